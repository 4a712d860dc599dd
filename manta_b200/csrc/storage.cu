// Packed candidate files: the stored form of a bound candidate set (codes + scales of the q8-row / q4-block32 /
// f16 layouts) on disk, so that a set is quantised once and later bound -- whole or as one row shard per GPU -- by
// streaming the stored bytes to the device.  The reference exports q4 / q8 tensors widened to float32 inside its
// MLL container (runtime/mll_export.go:833-866; read back by decodeTensorEntry, runtime/weight_file.go:304-367),
// i.e. 8x / 4x the packed size, and re-derives nothing at load; this file format keeps the packed bytes.
//
// Layout (little endian): 256-byte header, codes [rows][elem_row_bytes] at data_offset, scales
// [rows][scale_row_bytes] at scales_offset (both offsets multiples of 256).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <climits>
#include <cstring>
#include <vector>

#include "../../include/manta_b200.h"
#include "internal.h"

namespace {

struct PackedFileHeader {
    char magic[8];            // "MB2PACK\0"
    uint32_t version;         // 1
    uint32_t layout;          // MANTA_B200_LAYOUT_*
    int64_t rows;
    int32_t cols;
    int32_t elem_row_bytes;   // bytes of codes per row as stored (no padding)
    int32_t scale_row_bytes;  // bytes of scales per row
    int32_t reserved0;
    int64_t data_offset;
    int64_t scales_offset;
    int64_t row_base;         // id of row 0 of the file
    uint64_t payload_fnv1a;   // FNV-1a 64 over codes then scales
    unsigned char pad[256 - 72];
};
static_assert(sizeof(PackedFileHeader) == 256, "header is 256 bytes");

const char kMagic[8] = {'M', 'B', '2', 'P', 'A', 'C', 'K', '\0'};

int fail(char** err, const char* fmt, ...) {
    if (err) {
        char buf[512];
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(buf, sizeof buf, fmt, ap);
        va_end(ap);
        size_t n = strlen(buf) + 1;
        char* out = (char*)malloc(n);
        if (out) memcpy(out, buf, n);
        *err = out;
    }
    return 1;
}

int geometry(int layout, int cols, int* elem_row_bytes, int* scale_row_bytes) {
    switch (layout) {
        case MANTA_B200_LAYOUT_F16: *elem_row_bytes = cols * 2; *scale_row_bytes = 0; return 0;
        case MANTA_B200_LAYOUT_Q8_ROW_F32: *elem_row_bytes = cols; *scale_row_bytes = 4; return 0;
        case MANTA_B200_LAYOUT_Q4_B32_F16:
            if (cols % 32) return 1;
            *elem_row_bytes = cols / 2;
            *scale_row_bytes = (cols / 32) * 2;
            return 0;
    }
    return 1;
}

uint64_t fnv1a(uint64_t h, const unsigned char* p, size_t n) {
    for (size_t i = 0; i < n; ++i) {
        h ^= p[i];
        h *= 1099511628211ull;
    }
    return h;
}

int64_t align256(int64_t v) { return (v + 255) / 256 * 256; }

int read_header(const char* path, int fd, PackedFileHeader* h, int64_t* file_size, char** err) {
    struct stat st;
    if (fstat(fd, &st) != 0) return fail(err, "packed file %s: %s", path, strerror(errno));
    *file_size = (int64_t)st.st_size;
    if (*file_size < (int64_t)sizeof(PackedFileHeader) || pread(fd, h, sizeof *h, 0) != (ssize_t)sizeof *h)
        return fail(err, "packed file %s: shorter than its header", path);
    if (memcmp(h->magic, kMagic, 8) != 0) return fail(err, "packed file %s: not a packed candidate file", path);
    if (h->version != 1) return fail(err, "packed file %s: unsupported version %u", path, h->version);
    int erb = 0, srb = 0;
    if (h->rows < 0 || h->cols <= 0 || geometry((int)h->layout, h->cols, &erb, &srb) || erb != h->elem_row_bytes || srb != h->scale_row_bytes)
        return fail(err, "packed file %s: header geometry is inconsistent (layout %u, cols %d)", path, h->layout, h->cols);
    // Bounds are checked by division, so that a corrupt row count cannot wrap the products.
    if (h->data_offset < (int64_t)sizeof *h || (h->data_offset & 255) || (h->scales_offset & 255) || h->data_offset > *file_size ||
        h->rows > (*file_size - h->data_offset) / erb)
        return fail(err, "packed file %s: sections exceed the file (%lld bytes)", path, (long long)*file_size);
    if (srb && (h->scales_offset < h->data_offset + h->rows * erb || h->scales_offset > *file_size ||
                h->rows > (*file_size - h->scales_offset) / srb))
        return fail(err, "packed file %s: sections exceed the file (%lld bytes)", path, (long long)*file_size);
    if (h->row_base < 0 || h->row_base > (int64_t)INT32_MAX || h->rows > (int64_t)INT32_MAX - h->row_base)
        return fail(err, "packed file %s: row ids [%lld, %lld + %lld) do not fit int32", path, (long long)h->row_base, (long long)h->row_base,
                    (long long)h->rows);
    return 0;
}

}  // namespace

extern "C" {

int manta_b200_candidates_save(MantaB200Runtime* rt, const MantaB200Candidates* set, const char* path, char** err) {
    if (!rt || !set || !path) return fail(err, "candidates_save: NULL argument");
    mb200::RuntimeInfo ri = mb200::runtime_info(rt);
    if (mb200::candidates_device(set) != ri.device) return fail(err, "candidates_save: candidate set lives on another device");
    const mb200::CandView cv = *mb200::candidates_view(set);
    PackedFileHeader h;
    memset(&h, 0, sizeof h);
    memcpy(h.magic, kMagic, 8);
    h.version = 1;
    h.layout = (uint32_t)cv.layout;
    h.rows = cv.rows;
    h.cols = cv.cols;
    if (geometry(cv.layout, cv.cols, &h.elem_row_bytes, &h.scale_row_bytes)) return fail(err, "candidates_save: unknown layout %d", cv.layout);
    h.data_offset = 256;
    h.scales_offset = align256(h.data_offset + h.rows * h.elem_row_bytes);
    h.row_base = cv.row_base;
    FILE* f = fopen(path, "wb");
    if (!f) return fail(err, "candidates_save: cannot create %s: %s", path, strerror(errno));
    std::lock_guard<std::mutex> lk(*ri.mu);
    int rc = 0;
    cudaError_t ce = cudaSetDevice(ri.device);
    if (ce == cudaSuccess) ce = cudaStreamSynchronize(ri.stream);
    uint64_t hash = 14695981039346656037ull;
    const int64_t chunk_rows = std::max<int64_t>(1, ((int64_t)64 << 20) / std::max(h.elem_row_bytes, 1));
    std::vector<unsigned char> buf;
    auto put = [&](const void* p, size_t n) {
        if (!rc && n && fwrite(p, 1, n, f) != n) rc = fail(err, "candidates_save: write to %s failed: %s", path, strerror(errno));
    };
    put(&h, sizeof h);  // rewritten with the checksum at the end
    for (int64_t r0 = 0; r0 < h.rows && !rc && ce == cudaSuccess; r0 += chunk_rows) {
        const int64_t n = std::min(chunk_rows, h.rows - r0);
        buf.resize((size_t)n * h.elem_row_bytes);
        ce = cudaMemcpy2D(buf.data(), h.elem_row_bytes, cv.data + (size_t)r0 * cv.row_bytes, cv.row_bytes, h.elem_row_bytes, (size_t)n,
                          cudaMemcpyDeviceToHost);
        if (ce != cudaSuccess) break;
        hash = fnv1a(hash, buf.data(), buf.size());
        put(buf.data(), buf.size());
    }
    if (!rc && ce == cudaSuccess) {
        const int64_t pad = h.scales_offset - (h.data_offset + h.rows * h.elem_row_bytes);
        const unsigned char zeros[256] = {0};
        put(zeros, (size_t)pad);
        if (h.scale_row_bytes && h.rows) {
            buf.resize((size_t)h.rows * h.scale_row_bytes);
            ce = cudaMemcpy(buf.data(), cv.scales, buf.size(), cudaMemcpyDeviceToHost);
            if (ce == cudaSuccess) {
                hash = fnv1a(hash, buf.data(), buf.size());
                put(buf.data(), buf.size());
            }
        }
    }
    if (!rc && ce == cudaSuccess) {
        h.payload_fnv1a = hash;
        if (fseek(f, 0, SEEK_SET) != 0) rc = fail(err, "candidates_save: seek in %s failed", path);
        put(&h, sizeof h);
    }
    if (fclose(f) != 0 && !rc && ce == cudaSuccess) rc = fail(err, "candidates_save: closing %s failed: %s", path, strerror(errno));
    if (ce != cudaSuccess) return fail(err, "candidates_save: CUDA error: %s", cudaGetErrorString(ce));
    return rc;
}

int manta_b200_packed_file_info(const char* path, int* layout, int64_t* rows, int* cols, int64_t* row_base, int64_t* stored_bytes,
                                char** err) {
    if (!path) return fail(err, "packed_file_info: NULL path");
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(err, "packed file %s: %s", path, strerror(errno));
    PackedFileHeader h;
    int64_t size = 0;
    int rc = read_header(path, fd, &h, &size, err);
    close(fd);
    if (rc) return rc;
    if (layout) *layout = (int)h.layout;
    if (rows) *rows = h.rows;
    if (cols) *cols = h.cols;
    if (row_base) *row_base = h.row_base;
    if (stored_bytes) *stored_bytes = h.rows * ((int64_t)h.elem_row_bytes + h.scale_row_bytes);
    return 0;
}

int manta_b200_candidates_load(MantaB200Runtime* rt, const char* path, int64_t row_begin, int64_t row_end, int verify,
                               MantaB200Candidates** out, char** err) {
    if (!rt || !path || !out) return fail(err, "candidates_load: NULL argument");
    *out = nullptr;
    int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(err, "packed file %s: %s", path, strerror(errno));
    PackedFileHeader h;
    int64_t size = 0;
    if (read_header(path, fd, &h, &size, err)) {
        close(fd);
        return 1;
    }
    if (row_end < 0) row_end = h.rows;
    if (row_begin < 0 || row_begin > row_end || row_end > h.rows) {
        close(fd);
        return fail(err, "candidates_load: rows [%lld, %lld) are outside the file's %lld rows", (long long)row_begin, (long long)row_end,
                    (long long)h.rows);
    }
    void* map = size > 0 ? mmap(nullptr, (size_t)size, PROT_READ, MAP_PRIVATE, fd, 0) : MAP_FAILED;
    close(fd);
    if (map == MAP_FAILED) return fail(err, "packed file %s: mmap failed: %s", path, strerror(errno));
    const unsigned char* base = (const unsigned char*)map;
    int rc = 0;
    if (verify) {
        uint64_t hash = 14695981039346656037ull;
        hash = fnv1a(hash, base + h.data_offset, (size_t)(h.rows * h.elem_row_bytes));
        if (h.scale_row_bytes) hash = fnv1a(hash, base + h.scales_offset, (size_t)(h.rows * h.scale_row_bytes));
        if (hash != h.payload_fnv1a) rc = fail(err, "packed file %s: payload checksum mismatch", path);
    }
    if (!rc) {
        const void* data = base + h.data_offset + row_begin * h.elem_row_bytes;
        const void* scales = h.scale_row_bytes ? base + h.scales_offset + row_begin * h.scale_row_bytes : nullptr;
        rc = manta_b200_candidates_bind(rt, (int)h.layout, row_end - row_begin, h.cols, data, scales, h.row_base + row_begin,
                                        MANTA_B200_MEM_HOST, out, err);
    }
    munmap(map, (size_t)size);
    return rc;
}

}  // extern "C"
