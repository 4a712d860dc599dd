"""ctypes binding of ``libmanta_b200.so`` (the C ABI declared in ``include/manta_b200.h``).

This is the Python twin of the cgo layer a Go host would use: every call returns ``int`` and a malloc'd
error string, which is turned into :class:`MantaError` here the way ``cStringError`` does in the reference
(runtime/backends/cuda/native_linux.go:3069-3084).  There is no fallback: a missing library or a failing
call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, byref, c_char_p, c_int, c_int32, c_int64, c_uint64, c_void_p

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libmanta_b200.so")

LAYOUT_F16, LAYOUT_Q8_ROW_F32, LAYOUT_Q4_B32_F16 = 0, 1, 2
LAYOUTS = {"f16": LAYOUT_F16, "q8": LAYOUT_Q8_ROW_F32, "q4": LAYOUT_Q4_B32_F16}
METRIC_DOT, METRIC_COSINE, METRIC_L2_DISTANCE = 0, 1, 2
METRICS = {"dot": METRIC_DOT, "cosine": METRIC_COSINE, "l2_distance": METRIC_L2_DISTANCE}
ORDER_LARGEST, ORDER_SMALLEST = 0, 1
MEM_HOST, MEM_DEVICE_COPY, MEM_DEVICE_ADOPT = 0, 1, 2

# every symbol include/manta_b200.h declares (tests check that the library exports all of them)
EXPORTS = [
    "manta_b200_runtime_create", "manta_b200_runtime_destroy", "manta_b200_free_cstring",
    "manta_b200_runtime_stream", "manta_b200_runtime_synchronize", "manta_b200_runtime_stats",
    "manta_b200_runtime_profile", "manta_b200_runtime_scan_time", "manta_b200_runtime_last_launch",
    "manta_b200_kernel_launch_count", "manta_b200_candidates_bind", "manta_b200_candidates_unbind",
    "manta_b200_candidates_bytes", "manta_b200_pack_q8_rows", "manta_b200_pack_q4_b32",
    "manta_b200_pack_q8_rows_device", "manta_b200_pack_q4_b32_device", "manta_b200_score",
    "manta_b200_score_topk", "manta_b200_score_topk_device", "manta_b200_topk_merge_device",
    "manta_b200_gather_rows", "manta_b200_q8_accumulators", "manta_b200_score_topk_static",
    "manta_b200_embedder_bind", "manta_b200_embedder_unbind", "manta_b200_embed_pooled", "manta_b200_embed_score_topk",
    "manta_b200_embed_device", "manta_b200_score_batched", "manta_b200_score_topk_batched",
    "manta_b200_candidates_save", "manta_b200_candidates_load", "manta_b200_packed_file_info",
    "manta_b200_exchange_create", "manta_b200_exchange_connect", "manta_b200_exchange_destroy",
    "manta_b200_exchange_connect_local", "manta_b200_exchange_set_wait_limit", "manta_b200_exchange_disconnect",
    "manta_b200_topk_exchange_merge_device", "manta_b200_score_topk_exchange_device",
]


class MantaError(RuntimeError):
    pass


class LaunchInfo(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_char * 48), ("grid", c_int), ("block", c_int), ("shared_bytes", c_int), ("launches", c_int)]


class Stats(ctypes.Structure):
    _fields_ = [(n, c_uint64) for n in (
        "bind_calls", "bound_bytes", "score_calls", "score_topk_calls", "kernel_launches", "h2d_bytes",
        "d2h_bytes", "chunked_reruns", "mma_passes", "gemv_passes")]

    def as_dict(self):
        return {n: int(getattr(self, n)) for n, _ in self._fields_}


_lib = None


def load() -> ctypes.CDLL:
    """Loads the shared library; raises if it has not been built (``python -m manta_b200.build``)."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise MantaError(f"{LIB_PATH} is missing: build it with `python -m manta_b200.build`; there is no fallback path")
    lib = ctypes.CDLL(LIB_PATH)
    E = POINTER(c_char_p)
    lib.manta_b200_free_cstring.argtypes = [c_void_p]
    lib.manta_b200_free_cstring.restype = None
    lib.manta_b200_kernel_launch_count.restype = c_uint64
    lib.manta_b200_candidates_bytes.restype = c_int64
    lib.manta_b200_candidates_bytes.argtypes = [c_void_p]
    sigs = {
        "manta_b200_runtime_create": [c_int, c_void_p, POINTER(c_void_p), E],
        "manta_b200_runtime_destroy": [c_void_p, E],
        "manta_b200_runtime_stream": [c_void_p, POINTER(c_void_p), E],
        "manta_b200_runtime_synchronize": [c_void_p, E],
        "manta_b200_runtime_stats": [c_void_p, POINTER(Stats), E],
        "manta_b200_runtime_profile": [c_void_p, c_int, E],
        "manta_b200_runtime_last_launch": [c_void_p, POINTER(LaunchInfo), E],
        "manta_b200_runtime_scan_time": [c_void_p, POINTER(ctypes.c_double), POINTER(c_int), E],
        "manta_b200_candidates_bind": [c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, c_int64, c_int,
                                       POINTER(c_void_p), E],
        "manta_b200_candidates_unbind": [c_void_p, c_void_p, E],
        "manta_b200_pack_q8_rows": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, E],
        "manta_b200_pack_q4_b32": [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, E],
        "manta_b200_pack_q8_rows_device": [c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, E],
        "manta_b200_pack_q4_b32_device": [c_void_p, c_void_p, c_int, c_int64, c_int, c_void_p, c_void_p, E],
        "manta_b200_score": [c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p, E],
        "manta_b200_score_topk": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, E],
        "manta_b200_score_topk_device": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                         c_void_p, c_int, E],
        "manta_b200_score_topk_static": [c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p,
                                         c_void_p, c_int, E],
        "manta_b200_topk_merge_device": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p,
                                         c_void_p, c_int, E],
        "manta_b200_gather_rows": [c_void_p, c_void_p, c_void_p, c_int64, c_void_p, E],
        "manta_b200_exchange_create": [c_void_p, c_int, c_int, c_int, c_int, POINTER(c_void_p), c_void_p, E],
        "manta_b200_exchange_connect": [c_void_p, c_void_p, c_void_p, E],
        "manta_b200_exchange_destroy": [c_void_p, c_void_p, E],
        "manta_b200_exchange_disconnect": [c_void_p, c_void_p, E],
        "manta_b200_exchange_connect_local": [c_void_p, c_void_p, POINTER(c_void_p), E],
        "manta_b200_exchange_set_wait_limit": [c_void_p, ctypes.c_uint32, E],
        "manta_b200_score_topk_exchange_device": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p,
                                                  c_int, E],
        "manta_b200_topk_exchange_merge_device": [c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, E],
        "manta_b200_candidates_save": [c_void_p, c_void_p, c_char_p, E],
        "manta_b200_candidates_load": [c_void_p, c_char_p, c_int64, c_int64, c_int, POINTER(c_void_p), E],
        "manta_b200_packed_file_info": [c_char_p, POINTER(c_int), POINTER(c_int64), POINTER(c_int), POINTER(c_int64), POINTER(c_int64), E],
        "manta_b200_score_batched": [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_void_p, E],
        "manta_b200_score_topk_batched": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_int, c_int64, c_int, c_int, c_int, c_void_p,
                                          c_void_p, E],
        "manta_b200_embedder_bind": [c_void_p, c_int, c_int, c_int, c_void_p, c_void_p, c_int, POINTER(c_void_p), E],
        "manta_b200_embedder_unbind": [c_void_p, c_void_p, E],
        "manta_b200_embed_pooled": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, E],
        "manta_b200_embed_device": [c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_void_p, c_int, E],
        "manta_b200_embed_score_topk": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                        c_int, c_void_p, c_void_p, E],
        "manta_b200_q8_accumulators": [c_void_p, c_void_p, c_void_p, c_void_p, E],
    }
    for name, args in sigs.items():
        fn = getattr(lib, name)
        fn.argtypes = args
        fn.restype = c_int
    _lib = lib
    return lib


def call(name: str, *args):
    """Calls an ABI function with a trailing ``char** err`` and raises MantaError on failure."""
    lib = load()
    err = c_char_p()
    rc = getattr(lib, name)(*args, byref(err))
    if rc != 0:
        msg = err.value.decode("utf-8", "replace") if err.value else f"{name} failed (rc={rc})"
        if err.value:
            lib.manta_b200_free_cstring(ctypes.cast(err, c_void_p))
        raise MantaError(msg)
    return rc


def _ptr(a):
    if a is None:
        return None
    if isinstance(a, np.ndarray):
        return a.ctypes.data_as(c_void_p)
    if hasattr(a, "data_ptr"):  # torch tensor
        return c_void_p(a.data_ptr())
    return c_void_p(int(a))


def f16_bits(x) -> np.ndarray:
    """Query/candidate values as IEEE half bit patterns (uint16).  float arrays are rounded to nearest even."""
    a = np.asarray(x)
    if a.dtype == np.uint16:
        return np.ascontiguousarray(a)
    if a.dtype == np.float16:
        return np.ascontiguousarray(a).view(np.uint16)
    return np.ascontiguousarray(a.astype(np.float16)).view(np.uint16)


def packed_file_info(path: str) -> dict:
    layout, rows, cols, base, stored = c_int(), c_int64(), c_int(), c_int64(), c_int64()
    call("manta_b200_packed_file_info", os.fsencode(path), byref(layout), byref(rows), byref(cols), byref(base), byref(stored))
    return {"layout": layout.value, "rows": rows.value, "cols": cols.value, "row_base": base.value, "stored_bytes": stored.value}


class Candidates:
    """A packed candidate matrix resident on the device (``MantaB200Candidates``)."""

    def __init__(self, rt: "Runtime", handle, layout: int, rows: int, cols: int, row_base: int, keep=None):
        self.rt, self.handle, self.layout, self.rows, self.cols, self.row_base = rt, handle, layout, rows, cols, row_base
        self._keep = keep  # adopted device tensors must outlive the set

    @property
    def stored_bytes(self) -> int:
        return int(load().manta_b200_candidates_bytes(self.handle))

    def unbind(self):
        if self.handle is not None:
            call("manta_b200_candidates_unbind", self.rt.handle, self.handle)
            self.handle = None
            self._keep = None

    def __del__(self):
        try:
            if self.handle is not None and self.rt.handle is not None:
                self.unbind()
        except Exception:
            pass


class Runtime:
    """One device runtime (``MantaB200Runtime``): owns the stream and the scratch buffers."""

    def __init__(self, device: int = 0, stream=None):
        self.handle = None
        h = c_void_p()
        call("manta_b200_runtime_create", c_int(device), _ptr(stream), byref(h))
        self.handle = h
        self.device = device

    def close(self):
        if self.handle is not None:
            call("manta_b200_runtime_destroy", self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    @property
    def stream(self) -> int:
        s = c_void_p()
        call("manta_b200_runtime_stream", self.handle, byref(s))
        return int(s.value or 0)

    def synchronize(self):
        call("manta_b200_runtime_synchronize", self.handle)

    def profile(self, enable: bool):
        call("manta_b200_runtime_profile", self.handle, c_int(1 if enable else 0))

    def scan_time(self):
        """(summed device ms of the scan kernels, passes measured) since the last call."""
        ms, n = ctypes.c_double(), c_int()
        call("manta_b200_runtime_scan_time", self.handle, byref(ms), byref(n))
        return float(ms.value), int(n.value)

    def stats(self) -> dict:
        s = Stats()
        call("manta_b200_runtime_stats", self.handle, byref(s))
        return s.as_dict()

    def last_launch(self) -> dict:
        """Launch configuration of the scan kernel of the last score / fused pass."""
        li = LaunchInfo()
        call("manta_b200_runtime_last_launch", self.handle, byref(li))
        return {"kernel": li.kernel.decode(), "grid": li.grid, "block": li.block, "shared_bytes": li.shared_bytes, "launches": li.launches}

    # ---- exchange of per-shard lists over peer memory ---------------------------------------------
    def exchange_create(self, world: int, rank: int, nq_max: int, k_max: int):
        """Returns (exchange handle, 64-byte IPC handle to pass to the other ranks)."""
        h = c_void_p()
        ipc = (ctypes.c_ubyte * 64)()
        call("manta_b200_exchange_create", self.handle, c_int(world), c_int(rank), c_int(nq_max), c_int(k_max), byref(h), ipc)
        return h, bytes(ipc)

    def exchange_connect(self, ex, handles) -> None:
        blob = b"".join(handles)
        buf = (ctypes.c_ubyte * len(blob)).from_buffer_copy(blob)
        call("manta_b200_exchange_connect", self.handle, ex, buf)

    def exchange_connect_local(self, ex, ranks) -> None:
        """Connects exchanges that live in this process: ``ranks[r]`` is rank r's exchange handle."""
        arr = (c_void_p * len(ranks))(*[r.value if isinstance(r, c_void_p) else r for r in ranks])
        call("manta_b200_exchange_connect_local", self.handle, ex, arr)

    def exchange_set_wait_limit(self, ex, naps_200ns: int) -> None:
        call("manta_b200_exchange_set_wait_limit", ex, ctypes.c_uint32(naps_200ns))

    def exchange_disconnect(self, ex) -> None:
        """First half of the tear-down: unmaps the peers' inboxes.  A host barrier belongs between this and destroy."""
        call("manta_b200_exchange_disconnect", self.handle, ex)

    def exchange_destroy(self, ex) -> None:
        call("manta_b200_exchange_destroy", self.handle, ex)

    def score_topk_exchange_device(self, ex, cands: "Candidates", metric: str, d_queries, nq: int, k: int, d_out_ids, d_out_scores,
                                   smallest: bool = False, sync: bool = False):
        """Shard pass + exchange over peer memory + merge, one stream-ordered chain."""
        call("manta_b200_score_topk_exchange_device", self.handle, ex, cands.handle, c_int(METRICS[metric]),
             c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST), _ptr(d_queries), c_int(nq), c_int(k), _ptr(d_out_ids),
             _ptr(d_out_scores), c_int(1 if sync else 0))

    def topk_exchange_merge_device(self, ex, d_ids, d_scores, nq: int, k: int, d_out_ids, d_out_scores, smallest: bool = False,
                                   sync: bool = False):
        call("manta_b200_topk_exchange_merge_device", self.handle, ex, c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST),
             _ptr(d_ids), _ptr(d_scores), c_int(nq), c_int(k), _ptr(d_out_ids), _ptr(d_out_scores), c_int(1 if sync else 0))

    # ---- packed candidate files ---------------------------------------------------------------------
    def save_candidates(self, cands: "Candidates", path: str) -> None:
        call("manta_b200_candidates_save", self.handle, cands.handle, os.fsencode(path))

    def load_candidates(self, path: str, row_begin: int = 0, row_end: int = -1, verify: bool = False) -> "Candidates":
        """Binds rows [row_begin, row_end) of a packed candidate file (row_end < 0: to the end)."""
        info = packed_file_info(path)
        end = info["rows"] if row_end < 0 else row_end
        h = c_void_p()
        call("manta_b200_candidates_load", self.handle, os.fsencode(path), c_int64(row_begin), c_int64(row_end), c_int(1 if verify else 0),
             byref(h))
        return Candidates(self, h, info["layout"], int(end - row_begin), info["cols"], info["row_base"] + int(row_begin))

    # ---- candidates -------------------------------------------------------------------------------
    def bind(self, layout, data, scales=None, row_base: int = 0, rows=None, cols=None, mem=None) -> Candidates:
        """Binds host numpy arrays (copied) or device tensors (mem = MEM_DEVICE_COPY / MEM_DEVICE_ADOPT)."""
        lay = LAYOUTS[layout] if isinstance(layout, str) else int(layout)
        keep = None
        if isinstance(data, np.ndarray):
            mem = MEM_HOST if mem is None else mem
            data = np.ascontiguousarray(data)
            if lay == LAYOUT_F16:
                data = f16_bits(data)
            if rows is None:
                rows = data.shape[0]
            if cols is None:
                cols = data.shape[1] * (2 if lay == LAYOUT_Q4_B32_F16 else 1)
            if scales is not None:
                scales = np.ascontiguousarray(scales, dtype=np.float32 if lay == LAYOUT_Q8_ROW_F32 else np.uint16)
        else:
            mem = MEM_DEVICE_ADOPT if mem is None else mem
            if rows is None or cols is None:
                rows = data.shape[0]
                cols = data.shape[1] * (2 if lay == LAYOUT_Q4_B32_F16 else 1)
            keep = (data, scales)
        h = c_void_p()
        call("manta_b200_candidates_bind", self.handle, c_int(lay), c_int64(rows), c_int(cols), _ptr(data), _ptr(scales),
             c_int64(row_base), c_int(mem), byref(h))
        return Candidates(self, h, lay, int(rows), int(cols), int(row_base), keep if mem == MEM_DEVICE_ADOPT else None)

    # ---- quantisers ------------------------------------------------------------------------------------
    def pack_q8_rows(self, src):
        src = np.ascontiguousarray(src, dtype=np.float32)
        rows, cols = src.shape
        codes = np.empty((rows, cols), np.int8)
        scales = np.empty(rows, np.float32)
        call("manta_b200_pack_q8_rows", self.handle, _ptr(src), c_int64(rows), c_int(cols), _ptr(codes), _ptr(scales))
        return codes, scales

    def pack_q4_b32(self, src):
        src = np.ascontiguousarray(src, dtype=np.float32)
        rows, cols = src.shape
        codes = np.empty((rows, cols // 2), np.uint8)
        scales = np.empty((rows, max(cols // 32, 1)), np.uint16)
        call("manta_b200_pack_q4_b32", self.handle, _ptr(src), c_int64(rows), c_int(cols), _ptr(codes), _ptr(scales))
        return codes, scales

    def pack_q8_rows_device(self, d_src, src_is_f16: bool, rows: int, cols: int, d_codes, d_scales):
        call("manta_b200_pack_q8_rows_device", self.handle, _ptr(d_src), c_int(1 if src_is_f16 else 0), c_int64(rows),
             c_int(cols), _ptr(d_codes), _ptr(d_scales))

    def pack_q4_b32_device(self, d_src, src_is_f16: bool, rows: int, cols: int, d_codes, d_scales):
        call("manta_b200_pack_q4_b32_device", self.handle, _ptr(d_src), c_int(1 if src_is_f16 else 0), c_int64(rows),
             c_int(cols), _ptr(d_codes), _ptr(d_scales))

    # ---- scoring ---------------------------------------------------------------------------------------
    @staticmethod
    def _queries(queries, cols):
        q = f16_bits(queries)
        one = q.ndim == 1
        q2 = q[None, :] if one else q
        if q2.ndim != 2 or q2.shape[1] != cols:
            # message of scoreLayout, runtime/backend/tensor_ops.go:1500
            raise MantaError(f"score mismatch {list(q.shape)} x [N, {cols}]")
        return np.ascontiguousarray(q2), one

    def score(self, cands: Candidates, metric: str, queries) -> np.ndarray:
        q, one = self._queries(queries, cands.cols)
        out = np.empty((q.shape[0], cands.rows), np.float32)
        call("manta_b200_score", self.handle, cands.handle, c_int(METRICS[metric]), _ptr(q), c_int(q.shape[0]), _ptr(out))
        return out[0] if one else out

    def score_topk(self, cands: Candidates, metric: str, queries, k: int, smallest: bool = False):
        q, one = self._queries(queries, cands.cols)
        kk = max(int(k), 0)
        ids = np.empty((q.shape[0], kk), np.int32)
        scores = np.empty((q.shape[0], kk), np.float32)
        call("manta_b200_score_topk", self.handle, cands.handle, c_int(METRICS[metric]),
             c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST), _ptr(q), c_int(q.shape[0]), c_int(int(k)), _ptr(ids),
             _ptr(scores))
        return (ids[0], scores[0]) if one else (ids, scores)

    def score_topk_device(self, cands: Candidates, metric: str, d_queries, nq: int, k: int, d_ids, d_scores,
                          smallest: bool = False, sync: bool = False):
        call("manta_b200_score_topk_device", self.handle, cands.handle, c_int(METRICS[metric]),
             c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST), _ptr(d_queries), c_int(nq), c_int(k), _ptr(d_ids),
             _ptr(d_scores), c_int(1 if sync else 0))

    def score_topk_static(self, cands: Candidates, metric: str, d_queries, nq: int, k: int, d_ids, d_scores,
                          smallest: bool = False, sync: bool = True):
        """The fused pass on the library's fixed scratch array: no device allocation happens in this call."""
        call("manta_b200_score_topk_static", self.handle, cands.handle, c_int(METRICS[metric]),
             c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST), _ptr(d_queries), c_int(nq), c_int(k), _ptr(d_ids),
             _ptr(d_scores), c_int(1 if sync else 0))

    def topk_merge_device(self, d_ids, d_scores, lists: int, nq: int, k: int, d_out_ids, d_out_scores,
                          smallest: bool = False, sync: bool = False, list_stride: int = 0):
        call("manta_b200_topk_merge_device", self.handle, c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST), _ptr(d_ids),
             _ptr(d_scores), c_int(lists), c_int64(list_stride), c_int(nq), c_int(k), _ptr(d_out_ids), _ptr(d_out_scores),
             c_int(1 if sync else 0))

    # ---- per-query candidate sets [Q,D] x [Q,N,D] -----------------------------------------------------------
    @staticmethod
    def _batched_args(queries, docs):
        q = np.ascontiguousarray(queries, dtype=np.float32)
        d = np.ascontiguousarray(docs, dtype=np.float32)
        if q.ndim != 2 or d.ndim != 3:
            raise MantaError("score expects query/docs as [D] x [N,D] or [Q,D] x [Q,N,D]")  # tensor_ops.go:1520
        if q.shape[0] != d.shape[0] or q.shape[1] != d.shape[2]:
            raise MantaError(f"score mismatch {list(q.shape)} x {list(d.shape)}")
        return q, d

    def score_batched(self, metric: str, queries, docs) -> np.ndarray:
        q, d = self._batched_args(queries, docs)
        out = np.empty((d.shape[0], d.shape[1]), np.float32)
        call("manta_b200_score_batched", self.handle, c_int(METRICS[metric]), _ptr(q), _ptr(d), c_int(d.shape[0]), c_int64(d.shape[1]),
             c_int(d.shape[2]), c_int(MEM_HOST), _ptr(out))
        return out

    def score_topk_batched(self, metric: str, queries, docs, k: int, smallest: bool = False):
        q, d = self._batched_args(queries, docs)
        kk = max(int(k), 0)
        ids = np.empty((d.shape[0], kk), np.int32)
        scores = np.empty((d.shape[0], kk), np.float32)
        call("manta_b200_score_topk_batched", self.handle, c_int(METRICS[metric]), c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST),
             _ptr(q), _ptr(d), c_int(d.shape[0]), c_int64(d.shape[1]), c_int(d.shape[2]), c_int(MEM_HOST), c_int(int(k)), _ptr(ids),
             _ptr(scores))
        return ids, scores

    # ---- embedding front end -----------------------------------------------------------------------------
    def bind_embedder(self, table, projection):
        """table [V,D], projection [D,E] (float arrays are rounded to f16); returns an opaque handle."""
        t, p = f16_bits(table), f16_bits(projection)
        h = c_void_p()
        call("manta_b200_embedder_bind", self.handle, c_int(t.shape[0]), c_int(t.shape[1]), c_int(p.shape[1]), _ptr(t), _ptr(p),
             c_int(MEM_HOST), byref(h))
        return h

    def unbind_embedder(self, emb):
        call("manta_b200_embedder_unbind", self.handle, emb)

    def embed_pooled(self, emb, out_dim: int, tokens, mask, normalize_then_pool: bool = False) -> np.ndarray:
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        mask = np.ascontiguousarray(mask, dtype=np.int32)
        out = np.empty((tokens.shape[0], out_dim), np.float32)
        call("manta_b200_embed_pooled", self.handle, emb, _ptr(tokens), _ptr(mask), c_int(tokens.shape[0]), c_int(tokens.shape[1]),
             c_int(1 if normalize_then_pool else 0), _ptr(out))
        return out

    def embed_device(self, emb, d_tokens, d_mask, batch: int, seq: int, d_out_queries, normalize_then_pool: bool = False,
                     sync: bool = False):
        call("manta_b200_embed_device", self.handle, emb, _ptr(d_tokens), _ptr(d_mask), c_int(batch), c_int(seq),
             c_int(1 if normalize_then_pool else 0), _ptr(d_out_queries), c_int(1 if sync else 0))

    def embed_score_topk(self, emb, cands: Candidates, tokens, mask, metric: str, k: int, smallest: bool = False,
                         normalize_then_pool: bool = False):
        tokens = np.ascontiguousarray(tokens, dtype=np.int32)
        mask = np.ascontiguousarray(mask, dtype=np.int32)
        b = tokens.shape[0]
        ids = np.empty((b, max(k, 0)), np.int32)
        scores = np.empty((b, max(k, 0)), np.float32)
        call("manta_b200_embed_score_topk", self.handle, emb, cands.handle, _ptr(tokens), _ptr(mask), c_int(b), c_int(tokens.shape[1]),
             c_int(1 if normalize_then_pool else 0), c_int(METRICS[metric]), c_int(ORDER_SMALLEST if smallest else ORDER_LARGEST),
             c_int(int(k)), _ptr(ids), _ptr(scores))
        return ids, scores

    def gather_rows(self, cands: Candidates, ids) -> np.ndarray:
        ids = np.ascontiguousarray(ids, dtype=np.int32)
        out = np.empty((ids.shape[0], cands.cols), np.float32)
        call("manta_b200_gather_rows", self.handle, cands.handle, _ptr(ids), c_int64(ids.shape[0]), _ptr(out))
        return out

    def q8_accumulators(self, cands: Candidates, query) -> np.ndarray:
        q, _ = self._queries(query, cands.cols)
        out = np.empty((cands.rows, 3), np.int32)
        call("manta_b200_q8_accumulators", self.handle, cands.handle, _ptr(q), _ptr(out))
        return out


def kernel_launch_count() -> int:
    return int(load().manta_b200_kernel_launch_count())
