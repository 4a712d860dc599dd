// Host executor of the score/select path: Module JSON -> validated plan -> step walk with fused device passes.
// Mirrors, for this path only, ExecuteSymbolic / executeStep (runtime/backend/symbolic.go:14-163,
// tensor_ops.go:13-135) and the CUDA executor's dispatch (runtime/backends/cuda/cuda.go:222-429) of the
// reference (paths inside odvcencio/manta).  All arithmetic runs in the kernels behind include/manta_b200.h.
#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <string>
#include <vector>

#include "../../../include/manta_b200_host.h"
#include "half.h"
#include "json.h"
#include "sha256.h"

namespace {

using mjson::Value;
using mb200_host::half_bits;

const char* kVersion = "manta/v0alpha1";  // artifact/manta/module.go:9

int fail(char** err, const char* fmt, ...) {
    if (err) {
        char buf[768];
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

// ---- schema (the subset of artifact/manta/module.go:84-207 this path reads) -----------------------------------
struct ValueType {
    std::string kind;                 // tensor | candidate_pack | kv_cache
    std::string dtype;                // tensor
    std::vector<std::string> shape;   // tensor or candidate_pack shape symbols
};
struct Binding {
    std::string name;
    ValueType type;
};
struct Param {
    std::string name, binding;
    ValueType type;
    bool trainable = false;
};
struct EntryPoint {
    std::string name, kind;
    std::vector<Binding> inputs, outputs;
};
struct Variant {
    std::string backend, entry, source;
    std::map<std::string, std::string> meta;
    bool has_backend = false;
};
struct Hints {  // ScheduleHints, artifact/manta/module.go:168-176 (the fields the launch configuration reads)
    std::vector<int> tile, tile_2d;
    int vector_width = 0;
    std::string memory;
};
struct Kernel {
    std::string name, op;  // op = body[0].op
    std::vector<Binding> inputs, outputs;
    std::vector<Variant> variants;
    Hints hints;
    bool empty_body_op = false;
};
struct Step {
    std::string entry, kind, name, kernel;
    std::vector<std::string> inputs, outputs;
    std::map<std::string, std::string> attributes;
};
struct Module {
    std::string version, name;
    std::vector<std::string> supported_backends;
    std::vector<Param> params;
    std::vector<EntryPoint> entries;
    std::vector<Kernel> kernels;
    std::vector<Step> steps;
};

// ---- runtime values (runtime/backend/tensor.go:11-31, backend.go:18-25) -------------------------------------------
struct Tensor {
    std::string dtype;
    std::vector<int64_t> shape;
    std::vector<float> f32;
    std::vector<int32_t> i32;
    std::vector<int64_t> i64;
    int64_t elements() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
    const void* data() const {
        if (dtype == "i32") return i32.data();
        if (dtype == "i64") return i64.data();
        return f32.data();
    }
};
using TensorP = std::shared_ptr<Tensor>;
struct Pack {
    TensorP ids, scores, docs;
};
struct RValue {
    ValueType type;
    TensorP tensor;
    std::shared_ptr<Pack> pack;
    std::string producer;
    std::vector<std::string> inputs;
    Value metadata = Value::make_object();
};

bool float_like(const std::string& dt) { return dt != "i32" && dt != "i64"; }

std::vector<std::string> strings_of(const Value* v) {
    std::vector<std::string> out;
    if (v)
        for (const auto& e : v->items())
            if (e.is_string()) out.push_back(e.str);
    return out;
}

ValueType parse_type(const Value* v) {
    ValueType t;
    if (!v) return t;
    t.kind = v->get_string("kind");
    if (const Value* tt = v->get("tensor")) {
        t.dtype = tt->get_string("dtype");
        t.shape = strings_of(tt->get("shape"));
    }
    if (const Value* cp = v->get("candidate_pack")) t.shape = strings_of(cp->get("shape"));
    return t;
}

std::vector<Binding> parse_bindings(const Value* v) {
    std::vector<Binding> out;
    if (v)
        for (const auto& e : v->items()) out.push_back(Binding{e.get_string("name"), parse_type(e.get("type"))});
    return out;
}

bool parse_module(const std::string& text, Module* m, std::string* err) {
    Value root;
    mjson::Parser p(text);
    if (!p.parse(&root, err)) return false;
    if (!root.is_object()) { *err = "module JSON is not an object"; return false; }
    m->version = root.get_string("version");
    m->name = root.get_string("name");
    if (const Value* rq = root.get("requirements")) m->supported_backends = strings_of(rq->get("supported_backends"));
    if (const Value* ps = root.get("params"))
        for (const auto& e : ps->items()) {
            Param p{e.get_string("name"), e.get_string("binding"), parse_type(e.get("type"))};
            if (const Value* tr = e.get("trainable")) p.trainable = tr->kind == Value::Bool && tr->b;
            m->params.push_back(p);
        }
    if (const Value* es = root.get("entry_points"))
        for (const auto& e : es->items())
            m->entries.push_back(EntryPoint{e.get_string("name"), e.get_string("kind"), parse_bindings(e.get("inputs")), parse_bindings(e.get("outputs"))});
    if (const Value* ks = root.get("kernels"))
        for (const auto& e : ks->items()) {
            Kernel k;
            k.name = e.get_string("name");
            k.inputs = parse_bindings(e.get("inputs"));
            k.outputs = parse_bindings(e.get("outputs"));
            if (const Value* body = e.get("body")) {
                if (!body->items().empty()) k.op = body->items()[0].get_string("op");
                for (const auto& op : body->items()) k.empty_body_op = k.empty_body_op || op.get_string("op").empty();
            }
            if (const Value* h = e.get("hints")) {
                auto ints = [](const Value* a) {
                    std::vector<int> out;
                    if (a)
                        for (const auto& x : a->items())
                            if (x.kind == Value::Number) out.push_back((int)x.num);
                    return out;
                };
                k.hints.tile = ints(h->get("tile"));
                k.hints.tile_2d = ints(h->get("tile_2d"));
                if (const Value* vw = h->get("vector_width"))
                    if (vw->kind == Value::Number) k.hints.vector_width = (int)vw->num;
                k.hints.memory = h->get_string("memory");
            }
            if (const Value* vs = e.get("variants"))
                for (const auto& v : vs->items()) {
                    Variant var;
                    var.backend = v.get_string("backend");
                    var.entry = v.get_string("entry");
                    var.source = v.get_string("source");
                    if (const Value* mt = v.get("meta"))
                        if (mt->is_object())
                            for (const auto& kv : *mt->obj)
                                if (kv.second.is_string()) var.meta[kv.first] = kv.second.str;
                    k.variants.push_back(var);
                }
            m->kernels.push_back(k);
        }
    if (const Value* ss = root.get("steps"))
        for (const auto& e : ss->items()) {
            Step s;
            s.entry = e.get_string("entry");
            s.kind = e.get_string("kind");
            s.name = e.get_string("name");
            s.kernel = e.get_string("kernel");
            s.inputs = strings_of(e.get("inputs"));
            s.outputs = strings_of(e.get("outputs"));
            if (const Value* at = e.get("attributes"))
                if (at->is_object())
                    for (const auto& kv : *at->obj)
                        if (kv.second.is_string()) s.attributes[kv.first] = kv.second.str;
            m->steps.push_back(s);
        }
    return true;
}

const Kernel* kernel_by_name(const Module& m, const std::string& name) {
    for (const auto& k : m.kernels)
        if (k.name == name) return &k;
    return nullptr;
}
const EntryPoint* entry_by_name(const Module& m, const std::string& name) {
    for (const auto& e : m.entries)
        if (e.name == name) return &e;
    return nullptr;
}
const Param* param_by_name(const Module& m, const std::string& name) {
    for (const auto& p : m.params)
        if (p.name == name) return &p;
    return nullptr;
}
bool is_score_op(const std::string& op) { return op == "dot" || op == "cosine" || op == "l2_distance"; }
int metric_of(const std::string& op) {
    return op == "dot" ? MANTA_B200_METRIC_DOT : op == "cosine" ? MANTA_B200_METRIC_COSINE : MANTA_B200_METRIC_L2_DISTANCE;
}
const Variant* cuda_variant(const Kernel& k) {
    for (const auto& v : k.variants)
        if (v.backend == "cuda") return &v;
    return nullptr;
}

// validateKernelVariants (artifact/manta/module.go:426-449): one variant per backend, each with an entry and a
// source, and a variant for every backend the module says it supports (all five for a compiler-made module).
bool validate_kernel_variants(const std::vector<std::string>& required, const Kernel& k, std::string* err) {
    std::set<std::string> seen;
    for (const auto& v : k.variants) {
        if (v.backend.empty()) { *err = "kernel \"" + k.name + "\" variant backend is required"; return false; }
        if (!seen.insert(v.backend).second) { *err = "kernel \"" + k.name + "\" has duplicate variant for backend \"" + v.backend + "\""; return false; }
        if (v.entry.empty()) { *err = "kernel \"" + k.name + "\" variant entry is required for backend \"" + v.backend + "\""; return false; }
        if (v.source.empty()) { *err = "kernel \"" + k.name + "\" variant source is required for backend \"" + v.backend + "\""; return false; }
    }
    for (const auto& b : required)
        if (!seen.count(b)) { *err = "kernel \"" + k.name + "\" is missing variant for backend \"" + b + "\""; return false; }
    return true;
}

// Module.Validate, the part that concerns this path (artifact/manta/module.go:256-449), followed by what loading on
// the CUDA backend adds: the module must list "cuda" (Backend.CanLoad, runtime/backends/cuda/cuda.go:53-56), every
// kernel must carry a cuda variant (CompileVariants, runtime/backend/backend.go:275-296) whose source defines its
// entry (validateCompiledKernelSource, runtime/backend/native_kernel.go:37-63).
bool validate_module(const Module& m, std::string* err) {
    if (m.name.empty()) { *err = "module name is required"; return false; }
    if (m.version.empty()) { *err = "module version is required"; return false; }
    if (m.version != kVersion) { *err = "module version \"" + m.version + "\" is not supported, want \"" + kVersion + "\""; return false; }
    if (m.supported_backends.empty()) { *err = "at least one supported backend is required"; return false; }
    {
        std::set<std::string> seen;
        for (const auto& b : m.supported_backends) {
            if (b.empty()) { *err = "supported backend is required"; return false; }
            if (!seen.insert(b).second) { *err = "duplicate supported backend \"" + b + "\""; return false; }
        }
    }
    if (m.entries.empty()) { *err = "module requires at least one entry point"; return false; }
    std::set<std::string> seen;
    for (const auto& e : m.entries) {
        if (e.name.empty()) { *err = "entry point name is required"; return false; }
        if (!seen.insert(e.name).second) { *err = "duplicate entry point \"" + e.name + "\""; return false; }
    }
    std::set<std::string> kernel_names;
    for (const auto& k : m.kernels) {
        if (k.name.empty()) { *err = "kernel name is required"; return false; }
        if (!kernel_names.insert(k.name).second) { *err = "duplicate kernel \"" + k.name + "\""; return false; }
        if (k.empty_body_op) { *err = "kernel \"" + k.name + "\" has body op with empty op name"; return false; }
        if (!validate_kernel_variants(m.supported_backends, k, err)) return false;
    }
    for (const auto& s : m.steps) {
        if (!entry_by_name(m, s.entry)) { *err = "step \"" + s.name + "\" references unknown entry point \"" + s.entry + "\""; return false; }
        if (s.kind == "launch_kernel") {
            const Kernel* k = kernel_by_name(m, s.kernel);
            if (!k) { *err = "step \"" + s.name + "\" references unknown kernel \"" + s.kernel + "\""; return false; }
        }
    }
    // loading on the CUDA backend
    if (std::find(m.supported_backends.begin(), m.supported_backends.end(), "cuda") == m.supported_backends.end()) {
        *err = "cuda: unsupported backend";  // Runtime.Load's reason for a backend that cannot load the module (runtime.go:62-64)
        return false;
    }
    for (const auto& k : m.kernels) {
        const Variant* v = cuda_variant(k);
        if (!v) { *err = "kernel \"" + k.name + "\" missing variant for backend \"cuda\""; return false; }
        if (v->source.find("__global__ void " + v->entry + "(") == std::string::npos) {
            *err = "kernel \"" + k.name + "\" CUDA source does not define entry \"" + v->entry + "\"";
            return false;
        }
    }
    return true;
}

// firstTileSize / estimatedSharedBytes (runtime/backend/native_kernel.go:114-148): what the plan's hints ask for.
int first_tile_size(const Kernel& k, const Variant& v) {
    if (!k.hints.tile.empty() && k.hints.tile[0] > 0) return k.hints.tile[0];
    auto it = v.meta.find("tile");
    if (it != v.meta.end()) {
        std::string raw = it->second;
        if (!raw.empty() && raw.front() == '[') raw.erase(0, 1);
        if (!raw.empty() && raw.back() == ']') raw.pop_back();
        const int n = atoi(raw.c_str());
        if (n > 0) return n;
    }
    return 1;
}
int estimated_shared_bytes(const Kernel& k, int tile) {
    if (tile <= 0) tile = 1;
    if (k.hints.memory != "workgroup_local") return 0;
    const int width = k.hints.vector_width > 0 ? k.hints.vector_width : 1;
    int values = (int)(k.inputs.size() + k.outputs.size());
    if (values == 0) values = 1;
    return tile * width * values * 4;
}

// ---- candidate sets bound from float32-labelled tensors --------------------------------------------------------
struct BoundSet {
    MantaB200Candidates* set = nullptr;
    int layout = 0;
    int64_t rows = 0;
    int cols = 0;         // logical columns
    int stored_cols = 0;  // columns as bound (q4 pads to a multiple of 32 with zeros)
};

}  // namespace

struct MantaB200Program {
    MantaB200Runtime* rt = nullptr;
    Module mod;
    std::map<std::string, TensorP> weights;
    std::map<std::string, BoundSet> resident;  // params feeding score kernels, bound at first run
    std::map<std::string, std::string> residency;  // param -> residency of an applied memory plan
    uint64_t runs = 0;
};

struct MantaB200Result {
    std::map<std::string, RValue> outputs;
    std::string json;
};

namespace {

int layout_of_label(const std::string& dtype) {
    if (dtype == "q8") return MANTA_B200_LAYOUT_Q8_ROW_F32;
    if (dtype == "q4") return MANTA_B200_LAYOUT_Q4_B32_F16;
    return MANTA_B200_LAYOUT_F16;  // f16 / f32 labels
}

// Quantises a [rows, cols] float32 tensor into the packed layout its dtype label names and binds it.
int bind_docs(MantaB200Runtime* rt, const float* data, int64_t rows, int cols, const std::string& dtype, BoundSet* out, char** err) {
    out->layout = layout_of_label(dtype);
    out->rows = rows;
    out->cols = cols;
    out->stored_cols = cols;
    if (out->layout == MANTA_B200_LAYOUT_Q8_ROW_F32) {
        std::vector<int8_t> codes((size_t)rows * cols);
        std::vector<float> scales((size_t)rows);
        if (manta_b200_pack_q8_rows(rt, data, rows, cols, codes.data(), scales.data(), err)) return 1;
        return manta_b200_candidates_bind(rt, out->layout, rows, cols, codes.data(), scales.data(), 0, MANTA_B200_MEM_HOST, &out->set, err);
    }
    if (out->layout == MANTA_B200_LAYOUT_Q4_B32_F16) {
        const int pc = (cols + 31) / 32 * 32;  // zero columns change none of the three scores
        out->stored_cols = pc;
        std::vector<float> padded;
        const float* src = data;
        if (pc != cols) {
            padded.assign((size_t)rows * pc, 0.0f);
            for (int64_t r = 0; r < rows; ++r) memcpy(&padded[(size_t)r * pc], data + (size_t)r * cols, (size_t)cols * 4);
            src = padded.data();
        }
        std::vector<uint8_t> codes((size_t)rows * pc / 2);
        std::vector<uint16_t> scales((size_t)rows * (pc / 32));
        if (manta_b200_pack_q4_b32(rt, src, rows, pc, codes.data(), scales.data(), err)) return 1;
        return manta_b200_candidates_bind(rt, out->layout, rows, pc, codes.data(), scales.data(), 0, MANTA_B200_MEM_HOST, &out->set, err);
    }
    std::vector<uint16_t> bits((size_t)rows * cols);
    for (size_t i = 0; i < bits.size(); ++i) bits[i] = half_bits(data[i]);
    return manta_b200_candidates_bind(rt, out->layout, rows, cols, bits.data(), nullptr, 0, MANTA_B200_MEM_HOST, &out->set, err);
}

std::string shape_text(const std::vector<int64_t>& s) {
    std::string out = "[";
    for (size_t i = 0; i < s.size(); ++i) out += (i ? " " : "") + std::to_string(s[i]);
    return out + "]";
}

// validateTensorType + bindShape (runtime/backend/tensor.go:388-401, 491-517).
bool check_tensor(const ValueType& type, const Tensor& t, std::map<std::string, int64_t>* sym, std::string* err) {
    if (type.kind != "tensor") { *err = "expected tensor type metadata"; return false; }
    if (!type.dtype.empty() && t.dtype != type.dtype && !(type.dtype == "f16" && t.dtype == "f32")) {
        *err = "tensor dtype \"" + t.dtype + "\" does not match expected \"" + type.dtype + "\"";
        return false;
    }
    if (!type.shape.empty() && type.shape.size() != t.shape.size()) {
        *err = "tensor rank " + std::to_string(t.shape.size()) + " does not match expected rank " + std::to_string(type.shape.size());
        return false;
    }
    for (size_t i = 0; i < type.shape.size(); ++i) {
        const std::string& s = type.shape[i];
        if (s.empty()) continue;
        char* end = nullptr;
        long lit = strtol(s.c_str(), &end, 10);
        if (end && *end == 0) {
            if (lit != t.shape[i]) { *err = "dimension " + std::to_string(i) + " mismatch: expected " + s + ", got " + std::to_string(t.shape[i]); return false; }
            continue;
        }
        auto it = sym->find(s);
        if (it != sym->end()) {
            if (it->second != t.shape[i]) {
                *err = "symbol \"" + s + "\" mismatch: expected " + std::to_string(it->second) + ", got " + std::to_string(t.shape[i]);
                return false;
            }
            continue;
        }
        (*sym)[s] = t.shape[i];
    }
    return true;
}

TensorP tensor_from_arg(const MantaB200TensorArg& a, std::string* err) {
    auto t = std::make_shared<Tensor>();
    t->dtype = a.dtype ? a.dtype : "";
    for (int i = 0; i < a.rank; ++i) {
        if (a.shape[i] < 0) { *err = "negative dimension"; return nullptr; }
        t->shape.push_back(a.shape[i]);
    }
    const int64_t n = t->elements();
    if (n > 0 && !a.data) { *err = "tensor is nil"; return nullptr; }
    if (t->dtype == "i32") t->i32.assign((const int32_t*)a.data, (const int32_t*)a.data + n);
    else if (t->dtype == "i64") t->i64.assign((const int64_t*)a.data, (const int64_t*)a.data + n);
    else t->f32.assign((const float*)a.data, (const float*)a.data + n);
    return t;
}

Value shape_json(const std::vector<int64_t>& s) {
    Value a = Value::make_array();
    for (int64_t d : s) a.push(Value::make_number((double)d));
    return a;
}
Value strings_json(const std::vector<std::string>& s) {
    Value a = Value::make_array();
    for (const auto& x : s) a.push(Value::make_string(x));
    return a;
}

// What the walker decided for one score kernel launch of an entry point.
struct Fusion {
    int score_step = -1;              // index into the entry's step list
    int topk_step = -1;
    std::vector<int> gather_steps;    // gather(scores, ids)
    bool need_full_scores = false;    // scores are returned or read by a step that is not fused
    std::string scores_name, ids_name, query_name, docs_name, op;
    std::string bind_name;            // the value the candidate set is bound from: docs_name seen through dequant steps
    int k = 0;
};

std::vector<const Step*> steps_for_entry(const Module& m, const std::string& entry) {
    std::vector<const Step*> out;
    for (const auto& s : m.steps)
        if (s.entry == entry) out.push_back(&s);
    return out;
}

// Pre-pass over an entry's steps: launch_kernel{dot|cosine|l2_distance} -> topk -> gather(scores, ids).
std::vector<Fusion> plan_fusions(const Module& m, const std::vector<const Step*>& steps) {
    std::vector<Fusion> out;
    for (size_t i = 0; i < steps.size(); ++i) {
        const Step& s = *steps[i];
        if (s.kind != "launch_kernel") continue;
        const Kernel* k = kernel_by_name(m, s.kernel);
        if (!k || !is_score_op(k->op) || s.inputs.size() != 2 || s.outputs.size() != 1) continue;
        Fusion f;
        f.score_step = (int)i;
        f.op = k->op;
        f.query_name = s.inputs[0];
        f.docs_name = s.inputs[1];
        f.scores_name = s.outputs[0];
        // score(q, dequant(docs_q)): dequant only relabels (tensor_ops.go:136-148), so the pass binds docs_q itself, in
        // the packed layout its own label names
        f.bind_name = f.docs_name;
        for (bool again = true; again;) {
            again = false;
            for (size_t j = 0; j < i; ++j) {
                const Step& d = *steps[j];
                if (d.kind == "dequant" && d.inputs.size() == 1 && d.outputs.size() == 1 && d.outputs[0] == f.bind_name) {
                    f.bind_name = d.inputs[0];
                    again = true;
                    break;
                }
            }
        }
        for (size_t j = i + 1; j < steps.size(); ++j) {
            const Step& t = *steps[j];
            const bool reads_scores = std::find(t.inputs.begin(), t.inputs.end(), f.scores_name) != t.inputs.end();
            const bool returns_scores = t.kind == "return" && std::find(t.outputs.begin(), t.outputs.end(), f.scores_name) != t.outputs.end();
            if (t.kind == "topk" && f.topk_step < 0 && t.inputs.size() == 1 && t.inputs[0] == f.scores_name && t.outputs.size() == 1) {
                f.topk_step = (int)j;
                f.ids_name = t.outputs[0];
                auto it = t.attributes.find("k");
                f.k = (it == t.attributes.end()) ? 0 : atoi(it->second.c_str());
                continue;
            }
            if (t.kind == "gather" && f.topk_step >= 0 && t.inputs.size() == 2 && t.inputs[0] == f.scores_name && t.inputs[1] == f.ids_name) {
                f.gather_steps.push_back((int)j);
                continue;
            }
            if (reads_scores || returns_scores) f.need_full_scores = true;
        }
        if (f.topk_step < 0) f.need_full_scores = true;
        out.push_back(f);
    }
    return out;
}

Value fusion_json(const std::vector<const Step*>& steps, const std::vector<Fusion>& fusions) {
    Value arr = Value::make_array();
    for (size_t i = 0; i < steps.size(); ++i) {
        Value o = Value::make_object();
        o.set("kind", Value::make_string(steps[i]->kind));
        o.set("name", Value::make_string(steps[i]->name));
        std::string how = (steps[i]->kind == "return") ? "host" : "device";
        for (const auto& f : fusions) {
            if ((int)i == f.score_step) how = f.topk_step >= 0 ? (f.need_full_scores ? "fused_pass+full_scores" : "fused_pass") : "score_pass";
            if ((int)i == f.topk_step) how = "fused_with_score";
            for (int g : f.gather_steps)
                if ((int)i == g) how = "fused_with_score";
        }
        if (steps[i]->kind == "pack_candidates") how = "host";
        if (steps[i]->kind == "dequant") how = "relabel";
        o.set("execution", Value::make_string(how));
        arr.push(o);
    }
    return arr;
}

}  // namespace

namespace {

// tensorLogicalBytes (runtime/memory_plan.go:381-406): codes only, q4 = (n+1)/2, q8 = n.
int64_t logical_bytes(const Tensor& t) {
    int64_t n = 1;
    for (int64_t d : t.shape) {
        if (d <= 0) return 0;
        n *= d;
    }
    if (t.dtype == "q4") return (n + 1) / 2;
    if (t.dtype == "q8") return n;
    if (t.dtype == "f16") return n * 2;
    if (t.dtype == "i64") return n * 8;
    return n * 4;
}

// Bytes one shard really holds in HBM when the tensor is bound as a candidate set: padded codes + scales + the
// 4-byte row statistic.  Tensors that are not rank-2 float-like are counted as the reference counts them.
int64_t device_bytes(const Tensor& t, int shards) {
    if (t.shape.size() != 2 || !float_like(t.dtype) || t.shape[0] <= 0 || t.shape[1] <= 0) return logical_bytes(t);
    const int64_t rows = (t.shape[0] + shards - 1) / shards, cols = t.shape[1];
    if (t.dtype == "q8") return rows * ((cols + 15) / 16 * 16 + 4 + 4);
    if (t.dtype == "q4") {
        const int64_t pc = (cols + 31) / 32 * 32;
        return rows * (pc / 2 + (pc / 32) * 2 + 4);
    }
    return rows * ((cols + 7) / 8 * 16 + 4);  // stored as f16
}

}  // namespace

extern "C" {

/* NewMemoryPlan (runtime/memory_plan.go:59-138): same ordering (trainable first, then access count descending,
 * bytes ascending, name) and the same residency rule.  accounting 0 budgets the reference's logical bytes, 1 the
 * bytes a shard really holds on the device (codes + scales + row statistic). */
int manta_b200_program_memory_plan(MantaB200Program* prog, int64_t device_budget_bytes, int shared_host_weights, int shards,
                                   int accounting, char** out_json, char** err) {
    if (!prog || !out_json) return fail(err, "memory_plan: NULL argument");
    if (shards <= 0) return fail(err, "memory_plan: shard count %d out of range", shards);
    struct Item {
        std::string name, dtype, residency;
        std::vector<int64_t> shape;
        bool trainable;
        int64_t bytes, dev_bytes;
        int access;
    };
    std::map<std::string, int> access;
    for (const auto& s : prog->mod.steps)
        for (const auto& in : s.inputs)
            if (param_by_name(prog->mod, in)) access[in]++;
    std::vector<Item> items;
    int64_t total = 0;
    for (const auto& kv : prog->weights) {
        const Param* p = param_by_name(prog->mod, kv.first);
        Item it{kv.first, kv.second->dtype, "device_resident", kv.second->shape, p ? p->trainable : false,
                logical_bytes(*kv.second), device_bytes(*kv.second, shards), access[kv.first]};
        total += accounting ? it.dev_bytes : it.bytes;
        items.push_back(it);
    }
    auto cost = [&](const Item& it) { return accounting ? it.dev_bytes : it.bytes; };
    std::sort(items.begin(), items.end(), [&](const Item& a, const Item& b) {
        if (a.trainable != b.trainable) return a.trainable;
        if (a.access != b.access) return a.access > b.access;
        if (cost(a) != cost(b)) return cost(a) < cost(b);
        return a.name < b.name;
    });
    int64_t used = 0, dev = 0, host = 0, lazy = 0;
    const bool budgeted = device_budget_bytes > 0;
    for (auto& it : items) {
        const bool fits = !budgeted || used + cost(it) <= device_budget_bytes;
        if (it.trainable || fits) {
            it.residency = "device_resident";
            used += cost(it);
            dev += cost(it);
        } else if (shared_host_weights) {
            it.residency = "host_shared";
            host += cost(it);
        } else if (it.access <= 1) {
            it.residency = "lazy_staged";
            lazy += cost(it);
        } else {
            it.residency = "host_pinned";
            host += cost(it);
        }
    }
    std::sort(items.begin(), items.end(), [](const Item& a, const Item& b) { return a.name < b.name; });
    Value root = Value::make_object();
    root.set("version", Value::make_string("manta/memory/v0alpha1"));
    root.set("module_name", Value::make_string(prog->mod.name));
    root.set("backend", Value::make_string("cuda"));
    root.set("device_budget_bytes", Value::make_number((double)device_budget_bytes));
    root.set("accounting", Value::make_string(accounting ? "device_bytes_per_shard" : "logical_bytes"));
    root.set("shards", Value::make_number(shards));
    root.set("total_weight_bytes", Value::make_number((double)total));
    root.set("device_resident_bytes", Value::make_number((double)dev));
    root.set("host_resident_bytes", Value::make_number((double)host));
    root.set("lazy_staged_bytes", Value::make_number((double)lazy));
    Value ws = Value::make_array();
    for (const auto& it : items) {
        Value w = Value::make_object();
        w.set("name", Value::make_string(it.name));
        w.set("dtype", Value::make_string(it.dtype));
        w.set("shape", shape_json(it.shape));
        w.set("trainable", Value::make_bool(it.trainable));
        w.set("bytes", Value::make_number((double)it.bytes));
        w.set("device_bytes_per_shard", Value::make_number((double)it.dev_bytes));
        w.set("access_count", Value::make_number(it.access));
        w.set("residency", Value::make_string(it.residency));
        ws.push(w);
    }
    root.set("weights", ws);
    std::string text;
    mjson::write(root, &text);
    char* out = (char*)malloc(text.size() + 1);
    if (!out) return fail(err, "out of memory");
    memcpy(out, text.c_str(), text.size() + 1);
    *out_json = out;
    return 0;
}

/* WithMemoryPlan (applied at runtime.go:172-197): params whose residency is not device_resident are not kept on
 * the device between runs; they are bound for the run that needs them and released afterwards. */
int manta_b200_program_apply_memory_plan(MantaB200Program* prog, const char* plan_json, char** err) {
    if (!prog || !plan_json) return fail(err, "apply_memory_plan: NULL argument");
    Value root;
    std::string perr;
    const std::string plan_text(plan_json);
    mjson::Parser p(plan_text);
    if (!p.parse(&root, &perr)) return fail(err, "%s", perr.c_str());
    if (root.get_string("version") != "manta/memory/v0alpha1") return fail(err, "unsupported memory plan version \"%s\"", root.get_string("version").c_str());
    const Value* ws = root.get("weights");
    if (!ws) return fail(err, "memory plan has no weights");
    for (const auto& w : ws->items()) {
        const std::string name = w.get_string("name"), res = w.get_string("residency");
        if (res != "device_resident" && res != "host_pinned" && res != "host_shared" && res != "lazy_staged")
            return fail(err, "memory plan weight \"%s\" has unknown residency \"%s\"", name.c_str(), res.c_str());
        prog->residency[name] = res;
        auto it = prog->resident.find(name);
        if (res != "device_resident" && it != prog->resident.end()) {
            if (prog->rt && it->second.set) manta_b200_candidates_unbind(prog->rt, it->second.set, nullptr);
            prog->resident.erase(it);
        }
    }
    return 0;
}

int manta_b200_program_load(MantaB200Runtime* rt, const char* module_json, MantaB200Program** out, char** err) {
    if (!module_json || !out) return fail(err, "program_load: NULL argument");
    *out = nullptr;
    auto prog = std::make_unique<MantaB200Program>();
    std::string perr;
    if (!parse_module(module_json, &prog->mod, &perr)) return fail(err, "%s", perr.c_str());
    if (!validate_module(prog->mod, &perr)) return fail(err, "%s", perr.c_str());
    prog->rt = rt;
    *out = prog.release();
    return 0;
}

int manta_b200_program_bind_weight(MantaB200Program* prog, const MantaB200TensorArg* w, char** err) {
    if (!prog || !w || !w->name) return fail(err, "bind_weight: NULL argument");
    const Param* p = param_by_name(prog->mod, w->name);
    if (!p) return fail(err, "module does not declare param \"%s\"", w->name);
    std::string terr;
    TensorP t = tensor_from_arg(*w, &terr);
    if (!t) return fail(err, "param \"%s\": %s", w->name, terr.c_str());
    prog->weights[w->name] = t;
    auto it = prog->resident.find(w->name);
    if (it != prog->resident.end()) {  // a re-bound weight drops the resident copy
        if (prog->rt && it->second.set) manta_b200_candidates_unbind(prog->rt, it->second.set, nullptr);
        prog->resident.erase(it);
    }
    return 0;
}

int manta_b200_program_plan(MantaB200Program* prog, const char* entry, char** out_json, char** err) {
    if (!prog || !entry || !out_json) return fail(err, "program_plan: NULL argument");
    if (!entry_by_name(prog->mod, entry)) return fail(err, "unknown entrypoint \"%s\"", entry);
    auto steps = steps_for_entry(prog->mod, entry);
    if (steps.empty()) return fail(err, "entrypoint \"%s\" has no plan steps", entry);
    std::string text;
    mjson::write(fusion_json(steps, plan_fusions(prog->mod, steps)), &text);
    char* s = (char*)malloc(text.size() + 1);
    if (!s) return fail(err, "out of memory");
    memcpy(s, text.c_str(), text.size() + 1);
    *out_json = s;
    return 0;
}

int manta_b200_program_destroy(MantaB200Program* prog, char** err) {
    if (!prog) return 0;
    int rc = 0;
    for (auto& kv : prog->resident)
        if (prog->rt && kv.second.set) rc |= manta_b200_candidates_unbind(prog->rt, kv.second.set, err);
    delete prog;
    return rc;
}

void manta_b200_result_free(MantaB200Result* res) { delete res; }
const char* manta_b200_result_json(const MantaB200Result* res) { return res ? res->json.c_str() : ""; }

int manta_b200_result_tensor(const MantaB200Result* res, const char* output, const char* field, MantaB200TensorArg* view, char** err) {
    if (!res || !output || !view) return fail(err, "result_tensor: NULL argument");
    auto it = res->outputs.find(output);
    if (it == res->outputs.end()) return fail(err, "missing %s output", output);
    const Tensor* t = nullptr;
    const std::string f = field ? field : "";
    if (it->second.pack) {
        t = f == "ids" ? it->second.pack->ids.get() : f == "scores" ? it->second.pack->scores.get() : f == "docs" ? it->second.pack->docs.get() : nullptr;
        if (!t) return fail(err, "candidate pack field must be ids, scores or docs");
    } else {
        t = it->second.tensor.get();
    }
    if (!t) return fail(err, "output %s holds no tensor", output);
    view->name = it->first.c_str();
    view->dtype = t->dtype.c_str();
    view->rank = (int)t->shape.size();
    view->shape = t->shape.data();
    view->data = t->data();
    return 0;
}

int manta_b200_program_run(MantaB200Program* prog, const char* entry_name, const MantaB200TensorArg* inputs, int n_inputs,
                           MantaB200Result** out, char** err) {
    if (!prog || !entry_name || !out || (n_inputs > 0 && !inputs)) return fail(err, "program_run: NULL argument");
    *out = nullptr;
    if (!prog->rt) return fail(err, "program was loaded without a device runtime; this backend has no host fallback");
    const Module& mod = prog->mod;
    const EntryPoint* entry = entry_by_name(mod, entry_name);
    if (!entry) return fail(err, "unknown entrypoint \"%s\"", entry_name);
    // validateRequestInputs (symbolic.go:265-277)
    for (const auto& in : entry->inputs) {
        bool found = false;
        for (int i = 0; i < n_inputs; ++i) found = found || (inputs[i].name && in.name == inputs[i].name);
        if (!found) return fail(err, "entrypoint \"%s\" missing input \"%s\"", entry->name.c_str(), in.name.c_str());
    }
    for (int i = 0; i < n_inputs; ++i) {
        bool declared = false;
        for (const auto& in : entry->inputs) declared = declared || (inputs[i].name && in.name == inputs[i].name);
        if (!declared) return fail(err, "entrypoint \"%s\" does not declare input \"%s\"", entry->name.c_str(), inputs[i].name ? inputs[i].name : "");
    }

    std::map<std::string, int64_t> symbols;
    std::map<std::string, RValue> env;
    std::string terr;
    for (const auto& p : mod.params) {
        auto w = prog->weights.find(p.name);
        if (w == prog->weights.end()) return fail(err, "missing weight binding for param \"%s\"", p.name.c_str());
        if (!check_tensor(p.type, *w->second, &symbols, &terr)) return fail(err, "param \"%s\": %s", p.name.c_str(), terr.c_str());
        RValue v;
        v.type = p.type;
        v.tensor = w->second;
        v.producer = "param:" + p.name;
        v.metadata.set("materialized", Value::make_string("eager"));
        {
            auto rit = prog->residency.find(p.name);
            v.metadata.set("weight_residency", Value::make_string(rit == prog->residency.end() ? "device_resident" : rit->second));
        }
        env[p.name] = v;
    }
    for (const auto& in : entry->inputs) {
        for (int i = 0; i < n_inputs; ++i) {
            if (in.name != inputs[i].name) continue;
            TensorP t = tensor_from_arg(inputs[i], &terr);
            if (!t) return fail(err, "input \"%s\": %s", in.name.c_str(), terr.c_str());
            if (in.type.kind != "tensor") return fail(err, "input \"%s\": unsupported runtime value kind \"%s\"", in.name.c_str(), in.type.kind.c_str());
            if (!check_tensor(in.type, *t, &symbols, &terr)) return fail(err, "input \"%s\": %s", in.name.c_str(), terr.c_str());
            RValue v;
            v.type = in.type;
            v.tensor = t;
            v.producer = "input:" + in.name;
            env[in.name] = v;
        }
    }
    auto steps = steps_for_entry(mod, entry->name);
    if (steps.empty()) return fail(err, "entrypoint \"%s\" has no plan steps", entry->name.c_str());
    const std::vector<Fusion> fusions = plan_fusions(mod, steps);

    auto res = std::make_unique<MantaB200Result>();
    Value trace = Value::make_array();
    std::vector<BoundSet> temp_sets;  // docs that arrived as request inputs
    int temp_sets_released = 0;
    auto cleanup = [&]() {
        for (auto& b : temp_sets)
            if (b.set) {
                manta_b200_candidates_unbind(prog->rt, b.set, nullptr);
                b.set = nullptr;
                ++temp_sets_released;
            }
    };
    std::map<std::string, BoundSet> set_of_value;  // env name -> candidate set it is bound as
    // results of fused passes, keyed by the scores value name
    struct Fused {
        TensorP ids, top_scores;
        const Fusion* f;
    };
    std::map<std::string, Fused> fused;
    uint64_t launches_before = manta_b200_kernel_launch_count();

#define STEP_FAIL(...)                                                             \
    do {                                                                           \
        char* inner_ = nullptr;                                                    \
        fail(&inner_, __VA_ARGS__);                                                \
        int rc_ = fail(err, "entrypoint \"%s\" step \"%s\": %s", entry->name.c_str(), step.name.c_str(), inner_ ? inner_ : ""); \
        free(inner_);                                                              \
        cleanup();                                                                 \
        return rc_;                                                                \
    } while (0)

    for (size_t si = 0; si < steps.size(); ++si) {
        const Step& step = *steps[si];
        for (const auto& name : step.inputs)
            if (!env.count(name)) {
                cleanup();
                return fail(err, "entrypoint \"%s\" step \"%s\" missing runtime input \"%s\"", entry->name.c_str(), step.name.c_str(), name.c_str());
            }
        std::string variant_entry, source_hash;
        std::vector<RValue> produced;
        auto base_meta = [&](RValue* v) {
            v->metadata.set("backend", Value::make_string("cuda"));
            v->metadata.set("step", Value::make_string(step.kind));
            v->metadata.set("kernel", Value::make_string(step.kernel));
            v->metadata.set("variant_entry", Value::make_string(variant_entry));
            v->metadata.set("source_hash", Value::make_string(source_hash));
            v->producer = !step.kernel.empty() ? "kernel:" + step.kernel : (!step.name.empty() ? step.kind + ":" + step.name : step.kind);
            v->inputs = step.inputs;
        };
        auto device_meta = [&](RValue* v, const char* fused_steps) {
            v->metadata.set("device_execution", Value::make_bool(true));
            v->metadata.set("execution_mode", Value::make_string("device"));
            v->metadata.set("dispatch_mode", Value::make_string("backend_native"));
            v->metadata.set("launch_api", Value::make_string("cudaLaunchKernel"));
            v->metadata.set("launch_compiler", Value::make_string("nvcc-aot sm_100a"));
            v->metadata.set("fused_steps", Value::make_string(fused_steps));
        };
        auto out_type = [&](size_t idx, const Tensor& t) {
            ValueType vt;
            vt.kind = "tensor";
            vt.dtype = t.dtype;
            for (int64_t d : t.shape) vt.shape.push_back(std::to_string(d));
            (void)idx;
            return vt;
        };

        if (step.kind == "launch_kernel") {
            const Kernel* k = kernel_by_name(mod, step.kernel);
            if (!k) STEP_FAIL("unknown kernel \"%s\"", step.kernel.c_str());
            const Variant* var = cuda_variant(*k);
            variant_entry = var ? var->entry : "";
            source_hash = var ? mb200_host::sha256_hex(var->source) : "";  // CompileVariants, backend.go:286-293
            if (k->op == "dequant") {
                // kernel op dequant (tensor_ops.go:556-563): a clone relabelled f16; nothing to compute
                if (step.inputs.size() != 1 || step.outputs.size() != 1) STEP_FAIL("kernel \"%s\" expects 1 input and 1 output", k->name.c_str());
                const RValue& in = env[step.inputs[0]];
                if (!in.tensor) STEP_FAIL("value \"%s\" is not a tensor", step.inputs[0].c_str());
                RValue v;
                v.tensor = std::make_shared<Tensor>(*in.tensor);
                v.tensor->dtype = "f16";
                v.type = out_type(0, *v.tensor);
                base_meta(&v);
                v.metadata.set("execution_mode", Value::make_string("relabel"));
                produced.push_back(v);
            } else {
            if (!is_score_op(k->op)) STEP_FAIL("kernel op \"%s\" is outside the score/select path this backend implements", k->op.c_str());
            const Fusion* f = nullptr;
            for (const auto& c : fusions)
                if (c.score_step == (int)si) f = &c;
            if (!f) STEP_FAIL("score kernel expects 2 inputs and 1 output");
            const Tensor& query = *env[f->query_name].tensor;
            const Tensor& docs = *env[f->docs_name].tensor;
            // scoreLayout (tensor_ops.go:1492-1521) + the shared-candidate batch [Q,D] x [N,D]
            const bool rank1 = query.shape.size() == 1 && docs.shape.size() == 2;
            const bool shared = query.shape.size() == 2 && docs.shape.size() == 2;
            const bool per_query = query.shape.size() == 2 && docs.shape.size() == 3;
            if (!rank1 && !shared && !per_query) STEP_FAIL("score expects query/docs as [D] x [N,D] or [Q,D] x [Q,N,D]");
            if (per_query) {
                // [Q,D] x [Q,N,D]: every query against its own rows, streamed through the device for this call
                const int64_t bq = docs.shape[0], bn = docs.shape[1], bd = docs.shape[2];
                if (query.shape[0] != bq || query.shape[1] != bd) STEP_FAIL("score mismatch %s x %s", shape_text(query.shape).c_str(), shape_text(docs.shape).c_str());
                if (!float_like(query.dtype) || !float_like(docs.dtype)) STEP_FAIL("score inputs must be float-like tensors");
                const int metric = metric_of(k->op);
                RValue sv;
                auto t = std::make_shared<Tensor>();
                t->dtype = "f32";
                t->shape = {bq, bn};
                sv.tensor = t;
                if (f->need_full_scores) {
                    t->f32.resize((size_t)bq * bn);
                    char* serr = nullptr;
                    if (manta_b200_score_batched(prog->rt, metric, query.f32.data(), docs.f32.data(), (int)bq, bn, (int)bd, MANTA_B200_MEM_HOST,
                                                 t->f32.data(), &serr)) {
                        std::string m = serr ? serr : "score failed";
                        free(serr);
                        STEP_FAIL("%s", m.c_str());
                    }
                } else {
                    sv.metadata.set("materialized", Value::make_string("device_only"));
                }
                if (f->topk_step >= 0) {
                    const Step& ts = *steps[f->topk_step];
                    if (f->k <= 0) {
                        cleanup();
                        return fail(err, "entrypoint \"%s\" step \"%s\": topk step \"%s\" is missing limit attribute", entry->name.c_str(), ts.name.c_str(), ts.name.c_str());
                    }
                    Fused fu;
                    fu.f = f;
                    fu.ids = std::make_shared<Tensor>();
                    fu.top_scores = std::make_shared<Tensor>();
                    fu.ids->dtype = "i32";
                    fu.top_scores->dtype = "f32";
                    fu.ids->shape = fu.top_scores->shape = {bq, (int64_t)f->k};
                    fu.ids->i32.resize((size_t)bq * f->k);
                    fu.top_scores->f32.resize((size_t)bq * f->k);
                    char* serr = nullptr;
                    if (manta_b200_score_topk_batched(prog->rt, metric, MANTA_B200_ORDER_LARGEST, query.f32.data(), docs.f32.data(), (int)bq, bn,
                                                      (int)bd, MANTA_B200_MEM_HOST, f->k, fu.ids->i32.data(), fu.top_scores->f32.data(), &serr)) {
                        std::string m = serr ? serr : "score_topk failed";
                        free(serr);
                        cleanup();
                        return fail(err, "entrypoint \"%s\" step \"%s\": %s", entry->name.c_str(), ts.name.c_str(), m.c_str());
                    }
                    fused[f->scores_name] = fu;
                }
                sv.type = out_type(0, *sv.tensor);
                base_meta(&sv);
                device_meta(&sv, f->topk_step >= 0 ? "launch_kernel+topk+gather" : "launch_kernel");
                sv.metadata.set("candidate_sets", Value::make_string("per_query"));
                produced.push_back(sv);
            } else {
            const int64_t d = docs.shape[1], n = docs.shape[0];
            const int64_t qd = rank1 ? query.shape[0] : query.shape[1];
            const int nq = rank1 ? 1 : (int)query.shape[0];
            if (qd != d) STEP_FAIL("score mismatch %s x %s", shape_text(query.shape).c_str(), shape_text(docs.shape).c_str());
            if (!float_like(query.dtype) || !float_like(docs.dtype)) STEP_FAIL("score inputs must be float-like tensors");
            // candidate set: resident for params, bound for this call for request inputs
            BoundSet bs;
            // the set is bound from the value behind any dequant steps, with that value's own dtype label
            const std::string& bind_name = f->bind_name;
            const std::string bind_dtype = (env.count(bind_name) && env[bind_name].tensor) ? env[bind_name].tensor->dtype : docs.dtype;
            auto rit = prog->residency.find(bind_name);
            const bool keep_resident = rit == prog->residency.end() || rit->second.empty() || rit->second == "device_resident";
            if (param_by_name(mod, bind_name) && keep_resident) {
                auto it = prog->resident.find(bind_name);
                if (it == prog->resident.end()) {
                    char* berr = nullptr;
                    if (bind_docs(prog->rt, docs.f32.data(), n, (int)d, bind_dtype, &bs, &berr)) {
                        std::string m = berr ? berr : "bind failed";
                        free(berr);
                        STEP_FAIL("%s", m.c_str());
                    }
                    prog->resident[bind_name] = bs;
                } else {
                    bs = it->second;
                }
            } else {
                char* berr = nullptr;
                if (bind_docs(prog->rt, docs.f32.data(), n, (int)d, bind_dtype, &bs, &berr)) {
                    std::string m = berr ? berr : "bind failed";
                    free(berr);
                    STEP_FAIL("%s", m.c_str());
                }
                temp_sets.push_back(bs);
            }
            set_of_value[f->docs_name] = bs;
            set_of_value[bind_name] = bs;
            std::vector<uint16_t> qbits((size_t)nq * bs.stored_cols, 0);
            for (int q = 0; q < nq; ++q)
                for (int64_t c = 0; c < d; ++c) qbits[(size_t)q * bs.stored_cols + c] = half_bits(query.f32[(size_t)q * d + c]);
            const int metric = metric_of(k->op);
            RValue sv;
            if (f->need_full_scores) {
                auto t = std::make_shared<Tensor>();
                t->dtype = "f32";
                t->shape = rank1 ? std::vector<int64_t>{n} : std::vector<int64_t>{nq, n};
                t->f32.resize((size_t)nq * n);
                char* serr = nullptr;
                if (manta_b200_score(prog->rt, bs.set, metric, qbits.data(), nq, t->f32.data(), &serr)) {
                    std::string m = serr ? serr : "score failed";
                    free(serr);
                    STEP_FAIL("%s", m.c_str());
                }
                sv.tensor = t;
            } else {
                // the full score vector is never read outside the fused pass: it stays on the device
                auto t = std::make_shared<Tensor>();
                t->dtype = "f32";
                t->shape = rank1 ? std::vector<int64_t>{n} : std::vector<int64_t>{nq, n};
                sv.tensor = t;
                sv.metadata.set("materialized", Value::make_string("device_only"));
            }
            if (f->topk_step >= 0) {
                if (f->k <= 0) {
                    const Step& ts = *steps[f->topk_step];
                    cleanup();
                    return fail(err, "entrypoint \"%s\" step \"%s\": topk step \"%s\" is missing limit attribute", entry->name.c_str(), ts.name.c_str(), ts.name.c_str());
                }
                Fused fu;
                fu.f = f;
                fu.ids = std::make_shared<Tensor>();
                fu.top_scores = std::make_shared<Tensor>();
                fu.ids->dtype = "i32";
                fu.top_scores->dtype = "f32";
                fu.ids->shape = fu.top_scores->shape = rank1 ? std::vector<int64_t>{f->k} : std::vector<int64_t>{nq, f->k};
                fu.ids->i32.resize((size_t)nq * f->k);
                fu.top_scores->f32.resize((size_t)nq * f->k);
                char* serr = nullptr;
                if (manta_b200_score_topk(prog->rt, bs.set, metric, MANTA_B200_ORDER_LARGEST, qbits.data(), nq, f->k, fu.ids->i32.data(),
                                          fu.top_scores->f32.data(), &serr)) {
                    std::string m = serr ? serr : "score_topk failed";
                    free(serr);
                    // topKTensor's error belongs to the topk step in the reference's trace of errors
                    const Step& ts = *steps[f->topk_step];
                    cleanup();
                    return fail(err, "entrypoint \"%s\" step \"%s\": %s", entry->name.c_str(), ts.name.c_str(), m.c_str());
                }
                fused[f->scores_name] = fu;
            }
            sv.type = out_type(0, *sv.tensor);
            base_meta(&sv);
            device_meta(&sv, f->topk_step >= 0 ? "launch_kernel+topk+gather" : "launch_kernel");
            produced.push_back(sv);
            }  // shared / rank-1 candidate set
            {
                // nativeLaunchConfig (native_kernel.go:65-112): the plan-side keys as the reference derives them from
                // the variant, the launch_* keys from the kernel that really ran
                RValue& sv = produced.back();
                MantaB200LaunchInfo li{};
                manta_b200_runtime_last_launch(prog->rt, &li, nullptr);
                auto meta_of = [&](const char* key) {
                    if (!var) return std::string();
                    auto it = var->meta.find(key);
                    return it == var->meta.end() ? std::string() : it->second;
                };
                const int tile = var ? first_tile_size(*k, *var) : 1;
                sv.metadata.set("dispatch_backend", Value::make_string("cuda"));
                sv.metadata.set("launch_entry", Value::make_string(variant_entry));
                sv.metadata.set("launch_tile", Value::make_string(meta_of("tile")));
                sv.metadata.set("launch_tile_2d", Value::make_string(meta_of("tile_2d")));
                sv.metadata.set("launch_vector_width", Value::make_string(meta_of("vector_width")));
                sv.metadata.set("launch_memory", Value::make_string(meta_of("memory")));
                sv.metadata.set("launch_subgroup", Value::make_string(meta_of("subgroup")));
                sv.metadata.set("launch_subgroup_2d", Value::make_string(meta_of("subgroup_2d")));
                sv.metadata.set("launch_halo", Value::make_string(meta_of("halo")));
                sv.metadata.set("plan_block_size", Value::make_number(tile));
                sv.metadata.set("plan_shared_bytes", Value::make_number(estimated_shared_bytes(*k, tile)));
                sv.metadata.set("launch_grid", Value::make_string("1d"));
                sv.metadata.set("launch_kernel", Value::make_string(li.kernel));
                sv.metadata.set("launch_grid_size", Value::make_number(li.grid));
                sv.metadata.set("launch_block_size", Value::make_number(li.block));
                sv.metadata.set("launch_shared_bytes", Value::make_number(li.shared_bytes));
                sv.metadata.set("launch_count", Value::make_number(li.launches));
            }
            }  // score op
        } else if (step.kind == "dequant") {
            // StepDequant (tensor_ops.go:136-148): a clone of the input relabelled f16, values unchanged
            if (step.inputs.size() != 1 || step.outputs.size() != 1) STEP_FAIL("dequant step \"%s\" expects 1 input and 1 output", step.name.c_str());
            const RValue& in = env[step.inputs[0]];
            if (!in.tensor) STEP_FAIL("value \"%s\" is not a tensor", step.inputs[0].c_str());
            RValue v;
            v.tensor = std::make_shared<Tensor>(*in.tensor);
            if (v.tensor->dtype != "f16") v.tensor->dtype = "f16";
            v.type = out_type(0, *v.tensor);
            base_meta(&v);
            v.metadata.set("execution_mode", Value::make_string("relabel"));
            produced.push_back(v);
        } else if (step.kind == "topk") {
            if (step.inputs.size() != 1 || step.outputs.size() != 1) STEP_FAIL("topk step \"%s\" expects 1 input and 1 output", step.name.c_str());
            auto it = fused.find(step.inputs[0]);
            if (it == fused.end() || it->second.f->topk_step != (int)si)
                STEP_FAIL("topk over a value that no score kernel of this entry point produced is not on the device path");
            RValue v;
            v.tensor = it->second.ids;
            v.type = out_type(0, *v.tensor);
            base_meta(&v);
            device_meta(&v, "launch_kernel+topk+gather");
            produced.push_back(v);
        } else if (step.kind == "gather") {
            if (step.inputs.size() != 2 || step.outputs.size() != 1) STEP_FAIL("gather step \"%s\" expects 2 inputs and 1 output", step.name.c_str());
            const RValue& table = env[step.inputs[0]];
            const RValue& index = env[step.inputs[1]];
            if (!table.tensor || !index.tensor) STEP_FAIL("gather expects tensor inputs");
            if (index.tensor->dtype != "i32") STEP_FAIL("gather expects i32 indices");
            RValue v;
            auto fit = fused.find(step.inputs[0]);
            bool done = false;
            if (fit != fused.end() && fit->second.f->ids_name == step.inputs[1]) {
                v.tensor = fit->second.top_scores;  // gather(scores, ids) came out of the fused pass
                base_meta(&v);
                device_meta(&v, "launch_kernel+topk+gather");
                done = true;
            }
            auto sit = set_of_value.find(step.inputs[0]);
            if (!done && sit != set_of_value.end() && index.tensor->shape.size() <= 2) {
                // gather(docs, ids): de-quantised rows of the bound set, labelled with the table's dtype
                const BoundSet& bs = sit->second;
                const int64_t cnt = index.tensor->elements();
                std::vector<float> rows((size_t)cnt * bs.stored_cols);
                char* gerr = nullptr;
                if (manta_b200_gather_rows(prog->rt, bs.set, index.tensor->i32.data(), cnt, rows.data(), &gerr)) {
                    std::string m = gerr ? gerr : "gather failed";
                    free(gerr);
                    STEP_FAIL("%s", m.c_str());
                }
                auto t = std::make_shared<Tensor>();
                t->dtype = table.tensor->dtype;
                t->shape = index.tensor->shape;
                t->shape.push_back(bs.cols);
                t->f32.resize((size_t)cnt * bs.cols);
                for (int64_t r = 0; r < cnt; ++r) memcpy(&t->f32[(size_t)r * bs.cols], &rows[(size_t)r * bs.stored_cols], (size_t)bs.cols * 4);
                v.tensor = t;
                base_meta(&v);
                device_meta(&v, "gather");
                done = true;
            }
            if (!done) {
                // gatherTensor on a host table (candidate_ids and the like), tensor_ops.go:761-827
                const Tensor& tb = *table.tensor;
                const Tensor& ix = *index.tensor;
                auto t = std::make_shared<Tensor>();
                t->dtype = tb.dtype;
                auto copy_elems = [&](size_t src, size_t count) {
                    if (tb.dtype == "i32") t->i32.insert(t->i32.end(), tb.i32.begin() + src, tb.i32.begin() + src + count);
                    else if (tb.dtype == "i64") t->i64.insert(t->i64.end(), tb.i64.begin() + src, tb.i64.begin() + src + count);
                    else t->f32.insert(t->f32.end(), tb.f32.begin() + src, tb.f32.begin() + src + count);
                };
                if (tb.shape.size() == 1 && ix.shape.size() == 1) {
                    t->shape = {ix.shape[0]};
                    for (int32_t id : ix.i32) {
                        if (id < 0 || id >= tb.shape[0]) STEP_FAIL("gather index %d out of range", id);
                        copy_elems((size_t)id, 1);
                    }
                } else if (tb.shape.size() == 2 && ix.shape.size() == 1) {
                    const int64_t cols = tb.shape[1];
                    t->shape = {ix.shape[0], cols};
                    for (int32_t id : ix.i32) {
                        if (id < 0 || id >= tb.shape[0]) STEP_FAIL("gather index %d out of range", id);
                        copy_elems((size_t)id * cols, (size_t)cols);
                    }
                } else if (tb.shape.size() == 2 && ix.shape.size() == 2) {
                    // batched element gather [Q,N] x [Q,k] -> [Q,k] (tensor_ops.go:875-925)
                    if (tb.shape[0] != ix.shape[0]) STEP_FAIL("gather batch mismatch %s x %s", shape_text(tb.shape).c_str(), shape_text(ix.shape).c_str());
                    const int64_t rows = tb.shape[1], kk = ix.shape[1];
                    t->shape = {ix.shape[0], kk};
                    for (int64_t b = 0; b < ix.shape[0]; ++b)
                        for (int64_t i = 0; i < kk; ++i) {
                            const int32_t id = ix.i32[(size_t)(b * kk + i)];
                            if (id < 0 || id >= rows) STEP_FAIL("gather index %d out of range", id);
                            copy_elems((size_t)(b * rows + id), 1);
                        }
                } else if (tb.shape.size() == 3 && ix.shape.size() == 2) {
                    // batched row gather [Q,N,D] x [Q,k] -> [Q,k,D] (tensor_ops.go:926-975)
                    if (tb.shape[0] != ix.shape[0]) STEP_FAIL("gather batch mismatch %s x %s", shape_text(tb.shape).c_str(), shape_text(ix.shape).c_str());
                    const int64_t rows = tb.shape[1], cols = tb.shape[2], kk = ix.shape[1];
                    t->shape = {ix.shape[0], kk, cols};
                    for (int64_t b = 0; b < ix.shape[0]; ++b)
                        for (int64_t i = 0; i < kk; ++i) {
                            const int32_t id = ix.i32[(size_t)(b * kk + i)];
                            if (id < 0 || id >= rows) STEP_FAIL("gather index %d out of range", id);
                            copy_elems((size_t)((b * rows + id) * cols), (size_t)cols);
                        }
                } else {
                    STEP_FAIL("gather expects table rank 1, 2, or 3 with compatible indices");
                }
                v.tensor = t;
                base_meta(&v);
                v.metadata.set("execution_mode", Value::make_string("host_index"));
            }
            v.type = out_type(0, *v.tensor);
            produced.push_back(v);
        } else if (step.kind == "pack_candidates") {
            if (step.inputs.size() != 3 || step.outputs.size() != 1) STEP_FAIL("pack_candidates step \"%s\" expects 3 inputs and 1 output", step.name.c_str());
            RValue v;
            v.pack = std::make_shared<Pack>();
            v.pack->ids = env[step.inputs[0]].tensor;
            v.pack->scores = env[step.inputs[1]].tensor;
            v.pack->docs = env[step.inputs[2]].tensor;
            if (!v.pack->ids || !v.pack->scores || !v.pack->docs) STEP_FAIL("candidate pack requires ids, scores, and docs");
            // validateCandidatePackType, tensor.go:405-444
            if (v.pack->ids->dtype != "i64") STEP_FAIL("candidate pack ids dtype \"%s\" does not match expected \"i64\"", v.pack->ids->dtype.c_str());
            if (v.pack->scores->dtype != "f32") STEP_FAIL("candidate pack scores dtype \"%s\" does not match expected \"f32\"", v.pack->scores->dtype.c_str());
            if (v.pack->docs->dtype != "q4") STEP_FAIL("candidate pack docs dtype \"%s\" does not match expected \"q4\"", v.pack->docs->dtype.c_str());
            if (v.pack->docs->shape.size() == 2 && (v.pack->ids->shape.size() != 1 || v.pack->ids->shape[0] != v.pack->docs->shape[0] || v.pack->scores->shape[0] != v.pack->docs->shape[0]))
                STEP_FAIL("candidate pack leading dimension mismatch");
            if (v.pack->docs->shape.size() == 3) {
                if (v.pack->ids->shape.size() != 2 || v.pack->scores->shape.size() != 2) STEP_FAIL("candidate pack rank-3 docs require rank-2 ids and scores");
                if (v.pack->ids->shape[0] != v.pack->docs->shape[0] || v.pack->scores->shape[0] != v.pack->docs->shape[0] ||
                    v.pack->ids->shape[1] != v.pack->docs->shape[1] || v.pack->scores->shape[1] != v.pack->docs->shape[1])
                    STEP_FAIL("candidate pack leading dimensions mismatch");
            }
            v.type.kind = "candidate_pack";
            for (int64_t dd : v.pack->docs->shape) v.type.shape.push_back(std::to_string(dd));
            base_meta(&v);
            produced.push_back(v);
        } else if (step.kind == "return") {
            for (const auto& name : step.outputs) {
                auto it = env.find(name);
                if (it == env.end()) {
                    cleanup();
                    return fail(err, "entrypoint \"%s\" return references unknown value \"%s\"", entry->name.c_str(), name.c_str());
                }
                if (it->second.tensor && it->second.tensor->elements() > 0 && it->second.tensor->f32.empty() && it->second.tensor->i32.empty() && it->second.tensor->i64.empty()) {
                    cleanup();
                    return fail(err, "entrypoint \"%s\" return references value \"%s\" that was kept on the device", entry->name.c_str(), name.c_str());
                }
                res->outputs[name] = it->second;
            }
        } else {
            STEP_FAIL("step kind \"%s\" is outside the score/select path this backend implements", step.kind.c_str());
        }
        Value tr = Value::make_object();
        tr.set("entry", Value::make_string(step.entry));
        tr.set("kind", Value::make_string(step.kind));
        tr.set("name", Value::make_string(step.name));
        tr.set("kernel", Value::make_string(step.kernel));
        tr.set("variant", Value::make_string(variant_entry));
        tr.set("inputs", strings_json(step.inputs));
        tr.set("outputs", strings_json(step.outputs));
        trace.push(tr);
        if (step.kind != "return") {
            if (produced.size() < step.outputs.size()) STEP_FAIL("step produced %d values for %d outputs", (int)produced.size(), (int)step.outputs.size());
            for (size_t i = 0; i < step.outputs.size(); ++i) env[step.outputs[i]] = produced[i];
        }
    }
#undef STEP_FAIL
    cleanup();
    if (res->outputs.empty()) return fail(err, "entrypoint \"%s\" produced no outputs", entry->name.c_str());

    // ---- describe the result
    Value root = Value::make_object();
    Value outs = Value::make_object();
    for (const auto& kv : res->outputs) {
        Value o = Value::make_object();
        o.set("kind", Value::make_string(kv.second.type.kind));
        if (kv.second.tensor) {
            o.set("dtype", Value::make_string(kv.second.tensor->dtype));
            o.set("shape", shape_json(kv.second.tensor->shape));
        } else if (kv.second.pack) {
            o.set("shape", shape_json(kv.second.pack->docs->shape));
        }
        o.set("producer", Value::make_string(kv.second.producer));
        o.set("inputs", strings_json(kv.second.inputs));
        o.set("metadata", kv.second.metadata);
        outs.set(kv.first, o);
    }
    root.set("outputs", outs);
    root.set("trace", trace);
    int score_kernels = 0;
    for (const auto& k : mod.kernels) score_kernels += is_score_op(k.op) ? 1 : 0;
    Value md = Value::make_object();
    md.set("backend", Value::make_string("cuda"));
    md.set("status", Value::make_string("device"));
    md.set("kernel_dispatch", Value::make_string("backend_native"));
    md.set("weight_bindings", Value::make_string(std::to_string(prog->weights.size())));
    md.set("compiled_kernels", Value::make_string(std::to_string(mod.kernels.size())));
    md.set("entrypoint", Value::make_string(entry->name));
    md.set("step_count", Value::make_string(std::to_string(steps.size())));
    md.set("params_total", Value::make_string(std::to_string(mod.params.size())));
    md.set("params_eager_materialized", Value::make_string(std::to_string(mod.params.size())));
    md.set("fused_passes", Value::make_string(std::to_string(fused.size())));
    md.set("params_released", Value::make_string(std::to_string(temp_sets_released)));
    md.set("device_kernel_launches", Value::make_string(std::to_string(manta_b200_kernel_launch_count() - launches_before)));
    root.set("metadata", md);
    mjson::write(root, &res->json);
    prog->runs++;
    *out = res.release();
    return 0;
}

}  // extern "C"
