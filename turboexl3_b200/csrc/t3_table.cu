// The quant-plugin table (include/t3_table.h) over the C ABI: claim / validate / open / load / matmul / swiglu with the
// reference table's member names, claim rules and refusal texts (turboexl3 table/table.zig, table/config.zig). Weights
// are uploaded once at load; activations may live in host memory, in which case the call stages them through device
// buffers the table keeps and returns once the result is back on the host.
#include <cmath>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/t3.h"
#include "../../include/t3_table.h"
#include "t3_json.h"

namespace {

using t3json::Json;
using t3json::JsonReader;

bool parse_object(const char* text, Json& out) {
    if (!text) return false;
    JsonReader r{text, text + strlen(text)};
    out = r.value();
    r.skip();
    return r.ok && r.p == r.end && out.kind == Json::kObject;
}

// ---- the claimed block (table/config.zig:13-44) ------------------------------------------------------------------------

enum class Kind { trunk, bank };
struct Block {
    Kind kind = Kind::trunk;
    int codebook = T3_MUL1;
    int window_bits = 16;
    uint32_t n = 0;
};

// a block's kind: `format` exl3; a bank block declares its rate `k`, a trunk block does not (config.zig:78-83)
bool kind_of(const Json& o, Kind& kind) {
    const Json* f = o.get("format");
    if (!f || f->kind != Json::kString || f->s != "exl3") return false;
    kind = o.get("k") ? Kind::bank : Kind::trunk;
    return true;
}

// `k` as halfwords per tile: an even whole number in 16..128 (config.zig:85-96)
bool rate_of(const Json& k, uint32_t& n) {
    if (k.kind != Json::kInt && k.kind != Json::kFloat) return false;
    const double scaled = k.f * 16.0, r = std::round(scaled);
    if (std::fabs(scaled - r) > 1e-6 || r < 16 || r > 128) return false;
    const uint32_t whole = (uint32_t)r;
    if (whole % 2) return false;
    n = whole;
    return true;
}

// null = parsed; otherwise the refusal's name (config.zig:31-44)
const char* parse_block(const char* json, Block& b) {
    Json o;
    if (!parse_object(json, o)) return "NotExl3";
    if (!kind_of(o, b.kind)) return "NotExl3";
    if (const Json* c = o.get("codebook")) {
        if (c->kind != Json::kString) return "Exl3CodebookUnsupported";
        if (c->s == "mul1") b.codebook = T3_MUL1;
        else if (c->s == "mcg") b.codebook = T3_MCG;
        else return "Exl3CodebookUnsupported";
    } else if (b.kind == Kind::bank) {
        return "Exl3CodebookUnsupported";
    }
    if (const Json* w = o.get("window")) {
        if (w->kind != Json::kInt || w->i < 8 || w->i > 16) return "Exl3WindowUnsupported";
        b.window_bits = (int)w->i;
    }
    if (b.kind == Kind::bank && !rate_of(*o.get("k"), b.n)) return "Exl3RateUnsupported";
    return nullptr;
}

const Json* text_of(const Json* cfg) {  // config.zig:131-135
    if (!cfg) return nullptr;
    const Json* t = cfg->get("text_config");
    return (t && t->kind == Json::kObject) ? t : cfg;
}

bool profile(const Json* cfg) {  // config.zig:98-112: a fully EXL3 pack of the model family the numerics were measured on
    if (!cfg || !cfg->get("trunk_quant")) return false;
    for (const Json* o : {cfg, text_of(cfg)}) {
        const Json* mt = o ? o->get("model_type") : nullptr;
        if (mt && mt->kind == Json::kString && (mt->s == "qwen4_exp" || mt->s == "qwen4_exp_text")) return true;
    }
    return false;
}

bool clamped(const Json* cfg) {  // config.zig:116-127
    for (const Json* o : {cfg, text_of(cfg)}) {
        const Json* v = o ? o->get("swiglu_limit") : nullptr;
        if (v && (v->kind == Json::kInt || v->kind == Json::kFloat) && v->f > 0) return true;
    }
    return false;
}

t3_verdict ok() { return {T3_VERDICT_OK, nullptr}; }
t3_verdict refuse(int kind, const char* why) { return {kind, why}; }
// table/table.zig:591-593: a missing weight fails, every other refusal is "unsupported", named by the error
t3_verdict from_status(int status) {
    if (status == T3_OK) return ok();
    return refuse(status == T3_CUDA_ERROR || status == T3_NULL_POINTER ? T3_VERDICT_FAILED : T3_VERDICT_UNSUPPORTED,
                  t3_status_name(status));
}

int table_claims(const char* block_json, const char* config_json) {
    Json o;
    if (!parse_object(block_json, o)) return T3_CLAIM_NO;
    Kind kind;
    if (!kind_of(o, kind)) return T3_CLAIM_NO;
    if (kind == Kind::trunk) return T3_CLAIM_BY_MARKER;
    Block b;
    if (parse_block(block_json, b)) return T3_CLAIM_NO;
    Json cfg;
    const bool have = parse_object(config_json, cfg);
    // the reference also asks for its host GPU's matrix-unit gate (kit/nax.zig); this backend's tensor-core path always exists
    if (!profile(have ? &cfg : nullptr) || clamped(have ? &cfg : nullptr)) return T3_CLAIM_NO;
    return T3_CLAIM_BY_MARKER;
}

t3_verdict table_validate(const char* block_json, const char* config_json) {
    Block b;
    if (const char* why = parse_block(block_json, b)) return refuse(T3_VERDICT_UNSUPPORTED, why);
    if (b.kind == Kind::bank) {
        Json cfg;
        if (parse_object(config_json, cfg)) {
            const Json* k = text_of(&cfg)->get("num_experts_per_tok");
            if (k && k->kind == Json::kInt && k->i > T3_REDUCE_MAX_TOPK) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TopKExceedsReduceBank");
        }
    }
    return ok();
}

uint64_t table_bill(const char*, const char*, uint64_t stored) { return stored; }  // the arrays as stored

struct State {
    Kind kind;
    t3_decode dec;
    uint32_t n;
};

t3_verdict table_open(t3_load_ctx* ctx) {
    if (!ctx) return refuse(T3_VERDICT_FAILED, "turboexl3: no load context");
    Block b;
    if (const char* why = parse_block(ctx->block_json, b)) return refuse(T3_VERDICT_UNSUPPORTED, why);
    State* st = new (std::nothrow) State{b.kind, {b.codebook, b.window_bits}, b.n};
    if (!st) return refuse(T3_VERDICT_FAILED, "turboexl3: out of memory");
    ctx->state = st;
    return ok();
}

void table_close(t3_load_ctx* ctx) {
    if (!ctx) return;
    delete static_cast<State*>(ctx->state);
    ctx->state = nullptr;
}

// ---- device memory the table owns ------------------------------------------------------------------------------------

size_t elem_size(int dt) {
    switch (dt) {
        case T3_A_F32: case T3_A_I32: case T3_A_U32: return 4;
        default: return 2;
    }
}
size_t count_of(const t3_array* a) {
    size_t c = 1;
    for (int i = 0; i < a->ndim; ++i) c *= (size_t)(a->shape[i] > 0 ? a->shape[i] : 0);
    return c;
}

// one array to the device (or a device-to-device copy, so the weight owns its memory either way)
bool upload(const t3_array* a, void** out, size_t* bytes) {
    const size_t n = count_of(a) * elem_size(a->dtype);
    void* d = nullptr;
    if (cudaMalloc(&d, n ? n : 1) != cudaSuccess) return false;
    if (cudaMemcpy(d, a->data, n, a->device ? cudaMemcpyDeviceToDevice : cudaMemcpyHostToDevice) != cudaSuccess) {
        cudaFree(d);
        return false;
    }
    *out = d;
    *bytes += n;
    return true;
}

void table_release(t3_weight* w) {
    if (!w) return;
    cudaFree(w->w);
    cudaFree(w->scales);
    cudaFree(w->biases);
    memset(w, 0, sizeof *w);
}

t3_verdict fill(t3_weight* out, const t3_array* t, const t3_array* suh, const t3_array* svh, t3_decode dec, int n,
                int experts, int in_dim, int out_dim) {
    memset(out, 0, sizeof *out);
    if (!upload(t, &out->w, &out->bytes) || !upload(suh, &out->scales, &out->bytes) ||
        !upload(svh, &out->biases, &out->bytes)) {
        table_release(out);
        return refuse(T3_VERDICT_FAILED, "CudaError");
    }
    out->layout = dec.codebook;
    out->flags = dec.window_bits;
    out->block = n;
    out->experts = experts;
    out->in_dim = in_dim;
    out->out_dim = out_dim;
    return ok();
}

bool present(const t3_array* a) { return a && a->data; }
bool rate_ok(int64_t n) { return n >= 16 && n <= 128 && n % 2 == 0; }

// table/table.zig:119-145
t3_verdict table_load_tensor(const t3_load_ctx* ctx, const t3_array* t, const t3_array* suh, const t3_array* svh,
                             uint32_t in_dim, t3_weight* out) {
    const State* st = ctx ? static_cast<const State*>(ctx->state) : nullptr;
    if (!st) return refuse(T3_VERDICT_FAILED, "turboexl3: the format is not open");
    if (st->kind != Kind::trunk) return refuse(T3_VERDICT_UNSUPPORTED, "turboexl3: dense linears load under the trunk_quant block");
    if (!out || !present(t) || !present(suh) || !present(svh)) return refuse(T3_VERDICT_FAILED, "MissingWeight");
    if (t->ndim != 3 || (t->dtype != T3_A_U16 && t->dtype != T3_A_I16) || t->shape[0] <= 0 || t->shape[1] <= 0)
        return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TrellisGeometry");
    if (!rate_ok(t->shape[2])) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3RateUnsupported");
    const int64_t in = t->shape[0] * 16, width = t->shape[1] * 16;
    if (in % 128 || width % 128) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3WidthNotMultipleOf128");
    if (in_dim != 0 && in_dim != (uint32_t)in) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TrellisGeometry");
    if (suh->ndim != 1 || suh->shape[0] != in || svh->ndim != 1 || svh->shape[0] != width)
        return refuse(T3_VERDICT_UNSUPPORTED, "Exl3SideGeometry");
    if (suh->dtype != T3_A_F16 || svh->dtype != T3_A_F16) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3SideDtype");
    return fill(out, t, suh, svh, st->dec, (int)t->shape[2], 0, (int)in, (int)width);
}

// table/table.zig:147-172
t3_verdict table_load_bank(const t3_load_ctx* ctx, const t3_array* t, const t3_array* suh, const t3_array* svh,
                           uint32_t in_dim, t3_weight* out) {
    const State* st = ctx ? static_cast<const State*>(ctx->state) : nullptr;
    if (!st) return refuse(T3_VERDICT_FAILED, "turboexl3: the format is not open");
    if (st->kind != Kind::bank) return refuse(T3_VERDICT_UNSUPPORTED, "turboexl3: routed banks load under the expert_quant block");
    if (!out || !present(t) || !present(suh) || !present(svh)) return refuse(T3_VERDICT_FAILED, "MissingWeight");
    if (t->ndim != 4 || t->shape[0] <= 0 || t->shape[1] <= 0 || t->shape[2] <= 0) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TrellisGeometry");
    const uint32_t experts = (uint32_t)t->shape[0], in = (uint32_t)t->shape[1] * 16u, width = (uint32_t)t->shape[2] * 16u;
    if (in_dim != 0 && in_dim != in) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TrellisGeometry");
    if (!st->n) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3RateUnsupported");
    const int shape[4] = {(int)t->shape[0], (int)t->shape[1], (int)t->shape[2], (int)t->shape[3]};
    if (t->dtype != T3_A_U16 || !t3_trellis_admitted(shape, 4, experts, in, width, st->n))
        return refuse(T3_VERDICT_UNSUPPORTED, "Exl3TrellisGeometry");
    if (suh->ndim != 2 || suh->shape[0] != experts || suh->shape[1] != in || svh->ndim != 2 || svh->shape[0] != experts ||
        svh->shape[1] != width)
        return refuse(T3_VERDICT_UNSUPPORTED, "Exl3SideGeometry");
    if (suh->dtype != T3_A_F16 || svh->dtype != T3_A_F16) return refuse(T3_VERDICT_UNSUPPORTED, "Exl3SideDtype");
    return fill(out, t, suh, svh, st->dec, (int)t->shape[3], (int)experts, (int)in, (int)width);
}

// Staging buffers that only grow: activations in, results out, routing (one set per process; a host-array call that uses
// them holds the lock until its result is back on the host) and the engine workspaces, which are kept PER STREAM: a call on
// device arrays returns with its kernels still in flight, and a call on another stream must not write the same scratch.
struct Staging {
    std::mutex mu;
    int device = -1;  // the device whose memory the buffers are: a call with another device current is refused, never run
    bool owns_current() {
        int dev = -1;
        if (cudaGetDevice(&dev) != cudaSuccess) return false;
        if (device < 0) device = dev;
        return device == dev;
    }
    struct Buf {
        void* p = nullptr;
        size_t cap = 0;
    } x, y, inds, scores;
    // ws: the prefill and routed workspaces (written before they are read). rows: the decode-row linear's workspace, which
    // must start zero and is left zero-tagged by every call (t3_linear), so it is cleared when it is (re)allocated and
    // nothing else ever writes it.
    struct StreamWs {
        Buf ws, rows;
    };
    std::unordered_map<void*, StreamWs> per_stream;
    StreamWs& of(void* stream) { return per_stream[stream]; }
    bool fit_zeroed(Buf& b, size_t bytes) {
        if (bytes <= b.cap) return true;
        if (!fit(b, bytes)) return false;
        return cudaMemset(b.p, 0, b.cap) == cudaSuccess;
    }
    bool fit(Buf& b, size_t bytes) {
        if (bytes <= b.cap) return true;
        cudaFree(b.p);
        b.p = nullptr;
        b.cap = 0;
        const size_t want = (bytes + 0xFFFFu) & ~(size_t)0xFFFFu;
        if (cudaMalloc(&b.p, want) != cudaSuccess) return false;
        b.cap = want;
        return true;
    }
    // Small host calls skip the copy engine: a pair of pinned, device-mapped host buffers the kernels read x from and write
    // y to directly (the bytes cross the bus inside the kernel), filled and drained by plain memcpy.
    static constexpr size_t kMappedBytes = 128u * 1024u;
    void *hx = nullptr, *hy = nullptr, *hx_dev = nullptr, *hy_dev = nullptr;
    bool mapped() {
        if (hx && hy) return true;
        if (cudaHostAlloc(&hx, kMappedBytes, cudaHostAllocMapped) != cudaSuccess ||
            cudaHostAlloc(&hy, kMappedBytes, cudaHostAllocMapped) != cudaSuccess ||
            cudaHostGetDevicePointer(&hx_dev, hx, 0) != cudaSuccess || cudaHostGetDevicePointer(&hy_dev, hy, 0) != cudaSuccess) {
            cudaFreeHost(hx);
            cudaFreeHost(hy);
            hx = hy = hx_dev = hy_dev = nullptr;
            cudaGetLastError();
            return false;
        }
        return true;
    }
    size_t bytes() {
        size_t total = x.cap + y.cap + inds.cap + scores.cap + (hx ? 2u * kMappedBytes : 0u);
        for (auto& kv : per_stream) total += kv.second.ws.cap + kv.second.rows.cap;
        return total;
    }
    void release() {
        for (Buf* b : {&x, &y, &inds, &scores}) {
            cudaFree(b->p);
            b->p = nullptr;
            b->cap = 0;
        }
        for (auto& kv : per_stream) {
            cudaFree(kv.second.ws.p);
            cudaFree(kv.second.rows.p);
        }
        per_stream.clear();
        device = -1;
        cudaFreeHost(hx);
        cudaFreeHost(hy);
        hx = hy = hx_dev = hy_dev = nullptr;
    }
} g_staging;

bool act_dtype(int dt) { return dt == T3_A_F32 || dt == T3_A_F16 || dt == T3_A_BF16; }

// the device address of an input: itself, or a staged copy
bool stage_in(const t3_array* a, Staging::Buf& buf, size_t bytes, cudaStream_t s, const void** out) {
    if (a->device) {
        *out = a->data;
        return true;
    }
    if (!g_staging.fit(buf, bytes)) return false;
    if (cudaMemcpyAsync(buf.p, a->data, bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) return false;
    *out = buf.p;
    return true;
}

// table/table.zig:196-201
t3_verdict table_matmul(const t3_weight* w, const t3_array* x, void* stream, t3_array* out) {
    if (!w || !w->w || w->block == 0) return refuse(T3_VERDICT_FAILED, "turboexl3: a weight without its decode");
    if (!present(x) || !out || !out->data) return refuse(T3_VERDICT_FAILED, "NullPointer");
    if (x->ndim < 1 || x->ndim > 8 || x->shape[x->ndim - 1] != w->in_dim) return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Shape");
    if (!act_dtype(x->dtype)) return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Dtype");
    const size_t rows = count_of(x) / (size_t)w->in_dim;
    if (rows < 1) return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Shape");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = elem_size(x->dtype), xb = rows * w->in_dim * es, yb = rows * w->out_dim * es;
    const bool host = !x->device || !out->device;
    std::unique_lock<std::mutex> lock(g_staging.mu);
    if (!g_staging.owns_current()) return refuse(T3_VERDICT_FAILED, "CudaError");  // the staging buffers live on another device
    const size_t wsb = t3_linear_workspace_bytes(rows, w->in_dim, w->out_dim, w->block);
    Staging::StreamWs& sws = g_staging.of(stream);
    const bool decode_rows = rows <= T3_DECODE_ROWS_MAX;
    Staging::Buf& wsbuf = decode_rows ? sws.rows : sws.ws;
    if (wsb && !(decode_rows ? g_staging.fit_zeroed(wsbuf, wsb) : g_staging.fit(wsbuf, wsb))) return refuse(T3_VERDICT_FAILED, "CudaError");
    if (!x->device && !out->device && decode_rows && xb <= Staging::kMappedBytes && yb <= Staging::kMappedBytes &&
        g_staging.mapped()) {
        // decode rows on host arrays: one launch between two memcpys
        memcpy(g_staging.hx, x->data, xb);
        const t3_decode dec = {w->layout, w->flags};
        const int rc = t3_linear(g_staging.hx_dev, x->dtype, rows, w->w, w->scales, w->biases, w->in_dim, w->out_dim, w->block,
                                 dec, g_staging.hy_dev, wsbuf.p, wsbuf.cap, s);
        if (rc != T3_OK) return from_status(rc);
        if (cudaStreamSynchronize(s) != cudaSuccess) return refuse(T3_VERDICT_FAILED, "CudaError");
        memcpy(out->data, g_staging.hy, yb);
        out->dtype = x->dtype;
        out->ndim = x->ndim;
        for (int i = 0; i < x->ndim; ++i) out->shape[i] = x->shape[i];
        out->shape[x->ndim - 1] = w->out_dim;
        return ok();
    }
    const void* xd = nullptr;
    if (!stage_in(x, g_staging.x, xb, s, &xd)) return refuse(T3_VERDICT_FAILED, "CudaError");
    void* yd = out->data;
    if (!out->device) {
        if (!g_staging.fit(g_staging.y, yb)) return refuse(T3_VERDICT_FAILED, "CudaError");
        yd = g_staging.y.p;
    }
    const t3_decode dec = {w->layout, w->flags};
    const int rc = t3_linear(xd, x->dtype, rows, w->w, w->scales, w->biases, w->in_dim, w->out_dim, w->block, dec, yd,
                             wsbuf.p, wsbuf.cap, s);
    if (rc != T3_OK) return from_status(rc);
    if (!out->device && cudaMemcpyAsync(out->data, yd, yb, cudaMemcpyDeviceToHost, s) != cudaSuccess)
        return refuse(T3_VERDICT_FAILED, "CudaError");
    if (host && cudaStreamSynchronize(s) != cudaSuccess) return refuse(T3_VERDICT_FAILED, "CudaError");
    out->dtype = x->dtype;
    out->ndim = x->ndim;
    for (int i = 0; i < x->ndim; ++i) out->shape[i] = x->shape[i];
    out->shape[x->ndim - 1] = w->out_dim;
    return ok();
}

t3_verdict table_moe(const t3_weight*, const t3_array*, const t3_array*, const t3_array*, int, void*, t3_array*) {
    return refuse(T3_VERDICT_UNSUPPORTED, "turboexl3: a layer's banks run as one routed SwiGLU (swiglu)");
}

// table/table.zig:210-221
t3_verdict table_swiglu(const t3_weight* gate, const t3_weight* up, const t3_weight* down, const t3_array* x,
                        const t3_array* inds, const t3_array* scores, const t3_swiglu_opts* opts, void* stream,
                        t3_array* out) {
    if (!gate || !gate->w || gate->block == 0) return refuse(T3_VERDICT_FAILED, "turboexl3: a bank without its decode");
    if (!up || !down || up->layout != gate->layout || up->flags != gate->flags || down->layout != gate->layout ||
        down->flags != gate->flags || !up->w || !down->w)
        return refuse(T3_VERDICT_UNSUPPORTED, "turboexl3: a layer's banks decode differently");
    if (!present(x) || !present(inds) || !present(scores) || !out || !out->data) return refuse(T3_VERDICT_FAILED, "NullPointer");
    // root.validateCall, src/root.zig:128-141
    if (x->ndim != 3 || inds->ndim != 3 || scores->ndim != 3 || x->shape[0] <= 0 || x->shape[1] <= 0 ||
        x->shape[0] != inds->shape[0] || x->shape[1] != inds->shape[1] || inds->shape[2] <= 0 ||
        inds->shape[2] > T3_REDUCE_MAX_TOPK || scores->shape[0] != inds->shape[0] || scores->shape[1] != inds->shape[1] ||
        scores->shape[2] != inds->shape[2] || x->shape[2] != gate->in_dim)
        return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Shape");
    if (!act_dtype(x->dtype) || !act_dtype(scores->dtype) || (inds->dtype != T3_A_I32 && inds->dtype != T3_A_U32))
        return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Dtype");
    if (gate->experts <= 0 || up->experts != gate->experts || down->experts != gate->experts || up->in_dim != gate->in_dim ||
        up->out_dim != gate->out_dim || down->in_dim != gate->out_dim || down->out_dim != gate->in_dim)
        return refuse(T3_VERDICT_UNSUPPORTED, "BadExl3Shape");
    const size_t rows = (size_t)x->shape[0] * (size_t)x->shape[1];
    const int topk = (int)inds->shape[2];
    t3_bank bank = {};
    bank.gate = {gate->w, gate->scales, gate->biases};
    bank.up = {up->w, up->scales, up->biases};
    bank.down = {down->w, down->scales, down->biases};
    bank.experts = gate->experts;
    bank.hidden = gate->in_dim;
    bank.inter = gate->out_dim;
    bank.n_gate = gate->block;
    bank.n_up = up->block;
    bank.n_down = down->block;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t es = elem_size(x->dtype), xb = rows * bank.hidden * es;
    const bool host = !x->device || !out->device || !inds->device || !scores->device;
    std::unique_lock<std::mutex> lock(g_staging.mu);
    if (!g_staging.owns_current()) return refuse(T3_VERDICT_FAILED, "CudaError");  // the staging buffers live on another device
    const void *xd = nullptr, *id = nullptr, *sd = nullptr;
    if (!stage_in(x, g_staging.x, xb, s, &xd) || !stage_in(inds, g_staging.inds, rows * topk * 4u, s, &id) ||
        !stage_in(scores, g_staging.scores, rows * topk * elem_size(scores->dtype), s, &sd))
        return refuse(T3_VERDICT_FAILED, "CudaError");
    void* yd = out->data;
    if (!out->device) {
        if (!g_staging.fit(g_staging.y, xb)) return refuse(T3_VERDICT_FAILED, "CudaError");
        yd = g_staging.y.p;
    }
    const size_t wsb = t3_moe_workspace_bytes(rows, topk, &bank);
    Staging::Buf& wsbuf = g_staging.of(stream).ws;
    if (!g_staging.fit(wsbuf, wsb ? wsb : 1)) return refuse(T3_VERDICT_FAILED, "CudaError");
    const t3_decode dec = {gate->layout, gate->flags};
    const int limit = opts ? opts->limit : 0;
    const int rc = limit > 0 ? t3_moe_clamped(xd, x->dtype, rows, &bank, id, sd, scores->dtype, topk, dec, limit, yd,
                                              wsbuf.p, wsbuf.cap, s)
                             : t3_moe(xd, x->dtype, rows, &bank, id, sd, scores->dtype, topk, dec, yd, wsbuf.p,
                                      wsbuf.cap, s);
    if (rc != T3_OK) return from_status(rc);
    if (!out->device && cudaMemcpyAsync(out->data, yd, xb, cudaMemcpyDeviceToHost, s) != cudaSuccess)
        return refuse(T3_VERDICT_FAILED, "CudaError");
    if (host && cudaStreamSynchronize(s) != cudaSuccess) return refuse(T3_VERDICT_FAILED, "CudaError");
    out->dtype = x->dtype;
    out->ndim = 3;
    for (int i = 0; i < 3; ++i) out->shape[i] = x->shape[i];
    return ok();
}

const t3_quant_table g_table = {
    "turboexl3", table_claims, table_validate, table_bill, table_open, table_close, table_load_tensor, table_load_bank,
    table_release, table_matmul, table_moe, table_swiglu,
};

}  // namespace

extern "C" {

const t3_quant_table* t3_table(void) { return &g_table; }

size_t t3_table_staging_bytes(void) {
    std::lock_guard<std::mutex> lock(g_staging.mu);
    return g_staging.bytes();
}

void t3_table_release_staging(void) {
    std::lock_guard<std::mutex> lock(g_staging.mu);
    g_staging.release();
}

}  // extern "C"
