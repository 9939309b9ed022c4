// The C ABI (include/t3.h): admission, launch planning and dispatch. Every refusal happens before any launch, under the
// reference's error names (turboexl3 src/root.zig:93-141, 322-351, 839-904).
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <initializer_list>
#include <mutex>
#include <unordered_set>
#include <string>

#include "../../include/t3.h"
#include "t3_gemv.cuh"
#include "t3_internal.h"
#include "t3_json.h"

namespace t3 {

cudaError_t launch_dense_gemv_cb0(const DenseArgs&, cudaStream_t);
cudaError_t launch_dense_gemv_cb1(const DenseArgs&, cudaStream_t);
cudaError_t launch_dense_gemv_cb2(const DenseArgs&, cudaStream_t);  // timing probes: no codebook hash,
cudaError_t launch_dense_gemv_cb3(const DenseArgs&, cudaStream_t);  // no window extraction either,
cudaError_t launch_dense_gemv_cb4(const DenseArgs&, cudaStream_t);  // the code stream alone
cudaError_t launch_moe_gate_up_cb0(const MoeArgs&, cudaStream_t);
cudaError_t launch_moe_gate_up_cb1(const MoeArgs&, cudaStream_t);
cudaError_t launch_moe_down_cb0(const MoeArgs&, cudaStream_t);
cudaError_t launch_moe_down_cb1(const MoeArgs&, cudaStream_t);

namespace {

std::atomic<uint64_t> g_launches{0};

// The geometries served since the last t3_release_engines, by path: what the reference's engine caches would hold
// (src/root.zig:1183-1192). Nothing heavier hangs off an entry here: kernels are compiled ahead and plans are recomputed
// per call, so an entry is a key, not device memory.
std::mutex g_engines_mu;
std::unordered_set<uint64_t> g_engines[3];  // decode (routed GEMV chain), dense, prefill
void note_engine(int kind, uint64_t a, uint64_t b, uint64_t c, uint64_t d) {
    const uint64_t key = (a * 0x9E3779B97F4A7C15ull) ^ (b * 0xC2B2AE3D27D4EB4Full) ^ (c * 0x165667B19E3779F9ull) ^ (d << 48);
    std::lock_guard<std::mutex> lock(g_engines_mu);
    g_engines[kind].insert(key);
}

__device__ uint32_t g_dev_error_word;

std::mutex g_mu;
t3_config g_cfg = {1, 0, 0, 0, 0};
uint32_t* g_err_ptr[64] = {};
unsigned long long* g_trace = nullptr;

constexpr uint32_t kSmemCap = kGemvSmemLimit - kSmemSlack;  // what the carve-up of a GEMV CTA may add up to
constexpr uint32_t kDefaultRing = 64u * 1024u;

uint32_t* dev_error_ptr() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_err_ptr[dev]) {
        void* p = nullptr;
        if (cudaGetSymbolAddress(&p, g_dev_error_word) != cudaSuccess) return nullptr;
        g_err_ptr[dev] = static_cast<uint32_t*>(p);
    }
    return g_err_ptr[dev];
}

uint32_t pow2_at_most(uint32_t v, uint32_t cap) {
    uint32_t s = 1;
    while (s * 2u <= v && s * 2u <= cap) s *= 2u;
    return s;
}

// CTAs that fit on the device at once (two GEMV CTAs a multiprocessor)
uint32_t one_wave() {
    static std::atomic<uint32_t> ctas[64];  // per device ordinal; 0 = not asked yet
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 2u * 148u;
    uint32_t v = ctas[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        v = 2u * (uint32_t)sms;
        ctas[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}

// K slices for `units` independent (output block, job) pairs over nb 128-blocks of K: the smallest power of two, at most
// `cap`, that brings the grid (units x slices x `fan` CTAs a slice) to `target` CTAs, never past one wave. A dense linear
// aims at one CTA a multiprocessor (a second slot stays free for the next launch to start under this one); a routed call
// aims at an eighth of a wave for a nominal row's slots, because its grid grows with the rows and longer CTAs amortise
// their fixed part (measured on config 3: split 1 instead of 2 is as fast at 1 and 4 rows and 10 % faster at 16 and 32).
// (Other counts work too, slices may differ by a block, but measured slower than the nearest power of two below them.)
uint32_t pick_split(uint32_t nb, uint32_t units, uint32_t fan, uint32_t cap, uint32_t target) {
    uint32_t s = 1;
    while (s * 2u <= nb && s * 2u <= cap && (uint64_t)units * fan * s < target && (uint64_t)units * fan * s * 2u <= one_wave())
        s *= 2u;
    return s;
}

// K slices of a LARGE dense linear (tens of megabytes of codes: milliseconds of integer work, so what counts is that
// every multiprocessor gets the same share, not the launch's latency): the power of two whose CTAs all
// fit the device at once — two a multiprocessor, clusters of s — and leave the fullest multiprocessor the fewest
// 128-input blocks; ties go to the wider cluster (more warps a multiprocessor).
uint32_t pick_split_large(uint32_t nb, uint32_t out_blocks) {
    static const uint32_t cap_ctas[9] = {0, 296, 296, 279, 284, 280, 270, 259, 264};  // resident CTAs by cluster size (measured)
    const uint32_t sms = one_wave() / 2u;
    uint32_t best_s = 1, best = ~0u;
    for (uint32_t s = 1; s <= 8u && s <= nb; s *= 2u) {  // powers of two: clusters of 3, 5, 6, 7 measured slower (placement)
        const uint32_t ctas = out_blocks * s;
        if (ctas > cap_ctas[s] * sms / 148u) continue;
        const uint32_t cost = ((ctas + sms - 1u) / sms) * ((nb + s - 1u) / s);
        if (cost <= best) best = cost, best_s = s;
    }
    return best_s;
}

uint32_t largest_slice(uint32_t nb, uint32_t split) {
    uint32_t mx = 0;
    for (uint32_t r = 0; r < split; ++r) {
        uint32_t b0, b1;
        slice_blocks(nb, split, r, b0, b1);
        mx = b1 - b0 > mx ? b1 - b0 : mx;
    }
    return mx * 128u;
}

// The ring of one GEMV CTA: stages of kStageRows tk rows (two 128-input blocks), as many as the slab needs or the budget
// holds; three where the default budget holds fewer and two CTAs still fit a multiprocessor.
bool plan_ring(uint32_t row_cap, uint32_t xrows, uint32_t slice_max, uint32_t cluster, uint32_t n, RingPlan& ring) {
    const uint32_t row_bytes = 16u * n, nrows = slice_max / 16u;  // nrows is a multiple of 8 (whole 128-blocks)
    const uint32_t stage_rows = kStageRows;
    const uint32_t stage_bytes = stage_rows * row_bytes;
    const uint32_t need = (nrows + stage_rows - 1u) / stage_rows;
    const uint32_t fixed = gemv_smem(row_cap, xrows, slice_max, cluster, stage_bytes, 0).total;
    if (fixed + stage_bytes > kSmemCap) return false;
    uint32_t budget = g_cfg.ring_bytes ? g_cfg.ring_bytes : kDefaultRing;
    if (!g_cfg.ring_bytes && budget < 3u * stage_bytes && fixed + 3u * stage_bytes <= 108u * 1024u) budget = 3u * stage_bytes;
    if (budget > kSmemCap - fixed) budget = kSmemCap - fixed;
    uint32_t stages = budget / stage_bytes;
    stages = stages < 1u ? 1u : stages;
    stages = stages > need ? need : stages;
    stages = stages > kMaxStages ? kMaxStages : stages;
    ring.stage_rows = stage_rows;
    ring.stages = stages;
    return true;
}

bool dtype_ok(int dt) { return dt == T3_F32 || dt == T3_F16 || dt == T3_BF16; }
size_t dtype_size(int dt) { return dt == T3_F32 ? 4 : 2; }

int decode_mask(t3_decode dec, uint32_t& mask) {
    if (dec.codebook != T3_MUL1 && dec.codebook != T3_MCG) return T3_ENGINE_NOT_IMPLEMENTED;
    if (dec.window_bits < 8 || dec.window_bits > 16) return T3_WINDOW_UNSUPPORTED;
    mask = (1u << dec.window_bits) - 1u;
    return T3_OK;
}

bool rate_ok(int n) { return n >= 16 && n <= 128 && n % 2 == 0; }

int cuda_status(cudaError_t rc) { return rc == cudaSuccess ? T3_OK : T3_CUDA_ERROR; }

}  // namespace

uint32_t row_cap_for(uint32_t rows) { return rows <= 8u ? 8u : (rows <= 16u ? 16u : 32u); }

uint32_t gemv_smem_bytes(uint32_t row_cap, uint32_t xrows, uint32_t slice_max, uint32_t cluster, uint32_t n, RingPlan ring) {
    return gemv_smem(row_cap, xrows, slice_max, cluster, ring.stage_rows * 16u * n, ring.stages).total + kSmemSlack;
}

thread_local const void* g_last_kernel = nullptr;
void note_symbol(const void* kernel) { g_last_kernel = kernel; }

cudaError_t launch_dense_gemv(const DenseArgs& a, int codebook, cudaStream_t stream) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (codebook == 2) return launch_dense_gemv_cb2(a, stream);
    if (codebook == 3) return launch_dense_gemv_cb3(a, stream);
    if (codebook == 4) return launch_dense_gemv_cb4(a, stream);
    return codebook == T3_MCG ? launch_dense_gemv_cb1(a, stream) : launch_dense_gemv_cb0(a, stream);
}
cudaError_t launch_moe_gate_up(const MoeArgs& a, int codebook, cudaStream_t stream) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return codebook == T3_MCG ? launch_moe_gate_up_cb1(a, stream) : launch_moe_gate_up_cb0(a, stream);
}
cudaError_t launch_moe_down(const MoeArgs& a, int codebook, cudaStream_t stream) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return codebook == T3_MCG ? launch_moe_down_cb1(a, stream) : launch_moe_down_cb0(a, stream);
}

}  // namespace t3

using namespace t3;

extern "C" {

const char* t3_status_name(int status) {
    switch (status) {
        case T3_OK: return "Ok";
        case T3_BAD_EXL3_SHAPE: return "BadExl3Shape";
        case T3_BAD_EXL3_DTYPE: return "BadExl3Dtype";
        case T3_ENGINE_NOT_IMPLEMENTED: return "Exl3EngineNotImplemented";
        case T3_ENGINE_CACHE_FULL: return "Exl3EngineCacheFull";
        case T3_GATE_UP_RATE_MISMATCH: return "Exl3GateUpRateMismatch";
        case T3_INVALID_CLAMP: return "InvalidExl3Clamp";
        case T3_INVALID_CONFIG: return "InvalidTurboexl3Config";
        case T3_KERNEL_CREATE_FAILED: return "KernelCreateFailed";
        case T3_CUDA_ERROR: return "CudaError";
        case T3_TOPK_EXCEEDS_REDUCE_BANK: return "Exl3TopKExceedsReduceBank";
        case T3_WORKSPACE_TOO_SMALL: return "WorkspaceTooSmall";
        case T3_EXPERT_LAYOUT_UNSUPPORTED: return "ExpertLayoutUnsupported";
        case T3_WINDOW_UNSUPPORTED: return "Exl3WindowUnsupported";
        case T3_NULL_POINTER: return "NullPointer";
        case T3_SCRATCH_LIMIT_EXCEEDED: return "ScratchLimitExceeded";
        default: return "Unknown";
    }
}

int t3_uses_prefill_arm(size_t rows) { return rows > T3_DECODE_ROWS_MAX; }

int t3_admit_topk(uint32_t topk) { return topk > T3_REDUCE_MAX_TOPK ? T3_TOPK_EXCEEDS_REDUCE_BANK : T3_OK; }

int t3_trellis_admitted(const int* shape, int ndim, uint32_t experts, uint32_t in_dim, uint32_t out_dim, uint32_t n) {
    if (!shape || ndim != 4) return 0;
    for (int i = 0; i < 4; ++i)
        if (shape[i] <= 0) return 0;
    if (in_dim % 16u != 0 || out_dim % 16u != 0) return 0;
    if ((uint32_t)shape[0] != experts || (uint32_t)shape[1] != in_dim / 16u || (uint32_t)shape[2] != out_dim / 16u) return 0;
    if (!rate_ok(shape[3])) return 0;
    return (uint32_t)shape[3] <= n;
}

// ---- expert_quant ---------------------------------------------------------------------------------------------------

int t3_parse_expert_quant(const char* json, size_t len, t3_spec* out) {
    if (!json || !out) return T3_NULL_POINTER;
    // a top-level object field, as the reference reads it (src/core/spec.zig:38-50): a key of that name nested deeper, or
    // inside a string, is not the block
    t3json::JsonReader r{json, json + len};
    const t3json::Json root = r.value();
    r.skip();
    if (!r.ok || r.p != r.end || root.kind != t3json::Json::kObject) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    const t3json::Json* blk = root.get("expert_quant");
    if (!blk || blk->kind != t3json::Json::kObject) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    const t3json::Json* format = blk->get("format");
    if (!format || format->kind != t3json::Json::kString || format->s != "exl3") return T3_EXPERT_LAYOUT_UNSUPPORTED;
    const t3json::Json* k = blk->get("k");
    if (!k || (k->kind != t3json::Json::kInt && k->kind != t3json::Json::kFloat)) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    const double scaled = k->f * 16.0, rounded = std::round(scaled);
    if (std::fabs(scaled - rounded) > 1e-6 || rounded < 0 || rounded > 1024) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    if (!rate_ok((int)rounded)) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    const t3json::Json* codebook = blk->get("codebook");
    if (!codebook || codebook->kind != t3json::Json::kString) return T3_EXPERT_LAYOUT_UNSUPPORTED;
    int cb;
    if (codebook->s == "mul1") cb = T3_MUL1;
    else if (codebook->s == "mcg") cb = T3_MCG;
    else return T3_EXPERT_LAYOUT_UNSUPPORTED;
    int window = 16;
    if (const t3json::Json* w = blk->get("window")) {
        if (w->kind != t3json::Json::kInt || w->i < 8 || w->i > 16) return T3_WINDOW_UNSUPPORTED;
        window = (int)w->i;
    }
    out->n = (uint32_t)rounded;
    out->codebook = cb;
    out->window_bits = window;
    return T3_OK;
}

// ---- configuration --------------------------------------------------------------------------------------------------

void t3_config_default(t3_config* out) {
    if (!out) return;
    out->prefill = 1;
    out->ring_bytes = 0;
    out->dense_split = 0;
    out->no_overlap = 0;
    out->probe = 0;
}

int t3_configure(const t3_config* cfg) {
    if (!cfg) return T3_NULL_POINTER;
    const uint32_t s = cfg->dense_split;
    if (s > 16u) return T3_INVALID_CONFIG;
    if (cfg->no_overlap != 0 && cfg->no_overlap != 1) return T3_INVALID_CONFIG;
    if (cfg->ring_bytes != 0 && (cfg->ring_bytes < 4096u || cfg->ring_bytes > kGemvSmemLimit)) return T3_INVALID_CONFIG;
    if (cfg->prefill != 0 && cfg->prefill != 1) return T3_INVALID_CONFIG;
    if (cfg->probe < 0 || cfg->probe > 3) return T3_INVALID_CONFIG;
    std::lock_guard<std::mutex> lock(g_mu);
    g_cfg = *cfg;
    return T3_OK;
}

int t3_selftest_wait_runs_out(void* stream) {
    uint32_t* p = dev_error_ptr();
    if (!p) return T3_CUDA_ERROR;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_wait_runs_out(p, static_cast<cudaStream_t>(stream)));
}

int t3_device_error(void* stream, uint32_t* bits_out, int clear) {
    uint32_t* p = dev_error_ptr();
    if (!p) return T3_CUDA_ERROR;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint32_t bits = 0;
    if (cudaMemcpyAsync(&bits, p, sizeof bits, cudaMemcpyDeviceToHost, s) != cudaSuccess) return T3_CUDA_ERROR;
    if (clear && cudaMemsetAsync(p, 0, sizeof bits, s) != cudaSuccess) return T3_CUDA_ERROR;
    if (cudaStreamSynchronize(s) != cudaSuccess) return T3_CUDA_ERROR;
    if (bits_out) *bits_out = bits;
    return T3_OK;
}

void t3_set_trace(void* device_u64x8) {
    std::lock_guard<std::mutex> lock(g_mu);
    g_trace = static_cast<unsigned long long*>(device_u64x8);
}

uint64_t t3_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

void t3_engines_held(t3_engines* out) {
    if (!out) return;
    std::lock_guard<std::mutex> lock(g_engines_mu);
    out->decode = g_engines[0].size();
    out->dense = g_engines[1].size();
    out->prefill = g_engines[2].size();
}

void t3_release_engines(void) {
    std::lock_guard<std::mutex> lock(g_engines_mu);
    for (auto& e : g_engines) e.clear();
}

// ---- W_hat ----------------------------------------------------------------------------------------------------------

int t3_dequant(const void* trellis, int in_dim, int out_dim, int n, t3_decode dec, void* w_hat, void* stream) {
    if (!trellis || !w_hat) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n)) return T3_BAD_EXL3_SHAPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_dequant(static_cast<const uint8_t*>(trellis), (uint32_t)in_dim, (uint32_t)out_dim,
                                      (uint32_t)n, mask, dec.codebook, 0, w_hat, static_cast<cudaStream_t>(stream)));
}

size_t t3_resident_bytes(int in_dim, int out_dim) {
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0) return 0;
    return (size_t)in_dim * (size_t)out_dim * 2u;
}

int t3_resident_build(const void* trellis, int in_dim, int out_dim, int n, t3_decode dec, void* w_hat_t, void* stream) {
    if (!trellis || !w_hat_t) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n)) return T3_BAD_EXL3_SHAPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_dequant(static_cast<const uint8_t*>(trellis), (uint32_t)in_dim, (uint32_t)out_dim,
                                      (uint32_t)n, mask, dec.codebook, 1, w_hat_t, static_cast<cudaStream_t>(stream)));
}

int t3_linear_resident(const void* x, int x_dtype, size_t rows, const void* w_hat_t, const void* suh, const void* svh,
                       int in_dim, int out_dim, void* y, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !w_hat_t || !suh || !svh || !y) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || rows < 1 || rows > (size_t)1 << 30)
        return T3_BAD_EXL3_SHAPE;
    if (!dtype_ok(x_dtype)) return T3_BAD_EXL3_DTYPE;
    if (rows <= T3_DECODE_ROWS_MAX) return T3_ENGINE_NOT_IMPLEMENTED;  // decode rows read the codes, never W_hat
    if (rows > 0x7FFFFFFFu / (size_t)(in_dim > out_dim ? in_dim : out_dim)) return T3_BAD_EXL3_SHAPE;
    if (rows > kPrefillDenseRowsMax) return T3_BAD_EXL3_SHAPE;
    if (!workspace || workspace_bytes < t3_linear_workspace_bytes(rows, in_dim, out_dim, 16)) return T3_WORKSPACE_TOO_SMALL;
    PrefillLinearArgs p = {x, y, nullptr, w_hat_t, suh, svh, (uint32_t)rows, (uint32_t)in_dim, (uint32_t)out_dim, 16u, 0xFFFFu,
                           x_dtype, workspace, dev_error_ptr()};
    note_engine(2, (uint64_t)in_dim, (uint64_t)out_dim, 0, 1);
    int launches = 0;
    const cudaError_t rc = launch_prefill_linear(p, kMul1, static_cast<cudaStream_t>(stream), &launches);
    g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
    return cuda_status(rc);
}

int t3_unrot_build(const void* trellis, const void* suh, const void* svh, int in_dim, int out_dim, int n, t3_decode dec,
                   int act_dtype, void* w_std_t, void* stream) {
    if (!trellis || !suh || !svh || !w_std_t) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n)) return T3_BAD_EXL3_SHAPE;
    if (act_dtype != T3_F16 && act_dtype != T3_BF16) return T3_BAD_EXL3_DTYPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    g_launches.fetch_add(2, std::memory_order_relaxed);
    cudaError_t rc = launch_dequant(static_cast<const uint8_t*>(trellis), (uint32_t)in_dim, (uint32_t)out_dim, (uint32_t)n, mask,
                                    dec.codebook, 1, w_std_t, s);
    if (rc == cudaSuccess) rc = launch_unrot(w_std_t, suh, svh, (uint32_t)in_dim, (uint32_t)out_dim, act_dtype, s);
    return cuda_status(rc);
}

int t3_linear_unrot(const void* x, int x_dtype, size_t rows, const void* w_std_t, int in_dim, int out_dim, void* y, void* stream) {
    if (!x || !w_std_t || !y) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || rows < 1) return T3_BAD_EXL3_SHAPE;
    if (x_dtype != T3_F16 && x_dtype != T3_BF16) return T3_BAD_EXL3_DTYPE;
    if (rows <= T3_DECODE_ROWS_MAX) return T3_ENGINE_NOT_IMPLEMENTED;  // dense.unrot_min_rows: those rows keep the trellis paths
    if (rows > kPrefillDenseRowsMax || rows > 0x7FFFFFFFu / (size_t)(in_dim > out_dim ? in_dim : out_dim)) return T3_BAD_EXL3_SHAPE;
    note_engine(2, (uint64_t)in_dim, (uint64_t)out_dim, 0, 2);
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_plain_linear(x, x_dtype, (uint32_t)rows, w_std_t, (uint32_t)in_dim, (uint32_t)out_dim, y,
                                           dev_error_ptr(), static_cast<cudaStream_t>(stream)));
}

int t3_codebook_table(t3_decode dec, void* out, void* stream) {
    if (!out) return T3_NULL_POINTER;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_codebook_table(dec.codebook, mask, static_cast<uint16_t*>(out), static_cast<cudaStream_t>(stream)));
}

// ---- dense linear ---------------------------------------------------------------------------------------------------

namespace {
// Linears of 24 MB of codes and up with their workspace: any slice count s, CTAs placed one by one (no cluster), the slices'
// sums meeting in global memory. The cost of a count: the CTAs of the fullest multiprocessor times a slice's 128-input blocks
// (all CTAs resident at once, two a multiprocessor). Returns 0 when no count beats the cluster kernel's by a tenth (the
// global exchange costs a couple of microseconds a launch).
uint32_t pick_split_global(uint32_t nb, uint32_t out_blocks, uint32_t cluster_split) {
    const uint32_t sms = one_wave() / 2u;
    auto cost_of = [&](uint32_t s) { return ((out_blocks * s + sms - 1u) / sms) * ((nb + s - 1u) / s); };
    uint32_t best_s = 0, best = cost_of(cluster_split) * 9u / 10u;
    for (uint32_t s = 2; s <= 16u && s <= nb; ++s) {
        if (out_blocks * s > 2u * sms) break;
        const uint32_t cost = cost_of(s);
        if (cost < best) best = cost, best_s = s;
    }
    return best_s;
}

size_t align256(size_t v) { return (v + 255u) & ~(size_t)255u; }

// The workspace of a dense linear at decode rows, in this order: the rows rotated ahead of the GEMV (more than kFusedRows
// rows), the slices' partial sums and the blocks' arrival counters (large linears on the global exchange).
struct DenseWs {
    size_t xp, part, counters, total;
};
// Whether a call's rows are rotated once by a launch of their own instead of inside every CTA: past kFusedRows rows always;
// up to kFusedRows when a CTA's share of the work would be more than two rotations a warp (many rows on long K slices: each
// CTA repeats the rotation of its whole slice for every row before its first tensor-core step).
bool prep_ahead(uint32_t rows, uint32_t slice_max) { return rows > kFusedRows || rows * (slice_max / 128u) > 2u * kConsumerWarps; }

DenseWs dense_ws(uint32_t rows, uint32_t in, uint32_t out, uint32_t global_split, uint32_t slice_max) {
    DenseWs w;
    w.xp = 0;
    w.part = prep_ahead(rows, slice_max) ? align256((size_t)rows * in * 2u) : 0u;
    w.counters = w.part + (global_split ? align256((size_t)(out / 128u) * global_split * rows * 512u) : 0u);
    w.total = w.counters + (global_split ? align256((size_t)(out / 128u) * 4u) : 0u);
    return w;
}

bool large_linear(uint32_t in, uint32_t out, uint32_t n) { return (uint64_t)in * out * n >= (uint64_t)24u * 1024u * 1024u * 128u; }

// The launch shape of a dense linear at decode rows: the K split (cluster size) and the code ring. a.rows, in, out, n set.
// global_ok: the call has its workspace, so a large linear may take the global exchange (a.part is set non-null as a mark;
// the caller points it into the workspace).
int plan_dense(DenseArgs& a, const t3_config& cfg, bool global_ok) {
    const uint32_t nb = a.in / 128u;
    const bool large = large_linear(a.in, a.out, a.n);
    a.split = cfg.dense_split ? (cfg.dense_split < nb ? cfg.dense_split : nb)
                              : (large ? pick_split_large(nb, a.out / 128u) : pick_split(nb, a.out / 128u, 1u, 8u, one_wave() / 2u));
    a.part = nullptr;
    if (large && global_ok && !cfg.dense_split && !cfg.probe) {
        const uint32_t s = pick_split_global(nb, a.out / 128u, a.split);
        if (s) {
            a.split = s;
            a.part = reinterpret_cast<float*>(1);  // a mark: the caller sets the pointer
        }
    }
    a.overlap = !cfg.no_overlap;
    a.slice_max = largest_slice(nb, a.split);
    // a slice too long for shared memory (its prepared rows) is cut further, up to the widest cluster
    while (!plan_ring(row_cap_for(a.rows), a.rows, a.slice_max, a.part ? 1u : a.split, a.n, a.ring)) {
        if (a.part) {  // back to the cluster kernel
            a.part = nullptr;
            a.split = pick_split_large(nb, a.out / 128u);
            a.slice_max = largest_slice(nb, a.split);
            continue;
        }
        if (a.split * 2u > nb || a.split * 2u > 16u) return T3_ENGINE_NOT_IMPLEMENTED;
        a.split *= 2u;
        a.slice_max = largest_slice(nb, a.split);
    }
    return T3_OK;
}

// the rate as the kernels' names carry it: the integer rates have their own kernels, any other even rate runs the n0 ones
uint32_t named_rate(uint32_t n) { return (n % 16u == 0u && n >= 16u && n <= 128u) ? n : 0u; }

void fill_launch(t3_launch* l, const char* symbol, const char* group, dim3 grid, uint32_t block, uint32_t shared, uint32_t cluster,
                 std::initializer_list<int> roles) {
    std::memset(l, 0, sizeof *l);
    std::snprintf(l->symbol, sizeof l->symbol, "%s", symbol);
    std::snprintf(l->group, sizeof l->group, "%s", group);
    l->grid[0] = grid.x, l->grid[1] = grid.y, l->grid[2] = grid.z;
    l->block = block;
    l->shared = shared;
    l->cluster = cluster;
    for (int r : roles)
        if (l->nroles < (int)(sizeof l->roles / sizeof l->roles[0])) l->roles[l->nroles++] = r;
}

}  // namespace


size_t t3_linear_workspace_bytes(size_t rows, int in_dim, int out_dim, int n) {
    if (in_dim <= 0 || out_dim <= 0 || rows < 1) return 0;
    if (rows > T3_DECODE_ROWS_MAX) return prefill_linear_workspace(rows, (uint32_t)in_dim, (uint32_t)out_dim);
    if (in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n)) return 0;
    // Decode rows. Up to 8 rows of an ordinary linear: nothing (the kernel keeps everything on chip). 9 to 32 rows: the rows
    // rotated once ahead of the GEMV. Linears of 24 MB of codes and up: the K slices' partial sums, when a slice count that
    // fills the multiprocessors evenly exists for the shape. All optional: a call without it takes the cluster kernel.
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    DenseArgs a = {};
    a.in = (uint32_t)in_dim, a.out = (uint32_t)out_dim, a.n = (uint32_t)n, a.rows = (uint32_t)rows;
    if (plan_dense(a, cfg, true) != T3_OK) return 0;
    return dense_ws(a.rows, a.in, a.out, a.part ? a.split : 0u, a.slice_max).total;
}

int t3_linear(const void* x, int x_dtype, size_t rows, const void* trellis, const void* suh, const void* svh,
              int in_dim, int out_dim, int n, t3_decode dec, void* y, void* workspace, size_t workspace_bytes,
              void* stream) {
    if (!x || !trellis || !suh || !svh || !y) return T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n) || rows < 1 ||
        rows > (size_t)1 << 30)
        return T3_BAD_EXL3_SHAPE;
    if (!dtype_ok(x_dtype)) return T3_BAD_EXL3_DTYPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    if (rows > T3_DECODE_ROWS_MAX) {
        if (!cfg.prefill) return T3_ENGINE_NOT_IMPLEMENTED;
        if (rows > 0x7FFFFFFFu / (size_t)(in_dim > out_dim ? in_dim : out_dim)) return T3_BAD_EXL3_SHAPE;
        if (rows > kPrefillDenseRowsMax) return T3_BAD_EXL3_SHAPE;  // the prepare launch's row groups are a grid dimension
        if (!workspace || workspace_bytes < t3_linear_workspace_bytes(rows, in_dim, out_dim, n)) return T3_WORKSPACE_TOO_SMALL;
        PrefillLinearArgs p = {x, y, static_cast<const uint8_t*>(trellis), nullptr, suh, svh, (uint32_t)rows, (uint32_t)in_dim,
                               (uint32_t)out_dim, (uint32_t)n, mask, x_dtype, workspace, dev_error_ptr()};
        note_engine(2, (uint64_t)in_dim, (uint64_t)out_dim, (uint64_t)n, 0);
        int launches = 0;
        const cudaError_t rc = launch_prefill_linear(p, dec.codebook, static_cast<cudaStream_t>(stream), &launches);
        g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
        return cuda_status(rc);
    }

    DenseArgs a = {};
    a.trellis = static_cast<const uint8_t*>(trellis);
    a.suh = suh;
    a.svh = svh;
    a.in = (uint32_t)in_dim;
    a.out = (uint32_t)out_dim;
    a.n = (uint32_t)n;
    a.mask = mask;
    a.x_dt = x_dtype;
    note_engine(1, (uint64_t)in_dim, (uint64_t)out_dim, (uint64_t)n, 0);
    a.rows = (uint32_t)rows;
    if (int rc = plan_dense(a, cfg, workspace != nullptr)) return rc;
    DenseWs ws = dense_ws(a.rows, a.in, a.out, a.part ? a.split : 0u, a.slice_max);
    bool has_ws = workspace != nullptr && workspace_bytes >= ws.total;
    if (a.part && !has_ws) {  // too small for the global exchange: the cluster kernel, with the rotated rows if those fit
        if (int rc = plan_dense(a, cfg, false)) return rc;
        ws = dense_ws(a.rows, a.in, a.out, 0u, a.slice_max);
        has_ws = workspace != nullptr && workspace_bytes >= ws.total;
    }
    a.err = dev_error_ptr();
    a.trace = g_trace;
    if (a.part) {
        a.part = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + ws.part);
        a.counters = reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(workspace) + ws.counters);
        if (int rc = cuda_status(cudaMemsetAsync(a.counters, 0, (size_t)(a.out / 128u) * 4u, static_cast<cudaStream_t>(stream)))) return rc;
    }
    a.x = x;
    a.y = y;
    if (prep_ahead(a.rows, a.slice_max) && !cfg.probe && has_ws) {
        a.xp_g = workspace;
        g_launches.fetch_add(1, std::memory_order_relaxed);
        if (int rc = cuda_status(launch_dense_prep(a, static_cast<cudaStream_t>(stream)))) return rc;
    }
    if (cfg.probe) {  // a timing probe in the served kernel's place: y is not the linear's output
        if (rows > 8) return T3_ENGINE_NOT_IMPLEMENTED;
        return cuda_status(launch_dense_gemv(a, 1 + cfg.probe, static_cast<cudaStream_t>(stream)));
    }
    return cuda_status(launch_dense_gemv(a, dec.codebook, static_cast<cudaStream_t>(stream)));
}

const char* t3_last_kernel_symbol(void) {
    const char* name = nullptr;
    if (!g_last_kernel || cudaFuncGetName(&name, g_last_kernel) != cudaSuccess) return "";
    return name ? name : "";
}

int t3_plan_linear(size_t rows, int in_dim, int out_dim, int n, t3_decode dec, t3_launch* out, int max_launches) {
    if (!out) return -T3_NULL_POINTER;
    if (in_dim <= 0 || out_dim <= 0 || in_dim % 128 != 0 || out_dim % 128 != 0 || !rate_ok(n) || rows < 1) return -T3_BAD_EXL3_SHAPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return -rc;
    if (rows > T3_DECODE_ROWS_MAX) return -T3_ENGINE_NOT_IMPLEMENTED;  // the plan covers the decode-row kernels
    if (max_launches < 1) return -T3_BAD_EXL3_SHAPE;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    DenseArgs a = {};
    a.in = (uint32_t)in_dim, a.out = (uint32_t)out_dim, a.n = (uint32_t)n, a.rows = (uint32_t)rows;
    if (int rc = plan_dense(a, cfg, true)) return -rc;
    const uint32_t rm = row_cap_for(a.rows);
    char symbol[64];
    std::snprintf(symbol, sizeof symbol, "t3_dense_gemv_%s_n%u_r%u", dec.codebook == T3_MCG ? "mcg" : "mul1", named_rate(a.n), rm);
    int k = 0;
    const bool ahead = prep_ahead(a.rows, a.slice_max);
    if (ahead) {  // with the call's workspace: the rows rotated once ahead of the GEMV
        if (max_launches < 2) return -T3_BAD_EXL3_SHAPE;
        fill_launch(&out[k++], "t3_dense_prep", "dense", dim3((a.rows * (a.in / 128u) + 3u) / 4u, 1, 1), 128u, 0u, 1u,
                    {T3_ROLE_X, T3_ROLE_SUH, T3_ROLE_XP});
    }
    if (ahead)
        fill_launch(&out[k++], symbol, "dense", dim3(a.split, a.out / 128u, 1), 32u * 17u,
                    gemv_smem_bytes(rm, a.rows, a.slice_max, a.part ? 1u : a.split, a.n, a.ring), a.part ? 1u : a.split,
                    {T3_ROLE_XP, T3_ROLE_Y, T3_ROLE_TRELLIS, T3_ROLE_SVH});
    else
        fill_launch(&out[k++], symbol, "dense", dim3(a.split, a.out / 128u, 1), 32u * 17u,
                    gemv_smem_bytes(rm, a.rows, a.slice_max, a.part ? 1u : a.split, a.n, a.ring), a.part ? 1u : a.split,
                    {T3_ROLE_X, T3_ROLE_Y, T3_ROLE_TRELLIS, T3_ROLE_SUH, T3_ROLE_SVH});
    if (a.part) out[k - 1].roles[out[k - 1].nroles++] = T3_ROLE_Z;  // the slices' partial sums meet in global memory
    return k;
}

// ---- routed experts -------------------------------------------------------------------------------------------------

namespace {

int validate_bank(const t3_bank* b, int hidden_of_x) {
    if (!b) return T3_NULL_POINTER;
    const t3_proj* ps[3] = {&b->gate, &b->up, &b->down};
    for (const t3_proj* p : ps)
        if (!p->trellis || !p->suh || !p->svh) return T3_NULL_POINTER;
    if (b->experts <= 0 || b->hidden <= 0 || b->inter <= 0 || b->hidden % 128 != 0 || b->inter % 128 != 0 ||
        b->hidden != hidden_of_x || !rate_ok(b->n_gate) || !rate_ok(b->n_up) || !rate_ok(b->n_down))
        return T3_BAD_EXL3_SHAPE;
    if (b->n_gate != b->n_up) return T3_GATE_UP_RATE_MISMATCH;
    if (b->n_gate != b->n_down) return T3_ENGINE_NOT_IMPLEMENTED;  // src/root.zig:841
    return T3_OK;
}

// The routed chain at decode rows on filled arguments (geometry, rows, top-k, pointers): plans the launches and records
// them. workspace: t3_moe_workspace_bytes(rows, topk, bank) bytes.
// The launch shapes of the routed chain at decode rows: row capacity of a pass, K splits, code rings. Geometry, rows and
// top-k set.
int plan_moe_decode(MoeArgs& a, const t3_config& cfg) {
    const size_t slots = (size_t)a.rows * a.topk;
    // Rows one pass over an expert's weights serves. Sized from the geometry's expected members an expert (rows * topk /
    // experts, with headroom), not from the row count: with many experts a 32-row call still has one or two rows an
    // expert, and a 32-row pass would pay four times the shared memory and twice the tensor-core steps for nothing. An
    // expert with more members than this takes further passes over its weights. A row's bytes do not depend on it.
    const uint32_t expect = (uint32_t)((4u * slots + a.experts - 1u) / a.experts) + 4u;
    const uint32_t rm = row_cap_for(expect < a.rows ? expect : a.rows);
    a.row_cap = rm;
    a.overlap = !cfg.no_overlap;
    // The K splits depend on hidden and inter only (sized as if a row had eight slots), never on the row count, the top-k
    // or the bank's size: a row-slot's summation order, hence its bytes, is the same alone and in a batch, and the same in
    // a one-expert bank (a shared expert, an expert-parallel rank's share) as in the whole bank. A shared expert's chain,
    // run on a second stream beside the routed chain, then launches the same cluster shapes as the routed one (measured:
    // a 2-CTA-cluster launch beside 4- or 8-CTA-cluster launches costs a 1-row layer 7 us).
    constexpr uint32_t kNominalSlots = 8;
    a.split_gu = pick_split(a.hidden / 128u, (a.inter / 128u) * kNominalSlots, 2u, 4u, one_wave() / 8u);
    a.slice_max_gu = largest_slice(a.hidden / 128u, a.split_gu);
    a.split_d = pick_split(a.inter / 128u, (a.hidden / 128u) * kNominalSlots, 1u, 8u, one_wave() / 8u);
    a.slice_max_d = largest_slice(a.inter / 128u, a.split_d);
    // sized for the widest row capacity so the split does not move with the rows either
    while (!plan_ring(32u, 32u, a.slice_max_gu, 2u * a.split_gu, a.n, a.ring_gu)) {
        if (a.split_gu * 2u > a.hidden / 128u || a.split_gu * 2u > 8u) return T3_ENGINE_NOT_IMPLEMENTED;
        a.split_gu *= 2u;
        a.slice_max_gu = largest_slice(a.hidden / 128u, a.split_gu);
    }
    while (!plan_ring(32u, 32u, a.slice_max_d, a.split_d, a.n, a.ring_d)) {
        if (a.split_d * 2u > a.inter / 128u || a.split_d * 2u > 16u) return T3_ENGINE_NOT_IMPLEMENTED;
        a.split_d *= 2u;
        a.slice_max_d = largest_slice(a.inter / 128u, a.split_d);
    }
    if (!plan_ring(rm, rm, a.slice_max_gu, 2u * a.split_gu, a.n, a.ring_gu) || !plan_ring(rm, rm, a.slice_max_d, a.split_d, a.n, a.ring_d))
        return T3_ENGINE_NOT_IMPLEMENTED;
    return T3_OK;
}

int decode_chain(MoeArgs a, const t3_config& cfg, int codebook, void* workspace, cudaStream_t s, void* shared_ready) {
    const size_t slots = (size_t)a.rows * a.topk;
    a.hd = workspace;
    a.v = static_cast<uint8_t*>(workspace) + align256(slots * a.inter * 2u);
    if (int rc = plan_moe_decode(a, cfg)) return rc;
    a.err = dev_error_ptr();
    if (int rc = cuda_status(launch_moe_gate_up(a, codebook, s))) return rc;
    if (a.topk == 1u) {
        // one slot a row: the down launch stores y itself (and adds `shared`), there is nothing to merge
        if (shared_ready)
            if (int rc = cuda_status(cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(shared_ready), 0))) return rc;
        return cuda_status(launch_moe_down(a, codebook, s));
    }
    if (int rc = cuda_status(launch_moe_down(a, codebook, s))) return rc;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (shared_ready)  // only the merge reads `shared`: the two GEMV launches above do not wait for it
        if (int rc = cuda_status(cudaStreamWaitEvent(s, static_cast<cudaEvent_t>(shared_ready), 0))) return rc;
    return cuda_status(launch_moe_merge(a, s));
}

int moe_call(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
             int scores_dtype, int topk, t3_decode dec, uint32_t limit, int clamp_at, const void* shared, void* y,
             void* workspace, size_t workspace_bytes, void* stream, void* shared_ready = nullptr) {
    if (!x || !inds || !scores || !y) return T3_NULL_POINTER;
    if (rows < 1 || rows > (size_t)1 << 30 || topk <= 0) return T3_BAD_EXL3_SHAPE;
    if (topk > T3_REDUCE_MAX_TOPK) return T3_BAD_EXL3_SHAPE;  // validateCall, src/root.zig:131
    if (int rc = validate_bank(bank, bank ? bank->hidden : 0)) return rc;
    if (!dtype_ok(x_dtype) || !dtype_ok(scores_dtype)) return T3_BAD_EXL3_DTYPE;
    if (clamp_at != T3_CLAMP_GATE_IN && clamp_at != T3_CLAMP_SILU_OUT) return T3_INVALID_CLAMP;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    if (rows > T3_DECODE_ROWS_MAX && !cfg.prefill) return T3_ENGINE_NOT_IMPLEMENTED;  // src/root.zig:850-852
    // the prefill chain's launches carry row groups in a grid dimension (65535 at most): 8 rows a group in the last launch,
    // 64 row-slots a group in the prepare and the middle
    if (rows > T3_DECODE_ROWS_MAX && (rows > kPrefillMoeRowsMax || rows * (size_t)topk > kPrefillSlotsMax)) return T3_BAD_EXL3_SHAPE;
    if (rows * (size_t)topk > 0x7FFFFFFFu / (size_t)(bank->hidden > bank->inter ? bank->hidden : bank->inter)) return T3_BAD_EXL3_SHAPE;
    const size_t need = t3_moe_workspace_bytes(rows, topk, bank);
    if (!workspace || workspace_bytes < need) return T3_WORKSPACE_TOO_SMALL;

    MoeArgs a = {};
    a.x = x;
    a.x_dt = x_dtype;
    a.inds = inds;
    a.scores = scores;
    a.score_dt = scores_dtype;
    a.gate_t = static_cast<const uint8_t*>(bank->gate.trellis);
    a.up_t = static_cast<const uint8_t*>(bank->up.trellis);
    a.down_t = static_cast<const uint8_t*>(bank->down.trellis);
    a.gate_suh = bank->gate.suh;
    a.gate_svh = bank->gate.svh;
    a.up_suh = bank->up.suh;
    a.up_svh = bank->up.svh;
    a.down_suh = bank->down.suh;
    a.down_svh = bank->down.svh;
    a.experts = (uint32_t)bank->experts;
    a.hidden = (uint32_t)bank->hidden;
    a.inter = (uint32_t)bank->inter;
    a.topk = (uint32_t)topk;
    a.rows = (uint32_t)rows;
    a.n = (uint32_t)bank->n_gate;
    a.mask = mask;
    a.limit = (float)limit;
    a.clamp_at = clamp_at;
    const size_t slots = rows * (size_t)topk;
    a.y = y;
    a.shared = shared;
    a.y_dt = x_dtype;
    a.shared_ready = shared_ready;
    a.err = dev_error_ptr();
    note_engine(rows > T3_DECODE_ROWS_MAX ? 2 : 0, ((uint64_t)a.hidden << 32) | a.inter, a.experts, a.n, a.topk);
    if (rows > T3_DECODE_ROWS_MAX) {
        int launches = 0;
        const cudaError_t rc = launch_prefill_moe(a, workspace, dec.codebook, static_cast<cudaStream_t>(stream), &launches);
        g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
        return cuda_status(rc);
    }
    return decode_chain(a, cfg, dec.codebook, workspace, static_cast<cudaStream_t>(stream), shared_ready);
}

}  // namespace

int t3_plan_moe(size_t rows, int topk, const t3_bank* bank, t3_decode dec, t3_launch* out, int max_launches) {
    if (!out || !bank) return -T3_NULL_POINTER;
    if (rows < 1 || topk <= 0 || topk > T3_REDUCE_MAX_TOPK) return -T3_BAD_EXL3_SHAPE;
    if (bank->experts <= 0 || bank->hidden <= 0 || bank->inter <= 0 || bank->hidden % 128 != 0 || bank->inter % 128 != 0 ||
        !rate_ok(bank->n_gate) || !rate_ok(bank->n_up) || !rate_ok(bank->n_down))
        return -T3_BAD_EXL3_SHAPE;
    if (bank->n_gate != bank->n_up) return -T3_GATE_UP_RATE_MISMATCH;
    if (bank->n_gate != bank->n_down) return -T3_ENGINE_NOT_IMPLEMENTED;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return -rc;
    if (rows > T3_DECODE_ROWS_MAX) return -T3_ENGINE_NOT_IMPLEMENTED;  // the plan covers the decode-row kernels
    const int count = topk == 1 ? 2 : 3;
    if (max_launches < count) return -T3_BAD_EXL3_SHAPE;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    MoeArgs a = {};
    a.experts = (uint32_t)bank->experts, a.hidden = (uint32_t)bank->hidden, a.inter = (uint32_t)bank->inter;
    a.topk = (uint32_t)topk, a.rows = (uint32_t)rows, a.n = (uint32_t)bank->n_gate;
    if (int rc = plan_moe_decode(a, cfg)) return -rc;
    const char* cb = dec.codebook == T3_MCG ? "mcg" : "mul1";
    const uint32_t rm = a.row_cap, slots = a.rows * a.topk;
    char symbol[64];
    std::snprintf(symbol, sizeof symbol, "t3_dec_gate_up_%s_n%u_r%u", cb, named_rate(a.n), rm);
    fill_launch(&out[0], symbol, "decode", dim3(2u * a.split_gu, a.inter / 128u, slots), 32u * 17u,
                gemv_smem_bytes(rm, rm, a.slice_max_gu, 2u * a.split_gu, a.n, a.ring_gu), 2u * a.split_gu,
                {T3_ROLE_X, T3_ROLE_SLOTS, T3_ROLE_GATE_T, T3_ROLE_UP_T, T3_ROLE_GATE_SUH, T3_ROLE_UP_SUH, T3_ROLE_GATE_SVH,
                 T3_ROLE_UP_SVH, T3_ROLE_DOWN_SUH, T3_ROLE_HD});
    std::snprintf(symbol, sizeof symbol, "t3_dec_down_%s_n%u_r%u", cb, named_rate(a.n), rm);
    if (topk == 1) {
        fill_launch(&out[1], symbol, "decode", dim3(a.split_d, a.hidden / 128u, slots), 32u * 17u,
                    gemv_smem_bytes(rm, rm, a.slice_max_d, a.split_d, a.n, a.ring_d), a.split_d,
                    {T3_ROLE_HD, T3_ROLE_SLOTS, T3_ROLE_DOWN_T, T3_ROLE_DOWN_SVH, T3_ROLE_SCORES, T3_ROLE_Y});
        return 2;
    }
    fill_launch(&out[1], symbol, "decode", dim3(a.split_d, a.hidden / 128u, slots), 32u * 17u,
                gemv_smem_bytes(rm, rm, a.slice_max_d, a.split_d, a.n, a.ring_d), a.split_d,
                {T3_ROLE_HD, T3_ROLE_SLOTS, T3_ROLE_DOWN_T, T3_ROLE_DOWN_SVH, T3_ROLE_ZD});
    fill_launch(&out[2], "t3_dec_merge", "decode", dim3((a.hidden + 255u) / 256u, a.rows, 1), 256u, 0u, 1u,
                {T3_ROLE_ZD, T3_ROLE_SCORES, T3_ROLE_Y});
    return 3;
}

size_t t3_moe_workspace_bytes(size_t rows, int topk, const t3_bank* bank) {
    if (!bank || topk <= 0 || bank->inter <= 0 || bank->hidden <= 0 || bank->experts <= 0) return 0;
    const size_t slots = rows * (size_t)topk;
    if (rows > T3_DECODE_ROWS_MAX)
        return prefill_moe_workspace(rows, (uint32_t)topk, (uint32_t)bank->experts, (uint32_t)bank->hidden, (uint32_t)bank->inter);
    return align256(slots * (size_t)bank->inter * 2u) + align256(slots * (size_t)bank->hidden * 2u);
}

int t3_moe(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
           int scores_dtype, int topk, t3_decode dec, void* y, void* workspace, size_t workspace_bytes, void* stream) {
    return moe_call(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, 0, T3_CLAMP_GATE_IN, nullptr, y,
                    workspace, workspace_bytes, stream);
}

int t3_moe_swiglu(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
                  int scores_dtype, int topk, t3_decode dec, uint32_t limit, int clamp_at, void* y, void* workspace,
                  size_t workspace_bytes, void* stream) {
    return moe_call(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, limit, clamp_at, nullptr, y, workspace,
                    workspace_bytes, stream);
}

int t3_moe_clamped(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
                   int scores_dtype, int topk, t3_decode dec, int limit, void* y, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (limit <= 0 || limit > 128) return T3_INVALID_CLAMP;
    return moe_call(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, (uint32_t)limit, T3_CLAMP_GATE_IN,
                    nullptr, y, workspace, workspace_bytes, stream);
}

int t3_moe_clamped_banked(const void* x, int x_dtype, size_t rows, const t3_bank* banks, const void* ids, t3_decode dec,
                          int limit, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !banks || !ids || !y) return T3_NULL_POINTER;
    if (limit <= 0 || limit > 128) return T3_INVALID_CLAMP;               // deepseek_v41/api.zig:249
    if (rows < 1 || rows > T3_BANKED_ROWS_MAX) return T3_BAD_EXL3_SHAPE;  // api.zig:349
    if (int rc = validate_bank(&banks[0], banks[0].hidden)) return rc;
    for (int b = 1; b < 3; ++b) {  // every bank at bank 0's widths and rates, its own slot count (api.zig:375-386)
        if (int rc = validate_bank(&banks[b], banks[0].hidden)) return rc;
        if (banks[b].inter != banks[0].inter || banks[b].n_gate != banks[0].n_gate || banks[b].n_down != banks[0].n_down)
            return T3_BAD_EXL3_SHAPE;
    }
    for (int b = 0; b < 3; ++b)
        if (banks[b].experts > 0x1000000) return T3_BAD_EXL3_SHAPE;  // a slot is 24 bits of the id
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return T3_BAD_EXL3_DTYPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    if (!workspace || workspace_bytes < t3_moe_workspace_bytes(rows < 32 ? rows : 32, 1, &banks[0])) return T3_WORKSPACE_TOO_SMALL;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    const t3_bank* bank = &banks[0];
    MoeArgs a = {};
    a.x_dt = x_dtype;
    a.gate_t = static_cast<const uint8_t*>(bank->gate.trellis);
    a.up_t = static_cast<const uint8_t*>(bank->up.trellis);
    a.down_t = static_cast<const uint8_t*>(bank->down.trellis);
    a.gate_suh = bank->gate.suh;
    a.gate_svh = bank->gate.svh;
    a.up_suh = bank->up.suh;
    a.up_svh = bank->up.svh;
    a.down_suh = bank->down.suh;
    a.down_svh = bank->down.svh;
    a.experts = (uint32_t)bank->experts;
    for (int b = 1; b < 3; ++b) {
        BankTab& t = a.ext[b - 1];
        t.gate_t = static_cast<const uint8_t*>(banks[b].gate.trellis);
        t.up_t = static_cast<const uint8_t*>(banks[b].up.trellis);
        t.down_t = static_cast<const uint8_t*>(banks[b].down.trellis);
        t.gate_suh = banks[b].gate.suh;
        t.gate_svh = banks[b].gate.svh;
        t.up_suh = banks[b].up.suh;
        t.up_svh = banks[b].up.svh;
        t.down_suh = banks[b].down.suh;
        t.down_svh = banks[b].down.svh;
        t.experts = (uint32_t)banks[b].experts;
    }
    a.banked = 1;
    a.hidden = (uint32_t)bank->hidden;
    a.inter = (uint32_t)bank->inter;
    a.topk = 1;
    a.n = (uint32_t)bank->n_gate;
    a.mask = mask;
    a.limit = (float)limit;
    a.clamp_at = T3_CLAMP_GATE_IN;
    a.y_dt = y_dtype;
    a.err = dev_error_ptr();
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const size_t xs = x_dtype == T3_F32 ? 4u : 2u, ys = y_dtype == T3_F32 ? 4u : 2u;
    // a skipped row-slot's y row is 0 (banked.skip_id): no CTA writes it
    if (int rc = cuda_status(cudaMemsetAsync(y, 0, rows * (size_t)a.hidden * ys, s))) return rc;
    note_engine(0, ((uint64_t)a.hidden << 32) | a.inter, a.experts, a.n, 1u << 8);
    // an id may name one slot for every row-slot of the call, and a pass over a slot's weights serves 32: two calls past 32
    for (size_t r0 = 0; r0 < rows; r0 += 32u) {
        a.rows = (uint32_t)(rows - r0 < 32u ? rows - r0 : 32u);
        a.x = static_cast<const uint8_t*>(x) + r0 * a.hidden * xs;
        a.inds = static_cast<const uint32_t*>(ids) + r0;
        a.y = static_cast<uint8_t*>(y) + r0 * a.hidden * ys;
        if (int rc = decode_chain(a, cfg, dec.codebook, workspace, s, nullptr)) return rc;
    }
    return T3_OK;
}

int t3_ep_plan(const void* inds, size_t rows, int topk, int experts, int world, void* order, void* where, void* send_rows,
               void* meta, void* counts, void* stream) {
    if (!inds || !order || !where || !send_rows || !meta || !counts) return T3_NULL_POINTER;
    if (rows < 1 || topk <= 0 || topk > T3_REDUCE_MAX_TOPK || rows * (size_t)topk > 0x7FFFFFFFu || experts <= 0 || world < 1 ||
        world > T3_EP_WORLD_MAX || experts % world != 0)
        return T3_BAD_EXL3_SHAPE;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_ep_plan(static_cast<const uint32_t*>(inds), (uint32_t)rows, (uint32_t)topk, (uint32_t)experts,
                                      (uint32_t)world, static_cast<uint32_t*>(order), static_cast<uint32_t*>(where),
                                      static_cast<uint32_t*>(send_rows), meta, static_cast<int*>(counts),
                                      static_cast<cudaStream_t>(stream)));
}

int t3_moe_merge_mapped(const void* v, const void* where, const void* scores, int scores_dtype, size_t rows, int topk, int hidden,
                        const void* shared, void* y, int y_dtype, void* stream);

int t3_moe_merge(const void* v, const void* scores, int scores_dtype, size_t rows, int topk, int hidden,
                 const void* shared, void* y, int y_dtype, void* stream) {
    return t3_moe_merge_mapped(v, nullptr, scores, scores_dtype, rows, topk, hidden, shared, y, y_dtype, stream);
}

int t3_moe_merge_mapped(const void* v, const void* where, const void* scores, int scores_dtype, size_t rows, int topk, int hidden,
                        const void* shared, void* y, int y_dtype, void* stream) {
    if (!v || !scores || !y) return T3_NULL_POINTER;
    if (rows < 1 || rows > 0x7FFFFFFFu / 32u || topk <= 0 || topk > T3_REDUCE_MAX_TOPK || hidden <= 0) return T3_BAD_EXL3_SHAPE;
    if (rows > 65535u) return T3_BAD_EXL3_SHAPE;  // one grid row a row
    if (!dtype_ok(scores_dtype) || !dtype_ok(y_dtype)) return T3_BAD_EXL3_DTYPE;
    MoeArgs a = {};
    a.v = const_cast<void*>(v);
    a.row_map = static_cast<const uint32_t*>(where);
    a.scores = scores;
    a.score_dt = scores_dtype;
    a.rows = (uint32_t)rows;
    a.topk = (uint32_t)topk;
    a.hidden = (uint32_t)hidden;
    a.shared = shared;
    a.y = y;
    a.x_dt = y_dtype;
    a.overlap = 0;
    g_launches.fetch_add(1, std::memory_order_relaxed);
    return cuda_status(launch_moe_merge(a, static_cast<cudaStream_t>(stream)));
}

int t3_moe_with_shared(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds,
                       const void* scores, int scores_dtype, int topk, t3_decode dec, const void* shared, void* y,
                       void* workspace, size_t workspace_bytes, void* stream) {
    if (!shared) return T3_NULL_POINTER;
    return moe_call(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, 0, T3_CLAMP_GATE_IN, shared, y,
                    workspace, workspace_bytes, stream);
}

int t3_moe_swiglu_rows(const void* x, int x_dtype, size_t x_rows, const void* row_map, size_t slots, const t3_bank* bank,
                       const void* inds, const void* scores, int scores_dtype, t3_decode dec, int limit, int clamp_at,
                       void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream) {
    if (!x || !row_map || !inds || !scores || !y) return T3_NULL_POINTER;
    if (limit < 0 || limit > 128) return T3_INVALID_CLAMP;                       // src/root.zig:1058
    if (clamp_at != T3_CLAMP_GATE_IN && clamp_at != T3_CLAMP_SILU_OUT) return T3_INVALID_CLAMP;
    if (x_rows < 1 || slots < 1 || slots > (size_t)1 << 30) return T3_BAD_EXL3_SHAPE;
    if (int rc = validate_bank(bank, bank ? bank->hidden : 0)) return rc;
    if (!dtype_ok(x_dtype) || !dtype_ok(scores_dtype) || !dtype_ok(y_dtype)) return T3_BAD_EXL3_DTYPE;
    t3_config cfg;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        cfg = g_cfg;
    }
    if (!cfg.prefill || slots <= T3_DECODE_ROWS_MAX) return T3_ENGINE_NOT_IMPLEMENTED;  // src/root.zig:1059,1066
    if (slots > kPrefillMoeRowsMax) return T3_BAD_EXL3_SHAPE;  // row groups of the last launch are a grid dimension
    if (bank->n_gate != bank->n_down) return T3_ENGINE_NOT_IMPLEMENTED;                 // src/root.zig:1074
    if (slots > 0x7FFFFFFFu / (size_t)(bank->hidden > bank->inter ? bank->hidden : bank->inter)) return T3_BAD_EXL3_SHAPE;
    uint32_t mask;
    if (int rc = decode_mask(dec, mask)) return rc;
    if (!workspace || workspace_bytes < t3_moe_workspace_bytes(slots, 1, bank)) return T3_WORKSPACE_TOO_SMALL;
    MoeArgs a = {};
    a.x = x;
    a.x_dt = x_dtype;
    a.inds = inds;
    a.scores = scores;
    a.score_dt = scores_dtype;
    a.gate_t = static_cast<const uint8_t*>(bank->gate.trellis);
    a.up_t = static_cast<const uint8_t*>(bank->up.trellis);
    a.down_t = static_cast<const uint8_t*>(bank->down.trellis);
    a.gate_suh = bank->gate.suh;
    a.gate_svh = bank->gate.svh;
    a.up_suh = bank->up.suh;
    a.up_svh = bank->up.svh;
    a.down_suh = bank->down.suh;
    a.down_svh = bank->down.svh;
    a.experts = (uint32_t)bank->experts;
    a.hidden = (uint32_t)bank->hidden;
    a.inter = (uint32_t)bank->inter;
    a.topk = 1;
    a.rows = (uint32_t)slots;
    a.n = (uint32_t)bank->n_gate;
    a.mask = mask;
    a.limit = (float)limit;
    a.clamp_at = clamp_at;
    a.y = y;
    a.y_dt = y_dtype;
    a.row_map = static_cast<const uint32_t*>(row_map);
    a.err = dev_error_ptr();
    note_engine(2, ((uint64_t)a.hidden << 32) | a.inter, a.experts, a.n, 1);
    int launches = 0;
    const cudaError_t rc = launch_prefill_moe(a, workspace, dec.codebook, static_cast<cudaStream_t>(stream), &launches);
    g_launches.fetch_add((uint64_t)launches, std::memory_order_relaxed);
    return cuda_status(rc);
}

int t3_moe_with_shared_after(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds,
                             const void* scores, int scores_dtype, int topk, t3_decode dec, const void* shared,
                             void* shared_ready, void* y, void* workspace, size_t workspace_bytes, void* stream) {
    if (!shared || !shared_ready) return T3_NULL_POINTER;
    return moe_call(x, x_dtype, rows, bank, inds, scores, scores_dtype, topk, dec, 0, T3_CLAMP_GATE_IN, shared, y,
                    workspace, workspace_bytes, stream, shared_ready);
}

}  // extern "C"
