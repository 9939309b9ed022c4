/* t3.h: the C ABI of the B200-native EXL3 projection engine.
 *
 * A drop-in for the projection entry points of davidtai/turboexl3 (a Zig library over Metal/HIP kernels): every call
 * below names the reference interface it replaces (file:line relative to the reference's root). Arguments are plain
 * pointers and sizes; device pointers are CUDA device addresses of the current device; `stream` is a cudaStream_t passed
 * as void*. No call allocates device memory except where it says so; scratch is a caller-provided workspace whose size
 * the matching *_workspace_bytes call returns. Weights are read in the pack's own layout, never copied or repacked:
 *   trellis  u16 [in/16, out/16, n]      (banks: [E, in/16, out/16, n]), n even in [16, 128], bits per weight = n/16
 *   suh      f16 [in]   svh  f16 [out]   (banks: [E, in], [E, out])
 * Every call validates before it launches anything and returns a t3_status; nothing is launched on a refusal
 * (the reference's rule, docs/core/api.md:10-12). Calls are stream-ordered and never synchronise the device.
 */
#ifndef T3_H
#define T3_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes. t3_status_name returns the reference's error names (src/root.zig:93-141, table/table.zig:591-593). */
typedef enum {
    T3_OK = 0,
    T3_BAD_EXL3_SHAPE = 1,          /* "BadExl3Shape" */
    T3_BAD_EXL3_DTYPE = 2,          /* "BadExl3Dtype" */
    T3_ENGINE_NOT_IMPLEMENTED = 3,  /* "Exl3EngineNotImplemented" */
    T3_ENGINE_CACHE_FULL = 4,       /* "Exl3EngineCacheFull" */
    T3_GATE_UP_RATE_MISMATCH = 5,   /* "Exl3GateUpRateMismatch" */
    T3_INVALID_CLAMP = 6,           /* "InvalidExl3Clamp" */
    T3_INVALID_CONFIG = 7,          /* "InvalidTurboexl3Config" */
    T3_KERNEL_CREATE_FAILED = 8,    /* "KernelCreateFailed" */
    T3_CUDA_ERROR = 9,              /* "CudaError" (the reference's "MlxError") */
    T3_TOPK_EXCEEDS_REDUCE_BANK = 10, /* "Exl3TopKExceedsReduceBank" (src/core/spec.zig:75-77) */
    T3_WORKSPACE_TOO_SMALL = 11,    /* "WorkspaceTooSmall" (no counterpart: the reference allocates its scratch) */
    T3_EXPERT_LAYOUT_UNSUPPORTED = 12, /* "ExpertLayoutUnsupported" (src/core/spec.zig:38-50) */
    T3_WINDOW_UNSUPPORTED = 13,     /* "Exl3WindowUnsupported" (src/core/spec.zig:48) */
    T3_NULL_POINTER = 14,           /* "NullPointer" */
    T3_SCRATCH_LIMIT_EXCEEDED = 15  /* "ScratchLimitExceeded" (t3_moe_noalloc: the call needs more than the built-in scratch) */
} t3_status;

const char* t3_status_name(int status);

/* Activation dtypes, numbered as the reference's native kernels number them (src/kernels/hip/common.hpp:21). */
typedef enum { T3_F32 = 0, T3_F16 = 1, T3_BF16 = 2 } t3_dtype;
/* src/core/format.zig:18-21 */
typedef enum { T3_MUL1 = 0, T3_MCG = 1 } t3_codebook;
/* src/core/format.zig:83 */
typedef enum { T3_CLAMP_GATE_IN = 0, T3_CLAMP_SILU_OUT = 1 } t3_clamp_at;

/* How a pack's trellis decodes (format.Decode, src/core/format.zig:72-78): codebook and codeword width 8..16. */
typedef struct {
    int codebook;     /* t3_codebook */
    int window_bits;  /* 16 unless the pack names a narrower search width */
} t3_decode;

/* One projection (root.Proj, src/root.zig:74): device pointers. */
typedef struct {
    const void* trellis;
    const void* suh;
    const void* svh;
} t3_proj;

/* A routed bank (root.Bank, src/root.zig:75) with the shapes the reference reads off its arrays
 * (root.bankGeometry, src/root.zig:104-126). */
typedef struct {
    t3_proj gate, up, down;
    int experts, hidden, inter;
    int n_gate, n_up, n_down;  /* halfwords per tile of each projection's trellis */
} t3_bank;

/* Dispatch constants a host reads (root.kernels, src/root.zig:66-71; src/core/spec.zig:59-61). */
#define T3_DECODE_ROWS_MAX 32   /* rows up to this take the in-register GEMV chain (the reference's is 16) */
#define T3_REDUCE_MAX_TOPK 32
int t3_uses_prefill_arm(size_t rows);                    /* spec.usesPrefillArm, src/core/spec.zig:63-65 */
int t3_admit_topk(uint32_t topk);                        /* spec.admitTopK, src/core/spec.zig:75-77 */
/* spec.trellisAdmitted, src/core/spec.zig:80-88: 1 when a stacked trellis shape fits the config */
int t3_trellis_admitted(const int* shape, int ndim, uint32_t experts, uint32_t in_dim, uint32_t out_dim, uint32_t n);

/* The pack's `expert_quant` block (spec.parseExpertQuant, src/core/spec.zig:38-50): n, codebook and window from the
 * model config's JSON text. */
typedef struct {
    uint32_t n;
    int codebook;
    int window_bits;
} t3_spec;
int t3_parse_expert_quant(const char* json, size_t len, t3_spec* out);

/* Process-wide configuration (core.config.Config / configure, src/core/config.zig:7-181), set before the first call.
 * Only the knobs that mean something on this backend exist. */
typedef struct {
    int prefill;             /* 0: rows past T3_DECODE_ROWS_MAX refuse Exl3EngineNotImplemented (Config.prefill) */
    uint32_t ring_bytes;     /* shared-memory bytes a GEMV CTA's code ring may take; 0 = default */
    uint32_t dense_split;    /* K slices of a dense GEMV cluster (1..16); 0 = choose from the shape */
    int no_overlap;          /* 1: launches wait for the stream's previous kernel to finish before they start (no
                                programmatic dependent launch); for measurements */
    int probe;               /* timing probes only, never a served kernel (decode.Geometry.probe, src/core/decode.zig:34-35):
                                t3_linear calls of up to 8 rows launch the dense GEMV with 1 the codebook hash skipped, 2 the
                                window extraction skipped too, 3 nothing but the code stream (a stage is released as soon
                                as it has landed); y is then NOT the linear's output. 0 = serve */
} t3_config;
void t3_config_default(t3_config* out);
int t3_configure(const t3_config* cfg);                  /* InvalidTurboexl3Config on a bad value */

/* Bits a kernel sets when one of its bounded waits ran out (the context stays usable). Synchronises `stream`. */
int t3_device_error(void* stream, uint32_t* bits_out, int clear);
/* Test hook: launches one warp that waits, with the kernels' own bounded wait, for a barrier phase nothing completes. After
 * about a second the wait gives up, bit 0 (a copy never landed) is set in the error word and the kernel returns: what a
 * stalled copy looks like to the host. Nothing faults and the context stays usable. */
int t3_selftest_wait_runs_out(void* stream);

/* W_hat: the inner f16 weight [in, out] (format.reconstructInner, src/core/format.zig:276-291;
 * Dense.dequantize, src/core/dense.zig:909-922). */
int t3_dequant(const void* trellis, int in_dim, int out_dim, int n, t3_decode dec, void* w_hat, void* stream);

/* Test hook, the reference's codebook kernel test (src/hip_tests.zig:24-57): all 65,536 codewords through the device
 * decoders, out[cw] = f16 bits (device pointer to 65,536 uint16). */
int t3_codebook_table(t3_decode dec, void* out, void* stream);

/* root.linear (src/root.zig:309-351): y [rows, out] in x's dtype for x [rows, in]. `workspace` may be null when
 * t3_linear_workspace_bytes returns 0 for the call (up to 8 rows). For 9 to 32 rows the workspace (rows x in f16, 256-byte
 * aligned) is OPTIONAL: with it the rows are rotated once by a launch of their own ahead of the GEMV, without it every CTA
 * rotates its own copy; the same bytes either way. Past 32 rows it is required (256-byte aligned): the prepared rows, and
 * for calls of up to 512 rows on a linear with few 128-column blocks the partial sums of the K slices such a call is cut
 * into (the slices meet there; the slice counts of the two arms, 33..256 and 257..512 rows, follow in and out alone, so a
 * row's bytes do not depend on the row count within an arm, nor past 512 rows). */
size_t t3_linear_workspace_bytes(size_t rows, int in_dim, int out_dim, int n);
int t3_linear(const void* x, int x_dtype, size_t rows, const void* trellis, const void* suh, const void* svh,
              int in_dim, int out_dim, int n, t3_decode dec, void* y, void* workspace, size_t workspace_bytes,
              void* stream);

/* root.moe (src/root.zig:822-825): routed SwiGLU experts. x [rows, hidden]; inds (int32/uint32) and scores
 * [rows, topk]; y [rows, hidden] in x's dtype. scores_dtype is a t3_dtype. Gate, up and down must share a rate. */
size_t t3_moe_workspace_bytes(size_t rows, int topk, const t3_bank* bank);
int t3_moe(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
           int scores_dtype, int topk, t3_decode dec, void* y, void* workspace, size_t workspace_bytes, void* stream);
/* root.moeSwiglu (src/root.zig:831-833): t3_moe with the SwiGLU clamp `limit` (0 none) at `clamp_at`. */
int t3_moe_swiglu(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
                  int scores_dtype, int topk, t3_decode dec, uint32_t limit, int clamp_at, void* y, void* workspace,
                  size_t workspace_bytes, void* stream);
/* root.moeClamped (src/root.zig:1001-1004): limit in 1..128 at gate_in, else InvalidExl3Clamp. */
int t3_moe_clamped(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
                   int scores_dtype, int topk, t3_decode dec, int limit, void* y, void* workspace,
                   size_t workspace_bytes, void* stream);
/* root.moeWithShared (src/root.zig:976-984): t3_moe plus an already gated shared expert [rows, hidden] in x's dtype,
 * added at the routed output's rounding point. */
int t3_moe_with_shared(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds,
                       const void* scores, int scores_dtype, int topk, t3_decode dec, const void* shared, void* y,
                       void* workspace, size_t workspace_bytes, void* stream);

/* root.moeSwigluRows / moeClampedRows (src/root.zig:1007-1094): the routed chain at top-1 over GATHERED rows, for an expert
 * streamer's prompt calls over its slot bank. Row-slot p reads x's row row_map[p] (x [x_rows, hidden]; row_map u32 [slots],
 * each below x_rows: the caller's routing, not checked), runs the expert at slot inds[p] at weight scores[p], and y
 * [slots, hidden] in y_dtype holds its output at row p. No gathered copy of x is made. Row p is, bit for bit, row p of
 * t3_moe_swiglu at top-1 over the gathered rows, y rounded once to y_dtype. More than 32 row-slots (a caller pads a smaller
 * call), else Exl3EngineNotImplemented; limit 0 (none) .. 128, else InvalidExl3Clamp. Workspace: t3_moe_workspace_bytes(slots, 1, bank). */
int t3_moe_swiglu_rows(const void* x, int x_dtype, size_t x_rows, const void* row_map, size_t slots, const t3_bank* bank,
                       const void* inds, const void* scores, int scores_dtype, t3_decode dec, int limit, int clamp_at,
                       void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* deepseek_v41.moeClampedBanked / moeClampedBankedAs (src/models/deepseek_v41/api.zig:173-218): t3_moe_clamped over an expert
 * streamer's three slot banks at decode rows. Row-slot r is one routed pair: x's row r through the expert at ids[r], packed
 * (bank << 24 | slot), at weight 1; y [rows, hidden] in y_dtype holds each pair's output (the caller weighs and sums). Each
 * pair's bytes are t3_moe_clamped's on its bank at top-1 with score 1, rounded once to y_dtype. banks: three t3_bank at one
 * geometry and rate, each its own slot count (a bank no id names may repeat another's arrays). ids u32 / i32 [rows], rows
 * 1..T3_BANKED_ROWS_MAX; an id equal to T3_BANKED_SKIP_ID runs no expert and its y row is 0 (banked.skip_id,
 * src/models/deepseek_v41/banked.zig:87); a bank past 2 or a slot past its bank's count is clamped into range.
 * limit 1..128, else InvalidExl3Clamp. Workspace: t3_moe_workspace_bytes(min(rows, 32), 1, &banks[0]). */
#define T3_BANKED_ROWS_MAX 64          /* banked.banked_rows_max, src/models/deepseek_v41/banked.zig:185 */
#define T3_BANKED_SKIP_ID 0xFFFFFFFFu
int t3_moe_clamped_banked(const void* x, int x_dtype, size_t rows, const t3_bank* banks, const void* ids, t3_decode dec,
                          int limit, void* y, int y_dtype, void* workspace, size_t workspace_bytes, void* stream);

/* t3_moe_with_shared for a shared-expert output that another stream is still computing: `shared_ready` is a cudaEvent_t
 * recorded on that stream after `shared` was written. Only the call's last launch (the one that adds `shared`) waits for
 * the event, so the routed experts' launches run beside the shared expert's. The reference's moeWithShared
 * (src/root.zig:976-984) is moe followed by one add and leaves this overlap to MLX's graph scheduler; a stream-ordered C
 * ABI has to be told. Works under stream capture (the event becomes a graph edge into the last node). */
int t3_moe_with_shared_after(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds,
                             const void* scores, int scores_dtype, int topk, t3_decode dec, const void* shared,
                             void* shared_ready, void* y, void* workspace, size_t workspace_bytes, void* stream);

/* The routed chain's last step on its own: y[row] = sum over the row's slots, in slot order, of score * v, in f32 with a
 * multiply and an add (ref.moeRow, src/core/ref.zig:106), stored in y_dtype, plus the optional shared-expert add.
 * v is f16 [rows * topk, hidden]: each row-slot's finished down projection, the unit an expert-parallel combine returns
 * (the reference's per-slot outputs that a caller combines: src/kernels/hip/decode/decode.hip:11-13). */
int t3_moe_merge(const void* v, const void* scores, int scores_dtype, size_t rows, int topk, int hidden,
                 const void* shared, void* y, int y_dtype, void* stream);
/* t3_moe_merge on v rows that lie in another order: slot s's row is v[where[s]] (where u32 [rows * topk]; an
 * expert-parallel combine returns the rows grouped by owning rank, and t3_ep_plan's `where` says which is which). The
 * sum still runs in slot order, so y is t3_moe_merge's bit for bit. */
int t3_moe_merge_mapped(const void* v, const void* where, const void* scores, int scores_dtype, size_t rows, int topk,
                        int hidden, const void* shared, void* y, int y_dtype, void* stream);

/* Expert-parallel dispatch plan of one rank's routing, on the device (no counterpart in the reference, which serves one
 * device; the split is by experts, expert e on rank e / (experts / world)). inds u32 / i32 [rows, topk] holds GLOBAL expert
 * ids. All outputs are grouped by destination rank in rank order, ascending slot inside a rank (slot = row * topk + k):
 *   order u32 [S]      the slot sent at position p          where u32 [S]   slot s's position (order's inverse)
 *   send_rows u32 [S]  the rows to send, each (rank, row) pair ONCE, rows ascending inside a rank (the first
 *                      counts[1][*] summed entries are used)
 *   meta i32 [S, 2]    per sent slot: its row as an index into its rank's group of rows, its expert's index on the owner
 *   counts i32 [2, world]  slots to each rank, rows to each rank — the one array the host has to read
 * world 1..T3_EP_WORLD_MAX, experts a multiple of world; one launch. */
#define T3_EP_WORLD_MAX 8
int t3_ep_plan(const void* inds, size_t rows, int topk, int experts, int world, void* order, void* where, void* send_rows,
               void* meta, void* counts, void* stream);

/* t3_moe without a workspace argument, for callers that cannot allocate device memory (a host whose memory pool owns the
 * whole GPU, a plugin that is only handed activations and weights). It has no counterpart in the reference, which
 * allocates its scratch through MLX. The scratch lives in a fixed device array inside the library image:
 * T3_NOALLOC_SCRATCH_BYTES on every GPU that loads the library, until the process exits. Decode rows only (rows <=
 * T3_DECODE_ROWS_MAX) and t3_moe_workspace_bytes(rows, topk, bank) <= T3_NOALLOC_SCRATCH_BYTES, else
 * ScratchLimitExceeded before anything is launched. It calls no cudaMalloc/cudaFree. The first call on a device looks up
 * the array's address (cudaGetSymbolAddress) and should come before any stream capture. All calls share the one array:
 * calls whose kernels can overlap on the GPU (other streams or threads) race; keep them on one stream. */
#define T3_NOALLOC_SCRATCH_BYTES (4u << 20)
int t3_moe_noalloc(const void* x, int x_dtype, size_t rows, const t3_bank* bank, const void* inds, const void* scores,
                   int scores_dtype, int topk, t3_decode dec, void* y, void* stream);

/* Measurement hook (the reference has probe kernels for the same purpose, src/core/decode.zig:34-35): when set to a
 * device array of 8 uint64, the next t3_linear launches at decode rows record the SM cycle counter of their CTA (0, 0) at:
 * [0] entry, [1] barriers initialised, [2] activations prepared, [3] first code stage landed, [4] GEMV done and partials
 * pushed, [5] cluster reduce complete, [6] outputs stored. Null switches it off. */
void t3_set_trace(void* device_u64x8);

/* The resident trunk (src/core/dense.zig:1323-1530: "memory for compute; a host's opt-in"): a trunk linear's W_hat decoded
 * once and kept, so calls past 32 rows run a plain tensor-core GEMM instead of decoding every tile again. The caller owns
 * the memory: t3_resident_bytes (dense.residentBytesOf, src/core/dense.zig:1342-1345: 2 bytes a weight) sizes it,
 * t3_resident_build fills it — W_hat TRANSPOSED, f16 [out, in], so both GEMM operands stream by TMA as K-major tiles —
 * and t3_linear_resident is t3_linear on it. As in the reference the kept weight is the per-call one bit for bit, and so
 * is every output. Decode rows (<= 32) read the codes, never W_hat: Exl3EngineNotImplemented here, use t3_linear. */
size_t t3_resident_bytes(int in_dim, int out_dim);
int t3_resident_build(const void* trellis, int in_dim, int out_dim, int n, t3_decode dec, void* w_hat_t, void* stream);
int t3_linear_resident(const void* x, int x_dtype, size_t rows, const void* w_hat_t, const void* suh, const void* svh,
                       int in_dim, int out_dim, void* y, void* workspace, size_t workspace_bytes, void* stream);

/* The un-rotated trunk (root.trunkUnrot, src/root.zig:380-420; dense.unrotCols / unrotRows / residentPlain,
 * src/core/dense.zig:1587-1690, 1261-1263): the linear taken out of the Hadamard basis once,
 *   W_std = diag(suh) H W_hat H diag(svh),
 * so a call past 32 rows is ONE plain tensor-core GEMM y = x W_std in x's dtype: no prepare, no finish. t3_unrot_build
 * fills w_std_t (t3_resident_bytes bytes) with W_std TRANSPOSED [out, in] in act_dtype (T3_F16 or T3_BF16): the butterflies
 * run in f32 in the reference kernels' order, times 1/128, suh[i], svh[o], one rounding (the device form of
 * format.reconstructPublic, src/core/format.zig:295-331, whose f32 sums run in another order). t3_linear_unrot: x
 * [rows, in] and y [rows, out] in the weight's dtype, f32 accumulation, one rounding of each output — the same linear map
 * as t3_linear with other roundings (a reordering, as the reference says of it). Up to 32 rows: Exl3EngineNotImplemented
 * (dense.unrot_min_rows: decode rows keep the trellis paths). x and w_std_t 16-byte aligned. */
int t3_unrot_build(const void* trellis, const void* suh, const void* svh, int in_dim, int out_dim, int n, t3_decode dec,
                   int act_dtype, void* w_std_t, void* stream);
int t3_linear_unrot(const void* x, int x_dtype, size_t rows, const void* w_std_t, int in_dim, int out_dim, void* y, void* stream);

/* The native kernel seam (src/hip/plan.zig:9-70: "the launches of turboexl3's kernels, from a shape alone: kernel symbol,
 * grid, block, shared bytes and arguments by role"). The decode-row kernels carry extern "C" names after the reference's
 * pattern t3_<group>_<kernel>_<profile>...:
 *   t3_dense_gemv_<mul1|mcg>_n<n>_r<8|16|32>   t3_dense_prep   t3_dec_gate_up_<..>_n<n>_r<..>   t3_dec_down_<..>_n<n>_r<..>
 *   t3_dec_merge
 * (n = halfwords a tile for the rates with kernels of their own, 0 for the run-time-rate kernels). t3_plan_linear and
 * t3_plan_moe give, without launching, the launches t3_linear / t3_moe would record for a decode-row call under the
 * current configuration: each kernel takes ONE argument block (DenseArgs / MoeArgs of csrc/t3_internal.h) whose buffers are
 * listed by role, numbered as plan.Role is. They return the number of launches written, or minus a t3_status. Prefill
 * rows (> T3_DECODE_ROWS_MAX): -Exl3EngineNotImplemented. t3_last_kernel_symbol names the kernel the calling thread's last
 * decode-row launch ran (so a test can hold the plan against the launches). */
typedef enum {
    T3_ROLE_X, T3_ROLE_SUH, T3_ROLE_SVH, T3_ROLE_TRELLIS, T3_ROLE_XP, T3_ROLE_XS, T3_ROLE_Z, T3_ROLE_Y,
    T3_ROLE_SLOTS, T3_ROLE_SCORES, T3_ROLE_GATE_T, T3_ROLE_UP_T, T3_ROLE_DOWN_T, T3_ROLE_GATE_SUH, T3_ROLE_UP_SUH,
    T3_ROLE_GATE_SVH, T3_ROLE_UP_SVH, T3_ROLE_DOWN_SUH, T3_ROLE_DOWN_SVH,
    T3_ROLE_XG, T3_ROLE_XU, T3_ROLE_SG, T3_ROLE_SU, T3_ROLE_ZG, T3_ROLE_ZU, T3_ROLE_HD, T3_ROLE_HS, T3_ROLE_ZD,
    T3_ROLE_ORDER, T3_ROLE_INV, T3_ROLE_ITEMS, T3_ROLE_COUNTS
} t3_role;
typedef struct t3_launch {
    char symbol[64];    /* the kernel's name in the library's device code */
    char group[16];     /* "dense" | "decode" (plan.Launch.group) */
    uint32_t grid[3];
    uint32_t block;
    uint32_t shared;    /* dynamic shared-memory bytes */
    uint32_t cluster;   /* CTAs of a thread-block cluster along grid x; 1 = none */
    int nroles;
    int roles[24];      /* t3_role of every buffer the launch reads or writes */
} t3_launch;
int t3_plan_linear(size_t rows, int in_dim, int out_dim, int n, t3_decode dec, t3_launch* out, int max_launches);
int t3_plan_moe(size_t rows, int topk, const t3_bank* bank, t3_decode dec, t3_launch* out, int max_launches);
const char* t3_last_kernel_symbol(void);

/* root.enginesHeld / root.releaseEngines (src/root.zig:1148-1192). The reference caches a compiled engine per geometry and
 * frees them on request; here kernels are compiled ahead and a plan is recomputed per call, so an "engine" is only the
 * record that a geometry was served on a path. The counts are distinct geometries since the last release. */
typedef struct t3_engines {
    size_t decode;  /* routed GEMV chains (rows <= 32) */
    size_t dense;   /* dense linears at decode rows */
    size_t prefill; /* dense and routed calls past 32 rows */
} t3_engines;
void t3_engines_held(t3_engines* out);
void t3_release_engines(void);

/* Kernels this library launched since the process started (for benches that must report their launch count). */
uint64_t t3_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
