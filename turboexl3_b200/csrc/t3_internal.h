// Host-side declarations shared by the library's translation units (not part of the public C ABI).
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace t3 {

struct RingPlan {
    uint32_t stage_rows, stages;
};

// One dense linear at decode rows (rows <= 32)
struct DenseArgs {
    const void* x;            // [rows, in], dtype x_dt
    const void* xp_g;         // or null: the rows already prepared (f16 [rows, in], lane order inside every 16) by t3_dense_prep,
                              // which the CTAs copy in instead of rotating x themselves (calls of more than 8 rows)
    void* y;                  // [rows, out], dtype x_dt
    const uint8_t* trellis;   // [in/16, out/16, n] u16
    const void* suh;          // f16 [in]
    const void* svh;          // f16 [out]
    uint32_t rows, in, out, n, mask;
    int x_dt;
    float* part;              // or null. Set: the K slices' partial sums meet in global memory, [out/128][split][rows][128] f32, not
                              // in a cluster's shared memory (any slice count, CTAs placed one by one: large linears whose
                              // CTA count then fills the multiprocessors evenly)
    uint32_t* counters;       // with part: [out/128] arrivals a block, zero before the launch; the last arriver finishes the block
    uint32_t split;           // K slices (the cluster size unless `part` is set)
    uint32_t slice_max;       // inputs of the largest K slice
    RingPlan ring;
    int overlap;              // launch with the programmatic-dependent-launch attribute
    uint32_t* err;
    unsigned long long* trace;  // optional: SM cycle counts at the phases of CTA (0, 0) (see t3_set_trace)
};

// One more bank of a banked call (an expert streamer's slot banks: the same geometry and rate, its own slot count)
struct BankTab {
    const uint8_t *gate_t, *up_t, *down_t;
    const void *gate_suh, *gate_svh, *up_suh, *up_svh, *down_suh, *down_svh;
    uint32_t experts;
};
constexpr uint32_t kSkipId = 0xFFFFFFFFu;  // a banked call's id for a row-slot that runs no expert

// The routed chain at decode rows (rows <= 32): row-slot s = row * topk + k runs expert inds[s]
struct MoeArgs {
    const void* x;            // [rows, hidden], dtype x_dt
    int x_dt;
    const void* inds;         // [rows * topk] i32/u32
    const void* scores;       // [rows * topk], dtype score_dt
    int score_dt;
    const uint8_t *gate_t, *up_t, *down_t;
    const void *gate_suh, *gate_svh, *up_suh, *up_svh, *down_suh, *down_svh;  // f16, expert-major
    uint32_t experts, hidden, inter, topk, rows, n, mask;
    float limit;              // SwiGLU clamp, 0 = none
    int clamp_at;             // 0 gate_in, 1 silu_out
    void* hd;                 // scratch f16 [rows * topk, inter]: the down projection's prepared inputs
    void* v;                  // scratch f16 [rows * topk, hidden]: each row-slot's finished down output
    void* y;                  // [rows, hidden], dtype x_dt
    const void* shared;       // optional [rows, hidden] dtype x_dt added at y's rounding point, or null
    const uint32_t* row_map;  // prefill rows only: row-slot p reads x's row row_map[p] (top-1 over gathered rows), or null
    int y_dt;                 // y's dtype: x_dt, except for the gathered-rows and banked entries
    uint32_t banked;          // decode rows, top-1: inds holds packed ids (bank << 24 | slot); banks 1 and 2 in ext; scores null = 1
    BankTab ext[2];
    void* shared_ready;       // host side only: an event the last launch (the one that reads `shared`) waits for, or null
    uint32_t row_cap;                  // rows one pass over an expert's weights serves (8, 16 or 32): experts with more members take more passes
    uint32_t split_gu, slice_max_gu;   // K slices of gate|up (cluster = 2 * split_gu), largest slice
    uint32_t split_d, slice_max_d;     // K slices of down
    RingPlan ring_gu, ring_d;
    int overlap;
    uint32_t* err;
};

// remembers, per host thread, the kernel a decode-row launch is about to run (t3_last_kernel_symbol names it)
void note_symbol(const void* kernel);

cudaError_t launch_dense_gemv(const DenseArgs& a, int codebook, cudaStream_t stream);
// the input rotation of every row once, into a.xp_g (ahead of launch_dense_gemv on the same stream)
cudaError_t launch_dense_prep(const DenseArgs& a, cudaStream_t stream);
constexpr uint32_t kFusedRows = 8;  // up to this many rows a dense decode-row CTA rotates x itself
cudaError_t launch_moe_gate_up(const MoeArgs& a, int codebook, cudaStream_t stream);
cudaError_t launch_moe_down(const MoeArgs& a, int codebook, cudaStream_t stream);
cudaError_t launch_moe_merge(const MoeArgs& a, cudaStream_t stream);

// shared-memory bytes the GEMV CTAs of a plan need (for admission before launch)
uint32_t gemv_smem_bytes(uint32_t row_cap, uint32_t xrows, uint32_t slice_max, uint32_t cluster, uint32_t n, RingPlan ring);
// the most dynamic shared memory a GEMV CTA may be launched with
constexpr uint32_t kGemvSmemLimit = 200u * 1024u;
uint32_t row_cap_for(uint32_t rows);

// Row limits of the prefill launches, whose row groups are a grid dimension (65535 at most): the dense prepare takes 64
// rows a group; the routed chain's last launch 8 rows a group, its prepare and middle 64 row-slots a group.
constexpr size_t kPrefillDenseRowsMax = (size_t)65535 * 64;
constexpr size_t kPrefillMoeRowsMax = (size_t)65535 * 8;
constexpr size_t kPrefillSlotsMax = (size_t)65535 * 64;

// One dense linear at prefill rows (rows > 32): prepare -> tcgen05 GEMM with the decode in its weight loader -> finish
struct PrefillLinearArgs {
    const void* x;
    void* y;
    const uint8_t* trellis;
    const void* resident;  // W_hat transposed, f16 [out, in], kept by the caller: the GEMM loads it instead of decoding; or null
    const void* suh;
    const void* svh;
    uint32_t rows, in, out, n, mask;
    int x_dt;
    void* workspace;  // prefill_linear_workspace bytes
    uint32_t* err;
};
size_t prefill_linear_workspace(size_t rows, uint32_t in, uint32_t out);
cudaError_t launch_prefill_linear(const PrefillLinearArgs& p, int codebook, cudaStream_t stream, int* launches);
// The routed chain at prefill rows: route -> prepare -> GEMM(gate|up) -> mid -> GEMM(down) -> finish
size_t prefill_moe_workspace(size_t rows, uint32_t topk, uint32_t experts, uint32_t hidden, uint32_t inter);
cudaError_t launch_prefill_moe(const MoeArgs& a, void* workspace, int codebook, cudaStream_t stream, int* launches);

// W_hat f16 from the trellis: [in, out], or transposed [out, in]
cudaError_t launch_dequant(const uint8_t* trellis, uint32_t in, uint32_t out, uint32_t n, uint32_t mask, int codebook,
                           int transposed, void* what, cudaStream_t stream);
// W_hat transposed [out, in] f16 -> W_std transposed in dtype dt (f16 / bf16), in place: diag(suh) H W_hat H diag(svh)
cudaError_t launch_unrot(void* w_t, const void* suh, const void* svh, uint32_t in, uint32_t out, int dt, cudaStream_t stream);
// y = x W_std (x and the weight in the same 16-bit dtype, f32 accumulation, one rounding): the plain tensor-core GEMM
cudaError_t launch_plain_linear(const void* x, int dt, uint32_t rows, const void* w_std_t, uint32_t in, uint32_t out, void* y,
                                uint32_t* err, cudaStream_t stream);
// the expert-parallel dispatch plan of one rank's routing (see ep_plan_kernel); world 1..8, experts a multiple of world
cudaError_t launch_ep_plan(const uint32_t* inds, uint32_t rows, uint32_t topk, uint32_t experts, uint32_t world, uint32_t* order,
                           uint32_t* where, uint32_t* send_rows, void* meta, int* counts, cudaStream_t stream);
// test hook: a one-warp kernel whose bounded wait runs out (about a second) and sets the full-wait bit of `err`
cudaError_t launch_wait_runs_out(uint32_t* err, cudaStream_t stream);
// all 65,536 codewords through the kernels' decoders: out[cw] = f16 bits (test hook)
cudaError_t launch_codebook_table(int codebook, uint32_t mask, uint16_t* out, cudaStream_t stream);

}  // namespace t3
