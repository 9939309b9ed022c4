// Host-side declarations shared by the library's translation units (not part of the public C ABI).
#pragma once

#include <cuda_fp16.h>
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
    void* y;                  // [rows, out], dtype x_dt
    const uint8_t* trellis;   // [in/16, out/16, n] u16
    const void* suh;          // f16 [in]
    const void* svh;          // f16 [out]
    const __half* xp_g;       // the prepared rows f16 [rows, in] (lane order) when a prepare launch ran first, else null
    uint32_t rows, in, out, n, mask;
    int x_dt;
    uint32_t split;           // cluster size: K slices (a function of the geometry only, never of the rows)
    uint32_t chunk_blocks;    // 128-input blocks of prepared rows a CTA holds at once (>= a slice's blocks when xp_g is null)
    uint32_t xp_bufs;         // 1, or 2 when a slice takes several chunks
    uint32_t recv_bufs;       // 1, or 2 when a cluster walks more than one output block
    uint32_t dq_stages;       // ring stages a warp decodes ahead of the dependency wait
    RingPlan ring;
    int overlap;              // launch with the programmatic-dependent-launch attribute
    uint32_t* err;
    unsigned long long* trace;  // optional: 8 timestamps a CTA (see t3_set_trace)
};
constexpr uint32_t kTraceCtas = 512;   // CTAs of a launch whose timestamps are kept
constexpr uint32_t kTraceWords = 16;   // uint64 a CTA
constexpr uint32_t kFusedRows = 8;     // up to this many rows are rotated inside the GEMV's CTAs

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
    int y_dt;                 // prefill rows only: y's dtype (the decode-row chain stores y in x_dt)
    void* shared_ready;       // host side only: an event the last launch (the one that reads `shared`) waits for, or null
    uint32_t row_cap;                  // rows one pass over an expert's weights serves (8, 16 or 32): experts with more members take more passes
    uint32_t split_gu, slice_max_gu;   // K slices of gate|up (cluster = 2 * split_gu), largest slice
    uint32_t split_d, slice_max_d;     // K slices of down
    RingPlan ring_gu, ring_d;
    int overlap;
    uint32_t* err;
};

// the dense decode-row kernel: clusters to launch, the CTA's shared-memory bytes (dense_smem().total + kSmemSlack)
cudaError_t launch_dense_rows(const DenseArgs& a, int codebook, uint32_t rm, uint32_t clusters, uint32_t smem_bytes,
                              cudaStream_t stream);
// clusters of `split` such CTAs that the current device holds at once (0 when the query fails)
int dense_rows_max_clusters(int codebook, uint32_t n, uint32_t rm, bool prepared, uint32_t split, uint32_t smem_bytes);
// xp = the input rotation of every row (f16, lane order), for calls whose rows are not rotated inside the GEMV's CTAs
cudaError_t launch_dense_prepare(const void* x, int x_dt, const void* suh, uint32_t rows, uint32_t in, void* xp, bool overlap,
                                 cudaStream_t stream);
cudaError_t launch_moe_gate_up(const MoeArgs& a, int codebook, cudaStream_t stream);
cudaError_t launch_moe_down(const MoeArgs& a, int codebook, cudaStream_t stream);
cudaError_t launch_moe_merge(const MoeArgs& a, cudaStream_t stream);

// shared-memory bytes the GEMV CTAs of a plan need (for admission before launch)
uint32_t gemv_smem_bytes(uint32_t row_cap, uint32_t slice_max, uint32_t cluster, uint32_t n, RingPlan ring);
// the most dynamic shared memory a GEMV CTA may be launched with
constexpr uint32_t kGemvSmemLimit = 200u * 1024u;
uint32_t row_cap_for(uint32_t rows);

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
// all 65,536 codewords through the kernels' decoders: out[cw] = f16 bits (test hook)
cudaError_t launch_codebook_table(int codebook, uint32_t mask, uint16_t* out, cudaStream_t stream);

}  // namespace t3
