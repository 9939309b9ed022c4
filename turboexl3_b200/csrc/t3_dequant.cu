// W_hat: the trellis decoded to the inner (un-rotated) f16 weight [in, out], bit for bit what turboexl3's host
// reference reconstructs (format.reconstructInner, src/core/format.zig:276-291; the reference's kernel of the same job is
// turboexl3_dense_dequant, src/core/dense.zig:65-71). Used by the bit-exact decode check and by the dense prefill path.
//
// grid (out / 128, in / 16), 256 threads: warp w decodes tile (tk, 8 bx + w) from global memory in registers, the CTA
// transposes the 16 x 128 strip through shared memory and writes whole 256-byte rows.
#include <atomic>

#include "t3_common.cuh"
#include "t3_internal.h"

namespace t3 {
namespace {

constexpr uint32_t kStripStride = 128 + 8;  // halfs per strip row (padding spreads the 2-byte scatter over banks)

template <int N, int CB>
__global__ void __launch_bounds__(256) dequant_kernel(const uint8_t* __restrict__ trellis, uint32_t in, uint32_t out,
                                                      uint32_t n, uint32_t mask, int transposed, __half* __restrict__ what) {
    __shared__ __align__(16) uint16_t strip[16 * kStripStride];
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t tk = blockIdx.y, tn = blockIdx.x * 8u + warp, out_tiles = out / 16u;
    const uint32_t* tile = reinterpret_cast<const uint32_t*>(trellis + ((size_t)tk * out_tiles + tn) * 2u * n);
    uint32_t b[4];
    if (N > 0) {
        LanePlan<(N > 0 ? N : 16)> plan;
        plan.init(lane);
        decode_lane<(N > 0 ? N : 16), CB>(tile, plan, mask, b);
    } else {
        decode_lane_any<CB>(tile, n, lane, mask, b);
    }
#pragma unroll
    for (uint32_t m = 0; m < 8u; ++m)
        strip[tile_row(lane, m) * kStripStride + warp * 16u + tile_col(lane, m)] = (uint16_t)(b[m >> 1] >> ((m & 1u) * 16u));
    __syncthreads();
    if (!transposed) {
        const uint32_t r = tid >> 4, c = (tid & 15u) * 8u;  // 16 rows x 16 chunks of 8 halfs
        const uint4 v = *reinterpret_cast<const uint4*>(&strip[r * kStripStride + c]);
        *reinterpret_cast<uint4*>(what + ((size_t)tk * 16u + r) * out + blockIdx.x * 128u + c) = v;
    } else {
        // [out, in]: output column c's 16 inputs of this tile row are 32 contiguous bytes; a thread writes half of them
        const uint32_t c = tid >> 1, r0 = (tid & 1u) * 8u;
        uint32_t w[4];
#pragma unroll
        for (uint32_t i = 0; i < 4u; ++i)
            w[i] = (uint32_t)strip[(r0 + 2u * i) * kStripStride + c] | ((uint32_t)strip[(r0 + 2u * i + 1u) * kStripStride + c] << 16);
        *reinterpret_cast<uint4*>(what + (size_t)(blockIdx.x * 128u + c) * in + tk * 16u + r0) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}


// The un-rotated weight (the reference's turboexl3_unrot_cols / turboexl3_unrot_rows, src/core/dense.zig:1587-1630 and
// src/core/kernels/dense/unrot_cols.metal, unrot_rows.metal): W_std = diag(suh) H W_hat H diag(svh), one 128 x 128 tile at a
// time. wt is W_hat TRANSPOSED [out, in] f16 and is overwritten in place with W_std transposed in `dt` (f16 or bf16): the
// CTA holds its tile in shared memory as f32, runs the unscaled +-1 butterfly along the output index of every input row,
// then along the input index of every output column (the reference's order and statement order: lane L holds elements
// L + 32 j, five exchange stages over the lane bits, then the four-point stage), multiplies by 1/128, suh[i] and svh[o] in
// that order in f32 and rounds once.
// grid (in / 128, out / 128), 256 threads, 128 x 129 floats of dynamic shared memory.
constexpr uint32_t kUnrotStride = 129;
__global__ void __launch_bounds__(256) unrot_tile_kernel(uint16_t* wt, const __half* __restrict__ suh,
                                                         const __half* __restrict__ svh, uint32_t in, int dt) {
    extern __shared__ float tile[];  // tile[o][i]
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t i0 = blockIdx.x * 128u, o0 = blockIdx.y * 128u;
    for (uint32_t e = tid; e < 128u * 64u; e += 256u) {  // two inputs a load, a row of the tile a pass of 64 threads
        const uint32_t o = e >> 6, i = (e & 63u) * 2u;
        const __half2 h = *reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(wt) + (size_t)(o0 + o) * in + i0 + i);
        tile[o * kUnrotStride + i] = __low2float(h);
        tile[o * kUnrotStride + i + 1u] = __high2float(h);
    }
    __syncthreads();
    for (uint32_t i = warp; i < 128u; i += 8u) {  // along the outputs of input row i
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = tile[(lane + 32u * j) * kUnrotStride + i];
        h128_warp(v, lane);
#pragma unroll
        for (int j = 0; j < 4; ++j) tile[(lane + 32u * j) * kUnrotStride + i] = v[j];
    }
    __syncthreads();
    for (uint32_t o = warp; o < 128u; o += 8u) {  // along the inputs of output column o, then scale, round, store
        float v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] = tile[o * kUnrotStride + lane + 32u * j];
        h128_warp(v, lane);
        const float sv = __half2float(svh[o0 + o]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t i = i0 + lane + 32u * j;
            const float w = v[j] * 0.0078125f * __half2float(suh[i]) * sv;
            uint16_t bits;
            if (dt == (int)kBf16) {
                const __nv_bfloat16 b = __float2bfloat16_rn(w);
                bits = *reinterpret_cast<const uint16_t*>(&b);
            } else {
                const __half b = __float2half_rn(w);
                bits = *reinterpret_cast<const uint16_t*>(&b);
            }
            wt[(size_t)(o0 + o) * in + i] = bits;
        }
    }
}


// ---- expert-parallel dispatch plan ---------------------------------------------------------------------------------
// One CTA of 1024 threads. Slot s = row * topk + k goes to rank d = expert / per (clamped). Outputs, all grouped by
// destination rank in rank order, stable (ascending slot inside a rank):
//   order[p]      the slot sent at position p;          where[s]  the position of slot s (order's inverse)
//   meta[p]       (the slot's row as an index into its destination's group of rows, the expert's index on its owner)
//   send_rows[q]  the rows to send: each (destination, row) pair once, rows ascending inside a destination
//   counts[0][d]  slots to rank d;                       counts[1][d]  rows to rank d
// Thread t owns a run of consecutive rows; two passes over them with a block-wide exclusive scan of the per-rank counts
// between (world <= kEpWorldMax so the counters stay in registers).
constexpr uint32_t kEpWorldMax = 8;
struct EpPlanArgs {
    const uint32_t* inds;
    uint32_t rows, topk, per, world;
    uint32_t *order, *where, *send_rows;
    int2* meta;
    int* counts;  // [2][world]
};
__global__ void __launch_bounds__(1024) ep_plan_kernel(const EpPlanArgs a) {
    __shared__ uint32_t s_warp[2][kEpWorldMax][32];
    __shared__ uint32_t s_total[2][kEpWorldMax], s_base[2][kEpWorldMax];
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t chunk = (a.rows + 1023u) / 1024u;
    const uint32_t r0 = min(tid * chunk, a.rows), r1 = min(r0 + chunk, a.rows);
    uint32_t cs[kEpWorldMax], cr[kEpWorldMax];
#pragma unroll
    for (uint32_t d = 0; d < kEpWorldMax; ++d) cs[d] = cr[d] = 0u;
    for (uint32_t r = r0; r < r1; ++r) {
        uint32_t seen = 0u;
        for (uint32_t k = 0; k < a.topk; ++k) {
            const uint32_t d = min(a.inds[(size_t)r * a.topk + k] / a.per, a.world - 1u);
            seen |= 1u << d;
#pragma unroll
            for (uint32_t q = 0; q < kEpWorldMax; ++q) cs[q] += (q == d);
        }
#pragma unroll
        for (uint32_t q = 0; q < kEpWorldMax; ++q) cr[q] += (seen >> q) & 1u;
    }
    // exclusive scan over the threads, per rank, of both counters
    uint32_t bs[kEpWorldMax], br[kEpWorldMax];
#pragma unroll
    for (uint32_t d = 0; d < kEpWorldMax; ++d) {
        uint32_t vs = cs[d], vr = cr[d];
#pragma unroll
        for (uint32_t off = 1; off < 32u; off <<= 1) {
            const uint32_t ps = __shfl_up_sync(0xFFFFFFFFu, vs, off), pr = __shfl_up_sync(0xFFFFFFFFu, vr, off);
            if (lane >= off) vs += ps, vr += pr;
        }
        if (lane == 31u) s_warp[0][d][warp] = vs, s_warp[1][d][warp] = vr;
        bs[d] = vs - cs[d];
        br[d] = vr - cr[d];
    }
    __syncthreads();
    if (warp < 2u * kEpWorldMax) {  // warp w scans the 32 warp totals of counter w / 8, rank w % 8
        const uint32_t which = warp / kEpWorldMax, d = warp % kEpWorldMax;
        const uint32_t own = s_warp[which][d][lane];
        uint32_t v = own;
#pragma unroll
        for (uint32_t off = 1; off < 32u; off <<= 1) {
            const uint32_t p = __shfl_up_sync(0xFFFFFFFFu, v, off);
            if (lane >= off) v += p;
        }
        s_warp[which][d][lane] = v - own;
        if (lane == 31u) s_total[which][d] = v;
    }
    __syncthreads();
    if (tid < 2u) {  // where each rank's group starts
        uint32_t run = 0;
        for (uint32_t d = 0; d < kEpWorldMax; ++d) {
            s_base[tid][d] = run;
            run += s_total[tid][d];
        }
    }
    if (tid < 2u * a.world) a.counts[tid] = (int)s_total[tid / a.world][tid % a.world];
    __syncthreads();
#pragma unroll
    for (uint32_t d = 0; d < kEpWorldMax; ++d) {
        bs[d] += s_warp[0][d][warp];  // now: slots of rank d ahead of this thread's
        br[d] += s_warp[1][d][warp];  // rows of rank d ahead of this thread's
    }
    for (uint32_t r = r0; r < r1; ++r) {
        uint32_t seen = 0u;
        for (uint32_t k = 0; k < a.topk; ++k) {
            const uint32_t s = r * a.topk + k, e = a.inds[s];
            const uint32_t d = min(e / a.per, a.world - 1u);
            uint32_t at = 0, grp = 0;
#pragma unroll
            for (uint32_t q = 0; q < kEpWorldMax; ++q)
                if (q == d) at = bs[q]++, grp = br[q];
            const uint32_t p = s_base[0][d] + at;
            a.order[p] = s;
            a.where[s] = p;
            a.meta[p] = make_int2((int)grp, (int)(min(e, a.per * a.world - 1u) - d * a.per));
            if (!((seen >> d) & 1u)) a.send_rows[s_base[1][d] + grp] = r;
            seen |= 1u << d;
        }
#pragma unroll
        for (uint32_t q = 0; q < kEpWorldMax; ++q) br[q] += (seen >> q) & 1u;
    }
}

template <int CB>
__global__ void codebook_table_kernel(uint32_t mask, uint16_t* out) {
    const uint32_t cw = 2u * (blockIdx.x * blockDim.x + threadIdx.x);
    if (cw >= 65536u) return;
    const uint32_t w = decode2<CB>(cw & mask, (cw + 1u) & mask);
    out[cw] = (uint16_t)w;
    out[cw + 1u] = (uint16_t)(w >> 16);
}

// One warp waits, with the kernels' own bounded wait, for a barrier phase that nothing completes: the wait runs out, the
// error word gets `bit`, the kernel returns and the context stays usable (what a stalled copy would look like to the host).
__global__ void wait_runs_out_kernel(uint32_t* err, uint32_t bit) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1u);
        mbar_init_fence();
    }
    __syncthreads();
    if (threadIdx.x == 0) mbar_wait_report(smem_addr(&bar), 0u, err, bit);
}

template <int CB>
cudaError_t launch_dequant_cb(const uint8_t* trellis, uint32_t in, uint32_t out, uint32_t n, uint32_t mask, int transposed,
                              void* what, cudaStream_t stream) {
    const dim3 grid(out / 128u, in / 16u, 1);
    __half* w = static_cast<__half*>(what);
    switch (n) {
#define T3_CASE(NN) \
    case NN: dequant_kernel<NN, CB><<<grid, 256, 0, stream>>>(trellis, in, out, n, mask, transposed, w); break;
        T3_CASE(16) T3_CASE(32) T3_CASE(48) T3_CASE(64) T3_CASE(80) T3_CASE(96) T3_CASE(112) T3_CASE(128)
#undef T3_CASE
        default: dequant_kernel<0, CB><<<grid, 256, 0, stream>>>(trellis, in, out, n, mask, transposed, w); break;
    }
    return cudaGetLastError();
}

}  // namespace

cudaError_t launch_dequant(const uint8_t* trellis, uint32_t in, uint32_t out, uint32_t n, uint32_t mask, int codebook,
                           int transposed, void* what, cudaStream_t stream) {
    return codebook == kMcg ? launch_dequant_cb<kMcg>(trellis, in, out, n, mask, transposed, what, stream)
                            : launch_dequant_cb<kMul1>(trellis, in, out, n, mask, transposed, what, stream);
}

cudaError_t launch_unrot(void* w_t, const void* suh, const void* svh, uint32_t in, uint32_t out, int dt, cudaStream_t stream) {
    const int bytes = (int)(128u * kUnrotStride * sizeof(float));
    static std::atomic<unsigned long long> allowed{0};  // bit d: device d's kernel attribute is set
    int dev = 0;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return rc;
    if (dev >= 64 || !((allowed.load(std::memory_order_acquire) >> dev) & 1ull)) {
        rc = cudaFuncSetAttribute(reinterpret_cast<const void*>(unrot_tile_kernel), cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (rc != cudaSuccess) return rc;
        if (dev < 64) allowed.fetch_or(1ull << dev, std::memory_order_release);
    }
    unrot_tile_kernel<<<dim3(in / 128u, out / 128u, 1), 256, bytes, stream>>>(static_cast<uint16_t*>(w_t), static_cast<const __half*>(suh),
                                                                                static_cast<const __half*>(svh), in, dt);
    return cudaGetLastError();
}

cudaError_t launch_ep_plan(const uint32_t* inds, uint32_t rows, uint32_t topk, uint32_t experts, uint32_t world, uint32_t* order,
                           uint32_t* where, uint32_t* send_rows, void* meta, int* counts, cudaStream_t stream) {
    if (world < 1u || world > kEpWorldMax || experts % world != 0u) return cudaErrorInvalidValue;
    const EpPlanArgs a = {inds, rows, topk, experts / world, world, order, where, send_rows, static_cast<int2*>(meta), counts};
    ep_plan_kernel<<<1, 1024, 0, stream>>>(a);
    return cudaGetLastError();
}

cudaError_t launch_wait_runs_out(uint32_t* err, cudaStream_t stream) {
    wait_runs_out_kernel<<<1, 32, 0, stream>>>(err, kErrFullWait);
    return cudaGetLastError();
}

cudaError_t launch_codebook_table(int codebook, uint32_t mask, uint16_t* out, cudaStream_t stream) {
    if (codebook == kMcg) codebook_table_kernel<kMcg><<<128, 256, 0, stream>>>(mask, out);
    else codebook_table_kernel<kMul1><<<128, 256, 0, stream>>>(mask, out);
    return cudaGetLastError();
}

}  // namespace t3
