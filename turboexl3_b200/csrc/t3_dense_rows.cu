// The dense EXL3 linear at decode rows (up to 32 activation rows): t3_dense_<codebook>_n<rate>_r<row capacity>.
// Compiled once per codebook (-DT3_CB=0 MUL1, 1 MCG).
//
// What it computes is turboexl3's host reference (src/core/format.zig:334-389): xp = f16(H128(f16(x) suh)),
// z = f16(sum xp W_hat) with f32 accumulation, y = f16(H128(z) svh), in ONE launch where the reference takes three
// (prep_s -> dgemv -> dfinish, src/core/dense.zig:1229-1252, src/kernels/hip/dense/dense.hip:49-145).
//
// Shape of a launch. A thread-block cluster of S CTAs owns one 128-wide output block at a time (cluster c of the grid walks
// blocks c, c + clusters, ...). Rank r of the cluster streams the block's tile rows [T r / S, T (r + 1) / S) (T = in / 16,
// balanced to a tile row, not to a 128-input block) through a ring of shared-memory stages filled by bulk copies; sixteen
// consumer warps decode the tiles in registers straight into mma.sync B fragments and multiply them with the prepared
// rows. Partial sums leave a CTA as one-sided stores into the shared memory of the CTA that owns the row (row m belongs
// to rank m % S), counted on the owner's barrier; the owner adds the ranks in rank order, rounds, runs the output rotation
// and stores. Nobody waits for anybody but the owner for its data.
//
// Order on a stream of such launches (programmatic dependent launch). Everything that does not depend on the previous
// kernel runs ahead of griddepcontrol.wait: barrier set-up, the weight stream, and the DECODE of the first stages, whose
// B fragments are parked in shared memory (`dq`). After the wait come the input rotation, the tensor-core steps over the
// parked fragments, then the rest of the slab decoded as it streams. So a linear's integer work overlaps its
// predecessor's latency chain (x load, reduce, output rotation) instead of following it.
//
// Rows: up to kFusedRows rows are rotated inside the CTAs (every rank prepares its own K slice). Calls with more rows, or
// whose slice of prepared rows would not fit in shared memory, run t3_dense_prepare first (one Hadamard per row and block
// for the whole call instead of one per cluster) and the CTAs pull their slice of the prepared rows by bulk copy, in
// chunks of `chunk_blocks` 128-blocks through two buffers.
#include <mutex>
#include <unordered_map>

#include "t3_gemv.cuh"
#include "t3_internal.h"

#ifndef T3_CB
#error "compile with -DT3_CB=0 (MUL1) or -DT3_CB=1 (MCG)"
#endif

namespace t3 {
namespace {

constexpr int CB = T3_CB;

struct Carve {
    uint64_t *full, *empty, *recv_bar, *credit_bar, *xp_bar;
    __half* xp;
    float *local, *recv;
    uint8_t *dq, *ring;
};

__device__ __forceinline__ Carve carve(uint8_t* smem, const DenseSmem& L) {
    Carve c;
    c.full = reinterpret_cast<uint64_t*>(smem + L.bars);
    c.empty = c.full + kMaxStages;
    c.recv_bar = c.empty + kMaxStages;
    c.credit_bar = c.recv_bar + 2;
    c.xp_bar = c.credit_bar + 2;
    c.xp = reinterpret_cast<__half*>(smem + L.xp);
    c.local = reinterpret_cast<float*>(smem + L.local);
    c.recv = reinterpret_cast<float*>(smem + L.recv);
    c.dq = smem + L.dq;
    c.ring = smem + L.ring;
    return c;
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// rows [lo, hi) of the 8 tile rows of 128-input block b that belong to the slice [t0, t1)
__device__ __forceinline__ void stage_rows(uint32_t b, uint32_t t0, uint32_t t1, uint32_t& lo, uint32_t& hi) {
    const uint32_t r0 = 8u * b;
    lo = t0 > r0 ? t0 - r0 : 0u;
    hi = t1 < r0 + 8u ? t1 - r0 : 8u;
}

// What a consumer warp keeps for the whole kernel
template <int N>
struct WarpCtx {
    static constexpr int NP = N > 0 ? N : 16;
    LanePlan<NP> plan;
    uint32_t woff[raw_words(NP)];  // byte offsets of the lane's raw words inside a ring stage, tile row `kg`
    uint32_t n, mask, tcol, kg, lane;
    __device__ __forceinline__ uint32_t row_bytes() const { return N > 0 ? 16u * (uint32_t)N : 16u * n; }
};

// A whole ring stage (all 8 tile rows in the slice): the warp's four tiles — code words to registers, decode, then
// either the tensor-core steps (PARK = false) or the B fragments parked at `park` (16 bytes a lane a tile). Words, then
// decodes, then tensor-core steps, so four dependent chains overlap. With the rate a template constant every offset
// inside the stage is an immediate.
template <int N, int CBK, int RM, bool PARK>
__device__ __forceinline__ void stage_full(const uint8_t* st, const WarpCtx<N>& w, const __half* xs, uint32_t xstride,
                                           float (&acc)[RowCap<RM>::kMB][2][4], uint4* park) {
    constexpr int NP = WarpCtx<N>::NP;
    constexpr uint32_t kRaw = raw_words(NP);
    const uint32_t step = kKGroups * w.row_bytes();
    if (N > 0) {
        uint32_t raw[kBatch][kRaw];
#pragma unroll
        for (uint32_t i = 0; i < kBatch; ++i)
#pragma unroll
            for (uint32_t r = 0; r < kRaw; ++r) raw[i][r] = *reinterpret_cast<const uint32_t*>(st + w.woff[r] + i * step);
        uint32_t b[kBatch][4];
#pragma unroll
        for (uint32_t i = 0; i < kBatch; ++i) decode_raw<NP, CBK>(raw[i], w.plan, w.mask, b[i]);
#pragma unroll
        for (uint32_t i = 0; i < kBatch; ++i) {
            if (PARK) park[i * 32u] = make_uint4(b[i][0], b[i][1], b[i][2], b[i][3]);
            else mma_tile<RM>(acc, xs + i * kKGroups * 16u, xstride, b[i]);
        }
    } else {
#pragma unroll 1
        for (uint32_t i = 0; i < kBatch; ++i) {
            uint32_t b[4];
            decode_lane_any<CBK>(reinterpret_cast<const uint32_t*>(st + w.tcol * 2u * w.n + (i * kKGroups + w.kg) * w.row_bytes()),
                                 w.n, w.lane, w.mask, b);
            if (PARK) park[i * 32u] = make_uint4(b[0], b[1], b[2], b[3]);
            else mma_tile<RM>(acc, xs + i * kKGroups * 16u, xstride, b);
        }
    }
}

// A stage at the edge of the slice: only its tile rows [lo, hi) belong here. One tile at a time (the rare path: at most
// the first and the last stage of a slice); `park` non-null parks instead of multiplying.
template <int N, int CBK, int RM>
static __device__ __noinline__ void stage_edge(const uint8_t* st, uint32_t lo, uint32_t hi, const WarpCtx<N>& w, const __half* xs,
                                               uint32_t xstride, float (&acc)[RowCap<RM>::kMB][2][4], uint4* park) {
    constexpr int NP = WarpCtx<N>::NP;
    constexpr uint32_t kRaw = raw_words(NP);
#pragma unroll 1
    for (uint32_t i = 0; i < kBatch; ++i) {
        const uint32_t j = i * kKGroups + w.kg;
        if (j < lo || j >= hi) continue;
        uint32_t b[4];
        if (N > 0) {
            uint32_t raw[kRaw];
#pragma unroll
            for (uint32_t r = 0; r < kRaw; ++r) raw[r] = *reinterpret_cast<const uint32_t*>(st + w.woff[r] + i * kKGroups * w.row_bytes());
            decode_raw<NP, CBK>(raw, w.plan, w.mask, b);
        } else {
            decode_lane_any<CBK>(reinterpret_cast<const uint32_t*>(st + w.tcol * 2u * w.n + j * w.row_bytes()), w.n, w.lane, w.mask, b);
        }
        if (park) park[i * 32u] = make_uint4(b[0], b[1], b[2], b[3]);
        else mma_tile<RM>(acc, xs + i * kKGroups * 16u, xstride, b);
    }
}

// the tensor-core steps of a parked stage
template <int RM>
__device__ __forceinline__ void stage_parked(const uint4* pk, uint32_t lo, uint32_t hi, uint32_t kg, const __half* xs,
                                             uint32_t xstride, float (&acc)[RowCap<RM>::kMB][2][4]) {
#pragma unroll
    for (uint32_t i = 0; i < kBatch; ++i) {
        const uint32_t j = i * kKGroups + kg;
        if (j < lo || j >= hi) continue;
        const uint4 u = pk[i * 32u];
        const uint32_t b[4] = {u.x, u.y, u.z, u.w};
        mma_tile<RM>(acc, xs + i * kKGroups * 16u, xstride, b);
    }
}

// Sum over the cluster's ranks 0 .. count - 1, in that order, of owned row `slot`, for the lane's columns lane + 32 j
__device__ __forceinline__ void gather_ranks(const float* recv, uint32_t owned, uint32_t slot, uint32_t count, uint32_t lane,
                                             float (&v)[4]) {
    const float* rp = recv + slot * kPartialStride + lane;
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = rp[32 * j];
#pragma unroll 2
    for (uint32_t r = 1; r < count; ++r) {
        rp += owned * kPartialStride;
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] += rp[32 * j];
    }
}

// grid (S, clusters), cluster (S, 1, 1). PREP: the prepared rows come from global memory (a prepare launch ran first).
template <int N, int RM, bool PREP>
__global__ void __launch_bounds__(kGemvThreads, 2) dense_rows_kernel(const DenseArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = aligned_smem(smem_raw);
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank(), S = a.split;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;

    const uint32_t T = a.in / 16u, OB = a.out / 128u, clusters = gridDim.y;
    uint32_t t0, t1;
    slice_rows(T, S, rank, t0, t1);
    const uint32_t kb0 = t0 / 8u, nblk = (t1 + 7u) / 8u - kb0;            // the 128-input blocks the slice touches
    const uint32_t iters = (OB - blockIdx.y + clusters - 1u) / clusters;  // output blocks this cluster walks
    const uint32_t n = N > 0 ? (uint32_t)N : a.n;
    const uint32_t tile_bytes = 2u * n, row_bytes = 16u * n, out_tiles = a.out / 16u;
    const uint32_t stage_bytes = kStageRows * row_bytes;
    const uint32_t xstride = a.chunk_blocks * 128u + kXpPad;
    const DenseSmem L = dense_smem(RM, a.chunk_blocks, a.xp_bufs, a.recv_bufs, S, a.dq_stages, stage_bytes, a.ring.stages);
    const Carve c = carve(smem, L);
    const uint32_t owned = rows_owned(RM, S);
    const uint32_t n_owned = rank < a.rows ? (a.rows - rank + S - 1u) / S : 0u;  // live rows this CTA finishes
    const uint32_t owners = a.rows < S ? a.rows : S;                                // CTAs of the cluster that finish rows
    const uint32_t recv_bytes = n_owned * S * 512u;                                 // what one output block sends here
    const uint32_t recv_floats = S * owned * kPartialStride;                        // floats of one receive buffer
    // the slice's first and last stage may hold fewer than 8 of its tile rows
    const uint32_t lo_first = t0 - 8u * kb0, hi_last = t1 - 8u * (kb0 + nblk - 1u);

    unsigned long long* tr = nullptr;
    if (a.trace != nullptr && tid == 0) {
        const uint32_t cta = blockIdx.y * gridDim.x + blockIdx.x;
        if (cta < kTraceCtas) tr = a.trace + (size_t)cta * kTraceWords;
    }
    if (tr) {
        tr[0] = global_ns();
        uint32_t smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        tr[12] = smid;
    }

    if (tid < a.ring.stages) {
        mbar_init(&c.full[tid], 1u);
        mbar_init(&c.empty[tid], kConsumerWarps);
        mbar_init_fence();
    }
    if (tid == 32u) {
        for (uint32_t b = 0; b < 2u; ++b) {
            mbar_init(&c.recv_bar[b], 1u);
            mbar_init(&c.credit_bar[b], owners);
            mbar_init(&c.xp_bar[b], 1u);
        }
        mbar_init_fence();
        // armed for the first block that uses each buffer: complete when that block's partial sums have all landed
        if (n_owned) {
            mbar_arrive_expect_tx(&c.recv_bar[0], recv_bytes);
            if (iters > 1u) mbar_arrive_expect_tx(&c.recv_bar[1], recv_bytes);
        }
    }
    __syncthreads();
    cluster_arrive();  // "my barriers exist": peers wait for this before their first push

    const uint32_t full0 = smem_addr(c.full), empty0 = smem_addr(c.empty);

    if (warp == kConsumerWarps) {
        // ---- producer: the weights do not depend on the stream's previous kernel
        pdl_trigger();
        uint32_t slot = 0, lap = 0;
        const size_t src_stride = (size_t)out_tiles * tile_bytes;
#pragma unroll 1
        for (uint32_t it = 0; it < iters; ++it) {
            const uint32_t ob = blockIdx.y + it * clusters;
            const uint8_t* src = a.trellis + ((size_t)(8u * kb0) * out_tiles + ob * 8u) * tile_bytes + lane * src_stride;
#pragma unroll 1
            for (uint32_t s = 0; s < nblk; ++s, src += 8u * src_stride) {
                const uint32_t lo = s == 0u ? lo_first : 0u, hi = s + 1u == nblk ? hi_last : 8u;
                if (lap > 0 && !mbar_wait_addr(empty0 + slot * 8u, (lap - 1u) & 1u)) report(a.err, kErrEmptyWait);
                if (lane == 0) mbar_arrive_expect_tx(&c.full[slot], (hi - lo) * row_bytes);
                __syncwarp();
                if (lane >= lo && lane < hi)
                    bulk_copy_g2s(c.ring + slot * stage_bytes + lane * row_bytes, src, row_bytes, &c.full[slot]);
                if (++slot == a.ring.stages) slot = 0, ++lap;
            }
        }
        cluster_wait();
        return;
    }

    // ---- consumers
    pdl_trigger();
    WarpCtx<N> w;
    w.n = n, w.mask = a.mask, w.tcol = warp & (kTileWarps - 1u), w.kg = warp / kTileWarps, w.lane = lane;
    if (N > 0) w.plan.init(lane);
#pragma unroll
    for (uint32_t i = 0; i < raw_words(WarpCtx<N>::NP); ++i) w.woff[i] = w.tcol * tile_bytes + w.kg * row_bytes + w.plan.idx[i] * 4u;
    const uint32_t kg = w.kg, tcol = w.tcol;
    const bool lane0 = lane == 0;
    float sv0[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // the first output block's scales of the row this warp finishes
    if (warp < n_owned) load_scales(static_cast<const __half*>(a.svh) + blockIdx.y * 128u, lane, sv0);
    if (!PREP && warp == 0) prefetch_l2(static_cast<const __half*>(a.suh) + kb0 * 128u, nblk * 256u, lane);

    uint32_t slot = 0, par = 0;  // the ring stage this warp takes next and its phase parity
    float acc[RowCap<RM>::kMB][2][4];
    // parked decodes: the first `pre` stages of the first output block, ahead of the dependency wait
    const uint32_t pre = a.dq_stages < nblk ? a.dq_stages : nblk;
    uint4* const park = reinterpret_cast<uint4*>(c.dq) + (size_t)warp * a.dq_stages * kBatch * 32u + lane;
#pragma unroll 1
    for (uint32_t s = 0; s < pre; ++s) {
        const uint32_t lo = s == 0u ? lo_first : 0u, hi = s + 1u == nblk ? hi_last : 8u;
        if (!mbar_wait_addr(full0 + slot * 8u, par)) report(a.err, kErrFullWait);
        const uint8_t* st = c.ring + slot * stage_bytes;
        if (lo == 0u && hi == 8u) stage_full<N, CB, RM, true>(st, w, nullptr, 0u, acc, park + s * kBatch * 32u);
        else stage_edge<N, CB, RM>(st, lo, hi, w, nullptr, 0u, acc, park + s * kBatch * 32u);
        __syncwarp();
        if (lane0) mbar_arrive_addr(empty0 + slot * 8u);
        if (++slot == a.ring.stages) slot = 0, par ^= 1u;
    }
    if (tr) tr[1] = global_ns();
    pdl_wait();  // x (or the prepared rows) may be the previous kernel's output; y may be its input
    if (tr) tr[2] = global_ns();

    const uint32_t xp_buf_halfs = RM * xstride;
    uint32_t gc = 0;  // chunks of prepared rows pulled so far (PREP)
    // one chunk of prepared rows [rows][blocks of the chunk] from global memory into buffer `buf`: a bulk copy a row
    auto pull_chunk = [&](uint32_t chunk, uint32_t buf) {
        const uint32_t b0 = chunk * a.chunk_blocks, nb = min(a.chunk_blocks, nblk - b0);
        mbar_arrive_expect_tx(&c.xp_bar[buf], a.rows * nb * 256u);
#pragma unroll 1
        for (uint32_t r = 0; r < a.rows; ++r)
            bulk_copy_g2s(c.xp + buf * xp_buf_halfs + r * xstride, a.xp_g + (size_t)r * a.in + (kb0 + b0) * 128u, nb * 256u,
                          &c.xp_bar[buf]);
    };
    const uint32_t nchunks = PREP ? (nblk + a.chunk_blocks - 1u) / a.chunk_blocks : 1u;
    if (PREP) {
        if (tid == 0) pull_chunk(0, 0);
    } else {
        // the input rotation of this rank's slice, inside the CTA (one chunk by construction)
#pragma unroll 1
        for (uint32_t task = warp; task < a.rows * nblk; task += kConsumerWarps) {
            const uint32_t row = task / nblk, b = task - row * nblk;
            const uint32_t k0 = (kb0 + b) * 128u;
            prepare_block(a.x, a.x_dt, (size_t)row * a.in + k0, static_cast<const __half*>(a.suh) + k0,
                          c.xp + row * xstride + b * 128u, lane);
        }
        named_sync(1, kConsumerThreads);
    }
    if (tr) tr[3] = global_ns();

#pragma unroll 1
    for (uint32_t it = 0; it < iters; ++it) {
        const uint32_t ob = blockIdx.y + it * clusters;
#pragma unroll
        for (int mb = 0; mb < RowCap<RM>::kMB; ++mb)
#pragma unroll
            for (int nt = 0; nt < 2; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[mb][nt][e] = 0.0f;
        const uint32_t parked = it == 0u ? pre : 0u;
#pragma unroll 1
        for (uint32_t ch = 0; ch < nchunks; ++ch) {
            const uint32_t s0 = PREP ? ch * a.chunk_blocks : 0u, s1 = PREP ? min(nblk, s0 + a.chunk_blocks) : nblk;
            const __half* xpb = c.xp;
            if (PREP) {
                if (nchunks > 1u) {
                    // everyone is done with the chunk before this one, so the other buffer can take the chunk after it
                    named_sync(1, kConsumerThreads);
                    const uint32_t nxt = gc + 1u;
                    if (tid == 0 && nxt < iters * nchunks) pull_chunk(nxt % nchunks, nxt & 1u);
                    if (!mbar_wait(&c.xp_bar[gc & 1u], (gc >> 1) & 1u)) report(a.err, kErrFullWait);
                    xpb = c.xp + (gc & 1u) * xp_buf_halfs;
                    ++gc;
                } else if (it == 0) {
                    if (!mbar_wait(&c.xp_bar[0], 0u)) report(a.err, kErrFullWait);
                }
            }
            const __half* xs = xpb + (lane >> 2) * xstride + 4u * (lane & 3u) + kg * 16u;
            uint32_t s = s0;
            // the parked stages of this chunk: tensor-core steps only
#pragma unroll 1
            for (; s < s1 && s < parked; ++s, xs += 128u)
                stage_parked<RM>(park + s * kBatch * 32u, s == 0u ? lo_first : 0u, s + 1u == nblk ? hi_last : 8u, kg, xs, xstride, acc);
            // the rest streams through the ring
#pragma unroll 1
            for (; s < s1; ++s, xs += 128u) {
                if (!mbar_wait_addr(full0 + slot * 8u, par)) report(a.err, kErrFullWait);
                const uint8_t* st = c.ring + slot * stage_bytes;
                if ((s != 0u || lo_first == 0u) && (s + 1u != nblk || hi_last == 8u))
                    stage_full<N, CB, RM, false>(st, w, xs, xstride, acc, nullptr);
                else
                    stage_edge<N, CB, RM>(st, s == 0u ? lo_first : 0u, s + 1u == nblk ? hi_last : 8u, w, xs, xstride, acc, nullptr);
                __syncwarp();
                if (lane0) mbar_arrive_addr(empty0 + slot * 8u);
                if (++slot == a.ring.stages) slot = 0, par ^= 1u;
            }
        }
        if (tr && it == 0) tr[4] = global_ns();

        // the two K groups meet in this CTA's shared memory, then every live row goes to its owner
        if (kg == 1) store_local<RM>(c.local, acc, tcol, lane);
        named_sync(1, kConsumerThreads);
        const uint32_t buf = it & 1u, use = it >> 1;
        if (it == 0) cluster_wait();  // every peer's barriers exist
        if (use > 0 && !mbar_wait_cluster(&c.credit_bar[buf], (use - 1u) & 1u)) report(a.err, kErrEmptyWait);
        if (kg == 0) {
            const uint32_t g = lane >> 2, q = lane & 3u;
#pragma unroll
            for (int mb = 0; mb < RowCap<RM>::kMB; ++mb)
#pragma unroll
                for (int h = 0; h < (RowCap<RM>::kHalf ? 1 : 2); ++h) {
                    const uint32_t m = mb * 16 + h * 8 + g;
                    if (m >= a.rows) continue;
                    const uint32_t owner = m % S;
                    const float* dst = c.recv + buf * recv_floats + (rank * owned + m / S) * kPartialStride + tcol * 16u + 2u * q;
                    const float* src = c.local + m * kPartialStride + tcol * 16u + 2u * q;
                    const uint32_t bar = peer_addr(&c.recv_bar[buf], owner), to = peer_addr(dst, owner);
#pragma unroll
                    for (int nt = 0; nt < 2; ++nt) {
                        const float2 o = *reinterpret_cast<const float2*>(src + nt * 8);
                        push_f32x2(to + nt * 32u, acc[mb][nt][2 * h] + o.x, acc[mb][nt][2 * h + 1] + o.y, bar);
                    }
                }
        }
        if (tr && it == 0) tr[5] = global_ns();
        const bool last = it + 1u == iters;
        if (n_owned == 0u) {
            if (last) break;
            named_sync(1, kConsumerThreads);  // the K groups' tile is free for the next block
            continue;
        }
        // ---- owner: its rows' partial sums from every rank, in rank order; the output rotation; the store
        if (!mbar_wait_cluster(&c.recv_bar[buf], use & 1u)) report(a.err, kErrFullWait);
        if (tr && it == 0) tr[6] = global_ns();
#pragma unroll 1
        for (uint32_t i = warp; i < n_owned; i += kConsumerWarps) {
            const uint32_t row = i * S + rank;
            float v[4], sv[4];
            if (it == 0u && i == warp) {
#pragma unroll
                for (int j = 0; j < 4; ++j) sv[j] = sv0[j];
            } else {
                load_scales(static_cast<const __half*>(a.svh) + ob * 128u, lane, sv);
            }
            gather_ranks(c.recv + buf * recv_floats, owned, i, S, lane, v);
            finish_block(v, sv, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) store_act(a.y, a.x_dt, (size_t)row * a.out + ob * 128u + lane + 32u * j, v[j]);
        }
        if (last) break;
        named_sync(1, kConsumerThreads);  // every warp has read its rows: the buffer may be refilled
        if (tid == 0 && it + 2u < iters) {
            mbar_arrive_expect_tx(&c.recv_bar[buf], recv_bytes);
#pragma unroll 1
            for (uint32_t r = 0; r < S; ++r) peer_arrive(peer_addr(&c.credit_bar[buf], r));
        }
    }
    if (tr) tr[7] = global_ns();
}

// ---- the prepared rows of calls with many rows ---------------------------------------------------------------------

// grid (in / 128, rows), one warp a (row, block): format.prepareInput (src/core/format.zig:334-345) with the arithmetic of
// the in-CTA rotation, so a row's prepared values do not depend on which path its call took
__global__ void __launch_bounds__(32) dense_prepare_kernel(const void* x, int x_dt, const __half* suh, uint32_t in, __half* xp) {
    pdl_trigger();
    pdl_wait();
    const uint32_t b = blockIdx.x, row = blockIdx.y;
    prepare_block(x, x_dt, (size_t)row * in + b * 128u, suh + b * 128u, xp + (size_t)row * in + b * 128u, threadIdx.x);
}

// ---- launch plumbing -----------------------------------------------------------------------------------------------

using DenseFn = void (*)(const DenseArgs);

// rows up to kFusedRows rotate inside the CTAs (PREP = false, row capacity 8); everything else pulls prepared rows
#define T3_PICK_RM(NN, rm, prep)                                                                 \
    ((rm) == 8 ? ((prep) ? dense_rows_kernel<NN, 8, true> : dense_rows_kernel<NN, 8, false>)      \
               : ((rm) == 16 ? dense_rows_kernel<NN, 16, true> : dense_rows_kernel<NN, 32, true>))

DenseFn pick_kernel(uint32_t n, uint32_t rm, bool prep) {
    switch (n) {
        case 16: return T3_PICK_RM(16, rm, prep);
        case 32: return T3_PICK_RM(32, rm, prep);
        case 48: return T3_PICK_RM(48, rm, prep);
        case 64: return T3_PICK_RM(64, rm, prep);
        case 80: return T3_PICK_RM(80, rm, prep);
        case 96: return T3_PICK_RM(96, rm, prep);
        case 112: return T3_PICK_RM(112, rm, prep);
        case 128: return T3_PICK_RM(128, rm, prep);
        default: return T3_PICK_RM(0, rm, prep);
    }
}

// per (device, kernel): the dynamic shared-memory limit raised, and how many clusters of each size fit the device at once
struct FnInfo {
    bool ready = false;
    std::unordered_map<uint64_t, int> max_clusters;  // (cluster size << 32 | shared bytes) -> clusters resident at once
};
std::mutex g_fn_mu;
std::unordered_map<uint64_t, FnInfo> g_fn;  // device << 48 ^ function address

cudaError_t fn_info(DenseFn fn, FnInfo*& out) {
    int dev = 0;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return rc;
    FnInfo& fi = g_fn[((uint64_t)dev << 48) ^ reinterpret_cast<uint64_t>(fn)];
    if (!fi.ready) {
        rc = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvSmemLimit);
        if (rc == cudaSuccess) rc = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (rc != cudaSuccess) return rc;
        fi.ready = true;
    }
    out = &fi;
    return cudaSuccess;
}

void fill_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute (&attr)[2], uint32_t split, uint32_t clusters, uint32_t smem_bytes,
                 bool overlap, cudaStream_t stream) {
    cfg = {};
    cfg.gridDim = dim3(split, clusters, 1);
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = split;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 2 : 1;
}

}  // namespace

#define T3_CAT2(a, b) a##b
#define T3_CAT(a, b) T3_CAT2(a, b)

// clusters of `split` CTAs with `smem_bytes` of dynamic shared memory each that the current device holds at once
int T3_CAT(dense_rows_max_clusters_cb, T3_CB)(uint32_t n, uint32_t rm, bool prep, uint32_t split, uint32_t smem_bytes) {
    DenseFn fn = pick_kernel(n, rm, prep);
    std::lock_guard<std::mutex> lock(g_fn_mu);
    FnInfo* fi = nullptr;
    if (fn_info(fn, fi) != cudaSuccess) return 0;
    const uint64_t key = ((uint64_t)split << 32) | smem_bytes;
    auto hit = fi->max_clusters.find(key);
    if (hit != fi->max_clusters.end()) return hit->second;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    fill_config(cfg, attr, split, 1, smem_bytes, false, nullptr);
    int count = 0;
    if (cudaOccupancyMaxActiveClusters(&count, fn, &cfg) != cudaSuccess) {
        cudaGetLastError();
        count = 0;
    }
    fi->max_clusters[key] = count;
    return count;
}

cudaError_t T3_CAT(launch_dense_rows_cb, T3_CB)(const DenseArgs& a, uint32_t rm, uint32_t clusters, uint32_t smem_bytes,
                                                cudaStream_t stream) {
    if (smem_bytes > kGemvSmemLimit) return cudaErrorInvalidValue;
    DenseFn fn = pick_kernel(a.n, rm, a.xp_g != nullptr);
    {
        std::lock_guard<std::mutex> lock(g_fn_mu);
        FnInfo* fi = nullptr;
        cudaError_t rc = fn_info(fn, fi);
        if (rc != cudaSuccess) return rc;
    }
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[2];
    fill_config(cfg, attr, a.split, clusters, smem_bytes, a.overlap != 0, stream);
    return cudaLaunchKernelEx(&cfg, fn, a);
}

#if T3_CB == 0
cudaError_t launch_dense_prepare(const void* x, int x_dt, const void* suh, uint32_t rows, uint32_t in, void* xp, bool overlap,
                                 cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(in / 128u, rows, 1);
    cfg.blockDim = dim3(32, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, dense_prepare_kernel, x, x_dt, static_cast<const __half*>(suh), in, static_cast<__half*>(xp));
}
#endif

}  // namespace t3
