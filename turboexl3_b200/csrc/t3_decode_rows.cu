// Decode-row kernels (up to 32 activation rows): the fused dense linear, the routed experts' gate|up and down launches
// and the score-weighted merge. Compiled once per codebook (-DT3_CB=0 MUL1, 1 MCG) so the two halves build in parallel.
//
// Dense linear = one launch: prepare (input rotation) in shared memory, split-K GEMV over a thread-block cluster,
// output rotation by the cluster's leader. The reference takes three launches for the same values
// (prep_s -> dgemv -> dfinish, src/core/dense.zig:1229-1252, src/kernels/hip/dense/dense.hip).
//
// Routed chain = three launches: gate|up (+ SwiGLU + the down projection's prepare), down (+ its finish), merge.
// The reference's served chain is four or five (src/core/decode.zig:483-517). Row-slots that share an expert are found
// inside the kernels (each CTA scans the call's <= 1024 expert ids), so one decode of an expert's tiles feeds every row
// that routed to it, as the reference's grouped members do (src/core/kernels/decode/gemv_core.metal:4-21).
#include <mutex>
#include <unordered_set>

#include "t3_gemv.cuh"
#include "t3_internal.h"

#ifndef T3_CB
#error "compile with -DT3_CB=0 (MUL1), 1 (MCG), or 2..4 (the dense linear's timing probes: see t3_lane.cuh)"
#endif
#define T3_SERVED (T3_CB < 2)

namespace t3 {
namespace {

constexpr int CB = T3_CB;
constexpr uint32_t kMaxSlots = 1024;  // 32 rows x 32 top-k

// ---------------------------------------------------------------------------------------------- shared pieces

struct CtaSmem {
    uint64_t *full, *empty, *xp_full;
    __half* xp;
    float *local, *recv;
    uint8_t* ring;
};

__device__ __forceinline__ CtaSmem carve(uint8_t* smem, const GemvSmem& L) {
    CtaSmem c;
    c.full = reinterpret_cast<uint64_t*>(smem + L.bars);
    c.empty = c.full + kMaxStages;
    c.xp_full = c.full + 2u * kMaxStages;
    c.xp = reinterpret_cast<__half*>(smem + L.xp);
    c.local = reinterpret_cast<float*>(smem + L.local);
    c.recv = reinterpret_cast<float*>(smem + L.recv);
    c.ring = smem + L.ring;
    return c;
}

__device__ __forceinline__ void init_barriers(const CtaSmem& c, uint32_t stages) {
    if (threadIdx.x < stages) {  // one thread a stage
        mbar_init(&c.full[threadIdx.x], 1u);
        mbar_init(&c.empty[threadIdx.x], kConsumerWarps);
        mbar_init_fence();
    }
    if (threadIdx.x == kMaxStages) {
        mbar_init(c.xp_full, 1u);
        mbar_init_fence();
    }
}

__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory"); }

// The consumer side of one pass once xp is ready: GEMV over the slab, the two K groups joined, the partial pushed to the
// rows' owners. `count` live rows.
template <int N, int RM, int HB = 2>
__device__ __forceinline__ void gemv_and_push(cg::cluster_group& cluster, const CtaSmem& c, uint32_t nrows, uint32_t n,
                                              uint32_t mask, Ring rc, uint32_t xstride, uint32_t xrows, RingPos& pos, uint32_t count,
                                              uint32_t rank, uint32_t csize, uint32_t warp, uint32_t lane, uint32_t* err) {
    const uint32_t tcol = warp & (kTileWarps - 1u), kg = warp / kTileWarps;
    float acc[RowCap<RM>::kMB][2][4] = {};
    consume_slab<N, CB, RM, HB>(c.ring, c.full, c.empty, nrows, n, mask, rc, c.xp, xstride, xrows, pos, tcol, kg, lane, acc, err);
    if (kg == 1) store_local<RM>(c.local, acc, tcol, lane);
    named_sync(1, kConsumerThreads);
    if (kg == 0) push_partial<RM>(cluster, c.recv, c.local, acc, count, rank, csize, tcol, lane);
}

// ---------------------------------------------------------------------------------------------- dense linear

// grid (split, out / 128), cluster (split, 1, 1) — or no cluster when the partial sums meet in global memory (a.part)
template <int N, int RM>
__device__ __forceinline__ void dense_gemv_body(const DenseArgs& a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = aligned_smem(smem_raw);
    __shared__ uint32_t s_last;
    // up to 8 rows the accumulators are four registers, so four tiles' words and fragments fit beside them: more
    // independent chains a warp where few warps share a scheduler (the small linears)
    constexpr int kDenseBatch = RowCap<RM>::kHalf ? 4 : 2;
    cg::cluster_group cluster = cg::this_cluster();
    const bool global = a.part != nullptr;
    const uint32_t rank = global ? blockIdx.x : cluster.block_rank(), csize = global ? 1u : a.split, blk = blockIdx.y;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    uint32_t b0, b1;
    slice_blocks(a.in / 128u, a.split, rank, b0, b1);
    const uint32_t nblk = b1 - b0, nrows = nblk * 8u;
    const uint32_t tile_bytes = 2u * a.n, row_bytes = 16u * a.n, out_tiles = a.out / 16u;
    const Ring rc{a.ring.stage_rows, a.ring.stages};
    const CtaSmem c = carve(smem, gemv_smem(RM, a.rows, a.slice_max, csize, rc.stage_rows * row_bytes, rc.stages));
    const uint32_t xstride = a.slice_max + kXpPad;

    const bool traced = a.trace != nullptr && blockIdx.x == 0 && blockIdx.y == 0;
    if (traced && tid == 0) a.trace[0] = clock64();
    init_barriers(c, rc.stages);
    __syncthreads();
    if (traced && tid == 0) a.trace[1] = clock64();

    RingPos pos;
    float sv[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (warp == kConsumerWarps) {
        // the weights do not depend on the stream's previous kernel: start them, then let the next kernel do the same
        const uint8_t* src = a.trellis + ((size_t)(b0 * 8u) * out_tiles + blk * 8u) * tile_bytes;
        const size_t stride = (size_t)out_tiles * tile_bytes;
        if (a.xp_g == nullptr) {
            produce_slab(c.ring, c.full, c.empty, src, stride, nrows, row_bytes, rc, pos, lane, a.err);
            pdl_trigger();
        } else {
            // as many stages as the ring holds without waiting for a consumer (who waits for the prepared rows), then the
            // prepared rows of this CTA's K slice (the previous kernel's output), then the rest of the slab
            const uint32_t head = min(nrows, rc.stages * kStageRows);
            produce_slab(c.ring, c.full, c.empty, src, stride, head, row_bytes, rc, pos, lane, a.err);
            pdl_trigger();
            pdl_wait();
            const uint32_t slice_bytes = nblk * 256u;
            if (lane == 0) mbar_arrive_expect_tx(c.xp_full, a.rows * slice_bytes);
            __syncwarp();
            if (lane < a.rows)
                bulk_copy_g2s(c.xp + lane * xstride, static_cast<const __half*>(a.xp_g) + (size_t)lane * a.in + b0 * 128u, slice_bytes,
                              c.xp_full);
            produce_slab(c.ring, c.full, c.empty, src + (size_t)head * stride, stride, nrows - head, row_bytes, rc, pos, lane, a.err);
        }
    } else {
        pdl_trigger();
        load_scales(static_cast<const __half*>(a.svh) + blk * 128u, lane, sv);  // weights-side: ahead of the wait
        if (a.xp_g == nullptr) {
            if (warp == 0) prefetch_l2(static_cast<const __half*>(a.suh) + b0 * 128u, nblk * 256u, lane);
            pdl_wait();  // x may be the previous kernel's output
            for (uint32_t task = warp; task < a.rows * nblk; task += kConsumerWarps) {
                const uint32_t row = task / nblk, b = task - row * nblk;
                const uint32_t k0 = (b0 + b) * 128u;
                prepare_block(a.x, a.x_dt, (size_t)row * a.in + k0, static_cast<const __half*>(a.suh) + k0,
                              c.xp + row * xstride + b * 128u, lane);
            }
        } else {
            pdl_wait();
            mbar_wait_report(smem_addr(c.xp_full), 0u, a.err, kErrFullWait);
        }
        named_sync(1, kConsumerThreads);
        if (traced && tid == 0) {
            a.trace[2] = clock64();
            mbar_wait(&c.full[0], 0u);
            a.trace[3] = clock64();
        }
        if (!global) {
            gemv_and_push<N, RM, kDenseBatch>(cluster, c, nrows, a.n, a.mask, rc, xstride, a.rows, pos, a.rows, rank, csize, warp, lane, a.err);
        } else {
            // the slice's sums to global memory; the block's last arriver adds the slices in slice order and finishes
            const uint32_t tcol = warp & (kTileWarps - 1u), kg = warp / kTileWarps;
            float acc[RowCap<RM>::kMB][2][4] = {};
            consume_slab<N, CB, RM, kDenseBatch>(c.ring, c.full, c.empty, nrows, a.n, a.mask, rc, c.xp, xstride, a.rows, pos, tcol, kg, lane, acc, a.err);
            if (kg == 1) store_local<RM>(c.local, acc, tcol, lane);
            named_sync(1, kConsumerThreads);
            if (kg == 0) {
                float* mine = a.part + ((size_t)blk * a.split + rank) * a.rows * 128u;
#pragma unroll
                for (int mb = 0; mb < RowCap<RM>::kMB; ++mb)
#pragma unroll
                    for (int nt = 0; nt < Frags<RM>::kNt; ++nt)
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const uint32_t m = fragment_row<RM>(lane, mb, nt, e);
                            if (m >= a.rows) continue;
                            const uint32_t col = tcol * 16u + fragment_col<RM>(lane, e);
                            __stcg(mine + m * 128u + col, acc[mb][nt][e] + c.local[m * kPartialStride + col]);
                        }
            }
            __threadfence();
            named_sync(1, kConsumerThreads);
            if (tid == 0) s_last = atomicAdd(&a.counters[blk], 1u) == a.split - 1u;
            named_sync(1, kConsumerThreads);
            if (!s_last) return;
            __threadfence();
            for (uint32_t row = warp; row < a.rows; row += kConsumerWarps) {
                float v[4];
                for (uint32_t r = 0; r < a.split; ++r) {
                    const float* src = a.part + (((size_t)blk * a.split + r) * a.rows + row) * 128u + lane;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const float t = __ldcg(src + 32 * j);
                        v[j] = r == 0u ? t : v[j] + t;
                    }
                }
                finish_block(v, sv, lane);
#pragma unroll
                for (int j = 0; j < 4; ++j) store_act(a.y, a.x_dt, (size_t)row * a.out + blk * 128u + lane + 32u * j, v[j]);
            }
            if (tid == 0) a.counters[blk] = 0u;  // as the next call on this workspace expects it
            return;
        }
        if (traced && tid == 0) a.trace[4] = clock64();
    }
    if (global) return;  // the copy warp: its copies have landed (the consumers waited for each)
    cluster_arrive();
    if (rank >= a.rows) return;  // owns no row: nothing reads this CTA's shared memory after its arrival
    cluster_wait();
    if (traced && tid == 0) a.trace[5] = clock64();
    if (warp < kConsumerWarps) {
        const uint32_t owned = rows_owned(RM, csize);
        for (uint32_t i = warp; i * csize + rank < a.rows; i += kConsumerWarps) {
            const uint32_t row = i * csize + rank;
            float v[4];
            gather_owned(c.recv, owned, i, 0, 1, csize, lane, v);
            finish_block(v, sv, lane);
#pragma unroll
            for (int j = 0; j < 4; ++j) store_act(a.y, a.x_dt, (size_t)row * a.out + blk * 128u + lane + 32u * j, v[j]);
        }
    }
    if (traced && tid == 0) a.trace[6] = clock64();
}

#if T3_SERVED
// ---------------------------------------------------------------------------------------------- routed experts

struct Members {
    uint32_t expert, count;
    bool skip;
};

// A row-slot's id as the kernels use it: an expert of the bank, clamped into it; in a banked call the packed id with its
// bank clamped to 0..2 and its slot into that bank, or kSkipId as it is.
__device__ __forceinline__ uint32_t canon_id(const MoeArgs& a, uint32_t id) {
    if (!a.banked) return min(id, a.experts - 1u);
    if (id == kSkipId) return id;
    const uint32_t bk = min(id >> 24, 2u);
    const uint32_t cap = bk == 0u ? a.experts : (bk == 1u ? a.ext[0].experts : a.ext[1].experts);
    return (bk << 24) | min(id & 0xFFFFFFu, cap - 1u);
}

// The arrays of the bank a canonical id names (bank 0: the call's own)
#define T3_BANK_FIELD(a, id, f) (!(a).banked || ((id) >> 24) == 0u ? (a).f : (((id) >> 24) == 1u ? (a).ext[0].f : (a).ext[1].f))

// Row-slot j's expert and every row-slot of the call on that expert, ascending, into `members`; skip = an earlier
// row-slot already owns this expert (its CTAs do the work), or the row-slot runs no expert. All threads of the CTA must
// call this.
__device__ __forceinline__ Members find_members(const MoeArgs& a, uint32_t j, uint32_t* s_inds, uint16_t* members,
                                                uint32_t* s_count) {
    const uint32_t tid = threadIdx.x, slots = a.rows * a.topk;
    const uint32_t* inds = static_cast<const uint32_t*>(a.inds);
    for (uint32_t s = tid; s < slots; s += blockDim.x) s_inds[s] = canon_id(a, inds[s]);
    __syncthreads();
    Members m;
    m.expert = s_inds[j];
    int earlier = a.banked && m.expert == kSkipId;
    for (uint32_t s = tid; s < j; s += blockDim.x) earlier |= (s_inds[s] == m.expert);
    m.skip = __syncthreads_or(earlier) != 0;
    m.count = 0;
    if (m.skip) return m;
    if (tid < 32u) {
        uint32_t count = 0;
        for (uint32_t base = j & ~31u; base < slots; base += 32u) {
            const uint32_t s = base + tid;
            const bool hit = s >= j && s < slots && s_inds[s] == m.expert;
            const uint32_t votes = __ballot_sync(0xFFFFFFFFu, hit);
            if (hit) members[count + __popc(votes & ((1u << tid) - 1u))] = (uint16_t)s;
            count += __popc(votes);
        }
        if (tid == 0) *s_count = count;
    }
    __syncthreads();
    m.count = *s_count;
    return m;
}

// SwiGLU of one element in f32 with the optional clamp (turboexl3 src/core/ref.zig:124-140)
__device__ __forceinline__ float swiglu(float g, float u, float limit, int clamp_at) {
    if (limit > 0.0f) {
        u = u > limit ? limit : (u < -limit ? -limit : u);
        if (clamp_at == 0) g = g > limit ? limit : g;
    }
    float s = g / (1.0f + expf(-g));
    if (limit > 0.0f && clamp_at != 0) s = s > limit ? limit : s;
    return s * u;
}

// grid (2 SG, inter/128, row-slots), cluster (2 SG, 1, 1): cluster rank r streams projection r & 1 (0 gate, 1 up), K
// slice r >> 1. A row's owner finishes both projections, applies SwiGLU and prepares the 128 values as inputs of the
// down projection (ref.moeRow's middle, ref.zig:98-105; the reference kernels' "mid": src/kernels/hip/routed.hpp:64-112).
template <int N, int RM>
__device__ __forceinline__ void moe_gate_up_body(const MoeArgs& a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = aligned_smem(smem_raw);
    __shared__ uint32_t s_inds[kMaxSlots];
    __shared__ uint16_t s_members[kMaxSlots];
    __shared__ uint32_t s_count;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank(), csize = 2u * a.split_gu, ib = blockIdx.y, j = blockIdx.z;
    const uint32_t proj = rank & 1u, kpart = rank >> 1;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t H = a.hidden, I = a.inter;
    pdl_wait();     // the routing (and x) may be the previous kernel's output
    pdl_trigger();  // after the wait: the down launch reads the routing ahead of its own wait
    const Members mem = find_members(a, j, s_inds, s_members, &s_count);
    if (mem.skip) return;
    const uint32_t id = mem.expert, e = a.banked ? id & 0xFFFFFFu : id;

    uint32_t b0, b1;
    slice_blocks(H / 128u, a.split_gu, kpart, b0, b1);
    const uint32_t nblk = b1 - b0, nrows = nblk * 8u;
    const uint32_t tile_bytes = 2u * a.n, row_bytes = 16u * a.n, out_tiles = I / 16u;
    const Ring rc{a.ring_gu.stage_rows, a.ring_gu.stages};
    const CtaSmem c = carve(smem, gemv_smem(RM, RM, a.slice_max_gu, csize, rc.stage_rows * row_bytes, rc.stages));
    const uint32_t xstride = a.slice_max_gu + kXpPad;
    init_barriers(c, rc.stages);
    __syncthreads();

    const size_t expert_bytes = (size_t)(H / 16u) * out_tiles * tile_bytes;
    const uint8_t* wsrc = (proj ? T3_BANK_FIELD(a, id, up_t) : T3_BANK_FIELD(a, id, gate_t)) + e * expert_bytes +
                          ((size_t)(b0 * 8u) * out_tiles + ib * 8u) * tile_bytes;
    const __half* suh = static_cast<const __half*>(proj ? T3_BANK_FIELD(a, id, up_suh) : T3_BANK_FIELD(a, id, gate_suh)) + (size_t)e * H;
    if (warp == 0) {  // the expert's scale vectors are first used behind the weight stream and the cluster barrier
        const size_t eo = (size_t)e * I + ib * 128u;
        prefetch_l2(suh + b0 * 128u, nblk * 256u, lane);
        prefetch_l2(static_cast<const __half*>(T3_BANK_FIELD(a, id, gate_svh)) + eo, 256u, lane);
        prefetch_l2(static_cast<const __half*>(T3_BANK_FIELD(a, id, up_svh)) + eo, 256u, lane);
        prefetch_l2(static_cast<const __half*>(T3_BANK_FIELD(a, id, down_suh)) + eo, 256u, lane);
    }
    const uint32_t owned = rows_owned(RM, csize);
    RingPos pos;
    for (uint32_t m0 = 0; m0 < mem.count; m0 += RM) {
        const uint32_t mcount = min((uint32_t)RM, mem.count - m0);
        if (warp == kConsumerWarps) {
            produce_slab(c.ring, c.full, c.empty, wsrc, (size_t)out_tiles * tile_bytes, nrows, row_bytes, rc, pos, lane, a.err);
        } else {
            for (uint32_t i = mcount * xstride + tid; i < RM * xstride; i += kConsumerThreads) c.xp[i] = __float2half_rn(0.0f);
            for (uint32_t task = warp; task < mcount * nblk; task += kConsumerWarps) {
                const uint32_t m = task / nblk, b = task - m * nblk;
                const uint32_t row = s_members[m0 + m] / a.topk, k0 = (b0 + b) * 128u;
                prepare_block(a.x, a.x_dt, (size_t)row * H + k0, suh + k0, c.xp + m * xstride + b * 128u, lane);
            }
            named_sync(1, kConsumerThreads);
            gemv_and_push<N, RM>(cluster, c, nrows, a.n, a.mask, rc, xstride, RM, pos, mcount, rank, csize, warp, lane, a.err);
        }
        cluster_arrive();
        const bool last = m0 + RM >= mem.count;
        if (last && rank >= mcount) return;
        cluster_wait();
        if (warp < kConsumerWarps) {
            const size_t eo = (size_t)e * I + ib * 128u;
            for (uint32_t i = warp; i * csize + rank < mcount; i += kConsumerWarps) {
                const uint32_t m = i * csize + rank;
                float g[4], u[4];
                float sg[4], su[4], sd[4];
                load_scales(static_cast<const __half*>(T3_BANK_FIELD(a, id, gate_svh)) + eo, lane, sg);
                load_scales(static_cast<const __half*>(T3_BANK_FIELD(a, id, up_svh)) + eo, lane, su);
                load_scales(static_cast<const __half*>(T3_BANK_FIELD(a, id, down_suh)) + eo, lane, sd);
                gather_owned(c.recv, owned, i, 0, 2, a.split_gu, lane, g);
                gather_owned(c.recv, owned, i, 1, 2, a.split_gu, lane, u);
                finish_block(g, sg, lane);
                finish_block(u, su, lane);
                float d[4];
#pragma unroll
                for (int q = 0; q < 4; ++q) d[q] = round_half(swiglu(g[q], u[q], a.limit, a.clamp_at)) * sd[q];
                h128_warp(d, lane);
                __half* hd = static_cast<__half*>(a.hd) + (size_t)s_members[m0 + m] * I + ib * 128u;
#pragma unroll
                for (int q = 0; q < 4; ++q) hd[lane + 32u * q] = __float2half_rn(d[q] * kHadScale);
            }
        }
        if (!last) cluster.sync();  // the next pass overwrites the receive tiles
    }
}

// grid (SD, hidden/128, row-slots), cluster (SD, 1, 1): the down projection of every member of the slot's expert from the
// prepared rows hd, finished per row-slot into v (f16): the value the merge weights by the slot's score.
template <int N, int RM>
__device__ __forceinline__ void moe_down_body(const MoeArgs& a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    uint8_t* smem = aligned_smem(smem_raw);
    __shared__ uint32_t s_inds[kMaxSlots];
    __shared__ uint16_t s_members[kMaxSlots];
    __shared__ uint32_t s_count;
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = cluster.block_rank(), csize = a.split_d, hb = blockIdx.y, j = blockIdx.z;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t H = a.hidden, I = a.inter;
    // the routing was complete before the gate|up launch started, so it can be read ahead of pdl_wait
    const Members mem = find_members(a, j, s_inds, s_members, &s_count);
    if (mem.skip) return;
    const uint32_t id = mem.expert, e = a.banked ? id & 0xFFFFFFu : id;

    uint32_t b0, b1;
    slice_blocks(I / 128u, a.split_d, rank, b0, b1);
    const uint32_t nblk = b1 - b0, nrows = nblk * 8u;
    const uint32_t tile_bytes = 2u * a.n, row_bytes = 16u * a.n, out_tiles = H / 16u;
    const Ring rc{a.ring_d.stage_rows, a.ring_d.stages};
    const CtaSmem c = carve(smem, gemv_smem(RM, RM, a.slice_max_d, csize, rc.stage_rows * row_bytes, rc.stages));
    const uint32_t xstride = a.slice_max_d + kXpPad;
    init_barriers(c, rc.stages);
    __syncthreads();

    const size_t expert_bytes = (size_t)(I / 16u) * out_tiles * tile_bytes;
    const uint8_t* wsrc = T3_BANK_FIELD(a, id, down_t) + e * expert_bytes + ((size_t)(b0 * 8u) * out_tiles + hb * 8u) * tile_bytes;
    if (warp == 0) prefetch_l2(static_cast<const __half*>(T3_BANK_FIELD(a, id, down_svh)) + (size_t)e * H + hb * 128u, 256u, lane);
    const uint32_t owned = rows_owned(RM, csize);
    RingPos pos;
    for (uint32_t m0 = 0; m0 < mem.count; m0 += RM) {
        const uint32_t mcount = min((uint32_t)RM, mem.count - m0);
        if (warp == kConsumerWarps) {
            produce_slab(c.ring, c.full, c.empty, wsrc, (size_t)out_tiles * tile_bytes, nrows, row_bytes, rc, pos, lane, a.err);
            pdl_trigger();
        } else {
            pdl_trigger();
            pdl_wait();  // hd is the gate|up launch's output
            for (uint32_t i = mcount * xstride + tid; i < RM * xstride; i += kConsumerThreads) c.xp[i] = __float2half_rn(0.0f);
            for (uint32_t task = warp; task < mcount * nblk; task += kConsumerWarps) {
                const uint32_t m = task / nblk, b = task - m * nblk;
                const __half* src = static_cast<const __half*>(a.hd) + (size_t)s_members[m0 + m] * I + (b0 + b) * 128u;
                __half* dst = c.xp + m * xstride + b * 128u;
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const uint32_t i = lane + 32u * q;
                    dst[(i & ~15u) | lane_order16(i & 15u)] = src[i];
                }
            }
            named_sync(1, kConsumerThreads);
            gemv_and_push<N, RM>(cluster, c, nrows, a.n, a.mask, rc, xstride, RM, pos, mcount, rank, csize, warp, lane, a.err);
        }
        cluster_arrive();
        const bool last = m0 + RM >= mem.count;
        if (last && rank >= mcount) return;
        cluster_wait();
        if (warp < kConsumerWarps) {
            for (uint32_t i = warp; i * csize + rank < mcount; i += kConsumerWarps) {
                const uint32_t m = i * csize + rank;
                float v[4], sv[4];
                load_scales(static_cast<const __half*>(T3_BANK_FIELD(a, id, down_svh)) + (size_t)e * H + hb * 128u, lane, sv);
                gather_owned(c.recv, owned, i, 0, 1, csize, lane, v);
                finish_block(v, sv, lane);
                const uint32_t slot = s_members[m0 + m];
                if (a.topk == 1u) {
                    // One slot a row: the merge has nothing to gather, so the weighted value (and the shared-expert add)
                    // is stored here and the merge launch is skipped. The arithmetic is the merge kernel's, 0 + w v included.
                    const float w = a.scores ? load_act(a.scores, a.score_dt, slot) : 1.0f;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const size_t o = (size_t)slot * H + hb * 128u + lane + 32u * q;
                        float acc = __fadd_rn(0.0f, __fmul_rn(w, v[q]));
                        if (a.shared) {
                            store_act(a.y, a.y_dt, o, acc);
                            acc = __fadd_rn(load_act(a.y, a.y_dt, o), load_act(a.shared, a.y_dt, o));
                        }
                        store_act(a.y, a.y_dt, o, acc);
                    }
                    continue;
                }
                __half* vo = static_cast<__half*>(a.v) + (size_t)slot * H + hb * 128u;
#pragma unroll
                for (int q = 0; q < 4; ++q) vo[lane + 32u * q] = __float2half_rn(v[q]);
            }
        }
        if (!last) cluster.sync();
    }
}

// grid (ceil(hidden / 256), rows): y[row] = sum over the row's slots, in slot order, of score * v in f32 (a multiply and an
// add, as ref.moeRow has it, ref.zig:106), stored in x's dtype; then the optional shared-expert add in that dtype
// (root.moeWithShared, src/root.zig:976-984).
__device__ __forceinline__ void moe_merge_body(const MoeArgs& a) {
    const uint32_t i = blockIdx.x * 256u + threadIdx.x, row = blockIdx.y;
    pdl_trigger();
    pdl_wait();  // v is the down launch's output
    if (i >= a.hidden) return;
    float acc = 0.0f;
    for (uint32_t k = 0; k < a.topk; ++k) {
        const size_t s = (size_t)row * a.topk + k;
        const float w = load_act(a.scores, a.score_dt, s);
        const size_t at = a.row_map ? a.row_map[s] : s;  // where slot s's v row lies (an expert-parallel combine's order)
        acc = __fadd_rn(acc, __fmul_rn(w, __half2float(static_cast<const __half*>(a.v)[at * a.hidden + i])));
    }
    const size_t o = (size_t)row * a.hidden + i;
    if (a.shared) {
        store_act(a.y, a.x_dt, o, acc);
        acc = __fadd_rn(load_act(a.y, a.x_dt, o), load_act(a.shared, a.x_dt, o));
    }
    store_act(a.y, a.x_dt, o, acc);
}

#endif  // T3_SERVED

// ---------------------------------------------------------------------------------------------- launch plumbing

template <typename Args>
using KernelFn = void (*)(const Args);

// Raises a kernel's dynamic shared-memory limit once per device and kernel (the attribute is per device; the call is not
// free and the launches are hot).
cudaError_t allow_big_smem(const void* fn) {
    static std::mutex mu;
    static std::unordered_set<uint64_t> done;
    int dev = 0;
    cudaError_t rc = cudaGetDevice(&dev);
    if (rc != cudaSuccess) return rc;
    const uint64_t key = reinterpret_cast<uint64_t>(fn) ^ ((uint64_t)(dev + 1) << 56);
    std::lock_guard<std::mutex> lock(mu);
    if (done.count(key)) return cudaSuccess;
    rc = cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kGemvSmemLimit);
    if (rc == cudaSuccess) rc = cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);  // clusters of 16
    if (rc == cudaSuccess) done.insert(key);
    return rc;
}

// A cluster launch that may start while the stream's previous kernel is still running (the kernels order themselves
// with griddepcontrol).
template <typename Args>
cudaError_t launch_cluster(KernelFn<Args> fn, const Args& a, dim3 grid, uint32_t cluster_x, uint32_t smem_bytes,
                           bool overlap, cudaStream_t stream) {
    if (smem_bytes > kGemvSmemLimit) return cudaErrorInvalidValue;
    cudaError_t rc = allow_big_smem(reinterpret_cast<const void*>(fn));
    if (rc != cudaSuccess) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kGemvThreads, 1, 1);
    cfg.dynamicSmemBytes = smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 2 : 1;
    note_symbol(reinterpret_cast<const void*>(fn));
    return cudaLaunchKernelEx(&cfg, fn, a);
}

}  // namespace

// ---- entry points ---------------------------------------------------------------------------------------------------
// extern "C" names, as the reference's native kernels have them (t3_<group>_<kernel>_<profile>..., src/kernels/hip/decode/
// decode.hip:355-460), so that a host which binds kernels by name finds them and a launch plan can name them:
//   t3_dense_gemv_<codebook>_n<n>_r<rows>      t3_dec_gate_up_<codebook>_n<n>_r<rows>      t3_dec_down_<codebook>_n<n>_r<rows>
//   t3_dec_merge
// <codebook> mul1 | mcg (probe2..probe4: the dense kernel's timing probes); <n> the rate's halfwords a tile, 0 = any even
// rate at run time; <rows> the row capacity of a pass, 8 | 16 | 32.
#if T3_CB == 0
#define T3_CBNAME mul1
#elif T3_CB == 1
#define T3_CBNAME mcg
#elif T3_CB == 2
#define T3_CBNAME probe2
#elif T3_CB == 3
#define T3_CBNAME probe3
#else
#define T3_CBNAME probe4
#endif
#define T3_NAME2(stem, cb, nn, rm) stem##_##cb##_n##nn##_r##rm
#define T3_NAME(stem, cb, nn, rm) T3_NAME2(stem, cb, nn, rm)
#define T3_ENTRY(STEM, BODY, ARGS, NN, RM)                                                                      \
    extern "C" __global__ void __launch_bounds__(kGemvThreads, 2) T3_NAME(STEM, T3_CBNAME, NN, RM)(const ARGS a) { \
        BODY<NN, RM>(a);                                                                                        \
    }
#if T3_SERVED
#define T3_ENTRIES(STEM, BODY, ARGS, NN) T3_ENTRY(STEM, BODY, ARGS, NN, 8) T3_ENTRY(STEM, BODY, ARGS, NN, 16) T3_ENTRY(STEM, BODY, ARGS, NN, 32)
#else  // the probes exist at the 8-row capacity only
#define T3_ENTRIES(STEM, BODY, ARGS, NN) T3_ENTRY(STEM, BODY, ARGS, NN, 8)
#endif
#define T3_ALL_RATES(STEM, BODY, ARGS)                                                                          \
    T3_ENTRIES(STEM, BODY, ARGS, 0) T3_ENTRIES(STEM, BODY, ARGS, 16) T3_ENTRIES(STEM, BODY, ARGS, 32)           \
    T3_ENTRIES(STEM, BODY, ARGS, 48) T3_ENTRIES(STEM, BODY, ARGS, 64) T3_ENTRIES(STEM, BODY, ARGS, 80)          \
    T3_ENTRIES(STEM, BODY, ARGS, 96) T3_ENTRIES(STEM, BODY, ARGS, 112) T3_ENTRIES(STEM, BODY, ARGS, 128)
T3_ALL_RATES(t3_dense_gemv, dense_gemv_body, DenseArgs)
#if T3_SERVED
T3_ALL_RATES(t3_dec_gate_up, moe_gate_up_body, MoeArgs)
T3_ALL_RATES(t3_dec_down, moe_down_body, MoeArgs)
#endif
#if T3_CB == 0
extern "C" __global__ void __launch_bounds__(256) t3_dec_merge(const MoeArgs a) { moe_merge_body(a); }

// grid (ceil(rows in/128 / 4)), 128 threads: a warp one (row, 128-block) of the input rotation into a.xp_g
extern "C" __global__ void __launch_bounds__(128) t3_dense_prep(const DenseArgs a) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u, nb = a.in / 128u;
    const uint32_t task = blockIdx.x * 4u + warp;
    pdl_trigger();  // the GEMV that follows starts its weight stream now
    pdl_wait();     // x may be the previous kernel's output; the prepared rows' last reader has finished
    if (task >= a.rows * nb) return;
    const uint32_t row = task / nb, b = task - row * nb;
    prepare_block(a.x, a.x_dt, (size_t)row * a.in + b * 128u, static_cast<const __half*>(a.suh) + b * 128u,
                  static_cast<__half*>(const_cast<void*>(a.xp_g)) + (size_t)row * a.in + b * 128u, lane);
}
#endif

#if T3_SERVED
#define T3_PICK_RM(STEM, NN, rm) \
    ((rm) == 8 ? T3_NAME(STEM, T3_CBNAME, NN, 8) : ((rm) == 16 ? T3_NAME(STEM, T3_CBNAME, NN, 16) : T3_NAME(STEM, T3_CBNAME, NN, 32)))
#else
#define T3_PICK_RM(STEM, NN, rm) T3_NAME(STEM, T3_CBNAME, NN, 8)
#endif

#define T3_PICK(STEM, n, rm)                                                       \
    ((n) == 16    ? T3_PICK_RM(STEM, 16, rm)                                        \
     : (n) == 32  ? T3_PICK_RM(STEM, 32, rm)                                        \
     : (n) == 48  ? T3_PICK_RM(STEM, 48, rm)                                        \
     : (n) == 64  ? T3_PICK_RM(STEM, 64, rm)                                        \
     : (n) == 80  ? T3_PICK_RM(STEM, 80, rm)                                        \
     : (n) == 96  ? T3_PICK_RM(STEM, 96, rm)                                        \
     : (n) == 112 ? T3_PICK_RM(STEM, 112, rm)                                       \
     : (n) == 128 ? T3_PICK_RM(STEM, 128, rm)                                       \
                  : T3_PICK_RM(STEM, 0, rm))

#define T3_CAT2(a, b) a##b
#define T3_CAT(a, b) T3_CAT2(a, b)

cudaError_t T3_CAT(launch_dense_gemv_cb, T3_CB)(const DenseArgs& a, cudaStream_t stream) {
    const uint32_t rm = row_cap_for(a.rows);
    KernelFn<DenseArgs> fn = T3_PICK(t3_dense_gemv, a.n, rm);
    const uint32_t cluster = a.part ? 1u : a.split;
    return launch_cluster(fn, a, dim3(a.split, a.out / 128u, 1), cluster, gemv_smem_bytes(rm, a.rows, a.slice_max, cluster, a.n, a.ring),
                          a.overlap != 0, stream);
}

#if T3_CB == 0
cudaError_t launch_dense_prep(const DenseArgs& a, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.rows * (a.in / 128u) + 3u) / 4u, 1, 1);
    cfg.blockDim = dim3(128, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.overlap ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, t3_dense_prep, a);
}
#endif

#if T3_SERVED
cudaError_t T3_CAT(launch_moe_gate_up_cb, T3_CB)(const MoeArgs& a, cudaStream_t stream) {
    const uint32_t rm = a.row_cap;
    KernelFn<MoeArgs> fn = T3_PICK(t3_dec_gate_up, a.n, rm);
    return launch_cluster(fn, a, dim3(2u * a.split_gu, a.inter / 128u, a.rows * a.topk), 2u * a.split_gu,
                          gemv_smem_bytes(rm, rm, a.slice_max_gu, 2u * a.split_gu, a.n, a.ring_gu), a.overlap != 0, stream);
}

cudaError_t T3_CAT(launch_moe_down_cb, T3_CB)(const MoeArgs& a, cudaStream_t stream) {
    const uint32_t rm = a.row_cap;
    KernelFn<MoeArgs> fn = T3_PICK(t3_dec_down, a.n, rm);
    return launch_cluster(fn, a, dim3(a.split_d, a.hidden / 128u, a.rows * a.topk), a.split_d,
                          gemv_smem_bytes(rm, rm, a.slice_max_d, a.split_d, a.n, a.ring_d), a.overlap != 0, stream);
}

#endif  // T3_SERVED
#if T3_CB == 0
cudaError_t launch_moe_merge(const MoeArgs& a, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((a.hidden + 255u) / 256u, a.rows, 1);
    cfg.blockDim = dim3(256, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.overlap ? 1 : 0;
    note_symbol(reinterpret_cast<const void*>(t3_dec_merge));
    return cudaLaunchKernelEx(&cfg, t3_dec_merge, a);
}
#endif

}  // namespace t3
