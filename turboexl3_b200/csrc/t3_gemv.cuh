// The decode-row engine's core: one CTA streams a slab of trellis codes (a K slice of one 128-wide output block)
// through a ring of shared-memory stages filled by bulk copies, decodes each tile in registers straight into
// mma.sync B fragments, and multiplies it with up to 32 prepared activation rows held in shared memory. Decoded weights
// never leave registers. A thread-block cluster splits K; every CTA pushes its partial sums over distributed shared
// memory to the CTA that owns the row (a reduce-scatter in rank order, deterministic), and the owner runs the output
// rotation.
//
// Roles of the 544 threads: warps 0-15 are consumers (warp w owns output tile w % 8 of the block, 16 of its 128 columns,
// and every second tk row, starting at w / 8), warp 16 is the copy producer.
//
// What it computes follows turboexl3's host reference (src/core/format.zig:334-389): xp = f16(H128(f16(x) suh)),
// z = f16(sum xp W_hat) with f32 accumulation, y = f16(H128(z) svh). The launch shape has no counterpart in the
// reference, whose GEMV kernels write split-K planes to device memory and finish in a second launch
// (src/kernels/hip/dense/dense.hip:49-145).
#pragma once

#include <cooperative_groups.h>

#include "t3_common.cuh"

namespace t3 {

namespace cg = cooperative_groups;

constexpr uint32_t kTileWarps = 8;                         // output tiles of a 128-wide block
constexpr uint32_t kKGroups = 2;                           // warps sharing an output tile, interleaved over tk rows
constexpr uint32_t kConsumerWarps = kTileWarps * kKGroups;
constexpr uint32_t kConsumerThreads = 32u * kConsumerWarps;
constexpr uint32_t kGemvThreads = kConsumerThreads + 32u;
constexpr uint32_t kMaxStages = 32;
constexpr uint32_t kPartialStride = 136;  // floats per row of a partial-sum tile (128 + 8: conflict-free float2 stores)
constexpr uint32_t kXpPad = 16;           // halfs added to an xp row so a quad's 8-byte loads spread over the banks
constexpr uint32_t kBatch = 8;            // tiles of a full stage a warp owns (taken two at a time)
constexpr uint32_t kStageRows = kKGroups * kBatch;  // tk rows of a ring stage: two 128-input blocks (a slab's last stage may
                                                    // hold one: slabs are whole 128-input blocks)
constexpr uint32_t kBlockRows = 8;        // tk rows of a 128-input block

// How the ring is cut for one launch (host-chosen)
struct Ring {
    uint32_t stage_rows;  // tk rows a stage, always kStageRows (each row: the block's 8 tiles = 16 n bytes)
    uint32_t stages;      // 1..kMaxStages
};

template <int RM>
struct RowCap {
    static_assert(RM == 8 || RM == 16 || RM == 32, "row capacity");
    static constexpr int kMB = RM == 32 ? 2 : 1;  // 16-row MMA blocks
    static constexpr bool kHalf = RM == 8;        // rows 8-15 of the block are absent
};

// Shared-memory carve-up of a GEMV CTA (byte offsets from a 128-byte aligned base). `cluster` CTAs reduce together.
struct GemvSmem {
    uint32_t bars, xp, local, recv, ring, total;
};
__host__ __device__ inline uint32_t rows_owned(uint32_t rm, uint32_t cluster) { return (rm + cluster - 1u) / cluster; }
// xrows: prepared rows held (the routed kernels hold a pass's row capacity; the dense linear only its live rows: the
// tensor-core steps read a row past the last live one from the last live one, and nobody looks at what that gives)
__host__ __device__ inline GemvSmem gemv_smem(uint32_t rm, uint32_t xrows, uint32_t slice_k, uint32_t cluster, uint32_t stage_bytes,
                                              uint32_t stages) {
    GemvSmem s;
    s.bars = 0;
    s.xp = 2u * kMaxStages * 8u + 128u;  // the ring's full and empty barriers, then one for prepared rows copied in
    const uint32_t xp_bytes = xrows * (slice_k + kXpPad) * 2u;
    s.local = s.xp + ((xp_bytes + 127u) & ~127u);
    s.recv = s.local + ((rm * kPartialStride * 4u + 127u) & ~127u);
    s.ring = s.recv + ((cluster * rows_owned(rm, cluster) * kPartialStride * 4u + 127u) & ~127u);
    s.total = s.ring + stage_bytes * stages;
    return s;
}

// The CTA's dynamic shared memory rounded up to 128 bytes (launches ask for kSmemSlack bytes more than the carve-up).
constexpr uint32_t kSmemSlack = 128;
__device__ __forceinline__ uint8_t* aligned_smem(uint8_t* raw) {
    const uint32_t a = smem_addr(raw);
    return raw + (((a + 127u) & ~127u) - a);
}

// Programmatic dependent launch: `pdl_trigger` lets the next kernel of the stream start its own prologue (its weight
// copies do not depend on this kernel); `pdl_wait` blocks until the previous kernel of the stream has completed and its
// writes are visible. Both are no-ops for a launch without the attribute.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- producer -----------------------------------------------------------------------------------------------------

// Where a warp stands in the ring: the slot it uses next and how many times it has gone round (kept as running counters:
// the stage count is a launch value and integer division is not free).
struct RingPos {
    uint32_t slot = 0, lap = 0;
    __device__ __forceinline__ void advance(uint32_t stages) {
        if (++slot == stages) {
            slot = 0;
            ++lap;
        }
    }
};

// Streams tk rows [0, nrows) of a block's slab into the ring (nrows a multiple of kBlockRows): row r is `row_bytes`
// contiguous bytes at src + r * src_row_stride (bytes). `pos` continues across calls so barrier parities stay in step.
__device__ __forceinline__ void produce_slab(uint8_t* ring, uint64_t* full, uint64_t* empty, const uint8_t* src,
                                             size_t src_row_stride, uint32_t nrows, uint32_t row_bytes, Ring rc,
                                             RingPos& pos, uint32_t lane, uint32_t* err) {
    const uint32_t stage_bytes = kStageRows * row_bytes;
    for (uint32_t r0 = 0; r0 < nrows; r0 += kStageRows) {
        const uint32_t here = min(kStageRows, nrows - r0);  // a full stage, or the slab's last 128-input block
        if (pos.lap > 0) mbar_wait_report(smem_addr(&empty[pos.slot]), (pos.lap - 1u) & 1u, err, kErrEmptyWait);
        if (lane == 0) mbar_arrive_expect_tx(&full[pos.slot], here * row_bytes);
        __syncwarp();
        if (lane < here)
            bulk_copy_g2s(ring + pos.slot * stage_bytes + lane * row_bytes, src + (size_t)(r0 + lane) * src_row_stride,
                          row_bytes, &full[pos.slot]);
        pos.advance(rc.stages);
    }
}

// ---- consumer -----------------------------------------------------------------------------------------------------

// Where a lane finds its rows of the prepared-row buffer (half-element offsets): rows 16 mb + g and 16 mb + 8 + g of the
// tensor-core step's A operand, a row past the last live one read from the last live one
template <int RM>
struct RowOffsets {
    uint32_t lo[RowCap<RM>::kMB], hi[RowCap<RM>::kMB];  // byte offsets
    __device__ __forceinline__ void init(uint32_t lane, uint32_t live, uint32_t xstride) {
        const uint32_t g = lane >> 2, last = live - 1u;
#pragma unroll
        for (int mb = 0; mb < RowCap<RM>::kMB; ++mb) {
            lo[mb] = min((uint32_t)mb * 16u + g, last) * xstride * 2u;
            hi[mb] = min((uint32_t)mb * 16u + 8u + g, last) * xstride * 2u;
        }
    }
};

// loads from this CTA's shared memory by 32-bit shared address (constant parts of an address fold into the instruction)
__device__ __forceinline__ uint32_t lds_u32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds_u64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}

// one decoded tile times the prepared rows at inputs [16 tk, 16 tk + 16): xk is the shared address of the lane's columns there, row 0.
// The product is taken TRANSPOSED, (W tile)^T (16 outputs x 16 inputs) times x^T (16 inputs x 8 rows) a block of 8 rows:
// the decoded words, which are the B fragments of the tile's two column halves, are in another order exactly the A fragment
// of the transposed tile, and the lane's 8-byte load of a prepared row is the whole B fragment. One tensor-core step a tile
// and 8 rows, four accumulators an 8-row block, and no register is moved or zeroed to build an operand. Row block rb = 2 mb
// + nt of the pass is acc[mb][nt], whose element e is (row 8 rb + 2q + (e & 1), column g + 8 (e >> 1)) of the tile (see
// fragment_row, fragment_col). Up to 8 rows only acc[0][0] exists.
template <int RM>
__device__ __forceinline__ void mma_tile(float (&acc)[RowCap<RM>::kMB][2][4], uint32_t xk, const RowOffsets<RM>& ro,
                                         const uint32_t (&b)[4]) {
    if (RowCap<RM>::kHalf) {
        const uint2 lo = lds_u64(xk + ro.lo[0]);
        mma16816(acc[0][0], b[0], b[2], b[1], b[3], lo.x, lo.y);
        return;
    }
#pragma unroll
    for (int mb = 0; mb < RowCap<RM>::kMB; ++mb) {
        const uint2 lo = lds_u64(xk + ro.lo[mb]);
        const uint2 hi = lds_u64(xk + ro.hi[mb]);
        mma16816(acc[mb][0], b[0], b[2], b[1], b[3], lo.x, lo.y);
        mma16816(acc[mb][1], b[0], b[2], b[1], b[3], hi.x, hi.y);
    }
}

// Consumer warp (tile column `tcol`, K group `kg`) folds tk rows kg, kg + kKGroups, ... of [0, nrows) into acc (nrows a
// multiple of kBlockRows). xp: `live_rows` prepared rows in lane order, row stride `xstride` halfs, k = 0 at the slab's
// first input.
// acc[mb][nt] is the (transposed) mma C fragment of rows 8 (2 mb + nt) .. + 7, columns 16 tcol .. + 15.
// A full stage holds kStageRows tk rows, a warp's share of it kBatch tiles taken two at a time, and with the rate
// a template constant every shared-memory offset inside a stage is an immediate.
// HB: tiles whose words and fragments are in registers together (the routed kernels keep two: four spill there).
template <int N, int CB, int RM, int HB = 2>
__device__ __forceinline__ void consume_slab(const uint8_t* ring, uint64_t* full, uint64_t* empty, uint32_t nrows,
                                             uint32_t n_rt, uint32_t mask, Ring rc, const __half* xp, uint32_t xstride,
                                             uint32_t live_rows, RingPos& pos, uint32_t tcol, uint32_t kg, uint32_t lane,
                                             float (&acc)[RowCap<RM>::kMB][2][4], uint32_t* err) {
    constexpr int NP = N > 0 ? N : 16;
    constexpr uint32_t kRaw = raw_words(NP);
    constexpr uint32_t kHalfBatch = (uint32_t)HB;
    static_assert(kBatch % HB == 0 && (kBlockRows / kKGroups) % HB == 0, "a stage, and a last half stage, are whole batches");
    const uint32_t n = N > 0 ? (uint32_t)N : n_rt;
    const uint32_t tile_bytes = 2u * n, row_bytes = 16u * n, stage_bytes = kStageRows * row_bytes;
    LanePlan<NP> plan;
    if (N > 0) plan.init(lane);
    // byte offsets of the lane's raw words inside a stage, from the warp's first row
    uint32_t woff[kRaw];
#pragma unroll
    for (uint32_t i = 0; i < kRaw; ++i) woff[i] = tcol * tile_bytes + kg * row_bytes + plan.idx[i] * 4u;
    uint32_t xs = smem_addr(xp) + (4u * (lane & 3u) + kg * 16u) * 2u;  // shared address of the lane's columns, row 0, this stage
    RowOffsets<RM> ro;
    ro.init(lane, live_rows, xstride);
    const uint32_t full0 = smem_addr(full), empty0 = smem_addr(empty), ring0 = smem_addr(ring);
    uint32_t slot = pos.slot, par = pos.lap & 1u, lap = pos.lap;
    // the slot's barriers and stage as running addresses
    uint32_t full_a = full0 + slot * 8u, empty_a = empty0 + slot * 8u, st = ring0 + slot * stage_bytes;
    const bool lane0 = lane == 0;
#pragma unroll 1
    for (uint32_t r0 = 0; r0 < nrows; r0 += kStageRows, xs += kStageRows * 32u) {
        const uint32_t tiles = min(kStageRows, nrows - r0) / kKGroups;  // this warp's tiles of the stage: 8, or 4 in a last half stage
        mbar_wait_report(full_a, par, err, kErrFullWait);
        if (CB == kProbeStream) {
            // timing probe: the stage has landed, nothing reads it
        } else if (N > 0) {
            // the stage's four tiles of this warp, two at a time: words, then decodes, then tensor-core steps, so the
            // dependent chains of two tiles overlap and the registers of four are never needed at once
            uint32_t wa[kRaw];
#pragma unroll
            for (uint32_t w = 0; w < kRaw; ++w) wa[w] = st + woff[w];
#pragma unroll
            for (uint32_t h = 0; h < kBatch; h += kHalfBatch) {
                if (h >= tiles) break;
                uint32_t raw[kHalfBatch][kRaw];
#pragma unroll
                for (uint32_t i = 0; i < kHalfBatch; ++i)
#pragma unroll
                    for (uint32_t w = 0; w < kRaw; ++w) raw[i][w] = lds_u32(wa[w] + (h + i) * kKGroups * row_bytes);
                uint32_t b[kHalfBatch][4];
#pragma unroll
                for (uint32_t i = 0; i < kHalfBatch; ++i) decode_raw<NP, CB>(raw[i], plan, mask, b[i]);
#pragma unroll
                for (uint32_t i = 0; i < kHalfBatch; ++i) mma_tile<RM>(acc, xs + (h + i) * kKGroups * 32u, ro, b[i]);
            }
        } else {
            const uint8_t* stp = ring + (st - ring0);
#pragma unroll 1
            for (uint32_t i = 0; i < tiles; ++i) {
                uint32_t b[4];
                decode_lane_any<CB>(reinterpret_cast<const uint32_t*>(stp + tcol * tile_bytes + (kg + i * kKGroups) * row_bytes),
                                    n, lane, mask, b);
                mma_tile<RM>(acc, xs + i * kKGroups * 32u, ro, b);
            }
        }
        __syncwarp();
        if (lane0) mbar_arrive_addr(empty_a);
        full_a += 8u, empty_a += 8u, st += stage_bytes;
        if (++slot == rc.stages) slot = 0, par ^= 1u, ++lap, full_a = full0, empty_a = empty0, st = ring0;
    }
    pos.slot = slot, pos.lap = lap;
}

// ---- the cluster reduce-scatter -----------------------------------------------------------------------------------

// Where a lane's accumulators sit in a [rows][128] tile of partial sums: element e of acc[mb][nt] is row fragment_row,
// column tcol * 16 + fragment_col
template <int RM>
__device__ __forceinline__ uint32_t fragment_row(uint32_t lane, int mb, int nt, int e) {
    return 8u * (uint32_t)(2 * mb + nt) + 2u * (lane & 3u) + (uint32_t)(e & 1);
}
template <int RM>
__device__ __forceinline__ uint32_t fragment_col(uint32_t lane, int e) {
    return (lane >> 2) + ((e & 2) ? 8u : 0u);
}
// the 8-row blocks a lane holds a 16-row block of the pass: one up to 8 rows, else two
template <int RM>
struct Frags {
    static constexpr int kNt = RowCap<RM>::kHalf ? 1 : 2;
};

// K group 1's accumulators into the CTA's local tile [RM][kPartialStride]
template <int RM>
__device__ __forceinline__ void store_local(float* local, const float (&acc)[RowCap<RM>::kMB][2][4], uint32_t tcol,
                                            uint32_t lane) {
#pragma unroll
    for (int mb = 0; mb < RowCap<RM>::kMB; ++mb)
#pragma unroll
        for (int nt = 0; nt < Frags<RM>::kNt; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e)
                local[fragment_row<RM>(lane, mb, nt, e) * kPartialStride + tcol * 16u + fragment_col<RM>(lane, e)] = acc[mb][nt][e];
}

// K group 0 adds group 1's tile to its accumulators and pushes each live row m (< count) to the CTA that owns it,
// rank m % csize, into that CTA's recv[my rank][m / csize][column]. Remote stores; the cluster barrier that follows
// makes them visible.
template <int RM>
__device__ __forceinline__ void push_partial(cg::cluster_group& cluster, float* recv, const float* local,
                                             const float (&acc)[RowCap<RM>::kMB][2][4], uint32_t count, uint32_t rank,
                                             uint32_t csize, uint32_t tcol, uint32_t lane) {
    const uint32_t owned = rows_owned(RM, csize);
#pragma unroll
    for (int mb = 0; mb < RowCap<RM>::kMB; ++mb)
#pragma unroll
        for (int nt = 0; nt < Frags<RM>::kNt; ++nt)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const uint32_t m = fragment_row<RM>(lane, mb, nt, e);
                if (m >= count) continue;
                const uint32_t col = tcol * 16u + fragment_col<RM>(lane, e);
                float* dst = cluster.map_shared_rank(recv, m % csize) + (rank * owned + m / csize) * kPartialStride;
                dst[col] = acc[mb][nt][e] + local[m * kPartialStride + col];
            }
}

// Sum over ranks first, first + step, ... (count of them) of owned row `slot`, for the lane's columns lane + 32 j
__device__ __forceinline__ void gather_owned(const float* recv, uint32_t owned, uint32_t slot, uint32_t first,
                                             uint32_t step, uint32_t count, uint32_t lane, float (&v)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = 0.0f;
    // up to 16 ranks; the loads of four ranks are issued together, the sum stays in rank order
    for (uint32_t i0 = 0; i0 < count; i0 += 4u) {
        float t[4][4];
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k) {
            const uint32_t i = i0 + k < count ? i0 + k : count - 1u;
            const float* rp = recv + ((first + i * step) * owned + slot) * kPartialStride + lane;
#pragma unroll
            for (int j = 0; j < 4; ++j) t[k][j] = rp[32 * j];
        }
#pragma unroll
        for (uint32_t k = 0; k < 4u; ++k)
            if (i0 + k < count)
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = (i0 + k == 0u) ? t[k][j] : v[j] + t[k][j];
    }
}

// ---- prepare / finish ---------------------------------------------------------------------------------------------

// One (row, 128-block) of the input rotation by one warp (format.prepareInput, format.zig:334-345): the block's elements
// x[i] (dtype dt) times suh[i], H128, scaled, rounded to f16, into xp_blk at the block's lane-ordered slots.
__device__ __forceinline__ void prepare_block(const void* x, int dt, size_t x_off, const __half* suh, __half* xp_blk,
                                              uint32_t lane) {
    float v[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t i = lane + 32u * j;
        v[j] = round_half(load_act(x, dt, x_off + i)) * __half2float(suh[i]);
    }
    h128_warp(v, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const uint32_t i = lane + 32u * j;
        xp_blk[(i & ~15u) | lane_order16(i & 15u)] = __float2half_rn(v[j] * kHadScale);
    }
}

// The output rotation of one row's 128-block by one warp (format.finishOutput, format.zig:370-380): v[j] holds the
// f32 inner product of column lane + 32 j; returns y = f16(H128(f16(v)) svh) as f32 values in v.
__device__ __forceinline__ void finish_block(float (&v)[4], const float (&sv)[4], uint32_t lane) {
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = round_half(v[j]);
    h128_warp(v, lane);
#pragma unroll
    for (int j = 0; j < 4; ++j) v[j] = round_half(v[j] * kHadScale * sv[j]);
}

// the lane's four scale values of a 128-block (columns lane + 32 j), fetched ahead of the wait they would otherwise follow
__device__ __forceinline__ void load_scales(const __half* blk, uint32_t lane, float (&sv)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) sv[j] = __half2float(blk[lane + 32u * j]);
}

// K blocks [b0, b1) of rank r when nb 128-blocks are cut over s ranks
__host__ __device__ inline void slice_blocks(uint32_t nb, uint32_t s, uint32_t r, uint32_t& b0, uint32_t& b1) {
    b0 = nb * r / s;
    b1 = nb * (r + 1u) / s;
}

}  // namespace t3
