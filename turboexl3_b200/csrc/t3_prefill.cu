// Prefill-row kernels (more than 32 activation rows): the trellis is decoded inside the weight loader of a tcgen05 GEMM.
//
//   route   : counting sort of the row-slots by expert + a table of 128-row M tiles (the reference's route:
//             src/core/kernels/prefill/froute_count.metal, table_2.metal; src/kernels/hip/prefill/prefill.hip:22-71)
//   prep    : input rotation of every sorted row, f16, natural order (format.prepareInput, src/core/format.zig:334-345)
//   gemm    : z = f16(xp W_hat), a 256 x 128 (dense) or 128 x 128 (routed experts, two CTAs a multiprocessor) output tile
//             per CTA, K in stages of 64. One thread of warp 0 feeds two rings: the activation tile by TMA (tiled, 128-byte
//             swizzle) and the stage's code words by bulk copies. Warps 2-17 decode the stage's 32 weight tiles in
//             registers and store them as the K-major 128-byte-swizzled B operand; one thread of warp 1 issues tcgen05.mma
//             (f32 accumulators in tensor memory; with 256 rows two M = 128 halves share each decoded B tile); then warps
//             2-17 read the accumulators back (tcgen05.ld), round to f16 and store. (The reference's GEMM with the decode
//             in the loader: src/core/kernels/prefill/gemm_4.metal, src/kernels/hip/prefill/prefill.hip:125-216, on
//             Apple / gfx11 matrix units.)
//   mid     : gate and up finish, SwiGLU, the down projection's prepare (src/kernels/hip/routed.hpp:64-112)
//   fin     : per row, every slot's down finish and the score-weighted sum in slot order
//             (src/kernels/hip/prefill/prefill.hip:243-264); a dense linear's finish runs in its GEMM's epilogue.
// Every wait is bounded: a wait that runs out sets a bit of the device error word and the kernel walks to its exit,
// freeing its tensor memory on the way.
#include <cuda.h>

#include "t3_common.cuh"
#include "t3_internal.h"

namespace t3 {
namespace {

constexpr uint32_t kBN = 128, kBK = 64;
constexpr uint32_t kBBytes = kBN * kBK * 2u;  // 16 KB
// Decode warps a CTA: a warp takes one of the CTA's 8 tile columns and kTilesPerWarp of a stage's four tile rows. A warp's
// waits, fence, arrivals and ring arithmetic are paid a stage whatever its tiles, so fewer warps with more tiles each issue
// fewer instructions a tile.
constexpr uint32_t kDecodeWarps = 8;
constexpr uint32_t kTilesPerWarp = 32u / kDecodeWarps;           // 4 (8 warps) or 2 (16)
constexpr uint32_t kEpilogueCols = 128u / (kDecodeWarps / 4u);  // accumulator columns a warp moves: 64 or 32
static_assert(kDecodeWarps == 8 || kDecodeWarps == 16, "decode warps");
constexpr uint32_t kGemmThreads = 32u * (2u + kDecodeWarps);
constexpr uint32_t kMaxStages = 4;      // operand stages (A by TMA, B by the decode warps)
constexpr uint32_t kMaxCodeStages = 8;  // stages of the code ring that feeds the decode warps

// The tile heights: 512 rows (four M = 128 accumulators — all of tensor memory — share every decoded B tile, so a stage's
// MMAs outlast its decode and the kernel is bound by the tensor pipe; two operand stages; large dense calls), 256 rows
// (two accumulators, three stages; smaller dense calls) and 128 rows (half the shared memory and a quarter of tensor
// memory, so two CTAs fit a multiprocessor: routed experts, whose tiles are mostly part-full and whose cost is the decode).
// PAIR: 256-row tiles of the routed experts, two CTAs a multiprocessor (two operand stages each, half of tensor memory
// each): a routed tile's cost is its decode, and two CTAs' decode warps keep the multiprocessor's issue slots as busy as two
// 128-row CTAs would, on half the decodes.
template <int BM, bool PAIR = false>
struct Tile {
    static_assert(BM == 128 || BM == 256 || BM == 512, "tile height");
    static_assert(!PAIR || BM == 256, "only 256-row tiles come in the paired form");
    static constexpr uint32_t kABytes = BM * kBK * 2u;
    static constexpr uint32_t kStageBytes = kABytes + kBBytes;
    static constexpr uint32_t kStages = (BM == 512 || PAIR) ? 2u : 3u;
    static constexpr uint32_t kBoxRows = BM % 256u == 0u ? 256u : 128u;  // rows of one TMA box of the activation tile
    static constexpr uint32_t kCodeStages = PAIR ? 3u : (BM == 256 ? 6u : (BM == 512 ? 4u : 3u));
    static constexpr uint32_t kTmemCols = BM;  // 128 f32 columns an accumulator
    static constexpr int kMinBlocks = (BM == 128 || PAIR) ? 2 : 1;
    // dynamic shared memory: operand stages, the code ring (4 tile rows of 16 n bytes a stage), barriers, alignment slack
    static constexpr uint32_t smem(uint32_t n) { return kStages * kStageBytes + kCodeStages * 64u * n + 1024u + 512u; }
};

// ---- tcgen05 / TMA wrappers ----------------------------------------------------------------------------------------

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_addr(dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_addr(bar))
        : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* dst_smem, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(dst_smem)), "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// generic-proxy writes to shared memory made visible to the tensor core's (async proxy) reads
__device__ __forceinline__ void proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// K-major operand tile in shared memory, 128-byte swizzle: rows of 128 bytes, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_byte_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_byte_addr >> 4) & 0x3FFFu);  // start address
    d |= (uint64_t)1u << 16;                            // leading byte offset (unused with 128-byte swizzle)
    d |= (uint64_t)(1024u >> 4) << 32;                  // stride byte offset: next 8-row group
    d |= (uint64_t)1u << 46;                            // descriptor version of this architecture
    d |= (uint64_t)2u << 61;                            // 128-byte swizzle
    return d;
}

// kind::f16, f16 x f16 -> f32, both operands K-major, M = 128, N = kBN; kIdescBf16 switches both operands to bf16
constexpr uint32_t kIdesc = (1u << 4) | ((kBN >> 3) << 17) | ((128u >> 4) << 24);
constexpr uint32_t kIdescBf16 = (1u << 7) | (1u << 10);

__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// the barrier gets one arrival when every tcgen05.mma issued so far by this thread has completed
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar))
                 : "memory");
}

// 16 consecutive f32 columns of this thread's tensor-memory lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The output rotation of one block (format.finishOutput, format.zig:370-380): z and sv point at this lane's first
// element (block start + 4q); out = f16(H128(z) / sqrt(128) * sv).
__device__ __forceinline__ void finish_block_mma(const __half* z, const __half* sv, const HadB& hb, float (&out)[8][4]) {
    uint32_t a[8][2];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint2 u = *reinterpret_cast<const uint2*>(z + 16 * i);
        a[i][0] = u.x, a[i][1] = u.y;
    }
    h128_mma(a, a, false, hb, out);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        float sc[4];
        load_half4(sv + 16 * i, sc);
#pragma unroll
        for (int e = 0; e < 4; ++e) out[i][e] = round_half(out[i][e] * kHadScale * sc[e]);
    }
}

// ---- the GEMM ------------------------------------------------------------------------------------------------------

struct GemmArgs {
    const uint8_t* trellis[2];  // op 0 (gate / the dense weight) and op 1 (up), expert 0's first tile
    size_t expert_bytes;
    uint32_t K, N;              // one op's inner and outer widths
    uint32_t n, mask, ops;
    uint32_t a_op_rows;         // rows between op 0's and op 1's activations in the A buffer
    const int4* tiles;          // (expert, first row, rows, 0) per M tile; null: one matrix, M tiles of kBM rows
    uint32_t dense_rows;
    __half* z;                  // [ops][z_rows][N]
    size_t z_op_stride;         // elements between the ops' outputs
    // The output rotation in the epilogue (the CTA's 128 columns are one rotation block): svh[op] + expert * svh_stride is
    // the op's scale vector; the finished values go to y (dtype y_dt) when it is given, else to z as f16. Null svh[0]: the raw
    // inner products go to z.
    const __half* svh[2];
    size_t svh_stride;
    void* y;                    // [rows][N], one op
    int y_dt;
    uint32_t ab_bf16;           // both operands are bf16 (the un-rotated trunk on bf16 activations); else f16
    // K slices (dense linears of few CTAs; grid z): slice z runs K stages [ksteps z / ksplit, ksteps (z + 1) / ksplit) and
    // leaves its f32 accumulators in part[tile][z][BM][128]; the tile's last arriver (counters[tile], zero before the launch)
    // adds the slices in slice order and finishes. 0 or 1: one CTA runs all of K. With the fused finish only.
    uint32_t ksplit;
    float* part;
    uint32_t* counters;
    uint32_t* err;
};

// RES: the B operand is a kept W_hat (transposed, [N, K] f16) loaded by TMA like A; nothing is decoded.
// SLICED: the K-slice exchange (GemmArgs::ksplit > 1) is compiled in: 128-row tiles of dense linears only, so the routed
// experts' kernels do not carry its registers.
template <int NN, int CB, int BM, bool RES = false, bool PAIR = false, bool SLICED = false>
__global__ void __launch_bounds__(kGemmThreads, Tile<BM, PAIR>::kMinBlocks)
    gemm_decode_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmArgs a) {
    using T = Tile<BM, PAIR>;
    constexpr uint32_t kStages = T::kStages, kStageBytes = T::kStageBytes, kABytes = T::kABytes;
    int e = 0, first = 0, rows = 0;
    if (a.tiles) {
        const int4 t = a.tiles[blockIdx.y];
        e = t.x, first = t.y, rows = t.z;
    } else {
        first = (int)(blockIdx.y * BM);
        rows = min((int)BM, (int)a.dense_rows - first);
    }
    if (rows <= 0) return;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_addr(smem_raw);
    uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
    constexpr uint32_t kCodeStages = T::kCodeStages;
    const uint32_t code_stage_bytes = 64u * a.n;  // 4 tile rows x the CTA's 8 tiles x 2 n bytes
    uint8_t* codes = smem + kStages * kStageBytes;
    uint64_t* bars = reinterpret_cast<uint64_t*>(codes + kCodeStages * code_stage_bytes);
    uint64_t* full_a = bars;
    uint64_t* full_b = bars + kMaxStages;
    uint64_t* empty = bars + 2 * kMaxStages;
    uint64_t* full_c = bars + 3 * kMaxStages;
    uint64_t* empty_c = full_c + kMaxCodeStages;
    uint64_t* acc_full = empty_c + kMaxCodeStages;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t per_op = a.N / kBN, op = blockIdx.x / per_op, nt = blockIdx.x - op * per_op;
    uint32_t ks_lo = 0, ksteps = a.K / kBK;
    if (SLICED) {
        const uint32_t all = ksteps;
        ks_lo = all * blockIdx.z / a.ksplit;
        ksteps = all * (blockIdx.z + 1u) / a.ksplit - ks_lo;
    }
    const uint32_t tile_bytes = 2u * a.n, out_tiles = a.N / 16u;

    if (tid == 0) {
        for (uint32_t s = 0; s < kStages; ++s) {
            mbar_init(&full_a[s], 1u);
            mbar_init(&full_b[s], kDecodeWarps);
            mbar_init(&empty[s], 1u);
        }
        for (uint32_t s = 0; s < kCodeStages; ++s) {
            mbar_init(&full_c[s], 1u);
            mbar_init(&empty_c[s], kDecodeWarps);
        }
        mbar_init(acc_full, 1u);
        mbar_init_fence();
    }
    // the tile's 128 output scales, fetched now so that the epilogue finds them in shared memory
    __half* svh_s = reinterpret_cast<__half*>(reinterpret_cast<uint8_t*>(bars) + 256u);
    if (a.svh[0] != nullptr && tid >= 64u && tid < 64u + kBN)
        svh_s[tid - 64u] = (op ? a.svh[1] : a.svh[0])[(size_t)e * a.svh_stride + nt * kBN + (tid - 64u)];
    if (warp == 1) tmem_alloc(tmem_slot, T::kTmemCols);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // One thread feeds both rings and never blocks on either: it polls the two "slot free" barriers in turn, so the
            // code stream (which runs ahead of the decode) and the activation stream (which follows the MMAs) cannot starve
            // each other. Codes: a stage's four tile rows of the CTA's 8 tiles, 16 n contiguous bytes each.
            const uint8_t* src = (op ? a.trellis[1] : a.trellis[0]) + (size_t)e * a.expert_bytes + (size_t)(nt * 8u) * tile_bytes;
            const size_t tk_stride = (size_t)out_tiles * tile_bytes;
            const uint32_t row_bytes = 8u * tile_bytes;
            uint32_t ka = 0, kc = RES ? ksteps : 0u, idle = 0;
            while (ka < ksteps || kc < ksteps) {
                bool moved = false;
                if (kc < ksteps) {
                    const uint32_t cs = kc % kCodeStages, u = kc / kCodeStages;
                    if (u == 0 || mbar_try(smem_addr(&empty_c[cs]), (u - 1u) & 1u)) {
                        mbar_arrive_expect_tx(&full_c[cs], 4u * row_bytes);
#pragma unroll
                        for (uint32_t i = 0; i < 4u; ++i)
                            bulk_copy_g2s(codes + cs * code_stage_bytes + i * row_bytes,
                                          src + (size_t)((ks_lo + kc) * 4u + i) * tk_stride, row_bytes, &full_c[cs]);
                        ++kc;
                        moved = true;
                    }
                }
                if (ka < ksteps) {
                    const uint32_t s = ka % kStages, u = ka / kStages;
                    if (u == 0 || mbar_try(smem_addr(&empty[s]), (u - 1u) & 1u)) {
                        mbar_arrive_expect_tx(&full_a[s], RES ? kStageBytes : kABytes);
                        const int kx = (int)((ks_lo + ka) * kBK);
                        if (RES) tma_load_2d(smem + s * kStageBytes + kABytes, &tmap_b, kx, (int)(nt * kBN), &full_a[s]);
#pragma unroll
                        for (uint32_t h = 0; h < BM; h += T::kBoxRows)  // a TMA box holds at most 256 rows
                            tma_load_2d(smem + s * kStageBytes + h * kBK * 2u, &tmap_a, kx,
                                        (int)(op * a.a_op_rows) + first + (int)h, &full_a[s]);
                        ++ka;
                        moved = true;
                    }
                }
                idle = moved ? 0u : idle + 1u;
                if (idle > kSpinLimit) {  // neither ring has freed a slot for a very long time: give up, the others will too
                    report(a.err, kErrEmptyWait);
                    break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = kIdesc | (a.ab_bf16 ? kIdescBf16 : 0u);
            for (uint32_t ks = 0; ks < ksteps; ++ks) {
                const uint32_t s = ks % kStages, u = ks / kStages;
                if (!mbar_wait(&full_a[s], u & 1u)) report(a.err, kErrFullWait);
                if (!RES && !mbar_wait(&full_b[s], u & 1u)) report(a.err, kErrFullWait);
                tc_fence_after();
                const uint32_t a_addr = smem_addr(smem + s * kStageBytes), b_addr = a_addr + kABytes;
#pragma unroll
                for (uint32_t kk = 0; kk < kBK / 16u; ++kk) {
                    const uint64_t bdesc = umma_desc(b_addr + kk * 32u);
                    umma_f16(tmem, umma_desc(a_addr + kk * 32u), bdesc, (ks | kk) != 0u, idesc);
#pragma unroll
                    for (uint32_t h = 1; h < BM / 128u; ++h)
                        umma_f16(tmem + h * 128u, umma_desc(a_addr + h * 128u * 128u + kk * 32u), bdesc, (ks | kk) != 0u, idesc);
                }
                umma_commit(&empty[s]);
            }
            umma_commit(acc_full);
        }
    } else {
        // decode warp dw: output tile column dw % 8 of the CTA's 128, input tile rows kTilesPerWarp (dw / 8) .. of a stage (all
        // four with eight warps)
        const uint32_t dw = warp - 2u, tcol = dw & 7u, tk0 = (dw >> 3) * kTilesPerWarp;
        constexpr int NP = NN > 0 ? NN : 16;
        constexpr uint32_t kRaw = raw_words(NP);
        constexpr uint32_t T = kTilesPerWarp;
        LanePlan<NP> plan;
        plan.init(lane);
        // byte offsets of the lane's words of its tiles inside a code stage
        uint32_t woff[T][kRaw];
#pragma unroll
        for (uint32_t i = 0; i < T; ++i)
#pragma unroll
            for (uint32_t w = 0; w < kRaw; ++w) woff[i][w] = ((tk0 + i) * 8u + tcol) * tile_bytes + plan.idx[w] * 4u;
        const uint32_t g = lane >> 2, q = lane & 3u;
        // where the lane's eight half2 words of its tiles go in a B stage:
        // B[n][k] at n * 128 + ((k / 8) ^ (n % 8)) * 16 + (k % 8) * 2; k = 16 tk + 2 q (+8), n = 16 tcol + g (+8)
        const uint32_t row0 = (tcol * 16u + g) * 128u + 4u * q;
        uint32_t boff[T][2];
#pragma unroll
        for (uint32_t i = 0; i < T; ++i) {
            boff[i][0] = row0 + ((2u * (tk0 + i)) ^ g) * 16u;
            boff[i][1] = row0 + ((2u * (tk0 + i) + 1u) ^ g) * 16u;
        }
        for (uint32_t ks = RES ? ksteps : 0u; ks < ksteps; ++ks) {
            const uint32_t s = ks % kStages, u = ks / kStages, cs = ks % kCodeStages, uc = ks / kCodeStages;
            if (!mbar_wait(&full_c[cs], uc & 1u)) report(a.err, kErrFullWait);
            const uint8_t* cst = codes + cs * code_stage_bytes;
            uint32_t b[T][4];
            if (NN > 0) {
                uint32_t raw[T][kRaw];
#pragma unroll
                for (uint32_t i = 0; i < T; ++i)
#pragma unroll
                    for (uint32_t w = 0; w < kRaw; ++w) raw[i][w] = *reinterpret_cast<const uint32_t*>(cst + woff[i][w]);
#pragma unroll
                for (uint32_t i = 0; i < T; ++i) decode_raw<NP, CB>(raw[i], plan, a.mask, b[i]);
            } else {
#pragma unroll
                for (uint32_t i = 0; i < T; ++i)
                    decode_lane_any<CB>(reinterpret_cast<const uint32_t*>(cst + ((tk0 + i) * 8u + tcol) * tile_bytes), a.n, lane,
                                        a.mask, b[i]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_c[cs]);  // the words are in registers: the code stage may be refilled
            if (u > 0 && !mbar_wait(&empty[s], (u - 1u) & 1u)) report(a.err, kErrEmptyWait);
            uint8_t* bst = smem + s * kStageBytes + kABytes;
#pragma unroll
            for (uint32_t i = 0; i < T; ++i) {
                *reinterpret_cast<uint32_t*>(bst + boff[i][0]) = b[i][0];
                *reinterpret_cast<uint32_t*>(bst + boff[i][1]) = b[i][1];
                *reinterpret_cast<uint32_t*>(bst + boff[i][0] + 8u * 128u) = b[i][2];
                *reinterpret_cast<uint32_t*>(bst + boff[i][1] + 8u * 128u) = b[i][3];
            }
            proxy_fence();
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_b[s]);
        }
        // epilogue: a warp reads tensor-memory lanes 32 (warp % 4) .. + 31; the four warps of a lane quarter split the
        // accumulator halves (BM = 256) and the columns between them
        if (!mbar_wait(acc_full, 0u)) report(a.err, kErrMmaWait);
        tc_fence_after();
        // every accumulator's lane quarter `quarter`, columns kEpilogueCols grp .. of its 128, sixteen at a time
        const uint32_t quarter = warp & 3u, grp = dw >> 2;
        const uint32_t col0 = grp * kEpilogueCols;
        constexpr uint32_t kChunks = kEpilogueCols / 16u;
        if (a.svh[0] != nullptr) {
            // Fused finish (format.finishOutput): the accumulators go to shared memory as f16 (the operand stages are
            // free: every MMA and every copy has completed), then a warp takes eight rows at a time through the
            // tensor-core Hadamard, scales by svh, rounds and stores y.
            constexpr uint32_t kZStride = 128u + 8u;  // halfs a row: 16-byte aligned rows, staggered over the banks
            __half* ztile = reinterpret_cast<__half*>(smem);
            bool finisher = true;  // this CTA runs the finish (with K in slices: the tile's last arriver only)
            if (SLICED) {
                // this slice's accumulators to its place in the tile's slab
                const uint32_t tile = blockIdx.y * gridDim.x + blockIdx.x;
                float* slab = a.part + (size_t)tile * a.ksplit * (BM * 128u);
#pragma unroll 1
                for (uint32_t hc = 0; hc < (BM / 128u) * kChunks; ++hc) {
                    const uint32_t half = hc / kChunks, c = (hc % kChunks) * 16u;
                    const uint32_t r = half * 128u + quarter * 32u + lane;
                    uint32_t v[16];
                    tmem_ld16(tmem + ((quarter * 32u) << 16) + half * 128u + col0 + c, v);
                    if ((int)r < rows) {
                        float4* dst = reinterpret_cast<float4*>(slab + ((size_t)blockIdx.z * BM + r) * 128u + col0 + c);
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            __stcg(dst + j, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                        __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
                    }
                }
                tc_fence_before();
                __threadfence();
                named_sync(2, kDecodeWarps * 32u);
                volatile uint32_t* last_slot = tmem_slot + 2;
                if (dw == 0u && lane == 0u) *last_slot = atomicAdd(&a.counters[tile], 1u) == a.ksplit - 1u ? 1u : 0u;
                named_sync(2, kDecodeWarps * 32u);
                finisher = *last_slot != 0u;
                if (finisher) {
                    __threadfence();
                    if (dw == 0u && lane == 0u) a.counters[tile] = 0u;  // as the next call on this workspace expects it
                    // The slices' sums in slice order, by all the decode warps together: a thread takes float4 positions of
                    // the tile's live rows 256 apart (a warp reads whole 512-byte rows), two positions' loads of every slice
                    // in flight at once. (Rows past the tile's last are never stored.)
                    const uint32_t tid_d = dw * 32u + lane, live = (uint32_t)rows * 32u;
                    const uint32_t nz = a.ksplit;
#pragma unroll 1
                    for (uint32_t p0 = tid_d; p0 < live; p0 += 2u * kDecodeWarps * 32u) {
                        float4 t[2][8];
#pragma unroll
                        for (uint32_t b = 0; b < 2u; ++b) {
                            const uint32_t p = p0 + b * kDecodeWarps * 32u;
                            const float4* src = reinterpret_cast<const float4*>(slab) + p;
#pragma unroll
                            for (uint32_t z = 0; z < 8u; ++z)
                                if (z < nz && p < live) t[b][z] = __ldcg(src + (size_t)z * (BM * 32u));
                        }
#pragma unroll
                        for (uint32_t b = 0; b < 2u; ++b) {
                            const uint32_t p = p0 + b * kDecodeWarps * 32u;
                            if (p >= live) continue;
                            float4 acc = t[b][0];
#pragma unroll
                            for (uint32_t z = 1; z < 8u; ++z)
                                if (z < nz) acc.x += t[b][z].x, acc.y += t[b][z].y, acc.z += t[b][z].z, acc.w += t[b][z].w;
                            const __half2 lo = __floats2half2_rn(acc.x, acc.y), hi = __floats2half2_rn(acc.z, acc.w);
                            *reinterpret_cast<uint2*>(ztile + (p >> 5) * kZStride + (p & 31u) * 4u) =
                                make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
                        }
                    }
                }
            } else {
#pragma unroll 1
                for (uint32_t hc = 0; hc < (BM / 128u) * kChunks; ++hc) {
                    const uint32_t half = hc / kChunks, c = (hc % kChunks) * 16u;
                    const uint32_t r = half * 128u + quarter * 32u + lane;
                    uint32_t v[16];
                    tmem_ld16(tmem + ((quarter * 32u) << 16) + half * 128u + col0 + c, v);
                    uint32_t packed[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const __half2 h = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                    uint4* dst = reinterpret_cast<uint4*>(ztile + r * kZStride + col0 + c);
                    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                }
            }
            if (finisher) {
                tc_fence_before();
                named_sync(2, kDecodeWarps * 32u);
                const HadB hb = had_b(lane);
                const uint32_t pg = lane >> 2, pq = lane & 3u;
                const __half* sv = svh_s + 4u * pq;
                void* const dst = a.y ? a.y : static_cast<void*>(a.z);
                const int dst_dt = a.y ? a.y_dt : (int)kF16;
#pragma unroll 1
                for (uint32_t g8 = dw; g8 < BM / 8u; g8 += kDecodeWarps) {
                    const uint32_t r = g8 * 8u + pg;
                    float out[8][4];
                    finish_block_mma(ztile + r * kZStride + 4u * pq, sv, hb, out);
                    if ((int)r < rows) {
                        const size_t o = op * a.z_op_stride + (size_t)(first + (int)r) * a.N + nt * kBN + 4u * pq;
#pragma unroll
                        for (int i = 0; i < 8; ++i) store_act4(dst, dst_dt, o + 16u * i, out[i]);
                    }
                }
            }
        } else
#pragma unroll 1
        for (uint32_t hc = 0; hc < (BM / 128u) * kChunks; ++hc) {
            const uint32_t half = hc / kChunks, c = (hc % kChunks) * 16u;
            const int r = (int)(half * 128u + quarter * 32u + lane);
            // the inner products as they are: to y in its 16-bit dtype when it is given (one rounding: the un-rotated
            // trunk), else to z as f16
            __half* zrow = (a.y ? static_cast<__half*>(a.y) : a.z + op * a.z_op_stride) + (size_t)(first + r) * a.N + nt * kBN + col0;
            const bool to_bf16 = a.y != nullptr && a.y_dt == (int)kBf16;
            uint32_t v[16];
            tmem_ld16(tmem + ((quarter * 32u) << 16) + half * 128u + col0 + c, v);
            if (r < rows) {
                uint32_t packed[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (to_bf16) {
                        const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                    } else {
                        const __half2 h = __floats2half2_rn(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]));
                        packed[j] = *reinterpret_cast<const uint32_t*>(&h);
                    }
                }
                uint4* dst = reinterpret_cast<uint4*>(zrow + c);
                dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
        }
        tc_fence_before();
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, T::kTmemCols);
    }
}

// ---- route ---------------------------------------------------------------------------------------------------------

__global__ void route_count_kernel(const uint32_t* inds, uint32_t slots, uint32_t experts, uint32_t* counts) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < slots) atomicAdd(&counts[min(inds[s], experts - 1u)], 1u);
}

// How an expert's c rows are cut into M tiles: 512-row tiles while more than 384 rows are left, then one 256-row tile
// (and a 128-row one for what is past 256), or one 128-row tile. A tile decodes its expert's weights once whatever its
// height, and the decode is what a routed GEMM costs, so an expert's rows go into as few tiles as the accumulators hold
// (the reference sizes its tiles by the expert's row count for the same reason, src/core/kernels/prefill/table_2.metal).
struct TileCut {
    uint32_t n512, n256, n128;
};
__host__ __device__ inline TileCut cut_rows(uint32_t c, bool uniform) {
    TileCut t = {0u, 0u, 0u};
    if (uniform) {  // 128-row tiles only
        t.n128 = (c + 127u) / 128u;
        return t;
    }
    while (c > 384u) {
        ++t.n512;
        c -= c < 512u ? c : 512u;
    }
    if (c > 256u) t.n256 = 1u, t.n128 = 1u;
    else if (c > 128u) t.n256 = 1u;
    else if (c > 0u) t.n128 = 1u;
    return t;
}

// Tile tables by height: (expert, first row, rows, 0) each; a table's unused tail is zero rows
struct TileTables {
    int4* t[3];       // 512-, 256-, 128-row tiles
    uint32_t max[3];
    uint32_t uniform;  // 1: every tile is a 128-row tile (calls with few rows an expert: one launch a GEMM instead of three)
};

// one CTA: each expert's first sorted position (exclusive scan of the counts) into `cursor`, and the M-tile tables
__global__ void __launch_bounds__(1024) route_plan_kernel(const uint32_t* counts, uint32_t experts, uint32_t* cursor,
                                                          const TileTables tt) {
    __shared__ uint32_t s_scan[4][1024];
    __shared__ uint32_t base[4];
    const uint32_t tid = threadIdx.x;
    if (tid < 4u) base[tid] = 0;
    __syncthreads();
    // experts are walked in chunks of 1024 with running bases
    for (uint32_t e0 = 0; e0 < experts; e0 += 1024u) {
        const uint32_t e = e0 + tid;
        const uint32_t c = e < experts ? counts[e] : 0u;
        const TileCut cut = cut_rows(c, tt.uniform != 0u);
        const uint32_t mine[4] = {c, cut.n512, cut.n256, cut.n128};
#pragma unroll
        for (int k = 0; k < 4; ++k) s_scan[k][tid] = mine[k];
        __syncthreads();
        for (uint32_t off = 1; off < 1024u; off <<= 1) {  // inclusive Hillis-Steele scans
            uint32_t add[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) add[k] = tid >= off ? s_scan[k][tid - off] : 0u;
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 4; ++k) s_scan[k][tid] += add[k];
            __syncthreads();
        }
        if (e < experts) {
            const uint32_t pos0 = base[0] + s_scan[0][tid] - c;
            cursor[e] = pos0;
            uint32_t at[3];
#pragma unroll
            for (int k = 0; k < 3; ++k) at[k] = base[k + 1] + s_scan[k + 1][tid] - mine[k + 1];
            uint32_t first = pos0, left = c;
            for (uint32_t i = 0; i < cut.n512; ++i) {
                const uint32_t r = left < 512u ? left : 512u;
                if (at[0] + i < tt.max[0]) tt.t[0][at[0] + i] = make_int4((int)e, (int)first, (int)r, 0);
                first += r, left -= r;
            }
            if (cut.n256) {
                const uint32_t r = left < 256u ? left : 256u;
                if (at[1] < tt.max[1]) tt.t[1][at[1]] = make_int4((int)e, (int)first, (int)r, 0);
                first += r, left -= r;
            }
            for (uint32_t i = 0; i < cut.n128; ++i) {
                const uint32_t r = left < 128u ? left : 128u;
                if (at[2] + i < tt.max[2]) tt.t[2][at[2] + i] = make_int4((int)e, (int)first, (int)r, 0);
                first += r, left -= r;
            }
        }
        __syncthreads();
        if (tid < 4u) base[tid] += s_scan[tid][1023];
        __syncthreads();
    }
#pragma unroll
    for (int k = 0; k < 3; ++k)
        for (uint32_t i = base[k + 1] + tid; i < tt.max[k]; i += 1024u) tt.t[k][i] = make_int4(0, 0, 0, 0);
}

__global__ void route_scatter_kernel(const uint32_t* inds, uint32_t slots, uint32_t experts, uint32_t* cursor,
                                     uint32_t* order, uint32_t* inv) {
    const uint32_t s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s >= slots) return;
    const uint32_t p = atomicAdd(&cursor[min(inds[s], experts - 1u)], 1u);
    order[p] = s;
    inv[s] = p;
}

// ---- prepare / mid / finish ------------------------------------------------------------------------------------------

constexpr uint32_t kRowsPerCta = 64;  // 8 warps x 8 positions

// how many CTAs share a position group's 128-blocks, so that small calls still fill the GPU
uint32_t spread(uint32_t positions, uint32_t nblk) {
    const uint32_t groups = (positions + kRowsPerCta - 1u) / kRowsPerCta;
    const uint32_t want = (1184u + groups - 1u) / groups;
    return want < 1u ? 1u : (want > nblk ? nblk : want);
}

// this lane's position in a warp's group of eight; returns false when the whole warp is past the end
__device__ __forceinline__ bool my_position(uint32_t count, uint32_t lane, uint32_t& p, bool& live) {
    const uint32_t first = (blockIdx.y * 8u + (threadIdx.x >> 5)) * 8u;
    if (first >= count) return false;
    const uint32_t mine = first + (lane >> 2);
    live = mine < count;
    p = live ? mine : count - 1u;
    return true;
}

// grid (spread, ceil(P / 64)), 256 threads. Dense: position = row, suh shared. Routed: position p -> slot order[p] -> row
// slot / topk, suh of the slot's expert; the second op (up) reuses the row with its own suh.
struct PrepArgs {
    const void* x;
    int x_dt;
    const __half* suh[2];
    uint32_t K, positions, topk, experts, ops;
    const uint32_t *order, *inds;  // null for a dense linear
    const uint32_t* row_map;       // routed: the x row of each row-slot when the call gathers rows, else slot / topk
    __half* xp;                    // [ops][positions][K]
};
__global__ void __launch_bounds__(256, 3) prep_rows_kernel(const PrepArgs a) {
    const uint32_t lane = threadIdx.x & 31u, q = lane & 3u;
    uint32_t p;
    bool live;
    if (!my_position(a.positions, lane, p, live)) return;
    uint32_t row = p, e = 0;
    if (a.order) {
        const uint32_t slot = a.order[p];
        row = a.row_map ? a.row_map[slot] : slot / a.topk;
        e = min(a.inds[slot], a.experts - 1u);
    }
    const HadB hb = had_b(lane);
    for (uint32_t blk = blockIdx.x; blk < (a.K >> 7); blk += gridDim.x) {
        const uint32_t col = blk * 128u + 4u * q;
        float xv[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) load_act4(a.x, a.x_dt, (size_t)row * a.K + col + 16u * i, xv[i]);
        for (uint32_t op = 0; op < a.ops; ++op) {
            const __half* suh = (op ? a.suh[1] : a.suh[0]) + (size_t)e * a.K + col;
            float v[8][4], out[8][4];
            bool unit = true;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float sc[4];
                load_half4(suh + 16 * i, sc);
                unit = unit && all_unit(sc);
#pragma unroll
                for (int j = 0; j < 4; ++j) v[i][j] = round_half(xv[i][j]) * sc[j];
            }
            h128_split(v, __all_sync(0xFFFFFFFFu, unit) != 0, hb, out);
            if (live) {
                const size_t o = ((size_t)op * a.positions + p) * a.K + col;
#pragma unroll
                for (int i = 0; i < 8; ++i) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) out[i][j] *= kHadScale;
                    store_act4(a.xp, kF16, o + 16u * i, out[i]);
                }
            }
        }
    }
}

__device__ __forceinline__ float swiglu_f32(float g, float u, float limit, int clamp_at) {
    if (limit > 0.0f) {
        u = u > limit ? limit : (u < -limit ? -limit : u);
        if (clamp_at == 0) g = g > limit ? limit : g;
    }
    float s = g / (1.0f + expf(-g));
    if (limit > 0.0f && clamp_at != 0) s = s > limit ? limit : s;
    return s * u;
}

// grid (spread, ceil(P / 64)): SwiGLU of the finished gate and up values (the GEMM's epilogue finished them) and the
// down projection's prepare, per sorted position
struct MidArgs {
    const __half* z;  // [2][P][inter]: finished gate, finished up
    const __half* down_suh;
    const uint32_t *order, *inds;
    uint32_t positions, inter, experts;
    float limit;
    int clamp_at;
    __half* hd;  // [P][inter]
};
__global__ void __launch_bounds__(256, 3) mid_kernel(const MidArgs a) {
    const uint32_t lane = threadIdx.x & 31u, q = lane & 3u;
    uint32_t p;
    bool live;
    if (!my_position(a.positions, lane, p, live)) return;
    const uint32_t e = min(a.inds[a.order[p]], a.experts - 1u);
    const HadB hb = had_b(lane);
    for (uint32_t blk = blockIdx.x; blk < (a.inter >> 7); blk += gridDim.x) {
        const size_t eo = (size_t)e * a.inter + blk * 128u + 4u * q, zo = (size_t)p * a.inter + blk * 128u + 4u * q;
        float g[8][4], u[8][4];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            load_half4(a.z + zo + 16 * i, g[i]);
            load_half4(a.z + (size_t)a.positions * a.inter + zo + 16 * i, u[i]);
        }
        bool unit = true;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            float sd[4];
            load_half4(a.down_suh + eo + 16 * i, sd);
            unit = unit && all_unit(sd);
#pragma unroll
            for (int j = 0; j < 4; ++j) g[i][j] = round_half(swiglu_f32(g[i][j], u[i][j], a.limit, a.clamp_at)) * sd[j];
        }
        h128_split(g, __all_sync(0xFFFFFFFFu, unit) != 0, hb, u);
        if (live)
#pragma unroll
            for (int i = 0; i < 8; ++i) {
#pragma unroll
                for (int j = 0; j < 4; ++j) u[i][j] *= kHadScale;
                store_act4(a.hd, kF16, zo + 16u * i, u[i]);
            }
    }
}

// grid (spread, ceil(rows / 64)): per row, the score-weighted sum of its slots' finished down outputs (through inv) in
// slot order, then the optional shared-expert add in the output dtype
struct FinArgs {
    const __half* zd;  // [P][hidden]: each sorted position's finished down output (the per-slot v)
    const uint32_t* inv;
    const void* scores;
    int score_dt;
    const void* shared;
    void* y;
    int y_dt;
    uint32_t rows, hidden, topk;
};
__global__ void __launch_bounds__(256) moe_fin_kernel(const FinArgs a) {
    // a warp a row, a lane four consecutive elements of a 128-block: every slot's 256 bytes are one coalesced read
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t row = blockIdx.y * 8u + warp;
    if (row >= a.rows) return;
    for (uint32_t blk = blockIdx.x; blk < (a.hidden >> 7); blk += gridDim.x) {
        const uint32_t col = blk * 128u + 4u * lane;
        float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        for (uint32_t k0 = 0; k0 < a.topk; k0 += 4u) {  // four slots' loads in flight, the sum still in slot order
            float w[4], v[4][4];
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i) {
                const uint32_t k = k0 + i < a.topk ? k0 + i : a.topk - 1u;
                const size_t slot = (size_t)row * a.topk + k;
                w[i] = load_act(a.scores, a.score_dt, slot);
                load_half4(a.zd + (size_t)a.inv[slot] * a.hidden + col, v[i]);
            }
#pragma unroll
            for (uint32_t i = 0; i < 4u; ++i)
                if (k0 + i < a.topk)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[j] = __fadd_rn(acc[j], __fmul_rn(w[i], v[i][j]));
        }
        const size_t o = (size_t)row * a.hidden + col;
        if (a.shared) {
            float t[4], sh[4];
            store_act4(a.y, a.y_dt, o, acc);  // the routed output's rounding point
            load_act4(a.y, a.y_dt, o, t);
            load_act4(a.shared, a.y_dt, o, sh);
#pragma unroll
            for (int j = 0; j < 4; ++j) acc[j] = __fadd_rn(t[j], sh[j]);
        }
        store_act4(a.y, a.y_dt, o, acc);
    }
}

// ---- host side -----------------------------------------------------------------------------------------------------

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// f16 [rows, K] row-major, boxes of kBK x bm, 128-byte swizzle, rows past the end read as zero
bool make_a_map(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t bm) {
    EncodeTiledFn fn = encode_tiled();
    if (!fn) return false;
    const cuuint64_t dims[2] = {K, rows};
    const cuuint64_t strides[1] = {K * 2u};
    const cuuint32_t box[2] = {kBK, bm};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// the resident GEMM: both operands by TMA
template <int BM>
cudaError_t launch_gemm_resident(const CUtensorMap& map_a, const CUtensorMap& map_b, const GemmArgs& g, uint32_t max_tiles,
                                 cudaStream_t stream) {
    void (*fn)(const CUtensorMap, const CUtensorMap, const GemmArgs) = gemm_decode_kernel<0, 0, BM, true>;
    if (BM == 128 && g.ksplit > 1u) fn = gemm_decode_kernel<0, 0, 128, true, false, true>;
    const uint32_t smem_bytes = Tile<BM>::smem(0);
    cudaError_t rc = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)smem_bytes);
    if (rc != cudaSuccess) return rc;
    fn<<<dim3(g.N / kBN, max_tiles, g.ksplit > 1u ? g.ksplit : 1u), kGemmThreads, smem_bytes, stream>>>(map_a, map_b, g);
    return cudaGetLastError();
}

template <int CB, int BM, bool PAIR = false, bool kSliced = false>
cudaError_t launch_gemm_cb(const CUtensorMap& map, const GemmArgs& g, uint32_t max_tiles, cudaStream_t stream) {
    void (*fn)(const CUtensorMap, const CUtensorMap, const GemmArgs) = nullptr;
    switch (g.n) {
#define T3_CASE(NN) \
    case NN: fn = gemm_decode_kernel<NN, CB, BM, false, PAIR, kSliced>; break;
        T3_CASE(16) T3_CASE(32) T3_CASE(48) T3_CASE(64) T3_CASE(80) T3_CASE(96) T3_CASE(112) T3_CASE(128)
#undef T3_CASE
        default: fn = gemm_decode_kernel<0, CB, BM, false, PAIR, kSliced>; break;
    }
    const uint32_t smem_bytes = Tile<BM, PAIR>::smem(g.n);
    cudaError_t rc = cudaFuncSetAttribute(reinterpret_cast<const void*>(fn), cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)Tile<BM, PAIR>::smem(128u));
    if (rc != cudaSuccess) return rc;
    fn<<<dim3(g.ops * g.N / kBN, max_tiles, g.ksplit > 1u ? g.ksplit : 1u), kGemmThreads, smem_bytes, stream>>>(map, map, g);
    return cudaGetLastError();
}

// bm: the tile height (512, 256, 128); pair: 256-row tiles two CTAs a multiprocessor (the routed experts')
cudaError_t launch_gemm(const CUtensorMap& map, const GemmArgs& g, uint32_t max_tiles, uint32_t bm, int codebook,
                        cudaStream_t stream, bool pair = false) {
    if (bm == 512u)
        return codebook == kMcg ? launch_gemm_cb<kMcg, 512>(map, g, max_tiles, stream)
                                : launch_gemm_cb<kMul1, 512>(map, g, max_tiles, stream);
    if (bm == 256u && pair)
        return codebook == kMcg ? launch_gemm_cb<kMcg, 256, true>(map, g, max_tiles, stream)
                                : launch_gemm_cb<kMul1, 256, true>(map, g, max_tiles, stream);
    if (bm == 256u)
        return codebook == kMcg ? launch_gemm_cb<kMcg, 256>(map, g, max_tiles, stream)
                                : launch_gemm_cb<kMul1, 256>(map, g, max_tiles, stream);
    if (g.ksplit > 1u)  // the K-slice exchange compiled in (dense linears of few rows)
        return codebook == kMcg ? launch_gemm_cb<kMcg, 128, false, true>(map, g, max_tiles, stream)
                                : launch_gemm_cb<kMul1, 128, false, true>(map, g, max_tiles, stream);
    return codebook == kMcg ? launch_gemm_cb<kMcg, 128>(map, g, max_tiles, stream)
                            : launch_gemm_cb<kMul1, 128>(map, g, max_tiles, stream);
}

size_t up256(size_t v) { return (v + 255u) & ~(size_t)255u; }

// multiprocessors of the current device (one 512- or 256-row CTA fits each)
uint32_t one_wave_ctas() {
    static int sms = [] {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess)
            n = 148;
        return n;
    }();
    return (uint32_t)sms;
}

}  // namespace

// ---- dense linear, more than 32 rows ---------------------------------------------------------------------------------

// K slices of a dense linear of few rows: a call of up to 512 rows is one to four M tiles of 128 rows, out / 128 CTAs each,
// every one decoding all of its 128 columns' weights (a 6144 -> 2048 linear ran on 16 to 64 CTAs for 66 us whatever its
// rows). Such calls cut K into slices, a CTA a slice, that meet in global memory (see GemmArgs::ksplit). Two arms, 33..256
// rows (two M tiles at most) and 257..512 (four), each with a slice count that follows the geometry alone, so a row's bytes
// do not depend on the call's row count within an arm. The count: what fills two CTAs a multiprocessor at the arm's most
// tiles, eight at most (the tile's last arriver reads every slice), four K stages a slice at least — eight where K is short
// (under 64 stages), and there only while every CTA has a multiprocessor to itself and only in the first arm: with short K
// the slab's traffic and two CTAs sharing a multiprocessor cost what the slices save (measured: 2048 -> 6144 at 256 rows
// 35 us in three slices against 29, 2048 -> 2048 at 512 rows 32 us in four against 28).
uint32_t prefill_ksplit(size_t rows, uint32_t in, uint32_t out) {
    if (rows > 512u) return 1u;
    const uint32_t ncol = out / kBN, ksteps = in / kBK, sms = one_wave_ctas();
    const bool long_k = ksteps >= 64u;
    const uint32_t mtiles = rows <= 256u ? 2u : 4u;
    if (mtiles == 4u && !long_k) return 1u;
    uint32_t s = (2u * sms) / (mtiles * ncol);
    s = s < 8u ? s : 8u;
    const uint32_t by_k = long_k ? ksteps / 4u : ksteps / 8u;
    s = s < by_k ? s : by_k;
    if (s < 2u) return 1u;
    if (!long_k && mtiles * ncol * s > sms) return 1u;
    return s;
}

// the prepared rows (the GEMM's epilogue finishes into y, so the inner products of an unsliced call never reach memory);
// for a sliced call the slices' partial sums and the tiles' arrival counters as well
size_t prefill_linear_workspace(size_t rows, uint32_t in, uint32_t out) {
    size_t bytes = up256(rows * in * 2u);
    const uint32_t s = prefill_ksplit(rows, in, out);
    if (s > 1u) {
        const size_t mtiles = (rows + 127u) / 128u, ncol = out / kBN;
        bytes += up256(mtiles * ncol * s * 128u * 128u * 4u) + up256(mtiles * ncol * 4u);
    }
    return bytes;
}

cudaError_t launch_prefill_linear(const PrefillLinearArgs& p, int codebook, cudaStream_t stream, int* launches) {
    uint8_t* ws = static_cast<uint8_t*>(p.workspace);
    __half* xp = reinterpret_cast<__half*>(ws);
    PrepArgs pa = {};
    pa.x = p.x;
    pa.x_dt = p.x_dt;
    pa.suh[0] = pa.suh[1] = static_cast<const __half*>(p.suh);
    pa.K = p.in;
    pa.positions = p.rows;
    pa.topk = 1;
    pa.experts = 1;
    pa.xp = xp;
    pa.ops = 1;
    prep_rows_kernel<<<dim3(spread(p.rows, p.in / 128u), (p.rows + kRowsPerCta - 1u) / kRowsPerCta), 256, 0, stream>>>(pa);
    // Tile height: the one whose rounds of CTAs take the least time, a round of BM-row tiles costing about BM + 128 (a CTA's
    // fixed part: set-up, first loads, epilogue; and a shorter tile amortises its decoded B tile over fewer rows). Two
    // 128-row CTAs share a multiprocessor, so a full round of those costs twice one. Ties go to the taller tile. (Three
    // accumulators with three stages measured no faster than four with two.)
    const uint32_t sms = one_wave_ctas(), ncol = p.out / kBN;
    uint32_t bm = 512u, best = ~0u;
    for (uint32_t cand : {512u, 256u, 128u}) {
        const uint32_t ctas = ((p.rows + cand - 1u) / cand) * ncol;
        const uint32_t cost = cand == 128u ? (ctas <= sms ? 256u : ((ctas + 2u * sms - 1u) / (2u * sms)) * 512u)
                                           : ((ctas + sms - 1u) / sms) * (cand + 128u);
        if (cost < best) best = cost, bm = cand;
    }
    GemmArgs g = {};
    const uint32_t ksplit = prefill_ksplit(p.rows, p.in, p.out);
    if (ksplit > 1u) {
        // K slices on 128-row tiles: the slab of partial sums and the counters follow the prepared rows in the workspace
        bm = 128u;
        const size_t mtiles = (p.rows + 127u) / 128u;
        uint8_t* at = ws + up256((size_t)p.rows * p.in * 2u);
        g.ksplit = ksplit;
        g.part = reinterpret_cast<float*>(at);
        g.counters = reinterpret_cast<uint32_t*>(at + up256(mtiles * ncol * ksplit * 128u * 128u * 4u));
        const cudaError_t mrc = cudaMemsetAsync(g.counters, 0, mtiles * ncol * 4u, stream);
        if (mrc != cudaSuccess) return mrc;
    }
    CUtensorMap map;
    if (!make_a_map(&map, xp, p.rows, p.in, bm == 128u ? 128u : 256u)) return cudaErrorNotSupported;
    g.trellis[0] = g.trellis[1] = p.trellis;
    g.K = p.in;
    g.N = p.out;
    g.n = p.resident ? 0u : p.n;  // no code ring beside a kept weight: the barriers follow the operand stages directly
    g.mask = p.mask;
    g.ops = 1;
    g.dense_rows = p.rows;
    g.svh[0] = g.svh[1] = static_cast<const __half*>(p.svh);
    g.y = p.y;
    g.y_dt = p.x_dt;
    g.err = p.err;
    cudaError_t rc;
    if (p.resident) {
        CUtensorMap map_b;  // W_hat transposed [out, in]: boxes of 64 inputs x 128 outputs, the decoded B tile's layout
        if (!make_a_map(&map_b, p.resident, p.out, p.in, kBN)) return cudaErrorNotSupported;
        rc = bm == 512u   ? launch_gemm_resident<512>(map, map_b, g, (p.rows + bm - 1u) / bm, stream)
             : bm == 256u ? launch_gemm_resident<256>(map, map_b, g, (p.rows + bm - 1u) / bm, stream)
                          : launch_gemm_resident<128>(map, map_b, g, (p.rows + bm - 1u) / bm, stream);
    } else {
        rc = launch_gemm(map, g, (p.rows + bm - 1u) / bm, bm, codebook, stream);
    }
    if (rc != cudaSuccess) return rc;
    *launches += 2;  // the output rotation runs in the GEMM's epilogue
    return cudaGetLastError();
}

// ---- the un-rotated trunk, more than 32 rows ----------------------------------------------------------------------------

// One launch: both operands by TMA as they lie in memory (x [rows, in] and W_std transposed [out, in], the same 16-bit
// dtype), the epilogue rounds the f32 accumulators once into y (dense.residentPlain, src/core/dense.zig:1261-1263: "one
// matmul of x against its resident W_std in x's dtype").
cudaError_t launch_plain_linear(const void* x, int dt, uint32_t rows, const void* w_std_t, uint32_t in, uint32_t out, void* y,
                                uint32_t* err, cudaStream_t stream) {
    const uint32_t sms = one_wave_ctas(), ncol = out / kBN;
    uint32_t bm = 512u, best = ~0u;
    for (uint32_t cand : {512u, 256u, 128u}) {
        const uint32_t ctas = ((rows + cand - 1u) / cand) * ncol;
        const uint32_t cost = cand == 128u ? (ctas <= sms ? 256u : ((ctas + 2u * sms - 1u) / (2u * sms)) * 512u)
                                           : ((ctas + sms - 1u) / sms) * (cand + 128u);
        if (cost < best) best = cost, bm = cand;
    }
    CUtensorMap map_a, map_b;
    if (!make_a_map(&map_a, x, rows, in, bm == 128u ? 128u : 256u)) return cudaErrorNotSupported;
    if (!make_a_map(&map_b, w_std_t, out, in, kBN)) return cudaErrorNotSupported;
    GemmArgs g = {};
    g.K = in;
    g.N = out;
    g.ops = 1;
    g.dense_rows = rows;
    g.y = y;
    g.y_dt = dt;
    g.ab_bf16 = dt == (int)kBf16;
    g.err = err;
    const uint32_t tiles = (rows + bm - 1u) / bm;
    return bm == 512u   ? launch_gemm_resident<512>(map_a, map_b, g, tiles, stream)
           : bm == 256u ? launch_gemm_resident<256>(map_a, map_b, g, tiles, stream)
                        : launch_gemm_resident<128>(map_a, map_b, g, tiles, stream);
}

// ---- routed experts, more than 32 rows --------------------------------------------------------------------------------

namespace {
struct MoeWs {
    uint32_t *counts, *cursor, *order, *inv;
    TileTables tiles;
    __half *xp, *zgu, *hd, *zd;
    size_t total;
};
MoeWs carve_moe(uint8_t* base, size_t slots, uint32_t experts, uint32_t hidden, uint32_t inter) {
    MoeWs w;
    size_t off = 0;
    auto take = [&](size_t bytes) {
        uint8_t* p = base ? base + off : nullptr;
        off += up256(bytes);
        return p;
    };
    // the most tiles of each height any routing gives: a 512-row tile holds more than 384 rows, an expert has at most one
    // 256-row tile (more than 128 rows in it and whatever follows) and one 128-row tile
    // Calls that average under 96 rows an expert keep to 128-row tiles (most experts fit one, and three launches a GEMM
    // with two nearly empty cost more than the few second decodes they save): a function of the call's shape only.
    w.tiles.uniform = slots < (size_t)96u * experts;
    w.tiles.max[0] = w.tiles.uniform ? 0u : (uint32_t)(slots / 385u) + 1u;
    w.tiles.max[1] = w.tiles.uniform ? 0u : (uint32_t)(slots / 129u + 1u < experts ? slots / 129u + 1u : experts);
    w.tiles.max[2] = w.tiles.uniform ? (uint32_t)(slots / 128u) + experts : (uint32_t)(slots < experts ? slots : experts);
    w.counts = reinterpret_cast<uint32_t*>(take((size_t)experts * 4u));
    w.cursor = reinterpret_cast<uint32_t*>(take((size_t)experts * 4u));
    w.order = reinterpret_cast<uint32_t*>(take(slots * 4u));
    w.inv = reinterpret_cast<uint32_t*>(take(slots * 4u));
    for (int k = 0; k < 3; ++k) w.tiles.t[k] = reinterpret_cast<int4*>(take((size_t)w.tiles.max[k] * 16u));
    w.xp = reinterpret_cast<__half*>(take(2u * slots * hidden * 2u));
    w.zgu = reinterpret_cast<__half*>(take(2u * slots * inter * 2u));
    w.hd = reinterpret_cast<__half*>(take(slots * inter * 2u));
    w.zd = reinterpret_cast<__half*>(take(slots * hidden * 2u));
    w.total = off;
    return w;
}

// one routed GEMM: a launch a tile height, tallest first
cudaError_t launch_routed_gemm(const void* a_base, uint64_t a_rows, GemmArgs g, const TileTables& tt, int codebook,
                               cudaStream_t stream) {
    CUtensorMap map128, map256;
    if (!make_a_map(&map128, a_base, a_rows, g.K, 128u) || !make_a_map(&map256, a_base, a_rows, g.K, 256u))
        return cudaErrorNotSupported;
    static const uint32_t heights[3] = {512u, 256u, 128u};
    for (int k = 0; k < 3; ++k) {
        if (tt.max[k] == 0u) continue;
        g.tiles = tt.t[k];
        const cudaError_t rc = launch_gemm(k == 2 ? map128 : map256, g, tt.max[k], heights[k], codebook, stream, true);
        if (rc != cudaSuccess) return rc;
    }
    return cudaSuccess;
}
}  // namespace

size_t prefill_moe_workspace(size_t rows, uint32_t topk, uint32_t experts, uint32_t hidden, uint32_t inter) {
    return carve_moe(nullptr, rows * topk, experts, hidden, inter).total;
}

cudaError_t launch_prefill_moe(const MoeArgs& a, void* workspace, int codebook, cudaStream_t stream, int* launches) {
    const size_t slots = (size_t)a.rows * a.topk;
    const uint32_t S = (uint32_t)slots, H = a.hidden, I = a.inter;
    MoeWs w = carve_moe(static_cast<uint8_t*>(workspace), slots, a.experts, H, I);
    const uint32_t* inds = static_cast<const uint32_t*>(a.inds);
    cudaError_t rc = cudaMemsetAsync(w.counts, 0, (size_t)a.experts * 4u, stream);
    if (rc != cudaSuccess) return rc;
    route_count_kernel<<<(S + 255u) / 256u, 256, 0, stream>>>(inds, S, a.experts, w.counts);
    route_plan_kernel<<<1, 1024, 0, stream>>>(w.counts, a.experts, w.cursor, w.tiles);
    route_scatter_kernel<<<(S + 255u) / 256u, 256, 0, stream>>>(inds, S, a.experts, w.cursor, w.order, w.inv);

    PrepArgs pa = {};
    pa.x = a.x;
    pa.x_dt = a.x_dt;
    pa.suh[0] = static_cast<const __half*>(a.gate_suh);
    pa.suh[1] = static_cast<const __half*>(a.up_suh);
    pa.K = H;
    pa.positions = S;
    pa.topk = a.topk;
    pa.experts = a.experts;
    pa.order = w.order;
    pa.inds = inds;
    pa.row_map = a.row_map;
    pa.xp = w.xp;
    pa.ops = 2;
    prep_rows_kernel<<<dim3(spread(S, H / 128u), (S + kRowsPerCta - 1u) / kRowsPerCta), 256, 0, stream>>>(pa);

    const uint32_t tile_bytes = 2u * a.n;
    GemmArgs g = {};
    g.trellis[0] = a.gate_t;
    g.trellis[1] = a.up_t;
    g.expert_bytes = (size_t)(H / 16u) * (I / 16u) * tile_bytes;
    g.K = H;
    g.N = I;
    g.n = a.n;
    g.mask = a.mask;
    g.ops = 2;
    g.a_op_rows = S;
    g.z = w.zgu;
    g.z_op_stride = slots * I;
    g.svh[0] = static_cast<const __half*>(a.gate_svh);  // the epilogue finishes gate and up with the tile's expert's scales
    g.svh[1] = static_cast<const __half*>(a.up_svh);
    g.svh_stride = I;
    g.err = a.err;
    rc = launch_routed_gemm(w.xp, 2u * slots, g, w.tiles, codebook, stream);
    if (rc != cudaSuccess) return rc;

    MidArgs m = {w.zgu, static_cast<const __half*>(a.down_suh), w.order, inds, S, I, a.experts, a.limit, a.clamp_at, w.hd};
    mid_kernel<<<dim3(spread(S, I / 128u), (S + kRowsPerCta - 1u) / kRowsPerCta), 256, 0, stream>>>(m);

    GemmArgs d = {};
    d.trellis[0] = d.trellis[1] = a.down_t;
    d.expert_bytes = g.expert_bytes;
    d.K = I;
    d.N = H;
    d.n = a.n;
    d.mask = a.mask;
    d.ops = 1;
    d.z = w.zd;
    d.svh[0] = d.svh[1] = static_cast<const __half*>(a.down_svh);  // each slot's finished down output, the per-slot v
    d.svh_stride = H;
    d.err = a.err;
    rc = launch_routed_gemm(w.hd, slots, d, w.tiles, codebook, stream);
    if (rc != cudaSuccess) return rc;

    FinArgs f = {w.zd, w.inv, a.scores, a.score_dt, a.shared, a.y, a.y_dt, a.rows, H, a.topk};
    if (a.shared_ready) {  // only this launch reads `shared`
        rc = cudaStreamWaitEvent(stream, static_cast<cudaEvent_t>(a.shared_ready), 0);
        if (rc != cudaSuccess) return rc;
    }
    const uint32_t fin_groups = (a.rows + 7u) / 8u, fin_want = (1184u + fin_groups - 1u) / fin_groups;
    moe_fin_kernel<<<dim3(fin_want < H / 128u ? fin_want : H / 128u, fin_groups), 256, 0, stream>>>(f);
    *launches += w.tiles.uniform ? 8 : 12;
    return cudaGetLastError();
}

}  // namespace t3
