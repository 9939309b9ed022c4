// The per-lane trellis reader and the two codebooks, as the sm_100a kernels use them.
//
// A 256-weight tile is n halfwords (n even, 16..128); weight t's codeword is the 16-bit window of the tile's circular
// bitstream that ends at bit ((t + 1) n) >> 4 (turboexl3 src/core/format.zig:116-118, 182-200); stream bit j is bit
// 31 - (j % 32) of little-endian uint32 word j / 32 (format.zig:204-209). Lane L of a warp owns code positions
// 8L .. 8L+7, which format.tensorCorePerm (format.zig:237-256) places at tile rows 2(L%4)+{0,1,8,9}, column L/4
// (positions 0-3) and L/4+8 (positions 4-7): exactly the B fragment of mma.sync.m16n8k16 for the tile's two n8 halves.
//
// Because 8L n / 16 = L n/2 is whole, window m of lane L ends at bit L n/2 + d(m), d(m) = ((m + 1) n) >> 4, so the
// eight windows sit at lane-independent offsets p(m) = d(m) - d(0) inside the lane's span, which starts at bit
// L n/2 + d(0) - 16. The reader loads the span's raw words, shifts them once so the span starts at a word's top bit
// (skipped when n % 64 == 0, where every lane's shift is the same constant), and then every window is one constant
// shift and one mask. (The reference derives a per-lane plan with lane-dependent word selects instead:
// src/core/lane.zig:32-49, src/kernels/hip/lane.hpp:25-68.)
//
// Everything here is __host__ __device__ so that a CPU harness can replay the exact index arithmetic lane by lane.
#pragma once

#include <stdint.h>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#define T3_HD __host__ __device__ __forceinline__
#else
#define T3_HD inline
#endif

namespace t3 {

enum Codebook : int { kMul1 = 0, kMcg = 1 };  // format.zig:18-21

constexpr uint32_t kMul1Mult = 0x83DCD12Du;  // format.zig:16
constexpr uint32_t kMcgMult = 0xCBAC1FEDu;   // format.zig:15

// ---- small portable intrinsics ------------------------------------------------------------------------------------

// high word of (hi:lo) << s, s in [0, 31]
T3_HD uint32_t shl_pair(uint32_t hi, uint32_t lo, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_l(lo, hi, s);
#else
    return s == 0 ? hi : ((hi << s) | (lo >> (32u - s)));
#endif
}

// low word of (hi:lo) >> s, s in [0, 31]
T3_HD uint32_t shr_pair(uint32_t hi, uint32_t lo, uint32_t s) {
#if defined(__CUDA_ARCH__)
    return __funnelshift_r(lo, hi, s);
#else
    return s == 0 ? lo : ((lo >> s) | (hi << (32u - s)));
#endif
}

// c + the sum of v's four bytes
T3_HD uint32_t byte_sum_add(uint32_t v, uint32_t c) {
#if defined(__CUDA_ARCH__)
    return __dp4a(v, 0x01010101u, c);
#else
    return c + (v & 0xFFu) + ((v >> 8) & 0xFFu) + ((v >> 16) & 0xFFu) + (v >> 24);
#endif
}

// (b.lo16 << 16) | a.lo16
T3_HD uint32_t pack_lo(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, 0x5410);
#else
    return (a & 0xFFFFu) | (b << 16);
#endif
}

// (b.hi16 << 16) | a.hi16
T3_HD uint32_t pack_hi(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, 0x7632);
#else
    return (a >> 16) | (b & 0xFFFF0000u);
#endif
}

#if !defined(__CUDA_ARCH__)
namespace hostfp {
inline double h2d(uint16_t b) {
    _Float16 h;
    __builtin_memcpy(&h, &b, 2);
    return (double)h;
}
inline uint16_t d2h(double v) {  // one rounding, nearest even
    _Float16 h = (_Float16)v;
    uint16_t b;
    __builtin_memcpy(&b, &h, 2);
    return b;
}
}  // namespace hostfp
#endif

// two half-precision fused multiply-adds, a * b + c per 16-bit half, one rounding each
T3_HD uint32_t hfma2_bits(uint32_t a, uint32_t b, uint32_t c) {
#if defined(__CUDA_ARCH__)
    uint32_t d;
    asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
#else
    using namespace hostfp;  // operands have 11 significant bits each, so the double expression is exact
    const uint16_t lo = d2h(h2d((uint16_t)a) * h2d((uint16_t)b) + h2d((uint16_t)c));
    const uint16_t hi = d2h(h2d((uint16_t)(a >> 16)) * h2d((uint16_t)(b >> 16)) + h2d((uint16_t)(c >> 16)));
    return (uint32_t)lo | ((uint32_t)hi << 16);
#endif
}

// two half-precision adds
T3_HD uint32_t hadd2_bits(uint32_t a, uint32_t b) {
#if defined(__CUDA_ARCH__)
    uint32_t d;
    asm("add.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
#else
    using namespace hostfp;
    const uint16_t lo = d2h(h2d((uint16_t)a) + h2d((uint16_t)b));
    const uint16_t hi = d2h(h2d((uint16_t)(a >> 16)) + h2d((uint16_t)(b >> 16)));
    return (uint32_t)lo | ((uint32_t)hi << 16);
#endif
}

// ---- the codebooks: two codewords to one half2 ---------------------------------------------------------------------

// MUL1 (format.zig:158-167): t = byte sum of cw * 0x83DCD12D; w = f16(fma_f32(f16(0x6400 + t), f16(0x1EEE),
// f16(0xC931))). The f16 bit pattern 0x6400 + t IS 1024 + t, and the f32 fma is exact for every t (20 significant
// bits at most), so one half-precision fma rounds to the same bits (checked over every t by the CPU tests and over all
// 65,536 codewords by the GPU tests).
T3_HD uint32_t decode2_mul1(uint32_t cw0, uint32_t cw1) {
    const uint32_t h0 = byte_sum_add(cw0 * kMul1Mult, 0x6400u);
    const uint32_t h1 = byte_sum_add(cw1 * kMul1Mult, 0x6400u);
    return hfma2_bits(pack_lo(h0, h1), 0x1EEE1EEEu, 0xC931C931u);
}

// MCG (format.zig:149-155): pair = 0x3B603B60 ^ (cw * 0xCBAC1FED & 0x8FFF8FFF); w = f16(f32(lo) + f32(hi)). Both halves
// are normal f16 values within a factor 16 of each other, so the f32 sum is exact and one half-precision add rounds to
// the same bits.
T3_HD uint32_t decode2_mcg(uint32_t cw0, uint32_t cw1) {
    const uint32_t p0 = 0x3B603B60u ^ ((cw0 * kMcgMult) & 0x8FFF8FFFu);
    const uint32_t p1 = 0x3B603B60u ^ ((cw1 * kMcgMult) & 0x8FFF8FFFu);
    return hadd2_bits(pack_lo(p0, p1), pack_hi(p0, p1));
}

// Timing probes (never a served kernel; the reference's Geometry.probe, src/core/decode.zig:34-35): a "codebook" past the
// two real ones. kProbeNoHash skips the codebook hash (the codewords go to the tensor cores as they are), kProbeNoFunnel
// skips the window extraction too (the raw words go), kProbeStream leaves the stage as soon as it has landed.
constexpr int kProbeNoHash = 2, kProbeNoFunnel = 3, kProbeStream = 4;

template <int CB>
T3_HD uint32_t decode2(uint32_t cw0, uint32_t cw1) {
    if (CB >= kProbeNoHash) return cw0 | (cw1 << 16);
    if (CB == kMcg) return decode2_mcg(cw0, cw1);
    return decode2_mul1(cw0, cw1);
}

// ---- the lane plan -------------------------------------------------------------------------------------------------

// d(m): window m's end bit past L n/2
constexpr uint32_t win_end(uint32_t n, uint32_t m) { return ((m + 1u) * n) >> 4; }
// bits from the first window's first bit to the last window's last bit
constexpr uint32_t span_bits(uint32_t n) { return win_end(n, 7) - win_end(n, 0) + 16u; }
// whether every lane's span starts at the same bit of a word
constexpr bool uniform_shift(uint32_t n) { return n % 64u == 0u; }
// the lane's span start, one stream period added so it is never negative
T3_HD uint32_t span_start(uint32_t n, uint32_t lane) { return lane * (n >> 1) + win_end(n, 0) + 16u * n - 16u; }
// the largest in-word bit offset a lane's span starts at
constexpr uint32_t max_shift(uint32_t n) {
    uint32_t mx = 0;
    for (uint32_t l = 0; l < 32u; ++l) {
        const uint32_t o = (l * (n >> 1) + win_end(n, 0) + 16u * n - 16u) & 31u;
        mx = o > mx ? o : mx;
    }
    return mx;
}
constexpr uint32_t raw_words(uint32_t n) { return (max_shift(n) + span_bits(n) + 31u) / 32u; }      // 1..4
constexpr uint32_t aligned_words(uint32_t n) { return (span_bits(n) + 31u) / 32u; }                // 1..3

// What a lane needs to know about itself for rate N (loop-invariant: compute once per kernel).
template <int N>
struct LanePlan {
    static constexpr uint32_t kRaw = raw_words(N);
    uint32_t idx[kRaw];  // word indices into the tile (0 .. N/2 - 1), circular
    uint32_t shift;      // bit offset of the span inside word idx[0]

    T3_HD void init(uint32_t lane) {
        const uint32_t s = span_start(N, lane);
        const uint32_t hw = N / 2u;
        uint32_t w = s >> 5;  // in [hw - 1, 2 hw)
        w = w >= hw ? w - hw : w;
        shift = s & 31u;
#pragma unroll
        for (uint32_t i = 0; i < kRaw; ++i) {
            idx[i] = w;
            w = (w + 1u == hw) ? 0u : w + 1u;
        }
    }
};

// The 16-bit window that starts `pos` bits into the word array w (bit 0 = w[0]'s top bit), masked. `pos` is a
// compile-time constant wherever this is called from decode_lane, so the word picks and shifts fold.
template <uint32_t NW>
T3_HD uint32_t window_at(const uint32_t (&w)[NW], uint32_t pos, uint32_t mask) {
    const uint32_t q = pos >> 5, b = pos & 31u;
    if (b <= 16u) return (w[q] >> (16u - b)) & mask;
    return shr_pair(w[q], w[q + 1 < NW ? q + 1 : q], 48u - b) & mask;
}

// The lane's raw words of one tile (`tile` points at the tile's first word, shared or global memory).
template <int N>
T3_HD void load_lane(const uint32_t* tile, const LanePlan<N>& plan, uint32_t (&raw)[raw_words(N)]) {
#pragma unroll
    for (uint32_t i = 0; i < raw_words(N); ++i) raw[i] = tile[plan.idx[i]];
}

// The lane's eight weights from its raw words as four half2 words: {w0,w1}, {w2,w3}, {w4,w5}, {w6,w7}; b[0], b[1] are
// the mma.m16n8k16 B fragment of tile columns 0-7, b[2], b[3] of columns 8-15. `mask` is the pack's codeword-width mask
// (format.zig:60-62).
template <int N, int CB>
T3_HD void decode_raw(const uint32_t (&raw)[raw_words(N)], const LanePlan<N>& plan, uint32_t mask, uint32_t (&b)[4]) {
    constexpr uint32_t kRaw = raw_words(N);
    if (CB >= kProbeNoFunnel) {
#pragma unroll
        for (uint32_t j = 0; j < 4u; ++j) b[j] = raw[j < kRaw ? j : kRaw - 1u];
        return;
    }
    uint32_t cw[8];
    if (uniform_shift(N)) {
        constexpr uint32_t o = (win_end(N, 0) + 16u * N - 16u) & 31u;
#pragma unroll
        for (uint32_t m = 0; m < 8u; ++m) cw[m] = window_at<kRaw>(raw, o + win_end(N, m) - win_end(N, 0), mask);
    } else {
        constexpr uint32_t kAl = aligned_words(N);
        uint32_t al[kAl];
#pragma unroll
        for (uint32_t i = 0; i < kAl; ++i) al[i] = shl_pair(raw[i], raw[i + 1 < kRaw ? i + 1 : i], plan.shift);
#pragma unroll
        for (uint32_t m = 0; m < 8u; ++m) cw[m] = window_at<kAl>(al, win_end(N, m) - win_end(N, 0), mask);
    }
#pragma unroll
    for (uint32_t j = 0; j < 4u; ++j) b[j] = decode2<CB>(cw[2 * j], cw[2 * j + 1]);
}

// load_lane + decode_raw
template <int N, int CB>
T3_HD void decode_lane(const uint32_t* tile, const LanePlan<N>& plan, uint32_t mask, uint32_t (&b)[4]) {
    uint32_t raw[raw_words(N)];
    load_lane<N>(tile, plan, raw);
    decode_raw<N, CB>(raw, plan, mask, b);
}

// The same for a rate known only at run time (any even n in [16, 128]): the plain per-window read, two words a window.
// Slow; the integer rates take the templated reader.
template <int CB>
T3_HD void decode_lane_any(const uint32_t* tile, uint32_t n, uint32_t lane, uint32_t mask, uint32_t (&b)[4]) {
    const uint32_t hw = n >> 1;
    uint32_t cw[8];
#pragma unroll
    for (uint32_t m = 0; m < 8u; ++m) {
        const uint32_t end = lane * hw + (((m + 1u) * n) >> 4) + 16u * n;  // one period added
        uint32_t q = (end - 1u) >> 5;                                       // the word holding the window's last bit
        const uint32_t sh = 32u * (q + 1u) - end;                           // 0..31
        q = q % hw;
        const uint32_t lo = tile[q];
        const uint32_t hi = tile[q == 0u ? hw - 1u : q - 1u];
        cw[m] = shr_pair(hi, lo, sh) & mask;
    }
#pragma unroll
    for (uint32_t j = 0; j < 4u; ++j) b[j] = decode2<CB>(cw[2 * j], cw[2 * j + 1]);
}

// Where lane L's weight m (0..7) sits in the 16x16 tile (format.zig:237-256)
T3_HD uint32_t tile_row(uint32_t lane, uint32_t m) { return 2u * (lane & 3u) + (m & 1u) + ((m & 2u) ? 8u : 0u); }
T3_HD uint32_t tile_col(uint32_t lane, uint32_t m) { return (lane >> 2) + ((m & 4u) ? 8u : 0u); }

// The slot of input element r (0..15) of a 16-group in "lane order": the quad's four rows 2q, 2q+1, 2q+8, 2q+9 become
// one 8-byte load (the reference's order: src/kernels/hip/common.hpp:70-75).
T3_HD uint32_t lane_order16(uint32_t r) { return 4u * ((r & 7u) >> 1) + ((r & 1u) | ((r >> 3) << 1)); }

}  // namespace t3
