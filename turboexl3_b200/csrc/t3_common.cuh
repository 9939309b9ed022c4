// Device helpers shared by every kernel group: activation loads and stores, the 128-point Hadamard on a warp, the
// warp-level tensor-core step, and the mbarrier / bulk-copy plumbing with bounded waits.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "t3_lane.cuh"

namespace t3 {

// activation dtypes, numbered as the reference's kernels number them (src/kernels/hip/common.hpp:21)
enum Dtype : int { kF32 = 0, kF16 = 1, kBf16 = 2 };

constexpr float kHadScale = 0.08838834764831845f;  // 1 / sqrt(128), format.zig:14

// bits of the device error word (see t3.h: t3_device_error)
enum DevError : uint32_t {
    kErrFullWait = 1u,    // a consumer gave up waiting for a bulk copy to land
    kErrEmptyWait = 2u,   // the producer gave up waiting for a ring slot
    kErrMmaWait = 4u,     // a tensor-core completion never arrived
    kErrTmemAlloc = 8u,   // tensor memory could not be allocated
};

__device__ __forceinline__ float round_half(float v) { return __half2float(__float2half_rn(v)); }

// element i of an activation array as f32
__device__ __forceinline__ float load_act(const void* p, int dt, size_t i) {
    if (dt == kF32) return static_cast<const float*>(p)[i];
    if (dt == kF16) return __half2float(static_cast<const __half*>(p)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

// v into element i of an array of dtype dt (round to nearest even)
__device__ __forceinline__ void store_act(void* p, int dt, size_t i, float v) {
    if (dt == kF32) static_cast<float*>(p)[i] = v;
    else if (dt == kF16) static_cast<__half*>(p)[i] = __float2half_rn(v);
    else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

// Unscaled Walsh-Hadamard of a 128-block spread over a warp: lane L holds elements L + 32 j in v[j]. Index bits 0-4
// are butterflies across lanes, bits 5-6 inside the lane. (format.hadamard128, format.zig:265-273, is the dense
// 128x128 sum this equals up to f32 summation order.)
__device__ __forceinline__ void h128_warp(float (&v)[4], uint32_t lane) {
#pragma unroll
    for (uint32_t bit = 1; bit < 32u; bit <<= 1) {
        const bool upper = (lane & bit) != 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xFFFFFFFFu, v[j], bit);
            v[j] = upper ? other - v[j] : v[j] + other;
        }
    }
    const float s01 = v[0] + v[1], d01 = v[0] - v[1], s23 = v[2] + v[3], d23 = v[2] - v[3];
    v[0] = s01 + s23;
    v[1] = d01 + d23;
    v[2] = s01 - s23;
    v[3] = d01 - d23;
}

// The same transform for a lane that holds four CONSECUTIVE elements 4 L .. 4 L + 3 (so a warp's loads and stores of a
// 128-block are one contiguous 256- or 512-byte run): index bits 0-1 inside the lane, bits 2-6 across lanes.
__device__ __forceinline__ void h128_warp_v4(float (&v)[4], uint32_t lane) {
    const float s01 = v[0] + v[1], d01 = v[0] - v[1], s23 = v[2] + v[3], d23 = v[2] - v[3];
    v[0] = s01 + s23;
    v[1] = d01 + d23;
    v[2] = s01 - s23;
    v[3] = d01 - d23;
#pragma unroll
    for (uint32_t bit = 1; bit < 32u; bit <<= 1) {
        const bool upper = (lane & bit) != 0u;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float other = __shfl_xor_sync(0xFFFFFFFFu, v[j], bit);
            v[j] = upper ? other - v[j] : v[j] + other;
        }
    }
}

// four consecutive elements i .. i + 3 (i a multiple of 4) of an activation array as f32, one vector load
__device__ __forceinline__ void load_act4(const void* p, int dt, size_t i, float (&v)[4]) {
    if (dt == kF32) {
        const float4 f = *reinterpret_cast<const float4*>(static_cast<const float*>(p) + i);
        v[0] = f.x, v[1] = f.y, v[2] = f.z, v[3] = f.w;
    } else {
        const uint2 u = *reinterpret_cast<const uint2*>(static_cast<const uint16_t*>(p) + i);
        if (dt == kF16) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
            v[0] = a.x, v[1] = a.y, v[2] = b.x, v[3] = b.y;
        } else {
            v[0] = __uint_as_float(u.x << 16), v[1] = __uint_as_float(u.x & 0xFFFF0000u);
            v[2] = __uint_as_float(u.y << 16), v[3] = __uint_as_float(u.y & 0xFFFF0000u);
        }
    }
}

__device__ __forceinline__ void load_half4(const __half* p, float (&v)[4]) { load_act4(p, kF16, 0, v); }

// four consecutive elements stored in dtype dt (round to nearest even), one vector store
__device__ __forceinline__ void store_act4(void* p, int dt, size_t i, const float (&v)[4]) {
    if (dt == kF32) {
        *reinterpret_cast<float4*>(static_cast<float*>(p) + i) = make_float4(v[0], v[1], v[2], v[3]);
    } else if (dt == kF16) {
        const __half2 a = __floats2half2_rn(v[0], v[1]), b = __floats2half2_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(static_cast<__half*>(p) + i) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    } else {
        const __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(p) + i) =
            make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
    }
}

// D += A (16x16, row) * B (16x8, col), f16 operands, f32 accumulate
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---- the 128-point Hadamard on tensor cores (the prefill-row prepares and finishes) ---------------------------------
//
// The 128-point Hadamards of these kernels run on the tensor cores. The sign of entry (i, j) of H128 is the parity of
// popcount(i & j), which splits over the bit fields of i = 16 i8 + i16, so H128 = H8 (x) H16 and a block viewed as an
// 8 x 16 matrix X becomes H8 . X . H16: X . H16 is m16n8k16 steps against a constant +-1 fragment, H8 a three-level
// butterfly over values one thread already holds. A warp works on EIGHT positions at a time, one 128-block each: quad g
// (lanes 4g .. 4g + 3) owns position g, and lane q of the quad holds, for every i8, the four elements 16 i8 + 4q .. + 3:
// one 8-byte (f16) or 16-byte (f32) access per i8 on the way in and on the way out. The butterfly on a warp costs twenty
// shuffles per block, and the shuffle unit (one warp instruction per SM per cycle) bounded these kernels; this form has none.
// f32 accumulation of +-1 products is exact per term, so the result differs from the butterfly (and from the oracle's
// dense sum) only in summation order, as before.

struct HadB {
    uint32_t b[2][2];  // the +-1 H16 fragment of each 8-column half (t): {k 0-7 part, k 8-15 part}
};

// Matrix index <-> element maps (both free to choose): A/B index k of thread q covers elements 4q, 4q+1 (k = 2q, 2q+1) and
// 4q+2, 4q+3 (k = 2q+8, 2q+9); output column n = 2q+b of half t is element 4q + 2t + b. So a thread's inputs and outputs
// are the same four consecutive elements.
__device__ __forceinline__ HadB had_b(uint32_t lane) {
    const uint32_t g = lane >> 2, q = lane & 3u;
    HadB h;
#pragma unroll
    for (uint32_t t = 0; t < 2u; ++t) {
        const uint32_t en = 4u * (g >> 1) + 2u * t + (g & 1u);
        uint32_t s[4];
#pragma unroll
        for (uint32_t b = 0; b < 4u; ++b) s[b] = (__popc((4u * q + b) & en) & 1) ? 0xBC00u : 0x3C00u;
        h.b[t][0] = s[0] | (s[1] << 16);
        h.b[t][1] = s[2] | (s[3] << 16);
    }
    return h;
}

// out[i8][e] = sum over the block of sign * value, for the position this quad owns. a[i8] = the four f16 values
// {16 i8 + 4q .. + 3} as two packed pairs; a second set (the f16 remainders of values that are not f16 themselves) is
// accumulated into the same sums when `use_lo` is set.
__device__ __forceinline__ void h128_mma(const uint32_t (&a)[8][2], const uint32_t (&lo)[8][2], bool use_lo,
                                         const HadB& hb, float (&out)[8][4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int t = 0; t < 2; ++t) {
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            mma16816(c, a[2 * j][0], a[2 * j + 1][0], a[2 * j][1], a[2 * j + 1][1], hb.b[t][0], hb.b[t][1]);
            if (use_lo) mma16816(c, lo[2 * j][0], lo[2 * j + 1][0], lo[2 * j][1], lo[2 * j + 1][1], hb.b[t][0], hb.b[t][1]);
            out[2 * j][2 * t] = c[0], out[2 * j][2 * t + 1] = c[1];
            out[2 * j + 1][2 * t] = c[2], out[2 * j + 1][2 * t + 1] = c[3];
        }
#pragma unroll
    for (int bit = 1; bit < 8; bit <<= 1)
#pragma unroll
        for (int i = 0; i < 8; ++i)
            if (!(i & bit))
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float lo_v = out[i][e], hi_v = out[i | bit][e];
                    out[i][e] = lo_v + hi_v;
                    out[i | bit][e] = lo_v - hi_v;
                }
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

// v (f32 values, not necessarily f16) as an f16 part and the f16 of what is left; returns nonzero when any remainder is
__device__ __forceinline__ uint32_t split4(const float (&v)[4], uint32_t (&hi)[2], uint32_t (&lo)[2]) {
    float r[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) r[j] = v[j] - round_half(v[j]);
    hi[0] = pack_half2(v[0], v[1]), hi[1] = pack_half2(v[2], v[3]);
    lo[0] = pack_half2(r[0], r[1]), lo[1] = pack_half2(r[2], r[3]);
    return (lo[0] | lo[1]) & 0x7FFF7FFFu;
}

// H128 of the block whose values are `v` (v[i8] = elements 16 i8 + 4q .. + 3), any f32 values. `unit_scales`: the caller
// knows (for the whole warp) that every v is an f16 value times +-1 — sign vectors, the usual suh — so v is an f16 value
// itself and there are no remainders to compute.
__device__ __forceinline__ void h128_split(const float (&v)[8][4], bool unit_scales, const HadB& hb, float (&out)[8][4]) {
    uint32_t hi[8][2], lo[8][2], rest = 0;
    if (unit_scales) {
#pragma unroll
        for (int i = 0; i < 8; ++i) hi[i][0] = pack_half2(v[i][0], v[i][1]), hi[i][1] = pack_half2(v[i][2], v[i][3]);
        h128_mma(hi, hi, false, hb, out);
        return;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) rest |= split4(v[i], hi[i], lo[i]);
    h128_mma(hi, lo, __any_sync(0xFFFFFFFFu, rest != 0u) != 0, hb, out);
}

// whether four scales are all +1 or -1 (as f32 values converted from f16)
__device__ __forceinline__ bool all_unit(const float (&sc)[4]) {
    return fabsf(sc[0]) == 1.0f && fabsf(sc[1]) == 1.0f && fabsf(sc[2]) == 1.0f && fabsf(sc[3]) == 1.0f;
}

// ---- shared-memory barriers and bulk copies ------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

// makes freshly initialised barriers visible to the copy engine and to the cluster
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

// Waits for the barrier's phase of the given parity: one plain poll, then at most kSleepPolls polls that each sleep in
// the hardware for up to kSleepHintNs. Returns false after giving up; the caller records the error and carries on to
// its exit path, so a lost copy never hangs the device. (kSpinLimit bounds the polling loops that do not sleep.)
constexpr uint32_t kSpinLimit = 1u << 20;
__device__ __forceinline__ uint32_t mbar_try(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done;
}
// whether the phase has completed, without waiting at all
__device__ __forceinline__ uint32_t mbar_test(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done;
}
// The slow path sleeps inside try_wait (the hardware suspends the thread until the phase completes or the hint, in
// nanoseconds, runs out) instead of spinning: a waiting warp takes no issue slots from the warps that have work.
constexpr uint32_t kSleepPolls = 1u << 18;
constexpr uint32_t kSleepHintNs = 4000;
constexpr uint32_t kEagerPolls = 64;
static __device__ __noinline__ bool mbar_wait_slow(uint32_t addr, uint32_t parity) {
    for (uint32_t i = 0; i < kEagerPolls; ++i)
        if (mbar_try(addr, parity)) return true;
    for (uint32_t i = 0; i < kSleepPolls; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(kSleepHintNs)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ bool mbar_wait_addr(uint32_t addr, uint32_t parity) {
    if (mbar_try(addr, parity)) return true;  // the common case costs one poll and no loop
    return mbar_wait_slow(addr, parity);
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) { return mbar_wait_addr(smem_addr(bar), parity); }

// The same wait with the failure recorded in place (no call in the caller's hot loop: a call there makes the compiler
// keep its registers ready for one): on giving up, `bit` is or-ed into the device error word and the caller carries on.
__device__ __forceinline__ void mbar_wait_report(uint32_t addr, uint32_t parity, uint32_t* err, uint32_t bit) {
#pragma unroll 1
    for (uint32_t i = 0; i < kEagerPolls; ++i)  // a short wait is answered at once; only a long one goes to sleep
        if (mbar_try(addr, parity)) return;
#pragma unroll 1
    for (uint32_t i = 0; i < kSleepPolls; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(kSleepHintNs)
            : "memory");
        if (done) return;
    }
    if (err) atomicOr(err, bit);
}

__device__ __forceinline__ void mbar_arrive_addr(uint32_t addr) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(addr) : "memory");
}

// `bytes` (a multiple of 16) from 16-byte-aligned global memory to 16-byte-aligned shared memory of this CTA; completion
// is counted on `bar`. No multicast.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// a named barrier over `threads` threads of the CTA (id 1..15; 0 is __syncthreads')
__device__ __forceinline__ void named_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// asks L2 for `bytes` starting at p (lanes 0 .. bytes / 128 of the calling warp, one 128-byte line each): for small
// weight-side vectors whose first use sits behind a wait, so that the use finds them in L2 and not in DRAM
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes, uint32_t lane) {
    if (lane * 128u < bytes) asm volatile("prefetch.global.L2 [%0];" ::"l"(static_cast<const uint8_t*>(p) + lane * 128u));
}

static __device__ __noinline__ void report(uint32_t* err, uint32_t bit) {
    if (err) atomicOr(err, bit);
}

}  // namespace t3
