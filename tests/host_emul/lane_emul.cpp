// CPU replay of the kernels' per-lane trellis reader (turboexl3_b200/csrc/t3_lane.cuh) against the oracle's
// unpackTile / decodeTile, lane by lane. Built by tests/test_lane_host.py with g++; no GPU involved.
#include <cstdint>
#include <cstdio>
#include <cstring>

#include "../../oracle/t3_oracle.h"
#include "../../turboexl3_b200/csrc/t3_lane.cuh"

namespace {

uint64_t rng_state = 0x9E3779B97F4A7C15ull;
uint32_t next_u32() {
    rng_state += 0x9E3779B97F4A7C15ull;
    uint64_t z = rng_state;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return (uint32_t)((z ^ (z >> 31)) >> 16);
}

// the tile's 256 f16 weights in row-major order as the lane reader produces them
template <int N, int CB>
void tile_by_lanes(const uint32_t* words, uint32_t mask, uint16_t out[256]) {
    for (uint32_t lane = 0; lane < 32; ++lane) {
        t3::LanePlan<N> plan;
        plan.init(lane);
        uint32_t b[4];
        t3::decode_lane<N, CB>(words, plan, mask, b);
        for (uint32_t m = 0; m < 8; ++m) {
            const uint16_t v = (uint16_t)(b[m >> 1] >> ((m & 1) * 16));
            out[t3::tile_row(lane, m) * 16 + t3::tile_col(lane, m)] = v;
        }
    }
}

template <int CB>
void tile_by_lanes_any(const uint32_t* words, uint32_t n, uint32_t mask, uint16_t out[256]) {
    for (uint32_t lane = 0; lane < 32; ++lane) {
        uint32_t b[4];
        t3::decode_lane_any<CB>(words, n, lane, mask, b);
        for (uint32_t m = 0; m < 8; ++m)
            out[t3::tile_row(lane, m) * 16 + t3::tile_col(lane, m)] = (uint16_t)(b[m >> 1] >> ((m & 1) * 16));
    }
}

template <int N>
int check_rate(int trials) {
    int bad = 0;
    uint32_t words[64];
    uint16_t got[256], want[256];
    for (int t = 0; t < trials; ++t) {
        for (int i = 0; i < N / 2; ++i) words[i] = (next_u32() << 16) ^ next_u32();
        for (int wbits = 8; wbits <= 16; ++wbits) {
            const uint32_t mask = (1u << wbits) - 1u;
            for (int cb = 0; cb < 2; ++cb) {
                t3o_decode_tile((const uint16_t*)words, N, cb, wbits, want);
                if (cb == 0) tile_by_lanes<N, 0>(words, mask, got);
                else tile_by_lanes<N, 1>(words, mask, got);
                if (memcmp(got, want, sizeof got) != 0) ++bad;
                if (cb == 0) tile_by_lanes_any<0>(words, N, mask, got);
                else tile_by_lanes_any<1>(words, N, mask, got);
                if (memcmp(got, want, sizeof got) != 0) ++bad;
            }
        }
    }
    return bad;
}

}  // namespace

extern "C" int lane_emul_integer_rates(int trials) {
    return check_rate<16>(trials) + check_rate<32>(trials) + check_rate<48>(trials) + check_rate<64>(trials) +
           check_rate<80>(trials) + check_rate<96>(trials) + check_rate<112>(trials) + check_rate<128>(trials);
}

// templated reader at fractional rates too (it is written for any even n)
extern "C" int lane_emul_fractional_rates(int trials) {
    return check_rate<36>(trials) + check_rate<40>(trials) + check_rate<44>(trials) + check_rate<56>(trials) +
           check_rate<104>(trials) + check_rate<18>(trials) + check_rate<126>(trials);
}

// run-time reader at every even n
extern "C" int lane_emul_any_rate(int trials) {
    int bad = 0;
    uint32_t words[64];
    uint16_t got[256], want[256];
    for (uint32_t n = 16; n <= 128; n += 2)
        for (int t = 0; t < trials; ++t) {
            for (uint32_t i = 0; i < n / 2; ++i) words[i] = (next_u32() << 16) ^ next_u32();
            for (int cb = 0; cb < 2; ++cb) {
                t3o_decode_tile((const uint16_t*)words, n, cb, 16, want);
                if (cb == 0) tile_by_lanes_any<0>(words, n, 0xFFFFu, got);
                else tile_by_lanes_any<1>(words, n, 0xFFFFu, got);
                if (memcmp(got, want, sizeof got) != 0) ++bad;
            }
        }
    return bad;
}

// every codeword through the pair decoders against the oracle's scalar decoders
extern "C" int lane_emul_codebooks() {
    int bad = 0;
    for (uint32_t cw = 0; cw < 65536; cw += 2) {
        const uint32_t a = t3::decode2_mul1(cw, cw + 1), b = t3::decode2_mcg(cw, cw + 1);
        bad += (uint16_t)a != t3o_decode_mul1((uint16_t)cw);
        bad += (uint16_t)(a >> 16) != t3o_decode_mul1((uint16_t)(cw + 1));
        bad += (uint16_t)b != t3o_decode_mcg((uint16_t)cw);
        bad += (uint16_t)(b >> 16) != t3o_decode_mcg((uint16_t)(cw + 1));
    }
    return bad;
}

extern "C" int lane_emul_lane_order() {
    int bad = 0;
    bool seen[16] = {};
    for (uint32_t r = 0; r < 16; ++r) {
        const uint32_t s = t3::lane_order16(r);
        bad += s >= 16 || seen[s];
        seen[s] = true;
    }
    for (uint32_t q = 0; q < 4; ++q) {  // a quad's rows land in four consecutive slots, in fragment order
        bad += t3::lane_order16(2 * q) != 4 * q;
        bad += t3::lane_order16(2 * q + 1) != 4 * q + 1;
        bad += t3::lane_order16(2 * q + 8) != 4 * q + 2;
        bad += t3::lane_order16(2 * q + 9) != 4 * q + 3;
    }
    return bad;
}
