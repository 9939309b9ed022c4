/* CPU oracle of the EXL3 projection path (see t3_oracle.h for its role and its pins).
 * TEST INFRASTRUCTURE ONLY: never linked into, imported by or called from the shipped library.
 * Build: gcc -O2 -ffp-contract=off -fPIC -shared -pthread (oracle/Makefile). */
#include "t3_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------ scalars (format.zig:10-174) */

static const float kHadScale = 0.08838834764831845f; /* format.zig:14 */
static const uint32_t kMcgMult = 0xCBAC1FEDu;        /* format.zig:15 */
static const uint32_t kMul1Mult = 0x83DCD12Du;       /* format.zig:16 */

float t3o_had_scale(void) { return kHadScale; }

uint32_t t3o_multiplier(int codebook) { return codebook == T3O_MCG ? kMcgMult : kMul1Mult; }

int t3o_window_mask(int w) {
    if (w < 8 || w > 16) return -1;
    return (int)((1u << w) - 1u);
}

int t3o_rate_admitted(uint64_t n) { return (n % 2 == 0) && n >= 16 && n <= 128; }

uint64_t t3o_bit_end(uint32_t n, uint64_t t) { return ((t + 1) * (uint64_t)n) >> 4; }

uint64_t t3o_fresh_bits(uint32_t n, uint64_t t) {
    return t3o_bit_end(n, t) - (t == 0 ? 0 : t3o_bit_end(n, t - 1));
}

uint16_t t3o_f32_to_f16_bits(float v) {
    _Float16 h = (_Float16)v;
    uint16_t b;
    memcpy(&b, &h, 2);
    return b;
}

float t3o_f16_bits_to_f32(uint16_t bits) {
    _Float16 h;
    memcpy(&h, &bits, 2);
    return (float)h;
}

static inline float h2f(uint16_t b) { return t3o_f16_bits_to_f32(b); }
static inline uint16_t f2h(float v) { return t3o_f32_to_f16_bits(v); }
static inline float round_h(float v) { return h2f(f2h(v)); }

uint16_t t3o_decode_mcg(uint16_t cw) {
    const uint32_t mixed = (uint32_t)cw * kMcgMult;
    const uint32_t pair = 0x3B603B60u ^ (mixed & 0x8FFF8FFFu);
    return f2h(h2f((uint16_t)(pair & 0xFFFFu)) + h2f((uint16_t)(pair >> 16)));
}

uint32_t t3o_mul1_t(uint16_t cw) {
    const uint32_t mixed = (uint32_t)cw * kMul1Mult;
    return (mixed & 0xFFu) + ((mixed >> 8) & 0xFFu) + ((mixed >> 16) & 0xFFu) + (mixed >> 24);
}

uint16_t t3o_decode_mul1(uint16_t cw) {
    const float h = h2f((uint16_t)(0x6400u + t3o_mul1_t(cw)));
    return f2h(fmaf(h, h2f(0x1EEE), h2f(0xC931)));
}

uint16_t t3o_decode_codeword(uint16_t cw, int codebook) {
    return codebook == T3O_MCG ? t3o_decode_mcg(cw) : t3o_decode_mul1(cw);
}

/* ------------------------------------------------------------------ the bitstream (format.zig:176-256) */

static inline uint32_t word_u32(const uint16_t* hw, size_t i) {
    return (uint32_t)hw[2 * i] | ((uint32_t)hw[2 * i + 1] << 16);
}

void t3o_unpack_tile(const uint16_t* words, uint32_t n, uint16_t out[256]) {
    const size_t word_count = n / 2;
    const size_t total = (size_t)16 * n;
    for (size_t pair = 0; pair < 128; ++pair) {
        const size_t e0 = t3o_bit_end(n, 2 * pair);
        const size_t e1 = t3o_bit_end(n, 2 * pair + 1);
        const size_t first = (e0 + total - 16) / 32;
        const size_t last = (e1 + total - 1) / 32;
        const unsigned shift = (unsigned)((last + 1) * 32 - (e1 + total));
        const uint64_t merged =
            ((uint64_t)word_u32(words, first % word_count) << 32) | (uint64_t)word_u32(words, last % word_count);
        const uint32_t funnel = (uint32_t)(merged >> shift);
        const unsigned fresh = (unsigned)(e1 - e0);
        out[2 * pair] = (uint16_t)((funnel >> fresh) & 0xFFFFu);
        out[2 * pair + 1] = (uint16_t)(funnel & 0xFFFFu);
    }
}

int t3o_stream_bit(const uint16_t* words, uint32_t n, uint64_t bit) {
    const uint64_t j = bit % ((uint64_t)16 * n);
    return (int)((word_u32(words, (size_t)(j / 32)) >> (31 - (unsigned)(j % 32))) & 1u);
}

uint16_t t3o_codeword_by_definition(const uint16_t* words, uint32_t n, uint64_t t) {
    const uint64_t total = (uint64_t)16 * n;
    const uint64_t end = t3o_bit_end(n, t);
    uint16_t cw = 0;
    for (uint64_t i = 0; i < 16; ++i)
        cw = (uint16_t)((cw << 1) | (uint16_t)t3o_stream_bit(words, n, (end + total - 16 + i) % total));
    return cw;
}

void t3o_tensor_core_perm(uint32_t out[256]) {
    static const uint32_t row_add[4] = {0, 1, 8, 9};
    for (uint32_t lane = 0; lane < 32; ++lane)
        for (uint32_t j = 0; j < 8; ++j) {
            const uint32_t row = (lane % 4) * 2 + row_add[j & 3];
            const uint32_t col = lane / 4 + (j >= 4 ? 8 : 0);
            out[lane * 8 + j] = row * 16 + col;
        }
}

void t3o_decode_tile(const uint16_t* words, uint32_t n, int codebook, int window_bits, uint16_t out[256]) {
    uint16_t cw[256];
    uint32_t perm[256];
    t3o_unpack_tile(words, n, cw);
    t3o_tensor_core_perm(perm); /* per tile, as format.zig:228-229 does */
    const uint16_t mask = (uint16_t)t3o_window_mask(window_bits);
    for (int i = 0; i < 256; ++i) out[perm[i]] = t3o_decode_codeword((uint16_t)(cw[i] & mask), codebook);
}

void t3o_pack_symbols(const uint16_t symbols[256], uint32_t k, uint16_t* out) {
    uint16_t emitted[256];
    size_t i = 0, j = 0;
    for (int row = 0; row < 16; ++row) {
        uint32_t buf = 0;
        int room = 32;
        for (int col = 0; col < 16; ++col, ++i) {
            room -= (int)k;
            buf |= ((uint32_t)symbols[i] & ((1u << k) - 1u)) << room;
            if (room <= 16) {
                emitted[j++] = (uint16_t)(buf >> 16);
                buf <<= 16;
                room += 16;
            }
        }
    }
    const size_t words = (size_t)256 * k / 32;
    for (size_t w = 0; w < words; ++w) { /* SWAP16 within each uint32 */
        out[2 * w] = emitted[2 * w + 1];
        out[2 * w + 1] = emitted[2 * w];
    }
}

/* ------------------------------------------------------------------ H128 (format.zig:258-273) */

void t3o_hadamard128(float v[128]) {
    float tmp[128];
    for (unsigned r = 0; r < 128; ++r) {
        float acc = 0.0f;
        for (unsigned k = 0; k < 128; ++k) {
            const float entry = (__builtin_popcount(r & k) & 1) ? -1.0f * kHadScale : 1.0f * kHadScale;
            acc += entry * v[k];
        }
        tmp[r] = acc;
    }
    memcpy(v, tmp, sizeof tmp);
}

/* ------------------------------------------------------------------ weights (format.zig:276-331) */

void t3o_reconstruct_inner(const uint16_t* trellis, size_t in_f, size_t out_f, uint32_t n, int codebook,
                           int window_bits, uint16_t* out) {
    const size_t in_tiles = in_f / 16, out_tiles = out_f / 16;
    uint16_t tile[256];
    for (size_t tk = 0; tk < in_tiles; ++tk)
        for (size_t tn = 0; tn < out_tiles; ++tn) {
            t3o_decode_tile(trellis + (tk * out_tiles + tn) * n, n, codebook, window_bits, tile);
            for (size_t r = 0; r < 16; ++r)
                memcpy(out + (tk * 16 + r) * out_f + tn * 16, tile + r * 16, 16 * sizeof(uint16_t));
        }
}

int t3o_reconstruct_public(const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                           size_t out_f, uint32_t n, int codebook, int window_bits, uint16_t* out) {
    uint16_t* inner = malloc(in_f * out_f * sizeof(uint16_t));
    float* w = malloc(in_f * out_f * sizeof(float));
    if (!inner || !w) {
        free(inner);
        free(w);
        return -1;
    }
    t3o_reconstruct_inner(trellis, in_f, out_f, n, codebook, window_bits, inner);
    for (size_t i = 0; i < in_f * out_f; ++i) w[i] = h2f(inner[i]);
    float vec[128];
    for (size_t rb = 0; rb < in_f; rb += 128)
        for (size_t c = 0; c < out_f; ++c) {
            for (size_t r = 0; r < 128; ++r) vec[r] = w[(rb + r) * out_f + c];
            t3o_hadamard128(vec);
            for (size_t r = 0; r < 128; ++r) w[(rb + r) * out_f + c] = vec[r];
        }
    for (size_t r = 0; r < in_f; ++r) {
        const float s = h2f(suh[r]);
        for (size_t c = 0; c < out_f; ++c) w[r * out_f + c] *= s;
    }
    for (size_t cb = 0; cb < out_f; cb += 128)
        for (size_t r = 0; r < in_f; ++r) {
            memcpy(vec, w + r * out_f + cb, sizeof vec);
            t3o_hadamard128(vec);
            memcpy(w + r * out_f + cb, vec, sizeof vec);
        }
    for (size_t c = 0; c < out_f; ++c) {
        const float s = h2f(svh[c]);
        for (size_t r = 0; r < in_f; ++r) w[r * out_f + c] *= s;
    }
    for (size_t i = 0; i < in_f * out_f; ++i) out[i] = f2h(w[i]);
    free(inner);
    free(w);
    return 0;
}

/* ------------------------------------------------------------------ one row (format.zig:334-389) */

void t3o_prepare_input(const float* x, const uint16_t* suh, float* out, size_t len) {
    for (size_t i = 0; i < len; ++i) out[i] = round_h(x[i]) * h2f(suh[i]);
    float vec[128];
    for (size_t b = 0; b < len; b += 128) {
        memcpy(vec, out + b, sizeof vec);
        t3o_hadamard128(vec);
        for (size_t i = 0; i < 128; ++i) out[b + i] = round_h(vec[i]);
    }
}

/* outputs of tiles [tn0, tn1) only; every output's sum runs tk ascending, r ascending (format.zig:354-365) */
static void inner_gemv_range(const uint16_t* trellis, const float* transformed, size_t in_f, size_t out_f,
                             uint32_t n, int codebook, int window_bits, float* out, size_t tn0, size_t tn1) {
    const size_t in_tiles = in_f / 16, out_tiles = out_f / 16;
    uint16_t tile[256];
    memset(out + tn0 * 16, 0, (tn1 - tn0) * 16 * sizeof(float));
    for (size_t tk = 0; tk < in_tiles; ++tk)
        for (size_t tn = tn0; tn < tn1; ++tn) {
            t3o_decode_tile(trellis + (tk * out_tiles + tn) * n, n, codebook, window_bits, tile);
            for (size_t r = 0; r < 16; ++r) {
                const float xv = transformed[tk * 16 + r];
                for (size_t c = 0; c < 16; ++c) out[tn * 16 + c] += xv * h2f(tile[r * 16 + c]);
            }
        }
    for (size_t c = tn0 * 16; c < tn1 * 16; ++c) out[c] = round_h(out[c]);
}

void t3o_inner_gemv(const uint16_t* trellis, const float* transformed, size_t in_f, size_t out_f, uint32_t n,
                    int codebook, int window_bits, float* out) {
    inner_gemv_range(trellis, transformed, in_f, out_f, n, codebook, window_bits, out, 0, out_f / 16);
}

void t3o_finish_output(const float* inner, const uint16_t* svh, float* out, size_t len) {
    memcpy(out, inner, len * sizeof(float));
    for (size_t b = 0; b < len; b += 128) t3o_hadamard128(out + b);
    for (size_t i = 0; i < len; ++i) out[i] = round_h(out[i] * h2f(svh[i]));
}

void t3o_project(const float* x, const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                 size_t out_f, uint32_t n, int codebook, int window_bits, float* transformed, float* inner,
                 float* out) {
    t3o_prepare_input(x, suh, transformed, in_f);
    t3o_inner_gemv(trellis, transformed, in_f, out_f, n, codebook, window_bits, inner);
    t3o_finish_output(inner, svh, out, out_f);
}

void t3o_project_what(const float* x, const uint16_t* what, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                      size_t out_f, float* transformed, float* inner, float* out) {
    t3o_prepare_input(x, suh, transformed, in_f);
    memset(inner, 0, out_f * sizeof(float));
    for (size_t k = 0; k < in_f; ++k) {
        const float xv = transformed[k];
        const uint16_t* wrow = what + k * out_f;
        for (size_t c = 0; c < out_f; ++c) inner[c] += xv * h2f(wrow[c]);
    }
    for (size_t c = 0; c < out_f; ++c) inner[c] = round_h(inner[c]);
    t3o_finish_output(inner, svh, out, out_f);
}

/* ------------------------------------------------------------------ the routed layer (ref.zig:78-190) */

float t3o_swiglu_clamped_out(float g, float u, float limit) {
    const float sg = g / (1.0f + expf(-g));
    if (limit <= 0) return sg * u;
    const float sc = sg > limit ? limit : sg;
    const float uc = u > limit ? limit : (u < -limit ? -limit : u);
    return sc * uc;
}

float t3o_swiglu_clamped(float g, float u, float limit) {
    float gc = g, uc = u;
    if (limit > 0) {
        gc = g > limit ? limit : g;
        uc = u > limit ? limit : (u < -limit ? -limit : u);
    }
    return (gc / (1.0f + expf(-gc))) * uc;
}

int t3o_moe_row(const t3o_bank* b, int codebook, int window_bits, float limit, int clamp_at, const float* x,
                const uint32_t* slots, const float* scores, size_t topk, float* y, float* per_slot) {
    const size_t H = b->hidden, I = b->inter;
    const size_t big = H > I ? H : I;
    float* buf = malloc((2 * big + 3 * I + H) * sizeof(float));
    if (!buf) return -1;
    float *transformed = buf, *inner = buf + big, *gate_y = inner + big, *up_y = gate_y + I, *h = up_y + I,
          *down_y = h + I;
    const size_t stride = (H / 16) * (I / 16) * b->n;
    memset(y, 0, H * sizeof(float));
    for (size_t k = 0; k < topk; ++k) {
        const size_t e = slots[k];
        const float w = scores[k];
        t3o_project(x, b->gate_t + e * stride, b->gate_suh + e * H, b->gate_svh + e * I, H, I, b->n, codebook,
                    window_bits, transformed, inner, gate_y);
        t3o_project(x, b->up_t + e * stride, b->up_suh + e * H, b->up_svh + e * I, H, I, b->n, codebook,
                    window_bits, transformed, inner, up_y);
        for (size_t i = 0; i < I; ++i)
            h[i] = clamp_at == T3O_CLAMP_SILU_OUT ? t3o_swiglu_clamped_out(gate_y[i], up_y[i], limit)
                                                  : t3o_swiglu_clamped(gate_y[i], up_y[i], limit);
        t3o_project(h, b->down_t + e * stride, b->down_suh + e * I, b->down_svh + e * H, I, H, b->n, codebook,
                    window_bits, inner, transformed, down_y);
        if (per_slot) memcpy(per_slot + k * H, down_y, H * sizeof(float));
        for (size_t i = 0; i < H; ++i) y[i] += w * down_y[i];
    }
    free(buf);
    return 0;
}

void t3o_compare(const float* got, const float* ref, size_t len, double half_ulp, double out3[3]) {
    double max_abs = 0, ss = 0;
    for (size_t i = 0; i < len; ++i) {
        const double d = fabs((double)got[i] - (double)ref[i]) - half_ulp * fabs((double)ref[i]);
        if (d > max_abs) max_abs = d;
        ss += (double)ref[i] * (double)ref[i];
    }
    const double rms = sqrt(ss / (double)len);
    out3[0] = max_abs;
    out3[1] = rms;
    out3[2] = rms > 0 ? max_abs / rms : max_abs;
}

/* ------------------------------------------------------------------ threaded drivers */

typedef struct {
    void (*fn)(void*, size_t, size_t);
    void* ctx;
    size_t lo, hi;
} span_job;

static void* span_main(void* p) {
    span_job* j = p;
    j->fn(j->ctx, j->lo, j->hi);
    return NULL;
}

/* fn over [0, count) cut into `threads` contiguous spans */
static int run_spans(void (*fn)(void*, size_t, size_t), void* ctx, size_t count, int threads) {
    if (threads < 1) threads = 1;
    if ((size_t)threads > count) threads = (int)(count ? count : 1);
    if (threads == 1) {
        fn(ctx, 0, count);
        return 0;
    }
    pthread_t* th = malloc(sizeof(pthread_t) * (size_t)threads);
    span_job* jobs = malloc(sizeof(span_job) * (size_t)threads);
    if (!th || !jobs) {
        free(th);
        free(jobs);
        return -1;
    }
    int started = 0;
    for (int t = 0; t < threads; ++t) {
        jobs[t].fn = fn;
        jobs[t].ctx = ctx;
        jobs[t].lo = count * (size_t)t / (size_t)threads;
        jobs[t].hi = count * (size_t)(t + 1) / (size_t)threads;
        if (pthread_create(&th[t], NULL, span_main, &jobs[t]) != 0) break;
        ++started;
    }
    for (int t = 0; t < started; ++t) pthread_join(th[t], NULL);
    if (started < threads)
        for (int t = started; t < threads; ++t) fn(ctx, jobs[t].lo, jobs[t].hi);
    free(th);
    free(jobs);
    return 0;
}

typedef struct {
    const uint16_t *trellis, *svh;
    const float* transformed;
    size_t in_f, out_f;
    uint32_t n;
    int codebook, window_bits;
    float* inner;
} gemv_ctx;

static void gemv_span(void* p, size_t lo, size_t hi) {
    gemv_ctx* c = p;
    inner_gemv_range(c->trellis, c->transformed, c->in_f, c->out_f, c->n, c->codebook, c->window_bits, c->inner, lo,
                     hi);
}

int t3o_linear_rows(const float* x, size_t rows, const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh,
                    size_t in_f, size_t out_f, uint32_t n, int codebook, int window_bits, float* y, int threads) {
    float* transformed = malloc(in_f * sizeof(float));
    float* inner = malloc(out_f * sizeof(float));
    if (!transformed || !inner) {
        free(transformed);
        free(inner);
        return -1;
    }
    int rc = 0;
    for (size_t r = 0; r < rows && rc == 0; ++r) {
        t3o_prepare_input(x + r * in_f, suh, transformed, in_f);
        gemv_ctx c = {trellis, svh, transformed, in_f, out_f, n, codebook, window_bits, inner};
        rc = run_spans(gemv_span, &c, out_f / 16, threads);
        t3o_finish_output(inner, svh, y + r * out_f, out_f);
    }
    free(transformed);
    free(inner);
    return rc;
}

typedef struct {
    const float* x;
    const uint16_t *what, *suh, *svh;
    size_t in_f, out_f;
    float* y;
    int failed;
} what_ctx;

static void what_span(void* p, size_t lo, size_t hi) {
    what_ctx* c = p;
    float* scratch = malloc((c->in_f + c->out_f) * sizeof(float));
    if (!scratch) {
        c->failed = 1;
        return;
    }
    for (size_t r = lo; r < hi; ++r)
        t3o_project_what(c->x + r * c->in_f, c->what, c->suh, c->svh, c->in_f, c->out_f, scratch, scratch + c->in_f,
                         c->y + r * c->out_f);
    free(scratch);
}

int t3o_linear_rows_what(const float* x, size_t rows, const uint16_t* what, const uint16_t* suh, const uint16_t* svh,
                         size_t in_f, size_t out_f, float* y, int threads) {
    what_ctx c = {x, what, suh, svh, in_f, out_f, y, 0};
    if (run_spans(what_span, &c, rows, threads) != 0) return -1;
    return c.failed ? -1 : 0;
}

typedef struct {
    const t3o_bank* b;
    int codebook, window_bits, clamp_at;
    float limit;
    const float* x;
    const uint32_t* slots;
    const float* scores;
    size_t topk;
    float* y;
    int failed;
} moe_ctx;

static void moe_span(void* p, size_t lo, size_t hi) {
    moe_ctx* c = p;
    for (size_t r = lo; r < hi; ++r)
        if (t3o_moe_row(c->b, c->codebook, c->window_bits, c->limit, c->clamp_at, c->x + r * c->b->hidden,
                        c->slots + r * c->topk, c->scores + r * c->topk, c->topk, c->y + r * c->b->hidden,
                        NULL) != 0)
            c->failed = 1;
}

int t3o_moe_rows(const t3o_bank* b, int codebook, int window_bits, float limit, int clamp_at, const float* x,
                 size_t rows, const uint32_t* slots, const float* scores, size_t topk, float* y, int threads) {
    moe_ctx c = {b, codebook, window_bits, clamp_at, limit, x, slots, scores, topk, y, 0};
    if (run_spans(moe_span, &c, rows, threads) != 0) return -1;
    return c.failed ? -1 : 0;
}
