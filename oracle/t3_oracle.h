/* CPU oracle of the EXL3 projection path: a plain-C restatement of turboexl3's host reference
 * (src/core/format.zig and src/core/ref.zig).
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, imports or calls this file; it exists so the
 * parity tests, the smoke check and the bench's CPU-baseline leg have something to hold the CUDA kernels to.
 *
 * Parity pin: the reference is a Zig library and cannot be built where this oracle is developed, so the oracle is
 * pinned on the literal known-answer values and identities of the reference's own CPU tests
 * (src/core/format.zig:427-571, src/core/lane.zig:244-254, src/core/ref.zig:284-306); see tests/test_oracle_pins.py.
 *
 * Conventions: f16 values travel as their uint16 bit patterns; f16<->f32 conversions are IEEE round-to-nearest-even
 * (_Float16 casts); this file must be compiled with -ffp-contract=off so that a*b+c is two roundings exactly where the
 * reference writes a multiply and an add, and fmaf() only where the reference writes @mulAdd.
 */
#ifndef T3_ORACLE_H
#define T3_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { T3O_MUL1 = 0, T3O_MCG = 1 };          /* format.zig:18-21 Codebook */
enum { T3O_CLAMP_GATE_IN = 0, T3O_CLAMP_SILU_OUT = 1 }; /* format.zig:83 ClampAt */

/* format.zig:10-16 */
#define T3O_TILE 16
#define T3O_TILE_VALUES 256
#define T3O_HAD_DIM 128

float t3o_had_scale(void);
uint32_t t3o_multiplier(int codebook);                   /* format.zig:30-35 */
int t3o_window_mask(int window_bits);                    /* format.zig:60-69; -1 when the width is not admitted */
int t3o_rate_admitted(uint64_t n);                       /* format.zig:98-101 */
uint64_t t3o_bit_end(uint32_t n, uint64_t t);            /* format.zig:116-118 */
uint64_t t3o_fresh_bits(uint32_t n, uint64_t t);         /* format.zig:120-122 */

uint16_t t3o_f32_to_f16_bits(float v);                   /* format.zig:144-146 */
float t3o_f16_bits_to_f32(uint16_t bits);                /* format.zig:140-142 */

uint16_t t3o_decode_mcg(uint16_t cw);                    /* format.zig:149-155 */
uint16_t t3o_decode_mul1(uint16_t cw);                   /* format.zig:158-167 */
uint32_t t3o_mul1_t(uint16_t cw);                        /* the byte sum inside decodeMul1 (lane.zig:244-254 holds it to decodeMul1) */
uint16_t t3o_decode_codeword(uint16_t cw, int codebook); /* format.zig:169-174 */

void t3o_unpack_tile(const uint16_t* words, uint32_t n, uint16_t out[256]);              /* format.zig:182-200 */
int t3o_stream_bit(const uint16_t* words, uint32_t n, uint64_t bit);                     /* format.zig:204-209 */
uint16_t t3o_codeword_by_definition(const uint16_t* words, uint32_t n, uint64_t t);      /* format.zig:212-222 */
void t3o_tensor_core_perm(uint32_t out[256]);                                            /* format.zig:237-256 */
void t3o_decode_tile(const uint16_t* words, uint32_t n, int codebook, int window_bits, uint16_t out[256]); /* :225-234 */
void t3o_hadamard128(float v[128]);                                                      /* format.zig:265-273 */
void t3o_pack_symbols(const uint16_t symbols[256], uint32_t k, uint16_t* out);           /* format.zig:395-423 */

/* format.zig:276-291: W_hat [in, out] f16 bits */
void t3o_reconstruct_inner(const uint16_t* trellis, size_t in_f, size_t out_f, uint32_t n, int codebook,
                           int window_bits, uint16_t* out);
/* format.zig:295-331 */
int t3o_reconstruct_public(const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                           size_t out_f, uint32_t n, int codebook, int window_bits, uint16_t* out);
/* format.zig:334-345, 348-367, 370-380, 383-389 */
void t3o_prepare_input(const float* x, const uint16_t* suh, float* out, size_t len);
void t3o_inner_gemv(const uint16_t* trellis, const float* transformed, size_t in_f, size_t out_f, uint32_t n,
                    int codebook, int window_bits, float* out);
void t3o_finish_output(const float* inner, const uint16_t* svh, float* out, size_t len);
void t3o_project(const float* x, const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                 size_t out_f, uint32_t n, int codebook, int window_bits, float* transformed, float* inner,
                 float* out);

/* ref.zig:250-260 Linear.row: format.project's values from a W_hat decoded once (same per-output summation order). */
void t3o_project_what(const float* x, const uint16_t* what, const uint16_t* suh, const uint16_t* svh, size_t in_f,
                      size_t out_f, float* transformed, float* inner, float* out);

/* ref.zig:124-140 */
float t3o_swiglu_clamped(float g, float u, float limit);
float t3o_swiglu_clamped_out(float g, float u, float limit);

/* One routed bank (ref.zig:9-40), expert e on axis 0 of every array. */
typedef struct {
    size_t experts, hidden, inter;
    uint32_t n;
    const uint16_t *gate_t, *gate_suh, *gate_svh;
    const uint16_t *up_t, *up_suh, *up_svh;
    const uint16_t *down_t, *down_suh, *down_svh;
} t3o_bank;

/* ref.zig:154-190 moeRowClampedAt (limit 0 = moeRow/moeRowDec, ref.zig:78-113). y [hidden] in f32.
 * per_slot (optional, [topk, hidden]) receives each slot's down projection output before the score weighting. */
int t3o_moe_row(const t3o_bank* b, int codebook, int window_bits, float limit, int clamp_at, const float* x,
                const uint32_t* slots, const float* scores, size_t topk, float* y, float* per_slot);

/* ref.zig:195-218. out3 = {max_abs, rms_ref, max_ratio}. half_ulp 0 is `compare`. */
void t3o_compare(const float* got, const float* ref, size_t len, double half_ulp, double out3[3]);

/* ---- drivers over many rows (not in the reference: thread the faithful per-row functions, same values) ---- */

/* rows of format.project, faithful (decodes every tile on every call); `threads` workers split each row's output
 * tiles into contiguous ranges, so every output keeps format.innerGemv's summation order. */
int t3o_linear_rows(const float* x, size_t rows, const uint16_t* trellis, const uint16_t* suh, const uint16_t* svh,
                    size_t in_f, size_t out_f, uint32_t n, int codebook, int window_bits, float* y, int threads);
/* rows of t3o_project_what over `threads` workers (rows are independent). */
int t3o_linear_rows_what(const float* x, size_t rows, const uint16_t* what, const uint16_t* suh, const uint16_t* svh,
                         size_t in_f, size_t out_f, float* y, int threads);
/* rows of t3o_moe_row over `threads` workers (rows are independent). slots/scores [rows, topk], y [rows, hidden]. */
int t3o_moe_rows(const t3o_bank* b, int codebook, int window_bits, float limit, int clamp_at, const float* x,
                 size_t rows, const uint32_t* slots, const float* scores, size_t topk, float* y, int threads);

#ifdef __cplusplus
}
#endif
#endif
