/* t3_table.h: the quant-plugin table over the engine, for hosts that hold their tensors in HOST memory.
 *
 * The reference ships the same thing for its host application: a table of C function pointers
 * (`abi.QuantTable`, turboexl3 table/table.zig:30-60) whose members claim a pack's EXL3 blocks, take its tensors at load
 * time and run `matmul` (a dense linear) and `swiglu` (a layer's routed experts) on the engine. There the tensors are MLX
 * arrays in unified memory; here `load_tensor` / `load_bank` upload them once to the current CUDA device (the weights then
 * stay resident, in the pack's own layout), and `matmul` / `swiglu` take activations wherever they live: a host array is
 * copied in, the result copied out, and the call returns when the result is in place; device arrays run stream-ordered
 * with no copy. Member names, refusal texts and error names are the reference's (table/table.zig, table/config.zig,
 * docs/core/consuming.md:141-149). The binary layout of the reference's ABI structs lives in its host's plugin kit, which
 * is not part of the reference tree, so the structs below are this library's own.
 */
#ifndef T3_TABLE_H
#define T3_TABLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { T3_VERDICT_OK = 0, T3_VERDICT_UNSUPPORTED = 1, T3_VERDICT_FAILED = 2 } t3_verdict_kind;

/* abi.Verdict: ok, or a refusal with its reason (a static string: an error name or a sentence). */
typedef struct {
    int kind;            /* t3_verdict_kind */
    const char* reason;  /* null when ok */
} t3_verdict;

typedef enum { T3_CLAIM_NO = 0, T3_CLAIM_BY_MARKER = 1 } t3_claim;

/* A dense array. dtype: 0 f32, 1 f16, 2 bf16 (t3_dtype), 3 u16, 4 i16, 5 i32, 6 u32. `device` 0 = host memory. */
typedef enum { T3_A_F32 = 0, T3_A_F16 = 1, T3_A_BF16 = 2, T3_A_U16 = 3, T3_A_I16 = 4, T3_A_I32 = 5, T3_A_U32 = 6 } t3_array_dtype;
typedef struct {
    void* data;
    int dtype;
    int ndim;
    int64_t shape[8];
    int device;  /* 0: host pointer; 1: device pointer of the current CUDA device */
} t3_array;

/* abi.Weight as the table fills it (table/table.zig:175-187): the three arrays of a projection (device-resident after
 * load), `layout` = codebook (0 mul1, 1 mcg), `flags` = window bits, `block` = halfwords per tile. */
typedef struct {
    void* w;        /* trellis u16 [in/16, out/16, n] or [E, in/16, out/16, n] */
    void* scales;   /* suh f16 [in] or [E, in] */
    void* biases;   /* svh f16 [out] or [E, out] */
    int layout, flags, block;
    int experts;    /* 0 for a dense linear */
    int in_dim, out_dim;
    size_t bytes;   /* device bytes this weight holds */
} t3_weight;

/* abi.LoadCtx: the claimed block's JSON and the table's per-block state. */
typedef struct {
    const char* block_json;
    void* state;
} t3_load_ctx;

/* abi.Swiglu: the routed call's options (table/table.zig:210-221). */
typedef struct {
    int limit;        /* > 0: the clamped SwiGLU (root.moeClamped) */
    int verify_rows;  /* accepted and ignored, as the reference does */
} t3_swiglu_opts;

typedef struct {
    const char* name;  /* "turboexl3" */
    /* table/config.zig:46-62: a trunk block (`format` exl3, no `k`) is always claimed; a bank block (`k` present) when it
     * parses and the model config names no SwiGLU clamp. */
    int (*claims)(const char* block_json, const char* config_json);
    /* table/config.zig:64-76 */
    t3_verdict (*validate)(const char* block_json, const char* config_json);
    uint64_t (*bill)(const char* block_json, const char* model_dir, uint64_t stored);
    t3_verdict (*open)(t3_load_ctx* ctx);                       /* table/table.zig:77-98 */
    void (*close)(t3_load_ctx* ctx);                            /* table/table.zig:100-103 */
    /* table/table.zig:119-145: `<base>.weight|scales|biases` of a trunk linear; in_dim 0 = take it from the trellis */
    t3_verdict (*load_tensor)(const t3_load_ctx* ctx, const t3_array* weight, const t3_array* scales,
                              const t3_array* biases, uint32_t in_dim, t3_weight* out);
    /* table/table.zig:147-172: `<base>.trellis|suh|svh` of a routed bank */
    t3_verdict (*load_bank)(const t3_load_ctx* ctx, const t3_array* trellis, const t3_array* suh, const t3_array* svh,
                            uint32_t in_dim, t3_weight* out);
    void (*release)(t3_weight* w);                              /* table/table.zig:189-194 */
    /* table/table.zig:196-201: out->data must hold x's leading dims x out_dim elements of x's dtype */
    t3_verdict (*matmul)(const t3_weight* w, const t3_array* x, void* stream, t3_array* out);
    /* table/table.zig:203-205: always refuses; a layer's banks run as one routed SwiGLU */
    t3_verdict (*moe)(const t3_weight* w, const t3_array* x, const t3_array* inds, const t3_array* scores, int sorted,
                      void* stream, t3_array* out);
    /* table/table.zig:210-221: x [B, S, D]; inds, scores [B, S, K]; out like x */
    t3_verdict (*swiglu)(const t3_weight* gate, const t3_weight* up, const t3_weight* down, const t3_array* x,
                         const t3_array* inds, const t3_array* scores, const t3_swiglu_opts* opts, void* stream,
                         t3_array* out);
} t3_quant_table;

/* The table (table/table.zig:30). */
const t3_quant_table* t3_table(void);

/* Device bytes the table's staging buffers hold (activations in and out, engine workspace). */
size_t t3_table_staging_bytes(void);
/* Frees the staging buffers (root.releaseEngines' role, src/root.zig:1148-1192); weights are freed by `release`. */
void t3_table_release_staging(void);

#ifdef __cplusplus
}
#endif
#endif
