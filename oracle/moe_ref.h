/*
 * moe_ref.h -- CPU oracle for the teacher's mixture-of-experts forward path.
 *
 * TEST INFRASTRUCTURE ONLY.  This is a scalar C restatement of the reference's
 * GLSL kernels and of the host sequence that orders them; it is the checker
 * and the timed CPU baseline, never a product code path.  Only the tests, the
 * smoke check and the benchmark's cpu_baseline / reference arm may call it.
 *
 * PARITY UNPINNED: the reference holds no golden vector, known-answer test or
 * fixture for this path (its `make test` never loads a moe_* shader), and its
 * shaders cannot be compiled or run without a Vulkan stack.  The pins used
 * instead are this file's own invariants and an independent numpy restatement
 * in the test-suite.
 *
 * Every function names the reference file:line it follows.
 */
#ifndef MOE_REF_H
#define MOE_REF_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MOE_REF_NO_SLOT 0xffffffffu /* src/pc.h:6 MDA_PC_NO_SLOT */
#define MOE_REF_MAXK 16u            /* shader/moe_route.comp:18 */
#define MOE_REF_MAXE 512u           /* shader/moe_route.comp:17,24-26; moe_scan.comp:2 */

/* fp16 helpers (IEEE binary16, round to nearest even on narrowing). */
float moe_ref_h2f(uint16_t h);
uint16_t moe_ref_f2h(float f);

int moe_ref_threads(void);
void moe_ref_set_threads(int n);

/* shader/moe_route.comp:20-62.  Returns 0, or -1 if some row has fewer than
 * topk selectable candidates (logit > -3.0e38 and not NaN): the shader would
 * then index count[~0u]. */
int moe_ref_route(const float *proj, uint32_t rows, uint32_t experts, uint32_t topk,
                  uint32_t stride, uint32_t *idx, float *wt, uint32_t *count);

/* shader/moe_scan.comp:14-38.  tiles[] is only written for used tiles, as in
 * the shader; the caller pre-fills it (src/qwen.c:796). */
void moe_ref_scan(const uint32_t *count, uint32_t experts, uint32_t tile, uint32_t *off,
                  uint32_t *tiles);

/* shader/moe_scatter.comp:18-33, pairs visited in ascending order so that the
 * order inside an expert is by token index.  fill[] must be zero on entry. */
void moe_ref_scatter(const uint32_t *idx, const uint32_t *off, uint32_t *fill,
                     const uint16_t *x16, uint16_t *xp, uint32_t *slot, uint32_t rows,
                     uint32_t topk, uint32_t d8);

/* shader/matmul_f16_moe.comp:60-68 and shader/cast_f16.comp:20-28. */
float moe_ref_slot_scale(const uint32_t *amax, uint32_t s);

/* shader/matmul_f16_moe.comp:70-126.  A [m x k] fp16, B [experts][n x k] fp16,
 * C [m x n] fp32.  Row tile y (128 rows) uses expert tiles[y] and is skipped
 * when that is ~0u.  row_mask (may be NULL) has one byte per row of A; rows
 * with a zero byte are skipped -- a test-only shortcut to bound CPU time. */
void moe_ref_mm(const uint16_t *A, const uint16_t *B, float *C, const uint32_t *amax,
                const uint32_t *tiles, uint32_t m, uint32_t n, uint32_t k, uint32_t sa,
                uint32_t sb, const uint8_t *row_mask);

/* shader/qwen_elem.comp:20-31, op 0. */
void moe_ref_swiglu(const float *a, float *y, uint32_t rows, uint32_t n, uint32_t astride,
                    uint32_t ao, uint32_t bo);

/* shader/absmax.comp:13-31 (atomicMax on the float bits of a non-negative). */
void moe_ref_silu_scaled(const float *a, float *y, uint32_t rows, uint32_t n, uint32_t astride, uint32_t ao,
                         float scale); /* shader/qwen_elem.comp op 1 */
void moe_ref_norm(const float *x, const float *w, float *y, uint32_t rows, uint32_t groups, uint32_t gsize,
                  uint32_t w_off, uint32_t op, float eps, float scale); /* shader/qwen_norm.comp ops 0, 1 */
void moe_ref_hc(const float *a, const float *b, float *h, uint32_t rows, uint32_t d, uint32_t hc, uint32_t op,
                uint32_t inj_stride, uint32_t inj_off); /* shader/qwen_hc.comp */
void moe_ref_absmax(const float *x, uint64_t n, uint32_t *amax, uint32_t slot);

/* shader/cast_f16.comp:30-35. */
void moe_ref_cast_f16(const float *src, uint16_t *dst, uint64_t n, const uint32_t *amax,
                      uint32_t slot);

/* shader/moe_combine.comp:26-40.  sh may be NULL (no shared expert: the term
 * is dropped, equal to sh = 0); inj may be NULL (equal to inj = 0). */
void moe_ref_combine(const float *wt, const uint32_t *slot, const float *y, const float *proj,
                     const float *sh, const float *inj, float *h, uint32_t rows, uint32_t d,
                     uint32_t topk, uint32_t pstride, uint32_t sg_off, uint32_t inj_stride,
                     uint32_t inj_off, uint32_t hc);

/* Residual + RMSNorm used between the layers of the stacked configuration:
 * y = fp16( v * rsqrt(mean(v^2) + eps) ), v = x16 + delta   (weight 1),
 * after shader/qwen_norm.comp:55-61,79 op 0 with MDA_QWEN_EPS (src/qwen.h:16). */
void moe_ref_residual_rmsnorm(const uint16_t *x16, const float *delta, uint16_t *y16,
                              uint32_t rows, uint32_t d, float eps);

/* shader/qwen_bf16.comp:9-15 (call src/qwen.c:365-378): n 32-bit words, each two
 * bf16 values, rewritten in place as two fp16 values (round to nearest even,
 * overflow to infinity), as the upload of a layer's weights does. */
void moe_ref_bf16_to_f16(uint32_t *w, uint64_t n);

/* shader/kd_bytes.comp:96-147 (call mda_teach_sink, src/teach.c:108-128): the teacher's next-token
 * distribution over a byte-level vocabulary turned into per-byte distributions along the true
 * continuation.  logits [rows x vocab] fp32; toks [vocab x 5] u32 (16 bytes little-endian in four
 * words, then the length; length 0 = not a byte string); cont [rows x 5] (the 16 bytes that follow,
 * then how many of them count); outp [rows x 16 x 8] entries byte | fp16(probability) << 16:
 * entry 0 of depth l is the true byte, entries 1..7 the most probable other bytes. */
void moe_ref_kd_bytes(const float *logits, const uint32_t *toks, const uint32_t *cont, uint32_t *outp,
                      uint32_t rows, uint32_t vocab);

/* One whole layer in the order of src/qwen.c:788-907 (mda_qwen_route_rec then
 * mda_qwen_moe_rec from the first grouped product on).  All buffers are
 * caller-owned; see moe_ref_layer_t. */
typedef struct moe_ref_layer_t {
    uint32_t rows, d, experts, topk, inter, shared; /* shared = 0: no shared expert */
    uint32_t pstride;                               /* row stride of proj */
    uint32_t hc;                                    /* residual streams (1 for plain) */
    uint32_t tile;                                  /* 128: src/qwen.h:14 */
    const float *proj;     /* [rows x pstride]: logits in columns < experts, shared gate at column experts */
    const uint16_t *x16;   /* [rows x d] fp16 activations */
    const uint16_t *wgu;   /* [experts][2*inter x d] */
    const uint16_t *wdown; /* [experts][d x inter] */
    const uint16_t *wsgu;  /* [2*shared x d] or NULL */
    const uint16_t *wsdown;/* [d x shared] or NULL */
    const float *inj;      /* [rows x hc] or NULL */
    float *h;              /* [rows x hc x d], accumulated into */
    /* outputs kept for parity checks (all caller-allocated) */
    uint32_t *idx, *slot, *count, *off, *tiles;
    float *wt;
    uint32_t mrows;        /* round128(rows*topk + experts*127): src/qwen.c:68-70 */
    uint16_t *xp;          /* [mrows x d] */
    float *ye;             /* [mrows x d] */
    uint16_t *hp16;        /* [mrows x inter] or NULL */
    uint32_t *amax;        /* [4] scale slots: 0 = sh (expert h), 1 = ss (shared h) */
    const uint8_t *row_mask; /* optional [rows]: tokens whose expert products are computed */
} moe_ref_layer_t;

int moe_ref_layer(moe_ref_layer_t *L);

#ifdef __cplusplus
}
#endif
#endif
