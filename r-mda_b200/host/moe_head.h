/*
 * moe_head.h -- C host side of the two steps either side of the MoE layers, over
 * libmoe_cuda: the hyper-connection residual mixer (mda_qwen_res_rec,
 * src/qwen.c:641-663) and the teacher's head (mda_qwen_head,
 * src/qwen.c:1080-1099: mixer, cast, vocabulary product in row chunks, sink
 * callback), with the distillation sink of src/teach.c:108-128 as a ready-made
 * callback.  Same function order, buffers and push constants as the reference;
 * only the dispatch target differs.
 */
#ifndef MOE_HEAD_H
#define MOE_HEAD_H

#include <stdbool.h>
#include <stdint.h>

#include "moe_cuda.h"

#define MOE_MIX_MAX_SLOTS 256 /* MDA_QWEN_MAX_SLOTS, src/qwen.h:13 */

typedef struct moe_mix_t {
    moe_cuda_ctx_t *c;
    uint32_t d, hc, hc_rank, hc_pad; /* cfg.d, MDA_QWEN_HC, cfg.hc_rank, MDA_QWEN_HC_PAD */
    uint32_t rows;                   /* most rows one call handles (chunk / head_rows) */
    uint32_t vocab;                  /* 0: no head */
    /* mda_qwen_scratch_t members the mixer and the head use (src/qwen.c:149-185) */
    void *hn, *a16, *t, *u, *up, *x, *logits;
    void *amax; /* scale slots, u32[256] (src/qwen.c:250) */
    uint32_t n_slots;
} moe_mix_t;

/* the weights of one mixer: mda_qwen_res_t's offsets resolved to device pointers */
typedef struct moe_mix_w_t {
    const void *norm; /* fp32 [hc * d] */
    const void *down; /* fp16 [hc_pad x hc*d], rows >= hc_rank + hc used (mda_qwen_pad_to, src/qwen.c:406) */
    const void *up;   /* fp16 [hc*d x hc_rank] */
} moe_mix_w_t;

/* mda_qwen_sink_t (src/qwen.h:38): called after every chunk of head rows with the chunk's logits
 * (fp32 [rows x vocab], device) complete on the context's stream. */
typedef bool (*moe_head_sink_t)(void *ctx, moe_mix_t *q, uint32_t row0, uint32_t rows);

bool moe_mix_open(moe_mix_t *q, moe_cuda_ctx_t *c, uint32_t d, uint32_t hc, uint32_t hc_rank, uint32_t hc_pad, uint32_t rows,
                  uint32_t vocab);
void moe_mix_close(moe_mix_t *q);
void moe_mix_slots_begin(moe_mix_t *q);                                   /* src/qwen.c:500-503 */
uint32_t moe_mix_cast(moe_mix_t *q, const void *src, uint32_t n);         /* mda_qwen_cast, src/qwen.c:517-539 */
void moe_mix_mm(moe_mix_t *q, uint32_t sa, const void *w, void *out, uint32_t rows, uint32_t n, uint32_t k); /* mda_qwen_mm, :541-570 */
/* h: fp32 [rows x hc x d] (device).  Leaves the layer's input in q->x and the injection scalars in q->t. */
void moe_mix_res_rec(moe_mix_t *q, const void *h, uint32_t rows, const moe_mix_w_t *r);
/* h: fp32 [rows_total x hc x d]; lm_head: fp16 [vocab x d].  Returns true when every chunk was sunk. */
bool moe_head(moe_mix_t *q, const void *h, uint32_t rows_total, uint32_t head_rows, const moe_mix_w_t *mixer, const void *lm_head,
              moe_head_sink_t sink, void *ctx);

/* mda_teach_sink's device part (src/teach.c:108-128): byte distributions of the chunk's rows into outp. */
typedef struct moe_kd_sink_t {
    const void *toks; /* u32 [vocab x 5] */
    const void *cont; /* u32 [rows_total x 5] */
    void *outp;       /* u32 [rows_total x 16 x 8] */
    uint32_t chunks;  /* counts the calls */
} moe_kd_sink_t;
bool moe_kd_sink(void *ctx, moe_mix_t *q, uint32_t row0, uint32_t rows);

#endif
