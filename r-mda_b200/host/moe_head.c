/*
 * moe_head.c -- see moe_head.h.  Each function follows the reference function
 * named beside it.
 */
#include "moe_head.h"

#include <stdio.h>
#include <string.h>

bool moe_mix_open(moe_mix_t *q, moe_cuda_ctx_t *c, uint32_t d, uint32_t hc, uint32_t hc_rank, uint32_t hc_pad, uint32_t rows,
                  uint32_t vocab) {
    memset(q, 0, sizeof(*q));
    q->c = c;
    q->d = d;
    q->hc = hc;
    q->hc_rank = hc_rank;
    q->hc_pad = hc_pad;
    q->rows = rows;
    q->vocab = vocab;
    uint64_t r = rows, d4 = (uint64_t)hc * d; /* src/qwen.c:151 */
    q->hn = moe_cuda_alloc(c, r * d4 * sizeof(float));
    q->a16 = moe_cuda_alloc(c, r * d4 * sizeof(uint16_t));
    q->t = moe_cuda_alloc(c, r * hc_pad * sizeof(float));  /* :156 */
    q->u = moe_cuda_alloc(c, r * hc_rank * sizeof(float)); /* :157 */
    q->up = moe_cuda_alloc(c, r * d4 * sizeof(float));
    q->x = moe_cuda_alloc(c, r * d * sizeof(float));
    q->logits = vocab != 0 ? moe_cuda_alloc(c, r * vocab * sizeof(float)) : NULL;
    q->amax = moe_cuda_alloc(c, MOE_MIX_MAX_SLOTS * sizeof(uint32_t));
    return moe_cuda_status(c) == MOE_OK;
}

void moe_mix_close(moe_mix_t *q) {
    void *all[] = {q->hn, q->a16, q->t, q->u, q->up, q->x, q->logits, q->amax};
    for (uint32_t i = 0; i < sizeof(all) / sizeof(all[0]); i += 1) {
        moe_cuda_free(q->c, all[i]);
    }
    memset(q, 0, sizeof(*q));
}

void moe_mix_slots_begin(moe_mix_t *q) { /* src/qwen.c:500-503 */
    q->n_slots = 0;
    moe_cuda_fill(q->c, q->amax, MOE_MIX_MAX_SLOTS * sizeof(uint32_t), 0);
}

static uint32_t moe_mix_slot(moe_mix_t *q) { /* src/qwen.c:505-515 */
    if (q->n_slots == MOE_MIX_MAX_SLOTS) {
        fprintf(stderr, "moe_mix: out of fp16 scale slots\n");
        return MDA_PC_NO_SLOT;
    } else {
        uint32_t s = q->n_slots;
        q->n_slots += 1;
        return s;
    }
}

uint32_t moe_mix_cast(moe_mix_t *q, const void *src, uint32_t n) { /* src/qwen.c:517-539 */
    uint32_t slot = moe_mix_slot(q);
    struct mda_pc_absmax_t pa = {
        .n = n,
        .slot = slot,
    };
    moe_cuda_absmax(q->c, src, q->amax, pa);
    struct mda_pc_cast_t pc = {
        .n = n,
        .slot = slot,
    };
    moe_cuda_cast_f16(q->c, src, q->a16, q->amax, pc);
    return slot;
}

void moe_mix_mm(moe_mix_t *q, uint32_t sa, const void *w, void *out, uint32_t rows, uint32_t n, uint32_t k) { /* :541-570 */
    struct moe_pc_dense_t pc = {
        .rows = rows,
        .n = n,
        .k = k,
        .sa = sa,
    };
    moe_cuda_dense(q->c, q->a16, w, out, q->amax, pc);
}

void moe_mix_res_rec(moe_mix_t *q, const void *h, uint32_t rows, const moe_mix_w_t *r) { /* src/qwen.c:641-663 */
    uint32_t d4 = q->hc * q->d;
    struct mda_pc_qwen_norm_t pn = { /* mda_qwen_norm_pc(q, rows, HC, d, 0), src/qwen.c:582-604 */
        .rows = rows,
        .groups = q->hc,
        .gsize = q->d,
        .in_stride = d4,
        .in_off = 0,
        .in_gstride = q->d,
        .out_stride = d4,
        .out_off = 0,
        .out_gstride = q->d,
        .w_off = 0, /* r->norm is a pointer here, an offset into wvec in the reference */
        .wstride = q->d,
        .op = 0,
        .rot = 0,
        .seqlen = 1,
        .z_stride = 0,
        .z_off = 0,
        .z_gstride = 0,
        .eps = 1e-6f, /* MDA_QWEN_EPS */
        .scale = 1.0f,
        .theta = 1.0f,
    };
    moe_cuda_norm(q->c, h, r->norm, q->hn, h, pn);
    uint32_t s = moe_mix_cast(q, q->hn, rows * d4);
    moe_mix_mm(q, s, r->down, q->t, rows, q->hc_pad, d4);
    struct mda_pc_qwen_elem_t pe = {
        .rows = rows,
        .n = q->hc_rank,
        .astride = q->hc_pad,
        .ao = 0,
        .bo = 0,
        .op = 1,
        .scale = 1.0f / (float)q->hc,
    };
    moe_cuda_swiglu(q->c, q->t, q->u, pe);
    uint32_t su = moe_mix_cast(q, q->u, rows * q->hc_rank);
    moe_mix_mm(q, su, r->up, q->up, rows, d4, q->hc_rank);
    struct mda_pc_qwen_hc_t ph = { /* mda_qwen_hc(q, up, hn, x, rows, 0, rows * d), src/qwen.c:615-631 */
        .rows = rows,
        .d = q->d,
        .hc = q->hc,
        .op = 0,
        .inj_stride = q->hc_pad,
        .inj_off = q->hc_rank,
    };
    moe_cuda_hc(q->c, q->up, q->hn, q->x, ph);
}

bool moe_head(moe_mix_t *q, const void *h, uint32_t rows_total, uint32_t head_rows, const moe_mix_w_t *mixer, const void *lm_head,
              moe_head_sink_t sink, void *ctx) { /* src/qwen.c:1080-1099 */
    uint32_t sunk = 0;
    uint32_t hr = head_rows;
    if (hr == 0 || hr > q->rows || q->vocab == 0 || rows_total % hr != 0) {
        fprintf(stderr, "moe_head: head_rows %u does not fit (capacity %u, %u rows, vocab %u)\n", hr, q->rows, rows_total, q->vocab);
        return false;
    }
    for (uint32_t row0 = 0; row0 < rows_total && moe_cuda_status(q->c) == MOE_OK; row0 += hr) {
        const float *hrow = (const float *)h + (uint64_t)row0 * q->hc * q->d; /* mda_qwen_rows */
        moe_mix_slots_begin(q);
        moe_mix_res_rec(q, hrow, hr, mixer);
        uint32_t sx = moe_mix_cast(q, q->x, hr * q->d);
        moe_mix_mm(q, sx, lm_head, q->logits, hr, q->vocab, q->d);
        moe_cuda_flush(q->c);
        if (moe_cuda_status(q->c) == MOE_OK) {
            bool took = sink(ctx, q, row0, hr);
            sunk += took;
        }
    }
    return moe_cuda_status(q->c) == MOE_OK && sunk == rows_total / hr;
}

bool moe_kd_sink(void *ctx, moe_mix_t *q, uint32_t row0, uint32_t rows) { /* src/teach.c:108-128 */
    moe_kd_sink_t *t = ctx;
    struct mda_pc_kd_bytes_t pc = {
        .rows = rows,
        .vocab = q->vocab,
    };
    const uint32_t *cont = (const uint32_t *)t->cont + (uint64_t)row0 * 5u;
    uint32_t *outp = (uint32_t *)t->outp + (uint64_t)row0 * 16u * 8u;
    moe_cuda_kd_bytes(q->c, q->logits, t->toks, cont, outp, pc);
    moe_cuda_flush(q->c);
    t->chunks += 1;
    return moe_cuda_status(q->c) == MOE_OK;
}
