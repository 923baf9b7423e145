/*
 * moe_host.c -- C host side of the MoE path over libmoe_cuda (see moe_host.h).
 * Each function follows the reference function named beside it; the only
 * change is the dispatch target: mda_vkc_run(kernel, bufs, grid, &pc) becomes
 * the matching moe_cuda_* call with the same buffers in the same order and the
 * same push-constant values.
 */
#include "moe_host.h"

#include <stdio.h>
#include <string.h>

static uint32_t moe_host_round(uint32_t n, uint32_t to) { /* src/qwen.c:39-41 */
    return (n + to - 1) / to * to;
}

uint32_t moe_host_moe_cols(moe_host_cfg_t cfg) { /* src/qwen.c:55-57 */
    return cfg.experts + MOE_HOST_MOE_PAD + 2 * cfg.shared;
}

uint32_t moe_host_moe_rows(moe_host_cfg_t cfg, uint32_t rows) { /* src/qwen.c:68-70 */
    return moe_host_round(rows * cfg.topk + cfg.experts * (MOE_HOST_TILE - 1), MOE_HOST_TILE);
}

/* mda_qwen_scratch, src/qwen.c:149-185 (MoE members) */
bool moe_host_open(moe_host_t *q, moe_cuda_ctx_t *c, moe_host_cfg_t cfg, uint32_t chunk) {
    memset(q, 0, sizeof(*q));
    q->c = c;
    q->cfg = cfg;
    q->chunk = chunk;
    uint64_t r = chunk;
    uint32_t mrows = moe_host_moe_rows(cfg, chunk);
    uint64_t mr = mrows;
    uint64_t rp = moe_host_round(chunk, MOE_HOST_TILE);
    moe_host_scratch_t *sc = &q->sc;
    sc->p = moe_cuda_alloc(c, r * moe_host_moe_cols(cfg) * sizeof(float));
    sc->a16 = moe_cuda_alloc(c, rp * cfg.d * sizeof(uint16_t)); /* whole 128-row tiles for the shared expert's product */
    moe_cuda_fill(c, sc->a16, rp * cfg.d * sizeof(uint16_t), 0);
    sc->t = moe_cuda_alloc(c, r * cfg.hc_pad * sizeof(float));
    sc->idx = moe_cuda_alloc(c, r * cfg.topk * sizeof(uint32_t));
    sc->wt = moe_cuda_alloc(c, r * cfg.topk * sizeof(float));
    sc->slot = moe_cuda_alloc(c, r * cfg.topk * sizeof(uint32_t));
    sc->count = moe_cuda_alloc(c, cfg.experts * sizeof(uint32_t));
    sc->off = moe_cuda_alloc(c, cfg.experts * sizeof(uint32_t));
    sc->fill = moe_cuda_alloc(c, cfg.experts * sizeof(uint32_t));
    sc->tiles = moe_cuda_alloc(c, mr / MOE_HOST_TILE * sizeof(uint32_t));
    sc->xp = moe_cuda_alloc(c, mr * cfg.d * sizeof(uint16_t));
    sc->g = moe_cuda_alloc(c, mr * 2 * cfg.inter * sizeof(float));
    sc->hp = moe_cuda_alloc(c, mr * cfg.inter * sizeof(float));
    sc->hp16 = moe_cuda_alloc(c, mr * cfg.inter * sizeof(uint16_t));
    sc->ye = moe_cuda_alloc(c, mr * cfg.d * sizeof(float));
    if (cfg.shared != 0) {
        sc->hs = moe_cuda_alloc(c, rp * cfg.shared * sizeof(float));
        sc->sh = moe_cuda_alloc(c, rp * cfg.d * sizeof(float));
        sc->gs = moe_cuda_alloc(c, rp * 2 * cfg.shared * sizeof(float));
        sc->hs16 = moe_cuda_alloc(c, rp * cfg.shared * sizeof(uint16_t));
        sc->tiles0 = moe_cuda_alloc(c, rp / MOE_HOST_TILE * sizeof(uint32_t));
        moe_cuda_fill(c, sc->tiles0, rp / MOE_HOST_TILE * sizeof(uint32_t), 0);
    }
    sc->moe_rows = mrows;
    q->amax = moe_cuda_alloc(c, MOE_HOST_MAX_SLOTS * sizeof(uint32_t)); /* src/qwen.c:250 */
    return moe_cuda_status(c) == MOE_OK;
}

void moe_host_close(moe_host_t *q) {
    moe_host_scratch_t *sc = &q->sc;
    void *all[] = {sc->p, sc->a16, sc->t, sc->idx, sc->wt, sc->slot, sc->count, sc->off, sc->fill, sc->tiles,
                   sc->xp, sc->g, sc->hp, sc->hp16, sc->ye, sc->hs, sc->sh, sc->gs, sc->hs16, sc->tiles0, q->amax};
    for (uint32_t i = 0; i < sizeof(all) / sizeof(all[0]); i += 1) {
        moe_cuda_free(q->c, all[i]);
    }
    memset(q, 0, sizeof(*q));
}

void moe_host_slots_begin(moe_host_t *q) { /* src/qwen.c:500-503 */
    q->n_slots = 0;
    moe_cuda_fill(q->c, q->amax, MOE_HOST_MAX_SLOTS * sizeof(uint32_t), 0);
}

uint32_t moe_host_slot(moe_host_t *q) { /* src/qwen.c:505-515 */
    if (q->n_slots == MOE_HOST_MAX_SLOTS) {
        fprintf(stderr, "moe_host: out of fp16 scale slots\n");
        return MDA_PC_NO_SLOT;
    } else {
        uint32_t s = q->n_slots;
        q->n_slots += 1;
        return s;
    }
}

/* mda_qwen_convert, src/qwen.c:365-378: bf16 -> fp16 in place after the upload */
void moe_host_convert(moe_host_t *q, void *dev, uint64_t used_bytes) {
    uint32_t n = (uint32_t)(used_bytes / sizeof(uint32_t));
    if (n > 0) {
        struct mda_pc_qwen_bf16_t pc = {
            .n = n,
        };
        moe_cuda_bf16_to_f16(q->c, dev, pc);
    }
}

/* mda_qwen_moe_mm, src/qwen.c:770-786 */
static void moe_host_moe_mm(moe_host_t *q, void *a, uint32_t sa, void *w, void *out, void *tiles, uint32_t experts,
                            uint32_t m, uint32_t n, uint32_t k) {
    struct mda_pc_moe_mm_t pc = {
        .m = m,
        .n = n,
        .k = k,
        .sa = sa,
        .sb = MDA_PC_NO_SLOT,
    };
    moe_cuda_mm(q->c, a, w, out, q->amax, tiles, pc, experts);
}

/* mda_qwen_route_rec, src/qwen.c:788-836 */
void moe_host_route_rec(moe_host_t *q, uint32_t rows, uint32_t mrows) {
    moe_host_cfg_t cfg = q->cfg;
    moe_host_scratch_t *sc = &q->sc;
    moe_cuda_fill(q->c, sc->count, cfg.experts * sizeof(uint32_t), 0);
    moe_cuda_fill(q->c, sc->fill, cfg.experts * sizeof(uint32_t), 0);
    moe_cuda_fill(q->c, sc->tiles, (uint64_t)mrows / MOE_HOST_TILE * sizeof(uint32_t), 0xffffffffu);
    moe_cuda_fill(q->c, sc->xp, (uint64_t)mrows * cfg.d * sizeof(uint16_t), 0);
    struct mda_pc_moe_route_t pr = {
        .rows = rows,
        .experts = cfg.experts,
        .topk = cfg.topk,
        .stride = moe_host_moe_cols(cfg),
    };
    moe_cuda_route(q->c, sc->p, sc->idx, sc->wt, sc->count, pr);
    struct mda_pc_moe_scan_t ps = {
        .experts = cfg.experts,
        .tile = MOE_HOST_TILE,
    };
    moe_cuda_scan(q->c, sc->count, sc->off, sc->tiles, ps);
    struct mda_pc_moe_scatter_t pt = {
        .rows = rows,
        .topk = cfg.topk,
        .d8 = cfg.d / 8,
    };
    moe_cuda_scatter(q->c, sc->idx, sc->off, sc->fill, sc->a16, sc->xp, sc->slot, pt);
}

/* mda_qwen_moe_rec, src/qwen.c:838-907, from :846 on.  The reference casts x to
 * fp16 (:844) and runs the upstream dense product into p (:845) first; here a16
 * and p are inputs.  sx is NO_SLOT because a16 already holds fp16 values. */
void moe_host_moe_rec(moe_host_t *q, void *h, uint32_t rows) {
    moe_host_cfg_t cfg = q->cfg;
    moe_host_scratch_t *sc = &q->sc;
    uint32_t pcols = moe_host_moe_cols(cfg);
    uint32_t mrows = moe_host_moe_rows(cfg, rows);
    uint32_t sx = MDA_PC_NO_SLOT;
    moe_host_route_rec(q, rows, mrows);
    moe_cuda_fill(q->c, sc->g, (uint64_t)mrows * 2 * cfg.inter * sizeof(float), 0);
    moe_host_moe_mm(q, sc->xp, sx, q->wgu, sc->g, sc->tiles, cfg.experts, mrows, 2 * cfg.inter, cfg.d);
    struct mda_pc_qwen_elem_t pe = {
        .rows = mrows,
        .n = cfg.inter,
        .astride = 2 * cfg.inter,
        .ao = 0,
        .bo = cfg.inter,
        .op = 0,
        .scale = 1.0f,
    };
    moe_cuda_swiglu(q->c, sc->g, sc->hp, pe);
    uint32_t sh = moe_host_slot(q);
    struct mda_pc_absmax_t pa = {
        .n = mrows * cfg.inter,
        .slot = sh,
    };
    moe_cuda_absmax(q->c, sc->hp, q->amax, pa);
    struct mda_pc_cast_t pc = {
        .n = mrows * cfg.inter,
        .slot = sh,
    };
    moe_cuda_cast_f16(q->c, sc->hp, sc->hp16, q->amax, pc);
    moe_host_moe_mm(q, sc->hp16, sh, q->wdown, sc->ye, sc->tiles, cfg.experts, mrows, cfg.d, cfg.inter);
    if (cfg.shared != 0) {
        /* :879-886.  The reference reads the shared expert's gate/up
         * pre-activations from columns experts+128.. of p, written by the dense
         * product at :845; that product is outside this path, so the same
         * numbers are produced here by the grouped kernel with one expert. */
        uint32_t rp = moe_host_round(rows, MOE_HOST_TILE);
        struct mda_pc_moe_mm_t pg = {.m = rp, .n = 2 * cfg.shared, .k = cfg.d, .sa = sx, .sb = MDA_PC_NO_SLOT};
        moe_cuda_mm(q->c, sc->a16, q->wsgu, sc->gs, q->amax, sc->tiles0, pg, 1);
        pe.rows = rows;
        pe.n = cfg.shared;
        pe.astride = 2 * cfg.shared;
        pe.ao = 0;
        pe.bo = cfg.shared;
        moe_cuda_swiglu(q->c, sc->gs, sc->hs, pe);
        uint32_t ss = moe_host_slot(q);
        struct mda_pc_absmax_t pas = {.n = rows * cfg.shared, .slot = ss};
        moe_cuda_absmax(q->c, sc->hs, q->amax, pas);
        struct mda_pc_cast_t pcs = {.n = rows * cfg.shared, .slot = ss};
        moe_cuda_cast_f16(q->c, sc->hs, sc->hs16, q->amax, pcs);
        struct mda_pc_moe_mm_t pd = {.m = rp, .n = cfg.d, .k = cfg.shared, .sa = ss, .sb = MDA_PC_NO_SLOT};
        moe_cuda_mm(q->c, sc->hs16, q->wsdown, sc->sh, q->amax, sc->tiles0, pd, 1);
    }
    struct mda_pc_moe_combine_t pm = {
        .rows = rows,
        .d = cfg.d,
        .topk = cfg.topk,
        .pstride = pcols,
        .sg_off = cfg.experts,
        .inj_stride = cfg.hc_pad,
        .inj_off = cfg.hc_rank,
        .hc = cfg.hc,
    };
    moe_cuda_combine(q->c, sc->wt, sc->slot, sc->ye, sc->p, cfg.shared != 0 ? sc->sh : NULL, sc->t, h, pm);
}

void moe_host_moe_rec_fused(moe_host_t *q, void *h, uint32_t rows, uint32_t flags) {
    moe_host_cfg_t cfg = q->cfg;
    moe_host_scratch_t *sc = &q->sc;
    moe_cuda_layer_t L;
    memset(&L, 0, sizeof(L));
    L.rows = rows;
    L.d = cfg.d;
    L.experts = cfg.experts;
    L.topk = cfg.topk;
    L.inter = cfg.inter;
    L.shared = cfg.shared;
    L.pstride = moe_host_moe_cols(cfg);
    L.hc = cfg.hc;
    L.inj_stride = cfg.hc_pad;
    L.inj_off = cfg.hc_rank;
    L.proj = sc->p;
    L.x16 = sc->a16;
    L.wgu = q->wgu;
    L.wdown = q->wdown;
    L.wsgu = q->wsgu;
    L.wsdown = q->wsdown;
    L.inj = sc->t;
    L.h = h;
    L.idx = sc->idx;
    L.slot = sc->slot;
    L.count = sc->count;
    L.off = sc->off;
    L.tiles = sc->tiles;
    L.wt = sc->wt;
    L.flags = flags;
    moe_cuda_layer(q->c, &L);
}
