/*
 * moe_host.h -- the reference's MoE call sites, restated in C against
 * libmoe_cuda.  It mirrors, name for name, the parts of src/qwen.c that touch
 * the MoE path: the configuration fields (src/qwen.h:41-65), the scratch
 * buffers (src/qwen.c:149-185), the sizing helpers (src/qwen.c:55-57, 68-70),
 * the scale slots (src/qwen.c:500-515) and the two recording functions
 * mda_qwen_route_rec (src/qwen.c:788-836) and mda_qwen_moe_rec
 * (src/qwen.c:838-907).  Compiled with the reference's own flags (-std=gnu17).
 */
#ifndef MOE_HOST_H
#define MOE_HOST_H

#include <stdbool.h>
#include <stdint.h>

#include "moe_cuda.h"

#define MOE_HOST_TILE 128      /* MDA_QWEN_TILE, src/qwen.h:14 */
#define MOE_HOST_MOE_PAD 128   /* MDA_QWEN_MOE_PAD, src/qwen.h:22 */
#define MOE_HOST_MAX_SLOTS 256 /* MDA_QWEN_MAX_SLOTS, src/qwen.h:13 */

typedef struct moe_host_cfg_t {  /* the mda_qwen_cfg_t fields this path reads */
    uint32_t d, experts, topk, inter, shared;
    uint32_t hc;                 /* MDA_QWEN_HC (4) in the reference; 1 = plain residual */
    uint32_t hc_pad, hc_rank;    /* row stride / offset of the injection scalars (src/qwen.c:893-894) */
} moe_host_cfg_t;

typedef struct moe_host_scratch_t {  /* mda_qwen_scratch_t, MoE members only */
    void *p;      /* fp32 [chunk x moe_cols]: upstream projection (logits, shared gate) */
    void *a16;    /* fp16 [chunk x d]: activations after the cast at src/qwen.c:844 */
    void *t;      /* fp32 [chunk x hc_pad]: injection scalars */
    void *idx, *wt, *slot, *count, *off, *fill, *tiles;
    void *xp, *g, *hp, *hp16, *ye, *hs, *sh;
    void *gs, *hs16, *tiles0; /* shared expert: pre-activations the reference takes from p's columns */
    uint32_t moe_rows;
} moe_host_scratch_t;

typedef struct moe_host_t {
    moe_cuda_ctx_t *c;
    moe_host_cfg_t cfg;
    moe_host_scratch_t sc;
    void *wgu, *wdown, *wsgu, *wsdown; /* device weights of the current layer (src/qwen.c:235-246) */
    void *amax;                        /* scale slots, u32[256] (src/qwen.c:250) */
    uint32_t n_slots;
    uint32_t chunk;
} moe_host_t;

uint32_t moe_host_moe_cols(moe_host_cfg_t cfg);                  /* src/qwen.c:55-57 */
uint32_t moe_host_moe_rows(moe_host_cfg_t cfg, uint32_t rows);   /* src/qwen.c:68-70 */
bool moe_host_open(moe_host_t *q, moe_cuda_ctx_t *c, moe_host_cfg_t cfg, uint32_t chunk);
void moe_host_close(moe_host_t *q);
void moe_host_slots_begin(moe_host_t *q);                        /* src/qwen.c:500-503 */
uint32_t moe_host_slot(moe_host_t *q);                           /* src/qwen.c:505-515 */
void moe_host_convert(moe_host_t *q, void *dev, uint64_t used_bytes);          /* mda_qwen_convert, src/qwen.c:365-378 */
void moe_host_route_rec(moe_host_t *q, uint32_t rows, uint32_t mrows); /* src/qwen.c:788-836 */
/* src/qwen.c:838-907 from the routing on; p and a16 must hold the upstream
 * projection and the fp16 activations.  h: fp32 [rows x hc x d], accumulated. */
void moe_host_moe_rec(moe_host_t *q, void *h, uint32_t rows);
/* The same layer through the single fused entry point. */
void moe_host_moe_rec_fused(moe_host_t *q, void *h, uint32_t rows, uint32_t flags);

#endif
