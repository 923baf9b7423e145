/*
 * moe_weights.h -- the weight path of one MoE layer: from a directory of
 * safetensors shards, through page-locked staging banks, to fp16 tensors in
 * device memory.  It restates, for the MoE members only, what the reference's
 * loader does: the shard reader (src/safet.h, src/safet.c), mda_qwen_put /
 * mda_qwen_pad_to (src/qwen.c:310-339), mda_qwen_put_moe (src/qwen.c:441-452),
 * mda_qwen_stage_copy / mda_qwen_convert / mda_qwen_upload
 * (src/qwen.c:356-394) and the loader thread (src/qwen.c:488-498, 1101-1108).
 * On disk the weights are bf16; the device copy is converted in place to fp16
 * by moe_cuda_bf16_to_f16 (shader/qwen_bf16.comp).
 */
#ifndef MOE_WEIGHTS_H
#define MOE_WEIGHTS_H

#include <pthread.h>
#include <stdbool.h>
#include <stdint.h>

#include "moe_cuda.h"

#define MOE_ST_MAX_KEY 256   /* MDA_SAFET_MAX_KEY, src/safet.h:7 */
#define MOE_ST_MAX_DIMS 8
#define MOE_BANK_THREADS 16  /* MDA_QWEN_THREADS, src/qwen.h:25 */
#define MOE_HOST_PAD_ROWS 128 /* MDA_QWEN_MOE_PAD, src/qwen.h:22 */

enum { MOE_ST_BF16 = 0, MOE_ST_I64 = 1, MOE_ST_OTHER = 2 }; /* src/safet.h:15-18 */

typedef struct moe_st_entry_t { /* one tensor of a shard's header */
    const char *key;
    uint32_t key_len;
    uint32_t dtype;
    uint32_t elem; /* bytes per element, 0 if the dtype is not known */
    uint32_t ndim;
    uint64_t shape[MOE_ST_MAX_DIMS];
    uint64_t begin, end; /* data_offsets, relative to the end of the header */
} moe_st_entry_t;

typedef struct moe_st_file_t { /* mda_safet_file_t: one mapped shard */
    uint8_t *bytes;
    uint64_t mapped;
    const uint8_t *data; /* first byte after the header */
    uint64_t size;       /* bytes of tensor data */
    moe_st_entry_t *ent;
    uint32_t n;
    bool ok;
} moe_st_file_t;

typedef struct moe_st_tensor_t { /* mda_safet_tensor_t: leading dimensions folded into rows */
    const uint8_t *data;
    uint64_t rows;
    uint32_t cols;
    uint32_t dtype;
    bool ok;
} moe_st_tensor_t;

typedef struct moe_st_set_t { /* mda_safet_set_t: every *.safetensors of a directory */
    moe_st_file_t *files;
    uint32_t n;
} moe_st_set_t;

moe_st_file_t moe_st_read(const char *path);                                 /* mda_safet_read */
void moe_st_free(moe_st_file_t *f);                                          /* mda_safet_free */
bool moe_st_has(const moe_st_file_t *f, const char *name);                   /* mda_safet_has */
moe_st_tensor_t moe_st_tensor(const moe_st_file_t *f, const char *name);     /* mda_safet_tensor */
float moe_st_bf16(const uint8_t *data, uint64_t i);                          /* mda_safet_bf16 */
moe_st_set_t moe_st_open_set(const char *dir);                               /* mda_safet_open_set */
void moe_st_free_set(moe_st_set_t *s);                                       /* mda_safet_free_set */
moe_st_tensor_t moe_st_find(const moe_st_set_t *s, const char *name);        /* mda_safet_find */

typedef struct moe_stage_t { /* mda_qwen_stage_t: a host staging buffer that fills front to back */
    void *host;
    uint64_t size, used;
} moe_stage_t;

typedef struct moe_bank_t { /* mda_qwen_bank_t, MoE members */
    moe_stage_t dense; /* router rows, shared gate row, padding, shared gate_proj, up_proj, down_proj */
    moe_stage_t gu;    /* mlp.experts.gate_up_proj  [E][2I x d] */
    moe_stage_t down;  /* mlp.experts.down_proj     [E][d x I] */
    uint64_t moe;      /* element offset of the router block inside dense (mda_qwen_layer_t.moe) */
    uint64_t sdown;    /* element offset of the shared expert's down_proj inside dense (.sdown) */
    bool pinned, fail;
    moe_cuda_ctx_t *c;
} moe_bank_t;

typedef struct moe_bank_cfg_t {
    uint32_t d, experts, inter, shared;
} moe_bank_cfg_t;

/* Staging buffers sized for one layer.  c == NULL: pageable memory (host-only use). */
bool moe_bank_open(moe_bank_t *b, moe_cuda_ctx_t *c, moe_bank_cfg_t cfg);
void moe_bank_close(moe_bank_t *b);
void moe_bank_reset(moe_bank_t *b);                                           /* mda_qwen_stage_reset */
uint64_t moe_bank_put(moe_bank_t *b, moe_stage_t *s, moe_st_tensor_t t);      /* mda_qwen_put; returns the element offset */
void moe_bank_pad_to(moe_bank_t *b, moe_stage_t *s, uint64_t start, uint32_t rows, uint32_t cols); /* mda_qwen_pad_to */
/* mda_qwen_put_moe: the six tensors of layer l, named prefix + "layers.<l>.mlp...." */
void moe_bank_put_moe(moe_bank_t *b, const moe_st_set_t *set, const char *prefix, moe_bank_cfg_t cfg, uint32_t l);
/* Expert parallel: rank g of G stages only its experts [e_lo, e_hi) of the two fused expert tensors (rows
 * [e_lo*2I, e_hi*2I) of gate_up_proj and [e_lo*d, e_hi*d) of down_proj, read straight out of the mapped shard);
 * the router rows and the shared expert are replicated and staged whole.  The reference is single-device and
 * always stages all experts (src/qwen.c:441-452, 464-498).  moe_bank_open_slice sizes the expert stages for
 * `local` experts. */
bool moe_bank_open_slice(moe_bank_t *b, moe_cuda_ctx_t *c, moe_bank_cfg_t cfg, uint32_t local);
void moe_bank_put_moe_slice(moe_bank_t *b, const moe_st_set_t *set, const char *prefix, moe_bank_cfg_t cfg, uint32_t l,
                            uint32_t e_lo, uint32_t e_hi);
/* mda_qwen_upload: three host-to-device copies, then the bf16 -> fp16 conversion in place.
 * wd / wgu / wdown: device buffers at least as large as the bank's stages. */
void moe_bank_upload(moe_bank_t *b, void *wd, void *wgu, void *wdown, bool convert_gu);

typedef struct moe_bank_job_t { /* mda_qwen_job_t: loads one layer on a thread while the previous one computes */
    moe_bank_t *b;
    const moe_st_set_t *set;
    const char *prefix;
    moe_bank_cfg_t cfg;
    uint32_t layer;
    pthread_t th;
    bool started;
    uint32_t e_lo, e_hi; /* expert slice to stage; 0, 0 = all experts */
} moe_bank_job_t;
void moe_bank_prefetch(moe_bank_job_t *job); /* mda_qwen_prefetch */
void moe_bank_join(moe_bank_job_t *job);

#endif
