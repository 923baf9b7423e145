/*
 * moe_cuda.h -- C ABI of libmoe_cuda: the teacher's mixture-of-experts forward
 * path (route -> count/scan -> scatter -> grouped SwiGLU products -> combine)
 * as hand-written CUDA for sm_100a.
 *
 * The library replaces, for this path only, the reference's generic Vulkan
 * dispatch `mda_vkc_run(c, kernel, bufs[], gx, gy, gz, &pc)` (src/vkc.h:93,
 * src/vkc.c:771-789) and the buffer calls around it.  Each kernel entry point
 * takes the context, raw device pointers in the binding order of the shader it
 * replaces, and that shader's push-constant struct by value, unchanged.
 *
 * Conventions kept from the reference harness (src/vkc.c:15-20, 528-536):
 *  - no return values on the data path; the first failure makes the context's
 *    status sticky, prints one line to stderr, and every later call is a no-op;
 *  - calls are ordered: each runs after the previous one on the context's
 *    stream; moe_cuda_flush blocks until the device is idle on that stream;
 *  - all calls come from one host thread; buffers are caller-owned.
 * There is no CPU fallback: without a usable CUDA device every call fails.
 */
#ifndef MOE_CUDA_H
#define MOE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- push-constant structs: layout identical to src/pc.h:369-404 -------- */
#ifndef MDA_PC_H
#define MDA_PC_NO_SLOT 0xffffffffu /* src/pc.h:6 */
struct mda_pc_moe_route_t { uint32_t rows, experts, topk, stride; };                 /* src/pc.h:369-374 */
struct mda_pc_moe_scan_t { uint32_t experts, tile; };                                 /* src/pc.h:376-379 */
struct mda_pc_moe_scatter_t { uint32_t rows, topk, d8; };                             /* src/pc.h:381-385 */
struct mda_pc_moe_mm_t { uint32_t m, n, k, sa, sb; };                                 /* src/pc.h:387-393 */
struct mda_pc_moe_combine_t { uint32_t rows, d, topk, pstride, sg_off, inj_stride, inj_off, hc; }; /* src/pc.h:395-404 */
struct mda_pc_qwen_elem_t { uint32_t rows, n, astride, ao, bo, op; float scale; };    /* shader/qwen_elem.comp:6-14 */
struct mda_pc_absmax_t { uint32_t n, slot; };                                          /* shader/absmax.comp:6-9 */
struct mda_pc_cast_t { uint32_t n, slot; };                                            /* shader/cast_f16.comp:14-17 */
struct mda_pc_qwen_bf16_t { uint32_t n; };                                             /* src/pc.h:273-275 */
struct mda_pc_kd_bytes_t { uint32_t rows, vocab; };                                    /* src/pc.h:406-409 */
struct mda_pc_qwen_norm_t {                                                            /* src/pc.h:283-304 */
    uint32_t rows, groups, gsize, in_stride, in_off, in_gstride, out_stride, out_off, out_gstride, w_off, wstride, op, rot,
        seqlen, z_stride, z_off, z_gstride;
    float eps, scale, theta;
};
struct mda_pc_qwen_hc_t { uint32_t rows, d, hc, op, inj_stride, inj_off; };            /* src/pc.h:306-313 */
#endif
/* mda_qwen_mm's arguments (src/qwen.c:541-570) that matter here: C[rows x n] = A16[rows x k] * W[n x k]^T, sa = the
 * scale slot of A's fp16 cast (MDA_PC_NO_SLOT: scale 1). */
struct moe_pc_dense_t { uint32_t rows, n, k, sa; };
typedef struct mda_pc_moe_route_t moe_pc_route_t;
typedef struct mda_pc_moe_scan_t moe_pc_scan_t;
typedef struct mda_pc_moe_scatter_t moe_pc_scatter_t;
typedef struct mda_pc_moe_mm_t moe_pc_mm_t;
typedef struct mda_pc_moe_combine_t moe_pc_combine_t;
typedef struct mda_pc_qwen_elem_t moe_pc_elem_t;
typedef struct mda_pc_absmax_t moe_pc_absmax_t;
typedef struct mda_pc_cast_t moe_pc_cast_t;

/* ---- status ------------------------------------------------------------- */
enum {
    MOE_OK = 0,
    MOE_ERR_CUDA = 1,        /* a CUDA runtime/driver call failed */
    MOE_ERR_ARG = 2,         /* shape or pointer outside what the kernels accept */
    MOE_ERR_NOMEM = 3,       /* allocation refused */
    MOE_ERR_ROUTE = 4,       /* a row had fewer than topk selectable logits */
    MOE_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
    MOE_ERR_COMM = 6,        /* expert-parallel communicator failure */
    MOE_ERR_UNSUPPORTED = 7  /* device is not sm_100 */
};

typedef struct moe_cuda_ctx moe_cuda_ctx_t;

/* mda_vkc_init (src/vkc.c:95-161): bind one device and one in-order queue.
 * stream = an existing cudaStream_t to enqueue on, or NULL to create one.
 * Returns NULL only if the context object itself cannot be made; otherwise
 * check moe_cuda_status(). */
moe_cuda_ctx_t *moe_cuda_create(int device, void *stream);
void moe_cuda_destroy(moe_cuda_ctx_t *c);
/* c->fail (src/vkc.h:47): sticky.  Also folds in device-reported refusals
 * (MOE_ERR_ROUTE, MOE_ERR_TIMEOUT) seen so far; call after moe_cuda_flush for
 * a definitive answer. */
int moe_cuda_status(moe_cuda_ctx_t *c);
const char *moe_cuda_last_error(moe_cuda_ctx_t *c);
void *moe_cuda_stream(moe_cuda_ctx_t *c);
/* Test hook for host-side failure injection: the n-th allocation from now
 * (1 = the next one) is refused as if the device were out of memory. */
void moe_cuda_fail_alloc_after(moe_cuda_ctx_t *c, int n);
/* Every device-side wait (a pipeline barrier inside the grouped products, a
 * cross-GPU flag in the expert-parallel layer) gives up after this many
 * nanoseconds, records MOE_ERR_TIMEOUT and lets its kernel return.  Default
 * 2 000 000 000.  (The reference blocks in vkQueueWaitIdle without a bound,
 * src/vkc.c:655-668.) */
void moe_cuda_set_wait_ns(moe_cuda_ctx_t *c, uint64_t ns);
/* Test hook: runs the cross-GPU flag barrier against a peer that never
 * signals, so that the bounded wait runs out.  Afterwards (moe_cuda_flush) the
 * status is MOE_ERR_TIMEOUT and later calls are refused; no fault, no hang. */
void moe_cuda_wait_selftest(moe_cuda_ctx_t *c);

/* ---- buffers: mda_vkc_alloc / alloc_cached / free / fill / copy / write /
 *      read / flush (src/vkc.h:80-97) ------------------------------------- */
void *moe_cuda_alloc(moe_cuda_ctx_t *c, size_t bytes);        /* device-local (src/vkc.c:363-366) */
void *moe_cuda_alloc_pinned(moe_cuda_ctx_t *c, size_t bytes); /* host, page-locked (src/vkc.c:367-374) */
void moe_cuda_free(moe_cuda_ctx_t *c, void *p);
void moe_cuda_free_pinned(moe_cuda_ctx_t *c, void *p);
void moe_cuda_fill(moe_cuda_ctx_t *c, void *dst, size_t bytes, uint32_t word);       /* src/vkc.c:803-815 */
void moe_cuda_copy(moe_cuda_ctx_t *c, void *dst, const void *src, size_t bytes);     /* device to device, src/vkc.c:791-801 */
void moe_cuda_write(moe_cuda_ctx_t *c, void *dst, const void *host_src, size_t bytes); /* enqueued; host_src must stay valid until flush unless pageable (then staged) */
void moe_cuda_read(moe_cuda_ctx_t *c, void *host_dst, const void *src, size_t bytes);  /* blocking, src/vkc.c:817-826 */
void moe_cuda_read_async(moe_cuda_ctx_t *c, void *host_dst, const void *src, size_t bytes); /* enqueued; complete after the next flush.  host_dst should be page-locked.  Lets two contexts overlap one step's copies with the other's kernels. */
void moe_cuda_flush(moe_cuda_ctx_t *c);                                                /* src/vkc.c:655-668 */

/* ---- the five kernels --------------------------------------------------- */
/* shader/moe_route.comp (bindings proj, idx, wt, count; call src/qwen.c:799-811).
 * Candidates are experts e < pc.experts (the shader scans a fixed 512).  Ties go
 * to the lower expert index.  count[] must be zero on entry (src/qwen.c:794).
 * Limits: experts <= 512, 1 <= topk <= 16, topk <= experts. */
void moe_cuda_route(moe_cuda_ctx_t *c, const float *proj, uint32_t *idx, float *wt,
                    uint32_t *count, struct mda_pc_moe_route_t pc);
/* shader/moe_scan.comp (bindings count, off, tiles; call src/qwen.c:812-821).
 * tiles[] entries of unused tiles are left as the caller filled them. */
void moe_cuda_scan(moe_cuda_ctx_t *c, const uint32_t *count, uint32_t *off, uint32_t *tiles,
                   struct mda_pc_moe_scan_t pc);
/* shader/moe_scatter.comp (bindings idx, off, fill, x16, xp, slot; call
 * src/qwen.c:822-835).  Positions inside an expert are in token order (the
 * shader's atomic order is arbitrary).  fill[] must be zero on entry and ends
 * equal to the per-expert counts, as after the shader's atomics.  Uses the
 * context's scratch memory (grown on demand). */
void moe_cuda_scatter(moe_cuda_ctx_t *c, const uint32_t *idx, const uint32_t *off,
                      uint32_t *fill, const void *x16, void *xp, uint32_t *slot,
                      struct mda_pc_moe_scatter_t pc);
/* shader/matmul_f16_moe.comp (bindings A, B, C, amax, tiles; wrapper
 * src/qwen.c:770-786).  C[m x n] fp32 = A[m x k] * B[tiles[y]][n x k]^T /
 * (scale(sa) * scale(sb)); 128-row tile y is skipped when tiles[y] == ~0.
 * Requires m % 128 == 0, n % 128 == 0, k % 8 == 0; experts_in_B bounds tiles[]. */
void moe_cuda_mm(moe_cuda_ctx_t *c, const void *A, const void *B, float *C,
                 const uint32_t *amax, const uint32_t *tiles, struct mda_pc_moe_mm_t pc,
                 uint32_t experts_in_B);
/* shader/moe_combine.comp (bindings wt, slot, y, proj, sh, inj, h; call
 * src/qwen.c:887-906).  sh == NULL drops the shared-expert term; inj == NULL
 * means inj = 0 (so hc = 1 gives the plain residual h += acc). */
void moe_cuda_combine(moe_cuda_ctx_t *c, const float *wt, const uint32_t *slot, const float *y,
                      const float *proj, const float *sh, const float *inj, float *h,
                      struct mda_pc_moe_combine_t pc);

/* No counterpart in the reference.  moe_cuda_scatter for callers that must not
 * allocate device memory on the data path: a host that gave its whole device
 * budget to weights and pre-sized buffers at start-up (the reference itself
 * allocates all scratch once, in mda_qwen_scratch, and nothing on the path
 * allocates), or a loop that cannot afford the device-wide synchronisation a
 * cudaMalloc implies.  The per-block expert table that moe_cuda_scatter keeps in
 * growable context scratch lives here in a fixed array inside the library's
 * device image, so this call performs no cudaMalloc, cudaFree or other
 * allocating call.  Same arguments and results as moe_cuda_scatter, plus the
 * expert count (idx values must be < experts).
 *  - Limit: ceil(rows*topk/64) * experts <= MOE_NOALLOC_SCATTER_WORDS; larger
 *    calls are refused with MOE_ERR_ARG (sticky, like every refusal).
 *  - Every GPU that loads the library holds the 8 MiB table until exit.
 *  - The first call on a device looks up the table's device address (a query,
 *    not an allocation); make that first call before any stream capture starts.
 *  - All calls on a device share the one table: calls that overlap on the GPU
 *    (different streams or contexts) race.  Nothing in it has to be cleared
 *    between calls; each call overwrites what it reads. */
#define MOE_NOALLOC_SCATTER_WORDS (2u << 20)
void moe_cuda_scatter_noalloc(moe_cuda_ctx_t *c, const uint32_t *idx, const uint32_t *off,
                              uint32_t *fill, const void *x16, void *xp, uint32_t *slot,
                              struct mda_pc_moe_scatter_t pc, uint32_t experts);

/* ---- glue kernels between the two grouped products (unfused mode) ------- */
void moe_cuda_swiglu(moe_cuda_ctx_t *c, const float *a, float *y, struct mda_pc_qwen_elem_t pc); /* shader/qwen_elem.comp op 0, src/qwen.c:848-857 */
void moe_cuda_absmax(moe_cuda_ctx_t *c, const float *x, uint32_t *amax, struct mda_pc_absmax_t pc); /* shader/absmax.comp, src/qwen.c:858-867 */
void moe_cuda_cast_f16(moe_cuda_ctx_t *c, const float *src, void *dst, const uint32_t *amax,
                       struct mda_pc_cast_t pc); /* shader/cast_f16.comp, src/qwen.c:868-877 */

/* ---- the steps either side of the MoE path ---------------------------------
 * The hyper-connection residual mixer that produces a layer's input x and the
 * injection scalars the combine reads (mda_qwen_res_rec, src/qwen.c:641-663),
 * and the teacher's head (mda_qwen_head, src/qwen.c:1080-1099: the same mixer,
 * a cast, the vocabulary product in row chunks, then the sink below).
 * moe_cuda_swiglu above also takes op 1 of shader/qwen_elem.comp (silu(scale*a)),
 * moe_cuda_absmax + moe_cuda_cast_f16 are mda_qwen_cast (src/qwen.c:517-539). */
/* shader/qwen_norm.comp (bindings x, w, y, z), ops 0 and 1: grouped RMSNorm with
 * weight 1 + w (op 0), or x * scale / sqrt(sum x^2 + 1e-6) (op 1).  z is unused
 * by these ops and may be NULL. */
void moe_cuda_norm(moe_cuda_ctx_t *c, const float *x, const float *w, float *y, const float *z,
                   struct mda_pc_qwen_norm_t pc);
/* shader/qwen_hc.comp (bindings a, b, h): op 0 the mixer's read-out, op 1 the
 * stream injection, op 2 h += a + b (mda_qwen_hc, src/qwen.c:615-631). */
void moe_cuda_hc(moe_cuda_ctx_t *c, const float *a, const float *b, float *h, struct mda_pc_qwen_hc_t pc);
/* mda_qwen_mm (src/qwen.c:541-570; shader/matmul_f16_wide.comp and the small-tile
 * kernel it alternates with): dense fp16 x fp16 -> fp32 product on the tcgen05
 * kernel of the grouped products.  n % 128 == 0, k % 8 == 0; any rows >= 1. */
void moe_cuda_dense(moe_cuda_ctx_t *c, const void *A16, const void *W, float *C, const uint32_t *amax,
                    struct moe_pc_dense_t pc);

/* ---- weight upload step ---------------------------------------------------
 * shader/qwen_bf16.comp (binding w; call mda_qwen_convert, src/qwen.c:365-378):
 * pc.n 32-bit words of two bf16 values each, rewritten in place as fp16 (round
 * to nearest even) right after the host-to-device copy of a layer's weights. */
void moe_cuda_bf16_to_f16(moe_cuda_ctx_t *c, void *w, struct mda_pc_qwen_bf16_t pc);

/* ---- distillation sink behind the teacher's head --------------------------
 * shader/kd_bytes.comp (bindings logits, toks, cont, outp; call mda_teach_sink,
 * src/teach.c:108-128).  logits fp32 [rows x vocab]; toks [vocab x 5] u32: 16
 * bytes of the token (little-endian in four words) and its length, 0 = no byte
 * string; cont [rows x 5]: the 16 bytes that follow the row's position and how
 * many of them count; outp [rows x 16 x 8] entries byte | fp16(p) << 16 -- per
 * depth the true byte's probability, then the seven most probable other bytes. */
void moe_cuda_kd_bytes(moe_cuda_ctx_t *c, const float *logits, const uint32_t *toks, const uint32_t *cont,
                       uint32_t *outp, struct mda_pc_kd_bytes_t pc);

/* ---- the fused layer: mda_qwen_route_rec + mda_qwen_moe_rec from the first
 *      grouped product on (src/qwen.c:788-836, 847-906) in one call --------- */
typedef struct moe_cuda_layer_t {
    uint32_t rows, d, experts, topk, inter, shared; /* shared = 0: no shared expert */
    uint32_t pstride;      /* row stride of proj; shared gate logit at column `experts` */
    uint32_t hc;           /* residual streams; 1 = plain residual */
    uint32_t inj_stride, inj_off;
    const float *proj;     /* [rows x pstride] fp32 */
    const void *x16;       /* [rows x d] fp16 */
    const void *wgu;       /* [experts][2*inter x d] fp16: gate rows then up rows */
    const void *wdown;     /* [experts][d x inter] fp16 */
    const void *wsgu;      /* [2*shared x d] fp16 or NULL */
    const void *wsdown;    /* [d x shared] fp16 or NULL */
    const float *inj;      /* or NULL */
    float *h;              /* [rows x hc x d] fp32, accumulated into */
    /* optional outputs for inspection (NULL = kept in context scratch) */
    uint32_t *idx, *slot, *count, *off, *tiles;
    float *wt;
    /* optional: y16 [rows x d] fp16 = RMSNorm(x16 + moe(x)) with unit weight;
     * when set, h may be NULL.  (Residual + norm between stacked layers.) */
    void *y16;
    float eps;
    uint32_t flags;        /* MOE_LAYER_* */
} moe_cuda_layer_t;
#define MOE_LAYER_UNFUSED 1u /* run the reference's kernel sequence step by step (fp32 g, absmax rescale) */
#define MOE_LAYER_YE_F32 2u  /* keep expert outputs fp32 between the down product and the combine */
#define MOE_LAYER_CHUNKED 4u /* weight-stationary products over per-expert token chunks (MMA width rounded to 16, tcgen05 cta_group::2 pairs): the default whenever d % 128 == 0, so the flag only states it */
#define MOE_LAYER_NO_PAIR 8u /* weight-stationary products with one CTA per tile instead of tcgen05 cta_group::2 pairs */
#define MOE_LAYER_MATERIALIZE_XP 16u /* with MOE_LAYER_TILED: write the permuted activations xp to HBM as the reference does, instead of letting the gate_up product gather the rows of x16 itself */
#define MOE_LAYER_TILED 32u /* the reference's 128-row tile schedule (shader/matmul_f16_moe.comp) for both products instead of the weight-stationary chunks */

/* Rows of scratch the layer needs: round128(rows*topk + experts*127), src/qwen.c:68-70. */
uint32_t moe_cuda_moe_rows(uint32_t rows, uint32_t topk, uint32_t experts);
void moe_cuda_layer(moe_cuda_ctx_t *c, const moe_cuda_layer_t *L);

/* ---- expert parallel over the GPUs of one box (no counterpart in the
 *      reference, which keeps all experts of a layer on one device,
 *      src/qwen.c:235-246) ------------------------------------------------
 * One process per GPU.  Rank g owns experts [g*E/G, (g+1)*E/G) and passes only
 * their weights; every rank passes its own tokens.  Dispatch is fused into the
 * scatter (peer stores of each pair's row into the owner's expert-contiguous
 * buffer) and return into the combine (peer loads of each pair's output row);
 * or, with MOE_EP_TRANSFER_PER_GPU, each token row is stored once into the
 * receive buffer of every GPU that owns one of its experts plus small records
 * per pair, the owner's gate_up product gathers through those records, and the
 * owner returns one weighted partial row per token.  All of it is plain peer
 * stores / loads over NVLink; the per-expert counts and the three rendezvous points per layer are
 * flag exchanges over the same peer memory with bounded waits (a rank that
 * stops coming ends the others' call with MOE_ERR_TIMEOUT after 2 s).  NCCL is
 * needed once, at moe_cuda_ep_init, to hand round the memory handles. */
typedef struct moe_cuda_ep_cfg_t {
    uint32_t experts, topk, d, inter; /* global expert count; experts % world == 0, inter % 128 == 0 */
    uint32_t max_rows;                /* most tokens any rank will pass in one call */
    uint32_t micro_batches;           /* 1 to 4 slices of the local tokens (equal parts rounded up to 8 rows) that pipeline
                                         NVLink transfers against the products, each on its own stream;
                                         0 = automatic (2 with per-pair transfers over 4 or more ranks, else 1) */
    uint32_t transfer;                /* MOE_EP_TRANSFER_*: what crosses NVLink */
} moe_cuda_ep_cfg_t;
#define MOE_EP_TRANSFER_AUTO 0u     /* PER_GPU up to 4 ranks, PER_PAIR beyond (measured crossover on B200) */
#define MOE_EP_TRANSFER_PER_PAIR 1u /* one row per (token, expert) pair each way, written into / read from the owner's expert-contiguous buffers */
#define MOE_EP_TRANSFER_PER_GPU 2u  /* one row per (token, owning GPU) each way: the owner gathers its operand through a source-row table and returns one weighted partial row per token */
/* 128 bytes of NCCL unique id: call on one rank, hand the bytes to all. */
int moe_cuda_ep_unique_id(void *out128);
/* Rows of each rank's expert-contiguous buffers: sized for the worst case
 * (every token of every rank routed to this rank), so no token is ever dropped. */
uint32_t moe_cuda_ep_rows(uint32_t world, uint32_t max_rows, uint32_t experts, uint32_t topk);
/* Collective: joins the communicator, allocates and cross-maps the buffers.
 * All ranks succeed or fail together once the communicator exists.
 * moe_cuda_destroy of such a context is collective too: peers read and write
 * this rank's buffers, so every rank runs one more bounded flag barrier before
 * the memory is freed.  A context that has failed frees only what no peer can
 * reach and leaves its peer-visible buffers to process exit. */
void moe_cuda_ep_init(moe_cuda_ctx_t *c, const void *unique_id128, int rank, int world,
                      const moe_cuda_ep_cfg_t *cfg);
/* Collective: one MoE layer.  L->rows = this rank's tokens, L->experts = global
 * expert count, L->wgu / L->wdown = this rank's experts only.  L->slot receives
 * row numbers inside the owning rank's buffer (of the token's micro-batch),
 * L->off (one micro-batch only) this rank's first row per expert there.  The
 * shared expert (L->shared, L->wsgu, L->wsdown: replicated weights) runs on
 * every rank's own tokens and enters the combine as in the single-GPU layer
 * (src/qwen.c:879-886, shader/moe_combine.comp:35).  L->tiles and the flags
 * are not supported. */
void moe_cuda_ep_layer(moe_cuda_ctx_t *c, const moe_cuda_layer_t *L);

/* Per-stage device times of the last moe_cuda_layer call, in milliseconds, in
 * the order route, scan, scatter, gate_up, down, shared, combine (for
 * moe_cuda_ep_layer: router, counts + plan, dispatch + barrier (+ the shared
 * expert), gate_up, down, barrier, combine + return; with several token slices
 * each stage is the sum of the slices' times, every slice timed on its own
 * stream) (after
 * mda_vkc_prof_begin / prof_report, src/vkc.c:595-653).  Enabled with
 * moe_cuda_prof(c, 1); reading them synchronises the stream. */
#define MOE_PROF_STAGES 7
void moe_cuda_prof(moe_cuda_ctx_t *c, int on);
void moe_cuda_prof_read(moe_cuda_ctx_t *c, float ms[MOE_PROF_STAGES]);
/* Number of kernels this library has launched on the context so far. */
uint64_t moe_cuda_launches(moe_cuda_ctx_t *c);

#ifdef __cplusplus
}
#endif
#endif
