// Expert-parallel MoE layer over the GPUs of one box: one process per GPU,
// experts split contiguously (rank g owns experts [g*E/G, (g+1)*E/G)), tokens
// stay on their home GPU.  The reference is single-GPU (all experts of a layer
// live in one buffer, src/qwen.c:235-246); the result here must equal the
// single-GPU layer's.
//
// The two all-to-alls are fused into the kernels on either side of them instead
// of being library calls, in one of two schemes (moe_cuda_ep_cfg_t.transfer):
//   per pair: dispatch = the scatter kernel writes each (token, expert) pair's row
//             straight into the owning GPU's expert-contiguous buffer (peer stores
//             over NVLink); return = the combine kernel gathers each pair's output
//             row straight from the owning GPU's buffer (peer loads);
//   per GPU:  a token row crosses NVLink once per destination GPU, however many of
//             its experts live there: the send kernel stores it into that GPU's
//             receive buffer (slot = source rank, token), the scatter kernel stores,
//             for every pair, only a 4-byte record into the owner's source-row
//             table, and the owner's gate_up product gathers its operand rows
//             through that table.  The same the other way round: the owner sums
//             wt * (expert output row) over the token's experts it holds
//             (moe_ep_partial_kernel, from 8-byte records the scatter kernel stored
//             beside the source-row records) and the home GPU's combine kernel
//             loads that one fp16 partial row per owning GPU, adding the partial
//             rows in ascending GPU order.
// Peer buffers are plain cudaMalloc memory mapped with CUDA IPC; all accesses
// are ordinary ld/st (no multimem, no TMA from peer memory: the grouped
// products only ever read local HBM).  The per-expert counts travel the same way
// (each rank stores its row into every peer's table) and the three points where
// all ranks must have caught up -- counts complete, all rows landed, all products
// done -- are flag barriers over peer memory with bounded waits.  NCCL is used
// once, at set-up, to exchange the IPC handles.
//
// With top-8 routing over 8 GPUs a token has 7 remote expert copies but only 4.6
// distinct remote GPUs on average; over 2 GPUs 4 copies but 1 GPU.  The per-GPU
// scheme pays for the saved bytes with the owner-side sums and a gathering
// product; it is the default up to 4 GPUs, where it measured faster.
//
// Row order inside an expert is (source rank, token index); with contiguous
// token blocks per rank that is the global token order, so the permutation is
// the single-GPU one restricted to the expert.
#include <dlfcn.h>
#include <nccl.h>
#include <stdlib.h>
#include <string.h>

#include "moe_common.cuh"

struct moe_nccl_api {
    void *handle;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *);
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    ncclResult_t (*CommAbort)(ncclComm_t);
    const char *(*GetErrorString)(ncclResult_t);
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t);
    ncclResult_t (*AllReduce)(const void *, void *, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t);
};

static moe_nccl_api g_nccl;

static bool moe_nccl_load(char *why, size_t n) {
    if (g_nccl.handle != NULL) return true;
    void *h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);  // reuses a copy the process already loaded
    if (h == NULL) {
        snprintf(why, n, "libnccl.so.2 not loadable: %s", dlerror());
        return false;
    }
#define MOE_SYM(field, name)                                  \
    *(void **)(&g_nccl.field) = dlsym(h, name);               \
    if (g_nccl.field == NULL) {                               \
        snprintf(why, n, "libnccl.so.2 lacks %s", name);      \
        return false;                                         \
    }
    MOE_SYM(GetUniqueId, "ncclGetUniqueId")
    MOE_SYM(CommInitRank, "ncclCommInitRank")
    MOE_SYM(CommDestroy, "ncclCommDestroy")
    MOE_SYM(CommAbort, "ncclCommAbort")
    MOE_SYM(GetErrorString, "ncclGetErrorString")
    MOE_SYM(AllGather, "ncclAllGather")
    MOE_SYM(AllReduce, "ncclAllReduce")
#undef MOE_SYM
    g_nccl.handle = h;
    return true;
}

#define MOE_EP_MAX_WORLD 16
#define EP_FLAG_WORDS 256u  // 16 barrier sites x 16 ranks of epoch flags: 3 per micro-batch, the last one for teardown

#define EP_MAX_MB 4  // micro-batches per layer call

struct moe_ep_state {
    ncclComm_t comm;
    int rank, world;
    moe_cuda_ep_cfg_t cfg;
    uint32_t el;          // experts per rank
    uint32_t nmb;         // micro-batches: the local tokens are cut in nmb parts that pipeline transfer against products
    uint32_t mcap;        // rows of the expert-contiguous buffers of ONE micro-batch
    uint32_t cap;         // token rows one rank may send per micro-batch
    bool per_gpu;         // transfer scheme: rows cross NVLink once per (token, GPU) instead of once per (token, expert)
    uint32_t in_rows;     // rows per micro-batch of the two peer-visible buffers: world * cap (per_gpu) or mcap
    // xin: peer-visible operand rows (per_gpu: received rows, slot = (source rank, token); else expert-contiguous);
    // yout: peer-visible result rows (per_gpu: one partial row per received token; else the down product's output);
    // ye: the down product's output when it is not yout (per_gpu only); hp16 [nmb * mcap x inter]
    __half *xin, *yout, *ye, *hp16;
    void *xin_peer[MOE_EP_MAX_WORLD];     // every rank's xin as mapped here (own entry = local pointer)
    void *yout_peer[MOE_EP_MAX_WORLD];
    void **xin_peer_dev[EP_MAX_MB], **yout_peer_dev[EP_MAX_MB];  // per micro-batch: each rank's buffer of that micro-batch
    void **srow_peer_dev[EP_MAX_MB];     // per micro-batch: each rank's source-row table (inside its sync buffer)
    void **ret_peer_dev[EP_MAX_MB];      // per micro-batch: each rank's return-record table (inside its sync buffer)
    uint32_t *src_row[EP_MAX_MB];        // own tables: expert-contiguous row -> row of xr (~0: padding)
    uint2 *ret_tab[EP_MAX_MB];           // own tables: [world * cap][topk] (output row, weight) per received token, ~0 ends a list
    uint32_t *sync;                      // peer-visible: 6 x 16 epoch flags, nmb tables [world][experts] of counts, nmb source-row tables [mcap], nmb return tables
    void *sync_peer[MOE_EP_MAX_WORLD];
    void **sync_peer_dev;
    uint32_t epoch;
    uint32_t *dst_off[EP_MAX_MB];        // [experts]: first row of this rank's rows in the owner's buffer
    uint32_t *tiles[EP_MAX_MB];          // [mcap/128] local tile schedule
    uint32_t *count[EP_MAX_MB];
    // weight-stationary products: per micro-batch [el] rows per local expert, [el] first rows, 16 words (chunk count), chunk list
    uint32_t *wsbuf[EP_MAX_MB];
    uint32_t max_chunks;
    uint32_t *idx, *slot, *bar;
    float *wt;
    cudaStream_t side[EP_MAX_MB];        // streams of micro-batches 1.. (micro-batch 0 runs on the context's stream)
    cudaEvent_t ev_fork, ev_disp[EP_MAX_MB], ev_join[EP_MAX_MB];
    bool streams_made;
};

#define MOE_NCCL_TRY(c, expr)                                                                   \
    do {                                                                                        \
        ncclResult_t r__ = (expr);                                                              \
        if (r__ != ncclSuccess) {                                                               \
            moe_fail((c), MOE_ERR_COMM, "%s:%d: NCCL: %s", __FILE__, __LINE__, g_nccl.GetErrorString(r__)); \
            return;                                                                             \
        }                                                                                       \
    } while (0)

extern "C" int moe_cuda_ep_unique_id(void *out128) {
    char why[200];
    if (out128 == NULL || !moe_nccl_load(why, sizeof(why))) return MOE_ERR_COMM;
    ncclUniqueId id;
    if (g_nccl.GetUniqueId(&id) != ncclSuccess) return MOE_ERR_COMM;
    memcpy(out128, &id, sizeof(id));
    return MOE_OK;
}

extern "C" uint32_t moe_cuda_ep_rows(uint32_t world, uint32_t max_rows, uint32_t experts, uint32_t topk) {
    // Worst case one rank can be sent: every token of every rank picks min(topk, E/G) of its experts.
    if (world == 0 || experts % world != 0) return 0;
    uint32_t el = experts / world;
    uint64_t rows = (uint64_t)world * max_rows * (topk < el ? topk : el) + (uint64_t)el * (MOE_TILE - 1u);
    rows = (rows + MOE_TILE - 1u) / MOE_TILE * MOE_TILE;
    return rows < (1ull << 31) ? (uint32_t)rows : 0;
}

__global__ void moe_ep_barrier_kernel(uint32_t *const *sync_peers, uint32_t world, uint32_t rank, uint32_t site, uint32_t epoch,
                                      uint32_t *status, uint64_t wait_ns);

// Destroying an expert-parallel context is collective: peers write into and read
// from this rank's xin / yout / sync buffers, so they must all have finished
// their last layer before the memory goes away.  A healthy context runs one more
// bounded flag barrier (its own site) first.  A failed context cannot know what
// its peers still have in flight: it closes its mappings of their memory but
// leaves its own exported buffers allocated until the process exits.
#define EP_SITE_TEARDOWN 15u
void moe_ep_teardown(moe_cuda_ctx *c) {
    if (c == NULL || c->ep == NULL) return;
    moe_ep_state *ep = c->ep;
    bool mapped = ep->sync_peer_dev != NULL && ep->sync != NULL;
    for (int r = 0; r < ep->world && mapped; r += 1) mapped = ep->sync_peer[r] != NULL;
    bool rendezvous = false;
    if (c->stream != NULL && c->status == MOE_OK && mapped && ep->world > 1) {
        ep->epoch += 1;
        moe_ep_barrier_kernel<<<1, 32, 0, c->stream>>>((uint32_t *const *)ep->sync_peer_dev, (uint32_t)ep->world, (uint32_t)ep->rank,
                                                       EP_SITE_TEARDOWN, ep->epoch, c->dev_status_dev, c->wait_ns);
        rendezvous = cudaStreamSynchronize(c->stream) == cudaSuccess && moe_poll_device_status(c);
    } else if (c->stream != NULL) {
        cudaStreamSynchronize(c->stream);
        rendezvous = ep->world == 1 && c->status == MOE_OK;
    }
    for (int r = 0; r < ep->world; r += 1) {
        if (r == ep->rank) continue;
        if (ep->xin_peer[r] != NULL) cudaIpcCloseMemHandle(ep->xin_peer[r]);
        if (ep->yout_peer[r] != NULL) cudaIpcCloseMemHandle(ep->yout_peer[r]);
        if (ep->sync_peer[r] != NULL) cudaIpcCloseMemHandle(ep->sync_peer[r]);
    }
    void *mine[10 + 8 * EP_MAX_MB] = {ep->xin, ep->yout, ep->ye, ep->hp16, ep->sync_peer_dev, ep->sync, ep->idx, ep->slot};
    size_t n_mine = 8;
    mine[n_mine++] = ep->bar;
    mine[n_mine++] = ep->wt;
    for (uint32_t m = 0; m < EP_MAX_MB; m += 1) {
        void *per[] = {ep->xin_peer_dev[m], ep->yout_peer_dev[m], ep->srow_peer_dev[m], ep->ret_peer_dev[m], ep->dst_off[m], ep->tiles[m], ep->count[m], ep->wsbuf[m]};
        for (size_t i = 0; i < sizeof(per) / sizeof(per[0]) && n_mine < sizeof(mine) / sizeof(mine[0]); i += 1) mine[n_mine++] = per[i];
    }
    if (ep->streams_made) {
        cudaEventDestroy(ep->ev_fork);
        for (uint32_t m = 0; m < ep->nmb; m += 1) {
            if (m != 0 && ep->side[m] != NULL) {
                cudaStreamSynchronize(ep->side[m]);
                cudaStreamDestroy(ep->side[m]);
            }
            if (ep->ev_disp[m] != NULL) cudaEventDestroy(ep->ev_disp[m]);
            if (ep->ev_join[m] != NULL) cudaEventDestroy(ep->ev_join[m]);
        }
    }
    for (size_t i = 0; i < n_mine; i += 1) {
        const bool exported = mine[i] == (void *)ep->xin || mine[i] == (void *)ep->yout || mine[i] == (void *)ep->sync;
        if (mine[i] != NULL && (rendezvous || !exported)) cudaFree(mine[i]);
    }
    if (ep->comm != NULL) {
        if (c->status == MOE_OK) g_nccl.CommDestroy(ep->comm);
        else g_nccl.CommAbort(ep->comm);  // a failed rank must not wait for its peers
    }
    free(ep);
    c->ep = NULL;
}

__global__ void moe_ep_plan_kernel(const uint32_t *__restrict__ my_count, uint32_t *const *sync_peers, uint32_t epoch, uint32_t site,
                                   uint32_t table_off, uint32_t *__restrict__ dst_off, uint32_t *__restrict__ tiles,
                                   uint32_t experts, uint32_t world, uint32_t rank, uint32_t el, uint32_t mcap, uint32_t *status,
                                   uint64_t wait_ns, uint32_t *__restrict__ lcount, uint32_t *__restrict__ loff);

__global__ void moe_ep_send_kernel(const uint32_t *__restrict__ idx, const uint4 *__restrict__ x16, uint4 *const *__restrict__ xin_peers,
                                   uint32_t rows, uint32_t topk, uint32_t d8, uint32_t el, uint32_t world, uint32_t src_base);

__global__ void moe_ep_partial_kernel(const uint2 *__restrict__ ret_tab, const uint4 *__restrict__ ye, uint4 *__restrict__ part,
                                      uint32_t slots, uint32_t topk, uint32_t d8);

// Per-GPU scheme, owner side: the received rows (one per token) copied into expert order, one warp per row, so that
// the weight-stationary gate_up product can load them as tiles.  Padding rows (~0) are left as they are: a padding
// row only ever feeds padding rows.
__global__ void __launch_bounds__(256)
moe_ep_permute_kernel(const uint32_t *__restrict__ src_row, const uint4 *__restrict__ xin, uint4 *__restrict__ xp, uint32_t rows,
                      uint32_t d8) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t p = warp; p < rows; p += nwarps) {
        const uint32_t src = src_row[p];
        if (src == ~0u) continue;
        const uint4 *in = xin + (size_t)src * d8;
        uint4 *out = xp + (size_t)p * d8;
        for (uint32_t c0 = lane; c0 < d8; c0 += 32u) out[c0] = __ldg(in + c0);
    }
}

// Joins the communicator, allocates the peer-visible buffers for the stated
// maximum shape and maps every peer's buffers.  Collective over all ranks.
extern "C" void moe_cuda_ep_init(moe_cuda_ctx_t *c, const void *unique_id128, int rank, int world,
                                 const moe_cuda_ep_cfg_t *cfg) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, c->ep == NULL, "ep_init: already initialised");
    MOE_REQUIRE(c, unique_id128 != NULL && cfg != NULL, "ep_init: null argument");
    MOE_REQUIRE(c, world >= 1 && world <= MOE_EP_MAX_WORLD && rank >= 0 && rank < world, "ep_init: rank %d of %d", rank, world);
    MOE_REQUIRE(c, cfg->experts >= 1 && cfg->experts <= MOE_MAX_EXPERTS && cfg->experts % (uint32_t)world == 0,
                "ep_init: experts %u not divisible by world %d", cfg->experts, world);
    MOE_REQUIRE(c, cfg->topk >= 1 && cfg->topk <= MOE_MAX_TOPK && cfg->d % 8 == 0 && cfg->inter % 128 == 0 && cfg->max_rows >= 1,
                "ep_init: bad shape");
    char why[200];
    if (!moe_nccl_load(why, sizeof(why))) {
        moe_fail(c, MOE_ERR_COMM, "%s", why);
        return;
    }
    MOE_REQUIRE(c, cfg->micro_batches <= EP_MAX_MB, "ep_init: micro_batches %u > %d", cfg->micro_batches, EP_MAX_MB);
    MOE_REQUIRE(c, cfg->transfer <= MOE_EP_TRANSFER_PER_GPU, "ep_init: transfer %u", cfg->transfer);
    // Measured on B200 (30B-A3B shape, 4096 tokens per GPU, ms per layer): once-per-GPU transfers win
    // at 2 GPUs (0.512 against 0.588) and at 4 (0.610 against 0.642), per-pair transfers at 8 (0.672
    // against 0.754: 4.6 of 7 rows still travel, and the owner-side sums and the gathering product
    // cost more than the saved bytes).
    const bool per_gpu = cfg->transfer == MOE_EP_TRANSFER_AUTO ? world <= 4 : cfg->transfer == MOE_EP_TRANSFER_PER_GPU;
    // micro_batches 0 = automatic: with per-pair transfers over 4 or more ranks most rows cross NVLink,
    // and cutting the tokens in two lets one half's transfers run under the other half's products
    // (0.672 against 0.712 at 8 GPUs); with per-GPU transfers one slice measured faster (0.610
    // against 0.617 at 4 GPUs, 0.512 against 0.572 at 2)
    uint32_t nmb = cfg->micro_batches != 0 ? cfg->micro_batches : ((world >= 4 && !per_gpu) ? 2u : 1u);
    uint32_t rows_mb = nmb == 1 ? cfg->max_rows : (((cfg->max_rows + nmb - 1u) / nmb + 7u) & ~7u);
    uint32_t mcap = moe_cuda_ep_rows((uint32_t)world, rows_mb, cfg->experts, cfg->topk);
    MOE_REQUIRE(c, mcap != 0, "ep_init: buffer rows overflow");
    moe_ep_state *ep = (moe_ep_state *)calloc(1, sizeof(moe_ep_state));
    if (ep == NULL) {
        moe_fail(c, MOE_ERR_NOMEM, "ep_init: host allocation");
        return;
    }
    c->ep = ep;
    ep->rank = rank;
    ep->world = world;
    ep->cfg = *cfg;
    ep->el = cfg->experts / (uint32_t)world;
    ep->mcap = mcap;
    ep->cap = rows_mb;
    ep->nmb = nmb;
    ncclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    MOE_NCCL_TRY(c, g_nccl.CommInitRank(&ep->comm, world, id, rank));

    size_t R = cfg->max_rows, K = cfg->topk, E = cfg->experts;
    const size_t srow_words0 = EP_FLAG_WORDS + (size_t)nmb * world * E;
    const size_t ret_words0 = (srow_words0 + (size_t)nmb * mcap + 1u) & ~(size_t)1u;  // 8-byte records
    const size_t ret_words = (size_t)world * rows_mb * K * 2u;                          // per micro-batch
    const size_t sync_words = ret_words0 + (size_t)nmb * ret_words;
    ep->per_gpu = per_gpu;
    ep->in_rows = ep->per_gpu ? (uint32_t)world * rows_mb : mcap;
    ep->xin = (__half *)moe_cuda_alloc(c, (size_t)nmb * ep->in_rows * cfg->d * 2);
    ep->yout = (__half *)moe_cuda_alloc(c, (size_t)nmb * ep->in_rows * cfg->d * 2);
    ep->ye = ep->per_gpu ? (__half *)moe_cuda_alloc(c, (size_t)nmb * mcap * cfg->d * 2) : NULL;
    ep->hp16 = (__half *)moe_cuda_alloc(c, (size_t)nmb * mcap * cfg->inter * 2);
    ep->sync = (uint32_t *)moe_cuda_alloc(c, sync_words * 4);
    ep->sync_peer_dev = (void **)moe_cuda_alloc(c, MOE_EP_MAX_WORLD * sizeof(void *));
    for (uint32_t m = 0; m < nmb; m += 1) {
        ep->xin_peer_dev[m] = (void **)moe_cuda_alloc(c, MOE_EP_MAX_WORLD * sizeof(void *));
        ep->srow_peer_dev[m] = (void **)moe_cuda_alloc(c, MOE_EP_MAX_WORLD * sizeof(void *));
        ep->yout_peer_dev[m] = (void **)moe_cuda_alloc(c, MOE_EP_MAX_WORLD * sizeof(void *));
        ep->ret_peer_dev[m] = (void **)moe_cuda_alloc(c, MOE_EP_MAX_WORLD * sizeof(void *));
        ep->dst_off[m] = (uint32_t *)moe_cuda_alloc(c, E * 4);
        ep->tiles[m] = (uint32_t *)moe_cuda_alloc(c, (size_t)(mcap / MOE_TILE) * 4);
        ep->count[m] = (uint32_t *)moe_cuda_alloc(c, E * 4);
        ep->wsbuf[m] = (uint32_t *)moe_cuda_alloc(c, ((size_t)2 * ep->el + 16) * 4 + 16 + (size_t)(mcap / 256u + ep->el + 1u) * 16);
    }
    ep->max_chunks = mcap / 256u + ep->el + 1u;
    ep->idx = (uint32_t *)moe_cuda_alloc(c, R * K * 4);
    ep->slot = (uint32_t *)moe_cuda_alloc(c, R * K * 4);
    ep->wt = (float *)moe_cuda_alloc(c, R * K * 4);
    ep->bar = (uint32_t *)moe_cuda_alloc(c, 256);
    {
        // Every rank reaches this reduction whether or not its allocations succeeded, so that a rank
        // that ran out of memory makes all ranks return an error together instead of leaving the
        // others inside the handle exchange.
        uint32_t *agree = NULL;
        uint32_t flag[2] = {c->status == MOE_OK ? 0u : 1u, 0u};
        bool ran = cudaMalloc((void **)&agree, 64) == cudaSuccess &&
                   cudaMemcpyAsync(agree, flag, 8, cudaMemcpyHostToDevice, c->stream) == cudaSuccess &&
                   g_nccl.AllReduce(agree, agree + 1, 1, ncclUint32, ncclSum, ep->comm, c->stream) == ncclSuccess &&
                   cudaMemcpyAsync(flag, agree, 8, cudaMemcpyDeviceToHost, c->stream) == cudaSuccess &&
                   cudaStreamSynchronize(c->stream) == cudaSuccess;
        if (agree != NULL) cudaFree(agree);
        if (!ran) moe_fail(c, MOE_ERR_COMM, "ep_init: the ranks could not agree on their set-up");
        else if (flag[1] != 0) moe_fail(c, MOE_ERR_COMM, "ep_init: %u rank(s) failed to allocate their buffers", flag[1]);
    }
    if (c->status != MOE_OK) return;
    if (nmb > 1) {
        // the transfer kernels of one slice must be able to run on SMs that hold a product CTA of the other
        moe_overlap_prepare_combine(c);
        moe_overlap_prepare_scatter(c);
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_ep_send_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_ep_partial_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_ep_barrier_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_ep_plan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        if (c->status != MOE_OK) return;
        ep->streams_made = true;
        MOE_CUDA_TRY(c, cudaEventCreateWithFlags(&ep->ev_fork, cudaEventDisableTiming));
        for (uint32_t m = 0; m < nmb; m += 1) {
            if (m != 0) MOE_CUDA_TRY(c, cudaStreamCreateWithFlags(&ep->side[m], cudaStreamNonBlocking));
            MOE_CUDA_TRY(c, cudaEventCreateWithFlags(&ep->ev_disp[m], cudaEventDisableTiming));
            MOE_CUDA_TRY(c, cudaEventCreateWithFlags(&ep->ev_join[m], cudaEventDisableTiming));
        }
    }
    MOE_CUDA_TRY(c, cudaMemsetAsync(ep->bar, 0, 256, c->stream));
    MOE_CUDA_TRY(c, cudaMemsetAsync(ep->sync, 0, sync_words * 4, c->stream));

    // Exchange the IPC handles of xin, yout and sync through the communicator itself.
    struct Handles {
        cudaIpcMemHandle_t xin, yout, sync;
    };
    Handles mine;
    MOE_CUDA_TRY(c, cudaIpcGetMemHandle(&mine.xin, ep->xin));
    MOE_CUDA_TRY(c, cudaIpcGetMemHandle(&mine.yout, ep->yout));
    MOE_CUDA_TRY(c, cudaIpcGetMemHandle(&mine.sync, ep->sync));
    Handles *d_all = (Handles *)moe_cuda_alloc(c, sizeof(Handles) * (size_t)world);
    if (d_all == NULL) return;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(d_all + rank, &mine, sizeof(mine), cudaMemcpyHostToDevice, c->stream));
    MOE_NCCL_TRY(c, g_nccl.AllGather(d_all + rank, d_all, sizeof(Handles), ncclUint8, ep->comm, c->stream));
    Handles all[MOE_EP_MAX_WORLD];
    MOE_CUDA_TRY(c, cudaMemcpyAsync(all, d_all, sizeof(Handles) * (size_t)world, cudaMemcpyDeviceToHost, c->stream));
    MOE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    cudaFree(d_all);
    for (int r = 0; r < world; r += 1) {
        if (r == rank) {
            ep->xin_peer[r] = ep->xin;
            ep->yout_peer[r] = ep->yout;
            ep->sync_peer[r] = ep->sync;
            continue;
        }
        MOE_CUDA_TRY(c, cudaIpcOpenMemHandle(&ep->xin_peer[r], all[r].xin, cudaIpcMemLazyEnablePeerAccess));
        MOE_CUDA_TRY(c, cudaIpcOpenMemHandle(&ep->yout_peer[r], all[r].yout, cudaIpcMemLazyEnablePeerAccess));
        MOE_CUDA_TRY(c, cudaIpcOpenMemHandle(&ep->sync_peer[r], all[r].sync, cudaIpcMemLazyEnablePeerAccess));
    }
    for (uint32_t m = 0; m < nmb; m += 1) {  // micro-batch m: row m * in_rows of xin and yout, tables m
        void *xt[MOE_EP_MAX_WORLD] = {}, *yt[MOE_EP_MAX_WORLD] = {}, *st[MOE_EP_MAX_WORLD] = {}, *rt[MOE_EP_MAX_WORLD] = {};
        for (int r = 0; r < world; r += 1) {
            xt[r] = (__half *)ep->xin_peer[r] + (size_t)m * ep->in_rows * cfg->d;
            yt[r] = (__half *)ep->yout_peer[r] + (size_t)m * ep->in_rows * cfg->d;
            st[r] = (uint32_t *)ep->sync_peer[r] + srow_words0 + (size_t)m * mcap;
            rt[r] = (uint32_t *)ep->sync_peer[r] + ret_words0 + (size_t)m * ret_words;
        }
        ep->src_row[m] = ep->sync + srow_words0 + (size_t)m * mcap;
        ep->ret_tab[m] = (uint2 *)(ep->sync + ret_words0 + (size_t)m * ret_words);
        MOE_CUDA_TRY(c, cudaMemcpy(ep->xin_peer_dev[m], xt, sizeof(xt), cudaMemcpyHostToDevice));
        MOE_CUDA_TRY(c, cudaMemcpy(ep->yout_peer_dev[m], yt, sizeof(yt), cudaMemcpyHostToDevice));
        MOE_CUDA_TRY(c, cudaMemcpy(ep->srow_peer_dev[m], st, sizeof(st), cudaMemcpyHostToDevice));
        MOE_CUDA_TRY(c, cudaMemcpy(ep->ret_peer_dev[m], rt, sizeof(rt), cudaMemcpyHostToDevice));
    }
    MOE_CUDA_TRY(c, cudaMemcpyAsync(ep->sync_peer_dev, ep->sync_peer, sizeof(void *) * MOE_EP_MAX_WORLD, cudaMemcpyHostToDevice, c->stream));
    // nobody may write into a peer before every rank has finished mapping
    MOE_NCCL_TRY(c, g_nccl.AllReduce(ep->bar, ep->bar + 8, 1, ncclUint32, ncclSum, ep->comm, c->stream));
    MOE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
}

// Cross-GPU barrier without a library call: every rank stores the epoch into its
// slot of every peer's flag row, then waits until all slots of its own row have
// reached the epoch.  Flags only ever grow.  The wait is bounded (the context's
// wait limit, 2 s unless moe_cuda_set_wait_ns changed it): on timeout the kernel
// records MOE_ERR_TIMEOUT and returns, it never hangs.
__device__ __forceinline__ void ep_signal_and_wait(uint32_t *const *sync_peers, uint32_t world, uint32_t rank, uint32_t site,
                                                   uint32_t epoch, uint32_t *status, uint64_t wait_ns) {
    // called by threads 0..world-1 of a block after a __syncthreads(); thread p talks to rank p
    uint32_t p = threadIdx.x;
    if (p < world) {
        __threadfence_system();
        uint32_t *theirs = sync_peers[p] + site * MOE_EP_MAX_WORLD + rank;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(theirs), "r"(epoch) : "memory");
        const uint32_t *mine = sync_peers[rank] + site * MOE_EP_MAX_WORLD + p;
        uint64_t t0 = 0;
        for (uint32_t spins = 0;; spins += 1) {
            uint32_t v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
            if ((int32_t)(v - epoch) >= 0) break;
            if ((spins & 0x3ffu) == 0x3ffu) {
                uint64_t now;
                asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(now));
                if (t0 == 0) {
                    t0 = now;
                } else if (now - t0 > wait_ns) {
                    atomicCAS(status, 0u, (uint32_t)MOE_ERR_TIMEOUT | ((20u + site) << 8));
                    break;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(32)
moe_ep_barrier_kernel(uint32_t *const *sync_peers, uint32_t world, uint32_t rank, uint32_t site, uint32_t epoch,
                      uint32_t *status, uint64_t wait_ns) {
    ep_signal_and_wait(sync_peers, world, rank, site, epoch, status, wait_ns);
}

// Runs the cross-GPU flag barrier as rank 0 of a two-rank group whose second
// rank does not exist: both entries of the peer table point at one local,
// zeroed flag buffer, so the flag of rank 1 is never set and the wait must run
// into the context's limit, record MOE_ERR_TIMEOUT and return.  Nothing faults
// and nothing hangs; the context is left failed (sticky), as after a real
// timeout.
extern "C" void moe_cuda_wait_selftest(moe_cuda_ctx_t *c) {
    if (!MOE_LIVE(c)) return;
    uint8_t *buf = (uint8_t *)moe_scratch(c, MOE_SCR_EP, 4096);
    if (buf == NULL) return;
    MOE_CUDA_TRY(c, cudaMemsetAsync(buf, 0, 4096, c->stream));
    void *table[MOE_EP_MAX_WORLD] = {};
    table[0] = buf;
    table[1] = buf;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(buf + 2048, table, sizeof(table), cudaMemcpyHostToDevice, c->stream));
    moe_ep_barrier_kernel<<<1, 32, 0, c->stream>>>((uint32_t *const *)(buf + 2048), 2u, 0u, 0u, 1u, c->dev_status_dev, c->wait_ns);
    MOE_LAUNCHED(c);
}

// From all ranks' per-expert counts: where this rank's rows of expert e start in
// the owner's buffer (dst_off), and the owner-side tile schedule of this rank's
// own experts.  One block of 512 threads, thread = global expert.
// The counts exchange is part of this kernel: each rank stores its counts row
// into every peer's table, a flag barrier makes all rows visible, then the plan
// is computed -- one launch instead of an all-gather plus a kernel.
__global__ void __launch_bounds__(512)
moe_ep_plan_kernel(const uint32_t *__restrict__ my_count, uint32_t *const *sync_peers, uint32_t epoch, uint32_t site,
                   uint32_t table_off, uint32_t *__restrict__ dst_off, uint32_t *__restrict__ tiles,
                   uint32_t experts, uint32_t world, uint32_t rank, uint32_t el, uint32_t mcap, uint32_t *status,
                   uint64_t wait_ns, uint32_t *__restrict__ lcount, uint32_t *__restrict__ loff) {
    __shared__ uint32_t incl_s[512];
    uint32_t e = threadIdx.x;
    if (e < experts) {
        uint32_t v = my_count[e];
        for (uint32_t p = 0; p < world; p += 1) sync_peers[p][table_off + rank * experts + e] = v;
    }
    __syncthreads();
    ep_signal_and_wait(sync_peers, world, rank, site, epoch, status, wait_ns);
    __syncthreads();
    const volatile uint32_t *cnt_all = sync_peers[rank] + table_off;
    uint32_t tot = 0, before = 0;
    if (e < experts) {
        for (uint32_t s = 0; s < world; s += 1) {
            uint32_t v = cnt_all[s * experts + e];
            if (s < rank) before += v;
            tot += v;
        }
    }
    uint32_t p = (tot + MOE_TILE - 1u) / MOE_TILE * MOE_TILE;
    incl_s[e] = p;
    __syncthreads();
    for (uint32_t o = 1; o < 512; o <<= 1) {  // Hillis-Steele over at most 512 entries
        uint32_t v = e >= o ? incl_s[e - o] : 0;
        __syncthreads();
        incl_s[e] += v;
        __syncthreads();
    }
    if (e < experts) {
        uint32_t owner = e / el;
        uint32_t owner_start = owner * el;
        uint32_t base = owner_start > 0 ? incl_s[owner_start - 1] : 0;
        uint32_t off = incl_s[e] - p - base;  // rows before expert e inside its owner's buffer
        if (off + p > mcap) {
            atomicCAS(status, 0u, (uint32_t)MOE_ERR_ARG | (2u << 8));
        } else {
            dst_off[e] = off + before;
            if (owner == rank) {
                for (uint32_t t = off / MOE_TILE; t < (off + p) / MOE_TILE; t += 1) tiles[t] = e - owner_start;
                lcount[e - owner_start] = tot;  // the rows of this rank's own experts, for the chunk list
                loff[e - owner_start] = off;
            }
        }
    }
}

// Dispatch, bulk part: one warp per token reads the row once and stores it into the receive
// buffer of every GPU that owns at least one of the token's experts (its own included: the
// product gathers all its operand rows from the receive buffer), at row src_base + token.
__global__ void __launch_bounds__(256)
moe_ep_send_kernel(const uint32_t *__restrict__ idx, const uint4 *__restrict__ x16, uint4 *const *__restrict__ xin_peers,
                   uint32_t rows, uint32_t topk, uint32_t d8, uint32_t el, uint32_t world, uint32_t src_base) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t r = warp; r < rows; r += nwarps) {
        uint32_t bit = 0;
        if (lane < topk) {
            const uint32_t g = idx[(size_t)r * topk + lane] / el;
            if (g < world) bit = 1u << g;  // a row the router refused carries ~0 and goes nowhere
        }
        const uint32_t mask = __reduce_or_sync(0xffffffffu, bit);
        const uint4 *src = x16 + (size_t)r * d8;
        for (uint32_t c0 = 0; c0 < d8; c0 += 256u) {
            uint4 v[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; i += 1) {
                const uint32_t ci = c0 + i * 32u + lane;
                if (ci < d8) v[i] = __ldg(src + ci);
            }
            for (uint32_t mk = mask; mk != 0; mk &= mk - 1u) {
                uint4 *dst = xin_peers[__ffs((int)mk) - 1] + (size_t)(src_base + r) * d8;
#pragma unroll
                for (uint32_t i = 0; i < 8; i += 1) {
                    const uint32_t ci = c0 + i * 32u + lane;
                    if (ci < d8) dst[ci] = v[i];
                }
            }
        }
    }
}

// Return, owner side: a warp takes one received token slot and one 2 KB piece of its row, adds
// wt * (expert output row) over the token's records in list order (fp32, multiply and add rounded
// separately as in the combine) and leaves fp16; the next record's loads are issued before the
// current one is accumulated.  A slot whose list is empty is skipped and never read by its home GPU.
__global__ void __launch_bounds__(256)
moe_ep_partial_kernel(const uint2 *__restrict__ ret_tab, const uint4 *__restrict__ ye, uint4 *__restrict__ part,
                      uint32_t slots, uint32_t topk, uint32_t d8) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, nwarps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t pieces = (d8 + 127u) / 128u;  // 128 x 16 bytes per piece: four 16-byte loads per lane
    for (uint32_t u = warp; u < slots * pieces; u += nwarps) {
        const uint32_t t = u / pieces, c0 = (u - t * pieces) * 128u;
        const uint2 *rec = ret_tab + (size_t)t * topk;
        const uint2 mine = lane < topk ? rec[lane] : make_uint2(~0u, 0u);
        const uint32_t n = (uint32_t)__popc(__ballot_sync(0xffffffffu, mine.x != ~0u));  // lists are packed from entry 0
        if (n == 0) continue;
        float acc[4][8];
#pragma unroll
        for (uint32_t i = 0; i < 4; i += 1) {
#pragma unroll
            for (uint32_t q = 0; q < 8; q += 1) acc[i][q] = 0.0f;
        }
        uint4 cur[4], nxt[4];
        {
            const uint4 *src = ye + (size_t)__shfl_sync(0xffffffffu, mine.x, 0) * d8;
#pragma unroll
            for (uint32_t i = 0; i < 4; i += 1) {
                const uint32_t ci = c0 + i * 32u + lane;
                cur[i] = ci < d8 ? src[ci] : make_uint4(0u, 0u, 0u, 0u);
            }
        }
        for (uint32_t j = 0; j < n; j += 1) {
            const float w = __uint_as_float(__shfl_sync(0xffffffffu, mine.y, j));
            if (j + 1u < n) {
                const uint4 *src = ye + (size_t)__shfl_sync(0xffffffffu, mine.x, j + 1u) * d8;
#pragma unroll
                for (uint32_t i = 0; i < 4; i += 1) {
                    const uint32_t ci = c0 + i * 32u + lane;
                    nxt[i] = ci < d8 ? src[ci] : make_uint4(0u, 0u, 0u, 0u);
                }
            }
#pragma unroll
            for (uint32_t i = 0; i < 4; i += 1) {
                const __half2 *h = reinterpret_cast<const __half2 *>(&cur[i]);
#pragma unroll
                for (uint32_t q = 0; q < 4; q += 1) {
                    const float2 f = __half22float2(h[q]);
                    acc[i][2 * q] = __fadd_rn(acc[i][2 * q], __fmul_rn(w, f.x));
                    acc[i][2 * q + 1] = __fadd_rn(acc[i][2 * q + 1], __fmul_rn(w, f.y));
                }
                cur[i] = nxt[i];
            }
        }
        uint4 *dst = part + (size_t)t * d8;
#pragma unroll
        for (uint32_t i = 0; i < 4; i += 1) {
            const uint32_t ci = c0 + i * 32u + lane;
            if (ci < d8) {
                uint4 o;
                __half2 *h = reinterpret_cast<__half2 *>(&o);
#pragma unroll
                for (uint32_t q = 0; q < 4; q += 1) h[q] = __floats2half2_rn(acc[i][2 * q], acc[i][2 * q + 1]);
                dst[ci] = o;
            }
        }
    }
}

// Rows of micro-batch m when `rows` tokens are cut into nmb slices: equal parts rounded up to the router's
// 8-row blocks, the last slice takes what is left (possibly nothing).
static void ep_slice(uint32_t rows, uint32_t nmb, uint32_t m, uint32_t *row0, uint32_t *n) {
    const uint32_t part = nmb == 1 ? rows : (((rows + nmb - 1u) / nmb + 7u) & ~7u);
    const uint32_t lo = (uint64_t)m * part < rows ? m * part : rows;
    const uint32_t hi = m + 1u == nmb ? rows : ((uint64_t)(m + 1u) * part < rows ? (m + 1u) * part : rows);
    *row0 = lo;
    *n = hi - lo;
}

extern "C" void moe_cuda_ep_layer(moe_cuda_ctx_t *c, const moe_cuda_layer_t *L) {
    if (!MOE_LIVE(c)) return;
    moe_ep_state *ep = c->ep;
    MOE_REQUIRE(c, ep != NULL, "ep_layer: moe_cuda_ep_init has not run");
    MOE_REQUIRE(c, L != NULL && L->proj != NULL && L->x16 != NULL && L->wgu != NULL && L->wdown != NULL, "ep_layer: null input");
    MOE_REQUIRE(c, L->h != NULL || L->y16 != NULL, "ep_layer: no output");
    MOE_REQUIRE(c, L->experts == ep->cfg.experts && L->topk == ep->cfg.topk && L->d == ep->cfg.d && L->inter == ep->cfg.inter,
                "ep_layer: shape differs from moe_cuda_ep_init");
    MOE_REQUIRE(c, L->rows <= ep->cfg.max_rows, "ep_layer: rows %u > max_rows %u", L->rows, ep->cfg.max_rows);
    MOE_REQUIRE(c, L->shared % 128u == 0, "ep_layer: shared %u not a multiple of 128", L->shared);
    MOE_REQUIRE(c, L->shared == 0 || (L->wsgu != NULL && L->wsdown != NULL), "ep_layer: shared expert without weights");
    MOE_REQUIRE(c, L->hc >= 1, "ep_layer: hc 0");
    const uint32_t R = L->rows, K = L->topk, E = L->experts, d = L->d, I = L->inter, S = L->shared;
    const uint32_t mcap = ep->mcap, nmb = ep->nmb;
    uint32_t *idx = L->idx != NULL ? L->idx : ep->idx;
    uint32_t *slot = L->slot != NULL ? L->slot : ep->slot;
    float *wt = L->wt != NULL ? L->wt : ep->wt;
    cudaStream_t main_stream = c->stream;
    const bool prof = c->prof && c->ev_made;

    // stage marks of micro-batch m go on its own stream; moe_cuda_prof_read adds the slices up
    auto mark = [&](uint32_t m, int i) {
        if (prof && c->status == MOE_OK) cudaEventRecord(m == 0 ? c->ev[i] : c->ev_mb[m - 1][i], c->stream);
    };
    if (prof && nmb > 1 && c->ev_mb_made < (int)nmb - 1) {
        for (int m = c->ev_mb_made; m < (int)nmb - 1; m += 1) {
            for (int i = 0; i <= MOE_PROF_STAGES; i += 1) MOE_CUDA_TRY(c, cudaEventCreate(&c->ev_mb[m][i]));
            c->ev_mb_made = m + 1;
        }
    }
    mark(0, 0);
    for (uint32_t m = 0; m < nmb; m += 1) {
        moe_cuda_fill(c, ep->tiles[m], (size_t)(mcap / MOE_TILE) * 4, 0xffffffffu);
        if (ep->per_gpu) {
            // padding rows of used tiles read as zero; peers write the live entries after the first barrier
            moe_cuda_fill(c, ep->src_row[m], (size_t)mcap * 4, 0xffffffffu);
            // return records: ~0 ends a token's list
            moe_cuda_fill(c, ep->ret_tab[m], (size_t)ep->world * ep->cap * K * 8, 0xffffffffu);
        }
    }
    uint32_t *hist = (uint32_t *)moe_scratch(c, MOE_SCR_SCATTER, (size_t)((R + 7u) / 8u + 1u) * E * 4);
    if (hist == NULL) return;
    // The shared expert (src/qwen.c:879-886) is replicated: every rank runs it on its own tokens.
    const uint32_t Rp = (R + MOE_TILE - 1u) / MOE_TILE * MOE_TILE;
    __half *hs16 = NULL;
    float *sh = NULL;
    uint32_t *tiles0 = NULL;
    if (S != 0 && R != 0) {
        const size_t b_hs = ((size_t)Rp * S * 2 + 1023) & ~(size_t)1023, b_sh = ((size_t)Rp * d * 4 + 1023) & ~(size_t)1023;
        uint8_t *scr = (uint8_t *)moe_scratch(c, MOE_SCR_LAYER, b_hs + b_sh + (size_t)(Rp / MOE_TILE) * 4 + 1024);
        if (scr == NULL) return;
        hs16 = (__half *)scr;
        sh = (float *)(scr + b_hs);
        tiles0 = (uint32_t *)(scr + b_hs + b_sh);
    }
    if (R != 0) moe_launch_route_hist(c, L->proj, idx, wt, hist, R, E, K, L->pstride);
    mark(0, 1);
    if (!MOE_LIVE(c)) return;
    ep->epoch += 1;
    if (nmb > 1) {
        MOE_CUDA_TRY(c, cudaEventRecord(ep->ev_fork, main_stream));
        for (uint32_t m = 1; m < nmb; m += 1) MOE_CUDA_TRY(c, cudaStreamWaitEvent(ep->side[m], ep->ev_fork, 0));
    }
    for (uint32_t m = 0; m < nmb; m += 1) {
        // Micro-batch m runs on its own stream; every rank issues the same sequence, also for an empty slice.
        uint32_t row0, rows;
        ep_slice(R, nmb, m, &row0, &rows);
        const uint32_t site = 3u * m;
        c->stream = m == 0 ? main_stream : ep->side[m];
        if (m != 0) {
            mark(m, 0);
            mark(m, 1);
        }
        uint32_t *count = (m == 0 && nmb == 1 && L->count != NULL) ? L->count : ep->count[m];
        if (rows != 0) moe_launch_colscan_counts(c, hist + (size_t)(row0 / 8u) * E, count, rows, E);
        else moe_cuda_fill(c, count, (size_t)E * 4, 0);
        // counts of every rank + plan (also orders this layer after every peer's previous combine)
        moe_ep_plan_kernel<<<1, 512, 0, c->stream>>>(count, (uint32_t *const *)ep->sync_peer_dev, ep->epoch, site,
                                                     EP_FLAG_WORDS + m * (uint32_t)ep->world * E, ep->dst_off[m], ep->tiles[m], E,
                                                     (uint32_t)ep->world, (uint32_t)ep->rank, ep->el, mcap, c->dev_status_dev, c->wait_ns,
                                                     ep->wsbuf[m], ep->wsbuf[m] + ep->el);
        c->launches += 1;
        // the received rows of an expert are cut into chunks of at most 256 for the weight-stationary products
        uint32_t *n_chunks = ep->wsbuf[m] + 2u * ep->el;
        void *chunks = (void *)(((uintptr_t)(n_chunks + 16) + 15u) & ~(uintptr_t)15u);
        const bool ws = d % 256u == 0 && (L->flags & MOE_LAYER_TILED) == 0;
        if (ws) moe_launch_chunks(c, ep->wsbuf[m], ep->wsbuf[m] + ep->el, ep->el, chunks, n_chunks, ep->max_chunks);
        if (m == 0 && L->off != NULL && nmb == 1) moe_cuda_copy(c, L->off, ep->dst_off[0], (size_t)E * 4);
        mark(m, 2);
        // stagger: this slice's rows go out once the previous slice's are on their way, under its products
        if (m != 0) cudaStreamWaitEvent(c->stream, ep->ev_disp[m - 1], 0);
        __half *xin_m = ep->xin + (size_t)m * ep->in_rows * d, *yout_m = ep->yout + (size_t)m * ep->in_rows * d;
        __half *ye_m = ep->per_gpu ? ep->ye + (size_t)m * mcap * d : yout_m;
        if (rows != 0 && !ep->per_gpu) {
            // dispatch fused into the scatter: every pair's row goes straight into its owner's expert-contiguous buffer
            moe_launch_place(c, idx + (size_t)row0 * K, ep->dst_off[m], hist + (size_t)(row0 / 8u) * E,
                             (const __half *)L->x16 + (size_t)row0 * d, xin_m, slot + (size_t)row0 * K, rows, K, d / 8u, E,
                             ep->xin_peer_dev[m], ep->el);
        }
        // dispatch: each row once per destination GPU, then the records of every (token, expert) pair
        if (rows != 0 && ep->per_gpu) {
            const uint32_t src_base = (uint32_t)ep->rank * ep->cap;
            moe_ep_send_kernel<<<(rows + 7u) / 8u, 256, 0, c->stream>>>(
                idx + (size_t)row0 * K, (const uint4 *)((const __half *)L->x16 + (size_t)row0 * d),
                (uint4 *const *)ep->xin_peer_dev[m], rows, K, d / 8u, ep->el, (uint32_t)ep->world, src_base);
            c->launches += 1;
            moe_launch_place(c, idx + (size_t)row0 * K, ep->dst_off[m], hist + (size_t)(row0 / 8u) * E, L->x16, NULL,
                             slot + (size_t)row0 * K, rows, K, d / 8u, E, NULL, ep->el, NULL,
                             (uint32_t *const *)ep->srow_peer_dev[m], src_base, (uint2 *const *)ep->ret_peer_dev[m],
                             wt + (size_t)row0 * K);
        }
        if (nmb > 1) cudaEventRecord(ep->ev_disp[m], c->stream);
        if (m == 0 && S != 0 && R != 0) {
            // the shared expert's two products on all local tokens, while the other ranks' rows are still landing
            moe_cuda_fill(c, tiles0, (size_t)(Rp / MOE_TILE) * 4, 0);
            moe_launch_mm(c, MOE_MM_SWIGLU_F16, L->x16, L->wsgu, hs16, NULL, tiles0, Rp, 2u * S, d, MDA_PC_NO_SLOT, MDA_PC_NO_SLOT, 1, R);
            moe_launch_mm(c, MOE_MM_F32, hs16, L->wsdown, sh, NULL, tiles0, Rp, d, S, MDA_PC_NO_SLOT, MDA_PC_NO_SLOT, 1, Rp);
            if (nmb > 1) {  // the other slices' combines read sh too
                MOE_CUDA_TRY(c, cudaEventRecord(ep->ev_join[0], c->stream));
                for (uint32_t q = 1; q < nmb; q += 1) MOE_CUDA_TRY(c, cudaStreamWaitEvent(ep->side[q], ep->ev_join[0], 0));
            }
        }
        moe_ep_barrier_kernel<<<1, 32, 0, c->stream>>>((uint32_t *const *)ep->sync_peer_dev, (uint32_t)ep->world,
                                                       (uint32_t)ep->rank, site + 1u, ep->epoch, c->dev_status_dev, c->wait_ns);  // all rows landed
        c->launches += 1;
        mark(m, 3);
        if (ws && !ep->per_gpu) {
            moe_launch_mm_ws(c, MOE_MM_SWIGLU_F16, 2, xin_m, ep->in_rows, L->wgu, ep->el, ep->hp16 + (size_t)m * mcap * I, I, chunks,
                             n_chunks, ep->max_chunks, 2u * I, d);
        } else if (ws) {
            // per-GPU scheme: the received rows go into expert order first; ye's buffer is free until the down product
            moe_ep_permute_kernel<<<(mcap + 7u) / 8u, 256, 0, c->stream>>>(ep->src_row[m], (const uint4 *)xin_m, (uint4 *)ye_m, mcap,
                                                                          d / 8u);
            c->launches += 1;
            moe_launch_mm_ws(c, MOE_MM_SWIGLU_F16, 2, ye_m, mcap, L->wgu, ep->el, ep->hp16 + (size_t)m * mcap * I, I, chunks,
                             n_chunks, ep->max_chunks, 2u * I, d);
        } else {
            moe_launch_mm(c, MOE_MM_SWIGLU_F16, xin_m, L->wgu, ep->hp16 + (size_t)m * mcap * I, NULL, ep->tiles[m], mcap, 2u * I, d,
                          MDA_PC_NO_SLOT, MDA_PC_NO_SLOT, ep->el, ep->in_rows, true, ep->per_gpu ? ep->src_row[m] : NULL);
        }
        mark(m, 4);
        if (ws) {
            moe_launch_mm_ws(c, MOE_MM_F16, 2, ep->hp16 + (size_t)m * mcap * I, mcap, L->wdown, ep->el, ye_m, d, chunks, n_chunks,
                             ep->max_chunks, d, I);
        } else {
            moe_launch_mm(c, MOE_MM_F16, ep->hp16 + (size_t)m * mcap * I, L->wdown, ye_m, NULL,
                          ep->tiles[m], mcap, d, I, MDA_PC_NO_SLOT, MDA_PC_NO_SLOT, ep->el, mcap, true);
        }
        if (ep->per_gpu) {  // return, owner side: one weighted partial row per received token
            const uint32_t slots = (uint32_t)ep->world * ep->cap;
            const uint32_t units = slots * ((d / 8u + 127u) / 128u);  // one warp per (slot, 2 KB piece)
            moe_ep_partial_kernel<<<(units + 7u) / 8u, 256, 0, c->stream>>>(
                ep->ret_tab[m], (const uint4 *)ye_m, (uint4 *)yout_m, slots, K, d / 8u);
            c->launches += 1;
        }
        mark(m, 5);
        moe_ep_barrier_kernel<<<1, 32, 0, c->stream>>>((uint32_t *const *)ep->sync_peer_dev, (uint32_t)ep->world,
                                                       (uint32_t)ep->rank, site + 2u, ep->epoch, c->dev_status_dev, c->wait_ns);  // all result rows written
        c->launches += 1;
        mark(m, 6);
        if (rows != 0) {
            moe_combine_args a = {};
            a.wt = wt + (size_t)row0 * K;
            a.slot = slot + (size_t)row0 * K;
            a.y = ye_m;
            a.proj = L->proj + (size_t)row0 * L->pstride;
            a.sh = S != 0 ? sh + (size_t)row0 * d : NULL;
            a.inj = L->inj != NULL ? L->inj + (size_t)row0 * L->inj_stride : NULL;
            a.h = L->h != NULL ? L->h + (size_t)row0 * L->hc * d : NULL;
            a.x16 = (const __half *)L->x16 + (size_t)row0 * d;
            a.y16 = L->y16 != NULL ? (__half *)L->y16 + (size_t)row0 * d : NULL;
            a.eps = L->eps;
            a.rows = rows;
            a.d = d;
            a.topk = K;
            a.pstride = L->pstride;
            a.sg_off = E;
            a.inj_stride = L->inj_stride;
            a.inj_off = L->inj_off;
            a.hc = L->hc;
            a.y_is_f16 = true;
            a.idx = idx + (size_t)row0 * K;
            a.y_peers = (const void *const *)ep->yout_peer_dev[m];
            a.experts_per_rank = ep->el;
            a.world = (uint32_t)ep->world;
            a.src_base = (uint32_t)ep->rank * ep->cap;
            a.per_gpu = ep->per_gpu;
            moe_launch_combine(c, a);  // return all-to-all fused into the gather: one partial row per owning GPU
        }
        mark(m, 7);
    }
    c->stream = main_stream;
    for (uint32_t m = 1; m < nmb; m += 1) {
        cudaEventRecord(ep->ev_join[m], ep->side[m]);
        cudaStreamWaitEvent(main_stream, ep->ev_join[m], 0);
    }
    if (cudaGetLastError() != cudaSuccess) moe_fail(c, MOE_ERR_CUDA, "ep_layer: launch failed");
    if (prof && c->status == MOE_OK) {
        c->ev_valid = true;
        c->ev_slices = (int)nmb;
    }
}
