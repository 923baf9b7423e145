// Shared declarations of libmoe_cuda's translation units: the context object,
// status handling and small device helpers.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/moe_cuda.h"

#define MOE_MAX_EXPERTS 512u  // shader/moe_route.comp:24-26, shader/moe_scan.comp:2
#define MOE_MAX_TOPK 16u      // shader/moe_route.comp:18
#define MOE_TILE 128u         // MDA_QWEN_TILE, src/qwen.h:14

// Scratch areas inside the context (grown on demand, never shrunk).
enum { MOE_SCR_SCATTER = 0, MOE_SCR_LAYER = 1, MOE_SCR_STAGE = 2, MOE_SCR_EP = 3, MOE_SCR_COUNT = 4 };

struct moe_tmap_entry {
    const void *ptr;
    uint64_t rows, cols;
    uint32_t box_rows, box_cols;
    uint32_t kind;  // 0: plain 2-D; 1: gate/up interleaved 4-D
    CUtensorMap map;
};

struct moe_ep_state;  // moe_ep.cu

struct moe_cuda_ctx {
    int device;
    int sm_count;
    cudaStream_t stream;
    bool own_stream;
    int status;  // sticky, like mda_vkc_t.fail (src/vkc.h:47)
    char err[256];
    // Device-visible status word in mapped pinned memory: kernels record refusals
    // (MOE_ERR_ROUTE, MOE_ERR_TIMEOUT) here instead of trapping.
    uint32_t *dev_status_host;
    uint32_t *dev_status_dev;
    void *scratch[MOE_SCR_COUNT];
    size_t scratch_bytes[MOE_SCR_COUNT];
    moe_tmap_entry tmaps[128];
    int n_tmaps, next_tmap;
    void *encode_tiled;  // cuTensorMapEncodeTiled, resolved at create
    bool prof;
    cudaEvent_t ev[MOE_PROF_STAGES + 1];
    bool ev_made, ev_valid;
    cudaEvent_t ev_mb[3][MOE_PROF_STAGES + 1];  // expert parallel: the same marks of token slices 1..3, on their streams
    int ev_mb_made, ev_slices;
    uint64_t launches;
    int fail_alloc_countdown;
    bool mm_attr_set[4];
    uint32_t *ticket;  // device word, zero between kernels: "last block done" counter
    bool sw_attr_set[8];
    moe_ep_state *ep;
    uint64_t wait_ns;  // bound of every device-side wait (mbarriers, cross-GPU flags)
};

void moe_fail(moe_cuda_ctx *c, int code, const char *fmt, ...);
void *moe_scratch(moe_cuda_ctx *c, int area, size_t bytes);
bool moe_poll_device_status(moe_cuda_ctx *c);
void moe_ep_teardown(moe_cuda_ctx *c);
const CUtensorMap *moe_tmap_2d_f16(moe_cuda_ctx *c, const void *ptr, uint64_t rows, uint64_t cols,
                                   uint32_t box_rows, uint32_t box_cols);

// 4-D fp16 tensor map over an expert bank [experts][2][inter][k] (gate rows then up rows per expert) whose
// box (64 k, 2, 64 inter, 1 expert) lands in shared memory as 128 rows: row 2i = gate row i, row 2i+1 = up row i.
const CUtensorMap *moe_tmap_gate_up_f16(moe_cuda_ctx *c, const void *ptr, uint32_t experts, uint32_t inter, uint32_t k);

#define MOE_LIVE(c) ((c) != NULL && (c)->status == MOE_OK)

#define MOE_CUDA_TRY(c, expr)                                                             \
    do {                                                                                  \
        cudaError_t e__ = (expr);                                                         \
        if (e__ != cudaSuccess) {                                                         \
            moe_fail((c), MOE_ERR_CUDA, "%s:%d: %s", __FILE__, __LINE__,                  \
                     cudaGetErrorString(e__));                                            \
            return;                                                                       \
        }                                                                                 \
    } while (0)

#define MOE_LAUNCHED(c)                                                                   \
    do {                                                                                  \
        (c)->launches += 1;                                                               \
        MOE_CUDA_TRY((c), cudaGetLastError());                                            \
    } while (0)

#define MOE_REQUIRE(c, cond, ...)                                                         \
    do {                                                                                  \
        if (!(cond)) {                                                                    \
            moe_fail((c), MOE_ERR_ARG, __VA_ARGS__);                                      \
            return;                                                                       \
        }                                                                                 \
    } while (0)

// Internal launch helpers shared between the ABI entry points and the fused layer.
void moe_launch_route(moe_cuda_ctx *c, const float *proj, uint32_t *idx, float *wt, uint32_t *count,
                      uint32_t rows, uint32_t experts, uint32_t topk, uint32_t stride);
void moe_launch_scan(moe_cuda_ctx *c, const uint32_t *count, uint32_t *off, uint32_t *tiles,
                     uint32_t experts, uint32_t tile);
void moe_launch_scatter(moe_cuda_ctx *c, const uint32_t *idx, const uint32_t *off, uint32_t *fill,
                        const void *x16, void *xp, uint32_t *slot, uint32_t rows, uint32_t topk,
                        uint32_t d8, uint32_t experts_bound, void *const *xp_peers = NULL,
                        uint32_t experts_per_rank = 0);

// ones_a / ones_b: up to two word tables the router also fills with ~0 (tile schedule, source rows).
void moe_launch_route_hist(moe_cuda_ctx *c, const float *proj, uint32_t *idx, float *wt, uint32_t *hist,
                           uint32_t rows, uint32_t experts, uint32_t topk, uint32_t stride, uint32_t *ones_a = NULL,
                           uint32_t n_a = 0, uint32_t *ones_b = NULL, uint32_t n_b = 0);
// off / tiles non-NULL: the last block to finish also runs the reference's scan on the fresh counts.
void moe_launch_colscan_counts(moe_cuda_ctx *c, uint32_t *hist, uint32_t *count, uint32_t rows, uint32_t experts,
                               uint32_t *off = NULL, uint32_t *tiles = NULL, uint32_t tile = 0, void *chunks = NULL,
                               uint32_t *n_chunks = NULL, uint32_t max_chunks = 0);
void moe_launch_place(moe_cuda_ctx *c, const uint32_t *idx, const uint32_t *off, const uint32_t *hist, const void *x16,
                      void *xp, uint32_t *slot, uint32_t rows, uint32_t topk, uint32_t d8, uint32_t experts,
                      void *const *xp_peers, uint32_t experts_per_rank, uint32_t *src_row = NULL,
                      uint32_t *const *src_row_peers = NULL, uint32_t src_base = 0, uint2 *const *ret_peers = NULL,
                      const float *wt = NULL);

enum { MOE_MM_F32 = 0, MOE_MM_SWIGLU_F16 = 1, MOE_MM_F16 = 2 };
// Grouped product.  mode F32: C fp32 [m x n] = A*B^T * s;  SWIGLU_F16: B holds
// [gate n/2 rows | up n/2 rows] per expert and C fp16 [m x n/2] = silu(gate)*up;
// F16: C fp16 [m x n].
// a_rows = rows A really holds (<= m); rows beyond read as zero.  c_rows (fp32 mode; 0 = m) = rows C really
// holds; rows beyond are not stored.  With src_row (SWIGLU_F16 only)
// A is the un-permuted activation matrix [a_rows x k] and tile row p is its row src_row[p].
void moe_launch_mm(moe_cuda_ctx *c, int mode, const void *A, const void *B, void *C,
                   const uint32_t *amax, const uint32_t *tiles, uint32_t m, uint32_t n, uint32_t k,
                   uint32_t sa, uint32_t sb, uint32_t experts_in_B, uint32_t a_rows, bool prefix = false,
                   const uint32_t *src_row = NULL, uint32_t c_rows = 0);

// Weight-stationary grouped product over token chunks (moe_mm_ws.cu).
void moe_launch_chunks(moe_cuda_ctx *c, const uint32_t *count, const uint32_t *off, uint32_t experts, void *chunks,
                       uint32_t *n_chunks, uint32_t max_chunks);
void moe_launch_mm_ws(moe_cuda_ctx *c, int mode, int pair, const void *X, uint32_t rows_x, const void *W,
                        uint32_t experts_in_W, void *C, uint32_t ldc, const void *chunks, const uint32_t *n_chunks,
                        uint32_t max_chunks, uint32_t n, uint32_t k);

struct moe_combine_args {
    const float *wt;
    const uint32_t *slot;
    const void *y;       // fp32 or fp16 [M x d]
    const float *proj;
    const float *sh;     // fp32 [rows x d] or NULL
    const float *inj;    // or NULL
    float *h;            // or NULL when y16 is set
    const __half *x16;   // residual input for the fused norm (or NULL)
    __half *y16;         // fused residual + RMSNorm output (or NULL)
    float eps;
    uint32_t rows, d, topk, pstride, sg_off, inj_stride, inj_off, hc;
    bool y_is_f16;
    // expert-parallel: GPU g = idx[r,j] / experts_per_rank holds row j of the token in y_peers[g] at
    // row slot[r,j]; or, with per_gpu, at row src_base + r the token's weighted sum over all its
    // experts there (fp16; wt, slot and y are then unused)
    const uint32_t *idx;
    const void *const *y_peers;
    uint32_t experts_per_rank;
    uint32_t world;      // number of GPUs behind y_peers
    uint32_t src_base;
    bool per_gpu;
};
void moe_launch_combine(moe_cuda_ctx *c, const moe_combine_args &a);
void moe_overlap_prepare_combine(moe_cuda_ctx *c);
void moe_overlap_prepare_scatter(moe_cuda_ctx *c);

// ---- device helpers -------------------------------------------------------
// shader/moe_scan.comp:14-38, for a block of at least 512 threads (all threads of the block must
// call it; thread e < 512 handles expert e).  count is read past L1.
__device__ __forceinline__ void moe_scan_body(const uint32_t *count, uint32_t *off, uint32_t *tiles, uint32_t experts,
                                              uint32_t tile) {
    __shared__ uint32_t wsum[16];
    const uint32_t e = threadIdx.x;
    const uint32_t lane = e & 31u, warp = e >> 5;
    uint32_t p = 0;
    if (e < experts) p = (__ldcg(count + e) + tile - 1u) / tile * tile;  // :19
    uint32_t incl = p;
#pragma unroll
    for (uint32_t o = 1; o < 32; o <<= 1) {
        uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31 && warp < 16) wsum[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        uint32_t w = lane < 16 ? wsum[lane] : 0;
#pragma unroll
        for (uint32_t o = 1; o < 16; o <<= 1) {
            uint32_t v = __shfl_up_sync(0xffffffffu, w, o);
            if (lane >= o) w += v;
        }
        if (lane < 16) wsum[lane] = w;
    }
    __syncthreads();
    if (e < experts) {
        uint32_t lo = incl - p + (warp > 0 ? wsum[warp - 1] : 0);  // :31
        off[e] = lo;                                                // :33
        for (uint32_t t = lo / tile; t < (lo + p) / tile; t += 1) tiles[t] = e;  // :34-36
    }
}

// The chunk list of the weight-stationary products: every expert's rows cut into chunks of at most MOE_CHUNK_TOK
// tokens of near-equal size, MMA width rounded up to 16; entry = (expert, first row, MMA width, valid rows).  For a
// block of at least 512 threads (all threads of the block must call it; thread e < 512 handles expert e).
#define MOE_CHUNK_TOK 256u
__device__ __forceinline__ void moe_chunk_body(const uint32_t *count, const uint32_t *off, uint32_t experts, uint4 *chunks,
                                               uint32_t *n_chunks, uint32_t max_chunks) {
    __shared__ uint32_t csum[512];
    const uint32_t e = threadIdx.x;
    uint32_t cnt = 0, nch = 0;
    if (e < 512u) {
        cnt = e < experts ? __ldcg(count + e) : 0u;
        nch = (cnt + MOE_CHUNK_TOK - 1u) / MOE_CHUNK_TOK;
        csum[e] = nch;
    }
    __syncthreads();
    for (uint32_t o = 1; o < 512; o <<= 1) {
        uint32_t v = (e < 512u && e >= o) ? csum[e - o] : 0u;
        __syncthreads();
        if (e < 512u) csum[e] += v;
        __syncthreads();
    }
    if (e < 512u && nch != 0) {
        const uint32_t first = csum[e] - nch;
        const uint32_t per = ((cnt + nch - 1u) / nch + 15u) & ~15u;
        const uint32_t row0 = __ldcg(off + e);
        for (uint32_t j = 0; j < nch; j += 1) {
            const uint32_t start = j * per;
            const uint32_t valid = start < cnt ? min(per, cnt - start) : 0u;
            if (first + j < max_chunks) chunks[first + j] = make_uint4(e, row0 + start, (valid + 15u) & ~15u, valid);
        }
    }
    if (e == 511u) *n_chunks = min(csum[511], max_chunks);
}

__device__ __forceinline__ float moe_slot_scale(const uint32_t *amax, uint32_t s) {
    // shader/matmul_f16_moe.comp:60-68 = shader/cast_f16.comp:20-28
    if (s == MDA_PC_NO_SLOT) return 1.0f;
    uint32_t bits = amax[s];
    float a = __uint_as_float(bits);
    if (!(a > 0.0f) || isinf(a)) return 1.0f;
    return exp2f(141.0f - (float)((bits >> 23) & 0xffu));
}
