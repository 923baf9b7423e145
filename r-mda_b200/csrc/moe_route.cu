// Router top-k and the per-expert scan: CUDA for sm_100a.
//
// route: one warp per row (shader/moe_route.comp uses one 32-lane subgroup per
// row).  Lane l holds logits e = 4*l + 128*j + {0..3}, j < 4, fetched with
// 128-bit loads; k rounds of (lane-local best, warp arg-max by shuffle) pick
// the largest remaining logit, ties to the lower expert index -- the net rule of
// the shader's subgroupMax / subgroupMin pair (:30-50).
#include "moe_common.cuh"

#define ROUTE_WARPS 8
#define ROUTE_SENTINEL -3.0e38f  // shader/moe_route.comp:31

// HIST = false: counts by one atomicAdd per selection, as the shader does (:59).
// HIST = true (fused layer): block b owns rows [8b, 8b+8) and writes their
// per-expert pair counts to hist[b][*]; the counts then come out of the scatter's
// column scan, so no atomic is contended and the block table is ready for the
// stable ranking.
// NB = ceil(experts / 128): how many 128-expert blocks each lane really holds.
template <bool HIST, int NB>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float *__restrict__ proj, uint32_t *__restrict__ idx, float *__restrict__ wt,
                 uint32_t *__restrict__ count, uint32_t rows, uint32_t experts, uint32_t topk,
                 uint32_t stride, uint32_t *status, int vec_ok, uint32_t *__restrict__ ones_a, uint32_t n_a,
                 uint32_t *__restrict__ ones_b, uint32_t n_b) {
    __shared__ uint32_t s_hist[HIST ? MOE_MAX_EXPERTS : 1];
    if (HIST) {
        // the fills of src/qwen.c:796 ride along: tables that later kernels expect to start as ~0
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_a; i += gridDim.x * blockDim.x) ones_a[i] = ~0u;
        for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n_b; i += gridDim.x * blockDim.x) ones_b[i] = ~0u;
    }
    uint32_t lane = threadIdx.x & 31u;
    uint32_t warp = threadIdx.x >> 5;
    uint32_t nwarps = gridDim.x * ROUTE_WARPS;
    if (HIST) {
        for (uint32_t e = threadIdx.x; e < experts; e += ROUTE_WARPS * 32) s_hist[e] = 0;
        __syncthreads();
    }
    for (uint32_t r = blockIdx.x * ROUTE_WARPS + warp; r < rows; r += nwarps) {
        const float *row = proj + (size_t)r * stride;
        float l[4 * NB];
#pragma unroll
        for (uint32_t j = 0; j < NB; j += 1) {
            uint32_t e0 = 4u * lane + 128u * j;
            if (vec_ok && e0 + 3u < experts) {
                float4 v = __ldg(reinterpret_cast<const float4 *>(row + e0));
                l[4 * j + 0] = v.x;
                l[4 * j + 1] = v.y;
                l[4 * j + 2] = v.z;
                l[4 * j + 3] = v.w;
            } else {
#pragma unroll
                for (uint32_t q = 0; q < 4; q += 1) {
                    l[4 * j + q] = e0 + q < experts ? __ldg(row + e0 + q) : ROUTE_SENTINEL;
                }
            }
        }
        uint32_t taken = 0;
        float my_v = 0.0f;      // lane k keeps the k-th selected logit
        uint32_t my_e = ~0u;
        float v0 = 0.0f;
        bool bad = false;
        for (uint32_t k = 0; k < topk; k += 1) {
            float lb = ROUTE_SENTINEL;
            uint32_t li = ~0u;
#pragma unroll
            for (uint32_t j = 0; j < 4 * NB; j += 1) {
                // ascending expert index inside the lane: q fastest, then the 128-blocks
                uint32_t e = 4u * lane + 128u * (j >> 2) + (j & 3u);
                if (((taken >> j) & 1u) == 0u && l[j] > lb) {  // strict >: first of equals (:34)
                    lb = l[j];
                    li = e;
                }
            }
            // warp arg-max on (value desc, index asc)
            float gm = lb;
            uint32_t gi = li;
#pragma unroll
            for (uint32_t o = 16; o > 0; o >>= 1) {
                float ov = __shfl_xor_sync(0xffffffffu, gm, o);
                uint32_t oi = __shfl_xor_sync(0xffffffffu, gi, o);
                if (ov > gm || (ov == gm && oi < gi)) {
                    gm = ov;
                    gi = oi;
                }
            }
            if (gi == ~0u) {
                bad = true;
            } else if (((gi & 127u) >> 2) == lane) {
                taken |= 1u << (((gi >> 7) << 2) | (gi & 3u));  // :45-47
            }
            if (k == 0) v0 = gm;
            if (lane == k) {
                my_v = gm;
                my_e = gi;
            }
        }
        if (bad) {
            // the shader would index count[~0u] here; refuse instead.  The row's entries are written as
            // "no expert, weight 0" so that kernels already queued behind this one (place, send, combine)
            // skip it instead of acting on values a previous call left there.
            if (lane == 0) atomicCAS(status, 0u, (uint32_t)MOE_ERR_ROUTE | (r << 8));
            if (lane < topk) {
                idx[(size_t)r * topk + lane] = ~0u;
                wt[(size_t)r * topk + lane] = 0.0f;
            }
            continue;
        }
        // :52-60: z accumulated k = 0..topk-1 in fp32, then each weight
        float t = lane < topk ? expf(my_v - v0) : 0.0f;
        float z = 0.0f;
        for (uint32_t k = 0; k < topk; k += 1) z += __shfl_sync(0xffffffffu, t, k);
        if (lane < topk) {
            idx[(size_t)r * topk + lane] = my_e;
            wt[(size_t)r * topk + lane] = t / z;
            if (HIST) atomicAdd(&s_hist[my_e], 1u);
            else atomicAdd(&count[my_e], 1u);
        }
    }
    if (HIST) {
        __syncthreads();
        for (uint32_t e = threadIdx.x; e < experts; e += ROUTE_WARPS * 32) count[(size_t)blockIdx.x * experts + e] = s_hist[e];
    }
}

template <bool HIST>
static void route_dispatch(moe_cuda_ctx *c, uint32_t blocks, const float *proj, uint32_t *idx, float *wt, uint32_t *count,
                           uint32_t rows, uint32_t experts, uint32_t topk, uint32_t stride, int vec_ok,
                           uint32_t *ones_a = NULL, uint32_t n_a = 0, uint32_t *ones_b = NULL, uint32_t n_b = 0) {
    const uint32_t nb = (experts + 127u) / 128u;
    const dim3 g(blocks), t(ROUTE_WARPS * 32);
#define ROUTE_ARGS proj, idx, wt, count, rows, experts, topk, stride, c->dev_status_dev, vec_ok, ones_a, n_a, ones_b, n_b
    if (nb == 1) moe_route_kernel<HIST, 1><<<g, t, 0, c->stream>>>(ROUTE_ARGS);
    else if (nb == 2) moe_route_kernel<HIST, 2><<<g, t, 0, c->stream>>>(ROUTE_ARGS);
    else if (nb == 3) moe_route_kernel<HIST, 3><<<g, t, 0, c->stream>>>(ROUTE_ARGS);
    else moe_route_kernel<HIST, 4><<<g, t, 0, c->stream>>>(ROUTE_ARGS);
#undef ROUTE_ARGS
    MOE_LAUNCHED(c);
}

void moe_launch_route(moe_cuda_ctx *c, const float *proj, uint32_t *idx, float *wt, uint32_t *count,
                      uint32_t rows, uint32_t experts, uint32_t topk, uint32_t stride) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "route: experts %u outside 1..512", experts);
    MOE_REQUIRE(c, topk >= 1 && topk <= MOE_MAX_TOPK && topk <= experts, "route: topk %u outside 1..min(16, experts)", topk);
    MOE_REQUIRE(c, stride >= experts, "route: stride %u < experts %u", stride, experts);
    MOE_REQUIRE(c, proj != NULL && idx != NULL && wt != NULL && count != NULL, "route: null buffer");
    if (rows == 0) return;
    int vec_ok = ((uintptr_t)proj % 16 == 0) && (stride % 4 == 0);
    uint32_t blocks = (rows + ROUTE_WARPS - 1) / ROUTE_WARPS;
    uint32_t cap = (uint32_t)c->sm_count * 8u;
    if (blocks > cap) blocks = cap;
    route_dispatch<false>(c, blocks, proj, idx, wt, count, rows, experts, topk, stride, vec_ok);
}

// Fused-layer front end: routing plus the per-block expert table of the scatter
// (block = 8 consecutive rows = 8*topk pairs).  hist has ceil(rows/8) x experts words.
void moe_launch_route_hist(moe_cuda_ctx *c, const float *proj, uint32_t *idx, float *wt, uint32_t *hist,
                           uint32_t rows, uint32_t experts, uint32_t topk, uint32_t stride, uint32_t *ones_a,
                           uint32_t n_a, uint32_t *ones_b, uint32_t n_b) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "route: experts %u outside 1..512", experts);
    MOE_REQUIRE(c, topk >= 1 && topk <= MOE_MAX_TOPK && topk <= experts, "route: topk %u outside 1..min(16, experts)", topk);
    MOE_REQUIRE(c, stride >= experts, "route: stride %u < experts %u", stride, experts);
    MOE_REQUIRE(c, proj != NULL && idx != NULL && wt != NULL && hist != NULL, "route: null buffer");
    if (rows == 0) return;
    int vec_ok = ((uintptr_t)proj % 16 == 0) && (stride % 4 == 0);
    uint32_t blocks = (rows + ROUTE_WARPS - 1) / ROUTE_WARPS;  // exactly one block per 8 rows: no grid stride
    route_dispatch<true>(c, blocks, proj, idx, wt, hist, rows, experts, topk, stride, vec_ok, ones_a, n_a, ones_b, n_b);
}

extern "C" void moe_cuda_route(moe_cuda_ctx_t *c, const float *proj, uint32_t *idx, float *wt, uint32_t *count,
                               struct mda_pc_moe_route_t pc) {
    moe_launch_route(c, proj, idx, wt, count, pc.rows, pc.experts, pc.topk, pc.stride);
}

// shader/moe_scan.comp:14-38: one 512-thread block; pad each count to the tile,
// exclusive prefix sum, one tiles[] entry per padded tile (moe_scan_body, moe_common.cuh).
__global__ void __launch_bounds__(512)
moe_scan_kernel(const uint32_t *__restrict__ count, uint32_t *__restrict__ off, uint32_t *__restrict__ tiles,
                uint32_t experts, uint32_t tile) {
    moe_scan_body(count, off, tiles, experts, tile);
}

void moe_launch_scan(moe_cuda_ctx *c, const uint32_t *count, uint32_t *off, uint32_t *tiles, uint32_t experts,
                     uint32_t tile) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "scan: experts %u outside 1..512", experts);
    MOE_REQUIRE(c, tile >= 1, "scan: tile 0");
    MOE_REQUIRE(c, count != NULL && off != NULL && tiles != NULL, "scan: null buffer");
    moe_scan_kernel<<<1, 512, 0, c->stream>>>(count, off, tiles, experts, tile);
    MOE_LAUNCHED(c);
}

extern "C" void moe_cuda_scan(moe_cuda_ctx_t *c, const uint32_t *count, uint32_t *off, uint32_t *tiles,
                              struct mda_pc_moe_scan_t pc) {
    moe_launch_scan(c, count, off, tiles, pc.experts, pc.tile);
}
