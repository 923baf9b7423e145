// Token permutation into expert-contiguous order: CUDA for sm_100a.
//
// The reference (shader/moe_scatter.comp:22-27) hands out positions with an
// atomic per expert, so its order inside an expert depends on scheduling.  Here
// the position of pair pr = (row, j) is
//     off[e] + #{pr' < pr : idx[pr'] == e},
// i.e. stable by token index, computed without any atomic on the order:
//   1. hist:    blocks of 64 consecutive pairs count their pairs per expert;
//   2. colscan: exclusive prefix sum of those counts over the blocks, per expert;
//   3. place:   each block ranks its own 64 pairs in order, adds the block base,
//               writes slot[], and its 8 warps copy the rows with 128-bit accesses.
// The (blocks x experts) table of steps 1-2 lives in context scratch memory.
#include "moe_common.cuh"

#define SC_PAIRS 64u    // pairs per block
#define SC_MAX_PAIRS 128u
#define SC_THREADS 256u

__global__ void __launch_bounds__(SC_PAIRS)
moe_scatter_hist_kernel(const uint32_t *__restrict__ idx, uint32_t *__restrict__ hist, uint32_t pairs,
                        uint32_t ebound, uint32_t *status) {
    extern __shared__ uint32_t sh[];
    for (uint32_t e = threadIdx.x; e < ebound; e += SC_PAIRS) sh[e] = 0;
    __syncthreads();
    uint32_t pr = blockIdx.x * SC_PAIRS + threadIdx.x;
    if (pr < pairs) {
        uint32_t e = idx[pr];
        if (e < ebound) {
            atomicAdd(&sh[e], 1u);  // a count: order is irrelevant
        } else {
            atomicCAS(status, 0u, (uint32_t)MOE_ERR_ARG | (1u << 8));
        }
    }
    __syncthreads();
    for (uint32_t e = threadIdx.x; e < ebound; e += SC_PAIRS) hist[(size_t)blockIdx.x * ebound + e] = sh[e];
}

// One block per 32 experts; thread (seg, el) sums a contiguous segment of block
// rows for expert el (loads coalesced across el and unrolled so that they
// overlap), the 32 segment sums are scanned, then each thread rewrites its
// segment as exclusive prefixes.  fill[e] grows by the expert's total;
// count_out[e] receives it.
#define CS_EXPERTS 32u
__global__ void __launch_bounds__(1024)
moe_scatter_colscan_kernel(uint32_t *__restrict__ hist, uint32_t *__restrict__ fill, uint32_t nblocks,
                           uint32_t ebound, uint32_t *__restrict__ count_out, uint32_t *ticket, uint32_t *off,
                           uint32_t *tiles, uint32_t tile, uint4 *chunks, uint32_t *n_chunks, uint32_t max_chunks) {
    __shared__ uint32_t seg_sum[32][33];
    __shared__ uint32_t s_last;
    uint32_t el = threadIdx.x & 31u, seg = threadIdx.x >> 5;
    uint32_t e = blockIdx.x * 32u + el;
    uint32_t per = (nblocks + 31u) / 32u;
    uint32_t b0 = min(seg * per, nblocks), b1 = min(b0 + per, nblocks);
    uint32_t s = 0;
    if (e < ebound) {
        uint32_t b = b0;
        for (; b + 8u <= b1; b += 8u) {
            uint32_t v[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; i += 1) v[i] = hist[(size_t)(b + i) * ebound + e];
#pragma unroll
            for (uint32_t i = 0; i < 8; i += 1) s += v[i];
        }
        for (; b < b1; b += 1) s += hist[(size_t)b * ebound + e];
    }
    seg_sum[seg][el] = s;
    __syncthreads();
    uint32_t base = 0;
    for (uint32_t q = 0; q < seg; q += 1) base += seg_sum[q][el];
    if (e < ebound) {
        uint32_t run = base;
        uint32_t b = b0;
        for (; b + 8u <= b1; b += 8u) {
            uint32_t v[8];
#pragma unroll
            for (uint32_t i = 0; i < 8; i += 1) v[i] = hist[(size_t)(b + i) * ebound + e];
#pragma unroll
            for (uint32_t i = 0; i < 8; i += 1) {
                hist[(size_t)(b + i) * ebound + e] = run;
                run += v[i];
            }
        }
        for (; b < b1; b += 1) {
            uint32_t v = hist[(size_t)b * ebound + e];
            hist[(size_t)b * ebound + e] = run;
            run += v;
        }
        if (seg == 31) {
            // state after the shader's atomics (:25).  Only experts that occur are touched, as in the
            // shader: moe_cuda_scatter scans up to the reference's 512 experts, the caller's fill[] may be shorter.
            if (fill != NULL && run != 0) fill[e] += run;
            if (count_out != NULL) count_out[e] = run;  // per-expert totals double as the router's counts
        }
    }
    if (ticket != NULL) {
        // the block that finishes last sees every count and runs the scan (shader/moe_scan.comp) right here
        __threadfence();
        __syncthreads();
        if (threadIdx.x == 0) {
            s_last = atomicAdd(ticket, 1u) == gridDim.x - 1u ? 1u : 0u;
            if (s_last) *ticket = 0;  // ready for the next launch
        }
        __syncthreads();
        if (s_last) {
            __threadfence();
            moe_scan_body(count_out, off, tiles, ebound, tile);
            if (chunks != NULL) {  // and the chunk list of the weight-stationary products, from the same counts and offsets
                __syncthreads();
                moe_chunk_body(count_out, off, ebound, chunks, n_chunks, max_chunks);
            }
        }
    }
}

__global__ void __launch_bounds__(SC_THREADS)
moe_scatter_place_kernel(const uint32_t *__restrict__ idx, const uint32_t *__restrict__ off,
                         const uint32_t *__restrict__ base, const uint4 *__restrict__ x16,
                         uint4 *__restrict__ xp, uint32_t *__restrict__ slot, uint32_t pairs, uint32_t topk,
                         uint32_t d8, uint32_t ebound, uint4 *const *__restrict__ xp_peers, uint32_t experts_per_rank,
                         uint32_t ppb, uint32_t *__restrict__ src_row, uint32_t *const *__restrict__ src_row_peers,
                         uint32_t src_base, uint2 *const *__restrict__ ret_peers, const float *__restrict__ wt) {
    // ppb = pairs per block (<= SC_MAX_PAIRS): 64 in the stand-alone scatter, 8*topk behind the fused router.
    // A block takes pair groups blockIdx.x, blockIdx.x + gridDim.x, ...
    __shared__ uint32_t s_e[SC_MAX_PAIRS];
    __shared__ uint32_t s_slot[SC_MAX_PAIRS];
    __shared__ uint4 *s_dst[SC_MAX_PAIRS];
    const uint32_t ngroups = (pairs + ppb - 1u) / ppb;
    for (uint32_t grp = blockIdx.x; grp < ngroups; grp += gridDim.x) {
        uint32_t p0 = grp * ppb;
        uint32_t np = min(ppb, pairs - p0);
        if (threadIdx.x < SC_MAX_PAIRS) s_e[threadIdx.x] = threadIdx.x < np ? idx[p0 + threadIdx.x] : ~0u;
        __syncthreads();
        if (threadIdx.x < np) {
            uint32_t e = s_e[threadIdx.x];
            if (e < ebound) {
                uint32_t rank = 0;
                for (uint32_t q = 0; q < threadIdx.x; q += 1) rank += s_e[q] == e;
                uint32_t p = off[e] + base[(size_t)grp * ebound + e] + rank;
                s_slot[threadIdx.x] = p;
                // expert-parallel: the row goes straight into the owning GPU's buffer over NVLink
                s_dst[threadIdx.x] = xp_peers != NULL ? xp_peers[e / experts_per_rank] : xp;
                slot[p0 + threadIdx.x] = p;  // :27
                // gather mode: record where the row comes from instead of copying it; the product fetches it
                if (src_row != NULL) src_row[p] = (p0 + threadIdx.x) / topk;
                // expert-parallel gather mode: the record goes into the owning GPU's table; the row itself
                // travels once per destination GPU (moe_ep_send_kernel) and sits at src_base + its local index
                else if (src_row_peers != NULL) {
                    const uint32_t g = e / experts_per_rank, row = src_base + (p0 + threadIdx.x) / topk;
                    src_row_peers[g][p] = row;
                    if (ret_peers != NULL) {
                        // return record: (row of the expert's output, router weight), the token's records on one
                        // GPU packed in j order (ppb is a multiple of topk, so a token's pairs share the block)
                        const uint32_t t0 = threadIdx.x - threadIdx.x % topk;
                        uint32_t jj = 0;
                        for (uint32_t q = t0; q < threadIdx.x; q += 1) jj += (s_e[q] < ebound && s_e[q] / experts_per_rank == g) ? 1u : 0u;
                        ret_peers[g][(size_t)row * topk + jj] = make_uint2(p, __float_as_uint(wt[p0 + threadIdx.x]));
                    }
                }
            } else {
                s_slot[threadIdx.x] = ~0u;
                slot[p0 + threadIdx.x] = ~0u;  // a pair the router refused: the combine skips it
            }
        }
        __syncthreads();
        if (src_row == NULL && src_row_peers == NULL) {
            uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
            for (uint32_t q = warp; q < np; q += SC_THREADS / 32u) {
                uint32_t p = s_slot[q];
                if (p == ~0u) continue;
                uint32_t r = (p0 + q) / topk;  // :20
                const uint4 *src = x16 + (size_t)r * d8;
                uint4 *dst = s_dst[q] + (size_t)p * d8;
                uint32_t i = lane;
                for (; i + 96u < d8; i += 128u) {  // four 16-byte loads in flight per lane
                    uint4 a = __ldg(src + i), b = __ldg(src + i + 32u), c2 = __ldg(src + i + 64u), d2 = __ldg(src + i + 96u);
                    dst[i] = a;
                    dst[i + 32u] = b;
                    dst[i + 64u] = c2;
                    dst[i + 96u] = d2;
                }
                for (; i < d8; i += 32u) dst[i] = __ldg(src + i);  // :30-32
            }
            __syncthreads();  // the tables are rewritten by the next group
        }
    }
}

void moe_launch_scatter(moe_cuda_ctx *c, const uint32_t *idx, const uint32_t *off, uint32_t *fill, const void *x16,
                        void *xp, uint32_t *slot, uint32_t rows, uint32_t topk, uint32_t d8, uint32_t ebound,
                        void *const *xp_peers, uint32_t experts_per_rank) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, idx != NULL && off != NULL && x16 != NULL && xp != NULL && slot != NULL, "scatter: null buffer");
    MOE_REQUIRE(c, topk >= 1 && d8 >= 1 && ebound >= 1 && ebound <= MOE_MAX_EXPERTS, "scatter: bad shape");
    MOE_REQUIRE(c, ((uintptr_t)x16 & 15) == 0 && ((uintptr_t)xp & 15) == 0, "scatter: rows not 16-byte aligned");
    uint64_t pairs64 = (uint64_t)rows * topk;
    MOE_REQUIRE(c, pairs64 < (1ull << 31), "scatter: too many pairs");
    uint32_t pairs = (uint32_t)pairs64;
    if (pairs == 0) return;
    uint32_t nblocks = (pairs + SC_PAIRS - 1) / SC_PAIRS;
    uint32_t *hist = (uint32_t *)moe_scratch(c, MOE_SCR_SCATTER, (size_t)nblocks * ebound * sizeof(uint32_t));
    if (hist == NULL) return;
    moe_scatter_hist_kernel<<<nblocks, SC_PAIRS, ebound * sizeof(uint32_t), c->stream>>>(idx, hist, pairs, ebound,
                                                                                         c->dev_status_dev);
    MOE_LAUNCHED(c);
    moe_scatter_colscan_kernel<<<(ebound + CS_EXPERTS - 1u) / CS_EXPERTS, 1024, 0, c->stream>>>(hist, fill, nblocks, ebound, NULL, NULL, NULL, NULL, 0, NULL, NULL, 0);
    MOE_LAUNCHED(c);
    moe_scatter_place_kernel<<<nblocks, SC_THREADS, 0, c->stream>>>(idx, off, hist, (const uint4 *)x16, (uint4 *)xp,
                                                                    slot, pairs, topk, d8, ebound,
                                                                    (uint4 *const *)xp_peers, experts_per_rank, SC_PAIRS, NULL, NULL, 0, NULL, NULL);
    MOE_LAUNCHED(c);
}

// Fused front end, after the router wrote the per-8-row tables into `hist`:
// column scan in place (block bases for the ranking) which also yields count[].
void moe_launch_colscan_counts(moe_cuda_ctx *c, uint32_t *hist, uint32_t *count, uint32_t rows, uint32_t experts,
                               uint32_t *off, uint32_t *tiles, uint32_t tile, void *chunks, uint32_t *n_chunks,
                               uint32_t max_chunks) {
    if (!MOE_LIVE(c)) return;
    if (rows == 0) return;
    uint32_t nblocks = (rows + 7u) / 8u;
    uint32_t *ticket = NULL;
    if (off != NULL) {
        if (c->ticket == NULL) {
            c->ticket = (uint32_t *)moe_cuda_alloc(c, 64);
            if (c->ticket == NULL) return;
            MOE_CUDA_TRY(c, cudaMemsetAsync(c->ticket, 0, 64, c->stream));
        }
        ticket = c->ticket;
    }
    moe_scatter_colscan_kernel<<<(experts + CS_EXPERTS - 1u) / CS_EXPERTS, 1024, 0, c->stream>>>(hist, NULL, nblocks, experts, count,
                                                                                                 ticket, off, tiles, tile,
                                                                                                 (uint4 *)chunks, n_chunks, max_chunks);
    MOE_LAUNCHED(c);
}

void moe_overlap_prepare_scatter(moe_cuda_ctx *c) {
    MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_scatter_place_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared));
    MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_scatter_colscan_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared));
}

// Ranking + row copies for blocks of 8 rows (8*topk pairs), bases from `hist`.
void moe_launch_place(moe_cuda_ctx *c, const uint32_t *idx, const uint32_t *off, const uint32_t *hist, const void *x16,
                      void *xp, uint32_t *slot, uint32_t rows, uint32_t topk, uint32_t d8, uint32_t experts,
                      void *const *xp_peers, uint32_t experts_per_rank, uint32_t *src_row, uint32_t *const *src_row_peers,
                      uint32_t src_base, uint2 *const *ret_peers, const float *wt) {
    if (!MOE_LIVE(c)) return;
    if (rows == 0) return;
    MOE_REQUIRE(c, ((uintptr_t)x16 & 15) == 0 && ((uintptr_t)xp & 15) == 0, "scatter: rows not 16-byte aligned");
    uint32_t nblocks = (rows + 7u) / 8u;
    moe_scatter_place_kernel<<<nblocks, SC_THREADS, 0, c->stream>>>(idx, off, hist, (const uint4 *)x16, (uint4 *)xp, slot,
                                                                    rows * topk, topk, d8, experts,
                                                                    (uint4 *const *)xp_peers, experts_per_rank, 8u * topk, src_row,
                                                                    src_row_peers, src_base, ret_peers, wt);
    MOE_LAUNCHED(c);
}

extern "C" void moe_cuda_scatter(moe_cuda_ctx_t *c, const uint32_t *idx, const uint32_t *off, uint32_t *fill,
                                 const void *x16, void *xp, uint32_t *slot, struct mda_pc_moe_scatter_t pc) {
    // The push constants carry no expert count (src/pc.h:381-385); the table is
    // sized for the reference's limit of 512.
    moe_launch_scatter(c, idx, off, fill, x16, xp, slot, pc.rows, pc.topk, pc.d8, MOE_MAX_EXPERTS, NULL, 0);
}

// ---- scatter without any allocation ---------------------------------------
// Same three kernels, but the (blocks x experts) table lives in a fixed array in
// device global memory that the library image carries, instead of context
// scratch that grows with cudaMalloc.  Every GPU that loads the library holds
// these MOE_NOALLOC_SCATTER_WORDS * 4 bytes until the process exits.
static __device__ __align__(256) uint32_t g_scatter_noalloc_table[MOE_NOALLOC_SCATTER_WORDS];

#define MOE_NOALLOC_MAX_DEVICES 64
// In host code the array's name is only a handle for the runtime, not a device
// address; the address each device gives it is looked up once per device.
static uint32_t *g_scatter_noalloc_ptr[MOE_NOALLOC_MAX_DEVICES];

extern "C" void moe_cuda_scatter_noalloc(moe_cuda_ctx_t *c, const uint32_t *idx, const uint32_t *off,
                                         uint32_t *fill, const void *x16, void *xp, uint32_t *slot,
                                         struct mda_pc_moe_scatter_t pc, uint32_t experts) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, c->device >= 0 && c->device < MOE_NOALLOC_MAX_DEVICES, "scatter_noalloc: device %d outside 0..63", c->device);
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "scatter_noalloc: experts %u outside 1..512", experts);
    uint64_t pairs = (uint64_t)pc.rows * pc.topk;
    uint64_t nblocks = (pairs + SC_PAIRS - 1) / SC_PAIRS;
    MOE_REQUIRE(c, nblocks * experts <= (uint64_t)MOE_NOALLOC_SCATTER_WORDS,
                "scatter_noalloc: ceil(rows*topk/64)*experts = %llu exceeds the fixed table of %u words; "
                "use moe_cuda_scatter or fewer rows per call",
                (unsigned long long)(nblocks * experts), (unsigned)MOE_NOALLOC_SCATTER_WORDS);
    if (g_scatter_noalloc_ptr[c->device] == NULL) {
        // First call on this device: resolve the table's device address with that
        // device current.  This is a runtime query, not an allocation.
        int cur = -1;
        MOE_CUDA_TRY(c, cudaGetDevice(&cur));
        if (cur != c->device) MOE_CUDA_TRY(c, cudaSetDevice(c->device));
        uint32_t *p = NULL;
        cudaError_t e = cudaGetSymbolAddress((void **)&p, g_scatter_noalloc_table);
        if (cur != c->device) cudaSetDevice(cur);
        if (e != cudaSuccess || p == NULL) {
            moe_fail(c, MOE_ERR_CUDA, "scatter_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return;
        }
        g_scatter_noalloc_ptr[c->device] = p;
    }
    uint32_t *table = g_scatter_noalloc_ptr[c->device];
    MOE_REQUIRE(c, idx != NULL && off != NULL && x16 != NULL && xp != NULL && slot != NULL, "scatter_noalloc: null buffer");
    MOE_REQUIRE(c, pc.topk >= 1 && pc.d8 >= 1, "scatter_noalloc: bad shape");
    MOE_REQUIRE(c, ((uintptr_t)x16 & 15) == 0 && ((uintptr_t)xp & 15) == 0, "scatter_noalloc: rows not 16-byte aligned");
    if (pairs == 0) return;
    // The table keeps the previous call's contents; nothing has to start at zero
    // because the hist kernel writes every entry the later kernels read.
    moe_scatter_hist_kernel<<<(uint32_t)nblocks, SC_PAIRS, experts * sizeof(uint32_t), c->stream>>>(
        idx, table, (uint32_t)pairs, experts, c->dev_status_dev);
    MOE_LAUNCHED(c);
    moe_scatter_colscan_kernel<<<(experts + CS_EXPERTS - 1u) / CS_EXPERTS, 1024, 0, c->stream>>>(table, fill, (uint32_t)nblocks, experts, NULL, NULL, NULL, NULL, 0, NULL, NULL, 0);
    MOE_LAUNCHED(c);
    moe_scatter_place_kernel<<<(uint32_t)nblocks, SC_THREADS, 0, c->stream>>>(
        idx, off, table, (const uint4 *)x16, (uint4 *)xp, slot, (uint32_t)pairs, pc.topk, pc.d8, experts, NULL, 0, SC_PAIRS, NULL, NULL, 0, NULL, NULL);
    MOE_LAUNCHED(c);
}
