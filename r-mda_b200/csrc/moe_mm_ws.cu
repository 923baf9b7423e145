// Grouped expert products, weight-stationary form, for the fused layer: the
// MMA's M dimension runs over weight rows (output features), its N dimension
// over the tokens of one expert.  Compared with the token-major kernel in
// moe_mm.cu (the reference's 128-row tile schedule, shader/matmul_f16_moe.comp):
//   * an expert's rows are cut into chunks of at most 256 tokens whose MMA width
//     is rounded to 16, not 128, so ragged expert sizes waste almost no tensor
//     work (the reference pads every expert to 128 rows);
//   * with PAIR = 2 two CTAs of a cluster issue one tcgen05.mma.cta_group::2
//     (M 256) over a shared token tile: each CTA loads its own 128 weight rows
//     and only half of the token tile, i.e. 32 KB instead of 48 KB of operands
//     per 64-wide K step and SM.  The loads are plain per-CTA TMA tile loads.
// D lands transposed in tensor memory (lane = feature, column = token); the
// epilogue warps turn it round through a small shared-memory tile so that global
// stores are 16 bytes wide and row-contiguous.
// SWIGLU mode: a 4-D tensor map over [expert][gate|up][inter][d] lets TMA fetch 64
// gate rows and the matching 64 up rows interleaved (row 2i = gate i, row 2i+1 =
// up i), so the two values of an output sit in neighbouring lanes of one warp and
// meet with one shuffle; silu(gate)*up (shader/qwen_elem.comp:20-31 op 0) and the
// fp16 store are the epilogue.
// Every spin on an mbarrier is bounded; on timeout the kernel records
// MOE_ERR_TIMEOUT in the context's status word and unwinds.
#include <stdlib.h>

#include "moe_tc.cuh"

namespace {

using namespace moe_tc;

constexpr uint32_t BK = 64;
constexpr uint32_t W_BYTES = 128 * BK * 2;   // 16 KB: this CTA's 128 weight rows
constexpr uint32_t MAX_TOK = 256;            // tokens per chunk = MMA N
constexpr uint32_t WS_THREADS = 352;        // warps: 0 weight loads, 1 MMA issue, 2..5 epilogue, 6 token loads, 7..10 more loads
constexpr uint32_t NPROD = 3;               // issuing threads per operand, taking K steps in turn
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t ET = 32;                  // tokens per epilogue step (one tcgen05.ld of 32 columns)
constexpr uint32_t PITCH_SW = 160;           // bytes per token row of the turn-round tile, SwiGLU (64 fp16 + pad)
constexpr uint32_t PITCH_F16 = 256;          // the same for 128 fp16 features
constexpr uint32_t TURN_BYTES = 2 * ET * PITCH_F16;  // two buffers

template <int PAIR>
struct Geo {
    static constexpr uint32_t X_BYTES = MAX_TOK / PAIR * BK * 2;  // this CTA's share of the token tile
    static constexpr uint32_t STAGE_BYTES = W_BYTES + X_BYTES;
    static constexpr uint32_t STAGES = PAIR == 2 ? 6 : 4;         // 192 KB of operands either way (3 stages measured only 9 % slower)
};

struct __align__(8) WsBarriers {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};

template <int PAIR>
constexpr uint32_t ws_smem() {
    return Geo<PAIR>::STAGES * Geo<PAIR>::STAGE_BYTES + TURN_BYTES + sizeof(WsBarriers) + 1024;
}

struct WsArgs {
    void *C;
    const uint4 *chunks;       // (expert, first row, MMA width, valid rows)
    const uint32_t *n_chunks;
    uint32_t n;                // weight rows per expert (2*inter, or d)
    uint32_t k;
    uint32_t ldc;              // row stride of C in elements
    uint32_t *status;
    uint64_t wait_ns;
    unsigned long long *prof;  // per CTA 8 cycle counters, or NULL
    unsigned long long *trace; // profiling builds: event trace, or NULL
    uint32_t dbg;              // profiling builds only: 1 no MMA, 2 no token loads, 4 no weight loads, 8 no stores, 32 no epilogue
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t saddr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(saddr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// TMA tile loads issued by either CTA of a pair; the completion bytes are counted
// on the barrier at cluster address `bar` (the leader's).  Not multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1,
                                                 int32_t c2, int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1, int32_t c2,
                                            int32_t c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        :
        : "r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
template <int PAIR>
__device__ __forceinline__ void tma_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1) {
    if (PAIR == 2) tma_load_2d_pair(dst, map, bar, c0, c1);
    else tma_load_2d(dst, map, bar, c0, c1);
}
template <int PAIR>
__device__ __forceinline__ void tma_4d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1, int32_t c2,
                                       int32_t c3) {
    if (PAIR == 2) tma_load_4d_pair(dst, map, bar, c0, c1, c2, c3);
    else tma_load_4d(dst, map, bar, c0, c1, c2, c3);
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
}
// One commit that arrives on the barrier at the same shared-memory offset in both CTAs of the pair.
__device__ __forceinline__ void umma_commit_both(uint32_t local_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(local_bar),
                 "h"((uint16_t)3)
                 : "memory");
}
// All 128 epilogue threads agree on whether to go on (named barrier 1).
__device__ __forceinline__ bool epi_all(bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.and.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}\n"
        : "=r"(r)
        : "r"(ok ? 1u : 0u)
        : "memory");
    return r != 0;
}
__device__ __forceinline__ void epi_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Token rows per TMA box: the smallest multiple of 16 up to 128 that covers what is left.
__device__ __forceinline__ uint32_t x_box_rows(uint32_t left) { return left > 112u ? 128u : (left + 15u) & ~15u; }
__device__ __forceinline__ uint32_t x_rows_loaded(uint32_t half) {
    uint32_t rows = 0;
    for (uint32_t done = 0; done < half; done += x_box_rows(half - done)) rows += x_box_rows(half - done);
    return rows;
}
struct XMaps {
    CUtensorMap m[8];  // boxes of 16, 32, ... 128 token rows
#ifdef MOE_WS_PROF
    CUtensorMap wc;    // experiment: the weight bank as rows of 512 bytes, 16 KB contiguous per box
#endif
};

// Profiling builds: event trace of the first two CTAs (one pair), 8 timestamps per K step, 512 K steps.
#define WS_TRACE_STEPS 512u
__device__ __forceinline__ void ws_trace(unsigned long long *trace, uint32_t step, uint32_t slot) {
    if (trace != NULL && blockIdx.x < 2u && step < WS_TRACE_STEPS) {
        trace[((size_t)blockIdx.x * WS_TRACE_STEPS + step) * 8u + slot] = (unsigned long long)clock64();
    }
}

struct WsItem {
    uint32_t e, row0, ntok, nvalid, ft;
};

__device__ __forceinline__ void ws_item(const WsArgs &a, uint32_t w, uint32_t ft_count, WsItem &it) {
    uint32_t c = w / ft_count;
    it.ft = w - c * ft_count;
    uint4 ch = a.chunks[c];
    it.e = ch.x;
    it.row0 = ch.y;
    it.ntok = ch.z;
    it.nvalid = ch.w;
}

template <int MODE, int PAIR, bool PROF>
__global__ void __launch_bounds__(WS_THREADS, 1)
moe_mm_ws_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ XMaps tmX, WsArgs a) {
    using G = Geo<PAIR>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *turn = smem + G::STAGES * G::STAGE_BYTES;
    WsBarriers *bars = reinterpret_cast<WsBarriers *>(turn + TURN_BYTES);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = PAIR == 2 ? cluster_rank() : 0u;
    volatile uint32_t *abort = &bars->abort;

    // feature tiles: SwiGLU 64 outputs (64 gate + 64 up rows) per CTA, otherwise 128 weight rows per CTA
    const uint32_t ft_count = MODE == MOE_MM_SWIGLU_F16 ? (a.n / 2u) / (64u * PAIR) : a.n / (128u * PAIR);
    const uint32_t total = *a.n_chunks * ft_count;
    const uint32_t kblocks = (a.k + BK - 1) / BK;
    const uint32_t cluster_id = blockIdx.x / PAIR, n_clusters = gridDim.x / PAIR;
    long long t_begin = 0;
    if (PROF) t_begin = clock64();

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < G::STAGES; s += 1) {
            mbar_init(smem_u32(&bars->full[s]), 1);
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (uint32_t s = 0; s < 2; s += 1) {
            mbar_init(smem_u32(&bars->tmem_full[s]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[s]), 4 * PAIR);  // one arrival per epilogue warp of each CTA
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        if (PAIR == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                         "r"(TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) cluster_sync_all();  // the peer's barriers exist before anything is sent to them
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0 || warp >= 6) {
        // ---------------- TMA producers (both CTAs) ----------------
        // One thread gets at most one tile load issued per ~300 ns, whatever its size (measured: 4 KB to 32 KB
        // boxes, tiled or untiled, L2 or HBM source; threads of different warps add up).  A K step of the
        // tensor pipe is shorter than that, so each operand has NPROD issuing threads that take K steps in
        // turn: warps 0, 7, 9 load weight tiles, warps 6, 8, 10 token tiles.  All follow the same stage ring;
        // the completion bytes of the four loads of a stage (two CTAs x two operands) are counted on the
        // leader's full barrier, whose one arrival is the weight producer's expect_tx.
        if (lane == 0) {
            const bool wprod = warp == 0 || (warp >= 7 && (warp & 1u) != 0);
            const uint32_t turn_of = warp < 7 ? 0u : (warp - 5u) / 2u;  // 0, 1, 2: which K steps this thread takes
            const uint32_t dbg = PROF ? a.dbg : 0u;
            uint32_t s = 0, ph = 0, issued = 0, last_par = 0, step = 0, gstep = 0;
            long long waited = 0, issue_busy = 0;
            bool ok = true;
            for (uint32_t w = cluster_id; w < total && ok && !(dbg & 512u); w += n_clusters) {
                WsItem it;
                ws_item(a, w, ft_count, it);
                const uint32_t half = it.ntok / PAIR;            // token rows this CTA loads
                const uint32_t xbytes = (dbg & 2u) ? 0u : x_rows_loaded(half) * (BK * 2u);
                const uint32_t wbytes = (dbg & 4u) ? 0u : W_BYTES;
                const int32_t f0 = (int32_t)((it.ft * PAIR + rank) * (MODE == MOE_MM_SWIGLU_F16 ? 64u : 128u));
                const int32_t xrow = (int32_t)(it.row0 + rank * half);
                for (uint32_t kb = 0; kb < kblocks; kb += 1, gstep += 1) {
                    if (gstep % NPROD != turn_of) continue;
                    s = gstep % G::STAGES;
                    ph = (gstep / G::STAGES) & 1u;
                    long long t0 = 0;
                    if (PROF) t0 = clock64();
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort, a.status, wprod ? 11 : 15, a.wait_ns)) {
                        ok = false;
                        break;
                    }
                    long long t1 = 0;
                    if (PROF) {
                        t1 = clock64();
                        waited += t1 - t0;
                        ws_trace(a.trace, step, wprod ? 0u : 2u);
                    }
                    const uint32_t base = stage0 + s * G::STAGE_BYTES;
                    const int32_t kc = (int32_t)(kb * BK);
                    const uint32_t full = PAIR == 2 ? map_to_cta(smem_u32(&bars->full[s]), 0) : smem_u32(&bars->full[s]);
                    if (wprod) {
                        if (rank == 0) mbar_expect_tx(smem_u32(&bars->full[s]), (uint32_t)PAIR * (wbytes + xbytes));
                        if (PROF && (dbg & 64u)) {
#ifdef MOE_WS_PROF
                            // experiment: same bytes, but each tile one contiguous 16 KB piece of the bank
                            const uint32_t tile = (it.e * ft_count * PAIR + it.ft * PAIR + rank) * kblocks + kb;
                            tma_2d<PAIR>(base, &tmX.wc, full, 0, (int32_t)(tile * 32u));
#endif
                        } else if (wbytes != 0u) {
                            if (MODE == MOE_MM_SWIGLU_F16) tma_4d<PAIR>(base, &tmW, full, kc, 0, f0, (int32_t)it.e);
                            else tma_2d<PAIR>(base, &tmW, full, kc, (int32_t)(it.e * a.n) + f0);
                        }
                    } else if (xbytes != 0u) {
                        uint32_t done = 0;
                        while (done < half) {  // boxes of 16, 32, ... 128 token rows: at most 15 rows more than needed
                            const uint32_t rows = x_box_rows(half - done);
                            tma_2d<PAIR>(base + W_BYTES + done * (BK * 2u), &tmX.m[rows / 16u - 1u], full, kc, xrow + (int32_t)done);
                            done += rows;
                        }
                    }
                    if (PROF) {
                        issue_busy += clock64() - t1;
                        ws_trace(a.trace, step, wprod ? 1u : 3u);
                        step += 1;
                    }
                    issued |= 1u << s;
                    last_par = (last_par & ~(1u << s)) | (ph << s);
                }
            }
            if (!ok && rank == 0 && wprod) {
                for (uint32_t q = 0; q < G::STAGES; q += 1) {  // bounded wait for copies in flight
                    if (((issued >> q) & 1u) == 0) continue;
                    for (uint32_t spin = 0; spin < (1u << 16); spin += 1) {
                        if (mbar_try_wait(smem_u32(&bars->full[q]), (last_par >> q) & 1u)) break;
                    }
                }
            }
            if (PROF && a.prof != NULL && turn_of == 0) {
                a.prof[blockIdx.x * 16u + (wprod ? 1u : 8u)] = (unsigned long long)waited;
                a.prof[blockIdx.x * 16u + (wprod ? 9u : 10u)] = (unsigned long long)issue_busy;
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        // The whole warp runs the loop, so that barrier addresses and descriptors are warp-uniform values, and one
        // elected lane issues; one look at the full barriers covers the whole ring (mbar_ring_wait).
        if (rank == 0) {
            uint32_t gstep = 0, n_item = 0, ready = 0;
            long long wait_full = 0, wait_acc = 0;
            bool ok = true;
            for (uint32_t w = cluster_id; w < total && ok; w += n_clusters) {
                WsItem it;
                ws_item(a, w, ft_count, it);
                const uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
                long long t0 = 0;
                if (PROF) t0 = clock64();
                if (!mbar_wait(smem_u32(&bars->tmem_empty[as]), aph ^ 1u, abort, a.status, 12, a.wait_ns)) break;
                if (PROF) wait_acc += clock64() - t0;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * MAX_TOK;
                const uint32_t idesc = umma_idesc(128u * PAIR, it.ntok);
                for (uint32_t kb = 0; kb < kblocks; kb += 1, gstep += 1) {
                    const uint32_t s = gstep % G::STAGES;
                    if (PROF) t0 = clock64();
                    if (!(PROF && (a.dbg & 512u)) && ((ready >> s) & 1u) == 0 &&
                        !mbar_ring_wait<G::STAGES>(bars->full, gstep, ready, abort, a.status, 13, a.wait_ns)) {
                        ok = false;
                        break;
                    }
                    ready &= ~(1u << s);
                    if (PROF) {
                        wait_full += clock64() - t0;
                        if (lane == 0) ws_trace(a.trace, gstep, 4u);
                    }
                    tc_fence_after();
                    const uint32_t base = stage0 + s * G::STAGE_BYTES;
                    const uint64_t ad = umma_desc(base), bd = umma_desc(base + W_BYTES);
                    if (elect_one()) {
                        if (!(PROF && (a.dbg & 1u))) {
#pragma unroll
                            for (uint32_t kk = 0; kk < BK / 16; kk += 1) {
                                if (PAIR == 2) umma_f16_pair(tmem_d, ad + 2ull * kk, bd + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                                else umma_f16(tmem_d, ad + 2ull * kk, bd + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                            }
                        }
                        if (PROF && (a.dbg & 512u)) {  // experiment: tensor pipe alone, nothing is loaded, no stage hand-off
                        } else if (PAIR == 2) umma_commit_both(smem_u32(&bars->empty[s]));  // frees the stage in both CTAs
                        else umma_commit(smem_u32(&bars->empty[s]));
                    }
                    __syncwarp();
                    if (PROF && lane == 0) ws_trace(a.trace, gstep, 5u);
                }
                if (ok && elect_one()) {
                    if (PAIR == 2) umma_commit_both(smem_u32(&bars->tmem_full[as]));
                    else umma_commit(smem_u32(&bars->tmem_full[as]));
                }
                __syncwarp();
                n_item += 1;
            }
            if (PROF && a.prof != NULL && lane == 0) {
                a.prof[blockIdx.x * 16u + 2u] = (unsigned long long)wait_full;
                a.prof[blockIdx.x * 16u + 3u] = (unsigned long long)wait_acc;
                a.prof[blockIdx.x * 16u + 6u] = n_item;
                a.prof[blockIdx.x * 16u + 7u] = gstep;
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const uint32_t q = warp & 3u;    // TMEM lane quarter this warp may read
        const uint32_t ew = warp - 2u;   // 0..3: which rows of the turn-round tile this warp stores
        const uint32_t empty_leader = PAIR == 2 ? map_to_cta(smem_u32(&bars->tmem_empty[0]), 0) : smem_u32(&bars->tmem_empty[0]);
        uint32_t n_item = 0, tb = 0;
        long long wait_acc = 0, busy = 0;
        for (uint32_t w = cluster_id; w < total; w += n_clusters) {
            WsItem it;
            ws_item(a, w, ft_count, it);
            const uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
            long long t0 = 0;
            if (PROF) t0 = clock64();
            bool ok = true;
            if (lane == 0) ok = mbar_wait(smem_u32(&bars->tmem_full[as]), aph, abort, a.status, 14, a.wait_ns);
            if (!epi_all(ok)) break;
            long long t1 = 0;
            if (PROF) {
                t1 = clock64();
                wait_acc += t1 - t0;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + as * MAX_TOK + ((q * 32u) << 16);
            uint32_t nch = (it.ntok + ET - 1u) / ET;
            if (PROF && (a.dbg & 8u)) it.nvalid = 0;
            if (PROF && (a.dbg & 32u)) nch = 0;
            if (MODE == MOE_MM_SWIGLU_F16) {
                // lane 2i holds gate feature i of this warp's 16, lane 2i+1 the matching up feature
                const uint32_t fl = q * 16u + (lane >> 1);
                const uint32_t odd = lane & 1u;
                __half *out = reinterpret_cast<__half *>(a.C) + (size_t)it.row0 * a.ldc + (it.ft * PAIR + rank) * 64u + (lane & 7u) * 8u;
#pragma unroll 1
                for (uint32_t cch = 0; cch < nch; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * ET, v);
                    tmem_ld_wait();
                    uint8_t *tp = turn + tb * ET * PITCH_F16;
                    __half *mine = reinterpret_cast<__half *>(tp + odd * PITCH_SW) + fl;
#pragma unroll
                    for (uint32_t jj = 0; jj < 16; jj += 1) {
                        const uint32_t send = odd ? v[2 * jj] : v[2 * jj + 1];
                        const uint32_t recv = __shfl_xor_sync(0xffffffffu, send, 1);
                        const float g = __uint_as_float(odd ? recv : v[2 * jj]);
                        const float u = __uint_as_float(odd ? v[2 * jj + 1] : recv);
                        const float h = __fdividef(g, 1.0f + __expf(-g)) * u;
                        mine[jj * (2u * PITCH_SW / 2u)] = __float2half_rn(h);  // token 2jj + odd
                    }
                    epi_sync();
                    const uint32_t t0c = cch * ET;
#pragma unroll
                    for (uint32_t i = 0; i < 2; i += 1) {
                        const uint32_t r = ew * 8u + i * 4u + (lane >> 3);
                        if (t0c + r < it.nvalid) {
                            const uint4 val = *reinterpret_cast<const uint4 *>(tp + r * PITCH_SW + (lane & 7u) * 16u);
                            *reinterpret_cast<uint4 *>(out + (size_t)(t0c + r) * a.ldc) = val;
                        }
                    }
                    tb ^= 1u;
                }
            } else if (MODE == MOE_MM_F16) {
                const uint32_t fl = q * 32u + lane;
                __half *out = reinterpret_cast<__half *>(a.C) + (size_t)it.row0 * a.ldc + (it.ft * PAIR + rank) * 128u + (lane & 15u) * 8u;
#pragma unroll 1
                for (uint32_t cch = 0; cch < nch; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * ET, v);
                    tmem_ld_wait();
                    uint8_t *tp = turn + tb * ET * PITCH_F16;
                    __half *mine = reinterpret_cast<__half *>(tp) + fl;
#pragma unroll
                    for (uint32_t j = 0; j < 32; j += 1) mine[j * (PITCH_F16 / 2u)] = __float2half_rn(__uint_as_float(v[j]));
                    epi_sync();
                    const uint32_t t0c = cch * ET;
#pragma unroll
                    for (uint32_t i = 0; i < 4; i += 1) {
                        const uint32_t r = ew * 8u + i * 2u + (lane >> 4);
                        if (t0c + r < it.nvalid) {
                            const uint4 val = *reinterpret_cast<const uint4 *>(tp + r * PITCH_F16 + (lane & 15u) * 16u);
                            *reinterpret_cast<uint4 *>(out + (size_t)(t0c + r) * a.ldc) = val;
                        }
                    }
                    tb ^= 1u;
                }
            } else {
                // fp32 output: 32 lanes = 32 neighbouring features = one 128-byte piece of a token's row per store
                const uint32_t cfeat = (it.ft * PAIR + rank) * 128u + q * 32u + lane;
#pragma unroll 1
                for (uint32_t cch = 0; cch < nch; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * ET, v);
                    tmem_ld_wait();
                    const uint32_t t0c = cch * ET;
                    float *out = reinterpret_cast<float *>(a.C) + (size_t)(it.row0 + t0c) * a.ldc + cfeat;
#pragma unroll
                    for (uint32_t j = 0; j < 32; j += 1) {
                        if (t0c + j < it.nvalid) out[(size_t)j * a.ldc] = __uint_as_float(v[j]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR == 2) mbar_arrive_cluster(empty_leader + as * 8u);
                else mbar_arrive(empty_leader + as * 8u);
            }
            if (PROF) busy += clock64() - t1;
            n_item += 1;
        }
        if (PROF && a.prof != NULL && warp == 2 && lane == 0) {
            a.prof[blockIdx.x * 16u + 4u] = (unsigned long long)wait_acc;
            a.prof[blockIdx.x * 16u + 5u] = (unsigned long long)busy;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR == 2) cluster_sync_all();  // neither CTA leaves while the other may still touch its memory
    if (warp == 1) {
        tc_fence_after();
        if (PAIR == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
    if (PROF && a.prof != NULL && threadIdx.x == 0) a.prof[blockIdx.x * 16u] = (unsigned long long)(clock64() - t_begin);
}

// The chunk list as a kernel of its own (expert-parallel layer: the counts come from the plan): one block, thread =
// expert.  The single-GPU layer builds the same list in the last block of its column scan.
static_assert(MAX_TOK == MOE_CHUNK_TOK, "the chunk list is cut for the MMA width of this kernel");
__global__ void __launch_bounds__(512)
moe_chunk_kernel(const uint32_t *__restrict__ count, const uint32_t *__restrict__ off, uint32_t experts,
                 uint4 *__restrict__ chunks, uint32_t *__restrict__ n_chunks, uint32_t max_chunks) {
    moe_chunk_body(count, off, experts, chunks, n_chunks, max_chunks);
}

#ifdef MOE_WS_PROF
__device__ unsigned long long g_ws_prof[256 * 16];
__device__ unsigned long long g_ws_trace[2 * WS_TRACE_STEPS * 8];
#endif

template <int MODE, int PAIR>
void ws_launch(moe_cuda_ctx *c, const CUtensorMap *tmW, const XMaps &tmX, WsArgs &a, uint32_t grid) {
#ifdef MOE_WS_PROF
    constexpr bool PROF = true;
    MOE_CUDA_TRY(c, cudaGetSymbolAddress((void **)&a.prof, g_ws_prof));
    MOE_CUDA_TRY(c, cudaGetSymbolAddress((void **)&a.trace, g_ws_trace));
    const char *dbg = getenv("MOE_WS_DBG");
    a.dbg = dbg != NULL ? (uint32_t)atoi(dbg) : 0u;
    const char *only = getenv("MOE_WS_PROF_MODE");  // counters of one product only (1: gate_up, 2: down)
    if (only != NULL && atoi(only) != MODE) a.prof = NULL;
#else
    constexpr bool PROF = false;
#endif
    int slot = MODE * 2 + (PAIR - 1);
    if (!c->sw_attr_set[slot]) {
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_mm_ws_kernel<MODE, PAIR, PROF>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)ws_smem<PAIR>()));
        c->sw_attr_set[slot] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(WS_THREADS, 1, 1);
    cfg.dynamicSmemBytes = ws_smem<PAIR>();
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MOE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, moe_mm_ws_kernel<MODE, PAIR, PROF>, *tmW, tmX, a));
    c->launches += 1;
}

}  // namespace

#ifdef MOE_WS_PROF
extern "C" void moe_ws_prof_read(unsigned long long *out, int words) {
    cudaMemcpyFromSymbol(out, g_ws_prof, (size_t)words * 8);
}
extern "C" void moe_ws_trace_read(unsigned long long *out, int words) {
    cudaMemcpyFromSymbol(out, g_ws_trace, (size_t)words * 8);
}
#endif

void moe_launch_chunks(moe_cuda_ctx *c, const uint32_t *count, const uint32_t *off, uint32_t experts, void *chunks,
                       uint32_t *n_chunks, uint32_t max_chunks) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "chunks: experts %u outside 1..512", experts);
    moe_chunk_kernel<<<1, 512, 0, c->stream>>>(count, off, experts, (uint4 *)chunks, n_chunks, max_chunks);
    MOE_LAUNCHED(c);
}

// X [rows_x x k] fp16 token rows, W [experts_in_W][n x k] fp16, C token-major with row stride ldc.
void moe_launch_mm_ws(moe_cuda_ctx *c, int mode, int pair, const void *X, uint32_t rows_x, const void *W,
                      uint32_t experts_in_W, void *C, uint32_t ldc, const void *chunks, const uint32_t *n_chunks,
                      uint32_t max_chunks, uint32_t n, uint32_t k) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, X != NULL && W != NULL && C != NULL && chunks != NULL && n_chunks != NULL, "mm_ws: null buffer");
    MOE_REQUIRE(c, pair == 1 || pair == 2, "mm_ws: pair %d", pair);
    MOE_REQUIRE(c, n % (128u * (uint32_t)pair) == 0, "mm_ws: n %u does not tile into %d x 128 weight rows", n, pair);
    MOE_REQUIRE(c, k % 8u == 0 && k >= 8u && rows_x >= 1, "mm_ws: k %u", k);
    MOE_REQUIRE(c, (uint64_t)experts_in_W * n < (1ull << 31), "mm_ws: expert count");
    MOE_REQUIRE(c, ((uintptr_t)C & 15) == 0 && (mode == MOE_MM_F32 || ldc % 8u == 0), "mm_ws: C not 16-byte addressable");
    const CUtensorMap *tmW = mode == MOE_MM_SWIGLU_F16 ? moe_tmap_gate_up_f16(c, W, experts_in_W, n / 2u, k)
                                                       : moe_tmap_2d_f16(c, W, (uint64_t)experts_in_W * n, k, 128, BK);
    if (tmW == NULL) return;
    XMaps tmX;
    for (uint32_t i = 0; i < 8; i += 1) {
        const CUtensorMap *m = moe_tmap_2d_f16(c, X, rows_x, k, 16u * (i + 1u), BK);
        if (m == NULL) return;
        tmX.m[i] = *m;
    }
#ifdef MOE_WS_PROF
    {
        cuuint64_t dims[2] = {256, (cuuint64_t)experts_in_W * n * k * 2 / 512};
        cuuint64_t strides[1] = {512};
        cuuint32_t box[2] = {256, 32};
        cuuint32_t estr[2] = {1, 1};
        typedef CUresult (*enc_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                   const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
        CUresult r = ((enc_fn)c->encode_tiled)(&tmX.wc, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)W, dims, strides, box, estr,
                                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        MOE_REQUIRE(c, r == CUDA_SUCCESS, "mm_ws: contiguous weight map failed: %d", (int)r);
    }
#endif
    WsArgs a;
    a.C = C;
    a.chunks = (const uint4 *)chunks;
    a.n_chunks = n_chunks;
    a.n = n;
    a.k = k;
    a.ldc = ldc;
    a.status = c->dev_status_dev;
    a.wait_ns = c->wait_ns;
    a.prof = NULL;
    a.trace = NULL;
    a.dbg = 0;
    uint32_t ft = mode == MOE_MM_SWIGLU_F16 ? (n / 2u) / (64u * (uint32_t)pair) : n / (128u * (uint32_t)pair);
    uint64_t total = (uint64_t)max_chunks * ft * (uint32_t)pair;
    uint32_t sms = (uint32_t)c->sm_count / (uint32_t)pair * (uint32_t)pair;
    uint32_t grid = total < sms ? (uint32_t)total : sms;
#define WS_CASE(M, P)                                      \
    if (mode == M && pair == P) {                          \
        ws_launch<M, P>(c, tmW, tmX, a, grid);             \
        return;                                            \
    }
    WS_CASE(MOE_MM_SWIGLU_F16, 1)
    WS_CASE(MOE_MM_SWIGLU_F16, 2)
    WS_CASE(MOE_MM_F16, 1)
    WS_CASE(MOE_MM_F16, 2)
    WS_CASE(MOE_MM_F32, 1)
    WS_CASE(MOE_MM_F32, 2)
#undef WS_CASE
}
