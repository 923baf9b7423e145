// Grouped expert products, weight-stationary form ("swap-AB"), for the fused
// layer: the MMA's M dimension runs over weight rows (output features), its N
// dimension over the tokens of one expert.  Compared with the token-major kernel
// in moe_mm.cu (the reference's 128-row tile schedule, shader/matmul_f16_moe.comp):
//   * an expert's rows are cut into chunks of at most 256 tokens whose MMA width
//     is rounded to 16, not 128, so ragged expert sizes waste almost no tensor
//     work (the reference pads every expert to 128 rows);
//   * with PAIR = 2 two CTAs of a cluster issue one tcgen05.mma.cta_group::2
//     (M 256) over a shared token tile: each CTA loads its own 128 weight rows
//     and only half of the token tile, which cuts the shared-memory fill traffic
//     per flop by a third.  The loads are plain per-CTA TMA tile loads.
// D lands transposed in tensor memory (lane = feature, column = token); the
// epilogue warps write it back token-major.  SWIGLU mode gives each CTA 64 gate
// rows + the matching 64 up rows, so lanes i and i+64 pair up: the "up" warps
// hand their values to the "gate" warps through shared memory, which apply
// silu(gate)*up (shader/qwen_elem.comp:20-31 op 0) and store fp16.
#include "moe_tc.cuh"

namespace {

using namespace moe_tc;

constexpr uint32_t BK = 64;
constexpr uint32_t A_BYTES = 128 * BK * 2;   // 16 KB: this CTA's 128 weight rows
constexpr uint32_t BOX_BYTES = 64 * BK * 2;  // 8 KB: one 64-row TMA box
constexpr uint32_t MAX_TOK = 256;            // tokens per chunk = MMA N
constexpr uint32_t SW_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t EX_STRIDE = 33;           // floats per feature row of the exchange buffer

template <int PAIR>
struct Geo {
    static constexpr uint32_t B_BYTES = MAX_TOK / PAIR * BK * 2;  // this CTA's share of the token tile
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t STAGES = PAIR == 2 ? 6 : 4;         // 192 KB of operands either way
};

struct __align__(8) SwBarriers {
    uint64_t full[8];
    uint64_t empty[8];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};

template <int PAIR>
constexpr uint32_t sw_smem() {
    return Geo<PAIR>::STAGES * Geo<PAIR>::STAGE_BYTES + 2 * 64 * EX_STRIDE * 4 + sizeof(SwBarriers) + 1024;
}

struct SwArgs {
    void *C;
    const uint4 *chunks;       // (expert, first row, MMA width, valid rows)
    const uint32_t *n_chunks;
    uint32_t n;                // weight rows per expert (2*inter, or d)
    uint32_t k;
    uint32_t ldc;              // row stride of C in elements
    uint32_t *status;
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
// TMA tile load issued by either CTA of a pair; the completion bytes are counted
// on the barrier at cluster address `bar` (the leader's).  Not a multicast.
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
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
__device__ __forceinline__ void umma_commit_pair(uint32_t cluster_bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(cluster_bar) : "memory");
}

struct SwItem {
    uint32_t e, row0, ntok, nvalid, ft;
};

template <int MODE, int PAIR>
__device__ __forceinline__ void sw_item(const SwArgs &a, uint32_t w, uint32_t ft_count, SwItem &it) {
    uint32_t c = w / ft_count;
    it.ft = w - c * ft_count;
    uint4 ch = a.chunks[c];
    it.e = ch.x;
    it.row0 = ch.y;
    it.ntok = ch.z;
    it.nvalid = ch.w;
}

template <int MODE, int PAIR>
__global__ void __launch_bounds__(SW_THREADS, 1)
moe_mm_swap_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, SwArgs a) {
    using G = Geo<PAIR>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float *ex = reinterpret_cast<float *>(smem + G::STAGES * G::STAGE_BYTES);
    SwBarriers *bars = reinterpret_cast<SwBarriers *>(smem + G::STAGES * G::STAGE_BYTES + 2 * 64 * EX_STRIDE * 4);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t rank = PAIR == 2 ? cluster_rank() : 0u;
    volatile uint32_t *abort = &bars->abort;

    const uint32_t ft_count = MODE == MOE_MM_SWIGLU_F16 ? (a.n / 2u) / (64u * PAIR) : a.n / (128u * PAIR);
    const uint32_t total = *a.n_chunks * ft_count;
    const uint32_t kblocks = (a.k + BK - 1) / BK;
    const uint32_t cluster_id = blockIdx.x / PAIR, n_clusters = gridDim.x / PAIR;

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

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, issued = 0, last_par = 0;
            bool ok = true;
            for (uint32_t w = cluster_id; w < total && ok; w += n_clusters) {
                SwItem it;
                sw_item<MODE, PAIR>(a, w, ft_count, it);
                const uint32_t half = it.ntok / PAIR;            // token rows this CTA loads
                const uint32_t nbox = (half + 63u) / 64u;
                int32_t wrow0, wrow1;
                if (MODE == MOE_MM_SWIGLU_F16) {
                    uint32_t f0 = (it.ft * PAIR + rank) * 64u;
                    wrow0 = (int32_t)(it.e * a.n + f0);                // 64 gate rows
                    wrow1 = (int32_t)(it.e * a.n + a.n / 2u + f0);     // the matching 64 up rows
                } else {
                    wrow0 = (int32_t)(it.e * a.n + (it.ft * PAIR + rank) * 128u);
                    wrow1 = wrow0 + 64;
                }
                const int32_t xrow = (int32_t)(it.row0 + rank * half);
                for (uint32_t kb = 0; kb < kblocks; kb += 1) {
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort, a.status, 11)) {
                        ok = false;
                        break;
                    }
                    const uint32_t base = stage0 + s * G::STAGE_BYTES;
                    const int32_t kc = (int32_t)(kb * BK);
                    if (PAIR == 2) {
                        const uint32_t full = map_to_cta(smem_u32(&bars->full[s]), 0);  // the leader's barrier
                        if (rank == 0) mbar_expect_tx(smem_u32(&bars->full[s]), 2u * (A_BYTES + nbox * BOX_BYTES));
                        tma_load_2d_pair(base, &tmW, full, kc, wrow0);
                        tma_load_2d_pair(base + BOX_BYTES, &tmW, full, kc, wrow1);
                        for (uint32_t b = 0; b < nbox; b += 1) {
                            tma_load_2d_pair(base + A_BYTES + b * BOX_BYTES, &tmX, full, kc, xrow + (int32_t)(b * 64u));
                        }
                    } else {
                        const uint32_t full = smem_u32(&bars->full[s]);
                        mbar_expect_tx(full, A_BYTES + nbox * BOX_BYTES);
                        tma_load_2d(base, &tmW, full, kc, wrow0);
                        tma_load_2d(base + BOX_BYTES, &tmW, full, kc, wrow1);
                        for (uint32_t b = 0; b < nbox; b += 1) {
                            tma_load_2d(base + A_BYTES + b * BOX_BYTES, &tmX, full, kc, xrow + (int32_t)(b * 64u));
                        }
                    }
                    issued |= 1u << s;
                    last_par = (last_par & ~(1u << s)) | (ph << s);
                    s += 1;
                    if (s == G::STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (!ok && rank == 0) {
                for (uint32_t q = 0; q < G::STAGES; q += 1) {  // bounded wait for copies in flight
                    if (((issued >> q) & 1u) == 0) continue;
                    for (uint32_t spin = 0; spin < (1u << 16); spin += 1) {
                        if (mbar_try_wait(smem_u32(&bars->full[q]), (last_par >> q) & 1u)) break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (lane == 0 && rank == 0) {
            uint32_t s = 0, ph = 0, n_item = 0;
            bool ok = true;
            for (uint32_t w = cluster_id; w < total && ok; w += n_clusters) {
                SwItem it;
                sw_item<MODE, PAIR>(a, w, ft_count, it);
                const uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars->tmem_empty[as]), aph ^ 1u, abort, a.status, 12)) break;
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + as * MAX_TOK;
                const uint32_t idesc = umma_idesc(128u * PAIR, it.ntok);
                for (uint32_t kb = 0; kb < kblocks; kb += 1) {
                    if (!mbar_wait(smem_u32(&bars->full[s]), ph, abort, a.status, 13)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t base = stage0 + s * G::STAGE_BYTES;
                    const uint64_t ad = umma_desc(base), bd = umma_desc(base + A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / 16; kk += 1) {
                        if (PAIR == 2) umma_f16_pair(tmem_d, ad + 2ull * kk, bd + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                        else umma_f16(tmem_d, ad + 2ull * kk, bd + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                    }
                    if (PAIR == 2) {  // free the stage in both CTAs
                        umma_commit_pair(map_to_cta(smem_u32(&bars->empty[s]), 0));
                        umma_commit_pair(map_to_cta(smem_u32(&bars->empty[s]), 1));
                    } else {
                        umma_commit(smem_u32(&bars->empty[s]));
                    }
                    s += 1;
                    if (s == G::STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) {
                    if (PAIR == 2) {
                        umma_commit_pair(map_to_cta(smem_u32(&bars->tmem_full[as]), 0));
                        umma_commit_pair(map_to_cta(smem_u32(&bars->tmem_full[as]), 1));
                    } else {
                        umma_commit(smem_u32(&bars->tmem_full[as]));
                    }
                }
                n_item += 1;
            }
        }
        __syncwarp();
    } else {
        // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
        const uint32_t q = warp & 3u;  // TMEM lane quarter
        const uint32_t empty_leader = PAIR == 2 ? map_to_cta(smem_u32(&bars->tmem_empty[0]), 0) : smem_u32(&bars->tmem_empty[0]);
        uint32_t n_item = 0;
        uint32_t exbuf = 0;
        bool ok = true;
        for (uint32_t w = cluster_id; w < total && ok; w += n_clusters) {
            SwItem it;
            sw_item<MODE, PAIR>(a, w, ft_count, it);
            const uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
            if (!mbar_wait(smem_u32(&bars->tmem_full[as]), aph, abort, a.status, 14)) {
                ok = false;
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + as * MAX_TOK + ((q * 32u) << 16);
            const uint32_t nch = (it.ntok + 31u) / 32u;
            if (MODE == MOE_MM_SWIGLU_F16) {
                // lanes 0..63 hold gate features, lanes 64..127 the matching up features
                const uint32_t f = (it.ft * PAIR + rank) * 64u + (q & 1u) * 32u + lane;
                __half *out = reinterpret_cast<__half *>(a.C) + (size_t)it.row0 * a.ldc + f;
                for (uint32_t cch = 0; cch < nch; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * 32u, v);
                    tmem_ld_wait();
                    float *exb = ex + exbuf * 64u * EX_STRIDE + ((q & 1u) * 32u + lane) * EX_STRIDE;
                    if (q >= 2) {
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 1) exb[j] = __uint_as_float(v[j]);
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");  // up values visible to the gate warps
                    if (q < 2) {
                        const uint32_t t0 = cch * 32u;
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 1) {
                            float g = __uint_as_float(v[j]);
                            float h = __fdividef(g, 1.0f + __expf(-g)) * exb[j];
                            if (t0 + j < it.nvalid) out[(size_t)(t0 + j) * a.ldc] = __float2half_rn(h);
                        }
                    }
                    exbuf ^= 1u;
                }
            } else {
                const uint32_t cfeat = (it.ft * PAIR + rank) * 128u + q * 32u + lane;
                for (uint32_t cch = 0; cch < nch; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * 32u, v);
                    tmem_ld_wait();
                    const uint32_t t0 = cch * 32u;
                    if (MODE == MOE_MM_F16) {
                        __half *out = reinterpret_cast<__half *>(a.C) + (size_t)(it.row0 + t0) * a.ldc + cfeat;
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 1) {
                            if (t0 + j < it.nvalid) out[(size_t)j * a.ldc] = __float2half_rn(__uint_as_float(v[j]));
                        }
                    } else {
                        float *out = reinterpret_cast<float *>(a.C) + (size_t)(it.row0 + t0) * a.ldc + cfeat;
#pragma unroll
                        for (uint32_t j = 0; j < 32; j += 1) {
                            if (t0 + j < it.nvalid) out[(size_t)j * a.ldc] = __uint_as_float(v[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (PAIR == 2) mbar_arrive_cluster(empty_leader + as * 8u);
                else mbar_arrive(empty_leader + as * 8u);
            }
            n_item += 1;
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
}

// Cuts every expert's rows into chunks of at most 256 tokens of near-equal size,
// MMA width rounded up to 16.  One block; thread = expert.
__global__ void __launch_bounds__(512)
moe_chunk_kernel(const uint32_t *__restrict__ count, const uint32_t *__restrict__ off, uint32_t experts,
                 uint4 *__restrict__ chunks, uint32_t *__restrict__ n_chunks, uint32_t max_chunks) {
    __shared__ uint32_t s[512];
    uint32_t e = threadIdx.x;
    uint32_t cnt = e < experts ? count[e] : 0;
    uint32_t nch = (cnt + MAX_TOK - 1) / MAX_TOK;
    s[e] = nch;
    __syncthreads();
    for (uint32_t o = 1; o < 512; o <<= 1) {
        uint32_t v = e >= o ? s[e - o] : 0;
        __syncthreads();
        s[e] += v;
        __syncthreads();
    }
    uint32_t first = s[e] - nch;
    if (nch != 0) {
        uint32_t per = ((cnt + nch - 1) / nch + 15u) & ~15u;
        for (uint32_t j = 0; j < nch; j += 1) {
            uint32_t start = j * per;
            uint32_t valid = start < cnt ? min(per, cnt - start) : 0;
            if (first + j < max_chunks) chunks[first + j] = make_uint4(e, off[e] + start, (valid + 15u) & ~15u, valid);
        }
    }
    if (e == 511) *n_chunks = min(s[511], max_chunks);
}

template <int MODE, int PAIR>
void sw_launch(moe_cuda_ctx *c, const CUtensorMap *tmW, const CUtensorMap *tmX, const SwArgs &a, uint32_t grid) {
    int slot = MODE * 2 + (PAIR - 1);
    if (!c->sw_attr_set[slot]) {
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_mm_swap_kernel<MODE, PAIR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)sw_smem<PAIR>()));
        c->sw_attr_set[slot] = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(grid, 1, 1);
    cfg.blockDim = dim3(SW_THREADS, 1, 1);
    cfg.dynamicSmemBytes = sw_smem<PAIR>();
    cfg.stream = c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = PAIR;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    MOE_CUDA_TRY(c, cudaLaunchKernelEx(&cfg, moe_mm_swap_kernel<MODE, PAIR>, *tmW, *tmX, a));
    c->launches += 1;
}

}  // namespace

void moe_launch_chunks(moe_cuda_ctx *c, const uint32_t *count, const uint32_t *off, uint32_t experts, void *chunks,
                       uint32_t *n_chunks, uint32_t max_chunks) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, experts >= 1 && experts <= MOE_MAX_EXPERTS, "chunks: experts %u outside 1..512", experts);
    moe_chunk_kernel<<<1, 512, 0, c->stream>>>(count, off, experts, (uint4 *)chunks, n_chunks, max_chunks);
    MOE_LAUNCHED(c);
}

// A [rows_x x k] fp16 token rows, W [experts_in_W][n x k] fp16, C token-major with row stride ldc.
void moe_launch_mm_swap(moe_cuda_ctx *c, int mode, int pair, const void *X, uint32_t rows_x, const void *W,
                        uint32_t experts_in_W, void *C, uint32_t ldc, const void *chunks, const uint32_t *n_chunks,
                        uint32_t max_chunks, uint32_t n, uint32_t k) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, X != NULL && W != NULL && C != NULL && chunks != NULL && n_chunks != NULL, "mm_swap: null buffer");
    MOE_REQUIRE(c, pair == 1 || pair == 2, "mm_swap: pair %d", pair);
    MOE_REQUIRE(c, n % (128u * (uint32_t)pair) == 0, "mm_swap: n %u does not tile into %d x 128 weight rows", n, pair);
    MOE_REQUIRE(c, k % 8u == 0 && k >= 8u && rows_x >= 1, "mm_swap: k %u", k);
    MOE_REQUIRE(c, (uint64_t)experts_in_W * n < (1ull << 31), "mm_swap: expert count");
    const CUtensorMap *tmW = moe_tmap_2d_f16(c, W, (uint64_t)experts_in_W * n, k, 64, BK);
    const CUtensorMap *tmX = moe_tmap_2d_f16(c, X, rows_x, k, 64, BK);
    if (tmW == NULL || tmX == NULL) return;
    SwArgs a;
    a.C = C;
    a.chunks = (const uint4 *)chunks;
    a.n_chunks = n_chunks;
    a.n = n;
    a.k = k;
    a.ldc = ldc;
    a.status = c->dev_status_dev;
    uint32_t ft = mode == MOE_MM_SWIGLU_F16 ? (n / 2u) / (64u * (uint32_t)pair) : n / (128u * (uint32_t)pair);
    uint64_t total = (uint64_t)max_chunks * ft * (uint32_t)pair;
    uint32_t sms = (uint32_t)c->sm_count / (uint32_t)pair * (uint32_t)pair;
    uint32_t grid = total < sms ? (uint32_t)total : sms;
#define SW_CASE(M, P)                                      \
    if (mode == M && pair == P) {                          \
        sw_launch<M, P>(c, tmW, tmX, a, grid);             \
        return;                                            \
    }
    SW_CASE(MOE_MM_SWIGLU_F16, 1)
    SW_CASE(MOE_MM_SWIGLU_F16, 2)
    SW_CASE(MOE_MM_F16, 1)
    SW_CASE(MOE_MM_F16, 2)
    SW_CASE(MOE_MM_F32, 1)
    SW_CASE(MOE_MM_F32, 2)
#undef SW_CASE
}
