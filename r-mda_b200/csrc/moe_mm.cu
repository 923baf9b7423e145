// Grouped expert products on the 5th-generation tensor cores (sm_100a).
//
// C[m0:m0+128, :] = A[m0:m0+128, :k] * B[e]^T for every 128-row tile whose
// tiles[] entry e is not ~0 -- the tile schedule that the scan kernel builds
// from the per-expert offsets (shader/matmul_f16_moe.comp:70-78).
//
// One persistent CTA per SM walks the (row tile, column tile) list.  Roles:
//   warp 0     TMA producer: 128x64 fp16 boxes of A and two 128x64 boxes of B
//              per stage into a 4-stage shared-memory ring (128-byte swizzle);
//              plain per-CTA loads, never multicast.
//   warp 1     allocates tensor memory and issues tcgen05.mma (M128 N256 K16,
//              fp16 x fp16 -> fp32) into one of two 256-column accumulators.
//   warps 2-5  epilogue: tcgen05.ld the finished accumulator, apply the mode's
//              epilogue, store; overlaps the next tile's main loop.
// Modes: F32 (reference semantics: fp32 C, power-of-two slot scale), SWIGLU_F16
// (B tile = 128 gate rows + the matching 128 up rows; C = fp16 silu(gate)*up,
// i.e. shader/qwen_elem.comp op 0 + the fp16 store fused into the product) and
// F16 (fp16 C).  Every spin on an mbarrier is bounded; on timeout the kernel
// records MOE_ERR_TIMEOUT in the context's status word and unwinds.
#include "moe_tc.cuh"

namespace {

using namespace moe_tc;

#ifndef MM_BK
#define MM_BK 64
#endif
// K step per stage: 64 (128-byte rows, 128-byte swizzle, 4 stages of 48 KB).  32 (64-byte rows, 64-byte
// swizzle, 8 stages of 24 KB) also builds and passes the parity tests but is 40 % slower on B200: its
// half-line row requests stream worse, which outweighs the finer stage recycling.
constexpr uint32_t BM = 128, BN = 256, BK = MM_BK, STAGES = 256 / MM_BK;
constexpr uint32_t ROW_BYTES = BK * 2;          // bytes of one operand row per stage = the swizzle span
constexpr uint32_t A_BYTES = BM * BK * 2;
constexpr uint32_t BH_BYTES = 128 * BK * 2;     // half of the B tile
constexpr uint32_t STAGE_BYTES = A_BYTES + 2 * BH_BYTES;
constexpr uint32_t MM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(8) MmBarriers {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    uint32_t abort;
};
constexpr uint32_t MM_SMEM = STAGES * STAGE_BYTES + sizeof(MmBarriers) + 1024;

struct MmArgs {
    void *C;
    const uint32_t *amax;
    const uint32_t *tiles;
    uint32_t m, n, k, sa, sb, experts_in_B;
    uint32_t c_rows;  // rows C really holds (<= m): rows beyond are not stored (fp32 mode)
    uint32_t prefix;  // used tiles form a prefix of tiles[]: stop at the first unused one
    // row gather (fused layer): A row p is row src_row[p] of X (~0: padding row, reads as zero)
    const uint32_t *src_row;
    const __half *X;
    uint32_t ldx;
    uint32_t *status;
    uint64_t wait_ns;
};

struct WorkItem {
    uint32_t mt, nt, e, nvalid;
    int32_t rb0, rb1;
};

template <int MODE>
__device__ __forceinline__ bool mm_work(const MmArgs &a, uint32_t w, uint32_t nt_count, WorkItem &it) {
    it.mt = w / nt_count;
    it.nt = w - it.mt * nt_count;
    it.e = a.tiles[it.mt];
    if (it.e >= a.experts_in_B) return false;  // ~0: unused tile (matmul_f16_moe.comp:72-74)
    if (MODE == MOE_MM_SWIGLU_F16) {
        it.nvalid = BN;
        it.rb0 = (int32_t)(it.e * a.n + it.nt * 128u);
        it.rb1 = (int32_t)(it.e * a.n + a.n / 2u + it.nt * 128u);
    } else {
        uint32_t n0 = it.nt * BN;
        it.nvalid = a.n - n0 < BN ? a.n - n0 : BN;  // 128 or 256
        it.rb0 = (int32_t)(it.e * a.n + n0);
        it.rb1 = it.rb0 + 128;
    }
    return true;
}

// GATHER: four extra warps (6..9) fill the A tile themselves -- 16-byte async
// copies of rows of X picked by src_row[], written with the same 128-byte
// swizzle TMA would apply -- so the permuted copy of the activations never has
// to exist in HBM.  The weights still arrive by TMA from warp 0.
template <int MODE, bool GATHER>
__global__ void __launch_bounds__(MM_THREADS + (GATHER ? 128 : 0), 1)
moe_mm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, MmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    MmBarriers *bars = reinterpret_cast<MmBarriers *>(smem + STAGES * STAGE_BYTES);
    const uint32_t stage0 = smem_u32(smem);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    volatile uint32_t *abort = &bars->abort;

    const uint32_t nt_count = MODE == MOE_MM_SWIGLU_F16 ? a.n / BN : (a.n + BN - 1) / BN;
    const uint32_t total = (a.m / BM) * nt_count;
    const uint32_t kblocks = (a.k + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < STAGES; s += 1) {
            mbar_init(smem_u32(&bars->full[s]), GATHER ? 129 : 1);  // TMA thread + every gather thread
            mbar_init(smem_u32(&bars->empty[s]), 1);
        }
        for (uint32_t s = 0; s < 2; s += 1) {
            mbar_init(smem_u32(&bars->tmem_full[s]), 1);
            mbar_init(smem_u32(&bars->tmem_empty[s]), 128);
        }
        bars->abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&bars->tmem_base)),
                     "r"(TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = bars->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0;
            uint32_t issued = 0;  // bit s set once stage s has a load in flight or done
            uint32_t last_par = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < total && ok; w += gridDim.x) {
                WorkItem it;
                if (!mm_work<MODE>(a, w, nt_count, it)) {
                    if (a.prefix) break;
                    continue;
                }
                for (uint32_t kb = 0; kb < kblocks; kb += 1) {
                    if (!mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort, a.status, 1, a.wait_ns)) {
                        ok = false;
                        break;
                    }
                    uint32_t full = smem_u32(&bars->full[s]);
                    uint32_t base = stage0 + s * STAGE_BYTES;
                    mbar_expect_tx(full, (GATHER ? 0u : A_BYTES) + (it.nvalid == BN ? 2 * BH_BYTES : BH_BYTES));
                    if (!GATHER) tma_load_2d(base, &tmA, full, (int32_t)(kb * BK), (int32_t)(it.mt * BM));
                    tma_load_2d(base + A_BYTES, &tmB, full, (int32_t)(kb * BK), it.rb0);
                    if (it.nvalid == BN) tma_load_2d(base + A_BYTES + BH_BYTES, &tmB, full, (int32_t)(kb * BK), it.rb1);
                    issued |= 1u << s;
                    last_par = (last_par & ~(1u << s)) | (ph << s);
                    s += 1;
                    if (s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
            }
            if (!ok) {
                // unwinding: give copies already issued a bounded time to land
                for (uint32_t q = 0; q < STAGES; q += 1) {
                    if (((issued >> q) & 1u) == 0) continue;
                    for (uint32_t spin = 0; spin < (1u << 16); spin += 1) {
                        if (mbar_try_wait(smem_u32(&bars->full[q]), (last_par >> q) & 1u)) break;
                    }
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t s = 0, ph = 0, n_item = 0;
            bool ok = true;
            for (uint32_t w = blockIdx.x; w < total && ok; w += gridDim.x) {
                WorkItem it;
                if (!mm_work<MODE>(a, w, nt_count, it)) {
                    if (a.prefix) break;
                    continue;
                }
                uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
                if (!mbar_wait(smem_u32(&bars->tmem_empty[as]), aph ^ 1u, abort, a.status, 2, a.wait_ns)) break;
                tc_fence_after();
                uint32_t tmem_d = tmem_base + as * BN;
                uint32_t idesc = umma_idesc(BM, it.nvalid);
                for (uint32_t kb = 0; kb < kblocks; kb += 1) {
                    if (!mbar_wait(smem_u32(&bars->full[s]), ph, abort, a.status, 3, a.wait_ns)) {
                        ok = false;
                        break;
                    }
                    // gathered rows were written through the generic proxy; the tensor core reads through the async one
                    if (GATHER) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    tc_fence_after();
                    uint32_t base = stage0 + s * STAGE_BYTES;
                    uint64_t ad = BK == 64 ? umma_desc(base) : umma_desc_sw64(base);
                    uint64_t bd = BK == 64 ? umma_desc(base + A_BYTES) : umma_desc_sw64(base + A_BYTES);
#pragma unroll
                    for (uint32_t kk = 0; kk < BK / 16; kk += 1) {
                        // +32 bytes per K=16 step inside the 128-byte swizzle row
                        umma_f16(tmem_d, ad + 2ull * kk, bd + 2ull * kk, idesc, (kb | kk) != 0 ? 1u : 0u);
                    }
                    umma_commit(smem_u32(&bars->empty[s]));  // frees the stage when these MMAs retire
                    s += 1;
                    if (s == STAGES) {
                        s = 0;
                        ph ^= 1u;
                    }
                }
                if (ok) umma_commit(smem_u32(&bars->tmem_full[as]));
                n_item += 1;
            }
        }
        __syncwarp();
    } else if (GATHER && warp >= 6) {
        // ---------------- row gather (warps 6..9) ----------------
        // CPR = 16-byte chunks per operand row and stage.  Thread g of the 128 handles chunk g % CPR of rows
        // g / CPR + RPI * j: consecutive lanes fetch consecutive chunks of a row, so requests are whole
        // 64- or 128-byte pieces of a line.
        constexpr uint32_t CPR = ROW_BYTES / 16u, RPI = 128u / CPR, NJ = BM / RPI;
        const uint32_t g = (warp - 6u) * 32u + lane;
        const uint32_t sub = g / CPR, ch = g % CPR;
        // swizzle as TMA writes it: 128-byte rows: chunk ^ (row % 8); 64-byte rows: chunk ^ ((row / 2) % 4)
        const uint32_t dst_off = sub * ROW_BYTES + ((ch ^ (BK == 64 ? (sub & 7u) : ((sub >> 1) & 3u))) << 4);
        uint32_t s = 0, ph = 0;
        bool ok = true;
        for (uint32_t w = blockIdx.x; w < total && ok; w += gridDim.x) {
            WorkItem it;
            if (!mm_work<MODE>(a, w, nt_count, it)) {
                if (a.prefix) break;
                continue;
            }
            const __half *rowp[NJ];
            uint32_t live = 0;
#pragma unroll
            for (uint32_t j = 0; j < NJ; j += 1) {
                const uint32_t src = a.src_row[it.mt * BM + j * RPI + sub];
                rowp[j] = a.X + (size_t)(src == ~0u ? 0u : src) * a.ldx + ch * 8u;
                live |= (src != ~0u ? 1u : 0u) << j;
            }
            for (uint32_t kb = 0; kb < kblocks; kb += 1) {
                uint32_t got = 1;
                if (lane == 0) got = mbar_wait(smem_u32(&bars->empty[s]), ph ^ 1u, abort, a.status, 5, a.wait_ns) ? 1u : 0u;
                got = __shfl_sync(0xffffffffu, got, 0);
                if (!got) {
                    ok = false;
                    break;
                }
                const uint32_t dst = stage0 + s * STAGE_BYTES + dst_off;
                const uint32_t col = kb * BK + ch * 8u;
#pragma unroll
                for (uint32_t j = 0; j < NJ; j += 1) {
                    const uint32_t nbytes = (((live >> j) & 1u) != 0u && col < a.k) ? 16u : 0u;  // 0: zero-filled
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst + j * RPI * ROW_BYTES),
                                 "l"(rowp[j] + (nbytes != 0u ? kb * BK : 0u)), "r"(nbytes)
                                 : "memory");
                }
                // the hardware arrives on the stage's barrier once this thread's copies have landed
                asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&bars->full[s])) : "memory");
                s += 1;
                if (s == STAGES) {
                    s = 0;
                    ph ^= 1u;
                }
            }
        }
        asm volatile("cp.async.wait_all;" ::: "memory");  // nothing of this thread is in flight when it leaves
    } else {
        // ---------------- epilogue (warps 2..5) ----------------
        const uint32_t q = warp & 3u;  // TMEM lane quarter this warp may read
        float scale = 1.0f;
        if (MODE == MOE_MM_F32) scale = 1.0f / (moe_slot_scale(a.amax, a.sa) * moe_slot_scale(a.amax, a.sb));
        uint32_t n_item = 0;
        for (uint32_t w = blockIdx.x; w < total; w += gridDim.x) {
            WorkItem it;
            if (!mm_work<MODE>(a, w, nt_count, it)) {
                if (a.prefix) break;
                continue;
            }
            uint32_t as = n_item & 1u, aph = (n_item >> 1) & 1u;
            if (!mbar_wait(smem_u32(&bars->tmem_full[as]), aph, abort, a.status, 4, a.wait_ns)) break;
            tc_fence_after();
            uint32_t taddr = tmem_base + as * BN + ((q * 32u) << 16);
            size_t row = (size_t)it.mt * BM + q * 32u + lane;
            if (MODE == MOE_MM_SWIGLU_F16) {
                __half *out = reinterpret_cast<__half *>(a.C) + row * (a.n / 2u) + it.nt * 128u;
#pragma unroll 1
                for (uint32_t cch = 0; cch < 4; cch += 1) {
                    uint32_t g[32], u[32];
                    tmem_ld32(taddr + cch * 32u, g);
                    tmem_ld32(taddr + 128u + cch * 32u, u);
                    tmem_ld_wait();
                    uint32_t o[16];
#pragma unroll
                    for (uint32_t j = 0; j < 16; j += 1) {
                        float g0 = __uint_as_float(g[2 * j]), g1 = __uint_as_float(g[2 * j + 1]);
                        float h0 = __fdividef(g0, 1.0f + __expf(-g0)) * __uint_as_float(u[2 * j]);
                        float h1 = __fdividef(g1, 1.0f + __expf(-g1)) * __uint_as_float(u[2 * j + 1]);
                        o[j] = pack_h2(h0, h1);
                    }
                    uint4 *dst = reinterpret_cast<uint4 *>(out + cch * 32u);
#pragma unroll
                    for (uint32_t j = 0; j < 4; j += 1) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                }
            } else if (MODE == MOE_MM_F16) {
                __half *out = reinterpret_cast<__half *>(a.C) + row * a.n + it.nt * BN;
#pragma unroll 1
                for (uint32_t cch = 0; cch < it.nvalid / 32u; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * 32u, v);
                    tmem_ld_wait();
                    uint4 *dst = reinterpret_cast<uint4 *>(out + cch * 32u);
#pragma unroll
                    for (uint32_t j = 0; j < 4; j += 1) {
                        dst[j] = make_uint4(pack_h2(__uint_as_float(v[8 * j]), __uint_as_float(v[8 * j + 1])),
                                            pack_h2(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3])),
                                            pack_h2(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5])),
                                            pack_h2(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7])));
                    }
                }
            } else {
                float *out = reinterpret_cast<float *>(a.C) + row * a.n + it.nt * BN;
#pragma unroll 1
                for (uint32_t cch = 0; cch < it.nvalid / 32u; cch += 1) {
                    uint32_t v[32];
                    tmem_ld32(taddr + cch * 32u, v);
                    tmem_ld_wait();
                    float4 *dst = reinterpret_cast<float4 *>(out + cch * 32u);
                    if (row >= a.c_rows) continue;
#pragma unroll
                    for (uint32_t j = 0; j < 8; j += 1) {
                        dst[j] = make_float4(__uint_as_float(v[4 * j]) * scale, __uint_as_float(v[4 * j + 1]) * scale,
                                             __uint_as_float(v[4 * j + 2]) * scale, __uint_as_float(v[4 * j + 3]) * scale);
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(smem_u32(&bars->tmem_empty[as]));
            n_item += 1;
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

template <int MODE, bool GATHER>
void mm_launch(moe_cuda_ctx *c, const CUtensorMap *tmA, const CUtensorMap *tmB, const MmArgs &a, uint32_t grid) {
    const int slot = GATHER ? 3 : MODE;
    if (!c->mm_attr_set[slot]) {
        MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_mm_kernel<MODE, GATHER>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)MM_SMEM));
        c->mm_attr_set[slot] = true;
    }
    moe_mm_kernel<MODE, GATHER><<<grid, MM_THREADS + (GATHER ? 128 : 0), MM_SMEM, c->stream>>>(*tmA, *tmB, a);
    MOE_LAUNCHED(c);
}

}  // namespace

void moe_launch_mm(moe_cuda_ctx *c, int mode, const void *A, const void *B, void *C, const uint32_t *amax,
                   const uint32_t *tiles, uint32_t m, uint32_t n, uint32_t k, uint32_t sa, uint32_t sb,
                   uint32_t experts_in_B, uint32_t a_rows, bool prefix, const uint32_t *src_row, uint32_t c_rows) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, A != NULL && B != NULL && C != NULL && tiles != NULL, "mm: null buffer");
    MOE_REQUIRE(c, a_rows >= 1 && a_rows <= m, "mm: a_rows %u outside 1..m", a_rows);
    MOE_REQUIRE(c, m % BM == 0, "mm: m %u not a multiple of 128", m);
    MOE_REQUIRE(c, n % 128u == 0 && n >= 128u, "mm: n %u not a multiple of 128", n);
    MOE_REQUIRE(c, mode != MOE_MM_SWIGLU_F16 || n % 256u == 0, "mm: fused SwiGLU needs inter %% 128 == 0 (n = %u)", n);
    MOE_REQUIRE(c, k % 8u == 0 && k >= 8u, "mm: k %u not a multiple of 8", k);
    MOE_REQUIRE(c, experts_in_B >= 1 && (uint64_t)experts_in_B * n < (1ull << 31), "mm: expert count");
    MOE_REQUIRE(c, src_row == NULL || (mode == MOE_MM_SWIGLU_F16 && ((uintptr_t)A & 15) == 0), "mm: row gather is for the gate_up product");
    MOE_REQUIRE(c, (sa == MDA_PC_NO_SLOT && sb == MDA_PC_NO_SLOT) || amax != NULL, "mm: scale slot without amax");
    MOE_REQUIRE(c, ((uintptr_t)C & 15) == 0, "mm: C not 16-byte aligned");
    const CUtensorMap *tmA = moe_tmap_2d_f16(c, A, a_rows, k, 128, BK);
    const CUtensorMap *tmB = moe_tmap_2d_f16(c, B, (uint64_t)experts_in_B * n, k, 128, BK);
    if (tmA == NULL || tmB == NULL) return;
    MmArgs a;
    a.C = C;
    a.amax = amax;
    a.tiles = tiles;
    a.m = m;
    a.n = n;
    a.k = k;
    a.sa = sa;
    a.sb = sb;
    a.experts_in_B = experts_in_B;
    a.c_rows = c_rows == 0 ? m : c_rows;
    MOE_REQUIRE(c, a.c_rows == m || mode == MOE_MM_F32, "mm: a short C is only supported for fp32 output");
    a.prefix = prefix ? 1u : 0u;
    a.src_row = src_row;
    a.X = (const __half *)A;
    a.ldx = k;
    a.status = c->dev_status_dev;
    a.wait_ns = c->wait_ns;
    uint32_t nt = mode == MOE_MM_SWIGLU_F16 ? n / BN : (n + BN - 1) / BN;
    uint64_t total = (uint64_t)(m / BM) * nt;
    uint32_t grid = total < (uint64_t)c->sm_count ? (uint32_t)total : (uint32_t)c->sm_count;
    if (mode == MOE_MM_F32) mm_launch<MOE_MM_F32, false>(c, tmA, tmB, a, grid);
    else if (mode == MOE_MM_SWIGLU_F16 && src_row != NULL) mm_launch<MOE_MM_SWIGLU_F16, true>(c, tmA, tmB, a, grid);
    else if (mode == MOE_MM_SWIGLU_F16) mm_launch<MOE_MM_SWIGLU_F16, false>(c, tmA, tmB, a, grid);
    else mm_launch<MOE_MM_F16, false>(c, tmA, tmB, a, grid);
}

extern "C" void moe_cuda_mm(moe_cuda_ctx_t *c, const void *A, const void *B, float *C, const uint32_t *amax,
                            const uint32_t *tiles, struct mda_pc_moe_mm_t pc, uint32_t experts_in_B) {
    moe_launch_mm(c, MOE_MM_F32, A, B, C, amax, tiles, pc.m, pc.n, pc.k, pc.sa, pc.sb, experts_in_B, pc.m);
}
