// The teacher's distillation sink (shader/kd_bytes.comp; call mda_teach_sink,
// src/teach.c:108-128): next-token logits over a byte-level vocabulary become
// per-byte distributions along the true continuation.  For depth l < nd, among
// the tokens longer than l bytes that agree with the continuation on its first
// l bytes: the probability that byte l is the true one (entry 0) and the seven
// most probable other bytes (entries 1..7), each packed as byte | fp16(p) << 16.
//
// HBM bound by design: a persistent block of 1024 threads per SM takes rows in
// turn, so that at most one row per SM (148 x 600 KB at a 152 k vocabulary, less
// than L2) is between its two passes -- 16-byte loads for the maximum from DRAM,
// then the exponentials out of L2.  Nearly every token differs from the true
// continuation in its first byte and then only adds its mass to that byte's bin
// at depth 0; a table of (first byte, has a byte string) per token, 2 bytes
// instead of the vocabulary table's 20, built once per call, serves those, and
// only tokens that share the first byte read their full record.  Masses are
// accumulated with shared-memory float atomics, like the shader's (:122-125);
// depth 0 has one private copy per two warps to keep the atomics apart.  The
// per-depth totals and the top-7 selection run warp-parallel (one depth per warp,
// shuffles only) instead of the shader's 112 block-wide reductions per row.
#include "moe_common.cuh"

#define KD_D 16u        // MDA_KD_DEPTH, src/kd.h:11
#define KD_K 8u         // MDA_KD_K, src/kd.h:12
#define KD_THREADS 1024u
#define KD_WARPS (KD_THREADS / 32u)
#define KD_COPIES 16u   // private copies of the depth-0 bins (a power of two)

__device__ __forceinline__ uint32_t kd_byte_at(const uint32_t (&w)[4], uint32_t i) {  // :26-28
    return (w[i >> 2] >> ((i & 3u) * 8u)) & 0xffu;
}

// :30-39: index of the first of the 16 bytes in which a and b differ, or 16
__device__ __forceinline__ uint32_t kd_common_prefix(const uint32_t (&a)[4], const uint32_t (&b)[4]) {
    uint32_t n = 16u;
#pragma unroll
    for (int i = 3; i >= 0; i -= 1) {
        const uint32_t x = a[i] ^ b[i];
        if (x != 0u) n = (uint32_t)i * 4u + ((uint32_t)__ffs((int)x) - 1u) / 8u;
    }
    return n;
}

__device__ __forceinline__ uint32_t kd_pack_entry(uint32_t b, float p) {  // :70-72
    return b | ((uint32_t)__half_as_ushort(__float2half_rn(p)) << 16);
}

// first[t] = first byte | 0x100 if the token has a byte string
__global__ void moe_kd_first_kernel(const uint32_t *__restrict__ toks, uint16_t *__restrict__ first, uint32_t vocab) {
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t < vocab) first[t] = (uint16_t)((toks[(size_t)t * 5u] & 0xffu) | (toks[(size_t)t * 5u + 4u] != 0u ? 0x100u : 0u));
}

__global__ void __launch_bounds__(KD_THREADS, 1)
moe_kd_bytes_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ toks, const uint16_t *__restrict__ first,
                    const uint32_t *__restrict__ cont, uint32_t *__restrict__ outp, uint32_t vocab, uint32_t rows) {
    __shared__ float A[KD_D + 1u];
    __shared__ float H[KD_D][256];
    __shared__ float H0[KD_COPIES][256];
    __shared__ float s_max[KD_WARPS];
    const uint32_t lid = threadIdx.x, lane = lid & 31u, warp = lid >> 5;
    const bool vec = (vocab & 3u) == 0u && ((uintptr_t)logits & 15u) == 0u;
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
    uint32_t cw[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; i += 1) cw[i] = cont[(size_t)r * 5u + i];
    const uint32_t nd = min(cont[(size_t)r * 5u + 4u], KD_D);  // :100
    const uint32_t c0 = cw[0] & 0xffu;
    uint32_t *o = outp + (size_t)r * KD_D * KD_K;
    for (uint32_t i = nd * KD_K + lid; i < KD_D * KD_K; i += KD_THREADS) o[i] = 0u;  // :101-103
    if (lid <= KD_D) A[lid] = 0.0f;
    for (uint32_t i = lid; i < KD_D * 256u; i += KD_THREADS) (&H[0][0])[i] = 0.0f;
    for (uint32_t i = lid; i < KD_COPIES * 256u; i += KD_THREADS) (&H0[0][0])[i] = 0.0f;

    const float *lg = logits + (size_t)r * vocab;
    float m = -3.0e38f;  // :110-114
    if (vec) {
        const float4 *lg4 = reinterpret_cast<const float4 *>(lg);
        for (uint32_t q = lid; q < vocab / 4u; q += KD_THREADS) {
            const float4 v = lg4[q];
            m = fmaxf(fmaxf(m, fmaxf(v.x, v.y)), fmaxf(v.z, v.w));
        }
    } else {
        for (uint32_t t = lid; t < vocab; t += KD_THREADS) m = fmaxf(m, lg[t]);
    }
#pragma unroll
    for (uint32_t s = 16; s > 0; s >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, s));
    if (lane == 0) s_max[warp] = m;
    __syncthreads();  // also: the zeroed tables are visible
    m = s_max[0];
#pragma unroll 1
    for (uint32_t w = 1; w < KD_WARPS; w += 1) m = fmaxf(m, s_max[w]);

    // :115-127 for one token: x its logit, f its entry of first[]
    auto token = [&](uint32_t t, float x, uint32_t f) {
        if ((f & 0x100u) == 0u || nd == 0u) return;  // no byte string (len == 0), or no depth asked for
        const float e = expf(x - m);
        const uint32_t fb = f & 0xffu;
        if (fb != c0) {  // differs in the first byte: depth 0, bin = that byte, and nothing else (a = 0)
            atomicAdd(&H0[warp & (KD_COPIES - 1u)][fb], e);
            return;
        }
        const uint32_t *tp = toks + (size_t)t * 5u;
        const uint32_t len = tp[4];
        uint32_t tw[4];
#pragma unroll
        for (uint32_t i = 0; i < 4; i += 1) tw[i] = tp[i];
        const uint32_t lcp = kd_common_prefix(tw, cw);
        const uint32_t a = min(lcp, min(len, nd));
        if (a != 0u) atomicAdd(&A[a], e);  // A[0] is never read (:131-133)
        if (lcp < nd && lcp < len) {
            const uint32_t b = kd_byte_at(tw, lcp);
            if (lcp == 0u) atomicAdd(&H0[warp & (KD_COPIES - 1u)][b], e);
            else atomicAdd(&H[lcp][b], e);
        }
    };
    if (vec) {
        const float4 *lg4 = reinterpret_cast<const float4 *>(lg);
        const uint2 *f4 = reinterpret_cast<const uint2 *>(first);
        for (uint32_t q = lid; q < vocab / 4u; q += KD_THREADS) {
            const float4 v = lg4[q];
            const uint2 f = f4[q];
            token(q * 4u, v.x, f.x & 0xffffu);
            token(q * 4u + 1u, v.y, f.x >> 16);
            token(q * 4u + 2u, v.z, f.y & 0xffffu);
            token(q * 4u + 3u, v.w, f.y >> 16);
        }
    } else {
        for (uint32_t t = lid; t < vocab; t += KD_THREADS) token(t, lg[t], first[t]);
    }
    __syncthreads();
    if (lid < 256u) {
        float s = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < KD_COPIES; w += 1) s += H0[w][lid];
        H[0][lid] = s;
    }
    __syncthreads();

    for (uint32_t l = warp; l < nd; l += KD_WARPS) {  // :129-146, one warp per depth
        float ztrue = 0.0f;
        for (uint32_t k = l + 1u; k <= KD_D; k += 1) ztrue += A[k];
        float v[8];  // byte b = lane + 32 * i
        float sum = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 8; i += 1) {
            v[i] = H[l][lane + 32u * i];
            sum += v[i];
        }
#pragma unroll
        for (uint32_t s = 16; s > 0; s >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, s);
        const float total = fmaxf(ztrue + sum, 1e-30f);
        if (lane == 0) o[l * KD_K] = kd_pack_entry(kd_byte_at(cw, l), ztrue / total);
        for (uint32_t j = 1; j < KD_K; j += 1) {
            // largest remaining mass, lowest byte among equals (:74-94)
            float bv = v[0];
            uint32_t bi = lane;
#pragma unroll
            for (uint32_t i = 1; i < 8; i += 1) {
                if (v[i] > bv) {
                    bv = v[i];
                    bi = lane + 32u * i;
                }
            }
#pragma unroll
            for (uint32_t s = 16; s > 0; s >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, s);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, s);
                if (ov > bv || (ov == bv && oi < bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            if ((bi & 31u) == lane) {
                o[l * KD_K + j] = kd_pack_entry(bi, bv / total);
#pragma unroll
                for (uint32_t i = 0; i < 8; i += 1) {
                    if (i == (bi >> 5)) v[i] = -1.0f;
                }
            }
        }
    }
    __syncthreads();  // the tables are zeroed again for the next row
    }
}

extern "C" void moe_cuda_kd_bytes(moe_cuda_ctx_t *c, const float *logits, const uint32_t *toks, const uint32_t *cont,
                                  uint32_t *outp, struct mda_pc_kd_bytes_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, logits != NULL && toks != NULL && cont != NULL && outp != NULL, "kd_bytes: null buffer");
    MOE_REQUIRE(c, pc.vocab >= 1, "kd_bytes: empty vocabulary");
    if (pc.rows == 0) return;
    uint16_t *first = (uint16_t *)moe_scratch(c, MOE_SCR_STAGE, (size_t)pc.vocab * 2 + 16);
    if (first == NULL) return;
    moe_kd_first_kernel<<<(pc.vocab + 255u) / 256u, 256, 0, c->stream>>>(toks, first, pc.vocab);
    MOE_LAUNCHED(c);
    const uint32_t grid = pc.rows < (uint32_t)c->sm_count ? pc.rows : (uint32_t)c->sm_count;
    moe_kd_bytes_kernel<<<grid, KD_THREADS, 0, c->stream>>>(logits, toks, first, cont, outp, pc.vocab, pc.rows);
    MOE_LAUNCHED(c);
}
