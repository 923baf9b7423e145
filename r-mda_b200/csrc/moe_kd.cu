// The teacher's distillation sink (shader/kd_bytes.comp; call mda_teach_sink,
// src/teach.c:108-128): next-token logits over a byte-level vocabulary become
// per-byte distributions along the true continuation.  For depth l < nd, among
// the tokens longer than l bytes that agree with the continuation on its first
// l bytes: the probability that byte l is the true one (entry 0) and the seven
// most probable other bytes (entries 1..7), each packed as byte | fp16(p) << 16.
//
// Two persistent blocks of 512 threads per SM take rows in turn (one block's
// barriers and load latencies are covered by the other's work): 16-byte loads
// for the row maximum, then the exponentials of the same row, largely out of L2.  Nearly every token differs from the true continuation in its first
// byte and then only adds its mass to that byte's bin at depth 0.  The shader
// does that with one shared-memory atomic per token (:122-125); here the
// vocabulary is cut into chunks of 4096 tokens and, once per call, every chunk
// is sorted by first byte (moe_kd_sort_kernel: position -> token, position ->
// byte).  A row's chunk of logits is staged in shared memory and read back in
// sorted order, eight consecutive positions per thread, so that a thread -- and
// nearly always its whole warp -- adds up masses of one byte in registers and one
// lane issues one atomic per warp and chunk.  Only tokens that share the
// continuation's first byte read their 20-byte record and take the shader's path.
// The per-depth totals and the top-7 selection run warp-parallel (one depth per
// warp, shuffles only) instead of the shader's 112 block-wide reductions per row.
#include "moe_common.cuh"

#define KD_D 16u        // MDA_KD_DEPTH, src/kd.h:11
#define KD_K 8u         // MDA_KD_K, src/kd.h:12
#define KD_THREADS 512u
#define KD_WARPS (KD_THREADS / 32u)
#define KD_COPIES 4u    // private copies of the depth-0 bins (a power of two)
#define KD_CHUNK 4096u  // tokens per sorted chunk = 8 per thread
#define KD_NOKEY 256u   // sort key of a token without a byte string

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

// One block per chunk of KD_CHUNK tokens: counting sort by first byte (tokens without a byte string last).
// perm[chunk * KD_CHUNK + position] = index of the token inside the chunk, key[...] = its first byte or KD_NOKEY,
// bstart[chunk * 258 + b] = first position of byte b (entry 257 = KD_CHUNK).
__global__ void __launch_bounds__(KD_THREADS)
moe_kd_sort_kernel(const uint32_t *__restrict__ toks, uint16_t *__restrict__ perm, uint16_t *__restrict__ key,
                   uint16_t *__restrict__ bstart, uint32_t vocab) {
    __shared__ uint32_t cursor[KD_NOKEY + 1u];
    __shared__ uint32_t total[KD_NOKEY + 1u];
    const uint32_t base = blockIdx.x * KD_CHUNK, lid = threadIdx.x;
    for (uint32_t i = lid; i <= KD_NOKEY; i += KD_THREADS) total[i] = 0u;
    __syncthreads();
    uint32_t k[KD_CHUNK / KD_THREADS];
#pragma unroll
    for (uint32_t i = 0; i < KD_CHUNK / KD_THREADS; i += 1) {
        const uint32_t t = base + i * KD_THREADS + lid;
        k[i] = KD_NOKEY;
        if (t < vocab && toks[(size_t)t * 5u + 4u] != 0u) k[i] = toks[(size_t)t * 5u] & 0xffu;
        atomicAdd(&total[k[i]], 1u);  // tokens past the end of the vocabulary count as "no byte string"
    }
    __syncthreads();
    if (lid == 0) {
        uint32_t run = 0;
        for (uint32_t i = 0; i <= KD_NOKEY; i += 1) {
            cursor[i] = run;
            bstart[(size_t)blockIdx.x * 258u + i] = (uint16_t)run;
            run += total[i];
        }
        bstart[(size_t)blockIdx.x * 258u + 257u] = (uint16_t)run;
    }
    __syncthreads();
#pragma unroll
    for (uint32_t i = 0; i < KD_CHUNK / KD_THREADS; i += 1) {
        const uint32_t pos = atomicAdd(&cursor[k[i]], 1u);
        perm[(size_t)base + pos] = (uint16_t)(i * KD_THREADS + lid);
        key[(size_t)base + pos] = (uint16_t)k[i];
    }
}

__global__ void __launch_bounds__(KD_THREADS, 2)
moe_kd_bytes_kernel(const float *__restrict__ logits, const uint32_t *__restrict__ toks, const uint16_t *__restrict__ perm,
                    const uint16_t *__restrict__ key, const uint16_t *__restrict__ bstart, const uint32_t *__restrict__ cont,
                    uint32_t *__restrict__ outp, uint32_t vocab, uint32_t rows) {
    __shared__ float A[KD_D + 1u];
    __shared__ float H[KD_D][256];
    __shared__ float H0[KD_COPIES][256];
    __shared__ float s_max[KD_WARPS];
    extern __shared__ __align__(16) float stage[];  // two buffers of KD_CHUNK logits
    const uint32_t lid = threadIdx.x, lane = lid & 31u, warp = lid >> 5;
    const bool vec = (vocab & 3u) == 0u && ((uintptr_t)logits & 15u) == 0u;
    const uint32_t n_chunks = (vocab + KD_CHUNK - 1u) / KD_CHUNK;
    for (uint32_t r = blockIdx.x; r < rows; r += gridDim.x) {
    uint32_t cw[4];
#pragma unroll
    for (uint32_t i = 0; i < 4; i += 1) cw[i] = cont[(size_t)r * 5u + i];
    const uint32_t nd = min(cont[(size_t)r * 5u + 4u], KD_D);  // :100
    const uint32_t c0 = cw[0] & 0xffu;
    uint32_t *o = outp + (size_t)r * KD_D * KD_K;
    for (uint32_t i = nd * KD_K + lid; i < KD_D * KD_K; i += KD_THREADS) o[i] = 0u;  // :101-103
    if (nd == 0u) continue;  // no depth asked for: nothing but the zeros (the whole block takes this branch)
    if (lid <= KD_D) A[lid] = 0.0f;
    for (uint32_t i = lid; i < KD_D * 256u; i += KD_THREADS) (&H[0][0])[i] = 0.0f;
    for (uint32_t i = lid; i < KD_COPIES * 256u; i += KD_THREADS) (&H0[0][0])[i] = 0.0f;

    const float *lg = logits + (size_t)r * vocab;
    float m = -3.0e38f;  // :110-114
    if (vec) {
        const float4 *lg4 = reinterpret_cast<const float4 *>(lg);
        const uint32_t n4 = vocab / 4u;
        uint32_t q = lid;
        for (; q + 3u * KD_THREADS < n4; q += 4u * KD_THREADS) {  // four loads in flight per thread
            const float4 v0 = lg4[q], v1 = lg4[q + KD_THREADS], v2 = lg4[q + 2u * KD_THREADS], v3 = lg4[q + 3u * KD_THREADS];
            m = fmaxf(m, fmaxf(fmaxf(fmaxf(v0.x, v0.y), fmaxf(v0.z, v0.w)), fmaxf(fmaxf(v1.x, v1.y), fmaxf(v1.z, v1.w))));
            m = fmaxf(m, fmaxf(fmaxf(fmaxf(v2.x, v2.y), fmaxf(v2.z, v2.w)), fmaxf(fmaxf(v3.x, v3.y), fmaxf(v3.z, v3.w))));
        }
        for (; q < n4; q += KD_THREADS) {
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

    // :115-127, chunk by chunk; the next chunk's logits are fetched while this one is worked on
    struct Eight {
        float4 lo, hi;
    };
    auto fetch = [&](uint32_t c) -> Eight {  // tokens base + 8 lid .. + 7
        const uint32_t base = c * KD_CHUNK;
        Eight v;
        if (vec && base + KD_CHUNK <= vocab) {
            v.lo = reinterpret_cast<const float4 *>(lg + base)[2u * lid];
            v.hi = reinterpret_cast<const float4 *>(lg + base)[2u * lid + 1u];
            return v;
        }
        float f[8];
#pragma unroll
        for (uint32_t i = 0; i < 8; i += 1) {
            const uint32_t t = base + lid * 8u + i;
            f[i] = t < vocab ? lg[t] : 0.0f;
        }
        v.lo = make_float4(f[0], f[1], f[2], f[3]);
        v.hi = make_float4(f[4], f[5], f[6], f[7]);
        return v;
    };
    auto put = [&](float *buf, const Eight &v) {
        reinterpret_cast<float4 *>(buf)[2u * lid] = v.lo;
        reinterpret_cast<float4 *>(buf)[2u * lid + 1u] = v.hi;
    };
    put(stage, fetch(0));
    __syncthreads();
    for (uint32_t c = 0; c < n_chunks; c += 1) {
        const uint32_t base = c * KD_CHUNK;
        const float *st = stage + (c & 1u) * KD_CHUNK;
        Eight nxt;
        nxt.lo = nxt.hi = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        if (c + 1u < n_chunks) nxt = fetch(c + 1u);
        // the tokens that share the continuation's first byte: their records are asked for now and used after the sweep
        const uint32_t s0 = bstart[(size_t)c * 258u + c0], s1 = bstart[(size_t)c * 258u + c0 + 1u];
        uint32_t early_tl = 0, early_w[5] = {0u, 0u, 0u, 0u, 0u};
        if (s0 + lid < s1) {
            early_tl = perm[(size_t)base + s0 + lid];
            const uint32_t *tp = toks + (size_t)(base + early_tl) * 5u;
#pragma unroll
            for (uint32_t q = 0; q < 5; q += 1) early_w[q] = tp[q];
        }
        // eight consecutive positions of the sorted chunk
        const uint4 pp = reinterpret_cast<const uint4 *>(perm + (size_t)base)[lid];
        const uint4 kk = reinterpret_cast<const uint4 *>(key + (size_t)base)[lid];
        const uint32_t pos_tok[8] = {pp.x & 0xffffu, pp.x >> 16, pp.y & 0xffffu, pp.y >> 16, pp.z & 0xffffu, pp.z >> 16, pp.w & 0xffffu, pp.w >> 16};
        const uint32_t pos_key[8] = {kk.x & 0xffffu, kk.x >> 16, kk.y & 0xffffu, kk.y >> 16, kk.z & 0xffffu, kk.z >> 16, kk.w & 0xffffu, kk.w >> 16};
        uint32_t cur = KD_NOKEY;
        float acc = 0.0f;
#pragma unroll
        for (uint32_t i = 0; i < 8; i += 1) {
            const uint32_t b = pos_key[i];
            // no byte string (len == 0) or past the end of the vocabulary; or shares the first byte: handled below
            if (b == KD_NOKEY || b == c0) continue;
            const float e = expf(st[pos_tok[i]] - m);
            // differs in the first byte: depth 0, bin = that byte, and nothing else (a = 0)
            if (b != cur) {
                if (cur != KD_NOKEY) atomicAdd(&H0[warp & (KD_COPIES - 1u)][cur], acc);
                cur = b;
                acc = 0.0f;
            }
            acc += e;
        }
        // What is left in registers.  Positions are sorted, so lanes holding the same byte are neighbours: a
        // segmented scan over the warp leaves each byte's sum in the last lane of its run, which issues the
        // one atomic (lanes adding to one address would be serialised).
#pragma unroll
        for (uint32_t o = 1; o < 32; o <<= 1) {
            const float v = __shfl_up_sync(0xffffffffu, acc, o);
            const uint32_t cu = __shfl_up_sync(0xffffffffu, cur, o);
            if (lane >= o && cu == cur) acc += v;
        }
        const uint32_t nxc = __shfl_down_sync(0xffffffffu, cur, 1);
        if ((lane == 31u || nxc != cur) && cur != KD_NOKEY) atomicAdd(&H0[warp & (KD_COPIES - 1u)][cur], acc);
        // the tokens that share the continuation's first byte, one per thread: the shader's path with the full record
        for (uint32_t p0 = s0; p0 < s1; p0 += KD_THREADS) {  // whole warps stay together for the shuffles below
            const uint32_t p = p0 + lid;
            uint32_t a = 0u;
            float e = 0.0f;
            if (p < s1) {
                uint32_t tl = early_tl, len = early_w[4];
                uint32_t tw[4] = {early_w[0], early_w[1], early_w[2], early_w[3]};
                if (p0 != s0) {  // a run longer than the block: later rounds fetch their own
                    tl = perm[(size_t)base + p];
                    const uint32_t *tp = toks + (size_t)(base + tl) * 5u;
                    len = tp[4];
#pragma unroll
                    for (uint32_t q = 0; q < 4; q += 1) tw[q] = tp[q];
                }
                e = expf(st[tl] - m);
                const uint32_t lcp = kd_common_prefix(tw, cw);
                a = min(lcp, min(len, nd));
                if (lcp < nd && lcp < len) {
                    const uint32_t bb = kd_byte_at(tw, lcp);
                    if (lcp == 0u) atomicAdd(&H0[warp & (KD_COPIES - 1u)][bb], e);
                    else atomicAdd(&H[lcp][bb], e);
                }
            }
            // A[a] += e (A[0] is never read, :131-133): nearly all of these tokens agree on one byte only, so the
            // lanes of a warp are summed per value of a and one lane adds
            uint32_t todo = __ballot_sync(0xffffffffu, a != 0u);
            while (todo != 0u) {
                const uint32_t av = __shfl_sync(0xffffffffu, a, __ffs((int)todo) - 1);
                const bool mine = a == av;
                float sum = mine ? e : 0.0f;
#pragma unroll
                for (uint32_t sft = 16; sft > 0; sft >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, sft);
                if (lane == 0) atomicAdd(&A[av], sum);
                todo &= ~__ballot_sync(0xffffffffu, mine);
            }
        }
        put(stage + ((c + 1u) & 1u) * KD_CHUNK, nxt);
        __syncthreads();  // the next chunk is staged, this one's buffer is free
    }
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
    const uint32_t n_chunks = (pc.vocab + KD_CHUNK - 1u) / KD_CHUNK;
    uint16_t *perm = (uint16_t *)moe_scratch(c, MOE_SCR_STAGE, (size_t)n_chunks * (KD_CHUNK * 4 + 258 * 2) + 16);
    if (perm == NULL) return;
    uint16_t *key = perm + (size_t)n_chunks * KD_CHUNK;
    uint16_t *bstart = key + (size_t)n_chunks * KD_CHUNK;
    moe_kd_sort_kernel<<<n_chunks, KD_THREADS, 0, c->stream>>>(toks, perm, key, bstart, pc.vocab);
    MOE_LAUNCHED(c);
    const uint32_t grid = pc.rows < 2u * (uint32_t)c->sm_count ? pc.rows : 2u * (uint32_t)c->sm_count;
    const size_t stage_bytes = 2 * KD_CHUNK * sizeof(float);
    MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_kd_bytes_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)stage_bytes));
    moe_kd_bytes_kernel<<<grid, KD_THREADS, stage_bytes, c->stream>>>(logits, toks, perm, key, bstart, cont, outp, pc.vocab, pc.rows);
    MOE_LAUNCHED(c);
}
