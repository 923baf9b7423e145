// Weighted gather-sum back to token order, and the three elementwise glue
// kernels that sit between the two grouped products in the unfused sequence.
// CUDA for sm_100a; all HBM access is 128-bit and coalesced along the row.
#include "moe_common.cuh"

#define CB_THREADS 256
#define CB_MAXV 8  // float4 per thread kept for the fused norm: d <= 8192

__device__ __forceinline__ float moe_sigmoid(float v) {  // shader/moe_combine.comp:22-24
    return 1.0f / (1.0f + expf(-v));
}

__device__ __forceinline__ float4 moe_load4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float4 moe_load4(const __half *p) {
    uint2 raw = __ldg(reinterpret_cast<const uint2 *>(p));
    float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&raw.x));
    float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&raw.y));
    return make_float4(a.x, a.y, b.x, b.y);
}

// One block per row (shader/moe_combine.comp:26-40 uses one thread per element).
// acc = sum_j wt[r,j] * y[slot[r,j], c] in j order with separately rounded
// multiply and add, as the expression is written in the shader (:32-34).
template <typename YT, bool NORM, bool PEER>
__global__ void __launch_bounds__(CB_THREADS)
moe_combine_kernel(moe_combine_args a) {
    __shared__ uint32_t s_slot[MOE_MAX_TOPK];
    __shared__ float s_wt[MOE_MAX_TOPK];
    __shared__ float s_f[8];
    __shared__ float s_red[CB_THREADS / 32];
    __shared__ const YT *s_y[PEER ? MOE_MAX_TOPK : 1];
    __shared__ uint32_t s_mask, s_terms;
    const YT *y = reinterpret_cast<const YT *>(a.y);
    // One row per block and pass (rows blockIdx.x, blockIdx.x + gridDim.x, ...).
    for (uint32_t r = blockIdx.x; r < a.rows; r += gridDim.x) {
        if (PEER && a.per_gpu) {
            // Expert-parallel, one row per owning GPU: every GPU that owns some of the token's experts has
            // already summed wt * row over those experts (moe_ep_partial_kernel); one such partial row per
            // GPU comes over NVLink and the partial rows are added in ascending GPU order.
            if (threadIdx.x == 0) s_mask = 0;
            __syncthreads();
            if (threadIdx.x < a.topk) {
                uint32_t g = a.idx[(size_t)r * a.topk + threadIdx.x] / a.experts_per_rank;
                if (g < a.world) atomicOr(&s_mask, 1u << g);  // a row the router refused carries ~0: no term
            }
            __syncthreads();
            if (threadIdx.x == 0) {
                uint32_t n = 0;
                for (uint32_t mk = s_mask; mk != 0; mk &= mk - 1u, n += 1) {
                    s_y[n] = reinterpret_cast<const YT *>(a.y_peers[__ffs((int)mk) - 1]);
                    s_slot[n] = a.src_base + r;
                    s_wt[n] = 1.0f;
                }
                s_terms = n;
            }
        } else if (threadIdx.x < a.topk) {
            uint32_t sl = a.slot[(size_t)r * a.topk + threadIdx.x];
            if (PEER) {  // expert-parallel, one row per pair: read from the GPU that owns the expert, over NVLink
                const uint32_t g = a.idx[(size_t)r * a.topk + threadIdx.x] / a.experts_per_rank;
                s_y[threadIdx.x] = reinterpret_cast<const YT *>(a.y_peers[g < a.world ? g : 0u]);
                if (g >= a.world) sl = ~0u;
            }
            s_slot[threadIdx.x] = sl;  // ~0: a pair the router refused, contributes nothing
            s_wt[threadIdx.x] = a.wt[(size_t)r * a.topk + threadIdx.x];
        }
        if (threadIdx.x >= 32 && threadIdx.x < 32 + a.hc && a.hc <= 7) {
            uint32_t s = threadIdx.x - 32;
            float iv = a.inj != NULL ? a.inj[(size_t)r * a.inj_stride + a.inj_off + s] : 0.0f;
            s_f[s] = moe_sigmoid(iv / (float)a.hc);  // :37
        }
        if (threadIdx.x == 64) {
            s_f[7] = a.sh != NULL ? moe_sigmoid(a.proj[(size_t)r * a.pstride + a.sg_off]) : 0.0f;  // :35
        }
        __syncthreads();
        const uint32_t terms = (PEER && a.per_gpu) ? s_terms : a.topk;
        float sg = s_f[7];
        float4 keep[NORM ? CB_MAXV : 1];
        float ss = 0.0f;
        uint32_t it = 0;
        for (uint32_t c = threadIdx.x * 4u; c < a.d; c += CB_THREADS * 4u, it += 1) {
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t j = 0; j < terms; j += 1) {
                if (s_slot[j] == ~0u) continue;
                float4 v = moe_load4((PEER ? s_y[j] : y) + (size_t)s_slot[j] * a.d + c);
                float w = s_wt[j];
                acc.x = __fadd_rn(acc.x, __fmul_rn(w, v.x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(w, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(w, v.z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(w, v.w));
            }
            if (a.sh != NULL) {
                float4 v = moe_load4(a.sh + (size_t)r * a.d + c);
                acc.x = __fadd_rn(acc.x, __fmul_rn(sg, v.x));
                acc.y = __fadd_rn(acc.y, __fmul_rn(sg, v.y));
                acc.z = __fadd_rn(acc.z, __fmul_rn(sg, v.z));
                acc.w = __fadd_rn(acc.w, __fmul_rn(sg, v.w));
            }
            if (NORM) {
                float4 xv = moe_load4(a.x16 + (size_t)r * a.d + c);
                float f = s_f[0];
                float4 v;
                v.x = __fadd_rn(xv.x, __fmul_rn(__fmul_rn(acc.x, 2.0f), f));
                v.y = __fadd_rn(xv.y, __fmul_rn(__fmul_rn(acc.y, 2.0f), f));
                v.z = __fadd_rn(xv.z, __fmul_rn(__fmul_rn(acc.z, 2.0f), f));
                v.w = __fadd_rn(xv.w, __fmul_rn(__fmul_rn(acc.w, 2.0f), f));
                keep[it] = v;
                ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
            }
            if (a.h != NULL) {
                for (uint32_t s = 0; s < a.hc; s += 1) {  // :36-38
                    float f = a.hc <= 7 ? s_f[s]
                                        : moe_sigmoid((a.inj != NULL ? a.inj[(size_t)r * a.inj_stride + a.inj_off + s] : 0.0f) / (float)a.hc);
                    float4 *hp = reinterpret_cast<float4 *>(a.h + ((size_t)r * a.hc + s) * a.d + c);
                    float4 hv = *hp;
                    hv.x = __fadd_rn(hv.x, __fmul_rn(__fmul_rn(acc.x, 2.0f), f));
                    hv.y = __fadd_rn(hv.y, __fmul_rn(__fmul_rn(acc.y, 2.0f), f));
                    hv.z = __fadd_rn(hv.z, __fmul_rn(__fmul_rn(acc.z, 2.0f), f));
                    hv.w = __fadd_rn(hv.w, __fmul_rn(__fmul_rn(acc.w, 2.0f), f));
                    *hp = hv;
                }
            }
        }
        if (NORM) {
            // residual + RMSNorm with unit weight (shader/qwen_norm.comp:55-61,79 op 0)
#pragma unroll
            for (uint32_t o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if ((threadIdx.x & 31u) == 0) s_red[threadIdx.x >> 5] = ss;
            __syncthreads();
            float tot = 0.0f;
#pragma unroll
            for (uint32_t w = 0; w < CB_THREADS / 32; w += 1) tot += s_red[w];
            float inv = 1.0f / sqrtf(tot / (float)a.d + a.eps);
            it = 0;
            for (uint32_t c = threadIdx.x * 4u; c < a.d; c += CB_THREADS * 4u, it += 1) {
                float4 v = keep[it];
                __half2 lo = __floats2half2_rn(v.x * inv, v.y * inv);
                __half2 hi = __floats2half2_rn(v.z * inv, v.w * inv);
                uint2 out;
                out.x = *reinterpret_cast<uint32_t *>(&lo);
                out.y = *reinterpret_cast<uint32_t *>(&hi);
                *reinterpret_cast<uint2 *>(a.y16 + (size_t)r * a.d + c) = out;
            }
        }
        __syncthreads();  // the row's tables are rewritten by the next pass
    }
}

// Lets the kernels that move rows over NVLink share an SM with a resident grouped-product CTA: a
// kernel can only join an SM whose shared-memory carve-out matches its own, and the products run
// with the maximum carve-out.
void moe_overlap_prepare_combine(moe_cuda_ctx *c) {
    MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_combine_kernel<__half, false, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared));
    MOE_CUDA_TRY(c, cudaFuncSetAttribute(moe_combine_kernel<__half, true, true>, cudaFuncAttributePreferredSharedMemoryCarveout,
                                         cudaSharedmemCarveoutMaxShared));
}

void moe_launch_combine(moe_cuda_ctx *c, const moe_combine_args &a) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, (a.y_peers != NULL && a.per_gpu) || (a.wt != NULL && a.slot != NULL && (a.y != NULL || a.y_peers != NULL)),
                "combine: null buffer");
    MOE_REQUIRE(c, a.y_peers == NULL || (a.idx != NULL && a.experts_per_rank >= 1 && a.world >= 1 && a.world <= 16),
                "combine: peer rows need idx and the world size");
    MOE_REQUIRE(c, a.h != NULL || a.y16 != NULL, "combine: no output");
    MOE_REQUIRE(c, a.sh == NULL || a.proj != NULL, "combine: shared term needs proj");
    MOE_REQUIRE(c, a.topk >= 1 && a.topk <= MOE_MAX_TOPK, "combine: topk %u outside 1..16", a.topk);
    MOE_REQUIRE(c, a.d % 4 == 0 && a.d >= 4, "combine: d %u not a multiple of 4", a.d);
    MOE_REQUIRE(c, a.hc >= 1, "combine: hc 0");
    MOE_REQUIRE(c, ((uintptr_t)a.y & 15) == 0 && ((uintptr_t)a.h & 15) == 0 && ((uintptr_t)a.sh & 15) == 0,
                "combine: buffers not 16-byte aligned");
    if (a.y16 != NULL) {
        MOE_REQUIRE(c, a.x16 != NULL && a.hc == 1 && a.d <= CB_THREADS * 4 * CB_MAXV, "combine: fused norm needs x16, hc 1, d <= 8192");
    }
    if (a.rows == 0) return;
    const bool peer = a.y_peers != NULL;
    MOE_REQUIRE(c, !peer || a.y_is_f16, "combine: peer rows are fp16");
    // One block per row: the peer loads want every row in flight.  (A grid bounded to two blocks per SM, meant to
    // leave room for another token slice's product CTAs, measured 115 us against 47 us for the return over 2 GPUs
    // and 0.686 ms against 0.670 ms per layer over 8.)
    const uint32_t grid = a.rows;
    if (a.y16 != NULL) {
        if (peer) moe_combine_kernel<__half, true, true><<<grid, CB_THREADS, 0, c->stream>>>(a);
        else if (a.y_is_f16) moe_combine_kernel<__half, true, false><<<grid, CB_THREADS, 0, c->stream>>>(a);
        else moe_combine_kernel<float, true, false><<<grid, CB_THREADS, 0, c->stream>>>(a);
    } else {
        if (peer) moe_combine_kernel<__half, false, true><<<grid, CB_THREADS, 0, c->stream>>>(a);
        else if (a.y_is_f16) moe_combine_kernel<__half, false, false><<<grid, CB_THREADS, 0, c->stream>>>(a);
        else moe_combine_kernel<float, false, false><<<grid, CB_THREADS, 0, c->stream>>>(a);
    }
    MOE_LAUNCHED(c);
}

extern "C" void moe_cuda_combine(moe_cuda_ctx_t *c, const float *wt, const uint32_t *slot, const float *y,
                                 const float *proj, const float *sh, const float *inj, float *h,
                                 struct mda_pc_moe_combine_t pc) {
    moe_combine_args a = {};
    a.wt = wt;
    a.slot = slot;
    a.y = y;
    a.proj = proj;
    a.sh = sh;
    a.inj = inj;
    a.h = h;
    a.rows = pc.rows;
    a.d = pc.d;
    a.topk = pc.topk;
    a.pstride = pc.pstride;
    a.sg_off = pc.sg_off;
    a.inj_stride = pc.inj_stride;
    a.inj_off = pc.inj_off;
    a.hc = pc.hc;
    a.y_is_f16 = false;
    moe_launch_combine(c, a);
}

// ---- glue: shader/qwen_elem.comp op 0, shader/absmax.comp, shader/cast_f16.comp ----
__device__ __forceinline__ float moe_silu(float v) { return v / (1.0f + expf(-v)); }  // qwen_elem.comp:16-18

__global__ void moe_swiglu_kernel(const float *__restrict__ a, float *__restrict__ y, uint32_t rows, uint32_t n,
                                  uint32_t astride, uint32_t ao, uint32_t bo, uint32_t op, float scale) {
    size_t total = (size_t)rows * n;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        size_t r = i / n;
        uint32_t cidx = (uint32_t)(i - r * n);
        float g = a[r * astride + ao + cidx];
        if (op == 0u) y[i] = __fmul_rn(moe_silu(g), a[r * astride + bo + cidx]);  // qwen_elem.comp:27
        else y[i] = moe_silu(__fmul_rn(g, scale));                                // :29 (the mixer's gate, src/qwen.c:648-657)
    }
}

extern "C" void moe_cuda_swiglu(moe_cuda_ctx_t *c, const float *a, float *y, struct mda_pc_qwen_elem_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, pc.op <= 1u, "swiglu: op %u (the shader has 0: silu(gate)*up and 1: silu(scale*a))", pc.op);
    MOE_REQUIRE(c, a != NULL && y != NULL, "swiglu: null buffer");
    size_t total = (size_t)pc.rows * pc.n;
    if (total == 0) return;
    size_t blocks = (total + 255) / 256;
    if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
    moe_swiglu_kernel<<<(unsigned)blocks, 256, 0, c->stream>>>(a, y, pc.rows, pc.n, pc.astride, pc.ao, pc.bo, pc.op, pc.scale);
    MOE_LAUNCHED(c);
}

__global__ void __launch_bounds__(256)
moe_absmax_kernel(const float *__restrict__ x, uint32_t *__restrict__ amax, size_t n, uint32_t slot) {
    __shared__ float red[8];
    size_t stride = (size_t)gridDim.x * blockDim.x;
    float m = 0.0f;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) m = fmaxf(m, fabsf(x[i]));
#pragma unroll
    for (uint32_t o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w += 1) m = fmaxf(m, red[w]);
        atomicMax(&amax[slot], __float_as_uint(m));  // absmax.comp:29; valid for non-negative floats
    }
}

extern "C" void moe_cuda_absmax(moe_cuda_ctx_t *c, const float *x, uint32_t *amax, struct mda_pc_absmax_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, x != NULL && amax != NULL && pc.slot != MDA_PC_NO_SLOT, "absmax: null buffer or no slot");
    if (pc.n == 0) return;
    uint32_t blocks = (pc.n + 255u) / 256u;
    if (blocks > (uint32_t)c->sm_count * 8u) blocks = (uint32_t)c->sm_count * 8u;
    moe_absmax_kernel<<<blocks, 256, 0, c->stream>>>(x, amax, pc.n, pc.slot);
    MOE_LAUNCHED(c);
}

__global__ void moe_cast_f16_kernel(const float *__restrict__ src, __half *__restrict__ dst, size_t n,
                                    const uint32_t *__restrict__ amax, uint32_t slot) {
    float s = moe_slot_scale(amax, slot);
    size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        dst[i] = __float2half_rn(src[i] * s);  // cast_f16.comp:33
    }
}

extern "C" void moe_cuda_cast_f16(moe_cuda_ctx_t *c, const float *src, void *dst, const uint32_t *amax,
                                  struct mda_pc_cast_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, src != NULL && dst != NULL && (amax != NULL || pc.slot == MDA_PC_NO_SLOT), "cast: null buffer");
    if (pc.n == 0) return;
    uint32_t blocks = (pc.n + 255u) / 256u;
    if (blocks > (uint32_t)c->sm_count * 16u) blocks = (uint32_t)c->sm_count * 16u;
    moe_cast_f16_kernel<<<blocks, 256, 0, c->stream>>>(src, (__half *)dst, pc.n, amax, pc.slot);
    MOE_LAUNCHED(c);
}

// ---- weight upload step: shader/qwen_bf16.comp (call src/qwen.c:365-378) ----
// The reference uploads a layer's bf16 weights and rewrites them in place as fp16 on the
// device.  HBM bound (2 bytes read + 2 bytes written per value): 128-bit accesses, grid-stride.
__device__ __forceinline__ uint32_t moe_bf16x2_to_f16x2(uint32_t u) {
    __half2 h = __floats2half2_rn(__uint_as_float(u << 16), __uint_as_float(u & 0xffff0000u));  // qwen_bf16.comp:13
    return *reinterpret_cast<uint32_t *>(&h);
}

__global__ void moe_bf16_to_f16_kernel(uint32_t *__restrict__ w, size_t n) {
    size_t n4 = n / 4;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    uint4 *w4 = reinterpret_cast<uint4 *>(w);
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        uint4 v = w4[i];
        v.x = moe_bf16x2_to_f16x2(v.x);
        v.y = moe_bf16x2_to_f16x2(v.y);
        v.z = moe_bf16x2_to_f16x2(v.z);
        v.w = moe_bf16x2_to_f16x2(v.w);
        w4[i] = v;
    }
    size_t tail = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (tail < n) w[tail] = moe_bf16x2_to_f16x2(w[tail]);
}

extern "C" void moe_cuda_bf16_to_f16(moe_cuda_ctx_t *c, void *w, struct mda_pc_qwen_bf16_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, w != NULL && ((uintptr_t)w & 15) == 0, "bf16_to_f16: null or unaligned buffer");
    if (pc.n == 0) return;
    size_t blocks = ((size_t)pc.n / 4 + 255) / 256;
    if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
    if (blocks == 0) blocks = 1;
    moe_bf16_to_f16_kernel<<<(unsigned)blocks, 256, 0, c->stream>>>((uint32_t *)w, pc.n);
    MOE_LAUNCHED(c);
}
