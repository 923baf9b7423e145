// The kernels either side of the MoE path: the hyper-connection residual mixer
// that feeds every layer and the teacher's head (mda_qwen_res_rec,
// src/qwen.c:641-663; mda_qwen_head, src/qwen.c:1080-1099), and the dense fp16
// product both use (mda_qwen_mm, src/qwen.c:541-570).
//   moe_cuda_norm    shader/qwen_norm.comp op 0 / op 1 (grouped RMSNorm)
//   moe_cuda_hc      shader/qwen_hc.comp ops 0, 1, 2
//   moe_cuda_dense   C[rows x n] fp32 = A16[rows x k] * W[n x k]^T / scale(sa):
//                    the grouped tcgen05 kernel of moe_mm.cu over a dense tile
//                    schedule (one "expert", every 128-row tile used)
// Elementwise kernels are HBM bound: 128-bit accesses, coalesced along the row.
#include "moe_common.cuh"

#define NR_THREADS 256

__device__ __forceinline__ float dn_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }  // qwen_hc.comp:16-18

// One block per (row, group), as the shader (:64-67).  op 0: y = x * rsqrt(mean(x^2) + eps) * (1 + w);
// op 1: y = x * scale * rsqrt(sum(x^2) + 1e-6), no weight (:45-61).
__global__ void __launch_bounds__(NR_THREADS)
moe_norm_kernel(const float *__restrict__ x, const float *__restrict__ w, float *__restrict__ y, struct mda_pc_qwen_norm_t pc) {
    __shared__ float red[NR_THREADS / 32];
    const uint32_t r = blockIdx.x / pc.groups, g = blockIdx.x % pc.groups;
    const float *xi = x + (size_t)r * pc.in_stride + pc.in_off + (size_t)g * pc.in_gstride;
    float *yi = y + (size_t)r * pc.out_stride + pc.out_off + (size_t)g * pc.out_gstride;
    const float *wi = w != NULL ? w + pc.w_off + (size_t)g * pc.wstride : NULL;
    float acc = 0.0f;
    for (uint32_t c = threadIdx.x; c < pc.gsize; c += NR_THREADS) acc += xi[c] * xi[c];  // :71-73
#pragma unroll
    for (uint32_t o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if ((threadIdx.x & 31u) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    float ss = 0.0f;
#pragma unroll
    for (uint32_t q = 0; q < NR_THREADS / 32; q += 1) ss += red[q];
    const float f = pc.op == 1u ? pc.scale * rsqrtf(ss + 1e-6f) : rsqrtf(ss / (float)pc.gsize + pc.eps);  // :55-61
    for (uint32_t c = threadIdx.x; c < pc.gsize; c += NR_THREADS) {
        const float wt = (pc.op == 0u && wi != NULL) ? 1.0f + wi[c] : 1.0f;  // :45-53
        yi[c] = xi[c] * f * wt;                                              // :78,90
    }
}

extern "C" void moe_cuda_norm(moe_cuda_ctx_t *c, const float *x, const float *w, float *y, const float *z,
                              struct mda_pc_qwen_norm_t pc) {
    (void)z;  // binding 3 of the shader: only its op 2 reads it
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, pc.op <= 1u, "norm: only op 0 (weighted RMSNorm) and op 1 (scaled L2 norm) are part of this path");
    MOE_REQUIRE(c, x != NULL && y != NULL && (w != NULL || pc.op == 1u), "norm: null buffer");
    MOE_REQUIRE(c, pc.groups >= 1 && pc.gsize >= 1, "norm: empty group");
    if (pc.rows == 0) return;
    moe_norm_kernel<<<pc.rows * pc.groups, NR_THREADS, 0, c->stream>>>(x, w, y, pc);
    MOE_LAUNCHED(c);
}

// shader/qwen_hc.comp.  op 0: h[r,c] = mean_s sigmoid(a[r,s,c]) * b[r,s,c]  (the mixer's read-out, :24-30);
// op 1: h[r,s,c] += a[r,c] * 2*sigmoid(b[r*inj_stride + inj_off + s] / hc)  (:31-35);
// op 2: h[i] += a[i] + b[i]  (:36-38).
__global__ void moe_hc_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ h,
                              struct mda_pc_qwen_hc_t pc) {
    const size_t n = (size_t)pc.rows * pc.d * (pc.op == 2u ? pc.hc : 1u);
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        if (pc.op == 2u) {
            h[i] += a[i] + b[i];
            continue;
        }
        const size_t r = i / pc.d;
        const uint32_t col = (uint32_t)(i - r * pc.d);
        if (pc.op == 0u) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < pc.hc; s += 1) {
                const size_t j = (r * pc.hc + s) * pc.d + col;
                acc += dn_sigmoid(a[j]) * b[j];
            }
            h[i] = acc / (float)pc.hc;
        } else {
            for (uint32_t s = 0; s < pc.hc; s += 1) {
                const float g = 2.0f * dn_sigmoid(b[r * pc.inj_stride + pc.inj_off + s] / (float)pc.hc);
                h[(r * pc.hc + s) * pc.d + col] += a[i] * g;
            }
        }
    }
}

extern "C" void moe_cuda_hc(moe_cuda_ctx_t *c, const float *a, const float *b, float *h, struct mda_pc_qwen_hc_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, pc.op <= 2u && pc.hc >= 1 && pc.d >= 1, "hc: bad op or shape");
    MOE_REQUIRE(c, a != NULL && b != NULL && h != NULL, "hc: null buffer");
    const size_t n = (size_t)pc.rows * pc.d * (pc.op == 2u ? pc.hc : 1u);
    if (n == 0) return;
    size_t blocks = (n + 255) / 256;
    if (blocks > (size_t)c->sm_count * 16) blocks = (size_t)c->sm_count * 16;
    moe_hc_kernel<<<(unsigned)blocks, 256, 0, c->stream>>>(a, b, h, pc);
    MOE_LAUNCHED(c);
}

// mda_qwen_mm (src/qwen.c:541-570): the reference picks matmul_f16_wide.comp or the small-tile kernel by the
// number of 128 x 128 tiles; here one tcgen05 kernel serves both.  rows need not be a multiple of 128: rows of A
// beyond `rows` read as zero and rows of C beyond `rows` are not written.
extern "C" void moe_cuda_dense(moe_cuda_ctx_t *c, const void *A16, const void *W, float *C, const uint32_t *amax,
                               struct moe_pc_dense_t pc) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, A16 != NULL && W != NULL && C != NULL, "dense: null buffer");
    MOE_REQUIRE(c, pc.rows >= 1 && pc.n % 128u == 0 && pc.n >= 128u && pc.k % 8u == 0 && pc.k >= 8u,
                "dense: rows %u n %u k %u (n must be a multiple of 128, k of 8)", pc.rows, pc.n, pc.k);
    const uint32_t m = (pc.rows + MOE_TILE - 1u) / MOE_TILE * MOE_TILE;
    // the dense tile schedule: every 128-row tile belongs to "expert" 0
    uint32_t *tiles = (uint32_t *)moe_scratch(c, MOE_SCR_STAGE, (size_t)(m / MOE_TILE) * 4);
    if (tiles == NULL) return;
    MOE_CUDA_TRY(c, cudaMemsetAsync(tiles, 0, (size_t)(m / MOE_TILE) * 4, c->stream));
    moe_launch_mm(c, MOE_MM_F32, A16, W, C, amax, tiles, m, pc.n, pc.k, pc.sa, MDA_PC_NO_SLOT, 1, pc.rows, true, NULL, pc.rows);
}
