/*
 * moe_ref.c -- CPU oracle (TEST INFRASTRUCTURE ONLY; see moe_ref.h).
 *
 * Scalar restatement of the reference's MoE forward kernels.  PARITY UNPINNED:
 * the reference has no golden vectors for this path and its shaders cannot run
 * here, so nothing below has been compared with the reference's own output.
 *
 * Build: gcc -O3 -fopenmp -mavx2 -mf16c -mfma -ffp-contract=off -shared -fPIC
 * (contraction is off so that every elementwise expression rounds once per
 * operation as written; the only fused multiply-adds are the explicit ones in
 * the fp16 products, where a*b is exact in fp32 and fusing cannot change the
 * rounded sum).
 */
#include "moe_ref.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

float moe_ref_h2f(uint16_t h) {
    _Float16 v;
    memcpy(&v, &h, 2);
    return (float)v;
}

uint16_t moe_ref_f2h(float f) {
    _Float16 v = (_Float16)f; /* round to nearest even */
    uint16_t h;
    memcpy(&h, &v, 2);
    return h;
}

int moe_ref_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

/* Launchers such as torch.distributed.run export OMP_NUM_THREADS=1 to their
 * children; the timed CPU baseline asks for the machine's cores explicitly. */
void moe_ref_set_threads(int n) {
#ifdef _OPENMP
    if (n >= 1) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* shader/moe_route.comp:20-62.  The shader gives each of 32 lanes 16 candidate
 * columns and reduces (max value, then min index among the lanes holding it);
 * within a lane the scan keeps the first of equal values (strict >, :34).  The
 * net rule is: largest logit above the -3.0e38 sentinel among experts not yet
 * taken, ties to the lowest expert index.  The shader always scans 512 columns
 * (:24-26) and never reads `experts`; here candidates are e < experts. */
int moe_ref_route(const float *proj, uint32_t rows, uint32_t experts, uint32_t topk,
                  uint32_t stride, uint32_t *idx, float *wt, uint32_t *count) {
    int bad = 0;
    if (experts > MOE_REF_MAXE || topk > MOE_REF_MAXK) return -2;
#pragma omp parallel for schedule(static) reduction(| : bad)
    for (uint32_t r = 0; r < rows; r += 1) {
        const float *l = proj + (uint64_t)r * stride;
        uint8_t taken[MOE_REF_MAXE];
        uint32_t sel[MOE_REF_MAXK];
        float sv[MOE_REF_MAXK];
        memset(taken, 0, sizeof(taken));
        for (uint32_t k = 0; k < topk; k += 1) {
            float gm = -3.0e38f;   /* :31 */
            uint32_t gi = ~0u;     /* :32 */
            for (uint32_t e = 0; e < experts; e += 1) {
                if (!taken[e] && l[e] > gm) { /* :34, strict: first of equals wins */
                    gm = l[e];
                    gi = e;
                }
            }
            if (gi == ~0u) {
                bad |= 1;
            } else {
                taken[gi] = 1; /* :45-47 */
            }
            sel[k] = gi;
            sv[k] = gm;
        }
        float z = 0.0f; /* :52-55, accumulated k = 0..topk-1 in fp32 */
        for (uint32_t k = 0; k < topk; k += 1) {
            z += expf(sv[k] - sv[0]);
        }
        for (uint32_t k = 0; k < topk; k += 1) {
            idx[(uint64_t)r * topk + k] = sel[k];                  /* :57 */
            wt[(uint64_t)r * topk + k] = expf(sv[k] - sv[0]) / z;  /* :58 */
        }
    }
    if (bad) return -1;
    /* :59 atomicAdd(count[sel[k]], 1) -- order does not matter for a count */
    for (uint64_t i = 0; i < (uint64_t)rows * topk; i += 1) {
        count[idx[i]] += 1;
    }
    return 0;
}

/* shader/moe_scan.comp:14-38: pad each count to a multiple of tile, exclusive
 * prefix sum in rows, and one tiles[] entry per padded tile. */
void moe_ref_scan(const uint32_t *count, uint32_t experts, uint32_t tile, uint32_t *off,
                  uint32_t *tiles) {
    uint32_t run = 0;
    for (uint32_t e = 0; e < experts; e += 1) {
        uint32_t p = (count[e] + tile - 1u) / tile * tile; /* :19 */
        uint32_t lo = run;                                  /* :31 incl - p */
        off[e] = lo;                                        /* :33 */
        for (uint32_t t = lo / tile; t < (lo + p) / tile; t += 1) {
            tiles[t] = e;                                   /* :34-36 */
        }
        run += p;
    }
}

/* shader/moe_scatter.comp:18-33.  The shader takes positions with an atomic
 * (:25), so its order inside an expert is whatever order the groups land in;
 * visiting pr in ascending order gives the stable order by token index. */
void moe_ref_scatter(const uint32_t *idx, const uint32_t *off, uint32_t *fill,
                     const uint16_t *x16, uint16_t *xp, uint32_t *slot, uint32_t rows,
                     uint32_t topk, uint32_t d8) {
    uint64_t rowb = (uint64_t)d8 * 16u;
    for (uint64_t pr = 0; pr < (uint64_t)rows * topk; pr += 1) {
        uint32_t e = idx[pr];
        uint32_t p = off[e] + fill[e]; /* :25 */
        fill[e] += 1;
        slot[pr] = p;                  /* :27 */
    }
#pragma omp parallel for schedule(static)
    for (uint64_t pr = 0; pr < (uint64_t)rows * topk; pr += 1) {
        uint64_t r = pr / topk;        /* :20 */
        memcpy((uint8_t *)xp + slot[pr] * rowb, (const uint8_t *)x16 + r * rowb, rowb); /* :30-32 */
    }
}

/* shader/matmul_f16_moe.comp:60-68 = shader/cast_f16.comp:20-28. */
float moe_ref_slot_scale(const uint32_t *amax, uint32_t s) {
    if (s == MOE_REF_NO_SLOT) return 1.0f;
    float a;
    memcpy(&a, &amax[s], 4);
    if (!(a > 0.0f) || isinf(a)) return 1.0f;
    return exp2f(141.0f - (float)((amax[s] >> 23) & 0xffu));
}

#define NB 64u /* output columns per block of the CPU loop; not a reference constant */

/* shader/matmul_f16_moe.comp:70-126: C = A * B_e^T, fp16 operands widened to
 * fp32, fp32 accumulation (here in ascending k; the order inside the
 * reference's cooperative-matrix multiply is unspecified), epilogue scale
 * 1/(scale(sa)*scale(sb)) (:118-121). */
void moe_ref_mm(const uint16_t *A, const uint16_t *B, float *C, const uint32_t *amax,
                const uint32_t *tiles, uint32_t m, uint32_t n, uint32_t k, uint32_t sa,
                uint32_t sb, const uint8_t *row_mask) {
    const uint32_t TILE = 128u; /* :16 */
    float s = 1.0f / (moe_ref_slot_scale(amax, sa) * moe_ref_slot_scale(amax, sb));
    uint32_t ty = m / TILE;
    uint32_t nb = (n + NB - 1u) / NB;
#pragma omp parallel
    {
        float *bt = (float *)aligned_alloc(64, (size_t)k * NB * sizeof(float));
        float *ar = (float *)aligned_alloc(64, (size_t)((k + 15u) & ~15u) * sizeof(float));
#pragma omp for collapse(2) schedule(dynamic, 1)
        for (uint32_t y = 0; y < ty; y += 1) {
            for (uint32_t b = 0; b < nb; b += 1) {
                uint32_t e = tiles[y]; /* :71 */
                if (e == ~0u) continue; /* :72-74 */
                uint32_t m0 = y * TILE, n0 = b * NB;
                uint32_t nn = n - n0 < NB ? n - n0 : NB;
                int any = row_mask == NULL;
                for (uint32_t i = 0; i < TILE && !any; i += 1) any = row_mask[m0 + i] != 0;
                if (!any) continue;
                const uint16_t *Be = B + (uint64_t)e * n * k; /* :78 */
                for (uint32_t kk = 0; kk < k; kk += 1) {
                    for (uint32_t j = 0; j < NB; j += 1) {
                        bt[(size_t)kk * NB + j] =
                            j < nn ? moe_ref_h2f(Be[(uint64_t)(n0 + j) * k + kk]) : 0.0f;
                    }
                }
                for (uint32_t i = 0; i < TILE; i += 1) {
                    uint32_t r = m0 + i;
                    if (row_mask != NULL && row_mask[r] == 0) continue;
                    const uint16_t *a = A + (uint64_t)r * k;
                    for (uint32_t kk = 0; kk < k; kk += 1) ar[kk] = moe_ref_h2f(a[kk]);
                    float acc[NB];
                    for (uint32_t j = 0; j < NB; j += 1) acc[j] = 0.0f;
                    for (uint32_t kk = 0; kk < k; kk += 1) {
                        float av = ar[kk];
                        const float *bp = bt + (size_t)kk * NB;
#pragma omp simd
                        for (uint32_t j = 0; j < NB; j += 1) {
                            acc[j] = __builtin_fmaf(av, bp[j], acc[j]); /* a*b exact in fp32 */
                        }
                    }
                    for (uint32_t j = 0; j < nn; j += 1) {
                        C[(uint64_t)r * n + n0 + j] = acc[j] * s; /* :121-122 */
                    }
                }
            }
        }
        free(bt);
        free(ar);
    }
}

static float moe_ref_sigmoid(float v);

static float moe_ref_silu(float v) { /* shader/qwen_elem.comp:16-18 */
    return v / (1.0f + expf(-v));
}

/* shader/qwen_elem.comp:20-31 with op == 0: y = silu(a[ao+c]) * a[bo+c]. */
void moe_ref_swiglu(const float *a, float *y, uint32_t rows, uint32_t n, uint32_t astride,
                    uint32_t ao, uint32_t bo) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; r += 1) {
        for (uint32_t c = 0; c < n; c += 1) {
            float g = a[(uint64_t)r * astride + ao + c];
            y[(uint64_t)r * n + c] = moe_ref_silu(g) * a[(uint64_t)r * astride + bo + c];
        }
    }
}

/* shader/qwen_elem.comp:20-31 with op == 1: y = silu(a[ao+c] * scale)  (the mixer's gate, src/qwen.c:648-657). */
void moe_ref_silu_scaled(const float *a, float *y, uint32_t rows, uint32_t n, uint32_t astride, uint32_t ao,
                         float scale) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; r += 1) {
        for (uint32_t c = 0; c < n; c += 1) {
            y[(uint64_t)r * n + c] = moe_ref_silu(a[(uint64_t)r * astride + ao + c] * scale);
        }
    }
}

/* shader/qwen_norm.comp:63-92 with the contiguous strides of mda_qwen_norm_pc (src/qwen.c:582-604), ops 0 and 1:
 * per (row, group) ss = sum x^2 (the shader's tree reduction; here a plain sum in ascending c), then
 * op 0: y = x * rsqrt(ss / gsize + eps) * (1 + w[w_off + g * gsize + c]);  op 1: y = x * scale * rsqrt(ss + 1e-6). */
void moe_ref_norm(const float *x, const float *w, float *y, uint32_t rows, uint32_t groups, uint32_t gsize,
                  uint32_t w_off, uint32_t op, float eps, float scale) {
#pragma omp parallel for schedule(static)
    for (uint64_t rg = 0; rg < (uint64_t)rows * groups; rg += 1) {
        const uint32_t g = (uint32_t)(rg % groups);
        const float *xi = x + rg * gsize;
        float *yi = y + rg * gsize;
        float ss = 0.0f;
        for (uint32_t c = 0; c < gsize; c += 1) ss += xi[c] * xi[c];
        const float f = op == 1u ? scale / sqrtf(ss + 1e-6f) : 1.0f / sqrtf(ss / (float)gsize + eps);
        for (uint32_t c = 0; c < gsize; c += 1) {
            const float wt = op == 0u ? 1.0f + w[w_off + (uint64_t)g * gsize + c] : 1.0f;
            yi[c] = xi[c] * f * wt;
        }
    }
}

/* shader/qwen_hc.comp:20-39. */
void moe_ref_hc(const float *a, const float *b, float *h, uint32_t rows, uint32_t d, uint32_t hc, uint32_t op,
                uint32_t inj_stride, uint32_t inj_off) {
    if (op == 2u) {
        for (uint64_t i = 0; i < (uint64_t)rows * d * hc; i += 1) h[i] += a[i] + b[i];
        return;
    }
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < (uint64_t)rows * d; i += 1) {
        const uint64_t r = i / d, c = i % d;
        if (op == 0u) {
            float acc = 0.0f;
            for (uint32_t s = 0; s < hc; s += 1) {
                const uint64_t j = r * hc * d + (uint64_t)s * d + c;
                acc += moe_ref_sigmoid(a[j]) * b[j];
            }
            h[i] = acc / (float)hc;
        } else {
            for (uint32_t s = 0; s < hc; s += 1) {
                const float g = 2.0f * moe_ref_sigmoid(b[r * inj_stride + inj_off + s] / (float)hc);
                h[r * hc * d + (uint64_t)s * d + c] += a[i] * g;
            }
        }
    }
}

/* shader/absmax.comp:13-31: max |x| folded into amax[slot] as float bits. */
void moe_ref_absmax(const float *x, uint64_t n, uint32_t *amax, uint32_t slot) {
    float m = 0.0f;
#pragma omp parallel for schedule(static) reduction(max : m)
    for (uint64_t i = 0; i < n; i += 1) {
        float a = fabsf(x[i]);
        if (a > m) m = a; /* max(m, abs(x)) ; NaN never wins, as GLSL max(m, NaN) = m here */
    }
    uint32_t bits;
    memcpy(&bits, &m, 4);
    if (bits > amax[slot]) amax[slot] = bits; /* :29 atomicMax */
}

/* shader/cast_f16.comp:30-35. */
void moe_ref_cast_f16(const float *src, uint16_t *dst, uint64_t n, const uint32_t *amax,
                      uint32_t slot) {
    float s = moe_ref_slot_scale(amax, slot);
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; i += 1) {
        dst[i] = moe_ref_f2h(src[i] * s);
    }
}

static float moe_ref_sigmoid(float v) { /* shader/moe_combine.comp:22-24 */
    return 1.0f / (1.0f + expf(-v));
}

/* shader/moe_combine.comp:26-40. */
void moe_ref_combine(const float *wt, const uint32_t *slot, const float *y, const float *proj,
                     const float *sh, const float *inj, float *h, uint32_t rows, uint32_t d,
                     uint32_t topk, uint32_t pstride, uint32_t sg_off, uint32_t inj_stride,
                     uint32_t inj_off, uint32_t hc) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; r += 1) {
        float sg = sh != NULL ? moe_ref_sigmoid(proj[(uint64_t)r * pstride + sg_off]) : 0.0f;
        for (uint32_t c = 0; c < d; c += 1) {
            float acc = 0.0f;
            for (uint32_t j = 0; j < topk; j += 1) { /* :32-34, j ascending */
                acc += wt[(uint64_t)r * topk + j] * y[(uint64_t)slot[(uint64_t)r * topk + j] * d + c];
            }
            if (sh != NULL) acc += sg * sh[(uint64_t)r * d + c]; /* :35 */
            for (uint32_t s = 0; s < hc; s += 1) {               /* :36-38 */
                float iv = inj != NULL ? inj[(uint64_t)r * inj_stride + inj_off + s] : 0.0f;
                h[((uint64_t)r * hc + s) * d + c] += acc * 2.0f * moe_ref_sigmoid(iv / (float)hc);
            }
        }
    }
}

/* Residual add, RMSNorm with unit weight, fp16 store: the step between the
 * layers of the stacked configuration (shader/qwen_norm.comp:55-61,79 op 0:
 * sum of squares, y = x * inversesqrt(ss / n + eps)). */
void moe_ref_residual_rmsnorm(const uint16_t *x16, const float *delta, uint16_t *y16,
                              uint32_t rows, uint32_t d, float eps) {
#pragma omp parallel for schedule(static)
    for (uint32_t r = 0; r < rows; r += 1) {
        float ss = 0.0f;
        for (uint32_t c = 0; c < d; c += 1) {
            float v = moe_ref_h2f(x16[(uint64_t)r * d + c]) + delta[(uint64_t)r * d + c];
            ss += v * v;
        }
        float inv = 1.0f / sqrtf(ss / (float)d + eps);
        for (uint32_t c = 0; c < d; c += 1) {
            float v = moe_ref_h2f(x16[(uint64_t)r * d + c]) + delta[(uint64_t)r * d + c];
            y16[(uint64_t)r * d + c] = moe_ref_f2h(v * inv);
        }
    }
}

/* shader/qwen_bf16.comp:9-15: u -> packHalf2x16(float(lo bf16), float(hi bf16)). */
void moe_ref_bf16_to_f16(uint32_t *w, uint64_t n) {
#pragma omp parallel for schedule(static)
    for (uint64_t i = 0; i < n; i += 1) {
        uint32_t u = w[i];
        uint32_t lo_bits = u << 16, hi_bits = u & 0xffff0000u;
        float lo, hi;
        memcpy(&lo, &lo_bits, 4);
        memcpy(&hi, &hi_bits, 4);
        w[i] = (uint32_t)moe_ref_f2h(lo) | ((uint32_t)moe_ref_f2h(hi) << 16);
    }
}

/* shader/kd_bytes.comp:26-28 */
static uint32_t kd_byte_at(const uint32_t w[4], uint32_t i) {
    return (w[i >> 2] >> ((i & 3u) * 8u)) & 0xffu;
}

/* shader/kd_bytes.comp:30-39: index of the first byte in which the two 16-byte strings differ, or 16 */
static uint32_t kd_common_prefix(const uint32_t a[4], const uint32_t b[4]) {
    for (uint32_t i = 0; i < 16u; i += 1) {
        if (kd_byte_at(a, i) != kd_byte_at(b, i)) return i;
    }
    return 16u;
}

/* shader/kd_bytes.comp:70-72 */
static uint32_t kd_pack_entry(uint32_t b, float p) {
    return b | ((uint32_t)moe_ref_f2h(p) << 16);
}

/* shader/kd_bytes.comp:96-147.  The shader accumulates A and H with float atomics, i.e. in whatever
 * order the 256 threads arrive; here tokens are added in ascending order.  The 256-way sum of a
 * depth's byte masses follows the shader's halving tree (:55-68). */
void moe_ref_kd_bytes(const float *logits, const uint32_t *toks, const uint32_t *cont, uint32_t *outp,
                      uint32_t rows, uint32_t vocab) {
    enum { D = 16, K = 8 };
#pragma omp parallel for schedule(dynamic, 1)
    for (uint32_t r = 0; r < rows; r += 1) {
        const uint32_t *cw = cont + (size_t)r * 5u;
        const uint32_t nd = cont[(size_t)r * 5u + 4u] < D ? cont[(size_t)r * 5u + 4u] : D; /* :100 */
        uint32_t *o = outp + (size_t)r * D * K;
        for (uint32_t i = nd * K; i < D * K; i += 1) o[i] = 0u; /* :101-103 */
        float A[D + 1];
        static _Thread_local float H[D][256];
        memset(A, 0, sizeof(A));
        memset(H, 0, sizeof(H));
        const float *lg = logits + (size_t)r * vocab;
        float m = -3.0e38f; /* :110 */
        for (uint32_t t = 0; t < vocab; t += 1) m = lg[t] > m ? lg[t] : m;
        for (uint32_t t = 0; t < vocab; t += 1) { /* :115-127 */
            const uint32_t *tw = toks + (size_t)t * 5u;
            const uint32_t len = tw[4];
            if (len == 0u) continue;
            const float e = expf(lg[t] - m);
            const uint32_t lcp = kd_common_prefix(tw, cw);
            uint32_t a = len < nd ? len : nd;
            a = lcp < a ? lcp : a;
            A[a] += e;
            if (lcp < nd && lcp < len) H[lcp][kd_byte_at(tw, lcp)] += e;
        }
        for (uint32_t l = 0; l < nd; l += 1) { /* :129-146 */
            float ztrue = 0.0f;
            for (uint32_t k = l + 1u; k <= D; k += 1) ztrue += A[k];
            float red[256], v[256];
            memcpy(red, H[l], sizeof(red));
            memcpy(v, H[l], sizeof(v));
            for (uint32_t s = 128u; s > 0u; s >>= 1) {
                for (uint32_t i = 0; i < s; i += 1) red[i] += red[i + s];
            }
            float total = ztrue + red[0];
            total = total > 1e-30f ? total : 1e-30f;
            o[l * K] = kd_pack_entry(kd_byte_at(cw, l), ztrue / total);
            for (uint32_t j = 1; j < K; j += 1) {
                uint32_t b = 0; /* :74-94: largest mass, lowest byte among equals */
                for (uint32_t i = 1; i < 256u; i += 1) {
                    if (v[i] > v[b]) b = i;
                }
                o[l * K + j] = kd_pack_entry(b, v[b] / total);
                v[b] = -1.0f;
            }
        }
    }
}

/* src/qwen.c:788-836 (mda_qwen_route_rec) then src/qwen.c:847-906
 * (mda_qwen_moe_rec from the first grouped product on). */
int moe_ref_layer(moe_ref_layer_t *L) {
    uint32_t R = L->rows, K = L->topk, E = L->experts, d = L->d, I = L->inter, S = L->shared;
    uint32_t M = L->mrows, tile = L->tile;
    if (tile != 128u || M % 128u != 0u || d % 8u != 0u) return -2;
    /* src/qwen.c:793-798: count = 0, fill = 0, tiles = ~0, xp = 0 */
    uint32_t *fill = (uint32_t *)calloc(E, sizeof(uint32_t));
    memset(L->count, 0, E * sizeof(uint32_t));
    memset(L->tiles, 0xff, (size_t)(M / tile) * sizeof(uint32_t));
    memset(L->xp, 0, (size_t)M * d * sizeof(uint16_t));
    memset(L->amax, 0, 4 * sizeof(uint32_t)); /* src/qwen.c:500-503 */
    int rc = moe_ref_route(L->proj, R, E, K, L->pstride, L->idx, L->wt, L->count); /* :799-811 */
    if (rc != 0) {
        free(fill);
        return rc;
    }
    moe_ref_scan(L->count, E, tile, L->off, L->tiles);                               /* :812-821 */
    moe_ref_scatter(L->idx, L->off, fill, L->x16, L->xp, L->slot, R, K, d / 8u);     /* :822-835 */
    free(fill);

    /* rows of xp whose products are needed (all real rows unless the caller masks tokens) */
    uint8_t *pm = (uint8_t *)calloc(M, 1);
    for (uint64_t pr = 0; pr < (uint64_t)R * K; pr += 1) {
        if (L->row_mask == NULL || L->row_mask[pr / K]) pm[L->slot[pr]] = 1;
    }
    float *g = (float *)calloc((size_t)M * 2u * I, sizeof(float));
    float *hp = (float *)calloc((size_t)M * I, sizeof(float));
    uint16_t *hp16 = L->hp16 != NULL ? L->hp16 : (uint16_t *)malloc((size_t)M * I * sizeof(uint16_t));
    /* :847 gate_up product; sa = NO_SLOT because the activations are already
     * fp16 (a power-of-two rescale of fp16 data is an exact exponent shift) */
    moe_ref_mm(L->xp, L->wgu, g, L->amax, L->tiles, M, 2u * I, d, MOE_REF_NO_SLOT, MOE_REF_NO_SLOT, pm);
    moe_ref_swiglu(g, hp, M, I, 2u * I, 0u, I);       /* :848-857 */
    moe_ref_absmax(hp, (uint64_t)M * I, L->amax, 0u); /* :858-867 */
    moe_ref_cast_f16(hp, hp16, (uint64_t)M * I, L->amax, 0u); /* :868-877 */
    memset(L->ye, 0, (size_t)M * d * sizeof(float));
    moe_ref_mm(hp16, L->wdown, L->ye, L->amax, L->tiles, M, d, I, 0u, MOE_REF_NO_SLOT, pm); /* :878 */
    free(g);
    free(hp);
    if (L->hp16 == NULL) free(hp16);
    free(pm);

    float *sh = NULL;
    if (S != 0u) {
        /* The reference takes the shared expert's gate/up pre-activations from the
         * upstream dense product (src/qwen.c:845, columns experts+128...), which is
         * the same fp16 x fp16 -> fp32 arithmetic as the grouped product; then
         * src/qwen.c:879-886: SwiGLU, absmax + cast, dense product with the down
         * weights. */
        uint32_t Rp = (R + 127u) / 128u * 128u;
        uint32_t *t0 = (uint32_t *)calloc(Rp / 128u, sizeof(uint32_t));
        uint16_t *xpad = (uint16_t *)calloc((size_t)Rp * d, sizeof(uint16_t));
        memcpy(xpad, L->x16, (size_t)R * d * sizeof(uint16_t));
        uint8_t *rm = (uint8_t *)calloc(Rp, 1);
        for (uint32_t r = 0; r < R; r += 1) rm[r] = L->row_mask == NULL || L->row_mask[r];
        float *gs = (float *)calloc((size_t)Rp * 2u * S, sizeof(float));
        float *hs = (float *)calloc((size_t)Rp * S, sizeof(float));
        uint16_t *hs16 = (uint16_t *)malloc((size_t)Rp * S * sizeof(uint16_t));
        sh = (float *)calloc((size_t)Rp * d, sizeof(float));
        moe_ref_mm(xpad, L->wsgu, gs, L->amax, t0, Rp, 2u * S, d, MOE_REF_NO_SLOT, MOE_REF_NO_SLOT, rm);
        moe_ref_swiglu(gs, hs, Rp, S, 2u * S, 0u, S);
        moe_ref_absmax(hs, (uint64_t)Rp * S, L->amax, 1u);
        moe_ref_cast_f16(hs, hs16, (uint64_t)Rp * S, L->amax, 1u);
        moe_ref_mm(hs16, L->wsdown, sh, L->amax, t0, Rp, d, S, 1u, MOE_REF_NO_SLOT, rm);
        free(t0);
        free(xpad);
        free(rm);
        free(gs);
        free(hs);
        free(hs16);
    }
    moe_ref_combine(L->wt, L->slot, L->ye, L->proj, sh, L->inj, L->h, R, d, K, L->pstride, E,
                    L->hc, 0u, L->hc); /* :887-906 */
    free(sh);
    return 0;
}
