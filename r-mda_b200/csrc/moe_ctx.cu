// Context, status and buffer calls of libmoe_cuda: the part of the reference's
// Vulkan harness (src/vkc.c) that the MoE call sites use, restated over the CUDA
// runtime.  One context = one device + one in-order stream + a sticky status.
#include <stdlib.h>
#include <string.h>

#include "moe_common.cuh"

void moe_fail(moe_cuda_ctx *c, int code, const char *fmt, ...) {
    if (c == NULL || c->status != MOE_OK) return;  // first failure wins (src/vkc.c:15-20)
    c->status = code;
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(c->err, sizeof(c->err), fmt, ap);
    va_end(ap);
    fprintf(stderr, "moe_cuda: %s\n", c->err);
}

// Folds refusals recorded by kernels into the sticky status.  Returns true if
// the context is still live.
bool moe_poll_device_status(moe_cuda_ctx *c) {
    if (c == NULL) return false;
    if (c->status == MOE_OK && c->dev_status_host != NULL) {
        uint32_t w = *(volatile uint32_t *)c->dev_status_host;
        if (w != 0) {
            int code = (int)(w & 0xffu);
            if (code == MOE_ERR_ROUTE) {
                moe_fail(c, code, "route: row %u has fewer selectable logits than topk", w >> 8);
            } else if (code == MOE_ERR_TIMEOUT) {
                moe_fail(c, code, "device wait gave up (site %u)", w >> 8);
            } else {
                moe_fail(c, code, "device reported status 0x%x", w);
            }
        }
    }
    return c->status == MOE_OK;
}

extern "C" moe_cuda_ctx_t *moe_cuda_create(int device, void *stream) {
    moe_cuda_ctx *c = (moe_cuda_ctx *)calloc(1, sizeof(moe_cuda_ctx));
    if (c == NULL) return NULL;
    c->device = device;
    c->status = MOE_OK;
    c->wait_ns = 2000000000ull;
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) {
        moe_fail(c, MOE_ERR_CUDA, "no usable CUDA device %d: %s", device, cudaGetErrorString(e));
        return c;
    }
    cudaDeviceProp prop;
    e = cudaGetDeviceProperties(&prop, device);
    if (e != cudaSuccess) {
        moe_fail(c, MOE_ERR_CUDA, "device properties: %s", cudaGetErrorString(e));
        return c;
    }
    if (prop.major != 10) {  // the kernels are built for sm_100a only (cf. src/vkc.c:49-64 feature checks)
        moe_fail(c, MOE_ERR_UNSUPPORTED, "device %d is sm_%d%d, need sm_100", device, prop.major, prop.minor);
        return c;
    }
    c->sm_count = prop.multiProcessorCount;
    if (stream != NULL) {
        c->stream = (cudaStream_t)stream;
    } else {
        e = cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking);
        if (e != cudaSuccess) {
            moe_fail(c, MOE_ERR_CUDA, "stream: %s", cudaGetErrorString(e));
            return c;
        }
        c->own_stream = true;
    }
    e = cudaHostAlloc((void **)&c->dev_status_host, 64, cudaHostAllocMapped);
    if (e == cudaSuccess) {
        memset(c->dev_status_host, 0, 64);
        e = cudaHostGetDevicePointer((void **)&c->dev_status_dev, c->dev_status_host, 0);
    }
    if (e != cudaSuccess) {
        moe_fail(c, MOE_ERR_CUDA, "status word: %s", cudaGetErrorString(e));
        return c;
    }
    cudaDriverEntryPointQueryResult q;
    e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &c->encode_tiled, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || c->encode_tiled == NULL) {
        moe_fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled not available from this driver");
        return c;
    }
    return c;
}

extern "C" void moe_cuda_destroy(moe_cuda_ctx_t *c) {
    if (c == NULL) return;
    moe_ep_teardown(c);
    if (c->stream != NULL) cudaStreamSynchronize(c->stream);
    for (int i = 0; i < MOE_SCR_COUNT; i += 1) {
        if (c->scratch[i] != NULL) cudaFree(c->scratch[i]);
    }
    if (c->ev_made) {
        for (int i = 0; i <= MOE_PROF_STAGES; i += 1) cudaEventDestroy(c->ev[i]);
    }
    for (int m = 0; m < c->ev_mb_made; m += 1) {
        for (int i = 0; i <= MOE_PROF_STAGES; i += 1) cudaEventDestroy(c->ev_mb[m][i]);
    }
    if (c->ticket != NULL) cudaFree(c->ticket);
    if (c->dev_status_host != NULL) cudaFreeHost(c->dev_status_host);
    if (c->own_stream) cudaStreamDestroy(c->stream);
    free(c);
}

extern "C" int moe_cuda_status(moe_cuda_ctx_t *c) {
    if (c == NULL) return MOE_ERR_ARG;
    moe_poll_device_status(c);
    return c->status;
}

extern "C" const char *moe_cuda_last_error(moe_cuda_ctx_t *c) {
    return c == NULL ? "no context" : c->err;
}

extern "C" void *moe_cuda_stream(moe_cuda_ctx_t *c) { return c == NULL ? NULL : (void *)c->stream; }

extern "C" void moe_cuda_fail_alloc_after(moe_cuda_ctx_t *c, int n) {
    if (c != NULL) c->fail_alloc_countdown = n;
}

extern "C" void moe_cuda_set_wait_ns(moe_cuda_ctx_t *c, uint64_t ns) {
    if (c != NULL && ns != 0) c->wait_ns = ns;
}

extern "C" uint64_t moe_cuda_launches(moe_cuda_ctx_t *c) { return c == NULL ? 0 : c->launches; }

static bool moe_alloc_refused(moe_cuda_ctx *c) {
    if (c->fail_alloc_countdown > 0) {
        c->fail_alloc_countdown -= 1;
        if (c->fail_alloc_countdown == 0) return true;
    }
    return false;
}

extern "C" void *moe_cuda_alloc(moe_cuda_ctx_t *c, size_t bytes) {
    if (!MOE_LIVE(c)) return NULL;
    void *p = NULL;
    if (moe_alloc_refused(c)) {
        moe_fail(c, MOE_ERR_NOMEM, "alloc of %zu bytes refused (injected)", bytes);
        return NULL;
    }
    cudaError_t e = cudaMalloc(&p, bytes == 0 ? 1 : bytes);
    if (e != cudaSuccess) {
        moe_fail(c, MOE_ERR_NOMEM, "alloc of %zu bytes: %s", bytes, cudaGetErrorString(e));
        return NULL;
    }
    return p;
}

extern "C" void *moe_cuda_alloc_pinned(moe_cuda_ctx_t *c, size_t bytes) {
    if (!MOE_LIVE(c)) return NULL;
    void *p = NULL;
    if (moe_alloc_refused(c)) {
        moe_fail(c, MOE_ERR_NOMEM, "pinned alloc of %zu bytes refused (injected)", bytes);
        return NULL;
    }
    cudaError_t e = cudaHostAlloc(&p, bytes == 0 ? 1 : bytes, cudaHostAllocDefault);
    if (e != cudaSuccess) {
        moe_fail(c, MOE_ERR_NOMEM, "pinned alloc of %zu bytes: %s", bytes, cudaGetErrorString(e));
        return NULL;
    }
    return p;
}

extern "C" void moe_cuda_free(moe_cuda_ctx_t *c, void *p) {
    if (c == NULL || p == NULL) return;
    cudaStreamSynchronize(c->stream);
    cudaFree(p);
}

extern "C" void moe_cuda_free_pinned(moe_cuda_ctx_t *c, void *p) {
    if (c == NULL || p == NULL) return;
    cudaStreamSynchronize(c->stream);
    cudaFreeHost(p);
}

void *moe_scratch(moe_cuda_ctx *c, int area, size_t bytes) {
    if (!MOE_LIVE(c)) return NULL;
    if (c->scratch_bytes[area] >= bytes && c->scratch[area] != NULL) return c->scratch[area];
    if (c->scratch[area] != NULL) {
        cudaStreamSynchronize(c->stream);
        cudaFree(c->scratch[area]);
        c->scratch[area] = NULL;
        c->scratch_bytes[area] = 0;
    }
    size_t want = (bytes + 0xfffffu) & ~(size_t)0xfffffu;
    void *p = moe_cuda_alloc(c, want);
    if (p == NULL) return NULL;
    c->scratch[area] = p;
    c->scratch_bytes[area] = want;
    return p;
}

__global__ void moe_fill_kernel(uint4 *dst4, size_t n16, uint32_t *tail, uint32_t ntail, uint32_t word) {
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    size_t stride = (size_t)gridDim.x * blockDim.x;
    uint4 v = make_uint4(word, word, word, word);
    for (; i < n16; i += stride) dst4[i] = v;
    if (blockIdx.x == 0 && threadIdx.x < ntail) tail[threadIdx.x] = word;
}

// mda_vkc_fill (src/vkc.c:803-815): whole 32-bit words.
extern "C" void moe_cuda_fill(moe_cuda_ctx_t *c, void *dst, size_t bytes, uint32_t word) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, dst != NULL && bytes % 4 == 0 && ((uintptr_t)dst & 3) == 0, "fill: dst/bytes not word aligned");
    if (bytes == 0) return;
    uint32_t b = word & 0xffu;
    if (((word >> 8) & 0xffu) == b && ((word >> 16) & 0xffu) == b && (word >> 24) == b) {
        MOE_CUDA_TRY(c, cudaMemsetAsync(dst, (int)b, bytes, c->stream));
        return;
    }
    uintptr_t a = (uintptr_t)dst;
    size_t head = ((16 - (a & 15)) & 15);
    if (head > bytes) head = bytes;
    if (head != 0) {  // leading words up to 16-byte alignment
        moe_fill_kernel<<<1, 32, 0, c->stream>>>(NULL, 0, (uint32_t *)dst, (uint32_t)(head / 4), word);
        MOE_LAUNCHED(c);
    }
    size_t rest = bytes - head;
    size_t n16 = rest / 16;
    uint32_t ntail = (uint32_t)((rest % 16) / 4);
    uint8_t *body = (uint8_t *)dst + head;
    if (n16 != 0 || ntail != 0) {
        size_t blocks = (n16 + 255) / 256;
        if (blocks > (size_t)c->sm_count * 8) blocks = (size_t)c->sm_count * 8;
        if (blocks == 0) blocks = 1;
        moe_fill_kernel<<<(unsigned)blocks, 256, 0, c->stream>>>((uint4 *)body, n16, (uint32_t *)(body + n16 * 16), ntail, word);
        MOE_LAUNCHED(c);
    }
}

extern "C" void moe_cuda_copy(moe_cuda_ctx_t *c, void *dst, const void *src, size_t bytes) {
    if (!MOE_LIVE(c)) return;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, c->stream));
}

extern "C" void moe_cuda_write(moe_cuda_ctx_t *c, void *dst, const void *host_src, size_t bytes) {
    if (!MOE_LIVE(c)) return;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(dst, host_src, bytes, cudaMemcpyHostToDevice, c->stream));
}

extern "C" void moe_cuda_read(moe_cuda_ctx_t *c, void *host_dst, const void *src, size_t bytes) {
    if (!MOE_LIVE(c)) return;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
    MOE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
    moe_poll_device_status(c);
}

// Enqueued device-to-host copy; the data is on the host after the next moe_cuda_flush.
extern "C" void moe_cuda_read_async(moe_cuda_ctx_t *c, void *host_dst, const void *src, size_t bytes) {
    if (!MOE_LIVE(c)) return;
    MOE_CUDA_TRY(c, cudaMemcpyAsync(host_dst, src, bytes, cudaMemcpyDeviceToHost, c->stream));
}

extern "C" void moe_cuda_flush(moe_cuda_ctx_t *c) {
    if (c == NULL || c->stream == NULL) return;
    if (c->status == MOE_OK) {
        MOE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));
        moe_poll_device_status(c);
    }
}

extern "C" void moe_cuda_prof(moe_cuda_ctx_t *c, int on) {
    if (!MOE_LIVE(c)) return;
    if (on && !c->ev_made) {
        for (int i = 0; i <= MOE_PROF_STAGES; i += 1) MOE_CUDA_TRY(c, cudaEventCreate(&c->ev[i]));
        c->ev_made = true;
    }
    c->prof = on != 0;
    c->ev_valid = false;
}

extern "C" void moe_cuda_prof_read(moe_cuda_ctx_t *c, float ms[MOE_PROF_STAGES]) {
    for (int i = 0; i < MOE_PROF_STAGES; i += 1) ms[i] = 0.0f;
    if (!MOE_LIVE(c) || !c->ev_valid) return;
    MOE_CUDA_TRY(c, cudaStreamSynchronize(c->stream));  // the slices' streams have joined the context's stream
    for (int m = 0; m < (c->ev_slices > 1 ? c->ev_slices : 1); m += 1) {
        cudaEvent_t *ev = m == 0 ? c->ev : c->ev_mb[m - 1];
        for (int i = 0; i < MOE_PROF_STAGES; i += 1) {
            float t = 0.0f;
            MOE_CUDA_TRY(c, cudaEventElapsedTime(&t, ev[i], ev[i + 1]));
            ms[i] += t;
        }
    }
}

// 2-D fp16 tensor map [rows x cols], row-major, swizzle = the box's row width (128 or 64 bytes), zero fill
// outside the tensor; never multicast.  Cached per (pointer, shape, box).
typedef CUresult (*moe_encode_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

const CUtensorMap *moe_tmap_2d_f16(moe_cuda_ctx *c, const void *ptr, uint64_t rows, uint64_t cols,
                                   uint32_t box_rows, uint32_t box_cols) {
    if (!MOE_LIVE(c)) return NULL;
    for (int i = 0; i < c->n_tmaps; i += 1) {
        moe_tmap_entry *t = &c->tmaps[i];
        if (t->kind == 0 && t->ptr == ptr && t->rows == rows && t->cols == cols && t->box_rows == box_rows && t->box_cols == box_cols) {
            return &t->map;
        }
    }
    if (((uintptr_t)ptr & 15) != 0 || (cols * 2) % 16 != 0 || (box_cols * 2 != 128 && box_cols * 2 != 64) || box_rows > 256 || rows == 0) {
        moe_fail(c, MOE_ERR_ARG, "tensor map: base %p rows %llu cols %llu not TMA-addressable", ptr,
                 (unsigned long long)rows, (unsigned long long)cols);
        return NULL;
    }
    int at = c->n_tmaps < 128 ? c->n_tmaps++ : (c->next_tmap++ & 127);
    moe_tmap_entry *t = &c->tmaps[at];
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * 2};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = ((moe_encode_fn)c->encode_tiled)(&t->map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)ptr, dims,
                                                  strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                  box_cols * 2 == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        moe_fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled failed: %d", (int)r);
        c->n_tmaps = at < c->n_tmaps ? c->n_tmaps : at;
        t->ptr = NULL;
        return NULL;
    }
    t->ptr = ptr;
    t->rows = rows;
    t->cols = cols;
    t->box_rows = box_rows;
    t->box_cols = box_cols;
    t->kind = 0;
    return &t->map;
}

const CUtensorMap *moe_tmap_gate_up_f16(moe_cuda_ctx *c, const void *ptr, uint32_t experts, uint32_t inter, uint32_t k) {
    if (!MOE_LIVE(c)) return NULL;
    for (int i = 0; i < c->n_tmaps; i += 1) {
        moe_tmap_entry *t = &c->tmaps[i];
        if (t->kind == 1 && t->ptr == ptr && t->rows == experts && t->cols == k && t->box_rows == inter) return &t->map;
    }
    if (((uintptr_t)ptr & 15) != 0 || k % 8u != 0 || inter % 64u != 0 || experts == 0) {
        moe_fail(c, MOE_ERR_ARG, "tensor map: gate/up bank %p experts %u inter %u k %u not TMA-addressable", ptr, experts, inter, k);
        return NULL;
    }
    int at = c->n_tmaps < 128 ? c->n_tmaps++ : (c->next_tmap++ & 127);
    moe_tmap_entry *t = &c->tmaps[at];
    cuuint64_t dims[4] = {k, 2, inter, experts};
    cuuint64_t strides[3] = {(cuuint64_t)inter * k * 2, (cuuint64_t)k * 2, (cuuint64_t)2 * inter * k * 2};
    cuuint32_t box[4] = {64, 2, 64, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = ((moe_encode_fn)c->encode_tiled)(&t->map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, (void *)ptr, dims, strides, box,
                                                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        moe_fail(c, MOE_ERR_CUDA, "cuTensorMapEncodeTiled (gate/up bank) failed: %d", (int)r);
        t->ptr = NULL;
        return NULL;
    }
    t->ptr = ptr;
    t->rows = experts;
    t->cols = k;
    t->box_rows = inter;
    t->box_cols = 64;
    t->kind = 1;
    return &t->map;
}
