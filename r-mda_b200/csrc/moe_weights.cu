// Expert weights: re-tiling for HBM-friendly streaming.
//
// The reference keeps an expert's weights row-major [n x k] (HF layout,
// src/qwen.c:102-103) and converts them on the device right after the upload
// (bf16 -> fp16 in place, src/qwen.c:380-394, shader/qwen_bf16.comp).  A TMA box of
// 128 rows x 64 columns of that layout touches 128 separate 128-byte pieces 2k
// bytes apart -- a power-of-two stride that DRAM banks serve poorly when the
// weights are streamed once per layer.  moe_cuda_tile_weights rewrites them, in
// the same pass that the reference spends on the conversion, as contiguous
// 16 KB blocks: block (row / 128) * ceil(k / 64) + (col / 64) holds rows
// [128*(row/128), +128) x columns [64*(col/64), +64), row-major, zero-padded in k.
#include "moe_common.cuh"

__global__ void moe_tile_weights_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst, uint64_t rows,
                                        uint32_t k, uint32_t kblocks) {
    // one thread per 16-byte piece (8 halves) of the tiled output
    uint64_t total = rows * kblocks * 8u;
    uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        uint32_t piece = (uint32_t)(i & 7u);         // 16-byte piece inside the 128-byte row of the block
        uint64_t rb = i >> 3;                        // (block, row in block)
        uint32_t r = (uint32_t)(rb & 127u);
        uint64_t blk = rb >> 7;
        uint32_t kb = (uint32_t)(blk % kblocks);
        uint64_t r128 = blk / kblocks;
        uint64_t row = r128 * 128u + r;
        uint32_t col = kb * 64u + piece * 8u;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (col < k) v = __ldg(src + (row * k + col) / 8u);  // k % 8 == 0
        dst[i] = v;
    }
}

extern "C" size_t moe_cuda_tiled_bytes(uint32_t experts, uint32_t n, uint32_t k) {
    return (size_t)experts * n * ((k + 63u) / 64u) * 64u * 2u;
}

extern "C" void moe_cuda_tile_weights(moe_cuda_ctx_t *c, const void *src, void *dst, uint32_t experts, uint32_t n,
                                      uint32_t k) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, src != NULL && dst != NULL && src != dst, "tile_weights: null or aliased buffers");
    MOE_REQUIRE(c, n % 128u == 0 && k % 8u == 0 && experts >= 1, "tile_weights: n %u %% 128 or k %u %% 8", n, k);
    MOE_REQUIRE(c, ((uintptr_t)src & 15) == 0 && ((uintptr_t)dst & 15) == 0, "tile_weights: not 16-byte aligned");
    uint64_t rows = (uint64_t)experts * n;
    uint32_t kblocks = (k + 63u) / 64u;
    uint32_t blocks = (uint32_t)c->sm_count * 16u;
    moe_tile_weights_kernel<<<blocks, 256, 0, c->stream>>>((const uint4 *)src, (uint4 *)dst, rows, k, kblocks);
    MOE_LAUNCHED(c);
}
