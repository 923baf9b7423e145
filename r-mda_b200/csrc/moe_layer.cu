// The whole MoE layer in one call: the kernel order of mda_qwen_route_rec
// (src/qwen.c:788-836) followed by mda_qwen_moe_rec from the first grouped
// product on (src/qwen.c:847-906).
//
// Fused mode (default) differs from the reference's sequence in data movement
// only: SwiGLU and the fp16 store are the epilogue of the gate_up product (so the
// fp32 g and hp tensors are never written), the intermediate keeps scale 1
// instead of the global absmax power of two, expert outputs stay fp16 unless
// MOE_LAYER_YE_F32 is set, and the padding rows of xp are not zero-filled (a
// padding row only ever feeds padding rows).  MOE_LAYER_UNFUSED runs the
// reference's sequence step by step.
#include "moe_common.cuh"

extern "C" uint32_t moe_cuda_moe_rows(uint32_t rows, uint32_t topk, uint32_t experts) {
    // mda_qwen_moe_rows, src/qwen.c:68-70
    uint64_t n = (uint64_t)rows * topk + (uint64_t)experts * (MOE_TILE - 1u);
    return (uint32_t)((n + MOE_TILE - 1u) / MOE_TILE * MOE_TILE);
}

namespace {

struct Carver {
    uint8_t *base;
    size_t at;
    void *take(size_t bytes) {
        size_t a = (at + 1023) & ~(size_t)1023;  // 1 KB alignment: TMA bases need 16 B, keep tiles apart
        at = a + bytes;
        return base == NULL ? NULL : base + a;
    }
};

struct LayerBufs {
    uint32_t *idx, *slot, *count, *off, *fill, *tiles, *amax, *tiles0, *n_chunks, *src_row;
    void *chunks;
    float *wt;
    __half *xp, *hp16, *hs16;
    void *ye;
    float *g, *hp, *sh, *gs, *hs;
};

void carve(Carver &cv, LayerBufs &b, const moe_cuda_layer_t *L, uint32_t M, uint32_t Rp, bool unfused, bool ye32) {
    size_t R = L->rows, K = L->topk, E = L->experts, d = L->d, I = L->inter, S = L->shared;
    b.idx = (uint32_t *)cv.take(R * K * 4);
    b.slot = (uint32_t *)cv.take(R * K * 4);
    b.wt = (float *)cv.take(R * K * 4);
    b.count = (uint32_t *)cv.take(E * 4);
    b.off = (uint32_t *)cv.take(E * 4);
    b.fill = (uint32_t *)cv.take(E * 4);
    b.tiles = (uint32_t *)cv.take((size_t)(M / MOE_TILE) * 4);
    b.amax = (uint32_t *)cv.take(256 * 4);  // MDA_QWEN_MAX_SLOTS, src/qwen.h:13
    b.tiles0 = (uint32_t *)cv.take((size_t)(Rp / MOE_TILE) * 4);
    b.n_chunks = (uint32_t *)cv.take(64);
    b.src_row = (uint32_t *)cv.take((size_t)M * 4);
    b.chunks = cv.take((R * K / 256 + E + 1) * 16);
    b.xp = (__half *)cv.take((size_t)M * d * 2);
    b.hp16 = (__half *)cv.take((size_t)M * I * 2);
    b.ye = cv.take((size_t)M * d * ((unfused || ye32) ? 4 : 2));
    b.g = unfused ? (float *)cv.take((size_t)M * 2 * I * 4) : NULL;
    b.hp = unfused ? (float *)cv.take((size_t)M * I * 4) : NULL;
    b.hs16 = S != 0 ? (__half *)cv.take((size_t)Rp * S * 2) : NULL;
    b.sh = S != 0 ? (float *)cv.take((size_t)Rp * d * 4) : NULL;
    b.gs = (S != 0 && unfused) ? (float *)cv.take((size_t)Rp * 2 * S * 4) : NULL;
    b.hs = (S != 0 && unfused) ? (float *)cv.take((size_t)Rp * S * 4) : NULL;
}

void mark(moe_cuda_ctx *c, int i) {
    if (c->prof && c->ev_made && c->status == MOE_OK) cudaEventRecord(c->ev[i], c->stream);
}

}  // namespace

extern "C" void moe_cuda_layer(moe_cuda_ctx_t *c, const moe_cuda_layer_t *L) {
    if (!MOE_LIVE(c)) return;
    MOE_REQUIRE(c, L != NULL, "layer: null descriptor");
    MOE_REQUIRE(c, L->proj != NULL && L->x16 != NULL && L->wgu != NULL && L->wdown != NULL, "layer: null input");
    MOE_REQUIRE(c, L->h != NULL || L->y16 != NULL, "layer: no output");
    MOE_REQUIRE(c, L->experts >= 1 && L->experts <= MOE_MAX_EXPERTS, "layer: experts %u outside 1..512", L->experts);
    MOE_REQUIRE(c, L->topk >= 1 && L->topk <= MOE_MAX_TOPK && L->topk <= L->experts, "layer: topk %u", L->topk);
    MOE_REQUIRE(c, L->d % 8 == 0 && L->d >= 8, "layer: d %u not a multiple of 8", L->d);
    MOE_REQUIRE(c, L->inter % 64 == 0 && L->inter >= 64, "layer: inter %u not a multiple of 64", L->inter);
    MOE_REQUIRE(c, L->shared % 64 == 0, "layer: shared %u not a multiple of 64", L->shared);
    MOE_REQUIRE(c, L->shared == 0 || (L->wsgu != NULL && L->wsdown != NULL), "layer: shared expert without weights");
    MOE_REQUIRE(c, L->hc >= 1, "layer: hc 0");
    if (L->rows == 0) return;
    const uint32_t R = L->rows, K = L->topk, E = L->experts, d = L->d, I = L->inter, S = L->shared;
    const uint32_t M = moe_cuda_moe_rows(R, K, E);
    const uint32_t Rp = (R + MOE_TILE - 1u) / MOE_TILE * MOE_TILE;
    // The fused SwiGLU epilogue pairs 128 gate columns with 128 up columns.
    const bool unfused = (L->flags & MOE_LAYER_UNFUSED) != 0 || I % 128u != 0 || (S != 0 && S % 128u != 0);
    const bool ye32 = unfused || (L->flags & MOE_LAYER_YE_F32) != 0;
    // default: weight-stationary products over per-expert chunks; MOE_LAYER_TILED: the reference's 128-row tiles
    const bool chunked = !unfused && ((L->flags & MOE_LAYER_TILED) == 0 || (L->flags & MOE_LAYER_CHUNKED) != 0) && d % 128u == 0;
    // tiled: no permuted copy of the activations unless MOE_LAYER_MATERIALIZE_XP asks for the reference's xp
    const bool gather = !unfused && !chunked && (L->flags & MOE_LAYER_MATERIALIZE_XP) == 0;

    Carver measure = {NULL, 0};
    LayerBufs b;
    carve(measure, b, L, M, Rp, unfused, ye32);
    uint8_t *base = (uint8_t *)moe_scratch(c, MOE_SCR_LAYER, measure.at + 1024);
    if (base == NULL) return;
    Carver cv = {base, 0};
    carve(cv, b, L, M, Rp, unfused, ye32);
    uint32_t *idx = L->idx != NULL ? L->idx : b.idx;
    uint32_t *slot = L->slot != NULL ? L->slot : b.slot;
    uint32_t *count = L->count != NULL ? L->count : b.count;
    uint32_t *off = L->off != NULL ? L->off : b.off;
    uint32_t *tiles = L->tiles != NULL ? L->tiles : b.tiles;
    float *wt = L->wt != NULL ? L->wt : b.wt;

    mark(c, 0);
    // src/qwen.c:793-798
    if (unfused) {
        moe_cuda_fill(c, tiles, (size_t)(M / MOE_TILE) * 4, 0xffffffffu);
        moe_cuda_fill(c, count, (size_t)E * 4, 0);
        moe_cuda_fill(c, b.fill, (size_t)E * 4, 0);
        moe_cuda_fill(c, b.xp, (size_t)M * d * 2, 0);
        moe_cuda_fill(c, b.amax, 256 * 4, 0);  // mda_qwen_slots_begin, src/qwen.c:500-503
    }
    if (unfused) {
        moe_launch_route(c, L->proj, idx, wt, count, R, E, K, L->pstride);  // :799-811
        mark(c, 1);
        moe_launch_scan(c, count, off, tiles, E, MOE_TILE);  // :812-821
        mark(c, 2);
        moe_launch_scatter(c, idx, off, b.fill, L->x16, b.xp, slot, R, K, d / 8u, E);  // :822-835
    } else {
        // Same results with fewer launches and no contended atomics: the router leaves a
        // per-8-row expert table, whose column scan gives both count[] and the bases of
        // the stable ranking.
        uint32_t *hist = (uint32_t *)moe_scratch(c, MOE_SCR_SCATTER, (size_t)((R + 7u) / 8u) * E * 4);
        if (hist == NULL) return;
        // the router also fills the tile schedule and (gather mode) the source-row table with ~0
        moe_launch_route_hist(c, L->proj, idx, wt, hist, R, E, K, L->pstride, tiles, M / MOE_TILE,
                              gather ? b.src_row : NULL, gather ? M : 0u);
        mark(c, 1);
        // + the scan and (weight-stationary products) the chunk list, in its last block
        moe_launch_colscan_counts(c, hist, count, R, E, off, tiles, MOE_TILE, chunked ? b.chunks : NULL, b.n_chunks,
                                  R * K / 256u + E + 1u);
        mark(c, 2);
        moe_launch_place(c, idx, off, hist, L->x16, b.xp, slot, R, K, d / 8u, E, NULL, 0, gather ? b.src_row : NULL);
    }
    mark(c, 3);
    if (chunked) {
        // weight-stationary products over per-expert token chunks (MMA width rounded to 16, not 128)
        const uint32_t max_chunks = R * K / 256u + E + 1u;
        int pair1 = ((L->flags & MOE_LAYER_NO_PAIR) == 0 && I % 128u == 0) ? 2 : 1;
        int pair2 = ((L->flags & MOE_LAYER_NO_PAIR) == 0 && d % 256u == 0) ? 2 : 1;
        moe_launch_mm_ws(c, MOE_MM_SWIGLU_F16, pair1, b.xp, M, L->wgu, E, b.hp16, I, b.chunks, b.n_chunks, max_chunks,
                           2u * I, d);  // :847-877 in one kernel
        mark(c, 4);
        moe_launch_mm_ws(c, ye32 ? MOE_MM_F32 : MOE_MM_F16, pair2, b.hp16, M, L->wdown, E, b.ye, d, b.chunks, b.n_chunks,
                           max_chunks, d, I);  // :878
        mark(c, 5);
    }
    if (!unfused && !chunked) {
        if (gather) {  // the gate_up product fetches the rows of x16 itself; xp is never written
            moe_launch_mm(c, MOE_MM_SWIGLU_F16, L->x16, L->wgu, b.hp16, NULL, tiles, M, 2u * I, d, MDA_PC_NO_SLOT,
                          MDA_PC_NO_SLOT, E, R, true, b.src_row);  // :822-877 in one kernel
        } else {
            moe_launch_mm(c, MOE_MM_SWIGLU_F16, b.xp, L->wgu, b.hp16, NULL, tiles, M, 2u * I, d, MDA_PC_NO_SLOT,
                          MDA_PC_NO_SLOT, E, M, true);  // :847-877 in one kernel
        }
        mark(c, 4);
        moe_launch_mm(c, ye32 ? MOE_MM_F32 : MOE_MM_F16, b.hp16, L->wdown, b.ye, NULL, tiles, M, d, I, MDA_PC_NO_SLOT,
                      MDA_PC_NO_SLOT, E, M, true);  // :878
        mark(c, 5);
    }
    if (!unfused) {
        if (S != 0) {
            moe_cuda_fill(c, b.tiles0, (size_t)(Rp / MOE_TILE) * 4, 0);
            moe_launch_mm(c, MOE_MM_SWIGLU_F16, L->x16, L->wsgu, b.hs16, NULL, b.tiles0, Rp, 2u * S, d, MDA_PC_NO_SLOT,
                          MDA_PC_NO_SLOT, 1, R);
            moe_launch_mm(c, MOE_MM_F32, b.hs16, L->wsdown, b.sh, NULL, b.tiles0, Rp, d, S, MDA_PC_NO_SLOT,
                          MDA_PC_NO_SLOT, 1, Rp);  // :879-886
        }
    } else {
        // Row tiles the product skips keep whatever g held before (in the reference:
        // the previous call's values); zero them so the absmax below is a function
        // of this call's inputs only.
        moe_cuda_fill(c, b.g, (size_t)M * 2u * I * 4, 0);
        moe_launch_mm(c, MOE_MM_F32, b.xp, L->wgu, b.g, b.amax, tiles, M, 2u * I, d, MDA_PC_NO_SLOT, MDA_PC_NO_SLOT, E,
                      M);  // :847
        struct mda_pc_qwen_elem_t pe = {M, I, 2u * I, 0u, I, 0u, 1.0f};
        moe_cuda_swiglu(c, b.g, b.hp, pe);  // :848-857
        struct mda_pc_absmax_t pa = {M * I, 0u};
        moe_cuda_absmax(c, b.hp, b.amax, pa);  // :858-867
        struct mda_pc_cast_t pcst = {M * I, 0u};
        moe_cuda_cast_f16(c, b.hp, b.hp16, b.amax, pcst);  // :868-877
        mark(c, 4);
        moe_launch_mm(c, MOE_MM_F32, b.hp16, L->wdown, b.ye, b.amax, tiles, M, d, I, 0u, MDA_PC_NO_SLOT, E, M);  // :878
        mark(c, 5);
        if (S != 0) {
            moe_cuda_fill(c, b.tiles0, (size_t)(Rp / MOE_TILE) * 4, 0);
            moe_launch_mm(c, MOE_MM_F32, L->x16, L->wsgu, b.gs, b.amax, b.tiles0, Rp, 2u * S, d, MDA_PC_NO_SLOT,
                          MDA_PC_NO_SLOT, 1, R);
            struct mda_pc_qwen_elem_t ps = {Rp, S, 2u * S, 0u, S, 0u, 1.0f};
            moe_cuda_swiglu(c, b.gs, b.hs, ps);
            struct mda_pc_absmax_t pas = {Rp * S, 1u};
            moe_cuda_absmax(c, b.hs, b.amax, pas);
            struct mda_pc_cast_t pcs = {Rp * S, 1u};
            moe_cuda_cast_f16(c, b.hs, b.hs16, b.amax, pcs);
            moe_launch_mm(c, MOE_MM_F32, b.hs16, L->wsdown, b.sh, b.amax, b.tiles0, Rp, d, S, 1u, MDA_PC_NO_SLOT, 1, Rp);
        }
    }
    mark(c, 6);
    moe_combine_args a = {};
    a.wt = wt;
    a.slot = slot;
    a.y = b.ye;
    a.proj = L->proj;
    a.sh = S != 0 ? b.sh : NULL;
    a.inj = L->inj;
    a.h = L->h;
    a.x16 = (const __half *)L->x16;
    a.y16 = (__half *)L->y16;
    a.eps = L->eps;
    a.rows = R;
    a.d = d;
    a.topk = K;
    a.pstride = L->pstride;
    a.sg_off = E;
    a.inj_stride = L->inj_stride;
    a.inj_off = L->inj_off;
    a.hc = L->hc;
    a.y_is_f16 = !ye32;
    moe_launch_combine(c, a);  // :887-906
    mark(c, 7);
    if (c->prof && c->ev_made && c->status == MOE_OK) {
        c->ev_valid = true;
        c->ev_slices = 1;
    }
}
