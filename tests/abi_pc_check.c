/* Compile-time proof that libmoe_cuda's header and the reference share the
 * push-constant structs of the MoE path: the reference's own src/pc.h is
 * included first (unmodified), then include/moe_cuda.h, whose copies are
 * skipped by the MDA_PC_H guard; the assertions pin the sizes and field offsets
 * of src/pc.h:369-404 that the kernels were written against.  Built by
 * tests/test_abi.py (compile only) with -I <reference>/src when the reference tree is mounted. */
#include <stddef.h>

#include "pc.h"
#include "moe_cuda.h"

#define SAME(type, field, off) _Static_assert(offsetof(struct type, field) == (off), #type "." #field)

_Static_assert(sizeof(struct mda_pc_moe_route_t) == 16, "route");
SAME(mda_pc_moe_route_t, rows, 0);
SAME(mda_pc_moe_route_t, experts, 4);
SAME(mda_pc_moe_route_t, topk, 8);
SAME(mda_pc_moe_route_t, stride, 12);
_Static_assert(sizeof(struct mda_pc_moe_scan_t) == 8, "scan");
SAME(mda_pc_moe_scan_t, experts, 0);
SAME(mda_pc_moe_scan_t, tile, 4);
_Static_assert(sizeof(struct mda_pc_moe_scatter_t) == 12, "scatter");
SAME(mda_pc_moe_scatter_t, rows, 0);
SAME(mda_pc_moe_scatter_t, topk, 4);
SAME(mda_pc_moe_scatter_t, d8, 8);
_Static_assert(sizeof(struct mda_pc_moe_mm_t) == 20, "mm");
SAME(mda_pc_moe_mm_t, m, 0);
SAME(mda_pc_moe_mm_t, n, 4);
SAME(mda_pc_moe_mm_t, k, 8);
SAME(mda_pc_moe_mm_t, sa, 12);
SAME(mda_pc_moe_mm_t, sb, 16);
_Static_assert(sizeof(struct mda_pc_moe_combine_t) == 32, "combine");
SAME(mda_pc_moe_combine_t, rows, 0);
SAME(mda_pc_moe_combine_t, d, 4);
SAME(mda_pc_moe_combine_t, topk, 8);
SAME(mda_pc_moe_combine_t, pstride, 12);
SAME(mda_pc_moe_combine_t, sg_off, 16);
SAME(mda_pc_moe_combine_t, inj_stride, 20);
SAME(mda_pc_moe_combine_t, inj_off, 24);
SAME(mda_pc_moe_combine_t, hc, 28);
/* the glue and neighbour kernels' structs */
_Static_assert(sizeof(struct mda_pc_qwen_elem_t) == 28, "elem");
SAME(mda_pc_qwen_elem_t, scale, 24);
_Static_assert(sizeof(struct mda_pc_absmax_t) == 8 && sizeof(struct mda_pc_cast_t) == 8, "absmax/cast");
_Static_assert(sizeof(struct mda_pc_qwen_bf16_t) == 4, "bf16");
_Static_assert(sizeof(struct mda_pc_kd_bytes_t) == 8, "kd_bytes");

/* the entry points accept the reference's own struct types by value */
void abi_pc_check_use(moe_cuda_ctx_t *c) {
    struct mda_pc_moe_route_t r = {1, 1, 1, 1};
    struct mda_pc_moe_scan_t s = {1, 128};
    moe_cuda_route(c, NULL, NULL, NULL, NULL, r);
    moe_cuda_scan(c, NULL, NULL, NULL, s);
}
