// Inline-PTX building blocks shared by the tensor-core kernels: mbarriers with
// bounded waits, TMA tile loads (never multicast), tcgen05 descriptors, MMA
// issue / commit, tensor-memory loads.
#pragma once

#include "moe_common.cuh"

namespace moe_tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t globaltimer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// Bounded wait.  False = gave up (own timeout, or another role raised abort).
// wait_ns bounds any single wait (the context's limit, 2 s by default).
static __device__ __noinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile uint32_t *abort, uint32_t *status,
                                       uint32_t site, uint64_t wait_ns) {
    uint32_t spins = 0;
    uint64_t t0 = 0;
    while (!mbar_try_wait(bar, parity)) {
        spins += 1;
        if ((spins & 0xffu) == 0) {
            if (*abort != 0) return false;
            uint64_t now = globaltimer_ns();
            if (t0 == 0) {
                t0 = now;
            } else if (now - t0 > wait_ns) {
                *abort = 1;
                atomicCAS(status, 0u, (uint32_t)MOE_ERR_TIMEOUT | (site << 8));
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {  // never suspends the thread
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.b32 %0, 1, 0, p;\n\t}\n" : "=r"(pred));
    return pred != 0;
}
// Whole-warp wait for stage (gstep % STAGES) of a ring of `full` barriers that one consumer drains in order.
// A look at an mbarrier costs ~150 cycles even when the phase is complete, so one look covers the whole ring:
// lane l asks about the next use of stage l, and the answers are kept in `ready` (bit per stage) until used.
// False = gave up (own timeout, or another role raised abort).
template <uint32_t STAGES>
static __device__ __noinline__ bool mbar_ring_wait(const uint64_t *full, uint32_t gstep, uint32_t &ready, volatile uint32_t *abort,
                                                   uint32_t *status, uint32_t site, uint64_t wait_ns) {
    const uint32_t lane = threadIdx.x & 31u, s = gstep % STAGES;
    const uint32_t l = lane < STAGES ? lane : 0u;
    const uint32_t use = gstep + (l + STAGES - s) % STAGES;
    const uint32_t bar = smem_u32(full + l), parity = (use / STAGES) & 1u;
    uint32_t spins = 0;
    uint64_t t0 = 0;
    const uint32_t bar_s = smem_u32(full + s), parity_s = (gstep / STAGES) & 1u;
    for (;;) {
        ready = __ballot_sync(0xffffffffu, lane < STAGES && mbar_test_wait(bar, parity));
        if ((ready >> s) & 1u) return true;
        mbar_try_wait(bar_s, parity_s);  // not there yet: let the hardware park the warp on the stage it needs
        spins += 1;
        if ((spins & 0xfu) == 0) {
            uint32_t stop = *abort != 0 ? 1u : 0u;
            uint64_t now = globaltimer_ns();
            if (t0 == 0) t0 = now;
            else if (now - t0 > wait_ns) stop = 2u;
            stop = __reduce_max_sync(0xffffffffu, stop);
            if (stop != 0) {
                if (stop == 2u && lane == 0) {
                    *abort = 1;
                    atomicCAS(status, 0u, (uint32_t)MOE_ERR_TIMEOUT | (site << 8));
                }
                return false;
            }
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int32_t c0, int32_t c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        :
        : "r"(dst), "l"((uint64_t)map), "r"(bar), "r"(c0), "r"(c1)
        : "memory");
}

// Shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row
// groups 1024 bytes apart, descriptor version 1 (sm_100).
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// The same for a 64-byte swizzle (rows of 32 fp16): 8-row groups 512 bytes apart.
__device__ __forceinline__ uint64_t umma_desc_sw64(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3ffffu) >> 4) | ((uint64_t)(512u >> 4) << 32) | (1ull << 46) | (4ull << 61);
}
// Instruction descriptor, kind::f16: D fp32, A/B fp16, both K-major.
__device__ __forceinline__ uint32_t umma_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accum) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}\n"
        :
        : "r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accum)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}


}  // namespace moe_tc
