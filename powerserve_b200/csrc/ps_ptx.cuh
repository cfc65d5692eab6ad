// ps_ptx.cuh - inline-PTX building blocks shared by every kernel file: mbarrier, 1-D TMA bulk copies, programmatic dependent
// launch, and the tcgen05 (5th-generation tensor core) wrappers - shared-memory operand descriptors for the canonical
// K-major no-swizzle layout, the single-thread MMA issue, commit, fences, tensor-memory loads and the bounded mbarrier wait.
#pragma once
#include "ps_math.cuh"

#include <cstdint>

// ---------------------------------------------------------------------------------------------------- PTX helpers
PS_D uint32_t ps_smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
PS_D void ps_mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(ps_smem_u32(bar)), "r"(count));
}
PS_D void ps_mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(ps_smem_u32(bar)), "r"(bytes) : "memory");
}
PS_D void ps_mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(ps_smem_u32(bar)) : "memory");
}
PS_D void ps_mbar_wait(uint64_t *bar, uint32_t parity) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "WAIT_%=:\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%0], %1;\n\t"
        "@p bra DONE_%=;\n\t"
        "bra WAIT_%=;\n\t"
        "DONE_%=:\n\t}" ::"r"(ps_smem_u32(bar)),
        "r"(parity)
        : "memory");
}
// 1-D TMA: global -> shared, completion counted in bytes on an mbarrier
PS_D void ps_bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(ps_smem_u32(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(ps_smem_u32(bar))
                 : "memory");
}
PS_D void ps_fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
PS_D void ps_grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
PS_D void ps_grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
PS_D void ps_bar_sync(int id, int n) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(n) : "memory"); }

// ---------------------------------------------------------------------------------------------------- tcgen05 helpers
PS_D uint64_t ps_tc_smem_desc(uint32_t smem_addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    // cute::UMMA::SmemDescriptor: start address [0,14) >> 4, leading byte offset [16,30) >> 4, stride byte offset [32,46) >> 4,
    // version [46,48) = 1 (Blackwell), layout type [61,64) = 0 (no swizzle)
    return (uint64_t)((smem_addr & 0x3FFFF) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
}
PS_D void ps_tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
PS_D void ps_tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(ps_smem_u32(bar)) : "memory");
}
PS_D void ps_tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
PS_D void ps_tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
PS_D void ps_tc_ld8(uint32_t taddr, float v[8]) { // 32 lanes x 8 consecutive columns, one row (lane) per thread
    uint32_t r[8];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
#pragma unroll
    for (int t = 0; t < 8; t++) v[t] = __uint_as_float(r[t]);
}
PS_D void ps_tc_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// bounded mbarrier wait: a mis-sequenced pipeline must never hang the GPU (returns false after ~2^22 polls)
PS_D bool ps_tc_wait(uint64_t *bar, uint32_t parity) {
    for (int spin = 0; spin < (1 << 22); spin++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(ps_smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

