// Inline-PTX wrappers for the sm_100a features the matmul kernels use: mbarriers with bounded
// waits, bulk asynchronous copies, tensor memory (TMEM) management, tcgen05 MMA / commit / load,
// and the shared-memory and instruction descriptors of the fifth-generation tensor cores.
#pragma once
#include <cstdint>

namespace ttb {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier --------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// try_wait that lets the hardware suspend the thread for up to `ns` nanoseconds while the phase is incomplete (it wakes
// early when the phase completes): a waiting thread then issues an instruction every few microseconds instead of spinning
// through the issue slots of the warps that share its scheduler.
__device__ __forceinline__ bool mbar_try_wait_suspend(uint32_t bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(ok)
        : "r"(bar), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}

// Bounded wait. Gives up after `limit_cycles` SM clocks or as soon as another thread of the block
// has given up (*abort_flag != 0); on giving up it raises the block's abort flag, records `code`
// in the global status word and returns false. The caller then skips to the kernel's teardown.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status_word,
                                          int code, long long limit_cycles = 2000000000LL) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t spin = 1;; ++spin) {
        if (mbar_try_wait_suspend(bar, parity, 4000u)) return true;
        if ((spin & 7u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > limit_cycles) {
                *abort_flag = 1;
                atomicCAS(status_word, 0, code);
                return false;
            }
        }
    }
}

// One lane of a converged warp: the lane that issues for warp-uniform single-issuer roles (the others follow the same
// control flow, so addresses and descriptors stay uniform-datapath values).
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n\t"
        ".reg .pred P;\n\t"
        "elect.sync _|P, 0xffffffff;\n\t"
        "selp.u32 %0, 1, 0, P;\n\t"
        "}"
        : "=r"(pred));
    return pred != 0;
}

// ---- proxies and fences ------------------------------------------------------------------------
// Orders this thread's shared-memory writes (generic proxy) before later asynchronous-proxy reads
// (tcgen05.mma operand fetches, bulk copies).
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- programmatic dependent launch ----------------------------------------------------------------
// grid_dep_launch: lets a kernel that was launched as a programmatic dependent of this one be scheduled once every
// block of this grid has executed it (or exited). grid_dep_wait: returns when the grids this one depends on have
// completed and their writes are visible. Both do nothing in a launch without a programmatic dependency.
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// ---- bulk copy global -> shared, completion counted on an mbarrier ------------------------------
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src_gmem, uint32_t bytes, uint32_t bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            dst_smem),
        "l"(src_gmem), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}

// Same without a cache hint (data that other blocks will read again from L2).
__device__ __forceinline__ void bulk_g2s_plain(uint32_t dst_smem, const void *src_gmem, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_smem),
                 "l"(src_gmem), "r"(bytes), "r"(bar)
                 : "memory");
}

// Tiled tensor-map copy, three dimensions (x innermost), global -> shared, completion counted on an mbarrier. The x
// coordinate times the element size must be a multiple of 16 bytes (callers here always pass x = 0).
__device__ __forceinline__ void tma_load_3d(uint32_t dst_smem, const void *tensor_map, int x, int y, int z, uint32_t bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%2, %3, %4}], [%5], %6;" ::"r"(
            dst_smem),
        "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(bar), "l"(policy)
        : "memory");
}

// The same with five dimensions.
__device__ __forceinline__ void tma_load_5d(uint32_t dst_smem, const void *tensor_map, int c0, int c1, int c2, int c3, int c4, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.5d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5, %6}], [%7];" ::"r"(dst_smem),
        "l"(tensor_map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(c4), "r"(bar)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d_plain(uint32_t dst_smem, const void *tensor_map, int x, int y, int z, uint32_t bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(dst_smem),
        "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}
// Makes writes of other GPUs (or of earlier kernels) that this thread has observed through generic loads visible to the
// asynchronous proxy, i.e. to tensor-map copies this thread issues afterwards.
__device__ __forceinline__ void fence_proxy_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// ---- tensor memory -------------------------------------------------------------------------------
// Whole-warp calls. `ncols` is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// ---- descriptors ----------------------------------------------------------------------------------
// Shared-memory operand descriptor without swizzle. A core matrix is 8 rows of 16 bytes stored as 128
// contiguous bytes. `lbo` is the byte distance between core matrices adjacent along K, `sbo` between
// core matrices adjacent along M/N. Bits: [0,14) address>>4, [16,30) lbo>>4, [32,46) sbo>>4,
// [46,48) descriptor version 1, [61,64) swizzle mode 0.
__device__ __forceinline__ uint64_t smem_desc_noswizzle(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46);
}

// K-major operand with the 32-byte swizzle: rows of 32 bytes (16 bf16 = one MMA K step), eight rows form a 256-byte atom
// inside which the 16-byte half of a row is exchanged for rows 4..7 (address bit 4 ^= bit 7) - the pattern a tensor-map
// copy with CU_TENSOR_MAP_SWIZZLE_32B writes. `sbo` = bytes between 8-row groups; the leading offset is unused (1).
// The operand must start on a 256-byte boundary. Bits [61,64): 6 = 32-byte swizzle.
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t addr, uint32_t sbo) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | (1ull << 16) | ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | (6ull << 61);
}

// Instruction descriptor for kind::f16 with bf16 operands and an fp32 accumulator.
// Bits: [4,6) D format (1 = f32), [7,10) A format (1 = bf16), [10,13) B format, 15 A major
// (1 = M/N-contiguous), 16 B major, [17,23) N>>3, [24,29) M>>4.
__host__ __device__ constexpr uint32_t instr_desc_bf16_f32(int M, int N, bool a_mn_major, bool b_mn_major) {
    return (1u << 4) | (1u << 7) | (1u << 10) | ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the whole CTA.
__device__ __forceinline__ void mma_bf16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                            bool accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Each lane reads 16 consecutive 32-bit columns of its own TMEM lane (lane = 32*(warp%4) + laneid).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

}  // namespace ptx
}  // namespace ttb
