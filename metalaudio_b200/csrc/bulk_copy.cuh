// One-dimensional bulk asynchronous copies global -> shared (the TMA unit's untiled form,
// cp.async.bulk) completed on an mbarrier.  One elected thread moves a whole frame with a single
// instruction: no registers, and none of the load/store-pipe wavefronts a per-thread copy costs.
// No multicast; source, destination and size must be multiples of 16 bytes.  (The tiled form,
// through a tensor map, is bulk_tensor_load_3d below.)
//
// Every wait is bounded: after kBulkWaitLimit polls the waiter gives up, records the failure
// in a device flag the host reads at the next synchronisation, and carries on (the frame's
// output is then meaningless, but nothing hangs).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace ma {

constexpr int kBulkWaitLimit = 1 << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void bulk_barrier_init(uint64_t* bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders this thread's earlier ordinary shared-memory accesses (and, through the CTA barrier the
// callers place in front, everyone's) before the copy unit's writes to the same buffer.
__device__ __forceinline__ void bulk_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Arms the barrier for `bytes` and starts the copy.  Called by one thread.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    const uint32_t b = smem_u32(bar);
    bulk_proxy_fence();
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(b), "r"(bytes) : "memory");
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(b)
        : "memory");
}

// Several copies on one phase: one thread arms the barrier once for the total and then starts each
// copy with bulk_copy_part.
__device__ __forceinline__ void bulk_barrier_expect(uint64_t* bar, uint32_t total_bytes) {
    bulk_proxy_fence();
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(total_bytes) : "memory");
}
__device__ __forceinline__ void bulk_copy_part(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Tiled form: one box of a three-dimensional tensor (described by a host-built tensor map) lands in
// shared memory, row after row, dense.  Called by one thread after bulk_barrier_expect with the box's
// byte count.  x counts elements of the innermost dimension and x * element size must be a multiple
// of 16 bytes; dst must be 128-byte aligned.  No multicast.
__device__ __forceinline__ void bulk_tensor_load_3d(void* dst, const void* tensor_map, int x, int y, int z, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(dst)),
        "l"(tensor_map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

// Tiled store: a dense box in shared memory goes to its place in a three-dimensional tensor.  Every
// thread that wrote the box calls bulk_proxy_fence() and the CTA synchronises; then one thread calls
// this, which also waits until the copy unit has read the box (the shared memory may then be reused
// or released; the global writes complete on their own).  Coordinates must not be negative.
__device__ __forceinline__ void bulk_tensor_store_3d(const void* tensor_map, int x, int y, int z, const void* src) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.tile.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(tensor_map),
                 "r"(x), "r"(y), "r"(z), "r"(smem_u32(src))
                 : "memory");
}
__device__ __forceinline__ void bulk_store_commit_and_wait_read() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
    asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
}

// Waits for the phase with the given parity; false when the poll limit ran out.
__device__ __forceinline__ bool bulk_barrier_wait(uint64_t* bar, uint32_t parity, int limit = kBulkWaitLimit) {
    const uint32_t b = smem_u32(bar);
    for (int i = 0; i < limit; ++i) {
        uint32_t done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(b), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

}  // namespace ma
