// Bulk asynchronous copies (the TMA engine in its untiled form) with an mbarrier, for staging the contiguous
// per-block slices of the AoS parameter arrays.  No cluster launch and no multicast: every copy is between this
// GPU's global memory and the issuing block's shared memory.
// Rules obeyed by the callers: global address and shared address 16-byte aligned, size a multiple of 16 bytes.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace fsgs {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals));
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// global -> shared, completion counted in bytes on the mbarrier
__device__ __forceinline__ void bulk_load(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   smem_u32(dst_smem)),
               "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

// Waits for the given phase with an iteration limit; false when the limit ran out (the caller records the failure
// and falls back to plain loads -- nothing spins for ever).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, int limit = 1 << 20) {
  const uint32_t a = smem_u32(bar);
  for (int i = 0; i < limit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(a), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}

// Makes this thread's plain shared-memory writes visible to the async proxy.  Every thread that filled a buffer calls
// it before the block barrier that precedes bulk_store().
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// shared -> global, issued by one thread after fence_async_smem() + __syncthreads(); that thread must call
// bulk_store_wait() before the shared buffer is reused or the block exits.
__device__ __forceinline__ void bulk_store(void *dst_gmem, const void *src_smem, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst_gmem), "r"(smem_u32(src_smem)),
               "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

// shared -> global with element-wise float addition at the destination (the copy engine's reduction form); same
// issue and wait rules as bulk_store().
__device__ __forceinline__ void bulk_reduce_add_f32(void *dst_gmem, const void *src_smem, uint32_t bytes) {
  asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst_gmem),
               "r"(smem_u32(src_smem)), "r"(bytes)
               : "memory");
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}

__device__ __forceinline__ void bulk_store_wait() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

}  // namespace fsgs
