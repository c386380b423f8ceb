// mbarrier and TMA helpers shared by the kernels that stage tiles through
// shared memory: bounded waits, 2-D tiled loads, and the host-side encoding of
// tensor maps for bfloat16 matrices with 128-byte swizzled boxes.
#pragma once
#include <cuda.h>

#include "common.cuh"

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
#ifndef AF_TRY_WAIT_HINT_NS
#define AF_TRY_WAIT_HINT_NS 200000
#endif
// One try: the thread is suspended by the hardware until the phase completes
// or a time limit (the hint, in nanoseconds) passes; it wakes as soon as the
// barrier flips, without polling traffic.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity), "r"((uint32_t)AF_TRY_WAIT_HINT_NS)
      : "memory");
  return ok != 0;
}

constexpr unsigned long long AF_WAIT_LIMIT_NS = 2000000000ull;  // 2 s

// Waits until the barrier's phase `parity` is complete.  False when the time
// limit ran out (then *give_up is set) or another thread gave up already.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* give_up,
                                          unsigned long long limit_ns = AF_WAIT_LIMIT_NS) {
  if (mbar_try_wait(bar, parity)) return true;
  // try_wait itself suspends the thread for a while; the timer read between two polls
  // keeps waiting threads from crowding out working ones
  const unsigned long long t0 = now_ns();
  for (;;) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*give_up) return false;
    if (now_ns() - t0 > limit_ns) {
      *give_up = 1;
      return false;
    }
  }
}
// After a wait gave up: a grace period in which copies that were issued land
// before the block's shared memory is reused or released.
__device__ __forceinline__ void grace_period() {
  const unsigned long long t0 = now_ns();
  while (now_ns() - t0 < 1000000ull) {
  }
}
// c0: coordinate along the row (elements; * 2 bytes must be a multiple of 16), c1: row
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}

// The same for bytes that are read once (the weights of a decode step, a step's cache pages): they are marked
// first to leave L2, so that what streams through does not push out the small things every kernel comes back to
// (activations, partial sums, the step's tables).
__device__ __forceinline__ uint64_t l2_policy_read_once() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ void tma_load_2d_once(void* dst, const CUtensorMap* map, int c0, int c1, uint64_t* bar,
                                                 uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1, {%3, %4}], "
      "[%2], %5;"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}

// And the other way round, for small tables that every layer of a step comes back to (a layer's weights pass
// through L2 between two visits): loaded so that they are the last to leave.
__device__ __forceinline__ uint64_t l2_policy_keep() {
  uint64_t policy;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(policy));
  return policy;
}
__device__ __forceinline__ int4 ld_keep_int4(const int4* p, uint64_t policy) {
  int4 v;
  asm volatile("ld.global.nc.L2::cache_hint.v4.s32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(policy));
  return v;
}
__device__ __forceinline__ int ld_keep_int(const int* p, uint64_t policy) {
  int v;
  asm volatile("ld.global.nc.L2::cache_hint.s32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(policy));
  return v;
}

typedef CUresult (*AfEncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline AfEncodeTiledFn af_encode_tiled() {
  static AfEncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (AfEncodeTiledFn)p;
  }
  return fn;
}

// Tensor map of a [rows, cols] bfloat16 matrix with dense rows `ld` elements
// apart; boxes of 64 columns (128 bytes, hardware-swizzled) x box_rows rows;
// what lies outside the matrix reads as zero.
inline int af_make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld,
                            int box_rows) {
  AfEncodeTiledFn enc = af_encode_tiled();
  if (enc == nullptr) return af_fail(-1, "the driver has no cuTensorMapEncodeTiled");
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return af_fail(-1, "cuTensorMapEncodeTiled failed (%d)", (int)r);
  return 0;
}
