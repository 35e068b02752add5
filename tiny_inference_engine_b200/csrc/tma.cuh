// Shared pieces of the kernels that move tiles with TMA: mbarrier and bulk-tensor-copy wrappers
// (inline PTX), bounded waits, the host-side tensor-map encoder, and the status word.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace tie {

constexpr unsigned long long kWaitCycles = 4000000000ull;  // about two seconds

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait. Returns false (and records `where`) when the barrier did not flip in time or
// another role of this CTA already gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, int* status, int where) {
  if (mbar_try_wait(bar, parity)) return true;
  const unsigned long long start = clock64();
  while (!mbar_try_wait(bar, parity)) {
    if (*abort_flag != 0) return false;
    if (clock64() - start > kWaitCycles) {
      *abort_flag = 1;
      *reinterpret_cast<volatile int*>(status) = where;
      return false;
    }
  }
  return true;
}

// Bounded wait for up to three barriers at once (entries with `on` false are skipped): one round of polling
// and one return for what would otherwise be three waits in a row, each with its own latency.
struct BarrierPhase {
  uint64_t* bar;
  uint32_t parity;
  bool on;
};
__device__ __forceinline__ bool mbar_wait_all(const BarrierPhase& a, const BarrierPhase& b, const BarrierPhase& c,
                                              volatile int* abort_flag, int* status, int where) {
  bool da = !a.on, db = !b.on, dc = !c.on;
  const unsigned long long start = clock64();
  for (;;) {
    if (!da) da = mbar_try_wait(a.bar, a.parity);
    if (!db) db = mbar_try_wait(b.bar, b.parity);
    if (!dc) dc = mbar_try_wait(c.bar, c.parity);
    if (da && db && dc) return true;
    if (*abort_flag != 0) return false;
    if (clock64() - start > kWaitCycles) {
      *abort_flag = 1;
      *reinterpret_cast<volatile int*>(status) = where;
      return false;
    }
  }
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(smem_u32(bar))
      : "memory");
}

// ---------------------------------------------------------------------------------------------
// Host side (defined in errors.cu)

// [rows, cols] bfloat16 with row stride ld elements; box = box_cols x box_rows, 128-byte swizzle
// (box_cols * 2 must be 128), zeros outside the tensor.
bool make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols,
                   int box_rows);

// Device pointer of the status word (pinned, mapped host memory): kernels write a code there when a
// bounded wait runs out; the host reads and clears it with tie_kernel_status(). Null if it could
// not be allocated.
int* status_word();

}  // namespace tie
