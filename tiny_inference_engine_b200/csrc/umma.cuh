// tcgen05 pieces shared by the matrix-product kernels: shared-memory and instruction descriptors,
// MMA issue, commit and tensor-memory load wrappers (inline PTX).
#pragma once

#include "tma.cuh"

namespace tie {

// Shared-memory matrix descriptor of a k-major tile with 128-byte swizzle: rows of 128 bytes,
// groups of 8 rows 1024 bytes apart (stride byte offset), descriptor version 1 (Blackwell).
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);        // start address, 16-byte units
  d |= static_cast<uint64_t>(1) << 16;                      // leading byte offset: unused with swizzle
  d |= static_cast<uint64_t>(1024 >> 4) << 32;              // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                      // version
  d |= static_cast<uint64_t>(2) << 61;                      // SWIZZLE_128B
  return d;
}

// The same descriptor as two words, for issue loops: the high word is constant, and an operand tile
// that lies `bytes` further on (inside the 256 KB of shared memory) has `bytes >> 4` more in the low word.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo_sw128(uint32_t addr, uint32_t leading_bytes = 16) {
  return ((addr >> 4) & 0x3FFF) | ((leading_bytes >> 4) << 16);
}
__device__ __forceinline__ uint64_t desc_from_words(uint32_t lo, uint32_t hi) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(lo), "r"(hi));
  return d;
}

// Instruction descriptor: float accumulator, bfloat16 A and B, both k-major, M = bm, N = bn.
__host__ __device__ constexpr uint32_t instr_desc(int bn, int bm = 128) {
  return (1u << 4) | (1u << 7) | (1u << 10) | (static_cast<uint32_t>(bn >> 3) << 17) | (static_cast<uint32_t>(bm >> 4) << 24);
}

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// True in exactly one lane of a converged warp. An issue loop that stays warp-uniform and only wraps the
// tcgen05 instructions themselves in `if (elect_one())` lets the compiler keep descriptors and addresses
// in uniform registers, which is where those instructions take them from.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
}

}  // namespace tie
