// Pieces shared by the tensor-core attention kernels: cp.async, ldmatrix and mma.sync wrappers,
// the swizzled shared-memory layouts, and the per-warp tile steps (Q K^T, online softmax, P V).
#pragma once

#include <math.h>

#include "common.cuh"

namespace tie {

constexpr int kAttnThreads = 128;
constexpr int kKeysPerTile = 64;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Where 16-byte chunk c of row r lives in a shared-memory tile whose rows hold DH bfloat16 (DH a
// multiple of 64). Both layouts XOR the chunk index with the row, so that the 8 rows an ldmatrix
// reads at one chunk fall into 8 different bank groups.
//   RowLayout   rows of DH * 2 bytes, as the cp.async loaders write them.
//   HalfLayout  64-row tiles split into DH / 64 column blocks of 128-byte rows: what TMA writes with
//               its 128-byte swizzle when every box is 64 elements wide and starts 1024-byte aligned.
template <int DH> struct RowLayout {
  static __device__ __forceinline__ uint32_t at(int r, int c) { return static_cast<uint32_t>(r * (DH * 2) + ((c ^ (r & 7)) << 4)); }
};
template <int DH> struct HalfLayout {
  static __device__ __forceinline__ uint32_t at(int r, int c) {
    return static_cast<uint32_t>((c >> 3) * (64 * 128) + r * 128 + (((c & 7) ^ (r & 7)) << 4));
  }
};
template <int DH> __device__ __forceinline__ uint32_t swz(int r, int c) { return RowLayout<DH>::at(r, c); }

// Copies keys [key0, key0 + 64) of one kv head (rows of DH elements) from their pages into a
// swizzled K tile and the V tile behind it; keys outside [lo, hi] are zero-filled and their
// pages never touched. A thread always handles the same 16-byte column of the rows it copies,
// and the page of a key is looked up once for both planes.
template <int DH>
__device__ __forceinline__ void load_kv_tiles(uint32_t k_dst, uint32_t v_dst, const __nv_bfloat16* __restrict__ k_plane,
                                              const __nv_bfloat16* __restrict__ v_plane, const int* __restrict__ table,
                                              int kvh, int kv_heads, int page_size, int key0, int lo, int hi) {
  constexpr int CPR = DH / 8;                       // 16-byte chunks per row
  constexpr int RPP = kAttnThreads / CPR;           // rows covered by one pass of the block
  static_assert(kAttnThreads % CPR == 0 && kKeysPerTile % RPP == 0, "tile does not divide among the threads");
  const int c = threadIdx.x % CPR;
  const int r0 = threadIdx.x / CPR;
#pragma unroll
  for (int p = 0; p < kKeysPerTile / RPP; ++p) {
    const int r = r0 + p * RPP;
    const int key = key0 + r;
    const bool valid = key >= lo && key <= hi;
    long long off = 0;
    if (valid) {
      const int page = table[key / page_size];
      off = (static_cast<long long>(page * kv_heads + kvh) * page_size + key % page_size) * DH + c * 8;
    }
    const uint32_t sw = swz<DH>(r, c);
    cp_async16(k_dst + sw, k_plane + off, valid ? 16 : 0);
    cp_async16(v_dst + sw, v_plane + off, valid ? 16 : 0);
  }
}

// S[16 x (8 * NT)] += Q[16 x DH] . K^T for NT key tiles of 8 starting at row `key_row` of the K tile.
template <int DH, int NT, typename L = RowLayout<DH>>
__device__ __forceinline__ void qk_tile(float (&s)[NT][4], const uint32_t (&qf)[DH / 16][4], uint32_t k_tile, int key_row) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {   // two key tiles of 8 per ldmatrix.x4
      uint32_t b[4];
      const int r = key_row + np * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int c = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b, k_tile + L::at(r, c));
      mma_bf16(s[2 * np], qf[ks], b[0], b[1]);
      mma_bf16(s[2 * np + 1], qf[ks], b[2], b[3]);
    }
  }
}

// acc[16 x DH] += P[16 x (8 * NT)] . V for the NT * 8 keys starting at row `key_row` of the V tile.
template <int DH, int NT, typename L = RowLayout<DH>>
__device__ __forceinline__ void pv_tile(float (&acc)[DH / 8][4], const float (&p)[NT][4], uint32_t v_tile, int key_row) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int kk = 0; kk < NT / 2; ++kk) {     // 16 keys per MMA k-step
    uint32_t a[4];
    a[0] = pack_bf16(p[2 * kk][0], p[2 * kk][1]);
    a[1] = pack_bf16(p[2 * kk][2], p[2 * kk][3]);
    a[2] = pack_bf16(p[2 * kk + 1][0], p[2 * kk + 1][1]);
    a[3] = pack_bf16(p[2 * kk + 1][2], p[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < DH / 16; ++dp) {  // two output tiles of 8 dims per ldmatrix.x4.trans
      uint32_t b[4];
      const int r = key_row + kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
      const int c = dp * 2 + (lane >> 4);
      ldmatrix_x4_trans(b, v_tile + L::at(r, c));
      mma_bf16(acc[2 * dp], a, b[0], b[1]);
      mma_bf16(acc[2 * dp + 1], a, b[2], b[3]);
    }
  }
}

// Online softmax update of one warp's 16 rows over NT key tiles of 8. s holds scores already
// multiplied by scale * log2(e) with masked entries at -inf; on return s holds the weights p.
template <int DH, int NT>
__device__ __forceinline__ void softmax_update(float (&s)[NT][4], float (&m)[2], float (&l)[2], float (&acc)[DH / 8][4]) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {      // rows g and g + 8
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * half], s[j][2 * half + 1]));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m[half], mx);
    const float base = m_new == -INFINITY ? 0.0f : m_new;   // a row with no key yet: keep everything at zero
    const float corr = exp2f(m[half] - base);
    float sum = 0.0f;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      s[j][2 * half] = exp2f(s[j][2 * half] - base);
      s[j][2 * half + 1] = exp2f(s[j][2 * half + 1] - base);
      sum += s[j][2 * half] + s[j][2 * half + 1];
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l[half] = l[half] * corr + sum;
    m[half] = m_new;
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
      acc[j][2 * half] *= corr;
      acc[j][2 * half + 1] *= corr;
    }
  }
}

}  // namespace tie
