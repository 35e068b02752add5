// Embedding, norms, rotary position encoding, cache append and SiLU*mul: the memory-bound
// kernels between the matrix products. Each is templated on the storage type of the
// activations (float for the 32-bit path, bfloat16 for serving); every sum, scale, angle
// and the residual stream itself are float.
//
// What each computes follows the reference's CPU backend (src/backend/cpu/cpu_backend.cpp):
// embed :51-76, rms_norm :141-159, rope_neox :161-193, silu_mul :195-207, add :209-221,
// gather_rows :223-233, kv_write :235-259. The fusions are this engine's own.
#include "common.cuh"
#include "head_prep.cuh"
#include "launchers.h"

namespace tie {

// ---------------------------------------------------------------------------------------------
// x[t, :] = float(table[ids[t], :]). The residual stream is float in both paths.
// With k_block_rows > 0 the table is stored in k-blocks, [ceil(dim / 64)][k_block_rows][64] (the layout the
// matrix products stream best, gemm_tc.cu; a tied output table is this very tensor): element i of row id is at
// ((i / 64) * k_block_rows + id) * 64 + i % 64.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, float* __restrict__ x,
                             int dim, int vocab, int k_block_rows) {
  pdl_sync();
  const int t = blockIdx.x;
  int id = ids[t];
  // ids are validated on the host (an id that a step ahead could not sample arrives negative: its request ends
  // anyway); never read outside the table
  id = id < 0 ? 0 : (id >= vocab ? vocab - 1 : id);
  float* out = x + static_cast<size_t>(t) * dim;
  // 16 bytes of the table a thread and step where rows and addresses allow it (a 64-column block never ends inside one)
  constexpr int V = Vec16<T>::N;
  if (dim % V == 0 && reinterpret_cast<uintptr_t>(table) % 16 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0) {
    for (int i = threadIdx.x * V; i < dim; i += blockDim.x * V) {
      Vec16<T> v;
      v.load(k_block_rows > 0 ? table + (static_cast<size_t>(i >> 6) * k_block_rows + id) * 64 + (i & 63)
                              : table + static_cast<size_t>(id) * dim + i);
#pragma unroll
      for (int e = 0; e < V; e += 4)
        *reinterpret_cast<float4*>(out + i + e) = make_float4(v.v[e], v.v[e + 1], v.v[e + 2], v.v[e + 3]);
    }
    return;
  }
  if (k_block_rows > 0) {
    for (int i = threadIdx.x; i < dim; i += blockDim.x)
      out[i] = ld(table + (static_cast<size_t>(i >> 6) * k_block_rows + id) * 64 + (i & 63));
    return;
  }
  const T* row = table + static_cast<size_t>(id) * dim;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) out[i] = ld(row + i);
}

// tokens[dst[i]] = ids[src[i]]: a step that is queued before the host has seen the ids sampled by the step ahead
// of it takes them from the device; dst is the row of a request's token in this step, src its row in that step.
__global__ void scatter_ids_kernel(int* __restrict__ tokens, const int* __restrict__ dst, const int* __restrict__ src,
                                   const int* __restrict__ ids, int n) {
  pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) tokens[dst[i]] = ids[src[i]];
}

// ---------------------------------------------------------------------------------------------
// Residual add fused with the norm that follows it:
//   x[t] += delta[t]  (float sum, written back; skipped when delta is null)
//   out[t] = (x[t] * inv) * w,  inv = 1 / sqrt(mean(x[t]^2) + eps)
// With `rows` non-null, row t of the output comes from row rows[t] of x and delta, and x is
// not written back (the rows that reach the final norm are the last use of x).
// The delta may also come as float partial sums of a split matrix product: part[z][row][dim],
// z < splits, part_stride floats apart; they are added in split order.
template <typename T, int VPT>
__global__ void __launch_bounds__(1024) add_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta, const float* __restrict__ part,
                                   long long part_stride, int splits, const int* __restrict__ rows,
                                   const float* __restrict__ w, float eps, T* __restrict__ out, int dim) {
  pdl_sync();
  // VPT > 0: every thread keeps its VPT elements (index threadIdx.x + i * blockDim.x) in registers
  // between the sum and the scaling; VPT == 0: rows longer than that are read twice.
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[t] : t) * dim;
  float* xr = x + src;
  const T* dr = delta ? delta + src : nullptr;
  const float* pr = part ? part + src : nullptr;
  T* o = out + static_cast<size_t>(t) * dim;
  const bool has_delta = dr != nullptr || pr != nullptr;
  const bool write_back = has_delta && rows == nullptr;
  auto delta_at = [&](int k) -> float {
    if (dr) return ld(dr + k);
    float acc = pr[k];
    for (int z = 1; z < splits; ++z) acc += pr[static_cast<long long>(z) * part_stride + k];
    return acc;
  };
  float ss = 0.0f;
  if constexpr (VPT > 0) {
    float v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int k = threadIdx.x + i * blockDim.x;
      v[i] = k < dim ? xr[k] : 0.0f;
    }
    if (dr) {
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int k = threadIdx.x + i * blockDim.x;
        if (k < dim) v[i] += ld(dr + k);
      }
    } else if (pr) {   // split by split, the VPT loads of a split in flight together; each element still adds in split order
      float d[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) d[i] = 0.0f;
      for (int z = 0; z < splits; ++z) {
        const float* pz = pr + static_cast<long long>(z) * part_stride;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int k = threadIdx.x + i * blockDim.x;
          if (k < dim) d[i] += pz[k];
        }
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) v[i] += d[i];
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int k = threadIdx.x + i * blockDim.x;
      if (k < dim) {
        if (write_back) xr[k] = v[i];
        ss += v[i] * v[i];
      }
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int k = threadIdx.x + i * blockDim.x;
      if (k < dim) st(o + k, (v[i] * inv) * w[k]);
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      float v = xr[i];
      if (has_delta) v += delta_at(i);
      if (write_back) xr[i] = v;
      ss += v * v;
    }
    ss = block_sum(ss, scratch);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      float v = xr[i];
      if (has_delta && !write_back) v += delta_at(i);
      st(o + i, (v * inv) * w[i]);
    }
  }
}

// The same for rows whose length is a multiple of 4: every thread owns whole 16-byte pieces of the
// float row (and the matching 8 or 16 bytes of delta and output), NV of them, and the partial
// sums of a split product are read one 16-byte piece per split.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
  static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
  static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(t.x << 16), __uint_as_float(t.x & 0xffff0000u), __uint_as_float(t.y << 16),
                       __uint_as_float(t.y & 0xffff0000u));
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
    const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
  }
};

template <typename T, int NV>
__global__ void __launch_bounds__(1024) add_rmsnorm_vec4_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                                const float* __restrict__ part, long long part_stride,
                                                                int splits, const int* __restrict__ rows,
                                                                const float* __restrict__ w, float eps, T* __restrict__ out,
                                                                int dim) {
  // the norm weights do not depend on the kernels ahead in the stream: fetch them before waiting
  pdl_launch_dependents();
  const int pieces = dim >> 2;
  float4 wv[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    wv[i] = c < pieces ? *reinterpret_cast<const float4*>(w + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  pdl_wait();
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[t] : t) * dim;
  float* xr = x + src;
  const T* dr = delta ? delta + src : nullptr;
  const float* pr = part ? part + src : nullptr;
  T* o = out + static_cast<size_t>(t) * dim;
  const bool write_back = (dr != nullptr || pr != nullptr) && rows == nullptr;
  float4 v[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    v[i] = c < pieces ? *reinterpret_cast<const float4*>(xr + 4 * c) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (dr) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < pieces) {
        const float4 d = Vec4<T>::load(dr + 4 * c);
        v[i].x += d.x; v[i].y += d.y; v[i].z += d.z; v[i].w += d.w;
      }
    }
  } else if (pr) {
    float4 d[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) d[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 8
    for (int z = 0; z < splits; ++z) {   // every element still adds its splits in order
      const float* pz = pr + static_cast<long long>(z) * part_stride;
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = threadIdx.x + i * blockDim.x;
        if (c < pieces) {
          const float4 q = *reinterpret_cast<const float4*>(pz + 4 * c);
          d[i].x += q.x; d[i].y += q.y; d[i].z += q.z; d[i].w += q.w;
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) { v[i].x += d[i].x; v[i].y += d[i].y; v[i].z += d[i].z; v[i].w += d[i].w; }
  }
  float ss = 0.0f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < pieces) {
      if (write_back) *reinterpret_cast<float4*>(xr + 4 * c) = v[i];
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = threadIdx.x + i * blockDim.x;
    if (c < pieces) {
      const float4 ww = wv[i];
      Vec4<T>::store(o + 4 * c, make_float4((v[i].x * inv) * ww.x, (v[i].y * inv) * ww.y, (v[i].z * inv) * ww.z, (v[i].w * inv) * ww.w));
    }
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm of n rows of `size` elements of T (stride `row_stride`), one warp per row. Used for
// norms over something else than the residual stream (per-head norms outside the fused kernel).
template <typename T>
__global__ void rmsnorm_rows_kernel(const T* __restrict__ x, long long row_stride, const float* __restrict__ w,
                                    float eps, T* __restrict__ out, long long out_stride, int size, long long n) {
  pdl_sync();
  const long long r = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= n) return;
  const int lane = threadIdx.x & 31;
  const T* xr = x + r * row_stride;
  T* o = out + r * out_stride;
  float ss = 0.0f;
  for (int i = lane; i < size; i += 32) {
    const float v = ld(xr + i);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(size) + eps);
  for (int i = lane; i < size; i += 32) st(o + i, (ld(xr + i) * inv) * w[i]);
}

// ---------------------------------------------------------------------------------------------
// out[t, i] = silu(gu[t, i]) * gu[t, inter + i], silu(g) = g / (1 + exp(-g)).
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / inter;
  const int i = static_cast<int>(idx - t * inter);
  const float g = ld(gu + t * 2 * inter + i);
  const float u = ld(gu + t * 2 * inter + inter + i);
  st(out + idx, g / (1.0f + expf(-g)) * u);
}

// ---------------------------------------------------------------------------------------------
// Rotate-half RoPE in place over the first `rot` dims of every head:
//   angle = float(pos) * inv_freq[i];  (v[i], v[i + rot/2]) <- (v[i] c - v[i+rot/2] s, v[i+rot/2] c + v[i] s)
template <typename T>
__global__ void rope_kernel(T* __restrict__ x, long long row_stride, const int* __restrict__ positions,
                            const float* __restrict__ inv_freq, int heads, int head_dim, int rot, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int half = rot / 2;
  const int i = static_cast<int>(idx % half);
  const int h = static_cast<int>((idx / half) % heads);
  const long long t = idx / (static_cast<long long>(half) * heads);
  T* v = x + t * row_stride + static_cast<long long>(h) * head_dim;
  const float angle = static_cast<float>(positions[t]) * inv_freq[i];
  const float c = cosf(angle), s = sinf(angle);
  const float x1 = ld(v + i), x2 = ld(v + i + half);
  st(v + i, x1 * c - x2 * s);
  st(v + i + half, x2 * c + x1 * s);
}

// ---------------------------------------------------------------------------------------------
// k, v rows of token t go to slot s = slots[t]: page s / page_size, offset s % page_size, in
// planes laid out [page][kv_head][offset][head_dim]. A negative slot writes nothing.
template <typename T>
__global__ void kv_append_kernel(const T* __restrict__ k, const T* __restrict__ v, long long k_stride,
                                 long long v_stride, const int* __restrict__ slots, T* __restrict__ k_cache,
                                 T* __restrict__ v_cache, int kv_heads, int head_dim, int page_size, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int d = static_cast<int>(idx % head_dim);
  const int h = static_cast<int>((idx / head_dim) % kv_heads);
  const long long t = idx / (static_cast<long long>(head_dim) * kv_heads);
  const int slot = slots[t];
  if (slot < 0) return;
  const long long page = slot / page_size, off = slot % page_size;
  const long long dst = ((page * kv_heads + h) * page_size + off) * head_dim + d;
  k_cache[dst] = k[t * k_stride + static_cast<long long>(h) * head_dim + d];
  v_cache[dst] = v[t * v_stride + static_cast<long long>(h) * head_dim + d];
}

// ---------------------------------------------------------------------------------------------
// The work between the q/k/v projection and attention, one warp per (token, head):
//   q heads: RMSNorm over the head (weight qw, skipped when null), RoPE, written back in place;
//   k heads: RMSNorm (kw), RoPE, written to the key plane at the token's slot;
//   v heads: copied to the value plane at the token's slot.
// qkv is [T, (Hq + 2 Hkv) * Dh] with q first, then k, then v. With write_kv == 0 only the q
// heads are processed (a layer that reads another layer's cache). inv_freq null = no rotation.
// With `part` non-null the q, k, v values are read as the sum of `splits` float partial sums
// part[z][t][width] (the split product that made them) instead of from qkv; q still goes to qkv.
template <typename T>
__global__ void qk_norm_rope_append_kernel(T* __restrict__ qkv, long long row_stride, const float* __restrict__ part,
                                           long long part_stride, int splits, long long part_ld,
                                           const float* __restrict__ qw,
                                           const float* __restrict__ kw, float q_eps, float k_eps,
                                           const float* __restrict__ inv_freq, int rot,
                                           const int* __restrict__ positions, const int* __restrict__ slots,
                                           T* __restrict__ k_cache, T* __restrict__ v_cache, int q_heads, int kv_heads,
                                           int head_dim, int page_size, int heads_per_token, long long total) {
  pdl_launch_dependents();   // positions and frequencies are the step's own inputs: the rotation table is made before the wait
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int warps = blockDim.x >> 5;
  const long long t = blockIdx.x;
  const int head = blockIdx.y * warps + warp;
  // the token's rotation, once for the heads of this block: cos at [0, half), sin at [half, 2 half)
  float* cs = smem + warps * head_dim;
  const int half = inv_freq ? rot / 2 : 0;
  if (half > 0) {
    const float pos = static_cast<float>(positions[t]);
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float angle = pos * inv_freq[i];
      cs[i] = cosf(angle);
      cs[half + i] = sinf(angle);
    }
  }
  pdl_wait();
  __syncthreads();
  if (head >= heads_per_token) return;
  T* src = qkv + t * row_stride + static_cast<long long>(head) * head_dim;
  const float* psrc = part ? part + t * part_ld + static_cast<long long>(head) * head_dim : nullptr;
  auto value = [&](int i) -> float {
    if (!psrc) return ld(src + i);
    float acc = psrc[i];
    for (int z = 1; z < splits; ++z) acc += psrc[static_cast<long long>(z) * part_stride + i];
    return acc;
  };
  float* buf = smem + warp * head_dim;

  const bool is_q = head < q_heads;
  const bool is_k = !is_q && head < q_heads + kv_heads;
  T* dst = src;
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int h = is_k ? head - q_heads : head - q_heads - kv_heads;
    const long long page = slot / page_size, off = slot % page_size;
    dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + h) * page_size + off) * head_dim;
    if (!is_k) {  // values are stored as they are
      if (psrc) {
        for (int i = lane; i < head_dim; i += 32) st(dst + i, value(i));
      } else {
        for (int i = lane; i < head_dim; i += 32) dst[i] = src[i];
      }
      return;
    }
  }

  const float* w = is_q ? qw : kw;
  float ss = 0.0f;
  for (int i = lane; i < head_dim; i += 32) {
    const float v = value(i);
    buf[i] = v;
    ss += v * v;
  }
  if (w) {
    ss = warp_sum(ss);
    const float inv = 1.0f / sqrtf(ss / static_cast<float>(head_dim) + (is_q ? q_eps : k_eps));
    for (int i = lane; i < head_dim; i += 32) buf[i] = (buf[i] * inv) * w[i];
  }
  __syncwarp();
  if (half > 0) {
    for (int i = lane; i < half; i += 32) {
      const float c = cs[i], s = cs[half + i];
      const float x1 = buf[i], x2 = buf[i + half];
      st(dst + i, x1 * c - x2 * s);
      st(dst + i + half, x2 * c + x1 * s);
    }
  }
  for (int i = 2 * half + lane; i < head_dim; i += 32) st(dst + i, buf[i]);
}

// The same for head sizes 64, 128 and 256 with the whole head rotated (or none of it):
// a lane holds VEC = head_dim / 32 neighbouring elements (one vector load and store), lanes 0-15 the
// first half of the head and lanes 16-31 the second, so a rotation pair is one shuffle apart.

template <typename T, int VEC>
__global__ void __launch_bounds__(256) qk_norm_rope_append_vec_kernel(T* __restrict__ qkv, long long row_stride,
                                                                      const float* __restrict__ part, long long part_stride,
                                                                      int splits, long long part_ld,
                                                                      const float* __restrict__ qw, const float* __restrict__ kw,
                                                                      float q_eps, float k_eps, const float* __restrict__ inv_freq,
                                                                      const int* __restrict__ positions, const int* __restrict__ slots,
                                                                      T* __restrict__ k_cache, T* __restrict__ v_cache, int q_heads,
                                                                      int kv_heads, int page_size, int heads_per_token) {
  pdl_launch_dependents();   // positions and frequencies are the step's own inputs: the rotation table is made before the wait
  constexpr int DH = 32 * VEC, HALF = DH / 2;
  using Slice = HeadSlice<T, VEC>;
  __shared__ float cs[DH];   // the token's rotation: cos at [0, HALF), sin at [HALF, DH)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = blockIdx.x;
  const int head = blockIdx.y * (blockDim.x >> 5) + warp;
  if (inv_freq) rotation_table(cs, static_cast<float>(positions[t]), inv_freq, HALF, threadIdx.x, blockDim.x);
  pdl_wait();
  __syncthreads();
  if (head >= heads_per_token) return;
  T* src = qkv + t * row_stride + static_cast<long long>(head) * DH + lane * VEC;
  const bool is_q = head < q_heads;
  const bool is_k = !is_q && head < q_heads + kv_heads;
  T* dst = src;
  if (!is_q) {
    const int slot = slots[t];
    if (slot < 0) return;
    const int h = is_k ? head - q_heads : head - q_heads - kv_heads;
    const long long page = slot / page_size, off = slot % page_size;
    dst = (is_k ? k_cache : v_cache) + ((page * kv_heads + h) * page_size + off) * DH + lane * VEC;
  }
  float x[VEC];
  if (part) {   // the sum of the split product's partial sums, in split order
    using FloatSlice = HeadSlice<float, VEC>;
    const float* psrc = part + t * part_ld + static_cast<long long>(head) * DH + lane * VEC;
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] = 0.0f;
#pragma unroll 4
    for (int z = 0; z < splits; ++z) {
      const FloatSlice p = *reinterpret_cast<const FloatSlice*>(psrc + static_cast<long long>(z) * part_stride);
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] += p.v[e];
    }
  } else {
    const Slice in = *reinterpret_cast<const Slice*>(src);
#pragma unroll
    for (int e = 0; e < VEC; ++e) x[e] = Elem<T>::load(in.v + e);
  }
  if (!is_q && !is_k) {   // values are stored as they are
    Slice out;
#pragma unroll
    for (int e = 0; e < VEC; ++e) Elem<T>::store(out.v + e, x[e]);
    *reinterpret_cast<Slice*>(dst) = out;
    return;
  }
  prepare_head<VEC>(x, is_q ? qw : kw, is_q ? q_eps : k_eps, inv_freq ? cs : nullptr, lane);
  Slice out;
#pragma unroll
  for (int e = 0; e < VEC; ++e) Elem<T>::store(out.v + e, x[e]);
  *reinterpret_cast<Slice*>(dst) = out;
}

// The same for many tokens, where the kernel above is bound by the instructions it issues (about 250 a
// head), not by memory. A block works on TOK tokens, one after the other; a lane holds four neighbouring
// elements of the first half of a head and the four that rotate with them in the second half, so a head takes
// LPH = DH / 8 lanes, a warp works on 32 / LPH heads at once, and the rotation needs no exchange between lanes.
// What does not depend on the head (the lane's norm weights, and per token its cos and sin and its place in the
// cache) is made once.
template <typename T, int DH, int TOK>
__global__ void __launch_bounds__(256, 4) qk_norm_rope_append_rows_kernel(T* __restrict__ qkv, long long row_stride,
                                                                       const float* __restrict__ qw, const float* __restrict__ kw,
                                                                       float q_eps, float k_eps, const float* __restrict__ inv_freq,
                                                                       const int* __restrict__ positions, const int* __restrict__ slots,
                                                                       T* __restrict__ k_cache, T* __restrict__ v_cache, int q_heads,
                                                                       int kv_heads, int page_size, int heads_per_token, int tokens) {
  pdl_launch_dependents();
  constexpr int Q = 4, HALF = DH / 2, LPH = HALF / Q, WARP_HEADS = 32 / LPH;
  using Slice = HeadSlice<T, Q>;
  __shared__ __align__(16) float cs[TOK][DH];   // a token's rotation: cos at [0, HALF), sin at [HALF, DH)
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t0 = static_cast<long long>(blockIdx.x) * TOK;
  // positions, frequencies, slots and weights do not come from the kernel ahead
  if (inv_freq) {
    for (int i = threadIdx.x; i < TOK * HALF; i += blockDim.x) {
      const int tk = i / HALF, j = i % HALF;
      if (t0 + tk < tokens) sincosf(static_cast<float>(positions[t0 + tk]) * inv_freq[j], &cs[tk][HALF + j], &cs[tk][j]);
    }
  }
  const int e0 = (lane % LPH) * Q;        // this lane's elements of each half of its head
  float4 one = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
  const float4 qw_lo = qw ? *reinterpret_cast<const float4*>(qw + e0) : one, qw_hi = qw ? *reinterpret_cast<const float4*>(qw + HALF + e0) : one;
  const float4 kw_lo = kw ? *reinterpret_cast<const float4*>(kw + e0) : one, kw_hi = kw ? *reinterpret_cast<const float4*>(kw + HALF + e0) : one;
  const int stride_heads = warps * WARP_HEADS;
  pdl_wait();
  __syncthreads();
#pragma unroll 1
  for (int tk = 0; tk < TOK; ++tk) {
    const long long t = t0 + tk;
    if (t >= tokens) break;
    const int slot = slots ? slots[t] : -1;
    const long long cache_row = slot >= 0 ? static_cast<long long>(slot / page_size) * kv_heads * page_size + slot % page_size : 0;
    float4 c = one, sn = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (inv_freq) {
      c = *reinterpret_cast<const float4*>(&cs[tk][e0]);
      sn = *reinterpret_cast<const float4*>(&cs[tk][HALF + e0]);
    }
    T* row = qkv + t * row_stride + e0;
#pragma unroll 1
    for (int base = warp * WARP_HEADS; base < heads_per_token; base += stride_heads) {   // uniform over the warp
      const int head = base + lane / LPH;
      const bool is_q = head < q_heads;
      const bool is_v = head >= q_heads + kv_heads;
      const T* src = row + static_cast<long long>(head) * DH;
      T* dst = nullptr;
      if (head < heads_per_token) {
        if (is_q) {
          dst = const_cast<T*>(src);
        } else if (slot >= 0) {
          const int h = is_v ? head - q_heads - kv_heads : head - q_heads;
          dst = (is_v ? v_cache : k_cache) + (cache_row + static_cast<long long>(h) * page_size) * DH + e0;
        }
      }
      Slice lo, hi;
      if (dst != nullptr) {
        lo = *reinterpret_cast<const Slice*>(src);
        hi = *reinterpret_cast<const Slice*>(src + HALF);
      }
      if (__all_sync(0xffffffffu, is_v || dst == nullptr)) {   // a warp of value heads only copies
        if (dst != nullptr) {
          *reinterpret_cast<Slice*>(dst) = lo;
          *reinterpret_cast<Slice*>(dst + HALF) = hi;
        }
        continue;
      }
      float a[Q], b[Q];
#pragma unroll
      for (int e = 0; e < Q; ++e) {
        a[e] = dst != nullptr ? Elem<T>::load(lo.v + e) : 0.0f;
        b[e] = dst != nullptr ? Elem<T>::load(hi.v + e) : 0.0f;
      }
      float ss = 0.0f;
#pragma unroll
      for (int e = 0; e < Q; ++e) ss += a[e] * a[e] + b[e] * b[e];
#pragma unroll
      for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (!is_v) {   // values are stored as they are
        if ((is_q ? qw : kw) != nullptr) {
          const float inv = 1.0f / sqrtf(ss / static_cast<float>(DH) + (is_q ? q_eps : k_eps));
          const float4 wl = is_q ? qw_lo : kw_lo, wh = is_q ? qw_hi : kw_hi;
          a[0] = (a[0] * inv) * wl.x, a[1] = (a[1] * inv) * wl.y, a[2] = (a[2] * inv) * wl.z, a[3] = (a[3] * inv) * wl.w;
          b[0] = (b[0] * inv) * wh.x, b[1] = (b[1] * inv) * wh.y, b[2] = (b[2] * inv) * wh.z, b[3] = (b[3] * inv) * wh.w;
        }
        if (inv_freq != nullptr) {
          const float cc[Q] = {c.x, c.y, c.z, c.w}, ssn[Q] = {sn.x, sn.y, sn.z, sn.w};
#pragma unroll
          for (int e = 0; e < Q; ++e) {
            const float x0 = a[e], x1 = b[e];
            a[e] = x0 * cc[e] - x1 * ssn[e];
            b[e] = x1 * cc[e] + x0 * ssn[e];
          }
        }
      }
      if (dst != nullptr) {
        Slice out_lo, out_hi;
#pragma unroll
        for (int e = 0; e < Q; ++e) {
          Elem<T>::store(out_lo.v + e, a[e]);
          Elem<T>::store(out_hi.v + e, b[e]);
        }
        *reinterpret_cast<Slice*>(dst) = out_lo;
        *reinterpret_cast<Slice*>(dst + HALF) = out_hi;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
template <typename T>
int launch_embed(const void* table, const int* ids, float* x, int tokens, int dim, int vocab, int k_block_rows, cudaStream_t s) {
  if (tokens == 0) return kOk;
  TIE_LAUNCH((embed_kernel<T>), tokens, dim >= 1024 ? 256 : 128, 0, s, static_cast<const T*>(table), ids, x, dim, vocab, k_block_rows);
  TIE_RETURN_LAUNCH("embed");
}

template <typename T>
int launch_add_rmsnorm(float* x, const void* delta, const float* part, long long part_stride, int splits,
                       const int* rows, const float* w, float eps, void* out, int n, int dim, cudaStream_t s) {
  if (n == 0) return kOk;
  const T* d = static_cast<const T*>(delta);
  T* o = static_cast<T*>(out);
  const bool aligned = dim % 4 == 0 && reinterpret_cast<uintptr_t>(x) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(out) % 16 == 0 && reinterpret_cast<uintptr_t>(delta) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(part) % 16 == 0 && part_stride % 4 == 0;
  if (aligned && dim <= 16384) {
    // few rows (decode): many threads per row keep the latency short; many rows: 256 threads per row
    const int pieces = dim / 4;
    int threads = n <= 512 ? 1024 : 256;
    while (threads < 1024 && pieces > 4 * threads) threads *= 2;
    while (threads > 32 && threads / 2 >= pieces) threads /= 2;
    const int nv = (pieces + threads - 1) / threads;
    if (nv <= 1) TIE_LAUNCH((add_rmsnorm_vec4_kernel<T, 1>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
    else if (nv <= 2) TIE_LAUNCH((add_rmsnorm_vec4_kernel<T, 2>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
    else TIE_LAUNCH((add_rmsnorm_vec4_kernel<T, 4>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
    TIE_RETURN_LAUNCH("add_rmsnorm");
  }
  const int threads = dim >= 4096 ? 1024 : (dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128));
  if (dim <= 4 * threads) TIE_LAUNCH((add_rmsnorm_kernel<T, 4>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
  else if (dim <= 16 * threads) TIE_LAUNCH((add_rmsnorm_kernel<T, 16>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
  else TIE_LAUNCH((add_rmsnorm_kernel<T, 0>), n, threads, 0, s, x, d, part, part_stride, splits, rows, w, eps, o, dim);
  TIE_RETURN_LAUNCH("add_rmsnorm");
}

template <typename T>
int launch_rmsnorm_rows(const void* x, long long xs, const float* w, float eps, void* out, long long os, int size,
                        long long n, cudaStream_t s) {
  if (n == 0) return kOk;
  TIE_LAUNCH((rmsnorm_rows_kernel<T>), ceil_div(n, 4), 128, 0, s, static_cast<const T*>(x), xs, w, eps, static_cast<T*>(out), os,
                                                         size, n);
  TIE_RETURN_LAUNCH("rmsnorm_rows");
}

template <typename T>
int launch_silu_mul(const void* gu, void* out, int tokens, int inter, cudaStream_t s) {
  const long long total = static_cast<long long>(tokens) * inter;
  if (total == 0) return kOk;
  TIE_LAUNCH((silu_mul_kernel<T>), ceil_div(total, 256), 256, 0, s, static_cast<const T*>(gu), static_cast<T*>(out), inter, total);
  TIE_RETURN_LAUNCH("silu_mul");
}

template <typename T>
int launch_rope(void* x, long long stride, const int* pos, const float* inv_freq, int tokens, int heads, int head_dim,
                int rot, cudaStream_t s) {
  const long long total = static_cast<long long>(tokens) * heads * (rot / 2);
  if (total == 0) return kOk;
  TIE_LAUNCH((rope_kernel<T>), ceil_div(total, 256), 256, 0, s, static_cast<T*>(x), stride, pos, inv_freq, heads, head_dim, rot,
                                                      total);
  TIE_RETURN_LAUNCH("rope");
}

template <typename T>
int launch_kv_append(const void* k, const void* v, long long ks, long long vs, const int* slots, void* kc, void* vc,
                     int tokens, int kv_heads, int head_dim, int page_size, cudaStream_t s) {
  const long long total = static_cast<long long>(tokens) * kv_heads * head_dim;
  if (total == 0) return kOk;
  TIE_LAUNCH((kv_append_kernel<T>), ceil_div(total, 256), 256, 0, s, static_cast<const T*>(k), static_cast<const T*>(v), ks, vs,
                                                           slots, static_cast<T*>(kc), static_cast<T*>(vc), kv_heads,
                                                           head_dim, page_size, total);
  TIE_RETURN_LAUNCH("kv_append");
}

template <typename T>
int launch_qk_norm_rope_append(void* qkv, long long stride, const float* part, long long part_stride, int splits,
                               long long part_ld, const float* qw, const float* kw, float q_eps, float k_eps,
                               const float* inv_freq, int rot, const int* pos, const int* slots, void* kc, void* vc,
                               int tokens, int q_heads, int kv_heads, int head_dim, int page_size, int write_kv,
                               cudaStream_t s) {
  const int heads_per_token = write_kv ? q_heads + 2 * kv_heads : q_heads;
  const long long total = static_cast<long long>(tokens) * heads_per_token;
  if (total == 0) return kOk;
  const int warps = 8;
  const int vec = head_dim / 32;
  const size_t slice = sizeof(T) * vec > 16 ? 16 : sizeof(T) * vec;
  const size_t fslice = sizeof(float) * vec > 16 ? 16 : sizeof(float) * vec;
  const bool part_ok = part == nullptr || (reinterpret_cast<uintptr_t>(part) % fslice == 0 && part_stride % vec == 0 && part_ld % vec == 0);
  const bool whole = part_ok && (head_dim == 64 || head_dim == 128 || head_dim == 256) && (inv_freq == nullptr || rot == head_dim) &&
                     stride % vec == 0 && reinterpret_cast<uintptr_t>(qkv) % slice == 0 && reinterpret_cast<uintptr_t>(kc) % slice == 0 &&
                     reinterpret_cast<uintptr_t>(vc) % slice == 0;
  // many tokens, nothing to sum: the kernel that issues the fewest instructions a head
  const size_t half_slice = sizeof(T) * 4;
  const bool rows = whole && part == nullptr && tokens >= 256 && stride % 4 == 0 && reinterpret_cast<uintptr_t>(qkv) % half_slice == 0 &&
                    reinterpret_cast<uintptr_t>(kc) % half_slice == 0 && reinterpret_cast<uintptr_t>(vc) % half_slice == 0 &&
                    reinterpret_cast<uintptr_t>(qw) % 16 == 0 && reinterpret_cast<uintptr_t>(kw) % 16 == 0;
  if (rows) {
    T* q = static_cast<T*>(qkv);
    T* k = static_cast<T*>(kc);
    T* v = static_cast<T*>(vc);
    // four tokens a block where there are blocks enough for every SM several times over: the weights are fetched once
#define TIE_QK_ROWS_OF(D, TOK)                                                                                                          \
  TIE_LAUNCH((qk_norm_rope_append_rows_kernel<T, D, TOK>), ceil_div(tokens, TOK), 256, 0, s, q, stride, qw, kw, q_eps, k_eps, inv_freq, pos, \
             slots, k, v, q_heads, kv_heads, page_size, heads_per_token, tokens)
#define TIE_QK_ROWS(D)                   \
  do {                                   \
    if (tokens >= 2048) {                \
      TIE_QK_ROWS_OF(D, 4);              \
    } else {                             \
      TIE_QK_ROWS_OF(D, 1);              \
    }                                    \
  } while (0)
    if (head_dim == 64) TIE_QK_ROWS(64);
    else if (head_dim == 128) TIE_QK_ROWS(128);
    else TIE_QK_ROWS(256);
#undef TIE_QK_ROWS
#undef TIE_QK_ROWS_OF
    TIE_RETURN_LAUNCH("qk_norm_rope_append");
  }
  if (whole) {
    const dim3 grid(tokens, ceil_div(heads_per_token, warps));
    T* q = static_cast<T*>(qkv);
    T* k = static_cast<T*>(kc);
    T* v = static_cast<T*>(vc);
    if (vec == 2) {
      TIE_LAUNCH((qk_norm_rope_append_vec_kernel<T, 2>), grid, warps * 32, 0, s, q, stride, part, part_stride, splits, part_ld, qw, kw, q_eps, k_eps, inv_freq, pos, slots, k, v,
                 q_heads, kv_heads, page_size, heads_per_token);
    } else if (vec == 4) {
      TIE_LAUNCH((qk_norm_rope_append_vec_kernel<T, 4>), grid, warps * 32, 0, s, q, stride, part, part_stride, splits, part_ld, qw, kw, q_eps, k_eps, inv_freq, pos, slots, k, v,
                 q_heads, kv_heads, page_size, heads_per_token);
    } else {
      TIE_LAUNCH((qk_norm_rope_append_vec_kernel<T, 8>), grid, warps * 32, 0, s, q, stride, part, part_stride, splits, part_ld, qw, kw, q_eps, k_eps, inv_freq, pos, slots, k, v,
                 q_heads, kv_heads, page_size, heads_per_token);
    }
    TIE_RETURN_LAUNCH("qk_norm_rope_append");
  }
  const size_t smem = (static_cast<size_t>(warps) * head_dim + rot) * sizeof(float);
  TIE_LAUNCH((qk_norm_rope_append_kernel<T>), dim3(tokens, ceil_div(heads_per_token, warps)), warps * 32, smem, s, 
      static_cast<T*>(qkv), stride, part, part_stride, splits, part_ld, qw, kw, q_eps, k_eps, inv_freq, rot, pos, slots,
      static_cast<T*>(kc),
      static_cast<T*>(vc), q_heads, kv_heads, head_dim, page_size, heads_per_token, total);
  TIE_RETURN_LAUNCH("qk_norm_rope_append");
}

}  // namespace tie

using namespace tie;

#define TIE_DISPATCH(dtype, call_f32, call_bf16)                       \
  do {                                                                 \
    if ((dtype) == TIE_F32) return call_f32;                           \
    if ((dtype) == TIE_BF16) return call_bf16;                         \
    set_error("unknown dtype code %d", (dtype));                       \
    return kBadArgument;                                               \
  } while (0)

// k_block_rows > 0: the table is stored in k-blocks of 64 columns, k_block_rows rows each (see embed_kernel).
TIE_API int tie_embed(int dtype, const void* table, const int* ids, float* x, int tokens, int dim, int vocab,
                      int k_block_rows, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && dim > 0 && vocab > 0 && (k_block_rows == 0 || k_block_rows >= vocab),
              "embed: bad sizes tokens=%d dim=%d vocab=%d (k-blocks of %d rows)", tokens, dim, vocab, k_block_rows);
  TIE_DISPATCH(dtype, launch_embed<float>(table, ids, x, tokens, dim, vocab, k_block_rows, s),
               launch_embed<__nv_bfloat16>(table, ids, x, tokens, dim, vocab, k_block_rows, s));
}

TIE_API int tie_scatter_ids(int* tokens, const int* dst, const int* src, const int* ids, int n, cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && tokens != nullptr && dst != nullptr && src != nullptr && ids != nullptr, "scatter_ids: bad arguments n=%d", n);
  if (n == 0) return kOk;
  TIE_LAUNCH(scatter_ids_kernel, ceil_div(n, 128), 128, 0, s, tokens, dst, src, ids, n);
  TIE_RETURN_LAUNCH("scatter_ids");
}

// rows may be null (row t of out from row t of x); delta may be null (no add), or given as
// `splits` float partial sums at part (then delta must be null).
TIE_API int tie_add_rmsnorm(int dtype, float* x, const void* delta, const float* part, long long part_stride,
                            int splits, const int* rows, const float* w, float eps, void* out, int n, int dim,
                            cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && dim > 0, "add_rmsnorm: bad sizes n=%d dim=%d", n, dim);
  TIE_REQUIRE(part == nullptr || (delta == nullptr && splits >= 1), "add_rmsnorm: give a delta or partial sums, not both");
  TIE_DISPATCH(dtype, launch_add_rmsnorm<float>(x, delta, part, part_stride, splits, rows, w, eps, out, n, dim, s),
               launch_add_rmsnorm<__nv_bfloat16>(x, delta, part, part_stride, splits, rows, w, eps, out, n, dim, s));
}

TIE_API int tie_rmsnorm_rows(int dtype, const void* x, long long x_stride, const float* w, float eps, void* out,
                             long long out_stride, int size, long long n, cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && size > 0, "rmsnorm_rows: bad sizes n=%lld size=%d", n, size);
  TIE_DISPATCH(dtype, launch_rmsnorm_rows<float>(x, x_stride, w, eps, out, out_stride, size, n, s),
               launch_rmsnorm_rows<__nv_bfloat16>(x, x_stride, w, eps, out, out_stride, size, n, s));
}

TIE_API int tie_silu_mul(int dtype, const void* gu, void* out, int tokens, int inter, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && inter > 0, "silu_mul: bad sizes tokens=%d inter=%d", tokens, inter);
  TIE_DISPATCH(dtype, launch_silu_mul<float>(gu, out, tokens, inter, s),
               launch_silu_mul<__nv_bfloat16>(gu, out, tokens, inter, s));
}

TIE_API int tie_rope(int dtype, void* x, long long stride, const int* pos, const float* inv_freq, int tokens,
                     int heads, int head_dim, int rot, cudaStream_t s) {
  TIE_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= head_dim, "rope: rotary dim %d must be even and at most head_dim %d",
              rot, head_dim);
  TIE_DISPATCH(dtype, launch_rope<float>(x, stride, pos, inv_freq, tokens, heads, head_dim, rot, s),
               launch_rope<__nv_bfloat16>(x, stride, pos, inv_freq, tokens, heads, head_dim, rot, s));
}

TIE_API int tie_kv_append(int dtype, const void* k, const void* v, long long k_stride, long long v_stride,
                          const int* slots, void* k_cache, void* v_cache, int tokens, int kv_heads, int head_dim,
                          int page_size, cudaStream_t s) {
  TIE_REQUIRE(kv_heads > 0 && head_dim > 0 && page_size > 0, "kv_append: bad geometry");
  TIE_DISPATCH(dtype, launch_kv_append<float>(k, v, k_stride, v_stride, slots, k_cache, v_cache, tokens, kv_heads,
                                              head_dim, page_size, s),
               launch_kv_append<__nv_bfloat16>(k, v, k_stride, v_stride, slots, k_cache, v_cache, tokens, kv_heads,
                                               head_dim, page_size, s));
}

TIE_API int tie_qk_norm_rope_append(int dtype, void* qkv, long long stride, const float* part, long long part_stride,
                                    int splits, long long part_ld, const float* qw, const float* kw,
                                    float q_eps, float k_eps, const float* inv_freq, int rot, const int* pos,
                                    const int* slots, void* k_cache, void* v_cache, int tokens, int q_heads,
                                    int kv_heads, int head_dim, int page_size, int write_kv, cudaStream_t s) {
  TIE_REQUIRE(q_heads > 0 && kv_heads > 0 && head_dim > 0 && page_size > 0, "qk_norm_rope_append: bad geometry");
  TIE_REQUIRE(head_dim <= 1024, "qk_norm_rope_append: head_dim %d above 1024", head_dim);
  TIE_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= head_dim,
              "qk_norm_rope_append: rotary dim %d must be even and at most head_dim %d", rot, head_dim);
  TIE_DISPATCH(dtype,
               launch_qk_norm_rope_append<float>(qkv, stride, part, part_stride, splits, part_ld, qw, kw, q_eps, k_eps,
                                                 inv_freq, rot, pos, slots, k_cache,
                                                 v_cache, tokens, q_heads, kv_heads, head_dim, page_size, write_kv, s),
               launch_qk_norm_rope_append<__nv_bfloat16>(qkv, stride, part, part_stride, splits, part_ld, qw, kw, q_eps,
                                                         k_eps, inv_freq, rot, pos, slots, k_cache, v_cache, tokens, q_heads, kv_heads, head_dim,
                                                         page_size, write_kv, s));
}
