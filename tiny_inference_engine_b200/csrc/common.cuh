// Shared device helpers: element types, 16-byte vectors, warp and block reductions.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tie {

// Error codes that launchers return to Python (0 = launched).
enum Status : int {
  kOk = 0,
  kBadArgument = 1,   // a size the kernel does not take; the message names it
  kCudaError = 2,     // cudaGetLastError() after the launch
};

// The last launcher message, read by tie_last_error().
void set_error(const char* fmt, ...);

template <typename T> struct Elem;
template <> struct Elem<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
};
template <> struct Elem<__nv_bfloat16> {
  static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
};

template <typename T> __device__ __forceinline__ float ld(const T* p) { return Elem<T>::load(p); }
template <typename T> __device__ __forceinline__ void st(T* p, float v) { Elem<T>::store(p, v); }

// 16 bytes of T, read and written with one instruction when the address allows it.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  float v[4];
  __device__ __forceinline__ void load(const float* p) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
  }
  __device__ __forceinline__ void store(float* p) const {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  float v[8];
  __device__ __forceinline__ void load(const __nv_bfloat16* p) {
    const uint4 t = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(w[i] << 16);
      v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
  __device__ __forceinline__ void store(__nv_bfloat16* p) const {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
      w[i] = *reinterpret_cast<const uint32_t*>(&h);
    }
    *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
  }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result. `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.0f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

inline int ceil_div(long long a, long long b) { return static_cast<int>((a + b - 1) / b); }

// Programmatic dependent launch. Every kernel of this library starts with pdl_sync(): it waits
// until the kernels before it in the stream have completed and their writes are visible,
// then lets the kernel after it be scheduled. So the next kernel's blocks are already resident
// (launch latency, block scheduling and whatever they do before their own pdl_sync() are hidden
// behind this kernel) and start the moment this one is done. Nothing may touch global memory
// before pdl_sync().
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_sync() {
  pdl_wait();
  pdl_launch_dependents();
}

bool pdl_enabled();   // false when the environment sets TIE_NO_PDL=1

template <typename... KArgs, typename... Args>
inline void launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr.val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = pdl_enabled() ? 1 : 0;
  cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);   // errors surface in cudaGetLastError()
}

}  // namespace tie

#define TIE_LAUNCH(kernel, grid, block, smem, stream, ...) \
  tie::launch_kernel(kernel, dim3(grid), dim3(block), smem, stream, __VA_ARGS__)

#define TIE_API extern "C" __attribute__((visibility("default")))

// Every launcher ends with this: a launch error becomes a status and a message.
#define TIE_RETURN_LAUNCH(name)                                              \
  do {                                                                       \
    const cudaError_t e_ = cudaGetLastError();                               \
    if (e_ != cudaSuccess) {                                                 \
      tie::set_error("%s: %s", name, cudaGetErrorString(e_));                \
      return tie::kCudaError;                                                \
    }                                                                        \
    return tie::kOk;                                                         \
  } while (0)

#define TIE_REQUIRE(cond, ...)                                               \
  do {                                                                       \
    if (!(cond)) {                                                           \
      tie::set_error(__VA_ARGS__);                                           \
      return tie::kBadArgument;                                              \
    }                                                                        \
  } while (0)

// dtype codes shared with ops/library.py
#define TIE_F32 0
#define TIE_BF16 1
