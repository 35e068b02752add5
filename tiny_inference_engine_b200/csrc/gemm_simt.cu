// Matrix products on the CUDA cores: out[M, N] = a[M, K] . w[N, K]^T with float accumulation.
//
// These are the kernels of the true 32-bit path (float in, float out, FFMA only, no tensor
// cores and so no reduced-precision matrix mode), and they take every size; the bfloat16
// instantiations serve sizes that the tensor-core kernels refuse. The reference's
// counterpart is its dot-product matmul (src/backend/cpu/cpu_backend.cpp:78-139): weights
// in the checkpoint's [out, in] layout, y = x . W^T, no bias.
#include "common.cuh"
#include "launchers.h"

namespace tie {

// ---------------------------------------------------------------------------------------------
// Tiled kernel for any M, N, K: 64 x 64 output tile, 16-deep k slices, 256 threads, 4 x 4
// outputs per thread. Both operands are k-contiguous, so a slice is read along k and stored
// transposed in shared memory.
template <typename TI, typename TO>
__global__ void __launch_bounds__(256) gemm_tiled_kernel(const TI* __restrict__ a, const TI* __restrict__ w,
                                                         TO* __restrict__ out, int M, int N, int K, long long lda,
                                                         long long ldw, long long ldo) {
  pdl_sync();
  constexpr int BM = 64, BN = 64, BK = 16;
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  const int lr = tid / 4;        // row of the tile this thread loads (0..63)
  const int lk = (tid % 4) * 4;  // first of its 4 k's
  float acc[4][4] = {};

  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + lk + j;
      const int m = m0 + lr, n = n0 + lr;
      as[lk + j][lr] = (m < M && k < K) ? ld(a + static_cast<long long>(m) * lda + k) : 0.0f;
      ws[lk + j][lr] = (n < N && k < K) ? ld(w + static_cast<long long>(n) * ldw + k) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[4], wv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = as[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n < N) st(out + static_cast<long long>(m) * ldo + n, acc[i][j]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Few rows (decode): one warp per output column streams its weight row once with 16-byte
// loads and keeps MT accumulators; the MT activation rows come from L1/L2. Needs K to be a
// multiple of the 16-byte vector and 16-byte aligned rows.
template <typename TI, typename TO, int MT>
__global__ void __launch_bounds__(256) gemm_small_m_kernel(const TI* __restrict__ a, const TI* __restrict__ w,
                                                           TO* __restrict__ out, int M, int N, int K, long long lda,
                                                           long long ldw, long long ldo) {
  pdl_sync();
  constexpr int V = Vec16<TI>::N;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int m0 = blockIdx.y * MT;
  if (n >= N) return;
  const TI* wr = w + static_cast<long long>(n) * ldw;
  float acc[MT] = {};
  for (int k = lane * V; k < K; k += 32 * V) {
    Vec16<TI> wv;
    wv.load(wr + k);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (m0 + i < M) {
        Vec16<TI> av;
        av.load(a + static_cast<long long>(m0 + i) * lda + k);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[i] = fmaf(av.v[j], wv.v[j], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const float v = warp_sum(acc[i]);
    if (lane == 0 && m0 + i < M) st(out + static_cast<long long>(m0 + i) * ldo + n, v);
  }
}

template <typename TI, typename TO>
int launch_gemm(const void* a, const void* w, void* out, int M, int N, int K, long long lda, long long ldw,
                long long ldo, cudaStream_t s) {
  if (M == 0 || N == 0) return kOk;
  const TI* ap = static_cast<const TI*>(a);
  const TI* wp = static_cast<const TI*>(w);
  TO* op = static_cast<TO*>(out);
  constexpr int V = Vec16<TI>::N;
  const bool vec_ok = K % V == 0 && lda % V == 0 && ldw % V == 0 &&
                      reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0;
  if (M <= 16 && vec_ok) {
    const dim3 block(256);
    if (M <= 4) {
      TIE_LAUNCH((gemm_small_m_kernel<TI, TO, 4>), dim3(ceil_div(N, 8), 1), block, 0, s, ap, wp, op, M, N, K, lda, ldw, ldo);
    } else {
      TIE_LAUNCH((gemm_small_m_kernel<TI, TO, 8>), dim3(ceil_div(N, 8), ceil_div(M, 8)), block, 0, s, ap, wp, op, M, N, K, lda,
                                                                                            ldw, ldo);
    }
  } else {
    TIE_LAUNCH((gemm_tiled_kernel<TI, TO>), dim3(ceil_div(N, 64), ceil_div(M, 64)), 256, 0, s, ap, wp, op, M, N, K, lda, ldw, ldo);
  }
  TIE_RETURN_LAUNCH("gemm_simt");
}

}  // namespace tie

using namespace tie;

// in_dtype / out_dtype: TIE_F32 or TIE_BF16. Supported: f32->f32, bf16->bf16, bf16->f32.
// lda, ldw, ldo are row strides in elements.
TIE_API int tie_gemm_simt(int in_dtype, int out_dtype, const void* a, const void* w, void* out, int M, int N, int K,
                          long long lda, long long ldw, long long ldo, cudaStream_t s) {
  TIE_REQUIRE(M >= 0 && N >= 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
  TIE_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm: a row stride is smaller than the row");
  if (in_dtype == TIE_F32 && out_dtype == TIE_F32) return launch_gemm<float, float>(a, w, out, M, N, K, lda, ldw, ldo, s);
  if (in_dtype == TIE_BF16 && out_dtype == TIE_BF16)
    return launch_gemm<__nv_bfloat16, __nv_bfloat16>(a, w, out, M, N, K, lda, ldw, ldo, s);
  if (in_dtype == TIE_BF16 && out_dtype == TIE_F32)
    return launch_gemm<__nv_bfloat16, float>(a, w, out, M, N, K, lda, ldw, ldo, s);
  set_error("gemm: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
  return kBadArgument;
}
