// Picking the next token on the device: the first maximum (greedy), or a draw from
// softmax(logits / T) by inverse CDF with a Philox4x32-10 uniform keyed by the request's
// seed and the index of the generated token. One block per row of logits, a fixed block
// size and fixed segment boundaries, so a row's result never depends on the rows beside it.
//
// The reference samples on the host (src/sampling/sampler.cpp:18-81): greedy is the first
// maximum (ties go to the lowest id); otherwise logits are shifted by their maximum and
// scaled by 1/T before exp, and a uniform in [0, total) walks the candidates in id order.
// Its generator is std::mt19937_64 per sequence (src/engine/sequence.h:22); this engine's
// is counter-based so that a draw needs no state.
#include <math.h>

#include "common.cuh"

namespace tie {

constexpr int kSampleThreads = 1024;

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint64_t p0 = static_cast<uint64_t>(0xD2511F53u) * c[0];
    const uint64_t p1 = static_cast<uint64_t>(0xCD9E8D57u) * c[2];
    const uint32_t n0 = static_cast<uint32_t>(p1 >> 32) ^ c[1] ^ k0;
    const uint32_t n2 = static_cast<uint32_t>(p0 >> 32) ^ c[3] ^ k1;
    c[1] = static_cast<uint32_t>(p1);
    c[3] = static_cast<uint32_t>(p0);
    c[0] = n0;
    c[2] = n2;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

// (value, index) maximum with ties to the lower index.
__device__ __forceinline__ void arg_better(float& v, int& i, float ov, int oi) {
  if (ov > v || (ov == v && oi < i)) {
    v = ov;
    i = oi;
  }
}

__device__ __forceinline__ void block_argmax(float& v, int& i, float* sv, int* si) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    arg_better(v, i, ov, oi);
  }
  if (lane == 0) {
    sv[warp] = v;
    si[warp] = i;
  }
  __syncthreads();
  if (warp == 0) {
    const int nw = blockDim.x >> 5;
    v = lane < nw ? sv[lane] : -INFINITY;
    i = lane < nw ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, v, o);
      const int oi = __shfl_xor_sync(0xffffffffu, i, o);
      arg_better(v, i, ov, oi);
    }
    if (lane == 0) {
      sv[0] = v;
      si[0] = i;
    }
  }
  __syncthreads();
  v = sv[0];
  i = si[0];
}

// out[r] = sampled id of row r. inv_temperature[r] == 0 means greedy. A NaN logit never
// compares greater, so it is never chosen; rows are checked for NaN on the host only when the
// caller asks for the host sampler.
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const float* __restrict__ logits, long long row_stride,
                                                                int vocab, const float* __restrict__ inv_temperature,
                                                                const unsigned long long* __restrict__ seeds,
                                                                const unsigned long long* __restrict__ counters,
                                                                int* __restrict__ out) {
  pdl_sync();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float seg_sum[kSampleThreads];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* z = logits + static_cast<long long>(r) * row_stride;
  const int tid = threadIdx.x;

  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < vocab; i += kSampleThreads) arg_better(best, best_i, z[i], i);
  block_argmax(best, best_i, sv, si);
  const float inv_t = inv_temperature ? inv_temperature[r] : 0.0f;
  if (!(inv_t > 0.0f) || isinf(inv_t) || best == INFINITY) {  // greedy, or a certain token
    if (tid == 0) out[r] = best_i;
    return;
  }

  // Thread `tid` owns the contiguous ids [tid * seg, (tid + 1) * seg).
  const int seg = (vocab + kSampleThreads - 1) / kSampleThreads;
  const int begin = min(vocab, tid * seg), end = min(vocab, begin + seg);
  float mine = 0.0f;
  for (int i = begin; i < end; ++i) mine += expf((z[i] - best) * inv_t);
  seg_sum[tid] = mine;
  if (tid == 0) chosen = -1;
  __syncthreads();
  // Exclusive scan of the 1024 segment sums by warp 0: 32 per lane, then across lanes.
  if (tid < 32) {
    float local = 0.0f;
    for (int i = 0; i < 32; ++i) local += seg_sum[tid * 32 + i];
    float incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float n = __shfl_up_sync(0xffffffffu, incl, o);
      if (tid >= o) incl += n;
    }
    float run = incl - local;
    for (int i = 0; i < 32; ++i) {
      const float v = seg_sum[tid * 32 + i];
      seg_sum[tid * 32 + i] = run;  // exclusive prefix
      run += v;
    }
    if (tid == 31) sv[1] = run;  // total
  }
  __syncthreads();
  const float total = sv[1];
  uint32_t c[4] = {static_cast<uint32_t>(counters[r]), static_cast<uint32_t>(counters[r] >> 32), 0u, 0u};
  philox4x32_10(c, static_cast<uint32_t>(seeds[r]), static_cast<uint32_t>(seeds[r] >> 32));
  const float u = static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);
  const float target = u * total;
  const float start = seg_sum[tid];
  const float stop = tid + 1 < kSampleThreads ? seg_sum[tid + 1] : total;
  if (begin < end && target >= start && target < stop) {
    float run = start;
    int pick = end - 1;
    for (int i = begin; i < end; ++i) {
      run += expf((z[i] - best) * inv_t);
      if (target < run) {
        pick = i;
        break;
      }
    }
    chosen = pick;  // the ranges [start, stop) are disjoint: one writer
  }
  __syncthreads();
  if (tid == 0) out[r] = chosen >= 0 ? chosen : best_i;  // rounding left target at the very end
}

}  // namespace tie

using namespace tie;

TIE_API int tie_sample(const float* logits, long long row_stride, int rows, int vocab, const float* inv_temperature,
                       const unsigned long long* seeds, const unsigned long long* counters, int* out, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && vocab > 0, "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  TIE_REQUIRE(inv_temperature == nullptr || (seeds != nullptr && counters != nullptr),
              "sample: temperature sampling needs seeds and counters");
  if (rows == 0) return kOk;
  TIE_LAUNCH((sample_kernel), rows, kSampleThreads, 0, s, logits, row_stride, vocab, inv_temperature, seeds, counters, out);
  TIE_RETURN_LAUNCH("sample");
}
