// Picking the next token on the device: the first maximum (greedy), or a draw from
// softmax(logits / T) by inverse CDF with a Philox4x32-10 uniform keyed by the request's
// seed and the index of the generated token. One block per row of logits, a fixed block
// size and fixed chunk boundaries, so a row's result never depends on the rows beside it.
//
// The reference samples on the host (src/sampling/sampler.cpp:18-81): greedy is the first
// maximum (ties go to the lowest id); otherwise logits are shifted by their maximum and
// scaled by 1/T before exp, and a uniform in [0, total) walks the candidates in id order.
// Its generator is std::mt19937_64 per sequence (src/engine/sequence.h:22); this engine's
// is counter-based so that a draw needs no state.
#include <cooperative_groups.h>
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

// What the kernels answer for a row that cannot be sampled: one with a NaN among its logits, or with
// no value above -inf. The reference's sampler raises for both (src/sampling/sampler.cpp:18-26); here the
// refusal travels with the ids, and whoever reads them ends that request (the rows beside it are sampled).
constexpr int kUnsamplable = -2;

// out[r] = sampled id of row r, or kUnsamplable. inv_temperature[r] == 0 means greedy.
__global__ void __launch_bounds__(kSampleThreads) sample_kernel(const float* __restrict__ logits, long long row_stride,
                                                                int vocab, const float* __restrict__ inv_temperature,
                                                                const unsigned long long* __restrict__ seeds,
                                                                const unsigned long long* __restrict__ counters,
                                                                int* __restrict__ out) {
  pdl_sync();
  __shared__ float sv[32];
  __shared__ int si[32];
  __shared__ float seg_sum[32];
  __shared__ float batch_sum[32][64];
  __shared__ int chosen;
  const int r = blockIdx.x;
  const float* z = logits + static_cast<long long>(r) * row_stride;
  const int tid = threadIdx.x;

  float best = -INFINITY;
  int best_i = 0x7fffffff;
  int nan_seen = 0;
  // eight loads in flight per thread: one block reads the row, so what bounds it is the latency of its loads
  for (int i0 = tid; i0 < vocab; i0 += 8 * kSampleThreads) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * kSampleThreads;
      v[j] = i < vocab ? z[i] : -INFINITY;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j * kSampleThreads;
      nan_seen |= v[j] != v[j];
      if (i < vocab) arg_better(best, best_i, v[j], i);
    }
  }
  block_argmax(best, best_i, sv, si);
  if (__syncthreads_or(nan_seen) || best == -INFINITY) {   // a NaN somewhere, or nothing finite to choose from
    if (tid == 0) out[r] = kUnsamplable;
    return;
  }
  const float inv_t = inv_temperature ? inv_temperature[r] : 0.0f;
  if (!(inv_t > 0.0f) || isinf(inv_t) || best == INFINITY) {  // greedy, or a certain token
    if (tid == 0) out[r] = best_i;
    return;
  }

  // Warp w owns the contiguous ids [w * chunk, (w + 1) * chunk) and reads them in batches of 256 * m ids
  // (32 lanes x 8 loads in flight, m times; m = 1 up to 524,288 ids), keeping each batch's weight. The chunks'
  // weights are scanned; the warp whose chunk holds the target finds the batch among its (at most 64) batch
  // weights and reads only that batch again, 32 ids a step, for the id at which the running weight passes.
  const int lane = tid & 31, warp = tid >> 5;
  const int chunk = ((vocab + kSampleThreads - 1) / kSampleThreads) * 32;
  const int m = (chunk + 64 * 256 - 1) / (64 * 256);
  const int batch = 256 * m;
  const int begin = min(vocab, warp * chunk), end = min(vocab, begin + chunk);
  float chunk_sum = 0.0f;
  for (int b0 = begin, nb = 0; b0 < end; b0 += batch, ++nb) {
    float mine = 0.0f;
    for (int i0 = b0 + lane; i0 < min(end, b0 + batch); i0 += 256) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = i0 + 32 * j < min(end, b0 + batch) ? z[i0 + 32 * j] : -INFINITY;
#pragma unroll
      for (int j = 0; j < 8; ++j) mine += i0 + 32 * j < min(end, b0 + batch) ? expf((v[j] - best) * inv_t) : 0.0f;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if (lane == 0) batch_sum[warp][nb] = mine;
    chunk_sum += mine;
  }
  if (lane == 0) seg_sum[warp] = chunk_sum;
  if (tid == 0) chosen = -1;
  __syncthreads();
  // every warp scans the 32 chunk sums itself
  const float own = seg_sum[lane];
  float incl = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  const float total = __shfl_sync(0xffffffffu, incl, 31);
  uint32_t c[4] = {static_cast<uint32_t>(counters[r]), static_cast<uint32_t>(counters[r] >> 32), 0u, 0u};
  philox4x32_10(c, static_cast<uint32_t>(seeds[r]), static_cast<uint32_t>(seeds[r] >> 32));
  const float u = static_cast<float>(c[0] >> 8) * (1.0f / 16777216.0f);
  const float target = u * total;
  const float start = __shfl_sync(0xffffffffu, incl - own, warp);   // the weight before this warp's chunk
  const float stop = warp == 31 ? total : __shfl_sync(0xffffffffu, incl, warp);
  if (begin < end && target >= start && target < stop) {   // the ranges [start, stop) are disjoint: one warp
    float run = start;
    int b0 = begin;
    for (int nb = 0; b0 + batch < end; b0 += batch, ++nb) {   // the last batch takes what rounding leaves over
      const float w = batch_sum[warp][nb];
      if (target < run + w) break;
      run += w;
    }
    const int b1 = min(end, b0 + batch);
    int pick = b1 - 1;
    for (int i0 = b0; i0 < b1; i0 += 256) {
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = i0 + 32 * j + lane < b1 ? z[i0 + 32 * j + lane] : -INFINITY;
      bool found = false;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int i = i0 + 32 * j + lane;
        float in = i < b1 ? expf((v[j] - best) * inv_t) : 0.0f;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const float n = __shfl_up_sync(0xffffffffu, in, o);
          if (lane >= o) in += n;
        }
        const unsigned int passed = __ballot_sync(0xffffffffu, i < b1 && target < run + in);
        if (passed && !found) {
          pick = i0 + 32 * j + __ffs(passed) - 1;
          found = true;
        }
        run += __shfl_sync(0xffffffffu, in, 31);
      }
      if (found) break;
    }
    if (lane == 0) chosen = pick;
  }
  __syncthreads();
  if (tid == 0) out[r] = chosen >= 0 ? chosen : best_i;  // rounding left target at the very end
}


// ---------------------------------------------------------------------------------------------
// Top-k and top-p (src/sampling/sampler.cpp:33-81): the candidates are taken most likely first,
// ties by id; top_k keeps the first k of them; top_p then keeps the smallest prefix whose weight
// reaches top_p of the kept weight; the uniform draw walks the kept prefix in that order.
//
// Nothing is sorted as a whole. Every id has one place in the order, its 64-bit key
// (descending value, id), and each of the three questions (the k-th key; the key at which the
// running weight reaches a share of the total; the key at which it passes the draw) is a
// selection: seven passes over the row, one byte of the key per pass, each a histogram of counts
// or of weights over the ids that still match the bytes found so far. Weights are summed as
// 44-bit fixed-point integers so that a sum does not depend on the order of its additions.
// With top_k up to 1,024 the kept keys are gathered and sorted in shared memory instead, and
// their weights are summed in double precision in order.
constexpr int kFilterThreads = 1024;
constexpr int kFilterWarps = kFilterThreads / 32;
constexpr int kSortMax = 1024;
constexpr double kWeightScale = 17592186044416.0;   // 2^44

struct FilterShared {
  unsigned long long wgt[kFilterWarps][256];   // one histogram per warp; the sorted candidates and their sums reuse it
  unsigned int cnt[kFilterWarps][256];
  unsigned long long tot[256];
  unsigned long long prefix, above, target, total;
  float sv[32];
  int si[32];
  int n;
};

__device__ __forceinline__ float scaled_logit(float z, float best, float inv_t) {
  float s = (z - best) * inv_t;
  if (!(s == s)) s = -INFINITY;   // a NaN logit is never chosen
  return s == 0.0f ? 0.0f : s;    // -0 and +0 are one value
}

// Larger values get smaller keys; equal values equal keys.
__device__ __forceinline__ uint32_t descending_key(float s) {
  const uint32_t b = __float_as_uint(s);
  return ~((b & 0x80000000u) ? ~b : (b | 0x80000000u));
}

__device__ __forceinline__ float value_of_key(uint32_t k) {
  const uint32_t asc = ~k;
  return __uint_as_float((asc & 0x80000000u) ? (asc & 0x7fffffffu) : ~asc);
}

__device__ __forceinline__ unsigned long long fixed_weight(float s) {
  return static_cast<unsigned long long>(__double2ull_rn(static_cast<double>(expf(s)) * kWeightScale));
}

template <bool WEIGHTED>
__device__ __forceinline__ void histogram_add(unsigned int* cnt, unsigned long long* wgt, unsigned int bin, unsigned int count,
                                              unsigned long long weight) {
  if (WEIGHTED) atomicAdd(wgt + bin, weight);
  else atomicAdd(cnt + bin, count);
}

// After a pass, by warp 0: the byte at which the running sum reaches the target. `first` fixes the
// target from the total of this first pass. tot[256] holds the pass's sums; prefix, above, target
// and total are the selection's state (shared memory).
__device__ __forceinline__ void choose_byte(const unsigned long long* tot, bool first, bool weighted, unsigned long long count,
                                            double share, bool strict, int shift, unsigned long long prefix,
                                            unsigned long long* s_prefix, unsigned long long* s_above,
                                            unsigned long long* s_target, unsigned long long* s_total) {
  const int lane = threadIdx.x & 31;
  unsigned long long t[8], mine = 0;
#pragma unroll
  for (int b = 0; b < 8; ++b) {
    t[b] = tot[lane * 8 + b];
    mine += t[b];
  }
  unsigned long long incl = mine;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const unsigned long long n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  const unsigned long long total = __shfl_sync(0xffffffffu, incl, 31);
  unsigned long long target = *s_target;
  if (first) {
    target = count;
    if (weighted) {
      const double x = share * static_cast<double>(total);
      target = strict ? static_cast<unsigned long long>(floor(x)) + 1ull : static_cast<unsigned long long>(ceil(x));
    }
    target = max(1ull, min(target, total));
  }
  const unsigned long long above = *s_above;
  __syncwarp();
  const unsigned int reached = __ballot_sync(0xffffffffu, mine != 0ull && above + incl >= target);
  const unsigned int occupied = __ballot_sync(0xffffffffu, mine != 0ull);
  // the first lane whose bytes reach the target, else (rounding left the target beyond the end) the last one that holds anything
  const int owner = reached ? __ffs(reached) - 1 : (occupied ? 31 - __clz(occupied) : 0);
  if (lane == owner) {
    unsigned long long run = above + incl - mine;
    int pick = 0;
#pragma unroll
    for (int b = 0; b < 8; ++b) {
      if (t[b] == 0ull) continue;
      pick = b;
      if (run + t[b] >= target) break;
      run += t[b];
    }
    *s_above = run;
    *s_prefix = prefix | (static_cast<unsigned long long>(lane * 8 + pick) << shift);
    if (first) {
      *s_target = target;
      *s_total = total;
    }
  }
}


// One pass: sh.tot[b] = number (or weight) of the ids whose key is at most `limit`, agrees with
// `prefix` above byte `shift / 8` and has b in that byte.
template <bool WEIGHTED>
__device__ void filter_pass(const float* __restrict__ z, int vocab, float best, float inv_t, unsigned long long limit,
                            unsigned long long prefix, int shift, FilterShared& sh) {
  const int tid = threadIdx.x, warp = tid >> 5;
  for (int i = tid; i < kFilterWarps * 256; i += kFilterThreads) {
    if (WEIGHTED) (&sh.wgt[0][0])[i] = 0ull;
    else (&sh.cnt[0][0])[i] = 0u;
  }
  __syncthreads();
  const unsigned long long above_mask = shift >= 56 ? 0ull : ~0ull << (shift + 8);
  // A thread adds up runs of its ids that fall into the same byte before it touches the histogram.
  unsigned int run_bin = 0xffffffffu, run_count = 0;
  unsigned long long run_weight = 0;
#pragma unroll 4
  for (int i = tid; i < vocab; i += kFilterThreads) {
    const float s = scaled_logit(z[i], best, inv_t);
    const unsigned long long key = (static_cast<unsigned long long>(descending_key(s)) << 32) | static_cast<unsigned int>(i);
    if (key > limit || ((key ^ prefix) & above_mask) != 0) continue;
    const unsigned int bin = static_cast<unsigned int>(key >> shift) & 255u;
    if (bin != run_bin) {
      if (run_count) histogram_add<WEIGHTED>(sh.cnt[warp], sh.wgt[warp], run_bin, run_count, run_weight);
      run_bin = bin;
      run_count = 0;
      run_weight = 0;
    }
    run_count += 1;
    if (WEIGHTED) run_weight += fixed_weight(s);
  }
  if (run_count) histogram_add<WEIGHTED>(sh.cnt[warp], sh.wgt[warp], run_bin, run_count, run_weight);
  __syncthreads();
  if (tid < 256) {
    unsigned long long t = 0;
    for (int w2 = 0; w2 < kFilterWarps; ++w2) t += WEIGHTED ? sh.wgt[w2][tid] : sh.cnt[w2][tid];
    sh.tot[tid] = t;
  }
  __syncthreads();
}

// The smallest key X, among the ids with key <= limit, at which the running count (weight) of
// the ids up to and including X reaches the target. The target is `count` itself, or for
// weights ceil(share * total), or floor(share * total) + 1 with `strict` (the running weight
// must pass share * total). Leaves X in sh.prefix, the running sum before X in sh.above and
// the sum over all ids within the limit in sh.total.
template <bool WEIGHTED>
__device__ void filter_select(const float* __restrict__ z, int vocab, float best, float inv_t, unsigned long long limit,
                              unsigned long long count, double share, bool strict, FilterShared& sh) {
  if (threadIdx.x == 0) {
    sh.prefix = 0ull;
    sh.above = 0ull;
  }
  const int shifts[7] = {56, 48, 40, 32, 16, 8, 0};   // ids are below 2^24
  for (int p = 0; p < 7; ++p) {
    __syncthreads();
    const unsigned long long prefix = sh.prefix;
    filter_pass<WEIGHTED>(z, vocab, best, inv_t, limit, prefix, shifts[p], sh);
    if (threadIdx.x < 32)
      choose_byte(sh.tot, p == 0, WEIGHTED, count, share, strict, shifts[p], prefix, &sh.prefix, &sh.above, &sh.target, &sh.total);
  }
  __syncthreads();
}

__device__ __forceinline__ double warp_shfl_up_double(double v, int o) { return __shfl_up_sync(0xffffffffu, v, o); }

// Rows with top_k[r] in (0, vocab) or top_p[r] < 1 and a temperature: out[r] is overwritten with
// the filtered draw (the plain kernel has written the unfiltered one). Other rows are left alone,
// and so are rows that the plain kernel refused (kUnsamplable).
__global__ void __launch_bounds__(kFilterThreads) sample_filtered_kernel(const float* __restrict__ logits, long long row_stride,
                                                                         int vocab, const float* __restrict__ inv_temperature,
                                                                         const int* __restrict__ top_k,
                                                                         const float* __restrict__ top_p,
                                                                         const unsigned long long* __restrict__ seeds,
                                                                         const unsigned long long* __restrict__ counters,
                                                                         int* __restrict__ out) {
  pdl_sync();
  extern __shared__ __align__(16) unsigned char filter_smem[];
  FilterShared& sh = *reinterpret_cast<FilterShared*>(filter_smem);
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float inv_t = inv_temperature[r];
  const int k = top_k[r];
  const float p = top_p[r];
  const bool by_k = k > 0 && k < vocab, by_p = p < 1.0f;
  if (!(inv_t > 0.0f) || isinf(inv_t) || (!by_k && !by_p)) return;   // greedy or unfiltered: the plain kernel's id stands
  if (out[r] == kUnsamplable) return;                                 // the plain kernel refused the row: so does this one
  const float* z = logits + static_cast<long long>(r) * row_stride;
  float best = -INFINITY;
  int best_i = 0x7fffffff;
  for (int i = tid; i < vocab; i += kFilterThreads) arg_better(best, best_i, z[i], i);
  block_argmax(best, best_i, sh.sv, sh.si);
  if (best == INFINITY || best == -INFINITY) return;                  // a certain token (or nothing to weigh): the first maximum stands

  uint32_t c[4] = {static_cast<uint32_t>(counters[r]), static_cast<uint32_t>(counters[r] >> 32), 0u, 0u};
  philox4x32_10(c, static_cast<uint32_t>(seeds[r]), static_cast<uint32_t>(seeds[r] >> 32));
  const double u = static_cast<double>(c[0] >> 8) * (1.0 / 16777216.0);

  unsigned long long limit = ~0ull;
  if (by_k) {
    filter_select<false>(z, vocab, best, inv_t, limit, static_cast<unsigned long long>(k), 0.0, false, sh);
    limit = sh.prefix;   // the k-th key
  }
  if (by_k && k <= kSortMax) {
    // The kept keys, sorted; their weights summed in order in double precision.
    unsigned long long* cand = &sh.wgt[0][0];
    double* cum = reinterpret_cast<double*>(cand + kSortMax);
    __syncthreads();
    if (tid == 0) sh.n = 0;
    cand[tid] = ~0ull;
    __syncthreads();
    for (int i = tid; i < vocab; i += kFilterThreads) {
      const float s = scaled_logit(z[i], best, inv_t);
      const unsigned long long key = (static_cast<unsigned long long>(descending_key(s)) << 32) | static_cast<unsigned int>(i);
      if (key <= limit) {
        const int at = atomicAdd(&sh.n, 1);
        if (at < kSortMax) cand[at] = key;
      }
    }
    __syncthreads();
    for (int size = 2; size <= kSortMax; size <<= 1) {
      for (int j = size >> 1; j > 0; j >>= 1) {
        const int other = tid ^ j;
        if (other > tid) {
          const unsigned long long a = cand[tid], b = cand[other];
          if ((a > b) == ((tid & size) == 0)) {
            cand[tid] = b;
            cand[other] = a;
          }
        }
        __syncthreads();
      }
    }
    if (warp == 0) {
      const int n = min(sh.n, kSortMax);
      const int begin = min(n, lane * 32), end = min(n, begin + 32);
      double local = 0.0;
      for (int j = begin; j < end; ++j) {
        local += static_cast<double>(expf(value_of_key(static_cast<uint32_t>(cand[j] >> 32))));
        cum[j] = local;
      }
      double incl = local;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double t = warp_shfl_up_double(incl, o);
        if (lane >= o) incl += t;
      }
      const double before = incl - local;
      for (int j = begin; j < end; ++j) cum[j] += before;
      __syncwarp();
      double total = __shfl_sync(0xffffffffu, incl, 31);
      int keep = n;
      if (by_p) {
        const double target = static_cast<double>(p) * total;
        int first = n;
        for (int j = begin; j < end; ++j) {
          if (cum[j] >= target) {
            first = j;
            break;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
        keep = min(first + 1, n);
        total = cum[keep - 1];
      }
      const double draw = u * total;
      int first = keep - 1;
      for (int j = begin; j < min(end, keep); ++j) {
        if (cum[j] > draw) {
          first = j;
          break;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
      if (lane == 0) out[r] = static_cast<int>(cand[first] & 0xffffffffull);
    }
    return;
  }
  if (by_p) {
    filter_select<true>(z, vocab, best, inv_t, limit, 0ull, static_cast<double>(p), false, sh);
    limit = sh.prefix;   // the last key of the kept prefix
  }
  filter_select<true>(z, vocab, best, inv_t, limit, 0ull, u, true, sh);
  if (tid == 0) out[r] = static_cast<int>(sh.prefix & 0xffffffffull);
}


// ---------------------------------------------------------------------------------------------
// The same on a cluster of eight CTAs for a row, for vocabularies whose keys fit into the
// eight CTAs' shared memory (about 400,000 ids): the keys are made once, so the seven passes of
// a selection read shared memory only; each CTA counts into its own histogram and all of them
// add the eight histograms up through distributed shared memory (two histograms used in turn:
// one cluster barrier a pass). The kernel above stays for larger vocabularies.
constexpr int kClusterCtas = 8;

struct ClusterShared {
  unsigned long long wgt[2][256];
  unsigned int cnt[2][256];
  unsigned long long tot[256];
  unsigned long long prefix, above, target, total;
  unsigned long long cand[kSortMax];   // CTA 0: the kept keys, sorted
  double cum[kSortMax];
  float sv[32];
  int si[32];
  float best_v;
  int best_i;
  int n;
  int pass;                            // passes so far: picks the histogram
};

// keys[e * kFilterThreads + tid] = descending_key of id (e * kClusterCtas + rank) * kFilterThreads + tid, for e < E
template <bool WEIGHTED>
__device__ void cluster_select(const uint32_t* keys, int E, int vocab, int rank, unsigned long long limit, unsigned long long count,
                               double share, bool strict, ClusterShared& sh) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  const int tid = threadIdx.x;
  if (tid == 0) {
    sh.prefix = 0ull;
    sh.above = 0ull;
  }
  const int shifts[7] = {56, 48, 40, 32, 16, 8, 0};   // ids are below 2^24
  for (int p = 0; p < 7; ++p) {
    __syncthreads();
    const unsigned long long prefix = sh.prefix;
    const int buf = sh.pass & 1;
    __syncthreads();
    if (tid == 0) sh.pass += 1;
    if (tid < 256) {
      sh.wgt[buf][tid] = 0ull;
      sh.cnt[buf][tid] = 0u;
    }
    __syncthreads();
    const int shift = shifts[p];
    const unsigned long long above_mask = shift >= 56 ? 0ull : ~0ull << (shift + 8);
    // A thread adds up runs of its ids that fall into the same byte before it touches the histogram: early
    // bytes take few values, so most threads add once.
    unsigned int run_bin = 0xffffffffu, run_count = 0;
    unsigned long long run_weight = 0;
#pragma unroll 4
    for (int e = 0; e < E; ++e) {
      const int id = (e * kClusterCtas + rank) * kFilterThreads + tid;
      const uint32_t value_key = keys[e * kFilterThreads + tid];
      const unsigned long long key = (static_cast<unsigned long long>(value_key) << 32) | static_cast<unsigned int>(id);
      const bool in = id < vocab && key <= limit && ((key ^ prefix) & above_mask) == 0;
      if (!in) continue;
      const unsigned int bin = static_cast<unsigned int>(key >> shift) & 255u;
      if (bin != run_bin) {
        if (run_count) histogram_add<WEIGHTED>(sh.cnt[buf], sh.wgt[buf], run_bin, run_count, run_weight);
        run_bin = bin;
        run_count = 0;
        run_weight = 0;
      }
      run_count += 1;
      if (WEIGHTED) run_weight += fixed_weight(value_of_key(value_key));
    }
    if (run_count) histogram_add<WEIGHTED>(sh.cnt[buf], sh.wgt[buf], run_bin, run_count, run_weight);
    cluster.sync();   // every CTA's histogram of this pass is complete
    if (tid < 256) {
      unsigned long long t = 0;
      for (int c = 0; c < kClusterCtas; ++c) {
        const ClusterShared* other = cluster.map_shared_rank(&sh, c);
        t += WEIGHTED ? other->wgt[buf][tid] : other->cnt[buf][tid];
      }
      sh.tot[tid] = t;
    }
    __syncthreads();
    if (tid < 32)   // the same in every CTA
      choose_byte(sh.tot, p == 0, WEIGHTED, count, share, strict, shift, prefix, &sh.prefix, &sh.above, &sh.target, &sh.total);
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kFilterThreads, 1) sample_filtered_cluster_kernel(const float* __restrict__ logits, long long row_stride,
                                                                                    int vocab, int E, const float* __restrict__ inv_temperature,
                                                                                    const int* __restrict__ top_k,
                                                                                    const float* __restrict__ top_p,
                                                                                    const unsigned long long* __restrict__ seeds,
                                                                                    const unsigned long long* __restrict__ counters,
                                                                                    int* __restrict__ out) {
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  __shared__ ClusterShared sh;
  extern __shared__ uint32_t keys[];   // [E][kFilterThreads]
  const int rank = static_cast<int>(cluster.block_rank());
  const int r = blockIdx.x / kClusterCtas, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const float inv_t = inv_temperature[r];
  const int k = top_k[r];
  const float p = top_p[r];
  const bool by_k = k > 0 && k < vocab, by_p = p < 1.0f;
  if (!(inv_t > 0.0f) || isinf(inv_t) || (!by_k && !by_p)) return;   // the whole cluster: the plain kernel's id stands
  if (out[r] == kUnsamplable) return;                                 // the plain kernel refused the row (every CTA reads the same word)
  const float* z = logits + static_cast<long long>(r) * row_stride;

  // the row's maximum: each CTA over its ids, then the eight results in rank order
  float best = -INFINITY;
  int best_i = 0x7fffffff;
#pragma unroll 4
  for (int e = 0; e < E; ++e) {
    const int id = (e * kClusterCtas + rank) * kFilterThreads + tid;
    const float v = id < vocab ? z[id] : -INFINITY;
    keys[e * kFilterThreads + tid] = __float_as_uint(v);   // the logit itself until the maximum is known
    if (id < vocab) arg_better(best, best_i, v, id);
  }
  block_argmax(best, best_i, sh.sv, sh.si);
  if (tid == 0) {
    sh.best_v = best;
    sh.best_i = best_i;
    sh.pass = 0;
  }
  cluster.sync();
  best = -INFINITY;
  best_i = 0x7fffffff;
  for (int c = 0; c < kClusterCtas; ++c) {
    const ClusterShared* other = cluster.map_shared_rank(&sh, c);
    arg_better(best, best_i, other->best_v, other->best_i);
  }
  // No CTA may leave while another still reads its shared memory: every path below ends with a cluster barrier.
  if (best == INFINITY || best == -INFINITY) {   // a certain token (or nothing to weigh): the first maximum stands
    cluster.sync();
    return;
  }
  for (int e = 0; e < E; ++e) {   // a thread reads back what it wrote itself
    const int id = (e * kClusterCtas + rank) * kFilterThreads + tid;
    const float v = __uint_as_float(keys[e * kFilterThreads + tid]);
    keys[e * kFilterThreads + tid] = id < vocab ? descending_key(scaled_logit(v, best, inv_t)) : 0xffffffffu;
  }

  uint32_t c4[4] = {static_cast<uint32_t>(counters[r]), static_cast<uint32_t>(counters[r] >> 32), 0u, 0u};
  philox4x32_10(c4, static_cast<uint32_t>(seeds[r]), static_cast<uint32_t>(seeds[r] >> 32));
  const double u = static_cast<double>(c4[0] >> 8) * (1.0 / 16777216.0);

  unsigned long long limit = ~0ull;
  if (by_k) {
    cluster_select<false>(keys, E, vocab, rank, limit, static_cast<unsigned long long>(k), 0.0, false, sh);
    limit = sh.prefix;   // the k-th key
  }
  if (by_k && k <= kSortMax) {
    // The kept keys go to CTA 0, which sorts them and sums their weights in order in double precision.
    ClusterShared* first = cluster.map_shared_rank(&sh, 0);
    if (rank == 0) {
      if (tid == 0) sh.n = 0;
      sh.cand[tid] = ~0ull;
    }
    cluster.sync();
    for (int e = 0; e < E; ++e) {
      const int id = (e * kClusterCtas + rank) * kFilterThreads + tid;
      const unsigned long long key = (static_cast<unsigned long long>(keys[e * kFilterThreads + tid]) << 32) | static_cast<unsigned int>(id);
      if (id < vocab && key <= limit) {
        const int at = atomicAdd(&first->n, 1);
        if (at < kSortMax) first->cand[at] = key;
      }
    }
    cluster.sync();   // the last access to another CTA's memory
    if (rank != 0) return;
    unsigned long long* cand = sh.cand;
    double* cum = sh.cum;
    for (int size = 2; size <= kSortMax; size <<= 1) {
      for (int j = size >> 1; j > 0; j >>= 1) {
        const int other = tid ^ j;
        if (other > tid) {
          const unsigned long long a = cand[tid], b = cand[other];
          if ((a > b) == ((tid & size) == 0)) {
            cand[tid] = b;
            cand[other] = a;
          }
        }
        __syncthreads();
      }
    }
    if (warp == 0) {
      const int n = min(sh.n, kSortMax);
      const int begin = min(n, lane * 32), end = min(n, begin + 32);
      double local = 0.0;
      for (int j = begin; j < end; ++j) {
        local += static_cast<double>(expf(value_of_key(static_cast<uint32_t>(cand[j] >> 32))));
        cum[j] = local;
      }
      double incl = local;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const double t = warp_shfl_up_double(incl, o);
        if (lane >= o) incl += t;
      }
      const double before = incl - local;
      for (int j = begin; j < end; ++j) cum[j] += before;
      __syncwarp();
      double total = __shfl_sync(0xffffffffu, incl, 31);
      int keep = n;
      if (by_p) {
        const double target = static_cast<double>(p) * total;
        int at = n;
        for (int j = begin; j < end; ++j) {
          if (cum[j] >= target) {
            at = j;
            break;
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) at = min(at, __shfl_xor_sync(0xffffffffu, at, o));
        keep = min(at + 1, n);
        total = cum[keep - 1];
      }
      const double draw = u * total;
      int at = keep - 1;
      for (int j = begin; j < min(end, keep); ++j) {
        if (cum[j] > draw) {
          at = j;
          break;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) at = min(at, __shfl_xor_sync(0xffffffffu, at, o));
      if (lane == 0) out[r] = static_cast<int>(cand[at] & 0xffffffffull);
    }
    return;
  }
  if (by_p) {
    cluster_select<true>(keys, E, vocab, rank, limit, 0ull, static_cast<double>(p), false, sh);
    limit = sh.prefix;   // the last key of the kept prefix
  }
  cluster_select<true>(keys, E, vocab, rank, limit, 0ull, u, true, sh);
  if (rank == 0 && tid == 0) out[r] = static_cast<int>(sh.prefix & 0xffffffffull);
  cluster.sync();
}

constexpr int kClusterMaxE = 48;   // 192 KB of keys per CTA

static int launch_filtered_cluster(const float* logits, long long row_stride, int rows, int vocab, const float* inv_temperature,
                                   const int* top_k, const float* top_p, const unsigned long long* seeds,
                                   const unsigned long long* counters, int* out, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_filtered_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             kClusterMaxE * kFilterThreads * 4) != cudaSuccess) {
      set_error("sample: cannot reserve %d bytes of shared memory", kClusterMaxE * kFilterThreads * 4);
      return kCudaError;
    }
    configured = true;
  }
  const int E = ceil_div(vocab, kClusterCtas * kFilterThreads);
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(kClusterCtas * rows);
  cfg.blockDim = dim3(kFilterThreads);
  cfg.dynamicSmemBytes = static_cast<size_t>(E) * kFilterThreads * 4;
  cfg.stream = s;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeClusterDimension;   // clusters only: the kernel starts when the one ahead is done
  attrs[0].val.clusterDim.x = kClusterCtas;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  cudaLaunchKernelEx(&cfg, sample_filtered_cluster_kernel, logits, row_stride, vocab, E, inv_temperature, top_k, top_p, seeds,
                     counters, out);
  TIE_RETURN_LAUNCH("sample_filtered");
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

// Overwrites out[r] for the rows that filter (top_k[r] in (0, vocab) or top_p[r] < 1, with a temperature);
// call it after tie_sample on the same rows. one_cta != 0 runs the kernel for the largest vocabularies whatever
// the size (tests).
TIE_API int tie_sample_filtered(const float* logits, long long row_stride, int rows, int vocab, const float* inv_temperature,
                                const int* top_k, const float* top_p, const unsigned long long* seeds,
                                const unsigned long long* counters, int* out, int one_cta, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && vocab > 0 && vocab < (1 << 24), "sample: bad sizes rows=%d vocab=%d", rows, vocab);
  TIE_REQUIRE(inv_temperature != nullptr && top_k != nullptr && top_p != nullptr && seeds != nullptr && counters != nullptr,
              "sample: filtered sampling needs temperatures, top_k, top_p, seeds and counters");
  if (rows == 0) return kOk;
  if (!one_cta && vocab <= kClusterCtas * kFilterThreads * kClusterMaxE)
    return launch_filtered_cluster(logits, row_stride, rows, vocab, inv_temperature, top_k, top_p, seeds, counters, out, s);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(sample_filtered_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(sizeof(FilterShared))) != cudaSuccess) {
      set_error("sample: cannot reserve %zu bytes of shared memory", sizeof(FilterShared));
      return kCudaError;
    }
    configured = true;
  }
  TIE_LAUNCH((sample_filtered_kernel), rows, kFilterThreads, sizeof(FilterShared), s, logits, row_stride, vocab, inv_temperature,
             top_k, top_p, seeds, counters, out);
  TIE_RETURN_LAUNCH("sample_filtered");
}
