// Causal attention over the paged cache on the CUDA cores, for any head size that is a
// multiple of 8, any number of heads and groups, any page size; float or bfloat16 storage,
// float scores, softmax and accumulation. It is the attention of the 32-bit path and the
// fallback of the bfloat16 path.
//
// What it computes is the reference's paged_attention (src/backend/cpu/cpu_backend.cpp:261-319):
// query row t of sequence s has position pos = context_len[s] - n_queries(s) + (t - query_start[s])
// and sees keys 0..pos (with a window w > 0: keys pos-w+1..pos); query head h reads kv head
// h / (Hq/Hkv); online softmax of scale * q.k; out = acc / l.
//
// Two kernels share the inner loop:
//   rows kernel   one warp per (row, head) over all of its keys: prompt portions.
//   split kernel  one warp per (sequence, head, split of the keys) for sequences that bring
//                 one token: each split of `split_keys` keys leaves (max, sum, acc) in
//                 scratch memory and a merge kernel combines them in split order. The split
//                 size is a constant of the call, so the order of the sums for a token
//                 depends only on its own context, never on the batch around it.
#include <math.h>

#include "common.cuh"
#include "launchers.h"

namespace tie {

struct AttnArgs {
  const void* q;            // [T, ...] row stride q_stride, head h at h * head_dim
  const void* k_cache;      // [pages, kv_heads, page_size, head_dim]
  const void* v_cache;
  void* out;                // [T, q_heads * head_dim]
  const int* seq_of_row;    // [T]
  const int* query_start;   // [S + 1]
  const int* context_lens;  // [S]
  const int* block_tables;  // [S, max_blocks]
  long long q_stride;
  int max_blocks;
  int rows;                 // T
  int seqs;                 // S
  int q_heads, kv_heads, head_dim, page_size;
  int window;               // 0 = all keys
  float scale;
};

// One warp: online softmax over keys [lo, hi] of one (query vector, kv head).
// q is in shared memory (float, already multiplied by nothing: scale is applied to the score).
// Lane `l` owns output dims [l * DPL, (l + 1) * DPL). Returns m, l and acc in registers.
template <typename T, int DPL>
__device__ __forceinline__ void attend_range(const float* __restrict__ qs, const T* __restrict__ kc,
                                             const T* __restrict__ vc, const int* __restrict__ table, int kvh,
                                             int kv_heads, int head_dim, int page_size, float scale, int lo, int hi,
                                             float& m, float& l, float (&acc)[DPL]) {
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int d0 = lane * DPL;
  for (int base = lo; base <= hi; base += 32) {
    const int j = base + lane;
    const bool valid = j <= hi;
    int row = 0;  // index of the key's row in units of head_dim elements
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      row = (page * kv_heads + kvh) * page_size + j % page_size;
      const T* kr = kc + static_cast<long long>(row) * head_dim;
      float dot = 0.0f;
      for (int d = 0; d < head_dim; d += V) {
        Vec16<T> kv;
        kv.load(kr + d);
#pragma unroll
        for (int e = 0; e < V; ++e) dot = fmaf(qs[d + e], kv.v[e], dot);
      }
      s = scale * dot;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf at the start gives 0
    const float p = valid ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[e] *= corr;
    const int count = min(32, hi - base + 1);
    for (int jj = 0; jj < count; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const int rj = __shfl_sync(0xffffffffu, row, jj);
      if (d0 < head_dim) {
        const T* vr = vc + static_cast<long long>(rj) * head_dim + d0;
#pragma unroll
        for (int e = 0; e < DPL; ++e) acc[e] = fmaf(pj, ld(vr + e), acc[e]);
      }
    }
  }
}

template <typename T, int DPL>
__global__ void __launch_bounds__(128) attention_rows_kernel(AttnArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (item >= static_cast<long long>(a.rows) * a.q_heads) return;
  const int t = static_cast<int>(item / a.q_heads);
  const int h = static_cast<int>(item % a.q_heads);
  const int s = a.seq_of_row[t];
  const int qs0 = a.query_start[s], qs1 = a.query_start[s + 1];
  const int pos = a.context_lens[s] - (qs1 - qs0) + (t - qs0);
  const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int kvh = h / (a.q_heads / a.kv_heads);

  float* qs = smem + warp * a.head_dim;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride + static_cast<long long>(h) * a.head_dim;
  for (int d = lane; d < a.head_dim; d += 32) qs[d] = ld(qv + d);
  __syncwarp();

  float m = -INFINITY, l = 0.0f, acc[DPL] = {};
  attend_range<T, DPL>(qs, static_cast<const T*>(a.k_cache), static_cast<const T*>(a.v_cache),
                       a.block_tables + static_cast<long long>(s) * a.max_blocks, kvh, a.kv_heads, a.head_dim,
                       a.page_size, a.scale, lo, pos, m, l, acc);
  const int d0 = lane * DPL;
  if (d0 < a.head_dim) {
    T* o = static_cast<T*>(a.out) + (static_cast<long long>(t) * a.q_heads + h) * a.head_dim + d0;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;  // no keys (a padding row): zeros
#pragma unroll
    for (int e = 0; e < DPL; ++e) st(o + e, acc[e] * inv);
  }
}

// Split kernel: sequences listed in `seq_list` (each brings exactly one query row).
// scratch: [n_list, q_heads, max_splits, head_dim + 2] floats (acc, then m, l).
template <typename T, int DPL>
__global__ void __launch_bounds__(128) attention_split_kernel(AttnArgs a, const int* __restrict__ seq_list, int n_list,
                                                              int split_keys, int max_splits, float* __restrict__ scratch) {
  pdl_sync();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.y;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (item >= static_cast<long long>(n_list) * a.q_heads) return;
  const int li = static_cast<int>(item / a.q_heads);
  const int h = static_cast<int>(item % a.q_heads);
  const int s = seq_list[li];
  const int t = a.query_start[s];
  const int pos = a.context_lens[s] - 1;
  const int lo0 = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int lo = lo0 + split * split_keys;
  if (lo > pos) return;  // this sequence has fewer splits
  // The last split takes whatever is left, so that a context longer than max_splits * split_keys (a caller
  // who sized max_splits from something else than the longest context) costs time, never keys.
  const int hi = split == max_splits - 1 ? pos : min(pos, lo + split_keys - 1);
  const int kvh = h / (a.q_heads / a.kv_heads);

  float* qs = smem + warp * a.head_dim;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride + static_cast<long long>(h) * a.head_dim;
  for (int d = lane; d < a.head_dim; d += 32) qs[d] = ld(qv + d);
  __syncwarp();

  float m = -INFINITY, l = 0.0f, acc[DPL] = {};
  attend_range<T, DPL>(qs, static_cast<const T*>(a.k_cache), static_cast<const T*>(a.v_cache),
                       a.block_tables + static_cast<long long>(s) * a.max_blocks, kvh, a.kv_heads, a.head_dim,
                       a.page_size, a.scale, lo, hi, m, l, acc);
  float* dst = scratch + ((static_cast<long long>(li) * a.q_heads + h) * max_splits + split) * (a.head_dim + 2);
  const int d0 = lane * DPL;
  if (d0 < a.head_dim) {
#pragma unroll
    for (int e = 0; e < DPL; ++e) dst[d0 + e] = acc[e];
  }
  if (lane == 0) {
    dst[a.head_dim] = m;
    dst[a.head_dim + 1] = l;
  }
}

// Merge of the splits of one (sequence, head), in split order: one block each. The weights
// exp(m_i - m) of the splits are computed once into shared memory, then every thread sums its
// dims over the splits.
constexpr int kMergeThreads = 128;
constexpr int kMergeMaxSplits = 256;

template <typename T>
__global__ void __launch_bounds__(kMergeThreads) attention_merge_kernel(AttnArgs a, const int* __restrict__ seq_list,
                                                                        int n_list, int split_keys, int max_splits,
                                                                        const float* __restrict__ scratch) {
  pdl_sync();
  __shared__ float weight[kMergeMaxSplits];
  __shared__ float inv_l;
  const int item = blockIdx.x;
  const int li = item / a.q_heads, h = item % a.q_heads;
  const int s = seq_list[li];
  const int t = a.query_start[s];
  const int pos = a.context_lens[s] - 1;
  T* o = static_cast<T*>(a.out) + (static_cast<long long>(t) * a.q_heads + h) * a.head_dim;
  if (pos < 0) {  // a padding sequence: no keys, zeros
    for (int d = threadIdx.x; d < a.head_dim; d += kMergeThreads) st(o + d, 0.0f);
    return;
  }
  const int lo0 = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int splits = min((pos - lo0) / split_keys + 1, max_splits);   // the last one took the rest (split kernels)
  const int stride = a.head_dim + 2;
  const float* src = scratch + (static_cast<long long>(li) * a.q_heads + h) * max_splits * stride;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < splits; i += 32) m = fmaxf(m, src[i * stride + a.head_dim]);
    m = warp_max(m);
    float l = 0.0f;
    for (int i = threadIdx.x; i < splits; i += 32) {
      const float w = expf(src[i * stride + a.head_dim] - m);
      weight[i] = w;
      l += src[i * stride + a.head_dim + 1] * w;   // summed below in a fixed lane order
    }
    l = warp_sum(l);
    if (threadIdx.x == 0) inv_l = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < a.head_dim; d += kMergeThreads) {
    float acc = 0.0f;
    for (int i = 0; i < splits; ++i) acc = fmaf(src[i * stride + d], weight[i], acc);
    st(o + d, acc * inv_l);
  }
}

template <typename T>
int launch_attention(const AttnArgs& a, const int* row_seq_unused, const int* seq_list, int n_list, int split_keys,
                     int max_splits, float* scratch, int rows_kernel, cudaStream_t s) {
  (void)row_seq_unused;
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * a.head_dim * sizeof(float);
  const int dpl = (a.head_dim + 31) / 32;
#define TIE_ATTN_CASE(D)                                                                                         \
  do {                                                                                                           \
    if (rows_kernel) {                                                                                           \
      const long long items = static_cast<long long>(a.rows) * a.q_heads;                                        \
      if (items > 0) TIE_LAUNCH((attention_rows_kernel<T, D>), ceil_div(items, warps), warps * 32, smem, s, a);            \
    } else {                                                                                                     \
      const long long items = static_cast<long long>(n_list) * a.q_heads;                                        \
      if (items > 0) {                                                                                           \
        TIE_LAUNCH((attention_split_kernel<T, D>), dim3(ceil_div(items, warps), max_splits), warps * 32, smem, s,           \
            a, seq_list, n_list, split_keys, max_splits, scratch);                                               \
        TIE_LAUNCH((attention_merge_kernel<T>), static_cast<int>(items), kMergeThreads, 0, s, a, seq_list, n_list, split_keys, \
                                                                                    max_splits, scratch);         \
      }                                                                                                          \
    }                                                                                                            \
  } while (0)
  if (dpl <= 1) TIE_ATTN_CASE(1);
  else if (dpl <= 2) TIE_ATTN_CASE(2);
  else if (dpl <= 4) TIE_ATTN_CASE(4);
  else if (dpl <= 8) TIE_ATTN_CASE(8);
  else TIE_ATTN_CASE(16);
#undef TIE_ATTN_CASE
  TIE_RETURN_LAUNCH("paged_attention_simt");
}

}  // namespace tie

using namespace tie;

static int check_attn(const AttnArgs& a) {
  TIE_REQUIRE(a.q_heads > 0 && a.kv_heads > 0 && a.q_heads % a.kv_heads == 0,
              "attention: %d query heads are not a multiple of %d kv heads", a.q_heads, a.kv_heads);
  TIE_REQUIRE(a.head_dim > 0 && a.head_dim % 8 == 0 && a.head_dim <= 512,
              "attention: head_dim %d must be a multiple of 8 and at most 512", a.head_dim);
  TIE_REQUIRE(a.head_dim <= 256 || a.head_dim % 16 == 0, "attention: head_dim %d above 256 must be a multiple of 16",
              a.head_dim);
  TIE_REQUIRE(a.page_size > 0 && a.max_blocks > 0, "attention: bad page geometry");
  TIE_REQUIRE(a.window >= 0, "attention: negative window");
  return kOk;
}

// All rows of the step, each over all of its keys (prompt portions and, when no split is
// wanted, single tokens too).
TIE_API int tie_attention_rows(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                               void* out, const int* seq_of_row, const int* query_start, const int* context_lens,
                               const int* block_tables, int max_blocks, int rows, int seqs, int q_heads, int kv_heads,
                               int head_dim, int page_size, int window, float scale, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_stride, max_blocks,
                   rows, seqs, q_heads, kv_heads, head_dim, page_size, window, scale};
  if (const int st = check_attn(a)) return st;
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  if (dtype == TIE_BF16) return launch_attention<__nv_bfloat16>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// The sequences of seq_list bring one token each; their keys are cut into splits of
// `split_keys` keys. scratch holds n_list * q_heads * max_splits * (head_dim + 2) floats.
TIE_API int tie_attention_split(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                void* out, const int* query_start, const int* context_lens, const int* block_tables,
                                int max_blocks, int seqs, int q_heads, int kv_heads, int head_dim, int page_size,
                                int window, float scale, const int* seq_list, int n_list, int split_keys,
                                int max_splits, float* scratch, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale};
  if (const int st = check_attn(a)) return st;
  TIE_REQUIRE(split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits && scratch != nullptr,
              "attention split: bad split geometry (at most %d splits)", kMergeMaxSplits);
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// Combines the (acc, max, sum) that a split kernel (this file's or the tensor-core one) left in
// scratch [n_list, q_heads, max_splits, head_dim + 2] into out rows, in split order.
TIE_API int tie_attention_merge(int dtype, void* out, const int* query_start, const int* context_lens, int q_heads,
                                int head_dim, int window, const int* seq_list, int n_list, int split_keys, int max_splits,
                                const float* scratch, cudaStream_t s) {
  TIE_REQUIRE(q_heads > 0 && head_dim > 0 && split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits,
              "attention merge: bad geometry (at most %d splits)", kMergeMaxSplits);
  if (n_list == 0) return kOk;
  AttnArgs a{};
  a.out = out;
  a.query_start = query_start;
  a.context_lens = context_lens;
  a.q_heads = q_heads;
  a.head_dim = head_dim;
  a.window = window;
  const long long items = static_cast<long long>(n_list) * q_heads;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((attention_merge_kernel<float>), static_cast<int>(items), kMergeThreads, 0, s, a, seq_list, n_list, split_keys, max_splits, scratch);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((attention_merge_kernel<__nv_bfloat16>), static_cast<int>(items), kMergeThreads, 0, s, a, seq_list, n_list, split_keys, max_splits, scratch);
  } else {
    set_error("attention merge: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("attention_merge");
}

// ---------------------------------------------------------------------------------------------
// The variant of tie_attention_split that allocates nothing (see attention_noalloc.h).
#include "attention_noalloc.h"

namespace tie {
// Partial results of the splits. In host code this name is only a handle for
// cudaGetSymbolAddress; the address a kernel can use is looked up once per device below.
static __device__ __align__(256) float g_noalloc_scratch[TIE_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_noalloc_ptr[kMaxDevices] = {};   // device address of the array on each device, once known
}  // namespace tie

TIE_API int tie_attention_split_noalloc(int dtype, const void* q, long long q_stride, const void* k_cache,
                                        const void* v_cache, void* out, const int* query_start, const int* context_lens,
                                        const int* block_tables, int max_blocks, int seqs, int q_heads, int kv_heads,
                                        int head_dim, int page_size, int window, float scale, const int* seq_list,
                                        int n_list, int split_keys, int max_splits, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale};
  if (const int st = check_attn(a)) return st;
  TIE_REQUIRE(n_list >= 0 && split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits,
              "attention split (no alloc): bad split geometry (at most %d splits)", kMergeMaxSplits);
  const long long need = static_cast<long long>(n_list) * q_heads * max_splits * (head_dim + 2);
  TIE_REQUIRE(need <= TIE_NOALLOC_SCRATCH_FLOATS,
              "attention split (no alloc): %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of partial results "
              "exceed the built-in %d; use fewer splits or tie_attention_split with your own scratch",
              n_list, q_heads, max_splits, head_dim, need, TIE_NOALLOC_SCRATCH_FLOATS);
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    set_error("attention split (no alloc): cannot use device %d (at most %d devices)", device, kMaxDevices);
    return kCudaError;
  }
  if (g_noalloc_ptr[device] == nullptr) {   // set-up, once per device, with that device current
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("attention split (no alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return kCudaError;
    }
    g_noalloc_ptr[device] = p;
  }
  float* scratch = g_noalloc_ptr[device];
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}
