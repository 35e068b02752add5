// Causal attention over the paged bfloat16 cache on the tensor cores (mma.sync m16n8k16, float
// accumulation), for head sizes 64, 128 and 256, groups of up to 16 query heads per kv head, any
// page size. Other sizes are served by the CUDA-core kernels in attention_simt.cu.
//
// Same contract as there (the reference's paged_attention, src/backend/cpu/cpu_backend.cpp:261-319):
// query row t of sequence s sits at pos = context_len[s] - n_queries(s) + (t - query_start[s]) and
// sees keys 0..pos (window w > 0: pos-w+1..pos); query head h reads kv head h / G; scores, running
// maximum, sum and output accumulator are float.
//
// The G query heads that share a kv head are rows of one MMA tile, so every key and value is
// fetched once per group, not once per head. Keys and values travel from their pages to shared
// memory in 16-byte cp.async pieces (zero-filled beyond the last key) through a ring of stages,
// stored with an XOR swizzle so that ldmatrix reads them without bank conflicts.
//   prompt kernel  one CTA per (64 rows = queries x heads of the group, kv head, sequence); its
//                  four warps own 16 rows each and walk all key tiles up to the diagonal.
//   decode kernel  one CTA per (sequence, kv head, split of the keys); its four warps own 16 keys
//                  of every 64-key tile, combine their partial results in shared memory and leave
//                  (acc, max, sum) per split in scratch memory for attention_merge_kernel.
#include "attention_mma.cuh"
#include "launchers.h"

namespace tie {

struct AttnTcArgs {
  const __nv_bfloat16* q;     // row stride q_stride, head h at h * head_dim
  const __nv_bfloat16* k_cache;
  const __nv_bfloat16* v_cache;
  __nv_bfloat16* out;         // [T, q_heads * head_dim]
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  const int* seq_list;        // decode: sequences that bring one token; prompt: null (sequences 0..n-1)
  float* scratch;             // decode: [n_list, q_heads, max_splits, head_dim + 2]
  long long q_stride;
  int max_blocks, q_heads, kv_heads, page_size, window;
  int split_keys, max_splits;
  float scale_log2;           // scale * log2(e)
};

// ---------------------------------------------------------------------------------------------
// Prompt portions. grid = (row tiles of 64, kv heads, sequences with several tokens).
template <int DH, int STAGES>
__global__ void __launch_bounds__(kAttnThreads) attn_prompt_tc_kernel(AttnTcArgs a) {
  pdl_sync();
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE_BYTES = kKeysPerTile * DH * 2;
  const uint32_t q_tile = smem_addr(smem);                       // 64 rows x DH
  const uint32_t kv_base = q_tile + 64 * DH * 2;                 // STAGES x (K tile, V tile)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, kvh = blockIdx.y;
  const int G = a.q_heads / a.kv_heads;
  const int t0 = a.query_start[seq];
  const int nq = a.query_start[seq + 1] - t0;
  const int rows = nq * G;
  const int row0 = blockIdx.x * 64;
  if (row0 >= rows) return;
  const int ctx = a.context_lens[seq];
  const int pos0 = ctx - nq;                                      // position of the sequence's first query of this step
  const int last_row = min(rows, row0 + 64) - 1;
  const int hi_cta = pos0 + last_row / G;
  const int lo_cta = a.window > 0 ? max(0, pos0 + row0 / G - a.window + 1) : 0;
  const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;

  // Q rows of this tile -> shared memory (rows beyond the sequence: zeros)
  constexpr int CPR = DH / 8;
  for (int id = threadIdx.x; id < 64 * CPR; id += kAttnThreads) {
    const int r = id / CPR, c = id % CPR;
    const int row = row0 + r;
    const bool valid = row < rows;
    const __nv_bfloat16* src = a.q;
    if (valid) src = a.q + static_cast<long long>(t0 + row / G) * a.q_stride + static_cast<long long>(kvh * G + row % G) * DH + c * 8;
    cp_async16(q_tile + swz<DH>(r, c), src, valid ? 16 : 0);
  }
  cp_async_commit();

  const int kt_first = lo_cta / kKeysPerTile, kt_last = hi_cta / kKeysPerTile;
  const int n_tiles = kt_last - kt_first + 1;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles) {
      const int key0 = (kt_first + st) * kKeysPerTile;
      load_kv_tiles<DH>(kv_base + st * 2 * TILE_BYTES, kv_base + st * 2 * TILE_BYTES + TILE_BYTES, a.k_cache, a.v_cache, table, kvh, a.kv_heads, a.page_size, key0, lo_cta, hi_cta);
    }
    cp_async_commit();
  }
  cp_async_wait<STAGES - 1>();   // Q has landed (it was the first group)
  __syncthreads();
  uint32_t qf[DH / 16][4];
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) {
    const int r = warp * 16 + (lane & 15);
    const int c = ks * 2 + (lane >> 4);
    ldmatrix_x4(qf[ks], q_tile + swz<DH>(r, c));
  }

  const int g = lane >> 2, tq = lane & 3;
  int row_pos[2];   // position of this thread's two rows (g and g + 8 of the warp's 16)
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = row0 + warp * 16 + g + 8 * half;
    row_pos[half] = row < rows ? pos0 + row / G : -1;
  }
  // the largest position among this warp's rows (-1 if it has none): rows ascend with their index
  const int warp_hi = row0 + warp * 16 < rows ? pos0 + min(rows - 1, row0 + warp * 16 + 15) / G : -1;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float acc[DH / 8][4];
#pragma unroll
  for (int j = 0; j < DH / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

  for (int i = 0; i < n_tiles; ++i) {
    const int nxt = i + STAGES - 1;
    if (nxt < n_tiles) {
      const int key0 = (kt_first + nxt) * kKeysPerTile;
      const uint32_t dst = kv_base + (nxt % STAGES) * 2 * TILE_BYTES;
      load_kv_tiles<DH>(dst, dst + TILE_BYTES, a.k_cache, a.v_cache, table, kvh, a.kv_heads, a.page_size, key0, lo_cta, hi_cta);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const int key0 = (kt_first + i) * kKeysPerTile;
    if (key0 <= warp_hi) {   // the whole warp is above the diagonal otherwise
      const uint32_t k_tile = kv_base + (i % STAGES) * 2 * TILE_BYTES;
      float s[8][4];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      qk_tile<DH, 8>(s, qf, k_tile, 0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + tq * 2 + (e & 1);
          const int pos = row_pos[e >> 1];
          const bool ok = key <= pos && (a.window <= 0 || key > pos - a.window);
          s[j][e] = ok ? s[j][e] * a.scale_log2 : -INFINITY;
        }
      }
      softmax_update<DH, 8>(s, m, l, acc);
      pv_tile<DH, 8>(acc, s, k_tile + TILE_BYTES, 0);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int row = row0 + warp * 16 + g + 8 * half;
    if (row >= rows) continue;
    const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
    __nv_bfloat16* o = a.out + (static_cast<long long>(t0 + row / G) * a.q_heads + kvh * G + row % G) * DH;
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
      *reinterpret_cast<uint32_t*>(o + j * 8 + tq * 2) = pack_bf16(acc[j][2 * half] * inv, acc[j][2 * half + 1] * inv);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Sequences that bring one token. grid = (sequences of seq_list, kv heads, splits).
template <int DH, int STAGES>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_tc_kernel(AttnTcArgs a, int n_list) {
  pdl_sync();
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int TILE_BYTES = kKeysPerTile * DH * 2;
  const uint32_t q_tile = smem_addr(smem);                       // 16 rows x DH
  const uint32_t kv_base = q_tile + 16 * DH * 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int li = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = a.seq_list[li];
  const int G = a.q_heads / a.kv_heads;
  const int t = a.query_start[seq];
  const int pos = a.context_lens[seq] - 1;
  if (pos < 0) return;
  const int lo0 = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int lo = lo0 + split * a.split_keys;
  if (lo > pos) return;
  const int hi = split == a.max_splits - 1 ? pos : min(pos, lo + a.split_keys - 1);   // the last split takes the rest
  const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;

  constexpr int CPR = DH / 8;
  for (int id = threadIdx.x; id < 16 * CPR; id += kAttnThreads) {
    const int r = id / CPR, c = id % CPR;
    const bool valid = r < G;
    const __nv_bfloat16* src = valid ? a.q + static_cast<long long>(t) * a.q_stride + static_cast<long long>(kvh * G + r) * DH + c * 8 : a.q;
    cp_async16(q_tile + swz<DH>(r, c), src, valid ? 16 : 0);
  }
  cp_async_commit();

  const int kt_first = lo / kKeysPerTile, kt_last = hi / kKeysPerTile;
  const int n_tiles = kt_last - kt_first + 1;
#pragma unroll
  for (int st = 0; st < STAGES - 1; ++st) {
    if (st < n_tiles) {
      const int key0 = (kt_first + st) * kKeysPerTile;
      load_kv_tiles<DH>(kv_base + st * 2 * TILE_BYTES, kv_base + st * 2 * TILE_BYTES + TILE_BYTES, a.k_cache, a.v_cache, table, kvh, a.kv_heads, a.page_size, key0, lo, hi);
    }
    cp_async_commit();
  }
  cp_async_wait<STAGES - 1>();
  __syncthreads();
  uint32_t qf[DH / 16][4];
#pragma unroll
  for (int ks = 0; ks < DH / 16; ++ks) ldmatrix_x4(qf[ks], q_tile + swz<DH>(lane & 15, ks * 2 + (lane >> 4)));

  const int tq = lane & 3;
  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float acc[DH / 8][4];
#pragma unroll
  for (int j = 0; j < DH / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

  for (int i = 0; i < n_tiles; ++i) {
    const int nxt = i + STAGES - 1;
    if (nxt < n_tiles) {
      const int key0 = (kt_first + nxt) * kKeysPerTile;
      const uint32_t dst = kv_base + (nxt % STAGES) * 2 * TILE_BYTES;
      load_kv_tiles<DH>(dst, dst + TILE_BYTES, a.k_cache, a.v_cache, table, kvh, a.kv_heads, a.page_size, key0, lo, hi);
    }
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const int key0 = (kt_first + i) * kKeysPerTile + warp * 16;   // this warp's 16 keys of the tile
    if (key0 <= hi && key0 + 15 >= lo) {
      const uint32_t k_tile = kv_base + (i % STAGES) * 2 * TILE_BYTES;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      qk_tile<DH, 2>(s, qf, k_tile, warp * 16);
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + tq * 2 + (e & 1);
          s[j][e] = (key >= lo && key <= hi) ? s[j][e] * a.scale_log2 : -INFINITY;
        }
      }
      softmax_update<DH, 2>(s, m, l, acc);
      pv_tile<DH, 2>(acc, s, k_tile + TILE_BYTES, warp * 16);
    }
    __syncthreads();
  }
  cp_async_wait<0>();
  __syncthreads();

  // Combine the four warps (each saw a quarter of the keys) in shared memory: [warp][row][DH + 2] floats.
  float* part = reinterpret_cast<float*>(smem);
  constexpr int RS = DH + 2;
  const int g = lane >> 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = g + 8 * half;
    if (r >= G) continue;
    float* dst = part + (warp * 16 + r) * RS;
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) {
      dst[j * 8 + tq * 2] = acc[j][2 * half];
      dst[j * 8 + tq * 2 + 1] = acc[j][2 * half + 1];
    }
    if (tq == 0) {
      dst[DH] = m[half];
      dst[DH + 1] = l[half];
    }
  }
  __syncthreads();
  for (int id = threadIdx.x; id < G * DH; id += kAttnThreads) {
    const int r = id / DH, d = id % DH;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, part[(w * 16 + r) * RS + DH]);
    float o = 0.0f, ls = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = part[(w * 16 + r) * RS + DH];
      const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mx);
      o += part[(w * 16 + r) * RS + d] * f;
      ls += part[(w * 16 + r) * RS + DH + 1] * f;
    }
    float* dst = a.scratch + ((static_cast<long long>(li) * a.q_heads + kvh * G + r) * a.max_splits + split) * RS;
    dst[d] = o;
    if (d == 0) {
      dst[DH] = mx * 0.6931471805599453f;   // back to natural-log units, which the merge kernel uses
      dst[DH + 1] = ls;
    }
  }
}

template <int DH>
static int launch_prompt(const AttnTcArgs& a, int n_seqs, int max_rows, cudaStream_t s) {
  constexpr int STAGES = DH >= 256 ? 2 : 3;
  constexpr size_t smem = 64 * DH * 2 + static_cast<size_t>(STAGES) * 2 * kKeysPerTile * DH * 2;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prompt_tc_kernel<DH, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
      set_error("attention_tc: cannot reserve %zu bytes of shared memory", smem);
      return kCudaError;
    }
    configured = true;
  }
  TIE_LAUNCH((attn_prompt_tc_kernel<DH, STAGES>), dim3(ceil_div(max_rows, 64), a.kv_heads, n_seqs), kAttnThreads, smem, s, a);
  return kOk;
}

template <int DH>
static int launch_decode(const AttnTcArgs& a, int n_list, cudaStream_t s) {
  constexpr int STAGES = DH >= 256 ? 2 : 3;
  constexpr size_t kv = 16 * DH * 2 + static_cast<size_t>(STAGES) * 2 * kKeysPerTile * DH * 2;
  constexpr size_t merge = 4 * 16 * (DH + 2) * sizeof(float);
  constexpr size_t smem = kv > merge ? kv : merge;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_decode_tc_kernel<DH, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
      set_error("attention_tc: cannot reserve %zu bytes of shared memory", smem);
      return kCudaError;
    }
    configured = true;
  }
  TIE_LAUNCH((attn_decode_tc_kernel<DH, STAGES>), dim3(n_list, a.kv_heads, a.max_splits), kAttnThreads, smem, s, a, n_list);
  return kOk;
}

}  // namespace tie

using namespace tie;

static int check_tc(int q_heads, int kv_heads, int head_dim, int page_size) {
  TIE_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_tc: head_dim %d is not 64, 128 or 256", head_dim);
  TIE_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
              "attention_tc: %d query heads over %d kv heads (at most 16 per group)", q_heads, kv_heads);
  TIE_REQUIRE(page_size > 0, "attention_tc: bad page size");
  return kOk;
}

// Rows [0, rows) of the step belong to sequences 0..n_seqs-1, each bringing several tokens;
// max_queries is the largest number of tokens one of them brings.
TIE_API int tie_attention_prompt_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                    const int* query_start, const int* context_lens, const int* block_tables,
                                    int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                    int page_size, int window, float scale, cudaStream_t s) {
  if (const int st = check_tc(q_heads, kv_heads, head_dim, page_size)) return st;
  if (n_seqs == 0 || max_queries == 0) return kOk;
  TIE_REQUIRE(q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0, "attention_tc: q rows must be 16-byte aligned");
  AttnTcArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
               static_cast<const __nv_bfloat16*>(v_cache), static_cast<__nv_bfloat16*>(out), query_start, context_lens,
               block_tables, nullptr, nullptr, q_stride, max_blocks, q_heads, kv_heads, page_size, window, 0, 0,
               scale * 1.4426950408889634f};
  const int max_rows = max_queries * (q_heads / kv_heads);
  int st = kOk;
  if (head_dim == 64) st = launch_prompt<64>(a, n_seqs, max_rows, s);
  else if (head_dim == 128) st = launch_prompt<128>(a, n_seqs, max_rows, s);
  else st = launch_prompt<256>(a, n_seqs, max_rows, s);
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("attention_prompt_tc");
}

// The sequences of seq_list bring one token each; writes (acc, max, sum) per split to scratch
// [n_list, q_heads, max_splits, head_dim + 2]; tie_attention_merge then combines them.
TIE_API int tie_attention_decode_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                    const int* query_start, const int* context_lens, const int* block_tables,
                                    int max_blocks, int q_heads, int kv_heads, int head_dim, int page_size, int window,
                                    float scale, const int* seq_list, int n_list, int split_keys, int max_splits,
                                    float* scratch, cudaStream_t s) {
  if (const int st = check_tc(q_heads, kv_heads, head_dim, page_size)) return st;
  if (n_list == 0) return kOk;
  TIE_REQUIRE(q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0, "attention_tc: q rows must be 16-byte aligned");
  TIE_REQUIRE(split_keys > 0 && split_keys % kKeysPerTile == 0 && max_splits > 0 && scratch != nullptr,
              "attention_tc: splits must be positive multiples of %d keys", kKeysPerTile);
  AttnTcArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k_cache),
               static_cast<const __nv_bfloat16*>(v_cache), nullptr, query_start, context_lens, block_tables, seq_list,
               scratch, q_stride, max_blocks, q_heads, kv_heads, page_size, window, split_keys, max_splits,
               scale * 1.4426950408889634f};
  int st = kOk;
  if (head_dim == 64) st = launch_decode<64>(a, n_list, s);
  else if (head_dim == 128) st = launch_decode<128>(a, n_list, s);
  else st = launch_decode<256>(a, n_list, s);
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("attention_decode_tc");
}
