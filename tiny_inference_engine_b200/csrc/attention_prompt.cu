// Causal attention of prompt portions over the paged bfloat16 cache: keys and values come page by
// page through TMA into a ring of shared-memory stages filled by a producer warp; four consumer
// warps own 16 rows each (rows = queries x the query heads of one kv head) and walk the key tiles
// up to the diagonal with mma.sync m16n8k16, float softmax and accumulation. Head sizes 64, 128,
// 256; up to 16 query heads per kv head; page sizes that are powers of two from 8 up. Other sizes
// go to the cp.async kernel in attention_tc.cu or to the CUDA-core kernels.
//
// Contract as there (the reference's paged_attention, src/backend/cpu/cpu_backend.cpp:261-319): row
// t of sequence s sits at pos = context_len[s] - n_queries(s) + (t - query_start[s]) and sees keys
// 0..pos (window w > 0: pos-w+1..pos); the cached prefix and this step's own keys are both read
// from the pages, where the kernel before this one has put them.
//
// grid = (kv heads, row tiles of 64, sequences); CTAs start in that order with the last row tiles first, so the
// tiles with the most keys of every kv head run first.
// Tiles of keys that lie wholly below every row's position (and inside the window) need no mask.
#include "attention_mma.cuh"
#include "tma.cuh"
#include "launchers.h"

namespace tie {

constexpr int kPromptThreads = 160;

struct PromptArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  int* status;
  long long q_stride;
  int max_blocks, q_heads, kv_heads, page_size, page_shift, window;
  float scale_log2;
};

template <int DH, int STAGES>
__global__ void __launch_bounds__(kPromptThreads) attn_prompt_tma_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                         const __grid_constant__ CUtensorMap v_map, PromptArgs a) {
  pdl_sync();
  using L = HalfLayout<DH>;
  constexpr int HALVES = DH / 64;
  constexpr int PLANE_BYTES = HALVES * 64 * 128;
  constexpr int STAGE_BYTES = 2 * PLANE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_tile = smem;                                              // 64 rows x DH, row layout: borrowed from the ring until the
                                                                       // consumers hold Q in registers (the producer waits for that)
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  int* flags = reinterpret_cast<int*>(empty + STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, kvh = blockIdx.x;
  const int G = a.q_heads / a.kv_heads;
  const int t0 = a.query_start[seq];
  const int nq = a.query_start[seq + 1] - t0;
  const int rows = nq * G;
  const int row0 = (static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y)) * 64;   // last rows (most keys) first
  if (row0 >= rows) return;
  const int pos0 = a.context_lens[seq] - nq;                      // position of the sequence's first query of this step
  const int last_row = min(rows, row0 + 64) - 1;
  const int hi_cta = pos0 + last_row / G;
  const int lo_cta = a.window > 0 ? max(0, pos0 + row0 / G - a.window + 1) : 0;
  const int kt_first = lo_cta / kKeysPerTile, kt_last = hi_cta / kKeysPerTile;
  const int n_tiles = kt_last - kt_first + 1;
  const int box_rows = min(a.page_size, kKeysPerTile);
  const int boxes_per_tile = kKeysPerTile / box_rows;
  const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 4);
    }
    flags[0] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // Q rows of this tile (rows beyond the sequence: zeros)
  constexpr int CPR = DH / 8;
  for (int id = threadIdx.x; id < 64 * CPR; id += kPromptThreads) {
    const int r = id / CPR, c = id % CPR;
    const int row = row0 + r;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (row < rows)
      v = *reinterpret_cast<const uint4*>(a.q + static_cast<long long>(t0 + row / G) * a.q_stride +
                                          static_cast<long long>(kvh * G + row % G) * DH + c * 8);
    *reinterpret_cast<uint4*>(q_tile + RowLayout<DH>::at(r, c)) = v;
  }
  __syncthreads();
  volatile int* abort_flag = flags;
  uint32_t qf[DH / 16][4];
  if (warp < 4) {
    const uint32_t q_addr = smem_u32(q_tile);
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks) ldmatrix_x4(qf[ks], q_addr + RowLayout<DH>::at(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
  }
  __syncthreads();   // Q is in registers: the ring is free for keys and values

  if (warp == 4) {
    // ---- producer: lane b fetches box b of every tile (a page, or 64 keys of a larger page)
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(empty + s, ((i / STAGES) & 1) ^ 1, abort_flag, a.status, 11) ? 1 : 0;
        if (ok) mbar_expect_tx(full + s, STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < boxes_per_tile) {
        const int key = (kt_first + i) * kKeysPerTile + lane * box_rows;
        const int idx = key >> a.page_shift;
        const int page = idx < a.max_blocks ? table[idx] : 0;   // beyond the table: any real page; those keys are masked
        const int row = (page * a.kv_heads + kvh) * a.page_size + (key & (a.page_size - 1));
        uint8_t* kdst = smem + s * STAGE_BYTES + lane * box_rows * 128;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          tma_load_2d(kdst + h * (64 * 128), &k_map, h * 64, row, full + s);
          tma_load_2d(kdst + PLANE_BYTES + h * (64 * 128), &v_map, h * 64, row, full + s);
        }
      }
    }
  } else {
    // ---- consumers: warp w owns rows row0 + 16 w .. + 15
    const int g = lane >> 2, tq = lane & 3;
    int row_pos[2];
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int row = row0 + warp * 16 + g + 8 * half;
      row_pos[half] = row < rows ? pos0 + row / G : -1;
    }
    const bool warp_has_rows = row0 + warp * 16 < rows;
    const int warp_hi = warp_has_rows ? pos0 + min(rows - 1, row0 + warp * 16 + 15) / G : -1;   // largest position of the warp's rows
    const int warp_lo = warp_has_rows ? pos0 + (row0 + warp * 16) / G : -1;                     // smallest
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
    float acc[DH / 8][4];
#pragma unroll
    for (int j = 0; j < DH / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(full + s, (i / STAGES) & 1, abort_flag, a.status, 12)) break;
      const int key0 = (kt_first + i) * kKeysPerTile;
      const bool in_window = a.window <= 0 || key0 + 63 > warp_lo - a.window;   // some key of the tile is inside some row's window
      if (key0 <= warp_hi && in_window) {
        const uint32_t k_tile = smem_u32(smem + s * STAGE_BYTES);
        float sc[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
        qk_tile<DH, 8, L>(sc, qf, k_tile, 0);
        // no mask where every key of the tile is at or below every row's position and inside every row's window
        const bool full_tile = row0 + warp * 16 + 15 < rows && key0 + 63 <= warp_lo && (a.window <= 0 || key0 > warp_hi - a.window);
        if (full_tile) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) sc[j][e] *= a.scale_log2;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int key = key0 + j * 8 + tq * 2 + (e & 1);
              const int pos = row_pos[e >> 1];
              const bool ok = key <= pos && (a.window <= 0 || key > pos - a.window);
              sc[j][e] = ok ? sc[j][e] * a.scale_log2 : -INFINITY;
            }
          }
        }
        softmax_update<DH, 8>(sc, m, l, acc);
        pv_tile<DH, 8, L>(acc, sc, k_tile + PLANE_BYTES, 0);
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + s)) : "memory");
    }

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
  __syncthreads();
  if (flags[0] != 0) {   // a wait ran out: let copies that are still in flight land before the CTA goes away
    const unsigned long long t_start = clock64();
    while (clock64() - t_start < 4000000ull) {
    }
  }
}

template <int DH>
static int launch_prompt_tma(const CUtensorMap& km, const CUtensorMap& vm, const PromptArgs& a, int n_seqs, int max_rows,
                             cudaStream_t s) {
  constexpr int STAGES = DH >= 256 ? 2 : (DH == 128 ? 3 : 4);
  constexpr size_t smem = static_cast<size_t>(STAGES) * 2 * (DH / 64) * 64 * 128 + 2 * STAGES * 8 + 16 + 1024;
  static_assert(64 * DH * 2 <= STAGES * 2 * (DH / 64) * 64 * 128, "the Q tile borrows the ring");
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prompt_tma_kernel<DH, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
      set_error("attention_prompt: cannot reserve %zu bytes of shared memory", smem);
      return kCudaError;
    }
    configured = true;
  }
  TIE_LAUNCH((attn_prompt_tma_kernel<DH, STAGES>), dim3(a.kv_heads, ceil_div(max_rows, 64), n_seqs), kPromptThreads, smem, s, km, vm, a);
  return kOk;
}

}  // namespace tie

using namespace tie;

// Rows [0, rows) of the step belong to sequences 0..n_seqs-1, each bringing several tokens;
// max_queries is the largest number of tokens one of them brings; pages is the number of pages
// of the cache planes.
TIE_API int tie_attention_prompt_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                     const int* query_start, const int* context_lens, const int* block_tables,
                                     int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                     int page_size, int pages, int window, float scale, cudaStream_t s) {
  TIE_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_prompt: head_dim %d is not 64, 128 or 256", head_dim);
  TIE_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
              "attention_prompt: %d query heads over %d kv heads (at most 16 per group)", q_heads, kv_heads);
  TIE_REQUIRE(page_size >= 8 && (page_size & (page_size - 1)) == 0, "attention_prompt: page size %d is not a power of two from 8 up", page_size);
  TIE_REQUIRE(q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0, "attention_prompt: q rows must be 16-byte aligned");
  if (n_seqs == 0 || max_queries == 0) return kOk;
  TIE_REQUIRE(static_cast<long long>(max_queries) * (q_heads / kv_heads) <= 65535LL * 64, "attention_prompt: %d queries in one portion are too many", max_queries);
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  const int box_rows = page_size < kKeysPerTile ? page_size : kKeysPerTile;
  CUtensorMap km, vm;
  const long long rows = static_cast<long long>(pages) * kv_heads * page_size;
  TIE_REQUIRE(make_map_bf16(&km, k_cache, rows, head_dim, head_dim, 64, box_rows) &&
                  make_map_bf16(&vm, v_cache, rows, head_dim, head_dim, 64, box_rows),
              "attention_prompt: cuTensorMapEncodeTiled failed");
  TIE_REQUIRE(status_word() != nullptr, "attention_prompt: cannot allocate the status word");
  PromptArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), query_start, context_lens, block_tables,
               status_word(), q_stride, max_blocks, q_heads, kv_heads, page_size, shift, window, scale * 1.4426950408889634f};
  const int max_rows = max_queries * (q_heads / kv_heads);
  int st = kOk;
  if (head_dim == 64) st = launch_prompt_tma<64>(km, vm, a, n_seqs, max_rows, s);
  else if (head_dim == 128) st = launch_prompt_tma<128>(km, vm, a, n_seqs, max_rows, s);
  else st = launch_prompt_tma<256>(km, vm, a, n_seqs, max_rows, s);
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("attention_prompt_tma");
}
