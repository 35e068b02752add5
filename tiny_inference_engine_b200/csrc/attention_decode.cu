// Attention of sequences that bring one token (decode) over the paged bfloat16 cache: keys and
// values come page by page through TMA into a ring of shared-memory stages, a producer warp
// keeps the ring full, four consumer warps run the MMAs, and the CTA that finishes last among
// the splits of a (sequence, kv head) combines the splits itself. Head sizes 64, 128, 256; up
// to 16 query heads per kv head; page sizes that are powers of two from 8 up. Other sizes go to
// the cp.async kernel in attention_tc.cu or to the CUDA-core kernels.
//
// What it computes is the reference's paged_attention for one query row per sequence
// (src/backend/cpu/cpu_backend.cpp:261-319): pos = context_len - 1, keys lo..pos (lo > 0 only
// with a window), query head h reads kv head h / G, float scores, maximum, sum and accumulator.
//
// One CTA = (sequence, kv head, split of `split_keys` keys), 160 threads:
//   warp 4 (one lane) waits for a free stage (empty barrier), arms the stage's full barrier with
//       the byte count and issues one TMA box per page and 64-column block for K and for V;
//   warps 0-3 wait for the full barrier, each takes 16 of the tile's 64 keys (Q K^T, online
//       softmax, P V on mma.sync m16n8k16), and arrive on the empty barrier.
// The G query heads of the group are the rows of the MMA tile, so a key or value is read once per
// group. After the last tile the four warps' partial results are combined in shared memory and
// written as (acc, max, sum) to scratch; a counter per (sequence, kv head) tells the last CTA
// to arrive that all splits are there, and it merges them in split order (so the result does not
// depend on which CTA came last) and writes the output rows. With one split the output is
// written directly. Every mbarrier wait is bounded; on expiry the status word gets a code.
#include "attention_mma.cuh"
#include "head_prep.cuh"
#include "tma.cuh"
#include "launchers.h"

namespace tie {

constexpr int kDecThreads = 160;
constexpr int kNoCluster = -7;         // launch_decode_tma: the GPU does not hold the launch's clusters at once
constexpr int kMaxTablePages = 512;    // pages of one split that the CTA keeps in shared memory

struct DecodeArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  const int* seq_list;   // null: the sequences seq_first, seq_first + 1, ...
  int seq_first;
  float* scratch;        // [n_list, q_heads, max_splits, head_dim + 2]
  int* counters;         // [n_list, kv_heads], zero between launches
  int* status;
  long long q_stride;
  int max_blocks, q_heads, kv_heads, page_size, page_shift, window, split_keys, max_splits;
  float scale_log2;
  // Only for the kernel that prepares its heads itself (PREP): the output of the q/k/v product, [T, (q_heads + 2 kv_heads)
  // * head_dim] as bfloat16 rows (qkv) or as `part_splits` float partial sums (part + z * part_stride + t * part_ld + column),
  // the head norms' weights (null: no norm), the rotation's frequencies (null: none), the tokens' positions, the cache
  // planes to append the newest key and value to (append != 0).
  const __nv_bfloat16* qkv;
  const float* part;
  long long qkv_stride, part_stride, part_ld;
  int part_splits, append;
  const float *qw, *kw, *inv_freq;
  float q_eps, k_eps;
  const int* positions;
  __nv_bfloat16 *k_plane, *v_plane;
};

// A float into the shared memory of another CTA of the cluster (`mine`: the address in this CTA's own).
__device__ __forceinline__ void send_float(const float* mine, uint32_t rank, float v) {
  uint32_t addr;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(smem_u32(mine)), "r"(rank));
  asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// CLUSTER: the splits of a (sequence, kv head) are the CTAs of one thread-block cluster (grid z = cluster size =
// a.max_splits, 2 to 16): each sends its results into the shared memory of the CTAs that merge (one row of the
// group each), all meet at one cluster barrier, and the rows are merged from local shared memory, in split order; no
// scratch, no counter, no fence. A CTA whose split holds no key walks the same path with nothing to add.
template <int DH, int STAGES, bool PREP, bool CLUSTER>
__global__ void __launch_bounds__(kDecThreads) attn_decode_tma_kernel(const __grid_constant__ CUtensorMap k_map,
                                                                      const __grid_constant__ CUtensorMap v_map, DecodeArgs a) {
  // Keys and values of earlier tokens, the tables and the lengths do not depend on the kernels just ahead in
  // the stream (those write this step's q and the newest token's cache slot), so the ring starts filling before
  // this kernel waits for them; the wait comes before q is read, before the tile with the newest key is
  // fetched, and before anything is written.
  pdl_launch_dependents();
  using L = HalfLayout<DH>;
  constexpr int HALVES = DH / 64;
  constexpr int PLANE_BYTES = HALVES * 64 * 128;       // K (or V) of one 64-key tile
  constexpr int STAGE_BYTES = 2 * PLANE_BYTES;
  constexpr int RS = DH + 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_tile = smem + STAGES * STAGE_BYTES;                       // 16 rows x DH, row layout
  uint64_t* full = reinterpret_cast<uint64_t*>(q_tile + 16 * DH * 2);
  uint64_t* empty = full + STAGES;
  int* pages = reinterpret_cast<int*>(empty + STAGES);                 // page ids of this split
  int* flags = pages + kMaxTablePages;                                 // [0] abort, [1] last-arrival flag
  [[maybe_unused]] float* cs = reinterpret_cast<float*>(flags + 4);    // PREP: the token's cos and sin
  [[maybe_unused]] __nv_bfloat16* newest = reinterpret_cast<__nv_bfloat16*>(cs + DH);   // PREP: the newest key, then its value
  // CLUSTER: what the splits send for the rows this CTA merges, [16][RS] at most, and a row's weights. Memory of its own:
  // a split that is through early sends while this CTA's ring is still in use.
  [[maybe_unused]] float* inbox = reinterpret_cast<float*>(flags + 4) + (PREP ? 2 * DH : 0);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int li = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int seq = a.seq_list ? a.seq_list[li] : a.seq_first + li;
  const int G = a.q_heads / a.kv_heads;
  // Without a window a split's first key does not depend on the context length: the page ids of all the boxes the
  // split may need are asked for together with the length (one round of loads instead of two in a row); entries
  // beyond the sequence's own pages are never used.
  constexpr int kAhead = (kMaxTablePages + kDecThreads - 1) / kDecThreads;
  int ahead[kAhead];
  const int box_rows_ = min(a.page_size, kKeysPerTile);
  const int split_boxes = a.window > 0 ? 0 : (a.split_keys / kKeysPerTile) * (kKeysPerTile / box_rows_);
  {
    const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const int b = threadIdx.x + j * kDecThreads;
      const int idx = (split * a.split_keys + b * box_rows_) >> a.page_shift;
      ahead[j] = b < split_boxes && idx < a.max_blocks ? table[idx] : 0;
    }
  }
  const int t = a.query_start[seq];
  const int pos = a.context_lens[seq] - 1;
  if (pos < 0) {            // a padding sequence: no keys; split 0 writes zeros
    pdl_wait();
    if (split == 0) {
      for (int id = threadIdx.x; id < G * DH; id += kDecThreads)
        a.out[(static_cast<long long>(t) * a.q_heads + kvh * G) * DH + id] = __float2bfloat16_rn(0.0f);
    }
    return;
  }
  const int lo0 = a.window > 0 ? max(0, pos - a.window + 1) : 0;
  const int lo = lo0 + split * a.split_keys;
  const int n_splits = (pos - lo0) / a.split_keys + 1;     // the same in every CTA of the sequence
  const bool no_keys = lo > pos;
  if (no_keys && (!CLUSTER || n_splits == 1)) return;      // (with one split nobody meets at the cluster barrier)
  const int hi = min(pos, lo + a.split_keys - 1);
  if (n_splits > a.max_splits) {   // the caller sized max_splits for shorter contexts: say so, write nothing
    if (threadIdx.x == 0 && split == 0) *reinterpret_cast<volatile int*>(a.status) = 13;
    return;
  }
  const int kt_first = lo / kKeysPerTile, kt_last = hi / kKeysPerTile;
  const int n_tiles = no_keys ? 0 : kt_last - kt_first + 1;
  const int box_rows = min(a.page_size, kKeysPerTile);
  const int boxes_per_tile = kKeysPerTile / box_rows;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 4);
    }
    flags[0] = 0;
    flags[1] = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  // page ids of the split's tiles (one per TMA box), zero beyond the table: page 0 is real memory
  // and keys beyond `hi` are masked, so what it holds does not matter as long as it is finite
  if (a.window > 0) {
    const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
    const int first_key = kt_first * kKeysPerTile;
    for (int b = threadIdx.x; b < n_tiles * boxes_per_tile; b += kDecThreads) {
      const int idx = (first_key + b * box_rows) >> a.page_shift;
      pages[b] = idx < a.max_blocks ? table[idx] : 0;
    }
  } else {
#pragma unroll
    for (int j = 0; j < kAhead; ++j) {
      const int b = threadIdx.x + j * kDecThreads;
      if (b < split_boxes) pages[b] = ahead[j];
    }
  }
  __syncthreads();
  volatile int* abort_flag = flags;

  float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};
  float acc[DH / 8][4];
#pragma unroll
  for (int j = 0; j < DH / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;

  if (warp == 4) {
    // The whole warp walks the tiles: lane 0 arms the stage's barrier, then the lanes issue the tile's boxes side by
    // side (one lane after the other would spend most of a tile's time computing addresses).
    const int ops_per_tile = boxes_per_tile * HALVES * 2;
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      if (!__all_sync(0xffffffffu, mbar_wait(empty + s, ((i / STAGES) & 1) ^ 1, abort_flag, a.status, 11) ? 1 : 0)) break;
      // the tile with the newest key: written by the kernel ahead, unless this kernel appends it itself (then the
      // copy in shared memory is patched once it has landed)
      if (hi == pos && i == n_tiles - 1 && !(PREP && a.append)) pdl_wait();
      if (lane == 0) mbar_expect_tx(full + s, STAGE_BYTES);
      __syncwarp();
      uint8_t* kdst = smem + s * STAGE_BYTES;
      for (int op = lane; op < ops_per_tile; op += 32) {
        const int b = op / (2 * HALVES), h = (op % (2 * HALVES)) >> 1, is_v = op & 1;
        const int key = (kt_first + i) * kKeysPerTile + b * box_rows;
        const int row = (pages[i * boxes_per_tile + b] * a.kv_heads + kvh) * a.page_size + (key & (a.page_size - 1));
        tma_load_2d(kdst + is_v * PLANE_BYTES + h * (64 * 128) + b * box_rows * 128, is_v ? &v_map : &k_map, h * 64, row, full + s);
      }
      __syncwarp();
    }
  } else {
    // Q: the G heads of the group, rows G..15 zero
    constexpr int CPR = DH / 8;
    constexpr int VEC = DH / 32;
    using Slice = HeadSlice<__nv_bfloat16, VEC>;
    [[maybe_unused]] const bool appends = PREP && a.append != 0 && hi == pos && !no_keys;   // this split ends with the newest key
    if constexpr (PREP) {
      // the rotation depends on the step's own inputs only: made while the kernel ahead still runs
      if (a.inv_freq) rotation_table(cs, static_cast<float>(a.positions[t]), a.inv_freq, DH / 2, threadIdx.x, 128);
      for (int id = threadIdx.x; id < 16 * CPR; id += 128) {
        const int r = id / CPR, c = id % CPR;
        if (r >= G) *reinterpret_cast<uint4*>(q_tile + RowLayout<DH>::at(r, c)) = make_uint4(0u, 0u, 0u, 0u);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      pdl_wait();
      // A warp a head, as in the q/k norm + RoPE + append kernel: the group's query heads, and where this split ends
      // with the newest key, that key's head (normed and rotated) and its value's (as it is).
      const int heads = G + (appends ? 2 : 0);
      for (int r = warp; r < heads; r += 4) {
        const int head = r < G ? kvh * G + r : (r == G ? a.q_heads + kvh : a.q_heads + a.kv_heads + kvh);
        const long long col = static_cast<long long>(head) * DH + lane * VEC;
        float x[VEC];
        if (a.part) {   // the sum of the split product's partial sums, in split order
          using FloatSlice = HeadSlice<float, VEC>;
          const float* psrc = a.part + static_cast<long long>(t) * a.part_ld + col;
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[e] = 0.0f;
#pragma unroll 4
          for (int z = 0; z < a.part_splits; ++z) {
            const FloatSlice p = *reinterpret_cast<const FloatSlice*>(psrc + static_cast<long long>(z) * a.part_stride);
#pragma unroll
            for (int e = 0; e < VEC; ++e) x[e] += p.v[e];
          }
        } else {
          const Slice in = *reinterpret_cast<const Slice*>(a.qkv + static_cast<long long>(t) * a.qkv_stride + col);
#pragma unroll
          for (int e = 0; e < VEC; ++e) x[e] = __bfloat162float(in.v[e]);
        }
        if (r <= G) prepare_head<VEC>(x, r < G ? a.qw : a.kw, r < G ? a.q_eps : a.k_eps, a.inv_freq ? cs : nullptr, lane);
        Slice out;
#pragma unroll
        for (int e = 0; e < VEC; ++e) out.v[e] = __float2bfloat16_rn(x[e]);
        if (r < G) {
          *reinterpret_cast<Slice*>(q_tile + RowLayout<DH>::at(r, (lane * VEC) >> 3) + ((lane * VEC * 2) & 15)) = out;
        } else {
          // the page of the newest key is among this split's pages; the same row the TMA boxes of that page start from
          const int box = (pos - kt_first * kKeysPerTile) / box_rows;
          const long long row = static_cast<long long>(pages[box] * a.kv_heads + kvh) * a.page_size + (pos & (a.page_size - 1));
          *reinterpret_cast<Slice*>((r == G ? a.k_plane : a.v_plane) + row * DH + lane * VEC) = out;
          *reinterpret_cast<Slice*>(newest + (r - G) * DH + lane * VEC) = out;
        }
      }
    } else {
      pdl_wait();
      for (int id = threadIdx.x; id < 16 * CPR; id += 128) {
        const int r = id / CPR, c = id % CPR;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (r < G) v = *reinterpret_cast<const uint4*>(a.q + static_cast<long long>(t) * a.q_stride + static_cast<long long>(kvh * G + r) * DH + c * 8);
        *reinterpret_cast<uint4*>(q_tile + RowLayout<DH>::at(r, c)) = v;
      }
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");   // the four consumer warps
    uint32_t qf[DH / 16][4];
    const uint32_t q_addr = smem_u32(q_tile);
#pragma unroll
    for (int ks = 0; ks < DH / 16; ++ks) ldmatrix_x4(qf[ks], q_addr + RowLayout<DH>::at(lane & 15, ks * 2 + (lane >> 4)));
    const int tq = lane & 3;
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(full + s, (i / STAGES) & 1, abort_flag, a.status, 12)) break;
      if constexpr (PREP) {
        // The tile came from the cache as it was before this step: the newest key's row gets what this kernel made,
        // from the warp that works on that key (no other warp reads the row).
        const int rr = pos - (kt_first + i) * kKeysPerTile;
        if (appends && i == n_tiles - 1 && warp == (rr >> 4)) {
          uint8_t* tile = smem + s * STAGE_BYTES;
          const uint32_t at = L::at(rr, (lane * VEC) >> 3) + ((lane * VEC * 2) & 15);
          *reinterpret_cast<Slice*>(tile + at) = *reinterpret_cast<const Slice*>(newest + lane * VEC);
          *reinterpret_cast<Slice*>(tile + PLANE_BYTES + at) = *reinterpret_cast<const Slice*>(newest + DH + lane * VEC);
          __syncwarp();
        }
      }
      const int key0 = (kt_first + i) * kKeysPerTile + warp * 16;   // this warp's 16 keys of the tile
      if (key0 <= hi && key0 + 15 >= lo) {
        const uint32_t k_tile = smem_u32(smem + s * STAGE_BYTES);
        float sc[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) sc[j][0] = sc[j][1] = sc[j][2] = sc[j][3] = 0.0f;
        qk_tile<DH, 2, L>(sc, qf, k_tile, warp * 16);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int key = key0 + j * 8 + tq * 2 + (e & 1);
            sc[j][e] = (key >= lo && key <= hi) ? sc[j][e] * a.scale_log2 : -INFINITY;
          }
        }
        softmax_update<DH, 2>(sc, m, l, acc);
        pv_tile<DH, 2, L>(acc, sc, k_tile + PLANE_BYTES, warp * 16);
      }
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(empty + s)) : "memory");
    }
  }
  __syncthreads();   // every stage has been consumed (or a wait gave up): the ring can be reused
  pdl_wait();        // (the producer warp may not have waited yet)
  if (flags[0] != 0) {   // a wait ran out: let copies that are still in flight land before the ring is reused
    const unsigned long long t0 = clock64();
    while (clock64() - t0 < 4000000ull) {
    }
    __syncthreads();
  }

  // Combine the four consumer warps in shared memory: [warp][row][DH + 2] floats.
  float* part = reinterpret_cast<float*>(smem);
  if (warp < 4) {
    const int g = lane >> 2, tq = lane & 3;
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
  }
  __syncthreads();
  // per row: the warps' common maximum, the factor that brings each warp's sums to it, and the row sum
  float* fac = part + 4 * 16 * RS;          // [G][4] factors, then [G] maxima, then [G] sums
  if (threadIdx.x < G) {
    const int r = threadIdx.x;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) mx = fmaxf(mx, part[(w * 16 + r) * RS + DH]);
    float ls = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = part[(w * 16 + r) * RS + DH];
      const float f = mw == -INFINITY ? 0.0f : exp2f(mw - mx);
      fac[r * 4 + w] = f;
      ls += part[(w * 16 + r) * RS + DH + 1] * f;
    }
    fac[4 * G + r] = mx;
    fac[5 * G + r] = ls;
  }
  __syncthreads();
  if constexpr (CLUSTER) {
    if (n_splits > 1) {
      // Row r of the group is merged by the CTA r % C of the cluster (C = a.max_splits CTAs): every CTA sends its sums,
      // maximum and row sum of that row into the owner's shared memory, all meet at one cluster barrier, and the
      // owners merge what they were sent, in split order. Nobody reads another CTA's memory after the barrier, so
      // every CTA may leave when it is through.
      const int C = a.max_splits;
      float* wgt = inbox + 16 * RS;              // [C] weights of the row being merged, then 1 / its sum
      for (int id = threadIdx.x; id < G * RS; id += kDecThreads) {
        const int r = id / RS, e = id % RS;
        float v;
        if (e < DH) {
          v = 0.0f;
#pragma unroll
          for (int w = 0; w < 4; ++w) v += part[(w * 16 + r) * RS + e] * fac[r * 4 + w];
        } else {
          v = fac[(e == DH ? 4 : 5) * G + r];
        }
        send_float(inbox + ((r / C) * C + split) * RS + e, static_cast<uint32_t>(r % C), v);
      }
      cluster_barrier();
      for (int r = split; r < G; r += C) {       // (uniform over the CTA)
        const float* mine = inbox + (r / C) * C * RS;
        if (threadIdx.x == 0) {
          float mx = -INFINITY;
          for (int i = 0; i < n_splits; ++i) mx = fmaxf(mx, mine[i * RS + DH]);
          float ls = 0.0f;
          for (int i = 0; i < n_splits; ++i) {
            const float w = exp2f(mine[i * RS + DH] - mx);
            wgt[i] = w;
            ls += mine[i * RS + DH + 1] * w;
          }
          wgt[C] = ls > 0.0f ? 1.0f / ls : 0.0f;
        }
        __syncthreads();
        for (int d = threadIdx.x; d < DH; d += kDecThreads) {
          float o = 0.0f;
#pragma unroll 4
          for (int i = 0; i < n_splits; ++i) o = fmaf(mine[i * RS + d], wgt[i], o);
          a.out[(static_cast<long long>(t) * a.q_heads + kvh * G + r) * DH + d] = __float2bfloat16_rn(o * wgt[C]);
        }
        __syncthreads();
      }
      return;
    }
  }
  float* split_out = a.scratch + ((static_cast<long long>(li) * a.q_heads + kvh * G) * a.max_splits + split) * RS;
  for (int id = threadIdx.x; id < G * DH; id += kDecThreads) {
    const int r = id / DH, d = id % DH;
    float o = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) o += part[(w * 16 + r) * RS + d] * fac[r * 4 + w];
    const float ls = fac[5 * G + r];
    if (n_splits == 1) {
      a.out[(static_cast<long long>(t) * a.q_heads + kvh * G + r) * DH + d] = __float2bfloat16_rn(ls > 0.0f ? o / ls : 0.0f);
    } else {
      float* dst = split_out + static_cast<long long>(r) * a.max_splits * RS;
      dst[d] = o;
      if (d == 0) {
        dst[DH] = fac[4 * G + r];          // in log2 units: only this kernel reads it back
        dst[DH + 1] = ls;
      }
    }
  }
  if (n_splits == 1) return;

  // The last CTA of this (sequence, kv head) to get here merges all splits, in split order.
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int done = atomicAdd(a.counters + li * a.kv_heads + kvh, 1);
    flags[1] = done == n_splits - 1 ? 1 : 0;
  }
  __syncthreads();
  if (flags[1] == 0) return;
  __threadfence();
  // Every split's maximum and sum come in with one round of loads (a thread per row and split); then a thread
  // per row turns them into weights, adding in split order.
  float* wgt = part;                                   // [G][max_splits] weights
  float* msm = wgt + G * a.max_splits;                 // [G][max_splits] maxima
  float* lsm = msm + G * a.max_splits;                 // [G][max_splits] sums
  float* inv = lsm + G * a.max_splits;                 // [G] 1 / row sum
  const float* base = a.scratch + (static_cast<long long>(li) * a.q_heads + kvh * G) * a.max_splits * RS;
  for (int id = threadIdx.x; id < G * n_splits; id += kDecThreads) {
    const int r = id / n_splits, i = id % n_splits;
    const float* src = base + (static_cast<long long>(r) * a.max_splits + i) * RS;
    msm[r * a.max_splits + i] = __ldcg(src + DH);
    lsm[r * a.max_splits + i] = __ldcg(src + DH + 1);
  }
  __syncthreads();
  if (threadIdx.x < G) {
    const int r = threadIdx.x;
    float mx = -INFINITY;
    for (int i = 0; i < n_splits; ++i) mx = fmaxf(mx, msm[r * a.max_splits + i]);
    float ls = 0.0f;
    for (int i = 0; i < n_splits; ++i) {
      const float w = exp2f(msm[r * a.max_splits + i] - mx);
      wgt[r * a.max_splits + i] = w;
      ls += lsm[r * a.max_splits + i] * w;
    }
    inv[r] = ls > 0.0f ? 1.0f / ls : 0.0f;
  }
  __syncthreads();
  for (int id = threadIdx.x; id < G * DH; id += kDecThreads) {
    const int r = id / DH, d = id % DH;
    const float* src = base + static_cast<long long>(r) * a.max_splits * RS + d;
    const float* wr = wgt + r * a.max_splits;
    float o = 0.0f;
    for (int i0 = 0; i0 < n_splits; i0 += 8) {   // eight loads in flight, added in split order
      float v[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] = i0 + j < n_splits ? __ldcg(src + (i0 + j) * RS) : 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (i0 + j < n_splits) o = fmaf(v[j], wr[i0 + j], o);
      }
    }
    a.out[(static_cast<long long>(t) * a.q_heads + kvh * G + r) * DH + d] = __float2bfloat16_rn(o * inv[r]);
  }
  if (threadIdx.x == 0) a.counters[li * a.kv_heads + kvh] = 0;   // ready for the next launch
}

template <int DH, bool PREP, bool CLUSTER>
static int launch_decode_tma(const CUtensorMap& km, const CUtensorMap& vm, const DecodeArgs& a, int n_list, cudaStream_t s) {
  constexpr int STAGES = DH >= 256 ? 2 : (DH == 128 ? 3 : 4);
  constexpr size_t ring = static_cast<size_t>(STAGES) * 2 * (DH / 64) * 64 * 128;
  // the four warps' results and factors
  constexpr size_t combine = (4 * 16 * (DH + 2) + 6 * 16 + 0) * sizeof(float);
  constexpr size_t weights = (3 * 16 * 256 + 16) * sizeof(float);                    // the last CTA's merge: 16 rows, 256 splits at most
  constexpr size_t merge = combine > weights ? combine : weights;
  constexpr size_t prep = PREP ? DH * sizeof(float) + 2 * DH * 2 + 16 : 0;           // the rotation, the newest key and value
  constexpr size_t inbox = CLUSTER ? (16 * (DH + 2) + 32) * sizeof(float) : 0;        // what the splits send to the CTA that merges a row
  constexpr size_t smem = (ring > merge ? ring : merge) + 16 * DH * 2 + 2 * STAGES * 8 + (kMaxTablePages + 4) * 4 + prep + inbox + 1024;
  static bool configured = false;
  auto kernel = attn_decode_tma_kernel<DH, STAGES, PREP, CLUSTER>;
  if (!configured) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess ||
        (CLUSTER && cudaFuncSetAttribute(kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) != cudaSuccess)) {
      set_error("attention_decode: cannot reserve %zu bytes of shared memory (or clusters of 16)", smem);
      return kCudaError;
    }
    configured = true;
  }
  if constexpr (CLUSTER) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_list, a.kv_heads, a.max_splits);
    cfg.blockDim = dim3(kDecThreads);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 1;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = a.max_splits;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    // How many clusters of this size the GPU holds at once (asked once a size): with more than that in the launch,
    // splits without keys would keep others waiting for a place, and the launch goes through scratch memory instead.
    static int holds[17] = {};
    if (holds[a.max_splits] == 0) {
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
      }
      holds[a.max_splits] = n > 0 ? n : -1;
    }
    if (holds[a.max_splits] < n_list * a.kv_heads) return kNoCluster;
    cfg.numAttrs = pdl_enabled() ? 2 : 1;
    cudaLaunchKernelEx(&cfg, kernel, km, vm, a);
  } else {
    TIE_LAUNCH(kernel, dim3(n_list, a.kv_heads, a.max_splits), kDecThreads, smem, s, km, vm, a);
  }
  return kOk;
}

template <bool PREP, bool CLUSTER>
static int launch_decode_tma_of(int head_dim, const CUtensorMap& km, const CUtensorMap& vm, const DecodeArgs& a, int n_list, cudaStream_t s) {
  if (head_dim == 64) return launch_decode_tma<64, PREP, CLUSTER>(km, vm, a, n_list, s);
  if (head_dim == 128) return launch_decode_tma<128, PREP, CLUSTER>(km, vm, a, n_list, s);
  return launch_decode_tma<256, PREP, CLUSTER>(km, vm, a, n_list, s);
}

// What both entry points ask of their arguments, and the launch.
static int decode_tma(DecodeArgs a, bool prep, bool cluster, const void* k_cache, const void* v_cache, int head_dim, int pages, int n_list,
                      float scale, cudaStream_t s) {
  const int q_heads = a.q_heads, kv_heads = a.kv_heads, page_size = a.page_size, split_keys = a.split_keys, max_splits = a.max_splits;
  TIE_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_decode: head_dim %d is not 64, 128 or 256", head_dim);
  TIE_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
              "attention_decode: %d query heads over %d kv heads (at most 16 per group)", q_heads, kv_heads);
  TIE_REQUIRE(page_size >= 8 && (page_size & (page_size - 1)) == 0, "attention_decode: page size %d is not a power of two from 8 up", page_size);
  TIE_REQUIRE(split_keys > 0 && split_keys % kKeysPerTile == 0 && max_splits > 0 && a.scratch != nullptr && a.counters != nullptr,
              "attention_decode: splits must be positive multiples of %d keys", kKeysPerTile);
  const int box_rows = page_size < kKeysPerTile ? page_size : kKeysPerTile;
  TIE_REQUIRE((split_keys / kKeysPerTile + 1) * (kKeysPerTile / box_rows) <= kMaxTablePages && max_splits <= 256,
              "attention_decode: a split of %d keys over pages of %d (or %d splits) exceeds the kernel's tables", split_keys,
              page_size, max_splits);
  if (n_list == 0) return kOk;
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  CUtensorMap km, vm;
  const long long rows = static_cast<long long>(pages) * kv_heads * page_size;
  TIE_REQUIRE(make_map_bf16(&km, k_cache, rows, head_dim, head_dim, 64, box_rows) &&
                  make_map_bf16(&vm, v_cache, rows, head_dim, head_dim, 64, box_rows),
              "attention_decode: cuTensorMapEncodeTiled failed");
  TIE_REQUIRE(status_word() != nullptr, "attention_decode: cannot allocate the status word");
  a.status = status_word();
  a.page_shift = shift;
  a.scale_log2 = scale * 1.4426950408889634f;
  // cluster: the splits of a sequence and kv head as one thread-block cluster (2, 4, 8 or 16 CTAs), which merges them
  // through shared memory. The caller asks for it where every CTA of the launch is resident at once (a split without
  // keys holds its place until its cluster is through). Else, or with TIE_NO_CLUSTER_ATTENTION=1: through scratch
  // memory, merged by the CTA that finishes last.
  static const bool clusters = getenv("TIE_NO_CLUSTER_ATTENTION") == nullptr || getenv("TIE_NO_CLUSTER_ATTENTION")[0] != '1';
  TIE_REQUIRE(!cluster || max_splits == 2 || max_splits == 4 || max_splits == 8 || max_splits == 16,
              "attention_decode: a cluster of %d splits (2, 4, 8 or 16)", max_splits);
  cluster = cluster && clusters;
  int st = kNoCluster;
  if (cluster) st = prep ? launch_decode_tma_of<true, true>(head_dim, km, vm, a, n_list, s) : launch_decode_tma_of<false, true>(head_dim, km, vm, a, n_list, s);
  if (st == kNoCluster) st = prep ? launch_decode_tma_of<true, false>(head_dim, km, vm, a, n_list, s) : launch_decode_tma_of<false, false>(head_dim, km, vm, a, n_list, s);
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("attention_decode_tma");
}

}  // namespace tie

using namespace tie;

// Limits of the kernel that the host plans splits with (parts/attention.py keeps copies; a test holds them equal):
// 0 -> page ids of one split kept in shared memory, 1 -> the most splits of a sequence.
TIE_API int tie_attention_decode_limit(int which) { return which == 0 ? kMaxTablePages : which == 1 ? 256 : -1; }

// The sequences of seq_list (null: seq_first, seq_first + 1, ...; one load less at the start of every CTA) bring one token each. scratch holds n_list * q_heads * max_splits *
// (head_dim + 2) floats; counters holds n_list * kv_heads ints that are zero before the first
// launch (the kernel leaves them zero). pages is the number of pages of the cache planes. cluster != 0: the splits of
// a sequence and kv head run as one thread-block cluster and merge through shared memory (max_splits 2, 4, 8 or 16;
// scratch and counters are not touched); worth it where all n_list * kv_heads * max_splits CTAs are resident at once.
TIE_API int tie_attention_decode_tma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                     const int* query_start, const int* context_lens, const int* block_tables,
                                     int max_blocks, int q_heads, int kv_heads, int head_dim, int page_size, int pages,
                                     int window, float scale, const int* seq_list, int seq_first, int n_list,
                                     int split_keys,
                                     int max_splits, float* scratch, int* counters, int cluster, cudaStream_t s) {
  TIE_REQUIRE(q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0, "attention_decode: q rows must be 16-byte aligned");
  DecodeArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q);
  a.out = static_cast<__nv_bfloat16*>(out);
  a.query_start = query_start, a.context_lens = context_lens, a.block_tables = block_tables, a.seq_list = seq_list, a.seq_first = seq_first;
  a.scratch = scratch, a.counters = counters, a.q_stride = q_stride;
  a.max_blocks = max_blocks, a.q_heads = q_heads, a.kv_heads = kv_heads, a.page_size = page_size, a.window = window;
  a.split_keys = split_keys, a.max_splits = max_splits;
  return decode_tma(a, false, cluster != 0, k_cache, v_cache, head_dim, pages, n_list, scale, s);
}

// The same attention for a step in which every sequence brings one token, straight from the output of the q/k/v
// product: the kernel sums the product's partial sums (part, or reads the bfloat16 rows of qkv when part is null),
// norms and rotates the group's query heads itself (what tie_qk_norm_rope_append does, bit for bit), and, with
// append != 0, does the same for the newest key, stores it and its value in the cache planes and uses them. qw, kw
// and inv_freq may be null (no norm, no rotation); the rotation covers the whole head. Rows of qkv and of the
// partial sums: token t of sequence seq_list[i] is row query_start[seq_list[i]].
TIE_API int tie_attention_decode_prep(const void* qkv, long long qkv_stride, const float* part, long long part_stride,
                                      int part_splits, long long part_ld, const float* qw, const float* kw, float q_eps,
                                      float k_eps, const float* inv_freq, const int* positions, int append, void* k_cache,
                                      void* v_cache, void* out, const int* query_start, const int* context_lens,
                                      const int* block_tables, int max_blocks, int q_heads, int kv_heads, int head_dim,
                                      int page_size, int pages, int window, float scale, const int* seq_list, int seq_first,
                                      int n_list,
                                      int split_keys, int max_splits, float* scratch, int* counters, int cluster,
                                      cudaStream_t s) {
  const int vec = head_dim / 32;
  const size_t slice = static_cast<size_t>(vec) * 2 > 16 ? 16 : static_cast<size_t>(vec) * 2;
  const size_t fslice = static_cast<size_t>(vec) * 4 > 16 ? 16 : static_cast<size_t>(vec) * 4;
  TIE_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, "attention_decode: head_dim %d is not 64, 128 or 256", head_dim);
  TIE_REQUIRE(part != nullptr ? (part_splits >= 1 && reinterpret_cast<uintptr_t>(part) % fslice == 0 && part_stride % vec == 0 && part_ld % vec == 0)
                              : (qkv != nullptr && reinterpret_cast<uintptr_t>(qkv) % slice == 0 && qkv_stride % vec == 0),
              "attention_decode: the q/k/v rows (or their partial sums) must be aligned to %d elements", vec);
  TIE_REQUIRE(positions != nullptr && reinterpret_cast<uintptr_t>(k_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(v_cache) % 16 == 0,
              "attention_decode: positions and 16-byte aligned cache planes are needed");
  DecodeArgs a{};
  a.out = static_cast<__nv_bfloat16*>(out);
  a.query_start = query_start, a.context_lens = context_lens, a.block_tables = block_tables, a.seq_list = seq_list, a.seq_first = seq_first;
  a.scratch = scratch, a.counters = counters;
  a.max_blocks = max_blocks, a.q_heads = q_heads, a.kv_heads = kv_heads, a.page_size = page_size, a.window = window;
  a.split_keys = split_keys, a.max_splits = max_splits;
  a.qkv = static_cast<const __nv_bfloat16*>(qkv), a.part = part, a.qkv_stride = qkv_stride, a.part_stride = part_stride, a.part_ld = part_ld;
  a.part_splits = part_splits, a.append = append, a.qw = qw, a.kw = kw, a.inv_freq = inv_freq, a.q_eps = q_eps, a.k_eps = k_eps;
  a.positions = positions, a.k_plane = static_cast<__nv_bfloat16*>(k_cache), a.v_plane = static_cast<__nv_bfloat16*>(v_cache);
  return decode_tma(a, true, cluster != 0, k_cache, v_cache, head_dim, pages, n_list, scale, s);
}
