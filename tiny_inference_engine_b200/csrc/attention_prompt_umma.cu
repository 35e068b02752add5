// Causal attention of prompt portions on the 5th-generation tensor cores: S = Q K^T and O += P V are
// tcgen05.mma with the scores and the output accumulator in tensor memory; keys and values come page by
// page through TMA. Head sizes 64 and 128, up to 16 query heads per kv head, pages that are powers
// of two from 8 up; other sizes stay with the mma.sync kernels.
//
// Contract as in attention_prompt.cu (the reference's paged_attention,
// src/backend/cpu/cpu_backend.cpp:261-319): row t of sequence s sits at
// pos = context_len[s] - n_queries(s) + (t - query_start[s]) and sees keys 0..pos (window w > 0:
// pos-w+1..pos), all read from the pages.
//
// One CTA owns 256 rows (rows = queries x the query heads of one kv head) as two tiles of 128, so
// that the tensor cores work on one tile while the other tile's softmax runs, and both share every
// key/value tile of 64 keys. The MMAs' operand reads are what shared memory has to feed, so Q, which
// every key tile needs again, sits in tensor memory (the A operand of Q K^T comes from there) and only
// K, V and P are read from shared memory. Ten warps:
//   0-3, 4-7  softmax of tile 0 and 1: thread = one row. Puts its Q row into tensor memory once. Per key
//             tile it reads its 64 scores out of tensor memory, masks, exponentiates in float, writes P as
//             bfloat16 into one of two shared-memory buffers (the layout the MMA reads) and keeps the row
//             sum. The accumulator O stays in tensor memory; it is rescaled only when a row's maximum has
//             grown by more than 2^8 since the value it was last scaled for (any reference point gives
//             the same O / sum, as long as nothing overflows).
//   8         TMA producer: lane b fetches box b (a page, or 64 keys of a larger page) of every tile.
//   9         one thread issues the MMAs: Q K^T of tile i + 1 ahead of P V of tile i.
// Barriers: kv_full/kv_empty per stage, and for each row tile s_full (scores written), s_empty
// (scores read), p_full[2] (P written, O rescaled), p_empty[2] (P V retired). Every wait is bounded.
// grid = (kv heads, row tiles, sequences): CTAs start in that order with the last row tiles first, so the
// tiles with the most keys of every kv head run first.
#include "attention_mma.cuh"
#include "umma.cuh"
#include "launchers.h"

namespace tie {

constexpr int kUmmaAttnThreads = 320;

struct UmmaPromptArgs {
  const __nv_bfloat16* q;
  __nv_bfloat16* out;
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  int* status;
  long long q_stride;
  int max_blocks, q_heads, kv_heads, page_size, page_shift, window;
  float scale_log2;
  int cta_rows;   // 256: a CTA works on two row tiles side by side; 128: on one (more CTAs when there are few rows)
};

// Descriptor of an operand stored with its MN extent contiguous (V as [key][head dim]): 64 elements of
// MN per 128-byte row, 8 rows (k) per 1024-byte swizzle atom; `mn_block_bytes` apart lie successive blocks
// of 64 along MN.
__device__ __forceinline__ uint64_t smem_desc_sw128_mn(uint32_t addr, uint32_t mn_block_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr >> 4) & 0x3FFF);
  d |= static_cast<uint64_t>((mn_block_bytes >> 4) & 0x3FFF) << 16;   // leading byte offset
  d |= static_cast<uint64_t>(1024 >> 4) << 32;                         // stride byte offset: next 8 k
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
        "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// D[tmem_d] (+)= A[tmem_a] . B: the A operand read from tensor memory (lane = row, a 32-bit column = two
// consecutive k of 16 bits), B from shared memory.
__device__ __forceinline__ void umma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <int DH, int STAGES>
__global__ void __launch_bounds__(kUmmaAttnThreads, 1)
attn_prompt_umma_kernel(const __grid_constant__ CUtensorMap k_map, const __grid_constant__ CUtensorMap v_map, UmmaPromptArgs a) {
  pdl_sync();
  constexpr int HALVES = DH / 64;
  constexpr int P_BYTES = 128 * 128;              // 128 rows x 64 keys
  constexpr int PLANE_BYTES = HALVES * 64 * 128;  // 64 keys
  constexpr int STAGE_BYTES = 2 * PLANE_BYTES;
  constexpr int Q_COL = 128;                      // columns 0..127: the two score tiles; then Q of both tiles (two
  constexpr int O_COL = Q_COL + DH;               // elements a column); then the two accumulators
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(O_COL + 2 * DH <= 512, "tensor memory");
  constexpr float kRescaleStep = 8.0f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* p_smem = smem;                 // [row tile][buffer]
  uint8_t* ring = p_smem + 4 * P_BYTES;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(ring + STAGES * STAGE_BYTES);
  uint64_t* kv_empty = kv_full + STAGES;
  uint64_t* s_full = kv_empty + STAGES;   // [2]
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;         // [row tile][buffer]
  uint64_t* p_empty = p_full + 4;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(p_empty + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq = blockIdx.z, kvh = blockIdx.x;
  const int G = a.q_heads / a.kv_heads;
  const int t0 = a.query_start[seq];
  const int nq = a.query_start[seq + 1] - t0;
  const int rows = nq * G;
  const int row0 = (static_cast<int>(gridDim.y) - 1 - static_cast<int>(blockIdx.y)) * a.cta_rows;   // last rows (most keys) first
  if (row0 >= rows) return;
  const int pos0 = a.context_lens[seq] - nq;

  // key tiles each row tile needs: first[q]..last[q]; the CTA walks first[0]..last[1] (or last[0])
  bool has[2];
  int first[2], last[2];
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    const int r0 = row0 + 128 * q;
    has[q] = r0 < rows && 128 * q < a.cta_rows;
    const int lo_pos = pos0 + r0 / G, hi_pos = pos0 + min(rows - 1, r0 + 127) / G;
    first[q] = a.window > 0 ? max(0, lo_pos - a.window + 1) / kKeysPerTile : 0;
    last[q] = hi_pos / kKeysPerTile;
  }
  const int kt_first = first[0], kt_last = has[1] ? last[1] : last[0];
  const int n_tiles = kt_last - kt_first + 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(kv_full + s, 1);
      mbar_init(kv_empty + s, 1);
    }
    for (int q = 0; q < 2; ++q) {
      mbar_init(s_full + q, 1);
      mbar_init(s_empty + q, 4);
    }
    for (int b = 0; b < 4; ++b) {
      mbar_init(p_full + b, 4);
      mbar_init(p_empty + b, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 8) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(TMEM_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;
  if (warp < 8) {
    // Q: every softmax thread puts its own row into tensor memory (rows beyond the sequence: zeros)
    const int q = warp >> 2, rr = (warp & 3) * 32 + lane;
    const int row = row0 + 128 * q + rr;
    const uint4* src = row < rows ? reinterpret_cast<const uint4*>(a.q + static_cast<long long>(t0 + row / G) * a.q_stride +
                                                                  static_cast<long long>(kvh * G + row % G) * DH)
                                  : nullptr;
    const uint32_t q_tmem = tmem_base + (static_cast<uint32_t>((warp & 3) * 32) << 16) + Q_COL + q * (DH / 2);
#pragma unroll
    for (int c0 = 0; c0 < DH / 2; c0 += 16) {
      uint32_t w[16];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const uint4 v = src ? src[c0 / 4 + e] : make_uint4(0u, 0u, 0u, 0u);
        w[4 * e] = v.x, w[4 * e + 1] = v.y, w[4 * e + 2] = v.z, w[4 * e + 3] = v.w;
      }
      tmem_st16(q_tmem + c0, w);
    }
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

  if (warp == 8) {
    // ---- producer
    const int box_rows = min(a.page_size, kKeysPerTile);
    const int boxes_per_tile = kKeysPerTile / box_rows;
    const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % STAGES;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(kv_empty + s, ((i / STAGES) & 1) ^ 1, abort_flag, a.status, 11) ? 1 : 0;
        if (ok) mbar_expect_tx(kv_full + s, STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      if (lane < boxes_per_tile) {
        const int key = (kt_first + i) * kKeysPerTile + lane * box_rows;
        const int idx = key >> a.page_shift;
        const int page = idx < a.max_blocks ? table[idx] : 0;   // beyond the table: any real page; those keys are masked
        const int row = (page * a.kv_heads + kvh) * a.page_size + (key & (a.page_size - 1));
        uint8_t* kdst = ring + s * STAGE_BYTES + lane * box_rows * 128;
#pragma unroll
        for (int h = 0; h < HALVES; ++h) {
          tma_load_2d(kdst + h * (64 * 128), &k_map, h * 64, row, kv_full + s);
          tma_load_2d(kdst + PLANE_BYTES + h * (64 * 128), &v_map, h * 64, row, kv_full + s);
        }
      }
    }
  } else if (warp == 9) {
    // ---- MMA issuer: the whole warp walks the loop (uniform), one elected lane issues
    {
      constexpr uint32_t idesc_qk = instr_desc(kKeysPerTile);          // 128 x 64, both operands k-major
      constexpr uint32_t idesc_pv = instr_desc(DH) | (1u << 16);       // 128 x DH, B (= V) with its N extent contiguous
      // Descriptors as (low word, constant high word): one thread issues every MMA, so what it computes
      // per MMA is on the critical path of the tensor cores.
      const uint32_t k_lo0 = desc_lo_sw128(smem_u32(ring));
      const uint32_t v_lo0 = desc_lo_sw128(smem_u32(ring + PLANE_BYTES), 64 * 128);   // blocks of 64 head-dim columns lie 64 rows apart
      const uint32_t p_lo0 = desc_lo_sw128(smem_u32(p_smem));
      int n_qk[2] = {0, 0}, n_pv[2] = {0, 0};
      int s_qk = 0, s_pv = 0;
      uint32_t parity_qk = 0;
      bool ok = true;
      // Step i: Q K^T of key tile i for both row tiles, then P V of key tile i - 1 for both. The scores of
      // tile i are asked for as soon as the softmax groups have taken those of tile i - 1 out of tensor memory
      // (early in their work on them), so they are there when the groups come back for them; P V of tile i - 1
      // has to wait for the groups to finish that tile anyway. What a step waits for it waits for at once: a
      // wait costs this one thread a couple of hundred cycles even when the barrier has long flipped.
      for (int i = 0; i <= n_tiles && ok; ++i) {
        if (i < n_tiles) {
          const int t = kt_first + i;
          const bool on0 = has[0] && t >= first[0] && t <= last[0], on1 = has[1] && t >= first[1] && t <= last[1];
          const BarrierPhase w0{kv_full + s_qk, parity_qk, true};
          const BarrierPhase w1{s_empty + 0, static_cast<uint32_t>((n_qk[0] & 1) ^ 1), on0};
          const BarrierPhase w2{s_empty + 1, static_cast<uint32_t>((n_qk[1] & 1) ^ 1), on1};
          if (!__all_sync(0xffffffffu, mbar_wait_all(w0, w1, w2, abort_flag, a.status, 12) ? 1 : 0)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t k_lo = k_lo0 + s_qk * (STAGE_BYTES >> 4);
          if (elect_one()) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (!(q == 0 ? on0 : on1)) continue;
#pragma unroll
              for (int ks = 0; ks < DH / 16; ++ks) {
                umma_bf16_a_tmem(tmem_base + q * kKeysPerTile, tmem_base + Q_COL + q * (DH / 2) + ks * 8,
                                 desc_from_words(k_lo + (((ks >> 2) * (64 * 128) + (ks & 3) * 32) >> 4), kDescHiSw128), idesc_qk,
                                 ks > 0 ? 1u : 0u);
              }
              umma_commit(s_full + q);
            }
          }
          __syncwarp();
          n_qk[0] += on0 ? 1 : 0;
          n_qk[1] += on1 ? 1 : 0;
          if (++s_qk == STAGES) {
            s_qk = 0;
            parity_qk ^= 1;
          }
        }
        if (i >= 1) {
          const int t = kt_first + i - 1;
          const bool on0 = has[0] && t >= first[0] && t <= last[0], on1 = has[1] && t >= first[1] && t <= last[1];
          const int pb0 = n_pv[0] & 1, pb1 = 2 + (n_pv[1] & 1);          // the tiles' P buffers, each used for the (n_pv / 2)-th time
          const BarrierPhase w0{p_full + pb0, static_cast<uint32_t>((n_pv[0] >> 1) & 1), on0};
          const BarrierPhase w1{p_full + pb1, static_cast<uint32_t>((n_pv[1] >> 1) & 1), on1};
          const BarrierPhase w2{nullptr, 0u, false};
          if (!__all_sync(0xffffffffu, mbar_wait_all(w0, w1, w2, abort_flag, a.status, 14) ? 1 : 0)) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t v_lo = v_lo0 + s_pv * (STAGE_BYTES >> 4);
          if (elect_one()) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              if (!(q == 0 ? on0 : on1)) continue;
              const int pb = q == 0 ? pb0 : pb1;
              const uint32_t p_lo = p_lo0 + pb * (P_BYTES >> 4);
              const uint32_t keep = n_pv[q] > 0 ? 1u : 0u;
#pragma unroll
              for (int kk = 0; kk < kKeysPerTile / 16; ++kk) {
                umma_bf16(tmem_base + O_COL + q * DH, desc_from_words(p_lo + ((kk * 32) >> 4), kDescHiSw128),
                          desc_from_words(v_lo + ((kk * 16 * 128) >> 4), kDescHiSw128), idesc_pv, kk > 0 ? 1u : keep);
              }
              umma_commit(p_empty + pb);
            }
            umma_commit(kv_empty + s_pv);   // both products of key tile i - 1 have read the stage once everything issued so far retires
          }
          __syncwarp();
          n_pv[0] += on0 ? 1 : 0;
          n_pv[1] += on1 ? 1 : 0;
          if (++s_pv == STAGES) s_pv = 0;
        }
      }
    }
  } else {
    // ---- softmax: warps 0-3 own tile 0, warps 4-7 tile 1; thread = row
    const int q = warp >> 2, wq = warp & 3;
    const int rr = wq * 32 + lane;                           // row inside the tile = lane of tensor memory
    const int row = row0 + 128 * q + rr;
    const int pos = row < rows ? pos0 + row / G : -1;       // rows beyond the sequence see no key
    const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
    const uint32_t s_tmem = tmem_base + lane_base + q * kKeysPerTile;
    const uint32_t o_tmem = tmem_base + lane_base + O_COL + q * DH;
    uint8_t* p_rows = p_smem + 2 * q * P_BYTES + rr * 128;
    float m_run = -INFINITY, m_used = -INFINITY, l = 0.0f;
    bool ok = has[q];
    const int my_tiles = has[q] ? last[q] - first[q] + 1 : 0;
    for (int n = 0; n < my_tiles && ok; ++n) {
      const int key0 = (first[q] + n) * kKeysPerTile;
      ok = __all_sync(0xffffffffu, mbar_wait(s_full + q, n & 1, abort_flag, a.status, 13) ? 1 : 0) != 0;
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t sr[64];
      {
        uint32_t c0[16], c1[16], c2[16], c3[16];
        tmem_ld16(s_tmem, c0);
        tmem_ld16(s_tmem + 16, c1);
        tmem_ld16(s_tmem + 32, c2);
        tmem_ld16(s_tmem + 48, c3);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int e = 0; e < 16; ++e) {
          sr[e] = c0[e];
          sr[16 + e] = c1[e];
          sr[32 + e] = c2[e];
          sr[48 + e] = c3[e];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(s_empty + q)) : "memory");

      const bool full_tile = key0 + 63 <= pos && (a.window <= 0 || key0 > pos - a.window);
      if (!full_tile) {
#pragma unroll
        for (int c = 0; c < 64; ++c) {
          const int key = key0 + c;
          const bool seen = key <= pos && (a.window <= 0 || key > pos - a.window);
          sr[c] = seen ? sr[c] : 0xff800000u;   // -inf
        }
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 64; c += 4) {
#pragma unroll
        for (int e = 0; e < 4; ++e) mx4[e] = fmaxf(mx4[e], __uint_as_float(sr[c + e]));
      }
      m_run = fmaxf(m_run, fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * a.scale_log2);
      const bool need = m_run > m_used + kRescaleStep;       // also: the first finite maximum of the row
      if (__any_sync(0xffffffffu, need)) {
        float f = 1.0f;
        if (need) {
          f = m_used == -INFINITY ? 1.0f : ex2(m_used - m_run);
          m_used = m_run;
          l *= f;
        }
        if (n > 0) {
          // O may be touched once P V of the tile before has retired
          ok = __all_sync(0xffffffffu, mbar_wait(p_empty + 2 * q + ((n - 1) & 1), ((n - 1) >> 1) & 1, abort_flag, a.status, 13) ? 1 : 0) != 0;
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c0 = 0; c0 < DH; c0 += 16) {
            uint32_t o[16];
            tmem_ld16(o_tmem + c0, o);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 16; ++e) o[e] = __float_as_uint(__uint_as_float(o[e]) * f);
            tmem_st16(o_tmem + c0, o);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
      }
      const float base = m_used == -INFINITY ? 0.0f : m_used;
      float sum4[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p0 = ex2(fmaf(__uint_as_float(sr[c + 2 * e]), a.scale_log2, -base));
          const float p1 = ex2(fmaf(__uint_as_float(sr[c + 2 * e + 1]), a.scale_log2, -base));
          sum4[e] += p0 + p1;
          sr[(c >> 1) + e] = pack_bf16(p0, p1);
        }
      }
      l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
      // this buffer held P of the tile before the last one: its P V has to have retired
      const int pb = 2 * q + (n & 1);
      ok = __all_sync(0xffffffffu, mbar_wait(p_empty + pb, ((n >> 1) & 1) ^ 1, abort_flag, a.status, 13) ? 1 : 0) != 0;
      if (!ok) break;
      uint8_t* p_row = p_rows + (n & 1) * P_BYTES;
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(p_row + ((c ^ (rr & 7)) << 4)) = make_uint4(sr[4 * c], sr[4 * c + 1], sr[4 * c + 2], sr[4 * c + 3]);
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(p_full + pb)) : "memory");
    }
    if (ok && my_tiles > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(p_empty + 2 * q + ((my_tiles - 1) & 1), ((my_tiles - 1) >> 1) & 1, abort_flag, a.status, 13) ? 1 : 0) != 0;
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const float inv = l > 0.0f ? 1.0f / l : 0.0f;
        __nv_bfloat16* o_row = row < rows ? a.out + (static_cast<long long>(t0 + row / G) * a.q_heads + kvh * G + row % G) * DH : nullptr;
#pragma unroll 1
        for (int c0 = 0; c0 < DH; c0 += 16) {
          uint32_t o[16];
          tmem_ld16(o_tmem + c0, o);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (o_row) {
            uint32_t w[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) w[e] = pack_bf16(__uint_as_float(o[2 * e]) * inv, __uint_as_float(o[2 * e + 1]) * inv);
            *reinterpret_cast<uint4*>(o_row + c0) = make_uint4(w[0], w[1], w[2], w[3]);
            *reinterpret_cast<uint4*>(o_row + c0 + 8) = make_uint4(w[4], w[5], w[6], w[7]);
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag != 0) {   // a wait ran out: let copies and MMAs that are still in flight finish before the CTA goes away
    const unsigned long long t_start = clock64();
    while (clock64() - t_start < 4000000ull) {
    }
    __syncthreads();
  }
  if (warp == 8) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

template <int DH>
static int launch_prompt_umma(const CUtensorMap& km, const CUtensorMap& vm, const UmmaPromptArgs& a, int n_seqs, int max_rows,
                              cudaStream_t s) {
  constexpr int STAGES = DH == 128 ? 4 : 6;
  constexpr size_t smem = 4 * 128 * 128 + static_cast<size_t>(STAGES) * 2 * (DH / 64) * 64 * 128 + (2 * STAGES + 12) * 8 + 16 + 1024;
  static_assert(smem <= 227 * 1024, "shared memory of one CTA");
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(attn_prompt_umma_kernel<DH, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
      set_error("attention_prompt_umma: cannot reserve %zu bytes of shared memory", smem);
      return kCudaError;
    }
    configured = true;
  }
  TIE_LAUNCH((attn_prompt_umma_kernel<DH, STAGES>), dim3(a.kv_heads, ceil_div(max_rows, a.cta_rows), n_seqs), kUmmaAttnThreads, smem, s, km, vm, a);
  return kOk;
}

}  // namespace tie

using namespace tie;

// Rows [0, rows) of the step belong to sequences 0..n_seqs-1, each bringing several tokens;
// max_queries is the largest number of tokens one of them brings; pages is the number of pages
// of the cache planes.
TIE_API int tie_attention_prompt_umma(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                      const int* query_start, const int* context_lens, const int* block_tables,
                                      int max_blocks, int n_seqs, int max_queries, int q_heads, int kv_heads, int head_dim,
                                      int page_size, int pages, int window, float scale, cudaStream_t s) {
  TIE_REQUIRE(head_dim == 64 || head_dim == 128, "attention_prompt_umma: head_dim %d is not 64 or 128", head_dim);
  TIE_REQUIRE(q_heads > 0 && kv_heads > 0 && q_heads % kv_heads == 0 && q_heads / kv_heads <= 16,
              "attention_prompt_umma: %d query heads over %d kv heads (at most 16 per group)", q_heads, kv_heads);
  TIE_REQUIRE(page_size >= 8 && (page_size & (page_size - 1)) == 0, "attention_prompt_umma: page size %d is not a power of two from 8 up", page_size);
  TIE_REQUIRE(q_stride % 8 == 0 && reinterpret_cast<uintptr_t>(q) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "attention_prompt_umma: q and out rows must be 16-byte aligned");
  TIE_REQUIRE(scale > 0.0f, "attention_prompt_umma: the scale must be positive");
  if (n_seqs == 0 || max_queries == 0) return kOk;
  TIE_REQUIRE(static_cast<long long>(max_queries) * (q_heads / kv_heads) <= 65535LL * 256, "attention_prompt_umma: %d queries in one portion are too many", max_queries);
  int shift = 0;
  while ((1 << shift) < page_size) ++shift;
  const int box_rows = page_size < kKeysPerTile ? page_size : kKeysPerTile;
  CUtensorMap km, vm;
  const long long rows = static_cast<long long>(pages) * kv_heads * page_size;
  TIE_REQUIRE(make_map_bf16(&km, k_cache, rows, head_dim, head_dim, 64, box_rows) &&
                  make_map_bf16(&vm, v_cache, rows, head_dim, head_dim, 64, box_rows),
              "attention_prompt_umma: cuTensorMapEncodeTiled failed");
  TIE_REQUIRE(status_word() != nullptr, "attention_prompt_umma: cannot allocate the status word");
  UmmaPromptArgs a{static_cast<const __nv_bfloat16*>(q), static_cast<__nv_bfloat16*>(out), query_start, context_lens, block_tables,
                   status_word(), q_stride, max_blocks, q_heads, kv_heads, page_size, shift, window, scale * 1.4426950408889634f, 256};
  const int max_rows = max_queries * (q_heads / kv_heads);
  // Few rows: with two row tiles a CTA, half of the SMs or more would have none
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  if (static_cast<long long>(kv_heads) * ceil_div(max_rows, 256) * n_seqs * 2 <= sms) a.cta_rows = 128;
  const int st = head_dim == 64 ? launch_prompt_umma<64>(km, vm, a, n_seqs, max_rows, s) : launch_prompt_umma<128>(km, vm, a, n_seqs, max_rows, s);
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("attention_prompt_umma");
}
