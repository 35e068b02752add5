// bfloat16 matrix products for many rows (prompt portions) on pairs of SMs: tcgen05.mma with
// cta_group::2. Two CTAs of a cluster compute one 256 x BN tile of out[M, N] = a[M, K] . w[N, K]^T:
// each CTA stages its own 128 rows of a and its own half of the BN rows of w (32 KB per 64-deep
// k-block at BN = 256 instead of the 48 KB a lone CTA needs for 128 x 256), one thread of the leader CTA
// issues the MMAs for both, and each CTA's tensor memory receives its 128 x BN float
// accumulator. A third less operand traffic from L2 per flop is what this buys; the 1-CTA
// kernel in gemm_tc.cu is limited by exactly that feed. BN is 256, or narrower (multiples of 32 from 128 up)
// where that fills the last wave of tiles better: 128 tiles of 256 x 256 are 1.73 waves on 74 pairs and take
// two; 208 tiles of 256 x 160 take three waves of 0.625 each (the host picks, ops/gemm_select.py).
//
// Per CTA: warps 0-3 epilogue (tcgen05.ld, optional SiLU * up, stores), warp 4 TMA producer,
// warp 5 (leader CTA only) MMA issuer. Barriers: full[s] lives in the leader and counts the
// bytes of BOTH CTAs' loads (the loads carry .cta_group::2 and name the leader's barrier);
// empty[s] and acc_full[b] exist in both CTAs and are signalled by tcgen05.commit with a
// cluster multicast mask; acc_empty[b] lives in the leader and collects the eight epilogue
// warps of the pair. A pair walks the tiles pair, pair + pairs, ...; two accumulators let a
// tile's epilogue overlap the next tile's MMAs. No TMA multicast: every CTA fetches its own operands.
//
// Waits. Every mbarrier wait is bounded (status word as in gemm_tc.cu), and so is the handshake of the pair
// before it frees its tensor memory (`peer_done`: a remote arrive and a bounded wait, code 4). Three waits have
// no limit, because the instruction set gives them none: tcgen05.alloc (returns once 512 columns are free on both
// SMs; this kernel never shares an SM with another holder of tensor memory, since its 225 KB of shared memory
// exclude every kernel of this library that allocates some), the barrier.cluster right behind it (it waits for
// the partner CTA, which the hardware schedules together with this one and which has nothing ahead of it but the
// same allocation), and griddepcontrol.wait (never executed by this kernel as it is launched, see below).
//
// Programmatic dependent launch: the kernel behind this one may start while it runs (launch_dependents at the
// top), but this kernel itself is launched without the attribute and so starts only when the kernel ahead of it
// has finished. Started early, steps of 512 tokens that mixed two prompt portions with decoded tokens (Qwen3-8B
// shapes: 48 pairs of CTAs for the q/k/v product) hung about once in five runs with no bounded wait expired, so
// in one of the waits named above or in the cluster barrier that used to stand at the end; as it is, hundreds of
// runs of the same steps are clean. The prologue this gives up is a few microseconds of a product that takes
// hundreds. The pdl_wait() calls below stay (they return at once for a kernel launched this way) so that the
// order of loads and stores against the kernel ahead does not rest on the launch mode.
#include "umma.cuh"
#include "launchers.h"

namespace tie {

constexpr int k2Threads = 192;
constexpr int k2BK = 64;
constexpr int k2Stages = 7;
constexpr int k2StageA = 128 * k2BK * 2;      // this CTA's 128 rows of a
constexpr int k2StageB = 128 * k2BK * 2;      // this CTA's half of the tile's rows of w (128 at most: BN = 256)
constexpr int k2Stage = k2StageA + k2StageB;  // stages are as large for every BN: narrower tiles leave part of them unused
constexpr int k2TmemCols = 512;               // two accumulators of up to 256 columns
constexpr size_t k2Smem = static_cast<size_t>(k2Stages) * k2Stage + 1024 + 256;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address of `p` (in this CTA's shared memory) as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* p, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(p)), "r"(rank));
  return out;
}
__device__ __forceinline__ void tma_load_2d_pair(void* dst, const CUtensorMap* map, int x, int y, uint32_t leader_bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(smem_u32(dst)), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(leader_bar)
      : "memory");
}
__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once the MMAs issued so far retire.
__device__ __forceinline__ void umma2_commit_both(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void remote_arrive(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

template <typename OutT, int BN>
__global__ void __launch_bounds__(k2Threads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, OutT* __restrict__ out,
                int M, int N, int k_blocks, long long ldo, int silu, int tiles_m, int n_tiles, int* status, int w_rows, int w_row0) {
  pdl_launch_dependents();
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + k2Stages * k2Stage);   // used in the leader
  uint64_t* empty = full + k2Stages;                                         // both CTAs
  uint64_t* acc_full = empty + k2Stages;                                     // [2], both CTAs
  uint64_t* acc_empty = acc_full + 2;                                        // [2], used in the leader
  uint64_t* peer_done = acc_empty + 2;                                       // both CTAs: the partner is through
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(peer_done + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < k2Stages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 8);     // four epilogue warps of each CTA of the pair
    }
    mbar_init(peer_done, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(k2TmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  cluster_sync();      // both CTAs' barriers exist before anyone signals across the pair
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 4) {
    // ---- TMA producer (both CTAs): own rows of a, own half of the tile's rows of w; bytes count on the leader's barrier
    // The whole warp walks the loop (uniform) and one elected lane issues.
    {
      int s = 0;
      uint32_t parity = 1;   // a fresh barrier passes a wait on parity 1
      bool first = true, ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += pairs) {
        const int row_a = (tile % tiles_m) * 256 + static_cast<int>(rank) * 128;
        const int row_w = (tile / tiles_m) * BN + static_cast<int>(rank) * (BN / 2);
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(empty + s, parity, abort_flag, status, 1) ? 1 : 0)) {
            ok = false;
            break;
          }
          const uint32_t bar = map_to_cta(full + s, 0);
          uint8_t* sa = smem + s * k2Stage;
          if (elect_one()) {
            if (rank == 0) mbar_expect_tx(full + s, 2 * (k2StageA + (BN / 2) * k2BK * 2));
            // weights never change: before the wait. Stored in k-blocks (w_rows > 0) a box is 16 KB in one piece.
            if (w_rows > 0) tma_load_2d_pair(sa + k2StageA, &map_w, 0, kb * w_rows + w_row0 + row_w, bar);
            else tma_load_2d_pair(sa + k2StageA, &map_w, kb * k2BK, row_w, bar);
          }
          __syncwarp();
          if (first) {
            first = false;
            pdl_wait();
          }
          if (elect_one()) tma_load_2d_pair(sa, &map_a, kb * k2BK, row_a, bar);
          __syncwarp();
          if (++s == k2Stages) {
            s = 0;
            parity ^= 1;
          }
        }
      }
      if (first) pdl_wait();
    }
  } else if (warp == 5) {
    // ---- MMA issuer: a warp of the leader CTA walks the loop (uniform), one elected lane drives both CTAs' tensor cores
    if (rank == 0) {
      constexpr uint32_t idesc = instr_desc(BN, 256);
      const uint32_t ring_lo = desc_lo_sw128(smem_u32(smem));   // descriptors as (low word, constant high word)
      int s = 0, local = 0;
      uint32_t parity = 0;
      bool ok = true;
      for (int tile = pair; tile < n_tiles && ok; tile += pairs, ++local) {
        const int buf = local & 1;
        if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1, abort_flag, status, 2) ? 1 : 0)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * 256;      // the second accumulator at column 256 whatever BN
        for (int kb = 0; kb < k_blocks; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(full + s, parity, abort_flag, status, 2) ? 1 : 0)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_lo = ring_lo + s * (k2Stage >> 4), b_lo = a_lo + (k2StageA >> 4);
          const uint32_t keep = kb > 0 ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < k2BK / 16; ++k) {
              umma2_bf16(tmem_acc, desc_from_words(a_lo + 2 * k, kDescHiSw128), desc_from_words(b_lo + 2 * k, kDescHiSw128), idesc,
                         k > 0 ? 1u : keep);
            }
            umma2_commit_both(empty + s);
          }
          __syncwarp();
          if (++s == k2Stages) {
            s = 0;
            parity ^= 1;
          }
        }
        if (ok && elect_one()) umma2_commit_both(acc_full + buf);
        __syncwarp();
      }
    }
  } else {
    // ---- epilogue (both CTAs): rows i0 .. i0 + 127 of the pair's tile, all 256 columns
    int local = 0;
    for (int tile = pair; tile < n_tiles; tile += pairs, ++local) {
      const int buf = local & 1;
      const int i0 = (tile % tiles_m) * 256 + static_cast<int>(rank) * 128, j0 = (tile / tiles_m) * BN;
      if (!mbar_wait(acc_full + buf, (local >> 1) & 1, abort_flag, status, 3)) break;
      if (local == 0) pdl_wait();
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + buf * 256;
      const int i = i0 + warp * 32 + lane;
      if (silu) {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 32) {
          if (j0 + c0 >= N) break;
          uint32_t g[16], u[16];
          tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, g);
          tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0 + 16, u);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (i < M) {
            float v[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) {
              const float gv = __uint_as_float(g[e]);
              v[e] = gv / (1.0f + expf(-gv)) * __uint_as_float(u[e]);
            }
            const long long at = static_cast<long long>(i) * ldo + ((j0 + c0) >> 1);
            if (((at * sizeof(OutT)) & 15) == 0 && sizeof(OutT) == 2) {
              uint32_t w[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * e], v[2 * e + 1]);
                w[e] = *reinterpret_cast<const uint32_t*>(&h);
              }
              *reinterpret_cast<uint4*>(out + at) = make_uint4(w[0], w[1], w[2], w[3]);
              *reinterpret_cast<uint4*>(out + at + 8) = make_uint4(w[4], w[5], w[6], w[7]);
            } else {
#pragma unroll
              for (int e = 0; e < 16; ++e) st(out + at + e, v[e]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          if (j0 + c0 >= N) break;
          uint32_t r[16];
          tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (i < M) {
            const long long at = static_cast<long long>(i) * ldo + j0 + c0;
            const int n = min(16, N - (j0 + c0));
            if (n == 16 && ((at * sizeof(OutT)) & 15) == 0) {
              if constexpr (sizeof(OutT) == 2) {
                uint32_t w[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(r[2 * e]), __uint_as_float(r[2 * e + 1]));
                  w[e] = *reinterpret_cast<const uint32_t*>(&h);
                }
                *reinterpret_cast<uint4*>(out + at) = make_uint4(w[0], w[1], w[2], w[3]);
                *reinterpret_cast<uint4*>(out + at + 8) = make_uint4(w[4], w[5], w[6], w[7]);
              } else {
#pragma unroll
                for (int e = 0; e < 16; e += 4)
                  *reinterpret_cast<uint4*>(out + at + e) = make_uint4(r[e], r[e + 1], r[e + 2], r[e + 3]);
              }
            } else {
              for (int e = 0; e < n; ++e) st(out + at + e, __uint_as_float(r[e]));
            }
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) remote_arrive(map_to_cta(acc_empty + buf, 0));   // the leader's MMA thread may reuse this accumulator
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag != 0) {
    const unsigned long long t0 = clock64();
    while (clock64() - t0 < 4000000ull) {
    }
  }
  // Neither CTA leaves, or frees tensor memory, while its partner may still touch its shared or tensor memory:
  // each tells the other that it is through and waits (with the limit of every other wait) to be told. The
  // partner's arrive is its last access to this CTA's memory, and it comes before this wait can return.
  // A CTA that gave up a wait still waits here for its partner, which may need a limit of its own to get
  // here, so this limit is twice the usual one and does not look at the abort flag.
  if (threadIdx.x == 0) {
    remote_arrive(map_to_cta(peer_done, rank ^ 1u));
    const unsigned long long t0 = clock64();
    while (!mbar_try_wait(peer_done, 0)) {
      if (clock64() - t0 > 2 * kWaitCycles) {
        *reinterpret_cast<volatile int*>(status) = 4;
        break;
      }
    }
  }
  __syncthreads();
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(k2TmemCols) : "memory");
  }
}

// Pairs of SMs that can hold the kernel at once (SMs pair up inside a GPC, so it may be fewer than half the SMs);
// 0 if the query fails. The same for every instantiation: they differ in neither threads nor shared memory.
static int resident_pairs() {
  static int pairs = -1;
  if (pairs < 0) {
    pairs = 0;
    if (cudaFuncSetAttribute(gemm_tc2_kernel<__nv_bfloat16, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(k2Smem)) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.blockDim = dim3(k2Threads);
      cfg.dynamicSmemBytes = k2Smem;
      cfg.gridDim = dim3(2 * 74);
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel<__nv_bfloat16, 256>, &cfg) == cudaSuccess && n >= 1) pairs = n;
      else cudaGetLastError();
    }
  }
  return pairs;
}

template <typename OutT, int BN>
static int launch_tc2(const CUtensorMap& ma, const CUtensorMap& mw, void* out, int M, int N, int K, long long ldo, int silu,
                      int w_rows, int w_row0, cudaStream_t s) {
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc2_kernel<OutT, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(k2Smem)) != cudaSuccess) {
      set_error("gemm_tc2: cannot reserve %zu bytes of shared memory", k2Smem);
      return kCudaError;
    }
    configured = true;
  }
  const int tiles_m = ceil_div(M, 256), n_tiles = tiles_m * ceil_div(N, BN);
  cudaLaunchConfig_t cfg = {};
  cfg.blockDim = dim3(k2Threads);
  cfg.dynamicSmemBytes = k2Smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[1];     // the cluster shape and nothing else: no early start (see the top of this file)
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 2;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = 1;
  const int resident = resident_pairs();
  if (resident < 1) {
    set_error("gemm_tc2: no pair of SMs can hold the kernel");
    return kCudaError;
  }
  const int pairs = n_tiles < resident ? n_tiles : resident;
  cfg.gridDim = dim3(2 * pairs);
  cudaLaunchKernelEx(&cfg, gemm_tc2_kernel<OutT, BN>, ma, mw, static_cast<OutT*>(out), M, N, ceil_div(K, k2BK), ldo, silu, tiles_m,
                     n_tiles, status_word(), w_rows, w_row0);
  return kOk;
}

}  // namespace tie

using namespace tie;

// out[M, N] (or, with silu, out[M, N / 2] = silu(gate) * up for w in blocks of 16 gate + 16 up rows)
// = a[M, K] . w[N, K]^T on pairs of SMs. a, w bfloat16 with K and row strides multiples of 8. w_rows > 0: w is
// stored in k-blocks, [ceil(K / 64)][w_rows][64], and the product uses its rows w_row0 .. w_row0 + N - 1 (gemm_tc.cu).
// How many pairs of SMs hold the kernel at once: what the host counts waves of tiles with.
TIE_API int tie_gemm_tc2_pairs() { return resident_pairs(); }

// bn: the tile width, 128, 160, 192, 224 or 256 (0: 256).
TIE_API int tie_gemm_tc2(int out_dtype, const void* a, const void* w, void* out, int M, int N, int K, long long lda,
                         long long ldw, long long ldo, int silu, int w_rows, int w_row0, int bn, cudaStream_t s) {
  if (bn == 0) bn = 256;
  TIE_REQUIRE(bn == 128 || bn == 160 || bn == 192 || bn == 224 || bn == 256, "gemm_tc2: tile width %d", bn);
  TIE_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc2: bad sizes M=%d N=%d K=%d", M, N, K);
  TIE_REQUIRE(K % 8 == 0 && lda % 8 == 0 && (w_rows > 0 || ldw % 8 == 0), "gemm_tc2: K=%d and the row strides must be multiples of 8", K);
  TIE_REQUIRE(w_rows == 0 || (w_row0 >= 0 && w_row0 + N <= w_rows), "gemm_tc2: rows %d..%d of a weight of %d rows", w_row0, w_row0 + N, w_rows);
  TIE_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
              "gemm_tc2: operands must be 16-byte aligned");
  TIE_REQUIRE(out_dtype == TIE_BF16 || out_dtype == TIE_F32, "gemm_tc2: output dtype code %d", out_dtype);
  TIE_REQUIRE(!silu || N % 32 == 0, "gemm_tc2: the SiLU epilogue needs weight rows in blocks of 16 gate + 16 up (N=%d)", N);
  TIE_REQUIRE(status_word() != nullptr, "gemm_tc2: cannot allocate the status word");
  CUtensorMap ma, mw;
  const bool w_ok = w_rows > 0 ? make_map_bf16(&mw, w, static_cast<long long>(ceil_div(K, k2BK)) * w_rows, k2BK, k2BK, k2BK, bn / 2)
                               : make_map_bf16(&mw, w, N, K, ldw, k2BK, bn / 2);
  TIE_REQUIRE(make_map_bf16(&ma, a, M, K, lda, k2BK, 128) && w_ok, "gemm_tc2: cuTensorMapEncodeTiled failed (M %d, N %d, K %d)", M, N, K);
  int st = kOk;
#define TIE_TC2_CASE(B)                                                                                                  \
  case B:                                                                                                                \
    st = out_dtype == TIE_BF16 ? launch_tc2<__nv_bfloat16, B>(ma, mw, out, M, N, K, ldo, silu, w_rows, w_row0, s)         \
                               : launch_tc2<float, B>(ma, mw, out, M, N, K, ldo, silu, w_rows, w_row0, s);                \
    break;
  switch (bn) {
    TIE_TC2_CASE(128)
    TIE_TC2_CASE(160)
    TIE_TC2_CASE(192)
    TIE_TC2_CASE(224)
    TIE_TC2_CASE(256)
  }
#undef TIE_TC2_CASE
  if (st != kOk) return st;
  TIE_RETURN_LAUNCH("gemm_tc2");
}
