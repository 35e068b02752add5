// bfloat16 matrix products on the 5th-generation tensor cores (tcgen05), operands staged by TMA,
// accumulators in tensor memory:  out[M, N] = a[M, K] . w[N, K]^T, float accumulation.
//
// One CTA computes a 128 x BN tile of  P[i, j] = sum_k X[i, k] Y[j, k]  where X (the
// "row operand", 128 rows per tile) and Y (the "column operand", BN rows per tile, BN in
// {16, 32, 64, 128, 256}) are both k-contiguous, which is how activations [T, K] and
// checkpoint weights [out, in] are stored (the reference's matmul contract,
// src/backend/backend.h:44-50: y = x . W^T). Two ways to map a product onto it:
//   plain       X = activations, Y = weights : prompt portions (many tokens).
//   transposed  X = weights, Y = activations : few tokens (decode). The 128-row side of the
//               MMA is filled by weight rows, the tokens are the narrow BN side, so no
//               tensor-core work is wasted on padding and every weight byte streams through
//               shared memory exactly once. The epilogue writes P transposed.
// The weights may be stored row-major [rows, K] or in k-blocks (`w_rows` > 0): [K / 64][w_rows][64], all rows'
// 64 elements of k-block 0, then of k-block 1, and so on, so that the 128 x 64 box a stage loads is 16 KB of
// consecutive memory instead of 128 pieces of 128 bytes a row pitch apart (measured on the longest stream, the
// gate/up weights of a decode step: 6.45 against 5.87 TB/s). The operand then starts at row `w_row0` of every
// k-block (a row slice of a stacked weight needs no copy). A box that ends beyond the operand's rows holds rows
// of the next k-block there; they only reach outputs that the epilogue does not write.
// With `splits` > 1 the k range is cut into equal parts along gridDim.z; each part writes
// float partial sums to scratch memory and a second kernel adds them in split order
// (deterministic; no atomics).
//
// Roles inside a CTA of 192 threads: warps 0-3 read the accumulator out of tensor memory
// (warp w owns lanes 32w..32w+31) and store it, warp 4 issues the TMA loads, warp 5 issues
// the MMAs. A ring of STAGES shared-memory stages is handed back and forth with mbarriers:
// full[s] (TMA bytes landed) and empty[s] (the MMAs that read stage s retired, signalled by
// tcgen05.commit). Every wait is bounded: when it runs out the kernel records where in a
// status word, stops waiting, frees its tensor memory and returns; the host reads the word.
// No TMA multicast is used anywhere.
#include "umma.cuh"
#include "launchers.h"

namespace tie {

constexpr int kBM = 128;          // rows of the row operand per tile = MMA M
constexpr int kBK = 64;           // k per stage: 64 bf16 = 128 bytes = one swizzle row
constexpr int kUmmaK = 16;        // k per tcgen05.mma for 16-bit inputs
constexpr int kThreads = 192;

// DEEP: as many stages as fit in the 227 KB one CTA may use (at most 8), one CTA per SM.
// Not DEEP: about 100 KB of stages, so that two CTAs share an SM and one's start-up and
// epilogue hide behind the other's streaming.
template <int BN, bool DEEP> struct TcConfig {
  static constexpr int kStageA = kBM * kBK * 2;
  static constexpr int kStageB = BN * kBK * 2;
  static constexpr int kStage = kStageA + kStageB;
  static constexpr int kBudget = DEEP ? 200 * 1024 : 100 * 1024;
  static constexpr int kFit = kBudget / kStage < 2 ? 2 : kBudget / kStage;
  static constexpr int kStages = kFit > 8 ? 8 : kFit;
  static constexpr int kTmemCols = 2 * BN < 32 ? 32 : 2 * BN;   // two accumulators
  static constexpr size_t kSmem = static_cast<size_t>(kStages) * kStage + 1024 /*alignment*/ + 256 /*barriers*/;
  static_assert(2 * kStages * 8 + 4 * 8 + 16 <= 256, "barriers do not fit");
};

// out: OutT out[i * ldo + j] (plain) or out[j * ldo + i] (transposed); with partial != nullptr the
// same two layouts in float at partial + z * part_stride (row stride ldp). A CTA walks the
// output tiles blockIdx.x, blockIdx.x + gridDim.x, ... (tile t covers rows 128 * (t % tiles_x)
// of the row operand and BN * (t / tiles_x) of the column operand); two accumulators in tensor
// memory let the MMAs of the next tile run while the epilogue drains the last one.
template <int BN, typename OutT, bool DEEP>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_y, OutT* __restrict__ out,
               float* __restrict__ partial, long long part_stride, long long ldp, int rows_x, int rows_y, int k_blocks,
               int k_blocks_per_split, long long ldo, int transposed, int silu, int tiles_x, int n_tiles, int* status,
               int w_rows, int w_row0) {
  pdl_launch_dependents();   // the next kernel may get resident now; it waits for this one at its own pdl_wait()
  using C = TcConfig<BN, DEEP>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + C::kStages * C::kStage);
  uint64_t* empty = full + C::kStages;
  uint64_t* acc_full = empty + C::kStages;     // [2]
  uint64_t* acc_empty = acc_full + 2;          // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb_begin = blockIdx.z * k_blocks_per_split;
  const int kb_end = min(k_blocks, kb_begin + k_blocks_per_split);

  if (threadIdx.x == 0) {
    for (int s = 0; s < C::kStages; ++s) {
      mbar_init(full + s, 1);
      mbar_init(empty + s, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(acc_full + b, 1);
      mbar_init(acc_empty + b, 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 4) {  // this warp owns the tensor memory: it allocates here and frees at the end
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(C::kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 4) {
    // ---- TMA producer. The weights never change, so their tiles of the first stages are fetched
    // before this kernel waits for the one before it; the activations only after.
    // The whole warp walks the loop (uniform) and one elected lane issues, so that addresses and
    // coordinates live in uniform registers.
    {
      int s = 0;
      uint32_t parity = 1;   // a fresh barrier passes a wait on parity 1
      bool first = true, ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
        const int i0 = (tile % tiles_x) * kBM, j0 = (tile / tiles_x) * BN;
        int kb = kb_begin;
        if (first) {
          first = false;
          const CUtensorMap* map_static = transposed ? &map_x : &map_y;
          const CUtensorMap* map_dynamic = transposed ? &map_y : &map_x;
          const int off_static = transposed ? 0 : C::kStageA, off_dynamic = transposed ? C::kStageA : 0;
          const int row_static = transposed ? i0 : j0, row_dynamic = transposed ? j0 : i0;
          const int pre = min(C::kStages, kb_end - kb_begin);
          if (elect_one()) {
            for (int p = 0; p < pre; ++p) {   // fresh barriers: the stages are free
              mbar_expect_tx(full + p, C::kStage);
              if (w_rows > 0)
                tma_load_2d(smem + p * C::kStage + off_static, map_static, 0, (kb_begin + p) * w_rows + w_row0 + row_static, full + p);
              else
                tma_load_2d(smem + p * C::kStage + off_static, map_static, (kb_begin + p) * kBK, row_static, full + p);
            }
          }
          __syncwarp();
          pdl_wait();
          if (elect_one()) {
            for (int p = 0; p < pre; ++p) {
              tma_load_2d(smem + p * C::kStage + off_dynamic, map_dynamic, (kb_begin + p) * kBK, row_dynamic, full + p);
            }
          }
          __syncwarp();
          kb = kb_begin + pre;
          s = pre;
          if (s == C::kStages) {
            s = 0;
            parity = 0;
          }
        }
        for (; kb < kb_end; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(empty + s, parity, abort_flag, status, 1) ? 1 : 0)) {
            ok = false;
            break;
          }
          if (elect_one()) {
            uint8_t* sa = smem + s * C::kStage;
            mbar_expect_tx(full + s, C::kStage);
            // the weights are the row operand when transposed, else the column operand
            if (w_rows > 0 && transposed) tma_load_2d(sa, &map_x, 0, kb * w_rows + w_row0 + i0, full + s);
            else tma_load_2d(sa, &map_x, kb * kBK, i0, full + s);
            if (w_rows > 0 && !transposed) tma_load_2d(sa + C::kStageA, &map_y, 0, kb * w_rows + w_row0 + j0, full + s);
            else tma_load_2d(sa + C::kStageA, &map_y, kb * kBK, j0, full + s);
          }
          __syncwarp();
          if (++s == C::kStages) {
            s = 0;
            parity ^= 1;
          }
        }
      }
    }
  } else if (warp == 5) {
    // ---- MMA issuer: the whole warp walks the loop (uniform), one elected lane issues
    {
      constexpr uint32_t idesc = instr_desc(BN);
      const uint32_t ring_lo = desc_lo_sw128(smem_u32(smem));   // descriptors as (low word, constant high word)
      int s = 0, local = 0;
      uint32_t parity = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++local) {
        const int buf = local & 1;
        // the epilogue has drained this accumulator
        if (!__all_sync(0xffffffffu, mbar_wait(acc_empty + buf, ((local >> 1) & 1) ^ 1, abort_flag, status, 2) ? 1 : 0)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!__all_sync(0xffffffffu, mbar_wait(full + s, parity, abort_flag, status, 2) ? 1 : 0)) {
            ok = false;
            break;
          }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_lo = ring_lo + s * (C::kStage >> 4), b_lo = a_lo + (C::kStageA >> 4);
          const uint32_t keep = kb > kb_begin ? 1u : 0u;
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              umma_bf16(tmem_acc, desc_from_words(a_lo + ((k * kUmmaK * 2) >> 4), kDescHiSw128),
                        desc_from_words(b_lo + ((k * kUmmaK * 2) >> 4), kDescHiSw128), idesc, k > 0 ? 1u : keep);
            }
            umma_commit(empty + s);   // arrives once the MMAs above have read the stage
          }
          __syncwarp();
          if (++s == C::kStages) {
            s = 0;
            parity ^= 1;
          }
        }
        if (ok && elect_one()) umma_commit(acc_full + buf);
        __syncwarp();
      }
    }
  } else {
    // ---- epilogue: warp w reads lanes 32w..32w+31, 16 columns at a time
    float* part = partial ? partial + static_cast<long long>(blockIdx.z) * part_stride : nullptr;
    int local = 0;
    for (int tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++local) {
      const int buf = local & 1;
      const int i0 = (tile % tiles_x) * kBM, j0 = (tile / tiles_x) * BN;
      if (!mbar_wait(acc_full + buf, (local >> 1) & 1, abort_flag, status, 3)) break;
      if (local == 0) pdl_wait();   // nothing is stored before the kernels ahead in the stream are done
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + buf * BN;
      const int i = i0 + warp * 32 + lane;
      if (silu) {
        // The weight rows come in blocks of 16 gate rows followed by their 16 up rows; the output is
        // silu(gate) * up, half as wide as the product: out[token, 16 * block + r].
        if (transposed) {
          // lanes 0-15 of a warp hold gate rows, lanes 16-31 the matching up rows: exchange, then
          // the lower half finishes columns 0-7 of each chunk and the upper half columns 8-15
          const int o = (i0 >> 1) + warp * 16 + (lane & 15);
          const bool upper = lane >= 16;
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 16) {
            if (j0 + c0 >= rows_y) break;
            uint32_t r[16];
            tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              // the lower lane sends its gate of column e + 8 and receives the up of column e;
              // the upper lane sends its up of column e and receives the gate of column e + 8
              const uint32_t got = __shfl_xor_sync(0xffffffffu, upper ? r[e] : r[e + 8], 16);
              const float g = __uint_as_float(upper ? got : r[e]);
              const float u = __uint_as_float(upper ? r[e + 8] : got);
              const int j = j0 + c0 + e + (upper ? 8 : 0);
              if (j < rows_y && o < (rows_x >> 1)) st(out + static_cast<long long>(j) * ldo + o, g / (1.0f + expf(-g)) * u);
            }
          }
        } else {
#pragma unroll 1
          for (int c0 = 0; c0 < BN; c0 += 32) {
            if (j0 + c0 >= rows_y) break;
            uint32_t g[16], u[16];
            tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, g);
            tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0 + 16, u);
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (i < rows_x) {
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
        }
      } else {
#pragma unroll 1
        for (int c0 = 0; c0 < BN; c0 += 16) {
          if (j0 + c0 >= rows_y) break;   // uniform over the warp
          uint32_t r[16];
          tmem_ld16(tmem_acc + (static_cast<uint32_t>(warp * 32) << 16) + c0, r);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
          if (i < rows_x) {
            if (transposed) {
#pragma unroll
              for (int e = 0; e < 16; ++e) {
                const int j = j0 + c0 + e;
                if (j < rows_y) {
                  if (part) part[static_cast<long long>(j) * ldp + i] = __uint_as_float(r[e]);
                  else st(out + static_cast<long long>(j) * ldo + i, __uint_as_float(r[e]));
                }
              }
            } else {
              const long long at = static_cast<long long>(i) * ldo + j0 + c0;
              const int n = min(16, rows_y - (j0 + c0));
              if (part) {
                const long long pat = static_cast<long long>(i) * ldp + j0 + c0;
                if (n == 16 && (pat & 3) == 0) {
#pragma unroll
                  for (int e = 0; e < 16; e += 4)
                    *reinterpret_cast<uint4*>(part + pat + e) = make_uint4(r[e], r[e + 1], r[e + 2], r[e + 3]);
                } else {
                  for (int e = 0; e < n; ++e) part[pat + e] = __uint_as_float(r[e]);
                }
              } else if (n == 16 && ((at * sizeof(OutT)) & 15) == 0) {
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
      }
      // this accumulator may be overwritten by the tile after next
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(acc_empty + buf)) : "memory");
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag != 0) {  // a wait ran out: give copies that are still in flight time to land before the CTA goes away
    const unsigned long long t0 = clock64();
    while (clock64() - t0 < 4000000ull) {
    }
    __syncthreads();
  }
  if (warp == 4) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(C::kTmemCols) : "memory");
  }
}

// out[m, n] = sum over splits of partial[z][m, n], in split order, converted to OutT.
template <typename OutT>
__global__ void splitk_reduce_kernel(const float* __restrict__ partial, long long part_stride, int splits,
                                     OutT* __restrict__ out, long long ldo, int N, long long total) {
  pdl_sync();
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  float acc = partial[idx];
  for (int z = 1; z < splits; ++z) acc += partial[static_cast<long long>(z) * part_stride + idx];
  st(out + (idx / N) * ldo + idx % N, acc);
}

// ---------------------------------------------------------------------------------------------
// Host side

template <int BN, typename OutT, bool DEEP>
static int launch_tc(const CUtensorMap& mx, const CUtensorMap& my, void* out, float* partial, long long part_stride,
                     long long ldp, int rows_x, int rows_y, int K, long long ldo, int transposed, int silu, int splits, int w_rows,
                     int w_row0, cudaStream_t s) {
  using C = TcConfig<BN, DEEP>;
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(gemm_tc_kernel<BN, OutT, DEEP>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(C::kSmem)) != cudaSuccess) {
      set_error("gemm_tc: cannot reserve %zu bytes of shared memory", C::kSmem);
      return kCudaError;
    }
    configured = true;
  }
  const int k_blocks = ceil_div(K, kBK);
  const int per_split = ceil_div(k_blocks, splits);
  const int tiles_x = ceil_div(rows_x, kBM), n_tiles = tiles_x * ceil_div(rows_y, BN);
  const int z = ceil_div(k_blocks, per_split);
  // one CTA per SM walks the tiles when there are more tiles than SMs (deep ring); the narrow
  // rings (two CTAs per SM) get one CTA per tile
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0);
  const int ctas = DEEP ? (n_tiles * z > sms ? max(1, sms / z) : n_tiles) : n_tiles;
  const dim3 grid(min(ctas, n_tiles), 1, z);
  TIE_LAUNCH((gemm_tc_kernel<BN, OutT, DEEP>), grid, kThreads, C::kSmem, s, mx, my, static_cast<OutT*>(out), partial, part_stride, ldp,
             rows_x, rows_y, k_blocks, per_split, ldo, transposed, silu, tiles_x, n_tiles, status_word(), w_rows, w_row0);
  return kOk;
}

}  // namespace tie

using namespace tie;

// out[M, N] (OutT = bfloat16 or float, row stride ldo) = a[M, K] . w[N, K]^T, a and w bfloat16.
// transposed != 0 puts the weights on the 128-row side (few tokens). splits > 1 needs `scratch`
// with tie_gemm_tc_scratch_floats floats: the float partial sums [splits, M, N]; with reduce == 0
// they are left there for a consumer that adds them itself (tie_gemm_tc_real_splits says how
// many there are). silu != 0: w holds blocks of 16 gate rows followed by their 16 up rows and
// out[M, N / 2] = silu(gate) * up. deep != 0: the deepest shared-memory ring (one CTA per SM), else
// a ring of about 100 KB (two CTAs per SM). Returns kBadArgument
// with a message for sizes it does not take (K or a row stride not a multiple of 8, unaligned
// pointers): the caller then uses the CUDA-core kernel.
// How many splits a call with `splits` really makes (the k-blocks are divided evenly).
TIE_API int tie_gemm_tc_real_splits(int K, int splits) {
  const int k_blocks = ceil_div(K, kBK);
  return ceil_div(k_blocks, ceil_div(k_blocks, splits > 0 ? splits : 1));
}

TIE_API long long tie_gemm_tc_scratch_floats(int M, int N, int splits) {
  return splits > 1 ? static_cast<long long>(splits) * M * N : 0;
}

// w_rows > 0: w is stored in k-blocks, [ceil(K / 64)][w_rows][64] (zeros beyond K), and the product uses its rows
// w_row0 .. w_row0 + N - 1; ldw is then ignored.
TIE_API int tie_gemm_tc(int out_dtype, const void* a, const void* w, void* out, int M, int N, int K, long long lda,
                        long long ldw, long long ldo, int transposed, int bn, int splits, float* scratch, int silu,
                        int reduce, int deep, int w_rows, int w_row0, cudaStream_t s) {
  TIE_REQUIRE(M > 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
  TIE_REQUIRE(K % 8 == 0 && lda % 8 == 0 && (w_rows > 0 || ldw % 8 == 0), "gemm_tc: K=%d and the row strides must be multiples of 8", K);
  TIE_REQUIRE(w_rows == 0 || (w_row0 >= 0 && w_row0 + N <= w_rows), "gemm_tc: rows %d..%d of a weight of %d rows", w_row0, w_row0 + N, w_rows);
  TIE_REQUIRE(reinterpret_cast<uintptr_t>(a) % 16 == 0 && reinterpret_cast<uintptr_t>(w) % 16 == 0,
              "gemm_tc: operands must be 16-byte aligned");
  TIE_REQUIRE(bn == 16 || bn == 32 || bn == 64 || bn == 128 || bn == 256, "gemm_tc: tile width %d", bn);
  TIE_REQUIRE(splits >= 1 && (splits == 1 || scratch != nullptr), "gemm_tc: splits=%d needs scratch memory", splits);
  TIE_REQUIRE(out_dtype == TIE_BF16 || out_dtype == TIE_F32, "gemm_tc: output dtype code %d", out_dtype);
  TIE_REQUIRE(!silu || (splits == 1 && N % 32 == 0 && (transposed || bn >= 32)),
              "gemm_tc: the SiLU epilogue needs unsplit k and weight rows in blocks of 16 gate + 16 up (N=%d)", N);
  TIE_REQUIRE(status_word() != nullptr, "gemm_tc: cannot allocate the status word");
  // row operand X (128 per tile) and column operand Y (bn per tile)
  const void* x = transposed ? w : a;
  const void* y = transposed ? a : w;
  const int rows_x = transposed ? N : M, rows_y = transposed ? M : N;
  const long long ldx = transposed ? ldw : lda, ldy = transposed ? lda : ldw;
  CUtensorMap mx, my;
  const long long kb_rows = static_cast<long long>(ceil_div(K, kBK)) * w_rows;   // rows of the weight seen as [k-blocks x rows, 64]
  const bool x_ok = (w_rows > 0 && transposed) ? make_map_bf16(&mx, x, kb_rows, kBK, kBK, kBK, kBM) : make_map_bf16(&mx, x, rows_x, K, ldx, kBK, kBM);
  const bool y_ok = (w_rows > 0 && !transposed) ? make_map_bf16(&my, y, kb_rows, kBK, kBK, kBK, bn) : make_map_bf16(&my, y, rows_y, K, ldy, kBK, bn);
  TIE_REQUIRE(x_ok && y_ok, "gemm_tc: cuTensorMapEncodeTiled failed (rows %d/%d, K %d)", rows_x, rows_y, K);
  float* partial = splits > 1 ? scratch : nullptr;
  const long long part_stride = static_cast<long long>(M) * N;
  const long long ldp = N;
  int st = kOk;
#define TIE_TC_ARGS mx, my, out, partial, part_stride, ldp, rows_x, rows_y, K, ldo, transposed, silu, splits, w_rows, w_row0, s
#define TIE_TC_CASE(B)                                                                                     \
  case B:                                                                                                  \
    if (deep) {                                                                                            \
      st = out_dtype == TIE_BF16 ? launch_tc<B, __nv_bfloat16, true>(TIE_TC_ARGS) : launch_tc<B, float, true>(TIE_TC_ARGS);   \
    } else {                                                                                               \
      st = out_dtype == TIE_BF16 ? launch_tc<B, __nv_bfloat16, false>(TIE_TC_ARGS) : launch_tc<B, float, false>(TIE_TC_ARGS); \
    }                                                                                                      \
    break;
  switch (bn) {
    TIE_TC_CASE(16)
    TIE_TC_CASE(32)
    TIE_TC_CASE(64)
    TIE_TC_CASE(128)
    TIE_TC_CASE(256)
  }
#undef TIE_TC_ARGS
#undef TIE_TC_CASE
  if (st != kOk) return st;
  if (splits > 1 && reduce) {
    const int k_blocks = ceil_div(K, kBK);
    const int real_splits = ceil_div(k_blocks, ceil_div(k_blocks, splits));
    const long long total = part_stride;
    if (out_dtype == TIE_BF16) {
      TIE_LAUNCH((splitk_reduce_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, 
          partial, part_stride, real_splits, static_cast<__nv_bfloat16*>(out), ldo, N, total);
    } else {
      TIE_LAUNCH((splitk_reduce_kernel<float>), ceil_div(total, 256), 256, 0, s, partial, part_stride, real_splits,
                                                                      static_cast<float*>(out), ldo, N, total);
    }
  }
  TIE_RETURN_LAUNCH("gemm_tc");
}
