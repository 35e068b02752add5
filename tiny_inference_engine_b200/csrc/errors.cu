// The last error message of a launcher, per thread, and the library's version probe.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "tma.cuh"

namespace tie {
static thread_local char g_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
}
bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("TIE_NO_PDL");
    return !(v != nullptr && v[0] == '1');
  }();
  return on;
}
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime, so the library does not link against libcuda.
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  }
  return fn;
}

bool make_map_bf16(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols,
                   int box_rows) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return false;
  const cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  const cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2};
  const cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  const cuuint32_t elem[2] = {1, 1};
  return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, elem,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int* g_status_host = nullptr;
static int* g_status_dev = nullptr;

int* status_word() {
  if (g_status_host == nullptr) {
    if (cudaHostAlloc(reinterpret_cast<void**>(&g_status_host), sizeof(int), cudaHostAllocMapped) != cudaSuccess) return nullptr;
    *g_status_host = 0;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&g_status_dev), g_status_host, 0) != cudaSuccess) return nullptr;
  }
  return g_status_dev;
}
}  // namespace tie

// 0 when no kernel gave up a bounded wait since the last call; else where the first... the last one did:
// 1 = a matrix product's TMA producer on a free stage, 2 = its MMA issuer on landed bytes, 3 = its
// epilogue on the accumulator, 4 = a CTA of a pair on its partner at the end; 11 = an attention kernel's
// producer, 12 = its consumers, 13 = a context that needs more splits than the call allowed (nothing written for it).
// Reading clears it. Call after the stream has been synchronized.
TIE_API int tie_kernel_status() {
  if (tie::g_status_host == nullptr) return 0;
  const int v = *reinterpret_cast<volatile int*>(tie::g_status_host);
  *tie::g_status_host = 0;
  return v;
}

TIE_API const char* tie_last_error() { return tie::g_error; }

// The architecture this library was compiled for, so that Python can refuse another GPU loudly.
TIE_API int tie_compiled_arch() { return 100; }
