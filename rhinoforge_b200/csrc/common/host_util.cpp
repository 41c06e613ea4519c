#include "host_util.h"

#include <cudaTypedefs.h>
#include <stdarg.h>
#include <stdlib.h>

#include <atomic>
#include <mutex>

namespace rf {

static thread_local std::string g_last_error;

void set_error(const std::string& msg) { g_last_error = msg; }

int fail(int code, const char* fmt, ...) {
  char buf[1024];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof(buf), fmt, ap);
  va_end(ap);
  g_last_error = buf;
  return code;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tmap_2d(CUtensorMap* out, const void* base, int dtype, int elem_bytes, uint64_t inner,
                 uint64_t rows, uint64_t ld, uint32_t box_inner, uint32_t box_rows,
                 bool swizzle128) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(RF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0)
    return fail(RF_ERR_BAD_ARG, "TMA base %p is not 16-byte aligned", base);
  if ((ld * elem_bytes) % 16 != 0)
    return fail(RF_ERR_BAD_ARG, "TMA row pitch %llu B is not a multiple of 16",
                (unsigned long long)(ld * elem_bytes));
  if (box_rows == 0 || box_rows > 256 || box_inner * elem_bytes > 128 * (swizzle128 ? 1 : 16))
    return fail(RF_ERR_BAD_ARG, "TMA box [%u, %u] out of range", box_rows, box_inner);
  CUtensorMapDataType dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  if (elem_bytes == 1)
    dt = CU_TENSOR_MAP_DATA_TYPE_UINT8;
  else if (dtype == 1)
    dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  cuuint64_t gdim[2] = {inner, rows};
  cuuint64_t gstride[1] = {ld * elem_bytes};
  cuuint32_t box[2] = {box_inner, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return fail(RF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
  return RF_OK;
}

static std::atomic<uint64_t> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((uint64_t)n, std::memory_order_relaxed); }

bool pdl_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("RF_PDL");
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

int device_ordinal() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    (void)cudaGetLastError();   // no device: not an error of the caller's
    return -1;
  }
  return dev;
}

int sm_count() {
  constexpr int kMaxDev = 64;
  static std::atomic<int> cache[kMaxDev];   // zero-initialised: 0 = not looked up yet
  const int dev = device_ordinal();
  if (dev < 0) return 148;
  if (dev < kMaxDev) {
    const int c = cache[dev].load(std::memory_order_relaxed);
    if (c > 0) return c;
  }
  int n = 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
  if (dev < kMaxDev) cache[dev].store(n, std::memory_order_relaxed);
  return n;
}

}  // namespace rf

extern "C" const char* rf_last_error(void) { return rf::g_last_error.c_str(); }
extern "C" int rf_version(void) { return 100; }
extern "C" uint64_t rf_launch_count(void) { return rf::g_launches.load(); }
