// Host-side helpers: last-error string, CUDA error checks, TMA tensor-map
// encoding through the driver entry point (no link-time libcuda dependency, so
// the library also loads on a machine without a driver).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <atomic>
#include <string>

#include "../rf_api.h"

namespace rf {

void set_error(const std::string& msg);
int fail(int code, const char* fmt, ...);

#define RF_CUDA_CHECK(expr)                                                                  \
  do {                                                                                       \
    cudaError_t _e = (expr);                                                                 \
    if (_e != cudaSuccess)                                                                   \
      return ::rf::fail(RF_ERR_CUDA, "%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e), \
                        __FILE__, __LINE__);                                                 \
  } while (0)

#define RF_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return ::rf::fail(RF_ERR_BAD_ARG, __VA_ARGS__); \
  } while (0)

// 2-D K-major tensor map over a row-major [rows, inner] matrix of 16-bit (or
// 8-bit when elem_bytes == 1) elements with row pitch ld (elements).  The box is
// [box_rows, box_inner]; swizzle 128 B requires box_inner * elem_bytes == 128.
// Returns 0 or a negative RfError.
int make_tmap_2d(CUtensorMap* out, const void* base, int dtype, int elem_bytes, uint64_t inner,
                 uint64_t rows, uint64_t ld, uint32_t box_inner, uint32_t box_rows,
                 bool swizzle128);

inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline int round_up(int a, int b) { return ceil_div(a, b) * b; }
inline uint32_t next_pow2(uint32_t v) {
  uint32_t p = 1;
  while (p < v) p <<= 1;
  return p;
}

// SM count of the CURRENT device (cached per device ordinal; 148 when no device answers).
int sm_count();

// Ordinal of the current device, or -1 when there is none.
int device_ordinal();

// cudaFuncAttributeMaxDynamicSharedMemorySize is a per-device property of a kernel: a process that uses several
// GPUs must set it on each of them.  This sets it the first time the call site runs on each device (one bit per
// ordinal; ordinals >= 64 set it on every call).
#define RF_ALLOW_SMEM_PER_DEVICE(kfn, bytes)                                                               \
  do {                                                                                                     \
    static std::atomic<uint64_t> _rf_done{0};                                                              \
    const int _rf_dev = ::rf::device_ordinal();                                                            \
    const bool _rf_track = _rf_dev >= 0 && _rf_dev < 64;                                                   \
    if (!_rf_track || !((_rf_done.load(std::memory_order_acquire) >> _rf_dev) & 1ull)) {                   \
      RF_CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(bytes))); \
      if (_rf_track) _rf_done.fetch_or(1ull << _rf_dev, std::memory_order_release);                        \
    }                                                                                                      \
  } while (0)

// Whether kernels are launched with programmatic stream serialization (RF_PDL=0 turns it off).
bool pdl_enabled();

// Launch with the library's standard attributes: programmatic dependent launch and,
// when cluster_z > 1, a (1,1,cluster_z) thread-block cluster.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_k(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                            int cluster_z, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  int n = 0;
  if (pdl_enabled()) {
    attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[n].val.programmaticStreamSerializationAllowed = 1;
    ++n;
  }
  if (cluster_z > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = 1;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = (unsigned)cluster_z;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Launch WITHOUT programmatic dependent launch: the kernel starts after everything before it in the stream has
// completed, and a later kernel (even one launched with launch_k, whose prologue runs before its dependency wait)
// cannot start before this one has completed.  For kernels that write data which the next kernel reads in its
// prologue (a widened weight image that the GEMM prefetches before its dependency wait).
template <typename... KArgs, typename... Args>
inline cudaError_t launch_serial(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                 Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cfg.attrs = nullptr;
  cfg.numAttrs = 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// True while this thread is inside a graph scope in REPLAY mode: launchers return at once.
bool replay_mode();
#define RF_SKIP_IF_REPLAYING()             \
  do {                                     \
    if (::rf::replay_mode()) return RF_OK; \
  } while (0)

// Number of kernel launches this library has enqueued (captured launches count once).
void count_launch(int n = 1);

}  // namespace rf
