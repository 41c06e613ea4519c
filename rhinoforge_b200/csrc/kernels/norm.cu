// Row normalisation kernels: RMSNorm (Qwen/Llama and Gemma "(1+w)" flavours,
// optional fused residual add, optional adaRMS scale/shift), LayerNorm, L2 norm.
// Replaces the reference's llama_rms_norm*, layer_norm* and l2norm operators
// (src/ops/rpu_rmsnorm.cpp, src/ops/rpu_layernorm.cpp, src/ops/rpu_l2norm.cpp)
// and the adaRMS SUB/MUL/ADD chain (src/fused/rpu_pi05_denoise_step_model.cpp:848-857).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  __syncthreads();
  if (l == 0) red[w] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.f;
  if (w == 0) {
    t = warp_sum(t);
    if (l == 0) red[0] = t;
  }
  __syncthreads();
  return red[0];
}

// y = norm(x [+ residual]) ; if residual_out: residual_out = x + residual.
// mode bit0: gemma style weight (1 + w), product rounded once
// mod (optional, adaRMS): per-token [rows / rows_per_mod, 3H] = [scale | shift | gate];
//   y = norm(x) * (1 + scale) + shift   (weight is ignored when mod != null)
template <typename T>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ residual,
                               const T* __restrict__ w, T* __restrict__ y,
                               T* __restrict__ residual_out, const T* __restrict__ mod,
                               int rows_per_mod, int H, int64_t ldx, int64_t ldy, float eps,
                               int mode) {
  pdl_prologue();
  extern __shared__ float srow[];  // H floats + 32
  float* red = srow + H;
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * ldx;
  const T* rr = residual ? residual + (size_t)row * ldx : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8];
    load8(xr + i, f);
    if (rr) {
      float r[8];
      load8(rr + i, r);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = Num<T>::to_f(Num<T>::from_f(f[j] + r[j]));
      if (residual_out) store8(residual_out + (size_t)row * ldx + i, f);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      srow[i + j] = f[j];
      ss += f[j] * f[j];
    }
  }
  const float tot = block_sum(ss, red);
  const float rstd = rsqrtf(tot / (float)H + eps);
  const T* mrow = mod ? mod + (size_t)(row / rows_per_mod) * 3 * H : nullptr;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float o[8];
    if (mrow) {
      float sc[8], sh[8];
      load8(mrow + i, sc);
      load8(mrow + H + i, sh);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = srow[i + j] * rstd * (1.f + sc[j]) + sh[j];
    } else {
      float wf[8];
      if (w) {
        load8(w + i, wf);
      } else {   // no weight: plain x * rstd in either form
#pragma unroll
        for (int j = 0; j < 8; ++j) wf[j] = (mode & 1) ? 0.f : 1.f;
      }
      if (mode & 1) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = srow[i + j] * rstd * (1.f + wf[j]);
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j)
          o[j] = wf[j] * Num<T>::to_f(Num<T>::from_f(srow[i + j] * rstd));
      }
    }
    store8(y + (size_t)row * ldy + i, o);
  }
}

template <typename T>
__global__ void layernorm_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                 const T* __restrict__ b, T* __restrict__ y, int H, int64_t ldx,
                                 int64_t ldy, float eps) {
  pdl_prologue();
  extern __shared__ float srow[];
  float* red = srow + H;
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * ldx;
  float s = 0.f;
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float f[8];
    load8(xr + i, f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      srow[i + j] = f[j];
      s += f[j];
    }
  }
  const float mean = block_sum(s, red) / (float)H;
  float v = 0.f;
  for (int i = threadIdx.x; i < H; i += blockDim.x) {
    const float d = srow[i] - mean;
    v += d * d;
  }
  const float var = block_sum(v, red) / (float)H;
  const float rstd = rsqrtf(var + eps);
  for (int i = threadIdx.x * 8; i < H; i += blockDim.x * 8) {
    float wf[8], bf[8], o[8];
    load8(w + i, wf);
    if (b) load8(b + i, bf);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = (srow[i + j] - mean) * rstd * wf[j] + (b ? bf[j] : 0.f);
    store8(y + (size_t)row * ldy + i, o);
  }
}

template <typename T>
__global__ void l2norm_kernel(const T* __restrict__ x, T* __restrict__ y, int rows, int H,
                              float eps, float out_scale) {
  pdl_prologue();
  // one warp per row
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int l = threadIdx.x & 31;
  const T* xr = x + (size_t)row * H;
  float ss = 0.f;
  for (int i = l; i < H; i += 32) {
    const float f = Num<T>::to_f(xr[i]);
    ss += f * f;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss + eps) * out_scale;
  for (int i = l; i < H; i += 32) y[(size_t)row * H + i] = Num<T>::from_f(Num<T>::to_f(xr[i]) * r);
}

// x += gate * y  (adaRMS gated residual; gate per token-group [.., 3H] third block)
template <typename T>
__global__ void gated_residual_kernel(T* __restrict__ x, const T* __restrict__ y,
                                      const T* __restrict__ mod, int rows_per_mod, int H,
                                      int64_t total) {
  pdl_prologue();
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= total) return;
  const int row = (int)(i / H), col = (int)(i % H);
  float a[8], b[8], g[8];
  load8(x + i, a);
  load8(y + i, b);
  load8(mod + (size_t)(row / rows_per_mod) * 3 * H + 2 * H + col, g);
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] += g[j] * b[j];
  store8(x + i, a);
}

}  // namespace rf

using namespace rf;

extern "C" int rf_rmsnorm(const void* x, const void* residual, const void* w, void* y,
                          void* residual_out, const void* mod, int rows_per_mod, int rows, int H,
                          int64_t ldx, int64_t ldy, float eps, int mode, int dtype,
                          rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(rows >= 0 && H > 0 && H % 8 == 0, "rmsnorm H=%d must be a multiple of 8", H);
  RF_REQUIRE(ldx % 8 == 0 && ldy % 8 == 0, "rmsnorm pitches must be multiples of 8");
  if (rows == 0) return RF_OK;
  const int threads = H >= 2048 ? 256 : 128;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows_per_mod <= 0) rows_per_mod = 1;
  if (dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(rmsnorm_kernel<__half>, dim3(rows), dim3(threads), smem, s, 1, 
        (const __half*)x, (const __half*)residual, (const __half*)w, (__half*)y,
        (__half*)residual_out, (const __half*)mod, rows_per_mod, H, ldx, ldy, eps, mode));
  else
    RF_CUDA_CHECK(::rf::launch_k(rmsnorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, s, 1, 
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)residual, (const __nv_bfloat16*)w,
        (__nv_bfloat16*)y, (__nv_bfloat16*)residual_out, (const __nv_bfloat16*)mod, rows_per_mod,
        H, ldx, ldy, eps, mode));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_layernorm(const void* x, const void* w, const void* b, void* y, int rows, int H,
                            int64_t ldx, int64_t ldy, float eps, int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(rows >= 0 && H > 0 && H % 8 == 0, "layernorm H=%d must be a multiple of 8", H);
  if (rows == 0) return RF_OK;
  const int threads = H >= 2048 ? 256 : 128;
  const size_t smem = (size_t)(H + 32) * sizeof(float);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(layernorm_kernel<__half>, dim3(rows), dim3(threads), smem, s, 1, (const __half*)x, (const __half*)w,
                                                        (const __half*)b, (__half*)y, H, ldx, ldy,
                                                        eps));
  else
    RF_CUDA_CHECK(::rf::launch_k(layernorm_kernel<__nv_bfloat16>, dim3(rows), dim3(threads), smem, s, 1, 
        (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)b,
        (__nv_bfloat16*)y, H, ldx, ldy, eps));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_l2norm(const void* x, void* y, int rows, int H, float eps, float out_scale,
                         int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(rows >= 0 && H > 0, "l2norm shape");
  if (rows == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int wpb = 4;
  const int blocks = ceil_div(rows, wpb);
  if (dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(l2norm_kernel<__half>, dim3(blocks), dim3(wpb * 32), 0, s, 1, (const __half*)x, (__half*)y, rows, H, eps, out_scale));
  else
    RF_CUDA_CHECK(::rf::launch_k(l2norm_kernel<__nv_bfloat16>, dim3(blocks), dim3(wpb * 32), 0, s, 1, (const __nv_bfloat16*)x,
                                                             (__nv_bfloat16*)y, rows, H, eps, out_scale));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_gated_residual(void* x, const void* y, const void* mod, int rows_per_mod,
                                 int rows, int H, int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(H % 8 == 0 && rows >= 0, "gated_residual H=%d must be a multiple of 8", H);
  if (rows == 0) return RF_OK;
  const int64_t total = (int64_t)rows * H;
  const int threads = 256;
  const int blocks = (int)((total / 8 + threads - 1) / threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (rows_per_mod <= 0) rows_per_mod = 1;
  if (dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(gated_residual_kernel<__half>, dim3(blocks), dim3(threads), 0, s, 1, (__half*)x, (const __half*)y,
                                                           (const __half*)mod, rows_per_mod, H, total));
  else
    RF_CUDA_CHECK(::rf::launch_k(gated_residual_kernel<__nv_bfloat16>, dim3(blocks), dim3(threads), 0, s, 1, 
        (__nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)mod, rows_per_mod, H, total));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}
