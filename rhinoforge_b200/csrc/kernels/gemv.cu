// CUDA-core skinny GEMM for M <= 8 tokens: every warp streams two weight rows
// with 16-byte loads and keeps the tokens' activations in registers/L1.  Works
// on 16-bit weights and on int8 weights with a per-output-channel scale
// (dequantised in the loop: acc += x * float(q), scale applied once at the end,
// the same "(X . Q^T) * s" order as the tensor-core W8A16 kernel).
// Replaces llama_gemv / llama_gemv_wint8 (src/ops/rpu_linear_gemv.cpp:1-275).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

struct GemvParams {
  const void* x; int64_t ldx;
  const void* w; int64_t ldw;
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias; const void* scale; const float* row_scale;
  int M, N, K, act, dual_offset;
};

template <typename T, int MT, bool I8>
__device__ __forceinline__ void gemv_rows(const GemvParams& p, int n0, int n1, bool two,
                                          float (&acc0)[MT], float (&acc1)[MT]) {
  constexpr int VEC = I8 ? 16 : 8;
  const int lane = threadIdx.x & 31;
  const T* x = reinterpret_cast<const T*>(p.x);
#pragma unroll
  for (int m = 0; m < MT; ++m) { acc0[m] = 0.f; acc1[m] = 0.f; }
  for (int k = lane * VEC; k < p.K; k += 32 * VEC) {
    float w0[VEC], w1[VEC];
    if (I8) {
      const int8_t* wp = reinterpret_cast<const int8_t*>(p.w);
      const int4 q0 = *reinterpret_cast<const int4*>(wp + (size_t)n0 * p.ldw + k);
      const int8_t* b0 = reinterpret_cast<const int8_t*>(&q0);
#pragma unroll
      for (int j = 0; j < VEC; ++j) w0[j] = (float)b0[j];
      if (two) {
        const int4 q1 = *reinterpret_cast<const int4*>(wp + (size_t)n1 * p.ldw + k);
        const int8_t* b1 = reinterpret_cast<const int8_t*>(&q1);
#pragma unroll
        for (int j = 0; j < VEC; ++j) w1[j] = (float)b1[j];
      }
    } else {
      const T* wp = reinterpret_cast<const T*>(p.w);
      float t[8];
      load8(wp + (size_t)n0 * p.ldw + k, t);
#pragma unroll
      for (int j = 0; j < 8; ++j) w0[j] = t[j];
      if (two) {
        load8(wp + (size_t)n1 * p.ldw + k, t);
#pragma unroll
        for (int j = 0; j < 8; ++j) w1[j] = t[j];
      }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m) {
      if (m < p.M) {
#pragma unroll
        for (int v = 0; v < VEC; v += 8) {
          float xf[8];
          load8(x + (size_t)m * p.ldx + k + v, xf);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            acc0[m] = fmaf(xf[j], w0[v + j], acc0[m]);
            if (two) acc1[m] = fmaf(xf[j], w1[v + j], acc1[m]);
          }
        }
      }
    }
  }
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    acc0[m] = warp_sum(acc0[m]);
    acc1[m] = warp_sum(acc1[m]);
  }
}

template <typename T, int MT, bool I8>
__global__ void __launch_bounds__(256) gemv_kernel(const GemvParams p) {
  pdl_prologue();
  const int warp_global = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const bool dual = p.dual_offset > 0;
  int n0, n1;
  bool two;
  if (dual) {
    n0 = warp_global;
    n1 = p.dual_offset + warp_global;
    two = true;
    if (n0 >= p.N) return;
  } else {
    n0 = warp_global * 2;
    n1 = n0 + 1;
    if (n0 >= p.N) return;
    two = n1 < p.N;
  }
  float a0[MT], a1[MT];
  gemv_rows<T, MT, I8>(p, n0, n1, two, a0, a1);
  if (lane != 0) return;
  const T* bias = reinterpret_cast<const T*>(p.bias);
  const T* scale = reinterpret_cast<const T*>(p.scale);
  const T* resid = reinterpret_cast<const T*>(p.residual);
  T* out = reinterpret_cast<T*>(p.out);
#pragma unroll
  for (int m = 0; m < MT; ++m) {
    if (m >= p.M) break;
    float v0 = a0[m], v1 = a1[m];
    if (p.row_scale) { v0 *= p.row_scale[m]; v1 *= p.row_scale[m]; }
    if (scale) { v0 *= Num<T>::to_f(scale[n0]); if (two) v1 *= Num<T>::to_f(scale[n1]); }
    if (bias) { v0 += Num<T>::to_f(bias[n0]); if (two) v1 += Num<T>::to_f(bias[n1]); }
    if (dual) {
      float r = apply_act(p.act, v0, v1);
      if (resid) r += Num<T>::to_f(resid[(size_t)m * p.ldr + n0]);
      out[(size_t)m * p.ldo + n0] = Num<T>::from_f(r);
    } else {
      float r0 = apply_act(p.act, v0, 0.f);
      if (resid) r0 += Num<T>::to_f(resid[(size_t)m * p.ldr + n0]);
      out[(size_t)m * p.ldo + n0] = Num<T>::from_f(r0);
      if (two) {
        float r1 = apply_act(p.act, v1, 0.f);
        if (resid) r1 += Num<T>::to_f(resid[(size_t)m * p.ldr + n1]);
        out[(size_t)m * p.ldo + n1] = Num<T>::from_f(r1);
      }
    }
  }
}

template <typename T, bool I8>
static int launch_gemv(const GemvParams& p, cudaStream_t s) {
  const bool dual = p.dual_offset > 0;
  const int warps = dual ? p.N : (p.N + 1) / 2;
  const int wpb = 8;
  const int blocks = (warps + wpb - 1) / wpb;
  if (p.M <= 1) RF_CUDA_CHECK(::rf::launch_k(gemv_kernel<T, 1, I8>, dim3(blocks), dim3(wpb * 32), 0, s, 1, p));
  else if (p.M <= 2) RF_CUDA_CHECK(::rf::launch_k(gemv_kernel<T, 2, I8>, dim3(blocks), dim3(wpb * 32), 0, s, 1, p));
  else if (p.M <= 4) RF_CUDA_CHECK(::rf::launch_k(gemv_kernel<T, 4, I8>, dim3(blocks), dim3(wpb * 32), 0, s, 1, p));
  else RF_CUDA_CHECK(::rf::launch_k(gemv_kernel<T, 8, I8>, dim3(blocks), dim3(wpb * 32), 0, s, 1, p));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

}  // namespace rf

using namespace rf;

extern "C" int rf_gemv(const RfGemm* g, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(g && g->x && g->w && g->out, "gemv needs x, w and out");
  RF_REQUIRE(g->M >= 1 && g->M <= 8, "gemv handles 1..8 tokens, got %d", g->M);
  const int vec = g->w_int8 ? 16 : 8;
  RF_REQUIRE(g->K % vec == 0 && g->ldw % vec == 0 && g->ldx % 8 == 0,
             "gemv K=%d / pitches must be multiples of %d", g->K, vec);
  RF_REQUIRE(!g->w_int8 || g->scale, "int8 weights need a scale vector");
  RF_REQUIRE(g->ar_world <= 1, "gemv has no fused all-reduce");
  const bool dual_act = g->act == kActSiluMul || g->act == kActGeluTanhMul;
  RF_REQUIRE(dual_act == (g->dual_offset > 0), "dual_offset and a *_mul activation go together");
  GemvParams p;
  p.x = g->x; p.ldx = g->ldx; p.w = g->w; p.ldw = g->ldw; p.out = g->out; p.ldo = g->ldo;
  p.residual = g->residual; p.ldr = g->ldr; p.bias = g->bias; p.scale = g->scale;
  p.row_scale = g->row_scale; p.M = g->M; p.N = g->N; p.K = g->K; p.act = g->act;
  p.dual_offset = g->dual_offset;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (g->dtype == 0)
    return g->w_int8 ? launch_gemv<__half, true>(p, s) : launch_gemv<__half, false>(p, s);
  return g->w_int8 ? launch_gemv<__nv_bfloat16, true>(p, s) : launch_gemv<__nv_bfloat16, false>(p, s);
}
