// Small memory-bound kernels: embedding gather, row scatter (vision rows into
// text rows), elementwise algebra, uint8 -> 16-bit cast, two-stage arg-max.
// Replaces gather_embedding / assemble_inputs_embeds (src/ops/rpu_embedding.cpp),
// binary_* / unary_* / llama_silu_mul (src/ops/rpu_eltwise_binary.cpp,
// src/ops/rpu_eltwise_unary.cpp), cast_uint8_fp16 (src/ops/rpu_cast.cpp) and the
// host NEON lm_head_logits_top1 scan (src/core/rpu_backend.cpp:200-316).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

template <typename T>
__global__ void embedding_kernel(const T* __restrict__ table, const int32_t* __restrict__ ids,
                                 T* __restrict__ out, int H, int64_t ldo, float scale) {
  pdl_prologue();
  const int i = blockIdx.x;
  const int id = ids[i];
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float f[8];
    if (id >= 0) {
      load8(table + (size_t)id * H + c, f);
      if (scale != 1.f) {
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] *= scale;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = 0.f;
    }
    store8(out + (size_t)i * ldo + c, f);
  }
}

// int8 table with one 16-bit scale per row (W8A16 "quantized_embed_tokens")
template <typename T>
__global__ void embedding_i8_kernel(const int8_t* __restrict__ table, const T* __restrict__ rscale,
                                    const int32_t* __restrict__ ids, T* __restrict__ out, int H,
                                    int64_t ldo, float scale) {
  pdl_prologue();
  const int i = blockIdx.x;
  const int id = ids[i];
  const float s = id >= 0 ? Num<T>::to_f(rscale[id]) * scale : 0.f;
  for (int c = threadIdx.x; c < H; c += blockDim.x)
    out[(size_t)i * ldo + c] = Num<T>::from_f(id >= 0 ? (float)table[(size_t)id * H + c] * s : 0.f);
}

template <typename T>
__global__ void scatter_rows_kernel(T* __restrict__ dst, const T* __restrict__ src,
                                    const int32_t* __restrict__ rows, int H, int64_t ldd,
                                    int64_t lds, int accumulate) {
  pdl_prologue();
  const int i = blockIdx.x;
  const int r = rows[i];
  if (r < 0) return;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float f[8];
    load8(src + (size_t)i * lds + c, f);
    if (accumulate) {
      float d[8];
      load8(dst + (size_t)r * ldd + c, d);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += d[j];
    }
    store8(dst + (size_t)r * ldd + c, f);
  }
}

__device__ __forceinline__ float elt_op(int op, float a, float b, float alpha) {
  switch (op) {
    case 0: return a + b;
    case 1: return a * b;
    case 2: return silu_f(a) * b;
    case 3: return gelu_tanh_f(a) * b;
    case 4: return a + alpha * b;
    case 5: return gelu_tanh_f(a);
    case 6: return gelu_erf_f(a);
    case 7: return silu_f(a);
    case 8: return a * alpha;
    case 9: return b / (1.f + __expf(-a));
    case 10: return a * b;
    case 11: return tanhf(a);
    default: return a;
  }
}

template <typename T>
__global__ void eltwise_kernel(int op, const T* __restrict__ a, const T* __restrict__ b,
                               T* __restrict__ out, int64_t n, int64_t b_period, float alpha) {
  pdl_prologue();
  const int64_t i = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (i >= n) return;
  if (i + 8 <= n && (b_period == 0 || b_period % 8 == 0)) {
    float fa[8], fb[8] = {0, 0, 0, 0, 0, 0, 0, 0}, o[8];
    load8(a + i, fa);
    if (b) load8(b + (b_period ? i % b_period : i), fb);
#pragma unroll
    for (int j = 0; j < 8; ++j) o[j] = elt_op(op, fa[j], fb[j], alpha);
    store8(out + i, o);
  } else {
    for (int64_t k = i; k < n && k < i + 8; ++k) {
      const float fb = b ? Num<T>::to_f(b[b_period ? k % b_period : k]) : 0.f;
      out[k] = Num<T>::from_f(elt_op(op, Num<T>::to_f(a[k]), fb, alpha));
    }
  }
}

template <typename T>
__global__ void cast_u8_kernel(const uint8_t* __restrict__ src, T* __restrict__ dst, int64_t n,
                               float scale, float shift) {
  pdl_prologue();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = Num<T>::from_f((float)src[i] * scale + shift);
}

// ------------------------------------------------------------- argmax ----
constexpr int kArgmaxChunk = 4096;

struct ArgPair { float v; int32_t i; };

__device__ __forceinline__ ArgPair arg_better(ArgPair a, ArgPair b) {
  // larger value wins; ties go to the lower index (torch.argmax on CPU picks the first)
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgPair warp_argmax(ArgPair p) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgPair q;
    q.v = __shfl_xor_sync(0xffffffffu, p.v, o);
    q.i = __shfl_xor_sync(0xffffffffu, p.i, o);
    p = arg_better(p, q);
  }
  return p;
}
__device__ __forceinline__ ArgPair block_argmax(ArgPair p, ArgPair* red) {
  p = warp_argmax(p);
  const int w = threadIdx.x >> 5, l = threadIdx.x & 31;
  if (l == 0) red[w] = p;
  __syncthreads();
  const int nw = blockDim.x >> 5;
  if (w == 0) {
    ArgPair q = l < nw ? red[l] : ArgPair{-INFINITY, 0x7fffffff};
    q = warp_argmax(q);
    if (l == 0) red[0] = q;
  }
  __syncthreads();
  return red[0];
}

template <typename T>
__global__ void argmax_stage1(const T* __restrict__ x, int V, int64_t ld, ArgPair* __restrict__ part,
                              int chunks) {
  pdl_prologue();
  __shared__ ArgPair red[32];
  const int row = blockIdx.y, ch = blockIdx.x;
  const int beg = ch * kArgmaxChunk, end = min(V, beg + kArgmaxChunk);
  ArgPair best{-INFINITY, 0x7fffffff};
  const T* xr = x + (size_t)row * ld;
  for (int i = beg + threadIdx.x; i < end; i += blockDim.x) {
    const float v = Num<T>::to_f(xr[i]);
    if (v > best.v || (v == best.v && i < best.i)) { best.v = v; best.i = i; }
  }
  best = block_argmax(best, red);
  if (threadIdx.x == 0) part[(size_t)row * chunks + ch] = best;
}

__global__ void argmax_stage2(const ArgPair* __restrict__ part, int chunks, int32_t* out_ids,
                              float* out_vals, int32_t offset) {
  pdl_prologue();
  __shared__ ArgPair red[32];
  const int row = blockIdx.x;
  ArgPair best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < chunks; i += blockDim.x) best = arg_better(best, part[(size_t)row * chunks + i]);
  best = block_argmax(best, red);
  if (threadIdx.x == 0) {
    out_ids[row] = best.i + offset;
    if (out_vals) out_vals[row] = best.v;
  }
}

}  // namespace rf

using namespace rf;

#define RF_DISPATCH_T(dtype, ...)                      \
  if ((dtype) == 0) { using T = __half; __VA_ARGS__; } \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

extern "C" int rf_embedding(const void* table, const int32_t* ids, void* out, int n_ids, int H,
                            int64_t ldo, float scale, int dtype, const void* row_scale_i8,
                            rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(table && ids && out && H % 8 == 0 && ldo % 8 == 0, "embedding arguments");
  if (n_ids == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (row_scale_i8) {
    RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(embedding_i8_kernel<T>, dim3(n_ids), dim3(128), 0, s, 1, 
                             (const int8_t*)table, (const T*)row_scale_i8, ids, (T*)out, H, ldo, scale)));
  } else {
    RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(embedding_kernel<T>, dim3(n_ids), dim3(128), 0, s, 1, (const T*)table, ids, (T*)out, H, ldo, scale)));
  }
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_scatter_rows(void* dst, const void* src, const int32_t* rows, int n, int H,
                               int64_t ldd, int64_t lds, int accumulate, int dtype,
                               rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(dst && src && rows && H % 8 == 0 && ldd % 8 == 0 && lds % 8 == 0, "scatter_rows arguments");
  if (n == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(scatter_rows_kernel<T>, dim3(n), dim3(128), 0, s, 1, (T*)dst, (const T*)src, rows, H, ldd, lds, accumulate)));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_eltwise(int op, const void* a, const void* b, void* out, int64_t n,
                          int64_t b_period, float alpha, int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && out && n >= 0, "eltwise arguments");
  if (n == 0) return RF_OK;
  RF_REQUIRE((reinterpret_cast<uintptr_t>(a) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(b) & 15) == 0,
             "eltwise operands must be 16-byte aligned");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const int blocks = (int)(((n + 7) / 8 + threads - 1) / threads);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(eltwise_kernel<T>, dim3(blocks), dim3(threads), 0, s, 1, op, (const T*)a, (const T*)b, (T*)out, n, b_period, alpha)));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_cast_u8_f16(const uint8_t* src, void* dst, int64_t n, float scale, float shift,
                              int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(src && dst && n >= 0, "cast arguments");
  if (n == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 256;
  const int blocks = (int)((n + threads - 1) / threads);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(cast_u8_kernel<T>, dim3(blocks), dim3(threads), 0, s, 1, src, (T*)dst, n, scale, shift)));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

extern "C" uint64_t rf_argmax_scratch_bytes(int rows, int V) {
  const int chunks = (V + kArgmaxChunk - 1) / kArgmaxChunk;
  return (uint64_t)rows * chunks * sizeof(ArgPair);
}

extern "C" int rf_argmax(const void* logits, int rows, int V, int64_t ld, int32_t* out_ids,
                         float* out_vals, int32_t offset, void* scratch, uint64_t scratch_bytes,
                         int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(logits && out_ids && scratch && rows >= 0 && V > 0, "argmax arguments");
  if (rows == 0) return RF_OK;
  RF_REQUIRE(scratch_bytes >= rf_argmax_scratch_bytes(rows, V), "argmax scratch too small");
  const int chunks = (V + kArgmaxChunk - 1) / kArgmaxChunk;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 g1(chunks, rows);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(argmax_stage1<T>, dim3(g1), dim3(256), 0, s, 1, (const T*)logits, V, ld, (ArgPair*)scratch, chunks)));
  RF_CUDA_CHECK(::rf::launch_k(argmax_stage2, dim3(rows), dim3(128), 0, s, 1, (const ArgPair*)scratch, chunks, out_ids, out_vals, offset));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}
