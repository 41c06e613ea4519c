// Mixture-of-experts routing for TP-sharded expert MLPs.
//
// rf_moe_select: per token, scores = sigmoid(logits) (or softmax), selection by
// (score + correction bias) with ties going to the lower expert index, weights taken
// from the UNBIASED scores, optionally normalised over the selected experts and scaled
// (semantics of src/ops/rpu_moe_select.cpp:1-238 and the router of
// src/fused/rpu_lingbot_v2_moe_model.cpp:1029-1213).
//
// The expert MLPs themselves run as the "dense-einsum" form (the reference's
// rpu_lingbot_v2_moe_model.cpp:1215-1312 mode): all experts' gate/up projections are one
// GEMM [T, E*I], rf_moe_scale_blocks multiplies expert block e of token t by its routing
// weight (zero when not selected), and the down projections are one GEMM over K = E*I, which
// sums the weighted expert outputs.  For the token counts of an action expert (<= 256 rows)
// the GEMMs are bound by reading the expert weights once, which both forms must do.
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kMoeMaxPerLane = 8;   // up to 256 experts

template <typename T>
__global__ void moe_select_kernel(const T* __restrict__ logits, int64_t ld, const float* __restrict__ bias, int rows,
                                  int E, int k, int score_fn, int norm_topk, float scale, int32_t* __restrict__ out_ids,
                                  float* __restrict__ out_w, T* __restrict__ dense_w, int64_t ldd) {
  pdl_prologue();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  float sc[kMoeMaxPerLane], key[kMoeMaxPerLane];
  // expert e lives in lane e % 32, slot e / 32
  float mx = -INFINITY;
#pragma unroll
  for (int s = 0; s < kMoeMaxPerLane; ++s) {
    const int e = s * 32 + lane;
    sc[s] = e < E ? Num<T>::to_f(logits[(size_t)r * ld + e]) : -INFINITY;
    mx = fmaxf(mx, sc[s]);
  }
  if (score_fn == 1) {   // softmax over all experts
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int s = 0; s < kMoeMaxPerLane; ++s) {
      const int e = s * 32 + lane;
      sc[s] = e < E ? __expf(sc[s] - mx) : 0.f;
      sum += sc[s];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int s = 0; s < kMoeMaxPerLane; ++s) sc[s] /= sum;
  } else {
#pragma unroll
    for (int s = 0; s < kMoeMaxPerLane; ++s) {
      const int e = s * 32 + lane;
      sc[s] = e < E ? 1.f / (1.f + __expf(-sc[s])) : 0.f;
    }
  }
#pragma unroll
  for (int s = 0; s < kMoeMaxPerLane; ++s) {
    const int e = s * 32 + lane;
    key[s] = e < E ? sc[s] + (bias ? bias[e] : 0.f) : -INFINITY;
  }
  float wsel[kMoeMaxPerLane];
#pragma unroll
  for (int s = 0; s < kMoeMaxPerLane; ++s) wsel[s] = 0.f;
  float wsum = 0.f;
  int my_pick_id = -1;      // lane j < k remembers the j-th pick
  float my_pick_w = 0.f;
  for (int j = 0; j < k; ++j) {
    // arg-max of key with ties to the lower index
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int s = 0; s < kMoeMaxPerLane; ++s) {
      const int e = s * 32 + lane;
      if (key[s] > best || (key[s] == best && e < bi)) {
        best = key[s];
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    // the owner lane retires the expert and publishes its unbiased score
    float w = 0.f;
    if ((bi & 31) == lane) {
#pragma unroll
      for (int s = 0; s < kMoeMaxPerLane; ++s)
        if (s == (bi >> 5)) {
          w = sc[s];
          key[s] = -INFINITY;
          wsel[s] = sc[s];
        }
    }
    w = __shfl_sync(0xffffffffu, w, bi & 31);
    wsum += w;
    if (lane == j) {
      my_pick_id = bi;
      my_pick_w = w;
    }
  }
  const float mul = (norm_topk ? 1.f / (wsum + 1e-20f) : 1.f) * scale;
  if (lane < k) {
    if (out_ids) out_ids[(size_t)r * k + lane] = my_pick_id;
    if (out_w) out_w[(size_t)r * k + lane] = my_pick_w * mul;
  }
  if (dense_w) {
#pragma unroll
    for (int s = 0; s < kMoeMaxPerLane; ++s) {
      const int e = s * 32 + lane;
      if (e < E) dense_w[(size_t)r * ldd + e] = Num<T>::from_f(wsel[s] * mul);
    }
  }
}

// h[t, e*I + c] *= dense_w[t, e] for e < E; columns beyond E*I (shared expert) are left alone
template <typename T>
__global__ void moe_scale_blocks_kernel(T* __restrict__ h, int64_t ldh, const T* __restrict__ dense_w, int64_t ldd,
                                        int rows, int E, int I) {
  pdl_prologue();
  const int per_row = E * I / 8;
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (int64_t)rows * per_row) return;
  const int t = (int)(idx / per_row), c = (int)(idx % per_row) * 8;
  const float w = Num<T>::to_f(dense_w[(size_t)t * ldd + c / I]);
  T* p = h + (size_t)t * ldh + c;
  if (w == 0.f) {
    *reinterpret_cast<uint4*>(p) = make_uint4(0u, 0u, 0u, 0u);
    return;
  }
  float f[8];
  load8(p, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] *= w;
  store8(p, f);
}

// Counting sort of the (token, pick) pairs by expert, one CTA.  The order of an expert's rows among themselves
// is whatever the atomics give; every row is computed independently of its neighbours and the combine step adds
// a token's picks in pick order, so results do not depend on it.
__global__ void moe_group_kernel(const int32_t* __restrict__ ids, const float* __restrict__ w, int pairs, int E,
                                 int32_t* __restrict__ slot_of, int32_t* __restrict__ token_of_slot,
                                 float* __restrict__ slot_w, int32_t* __restrict__ tiles, int k) {
  pdl_prologue();
  __shared__ int32_t count[256], start[257], cursor[256];
  const int tid = threadIdx.x;
  for (int e = tid; e < 256; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int acc = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = acc;
      cursor[e] = acc;
      for (int r0 = 0; r0 < count[e]; r0 += 128) {     // one tile entry per 128-row block of this expert
        tiles[1 + 4 * nt + 0] = e;
        tiles[1 + 4 * nt + 1] = acc + r0;
        tiles[1 + 4 * nt + 2] = acc + count[e];
        tiles[1 + 4 * nt + 3] = 0;
        ++nt;
      }
      acc += count[e];
    }
    start[E] = acc;
    tiles[0] = nt;
  }
  __syncthreads();
  for (int i = tid; i < pairs; i += blockDim.x) {
    const int e = ids[i];
    if (e < 0 || e >= E) { slot_of[i] = -1; continue; }
    const int s = atomicAdd(&cursor[e], 1);
    slot_of[i] = s;
    token_of_slot[s] = i / k;
    slot_w[s] = w[i];
  }
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, int64_t ldo, const T* __restrict__ y, int64_t ldy,
                                   const int32_t* __restrict__ slot_of, int k, int H) {
  pdl_prologue();
  const int t = blockIdx.x;
  for (int c = threadIdx.x * 8; c < H; c += blockDim.x * 8) {
    float acc[8];
    load8(out + (size_t)t * ldo + c, acc);
    for (int j = 0; j < k; ++j) {
      const int s = slot_of[(size_t)t * k + j];
      if (s < 0) continue;
      float f[8];
      load8(y + (size_t)s * ldy + c, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    store8(out + (size_t)t * ldo + c, acc);
  }
}

}  // namespace rf

using namespace rf;

#define RF_DISPATCH_T(dtype, ...)                      \
  if ((dtype) == 0) { using T = __half; __VA_ARGS__; } \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

extern "C" int rf_moe_select(const void* logits, int64_t ld, const float* bias, int rows, int E, int k, int score_fn,
                             int norm_topk, float scale, int32_t* out_ids, float* out_w, void* dense_w, int64_t ldd,
                             int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(logits && E > 0 && E <= 32 * kMoeMaxPerLane && k > 0 && k <= 32 && k <= E, "moe_select: E=%d k=%d", E, k);
  RF_REQUIRE(out_ids || out_w || dense_w, "moe_select: no output requested");
  if (rows == 0) return RF_OK;
  const int wpb = 4;
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(moe_select_kernel<T>, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0,
                                                    static_cast<cudaStream_t>(stream), 1, (const T*)logits, ld, bias, rows, E,
                                                    k, score_fn, norm_topk, scale, out_ids, out_w, (T*)dense_w, ldd)));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_moe_scale_blocks(void* h, int64_t ldh, const void* dense_w, int64_t ldd, int rows, int E, int I,
                                   int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(h && dense_w && I % 8 == 0 && ldh % 8 == 0, "moe_scale_blocks: expert width %d / pitch must be multiples of 8", I);
  if (rows == 0) return RF_OK;
  const int64_t n = (int64_t)rows * (E * I / 8);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(moe_scale_blocks_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0,
                                                    static_cast<cudaStream_t>(stream), 1, (T*)h, ldh, (const T*)dense_w, ldd,
                                                    rows, E, I)));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_moe_group(const int32_t* ids, const float* w, int rows, int k, int E, int32_t* slot_of,
                            int32_t* token_of_slot, float* slot_w, int32_t* tiles, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(ids && w && slot_of && token_of_slot && slot_w && tiles, "moe_group arguments");
  RF_REQUIRE(rows > 0 && k > 0 && E > 0 && E <= 256 && (int64_t)rows * k <= (1 << 20), "moe_group: rows=%d k=%d E=%d", rows, k, E);
  RF_CUDA_CHECK(::rf::launch_k(moe_group_kernel, dim3(1), dim3(1024), 0, static_cast<cudaStream_t>(stream), 1, ids, w,
                               rows * k, E, slot_of, token_of_slot, slot_w, tiles, k));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_moe_combine(void* out, int64_t ldo, const void* y, int64_t ldy, const int32_t* slot_of, int rows, int k,
                              int H, int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(out && y && slot_of && H % 8 == 0 && ldo % 8 == 0 && ldy % 8 == 0, "moe_combine: widths and pitches must be multiples of 8");
  if (rows == 0) return RF_OK;
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(moe_combine_kernel<T>, dim3(rows), dim3(128), 0,
                                                    static_cast<cudaStream_t>(stream), 1, (T*)out, ldo, (const T*)y, ldy,
                                                    slot_of, k, H)));
  ::rf::count_launch();
  return RF_OK;
}
