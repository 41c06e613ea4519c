// Fused per-head RMSNorm(q,k) -> RoPE -> KV-page insert, one launch after the
// QKV GEMM.  Covers 1-D rotate-half RoPE, interleaved/sectioned M-RoPE (per
// frequency lane axis select), partial rotary (rot_dim < head_dim) and 2-D
// vision RoPE (two position axes), and writes K/V straight into 16-token pages.
// Replaces five reference launches per layer: llama_rms_norm (per head),
// llama_rope / llama_mrope_interleave / partial_mrope / rope_2d and
// llama_insert_{k,v}cache (src/fused/rpu_qwen3_model.h:3378-3453,
// src/ops/rpu_rope.cpp, src/ops/rpu_mrope.cpp:37-124, src/ops/rpu_llama_kvcache.cpp).
#include <cstdlib>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

template <typename T>
__global__ void qk_norm_rope_kv_kernel(const RfRopeKv a) {
  pdl_prologue();
  extern __shared__ float sh[];  // warps * hd floats
  const int tok = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* buf = sh + warp * a.hd;
  const int hd = a.hd, rot = a.rot_dim, half = rot >> 1;
  const int heads = a.Hq + 2 * a.Hkv;
  T* row = reinterpret_cast<T*>(a.qkv) + (size_t)tok * a.ld;

  int page = -1, slot = 0;
  if (a.k_pool) {
    const int seq = a.seq_of_tok ? a.seq_of_tok[tok] : tok;
    const int cpos = a.cache_pos ? a.cache_pos[tok] : a.pos[(size_t)tok * a.pos_stride];
    if (seq >= 0 && cpos >= 0) {
      page = a.page_table[(size_t)seq * a.pt_stride + (cpos >> 4)];
      slot = cpos & 15;
    }
  }

  // heads are spread over the warps of the block and over blockIdx.y (few tokens: more blocks)
  for (int h = blockIdx.y * nwarps + warp; h < heads; h += nwarps * gridDim.y) {
    const bool is_q = h < a.Hq, is_k = !is_q && h < a.Hq + a.Hkv;
    T* src = row + (size_t)h * hd;
    if (is_q || is_k) {
      const T* nw = reinterpret_cast<const T*>(is_q ? a.q_norm_w : a.k_norm_w);
      float ss = 0.f;
      for (int i = lane; i < hd; i += 32) {
        const float f = Num<T>::to_f(src[i]);
        buf[i] = f;
        ss += f * f;
      }
      __syncwarp();
      auto do_norm = [&]() {
        if (!nw) return;
        float s2 = 0.f;
        for (int i = lane; i < hd; i += 32) s2 += buf[i] * buf[i];
        s2 = warp_sum(s2);
        const float rstd = rsqrtf(s2 / (float)hd + a.eps);
        for (int i = lane; i < hd; i += 32) {
          const float w = Num<T>::to_f(nw[i]);
          buf[i] = (a.norm_mode & 1) ? buf[i] * rstd * (1.f + w)
                                     : w * Num<T>::to_f(Num<T>::from_f(buf[i] * rstd));
        }
        __syncwarp();
      };
      auto do_rope = [&]() {
        if (!a.cos || rot <= 0) return;
        // round to storage precision first: the rotation acts on 16-bit values
        for (int i = lane; i < half; i += 32) {
          int axis = a.axis_of_freq ? a.axis_of_freq[i] : 0;
          const int p = a.pos[(size_t)tok * a.pos_stride + axis];
          const float c = a.cos[(size_t)p * half + i], s = a.sin[(size_t)p * half + i];
          const float x0 = Num<T>::to_f(Num<T>::from_f(buf[i]));
          const float x1 = Num<T>::to_f(Num<T>::from_f(buf[i + half]));
          buf[i] = x0 * c - x1 * s;
          buf[i + half] = x1 * c + x0 * s;
        }
        __syncwarp();
      };
      if (a.rope_before_norm) { do_rope(); do_norm(); } else { do_norm(); do_rope(); }
      (void)ss;
      if (is_q) {
        T* dst = a.q_out ? reinterpret_cast<T*>(a.q_out) + (size_t)tok * a.ldq + (size_t)h * hd : src;
        for (int i = lane; i < hd; i += 32) dst[i] = Num<T>::from_f(buf[i]);
      } else {
        const int kh = h - a.Hq;
        if (page >= 0) {
          T* dst = reinterpret_cast<T*>(a.k_pool) + (((size_t)page * a.Hkv + kh) * 16 + slot) * hd;
          for (int i = lane; i < hd; i += 32) dst[i] = Num<T>::from_f(buf[i]);
        }
        if (!a.k_pool || a.write_k_inplace)
          for (int i = lane; i < hd; i += 32) src[i] = Num<T>::from_f(buf[i]);
      }
      __syncwarp();
    } else {
      if (a.v_norm) {                                      // unweighted RMS over the value head, in place
        float s2 = 0.f;
        for (int i = lane; i < hd; i += 32) {
          const float f = Num<T>::to_f(src[i]);
          buf[i] = f;
          s2 += f * f;
        }
        s2 = warp_sum(s2);
        const float rstd = rsqrtf(s2 / (float)hd + a.eps);
        for (int i = lane; i < hd; i += 32) src[i] = Num<T>::from_f(buf[i] * rstd);
        __syncwarp();
      }
      if (page >= 0) {
        const int vh = h - a.Hq - a.Hkv;
        T* dst = reinterpret_cast<T*>(a.v_pool) + (((size_t)page * a.Hkv + vh) * 16 + slot) * hd;
        for (int i = lane; i < hd; i += 32) dst[i] = src[i];
      }
    }
  }
}

// Prefill-sized launches: the same computation with 16-byte accesses.  A head of 64 / 128 / 256 elements is held by 8 / 16 /
// 32 lanes with eight consecutive elements each, so one warp instruction moves four / two / one head(s); sums of squares
// are reduced inside the lane group and the rotate-half partner comes from the lane rot_dim / 16 away (rot_dim % 16 == 0).
// The scalar kernel above keeps a warp on 64 - 128 bytes per load and runs at a fraction of memory speed on thousands of
// tokens (6 272 vision patches x 48 heads of 64: 53 us); it stays for decode-sized launches and odd geometries.
template <typename T, int HD>
__global__ void __launch_bounds__(256) qk_norm_rope_kv_vec_kernel(const RfRopeKv a) {
  pdl_prologue();
  constexpr int GROUP = HD / 8;                  // lanes per head
  constexpr int HPW = 32 / GROUP;                // heads per warp instruction
  const int tok = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int rot = a.rot_dim, half = rot >> 1, hl = half >> 3;   // hl: lanes between rotate-half partners
  const int heads = a.Hq + 2 * a.Hkv;
  const int gl = lane % GROUP, o = gl * 8;       // this lane's first element inside its head
  T* row = reinterpret_cast<T*>(a.qkv) + (size_t)tok * a.ld;
  int page = -1, slot = 0;
  if (a.k_pool) {
    const int seq = a.seq_of_tok ? a.seq_of_tok[tok] : tok;
    const int cpos = a.cache_pos ? a.cache_pos[tok] : a.pos[(size_t)tok * a.pos_stride];
    if (seq >= 0 && cpos >= 0) {
      page = a.page_table[(size_t)seq * a.pt_stride + (cpos >> 4)];
      slot = cpos & 15;
    }
  }
  const bool do_rope = a.cos != nullptr && rot > 0;
  const int region = o < half ? 0 : (o < rot ? 1 : 2);           // first half, second half, not rotated
  const int partner = lane + (region == 0 ? hl : (region == 1 ? -hl : 0));
  // cos / sin of this lane's eight frequencies (the same for every head of the token)
  float cs[8], sn[8];
  if (do_rope && region < 2) {
    const int i0 = region == 0 ? o : o - half;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = i0 + j;
      const int axis = a.axis_of_freq ? a.axis_of_freq[i] : 0;
      const int p = a.pos[(size_t)tok * a.pos_stride + axis];
      cs[j] = a.cos[(size_t)p * half + i];
      sn[j] = a.sin[(size_t)p * half + i];
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) { cs[j] = 1.f; sn[j] = 0.f; }
  }
  for (int h0 = warp * HPW; h0 < heads; h0 += nwarps * HPW) {
    const int h = h0 + lane / GROUP;
    const bool live = h < heads;
    const bool is_q = live && h < a.Hq, is_k = live && !is_q && h < a.Hq + a.Hkv, is_v = live && !is_q && !is_k;
    T* src = row + (size_t)(live ? h : 0) * HD + o;
    float x[8];
    if (live) load8(src, x);
    else {
#pragma unroll
      for (int j = 0; j < 8; ++j) x[j] = 0.f;
    }
    const T* nw = reinterpret_cast<const T*>(is_q ? a.q_norm_w : (is_k ? a.k_norm_w : nullptr));
    auto group_sum = [&](float v) {
#pragma unroll
      for (int d = GROUP / 2; d >= 1; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
      return v;
    };
    auto norm = [&]() {                          // every lane takes part in the shuffles; only q / k lanes with a weight change
      float s2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s2 += x[j] * x[j];
      s2 = group_sum(s2);
      if (nw) {
        const float rstd = rsqrtf(s2 / (float)HD + a.eps);
        float w[8];
        load8(nw + o, w);
#pragma unroll
        for (int j = 0; j < 8; ++j)
          x[j] = (a.norm_mode & 1) ? x[j] * rstd * (1.f + w[j]) : w[j] * Num<T>::to_f(Num<T>::from_f(x[j] * rstd));
      }
    };
    auto rope = [&]() {
      if (!do_rope) return;                      // uniform over the block
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float own = Num<T>::to_f(Num<T>::from_f(x[j]));        // the rotation acts on 16-bit values
        const float oth = __shfl_sync(0xffffffffu, own, partner);
        if ((is_q || is_k) && region < 2) x[j] = region == 0 ? own * cs[j] - oth * sn[j] : own * cs[j] + oth * sn[j];
      }
    };
    if (a.rope_before_norm) { rope(); norm(); } else { norm(); rope(); }
    if (is_q) {
      T* dst = a.q_out ? reinterpret_cast<T*>(a.q_out) + (size_t)tok * a.ldq + (size_t)h * HD + o : src;
      store8(dst, x);
    } else if (is_k) {
      const int kh = h - a.Hq;
      if (page >= 0) store8(reinterpret_cast<T*>(a.k_pool) + (((size_t)page * a.Hkv + kh) * 16 + slot) * HD + o, x);
      if (!a.k_pool || a.write_k_inplace) store8(src, x);
    }
    // value heads: optional unweighted RMS in place, then the page copy
    if (a.v_norm) {
      float raw[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) raw[j] = is_v ? x[j] : 0.f;
      float s2 = 0.f;
#pragma unroll
      for (int j = 0; j < 8; ++j) s2 += raw[j] * raw[j];
      s2 = group_sum(s2);
      if (is_v) {
        const float rstd = rsqrtf(s2 / (float)HD + a.eps);
#pragma unroll
        for (int j = 0; j < 8; ++j) x[j] = raw[j] * rstd;
        store8(src, x);
      }
    }
    if (is_v && page >= 0) {
      const int vh = h - a.Hq - a.Hkv;
      T* dst = reinterpret_cast<T*>(a.v_pool) + (((size_t)page * a.Hkv + vh) * 16 + slot) * HD + o;
      if (a.v_norm) store8(dst, x);
      else *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
    }
  }
}

// Rotate-half RoPE on a plain [tokens, heads, hd] tensor (public
// apply_rotary_pos_emb op; 2-D vision RoPE passes two axes via axis_of_freq).
}  // namespace rf

using namespace rf;

extern "C" int rf_qk_norm_rope_kv(const RfRopeKv* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->qkv, "rope_kv: null arguments");
  RF_REQUIRE(a->hd > 0 && a->hd % 2 == 0 && a->rot_dim <= a->hd && a->rot_dim % 2 == 0,
             "rope_kv: head_dim %d / rot_dim %d", a->hd, a->rot_dim);
  RF_REQUIRE(a->pos_stride >= 1, "rope_kv: pos_stride");
  if (a->k_pool) RF_REQUIRE(a->v_pool && a->page_table && a->hd % 8 == 0, "rope_kv: KV pool arguments");
  if (a->tokens == 0) return RF_OK;
  const int heads = a->Hq + 2 * a->Hkv;
  int warps = heads < 8 ? heads : 8;
  int gy = 1;
  if (a->tokens < 512) {  // decode-sized launches: one head per warp, heads across blockIdx.y
    warps = heads < 4 ? heads : 4;
    gy = ceil_div(heads, warps);
  }
  const size_t smem = (size_t)warps * a->hd * sizeof(float);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // prefill-sized launches on the common geometries take the 16-byte kernel (RF_ROPE_VEC=0: never)
  static const bool vec_on = [] { const char* e = getenv("RF_ROPE_VEC"); return !(e && e[0] == '0'); }();
  const bool aligned = a->ld % 8 == 0 && (reinterpret_cast<uintptr_t>(a->qkv) & 15) == 0 &&
                       (!a->q_out || (a->ldq % 8 == 0 && (reinterpret_cast<uintptr_t>(a->q_out) & 15) == 0)) &&
                       (!a->k_pool || ((reinterpret_cast<uintptr_t>(a->k_pool) | reinterpret_cast<uintptr_t>(a->v_pool)) & 15) == 0) &&
                       (!a->q_norm_w || (reinterpret_cast<uintptr_t>(a->q_norm_w) & 15) == 0) &&
                       (!a->k_norm_w || (reinterpret_cast<uintptr_t>(a->k_norm_w) & 15) == 0);
  if (vec_on && a->tokens >= 512 && aligned && a->rot_dim % 16 == 0 && (a->hd == 64 || a->hd == 128 || a->hd == 256)) {
    cudaError_t e;
#define RF_ROPE_VEC(T)                                                                                              \
    e = a->hd == 64 ? ::rf::launch_k(qk_norm_rope_kv_vec_kernel<T, 64>, dim3(a->tokens), dim3(256), 0, s, 1, *a)    \
      : a->hd == 128 ? ::rf::launch_k(qk_norm_rope_kv_vec_kernel<T, 128>, dim3(a->tokens), dim3(256), 0, s, 1, *a)  \
                     : ::rf::launch_k(qk_norm_rope_kv_vec_kernel<T, 256>, dim3(a->tokens), dim3(256), 0, s, 1, *a);
    if (a->dtype == 0) { RF_ROPE_VEC(__half) } else { RF_ROPE_VEC(__nv_bfloat16) }
#undef RF_ROPE_VEC
    RF_CUDA_CHECK(e);
    ::rf::count_launch();
    return RF_OK;
  }
  if (a->dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(qk_norm_rope_kv_kernel<__half>, dim3(a->tokens, gy), dim3(warps * 32), smem, s, 1, *a));
  else
    RF_CUDA_CHECK(::rf::launch_k(qk_norm_rope_kv_kernel<__nv_bfloat16>, dim3(a->tokens, gy), dim3(warps * 32), smem, s, 1, *a));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}
