// Fused per-head RMSNorm(q,k) -> RoPE -> KV-page insert, one launch after the
// QKV GEMM.  Covers 1-D rotate-half RoPE, interleaved/sectioned M-RoPE (per
// frequency lane axis select), partial rotary (rot_dim < head_dim) and 2-D
// vision RoPE (two position axes), and writes K/V straight into 16-token pages.
// Replaces five reference launches per layer: llama_rms_norm (per head),
// llama_rope / llama_mrope_interleave / partial_mrope / rope_2d and
// llama_insert_{k,v}cache (src/fused/rpu_qwen3_model.h:3378-3453,
// src/ops/rpu_rope.cpp, src/ops/rpu_mrope.cpp:37-124, src/ops/rpu_llama_kvcache.cpp).
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
  if (a->dtype == 0)
    RF_CUDA_CHECK(::rf::launch_k(qk_norm_rope_kv_kernel<__half>, dim3(a->tokens, gy), dim3(warps * 32), smem, s, 1, *a));
  else
    RF_CUDA_CHECK(::rf::launch_k(qk_norm_rope_kv_kernel<__nv_bfloat16>, dim3(a->tokens, gy), dim3(warps * 32), smem, s, 1, *a));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}
