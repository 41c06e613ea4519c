// Flash-style attention for head sizes beyond the tensor-memory kernels (head_dim 512: the global layers of Gemma4).
//
// With 512 output columns per head the O accumulator of a 128-row tile alone would fill all of tensor memory, so this
// path keeps O in registers on the warp-level tensor cores (mma.sync m16n8k16, fp32 accumulation): a CTA owns 64 query
// rows of one head; its eight warps are four row groups of 16 queries times two column halves of the head.  Both warps
// of a row group compute the same 16 x 32 score tile (S = Q K^T over all 512 channels) and each accumulates its 256
// output columns (O += P V), 128 fp32 registers per thread.  K / V arrive in 32-key tiles through cp.async, Q once.
// Varlen batches, causal / sliding-window masks and grouped KV heads follow the RfAttn contract of the other kernels
// (contiguous K / V rows; query row i of a sequence sits at position kv_len - q_len + i), so one launch serves prefill
// and decode (q_len = 1).  Reference behaviour: src/ops/rpu_sdpa.cpp:1-120 (mask kinds, softmax over the valid range),
// src/fused/rpu_gemma4_model.cpp:1-24 (per-layer head size, qk scale 1).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kWideBM = 64;       // query rows per CTA
constexpr int kWideBN = 32;       // keys per tile
constexpr int kWideThreads = 256;
constexpr int kWidePad = 8;       // elements of row padding: a 16-byte shift per row keeps ldmatrix conflict-free

struct WideParams {
  const void* q; int64_t ldq;
  void* out; int64_t ldo;
  const void* k; const void* v; int64_t ldk, ldv;
  const int32_t* q_start; const int32_t* q_len; const int32_t* kv_start; const int32_t* kv_len;
  int32_t Hq, G, causal, window;
  float scale_log2;
};

__device__ __forceinline__ void wide_cp16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  const __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h);
}

template <typename T, int HD>
__global__ void __launch_bounds__(kWideThreads, 1)
attn_wide_kernel(const WideParams p) {
  pdl_prologue();
  constexpr int LD = HD + kWidePad;            // shared-memory row pitch in elements
  constexpr int HALF = HD / 2;                 // output columns per warp
  constexpr int NT = HALF / 8;                 // 8-column output tiles per warp
  extern __shared__ __align__(16) uint8_t wsm[];
  T* sQ = reinterpret_cast<T*>(wsm);           // [64][LD]
  T* sK = sQ + kWideBM * LD;                   // [32][LD]
  T* sV = sK + kWideBN * LD;                   // [32][LD]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int rg = warp & 3, ch = warp >> 2;
  const int seq = blockIdx.z, h = blockIdx.y, q0 = blockIdx.x * kWideBM;
  const int qlen = p.q_len ? p.q_len[seq] : 1;
  if (q0 >= qlen) return;
  const int qs = p.q_start ? p.q_start[seq] : seq;
  const int kvs = p.kv_start[seq], kvl = p.kv_len[seq];
  const int hk = h / p.G;
  const int pos0 = kvl - qlen;                 // position of query row 0
  const T* Q = reinterpret_cast<const T*>(p.q);
  const T* Kp = reinterpret_cast<const T*>(p.k);
  const T* Vp = reinterpret_cast<const T*>(p.v);
  T* O = reinterpret_cast<T*>(p.out);

  // ---- Q tile (rows past the sequence read as zero)
  constexpr int PIECES = HD / 8;               // 16-byte pieces per row
  for (int i = tid; i < kWideBM * PIECES; i += kWideThreads) {
    const int r = i / PIECES, c = i % PIECES;
    const bool valid = q0 + r < qlen;
    wide_cp16(sQ + r * LD + c * 8, Q + (size_t)(qs + (valid ? q0 + r : 0)) * p.ldq + (size_t)h * HD + c * 8, valid);
  }
  asm volatile("cp.async.commit_group;" ::: "memory");

  // keys this tile can see
  const int q_last = min(q0 + kWideBM, qlen) - 1;
  int key_hi = p.causal ? min(kvl, pos0 + q_last + 1) : kvl;             // exclusive
  int key_lo = (p.window > 0) ? max(0, pos0 + q0 - p.window + 1) : 0;
  if (key_hi < 0) key_hi = 0;
  const int j_lo = key_lo / kWideBN, j_hi = (key_hi + kWideBN - 1) / kWideBN;

  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[n][e] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = q0 + rg * 16 + g, row_b = row_a + 8;                // this thread's two query rows
  const int pos_a = pos0 + row_a, pos_b = pos0 + row_b;

  for (int j = j_lo; j < j_hi; ++j) {
    __syncthreads();                                                      // the previous tile is no longer read
    const int k0 = j * kWideBN;
    for (int i = tid; i < kWideBN * PIECES; i += kWideThreads) {
      const int r = i / PIECES, c = i % PIECES;
      const bool valid = k0 + r < kvl;
      const size_t row = (size_t)(kvs + (valid ? k0 + r : 0));
      wide_cp16(sK + r * LD + c * 8, Kp + row * p.ldk + (size_t)hk * HD + c * 8, valid);
      wide_cp16(sV + r * LD + c * 8, Vp + row * p.ldv + (size_t)hk * HD + c * 8, valid);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();

    // ---- S = Q K^T (16 x 32 per warp)
    float s[4][4];
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) s[n][e] = 0.f;
#pragma unroll 4
    for (int ks = 0; ks < HD / 16; ++ks) {
      uint32_t a[4], b01[4], b23[4];
      ldsm_x4(a, sQ + (rg * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ks * 16 + (lane >> 4) * 8);
      ldsm_x4(b01, sK + ((lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
      ldsm_x4(b23, sK + (16 + (lane & 7) + (lane >> 4) * 8) * LD + ks * 16 + ((lane >> 3) & 1) * 8);
      mma_16816<T>(s[0], a, b01[0], b01[1]);
      mma_16816<T>(s[1], a, b01[2], b01[3]);
      mma_16816<T>(s[2], a, b23[0], b23[1]);
      mma_16816<T>(s[3], a, b23[2], b23[3]);
    }

    // ---- mask, online softmax (base-2 exponent with the scale folded in)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int n = 0; n < 4; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + n * 8 + 2 * t + (e & 1);
        const int pos = (e >> 1) ? pos_b : pos_a;
        bool ok = key < kvl;
        if (p.causal) ok = ok && key <= pos;
        if (p.window > 0) ok = ok && key > pos - p.window;
        const float v = ok ? s[n][e] * p.scale_log2 : -INFINITY;
        s[n][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    float alpha[2], m_use[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
      mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      const float m_new = fmaxf(m_run[r], mx[r]);
      m_use[r] = m_new == -INFINITY ? 0.f : m_new;                        // a row with nothing visible yet
      alpha[r] = exp2f(m_run[r] - m_use[r]);                              // exp2(-inf) = 0 on the first visible tile
      m_run[r] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pa[2][4];
#pragma unroll
    for (int n = 0; n < 4; ++n) {
      float e0 = exp2f(s[n][0] - m_use[0]), e1 = exp2f(s[n][1] - m_use[0]);
      float e2 = exp2f(s[n][2] - m_use[1]), e3 = exp2f(s[n][3] - m_use[1]);
      rs[0] += e0 + e1;
      rs[1] += e2 + e3;
      pa[n >> 1][(n & 1) * 2 + 0] = pack2<T>(e0, e1);
      pa[n >> 1][(n & 1) * 2 + 1] = pack2<T>(e2, e3);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
      rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
      l_run[r] = l_run[r] * alpha[r] + rs[r];
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= alpha[0];
      o[n][1] *= alpha[0];
      o[n][2] *= alpha[1];
      o[n][3] *= alpha[1];
    }

    // ---- O += P V over this warp's column half
#pragma unroll
    for (int kk = 0; kk < 2; ++kk) {
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        uint32_t b[4];
        ldsm_x4_trans(b, sV + (kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8) * LD + ch * HALF + n * 8 + (lane >> 4) * 8);
        mma_16816<T>(o[n], pa[kk], b[0], b[1]);
        mma_16816<T>(o[n + 1], pa[kk], b[2], b[3]);
      }
    }
  }
  if (j_lo >= j_hi) {                          // nothing visible: the Q copy is still in flight
    asm volatile("cp.async.wait_group 0;" ::: "memory");
  }

  // ---- normalise and store
  const float inv_a = l_run[0] > 0.f ? 1.f / l_run[0] : 0.f, inv_b = l_run[1] > 0.f ? 1.f / l_run[1] : 0.f;
#pragma unroll
  for (int n = 0; n < NT; ++n) {
    const int col = ch * HALF + n * 8 + 2 * t;
    if (row_a < qlen)
      *reinterpret_cast<uint32_t*>(O + (size_t)(qs + row_a) * p.ldo + (size_t)h * HD + col) = pack2<T>(o[n][0] * inv_a, o[n][1] * inv_a);
    if (row_b < qlen)
      *reinterpret_cast<uint32_t*>(O + (size_t)(qs + row_b) * p.ldo + (size_t)h * HD + col) = pack2<T>(o[n][2] * inv_b, o[n][3] * inv_b);
  }
}

}  // namespace rf

using namespace rf;

// Short problems on heads of 64 / 128 (a few dozen query rows over at most a few hundred keys: the self- and
// cross-attention of the action heads) also run here: no tensor maps, no tensor memory, one cp.async round trip per
// 32-key tile, which is less fixed cost than the tensor-memory kernel's set-up.  RF_ATTN_TINY=0 turns that routing off.
bool rf_attn_tiny_eligible(const RfAttn* a) {
  static const bool on = [] { const char* e = getenv("RF_ATTN_TINY"); return !(e && e[0] == '0'); }();
  if (!on || !a || a->k_pool || !a->k || !a->v || a->mask || a->seg_q || a->seg_k) return false;
  if (a->hd != 64 && a->hd != 128) return false;
  if (a->ldq % 8 || a->ldk % 8 || a->ldv % 8 || a->ldo % 2) return false;
  const int max_q = a->q_len ? a->max_q_len : 1;
  return max_q > 0 && max_q <= 64 && a->max_kv_len > 0 && a->max_kv_len <= 512;
}

template <typename T, int HD>
static int launch_wide(const WideParams& p, dim3 grid, cudaStream_t s) {
  constexpr size_t smem = (size_t)(kWideBM + 2 * kWideBN) * (HD + kWidePad) * 2;
  RF_ALLOW_SMEM_PER_DEVICE((attn_wide_kernel<T, HD>), smem);
  RF_CUDA_CHECK(::rf::launch_k(attn_wide_kernel<T, HD>, grid, dim3(kWideThreads), smem, s, 1, p));
  ::rf::count_launch();
  return RF_OK;
}

// Entry used by rf_attn_prefill for head sizes the tensor-memory kernels do not take, and for short problems.
int rf_attn_wide(const RfAttn* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->q && a->out, "attention needs q and out");
  RF_REQUIRE(a->hd == 512 || a->hd == 128 || a->hd == 64, "register-accumulator attention takes head_dim 64 / 128 / 512, got %d", a->hd);
  RF_REQUIRE(a->Hkv > 0 && a->Hq % a->Hkv == 0, "attention heads %d / kv heads %d", a->Hq, a->Hkv);
  RF_REQUIRE(a->k && a->v && a->kv_start && a->kv_len && !a->k_pool, "this attention path takes contiguous K / V rows (k, v, kv_start, kv_len)");
  RF_REQUIRE(!a->mask && !a->seg_q && !a->seg_k, "this attention path takes causal / window masks only");
  RF_REQUIRE(a->ldq % 8 == 0 && a->ldk % 8 == 0 && a->ldv % 8 == 0 && a->ldo % 2 == 0, "attention row pitches must be multiples of 16 bytes");
  RF_REQUIRE(a->num_seqs > 0 && (a->dtype == 0 || a->dtype == 1), "attention needs sequences and a 16-bit dtype");
  WideParams p;
  p.q = a->q; p.ldq = a->ldq; p.out = a->out; p.ldo = a->ldo;
  p.k = a->k; p.v = a->v; p.ldk = a->ldk; p.ldv = a->ldv;
  p.q_start = a->q_start; p.q_len = a->q_len; p.kv_start = a->kv_start; p.kv_len = a->kv_len;
  p.Hq = a->Hq; p.G = a->Hq / a->Hkv; p.causal = a->causal; p.window = a->window;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)a->hd);
  p.scale_log2 = scale * 1.4426950408889634f;
  const int max_q = a->q_len ? (a->max_q_len > 0 ? a->max_q_len : 1) : 1;
  const dim3 grid((max_q + kWideBM - 1) / kWideBM, a->Hq, a->num_seqs);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (a->dtype == 0) {
    if (a->hd == 512) return launch_wide<__half, 512>(p, grid, s);
    if (a->hd == 128) return launch_wide<__half, 128>(p, grid, s);
    return launch_wide<__half, 64>(p, grid, s);
  }
  if (a->hd == 512) return launch_wide<__nv_bfloat16, 512>(p, grid, s);
  if (a->hd == 128) return launch_wide<__nv_bfloat16, 128>(p, grid, s);
  return launch_wide<__nv_bfloat16, 64>(p, grid, s);
}
