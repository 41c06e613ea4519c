// Gated-DeltaNet (linear attention) kernels for the Qwen3.5 hybrid decoder:
//   * causal depthwise conv1d (kernel 4) with a carried per-sequence state + SiLU,
//   * the gated delta-rule recurrence over a [Dk, Dv] fp32 state per value head
//     (one launch covers decode -- one step from the stored state -- and prefill -- n
//     steps with the state held in registers, written back once),
//   * RMSNorm over Dv gated by silu(z),
//   * sigmoid output gate of the full-attention layers,
//   * the same rule in its chunked (block-parallel) form for prefill: 64 tokens per step as TF32 tensor-core products,
//   * last-dim cumulative sum and (I - M)^-1 of strictly-lower-triangular blocks, the two
//     helper operators of the chunked formulation.
// Semantics follow src/ops/rpu_gdn_recurrent.cpp:1-120 (decode step), src/ops/rpu_fla_conv1d.cpp,
// src/ops/rpu_cumsum.cpp, src/ops/rpu_unit_tril_inv.cpp and the op order of
// src/fused/rpu_qwen3_5_model.cpp:1301-1661.  The state of a head is split by COLUMNS over
// CTAs: column j of S only ever needs k, q, v[j], so Dv/32 CTAs per head run independently
// and a batch-1 decode step still fills Hv * Dv/32 SMs.
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

// ------------------------------------------------------------------ conv1d ----
// y[t, c] = silu( sum_j w[c, j] * xin[t - (K-1) + j, c] ), xin = [state | x] per sequence.
// One thread owns 8 adjacent channels of one token.
template <typename T, int KW>
__global__ void conv1d_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ y, int64_t ldy,
                              const T* __restrict__ w, const T* __restrict__ state,
                              const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len,
                              const int32_t* __restrict__ slot, int C, int tokens_per_block, int silu) {
  pdl_prologue();
  const int seq = blockIdx.z;
  const int s0 = q_start ? q_start[seq] : seq;
  const int n = q_len ? q_len[seq] : 1;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int sl = slot ? slot[seq] : seq;
  const T* st = state + (size_t)sl * (KW - 1) * C;
  float wk[KW][8];
#pragma unroll
  for (int ch = 0; ch < 8; ++ch) {
#pragma unroll
    for (int j = 0; j < KW; ++j) wk[j][ch] = Num<T>::to_f(w[(size_t)(c + ch) * KW + j]);
  }
  const int t0 = blockIdx.y * tokens_per_block;
  const int t1 = min(n, t0 + tokens_per_block);
  if (t0 >= n) return;
  // sliding window of the last KW-1 inputs
  float win[KW - 1][8];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) {
    const int ti = t0 - (KW - 1) + j;     // input index relative to the sequence start
    if (ti >= 0) load8(x + (size_t)(s0 + ti) * ldx + c, win[j]);
    else load8(st + (size_t)(KW - 1 + ti) * C + c, win[j]);
  }
  for (int t = t0; t < t1; ++t) {
    float cur[8], acc[8];
    load8(x + (size_t)(s0 + t) * ldx + c, cur);
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) {
      float a = wk[KW - 1][ch] * cur[ch];
#pragma unroll
      for (int j = 0; j < KW - 1; ++j) a += wk[j][ch] * win[j][ch];
      acc[ch] = silu ? silu_f(a) : a;
    }
    store8(y + (size_t)(s0 + t) * ldy + c, acc);
#pragma unroll
    for (int j = 0; j < KW - 2; ++j)
#pragma unroll
      for (int ch = 0; ch < 8; ++ch) win[j][ch] = win[j + 1][ch];
#pragma unroll
    for (int ch = 0; ch < 8; ++ch) win[KW - 2][ch] = cur[ch];
  }
}

// new state = last KW-1 rows of [old state | x]; runs after conv1d_kernel of the same call.
template <typename T, int KW>
__global__ void conv1d_state_kernel(const T* __restrict__ x, int64_t ldx, T* __restrict__ state,
                                    const int32_t* __restrict__ q_start, const int32_t* __restrict__ q_len,
                                    const int32_t* __restrict__ slot, int C) {
  pdl_prologue();
  const int seq = blockIdx.y;
  const int s0 = q_start ? q_start[seq] : seq;
  const int n = q_len ? q_len[seq] : 1;
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 8;
  if (c >= C) return;
  const int sl = slot ? slot[seq] : seq;
  T* st = state + (size_t)sl * (KW - 1) * C;
  float rows[KW - 1][8];
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) {
    const int ti = n - (KW - 1) + j;
    if (ti >= 0) load8(x + (size_t)(s0 + ti) * ldx + c, rows[j]);
    else load8(st + (size_t)(KW - 1 + ti) * C + c, rows[j]);
  }
#pragma unroll
  for (int j = 0; j < KW - 1; ++j) store8(st + (size_t)j * C + c, rows[j]);
}

// --------------------------------------------------------- delta rule ----
constexpr int kGdnCols = 32;     // state columns per CTA
constexpr int kGdnThreads = 128;  // 4 row groups x 32 columns

template <typename T, int DK>
__global__ void __launch_bounds__(kGdnThreads)
gdn_recurrent_kernel(const RfGdn p) {
  pdl_prologue();
  constexpr int RG = kGdnThreads / kGdnCols;   // row groups
  constexpr int RPT = DK / RG;                 // state rows per thread
  const int seq = blockIdx.z, hv = blockIdx.y;
  const int col = threadIdx.x % kGdnCols, rg = threadIdx.x / kGdnCols;
  const int j = blockIdx.x * kGdnCols + col;   // state column = value channel
  const int hk = hv / (p.Hv / p.Hk);
  const int s0 = p.q_start ? p.q_start[seq] : seq;
  const int n = p.q_len ? p.q_len[seq] : 1;
  const int sl = p.slot ? p.slot[seq] : seq;
  const int fresh = p.fresh ? p.fresh[seq] : 0;
  float* S = p.state + (((size_t)sl * p.Hv + hv) * DK) * p.Dv;
  const T* qkv = reinterpret_cast<const T*>(p.qkv);
  const T* bp = reinterpret_cast<const T*>(p.b);
  const T* ap = reinterpret_cast<const T*>(p.a);
  T* out = reinterpret_cast<T*>(p.out);
  const int q_off = hk * DK, k_off = p.Hk * DK + hk * DK, v_off = 2 * p.Hk * DK + hv * p.Dv;
  const float A = -__expf(p.A_log[hv]), dtb = p.dt_bias[hv];
  const float qscale = rsqrtf((float)DK);

  __shared__ float sq[DK], sk[DK];
  __shared__ float red[2][RG][kGdnCols];
  __shared__ float ssum[2][kGdnThreads / 32];

  float st[RPT];
#pragma unroll
  for (int r = 0; r < RPT; ++r) st[r] = fresh ? 0.f : S[(size_t)(rg * RPT + r) * p.Dv + j];

  for (int t = 0; t < n; ++t) {
    const size_t row = (size_t)(s0 + t);
    // L2-normalise q and k of this head (all 128 threads; DK == 128 -> one element each)
    float qv = 0.f, kv = 0.f;
    for (int i = threadIdx.x; i < DK; i += kGdnThreads) {
      qv = Num<T>::to_f(qkv[row * p.ld + q_off + i]);
      kv = Num<T>::to_f(qkv[row * p.ld + k_off + i]);
    }
    float q2 = qv * qv, k2 = kv * kv;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      q2 += __shfl_xor_sync(0xffffffffu, q2, o);
      k2 += __shfl_xor_sync(0xffffffffu, k2, o);
    }
    if ((threadIdx.x & 31) == 0) {
      ssum[0][threadIdx.x >> 5] = q2;
      ssum[1][threadIdx.x >> 5] = k2;
    }
    __syncthreads();
    float qn = 0.f, kn = 0.f;
#pragma unroll
    for (int w = 0; w < kGdnThreads / 32; ++w) {
      qn += ssum[0][w];
      kn += ssum[1][w];
    }
    if (threadIdx.x < DK) {
      sq[threadIdx.x] = qv * rsqrtf(qn + 1e-6f) * qscale;
      sk[threadIdx.x] = kv * rsqrtf(kn + 1e-6f);
    }
    const float beta = 1.f / (1.f + __expf(-Num<T>::to_f(bp[row * p.ld_ba + hv])));
    const float ar = Num<T>::to_f(ap[row * p.ld_ba + hv]) + dtb;
    const float sp = ar > 20.f ? ar : log1pf(__expf(ar));
    const float decay = __expf(A * sp);
    const float vj = Num<T>::to_f(qkv[row * p.ld + v_off + j]);
    __syncthreads();
    // S *= decay ; kv_mem[j] = sum_i S[i, j] k[i]
    float part = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      st[r] *= decay;
      part += st[r] * sk[rg * RPT + r];
    }
    red[0][rg][col] = part;
    __syncthreads();
    float kvm = 0.f;
#pragma unroll
    for (int g = 0; g < RG; ++g) kvm += red[0][g][col];
    const float delta = (vj - kvm) * beta;
    float po = 0.f;
#pragma unroll
    for (int r = 0; r < RPT; ++r) {
      st[r] += sk[rg * RPT + r] * delta;
      po += st[r] * sq[rg * RPT + r];
    }
    red[1][rg][col] = po;
    __syncthreads();
    if (rg == 0) {
      float o = 0.f;
#pragma unroll
      for (int g = 0; g < RG; ++g) o += red[1][g][col];
      out[row * p.ldo + hv * p.Dv + j] = Num<T>::from_f(o);
    }
  }
#pragma unroll
  for (int r = 0; r < RPT; ++r) S[(size_t)(rg * RPT + r) * p.Dv + j] = st[r];
}

// ------------------------------------------------ chunked delta rule (prefill) ----
// The same recurrence evaluated 64 tokens at a time on the tensor cores.  With G_i the cumulative log decay inside a
// chunk, S0 the incoming state and L_ij = beta_i e^{G_i - G_j} (k_i . k_j) for j < i:
//     (I + L) U = beta * (V - e^G * (K S0))
//     O  = e^G * (Q S0) + tril(e^{G_i - G_j} (q_i . k_j)) U
//     S' = e^{G_C} S0 + K^T (e^{G_C - G} * U)
// One CTA owns 32 state columns of one value head of one sequence (the same split as the recurrent kernel) and walks
// the sequence's chunks with its [128 x 32] state slice resident in shared memory.  Every product is an fp32-accumulate
// TF32 mma.sync (operands rounded to nearest): the state stays fp32 between chunks, and every decay factor that appears
// is e^{G_i - G_j} with j <= i, at most one.  The unit-triangular system is solved in 16-row blocks: the four diagonal
// blocks are inverted by forward substitution (one warp each), the rest is block forward substitution on the 32
// right-hand-side columns.  Rows past the end of a sequence are zero tokens with beta = 0 and no decay, which leave both
// the outputs of the real rows and the state untouched.
constexpr int kGcC = 64;          // tokens per chunk
constexpr int kGcThreads = 256;
constexpr int kGcLdQK = 132;      // fp32 row pitch of the q / k tiles: (4 * row + col) mod 32 is distinct over a fragment
constexpr int kGcLdS = 40;        // row pitch of the state slice and of the v / rhs / u tile
constexpr int kGcLdL = 68;        // row pitch of the two chunk x chunk matrices
constexpr int kGcLdD = 17;
constexpr int kGcSmemFloats = 2 * kGcC * kGcLdQK + 128 * kGcLdS + 2 * kGcC * kGcLdS + 2 * kGcC * kGcLdL + 4 * 16 * kGcLdD + 3 * kGcC;
// + the raw 16-bit q | k rows and v slice of the NEXT chunk, fetched with cp.async while this chunk is computed
constexpr int kGcRawElems = kGcC * 256 + kGcC * kGdnCols;
constexpr size_t kGcSmemBytes = (size_t)kGcSmemFloats * sizeof(float) + (size_t)kGcRawElems * 2;

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? 16 : 0;                      // 0 source bytes: the 16 destination bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gsrc), "r"(n) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// A fragment of a row-major fp32 tile: rows r0 + {g, g + 8}, columns c0 + {t, t + 4}
__device__ __forceinline__ void frag_a(uint32_t (&a)[4], const float* m, int ld, int r0, int c0, int g, int t) {
  a[0] = to_tf32(m[(r0 + g) * ld + c0 + t]);
  a[1] = to_tf32(m[(r0 + g + 8) * ld + c0 + t]);
  a[2] = to_tf32(m[(r0 + g) * ld + c0 + t + 4]);
  a[3] = to_tf32(m[(r0 + g + 8) * ld + c0 + t + 4]);
}

// the same for a tile whose values were rounded to TF32 when they were stored
__device__ __forceinline__ void frag_a_bits(uint32_t (&a)[4], const float* m, int ld, int r0, int c0, int g, int t) {
  a[0] = __float_as_uint(m[(r0 + g) * ld + c0 + t]);
  a[1] = __float_as_uint(m[(r0 + g + 8) * ld + c0 + t]);
  a[2] = __float_as_uint(m[(r0 + g) * ld + c0 + t + 4]);
  a[3] = __float_as_uint(m[(r0 + g + 8) * ld + c0 + t + 4]);
}

template <typename T>
__global__ void __launch_bounds__(kGcThreads, 1)
gdn_chunked_kernel(const RfGdn p) {
  pdl_prologue();
  constexpr int DK = 128, C = kGcC, NV = kGdnCols;
  extern __shared__ __align__(16) float gsm[];
  float* sQ = gsm;
  float* sK = sQ + C * kGcLdQK;
  float* sS = sK + C * kGcLdQK;
  float* sV = sS + DK * kGcLdS;
  float* sU = sV + C * kGcLdS;
  float* sL = sU + C * kGcLdS;
  float* sP = sL + C * kGcLdL;
  float* sD = sP + C * kGcLdL;
  float* sG = sD + 4 * 16 * kGcLdD;
  float* sBeta = sG + C;
  float* sg = sBeta + C;
  T* rawQK = reinterpret_cast<T*>(sg + C);             // [C][q 128 | k 128]
  T* rawV = rawQK + C * 256;                           // [C][32]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int seq = blockIdx.z, hv = blockIdx.y, j0 = blockIdx.x * NV;
  const int hk = hv / (p.Hv / p.Hk);
  const int s0 = p.q_start ? p.q_start[seq] : seq;
  const int n = p.q_len ? p.q_len[seq] : 1;
  const int sl = p.slot ? p.slot[seq] : seq;
  const int fresh = p.fresh ? p.fresh[seq] : 0;
  float* S = p.state + (((size_t)sl * p.Hv + hv) * DK) * p.Dv + j0;
  const T* qkv = reinterpret_cast<const T*>(p.qkv);
  const T* bp = reinterpret_cast<const T*>(p.b);
  const T* ap = reinterpret_cast<const T*>(p.a);
  T* out = reinterpret_cast<T*>(p.out);
  const int q_off = hk * DK, k_off = p.Hk * DK + hk * DK, v_off = 2 * p.Hk * DK + hv * p.Dv + j0;
  const float A = -__expf(p.A_log[hv]), dtb = p.dt_bias[hv];
  const float qscale = rsqrtf((float)DK);

  for (int i = tid; i < DK * NV; i += kGcThreads) {
    const int m = i / NV, c = i % NV;
    sS[m * kGcLdS + c] = fresh ? 0.f : S[(size_t)m * p.Dv + c];
  }

  float nb = 0.f, na = 0.f;                            // beta / decay inputs of row `tid` of the chunk in flight
  auto prefetch = [&](int cn) {
    if (cn < n) {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int idx = tid + kGcThreads * k, i = idx >> 5, part = idx & 31;
        const bool valid = cn + i < n;
        const size_t row = (size_t)(s0 + (valid ? cn + i : 0));
        cp_async16(rawQK + i * 256 + part * 8, qkv + row * p.ld + (part < 16 ? q_off + part * 8 : k_off + (part - 16) * 8), valid);
      }
      {
        const int i = tid >> 2, part = tid & 3;
        const bool valid = cn + i < n;
        const size_t row = (size_t)(s0 + (valid ? cn + i : 0));
        cp_async16(rawV + i * NV + part * 8, qkv + row * p.ld + v_off + part * 8, valid);
      }
      if (tid < C && cn + tid < n) {
        const size_t row = (size_t)(s0 + cn + tid);
        nb = Num<T>::to_f(bp[row * p.ld_ba + hv]);
        na = Num<T>::to_f(ap[row * p.ld_ba + hv]);
      }
    }
    cp_async_commit();
  };
  prefetch(0);

  for (int c0 = 0; c0 < n; c0 += C) {
    // ---- this chunk's rows arrived through cp.async: L2-normalise q (pre-scaled) and k, widen the v slice
    cp_async_wait_all();
    __syncthreads();
#pragma unroll
    for (int rr = 0; rr < 8; ++rr) {
      const int i = warp * 8 + rr;
      const int half = lane >> 4, l16 = lane & 15;
      float f[8];
      load8(rawQK + i * 256 + half * 128 + l16 * 8, f);
      float ss = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += f[e] * f[e];
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float sc = rsqrtf(ss + 1e-6f) * (half ? 1.f : qscale);
      float* dst = (half ? sK : sQ) + i * kGcLdQK + l16 * 8;
#pragma unroll
      for (int e = 0; e < 8; ++e) dst[e] = __uint_as_float(to_tf32(f[e] * sc));   // rounded once here, read as TF32 bits below
    }
    {
      const int i = tid >> 2, part = tid & 3;
      float vv[8];
      load8(rawV + i * NV + part * 8, vv);
#pragma unroll
      for (int e = 0; e < 8; ++e) sV[i * kGcLdS + part * 8 + e] = vv[e];
    }
    if (tid < C) {
      float beta = 0.f, lg = 0.f;
      if (c0 + tid < n) {
        beta = 1.f / (1.f + __expf(-nb));
        const float ar = na + dtb;
        lg = A * (ar > 20.f ? ar : log1pf(__expf(ar)));
      }
      sBeta[tid] = beta;
      sg[tid] = lg;
    }
    __syncthreads();
    prefetch(c0 + C);                                  // the raw buffers are free again: fetch the next chunk behind the math
    if (warp == 0) {      // inclusive prefix sum of the log decays
      const float x0 = sg[2 * lane], x1 = sg[2 * lane + 1];
      float run = x0 + x1;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, run, o);
        if (lane >= o) run += y;
      }
      sG[2 * lane] = run - x1;
      sG[2 * lane + 1] = run;
    }
    __syncthreads();

    // ---- L = beta_i e^{G_i - G_j} (k_i . k_j) [j < i],  P = e^{G_i - G_j} (q_i . k_j) [j <= i]
    {
      const int rt = warp >> 1, cnt = rt + 1, nt0 = (warp & 1) * cnt;   // row tile rt has 2 (rt + 1) column tiles on or below the diagonal
      float accL[4][4], accP[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) accL[a][b] = accP[a][b] = 0.f;
#pragma unroll 4
      for (int ks = 0; ks < DK / 8; ++ks) {
        uint32_t aK[4], aQ[4];
        frag_a_bits(aK, sK, kGcLdQK, rt * 16, ks * 8, g, t);
        frag_a_bits(aQ, sQ, kGcLdQK, rt * 16, ks * 8, g, t);
#pragma unroll
        for (int ti = 0; ti < 4; ++ti) {
          if (ti < cnt) {
            const int col = (nt0 + ti) * 8 + g;
            uint32_t b[2];
            b[0] = __float_as_uint(sK[col * kGcLdQK + ks * 8 + t]);
            b[1] = __float_as_uint(sK[col * kGcLdQK + ks * 8 + t + 4]);
            mma_tf32(accL[ti], aK, b);
            mma_tf32(accP[ti], aQ, b);
          }
        }
      }
#pragma unroll
      for (int ti = 0; ti < 4; ++ti) {
        if (ti < cnt) {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int i = rt * 16 + g + (e >> 1) * 8, j = (nt0 + ti) * 8 + 2 * t + (e & 1);
            const float dec = j <= i ? __expf(sG[i] - sG[j]) : 0.f;
            sL[i * kGcLdL + j] = j < i ? sBeta[i] * dec * accL[ti][e] : 0.f;
            sP[i * kGcLdL + j] = __uint_as_float(to_tf32(dec * accP[ti][e]));
          }
        }
      }
    }
    __syncthreads();

    // ---- inverses of the four 16 x 16 diagonal blocks of I + L (warps 0..3, one column per lane)
    if (warp < 4 && lane < 16) {
      float x[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float acc = i == lane ? 1.f : 0.f;
#pragma unroll
        for (int j = 0; j < i; ++j) acc -= sL[(warp * 16 + i) * kGcLdL + warp * 16 + j] * x[j];
        x[i] = acc;
        sD[(warp * 16 + i) * kGcLdD + lane] = acc;
      }
    }

    // ---- rhs = beta (V - e^G (K S0)) in place of V;  accO = e^G (Q S0)
    const int rt = warp & 3, nh = warp >> 2;
    float accO[2][4];
    {
      float accR[2][4];
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int b = 0; b < 4; ++b) accR[a][b] = accO[a][b] = 0.f;
#pragma unroll 4
      for (int ks = 0; ks < DK / 8; ++ks) {
        uint32_t aK[4], aQ[4];
        frag_a_bits(aK, sK, kGcLdQK, rt * 16, ks * 8, g, t);
        frag_a_bits(aQ, sQ, kGcLdQK, rt * 16, ks * 8, g, t);
#pragma unroll
        for (int a = 0; a < 2; ++a) {
          const int col = (nh * 2 + a) * 8 + g;
          uint32_t b[2];
          b[0] = to_tf32(sS[(ks * 8 + t) * kGcLdS + col]);
          b[1] = to_tf32(sS[(ks * 8 + t + 4) * kGcLdS + col]);
          mma_tf32(accR[a], aK, b);
          mma_tf32(accO[a], aQ, b);
        }
      }
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int i = rt * 16 + g + (e >> 1) * 8, j = (nh * 2 + a) * 8 + 2 * t + (e & 1);
          const float eg = __expf(sG[i]);
          sV[i * kGcLdS + j] = sBeta[i] * (sV[i * kGcLdS + j] - eg * accR[a][e]);
          accO[a][e] *= eg;
        }
    }
    __syncthreads();

    // ---- U = (I + L)^-1 rhs by block forward substitution: rhs rows in sV, finished rows in sU
    {
      const int r = tid >> 4, cc = (tid & 15) * 2;
      for (int b = 0; b < 4; ++b) {
        const int i = b * 16 + r;
        float a0 = sV[i * kGcLdS + cc], a1 = sV[i * kGcLdS + cc + 1];
#pragma unroll 4
        for (int j = 0; j < b * 16; ++j) {
          const float l = sL[i * kGcLdL + j];
          a0 -= l * sU[j * kGcLdS + cc];
          a1 -= l * sU[j * kGcLdS + cc + 1];
        }
        sV[i * kGcLdS + cc] = a0;          // a row of block b is touched by its owner only until the barrier
        sV[i * kGcLdS + cc + 1] = a1;
        __syncthreads();
        float u0 = 0.f, u1 = 0.f;
        for (int r2 = 0; r2 <= r; ++r2) {
          const float d = sD[i * kGcLdD + r2];
          u0 += d * sV[(b * 16 + r2) * kGcLdS + cc];
          u1 += d * sV[(b * 16 + r2) * kGcLdS + cc + 1];
        }
        sU[i * kGcLdS + cc] = u0;
        sU[i * kGcLdS + cc + 1] = u1;
        __syncthreads();
      }
    }

    // ---- O = accO + P U
    for (int ks = 0; ks <= 2 * rt + 1; ++ks) {
      uint32_t aP[4];
      frag_a_bits(aP, sP, kGcLdL, rt * 16, ks * 8, g, t);
#pragma unroll
      for (int a = 0; a < 2; ++a) {
        const int col = (nh * 2 + a) * 8 + g;
        uint32_t b[2];
        b[0] = to_tf32(sU[(ks * 8 + t) * kGcLdS + col]);
        b[1] = to_tf32(sU[(ks * 8 + t + 4) * kGcLdS + col]);
        mma_tf32(accO[a], aP, b);
      }
    }
#pragma unroll
    for (int a = 0; a < 2; ++a)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = rt * 16 + g + (e >> 1) * 8, j = (nh * 2 + a) * 8 + 2 * t + (e & 1);
        if (c0 + i < n) out[(size_t)(s0 + c0 + i) * p.ldo + hv * p.Dv + j0 + j] = Num<T>::from_f(accO[a][e]);
      }

    // ---- S' = e^{G_C} S0 + K^T (e^{G_C - G} * U): warp w owns state rows 16 w .. 16 w + 15
    {
      const float gl = sG[C - 1], egl = __expf(gl);
      float accS[4][4];
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          accS[a][e] = egl * sS[(warp * 16 + g + (e >> 1) * 8) * kGcLdS + a * 8 + 2 * t + (e & 1)];
#pragma unroll
      for (int ks = 0; ks < C / 8; ++ks) {
        const int ca = ks * 8 + t, cb = ks * 8 + t + 4;
        uint32_t aT[4];
        aT[0] = __float_as_uint(sK[ca * kGcLdQK + warp * 16 + g]);
        aT[1] = __float_as_uint(sK[ca * kGcLdQK + warp * 16 + g + 8]);
        aT[2] = __float_as_uint(sK[cb * kGcLdQK + warp * 16 + g]);
        aT[3] = __float_as_uint(sK[cb * kGcLdQK + warp * 16 + g + 8]);
        const float wa = __expf(gl - sG[ca]), wb = __expf(gl - sG[cb]);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          uint32_t b[2];
          b[0] = to_tf32(wa * sU[ca * kGcLdS + a * 8 + g]);
          b[1] = to_tf32(wb * sU[cb * kGcLdS + a * 8 + g]);
          mma_tf32(accS[a], aT, b);
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int e = 0; e < 4; ++e)
          sS[(warp * 16 + g + (e >> 1) * 8) * kGcLdS + a * 8 + 2 * t + (e & 1)] = accS[a][e];
    }
    __syncthreads();
  }

  for (int i = tid; i < DK * NV; i += kGcThreads) {
    const int m = i / NV, c = i % NV;
    S[(size_t)m * p.Dv + c] = sS[m * kGcLdS + c];
  }
}

// ------------------------------------------------- gated RMSNorm over Dv ----
// y = (w * rmsnorm(x)) * silu(z); one warp per (token, head) row of D <= 256 values.
template <typename T>
__global__ void rmsnorm_gated_kernel(const T* __restrict__ x, int64_t ldx, const T* __restrict__ z, int64_t ldz,
                                     const T* __restrict__ w, T* __restrict__ y, int64_t ldy, int rows, int heads,
                                     int D, float eps) {
  pdl_prologue();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  const int t = r / heads, h = r % heads;
  const T* xr = x + (size_t)t * ldx + (size_t)h * D;
  const T* zr = z + (size_t)t * ldz + (size_t)h * D;
  T* yr = y + (size_t)t * ldy + (size_t)h * D;
  float v[8];
  float ss = 0.f;
  const int per = D / 32;      // 2, 4 or 8
  for (int i = 0; i < per; ++i) {
    v[i] = Num<T>::to_f(xr[lane * per + i]);
    ss += v[i] * v[i];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = rsqrtf(ss / (float)D + eps);
  for (int i = 0; i < per; ++i) {
    const int c = lane * per + i;
    const float nx = Num<T>::to_f(Num<T>::from_f(v[i] * inv));   // rounded like the unfused form
    yr[c] = Num<T>::from_f(Num<T>::to_f(w[c]) * nx * silu_f(Num<T>::to_f(zr[c])));
  }
}

// a[t, c] *= sigmoid(g[t, c])  (8 channels per thread; pitches in elements)
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ a, int64_t lda, const T* __restrict__ g, int64_t ldg,
                                    int rows, int cols) {
  pdl_prologue();
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int per_row = cols / 8;
  if (idx >= (int64_t)rows * per_row) return;
  const int t = (int)(idx / per_row), c = (int)(idx % per_row) * 8;
  float x[8], y[8];
  load8(a + (size_t)t * lda + c, x);
  load8(g + (size_t)t * ldg + c, y);
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] *= 1.f / (1.f + __expf(-y[i]));
  store8(a + (size_t)t * lda + c, x);
}

// inclusive cumulative sum over the last dim (n <= 1024), one warp per row, fp32
__global__ void cumsum_kernel(const float* __restrict__ x, float* __restrict__ y, int rows, int n) {
  pdl_prologue();
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (r >= rows) return;
  const int lane = threadIdx.x & 31;
  float carry = 0.f;
  for (int base = 0; base < n; base += 32) {
    const int i = base + lane;
    float v = i < n ? x[(size_t)r * n + i] : 0.f;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float u = __shfl_up_sync(0xffffffffu, v, o);
      if (lane >= o) v += u;
    }
    v += carry;
    if (i < n) y[(size_t)r * n + i] = v;
    carry = __shfl_sync(0xffffffffu, v, 31);
  }
}

// X = (I - M)^-1 for a batch of n x n (n <= 64) blocks whose strict lower triangle is M
// (everything on and above the diagonal of the input is ignored).  Forward substitution,
// one CTA per block, one thread per column: X[i, :] = e_i + sum_{k<i} M[i, k] X[k, :].
__global__ void unit_tril_inv_kernel(const float* __restrict__ m, float* __restrict__ out, int n) {
  pdl_prologue();
  __shared__ float M[64][65], X[64][65];
  const float* mb = m + (size_t)blockIdx.x * n * n;
  float* ob = out + (size_t)blockIdx.x * n * n;
  for (int i = threadIdx.x; i < n * n; i += blockDim.x) {
    M[i / n][i % n] = mb[i];
    X[i / n][i % n] = 0.f;
  }
  __syncthreads();
  const int c = threadIdx.x;
  for (int i = 0; i < n; ++i) {
    if (c < n) {
      float acc = (c == i) ? 1.f : 0.f;
      for (int k = 0; k < i; ++k) acc += M[i][k] * X[k][c];
      X[i][c] = acc;
    }
    __syncthreads();
  }
  for (int i = threadIdx.x; i < n * n; i += blockDim.x) ob[i] = X[i / n][i % n];
}

}  // namespace rf

using namespace rf;

#define RF_DISPATCH_T(dtype, ...)                      \
  if ((dtype) == 0) { using T = __half; __VA_ARGS__; } \
  else { using T = __nv_bfloat16; __VA_ARGS__; }

extern "C" int rf_causal_conv1d(const RfConv1d* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->x && a->y && a->w && a->state, "conv1d: null argument");
  RF_REQUIRE(a->K == 4, "conv1d: kernel size %d (only 4 is built)", a->K);
  RF_REQUIRE(a->C % 8 == 0 && a->ldx % 8 == 0 && a->ldy % 8 == 0, "conv1d: channels and pitches must be multiples of 8");
  RF_REQUIRE(a->num_seqs > 0, "conv1d: no sequences");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int threads = 128;
  const int cblocks = (a->C / 8 + threads - 1) / threads;
  const int max_len = a->q_len ? (a->max_q_len > 0 ? a->max_q_len : 1) : 1;
  const int tpb = 32;
  const int tblocks = (max_len + tpb - 1) / tpb;
  RF_DISPATCH_T(a->dtype, {
    RF_CUDA_CHECK(::rf::launch_k(conv1d_kernel<T, 4>, dim3(cblocks, tblocks, a->num_seqs), dim3(threads), 0, s, 1,
                                 (const T*)a->x, a->ldx, (T*)a->y, a->ldy, (const T*)a->w, (const T*)a->state,
                                 a->q_start, a->q_len, a->slot, a->C, tpb, a->silu));
    ::rf::count_launch();
    RF_CUDA_CHECK(::rf::launch_k(conv1d_state_kernel<T, 4>, dim3(cblocks, a->num_seqs), dim3(threads), 0, s, 1,
                                 (const T*)a->x, a->ldx, (T*)a->state, a->q_start, a->q_len, a->slot, a->C));
    ::rf::count_launch();
  });
  return RF_OK;
}

extern "C" int rf_gdn_recurrent(const RfGdn* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->qkv && a->b && a->a && a->out && a->state && a->A_log && a->dt_bias, "gdn: null argument");
  RF_REQUIRE(a->Dk == 128, "gdn: key head dim %d (only 128 is built)", a->Dk);
  RF_REQUIRE(a->Dv % kGdnCols == 0 && a->Hv % a->Hk == 0 && a->Hk > 0, "gdn: head geometry Hk=%d Hv=%d Dv=%d", a->Hk, a->Hv, a->Dv);
  RF_REQUIRE(a->num_seqs > 0, "gdn: no sequences");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(a->Dv / kGdnCols, a->Hv, a->num_seqs);
  if (a->dtype == 0) RF_CUDA_CHECK(::rf::launch_k(gdn_recurrent_kernel<__half, 128>, grid, dim3(kGdnThreads), 0, s, 1, *a));
  else RF_CUDA_CHECK(::rf::launch_k(gdn_recurrent_kernel<__nv_bfloat16, 128>, grid, dim3(kGdnThreads), 0, s, 1, *a));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_gdn_chunked(const RfGdn* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->qkv && a->b && a->a && a->out && a->state && a->A_log && a->dt_bias, "gdn: null argument");
  RF_REQUIRE(a->Dk == 128, "gdn: key head dim %d (only 128 is built)", a->Dk);
  RF_REQUIRE(a->Dv % kGdnCols == 0 && a->Hv % a->Hk == 0 && a->Hk > 0, "gdn: head geometry Hk=%d Hv=%d Dv=%d", a->Hk, a->Hv, a->Dv);
  RF_REQUIRE(a->ld % 8 == 0 && (a->Hk * a->Dk) % 8 == 0 && a->Dv % 8 == 0, "gdn: the chunked form reads 16-byte vectors (pitch %lld)", (long long)a->ld);
  RF_REQUIRE(a->num_seqs > 0, "gdn: no sequences");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const dim3 grid(a->Dv / kGdnCols, a->Hv, a->num_seqs);
  constexpr size_t smem = kGcSmemBytes;
  if (a->dtype == 0) {
    RF_ALLOW_SMEM_PER_DEVICE(gdn_chunked_kernel<__half>, smem);
    RF_CUDA_CHECK(::rf::launch_k(gdn_chunked_kernel<__half>, grid, dim3(kGcThreads), smem, s, 1, *a));
  } else {
    RF_ALLOW_SMEM_PER_DEVICE(gdn_chunked_kernel<__nv_bfloat16>, smem);
    RF_CUDA_CHECK(::rf::launch_k(gdn_chunked_kernel<__nv_bfloat16>, grid, dim3(kGcThreads), smem, s, 1, *a));
  }
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_rmsnorm_gated(const void* x, int64_t ldx, const void* z, int64_t ldz, const void* w, void* y,
                                int64_t ldy, int tokens, int heads, int D, float eps, int dtype, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(x && z && w && y, "rmsnorm_gated: null argument");
  RF_REQUIRE(D % 32 == 0 && D <= 256, "rmsnorm_gated: width %d must be a multiple of 32, at most 256", D);
  if (tokens == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int rows = tokens * heads, wpb = 8;
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(rmsnorm_gated_kernel<T>, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0,
                                                    s, 1, (const T*)x, ldx, (const T*)z, ldz, (const T*)w, (T*)y, ldy,
                                                    rows, heads, D, eps)));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_sigmoid_gate(void* a, int64_t lda, const void* g, int64_t ldg, int rows, int cols, int dtype,
                               rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && g && cols % 8 == 0 && lda % 8 == 0 && ldg % 8 == 0, "sigmoid_gate arguments");
  if (rows == 0) return RF_OK;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int64_t n = (int64_t)rows * (cols / 8);
  RF_DISPATCH_T(dtype, RF_CUDA_CHECK(::rf::launch_k(sigmoid_gate_kernel<T>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, s,
                                                    1, (T*)a, lda, (const T*)g, ldg, rows, cols)));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_cumsum_f32(const float* x, float* y, int rows, int n, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(x && y && n > 0, "cumsum arguments");
  if (rows == 0) return RF_OK;
  RF_CUDA_CHECK(::rf::launch_k(cumsum_kernel, dim3((rows + 3) / 4), dim3(128), 0, static_cast<cudaStream_t>(stream), 1, x, y,
                               rows, n));
  ::rf::count_launch();
  return RF_OK;
}

extern "C" int rf_unit_tril_inv_f32(const float* m, float* out, int batch, int n, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(m && out && n > 0 && n <= 64, "unit_tril_inv: n=%d (1..64)", n);
  if (batch == 0) return RF_OK;
  RF_CUDA_CHECK(::rf::launch_k(unit_tril_inv_kernel, dim3(batch), dim3(64), 0, static_cast<cudaStream_t>(stream), 1, m, out, n));
  ::rf::count_launch();
  return RF_OK;
}
