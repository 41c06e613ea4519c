// Latency-bound GEMMs: at most a few hundred token rows against a weight of a few megabytes (the per-layer projections
// of the action heads and diffusion policies: 31 - 128 rows, widths 384 - 6144).
//
// For these shapes the tcgen05 streaming kernel spends its time on set-up - tensor maps, tensor-memory allocation, a ring
// that is deeper than the problem - and on too few CTAs, each limited to what one SM can load (measured: 11 - 20 us
// where the arithmetic and the bytes need 2 - 3 us).  This kernel is built for the opposite regime:
//   * no tensor memory, no tensor maps: warp-level mma.sync (m16n8k16, fp32 accumulation) on tiles staged with cp.async;
//   * a CTA owns 64 output features (half a 128-row block of the tile-major weight image, whose 128-byte swizzle is
//     exactly what ldmatrix wants) and up to 128 token rows; the token tile is staged with the same swizzle;
//   * split K across a thread-block cluster (2 / 4 / 8 CTAs): both operands are split, so a CTA loads only its K range
//     of the tokens; partial tiles are summed over distributed shared memory, each CTA finishing its share of the rows;
//   * bias, activation (also the GLU forms: the CTA then carries the gate and the up tile) and residual in the epilogue.
// Reference behaviour: the epilogue options of src/ops/rpu_linear.cpp:1119-1209 (bias, activation, residual add).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <algorithm>
#include <cstdlib>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kSmThreads = 256;
constexpr int kSmBN = 64;         // output features per CTA
constexpr int kSmBK = 64;         // K per stage
constexpr int kSmPartLd = kSmBN + 4;   // fp32 row pitch of the split-K partial (68 words: conflict-free column pairs)

struct SmallParams {
  const void* x; int64_t ldx;
  const void* w; int64_t ldw;
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias;
  const void* scale;          // optional per-output-column factor, applied before the bias (16-bit weights only)
  int M, N, K, act, dual_offset, packed, kb_total, dual_tiles, splits;
};

__device__ __forceinline__ void sm_cp16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void sm_ldsm4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void sm_mma(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void sm_mma<__half>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void sm_mma<__nv_bfloat16>(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// BM: token rows per CTA.  Eight warps: 128 rows = 4 row groups x 2 feature halves, 64 rows = 2 row groups x 4 feature
// quarters.  STAGES: depth of the cp.async ring; a CTA's whole K range is usually in flight at once (what bounds these
// GEMMs is one memory round trip).
template <typename T, int BM, bool DUAL, int STAGES>
__global__ void __launch_bounds__(kSmThreads)
gemm_small_kernel(const SmallParams p) {
  pdl_launch_dependents();                              // the dependency wait comes after the weight prefetch below
  constexpr int kSmStages = STAGES;
  constexpr int WM = BM / 32;                           // warps along the token axis
  constexpr int WN = (kSmThreads / 32) / WM;            // warps along the feature axis
  constexpr int NT = kSmBN / WN / 8;                    // 8-feature tiles per warp
  constexpr int kWT = DUAL ? 2 : 1;
  constexpr int kXBytes = BM * 128, kWBytes = kSmBN * 128;
  constexpr int kStage = kXBytes + kWT * kWBytes;
  constexpr int kXIter = BM * 8 / kSmThreads, kWIter = kSmBN * 8 / kSmThreads;   // 16-byte pieces per thread and tile
  extern __shared__ __align__(128) uint8_t ssm[];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
  const int wm = warp % WM, wn = warp / WM;
  const int f0 = blockIdx.x * kSmBN, m0 = blockIdx.y * BM, z = blockIdx.z;
  const int kb_all = (p.K + kSmBK - 1) / kSmBK;
  const int kb_base = kb_all / p.splits, kb_rem = kb_all % p.splits;
  const int kb0 = z * kb_base + min(z, kb_rem), kb_cnt = kb_base + (z < kb_rem ? 1 : 0);
  const T* X = reinterpret_cast<const T*>(p.x);
  const T* W = reinterpret_cast<const T*>(p.w);

  // this thread's pieces of a tile: rows lr + j * (threads / 8), 16-byte chunk lc; the swizzled chunk does not depend on j
  const int lr = tid >> 3, lc = tid & 7;
  const uint32_t l_off = (uint32_t)(lr * 128 + ((lc ^ (lr & 7)) << 4));
  const T* x_src = X + (size_t)(m0 + lr) * p.ldx + lc * 8;
  const size_t x_step = (size_t)(kSmThreads / 8) * p.ldx;
  const uint8_t* wp_src[kWT];
  const T* wu_src[kWT];
#pragma unroll
  for (int wt = 0; wt < kWT; ++wt) {
    const int ft = blockIdx.x + wt * 2 * p.dual_tiles;               // 64-row feature tile index in the tile-major image
    wp_src[wt] = reinterpret_cast<const uint8_t*>(W) + ((size_t)(ft >> 1) * p.kb_total) * 16384 + (ft & 1) * 8192 + tid * 16;
    wu_src[wt] = W + (size_t)(f0 + wt * p.dual_offset + lr) * p.ldw + lc * 8;
  }
  const size_t w_step = (size_t)(kSmThreads / 8) * p.ldw;

  // the two halves of a stage: the token tile depends on the previous kernel, the weight tile does not
  auto load_x = [&](int i, int s) {
    uint8_t* st = ssm + s * kStage;
    const int kc = (kb0 + i) * kSmBK;
    const bool kok = kc + lc * 8 < p.K;
#pragma unroll
    for (int j = 0; j < kXIter; ++j) {
      const bool ok = kok && (m0 + lr + j * (kSmThreads / 8) < p.M);
      sm_cp16(st + l_off + j * (kSmThreads / 8) * 128, ok ? x_src + j * x_step + kc : X, ok);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  auto load_w = [&](int i, int s) {
    uint8_t* st = ssm + s * kStage;
    const int kc = (kb0 + i) * kSmBK;
    const bool kok = kc + lc * 8 < p.K;
#pragma unroll
    for (int wt = 0; wt < kWT; ++wt) {
      uint8_t* dst = st + kXBytes + wt * kWBytes;
      if (p.packed) {
        // 64 rows of a 128 x 64 block of the tile-major image: 8 KB, already in the swizzled order
        const uint8_t* src = wp_src[wt] + (size_t)(kb0 + i) * 16384;
#pragma unroll
        for (int j = 0; j < kWIter; ++j) sm_cp16(dst + tid * 16 + j * kSmThreads * 16, src + j * kSmThreads * 16, true);
      } else {
#pragma unroll
        for (int j = 0; j < kWIter; ++j) {
          const bool ok = kok && (f0 + lr + j * (kSmThreads / 8) < p.N);
          sm_cp16(dst + l_off + j * (kSmThreads / 8) * 128, ok ? wu_src[wt] + j * w_step + kc : W, ok);
        }
      }
    }
  };

  float acc[kWT][2][NT][4];
#pragma unroll
  for (int a = 0; a < kWT; ++a)
#pragma unroll
    for (int b = 0; b < 2; ++b)
#pragma unroll
      for (int c = 0; c < NT; ++c)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[a][b][c][e] = 0.f;

  // fragment addresses: row offset and the XOR term of the swizzle are fixed per thread; the k step only flips chunk bits
  uint32_t a_row[2], a_x[2], b_row[NT / 2 > 0 ? NT / 2 : 1], b_x[NT / 2 > 0 ? NT / 2 : 1];
#pragma unroll
  for (int mt = 0; mt < 2; ++mt) {
    const int r = wm * 32 + mt * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
    a_row[mt] = (uint32_t)r * 128;
    a_x[mt] = (uint32_t)((lane >> 4) ^ (r & 7));
  }
#pragma unroll
  for (int np = 0; np < NT / 2; ++np) {
    const int r = wn * (kSmBN / WN) + np * 16 + (lane & 7) + (lane >> 4) * 8;
    b_row[np] = (uint32_t)r * 128;
    b_x[np] = (uint32_t)(((lane >> 3) & 1) ^ (r & 7));
  }

  // ---- main loop: a ring of cp.async groups (empty groups keep the count uniform)
  for (int i = 0; i < kSmStages - 1; ++i)
    if (i < kb_cnt) load_w(i, i);                       // weights first: they stream while the previous kernel finishes
  pdl_wait();
  for (int i = 0; i < kSmStages - 1; ++i) {
    if (i < kb_cnt) load_x(i, i);                       // commits the group of stage i (the first one also carries every weight tile above)
    else asm volatile("cp.async.commit_group;" ::: "memory");
  }
  const uint32_t ring = smem_u32(ssm);
  for (int i = 0; i < kb_cnt; ++i) {
    asm volatile("cp.async.wait_group %0;" ::"n"(kSmStages - 2) : "memory");
    __syncthreads();
    if (i + kSmStages - 1 < kb_cnt) {
      load_w(i + kSmStages - 1, (i + kSmStages - 1) % kSmStages);
      load_x(i + kSmStages - 1, (i + kSmStages - 1) % kSmStages);
    } else {
      asm volatile("cp.async.commit_group;" ::: "memory");
    }
    const uint32_t sx = ring + (uint32_t)((i % kSmStages) * kStage), sw = sx + kXBytes;
#pragma unroll
    for (int ks = 0; ks < kSmBK / 16; ++ks) {
      uint32_t a[2][4];
#pragma unroll
      for (int mt = 0; mt < 2; ++mt) sm_ldsm4(a[mt], sx + a_row[mt] + (((uint32_t)(2 * ks) ^ a_x[mt]) << 4));
#pragma unroll
      for (int wt = 0; wt < kWT; ++wt)
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
          uint32_t b[4];
          sm_ldsm4(b, sw + wt * kWBytes + b_row[np] + (((uint32_t)(2 * ks) ^ b_x[np]) << 4));
#pragma unroll
          for (int mt = 0; mt < 2; ++mt) {
            sm_mma<T>(acc[wt][mt][np * 2], a[mt], b[0], b[1]);
            sm_mma<T>(acc[wt][mt][np * 2 + 1], a[mt], b[2], b[3]);
          }
        }
    }
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");

  const T* bias = reinterpret_cast<const T*>(p.bias);
  const T* scale = reinterpret_cast<const T*>(p.scale);
  const T* res = reinterpret_cast<const T*>(p.residual);
  T* out = reinterpret_cast<T*>(p.out);
  auto finish_pair = [&](int m, int n, float g0, float g1, float u0, float u1) {
    // features n and n + 1 of token row m (n is even; N is a multiple of 8)
    if (m >= p.M || n >= p.N) return;
    if (scale) {
      g0 *= Num<T>::to_f(scale[n]);
      g1 *= Num<T>::to_f(scale[n + 1]);
      if (DUAL) {
        u0 *= Num<T>::to_f(scale[p.dual_offset + n]);
        u1 *= Num<T>::to_f(scale[p.dual_offset + n + 1]);
      }
    }
    if (bias) {
      g0 += Num<T>::to_f(bias[n]);
      g1 += Num<T>::to_f(bias[n + 1]);
      if (DUAL) {
        u0 += Num<T>::to_f(bias[p.dual_offset + n]);
        u1 += Num<T>::to_f(bias[p.dual_offset + n + 1]);
      }
    }
    float v0 = apply_act(p.act, g0, u0), v1 = apply_act(p.act, g1, u1);
    if (res) {
      v0 += Num<T>::to_f(res[(size_t)m * p.ldr + n]);
      v1 += Num<T>::to_f(res[(size_t)m * p.ldr + n + 1]);
    }
    T pair[2] = {Num<T>::from_f(v0), Num<T>::from_f(v1)};
    *reinterpret_cast<uint32_t*>(out + (size_t)m * p.ldo + n) = *reinterpret_cast<const uint32_t*>(pair);
  };

  if (p.splits == 1) {
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int m = m0 + wm * 32 + mt * 16 + g + h * 8, n = f0 + wn * (kSmBN / WN) + nt * 8 + 2 * t;
          finish_pair(m, n, acc[0][mt][nt][2 * h], acc[0][mt][nt][2 * h + 1], DUAL ? acc[kWT - 1][mt][nt][2 * h] : 0.f,
                      DUAL ? acc[kWT - 1][mt][nt][2 * h + 1] : 0.f);
        }
    return;
  }

  // ---- split K: park the partial tile(s) in shared memory, sum over the cluster, each CTA finishing BM / splits rows
  __syncthreads();                                            // the ring is no longer read
  float* part = reinterpret_cast<float*>(ssm);                // [kWT][BM][kSmPartLd]
#pragma unroll
  for (int wt = 0; wt < kWT; ++wt)
#pragma unroll
    for (int mt = 0; mt < 2; ++mt)
#pragma unroll
      for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = wm * 32 + mt * 16 + g + h * 8, c = wn * (kSmBN / WN) + nt * 8 + 2 * t;
          *reinterpret_cast<float2*>(part + ((size_t)wt * BM + r) * kSmPartLd + c) =
              make_float2(acc[wt][mt][nt][2 * h], acc[wt][mt][nt][2 * h + 1]);
        }
  cluster_sync_all();
  {
    const int rows = BM / p.splits;                           // splits is 2, 4 or 8
    const int r_lo = (int)cluster_ctarank() * rows;
    const uint32_t base = smem_u32(part);
    for (int idx = tid; idx < rows * (kSmBN / 2); idx += kSmThreads) {
      const int r = r_lo + idx / (kSmBN / 2), c = (idx % (kSmBN / 2)) * 2;
      // every CTA's pair in flight before the first add (a loop over a run-time split count would chain the
      // distributed-shared-memory round trips one behind the other)
      float2 v[kWT][8];
#pragma unroll
      for (int k = 0; k < 8; ++k)
#pragma unroll
        for (int wt = 0; wt < kWT; ++wt)
          v[wt][k] = k < p.splits
                         ? ld_dsmem_f32x2(dsmem_addr(base + (uint32_t)((((size_t)wt * BM + r) * kSmPartLd + c) * sizeof(float)), (uint32_t)k))
                         : make_float2(0.f, 0.f);
      float s[kWT][2];
#pragma unroll
      for (int wt = 0; wt < kWT; ++wt) {
        s[wt][0] = s[wt][1] = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) { s[wt][0] += v[wt][k].x; s[wt][1] += v[wt][k].y; }
      }
      finish_pair(m0 + r, f0 + c, s[0][0], s[0][1], DUAL ? s[kWT - 1][0] : 0.f, DUAL ? s[kWT - 1][1] : 0.f);
    }
  }
  cluster_sync_relaxed();                                     // peers may still be reading this CTA's partial
}

template <int BM, bool DUAL, int STAGES>
constexpr size_t small_smem() {
  constexpr size_t ring = (size_t)STAGES * (BM * 128 + (DUAL ? 2 : 1) * kSmBN * 128);
  constexpr size_t part = (size_t)(DUAL ? 2 : 1) * BM * kSmPartLd * sizeof(float);
  return ring > part ? ring : part;
}

static bool small_enabled() {
  static const bool v = [] { const char* e = getenv("RF_GEMM_SMALL"); return !(e && e[0] == '0'); }();
  return v;
}

// Shapes this kernel takes over from the streaming kernel: few token rows, a weight that an SM-count's worth of CTAs
// finishes in one short wave, and only the plain epilogue options.
bool gemm_small_eligible(const RfGemm* g) {
  if (!small_enabled() || g->w_int8 || g->w_bits || g->row_scale || g->ar_world > 1 || g->ar_publish || g->ss_in || g->ss_out ||
      g->prefetch || g->force_splits || g->force_bn || g->force_swap >= 0 || g->streaming_only)
    return false;
  // Up to 256 rows the weight-size cap below decides.  Up to RF_GEMM_SMALL_MAX_ROWS rows (default 2048) only weights of at
  // most 1 Mi elements qualify: such GEMMs (ViT-S towers: ~1 000 patch rows, 384-wide) are still bound by launch and
  // set-up cost, not by tensor throughput (RGB-D encoder 4.07 -> 2.82 ms per call); with SigLIP-sized weights
  // (1152 x 1152 and up, 768 rows) the tcgen05 kernels win (Pi0.5 vision tower 4.4 ms against 6.2 ms here).
  static const int max_rows = [] { const char* e = getenv("RF_GEMM_SMALL_MAX_ROWS"); return e ? atoi(e) : 2048; }();
  if (g->M > 256 && (g->M > max_rows || (long)g->N * g->K * (g->dual_offset > 0 ? 2 : 1) > (1L << 20))) return false;
  if (g->N % 8 || g->K % 8 || g->ldx % 8 || g->ldo % 2 || (g->residual && g->ldr % 2)) return false;
  if (!g->w_packed && g->ldw % 8) return false;
  const bool dual = g->dual_offset > 0;
  if (dual && !g->w_packed && g->dual_offset % 8) return false;
  // up to 64 rows the two kernels are close once K is long (41 x 1536 x 6144: 12.0 us on the streaming kernel, 11.6 us
  // here; 50 x 1024 x 2048: 8.5 against 5.7; inside the Pi0.5 denoise loop, K = 2048 / 4096 at 50 rows: 24.8 ms per chunk with
  // this bound at 2048, 23.9 ms at 8192); above 64 rows this kernel wins everywhere that was measured
  // (128 x 1536 x 384: 5.6 us against 19.6 us)
  static const int max_k64 = [] { const char* e = getenv("RF_GEMM_SMALL_MAX_K"); return e ? atoi(e) : 8192; }();
  if (g->M <= 64 && g->K > max_k64) return false;
  // up to 32 rows the streaming kernel runs 32-column tiles; it won on all but the smallest weights before the split-K
  // reduction here had its loads batched (31 x 2560 x 1024: 6.8 us there against 9.2 us here), and loses since then
  // inside the loops that matter (RhinoVLA expert, 31 rows: 12.6 ms per call with this bound at 1 Mi elements, 11.9 ms
  // without it), so the bound now sits above the kernel's general weight cap
  static const long max_elems32 = [] { const char* e = getenv("RF_GEMM_SMALL_ROWS32_MAX_KELEMS"); return (long)(e ? atoi(e) : 16384) << 10; }();
  if (g->M <= 32 && (long)g->N * g->K * (dual ? 2 : 1) > max_elems32) return false;
  static const long max_elems = [] { const char* e = getenv("RF_GEMM_SMALL_MAX_MELEMS"); return (long)(e ? atoi(e) : 12) << 20; }();
  return (long)g->N * g->K * (dual ? 2 : 1) <= max_elems;
}

template <typename T, int BM, bool DUAL, int STAGES>
static int launch_small_st(const SmallParams& p, dim3 grid, cudaStream_t s) {
  constexpr size_t smem = small_smem<BM, DUAL, STAGES>();
  RF_ALLOW_SMEM_PER_DEVICE((gemm_small_kernel<T, BM, DUAL, STAGES>), smem);
  RF_CUDA_CHECK(::rf::launch_k(gemm_small_kernel<T, BM, DUAL, STAGES>, grid, dim3(kSmThreads), smem, s, p.splits, p));
  ::rf::count_launch();
  return RF_OK;
}

// Ring depth: a CTA's k blocks are all in flight when they fit: 4 stages, or the deep ring (64-row tiles: 6 stages, 96 KB,
// two CTAs per SM; 128-row tiles: 8 stages, 192 KB) when the CTA has more than 4 blocks.
template <typename T, int BM, bool DUAL>
static int launch_small(const SmallParams& p, dim3 grid, cudaStream_t s) {
  const int kb_cnt = (p.kb_total + p.splits - 1) / p.splits;
  constexpr int kDeep = BM == 64 ? (DUAL ? 4 : 6) : (DUAL ? 4 : 8);
  if constexpr (kDeep > 4) {
    if (kb_cnt > 4) return launch_small_st<T, BM, DUAL, kDeep>(p, grid, s);
  }
  return launch_small_st<T, BM, DUAL, 4>(p, grid, s);
}

int gemm_small_run(const RfGemm* g, cudaStream_t s) {
  const bool dual = g->dual_offset > 0;
  SmallParams p;
  p.x = g->x; p.ldx = g->ldx; p.w = g->w; p.ldw = g->ldw; p.out = g->out; p.ldo = g->ldo;
  p.residual = g->residual; p.ldr = g->ldr; p.bias = g->bias; p.scale = g->scale;
  p.M = g->M; p.N = g->N; p.K = g->K; p.act = g->act; p.dual_offset = g->dual_offset; p.packed = g->w_packed ? 1 : 0;
  p.kb_total = (g->K + 63) / 64;
  p.dual_tiles = dual ? (g->dual_offset + 127) / 128 : 0;    // the up section starts this many 128-row tiles after the gate section
  const int bm = g->M > 64 ? 128 : 64;
  const int tiles = ((g->N + kSmBN - 1) / kSmBN) * ((g->M + bm - 1) / bm);
  // split K until about two SMs' worth... of CTAs exist or a CTA is down to a few k blocks (then its whole K range is
  // one burst of loads); never below one block per CTA
  int splits = 1;
  while (splits < 8 && tiles * splits * 2 <= 2 * sm_count() && p.kb_total >= splits * 2 && (p.kb_total + splits - 1) / splits > 2)
    splits *= 2;
  p.splits = splits;
  const dim3 grid((g->N + kSmBN - 1) / kSmBN, (g->M + bm - 1) / bm, splits);
#define RF_SMALL(T)                                                                    \
  do {                                                                                 \
    if (bm == 128) return dual ? launch_small<T, 128, true>(p, grid, s) : launch_small<T, 128, false>(p, grid, s); \
    return dual ? launch_small<T, 64, true>(p, grid, s) : launch_small<T, 64, false>(p, grid, s);                  \
  } while (0)
  if (g->dtype == 0) RF_SMALL(__half);
  RF_SMALL(__nv_bfloat16);
#undef RF_SMALL
}

}  // namespace rf
