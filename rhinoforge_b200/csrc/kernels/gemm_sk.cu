// Persistent stream-K tcgen05 GEMM for weight-streaming shapes (at most 256 tokens: decode steps, small
// prefills, action chunks):  out[M,N] = epilogue( x[M,K] . w[N,K]^T ).
//
// A decode GEMM is a pass over the weight matrix; it is as fast as the weight bytes can be kept in flight from
// every SM for the whole duration of the kernel.  One-tile CTAs (gemm_tc.cu) cannot do that: 96 output tiles on
// 148 SMs leave a third of the machine idle, 192 half-tiles make some SMs stream twice as much as others, and
// every CTA pays barrier set-up, tensor-memory allocation and the first DRAM round trip before it streams.
//
// Here the work is the flat list of (128-row weight tile, 64-column k block) units; one CTA per SM takes an equal
// contiguous share of it and streams that share through one operand ring that never drains between tiles:
//   warp 0      producer: weight blocks (tile-major image) by bulk copy, activation tiles by tensor map;
//   warp 1      MMA issuer: weights on the 128-wide MMA M axis, tokens on the N axis, fp32 accumulators in tensor
//               memory, two accumulator buffers so the epilogue of one tile segment runs under the next one's MMAs;
//   warps 2-5   epilogue: one thread per output feature.
// A CTA's share starts and ends anywhere inside a tile, so a tile's k range may be split over two or three
// neighbouring CTAs ("segments").  The CTA that holds the segment starting at k = 0 finishes the tile; the others
// park their fp32 partial in global scratch (slot = CTA index) and raise a flag.  Because shares are contiguous,
// a CTA parks only the FIRST segment of its share -- at the very start of the kernel -- and finishes only at the
// END of its share, so the finisher practically never waits, nothing waits in a cycle, and partials are added in
// segment order (deterministic).  The waits are bounded like every other wait in this library.
//
// The epilogue parks a finished tile as rows [token][128 features] in shared memory and writes it out (or, under
// tensor parallelism, pushes it into every rank's receive buffer -- the "publish" half of the all-reduce whose
// other half is rf_ar_consume) as 16-byte vectors.
//
// Replaces the reference's parallel_linear_* tile family at small M, llama_gemv and the ring-buffered K pipeline
// of src/ops/rpu_linear_gemv.cpp:1-275 (src/ops/rpu_linear.cpp:1047-1544, src/fused/rpu_qwen3_model.h:3653-3700).
#include <algorithm>
#include <atomic>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kSkBM = 128, kSkBK = 64;
constexpr int kSkWBlock = kSkBM * kSkBK * 2;    // one packed 16-bit weight block: 16 KB
constexpr int kSkMaxStages = 12;
constexpr int kSkThreads = 192;
constexpr int kSkEpiThreads = 128;
constexpr int kSkMaxPartners = 8;               // CTAs that may hold the rest of a finisher's tile

struct GemmSkParams {
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias; const void* scale; const float* row_scale;
  const uint8_t* w_packed;
  float* ws; uint32_t* flags; int32_t* status;
  int M, N, k_blocks, bn, stages, act, dual_offset, dual_tiles, tiles;
  long long units;
  int stage_off;             // shared-memory offset of the [token][128] staging rows
  int ctl_off;
  int tmem_cols;             // tensor-memory columns this CTA allocates (a power of two covering its accumulator buffers)
  // tensor-parallel publish (see gemm_tc.cu / ar_consume.cu)
  int ar_world, ar_rank, ar_publish, ar_cnt_base;
  int w_evict_first;       // weights are read with the L2 evict-first policy (streamed once)
  void* const* ar_recv; uint32_t* const* ar_flags; uint32_t* ar_state; uint64_t ar_half_bytes;
};

struct alignas(8) GemmSkCtl {
  uint64_t full[kSkMaxStages], empty[kSkMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int32_t abort_flag;
  int32_t partner_bad;
  int32_t partner_count;
};

__device__ __forceinline__ void st_release_gpu(uint32_t* p, uint32_t v) {
  asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void epi_bar_sync() {   // the four epilogue warps only (named barrier 1)
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

// The share of CTA c: units [c * U / P, (c + 1) * U / P)
__device__ __forceinline__ long long sk_share_begin(long long units, int ctas, int c) {
  return units * c / ctas;
}
__device__ __forceinline__ long long sk_min(long long a, long long b) { return a < b ? a : b; }

template <typename T, bool DUAL>
__global__ void __launch_bounds__(kSkThreads)
gemm_sk_kernel(const __grid_constant__ CUtensorMap tmX, const GemmSkParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bn = p.bn, KB = p.k_blocks;
  constexpr int kW = DUAL ? 2 : 1;
  const int x_bytes = bn * kSkBK * 2;
  const int stage_bytes = kW * kSkWBlock + x_bytes;
  const int acc_cols = kW * bn;
  const int nbuf = 2 * acc_cols <= 512 ? 2 : 1;
  GemmSkCtl* ctl = reinterpret_cast<GemmSkCtl*>(smem + p.ctl_off);
  const int cta = blockIdx.x, ctas = gridDim.x;
  const long long u_begin = sk_share_begin(p.units, ctas, cta), u_end = sk_share_begin(p.units, ctas, cta + 1);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl->acc_full[b], 1);
      mbar_init(&ctl->acc_empty[b], 4);
    }
    ctl->abort_flag = 0;
    ctl->partner_bad = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmX);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  pdl_launch_dependents();         // after this CTA owns its tensor-memory columns
  volatile int32_t* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer ----
    if (lane == 0) {
      auto load_w = [&](long long u, int s) {
        const int t = (int)(u / KB), kb = (int)(u - (long long)t * KB);
        uint8_t* st = smem + (size_t)s * stage_bytes;
#pragma unroll
        for (int wt = 0; wt < kW; ++wt)
          if (p.w_evict_first)
            bulk_load_1d_hint(st + wt * kSkWBlock, p.w_packed + ((size_t)(t + wt * p.dual_tiles) * KB + kb) * kSkWBlock,
                              kSkWBlock, &ctl->full[s], l2_policy_evict_first());
          else
            bulk_load_1d(st + wt * kSkWBlock, p.w_packed + ((size_t)(t + wt * p.dual_tiles) * KB + kb) * kSkWBlock, kSkWBlock,
                         &ctl->full[s]);
      };
      auto load_x = [&](long long u, int s) {
        const int kb = (int)(u % KB);
        tma_load_2d(smem + (size_t)s * stage_bytes + kW * kSkWBlock, &tmX, &ctl->full[s], kb * kSkBK, 0);
      };
      // weights never depend on the previous kernel: the first ring fill starts before the dependency wait
      const long long total = u_end - u_begin;
      const int pre = (int)sk_min(p.stages, total);
      for (int i = 0; i < pre; ++i) {
        mbar_arrive_expect_tx(&ctl->full[i], (uint32_t)stage_bytes);
        load_w(u_begin + i, i);
      }
      pdl_wait();
      for (int i = 0; i < pre; ++i) load_x(u_begin + i, i);
      bool ok = true;
      long long issued = pre;
      for (long long i = pre; i < total; ++i) {
        const int s = (int)(i % p.stages);
        if (!mbar_wait(&ctl->empty[s], (((uint32_t)(i / p.stages)) & 1u) ^ 1u, kLocalWaitNs, 32) || *abort_flag) {
          if (!*abort_flag) report_status(p.status, kStatusTmaTimeout, kTagGemmTc, (int)i);
          ok = false;
          break;
        }
        mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)stage_bytes);
        load_w(u_begin + i, s);
        load_x(u_begin + i, s);
        issued = i + 1;
      }
      if (!ok) {
        ctl->abort_flag = 1;
        const long long first = issued > p.stages ? issued - p.stages : 0;
        for (long long i = first; i < issued; ++i)
          mbar_wait(&ctl->full[i % p.stages], (uint32_t)(i / p.stages) & 1u, 20ull * 1000 * 1000);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer ----
    pdl_wait();
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(kSkBM, bn, Num<T>::kFmt);
      long long it = 0;
      int seg = 0;
      bool ok = true;
      for (long long u = u_begin; ok && u < u_end; ++seg) {
        const int t = (int)(u / KB);
        const long long seg_end = sk_min(u_end, (long long)(t + 1) * KB);
        const int b = seg % nbuf;
        if (!mbar_wait(&ctl->acc_empty[b], (((uint32_t)(seg / nbuf)) & 1u) ^ 1u, kLocalWaitNs, 32)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(b * acc_cols);
        bool first_mma = true;
        for (; u < seg_end; ++u, ++it) {
          const int s = (int)(it % p.stages);
          if (!mbar_wait(&ctl->full[s], (uint32_t)(it / p.stages) & 1u, kLocalWaitNs, 0)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t w_addr = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t x_addr = w_addr + kW * kSkWBlock;
#pragma unroll
          for (int k = 0; k < kSkBK / 16; ++k) {
            const uint32_t accum = (first_mma && k == 0) ? 0u : 1u;
            const uint64_t dx = umma_desc_k128(x_addr + k * 32);
            umma_f16(acc, umma_desc_k128(w_addr + k * 32), dx, idesc, accum);
            if (DUAL) umma_f16(acc + bn, umma_desc_k128(w_addr + kSkWBlock + k * 32), dx, idesc, accum);
          }
          first_mma = false;
          umma_commit(&ctl->empty[s]);
        }
        if (ok) umma_commit(&ctl->acc_full[b]);
      }
      if (!ok) {
        if (!*abort_flag) report_status(p.status, kStatusMmaTimeout, kTagGemmTc, (int)it);
        ctl->abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue ----
    pdl_wait();
    const int quarter = warp & 3;                          // the tensor-memory lanes this warp may read
    const int r = quarter * 32 + lane;                     // feature row of this thread inside a tile
    const int et = tid - 64;                               // 0..127 among the epilogue threads
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* scale = reinterpret_cast<const T*>(p.scale);
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    const int M = p.M, N = p.N;
    const bool pub = p.ar_world > 1 && p.ar_publish;
    const bool pub_f32 = pub && M <= RF_AR_F32_MAX_ROWS;
    const bool use_bias = bias != nullptr && (p.ar_world <= 1 || p.ar_rank == 0);
    const bool affine = p.row_scale || scale || use_bias;
    uint8_t* stage = smem + p.stage_off;
    const size_t slot_floats = (size_t)acc_cols * kSkBM;
    uint8_t* peer_buf[8];
    {
      const uint32_t call = pub ? *reinterpret_cast<volatile uint32_t*>(p.ar_state) : 0u;
      const uint64_t slot_off = (uint64_t)(call & 1u) * p.ar_half_bytes;
#pragma unroll
      for (int d = 0; d < 8; ++d)
        peer_buf[d] = (pub && d < p.ar_world) ? reinterpret_cast<uint8_t*>(p.ar_recv[d]) + slot_off : nullptr;
    }
    int seg = 0;
    bool dead = false;
    for (long long u = u_begin; u < u_end && !dead; ++seg) {
      const int t = (int)(u / KB);
      const int k0 = (int)(u - (long long)t * KB);
      const long long seg_end = sk_min(u_end, (long long)(t + 1) * KB);
      const int k1 = (int)(seg_end - (long long)t * KB);
      u = seg_end;
      const int b = seg % nbuf;
      if (!mbar_wait(&ctl->acc_full[b], (uint32_t)(seg / nbuf) & 1u)) {
        if (!*abort_flag) report_status(p.status, kStatusEpilogueTimeout, kTagGemmTc, t);
        ctl->abort_flag = 1;
      }
      // one decision for all four warps: the named barriers below need every epilogue thread or none
      epi_bar_sync();
      if (*abort_flag) {
        dead = true;
        break;
      }
      tc_fence_after_sync();
      const uint32_t acc = lane_base + (uint32_t)(b * acc_cols);
      if (k0 != 0) {
        // ---- not the finisher of this tile: park the fp32 partial in this CTA's scratch slot, raise the flag
        float* slot = p.ws + (size_t)cta * slot_floats;
        for (int c = 0; c < acc_cols; c += 16) {
          uint32_t rg[16];
          tmem_ld16(acc + c, rg);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) slot[(size_t)(c + j) * kSkBM + r] = __uint_as_float(rg[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
        __threadfence();
        epi_bar_sync();
        if (et == 0) st_release_gpu(p.flags + cta, 1u);
        continue;
      }
      // ---- finisher: the rest of the tile's k range (if any) sits in the slots of the following CTAs
      int partners = 0;
      if (k1 < KB) {
        if (et == 0) {
          int cov = k1, j = cta + 1, n = 0;
          while (cov < KB && j < ctas && n < kSkMaxPartners) {
            if (!wait_flag_ge_sys(p.flags + j, 1u, kLocalWaitNs)) {   // flags are 0 or 1; a device-scope acquire load suffices, the helper's is stronger
              report_status(p.status, kStatusSplitKTimeout, kTagGemmTc, j);
              ctl->partner_bad = 1;
              break;
            }
            const long long uj1 = sk_share_begin(p.units, ctas, j + 1);
            cov = (int)sk_min(KB, uj1 - (long long)t * KB);
            ++j; ++n;
          }
          if (cov < KB && !ctl->partner_bad) {
            report_status(p.status, kStatusBadArgument, kTagGemmTc, t);
            ctl->partner_bad = 1;
          }
          ctl->partner_count = n;
        }
        epi_bar_sync();
        partners = *reinterpret_cast<volatile int32_t*>(&ctl->partner_count);
        if (*reinterpret_cast<volatile int32_t*>(&ctl->partner_bad)) { dead = true; ctl->abort_flag = 1; }
      }
      const int n_feat = t * kSkBM + r;                    // output feature of this thread
      if (!dead) {
        for (int c = 0; c < bn; c += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld16(acc + c, rg);
          if (DUAL) tmem_ld16(acc + bn + c, ru);
          tmem_ld_wait();
          float g[16], uu[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            g[j] = __uint_as_float(rg[j]);
            uu[j] = DUAL ? __uint_as_float(ru[j]) : 0.f;
          }
          for (int q = 0; q < partners; ++q) {             // segment order: deterministic sum
            const float* slot = p.ws + (size_t)(cta + 1 + q) * slot_floats;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              g[j] += __ldcg(slot + (size_t)(c + j) * kSkBM + r);
              if (DUAL) uu[j] += __ldcg(slot + (size_t)(bn + c + j) * kSkBM + r);
            }
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = c + j;
            float vg = g[j], vu = uu[j], v = 0.f;
            if (tok < M && n_feat < N) {
              if (affine) {
                if (p.row_scale) { const float rs = p.row_scale[tok]; vg *= rs; vu *= rs; }
                if (scale) { vg *= Num<T>::to_f(scale[n_feat]); if (DUAL) vu *= Num<T>::to_f(scale[p.dual_offset + n_feat]); }
                if (use_bias) { vg += Num<T>::to_f(bias[n_feat]); if (DUAL) vu += Num<T>::to_f(bias[p.dual_offset + n_feat]); }
              }
              v = apply_act(p.act, vg, vu);
              if (resid && !pub) v += Num<T>::to_f(resid[(size_t)tok * p.ldr + n_feat]);
            }
            if (pub_f32) reinterpret_cast<float*>(stage)[tok * kSkBM + r] = v;
            else reinterpret_cast<T*>(stage)[tok * kSkBM + r] = Num<T>::from_f(v);
          }
        }
      }
      // the accumulator buffer is free for a later segment
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
      epi_bar_sync();                                      // the staged rows are complete
      if (!dead) {
        if (et < partners) p.flags[cta + 1 + et] = 0u;     // consumed: ready for the next launch on this scratch
        const int rows = min(bn, M);
        const int nfeat = min(kSkBM, N - t * kSkBM);        // valid features of this tile
        if (pub) {
          const int vpr = pub_f32 ? 32 : 16, epv = pub_f32 ? 4 : 8, esz = pub_f32 ? 4 : 2;
          for (int idx = et; idx < rows * vpr; idx += kSkEpiThreads) {
            const int tok = idx / vpr, ch = idx - tok * vpr;
            if (ch * epv >= nfeat) continue;
            const uint4 val = *reinterpret_cast<const uint4*>(stage + ((size_t)tok * kSkBM * esz) + ch * 16);
            const size_t off = (((size_t)p.ar_rank * M + tok) * N + (size_t)t * kSkBM) * esz + (size_t)ch * 16;
#pragma unroll
            for (int d = 0; d < 8; ++d)
              if (d < p.ar_world) *reinterpret_cast<uint4*>(peer_buf[d] + off) = val;
          }
        } else if ((N & 7) == 0 && (p.ldo & 7) == 0) {
          for (int idx = et; idx < rows * 16; idx += kSkEpiThreads) {
            const int tok = idx >> 4, ch = idx & 15;
            if (ch * 8 >= nfeat) continue;
            *reinterpret_cast<uint4*>(out + (size_t)tok * p.ldo + (size_t)t * kSkBM + ch * 8) =
                *reinterpret_cast<const uint4*>(stage + ((size_t)tok * kSkBM * 2) + ch * 16);
          }
        } else {
          for (int idx = et; idx < rows * kSkBM; idx += kSkEpiThreads) {
            const int tok = idx >> 7, f = idx & 127;
            if (f < nfeat) out[(size_t)tok * p.ldo + (size_t)t * kSkBM + f] = reinterpret_cast<const T*>(stage)[tok * kSkBM + f];
          }
        }
      }
      epi_bar_sync();                                      // the staging rows may be overwritten
    }
    if (pub) {
      // every remote row of this CTA is visible system-wide before its arrival is counted
      __threadfence_system();
      epi_bar_sync();
      if (et < p.ar_world && !dead && !*abort_flag) red_release_sys_add(p.ar_flags[et] + p.ar_cnt_base + p.ar_rank, 1u);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// ------------------------------------------------------------------ host side ----
struct SkPlan {
  int bn, stages, ctas, stage_off, ctl_off, tiles, k_blocks, tmem_cols;
  long long units;
  size_t smem;
  uint64_t ws_bytes;
};

// 0: never; 1 (default): shapes with at least four output tiles per SM, where almost every tile is streamed whole by
// one CTA and the partial-tile fix-up is noise (measured on B200 at 64 tokens: the 151936-row vocabulary projection
// 244 -> 203 us, 0.97 of the copy bandwidth; with fewer tiles than SMs - 32 to 96 for the projections of a decoder
// layer - every tile is cut into 4 to 8 pieces, the fix-up through global memory is a serial tail, and the cluster
// split-K kernel of gemm_tc.cu with its on-chip reduction is 1.1x to 1.9x faster); 2: every shape that fits (tests).
static std::atomic<int> g_sk_mode{-1};
static int sk_mode() {
  int m = g_sk_mode.load(std::memory_order_relaxed);
  if (m < 0) {
    const char* e = getenv("RF_GEMM_STREAMK");
    m = e ? atoi(e) : 1;
    if (m < 0 || m > 2) m = 1;
    g_sk_mode.store(m, std::memory_order_relaxed);
  }
  return m;
}

// Shapes the stream-K kernel takes: tokens on the MMA N axis (at most 256), tile-major 16-bit weights, enough
// (tile, k block) units that every CTA streams a few.
static bool sk_plan(const RfGemm* g, SkPlan* pl) {
  const int mode = sk_mode();
  if (mode == 0 || !g->w_packed || g->w_int8 || g->M > 256 || g->force_swap == 0 || g->force_splits > 0 || g->force_bn > 0)
    return false;
  if (mode == 1 && ceil_div(g->N, kSkBM) < 4 * sm_count()) return false;
  if (g->ar_world > 1 && !g->ar_publish) return false;     // the in-kernel all-reduce form stays with gemm_tc.cu
  if (g->ss_in || g->ss_out) return false;                 // folded RMSNorm lives in gemm_tc.cu's epilogue
  const bool dual = g->dual_offset > 0;
  const int bn = round_up(std::max(g->M, 16), 16);
  if ((dual ? 2 : 1) * bn > 512) return false;
  pl->bn = bn;
  pl->tiles = ceil_div(g->N, kSkBM);
  pl->k_blocks = ceil_div(g->K, kSkBK);
  pl->units = (long long)pl->tiles * pl->k_blocks;
  static const int min_units = [] { const char* e = getenv("RF_GEMM_STREAMK_MIN_UNITS"); return e ? atoi(e) : 2; }();
  if (pl->units < (long long)min_units * 16) return false;  // tiny GEMMs: set-up dominates either way
  // a tile's k range may spread over at most kSkMaxPartners + 1 shares: a share holds at least k_blocks / kSkMaxPartners units
  const long long per_cta = std::max<long long>(std::max(1, min_units), ceil_div(pl->k_blocks, kSkMaxPartners));
  // CTAs per SM: 2 (default) = two half-size rings with their own producer and MMA issuer, and a CTA of the next
  // kernel can move in as soon as one of them retires (vocabulary projection at 64 tokens: 203 us against 248 us
  // with one CTA per SM); 1 = the whole shared memory is one deep ring (RF_GEMM_STREAMK_PER_SM=1, A/B timing)
  static const int per_sm = [] { const char* e = getenv("RF_GEMM_STREAMK_PER_SM"); const int v = e ? atoi(e) : 2; return v == 1 ? 1 : 2; }();
  const int acc_cols = (dual ? 2 : 1) * bn;
  pl->tmem_cols = (int)next_pow2((uint32_t)std::max(32, (2 * acc_cols <= 512 ? 2 : 1) * acc_cols));
  const int ctas_per_sm = (per_sm == 2 && pl->tmem_cols <= 256) ? 2 : 1;
  pl->ctas = (int)std::min<long long>((long long)sm_count() * ctas_per_sm, std::max<long long>(1, pl->units / per_cta));
  if ((long long)pl->k_blocks > (long long)kSkMaxPartners * (pl->units / pl->ctas)) return false;
  const int stage_bytes = (dual ? 2 : 1) * kSkWBlock + bn * kSkBK * 2;
  const bool pub_f32 = g->ar_world > 1 && g->ar_publish && g->M <= RF_AR_F32_MAX_ROWS;
  const int staging = bn * kSkBM * (pub_f32 ? 4 : 2);
  const int ctl_bytes = (int)sizeof(GemmSkCtl) + 64;
  const int budget = (ctas_per_sm == 2 ? 113 : 227) * 1024 - 1024 /*alignment slack*/ - round_up(staging, 1024) - ctl_bytes;
  pl->stages = std::min(kSkMaxStages, budget / stage_bytes);
  if (pl->stages < 2) return false;
  pl->stage_off = round_up(pl->stages * stage_bytes, 1024);
  pl->ctl_off = pl->stage_off + round_up(staging, 1024);
  pl->smem = (size_t)pl->ctl_off + ctl_bytes + 1024;
  pl->ws_bytes = (uint64_t)pl->ctas * (dual ? 2 : 1) * bn * kSkBM * sizeof(float);
  return true;
}

// Scratch (bytes of fp32 partial slots, number of flags) a stream-K launch of this shape needs; 0 / 0 when the
// shape does not take this kernel.
void gemm_sk_scratch(const RfGemm* g, uint64_t* ws_bytes, int32_t* flags) {
  SkPlan pl;
  const bool yes = sk_plan(g, &pl);
  *ws_bytes = yes ? pl.ws_bytes : 0;
  *flags = yes ? pl.ctas : 0;
}

// True (and *ctas set) when rf_gemm will run this shape on the stream-K kernel with the scratch it was given.
bool gemm_sk_eligible(const RfGemm* g, int* ctas) {
  SkPlan pl;
  if (!sk_plan(g, &pl)) return false;
  if (!g->ws || !g->sem || g->ws_bytes < pl.ws_bytes || g->sem_count < pl.ctas) return false;
  if (ctas) *ctas = pl.ctas;
  return true;
}

template <typename T, bool DUAL>
static int launch_sk(const RfGemm* g, const SkPlan& pl, cudaStream_t stream) {
  auto kfn = gemm_sk_kernel<T, DUAL>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 227 * 1024);
  CUtensorMap tmX;
  int rc = make_tmap_2d(&tmX, g->x, g->dtype, 2, g->K, g->M, g->ldx, kSkBK, pl.bn, true);
  if (rc) return rc;
  GemmSkParams p = {};
  p.out = g->out; p.ldo = g->ldo; p.residual = g->residual; p.ldr = g->ldr;
  p.bias = g->bias; p.scale = g->scale; p.row_scale = g->row_scale;
  p.w_packed = reinterpret_cast<const uint8_t*>(g->w);
  p.ws = g->ws; p.flags = g->sem; p.status = g->status;
  p.M = g->M; p.N = g->N; p.k_blocks = pl.k_blocks; p.bn = pl.bn; p.stages = pl.stages; p.act = g->act;
  p.dual_offset = g->dual_offset; p.dual_tiles = pl.tiles; p.tiles = pl.tiles; p.units = pl.units;
  p.stage_off = pl.stage_off; p.ctl_off = pl.ctl_off; p.tmem_cols = pl.tmem_cols;
  p.ar_world = g->ar_world; p.ar_rank = g->ar_rank; p.ar_publish = g->ar_publish; p.ar_cnt_base = g->ar_cnt_base;
  {
    static const int ef_env = [] { const char* e = getenv("RF_GEMM_W_EVICT_FIRST"); return e ? atoi(e) : 1; }();
    p.w_evict_first = ef_env ? 1 : 0;
  }
  p.ar_recv = g->ar_recv; p.ar_flags = g->ar_flags; p.ar_state = g->ar_state; p.ar_half_bytes = g->ar_recv_bytes;
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(pl.ctas), dim3(kSkThreads), pl.smem, stream, 1, tmX, p));
  ::rf::count_launch();
  return RF_OK;
}

int launch_gemm_sk(const RfGemm* g, cudaStream_t stream) {
  SkPlan pl;
  if (!sk_plan(g, &pl)) return fail(RF_ERR_STATE, "stream-K GEMM: shape is not eligible");
  const bool dual = g->dual_offset > 0;
  if (g->dtype == 0) return dual ? launch_sk<__half, true>(g, pl, stream) : launch_sk<__half, false>(g, pl, stream);
  return dual ? launch_sk<__nv_bfloat16, true>(g, pl, stream) : launch_sk<__nv_bfloat16, false>(g, pl, stream);
}

}  // namespace rf

// 0 never, 1 automatic (large N only), 2 every eligible shape; returns the previous mode.  For tests and A/B timing.
extern "C" int rf_gemm_streamk_mode(int mode) {
  const int old = rf::sk_mode();
  if (mode >= 0 && mode <= 2) rf::g_sk_mode.store(mode, std::memory_order_relaxed);
  return old;
}
