// Persistent tcgen05 GEMM for large token counts (prefill):  out[M,N] = epilogue( x[M,K] . w[N,K]^T ).
//
// One CTA per SM walks a list of 128 x BN output tiles.  Three roles run concurrently and never wait for
// each other at tile boundaries:
//   warp 0      TMA producer: the activation tile by tensor map, the weight blocks (tile-major layout) by
//               bulk copy; its ring runs ahead into the next tile while the current one is still multiplying;
//   warp 1      MMA issuer: accumulates a tile into one of TWO accumulator buffers in tensor memory;
//   warps 2-5   epilogue: drain the other accumulator buffer (scale, bias, activation / GLU, residual, store)
//               while the tensor core already works on the next tile.
// This removes the per-tile start-up and epilogue bubbles of gemm_tc.cu's one-tile CTAs, which is what limits
// that kernel on compute-bound shapes.  Tiles are numbered with the M index fastest, so the CTAs that run
// side by side share one weight panel and the activation matrix stays in L2.
// Scope: tokens on the MMA M axis, tile-major 16-bit weights, no split-K, no fused all-reduce (those shapes
// stay with gemm_tc.cu).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kPsBM = 128, kPsBK = 64;
constexpr int kPsATile = kPsBM * kPsBK * 2;      // 16 KB
constexpr int kPsBlock = 128 * kPsBK * 2;        // one packed weight block
constexpr int kPsThreads = 192;
constexpr int kPsMaxStages = 8;

struct GemmPsParams {
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias; const void* scale; const float* row_scale;
  const uint8_t* w_packed;
  int32_t* status;
  int M, N, k_blocks, bn, stages, act, dual_offset, dual_tiles;
  int tiles_m, tiles_n;
};

struct alignas(8) GemmPsCtl {
  uint64_t full[kPsMaxStages], empty[kPsMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int32_t abort_flag;
};

template <typename T, bool DUAL>
__global__ void __launch_bounds__(kPsThreads)
gemm_ps_kernel(const __grid_constant__ CUtensorMap tmA, const GemmPsParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bn = p.bn;
  constexpr int kW = DUAL ? 2 : 1;                         // weight tiles per stage
  const int b_bytes = bn * kPsBK * 2;
  const int stage_bytes = kPsATile + kW * b_bytes;
  const int acc_cols = kW * bn;                            // TMEM columns of one accumulator buffer
  GemmPsCtl* ctl = reinterpret_cast<GemmPsCtl*>(smem + (size_t)p.stages * stage_bytes);
  const int tiles = p.tiles_m * p.tiles_n;

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
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, 512u);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  pdl_launch_dependents();         // after this CTA owns its TMEM columns
  volatile int32_t* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ producer ----
    if (lane == 0) {
      const int nsub = bn / 128;
      auto load_w = [&](int tn, int kb, int s) {
        uint8_t* sb = smem + (size_t)s * stage_bytes + kPsATile;
        const int rt0 = tn * nsub;
#pragma unroll
        for (int wt = 0; wt < kW; ++wt)
          for (int sub = 0; sub < nsub; ++sub)
            bulk_load_1d(sb + wt * b_bytes + sub * kPsBlock,
                         p.w_packed + ((size_t)(rt0 + sub + wt * p.dual_tiles) * p.k_blocks + kb) * kPsBlock, kPsBlock,
                         &ctl->full[s]);
      };
      auto load_x = [&](int tm, int kb, int s) {
        tma_load_2d(smem + (size_t)s * stage_bytes, &tmA, &ctl->full[s], kb * kPsBK, tm * kPsBM);
      };
      // weights never depend on the previous kernel: the first ring fill starts before the dependency wait
      int it = 0;
      int tile = blockIdx.x;
      const int first_pre = tile < tiles ? min(p.stages, p.k_blocks) : 0;
      for (int i = 0; i < first_pre; ++i) {
        mbar_arrive_expect_tx(&ctl->full[i], (uint32_t)stage_bytes);
        load_w(tile / p.tiles_m, i, i);
      }
      pdl_wait();
      for (int i = 0; i < first_pre; ++i) load_x(tile % p.tiles_m, i, i);
      bool ok = true;
      int issued = first_pre;
      for (; ok && tile < tiles; tile += gridDim.x) {
        const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
        for (int kb = (tile == (int)blockIdx.x ? first_pre : 0); kb < p.k_blocks; ++kb) {
          const int gi = it + kb;                          // global k-block index of this CTA
          const int s = gi % p.stages;
          if (!mbar_wait(&ctl->empty[s], (((uint32_t)(gi / p.stages)) & 1u) ^ 1u, kLocalWaitNs, 32) || *abort_flag) {
            if (!*abort_flag) report_status(p.status, kStatusTmaTimeout, kTagGemmTc, gi);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)stage_bytes);
          load_w(tn, kb, s);
          load_x(tm, kb, s);
          issued = gi + 1;
        }
        it += p.k_blocks;
      }
      if (!ok) {
        ctl->abort_flag = 1;
        const int first = issued > p.stages ? issued - p.stages : 0;
        for (int gi = first; gi < issued; ++gi)
          mbar_wait(&ctl->full[gi % p.stages], (uint32_t)(gi / p.stages) & 1u, 20ull * 1000 * 1000);
      }
    } else {
      pdl_wait();
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer ----
    pdl_wait();
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_f16(kPsBM, bn, Num<T>::kFmt);
      int it = 0, lt = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x, ++lt) {
        const int b = lt & 1;
        if (!mbar_wait(&ctl->acc_empty[b], (((uint32_t)(lt >> 1)) & 1u) ^ 1u, kLocalWaitNs, 32)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(b * acc_cols);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % p.stages;
          if (!mbar_wait(&ctl->full[s], (uint32_t)(it / p.stages) & 1u, kLocalWaitNs, 0)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t b_addr = a_addr + kPsATile;
#pragma unroll
          for (int k = 0; k < kPsBK / 16; ++k) {
            const uint32_t accum = (kb | k) ? 1u : 0u;
            const uint64_t da = umma_desc_k128(a_addr + k * 32);
            umma_f16(acc, da, umma_desc_k128(b_addr + k * 32), idesc, accum);
            if (DUAL) umma_f16(acc + bn, da, umma_desc_k128(b_addr + b_bytes + k * 32), idesc, accum);
          }
          umma_commit(&ctl->empty[s]);
        }
        if (ok) umma_commit(&ctl->acc_full[b]);
      }
      if (!ok) {
        if (!*abort_flag) report_status(p.status, kStatusMmaTimeout, kTagGemmTc, it);
        ctl->abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------------------------ epilogue ----
    pdl_wait();
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* scale = reinterpret_cast<const T*>(p.scale);
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    const int M = p.M, N = p.N;
    const bool vec_ok = (p.ldo & 7) == 0 && (!resid || (p.ldr & 7) == 0);
    int lt = 0;
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++lt) {
      const int b = lt & 1;
      const int tm = tile % p.tiles_m, tn = tile / p.tiles_m;
      if (!mbar_wait(&ctl->acc_full[b], (uint32_t)(lt >> 1) & 1u) || *abort_flag) {
        if (!*abort_flag) report_status(p.status, kStatusEpilogueTimeout, kTagGemmTc, tile);
        ctl->abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = tm * kPsBM + r;
      const int n_base = tn * bn;
      const uint32_t acc = lane_base + (uint32_t)(b * acc_cols);
      const float rs = (p.row_scale && row < M) ? p.row_scale[row] : 1.f;
      for (int c = 0; c < bn; c += 16) {
        uint32_t rg[16], ru[16];
        tmem_ld16(acc + c, rg);
        if (DUAL) tmem_ld16(acc + bn + c, ru);
        tmem_ld_wait();
        const int n0 = n_base + c;
        if (row >= M || n0 >= N) continue;
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int n = n0 + j;
          float vg = __uint_as_float(rg[j]) * rs, vu = DUAL ? __uint_as_float(ru[j]) * rs : 0.f;
          if (n < N) {
            if (scale) {
              vg *= Num<T>::to_f(scale[n]);
              if (DUAL) vu *= Num<T>::to_f(scale[p.dual_offset + n]);
            }
            if (bias) {
              vg += Num<T>::to_f(bias[n]);
              if (DUAL) vu += Num<T>::to_f(bias[p.dual_offset + n]);
            }
          }
          v[j] = apply_act(p.act, vg, vu);
        }
        if (vec_ok && n0 + 16 <= N) {
          if (resid) {
            float r0[8], r1[8];
            load8(resid + (size_t)row * p.ldr + n0, r0);
            load8(resid + (size_t)row * p.ldr + n0 + 8, r1);
#pragma unroll
            for (int j = 0; j < 8; ++j) { v[j] += r0[j]; v[8 + j] += r1[j]; }
          }
          float lo[8], hi[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
          store8(out + (size_t)row * p.ldo + n0, lo);
          store8(out + (size_t)row * p.ldo + n0 + 8, hi);
        } else {
          for (int j = 0; j < 16; ++j) {
            const int n = n0 + j;
            if (n < N) {
              float x = v[j];
              if (resid) x += Num<T>::to_f(resid[(size_t)row * p.ldr + n]);
              out[(size_t)row * p.ldo + n] = Num<T>::from_f(x);
            }
          }
        }
      }
      // this accumulator buffer may be overwritten by the tile after next
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512u);
}

template <typename T, bool DUAL>
static int launch_ps(const RfGemm* g, int bn, cudaStream_t stream) {
  auto kfn = gemm_ps_kernel<T, DUAL>;
  static bool attr_set = false;
  if (!attr_set) {
    RF_CUDA_CHECK(cudaFuncSetAttribute(kfn, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    attr_set = true;
  }
  CUtensorMap tmA;
  int rc = make_tmap_2d(&tmA, g->x, g->dtype, 2, g->K, g->M, g->ldx, kPsBK, kPsBM, true);
  if (rc) return rc;
  GemmPsParams p = {};
  p.out = g->out; p.ldo = g->ldo; p.residual = g->residual; p.ldr = g->ldr;
  p.bias = g->bias; p.scale = g->scale; p.row_scale = g->row_scale;
  p.w_packed = reinterpret_cast<const uint8_t*>(g->w);
  p.status = g->status;
  p.M = g->M; p.N = g->N; p.k_blocks = ceil_div(g->K, kPsBK); p.bn = bn;
  p.act = g->act; p.dual_offset = g->dual_offset; p.dual_tiles = ceil_div(g->N, 128);
  p.tiles_m = ceil_div(g->M, kPsBM); p.tiles_n = ceil_div(g->N, bn);
  const int stage_bytes = kPsATile + (DUAL ? 2 : 1) * bn * kPsBK * 2;
  const int ctl_bytes = (int)sizeof(GemmPsCtl) + 1024;
  p.stages = std::min(kPsMaxStages, (224 * 1024 - ctl_bytes) / stage_bytes);
  const size_t smem = (size_t)p.stages * stage_bytes + ctl_bytes;
  const int grid = std::min(p.tiles_m * p.tiles_n, sm_count());
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(grid), dim3(kPsThreads), smem, stream, 1, tmA, p));
  ::rf::count_launch();
  return RF_OK;
}

// True when the persistent kernel takes this GEMM (called by rf_gemm after its argument checks).
bool gemm_ps_eligible(const RfGemm* g, bool swap, int splits) {
  static const bool enabled = [] { const char* e = getenv("RF_GEMM_PERSISTENT"); return !(e && e[0] == '0'); }();
  if (!enabled || swap || splits != 1 || g->ar_world > 1 || !g->w_packed || g->w_int8) return false;
  const bool dual = g->dual_offset > 0;
  const int bn = (!dual && g->N % 256 == 0) ? 256 : 128;
  return ceil_div(g->M, kPsBM) * ceil_div(g->N, bn) >= sm_count();
}

int launch_gemm_ps(const RfGemm* g, cudaStream_t stream) {
  const bool dual = g->dual_offset > 0;
  const int bn = (!dual && g->N % 256 == 0) ? 256 : 128;
  if (g->dtype == 0) return dual ? launch_ps<__half, true>(g, bn, stream) : launch_ps<__half, false>(g, bn, stream);
  return dual ? launch_ps<__nv_bfloat16, true>(g, bn, stream) : launch_ps<__nv_bfloat16, false>(g, bn, stream);
}

}  // namespace rf
