// Persistent tcgen05 GEMM for large token counts (prefill):  out[M,N] = epilogue( x[M,K] . w[N,K]^T ).
//
// One CTA per SM walks a list of (128*MT) x BN output tiles.  Three roles run concurrently:
//   warp 0      TMA producer: the activation tile(s) by tensor map, the weight blocks (tile-major layout) by
//               bulk copy; its ring runs ahead into the next tile while the current one is still multiplying;
//   warp 1      MMA issuer: accumulates a tile into an accumulator buffer in tensor memory;
//   warps 2..   epilogue (four warps per 128-row half): scale, bias, activation / GLU, residual, store.
// MT = 1: 128 x BN tiles and TWO accumulator buffers, so a tile's epilogue runs under the next tile's MMAs.
// MT = 2: 256 x BN tiles; each weight tile in shared memory feeds two MMAs (rows 0-127 and 128-255), which
//         cuts the shared-memory fill per FLOP by a third - the limit of the 128-row tile, whose operand
//         stream (48 KB per 4.2 MFLOP) cannot be kept in flight deep enough to cover the L2 latency.  The two
//         halves take all 512 tensor-memory columns, so the epilogue (eight warps) is not overlapped; the
//         producer still runs ahead into the next tile meanwhile.
// This removes the per-tile start-up bubbles of gemm_tc.cu's one-tile CTAs, which is what limits that kernel
// on compute-bound shapes.  Tiles are numbered with the M index fastest, so the CTAs that run side by side
// share one weight panel and the activation matrix stays in L2.
// Scope: tokens on the MMA M axis, tile-major 16-bit weights, no split-K, no fused all-reduce (those shapes
// stay with gemm_tc.cu).
//
// Grouped form (mixture of experts, rf_moe_grouped_gemm): the rows are (token, pick) pairs sorted by expert and
// the tile list comes from device memory - one entry {expert, first row, end row} per 128-row block of one
// expert's rows.  A tile reads its rows from the sorted activation matrix and its weight blocks from that
// expert's row tiles (up / gate projections) or k blocks (down projection) of the one packed expert bank; rows
// of the block that belong to the next expert are multiplied but never stored.  The number of tiles is only
// known on the device, so every CTA reads it there: the launch itself is shape-independent and graph-capturable.
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kPsBM = 128, kPsBK = 64;
constexpr int kPsATile = kPsBM * kPsBK * 2;      // 16 KB
constexpr int kPsBlock = 128 * kPsBK * 2;        // one packed weight block
constexpr int kPsMaxStages = 8;
constexpr int kPsEpiBytes = 32 * 64 * 2;          // staging of one epilogue warp: 32 rows x 64 columns, 16-bit

struct GemmPsParams {
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias; const void* scale; const float* row_scale;
  const uint8_t* w_packed;
  int32_t* status;
  int M, N, k_blocks, bn, stages, act, dual_offset, dual_tiles;
  int tiles_m, tiles_n;   // tiles_m counts tiles of 128*MT rows
  int band;               // row tiles per band of the tile order
  int pf_blocks;          // k blocks prefetched into L2 ahead of the ring
  int tma_out;            // results leave through shared-memory staging: 1 tiled bulk stores, 2 bulk reduce-adds
                          // into an output that already holds the residual (out == residual)
  // grouped form: grp[0] = number of row blocks, then {expert, row0, row_end, 0} per block (device memory)
  const int32_t* grp;
  int grp_rt_per_expert;  // row tiles of the weight image between two experts (projection whose N axis is split by expert)
  int grp_kb_per_expert;  // k blocks of the weight image between two experts (projection whose K axis is split by expert)
  int kb_total;           // k blocks of a row tile of the whole weight image (stride between row tiles)
};

// Tile order: bands of `band` row tiles; inside a band the row index runs fastest and the weight panel
// advances slowly.  The CTAs that run side by side then share a few weight panels and one band of the
// activation matrix, and the band (sized to a fraction of L2) is reused from L2 by every panel of the sweep
// instead of being streamed from DRAM once per wave.
__device__ __forceinline__ void ps_tile_coords(const GemmPsParams& p, int tile, int* tm, int* tn) {
  const int per_band = p.band * p.tiles_n;
  const int b = tile / per_band, r = tile - b * per_band;
  const int rows_here = min(p.band, p.tiles_m - b * p.band);
  *tn = r / rows_here;
  *tm = b * p.band + r % rows_here;
}

// Coordinates of one tile: first activation row, end of the valid rows, weight column tile, and the offsets of
// the tile's expert inside the packed weight image (zero in the plain form).
struct PsTile { int row0, row_end, tm, tn, rt_add, kb_add; };
template <int MT>
__device__ __forceinline__ PsTile ps_tile(const GemmPsParams& p, int tile) {
  PsTile t;
  if (p.grp) {
    const int entry = tile / p.tiles_n;
    t.tn = tile - entry * p.tiles_n;
    const int e = p.grp[1 + 4 * entry];
    t.row0 = p.grp[2 + 4 * entry];
    t.row_end = p.grp[3 + 4 * entry];
    t.tm = 0;
    t.rt_add = e * p.grp_rt_per_expert;
    t.kb_add = e * p.grp_kb_per_expert;
  } else {
    ps_tile_coords(p, tile, &t.tm, &t.tn);
    t.row0 = t.tm * MT * kPsBM;
    t.row_end = p.M;
    t.rt_add = 0;
    t.kb_add = 0;
  }
  return t;
}

struct alignas(8) GemmPsCtl {
  uint64_t full[kPsMaxStages], empty[kPsMaxStages], acc_full[2], acc_empty[2];
  uint32_t tmem_base;
  int32_t abort_flag;
};

template <typename T, bool DUAL, int MT>
__global__ void __launch_bounds__(64 + 128 * MT)
gemm_ps_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmO, const GemmPsParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int bn = p.bn;
  constexpr int kW = DUAL ? 2 : 1;                         // weight tiles per stage
  const int b_bytes = bn * kPsBK * 2;
  constexpr int kAStage = MT * kPsATile;                   // activation bytes of one stage
  const int stage_bytes = kAStage + kW * b_bytes;
  const int half_cols = kW * bn;                           // TMEM columns of one 128-row half
  const int acc_cols = MT * half_cols;                     // ... of one accumulator buffer
  const int nbuf = 2 * acc_cols <= 512 ? 2 : 1;
  // after the ring: one 4 KB output staging buffer per epilogue warp, then the control block
  uint8_t* epi_stage = smem + (size_t)p.stages * stage_bytes;
  GemmPsCtl* ctl = reinterpret_cast<GemmPsCtl*>(epi_stage + 4 * MT * kPsEpiBytes);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&ctl->acc_full[b], 1);
      mbar_init(&ctl->acc_empty[b], 4 * MT);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    if (p.tma_out) tma_prefetch_desc(&tmO);
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
  // Plain form: the tile count is a launch constant.  Grouped form: it (and the list) was written by the kernel
  // before this one, so it may only be read after the dependency wait; nothing of a tile is touched before that.
  auto tile_count = [&]() { return p.grp ? p.grp[0] * p.tiles_n : p.tiles_m * p.tiles_n; };

  if (warp == 0) {
    // ------------------------------------------------------------------ producer ----
    if (lane == 0) {
      const int nsub = bn / 128;
      auto load_w = [&](const PsTile& t, int kb, int s) {
        uint8_t* sb = smem + (size_t)s * stage_bytes + kAStage;
        const int rt0 = t.tn * nsub + t.rt_add;
#pragma unroll
        for (int wt = 0; wt < kW; ++wt)
          for (int sub = 0; sub < nsub; ++sub)
            bulk_load_1d(sb + wt * b_bytes + sub * kPsBlock,
                         p.w_packed + ((size_t)(rt0 + sub + wt * p.dual_tiles) * p.kb_total + t.kb_add + kb) * kPsBlock,
                         kPsBlock, &ctl->full[s]);
      };
      auto load_x = [&](const PsTile& t, int kb, int s) {
#pragma unroll
        for (int h = 0; h < MT; ++h)   // a half wholly past the last row is zero-filled by the copy engine
          tma_load_2d(smem + (size_t)s * stage_bytes + h * kPsATile, &tmA, &ctl->full[s], kb * kPsBK,
                      t.row0 + h * kPsBM);
      };
      // L2 prefetch cursor: runs p.pf_blocks k blocks ahead of the ring (into the following tiles as well), so
      // the ring's own copies complete with L2 latency and the bytes in flight towards DRAM are not limited by
      // shared memory
      const int tiles = p.grp ? 0 : p.tiles_m * p.tiles_n;   // the prefetch cursor and the early ring fill are plain-form only
      int pf_tile = blockIdx.x, pf_kb = 0, pf_tm = 0, pf_tn = 0;
      if (pf_tile < tiles) ps_tile_coords(p, pf_tile, &pf_tm, &pf_tn);
      auto prefetch_next = [&](bool weights, bool acts) {
        if (pf_tile >= tiles) return;
        if (weights) {
          const int rt0 = pf_tn * nsub;
#pragma unroll
          for (int wt = 0; wt < kW; ++wt)
            for (int sub = 0; sub < nsub; ++sub)
              bulk_prefetch_l2(p.w_packed + ((size_t)(rt0 + sub + wt * p.dual_tiles) * p.k_blocks + pf_kb) * kPsBlock,
                               kPsBlock);
        }
        if (acts) {
#pragma unroll
          for (int h = 0; h < MT; ++h)
            if ((pf_tm * MT + h) * kPsBM < p.M) tma_prefetch_2d(&tmA, pf_kb * kPsBK, (pf_tm * MT + h) * kPsBM);
        }
        if (++pf_kb == p.k_blocks) {
          pf_kb = 0;
          pf_tile += gridDim.x;
          if (pf_tile < tiles) ps_tile_coords(p, pf_tile, &pf_tm, &pf_tn);
        }
      };
      // weights never depend on the previous kernel: the first ring fill starts before the dependency wait
      int it = 0;
      int tile = blockIdx.x;
      PsTile t0 = {};
      if (tile < tiles) t0 = ps_tile<MT>(p, tile);
      const int first_pre = tile < tiles ? min(p.stages, p.k_blocks) : 0;
      for (int i = 0; i < first_pre; ++i) {
        mbar_arrive_expect_tx(&ctl->full[i], (uint32_t)stage_bytes);
        load_w(t0, i, i);
      }
      // the cursor passes the blocks the ring has just asked for, then takes its lead (weights only: the
      // activations may still be written by the previous kernel)
      const int lead = p.pf_blocks > 0 ? first_pre + p.pf_blocks : 0;
      for (int i = 0; i < lead; ++i) prefetch_next(i >= first_pre, false);
      pdl_wait();
      for (int i = 0; i < first_pre; ++i) load_x(t0, i, i);
      bool ok = true;
      int issued = first_pre;
      const int ntiles = tile_count();
      for (; ok && tile < ntiles; tile += gridDim.x) {
        const PsTile t = ps_tile<MT>(p, tile);
        for (int kb = (tile == (int)blockIdx.x ? first_pre : 0); kb < p.k_blocks; ++kb) {
          const int gi = it + kb;                          // global k-block index of this CTA
          const int s = gi % p.stages;
          if (!mbar_wait(&ctl->empty[s], (((uint32_t)(gi / p.stages)) & 1u) ^ 1u, kLocalWaitNs, 32) || *abort_flag) {
            if (!*abort_flag) report_status(p.status, kStatusTmaTimeout, kTagGemmTc, gi);
            ok = false;
            break;
          }
          mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)stage_bytes);
          load_w(t, kb, s);
          load_x(t, kb, s);
          if (p.pf_blocks > 0) prefetch_next(true, true);
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
      const int tiles = tile_count();
      for (int tile = blockIdx.x; ok && tile < tiles; tile += gridDim.x, ++lt) {
        const int b = lt % nbuf;
        if (!mbar_wait(&ctl->acc_empty[b], (((uint32_t)(lt / nbuf)) & 1u) ^ 1u, kLocalWaitNs, 32)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t acc = tmem_base + (uint32_t)(b * acc_cols);
        for (int kb = 0; kb < p.k_blocks; ++kb, ++it) {
          const int s = it % p.stages;
          if (!mbar_wait(&ctl->full[s], (uint32_t)(it / p.stages) & 1u, kLocalWaitNs, 0)) { ok = false; break; }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
          const uint32_t b_addr = a_addr + kAStage;
#pragma unroll
          for (int k = 0; k < kPsBK / 16; ++k) {
            const uint32_t accum = (kb | k) ? 1u : 0u;
            const uint64_t db = umma_desc_k128(b_addr + k * 32);
            const uint64_t db2 = umma_desc_k128(b_addr + b_bytes + k * 32);
#pragma unroll
            for (int h = 0; h < MT; ++h) {
              const uint64_t da = umma_desc_k128(a_addr + h * kPsATile + k * 32);
              umma_f16(acc + h * half_cols, da, db, idesc, accum);
              if (DUAL) umma_f16(acc + h * half_cols + bn, da, db2, idesc, accum);
            }
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
    const int quarter = warp & 3;                          // the TMEM lanes a warp may read
    const int half = (warp - 2) >> 2;                      // which 128-row half of the tile it drains
    const int r = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const T* bias = reinterpret_cast<const T*>(p.bias);
    const T* scale = reinterpret_cast<const T*>(p.scale);
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    const int N = p.N;
    const bool vec_ok = (p.ldo & 7) == 0 && (!resid || (p.ldr & 7) == 0);
    int lt = 0;
    const int tiles = tile_count();
    for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++lt) {
      const int b = lt % nbuf;
      const PsTile pt = ps_tile<MT>(p, tile);
      const int tn = pt.tn;
      const int M = pt.row_end;                            // rows at and past it are not this tile's to store
      if (!mbar_wait(&ctl->acc_full[b], (uint32_t)(lt / nbuf) & 1u) || *abort_flag) {
        if (!*abort_flag) report_status(p.status, kStatusEpilogueTimeout, kTagGemmTc, tile);
        ctl->abort_flag = 1;
        break;
      }
      tc_fence_after_sync();
      const int row = pt.row0 + half * kPsBM + r;
      const int n_base = tn * bn;
      const uint32_t acc = lane_base + (uint32_t)(b * acc_cols + half * half_cols);
      const float rs = (p.row_scale && row < M) ? p.row_scale[row] : 1.f;
      // Results go straight from registers to global memory, 16 columns (of each accumulator) per tensor-memory
      // round trip for one accumulator and 32 for the GLU pair.  Measured alternatives on 8192 x 4096 x 4096:
      // 64-column round trips 30 % slower, a shared-memory transpose for full-line stores 35 % slower - long
      // instruction bursts of the epilogue warps delay the single MMA-issuing lane that shares their schedulers,
      // so the loop is kept short: scale / bias work and the activation switch are hoisted out of the element loop.
      const bool affine = scale || bias || p.row_scale;   // per-element scale / bias work, hoisted out of the loop
      // Output path without a residual, or with the residual already in place (out == residual, the decoder's
      // out-projection and down-projection): 64 finished columns of the warp's 32 rows are parked in a swizzled
      // staging tile and leave as ONE tiled bulk store (or bulk reduce-add, which makes the residual add an L2
      // operation) issued by lane 0 - whole 128-byte lines, asynchronous, no load or store instructions on the
      // epilogue warps (16-byte stores to 32 rows per instruction kept the store queue saturated: 537 MB on the
      // L1->L2 path for 67 MB of output).
      const bool tma_out = p.tma_out != 0;
      uint8_t* stg = epi_stage + (size_t)(warp - 2) * kPsEpiBytes;
      const int row0 = pt.row0 + half * kPsBM + quarter * 32;
      auto chunk_begin = [&]() {                       // the previous bulk store has read the staging tile
        if (lane == 0) bulk_wait_read_all();
        __syncwarp();
      };
      auto chunk_end = [&](int c_first) {              // c_first: first column of the 64-column chunk in the tile
        fence_proxy_async();
        __syncwarp();
        if (lane == 0 && row0 < M && n_base + c_first < N) {
          if (p.tma_out == 2) tma_reduce_add_2d(&tmO, stg, n_base + c_first, row0);
          else tma_store_2d(&tmO, stg, n_base + c_first, row0);
          bulk_commit_group();
        }
      };
      auto finish16 = [&](int n0, const uint32_t* g16, const uint32_t* u16) {
        float g[16], u[16], v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          g[j] = __uint_as_float(g16[j]);
          u[j] = DUAL ? __uint_as_float(u16[j]) : 0.f;
        }
        if (affine) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int n = n0 + j;
            g[j] *= rs;
            if (DUAL) u[j] *= rs;
            if (n < N) {
              if (scale) {
                g[j] *= Num<T>::to_f(scale[n]);
                if (DUAL) u[j] *= Num<T>::to_f(scale[p.dual_offset + n]);
              }
              if (bias) {
                g[j] += Num<T>::to_f(bias[n]);
                if (DUAL) u[j] += Num<T>::to_f(bias[p.dual_offset + n]);
              }
            }
          }
        }
        apply_act_n<16>(p.act, g, u, v);
        if (tma_out) {
          // row `lane` of the warp's staging tile, 128-byte swizzled as the bulk store expects it
          const int ch = ((n0 - n_base) >> 3) & 7;
          float lo[8], hi[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
          store8(reinterpret_cast<T*>(stg + lane * 128 + ((ch ^ (lane & 7)) << 4)), lo);
          store8(reinterpret_cast<T*>(stg + lane * 128 + (((ch + 1) ^ (lane & 7)) << 4)), hi);
        } else if (vec_ok && n0 + 16 <= N) {
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
      };
      if constexpr (DUAL) {
        for (int c0 = 0; c0 < bn; c0 += 32) {
          uint32_t ra[32], rb[32];
          tmem_ld32(acc + c0, ra);
          tmem_ld32(acc + bn + c0, rb);
          tmem_ld_wait();
          if (tma_out && (c0 & 63) == 0) chunk_begin();
          if (row < M || tma_out) {
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int n0 = n_base + c0 + q * 16;
              if (n0 < N || tma_out) finish16(n0, ra + q * 16, rb + q * 16);
            }
          }
          if (tma_out && (c0 & 63) == 32) chunk_end(c0 - 32);
        }
      } else {
        for (int c0 = 0; c0 < bn; c0 += 16) {
          uint32_t ra[16];
          tmem_ld16(acc + c0, ra);
          tmem_ld_wait();
          const int n0 = n_base + c0;
          if (tma_out && (c0 & 63) == 0) chunk_begin();
          if ((row < M && n0 < N) || tma_out) finish16(n0, ra, ra);
          if (tma_out && (c0 & 63) == 48) chunk_end(c0 - 48);
        }
      }
      // this accumulator buffer may now be overwritten by a later tile
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->acc_empty[b]);
    }
    if (p.tma_out && lane == 0) bulk_wait_all();       // the last stores are complete before the CTA retires
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, 512u);
}

template <typename T, bool DUAL, int MT>
static int launch_ps(const RfGemm* g, int bn, cudaStream_t stream) {
  auto kfn = gemm_ps_kernel<T, DUAL, MT>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 227 * 1024);
  CUtensorMap tmA, tmO;
  int rc = make_tmap_2d(&tmA, g->x, g->dtype, 2, g->K, g->M, g->ldx, kPsBK, kPsBM, true);
  if (rc) return rc;
  static const bool tma_out_enabled = [] { const char* e = getenv("RF_GEMM_PS_TMA_OUT"); return !(e && e[0] == '0'); }();
  const bool inplace_resid = g->residual == g->out && g->ldr == g->ldo;
  const bool tma_out = tma_out_enabled && (!g->residual || inplace_resid) && (g->ldo & 7) == 0 &&
                       (reinterpret_cast<uintptr_t>(g->out) & 15) == 0;
  if (tma_out) {
    rc = make_tmap_2d(&tmO, g->out, g->dtype, 2, g->N, g->M, g->ldo, 64, 32, true);
    if (rc) return rc;
  } else {
    tmO = tmA;
  }
  GemmPsParams p = {};
  p.out = g->out; p.ldo = g->ldo; p.residual = g->residual; p.ldr = g->ldr;
  p.bias = g->bias; p.scale = g->scale; p.row_scale = g->row_scale;
  p.w_packed = reinterpret_cast<const uint8_t*>(g->w);
  p.status = g->status;
  p.tma_out = tma_out ? (g->residual ? 2 : 1) : 0;
  p.M = g->M; p.N = g->N; p.k_blocks = ceil_div(g->K, kPsBK); p.bn = bn;
  p.kb_total = p.k_blocks;
  p.act = g->act; p.dual_offset = g->dual_offset; p.dual_tiles = ceil_div(g->N, 128);
  p.tiles_m = ceil_div(g->M, kPsBM * MT); p.tiles_n = ceil_div(g->N, bn);
  const int stage_bytes = MT * kPsATile + (DUAL ? 2 : 1) * bn * kPsBK * 2;
  {
    // a band of activation rows of about 16 MB: it and a weight matrix of a few tens of MB stay in L2 together
    const int64_t row_tile_bytes = (int64_t)kPsBM * MT * g->K * 2;
    p.band = (int)std::max<int64_t>(1, std::min<int64_t>(p.tiles_m, (16ll << 20) / std::max<int64_t>(1, row_tile_bytes)));
    static const int band_env = [] { const char* e = getenv("RF_GEMM_PS_BAND"); return e ? atoi(e) : 0; }();
    if (band_env > 0) p.band = std::min(p.tiles_m, band_env);
    static const int pf_kb = [] { const char* e = getenv("RF_GEMM_L2_PREFETCH_KB"); return e ? atoi(e) : 0; }();
    p.pf_blocks = std::min(16, pf_kb * 1024 / stage_bytes);
  }
  const int ctl_bytes = (int)sizeof(GemmPsCtl) + 1024 /*alignment slack*/ + 4 * MT * kPsEpiBytes;
  p.stages = std::min(kPsMaxStages, (227 * 1024 - ctl_bytes) / stage_bytes);
  RF_REQUIRE(p.stages >= 2, "persistent GEMM: a %d-byte stage does not fit twice in shared memory", stage_bytes);
  const size_t smem = (size_t)p.stages * stage_bytes + ctl_bytes;
  const int grid = std::min(p.tiles_m * p.tiles_n, sm_count());
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(grid), dim3(64 + 128 * MT), smem, stream, 1, tmA, tmO, p));
  ::rf::count_launch();
  return RF_OK;
}

// Rows per tile: 256 (MT = 2) once that still gives about one tile per SM, else 128 down to half a tile per SM;
// 0 = not a persistent shape.
static int ps_rows_per_tile(const RfGemm* g, int bn) {
  static const int forced = [] { const char* e = getenv("RF_GEMM_PS_ROWS"); return e ? atoi(e) : 0; }();
  const int t1 = ceil_div(g->M, kPsBM) * ceil_div(g->N, bn), t2 = ceil_div(g->M, 2 * kPsBM) * ceil_div(g->N, bn);
  if (forced == 128 || forced == 256) return (forced == 256 ? t2 : t1) >= sm_count() / 2 ? forced : 0;
  if (t2 * 4 >= sm_count() * 3) return 256;
  return t1 * 2 >= sm_count() ? 128 : 0;   // half a wave of 128-row tiles still beats one-tile CTAs (Pi0.5 chunk 28.3 -> 26.6 ms)
}

// True when the persistent kernel takes this GEMM (called by rf_gemm after its argument checks).
bool gemm_ps_eligible(const RfGemm* g, bool swap, int splits) {
  static const bool enabled = [] { const char* e = getenv("RF_GEMM_PERSISTENT"); return !(e && e[0] == '0'); }();
  if (!enabled || swap || splits != 1 || g->ar_world > 1 || !g->w_packed || g->w_int8) return false;
  const bool dual = g->dual_offset > 0;
  const int bn = (!dual && g->N % 256 == 0) ? 256 : 128;
  return ps_rows_per_tile(g, bn) != 0;
}

template <typename T>
static int launch_ps_t(const RfGemm* g, bool dual, int bn, int rows, cudaStream_t stream) {
  if (rows == 256) return dual ? launch_ps<T, true, 2>(g, bn, stream) : launch_ps<T, false, 2>(g, bn, stream);
  return dual ? launch_ps<T, true, 1>(g, bn, stream) : launch_ps<T, false, 1>(g, bn, stream);
}

int launch_gemm_ps(const RfGemm* g, cudaStream_t stream) {
  const bool dual = g->dual_offset > 0;
  const int bn = (!dual && g->N % 256 == 0) ? 256 : 128;
  const int rows = ps_rows_per_tile(g, bn);
  if (g->dtype == 0) return launch_ps_t<__half>(g, dual, bn, rows, stream);
  return launch_ps_t<__nv_bfloat16>(g, dual, bn, rows, stream);
}

// Grouped (mixture-of-experts) launch: see the file comment.  One accumulator or a GLU pair, 128-row tiles.
template <typename T, bool DUAL>
static int launch_ps_grouped(const RfMoeGroupedGemm* a, cudaStream_t stream) {
  auto kfn = gemm_ps_kernel<T, DUAL, 1>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 227 * 1024);
  CUtensorMap tmA;
  int rc = make_tmap_2d(&tmA, a->x, a->dtype, 2, a->K, a->max_rows, a->ldx, kPsBK, kPsBM, true);
  if (rc) return rc;
  const int bn = (!DUAL && a->N % 256 == 0) ? 256 : 128;
  GemmPsParams p = {};
  p.out = a->out; p.ldo = a->ldo;
  p.row_scale = a->row_scale;
  p.w_packed = reinterpret_cast<const uint8_t*>(a->w);
  p.status = a->status;
  p.M = a->max_rows; p.N = a->N; p.k_blocks = ceil_div(a->K, kPsBK); p.bn = bn;
  p.act = a->act; p.dual_offset = DUAL ? a->N : 0; p.dual_tiles = a->bank_section_row_tiles;
  p.tiles_m = 0; p.tiles_n = ceil_div(a->N, bn);
  p.band = 1;
  p.grp = a->tiles; p.grp_rt_per_expert = a->rt_per_expert; p.grp_kb_per_expert = a->kb_per_expert;
  p.kb_total = a->bank_kb_total;
  const int stage_bytes = kPsATile + (DUAL ? 2 : 1) * bn * kPsBK * 2;
  const int ctl_bytes = (int)sizeof(GemmPsCtl) + 1024 + 4 * kPsEpiBytes;
  p.stages = std::min(kPsMaxStages, (227 * 1024 - ctl_bytes) / stage_bytes);
  const size_t smem = (size_t)p.stages * stage_bytes + ctl_bytes;
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(sm_count()), dim3(64 + 128), smem, stream, 1, tmA, tmA, p));
  ::rf::count_launch();
  return RF_OK;
}

int launch_moe_grouped(const RfMoeGroupedGemm* a, cudaStream_t stream) {
  if (a->dtype == 0) return a->dual ? launch_ps_grouped<__half, true>(a, stream) : launch_ps_grouped<__half, false>(a, stream);
  return a->dual ? launch_ps_grouped<__nv_bfloat16, true>(a, stream) : launch_ps_grouped<__nv_bfloat16, false>(a, stream);
}

// int8 tile-major weight image -> 16-bit tile-major image (the 128-byte-swizzled block layout the MMA reads).
// One thread widens eight values: 8 bytes in, 16 bytes out.  Exact in fp16 and bf16 (|q| <= 127).
template <typename T>
__global__ void widen_packed_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int64_t pieces) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < pieces; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t block = i >> 10;                     // 128 rows x 8 pieces
    const int row = (int)(i & 1023) >> 3, c = (int)(i & 7);
    const uint2 q = *reinterpret_cast<const uint2*>(src + block * 8192 + row * 64 + c * 8);
    *reinterpret_cast<uint4*>(dst + block * 16384 + row * 128 + ((c ^ (row & 7)) << 4)) = widen_i8x8<T>(q);
  }
}

int widen_packed(const void* src, void* dst, int64_t blocks, int dtype, cudaStream_t stream) {
  const int64_t pieces = blocks * 1024;
  const int grid = (int)std::min<int64_t>((pieces + 255) / 256, (int64_t)sm_count() * 16);
  // no programmatic dependent launch here: the GEMM that follows prefetches this image before its dependency wait
  const uint8_t* sp = reinterpret_cast<const uint8_t*>(src);
  uint8_t* dp = reinterpret_cast<uint8_t*>(dst);
  if (dtype == 0) RF_CUDA_CHECK(::rf::launch_serial(widen_packed_kernel<__half>, dim3(grid), dim3(256), 0, stream, sp, dp, pieces));
  else RF_CUDA_CHECK(::rf::launch_serial(widen_packed_kernel<__nv_bfloat16>, dim3(grid), dim3(256), 0, stream, sp, dp, pieces));
  ::rf::count_launch();
  return RF_OK;
}

}  // namespace rf

extern "C" int rf_moe_grouped_gemm(const RfMoeGroupedGemm* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a && a->x && a->w && a->out && a->tiles, "moe_grouped_gemm needs x, w, out and the tile list");
  RF_REQUIRE(a->max_rows > 0 && a->N > 0 && a->K > 0 && a->K % 8 == 0 && a->ldx % 8 == 0, "moe_grouped_gemm shape %d x %d x %d",
             a->max_rows, a->N, a->K);
  RF_REQUIRE(a->dtype == 0 || a->dtype == 1, "moe_grouped_gemm dtype");
  RF_REQUIRE(a->bank_kb_total > 0 && a->rt_per_expert >= 0 && a->kb_per_expert >= 0, "moe_grouped_gemm bank geometry");
  RF_REQUIRE((reinterpret_cast<uintptr_t>(a->w) & 127) == 0, "packed expert bank must be 128-byte aligned");
  if (a->dual) RF_REQUIRE(a->bank_section_row_tiles > 0 && (a->act == rf::kActSiluMul || a->act == rf::kActGeluTanhMul),
                          "a GLU grouped GEMM needs the section size and a *_mul activation");
  return rf::launch_moe_grouped(a, static_cast<cudaStream_t>(stream));
}
