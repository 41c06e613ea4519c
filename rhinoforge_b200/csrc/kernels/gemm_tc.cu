// tcgen05 GEMM for sm_100a:  out[M,N] = epilogue( x[M,K] . w[N,K]^T ).
//
// One kernel covers decode (M <= 256 tokens) and prefill:
//  * operands are staged by TMA into 128-byte-swizzled K-major smem tiles and
//    multiplied by tcgen05.mma (kind::f16, fp32 accumulators in TMEM);
//  * "swap" mode puts the WEIGHT rows on the 128-wide MMA M axis and the tokens
//    on the MMA N axis (16..256), so a decode step streams every weight byte
//    exactly once with no padded-token traffic; "normal" mode puts tokens on M;
//  * "dual" mode keeps two accumulators (gate and up projection of the same
//    output feature) and applies act(gate) * up in the epilogue (SwiGLU/GeGLU);
//  * split-K spreads one output tile over a thread-block CLUSTER (up to 8 CTAs
//    along z) so that skinny decode GEMMs still fill 148 SMs; each CTA parks its
//    fp32 partial in its own shared memory and the cluster reduces over
//    distributed shared memory in split order (deterministic, no global scratch);
//  * the epilogue can push its tile to every tensor-parallel peer over NVLink
//    (plain peer stores), wait (bounded) for the peers' tiles and finish the
//    all-reduce + residual in the same kernel.
//
// Replaces the reference's parallel_linear_* tile family, llama_gemv, the
// SiLU/GELU + multiply launches and llama_reduce_sum (src/ops/rpu_linear.cpp:1047-1544,
// src/ops/rpu_linear_gemv.cpp, src/core/fused_model_base.cpp:8515-8567,
// src/core/rpu_runtime_extras.cpp:1035-1092).
#include <map>
#include <mutex>

#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kBM = 128;          // MMA M (rows of operand A per CTA)
constexpr int kBK = 64;           // K elements per smem stage (128 bytes)
constexpr int kATileBytes = kBM * kBK * 2;
constexpr int kMaxStages = 8;   // ring depth (barrier slots); extra smem beyond it only backs the split-K partial

struct GemmTcParams {
  void* out; int64_t ldo;
  const void* residual; int64_t ldr;
  const void* bias; const void* scale; const float* row_scale;
  float* ws; uint32_t* sem; int32_t* status;
  int M, N;
  int k_blocks, splits, bn, stages, act, dual_offset, tmem_cols, ctl_offset;
  int ar_world, ar_rank;
  void* const* ar_recv; uint32_t* const* ar_flags; uint32_t* ar_state;
  uint64_t ar_half_bytes;
  const uint8_t* w_packed;  // tile-major weight image (null: row-major weights through the tensor maps)
  int kb_total;             // k blocks of the whole weight (row-tile stride of the packed image)
  int dual_tiles;           // row tiles of the first (gate) section
  int k_rotate;             // 1: every output tile starts its K loop at a different block
  int ar_two_shot;    // large-M path: 16-bit reduce-scatter to the tile's owner, then broadcast
  int ar_flag2_base;  // first flag of the "result has landed" range
  int ar_publish;     // small-M path: push the partial rows to every rank, bump the arrival counters, exit
  int ar_cnt_base;    // first arrival counter in every rank's flag array
  int ar_stage_off;   // shared-memory offset of the staging rows of the publish path
  const uint8_t* pf_ptr;   // L2 prefetch hint: memory the next kernel will read
  uint32_t pf_chunks;      // number of kPrefetchChunk-byte pieces of it, dealt out over the CTAs
  int w4;                  // 1: int4 weight image (4096 bytes of nibbles + in-block scales per 128 x 64 block)
  int w4_ns;               // scales per row of a block: 0 (per-channel scale in the epilogue), 1, 2 or 4
  int w4_fp4;              // 1: the nibbles are e2m1 floating-point codes
  int pf_ahead;            // packed weights: k blocks beyond the ring that are asked into L2 ahead of their bulk copy
  int w_evict_first;       // packed weights are read with the L2 evict-first policy (streamed once)
  int q_blk_bytes;         // bytes of one quantised 128 x 64 block in the staging area / the packed image
  float* ss_out;           // per (128-column tile, token) sum of squares of the finished values (swap mode)
  const float* ss_in;      // per (tile, token) sums of squares of the input rows: the result is scaled by their rstd
  int ss_tiles, ss_ld;
  float ss_inv_dim, ss_eps;
};
constexpr uint32_t kPrefetchChunk = 8192;

struct alignas(8) GemmSmemCtl {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t ready[kMaxStages];  // W8A16: the converter warps have written the 16-bit weight tile
  uint64_t qfull[kMaxStages];  // W8A16: the int8 staging tile has landed
  uint64_t qempty[kMaxStages]; // W8A16: the converter warps have read the int8 staging tile
  uint64_t accum;
  uint32_t tmem_base;
  int32_t abort_flag;
};
// Scratch behind the control block, present only in launches with a folded RMSNorm (ss_in / ss_out):
// rs[256] = reciprocal RMS of this tile's token columns, then ssw[4][256] = the four epilogue warps' partial sums of
// squares per token column.
constexpr int kSsScratchBytes = (256 + 4 * 256) * (int)sizeof(float);

// Converter warps of the quantised kernels: the block is 128 threads (producer, MMA issuer, epilogue) plus these.
constexpr int kMaxConvWarps = 6;     // two CTAs of 128 + 192 threads still fit an SM's register file

// W8 = int8 weights (W8A16): TMA brings the int8 tile into a staging area of the stage, the extra
// converter warps widen it into the 128-byte-swizzled 16-bit tile the MMA reads, and the
// per-output-channel scale is applied in the epilogue: (X . Q^T) * s.
template <typename T, bool SWAP, bool DUAL, bool W8>
__global__ void __launch_bounds__(W8 ? 128 + 32 * kMaxConvWarps : 128, W8 ? 2 : 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmW, const GemmTcParams p) {
  // No alignment slack: the W8A16 decode configuration fits two CTAs per SM only without it.  The swizzled
  // tiles need a 1024-byte aligned base, which the runtime provides when the kernel has no static shared
  // memory; a misaligned base is reported instead of being used.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(p.status, kStatusBadArgument, kTagGemmTc, (int)(smem_u32(smem_raw) & 1023u));
    return;
  }
  uint8_t* smem = smem_raw;

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int bn = p.bn;
  constexpr int kATiles = (SWAP && DUAL) ? 2 : 1;
  constexpr int kBTiles = (!SWAP && DUAL) ? 2 : 1;
  const int b_tile_bytes = bn * kBK * 2;
  constexpr int kWTiles = DUAL ? 2 : 1;                    // weight tiles per stage
  const int w_rows = SWAP ? kBM : bn;                      // rows of one weight tile
  const int q_tile_bytes = W8 ? (w_rows / kBM) * p.q_blk_bytes + (w_rows % kBM) * kBK : 0;   // staging of one weight tile
  const int half_bytes = kATiles * kATileBytes + kBTiles * b_tile_bytes;   // the 16-bit tiles
  // the next stage's swizzled 16-bit tiles must start on a 1024-byte boundary (an int4 block with its scales is not
  // a multiple of that)
  const int stage_bytes = half_bytes + ((kWTiles * q_tile_bytes + 1023) & ~1023);
  const int act_bytes = SWAP ? b_tile_bytes : kATileBytes;
  GemmSmemCtl* ctl = reinterpret_cast<GemmSmemCtl*>(smem + p.ctl_offset);

  const int a0 = blockIdx.x * kBM;
  const int b0 = blockIdx.y * bn;
  const int z = blockIdx.z;
  const int kb_base = p.k_blocks / p.splits, kb_rem = p.k_blocks % p.splits;
  const int kb0 = z * kb_base + min(z, kb_rem);
  const int kb_count = kb_base + (z < kb_rem ? 1 : 0);

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
      mbar_init(&ctl->ready[s], (blockDim.x - 128) >> 5);     // one arrival per converter warp
      mbar_init(&ctl->qfull[s], 1);
      mbar_init(&ctl->qempty[s], (blockDim.x - 128) >> 5);
    }
    mbar_init(&ctl->accum, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    if (W8) tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, (uint32_t)p.tmem_cols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  // Only now may the next kernel start launching: its CTAs could take the last
  // TMEM columns of this SM and then sit in their dependency wait, so this CTA
  // must already own its columns (tcgen05.alloc blocks without a time limit).
  // This kernel's own dependency wait comes later, after the weight prefetch.
  pdl_launch_dependents();

  // ------------------------------------------------------- TMA producer ----
  if (warp == 0 && lane_id() == 0) {
    // W8A16 splits a stage's traffic over two barriers: the int8 staging tile (qfull) is refilled as soon as
    // the converter warps have widened it (qempty), without waiting for the MMAs that still read the 16-bit
    // tile of the same stage, so the DRAM latency of the next weights hides behind conversion and MMA.
    const uint32_t tx = W8 ? (uint32_t)act_bytes : (uint32_t)stage_bytes;
    const uint32_t txq = (uint32_t)(kWTiles * q_tile_bytes);
    int issued = 0, issued_q = 0;
    bool ok = true;
    // Weight-streaming CTAs would otherwise all walk their (power-of-two sized) weight panels in lock step and
    // present DRAM with one address offset at a time; each output tile starts its K loop at a different block
    // and wraps around (the accumulation order changes, deterministically per shape).
    const int rot = (SWAP && p.k_rotate) ? (int)((blockIdx.x * 11u + blockIdx.y * 7u) % (uint32_t)kb_count) : 0;
    auto kblock = [&](int i) { const int j = i + rot; return kb0 + (j >= kb_count ? j - kb_count : j); };
    auto load_weights = [&](int i, int s) {
      uint64_t* wbar = W8 ? &ctl->qfull[s] : &ctl->full[s];
      uint8_t* st = smem + (size_t)s * stage_bytes;
      const int kc = kblock(i) * kBK;
      if (p.w_packed) {
        // contiguous 128-row x 64-column blocks: one bulk copy each
        const uint32_t kBlk = W8 ? (uint32_t)p.q_blk_bytes : (uint32_t)kATileBytes;
        const int rt0 = (SWAP ? a0 : b0) / kBM;
        const int nsub = SWAP ? 1 : bn / kBM;
#pragma unroll
        for (int wt = 0; wt < kWTiles; ++wt) {
          uint8_t* dst = W8 ? st + half_bytes + wt * q_tile_bytes
                            : (SWAP ? st + wt * kATileBytes : st + kATiles * kATileBytes + wt * b_tile_bytes);
          for (int sub = 0; sub < nsub; ++sub) {
            const uint8_t* src = p.w_packed + ((size_t)(rt0 + sub + wt * p.dual_tiles) * p.kb_total + kblock(i)) * kBlk;
            if (p.w_evict_first) bulk_load_1d_hint(dst + (size_t)sub * kBlk, src, kBlk, wbar, l2_policy_evict_first());
            else bulk_load_1d(dst + (size_t)sub * kBlk, src, kBlk, wbar);
            // keep more bytes in flight towards HBM than the ring holds: the block that will be copied pf_ahead ring
            // slots from now is asked into L2 already, so that its copy later completes with L2 latency
            if (p.pf_ahead && i + p.pf_ahead < kb_count)
              bulk_prefetch_l2(p.w_packed + ((size_t)(rt0 + sub + wt * p.dual_tiles) * p.kb_total + kblock(i + p.pf_ahead)) * kBlk, kBlk);
          }
        }
      } else if (W8) {
        const int r0 = SWAP ? a0 : b0;
        tma_load_2d(st + half_bytes, &tmW, wbar, kc, r0);
        if (kWTiles == 2) tma_load_2d(st + half_bytes + q_tile_bytes, &tmW, wbar, kc, p.dual_offset + r0);
      } else if (SWAP) {
        tma_load_2d(st, &tmA, &ctl->full[s], kc, a0);
        if (kATiles == 2) tma_load_2d(st + kATileBytes, &tmA, &ctl->full[s], kc, p.dual_offset + a0);
      } else {
        uint8_t* sb = st + kATiles * kATileBytes;
        tma_load_2d(sb, &tmB, &ctl->full[s], kc, b0);
        if (kBTiles == 2) tma_load_2d(sb + b_tile_bytes, &tmB, &ctl->full[s], kc, p.dual_offset + b0);
      }
    };
    auto load_acts = [&](int i, int s) {
      uint8_t* st = smem + (size_t)s * stage_bytes;
      const int kc = kblock(i) * kBK;
      if (SWAP) tma_load_2d(st + kATiles * kATileBytes, &tmB, &ctl->full[s], kc, b0);
      else tma_load_2d(st, &tmA, &ctl->full[s], kc, a0);
    };
    // weights never depend on the previous kernel: fill the ring with them first
    const int pre = min(p.stages, kb_count);
    for (int i = 0; i < pre; ++i) {
      if (W8) mbar_arrive_expect_tx(&ctl->qfull[i], txq);
      else mbar_arrive_expect_tx(&ctl->full[i], tx);
      load_weights(i, i);
    }
    issued_q = pre;
    pdl_wait();
    for (int i = 0; i < pre; ++i) {
      if (W8) mbar_arrive_expect_tx(&ctl->full[i], tx);
      load_acts(i, i);
    }
    issued = pre;
    for (int i = pre; i < kb_count; ++i) {
      const int s = i % p.stages;
      const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
      if (W8) {
        if (!mbar_wait(&ctl->qempty[s], ph ^ 1u)) {
          report_status(p.status, kStatusTmaTimeout, kTagW8A16, i);
          ok = false;
          break;
        }
        if (*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag)) { ok = false; break; }
        mbar_arrive_expect_tx(&ctl->qfull[s], txq);
        load_weights(i, s);
        issued_q = i + 1;
      }
      if (!mbar_wait(&ctl->empty[s], ph ^ 1u)) {
        report_status(p.status, kStatusTmaTimeout, kTagGemmTc, i);
        ok = false;
        break;
      }
      if (*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag)) { ok = false; break; }
      mbar_arrive_expect_tx(&ctl->full[s], tx);
      if (!W8) load_weights(i, s);
      load_acts(i, s);
      issued = i + 1;
    }
    if (ok && p.pf_chunks) {
      // this CTA's own weight loads are all in flight: spend the rest of its life keeping HBM busy for the next kernel
      const uint32_t ncta = gridDim.x * gridDim.y * gridDim.z;
      const uint32_t cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
      for (uint32_t c = cta; c < p.pf_chunks; c += ncta) bulk_prefetch_l2(p.pf_ptr + (size_t)c * kPrefetchChunk, kPrefetchChunk);
    }
    if (!ok) {
      ctl->abort_flag = 1;
      // Let every copy that was issued land before the CTA can exit.
      const int first = issued > p.stages ? issued - p.stages : 0;
      for (int i = first; i < issued; ++i)
        mbar_wait(&ctl->full[i % p.stages], (uint32_t)(i / p.stages) & 1u, 20ull * 1000 * 1000);
      if (W8) {
        const int firstq = issued_q > p.stages ? issued_q - p.stages : 0;
        for (int i = firstq; i < issued_q; ++i)
          mbar_wait(&ctl->qfull[i % p.stages], (uint32_t)(i / p.stages) & 1u, 20ull * 1000 * 1000);
      }
    }
  } else {
    pdl_wait();
  }
  // ------------------------------------------------- W8A16 converter warps ----
  if (W8 && warp >= 4) {
    const int ct = tid - 128, cstep = (int)blockDim.x - 128;
    for (int i = 0; i < kb_count; ++i) {
      const int s = i % p.stages;
      const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
      // the int8 tile has landed, and the MMAs that read this stage's 16-bit tile one ring turn ago are done
      if (!mbar_wait(&ctl->qfull[s], ph) || !mbar_wait(&ctl->empty[s], ph ^ 1u)) {
        report_status(p.status, kStatusMmaTimeout, kTagW8A16, i);
        ctl->abort_flag = 1;
        break;
      }
      if (*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag)) break;
      uint8_t* st = smem + (size_t)s * stage_bytes;
#pragma unroll
      for (int wt = 0; wt < kWTiles; ++wt) {
        const uint8_t* src = st + half_bytes + wt * q_tile_bytes;
        uint8_t* dst = SWAP ? st + wt * kATileBytes : st + kATiles * kATileBytes + wt * b_tile_bytes;
        if (p.w4) {
          // 32 nibbles (one 16-byte piece = half a row) per thread and round -> four 16-byte pieces of the 16-bit tile
          for (int idx = ct; idx < w_rows * 2; idx += cstep) {
            const int row = idx >> 1, h = idx & 1;
            const uint8_t* blk = src + (size_t)(row >> 7) * p.q_blk_bytes;
            const int r = row & 127;
            const uint4 q = *reinterpret_cast<const uint4*>(blk + r * 32 + h * 16);
            // word w of the piece covers columns [32 h + 8 w, +8): its scale is number (4 h + w) * ns / 8 of the row
            const T one = Num<T>::from_f(1.f);
            const T* srow = reinterpret_cast<const T*>(blk + 4096) + r * p.w4_ns;
            const T s0 = p.w4_ns ? srow[(4 * h + 0) * p.w4_ns >> 3] : one, s1 = p.w4_ns ? srow[(4 * h + 1) * p.w4_ns >> 3] : one;
            const T s2 = p.w4_ns ? srow[(4 * h + 2) * p.w4_ns >> 3] : one, s3 = p.w4_ns ? srow[(4 * h + 3) * p.w4_ns >> 3] : one;
            uint8_t* drow = dst + row * 128;
            const int c = 4 * h, sw = row & 7;
            if (p.w4_fp4) {
              *reinterpret_cast<uint4*>(drow + (((c + 0) ^ sw) << 4)) = widen_e2m1x8<T>(q.x, s0);
              *reinterpret_cast<uint4*>(drow + (((c + 1) ^ sw) << 4)) = widen_e2m1x8<T>(q.y, s1);
              *reinterpret_cast<uint4*>(drow + (((c + 2) ^ sw) << 4)) = widen_e2m1x8<T>(q.z, s2);
              *reinterpret_cast<uint4*>(drow + (((c + 3) ^ sw) << 4)) = widen_e2m1x8<T>(q.w, s3);
            } else {
              *reinterpret_cast<uint4*>(drow + (((c + 0) ^ sw) << 4)) = widen_i4x8<T>(q.x, s0);
              *reinterpret_cast<uint4*>(drow + (((c + 1) ^ sw) << 4)) = widen_i4x8<T>(q.y, s1);
              *reinterpret_cast<uint4*>(drow + (((c + 2) ^ sw) << 4)) = widen_i4x8<T>(q.z, s2);
              *reinterpret_cast<uint4*>(drow + (((c + 3) ^ sw) << 4)) = widen_i4x8<T>(q.w, s3);
            }
          }
          continue;
        }
        // 16 int8 (one 16-byte piece) per thread and round; consecutive threads take consecutive pieces, so a
        // warp reads 512 contiguous bytes (8 rows x 64) without bank conflicts
        for (int idx = ct; idx < w_rows * 4; idx += cstep) {
          const int row = idx >> 2, h = idx & 3;
          const uint4 q = *reinterpret_cast<const uint4*>(src + row * kBK + h * 16);
          const int c0 = 2 * h, c1 = 2 * h + 1;
          *reinterpret_cast<uint4*>(dst + row * 128 + ((c0 ^ (row & 7)) << 4)) = widen_i8x8<T>(make_uint2(q.x, q.y));
          *reinterpret_cast<uint4*>(dst + row * 128 + ((c1 ^ (row & 7)) << 4)) = widen_i8x8<T>(make_uint2(q.z, q.w));
        }
      }
      fence_proxy_async();   // generic-proxy writes -> visible to the tensor core's async-proxy reads
      __syncwarp();
      if (lane_id() == 0) {
        mbar_arrive(&ctl->ready[s]);
        mbar_arrive(&ctl->qempty[s]);
      }
    }
  }
  // ------------- folded RMSNorm: reciprocal RMS of this tile's token columns ----
  // Warps 2 and 3 have nothing to do until the accumulator is complete: they add up the producer kernel's per-tile sums
  // of squares (fixed order) while the weights stream.  The block-wide barrier ahead of the epilogue publishes ss_rs.
  if (SWAP && p.ss_in != nullptr && warp >= 2 && warp < 4) {
    float* rs_out = reinterpret_cast<float*>(ctl + 1);
    for (int c = tid - 64; c < bn; c += 64) {
      const int tok = blockIdx.y * bn + c;
      float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
      if (tok < p.M) {
        const float* src = p.ss_in + tok;
        int t = 0;
        for (; t + 4 <= p.ss_tiles; t += 4) {          // four independent loads in flight per round
          s0 += src[(size_t)(t + 0) * p.ss_ld];
          s1 += src[(size_t)(t + 1) * p.ss_ld];
          s2 += src[(size_t)(t + 2) * p.ss_ld];
          s3 += src[(size_t)(t + 3) * p.ss_ld];
        }
        for (; t < p.ss_tiles; ++t) s0 += src[(size_t)t * p.ss_ld];
      }
      rs_out[c] = rsqrtf(((s0 + s1) + (s2 + s3)) * p.ss_inv_dim + p.ss_eps);
    }
  }
  // --------------------------------------------------------- MMA issuer ----
  if (warp == 1 && lane_id() == 0) {
    const uint32_t idesc = umma_idesc_f16(kBM, bn, Num<T>::kFmt);
    bool ok = true;
    for (int i = 0; i < kb_count; ++i) {
      const int s = i % p.stages;
      const uint32_t ph = (uint32_t)(i / p.stages) & 1u;
      if (!mbar_wait(&ctl->full[s], ph)) {
        report_status(p.status, kStatusMmaTimeout, kTagGemmTc, i);
        ok = false;
        break;
      }
      if (W8 && !mbar_wait(&ctl->ready[s], ph)) {
        report_status(p.status, kStatusMmaTimeout, kTagW8A16, 1000 + i);
        ok = false;
        break;
      }
      tc_fence_after_sync();
      const uint32_t a_addr = smem_u32(smem + (size_t)s * stage_bytes);
      const uint32_t b_addr = a_addr + kATiles * kATileBytes;
#pragma unroll
      for (int k = 0; k < kBK / 16; ++k) {
        const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
        const uint64_t da = umma_desc_k128(a_addr + k * 32);
        const uint64_t db = umma_desc_k128(b_addr + k * 32);
        umma_f16(tmem_base, da, db, idesc, acc);
        if (DUAL) {
          if (SWAP) {
            const uint64_t da1 = umma_desc_k128(a_addr + kATileBytes + k * 32);
            umma_f16(tmem_base + bn, da1, db, idesc, acc);
          } else {
            const uint64_t db1 = umma_desc_k128(b_addr + b_tile_bytes + k * 32);
            umma_f16(tmem_base + bn, da, db1, idesc, acc);
          }
        }
      }
      umma_commit(&ctl->empty[s]);
    }
    if (ok) umma_commit(&ctl->accum);
    else ctl->abort_flag = 1;
  }
  __syncwarp();

  // ----------------------------------------------------------- epilogue ----
  bool have_acc = mbar_wait(&ctl->accum, 0);
  if (!have_acc) {
    if (!*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag))
      report_status(p.status, kStatusEpilogueTimeout, kTagGemmTc, (int)blockIdx.y);
    ctl->abort_flag = 1;
  }
  tc_fence_after_sync();
  __syncwarp();

  // a warp reads the TMEM lanes of its own quarter (warp % 4); converter warps alias warps 0-3
  const uint32_t trow = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);
  const bool epi = tid < kBM;                              // converter warps only keep the barriers company
  const int a_idx = epi ? a0 + tid : 0x3fffffff;
  const int M = p.M, N = p.N;
  const int tile_id = blockIdx.y * gridDim.x + blockIdx.x;
  constexpr int kAcc = DUAL ? 2 : 1;

  const T* bias = reinterpret_cast<const T*>(p.bias);
  const T* scale = reinterpret_cast<const T*>(p.scale);
  const T* resid = reinterpret_cast<const T*>(p.residual);
  T* out = reinterpret_cast<T*>(p.out);
  const bool use_bias = bias != nullptr && (p.ar_world <= 1 || p.ar_rank == 0);
  const uint32_t call = (p.ar_world > 1) ? *reinterpret_cast<volatile uint32_t*>(p.ar_state) : 0u;
  const uint64_t slot_off = (uint64_t)(call & 1u) * p.ar_half_bytes;
  const uint32_t crank = p.splits > 1 ? cluster_ctarank() : 0u;

  // folded RMSNorm: reciprocal RMS of every token column of this tile from the producer's per-tile sums of squares
  float* ss_rs = reinterpret_cast<float*>(ctl + 1);
  float (*ss_w)[256] = reinterpret_cast<float (*)[256]>(ss_rs + 256);
  const bool use_rs = SWAP && p.ss_in != nullptr;   // ss_rs was filled by warps 2 and 3 while the main loop ran
  const bool emit_ss = SWAP && p.ss_out != nullptr && p.ar_world <= 1;
  // sum over this warp's 32 output features of the square of one finished value per lane, for token column c
  auto ss_add = [&](int c, float v) {
    float q = v * v;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    if (lane_id() == 0 && warp < 4) ss_w[warp][c] = q;
  };

  // per-element epilogue math shared by both paths
  const bool affine = p.row_scale || scale || use_bias || use_rs;
  auto finish = [&](int tok, int n, float vg, float vu) -> float {
    if (!affine) return apply_act(p.act, vg, vu);
    if (use_rs) {
      const float rs = ss_rs[tok - blockIdx.y * bn];
      vg *= rs;
      vu *= rs;
    }
    if (p.row_scale) {
      const float rs = p.row_scale[tok];
      vg *= rs;
      vu *= rs;
    }
    if (scale) {
      vg *= Num<T>::to_f(scale[n]);
      if (DUAL) vu *= Num<T>::to_f(scale[p.dual_offset + n]);
    }
    if (use_bias) {
      vg += Num<T>::to_f(bias[n]);
      if (DUAL) vu += Num<T>::to_f(bias[p.dual_offset + n]);
    }
    return apply_act(p.act, vg, vu);
  };
  // Peer buffer addresses are read ONCE: the table lives in global memory and nothing tells the compiler
  // that the remote stores below cannot alias it, so a lookup per element would sit between every two stores.
  uint8_t* peer_buf[8];
#pragma unroll
  for (int d = 0; d < 8; ++d)
    peer_buf[d] = (p.ar_world > 1 && d < p.ar_world) ? reinterpret_cast<uint8_t*>(p.ar_recv[d]) + slot_off : nullptr;
  auto push_partial = [&](int tok, int n, float v) {
    const size_t at = ((size_t)p.ar_rank * M + tok) * N + n;
#pragma unroll
    for (int d = 0; d < 8; ++d)
      if (d < p.ar_world) reinterpret_cast<float*>(peer_buf[d])[at] = v;
  };

  // Publish path (swap mode): finished values are parked as rows [token][128 features] in shared memory and leave
  // the CTA as 16-byte vectors, one contiguous 256- or 512-byte row segment per group of 16 or 32 threads.
  const bool pub = SWAP && p.ar_world > 1 && p.ar_publish;
  const bool pub_f32 = M <= RF_AR_F32_MAX_ROWS;
  uint8_t* pub_stage = smem + p.ar_stage_off;
  auto stage_put = [&](int j, float v) {   // j: row of the staging area (this CTA's j-th token)
    if (pub_f32) reinterpret_cast<float*>(pub_stage)[j * kBM + tid] = v;
    else reinterpret_cast<T*>(pub_stage)[j * kBM + tid] = Num<T>::from_f(v);
  };

  bool aborted = __syncthreads_or(*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag) != 0);
  const int ncols = min(bn, (SWAP ? M : N) - b0);  // valid accumulator columns of this tile
  uint8_t* owner_buf = nullptr;                    // two-shot: the buffer of this tile's owner rank
  if (p.ar_world > 1 && p.ar_two_shot) {
    const int owner = tile_id % p.ar_world;
#pragma unroll
    for (int d = 0; d < 8; ++d)
      if (d == owner) owner_buf = peer_buf[d];
  }

  if (p.splits > 1) {
    // ---- split-K: the CTAs of one output tile form a cluster (cluster dim z =
    // splits).  Each parks its fp32 partial in its own shared memory
    // ([column][lane], conflict-free), then CTA r reduces columns r, r+S, ...
    // over distributed shared memory in split order and finishes them.
    float* part = reinterpret_cast<float*>(smem);
    // Token-row tiles PUSH instead: a thread owns one output row and 8-column groups are dealt round-robin to the
    // cluster's CTAs, so every CTA stores each group of its partial straight into the owner's shared memory (slot =
    // sender, [column][lane]); remote stores do not wait for a round trip, and the owner then sums from its own shared
    // memory.  (Pulling the same values cost one distributed-shared-memory round trip per split and column group:
    // ~10 us for a 128 x 128 tile split in four.)  The peers' operand rings must be idle first: one more rendezvous.
    const int gpo = (((bn + 7) >> 3) + p.splits - 1) / p.splits;   // column groups per owner
    const int cpo = gpo * 8;                                       // receive columns per owner and sender
    const uint32_t acc2 = (uint32_t)p.splits * cpo * kBM;          // floats before the second accumulator's slots
    if constexpr (!SWAP) {
      cluster_sync_all();
      if (!aborted) {
        const uint32_t my_slot = smem_u32(part) + ((uint32_t)crank * cpo * kBM + tid) * 4u;
        auto push16 = [&](int c, const uint32_t* rg, const uint32_t* ru) {   // columns c .. c + 15 of this row
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int gi = (c >> 3) + h;
            const uint32_t dst = dsmem_addr(my_slot + (uint32_t)((gi / p.splits) * 8 * kBM) * 4u, (uint32_t)(gi % p.splits));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              st_dsmem_u32(dst + (uint32_t)(j * kBM) * 4u, rg[h * 8 + j]);
              if (DUAL) st_dsmem_u32(dst + (acc2 + (uint32_t)(j * kBM)) * 4u, ru[h * 8 + j]);
            }
          }
        };
        if ((bn & 31) == 0) {
          for (int c = 0; c < bn; c += 32) {
            uint32_t rg[32], ru[32];
            tmem_ld32(trow + c, rg);
            if (DUAL) tmem_ld32(trow + bn + c, ru);
            tmem_ld_wait();
            if (epi) {
              push16(c, rg, ru);
              push16(c + 16, rg + 16, ru + 16);
            }
          }
        } else {
          for (int c = 0; c < bn; c += 16) {
            uint32_t rg[16], ru[16];
            tmem_ld16(trow + c, rg);
            if (DUAL) tmem_ld16(trow + bn + c, ru);
            tmem_ld_wait();
            if (epi) push16(c, rg, ru);
          }
        }
      }
    } else
    if (!aborted) {
      if ((bn & 31) == 0) {
        // 32 columns (of each accumulator) per tensor-memory round trip: the round trip, not the copy, is the cost
        for (int c = 0; c < bn; c += 32) {
          uint32_t rg[32], ru[32];
          tmem_ld32(trow + c, rg);
          if (DUAL) tmem_ld32(trow + bn + c, ru);
          tmem_ld_wait();
          if (epi) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              part[(c + j) * kBM + tid] = __uint_as_float(rg[j]);
              if (DUAL) part[(bn + c + j) * kBM + tid] = __uint_as_float(ru[j]);
            }
          }
        }
      } else {
        for (int c = 0; c < bn; c += 16) {
          uint32_t rg[16], ru[16];
          tmem_ld16(trow + c, rg);
          if (DUAL) tmem_ld16(trow + bn + c, ru);
          tmem_ld_wait();
          if (epi) {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              part[(c + j) * kBM + tid] = __uint_as_float(rg[j]);
              if (DUAL) part[(bn + c + j) * kBM + tid] = __uint_as_float(ru[j]);
            }
          }
        }
      }
    }
    cluster_sync_all();
    if (!aborted) {
      const uint32_t my_part = smem_u32(part);
      uint32_t peer_part[8];
#pragma unroll
      for (int s = 0; s < 8; ++s) peer_part[s] = dsmem_addr(my_part, (uint32_t)(s < p.splits ? s : 0));
      if constexpr (!SWAP) {
        // tokens on the rows: a thread owns one output row, so it takes EIGHT ADJACENT columns per
        // round (column groups are dealt round-robin to the cluster's CTAs) and stores them as one
        // 16-byte vector; single interleaved columns would make every store a lone 2-byte sector write
        for (int g0 = (int)crank * 8; g0 < ncols; g0 += 8 * p.splits) {
          float ag[8], au[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { ag[j] = 0.f; au[j] = 0.f; }
          // the senders' slots of this group, from this CTA's own shared memory, summed in split order
          const float* slot0 = part + (size_t)((g0 >> 3) / p.splits) * 8 * kBM + tid;
          for (int s = 0; s < p.splits; ++s) {
            const float* sp = slot0 + (size_t)s * cpo * kBM;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const bool on = g0 + j < ncols && epi;
              ag[j] += on ? sp[j * kBM] : 0.f;
              if (DUAL) au[j] += on ? sp[acc2 + j * kBM] : 0.f;
            }
          }
          const int n0 = b0 + g0;
          if (a_idx < M) {
            float v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) v[j] = (n0 + j < N) ? finish(a_idx, n0 + j, ag[j], au[j]) : 0.f;
            if (p.ar_world > 1) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                if (n0 + j < N) push_partial(a_idx, n0 + j, v[j]);
            } else if (n0 + 8 <= N && (p.ldo & 7) == 0 && (!resid || (p.ldr & 7) == 0)) {
              if (resid) {
                float r8[8];
                load8(resid + (size_t)a_idx * p.ldr + n0, r8);
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] += r8[j];
              }
              store8(out + (size_t)a_idx * p.ldo + n0, v);
            } else {
              for (int j = 0; j < 8; ++j) {
                if (n0 + j < N) {
                  float r = v[j];
                  if (resid) r += Num<T>::to_f(resid[(size_t)a_idx * p.ldr + n0 + j]);
                  out[(size_t)a_idx * p.ldo + n0 + j] = Num<T>::from_f(r);
                }
              }
            }
          }
        }
      } else
      // four columns per round: all remote loads are issued before the first add
      for (int c0 = (int)crank; c0 < ncols; c0 += 4 * p.splits) {
        float pg[4][8], pu[4][8];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = c0 + q * p.splits;
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            pg[q][s] = 0.f;
            pu[q][s] = 0.f;
            if (s < p.splits && c < ncols && epi) {
              pg[q][s] = ld_dsmem_f32(peer_part[s] + (uint32_t)(c * kBM + tid) * 4u);
              if (DUAL) pu[q][s] = ld_dsmem_f32(peer_part[s] + (uint32_t)((bn + c) * kBM + tid) * 4u);
            }
          }
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = c0 + q * p.splits;
          if (c >= ncols) break;
          float g = 0.f, u = 0.f;
#pragma unroll
          for (int s = 0; s < 8; ++s) {
            g += pg[q][s];
            u += pu[q][s];
          }
          const int tok = SWAP ? (b0 + c) : a_idx;
          const int n = SWAP ? a_idx : (b0 + c);
          if (pub) {
            if (epi) stage_put((c - (int)crank) / p.splits, (tok < M && n < N) ? finish(tok, n, g, u) : 0.f);
          } else {
            float fin = 0.f;                       // the value as stored (0 outside the matrix)
            if (tok < M && n < N) {
              const float v = finish(tok, n, g, u);
              if (p.ar_world > 1) {
                push_partial(tok, n, v);
              } else {
                float r = v;
                if (resid) r += Num<T>::to_f(resid[(size_t)tok * p.ldr + n]);
                const T rt = Num<T>::from_f(r);
                out[(size_t)tok * p.ldo + n] = rt;
                fin = Num<T>::to_f(rt);
              }
            }
            if (emit_ss) ss_add(c, fin);
          }
        }
      }
      if (emit_ss) {
        // the columns this CTA finished (crank, crank + S, ...): one thread each adds the four warps' sums
        __syncthreads();
        for (int c = (int)crank + tid * p.splits; c < ncols; c += (int)blockDim.x * p.splits)
          p.ss_out[(size_t)blockIdx.x * p.ss_ld + b0 + c] = ss_w[0][c] + ss_w[1][c] + ss_w[2][c] + ss_w[3][c];
      }
    }
  } else if (!aborted) {
    for (int c = 0; c < bn; c += 16) {
      uint32_t rg[16], ru[16];
      tmem_ld16(trow + c, rg);
      if (DUAL) tmem_ld16(trow + bn + c, ru);
      tmem_ld_wait();
      float v[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const int tok = SWAP ? (b0 + c + j) : a_idx;
        const int n = SWAP ? a_idx : (b0 + c + j);
        const float vg = __uint_as_float(rg[j]);
        const float vu = DUAL ? __uint_as_float(ru[j]) : 0.f;
        v[j] = (tok < M && n < N) ? finish(tok, n, vg, vu) : 0.f;
      }
      if (p.ar_world > 1 && p.ar_two_shot) {
        // The 16-bit partial of this tile is parked in the operand ring (idle once the accumulator is
        // complete): row r at r * bn elements, its 16-byte chunks XOR-swizzled by r so that both this
        // row-per-thread write and the row-per-warp reads below are free of bank conflicts.  It leaves the
        // CTA as whole rows, because 16-byte stores scattered over 32 rows cross NVLink at a fraction of
        // the link rate.
        if (!SWAP && epi) {
          T* srow = reinterpret_cast<T*>(smem) + (size_t)tid * bn;
          const int cmask = min(bn >> 3, 32) - 1;
          float lo[8], hi[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
          store8(srow + ((((c >> 3)) ^ (tid & cmask)) << 3), lo);
          store8(srow + ((((c >> 3) + 1) ^ (tid & cmask)) << 3), hi);
        }
      } else if (pub) {
        if (epi) {
#pragma unroll
          for (int j = 0; j < 16; ++j) stage_put(c + j, v[j]);
        }
      } else if (p.ar_world > 1) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = SWAP ? (b0 + c + j) : a_idx;
          const int n = SWAP ? a_idx : (b0 + c + j);
          if (tok < M && n < N) push_partial(tok, n, v[j]);
        }
      } else if (SWAP) {
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int tok = b0 + c + j;
          float fin = 0.f;
          if (tok < M && a_idx < N) {
            float r = v[j];
            if (resid) r += Num<T>::to_f(resid[(size_t)tok * p.ldr + a_idx]);
            const T rt = Num<T>::from_f(r);
            out[(size_t)tok * p.ldo + a_idx] = rt;
            fin = Num<T>::to_f(rt);
          }
          if (emit_ss) ss_add(c + j, fin);
        }
        if (emit_ss && c + 16 >= bn) {
          // last column group: one thread per token column adds the four warps' sums
          __syncthreads();
          for (int cc = tid; cc < ncols; cc += (int)blockDim.x)
            p.ss_out[(size_t)blockIdx.x * p.ss_ld + b0 + cc] = ss_w[0][cc] + ss_w[1][cc] + ss_w[2][cc] + ss_w[3][cc];
        }
      } else {
        const int n0 = b0 + c;
        if (a_idx < M) {
          const bool vec = (n0 + 16 <= N) && ((p.ldo & 7) == 0) && (!resid || (p.ldr & 7) == 0);
          if (vec) {
            if (resid) {
              float r0[8], r1[8];
              load8(resid + (size_t)a_idx * p.ldr + n0, r0);
              load8(resid + (size_t)a_idx * p.ldr + n0 + 8, r1);
#pragma unroll
              for (int j = 0; j < 8; ++j) { v[j] += r0[j]; v[8 + j] += r1[j]; }
            }
            float lo[8], hi[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) { lo[j] = v[j]; hi[j] = v[8 + j]; }
            store8(out + (size_t)a_idx * p.ldo + n0, lo);
            store8(out + (size_t)a_idx * p.ldo + n0 + 8, hi);
          } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const int n = n0 + j;
              if (n < N) {
                float r = v[j];
                if (resid) r += Num<T>::to_f(resid[(size_t)a_idx * p.ldr + n]);
                out[(size_t)a_idx * p.ldo + n] = Num<T>::from_f(r);
              }
            }
          }
        }
      }
    }
  }

  if (p.ar_world > 1 && p.ar_two_shot) {
    // Two-shot all-reduce for large M, one output tile per CTA.  Leg 1: every rank copies its 16-bit partial
    // tile (parked in shared memory above) into the buffer of the tile's owner rank.  The owner waits for all
    // ranks, sums in rank order in fp32, adds the residual and writes the finished tile into every rank's
    // result region (leg 2); every rank then copies the tile into its own output.  All global traffic is
    // row-per-warp: the lanes of a warp cover whole rows of the tile with 16 bytes each.
    const int owner = tile_id % p.ar_world;
    const uint32_t want = call + 1u;
    const size_t fbase = ((size_t)tile_id * 8) * p.ar_world;
    const size_t f2 = (size_t)p.ar_flag2_base + tile_id;
    const size_t result_rel = (uint64_t)p.ar_world * M * N * sizeof(T);   // result region, after the partials
    const size_t result_off = slot_off + result_rel;
    const bool vecio = (N & 7) == 0 && (p.ldo & 7) == 0 && (!resid || (p.ldr & 7) == 0);
    const int cpr = bn >> 3;                       // 16-byte chunks per tile row (a power of two, <= 32)
    const int rpi = 32 / cpr;                      // tile rows one warp instruction covers
    const int cmask = cpr - 1;
    const int nwarps = (int)blockDim.x >> 5;
    const int lrow = lane_id() / cpr, lchunk = lane_id() % cpr;
    const int ncol0 = b0 + lchunk * 8;             // first output column of this lane
    const T* tile_s = reinterpret_cast<const T*>(smem);
    __syncthreads();                               // the parked tile is complete
    if (!aborted && !SWAP && ncol0 < N) {
      T* pdst = reinterpret_cast<T*>(owner_buf) + (size_t)p.ar_rank * M * N;
      for (int r0 = warp * rpi; r0 < kBM; r0 += nwarps * rpi) {
        const int r = r0 + lrow, grow = a0 + r;
        if (grow >= M) continue;
        const T* sp = tile_s + (size_t)r * bn + ((lchunk ^ (r & cmask)) << 3);
        T* gp = pdst + (size_t)grow * N + ncol0;
        if (vecio && ncol0 + 8 <= N) {
          *reinterpret_cast<uint4*>(gp) = *reinterpret_cast<const uint4*>(sp);
        } else {
          for (int j = 0; j < 8; ++j)
            if (ncol0 + j < N) gp[j] = sp[j];
        }
      }
    }
    __threadfence_system();
    __syncthreads();
    if (tid == 0 && !aborted) st_release_sys(p.ar_flags[owner] + fbase + p.ar_rank, want);
    if (p.ar_rank == owner) {
      if (tid < p.ar_world && !aborted) {
        if (!wait_flag_ge_sys(p.ar_flags[p.ar_rank] + fbase + tid, want)) {
          report_status(p.status, kStatusPeerTimeout, kTagGemmAr, tid);
          ctl->abort_flag = 1;
        }
      }
      aborted = __syncthreads_or(*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag) != 0);
      if (!aborted && !SWAP && ncol0 < N) {
        const T* part = reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(p.ar_recv[p.ar_rank]) + slot_off);
        for (int r0 = warp * rpi; r0 < kBM; r0 += nwarps * rpi) {
          const int grow = a0 + r0 + lrow;
          if (grow >= M) continue;
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          const bool vec = vecio && ncol0 + 8 <= N;
          if (vec) {
            // every rank's vector (and the residual's) is in flight before the first add
            uint4 raw[8];
#pragma unroll
            for (int rr = 0; rr < 8; ++rr)
              raw[rr] = rr < p.ar_world
                            ? __ldcg(reinterpret_cast<const uint4*>(part + ((size_t)rr * M + grow) * N + ncol0))
                            : make_uint4(0u, 0u, 0u, 0u);
            float r8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            if (resid) load8(resid + (size_t)grow * p.ldr + ncol0, r8);
#pragma unroll
            for (int rr = 0; rr < 8; ++rr) {
              if (rr < p.ar_world) {
                const typename Num<T>::T2* h = reinterpret_cast<const typename Num<T>::T2*>(&raw[rr]);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float2 f = Num<T>::to_f2(h[j]);
                  acc[2 * j] += f.x;
                  acc[2 * j + 1] += f.y;
                }
              }
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += r8[j];
          } else {
            for (int rr = 0; rr < p.ar_world; ++rr) {
              const T* src = part + ((size_t)rr * M + grow) * N + ncol0;
              for (int j = 0; j < 8; ++j)
                if (ncol0 + j < N) acc[j] += Num<T>::to_f(src[j]);
            }
            if (resid) {
              for (int j = 0; j < 8; ++j)
                if (ncol0 + j < N) acc[j] += Num<T>::to_f(resid[(size_t)grow * p.ldr + ncol0 + j]);
            }
          }
#pragma unroll
          for (int dst = 0; dst < 8; ++dst) {
            if (dst < p.ar_world) {
              T* rp = reinterpret_cast<T*>(peer_buf[dst] + result_rel) + (size_t)grow * N + ncol0;
              if (vec) store8(rp, acc);
              else
                for (int j = 0; j < 8; ++j)
                  if (ncol0 + j < N) rp[j] = Num<T>::from_f(acc[j]);
            }
          }
        }
      }
      __threadfence_system();
      __syncthreads();
      if (tid < p.ar_world && !aborted) st_release_sys(p.ar_flags[tid] + f2, want);
    }
    if (tid == 0 && !aborted) {
      if (!wait_flag_ge_sys(p.ar_flags[p.ar_rank] + f2, want)) {
        report_status(p.status, kStatusPeerTimeout, kTagGemmAr, 100 + owner);
        ctl->abort_flag = 1;
      }
    }
    aborted = __syncthreads_or(*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag) != 0);
    if (!aborted && !SWAP && ncol0 < N) {
      const T* res = reinterpret_cast<const T*>(reinterpret_cast<const uint8_t*>(p.ar_recv[p.ar_rank]) + result_off);
      if (vecio && ncol0 + 8 <= N) {
        // four row groups per round: a store to `out` may alias `res` as far as the compiler knows, so a
        // load-store pair per row would run one memory latency at a time
        for (int r0 = warp * rpi; r0 < kBM; r0 += 4 * nwarps * rpi) {
          uint4 t[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int grow = a0 + r0 + q * nwarps * rpi + lrow;
            t[q] = (r0 + q * nwarps * rpi < kBM && grow < M)
                       ? __ldcg(reinterpret_cast<const uint4*>(res + (size_t)grow * N + ncol0)) : make_uint4(0u, 0u, 0u, 0u);
          }
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int grow = a0 + r0 + q * nwarps * rpi + lrow;
            if (r0 + q * nwarps * rpi < kBM && grow < M)
              *reinterpret_cast<uint4*>(out + (size_t)grow * p.ldo + ncol0) = t[q];
          }
        }
      } else {
        for (int r0 = warp * rpi; r0 < kBM; r0 += nwarps * rpi) {
          const int grow = a0 + r0 + lrow;
          if (grow >= M) continue;
          for (int j = 0; j < 8; ++j)
            if (ncol0 + j < N) out[(size_t)grow * p.ldo + ncol0 + j] = res[(size_t)grow * N + ncol0 + j];
        }
      }
    }
    __syncthreads();
    if (tid == 0) {
      const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
      const uint32_t done = atomicAdd(p.ar_state + 1, 1u);
      if (done == total - 1u) {
        p.ar_state[1] = 0u;
        __threadfence();
        p.ar_state[0] = call + 1u;
      }
    }
  } else if (pub) {
    // Publish and exit: copy the staged rows into slot [rank] of every rank's receive buffer, make the copies
    // visible system-wide, bump this rank's arrival counter on every rank.  Nothing here waits for a peer; the
    // reduction, the residual and the following norm belong to rf_ar_consume.
    __syncthreads();                                       // the staging rows are complete
    if (!aborted) {
      const int vpr = pub_f32 ? 32 : 16;                   // 16-byte vectors per staged row
      const int epv = pub_f32 ? 4 : 8;                     // elements per vector
      const int esz = pub_f32 ? 4 : 2;
      const int nfeat = min(kBM, N - a0);                  // valid features of this tile (N % 8 == 0)
      const int nst = p.splits > 1 ? (ncols > (int)crank ? (ncols - (int)crank + p.splits - 1) / p.splits : 0) : ncols;
      for (int idx = tid; idx < nst * vpr; idx += (int)blockDim.x) {
        const int j = idx / vpr, ch = idx - j * vpr;
        if (ch * epv >= nfeat) continue;
        const int tok = b0 + (p.splits > 1 ? (int)crank + j * p.splits : j);
        if (tok >= M) continue;
        const uint4 val = *reinterpret_cast<const uint4*>(pub_stage + ((size_t)j * kBM * esz) + ch * 16);
        const size_t off = (((size_t)p.ar_rank * M + tok) * N + a0) * esz + (size_t)ch * 16;
#pragma unroll
        for (int d = 0; d < 8; ++d)
          if (d < p.ar_world) *reinterpret_cast<uint4*>(peer_buf[d] + off) = val;
      }
    }
    __threadfence_system();
    __syncthreads();
    if (tid < p.ar_world && !aborted) red_release_sys_add(p.ar_flags[tid] + p.ar_cnt_base + p.ar_rank, 1u);
  } else if (p.ar_world > 1) {
    // Publish this CTA's share of the tile to every rank, wait (bounded) for
    // every rank's share, then reduce in rank order and add the residual.
    // Flags are per (tile, cluster rank, source rank) and carry the call number.
    __threadfence_system();
    __syncthreads();
    const uint32_t want = call + 1u;
    const size_t fbase = ((size_t)tile_id * 8 + crank) * p.ar_world;
    if (tid < p.ar_world && !aborted) st_release_sys(p.ar_flags[tid] + fbase + p.ar_rank, want);
    if (tid < p.ar_world && !aborted) {
      if (!wait_flag_ge_sys(p.ar_flags[p.ar_rank] + fbase + tid, want)) {
        report_status(p.status, kStatusPeerTimeout, kTagGemmAr, tid);
        ctl->abort_flag = 1;
      }
    }
    aborted = __syncthreads_or(*reinterpret_cast<volatile int32_t*>(&ctl->abort_flag) != 0);
    if (!aborted) {
      const float* rb = reinterpret_cast<const float*>(
          reinterpret_cast<const uint8_t*>(p.ar_recv[p.ar_rank]) + slot_off);
      const int cstep = p.splits > 1 ? p.splits : 1;
      // the i-th column this CTA pushed: single columns (swap) or groups of eight (tokens on rows)
      auto own_col = [&](int i) -> int {
        return SWAP ? ((int)crank + i * cstep) : ((((int)crank + (i >> 3) * cstep) << 3) + (i & 7));
      };
      // four columns x every rank's partial are in flight before the first add
      for (int i0 = 0; own_col(i0) < ncols; i0 += 4) {
        float v[4][8], rs[4];
        bool ok[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int c = own_col(i0 + q);
          const int tok = SWAP ? (b0 + c) : a_idx;
          const int n = SWAP ? a_idx : (b0 + c);
          ok[q] = c < ncols && tok < M && n < N;
#pragma unroll
          for (int r = 0; r < 8; ++r)
            v[q][r] = (ok[q] && r < p.ar_world) ? __ldcg(rb + ((size_t)r * M + tok) * N + n) : 0.f;
          rs[q] = (ok[q] && resid) ? Num<T>::to_f(resid[(size_t)tok * p.ldr + n]) : 0.f;
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          if (!ok[q]) continue;
          const int c = own_col(i0 + q);
          const int tok = SWAP ? (b0 + c) : a_idx;
          const int n = SWAP ? a_idx : (b0 + c);
          float acc = 0.f;
#pragma unroll
          for (int r = 0; r < 8; ++r) acc += v[q][r];   // rank order; absent ranks contribute +0
          out[(size_t)tok * p.ldo + n] = Num<T>::from_f(acc + rs[q]);
        }
      }
    }
    // the last CTA to finish advances the call counter for the next launch
    __syncthreads();
    if (tid == 0) {
      const uint32_t total = gridDim.x * gridDim.y * gridDim.z;
      const uint32_t done = atomicAdd(p.ar_state + 1, 1u);
      if (done == total - 1u) {
        p.ar_state[1] = 0u;
        __threadfence();
        p.ar_state[0] = call + 1u;
      }
    }
  }
  // peers may still be reading this CTA's partial over DSMEM: a rendezvous without memory ordering (the values read
  // were consumed before the arrive; a release here would make every CTA wait for its output stores to drain)
  if (SWAP && p.splits > 1) cluster_sync_relaxed();   // token-row tiles push: nothing reads a peer after their second rendezvous

  // ----------------------------------------------------------- teardown ----
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
}

// ------------------------------------------------------------ host side ----
struct GemmPlan {
  int swap, bn, splits, stages, tmem_cols, grid_x, grid_y, k_blocks, ctl_offset;
  size_t smem_bytes;
  uint64_t ws_bytes;
  int sem_count;
};

static int plan_gemm(const RfGemm* g, GemmPlan* pl) {
  const bool dual = g->dual_offset > 0;
  pl->k_blocks = ceil_div(g->K, kBK);
  int swap = g->force_swap >= 0 ? g->force_swap : (g->M <= 256 ? 1 : 0);
  if (swap && g->M > 256 && g->force_swap < 0) swap = 0;
  pl->swap = swap;
  if (swap) {
    int bn = g->force_bn > 0 ? g->force_bn : round_up(g->M < 16 ? 16 : g->M, 16);
    if (bn > 256) bn = 256;
    if (dual && bn > 256) bn = 256;
    pl->bn = bn;
    pl->grid_x = ceil_div(g->N, kBM);
    pl->grid_y = ceil_div(g->M, bn);
  } else {
    // 256-wide tiles only where they fill the GPU on their own: with fewer of them than SMs the kernel would split K to
    // make CTAs, and the split-K reduction of a 128 x 256 fp32 tile over distributed shared memory costs more than the
    // operand re-reads that 128-wide tiles add (measured, with a residual epilogue: 968 x 2048 x 2048 42.9 us at 256 x 2
    // splits against 32.3 us at 128 x 2; 968 x 2048 x 16384 113.2 against 97.2; 400 x 1024 x 4096 40.6 against 20.9)
    const bool wide_fills = (long)ceil_div(g->M, kBM) * (g->N / 256) >= sm_count() || (g->ar_world > 1 && g->M > 256);
    int bn = g->force_bn > 0 ? g->force_bn : ((g->N % 256 == 0 && !dual && wide_fills) ? 256 : 128);
    if (g->N < 128 && !g->w_packed) bn = round_up(g->N, 16);
    if (g->w_packed && bn != 128 && bn != 256) bn = 128;   // packed weights come in 128-row blocks
    // a 256-wide tile is two 128-row blocks of the tile-major image: with an odd number of blocks the last tile's second
    // block would lie past the end of the image (a forced width can ask for this; the planner's own choice cannot)
    if (g->w_packed && bn == 256 && ceil_div(dual ? g->dual_offset : g->N, 128) % 2 != 0) bn = 128;
    pl->bn = bn;
    pl->grid_x = ceil_div(g->M, kBM);
    pl->grid_y = ceil_div(g->N, bn);
  }
  pl->tmem_cols = (int)next_pow2((uint32_t)std::max(32, pl->bn * (dual ? 2 : 1)));
  if (pl->tmem_cols > 512) return fail(RF_ERR_BAD_ARG, "accumulator needs %d TMEM columns", pl->tmem_cols);

  const int tiles = pl->grid_x * pl->grid_y;
  const int a_tiles = (swap && dual) ? 2 : 1, b_tiles = (!swap && dual) ? 2 : 1;
  int stage_bytes = a_tiles * kATileBytes + b_tiles * pl->bn * kBK * 2;
  if (g->w_int8) {   // staging tiles of the quantised weights
    const int rows = swap ? kBM : pl->bn;
    stage_bytes += round_up((dual ? 2 : 1) * (g->w_bits == 4 ? ceil_div(rows, kBM) * rf_w4_block_bytes(g->w_group) : rows * kBK), 1024);
  }
  const int ctl_bytes = (int)sizeof(GemmSmemCtl) + 64 + ((g->ss_in || g->ss_out) ? kSsScratchBytes : 0);
  const bool publish = g->ar_world > 1 && g->ar_publish && swap;
  static const int env_smem_kb = [] { const char* e = getenv("RF_GEMM_SMEM_KB"); return e ? atoi(e) : 0; }();

  // shared-memory plan for a given split count and ring budget
  auto layout = [&](int S, int budget, int* stages_out, int* part_out) -> size_t {
    int st = (budget - ctl_bytes) / stage_bytes;
    st = std::min(st, kMaxStages);
    st = std::min(st, std::max(2, ceil_div(pl->k_blocks, S)));
    // the split-K partial ([columns][128] fp32 per accumulator) reuses the stage ring; the publish path parks this
    // CTA's finished rows behind it (peers still read the partial over DSMEM while the rows are pushed)
    // (token-row tiles receive pushed slices: splits x ceil(groups / splits) 8-column groups per accumulator)
    const int part_cols = swap ? pl->bn : ceil_div(ceil_div(pl->bn, 8), S) * 8 * S;
    int part = S > 1 ? part_cols * (dual ? 2 : 1) * kBM * 4 : 0;
    if (S > 1 && publish) part += ceil_div(pl->bn, S) * kBM * (g->M <= RF_AR_F32_MAX_ROWS ? 4 : 2);
    *stages_out = st;
    *part_out = part;
    return (size_t)round_up(std::max(st * stage_bytes, part), 1024) + ctl_bytes;
  };

  // largest dynamic shared memory with which two CTAs share an SM: (228 KB - 1 KB reserved per CTA) / 2
  constexpr int kTwoCtaSmem = 113 * 1024;
  int splits = 1, budget = 224 * 1024;
  const bool two_shot = g->ar_world > 1 && !swap && g->M > 256;   // its epilogue works on whole tiles
  if (g->force_splits > 0) {
    splits = std::min(std::min(g->force_splits, 8), pl->k_blocks);
    if (two_shot) splits = 1;
    int st, part;
    if (layout(splits, kTwoCtaSmem, &st, &part) && st >= 2 && tiles * splits > sm_count()) budget = kTwoCtaSmem;
  } else {
    // Split rule from timing sweeps of decode and mid-size shapes on B200:
    //  * power-of-two cluster sizes only (3 and 6 place badly on the GPCs and cost up to 2x);
    //  * weight-streaming shapes (tokens on the MMA N axis) and 128-wide token-row tiles want about two CTAs per
    //    SM in flight: more splits until tiles * splits would exceed 2 * SMs;
    //  * 256-wide token-row tiles are tensor-core bound and want ONE CTA per SM with a deep ring, so they split
    //    only up to tiles * splits <= SMs (grids beyond that run two CTAs per SM with a two-stage ring each, which
    //    measured faster than one CTA with four stages once there are several waves);
    //  * a small second wave costs less than halving the split (measured), so residency is not required.
    // at least one k block per split: short-K shapes (tensor-parallel out-projections, K = 512) measured 16.3 us
    // unsplit-ish (S <= k_blocks / 4) against 8.8 us at one block per CTA - the fixed cost of a CTA is paid in
    // parallel, its streaming time is not
    const int max_by_k = std::max(1, pl->k_blocks);
    const int cap = (!swap && pl->bn > 128) ? sm_count() : 2 * sm_count();
    splits = 1;
    if (!two_shot) {
      for (int S = 8; S >= 2; S >>= 1) {
        if (S > max_by_k || tiles * S > cap) continue;
        int st, part;
        const int b = tiles * S > sm_count() ? kTwoCtaSmem : 224 * 1024;
        const size_t smem = layout(S, b, &st, &part);
        if (st < 2 || smem > 227 * 1024) continue;
        splits = S;
        break;
      }
    }
    {
      int st, part;
      layout(splits, kTwoCtaSmem, &st, &part);
      budget = (tiles * splits > sm_count() && st >= 2) ? kTwoCtaSmem : 224 * 1024;
    }
  }
  if (env_smem_kb > 0) budget = std::min(224, std::max(48, env_smem_kb)) * 1024;
  pl->splits = splits;
  pl->ws_bytes = 0;
  pl->sem_count = 0;
  int stages, part_bytes;
  size_t smem_total = layout(splits, budget, &stages, &part_bytes);
  if (stages < 2) smem_total = layout(splits, 224 * 1024, &stages, &part_bytes);
  if (stages < 2) return fail(RF_ERR_UNSUPPORTED, "GEMM tile does not fit in shared memory");
  if (smem_total > 227 * 1024) {
    if (g->force_splits > 1) return fail(RF_ERR_UNSUPPORTED, "split-K partial does not fit in shared memory");
    pl->splits = 1;
    smem_total = layout(1, budget, &stages, &part_bytes);
  }
  pl->stages = stages;
  pl->ctl_offset = round_up(std::max(stages * stage_bytes, part_bytes), 1024);
  pl->smem_bytes = (size_t)pl->ctl_offset + ctl_bytes;
  (void)smem_total;
  return RF_OK;
}

// Converter warps per CTA of the quantised kernels (RF_W8_CONV_WARPS: 4 .. 6).  The widening is a chain of shared-memory
// loads, byte permutes and stores; more warps per scheduler hide its latencies.
static int conv_warps() {
  static const int v = [] {
    const char* e = getenv("RF_W8_CONV_WARPS");
    const int n = e ? atoi(e) : 4;
    return std::min(std::max(n, 4), kMaxConvWarps);
  }();
  return v;
}

template <typename T, bool SWAP, bool DUAL, bool W8>
static int launch_gemm(const RfGemm* g, const GemmPlan& pl, cudaStream_t stream) {
  auto kfn = gemm_tc_kernel<T, SWAP, DUAL, W8>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 227 * 1024);
  const bool dual = DUAL;
  const uint64_t w_rows = (uint64_t)(dual ? g->dual_offset + g->N : g->N);
  CUtensorMap tmA, tmB, tmW;
  int rc;
  if (g->w_packed) {
    // only the activations go through a tensor map; the weight blocks are plain bulk copies
    if (SWAP) rc = make_tmap_2d(&tmB, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, pl.bn, true);
    else rc = make_tmap_2d(&tmA, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, kBM, true);
    if (rc) return rc;
    if (SWAP) tmA = tmB; else tmB = tmA;
    tmW = tmA;
  } else if (W8) {
    // int8 weights: their own byte-typed, unswizzled map; the 16-bit map of that operand is unused
    rc = make_tmap_2d(&tmW, g->w, 0, 1, g->K, w_rows, g->ldw, kBK, SWAP ? kBM : pl.bn, false);
    if (rc) return rc;
    if (SWAP) rc = make_tmap_2d(&tmB, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, pl.bn, true);
    else rc = make_tmap_2d(&tmA, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, kBM, true);
    if (rc) return rc;
    if (SWAP) tmA = tmB; else tmB = tmA;
  } else if (SWAP) {
    rc = make_tmap_2d(&tmA, g->w, g->dtype, 2, g->K, w_rows, g->ldw, kBK, kBM, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, pl.bn, true);
    if (rc) return rc;
    tmW = tmA;
  } else {
    rc = make_tmap_2d(&tmA, g->x, g->dtype, 2, g->K, g->M, g->ldx, kBK, kBM, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmB, g->w, g->dtype, 2, g->K, w_rows, g->ldw, kBK, pl.bn, true);
    if (rc) return rc;
    tmW = tmA;
  }
  GemmTcParams p;
  p.out = g->out; p.ldo = g->ldo;
  p.residual = g->residual; p.ldr = g->ldr;
  p.bias = g->bias; p.scale = g->scale; p.row_scale = g->row_scale;
  p.ws = g->ws; p.sem = g->sem; p.status = g->status;
  p.M = g->M; p.N = g->N;
  p.k_blocks = pl.k_blocks; p.splits = pl.splits; p.bn = pl.bn; p.stages = pl.stages; p.ctl_offset = pl.ctl_offset;
  p.act = g->act; p.dual_offset = g->dual_offset; p.tmem_cols = pl.tmem_cols;
  p.ar_world = g->ar_world; p.ar_rank = g->ar_rank;
  p.ar_recv = g->ar_recv; p.ar_flags = g->ar_flags; p.ar_state = g->ar_state;
  p.ar_half_bytes = g->ar_recv_bytes;
  p.w_packed = g->w_packed ? reinterpret_cast<const uint8_t*>(g->w) : nullptr;
  p.kb_total = pl.k_blocks;
  p.dual_tiles = ceil_div(g->N, kBM);
  {
    static const int rot_env = [] { const char* e = getenv("RF_GEMM_K_ROTATE"); return e ? atoi(e) : 1; }();
    p.k_rotate = rot_env;
  }
  p.ar_two_shot = (g->ar_world > 1 && !SWAP && g->M > 256) ? 1 : 0;
  p.ar_flag2_base = g->ar_flag_count / 2;
  p.ar_publish = (g->ar_world > 1 && g->ar_publish && SWAP) ? 1 : 0;
  p.ar_cnt_base = g->ar_cnt_base;
  p.ar_stage_off = pl.splits > 1 ? pl.bn * (DUAL ? 2 : 1) * kBM * 4 : 0;
  p.ss_out = SWAP ? g->ss_out : nullptr;
  p.ss_in = SWAP ? g->ss_in : nullptr;
  p.ss_tiles = g->ss_tiles; p.ss_ld = g->ss_ld;
  p.ss_inv_dim = g->ss_dim > 0 ? 1.f / (float)g->ss_dim : 0.f;
  p.ss_eps = g->ss_eps;
  p.w4 = (W8 && g->w_bits == 4) ? 1 : 0;
  p.w4_ns = p.w4 && g->w_group > 0 ? kBK / std::min(g->w_group, kBK) : 0;
  p.w4_fp4 = p.w4 && g->w_fp4 ? 1 : 0;
  {
    static const int ahead_env = [] { const char* e = getenv("RF_GEMM_PF_AHEAD"); return e ? atoi(e) : 0; }();
    p.pf_ahead = (g->w_packed && SWAP && ahead_env > 0) ? pl.stages + ahead_env - 1 : 0;
    static const int ef_env = [] { const char* e = getenv("RF_GEMM_W_EVICT_FIRST"); return e ? atoi(e) : 1; }();
    p.w_evict_first = (g->w_packed && SWAP && g->M <= 256 && ef_env) ? 1 : 0;
  }
  p.q_blk_bytes = p.w4 ? rf_w4_block_bytes(g->w_group) : kBM * kBK;
  p.pf_ptr = nullptr; p.pf_chunks = 0;
  if (SWAP && g->prefetch && g->prefetch_bytes >= kPrefetchChunk && g->M <= 256 &&
      (reinterpret_cast<uintptr_t>(g->prefetch) & 15u) == 0) {
    p.pf_ptr = reinterpret_cast<const uint8_t*>(g->prefetch);
    p.pf_chunks = (uint32_t)std::min<uint64_t>(g->prefetch_bytes / kPrefetchChunk, 1u << 20);
  }
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(pl.grid_x, pl.grid_y, pl.splits), dim3(W8 ? 128 + 32 * conv_warps() : 128), pl.smem_bytes, stream,
                               pl.splits, tmA, tmB, tmW, p));
  ::rf::count_launch();
  return RF_OK;
}

static int check_gemm(const RfGemm* g) {
  RF_REQUIRE(g != nullptr, "null RfGemm");
  RF_REQUIRE(g->x && g->w && g->out, "GEMM needs x, w and out");
  RF_REQUIRE(g->M > 0 && g->N > 0 && g->K > 0, "GEMM shape %dx%dx%d", g->M, g->N, g->K);
  RF_REQUIRE(g->K % 8 == 0, "GEMM K=%d must be a multiple of 8 (16-byte rows)", g->K);
  RF_REQUIRE(g->ldx % 8 == 0 && (g->w_packed || g->ldw % (g->w_int8 ? 16 : 8) == 0), "GEMM row pitches must be multiples of 16 bytes");
  if (g->w_packed) RF_REQUIRE((reinterpret_cast<uintptr_t>(g->w) & 127) == 0, "packed weights must be 128-byte aligned");
  if (g->ss_in || g->ss_out) {
    RF_REQUIRE(g->M <= 256 && g->force_swap != 0, "folded RMSNorm (ss_in / ss_out) is for at most 256 tokens (got %d)", g->M);
    RF_REQUIRE(g->ss_ld >= g->M, "ss_ld %d is smaller than the token count %d", g->ss_ld, g->M);
    if (g->ss_in) RF_REQUIRE(g->ss_tiles > 0 && g->ss_dim > 0, "ss_in needs ss_tiles and ss_dim");
    if (g->ss_out) RF_REQUIRE(g->ar_world <= 1, "ss_out is not available together with the fused all-reduce");
  }
  if (g->w_bits == 4) {
    RF_REQUIRE(g->w_int8 && g->w_packed, "int4 weights come as the tile-major image (w_int8 = 1, w_packed = 1)");
    RF_REQUIRE(g->w_group == 0 || g->w_group == 32 || g->w_group == 64 || g->w_group == 128 || (g->w_fp4 && g->w_group == 16),
               "4-bit scale group must be 0 (per channel), 32, 64 or 128 (e2m1 codes also 16), got %d", g->w_group);
    RF_REQUIRE(g->w_group > 0 || g->scale != nullptr, "per-channel int4 weights need a scale vector");
    RF_REQUIRE(g->w_group == 0 || g->K % g->w_group == 0, "K=%d is not a multiple of the scale group %d", g->K, g->w_group);
  } else {
    RF_REQUIRE(g->w_bits == 0 || g->w_bits == 8 || g->w_bits == 16, "w_bits must be 0, 4, 8 or 16, got %d", g->w_bits);
    if (g->w_int8) RF_REQUIRE(g->scale != nullptr && g->K % 16 == 0, "int8 weights need a scale vector and K %% 16 == 0");
  }
  RF_REQUIRE(g->dtype == 0 || g->dtype == 1, "GEMM dtype must be fp16 or bf16");
  const bool dual_act = g->act == kActSiluMul || g->act == kActGeluTanhMul;
  RF_REQUIRE(dual_act == (g->dual_offset > 0), "dual_offset and a *_mul activation go together");
  if (g->ar_world > 1) {
    RF_REQUIRE(g->ar_world <= 8 && g->ar_rank >= 0 && g->ar_rank < g->ar_world, "bad ar rank/world");
    RF_REQUIRE(g->ar_recv && g->ar_flags && g->ar_state, "fused all-reduce needs recv/flags/state");
    const uint64_t need = (g->M > 256 && g->force_swap != 1) ? (uint64_t)(g->ar_world + 1) * g->M * g->N * 2
                                     : (uint64_t)g->ar_world * g->M * g->N * sizeof(float);
    RF_REQUIRE(need <= g->ar_recv_bytes, "all-reduce receive buffer too small for %dx%d: need %llu B, have %llu B",
               g->M, g->N, (unsigned long long)need, (unsigned long long)g->ar_recv_bytes);
    if (g->ar_publish) {
      RF_REQUIRE(g->M <= 256 && g->force_swap != 0, "ar_publish is the path for at most 256 tokens (got %d)", g->M);
      RF_REQUIRE(g->N % 8 == 0 && g->dual_offset == 0, "ar_publish needs N %% 8 == 0 and a single accumulator");
      RF_REQUIRE(g->ar_cnt_base >= 0 && g->ar_cnt_base + g->ar_world <= g->ar_flag_count + 64,
                 "ar_publish arrival counters [%d, %d) lie outside the flag array", g->ar_cnt_base,
                 g->ar_cnt_base + g->ar_world);
    }
  }
  return RF_OK;
}

}  // namespace rf

using namespace rf;

extern "C" uint64_t rf_pack_weight_bytes(int64_t rows, int64_t K, int32_t sections, int32_t elem_bytes) {
  if (rows <= 0 || K <= 0 || sections <= 0 || rows % sections) return 0;
  const int64_t tiles = ((rows / sections + kBM - 1) / kBM) * sections, kb = (K + kBK - 1) / kBK;
  return (uint64_t)(tiles * kb) * kBM * kBK * (uint64_t)elem_bytes;
}

namespace rf { void gemm_sk_scratch(const RfGemm* g, uint64_t* ws_bytes, int32_t* flags); }

extern "C" int rf_gemm_scratch(const RfGemm* g, uint64_t* ws_bytes, int32_t* sem_count) {
  int rc = check_gemm(g);
  if (rc) return rc;
  GemmPlan pl;
  rc = plan_gemm(g, &pl);
  if (rc) return rc;
  // the persistent stream-K kernel (small token counts) parks partial tiles in global scratch, one slot and one
  // flag per CTA; a caller that provides them gets that kernel
  uint64_t sk_ws = 0;
  int32_t sk_flags = 0;
  if (!g->w_int8) rf::gemm_sk_scratch(g, &sk_ws, &sk_flags);
  if (ws_bytes) *ws_bytes = std::max<uint64_t>(pl.ws_bytes, sk_ws);
  if (sem_count) *sem_count = std::max<int32_t>(pl.sem_count, sk_flags);
  return RF_OK;
}

// The launch plan rf_gemm / rf_gemm_w8a16 would use for this shape, without launching (host-only; usable without
// a GPU, where 148 SMs are assumed): out = {swap, bn, splits, stages, grid_x, grid_y, shared-memory bytes, k_blocks,
// persistent kernel?, two-shot all-reduce?}.  For tests of the planner's invariants and for diagnostics.
extern "C" int rf_gemm_plan_info(const RfGemm* g, int32_t* out);

namespace rf {
bool gemm_sk_eligible(const RfGemm* g, int* ctas);               // gemm_sk.cu: persistent stream-K kernel for small M
bool gemm_small_eligible(const RfGemm* g);                         // gemm_small.cu: latency-bound shapes (few rows, small weight)
int gemm_small_run(const RfGemm* g, cudaStream_t stream);
void gemm_sk_scratch(const RfGemm* g, uint64_t* ws_bytes, int32_t* flags);
int launch_gemm_sk(const RfGemm* g, cudaStream_t stream);
bool gemm_ps_eligible(const RfGemm* g, bool swap, int splits);   // gemm_ps.cu: persistent kernel for large M
int launch_gemm_ps(const RfGemm* g, cudaStream_t stream);
int widen_packed(const void* src, void* dst, int64_t blocks, int dtype, cudaStream_t stream);   // gemm_ps.cu
}

static int run_gemm(const RfGemm* g, cudaStream_t stream, bool w8) {
  int rc = check_gemm(g);
  if (rc) return rc;
  if (!w8 && rf::gemm_small_eligible(g)) return rf::gemm_small_run(g, stream);      // latency-bound shapes: gemm_small.cu
  if (!w8 && rf::gemm_sk_eligible(g, nullptr)) return rf::launch_gemm_sk(g, stream);
  GemmPlan pl;
  rc = plan_gemm(g, &pl);
  if (rc) return rc;
  if (!w8 && g->force_splits == 0 && g->force_bn == 0 && rf::gemm_ps_eligible(g, pl.swap != 0, pl.splits))
    return rf::launch_gemm_ps(g, stream);
  if (w8 && g->w_bits != 4 && !pl.swap && g->M > 256 && g->w_packed && g->w_scratch && g->force_splits == 0 && g->force_bn == 0) {
    // Large token counts are compute-bound: widen the int8 weight image once into the caller's scratch (a pass
    // over the weights costs a few per cent of the GEMM) and run the 16-bit kernels, whose main loop has no
    // converter stage; the per-channel scale stays in the epilogue, so the result is (X . Q^T) * s as before.
    const int64_t blocks = (int64_t)(g->dual_offset > 0 ? 2 : 1) * ceil_div(g->N, kBM) * ceil_div(g->K, kBK);
    if ((uint64_t)blocks * kATileBytes <= g->w_scratch_bytes) {
      rc = rf::widen_packed(g->w, g->w_scratch, blocks, g->dtype, stream);
      if (rc) return rc;
      RfGemm g2 = *g;
      g2.w = g->w_scratch;
      g2.w_int8 = 0;
      return run_gemm(&g2, stream, false);
    }
  }
  if (g->ar_world > 1)
    RF_REQUIRE(pl.grid_x * pl.grid_y * 8 * g->ar_world <= g->ar_flag_count / 2,
               "all-reduce needs %d flags, have %d", pl.grid_x * pl.grid_y * 8 * g->ar_world, g->ar_flag_count / 2);
  const bool dual = g->dual_offset > 0;
#define RF_GEMM_DISPATCH(T, W8)                                                          \
  if (pl.swap) {                                                                         \
    return dual ? launch_gemm<T, true, true, W8>(g, pl, stream)                          \
                : launch_gemm<T, true, false, W8>(g, pl, stream);                        \
  } else {                                                                               \
    return dual ? launch_gemm<T, false, true, W8>(g, pl, stream)                         \
                : launch_gemm<T, false, false, W8>(g, pl, stream);                       \
  }
  if (w8) {
    if (g->dtype == 0) { RF_GEMM_DISPATCH(__half, true) }
    RF_GEMM_DISPATCH(__nv_bfloat16, true)
  }
  if (g->dtype == 0) { RF_GEMM_DISPATCH(__half, false) }
  RF_GEMM_DISPATCH(__nv_bfloat16, false)
#undef RF_GEMM_DISPATCH
}

extern "C" int rf_gemm_plan_info(const RfGemm* g, int32_t* out) {
  RF_REQUIRE(g && out, "rf_gemm_plan_info: null argument");
  int rc = check_gemm(g);
  if (rc) return rc;
  GemmPlan pl;
  rc = plan_gemm(g, &pl);
  if (rc) return rc;
  out[0] = pl.swap; out[1] = pl.bn; out[2] = pl.splits; out[3] = pl.stages; out[4] = pl.grid_x; out[5] = pl.grid_y;
  out[6] = (int32_t)pl.smem_bytes; out[7] = pl.k_blocks;
  out[8] = (!g->w_int8 && g->force_splits == 0 && g->force_bn == 0 && rf::gemm_ps_eligible(g, pl.swap != 0, pl.splits)) ? 1 : 0;
  if (!g->w_int8 && rf::gemm_sk_eligible(g, nullptr)) out[8] = 2;   // persistent stream-K kernel
  out[9] = (g->ar_world > 1 && !pl.swap && g->M > 256) ? 1 : 0;
  return RF_OK;
}

extern "C" int rf_gemm_grid_ctas(const RfGemm* g) {
  int rc = check_gemm(g);
  if (rc) return rc;
  int sk_ctas = 0;
  if (!g->w_int8 && rf::gemm_sk_eligible(g, &sk_ctas)) return sk_ctas;
  GemmPlan pl;
  rc = plan_gemm(g, &pl);
  if (rc) return rc;
  return pl.grid_x * pl.grid_y * pl.splits;
}

extern "C" int rf_gemm(const RfGemm* g, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(g && !g->w_int8, "rf_gemm takes 16-bit weights; use rf_gemm_w8a16 for int8");
  return run_gemm(g, static_cast<cudaStream_t>(stream), false);
}

// int8 weights [N,K] with a per-output-channel scale: widened to the activation dtype inside the
// mainloop, (X . Q^T) * scale in the epilogue.  Same epilogue options as rf_gemm (bias, residual,
// GLU, cluster split-K, fused all-reduce).
extern "C" int rf_gemm_w8a16(const RfGemm* g, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(g && g->w_int8 && (g->scale || (g->w_bits == 4 && g->w_group > 0)),
             "rf_gemm_w8a16 takes quantised weights and their scales");
  return run_gemm(g, static_cast<cudaStream_t>(stream), true);
}

// int4 weights in the tile-major image (nibbles + in-block group scales, or a per-channel scale vector): the same
// main loop, whose converter warps widen the nibbles and apply the group scale on the way into the 16-bit tile.
extern "C" int rf_gemm_w4a16(const RfGemm* g, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(g && g->w_int8 && g->w_bits == 4, "rf_gemm_w4a16 takes the int4 weight image (w_int8 = 1, w_bits = 4)");
  return run_gemm(g, static_cast<cudaStream_t>(stream), true);
}

extern "C" int32_t rf_w4_block_bytes(int32_t group) {
  return kBM * kBK / 2 + (group > 0 ? kBM * (kBK / std::min(group, kBK)) * 2 : 0);
}

extern "C" uint64_t rf_pack_w4_bytes(int64_t rows, int64_t K, int32_t sections, int32_t group) {
  if (rows <= 0 || K <= 0 || sections <= 0 || rows % sections) return 0;
  const int64_t tiles = ((rows / sections + kBM - 1) / kBM) * sections, kb = (K + kBK - 1) / kBK;
  return (uint64_t)(tiles * kb) * (uint64_t)rf_w4_block_bytes(group);
}
