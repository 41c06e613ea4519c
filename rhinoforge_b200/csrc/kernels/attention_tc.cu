// Flash attention (prefill) on the 5th-generation tensor cores.
//
// One CTA owns 128 query rows of one head.  Both GEMMs of attention run as tcgen05.mma with
// accumulators in tensor memory:
//   S = Q . K^T   A = Q tile  [128 x HD]  (K-major, smem)   B = K tile [KVB x HD] (K-major, smem)   D = S in TMEM
//   O += P . V    A = P tile  [128 x KVB] (K-major, smem)   B = V tile [KVB x HD] (MN-major, smem)  D = O in TMEM
// Warp roles: warp 0 = TMA producer (K/V pages or rows, double buffered), warp 1 = MMA issuer (and
// TMEM owner), warps 2-5 = softmax: thread r owns query row r, which is TMEM lane r, so row max and
// row sum need no shuffles.  S is double buffered in TMEM: Q.K^T of block j+1 runs on the tensor core
// while the softmax warps work on block j.  The running maximum is only raised when a block exceeds
// it by more than 2^8 (the accumulator and the row sum share the stale maximum, so the final
// O / l is exact); raising it rescales the O accumulator in TMEM (tcgen05.ld / tcgen05.st).
// V needs no transpose: the [tokens x 64] slabs a TMA box leaves in shared memory are exactly the
// MN-major 128-byte-swizzle operand layout.
//
// Same contract as the mma.sync kernel in attention.cu (varlen packed q, paged or contiguous KV,
// causal / window / boolean mask / segment ids, GQA).  Every wait is bounded.
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"
#include "attn_params.cuh"

namespace rf {

constexpr int kFaRows = 128;          // query rows per CTA
constexpr int kFaBox = 16 * 128;      // one TMA box: 16 rows x 64 x 16-bit
constexpr int kFaThreads = 192;
constexpr float kFaRaise = 8.0f;      // raise the reference maximum only beyond 2^8

struct alignas(8) FaCtl {
  uint64_t q_full, kv_full[2], kv_empty[2], s_full[2], s_empty[2], p_full, p_empty, o_full;
  uint32_t tmem_base;
  int32_t abort_flag;
};

template <int HD> struct FaGeom {
  static constexpr int J = HD / 64;                      // 64-column chunks of the head dimension
  static constexpr int KVB = 64;                         // kv tokens per block: small enough for TWO CTAs per SM
                                                         // (HD <= 128), whose softmax and MMA phases interleave
  static constexpr int PC = KVB / 64;                    // 64-token chunks of P
  static constexpr int kQBytes = J * kFaRows * 128;
  static constexpr int kKBytes = J * KVB * 128;          // K (and V) of one stage
  static constexpr int kStageBytes = 2 * kKBytes;
  static constexpr int kPBytes = PC * kFaRows * 128;
  static constexpr int kSmem = kQBytes + 2 * kStageBytes + kPBytes;
  static constexpr int kTmemCols = HD == 256 ? 512 : 256; // 2 x KVB (S) + HD (O), rounded up to a power of two
  static constexpr int kOCol = 2 * KVB;
};

template <typename T, int HD>
__global__ void __launch_bounds__(kFaThreads)
attn_prefill_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                       const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using G = FaGeom<HD>;
  constexpr int J = G::J, KVB = G::KVB;
  // No alignment slack: two CTAs of the HD <= 128 configuration fill the SM's shared memory to within 2 KB.
  // The swizzled tiles need a 1024-byte aligned base, which the runtime provides when the kernel has no
  // static shared memory; a misaligned base is reported instead of being used.
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if ((smem_u32(smem_raw) & 1023u) != 0) {
    if (threadIdx.x == 0) report_status(p.status, kStatusBadArgument, kTagAttnPrefill, (int)(smem_u32(smem_raw) & 1023u));
    return;
  }
  uint8_t* qsm = smem;
  uint8_t* kvsm = smem + G::kQBytes;
  uint8_t* psm = kvsm + 2 * G::kStageBytes;
  FaCtl* ctl = reinterpret_cast<FaCtl*>(psm + G::kPBytes);

  const int qt = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qlen = p.q_len[seq];
  if (qt * kFaRows >= qlen) return;                       // before any barrier or allocation
  const int kvlen = p.kv_len[seq];
  const int kvh = h / p.G;
  const int qpos0 = kvlen - qlen;                         // position of query row 0 on the kv axis
  const int q_row0 = p.q_start[seq] + qt * kFaRows;
  const int rows_here = min(kFaRows, qlen - qt * kFaRows);
  int kv_hi = kvlen;
  if (p.causal) kv_hi = min(kvlen, qpos0 + qt * kFaRows + rows_here);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, qpos0 + qt * kFaRows - p.window + 1) & ~(KVB - 1);
  const int nblk = kv_hi > kv_lo ? (kv_hi - kv_lo + KVB - 1) / KVB : 0;

  if (tid == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&ctl->kv_full[s], 1);
      mbar_init(&ctl->kv_empty[s], 1);
      mbar_init(&ctl->s_full[s], 1);
      mbar_init(&ctl->s_empty[s], 4);
    }
    mbar_init(&ctl->p_full, 4);
    mbar_init(&ctl->p_empty, 1);
    mbar_init(&ctl->o_full, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, (uint32_t)G::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = ctl->tmem_base;
  pdl_launch_dependents();     // only after this CTA owns its TMEM columns
  pdl_wait();                  // q, k, v come from the previous kernel
  volatile int32_t* abort_flag = &ctl->abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      mbar_arrive_expect_tx(&ctl->q_full, (uint32_t)G::kQBytes);
#pragma unroll
      for (int c = 0; c < J; ++c)
#pragma unroll
        for (int rg = 0; rg < kFaRows / 16; ++rg)
          tma_load_2d(qsm + c * (kFaRows * 128) + rg * kFaBox, &tmQ, &ctl->q_full, h * HD + c * 64, q_row0 + rg * 16);
      int issued = 0;
      for (int j = 0; j < nblk; ++j) {
        const int s = j & 1;
        const uint32_t ph = (uint32_t)(j >> 1) & 1u;
        if (!mbar_wait(&ctl->kv_empty[s], ph ^ 1u, kLocalWaitNs, 64)) {
          report_status(p.status, kStatusTmaTimeout, kTagAttnPrefill, j);
          ctl->abort_flag = 1;
          break;
        }
        if (*abort_flag) break;
        const int t0 = kv_lo + j * KVB;
        uint8_t* ks = kvsm + (size_t)s * G::kStageBytes;
        uint8_t* vs = ks + G::kKBytes;
        mbar_arrive_expect_tx(&ctl->kv_full[s], (uint32_t)G::kStageBytes);
        // Whole blocks are always loaded: rows past the sequence end are other (finite) cache rows or the
        // zero fill beyond the tensor, and their probabilities are forced to zero.
        for (int w = 0; w < KVB / 16; ++w) {
          int row, col0;
          if (p.paged) {
            const int pi = min((t0 >> 4) + w, p.pt_stride - 1);
            const int page_id = p.page_table[(size_t)seq * p.pt_stride + pi];
            row = (page_id * p.Hkv + kvh) * 16;
            col0 = 0;
          } else {
            row = p.kv_start[seq] + t0 + w * 16;
            col0 = kvh * HD;
          }
#pragma unroll
          for (int c = 0; c < J; ++c) {
            tma_load_2d(ks + c * (KVB * 128) + w * kFaBox, &tmK, &ctl->kv_full[s], col0 + c * 64, row);
            tma_load_2d(vs + c * (KVB * 128) + w * kFaBox, &tmV, &ctl->kv_full[s], col0 + c * 64, row);
          }
        }
        issued = j + 1;
      }
      if (*abort_flag) {   // let every copy that was issued land before the CTA can exit
        mbar_wait(&ctl->q_full, 0, 20ull * 1000 * 1000);
        for (int j = max(0, issued - 2); j < issued; ++j)
          mbar_wait(&ctl->kv_full[j & 1], (uint32_t)(j >> 1) & 1u, 20ull * 1000 * 1000);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------- MMA issuer ----
    if (lane == 0 && nblk > 0) {
      const uint32_t idesc_qk = umma_idesc_f16(kFaRows, KVB, Num<T>::kFmt, 0);
      const uint32_t idesc_pv = umma_idesc_f16(kFaRows, HD, Num<T>::kFmt, 1);
      const uint32_t q_addr = smem_u32(qsm), p_addr = smem_u32(psm);
      bool ok = mbar_wait(&ctl->q_full, 0, kLocalWaitNs, 32);
      auto issue_qk = [&](int j) -> bool {
        const int s = j & 1, b = j & 1;
        if (!mbar_wait(&ctl->kv_full[s], (uint32_t)(j >> 1) & 1u, kLocalWaitNs, 32)) return false;
        if (!mbar_wait(&ctl->s_empty[b], ((uint32_t)(j >> 1) & 1u) ^ 1u, kLocalWaitNs, 32)) return false;
        tc_fence_after_sync();
        const uint32_t k_addr = smem_u32(kvsm + (size_t)s * G::kStageBytes);
#pragma unroll
        for (int c = 0; c < J; ++c)
#pragma unroll
          for (int kk = 0; kk < 4; ++kk)
            umma_f16(tmem_base + (uint32_t)(b * KVB), umma_desc_k128(q_addr + c * (kFaRows * 128) + kk * 32),
                     umma_desc_k128(k_addr + c * (KVB * 128) + kk * 32), idesc_qk, (c | kk) ? 1u : 0u);
        umma_commit(&ctl->s_full[b]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; ok && j < nblk; ++j) {
        if (j + 1 < nblk) ok = issue_qk(j + 1);          // runs while the softmax warps work on block j
        if (!ok) break;
        if (!mbar_wait(&ctl->p_full, (uint32_t)j & 1u, kLocalWaitNs, 32)) { ok = false; break; }
        tc_fence_after_sync();
        const int s = j & 1;
        const uint32_t v_addr = smem_u32(kvsm + (size_t)s * G::kStageBytes + G::kKBytes);
#pragma unroll
        for (int t = 0; t < KVB / 16; ++t)
          umma_f16(tmem_base + (uint32_t)G::kOCol, umma_desc_k128(p_addr + (t >> 2) * (kFaRows * 128) + (t & 3) * 32),
                   umma_desc_mn128(v_addr + t * kFaBox, (uint32_t)(KVB * 128)), idesc_pv, (j | t) ? 1u : 0u);
        umma_commit(&ctl->kv_empty[s]);
        umma_commit(&ctl->p_empty);
        if (j + 1 == nblk) umma_commit(&ctl->o_full);
      }
      if (!ok) {
        if (!*abort_flag) report_status(p.status, kStatusMmaTimeout, kTagAttnPrefill, 1000);
        ctl->abort_flag = 1;
      }
    }
  } else {
    // ------------------------------------------------- softmax / correction / epilogue ----
    const int quarter = warp & 3;                         // TMEM lanes this warp may touch
    const int r = quarter * 32 + lane;                    // query row of this thread inside the tile
    const int qi = qt * kFaRows + r;                      // row index inside the sequence
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint8_t* mrow = p.mask ? p.mask + (size_t)seq * p.mask_seq_stride + (size_t)min(qi, qlen - 1) * p.mask_ld : nullptr;
    const int sq = (p.seg_q && qi < qlen) ? p.seg_q[p.q_start[seq] + qi] : 0;
    const int kv0 = p.paged ? 0 : p.kv_start[seq];
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    uint8_t* prow = psm + r * 128;
    // bounds of the valid kv positions of this row that do not depend on data: [lo, hi]
    const int hi_row = min(kvlen - 1, p.causal ? qpos0 + qi : 0x7fffffff);
    const int lo_row = p.window > 0 ? qpos0 + qi - p.window + 1 : 0;
    const bool data_mask = mrow != nullptr || p.seg_q != nullptr;
    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      if (!mbar_wait(&ctl->s_full[b], (uint32_t)(j >> 1) & 1u) || *abort_flag) { ok = false; break; }
      tc_fence_after_sync();
      const int t0 = kv_lo + j * KVB;
      const uint32_t s_addr = lane_base + (uint32_t)(b * KVB);
      // the whole row of S for this block: all loads in flight, one wait
      uint32_t sv[KVB];
#pragma unroll
      for (int c0 = 0; c0 < KVB; c0 += 32) tmem_ld32(s_addr + c0, *reinterpret_cast<uint32_t(*)[32]>(&sv[c0]));
      tmem_ld_wait();
      // S[b] may now be overwritten by Q.K^T of block j+2
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->s_empty[b]);
      // masking: interior blocks need none; edge blocks compare against the row's [lo, hi]; boolean
      // masks and segment ids (rare) take the per-element path
      const bool edge = __any_sync(0xffffffffu, t0 < lo_row || t0 + KVB - 1 > hi_row) || data_mask;
      float mx = -INFINITY;
      if (!edge) {
#pragma unroll
        for (int i = 0; i < KVB; ++i) {
          const float v = __uint_as_float(sv[i]) * p.scale_log2;
          sv[i] = __float_as_uint(v);
          mx = fmaxf(mx, v);
        }
      } else if (mrow != nullptr && p.seg_q == nullptr && ((reinterpret_cast<uintptr_t>(mrow) + (uintptr_t)t0) & 15u) == 0 &&
                 t0 + KVB <= p.mask_ld) {
        // boolean mask, 16-byte aligned and wholly inside the row: the block's KVB mask bytes come as 16-byte
        // loads that are all in flight at once (byte loads chained behind the range test cost a cache round
        // trip each and made a 31 x 331 problem take 60 us)
        uint4 mv[KVB / 16];
        const uint4* m16 = reinterpret_cast<const uint4*>(mrow + t0);
#pragma unroll
        for (int c = 0; c < KVB / 16; ++c) mv[c] = __ldg(m16 + c);
#pragma unroll
        for (int i = 0; i < KVB; ++i) {
          const int tk = t0 + i;
          const uint32_t word = reinterpret_cast<const uint32_t*>(&mv[i >> 4])[(i >> 2) & 3];
          const bool v = tk >= lo_row && tk <= hi_row && ((word >> ((i & 3) * 8)) & 0xffu) != 0;
          const float x = v ? __uint_as_float(sv[i]) * p.scale_log2 : -INFINITY;
          sv[i] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      } else {
#pragma unroll
        for (int i = 0; i < KVB; ++i) {
          const int tk = t0 + i;
          bool v = tk >= lo_row && tk <= hi_row;
          if (data_mask && v) {
            if (mrow) v = mrow[tk] != 0;
            if (p.seg_q && v) v = p.seg_k[kv0 + tk] == sq;
          }
          const float x = v ? __uint_as_float(sv[i]) * p.scale_log2 : -INFINITY;
          sv[i] = __float_as_uint(x);
          mx = fmaxf(mx, x);
        }
      }
      // P and O belong to the tensor core until P.V of the previous block has finished
      if (j > 0 && !mbar_wait(&ctl->p_empty, (uint32_t)(j - 1) & 1u)) { ok = false; break; }
      tc_fence_after_sync();
      const bool raise = mx > m_ref + kFaRaise || (m_ref == -INFINITY && mx > -INFINITY);
      if (__any_sync(0xffffffffu, raise)) {               // tcgen05.ld/st are warp-wide
        const float m_new = raise ? mx : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
        if (j > 0) {
#pragma unroll 1
          for (int c0 = 0; c0 < HD; c0 += 32) {
            uint32_t ov[32];
            tmem_ld32(lane_base + (uint32_t)(G::kOCol + c0), ov);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * (raise ? alpha : 1.f));
            tmem_st32(lane_base + (uint32_t)(G::kOCol + c0), ov);
          }
          tmem_st_wait();
        }
        if (raise) {
          l *= alpha;
          m_ref = m_new;
        }
      }
      // probabilities against the reference maximum -> 16-bit P tile (K-major, 128-byte swizzle)
      const float mref = m_ref == -INFINITY ? 0.f : m_ref;
      float rs = 0.f;
#pragma unroll
      for (int u = 0; u < KVB / 8; ++u) {                 // 16-byte units of 8 values
        float f8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          f8[i] = exp2f(__uint_as_float(sv[u * 8 + i]) - mref);   // masked entries are -inf -> 0
          rs += f8[i];
        }
        uint8_t* chunk_base = prow + (u >> 3) * (kFaRows * 128);
        store8(reinterpret_cast<T*>(chunk_base + (((u & 7) ^ (r & 7)) << 4)), f8);
      }
      l += rs;
      // P (and a rescaled O) are ready for the tensor core
      tc_fence_before_sync();
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->p_full);
    }
    // epilogue: O / l
    if (ok && nblk > 0) ok = mbar_wait(&ctl->o_full, 0);
    if (!ok) {
      if (!*abort_flag) report_status(p.status, kStatusEpilogueTimeout, kTagAttnPrefill, r);
      ctl->abort_flag = 1;
    }
    tc_fence_after_sync();
    if (ok) {
      const float inv = l > 0.f ? 1.f / l : 0.f;
      T* orow = reinterpret_cast<T*>(p.out) + (size_t)(p.q_start[seq] + qi) * p.ldo + (size_t)h * HD;
#pragma unroll 1
      for (int c0 = 0; c0 < HD; c0 += 32) {
        uint32_t ov[32];
        if (nblk > 0) {
          tmem_ld32(lane_base + (uint32_t)(G::kOCol + c0), ov);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) ov[i] = 0u;
        }
        if (qi < qlen) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            float f8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) f8[i] = __uint_as_float(ov[u * 8 + i]) * inv;
            store8(orow + c0 + u * 8, f8);
          }
        }
      }
    }
  }
  // ----------------------------------------------------------------- teardown ----
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, (uint32_t)G::kTmemCols);
}

template <typename T, int HD>
static int launch_prefill_tc_t(const RfAttn* a, const AttnParams& p, cudaStream_t s) {
  using G = FaGeom<HD>;
  CUtensorMap tmQ, tmK, tmV;
  int rc;
  if (a->k_pool) {
    const uint64_t rows = (uint64_t)a->pool_pages * a->Hkv * 16;
    rc = make_tmap_2d(&tmK, a->k_pool, a->dtype, 2, a->hd, rows, a->hd, 64, 16, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmV, a->v_pool, a->dtype, 2, a->hd, rows, a->hd, 64, 16, true);
  } else {
    rc = make_tmap_2d(&tmK, a->k, a->dtype, 2, (uint64_t)a->Hkv * a->hd, a->kv_rows_total, a->ldk, 64, 16, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tmV, a->v, a->dtype, 2, (uint64_t)a->Hkv * a->hd, a->kv_rows_total, a->ldv, 64, 16, true);
  }
  if (rc) return rc;
  rc = make_tmap_2d(&tmQ, a->q, a->dtype, 2, (uint64_t)a->Hq * a->hd, a->q_rows_total, a->ldq, 64, 16, true);
  if (rc) return rc;
  const size_t smem = (size_t)G::kSmem + sizeof(FaCtl);
  auto kfn = attn_prefill_tc_kernel<T, HD>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 227 * 1024);
  dim3 grid(ceil_div(a->max_q_len, kFaRows), a->Hq, a->num_seqs);
  RF_CUDA_CHECK(::rf::launch_k(kfn, grid, dim3(kFaThreads), smem, s, 1, tmQ, tmK, tmV, p));
  ::rf::count_launch();
  return RF_OK;
}

// Entry used by rf_attn_prefill (attention.cu): `p` is already filled from `a`.
int launch_prefill_tc(const RfAttn* a, const AttnParams& p, cudaStream_t s) {
  RF_REQUIRE(a->q_start && a->q_len && a->max_q_len > 0 && a->q_rows_total > 0,
             "prefill attention needs q_start, q_len, max_q_len, q_rows_total");
  if (a->dtype == 0) {
    if (a->hd == 64) return launch_prefill_tc_t<__half, 64>(a, p, s);
    if (a->hd == 128) return launch_prefill_tc_t<__half, 128>(a, p, s);
    return launch_prefill_tc_t<__half, 256>(a, p, s);
  }
  if (a->hd == 64) return launch_prefill_tc_t<__nv_bfloat16, 64>(a, p, s);
  if (a->hd == 128) return launch_prefill_tc_t<__nv_bfloat16, 128>(a, p, s);
  return launch_prefill_tc_t<__nv_bfloat16, 256>(a, p, s);
}

}  // namespace rf
