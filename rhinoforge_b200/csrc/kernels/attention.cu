// Attention for sm_100a: flash-style prefill and split-KV paged decode.
//
// K and V arrive by TMA (cp.async.bulk.tensor.2d, 128-byte swizzle) in blocks
// of 16 tokens x 64 head-dim elements -- exactly one KV page (16 tokens) of the
// paged pool, or 16 rows of a contiguous [tokens, heads*hd] buffer (vision
// towers) -- into a multi-stage shared-memory ring guarded by mbarriers; a
// dedicated producer warp issues the copies.  Four consumer warps run
// m16n8k16 tensor-core MMAs with fp32 online softmax.
//
//  * prefill: one CTA per (64 query rows, q head, sequence); causal,
//    bidirectional, sliding-window, boolean 2-D mask and segment-id (block
//    diagonal / packed images) masking; GQA by kv head = q head / group.
//  * decode: one CTA per (KV split, kv head, sequence); the GQA group's query
//    heads are the MMA rows, every consumer warp owns one page per stage, warps
//    and splits are merged with log-sum-exp weights.
//
// Replaces llm_fp16_32b_prefill_flash_attn_univ_* and its vctxlen / minibatch
// variants (src/ops/rpu_sdpa.cpp:30-37,202-203, src/ops/rpu_sdpa_vctxlen.cpp,
// src/ops/rpu_sdpa_minibatch.cpp) and the per-sequence decode SDPA loop
// (src/fused/rpu_qwen3_model.h:3504-3513).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/mma.cuh"
#include "../common/ptx.cuh"
#include "../rf_api.h"
#include "attn_params.cuh"

namespace rf {

constexpr int kAttnMaxStages = 4;
constexpr int kBoxBytes = 16 * 128;  // one TMA box: 16 rows x 64 x 16-bit

struct alignas(8) AttnCtl {
  uint64_t full[kAttnMaxStages];
  uint64_t empty[kAttnMaxStages];
  uint64_t qbar;
  int32_t abort_flag;
};

// STREAM: the page is read once in this launch (decode): it takes the L2 evict-first policy, so that a step's KV
// traffic does not push the activations and the next kernel's first weight blocks out of L2.
template <int HD, bool STREAM = false>
__device__ __forceinline__ void load_kv_page(const CUtensorMap* tmK, const CUtensorMap* tmV,
                                             uint8_t* page_smem, uint64_t* bar, int col0, int row) {
  constexpr int J = HD / 64;
  uint64_t pol = 0;
  if (STREAM) pol = l2_policy_evict_first();
#pragma unroll
  for (int j = 0; j < J; ++j) {
    if (STREAM) {
      tma_load_2d_hint(page_smem + j * kBoxBytes, tmK, bar, col0 + j * 64, row, pol);
      tma_load_2d_hint(page_smem + (J + j) * kBoxBytes, tmV, bar, col0 + j * 64, row, pol);
    } else {
      tma_load_2d(page_smem + j * kBoxBytes, tmK, bar, col0 + j * 64, row);
      tma_load_2d(page_smem + (J + j) * kBoxBytes, tmV, bar, col0 + j * 64, row);
    }
  }
}

// S[16 rows x 16 tokens] += Qfrag(ks) . K_page^T for one k-step.
template <typename T>
__device__ __forceinline__ void qk_step(float (&s0)[4], float (&s1)[4], const uint32_t (&qf)[4],
                                        uint32_t kbase, int ks, int lane) {
  const int mi = lane >> 3, r8 = lane & 7;
  const int row = ((mi >> 1) << 3) + r8;
  const int chunk = ks * 2 + (mi & 1);
  uint32_t b0, b1, b2, b3;
  ldsm_x4(swz128(kbase + (chunk >> 3) * kBoxBytes, row, chunk & 7), b0, b1, b2, b3);
  MmaOp<T>::mma(s0, qf, b0, b1);
  MmaOp<T>::mma(s1, qf, b2, b3);
}

// O[16 rows x HD] += P[16 x 16 tokens] . V_page
template <typename T, int HD>
__device__ __forceinline__ void pv_page(float (&o)[HD / 8][4], const uint32_t (&pf)[4],
                                        uint32_t vbase, int lane) {
  const int mi = lane >> 3, r8 = lane & 7;
  const int row = ((mi & 1) << 3) + r8;
#pragma unroll
  for (int pair = 0; pair < HD / 16; ++pair) {
    const int chunk = pair * 2 + (mi >> 1);
    uint32_t b0, b1, b2, b3;
    ldsm_x4_t(swz128(vbase + (chunk >> 3) * kBoxBytes, row, chunk & 7), b0, b1, b2, b3);
    MmaOp<T>::mma(o[pair * 2], pf, b0, b1);
    MmaOp<T>::mma(o[pair * 2 + 1], pf, b2, b3);
  }
}

// ------------------------------------------------------------------ decode --
template <typename T, int HD>
__global__ void __launch_bounds__(160)
attn_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const AttnParams p) {
  pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  constexpr int kPageBytes = 2 * (HD / 64) * kBoxBytes;
  constexpr int kStageBytes = 4 * kPageBytes;
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(smem + (size_t)p.stages * kStageBytes);

  const int split = blockIdx.x, kvh = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvlen = p.kv_len[seq];
  const int total_pages = (kvlen + 15) >> 4;
  const int pg_begin = split * p.pages_per_split;
  const int pg_end = min(total_pages, pg_begin + p.pages_per_split);
  const int npg = max(0, pg_end - pg_begin);
  const int iters = (npg + 3) >> 2;
  const int G = p.G;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 4);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  __syncthreads();

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[HD / 8][4];
#pragma unroll
  for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }

  if (warp == 4) {
    if (lane == 0) {
      for (int it = 0; it < iters; ++it) {
        const int s = it % p.stages;
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(&ctl->empty[s], ph ^ 1u)) {
          report_status(p.status, kStatusTmaTimeout, kTagAttnDecode, it);
          ctl->abort_flag = 1;
          break;
        }
        const int nvalid = min(4, npg - it * 4);
        mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)(nvalid * kPageBytes));
        for (int w = 0; w < nvalid; ++w) {
          const int pg = pg_begin + it * 4 + w;
          int row, col0;
          if (p.paged) {
            const int page_id = p.page_table[(size_t)seq * p.pt_stride + pg];
            row = (page_id * p.Hkv + kvh) * 16;
            col0 = 0;
          } else {
            row = p.kv_start[seq] + pg * 16;
            col0 = kvh * HD;
          }
          if (p.kv_stream)
            load_kv_page<HD, true>(&tmK, &tmV, smem + (size_t)s * kStageBytes + w * kPageBytes, &ctl->full[s], col0, row);
          else
            load_kv_page<HD>(&tmK, &tmV, smem + (size_t)s * kStageBytes + w * kPageBytes, &ctl->full[s], col0, row);
        }
      }
    }
  } else {
    // query fragments of this kv head's group: row g = lane/4 (and g + 8)
    uint32_t qf[HD / 16][4];
    {
      const int g0 = lane >> 2, g1 = g0 + 8;
      const T* qbase = reinterpret_cast<const T*>(p.q) + (size_t)seq * p.ldq + (size_t)kvh * G * HD;
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int col = ks * 16 + (lane & 3) * 2;
        qf[ks][0] = g0 < G ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g0 * HD + col) : 0u;
        qf[ks][1] = g1 < G ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g1 * HD + col) : 0u;
        qf[ks][2] = g0 < G ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g0 * HD + col + 8) : 0u;
        qf[ks][3] = g1 < G ? *reinterpret_cast<const uint32_t*>(qbase + (size_t)g1 * HD + col + 8) : 0u;
      }
    }
    for (int it = 0; it < iters; ++it) {
      const int s = it % p.stages;
      const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
      if (!mbar_wait(&ctl->full[s], ph)) {
        report_status(p.status, kStatusMmaTimeout, kTagAttnDecode, it);
        ctl->abort_flag = 1;
        break;
      }
      const int pgl = it * 4 + warp;
      if (pgl < npg) {
        const uint32_t kbase = smem_u32(smem + (size_t)s * kStageBytes + warp * kPageBytes);
        const uint32_t vbase = kbase + (HD / 64) * kBoxBytes;
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) qk_step<T>(s0, s1, qf[ks], kbase, ks, lane);
        const int tok0 = (pg_begin + pgl) * 16 + (lane & 3) * 2;
        float x[2][4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t0 = tok0 + (e & 1), t1 = tok0 + 8 + (e & 1);
          x[0][e] = t0 < kvlen ? s0[e] * p.scale_log2 : -INFINITY;
          x[1][e] = t1 < kvlen ? s1[e] * p.scale_log2 : -INFINITY;
        }
        const float mx0 = quad_max(fmaxf(fmaxf(x[0][0], x[0][1]), fmaxf(x[1][0], x[1][1])));
        const float mx1 = quad_max(fmaxf(fmaxf(x[0][2], x[0][3]), fmaxf(x[1][2], x[1][3])));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
        const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
        m0 = mn0; m1 = mn1;
        float pr[2][4];
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
          pr[nt][0] = exp2f(x[nt][0] - ms0); pr[nt][1] = exp2f(x[nt][1] - ms0);
          pr[nt][2] = exp2f(x[nt][2] - ms1); pr[nt][3] = exp2f(x[nt][3] - ms1);
        }
        l0 = l0 * a0 + pr[0][0] + pr[0][1] + pr[1][0] + pr[1][1];
        l1 = l1 * a1 + pr[0][2] + pr[0][3] + pr[1][2] + pr[1][3];
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
        uint32_t pf[4];
        pf[0] = MmaOp<T>::pack(pr[0][0], pr[0][1]);
        pf[1] = MmaOp<T>::pack(pr[0][2], pr[0][3]);
        pf[2] = MmaOp<T>::pack(pr[1][0], pr[1][1]);
        pf[3] = MmaOp<T>::pack(pr[1][2], pr[1][3]);
        pv_page<T, HD>(o, pf, vbase, lane);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->empty[s]);
    }
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);
  }
  __syncthreads();  // every issued copy has landed and been consumed

  // merge the four warps (stage memory is free now)
  float* mo = reinterpret_cast<float*>(smem);            // [4][16][HD]
  float* mm = mo + 4 * 16 * HD;                          // [4][16]
  float* ml = mm + 4 * 16;                               // [4][16]
  if (warp < 4) {
    const int r0 = lane >> 2, r1 = r0 + 8, c = (lane & 3) * 2;
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) {
      float* d0 = mo + ((size_t)warp * 16 + r0) * HD + i * 8 + c;
      float* d1 = mo + ((size_t)warp * 16 + r1) * HD + i * 8 + c;
      d0[0] = o[i][0]; d0[1] = o[i][1];
      d1[0] = o[i][2]; d1[1] = o[i][3];
    }
    if ((lane & 3) == 0) {
      mm[warp * 16 + r0] = m0; mm[warp * 16 + r1] = m1;
      ml[warp * 16 + r0] = l0; ml[warp * 16 + r1] = l1;
    }
  }
  __syncthreads();
  if (ctl->abort_flag) {
    // A bounded wait ran out (the status word says where).  The merge pass still runs after this kernel, so this
    // CTA's slots must not keep an earlier call's partials: mark them empty (weight 0 in the merge).
    if (p.splits > 1) {
      for (int idx = tid; idx < G * HD; idx += blockDim.x) {
        const int g = idx / HD, col = idx % HD;
        const size_t base = ((size_t)seq * p.Hq + (size_t)kvh * G + g) * p.splits + split;
        p.ws_o[base * HD + col] = 0.f;
        if (col == 0) p.ws_lse[base] = -INFINITY;
      }
    }
    return;
  }
  for (int idx = tid; idx < G * HD; idx += blockDim.x) {
    const int g = idx / HD, col = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, mm[w * 16 + g]);
    float num = 0.f, den = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float f = exp2f(mm[w * 16 + g] - M);
        num += f * mo[((size_t)w * 16 + g) * HD + col];
        den += f * ml[w * 16 + g];
      }
    }
    const float val = den > 0.f ? num / den : 0.f;
    const int head = kvh * G + g;
    if (p.splits == 1) {
      reinterpret_cast<T*>(p.out)[(size_t)seq * p.ldo + (size_t)head * HD + col] = Num<T>::from_f(val);
    } else {
      const size_t base = ((size_t)seq * p.Hq + head) * p.splits + split;
      p.ws_o[base * HD + col] = val;
      if (col == 0) p.ws_lse[base] = den > 0.f ? M + log2f(den) : -INFINITY;
    }
  }
}

template <typename T>
__global__ void attn_decode_combine_kernel(const float* __restrict__ ws_o,
                                           const float* __restrict__ ws_lse, T* __restrict__ out,
                                           int64_t ldo, int Hq, int hd, int splits) {
  pdl_prologue();
  const int head = blockIdx.x, seq = blockIdx.y;
  const size_t base = ((size_t)seq * Hq + head) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, ws_lse[base + s]);
  for (int col = threadIdx.x; col < hd; col += blockDim.x) {
    float num = 0.f, den = 0.f;
    if (M != -INFINITY) {
      for (int s = 0; s < splits; ++s) {
        const float f = exp2f(ws_lse[base + s] - M);
        num += f * ws_o[(base + s) * hd + col];
        den += f;
      }
    }
    out[(size_t)seq * ldo + (size_t)head * hd + col] = Num<T>::from_f(den > 0.f ? num / den : 0.f);
  }
}

// ----------------------------------------------------------------- prefill --
template <typename T, int HD>
__global__ void __launch_bounds__(160)
attn_prefill_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  pdl_prologue();
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
  constexpr int J = HD / 64;
  constexpr int kPageBytes = 2 * J * kBoxBytes;
  constexpr int kStageBytes = 4 * kPageBytes;
  constexpr int kQBytes = 4 * J * kBoxBytes;
  uint8_t* qsm = smem;
  uint8_t* kvsm = smem + kQBytes;
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(kvsm + (size_t)p.stages * kStageBytes);

  const int qt = blockIdx.x, h = blockIdx.y, seq = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int qlen = p.q_len[seq];
  if (qt * 64 >= qlen) return;
  const int kvlen = p.kv_len[seq];
  const int kvh = h / p.G;
  const int qpos0 = kvlen - qlen;
  const int q_row0 = p.q_start[seq] + qt * 64;
  const int rows_here = min(64, qlen - qt * 64);
  int kv_hi = kvlen;
  if (p.causal) kv_hi = min(kvlen, qpos0 + qt * 64 + rows_here);
  int kv_lo = 0;
  if (p.window > 0) kv_lo = max(0, (qpos0 + qt * 64 - p.window + 1)) & ~63;
  const int nblk = kv_hi > kv_lo ? (kv_hi - kv_lo + 63) >> 6 : 0;

  if (tid == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 4);
    }
    mbar_init(&ctl->qbar, 1);
    ctl->abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  __syncthreads();

  if (warp == 4) {
    if (lane == 0) {
      mbar_arrive_expect_tx(&ctl->qbar, (uint32_t)kQBytes);
#pragma unroll
      for (int rg = 0; rg < 4; ++rg)
#pragma unroll
        for (int j = 0; j < J; ++j)
          tma_load_2d(qsm + (rg * J + j) * kBoxBytes, &tmQ, &ctl->qbar, h * HD + j * 64, q_row0 + rg * 16);
      for (int it = 0; it < nblk; ++it) {
        const int s = it % p.stages;
        const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
        if (!mbar_wait(&ctl->empty[s], ph ^ 1u)) {
          report_status(p.status, kStatusTmaTimeout, kTagAttnPrefill, it);
          ctl->abort_flag = 1;
          break;
        }
        const int t0 = kv_lo + it * 64;
        const int nvalid = min(4, (kv_hi - t0 + 15) >> 4);
        mbar_arrive_expect_tx(&ctl->full[s], (uint32_t)(nvalid * kPageBytes));
        for (int w = 0; w < nvalid; ++w) {
          int row, col0;
          if (p.paged) {
            const int page_id = p.page_table[(size_t)seq * p.pt_stride + ((t0 >> 4) + w)];
            row = (page_id * p.Hkv + kvh) * 16;
            col0 = 0;
          } else {
            row = p.kv_start[seq] + t0 + w * 16;
            col0 = kvh * HD;
          }
          load_kv_page<HD>(&tmK, &tmV, kvsm + (size_t)s * kStageBytes + w * kPageBytes, &ctl->full[s],
                           col0, row);
        }
      }
    }
  } else {
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    bool ok = mbar_wait(&ctl->qbar, 0);
    if (!ok) {
      report_status(p.status, kStatusMmaTimeout, kTagAttnPrefill, -1);
      ctl->abort_flag = 1;
    }
    const int qi0 = qt * 64 + warp * 16 + (lane >> 2), qi1 = qi0 + 8;
    const uint32_t qwarp = smem_u32(qsm) + warp * J * kBoxBytes;
    const uint8_t* mrow0 = p.mask ? p.mask + (size_t)seq * p.mask_seq_stride + (size_t)qi0 * p.mask_ld : nullptr;
    const uint8_t* mrow1 = p.mask ? p.mask + (size_t)seq * p.mask_seq_stride + (size_t)qi1 * p.mask_ld : nullptr;
    const int sq0 = (p.seg_q && qi0 < qlen) ? p.seg_q[p.q_start[seq] + qi0] : 0;
    const int sq1 = (p.seg_q && qi1 < qlen) ? p.seg_q[p.q_start[seq] + qi1] : 0;
    const int kv0 = p.paged ? 0 : p.kv_start[seq];

    for (int it = 0; ok && it < nblk; ++it) {
      const int s = it % p.stages;
      const uint32_t ph = (uint32_t)(it / p.stages) & 1u;
      if (!mbar_wait(&ctl->full[s], ph)) {
        report_status(p.status, kStatusMmaTimeout, kTagAttnPrefill, it);
        ctl->abort_flag = 1;
        break;
      }
      const int t0 = kv_lo + it * 64;
      const int nvalid = min(4, (kv_hi - t0 + 15) >> 4);
      const uint32_t stage = smem_u32(kvsm + (size_t)s * kStageBytes);
      float sc[8][4];
#pragma unroll
      for (int i = 0; i < 8; ++i) { sc[i][0] = sc[i][1] = sc[i][2] = sc[i][3] = 0.f; }
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        uint32_t qf[4];
        {
          const int mi = lane >> 3, r8 = lane & 7;
          const int row = ((mi & 1) << 3) + r8;
          const int chunk = ks * 2 + (mi >> 1);
          ldsm_x4(swz128(qwarp + (chunk >> 3) * kBoxBytes, row, chunk & 7), qf[0], qf[1], qf[2], qf[3]);
        }
#pragma unroll
        for (int pi = 0; pi < 4; ++pi)
          if (pi < nvalid) qk_step<T>(sc[2 * pi], sc[2 * pi + 1], qf, stage + pi * kPageBytes, ks, lane);
      }
      // mask + online softmax over this block of 64 tokens
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tk = t0 + nt * 8 + (lane & 3) * 2 + (e & 1);
          const int qi = (e < 2) ? qi0 : qi1;
          bool valid = (nt >> 1) < nvalid && tk < kvlen;
          if (p.causal) valid = valid && tk <= qpos0 + qi;
          if (p.window > 0) valid = valid && tk > qpos0 + qi - p.window;
          if (p.mask && valid && qi < qlen) valid = ((e < 2) ? mrow0 : mrow1)[tk] != 0;
          if (p.seg_q && valid) valid = p.seg_k[kv0 + tk] == ((e < 2) ? sq0 : sq1);
          const float v = valid ? sc[nt][e] * p.scale_log2 : -INFINITY;
          sc[nt][e] = v;
          if (e < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
        }
      }
      mx0 = quad_max(mx0);
      mx1 = quad_max(mx1);
      const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
      const float ms0 = mn0 == -INFINITY ? 0.f : mn0, ms1 = mn1 == -INFINITY ? 0.f : mn1;
      const float a0 = exp2f(m0 - ms0), a1 = exp2f(m1 - ms1);
      m0 = mn0; m1 = mn1;
      float rs0 = 0.f, rs1 = 0.f;
#pragma unroll
      for (int nt = 0; nt < 8; ++nt) {
        sc[nt][0] = exp2f(sc[nt][0] - ms0); sc[nt][1] = exp2f(sc[nt][1] - ms0);
        sc[nt][2] = exp2f(sc[nt][2] - ms1); sc[nt][3] = exp2f(sc[nt][3] - ms1);
        rs0 += sc[nt][0] + sc[nt][1];
        rs1 += sc[nt][2] + sc[nt][3];
      }
      l0 = l0 * a0 + rs0;
      l1 = l1 * a1 + rs1;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
#pragma unroll
      for (int pi = 0; pi < 4; ++pi) {
        if (pi < nvalid) {
          uint32_t pf[4];
          pf[0] = MmaOp<T>::pack(sc[2 * pi][0], sc[2 * pi][1]);
          pf[1] = MmaOp<T>::pack(sc[2 * pi][2], sc[2 * pi][3]);
          pf[2] = MmaOp<T>::pack(sc[2 * pi + 1][0], sc[2 * pi + 1][1]);
          pf[3] = MmaOp<T>::pack(sc[2 * pi + 1][2], sc[2 * pi + 1][3]);
          pv_page<T, HD>(o, pf, stage + pi * kPageBytes + J * kBoxBytes, lane);
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->empty[s]);
    }
    l0 = quad_sum(l0);
    l1 = quad_sum(l1);
    if (!ctl->abort_flag) {
      const float inv0 = l0 > 0.f ? 1.f / l0 : 0.f, inv1 = l1 > 0.f ? 1.f / l1 : 0.f;
      T* out = reinterpret_cast<T*>(p.out);
      const int c = (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < HD / 8; ++i) {
        if (qi0 < qlen) {
          typename Num<T>::T2 v = Num<T>::from_f2(o[i][0] * inv0, o[i][1] * inv0);
          *reinterpret_cast<typename Num<T>::T2*>(out + (size_t)(p.q_start[seq] + qi0) * p.ldo + (size_t)h * HD + i * 8 + c) = v;
        }
        if (qi1 < qlen) {
          typename Num<T>::T2 v = Num<T>::from_f2(o[i][2] * inv1, o[i][3] * inv1);
          *reinterpret_cast<typename Num<T>::T2*>(out + (size_t)(p.q_start[seq] + qi1) * p.ldo + (size_t)h * HD + i * 8 + c) = v;
        }
      }
    }
  }
  __syncthreads();
}

// ----------------------------------------------------------------- host -----
static int fill_params(const RfAttn* a, AttnParams* p) {
  RF_REQUIRE(a && a->q && a->out, "attention needs q and out");
  RF_REQUIRE(a->hd == 64 || a->hd == 128 || a->hd == 256, "attention head_dim %d (64/128/256; pad others)", a->hd);
  RF_REQUIRE(a->Hkv > 0 && a->Hq % a->Hkv == 0, "attention heads %d / kv heads %d", a->Hq, a->Hkv);
  RF_REQUIRE(a->kv_len && a->num_seqs > 0, "attention needs kv_len and sequences");
  RF_REQUIRE(a->dtype == 0 || a->dtype == 1, "attention dtype");
  const bool paged = a->k_pool != nullptr;
  if (paged) RF_REQUIRE(a->v_pool && a->page_table && a->pool_pages > 0, "paged attention needs v_pool, page_table, pool_pages");
  else RF_REQUIRE(a->k && a->v && a->kv_start && a->kv_rows_total > 0, "contiguous attention needs k, v, kv_start, kv_rows_total");
  p->q = a->q; p->ldq = a->ldq; p->out = a->out; p->ldo = a->ldo;
  p->kv_stream = 0;
  p->page_table = a->page_table; p->pt_stride = a->pt_stride; p->paged = paged ? 1 : 0;
  p->num_seqs = a->num_seqs; p->Hq = a->Hq; p->Hkv = a->Hkv; p->G = a->Hq / a->Hkv;
  p->q_start = a->q_start; p->q_len = a->q_len; p->kv_start = a->kv_start; p->kv_len = a->kv_len;
  p->max_q_len = a->max_q_len; p->causal = a->causal; p->window = a->window;
  p->mask = a->mask; p->mask_ld = a->mask_ld; p->mask_seq_stride = a->mask_seq_stride;
  p->seg_q = a->seg_q; p->seg_k = a->seg_k;
  const float scale = a->scale > 0.f ? a->scale : 1.0f / sqrtf((float)a->hd);
  p->scale_log2 = scale * 1.4426950408889634f;
  p->ws_o = nullptr; p->ws_lse = nullptr; p->splits = 1; p->pages_per_split = 1 << 28; p->stages = 2;
  p->status = a->status;
  return RF_OK;
}

static int kv_tmaps(const RfAttn* a, CUtensorMap* tmK, CUtensorMap* tmV) {
  int rc;
  if (a->k_pool) {
    const uint64_t rows = (uint64_t)a->pool_pages * a->Hkv * 16;
    rc = make_tmap_2d(tmK, a->k_pool, a->dtype, 2, a->hd, rows, a->hd, 64, 16, true);
    if (rc) return rc;
    return make_tmap_2d(tmV, a->v_pool, a->dtype, 2, a->hd, rows, a->hd, 64, 16, true);
  }
  rc = make_tmap_2d(tmK, a->k, a->dtype, 2, (uint64_t)a->Hkv * a->hd, a->kv_rows_total, a->ldk, 64, 16, true);
  if (rc) return rc;
  return make_tmap_2d(tmV, a->v, a->dtype, 2, (uint64_t)a->Hkv * a->hd, a->kv_rows_total, a->ldv, 64, 16, true);
}

// Split-KV plan of the decode kernel: how many CTAs share one (sequence, kv head)'s KV range and how many pages each
// takes.  Small batches are split until about two CTAs per SM exist; a split covers at least 8 pages and a multiple
// of 4 (one ring stage).  `allow_split` is false when the caller gave no scratch for the partials.
struct DecodeSplitPlan {
  int splits, pages_per_split;
  uint64_t scratch_bytes;   // fp32 partial outputs + one log-sum-exp per (sequence, head, split); 0 when unsplit
};
static DecodeSplitPlan plan_decode_split(int num_seqs, int Hq, int Hkv, int hd, int max_kv_len, bool allow_split) {
  const int max_pages = std::max(1, (max_kv_len + 15) / 16);
  const int ctas = num_seqs * Hkv;
  int splits = 1;
  // RF_ATTN_DECODE_CTAS_PER_SM (default 2; 1 for heads of 256): CTAs per SM the split aims at; RF_ATTN_DECODE_MIN_PAGES (default 8): fewest
  // pages a split may cover
  // (heads of 256 run one CTA per SM: measured on the Pi0.5 denoise loop, 50 rows x 1 KV head over ~870 keys, 12.5 ms at
  // two per SM against 11.6 ms at one; heads of 128, Qwen3-8B decode at batch 1 / 8: 3.41 / 3.83 ms against 3.51 / 4.03)
  static const int per_sm_env = [] { const char* e = getenv("RF_ATTN_DECODE_CTAS_PER_SM"); return e ? std::max(1, atoi(e)) : 0; }();
  const int per_sm = per_sm_env > 0 ? per_sm_env : (hd >= 256 ? 1 : 2);
  static const int min_pages = [] { const char* e = getenv("RF_ATTN_DECODE_MIN_PAGES"); return e ? std::max(4, atoi(e)) : 8; }();
  if (allow_split && ctas < per_sm * sm_count()) {
    splits = std::min(std::max(1, (per_sm * sm_count()) / ctas), std::max(1, max_pages / min_pages));
    splits = std::min(splits, 64);
  }
  DecodeSplitPlan pl;
  pl.pages_per_split = round_up(ceil_div(max_pages, splits), 4);
  pl.splits = std::max(1, ceil_div(max_pages, pl.pages_per_split));
  pl.scratch_bytes = pl.splits > 1 ? (uint64_t)num_seqs * Hq * pl.splits * (hd + 1) * sizeof(float) : 0;
  return pl;
}

template <typename T, int HD>
static int launch_decode(const RfAttn* a, AttnParams& p, cudaStream_t s) {
  CUtensorMap tmK, tmV;
  int rc = kv_tmaps(a, &tmK, &tmV);
  if (rc) return rc;
  constexpr int kStageBytes = 4 * 2 * (HD / 64) * kBoxBytes;
  const int merge_bytes = (4 * 16 * HD + 128) * 4;
  int stages = HD == 256 ? 2 : (HD == 128 ? 3 : 4);
  while (stages * kStageBytes < merge_bytes) ++stages;
  p.stages = stages;
  const size_t smem = (size_t)stages * kStageBytes + sizeof(AttnCtl) + 1024 + 64;
  auto kfn = attn_decode_kernel<T, HD>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 200 * 1024);
  // split the KV range so that small batches still fill the machine
  const DecodeSplitPlan pl = plan_decode_split(a->num_seqs, a->Hq, a->Hkv, HD, a->max_kv_len, a->ws != nullptr);
  const int splits = pl.splits;
  if (splits > 1) {
    RF_REQUIRE(pl.scratch_bytes <= a->ws_bytes, "decode attention scratch too small: need %llu B",
               (unsigned long long)pl.scratch_bytes);
    p.ws_o = a->ws;
    p.ws_lse = a->ws + (size_t)a->num_seqs * a->Hq * splits * HD;
  }
  p.splits = splits;
  p.pages_per_split = pl.pages_per_split;
  {
    static const int ef = [] { const char* e = getenv("RF_ATTN_KV_EVICT_FIRST"); return e ? atoi(e) : 1; }();
    p.kv_stream = ef;
  }
  dim3 grid(splits, a->Hkv, a->num_seqs);
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(grid), dim3(160), smem, s, 1, tmK, tmV, p));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  if (splits > 1) {
    dim3 g2(a->Hq, a->num_seqs);
    RF_CUDA_CHECK(::rf::launch_k(attn_decode_combine_kernel<T>, dim3(g2), dim3(HD < 128 ? HD : 128), 0, s, 1, p.ws_o, p.ws_lse, (T*)a->out, a->ldo, a->Hq, HD, splits));
    RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  }
  return RF_OK;
}

template <typename T, int HD>
static int launch_prefill(const RfAttn* a, AttnParams& p, cudaStream_t s) {
  CUtensorMap tmQ, tmK, tmV;
  int rc = kv_tmaps(a, &tmK, &tmV);
  if (rc) return rc;
  RF_REQUIRE(a->q_start && a->q_len && a->max_q_len > 0 && a->q_rows_total > 0, "prefill attention needs q_start, q_len, max_q_len, q_rows_total");
  rc = make_tmap_2d(&tmQ, a->q, a->dtype, 2, (uint64_t)a->Hq * a->hd, a->q_rows_total, a->ldq, 64, 16, true);
  if (rc) return rc;
  constexpr int kStageBytes = 4 * 2 * (HD / 64) * kBoxBytes;
  constexpr int kQBytes = 4 * (HD / 64) * kBoxBytes;
  // two resident CTAs per SM (registers allow two): their warps hide each other's MMA and ldmatrix latency,
  // which matters more than a deeper K/V ring
  p.stages = HD == 64 ? 3 : 2;
  const size_t smem = (size_t)kQBytes + (size_t)p.stages * kStageBytes + sizeof(AttnCtl) + 1024 + 64;
  auto kfn = attn_prefill_kernel<T, HD>;
  RF_ALLOW_SMEM_PER_DEVICE(kfn, 200 * 1024);
  dim3 grid(ceil_div(a->max_q_len, 64), a->Hq, a->num_seqs);
  RF_CUDA_CHECK(::rf::launch_k(kfn, dim3(grid), dim3(160), smem, s, 1, tmQ, tmK, tmV, p));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}

}  // namespace rf

using namespace rf;

#define RF_ATTN_DISPATCH(fn)                                                        \
  if (a->dtype == 0) {                                                              \
    if (a->hd == 64) return fn<__half, 64>(a, p, s);                                \
    if (a->hd == 128) return fn<__half, 128>(a, p, s);                              \
    return fn<__half, 256>(a, p, s);                                                \
  }                                                                                 \
  if (a->hd == 64) return fn<__nv_bfloat16, 64>(a, p, s);                           \
  if (a->hd == 128) return fn<__nv_bfloat16, 128>(a, p, s);                         \
  return fn<__nv_bfloat16, 256>(a, p, s);

extern "C" uint64_t rf_attn_decode_scratch_bytes(int num_seqs, int Hq, int hd) {
  return (uint64_t)num_seqs * Hq * 64 * (hd + 1) * sizeof(float);
}

extern "C" int rf_attn_decode(const RfAttn* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  AttnParams p;
  int rc = fill_params(a, &p);
  if (rc) return rc;
  RF_REQUIRE(a->Hq / a->Hkv <= 16, "decode attention handles GQA groups up to 16, got %d", a->Hq / a->Hkv);
  RF_REQUIRE(a->max_kv_len > 0, "decode attention needs max_kv_len");
  RF_REQUIRE(a->window <= 0, "decode attention has no sliding-window form (window=%d): every query would see the whole "
             "context", a->window);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  RF_ATTN_DISPATCH(launch_decode)
}

namespace rf {
int launch_prefill_tc(const RfAttn* a, const AttnParams& p, cudaStream_t s);   // attention_tc.cu
}

int rf_attn_wide(const RfAttn* a, rf_stream_t stream);   // attention_wide.cu: head sizes beyond 256, and short problems
bool rf_attn_tiny_eligible(const RfAttn* a);

extern "C" int rf_attn_prefill(const RfAttn* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  if (a && (a->hd == 512 || rf_attn_tiny_eligible(a))) return rf_attn_wide(a, stream);
  AttnParams p;
  int rc = fill_params(a, &p);
  if (rc) return rc;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // tcgen05 kernel by default; RF_ATTN_TC=0 selects the mma.sync kernel (A/B timing)
  static const bool use_tc = [] { const char* e = getenv("RF_ATTN_TC"); return !(e && e[0] == '0'); }();
  if (use_tc) return rf::launch_prefill_tc(a, p, s);
  RF_ATTN_DISPATCH(launch_prefill)
}

// ---------------------------------------------------------------------------
// Decode attention with built-in scratch (see attn_decode_static.h).
#include "attn_decode_static.h"

#include <mutex>

// Split-KV partials of rf_attn_decode_static().  In host code this name is only
// a stand-in for the symbol, never a device address: the address handed to the
// kernels comes from cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_attn_decode_static_scratch[RF_ATTN_DECODE_STATIC_SCRATCH_BYTES];

namespace rf {

constexpr int kMaxStaticDevices = 64;
static std::mutex g_static_mu;
static void* g_static_ptr[kMaxStaticDevices] = {};

// Device address of the built-in scratch on the current device (looked up once per device).
static int static_scratch_ptr(void** out) {
  int dev = -1;
  RF_CUDA_CHECK(cudaGetDevice(&dev));
  RF_REQUIRE(dev >= 0 && dev < kMaxStaticDevices, "device ordinal %d is outside the supported range", dev);
  std::lock_guard<std::mutex> g(g_static_mu);
  if (g_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    RF_CUDA_CHECK(cudaGetSymbolAddress(&p, g_attn_decode_static_scratch));
    RF_REQUIRE(p != nullptr && (reinterpret_cast<uintptr_t>(p) & 255) == 0,
               "built-in scratch has no usable device address on device %d", dev);
    g_static_ptr[dev] = p;
  }
  *out = g_static_ptr[dev];
  return RF_OK;
}

// Bytes of split-KV partials the launcher will ask for: the launcher's own plan, with splitting allowed.
static uint64_t decode_scratch_need(const RfAttn* a) {
  return plan_decode_split(a->num_seqs, a->Hq, a->Hkv, a->hd, a->max_kv_len, true).scratch_bytes;
}

}  // namespace rf

extern "C" int rf_attn_decode_static(const RfAttn* a, rf_stream_t stream) {
  RF_REQUIRE(a != nullptr, "null RfAttn");
  RF_REQUIRE(a->num_seqs > 0 && a->Hkv > 0 && a->Hq > 0 && a->hd > 0 && a->max_kv_len > 0,
             "decode attention shape: seqs=%d Hq=%d Hkv=%d hd=%d max_kv_len=%d", a->num_seqs, a->Hq, a->Hkv,
             a->hd, a->max_kv_len);
  const uint64_t need = decode_scratch_need(a);
  if (need > RF_ATTN_DECODE_STATIC_SCRATCH_BYTES)
    return fail(RF_ERR_NO_MEMORY,
                "decode attention for %d sequences x %d heads needs %llu B of split-KV scratch; the built-in buffer "
                "holds %u B -- call rf_attn_decode() with caller-provided scratch",
                a->num_seqs, a->Hq, (unsigned long long)need, (unsigned)RF_ATTN_DECODE_STATIC_SCRATCH_BYTES);
  void* ptr = nullptr;
  int rc = static_scratch_ptr(&ptr);
  if (rc) return rc;
  RfAttn b = *a;
  b.ws = static_cast<float*>(ptr);
  b.ws_bytes = RF_ATTN_DECODE_STATIC_SCRATCH_BYTES;
  return rf_attn_decode(&b, stream);
}
