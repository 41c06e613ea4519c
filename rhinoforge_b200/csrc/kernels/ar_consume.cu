// Second half of the tensor-parallel all-reduce of a row-parallel GEMM: wait for every rank's
// partial rows, reduce, add the residual and apply the RMSNorm that follows in the layer.
//
// The producing GEMM (gemm_tc.cu, ar_publish) pushes its partial rows into slot [rank] of every
// rank's receive buffer over NVLink and exits without waiting for anyone.  This kernel is the only
// place that waits: thread r polls (bounded) the arrival counter of rank r in this GPU's own flag
// array until it shows that all CTAs of that rank's GEMM have published.  One CTA then owns one
// token row: it sums the ranks' partials in rank order in fp32, adds the residual, writes the
// row of the residual stream and -- when the layer continues with an RMSNorm -- the normalised row
// that the next GEMM reads, so neither the wait nor the norm costs a launch of its own.
//
// Because the kernel lets its dependents launch at once, the next GEMM's CTAs are already resident
// and prefetching their weight tiles while this kernel waits for the slowest peer.
//
// Replaces the reference's single-launch all-reduce + residual operators
// (src/core/rpu_runtime_extras.cpp:202-460,1035-1092) and the RMSNorm launch after them
// (src/fused/rpu_qwen3_model.h:3526-3557).
#include "../common/dtype.cuh"
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

constexpr int kArThreads = 512;
constexpr int kArMaxVec = 4;   // 8-column vectors a thread keeps in registers: rows up to 512 * 4 * 8 columns

struct ArConsumeParams {
  void* const* recv_tab;         // device table of receive-buffer bases; entry [rank] is this GPU's own
  uint32_t* const* flag_tab;     // device table of flag-array bases; entry [rank] is this GPU's own
  uint64_t half_bytes;
  int cnt_base, rank;
  uint32_t* state;
  int world, M, N, pub_ctas;
  const void* residual; int64_t ldr;
  void* out; int64_t ldo;
  const void* norm_w; void* norm_out; int64_t ldn;
  float eps; int norm_mode;
  int32_t* status;
};

// One rank's eight partial columns as fp32
template <typename T, bool F32>
__device__ __forceinline__ void load_partial8(const uint8_t* base, size_t elem, float (&f)[8]) {
  if constexpr (F32) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(base + elem * 4));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(base + elem * 4 + 16));
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
  } else {
    const uint4 raw = __ldcg(reinterpret_cast<const uint4*>(base + elem * 2));
    const typename Num<T>::T2* h = reinterpret_cast<const typename Num<T>::T2*>(&raw);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 t = Num<T>::to_f2(h[j]);
      f[2 * j] = t.x;
      f[2 * j + 1] = t.y;
    }
  }
}

template <typename T, bool F32, int VPT>
__global__ void __launch_bounds__(kArThreads) ar_consume_kernel(const ArConsumeParams p) {
  pdl_prologue();
  __shared__ float red[kArThreads / 32 + 1];
  __shared__ int bad;
  const int tid = threadIdx.x, row = blockIdx.x;
  const uint32_t call = *reinterpret_cast<volatile uint32_t*>(p.state);
  const uint32_t target = *reinterpret_cast<volatile uint32_t*>(p.state + 4) + (uint32_t)p.pub_ctas;
  if (tid == 0) bad = 0;
  __syncthreads();
  const uint32_t* counters = p.flag_tab[p.rank] + p.cnt_base;   // this rank's arrival counters, one per source rank
  if (tid < p.world) {
    // after the first reported failure of this status block nothing waits again: one second, not one per launch
    const bool poisoned = p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0;
    if (poisoned || !wait_flag_ge_sys(counters + tid, target)) {
      if (!poisoned) report_status(p.status, kStatusPeerTimeout, kTagGemmAr, 200 + tid);
      bad = 1;
    }
  }
  __syncthreads();
  if (!bad) {
    const uint8_t* slot = static_cast<const uint8_t*>(p.recv_tab[p.rank]) + (uint64_t)(call & 1u) * p.half_bytes;
    const T* resid = reinterpret_cast<const T*>(p.residual);
    T* out = reinterpret_cast<T*>(p.out);
    const int nvec = p.N >> 3;
    float h[VPT][8];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
      const int v = tid + k * kArThreads;
      if (v < nvec) {
        // every rank's vector (and the residual's) is in flight before the first add; sum in rank order
        float part[8][8];
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < p.world) load_partial8<T, F32>(slot, ((size_t)r * p.M + row) * p.N + (size_t)v * 8, part[r]);
        }
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float r8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (resid) load8(resid + (size_t)row * p.ldr + (size_t)v * 8, r8);
#pragma unroll
        for (int r = 0; r < 8; ++r) {
          if (r < p.world) {
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] += part[r][j];
          }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          h[k][j] = Num<T>::to_f(Num<T>::from_f(acc[j] + r8[j]));   // the value the residual stream holds
          ss += h[k][j] * h[k][j];
        }
        store8(out + (size_t)row * p.ldo + (size_t)v * 8, h[k]);
      }
    }
    if (p.norm_mode != 0) {
      // block sum of squares in a fixed order (lanes, then warps)
      ss = warp_sum(ss);
      if ((tid & 31) == 0) red[tid >> 5] = ss;
      __syncthreads();
      if (tid < 32) {
        float t = tid < (int)(blockDim.x >> 5) ? red[tid] : 0.f;
        t = warp_sum(t);
        if (tid == 0) red[kArThreads / 32] = t;
      }
      __syncthreads();
      const float rstd = rsqrtf(red[kArThreads / 32] / (float)p.N + p.eps);
      const T* w = reinterpret_cast<const T*>(p.norm_w);
      T* y = reinterpret_cast<T*>(p.norm_out);
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tid + k * kArThreads;
        if (v < nvec) {
          float wf[8], o[8];
          load8(w + (size_t)v * 8, wf);
          if (p.norm_mode == 2) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = h[k][j] * rstd * (1.f + wf[j]);
          } else {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = wf[j] * Num<T>::to_f(Num<T>::from_f(h[k][j] * rstd));
          }
          store8(y + (size_t)row * p.ldn + (size_t)v * 8, o);
        }
      }
    }
  }
  // the last CTA to finish closes this all-reduce: the counters it consumed and the next call number
  __syncthreads();
  if (tid == 0) {
    const uint32_t done = atomicAdd(p.state + 5, 1u);
    if (done == gridDim.x - 1u) {
      p.state[5] = 0u;
      p.state[4] = target;
      __threadfence();
      p.state[0] = call + 1u;
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Two-shot all-reduce of whole rows for prefill-sized token counts (see RfArRows in rf_api.h).
struct ArRowsParams {
  void* const* partial_tab; void* const* out_tab; void* const* norm_tab;
  uint32_t* const* flag_tab; uint32_t* state;
  int world, rank, M, N, flag_base, add_residual, out_local;
  const void* norm_w; float eps; int norm_mode;
  int32_t* status;
};

template <typename T, int VPT>
__global__ void __launch_bounds__(kArThreads) ar_rows_kernel(const ArRowsParams p) {
  pdl_prologue();
  __shared__ float red[kArThreads / 32 + 1];
  __shared__ int bad;
  __shared__ unsigned last_cta;
  const int tid = threadIdx.x;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(p.state + 6) + 1u;
  uint32_t* my_flags = p.flag_tab[p.rank] + p.flag_base;
  if (tid == 0) bad = 0;
  // this rank's partial (written by the kernel before this one) is complete: tell every peer, once
  if (blockIdx.x == 0 && tid < p.world) {
    __threadfence_system();
    st_release_sys(p.flag_tab[tid] + p.flag_base + p.rank, epoch);
  }
  __syncthreads();
  if (tid < p.world) {
    const bool poisoned = p.status != nullptr && *reinterpret_cast<volatile int32_t*>(p.status) != 0;
    if (poisoned || !wait_flag_ge_sys(my_flags + tid, epoch)) {
      if (!poisoned) report_status(p.status, kStatusPeerTimeout, kTagGemmAr, 300 + tid);
      bad = 1;
    }
  }
  __syncthreads();
  const int per = (p.M + p.world - 1) / p.world;
  const int row_begin = p.rank * per, row_end = min(p.M, row_begin + per);
  const int nvec = p.N >> 3;
  if (!bad) {
    const T* parts[8];
    T* outs[8];
    T* norms[8];
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      parts[r] = r < p.world ? reinterpret_cast<const T*>(p.partial_tab[r]) : nullptr;
      outs[r] = r < p.world ? reinterpret_cast<T*>(p.out_tab[r]) : nullptr;
      norms[r] = (r < p.world && p.norm_mode != 0) ? reinterpret_cast<T*>(p.norm_tab[r]) : nullptr;
    }
    const T* resid = p.add_residual ? outs[0] : nullptr;
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r == p.rank && p.add_residual) resid = outs[r];
    const T* w = reinterpret_cast<const T*>(p.norm_w);
    for (int row = row_begin + blockIdx.x; row < row_end; row += gridDim.x) {
      float h[VPT][8];
      float ss = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; ++k) {
        const int v = tid + k * kArThreads;
        if (v < nvec) {
          const size_t at = (size_t)row * p.N + (size_t)v * 8;
          uint4 raw[8];
#pragma unroll
          for (int r = 0; r < 8; ++r)
            raw[r] = r < p.world ? __ldcg(reinterpret_cast<const uint4*>(parts[r] + at)) : make_uint4(0u, 0u, 0u, 0u);
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          float r8[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          if (resid) load8(resid + at, r8);
#pragma unroll
          for (int r = 0; r < 8; ++r) {
            if (r < p.world) {
              const typename Num<T>::T2* hh = reinterpret_cast<const typename Num<T>::T2*>(&raw[r]);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const float2 f = Num<T>::to_f2(hh[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
              }
            }
          }
          Vec8<T> packed;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            packed.v[j] = Num<T>::from_f2(acc[2 * j] + r8[2 * j], acc[2 * j + 1] + r8[2 * j + 1]);
            const float2 back = Num<T>::to_f2(packed.v[j]);
            h[k][2 * j] = back.x;
            h[k][2 * j + 1] = back.y;
            ss += back.x * back.x + back.y * back.y;
          }
#pragma unroll
          for (int d = 0; d < 8; ++d)
            if (d < p.world && (!p.out_local || d == p.rank)) *reinterpret_cast<Vec8<T>*>(outs[d] + at) = packed;
        }
      }
      if (p.norm_mode != 0) {
        ss = warp_sum(ss);
        __syncthreads();                       // red[] of the previous row has been read
        if ((tid & 31) == 0) red[tid >> 5] = ss;
        __syncthreads();
        if (tid < 32) {
          float t = tid < (int)(blockDim.x >> 5) ? red[tid] : 0.f;
          t = warp_sum(t);
          if (tid == 0) red[kArThreads / 32] = t;
        }
        __syncthreads();
        const float rstd = rsqrtf(red[kArThreads / 32] / (float)p.N + p.eps);
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
          const int v = tid + k * kArThreads;
          if (v < nvec) {
            const size_t at = (size_t)row * p.N + (size_t)v * 8;
            float wf[8], o[8];
            load8(w + (size_t)v * 8, wf);
            if (p.norm_mode == 2) {
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = h[k][j] * rstd * (1.f + wf[j]);
            } else {
#pragma unroll
              for (int j = 0; j < 8; ++j) o[j] = wf[j] * Num<T>::to_f(Num<T>::from_f(h[k][j] * rstd));
            }
            Vec8<T> packed;
#pragma unroll
            for (int j = 0; j < 4; ++j) packed.v[j] = Num<T>::from_f2(o[2 * j], o[2 * j + 1]);
#pragma unroll
            for (int d = 0; d < 8; ++d)
              if (d < p.world) *reinterpret_cast<Vec8<T>*>(norms[d] + at) = packed;
          }
        }
      }
    }
  }
  // Every row this rank owns is written on every rank: the last CTA says so to every peer and then waits until
  // every peer has said the same, so that the kernel after this one finds all rows of its buffers complete.
  __threadfence_system();
  __syncthreads();
  if (tid == 0) {
    const unsigned done = atomicAdd(p.state + 7, 1u);
    last_cta = (done == gridDim.x - 1u) ? 1u : 0u;
  }
  __syncthreads();
  if (last_cta) {
    __threadfence_system();
    if (tid < p.world && !bad) st_release_sys(p.flag_tab[tid] + p.flag_base + 8 + p.rank, epoch);
    if (tid < p.world && !bad) {
      if (!wait_flag_ge_sys(my_flags + 8 + tid, epoch)) report_status(p.status, kStatusPeerTimeout, kTagGemmAr, 400 + tid);
    }
    __syncthreads();
    if (tid == 0) {
      p.state[7] = 0u;
      __threadfence();
      p.state[6] = epoch;
    }
  }
}

template <typename T, bool F32>
static int launch_consume(const RfArConsume* a, const ArConsumeParams& p, cudaStream_t st) {
  const int nvec = a->N / 8;
  const int vpt = ceil_div(nvec, kArThreads);
  const int threads = vpt > 1 ? kArThreads : std::max(32, round_up(nvec, 32));
  cudaError_t e;
  switch (vpt) {
    case 1: e = launch_k(ar_consume_kernel<T, F32, 1>, dim3(a->M), dim3(threads), 0, st, 1, p); break;
    case 2: e = launch_k(ar_consume_kernel<T, F32, 2>, dim3(a->M), dim3(threads), 0, st, 1, p); break;
    default: e = launch_k(ar_consume_kernel<T, F32, kArMaxVec>, dim3(a->M), dim3(threads), 0, st, 1, p); break;
  }
  RF_CUDA_CHECK(e);
  count_launch();
  return RF_OK;
}

}  // namespace rf

using namespace rf;

extern "C" int rf_ar_consume(const RfArConsume* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a != nullptr, "null RfArConsume");
  RF_REQUIRE(a->M > 0 && a->M <= 256 && a->N > 0 && a->N % 8 == 0, "ar_consume shape %dx%d (rows <= 256, columns %% 8)", a->M, a->N);
  RF_REQUIRE(a->N <= kArThreads * kArMaxVec * 8, "ar_consume rows of %d columns exceed %d", a->N, kArThreads * kArMaxVec * 8);
  RF_REQUIRE(a->world >= 2 && a->world <= 8 && a->rank >= 0 && a->rank < a->world, "ar_consume rank %d of %d", a->rank, a->world);
  RF_REQUIRE(a->ar_recv && a->ar_flags && a->ar_state && a->out && a->pub_ctas > 0, "ar_consume needs buffers and the producer's CTA count");
  RF_REQUIRE(a->dtype == 0 || a->dtype == 1, "ar_consume dtype");
  RF_REQUIRE(a->ldo % 8 == 0 && (!a->residual || a->ldr % 8 == 0), "ar_consume row pitches must be multiples of 8 elements");
  if (a->norm_mode != 0) RF_REQUIRE(a->norm_w && a->norm_out && a->ldn % 8 == 0 && (a->norm_mode == 1 || a->norm_mode == 2), "ar_consume fused norm arguments");
  const bool f32 = a->M <= RF_AR_F32_MAX_ROWS;
  const uint64_t need = (uint64_t)a->world * a->M * a->N * (f32 ? 4 : 2);
  RF_REQUIRE(need <= a->ar_recv_bytes, "ar_consume: receive buffer half of %llu B is smaller than %llu B", (unsigned long long)a->ar_recv_bytes, (unsigned long long)need);
  ArConsumeParams p;
  p.recv_tab = a->ar_recv;
  p.flag_tab = a->ar_flags;
  p.half_bytes = a->ar_recv_bytes;
  p.cnt_base = a->ar_cnt_base;
  p.rank = a->rank;
  p.state = a->ar_state;
  p.world = a->world; p.M = a->M; p.N = a->N; p.pub_ctas = a->pub_ctas;
  p.residual = a->residual; p.ldr = a->ldr; p.out = a->out; p.ldo = a->ldo;
  p.norm_w = a->norm_w; p.norm_out = a->norm_out; p.ldn = a->ldn; p.eps = a->eps; p.norm_mode = a->norm_mode;
  p.status = a->status;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (a->dtype == 0) return f32 ? launch_consume<__half, true>(a, p, st) : launch_consume<__half, false>(a, p, st);
  return f32 ? launch_consume<__nv_bfloat16, true>(a, p, st) : launch_consume<__nv_bfloat16, false>(a, p, st);
}

extern "C" int rf_ar_rows(const RfArRows* a, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(a != nullptr, "null RfArRows");
  RF_REQUIRE(a->M > 0 && a->N > 0 && a->N % 8 == 0 && a->N <= kArThreads * kArMaxVec * 8, "ar_rows shape %dx%d", a->M, a->N);
  RF_REQUIRE(a->world >= 2 && a->world <= 8 && a->rank >= 0 && a->rank < a->world, "ar_rows rank %d of %d", a->rank, a->world);
  RF_REQUIRE(a->partial_tab && a->out_tab && a->ar_flags && a->ar_state && a->flag_base >= 0, "ar_rows needs the buffer tables, flags and state");
  RF_REQUIRE(a->dtype == 0 || a->dtype == 1, "ar_rows dtype");
  if (a->norm_mode != 0) RF_REQUIRE(a->norm_w && a->norm_tab && (a->norm_mode == 1 || a->norm_mode == 2), "ar_rows fused norm arguments");
  RF_REQUIRE(!a->out_local || a->norm_mode != 0, "ar_rows: rows that stay on their owner need the gathered normalised rows as the result every rank reads");
  ArRowsParams p;
  p.partial_tab = a->partial_tab; p.out_tab = a->out_tab; p.norm_tab = a->norm_tab;
  p.flag_tab = a->ar_flags; p.state = a->ar_state;
  p.world = a->world; p.rank = a->rank; p.M = a->M; p.N = a->N; p.flag_base = a->flag_base; p.add_residual = a->add_residual;
  p.out_local = a->out_local;
  p.norm_w = a->norm_w; p.eps = a->eps; p.norm_mode = a->norm_mode; p.status = a->status;
  const int nvec = a->N / 8;
  const int vpt = ceil_div(nvec, kArThreads);
  const int threads = vpt > 1 ? kArThreads : std::max(32, round_up(nvec, 32));
  const int own = ceil_div(a->M, a->world);
  const int grid = std::max(1, std::min(own, 8 * sm_count()));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  cudaError_t e;
#define RF_AR_ROWS(T)                                                                                        \
  switch (vpt) {                                                                                             \
    case 1: e = launch_k(ar_rows_kernel<T, 1>, dim3(grid), dim3(threads), 0, st, 1, p); break;               \
    case 2: e = launch_k(ar_rows_kernel<T, 2>, dim3(grid), dim3(threads), 0, st, 1, p); break;               \
    default: e = launch_k(ar_rows_kernel<T, kArMaxVec>, dim3(grid), dim3(threads), 0, st, 1, p); break;      \
  }
  if (a->dtype == 0) { RF_AR_ROWS(__half) } else { RF_AR_ROWS(__nv_bfloat16) }
#undef RF_AR_ROWS
  RF_CUDA_CHECK(e);
  count_launch();
  return RF_OK;
}
