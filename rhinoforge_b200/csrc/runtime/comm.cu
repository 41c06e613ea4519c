// Peer-memory plumbing for the fused compute+collective kernels: a
// cudaMalloc'ed, zero-filled communication buffer per rank, exported to the
// other ranks of the node through CUDA IPC handles (the handles themselves
// travel over torch.distributed), plus a bounded device-side barrier used at
// set-up and in tests.  No NCCL and no multicast objects are involved: the
// kernels use plain peer loads/stores over NVLink.
//
// B200 counterpart of the reference's per-core SPM address tables
// (SCM registers 4096+j, src/core/rpu_runtime_extras.cpp:202-273).
#include "../common/host_util.h"
#include "../common/ptx.cuh"
#include "../rf_api.h"

namespace rf {

// Every rank bumps its slot on every peer, then waits until all slots on its own
// flag line reach the same epoch.  One block, `world` threads.
__global__ void peer_barrier_kernel(uint32_t* const* flags, int flag_base, uint32_t* state, int world,
                                    int rank, int32_t* status) {
  pdl_prologue();
  const int t = threadIdx.x;
  const uint32_t want = state[2] + 1u;
  __threadfence_system();
  if (t < world) st_release_sys(flags[t] + flag_base + rank, want);
  if (t < world) {
    if (!wait_flag_ge_sys(flags[rank] + flag_base + t, want))
      report_status(status, kStatusPeerTimeout, kTagBarrier, t);
  }
  __syncthreads();
  if (t == 0) state[2] = want;
}

// Cross-rank greedy pick: every rank publishes (value, id) of its vocab shard for
// each row to every peer's aux buffer, waits (bounded) for all ranks, and keeps the
// best pair (larger value, then lower id) -- identical on every rank.
struct ValIdx { float v; int32_t i; };
__global__ void tp_argmax_merge_kernel(void* const* aux, uint32_t* const* flags, int flag_base,
                                       uint32_t* state, int world, int rank, int rows, int max_rows,
                                       const float* vals, int32_t* ids, int32_t* status) {
  pdl_prologue();
  const int t = threadIdx.x;
  const uint32_t call = state[3];
  const uint32_t want = call + 1u;
  const size_t half = (size_t)(call & 1u) * world * max_rows;
  for (int i = t; i < rows; i += blockDim.x) {
    ValIdx p{vals[i], ids[i]};
    for (int d = 0; d < world; ++d)
      reinterpret_cast<ValIdx*>(aux[d])[half + (size_t)rank * max_rows + i] = p;
  }
  __threadfence_system();
  __syncthreads();
  if (t < world) st_release_sys(flags[t] + flag_base + rank, want);
  __shared__ int bad;
  if (t == 0) bad = 0;
  __syncthreads();
  if (t < world) {
    if (!wait_flag_ge_sys(flags[rank] + flag_base + t, want)) {
      report_status(status, kStatusPeerTimeout, kTagBarrier, 100 + t);
      bad = 1;
    }
  }
  __syncthreads();
  if (!bad) {
    const ValIdx* mine = reinterpret_cast<const ValIdx*>(aux[rank]) + half;
    for (int i = t; i < rows; i += blockDim.x) {
      ValIdx best{-INFINITY, 0x7fffffff};
      for (int r = 0; r < world; ++r) {
        ValIdx q;
        q.v = __ldcg(&mine[(size_t)r * max_rows + i].v);
        q.i = __ldcg(&mine[(size_t)r * max_rows + i].i);
        if (q.v > best.v || (q.v == best.v && q.i < best.i)) best = q;
      }
      ids[i] = best.i;
    }
  }
  __syncthreads();
  if (t == 0) state[3] = want;
}

}  // namespace rf

using namespace rf;

extern "C" int rf_tp_argmax_merge(void* const* aux, uint32_t* const* flags, int flag_base, uint32_t* state,
                                  int world, int rank, int rows, int max_rows, const float* vals,
                                  int32_t* ids, int32_t* status, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(aux && flags && state && vals && ids, "tp_argmax_merge arguments");
  RF_REQUIRE(world >= 1 && world <= 8 && rows > 0 && rows <= max_rows, "tp_argmax_merge shape");
  RF_CUDA_CHECK(::rf::launch_k(tp_argmax_merge_kernel, dim3(1), dim3(128), 0, static_cast<cudaStream_t>(stream), 1, aux, flags, flag_base, state, world, rank,
                                                                         rows, max_rows, vals, ids, status));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}


extern "C" int rf_comm_alloc(uint64_t bytes, void** out) {
  RF_REQUIRE(out && bytes > 0, "comm_alloc arguments");
  void* p = nullptr;
  RF_CUDA_CHECK(cudaMalloc(&p, bytes));
  RF_CUDA_CHECK(cudaMemset(p, 0, bytes));
  RF_CUDA_CHECK(cudaDeviceSynchronize());
  *out = p;
  return RF_OK;
}

extern "C" int rf_comm_free(void* p) {
  if (p) RF_CUDA_CHECK(cudaFree(p));
  return RF_OK;
}

extern "C" int rf_ipc_export(void* p, uint8_t* handle64) {
  RF_REQUIRE(p && handle64, "ipc_export arguments");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  cudaIpcMemHandle_t h;
  RF_CUDA_CHECK(cudaIpcGetMemHandle(&h, p));
  memcpy(handle64, &h, 64);
  return RF_OK;
}

extern "C" int rf_ipc_import(const uint8_t* handle64, void** out) {
  RF_REQUIRE(handle64 && out, "ipc_import arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  RF_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
  *out = p;
  return RF_OK;
}

extern "C" int rf_ipc_close(void* p) {
  if (p) RF_CUDA_CHECK(cudaIpcCloseMemHandle(p));
  return RF_OK;
}

// flags: device array [world] of flag-array bases; the barrier uses flags
// [flag_base, flag_base + world) on every rank and state[2] as its epoch.
extern "C" int rf_peer_barrier(uint32_t* const* flags, int flag_base, uint32_t* state, int world, int rank,
                               int32_t* status, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  RF_REQUIRE(flags && state && world >= 1 && world <= 8 && rank >= 0 && rank < world, "peer_barrier arguments");
  RF_CUDA_CHECK(::rf::launch_k(peer_barrier_kernel, dim3(1), dim3(32), 0, static_cast<cudaStream_t>(stream), 1, flags, flag_base, state, world, rank, status));
  RF_CUDA_CHECK(cudaGetLastError());
  ::rf::count_launch();
  return RF_OK;
}
