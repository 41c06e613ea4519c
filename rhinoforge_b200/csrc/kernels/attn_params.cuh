// Kernel-side argument block shared by the attention kernels (attention.cu: mma.sync prefill and
// split-KV decode; attention_tc.cu: tcgen05 prefill).
#pragma once
#include <stdint.h>

namespace rf {

struct AttnParams {
  const void* q; int64_t ldq;
  void* out; int64_t ldo;
  const int32_t* page_table; int32_t pt_stride;
  int32_t paged;
  int32_t num_seqs, Hq, Hkv, G;
  const int32_t* q_start; const int32_t* q_len; const int32_t* kv_start; const int32_t* kv_len;
  int32_t max_q_len;
  int32_t causal, window;
  const uint8_t* mask; int64_t mask_ld, mask_seq_stride;
  const int32_t* seg_q; const int32_t* seg_k;
  float scale_log2;
  float* ws_o; float* ws_lse;
  int32_t splits, pages_per_split, stages;
  int32_t kv_stream;      // decode: K/V pages are read with the L2 evict-first policy
  int32_t* status;
};


}  // namespace rf
