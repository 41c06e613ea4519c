// W8A16 tensor-core GEMM entry point (int8 per-output-channel weights, 16-bit
// activations).  Placeholder dispatch: token counts up to 8 run on the
// CUDA-core GEMV with in-loop dequantisation.
#include "../common/host_util.h"
#include "../rf_api.h"

extern "C" int rf_gemm_w8a16(const RfGemm* g, rf_stream_t stream) {
  RF_SKIP_IF_REPLAYING();
  if (g && g->M <= 8 && g->ar_world <= 1) return rf_gemv(g, stream);
  return rf::fail(RF_ERR_UNSUPPORTED, "W8A16 tensor-core GEMM for M=%d is not built yet", g ? g->M : -1);
}
