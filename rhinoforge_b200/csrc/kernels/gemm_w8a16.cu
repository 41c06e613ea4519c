// The W8A16 tensor-core path lives in gemm_tc.cu (template parameter W8 of gemm_tc_kernel and
// the entry point rf_gemm_w8a16): the int8 weight tile is brought in by TMA, widened to the
// activation dtype by four converter warps into the swizzled MMA tile, and the per-channel scale
// is applied in the epilogue.  The CUDA-core path for up to 8 tokens is rf_gemv (gemv.cu).
// Replaces parallel_linear_w8a16_* and llama_gemv_wint8 (src/ops/rpu_linear.cpp:1119-1209,1546-1670).
