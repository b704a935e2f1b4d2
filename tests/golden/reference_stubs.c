/* The reference's NPU backend (src/npu/rk3588/vllm_npu_direct.c) builds only on its board.
 * Its four entry points that the model file links against are stubbed; the float32 path that
 * the golden run takes never calls them. */
int vllm_npu_available(void *npu) { (void)npu; return 0; }
int vllm_npu_backend(void *npu) { (void)npu; return 0; }
int vllm_npu_gemm_gw(void) { return -1; }
int vllm_npu_gemm_i8(void) { return -1; }
