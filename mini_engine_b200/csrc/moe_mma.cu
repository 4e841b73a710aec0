// The routed feed-forward's per-expert products on the tensor cores (bfloat16 operands, float32 accumulation).
// Placeholder entry points: no shape is taken yet, every product runs the CUDA-core kernel of moe.cu.
#include "common.cuh"

bool me_moe_gemm_mma_takes(int a_dtype, int w_dtype, int64_t a_stride, int N, int K) { return false; }

int me_moe_gemm_mma(const void* a, int64_t a_stride, const int* sorted, int top, const void* w, int64_t w_expert_stride,
                    const int* offsets, int E, void* out, int out_dtype, int64_t out_stride, int rows, int N, int K, int glu,
                    float limit, float alpha, cudaStream_t stream) {
  me_set_error("me_moe_gemm_mma: no shape is taken");
  return 1;
}
