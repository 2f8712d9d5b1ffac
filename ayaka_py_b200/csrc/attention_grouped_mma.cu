// The grouped softmax attention (attention_grouped.cu) in bfloat16 on the tensor cores.
#include "attention_grouped.cuh"

// 0: launched; 1: this geometry is left to the kernel on the FP32 pipes; < 0: an error.
int ayk_grouped_attention_mma(const GroupedArgs& a, cudaStream_t stream) {
  (void)a; (void)stream;
  return 1;
}
