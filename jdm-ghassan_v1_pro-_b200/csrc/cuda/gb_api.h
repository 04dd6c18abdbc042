// C ABI of the sm_100a kernel library (_gb200_cuda.so).  Every function takes raw device
// pointers plus the CUDA stream to launch on and returns 0 on success (negative = rejected
// arguments or a launch error).  Kernels that wait on barriers or peers report timeouts through a
// device-side status word instead of trapping; the host reads it with gb_status_read().
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

// ----------------------------------------------------------------------------- GEMM
// C[M,N] (+)= A[M,K] * B[N,K]^T with 16-bit operands and fp32 accumulation on tcgen05.
typedef struct gb_gemm_args {
  const void* A;            // stored matrix holding the A operand
  const void* B;            // stored matrix holding the B operand
  int M, N, K;              // logical problem; per group in grouped modes
  long long a_rows, a_cols, lda;   // stored A: [a_rows, a_cols], row stride lda (elements)
  long long b_rows, b_cols, ldb;   // stored B
  int a_mn_major;           // 0: stored [M,K] (K contiguous); 1: stored [K,M]
  int b_mn_major;           // 0: stored [N,K]; 1: stored [K,N]
  int is_bf16;              // operand type: 0 fp16, 1 bf16
  int out_dtype;            // 0 fp16, 1 bf16, 2 fp32
  int epilogue;             // 0 store (+ optional fp32 addend), 1 SwiGLU forward, 2 SwiGLU backward
  int block_n;              // 64 / 128 / 256 (0 = 128)
  int mode;                 // 0 dense, 1 grouped over rows (tile map), 2 grouped over the reduction dim
  const int* tile_expert;   // mode 1
  const int* num_m_tiles;   // mode 1 (device scalar)
  const int* seg_offsets;   // mode 2
  int groups;               // mode 2
  int b_group_rows;         // mode 1: stored-B rows per group
  void* out; int ldo; long long out_group_stride;
  const float* addend; int ld_add;   // out = acc + addend (fp32), may alias out when out is fp32
  void* aux_out; const void* aux_in; int ld_aux;
  int* status;              // device status word (see gb_status_*)
} gb_gemm_args;
int gb_gemm(const gb_gemm_args* args, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
