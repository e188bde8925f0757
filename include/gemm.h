// Transpose-aware GEMM and strided-batched GEMM with the reference's
// signatures (src/gemm.h:17-29).  Row-major, dense leading dimensions:
//   C[M,N] = alpha * op(A) @ op(B) + beta * C
//   op(A) = A   (A stored M x K)  or  A^T (A stored K x M) when transA
//   op(B) = B   (B stored K x N)  or  B^T (B stored N x K) when transB
// Arithmetic follows bmb_get_math_mode(): fp32 FFMA unless the process opted
// into TF32/BF16 tensor cores (BMB_MATH=tf32|bf16 or bmb_set_math_mode).
// A failing status from the C ABI is fatal here, as CUDA errors are in the
// reference's callers (message on stderr, exit(1)).
#pragma once
#include <cuda_runtime.h>

void gemm(bool transA, bool transB, int M, int N, int K, float alpha,
          const float *A, const float *B, float beta, float *C,
          cudaStream_t stream = 0);

// `batch` independent problems; problem i uses A + i*strideA, B + i*strideB,
// C + i*strideC (strides in elements).  One launch: the batch index is a grid
// dimension.
void batched_gemm(bool transA, bool transB, int batch, int M, int N, int K,
                  float alpha, const float *A, long long strideA,
                  const float *B, long long strideB, float beta, float *C,
                  long long strideC, cudaStream_t stream = 0);
