// C entry points of libllmq_b200_kernels.so.  Every function takes raw device pointers, sizes and
// a CUDA stream, launches asynchronously and returns 0 or a CUDA/driver error code (negative values
// are argument errors).  Python binds these through ctypes (llmq_b200/ops/lib.py).
//
// dtype codes: 0 = bf16, 1 = e4m3, 2 = e5m2, 3 = fp32, 4 = fp16, 5 = int32, 6 = int8
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

int llmq_encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, long long rows, long long cols,
                        long long ld, int box_rows);

extern "C" {

// C[M,N] (+)= alpha*scale_a*scale_b * op(A) op(B)^T + bias.   See gemm_tcgen05.cu.
int llmq_gemm(const void* A, const void* B, void* C, const void* bias, int M, int N, int K, int a_dtype, int b_dtype,
              int a_mn_major, int b_mn_major, long long lda, long long ldb, long long ldc, int c_dtype, int bias_dtype,
              int accumulate, const float* scale_a, const float* scale_b, float alpha, float* absmax_out,
              unsigned int* status, int num_sms, cudaStream_t stream);

}  // extern "C"
