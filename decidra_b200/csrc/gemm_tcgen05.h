// Host interface of the tcgen05 bf16 GEMM (gemm_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

// Opaque 128-byte TMA descriptor (same size and alignment as the driver's CUtensorMap).
struct alignas(64) TcTensorMap { uint64_t opaque[16]; };

// Descriptors for the activation operand X[M,K] (box 128 rows) and the weight operand
// W[N,K] (box 256 rows); both row-major bf16 with K contiguous. 0 on success.
int tc_make_tmap_a(TcTensorMap* out, const void* X, uint64_t M, uint64_t K);
int tc_make_tmap_b(TcTensorMap* out, const void* W, uint64_t N, uint64_t K);
bool tc_shape_ok(int M, int N, int K);
// Raises the kernel's dynamic shared-memory limit on the current device (call once per device).
cudaError_t tc_gemm_prepare_device();
// epi 0: C[M,N] (row stride ldc). epi 1: SwiGLU over gate/up-interleaved weights, C[M,N/2].
cudaError_t tc_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, void* C, int M, int N, int K, int ldc, int epi,
                           int sm_count, int* err, cudaStream_t stream);
