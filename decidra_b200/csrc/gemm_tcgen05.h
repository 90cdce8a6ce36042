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
// Strided 2-D view (row stride in elements) with a box of box_rows x 64 columns, and a 3-D view
// [d2, d1, d0] (d0 contiguous) with a box of box2 x box1 x 64; both bf16, 128-byte swizzle.
int tc_make_tmap_strided(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows);
int tc_make_tmap_3d(TcTensorMap* out, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1, uint64_t stride2,
                    uint32_t box1, uint32_t box2);
// Strided 2-D f32 view (row stride in elements), box of box_rows x 32 columns, 128-byte swizzle.
int tc_make_tmap_f32(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows);
bool tc_shape_ok(int M, int N, int K);
// Raises the kernel's dynamic shared-memory limit on the current device (call once per device).
cudaError_t tc_gemm_prepare_device();
// epi 0: C[M,N] (row stride ldc). epi 1: SwiGLU over gate/up-interleaved weights, C[M,N/2].
// alpha: optional device scalar multiplied into the accumulator before rounding.
// resid (epi 0 only): optional bf16 [M, ldc]; C = bf16(resid + bf16(product)).
// M tiles per rasterisation group of the bf16 / e4m3 GEMM (0 = the built-in choice); for measurements.
void tc_gemm_set_group_m(int group_m);
cudaError_t tc_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, void* C, int M, int N, int K, int ldc, int epi,
                           int sm_count, int* err, cudaStream_t stream, const float* alpha = nullptr, const void* resid = nullptr);

// e4m3 (FP8) operand form: X[M,K] and W[N,K] hold one byte per element; the f32 accumulator is
// scaled by w_scale[n] * a_scale[m] before rounding to bf16. Needs K % 16 == 0, N % 8 == 0.
int tc_make_tmap_fp8_a(TcTensorMap* out, const void* X, uint64_t M, uint64_t K);
int tc_make_tmap_fp8_b(TcTensorMap* out, const void* W, uint64_t N, uint64_t K);
bool tc_fp8_shape_ok(int M, int N, int K);
cudaError_t tc_gemm_fp8_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, void* C, int M, int N, int K, int ldc, int epi,
                               const float* a_scale, const float* w_scale, int sm_count, int* err, cudaStream_t stream, const void* resid = nullptr);

// NVFP4 block-scaled GEMM (gemm_nvfp4.cu): e2m1 codes [rows, K/2] bytes (byte maps from tc_make_tmap_fp8_a, 128-row
// boxes, for both operands), unsigned e4m3 scales per 16 elements in the 128 x 4 tiled layout padded to an even number of 128-row
// blocks (launch_nvfp4_sf_tile converts from row-major [rows, K/16]); bf16 C = alpha * (Xq . Wq^T). K % 256 == 0.
bool nvfp4_tc_shape_ok(int M, int N, int K);
size_t nvfp4_sf_tiled_bytes(int rows, int K);
cudaError_t nvfp4_gemm_prepare_device();
cudaError_t launch_nvfp4_sf_tile(const uint8_t* lin, uint8_t* tiled, int rows, int K, cudaStream_t s, bool pad_even = true);
// bf16 rows (tensor scale 1) -> codes [rows, K/2] + scales in the tiled layout (rows of the last block beyond `rows` are left
// as they are: they only meet zero-filled codes). K % 64 == 0.
struct __nv_bfloat16;
cudaError_t launch_nvfp4_act_quant_tiled(const __nv_bfloat16* x, size_t x_stride, uint8_t* packed, uint8_t* tiled, int rows, int K, cudaStream_t s);
// SwiGLU over the tile-interleaved gate/up GEMM output [rows, gu_stride] (256-column tiles: 128 gate, 128 up) fused with the same
// quantiser: codes [rows, I/2] + tiled scales of the [rows, I] activation. I % 128 == 0.
cudaError_t launch_nvfp4_swiglu_quant_tiled(const __nv_bfloat16* gu, int gu_stride, uint8_t* packed, uint8_t* tiled, int rows, int I, cudaStream_t s);
// bn: output tile width, 128 or 256; tmB must have bn-row boxes (tc_make_tmap_fp8_a / tc_make_tmap_fp8_b over the codes).
// resid (optional, bf16 [M, ldc]): C = bf16(resid + bf16(alpha * acc)). q_packed / q_tiled (optional, bn 256, N = 2 * ldc, W rows interleaved
// 128 gate / 128 up per tile): instead of C, the NVFP4 image of the SwiGLU activation [M, ldc] (codes + tiled scales).
cudaError_t nvfp4_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, const uint8_t* sfa_tiled, const uint8_t* sfb_tiled, void* C, int M,
                              int N, int K, int ldc, const float* alpha, int sm_count, int* err, cudaStream_t stream, int bn,
                              const void* resid = nullptr, uint8_t* q_packed = nullptr, uint8_t* q_tiled = nullptr);

// W4A16 GEMM without a bf16 copy of W (gemm_w4a16.cu): int4 group-128 weights in the engine's own image (words with the nibble
// order k0 k2 k4 k6 k1 k3 k5 k7, fp16 scales transposed to [K/128][N]); bit-identical to dequantising and running the bf16 GEMM.
bool w4a16_tc_shape_ok(int M, int N, int K);           // K % 128 == 0, N % 8 == 0
bool w4a16_tc_prefer(int M, int N, int sm_count);       // the fused kernel is the faster route for this launch (weight-streaming-bound passes)
cudaError_t w4a16_gemm_prepare_device();
int w4a16_make_tmap_packed(TcTensorMap* out, const void* packed, uint64_t N, uint64_t K);
cudaError_t launch_w4_repack(const uint32_t* packed, uint32_t* out, size_t words, cudaStream_t s);   // in place is fine
cudaError_t launch_w4_scale_transpose(const void* scales, void* out, int N, int groups, cudaStream_t s);
cudaError_t w4a16_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmP, const void* scale_t, void* C, int M, int N, int K, int ldc, int epi,
                              int sm_count, int* err, cudaStream_t stream, const void* resid = nullptr);
