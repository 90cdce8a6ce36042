// Launch wrappers of kernels.cu (all enqueue on the given stream and return the launch status).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

cudaError_t launch_pack(const int32_t* lens, int B, int total, int pos_start, int32_t* cu, int32_t* last_row, int32_t* tok_q,
                        int32_t* tok_pos, int* err, cudaStream_t s, const int32_t* pos_start_q = nullptr);
template <typename T>
cudaError_t launch_embed(const T* table, const uint32_t* ids, T* out, int rows, int H, int vocab, int* err, cudaStream_t s);
template <typename T>
cudaError_t launch_rmsnorm(const T* x, const T* w, T* out, int rows, int cols, float eps, bool zero_centered, cudaStream_t s);
template <typename T>
cudaError_t launch_add_rmsnorm(const T* x, const T* mix, const T* w, T* residual, T* out, int rows, int cols, float eps, cudaStream_t s);
// RMSNorm(1+w) / residual add + RMSNorm(1+w) whose output row goes straight to the NVFP4 operand format of the block-scaled GEMM
// (codes [rows, cols/2], e4m3 scales in the 128 x 4 tiled layout); the bf16 output is not written. cols % 64 == 0.
cudaError_t launch_rmsnorm_nvfp4(const __nv_bfloat16* x, const __nv_bfloat16* w, uint8_t* q_packed, uint8_t* q_tiled, int rows, int cols, float eps,
                                 cudaStream_t s);
cudaError_t launch_add_rmsnorm_nvfp4(const __nv_bfloat16* x, const __nv_bfloat16* mix, const __nv_bfloat16* w, __nv_bfloat16* residual,
                                     uint8_t* q_packed, uint8_t* q_tiled, int rows, int cols, float eps, cudaStream_t s);
template <typename T>
cudaError_t launch_final_norm_rows(const T* x, const T* w, float* out, const int32_t* rows_idx, int B, int cols, float eps, cudaStream_t s);
cudaError_t launch_rmsnorm_gated_nvfp4(const __nv_bfloat16* x, const __nv_bfloat16* z, int z_stride, const __nv_bfloat16* w, uint8_t* q_packed, uint8_t* q_tiled,
                                       int tokens, int heads, float eps, cudaStream_t s);
template <typename T>
cudaError_t launch_rmsnorm_gated(const T* x, const T* z, int z_stride, const T* w, T* out, int tokens, int heads, int cols, float eps, cudaStream_t s);
template <typename T>
cudaError_t launch_add(const T* a, const T* b, T* out, size_t n, cudaStream_t s);
template <typename T>
cudaError_t launch_silu_mul(const T* g, const T* u, T* out, size_t n, cudaStream_t s);
template <typename T>
cudaError_t launch_silu_mul_interleaved(const T* gu, int gu_stride, T* out, int tokens, int I, cudaStream_t s);
template <typename T>
cudaError_t launch_qk_norm_rope(const T* qg, int qg_stride, const T* kraw, int k_stride, const T* qw, const T* kw, const T* cos_t,
                                const T* sin_t, const int32_t* positions, int pos_base, int max_pos, T* q, T* k, int k_out_stride,
                                int tokens, int heads, int kv, int hd, int rotary_dim, float eps, int* err, cudaStream_t s);
template <typename T>
cudaError_t launch_attn_fma(const T* q, const T* k_own, int k_stride, const T* v_own, int v_stride, const T* k_state,
                            const T* v_state, int n_state, const T* gate_qg, int qg_stride, T* out, const int32_t* cu,
                            const int32_t* tok_q, int tokens, int heads, int kv, int hd, int split, cudaStream_t s, int tok_base = 0);
template <typename T>
cudaError_t launch_conv1d_silu(const T* x, int x_stride, const T* hist, const T* w, T* out, const int32_t* cu,
                               const int32_t* tok_q, int tokens, int ch, cudaStream_t s, int tok_base = 0);
template <typename T>
cudaError_t launch_gdn_prepare(const T* conv, int conv_stride, const T* b, const T* a, int ba_stride, const float* A_log,
                               const float* dt_bias, float* qf, float* kf, float* g, float* beta, int tokens, int nk, int nv,
                               int dk, cudaStream_t s);
template <typename T>
cudaError_t launch_gdn_recurrent(const float* qf, const float* kf, const T* conv, int conv_stride, const float* g, const float* beta,
                                 const float* seed, float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int dk,
                                 int dv, bool few_sequences, cudaStream_t s);
cudaError_t launch_readout(const float* x, const float* W, float* out, int B, int H, int R, cudaStream_t s);
template <typename T>
cudaError_t launch_gemm_fma(const T* X, const T* W, T* C, int M, int N, int K, int ldc, cudaStream_t s);
template <typename T>
cudaError_t launch_copy_rows(const T* src, int src_stride, T* dst, int dst_stride, int rows, int cols, cudaStream_t s);
template <typename T>
cudaError_t launch_to_f32(const T* src, float* dst, size_t n, cudaStream_t s);
template <typename T>
cudaError_t launch_from_f32(const float* src, T* dst, size_t n, cudaStream_t s);

uint64_t gen_tensor_key(uint64_t seed, int layer, int kind);
template <typename T>
cudaError_t launch_gen_tensor(T* dst, uint64_t key, uint64_t first, uint64_t count, int cols, int dist, float p0, float p1, float c,
                              bool round_bf, int mode, int row_offset, int dst_stride, cudaStream_t s);
template <typename T>
cudaError_t launch_place_rows(const T* src, T* dst, size_t rows, int cols, int mode, int row_offset, int dst_stride, bool inverse,
                              cudaStream_t s);
// Checkpoint formats -> engine layout (a chunk of rows starting at row_start of the logical tensor).
// src_dt: 0 = f32, 1 = f16, 2 = bf16.
template <typename T>
cudaError_t launch_place_rows_cvt(const void* src, int src_dt, T* dst, size_t n_rows, int cols, size_t row_start, int mode, int row_offset,
                                  int dst_stride, cudaStream_t s);
// compressed-tensors pack-quantized int4 (zp == nullptr: symmetric, zero point 8); row_start must be a multiple of 8
// compressed-tensors int4 group-128 rows into a W4 engine image as they are (nibble order permuted, scales bf16 -> fp16); *flag is
// raised when a zero point is not 8 or a scale is not exact in fp16
cudaError_t launch_adopt_ct_w4_rows(const int32_t* packed, const __nv_bfloat16* scale, const int32_t* zp, uint32_t* dst_q, void* dst_scale, size_t n_rows,
                                    int in_dim, size_t row_start, int mode, int row_offset, int* flag, cudaStream_t s);
template <typename T>
cudaError_t launch_dequant_ct_w4_place(const int32_t* packed, const __nv_bfloat16* scale, const int32_t* zp, T* dst, size_t n_rows, int in_dim,
                                       int group_size, size_t row_start, int mode, int row_offset, int dst_stride, cudaStream_t s);
// compressed-tensors nvfp4-pack-quantized weights: e2m1 pairs, row-major e4m3 scale per 16, f32 tensor scale
template <typename T>
cudaError_t launch_dequant_ct_nvfp4_place(const uint8_t* packed, const uint8_t* scales, float global, T* dst, size_t n_rows, int K,
                                          size_t row_start, int mode, int row_offset, int dst_stride, cudaStream_t s);

// Chunked tensor-core form of the gated delta rule (gdn_chunked.cu); dk must be 128 and dv a multiple of 64.
bool gdn_chunked_supported(int dk, int dv);
template <typename T>
cudaError_t gdn_chunked_prepare_device();
template <typename T>
cudaError_t launch_gdn_chunked(const float* qf, const float* kf, const T* conv, int conv_stride, const float* g, const float* beta,
                               const float* seed, float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int dk, int dv,
                               bool few_sequences, cudaStream_t s);

// tcgen05 (kind::tf32) form of the chunked gated delta rule (gdn_tcgen05.cu); dk and dv must both be 128.
// maps[0..2] are TMA descriptors of the f32 q/k buffers [tokens, nk*128] and (16-bit storage) of the conv
// output [tokens, conv_cols], made by gdn_tc_make_maps with rows = the token count of this launch, so that
// a partial last chunk reads the zero fill.
struct TcTensorMap;
bool gdn_tc_supported(int dk, int dv);
template <typename T>
cudaError_t gdn_tc_prepare_device();
int gdn_tc_make_maps(TcTensorMap maps[3], const float* qf, const float* kf, const void* conv, int conv_stride, int conv_cols, int elem_size,
                     int tokens, int nk);
template <typename T>
cudaError_t launch_gdn_tc(const TcTensorMap maps[3], const T* conv, int conv_stride, const float* g, const float* beta, const float* seed,
                          float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int* err, cudaStream_t s);
// The same function in WY form (gdn_wy.cu): the triangular system of a chunk is inverted blockwise once, everything else is a
// tensor-core product. Same tensor maps, same arguments.
template <typename T>
cudaError_t gdn_wy_prepare_device();
template <typename T>
cudaError_t launch_gdn_wy(const TcTensorMap maps[3], const T* conv, int conv_stride, const float* g, const float* beta, const float* seed,
                          float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int* err, cudaStream_t s, unsigned long long* phases = nullptr);

// Per-row FP8 E4M3 quantisation: scale[row] = max(absmax*clip, 1e-10)/448, out = e4m3(x/scale).
template <typename T>
cudaError_t launch_quant_fp8_rows(const T* x, size_t x_stride, uint8_t* out, float* scales, int rows, int cols, float clip, cudaStream_t s);

// W4A16 group-128 weights: packed [N, K/8] words (nibble k of word j = input 8j+k, zero-point 8) and
// fp16 scales [N, ceil(K/128)]. K % 8 == 0.
// perm: words in the engine's nibble order [k0 k2 k4 k6 k1 k3 k5 k7] instead of the compressed-tensors order k0..k7
cudaError_t launch_quant_w4_g128(const __nv_bfloat16* W, uint32_t* packed, void* scales, int N, int K, cudaStream_t s, bool perm = false);
cudaError_t launch_dequant_w4_g128(const uint32_t* packed, const void* scales, __nv_bfloat16* W, int N, int K, cudaStream_t s, bool perm = false);

// NVFP4 (e2m1 + e4m3 per 16 + f32 per tensor). K % 16 == 0. Scales row-major [rows, K/16].
cudaError_t launch_absmax_bf16(const __nv_bfloat16* x, size_t n, unsigned int* out, cudaStream_t s);
cudaError_t launch_nvfp4_global(const unsigned int* amax, float* global, float* alpha, float input_global, cudaStream_t s);
cudaError_t launch_nvfp4_quant_rows(const __nv_bfloat16* x, size_t x_stride, const float* global_ptr, float global_imm, uint8_t* packed,
                                    uint8_t* scales, int rows, int K, cudaStream_t s);
cudaError_t launch_nvfp4_fakequant_rows(const __nv_bfloat16* x, size_t x_stride, float global_imm, __nv_bfloat16* out, int rows, int K,
                                        cudaStream_t s);
cudaError_t launch_nvfp4_dequant_rows(const uint8_t* packed, const uint8_t* scales, const float* global_ptr, __nv_bfloat16* out, int rows,
                                      int K, cudaStream_t s);
