// Kernel-level C entry points: raw device pointers in, one launch out. They exist so that every
// kernel can be checked against the CPU oracle and timed on its own through the C ABI.
#include "../../include/decidra_b200.h"
#include "attn_tcgen05.h"
#include "common.cuh"
#include "gemm_tcgen05.h"
#include "kernels.h"

namespace {
inline int rc_of(cudaError_t e) { return e == cudaSuccess ? DCD_OK : (e == cudaErrorInvalidValue ? DCD_E_INVALID : DCD_E_CUDA); }
inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }
}  // namespace

#define DISPATCH(dtype, call_f32, call_bf16) ((dtype) == 0 ? rc_of(call_f32) : (dtype) == 1 ? rc_of(call_bf16) : DCD_E_INVALID)

extern "C" {

int dcd_k_gemm_bf16_tc(const void* X, const void* W, void* C, int M, int N, int K, int ldc, int epi, int sm_count, int* err, void* stream) {
  if (!tc_shape_ok(M, N, K) || sm_count <= 0 || (epi != 0 && epi != 1)) return DCD_E_INVALID;
  TcTensorMap ta, tb;
  if (tc_make_tmap_a(&ta, X, M, K) || tc_make_tmap_b(&tb, W, N, K)) return DCD_E_CUDA;
  if (tc_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  return rc_of(tc_gemm_launch(&ta, &tb, C, M, N, K, ldc, epi, sm_count, err, S(stream)));
}

int dcd_k_gemm_bf16_tc_resid(const void* X, const void* W, const void* resid, void* C, int M, int N, int K, int ldc, int sm_count, int* err,
                             void* stream) {
  if (!tc_shape_ok(M, N, K) || sm_count <= 0 || !resid) return DCD_E_INVALID;
  TcTensorMap ta, tb;
  if (tc_make_tmap_a(&ta, X, M, K) || tc_make_tmap_b(&tb, W, N, K)) return DCD_E_CUDA;
  if (tc_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  return rc_of(tc_gemm_launch(&ta, &tb, C, M, N, K, ldc, 0, sm_count, err, S(stream), nullptr, resid));
}

int dcd_k_gemm_fp8_tc(const void* Xq, const void* Wq, void* C, int M, int N, int K, int ldc, int epi, const float* a_scale,
                      const float* w_scale, int sm_count, int* err, void* stream) {
  if (!tc_fp8_shape_ok(M, N, K) || sm_count <= 0 || (epi != 0 && epi != 1) || !a_scale || !w_scale) return DCD_E_INVALID;
  TcTensorMap ta, tb;
  if (tc_make_tmap_fp8_a(&ta, Xq, M, K) || tc_make_tmap_fp8_b(&tb, Wq, N, K)) return DCD_E_CUDA;
  if (tc_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  return rc_of(tc_gemm_fp8_launch(&ta, &tb, C, M, N, K, ldc, epi, a_scale, w_scale, sm_count, err, S(stream)));
}

int dcd_k_quant_fp8_rows(const void* x, size_t x_stride, void* out, float* scales, int rows, int cols, float clip, int dtype, void* stream) {
  return DISPATCH(dtype, launch_quant_fp8_rows<float>((const float*)x, x_stride, (uint8_t*)out, scales, rows, cols, clip, S(stream)),
                  launch_quant_fp8_rows<bf16>((const bf16*)x, x_stride, (uint8_t*)out, scales, rows, cols, clip, S(stream)));
}

int dcd_k_quant_w4_g128(const void* W, void* packed, void* scales, int N, int K, void* stream) {
  return rc_of(launch_quant_w4_g128((const bf16*)W, (uint32_t*)packed, scales, N, K, S(stream)));
}
int dcd_k_w4_repack(const void* packed, const void* scales, void* packed_out, void* scales_t, int N, int K, void* stream) {
  if (N <= 0 || K <= 0 || (K % 128) != 0) return DCD_E_INVALID;
  cudaError_t ce = launch_w4_repack((const uint32_t*)packed, (uint32_t*)packed_out, (size_t)N * (K / 8), S(stream));
  if (ce == cudaSuccess) ce = launch_w4_scale_transpose(scales, scales_t, N, K / 128, S(stream));
  return rc_of(ce);
}
int dcd_k_gemm_w4a16_tc(const void* X, const void* packed, const void* scales_t, const void* resid, void* C, int M, int N, int K, int ldc, int epi,
                        int sm_count, int* err, void* stream) {
  if (!w4a16_tc_shape_ok(M, N, K) || sm_count <= 0 || (epi != 0 && epi != 1) || (resid && epi)) return DCD_E_INVALID;
  if (w4a16_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap ta, tp;
  if (tc_make_tmap_a(&ta, X, M, K) || w4a16_make_tmap_packed(&tp, packed, N, K)) return DCD_E_CUDA;
  return rc_of(w4a16_gemm_launch(&ta, &tp, scales_t, C, M, N, K, ldc, epi, sm_count, err, S(stream), resid));
}
int dcd_k_dequant_w4_g128(const void* packed, const void* scales, void* W, int N, int K, void* stream) {
  return rc_of(launch_dequant_w4_g128((const uint32_t*)packed, scales, (bf16*)W, N, K, S(stream)));
}

int dcd_k_nvfp4_quant_rows(const void* x, size_t x_stride, float global, void* packed, void* scales, int rows, int K, void* stream) {
  return rc_of(launch_nvfp4_quant_rows((const bf16*)x, x_stride, nullptr, global, (uint8_t*)packed, (uint8_t*)scales, rows, K, S(stream)));
}
int dcd_k_nvfp4_dequant_rows(const void* packed, const void* scales, void* out, int rows, int K, void* stream) {
  return rc_of(launch_nvfp4_dequant_rows((const uint8_t*)packed, (const uint8_t*)scales, nullptr, (bf16*)out, rows, K, S(stream)));
}
int dcd_k_nvfp4_fakequant_rows(const void* x, size_t x_stride, float global, void* out, int rows, int K, void* stream) {
  return rc_of(launch_nvfp4_fakequant_rows((const bf16*)x, x_stride, global, (bf16*)out, rows, K, S(stream)));
}

int dcd_k_nvfp4_tile_scales(const void* scales, void* tiled, int rows, int K, void* stream) {
  if (rows <= 0 || K <= 0 || (K % 64) != 0) return DCD_E_INVALID;
  return rc_of(launch_nvfp4_sf_tile((const uint8_t*)scales, (uint8_t*)tiled, rows, K, S(stream), false));
}

int dcd_k_nvfp4_quant_act_tiled(const void* x, size_t x_stride, void* packed, void* tiled, int rows, int K, void* stream) {
  return rc_of(launch_nvfp4_act_quant_tiled((const bf16*)x, x_stride, (uint8_t*)packed, (uint8_t*)tiled, rows, K, S(stream)));
}

int dcd_k_nvfp4_swiglu_quant_tiled(const void* gu, int gu_stride, void* packed, void* tiled, int rows, int I, void* stream) {
  return rc_of(launch_nvfp4_swiglu_quant_tiled((const bf16*)gu, gu_stride, (uint8_t*)packed, (uint8_t*)tiled, rows, I, S(stream)));
}

int dcd_k_gemm_nvfp4_tc(const void* xq, const void* x_scales, const void* wq, const void* w_scales, void* C, int M, int N, int K, int ldc,
                        const float* alpha, int sm_count, int* err, int tile_n, void* stream) {
  const int tile_w = tile_n >= 1000 ? tile_n - 1000 : tile_n;  // + 1000: scale copies issued by a thread of their own
  if (!nvfp4_tc_shape_ok(M, N, K) || sm_count <= 0 || (tile_w != 128 && tile_w != 256)) return DCD_E_INVALID;
  if (nvfp4_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap ta, tb;
  if (tc_make_tmap_fp8_a(&ta, xq, M, K / 2) || (tile_w == 128 ? tc_make_tmap_fp8_a(&tb, wq, N, K / 2) : tc_make_tmap_fp8_b(&tb, wq, N, K / 2))) return DCD_E_CUDA;
  uint8_t *sa = nullptr, *sb = nullptr;  // scales re-laid in 128 x 4 tiles for the duration of the call
  cudaStream_t st = S(stream);
  if (cudaMallocAsync(&sa, nvfp4_sf_tiled_bytes(M, K), st) != cudaSuccess) return DCD_E_OOM;
  if (cudaMallocAsync(&sb, nvfp4_sf_tiled_bytes(N, K), st) != cudaSuccess) { cudaFreeAsync(sa, st); return DCD_E_OOM; }
  cudaError_t ce = launch_nvfp4_sf_tile((const uint8_t*)x_scales, sa, M, K, st);
  if (ce == cudaSuccess) ce = launch_nvfp4_sf_tile((const uint8_t*)w_scales, sb, N, K, st);
  if (ce == cudaSuccess) ce = nvfp4_gemm_launch(&ta, &tb, sa, sb, C, M, N, K, ldc, alpha, sm_count, err, st, tile_n);
  cudaFreeAsync(sa, st);
  cudaFreeAsync(sb, st);
  return rc_of(ce);
}

int dcd_k_gemm_nvfp4_tc_tiled(const void* xq, const void* x_tiled, const void* wq, const void* w_tiled, void* C, int M, int N, int K, int ldc,
                              const float* alpha, int sm_count, int* err, int tile_n, const void* resid, void* q_packed, void* q_tiled, void* stream) {
  const int tile_w = tile_n >= 1000 ? tile_n - 1000 : tile_n;
  if (!nvfp4_tc_shape_ok(M, N, K) || sm_count <= 0 || (tile_w != 128 && tile_w != 256)) return DCD_E_INVALID;
  if (nvfp4_gemm_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap ta, tb;
  if (tc_make_tmap_fp8_a(&ta, xq, M, K / 2) || (tile_w == 128 ? tc_make_tmap_fp8_a(&tb, wq, N, K / 2) : tc_make_tmap_fp8_b(&tb, wq, N, K / 2))) return DCD_E_CUDA;
  return rc_of(nvfp4_gemm_launch(&ta, &tb, (const uint8_t*)x_tiled, (const uint8_t*)w_tiled, C, M, N, K, ldc, alpha, sm_count, err, S(stream), tile_n, resid,
                                 (uint8_t*)q_packed, (uint8_t*)q_tiled));
}

void dcd_debug_set_gemm_group_m(int group_m) { tc_gemm_set_group_m(group_m); }

int dcd_k_gemm_fma(const void* X, const void* W, void* C, int M, int N, int K, int dtype, void* stream) {
  return DISPATCH(dtype, launch_gemm_fma<float>((const float*)X, (const float*)W, (float*)C, M, N, K, N, S(stream)),
                  launch_gemm_fma<bf16>((const bf16*)X, (const bf16*)W, (bf16*)C, M, N, K, N, S(stream)));
}

int dcd_k_rmsnorm(const void* x, const void* w, void* out, int rows, int cols, float eps, int zero_centered, int dtype, void* stream) {
  return DISPATCH(dtype, launch_rmsnorm<float>((const float*)x, (const float*)w, (float*)out, rows, cols, eps, zero_centered != 0, S(stream)),
                  launch_rmsnorm<bf16>((const bf16*)x, (const bf16*)w, (bf16*)out, rows, cols, eps, zero_centered != 0, S(stream)));
}

int dcd_k_add_rmsnorm(const void* x, const void* mix, const void* w, void* residual, void* out, int rows, int cols, float eps, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_add_rmsnorm<float>((const float*)x, (const float*)mix, (const float*)w, (float*)residual, (float*)out, rows, cols, eps, S(stream)),
                  launch_add_rmsnorm<bf16>((const bf16*)x, (const bf16*)mix, (const bf16*)w, (bf16*)residual, (bf16*)out, rows, cols, eps, S(stream)));
}

int dcd_k_rmsnorm_gated(const void* x, const void* z, int z_stride, const void* w, void* out, int tokens, int heads, int cols, float eps, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_rmsnorm_gated<float>((const float*)x, (const float*)z, z_stride, (const float*)w, (float*)out, tokens, heads, cols, eps, S(stream)),
                  launch_rmsnorm_gated<bf16>((const bf16*)x, (const bf16*)z, z_stride, (const bf16*)w, (bf16*)out, tokens, heads, cols, eps, S(stream)));
}

int dcd_k_silu_mul(const void* gate, const void* up, void* out, size_t n, int dtype, void* stream) {
  return DISPATCH(dtype, launch_silu_mul<float>((const float*)gate, (const float*)up, (float*)out, n, S(stream)),
                  launch_silu_mul<bf16>((const bf16*)gate, (const bf16*)up, (bf16*)out, n, S(stream)));
}

int dcd_k_add(const void* a, const void* b, void* out, size_t n, int dtype, void* stream) {
  return DISPATCH(dtype, launch_add<float>((const float*)a, (const float*)b, (float*)out, n, S(stream)),
                  launch_add<bf16>((const bf16*)a, (const bf16*)b, (bf16*)out, n, S(stream)));
}

int dcd_k_conv1d_silu(const void* x, int x_stride, const void* hist, const void* w, void* out, const int32_t* cu_seqlens,
                      const int32_t* tok_q, int total, int ch, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_conv1d_silu<float>((const float*)x, x_stride, (const float*)hist, (const float*)w, (float*)out, cu_seqlens, tok_q, total, ch, S(stream)),
                  launch_conv1d_silu<bf16>((const bf16*)x, x_stride, (const bf16*)hist, (const bf16*)w, (bf16*)out, cu_seqlens, tok_q, total, ch, S(stream)));
}

int dcd_k_gdn_prepare(const void* conv, int conv_stride, const void* b, const void* a, int ba_stride, const float* A_log, const float* dt_bias,
                      float* qf, float* kf, float* g, float* beta, int T, int nk, int nv, int dk, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_gdn_prepare<float>((const float*)conv, conv_stride, (const float*)b, (const float*)a, ba_stride, A_log, dt_bias, qf, kf, g, beta, T, nk, nv, dk, S(stream)),
                  launch_gdn_prepare<bf16>((const bf16*)conv, conv_stride, (const bf16*)b, (const bf16*)a, ba_stride, A_log, dt_bias, qf, kf, g, beta, T, nk, nv, dk, S(stream)));
}

int dcd_k_gdn_recurrent(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                        const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int nk, int nv, int dk,
                        int dv, int narrow, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_gdn_recurrent<float>(qf, kf, (const float*)conv, conv_stride, g, beta, seed, final_state, (float*)out, cu_seqlens, B, nk, nv, dk, dv, narrow != 0, S(stream)),
                  launch_gdn_recurrent<bf16>(qf, kf, (const bf16*)conv, conv_stride, g, beta, seed, final_state, (bf16*)out, cu_seqlens, B, nk, nv, dk, dv, narrow != 0, S(stream)));
}

int dcd_k_gdn_chunked(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                      const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int nk, int nv, int dk, int dv,
                      int narrow, int dtype, void* stream) {
  if (!gdn_chunked_supported(dk, dv)) return DCD_E_INVALID;
  if ((dtype == 0 ? gdn_chunked_prepare_device<float>() : gdn_chunked_prepare_device<bf16>()) != cudaSuccess) return DCD_E_CUDA;
  return DISPATCH(dtype,
                  launch_gdn_chunked<float>(qf, kf, (const float*)conv, conv_stride, g, beta, seed, final_state, (float*)out, cu_seqlens, B, nk, nv, dk, dv, narrow != 0, S(stream)),
                  launch_gdn_chunked<bf16>(qf, kf, (const bf16*)conv, conv_stride, g, beta, seed, final_state, (bf16*)out, cu_seqlens, B, nk, nv, dk, dv, narrow != 0, S(stream)));
}

int dcd_k_gdn_chunked_tc(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                         const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens, int nk,
                         int nv, int dk, int dv, int* err, int dtype, void* stream) {
  if (!gdn_tc_supported(dk, dv) || total_tokens <= 0 || nk <= 0 || nv % nk != 0) return DCD_E_INVALID;
  if ((dtype == 0 ? gdn_tc_prepare_device<float>() : gdn_tc_prepare_device<bf16>()) != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap maps[3];
  if (gdn_tc_make_maps(maps, qf, kf, conv, conv_stride, 2 * nk * dk + nv * dv, dtype == 0 ? 4 : 2, total_tokens, nk) != 0) return DCD_E_CUDA;
  return DISPATCH(dtype,
                  launch_gdn_tc<float>(maps, (const float*)conv, conv_stride, g, beta, seed, final_state, (float*)out, cu_seqlens, B, nk, nv, err, S(stream)),
                  launch_gdn_tc<bf16>(maps, (const bf16*)conv, conv_stride, g, beta, seed, final_state, (bf16*)out, cu_seqlens, B, nk, nv, err, S(stream)));
}

int dcd_k_gdn_wy_tc(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                         const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens, int nk,
                         int nv, int dk, int dv, int* err, int dtype, void* stream) {
  if (!gdn_tc_supported(dk, dv) || total_tokens <= 0 || nk <= 0 || nv % nk != 0) return DCD_E_INVALID;
  if ((dtype == 0 ? gdn_wy_prepare_device<float>() : gdn_wy_prepare_device<bf16>()) != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap maps[3];
  if (gdn_tc_make_maps(maps, qf, kf, conv, conv_stride, 2 * nk * dk + nv * dv, dtype == 0 ? 4 : 2, total_tokens, nk) != 0) return DCD_E_CUDA;
  return DISPATCH(dtype,
                  launch_gdn_wy<float>(maps, (const float*)conv, conv_stride, g, beta, seed, final_state, (float*)out, cu_seqlens, B, nk, nv, err, S(stream)),
                  launch_gdn_wy<bf16>(maps, (const bf16*)conv, conv_stride, g, beta, seed, final_state, (bf16*)out, cu_seqlens, B, nk, nv, err, S(stream)));
}

int dcd_k_gdn_wy_tc_phases(const float* qf, const float* kf, const void* conv, int conv_stride, const float* g, const float* beta,
                         const float* seed, float* final_state, void* out, const int32_t* cu_seqlens, int B, int total_tokens, int nk,
                         int nv, int dk, int dv, int* err, int dtype, unsigned long long* phases, void* stream) {
  if (!gdn_tc_supported(dk, dv) || total_tokens <= 0 || nk <= 0 || nv % nk != 0) return DCD_E_INVALID;
  if ((dtype == 0 ? gdn_wy_prepare_device<float>() : gdn_wy_prepare_device<bf16>()) != cudaSuccess) return DCD_E_CUDA;
  TcTensorMap maps[3];
  if (gdn_tc_make_maps(maps, qf, kf, conv, conv_stride, 2 * nk * dk + nv * dv, dtype == 0 ? 4 : 2, total_tokens, nk) != 0) return DCD_E_CUDA;
  return DISPATCH(dtype,
                  launch_gdn_wy<float>(maps, (const float*)conv, conv_stride, g, beta, seed, final_state, (float*)out, cu_seqlens, B, nk, nv, err, S(stream), phases),
                  launch_gdn_wy<bf16>(maps, (const bf16*)conv, conv_stride, g, beta, seed, final_state, (bf16*)out, cu_seqlens, B, nk, nv, err, S(stream), phases));
}

int dcd_k_qk_norm_rope(const void* qg, int qg_stride, const void* kraw, int k_stride, const void* qw, const void* kw, const void* cos_t,
                       const void* sin_t, const int32_t* positions, int max_pos, void* q, void* k, int T, int heads, int kv, int hd,
                       int rotary_dim, float eps, int* err, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_qk_norm_rope<float>((const float*)qg, qg_stride, (const float*)kraw, k_stride, (const float*)qw, (const float*)kw, (const float*)cos_t, (const float*)sin_t, positions, 0, max_pos, (float*)q, (float*)k, kv * hd, T, heads, kv, hd, rotary_dim, eps, err, S(stream)),
                  launch_qk_norm_rope<bf16>((const bf16*)qg, qg_stride, (const bf16*)kraw, k_stride, (const bf16*)qw, (const bf16*)kw, (const bf16*)cos_t, (const bf16*)sin_t, positions, 0, max_pos, (bf16*)q, (bf16*)k, kv * hd, T, heads, kv, hd, rotary_dim, eps, err, S(stream)));
}

int dcd_k_attention(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                    const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out, const int32_t* cu_seqlens,
                    const int32_t* tok_q, int T, int heads, int kv, int hd, int split, int dtype, void* stream) {
  return DISPATCH(dtype,
                  launch_attn_fma<float>((const float*)q, (const float*)k_own, k_stride, (const float*)v_own, v_stride, (const float*)k_state, (const float*)v_state, n_state, (const float*)gate_qg, qg_stride, (float*)out, cu_seqlens, tok_q, T, heads, kv, hd, split, S(stream)),
                  launch_attn_fma<bf16>((const bf16*)q, (const bf16*)k_own, k_stride, (const bf16*)v_own, v_stride, (const bf16*)k_state, (const bf16*)v_state, n_state, (const bf16*)gate_qg, qg_stride, (bf16*)out, cu_seqlens, tok_q, T, heads, kv, hd, split, S(stream)));
}

int dcd_k_attention_tc(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                       const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out, const int32_t* cu_seqlens,
                       int32_t* tile_cu, int B, int T, int heads, int kv, int hd, int* err, void* stream) {
  if (!attn_tc_supported(heads, kv, hd) || B <= 0 || T <= 0) return DCD_E_INVALID;
  if (attn_tc_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  const int tt = attn_tc_tokens_per_tile(heads, kv);
  AttnTcMaps maps;
  if (attn_tc_make_maps(&maps, q, k_own, k_stride, v_own, v_stride, k_state, v_state, n_state, T, heads, kv, hd)) return DCD_E_CUDA;
  cudaError_t ce = attn_tc_build_tiles(cu_seqlens, B, tt, tile_cu, S(stream));
  if (ce != cudaSuccess) return rc_of(ce);
  return rc_of(attn_tc_launch(&maps, cu_seqlens, tile_cu, B, n_state, T, (T + tt - 1) / tt + B, heads, kv, hd, gate_qg, qg_stride, out, err, S(stream)));
}

int dcd_k_attention_tc_split(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                             const void* v_state, int n_state, const void* gate_qg, int qg_stride, void* out, const int32_t* cu_seqlens,
                             int32_t* tile_cu, int B, int T, int heads, int kv, int hd, int* err, int n_split, void* workspace,
                             size_t workspace_bytes, void* stream) {
  if (!attn_tc_supported(heads, kv, hd) || B <= 0 || T <= 0 || n_split < 0) return DCD_E_INVALID;
  if (attn_tc_prepare_device() != cudaSuccess) return DCD_E_CUDA;
  const int tt = attn_tc_tokens_per_tile(heads, kv), max_tiles = (T + tt - 1) / tt + B;
  if (n_split == 0) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return DCD_E_CUDA;
    n_split = attn_tc_pick_split(max_tiles, kv, n_state, sms);
  }
  if (n_split > 1 && (!workspace || workspace_bytes < (size_t)n_split * max_tiles * kv * 128 * 1032)) return DCD_E_INVALID;
  AttnTcMaps maps;
  if (attn_tc_make_maps(&maps, q, k_own, k_stride, v_own, v_stride, k_state, v_state, n_state, T, heads, kv, hd)) return DCD_E_CUDA;
  cudaError_t ce = attn_tc_build_tiles(cu_seqlens, B, tt, tile_cu, S(stream));
  if (ce != cudaSuccess) return rc_of(ce);
  return rc_of(attn_tc_launch(&maps, cu_seqlens, tile_cu, B, n_state, T, max_tiles, heads, kv, hd, gate_qg, qg_stride, out, err, S(stream), n_split, workspace));
}

int dcd_k_readout(const float* x, const float* W, float* out, int B, int H, int R, void* stream) {
  return rc_of(launch_readout(x, W, out, B, H, R, S(stream)));
}

}  // extern "C"
