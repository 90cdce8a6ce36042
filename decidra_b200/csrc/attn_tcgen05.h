// Host interface of the tcgen05 varlen attention kernel (attn_tcgen05.cu).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "gemm_tcgen05.h"

struct AttnTcMaps { TcTensorMap q, k_own, v_own, k_state, v_state; };

// bf16, head_dim 256, 6 query heads per KV head (the d3-turbo shape).
bool attn_tc_supported(int heads, int kv, int hd);
int attn_tc_tokens_per_tile(int heads, int kv);
cudaError_t attn_tc_prepare_device();
// tile_cu[B+1] = prefix sum over sequences of ceil(len / tokens_per_tile); one launch per pass.
cudaError_t attn_tc_build_tiles(const int32_t* cu, int B, int tokens_per_tile, int32_t* tile_cu, cudaStream_t s);
// TMA descriptors of one layer's operands. q [T,heads,hd]; own K/V rows with element strides;
// state K/V [n_state, kv*hd] contiguous (ignored when n_state == 0). 0 on success.
int attn_tc_make_maps(AttnTcMaps* m, const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                      const void* v_state, int n_state, int T, int heads, int kv, int hd);
// max_tiles >= tile_cu[B] (e.g. ceil(T / tokens_per_tile) + B); surplus CTAs exit at once.
// n_split > 1: the key tiles of every (token tile, KV head) are split over n_split CTAs whose parts a second kernel merges;
// workspace then holds n_split * max_tiles * kv * 128 rows of (256 + 2) floats (attn_tc_pick_split never asks for more than
// attn_tc_split_workspace_bytes(sm_count)).
cudaError_t attn_tc_launch(const AttnTcMaps* m, const int32_t* cu, const int32_t* tile_cu, int B, int n_state, int T, int max_tiles,
                           int heads, int kv, int hd, const void* gate_qg, int qg_stride, void* out, int* err, cudaStream_t s, int n_split = 1,
                           void* workspace = nullptr);
// Parts per (token tile, KV head) for a launch of max_tiles x kv CTAs over n_state cached keys: 1 unless the launch has no more CTAs
// than there are SMs and the state is at least eight key tiles long; then as many as bring the grid to about two CTAs per SM, with
// at least two key tiles per part.
int attn_tc_pick_split(int max_tiles, int kv, int n_state, int sm_count);
size_t attn_tc_split_workspace_bytes(int sm_count);
