// dcd_k_attention_tc_noalloc: the tensor-core attention launch for callers that must not allocate.
//
// Who needs this: a serving worker that drives the kernels from its request thread cannot afford
// cudaMalloc/cudaFree there — both synchronise the whole device, so one call stalls every other
// stream (other replicas' engines in the same process included) — and a host that has already
// committed the GPU's memory to weights and state caches, with its own head-room accounting, cannot
// risk an allocation that fails in the middle of a request. The ordinary entry point,
// dcd_k_attention_tc, asks the caller for a device scratch array (the per-sequence tile prefix sum);
// a caller that has no allocator to take that from uses this variant, whose scratch is a fixed
// array inside the library image.
//
// The scratch is a file-scope __device__ array, so every GPU that loads the library carries its
// 16 KB until the process exits, and the batch size is capped at DCD_NOALLOC_MAX_SEQUENCES.
#include <cstdio>
#include <mutex>

#include "../../include/decidra_b200.h"
#include "attn_tcgen05.h"
#include "common.cuh"

namespace {

constexpr int MAX_SEQ = DCD_NOALLOC_MAX_SEQUENCES;
constexpr int MAX_DEVICES = 64;

// Prefix sum of token tiles per packed sequence: MAX_SEQ + 1 entries, rewritten in full
// ([0, B]) by the tile-scan kernel at the start of every call.
static __device__ __align__(256) int32_t g_tile_scratch[MAX_SEQ + 1];

// In host code `g_tile_scratch` is only a stand-in for the symbol; the address a kernel may
// dereference has to be asked for, per device, with that device current.
int32_t* g_scratch_addr[MAX_DEVICES] = {};
std::mutex g_setup_mutex;

void say(char* msg, size_t len, const char* text) {
  if (msg && len) snprintf(msg, len, "%s", text);
}

// Returns the device address of the scratch array on the current device (set-up on first use).
int32_t* scratch_for_current_device(char* msg, size_t len) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) {
    say(msg, len, "dcd_k_attention_tc_noalloc: cannot identify the current device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    void* ptr = nullptr;
    const cudaError_t ce = cudaGetSymbolAddress(&ptr, g_tile_scratch);
    if (ce != cudaSuccess || !ptr) {
      if (msg && len) snprintf(msg, len, "dcd_k_attention_tc_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(ce));
      return nullptr;
    }
    if (attn_tc_prepare_device() != cudaSuccess) {
      say(msg, len, "dcd_k_attention_tc_noalloc: could not raise the kernel's shared-memory limit");
      return nullptr;
    }
    g_scratch_addr[dev] = static_cast<int32_t*>(ptr);
  }
  return g_scratch_addr[dev];
}

}  // namespace

extern "C" int dcd_k_attention_tc_noalloc(const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride,
                                          const void* k_state, const void* v_state, int n_state, const void* gate_qg, int qg_stride,
                                          void* out, const int32_t* cu_seqlens, int B, int T, int heads, int kv, int hd, int* err,
                                          void* stream, char* msg, size_t msg_len) {
  if (msg && msg_len) msg[0] = 0;
  if (!attn_tc_supported(heads, kv, hd)) {
    say(msg, msg_len, "dcd_k_attention_tc_noalloc: only bf16, head_dim 256 with 6 query heads per KV head is supported");
    return DCD_E_UNSUPPORTED;
  }
  if (B <= 0 || T <= 0 || !q || !k_own || !v_own || !out || !cu_seqlens) {
    say(msg, msg_len, "dcd_k_attention_tc_noalloc: empty batch or null operand");
    return DCD_E_INVALID;
  }
  if (B > MAX_SEQ) {
    if (msg && msg_len)
      snprintf(msg, msg_len, "dcd_k_attention_tc_noalloc: %d packed sequences exceed the built-in scratch of %d; use dcd_k_attention_tc with caller scratch", B, MAX_SEQ);
    return DCD_E_INVALID;
  }
  int32_t* tile_cu = scratch_for_current_device(msg, msg_len);
  if (!tile_cu) return DCD_E_CUDA;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int tt = attn_tc_tokens_per_tile(heads, kv);
  AttnTcMaps maps;
  if (attn_tc_make_maps(&maps, q, k_own, k_stride, v_own, v_stride, k_state, v_state, n_state, T, heads, kv, hd)) {
    say(msg, msg_len, "dcd_k_attention_tc_noalloc: cuTensorMapEncodeTiled rejected an operand (alignment or stride)");
    return DCD_E_CUDA;
  }
  // The scan rewrites entries [0, B] before the attention kernel reads them, so nothing left by an
  // earlier call is ever consumed and nothing has to be cleared.
  cudaError_t ce = attn_tc_build_tiles(cu_seqlens, B, tt, tile_cu, s);
  if (ce == cudaSuccess)
    ce = attn_tc_launch(&maps, cu_seqlens, tile_cu, B, n_state, T, (T + tt - 1) / tt + B, heads, kv, hd, gate_qg, qg_stride, out, err, s);
  if (ce != cudaSuccess) {
    if (msg && msg_len) snprintf(msg, msg_len, "dcd_k_attention_tc_noalloc: launch failed: %s", cudaGetErrorString(ce));
    return DCD_E_CUDA;
  }
  return DCD_OK;
}
