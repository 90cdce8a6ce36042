// Host orchestration and C ABI of the state-once question path.
//
// Mirrors, in C++ behind include/decidra_b200.h, what juanqui/decidra's Engine does for this
// path: Engine::capture_state_mm (native/src/engine.rs:4616-4763),
// Engine::state_once_batch_rows(_inner) (:4866-4987), run_layer_batch (:1725-1788),
// full_attention_batch (:1790-2142), gdn_batch (:2144-2591), mlp (:2794-2885),
// decision_logits_split (:4585-4601) and StateCache offload/restore (:559-648).
// Differences by design: one fused projection GEMM per mixer (q|gate|k|v, and
// qkv|z|b|a), SwiGLU folded into the gate/up GEMM epilogue, no K/V concatenation copies
// (attention reads the cached state and the question's own rows in place), no host round
// trip before the readout, packing metadata built on the device.
#include <algorithm>
#include <cmath>
#include <unistd.h>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <thread>
#include <vector>

#include "../../include/decidra_b200.h"
#include "attn_tcgen05.h"
#include "checkpoint.h"
#include "common.cuh"
#include "gemm_tcgen05.h"
#include "host_logic.h"
#include "kernels.h"
#include "tc_common.cuh"

namespace {

// The give-up path of the tensor-core kernels on its own, for the test that makes a bounded wait run out: one warp holds a
// TMEM allocation (as every tcgen05 kernel here does) and waits, with the same bounded wait, on an mbarrier that nothing will
// ever arrive at. After `polls` polls it does what the real kernels do: raise the error word, pause for work in flight (there
// is none here), free the TMEM, return. Nothing traps, spins without limit or touches memory it does not own.
__global__ void __launch_bounds__(32, 1) bounded_wait_probe_kernel(int* __restrict__ err, uint32_t polls, int code) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    tcc::mbar_init(tcc::smem_u32(&bar), 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tcc::smem_u32(&tmem_holder)), "r"(32u) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  tcc::tc_fence_before();
  __syncthreads();
  tcc::tc_fence_after();
  const uint32_t tmem_base = tmem_holder;
  bool ok = true;
  if (threadIdx.x == 0) ok = tcc::mbar_wait_limit(tcc::smem_u32(&bar), 0, abort_flag, polls);
  ok = __all_sync(0xffffffffu, ok);
  tcc::tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) set_err(err, code);
    for (int i = 0; i < 20; ++i) __nanosleep(1000);
    __syncthreads();
  }
  tcc::tc_fence_after();
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(32u) : "memory");
}

thread_local std::string g_create_error;

struct Prof {
  struct Pair { cudaEvent_t a, b; int kind; double work; };
  std::vector<Pair> pairs;
  std::vector<cudaEvent_t> pool;
  bool on = false;
  dcd_prof_entry acc[DCD_PROF_COUNT] = {};
};

struct LayerW {
  bool full = false;
  void *input_norm = nullptr, *post_norm = nullptr, *w_gu = nullptr, *w_down = nullptr;
  void *w_qkv = nullptr, *w_o = nullptr, *qnorm = nullptr, *knorm = nullptr;
  void *w_gin = nullptr, *w_out = nullptr, *conv = nullptr, *gnorm = nullptr;
  float *A_log = nullptr, *dt_bias = nullptr;
  TcTensorMap tm_gu, tm_down, tm_qkv, tm_o, tm_gin, tm_out;
  // FP8 (e4m3) images of the six GEMM weights: values, per-output-row scales, TMA descriptors
  struct Fp8W { uint8_t* q = nullptr; float* scale = nullptr; TcTensorMap tm; };
  Fp8W f_gu, f_down, f_qkv, f_o, f_gin, f_out;
  // W4A16 group-128 images (precision 1): the only resident copy of the six GEMM weights
  // q: words in the nibble order [k0 k2 k4 k6 k1 k3 k5 k7]; scale: fp16 [N, K/128]; scale_t: the same transposed to [K/128][N] and
  // tm_q: TMA descriptor over q, both for the fused W4A16 GEMM (K % 128 == 0)
  struct W4 { uint32_t* q = nullptr; void* scale = nullptr; void* scale_t = nullptr; int N = 0, K = 0; bool fused = false; TcTensorMap tm_q;
              TcTensorMap tm_stage[2]; };  // this weight's [N, K] bf16 image in either of the two dequantisation stages
  W4 g_gu, g_down, g_qkv, g_o, g_gin, g_out;
  // NVFP4 images (precision 3): e2m1 codes, e4m3 scale per 16, f32 tensor scale and GEMM alpha on the device
  // codes, row-major scales, the same scales in the 128 x 4 tiled layout of the block-scaled MMA, tensor scale, 1/tensor scale
  struct NV4 { uint8_t* q = nullptr; uint8_t* sf = nullptr; uint8_t* sft = nullptr; float* wg = nullptr; float* alpha = nullptr; int N = 0, K = 0; TcTensorMap tm, tm256; };
  NV4 n_gu, n_down, n_qkv, n_o, n_gin, n_out;
};

}  // namespace

struct dcd_state {
  size_t state_len = 0, pos_end = 0, bytes = 0;
  void* block = nullptr;
  std::vector<void*> k, v, hist;
  std::vector<float*> gstate;
};

struct dcd_host_state {
  size_t state_len = 0, pos_end = 0, bytes = 0;
  void* block = nullptr;  // pinned host copy of the device block
};

struct dcd_engine {
  dcd_model_config c;
  dcd_options o;
  int device = 0, sm_count = 0, cc_major = 0, cc_minor = 0;
  char device_name[128] = {};
  bool bf = false;
  size_t esz = 4;
  cudaStream_t stream = nullptr;
  std::string err;
  int64_t launches = 0;

  // derived sizes
  int H = 0, I = 0, qcols = 0, kvcols = 0, qkv_n = 0, conv_dim = 0, vd = 0, gin_n = 0, gu_rows = 0, rhalf = 0;
  int Tm = 0;  // workspace rows

  // weights
  std::vector<void*> allocs;
  std::vector<LayerW> layers;
  void *embed = nullptr, *final_norm = nullptr;
  float* readout = nullptr;
  void *cos_t = nullptr, *sin_t = nullptr;
  size_t weight_bytes = 0, workspace_bytes = 0;
  bool weights_ready = false;

  // workspace
  void *x = nullptr, *h = nullptr, *x1 = nullptr, *mix = nullptr, *big = nullptr, *q = nullptr, *kown = nullptr;
  void *bufA = nullptr, *bufB = nullptr, *conv = nullptr, *act = nullptr;
  float *qf = nullptr, *kf = nullptr, *g = nullptr, *beta = nullptr, *hid = nullptr, *d_logits = nullptr, *tap_dev = nullptr;
  uint32_t* d_ids = nullptr;
  int32_t *d_lens = nullptr, *d_cu = nullptr, *d_last = nullptr, *d_tokq = nullptr, *d_tokpos = nullptr, *d_tile_cu = nullptr;
  void* attn_ws = nullptr;  // partial outputs of split attention launches
  bool attn_tc = false, gdn_chunked = false, gdn_tc = false, gdn_wy = false;
  TcTensorMap tm_gdn[3];  // q/k/conv views for the tcgen05 GDN kernel, rebuilt when the pass's token count changes
  int tm_gdn_tokens = -1;
  bool nv4 = false;                    // precision 3: NVFP4 weights and NVFP4-quantised activations (W4A4 semantics)
  bool nv4_native = false;             // ... on the block-scaled FP4 tensor-core GEMM (gemm_path 0) instead of dequantise + bf16 GEMM (2)
  uint8_t *xq = nullptr, *xsf = nullptr, *xsft = nullptr;  // activation codes, row-major scales, tiled scales
  uint8_t *aq4 = nullptr, *asft4 = nullptr;                // second set: the SwiGLU activation quantised by the gate/up GEMM's epilogue
  void* xstage = nullptr;              // bf16 [Tm, max K]: activations after the NVFP4 round trip
  unsigned int* amax_tmp = nullptr;
  bool w4 = false;                     // precision 1: int4 g128 weights, dequantised per GEMM into wstage
  void* wstage = nullptr;              // bf16 [max N*K] stage shared by all W4 GEMMs
  // precision 1, staged route, w4a16_prefetch = 1: a second stage and a second stream, so that the weight of the NEXT projection is
  // dequantised while the tensor cores run the current one. Off by default: under the power cap the GEMM slows by more than the
  // dequantisation it hides (8 layers: 54.96 ms per step with it, 53.56 without; identical results)
  void* wstage2 = nullptr;
  cudaStream_t stream2 = nullptr;
  // gdn_overlap = 0: the state's delta rule of a one-pass cold request runs here while the questions' conv and preparation run on `stream`
  cudaStream_t stream_gdn = nullptr;
  cudaEvent_t gdn_fork = nullptr, gdn_join = nullptr;
  cudaEvent_t w4_free[2] = {nullptr, nullptr}, w4_ready[2] = {nullptr, nullptr};  // stage b: last GEMM that read it launched / image complete
  const void* w4_holds[2] = {nullptr, nullptr};                                    // the W4 whose image stage b holds or is being given
  bool w4_pending[2] = {false, false};                                             // written on stream2, not yet awaited by the main stream
  int w4_cur = 0;                                                                  // stage read by the last staged GEMM
  bool fp8 = false, fp8_dirty = true;  // precision 2: e4m3 GEMMs in question passes of >= fp8_min_rows rows
  uint8_t* aq = nullptr;               // [Tm, max K] quantised activations
  float* a_scale = nullptr;            // [Tm] per-token scales
  int max_k = 0;
  int* d_err = nullptr;
  int max_batch = 0;

  // pinned staging
  uint32_t* h_ids = nullptr;
  int32_t* h_lens = nullptr;
  int32_t *h_posq = nullptr, *d_posq = nullptr;  // per-question start positions of a pass over several states
  float* h_logits = nullptr;
  int* h_err = nullptr;

  cudaEvent_t t0 = nullptr, t1 = nullptr;
  Prof prof;
  float* tap_sink = nullptr;
  size_t tap_cap = 0;
};

namespace {

int fail(dcd_engine* e, int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  if (e) e->err = buf; else g_create_error = buf;
  return code;
}
int cuda_fail(dcd_engine* e, cudaError_t ce, const char* what) {
  if (ce == cudaErrorMemoryAllocation) return fail(e, DCD_E_OOM, "%s: CUDA out of memory", what);
  return fail(e, DCD_E_CUDA, "%s: %s", what, cudaGetErrorString(ce));
}
#define CK(e, expr, what)                              \
  do {                                                 \
    cudaError_t _ce = (expr);                          \
    if (_ce != cudaSuccess) return cuda_fail(e, _ce, what); \
  } while (0)

const double IH8_STD = 53509.919921;  // sqrt(8 * (65536^2 - 1) / 12)
struct GenSpec { int dist; float p0, p1; bool round_bf; };
GenSpec spec_for(int kind, bool bf) {
  switch (kind) {
    case DCD_T_READOUT: return {0, 0.02f, 0.f, false};
    case DCD_T_A_LOG: return {1, 0.0f, 2.7725887f, false};
    case DCD_T_DT_BIAS: return {1, -6.9f, -2.3f, false};
    case DCD_T_CONV: return {1, -0.5f, 0.5f, bf};
    case DCD_T_GNORM: return {0, 0.02f, 1.0f, bf};
    default: return {0, 0.02f, 0.f, bf};
  }
}

// Where a logical tensor lives: base pointer of the (possibly fused) destination, its logical
// shape, the row mapping into the destination and whether it is stored as f32.
struct Loc { void* base; size_t rows, cols; int mode, row_offset, dst_stride; bool f32; LayerW::W4* w4 = nullptr; LayerW::NV4* nv = nullptr; };

bool locate(dcd_engine* e, int layer, int kind, Loc* out) {
  const dcd_model_config& c = e->c;
  const size_t H = e->H;
  auto L = [&](void* b, size_t r, size_t cc, int mode, int ro, int ds, bool f) { *out = Loc{b, r, cc, mode, ro, ds, f, nullptr}; return b != nullptr; };
  // GEMM weights of a W4 engine live as int4 images; the logical tensor is staged through wstage
  auto G = [&](void* b, LayerW::W4& img, LayerW::NV4& nimg, size_t r, size_t cc, int mode, int ro, int ds) {
    if (e->w4) { *out = Loc{e->wstage, r, cc, mode, ro, ds, false, &img, nullptr}; return true; }
    if (e->nv4) { *out = Loc{e->wstage, r, cc, mode, ro, ds, false, nullptr, &nimg}; return true; }
    return L(b, r, cc, mode, ro, ds, false);
  };
  if (layer < 0) {
    switch (kind) {
      case DCD_T_EMBED: return L(e->embed, c.vocab, H, 0, 0, (int)H, false);
      case DCD_T_FINAL_NORM: return L(e->final_norm, 1, H, 0, 0, (int)H, false);
      case DCD_T_READOUT: return L(e->readout, c.readout_rows, H, 0, 0, (int)H, true);
      default: return false;
    }
  }
  if (layer >= c.num_layers) return false;
  LayerW& w = e->layers[layer];
  const int hd = c.head_dim;
  switch (kind) {
    case DCD_T_INPUT_NORM: return L(w.input_norm, 1, H, 0, 0, (int)H, false);
    case DCD_T_POST_NORM: return L(w.post_norm, 1, H, 0, 0, (int)H, false);
    case DCD_T_GATE: return G(w.w_gu, w.g_gu, w.n_gu, e->I, H, 1, 0, (int)H);
    case DCD_T_UP: return G(w.w_gu, w.g_gu, w.n_gu, e->I, H, 2, 0, (int)H);
    case DCD_T_DOWN: return G(w.w_down, w.g_down, w.n_down, H, e->I, 0, 0, e->I);
  }
  if (w.full) {
    switch (kind) {
      case DCD_T_Q: return G(w.w_qkv, w.g_qkv, w.n_qkv, e->qcols, H, 0, 0, (int)H);
      case DCD_T_K: return G(w.w_qkv, w.g_qkv, w.n_qkv, e->kvcols, H, 0, e->qcols, (int)H);
      case DCD_T_V: return G(w.w_qkv, w.g_qkv, w.n_qkv, e->kvcols, H, 0, e->qcols + e->kvcols, (int)H);
      case DCD_T_O: return G(w.w_o, w.g_o, w.n_o, H, (size_t)c.heads * hd, 0, 0, c.heads * hd);
      case DCD_T_QNORM: return L(w.qnorm, 1, hd, 0, 0, hd, false);
      case DCD_T_KNORM: return L(w.knorm, 1, hd, 0, 0, hd, false);
      default: return false;
    }
  }
  switch (kind) {
    case DCD_T_IN_QKV: return G(w.w_gin, w.g_gin, w.n_gin, e->conv_dim, H, 0, 0, (int)H);
    case DCD_T_IN_Z: return G(w.w_gin, w.g_gin, w.n_gin, e->vd, H, 0, e->conv_dim, (int)H);
    case DCD_T_IN_B: return G(w.w_gin, w.g_gin, w.n_gin, c.gdn_v_heads, H, 0, e->conv_dim + e->vd, (int)H);
    case DCD_T_IN_A: return G(w.w_gin, w.g_gin, w.n_gin, c.gdn_v_heads, H, 0, e->conv_dim + e->vd + c.gdn_v_heads, (int)H);
    case DCD_T_OUT: return G(w.w_out, w.g_out, w.n_out, H, e->vd, 0, 0, e->vd);
    case DCD_T_CONV: return L(w.conv, e->conv_dim, 4, 0, 0, 4, false);
    case DCD_T_A_LOG: return L(w.A_log, 1, c.gdn_v_heads, 0, 0, c.gdn_v_heads, true);
    case DCD_T_DT_BIAS: return L(w.dt_bias, 1, c.gdn_v_heads, 0, 0, c.gdn_v_heads, true);
    case DCD_T_GNORM: return L(w.gnorm, 1, c.gdn_dv, 0, 0, c.gdn_dv, false);
    default: return false;
  }
}

int dev_alloc(dcd_engine* e, void** p, size_t bytes, bool zero, size_t* tally) {
  bytes = (bytes + 255) & ~(size_t)255;
  cudaError_t ce = cudaMalloc(p, bytes ? bytes : 256);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "cudaMalloc");
  e->allocs.push_back(*p);
  if (zero) CK(e, cudaMemsetAsync(*p, 0, bytes, e->stream), "memset");
  if (tally) *tally += bytes;
  return DCD_OK;
}
#define ALLOC(e, ptr, bytes, zero, tally)                                             \
  do {                                                                                \
    int _rc = dev_alloc(e, reinterpret_cast<void**>(&(ptr)), (bytes), (zero), (tally)); \
    if (_rc) return _rc;                                                              \
  } while (0)

uint16_t host_bf16(float x) {
  uint32_t u;
  memcpy(&u, &x, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
  u += 0x7fffu + ((u >> 16) & 1u);
  return (uint16_t)(u >> 16);
}

// ---- profiling -----------------------------------------------------------------
struct Scope {
  dcd_engine* e;
  int idx = -1;
  Scope(dcd_engine* e_, int kind, double work, int n_launch) : e(e_) {
    e->launches += n_launch;
    if (!e->prof.on) return;
    cudaEvent_t a, b;
    auto get = [&](cudaEvent_t* ev) {
      if (!e->prof.pool.empty()) { *ev = e->prof.pool.back(); e->prof.pool.pop_back(); }
      else cudaEventCreate(ev);
    };
    get(&a);
    get(&b);
    cudaEventRecord(a, e->stream);
    e->prof.pairs.push_back({a, b, kind, work});
    idx = (int)e->prof.pairs.size() - 1;
  }
  ~Scope() {
    if (idx >= 0) cudaEventRecord(e->prof.pairs[idx].b, e->stream);
  }
};

// ---- GEMM dispatch -------------------------------------------------------------
// C[M,N] = X[M,K] . W[N,K]^T. bf16 engine: tcgen05 path (bf16 operands, or e4m3 operands when
// `fw` is given: the activations are quantised per token first, Engine::fp8_gemm,
// native/src/engine.rs:4144-4296); plain FMA otherwise.
template <typename T>
int gemm(dcd_engine* e, const void* X, const TcTensorMap* tmA, const void* W, const TcTensorMap* tmB, const LayerW::Fp8W* fw,
         const LayerW::W4* g4, const LayerW::NV4* n4, void* C, int M, int N, int K, int ldc, int epi, bool x_quantised = false,
         const void* resid = nullptr, int x_set = 0, bool act_out = false) {
  // resid: C = bf16(resid + bf16(X W^T)) in the epilogue (tensor-core paths). x_set: which of the two NVFP4 activation buffer sets
  // holds a pre-quantised X (0: xq / xsft, 1: aq4 / asft4). act_out (native NVFP4, gate/up projection): the epilogue applies SwiGLU
  // and writes the NVFP4 image of the activation into set 1 instead of C.
  int w4_stage_used = -1;
  if (resid && !(e->nv4_native && n4->sft && nvfp4_tc_shape_ok(M, N, K)) && (e->nv4 || !(e->bf && e->o.gemm_path == 0 && tc_shape_ok(M, N, K))))
    return fail(e, DCD_E_INVALID, "internal: fused residual on a GEMM path without that epilogue");
  if (e->nv4_native && epi == 0 && n4->sft && nvfp4_tc_shape_ok(M, N, K)) {
    // NVFP4 W4A4 (Engine::nvfp4_gemm, native/src/engine.rs:3962-4131) on the block-scaled FP4 MMA: activations are
    // quantised per 16 elements (tensor scale 1), both scale sets are read in the 128 x 4 tiled layout, alpha =
    // 1/(weight_global*input_global) in the epilogue.
    if (!x_quantised) {  // else the producer of X already left its codes and tiled scales in xq / xsft
      Scope sc(e, DCD_PROF_ELEMENTWISE, 2.5625 * M * (double)K, 1);
      CK(e, launch_nvfp4_act_quant_tiled((const bf16*)X, (size_t)K, e->xq, e->xsft, M, K, e->stream), "nvfp4 activation quantisation");
    }
    const uint8_t* xq = x_set ? e->aq4 : e->xq;
    const uint8_t* xsf = x_set ? e->asft4 : e->xsft;
    TcTensorMap ta;
    if (tc_make_tmap_fp8_a(&ta, xq, M, K / 2)) return fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an nvfp4 activation operand");
    Scope sc(e, DCD_PROF_GEMM, 2.0 * M * (double)N * K, 1);
    const int bn = N >= 256 ? 256 : 128;
    CK(e, nvfp4_gemm_launch(&ta, bn == 256 ? &n4->tm256 : &n4->tm, xsf, n4->sft, C, M, N, K, ldc, n4->alpha, e->sm_count, e->d_err, e->stream,
                            bn + (e->o.nvfp4_scale_copy == 1 ? 0 : 1000), resid, act_out ? e->aq4 : nullptr, act_out ? e->asft4 : nullptr),
       "tcgen05 nvfp4 gemm");
    return DCD_OK;
  }
  if (act_out) return fail(e, DCD_E_INVALID, "internal: fused SwiGLU quantisation on a GEMM that does not take the block-scaled path");
  if (x_quantised) return fail(e, DCD_E_INVALID, "internal: pre-quantised operand for a GEMM that does not take the block-scaled path");
  if (e->nv4) {
    // The same product by the long route (gemm_path 2, or a shape the native kernel does not take): both operands go through the
    // e2m1/e4m3 round trip; their dequantised values are exact in bf16, so the bf16 tensor-core GEMM
    // gives the block-scaled product; alpha = 1/(weight_global*input_global) in the epilogue.
    {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 0.5625 * N * (double)K + 2.0 * N * (double)K + 4.0 * M * (double)K, 2);
      CK(e, launch_nvfp4_dequant_rows(n4->q, n4->sf, nullptr, (bf16*)e->wstage, N, K, e->stream), "nvfp4 weight dequantisation");
      CK(e, launch_nvfp4_fakequant_rows((const bf16*)X, (size_t)K, 1.0f, (bf16*)e->xstage, M, K, e->stream), "nvfp4 activation quantisation");
    }
    TcTensorMap ta;
    if (tc_make_tmap_a(&ta, e->xstage, M, K)) return fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an nvfp4 activation operand");
    Scope sc(e, DCD_PROF_GEMM, 2.0 * M * (double)N * K, 1);
    CK(e, tc_gemm_launch(&ta, tmB, C, M, N, K, ldc, epi, e->sm_count, e->d_err, e->stream, n4->alpha), "tcgen05 gemm (nvfp4 operands)");
    return DCD_OK;
  }
  if (e->w4 && g4->fused && e->o.gemm_path == 0 && e->o.w4a16_gemm != 1 && w4a16_tc_shape_ok(M, N, K) &&
      (e->o.w4a16_gemm == 2 || w4a16_tc_prefer(M, N, e->sm_count))) {
    // W4A16 on the fused kernel: nibbles become bf16 inside the GEMM's producer warps, no bf16 copy of W
    // (the role of the reference's Marlin kernel, native/kernels/marlin.cu:398-408)
    Scope sc(e, DCD_PROF_GEMM, 2.0 * M * (double)N * K, 1);
    CK(e, w4a16_gemm_launch(tmA, &g4->tm_q, g4->scale_t, C, M, N, K, ldc, epi, e->sm_count, e->d_err, e->stream, resid), "tcgen05 w4a16 gemm");
    return DCD_OK;
  }
  if (e->w4) {
    // ... or, where 256-row tiles would leave the GPU half empty (or the shape is not the kernel's): int4 -> bf16 into the shared
    // stage, then the bf16 tensor-core GEMM reads the stage (the reference's dequant_w4a16_bf16 + BF16 GEMM route,
    // native/src/engine.rs:4516-4558)
    int b = -1;
    for (int i = 0; i < 2; ++i)
      if (e->wstage2 && e->w4_pending[i] && e->w4_holds[i] == g4) b = i;
    if (b >= 0) {  // dequantised ahead on the second stream (w4_prefetch)
      CK(e, cudaStreamWaitEvent(e->stream, e->w4_ready[b], 0), "w4 stage ready");
      e->w4_pending[b] = false;
    } else {
      b = e->wstage2 ? e->w4_cur ^ 1 : 0;
      if (e->w4_pending[b]) {  // a prefetch nobody asked for after all: let it finish before the stage is rewritten
        CK(e, cudaStreamWaitEvent(e->stream, e->w4_ready[b], 0), "w4 stage ready");
        e->w4_pending[b] = false;
      }
      Scope sc(e, DCD_PROF_ELEMENTWISE, 2.5 * N * (double)K, 1);
      CK(e, launch_dequant_w4_g128(g4->q, g4->scale, (bf16*)(b ? e->wstage2 : e->wstage), N, K, e->stream, true), "w4 dequantisation");
      e->w4_holds[b] = g4;
    }
    W = b ? e->wstage2 : e->wstage;
    tmB = &g4->tm_stage[b];
    e->w4_cur = b;
    w4_stage_used = b;
  }
  if (fw && e->bf && e->o.gemm_path == 0 && tc_fp8_shape_ok(M, N, K)) {
    {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 3.0 * M * (double)K, 1);
      CK(e, launch_quant_fp8_rows<bf16>((const bf16*)X, (size_t)K, e->aq, e->a_scale, M, K, 1.0f, e->stream), "fp8 activation quantisation");
    }
    TcTensorMap ta;
    if (tc_make_tmap_fp8_a(&ta, e->aq, M, K)) return fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an fp8 activation operand");
    Scope sc(e, DCD_PROF_GEMM, 2.0 * M * (double)N * K, 1);
    CK(e, tc_gemm_fp8_launch(&ta, &fw->tm, C, M, N, K, ldc, epi, e->a_scale, fw->scale, e->sm_count, e->d_err, e->stream, resid), "tcgen05 fp8 gemm");
    return DCD_OK;
  }
  Scope sc(e, DCD_PROF_GEMM, 2.0 * M * (double)N * K, 1);
  if (e->bf && e->o.gemm_path == 0 && tc_shape_ok(M, N, K)) {
    CK(e, tc_gemm_launch(tmA, tmB, C, M, N, K, ldc, epi, e->sm_count, e->d_err, e->stream, nullptr, resid), "tcgen05 gemm");
    if (w4_stage_used >= 0 && e->wstage2) CK(e, cudaEventRecord(e->w4_free[w4_stage_used], e->stream), "w4 stage free");
    return DCD_OK;
  }
  if (epi != 0) return fail(e, DCD_E_INVALID, "internal: fused epilogue without tensor-core path");
  CK(e, launch_gemm_fma<T>((const T*)X, (const T*)W, (T*)C, M, N, K, ldc, e->stream), "fma gemm");
  return DCD_OK;
}

// Staged W4A16 route: would gemm() dequantise this weight into a stage for a pass of M rows?
bool w4_takes_stage(const dcd_engine* e, const LayerW::W4* g4, int M) {
  if (!e->w4 || !g4 || !g4->q) return false;
  const bool fused = g4->fused && e->o.gemm_path == 0 && e->o.w4a16_gemm != 1 && w4a16_tc_shape_ok(M, g4->N, g4->K) &&
                     (e->o.w4a16_gemm == 2 || w4a16_tc_prefer(M, g4->N, e->sm_count));
  return !fused;
}
// Start dequantising the weight of the NEXT projection on the second stream into the stage the GEMM launched last does not read.
// That stage was last read by the GEMM before it, whose completion event the second stream awaits first.
int w4_prefetch(dcd_engine* e, const LayerW::W4* next, int M) {
  if (!e->wstage2 || !w4_takes_stage(e, next, M) || !(e->bf && e->o.gemm_path == 0 && tc_shape_ok(M, next->N, next->K))) return DCD_OK;
  const int b = e->w4_cur ^ 1;
  if (e->w4_pending[b]) return DCD_OK;  // still holds an image nobody consumed
  CK(e, cudaStreamWaitEvent(e->stream2, e->w4_free[b], 0), "w4 stage free");
  CK(e, launch_dequant_w4_g128(next->q, next->scale, (bf16*)(b ? e->wstage2 : e->wstage), next->N, next->K, e->stream2, true), "w4 dequantisation ahead");
  CK(e, cudaEventRecord(e->w4_ready[b], e->stream2), "w4 stage ready");
  e->w4_holds[b] = next;
  e->w4_pending[b] = true;
  e->launches += 1;
  return DCD_OK;
}

// A run of consecutive questions of the packed batch that fork the same state.
struct Group {
  const dcd_state* st;  // the state these sequences fork; null: none (a state sequence that attends to itself only)
  int q0, nq;      // questions [q0, q0 + nq)
  int tok0, ntok;  // their packed tokens [tok0, tok0 + ntok)
  int max_len;
  // Cold request in ONE pass (mode 1): a group of one sequence, the state itself, whose K/V, conv tail and final recurrent state
  // are written into `cap` layer by layer; a later group of the same pass names `cap` as its `st` and reads, in each layer, what
  // the state's kernels of that layer have just written (same stream). The token-parallel kernels see one batch of
  // state + question rows: the weights stream once per layer for the whole request.
  dcd_state* cap = nullptr;
};

struct Pass {
  int mode;  // 0 capture, 1 state-once question pass, 2 per-row reference
  int T, B, max_len;
  const dcd_state* cache = nullptr;
  dcd_state* cap = nullptr;
  int split = 0;
  // mode 1 over several states: the token-parallel kernels (GEMMs, norms, RoPE, GDN preparation) run once over the whole
  // batch; the kernels that read a state (attention, conv tail, recurrent seed) run once per group on its slice
  const Group* groups = nullptr;
  int n_groups = 0;
  const int32_t* d_posq = nullptr;  // per-question start position (device), with groups
};

template <typename T>
int run_layers(dcd_engine* e, const Pass& p) {
  const dcd_model_config& c = e->c;
  const int T_ = p.T, H = e->H, heads = c.heads, kv = c.kv_heads, hd = c.head_dim;
  const int nk = c.gdn_k_heads, nv = c.gdn_v_heads, dk = c.gdn_dk, dv = c.gdn_dv;
  cudaStream_t s = e->stream;
  const bool tc = e->bf && e->o.gemm_path == 0;
  const bool fused_swiglu = tc && !e->nv4_native;  // the block-scaled FP4 kernel has the plain epilogue only
  // ... so SwiGLU runs as its own kernel, which then writes the down projection's operand as NVFP4 directly
  const bool act_fused_quant = e->nv4_native && sizeof(T) == 2 && (e->I % 256) == 0 && nvfp4_tc_shape_ok(T_, H, e->I);
  // ... and the norms that feed the q/k/v, GDN input and gate/up projections write NVFP4 instead of bf16 h
  const bool h_fused_quant = e->nv4_native && sizeof(T) == 2 && (H % 256) == 0 && H <= 8192;
  // bf16 / fp8 / w4a16 tensor-core GEMMs add the residual in their epilogue: the projection that closes a block writes the new
  // residual stream itself and the norm that follows reads one tensor instead of two
  const bool fuse4 = e->nv4_native && e->o.nvfp4_fusion != 1 && sizeof(T) == 2;  // the NVFP4 epilogue / producer fusions below
  // ... the block-scaled kernel has the residual epilogue too, where all three closing projections take it
  const bool resid4 = fuse4 && nvfp4_tc_shape_ok(T_, H, heads * hd) && nvfp4_tc_shape_ok(T_, H, e->vd) && nvfp4_tc_shape_ok(T_, H, e->I);
  const bool fused_resid = (tc && !e->nv4 && tc_shape_ok(T_, H, H)) || resid4;
  // ... its gate/up epilogue can apply SwiGLU and write the down projection's NVFP4 operand itself (set 1)
  const bool act_epi4 = fuse4 && act_fused_quant && h_fused_quant && (e->I % 128) == 0 && e->gu_rows == 2 * e->I && nvfp4_tc_shape_ok(T_, e->gu_rows, H);
  // ... and the gated norm writes the out projection's NVFP4 operand
  const bool gnorm4 = fuse4 && dv == 128 && (e->vd % 256) == 0 && nvfp4_tc_shape_ok(T_, H, e->vd);
  // FP8 only in question passes with enough rows; capture and the per-row reference stay bf16
  // (native/src/engine.rs:4321-4326, fp8_min_rows :246-257)
  const bool q8 = e->fp8 && tc && p.mode == 1 && p.T >= e->o.fp8_min_rows;
  TcTensorMap tm_h, tm_A, tm_B, tm_act;
  if (tc) {
    if (tc_make_tmap_a(&tm_h, e->h, T_, H) || tc_make_tmap_a(&tm_A, e->bufA, T_, heads * hd) ||
        tc_make_tmap_a(&tm_B, e->bufB, T_, e->vd) || tc_make_tmap_a(&tm_act, e->act, T_, e->I))
      return fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an activation operand");
  }
  const size_t xbytes = (size_t)T_ * H * e->esz;
  const Group whole{p.cache, 0, p.B, 0, T_, p.max_len};
  const Group* groups = p.n_groups > 0 ? p.groups : &whole;
  const int n_groups = p.n_groups > 0 ? p.n_groups : 1;
  for (int li = 0; li < c.num_layers; ++li) {
    LayerW& w = e->layers[li];
    if (li == 0) {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 2.0 * xbytes, 1);
      if (h_fused_quant) CK(e, launch_rmsnorm_nvfp4((const bf16*)e->x, (const bf16*)w.input_norm, e->xq, e->xsft, T_, H, c.rms_eps, s), "rmsnorm + nvfp4");
      else CK(e, launch_rmsnorm<T>((const T*)e->x, (const T*)w.input_norm, (T*)e->h, T_, H, c.rms_eps, true, s), "rmsnorm");
    }
    if (w.full) {
      int rc = gemm<T>(e, e->h, &tm_h, w.w_qkv, &w.tm_qkv, q8 ? &w.f_qkv : nullptr, &w.g_qkv, &w.n_qkv, e->big, T_, e->qkv_n, H, e->qkv_n, 0, h_fused_quant);
      if (!rc) rc = w4_prefetch(e, &w.g_o, T_);
      if (rc) return rc;
      T* big = (T*)e->big;
      T* kdst = p.mode == 0 ? (T*)p.cap->k[li] : (T*)e->kown;
      {
        Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * (heads + kv) * hd * e->esz * 2.0, 1);
        CK(e, launch_qk_norm_rope<T>(big, e->qkv_n, big + e->qcols, e->qkv_n, (const T*)w.qnorm, (const T*)w.knorm, (const T*)e->cos_t,
                                     (const T*)e->sin_t, e->d_tokpos, 0, e->o.max_positions, (T*)e->q, kdst, kv * hd, T_, heads, kv, hd,
                                     c.rotary_dim, c.rms_eps, e->d_err, s), "qk_norm_rope");
      }
      const T* vsrc = big + e->qcols + e->kvcols;
      if (p.mode == 0) {
        Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * kv * hd * e->esz * 2.0, 1);
        CK(e, launch_copy_rows<T>(vsrc, e->qkv_n, (T*)p.cap->v[li], kv * hd, T_, kv * hd, s), "copy V");
      }
      for (int gi = 0; gi < n_groups && p.mode == 1; ++gi) {
        const Group& g = groups[gi];
        if (!g.cap) continue;
        Scope sc(e, DCD_PROF_ELEMENTWISE, (double)g.ntok * kv * hd * e->esz * 4.0, 2);
        CK(e, launch_copy_rows<T>(kdst + (size_t)g.tok0 * kv * hd, kv * hd, (T*)g.cap->k[li], kv * hd, g.ntok, kv * hd, s), "copy K");
        CK(e, launch_copy_rows<T>(vsrc + (size_t)g.tok0 * e->qkv_n, e->qkv_n, (T*)g.cap->v[li], kv * hd, g.ntok, kv * hd, s), "copy V");
      }
      // Capture keeps nothing of the last layer beyond its cache entries: the reference computes the
      // rest of that layer and discards it (native/src/engine.rs:4616-4763 builds no final norm or readout).
      if (p.mode == 0 && li + 1 == c.num_layers) break;
      for (int gi = 0; gi < n_groups; ++gi) {
        const Group& g = groups[gi];
        const int n_state = p.mode == 1 && g.st ? (int)g.st->state_len : 0;
        double keys = 0;  // sum over rows of visible keys
        if (p.mode == 1) keys = (double)g.ntok * n_state + (double)g.ntok * g.max_len;  // upper bound on own keys
        else if (p.mode == 0) keys = (double)T_ * T_;
        else keys = (double)p.split * p.split + (double)(T_ - p.split) * T_;
        const T* ks = p.mode == 1 && g.st ? (const T*)g.st->k[li] : nullptr;
        const T* vs = p.mode == 1 && g.st ? (const T*)g.st->v[li] : nullptr;
        Scope sc(e, DCD_PROF_ATTN, 4.0 * heads * hd * keys, 1);
        if (e->attn_tc && p.mode != 2) {
          const int tt = attn_tc_tokens_per_tile(heads, kv);
          if (n_groups > 1) {  // the tile table is per launch: rebuilt for this group's sequences (same stream, so in order)
            e->launches += 1;
            CK(e, attn_tc_build_tiles(e->d_cu + g.q0, g.nq, tt, e->d_tile_cu, s), "attention tiles");
          }
          AttnTcMaps maps;
          if (attn_tc_make_maps(&maps, e->q, kdst, kv * hd, vsrc, e->qkv_n, ks, vs, n_state, T_, heads, kv, hd))
            return fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an attention operand");
          const int max_tiles = (g.ntok + tt - 1) / tt + g.nq;
          const int n_split = e->attn_ws ? attn_tc_pick_split(max_tiles, kv, n_state, e->sm_count) : 1;
          if (n_split > 1) e->launches += 1;  // the merge kernel
          CK(e, attn_tc_launch(&maps, e->d_cu + g.q0, e->d_tile_cu, g.nq, n_state, T_, max_tiles, heads, kv, hd, big, e->qkv_n, e->bufA, e->d_err, s,
                               n_split, e->attn_ws), "tcgen05 attention");
        } else {
          const size_t t0 = (size_t)g.tok0;
          CK(e, launch_attn_fma<T>((const T*)e->q + t0 * heads * hd, kdst + t0 * kv * hd, kv * hd, vsrc + t0 * e->qkv_n, e->qkv_n, ks, vs, n_state,
                                   big + t0 * e->qkv_n, e->qkv_n, (T*)e->bufA + t0 * heads * hd, e->d_cu, e->d_tokq + t0, g.ntok, heads, kv, hd,
                                   p.mode == 2 ? p.split : 0, s, g.tok0), "attention");
        }
      }
      rc = gemm<T>(e, e->bufA, &tm_A, w.w_o, &w.tm_o, q8 ? &w.f_o : nullptr, &w.g_o, &w.n_o, fused_resid ? e->x1 : e->mix, T_, H, heads * hd, H, 0, false,
                   fused_resid ? e->x : nullptr);
      if (!rc) rc = w4_prefetch(e, &w.g_gu, T_);
      if (rc) return rc;
    } else {
      int rc = gemm<T>(e, e->h, &tm_h, w.w_gin, &w.tm_gin, q8 ? &w.f_gin : nullptr, &w.g_gin, &w.n_gin, e->big, T_, e->gin_n, H, e->gin_n, 0, h_fused_quant);
      if (!rc) rc = w4_prefetch(e, &w.g_out, T_);
      if (rc) return rc;
      T* big = (T*)e->big;
      if (p.mode == 0) {
        // last three pre-convolution rows, left-zero-padded (native/src/engine.rs:3348-3361)
        CK(e, cudaMemsetAsync(p.cap->hist[li], 0, (size_t)3 * e->conv_dim * e->esz, s), "memset hist");
        const int keep = T_ < 3 ? T_ : 3;
        Scope sc(e, DCD_PROF_ELEMENTWISE, 0, 1);
        CK(e, launch_copy_rows<T>(big + (size_t)(T_ - keep) * e->gin_n, e->gin_n, (T*)p.cap->hist[li] + (size_t)(3 - keep) * e->conv_dim,
                                  e->conv_dim, keep, e->conv_dim, s), "copy conv tail");
      }
      for (int gi = 0; gi < n_groups && p.mode == 1; ++gi) {
        const Group& g = groups[gi];
        if (!g.cap) continue;
        CK(e, cudaMemsetAsync(g.cap->hist[li], 0, (size_t)3 * e->conv_dim * e->esz, s), "memset hist");
        const int keep = g.ntok < 3 ? g.ntok : 3;
        Scope sc(e, DCD_PROF_ELEMENTWISE, 0, 1);
        CK(e, launch_copy_rows<T>(big + (size_t)(g.tok0 + g.ntok - keep) * e->gin_n, e->gin_n, (T*)g.cap->hist[li] + (size_t)(3 - keep) * e->conv_dim,
                                  e->conv_dim, keep, e->conv_dim, s), "copy conv tail");
      }
      // A cold request in one pass = the state (group 0, rows [0, n)) and its questions (group 1). The state's delta rule occupies one
      // CTA per value head (48 of the SMs) for 32 chunks in a row and the questions' needs its final state, so with gdn_overlap = 0
      // it runs on a stream of its own while the conv and the preparation of the questions' rows run here; same kernels, same bits.
      const bool overlap = e->stream_gdn && e->gdn_wy && p.mode == 1 && n_groups == 2 && groups[0].cap && groups[0].tok0 == 0 &&
                           groups[1].tok0 == groups[0].ntok && groups[1].st == groups[0].cap;
      auto conv_group = [&](const Group& g) {
        const size_t t0 = (size_t)g.tok0;
        return launch_conv1d_silu<T>(big + t0 * e->gin_n, e->gin_n, p.mode == 1 && g.st ? (const T*)g.st->hist[li] : nullptr, (const T*)w.conv,
                                     (T*)e->conv + t0 * e->conv_dim, e->d_cu, e->d_tokq + t0, g.ntok, e->conv_dim, s, g.tok0);
      };
      auto prepare_rows = [&](size_t t0, int rows) {
        const T* bsrc = big + t0 * e->gin_n + e->conv_dim + e->vd;
        return launch_gdn_prepare<T>((const T*)e->conv + t0 * e->conv_dim, e->conv_dim, bsrc, bsrc + nv, e->gin_n, w.A_log, w.dt_bias,
                                     e->qf + t0 * nk * dk, e->kf + t0 * nk * dk, e->g + t0 * nv, e->beta + t0 * nv, rows, nk, nv, dk, s);
      };
      auto gdn_group = [&](const Group& g, float* fin0, cudaStream_t gs) -> cudaError_t {  // sequences index the packed buffers through cu, so a group is a slice of cu
        const float* seed = p.mode == 1 && g.st ? g.st->gstate[li] : nullptr;
        float* fin = g.cap ? g.cap->gstate[li] : fin0;
        const int32_t* cu = e->d_cu + g.q0;
        if (e->gdn_wy) return launch_gdn_wy<T>(e->tm_gdn, (const T*)e->conv, e->conv_dim, e->g, e->beta, seed, fin, (T*)e->bufA, cu, g.nq, nk, nv, e->d_err, gs);
        if (e->gdn_tc) return launch_gdn_tc<T>(e->tm_gdn, (const T*)e->conv, e->conv_dim, e->g, e->beta, seed, fin, (T*)e->bufA, cu, g.nq, nk, nv, e->d_err, gs);
        if (e->gdn_chunked)
          return launch_gdn_chunked<T>(e->qf, e->kf, (const T*)e->conv, e->conv_dim, e->g, e->beta, seed, fin, (T*)e->bufA, cu, g.nq, nk, nv, dk, dv, g.nq < 2, gs);
        return launch_gdn_recurrent<T>(e->qf, e->kf, (const T*)e->conv, e->conv_dim, e->g, e->beta, seed, fin, (T*)e->bufA, cu, g.nq, nk, nv, dk, dv, g.nq < 8, gs);
      };
      if (e->gdn_tc && e->tm_gdn_tokens != T_) {
        if (gdn_tc_make_maps(e->tm_gdn, e->qf, e->kf, e->conv, e->conv_dim, e->conv_dim, (int)e->esz, T_, nk) != 0) return fail(e, DCD_E_CUDA, "GDN q/k tensor maps");
        e->tm_gdn_tokens = T_;
      }
      if (overlap) {
        {
          Scope sc(e, DCD_PROF_ELEMENTWISE, (double)groups[0].ntok * (e->conv_dim * e->esz * 2.0 + nk * dk * (2.0 * e->esz + 8.0)), 1);
          e->launches += 1;
          CK(e, conv_group(groups[0]), "conv1d");
          CK(e, prepare_rows(0, groups[0].ntok), "gdn_prepare");
        }
        CK(e, cudaEventRecord(e->gdn_fork, s), "GDN fork");
        CK(e, cudaStreamWaitEvent(e->stream_gdn, e->gdn_fork, 0), "GDN fork");
        CK(e, gdn_group(groups[0], nullptr, e->stream_gdn), "gdn_wy");
        CK(e, cudaEventRecord(e->gdn_join, e->stream_gdn), "GDN join");
        {
          Scope sc(e, DCD_PROF_ELEMENTWISE, (double)groups[1].ntok * (e->conv_dim * e->esz * 2.0 + nk * dk * (2.0 * e->esz + 8.0)), 1);
          e->launches += 1;
          CK(e, conv_group(groups[1]), "conv1d");
          CK(e, prepare_rows((size_t)groups[1].tok0, groups[1].ntok), "gdn_prepare");
        }
        {
          Scope sc(e, DCD_PROF_GDN, 6.0 * dk * dv * (double)T_ * nv, 1);
          e->launches += 1;
          CK(e, cudaStreamWaitEvent(s, e->gdn_join, 0), "GDN join");
          CK(e, gdn_group(groups[1], nullptr, s), "gdn_wy");
        }
      } else {
        {
          Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * e->conv_dim * e->esz * 2.0, 1);
          e->launches += n_groups - 1;
          for (int gi = 0; gi < n_groups; ++gi) CK(e, conv_group(groups[gi]), "conv1d");
        }
        {
          Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * nk * dk * (2.0 * e->esz + 8.0), 1);
          CK(e, prepare_rows(0, T_), "gdn_prepare");
        }
        {
          Scope sc(e, DCD_PROF_GDN, 6.0 * dk * dv * (double)T_ * nv, 1);
          float* fin0 = p.mode == 0 ? p.cap->gstate[li] : nullptr;
          e->launches += n_groups - 1;
          for (int gi = 0; gi < n_groups; ++gi) CK(e, gdn_group(groups[gi], fin0, s), "gdn");
        }
      }
      if (p.mode == 0 && li + 1 == c.num_layers) break;  // last capture layer: the state and conv tail are stored
      {
        Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * e->vd * e->esz * (gnorm4 ? 2.3 : 3.0), 1);
        if (gnorm4)
          CK(e, launch_rmsnorm_gated_nvfp4((const bf16*)e->bufA, (const bf16*)(big + e->conv_dim), e->gin_n, (const bf16*)w.gnorm, e->xq, e->xsft, T_, nv,
                                           c.rms_eps, s), "rmsnorm_gated + nvfp4");
        else
          CK(e, launch_rmsnorm_gated<T>((const T*)e->bufA, big + e->conv_dim, e->gin_n, (const T*)w.gnorm, (T*)e->bufB, T_, nv, dv,
                                        c.rms_eps, s), "rmsnorm_gated");
      }
      rc = gemm<T>(e, e->bufB, &tm_B, w.w_out, &w.tm_out, q8 ? &w.f_out : nullptr, &w.g_out, &w.n_out, fused_resid ? e->x1 : e->mix, T_, H, e->vd, H, 0, gnorm4,
                   fused_resid ? e->x : nullptr);
      if (!rc) rc = w4_prefetch(e, &w.g_gu, T_);
      if (rc) return rc;
    }
    {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 4.0 * xbytes, 1);
      if (fused_resid && h_fused_quant)
        CK(e, launch_rmsnorm_nvfp4((const bf16*)e->x1, (const bf16*)w.post_norm, e->xq, e->xsft, T_, H, c.rms_eps, s), "rmsnorm + nvfp4");
      else if (fused_resid)
        CK(e, launch_rmsnorm<T>((const T*)e->x1, (const T*)w.post_norm, (T*)e->h, T_, H, c.rms_eps, true, s), "rmsnorm");
      else if (h_fused_quant)
        CK(e, launch_add_rmsnorm_nvfp4((const bf16*)e->x, (const bf16*)e->mix, (const bf16*)w.post_norm, (bf16*)e->x1, e->xq, e->xsft, T_, H, c.rms_eps, s),
           "add_rmsnorm + nvfp4");
      else
        CK(e, launch_add_rmsnorm<T>((const T*)e->x, (const T*)e->mix, (const T*)w.post_norm, (T*)e->x1, (T*)e->h, T_, H, c.rms_eps, s),
           "add_rmsnorm");
    }
    if (fused_swiglu) {
      int rc = gemm<T>(e, e->h, &tm_h, w.w_gu, &w.tm_gu, q8 ? &w.f_gu : nullptr, &w.g_gu, &w.n_gu, e->act, T_, e->gu_rows, H, e->I, 1);
      if (!rc) rc = w4_prefetch(e, &w.g_down, T_);
      if (rc) return rc;
    } else if (act_epi4) {
      // gate/up projection whose epilogue applies SwiGLU and leaves the activation as NVFP4 in set 1 (ldc = the activation width)
      int rc = gemm<T>(e, e->h, &tm_h, w.w_gu, &w.tm_gu, nullptr, &w.g_gu, &w.n_gu, nullptr, T_, e->gu_rows, H, e->I, 0, true, nullptr, 0, true);
      if (rc) return rc;
    } else {
      int rc = gemm<T>(e, e->h, &tm_h, w.w_gu, &w.tm_gu, nullptr, &w.g_gu, &w.n_gu, e->big, T_, e->gu_rows, H, e->gu_rows, 0, h_fused_quant);
      if (rc) return rc;
      Scope sc(e, DCD_PROF_ELEMENTWISE, (double)T_ * e->I * e->esz * 3.0, 1);
      if (act_fused_quant) CK(e, launch_nvfp4_swiglu_quant_tiled((const bf16*)e->big, e->gu_rows, e->xq, e->xsft, T_, e->I, s), "silu_mul + nvfp4 quantisation");
      else CK(e, launch_silu_mul_interleaved<T>((const T*)e->big, e->gu_rows, (T*)e->act, T_, e->I, s), "silu_mul");
    }
    int rc = gemm<T>(e, e->act, &tm_act, w.w_down, &w.tm_down, q8 ? &w.f_down : nullptr, &w.g_down, &w.n_down, fused_resid ? e->x : e->mix, T_, H, e->I, H, 0, act_fused_quant,
                     fused_resid ? e->x1 : nullptr, act_epi4 ? 1 : 0);
    if (!rc && li + 1 < c.num_layers)
      rc = w4_prefetch(e, e->layers[li + 1].full ? &e->layers[li + 1].g_qkv : &e->layers[li + 1].g_gin, T_);
    if (rc) return rc;
    if (li + 1 < c.num_layers) {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 4.0 * xbytes, 1);
      if (fused_resid && h_fused_quant)
        CK(e, launch_rmsnorm_nvfp4((const bf16*)e->x, (const bf16*)e->layers[li + 1].input_norm, e->xq, e->xsft, T_, H, c.rms_eps, s), "rmsnorm + nvfp4");
      else if (fused_resid)
        CK(e, launch_rmsnorm<T>((const T*)e->x, (const T*)e->layers[li + 1].input_norm, (T*)e->h, T_, H, c.rms_eps, true, s), "rmsnorm");
      else if (h_fused_quant)
        CK(e, launch_add_rmsnorm_nvfp4((const bf16*)e->x1, (const bf16*)e->mix, (const bf16*)e->layers[li + 1].input_norm, (bf16*)e->x, e->xq, e->xsft,
                                       T_, H, c.rms_eps, s), "add_rmsnorm + nvfp4");
      else
        CK(e, launch_add_rmsnorm<T>((const T*)e->x1, (const T*)e->mix, (const T*)e->layers[li + 1].input_norm, (T*)e->x, (T*)e->h, T_, H,
                                    c.rms_eps, s), "add_rmsnorm");
    } else if (!fused_resid) {
      Scope sc(e, DCD_PROF_ELEMENTWISE, 3.0 * xbytes, 1);
      CK(e, launch_add<T>((const T*)e->x1, (const T*)e->mix, (T*)e->x, (size_t)T_ * H, s), "add");
    }
    if (e->tap_sink && (size_t)(li + 1) * T_ * H <= e->tap_cap) {
      CK(e, launch_to_f32<T>((const T*)e->x, e->tap_dev, (size_t)T_ * H, s), "tap");
      CK(e, cudaMemcpyAsync(e->tap_sink + (size_t)li * T_ * H, e->tap_dev, (size_t)T_ * H * 4, cudaMemcpyDeviceToHost, s), "tap copy");
      CK(e, cudaStreamSynchronize(s), "tap sync");
    }
  }
  return DCD_OK;
}

// Pack + embed + layers (+ final norm of last rows + readout unless capturing).
template <typename T>
int run_pass(dcd_engine* e, const Pass& p, const uint32_t* d_ids, const int32_t* d_lens, int pos_start, float* d_out) {
  cudaStream_t s = e->stream;
  {
    Scope sc(e, DCD_PROF_ELEMENTWISE, 12.0 * p.T, 2);
    CK(e, launch_pack(d_lens, p.B, p.T, pos_start, e->d_cu, e->d_last, e->d_tokq, e->d_tokpos, e->d_err, s, p.d_posq), "pack");
    if (e->attn_tc && p.mode != 2 && p.n_groups <= 1) {
      e->launches += 1;
      CK(e, attn_tc_build_tiles(e->d_cu, p.B, attn_tc_tokens_per_tile(e->c.heads, e->c.kv_heads), e->d_tile_cu, s), "attention tiles");
    }
  }
  {
    Scope sc(e, DCD_PROF_ELEMENTWISE, 2.0 * p.T * e->H * e->esz, 1);
    CK(e, launch_embed<T>((const T*)e->embed, d_ids, (T*)e->x, p.T, e->H, e->c.vocab, e->d_err, s), "embed");
  }
  int rc = run_layers<T>(e, p);
  if (rc) return rc;
  if (p.mode != 0) {
    {
      Scope sc(e, DCD_PROF_ELEMENTWISE, (double)p.B * e->H * (e->esz + 4.0), 1);
      CK(e, launch_final_norm_rows<T>((const T*)e->x, (const T*)e->final_norm, e->hid, e->d_last, p.B, e->H, e->c.rms_eps, s), "final norm");
    }
    Scope sc(e, DCD_PROF_READOUT, 2.0 * p.B * e->H * e->c.readout_rows, 1);
    CK(e, launch_readout(e->hid, e->readout, d_out, p.B, e->H, e->c.readout_rows, s), "readout");
  }
  return DCD_OK;
}

// (Re)build the e4m3 weight images from the bf16 weights: per-output-row scale, as
// weights.rs:472-492 does with quant_fp8_bf16 at load time.
int ensure_fp8_weights(dcd_engine* e) {
  if (!e->fp8 || !e->fp8_dirty) return DCD_OK;
  auto q = [&](const void* w, LayerW::Fp8W& f, int n, int k) -> cudaError_t {
    e->launches += 1;
    return launch_quant_fp8_rows<bf16>((const bf16*)w, (size_t)k, f.q, f.scale, n, k, 1.0f, e->stream);
  };
  for (LayerW& w : e->layers) {
    CK(e, q(w.w_gu, w.f_gu, e->gu_rows, e->H), "fp8 weight quantisation");
    CK(e, q(w.w_down, w.f_down, e->H, e->I), "fp8 weight quantisation");
    if (w.full) {
      CK(e, q(w.w_qkv, w.f_qkv, e->qkv_n, e->H), "fp8 weight quantisation");
      CK(e, q(w.w_o, w.f_o, e->H, e->c.heads * e->c.head_dim), "fp8 weight quantisation");
    } else {
      CK(e, q(w.w_gin, w.f_gin, e->gin_n, e->H), "fp8 weight quantisation");
      CK(e, q(w.w_out, w.f_out, e->H, e->vd), "fp8 weight quantisation");
    }
  }
  e->fp8_dirty = false;
  return DCD_OK;
}

int run_pass_any(dcd_engine* e, const Pass& p, const uint32_t* d_ids, const int32_t* d_lens, int pos_start, float* d_out) {
  if (int rc = ensure_fp8_weights(e)) return rc;
  return e->bf ? run_pass<bf16>(e, p, d_ids, d_lens, pos_start, d_out) : run_pass<float>(e, p, d_ids, d_lens, pos_start, d_out);
}

int check_device_error(dcd_engine* e) {
  // caller has synchronised the stream after copying d_err into h_err
  const int code = *e->h_err;
  if (code == DERR_NONE) return DCD_OK;
  cudaMemsetAsync(e->d_err, 0, sizeof(int), e->stream);
  cudaStreamSynchronize(e->stream);
  switch (code) {
    case DERR_TOKEN_RANGE: return fail(e, DCD_E_INVALID, "token id out of range for vocabulary %d", e->c.vocab);
    case DERR_EMPTY_ITEM: return fail(e, DCD_E_INVALID, "batch item has no tokens");
    case DERR_POSITION_RANGE: return fail(e, DCD_E_INVALID, "position beyond the RoPE table (%d)", e->o.max_positions);
    case DERR_GEMM_TIMEOUT: return fail(e, DCD_E_TIMEOUT, "tcgen05 GEMM: a bounded barrier wait gave up");
    case DERR_ATTN_TIMEOUT: return fail(e, DCD_E_TIMEOUT, "tcgen05 attention: a bounded barrier wait gave up");
    case DERR_GDN_TIMEOUT: return fail(e, DCD_E_TIMEOUT, "tcgen05 gated delta rule: a bounded barrier wait gave up");
    default: return fail(e, DCD_E_CUDA, "device error word %d", code);
  }
}

int sync_and_check(dcd_engine* e) {
  CK(e, cudaMemcpyAsync(e->h_err, e->d_err, sizeof(int), cudaMemcpyDeviceToHost, e->stream), "err copy");
  CK(e, cudaStreamSynchronize(e->stream), "stream sync");
  return check_device_error(e);
}

size_t state_bytes_for(const dcd_engine* e, size_t S) {
  const dcd_model_config& c = e->c;
  size_t b = 0;
  auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
  for (int i = 0; i < c.num_layers; ++i) {
    if (c.layer_is_full[i]) b += 2 * al(S * c.kv_heads * c.head_dim * e->esz);
    else b += al((size_t)c.gdn_v_heads * c.gdn_dk * c.gdn_dv * 4) + al((size_t)3 * e->conv_dim * e->esz);
  }
  return b;
}

void carve_state(const dcd_engine* e, dcd_state* st) {
  const dcd_model_config& c = e->c;
  const int L = c.num_layers;
  st->k.assign(L, nullptr); st->v.assign(L, nullptr); st->hist.assign(L, nullptr); st->gstate.assign(L, nullptr);
  char* p = (char*)st->block;
  auto al = [](size_t x) { return (x + 255) & ~(size_t)255; };
  for (int i = 0; i < L; ++i) {
    if (c.layer_is_full[i]) {
      const size_t n = al(st->state_len * c.kv_heads * c.head_dim * e->esz);
      st->k[i] = p; p += n;
      st->v[i] = p; p += n;
    } else {
      st->gstate[i] = (float*)p; p += al((size_t)c.gdn_v_heads * c.gdn_dk * c.gdn_dv * 4);
      st->hist[i] = p; p += al((size_t)3 * e->conv_dim * e->esz);
    }
  }
}

int new_state(dcd_engine* e, size_t S, dcd_state** out) {
  dcd_state* st = new dcd_state();
  st->state_len = S;
  st->pos_end = S;
  st->bytes = state_bytes_for(e, S);
  cudaError_t ce = cudaMallocAsync(&st->block, st->bytes, e->stream);
  if (ce != cudaSuccess) {
    delete st;
    cudaGetLastError();
    return cuda_fail(e, ce, "state cache allocation");
  }
  carve_state(e, st);
  *out = st;
  return DCD_OK;
}

}  // namespace

// =================================================================================
// C ABI
// =================================================================================
extern "C" {

const char* dcd_last_error(const dcd_engine* e) { return e ? e->err.c_str() : g_create_error.c_str(); }

int dcd_engine_create(const dcd_model_config* cfg, const dcd_options* opt, int device, dcd_engine** out) {
  if (!out) return DCD_E_INVALID;
  *out = nullptr;
  if (!cfg) return fail(nullptr, DCD_E_INVALID, "null config");
  const dcd_model_config& c = *cfg;
  if (c.num_layers <= 0 || c.num_layers > 256 || c.hidden <= 0 || c.heads <= 0 || c.kv_heads <= 0 || c.heads % c.kv_heads ||
      c.intermediate <= 0 || c.vocab <= 0 || c.readout_rows <= 0)
    return fail(nullptr, DCD_E_INVALID, "invalid model config");
  if (c.conv_kernel != 4) return fail(nullptr, DCD_E_UNSUPPORTED, "conv kernel %d unsupported (4 only)", c.conv_kernel);
  if (c.head_dim != 64 && c.head_dim != 128 && c.head_dim != 256) return fail(nullptr, DCD_E_UNSUPPORTED, "head_dim %d unsupported", c.head_dim);
  if ((c.gdn_dk != 64 && c.gdn_dk != 128) || c.gdn_dv % 16 || c.gdn_v_heads % c.gdn_k_heads)
    return fail(nullptr, DCD_E_UNSUPPORTED, "GDN dims unsupported");
  if (c.rotary_dim % 2 || c.rotary_dim > c.head_dim) return fail(nullptr, DCD_E_INVALID, "rotary_dim invalid");
  if (c.dtype != 0 && c.dtype != 1) return fail(nullptr, DCD_E_INVALID, "dtype must be 0 (f32) or 1 (bf16)");
  dcd_options o = {};
  if (opt) o = *opt;
  if (o.precision < 0 || o.precision > 3) return fail(nullptr, DCD_E_UNSUPPORTED, "precision %d unknown (0 = config dtype, 1 = w4a16 g128, 2 = fp8, 3 = nvfp4)", o.precision);
  if (o.precision == 3 && ((c.hidden % 16) || (c.intermediate % 16) || ((c.heads * c.head_dim) % 16) || ((c.gdn_v_heads * c.gdn_dv) % 16) || (o.gemm_path != 0 && o.gemm_path != 2)))
    return fail(nullptr, DCD_E_UNSUPPORTED, "nvfp4 needs every GEMM K to be a multiple of 16 and the tensor-core GEMM path");
  if (o.precision != 0 && c.dtype != 1) return fail(nullptr, DCD_E_UNSUPPORTED, "w4a16 / fp8 precision needs a bf16 engine (dtype 1)");
  if (o.precision == 1 && ((c.hidden % 8) || (c.intermediate % 8))) return fail(nullptr, DCD_E_UNSUPPORTED, "w4a16 needs K multiples of 8");
  if (o.fp8_min_rows <= 0) o.fp8_min_rows = 512;
  if (o.nvfp4_scale_copy < 0 || o.nvfp4_scale_copy > 2) return fail(nullptr, DCD_E_INVALID, "nvfp4_scale_copy must be 0, 1 or 2");
  if (o.w4a16_gemm < 0 || o.w4a16_gemm > 2) return fail(nullptr, DCD_E_INVALID, "w4a16_gemm must be 0, 1 or 2");
  if (o.nvfp4_fusion < 0 || o.nvfp4_fusion > 1) return fail(nullptr, DCD_E_INVALID, "nvfp4_fusion must be 0 or 1");
  if (o.attn_split < 0 || o.attn_split > 1) return fail(nullptr, DCD_E_INVALID, "attn_split must be 0 or 1");
  if (o.w4a16_prefetch < 0 || o.w4a16_prefetch > 1) return fail(nullptr, DCD_E_INVALID, "w4a16_prefetch must be 0 or 1");
  if (o.gdn_overlap < 0 || o.gdn_overlap > 1) return fail(nullptr, DCD_E_INVALID, "gdn_overlap must be 0 or 1");
  if (o.max_pass_tokens <= 0) o.max_pass_tokens = 16384;
  if (o.max_rows <= 0) o.max_rows = 256;
  if (o.max_keys <= 0) o.max_keys = (int64_t)1 << 22;
  if (o.max_scores <= 0) o.max_scores = (int64_t)1 << 33;
  if (o.max_positions <= 0) o.max_positions = 65536;

  int ndev = 0;
  cudaError_t ce = cudaGetDeviceCount(&ndev);
  if (ce != cudaSuccess || ndev == 0) {
    cudaGetLastError();
    return fail(nullptr, DCD_E_CUDA, "no CUDA device: %s", ce == cudaSuccess ? "count is 0" : cudaGetErrorString(ce));
  }
  if (device < 0 || device >= ndev) return fail(nullptr, DCD_E_INVALID, "device %d out of range (%d devices)", device, ndev);
  ce = cudaSetDevice(device);
  if (ce != cudaSuccess) return fail(nullptr, DCD_E_CUDA, "cudaSetDevice: %s", cudaGetErrorString(ce));
  cudaDeviceProp prop;
  cudaGetDeviceProperties(&prop, device);
  if (prop.major != 10) return fail(nullptr, DCD_E_UNSUPPORTED, "device %s is sm_%d%d; this library is built for sm_100a only", prop.name, prop.major, prop.minor);

  dcd_engine* e = new dcd_engine();
  e->c = c;
  e->o = o;
  e->device = device;
  e->sm_count = prop.multiProcessorCount;
  e->cc_major = prop.major;
  e->cc_minor = prop.minor;
  snprintf(e->device_name, sizeof e->device_name, "%s", prop.name);
  e->bf = c.dtype == 1;
  e->esz = e->bf ? 2 : 4;
  e->H = c.hidden;
  e->I = c.intermediate;
  e->qcols = c.heads * 2 * c.head_dim;
  e->kvcols = c.kv_heads * c.head_dim;
  e->qkv_n = e->qcols + 2 * e->kvcols;
  e->conv_dim = 2 * c.gdn_k_heads * c.gdn_dk + c.gdn_v_heads * c.gdn_dv;
  e->vd = c.gdn_v_heads * c.gdn_dv;
  e->gin_n = (e->conv_dim + e->vd + 2 * c.gdn_v_heads + 7) & ~7;
  e->gu_rows = ((e->I + 127) / 128) * 256;
  e->rhalf = c.rotary_dim / 2;
  e->Tm = o.max_pass_tokens;
  e->max_batch = o.max_pass_tokens;  // a question has >= 1 token
  if ((e->H * e->esz) % 16 || (e->conv_dim % 8) || (e->qkv_n % 8)) {
    delete e;
    return fail(nullptr, DCD_E_UNSUPPORTED, "hidden/projection widths must keep rows 16-byte aligned");
  }

#define CRE(expr, what)                                            \
  do {                                                             \
    cudaError_t _ce = (expr);                                      \
    if (_ce != cudaSuccess) {                                      \
      int _rc = cuda_fail(nullptr, _ce, what);                     \
      dcd_engine_destroy(e);                                       \
      return _rc;                                                  \
    }                                                              \
  } while (0)
#define CRA(ptr, bytes, zero, tally)                                                   \
  do {                                                                                 \
    int _rc = dev_alloc(e, reinterpret_cast<void**>(&(ptr)), (bytes), (zero), (tally)); \
    if (_rc) { g_create_error = e->err; dcd_engine_destroy(e); return _rc; }           \
  } while (0)

  CRE(cudaStreamCreateWithFlags(&e->stream, cudaStreamNonBlocking), "stream");
  {
    // State blocks come from the device's default stream-ordered pool. Its default release threshold (0) hands
    // freed blocks back to the driver at the next synchronisation, so a host that frees a state and captures
    // the next one around a blocking readout pays a fresh ~300 MB reservation each time. Keep freed blocks
    // cached; dcd_trim_pools returns them on request (Engine::trim_pools, native/src/engine.rs:1044, has the same role).
    cudaMemPool_t pool;
    uint64_t keep = UINT64_MAX;
    CRE(cudaDeviceGetDefaultMemPool(&pool, e->device), "mem pool");
    CRE(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep), "mem pool release threshold");
  }
  CRE(cudaEventCreate(&e->t0), "event");
  CRE(cudaEventCreate(&e->t1), "event");
  if (e->bf) CRE(tc_gemm_prepare_device(), "tcgen05 GEMM shared-memory attribute");
  e->attn_tc = e->bf && o.attn_path == 0 && attn_tc_supported(c.heads, c.kv_heads, c.head_dim);
  if (e->attn_tc) CRE(attn_tc_prepare_device(), "tcgen05 attention shared-memory attribute");
  e->fp8 = o.precision == 2 && o.gemm_path == 0;
  e->w4 = o.precision == 1;
  e->nv4 = o.precision == 3;
  e->nv4_native = e->nv4 && o.gemm_path == 0;
  if (e->nv4_native) CRE(nvfp4_gemm_prepare_device(), "nvfp4 GEMM shared-memory attribute");
  if (e->w4 && o.gemm_path == 0) CRE(w4a16_gemm_prepare_device(), "w4a16 GEMM shared-memory attribute");
  e->gdn_tc = e->bf && (o.gdn_path == 0 || o.gdn_path == 3) && gdn_tc_supported(c.gdn_dk, c.gdn_dv);
  e->gdn_wy = e->gdn_tc && o.gdn_path == 0;
  if (e->gdn_tc) CRE(gdn_tc_prepare_device<bf16>(), "tcgen05 GDN shared-memory attribute");
  if (e->gdn_wy) CRE(gdn_wy_prepare_device<bf16>(), "tcgen05 WY GDN shared-memory attribute");
  if (e->gdn_wy && o.gdn_overlap == 0) {
    CRE(cudaStreamCreateWithFlags(&e->stream_gdn, cudaStreamNonBlocking), "GDN stream");
    CRE(cudaEventCreateWithFlags(&e->gdn_fork, cudaEventDisableTiming), "event");
    CRE(cudaEventCreateWithFlags(&e->gdn_join, cudaEventDisableTiming), "event");
  }
  e->gdn_chunked = e->bf && !e->gdn_tc && (o.gdn_path == 0 || o.gdn_path == 2) && gdn_chunked_supported(c.gdn_dk, c.gdn_dv);
  if (e->gdn_chunked) CRE(gdn_chunked_prepare_device<bf16>(), "chunked GDN shared-memory attribute");

  const size_t es = e->esz, H = e->H;
  // ---- weights
  e->layers.resize(c.num_layers);
  if (e->w4 || e->nv4) {
    size_t mx = (size_t)e->gu_rows * H;
    auto up = [&](size_t n) { if (n > mx) mx = n; };
    up(H * (size_t)e->I); up((size_t)e->qkv_n * H); up(H * (size_t)c.heads * c.head_dim); up((size_t)e->gin_n * H); up(H * (size_t)e->vd);
    CRA(e->wstage, mx * 2, true, &e->weight_bytes);
    if (e->nv4) CRA(e->amax_tmp, 256, true, &e->weight_bytes);
    if (e->w4 && e->bf && o.w4a16_prefetch == 1) {
      CRA(e->wstage2, mx * 2, true, &e->weight_bytes);
      CRE(cudaStreamCreateWithFlags(&e->stream2, cudaStreamNonBlocking), "second stream");
      for (int i = 0; i < 2; ++i) {
        CRE(cudaEventCreateWithFlags(&e->w4_free[i], cudaEventDisableTiming), "event");
        CRE(cudaEventCreateWithFlags(&e->w4_ready[i], cudaEventDisableTiming), "event");
      }
    }
  }
  CRA(e->embed, (size_t)c.vocab * H * es, false, &e->weight_bytes);
  CRA(e->final_norm, H * es, true, &e->weight_bytes);
  CRA(e->readout, (size_t)c.readout_rows * H * 4, true, &e->weight_bytes);
  for (int i = 0; i < c.num_layers; ++i) {
    LayerW& w = e->layers[i];
    w.full = c.layer_is_full[i] != 0;
    CRA(w.input_norm, H * es, true, &e->weight_bytes);
    CRA(w.post_norm, H * es, true, &e->weight_bytes);
    if (e->nv4) {
      auto mkn = [&](LayerW::NV4& g, size_t n, size_t k) -> int {
        g.N = (int)n; g.K = (int)k;
        int rc = dev_alloc(e, reinterpret_cast<void**>(&g.q), n * k / 2, true, &e->weight_bytes);
        if (!rc) rc = dev_alloc(e, reinterpret_cast<void**>(&g.sf), n * k / 16, true, &e->weight_bytes);
        if (!rc) rc = dev_alloc(e, reinterpret_cast<void**>(&g.wg), 256, true, &e->weight_bytes);
        if (!rc && e->nv4_native && (k % 256) == 0) {  // shapes the block-scaled kernel takes; others go the dequantise + bf16 route
          rc = dev_alloc(e, reinterpret_cast<void**>(&g.sft), nvfp4_sf_tiled_bytes((int)n, (int)k), true, &e->weight_bytes);
          if (!rc && (tc_make_tmap_fp8_a(&g.tm, g.q, n, k / 2) || tc_make_tmap_fp8_b(&g.tm256, g.q, n, k / 2)))
            rc = fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an nvfp4 weight operand");
        }
        g.alpha = g.wg + 1;
        return rc;
      };
      int rc = mkn(w.n_gu, e->gu_rows, H);
      if (!rc) rc = mkn(w.n_down, H, e->I);
      if (!rc && w.full) { rc = mkn(w.n_qkv, e->qkv_n, H); if (!rc) rc = mkn(w.n_o, H, (size_t)c.heads * c.head_dim); }
      if (!rc && !w.full) { rc = mkn(w.n_gin, e->gin_n, H); if (!rc) rc = mkn(w.n_out, H, e->vd); }
      if (rc) { g_create_error = e->err; dcd_engine_destroy(e); return rc; }
    }
    if (e->w4 || e->nv4) {
      auto mk4 = [&](LayerW::W4& g, size_t n, size_t k) -> int {
        if (!e->w4) return DCD_OK;
        g.N = (int)n; g.K = (int)k;
        int rc = dev_alloc(e, reinterpret_cast<void**>(&g.q), n * ((k + 7) / 8) * 4, true, &e->weight_bytes);
        if (!rc) rc = dev_alloc(e, &g.scale, n * ((k + 127) / 128) * 2, true, &e->weight_bytes);
        if (!rc && (k % 128) == 0 && o.gemm_path == 0) {  // shapes the fused W4A16 GEMM takes
          rc = dev_alloc(e, &g.scale_t, n * (k / 128) * 2, true, &e->weight_bytes);
          if (!rc && w4a16_make_tmap_packed(&g.tm_q, g.q, n, k)) rc = fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an int4 weight operand");
          g.fused = !rc;
        }
        if (!rc && e->bf && o.gemm_path == 0) {  // the weight's image in either dequantisation stage, as a GEMM operand
          if (tc_make_tmap_b(&g.tm_stage[0], e->wstage, n, k) || (e->wstage2 && tc_make_tmap_b(&g.tm_stage[1], e->wstage2, n, k)))
            rc = tc_shape_ok(128, (int)n, (int)k) ? fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for a staged weight operand") : DCD_OK;
        }
        return rc;
      };
      int rc = mk4(w.g_gu, e->gu_rows, H);
      if (!rc) rc = mk4(w.g_down, H, e->I);
      if (!rc && w.full) { rc = mk4(w.g_qkv, e->qkv_n, H); if (!rc) rc = mk4(w.g_o, H, (size_t)c.heads * c.head_dim); }
      if (!rc && !w.full) { rc = mk4(w.g_gin, e->gin_n, H); if (!rc) rc = mk4(w.g_out, H, e->vd); }
      if (rc) { g_create_error = e->err; dcd_engine_destroy(e); return rc; }
      // every bf16 weight pointer aliases the shared stage (filled by the dequantiser before each GEMM)
      w.w_gu = w.w_down = e->wstage;
      if (w.full) { w.w_qkv = w.w_o = e->wstage; CRA(w.qnorm, c.head_dim * es, true, &e->weight_bytes); CRA(w.knorm, c.head_dim * es, true, &e->weight_bytes); }
      else {
        w.w_gin = w.w_out = e->wstage;
        CRA(w.conv, (size_t)e->conv_dim * 4 * es, true, &e->weight_bytes);
        CRA(w.gnorm, c.gdn_dv * es, true, &e->weight_bytes);
        CRA(w.A_log, c.gdn_v_heads * 4, true, &e->weight_bytes);
        CRA(w.dt_bias, c.gdn_v_heads * 4, true, &e->weight_bytes);
      }
    } else {
    CRA(w.w_gu, (size_t)e->gu_rows * H * es, true, &e->weight_bytes);
    CRA(w.w_down, H * (size_t)e->I * es, true, &e->weight_bytes);
    if (w.full) {
      CRA(w.w_qkv, (size_t)e->qkv_n * H * es, true, &e->weight_bytes);
      CRA(w.w_o, H * (size_t)c.heads * c.head_dim * es, true, &e->weight_bytes);
      CRA(w.qnorm, c.head_dim * es, true, &e->weight_bytes);
      CRA(w.knorm, c.head_dim * es, true, &e->weight_bytes);
    } else {
      CRA(w.w_gin, (size_t)e->gin_n * H * es, true, &e->weight_bytes);
      CRA(w.w_out, H * (size_t)e->vd * es, true, &e->weight_bytes);
      CRA(w.conv, (size_t)e->conv_dim * 4 * es, true, &e->weight_bytes);
      CRA(w.gnorm, c.gdn_dv * es, true, &e->weight_bytes);
      CRA(w.A_log, c.gdn_v_heads * 4, true, &e->weight_bytes);
      CRA(w.dt_bias, c.gdn_v_heads * 4, true, &e->weight_bytes);
    }
    }
    if (e->fp8) {
      auto mk = [&](LayerW::Fp8W& f, size_t n, size_t k) -> int {
        int rc = dev_alloc(e, reinterpret_cast<void**>(&f.q), n * k, false, &e->weight_bytes);
        if (!rc) rc = dev_alloc(e, reinterpret_cast<void**>(&f.scale), n * 4, false, &e->weight_bytes);
        if (!rc && tc_make_tmap_fp8_b(&f.tm, f.q, n, k)) rc = fail(e, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for an fp8 weight operand");
        return rc;
      };
      int rc = mk(w.f_gu, e->gu_rows, H);
      if (!rc) rc = mk(w.f_down, H, e->I);
      if (!rc && w.full) { rc = mk(w.f_qkv, e->qkv_n, H); if (!rc) rc = mk(w.f_o, H, (size_t)c.heads * c.head_dim); }
      if (!rc && !w.full) { rc = mk(w.f_gin, e->gin_n, H); if (!rc) rc = mk(w.f_out, H, e->vd); }
      if (rc) { g_create_error = e->err; dcd_engine_destroy(e); return rc; }
    }
    if (e->bf) {
      int bad = tc_make_tmap_b(&w.tm_gu, w.w_gu, e->gu_rows, H) | tc_make_tmap_b(&w.tm_down, w.w_down, H, e->I);
      if (w.full) bad |= tc_make_tmap_b(&w.tm_qkv, w.w_qkv, e->qkv_n, H) | tc_make_tmap_b(&w.tm_o, w.w_o, H, (uint64_t)c.heads * c.head_dim);
      else bad |= tc_make_tmap_b(&w.tm_gin, w.w_gin, e->gin_n, H) | tc_make_tmap_b(&w.tm_out, w.w_out, H, e->vd);
      if (bad && o.gemm_path == 0) {
        dcd_engine_destroy(e);
        return fail(nullptr, DCD_E_CUDA, "cuTensorMapEncodeTiled failed for a weight operand (layer %d)", i);
      }
    }
  }
  // ---- RoPE tables, built on the host exactly as Engine::rope_tables_positions does
  // (native/src/engine.rs:1619-1643), once for every position.
  {
    const int half = e->rhalf, P = o.max_positions;
    std::vector<float> inv(half > 0 ? half : 1);
    for (int i = 0; i < half; ++i) inv[i] = 1.0f / powf(c.rope_theta, (float)(2 * i) / (float)c.rotary_dim);
    const size_t n = (size_t)P * (half > 0 ? half : 1);
    std::vector<unsigned char> cs(n * es), sn(n * es);
    for (int p = 0; p < P && half > 0; ++p)
      for (int i = 0; i < half; ++i) {
        const float ang = (float)p * inv[i];
        const float cv = cosf(ang), sv = sinf(ang);
        const size_t at = (size_t)p * half + i;
        if (e->bf) { ((uint16_t*)cs.data())[at] = host_bf16(cv); ((uint16_t*)sn.data())[at] = host_bf16(sv); }
        else { ((float*)cs.data())[at] = cv; ((float*)sn.data())[at] = sv; }
      }
    CRA(e->cos_t, n * es, false, &e->weight_bytes);
    CRA(e->sin_t, n * es, false, &e->weight_bytes);
    CRE(cudaMemcpyAsync(e->cos_t, cs.data(), n * es, cudaMemcpyHostToDevice, e->stream), "rope upload");
    CRE(cudaMemcpyAsync(e->sin_t, sn.data(), n * es, cudaMemcpyHostToDevice, e->stream), "rope upload");
    CRE(cudaStreamSynchronize(e->stream), "rope upload");
  }
  // ---- workspace
  const size_t Tm = e->Tm;
  size_t bigw = e->qkv_n;
  if ((size_t)e->gin_n > bigw) bigw = e->gin_n;
  if ((size_t)e->gu_rows > bigw) bigw = e->gu_rows;
  size_t aw = (size_t)c.heads * c.head_dim;
  if ((size_t)e->vd > aw) aw = e->vd;
  size_t* ws = &e->workspace_bytes;
  CRA(e->x, Tm * H * es, false, ws);
  CRA(e->h, Tm * H * es, false, ws);
  CRA(e->x1, Tm * H * es, false, ws);
  CRA(e->mix, Tm * H * es, false, ws);
  CRA(e->big, Tm * bigw * es, false, ws);
  CRA(e->q, Tm * (size_t)c.heads * c.head_dim * es, false, ws);
  CRA(e->kown, Tm * (size_t)e->kvcols * es, false, ws);
  CRA(e->bufA, Tm * aw * es, false, ws);
  CRA(e->bufB, Tm * aw * es, false, ws);
  CRA(e->conv, Tm * (size_t)e->conv_dim * es, false, ws);
  CRA(e->act, Tm * (size_t)e->I * es, false, ws);
  e->max_k = e->I;
  if (e->H > e->max_k) e->max_k = e->H;
  if ((int)aw > e->max_k) e->max_k = (int)aw;
  if (e->nv4) CRA(e->xstage, Tm * (size_t)e->max_k * 2, false, ws);
  if (e->nv4_native) {
    CRA(e->xq, Tm * (size_t)e->max_k / 2, false, ws);
    CRA(e->xsf, Tm * (size_t)e->max_k / 16, false, ws);
    CRA(e->xsft, nvfp4_sf_tiled_bytes((int)Tm, (e->max_k + 63) / 64 * 64) + 512, false, ws);
    CRA(e->aq4, Tm * (size_t)e->I / 2, false, ws);
    CRA(e->asft4, nvfp4_sf_tiled_bytes((int)Tm, (e->I + 63) / 64 * 64) + 512, false, ws);
  }
  if (e->fp8) {
    CRA(e->aq, Tm * (size_t)e->max_k, false, ws);
    CRA(e->a_scale, Tm * 4, false, ws);
  }
  CRA(e->qf, Tm * (size_t)c.gdn_k_heads * c.gdn_dk * 4, false, ws);
  CRA(e->kf, Tm * (size_t)c.gdn_k_heads * c.gdn_dk * 4, false, ws);
  CRA(e->g, Tm * (size_t)c.gdn_v_heads * 4, false, ws);
  CRA(e->beta, Tm * (size_t)c.gdn_v_heads * 4, false, ws);
  CRA(e->hid, (size_t)e->max_batch * H * 4, false, ws);
  CRA(e->d_logits, (size_t)e->max_batch * c.readout_rows * 4, false, ws);
  CRA(e->d_ids, Tm * 4, false, ws);
  CRA(e->d_lens, (size_t)e->max_batch * 4, false, ws);
  CRA(e->d_posq, (size_t)e->max_batch * 4, false, ws);
  CRA(e->d_cu, ((size_t)e->max_batch + 1) * 4, false, ws);
  CRA(e->d_last, (size_t)e->max_batch * 4, false, ws);
  CRA(e->d_tile_cu, ((size_t)e->max_batch + 1) * 4, false, ws);
  if (e->attn_tc && o.attn_split == 0) CRA(e->attn_ws, attn_tc_split_workspace_bytes(e->sm_count), false, ws);  // parts of split launches
  CRA(e->d_tokq, Tm * 4, false, ws);
  CRA(e->d_tokpos, Tm * 4, false, ws);
  CRA(e->d_err, 256, true, ws);
  CRE(cudaMallocHost(&e->h_ids, Tm * 4), "pinned ids");
  CRE(cudaMallocHost(&e->h_lens, (size_t)e->max_batch * 4), "pinned lens");
  CRE(cudaMallocHost(&e->h_posq, (size_t)e->max_batch * 4), "pinned positions");
  CRE(cudaMallocHost(&e->h_logits, (size_t)e->max_batch * c.readout_rows * 4), "pinned logits");
  CRE(cudaMallocHost(&e->h_err, 64), "pinned err");
  *e->h_err = 0;
  CRE(cudaStreamSynchronize(e->stream), "create sync");
#undef CRE
#undef CRA
  *out = e;
  return DCD_OK;
}

void dcd_engine_destroy(dcd_engine* e) {
  if (!e) return;
  cudaSetDevice(e->device);
  if (e->stream) cudaStreamSynchronize(e->stream);
  for (void* p : e->allocs) cudaFree(p);
  if (e->h_ids) cudaFreeHost(e->h_ids);
  if (e->h_lens) cudaFreeHost(e->h_lens);
  if (e->h_posq) cudaFreeHost(e->h_posq);
  if (e->h_logits) cudaFreeHost(e->h_logits);
  if (e->h_err) cudaFreeHost(e->h_err);
  for (auto& pr : e->prof.pairs) { cudaEventDestroy(pr.a); cudaEventDestroy(pr.b); }
  for (auto ev : e->prof.pool) cudaEventDestroy(ev);
  if (e->t0) cudaEventDestroy(e->t0);
  if (e->t1) cudaEventDestroy(e->t1);
  if (e->stream2) { cudaStreamSynchronize(e->stream2); cudaStreamDestroy(e->stream2); }
  if (e->stream_gdn) { cudaStreamSynchronize(e->stream_gdn); cudaStreamDestroy(e->stream_gdn); }
  if (e->gdn_fork) cudaEventDestroy(e->gdn_fork);
  if (e->gdn_join) cudaEventDestroy(e->gdn_join);
  for (int i = 0; i < 2; ++i) {
    if (e->w4_free[i]) cudaEventDestroy(e->w4_free[i]);
    if (e->w4_ready[i]) cudaEventDestroy(e->w4_ready[i]);
  }
  if (e->stream) cudaStreamDestroy(e->stream);
  delete e;
}

int dcd_engine_info(const dcd_engine* e, dcd_info* out) {
  if (!e || !out) return DCD_E_INVALID;
  memset(out, 0, sizeof *out);
  out->device = e->device;
  out->sm_count = e->sm_count;
  out->cc_major = e->cc_major;
  out->cc_minor = e->cc_minor;
  snprintf(out->device_name, sizeof out->device_name, "%s", e->device_name);
  out->hidden = e->c.hidden;
  out->num_layers = e->c.num_layers;
  out->readout_rows = e->c.readout_rows;
  out->supports_vision = 0;
  out->weight_bytes = e->weight_bytes;
  out->workspace_bytes = e->workspace_bytes;
  return DCD_OK;
}

int dcd_rebind_blas(dcd_engine* e) { return e ? DCD_OK : DCD_E_INVALID; }

// W4 engines: a logical GEMM tensor is edited in the bf16 stage — bring the whole fused matrix in
// (dequantise), let the caller write or read its rows, then quantise the matrix back.
static int w4_stage_in(dcd_engine* e, const Loc& L) {
  if (L.nv) {
    e->launches += 1;
    CK(e, launch_nvfp4_dequant_rows(L.nv->q, L.nv->sf, L.nv->wg, (bf16*)e->wstage, L.nv->N, L.nv->K, e->stream), "nvfp4 stage in");
    return DCD_OK;
  }
  if (!L.w4) return DCD_OK;
  e->launches += 1;
  CK(e, launch_dequant_w4_g128(L.w4->q, L.w4->scale, (bf16*)e->wstage, L.w4->N, L.w4->K, e->stream, true), "w4 stage in");
  return DCD_OK;
}
static int w4_stage_out(dcd_engine* e, const Loc& L) {
  if (L.nv) {
    // tensor scale 2688/absmax of the whole fused matrix, then per-16 e4m3 scales and e2m1 codes
    e->launches += 3;
    CK(e, launch_absmax_bf16((const bf16*)e->wstage, (size_t)L.nv->N * L.nv->K, e->amax_tmp, e->stream), "nvfp4 absmax");
    CK(e, launch_nvfp4_global(e->amax_tmp, L.nv->wg, L.nv->alpha, 1.0f, e->stream), "nvfp4 tensor scale");
    CK(e, launch_nvfp4_quant_rows((const bf16*)e->wstage, (size_t)L.nv->K, L.nv->wg, 0.f, L.nv->q, L.nv->sf, L.nv->N, L.nv->K, e->stream), "nvfp4 stage out");
    if (L.nv->sft) {
      e->launches += 1;
      CK(e, launch_nvfp4_sf_tile(L.nv->sf, L.nv->sft, L.nv->N, L.nv->K, e->stream), "nvfp4 scale tiling");
    }
    return DCD_OK;
  }
  if (!L.w4) return DCD_OK;
  e->launches += 1;
  CK(e, launch_quant_w4_g128((const bf16*)e->wstage, L.w4->q, L.w4->scale, L.w4->N, L.w4->K, e->stream, true), "w4 stage out");
  if (L.w4->scale_t) {
    e->launches += 1;
    CK(e, launch_w4_scale_transpose(L.w4->scale, L.w4->scale_t, L.w4->N, (L.w4->K + 127) / 128, e->stream), "w4 scale transpose");
  }
  return DCD_OK;
}

// first/last: position of this logical tensor inside its fused matrix. Quantised engines zero the
// stage before the first tensor and quantise the whole fused matrix once after the last one (the
// NVFP4 tensor scale is taken over the complete matrix).
static int gen_one(dcd_engine* e, uint64_t seed, int layer, int kind, bool first = true, bool last = true) {
  Loc L;
  if (!locate(e, layer, kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", kind, layer);
  if ((L.w4 || L.nv) && first) {
    const size_t n = L.w4 ? (size_t)L.w4->N * L.w4->K : (size_t)L.nv->N * L.nv->K;
    CK(e, cudaMemsetAsync(e->wstage, 0, n * 2, e->stream), "stage clear");
  }
  const GenSpec sp = spec_for(kind, e->bf);
  const float cc = (float)((double)sp.p0 / IH8_STD);
  const uint64_t key = gen_tensor_key(seed, layer, kind);
  const uint64_t count = (uint64_t)L.rows * L.cols;
  e->launches += 1;
  if (L.f32) CK(e, launch_gen_tensor<float>((float*)L.base, key, 0, count, (int)L.cols, sp.dist, sp.p0, sp.p1, cc, sp.round_bf, L.mode, L.row_offset, L.dst_stride, e->stream), "gen");
  else if (e->bf) CK(e, launch_gen_tensor<bf16>((bf16*)L.base, key, 0, count, (int)L.cols, sp.dist, sp.p0, sp.p1, cc, sp.round_bf, L.mode, L.row_offset, L.dst_stride, e->stream), "gen");
  else CK(e, launch_gen_tensor<float>((float*)L.base, key, 0, count, (int)L.cols, sp.dist, sp.p0, sp.p1, cc, sp.round_bf, L.mode, L.row_offset, L.dst_stride, e->stream), "gen");
  return last ? w4_stage_out(e, L) : DCD_OK;
}

int dcd_engine_init_random(dcd_engine* e, uint64_t seed) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  struct K { int kind; bool first, last; };
  static const K globals[] = {{DCD_T_EMBED, true, true}, {DCD_T_FINAL_NORM, true, true}, {DCD_T_READOUT, true, true}};
  static const K common[] = {{DCD_T_INPUT_NORM, true, true}, {DCD_T_POST_NORM, true, true}, {DCD_T_GATE, true, false}, {DCD_T_UP, false, true},
                             {DCD_T_DOWN, true, true}};
  static const K full[] = {{DCD_T_Q, true, false}, {DCD_T_K, false, false}, {DCD_T_V, false, true}, {DCD_T_O, true, true},
                           {DCD_T_QNORM, true, true}, {DCD_T_KNORM, true, true}};
  static const K gdn[] = {{DCD_T_IN_QKV, true, false}, {DCD_T_IN_Z, false, false}, {DCD_T_IN_B, false, false}, {DCD_T_IN_A, false, true},
                          {DCD_T_OUT, true, true}, {DCD_T_CONV, true, true}, {DCD_T_A_LOG, true, true}, {DCD_T_DT_BIAS, true, true},
                          {DCD_T_GNORM, true, true}};
  int rc;
  for (const K& k : globals) if ((rc = gen_one(e, seed, -1, k.kind, k.first, k.last))) return rc;
  for (int i = 0; i < e->c.num_layers; ++i) {
    for (const K& k : common) if ((rc = gen_one(e, seed, i, k.kind, k.first, k.last))) return rc;
    if (e->layers[i].full) { for (const K& k : full) if ((rc = gen_one(e, seed, i, k.kind, k.first, k.last))) return rc; }
    else { for (const K& k : gdn) if ((rc = gen_one(e, seed, i, k.kind, k.first, k.last))) return rc; }
  }
  CK(e, cudaStreamSynchronize(e->stream), "init_random sync");
  e->weights_ready = true;
  e->fp8_dirty = true;
  return DCD_OK;
}

int dcd_engine_load_tensor(dcd_engine* e, int layer, int kind, const float* host, size_t count) {
  if (!e || !host) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  Loc L;
  if (!locate(e, layer, kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", kind, layer);
  if (count != L.rows * L.cols) return fail(e, DCD_E_INVALID, "tensor kind %d expects %zu values, got %zu", kind, L.rows * L.cols, count);
  if (int rc0 = w4_stage_in(e, L)) return rc0;
  float* tmp = nullptr;
  void* tmpT = nullptr;
  cudaError_t ce = cudaMalloc(&tmp, count * 4);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "load_tensor staging");
  int rc = DCD_OK;
  do {
    if ((ce = cudaMemcpyAsync(tmp, host, count * 4, cudaMemcpyHostToDevice, e->stream)) != cudaSuccess) break;
    e->launches += 2;
    if (L.f32 || !e->bf) {
      ce = launch_place_rows<float>(tmp, (float*)L.base, L.rows, (int)L.cols, L.mode, L.row_offset, L.dst_stride, false, e->stream);
    } else {
      if ((ce = cudaMalloc(&tmpT, count * 2)) != cudaSuccess) break;
      if ((ce = launch_from_f32<bf16>(tmp, (bf16*)tmpT, count, e->stream)) != cudaSuccess) break;
      ce = launch_place_rows<bf16>((const bf16*)tmpT, (bf16*)L.base, L.rows, (int)L.cols, L.mode, L.row_offset, L.dst_stride, false, e->stream);
    }
    if (ce != cudaSuccess) break;
    if (w4_stage_out(e, L)) { rc = DCD_E_CUDA; break; }
    ce = cudaStreamSynchronize(e->stream);
  } while (0);
  if (ce != cudaSuccess) rc = cuda_fail(e, ce, "load_tensor");
  cudaFree(tmp);
  if (tmpT) cudaFree(tmpT);
  if (rc == DCD_OK) { e->weights_ready = true; e->fp8_dirty = true; }
  return rc;
}

int dcd_engine_read_tensor(dcd_engine* e, int layer, int kind, float* host, size_t count) {
  if (!e || !host) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  Loc L;
  if (!locate(e, layer, kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", kind, layer);
  if (count != L.rows * L.cols) return fail(e, DCD_E_INVALID, "tensor kind %d holds %zu values, asked for %zu", kind, L.rows * L.cols, count);
  if (int rc0 = w4_stage_in(e, L)) return rc0;
  float* tmp = nullptr;
  void* tmpT = nullptr;
  cudaError_t ce = cudaMalloc(&tmp, count * 4);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "read_tensor staging");
  do {
    e->launches += 2;
    if (L.f32 || !e->bf) {
      ce = launch_place_rows<float>((const float*)L.base, tmp, L.rows, (int)L.cols, L.mode, L.row_offset, L.dst_stride, true, e->stream);
    } else {
      if ((ce = cudaMalloc(&tmpT, count * 2)) != cudaSuccess) break;
      if ((ce = launch_place_rows<bf16>((const bf16*)L.base, (bf16*)tmpT, L.rows, (int)L.cols, L.mode, L.row_offset, L.dst_stride, true, e->stream)) != cudaSuccess) break;
      ce = launch_to_f32<bf16>((const bf16*)tmpT, tmp, count, e->stream);
    }
    if (ce != cudaSuccess) break;
    if ((ce = cudaMemcpyAsync(host, tmp, count * 4, cudaMemcpyDeviceToHost, e->stream)) != cudaSuccess) break;
    ce = cudaStreamSynchronize(e->stream);
  } while (0);
  cudaFree(tmp);
  if (tmpT) cudaFree(tmpT);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "read_tensor");
  return DCD_OK;
}

}  // extern "C"

// ---- checkpoint loading ----------------------------------------------------------------
// WeightProvider::layer / linear / final_norm (native/src/weights.rs:283-630) and the readout head
// (HeadMatrix::load, native/src/engine.rs:747-783), re-hosted: tensors stream from the memory-mapped
// shards through a ring of pinned buffers, and one kernel per chunk converts the stored format
// (BF16 / F16 / F32, compressed-tensors int4, compressed-tensors NVFP4) and writes it to its place in
// the engine's fused matrices. Quantised engines (precision 1 and 3) collect a fused matrix in the bf16
// stage and quantise it once after its last member.
namespace {

// Page cache -> pinned buffer. One thread moves about 9 GB/s, well under the host link; large chunks are split
// over a few threads so that the staging copy keeps up with the H2D copy it overlaps with.
void parallel_copy(void* dst, const void* src, size_t bytes) {
  constexpr size_t MIN_PART = 4u << 20;
  unsigned hw = std::thread::hardware_concurrency();
  size_t parts = std::min<size_t>(std::min<size_t>(8, hw ? hw : 1), bytes / MIN_PART);
  if (parts <= 1) { memcpy(dst, src, bytes); return; }
  const size_t per = ((bytes / parts) + 4095) & ~(size_t)4095;
  std::vector<std::thread> th;
  for (size_t i = 1; i < parts; ++i) {
    const size_t off = i * per;
    if (off >= bytes) break;
    const size_t n = std::min(per, bytes - off);
    th.emplace_back([=] { memcpy((char*)dst + off, (const char*)src + off, n); });
  }
  memcpy(dst, src, std::min(per, bytes));
  for (auto& t : th) t.join();
}

// The same split for a range of an open file: pread copies straight out of the page cache (a first touch of the
// mapping would instead take one page fault per 4 KB, which caps a thread near 8 GB/s). Falls back to the mapping
// if a read comes back short.
void parallel_pread(int fd, size_t offset, void* dst, const void* mapped, size_t bytes) {
  constexpr size_t MIN_PART = 4u << 20;
  unsigned hw = std::thread::hardware_concurrency();
  const size_t parts = std::max<size_t>(1, std::min<size_t>(std::min<size_t>(8, hw ? hw : 1), bytes / MIN_PART));
  const size_t per = ((bytes / parts) + 4095) & ~(size_t)4095;
  auto part = [=](size_t off, size_t n) {
    size_t done = 0;
    while (done < n) {
      const ssize_t r = pread(fd, (char*)dst + off + done, n - done, (off_t)(offset + off + done));
      if (r <= 0) { memcpy((char*)dst + off + done, (const char*)mapped + off + done, n - done); return; }
      done += (size_t)r;
    }
  };
  std::vector<std::thread> th;
  for (size_t i = 1; i < parts; ++i) {
    const size_t off = i * per;
    if (off >= bytes) break;
    th.emplace_back(part, off, std::min(per, bytes - off));
  }
  part(0, std::min(per, bytes));
  for (auto& t : th) t.join();
}

struct Stager {
  static constexpr int N = 6;
  size_t cap = 0;
  void* h[N] = {};
  void* d[N] = {};
  cudaEvent_t idle[N] = {};
  int cur = 0;
  cudaStream_t s = nullptr;
  const ckpt::Store* store = nullptr;  // when set, sources inside its mappings are read with pread

  cudaError_t init(size_t cap_, cudaStream_t s_) {
    cap = cap_;
    s = s_;
    for (int i = 0; i < N; ++i) {
      cudaError_t ce = cudaMallocHost(&h[i], cap);
      if (ce == cudaSuccess) ce = cudaMalloc(&d[i], cap);
      if (ce == cudaSuccess) ce = cudaEventCreateWithFlags(&idle[i], cudaEventDisableTiming);
      if (ce != cudaSuccess) return ce;
    }
    return cudaSuccess;
  }
  void destroy() {
    for (int i = 0; i < N; ++i) {
      if (h[i]) cudaFreeHost(h[i]);
      if (d[i]) cudaFree(d[i]);
      if (idle[i]) cudaEventDestroy(idle[i]);
      h[i] = d[i] = nullptr;
      idle[i] = nullptr;
    }
  }
  // Copies `bytes` into the next slot (after the kernel that last read the slot has finished) and enqueues
  // the H2D copy. The caller enqueues the consumer and then calls release(slot).
  cudaError_t push(const void* src, size_t bytes, void** dev, int* slot) {
    if (bytes > cap) return cudaErrorInvalidValue;
    const int b = cur;
    cur = (cur + 1) % N;
    cudaError_t ce = cudaEventSynchronize(idle[b]);
    if (ce != cudaSuccess) return ce;
    int fd;
    size_t off;
    if (store && store->file_of(src, &fd, &off)) parallel_pread(fd, off, h[b], src, bytes);
    else parallel_copy(h[b], src, bytes);
    ce = cudaMemcpyAsync(d[b], h[b], bytes, cudaMemcpyHostToDevice, s);
    *dev = d[b];
    *slot = b;
    return ce;
  }
  cudaError_t release(int slot) { return cudaEventRecord(idle[slot], s); }
};

constexpr size_t STAGE_CHUNK = 32u << 20;

int src_dt_of(int ckpt_dtype) {
  switch (ckpt_dtype) {
    case ckpt::F32: return 0;
    case ckpt::F16: return 1;
    case ckpt::BF16: return 2;
    default: return -1;
  }
}

template <typename F>
int with_dst_type(dcd_engine* e, const Loc& L, F&& f) {
  return (L.f32 || !e->bf) ? f((float*)L.base) : f((bf16*)L.base);
}

// A plain tensor of `count` values in F32 / F16 / BF16 storage -> L.
int place_plain(dcd_engine* e, Stager& st, const char* name, const uint8_t* data, int ckpt_dtype, size_t count, const Loc& L) {
  const int sdt = src_dt_of(ckpt_dtype);
  if (sdt < 0) return fail(e, DCD_E_INVALID, "%s: expected F32, F16 or BF16 storage", name);
  if (count != L.rows * L.cols) return fail(e, DCD_E_INVALID, "%s: holds %zu values, the engine expects %zu x %zu", name, count, L.rows, L.cols);
  const size_t esz = ckpt::dtype_size(ckpt_dtype), row_bytes = L.cols * esz;
  const size_t chunk_rows = std::max<size_t>(1, st.cap / row_bytes);
  if (row_bytes > st.cap) return fail(e, DCD_E_INVALID, "%s: one row exceeds the staging buffer", name);
  for (size_t r0 = 0; r0 < L.rows; r0 += chunk_rows) {
    const size_t n = std::min(chunk_rows, L.rows - r0);
    void* dev;
    int slot;
    CK(e, st.push(data + r0 * row_bytes, n * row_bytes, &dev, &slot), "checkpoint upload");
    e->launches += 1;
    const int rc = with_dst_type(e, L, [&](auto* dst) {
      CK(e, launch_place_rows_cvt(dev, sdt, dst, n, (int)L.cols, r0, L.mode, L.row_offset, L.dst_stride, e->stream), "checkpoint placement");
      return (int)DCD_OK;
    });
    if (rc) return rc;
    CK(e, st.release(slot), "checkpoint staging");
  }
  return DCD_OK;
}

int need(dcd_engine* e, const ckpt::Store& s, const std::string& name, const ckpt::Tensor** out) {
  *out = s.info(name);
  if (!*out) return fail(e, DCD_E_INVALID, "tensor %s not found", name.c_str());
  return DCD_OK;
}

int load_vector(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& name, int layer, int kind) {
  Loc L;
  if (!locate(e, layer, kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", kind, layer);
  const ckpt::Tensor* t;
  if (int rc = need(e, s, name, &t)) return rc;
  return place_plain(e, st, name.c_str(), s.data(*t), t->dtype, t->count(), L);
}

// compressed-tensors pack-quantized int4 module -> bf16 values at L (weights.rs:292-330)
int place_ct_w4(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& module, const Loc& L) {
  const ckpt::Tensor *tp, *tsh, *tsc;
  if (int rc = need(e, s, module + ".weight_packed", &tp)) return rc;
  if (int rc = need(e, s, module + ".weight_shape", &tsh)) return rc;
  if (int rc = need(e, s, module + ".weight_scale", &tsc)) return rc;
  const ckpt::Tensor* tz = s.info(module + ".weight_zero_point");
  size_t out = 0, in = 0;
  if (tsh->count() != 2) return fail(e, DCD_E_INVALID, "%s.weight_shape: expected 2 entries", module.c_str());
  if (tsh->dtype == ckpt::I64) { const int64_t* v = (const int64_t*)s.data(*tsh); out = (size_t)v[0]; in = (size_t)v[1]; }
  else if (tsh->dtype == ckpt::I32) { const int32_t* v = (const int32_t*)s.data(*tsh); out = (size_t)v[0]; in = (size_t)v[1]; }
  else return fail(e, DCD_E_INVALID, "%s.weight_shape: expected I64", module.c_str());
  if (out != L.rows || in != L.cols) return fail(e, DCD_E_INVALID, "%s: checkpoint shape %zu x %zu, the engine expects %zu x %zu", module.c_str(), out, in, L.rows, L.cols);
  const size_t groups = tsc->shape.empty() ? 0 : tsc->shape.back();
  if (groups == 0 || in % groups) return fail(e, DCD_E_INVALID, "%s: in=%zu not divisible by groups=%zu", module.c_str(), in, groups);
  const size_t gs = in / groups;
  if (gs != 64 && gs != 128) return fail(e, DCD_E_INVALID, "%s: unsupported group size %zu", module.c_str(), gs);
  const size_t words = (in + 7) / 8, zp_rows = (out + 7) / 8;
  if (tp->dtype != ckpt::I32 || tp->count() != out * words) return fail(e, DCD_E_INVALID, "%s: packed has %zu words, expected %zu", module.c_str(), tp->count(), out * words);
  if (tsc->dtype != ckpt::BF16 || tsc->count() != out * groups || (tz && (tz->dtype != ckpt::I32 || tz->count() != zp_rows * groups)))
    return fail(e, DCD_E_INVALID, "%s: scale/zp size mismatch", module.c_str());
  const uint8_t *pp = s.data(*tp), *ps = s.data(*tsc), *pz = tz ? s.data(*tz) : nullptr;
  const size_t chunk_rows = std::max<size_t>(8, (st.cap / (words * 4)) & ~(size_t)7);
  if (8 * words * 4 > st.cap) return fail(e, DCD_E_INVALID, "%s: eight rows exceed the staging buffer", module.c_str());
  for (size_t r0 = 0; r0 < out; r0 += chunk_rows) {
    const size_t n = std::min(chunk_rows, out - r0);
    void *dp, *ds, *dz = nullptr;
    int sp, ss, sz = -1;
    CK(e, st.push(pp + r0 * words * 4, n * words * 4, &dp, &sp), "checkpoint upload");
    CK(e, st.push(ps + r0 * groups * 2, n * groups * 2, &ds, &ss), "checkpoint upload");
    if (pz) CK(e, st.push(pz + (r0 / 8) * groups * 4, ((n + 7) / 8) * groups * 4, &dz, &sz), "checkpoint upload");
    e->launches += 1;
    const int rc = with_dst_type(e, L, [&](auto* dst) {
      CK(e, launch_dequant_ct_w4_place((const int32_t*)dp, (const bf16*)ds, (const int32_t*)dz, dst, n, (int)in, (int)gs, r0, L.mode, L.row_offset,
                                       L.dst_stride, e->stream), "int4 checkpoint dequantisation");
      return (int)DCD_OK;
    });
    if (rc) return rc;
    CK(e, st.release(sp), "checkpoint staging");
    CK(e, st.release(ss), "checkpoint staging");
    if (sz >= 0) CK(e, st.release(sz), "checkpoint staging");
  }
  return DCD_OK;
}

// compressed-tensors nvfp4-pack-quantized module -> bf16 values at L (weights.rs:502-547)
int place_ct_nvfp4(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& module, const Loc& L) {
  const ckpt::Tensor *tp, *tsc, *tg;
  if (int rc = need(e, s, module + ".weight_packed", &tp)) return rc;
  if (int rc = need(e, s, module + ".weight_scale", &tsc)) return rc;
  if (int rc = need(e, s, module + ".weight_global_scale", &tg)) return rc;
  if (tp->shape.size() != 2) return fail(e, DCD_E_INVALID, "%s.weight_packed must be 2-D", module.c_str());
  const size_t out = tp->shape[0], in = tp->shape[1] * 2;
  if (in % 64) return fail(e, DCD_E_INVALID, "%s: K=%zu is not a multiple of 64", module.c_str(), in);
  if (tsc->shape.size() != 2 || tsc->shape[0] != out || tsc->shape[1] != in / 16 || ckpt::dtype_size(tsc->dtype) != 1 || ckpt::dtype_size(tp->dtype) != 1)
    return fail(e, DCD_E_INVALID, "%s: weight_scale must be [%zu, %zu] of 8-bit values", module.c_str(), out, in / 16);
  if (out != L.rows || in != L.cols) return fail(e, DCD_E_INVALID, "%s: checkpoint shape %zu x %zu, the engine expects %zu x %zu", module.c_str(), out, in, L.rows, L.cols);
  float global = 0.f;
  if (tg->count() < 1) return fail(e, DCD_E_INVALID, "%s: weight_global_scale empty", module.c_str());
  if (tg->dtype == ckpt::F32) memcpy(&global, s.data(*tg), 4);
  else if (tg->dtype == ckpt::BF16) { uint16_t hv; memcpy(&hv, s.data(*tg), 2); const uint32_t u = (uint32_t)hv << 16; memcpy(&global, &u, 4); }
  else return fail(e, DCD_E_INVALID, "%s.weight_global_scale: expected F32/BF16", module.c_str());
  const uint8_t *pp = s.data(*tp), *ps = s.data(*tsc);
  const size_t row_bytes = in / 2, chunk_rows = std::max<size_t>(1, st.cap / row_bytes);
  if (row_bytes > st.cap) return fail(e, DCD_E_INVALID, "%s: one row exceeds the staging buffer", module.c_str());
  for (size_t r0 = 0; r0 < out; r0 += chunk_rows) {
    const size_t n = std::min(chunk_rows, out - r0);
    void *dp, *ds;
    int sp, ss;
    CK(e, st.push(pp + r0 * row_bytes, n * row_bytes, &dp, &sp), "checkpoint upload");
    CK(e, st.push(ps + r0 * (in / 16), n * (in / 16), &ds, &ss), "checkpoint upload");
    e->launches += 1;
    const int rc = with_dst_type(e, L, [&](auto* dst) {
      CK(e, launch_dequant_ct_nvfp4_place((const uint8_t*)dp, (const uint8_t*)ds, global, dst, n, (int)in, r0, L.mode, L.row_offset, L.dst_stride,
                                          e->stream), "nvfp4 checkpoint dequantisation");
      return (int)DCD_OK;
    });
    if (rc) return rc;
    CK(e, st.release(sp), "checkpoint staging");
    CK(e, st.release(ss), "checkpoint staging");
  }
  return DCD_OK;
}

// WeightProvider::linear (weights.rs:283-499): the stored format of a module is detected by the tensors it has.
int load_linear(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& module, const Loc& L) {
  if (s.contains(module + ".weight_global_scale")) return place_ct_nvfp4(e, st, s, module, L);
  if (s.contains(module + ".weight_packed")) return place_ct_w4(e, st, s, module, L);
  const std::string wname = module + ".weight";
  const ckpt::Tensor* t = s.info(wname);
  if (!t) return fail(e, DCD_E_INVALID, "linear %s not found", wname.c_str());
  if (t->shape.size() != 2) return fail(e, DCD_E_INVALID, "%s: expected 2-D weight", wname.c_str());
  if (t->shape[0] != L.rows || t->shape[1] != L.cols)
    return fail(e, DCD_E_INVALID, "%s: checkpoint shape %zu x %zu, the engine expects %zu x %zu", wname.c_str(), t->shape[0], t->shape[1], L.rows, L.cols);
  return place_plain(e, st, wname.c_str(), s.data(*t), t->dtype, t->count(), L);
}

struct Member { int kind; const char* module; };

// A compressed-tensors int4 module whose codes a W4 engine can keep as they are: group 128 over the whole input width.
// (Zero points and the fp16 exactness of the scales are checked on the device while the rows are copied.)
bool w4_adoptable(const ckpt::Store& s, const std::string& module, const Loc& L) {
  if (s.contains(module + ".weight_global_scale") || !s.contains(module + ".weight_packed")) return false;
  const ckpt::Tensor *tp = s.info(module + ".weight_packed"), *tsc = s.info(module + ".weight_scale"), *tz = s.info(module + ".weight_zero_point");
  if (!tp || !tsc || (L.cols % 128) != 0 || tsc->shape.empty()) return false;
  const size_t groups = L.cols / 128, words = L.cols / 8;
  if (tsc->shape.back() != groups || tsc->dtype != ckpt::BF16 || tsc->count() != L.rows * groups) return false;
  if (tp->dtype != ckpt::I32 || tp->count() != L.rows * words) return false;
  if (tz && (tz->dtype != ckpt::I32 || tz->count() != ((L.rows + 7) / 8) * groups)) return false;
  return true;
}

// Copies the module's words and scales into the engine image (rows mapped like every other loader maps them).
int adopt_ct_w4(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& module, const Loc& L, int* d_flag) {
  const ckpt::Tensor *tp = s.info(module + ".weight_packed"), *tsc = s.info(module + ".weight_scale"), *tz = s.info(module + ".weight_zero_point");
  const size_t groups = L.cols / 128, words = L.cols / 8, out = L.rows;
  const uint8_t *pp = s.data(*tp), *ps = s.data(*tsc), *pz = tz ? s.data(*tz) : nullptr;
  const size_t chunk_rows = std::max<size_t>(8, (st.cap / (words * 4)) & ~(size_t)7);
  if (8 * words * 4 > st.cap) return fail(e, DCD_E_INVALID, "%s: eight rows exceed the staging buffer", module.c_str());
  for (size_t r0 = 0; r0 < out; r0 += chunk_rows) {
    const size_t n = std::min(chunk_rows, out - r0);
    void *dp, *ds, *dz = nullptr;
    int sp, ss, sz = -1;
    CK(e, st.push(pp + r0 * words * 4, n * words * 4, &dp, &sp), "checkpoint upload");
    CK(e, st.push(ps + r0 * groups * 2, n * groups * 2, &ds, &ss), "checkpoint upload");
    if (pz) CK(e, st.push(pz + (r0 / 8) * groups * 4, ((n + 7) / 8) * groups * 4, &dz, &sz), "checkpoint upload");
    e->launches += 1;
    CK(e, launch_adopt_ct_w4_rows((const int32_t*)dp, (const bf16*)ds, (const int32_t*)dz, L.w4->q, L.w4->scale, n, (int)L.cols, r0, L.mode, L.row_offset,
                                  d_flag, e->stream), "int4 checkpoint adoption");
    CK(e, st.release(sp), "checkpoint staging");
    CK(e, st.release(ss), "checkpoint staging");
    if (sz >= 0) CK(e, st.release(sz), "checkpoint staging");
  }
  return DCD_OK;
}

// One fused engine matrix = one or more checkpoint modules.
int load_group(dcd_engine* e, Stager& st, const ckpt::Store& s, const std::string& layer_prefix, int layer, const Member* m, int count) {
  Loc L;
  // A W4 engine serves the checkpoint's own int4 codes and scales where it can (every member of the fused matrix symmetric, group
  // 128, scales exact in fp16): nothing is re-quantised, so the served weights are the reference's dequant_w4a16_bf16 values bit
  // for bit. Anything else (bf16 members, group 64, zero points, a mix) goes through the bf16 stage and is quantised again.
  if (e->w4) {
    bool all = true;
    for (int i = 0; i < count && all; ++i) all = locate(e, layer, m[i].kind, &L) && L.w4 && w4_adoptable(s, layer_prefix + m[i].module, L);
    if (all) {
      int* d_flag = e->d_err + 8;
      const size_t words = (size_t)L.w4->N * (L.w4->K / 8), nsc = (size_t)L.w4->N * (L.w4->K / 128);
      CK(e, cudaMemsetAsync(d_flag, 0, sizeof(int), e->stream), "adoption flag");
      CK(e, cudaMemsetAsync(L.w4->q, 0x88, words * 4, e->stream), "int4 image clear");   // padding rows: code 8 = 0
      CK(e, cudaMemsetAsync(L.w4->scale, 0, nsc * 2, e->stream), "int4 scale clear");
      for (int i = 0; i < count; ++i) {
        locate(e, layer, m[i].kind, &L);
        if (int rc = adopt_ct_w4(e, st, s, layer_prefix + m[i].module, L, d_flag)) return rc;
      }
      int flag = 0;
      CK(e, cudaMemcpyAsync(&flag, d_flag, sizeof(int), cudaMemcpyDeviceToHost, e->stream), "adoption flag");
      CK(e, cudaStreamSynchronize(e->stream), "adoption sync");
      if (flag == 0) {
        if (L.w4->scale_t) {
          e->launches += 1;
          CK(e, launch_w4_scale_transpose(L.w4->scale, L.w4->scale_t, L.w4->N, L.w4->K / 128, e->stream), "w4 scale transpose");
        }
        return DCD_OK;
      }
    }
  }
  for (int i = 0; i < count; ++i) {
    if (!locate(e, layer, m[i].kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", m[i].kind, layer);
    if ((L.w4 || L.nv) && i == 0) {
      const size_t n = L.w4 ? (size_t)L.w4->N * L.w4->K : (size_t)L.nv->N * L.nv->K;
      CK(e, cudaMemsetAsync(e->wstage, 0, n * 2, e->stream), "stage clear");
    }
    if (int rc = load_linear(e, st, s, layer_prefix + m[i].module, L)) return rc;
  }
  return w4_stage_out(e, L);
}

int load_checkpoint_impl(dcd_engine* e, Stager& st, const ckpt::Store& s, const char* readout_path) {
  static const char* prefixes[] = {"model.language_model.", "language_model.", "model.", ""};
  const char* prefix = nullptr;
  for (const char* p : prefixes) if (s.contains(std::string(p) + "embed_tokens.weight")) { prefix = p; break; }
  if (!prefix) return fail(e, DCD_E_INVALID, "could not locate embed_tokens.weight in checkpoint");
  const std::string P = prefix;
  int rc;
  {
    const ckpt::Tensor* t;
    if ((rc = need(e, s, P + "embed_tokens.weight", &t))) return rc;
    if (t->shape.size() != 2 || t->shape[0] != (size_t)e->c.vocab || t->shape[1] != e->H)
      return fail(e, DCD_E_INVALID, "embed_tokens.weight: expected [%d, %zu]", e->c.vocab, e->H);
    if ((rc = load_vector(e, st, s, P + "embed_tokens.weight", -1, DCD_T_EMBED))) return rc;
  }
  if ((rc = load_vector(e, st, s, P + "norm.weight", -1, DCD_T_FINAL_NORM))) return rc;
  static const Member gate_up[] = {{DCD_T_GATE, "mlp.gate_proj"}, {DCD_T_UP, "mlp.up_proj"}};
  static const Member down[] = {{DCD_T_DOWN, "mlp.down_proj"}};
  static const Member qkv[] = {{DCD_T_Q, "self_attn.q_proj"}, {DCD_T_K, "self_attn.k_proj"}, {DCD_T_V, "self_attn.v_proj"}};
  static const Member o[] = {{DCD_T_O, "self_attn.o_proj"}};
  static const Member gin[] = {{DCD_T_IN_QKV, "linear_attn.in_proj_qkv"}, {DCD_T_IN_Z, "linear_attn.in_proj_z"}, {DCD_T_IN_B, "linear_attn.in_proj_b"},
                               {DCD_T_IN_A, "linear_attn.in_proj_a"}};
  static const Member gout[] = {{DCD_T_OUT, "linear_attn.out_proj"}};
  for (int i = 0; i < e->c.num_layers; ++i) {
    const std::string l = P + "layers." + std::to_string(i) + ".";
    if ((rc = load_vector(e, st, s, l + "input_layernorm.weight", i, DCD_T_INPUT_NORM))) return rc;
    if ((rc = load_vector(e, st, s, l + "post_attention_layernorm.weight", i, DCD_T_POST_NORM))) return rc;
    if ((rc = load_group(e, st, s, l, i, gate_up, 2))) return rc;
    if ((rc = load_group(e, st, s, l, i, down, 1))) return rc;
    if (e->layers[i].full) {
      if ((rc = load_group(e, st, s, l, i, qkv, 3))) return rc;
      if ((rc = load_group(e, st, s, l, i, o, 1))) return rc;
      if ((rc = load_vector(e, st, s, l + "self_attn.q_norm.weight", i, DCD_T_QNORM))) return rc;
      if ((rc = load_vector(e, st, s, l + "self_attn.k_norm.weight", i, DCD_T_KNORM))) return rc;
    } else {
      if ((rc = load_group(e, st, s, l, i, gin, 4))) return rc;
      if ((rc = load_group(e, st, s, l, i, gout, 1))) return rc;
      if ((rc = load_vector(e, st, s, l + "linear_attn.conv1d.weight", i, DCD_T_CONV))) return rc;
      if ((rc = load_vector(e, st, s, l + "linear_attn.A_log", i, DCD_T_A_LOG))) return rc;
      if ((rc = load_vector(e, st, s, l + "linear_attn.dt_bias", i, DCD_T_DT_BIAS))) return rc;
      if ((rc = load_vector(e, st, s, l + "linear_attn.norm.weight", i, DCD_T_GNORM))) return rc;
    }
  }
  if (readout_path) {
    ckpt::Store head;
    std::string err;
    if (!head.open(readout_path, &err)) return fail(e, DCD_E_INVALID, "%s", err.c_str());
    const ckpt::Tensor* w = head.info("weight");
    if (!w) return fail(e, DCD_E_INVALID, "readout.weight not found in %s", readout_path);
    if (w->shape.size() != 2) return fail(e, DCD_E_INVALID, "readout.weight must be 2-D");
    if (w->dtype != ckpt::F32 && w->dtype != ckpt::BF16) return fail(e, DCD_E_INVALID, "readout.weight dtype unsupported");
    if (w->shape[0] != (size_t)e->c.readout_rows || w->shape[1] != e->H)
      return fail(e, DCD_E_INVALID, "readout.weight is %zu x %zu, the engine expects %d x %zu", w->shape[0], w->shape[1], e->c.readout_rows, e->H);
    Loc L;
    if (!locate(e, -1, DCD_T_READOUT, &L)) return fail(e, DCD_E_INVALID, "no readout tensor");
    if ((rc = place_plain(e, st, "readout.weight", head.data(*w), w->dtype, w->count(), L))) return rc;
    // the mapping of `head` ends with this scope: finish the copies out of it first
    CK(e, cudaStreamSynchronize(e->stream), "readout upload");
  }
  return DCD_OK;
}

}  // namespace

extern "C" {

int dcd_checkpoint_open(const char* path, dcd_checkpoint** out) {
  if (!out) return DCD_E_INVALID;
  *out = nullptr;
  if (!path) return fail(nullptr, DCD_E_INVALID, "null checkpoint path");
  dcd_checkpoint* ck = new dcd_checkpoint();
  std::string err;
  if (!ck->store.open(path, &err)) {
    delete ck;
    return fail(nullptr, DCD_E_INVALID, "%s", err.c_str());
  }
  *out = ck;
  return DCD_OK;
}
void dcd_checkpoint_close(dcd_checkpoint* ck) { delete ck; }
size_t dcd_checkpoint_count(const dcd_checkpoint* ck) { return ck ? ck->store.size() : 0; }
const char* dcd_checkpoint_name(const dcd_checkpoint* ck, size_t i) { return ck && i < ck->store.size() ? ck->store.name_at(i).c_str() : nullptr; }
int dcd_checkpoint_tensor(const dcd_checkpoint* ck, const char* name, dcd_tensor_info* out) {
  if (!ck || !name || !out) return DCD_E_INVALID;
  const ckpt::Tensor* t = ck->store.info(name);
  if (!t) return fail(nullptr, DCD_E_INVALID, "tensor %s not found", name);
  memset(out, 0, sizeof *out);
  if (t->shape.size() > 8) return fail(nullptr, DCD_E_UNSUPPORTED, "tensor %s has more than 8 dimensions", name);
  out->dtype = t->dtype;
  out->rank = (int32_t)t->shape.size();
  for (size_t i = 0; i < t->shape.size(); ++i) out->shape[i] = t->shape[i];
  out->bytes = t->end - t->start;
  out->data = ck->store.data(*t);
  return DCD_OK;
}
int dcd_config_from_dir(const char* dir, dcd_model_config* out) {
  if (!dir || !out) return DCD_E_INVALID;
  std::string err;
  if (!ckpt::config_from_dir(dir, out, &err)) return fail(nullptr, DCD_E_INVALID, "%s", err.c_str());
  return DCD_OK;
}

int dcd_engine_load_checkpoint(dcd_engine* e, const dcd_checkpoint* ck, const char* readout_path) {
  if (!e || !ck) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  Stager st;
  cudaError_t ce = st.init(STAGE_CHUNK, e->stream);
  st.store = &ck->store;
  int rc = ce == cudaSuccess ? load_checkpoint_impl(e, st, ck->store, readout_path) : cuda_fail(e, ce, "checkpoint staging buffers");
  const cudaError_t se = cudaStreamSynchronize(e->stream);
  st.destroy();
  if (rc == DCD_OK && se != cudaSuccess) rc = cuda_fail(e, se, "load_checkpoint");
  if (rc == DCD_OK) { e->weights_ready = true; e->fp8_dirty = true; }
  return rc;
}

int dcd_engine_load_tensor_typed(dcd_engine* e, int layer, int kind, const void* host, int dtype, size_t count) {
  if (!e || !host) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  Loc L;
  if (!locate(e, layer, kind, &L)) return fail(e, DCD_E_INVALID, "no tensor kind %d in layer %d", kind, layer);
  if (int rc0 = w4_stage_in(e, L)) return rc0;
  Stager st;
  cudaError_t ce = st.init(STAGE_CHUNK, e->stream);
  int rc = ce == cudaSuccess ? place_plain(e, st, "tensor", (const uint8_t*)host, dtype, count, L) : cuda_fail(e, ce, "tensor staging buffers");
  if (rc == DCD_OK) rc = w4_stage_out(e, L);
  const cudaError_t se = cudaStreamSynchronize(e->stream);
  st.destroy();
  if (rc == DCD_OK && se != cudaSuccess) rc = cuda_fail(e, se, "load_tensor_typed");
  if (rc == DCD_OK) { e->weights_ready = true; e->fp8_dirty = true; }
  return rc;
}

// ---- hot path ---------------------------------------------------------------------

int dcd_capture_state_device(dcd_engine* e, const uint32_t* d_ids, size_t n, dcd_state** out) {
  if (!e || !out) return DCD_E_INVALID;
  *out = nullptr;
  cudaSetDevice(e->device);
  if (!e->weights_ready) return fail(e, DCD_E_INVALID, "weights are not loaded");
  if (n < 2) return fail(e, DCD_E_INVALID, "a state block needs at least two tokens, got %zu", n);
  if (n > (size_t)e->Tm) return fail(e, DCD_E_INVALID, "state of %zu tokens exceeds max_pass_tokens %d", n, e->Tm);
  if (n > (size_t)e->o.max_positions) return fail(e, DCD_E_INVALID, "state of %zu tokens exceeds the RoPE table", n);
  dcd_state* st = nullptr;
  int rc = new_state(e, n, &st);
  if (rc) return rc;
  const int32_t len = (int32_t)n;
  cudaError_t ce = cudaMemcpyAsync(e->d_lens, &len, 4, cudaMemcpyHostToDevice, e->stream);  // 4-byte pageable copy: staged by the driver
  if (ce != cudaSuccess) { dcd_state_free(e, st); return cuda_fail(e, ce, "lens upload"); }
  Pass p{0, (int)n, 1, (int)n};
  p.cap = st;
  rc = run_pass_any(e, p, d_ids, e->d_lens, 0, nullptr);
  if (rc) { dcd_state_free(e, st); return rc; }
  *out = st;
  return DCD_OK;
}

int dcd_capture_state(dcd_engine* e, const uint32_t* ids, size_t n, const uint32_t (*pos)[3], dcd_state** out) {
  if (!e || !out) return DCD_E_INVALID;
  *out = nullptr;
  if (!ids) return fail(e, DCD_E_INVALID, "null ids");
  cudaSetDevice(e->device);
  if (n < 2) return fail(e, DCD_E_INVALID, "a state block needs at least two tokens, got %zu", n);
  if (n > (size_t)e->Tm) return fail(e, DCD_E_INVALID, "state of %zu tokens exceeds max_pass_tokens %d", n, e->Tm);
  if (pos) {
    // text-only: every triple must be (t,t,t); anything else belongs to the image path
    for (size_t t = 0; t < n; ++t)
      if (pos[t][0] != t || pos[t][1] != t || pos[t][2] != t)
        return fail(e, DCD_E_UNSUPPORTED, "mRoPE positions other than (t,t,t) need the vision path, which is not built");
  }
  memcpy(e->h_ids, ids, n * 4);
  CK(e, cudaMemcpyAsync(e->d_ids, e->h_ids, n * 4, cudaMemcpyHostToDevice, e->stream), "ids upload");
  dcd_state* st = nullptr;
  int rc = dcd_capture_state_device(e, e->d_ids, n, &st);
  if (rc) return rc;
  rc = sync_and_check(e);
  if (rc) { dcd_state_free(e, st); return rc; }
  *out = st;
  return DCD_OK;
}

int dcd_readout_state_once_device(dcd_engine* e, const dcd_state* st, const uint32_t* d_ids, const int32_t* d_lens, size_t B,
                                  size_t total, size_t max_len, float* d_out) {
  if (!e || !st || !d_ids || !d_lens || !d_out) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  if (!e->weights_ready) return fail(e, DCD_E_INVALID, "weights are not loaded");
  if (B == 0) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  if (total > (size_t)e->Tm || B > (size_t)e->max_batch) return fail(e, DCD_E_INVALID, "pass of %zu tokens exceeds max_pass_tokens %d", total, e->Tm);
  if (st->pos_end + max_len > (size_t)e->o.max_positions) return fail(e, DCD_E_INVALID, "positions exceed the RoPE table");
  Pass p{1, (int)total, (int)B, (int)max_len};
  p.cache = st;
  return run_pass_any(e, p, d_ids, d_lens, (int)st->pos_end, d_out);
}

// One chunk through the host-buffer path: ids/lens already in pinned staging.
static int run_chunk_host(dcd_engine* e, const dcd_state* st, size_t B, size_t total, size_t max_len) {
  CK(e, cudaMemcpyAsync(e->d_ids, e->h_ids, total * 4, cudaMemcpyHostToDevice, e->stream), "ids upload");
  CK(e, cudaMemcpyAsync(e->d_lens, e->h_lens, B * 4, cudaMemcpyHostToDevice, e->stream), "lens upload");
  int rc = dcd_readout_state_once_device(e, st, e->d_ids, e->d_lens, B, total, max_len, e->d_logits);
  if (rc) return rc;
  CK(e, cudaMemcpyAsync(e->h_logits, e->d_logits, B * e->c.readout_rows * 4, cudaMemcpyDeviceToHost, e->stream), "logits download");
  return sync_and_check(e);
}

int dcd_readout_state_once_batch(dcd_engine* e, const dcd_state* st, const uint32_t* const* questions, const size_t* lens, size_t B,
                                 float* out) {
  if (!e) return DCD_E_INVALID;
  if (!st || !out) return fail(e, DCD_E_INVALID, "null argument");
  if (B == 0 || !questions || !lens) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  for (size_t i = 0; i < B; ++i)
    if (lens[i] == 0 || !questions[i]) return fail(e, DCD_E_INVALID, "batch item %zu has no tokens", i);
  cudaSetDevice(e->device);
  std::vector<int32_t> order(B), chunk_of(B);
  int32_t n_chunks = 0;
  int rc = plan_chunks_host(lens, B, st->state_len, (size_t)e->o.max_rows, (size_t)e->o.max_keys, (size_t)e->o.max_scores,
                            (size_t)e->Tm, order.data(), chunk_of.data(), &n_chunks);
  if (rc == -5) return fail(e, DCD_E_INVALID, "one question exceeds the key/score/token caps of a pass");
  if (rc) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  const int R = e->c.readout_rows;
  if (n_chunks <= 1) {
    size_t total = 0, mx = 0;
    for (size_t i = 0; i < B; ++i) {
      memcpy(e->h_ids + total, questions[i], lens[i] * 4);
      e->h_lens[i] = (int32_t)lens[i];
      total += lens[i];
      if (lens[i] > mx) mx = lens[i];
    }
    rc = run_chunk_host(e, st, B, total, mx);
    if (rc) return rc;
    memcpy(out, e->h_logits, B * R * sizeof(float));
    return DCD_OK;
  }
  // several chunks: questions of a chunk run in sorted order; rows go back to input order
  size_t n = 0;
  for (int ch = 0; ch < n_chunks; ++ch) {
    size_t first = n, total = 0, mx = 0, nb = 0;
    while (n < B && chunk_of[order[n]] == ch) {
      const size_t i = order[n];
      memcpy(e->h_ids + total, questions[i], lens[i] * 4);
      e->h_lens[nb++] = (int32_t)lens[i];
      total += lens[i];
      if (lens[i] > mx) mx = lens[i];
      ++n;
    }
    rc = run_chunk_host(e, st, nb, total, mx);
    if (rc) return rc;
    for (size_t j = 0; j < nb; ++j) memcpy(out + (size_t)order[first + j] * R, e->h_logits + j * R, R * sizeof(float));
  }
  return DCD_OK;
}

int dcd_readout_state_once_flat(dcd_engine* e, const dcd_state* st, const uint32_t* flat_ids, const uint32_t* lens, size_t B, float* out) {
  if (!e) return DCD_E_INVALID;
  if (B == 0 || !flat_ids || !lens) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  std::vector<const uint32_t*> ptrs(B);
  std::vector<size_t> ls(B);
  size_t off = 0;
  for (size_t i = 0; i < B; ++i) {
    ptrs[i] = flat_ids + off;
    ls[i] = lens[i];
    off += lens[i];
  }
  return dcd_readout_state_once_batch(e, st, ptrs.data(), ls.data(), B, out);
}

// One question pass over questions that fork DIFFERENT states. Questions are reordered so that those of one state are
// consecutive (stable, states in index order); rows come back in input order.
int dcd_readout_multi_state_batch(dcd_engine* e, const dcd_state* const* states, size_t n_states, const uint32_t* const* questions,
                                  const size_t* lens, const uint32_t* state_of, size_t B, float* out) {
  if (!e) return DCD_E_INVALID;
  if (!states || n_states == 0 || !out) return fail(e, DCD_E_INVALID, "null argument");
  if (B == 0 || !questions || !lens || !state_of) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  cudaSetDevice(e->device);
  if (!e->weights_ready) return fail(e, DCD_E_INVALID, "weights are not loaded");
  size_t total = 0, mx = 0;
  for (size_t i = 0; i < B; ++i) {
    if (lens[i] == 0 || !questions[i]) return fail(e, DCD_E_INVALID, "batch item %zu has no tokens", i);
    if (state_of[i] >= n_states || !states[state_of[i]]) return fail(e, DCD_E_INVALID, "batch item %zu names state %u of %zu", i, state_of[i], n_states);
    total += lens[i];
    if (lens[i] > mx) mx = lens[i];
  }
  if (mx > (size_t)e->Tm) return fail(e, DCD_E_INVALID, "a question of %zu tokens exceeds max_pass_tokens %d", mx, e->Tm);
  std::vector<int32_t> order(B);
  for (size_t i = 0; i < B; ++i) order[i] = (int32_t)i;
  std::stable_sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return state_of[a] < state_of[b]; });
  const int R = e->c.readout_rows;
  // as many passes as the workspace needs: each takes the next run of (sorted) questions that fits max_pass_tokens
  for (size_t n0 = 0; n0 < B;) {
    std::vector<Group> groups;
    size_t tok = 0, n = n0, pass_max = 0;
    for (; n < B; ++n) {
      const size_t i = (size_t)order[n];
      if (n > n0 && (tok + lens[i] > (size_t)e->Tm || n - n0 >= (size_t)e->max_batch)) break;
      const dcd_state* st = states[state_of[i]];
      if (st->pos_end + lens[i] > (size_t)e->o.max_positions) return fail(e, DCD_E_INVALID, "positions exceed the RoPE table");
      if (groups.empty() || state_of[i] != state_of[(size_t)order[n - 1]]) groups.push_back(Group{st, (int)(n - n0), 0, (int)tok, 0, 0});
      Group& g = groups.back();
      g.nq += 1;
      g.ntok += (int)lens[i];
      if ((int)lens[i] > g.max_len) g.max_len = (int)lens[i];
      if (lens[i] > pass_max) pass_max = lens[i];
      memcpy(e->h_ids + tok, questions[i], lens[i] * 4);
      e->h_lens[n - n0] = (int32_t)lens[i];
      e->h_posq[n - n0] = (int32_t)st->pos_end;
      tok += lens[i];
    }
    const size_t nb = n - n0;
    CK(e, cudaMemcpyAsync(e->d_ids, e->h_ids, tok * 4, cudaMemcpyHostToDevice, e->stream), "ids upload");
    CK(e, cudaMemcpyAsync(e->d_lens, e->h_lens, nb * 4, cudaMemcpyHostToDevice, e->stream), "lens upload");
    CK(e, cudaMemcpyAsync(e->d_posq, e->h_posq, nb * 4, cudaMemcpyHostToDevice, e->stream), "positions upload");
    Pass p{1, (int)tok, (int)nb, (int)pass_max};
    p.cache = groups[0].st;
    p.groups = groups.data();
    p.n_groups = (int)groups.size();
    p.d_posq = e->d_posq;
    int rc = run_pass_any(e, p, e->d_ids, e->d_lens, 0, e->d_logits);
    if (rc) return rc;
    CK(e, cudaMemcpyAsync(e->h_logits, e->d_logits, nb * R * 4, cudaMemcpyDeviceToHost, e->stream), "logits download");
    rc = sync_and_check(e);
    if (rc) return rc;
    for (size_t j = 0; j < nb; ++j) memcpy(out + (size_t)order[n0 + j] * R, e->h_logits + j * R, (size_t)R * sizeof(float));
    n0 = n;
  }
  return DCD_OK;
}

// ---- cold request in one pass ---------------------------------------------------------------------------------------------
// Capture of a state and the question pass over it as ONE sweep over the layers: rows [0, n_state) are the state (a sequence
// that attends to itself and whose K/V, conv tail and recurrent state are kept), the rest the questions, which read in every
// layer what the state's kernels of that layer have just written. Every row goes through the same kernels as in the two-pass
// order (capture, then readout), so the cache and the logits are bit-identical to it; the weights stream once per layer instead of
// twice and the projections see 25-30 % more rows per launch. The reference has no such call: it captures, then runs the
// question pass (src/batch.rs:752-905).
static bool cold_pass_fits(const dcd_engine* e, size_t n_state, size_t B, size_t total_q, size_t max_len) {
  return !e->fp8 /* the capture half of an FP8 engine stays bf16, the question half does not */ && n_state >= 2 &&
         n_state + total_q <= (size_t)e->Tm && B + 1 <= (size_t)e->max_batch && n_state + max_len <= (size_t)e->o.max_positions;
}

int dcd_capture_and_readout_device(dcd_engine* e, const uint32_t* d_ids, const int32_t* d_lens, size_t n_state, size_t B, size_t total,
                                   size_t max_len, dcd_state** out_state, float* d_out) {
  if (!e || !out_state) return DCD_E_INVALID;
  *out_state = nullptr;
  if (!d_ids || !d_lens || !d_out) return fail(e, DCD_E_INVALID, "null argument");
  cudaSetDevice(e->device);
  if (!e->weights_ready) return fail(e, DCD_E_INVALID, "weights are not loaded");
  if (B == 0) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  if (total <= n_state || !cold_pass_fits(e, n_state, B, total - n_state, max_len))
    return fail(e, DCD_E_INVALID, "a cold request of %zu + %zu tokens does not fit one pass of this engine (max_pass_tokens %d)", n_state, total - n_state, e->Tm);
  dcd_state* st = nullptr;
  int rc = new_state(e, n_state, &st);
  if (rc) return rc;
  e->h_posq[0] = 0;
  for (size_t i = 1; i <= B; ++i) e->h_posq[i] = (int32_t)n_state;
  cudaError_t ce = cudaMemcpyAsync(e->d_posq, e->h_posq, (B + 1) * 4, cudaMemcpyHostToDevice, e->stream);
  if (ce != cudaSuccess) { dcd_state_free(e, st); return cuda_fail(e, ce, "positions upload"); }
  Group groups[2] = {Group{nullptr, 0, 1, 0, (int)n_state, (int)n_state, st},
                     Group{st, 1, (int)B, (int)n_state, (int)(total - n_state), (int)max_len, nullptr}};
  Pass p{1, (int)total, (int)B + 1, (int)(n_state > max_len ? n_state : max_len)};
  p.cache = nullptr;
  p.groups = groups;
  p.n_groups = 2;
  p.d_posq = e->d_posq;
  rc = run_pass_any(e, p, d_ids, d_lens, 0, d_out);
  if (rc) { dcd_state_free(e, st); return rc; }
  *out_state = st;
  return DCD_OK;
}

int dcd_capture_and_readout(dcd_engine* e, const uint32_t* state_ids, size_t n_state, const uint32_t* const* questions, const size_t* lens,
                            size_t B, dcd_state** out_state, float* out) {
  if (!e || !out_state) return DCD_E_INVALID;
  *out_state = nullptr;
  if (!state_ids || !out) return fail(e, DCD_E_INVALID, "null argument");
  if (B == 0 || !questions || !lens) return fail(e, DCD_E_INVALID, "empty state-once question batch");
  size_t total_q = 0, mx = 0;
  for (size_t i = 0; i < B; ++i) {
    if (lens[i] == 0 || !questions[i]) return fail(e, DCD_E_INVALID, "batch item %zu has no tokens", i);
    total_q += lens[i];
    if (lens[i] > mx) mx = lens[i];
  }
  cudaSetDevice(e->device);
  // one pass only where the reference's planner would also take the questions in one chunk; otherwise the two-pass order
  bool one = cold_pass_fits(e, n_state, B, total_q, mx);
  if (one) {
    std::vector<int32_t> order(B), chunk_of(B);
    int32_t n_chunks = 0;
    const int prc = plan_chunks_host(lens, B, n_state, (size_t)e->o.max_rows, (size_t)e->o.max_keys, (size_t)e->o.max_scores, (size_t)e->Tm, order.data(),
                                     chunk_of.data(), &n_chunks);
    one = prc == 0 && n_chunks <= 1;
  }
  if (!one) {
    dcd_state* st = nullptr;
    int rc = dcd_capture_state(e, state_ids, n_state, nullptr, &st);
    if (rc) return rc;
    rc = dcd_readout_state_once_batch(e, st, questions, lens, B, out);
    if (rc) { dcd_state_free(e, st); return rc; }
    *out_state = st;
    return DCD_OK;
  }
  memcpy(e->h_ids, state_ids, n_state * 4);
  e->h_lens[0] = (int32_t)n_state;
  size_t total = n_state;
  for (size_t i = 0; i < B; ++i) {
    memcpy(e->h_ids + total, questions[i], lens[i] * 4);
    e->h_lens[i + 1] = (int32_t)lens[i];
    total += lens[i];
  }
  CK(e, cudaMemcpyAsync(e->d_ids, e->h_ids, total * 4, cudaMemcpyHostToDevice, e->stream), "ids upload");
  CK(e, cudaMemcpyAsync(e->d_lens, e->h_lens, (B + 1) * 4, cudaMemcpyHostToDevice, e->stream), "lens upload");
  dcd_state* st = nullptr;
  int rc = dcd_capture_and_readout_device(e, e->d_ids, e->d_lens, n_state, B, total, mx, &st, e->d_logits);
  if (rc) return rc;
  const int R = e->c.readout_rows;
  cudaError_t ce = cudaMemcpyAsync(e->h_logits, e->d_logits + R, B * R * 4, cudaMemcpyDeviceToHost, e->stream);  // row 0 is the state's own last token
  if (ce != cudaSuccess) { dcd_state_free(e, st); return cuda_fail(e, ce, "logits download"); }
  rc = sync_and_check(e);
  if (rc) { dcd_state_free(e, st); return rc; }
  memcpy(out, e->h_logits, B * R * sizeof(float));
  *out_state = st;
  return DCD_OK;
}

int dcd_decision_logits_split(dcd_engine* e, const uint32_t* ids, size_t seq, size_t split, float* out) {
  if (!e) return DCD_E_INVALID;
  if (!ids || !out) return fail(e, DCD_E_INVALID, "null argument");
  cudaSetDevice(e->device);
  if (!e->weights_ready) return fail(e, DCD_E_INVALID, "weights are not loaded");
  if (split == 0 || split >= seq) return fail(e, DCD_E_INVALID, "block split %zu out of range for %zu tokens", split, seq);
  if (seq > (size_t)e->Tm || seq > (size_t)e->o.max_positions) return fail(e, DCD_E_INVALID, "sequence of %zu tokens exceeds max_pass_tokens %d", seq, e->Tm);
  memcpy(e->h_ids, ids, seq * 4);
  e->h_lens[0] = (int32_t)seq;
  CK(e, cudaMemcpyAsync(e->d_ids, e->h_ids, seq * 4, cudaMemcpyHostToDevice, e->stream), "ids upload");
  CK(e, cudaMemcpyAsync(e->d_lens, e->h_lens, 4, cudaMemcpyHostToDevice, e->stream), "lens upload");
  Pass p{2, (int)seq, 1, (int)seq};
  p.split = (int)split;
  int rc = run_pass_any(e, p, e->d_ids, e->d_lens, 0, e->d_logits);
  if (rc) return rc;
  CK(e, cudaMemcpyAsync(e->h_logits, e->d_logits, (size_t)e->c.readout_rows * 4, cudaMemcpyDeviceToHost, e->stream), "logits download");
  rc = sync_and_check(e);
  if (rc) return rc;
  memcpy(out, e->h_logits, (size_t)e->c.readout_rows * 4);
  return DCD_OK;
}

// ---- StateCache ---------------------------------------------------------------------
void dcd_state_free(dcd_engine* e, dcd_state* st) {
  if (!st) return;
  if (st->block && e) {
    cudaSetDevice(e->device);
    cudaFreeAsync(st->block, e->stream);
  }
  delete st;
}
size_t dcd_state_tokens(const dcd_state* st) { return st ? st->state_len : 0; }
size_t dcd_state_pos_end(const dcd_state* st) { return st ? st->pos_end : 0; }
size_t dcd_state_bytes(const dcd_state* st) { return st ? st->bytes : 0; }
size_t dcd_state_bytes_for(const dcd_engine* e, size_t state_len) { return e ? state_bytes_for(e, state_len) : 0; }
// Every working buffer of a pass is sized at engine creation (max_pass_tokens); a pass allocates nothing beyond the state
// itself, so what has to stay free besides a state is the stream-ordered pool's granularity and the CUDA context's own needs.
size_t dcd_pass_reserve_bytes(const dcd_engine* e, size_t state_len) {
  (void)state_len;
  return e ? (size_t)256 << 20 : 0;
}

int dcd_state_offload(dcd_engine* e, const dcd_state* st, dcd_host_state** out) {
  if (!e || !st || !out) return DCD_E_INVALID;
  *out = nullptr;
  cudaSetDevice(e->device);
  dcd_host_state* hs = new dcd_host_state();
  hs->state_len = st->state_len;
  hs->pos_end = st->pos_end;
  hs->bytes = st->bytes;
  cudaError_t ce = cudaMallocHost(&hs->block, st->bytes);
  if (ce != cudaSuccess) {
    delete hs;
    cudaGetLastError();
    return fail(e, DCD_E_OOM, "host state cache: out of memory (%zu bytes pinned)", st->bytes);
  }
  ce = cudaMemcpyAsync(hs->block, st->block, st->bytes, cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) { dcd_host_state_free(hs); return cuda_fail(e, ce, "state offload"); }
  *out = hs;
  return DCD_OK;
}

int dcd_state_restore(dcd_engine* e, const dcd_host_state* hs, dcd_state** out) {
  if (!e || !hs || !out) return DCD_E_INVALID;
  *out = nullptr;
  cudaSetDevice(e->device);
  if (hs->bytes != state_bytes_for(e, hs->state_len)) return fail(e, DCD_E_INVALID, "host state does not match this engine's model");
  dcd_state* st = nullptr;
  int rc = new_state(e, hs->state_len, &st);
  if (rc) return rc;
  st->pos_end = hs->pos_end;
  cudaError_t ce = cudaMemcpyAsync(st->block, hs->block, hs->bytes, cudaMemcpyHostToDevice, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  if (ce != cudaSuccess) { dcd_state_free(e, st); return cuda_fail(e, ce, "state restore"); }
  *out = st;
  return DCD_OK;
}

void dcd_host_state_free(dcd_host_state* hs) {
  if (!hs) return;
  if (hs->block) cudaFreeHost(hs->block);
  delete hs;
}

int dcd_state_zero_gdn_state(dcd_engine* e, dcd_state* st, int layer) {
  if (!e || !st || layer < 0 || layer >= e->c.num_layers || !st->gstate[layer]) return fail(e, DCD_E_INVALID, "layer %d has no GDN state", layer);
  cudaSetDevice(e->device);
  CK(e, cudaMemsetAsync(st->gstate[layer], 0, (size_t)e->c.gdn_v_heads * e->c.gdn_dk * e->c.gdn_dv * 4, e->stream), "zero state");
  CK(e, cudaStreamSynchronize(e->stream), "sync");
  return DCD_OK;
}
int dcd_state_zero_gdn_hist(dcd_engine* e, dcd_state* st, int layer) {
  if (!e || !st || layer < 0 || layer >= e->c.num_layers || !st->hist[layer]) return fail(e, DCD_E_INVALID, "layer %d has no conv tail", layer);
  cudaSetDevice(e->device);
  CK(e, cudaMemsetAsync(st->hist[layer], 0, (size_t)3 * e->conv_dim * e->esz, e->stream), "zero hist");
  CK(e, cudaStreamSynchronize(e->stream), "sync");
  return DCD_OK;
}

int dcd_state_read_tensor(dcd_engine* e, const dcd_state* st, int layer, int what, float* host, size_t* count) {
  if (!e || !st || !count || layer < 0 || layer >= e->c.num_layers) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  const dcd_model_config& c = e->c;
  const void* src = nullptr;
  size_t n = 0;
  bool f32 = false;
  if (what == 0 || what == 1) { src = what == 0 ? st->k[layer] : st->v[layer]; n = st->state_len * c.kv_heads * c.head_dim; }
  else if (what == 2) { src = st->gstate[layer]; n = (size_t)c.gdn_v_heads * c.gdn_dk * c.gdn_dv; f32 = true; }
  else if (what == 3) { src = st->hist[layer]; n = (size_t)3 * e->conv_dim; }
  if (!src) return fail(e, DCD_E_INVALID, "layer %d has no cached tensor %d", layer, what);
  *count = n;
  if (!host) return DCD_OK;
  float* tmp = nullptr;
  cudaError_t ce = cudaMalloc(&tmp, n * 4);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "state read staging");
  e->launches += 1;
  if (f32 || !e->bf) ce = cudaMemcpyAsync(tmp, src, n * 4, cudaMemcpyDeviceToDevice, e->stream);
  else ce = launch_to_f32<bf16>((const bf16*)src, tmp, n, e->stream);
  if (ce == cudaSuccess) ce = cudaMemcpyAsync(host, tmp, n * 4, cudaMemcpyDeviceToHost, e->stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize(e->stream);
  cudaFree(tmp);
  if (ce != cudaSuccess) return cuda_fail(e, ce, "state read");
  return DCD_OK;
}

// ---- pools, memory, timers ----------------------------------------------------------
int dcd_trim_pools(dcd_engine* e) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  cudaMemPool_t pool;
  CK(e, cudaStreamSynchronize(e->stream), "sync");
  CK(e, cudaDeviceGetDefaultMemPool(&pool, e->device), "mem pool");
  CK(e, cudaMemPoolTrimTo(pool, 0), "pool trim");
  return DCD_OK;
}
int dcd_mem_info(dcd_engine* e, size_t* free_bytes, size_t* total_bytes) {
  if (!e || !free_bytes || !total_bytes) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  CK(e, cudaMemGetInfo(free_bytes, total_bytes), "mem info");
  return DCD_OK;
}
int dcd_timer_begin(dcd_engine* e) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  CK(e, cudaEventRecord(e->t0, e->stream), "timer begin");
  return DCD_OK;
}
int dcd_timer_end(dcd_engine* e) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  CK(e, cudaEventRecord(e->t1, e->stream), "timer end");
  return DCD_OK;
}
double dcd_timer_seconds(dcd_engine* e) {
  if (!e) return -1.0;
  cudaSetDevice(e->device);
  float ms = 0.f;
  if (cudaEventSynchronize(e->t1) != cudaSuccess || cudaEventElapsedTime(&ms, e->t0, e->t1) != cudaSuccess) return -1.0;
  return (double)ms * 1e-3;
}
int dcd_vision_encode(dcd_engine* e, const void*, size_t) { return fail(e, DCD_E_UNSUPPORTED, "the vision tower is not part of this library"); }
int dcd_engine_sync(dcd_engine* e) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  return sync_and_check(e);
}

int dcd_profile_enable(dcd_engine* e, int on) {
  if (!e) return DCD_E_INVALID;
  e->prof.on = on != 0;
  return DCD_OK;
}
int dcd_profile_read(dcd_engine* e, dcd_prof_entry out[DCD_PROF_COUNT]) {
  if (!e || !out) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  CK(e, cudaStreamSynchronize(e->stream), "sync");
  for (auto& pr : e->prof.pairs) {
    float ms = 0.f;
    if (cudaEventElapsedTime(&ms, pr.a, pr.b) == cudaSuccess) {
      e->prof.acc[pr.kind].ms += ms;
      e->prof.acc[pr.kind].work += pr.work;
      e->prof.acc[pr.kind].launches += 1;
    }
    e->prof.pool.push_back(pr.a);
    e->prof.pool.push_back(pr.b);
  }
  e->prof.pairs.clear();
  for (int i = 0; i < DCD_PROF_COUNT; ++i) { out[i] = e->prof.acc[i]; e->prof.acc[i] = dcd_prof_entry{}; }
  return DCD_OK;
}
int64_t dcd_launch_count(const dcd_engine* e) { return e ? e->launches : 0; }

int dcd_debug_layer_outputs(dcd_engine* e, float* host_sink, size_t capacity) {
  if (!e) return DCD_E_INVALID;
  cudaSetDevice(e->device);
  if (host_sink && !e->tap_dev) {
    cudaError_t ce = cudaMalloc(&e->tap_dev, (size_t)e->Tm * e->H * 4);
    if (ce != cudaSuccess) return cuda_fail(e, ce, "tap buffer");
    e->allocs.push_back(e->tap_dev);
  }
  e->tap_sink = host_sink;
  e->tap_cap = host_sink ? capacity : 0;
  return DCD_OK;
}

int dcd_debug_bounded_wait_probe(dcd_engine* e, int polls) {
  if (!e) return DCD_E_INVALID;
  if (polls < 1 || polls > (1 << 20)) return fail(e, DCD_E_INVALID, "polls must be in [1, 2^20]");
  cudaSetDevice(e->device);
  e->launches += 1;
  bounded_wait_probe_kernel<<<1, 32, 0, e->stream>>>(e->d_err, (uint32_t)polls, DERR_GEMM_TIMEOUT);
  CK(e, cudaGetLastError(), "bounded-wait probe");
  return sync_and_check(e);
}

int dcd_pack(dcd_engine* e, const int32_t* lens, size_t B, int32_t pos_start, int32_t* cu_seqlens, int32_t* positions, int32_t* tok_q,
             int32_t* last_row) {
  if (!e) return DCD_E_INVALID;
  if (B == 0 || !lens) return fail(e, DCD_E_INVALID, "empty batch");
  cudaSetDevice(e->device);
  size_t total = 0;
  for (size_t i = 0; i < B; ++i) total += lens[i] > 0 ? (size_t)lens[i] : 0;
  if (B > (size_t)e->max_batch || total > (size_t)e->Tm) return fail(e, DCD_E_INVALID, "batch exceeds max_pass_tokens %d", e->Tm);
  memcpy(e->h_lens, lens, B * 4);
  CK(e, cudaMemcpyAsync(e->d_lens, e->h_lens, B * 4, cudaMemcpyHostToDevice, e->stream), "lens upload");
  e->launches += 2;
  CK(e, launch_pack(e->d_lens, (int)B, (int)total, pos_start, e->d_cu, e->d_last, e->d_tokq, e->d_tokpos, e->d_err, e->stream), "pack");
  CK(e, cudaMemcpyAsync(cu_seqlens, e->d_cu, (B + 1) * 4, cudaMemcpyDeviceToHost, e->stream), "download");
  CK(e, cudaMemcpyAsync(last_row, e->d_last, B * 4, cudaMemcpyDeviceToHost, e->stream), "download");
  if (total) {
    CK(e, cudaMemcpyAsync(positions, e->d_tokpos, total * 4, cudaMemcpyDeviceToHost, e->stream), "download");
    CK(e, cudaMemcpyAsync(tok_q, e->d_tokq, total * 4, cudaMemcpyDeviceToHost, e->stream), "download");
  }
  return sync_and_check(e);
}

}  // extern "C"
