// Chunked gated delta rule on the 5th-generation tensor cores (tcgen05.mma kind::tf32, TMEM
// accumulators, TMA-fed K/Q tiles), seeded from the cached f32 recurrent state.
//
// Same function as the sequential kernel (gdn_recurrent_kernel; reference: gdn_recurrent,
// native/kernels/kernels.cu:834-865 in juanqui/decidra) and as the reference's chunked form
// (gdn_chunked_tc_body, native/kernels/kernels.cu:1671-1933; formulation :1340-1352), chunk C = 64:
//   G_t   = cumulative log decay inside the chunk (inclusive), Gam_t = exp(G_t)
//   A_ts  = beta_t exp(G_t-G_s) (k_t.k_s)            s <  t   (strictly lower)
//   (I+A) D = beta (V - Gam (K S))                    forward substitution, D = per-step deltas
//   P_ts  = exp(G_t-G_s) (q_t.k_s)                   s <= t
//   O     = Gam (Q S) + P D
//   S'    = exp(G_C) S + (exp(G_C-G) K)^T D
// Only differences of cumulative log decays are exponentiated (never ratios of products).
//
// One CTA = (packed sequence, value head) with all 128 value columns; 128 threads. Everything
// that depends on the state is kept transposed so that TMEM lane = value column = thread:
//   D1 [row, s]   = [K;Q] K^T            (rows 0-63 key tokens, 64-127 query tokens)
//   D2 [vc, t]    = S^T [K;Q]^T          (columns 0-63 (K S)^T, 64-127 (Q S)^T)
//   O2 [vc, t]    = D^T P^T
//   RD [vc, dk]   = D^T (exp(G_C-G) K)     (B operand: a transposed, decay-scaled copy of the K tile that
//                                          the threads write while the first two products run)
//   RS [vc, dk]   = f32 master copy of S^T, updated in place by the epilogue
// so thread vc reads (K S)[., vc] for all 64 tokens from its own TMEM lane, runs the forward
// substitution for its column in registers (right-looking, A^T broadcast from shared memory),
// and writes its rows of D^T and S^T as K-major tf32 operands with the 128-byte swizzle the MMA
// descriptors expect (every operand is K-major). K and Q tiles arrive by TMA straight from the f32 q/k
// buffers; the tensor core ignores the low 13 mantissa bits of those.
// Rows of a partial chunk beyond the sequence get beta = 0 and g = 0: their deltas are exactly
// zero, the decay stays flat, and their outputs are not stored. (They read the next sequence's
// rows or the TMA zero fill, both finite.)
// Every mbarrier wait is bounded; on a timeout the CTA sets the error word, waits for copies in
// flight, frees its TMEM and returns.
#include "gemm_tcgen05.h"
#include "kernels.h"
#include "tc_common.cuh"

namespace gtc {
using namespace tcc;

constexpr int C = 64, DK = 128, DV = 128;
constexpr uint32_t REG = 16384;            // one 32-column (128-byte) slab of a 128-row operand
constexpr uint32_t KQ_OFF = 0;             // [4 slabs][K rows 0-63 | Q rows 64-127][128 B]
constexpr uint32_t ST_OFF = 4 * REG;       // S^T  [4 slabs over dk][vc][128 B]
constexpr uint32_t DT_OFF = 8 * REG;       // D^T  [2 slabs over s][vc][128 B]; A^T (64x64 f32) aliases it until the solve is done
constexpr uint32_t KT_OFF = 10 * REG;      // (exp(G_C-G) K)^T [2 slabs over t][dk][128 B]
constexpr uint32_t P_OFF = 12 * REG;       // P    [2 slabs over s][t][128 B] (8 KB each)
constexpr uint32_t SC_OFF = 13 * REG;      // scalars: G, beta, exp(G_C-G), exp(G) (64 floats each), two sets
constexpr uint32_t BAR_OFF = SC_OFF + 2 * 4 * 64 * 4;
constexpr uint32_t SMEM_BYTES = BAR_OFF + 64 + 1024;  // + alignment slack
constexpr uint32_t D2_COL = 0, D1_COL = 128, O2_COL = 192, RS_COL = 256, RD_COL = 384;
constexpr uint32_t IDESC_N64 = umma_idesc_tf32(128, 64, 0);
constexpr uint32_t IDESC_N128 = umma_idesc_tf32(128, 128, 0);

// byte offset of 16-byte chunk c16 of row `row` inside a slab (128-byte swizzle)
__device__ __forceinline__ uint32_t sw_off(int row, int c16) { return (uint32_t)row * 128u + (uint32_t)((c16 ^ (row & 7)) << 4); }

__device__ __forceinline__ float4 tf32x4(float a, float b, float c, float d) {
  return make_float4(__uint_as_float(cvt_tf32(a)), __uint_as_float(cvt_tf32(b)), __uint_as_float(cvt_tf32(c)), __uint_as_float(cvt_tf32(d)));
}

template <typename T>
__global__ void __launch_bounds__(128, 1)
gdn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const T* __restrict__ conv, int conv_stride,
              const float* __restrict__ gl, const float* __restrict__ beta, const float* __restrict__ seed, float* __restrict__ final_state,
              T* __restrict__ out, const int32_t* __restrict__ cu, int nk, int nv, int* err) {
  const int head = blockIdx.x, b = blockIdx.y;
  const int off = cu[b], len = cu[b + 1] - off;
  const int kh = head / (nv / nk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int vcol0 = 2 * nk * DK + head * DV;

  if (len <= 0) {  // nothing to run: the final state is the seed
    if (final_state)
      for (int r = 0; r < DK; ++r) final_state[(((size_t)b * nv + head) * DK + r) * DV + tid] = seed ? seed[((size_t)head * DK + r) * DV + tid] : 0.f;
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sbase = raw + pad;
  float* sAT = reinterpret_cast<float*>(smem + DT_OFF);
  const uint32_t bar_kq = sbase + BAR_OFF, bar_mma = bar_kq + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + BAR_OFF + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + BAR_OFF + 20);

  if (tid == 0) {
    mbar_init(bar_kq, 1);
    mbar_init(bar_mma, 1);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tlane = tmem_base + ((uint32_t)(warp * 32) << 16);

  auto load_kq = [&](int t0) {  // one elected thread
    mbar_expect_tx(bar_kq, 4 * REG);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tma_load_2d(sbase + KQ_OFF + j * REG, &tmK, bar_kq, kh * DK + j * 32, off + t0);
      tma_load_2d(sbase + KQ_OFF + j * REG + 8192, &tmQ, bar_kq, kh * DK + j * 32, off + t0);
    }
  };
  if (tid == 0) load_kq(0);

  // ---- seed: S^T row of this thread's value column into TMEM (f32 master) and shared memory (tf32) ----
#pragma unroll 1
  for (int j = 0; j < 4; ++j) {
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = seed ? __float_as_uint(seed[((size_t)head * DK + j * 32 + i) * DV + tid]) : 0u;
    tmem_st32(tlane + RS_COL + j * 32, v);
#pragma unroll
    for (int c = 0; c < 8; ++c)
      *reinterpret_cast<float4*>(smem + ST_OFF + j * REG + sw_off(tid, c)) =
          tf32x4(__uint_as_float(v[4 * c]), __uint_as_float(v[4 * c + 1]), __uint_as_float(v[4 * c + 2]), __uint_as_float(v[4 * c + 3]));
  }
  tmem_st_wait();
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();

  const int n_chunks = (len + C - 1) / C;
  uint32_t mma_phase = 0;
  bool ok = true;
#pragma unroll 1
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int t0 = ci * C;
    const int nt = min(C, len - t0);
    const bool last = ci + 1 == n_chunks;
    // the scalar set alternates so that a warp may start the next chunk while others finish this one
    float* sG = reinterpret_cast<float*>(smem + SC_OFF) + (ci & 1) * 256;
    float* sB = sG + 64;
    float* sE = sG + 128;
    float* sGam = sG + 192;

    // ---- per-chunk scalars (warp 0: decays, warp 1: beta) and this column's V values --------------
    if (warp == 0) {
      float g0 = lane < nt ? gl[(size_t)(off + t0 + lane) * nv + head] : 0.f;
      float g1 = lane + 32 < nt ? gl[(size_t)(off + t0 + lane + 32) * nv + head] : 0.f;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n0 = __shfl_up_sync(0xffffffffu, g0, o), n1 = __shfl_up_sync(0xffffffffu, g1, o);
        if (lane >= o) { g0 += n0; g1 += n1; }
      }
      g1 += __shfl_sync(0xffffffffu, g0, 31);
      const float gend = __shfl_sync(0xffffffffu, g1, 31);
      sG[lane] = g0;
      sG[lane + 32] = g1;
      sGam[lane] = expf(g0);
      sGam[lane + 32] = expf(g1);
      sE[lane] = expf(gend - g0);
      sE[lane + 32] = expf(gend - g1);
    } else if (warp == 1) {
      sB[lane] = lane < nt ? beta[(size_t)(off + t0 + lane) * nv + head] : 0.f;
      sB[lane + 32] = lane + 32 < nt ? beta[(size_t)(off + t0 + lane + 32) * nv + head] : 0.f;
    }
    float rhs[C];
    {
      const T* vp = conv + (size_t)(off + t0) * conv_stride + vcol0 + tid;
#pragma unroll
      for (int t = 0; t < C; ++t) rhs[t] = t < nt ? Ty<T>::ld(vp + (size_t)t * conv_stride) : 0.f;
    }
    __syncthreads();  // scalars visible; S^T of the previous chunk written and fenced by every thread

    // ---- MMA 1: D1 = [K;Q] K^T, D2 = S^T [K;Q]^T --------------------------------------------------------
    ok = mbar_wait(bar_kq, (uint32_t)(ci & 1), abort_flag);  // every thread reads the K tile below
    if (tid == 0 && ok) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t dkq = umma_desc(sbase + KQ_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        umma_tf32(tmem_base + D1_COL, dkq, dkq, IDESC_N64, kk != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t dst = umma_desc(sbase + ST_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        const uint64_t dkq = umma_desc(sbase + KQ_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        umma_tf32(tmem_base + D2_COL, dst, dkq, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      umma_commit_to(bar_mma);
    }
    // ---- meanwhile: row dk = tid of (exp(G_C-G) K)^T, the K-major B operand of the state update ---------------
    if (ok) {
      const uint8_t* kcol = smem + KQ_OFF + (tid >> 5) * REG + (tid & 3) * 4;
      const int c16 = (tid & 31) >> 2;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        float kv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = 4 * c + i;
          kv[i] = sE[t] * *reinterpret_cast<const float*>(kcol + t * 128 + ((c16 ^ (t & 7)) << 4));
        }
        *reinterpret_cast<float4*>(smem + KT_OFF + (uint32_t)(c >> 3) * REG + sw_off(tid, c & 7)) = tf32x4(kv[0], kv[1], kv[2], kv[3]);
      }
    }
    ok = ok && mbar_wait(bar_mma, mma_phase, abort_flag);
    mma_phase ^= 1u;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();

    // ---- D1 rows: key-token rows give A^T, query-token rows give P -------------------------------------
    if (tid < 64) {
      const int t = tid;
      const float Gt = sG[t], bt = sB[t];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld32(tlane + D1_COL + h * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int s = h * 32 + i;
          if (s < t) sAT[s * C + t] = bt * __expf(Gt - sG[s]) * __uint_as_float(v[i]);
        }
      }
    } else {
      const int t = tid - 64;
      const float Gt = sG[t];
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t v[32];
        tmem_ld32(tlane + D1_COL + h * 32, v);
        tmem_ld_wait();
        float pr[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int s = h * 32 + i;
          pr[i] = s <= t ? __expf(Gt - sG[s]) * __uint_as_float(v[i]) : 0.f;
        }
#pragma unroll
        for (int c = 0; c < 8; ++c)
          *reinterpret_cast<float4*>(smem + P_OFF + h * 8192 + sw_off(t, c)) = tf32x4(pr[4 * c], pr[4 * c + 1], pr[4 * c + 2], pr[4 * c + 3]);
      }
    }
    // ---- right-hand side beta (V - Gam (K S)) for this value column ----------------------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      uint32_t v[32];
      tmem_ld32(tlane + D2_COL + h * 32, v);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int t = h * 32 + i;
        rhs[t] = sB[t] * (rhs[t] - sGam[t] * __uint_as_float(v[i]));
      }
    }
    __syncthreads();  // A^T complete

    // ---- forward substitution, right-looking: after step p, rhs[p] is the delta of token p -----------------
#pragma unroll
    for (int p = 0; p < C - 1; ++p) {
      const float d = rhs[p];
#pragma unroll
      for (int r4 = (p + 1) / 4; r4 < C / 4; ++r4) {
        const float4 a = *reinterpret_cast<const float4*>(sAT + p * C + r4 * 4);
        if (r4 * 4 + 0 > p) rhs[r4 * 4 + 0] = fmaf(-a.x, d, rhs[r4 * 4 + 0]);
        if (r4 * 4 + 1 > p) rhs[r4 * 4 + 1] = fmaf(-a.y, d, rhs[r4 * 4 + 1]);
        if (r4 * 4 + 2 > p) rhs[r4 * 4 + 2] = fmaf(-a.z, d, rhs[r4 * 4 + 2]);
        if (r4 * 4 + 3 > p) rhs[r4 * 4 + 3] = fmaf(-a.w, d, rhs[r4 * 4 + 3]);
      }
    }
    __syncthreads();  // every thread is done with A^T (D^T below overwrites it)

    // ---- D^T row as a K-major tf32 operand ---------------------------------------------------------------------
#pragma unroll
    for (int c = 0; c < 16; ++c)
      *reinterpret_cast<float4*>(smem + DT_OFF + (uint32_t)(c >> 3) * REG + sw_off(tid, c & 7)) =
          tf32x4(rhs[4 * c], rhs[4 * c + 1], rhs[4 * c + 2], rhs[4 * c + 3]);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();

    // ---- MMA 2: O2 = D^T P^T, RD = D^T (exp(G_C-G) K) --------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t dd = umma_desc(sbase + DT_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        const uint64_t dp = umma_desc(sbase + P_OFF + (kk >> 2) * 8192 + (kk & 3) * 32, 16, 1024);
        umma_tf32(tmem_base + O2_COL, dd, dp, IDESC_N64, kk != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t dd = umma_desc(sbase + DT_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        const uint64_t dk = umma_desc(sbase + KT_OFF + (kk >> 2) * REG + (kk & 3) * 32, 16, 1024);
        umma_tf32(tmem_base + RD_COL, dd, dk, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      umma_commit_to(bar_mma);
    }
    ok = mbar_wait(bar_mma, mma_phase, abort_flag);
    mma_phase ^= 1u;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && !last) load_kq(t0 + C);  // the K/Q tile is free again

    // ---- outputs O[t, vc] = Gam_t (Q S)[t, vc] + (P D)[t, vc] ----------------------------------------------------
    {
      T* op = out + (size_t)(off + t0) * nv * DV + (size_t)head * DV + tid;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t qs[32], pd[32];
        tmem_ld32(tlane + D2_COL + 64 + h * 32, qs);
        tmem_ld32(tlane + O2_COL + h * 32, pd);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const int t = h * 32 + i;
          if (t < nt) Ty<T>::st(op + (size_t)t * nv * DV, fmaf(sGam[t], __uint_as_float(qs[i]), __uint_as_float(pd[i])));
        }
      }
    }
    // ---- state S' = exp(G_C) S + RD: f32 master in TMEM, tf32 operand copy (or the final state) ------------------
    {
      const float gamC = sGam[C - 1];
#pragma unroll 1
      for (int j = 0; j < 4; ++j) {
        uint32_t a[32], dl[32];
        tmem_ld32(tlane + RS_COL + j * 32, a);
        tmem_ld32(tlane + RD_COL + j * 32, dl);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(fmaf(gamC, __uint_as_float(a[i]), __uint_as_float(dl[i])));
        if (!last) {
          tmem_st32(tlane + RS_COL + j * 32, a);
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(smem + ST_OFF + j * REG + sw_off(tid, c)) =
                tf32x4(__uint_as_float(a[4 * c]), __uint_as_float(a[4 * c + 1]), __uint_as_float(a[4 * c + 2]), __uint_as_float(a[4 * c + 3]));
        } else if (final_state) {
          float* fp = final_state + (((size_t)b * nv + head) * DK + j * 32) * DV + tid;
#pragma unroll
          for (int i = 0; i < 32; ++i) fp[(size_t)i * DV] = __uint_as_float(a[i]);
        }
      }
      tmem_st_wait();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) set_err(err, DERR_GDN_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

}  // namespace gtc

bool gdn_tc_supported(int dk, int dv) { return dk == gtc::DK && dv == gtc::DV; }

template <typename T>
cudaError_t gdn_tc_prepare_device() {
  return cudaFuncSetAttribute(gtc::gdn_tc_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gtc::SMEM_BYTES);
}
template cudaError_t gdn_tc_prepare_device<float>();
template cudaError_t gdn_tc_prepare_device<bf16>();

int gdn_tc_make_maps(TcTensorMap maps[2], const float* qf, const float* kf, int tokens, int nk) {
  const uint64_t cols = (uint64_t)nk * gtc::DK;
  int r = tc_make_tmap_f32(&maps[0], qf, (uint64_t)tokens, cols, cols, gtc::C);
  if (r) return r;
  return tc_make_tmap_f32(&maps[1], kf, (uint64_t)tokens, cols, cols, gtc::C);
}

template <typename T>
cudaError_t launch_gdn_tc(const TcTensorMap maps[2], const T* conv, int conv_stride, const float* g, const float* beta, const float* seed,
                          float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int* err, cudaStream_t s) {
  if (B <= 0) return cudaSuccess;
  if (B > 65535 || nk <= 0 || nv % nk != 0) return cudaErrorInvalidValue;
  dim3 grid(nv, B);
  gtc::gdn_tc_kernel<T><<<grid, 128, gtc::SMEM_BYTES, s>>>(*reinterpret_cast<const CUtensorMap*>(&maps[0]), *reinterpret_cast<const CUtensorMap*>(&maps[1]),
                                                            conv, conv_stride, g, beta, seed, final_state, out, cu, nk, nv, err);
  return cudaGetLastError();
}
template cudaError_t launch_gdn_tc<float>(const TcTensorMap*, const float*, int, const float*, const float*, const float*, float*, float*, const int32_t*, int, int, int, int*, cudaStream_t);
template cudaError_t launch_gdn_tc<bf16>(const TcTensorMap*, const bf16*, int, const float*, const float*, const float*, float*, bf16*, const int32_t*, int, int, int, int*, cudaStream_t);
