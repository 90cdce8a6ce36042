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
// One CTA = (packed sequence, value head) with all 128 value columns; 256 threads = two warpgroups.
// Everything that depends on the state is kept transposed so that TMEM lane = value column; thread
// `ln` of each warpgroup owns lane ln, and the two warpgroups split every per-lane loop in halves
// (with one warp per scheduler the chunk body ran at a third of an instruction per cycle, all of it
// exposed latency). The forward substitution is sequential per column and runs on warpgroup 0; warpgroup 1
// meanwhile turns the query-token rows of D1 into P and writes the transposed, decay-scaled K operand.
//   D1 [row, s]   = [K;Q] K^T            (rows 0-63 key tokens, 64-127 query tokens)
//   D2 [vc, t]    = S^T [K;Q]^T          (columns 0-63 (K S)^T, 64-127 (Q S)^T)
//   O2 [vc, t]    = D^T P^T
//   RD [vc, dk]   = D^T (exp(G_C-G) K)     (B operand: a transposed, decay-scaled copy of the K tile)
//   VR [vc, t]    = per-thread scratch: the right-hand side, then D
// so thread vc reads (K S)[., vc] for all 64 tokens from its own TMEM lane and runs the forward
// substitution for its column. S^T lives in shared memory as full f32 (it is both the master copy
// and the A operand of D2; the tensor core ignores the low 13 mantissa bits), D^T, P and the
// scaled K^T are written as K-major tf32 operands with the 128-byte swizzle the MMA descriptors
// expect. K and Q tiles arrive by TMA straight from the f32 q/k buffers, and (16-bit storage) the
// chunk's V tile from the conv output into the space that later holds P.
// The per-thread vectors (64 or 128 values) stay in TMEM and are processed in blocks of 16 by
// loops that are not unrolled: unrolled over whole vectors, the chunk body was 170 KB of
// straight-line code and the kernel was bound by instruction fetch.
// The forward substitution is blocked 16x16, left-looking: block j subtracts A[j,i] D[i] for the
// finished blocks i < j, then solves its own triangle in registers.
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

constexpr int C = 64, DK = 128, DV = 128, BLK = 16;
constexpr uint32_t REG = 16384;            // one 32-column (128-byte) slab of a 128-row operand
constexpr uint32_t KQ_OFF = 0;             // [4 slabs][K rows 0-63 | Q rows 64-127][128 B]
constexpr uint32_t ST_OFF = 4 * REG;       // S^T  [4 slabs over dk][vc][128 B], full f32
constexpr uint32_t DT_OFF = 8 * REG;       // D^T  [2 slabs over s][vc][128 B]; A^T (64x64 f32) aliases it until the solve is done
constexpr uint32_t KT_OFF = 10 * REG;      // (exp(G_C-G) K)^T [2 slabs over t][dk][128 B]
constexpr uint32_t P_OFF = 12 * REG;       // P    [2 slabs over s][t][128 B] (8 KB each); before that the V tile
                                           // [2 halves of 64 columns][t][128 B] (16-bit storage only)
constexpr uint32_t SC_OFF = 13 * REG;      // scalars: G, beta, exp(G_C-G), exp(G) (64 floats each), two sets
constexpr uint32_t BAR_OFF = SC_OFF + 2 * 4 * 64 * 4;
constexpr uint32_t SMEM_BYTES = BAR_OFF + 64 + 1024;  // + alignment slack
constexpr uint32_t D2_COL = 0, D1_COL = 128, O2_COL = 192, RD_COL = 256, VR_COL = 384;
constexpr uint32_t IDESC_N64 = umma_idesc_tf32(128, 64, 0);
constexpr uint32_t IDESC_N128 = umma_idesc_tf32(128, 128, 0);

// byte offset of 16-byte chunk c16 of row `row` inside a slab (128-byte swizzle)
__device__ __forceinline__ uint32_t sw_off(int row, int c16) { return (uint32_t)row * 128u + (uint32_t)((c16 ^ (row & 7)) << 4); }

__device__ __forceinline__ float4 tf32x4(float a, float b, float c, float d) {
  return make_float4(__uint_as_float(cvt_tf32(a)), __uint_as_float(cvt_tf32(b)), __uint_as_float(cvt_tf32(c)), __uint_as_float(cvt_tf32(d)));
}
__device__ __forceinline__ float u2f(uint32_t x) { return __uint_as_float(x); }
__device__ __forceinline__ uint32_t f2u(float x) { return __float_as_uint(x); }

template <typename T> __device__ __forceinline__ void st_if(T* p, float v, bool pred);
template <> __device__ __forceinline__ void st_if<float>(float* p, float v, bool pred) {
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %2, 0;\n@p st.global.f32 [%0], %1;\n}\n" ::"l"(p), "f"(v), "r"((int)pred) : "memory");
}
template <> __device__ __forceinline__ void st_if<bf16>(bf16* p, float v, bool pred) {
  const bf16 h = __float2bfloat16_rn(v);
  asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %2, 0;\n@p st.global.b16 [%0], %1;\n}\n" ::"l"(p), "h"(*reinterpret_cast<const uint16_t*>(&h)), "r"((int)pred)
               : "memory");
}

template <typename T>
__global__ void __launch_bounds__(256, 1)
gdn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              const T* __restrict__ conv, int conv_stride,
              const float* __restrict__ gl, const float* __restrict__ beta, const float* __restrict__ seed, float* __restrict__ final_state,
              T* __restrict__ out, const int32_t* __restrict__ cu, int nk, int nv, int* err) {
  const int head = blockIdx.x, b = blockIdx.y;
  const int off = cu[b], len = cu[b + 1] - off;
  const int kh = head / (nv / nk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int wg = warp >> 2, ln = tid & 127;  // warpgroup; TMEM lane / operand row owned by this thread
  const int vcol0 = 2 * nk * DK + head * DV;

  if (len <= 0) {  // nothing to run: the final state is the seed
    if (final_state && wg == 0)
      for (int r = 0; r < DK; ++r) final_state[(((size_t)b * nv + head) * DK + r) * DV + ln] = seed ? seed[((size_t)head * DK + r) * DV + ln] : 0.f;
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sbase = raw + pad;
  float* sAT = reinterpret_cast<float*>(smem + DT_OFF);
  float* sc = reinterpret_cast<float*>(smem + SC_OFF);
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
  const uint32_t tlane = tmem_base + ((uint32_t)((warp & 3) * 32) << 16);

  constexpr bool V_TMA = sizeof(T) == 2;  // the V tile of a 16-bit conv output fits the P space
  auto load_kq = [&](int t0) {  // one elected thread; K/Q tiles and (16-bit storage) the V tile of the chunk at t0
    mbar_expect_tx(bar_kq, 4 * REG + (V_TMA ? REG : 0));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      tma_load_2d(sbase + KQ_OFF + j * REG, &tmK, bar_kq, kh * DK + j * 32, off + t0);
      tma_load_2d(sbase + KQ_OFF + j * REG + 8192, &tmQ, bar_kq, kh * DK + j * 32, off + t0);
    }
    if (V_TMA) {
      tma_load_2d(sbase + P_OFF, &tmV, bar_kq, vcol0, off + t0);
      tma_load_2d(sbase + P_OFF + 8192, &tmV, bar_kq, vcol0 + 64, off + t0);
    }
  };
  // Scalars of the chunk at t0 into set `set` (warp 6: decays, warp 7: beta; warp 0 issues the MMAs meanwhile). A set is rewritten two
  // chunks later, after every thread has passed a barrier that follows its last read.
  auto scalars = [&](int t0, int set) {
    const int nt = min(C, len - t0);
    float* sG = sc + set * 256;
    if (warp == 6) {
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
      sG[192 + lane] = expf(g0);
      sG[192 + lane + 32] = expf(g1);
      sG[128 + lane] = expf(gend - g0);
      sG[128 + lane + 32] = expf(gend - g1);
    } else if (warp == 7) {
      sG[64 + lane] = lane < nt ? beta[(size_t)(off + t0 + lane) * nv + head] : 0.f;
      sG[64 + lane + 32] = lane + 32 < nt ? beta[(size_t)(off + t0 + lane + 32) * nv + head] : 0.f;
    }
  };
  // 32-bit storage: this thread's V column of the chunk at t0 into its TMEM scratch (all loads in flight together).
  auto park_v = [&](int t0) {  // each warpgroup parks its half of the chunk's rows
    const int nt = min(C, len - t0);
    const T* vp = conv + (size_t)(off + t0) * conv_stride + vcol0 + ln;
    uint32_t v[C / 2];
#pragma unroll
    for (int i = 0; i < C / 2; ++i) {
      const int t = wg * (C / 2) + i;
      const float x = Ty<T>::ld(vp + (size_t)min(t, nt - 1) * conv_stride);
      v[i] = f2u(t < nt ? x : 0.f);
    }
#pragma unroll
    for (int j = 0; j < C / BLK / 2; ++j) tmem_st16(tlane + VR_COL + (wg * 2 + j) * BLK, v + j * BLK);
    tmem_st_wait();
  };

  if (tid == 0) load_kq(0);
  scalars(0, 0);
  if (!V_TMA) park_v(0);
  // ---- seed: S^T row of this thread's value column into shared memory ------------------------------------
#pragma unroll 1
  for (int j = wg * 4; j < wg * 4 + 4; ++j) {
    float v[BLK];
#pragma unroll
    for (int i = 0; i < BLK; ++i) v[i] = seed ? seed[((size_t)head * DK + j * BLK + i) * DV + ln] : 0.f;
#pragma unroll
    for (int q = 0; q < 4; ++q)
      *reinterpret_cast<float4*>(smem + ST_OFF + (uint32_t)(j >> 1) * REG + sw_off(ln, (j & 1) * 4 + q)) = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();

  // operand descriptors of slab 0; a k-step of 8 columns advances the start address by 32 bytes, a slab by REG
  const uint64_t d_kq = umma_desc(sbase + KQ_OFF, 16, 1024), d_st = umma_desc(sbase + ST_OFF, 16, 1024), d_dt = umma_desc(sbase + DT_OFF, 16, 1024),
                 d_kt = umma_desc(sbase + KT_OFF, 16, 1024), d_p = umma_desc(sbase + P_OFF, 16, 1024);
  const int n_chunks = (len + C - 1) / C;
  uint32_t mma_phase = 0;
  bool ok = true;
#pragma unroll 1
  for (int ci = 0; ci < n_chunks; ++ci) {
    const int t0 = ci * C;
    const int nt = min(C, len - t0);
    const bool last = ci + 1 == n_chunks;
    const float* sG = sc + (ci & 1) * 256;
    const float* sB = sG + 64;
    const float* sE = sG + 128;
    const float* sGam = sG + 192;
    __syncthreads();  // scalars visible; S^T of the previous chunk written and fenced by every thread

    // ---- MMA 1: D1 = [K;Q] K^T, D2 = S^T [K;Q]^T --------------------------------------------------------
    ok = mbar_wait(bar_kq, (uint32_t)(ci & 1), abort_flag);  // every thread reads the K tile below
    if (tid == 0 && ok) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        umma_tf32(tmem_base + D1_COL, d_kq + o, d_kq + o, IDESC_N64, kk != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        umma_tf32(tmem_base + D2_COL, d_st + o, d_kq + o, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      umma_commit_to(bar_mma);
    }
    ok = ok && mbar_wait(bar_mma, mma_phase, abort_flag);
    mma_phase ^= 1u;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();

    // ---- right-hand side beta (V - Gam (K S)) for this value column into the scratch ------------------------------
#pragma unroll 1
    for (int j = wg * 2; j < wg * 2 + 2; ++j) {
      uint32_t x[BLK], v[BLK];
      tmem_ld16(tlane + D2_COL + j * BLK, x);
      if (V_TMA) {
        const uint8_t* vcol = smem + P_OFF + (ln >> 6) * 8192 + (ln & 7) * 2;
        const int c16 = (ln & 63) >> 3;
#pragma unroll
        for (int i = 0; i < BLK; ++i) {
          const int t = j * BLK + i;
          v[i] = (uint32_t)(*reinterpret_cast<const uint16_t*>(vcol + t * 128 + ((c16 ^ (t & 7)) << 4))) << 16;  // bf16 -> f32 bits
        }
      } else {
        tmem_ld16(tlane + VR_COL + j * BLK, v);
      }
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 b4 = *reinterpret_cast<const float4*>(sB + j * BLK + q * 4);
        const float4 g4 = *reinterpret_cast<const float4*>(sGam + j * BLK + q * 4);
        v[4 * q + 0] = f2u(b4.x * (u2f(v[4 * q + 0]) - g4.x * u2f(x[4 * q + 0])));
        v[4 * q + 1] = f2u(b4.y * (u2f(v[4 * q + 1]) - g4.y * u2f(x[4 * q + 1])));
        v[4 * q + 2] = f2u(b4.z * (u2f(v[4 * q + 2]) - g4.z * u2f(x[4 * q + 2])));
        v[4 * q + 3] = f2u(b4.w * (u2f(v[4 * q + 3]) - g4.w * u2f(x[4 * q + 3])));
      }
      tmem_st16(tlane + VR_COL + j * BLK, v);
    }
    tmem_st_wait();
    tc_fence_before();  // the other warpgroup's half of the right-hand side is read by the solve below

    // ---- D1 rows of the key tokens give A^T (the query-token rows, P, are taken by warpgroup 1 during the solve) ---------
    // (exponents are clamped to <= 0 and the result selected, so the loops stay branch-free)
    if (ln < 64) {
      const int t = ln;
      const float Gt = sG[t], bt = sB[t];
#pragma unroll 1
      for (int j = wg * 2; j < wg * 2 + 2; ++j) {
        uint32_t v[BLK];
        tmem_ld16(tlane + D1_COL + j * BLK, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 gs = *reinterpret_cast<const float4*>(sG + j * BLK + q * 4);
          const float ge[4] = {gs.x, gs.y, gs.z, gs.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int s = j * BLK + q * 4 + i;
            const float a = bt * __expf(fminf(Gt - ge[i], 0.f)) * u2f(v[q * 4 + i]);
            sAT[s * C + t] = s < t ? a : 0.f;
          }
        }
      }
    }
    __syncthreads();  // A^T complete; the right-hand sides of both warpgroups are in the scratch

    // ---- forward substitution, blocked 16x16, left-looking; block j ends up holding D[16j .. 16j+15] ----------
    if (wg == 1) {
      // ---- warpgroup 1, while warpgroup 0 runs the forward substitution: P from the query-token rows of D1 (over the V tile,
      // which every thread has read by now), then row dk = ln of (exp(G_C-G) K)^T, the K-major B operand of the state update
      if (ln >= 64) {
        const int t = ln - 64;
        const float Gt = sG[t];
#pragma unroll 1
        for (int j = 0; j < C / BLK; ++j) {
          uint32_t v[BLK];
          tmem_ld16(tlane + D1_COL + j * BLK, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 gs = *reinterpret_cast<const float4*>(sG + j * BLK + q * 4);
            const float ge[4] = {gs.x, gs.y, gs.z, gs.w};
            float pr[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int s = j * BLK + q * 4 + i;
              const float e = __expf(fminf(Gt - ge[i], 0.f)) * u2f(v[q * 4 + i]);
              pr[i] = s <= t ? e : 0.f;
            }
            *reinterpret_cast<float4*>(smem + P_OFF + (uint32_t)(j >> 1) * 8192 + sw_off(t, (j & 1) * 4 + q)) = tf32x4(pr[0], pr[1], pr[2], pr[3]);
          }
        }
      }
      // K^T rows: warps 4 and 5 (no P rows to do) take their own row in full and the first 32 tokens of row ln + 64; warps 6 and 7
      // take the last 32 tokens of their own row
      auto kt_row = [&](int r, int c_lo, int c_hi) {
        const uint8_t* kcol = smem + KQ_OFF + (r >> 5) * REG + (r & 3) * 4;
        const int c16 = (r & 31) >> 2;
#pragma unroll 4
        for (int c = c_lo; c < c_hi; ++c) {
          const float4 e4 = *reinterpret_cast<const float4*>(sE + 4 * c);
          const float k0 = e4.x * *reinterpret_cast<const float*>(kcol + (4 * c + 0) * 128 + ((c16 ^ ((4 * c + 0) & 7)) << 4));
          const float k1 = e4.y * *reinterpret_cast<const float*>(kcol + (4 * c + 1) * 128 + ((c16 ^ ((4 * c + 1) & 7)) << 4));
          const float k2 = e4.z * *reinterpret_cast<const float*>(kcol + (4 * c + 2) * 128 + ((c16 ^ ((4 * c + 2) & 7)) << 4));
          const float k3 = e4.w * *reinterpret_cast<const float*>(kcol + (4 * c + 3) * 128 + ((c16 ^ ((4 * c + 3) & 7)) << 4));
          *reinterpret_cast<float4*>(smem + KT_OFF + (uint32_t)(c >> 3) * REG + sw_off(r, c & 7)) = tf32x4(k0, k1, k2, k3);
        }
      };
      if (ln < 64) {
        kt_row(ln, 0, 16);
        kt_row(ln + 64, 0, 8);
      } else {
        kt_row(ln, 8, 16);
      }
    }
    if (wg == 0) {
    tc_fence_after();
#pragma unroll 1
    for (int jb = 0; jb < C / BLK; ++jb) {
      float r[BLK];
      {
        uint32_t rv[BLK];
        tmem_ld16(tlane + VR_COL + jb * BLK, rv);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < BLK; ++i) r[i] = u2f(rv[i]);
      }
#pragma unroll 1
      for (int ib = 0; ib < jb; ++ib) {
        uint32_t d[BLK];
        tmem_ld16(tlane + VR_COL + ib * BLK, d);
        tmem_ld_wait();
        const float* a = sAT + (ib * BLK) * C + jb * BLK;  // a[p*C + i] = A[16jb+i][16ib+p]
#pragma unroll
        for (int p = 0; p < BLK; ++p) {
          const float dp = u2f(d[p]);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float4 av = *reinterpret_cast<const float4*>(a + p * C + 4 * q);
            r[4 * q + 0] = fmaf(-av.x, dp, r[4 * q + 0]);
            r[4 * q + 1] = fmaf(-av.y, dp, r[4 * q + 1]);
            r[4 * q + 2] = fmaf(-av.z, dp, r[4 * q + 2]);
            r[4 * q + 3] = fmaf(-av.w, dp, r[4 * q + 3]);
          }
        }
      }
      {
        const float* a = sAT + (jb * BLK) * C + jb * BLK;
#pragma unroll
        for (int p = 0; p < BLK - 1; ++p) {
          const float dp = r[p];
#pragma unroll
          for (int q = (p + 1) / 4; q < 4; ++q) {
            const float4 av = *reinterpret_cast<const float4*>(a + p * C + 4 * q);
            if (4 * q + 0 > p) r[4 * q + 0] = fmaf(-av.x, dp, r[4 * q + 0]);
            if (4 * q + 1 > p) r[4 * q + 1] = fmaf(-av.y, dp, r[4 * q + 1]);
            if (4 * q + 2 > p) r[4 * q + 2] = fmaf(-av.z, dp, r[4 * q + 2]);
            if (4 * q + 3 > p) r[4 * q + 3] = fmaf(-av.w, dp, r[4 * q + 3]);
          }
        }
      }
      uint32_t rv[BLK];
#pragma unroll
      for (int i = 0; i < BLK; ++i) rv[i] = f2u(r[i]);
      tmem_st16(tlane + VR_COL + jb * BLK, rv);
      tmem_st_wait();
    }
    }
    tc_fence_before();
    __syncthreads();  // every thread is done with A^T (D^T below overwrites it)

    // ---- D^T row as a K-major tf32 operand ---------------------------------------------------------------------
    tc_fence_after();
#pragma unroll 1
    for (int j = wg * 2; j < wg * 2 + 2; ++j) {
      uint32_t d[BLK];
      tmem_ld16(tlane + VR_COL + j * BLK, d);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q)
        *reinterpret_cast<float4*>(smem + DT_OFF + (uint32_t)(j >> 1) * REG + sw_off(ln, (j & 1) * 4 + q)) =
            tf32x4(u2f(d[4 * q]), u2f(d[4 * q + 1]), u2f(d[4 * q + 2]), u2f(d[4 * q + 3]));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();

    // ---- MMA 2: O2 = D^T P^T, RD = D^T (exp(G_C-G) K) --------------------------------------------------------------
    if (tid == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4), op = (uint64_t)(((kk >> 2) * 8192 + (kk & 3) * 32) >> 4);
        umma_tf32(tmem_base + O2_COL, d_dt + o, d_p + op, IDESC_N64, kk != 0 ? 1u : 0u);
      }
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        umma_tf32(tmem_base + RD_COL, d_dt + o, d_kt + o, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      umma_commit_to(bar_mma);
    }
    // ---- meanwhile: scalars and V column of the next chunk (the scratch is free again) ---------------------------
    if (!last) {
      scalars(t0 + C, (ci + 1) & 1);
      if (!V_TMA) park_v(t0 + C);
    }
    ok = mbar_wait(bar_mma, mma_phase, abort_flag);
    mma_phase ^= 1u;
    if (!__syncthreads_and(ok)) { ok = false; break; }
    tc_fence_after();
    if (tid == 0 && !last) load_kq(t0 + C);  // the K/Q tile is free again

    // ---- outputs O[t, vc] = Gam_t (Q S)[t, vc] + (P D)[t, vc] ----------------------------------------------------
    {
      T* op = out + (size_t)(off + t0) * nv * DV + (size_t)head * DV + ln;
      const size_t os = (size_t)nv * DV;
#pragma unroll 1
      for (int j = wg * 2; j < wg * 2 + 2; ++j) {
        uint32_t qs[BLK], pd[BLK];
        tmem_ld16(tlane + D2_COL + 64 + j * BLK, qs);
        tmem_ld16(tlane + O2_COL + j * BLK, pd);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float4 g4 = *reinterpret_cast<const float4*>(sGam + j * BLK + q * 4);
          const float ge[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int t = j * BLK + q * 4 + i;
            st_if<T>(op + (size_t)t * os, fmaf(ge[i], u2f(qs[q * 4 + i]), u2f(pd[q * 4 + i])), t < nt);
          }
        }
      }
    }
    // ---- state S' = exp(G_C) S + RD, in place in shared memory (or out to the final state) ---------------------
    {
      const float gamC = sGam[C - 1];
#pragma unroll 1
      for (int j = wg * 4; j < wg * 4 + 4; ++j) {
        uint32_t dl[BLK];
        tmem_ld16(tlane + RD_COL + j * BLK, dl);
        float4 o4[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) o4[q] = *reinterpret_cast<const float4*>(smem + ST_OFF + (uint32_t)(j >> 1) * REG + sw_off(ln, (j & 1) * 4 + q));
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          o4[q].x = fmaf(gamC, o4[q].x, u2f(dl[4 * q + 0]));
          o4[q].y = fmaf(gamC, o4[q].y, u2f(dl[4 * q + 1]));
          o4[q].z = fmaf(gamC, o4[q].z, u2f(dl[4 * q + 2]));
          o4[q].w = fmaf(gamC, o4[q].w, u2f(dl[4 * q + 3]));
        }
        if (!last) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<float4*>(smem + ST_OFF + (uint32_t)(j >> 1) * REG + sw_off(ln, (j & 1) * 4 + q)) = o4[q];
        } else if (final_state) {
          float* fp = final_state + (((size_t)b * nv + head) * DK + j * BLK) * DV + ln;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            fp[(size_t)(4 * q + 0) * DV] = o4[q].x;
            fp[(size_t)(4 * q + 1) * DV] = o4[q].y;
            fp[(size_t)(4 * q + 2) * DV] = o4[q].z;
            fp[(size_t)(4 * q + 3) * DV] = o4[q].w;
          }
        }
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) set_err(err, DERR_GDN_TIMEOUT);
#pragma unroll 1
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

int gdn_tc_make_maps(TcTensorMap maps[3], const float* qf, const float* kf, const void* conv, int conv_stride, int conv_cols, int elem_size,
                     int tokens, int nk) {
  const uint64_t cols = (uint64_t)nk * gtc::DK;
  int r = tc_make_tmap_f32(&maps[0], qf, (uint64_t)tokens, cols, cols, gtc::C);
  if (r) return r;
  r = tc_make_tmap_f32(&maps[1], kf, (uint64_t)tokens, cols, cols, gtc::C);
  if (r) return r;
  if (elem_size == 2) return tc_make_tmap_strided(&maps[2], conv, (uint64_t)tokens, (uint64_t)conv_cols, (uint64_t)conv_stride, gtc::C);
  maps[2] = maps[1];  // unused by the 32-bit kernel
  return 0;
}

template <typename T>
cudaError_t launch_gdn_tc(const TcTensorMap maps[3], const T* conv, int conv_stride, const float* g, const float* beta, const float* seed,
                          float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int* err, cudaStream_t s) {
  if (B <= 0) return cudaSuccess;
  if (B > 65535 || nk <= 0 || nv % nk != 0) return cudaErrorInvalidValue;
  dim3 grid(nv, B);
  gtc::gdn_tc_kernel<T><<<grid, 256, gtc::SMEM_BYTES, s>>>(*reinterpret_cast<const CUtensorMap*>(&maps[0]), *reinterpret_cast<const CUtensorMap*>(&maps[1]),
                                                            *reinterpret_cast<const CUtensorMap*>(&maps[2]), conv, conv_stride, g, beta, seed, final_state,
                                                            out, cu, nk, nv, err);
  return cudaGetLastError();
}
template cudaError_t launch_gdn_tc<float>(const TcTensorMap*, const float*, int, const float*, const float*, const float*, float*, float*, const int32_t*, int, int, int, int*, cudaStream_t);
template cudaError_t launch_gdn_tc<bf16>(const TcTensorMap*, const bf16*, int, const float*, const float*, const float*, float*, bf16*, const int32_t*, int, int, int, int*, cudaStream_t);
