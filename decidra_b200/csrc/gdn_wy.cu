// Chunked gated delta rule in WY form on the 5th-generation tensor cores (tcgen05.mma kind::tf32, TMEM accumulators and TMEM A
// operands, TMA-fed K/Q/V tiles), seeded from the cached f32 recurrent state.
//
// Same function as the sequential kernel (gdn_recurrent_kernel; reference: gdn_recurrent, native/kernels/kernels.cu:834-865 in
// juanqui/decidra) and the same algebra as the reference's chunked form (native/kernels/kernels.cu:1340-1352, body :1671-1933),
// chunk C = 64:
//   G_t   = cumulative log decay inside the chunk (inclusive), Gam_t = exp(G_t)
//   A_ts  = beta_t exp(G_t-G_s) (k_t.k_s)            s <  t   (strictly lower)
//   T     = (I+A)^-1
//   W     = T (beta Gam K),  U = T (beta V)           state-independent
//   D     = U - W S                                   the per-step deltas
//   P_ts  = exp(G_t-G_s) (q_t.k_s)                   s <= t
//   O     = Gam (Q S) + P D
//   S'    = exp(G_C) S + (exp(G_C-G) K)^T D
// Only differences of cumulative log decays are exponentiated (never ratios of products).
//
// gdn_tc_kernel (gdn_tcgen05.cu) solves (I+A) D = beta (V - Gam K S) by forward substitution, one value column per thread: 2016
// multiply-adds per thread and chunk on the sequential path. Here the triangular system is inverted once per chunk and head, blockwise,
// and D = T R with R = beta (V - Gam K S) (which equals U - W S) is one more tensor-core product:
//   - the four 16x16 diagonal blocks by substitution in registers (64 threads, 120 multiply-adds each);
//   - with X = blockdiag(inverses) and F = X E (E = the block-strictly-lower part of A, F^4 = 0):
//     T = (I - F + F^2 - F^3) X, seventeen 16x16x16 products on mma.sync m16n8k8 with every operand split in two tf32 halves
//     (a_hi b_hi + a_hi b_lo + a_lo b_hi), i.e. f32-grade, spread over the warps. tcgen05 has no shape this small and each of
//     its results would have to go through TMEM and back into an operand: this part is latency, not throughput;
//   - T is written as a K-major tf32 operand; R^T is written by its owners into TMEM and is the A operand of D^T = R^T T^T.
//
// One CTA = (packed sequence, value head) with all 128 value columns; 512 threads = four warpgroups. Everything that depends on the
// state is kept transposed so that TMEM lane = value column; thread `ln` of each warpgroup owns lane ln, and the four warpgroups
// split every per-lane loop in quarters.
//   D1 [row, s]   = [K;Q] K^T             (rows 0-63 key tokens -> A, 64-127 query tokens -> P)          smem x smem
//   D2 [vc, t]    = S^T [K;Q]^T           (columns 0-63 (K S)^T, 64-127 (Q S)^T)                         TMEM x smem
//   RT [vc, s]    = beta_s (V^T - Gam_s (K S)^T)     written to TMEM by the threads
//   DR [vc, t]    = RT T^T                                                                               TMEM x smem
//   DT [vc, t]    = DR rounded to tf32, written back to TMEM as the A operand of the next two
//   O2 [vc, t]    = DT P^T                                                                               TMEM x smem
//   RD [vc, dk]   = DT (exp(G_C-G) K)     (B = a transposed copy of K with its columns scaled)           TMEM x smem
// S^T lives in TMEM as full f32 (master copy and A operand of D2; the tensor core ignores the low 13 mantissa bits): the state update
// is a TMEM read-modify-write and the state products read only their B operand from shared memory.
// The next chunk's K/Q/V tiles are requested as soon as this chunk's D2 and R are done, two thirds of a chunk ahead of their use.
// Rows of a partial chunk beyond the sequence get beta = 0 and g = 0: their rows of A and of R are zero, so their deltas are exactly
// zero, the decay stays flat, and their outputs are not stored. (They read the next sequence's rows or the TMA zero fill, both
// finite.)
// Every mbarrier wait is bounded; on a timeout the CTA sets the error word, waits for copies in flight, frees its TMEM and returns.
#include "gemm_tcgen05.h"
#include "kernels.h"
#include "tc_common.cuh"

namespace gwy {
using namespace tcc;

constexpr int C = 64, DK = 128, DV = 128, BLK = 16, NWG = 4, THREADS = 128 * NWG;
constexpr int LDM = 68;                              // row stride of the two f32 scratch matrices (conflict-free A fragments)
constexpr uint32_t REG = 16384;                      // one 32-column (128-byte) slab of a 128-row operand
constexpr uint32_t KQ_OFF = 0;                       // [4 slabs over dk][K rows 0-63 | Q rows 64-127][128 B]
constexpr uint32_t KE_OFF = 4 * REG;                 // (exp(G_C-G) K)^T [2 slabs over t][dk][128 B]
constexpr uint32_t X_OFF = 6 * REG;                  // scratch M0 | M1 (64 x LDM f32 each)
constexpr uint32_t X_BYTES = 36864;
constexpr uint32_t T_OFF = X_OFF + X_BYTES;          // T [2 slabs over s][t][128 B] (8 KB each)
constexpr uint32_t P_OFF = T_OFF + REG;              // P [2 slabs over s][t][128 B]
constexpr uint32_t V_OFF = P_OFF + REG;              // the V tile [2 halves of 64 columns][t][128 B] (16-bit storage)
constexpr uint32_t SC_OFF = V_OFF + REG;             // scalars: G, beta, exp(G_C-G), exp(G) (64 floats each), two sets
constexpr uint32_t BAR_OFF = SC_OFF + 2 * 4 * 64 * 4;
constexpr uint32_t SMEM_BYTES = BAR_OFF + 64 + 1024;  // + alignment slack
static_assert(2 * 64 * LDM * 4 <= X_BYTES, "scratch region");
// TMEM columns (all 512): S^T, the master copy of the state in full f32 and the A operand of D2; D2; RD; D1 (later DR, then O2);
// R^T (later D^T)
constexpr uint32_t ST_COL = 0, D2_COL = 128, RD_COL = 256, D1_COL = 384, VT_COL = 448;
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

// A operand from TMEM (lane = row, one 32-bit element per column, K-major), B from shared memory
__device__ __forceinline__ void umma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, p;\n"
      "}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

// ---- 16 x 16 x 16 block products of the triangular inverse: warp-level mma.sync m16n8k8, operands split in two tf32 halves ---------
__device__ __forceinline__ void mma_m16n8k8(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
// c[16 x 8] += A[16 x 16] B[16 x 8]; A, B point at the blocks' origins in matrices of row stride LDM. With A2 == A the left operand is
// -A, with another A2 it is A2 - A. The six tensor-core instructions (two k-steps, three products of the split) are independent.
__device__ __forceinline__ void blk_mma(float (&c)[4], const float* A, const float* A2, const float* B, int lane) {
  const int r = lane >> 2, q = lane & 3;
  float acc[6][4];
#pragma unroll
  for (int ks = 0; ks < 2; ++ks) {
    float a[4], b[2];
    const int o0 = r * LDM + 8 * ks + q, o1 = o0 + 8 * LDM;
    a[0] = A[o0];
    a[1] = A[o1];
    a[2] = A[o0 + 4];
    a[3] = A[o1 + 4];
    if (A2 == A) {
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = -a[i];
    } else if (A2) {
      a[0] = A2[o0] - a[0];
      a[1] = A2[o1] - a[1];
      a[2] = A2[o0 + 4] - a[2];
      a[3] = A2[o1 + 4] - a[3];
    }
    b[0] = B[(8 * ks + q) * LDM + r];
    b[1] = B[(8 * ks + q + 4) * LDM + r];
    uint32_t ah[4], al[4], bh[2], bl[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      ah[i] = cvt_tf32(a[i]);
      al[i] = cvt_tf32(a[i] - u2f(ah[i]));
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      bh[i] = cvt_tf32(b[i]);
      bl[i] = cvt_tf32(b[i] - u2f(bh[i]));
    }
#pragma unroll
    for (int j = 0; j < 3; ++j)
#pragma unroll
      for (int i = 0; i < 4; ++i) acc[3 * ks + j][i] = 0.f;
    mma_m16n8k8(acc[3 * ks + 0], al, bh);
    mma_m16n8k8(acc[3 * ks + 1], ah, bl);
    mma_m16n8k8(acc[3 * ks + 2], ah, bh);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) c[i] += ((acc[0][i] + acc[1][i]) + (acc[3][i] + acc[4][i])) + (acc[2][i] + acc[5][i]);
}
// element (row, col) of a 16 x 8 C fragment held by this lane: c[0], c[1] at (lane / 4, 2 (lane % 4) + {0, 1}); c[2], c[3] eight rows below

// PROF: thread 0 adds the clock cycles of each of the 16 phases of a chunk to prof[0..15] (diagnostics; the reference's chunked
// kernel has the same switch, native/kernels/kernels.cu:1671-1690)
#define GWY_PH(i)                                    \
  if (PROF && tid == 0) {                            \
    const long long now_ = clock64();                \
    pacc[i] += (unsigned long long)(now_ - plast);   \
    plast = now_;                                    \
  }
template <typename T, bool PROF>
__global__ void __launch_bounds__(THREADS, 1)
gdn_wy_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
              const T* __restrict__ conv, int conv_stride,
              const float* __restrict__ gl, const float* __restrict__ beta, const float* __restrict__ seed, float* __restrict__ final_state,
              T* __restrict__ out, const int32_t* __restrict__ cu, int nk, int nv, int* err, unsigned long long* __restrict__ prof) {
  const int head = blockIdx.x, b = blockIdx.y;
  unsigned long long pacc[PROF ? 16 : 1];
  long long plast = 0;
  const long long t_entry = PROF ? clock64() : 0;  // phase 13: kernel entry to the first chunk (allocation, seed, first tiles)
  if (PROF) {
#pragma unroll
    for (int i = 0; i < 16; ++i) pacc[i] = 0;
  }
  const int off = cu[b], len = cu[b + 1] - off;
  const int kh = head / (nv / nk);
  const int tid = threadIdx.x, warp = uniform_warp_idx(), lane = tid & 31;
  // The tensor-core and TMA instructions are issued by the elected lane of a warp that runs the surrounding code as a whole: operands
  // built by the whole warp sit in uniform registers, and the instructions then issue every ~21 cycles instead of every ~57 from
  // a lone thread inside a divergent branch.
  const bool el = elect_one();
  const int wg = warp >> 2, ln = tid & 127;  // warpgroup; TMEM lane / operand row owned by this thread
  const int vcol0 = 2 * nk * DK + head * DV;

  if (len <= 0) {  // nothing to run: the final state is the seed
    if (final_state)
      for (int r = wg * 32; r < wg * 32 + 32; ++r) final_state[(((size_t)b * nv + head) * DK + r) * DV + ln] = seed ? seed[((size_t)head * DK + r) * DV + ln] : 0.f;
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t sbase = raw + pad;
  float* M0 = reinterpret_cast<float*>(smem + X_OFF);  // A, later F^2 (and F^2 - F^3) in the blocks two and three below the diagonal
  float* M1 = M0 + 64 * LDM;                           // X on the diagonal blocks, F below
  float* sc = reinterpret_cast<float*>(smem + SC_OFF);
  const uint32_t bar_kq = sbase + BAR_OFF, bar_a = bar_kq + 8, bar_q = bar_kq + 16, bar_o = bar_kq + 24;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + BAR_OFF + 32);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + BAR_OFF + 36);

  if (tid == 0) {
    mbar_init(bar_kq, 1);
    mbar_init(bar_a, 1);
    mbar_init(bar_q, 1);
    mbar_init(bar_o, 1);
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

  constexpr bool V_TMA = sizeof(T) == 2;  // a 16-bit conv output: the chunk's V tile comes by TMA
  auto load_kq = [&](int t0) {  // called by a whole warp; K/Q tiles and (16-bit storage) the V tile of the chunk at t0
    if (el) mbar_expect_tx(bar_kq, 4 * REG + (V_TMA ? REG : 0));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (el) tma_load_2d(sbase + KQ_OFF + j * REG, &tmK, bar_kq, kh * DK + j * 32, off + t0);
      if (el) tma_load_2d(sbase + KQ_OFF + j * REG + 8192, &tmQ, bar_kq, kh * DK + j * 32, off + t0);
    }
    if (V_TMA) {
      if (el) tma_load_2d(sbase + V_OFF, &tmV, bar_kq, vcol0, off + t0);
      if (el) tma_load_2d(sbase + V_OFF + 8192, &tmV, bar_kq, vcol0 + 64, off + t0);
    }
  };
  // Scalars of the chunk at t0 into set `set` (warp 6: decays, warp 7: beta). A set is rewritten two chunks later, after every thread
  // has passed a barrier that follows its last read.
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

  if (warp == 0) load_kq(0);
  scalars(0, 0);
  // ---- the blocks of T above the diagonal stay zero for the whole kernel ------------------------------------------
#pragma unroll
  for (int i = 0; i < 2; ++i) *reinterpret_cast<float4*>(smem + T_OFF + (uint32_t)(tid + THREADS * i) * 16u) = make_float4(0.f, 0.f, 0.f, 0.f);
  // ---- seed: S^T row of this thread's value column into its TMEM lane, 32 dk columns per warpgroup ----------------------------------
  {
    uint32_t v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = f2u(seed ? seed[((size_t)head * DK + wg * 32 + i) * DV + ln] : 0.f);
    tmem_st32(tlane + ST_COL + wg * 32, v);
    tmem_st_wait();
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  tc_fence_before();

  // operand descriptors of slab 0; a k-step of 8 columns advances the start address by 32 bytes and a slab by its size
  const uint64_t d_kq = umma_desc(sbase + KQ_OFF, 16, 1024), d_ke = umma_desc(sbase + KE_OFF, 16, 1024), d_t = umma_desc(sbase + T_OFF, 16, 1024),
                 d_p = umma_desc(sbase + P_OFF, 16, 1024);
  const int n_chunks = (len + C - 1) / C;
  uint32_t ph_a = 0;
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
    if (PROF && tid == 0 && ci == 0) {
      plast = clock64();
      pacc[13] += (unsigned long long)(plast - t_entry);
    }

    // ---- D1 = [K;Q] K^T ---------------------------------------------------------------------------------------------------------
    ok = mbar_wait(bar_kq, (uint32_t)(ci & 1), abort_flag);  // every thread reads the K tile below
    GWY_PH(0);
    if (warp == 0 && ok) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        if (el) umma_tf32(tmem_base + D1_COL, d_kq + o, d_kq + o, IDESC_N64, kk != 0 ? 1u : 0u);
      }
      if (el) umma_commit_to(bar_a);
    }
    // ---- (exp(G_C-G) K)^T: row dk = ln, 16 tokens per warpgroup, a K-major tf32 operand (while D1 runs) --------------------------------
    if (ok) {
      const uint8_t* kcol = smem + KQ_OFF + (ln >> 5) * REG + (ln & 3) * 4;
      const int c16 = (ln & 31) >> 2;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        float kv[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = wg * BLK + q * 4 + i;
          kv[i] = *reinterpret_cast<const float*>(kcol + t * 128 + ((c16 ^ (t & 7)) << 4));
        }
        const float4 e4 = *reinterpret_cast<const float4*>(sE + wg * BLK + q * 4);
        *reinterpret_cast<float4*>(smem + KE_OFF + (uint32_t)(wg >> 1) * REG + sw_off(ln, (wg & 1) * 4 + q)) =
            tf32x4(kv[0] * e4.x, kv[1] * e4.y, kv[2] * e4.z, kv[3] * e4.w);
      }
    }
    ok = ok && mbar_wait(bar_a, ph_a, abort_flag);
    ph_a ^= 1u;
    ok = __all_sync(0xffffffffu, ok);
    GWY_PH(1);
    tc_fence_after();

    // ---- D1 rows of the key tokens give A (scratch M0), the rows of the query tokens P ---------------------------------------
    // (exponents are clamped to <= 0 and the result selected, so the loops stay branch-free)
    if (ok) {
      uint32_t v[BLK];
      tmem_ld16(tlane + D1_COL + wg * BLK, v);
      tmem_ld_wait();
      const int t = ln & 63;
      const float Gt = sG[t], bt = ln < 64 ? sB[t] : 1.0f;
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 gs = *reinterpret_cast<const float4*>(sG + wg * BLK + q * 4);
        const float ge[4] = {gs.x, gs.y, gs.z, gs.w};
        float pr[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int s = wg * BLK + q * 4 + i;
          const float e = bt * __expf(fminf(Gt - ge[i], 0.f)) * u2f(v[q * 4 + i]);
          pr[i] = (ln < 64 ? s < t : s <= t) ? e : 0.f;
        }
        if (ln < 64)
          *reinterpret_cast<float4*>(M0 + t * LDM + wg * BLK + q * 4) = make_float4(pr[0], pr[1], pr[2], pr[3]);
        else
          *reinterpret_cast<float4*>(smem + P_OFF + (uint32_t)(wg >> 1) * 8192 + sw_off(t, (wg & 1) * 4 + q)) = tf32x4(pr[0], pr[1], pr[2], pr[3]);
      }
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }  // A complete
    GWY_PH(2);

    // ---- X: inverses of the four 16 x 16 diagonal blocks of I + A, one column per thread, in registers ------------------------------
    if (tid < 64) {
      const int bb = tid >> 4, j = tid & 15;
      const float* Ab = M0 + (bb * BLK) * LDM + bb * BLK;
      float x[BLK];
#pragma unroll
      for (int i = 0; i < BLK; ++i) x[i] = i == j ? 1.f : 0.f;
#pragma unroll
      for (int i = 1; i < BLK; ++i) {
        float row[BLK];
#pragma unroll
        for (int q = 0; q < (i + 3) / 4; ++q) {
          const float4 r4 = *reinterpret_cast<const float4*>(Ab + i * LDM + 4 * q);
          row[4 * q] = r4.x; row[4 * q + 1] = r4.y; row[4 * q + 2] = r4.z; row[4 * q + 3] = r4.w;
        }
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int p = 0; p < i; ++p) {
          if (p & 1) acc1 = fmaf(row[p], x[p], acc1);
          else acc0 = fmaf(row[p], x[p], acc0);
        }
        x[i] = i > j ? -(acc0 + acc1) : x[i];
      }
      float* Xb = M1 + (bb * BLK) * LDM + bb * BLK + j;
#pragma unroll
      for (int i = 0; i < BLK; ++i) Xb[i * LDM] = x[i];
    } else if (warp == 12) {
      // ---- meanwhile D2 = S^T [K;Q]^T, not needed before R: issued from a warp that has nothing to do until T is stored (the issuing
      //      thread is held while the tensor core's queue is full) ---------------------------------------------------------------------
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 16; ++kk) {
        const uint64_t o = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        if (el) umma_tf32_ts(tmem_base + D2_COL, tmem_base + ST_COL + kk * 8, d_kq + o, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      if (el) umma_commit_to(bar_q);
    }
    __syncthreads();
    GWY_PH(3);

    // ---- F = X E (six blocks, two 8-column halves each: twelve warps) ------------------------------------------------------------
    const int r8 = lane >> 2, q2 = 2 * (lane & 3);
    if (warp < 12) {
      const int blk = warp >> 1, h = warp & 1;
      const int bi = blk < 1 ? 1 : blk < 3 ? 2 : 3, bj = blk - (bi == 1 ? 0 : bi == 2 ? 1 : 3);
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      blk_mma(c, M1 + (bi * BLK) * LDM + bi * BLK, nullptr, M0 + (bi * BLK) * LDM + bj * BLK + 8 * h, lane);
      float* o = M1 + (bi * BLK + r8) * LDM + bj * BLK + 8 * h + q2;
      *reinterpret_cast<float2*>(o) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2*>(o + 8 * LDM) = make_float2(c[2], c[3]);
    }
    __syncthreads();
    GWY_PH(4);
    // ---- F^2: blocks (2,0) = F21 F10, (3,1) = F32 F21, (3,0) = F31 F10 + F32 F20, into M0 (E is dead) ---------------------------------
    if (warp < 6) {
      const int task = warp >> 1, h = warp & 1;
      const int bi = task == 0 ? 2 : 3, bj = task == 1 ? 1 : 0;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      for (int bk = bj + 1; bk < bi; ++bk) blk_mma(c, M1 + (bi * BLK) * LDM + bk * BLK, nullptr, M1 + (bk * BLK) * LDM + bj * BLK + 8 * h, lane);
      float* o = M0 + (bi * BLK + r8) * LDM + bj * BLK + 8 * h + q2;
      *reinterpret_cast<float2*>(o) = make_float2(c[0], c[1]);
      *reinterpret_cast<float2*>(o + 8 * LDM) = make_float2(c[2], c[3]);
    }
    __syncthreads();
    GWY_PH(5);
    // ---- F^3 has one block, (3,0) = F32 (F^2)20; M0 (3,0) becomes F^2 - F^3 --------------------------------------------------------
    if (warp < 2) {
      const int h = warp;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      blk_mma(c, M1 + (3 * BLK) * LDM + 2 * BLK, nullptr, M0 + (2 * BLK) * LDM + 8 * h, lane);
      float* o = M0 + (3 * BLK + r8) * LDM + 8 * h + q2;
      float2 lo = *reinterpret_cast<float2*>(o), hi = *reinterpret_cast<float2*>(o + 8 * LDM);
      *reinterpret_cast<float2*>(o) = make_float2(lo.x - c[0], lo.y - c[1]);
      *reinterpret_cast<float2*>(o + 8 * LDM) = make_float2(hi.x - c[2], hi.y - c[3]);
    }
    __syncthreads();
    GWY_PH(6);
    // ---- T = (I - F + F^2 - F^3) X: the six blocks below the diagonal (twelve warps) and the diagonal blocks X (four warps), written
    //      as a K-major tf32 operand ---------------------------------------------------------------------------------------------------
    if (warp < 12) {
      const int blk = warp >> 1, h = warp & 1;
      const int bi = blk < 1 ? 1 : blk < 3 ? 2 : 3, bj = blk - (bi == 1 ? 0 : bi == 2 ? 1 : 3);
      const float* F = M1 + (bi * BLK) * LDM + bj * BLK;
      float c[4] = {0.f, 0.f, 0.f, 0.f};
      blk_mma(c, F, bi - bj >= 2 ? M0 + (bi * BLK) * LDM + bj * BLK : F, M1 + (bj * BLK) * LDM + bj * BLK + 8 * h, lane);
      const int s = bj * BLK + 8 * h + q2;  // even: the pair s, s + 1 shares a 16-byte chunk
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int t = bi * BLK + r8 + 8 * hh;
        const uint32_t o = (uint32_t)(s >> 5) * 8192u + sw_off(t, (s & 31) >> 2) + (uint32_t)(s & 3) * 4u;
        *reinterpret_cast<float2*>(smem + T_OFF + o) = make_float2(u2f(cvt_tf32(c[2 * hh])), u2f(cvt_tf32(c[2 * hh + 1])));
      }
    } else {
      const int bb = warp - 12, r = lane >> 1, c0 = (lane & 1) * 8;
      const int t = bb * BLK + r;
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int s = bb * BLK + c0 + 4 * q;
        const float4 x4 = *reinterpret_cast<const float4*>(M1 + t * LDM + s);
        *reinterpret_cast<float4*>(smem + T_OFF + (uint32_t)(s >> 5) * 8192u + sw_off(t, (s & 31) >> 2)) = tf32x4(x4.x, x4.y, x4.z, x4.w);
      }
    }
    // ---- R^T = beta (V^T - Gam (K S)^T): this thread's value column, tokens 16 wg .. 16 wg + 15, into TMEM ------------------------------
    ok = mbar_wait(bar_q, (uint32_t)(ci & 1), abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok) {
      uint32_t x[BLK], v[BLK];
      tmem_ld16(tlane + D2_COL + wg * BLK, x);
      if (V_TMA) {
        const uint8_t* vcol = smem + V_OFF + (ln >> 6) * 8192 + (ln & 7) * 2;
        const int c16 = (ln & 63) >> 3;
#pragma unroll
        for (int i = 0; i < BLK; ++i) {
          const int t = wg * BLK + i;
          v[i] = (uint32_t)(*reinterpret_cast<const uint16_t*>(vcol + t * 128 + ((c16 ^ (t & 7)) << 4))) << 16;  // bf16 -> f32 bits
        }
      } else {
        const T* vp = conv + (size_t)(off + t0) * conv_stride + vcol0 + ln;
#pragma unroll
        for (int i = 0; i < BLK; ++i) {
          const int t = wg * BLK + i;
          const float xv = Ty<T>::ld(vp + (size_t)min(t, nt - 1) * conv_stride);
          v[i] = f2u(t < nt ? xv : 0.f);
        }
      }
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 b4 = *reinterpret_cast<const float4*>(sB + wg * BLK + q * 4);
        const float4 g4 = *reinterpret_cast<const float4*>(sGam + wg * BLK + q * 4);
        v[4 * q + 0] = cvt_tf32(b4.x * (u2f(v[4 * q + 0]) - g4.x * u2f(x[4 * q + 0])));
        v[4 * q + 1] = cvt_tf32(b4.y * (u2f(v[4 * q + 1]) - g4.y * u2f(x[4 * q + 1])));
        v[4 * q + 2] = cvt_tf32(b4.z * (u2f(v[4 * q + 2]) - g4.z * u2f(x[4 * q + 2])));
        v[4 * q + 3] = cvt_tf32(b4.w * (u2f(v[4 * q + 3]) - g4.w * u2f(x[4 * q + 3])));
      }
      tmem_st16(tlane + VT_COL + wg * BLK, v);
      tmem_st_wait();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    GWY_PH(7);

    // ---- DR = R^T T^T; the K/Q/V tiles are free: request the next chunk's -----------------------------------------------------------
    if (warp == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t ob = (uint64_t)(((kk >> 2) * 8192 + (kk & 3) * 32) >> 4);
        if (el) umma_tf32_ts(tmem_base + D1_COL, tmem_base + VT_COL + kk * 8, d_t + ob, IDESC_N64, kk != 0 ? 1u : 0u);
      }
      if (el) umma_commit_to(bar_a);
    } else if (warp == 13 && !last) {
      load_kq(t0 + C);
    }
    ok = mbar_wait(bar_a, ph_a, abort_flag);
    ph_a ^= 1u;
    ok = __all_sync(0xffffffffu, ok);
    GWY_PH(8);
    tc_fence_after();
    // ---- D^T = DR rounded to tf32, over R^T: the A operand of O2 and RD -----------------------------------------------------------
    if (ok) {
      uint32_t u[BLK];
      tmem_ld16(tlane + D1_COL + wg * BLK, u);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < BLK; ++i) u[i] = cvt_tf32(u2f(u[i]));
      tmem_st16(tlane + VT_COL + wg * BLK, u);
      tmem_st_wait();
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    GWY_PH(9);

    // ---- RD = D^T (exp(G_C-G) K), O2 = D^T P^T ---------------------------------------------------------------------------------
    if (warp == 0) {
      tc_fence_after();
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t ob = (uint64_t)(((kk >> 2) * REG + (kk & 3) * 32) >> 4);
        if (el) umma_tf32_ts(tmem_base + RD_COL, tmem_base + VT_COL + kk * 8, d_ke + ob, IDESC_N128, kk != 0 ? 1u : 0u);
      }
      if (el) umma_commit_to(bar_a);
#pragma unroll
      for (int kk = 0; kk < 8; ++kk) {
        const uint64_t op = (uint64_t)(((kk >> 2) * 8192 + (kk & 3) * 32) >> 4);
        if (el) umma_tf32_ts(tmem_base + D1_COL, tmem_base + VT_COL + kk * 8, d_p + op, IDESC_N64, kk != 0 ? 1u : 0u);
      }
      if (el) umma_commit_to(bar_o);
    }
    if (!last) scalars(t0 + C, (ci + 1) & 1);  // meanwhile (warps 6 and 7): scalars of the next chunk
    ok = mbar_wait(bar_a, ph_a, abort_flag);
    ph_a ^= 1u;
    ok = __all_sync(0xffffffffu, ok);
    GWY_PH(10);
    tc_fence_after();
    // ---- state S' = exp(G_C) S + RD in TMEM (or out to the final state); 32 dk columns per warpgroup ------------------------------------
    if (ok) {
      const float gamC = sGam[C - 1];
      uint32_t dl[32], st[32];
      tmem_ld32(tlane + RD_COL + wg * 32, dl);
      tmem_ld32(tlane + ST_COL + wg * 32, st);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) st[i] = f2u(fmaf(gamC, u2f(st[i]), u2f(dl[i])));
      if (!last) {
        tmem_st32(tlane + ST_COL + wg * 32, st);
        tmem_st_wait();
      } else if (final_state) {
        float* fp = final_state + (((size_t)b * nv + head) * DK + wg * 32) * DV + ln;
#pragma unroll
        for (int i = 0; i < 32; ++i) fp[(size_t)i * DV] = u2f(st[i]);
      }
    }
    GWY_PH(11);
    // ---- outputs O[t, vc] = Gam_t (Q S)[t, vc] + (P D)[t, vc]; 16 tokens per warpgroup -----------------------------------------------
    ok = ok && mbar_wait(bar_o, (uint32_t)(ci & 1), abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    tc_fence_after();
    if (ok) {
      T* op = out + (size_t)(off + t0) * nv * DV + (size_t)head * DV + ln;
      const size_t os = (size_t)nv * DV;
      uint32_t qs[BLK], pd[BLK];
      tmem_ld16(tlane + D2_COL + 64 + wg * BLK, qs);
      tmem_ld16(tlane + D1_COL + wg * BLK, pd);
      tmem_ld_wait();
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float4 g4 = *reinterpret_cast<const float4*>(sGam + wg * BLK + q * 4);
        const float ge[4] = {g4.x, g4.y, g4.z, g4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int t = wg * BLK + q * 4 + i;
          st_if<T>(op + (size_t)t * os, fmaf(ge[i], u2f(qs[q * 4 + i]), u2f(pd[q * 4 + i])), t < nt);
        }
      }
    }
    tc_fence_before();
    if (!__syncthreads_and(ok)) { ok = false; break; }
    GWY_PH(12);
  }
  if (PROF && tid == 0 && prof) {
#pragma unroll
    for (int i = 0; i < 16; ++i) atomicAdd(prof + i, pacc[i]);
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

}  // namespace gwy

template <typename T>
cudaError_t gdn_wy_prepare_device() {
  cudaError_t e = cudaFuncSetAttribute(gwy::gdn_wy_kernel<T, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gwy::SMEM_BYTES);
  if (e != cudaSuccess) return e;
  return cudaFuncSetAttribute(gwy::gdn_wy_kernel<T, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gwy::SMEM_BYTES);
}
template cudaError_t gdn_wy_prepare_device<float>();
template cudaError_t gdn_wy_prepare_device<bf16>();

// maps: the three tensor maps of gdn_tc_make_maps (the same 64-row boxes). phases (may be null): 16 device counters that receive the
// clock cycles thread 0 of every CTA spent in each phase of its chunks.
template <typename T>
cudaError_t launch_gdn_wy(const TcTensorMap maps[3], const T* conv, int conv_stride, const float* g, const float* beta, const float* seed,
                          float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int* err, cudaStream_t s, unsigned long long* phases) {
  if (B <= 0) return cudaSuccess;
  if (B > 65535 || nk <= 0 || nv % nk != 0) return cudaErrorInvalidValue;
  dim3 grid(nv, B);
  const CUtensorMap &mq = *reinterpret_cast<const CUtensorMap*>(&maps[0]), &mk = *reinterpret_cast<const CUtensorMap*>(&maps[1]),
                    &mv = *reinterpret_cast<const CUtensorMap*>(&maps[2]);
  if (phases)
    gwy::gdn_wy_kernel<T, true><<<grid, gwy::THREADS, gwy::SMEM_BYTES, s>>>(mq, mk, mv, conv, conv_stride, g, beta, seed, final_state, out, cu, nk, nv, err, phases);
  else
    gwy::gdn_wy_kernel<T, false><<<grid, gwy::THREADS, gwy::SMEM_BYTES, s>>>(mq, mk, mv, conv, conv_stride, g, beta, seed, final_state, out, cu, nk, nv, err, nullptr);
  return cudaGetLastError();
}
template cudaError_t launch_gdn_wy<float>(const TcTensorMap*, const float*, int, const float*, const float*, const float*, float*, float*, const int32_t*, int, int, int, int*, cudaStream_t, unsigned long long*);
template cudaError_t launch_gdn_wy<bf16>(const TcTensorMap*, const bf16*, int, const float*, const float*, const float*, float*, bf16*, const int32_t*, int, int, int, int*, cudaStream_t, unsigned long long*);
