// Chunked gated delta rule with tensor-core contractions (TF32 mma.sync, f32 accumulate), seeded
// from the cached f32 recurrent state.
//
// Same function as the sequential kernel (gdn_recurrent_kernel; reference: gdn_recurrent,
// native/kernels/kernels.cu:834-865 in juanqui/decidra) in the chunked WY form the reference uses
// in gdn_chunked_tc_body (native/kernels/kernels.cu:1671-1933; formulation :1340-1352), chunk C = 32:
//   G_t   = cumulative log decay inside the chunk (inclusive), Gam_t = exp(G_t)
//   A_ts  = beta_t exp(G_t-G_s) (k_t.k_s)            s <  t   (strictly lower)
//   (I+A) D = beta (V - Gam (K S))                    forward substitution, D = per-step deltas
//   P_ts  = exp(G_t-G_s) (q_t.k_s)                   s <= t
//   O     = Gam (Q S) + P D
//   S'    = exp(G_C) S + (exp(G_C-G) K)^T D
// Only differences of cumulative log decays are exponentiated (never ratios of products).
// One CTA = (packed sequence, value head, slice of VC value columns); the state slice
// S[dk=128, VC] stays in shared memory in f32 across chunks. K S, Q S, K K^T, Q K^T, P D and the
// state update run on mma.sync.m16n8k8 TF32; the triangular solve is a right-looking
// substitution with one thread per value column, overlapped with the Q-side products, and the
// next chunk's rows are prefetched into registers while the current chunk is computed.
// K, Q, P and the deltas are rounded to TF32 (cvt.rna) when they are written to shared memory; the
// f32 state is fed to the tensor core as stored (the unit ignores the low mantissa bits), which
// saves one conversion per B fragment in the two state products.
#include "common.cuh"
#include "kernels.h"

namespace gdc {

constexpr int C = 32, DK = 128, LDK = DK + 4, LDA = C + 4;

__device__ __forceinline__ uint32_t tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T, int VC>
__global__ void __launch_bounds__(256)
gdn_chunked_kernel(const float* __restrict__ qf, const float* __restrict__ kf, const T* __restrict__ conv, int conv_stride,
                   const float* __restrict__ gl, const float* __restrict__ beta, const float* __restrict__ seed,
                   float* __restrict__ final_state, T* __restrict__ out, const int32_t* __restrict__ cu, int nk, int nv, int dv) {
  constexpr int LDS = VC + 8;   // row stride of S, D, O tiles
  constexpr int NT = VC / 8;    // n-tiles across the value slice
  extern __shared__ __align__(16) float sm[];
  float* sK = sm;                    // [C][LDK]   tf32-rounded keys
  float* sQ = sK + C * LDK;          // [C][LDK]   tf32-rounded queries
  float* sS = sQ + C * LDK;          // [DK][LDS]  f32 state slice
  float* sD = sS + DK * LDS;         // [C][LDS]   rhs, then deltas
  float* sO = sD + C * LDS;          // [C][LDS]   Gam * (Q S)
  float* sAT = sO + C * LDS;         // [C][LDA]   A transposed: sAT[s][t]
  float* sP = sAT + C * LDA;         // [C][LDA]   P[t][s]
  float* sV = sP + C * LDA;          // [C][VC]
  float* sG = sV + C * VC;           // [C] cumulative log decay
  float* sB = sG + C;                // [C] beta
  float* sE = sB + C;                // [C] exp(G_last - G_t)

  const int slices = dv / VC;
  const int head = blockIdx.x / slices, cbase = (blockIdx.x - head * slices) * VC;
  const int b = blockIdx.y;
  const int off = cu[b], len = cu[b + 1] - off;
  const int kh = head / (nv / nk);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
  const int vcol0 = 2 * nk * DK + head * dv + cbase;

  for (int i = tid; i < DK * VC; i += 256) {
    const int r = i / VC, c = i - r * VC;
    sS[r * LDS + c] = seed ? seed[((size_t)head * DK + r) * dv + cbase + c] : 0.f;
  }

  // register prefetch of one chunk's K/Q rows (4 float4 each per thread) and V values
  constexpr int VPT = C * VC / 256;  // V elements per thread
  float4 pk[4], pq[4];
  float pv[VPT];
  float pg = 0.f, pb = 0.f;
  auto fetch = [&](int t0) {
    const int nt = min(C, len - t0);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + j * 256;
      const int r = i / (DK / 4), c4 = (i - r * (DK / 4)) * 4;
      pk[j] = make_float4(0.f, 0.f, 0.f, 0.f);
      pq[j] = pk[j];
      if (r < nt) {
        const size_t src = ((size_t)(off + t0 + r) * nk + kh) * DK + c4;
        pk[j] = *reinterpret_cast<const float4*>(kf + src);
        pq[j] = *reinterpret_cast<const float4*>(qf + src);
      }
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) {
      const int i = tid + j * 256;
      const int r = i / VC, c = i - r * VC;
      pv[j] = r < nt ? Ty<T>::ld(conv + (size_t)(off + t0 + r) * conv_stride + vcol0 + c) : 0.f;
    }
    if (warp == 0) {
      pg = lane < nt ? gl[(size_t)(off + t0 + lane) * nv + head] : 0.f;
      pb = lane < nt ? beta[(size_t)(off + t0 + lane) * nv + head] : 0.f;
    }
  };
  if (len > 0) fetch(0);

  for (int t0 = 0; t0 < len; t0 += C) {
    const int nt = min(C, len - t0);
    __syncthreads();  // previous chunk done with every buffer; S updated
    // ---- stage the prefetched chunk (rows beyond the sequence are zero: no decay, no update) ------
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + j * 256;
      const int r = i / (DK / 4), c4 = (i - r * (DK / 4)) * 4;
      *reinterpret_cast<float4*>(sK + r * LDK + c4) = make_float4(__uint_as_float(tf32(pk[j].x)), __uint_as_float(tf32(pk[j].y)),
                                                                  __uint_as_float(tf32(pk[j].z)), __uint_as_float(tf32(pk[j].w)));
      *reinterpret_cast<float4*>(sQ + r * LDK + c4) = make_float4(__uint_as_float(tf32(pq[j].x)), __uint_as_float(tf32(pq[j].y)),
                                                                  __uint_as_float(tf32(pq[j].z)), __uint_as_float(tf32(pq[j].w)));
    }
#pragma unroll
    for (int j = 0; j < VPT; ++j) sV[tid + j * 256] = pv[j];
    if (warp == 0) {
      float gv = pg;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, gv, o);
        if (lane >= o) gv += n;
      }
      const float glast = __shfl_sync(0xffffffffu, gv, 31);
      sG[lane] = gv;
      sB[lane] = pb;
      sE[lane] = expf(glast - gv);
    }
    __syncthreads();
    if (t0 + C < len) fetch(t0 + C);  // loads for the next chunk stay in flight during this chunk's math

    // ---- phase 1: warps 0-3: K S -> rhs;  warps 4-7: K K^T -> A^T -------------------------------------
    if (warp < 4) {
      const int mt = warp >> 1, nh = warp & 1;
      float acc[NT / 2][4];
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const int r0 = mt * 16 + g;
#pragma unroll 4
      for (int k0 = 0; k0 < DK; k0 += 8) {
        uint32_t a[4];
        a[0] = __float_as_uint(sK[r0 * LDK + k0 + tig]);
        a[1] = __float_as_uint(sK[(r0 + 8) * LDK + k0 + tig]);
        a[2] = __float_as_uint(sK[r0 * LDK + k0 + tig + 4]);
        a[3] = __float_as_uint(sK[(r0 + 8) * LDK + k0 + tig + 4]);
#pragma unroll
        for (int n = 0; n < NT / 2; ++n) {
          const int n0 = (nh * (NT / 2) + n) * 8 + g;
          mma_tf32(acc[n], a, __float_as_uint(sS[(k0 + tig) * LDS + n0]), __float_as_uint(sS[(k0 + tig + 4) * LDS + n0]));
        }
      }
      const float gam0 = expf(sG[r0]), gam1 = expf(sG[r0 + 8]);
      const float b0 = sB[r0], b1 = sB[r0 + 8];
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) {
        const int c = (nh * (NT / 2) + n) * 8 + 2 * tig;
        sD[r0 * LDS + c] = b0 * (sV[r0 * VC + c] - gam0 * acc[n][0]);
        sD[r0 * LDS + c + 1] = b0 * (sV[r0 * VC + c + 1] - gam0 * acc[n][1]);
        sD[(r0 + 8) * LDS + c] = b1 * (sV[(r0 + 8) * VC + c] - gam1 * acc[n][2]);
        sD[(r0 + 8) * LDS + c + 1] = b1 * (sV[(r0 + 8) * VC + c + 1] - gam1 * acc[n][3]);
      }
    } else {
      // K K^T: 2 m-tiles x 4 n-tiles; warp (4+i): m-tile = i>>1, n-tiles (i&1)*2 .. +1
      const int mt = (warp - 4) >> 1, nh = (warp - 4) & 1;
      float acc[2][4];
#pragma unroll
      for (int n = 0; n < 2; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const int r0 = mt * 16 + g;
      if (!(mt == 0 && nh == 1)) {  // tiles entirely above the diagonal stay zero
#pragma unroll 4
        for (int k0 = 0; k0 < DK; k0 += 8) {
          uint32_t a[4];
          a[0] = __float_as_uint(sK[r0 * LDK + k0 + tig]);
          a[1] = __float_as_uint(sK[(r0 + 8) * LDK + k0 + tig]);
          a[2] = __float_as_uint(sK[r0 * LDK + k0 + tig + 4]);
          a[3] = __float_as_uint(sK[(r0 + 8) * LDK + k0 + tig + 4]);
#pragma unroll
          for (int n = 0; n < 2; ++n) {
            const int n0 = (nh * 2 + n) * 8 + g;
            mma_tf32(acc[n], a, __float_as_uint(sK[n0 * LDK + k0 + tig]), __float_as_uint(sK[n0 * LDK + k0 + tig + 4]));
          }
        }
      }
#pragma unroll
      for (int n = 0; n < 2; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t = r0 + (e >> 1) * 8, sidx = (nh * 2 + n) * 8 + 2 * tig + (e & 1);
          sAT[sidx * LDA + t] = sidx < t ? sB[t] * __expf(sG[t] - sG[sidx]) * acc[n][e] : 0.f;
        }
    }
    __syncthreads();
    // ---- phase 2: warps 0-1 solve (I + A) D = rhs (one thread per value column, right-looking);
    //      meanwhile warps 2-5: Gam (Q S) -> sO, warps 6-7: Q K^T -> P -------------------------------------
    if (tid < VC) {
      float r[C];
#pragma unroll
      for (int t = 0; t < C; ++t) r[t] = sD[t * LDS + tid];
#pragma unroll
      for (int sidx = 0; sidx < C - 1; ++sidx) {
        const float x = r[sidx];
#pragma unroll
        for (int t4 = ((sidx + 1) / 4) * 4; t4 < C; t4 += 4) {
          const float4 av = *reinterpret_cast<const float4*>(sAT + sidx * LDA + t4);
          if (t4 + 0 > sidx) r[t4 + 0] = fmaf(-av.x, x, r[t4 + 0]);
          if (t4 + 1 > sidx) r[t4 + 1] = fmaf(-av.y, x, r[t4 + 1]);
          if (t4 + 2 > sidx) r[t4 + 2] = fmaf(-av.z, x, r[t4 + 2]);
          if (t4 + 3 > sidx) r[t4 + 3] = fmaf(-av.w, x, r[t4 + 3]);
        }
      }
#pragma unroll
      for (int t = 0; t < C; ++t) sD[t * LDS + tid] = __uint_as_float(tf32(r[t]));
    } else if (warp >= 2 && warp < 6) {
      const int mt = (warp - 2) >> 1, nh = (warp - 2) & 1;
      float acc[NT / 2][4];
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const int r0 = mt * 16 + g;
#pragma unroll 4
      for (int k0 = 0; k0 < DK; k0 += 8) {
        uint32_t a[4];
        a[0] = __float_as_uint(sQ[r0 * LDK + k0 + tig]);
        a[1] = __float_as_uint(sQ[(r0 + 8) * LDK + k0 + tig]);
        a[2] = __float_as_uint(sQ[r0 * LDK + k0 + tig + 4]);
        a[3] = __float_as_uint(sQ[(r0 + 8) * LDK + k0 + tig + 4]);
#pragma unroll
        for (int n = 0; n < NT / 2; ++n) {
          const int n0 = (nh * (NT / 2) + n) * 8 + g;
          mma_tf32(acc[n], a, __float_as_uint(sS[(k0 + tig) * LDS + n0]), __float_as_uint(sS[(k0 + tig + 4) * LDS + n0]));
        }
      }
      const float gam0 = expf(sG[r0]), gam1 = expf(sG[r0 + 8]);
#pragma unroll
      for (int n = 0; n < NT / 2; ++n) {
        const int c = (nh * (NT / 2) + n) * 8 + 2 * tig;
        sO[r0 * LDS + c] = gam0 * acc[n][0];
        sO[r0 * LDS + c + 1] = gam0 * acc[n][1];
        sO[(r0 + 8) * LDS + c] = gam1 * acc[n][2];
        sO[(r0 + 8) * LDS + c + 1] = gam1 * acc[n][3];
      }
    } else if (warp >= 6) {
      // Q K^T: warp 6 -> m-tile 0 (n-tiles 0,1), warp 7 -> m-tile 1 (n-tiles 0..3)
      const int mt = warp - 6;
      float acc[4][4];
#pragma unroll
      for (int n = 0; n < 4; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
      const int r0 = mt * 16 + g;
#pragma unroll 4
      for (int k0 = 0; k0 < DK; k0 += 8) {
        uint32_t a[4];
        a[0] = __float_as_uint(sQ[r0 * LDK + k0 + tig]);
        a[1] = __float_as_uint(sQ[(r0 + 8) * LDK + k0 + tig]);
        a[2] = __float_as_uint(sQ[r0 * LDK + k0 + tig + 4]);
        a[3] = __float_as_uint(sQ[(r0 + 8) * LDK + k0 + tig + 4]);
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          if (n < 2 * (mt + 1)) {
            const int n0 = n * 8 + g;
            mma_tf32(acc[n], a, __float_as_uint(sK[n0 * LDK + k0 + tig]), __float_as_uint(sK[n0 * LDK + k0 + tig + 4]));
          }
        }
      }
#pragma unroll
      for (int n = 0; n < 4; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int t = r0 + (e >> 1) * 8, sidx = n * 8 + 2 * tig + (e & 1);
          sP[t * LDA + sidx] = sidx <= t ? __uint_as_float(tf32(__expf(sG[t] - sG[sidx]) * acc[n][e])) : 0.f;
        }
    }
    __syncthreads();
    // ---- phase 3a: O = Gam (Q S) + P D  ([32 x VC], k = 32). warp -> (m-tile, quarter of the n-tiles)
    {
      const int mt = warp & 1, nq = warp >> 1;  // NT/4 n-tiles per warp
      const int r0 = mt * 16 + g;
      float acc[NT / 4][4];
#pragma unroll
      for (int n = 0; n < NT / 4; ++n) {
        const int c = (nq * (NT / 4) + n) * 8 + 2 * tig;
        acc[n][0] = sO[r0 * LDS + c];
        acc[n][1] = sO[r0 * LDS + c + 1];
        acc[n][2] = sO[(r0 + 8) * LDS + c];
        acc[n][3] = sO[(r0 + 8) * LDS + c + 1];
      }
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 8) {
        uint32_t a[4];
        a[0] = __float_as_uint(sP[r0 * LDA + k0 + tig]);
        a[1] = __float_as_uint(sP[(r0 + 8) * LDA + k0 + tig]);
        a[2] = __float_as_uint(sP[r0 * LDA + k0 + tig + 4]);
        a[3] = __float_as_uint(sP[(r0 + 8) * LDA + k0 + tig + 4]);
#pragma unroll
        for (int n = 0; n < NT / 4; ++n) {
          const int n0 = (nq * (NT / 4) + n) * 8 + g;
          mma_tf32(acc[n], a, __float_as_uint(sD[(k0 + tig) * LDS + n0]), __float_as_uint(sD[(k0 + tig + 4) * LDS + n0]));
        }
      }
#pragma unroll
      for (int n = 0; n < NT / 4; ++n) {
        const int c = (nq * (NT / 4) + n) * 8 + 2 * tig;
        T* o0 = out + (size_t)(off + t0 + r0) * (nv * dv) + head * dv + cbase + c;
        T* o1 = out + (size_t)(off + t0 + r0 + 8) * (nv * dv) + head * dv + cbase + c;
        if (r0 < nt) { Ty<T>::st(o0, acc[n][0]); Ty<T>::st(o0 + 1, acc[n][1]); }
        if (r0 + 8 < nt) { Ty<T>::st(o1, acc[n][2]); Ty<T>::st(o1 + 1, acc[n][3]); }
      }
    }
    // ---- phase 3b: S' = exp(G_C) S + (exp(G_C - G) K)^T D  ([128 x VC], k = 32). warp -> m-tile
    {
      const int m0 = warp * 16 + g;
      const float gamC = expf(sG[C - 1]);
      float acc[NT][4];
#pragma unroll
      for (int n = 0; n < NT; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
#pragma unroll
      for (int k0 = 0; k0 < C; k0 += 8) {
        const float e0 = sE[k0 + tig], e1 = sE[k0 + tig + 4];
        uint32_t a[4];
        a[0] = tf32(sK[(k0 + tig) * LDK + m0] * e0);
        a[1] = tf32(sK[(k0 + tig) * LDK + m0 + 8] * e0);
        a[2] = tf32(sK[(k0 + tig + 4) * LDK + m0] * e1);
        a[3] = tf32(sK[(k0 + tig + 4) * LDK + m0 + 8] * e1);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
          const int n0 = n * 8 + g;
          mma_tf32(acc[n], a, __float_as_uint(sD[(k0 + tig) * LDS + n0]), __float_as_uint(sD[(k0 + tig + 4) * LDS + n0]));
        }
      }
      // every warp passed the barrier after phase 2, so nobody still reads S
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int c = n * 8 + 2 * tig;
        float* s0 = sS + m0 * LDS + c;
        float* s1 = sS + (m0 + 8) * LDS + c;
        s0[0] = fmaf(gamC, s0[0], acc[n][0]);
        s0[1] = fmaf(gamC, s0[1], acc[n][1]);
        s1[0] = fmaf(gamC, s1[0], acc[n][2]);
        s1[1] = fmaf(gamC, s1[1], acc[n][3]);
      }
    }
  }
  if (final_state) {
    __syncthreads();
    for (int i = tid; i < DK * VC; i += 256) {
      const int r = i / VC, c = i - r * VC;
      final_state[(((size_t)b * nv + head) * DK + r) * dv + cbase + c] = sS[r * LDS + c];
    }
  }
}

template <int VC>
constexpr size_t smem_bytes() {
  return sizeof(float) * (size_t)(2 * C * LDK + DK * (VC + 8) + 2 * C * (VC + 8) + 2 * C * LDA + C * VC + 3 * C);
}

}  // namespace gdc

bool gdn_chunked_supported(int dk, int dv) { return dk == 128 && dv % 64 == 0; }

template <typename T>
cudaError_t gdn_chunked_prepare_device() {
  CUDA_TRY(cudaFuncSetAttribute(gdc::gdn_chunked_kernel<T, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdc::smem_bytes<64>()));
  CUDA_TRY(cudaFuncSetAttribute(gdc::gdn_chunked_kernel<T, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)gdc::smem_bytes<32>()));
  return cudaSuccess;
}
template cudaError_t gdn_chunked_prepare_device<float>();
template cudaError_t gdn_chunked_prepare_device<bf16>();

template <typename T>
cudaError_t launch_gdn_chunked(const float* qf, const float* kf, const T* conv, int conv_stride, const float* g, const float* beta,
                               const float* seed, float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int dk, int dv,
                               bool few_sequences, cudaStream_t s) {
  if (!gdn_chunked_supported(dk, dv)) return cudaErrorInvalidValue;
  if (few_sequences) {
    dim3 grid(nv * (dv / 32), B);
    gdc::gdn_chunked_kernel<T, 32><<<grid, 256, gdc::smem_bytes<32>(), s>>>(qf, kf, conv, conv_stride, g, beta, seed, final_state, out, cu, nk, nv, dv);
  } else {
    dim3 grid(nv * (dv / 64), B);
    gdc::gdn_chunked_kernel<T, 64><<<grid, 256, gdc::smem_bytes<64>(), s>>>(qf, kf, conv, conv_stride, g, beta, seed, final_state, out, cu, nk, nv, dv);
  }
  return cudaGetLastError();
}
template cudaError_t launch_gdn_chunked<float>(const float*, const float*, const float*, int, const float*, const float*, const float*, float*, float*, const int32_t*, int, int, int, int, int, bool, cudaStream_t);
template cudaError_t launch_gdn_chunked<bf16>(const float*, const float*, const bf16*, int, const float*, const float*, const float*, float*, bf16*, const int32_t*, int, int, int, int, int, bool, cudaStream_t);
