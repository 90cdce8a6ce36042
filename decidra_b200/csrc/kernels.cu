// Bandwidth / latency kernels of the state-once question path (everything except the
// tensor-core GEMM): packing, embedding gather, norms, RoPE, varlen prefix-bidirectional
// attention (plain-FMA form), causal conv, gated-delta-net prepare + recurrence, gated norm,
// residuals, last-row gather + readout, and the seeded weight generator.
//
// Each kernel names the reference code (paths inside juanqui/decidra) whose arithmetic it
// reproduces. All are templated on the storage type T (float for the f32 engine, bf16 for
// the bf16 engine); Ty<T>::rnd() rounds at the points where the reference rounds through bf16.
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.h"

// ---------------------------------------------------------------------------
// Packing: lens[B] -> cu_seqlens[B+1], last_row[B]; then per token (question, position).
// Replaces the host loops of BatchInfo::new / positions / last_row_indices
// (native/src/engine.rs:693-735, 1669-1674) and their H2D copies.
// ---------------------------------------------------------------------------
__global__ void pack_scan_kernel(const int32_t* __restrict__ lens, int B, int32_t* __restrict__ cu,
                                 int32_t* __restrict__ last_row, int* __restrict__ err) {
  __shared__ int part[1024];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int per = (B + nt - 1) / nt;
  const int lo = min(tid * per, B), hi = min(lo + per, B);
  int s = 0;
  bool bad = false;
  for (int i = lo; i < hi; ++i) {
    const int l = lens[i];
    bad |= (l <= 0);
    s += l;
  }
  if (bad) set_err(err, DERR_EMPTY_ITEM);
  part[tid] = s;
  __syncthreads();
  for (int off = 1; off < nt; off <<= 1) {
    int v = tid >= off ? part[tid - off] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  int run = part[tid] - s;  // exclusive prefix
  for (int i = lo; i < hi; ++i) {
    cu[i] = run;
    run += lens[i];
    last_row[i] = run - 1;
  }
  if (tid == nt - 1) cu[B] = part[tid];
}

__global__ void pack_fill_kernel(const int32_t* __restrict__ cu, int B, int total, int pos_start, const int32_t* __restrict__ pos_start_q,
                                 int32_t* __restrict__ tok_q, int32_t* __restrict__ tok_pos) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= total) return;
  int lo = 0, hi = B;  // largest b with cu[b] <= t
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (cu[mid] <= t) lo = mid; else hi = mid;
  }
  tok_q[t] = lo;
  tok_pos[t] = (pos_start_q ? pos_start_q[lo] : pos_start) + (t - cu[lo]);  // per question when the batch mixes states
}

cudaError_t launch_pack(const int32_t* lens, int B, int total, int pos_start, int32_t* cu, int32_t* last_row,
                        int32_t* tok_q, int32_t* tok_pos, int* err, cudaStream_t s, const int32_t* pos_start_q) {
  pack_scan_kernel<<<1, 1024, 0, s>>>(lens, B, cu, last_row, err);
  if (total > 0) pack_fill_kernel<<<(total + 255) / 256, 256, 0, s>>>(cu, B, total, pos_start, pos_start_q, tok_q, tok_pos);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Embedding gather with vocabulary bound check (error word, rows zeroed; never clamps):
// Engine::embed (native/src/engine.rs:1364-1439), embed_gather_bf16 (native/kernels/kernels.cu:84-94).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const uint32_t* __restrict__ ids, T* __restrict__ out, int H,
                             uint32_t vocab, int* __restrict__ err) {
  const int row = blockIdx.x;
  const uint32_t id = ids[row];
  const int n16 = (int)((size_t)H * sizeof(T) / 16);
  uint4* dst = reinterpret_cast<uint4*>(out + (size_t)row * H);
  if (id >= vocab) {
    if (threadIdx.x == 0) set_err(err, DERR_TOKEN_RANGE);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * H);
  for (int i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = src[i];
}

template <typename T>
cudaError_t launch_embed(const T* table, const uint32_t* ids, T* out, int T_rows, int H, int vocab, int* err, cudaStream_t s) {
  embed_kernel<T><<<T_rows, 128, 0, s>>>(table, ids, out, H, (uint32_t)vocab, err);
  return cudaGetLastError();
}
template cudaError_t launch_embed<float>(const float*, const uint32_t*, float*, int, int, int, int*, cudaStream_t);
template cudaError_t launch_embed<bf16>(const bf16*, const uint32_t*, bf16*, int, int, int, int*, cudaStream_t);

// ---------------------------------------------------------------------------
// RMSNorm family. One CTA per row; f32 sum of squares; scale = 1/sqrt(mean+eps);
// out = T(x * scale * (w + zero_centered)).  rmsnorm_bf16 / add_rmsnorm_bf16,
// native/kernels/kernels.cu:378-426. `rows_idx` (optional) gathers input rows
// (gather_rows_bf16, native/kernels/kernels.cu:2351-2361 — the last-row gather is applied
// before the final norm here, which is the same function row by row).
// ---------------------------------------------------------------------------
template <typename T, typename TO>
__global__ void rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ w, TO* __restrict__ out, int cols, float eps,
                               float wofs, const int32_t* __restrict__ rows_idx) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)(rows_idx ? rows_idx[row] : row) * cols;
  TO* orow = out + (size_t)row * cols;
  float ss = 0.f;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    const float v = Ty<T>::ld(xr + j);
    ss += v * v;
  }
  const float mean = block_sum(ss, red) / (float)cols;
  const float scale = 1.0f / sqrtf(mean + eps);
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    const float wv = Ty<T>::ld(w + j) + wofs;
    const float y = Ty<T>::rnd(Ty<T>::ld(xr + j) * scale * wv);
    orow[j] = (TO)y;
  }
}
template <typename T>
__global__ void add_rmsnorm_kernel(const T* __restrict__ x, const T* __restrict__ mix, const T* __restrict__ w,
                                   T* __restrict__ residual, T* __restrict__ out, int cols, float eps) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * cols;
  const T* mr = mix + (size_t)row * cols;
  T* rr = residual + (size_t)row * cols;
  T* orow = out + (size_t)row * cols;
  float ss = 0.f;
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    const float r = Ty<T>::rnd(Ty<T>::ld(xr + j) + Ty<T>::ld(mr + j));
    Ty<T>::st(rr + j, r);
    ss += r * r;
  }
  const float mean = block_sum(ss, red) / (float)cols;
  const float scale = 1.0f / sqrtf(mean + eps);
  for (int j = threadIdx.x; j < cols; j += blockDim.x) {
    const float wv = Ty<T>::ld(w + j) + 1.0f;
    Ty<T>::st(orow + j, Ty<T>::ld(rr + j) * scale * wv);
  }
}


// ---- 16-byte vectorised bf16 forms (cols % 8 == 0, cols <= 8 * 4 * blockDim): one pass, the row is
// held in registers between the sum of squares and the scaling. Same arithmetic as the kernels above.
// SiLU with the hardware exp2/reciprocal approximations (about 2 ulp in f32): used only where the
// result is rounded to bf16 straight away, which hides the difference except on rare rounding ties.
__device__ __forceinline__ float silu_fast(float g) { return __fdividef(g, 1.0f + __expf(-g)); }

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = __low2float(h[i]);
    f[2 * i + 1] = __high2float(h[i]);
  }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 v;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return v;
}

// NVFP4 quantisation of 16 consecutive values held 8 + 8 by two neighbouring lanes (tensor scale 1; same rule as
// quant_nvfp4_act_bf16 / fp4_encode, native/kernels/kernels.cu:222-277, the codes by nvfp4_codes8). Returns this lane's 8 codes; *sb = the group's e4m3 scale byte.
__device__ __forceinline__ uint32_t nvfp4_encode_half_group(const float (&y)[8], uint32_t* sb_out) {
  float m = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(y[j]));
  m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, 1));
  const float sf = fmaxf(m / 6.0f, 1e-10f);
  const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(sf, __NV_SATFINITE, __NV_E4M3);
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(sb, __NV_E4M3);
  const float sd = __half2float(*reinterpret_cast<const __half*>(&hr));
  *sb_out = sb;
  return nvfp4_codes8(y, sd);
}

// QUANT: instead of the bf16 output row, write its NVFP4 image: codes to q_packed [rows, cols/2] and the e4m3 group scales
// into the 128 x 4 tiled layout q_tiled (the operand format of the block-scaled GEMM). cols % 64 == 0.
template <int NV, bool ADD, typename TO, bool QUANT = false>
__global__ void __launch_bounds__(256) rmsnorm_vec_kernel(const bf16* __restrict__ x, const bf16* __restrict__ mix, const bf16* __restrict__ w,
                                                          bf16* __restrict__ residual, TO* __restrict__ out, int cols, float eps, float wofs,
                                                          const int32_t* __restrict__ rows_idx, uint8_t* __restrict__ q_packed = nullptr,
                                                          uint8_t* __restrict__ q_tiled = nullptr) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const size_t in_row = rows_idx ? (size_t)rows_idx[row] : (size_t)row;
  const int n8 = cols >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + in_row * cols);
  const uint4* mr = ADD ? reinterpret_cast<const uint4*>(mix + in_row * cols) : nullptr;
  float v[NV][8];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int i = threadIdx.x + c * 256;
    if (i < n8) {
      unpack8(xr[i], v[c]);
      if (ADD) {
        float m[8];
        unpack8(mr[i], m);
#pragma unroll
        for (int j = 0; j < 8; ++j) v[c][j] = Ty<bf16>::rnd(v[c][j] + m[j]);
        reinterpret_cast<uint4*>(residual + (size_t)row * cols)[i] = pack8(v[c]);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += v[c][j] * v[c][j];
    }
  }
  const float mean = block_sum(ss, red) / (float)cols;
  const float scale = 1.0f / sqrtf(mean + eps);
  const uint4* wr = reinterpret_cast<const uint4*>(w);
#pragma unroll
  for (int c = 0; c < NV; ++c) {
    const int i = threadIdx.x + c * 256;
    if constexpr (QUANT) {  // every lane takes part in the pair exchange; lanes beyond the row carry zeros and store nothing
      float y[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (i < n8) {
        float wv[8];
        unpack8(wr[i], wv);
#pragma unroll
        for (int j = 0; j < 8; ++j) y[j] = Ty<bf16>::rnd(v[c][j] * scale * (wv[j] + wofs));
      }
      uint32_t sb;
      const uint32_t codes = nvfp4_encode_half_group(y, &sb);
      if (i < n8) {
        reinterpret_cast<uint32_t*>(q_packed + (size_t)row * (cols >> 1))[i] = codes;
        if ((i & 1) == 0) {
          const int g = i >> 1;  // group of 16 along the row
          q_tiled[((size_t)(row >> 7) * (cols >> 6) + (g >> 2)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (g & 3)] = (uint8_t)sb;
        }
      }
    } else if (i < n8) {
      float wv[8], y[8];
      unpack8(wr[i], wv);
#pragma unroll
      for (int j = 0; j < 8; ++j) y[j] = Ty<bf16>::rnd(v[c][j] * scale * (wv[j] + wofs));
      if constexpr (sizeof(TO) == 2) {
        reinterpret_cast<uint4*>(out + (size_t)row * cols)[i] = pack8(y);
      } else {
        float4* o = reinterpret_cast<float4*>(out + (size_t)row * cols + (size_t)i * 8);
        o[0] = make_float4(y[0], y[1], y[2], y[3]);
        o[1] = make_float4(y[4], y[5], y[6], y[7]);
      }
    }
  }
}
static inline bool vec_norm_ok(int cols) { return (cols % 8) == 0 && cols <= 8 * 4 * 256; }

template <typename T>
cudaError_t launch_rmsnorm(const T* x, const T* w, T* out, int rows, int cols, float eps, bool zero_centered, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if (vec_norm_ok(cols)) {
      rmsnorm_vec_kernel<4, false, bf16><<<rows, 256, 0, s>>>(x, nullptr, w, nullptr, out, cols, eps, zero_centered ? 1.0f : 0.0f, nullptr);
      return cudaGetLastError();
    }
  }
  rmsnorm_kernel<T, T><<<rows, 256, 0, s>>>(x, w, out, cols, eps, zero_centered ? 1.0f : 0.0f, nullptr);
  return cudaGetLastError();
}
// The two norms that feed a GEMM, writing that GEMM's NVFP4 operand instead of bf16 (bf16 engines; cols % 64 == 0, cols <= 8192).
cudaError_t launch_rmsnorm_nvfp4(const bf16* x, const bf16* w, uint8_t* q_packed, uint8_t* q_tiled, int rows, int cols, float eps, cudaStream_t s) {
  if ((cols % 64) != 0 || !vec_norm_ok(cols)) return cudaErrorInvalidValue;
  rmsnorm_vec_kernel<4, false, bf16, true><<<rows, 256, 0, s>>>(x, nullptr, w, nullptr, nullptr, cols, eps, 1.0f, nullptr, q_packed, q_tiled);
  return cudaGetLastError();
}
cudaError_t launch_add_rmsnorm_nvfp4(const bf16* x, const bf16* mix, const bf16* w, bf16* residual, uint8_t* q_packed, uint8_t* q_tiled, int rows,
                                     int cols, float eps, cudaStream_t s) {
  if ((cols % 64) != 0 || !vec_norm_ok(cols)) return cudaErrorInvalidValue;
  rmsnorm_vec_kernel<4, true, bf16, true><<<rows, 256, 0, s>>>(x, mix, w, residual, nullptr, cols, eps, 1.0f, nullptr, q_packed, q_tiled);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_add_rmsnorm(const T* x, const T* mix, const T* w, T* residual, T* out, int rows, int cols, float eps, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if (vec_norm_ok(cols)) {
      rmsnorm_vec_kernel<4, true, bf16><<<rows, 256, 0, s>>>(x, mix, w, residual, out, cols, eps, 1.0f, nullptr);
      return cudaGetLastError();
    }
  }
  add_rmsnorm_kernel<T><<<rows, 256, 0, s>>>(x, mix, w, residual, out, cols, eps);
  return cudaGetLastError();
}
// Final norm of the gathered last rows, widened to f32 for the readout
// (native/src/engine.rs:4968-4975).
template <typename T>
cudaError_t launch_final_norm_rows(const T* x, const T* w, float* out, const int32_t* rows_idx, int B, int cols, float eps, cudaStream_t s) {
  if constexpr (sizeof(T) == 2) {
    if (vec_norm_ok(cols)) {
      rmsnorm_vec_kernel<4, false, float><<<B, 256, 0, s>>>(x, nullptr, w, nullptr, out, cols, eps, 1.0f, rows_idx);
      return cudaGetLastError();
    }
  }
  rmsnorm_kernel<T, float><<<B, 256, 0, s>>>(x, w, out, cols, eps, 1.0f, rows_idx);
  return cudaGetLastError();
}
#define INST_NORM(T)                                                                                                   \
  template cudaError_t launch_rmsnorm<T>(const T*, const T*, T*, int, int, float, bool, cudaStream_t);                  \
  template cudaError_t launch_add_rmsnorm<T>(const T*, const T*, const T*, T*, T*, int, int, float, cudaStream_t);      \
  template cudaError_t launch_final_norm_rows<T>(const T*, const T*, float*, const int32_t*, int, int, float, cudaStream_t);
INST_NORM(float)
INST_NORM(bf16)

// Gated RMSNorm, one warp per (token, value head) row of `cols` = dv:
// n = T(x*scale); y = T(n*w) (weight not zero-centred); out = T(y * T(silu(z))).
// rmsnorm_gated_bf16, native/kernels/kernels.cu:430-455. z is read with a row stride
// because it lives inside the fused input-projection output.
template <typename T>
__global__ void rmsnorm_gated_kernel(const T* __restrict__ x, const T* __restrict__ z, int z_stride, const T* __restrict__ w,
                                     T* __restrict__ out, int rows, int heads, int cols, float eps) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const int t = row / heads, h = row - t * heads;
  const T* xr = x + (size_t)row * cols;
  const T* zr = z + (size_t)t * z_stride + (size_t)h * cols;
  T* orow = out + (size_t)row * cols;
  float ss = 0.f;
  for (int j = lane; j < cols; j += 32) {
    const float v = Ty<T>::ld(xr + j);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)cols + eps);
  for (int j = lane; j < cols; j += 32) {
    const float normed = Ty<T>::rnd(Ty<T>::ld(xr + j) * scale);
    const float scaled = Ty<T>::rnd(normed * Ty<T>::ld(w + j));
    const float g = Ty<T>::ld(zr + j);
    Ty<T>::st(orow + j, scaled * Ty<T>::rnd(silu_f(g)));
  }
}
// 16 values (bf16-representable) -> e4m3 scale byte and 16 e2m1 codes in two words; the rule of quant_nvfp4_act_bf16 / fp4_encode
// (native/kernels/kernels.cu:222-277) with tensor scale 1; the codes by nvfp4_codes8.
__device__ __forceinline__ void nvfp4_encode_group16(const float (&v)[16], uint32_t& c0, uint32_t& c1, uint32_t& sb_out) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
  const float sf = fmaxf(m / 6.0f, 1e-10f);
  const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(sf, __NV_SATFINITE, __NV_E4M3);
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(sb, __NV_E4M3);
  const float sd = __half2float(*reinterpret_cast<const __half*>(&hr));
  sb_out = sb;
  c0 = nvfp4_codes8(&v[0], sd);
  c1 = nvfp4_codes8(&v[8], sd);
}

// bf16, cols == 128: 8 lanes per row, 16 consecutive elements per lane (16-byte loads and stores); same arithmetic.
// QUANT: instead of the bf16 rows, their NVFP4 image as the out-projection's operand: a lane's 16 outputs are one scale group;
// codes to q_packed [tokens, heads * 64] bytes, scale bytes into the 128 x 4 tiled layout of the [tokens, heads * 128] matrix.
template <bool QUANT>
__global__ void __launch_bounds__(256) rmsnorm_gated_vec128_kernel(const bf16* __restrict__ x, const bf16* __restrict__ z, int z_stride,
                                                                    const bf16* __restrict__ w, bf16* __restrict__ out, int rows, int heads,
                                                                    float eps, uint8_t* __restrict__ q_packed = nullptr,
                                                                    uint8_t* __restrict__ q_tiled = nullptr) {
  // 8 lanes per row, 16 consecutive elements (two 16-byte vectors) per lane: three shuffle steps per row instead of five
  const int row = blockIdx.x * 32 + (threadIdx.x >> 3);
  const int sub = threadIdx.x & 7;
  const bool live = row < rows;
  const int r = live ? row : rows - 1;  // every lane stays in the shuffles; rows past the end recompute the last row and store nothing
  const int t = r / heads, h = r - t * heads;
  const uint4* xp = reinterpret_cast<const uint4*>(x + (size_t)r * 128) + sub * 2;
  const uint4* zp = reinterpret_cast<const uint4*>(z + (size_t)t * z_stride + (size_t)h * 128) + sub * 2;
  const uint4* wp = reinterpret_cast<const uint4*>(w) + sub * 2;
  float xf[16], zf[16], wf[16];
  unpack8(xp[0], *reinterpret_cast<float(*)[8]>(&xf[0]));
  unpack8(xp[1], *reinterpret_cast<float(*)[8]>(&xf[8]));
  unpack8(zp[0], *reinterpret_cast<float(*)[8]>(&zf[0]));
  unpack8(zp[1], *reinterpret_cast<float(*)[8]>(&zf[8]));
  unpack8(wp[0], *reinterpret_cast<float(*)[8]>(&wf[0]));
  unpack8(wp[1], *reinterpret_cast<float(*)[8]>(&wf[8]));
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 16; ++j) ss += xf[j] * xf[j];
#pragma unroll
  for (int o = 1; o < 8; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float scale = 1.0f / sqrtf(ss / 128.0f + eps);
  float y[16];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const float normed = Ty<bf16>::rnd(xf[j] * scale);
    const float scaled = Ty<bf16>::rnd(normed * wf[j]);
    y[j] = scaled * Ty<bf16>::rnd(silu_fast(zf[j]));
  }
  if constexpr (QUANT) {
    float v[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) v[j] = Ty<bf16>::rnd(y[j]);
    uint32_t c0, c1, sb;
    nvfp4_encode_group16(v, c0, c1, sb);
    if (live) {
      const int K = heads * 128, g = h * 8 + sub;  // scale group of this lane inside the token's row
      *reinterpret_cast<uint2*>(q_packed + (size_t)t * (K >> 1) + (size_t)g * 8) = make_uint2(c0, c1);
      q_tiled[((size_t)(t >> 7) * (K >> 6) + (g >> 2)) * 512 + (t & 31) * 16 + ((t & 127) >> 5) * 4 + (g & 3)] = (uint8_t)sb;
    }
  } else if (live) {
    uint4* op = reinterpret_cast<uint4*>(out + (size_t)row * 128) + sub * 2;
    op[0] = pack8(*reinterpret_cast<float(*)[8]>(&y[0]));
    op[1] = pack8(*reinterpret_cast<float(*)[8]>(&y[8]));
  }
}

template <typename T>
cudaError_t launch_rmsnorm_gated(const T* x, const T* z, int z_stride, const T* w, T* out, int tokens, int heads, int cols, float eps, cudaStream_t s) {
  const int rows = tokens * heads;
  if constexpr (sizeof(T) == 2) {
    if (cols == 128 && rows > 0 && (z_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(z) % 16) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0 &&
        (reinterpret_cast<uintptr_t>(w) % 16) == 0 && (reinterpret_cast<uintptr_t>(out) % 16) == 0) {
      rmsnorm_gated_vec128_kernel<false><<<(rows + 31) / 32, 256, 0, s>>>(x, z, z_stride, w, out, rows, heads, eps);
      return cudaGetLastError();
    }
  }
  rmsnorm_gated_kernel<T><<<(rows + 7) / 8, 256, 0, s>>>(x, z, z_stride, w, out, rows, heads, cols, eps);
  return cudaGetLastError();
}
// The gated norm writing the out-projection's NVFP4 operand (bf16 inputs, value heads of 128; heads * 128 a multiple of 64).
cudaError_t launch_rmsnorm_gated_nvfp4(const bf16* x, const bf16* z, int z_stride, const bf16* w, uint8_t* q_packed, uint8_t* q_tiled, int tokens, int heads,
                                       float eps, cudaStream_t s) {
  const int rows = tokens * heads;
  if (rows <= 0) return cudaSuccess;
  if ((z_stride % 8) || (reinterpret_cast<uintptr_t>(z) % 16) || (reinterpret_cast<uintptr_t>(x) % 16) || (reinterpret_cast<uintptr_t>(w) % 16)) return cudaErrorInvalidValue;
  rmsnorm_gated_vec128_kernel<true><<<(rows + 31) / 32, 256, 0, s>>>(x, z, z_stride, w, nullptr, rows, heads, eps, q_packed, q_tiled);
  return cudaGetLastError();
}
template cudaError_t launch_rmsnorm_gated<float>(const float*, const float*, int, const float*, float*, int, int, int, float, cudaStream_t);
template cudaError_t launch_rmsnorm_gated<bf16>(const bf16*, const bf16*, int, const bf16*, bf16*, int, int, int, float, cudaStream_t);

// ---------------------------------------------------------------------------
// Elementwise: residual add (add_bf16, kernels.cu:485-490) and SwiGLU over the
// tile-interleaved gate/up GEMM output (silu_mul_bf16, kernels.cu:492-501).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Ty<T>::st(out + i, Ty<T>::ld(a + i) + Ty<T>::ld(b + i));
}
template <typename T>
cudaError_t launch_add(const T* a, const T* b, T* out, size_t n, cudaStream_t s) {
  add_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, b, out, n);
  return cudaGetLastError();
}
template cudaError_t launch_add<float>(const float*, const float*, float*, size_t, cudaStream_t);
template cudaError_t launch_add<bf16>(const bf16*, const bf16*, bf16*, size_t, cudaStream_t);

// gu: [T, gu_stride] where each 256-column tile holds 128 gate then 128 up columns.
template <typename T>
__global__ void silu_mul_interleaved_kernel(const T* __restrict__ gu, int gu_stride, T* __restrict__ out, int I, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t t = i / I;
  const int c = (int)(i - t * I);
  const T* row = gu + t * gu_stride + (size_t)(c >> 7) * 256 + (c & 127);
  const float g = Ty<T>::ld(row), u = Ty<T>::ld(row + 128);
  Ty<T>::st(out + i, Ty<T>::rnd(silu_f(g)) * u);
}
template <typename T>
cudaError_t launch_silu_mul_interleaved(const T* gu, int gu_stride, T* out, int tokens, int I, cudaStream_t s) {
  const size_t n = (size_t)tokens * I;
  silu_mul_interleaved_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(gu, gu_stride, out, I, n);
  return cudaGetLastError();
}
template cudaError_t launch_silu_mul_interleaved<float>(const float*, int, float*, int, int, cudaStream_t);
template cudaError_t launch_silu_mul_interleaved<bf16>(const bf16*, int, bf16*, int, int, cudaStream_t);

template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ g, const T* __restrict__ u, T* __restrict__ out, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Ty<T>::st(out + i, Ty<T>::rnd(silu_f(Ty<T>::ld(g + i))) * Ty<T>::ld(u + i));
}
template <typename T>
cudaError_t launch_silu_mul(const T* g, const T* u, T* out, size_t n, cudaStream_t s) {
  silu_mul_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(g, u, out, n);
  return cudaGetLastError();
}
template cudaError_t launch_silu_mul<float>(const float*, const float*, float*, size_t, cudaStream_t);
template cudaError_t launch_silu_mul<bf16>(const bf16*, const bf16*, bf16*, size_t, cudaStream_t);

// ---------------------------------------------------------------------------
// split_q_gate + head RMSNorm(1+w) + partial NeoX RoPE, one warp per (token, head).
// split_q_gate_bf16 / rmsnorm_bf16 / rope_bf16: native/kernels/kernels.cu:516-557, 406-426.
// q heads are read from the fused projection [T, *, 2*hd] (first hd of each head), k heads
// from [T, kv, hd]; both with a row stride. cos/sin are tables [max_pos, rhalf] in T
// (host-built exactly like Engine::rope_tables_positions, native/src/engine.rs:1619-1643).
// ---------------------------------------------------------------------------
template <typename T, int HD>
__global__ void qk_norm_rope_kernel(const T* __restrict__ qg, int qg_stride, const T* __restrict__ kraw, int k_stride,
                                    const T* __restrict__ qw, const T* __restrict__ kw, const T* __restrict__ cos_t,
                                    const T* __restrict__ sin_t, const int32_t* __restrict__ positions, int pos_base,
                                    int max_pos, T* __restrict__ q, T* __restrict__ k, int k_out_stride, int tokens,
                                    int heads, int kv, int rhalf, float eps, int* __restrict__ err) {
  constexpr int V = HD / 32;
  __shared__ float sh[8][HD];
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int idx = blockIdx.x * 8 + wi;
  const int slots = heads + kv;
  if (idx >= tokens * slots) return;
  const int t = idx / slots, hs = idx - t * slots;
  const T* src;
  const T* w;
  T* dst;
  if (hs < heads) {
    src = qg + (size_t)t * qg_stride + (size_t)hs * 2 * HD;
    w = qw;
    dst = q + ((size_t)t * heads + hs) * HD;
  } else {
    src = kraw + (size_t)t * k_stride + (size_t)(hs - heads) * HD;
    w = kw;
    dst = k + (size_t)t * k_out_stride + (size_t)(hs - heads) * HD;
  }
  float v[V];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    v[i] = Ty<T>::ld(src + lane * V + i);
    ss += v[i] * v[i];
  }
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
  for (int i = 0; i < V; ++i) {
    v[i] = Ty<T>::rnd(v[i] * scale * (Ty<T>::ld(w + lane * V + i) + 1.0f));
    sh[wi][lane * V + i] = v[i];
  }
  __syncwarp();
  int pos = positions ? positions[t] : pos_base + t;
  if (pos < 0 || pos >= max_pos) {
    if (lane == 0) set_err(err, DERR_POSITION_RANGE);
    pos = 0;
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    const int d = lane * V + i;
    float y = v[i];
    if (d < 2 * rhalf) {
      const int f = d < rhalf ? d : d - rhalf;
      const float c = Ty<T>::ld(cos_t + (size_t)pos * rhalf + f);
      const float s = Ty<T>::ld(sin_t + (size_t)pos * rhalf + f);
      const float a = sh[wi][f], b = sh[wi][f + rhalf];
      if (d < rhalf)
        y = Ty<T>::rnd(__fsub_rn(Ty<T>::rnd(__fmul_rn(a, c)), Ty<T>::rnd(__fmul_rn(b, s))));
      else
        y = Ty<T>::rnd(__fadd_rn(Ty<T>::rnd(__fmul_rn(b, c)), Ty<T>::rnd(__fmul_rn(a, s))));
    }
    Ty<T>::st(dst + d, y);
  }
}

// bf16, head_dim 256: lane l owns dims 8l..8l+7 (one 16-byte load and store per lane); the rotation partner (dim +- rhalf) sits
// rhalf/8 lanes away and comes by shuffle. Same arithmetic and rounding points as the generic kernel.
__global__ void __launch_bounds__(256) qk_norm_rope_vec256_kernel(const bf16* __restrict__ qg, int qg_stride, const bf16* __restrict__ kraw,
                                                                  int k_stride, const bf16* __restrict__ qw, const bf16* __restrict__ kw,
                                                                  const bf16* __restrict__ cos_t, const bf16* __restrict__ sin_t,
                                                                  const int32_t* __restrict__ positions, int pos_base, int max_pos,
                                                                  bf16* __restrict__ q, bf16* __restrict__ k, int k_out_stride, int tokens,
                                                                  int heads, int kv, int rhalf, float eps, int* __restrict__ err) {
  constexpr int HD = 256;
  const int wi = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int idx = blockIdx.x * 8 + wi;
  const int slots = heads + kv;
  if (idx >= tokens * slots) return;
  const int t = idx / slots, hs = idx - t * slots;
  const bf16* src;
  const bf16* w;
  bf16* dst;
  if (hs < heads) {
    src = qg + (size_t)t * qg_stride + (size_t)hs * 2 * HD;
    w = qw;
    dst = q + ((size_t)t * heads + hs) * HD;
  } else {
    src = kraw + (size_t)t * k_stride + (size_t)(hs - heads) * HD;
    w = kw;
    dst = k + (size_t)t * k_out_stride + (size_t)(hs - heads) * HD;
  }
  float v[8], wv[8];
  unpack8(reinterpret_cast<const uint4*>(src)[lane], v);
  unpack8(reinterpret_cast<const uint4*>(w)[lane], wv);
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
  ss = warp_sum(ss);
  const float scale = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = Ty<bf16>::rnd(v[i] * scale * (wv[i] + 1.0f));
  int pos = positions ? positions[t] : pos_base + t;
  if (pos < 0 || pos >= max_pos) {
    if (lane == 0) set_err(err, DERR_POSITION_RANGE);
    pos = 0;
  }
  const int rl = rhalf >> 3;  // lanes per rotary half
  const bool lo = lane < rl, rot = lane < 2 * rl;
  const int partner = rot ? (lo ? lane + rl : lane - rl) : lane;
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = __shfl_sync(0xffffffffu, v[i], partner);
  if (rot) {
    float c[8], sn[8];
    const int f0 = (lo ? lane : lane - rl) * 8;
    unpack8(*reinterpret_cast<const uint4*>(cos_t + (size_t)pos * rhalf + f0), c);
    unpack8(*reinterpret_cast<const uint4*>(sin_t + (size_t)pos * rhalf + f0), sn);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // first half: a = own, b = partner: a c - b s; second half: a = partner, b = own: b c + a s. Both are own * c -/+ partner * s;
      // a - b and a + (-b) are the same sum, so the halves share one instruction stream instead of diverging
      const float bs = Ty<bf16>::rnd(__fmul_rn(o[i], sn[i]));
      v[i] = Ty<bf16>::rnd(__fadd_rn(Ty<bf16>::rnd(__fmul_rn(v[i], c[i])), lo ? -bs : bs));
    }
  }
  reinterpret_cast<uint4*>(dst)[lane] = pack8(v);
}

template <typename T>
cudaError_t launch_qk_norm_rope(const T* qg, int qg_stride, const T* kraw, int k_stride, const T* qw, const T* kw, const T* cos_t,
                                const T* sin_t, const int32_t* positions, int pos_base, int max_pos, T* q, T* k, int k_out_stride,
                                int tokens, int heads, int kv, int hd, int rotary_dim, float eps, int* err, cudaStream_t s) {
  const int n = tokens * (heads + kv);
  const int grid = (n + 7) / 8;
  if constexpr (sizeof(T) == 2) {
    const int rh = rotary_dim / 2;
    auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) % 16) == 0; };
    if (hd == 256 && (rh % 8) == 0 && rh <= 128 && (qg_stride % 8) == 0 && (k_stride % 8) == 0 && (k_out_stride % 8) == 0 && al16(qg) && al16(kraw) &&
        al16(qw) && al16(kw) && al16(cos_t) && al16(sin_t) && al16(q) && al16(k)) {
      qk_norm_rope_vec256_kernel<<<grid, 256, 0, s>>>(qg, qg_stride, kraw, k_stride, qw, kw, cos_t, sin_t, positions, pos_base, max_pos, q, k,
                                                      k_out_stride, tokens, heads, kv, rh, eps, err);
      return cudaGetLastError();
    }
  }
#define QK_CASE(HD_)                                                                                                     \
  case HD_:                                                                                                              \
    qk_norm_rope_kernel<T, HD_><<<grid, 256, 0, s>>>(qg, qg_stride, kraw, k_stride, qw, kw, cos_t, sin_t, positions,     \
                                                     pos_base, max_pos, q, k, k_out_stride, tokens, heads, kv,           \
                                                     rotary_dim / 2, eps, err);                                         \
    break;
  switch (hd) {
    QK_CASE(64)
    QK_CASE(128)
    QK_CASE(256)
    default: return cudaErrorInvalidValue;
  }
#undef QK_CASE
  return cudaGetLastError();
}
template cudaError_t launch_qk_norm_rope<float>(const float*, int, const float*, int, const float*, const float*, const float*, const float*, const int32_t*, int, int, float*, float*, int, int, int, int, int, int, float, int*, cudaStream_t);
template cudaError_t launch_qk_norm_rope<bf16>(const bf16*, int, const bf16*, int, const bf16*, const bf16*, const bf16*, const bf16*, const int32_t*, int, int, bf16*, bf16*, int, int, int, int, int, int, float, int*, cudaStream_t);

// ---------------------------------------------------------------------------
// Varlen prefix-bidirectional attention, plain-FMA form: one warp per (token, head), keys
// streamed four at a time with an online softmax. Each packed question attends to
// [state K/V (n_state rows) || its own K/V rows]; no causal mask. Output is multiplied by
// the sigmoid output gate when gate_qg is given.
//   Engine::full_attention_batch cascade branch (native/src/engine.rs:1985-2042),
//   fi_prefill_bf16_ext (native/third_party/flashinfer/fi_prefill.cu:161-173; scale 1/sqrt(hd),
//   GQA group heads/kv, probabilities rounded to the storage type before P.V),
//   sigmoid_gate_bf16 (native/kernels/kernels.cu:504-512).
// split > 0: single sequence [state || question] with the block-cascade mask of
//   block_cascade_mask (native/src/engine.rs:490-504): rows < split see keys < split.
// ---------------------------------------------------------------------------
template <typename T, int HD>
__global__ void attn_fma_kernel(const T* __restrict__ q, const T* __restrict__ k_own, int k_stride, const T* __restrict__ v_own,
                                int v_stride, const T* __restrict__ k_state, const T* __restrict__ v_state, int n_state,
                                const T* __restrict__ gate_qg, int qg_stride, T* __restrict__ out,
                                const int32_t* __restrict__ cu, const int32_t* __restrict__ tok_q, int tokens, int heads, int kv,
                                int split, int tok_base) {
  constexpr int V = HD / 32;
  const int idx = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (idx >= tokens * heads) return;
  const int lane = threadIdx.x & 31;
  const int t = idx / heads, h = idx - t * heads;
  const int kh = h / (heads / kv);
  const int qi = tok_q ? tok_q[t] : 0;
  const int off_packed = cu ? cu[qi] : 0;
  int len = cu ? cu[qi + 1] - off_packed : tokens;
  const int off = off_packed - tok_base;  // tok_base: packed index of row 0 when q/k/v/out/tok_q point into a larger batch
  if (split > 0 && t < split) len = split;
  const float scale = 1.0f / sqrtf((float)HD);
  float qv[V], acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    qv[i] = Ty<T>::ld(q + ((size_t)t * heads + h) * HD + lane * V + i);
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int nk = n_state + len;
  for (int j0 = 0; j0 < nk; j0 += 4) {
    float sc[4];
    const T* vp[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      float d = 0.f;
      vp[u] = nullptr;
      if (j < nk) {
        const T* kp;
        if (j < n_state) {
          kp = k_state + ((size_t)j * kv + kh) * HD;
          vp[u] = v_state + ((size_t)j * kv + kh) * HD;
        } else {
          kp = k_own + (size_t)(off + j - n_state) * k_stride + (size_t)kh * HD;
          vp[u] = v_own + (size_t)(off + j - n_state) * v_stride + (size_t)kh * HD;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) d += qv[i] * Ty<T>::ld(kp + lane * V + i);
      }
      sc[u] = d;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
      for (int u = 0; u < 4; ++u) sc[u] += __shfl_xor_sync(0xffffffffu, sc[u], o);
    }
    float mx = m;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      sc[u] = (j0 + u < nk) ? sc[u] * scale : -INFINITY;
      mx = fmaxf(mx, sc[u]);
    }
    const float corr = expf(m - mx);
    l *= corr;
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] *= corr;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u < nk) {
        const float p = Ty<T>::rnd(expf(sc[u] - mx));
        l += p;
#pragma unroll
        for (int i = 0; i < V; ++i) acc[i] += p * Ty<T>::ld(vp[u] + lane * V + i);
      }
    }
    m = mx;
  }
  const float inv = 1.0f / l;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    float o = Ty<T>::rnd(acc[i] * inv);
    if (gate_qg) {
      const float g = Ty<T>::ld(gate_qg + (size_t)t * qg_stride + (size_t)h * 2 * HD + HD + lane * V + i);
      o = o * Ty<T>::rnd(sigmoid_f(g));
    }
    Ty<T>::st(out + ((size_t)t * heads + h) * HD + lane * V + i, o);
  }
}

template <typename T>
cudaError_t launch_attn_fma(const T* q, const T* k_own, int k_stride, const T* v_own, int v_stride, const T* k_state,
                            const T* v_state, int n_state, const T* gate_qg, int qg_stride, T* out, const int32_t* cu,
                            const int32_t* tok_q, int tokens, int heads, int kv, int hd, int split, cudaStream_t s, int tok_base) {
  const int n = tokens * heads;
  const int grid = (n + 3) / 4;
#define AT_CASE(HD_)                                                                                                      \
  case HD_:                                                                                                               \
    attn_fma_kernel<T, HD_><<<grid, 128, 0, s>>>(q, k_own, k_stride, v_own, v_stride, k_state, v_state, n_state, gate_qg, \
                                                 qg_stride, out, cu, tok_q, tokens, heads, kv, split, tok_base);         \
    break;
  switch (hd) {
    AT_CASE(64)
    AT_CASE(128)
    AT_CASE(256)
    default: return cudaErrorInvalidValue;
  }
#undef AT_CASE
  return cudaGetLastError();
}
template cudaError_t launch_attn_fma<float>(const float*, const float*, int, const float*, int, const float*, const float*, int, const float*, int, float*, const int32_t*, const int32_t*, int, int, int, int, int, cudaStream_t, int);
template cudaError_t launch_attn_fma<bf16>(const bf16*, const bf16*, int, const bf16*, int, const bf16*, const bf16*, int, const bf16*, int, bf16*, const int32_t*, const int32_t*, int, int, int, int, int, cudaStream_t, int);

// ---------------------------------------------------------------------------
// Depthwise causal conv (4 taps) + SiLU over a packed batch; taps before a sequence start
// come from the cached 3-row tail `hist` (or zero). fmaf chain in tap order, round, SiLU:
// conv1d_silu_seeded_tiled_bf16, native/kernels/kernels.cu:2085-2122.
// x is read with a row stride (it is the first conv_dim columns of the fused projection).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void conv1d_silu_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ hist, const T* __restrict__ w,
                                   T* __restrict__ out, const int32_t* __restrict__ cu, const int32_t* __restrict__ tok_q,
                                   int ch, int tok_base) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= ch) return;
  const int t = blockIdx.y;
  const int off = cu ? cu[tok_q[t]] - tok_base : 0;  // tok_base: packed index of row 0 when x/out/tok_q point into a larger batch
  const int lt = t - off;
  float xs[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int src = lt - 3 + j;
    if (src < 0)
      xs[j] = hist ? Ty<T>::ld(hist + (size_t)(src + 3) * ch + c) : 0.f;
    else
      xs[j] = Ty<T>::ld(x + (size_t)(off + src) * x_stride + c);
  }
  float acc = fmaf(xs[0], Ty<T>::ld(w + c * 4 + 0), 0.f);
  acc = fmaf(xs[1], Ty<T>::ld(w + c * 4 + 1), acc);
  acc = fmaf(xs[2], Ty<T>::ld(w + c * 4 + 2), acc);
  acc = fmaf(xs[3], Ty<T>::ld(w + c * 4 + 3), acc);
  const float v = Ty<T>::rnd(acc);
  Ty<T>::st(out + (size_t)t * ch + c, silu_f(v));
}
// bf16, ch % 8 == 0: each thread owns 8 consecutive channels and CONV_TT consecutive packed tokens,
// sliding the three previous rows through registers (16-byte loads and stores). Same fmaf chain,
// rounding and SiLU per channel; the window restarts from the cached tail at every sequence start.
// Packed row t of x is token t whatever its sequence, so the CONV_TT + 3 rows of a tile, the cached
// tail and the per-token sequence offsets are all fetched up front (independent loads in flight
// together); only the choice between an x row and a tail row depends on the offsets.
constexpr int CONV_TT = 8;
__global__ void __launch_bounds__(128) conv1d_silu_vec8_kernel(const bf16* __restrict__ x, int x_stride, const bf16* __restrict__ hist,
                                                               const bf16* __restrict__ w, bf16* __restrict__ out,
                                                               const int32_t* __restrict__ cu, const int32_t* __restrict__ tok_q, int ch,
                                                               int tokens, int tok_base) {
  const int c8 = blockIdx.x * blockDim.x + threadIdx.x;
  if (c8 * 8 >= ch) return;
  const int c = c8 * 8;
  const int t_begin = blockIdx.y * CONV_TT, t_end = min(t_begin + CONV_TT, tokens);
  int offs[CONV_TT];
#pragma unroll
  for (int i = 0; i < CONV_TT; ++i) offs[i] = cu ? cu[tok_q[min(t_begin + i, tokens - 1)]] - tok_base : 0;
  uint4 xr[CONV_TT + 3];
#pragma unroll
  for (int k = 0; k < CONV_TT + 3; ++k) {
    const int r = min(max(t_begin - 3 + k, 0), tokens - 1);
    xr[k] = *reinterpret_cast<const uint4*>(x + (size_t)r * x_stride + c);
  }
  uint4 hr[3];
#pragma unroll
  for (int k = 0; k < 3; ++k) hr[k] = hist ? *reinterpret_cast<const uint4*>(hist + (size_t)k * ch + c) : make_uint4(0, 0, 0, 0);
  float wt[8][4];
  {
    const uint4* wp = reinterpret_cast<const uint4*>(w + (size_t)c * 4);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      float f[8];
      unpack8(wp[q], f);
#pragma unroll
      for (int i = 0; i < 8; ++i) wt[q * 2 + (i >> 2)][i & 3] = f[i];
    }
  }
  float x3[8], x2[8], x1[8], x0[8];
  {  // window of the tile's first token: rows lt-3..lt-1, from x while they are inside the sequence, else from the tail
    const int lt = t_begin - offs[0];
    auto pick = [&](int j, const uint4& xrow, float (&f)[8]) {  // j = 3, 2, 1: row lt - j
      const int src = lt - j;
      uint4 v = xrow;
      if (src < 0) v = src == -3 ? hr[0] : (src == -2 ? hr[1] : hr[2]);
      unpack8(v, f);
    };
    pick(3, xr[0], x3);
    pick(2, xr[1], x2);
    pick(1, xr[2], x1);
  }
#pragma unroll
  for (int i = 0; i < CONV_TT; ++i) {
    const int t = t_begin + i;
    if (t < t_end) {
      if (i > 0 && t == offs[i]) {  // a new sequence starts here: restart from the tail
        unpack8(hr[0], x3);
        unpack8(hr[1], x2);
        unpack8(hr[2], x1);
      }
      unpack8(xr[i + 3], x0);
      float y[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        float acc = fmaf(x3[e], wt[e][0], 0.f);
        acc = fmaf(x2[e], wt[e][1], acc);
        acc = fmaf(x1[e], wt[e][2], acc);
        acc = fmaf(x0[e], wt[e][3], acc);
        y[e] = silu_fast(Ty<bf16>::rnd(acc));
        x3[e] = x2[e];
        x2[e] = x1[e];
        x1[e] = x0[e];
      }
      *reinterpret_cast<uint4*>(out + (size_t)t * ch + c) = pack8(y);
    }
  }
}

template <typename T>
cudaError_t launch_conv1d_silu(const T* x, int x_stride, const T* hist, const T* w, T* out, const int32_t* cu,
                               const int32_t* tok_q, int tokens, int ch, cudaStream_t s, int tok_base) {
  if constexpr (sizeof(T) == 2) {
    if ((ch % 8) == 0 && (x_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0) {
      dim3 gridv((ch / 8 + 127) / 128, (tokens + CONV_TT - 1) / CONV_TT);
      conv1d_silu_vec8_kernel<<<gridv, 128, 0, s>>>(x, x_stride, hist, w, out, cu, tok_q, ch, tokens, tok_base);
      return cudaGetLastError();
    }
  }
  dim3 grid((ch + 255) / 256, tokens);
  conv1d_silu_kernel<T><<<grid, 256, 0, s>>>(x, x_stride, hist, w, out, cu, tok_q, ch, tok_base);
  return cudaGetLastError();
}
template cudaError_t launch_conv1d_silu<float>(const float*, int, const float*, const float*, float*, const int32_t*, const int32_t*, int, int, cudaStream_t, int);
template cudaError_t launch_conv1d_silu<bf16>(const bf16*, int, const bf16*, const bf16*, bf16*, const int32_t*, const int32_t*, int, int, cudaStream_t, int);

// ---------------------------------------------------------------------------
// GDN prepare (compact form): per (token, key head) L2-normalised q (also scaled by
// dk^-1/2) and k in f32; per (token, value head) g = -exp(A_log)*softplus(a+dt_bias) and
// beta = T(sigmoid(b)). gdn_prepare_compact_bf16, native/kernels/kernels.cu:765-815.
// b and a are read from the fused projection output with a row stride.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void gdn_prepare_kernel(const T* __restrict__ conv, int conv_stride, const T* __restrict__ b, const T* __restrict__ a,
                                   int ba_stride, const float* __restrict__ A_log, const float* __restrict__ dt_bias,
                                   float* __restrict__ qf, float* __restrict__ kf, float* __restrict__ g, float* __restrict__ beta,
                                   int nk, int nv, int dk) {
  __shared__ float red[32];
  const int t = blockIdx.x, kh = blockIdx.y;
  const int key_dim = nk * dk;
  const T* row = conv + (size_t)t * conv_stride;
  const int j = threadIdx.x;  // blockDim.x == dk
  const float qv = Ty<T>::ld(row + kh * dk + j);
  const float kvv = Ty<T>::ld(row + key_dim + kh * dk + j);
  const float qn = block_sum(qv * qv, red);
  const float kn = block_sum(kvv * kvv, red);
  const float qscale = (1.0f / sqrtf(qn + 1e-6f)) * (1.0f / sqrtf((float)dk));
  const float kscale = 1.0f / sqrtf(kn + 1e-6f);
  qf[((size_t)t * nk + kh) * dk + j] = qv * qscale;
  kf[((size_t)t * nk + kh) * dk + j] = kvv * kscale;
  const int rep = nv / nk;
  if (j < rep) {
    const int vh = kh * rep + j;
    const float av = Ty<T>::ld(a + (size_t)t * ba_stride + vh) + dt_bias[vh];
    const float sp = av > 20.f ? av : log1pf(expf(av));
    g[(size_t)t * nv + vh] = -expf(A_log[vh]) * sp;
    beta[(size_t)t * nv + vh] = Ty<T>::rnd(sigmoid_f(Ty<T>::ld(b + (size_t)t * ba_stride + vh)));
  }
}
// dk == 128, bf16: 16 lanes per (token, key head), 8 consecutive elements per lane (16-byte loads), four shuffle steps per
// reduction, float4 stores. Same arithmetic as the generic kernel.
__global__ void __launch_bounds__(256) gdn_prepare_vec128_kernel(const bf16* __restrict__ conv, int conv_stride, const bf16* __restrict__ b,
                                                                 const bf16* __restrict__ a, int ba_stride, const float* __restrict__ A_log,
                                                                 const float* __restrict__ dt_bias, float* __restrict__ qf,
                                                                 float* __restrict__ kf, float* __restrict__ g, float* __restrict__ beta,
                                                                 int tokens, int nk, int nv) {
  const int pair = blockIdx.x * 16 + (threadIdx.x >> 4);
  const int sub = threadIdx.x & 15;
  const bool live = pair < tokens * nk;
  const int idx = live ? pair : tokens * nk - 1;  // every lane stays in the shuffles; the tail recomputes the last pair and stores nothing
  const int t = idx / nk, kh = idx - t * nk;
  const bf16* row = conv + (size_t)t * conv_stride;
  float q[8], k[8];
  unpack8(*reinterpret_cast<const uint4*>(row + kh * 128 + sub * 8), q);
  unpack8(*reinterpret_cast<const uint4*>(row + nk * 128 + kh * 128 + sub * 8), k);
  float qn = 0.f, kn = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    qn += q[j] * q[j];
    kn += k[j] * k[j];
  }
#pragma unroll
  for (int o = 1; o < 16; o <<= 1) {
    qn += __shfl_xor_sync(0xffffffffu, qn, o);
    kn += __shfl_xor_sync(0xffffffffu, kn, o);
  }
  if (!live) return;
  const float qscale = (1.0f / sqrtf(qn + 1e-6f)) * (1.0f / sqrtf(128.0f));
  const float kscale = 1.0f / sqrtf(kn + 1e-6f);
  float4* qd = reinterpret_cast<float4*>(qf + ((size_t)t * nk + kh) * 128 + sub * 8);
  float4* kd = reinterpret_cast<float4*>(kf + ((size_t)t * nk + kh) * 128 + sub * 8);
  qd[0] = make_float4(q[0] * qscale, q[1] * qscale, q[2] * qscale, q[3] * qscale);
  qd[1] = make_float4(q[4] * qscale, q[5] * qscale, q[6] * qscale, q[7] * qscale);
  kd[0] = make_float4(k[0] * kscale, k[1] * kscale, k[2] * kscale, k[3] * kscale);
  kd[1] = make_float4(k[4] * kscale, k[5] * kscale, k[6] * kscale, k[7] * kscale);
  const int rep = nv / nk;
  if (sub < rep) {
    const int vh = kh * rep + sub;
    const float av = __bfloat162float(a[(size_t)t * ba_stride + vh]) + dt_bias[vh];
    const float sp = av > 20.f ? av : log1pf(expf(av));
    g[(size_t)t * nv + vh] = -expf(A_log[vh]) * sp;
    beta[(size_t)t * nv + vh] = Ty<bf16>::rnd(sigmoid_f(__bfloat162float(b[(size_t)t * ba_stride + vh])));
  }
}
// dk == 128: one warp per (token, key head), 4 elements per lane, shuffle reductions, float4 stores.
template <typename T>
__global__ void __launch_bounds__(256) gdn_prepare_warp128_kernel(const T* __restrict__ conv, int conv_stride, const T* __restrict__ b,
                                                                  const T* __restrict__ a, int ba_stride, const float* __restrict__ A_log,
                                                                  const float* __restrict__ dt_bias, float* __restrict__ qf,
                                                                  float* __restrict__ kf, float* __restrict__ g, float* __restrict__ beta,
                                                                  int tokens, int nk, int nv) {
  const int idx = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (idx >= tokens * nk) return;
  const int lane = threadIdx.x & 31;
  const int t = idx / nk, kh = idx - t * nk;
  const T* row = conv + (size_t)t * conv_stride;
  float q[4], k[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    q[j] = Ty<T>::ld(row + kh * 128 + lane * 4 + j);
    k[j] = Ty<T>::ld(row + nk * 128 + kh * 128 + lane * 4 + j);
  }
  const float qn = warp_sum(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
  const float kn = warp_sum(k[0] * k[0] + k[1] * k[1] + k[2] * k[2] + k[3] * k[3]);
  const float qscale = (1.0f / sqrtf(qn + 1e-6f)) * (1.0f / sqrtf(128.0f));
  const float kscale = 1.0f / sqrtf(kn + 1e-6f);
  reinterpret_cast<float4*>(qf + ((size_t)t * nk + kh) * 128)[lane] = make_float4(q[0] * qscale, q[1] * qscale, q[2] * qscale, q[3] * qscale);
  reinterpret_cast<float4*>(kf + ((size_t)t * nk + kh) * 128)[lane] = make_float4(k[0] * kscale, k[1] * kscale, k[2] * kscale, k[3] * kscale);
  const int rep = nv / nk;
  if (lane < rep) {
    const int vh = kh * rep + lane;
    const float av = Ty<T>::ld(a + (size_t)t * ba_stride + vh) + dt_bias[vh];
    const float sp = av > 20.f ? av : log1pf(expf(av));
    g[(size_t)t * nv + vh] = -expf(A_log[vh]) * sp;
    beta[(size_t)t * nv + vh] = Ty<T>::rnd(sigmoid_f(Ty<T>::ld(b + (size_t)t * ba_stride + vh)));
  }
}

template <typename T>
cudaError_t launch_gdn_prepare(const T* conv, int conv_stride, const T* b, const T* a, int ba_stride, const float* A_log,
                               const float* dt_bias, float* qf, float* kf, float* g, float* beta, int tokens, int nk, int nv,
                               int dk, cudaStream_t s) {
  if (dk % 32 != 0 || dk > 1024 || nv / nk > dk) return cudaErrorInvalidValue;
  if constexpr (sizeof(T) == 2) {
    if (dk == 128 && nv / nk <= 16 && tokens > 0 && (conv_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(conv) % 16) == 0) {
      gdn_prepare_vec128_kernel<<<(tokens * nk + 15) / 16, 256, 0, s>>>(conv, conv_stride, b, a, ba_stride, A_log, dt_bias, qf, kf, g, beta, tokens, nk, nv);
      return cudaGetLastError();
    }
  }
  if (dk == 128 && nv / nk <= 32) {
    gdn_prepare_warp128_kernel<T><<<(tokens * nk + 7) / 8, 256, 0, s>>>(conv, conv_stride, b, a, ba_stride, A_log, dt_bias, qf, kf, g, beta, tokens, nk, nv);
    return cudaGetLastError();
  }
  dim3 grid(tokens, nk);
  gdn_prepare_kernel<T><<<grid, dk, 0, s>>>(conv, conv_stride, b, a, ba_stride, A_log, dt_bias, qf, kf, g, beta, nk, nv, dk);
  return cudaGetLastError();
}
template cudaError_t launch_gdn_prepare<float>(const float*, int, const float*, const float*, int, const float*, const float*, float*, float*, float*, float*, int, int, int, int, cudaStream_t);
template cudaError_t launch_gdn_prepare<bf16>(const bf16*, int, const bf16*, const bf16*, int, const float*, const float*, float*, float*, float*, float*, int, int, int, int, cudaStream_t);

// ---------------------------------------------------------------------------
// Gated delta rule, sequential in time, f32 state in registers. One CTA per
// (value head, slice of VC value columns, packed sequence); 4 lanes share a column and
// each holds DK/4 state rows. Starts from the immutable cached state `seed` (or zero) and
// optionally stores the final state (capture). Per step:
//   S *= exp(g); kv = S^T k; delta = (v - kv) * beta; S += k delta^T; o = S^T q.
// gdn_recurrent (scalar statement, native/kernels/kernels.cu:834-865) and
// gdn_recurrent_reg_split_seeded_bf16 (production form, :2245-2300).
// v is read straight from the conv output (value columns start at 2*nk*dk).
// ---------------------------------------------------------------------------
template <typename T, int DK, int VC>
__global__ void __launch_bounds__(VC * 4)
gdn_recurrent_kernel(const float* __restrict__ qf, const float* __restrict__ kf, const T* __restrict__ conv, int conv_stride,
                     const float* __restrict__ g, const float* __restrict__ beta, const float* __restrict__ seed,
                     float* __restrict__ final_state, T* __restrict__ out, const int32_t* __restrict__ cu, int nk, int nv, int dv) {
  constexpr int R = DK / 4;     // state rows per lane
  constexpr int TS = 8;         // time steps staged per shared-memory tile
  constexpr int KP = R + 4;     // padded chunk stride (avoids 4-way bank conflicts)
  __shared__ __align__(16) float sk[TS][4 * KP];
  __shared__ __align__(16) float sq[TS][4 * KP];
  __shared__ float sv[TS][VC];
  __shared__ float sg[TS], sb[TS];
  const int slices = dv / VC;
  const int head = blockIdx.x / slices, cbase = (blockIdx.x - head * slices) * VC;
  const int b = blockIdx.y;
  const int off = cu ? cu[b] : 0;
  const int len = cu ? cu[b + 1] - off : 0;
  const int kh = head / (nv / nk);
  const int tid = threadIdx.x, col = tid >> 2, sub = tid & 3;
  const int vcol0 = 2 * nk * DK + head * dv + cbase;

  float S[R];
  if (seed) {
#pragma unroll
    for (int m = 0; m < R; ++m) S[m] = seed[((size_t)head * DK + sub * R + m) * dv + cbase + col];
  } else {
#pragma unroll
    for (int m = 0; m < R; ++m) S[m] = 0.f;
  }

  for (int t0 = 0; t0 < len; t0 += TS) {
    const int nt = min(TS, len - t0);
    __syncthreads();
    for (int i = tid; i < nt * DK; i += VC * 4) {
      const int tt = i / DK, d = i - tt * DK;
      const size_t src = ((size_t)(off + t0 + tt) * nk + kh) * DK + d;
      const int dst = (d / R) * KP + (d % R);
      sk[tt][dst] = kf[src];
      sq[tt][dst] = qf[src];
    }
    for (int i = tid; i < nt * VC; i += VC * 4) {
      const int tt = i / VC, c = i - tt * VC;
      sv[tt][c] = Ty<T>::ld(conv + (size_t)(off + t0 + tt) * conv_stride + vcol0 + c);
    }
    if (tid < nt) {
      sg[tid] = expf(g[(size_t)(off + t0 + tid) * nv + head]);
      sb[tid] = beta[(size_t)(off + t0 + tid) * nv + head];
    }
    __syncthreads();
    for (int tt = 0; tt < nt; ++tt) {
      const float dec = sg[tt], bt = sb[tt];
      const float* kp = &sk[tt][sub * KP];
      const float* qp = &sq[tt][sub * KP];
      float kvp = 0.f;
#pragma unroll
      for (int m = 0; m < R; m += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kp + m);
        S[m] *= dec; S[m + 1] *= dec; S[m + 2] *= dec; S[m + 3] *= dec;
        kvp += S[m] * k4.x; kvp += S[m + 1] * k4.y; kvp += S[m + 2] * k4.z; kvp += S[m + 3] * k4.w;
      }
      kvp += __shfl_xor_sync(0xffffffffu, kvp, 1);
      kvp += __shfl_xor_sync(0xffffffffu, kvp, 2);
      const float del = (sv[tt][col] - kvp) * bt;
      float op = 0.f;
#pragma unroll
      for (int m = 0; m < R; m += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kp + m);
        const float4 q4 = *reinterpret_cast<const float4*>(qp + m);
        S[m] += k4.x * del; S[m + 1] += k4.y * del; S[m + 2] += k4.z * del; S[m + 3] += k4.w * del;
        op += S[m] * q4.x; op += S[m + 1] * q4.y; op += S[m + 2] * q4.z; op += S[m + 3] * q4.w;
      }
      op += __shfl_xor_sync(0xffffffffu, op, 1);
      op += __shfl_xor_sync(0xffffffffu, op, 2);
      if (sub == 0) Ty<T>::st(out + (size_t)(off + t0 + tt) * (nv * dv) + head * dv + cbase + col, op);
    }
  }
  if (final_state) {
#pragma unroll
    for (int m = 0; m < R; ++m)
      final_state[(((size_t)b * nv + head) * DK + sub * R + m) * dv + cbase + col] = S[m];
  }
}

template <typename T>
cudaError_t launch_gdn_recurrent(const float* qf, const float* kf, const T* conv, int conv_stride, const float* g, const float* beta,
                                 const float* seed, float* final_state, T* out, const int32_t* cu, int B, int nk, int nv, int dk,
                                 int dv, bool few_sequences, cudaStream_t s) {
  // Many sequences (question pass): 64 columns per CTA. One long sequence (capture): 16
  // columns per CTA so that the grid still covers the GPU.
  const int vc = (few_sequences && dv % 16 == 0) ? 16 : 64;
  if (dv % vc != 0) return cudaErrorInvalidValue;
  dim3 grid(nv * (dv / vc), B);
#define GDN_CASE(DK_, VC_)                                                                                              \
  gdn_recurrent_kernel<T, DK_, VC_><<<grid, VC_ * 4, 0, s>>>(qf, kf, conv, conv_stride, g, beta, seed, final_state, out, \
                                                             cu, nk, nv, dv)
  if (dk == 128 && vc == 64) GDN_CASE(128, 64);
  else if (dk == 128 && vc == 16) GDN_CASE(128, 16);
  else if (dk == 64 && vc == 64) GDN_CASE(64, 64);
  else if (dk == 64 && vc == 16) GDN_CASE(64, 16);
  else return cudaErrorInvalidValue;
#undef GDN_CASE
  return cudaGetLastError();
}
template cudaError_t launch_gdn_recurrent<float>(const float*, const float*, const float*, int, const float*, const float*, const float*, float*, float*, const int32_t*, int, int, int, int, int, bool, cudaStream_t);
template cudaError_t launch_gdn_recurrent<bf16>(const float*, const float*, const bf16*, int, const float*, const float*, const float*, float*, bf16*, const int32_t*, int, int, int, int, int, bool, cudaStream_t);

// ---------------------------------------------------------------------------
// F32 readout: logits[B, R] = x[B, H] . W[R, H]^T, all f32
// (blas_gemm_f32 call at native/src/engine.rs:4977-4984; HeadMatrix kept in F32, :737-783).
// One CTA per readout row; the row of W is staged in shared memory once and each warp
// produces logits for a strided subset of the B hidden rows.
// ---------------------------------------------------------------------------
__global__ void readout_kernel(const float* __restrict__ x, const float* __restrict__ W, float* __restrict__ out, int B, int H, int R) {
  extern __shared__ float wrow[];
  const int n = blockIdx.x;
  for (int i = threadIdx.x; i < H; i += blockDim.x) wrow[i] = W[(size_t)n * H + i];
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int b = warp; b < B; b += nw) {
    const float* xr = x + (size_t)b * H;
    float acc = 0.f;
    for (int i = lane; i < H; i += 32) acc += xr[i] * wrow[i];
    acc = warp_sum(acc);
    if (lane == 0) out[(size_t)b * R + n] = acc;
  }
}
cudaError_t launch_readout(const float* x, const float* W, float* out, int B, int H, int R, cudaStream_t s) {
  readout_kernel<<<R, 256, (size_t)H * sizeof(float), s>>>(x, W, out, B, H, R);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Plain-FMA GEMM C[M,N] = X[M,K] . W[N,K]^T with f32 accumulation (f32 engine; diagnostic
// path of the bf16 engine). 64x64 tile, 16-wide K slices, 256 threads, 4x4 per thread.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) gemm_fma_kernel(const T* __restrict__ X, const T* __restrict__ W, T* __restrict__ C, int M,
                                                        int N, int K, int ldc) {
  __shared__ float xs[16][64 + 4];
  __shared__ float ws[16][64 + 4];
  const int m0 = blockIdx.y * 64, n0 = blockIdx.x * 64;
  const int tid = threadIdx.x;
  const int tm = (tid / 16) * 4, tn = (tid % 16) * 4;
  float acc[4][4] = {};
  for (int k0 = 0; k0 < K; k0 += 16) {
    for (int i = tid; i < 64 * 16; i += 256) {
      const int r = i / 16, kk = i % 16;
      const int gm = m0 + r, gn = n0 + r, gk = k0 + kk;
      xs[kk][r] = (gm < M && gk < K) ? Ty<T>::ld(X + (size_t)gm * K + gk) : 0.f;
      ws[kk][r] = (gn < N && gk < K) ? Ty<T>::ld(W + (size_t)gn * K + gk) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < 16; ++kk) {
      float a[4], b[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) { a[i] = xs[kk][tm + i]; b[i] = ws[kk][tn + i]; }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] += a[i] * b[j];
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int gm = m0 + tm + i, gn = n0 + tn + j;
      if (gm < M && gn < N) Ty<T>::st(C + (size_t)gm * ldc + gn, acc[i][j]);
    }
}
template <typename T>
cudaError_t launch_gemm_fma(const T* X, const T* W, T* C, int M, int N, int K, int ldc, cudaStream_t s) {
  dim3 grid((N + 63) / 64, (M + 63) / 64);
  gemm_fma_kernel<T><<<grid, 256, 0, s>>>(X, W, C, M, N, K, ldc);
  return cudaGetLastError();
}
template cudaError_t launch_gemm_fma<float>(const float*, const float*, float*, int, int, int, int, cudaStream_t);
template cudaError_t launch_gemm_fma<bf16>(const bf16*, const bf16*, bf16*, int, int, int, int, cudaStream_t);

// ---------------------------------------------------------------------------
// Strided row copy (V rows of the fused projection into the contiguous StateCache,
// last three pre-conv rows into the conv tail; native/src/engine.rs:3014-3025, 3348-3361).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void copy_rows_kernel(const T* __restrict__ src, int src_stride, T* __restrict__ dst, int dst_stride, int rows, int cols) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)rows * cols) return;
  const size_t r = i / cols, c = i - r * cols;
  dst[r * dst_stride + c] = src[r * src_stride + c];
}
template <typename T>
cudaError_t launch_copy_rows(const T* src, int src_stride, T* dst, int dst_stride, int rows, int cols, cudaStream_t s) {
  const size_t n = (size_t)rows * cols;
  if (n == 0) return cudaSuccess;
  copy_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, src_stride, dst, dst_stride, rows, cols);
  return cudaGetLastError();
}
template cudaError_t launch_copy_rows<float>(const float*, int, float*, int, int, int, cudaStream_t);
template cudaError_t launch_copy_rows<bf16>(const bf16*, int, bf16*, int, int, int, cudaStream_t);

// T -> f32 widening copy (debug taps, state reads) and f32 -> T narrowing (tensor upload).
template <typename T>
__global__ void to_f32_kernel(const T* __restrict__ src, float* __restrict__ dst, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = Ty<T>::ld(src + i);
}
template <typename T>
__global__ void from_f32_kernel(const float* __restrict__ src, T* __restrict__ dst, size_t n) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) Ty<T>::st(dst + i, src[i]);
}
template <typename T>
cudaError_t launch_to_f32(const T* src, float* dst, size_t n, cudaStream_t s) {
  if (n) to_f32_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}
template <typename T>
cudaError_t launch_from_f32(const float* src, T* dst, size_t n, cudaStream_t s) {
  if (n) from_f32_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n);
  return cudaGetLastError();
}
template cudaError_t launch_to_f32<float>(const float*, float*, size_t, cudaStream_t);
template cudaError_t launch_to_f32<bf16>(const bf16*, float*, size_t, cudaStream_t);
template cudaError_t launch_from_f32<float>(const float*, float*, size_t, cudaStream_t);
template cudaError_t launch_from_f32<bf16>(const float*, bf16*, size_t, cudaStream_t);

// ---------------------------------------------------------------------------
// Seeded weight generator (device twin; integer hashing plus one float multiply, so the
// values are bit-identical to a host evaluation of the same rule):
//   key = mix64(mix64(seed) ^ tensor_id); a = mix64(key+2i); b = mix64(key+2i+1)
//   normal : (sum of the eight 16-bit lanes of a,b - 262140) * c + shift   (Irwin-Hall 8)
//   uniform: fmaf(hi-lo, (a>>40) * 2^-24, lo)
// Rows are scattered through `row_map`: mode 0 dst_row = row_offset + r; mode 1/2 place
// gate/up rows in 256-row tiles (128 gate rows then 128 up rows) for the SwiGLU epilogue.
// ---------------------------------------------------------------------------
__host__ __device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
uint64_t gen_tensor_key(uint64_t seed, int layer, int kind) {
  return mix64(mix64(seed) ^ ((uint64_t)(layer + 1) * 64 + (uint64_t)kind));
}
__device__ __forceinline__ size_t map_row(size_t r, int mode, int row_offset) {
  if (mode == 0) return (size_t)row_offset + r;
  return (r >> 7) * 256 + (r & 127) + (mode == 2 ? 128 : 0);
}
template <typename T>
__global__ void gen_tensor_kernel(T* __restrict__ dst, uint64_t key, uint64_t first, uint64_t count, int cols, int dist, float p0,
                                  float p1, float c, int round_bf, int mode, int row_offset, int dst_stride) {
  const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= count) return;
  const uint64_t e = first + i;
  const uint64_t a = mix64(key + 2 * e);
  float v;
  if (dist == 0) {
    const uint64_t b = mix64(key + 2 * e + 1);
    int s = 0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      s += (int)((a >> (16 * q)) & 0xffff);
      s += (int)((b >> (16 * q)) & 0xffff);
    }
    v = __fadd_rn(__fmul_rn((float)(s - 262140), c), p1);
  } else {
    const float u = __fmul_rn((float)(a >> 40), 1.0f / 16777216.0f);
    v = __fmaf_rn(__fsub_rn(p1, p0), u, p0);
  }
  if (round_bf) v = __bfloat162float(__float2bfloat16_rn(v));
  const size_t r = (size_t)(i / cols), cc = (size_t)(i % cols);
  Ty<T>::st(dst + map_row(r, mode, row_offset) * dst_stride + cc, v);
}
template <typename T>
cudaError_t launch_gen_tensor(T* dst, uint64_t key, uint64_t first, uint64_t count, int cols, int dist, float p0, float p1, float c,
                              bool round_bf, int mode, int row_offset, int dst_stride, cudaStream_t s) {
  if (count == 0) return cudaSuccess;
  gen_tensor_kernel<T><<<(unsigned)((count + 255) / 256), 256, 0, s>>>(dst, key, first, count, cols, dist, p0, p1, c, round_bf ? 1 : 0,
                                                                      mode, row_offset, dst_stride);
  return cudaGetLastError();
}
template cudaError_t launch_gen_tensor<float>(float*, uint64_t, uint64_t, uint64_t, int, int, float, float, float, bool, int, int, int, cudaStream_t);
template cudaError_t launch_gen_tensor<bf16>(bf16*, uint64_t, uint64_t, uint64_t, int, int, float, float, float, bool, int, int, int, cudaStream_t);

// Scatter / gather rows between the standard [rows, cols] layout and a placed layout.
template <typename T>
__global__ void place_rows_kernel(const T* __restrict__ src, T* __restrict__ dst, size_t n, int cols, int mode, int row_offset,
                                  int dst_stride, int inverse) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t r = i / cols, c = i - r * cols;
  const size_t p = map_row(r, mode, row_offset) * dst_stride + c;
  if (inverse) dst[i] = src[p]; else dst[p] = src[i];
}
template <typename T>
cudaError_t launch_place_rows(const T* src, T* dst, size_t rows, int cols, int mode, int row_offset, int dst_stride, bool inverse,
                              cudaStream_t s) {
  const size_t n = rows * cols;
  if (n == 0) return cudaSuccess;
  place_rows_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, dst, n, cols, mode, row_offset, dst_stride, inverse ? 1 : 0);
  return cudaGetLastError();
}
template cudaError_t launch_place_rows<float>(const float*, float*, size_t, int, int, int, int, bool, cudaStream_t);
template cudaError_t launch_place_rows<bf16>(const bf16*, bf16*, size_t, int, int, int, int, bool, cudaStream_t);

// ---------------------------------------------------------------------------
// Per-row symmetric FP8 E4M3 quantisation (activations per token, weights per output row):
// scale = max(absmax * clip, 1e-10) / 448; q = e4m3_satfinite(x / scale).
// quant_fp8_per_token_bf16, native/kernels/kernels.cu:182-205. x rows may be strided.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) quant_fp8_rows_kernel(const T* __restrict__ x, size_t x_stride, uint8_t* __restrict__ out,
                                                             float* __restrict__ scales, int cols, float clip) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const T* xr = x + (size_t)row * x_stride;
  float m = 0.f;
  for (int i = threadIdx.x; i < cols; i += blockDim.x) m = fmaxf(m, fabsf(Ty<T>::ld(xr + i)));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  float t = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
  t = warp_max(t);
  const float scale = fmaxf(t * clip, 1e-10f) / 448.f;
  if (threadIdx.x == 0) scales[row] = scale;
  uint8_t* orow = out + (size_t)row * cols;
  for (int i = threadIdx.x; i < cols; i += blockDim.x)
    orow[i] = (uint8_t)__nv_cvt_float_to_fp8(Ty<T>::ld(xr + i) / scale, __NV_SATFINITE, __NV_E4M3);
}
// bf16, cols % 8 == 0: 16-byte loads, 8-byte stores.
__global__ void __launch_bounds__(256) quant_fp8_rows_vec_kernel(const bf16* __restrict__ x, size_t x_stride, uint8_t* __restrict__ out,
                                                                 float* __restrict__ scales, int cols, float clip) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * x_stride);
  const int n8 = cols >> 3;
  float m = 0.f;
  for (int i = threadIdx.x; i < n8; i += 256) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  float t = (threadIdx.x & 31) < 8 ? red[threadIdx.x & 31] : 0.f;
  t = warp_max(t);
  const float scale = fmaxf(t * clip, 1e-10f) / 448.f;
  if (threadIdx.x == 0) scales[row] = scale;
  uint2* orow = reinterpret_cast<uint2*>(out + (size_t)row * cols);
  for (int i = threadIdx.x; i < n8; i += 256) {
    float f[8];
    unpack8(xr[i], f);
    uint32_t w[2] = {0, 0};
#pragma unroll
    for (int j = 0; j < 8; ++j)
      w[j >> 2] |= (uint32_t)__nv_cvt_float_to_fp8(f[j] / scale, __NV_SATFINITE, __NV_E4M3) << (8 * (j & 3));
    orow[i] = make_uint2(w[0], w[1]);
  }
}
template <typename T>
cudaError_t launch_quant_fp8_rows(const T* x, size_t x_stride, uint8_t* out, float* scales, int rows, int cols, float clip, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if constexpr (sizeof(T) == 2) {
    if ((cols % 8) == 0 && (x_stride % 8) == 0 && (reinterpret_cast<uintptr_t>(x) % 16) == 0 && (reinterpret_cast<uintptr_t>(out) % 8) == 0) {
      quant_fp8_rows_vec_kernel<<<rows, 256, 0, s>>>(x, x_stride, out, scales, cols, clip);
      return cudaGetLastError();
    }
  }
  quant_fp8_rows_kernel<T><<<rows, 256, 0, s>>>(x, x_stride, out, scales, cols, clip);
  return cudaGetLastError();
}
template cudaError_t launch_quant_fp8_rows<float>(const float*, size_t, uint8_t*, float*, int, int, float, cudaStream_t);
template cudaError_t launch_quant_fp8_rows<bf16>(const bf16*, size_t, uint8_t*, float*, int, int, float, cudaStream_t);

// ---------------------------------------------------------------------------
// W4A16, group 128: compressed-tensors pack-quantized layout as the reference reads it
// (native/src/weights.rs:292-330): packed [N, ceil(K/8)] words, nibble k of word j = input 8j+k,
// symmetric zero-point 8, scales [N, ceil(K/128)] (fp16 here).
//   dequant: w[o,i] = bf16(float(q - 8) * float(scale[o, i/128]))   dequant_w4a16_bf16, kernels.cu:867-892
//   quant  : scale = fp16(absmax/7), q = clamp(rint(w/scale), -8, 7)  (round to nearest; one warp per group)
// ---------------------------------------------------------------------------
// perm: the engine's own word layout, nibble order [k0 k2 k4 k6 k1 k3 k5 k7] (what the fused W4A16 GEMM unpacks in two-element
// steps); otherwise the compressed-tensors order k0..k7.
__device__ __forceinline__ uint32_t w4_nibble_permute(uint32_t w) {
  uint32_t o = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) o |= ((w >> (4 * j)) & 0xFu) << (4 * ((j & 1) * 4 + (j >> 1)));
  return o;
}
__global__ void __launch_bounds__(256) quant_w4_g128_kernel(const bf16* __restrict__ W, uint32_t* __restrict__ packed,
                                                            __half* __restrict__ scales, int N, int K, bool perm) {
  const int groups = (K + 127) / 128, words = (K + 7) / 8;
  const int gidx = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (gidx >= N * groups) return;
  const int lane = threadIdx.x & 31;
  const int o = gidx / groups, gi = gidx - o * groups;
  const int k0 = gi * 128 + lane * 4;
  float v[4];
  float amax = 0.f;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    v[j] = (k0 + j) < K ? __bfloat162float(W[(size_t)o * K + k0 + j]) : 0.f;
    amax = fmaxf(amax, fabsf(v[j]));
  }
  amax = warp_max(amax);
  const __half sh = __float2half_rn(amax / 7.0f);
  const float sc = __half2float(sh);
  if (lane == 0) scales[(size_t)o * groups + gi] = sh;
  uint32_t nib = 0;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    int q = 0;
    if (sc > 0.f) q = (int)fminf(fmaxf(rintf(v[j] / sc), -8.f), 7.f);
    nib |= (uint32_t)((q + 8) & 0xf) << (4 * j);
  }
  // lanes 2m and 2m+1 hold the low and high halves of word m of the group
  const uint32_t other = __shfl_xor_sync(0xffffffffu, nib, 1);
  if ((lane & 1) == 0) {
    const int w = (gi * 128 + lane * 4) >> 3;
    const uint32_t word = nib | (other << 16);
    if (w < words) packed[(size_t)o * words + w] = perm ? w4_nibble_permute(word) : word;
  }
}

__global__ void __launch_bounds__(256) dequant_w4_g128_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scales,
                                                              bf16* __restrict__ W, int N, int K, bool perm) {
  const int words = (K + 7) / 8, groups = (K + 127) / 128;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)N * words) return;
  const int o = (int)(idx / words), w = (int)(idx - (size_t)o * words);
  const uint32_t word = packed[idx];
  const float sc = __half2float(scales[(size_t)o * groups + (w * 8) / 128]);
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = (float)((int)((word >> (4 * (perm ? (j & 1) * 4 + (j >> 1) : j))) & 0xf) - 8) * sc;
  bf16* dst = W + (size_t)o * K + (size_t)w * 8;
  if (w * 8 + 8 <= K && (K % 8) == 0) {
    *reinterpret_cast<uint4*>(dst) = pack8(f);
  } else {
    for (int j = 0; j < 8 && w * 8 + j < K; ++j) dst[j] = __float2bfloat16_rn(f[j]);
  }
}

cudaError_t launch_quant_w4_g128(const bf16* W, uint32_t* packed, void* scales, int N, int K, cudaStream_t s, bool perm) {
  if (N <= 0 || (K % 8) != 0) return N <= 0 ? cudaSuccess : cudaErrorInvalidValue;
  const int groups = (K + 127) / 128;
  quant_w4_g128_kernel<<<(N * groups + 7) / 8, 256, 0, s>>>(W, packed, (__half*)scales, N, K, perm);
  return cudaGetLastError();
}
cudaError_t launch_dequant_w4_g128(const uint32_t* packed, const void* scales, bf16* W, int N, int K, cudaStream_t s, bool perm) {
  if (N <= 0) return cudaSuccess;
  const size_t n = (size_t)N * ((K + 7) / 8);
  dequant_w4_g128_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(packed, (const __half*)scales, W, N, K, perm);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// NVFP4: e2m1 values, one e4m3 scale per 16 elements along K, one f32 scale per tensor.
// Quantisation rule of quant_nvfp4_act_bf16 / fp4_encode (native/kernels/kernels.cu:222-277):
//   v = x * global; sf = e4m3_satfinite(max(absmax16(v)/6, 1e-10)); code = fp4_encode(v / decode(sf));
//   packed byte = low nibble even k, high nibble odd k. (Scales are kept row-major [rows, K/16] here.)
// e2m1 * e4m3 has at most five significant bits, so the dequantised element decode(code)*decode(sf)
// is exact in bf16: the bf16 tensor-core GEMM on dequantised operands reproduces the block-scaled
// FP4 product exactly up to the f32 summation order; alpha = 1/(weight_global*input_global) is
// applied in the GEMM epilogue (native/src/engine.rs:4108).
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint8_t fp4_encode(float x) {
  const float a = fabsf(x);
  uint8_t e;
  if (a < 0.25f) e = 0;
  else if (a < 0.75f) e = 1;
  else if (a < 1.25f) e = 2;
  else if (a < 1.75f) e = 3;
  else if (a < 2.5f) e = 4;
  else if (a < 3.5f) e = 5;
  else if (a < 5.0f) e = 6;
  else e = 7;
  return (x < 0.f) ? (uint8_t)(e | 8) : e;
}
__device__ __forceinline__ float fp4_decode(uint8_t c) {
  const float mag[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = mag[c & 7];
  return (c & 8) ? -v : v;
}
__device__ __forceinline__ float e4m3_decode(uint8_t c) {
  const __half_raw hr = __nv_cvt_fp8_to_halfraw(c, __NV_E4M3);
  return __half2float(*reinterpret_cast<const __half*>(&hr));
}

// |x| maximum of a bf16 matrix into *out (float bits; non-negative floats order like unsigned ints).
__global__ void absmax_bf16_kernel(const bf16* __restrict__ x, size_t n, unsigned int* __restrict__ out) {
  float m = 0.f;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    m = fmaxf(m, fabsf(__bfloat162float(x[i])));
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) atomicMax(out, __float_as_uint(m));
}
// *global = 2688 / absmax (448 * 6: the largest group scale lands on the top of the e4m3 range)
__global__ void nvfp4_global_from_absmax_kernel(const unsigned int* __restrict__ amax, float* __restrict__ global, float* __restrict__ alpha,
                                                float input_global) {
  const float a = __uint_as_float(*amax);
  const float g = a > 0.f ? 2688.0f / a : 1.0f;
  *global = g;
  *alpha = 1.0f / (g * input_global);
}

// mode 0: store codes + scales. mode 1: store the dequantised value decode(code)*decode(sf) (no global) as bf16.
template <int MODE>
__global__ void __launch_bounds__(256) nvfp4_rows_kernel(const bf16* __restrict__ x, size_t x_stride, const float* __restrict__ global_ptr,
                                                         float global_imm, uint8_t* __restrict__ packed, uint8_t* __restrict__ scales,
                                                         bf16* __restrict__ deq, int K) {
  const int row = blockIdx.x;
  const float gl = global_ptr ? __ldg(global_ptr) : global_imm;
  const bf16* src = x + (size_t)row * x_stride;
  const int groups = K / 16;
  for (int j = threadIdx.x; j < groups; j += blockDim.x) {
    float v[16];
    float m = 0.f;
    const uint4 lo = *reinterpret_cast<const uint4*>(src + j * 16);
    const uint4 hi = *reinterpret_cast<const uint4*>(src + j * 16 + 8);
    float f[8];
    unpack8(lo, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = f[i] * gl;
    unpack8(hi, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[8 + i] = f[i] * gl;
#pragma unroll
    for (int i = 0; i < 16; ++i) m = fmaxf(m, fabsf(v[i]));
    const float sf = fmaxf(m / 6.0f, 1e-10f);
    const uint8_t sb = (uint8_t)__nv_cvt_float_to_fp8(sf, __NV_SATFINITE, __NV_E4M3);
    const float sd = e4m3_decode(sb);
    if (MODE == 0) {
      uint32_t w[2] = {0, 0};
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint32_t byte = (uint32_t)fp4_encode(v[2 * i] / sd) | ((uint32_t)fp4_encode(v[2 * i + 1] / sd) << 4);
        w[i >> 2] |= byte << (8 * (i & 3));
      }
      *reinterpret_cast<uint2*>(packed + (size_t)row * (K / 2) + j * 8) = make_uint2(w[0], w[1]);
      scales[(size_t)row * groups + j] = sb;
    } else {
      float o[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = fp4_decode(fp4_encode(v[i] / sd)) * sd;
      *reinterpret_cast<uint4*>(deq + (size_t)row * K + j * 16) = pack8(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = fp4_decode(fp4_encode(v[8 + i] / sd)) * sd;
      *reinterpret_cast<uint4*>(deq + (size_t)row * K + j * 16 + 8) = pack8(o);
    }
  }
}
// codes + scales -> bf16 decode(code)*decode(sf) [* inv_global when given]
__global__ void __launch_bounds__(256) nvfp4_dequant_rows_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales,
                                                                 const float* __restrict__ global_ptr, bf16* __restrict__ out, size_t total_groups,
                                                                 int K) {
  const size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gi >= total_groups) return;
  const int groups = K / 16;
  const size_t row = gi / groups;
  const int j = (int)(gi - row * groups);
  float sd = e4m3_decode(scales[gi]);
  if (global_ptr) {
    const float gsc = __ldg(global_ptr);
    if (gsc > 0.f) sd = sd / gsc;
  }
  const uint2 w = *reinterpret_cast<const uint2*>(packed + row * (K / 2) + j * 8);
  const uint32_t ww[2] = {w.x, w.y};
  float o[16];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t byte = (ww[i >> 2] >> (8 * (i & 3))) & 0xff;
    o[2 * i] = fp4_decode((uint8_t)(byte & 0xf)) * sd;
    o[2 * i + 1] = fp4_decode((uint8_t)(byte >> 4)) * sd;
  }
  float a[8], b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { a[i] = o[i]; b[i] = o[8 + i]; }
  *reinterpret_cast<uint4*>(out + row * K + j * 16) = pack8(a);
  *reinterpret_cast<uint4*>(out + row * K + j * 16 + 8) = pack8(b);
}

cudaError_t launch_absmax_bf16(const bf16* x, size_t n, unsigned int* out, cudaStream_t s) {
  cudaError_t e = cudaMemsetAsync(out, 0, 4, s);
  if (e != cudaSuccess) return e;
  absmax_bf16_kernel<<<1024, 256, 0, s>>>(x, n, out);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_global(const unsigned int* amax, float* global, float* alpha, float input_global, cudaStream_t s) {
  nvfp4_global_from_absmax_kernel<<<1, 1, 0, s>>>(amax, global, alpha, input_global);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_quant_rows(const bf16* x, size_t x_stride, const float* global_ptr, float global_imm, uint8_t* packed, uint8_t* scales,
                                    int rows, int K, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if ((K % 16) || (x_stride % 8)) return cudaErrorInvalidValue;
  nvfp4_rows_kernel<0><<<rows, 256, 0, s>>>(x, x_stride, global_ptr, global_imm, packed, scales, nullptr, K);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_fakequant_rows(const bf16* x, size_t x_stride, float global_imm, bf16* out, int rows, int K, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if ((K % 16) || (x_stride % 8)) return cudaErrorInvalidValue;
  nvfp4_rows_kernel<1><<<rows, 256, 0, s>>>(x, x_stride, nullptr, global_imm, nullptr, nullptr, out, K);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_dequant_rows(const uint8_t* packed, const uint8_t* scales, const float* global_ptr, bf16* out, int rows, int K,
                                      cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  const size_t groups = (size_t)rows * (K / 16);
  nvfp4_dequant_rows_kernel<<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(packed, scales, global_ptr, out, groups, K);
  return cudaGetLastError();
}

// ---------------------------------------------------------------------------
// Checkpoint formats -> engine layout. A chunk of `n_rows` source rows (the first one is row
// `row_start` of the logical tensor) is converted and written to its place inside the (possibly
// fused / interleaved) engine matrix; map_row() is the same placement every other loader uses.
//
// place_rows_cvt: plain tensors stored as F32, F16 or BF16 (Store::bf16 / Store::f32,
//   native/src/tensor.rs:187-215 in juanqui/decidra).
// dequant_ct_w4_place: compressed-tensors pack-quantized int4 (LinearWeight::PackedW4A16,
//   native/src/weights.rs:73-87): packed I32 [out, ceil(in/8)], nibble j of a word = input
//   8*word + j; scale BF16 [out, in/group]; zero point I32 [ceil(out/8), in/group], nibble
//   (o & 7) of word (o >> 3); symmetric checkpoints have no zero-point tensor and mean 8
//   (weights.rs:314-320). Value = bf16((q - z) * scale), the arithmetic of dequant_w4a16_bf16
//   (native/kernels/kernels.cu:874-892).
// dequant_ct_nvfp4_place: compressed-tensors nvfp4-pack-quantized (nvfp4_linear,
//   native/src/weights.rs:502-547): packed U8 [out, in/2] (low nibble = even input), scale
//   E4M3 [out, in/16] row-major, f32 weight_global_scale; value = bf16(e2m1 * (scale / global)),
//   the weight factor of Engine::nvfp4_gemm's alpha = 1/(weight_global*input_global)
//   (native/src/engine.rs:4109).
// ---------------------------------------------------------------------------
template <typename T>
__global__ void place_rows_cvt_kernel(const void* __restrict__ src, int src_dt, T* __restrict__ dst, size_t n, int cols, size_t row_start,
                                      int mode, int row_offset, int dst_stride) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const size_t r = i / cols, c = i - r * cols;
  float v;
  if (src_dt == 0) v = reinterpret_cast<const float*>(src)[i];
  else if (src_dt == 1) v = __half2float(reinterpret_cast<const __half*>(src)[i]);
  else v = __bfloat162float(reinterpret_cast<const bf16*>(src)[i]);
  Ty<T>::st(dst + map_row(row_start + r, mode, row_offset) * dst_stride + c, v);
}
template <typename T>
cudaError_t launch_place_rows_cvt(const void* src, int src_dt, T* dst, size_t n_rows, int cols, size_t row_start, int mode, int row_offset,
                                  int dst_stride, cudaStream_t s) {
  const size_t n = n_rows * cols;
  if (n == 0) return cudaSuccess;
  if (src_dt < 0 || src_dt > 2) return cudaErrorInvalidValue;
  place_rows_cvt_kernel<T><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(src, src_dt, dst, n, cols, row_start, mode, row_offset, dst_stride);
  return cudaGetLastError();
}
template cudaError_t launch_place_rows_cvt<float>(const void*, int, float*, size_t, int, size_t, int, int, int, cudaStream_t);
template cudaError_t launch_place_rows_cvt<bf16>(const void*, int, bf16*, size_t, int, size_t, int, int, int, cudaStream_t);

template <typename T>
__global__ void dequant_ct_w4_place_kernel(const int32_t* __restrict__ packed, const bf16* __restrict__ scale, const int32_t* __restrict__ zp,
                                           T* __restrict__ dst, size_t n_words, int in_dim, int group_size, size_t row_start, int mode,
                                           int row_offset, int dst_stride) {
  const size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (wi >= n_words) return;
  const int words_per_row = (in_dim + 7) / 8;
  const int groups = (in_dim + group_size - 1) / group_size;
  const size_t o = wi / words_per_row;  // row inside the chunk; the chunk starts on a multiple of 8 rows
  const int w = (int)(wi - o * words_per_row);
  const uint32_t word = (uint32_t)packed[wi];
  T* out = dst + map_row(row_start + o, mode, row_offset) * dst_stride;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int i = w * 8 + j;
    if (i >= in_dim) break;
    const int g = i / group_size;
    const int q = (int)((word >> (4 * j)) & 0xFu);
    const int z = zp ? (int)(((uint32_t)zp[(o >> 3) * groups + g] >> (4 * (int)(o & 7))) & 0xFu) : 8;
    const float sc = __bfloat162float(scale[o * groups + g]);
    Ty<T>::st(out + i, __bfloat162float(__float2bfloat16_rn((float)(q - z) * sc)));
  }
}
template <typename T>
cudaError_t launch_dequant_ct_w4_place(const int32_t* packed, const bf16* scale, const int32_t* zp, T* dst, size_t n_rows, int in_dim,
                                       int group_size, size_t row_start, int mode, int row_offset, int dst_stride, cudaStream_t s) {
  if (n_rows == 0) return cudaSuccess;
  if (in_dim <= 0 || group_size <= 0 || (row_start & 7)) return cudaErrorInvalidValue;
  const size_t n_words = n_rows * (size_t)((in_dim + 7) / 8);
  dequant_ct_w4_place_kernel<T><<<(unsigned)((n_words + 255) / 256), 256, 0, s>>>(packed, scale, zp, dst, n_words, in_dim, group_size, row_start,
                                                                                 mode, row_offset, dst_stride);
  return cudaGetLastError();
}
template cudaError_t launch_dequant_ct_w4_place<float>(const int32_t*, const bf16*, const int32_t*, float*, size_t, int, int, size_t, int, int,
                                                       int, cudaStream_t);
template cudaError_t launch_dequant_ct_w4_place<bf16>(const int32_t*, const bf16*, const int32_t*, bf16*, size_t, int, int, size_t, int, int, int,
                                                      cudaStream_t);

// compressed-tensors int4 rows (group 128) adopted as they are by a W4 engine: the words go to their (fused / interleaved) rows in
// the engine's nibble order, the bf16 scales become fp16. A zero point other than 8 or a scale that fp16 cannot hold exactly
// raises *flag (the caller then takes the dequantise-and-requantise route for the whole fused matrix).
__global__ void adopt_ct_w4_rows_kernel(const int32_t* __restrict__ packed, const bf16* __restrict__ scale, const int32_t* __restrict__ zp,
                                        uint32_t* __restrict__ dst_q, __half* __restrict__ dst_scale, size_t n_words, int in_dim, size_t row_start,
                                        int mode, int row_offset, int* __restrict__ flag) {
  const size_t wi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (wi >= n_words) return;
  const int words_per_row = in_dim / 8, groups = in_dim / 128;
  const size_t o = wi / words_per_row;  // row inside the chunk; the chunk starts on a multiple of 8 rows
  const int w = (int)(wi - o * words_per_row);
  const size_t drow = map_row(row_start + o, mode, row_offset);
  dst_q[drow * words_per_row + w] = w4_nibble_permute((uint32_t)packed[wi]);
  if ((w & 15) == 0) {  // first word of a group: its scale and zero point
    const int g = w >> 4;
    const float sc = __bfloat162float(scale[o * groups + g]);
    const __half sh = __float2half_rn(sc);
    dst_scale[drow * groups + g] = sh;
    const int z = zp ? (int)(((uint32_t)zp[(o >> 3) * groups + g] >> (4 * (int)(o & 7))) & 0xFu) : 8;
    if (__half2float(sh) != sc || z != 8) atomicExch(flag, 1);
  }
}
cudaError_t launch_adopt_ct_w4_rows(const int32_t* packed, const bf16* scale, const int32_t* zp, uint32_t* dst_q, void* dst_scale, size_t n_rows,
                                    int in_dim, size_t row_start, int mode, int row_offset, int* flag, cudaStream_t s) {
  if (n_rows == 0) return cudaSuccess;
  if (in_dim <= 0 || (in_dim % 128) || (row_start & 7)) return cudaErrorInvalidValue;
  const size_t n_words = n_rows * (size_t)(in_dim / 8);
  adopt_ct_w4_rows_kernel<<<(unsigned)((n_words + 255) / 256), 256, 0, s>>>(packed, scale, zp, dst_q, (__half*)dst_scale, n_words, in_dim, row_start,
                                                                           mode, row_offset, flag);
  return cudaGetLastError();
}

template <typename T>
__global__ void dequant_ct_nvfp4_place_kernel(const uint8_t* __restrict__ packed, const uint8_t* __restrict__ scales, float global,
                                              T* __restrict__ dst, size_t total_groups, int K, size_t row_start, int mode, int row_offset,
                                              int dst_stride) {
  const size_t gi = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (gi >= total_groups) return;
  const int groups = K / 16;
  const size_t row = gi / groups;
  const int j = (int)(gi - row * groups);
  float sd = e4m3_decode(scales[gi]);
  if (global > 0.f) sd = sd / global;
  const uint2 w = *reinterpret_cast<const uint2*>(packed + row * (size_t)(K / 2) + j * 8);
  const uint32_t ww[2] = {w.x, w.y};
  T* out = dst + map_row(row_start + row, mode, row_offset) * dst_stride + j * 16;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t byte = (ww[i >> 2] >> (8 * (i & 3))) & 0xff;
    Ty<T>::st(out + 2 * i, __bfloat162float(__float2bfloat16_rn(fp4_decode((uint8_t)(byte & 0xf)) * sd)));
    Ty<T>::st(out + 2 * i + 1, __bfloat162float(__float2bfloat16_rn(fp4_decode((uint8_t)(byte >> 4)) * sd)));
  }
}
template <typename T>
cudaError_t launch_dequant_ct_nvfp4_place(const uint8_t* packed, const uint8_t* scales, float global, T* dst, size_t n_rows, int K,
                                          size_t row_start, int mode, int row_offset, int dst_stride, cudaStream_t s) {
  if (n_rows == 0) return cudaSuccess;
  if (K <= 0 || (K % 16)) return cudaErrorInvalidValue;
  const size_t groups = n_rows * (size_t)(K / 16);
  dequant_ct_nvfp4_place_kernel<T><<<(unsigned)((groups + 255) / 256), 256, 0, s>>>(packed, scales, global, dst, groups, K, row_start, mode,
                                                                                   row_offset, dst_stride);
  return cudaGetLastError();
}
template cudaError_t launch_dequant_ct_nvfp4_place<float>(const uint8_t*, const uint8_t*, float, float*, size_t, int, size_t, int, int, int,
                                                          cudaStream_t);
template cudaError_t launch_dequant_ct_nvfp4_place<bf16>(const uint8_t*, const uint8_t*, float, bf16*, size_t, int, size_t, int, int, int,
                                                         cudaStream_t);
