// Shared device helpers: storage-type traits (f32 / bf16), rounding, warp reductions.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp4.h>
#include <cuda_runtime.h>
#include <stdint.h>

typedef __nv_bfloat16 bf16;

// Device error word codes (written with atomicCAS so the first error wins).
enum : int {
  DERR_NONE = 0,
  DERR_TOKEN_RANGE = 1,   // token id >= vocab
  DERR_EMPTY_ITEM = 2,    // a packed sequence has length <= 0
  DERR_GEMM_TIMEOUT = 3,  // a bounded mbarrier wait gave up in the tcgen05 GEMM
  DERR_ATTN_TIMEOUT = 4,
  DERR_POSITION_RANGE = 5, // RoPE position beyond the table
  DERR_GDN_TIMEOUT = 6
};

__device__ __forceinline__ void set_err(int* err, int code) {
  if (err) atomicCAS(err, 0, code);
}

template <typename T> struct Ty;
template <> struct Ty<float> {
  static __device__ __forceinline__ float ld(const float* p) { return *p; }
  static __device__ __forceinline__ void st(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float rnd(float v) { return v; }
};
template <> struct Ty<bf16> {
  static __device__ __forceinline__ float ld(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void st(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float rnd(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for blockDim.x <= 1024 (multiple of 32). `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = lane < nw ? red[lane] : 0.f;
  t = warp_sum(t);
  __syncthreads();
  return t;
}

__device__ __forceinline__ float silu_f(float g) { return g / (1.0f + expf(-g)); }
__device__ __forceinline__ float sigmoid_f(float g) { return 1.0f / (1.0f + expf(-g)); }

#define CUDA_TRY(expr)                          \
  do {                                          \
    cudaError_t _e = (expr);                    \
    if (_e != cudaSuccess) return _e;           \
  } while (0)

// e2m1 codes of eight bf16-representable values divided by the decoded group scale sd, value j in nibble j, under the rule of
// fp4_encode (juanqui/decidra native/kernels/kernels.cu:222-239: magnitude thresholds 0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5 taken with
// >=, the sign bit only for v < 0). cvt.rn.satfinite.e2m1x2.f32 rounds to nearest with the same midpoints; it differs from the rule
// on exact ties (nearest-even instead of up) and on -0 only, and both are steered here: the quotient is v * (1/sd)(1 + 2^-12). v has
// at most 8 significant bits and threshold * sd at most 7, so a quotient that is not a tie is at least 2^-8 away from every midpoint
// in relative terms and stays on its side of it, a tie lands just above; the added +0 turns a -0 product into +0. sd = 0 (every value
// of the group below half the smallest scale): magnitude code 7 throughout, which is what comparing with zero thresholds gives and
// what fp4_encode returns for the inf and NaN of v / 0. One conversion per pair instead of fourteen compare-and-add steps.
__device__ __forceinline__ uint32_t nvfp4_codes8(const float* y, float sd) {
  uint32_t c = 0;
  if (sd == 0.f) {
#pragma unroll
    for (int j = 0; j < 8; ++j) c |= (7u | (y[j] < 0.f ? 8u : 0u)) << (4 * j);
    return c;
  }
  const float r = (1.0f / sd) * 1.000244140625f;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const float2 q = make_float2(fmaf(y[2 * p], r, 0.f), fmaf(y[2 * p + 1], r, 0.f));
    c |= (uint32_t)__nv_cvt_float2_to_fp4x2(q, __NV_E2M1, cudaRoundNearest) << (8 * p);
  }
  return c;
}
