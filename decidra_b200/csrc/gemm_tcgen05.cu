// C[M,N] = X[M,K] . W[N,K]^T for bf16 operands on the sm_100a tensor cores.
//
// Replaces the cuBLAS BF16 GEMM of Engine::gemm_core (native/src/engine.rs:4321-4350 in
// juanqui/decidra): same contraction, f32 accumulation, bf16 output.
//
// Design (one CTA per SM, persistent over output tiles, no clusters):
//   * tile 128 (M) x 256 (N), K sliced in 64-element (128-byte) blocks;
//   * warp 0   : TMA producer. cp.async.bulk.tensor.2d loads of the X tile (128x64) and the
//                W tile (256x64) into a 4-stage shared-memory ring, 128-byte swizzle;
//   * warp 1   : MMA issuer. One elected thread issues tcgen05.mma (M128 N256 K16,
//                kind::f16, bf16 in / f32 out) reading both operands from shared memory
//                through UMMA descriptors; accumulators live in TMEM (2 x 256 columns so
//                the epilogue of tile i overlaps the main loop of tile i+1);
//   * warps 2-5: epilogue. tcgen05.ld 32 lanes x 32 columns at a time, convert to bf16
//                (optionally SwiGLU-combine the two column halves), 16-byte global stores.
// Every mbarrier wait is bounded: when a wait gives up the kernel raises an error word,
// lets in-flight copies land, frees its TMEM and returns.
#include <cuda.h>

#include "common.cuh"
#include "gemm_tcgen05.h"
#include "tc_common.cuh"

namespace tcg {
using namespace tcc;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16, ACC_STAGES = 2;
constexpr uint32_t A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr uint32_t BAR_BYTES = 256;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + BAR_BYTES + 1024;
constexpr int GROUP_M = 16;  // default rasterisation: 16 M-tiles share each W tile while it is hot in L2 (see pick_group_m)

// Shared-memory operand descriptor: K-major tile, rows of 128 bytes, 128-byte swizzle,
// 8-row groups 1024 bytes apart. Bits: [0,14) address>>4, [16,30) leading offset>>4 (unused
// for swizzled K-major, set to 1), [32,46) stride offset>>4 = 64, [46,48) version 1,
// [61,64) layout 2 = SWIZZLE_128B.
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
  d |= (uint64_t)1 << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// Instruction descriptor: D f32 (bit 4); A/B format at bits 7 and 10 (kind::f16: 1 = bf16;
// kind::f8f6f4: 0 = e4m3); both K-major; N>>3 at [17,23), M>>4 at [24,29).
constexpr uint32_t IDESC_BF16 = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
constexpr uint32_t IDESC_E4M3 = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// ESZ 2: bf16 operands (kind::f16, K = 16 per instruction); ESZ 1: e4m3 operands (kind::f8f6f4, K = 32).
template <int ESZ>
__device__ __forceinline__ void umma(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  if (ESZ == 2) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(IDESC_BF16), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(da), "l"(db), "r"(IDESC_E4M3), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int group_m, int& m_idx, int& n_idx) {
  const int per_group = group_m * num_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int gsize = min(group_m, num_m - first_m);
  const int r = tile - g * per_group;
  m_idx = first_m + r % gsize;
  n_idx = r / gsize;
}

// EPI 0: C[M,N] bf16. EPI 1: SwiGLU — W rows are interleaved per 256-row tile as
// [128 gate rows | 128 up rows]; the kernel writes act[M, N/2] = bf16(bf16(silu(bf16(gate))) * bf16(up))
// (silu_mul_bf16, native/kernels/kernels.cu:492-501, applied to the bf16-rounded GEMM outputs).
// ESZ 1 (e4m3 operands): the accumulator is scaled by w_scale[column] * a_scale[row] before rounding
// (scale_fp8_gemm_bf16, native/kernels/kernels.cu:208-220); ESZ 2 ignores the scale pointers.
// alpha (device scalar, may be null): the accumulator is multiplied by *alpha before rounding
// (cuBLASLt alpha = 1/(weight_global*input_global) of the NVFP4 path, native/src/engine.rs:4108).
// resid (EPI 0, may be null; [M, ldc] like C): C = bf16(resid + bf16(product)), the residual add of add_bf16 /
// add_rmsnorm_bf16 (native/kernels/kernels.cu:406-426, 485-490) applied to the rounded GEMM output.
template <int EPI, int ESZ>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, bf16* __restrict__ C,
                    int M, int N, int K, int ldc, const float* __restrict__ a_scale, const float* __restrict__ w_scale,
                    const float* __restrict__ alpha, int* __restrict__ err, const bf16* __restrict__ resid, int group_m) {
  constexpr int BKE = 128 / ESZ;  // K elements per 128-byte swizzled row
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t tiles_base = raw + pad;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  const uint32_t bars_base = tiles_base + STAGES * STAGE_BYTES;
  // barrier layout: full[STAGES], empty[STAGES], tfull[ACC], tempty[ACC]
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * STAGES + ACC_STAGES + a); };
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2 * ACC_STAGES);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN, num_tiles = num_m * num_n;
  const int num_kb = (K + BKE - 1) / BKE;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < ACC_STAGES; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, group_m, m_idx, n_idx);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))) break;
          mbar_expect_tx(full_bar(stage), STAGE_BYTES);
          const uint32_t a_dst = tiles_base + stage * STAGE_BYTES;
          tma_load_2d(a_dst, &tmA, full_bar(stage), kb * BKE, m_idx * BM);
          tma_load_2d(a_dst + A_BYTES, &tmB, full_bar(stage), kb * BKE, n_idx * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!(ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(full_bar(stage), phase, abort_flag))) break;
          tc_fence_after();
          const uint32_t a_src = tiles_base + stage * STAGE_BYTES;
          const uint64_t da = make_desc(a_src), db = make_desc(a_src + A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            // advance 32 bytes (one instruction's K) inside the swizzled 128-byte row
            umma<ESZ>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit(tfull_bar(acc));
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // Epilogue warps 2..5; a warp may only touch TMEM lanes 32*(warp%4) .. +31.
    const int lane_base = 32 * (warp & 3);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_idx, n_idx;
      tile_coords(tile, num_m, num_n, group_m, m_idx, n_idx);
      ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const int row = m_idx * BM + lane_base + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(acc * BN);
      const float rs = (ESZ == 1 && row < M) ? a_scale[row] : 1.0f;
      const float al = alpha ? __ldg(alpha) : 1.0f;
      if (EPI == 0) {
        bf16* crow = C + (size_t)row * ldc + (size_t)n_idx * BN;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = n_idx * BN + c * 32 + v * 8;
              if (col + 8 <= N) {
                float f[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]) * al;
                if (ESZ == 1) {
                  const float4 w0 = __ldg(reinterpret_cast<const float4*>(w_scale + col));
                  const float4 w1 = __ldg(reinterpret_cast<const float4*>(w_scale + col + 4));
                  f[0] = f[0] * w0.x * rs; f[1] = f[1] * w0.y * rs; f[2] = f[2] * w0.z * rs; f[3] = f[3] * w0.w * rs;
                  f[4] = f[4] * w1.x * rs; f[5] = f[5] * w1.y * rs; f[6] = f[6] * w1.z * rs; f[7] = f[7] * w1.w * rs;
                }
                if (resid) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(resid + (size_t)row * ldc + col);
                  const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] = Ty<bf16>::rnd(f[2 * j]) + __uint_as_float(rw[j] << 16);
                    f[2 * j + 1] = Ty<bf16>::rnd(f[2 * j + 1]) + __uint_as_float(rw[j] & 0xffff0000u);
                  }
                }
                uint4 o;
                o.x = pack_bf16(f[0], f[1]);
                o.y = pack_bf16(f[2], f[3]);
                o.z = pack_bf16(f[4], f[5]);
                o.w = pack_bf16(f[6], f[7]);
                *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = o;
              }
            }
          }
        }
      } else {
        // gate = columns [0,128), up = columns [128,256) of this tile → 128 output columns
        bf16* crow = C + (size_t)row * ldc + (size_t)n_idx * (BN / 2);
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld32(taddr + c * 32, g);
          tmem_ld32(taddr + BN / 2 + c * 32, u);
          tmem_ld_wait();
          if (row < M) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = n_idx * (BN / 2) + c * 32 + v * 8;
              if (col + 8 <= ldc) {  // ldc = true output width I (the interleaved N/2 may be padded)
                float a[8];
                float wg[8], wu[8];
                if (ESZ == 1) {
                  const int gcol = n_idx * BN + c * 32 + v * 8;  // interleaved row index of the gate weights
                  *reinterpret_cast<float4*>(&wg[0]) = __ldg(reinterpret_cast<const float4*>(w_scale + gcol));
                  *reinterpret_cast<float4*>(&wg[4]) = __ldg(reinterpret_cast<const float4*>(w_scale + gcol + 4));
                  *reinterpret_cast<float4*>(&wu[0]) = __ldg(reinterpret_cast<const float4*>(w_scale + gcol + BN / 2));
                  *reinterpret_cast<float4*>(&wu[4]) = __ldg(reinterpret_cast<const float4*>(w_scale + gcol + BN / 2 + 4));
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float ga = __uint_as_float(g[v * 8 + j]) * al, ua = __uint_as_float(u[v * 8 + j]) * al;
                  if (ESZ == 1) { ga = ga * wg[j] * rs; ua = ua * wu[j] * rs; }
                  const float gg = Ty<bf16>::rnd(ga);
                  const float uu = Ty<bf16>::rnd(ua);
                  a[j] = Ty<bf16>::rnd(__fdividef(gg, 1.0f + __expf(-gg))) * uu;
                }
                uint4 o;
                o.x = pack_bf16(a[0], a[1]);
                o.y = pack_bf16(a[2], a[3]);
                o.z = pack_bf16(a[4], a[5]);
                o.w = pack_bf16(a[6], a[7]);
                *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = o;
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    // A wait gave up: report, then give copies and MMAs already in flight time to land
    // before shared memory and TMEM are released.
    if (threadIdx.x == 0) set_err(err, DERR_GEMM_TIMEOUT);
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

}  // namespace tcg

// Row-major [rows, cols] bf16 matrix, box = box_rows x 64 columns, 128-byte swizzle, zero fill
// outside the matrix.
int tc_make_tmap(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  static_assert(sizeof(TcTensorMap) == sizeof(CUtensorMap), "tensor map size");
  auto fn = tcg::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols * 2};
  cuuint32_t box[2] = {(cuuint32_t)tcg::BK, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
// Row-major [rows, cols] bf16 view with an explicit row stride (elements); box = box_rows x 64.
int tc_make_tmap_strided(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows) {
  auto fn = tcg::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride * 2};
  cuuint32_t box[2] = {64, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
// [d2, d1, d0] bf16 tensor (d0 contiguous), strides in elements; box = box2 x box1 x 64.
int tc_make_tmap_3d(TcTensorMap* out, const void* ptr, uint64_t d0, uint64_t d1, uint64_t d2, uint64_t stride1, uint64_t stride2,
                    uint32_t box1, uint32_t box2) {
  auto fn = tcg::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1 * 2, stride2 * 2};
  cuuint32_t box[3] = {64, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
// Row-major [rows, cols] f32 view with an explicit row stride (elements); box = box_rows x 32 columns
// (128 bytes), 128-byte swizzle, zero fill outside the matrix. Feeds kind::tf32 operands.
int tc_make_tmap_f32(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint64_t row_stride, uint32_t box_rows) {
  auto fn = tcg::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {row_stride * 4};
  cuuint32_t box[2] = {32, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box,
                  estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
int tc_make_tmap_a(TcTensorMap* out, const void* X, uint64_t M, uint64_t K) { return tc_make_tmap(out, X, M, K, tcg::BM); }
int tc_make_tmap_b(TcTensorMap* out, const void* W, uint64_t N, uint64_t K) { return tc_make_tmap(out, W, N, K, tcg::BN); }

bool tc_shape_ok(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && (K % 8) == 0 && (N % 8) == 0; }

cudaError_t tc_gemm_prepare_device() {
  CUDA_TRY(cudaFuncSetAttribute(tcg::gemm_bf16_tc_kernel<0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tcg::SMEM_BYTES));
  CUDA_TRY(cudaFuncSetAttribute(tcg::gemm_bf16_tc_kernel<1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, tcg::SMEM_BYTES));
  CUDA_TRY(cudaFuncSetAttribute(tcg::gemm_bf16_tc_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, tcg::SMEM_BYTES));
  CUDA_TRY(cudaFuncSetAttribute(tcg::gemm_bf16_tc_kernel<1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, tcg::SMEM_BYTES));
  return cudaSuccess;
}

// M tiles per rasterisation group. A group sweeps all N tiles with its M tiles innermost, so the W panel streams from DRAM once
// per group while the group's rows of X stay in L2: fewer, larger groups re-read W less. The override is for measurements.
static int g_group_m_override = 0;
void tc_gemm_set_group_m(int group_m) { g_group_m_override = group_m; }
static int pick_group_m(int M, int K, int esz) {
  (void)K; (void)esz;
  const int num_m = (M + tcg::BM - 1) / tcg::BM;
  int g = g_group_m_override > 0 ? g_group_m_override : tcg::GROUP_M;
  return g < num_m ? g : (num_m > 0 ? num_m : 1);
}

cudaError_t tc_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, void* C, int M, int N, int K, int ldc, int epi,
                           int sm_count, int* err, cudaStream_t stream, const float* alpha, const void* resid) {
  if (resid && epi != 0) return cudaErrorInvalidValue;
  const int num_tiles = ((M + tcg::BM - 1) / tcg::BM) * ((N + tcg::BN - 1) / tcg::BN);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  const CUtensorMap& a = *reinterpret_cast<const CUtensorMap*>(tmA);
  const CUtensorMap& b = *reinterpret_cast<const CUtensorMap*>(tmB);
  if (epi == 0) tcg::gemm_bf16_tc_kernel<0, 2><<<grid, tcg::NUM_THREADS, tcg::SMEM_BYTES, stream>>>(a, b, (bf16*)C, M, N, K, ldc, nullptr, nullptr, alpha, err, (const bf16*)resid, pick_group_m(M, K, 2));
  else tcg::gemm_bf16_tc_kernel<1, 2><<<grid, tcg::NUM_THREADS, tcg::SMEM_BYTES, stream>>>(a, b, (bf16*)C, M, N, K, ldc, nullptr, nullptr, alpha, err, nullptr, pick_group_m(M, K, 2));
  return cudaGetLastError();
}

// e4m3 operands (1 byte per element; maps made with tc_make_tmap_fp8_*), bf16 output scaled by
// w_scale[n] * a_scale[m].
cudaError_t tc_gemm_fp8_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, void* C, int M, int N, int K, int ldc, int epi,
                               const float* a_scale, const float* w_scale, int sm_count, int* err, cudaStream_t stream, const void* resid) {
  if (resid && epi != 0) return cudaErrorInvalidValue;
  const int num_tiles = ((M + tcg::BM - 1) / tcg::BM) * ((N + tcg::BN - 1) / tcg::BN);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  const CUtensorMap& a = *reinterpret_cast<const CUtensorMap*>(tmA);
  const CUtensorMap& b = *reinterpret_cast<const CUtensorMap*>(tmB);
  if (epi == 0) tcg::gemm_bf16_tc_kernel<0, 1><<<grid, tcg::NUM_THREADS, tcg::SMEM_BYTES, stream>>>(a, b, (bf16*)C, M, N, K, ldc, a_scale, w_scale, nullptr, err, (const bf16*)resid, pick_group_m(M, K, 1));
  else tcg::gemm_bf16_tc_kernel<1, 1><<<grid, tcg::NUM_THREADS, tcg::SMEM_BYTES, stream>>>(a, b, (bf16*)C, M, N, K, ldc, a_scale, w_scale, nullptr, err, nullptr, pick_group_m(M, K, 1));
  return cudaGetLastError();
}

// Row-major [rows, cols] e4m3 (1 byte) matrix, box = box_rows x 128 columns, 128-byte swizzle.
static int make_tmap_u8(TcTensorMap* out, const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  auto fn = tcg::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {cols};
  cuuint32_t box[2] = {128, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}
int tc_make_tmap_fp8_a(TcTensorMap* out, const void* X, uint64_t M, uint64_t K) { return make_tmap_u8(out, X, M, K, tcg::BM); }
int tc_make_tmap_fp8_b(TcTensorMap* out, const void* W, uint64_t N, uint64_t K) { return make_tmap_u8(out, W, N, K, tcg::BN); }
bool tc_fp8_shape_ok(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && (K % 16) == 0 && (N % 8) == 0; }
