// C[M,N] = X[M,K] . dequant(Wq)[N,K]^T with int4 group-128 weights, on the sm_100a tensor cores, without a bf16 copy of W.
//
// Replaces the Marlin W4A16 GEMM of juanqui/decidra (native/kernels/marlin.cu:398-408) and its fallback route
// dequant_w4a16_bf16 + BF16 GEMM (native/src/engine.rs:4516-4558, native/kernels/kernels.cu:867-892): every weight is
// w = bf16(float(q - 8) * float(scale)) exactly as the reference rounds it, then enters a bf16 x bf16 -> f32 product.
// The result is bit-identical to dequantising into a bf16 matrix and running gemm_bf16_tc_kernel on it (same MMA shape and
// the same order of K steps per accumulator).
//
// One CTA per SM, persistent over 256 x 256 output tiles (two M128 accumulators share every dequantised W tile, which halves
// the dequantisation work per FLOP against a 128-row tile), K in blocks of 64:
//   warp 16: TMA of the two X half tiles (128 x 64 bf16 each, 128-byte swizzle) into a 3-stage ring;
//   warp 17: TMA of the packed W tile (256 rows x 32 bytes, 32-byte swizzle so that the workers' 16-byte reads spread over all
//            banks) and a bulk copy of the tile's 256 group scales into a 3-slot ring;
//   warps 0-15 ("workers", thread t owns half h = t / 256 of W row t % 256 of the tile): read the half row's 4 words, turn 32
//            nibbles into bf16 and write 64 bytes of the K-major B operand with the swizzle the MMA descriptor expects. The
//            loop of a worker is a chain of waits (packed words, free B slot) and fences, so it takes many warps to keep the
//            ALUs busy: with 8 warps (a whole row per thread) a K block took ~1600 cycles against 1024 of MMA time. After the
//            last K block of a tile the same warps are the epilogue (warp w: TMEM lanes 32 (w % 4)..., accumulator (w / 4) % 2,
//            columns 128 (w / 8)...);
//   warp 18: MMA issuer: 2 x 4 tcgen05.mma (M128 N256 K16, kind::f16) per K block; TMEM holds the two accumulators (512 columns).
// Dequantisation, 2.4 instructions per weight, bit-exact: the engine stores each word's nibbles in the order
// [k0 k2 k4 k6 k1 k3 k5 k7], so (w >> 4p) & 0x000F000F | 0x43004300 is the bf16 pair (128 + q[2p], 128 + q[2p+1]); minus 136
// gives (q - 8) exactly; with the fp16 scale split as s = s_hi + s_lo (s_hi = bf16(s); s_lo has at most 3 significant bits),
// (q-8)*s_lo is exact in bf16 and fma(q-8, s_hi, (q-8)*s_lo) rounds the exact product once to bf16: bf16(float(q-8)*float(s)).
// Scales come from a transposed copy [K/128][N], so that the 256 scales a tile needs for a K block are 512 contiguous bytes: they
// travel with the packed words (a load from global memory in the worker loop stalled every group on its latency).
// Every mbarrier wait is bounded; a wait that gives up raises the error word, the CTA drains and frees its TMEM.
#include <cuda.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "gemm_tcgen05.h"
#include "tc_common.cuh"

namespace w4g {
using namespace tcc;

constexpr int BM = 256, BN = 256, BK = 64, STAGES = 3, PSTAGES = 3;
constexpr uint32_t A_HALF = 128 * BK * 2, A_BYTES = 2 * A_HALF, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;  // 64 KB
constexpr uint32_t PK_BYTES = BN * (BK / 2), SC_BYTES = BN * 2, P_BYTES = PK_BYTES + SC_BYTES;  // 8 KB of words + the tile's 256 fp16 scales
constexpr int WORKER_WARPS = 16, A_WARP = 16, P_WARP = 17, MMA_WARP = 18, NUM_THREADS = 608;
constexpr uint32_t BAR_BYTES = 256;
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + PSTAGES * P_BYTES + BAR_BYTES + 1024;
constexpr int GROUP_M = 8;  // rasterisation: 8 M-tiles (2048 rows) share each W tile while it is hot in L2
constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);

__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {  // K-major, 128-byte rows, 128-byte swizzle, 8-row groups 1024 B apart
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ void tile_coords(int tile, int num_m, int num_n, int& m_idx, int& n_idx) {
  const int per_group = GROUP_M * num_n;
  const int g = tile / per_group;
  const int first_m = g * GROUP_M;
  const int gsize = min(GROUP_M, num_m - first_m);
  const int r = tile - g * per_group;
  m_idx = first_m + r % gsize;
  n_idx = r / gsize;
}

// one stored word (nibble order k0 k2 k4 k6 k1 k3 k5 k7) -> 8 bf16 in K order
__device__ __forceinline__ uint4 dequant_word(uint32_t w, __nv_bfloat162 s_hi, __nv_bfloat162 s_lo) {
  const __nv_bfloat162 c136 = __floats2bfloat162_rn(136.f, 136.f);
  uint32_t o[4];
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const uint32_t y = ((w >> (4 * p)) & 0x000F000Fu) | 0x43004300u;
    const __nv_bfloat162 q = __hsub2(*reinterpret_cast<const __nv_bfloat162*>(&y), c136);
    const __nv_bfloat162 r = __hfma2(q, s_hi, __hmul2(q, s_lo));
    o[p] = *reinterpret_cast<const uint32_t*>(&r);
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

// EPI 0: C[M,N] bf16 (+ optional residual: C = bf16(resid + bf16(product))). EPI 1: SwiGLU over gate/up-interleaved W rows
// (per 256-row tile: 128 gate rows, then the matching 128 up rows): act[M, N/2] = bf16(bf16(silu(bf16(gate))) * bf16(up)).
template <int EPI>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_w4a16_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmP, const __half* __restrict__ scale_t,
                     bf16* __restrict__ C, int M, int N, int K, int ldc, int* __restrict__ err, const bf16* __restrict__ resid) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t tiles_base = raw + pad;
  const uint32_t p_base = tiles_base + STAGES * STAGE_BYTES;
  const uint32_t bars_base = p_base + PSTAGES * P_BYTES;
  uint8_t* bars_ptr = smem + STAGES * STAGE_BYTES + PSTAGES * P_BYTES;
  auto full_a = [&](int s) { return bars_base + 8u * s; };                                // TMA bytes of the X tiles
  auto full_b = [&](int s) { return bars_base + 8u * (STAGES + s); };                      // all 512 worker threads wrote their part of B
  auto empty_bar = [&](int s) { return bars_base + 8u * (2 * STAGES + s); };               // the MMAs of the stage are done
  auto pfull = [&](int s) { return bars_base + 8u * (3 * STAGES + s); };                   // TMA bytes of the packed tile
  auto pempty = [&](int s) { return bars_base + 8u * (3 * STAGES + PSTAGES + s); };        // 16 worker warps read it
  const uint32_t tfull = bars_base + 8u * (3 * STAGES + 2 * PSTAGES), tempty = tfull + 8;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars_ptr + 8 * (3 * STAGES + 2 * PSTAGES + 2));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN, num_tiles = num_m * num_n;
  const int num_kb = K / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_a(s), 1);
      mbar_init(full_b(s), WORKER_WARPS * 32);
      mbar_init(empty_bar(s), 1);
    }
    for (int s = 0; s < PSTAGES; ++s) {
      mbar_init(pfull(s), 1);
      mbar_init(pempty(s), WORKER_WARPS);
    }
    mbar_init(tfull, 1);
    mbar_init(tempty, WORKER_WARPS);
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == MMA_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == A_WARP) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, m_idx, n_idx);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag))) break;
          mbar_expect_tx(full_a(stage), A_BYTES);
          const uint32_t dst = tiles_base + stage * STAGE_BYTES;
          tma_load_2d(dst, &tmA, full_a(stage), kb * BK, m_idx * BM);
          tma_load_2d(dst + A_HALF, &tmA, full_a(stage), kb * BK, m_idx * BM + 128);  // rows beyond M read the zero fill
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == P_WARP) {
    if (lane == 0) {
      int ps = 0;
      uint32_t pphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, m_idx, n_idx);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(pempty(ps), pphase ^ 1u, abort_flag))) break;
          const int n0 = n_idx * BN;
          const uint32_t sc_bytes = (uint32_t)min(BN, N - n0) * 2u;  // N % 8 == 0: a multiple of 16 bytes; rows beyond N keep stale scales
          mbar_expect_tx(pfull(ps), PK_BYTES + sc_bytes);
          tma_load_2d(p_base + ps * P_BYTES, &tmP, pfull(ps), kb * (BK / 2), n0);
          asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(p_base + ps * P_BYTES + PK_BYTES),
                       "l"(scale_t + (size_t)(kb >> 1) * N + n0), "r"(sc_bytes), "r"(pfull(ps))
                       : "memory");
          if (++ps == PSTAGES) { ps = 0; pphase ^= 1u; }
        }
      }
    }
  } else if (warp == MMA_WARP) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, m_idx, n_idx);
        const bool two = m_idx * BM + 128 < M;  // the second accumulator has rows to compute
        if (!(ok = mbar_wait(tempty, tphase ^ 1u, abort_flag))) break;
        tc_fence_after();
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait(full_a(stage), phase, abort_flag))) break;
          if (!(ok = mbar_wait(full_b(stage), phase, abort_flag))) break;
          tc_fence_after();
          const uint32_t src = tiles_base + stage * STAGE_BYTES;
          const uint64_t da0 = make_desc(src), da1 = make_desc(src + A_HALF), db = make_desc(src + A_BYTES);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_base, da0 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), IDESC, (kb | k) != 0 ? 1u : 0u);
          if (two) {
#pragma unroll
            for (int k = 0; k < 4; ++k) umma_f16(tmem_base + BN, da1 + (uint64_t)(k * 2), db + (uint64_t)(k * 2), IDESC, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_to(empty_bar(stage));
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        umma_commit_to(tfull);
        tphase ^= 1u;
      }
    }
  } else {
    // ---- workers: dequantise during the K loop, then store the tile -----------------------------------------------------
    const int row = threadIdx.x & 255, hh = threadIdx.x >> 8;  // W row of the tile and the half of it (32 of 64 weights) owned by this thread
    int stage = 0, ps = 0;
    uint32_t phase = 0, pphase = 0, tphase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_idx, n_idx;
      tile_coords(tile, num_m, num_n, m_idx, n_idx);
      const int n_row = n_idx * BN + row;
      const bool live = n_row < N;  // rows beyond N: zero scale (their packed words are the TMA zero fill)
      for (int kb = 0; kb < num_kb; ++kb) {
        ok = mbar_wait(pfull(ps), pphase, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const uint8_t* slot = smem + STAGES * STAGE_BYTES + ps * P_BYTES;
        // 32-byte swizzle of the TMA: the 16-byte half h of row r sits at chunk h ^ ((r >> 2) & 1)
        const uint4 w = *reinterpret_cast<const uint4*>(slot + row * 32 + ((hh ^ ((row >> 2) & 1)) << 4));
        const float sc = live ? __half2float(*reinterpret_cast<const __half*>(slot + PK_BYTES + row * 2)) : 0.f;
        const __nv_bfloat16 sh = __float2bfloat16_rn(sc);
        const __nv_bfloat16 sl = __float2bfloat16_rn(sc - __bfloat162float(sh));
        const __nv_bfloat162 s_hi = __halves2bfloat162(sh, sh), s_lo = __halves2bfloat162(sl, sl);
        uint4 o[4];
        o[0] = dequant_word(w.x, s_hi, s_lo);
        o[1] = dequant_word(w.y, s_hi, s_lo);
        o[2] = dequant_word(w.z, s_hi, s_lo);
        o[3] = dequant_word(w.w, s_hi, s_lo);
        // the packed slot is handed back only now that the words have been consumed (the loads have certainly returned)
        __syncwarp();
        if (lane == 0) mbar_arrive(pempty(ps));
        if (++ps == PSTAGES) { ps = 0; pphase ^= 1u; }
        ok = mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag);  // the MMAs that read this B slot are done
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after();
        uint8_t* brow = smem + stage * STAGE_BYTES + A_BYTES + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c) *reinterpret_cast<uint4*>(brow + (((hh * 4 + c) ^ (row & 7)) << 4)) = o[c];
        // Every thread makes its own stores visible to the tensor core's (async proxy) reads and then signals for itself. (With one
        // elected arrival per warp behind a __syncwarp, and the packed slot released right after the loads, two runs of the kernel
        // disagreed on long K loops.)
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        mbar_arrive(full_b(stage));
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
      if (!ok) break;
      // ---- epilogue of this tile: warp w reads TMEM lanes 32 (w % 4) .. + 31 of accumulator (w / 4) % 2, its half of the columns ---
      ok = mbar_wait(tfull, tphase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tphase ^= 1u;
      tc_fence_after();
      const int half = (warp >> 2) & 1, ch = warp >> 3, lane_base = 32 * (warp & 3);  // accumulator, column half, TMEM lane quarter
      const int orow = m_idx * BM + half * 128 + lane_base + lane;
      const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(half * BN);
      if (m_idx * BM + half * 128 < M) {
        if (EPI == 0) {
          bf16* crow = C + (size_t)orow * ldc + (size_t)n_idx * BN;
#pragma unroll 1
          for (int c = ch * (BN / 64); c < (ch + 1) * (BN / 64); ++c) {
            uint32_t r[32];
            tmem_ld32(taddr + c * 32, r);
            tmem_ld_wait();
            if (orow < M) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const int col = n_idx * BN + c * 32 + v * 8;
                if (col + 8 <= N) {
                  float f[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) f[j] = __uint_as_float(r[v * 8 + j]);
                  if (resid) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(resid + (size_t)orow * ldc + col);
                    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                      f[2 * j] = Ty<bf16>::rnd(f[2 * j]) + __uint_as_float(rw[j] << 16);
                      f[2 * j + 1] = Ty<bf16>::rnd(f[2 * j + 1]) + __uint_as_float(rw[j] & 0xffff0000u);
                    }
                  }
                  uint4 ov;
                  ov.x = pack_bf16(f[0], f[1]);
                  ov.y = pack_bf16(f[2], f[3]);
                  ov.z = pack_bf16(f[4], f[5]);
                  ov.w = pack_bf16(f[6], f[7]);
                  *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = ov;
                }
              }
            }
          }
        } else {
          bf16* crow = C + (size_t)orow * ldc + (size_t)n_idx * (BN / 2);
#pragma unroll 1
          for (int c = ch * (BN / 128); c < (ch + 1) * (BN / 128); ++c) {
            uint32_t g[32], u[32];
            tmem_ld32(taddr + c * 32, g);
            tmem_ld32(taddr + BN / 2 + c * 32, u);
            tmem_ld_wait();
            if (orow < M) {
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const int col = n_idx * (BN / 2) + c * 32 + v * 8;
                if (col + 8 <= ldc) {  // ldc = true output width (the interleaved N/2 may be padded)
                  float a[8];
#pragma unroll
                  for (int j = 0; j < 8; ++j) {
                    const float gg = Ty<bf16>::rnd(__uint_as_float(g[v * 8 + j]));
                    const float uu = Ty<bf16>::rnd(__uint_as_float(u[v * 8 + j]));
                    a[j] = Ty<bf16>::rnd(__fdividef(gg, 1.0f + __expf(-gg))) * uu;
                  }
                  uint4 ov;
                  ov.x = pack_bf16(a[0], a[1]);
                  ov.y = pack_bf16(a[2], a[3]);
                  ov.z = pack_bf16(a[4], a[5]);
                  ov.w = pack_bf16(a[6], a[7]);
                  *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = ov;
                }
              }
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) set_err(err, DERR_GEMM_TIMEOUT);
#pragma unroll 1
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == MMA_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// ---- the engine's own int4 image: nibble order [k0 k2 k4 k6 k1 k3 k5 k7] per word, scales transposed to [groups][N] ----------
__device__ __host__ __forceinline__ uint32_t nibble_permute(uint32_t w) {
  uint32_t o = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) o |= ((w >> (4 * j)) & 0xFu) << (4 * ((j & 1) * 4 + (j >> 1)));
  return o;
}
__global__ void w4_repack_kernel(const uint32_t* __restrict__ packed, uint32_t* __restrict__ out, size_t words) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < words) out[i] = nibble_permute(packed[i]);
}
__global__ void w4_scale_transpose_kernel(const __half* __restrict__ scales, __half* __restrict__ out, int N, int groups) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (size_t)N * groups) return;
  const int g = (int)(i / N), n = (int)(i - (size_t)g * N);
  out[i] = scales[(size_t)n * groups + g];
}

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

}  // namespace w4g

bool w4a16_tc_shape_ok(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && (K % 128) == 0 && (N % 8) == 0; }

// Which route a launch takes. Measured on a B200 (N = 10240, K = 5120; fused kernel against dequantisation pass + bf16 kernel):
// M = 64: 70 vs 74 us, M = 512: 77 vs 105 us, M = 2048: 222 vs 195 us, M = 6835: 589 vs 535 us (gate/up at M = 6835: 1868 vs
// 1774 us). The fused kernel wins while the pass is bound by streaming the weights (4.5 bytes per weight by the two-step route,
// 0.5 here); in the tensor-bound regime it reaches 0.87-0.93 of the bf16 kernel's rate (the dequantising warps share the SM's
// issue slots and power budget with the tensor core, and the single set of accumulators leaves the epilogue uncovered), which
// is less than the 4-7 % the separate dequantisation pass costs. Both routes give the same bits.
bool w4a16_tc_prefer(int M, int N, int sm_count) {
  (void)N;
  (void)sm_count;
  return M <= 640;
}

cudaError_t w4a16_gemm_prepare_device() {
  CUDA_TRY(cudaFuncSetAttribute(w4g::gemm_w4a16_tc_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, w4g::SMEM_BYTES));
  CUDA_TRY(cudaFuncSetAttribute(w4g::gemm_w4a16_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, w4g::SMEM_BYTES));
  return cudaSuccess;
}

// packed words [N, K/8] as bytes [N, K/2]; box = 256 rows x 32 bytes (one K block), 32-byte swizzle, zero fill beyond N
int w4a16_make_tmap_packed(TcTensorMap* out, const void* packed, uint64_t N, uint64_t K) {
  auto fn = w4g::encode_fn();
  if (!fn) return -1;
  cuuint64_t dims[2] = {K / 2, N};
  cuuint64_t strides[1] = {K / 2};
  cuuint32_t box[2] = {(cuuint32_t)(w4g::BK / 2), (cuuint32_t)w4g::BN};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(packed), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : (int)r;
}

cudaError_t launch_w4_repack(const uint32_t* packed, uint32_t* out, size_t words, cudaStream_t s) {
  if (!words) return cudaSuccess;
  w4g::w4_repack_kernel<<<(unsigned)((words + 255) / 256), 256, 0, s>>>(packed, out, words);
  return cudaGetLastError();
}
cudaError_t launch_w4_scale_transpose(const void* scales, void* out, int N, int groups, cudaStream_t s) {
  const size_t n = (size_t)N * groups;
  if (!n) return cudaSuccess;
  w4g::w4_scale_transpose_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>((const __half*)scales, (__half*)out, N, groups);
  return cudaGetLastError();
}

// tmA: the bf16 activation map of tc_make_tmap_a (128-row boxes); tmP: w4a16_make_tmap_packed over the permuted words;
// scale_t: fp16 [K/128][N]. epi / resid as tc_gemm_launch.
cudaError_t w4a16_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmP, const void* scale_t, void* C, int M, int N, int K, int ldc, int epi,
                              int sm_count, int* err, cudaStream_t stream, const void* resid) {
  if (!w4a16_tc_shape_ok(M, N, K) || (resid && epi != 0)) return cudaErrorInvalidValue;
  const int num_tiles = ((M + w4g::BM - 1) / w4g::BM) * ((N + w4g::BN - 1) / w4g::BN);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  const CUtensorMap& a = *reinterpret_cast<const CUtensorMap*>(tmA);
  const CUtensorMap& p = *reinterpret_cast<const CUtensorMap*>(tmP);
  if (epi == 0)
    w4g::gemm_w4a16_tc_kernel<0><<<grid, w4g::NUM_THREADS, w4g::SMEM_BYTES, stream>>>(a, p, (const __half*)scale_t, (bf16*)C, M, N, K, ldc, err, (const bf16*)resid);
  else
    w4g::gemm_w4a16_tc_kernel<1><<<grid, w4g::NUM_THREADS, w4g::SMEM_BYTES, stream>>>(a, p, (const __half*)scale_t, (bf16*)C, M, N, K, ldc, err, nullptr);
  return cudaGetLastError();
}
