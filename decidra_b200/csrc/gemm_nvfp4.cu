// C[M,N] = alpha * (Xq . Wq^T) for NVFP4 operands on the sm_100a block-scaled tensor-core path:
// e2m1 codes (two per byte), one unsigned e4m3 scale per 16 elements along K, f32 accumulation
// (tcgen05.mma kind::mxf4nvf4.block_scale, 16-element blocks), bf16 output.
//
// Replaces the cuBLASLt block-scaled FP4 GEMM of Engine::nvfp4_gemm (native/src/engine.rs:3962-4131
// in juanqui/decidra): same operand formats (codes K-major, scales in the 128 x 4 tiled layout that
// cuBLASLt and the reference's quantisers use: tile (row block of 128, group of 4 scales) is 512
// bytes with scale (r, g) at (r % 32) * 16 + (r / 32) * 4 + g), alpha = 1 / (weight_global *
// input_global) applied to the accumulator before rounding.
//
// Structure (one CTA per SM, persistent over 128 x 128 output tiles, K in 256-element = 128-byte blocks):
//   warps 0, 6, 7: producers, one thread each. Per K block: the X codes tile (128 rows x 128 bytes, TMA, 128-byte
//           swizzle), the W codes tile, and two plain bulk copies of 2 KB (the four 512-byte scale tiles of each
//           operand, contiguous in the tiled layout) into a 5-stage ring. One thread issuing all four copies
//           (about 100 cycles each) was slower than the four MMAs they feed;
//   warp 1: MMA issuer. Copies the eight scale tiles of the stage into TMEM (tcgen05.cp 32x128b.warpx4: a
//           512-byte tile becomes 4 columns, lane r % 32 of every 32-lane quarter holding the four scales
//           of rows r, r+32, r+64, r+96 in its four columns) and issues 4 MMAs (M128 N128 K64);
//   warps 2-5: epilogue. tcgen05.ld, * alpha, bf16, 16-byte stores; two accumulators of 128 columns so
//           the epilogue of a tile overlaps the main loop of the next.
// TMEM: columns 0-255 accumulators, 256 + 32*stage: 16 columns of X scales then 16 of W scales.
// Rows beyond M or N read the TMA zero fill for codes; their scale tiles exist (the scale buffers are
// padded to whole 128-row blocks) and whatever they hold multiplies zeros or lands in rows/columns that
// are not stored.
// Every mbarrier wait is bounded: when a wait gives up the kernel raises an error word, lets in-flight
// copies land, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "gemm_tcgen05.h"
#include "tc_common.cuh"

namespace nvg {
using namespace tcc;

// Two tile widths: BN = 128 (5 stages, two accumulators) and BN = 256 (4 stages, one accumulator: TMEM holds 256
// accumulator columns plus 48 scale columns per stage, so the epilogue of a tile does not overlap the next main loop,
// but every MMA and every scale copy covers twice the columns).
constexpr int BM = 128, BKB = 128 /* bytes of codes per row per K block = 256 elements */;
constexpr uint32_t A_BYTES = BM * BKB, SF_BYTES = 2048;
template <int BN> struct Cfg {
  static constexpr int STAGES = BN == 128 ? 5 : 4, ACC_STAGES = BN == 128 ? 2 : 1, NB = BN / 128 /* 128-row scale blocks of W per tile */;
  static constexpr uint32_t B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES + (1 + NB) * SF_BYTES;
  static constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
  static constexpr uint32_t SF_COLS = 16 + 16 * NB;  // per stage: 16 columns of X scales, then 4 * NB per K step of W scales
  // block-scaled instruction descriptor: A/B format e2m1 (1) at bits 7 and 10, N>>3 at [17,23), scale format
  // UE4M3 (0) at bit 23, M>>4 at [24,29), K = 64 (bit 31 = 0), scale-factor ids 0
  static constexpr uint32_t IDESC = (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
};
constexpr int NUM_THREADS = 320;        // BN 128: warps 0 / 6 / 7 producers, 1 MMA issuer, 2-5 epilogue, 8 and 9 scale copiers
constexpr int NUM_THREADS_WIDE = 480;   // BN 256: four more epilogue warps (9-12) and scale copiers 8, 13, 14. There is one accumulator, so
                                        // the next tile's MMAs wait for the epilogue: eight warps first drain it into registers as bf16
                                        // pairs (32 rows x 128 columns each), hand it back, and only then add, activate, quantise and
                                        // store, beside the next main loop
// A thread issues one tcgen05.cp every 57 cycles (measured; the instruction itself completes faster: three threads of three warps
// issue three in 57). A stage needs 4 + 4 NB of them and its four MMAs run for 256 (BN 128) or 512 cycles (BN 256), so one copier
// (12 x 57 = 684 cycles per stage at BN 256) holds the tensor core back; the copies are therefore spread over 1 + NB threads, one
// for the X scales and one per 128-row block of W scales, each committing to the stage's barrier (count 1 + NB).
constexpr uint32_t SF_COL = 256;
constexpr int GROUP_M = 16;

__device__ __forceinline__ uint64_t desc_sw128(uint32_t smem_addr) {  // K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t desc_sf(uint32_t smem_addr) {  // 32 rows of 16 bytes, no swizzle, 8-row groups 128 bytes apart
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}
__device__ __forceinline__ void cp_sf(uint32_t tmem_col, uint64_t sdesc) {
  asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(sdesc) : "memory");
}
__device__ __forceinline__ void umma_fp4(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "setp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.scale_vec::4X [%0], %1, %2, %3, [%5], [%6], p;\n"
      "}\n" ::"r"(tmem_d),
      "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
      : "memory");
}
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
               : "memory");
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

// Activation quantiser for the block-scaled GEMM: bf16 rows (tensor scale 1) -> e2m1 codes [rows, K/2] and e4m3 scales
// written straight into the 128 x 4 tiled layout. Same rule as quant_nvfp4_act_bf16 / fp4_encode
// (native/kernels/kernels.cu:222-277): sf = e4m3_satfinite(max(absmax16/6, 1e-10)), code = fp4_encode(v / decode(sf)).
// The codes come from the e2m1 conversion instruction, steered onto fp4_encode's rule on exact ties, -0 and decode(sf) = 0
// (nvfp4_codes8 in common.cuh says how). One thread per 64 elements (four scale groups = one 32-bit word of a tile).
// 16 values (already bf16-representable) -> scale byte and two words of codes
__device__ __forceinline__ void quant_group16(const float (&v)[16], uint32_t& c0, uint32_t& c1, uint32_t& sb_out) {
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
// SPLIT: the scale tiles are copied into TMEM by threads of their own (one per 2 KB scale set of the stage, each in a warp of
// its own) that signal the MMA issuer through one more barrier per stage, so that the copies of a K block are not queued in front of that block's MMAs on the issuer's in-order
// stream of tensor-core work.
// EPI 0: C[M, ldc] = bf16(alpha * acc), or with resid (bf16 [M, ldc]): bf16(resid + bf16(alpha * acc)), the residual add of a
// pre-norm block (add_bf16 / add_rmsnorm_bf16, native/kernels/kernels.cu:378-404, 485-490) applied to the rounded product.
// EPI 1 (BN = 256; W rows interleaved per tile as 128 gate rows then the matching 128 up rows): the tile's 128 activations
// bf16(bf16(silu(bf16(gate))) * bf16(up)) (silu_mul_bf16, native/kernels/kernels.cu:492-501) are quantised to NVFP4 on the spot,
// 16 at a time (quant_nvfp4_act_bf16's rule), as the down projection's operand: codes to q_packed [M, ldc / 2], scales into the
// 128 x 4 tiled layout q_tiled (ldc = the activation width I). Neither the gate/up matrix nor the bf16 activation reach memory.
template <int BN, bool SPLIT, int EPI>
__global__ void __launch_bounds__(BN == 256 ? NUM_THREADS_WIDE : NUM_THREADS, 1)
gemm_nvfp4_tc_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const uint8_t* __restrict__ sfa,
                     const uint8_t* __restrict__ sfb, bf16* __restrict__ C, int M, int N, int K, int ldc, const float* __restrict__ alpha,
                     int* __restrict__ err, const bf16* __restrict__ resid, uint8_t* __restrict__ q_packed, uint8_t* __restrict__ q_tiled) {
  using CF = Cfg<BN>;
  constexpr int STAGES = CF::STAGES, ACC_STAGES = CF::ACC_STAGES, NB = CF::NB;
  constexpr uint32_t B_BYTES = CF::B_BYTES, STAGE_BYTES = CF::STAGE_BYTES;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t tiles_base = raw + pad;
  const uint32_t bars_base = tiles_base + STAGES * STAGE_BYTES;
  auto full_bar = [&](int s) { return bars_base + 8u * s; };
  auto empty_bar = [&](int s) { return bars_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int a) { return bars_base + 8u * (2 * STAGES + a); };
  auto tempty_bar = [&](int a) { return bars_base + 8u * (2 * STAGES + ACC_STAGES + a); };
  auto sfull_bar = [&](int s) { return bars_base + 8u * (2 * STAGES + 2 * ACC_STAGES + s); };  // scales of the stage are in TMEM
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(smem + STAGES * STAGE_BYTES + 8 * (3 * STAGES + 2 * ACC_STAGES));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;
  const int num_m = (M + BM - 1) / BM, num_n = (N + BN - 1) / BN, num_tiles = num_m * num_n;
  const int num_kb = K / 256;      // K blocks of 256 elements
  const int kb64 = K / 64;         // 512-byte scale tiles per 128-row block

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
      mbar_init(sfull_bar(s), SPLIT ? 1 + NB : 1);
    }
    for (int a = 0; a < ACC_STAGES; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), ACC_STAGES == 1 ? 8 : 4);
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

  // the tcgen05.cp copies of one stage: X scales of K step k into 4 columns, W scales 4 columns per 128-row block, blocks side by side
  auto copy_scales = [&](uint32_t src, uint32_t sf_tmem) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      cp_sf(sf_tmem + 4 * k, desc_sf(src + A_BYTES + B_BYTES + 512 * k));
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) cp_sf(sf_tmem + 16 + 4 * NB * k + 4 * nb, desc_sf(src + A_BYTES + B_BYTES + (1 + nb) * SF_BYTES + 512 * k));
    }
  };

  constexpr int COPIER1 = BN == 256 ? 13 : 9;  // warp of the second copier; the first is warp 8
  const int copier = warp == 8 ? 0 : (warp >= COPIER1 && warp < COPIER1 + NB) ? warp - COPIER1 + 1 : -1;
  if (copier >= 0) {
    if (SPLIT) {
      // Scale copiers: number 0 takes the X scales, number 1 + nb the W scales of 128-row block nb. A stage's TMEM columns are
      // rewritten only after the MMAs that read them have completed: the producers refill the stage after empty_bar, and these
      // warps wait for the refill. (Every role below: the whole warp runs the loop, the elected lane issues.)
      const bool el = elect_one();
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait_warp(full_bar(stage), phase, abort_flag))) break;
          tc_fence_after();
          const uint32_t src = tiles_base + stage * STAGE_BYTES + A_BYTES + B_BYTES + (uint32_t)copier * SF_BYTES;
          const uint32_t col = tmem_base + SF_COL + (uint32_t)stage * CF::SF_COLS + (copier == 0 ? 0u : 16u + 4u * (uint32_t)(copier - 1));
          if (el) {
#pragma unroll
            for (int k = 0; k < 4; ++k) cp_sf(col + (copier == 0 ? 4 : 4 * NB) * k, desc_sf(src + 512 * k));
            umma_commit_to(sfull_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 0 || warp == 6 || warp == 7) {
    {
      const bool el = elect_one();
      // warp 0: X codes (and the expected byte count of the stage); warp 6: W codes; warp 7: both scale sets
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        int m_idx, n_idx;
        tile_coords(tile, num_m, num_n, m_idx, n_idx);
        const uint8_t* sa = sfa + ((size_t)m_idx * kb64) * 512;
        const uint8_t* sb = sfb + ((size_t)n_idx * NB * kb64) * 512;  // first of the NB 128-row scale blocks of this W tile
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!(ok = mbar_wait_warp(empty_bar(stage), phase ^ 1u, abort_flag))) break;
          const uint32_t dst = tiles_base + stage * STAGE_BYTES;
          if (!el) {
          } else if (warp == 0) {
            mbar_expect_tx(full_bar(stage), STAGE_BYTES);
            tma_load_2d(dst, &tmA, full_bar(stage), kb * BKB, m_idx * BM);
          } else if (warp == 6) {
            tma_load_2d(dst + A_BYTES, &tmB, full_bar(stage), kb * BKB, n_idx * BN);
          } else {
            bulk_load(dst + A_BYTES + B_BYTES, sa + (size_t)kb * SF_BYTES, SF_BYTES, full_bar(stage));
#pragma unroll
            for (int nb = 0; nb < NB; ++nb)
              bulk_load(dst + A_BYTES + B_BYTES + (1 + nb) * SF_BYTES, sb + ((size_t)nb * kb64) * 512 + (size_t)kb * SF_BYTES, SF_BYTES, full_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    {
      const bool el = elect_one();
      int stage = 0, acc = 0;
      uint32_t phase = 0, acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!(ok = mbar_wait_warp(tempty_bar(acc), acc_phase ^ 1u, abort_flag))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + (uint32_t)(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          const uint32_t src = tiles_base + stage * STAGE_BYTES;
          const uint32_t sf_tmem = tmem_base + SF_COL + (uint32_t)stage * CF::SF_COLS;
          if (SPLIT) {
            // the copiers commit to sfull_bar after they have seen full_bar (codes and scales of the stage, one byte count),
            // so this one wait covers both; a second wait only lengthens this thread's stream of about 57 cycles per tcgen05
            // instruction, which is what the tensor core waits for (measured: 548 -> 623 us on the gate/up shape)
            if (!(ok = mbar_wait_warp(sfull_bar(stage), phase, abort_flag))) break;
            tc_fence_after();
          } else {
            if (!(ok = mbar_wait_warp(full_bar(stage), phase, abort_flag))) break;
            tc_fence_after();
            if (el) copy_scales(src, sf_tmem);
          }
          const uint64_t da = desc_sw128(src), db = desc_sw128(src + A_BYTES);
          if (el) {
#pragma unroll
            for (int k = 0; k < 4; ++k)  // 64 elements = 32 bytes of codes per instruction
              umma_fp4(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), CF::IDESC, sf_tmem + 4 * k, sf_tmem + 16 + 4 * NB * k, (kb | k) != 0 ? 1u : 0u);
            umma_commit_to(empty_bar(stage));
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (el) umma_commit_to(tfull_bar(acc));
        if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    const int lane_base = 32 * (warp & 3);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const float al = alpha ? __ldg(alpha) : 1.0f;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
      int m_idx, n_idx;
      tile_coords(tile, num_m, num_n, m_idx, n_idx);
      const int row = m_idx * BM + lane_base + lane;
      ok = mbar_wait(tfull_bar(acc), acc_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)lane_base << 16) + (uint32_t)(acc * BN);
      if constexpr (ACC_STAGES == 1) {
        // Drain first: four 32-column chunks of this thread's row, scaled, rounded to bf16 and packed in pairs. EPI 0: the chunks
        // of one half of the tile; EPI 1: two gate chunks and the two up chunks that go with them.
        const int slot = warp < 9 ? 0 : 1;
        uint32_t pk[64];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = EPI == 1 ? (i < 2 ? 2 * slot + i : 2 + 2 * slot + i) : 4 * slot + i;
          uint32_t r[32];
          tmem_ld32(taddr + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) pk[16 * i + j] = pack_bf16(__uint_as_float(r[2 * j]) * al, __uint_as_float(r[2 * j + 1]) * al);
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));  // the next tile's MMAs may overwrite the accumulator from here on
        if constexpr (EPI == 0) {
          if (row < M) {
            bf16* crow = C + (size_t)row * ldc + (size_t)n_idx * BN;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = 4 * slot + i;
#pragma unroll
              for (int v = 0; v < 4; ++v) {
                const int col = n_idx * BN + c * 32 + v * 8;
                if (col + 8 <= N) {
                  uint32_t o[4] = {pk[16 * i + 4 * v], pk[16 * i + 4 * v + 1], pk[16 * i + 4 * v + 2], pk[16 * i + 4 * v + 3]};
                  if (resid) {
                    const uint4 rv = *reinterpret_cast<const uint4*>(resid + (size_t)row * ldc + col);
                    const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                      o[j] = pack_bf16(__uint_as_float(o[j] << 16) + __uint_as_float(rw[j] << 16),
                                       __uint_as_float(o[j] & 0xffff0000u) + __uint_as_float(rw[j] & 0xffff0000u));
                  }
                  *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                }
              }
            }
          }
        } else {
          // gate = columns [0,128), up = columns [128,256) of this tile -> 128 activations per row; gate chunk c and up chunk c
          // give outputs [32 c, 32 c + 32): two scale groups = 16 bytes of codes and two bytes of the tiled scale layout
          const int chunks = ldc / 64;
#pragma unroll
          for (int i = 0; i < 2; ++i) {
            const int c = 2 * slot + i;
            uint8_t* prow = q_packed + (size_t)row * (ldc / 2) + (size_t)n_idx * (BN / 4) + c * 16;
            uint32_t sb2 = 0u;
#pragma unroll
            for (int grp = 0; grp < 2; ++grp) {
              float v[16];
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const uint32_t gw = pk[16 * i + 8 * grp + j], uw = pk[32 + 16 * i + 8 * grp + j];
                const float g0 = __uint_as_float(gw << 16), g1 = __uint_as_float(gw & 0xffff0000u);
                const float u0 = __uint_as_float(uw << 16), u1 = __uint_as_float(uw & 0xffff0000u);
                v[2 * j] = Ty<bf16>::rnd(Ty<bf16>::rnd(__fdividef(g0, 1.0f + __expf(-g0))) * u0);
                v[2 * j + 1] = Ty<bf16>::rnd(Ty<bf16>::rnd(__fdividef(g1, 1.0f + __expf(-g1))) * u1);
              }
              uint32_t c0, c1, sb;
              quant_group16(v, c0, c1, sb);
              if (row < M) *reinterpret_cast<uint2*>(prow + grp * 8) = make_uint2(c0, c1);
              sb2 |= sb << (8 * grp);
            }
            if (row < M) {
              uint8_t* trow = q_tiled + ((size_t)(row >> 7) * chunks + (size_t)n_idx * 2 + (c >> 1)) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (c & 1) * 2;
              *reinterpret_cast<uint16_t*>(trow) = (uint16_t)sb2;
            }
          }
        }
      } else {
        // two accumulators: this epilogue already runs beside the next tile's main loop
        bf16* crow = C + (size_t)row * ldc + (size_t)n_idx * BN;
#pragma unroll
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
                if (resid) {
                  const uint4 rv = *reinterpret_cast<const uint4*>(resid + (size_t)row * ldc + col);
                  const uint32_t rw[4] = {rv.x, rv.y, rv.z, rv.w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) {
                    f[2 * j] = Ty<bf16>::rnd(f[2 * j]) + __uint_as_float(rw[j] << 16);
                    f[2 * j + 1] = Ty<bf16>::rnd(f[2 * j + 1]) + __uint_as_float(rw[j] & 0xffff0000u);
                  }
                }
                *reinterpret_cast<uint4*>(crow + c * 32 + v * 8) = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
              }
            }
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
      }
      if (++acc == ACC_STAGES) { acc = 0; acc_phase ^= 1u; }
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
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// scales [rows, K/16] row-major -> `blocks` 128-row blocks of the 128 x 4 tiled layout (rows beyond `rows` zero)
__global__ void sf_tile_kernel(const uint8_t* __restrict__ lin, uint8_t* __restrict__ tiled, int rows, int groups, int blocks) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int kb64 = groups / 4;
  const size_t total = (size_t)blocks * kb64 * 512;
  if (i >= total) return;
  const size_t tile = i / 512;
  const int in = (int)(i - tile * 512);
  const int rb = (int)(tile / kb64), kc = (int)(tile - (size_t)rb * kb64);
  const int r = rb * 128 + (in >> 4) + ((in >> 2) & 3) * 32, g = kc * 4 + (in & 3);
  tiled[i] = r < rows ? lin[(size_t)r * groups + g] : (uint8_t)0;
}

__device__ __forceinline__ void unpack16(const uint4& lo, const uint4& hi, float (&v)[16]) {
  const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    v[2 * i] = __uint_as_float(w[i] << 16);
    v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
__device__ __forceinline__ void store_chunk64(uint8_t* packed, uint8_t* tiled, int row, int ch, int chunks, int K, const uint32_t (&codes)[8], uint32_t sfw) {
  uint4* dst = reinterpret_cast<uint4*>(packed + (size_t)row * (K / 2) + ch * 32);
  dst[0] = make_uint4(codes[0], codes[1], codes[2], codes[3]);
  dst[1] = make_uint4(codes[4], codes[5], codes[6], codes[7]);
  *reinterpret_cast<uint32_t*>(tiled + ((size_t)(row >> 7) * chunks + ch) * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4) = sfw;
}

__global__ void __launch_bounds__(128) act_quant_tiled_kernel(const bf16* __restrict__ x, size_t x_stride, uint8_t* __restrict__ packed,
                                                              uint8_t* __restrict__ tiled, int rows, int K) {
  const int chunks = K / 64;
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (size_t)rows * chunks) return;
  const int row = (int)(t / chunks), ch = (int)(t - (size_t)row * chunks);
  const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)row * x_stride + ch * 64);
  uint32_t codes[8];
  uint32_t sfw = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float v[16];
    unpack16(src[2 * g], src[2 * g + 1], v);
    uint32_t sb;
    quant_group16(v, codes[2 * g], codes[2 * g + 1], sb);
    sfw |= sb << (8 * g);
  }
  store_chunk64(packed, tiled, row, ch, chunks, K, codes, sfw);
}

// SwiGLU over the tile-interleaved gate/up GEMM output (each 256-column tile: 128 gate then 128 up columns), rounded as
// silu_mul_bf16 does (native/kernels/kernels.cu:492-501: bf16(bf16(silu(g)) * u)), quantised on the spot: the bf16
// activation matrix is never written. One thread per 64 outputs.
__global__ void __launch_bounds__(128) swiglu_quant_tiled_kernel(const bf16* __restrict__ gu, int gu_stride, uint8_t* __restrict__ packed,
                                                                 uint8_t* __restrict__ tiled, int rows, int I) {
  const int chunks = I / 64;
  const size_t t = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= (size_t)rows * chunks) return;
  const int row = (int)(t / chunks), ch = (int)(t - (size_t)row * chunks);
  const int c0 = ch * 64;
  const uint4* gsrc = reinterpret_cast<const uint4*>(gu + (size_t)row * gu_stride + (size_t)(c0 >> 7) * 256 + (c0 & 127));
  const uint4* usrc = gsrc + 16;  // + 128 columns
  uint32_t codes[8];
  uint32_t sfw = 0;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    float gv[16], uv[16], v[16];
    unpack16(gsrc[2 * g], gsrc[2 * g + 1], gv);
    unpack16(usrc[2 * g], usrc[2 * g + 1], uv);
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = Ty<bf16>::rnd(Ty<bf16>::rnd(__fdividef(gv[i], 1.0f + __expf(-gv[i]))) * uv[i]);
    uint32_t sb;
    quant_group16(v, codes[2 * g], codes[2 * g + 1], sb);
    sfw |= sb << (8 * g);
  }
  store_chunk64(packed, tiled, row, ch, chunks, I, codes, sfw);
}

}  // namespace nvg

bool nvfp4_tc_shape_ok(int M, int N, int K) { return M > 0 && N > 0 && K > 0 && (K % 256) == 0 && (N % 8) == 0; }
size_t nvfp4_sf_tiled_bytes(int rows, int K) { return (size_t)((rows + 255) / 256) * 2 * (K / 64) * 512; }

cudaError_t nvfp4_gemm_prepare_device() {
#define NVG_SMEM(BN_, SP_, EPI_) \
  CUDA_TRY(cudaFuncSetAttribute(nvg::gemm_nvfp4_tc_kernel<BN_, SP_, EPI_>, cudaFuncAttributeMaxDynamicSharedMemorySize, nvg::Cfg<BN_>::SMEM_BYTES))
  NVG_SMEM(128, false, 0);
  NVG_SMEM(128, true, 0);
  NVG_SMEM(256, false, 0);
  NVG_SMEM(256, true, 0);
  NVG_SMEM(256, false, 1);
  NVG_SMEM(256, true, 1);
#undef NVG_SMEM
  return cudaSuccess;
}
cudaError_t launch_nvfp4_act_quant_tiled(const bf16* x, size_t x_stride, uint8_t* packed, uint8_t* tiled, int rows, int K, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if ((K % 64) || (x_stride % 8)) return cudaErrorInvalidValue;
  const size_t n = (size_t)rows * (K / 64);
  nvg::act_quant_tiled_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(x, x_stride, packed, tiled, rows, K);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_swiglu_quant_tiled(const bf16* gu, int gu_stride, uint8_t* packed, uint8_t* tiled, int rows, int I, cudaStream_t s) {
  if (rows <= 0) return cudaSuccess;
  if ((I % 128) || (gu_stride % 8)) return cudaErrorInvalidValue;
  const size_t n = (size_t)rows * (I / 64);
  nvg::swiglu_quant_tiled_kernel<<<(unsigned)((n + 127) / 128), 128, 0, s>>>(gu, gu_stride, packed, tiled, rows, I);
  return cudaGetLastError();
}
cudaError_t launch_nvfp4_sf_tile(const uint8_t* lin, uint8_t* tiled, int rows, int K, cudaStream_t s, bool pad_even) {
  // pad_even: as the GEMM wants its operands (nvfp4_sf_tiled_bytes); otherwise whole 128-row blocks only, as the reference's repack
  const int blocks = pad_even ? (rows + 255) / 256 * 2 : (rows + 127) / 128;
  const size_t total = (size_t)blocks * (K / 64) * 512;
  if (!total) return cudaSuccess;
  nvg::sf_tile_kernel<<<(unsigned)((total + 255) / 256), 256, 0, s>>>(lin, tiled, rows, K / 16, blocks);
  return cudaGetLastError();
}
// tmA: byte map over the X codes [M, K/2] with 128-row boxes (tc_make_tmap_fp8_a); tmB: the same over the W codes with bn-row boxes
// (tc_make_tmap_fp8_a for bn 128, tc_make_tmap_fp8_b for bn 256).
cudaError_t nvfp4_gemm_launch(const TcTensorMap* tmA, const TcTensorMap* tmB, const uint8_t* sfa_tiled, const uint8_t* sfb_tiled, void* C, int M,
                              int N, int K, int ldc, const float* alpha, int sm_count, int* err, cudaStream_t stream, int bn, const void* resid,
                              uint8_t* q_packed, uint8_t* q_tiled) {
  const bool split = bn >= 1000;  // bn 1128 / 1256: the variant with the scale copies on a thread of their own
  if (split) bn -= 1000;
  const bool swiglu_quant = q_packed != nullptr;
  if (!nvfp4_tc_shape_ok(M, N, K) || (bn != 128 && bn != 256)) return cudaErrorInvalidValue;
  if (swiglu_quant && (bn != 256 || resid || !q_tiled || (N % 256) || (ldc % 128) || N != 2 * ldc)) return cudaErrorInvalidValue;
  const int num_tiles = ((M + nvg::BM - 1) / nvg::BM) * ((N + bn - 1) / bn);
  const int grid = num_tiles < sm_count ? num_tiles : sm_count;
  const CUtensorMap& a = *reinterpret_cast<const CUtensorMap*>(tmA);
  const CUtensorMap& b = *reinterpret_cast<const CUtensorMap*>(tmB);
  const bf16* rs = (const bf16*)resid;
#define NVG_LAUNCH(BN_, SP_, EPI_)                                                                                                              \
  nvg::gemm_nvfp4_tc_kernel<BN_, SP_, EPI_><<<grid, BN_ == 256 ? nvg::NUM_THREADS_WIDE : nvg::NUM_THREADS, nvg::Cfg<BN_>::SMEM_BYTES, stream>>>( \
      a, b, sfa_tiled, sfb_tiled, (bf16*)C, M, N, K, ldc, alpha, err, rs, q_packed, q_tiled)
  if (swiglu_quant) { if (split) NVG_LAUNCH(256, true, 1); else NVG_LAUNCH(256, false, 1); }
  else if (bn == 128) { if (split) NVG_LAUNCH(128, true, 0); else NVG_LAUNCH(128, false, 0); }
  else { if (split) NVG_LAUNCH(256, true, 0); else NVG_LAUNCH(256, false, 0); }
#undef NVG_LAUNCH
  return cudaGetLastError();
}
