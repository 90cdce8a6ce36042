// Varlen prefix-bidirectional attention on the sm_100a tensor cores (bf16, head_dim 256).
//
// Replaces, for the whole packed batch in ONE launch per layer, what juanqui/decidra does with
// (2+2B) device copies and B FlashInfer launches per layer (Engine::full_attention_batch cascade
// branch, native/src/engine.rs:1985-2042; fi_prefill_bf16_ext,
// native/third_party/flashinfer/fi_prefill.cu:161-173), plus the sigmoid output gate
// (sigmoid_gate_bf16, native/kernels/kernels.cu:504-512). Each question attends, without a causal
// mask, to [cached state K/V || its own K/V]; the two segments are read in place through two pairs
// of TMA descriptors — nothing is concatenated.
//
// One CTA = (question, KV head, tile of 128/G tokens), G = query heads per KV head. The G heads of
// a token share K/V, so the M=128 MMA tile is packed with (token, head) rows by a 3-D TMA box
// {64 dims, G heads, 128/G tokens}. Keys stream in tiles of 128:
//   S[128,128] = Q[128,256] . K^T        tcgen05.mma, Q and K from shared memory, S in TMEM. K arrives as four
//                64-dim slabs (16 KB) through a ring of five slab slots; the products of a slab are issued as
//                soon as it lands and the slot is handed back when they are done, so the loads run about a tile
//                ahead of the tensor core with 80 KB of shared memory instead of two whole K tiles
//   softmax    : threads r and r+128 own row r, 64 key columns each: tcgen05.ld S, base-2 online softmax with
//                a lazy rescale (O is only rescaled when the running max grows by more than 2^8), P -> bf16
//                written back over S in TMEM. The scores stay unscaled in registers: the maximum is taken on
//                them and 1/sqrt(d)*log2(e) rides in the multiply-add in front of ex2.approx.ftz; only a
//                partial last tile pays for the column mask (11 -> ~7 instructions per score)
//   O[128,256] += P[128,128] . V[128,256] tcgen05.mma, P as the TMEM A operand, V (one 64 KB slot, refilled as
//                soon as the product that read it is done) as an MN-major shared-memory operand, O in TMEM
// S is double-buffered in TMEM (2 x 128 columns beside the 256 of O): S of tile j+1 is issued before the softmax
// of tile j is awaited, so the tensor core works on S[j+1] and P.V[j-1] while the threads run the softmax of
// tile j. With 128-key tiles every S instruction is 128 x 128 x 16 (the 64-wide ones ran at about a third of
// their nominal rate) and the per-tile costs of the softmax (barrier waits, the exchange of the row maximum
// between the two threads of a row, TMEM load/store round trips) are paid half as often.
// Warps 0-7 are the softmax/epilogue warps: warps w and w+4 share TMEM lanes 32w..32w+31 (they exchange the row
// maximum through shared memory once per tile and their partial denominators once at the end); one thread of
// warp 8 issues the MMAs, one of warp 9 loads Q and the K slabs, one of warp 10 the V tiles, so that no wait
// sits behind another.
// Few rows over a long state leave most SMs without a CTA, so the key tiles of a (token tile, KV head) can be split over
// gridDim.z CTAs: each takes a contiguous range of tiles, leaves its unnormalised O with the maximum and denominator it is
// relative to in a workspace, and attn_merge_kernel adds the parts up with the base-2 identity of the reference's
// merge_attn_lse_bf16 (native/kernels/kernels.cu:461-483; the reference takes the same decision inside FlashInfer's planner,
// native/third_party/flashinfer/fi_prefill.cu:42-86), normalises, applies the output gate and stores.
// All waits are bounded; a wait that gives up raises the error word and the CTA drains and exits.
#include <cuda.h>

#include "attn_tcgen05.h"
#include "common.cuh"
#include "tc_common.cuh"

namespace atc {
using namespace tcc;

constexpr int HD = 256, KT = 128, NKB = HD / 64;
constexpr uint32_t Q_KB_BYTES = 128 * 128, Q_BYTES = NKB * Q_KB_BYTES;          // 64 KB
constexpr uint32_t KV_CHUNK = KT * 128;                                         // one 64-dim slab of a K or V tile: 16 KB
constexpr int K_SLOTS = 5;                                                       // ring of K slabs (a K tile is NKB = 4 slabs)
constexpr uint32_t K_RING_BYTES = K_SLOTS * KV_CHUNK, V_BYTES = NKB * KV_CHUNK;  // 80 KB, 64 KB
constexpr uint32_t XCH_BYTES = 2 * 256 * 4;  // row-maximum exchange, two sets of 2 x 128 floats
constexpr uint32_t SMEM_BYTES = Q_BYTES + K_RING_BYTES + V_BYTES + XCH_BYTES + 256 + 1024;
constexpr int NUM_THREADS = 352;
constexpr int ISSUER_WARP = 8, K_LOADER_WARP = 9, V_LOADER_WARP = 10;
constexpr uint32_t O_COL = 0, S_COL = 256;  // O 256 columns, S 2 x 128
constexpr uint32_t IDESC_QK = umma_idesc(128, KT, 0);
constexpr uint32_t IDESC_PV = umma_idesc(128, HD, 1);
constexpr float RESCALE_THRESHOLD = 8.0f;  // log2 units

// 2^x by the special-function unit alone (inputs below -126 give 0, which is what a masked or far-away key should weigh)
__device__ __forceinline__ float ex2_ftz(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// the same, kept in program order behind the barrier arrive that precedes it (so that the work stays between an arrive and its wait)
__device__ __forceinline__ float ex2_ftz_ordered(float x) {
  float y;
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// The output gate: sigmoid with the hardware exponential and reciprocal approximations (about 2 ulp in f32). Its result is rounded to
// bf16 straight away (sigmoid_gate_bf16, native/kernels/kernels.cu:504-512, rounds there too), which hides the difference except on
// rare rounding ties; the accurate expf and division cost about 25 instructions per element, 128 elements per thread, and made the
// epilogue a third of a CTA's time at 2048 keys (30 k of 93 k cycles).
__device__ __forceinline__ float sigmoid_gate(float g) { return __fdividef(1.0f, 1.0f + __expf(-g)); }

struct Params {
  const int32_t* cu;       // [B+1] packed sequence offsets
  const int32_t* tile_cu;  // [B+1] prefix sum of token tiles per sequence
  int B, n_state, heads, kv, total_tokens;
  const bf16* gate_qg;     // fused q projection [T, qg_stride]; gate = dims [hd, 2hd) of each head; may be null
  int qg_stride;
  bf16* out;               // [T, heads, hd]
  float scale_log2e;
  int* err;
  float* ws_o;             // gridDim.z > 1: unnormalised partial outputs [CTA][128 rows][256]
  float2* ws_ml;           //                (maximum in log2 units, denominator) [CTA][128 rows]
};

template <int G>
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmKs,
               const __grid_constant__ CUtensorMap tmVs, const __grid_constant__ CUtensorMap tmKo,
               const __grid_constant__ CUtensorMap tmVo, const Params p) {
  constexpr int TT = 128 / G;  // tokens per tile
  // ---- which (sequence, token tile) is this CTA? ------------------------------------------------
  const int ti = blockIdx.x, kh = blockIdx.y;
  if (ti >= p.tile_cu[p.B]) return;
  int b = 0;
  {
    int lo = 0, hi = p.B;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.tile_cu[mid] <= ti) lo = mid; else hi = mid;
    }
    b = lo;
  }
  const int off = p.cu[b], L = p.cu[b + 1] - off;
  const int t0 = (ti - p.tile_cu[b]) * TT;
  const int ntok = min(TT, L - t0);
  const int n_st = (p.n_state + KT - 1) / KT, n_own = (L + KT - 1) / KT, n_all = n_st + n_own;
  // this CTA's range of key tiles [j_lo, j_lo + n_tiles); j below counts from j_lo
  const int per_split = (n_all + (int)gridDim.z - 1) / (int)gridDim.z;
  const int j_lo = (int)blockIdx.z * per_split, n_tiles = max(0, min(n_all, j_lo + per_split) - j_lo);
  const size_t cta_lin = ((size_t)blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;
  if (n_tiles == 0) {  // more parts than tiles: an empty part
    if (gridDim.z > 1 && threadIdx.x < 128) p.ws_ml[cta_lin * 128 + threadIdx.x] = make_float2(-INFINITY, 0.f);
    return;
  }

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = smem_u32(smem_raw);
  const uint32_t pad = ((raw + 1023u) & ~1023u) - raw;
  uint8_t* smem = smem_raw + pad;
  const uint32_t q_base = raw + pad;
  const uint32_t k_base = q_base + Q_BYTES;
  const uint32_t v_base = k_base + K_RING_BYTES;
  const uint32_t bars = v_base + V_BYTES + XCH_BYTES;
  float* xch = reinterpret_cast<float*>(smem + Q_BYTES + K_RING_BYTES + V_BYTES);
  uint8_t* bars_ptr = smem + Q_BYTES + K_RING_BYTES + V_BYTES + XCH_BYTES;
  // bar_s / bar_p: two each (by tile parity); k_full / k_empty: one pair per K slab slot
  const uint32_t bar_q = bars, bar_v = bars + 24, bar_s = bars + 40, bar_p = bars + 56, bar_o = bars + 72;
  const uint32_t k_full = bars + 128, k_empty = bars + 128 + 8 * K_SLOTS;
  // bar_o counts one phase per tile and its waiters test a phase PARITY, which is only sound while the barrier is at most one
  // phase behind what they wait for. That holds for the V loader (in lockstep) and for the rescale (S[j] done implies P.V[j-2]
  // done: the tensor core runs the issuer's instructions in order), but not for the epilogue: the softmax can finish the last
  // tile while P.V of the tile before it still waits for its V tile, and the parity of the last phase then reads as complete.
  // The end of the last product therefore has a barrier of its own, used once.
  const uint32_t bar_done = k_empty + 8 * K_SLOTS;
  static_assert(128 + 16 * K_SLOTS + 8 <= 256, "barrier area");
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars_ptr + 80);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(bars_ptr + 84);

  const int warp = uniform_warp_idx(), lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    mbar_init(bar_v, 1);
    mbar_init(bar_s, 1);
    mbar_init(bar_s + 8, 1);
    mbar_init(bar_p, 256);
    mbar_init(bar_p + 8, 256);
    mbar_init(bar_o, 1);
    mbar_init(bar_done, 1);
    for (int i = 0; i < 4; ++i) mbar_init(bars + 88 + 8 * i, 64);  // one per pair of softmax warps
    for (int i = 0; i < K_SLOTS; ++i) {
      mbar_init(k_full + 8 * i, 1);
      mbar_init(k_empty + 8 * i, 1);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  // rows TT*G .. 127 of the Q tile are never written by TMA: zero them so that they stay finite
  if (threadIdx.x < 128) {
    constexpr int ROW0 = TT * G;
    constexpr int NZ = (128 - ROW0) * 8;  // 16-byte chunks per k-block
    for (int i = threadIdx.x; i < NKB * NZ; i += 128) {
      const int kb = i / NZ, c = i - kb * NZ;
      *reinterpret_cast<uint4*>(smem + kb * Q_KB_BYTES + ROW0 * 128 + c * 16) = make_uint4(0, 0, 0, 0);
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  if (warp == ISSUER_WARP) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)), "r"(512u) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  // The three roles below run as whole warps with uniform control flow; the elected lane executes the asynchronous instructions.
  if (warp == K_LOADER_WARP) {
    {
      // ---- K loader: Q once, then the K slabs (tile j, 64-dim slab c) through a ring that runs ahead of the S products --
      const bool el = elect_one();
      if (el) {
        mbar_expect_tx(bar_q, (uint32_t)(NKB * TT * G * 128));
#pragma unroll
        for (int c = 0; c < NKB; ++c) tma_load_3d(q_base + c * Q_KB_BYTES, &tmQ, bar_q, c * 64, kh * G, off + t0);
      }
      bool ok = true;
      const int n_slabs = n_tiles * NKB;
      for (int i = 0; i < n_slabs && ok; ++i) {
        const int slot = i % K_SLOTS, use = i / K_SLOTS, j = i / NKB, c = i % NKB;
        if (use >= 1 && !(ok = mbar_wait_warp(k_empty + 8 * slot, (uint32_t)((use - 1) & 1), abort_flag))) break;
        const bool st = j_lo + j < n_st;
        const int row0 = st ? (j_lo + j) * KT : off + (j_lo + j - n_st) * KT;
        if (el) {
          mbar_expect_tx(k_full + 8 * slot, KV_CHUNK);
          tma_load_2d(k_base + slot * KV_CHUNK, st ? &tmKs : &tmKo, k_full + 8 * slot, kh * HD + c * 64, row0);
        }
      }
    }
  } else if (warp == V_LOADER_WARP) {
    {
      // ---- V loader: one tile slot, refilled as soon as the P.V product that read it is done ----------------------------
      const bool el = elect_one();
      bool ok = true;
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j >= 1 && !(ok = mbar_wait_warp(bar_o, (uint32_t)((j - 1) & 1), abort_flag))) break;
        const bool st = j_lo + j < n_st;
        const int row0 = st ? (j_lo + j) * KT : off + (j_lo + j - n_st) * KT;
        if (el) {
          mbar_expect_tx(bar_v, V_BYTES);
#pragma unroll
          for (int c = 0; c < NKB; ++c) tma_load_2d(v_base + c * KV_CHUNK, st ? &tmVs : &tmVo, bar_v, kh * HD + c * 64, row0);
        }
      }
    }
  } else if (warp == ISSUER_WARP) {
    {
      // ---- MMA issuer --------------------------------------------------------------------------------------------
      const bool el = elect_one();
      bool ok = mbar_wait_warp(bar_q, 0, abort_flag);
      auto issue_s = [&](int j) {  // S[j] = Q K[j]^T into S buffer j & 1, one 64-dim slab at a time as the slabs land
        const int s = j & 1;
        for (int c = 0; c < NKB && ok; ++c) {
          const int i = j * NKB + c, slot = i % K_SLOTS, use = i / K_SLOTS;
          if (!(ok = mbar_wait_warp(k_full + 8 * slot, (uint32_t)(use & 1), abort_flag))) break;
          tc_fence_after();
          const uint64_t dq = umma_desc(q_base + c * Q_KB_BYTES, 16, 1024);
          const uint64_t dk = umma_desc(k_base + slot * KV_CHUNK, 16, 1024);
          if (el) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
              umma_f16(tmem_base + S_COL + s * KT, dq + (uint64_t)(k * 2), dk + (uint64_t)(k * 2), IDESC_QK, (c | k) != 0 ? 1u : 0u);
            umma_commit_to(k_empty + 8 * slot);  // the slab can be refilled once these products are done
          }
        }
        if (ok && el) umma_commit_to(bar_s + 8 * s);
      };
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j & 1;
        if (j + 1 < n_tiles) {  // S of the next tile goes to the tensor core before this tile's softmax is awaited
          issue_s(j + 1);
          if (!ok) break;
        }
        if (!(ok = mbar_wait_warp(bar_p + 8 * s, (uint32_t)((j >> 1) & 1), abort_flag))) break;
        if (!(ok = mbar_wait_warp(bar_v, (uint32_t)(j & 1), abort_flag))) break;
        tc_fence_after();
        const uint64_t dv = umma_desc(v_base, KV_CHUNK, 1024);
        if (el) {
#pragma unroll
          for (int k = 0; k < KT / 16; ++k)  // P[j] sits over S[j]: 16 keys = 8 packed columns per step
            umma_f16_ts(tmem_base + O_COL, tmem_base + S_COL + s * KT + k * 8, dv + (uint64_t)(k * (16 * 128 / 16)), IDESC_PV, (j | k) != 0 ? 1u : 0u);
          umma_commit_to(bar_o);
          if (j + 1 == n_tiles) umma_commit_to(bar_done);
        }
      }
    }
  } else {
    // ---- softmax + epilogue: threads r and r + 128 own row r of the tile, key columns [32h, 32h + 32) each ------
    const int r = threadIdx.x & 127, h = threadIdx.x >> 7;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t pair_bar = bars + 88 + 8 * (warp & 3);  // mbarrier of the two warps that share these rows (bounded wait)
    uint32_t pair_phase = 0;
    constexpr int HK = KT / 2;                 // key columns per thread
    float m_used = -INFINITY, l = 0.f;         // l: this thread's part of the denominator
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int jg = j_lo + j;
      const int valid = jg < n_st ? min(KT, p.n_state - jg * KT) : min(KT, L - (jg - n_st) * KT);
      ok = mbar_wait(bar_s + 8 * (j & 1), (uint32_t)((j >> 1) & 1), abort_flag);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after();
      // raw scores stay unscaled: the row maximum is taken on them (the scale is positive) and the scale is folded
      // into the exponent's multiply-add; only a partial last tile pays for the column mask
      float x[HK];
      {
        uint32_t v[HK];
        tmem_ld32(tmem_base + lane_addr + S_COL + (j & 1) * KT + h * HK, &v[0]);
        tmem_ld32(tmem_base + lane_addr + S_COL + (j & 1) * KT + h * HK + 32, &v[32]);
        tmem_ld_wait();
        if (valid == KT) {
#pragma unroll
          for (int i = 0; i < HK; ++i) x[i] = __uint_as_float(v[i]);
        } else {
#pragma unroll
          for (int i = 0; i < HK; ++i) x[i] = h * HK + i < valid ? __uint_as_float(v[i]) : -INFINITY;
        }
      }
      // P = exp2(x * scale - m_used) rounded to bf16, packed in pairs over this thread's half of S[j]; the denominator sums the
      // rounded values. From the second tile on the exponentials are taken against the maximum in use BEFORE this tile's own
      // maximum is known (it only changes when a row's maximum grows by more than 2^8, which is rare after the first tiles):
      // the maximum is folded into the first half of the loop, handed to the partner thread at the midpoint, and the partner's
      // value is read after the second half, so that neither the 64 max instructions nor the exchange sit in front of the
      // special-function unit. A row whose maximum did grow takes the exponentials again against the new one.
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      uint32_t w[HK / 2];
      auto pair = [&](int i, float neg_m, bool ordered) {
        const float a0 = fmaf(x[2 * i], p.scale_log2e, neg_m), a1 = fmaf(x[2 * i + 1], p.scale_log2e, neg_m);
        const __nv_bfloat162 pr = ordered ? __floats2bfloat162_rn(ex2_ftz_ordered(a0), ex2_ftz_ordered(a1)) : __floats2bfloat162_rn(ex2_ftz(a0), ex2_ftz(a1));
        w[i] = *reinterpret_cast<const uint32_t*>(&pr);
        l4[i & 3] += __uint_as_float(w[i] << 16) + __uint_as_float(w[i] & 0xffff0000u);
      };
      float* xs = xch + (j & 1) * 256;
      float tmax;
      {
        float t4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (j >= 1) {
          const float neg_m = -m_used;
#pragma unroll
          for (int i = 0; i < HK / 4; ++i) {
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) t4[q4] = fmaxf(t4[q4], x[4 * i + q4]);
            pair(i, neg_m, false);
          }
        } else {
#pragma unroll
          for (int i = 0; i < HK; ++i) t4[i & 3] = fmaxf(t4[i & 3], x[i]);
        }
        tmax = fmaxf(fmaxf(t4[0], t4[1]), fmaxf(t4[2], t4[3])) * p.scale_log2e;
      }
      xs[h * 128 + r] = tmax;
      mbar_arrive(pair_bar);
      if (j >= 1) {
        const float neg_m = -m_used;
#pragma unroll
        for (int i = HK / 4; i < HK / 2; ++i) pair(i, neg_m, true);
      }
      ok = mbar_wait(pair_bar, pair_phase, abort_flag);
      pair_phase ^= 1u;
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tmax = fmaxf(tmax, xs[(h ^ 1) * 128 + r]);
      const bool need = tmax > m_used + RESCALE_THRESHOLD;  // also true on the first tile (m_used = -inf); same for the pair
      if (j >= 1 && __any_sync(0xffffffffu, need)) {
        ok = mbar_wait(bar_o, (uint32_t)((j - 1) & 1), abort_flag);  // PV of tile j-1 done: O stable
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        {
          tc_fence_after();
          const float f = need ? exp2f(m_used - tmax) : 1.0f;
#pragma unroll 1
          for (int c = h * (HD / 64); c < (h + 1) * (HD / 64); ++c) {
            uint32_t v[32];
            tmem_ld32(tmem_base + lane_addr + O_COL + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * f);
            tmem_st32(tmem_base + lane_addr + O_COL + c * 32, v);
          }
          tmem_st_wait();
          l *= f;
        }
      }
      if (need) {  // the first tile, or a row whose maximum grew: the exponentials against the new maximum
        m_used = tmax;
        const float neg_m = -m_used;
        l4[0] = l4[1] = l4[2] = l4[3] = 0.f;
#pragma unroll
        for (int i = 0; i < HK / 2; ++i) pair(i, neg_m, false);
      }
      l += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      tmem_st32(tmem_base + lane_addr + S_COL + (j & 1) * KT + h * (HK / 2), w);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(bar_p + 8 * (j & 1));
    }
    // ---- epilogue: O / l, output gate, store (each thread of the pair takes half of the head dims) -----------------
    if (ok) {
      ok = mbar_wait(bar_done, 0, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after();
      float* xs = xch + (n_tiles & 1) * 256;  // the set the last tile did not use
      xs[h * 128 + r] = l;
      mbar_arrive(pair_bar);
      ok = mbar_wait(pair_bar, pair_phase, abort_flag);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && gridDim.z > 1) {
      // ---- a part of a split: unnormalised O (f32) and what it is relative to ---------------------------------------------
      float* xs = xch + (n_tiles & 1) * 256;
      l += xs[(h ^ 1) * 128 + r];
      if (h == 0) p.ws_ml[cta_lin * 128 + r] = make_float2(m_used, l);
      float* orow = p.ws_o + (cta_lin * 128 + r) * HD;
#pragma unroll 1
      for (int c = h * (HD / 64); c < (h + 1) * (HD / 64); ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_addr + O_COL + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q4 = 0; q4 < 8; ++q4)
          *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 4) = make_uint4(v[q4 * 4], v[q4 * 4 + 1], v[q4 * 4 + 2], v[q4 * 4 + 3]);
      }
    } else if (ok) {
      float* xs = xch + (n_tiles & 1) * 256;
      l += xs[(h ^ 1) * 128 + r];
      const int tt = r / G, g = r - tt * G;
      const bool live = tt < ntok;
      const int t = off + t0 + tt, head = kh * G + g;
      const float inv = 1.0f / l;
      bf16* orow = p.out + ((size_t)t * p.heads + head) * HD;
      const bf16* grow = p.gate_qg && live ? p.gate_qg + (size_t)t * p.qg_stride + (size_t)head * 2 * HD + HD : nullptr;
      // the gate values of a 32-column chunk are requested before the chunk's accumulator is read from TMEM, those of the next chunk
      // while this one is worked on, so that no load latency sits between the chunks
      uint4 gv[4], gn[4];
      const int c_lo = h * (HD / 64), c_hi = (h + 1) * (HD / 64);
      if (grow) {
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) gv[q4] = __ldg(reinterpret_cast<const uint4*>(grow + c_lo * 32 + q4 * 8));
      }
#pragma unroll 1
      for (int c = c_lo; c < c_hi; ++c) {
        uint32_t v[32];
        tmem_ld32(tmem_base + lane_addr + O_COL + c * 32, v);
        if (grow && c + 1 < c_hi) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) gn[q4] = __ldg(reinterpret_cast<const uint4*>(grow + (c + 1) * 32 + q4 * 8));
        }
        tmem_ld_wait();
        if (live) {
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4) {
            float o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = Ty<bf16>::rnd(__uint_as_float(v[q4 * 8 + i]) * inv);
            if (grow) {
              const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv[q4]);
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                o[2 * i] *= Ty<bf16>::rnd(sigmoid_gate(__low2float(g2[i])));
                o[2 * i + 1] *= Ty<bf16>::rnd(sigmoid_gate(__high2float(g2[i])));
              }
            }
            uint4 ov;
            ov.x = pack_bf16(o[0], o[1]);
            ov.y = pack_bf16(o[2], o[3]);
            ov.z = pack_bf16(o[4], o[5]);
            ov.w = pack_bf16(o[6], o[7]);
            *reinterpret_cast<uint4*>(orow + c * 32 + q4 * 8) = ov;
          }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) gv[q4] = gn[q4];
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) set_err(p.err, DERR_ATTN_TIMEOUT);
#pragma unroll 1
    for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == ISSUER_WARP) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
  }
}

// Adds up the parts of a split launch: out = sum_z O_z 2^(m_z - M) / sum_z l_z 2^(m_z - M), M = max_z m_z, then the output gate.
// One warp per row of a (token tile, KV head), eight head dims per lane; grid (token tiles, KV heads, 128 / 4 rows). The maxima and
// denominators of all parts are fetched first, one part per lane, so that the loop over the parts has no dependent loads.
template <int G>
__global__ void __launch_bounds__(128) attn_merge_kernel(const Params p, int n_split, int grid_x, int grid_y) {
  constexpr int TT = 128 / G;
  const int ti = blockIdx.x, kh = blockIdx.y;
  if (ti >= p.tile_cu[p.B]) return;
  int b = 0;
  {
    int lo = 0, hi = p.B;
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (p.tile_cu[mid] <= ti) lo = mid; else hi = mid;
    }
    b = lo;
  }
  const int off = p.cu[b], L = p.cu[b + 1] - off;
  const int t0 = (ti - p.tile_cu[b]) * TT;
  const int ntok = min(TT, L - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = blockIdx.z * 4 + warp;
  if (r >= ntok * G) return;
  const int tt = r / G, g = r - tt * G;
  const size_t part_stride = (size_t)grid_y * grid_x * 128, row0 = ((size_t)kh * grid_x + ti) * 128 + r;
  constexpr int MAXP = 4;  // parts per lane: up to 128 parts
  float2 ml[MAXP];
  float M = -INFINITY;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    const int z = lane + 32 * i;
    ml[i] = z < n_split ? p.ws_ml[(size_t)z * part_stride + row0] : make_float2(-INFINITY, 0.f);
    if (ml[i].y > 0.f) M = fmaxf(M, ml[i].x);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
  float den = 0.f;
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    ml[i].x = ml[i].y > 0.f ? exp2f(ml[i].x - M) : 0.f;  // the weight of the part
    den = fmaf(ml[i].x, ml[i].y, den);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < MAXP; ++i) {
    if (32 * i >= n_split) break;
#pragma unroll 8
    for (int zz = 0; zz < 32; ++zz) {
      const int z = 32 * i + zz;
      if (z >= n_split) break;
      const float w = __shfl_sync(0xffffffffu, ml[i].x, zz);
      if (w == 0.f) continue;  // an empty part wrote no output
      const float* src = p.ws_o + ((size_t)z * part_stride + row0) * HD + lane * 8;
      const float4 a = *reinterpret_cast<const float4*>(src);
      const float4 c = *reinterpret_cast<const float4*>(src + 4);
      acc[0] = fmaf(w, a.x, acc[0]); acc[1] = fmaf(w, a.y, acc[1]); acc[2] = fmaf(w, a.z, acc[2]); acc[3] = fmaf(w, a.w, acc[3]);
      acc[4] = fmaf(w, c.x, acc[4]); acc[5] = fmaf(w, c.y, acc[5]); acc[6] = fmaf(w, c.z, acc[6]); acc[7] = fmaf(w, c.w, acc[7]);
    }
  }
  const int t = off + t0 + tt, head = kh * G + g;
  const float inv = 1.0f / den;
  float o[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] = Ty<bf16>::rnd(acc[i] * inv);
  if (p.gate_qg) {
    const uint4 gv = *reinterpret_cast<const uint4*>(p.gate_qg + (size_t)t * p.qg_stride + (size_t)head * 2 * HD + HD + lane * 8);
    const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      o[2 * i] *= Ty<bf16>::rnd(sigmoid_gate(__low2float(g2[i])));
      o[2 * i + 1] *= Ty<bf16>::rnd(sigmoid_gate(__high2float(g2[i])));
    }
  }
  *reinterpret_cast<uint4*>(p.out + ((size_t)t * p.heads + head) * HD + lane * 8) =
      make_uint4(pack_bf16(o[0], o[1]), pack_bf16(o[2], o[3]), pack_bf16(o[4], o[5]), pack_bf16(o[6], o[7]));
}

// tile_cu[b] = number of token tiles of the sequences before b (single CTA scan).
__global__ void attn_tiles_kernel(const int32_t* __restrict__ cu, int B, int tokens_per_tile, int32_t* __restrict__ tile_cu) {
  __shared__ int part[1024];
  const int tid = threadIdx.x, nt = blockDim.x;
  const int per = (B + nt - 1) / nt;
  const int lo = min(tid * per, B), hi = min(lo + per, B);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += (cu[i + 1] - cu[i] + tokens_per_tile - 1) / tokens_per_tile;
  part[tid] = s;
  __syncthreads();
  for (int o = 1; o < nt; o <<= 1) {
    const int v = tid >= o ? part[tid - o] : 0;
    __syncthreads();
    part[tid] += v;
    __syncthreads();
  }
  int run = part[tid] - s;
  for (int i = lo; i < hi; ++i) {
    tile_cu[i] = run;
    run += (cu[i + 1] - cu[i] + tokens_per_tile - 1) / tokens_per_tile;
  }
  if (tid == nt - 1) tile_cu[B] = part[tid];
}

}  // namespace atc

bool attn_tc_supported(int heads, int kv, int hd) { return hd == 256 && kv > 0 && heads % kv == 0 && heads / kv == 6; }
int attn_tc_tokens_per_tile(int heads, int kv) { return 128 / (heads / kv); }

cudaError_t attn_tc_prepare_device() {
  return cudaFuncSetAttribute(atc::attn_tc_kernel<6>, cudaFuncAttributeMaxDynamicSharedMemorySize, atc::SMEM_BYTES);
}

cudaError_t attn_tc_build_tiles(const int32_t* cu, int B, int tokens_per_tile, int32_t* tile_cu, cudaStream_t s) {
  atc::attn_tiles_kernel<<<1, 1024, 0, s>>>(cu, B, tokens_per_tile, tile_cu);
  return cudaGetLastError();
}

int attn_tc_make_maps(AttnTcMaps* m, const void* q, const void* k_own, int k_stride, const void* v_own, int v_stride, const void* k_state,
                      const void* v_state, int n_state, int T, int heads, int kv, int hd) {
  const int G = heads / kv, TT = 128 / G;
  int bad = tc_make_tmap_3d(&m->q, q, hd, heads, T, hd, (uint64_t)heads * hd, G, TT);
  bad |= tc_make_tmap_strided(&m->k_own, k_own, T, (uint64_t)kv * hd, k_stride, atc::KT);
  bad |= tc_make_tmap_strided(&m->v_own, v_own, T, (uint64_t)kv * hd, v_stride, atc::KT);
  if (n_state > 0) {
    bad |= tc_make_tmap_strided(&m->k_state, k_state, n_state, (uint64_t)kv * hd, (uint64_t)kv * hd, atc::KT);
    bad |= tc_make_tmap_strided(&m->v_state, v_state, n_state, (uint64_t)kv * hd, (uint64_t)kv * hd, atc::KT);
  } else {
    m->k_state = m->k_own;
    m->v_state = m->v_own;
  }
  return bad;
}

size_t attn_tc_split_workspace_bytes(int sm_count) { return (size_t)2 * sm_count * 128 * (atc::HD * sizeof(float) + sizeof(float2)); }

int attn_tc_pick_split(int max_tiles, int kv, int n_state, int sm_count) {
  const int ctas = max_tiles * kv, st_tiles = (n_state + atc::KT - 1) / atc::KT;
  if (ctas <= 0 || ctas > sm_count || st_tiles < 8) return 1;  // a CTA per SM already, or too few key tiles to be worth a second pass
  int z = (2 * sm_count) / ctas;
  if (z > st_tiles / 2) z = st_tiles / 2;  // at least two key tiles per part
  if (z > 128) z = 128;
  return z < 2 ? 1 : z;
}

cudaError_t attn_tc_launch(const AttnTcMaps* m, const int32_t* cu, const int32_t* tile_cu, int B, int n_state, int T, int max_tiles,
                           int heads, int kv, int hd, const void* gate_qg, int qg_stride, void* out, int* err, cudaStream_t s, int n_split,
                           void* workspace) {
  if (!attn_tc_supported(heads, kv, hd)) return cudaErrorInvalidValue;
  if (n_split < 1 || n_split > 128 || (n_split > 1 && !workspace)) return cudaErrorInvalidValue;
  atc::Params p;
  p.cu = cu;
  p.tile_cu = tile_cu;
  p.B = B;
  p.n_state = n_state;
  p.heads = heads;
  p.kv = kv;
  p.total_tokens = T;
  p.gate_qg = (const bf16*)gate_qg;
  p.qg_stride = qg_stride;
  p.out = (bf16*)out;
  p.scale_log2e = (1.0f / sqrtf((float)hd)) * 1.4426950408889634f;
  p.err = err;
  // workspace: the maxima and denominators of all parts, then the partial outputs
  p.ws_ml = (float2*)workspace;
  p.ws_o = (float*)((char*)workspace + (size_t)n_split * max_tiles * kv * 128 * sizeof(float2));
  dim3 grid(max_tiles, kv, n_split);
  atc::attn_tc_kernel<6><<<grid, atc::NUM_THREADS, atc::SMEM_BYTES, s>>>(
      *reinterpret_cast<const CUtensorMap*>(&m->q), *reinterpret_cast<const CUtensorMap*>(&m->k_state),
      *reinterpret_cast<const CUtensorMap*>(&m->v_state), *reinterpret_cast<const CUtensorMap*>(&m->k_own),
      *reinterpret_cast<const CUtensorMap*>(&m->v_own), p);
  cudaError_t ce = cudaGetLastError();
  if (ce != cudaSuccess || n_split == 1) return ce;
  atc::attn_merge_kernel<6><<<dim3(max_tiles, kv, 32), 128, 0, s>>>(p, n_split, max_tiles, kv);
  return cudaGetLastError();
}
