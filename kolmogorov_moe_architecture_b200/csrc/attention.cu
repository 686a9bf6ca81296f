// Causal grouped-query flash attention for sm_100a: tcgen05 MMAs with TMEM accumulators,
// TMA-fed 128B-swizzled shared memory, online softmax in registers.
//
// Layouts: q, o, do, dq [B, S, H, D]; k, v, dk, dv [B, S, Hkv, D] (bf16, contiguous);
// lse [B, H, S] fp32 (natural log).  Query head h reads KV head h / (H / Hkv) directly -
// K and V are never expanded to H heads.
//
// head_dim 128 (the model's): 320-thread CTAs - eight softmax warps in two warpgroups, a TMA producer warp, an
// MMA warp - and 128-key / 128-query steps.
//   forward   attn_fwd2_kernel: two 128-query tiles per CTA, one per warpgroup; S = Q K^T in TMEM, the score row
//             is read into registers once, P is written as packed bf16 over the S columns and feeds O += P V as
//             the A operand from tensor memory; O is rescaled only when the row maximum grew by more than 2^8.
//   backward  attn_bwd_dq2_kernel (loop over key blocks of a query block) and attn_bwd_dkv2_kernel (loop over
//             the query heads of the group and their query blocks for a key block); both recompute P from the
//             saved lse (no atomics, deterministic); the warpgroups split the 128 columns of an accumulator in
//             halves; P^T / dS^T / dS are packed over consumed accumulator columns and enter the next MMA from
//             tensor memory.
// head_dim 64 keeps the earlier kernels (attn_fwd_kernel, attn_bwd_dq_kernel, attn_bwd_dkv_kernel): 192-thread
// CTAs, one softmax warpgroup (thread = row), 64-wide steps, P / dS staged through swizzled shared memory.
// In the head_dim-128 kernels the tile index is the slowest grid dimension, so the heavy tiles of all heads run
// first.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <cstdlib>

#include <mutex>

#include "kmoe_api.h"
#include "ptx.cuh"
#include "tmap_host.h"

namespace kmoe {

constexpr int ATT_BLK = 128;             // query rows per CTA and keys per step
constexpr int PANEL_BYTES = ATT_BLK * 128;  // one 64-column bf16 panel of a 128-row tile
constexpr int ATT_THREADS = 192;

struct AttnArgs {
  int B, S, H, Hkv;
  float scale_log2;  // softmax scale * log2(e)
  __nv_bfloat16* out;
  float* lse;
  int* status;
  // optional (B, S): first position of the packed document that contains each position; a query then sees
  // only keys k with doc_start[q] <= k <= q (block-diagonal causal mask of packed sequences)
  const int* doc_start;
};

// Byte offset of the 16-byte chunk holding (row, col..col+7) in a K-major 128B-swizzled tile
// made of 64-column panels.
__device__ __forceinline__ uint32_t swz_kmajor(int row, int col) {
  const int panel = col >> 6;
  const int chunk = (col & 63) >> 3;
  return panel * PANEL_BYTES + row * 128 + ((chunk ^ (row & 7)) << 4);
}

// 16-byte chunk offset inside a [rows x 64] K-major swizzled panel
__device__ __forceinline__ uint32_t swz64(int row, int col) { return row * 128 + ((((col & 63) >> 3) ^ (row & 7)) << 4); }

constexpr int FWD_BN = 64;                         // keys per forward step
constexpr int FWD_KPANEL = FWD_BN * 128;           // 64 key rows x 64 bf16 columns
constexpr float RESCALE_THRESHOLD = 8.0f;          // log2 units: rescale O only when the row max grew by > 2^8

// Forward.  O stays in TMEM across the whole KV loop (the PV MMA accumulates into it); the running
// maximum used for the exponent is only advanced - and O rescaled in place - when the true row
// maximum has grown by more than RESCALE_THRESHOLD, so most steps never touch O.  64-key steps keep
// the footprint at 112 KB of shared memory and 256 TMEM columns: two CTAs share an SM and the
// softmax of one overlaps the MMAs of the other.
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  constexpr int NP = D / 64;
  constexpr int QTILE = NP * PANEL_BYTES;       // 128 query rows
  constexpr int KTILE = NP * FWD_KPANEL;        // 64 key rows
  constexpr uint32_t IDESC_S = make_idesc_f16(128, FWD_BN, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_PV = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  constexpr uint32_t TMEM_COLS = 256;
  constexpr uint32_t COL_S0 = 0, COL_O = 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + QTILE;             // 2 stages
  uint8_t* sV = sK + 2 * KTILE;         // 2 stages
  uint8_t* sP = sV + 2 * KTILE;         // 128 x 64 bf16, one K-major panel
  __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], s_free[2], p_full, pv_full;
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;  // heavy (late) query blocks first
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (a.H / a.Hkv);
  const int q0 = qb * ATT_BLK;
  const int kmax = min(q0 + ATT_BLK, a.S);
  // packed documents: key blocks that end before the document of the block's first query are invisible to
  // every row of the block (document starts do not decrease along the sequence) and are not visited at all
  const int jlo = a.doc_start != nullptr ? a.doc_start[(size_t)b * a.S + q0] / FWD_BN : 0;
  const int nblk = (kmax + FWD_BN - 1) / FWD_BN - jlo;       // j below counts visited blocks; key block = jlo + j

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 128);
    }
    mbar_init(&p_full, 128);
    mbar_init(&pv_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 5) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    if (elect_one()) {
      mbar_expect_tx(&q_full, QTILE);
#pragma unroll
      for (int p = 0; p < NP; ++p) tma_load_4d(sQ + p * PANEL_BYTES, &tmQ, &q_full, p * 64, h, q0, b);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { atomicExch(a.status, 11); goto teardown; }
        mbar_expect_tx(&k_full[st], KTILE);
#pragma unroll
        for (int p = 0; p < NP; ++p)
          tma_load_4d(sK + st * KTILE + p * FWD_KPANEL, &tmK, &k_full[st], p * 64, hkv, (jlo + j) * FWD_BN, b);
        if (!mbar_wait(&v_empty[st], par)) { atomicExch(a.status, 12); goto teardown; }
        mbar_expect_tx(&v_full[st], KTILE);
#pragma unroll
        for (int p = 0; p < NP; ++p)
          tma_load_4d(sV + st * KTILE + p * FWD_KPANEL, &tmV, &v_full[st], p * 64, hkv, (jlo + j) * FWD_BN, b);
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      auto issue_S = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1)) return false;
        if (!mbar_wait(&s_free[st], ((j >> 1) & 1) ^ 1)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ), ka = smem_u32(sK + st * KTILE);
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t aoff = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          const uint32_t boff = (k4 >> 2) * FWD_KPANEL + (k4 & 3) * 32;
          umma_f16(tmem + COL_S0 + st * FWD_BN, make_smem_desc_sw128(qa + aoff, 16, 1024),
                   make_smem_desc_sw128(ka + boff, 16, 1024), IDESC_S, k4 > 0);
        }
        umma_commit(&s_full[st]);
        umma_commit(&k_empty[st]);
        return true;
      };
      if (!mbar_wait(&q_full, 0)) { atomicExch(a.status, 13); goto teardown; }
      if (!issue_S(0)) { atomicExch(a.status, 14); goto teardown; }
      for (int j = 0; j < nblk; ++j) {
        if (j + 1 < nblk && !issue_S(j + 1)) { atomicExch(a.status, 15); goto teardown; }
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1)) { atomicExch(a.status, 16); goto teardown; }
        if (!mbar_wait(&p_full, j & 1)) { atomicExch(a.status, 17); goto teardown; }
        tc_fence_after();
        const uint32_t pa = smem_u32(sP), va = smem_u32(sV + st * KTILE);
#pragma unroll
        for (int k4 = 0; k4 < FWD_BN / 16; ++k4)
          umma_f16(tmem + COL_O, make_smem_desc_sw128(pa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(va + k4 * 16 * 128, FWD_KPANEL, 1024), IDESC_PV, (j > 0 || k4 > 0));
        umma_commit(&pv_full);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ----------------------------------------------------------- softmax warps
    const int r = warp * 32 + lane;                 // query row within the block
    const int qi = q0 + r;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    const int qstart = (a.doc_start != nullptr && qi < a.S) ? a.doc_start[(size_t)b * a.S + qi] : 0;
    for (int j = 0; j < nblk; ++j) {
      const int st = j & 1;
      if (!mbar_wait(&s_full[st], (j >> 1) & 1)) { if (lane == 0) atomicExch(a.status, 18); goto teardown; }
      tc_fence_after();
      const uint32_t ts = tmem + lane_base + COL_S0 + st * FWD_BN;
      const int k0 = (jlo + j) * FWD_BN;
      const bool need_mask = (k0 + FWD_BN > q0) || (k0 + FWD_BN > a.S) || (k0 < qstart);
      uint32_t sv[FWD_BN];
      {
        uint32_t (&lo)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[0]);
        uint32_t (&hi)[32] = *reinterpret_cast<uint32_t (*)[32]>(&sv[32]);
        tmem_ld_32x32(ts, lo);
        tmem_ld_32x32(ts + 32, hi);
        tmem_ld_wait();
      }
      tc_fence_before();
      mbar_arrive(&s_free[st]);          // S_j is in registers: its TMEM buffer may be overwritten
      float mx = -INFINITY;
#pragma unroll
      for (int i = 0; i < FWD_BN; ++i) {
        float s = __uint_as_float(sv[i]) * a.scale_log2;
        if (need_mask && (k0 + i > qi || k0 + i >= a.S || k0 + i < qstart)) s = -INFINITY;
        sv[i] = __float_as_uint(s);
        mx = fmaxf(mx, s);
      }
      const bool grow = mx > m_used + RESCALE_THRESHOLD;      // always true on the first step
      const float m_new = grow ? mx : m_used;
      const float alpha = grow ? exp2f(m_used - m_new) : 1.f;
      // a row that has not met a visible key yet (its document starts in a later block) has m_new = -inf
      const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;
      float rs = 0.f;
      uint32_t pk[FWD_BN / 2];
#pragma unroll
      for (int i = 0; i < FWD_BN; i += 2) {
        const float p0 = exp2f(__uint_as_float(sv[i]) - m_exp), p1 = exp2f(__uint_as_float(sv[i + 1]) - m_exp);
        rs += p0 + p1;
        pk[i >> 1] = pack_bf16(p0, p1);
      }
      l = l * alpha + rs;
      m_used = m_new;
      if (j > 0) {
        // PV_{j-1} must have retired before P is overwritten or O is rescaled
        if (!mbar_wait(&pv_full, (j - 1) & 1)) { if (lane == 0) atomicExch(a.status, 19); goto teardown; }
        tc_fence_after();
        if (__any_sync(0xffffffffu, grow)) {
#pragma unroll
          for (int c = 0; c < D; c += 32) {
            uint32_t v[32];
            tmem_ld_32x32(tmem + lane_base + COL_O + c, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(tmem + lane_base + COL_O + c, v);
          }
          tmem_st_wait();
        }
      }
#pragma unroll
      for (int c = 0; c < FWD_BN; c += 8)
        *reinterpret_cast<uint4*>(sP + swz64(r, c)) = make_uint4(pk[c / 2], pk[c / 2 + 1], pk[c / 2 + 2], pk[c / 2 + 3]);
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&p_full);
    }
    if (!mbar_wait(&pv_full, (nblk - 1) & 1)) { if (lane == 0) atomicExch(a.status, 20); goto teardown; }
    tc_fence_after();
    const bool row_ok = qi < a.S;
    const float inv = 1.f / l;
    __nv_bfloat16* orow = a.out + (((size_t)b * a.S + (row_ok ? qi : 0)) * a.H + h) * D;
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + COL_O + c, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(orow + c + i) =
              make_uint4(pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv),
                         pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv),
                         pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv),
                         pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv));
      }
    }
    if (row_ok) a.lse[((size_t)b * a.H + h) * a.S + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
    tc_fence_before();
  }

teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 5) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}


// ------------------------------------------------------------ forward, two query tiles per CTA
// One CTA per SM owns 256 query rows as two 128-row tiles, each with its own softmax warpgroup, S and O
// accumulators (4 x 128 TMEM columns in all) and barriers; both tiles share the K/V tiles of a 128-key step.
//   warps 0-3 / 4-7  softmax of tile 0 / 1 (thread = query row)
//   warp 8           TMA producer: Q tiles once, K_j / V_j into 2-stage rings
//   warp 9           MMA issuer: S_t = Q_t K_j^T (128 x 128 x 128), O_t += P_t V_j with P_t read from TMEM
// P is written as packed bf16 over the first 64 columns of the tile's own S accumulator (the softmax has the whole
// 128-value score row in registers by then), so no shared memory is spent on P and the PV MMA takes its A operand
// from tensor memory.  The tensor pipe executes one tile's MMAs while the
// other tile's warpgroup is in its softmax; 128-key steps halve the number of barrier round trips per key.
constexpr int F2_KEYS = 128;
constexpr int F2_THREADS = 320;
constexpr int F2_TILE_BYTES = 2 * PANEL_BYTES;     // 128 rows x 128 bf16 columns, two 64-column panels

// 2^x on the FMA pipe (x <= ~10): round-to-nearest split x = n + f, f in [-0.5, 0.5], cubic for 2^f, exponent
// added in integer.  Relative error ~1e-4, far below the bf16 rounding of P.  Used for a share of the
// exponentials so that the MUFU pipe (16 per clock and SM) is not the only limit of the softmax.
__device__ __forceinline__ float ex2_fma(float x) {
  x = fmaxf(x, -125.f);
  const float t = x + 12582912.f;                   // 1.5 * 2^23: the integer part lands in the low mantissa bits
  const float f = x - (t - 12582912.f);
  float p = 0.0555041f;
  p = fmaf(p, f, 0.2402265f);
  p = fmaf(p, f, 0.6931472f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (__float_as_int(t) << 23));
}

template <int D>
__global__ void __launch_bounds__(F2_THREADS, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  static_assert(D == 128, "two-tile forward is written for head_dim 128");
  constexpr uint32_t IDESC_S = make_idesc_f16(128, F2_KEYS, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_PV = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  constexpr uint32_t TMEM_COLS = 512;
  constexpr uint32_t COL_S = 0, COL_O = 256;          // S_t at COL_S + 128 t, O_t at COL_O + 128 t

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                           // 2 tiles
  uint8_t* sK = sQ + 2 * F2_TILE_BYTES;         // 2 stages
  uint8_t* sV = sK + 2 * F2_TILE_BYTES;         // 2 stages
  __shared__ uint64_t q_full, k_full[2], v_full[2], k_empty[2], v_empty[2], s_full[2], p_full[2], pv_done[2];
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the block index is the slowest grid dimension: all heavy (late) query blocks are scheduled before any lighter one
  const int qb = gridDim.z - 1 - blockIdx.z;
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / (a.H / a.Hkv);
  const int q0 = qb * 256;
  // packed documents: key blocks that end before the document of the CTA's first query are invisible to all rows
  const int jlo = a.doc_start != nullptr ? a.doc_start[(size_t)b * a.S + q0] / F2_KEYS : 0;
  // visited key blocks per tile (causal): tile t sees keys < min(q0 + 128 (t + 1), S)
  int nb[2];
#pragma unroll
  for (int t = 0; t < 2; ++t) {
    const int kmax = min(q0 + 128 * (t + 1), a.S);
    nb[t] = (q0 + 128 * t < a.S) ? max((kmax + F2_KEYS - 1) / F2_KEYS - jlo, 0) : 0;
  }
  const int nblk = max(nb[0], nb[1]);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1); mbar_init(&p_full[i], 128); mbar_init(&pv_done[i], 1);
    }
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 9) {
    tmem_alloc(&tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------ TMA producer
    if (elect_one() && nblk > 0) {
      mbar_expect_tx(&q_full, 2 * F2_TILE_BYTES);
#pragma unroll
      for (int t = 0; t < 2; ++t)
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sQ + t * F2_TILE_BYTES + p * PANEL_BYTES, &tmQ, &q_full, p * 64, h, q0 + t * 128, b);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { atomicExch(a.status, 31); goto teardown; }
        mbar_expect_tx(&k_full[st], F2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sK + st * F2_TILE_BYTES + p * PANEL_BYTES, &tmK, &k_full[st], p * 64, hkv, (jlo + j) * F2_KEYS, b);
        if (!mbar_wait(&v_empty[st], par)) { atomicExch(a.status, 32); goto teardown; }
        mbar_expect_tx(&v_full[st], F2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sV + st * F2_TILE_BYTES + p * PANEL_BYTES, &tmV, &v_full[st], p * 64, hkv, (jlo + j) * F2_KEYS, b);
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && nblk > 0) {
      auto issue_S = [&](int t, int j) {
        const uint32_t qa = smem_u32(sQ + t * F2_TILE_BYTES), ka = smem_u32(sK + (j & 1) * F2_TILE_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t off = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tmem + COL_S + t * 128, make_smem_desc_sw128(qa + off, 16, 1024),
                   make_smem_desc_sw128(ka + off, 16, 1024), IDESC_S, k4 > 0);
        }
        umma_commit(&s_full[t]);
      };
      if (!mbar_wait(&q_full, 0)) { atomicExch(a.status, 33); goto teardown; }
      if (!mbar_wait(&k_full[0], 0)) { atomicExch(a.status, 34); goto teardown; }
      tc_fence_after();
#pragma unroll
      for (int t = 0; t < 2; ++t)
        if (nb[t] > 0) issue_S(t, 0);
      umma_commit(&k_empty[0]);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1)) { atomicExch(a.status, 35); goto teardown; }
        if (j + 1 < nblk && !mbar_wait(&k_full[(j + 1) & 1], ((j + 1) >> 1) & 1)) {
          atomicExch(a.status, 36);
          goto teardown;
        }
#pragma unroll
        for (int t = 0; t < 2; ++t) {
          if (j >= nb[t]) continue;
          if (!mbar_wait(&p_full[t], j & 1)) { atomicExch(a.status, 37); goto teardown; }
          tc_fence_after();
          const uint32_t va = smem_u32(sV + st * F2_TILE_BYTES);
#pragma unroll
          for (int k4 = 0; k4 < F2_KEYS / 16; ++k4)   // A = P_t from tensor memory: 16 keys = 8 packed columns
            umma_f16_ts(tmem + COL_O + t * 128, tmem + COL_S + t * 128 + k4 * 8,
                        make_smem_desc_sw128(va + k4 * 16 * 128, PANEL_BYTES, 1024), IDESC_PV, (j > 0 || k4 > 0));
          umma_commit(&pv_done[t]);
          if (j + 1 < nb[t]) issue_S(t, j + 1);       // overwrites S_t / P_t: ordered behind the PV just issued
        }
        if (j + 1 < nblk) umma_commit(&k_empty[(j + 1) & 1]);
        umma_commit(&v_empty[st]);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups
    const int t = warp >> 2;
    const int r = (warp & 3) * 32 + lane;
    const int qt0 = q0 + t * 128;                 // first query row of this tile
    const int qi = qt0 + r;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t ts = tmem + lane_base + COL_S + t * 128;
    const uint32_t to = tmem + lane_base + COL_O + t * 128;
    float m_used = -INFINITY, l = 0.f;
    const int qstart = (a.doc_start != nullptr && qi < a.S) ? a.doc_start[(size_t)b * a.S + qi] : 0;
    const float sc = a.scale_log2;
    for (int j = 0; j < nb[t]; ++j) {
      if (!mbar_wait(&s_full[t], j & 1)) { if (lane == 0) atomicExch(a.status, 38); goto teardown; }
      tc_fence_after();
      const int k0 = (jlo + j) * F2_KEYS;
      const bool need_mask = (k0 + F2_KEYS > qt0) || (k0 + F2_KEYS > a.S) || (k0 < qstart);
      // The whole row of scores (128 values) is read into registers once; the mask is applied in a separate,
      // rarely taken branch.
      uint32_t v[F2_KEYS];
#pragma unroll
      for (int c = 0; c < F2_KEYS; c += 32) tmem_ld_32x32(ts + c, *reinterpret_cast<uint32_t(*)[32]>(&v[c]));
      tmem_ld_wait();
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < F2_KEYS; ++i) {
          const int kk = k0 + i;
          if (kk > qi || kk >= a.S || kk < qstart) v[i] = 0xff800000u;      // -inf
        }
      }
      float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
      for (int i = 0; i < F2_KEYS; i += 4) {
        m0 = fmaxf(m0, __uint_as_float(v[i]));
        m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
        m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
        m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
      }
      const float mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3)) * sc;      // scale > 0: max of the scaled scores
      const bool grow = mx > m_used + RESCALE_THRESHOLD;      // always true on the first step
      const float m_new = grow ? mx : m_used;
      const float alpha = grow ? exp2f(m_used - m_new) : 1.f;
      const float m_exp = (m_new == -INFINITY) ? 0.f : m_new;   // rows that have not met a visible key yet
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // s_full for step j was committed after PV of step j-1 in the same in-order pipe: O is at rest
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_32x32(to + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(to + c, o);
        }
        tmem_st_wait();
      }
      // p = 2^(s * scale - m), packed bf16 written over the first 64 columns of S (all of S is in registers)
      const uint64_t sc2 = pack_f32x2(sc, sc), nm2 = pack_f32x2(-m_exp, -m_exp);
      uint64_t rsum = pack_f32x2(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < F2_KEYS; c += 32) {
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(v[c + i]), __uint_as_float(v[c + i + 1])), sc2, nm2), x0, x1);
          // every fourth pair on the FMA pipe, the rest on MUFU
          const float p0 = ((i & 6) == 6) ? ex2_fma(x0) : ex2_approx(x0);
          const float p1 = ((i & 6) == 6) ? ex2_fma(x1) : ex2_approx(x1);
          rsum = add_f32x2(rsum, pack_f32x2(p0, p1));
          pk[i >> 1] = pack_bf16(p0, p1);
        }
        tmem_st_32x16(ts + (c >> 1), pk);
      }
      float rs0, rs1;
      unpack_f32x2(rsum, rs0, rs1);
      const float rs = rs0 + rs1;
      tmem_st_wait();
      l = l * alpha + rs;
      m_used = m_new;
      tc_fence_before();
      mbar_arrive(&p_full[t]);
    }
    if (nb[t] > 0) {
      if (!mbar_wait(&pv_done[t], (nb[t] - 1) & 1)) { if (lane == 0) atomicExch(a.status, 39); goto teardown; }
      tc_fence_after();
      const bool row_ok = qi < a.S;
      const float inv = 1.f / l;
      __nv_bfloat16* orow = a.out + (((size_t)b * a.S + (row_ok ? qi : 0)) * a.H + h) * D;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(to + c, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(orow + c + i) =
                make_uint4(pack_bf16(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv),
                           pack_bf16(__uint_as_float(v[i + 2]) * inv, __uint_as_float(v[i + 3]) * inv),
                           pack_bf16(__uint_as_float(v[i + 4]) * inv, __uint_as_float(v[i + 5]) * inv),
                           pack_bf16(__uint_as_float(v[i + 6]) * inv, __uint_as_float(v[i + 7]) * inv));
        }
      }
      if (row_ok) a.lse[((size_t)b * a.H + h) * a.S + qi] = (m_used + log2f(l)) * 0.6931471805599453f;
      tc_fence_before();
    }
  }

teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem, TMEM_COLS);
  }
}

}  // namespace kmoe

// ------------------------------------------------------------------- backward
namespace kmoe {

constexpr int BWD_SUB = 64;                       // keys (dQ kernel) / queries (dK/dV kernel) per step
constexpr int SUBPANEL_BYTES = BWD_SUB * 128;     // 64 rows x 64 bf16 columns

struct AttnBwdArgs {
  int B, S, H, Hkv;
  float scale, scale_log2;
  const float* lse;     // [B,H,S]
  const float* delta;   // [B,H,S]  rowsum(dO * O)
  __nv_bfloat16* dq;    // [B,S,H,D]
  __nv_bfloat16* dk;    // [B,S,Hkv,D]
  __nv_bfloat16* dv;
  int* status;
  const int* doc_start;  // optional (B, S), see AttnArgs
};

// delta[b,h,s] = sum_d dO * O.  One warp per (b,s,h) row.
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                  float* __restrict__ delta, int B, int S, int H, int D) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long long rows = (long long)B * S * H;
  for (long long row = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const int h = (int)(row % H);
    const long long bs = row / H;
    const int s_ = (int)(bs % S);
    const int b = (int)(bs / S);
    float acc = 0.f;
    for (int c = lane * 8; c < D; c += 256) {
      uint4 r1 = *reinterpret_cast<const uint4*>(o + row * D + c);
      uint4 r2 = *reinterpret_cast<const uint4*>(d_o + row * D + c);
      const __nv_bfloat162* p1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&r2);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float2 f1 = __bfloat1622float2(p1[i]), f2 = __bfloat1622float2(p2[i]);
        acc += f1.x * f2.x + f1.y * f2.y;
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) delta[((size_t)b * H + h) * S + s_] = acc;
  }
}


// dQ for one (128-query block, head, batch): dQ = sum_j dS_j K_j, dS = P * (dO V^T - delta) * scale
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                   const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const AttnBwdArgs a) {
  constexpr int NP = D / 64;
  constexpr int QTILE = NP * PANEL_BYTES;       // 128 rows
  constexpr int KTILE = NP * SUBPANEL_BYTES;    // 64 rows
  constexpr uint32_t IDESC_S = make_idesc_f16(128, BWD_SUB, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_DQ = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  // S and dP are double buffered in TMEM (buffer = block parity): the MMAs of block j+1 run while the
  // threads turn block j into dS, and the dQ MMA of block j runs under the softmax of block j+1.
  constexpr uint32_t TMEM_COLS = 512, COL_S = 0, COL_DP = 64, COL_BUF = 128, COL_DQ = 256;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + QTILE;
  uint8_t* sK = sdO + QTILE;          // 2 stages
  uint8_t* sV = sK + 2 * KTILE;       // 2 stages
  uint8_t* sdS = sV + 2 * KTILE;      // 128 x 64 bf16
  __shared__ uint64_t qdo_full, k_full[2], v_full[2], k_empty[2], v_empty[2], sdp_full[2], ds_full, ds_free, dq_full;
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.x - 1 - blockIdx.x;
  const int h = blockIdx.y, b = blockIdx.z;
  const int hkv = h / (a.H / a.Hkv);
  const int q0 = qb * ATT_BLK;
  const int kmax = min(q0 + ATT_BLK, a.S);
  const int jlo = a.doc_start != nullptr ? a.doc_start[(size_t)b * a.S + q0] / BWD_SUB : 0;   // see the forward kernel
  const int nblk = (kmax + BWD_SUB - 1) / BWD_SUB - jlo;

  if (threadIdx.x == 0) {
    mbar_init(&qdo_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&k_empty[i], 1); mbar_init(&v_empty[i], 1);
    }
    mbar_init(&sdp_full[0], 1); mbar_init(&sdp_full[1], 1);
    mbar_init(&ds_full, 128); mbar_init(&ds_free, 1); mbar_init(&dq_full, 1);
    mbar_fence_init();
  }
  if (warp == 5) { tmem_alloc(&tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    if (elect_one()) {
      mbar_expect_tx(&qdo_full, 2 * QTILE);
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        tma_load_4d(sQ + p * PANEL_BYTES, &tmQ, &qdo_full, p * 64, h, q0, b);
        tma_load_4d(sdO + p * PANEL_BYTES, &tmdO, &qdo_full, p * 64, h, q0, b);
      }
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(&k_empty[st], par)) { atomicExch(a.status, 21); goto teardown; }
        mbar_expect_tx(&k_full[st], KTILE);
#pragma unroll
        for (int p = 0; p < NP; ++p)
          tma_load_4d(sK + st * KTILE + p * SUBPANEL_BYTES, &tmK, &k_full[st], p * 64, hkv, (jlo + j) * BWD_SUB, b);
        if (!mbar_wait(&v_empty[st], par)) { atomicExch(a.status, 22); goto teardown; }
        mbar_expect_tx(&v_full[st], KTILE);
#pragma unroll
        for (int p = 0; p < NP; ++p)
          tma_load_4d(sV + st * KTILE + p * SUBPANEL_BYTES, &tmV, &v_full[st], p * 64, hkv, (jlo + j) * BWD_SUB, b);
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      if (!mbar_wait(&qdo_full, 0)) { atomicExch(a.status, 23); goto teardown; }
      const uint32_t qa = smem_u32(sQ), da = smem_u32(sdO);
      // S_j = Q K_j^T and dP_j = dO V_j^T into TMEM buffer j & 1
      auto issue_sdp = [&](int j) -> bool {
        const int st = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        if (!mbar_wait(&k_full[st], ph) || !mbar_wait(&v_full[st], ph)) return false;
        tc_fence_after();
        const uint32_t ka = smem_u32(sK + st * KTILE), va = smem_u32(sV + st * KTILE);
        const uint32_t tb = tmem + st * COL_BUF;
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t aoff = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          const uint32_t boff = (k4 >> 2) * SUBPANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tb + COL_S, make_smem_desc_sw128(qa + aoff, 16, 1024), make_smem_desc_sw128(ka + boff, 16, 1024),
                   IDESC_S, k4 > 0);
        }
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t aoff = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          const uint32_t boff = (k4 >> 2) * SUBPANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tb + COL_DP, make_smem_desc_sw128(da + aoff, 16, 1024), make_smem_desc_sw128(va + boff, 16, 1024),
                   IDESC_S, k4 > 0);
        }
        umma_commit(&sdp_full[st]);
        umma_commit(&v_empty[st]);
        return true;
      };
      if (nblk > 0 && !issue_sdp(0)) { atomicExch(a.status, 24); goto teardown; }
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1;
        // buffer (j+1)&1 was last read for block j-1, whose dS arrival was awaited in the previous iteration
        if (j + 1 < nblk && !issue_sdp(j + 1)) { atomicExch(a.status, 24); goto teardown; }
        if (!mbar_wait(&ds_full, j & 1)) { atomicExch(a.status, 25); goto teardown; }
        tc_fence_after();
        const uint32_t sa = smem_u32(sdS);
        const uint32_t ka = smem_u32(sK + st * KTILE);
#pragma unroll
        for (int k4 = 0; k4 < BWD_SUB / 16; ++k4)
          umma_f16(tmem + COL_DQ, make_smem_desc_sw128(sa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(ka + k4 * 16 * 128, SUBPANEL_BYTES, 1024), IDESC_DQ, (j > 0 || k4 > 0));
        umma_commit(&ds_free);
        umma_commit(&k_empty[st]);
      }
      umma_commit(&dq_full);
    }
  } else {
    const int r = warp * 32 + lane;
    const int qi = q0 + r;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    const bool row_ok = qi < a.S;
    const size_t stat = ((size_t)b * a.H + h) * a.S + (row_ok ? qi : 0);
    const float lse2 = a.lse[stat] * 1.4426950408889634f;
    const float dlt = a.delta[stat];
    const int qstart = (a.doc_start != nullptr && row_ok) ? a.doc_start[(size_t)b * a.S + qi] : 0;
    for (int j = 0; j < nblk; ++j) {
      if (!mbar_wait(&sdp_full[j & 1], (j >> 1) & 1)) { if (lane == 0) atomicExch(a.status, 26); goto teardown; }
      const uint32_t tbuf = tmem + lane_base + (j & 1) * COL_BUF;
      tc_fence_after();
      const int k0 = (jlo + j) * BWD_SUB;
      // only blocks that touch the diagonal, the sequence end or a document start need per-element tests; the
      // tests live in their own branch, off the common path (instruction-cache footprint)
      const bool need_mask = (k0 + BWD_SUB > q0) || (k0 + BWD_SUB > a.S) || (k0 < qstart) || !row_ok;
      uint32_t ds_packed[BWD_SUB / 2];
#pragma unroll
      for (int c = 0; c < BWD_SUB; c += 32) {        // two chunks: unrolled so the packed results stay in registers
        uint32_t sv[32], dv_[32];
        tmem_ld_32x32(tbuf + COL_S + c, sv);
        tmem_ld_32x32(tbuf + COL_DP + c, dv_);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int kj = k0 + c + i;
            if ((kj > qi) || (kj >= a.S) || !row_ok || (kj < qstart)) sv[i] = 0xff800000u;   // -inf: p = 0
          }
        }
        uint32_t* dsp = &ds_packed[c >> 1];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), a.scale_log2, -lse2));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), a.scale_log2, -lse2));
          dsp[i >> 1] = pack_bf16(p0 * (__uint_as_float(dv_[i]) - dlt) * a.scale,
                                  p1 * (__uint_as_float(dv_[i + 1]) - dlt) * a.scale);
        }
      }
      tc_fence_before();
      if (!mbar_wait(&ds_free, (j & 1) ^ 1)) { if (lane == 0) atomicExch(a.status, 27); goto teardown; }
#pragma unroll
      for (int c = 0; c < BWD_SUB; c += 8)
        *reinterpret_cast<uint4*>(sdS + swz64(r, c)) =
            make_uint4(ds_packed[c / 2], ds_packed[c / 2 + 1], ds_packed[c / 2 + 2], ds_packed[c / 2 + 3]);
      fence_async_smem();
      mbar_arrive(&ds_full);
    }
    if (!mbar_wait(&dq_full, 0)) { if (lane == 0) atomicExch(a.status, 28); goto teardown; }
    tc_fence_after();
    __nv_bfloat16* drow = a.dq + (((size_t)b * a.S + (row_ok ? qi : 0)) * a.H + h) * D;
#pragma unroll
    for (int c = 0; c < D; c += 32) {
      uint32_t v[32];
      tmem_ld_32x32(tmem + lane_base + COL_DQ + c, v);
      tmem_ld_wait();
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(drow + c + i) =
              make_uint4(pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                         pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                         pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                         pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
      }
    }
    tc_fence_before();
  }
teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// dK, dV for one (128-key block, KV head, batch): loops over the query heads of the group and the
// 64-query blocks at or after the key block.
template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attn_bwd_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const AttnBwdArgs a) {
  constexpr int NP = D / 64;
  constexpr int KTILE = NP * PANEL_BYTES;       // 128 key rows
  constexpr int QTILE = NP * SUBPANEL_BYTES;    // 64 query rows
  constexpr uint32_t IDESC_ST = make_idesc_f16(128, BWD_SUB, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_ACC = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  // S^T and dP^T are double buffered in TMEM (buffer = iteration parity) so that the MMAs of iteration it+1
  // run while the threads turn iteration it into P^T / dS^T, and the dV / dK MMAs run under the next softmax.
  constexpr uint32_t TMEM_COLS = 512, COL_ST = 0, COL_DPT = 64, COL_BUF = 128, COL_DV = 256, COL_DK = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KTILE;
  uint8_t* sQ = sV + KTILE;            // 2 stages
  uint8_t* sdO = sQ + 2 * QTILE;       // 2 stages
  uint8_t* sPT = sdO + 2 * QTILE;      // 128 x 64
  uint8_t* sdST = sPT + ATT_BLK * 128; // 128 x 64
  __shared__ uint64_t kv_full, q_full[2], q_empty[2], st_full[2], pds_full, pds_free, acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ float s_lse[BWD_SUB], s_delta[BWD_SUB];
  __shared__ int s_start[BWD_SUB];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kb = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = a.H / a.Hkv;
  const int k0 = kb * ATT_BLK;
  const int qblk0 = k0 / BWD_SUB;
  const int qblk1 = (a.S + BWD_SUB - 1) / BWD_SUB;
  int per_head = qblk1 - qblk0;
  if (a.doc_start != nullptr) {
    // packed documents: once a query block starts in a document that begins after this key block's last key,
    // it and all later query blocks cannot see the block (document starts do not decrease along the sequence)
    const int klast = min(k0 + ATT_BLK, a.S) - 1;
    for (int i = 1; i < per_head; ++i) {
      if (a.doc_start[(size_t)b * a.S + (qblk0 + i) * BWD_SUB] > klast) { per_head = i; break; }
    }
  }
  const int niter = per_head * G;

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(&st_full[0], 1); mbar_init(&st_full[1], 1);
    mbar_init(&pds_full, 128); mbar_init(&pds_free, 1); mbar_init(&acc_full, 1);
    mbar_fence_init();
  }
  if (warp == 5) { tmem_alloc(&tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 4) {
    if (elect_one()) {
      mbar_expect_tx(&kv_full, 2 * KTILE);
#pragma unroll
      for (int p = 0; p < NP; ++p) {
        tma_load_4d(sK + p * PANEL_BYTES, &tmK, &kv_full, p * 64, hkv, k0, b);
        tma_load_4d(sV + p * PANEL_BYTES, &tmV, &kv_full, p * 64, hkv, k0, b);
      }
      for (int it = 0; it < niter; ++it) {
        const int st = it & 1;
        const int h = hkv * G + it / per_head;
        const int qrow = (qblk0 + it % per_head) * BWD_SUB;
        if (!mbar_wait(&q_empty[st], ((it >> 1) & 1) ^ 1)) { atomicExch(a.status, 31); goto teardown; }
        mbar_expect_tx(&q_full[st], 2 * QTILE);
#pragma unroll
        for (int p = 0; p < NP; ++p) {
          tma_load_4d(sQ + st * QTILE + p * SUBPANEL_BYTES, &tmQ, &q_full[st], p * 64, h, qrow, b);
          tma_load_4d(sdO + st * QTILE + p * SUBPANEL_BYTES, &tmdO, &q_full[st], p * 64, h, qrow, b);
        }
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      if (!mbar_wait(&kv_full, 0)) { atomicExch(a.status, 32); goto teardown; }
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      // S^T = K Q^T and dP^T = V dO^T of iteration `it` into TMEM buffer it & 1
      auto issue_st = [&](int it) -> bool {
        const int st = it & 1;
        if (!mbar_wait(&q_full[st], (it >> 1) & 1)) return false;
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * QTILE), da = smem_u32(sdO + st * QTILE);
        const uint32_t tb = tmem + st * COL_BUF;
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t aoff = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          const uint32_t boff = (k4 >> 2) * SUBPANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tb + COL_ST, make_smem_desc_sw128(ka + aoff, 16, 1024), make_smem_desc_sw128(qa + boff, 16, 1024),
                   IDESC_ST, k4 > 0);
        }
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t aoff = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          const uint32_t boff = (k4 >> 2) * SUBPANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tb + COL_DPT, make_smem_desc_sw128(va + aoff, 16, 1024),
                   make_smem_desc_sw128(da + boff, 16, 1024), IDESC_ST, k4 > 0);
        }
        umma_commit(&st_full[st]);
        return true;
      };
      if (niter > 0 && !issue_st(0)) { atomicExch(a.status, 33); goto teardown; }
      for (int it = 0; it < niter; ++it) {
        const int st = it & 1;
        // TMEM buffer (it+1)&1 was last read for iteration it-1, whose P^T/dS^T arrival was awaited last time;
        // the Q/dO stage (it+1)&1 is handed back by q_empty after the accumulation MMAs of iteration it-1
        if (it + 1 < niter && !issue_st(it + 1)) { atomicExch(a.status, 33); goto teardown; }
        if (!mbar_wait(&pds_full, it & 1)) { atomicExch(a.status, 34); goto teardown; }
        tc_fence_after();
        const uint32_t qa = smem_u32(sQ + st * QTILE), da = smem_u32(sdO + st * QTILE);
        const uint32_t pa = smem_u32(sPT), sa = smem_u32(sdST);
#pragma unroll
        for (int k4 = 0; k4 < BWD_SUB / 16; ++k4) {
          umma_f16(tmem + COL_DV, make_smem_desc_sw128(pa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(da + k4 * 16 * 128, SUBPANEL_BYTES, 1024), IDESC_ACC, (it > 0 || k4 > 0));
          umma_f16(tmem + COL_DK, make_smem_desc_sw128(sa + k4 * 32, 16, 1024),
                   make_smem_desc_sw128(qa + k4 * 16 * 128, SUBPANEL_BYTES, 1024), IDESC_ACC, (it > 0 || k4 > 0));
        }
        umma_commit(&pds_free);
        umma_commit(&q_empty[st]);
      }
      umma_commit(&acc_full);
    }
  } else {
    const int r = warp * 32 + lane;     // key row
    const int kj = k0 + r;
    const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
    for (int it = 0; it < niter; ++it) {
      const int h = hkv * G + it / per_head;
      const int qrow = (qblk0 + it % per_head) * BWD_SUB;
      // stage lse / delta of the 64 queries (previous iteration's readers are past their loop:
      // they arrived on pds_full after their last read, and this point is after waiting st_full)
      if (!mbar_wait(&st_full[it & 1], (it >> 1) & 1)) { if (lane == 0) atomicExch(a.status, 35); goto teardown; }
      const uint32_t tbuf = tmem + lane_base + (it & 1) * COL_BUF;
      tc_fence_after();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (r < BWD_SUB) {
        const int qi = qrow + r;
        const size_t si = ((size_t)b * a.H + h) * a.S + (qi < a.S ? qi : 0);
        s_lse[r] = a.lse[si] * 1.4426950408889634f;
        s_delta[r] = a.delta[si];
        s_start[r] = (a.doc_start != nullptr && qi < a.S) ? a.doc_start[(size_t)b * a.S + qi] : 0;
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      uint32_t pt[BWD_SUB / 2], dst[BWD_SUB / 2];
      // per-element tests only for query blocks that touch this key block's diagonal, the sequence end or a
      // document boundary (s_start > first key of the block); the tests live in their own branch
      bool need_mask = (qrow < k0 + ATT_BLK) || (qrow + BWD_SUB > a.S) || (k0 + ATT_BLK > a.S);
      if (a.doc_start != nullptr) need_mask = need_mask || (s_start[BWD_SUB - 1] > k0);
#pragma unroll
      for (int c = 0; c < BWD_SUB; c += 32) {        // two chunks: unrolled so the packed results stay in registers
        uint32_t sv[32], dv_[32];
        tmem_ld_32x32(tbuf + COL_ST + c, sv);
        tmem_ld_32x32(tbuf + COL_DPT + c, dv_);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int qi = qrow + c + i;
            if ((kj > qi) || (qi >= a.S) || (kj >= a.S) || (kj < s_start[c + i])) sv[i] = 0xff800000u;   // p = 0
          }
        }
        uint32_t* ptp = &pt[c >> 1];
        uint32_t* dsp = &dst[c >> 1];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2f(fmaf(__uint_as_float(sv[i]), a.scale_log2, -s_lse[c + i]));
          const float p1 = exp2f(fmaf(__uint_as_float(sv[i + 1]), a.scale_log2, -s_lse[c + i + 1]));
          ptp[i >> 1] = pack_bf16(p0, p1);
          dsp[i >> 1] = pack_bf16(p0 * (__uint_as_float(dv_[i]) - s_delta[c + i]) * a.scale,
                                  p1 * (__uint_as_float(dv_[i + 1]) - s_delta[c + i + 1]) * a.scale);
        }
      }
      tc_fence_before();
      if (!mbar_wait(&pds_free, (it & 1) ^ 1)) { if (lane == 0) atomicExch(a.status, 36); goto teardown; }
#pragma unroll
      for (int c = 0; c < BWD_SUB; c += 8) {
        *reinterpret_cast<uint4*>(sPT + swz64(r, c)) = make_uint4(pt[c / 2], pt[c / 2 + 1], pt[c / 2 + 2], pt[c / 2 + 3]);
        *reinterpret_cast<uint4*>(sdST + swz64(r, c)) =
            make_uint4(dst[c / 2], dst[c / 2 + 1], dst[c / 2 + 2], dst[c / 2 + 3]);
      }
      fence_async_smem();
      mbar_arrive(&pds_full);
    }
    if (!mbar_wait(&acc_full, 0)) { if (lane == 0) atomicExch(a.status, 37); goto teardown; }
    tc_fence_after();
    const bool row_ok = kj < a.S;
    const size_t off = (((size_t)b * a.S + (row_ok ? kj : 0)) * a.Hkv + hkv) * D;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* drow = (which == 0 ? a.dv : a.dk) + off;
      const uint32_t col0 = which == 0 ? COL_DV : COL_DK;
#pragma unroll
      for (int c = 0; c < D; c += 32) {
        uint32_t v[32];
        tmem_ld_32x32(tmem + lane_base + col0 + c, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(drow + c + i) =
                make_uint4(pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                           pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                           pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                           pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
        }
      }
    }
    tc_fence_before();
  }
teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// ------------------------------------------------- backward for head_dim 128: 128 x 128 steps, P and dS in TMEM
// Both kernels below keep the structure of the two-tile forward: 8 softmax warps (two warpgroups that split the
// 128 columns of an accumulator in halves; thread = accumulator row), warp 8 is the TMA producer, warp 9 issues
// the MMAs.  The bf16 operands made by the threads (P^T and dS^T for dK/dV, dS for dQ) are written as packed
// pairs over accumulator columns the same warpgroup has already consumed and enter the next MMA as its A
// operand from tensor memory, so no shared memory and no proxy fence is spent on them.  The work of a step is
// two chains that the tensor pipe interleaves: S -> P (exponentials) and dP -> dS (needs P, kept in
// registers); while the threads are in one chain the pipe executes the MMAs of the other.
constexpr int B2_THREADS = 320;
constexpr int B2_TILE_BYTES = 2 * PANEL_BYTES;     // 128 rows x 128 bf16 columns
constexpr int DKV2_Q_STAGES = 2;                   // a third stage would not fit beside K, V, two dO stages and the statistics

// dK, dV of one (128-key block, KV head, batch): loops over the query heads of the group and over the
// 128-query blocks at or after the key block.  TMEM: S^T | dP^T | dV | dK, 128 columns each.
__global__ void __launch_bounds__(B2_THREADS, 1)
attn_bwd_dkv2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                     const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                     const AttnBwdArgs a) {
  constexpr int D = 128;
  constexpr int NQ = DKV2_Q_STAGES;
  constexpr uint32_t IDESC_ST = make_idesc_f16(128, 128, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_ACC = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  constexpr uint32_t TMEM_COLS = 512, COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 384;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + B2_TILE_BYTES;
  // Q is held until the dK MMAs of its step, the last of the step;
  // dO is released by the dV MMAs in mid-step.
  uint8_t* sQ = sV + B2_TILE_BYTES;             // NQ stages (with the row statistics)
  uint8_t* sdO = sQ + NQ * B2_TILE_BYTES;        // 2 stages
  __shared__ uint64_t kv_full, q_full[NQ], q_empty[NQ], stat_full[NQ], do_full[2], do_empty[2];
  __shared__ uint64_t st_full, dpt_full, p_full, ds_full, acc_full;
  __shared__ uint32_t tmem_slot;
  __shared__ __align__(16) float s_lse[NQ][128], s_delta[NQ][128];   // -lse * log2(e), -delta * scale
  __shared__ __align__(16) int s_start[NQ][128];

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // the key block is the slowest grid dimension: the heavy (early) key blocks of all heads are scheduled first
  const int kb = blockIdx.z, hkv = blockIdx.x, b = blockIdx.y;
  const int G = a.H / a.Hkv;
  const int k0 = kb * ATT_BLK;
  const int qblk1 = (a.S + ATT_BLK - 1) / ATT_BLK;
  int per_head = qblk1 - kb;
  if (a.doc_start != nullptr) {
    // packed documents: once a query block starts in a document that begins after this key block's last key,
    // it and all later query blocks cannot see the block (document starts do not decrease along the sequence)
    const int klast = min(k0 + ATT_BLK, a.S) - 1;
    for (int i = 1; i < per_head; ++i) {
      if (a.doc_start[(size_t)b * a.S + (kb + i) * ATT_BLK] > klast) { per_head = i; break; }
    }
  }
  const int niter = per_head * G;

  if (threadIdx.x == 0) {
    mbar_init(&kv_full, 1);
    for (int i = 0; i < NQ; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); mbar_init(&stat_full[i], 32); }
    for (int i = 0; i < 2; ++i) { mbar_init(&do_full[i], 1); mbar_init(&do_empty[i], 1); }
    mbar_init(&st_full, 1); mbar_init(&dpt_full, 1);
    mbar_init(&p_full, 256); mbar_init(&ds_full, 256); mbar_init(&acc_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmdO); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 9) { tmem_alloc(&tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------------ producer: tiles by TMA, row statistics
    if (elect_one()) {
      mbar_expect_tx(&kv_full, 2 * B2_TILE_BYTES);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        tma_load_4d(sK + p * PANEL_BYTES, &tmK, &kv_full, p * 64, hkv, k0, b);
        tma_load_4d(sV + p * PANEL_BYTES, &tmV, &kv_full, p * 64, hkv, k0, b);
      }
    }
    __syncwarp();
    for (int it = 0; it < niter; ++it) {
      const int qs = it % NQ, os = it & 1;
      const int h = hkv * G + it / per_head;
      const int qrow = (kb + it % per_head) * ATT_BLK;
      // the Q stage (tile and statistics) is free once the dK MMAs of step it - 3 have completed
      if (!mbar_wait(&q_empty[qs], ((it / NQ) & 1) ^ 1)) { if (lane == 0) atomicExch(a.status, 41); goto teardown; }
      __syncwarp();
      if (elect_one()) {
        mbar_expect_tx(&q_full[qs], B2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sQ + qs * B2_TILE_BYTES + p * PANEL_BYTES, &tmQ, &q_full[qs], p * 64, h, qrow, b);
      }
      __syncwarp();
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = lane + 32 * i;
        const int qi = qrow + r;
        const size_t si = ((size_t)b * a.H + h) * a.S + (qi < a.S ? qi : 0);
        s_lse[qs][r] = -a.lse[si] * 1.4426950408889634f;       // the exponent is s * scale_log2 + this
        s_delta[qs][r] = -a.delta[si] * a.scale;                // dS = P * (dP * scale + this)
        s_start[qs][r] = (a.doc_start != nullptr && qi < a.S) ? a.doc_start[(size_t)b * a.S + qi] : 0;
      }
      mbar_arrive(&stat_full[qs]);
      // the dO stage is free once the dV MMAs of step it - 2 have completed
      if (!mbar_wait(&do_empty[os], ((it >> 1) & 1) ^ 1)) { if (lane == 0) atomicExch(a.status, 40); goto teardown; }
      __syncwarp();
      if (elect_one()) {
        mbar_expect_tx(&do_full[os], B2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sdO + os * B2_TILE_BYTES + p * PANEL_BYTES, &tmdO, &do_full[os], p * 64, h, qrow, b);
      }
      __syncwarp();
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------------ MMA issuer
    if (elect_one() && niter > 0) {
      const uint32_t ka = smem_u32(sK), va = smem_u32(sV);
      // S^T = K Q^T or dP^T = V dO^T of one stage: 128 x 128 x 128
      auto issue_t = [&](uint32_t col, uint32_t a_base, uint32_t b_base) {
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t off = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tmem + col, make_smem_desc_sw128(a_base + off, 16, 1024),
                   make_smem_desc_sw128(b_base + off, 16, 1024), IDESC_ST, k4 > 0);
        }
      };
      // acc += X^T Y with X^T (128 keys x 128 queries, packed bf16) in tensor memory: queries 0-63 sit in the
      // 32 columns at `col`, queries 64-127 in the 32 columns at `col` + 64 (each warpgroup packs over its own half)
      auto issue_acc = [&](uint32_t acc, uint32_t col, uint32_t y_base, bool first) {
#pragma unroll
        for (int k4 = 0; k4 < ATT_BLK / 16; ++k4)
          umma_f16_ts(tmem + acc, tmem + col + (k4 >> 2) * 64 + (k4 & 3) * 8,
                      make_smem_desc_sw128(y_base + k4 * 16 * 128, PANEL_BYTES, 1024), IDESC_ACC, (!first || k4 > 0));
      };
      if (!mbar_wait(&kv_full, 0)) { atomicExch(a.status, 42); goto teardown; }
      if (!mbar_wait(&q_full[0], 0)) { atomicExch(a.status, 43); goto teardown; }
      tc_fence_after();
      issue_t(COL_ST, ka, smem_u32(sQ));
      umma_commit(&st_full);
      if (!mbar_wait(&do_full[0], 0)) { atomicExch(a.status, 43); goto teardown; }
      tc_fence_after();
      issue_t(COL_DPT, va, smem_u32(sdO));
      umma_commit(&dpt_full);
      for (int it = 0; it < niter; ++it) {
        const int qs = it % NQ, qn = (it + 1) % NQ, os = it & 1, on = os ^ 1;
        const uint32_t qa = smem_u32(sQ + qs * B2_TILE_BYTES), da = smem_u32(sdO + os * B2_TILE_BYTES);
        // chain 1: P^T(it) -> dV, then S^T(it + 1) over the same columns (in order behind the dV MMAs)
        if (!mbar_wait(&p_full, it & 1)) { atomicExch(a.status, 44); goto teardown; }
        tc_fence_after();
        issue_acc(COL_DV, COL_ST, da, it == 0);
        umma_commit(&do_empty[os]);
        if (it + 1 < niter) {
          if (!mbar_wait(&q_full[qn], ((it + 1) / NQ) & 1)) { atomicExch(a.status, 45); goto teardown; }
          tc_fence_after();
          issue_t(COL_ST, ka, smem_u32(sQ + qn * B2_TILE_BYTES));
          umma_commit(&st_full);
        }
        // chain 2: dS^T(it) -> dK, then dP^T(it + 1)
        if (!mbar_wait(&ds_full, it & 1)) { atomicExch(a.status, 46); goto teardown; }
        tc_fence_after();
        issue_acc(COL_DK, COL_DPT, qa, it == 0);
        umma_commit(&q_empty[qs]);
        if (it + 1 < niter) {
          if (!mbar_wait(&do_full[on], ((it + 1) >> 1) & 1)) { atomicExch(a.status, 45); goto teardown; }
          tc_fence_after();
          issue_t(COL_DPT, va, smem_u32(sdO + on * B2_TILE_BYTES));
          umma_commit(&dpt_full);
        }
      }
      umma_commit(&acc_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups (thread = key row)
    const int wg = warp >> 2;
    const int cb = wg * 64;                        // this warpgroup's query columns of the step
    const int r = (warp & 3) * 32 + lane;
    const int kj = k0 + r;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + COL_ST + cb;
    const uint32_t t_dp = tmem + lane_base + COL_DPT + cb;
    const uint64_t sl2 = pack_f32x2(a.scale_log2, a.scale_log2), sc2 = pack_f32x2(a.scale, a.scale);
    for (int it = 0; it < niter; ++it) {
      const int st = it % NQ;
      const int qrow = (kb + it % per_head) * ATT_BLK;
      if (!mbar_wait(&stat_full[st], (it / NQ) & 1)) { if (lane == 0) atomicExch(a.status, 47); goto teardown; }
      if (!mbar_wait(&st_full, it & 1)) { if (lane == 0) atomicExch(a.status, 48); goto teardown; }
      tc_fence_after();
      // per-element tests only for steps that touch the diagonal, the sequence end or a document boundary
      bool need_mask = (qrow < k0 + ATT_BLK) || (qrow + ATT_BLK > a.S) || (k0 + ATT_BLK > a.S);
      if (a.doc_start != nullptr) need_mask = need_mask || (s_start[st][ATT_BLK - 1] > k0);
      uint64_t p2[32];                             // P of this thread's 64 queries, fp32 pairs
      {
        uint32_t sv[64];
        tmem_ld_32x32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int qi = qrow + cb + i;
            if ((kj > qi) || (qi >= a.S) || (kj >= a.S) || (kj < s_start[st][cb + i])) sv[i] = 0xff800000u;  // p = 0
          }
        }
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const uint64_t x = fma_f32x2(pack_f32x2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), sl2,
                                       *reinterpret_cast<const uint64_t*>(&s_lse[st][cb + 2 * i]));
          float x0, x1;
          unpack_f32x2(x, x0, x1);
          const float e0 = ex2_approx(x0), e1 = ex2_approx(x1);
          p2[i] = pack_f32x2(e0, e1);
          pk[i] = pack_bf16(e0, e1);
        }
        tmem_st_32x32(t_s, pk);                     // over columns this warpgroup has consumed
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full);
      if (!mbar_wait(&dpt_full, it & 1)) { if (lane == 0) atomicExch(a.status, 49); goto teardown; }
      tc_fence_after();
      {
        uint32_t dv_[64];
        tmem_ld_32x32(t_dp, *reinterpret_cast<uint32_t(*)[32]>(&dv_[0]));
        tmem_ld_32x32(t_dp + 32, *reinterpret_cast<uint32_t(*)[32]>(&dv_[32]));
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // dS = P * (dP - delta) * scale = P * (dP * scale - delta * scale)
          const uint64_t t = fma_f32x2(pack_f32x2(__uint_as_float(dv_[2 * i]), __uint_as_float(dv_[2 * i + 1])), sc2,
                                       *reinterpret_cast<const uint64_t*>(&s_delta[st][cb + 2 * i]));
          float d0, d1;
          unpack_f32x2(mul_f32x2(p2[i], t), d0, d1);
          pk[i] = pack_bf16(d0, d1);
        }
        tmem_st_32x32(t_dp, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full);
    }
    if (niter > 0) {
      if (!mbar_wait(&acc_full, 0)) { if (lane == 0) atomicExch(a.status, 50); goto teardown; }
      tc_fence_after();
    }
    const bool row_ok = kj < a.S;
    const size_t off = (((size_t)b * a.S + (row_ok ? kj : 0)) * a.Hkv + hkv) * D + cb;
#pragma unroll
    for (int which = 0; which < 2; ++which) {
      __nv_bfloat16* drow = (which == 0 ? a.dv : a.dk) + off;
      const uint32_t col0 = (which == 0 ? COL_DV : COL_DK) + cb;
#pragma unroll 1
      for (int c = 0; c < 64; c += 32) {
        uint32_t v[32];
        if (niter > 0) {
          tmem_ld_32x32(tmem + lane_base + col0 + c, v);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 32; i += 8)
            *reinterpret_cast<uint4*>(drow + c + i) =
                make_uint4(pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                           pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                           pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                           pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
        }
      }
    }
    tc_fence_before();
  }
teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

// dQ of one (128-query block, head, batch): loops over the 128-key blocks the block can see.
// TMEM: S | dP (two buffers, step parity) | dQ, 128 columns each.  S and dP of step j + 1 are issued as soon as
// the threads have read S of step j into registers, a whole thread phase ahead of their use.
__global__ void __launch_bounds__(B2_THREADS, 1)
attn_bwd_dq2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmdO,
                    const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                    const AttnBwdArgs a) {
  constexpr int D = 128;
  constexpr uint32_t IDESC_S = make_idesc_f16(128, 128, 1, KMOE_MAJOR_K, KMOE_MAJOR_K);
  constexpr uint32_t IDESC_DQ = make_idesc_f16(128, D, 1, KMOE_MAJOR_K, KMOE_MAJOR_MN);
  constexpr uint32_t TMEM_COLS = 512, COL_S = 0, COL_DP = 128, COL_DQ = 384;   // dP buffer b at COL_DP + 128 b

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sdO = sQ + B2_TILE_BYTES;
  // K is held until the dQ MMAs of its step: a third stage lets the load of step j + 1 start a whole step ahead
  uint8_t* sK = sdO + B2_TILE_BYTES;            // 3 stages
  uint8_t* sV = sK + 3 * B2_TILE_BYTES;         // 2 stages
  __shared__ uint64_t qdo_full, k_full[3], v_full[2], k_empty[3], v_empty[2], s_full, s_free, dp_full[2], ds_full[2], dq_full;
  __shared__ uint32_t tmem_slot;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qb = gridDim.z - 1 - blockIdx.z;    // slowest grid dimension: heavy (late) query blocks first
  const int h = blockIdx.x, b = blockIdx.y;
  const int hkv = h / (a.H / a.Hkv);
  const int q0 = qb * ATT_BLK;
  const int kmax = min(q0 + ATT_BLK, a.S);
  // packed documents: key blocks that end before the document of the block's first query are invisible to all rows
  const int jlo = a.doc_start != nullptr ? a.doc_start[(size_t)b * a.S + q0] / ATT_BLK : 0;
  const int nblk = (kmax + ATT_BLK - 1) / ATT_BLK - jlo;

  if (threadIdx.x == 0) {
    mbar_init(&qdo_full, 1);
    for (int i = 0; i < 3; ++i) { mbar_init(&k_full[i], 1); mbar_init(&k_empty[i], 1); }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&v_full[i], 1); mbar_init(&v_empty[i], 1); mbar_init(&dp_full[i], 1); mbar_init(&ds_full[i], 256);
    }
    mbar_init(&s_full, 1); mbar_init(&s_free, 256); mbar_init(&dq_full, 1);
    mbar_fence_init();
    prefetch_tmap(&tmQ); prefetch_tmap(&tmdO); prefetch_tmap(&tmK); prefetch_tmap(&tmV);
  }
  if (warp == 9) { tmem_alloc(&tmem_slot, TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = tmem_slot;

  if (warp == 8) {
    if (elect_one() && nblk > 0) {
      mbar_expect_tx(&qdo_full, 2 * B2_TILE_BYTES);
#pragma unroll
      for (int p = 0; p < 2; ++p) {
        tma_load_4d(sQ + p * PANEL_BYTES, &tmQ, &qdo_full, p * 64, h, q0, b);
        tma_load_4d(sdO + p * PANEL_BYTES, &tmdO, &qdo_full, p * 64, h, q0, b);
      }
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1, ks = j % 3;
        if (!mbar_wait(&k_empty[ks], ((j / 3) & 1) ^ 1)) { atomicExch(a.status, 51); goto teardown; }
        mbar_expect_tx(&k_full[ks], B2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sK + ks * B2_TILE_BYTES + p * PANEL_BYTES, &tmK, &k_full[ks], p * 64, hkv, (jlo + j) * ATT_BLK, b);
        if (!mbar_wait(&v_empty[st], ((j >> 1) & 1) ^ 1)) { atomicExch(a.status, 52); goto teardown; }
        mbar_expect_tx(&v_full[st], B2_TILE_BYTES);
#pragma unroll
        for (int p = 0; p < 2; ++p)
          tma_load_4d(sV + st * B2_TILE_BYTES + p * PANEL_BYTES, &tmV, &v_full[st], p * 64, hkv, (jlo + j) * ATT_BLK, b);
      }
    }
  } else if (warp == 9) {
    if (elect_one() && nblk > 0) {
      const uint32_t qa = smem_u32(sQ), da = smem_u32(sdO);
      auto issue_t = [&](uint32_t col, uint32_t a_base, uint32_t b_base) {
#pragma unroll
        for (int k4 = 0; k4 < D / 16; ++k4) {
          const uint32_t off = (k4 >> 2) * PANEL_BYTES + (k4 & 3) * 32;
          umma_f16(tmem + col, make_smem_desc_sw128(a_base + off, 16, 1024),
                   make_smem_desc_sw128(b_base + off, 16, 1024), IDESC_S, k4 > 0);
        }
      };
      if (!mbar_wait(&qdo_full, 0)) { atomicExch(a.status, 53); goto teardown; }
      if (!mbar_wait(&k_full[0], 0)) { atomicExch(a.status, 54); goto teardown; }
      tc_fence_after();
      issue_t(COL_S, qa, smem_u32(sK));
      umma_commit(&s_full);
      if (!mbar_wait(&v_full[0], 0)) { atomicExch(a.status, 55); goto teardown; }
      tc_fence_after();
      issue_t(COL_DP, da, smem_u32(sV));
      umma_commit(&dp_full[0]);
      umma_commit(&v_empty[0]);
      for (int j = 0; j < nblk; ++j) {
        const int st = j & 1, nx = st ^ 1, ks = j % 3, kn = (j + 1) % 3;
        if (j + 1 < nblk) {
          if (!mbar_wait(&k_full[kn], ((j + 1) / 3) & 1) || !mbar_wait(&v_full[nx], ((j + 1) >> 1) & 1)) {
            atomicExch(a.status, 54);
            goto teardown;
          }
          // S(j) is in the threads' registers: S(j + 1) may overwrite it.  dP(j + 1) goes to the other dP buffer,
          // whose dS(j - 1) the dQ MMAs of step j - 1 (earlier in this pipe) have consumed.
          if (!mbar_wait(&s_free, j & 1)) { atomicExch(a.status, 60); goto teardown; }
          tc_fence_after();
          issue_t(COL_S, qa, smem_u32(sK + kn * B2_TILE_BYTES));
          umma_commit(&s_full);
          issue_t(COL_DP + nx * 128, da, smem_u32(sV + nx * B2_TILE_BYTES));
          umma_commit(&dp_full[nx]);
          umma_commit(&v_empty[nx]);
        }
        // one barrier per dP buffer: a thread may finish dS(j + 1) (it needs only s_free of step j, not this
        // step's dQ MMAs) before a slower thread has arrived for dS(j), and the two must not share a phase
        if (!mbar_wait(&ds_full[st], (j >> 1) & 1)) { atomicExch(a.status, 56); goto teardown; }
        tc_fence_after();
        // dQ += dS K_j with dS (128 queries x 128 keys, packed bf16) in the step's dP buffer: keys 0-63 in its
        // first 32 columns, keys 64-127 in the 32 columns from column 64
        const uint32_t ka = smem_u32(sK + ks * B2_TILE_BYTES);
#pragma unroll
        for (int k4 = 0; k4 < ATT_BLK / 16; ++k4)
          umma_f16_ts(tmem + COL_DQ, tmem + COL_DP + st * 128 + (k4 >> 2) * 64 + (k4 & 3) * 8,
                      make_smem_desc_sw128(ka + k4 * 16 * 128, PANEL_BYTES, 1024), IDESC_DQ, (j > 0 || k4 > 0));
        umma_commit(&k_empty[ks]);
      }
      umma_commit(&dq_full);
    }
  } else {
    // ------------------------------------------------------------------ softmax warpgroups (thread = query row)
    const int wg = warp >> 2;
    const int cb = wg * 64;                        // this warpgroup's key columns of the step
    const int r = (warp & 3) * 32 + lane;
    const int qi = q0 + r;
    const uint32_t lane_base = (uint32_t)((warp & 3) * 32) << 16;
    const bool row_ok = qi < a.S;
    const size_t stat = ((size_t)b * a.H + h) * a.S + (row_ok ? qi : 0);
    const float lse2 = a.lse[stat] * 1.4426950408889634f;
    const float dlt = a.delta[stat];
    const int qstart = (a.doc_start != nullptr && row_ok) ? a.doc_start[(size_t)b * a.S + qi] : 0;
    const uint32_t t_s = tmem + lane_base + COL_S + cb;
    const uint64_t sl2 = pack_f32x2(a.scale_log2, a.scale_log2), nlse = pack_f32x2(-lse2, -lse2);
    const uint64_t sc2 = pack_f32x2(a.scale, a.scale), nds = pack_f32x2(-dlt * a.scale, -dlt * a.scale);
    for (int j = 0; j < nblk; ++j) {
      if (!mbar_wait(&s_full, j & 1)) { if (lane == 0) atomicExch(a.status, 57); goto teardown; }
      tc_fence_after();
      const uint32_t t_dp = tmem + lane_base + COL_DP + (j & 1) * 128 + cb;
      const int k0 = (jlo + j) * ATT_BLK;
      const bool need_mask = (k0 + ATT_BLK > q0) || (k0 + ATT_BLK > a.S) || (k0 < qstart) || !row_ok;
      uint64_t p2[32];                             // P of this thread's 64 keys, fp32 pairs
      {
        uint32_t sv[64];
        tmem_ld_32x32(t_s, *reinterpret_cast<uint32_t(*)[32]>(&sv[0]));
        tmem_ld_32x32(t_s + 32, *reinterpret_cast<uint32_t(*)[32]>(&sv[32]));
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&s_free);                      // S is in registers: the next S may be issued
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 64; ++i) {
            const int kj = k0 + cb + i;
            if ((kj > qi) || (kj >= a.S) || !row_ok || (kj < qstart)) sv[i] = 0xff800000u;   // -inf: p = 0
          }
        }
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float x0, x1;
          unpack_f32x2(fma_f32x2(pack_f32x2(__uint_as_float(sv[2 * i]), __uint_as_float(sv[2 * i + 1])), sl2, nlse),
                       x0, x1);
          p2[i] = pack_f32x2(ex2_approx(x0), ex2_approx(x1));
        }
      }
      if (!mbar_wait(&dp_full[j & 1], (j >> 1) & 1)) { if (lane == 0) atomicExch(a.status, 58); goto teardown; }
      tc_fence_after();
      {
        uint32_t dv_[64];
        tmem_ld_32x32(t_dp, *reinterpret_cast<uint32_t(*)[32]>(&dv_[0]));
        tmem_ld_32x32(t_dp + 32, *reinterpret_cast<uint32_t(*)[32]>(&dv_[32]));
        tmem_ld_wait();
        uint32_t pk[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          // dS = P * (dP - delta) * scale = P * (dP * scale - delta * scale)
          const uint64_t t =
              fma_f32x2(pack_f32x2(__uint_as_float(dv_[2 * i]), __uint_as_float(dv_[2 * i + 1])), sc2, nds);
          float d0, d1;
          unpack_f32x2(mul_f32x2(p2[i], t), d0, d1);
          pk[i] = pack_bf16(d0, d1);
        }
        tmem_st_32x32(t_dp, pk);                    // over columns this warpgroup has consumed
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full[j & 1]);
    }
    if (nblk > 0) {
      if (!mbar_wait(&dq_full, 0)) { if (lane == 0) atomicExch(a.status, 59); goto teardown; }
      tc_fence_after();
    }
    __nv_bfloat16* drow = a.dq + (((size_t)b * a.S + (row_ok ? qi : 0)) * a.H + h) * D + cb;
#pragma unroll 1
    for (int c = 0; c < 64; c += 32) {
      uint32_t v[32];
      if (nblk > 0) {
        tmem_ld_32x32(tmem + lane_base + COL_DQ + cb + c, v);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (row_ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 8)
          *reinterpret_cast<uint4*>(drow + c + i) =
              make_uint4(pack_bf16(__uint_as_float(v[i]), __uint_as_float(v[i + 1])),
                         pack_bf16(__uint_as_float(v[i + 2]), __uint_as_float(v[i + 3])),
                         pack_bf16(__uint_as_float(v[i + 4]), __uint_as_float(v[i + 5])),
                         pack_bf16(__uint_as_float(v[i + 6]), __uint_as_float(v[i + 7])));
      }
    }
    tc_fence_before();
  }
teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem, TMEM_COLS); }
}

}  // namespace kmoe

// ------------------------------------------------------------------ host side
namespace kmoe {

// [B, S, Hx, D] bf16 tensor viewed as dims {D, Hx, S, B}; box = 64 columns of one head for `rows` positions.
static int make_bshd_tmap(CUtensorMap* out, const void* base, int B, int S, int Hx, int D, int rows) {
  cuuint64_t dims[4] = {(cuuint64_t)D, (cuuint64_t)Hx, (cuuint64_t)S, (cuuint64_t)B};
  cuuint64_t strides[3] = {(cuuint64_t)D * 2, (cuuint64_t)Hx * D * 2, (cuuint64_t)S * Hx * D * 2};
  cuuint32_t box[4] = {64, 1, (cuuint32_t)rows, 1};
  return encode_bf16_4d(out, base, dims, strides, box);
}

template <int D>
static int launch_attn_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a,
                           cudaStream_t st) {
  constexpr int NP = D / 64;
  const int smem = NP * PANEL_BYTES + 4 * NP * FWD_KPANEL + ATT_BLK * 128 + 1024;
  auto kern = attn_fwd_kernel<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    attr = true;
  }
  dim3 grid((a.S + ATT_BLK - 1) / ATT_BLK, a.H, a.B);
  kern<<<grid, ATT_THREADS, smem, st>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

static int launch_attn_fwd2(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnArgs& a,
                            cudaStream_t st) {
  const int smem = 6 * F2_TILE_BYTES + 1024;
  auto kern = attn_fwd2_kernel<128>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    attr = true;
  }
  dim3 grid(a.H, a.B, (a.S + 255) / 256);
  kern<<<grid, F2_THREADS, smem, st>>>(tq, tk, tv, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

}  // namespace kmoe

extern "C" int kmoe_attn_fwd(const void* q, const void* k, const void* v, void* out, float* lse, int B, int S, int H,
                             int Hkv, int D, float scale, const int* doc_start, int* status, cudaStream_t st) {
  using namespace kmoe;
  if (D != 64 && D != 128) return -1;
  if (H % Hkv) return -2;
  CUtensorMap tq, tk, tv;
  int rc = make_bshd_tmap(&tq, q, B, S, H, D, ATT_BLK);
  if (rc) return rc;
  AttnArgs a{B, S, H, Hkv, scale * 1.4426950408889634f, (__nv_bfloat16*)out, lse, status, doc_start};
  // head_dim 128: two query tiles per CTA, 128-key steps (KMOE_ATTN_FWD2=0 keeps the one-tile kernel)
  static int fwd2 = -1;
  if (fwd2 < 0) {
    const char* e = getenv("KMOE_ATTN_FWD2");
    fwd2 = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  if (D == 128 && fwd2 == 1) {
    if ((rc = make_bshd_tmap(&tk, k, B, S, Hkv, D, F2_KEYS))) return rc;
    if ((rc = make_bshd_tmap(&tv, v, B, S, Hkv, D, F2_KEYS))) return rc;
    return launch_attn_fwd2(tq, tk, tv, a, st);
  }
  if ((rc = make_bshd_tmap(&tk, k, B, S, Hkv, D, FWD_BN))) return rc;
  if ((rc = make_bshd_tmap(&tv, v, B, S, Hkv, D, FWD_BN))) return rc;
  return D == 128 ? launch_attn_fwd<128>(tq, tk, tv, a, st) : launch_attn_fwd<64>(tq, tk, tv, a, st);
}

namespace kmoe {
template <int D>
static int launch_attn_bwd(const void* q, const void* k, const void* v, const void* d_o, const AttnBwdArgs& a,
                           cudaStream_t st) {
  CUtensorMap tq128, tdo128, tk64, tv64, tq64, tdo64, tk128, tv128;
  int rc;
  if ((rc = make_bshd_tmap(&tq128, q, a.B, a.S, a.H, D, 128))) return rc;
  if ((rc = make_bshd_tmap(&tdo128, d_o, a.B, a.S, a.H, D, 128))) return rc;
  if ((rc = make_bshd_tmap(&tk64, k, a.B, a.S, a.Hkv, D, 64))) return rc;
  if ((rc = make_bshd_tmap(&tv64, v, a.B, a.S, a.Hkv, D, 64))) return rc;
  if ((rc = make_bshd_tmap(&tq64, q, a.B, a.S, a.H, D, 64))) return rc;
  if ((rc = make_bshd_tmap(&tdo64, d_o, a.B, a.S, a.H, D, 64))) return rc;
  if ((rc = make_bshd_tmap(&tk128, k, a.B, a.S, a.Hkv, D, 128))) return rc;
  if ((rc = make_bshd_tmap(&tv128, v, a.B, a.S, a.Hkv, D, 128))) return rc;
  constexpr int NP = D / 64;
  const int smem_dq = 2 * NP * PANEL_BYTES + 4 * NP * SUBPANEL_BYTES + ATT_BLK * 128 + 1024;
  const int smem_dkv = 2 * NP * PANEL_BYTES + 4 * NP * SUBPANEL_BYTES + 2 * ATT_BLK * 128 + 1024;
  auto k1 = attn_bwd_dq_kernel<D>;
  auto k2 = attn_bwd_dkv_kernel<D>;
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(k1, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dq) != cudaSuccess) return -20;
    if (cudaFuncSetAttribute(k2, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv) != cudaSuccess) return -20;
    attr = true;
  }
  const int nb = (a.S + ATT_BLK - 1) / ATT_BLK;
  // head_dim 128: 128 x 128 steps with P / dS in tensor memory.  KMOE_ATTN_BWD2=0 keeps the 64-wide kernels,
  // =dq / =dkv moves only that kernel.
  static int bwd2 = -1;
  constexpr int smem2 = 7 * B2_TILE_BYTES + 1024, smem_dkv2 = (4 + DKV2_Q_STAGES) * B2_TILE_BYTES + 1024;
  if (bwd2 < 0) {
    const char* e = getenv("KMOE_ATTN_BWD2");
    int mode = 3;
    if (e != nullptr && e[0] == '0') mode = 0;
    else if (e != nullptr && e[0] == 'd' && e[1] == 'q') mode = 1;
    else if (e != nullptr && e[0] == 'd' && e[1] == 'k') mode = 2;
    if (D == 128 && mode != 0) {
      if (cudaFuncSetAttribute(attn_bwd_dq2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem2) !=
              cudaSuccess ||
          cudaFuncSetAttribute(attn_bwd_dkv2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_dkv2) !=
              cudaSuccess)
        return -20;
    }
    bwd2 = mode;
  }
  if (D == 128 && (bwd2 & 1))
    attn_bwd_dq2_kernel<<<dim3(a.H, a.B, nb), B2_THREADS, smem2, st>>>(tq128, tdo128, tk128, tv128, a);
  else
    k1<<<dim3(nb, a.H, a.B), ATT_THREADS, smem_dq, st>>>(tq128, tdo128, tk64, tv64, a);
  if (D == 128 && (bwd2 & 2))
    attn_bwd_dkv2_kernel<<<dim3(a.Hkv, a.B, nb), B2_THREADS, smem_dkv2, st>>>(tq128, tdo128, tk128, tv128, a);
  else
    k2<<<dim3(nb, a.Hkv, a.B), ATT_THREADS, smem_dkv, st>>>(tq64, tdo64, tk128, tv128, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
}  // namespace kmoe

// delta is scratch of B*H*S floats.
extern "C" int kmoe_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                             const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int S, int H,
                             int Hkv, int D, float scale, const int* doc_start, int* status, cudaStream_t st) {
  using namespace kmoe;
  if (D != 64 && D != 128) return -1;
  if (H % Hkv) return -2;
  attn_delta_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)d_o, delta, B, S, H, D);
  AttnBwdArgs a{B, S, H, Hkv, scale, scale * 1.4426950408889634f, lse, delta, (__nv_bfloat16*)dq,
                (__nv_bfloat16*)dk, (__nv_bfloat16*)dv, status, doc_start};
  return D == 128 ? launch_attn_bwd<128>(q, k, v, d_o, a, st) : launch_attn_bwd<64>(q, k, v, d_o, a, st);
}
