// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   warp 0      : TMA producer  (cp.async.bulk.tensor -> 128B-swizzled smem ring, mbarrier tx counts)
//   warp 1      : MMA issuer    (tcgen05.mma 128 x BN x 16, accumulators in TMEM, double buffered)
//   warps 2..5  : epilogue      (tcgen05.ld -> registers -> fused epilogue -> global)
//
// One CTA per SM walks a static tile list, so the epilogue of tile i overlaps the
// main loop of tile i+1.  Operands may be K-major or MN-major (the MMA reads either
// from swizzled smem), which covers forward, dgrad and wgrad without transposes.
// Three tile schedules: dense, grouped along M (expert-sorted rows padded to 128
// per expert, tile->expert table and live tile count read from device memory: no
// host synchronisation), and batched (independent GEMMs, optionally with a ragged
// reduction range per group: the wgrad of the experts).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>

#include "kmoe_api.h"
#include "ptx.cuh"
#include "tmap_host.h"

namespace kmoe {

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int A_STAGE_BYTES = BM * BK * 2;
constexpr int NUM_THREADS = 192;

struct GemmArgs {
  void* C;
  const void* D;
  const void* D2;
  void* G_out;
  void* U_out;
  int mode, epilogue;
  int M, N, K, groups;
  long long ldc, ldd, c_gstride;
  int a_grouped, b_grouped;
  const int* tile_group;
  const int* num_m_tiles;
  const int* k_begin;
  const int* k_len;
  int out_f32;
  float alpha, beta, beta2;
  const float* row_scale;
  const float* alpha_dev;     // optional per-group multipliers of alpha / beta (BATCHED: index = group)
  const float* beta_dev;
  int sym_upper;              // C is symmetric (A == B): compute only tiles that touch the upper triangle
  float diag_add;             // added to C[i][i] after alpha (bf16 store path)
  int k_split;                // > 0: reduction elements [k_split, K) of B come from the second tensor map
  const long long* row_ptr;   // optional: address of each output row (may be peer memory); 0 = row not stored
  int* status;
};

struct Tile {
  int m_tile, n_tile, g_a, g_b, g_c, k0, k_blocks;
};

__device__ __forceinline__ int ceil_div(int a, int b) { return (a + b - 1) / b; }

// Maps a linear work index to a tile of TM x BN outputs. Returns false past the end.
template <int BN, int TM = BM>
__device__ __forceinline__ bool get_tile(const GemmArgs& a, int idx, int num_m, int num_n, Tile& t) {
  const int n_out = (a.epilogue == KMOE_EPI_SWIGLU) ? BN / 2 : BN;
  (void)n_out;
  int per_group = num_m * num_n;
  int g = 0, local = idx;
  if (a.sym_upper) {
    // enumerate only the tiles that touch the upper triangle, row by row, so that the work is spread evenly
    int kept = 0;
    for (int m = 0; m < num_m; ++m) kept += num_n - min(num_n, (m * TM) / BN);
    g = idx / kept;
    local = idx - g * kept;
    if (g >= (a.mode == KMOE_GEMM_BATCHED ? a.groups : 1)) return false;
    int m = 0;
    while (true) {
      const int km = num_n - min(num_n, (m * TM) / BN);
      if (local < km) break;
      local -= km;
      ++m;
    }
    t.m_tile = m;
    t.n_tile = min(num_n, (m * TM) / BN) + local;
  } else {
    if (a.mode == KMOE_GEMM_BATCHED) {
      g = idx / per_group;
      local = idx - g * per_group;
      if (g >= a.groups) return false;
    } else if (idx >= per_group) {
      return false;
    }
    // supertile of 8 m-tiles: neighbouring CTAs share B tiles and a narrow band of A
    const int GM = 8;
    int band = local / (GM * num_n);
    int first_m = band * GM;
    int gsz = min(num_m - first_m, GM);
    int r = local - band * GM * num_n;
    t.m_tile = first_m + r % gsz;
    t.n_tile = r / gsz;
  }
  t.k0 = 0;
  t.k_blocks = ceil_div(a.K, BK);
  if (a.mode == KMOE_GEMM_GROUPED_M) {
    int e = a.tile_group[t.m_tile];
    t.g_a = 0;
    t.g_b = e;
    t.g_c = 0;
  } else if (a.mode == KMOE_GEMM_BATCHED) {
    t.g_a = a.a_grouped ? g : 0;
    t.g_b = a.b_grouped ? g : 0;
    t.g_c = g;
    if (a.k_begin != nullptr) {
      t.k0 = a.k_begin[g];
      t.k_blocks = ceil_div(a.k_len[g], BK);
    }
  } else {
    t.g_a = t.g_b = t.g_c = 0;
  }
  return true;
}

template <typename T>
__device__ __forceinline__ void store8(T* dst, const float* v);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* dst, const float* v) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = o;
}
template <>
__device__ __forceinline__ void store8<float>(float* dst, const float* v) {
  *reinterpret_cast<float4*>(dst) = make_float4(v[0], v[1], v[2], v[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(v[4], v[5], v[6], v[7]);
}
__device__ __forceinline__ void load8(const __nv_bfloat16* src, float* v) {
  uint4 r = *reinterpret_cast<const uint4*>(src);
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ void load8(const float* src, float* v) {
  float4 a = *reinterpret_cast<const float4*>(src);
  float4 b = *reinterpret_cast<const float4*>(src + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
  v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

// Writes one 32-column chunk of one row: out = alpha*scale*acc + beta*D
template <typename T>
__device__ __forceinline__ void epilogue_store_chunk(const GemmArgs& a, const uint32_t (&acc)[32], bool have_acc,
                                                     long long row_off_c, long long row_off_d, int col, float scale,
                                                     float beta, long long row_addr, int row = -1) {
  // row_addr != 0: the row's own base address (possibly on a peer GPU) replaces C + row offset
  T* C = row_addr ? reinterpret_cast<T*>(row_addr) - row_off_c : reinterpret_cast<T*>(a.C);
  const T* D = reinterpret_cast<const T*>(a.D);
#pragma unroll
  for (int j = 0; j < 32; j += 8) {
    if (col + j >= a.N) break;
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = have_acc ? __uint_as_float(acc[j + i]) * scale : 0.f;
    if (a.diag_add != 0.f && row >= col + j && row < col + j + 8) {
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += (col + j + i == row) ? a.diag_add : 0.f;
    }
    if (D != nullptr) {
      float d[8];
      load8(D + row_off_d + col + j, d);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += beta * d[i];
    }
    store8<T>(C + row_off_c + col + j, v);
  }
}

template <int BN, int A_MAJOR, int B_MAJOR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
umma_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmB2, const GemmArgs args, const int stages) {
  constexpr int B_STAGE_BYTES = BN * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BN;  // two accumulators
  constexpr uint32_t IDESC = make_idesc_f16(BM, BN, /*bf16*/ 1, A_MAJOR, B_MAJOR);
  constexpr int MAX_STAGES = 8;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[MAX_STAGES];
  __shared__ uint64_t empty_bar[MAX_STAGES];
  __shared__ uint64_t tmem_full[2];
  __shared__ uint64_t tmem_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ __align__(16) __nv_bfloat16 peer_stage[4][32][72];   // per epilogue warp: 32 rows x 64 columns (+pad)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);  // one arrival per epilogue warp
    }
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const bool swiglu = args.epilogue == KMOE_EPI_SWIGLU;
  const int n_per_tile = swiglu ? BN / 2 : BN;  // output columns per tile
  int num_m = ceil_div(args.M, BM);
  if (args.mode == KMOE_GEMM_GROUPED_M) num_m = min(num_m, *args.num_m_tiles);
  const int num_n = ceil_div(args.N, n_per_tile);

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      Tile t;
      for (int idx = blockIdx.x; get_tile<BN>(args, idx, num_m, num_n, t); idx += gridDim.x) {
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            atomicExch(args.status, 1);
            goto teardown;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k = t.k0 + kb * BK;
          if (A_MAJOR == KMOE_MAJOR_K)
            tma_load_4d(sa, &tmA, &full_bar[s], k, t.m_tile * BM, 0, t.g_a);
          else
            tma_load_4d(sa, &tmA, &full_bar[s], 0, k, t.m_tile * (BM / 64), t.g_a);
          if (!swiglu) {
            const bool second = args.k_split > 0 && k >= args.k_split;
            const CUtensorMap* tb = second ? &tmB2 : &tmB;
            const int kb2 = second ? k - args.k_split : k;
            if (B_MAJOR == KMOE_MAJOR_K)
              tma_load_4d(sb, tb, &full_bar[s], kb2, t.n_tile * BN, 0, t.g_b);
            else
              tma_load_4d(sb, tb, &full_bar[s], 0, kb2, t.n_tile * (BN / 64), t.g_b);
          } else {
            constexpr int HB = BN / 2;
            if (B_MAJOR == KMOE_MAJOR_K) {
              tma_load_4d(sb, &tmB, &full_bar[s], k, t.n_tile * HB, 0, t.g_b);
              tma_load_4d(sb + B_STAGE_BYTES / 2, &tmB2, &full_bar[s], k, t.n_tile * HB, 0, t.g_b);
            } else {
              tma_load_4d(sb, &tmB, &full_bar[s], 0, k, t.n_tile * (HB / 64), t.g_b);
              tma_load_4d(sb + B_STAGE_BYTES / 2, &tmB2, &full_bar[s], 0, k, t.n_tile * (HB / 64), t.g_b);
            }
          }
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      Tile t;
      for (int idx = blockIdx.x; get_tile<BN>(args, idx, num_m, num_n, t); idx += gridDim.x) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) {
          atomicExch(args.status, 2);
          goto teardown;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[s], ph)) {
            atomicExch(args.status, 3);
            goto teardown;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            // K-major: 16 bf16 = 32 B along the swizzled row. MN-major: 16 k-rows of 128 B.
            const uint32_t a_off = (A_MAJOR == KMOE_MAJOR_K) ? k4 * 32 : k4 * 16 * 128;
            const uint32_t b_off = (B_MAJOR == KMOE_MAJOR_K) ? k4 * 32 : k4 * 16 * 128;
            const uint64_t adesc = make_smem_desc_sw128(sa + a_off, (A_MAJOR == KMOE_MAJOR_K) ? 16 : BK * 128, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sb + b_off, (B_MAJOR == KMOE_MAJOR_K) ? 16 : BK * 128, 1024);
            umma_f16(d_tmem, adesc, bdesc, IDESC, (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the smem stage once these MMAs retire
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        if (t.k_blocks > 0)
          umma_commit(&tmem_full[acc]);
        else
          mbar_arrive(&tmem_full[acc]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int it = 0;
    Tile t;
    for (int idx = blockIdx.x; get_tile<BN>(args, idx, num_m, num_n, t); idx += gridDim.x) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      ++it;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) {
        if (lane == 0) atomicExch(args.status, 4);
        goto teardown;
      }
      tc_fence_after();
      const bool have_acc = t.k_blocks > 0;
      const int row = t.m_tile * BM + q * 32 + lane;
      const bool row_ok = row < args.M;
      const long long coff = (long long)t.g_c * args.c_gstride + (long long)row * args.ldc;
      const long long doff = (long long)t.g_c * args.c_gstride + (long long)row * args.ldd;
      float scale = args.alpha;
      float beta = args.beta;
      if (args.alpha_dev != nullptr) scale *= args.alpha_dev[t.g_c];
      if (args.beta_dev != nullptr) beta *= args.beta_dev[t.g_c];
      if (args.row_scale != nullptr && row_ok) scale *= args.row_scale[row];
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      long long row_addr = 0;
      bool store_ok = row_ok;
      if (args.row_ptr != nullptr) {
        row_addr = row_ok ? args.row_ptr[row] : 0;
        store_ok = row_addr != 0;
      }
      if (!swiglu && args.row_ptr != nullptr) {
        // Rows go to individual addresses, possibly on peer GPUs.  A lane holds one row, so a direct store
        // would emit 32 scattered 16-byte writes per instruction; the 64-column slab is staged in shared
        // memory instead and written back with 8 lanes per row: four full 128-byte lines per instruction.
        __nv_bfloat16(*stg)[72] = peer_stage[q];
        const __nv_bfloat16* Dp = reinterpret_cast<const __nv_bfloat16*>(args.D);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            uint32_t r[32];
            if (have_acc) {
              tmem_ld_32x32(t_row + c + h * 32, r);
              tmem_ld_wait();
            }
            const int col = t.n_tile * BN + c + h * 32;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              float v[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = have_acc ? __uint_as_float(r[j + i]) * scale : 0.f;
              if (Dp != nullptr && row_ok && col + j < args.N) {
                float d[8];
                load8(Dp + doff + col + j, d);
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += beta * d[i];
              }
              store8<__nv_bfloat16>(&stg[lane][h * 32 + j], v);
            }
          }
          __syncwarp();
#pragma unroll
          for (int it = 0; it < 8; ++it) {
            const int rr = it * 4 + (lane >> 3);
            const int cc = (lane & 7) * 8;
            const long long addr = __shfl_sync(0xffffffffu, row_addr, rr);
            const int gcol = t.n_tile * BN + c + cc;
            if (addr != 0 && gcol < args.N)
              *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(addr) + gcol) =
                  *reinterpret_cast<const uint4*>(&stg[rr][cc]);
          }
          __syncwarp();
        }
      } else if (!swiglu) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          if (have_acc) {
            tmem_ld_32x32(t_row + c, r);
            tmem_ld_wait();
          }
          const int col = t.n_tile * BN + c;
          if (store_ok && col < args.N) {
            if (args.out_f32)
              epilogue_store_chunk<float>(args, r, have_acc, coff, doff, col, scale, beta, row_addr);
            else
              epilogue_store_chunk<__nv_bfloat16>(args, r, have_acc, coff, doff, col, scale, beta, row_addr, row);
          }
        }
      } else {
        constexpr int HB = BN / 2;
        __nv_bfloat16* H = reinterpret_cast<__nv_bfloat16*>(args.C);
        __nv_bfloat16* G = reinterpret_cast<__nv_bfloat16*>(args.G_out);
        __nv_bfloat16* U = reinterpret_cast<__nv_bfloat16*>(args.U_out);
#pragma unroll 1
        for (int c = 0; c < HB; c += 32) {
          uint32_t g[32], u[32];
          if (have_acc) {
            tmem_ld_32x32(t_row + c, g);
            tmem_ld_32x32(t_row + HB + c, u);
            tmem_ld_wait();
          }
          const int col = t.n_tile * HB + c;
          if (row_ok && col < args.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j >= args.N) break;
              float gv[8], uv[8], hv[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                gv[i] = have_acc ? __uint_as_float(g[j + i]) : 0.f;
                uv[i] = have_acc ? __uint_as_float(u[j + i]) : 0.f;
                hv[i] = silu_f(gv[i]) * uv[i] * scale;
              }
              store8<__nv_bfloat16>(H + coff + col + j, hv);
              if (G != nullptr) store8<__nv_bfloat16>(G + coff + col + j, gv);
              if (U != nullptr) store8<__nv_bfloat16>(U + coff + col + j, uv);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[acc]);
    }
  }

teardown:
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ CTA-pair kernel
// The same GEMM with tcgen05.mma.cta_group::2: the two CTAs of a cluster share one 256 x BN tile.  Each CTA
// loads its own 128 rows of A and its own half of B's columns (plain per-CTA TMA loads), the even CTA issues
// 256 x BN x 16 MMAs that read both CTAs' shared memory, and each CTA ends up with its 128 rows of the
// accumulator in its own tensor memory.  Halving the B traffic per CTA is what lifts the tensor pipe off the
// shared-memory bandwidth limit of the single-CTA 128 x 256 tile.
//
// Barriers: `full` lives in the leader and is credited by both CTAs' loads; `empty` and `tmem_full` exist in
// both CTAs and are signalled by the leader's commits (multicast arrive); `tmem_empty` lives in the leader
// and collects the epilogue warps of both CTAs.  DENSE and BATCHED schedules, all epilogues except per-row
// destination addresses.
constexpr int PAIR_TM = 2 * BM;

template <int BN, int A_MAJOR, int B_MAJOR>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
umma_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      const __grid_constant__ CUtensorMap tmB2, const GemmArgs args, const int stages) {
  constexpr int HALF_N = BN / 2;
  constexpr int B_STAGE_BYTES = HALF_N * BK * 2;
  constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;   // per CTA
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr uint32_t IDESC = make_idesc_f16(PAIR_TM, BN, /*bf16*/ 1, A_MAJOR, B_MAJOR);
  constexpr int MAX_STAGES = 8;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[MAX_STAGES];
  __shared__ uint64_t empty_bar[MAX_STAGES];
  __shared__ uint64_t tmem_full[2];
  __shared__ uint64_t tmem_empty[2];
  __shared__ uint32_t tmem_base_slot;
  __shared__ __align__(16) __nv_bfloat16 out_stage[4][32][72];   // per epilogue warp: 32 rows x 64 columns (+pad)

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const bool leader = rank == 0;
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < stages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 8);   // four epilogue warps in each CTA of the pair
    }
    mbar_fence_init();
    prefetch_tmap(&tmA);
    prefetch_tmap(&tmB);
  }
  if (warp == 1) {                    // collective over the pair: the same warp of both CTAs
    tmem_alloc_pair(&tmem_base_slot, TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // the peer's barriers exist before anything is signalled across
  tc_fence_after();
  const uint32_t tmem_base = tmem_base_slot;

  const bool swiglu = args.epilogue == KMOE_EPI_SWIGLU;
  const int n_per_tile = swiglu ? BN / 2 : BN;
  const int num_m = ceil_div(args.M, PAIR_TM);
  const int num_n = ceil_div(args.N, n_per_tile);

  if (warp == 0) {
    // ------------------------------------------------------------ producer (both CTAs)
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      Tile t;
      for (int idx = pair; get_tile<BN, PAIR_TM>(args, idx, num_m, num_n, t); idx += num_pairs) {
        const int arow = t.m_tile * PAIR_TM + (int)rank * BM;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            atomicExch(args.status, 11);
            goto teardown;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + A_STAGE_BYTES;
          if (leader) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          const uint32_t fb = map_to_cta(&full_bar[s], 0);
          const int k = t.k0 + kb * BK;
          if (A_MAJOR == KMOE_MAJOR_K)
            tma_load_4d_pair(sa, &tmA, fb, k, arow, 0, t.g_a);
          else
            tma_load_4d_pair(sa, &tmA, fb, 0, k, arow / 64, t.g_a);
          // B: this CTA's half of the tile's columns; with the SwiGLU epilogue the halves are the gate
          // weight (leader) and the up weight (peer), so accumulator columns [0, BN/2) hold the gate
          const bool second = !swiglu && args.k_split > 0 && k >= args.k_split;
          const CUtensorMap* tb = ((swiglu && !leader) || second) ? &tmB2 : &tmB;
          const int kb2 = second ? k - args.k_split : k;
          const int brow = swiglu ? t.n_tile * HALF_N : t.n_tile * BN + (int)rank * HALF_N;
          if (B_MAJOR == KMOE_MAJOR_K)
            tma_load_4d_pair(sb, tb, fb, kb2, brow, 0, t.g_b);
          else
            tma_load_4d_pair(sb, tb, fb, 0, kb2, brow / 64, t.g_b);
          if (++s == stages) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------- MMA issuer (leader only)
    if (leader && elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      Tile t;
      for (int idx = pair; get_tile<BN, PAIR_TM>(args, idx, num_m, num_n, t); idx += num_pairs) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
        ++it;
        if (!mbar_wait(&tmem_empty[acc], acc_ph ^ 1)) {
          atomicExch(args.status, 12);
          goto teardown;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&full_bar[s], ph)) {
            atomicExch(args.status, 13);
            goto teardown;
          }
          tc_fence_after();
          const uint32_t sa = smem_u32(smem + s * STAGE_BYTES);
          const uint32_t sb = sa + A_STAGE_BYTES;
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint32_t a_off = (A_MAJOR == KMOE_MAJOR_K) ? k4 * 32 : k4 * 16 * 128;
            const uint32_t b_off = (B_MAJOR == KMOE_MAJOR_K) ? k4 * 32 : k4 * 16 * 128;
            const uint64_t adesc = make_smem_desc_sw128(sa + a_off, (A_MAJOR == KMOE_MAJOR_K) ? 16 : BK * 128, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sb + b_off, (B_MAJOR == KMOE_MAJOR_K) ? 16 : BK * 128, 1024);
            umma_f16_pair(d_tmem, adesc, bdesc, IDESC, (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[s], 3);      // frees the stage in both CTAs
          if (++s == stages) { s = 0; ph ^= 1; }
        }
        if (t.k_blocks > 0) {
          umma_commit_pair(&tmem_full[acc], 3);
        } else {
          mbar_arrive(&tmem_full[acc]);
          mbar_arrive_cluster(map_to_cta(&tmem_full[acc], 1));
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs)
    const int q = warp & 3;
    int it = 0;
    Tile t;
    __nv_bfloat16(*stg)[72] = out_stage[q];
    for (int idx = pair; get_tile<BN, PAIR_TM>(args, idx, num_m, num_n, t); idx += num_pairs) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      ++it;
      const bool staged = !swiglu && !args.out_f32;   // this path awaits the accumulator itself
      if (!staged) {
        if (!mbar_wait(&tmem_full[acc], acc_ph)) {
          if (lane == 0) atomicExch(args.status, 14);
          goto teardown;
        }
        tc_fence_after();
      }
      const bool have_acc = t.k_blocks > 0;
      const int row0 = t.m_tile * PAIR_TM + (int)rank * BM + q * 32;
      const int row = row0 + lane;
      const bool row_ok = row < args.M;
      const long long goff = (long long)t.g_c * args.c_gstride;
      const long long coff = goff + (long long)row * args.ldc;
      const long long doff = goff + (long long)row * args.ldd;
      float scale = args.alpha;
      float beta = args.beta;
      if (args.alpha_dev != nullptr) scale *= args.alpha_dev[t.g_c];
      if (args.beta_dev != nullptr) beta *= args.beta_dev[t.g_c];
      if (args.row_scale != nullptr && row_ok) scale *= args.row_scale[row];
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
      if (!swiglu && !args.out_f32) {
        // bf16 output: a lane holds one row, so each 64-column slab is staged in shared memory and written
        // back with 8 lanes per row (four full 128-byte lines per store instruction).  The addend is read
        // with the same pattern.
        __nv_bfloat16* Cb = reinterpret_cast<__nv_bfloat16*>(args.C);
        const __nv_bfloat16* Dp = reinterpret_cast<const __nv_bfloat16*>(args.D);
        constexpr int SLABS = BN / 64;
        if (!mbar_wait(&tmem_full[acc], acc_ph)) {
          if (lane == 0) atomicExch(args.status, 14);
          goto teardown;
        }
        tc_fence_after();
        // symmetric product: a tile strictly above the diagonal also writes its transpose
        const bool mirror = args.sym_upper && t.n_tile * BN >= (t.m_tile + 1) * PAIR_TM;
        const bool diag = args.diag_add != 0.f && t.n_tile * BN < row0 + 32 && (t.n_tile + 1) * BN > row0;
        // Addends of a symmetric product (and every second addend) are added before the slab is staged, each lane
        // reading its own row, so that the mirrored tile is written from final values.
        const __nv_bfloat16* D2p = reinterpret_cast<const __nv_bfloat16*>(args.D2);
        const bool d_early = Dp != nullptr && (args.sym_upper || D2p != nullptr);
        float beta2 = args.beta2;
        if (args.beta_dev != nullptr) beta2 *= args.beta_dev[t.g_c];
        // the slab loop stays rolled: unrolled, the epilogue outgrows the instruction cache and every tile
        // of a short-reduction product stalls on instruction fetch
#pragma unroll 1
        for (int sl = 0; sl < SLABS; ++sl) {
          const int c = sl * 64;
          if (t.n_tile * BN + c >= args.N) break;
          // the addend of this slab is requested first: its latency falls under the accumulator reads below
          uint4 dpre[8];
          auto load_addend = [&](const __nv_bfloat16* P) {      // 8 lanes per row: full 128-byte lines
#pragma unroll
            for (int i8 = 0; i8 < 8; ++i8) {
              const int grow = row0 + i8 * 4 + (lane >> 3);
              const int gcol = t.n_tile * BN + c + (lane & 7) * 8;
              dpre[i8] = (grow < args.M && gcol < args.N)
                             ? __ldg(reinterpret_cast<const uint4*>(P + goff + (long long)grow * args.ldd + gcol))
                             : make_uint4(0, 0, 0, 0);
            }
          };
          if (Dp != nullptr) load_addend(Dp);
          uint32_t r[64];
          if (have_acc) {
            tmem_ld_32x32(t_row + c, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
            tmem_ld_32x32(t_row + c + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
            tmem_ld_wait();
          }
#pragma unroll
          for (int i = 0; i < 64; ++i) r[i] = have_acc ? __float_as_uint(__uint_as_float(r[i]) * scale) : 0u;
          if (diag) {
            const int col0 = t.n_tile * BN + c;
#pragma unroll
            for (int i = 0; i < 64; ++i)
              if (col0 + i == row) r[i] = __float_as_uint(__uint_as_float(r[i]) + args.diag_add);
          }
          if (d_early) {
            // the addends pass through the staging buffer to reach the lane that owns their row
#pragma unroll 1
            for (int pass = 0; pass < (D2p != nullptr ? 2 : 1); ++pass) {
              const float bcoef = pass == 0 ? beta : beta2;
              if (pass == 1) load_addend(D2p);
#pragma unroll
              for (int i8 = 0; i8 < 8; ++i8)
                *reinterpret_cast<uint4*>(&stg[i8 * 4 + (lane >> 3)][(lane & 7) * 8]) = dpre[i8];
              __syncwarp();
#pragma unroll
              for (int j8 = 0; j8 < 8; ++j8) {
                const uint4 q4 = *reinterpret_cast<const uint4*>(&stg[lane][j8 * 8]);
                const __nv_bfloat162* pq = reinterpret_cast<const __nv_bfloat162*>(&q4);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(pq[i]);
                  r[j8 * 8 + 2 * i] = __float_as_uint(__uint_as_float(r[j8 * 8 + 2 * i]) + bcoef * f.x);
                  r[j8 * 8 + 2 * i + 1] = __float_as_uint(__uint_as_float(r[j8 * 8 + 2 * i + 1]) + bcoef * f.y);
                }
              }
              __syncwarp();
            }
          }
#pragma unroll
          for (int j = 0; j < 64; j += 8) store8<__nv_bfloat16>(&stg[lane][j], reinterpret_cast<const float*>(&r[j]));
          __syncwarp();
#pragma unroll
          for (int i8 = 0; i8 < 8; ++i8) {
            const int rr = i8 * 4 + (lane >> 3);
            const int cc = (lane & 7) * 8;
            const int grow = row0 + rr;
            const int gcol = t.n_tile * BN + c + cc;
            if (grow < args.M && gcol < args.N) {
              uint4 o = *reinterpret_cast<const uint4*>(&stg[rr][cc]);
              if (Dp != nullptr && !d_early) {
                float v[8];
                const __nv_bfloat162* pv = reinterpret_cast<const __nv_bfloat162*>(&o);
                const __nv_bfloat162* pd = reinterpret_cast<const __nv_bfloat162*>(&dpre[i8]);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(pv[i]);
                  const float2 d = __bfloat1622float2(pd[i]);
                  v[2 * i] = f.x + beta * d.x;
                  v[2 * i + 1] = f.y + beta * d.y;
                }
                o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]);
                o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
              }
              *reinterpret_cast<uint4*>(Cb + goff + (long long)grow * args.ldc + gcol) = o;
            }
          }
          if (mirror) {
            // C[col][row] = C[row][col]: a lane gathers 8 rows of one staged column (16 bytes of the
            // destination row), 4 lanes cover the 32 rows of the slab
#pragma unroll
            for (int i8 = 0; i8 < 8; ++i8) {
              const int jc = i8 * 8 + (lane >> 2);          // staged column = destination row
              const int r8 = (lane & 3) * 8;                // first of 8 staged rows = destination columns
              const int drow = t.n_tile * BN + c + jc;
              const int dcol = row0 + r8;
              if (drow < args.N && dcol < args.M) {
                __nv_bfloat16 e[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) e[i] = stg[r8 + i][jc];
                *reinterpret_cast<uint4*>(Cb + goff + (long long)drow * args.ldc + dcol) =
                    *reinterpret_cast<const uint4*>(e);
              }
            }
          }
          __syncwarp();
        }
      } else if (!swiglu) {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t r[32];
          if (have_acc) {
            tmem_ld_32x32(t_row + c, r);
            tmem_ld_wait();
          }
          const int col = t.n_tile * BN + c;
          if (row_ok && col < args.N) epilogue_store_chunk<float>(args, r, have_acc, coff, doff, col, scale, beta, 0);
        }
      } else {
        __nv_bfloat16* H = reinterpret_cast<__nv_bfloat16*>(args.C);
        __nv_bfloat16* G = reinterpret_cast<__nv_bfloat16*>(args.G_out);
        __nv_bfloat16* U = reinterpret_cast<__nv_bfloat16*>(args.U_out);
#pragma unroll 1
        for (int c = 0; c < HALF_N; c += 32) {
          uint32_t g[32], u[32];
          if (have_acc) {
            tmem_ld_32x32(t_row + c, g);
            tmem_ld_32x32(t_row + HALF_N + c, u);
            tmem_ld_wait();
          }
          const int col = t.n_tile * HALF_N + c;
          if (row_ok && col < args.N) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              if (col + j >= args.N) break;
              float gv[8], uv[8], hv[8];
#pragma unroll
              for (int i = 0; i < 8; ++i) {
                gv[i] = have_acc ? __uint_as_float(g[j + i]) : 0.f;
                uv[i] = have_acc ? __uint_as_float(u[j + i]) : 0.f;
                hv[i] = silu_f(gv[i]) * uv[i] * scale;
              }
              store8<__nv_bfloat16>(H + coff + col + j, hv);
              if (G != nullptr) store8<__nv_bfloat16>(G + coff + col + j, gv);
              if (U != nullptr) store8<__nv_bfloat16>(U + coff + col + j, uv);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (leader) mbar_arrive(&tmem_empty[acc]);
        else mbar_arrive_cluster(map_to_cta(&tmem_empty[acc], 0));
      }
    }
  }

teardown:
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // nothing of the peer may still point at this CTA's memory
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// Fills the tiles that a symmetric GEMM skipped: C[g][i][j] = C[g][j][i] for every 32x32 block that lies in a
// tile entirely below the diagonal.  grid = (n/32, n/32, groups), block = (32, 8).
__global__ void sym_mirror_kernel(__nv_bfloat16* __restrict__ C, int n, long long ldc, long long gstride, int bn,
                                  int tm) {
  const int bx = blockIdx.x, by = blockIdx.y;
  const int mt = (by * 32) / tm, nt = (bx * 32) / bn;
  if ((nt + 1) * bn > mt * tm) return;                      // destination was computed
  __shared__ __nv_bfloat16 tile[32][33];
  __nv_bfloat16* Cg = C + (long long)blockIdx.z * gstride;
  for (int r = threadIdx.y; r < 32; r += 8)                  // source block: rows 32*bx.., cols 32*by..
    tile[r][threadIdx.x] = Cg[(long long)(bx * 32 + r) * ldc + by * 32 + threadIdx.x];
  __syncthreads();
  for (int r = threadIdx.y; r < 32; r += 8)
    Cg[(long long)(by * 32 + r) * ldc + bx * 32 + threadIdx.x] = tile[threadIdx.x][r];
}

// ------------------------------------------------------------------ host side
using TmapKey = std::tuple<const void*, int, long long, long long, long long, long long, int, int>;
static std::map<TmapKey, CUtensorMap> g_tmap_cache;
static std::mutex g_tmap_mutex;

// Operand tensor map (bf16, 128B swizzle), always rank 4 so one TMA instruction form serves all cases.
//   K-major : dims {K, rows, 1, G}       box {64, tile_rows, 1, 1}
//   MN-major: dims {64, K, rows/64, G}   box {64, 64, tile_rows/64, 1}   (memory is [K][rows], rows contiguous)
static int make_operand_tmap(CUtensorMap* out, const void* base, int major, long long rows, long long K,
                             long long ld, long long gstride, int groups, int tile_rows) {
  TmapKey key{base, major, rows, K, ld, gstride, groups, tile_rows};
  {
    std::lock_guard<std::mutex> lk(g_tmap_mutex);
    auto it = g_tmap_cache.find(key);
    if (it != g_tmap_cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  const long long gs = (groups > 1 && gstride > 0) ? gstride : (major == KMOE_MAJOR_K ? rows * ld : K * ld);
  const int G = (groups > 1 && gstride > 0) ? groups : 1;
  if (major == KMOE_MAJOR_K) {
    dims[0] = (cuuint64_t)K; dims[1] = (cuuint64_t)rows; dims[2] = 1; dims[3] = (cuuint64_t)G;
    strides[0] = (cuuint64_t)ld * 2; strides[1] = (cuuint64_t)rows * ld * 2; strides[2] = (cuuint64_t)gs * 2;
    box[0] = BK; box[1] = (cuuint32_t)tile_rows; box[2] = 1; box[3] = 1;
  } else {
    if (rows % 64 != 0) return -11;
    dims[0] = 64; dims[1] = (cuuint64_t)K; dims[2] = (cuuint64_t)(rows / 64); dims[3] = (cuuint64_t)G;
    strides[0] = (cuuint64_t)ld * 2; strides[1] = 128; strides[2] = (cuuint64_t)gs * 2;
    box[0] = 64; box[1] = BK; box[2] = (cuuint32_t)(tile_rows / 64); box[3] = 1;
  }
  const int rc = encode_bf16_4d(out, base, dims, strides, box);
  if (rc) return rc;
  {
    std::lock_guard<std::mutex> lk(g_tmap_mutex);
    if (g_tmap_cache.size() > 4096) g_tmap_cache.clear();
    g_tmap_cache[key] = *out;
  }
  return 0;
}

template <int BN, int AM, int BMj>
static int launch_variant(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2, const GemmArgs& args,
                          int grid, cudaStream_t stream) {
  constexpr int stage_bytes = A_STAGE_BYTES + BN * BK * 2;
  int stages = (196 * 1024) / stage_bytes;      // leaves room for the 18 KB static staging buffer
  if (stages > 8) stages = 8;
  const int smem = stages * stage_bytes + 1024;
  auto kern = umma_gemm_kernel<BN, AM, BMj>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    attr_set = true;
  }
  kern<<<grid, NUM_THREADS, smem, stream>>>(tA, tB, tB2, args, stages);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

template <int BN, int AM, int BMj>
static int launch_pair_variant(const CUtensorMap& tA, const CUtensorMap& tB, const CUtensorMap& tB2,
                               const GemmArgs& args, long long pair_tiles, int sms, cudaStream_t stream) {
  constexpr int stage_bytes = A_STAGE_BYTES + (BN / 2) * BK * 2;
  int stages = (196 * 1024) / stage_bytes;
  if (stages > 8) stages = 8;
  const int smem = stages * stage_bytes + 1024;
  auto kern = umma_gemm_pair_kernel<BN, AM, BMj>;
  static int max_clusters = 0;
  if (max_clusters == 0) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return -20;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(2 * (sms / 2)));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = (size_t)smem;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeClusterDimension;
    at[0].val.clusterDim.x = 2; at[0].val.clusterDim.y = 1; at[0].val.clusterDim.z = 1;
    cfg.attrs = at; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n < 1) n = sms / 2;
    max_clusters = n;
  }
  long long pairs = pair_tiles < max_clusters ? pair_tiles : max_clusters;
  if (pairs < 1) pairs = 1;
  kern<<<(unsigned)(2 * pairs), NUM_THREADS, smem, stream>>>(tA, tB, tB2, args, stages);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}

// KMOE_GEMM_PAIR=0 keeps every GEMM on the single-CTA kernel.
static bool pair_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("KMOE_GEMM_PAIR");
    v = (e != nullptr && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

}  // namespace kmoe

extern "C" void kmoe_gemm_clear_tensormap_cache(void) {
  std::lock_guard<std::mutex> lk(kmoe::g_tmap_mutex);
  kmoe::g_tmap_cache.clear();
}

extern "C" int kmoe_gemm(const KmoeGemmDesc* d, cudaStream_t stream) {
  using namespace kmoe;
  // 16-byte rows for TMA: the reduction length only matters for an operand whose rows run along it
  if (d->N % 8 != 0) return -1;
  if ((d->a_major == KMOE_MAJOR_K || d->b_major == KMOE_MAJOR_K) && d->K % 8 != 0) return -1;
  if (d->K <= 0 || d->M <= 0 || d->N <= 0) return -2;
  if (d->c_row_ptr != nullptr && (d->out_f32 || d->epilogue != KMOE_EPI_STORE)) return -3;
  if (d->k_split != 0 && (d->k_split % BK || d->k_split <= 0 || d->k_split >= d->K || d->B2 == nullptr ||
                          d->epilogue != KMOE_EPI_STORE || d->k_begin != nullptr))
    return -5;
  const bool swiglu = d->epilogue == KMOE_EPI_SWIGLU;
  // narrow outputs use the 128-wide tile so more CTAs get work
  const int n_tiles_256 = (d->N + (swiglu ? 127 : 255)) / (swiglu ? 128 : 256);
  const long long m_tiles = (d->M + BM - 1) / BM;
  const long long groups = d->mode == KMOE_GEMM_BATCHED ? d->groups : 1;
  int sms = d->num_sms;
  if (sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  // CTA-pair kernel (256-row tiles): every schedule except the expert-padded one (its row blocks are 128 high
  // and neighbouring blocks may belong to different experts) and per-row destination addresses
  const bool pair = pair_enabled() && d->mode != KMOE_GEMM_GROUPED_M && d->c_row_ptr == nullptr && d->M > BM;
  const int TM = pair ? PAIR_TM : BM;
  const long long tm_tiles = (d->M + TM - 1) / TM;
  const int units = pair ? sms / 2 : sms;       // CTAs or CTA pairs that run at once
  // 256-wide tiles unless that would leave most of the machine idle.  A CTA pair on 256 x 128 tiles asks the L2
  // for about 1.5x the bytes per FLOP of a 256 x 256 tile and runs at nearly the same time per reduction block,
  // so two waves of narrow tiles are slower than one partly filled wave of wide ones.
  const long long tiles256 = tm_tiles * n_tiles_256 * groups;
  const bool use256 = swiglu || (d->N >= 256 && (pair ? 2 * tiles256 > units : tiles256 >= units));
  const int BN = use256 ? 256 : 128;
  const int b_box_rows = pair ? BN / 2 : (swiglu ? BN / 2 : BN);

  GemmArgs a;
  a.C = d->C; a.D = d->D; a.D2 = d->D2; a.beta2 = d->beta2; a.G_out = d->G_out; a.U_out = d->U_out;
  a.mode = d->mode; a.epilogue = d->epilogue;
  a.M = d->M; a.N = d->N; a.K = d->K; a.groups = d->groups;
  a.ldc = d->ldc; a.ldd = d->ldd ? d->ldd : d->ldc; a.c_gstride = d->c_gstride;
  a.a_grouped = d->a_gstride != 0; a.b_grouped = d->b_gstride != 0;
  a.tile_group = d->tile_group; a.num_m_tiles = d->num_m_tiles;
  a.k_begin = d->k_begin; a.k_len = d->k_len;
  a.out_f32 = d->out_f32; a.alpha = d->alpha; a.beta = d->beta;
  a.row_scale = d->row_scale; a.row_ptr = d->c_row_ptr; a.status = d->status;
  a.alpha_dev = d->alpha_dev; a.beta_dev = d->beta_dev;
  a.sym_upper = d->sym_upper;
  a.diag_add = d->diag_add;
  a.k_split = d->k_split;
  if (d->sym_upper && (d->M != d->N || swiglu || d->mode == KMOE_GEMM_GROUPED_M || d->out_f32 || d->N % 32 ||
                       (d->D != nullptr && !pair)))
    return -4;
  // the second addend exists in the bf16 epilogue of the CTA-pair kernel only
  if (d->D2 != nullptr && (!pair || swiglu || d->out_f32 || d->D == nullptr)) return -6;

  // The reduction extent seen by TMA: ragged batched GEMMs index a shared [sum K, rows] buffer.
  long long k_extent_a = d->K, k_extent_b = d->K;
  if (d->mode == KMOE_GEMM_BATCHED && d->k_begin != nullptr) {
    k_extent_a = d->a_gstride == 0 ? (long long)d->K : d->K;
    k_extent_b = k_extent_a;
  }
  const int a_groups = (d->mode == KMOE_GEMM_BATCHED && d->a_gstride != 0) ? d->groups : 1;
  const int b_groups = d->b_gstride != 0 ? d->groups : 1;
  CUtensorMap tA, tB, tB2;
  int rc = make_operand_tmap(&tA, d->A, d->a_major, d->M, k_extent_a, d->lda, d->a_gstride, a_groups, BM);
  if (rc) return rc;
  if (d->k_split > 0) k_extent_b = d->k_split;
  rc = make_operand_tmap(&tB, d->B, d->b_major, d->N, k_extent_b, d->ldb, d->b_gstride, b_groups, b_box_rows);
  if (rc) return rc;
  if (d->k_split > 0) {
    rc = make_operand_tmap(&tB2, d->B2, d->b_major, d->N, d->K - d->k_split, d->ldb, d->b_gstride, b_groups,
                           b_box_rows);
    if (rc) return rc;
  } else if (swiglu) {
    rc = make_operand_tmap(&tB2, d->B2, d->b_major, d->N, k_extent_b, d->ldb, d->b_gstride, b_groups, b_box_rows);
    if (rc) return rc;
  } else {
    tB2 = tB;
  }
  const int n_per_tile = swiglu ? BN / 2 : BN;
  long long total = tm_tiles * ((d->N + n_per_tile - 1) / n_per_tile) * groups;
  if (d->sym_upper) {
    const long long nn = (d->N + BN - 1) / BN;
    long long kept = 0;
    for (long long m = 0; m < tm_tiles; ++m) kept += nn - std::min<long long>(nn, (m * TM) / BN);
    total = kept * groups;
  }
  int grid = (int)(total < sms ? total : sms);
  if (grid < 1) grid = 1;

  int lrc = 0;
#define KMOE_LAUNCH_PAIR(BN_, AM_, BM_) lrc = launch_pair_variant<BN_, AM_, BM_>(tA, tB, tB2, a, total, sms, stream)
#define KMOE_LAUNCH(BN_, AM_, BM_) lrc = launch_variant<BN_, AM_, BM_>(tA, tB, tB2, a, grid, stream)
  if (pair && BN == 256) {
    if (d->a_major == 0 && d->b_major == 0) KMOE_LAUNCH_PAIR(256, 0, 0);
    else if (d->a_major == 0 && d->b_major == 1) KMOE_LAUNCH_PAIR(256, 0, 1);
    else if (d->a_major == 1 && d->b_major == 0) KMOE_LAUNCH_PAIR(256, 1, 0);
    else KMOE_LAUNCH_PAIR(256, 1, 1);
  } else if (pair) {
    if (d->a_major == 0 && d->b_major == 0) KMOE_LAUNCH_PAIR(128, 0, 0);
    else if (d->a_major == 0 && d->b_major == 1) KMOE_LAUNCH_PAIR(128, 0, 1);
    else if (d->a_major == 1 && d->b_major == 0) KMOE_LAUNCH_PAIR(128, 1, 0);
    else KMOE_LAUNCH_PAIR(128, 1, 1);
  } else if (BN == 256) {
    if (d->a_major == 0 && d->b_major == 0) KMOE_LAUNCH(256, 0, 0);
    else if (d->a_major == 0 && d->b_major == 1) KMOE_LAUNCH(256, 0, 1);
    else if (d->a_major == 1 && d->b_major == 0) KMOE_LAUNCH(256, 1, 0);
    else KMOE_LAUNCH(256, 1, 1);
  } else {
    if (d->a_major == 0 && d->b_major == 0) KMOE_LAUNCH(128, 0, 0);
    else if (d->a_major == 0 && d->b_major == 1) KMOE_LAUNCH(128, 0, 1);
    else if (d->a_major == 1 && d->b_major == 0) KMOE_LAUNCH(128, 1, 0);
    else KMOE_LAUNCH(128, 1, 1);
  }
#undef KMOE_LAUNCH
#undef KMOE_LAUNCH_PAIR
  if (lrc) return lrc;
  if (d->sym_upper && !pair) {
    // the tiles below the diagonal were skipped: mirror them from the computed upper part (the CTA-pair
    // kernel writes the transposed tiles from its epilogue instead)
    dim3 mg((unsigned)(d->N / 32), (unsigned)(d->N / 32), (unsigned)groups);
    sym_mirror_kernel<<<mg, dim3(32, 8), 0, stream>>>((__nv_bfloat16*)d->C, d->N, d->ldc, d->c_gstride, BN, TM);
    if (cudaGetLastError() != cudaSuccess) return -22;
  }
  return 0;
}
