// Block-scaled MXFP8 GEMM for sm_100a:  C (M, N) = A (M, K) * B (N, K)^T, both operands e4m3 with the
// reduction dimension contiguous, one e8m0 scale per 32 reduction elements, fp32 accumulation in TMEM.
//
//   warp 0     : producer - TMA tiles of A and B (128-byte swizzle, 128 x 128 e4m3 per operand and stage)
//                plus one 512-byte bulk copy per operand for the stage's scale factors
//   warp 1     : tcgen05.cp of the scale chunks shared -> tensor memory, then four
//                tcgen05.mma.kind::mxf8f6f4.block_scale (128 x 128 x 32) per stage; the k-th MMA of a stage
//                selects byte k of the scale columns through the instruction descriptor
//   warps 2..5 : epilogue, tcgen05.ld -> alpha * acc + beta * D -> bf16 / fp32
//
// Tensor memory: two 128-column accumulators (epilogue of tile i overlaps the main loop of tile i+1),
// then 4 columns of A scales and 4 columns of B scales.  The scale columns are rewritten every stage;
// tcgen05.cp and tcgen05.mma issued by one thread execute in order, so no extra barrier is needed.
// Tile schedules match the bf16 kernel: dense, grouped along M (expert-major padded rows, tile -> expert
// table on the device) and batched with an optional ragged reduction range per group (expert wgrad).
// Every wait is bounded; on expiry the kernel records a status code, frees its TMEM and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <tuple>

#include "kmoe_api.h"
#include "ptx.cuh"
#include "tmap_host.h"

namespace kmoe {
namespace mx {

constexpr int BM = 128, BN = 128, BK = 128;          // BK e4m3 elements = one 128-byte swizzled row
constexpr int TILE_BYTES = BM * BK;                  // 16 KB per operand
constexpr int SF_BYTES = 512;                        // 128 rows x 4 scale groups
constexpr int STAGE_BYTES = 2 * TILE_BYTES + 2 * SF_BYTES;
constexpr int STAGES = 6;
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;                  // 2 x 128 accumulators + 8 scale columns, power of two
constexpr uint32_t SFA_COL = 2 * BN;
constexpr uint32_t SFB_COL = 2 * BN + 4;

struct Args {
  void* C;
  const void* D;
  const uint8_t* sfa;
  const uint8_t* sfb;
  int mode;
  int M, N, K, groups;
  long long ldc, ldd, c_gstride;
  long long sfa_gchunks, sfb_gchunks;               // scale chunks per group (0 = operand shared by all groups)
  int k_chunks_total;                               // K / 128 of the underlying buffers
  int a_grouped, b_grouped;
  const int* tile_group;
  const int* num_m_tiles;
  const int* k_begin;
  const int* k_len;
  int out_f32;
  float alpha, beta;
  int* status;
};

struct Tile {
  int m_tile, n_tile, g_a, g_b, g_c, k0, k_blocks;
};

__device__ __forceinline__ int cdiv(int a, int b) { return (a + b - 1) / b; }

__device__ __forceinline__ bool get_tile(const Args& a, int idx, int num_m, int num_n, Tile& t) {
  const int per_group = num_m * num_n;
  int g = 0, local = idx;
  if (a.mode == KMOE_GEMM_BATCHED) {
    g = idx / per_group;
    local = idx - g * per_group;
    if (g >= a.groups) return false;
  } else if (idx >= per_group) {
    return false;
  }
  const int GM = 8;                                  // bands of 8 m-tiles share B tiles in L2
  const int band = local / (GM * num_n);
  const int first_m = band * GM;
  const int gsz = min(num_m - first_m, GM);
  const int r = local - band * GM * num_n;
  t.m_tile = first_m + r % gsz;
  t.n_tile = r / gsz;
  t.k0 = 0;
  t.k_blocks = a.K / BK;
  t.g_a = t.g_b = t.g_c = 0;
  if (a.mode == KMOE_GEMM_GROUPED_M) {
    t.g_b = a.tile_group[t.m_tile];
  } else if (a.mode == KMOE_GEMM_BATCHED) {
    t.g_a = a.a_grouped ? g : 0;
    t.g_b = a.b_grouped ? g : 0;
    t.g_c = g;
    if (a.k_begin != nullptr) {
      t.k0 = a.k_begin[g];
      t.k_blocks = cdiv(a.k_len[g], BK);
    }
  }
  return true;
}

// descriptor for the scale chunk in shared memory: no swizzle, 8-row x 16-byte core matrices 128 bytes apart
__device__ __forceinline__ uint64_t make_sf_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(128 >> 4) << 32;                  // stride between 8-row groups
  d |= (uint64_t)1 << 46;                           // descriptor version for sm_100
  return d;
}

// block-scaled instruction descriptor: e4m3 x e4m3, e8m0 scales, K-major operands, M x N tile
__device__ __forceinline__ uint32_t make_idesc_mx(int M, int N, int sf_id) {
  return ((uint32_t)sf_id << 4) |                   // byte of the B scale columns used by this MMA
         (0u << 7) | (0u << 10) |                   // A, B formats: e4m3
         ((uint32_t)(N >> 3) << 17) | (1u << 23) |  // N, scale format e8m0
         ((uint32_t)(M >> 4) << 24) | ((uint32_t)sf_id << 29);   // M, byte of the A scale columns
}

__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar))
               : "memory");
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
mxfp8_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  __shared__ uint64_t full_bar[STAGES];
  __shared__ uint64_t empty_bar[STAGES];
  __shared__ uint64_t tmem_full[2];
  __shared__ uint64_t tmem_empty[2];
  __shared__ uint32_t tmem_base_slot;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full[i], 1);
      mbar_init(&tmem_empty[i], 4);
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

  int num_m = cdiv(args.M, BM);
  if (args.mode == KMOE_GEMM_GROUPED_M) num_m = min(num_m, *args.num_m_tiles);
  const int num_n = cdiv(args.N, BN);
  // stage layout: [A tile][B tile][A scales][B scales]; the tiles stay 1024-byte aligned
  if (warp == 0) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      Tile t;
      for (int idx = blockIdx.x; get_tile(args, idx, num_m, num_n, t); idx += gridDim.x) {
        for (int kb = 0; kb < t.k_blocks; ++kb) {
          if (!mbar_wait(&empty_bar[s], ph ^ 1)) {
            atomicExch(args.status, 11);
            goto teardown;
          }
          uint8_t* sa = smem + s * STAGE_BYTES;
          uint8_t* sb = sa + TILE_BYTES;
          uint8_t* ssa = sb + TILE_BYTES;
          uint8_t* ssb = ssa + SF_BYTES;
          mbar_expect_tx(&full_bar[s], STAGE_BYTES);
          const int k = t.k0 + kb * BK;
          tma_load_4d(sa, &tmA, &full_bar[s], k, t.m_tile * BM, 0, t.g_a);
          tma_load_4d(sb, &tmB, &full_bar[s], k, t.n_tile * BN, 0, t.g_b);
          const long long kc = k / BK;
          bulk_load(ssa, args.sfa + ((long long)t.g_a * args.sfa_gchunks + (long long)t.m_tile * args.k_chunks_total + kc) * SF_BYTES,
                    SF_BYTES, &full_bar[s]);
          bulk_load(ssb, args.sfb + ((long long)t.g_b * args.sfb_gchunks + (long long)t.n_tile * args.k_chunks_total + kc) * SF_BYTES,
                    SF_BYTES, &full_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      Tile t;
      for (int idx = blockIdx.x; get_tile(args, idx, num_m, num_n, t); idx += gridDim.x, ++it) {
        const int acc = it & 1;
        const uint32_t acc_ph = (it >> 1) & 1;
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
          const uint32_t sb = sa + TILE_BYTES;
          tcgen05_cp_32x128b_warpx4(tmem_base + SFA_COL, make_sf_desc(sb + TILE_BYTES));
          tcgen05_cp_32x128b_warpx4(tmem_base + SFB_COL, make_sf_desc(sb + TILE_BYTES + SF_BYTES));
#pragma unroll
          for (int k4 = 0; k4 < BK / 32; ++k4) {
            const uint64_t adesc = make_smem_desc_sw128(sa + k4 * 32, 16, 1024);
            const uint64_t bdesc = make_smem_desc_sw128(sb + k4 * 32, 16, 1024);
            umma_mxf8(d_tmem, adesc, bdesc, make_idesc_mx(BM, BN, k4), tmem_base + SFA_COL, tmem_base + SFB_COL,
                      (kb > 0 || k4 > 0) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);
          if (++s == STAGES) { s = 0; ph ^= 1; }
        }
        if (t.k_blocks > 0)
          umma_commit(&tmem_full[acc]);
        else
          mbar_arrive(&tmem_full[acc]);
      }
    }
  } else {
    const int q = warp & 3;
    int it = 0;
    Tile t;
    for (int idx = blockIdx.x; get_tile(args, idx, num_m, num_n, t); idx += gridDim.x, ++it) {
      const int acc = it & 1;
      const uint32_t acc_ph = (it >> 1) & 1;
      if (!mbar_wait(&tmem_full[acc], acc_ph)) {
        if (lane == 0) atomicExch(args.status, 14);
        goto teardown;
      }
      tc_fence_after();
      const bool have_acc = t.k_blocks > 0;
      const int row = t.m_tile * BM + q * 32 + lane;
      const bool row_ok = row < args.M;
      const long long coff = (long long)t.g_c * args.c_gstride + (long long)row * args.ldc;
      const long long doff = (long long)t.g_c * args.c_gstride + (long long)row * args.ldd;
      const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = 0; c < BN; c += 32) {
        uint32_t r[32];
        if (have_acc) {
          tmem_ld_32x32(t_row + c, r);
          tmem_ld_wait();
        }
        const int col0 = t.n_tile * BN + c;
        if (row_ok && col0 < args.N) {
#pragma unroll
          for (int j = 0; j < 32; j += 8) {
            if (col0 + j >= args.N) break;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = have_acc ? __uint_as_float(r[j + i]) * args.alpha : 0.f;
            if (args.out_f32) {
              float* Cp = reinterpret_cast<float*>(args.C) + coff + col0 + j;
              if (args.D != nullptr) {
                const float* Dp = reinterpret_cast<const float*>(args.D) + doff + col0 + j;
#pragma unroll
                for (int i = 0; i < 8; ++i) v[i] += args.beta * Dp[i];
              }
              *reinterpret_cast<float4*>(Cp) = make_float4(v[0], v[1], v[2], v[3]);
              *reinterpret_cast<float4*>(Cp + 4) = make_float4(v[4], v[5], v[6], v[7]);
            } else {
              __nv_bfloat16* Cp = reinterpret_cast<__nv_bfloat16*>(args.C) + coff + col0 + j;
              if (args.D != nullptr) {
                const uint4 dr = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(args.D) +
                                                                  doff + col0 + j);
                const __nv_bfloat162* dp = reinterpret_cast<const __nv_bfloat162*>(&dr);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float2 f = __bfloat1622float2(dp[i]);
                  v[2 * i] += args.beta * f.x;
                  v[2 * i + 1] += args.beta * f.y;
                }
              }
              uint4 o;
              o.x = pack_bf16(v[0], v[1]); o.y = pack_bf16(v[2], v[3]);
              o.z = pack_bf16(v[4], v[5]); o.w = pack_bf16(v[6], v[7]);
              *reinterpret_cast<uint4*>(Cp) = o;
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

// e4m3 operand map: dims {K, rows, 1, G}, box {128, 128, 1, 1}, 128-byte swizzle
static std::map<std::tuple<const void*, long long, long long, long long, int>, CUtensorMap> g_cache;
static std::mutex g_mutex;

static int make_tmap(CUtensorMap* out, const void* base, long long rows, long long K, long long gstride, int groups) {
  auto key = std::make_tuple(base, rows, K, gstride, groups);
  {
    std::lock_guard<std::mutex> lk(g_mutex);
    auto it = g_cache.find(key);
    if (it != g_cache.end()) { *out = it->second; return 0; }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return -10;
  if (K % 16 != 0 || (reinterpret_cast<uintptr_t>(base) & 15) != 0) return -12;
  const int G = (groups > 1 && gstride > 0) ? groups : 1;
  const long long gs = G > 1 ? gstride : rows * K;
  if (gs % 16 != 0) return -12;
  cuuint64_t dims[4] = {(cuuint64_t)K, (cuuint64_t)rows, 1, (cuuint64_t)G};
  cuuint64_t strides[3] = {(cuuint64_t)K, (cuuint64_t)(rows * K), (cuuint64_t)gs};
  cuuint32_t box[4] = {BK, BM, 1, 1};
  cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return -14;
  std::lock_guard<std::mutex> lk(g_mutex);
  if (g_cache.size() > 4096) g_cache.clear();
  g_cache[key] = *out;
  return 0;
}

}  // namespace mx
}  // namespace kmoe

extern "C" void kmoe_mxfp8_clear_tensormap_cache(void) {
  std::lock_guard<std::mutex> lk(kmoe::mx::g_mutex);
  kmoe::mx::g_cache.clear();
}

extern "C" int kmoe_gemm_mxfp8(const KmoeMxGemmDesc* d, cudaStream_t stream) {
  using namespace kmoe;
  using namespace kmoe::mx;
  if (d->K % BK != 0 || d->N % 8 != 0 || d->K <= 0 || d->M <= 0 || d->N <= 0) return -1;
  if (d->mode == KMOE_GEMM_GROUPED_M && d->M % BM != 0) return -2;
  Args a;
  a.C = d->C; a.D = d->D; a.sfa = (const uint8_t*)d->sfa; a.sfb = (const uint8_t*)d->sfb;
  a.mode = d->mode; a.M = d->M; a.N = d->N; a.K = d->K; a.groups = d->groups;
  a.ldc = d->ldc; a.ldd = d->ldd ? d->ldd : d->ldc; a.c_gstride = d->c_gstride;
  a.k_chunks_total = d->K / BK;
  const bool a_grp = d->mode == KMOE_GEMM_BATCHED && d->a_grouped;
  const bool b_grp = d->b_grouped != 0;
  a.a_grouped = a_grp; a.b_grouped = b_grp;
  const long long m_blocks = (d->M + BM - 1) / BM, n_blocks = (d->N + BN - 1) / BN;
  // grouped operands: every group has its own (rows x K) block and its own run of scale chunks
  a.sfa_gchunks = a_grp ? m_blocks * a.k_chunks_total : 0;
  a.sfb_gchunks = b_grp ? n_blocks * a.k_chunks_total : 0;
  if (b_grp && d->N % BN != 0) return -3;            // scale chunks of neighbouring groups must not share a block
  if (a_grp && d->M % BM != 0) return -3;
  a.tile_group = d->tile_group; a.num_m_tiles = d->num_m_tiles;
  a.k_begin = d->k_begin; a.k_len = d->k_len;
  a.out_f32 = d->out_f32; a.alpha = d->alpha; a.beta = d->beta; a.status = d->status;

  CUtensorMap tA, tB;
  int rc = make_tmap(&tA, d->A, d->M, d->K, a_grp ? (long long)d->M * d->K : 0, a_grp ? d->groups : 1);
  if (rc) return rc;
  rc = make_tmap(&tB, d->B, d->N, d->K, b_grp ? (long long)d->N * d->K : 0, b_grp ? d->groups : 1);
  if (rc) return rc;
  int sms = d->num_sms;
  if (sms <= 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  const long long groups = d->mode == KMOE_GEMM_BATCHED ? d->groups : 1;
  const long long total = m_blocks * n_blocks * groups;
  int grid = (int)(total < sms ? total : sms);
  if (grid < 1) grid = 1;
  const int smem = STAGES * STAGE_BYTES + 1024;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(mxfp8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -20;
    attr_set = true;
  }
  mxfp8_gemm_kernel<<<grid, NUM_THREADS, smem, stream>>>(tA, tB, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -21;
}
