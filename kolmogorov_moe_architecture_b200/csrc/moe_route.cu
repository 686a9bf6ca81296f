// Token-choice MoE bookkeeping without host synchronisation.
//
// Layout ("padded expert-major"): the assignments of expert e occupy rows
// [off[e], off[e] + cnt[e]) of a [max_rows, d] buffer, with off[e] a multiple of 128,
// so a 128-row GEMM tile never spans two experts; rows between cnt[e] and the next
// multiple of 128 are zero.  Within an expert, rows keep (token, slot) order - the
// sort is stable, so results are deterministic.  max_rows = T*k + E*127 rounded up
// is a static bound, which keeps every buffer shape fixed across steps.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int PLAN_THREADS = 256;
constexpr int ROW_TILE = 128;

// Single-block stable counting sort of n = T*k assignments over E experts.
//   idx      [n] int64 expert of each assignment (flat (token, slot) order)
//   keep     [n] bool/uint8 or null: 0 = dropped assignment
//   pos      [n] int32  row of the assignment in the padded layout, -1 if dropped
//   row_src  [max_rows] int32 flat assignment index feeding each row, -1 for padding
//   counts   [E] int32 ; offsets [E+1] int32 (padded) ; tile_group [max_rows/128] ; meta[0] = live m-tiles,
//   meta[1] = live padded rows
__global__ void __launch_bounds__(PLAN_THREADS)
moe_plan_kernel(const long long* __restrict__ idx, const unsigned char* __restrict__ keep, int n, int E, int max_rows,
                int expert_base, int stage_ids, int* __restrict__ pos, int* __restrict__ row_src,
                int* __restrict__ counts, int* __restrict__ offsets, int* __restrict__ tile_group,
                int* __restrict__ meta) {
  // hist[PLAN_THREADS][ES] (ES = E rounded up to an odd number: threads of a warp hit different banks), then
  // wtot[PLAN_THREADS / 32][E], off[E + 1], and, when they fit, the n local expert ids as 16-bit values
  extern __shared__ int sh[];
  const int ES = E | 1;
  int* hist = sh;
  int* wtot = hist + PLAN_THREADS * ES;
  int* off = wtot + (PLAN_THREADS / 32) * E;
  unsigned short* eid = reinterpret_cast<unsigned short*>(off + E + 1);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int seg = (n + PLAN_THREADS - 1) / PLAN_THREADS;
  const int lo = min(tid * seg, n), hi = min(lo + seg, n);
  auto local_expert = [&](int i) -> int {             // 0xffff: not routed to an expert of this plan
    const int e = (int)idx[i] - expert_base;
    return (e >= 0 && e < E && (keep == nullptr || keep[i])) ? e : 0xffff;
  };
  for (int e = 0; e < E; ++e) hist[tid * ES + e] = 0;
  for (int i = tid; i < max_rows; i += PLAN_THREADS) row_src[i] = -1;
  if (stage_ids) {
    // coalesced read of the ids; the two passes below then walk each thread's contiguous segment in shared memory
    for (int i = tid; i < n; i += PLAN_THREADS) eid[i] = (unsigned short)local_expert(i);
    __syncthreads();
  }
  for (int i = lo; i < hi; ++i) {
    const int e = stage_ids ? (int)eid[i] : local_expert(i);
    if (e != 0xffff) hist[tid * ES + e]++;
  }
  __syncthreads();
  // exclusive scan over the threads, per expert: shuffles inside a warp, then the warp totals
  for (int e = 0; e < E; ++e) {
    const int v = hist[tid * ES + e];
    int inc = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, inc, o);
      if (lane >= o) inc += t;
    }
    hist[tid * ES + e] = inc - v;
    if (lane == 31) wtot[warp * E + e] = inc;
  }
  __syncthreads();
  for (int e = tid; e < E; e += PLAN_THREADS) {
    int run = 0;
    for (int w = 0; w < PLAN_THREADS / 32; ++w) {
      const int v = wtot[w * E + e];
      wtot[w * E + e] = run;
      run += v;
    }
    counts[e] = run;
    off[e] = run;  // temporarily the count
  }
  __syncthreads();
  if (tid == 0) {
    int run = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      const int cnt = off[e];
      off[e] = run;
      offsets[e] = run;
      const int nt = (cnt + ROW_TILE - 1) / ROW_TILE;
      for (int j = 0; j < nt; ++j) tile_group[tiles + j] = e;
      tiles += nt;
      run += nt * ROW_TILE;
    }
    off[E] = run;
    offsets[E] = run;
    meta[0] = tiles;
    meta[1] = run;
    for (int j = tiles; j < max_rows / ROW_TILE; ++j) tile_group[j] = 0;
  }
  __syncthreads();
  for (int i = lo; i < hi; ++i) {
    const int e = stage_ids ? (int)eid[i] : local_expert(i);
    int p = -1;
    if (e != 0xffff) {
      p = off[e] + wtot[warp * E + e] + hist[tid * ES + e]++;
      if (p < max_rows) row_src[p] = i; else p = -1;
    }
    pos[i] = p;
  }
}

// Capacity with drops for token choice: keep[i] = 1 iff assignment i is among the first `cap` assignments of its
// expert in flat (token, slot) order.  Same single-block stable ranking as the plan kernel.
__global__ void __launch_bounds__(PLAN_THREADS)
moe_capacity_mask_kernel(const long long* __restrict__ idx, int n, int E, int cap, unsigned char* __restrict__ keep) {
  extern __shared__ int sh[];     // hist[PLAN_THREADS][E]
  int* hist = sh;
  const int tid = threadIdx.x;
  const int seg = (n + PLAN_THREADS - 1) / PLAN_THREADS;
  const int lo = min(tid * seg, n), hi = min(lo + seg, n);
  for (int e = 0; e < E; ++e) hist[tid * E + e] = 0;
  for (int i = lo; i < hi; ++i) {
    const int e = (int)idx[i];
    if (e >= 0 && e < E) hist[tid * E + e]++;
  }
  __syncthreads();
  for (int e = tid; e < E; e += PLAN_THREADS) {
    int run = 0;
    for (int t = 0; t < PLAN_THREADS; ++t) {
      const int v = hist[t * E + e];
      hist[t * E + e] = run;
      run += v;
    }
  }
  __syncthreads();
  for (int i = lo; i < hi; ++i) {
    const int e = (int)idx[i];
    keep[i] = (e >= 0 && e < E && hist[tid * E + e]++ < cap) ? 1 : 0;
  }
}

// One slot of the balanced token-choice assignment: every token takes its most probable expert among those it
// has not used and that were not full (count >= cap) when the slot began; a token whose unused experts are all
// full takes its most probable unused expert regardless.  One warp per token; ties go to the lower index.
//   taken [T, E] uint8 (in/out), counts_in [E] (read), counts_out [E] (incremented), sel [T] int64
__global__ void moe_balanced_slot_kernel(const float* __restrict__ probs, unsigned char* __restrict__ taken,
                                         const int* __restrict__ counts_in, int* __restrict__ counts_out,
                                         long long* __restrict__ sel, long long sel_stride, int T, int E, int cap) {
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    float best = -INFINITY, fb = -INFINITY;
    int bi = E, fi = E;
    for (int e = lane; e < E; e += 32) {
      if (taken[(size_t)t * E + e]) continue;
      const float p = probs[(size_t)t * E + e];
      if (p > fb) { fb = p; fi = e; }
      if (counts_in[e] < cap && p > best) { best = p; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o), of = __shfl_xor_sync(0xffffffffu, fb, o);
      const int obi = __shfl_xor_sync(0xffffffffu, bi, o), ofi = __shfl_xor_sync(0xffffffffu, fi, o);
      if (ob > best || (ob == best && obi < bi)) { best = ob; bi = obi; }
      if (of > fb || (of == fb && ofi < fi)) { fb = of; fi = ofi; }
    }
    const int pick = bi < E ? bi : (fi < E ? fi : 0);
    if (lane == 0) {
      sel[(size_t)t * sel_stride] = pick;
      taken[(size_t)t * E + pick] = 1;
      atomicAdd(&counts_out[pick], 1);
    }
  }
}

// dst[row] = scale(row) * src[row_src[row] / div]  (zero for padding rows), rows < meta[1].
//   row_scale: optional fp32 per *assignment* multiplier (indexed by row_src), used by the
//   backward of the combine: dY[row] = w[assignment] * dout[token].
__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ row_src,
                                       const float* __restrict__ assign_scale, const int* __restrict__ meta,
                                       __nv_bfloat16* __restrict__ dst, int max_rows, int d, int div) {
  const int live_rows = min(meta[1], max_rows);
  const int vec = d / 8;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < live_rows; row += warps) {
    const int a = row_src[row];
    uint4* drow = reinterpret_cast<uint4*>(dst + (size_t)row * d);
    if (a < 0) {
      for (int v = lane; v < vec; v += 32) drow[v] = make_uint4(0, 0, 0, 0);
      continue;
    }
    const uint4* srow = reinterpret_cast<const uint4*>(src + (size_t)(a / div) * d);
    if (assign_scale == nullptr) {
      for (int v = lane; v < vec; v += 32) drow[v] = srow[v];
    } else {
      const float s = assign_scale[a];
      for (int v = lane; v < vec; v += 32) {
        uint4 r = srow[v];
        __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(p[i]);
          p[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
        }
        drow[v] = r;
      }
    }
  }
}

// out[t] = sum_k w[t,k] * Y[pos[t,k]]   (pos < 0 skipped; w null = 1).  One warp per token.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ Y, const int* __restrict__ pos,
                                   const float* __restrict__ w, __nv_bfloat16* __restrict__ out, int T, int k, int d) {
  const int vec = d / 8;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; t < T; t += warps) {
    for (int v = lane; v < vec; v += 32) {
      float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      for (int j = 0; j < k; ++j) {
        const int p = pos[t * k + j];
        if (p < 0) continue;
        const float s = w ? w[t * k + j] : 1.f;
        uint4 r = *reinterpret_cast<const uint4*>(Y + (size_t)p * d + v * 8);
        const __nv_bfloat162* q = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f = __bfloat1622float2(q[i]);
          acc[2 * i] += s * f.x;
          acc[2 * i + 1] += s * f.y;
        }
      }
      uint4 o;
      o.x = pack_bf16(acc[0], acc[1]);
      o.y = pack_bf16(acc[2], acc[3]);
      o.z = pack_bf16(acc[4], acc[5]);
      o.w = pack_bf16(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(out + (size_t)t * d + v * 8) = o;
    }
  }
}

// dw[t,k] = <dout[t], Y[pos[t,k]]>.  One warp per assignment.
__global__ void moe_combine_dw_kernel(const __nv_bfloat16* __restrict__ Y, const __nv_bfloat16* __restrict__ dout,
                                      const int* __restrict__ pos, float* __restrict__ dw, int n, int k, int d) {
  const int vec = d / 8;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  for (int a = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; a < n; a += warps) {
    const int p = pos[a];
    float s = 0.f;
    if (p >= 0) {
      const uint4* yr = reinterpret_cast<const uint4*>(Y + (size_t)p * d);
      const uint4* gr = reinterpret_cast<const uint4*>(dout + (size_t)(a / k) * d);
      for (int v = lane; v < vec; v += 32) {
        uint4 r1 = yr[v], r2 = gr[v];
        const __nv_bfloat162* q1 = reinterpret_cast<const __nv_bfloat162*>(&r1);
        const __nv_bfloat162* q2 = reinterpret_cast<const __nv_bfloat162*>(&r2);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          float2 f1 = __bfloat1622float2(q1[i]), f2 = __bfloat1622float2(q2[i]);
          s += f1.x * f2.x + f1.y * f2.y;
        }
      }
    }
    s = warp_sum(s);
    if (lane == 0) dw[a] = s;
  }
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_moe_max_rows(int n_assign, int E) {
  const int r = n_assign + E * (ROW_TILE - 1);
  return (r + ROW_TILE - 1) / ROW_TILE * ROW_TILE;
}

extern "C" int kmoe_moe_plan(const long long* idx, const unsigned char* keep, int n, int E, int max_rows,
                             int expert_base, int* pos, int* row_src, int* counts, int* offsets, int* tile_group,
                             int* meta, cudaStream_t st) {
  const size_t base = ((size_t)PLAN_THREADS * (E | 1) + (size_t)(PLAN_THREADS / 32) * E + E + 1) * sizeof(int);
  if (base > 200 * 1024 || E >= 0xffff) return -1;
  // the expert ids are staged in shared memory when they fit beside the histograms
  const int stage_ids = base + (size_t)n * 2 <= 200 * 1024 ? 1 : 0;
  const size_t smem = base + (stage_ids ? (size_t)n * 2 : 0);
  static size_t attr_set = 0;
  if (smem > 48 * 1024 && smem > attr_set) {
    if (cudaFuncSetAttribute(moe_plan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return -3;
    attr_set = smem;
  }
  moe_plan_kernel<<<1, PLAN_THREADS, smem, st>>>(idx, keep, n, E, max_rows, expert_base, stage_ids, pos, row_src,
                                                 counts, offsets, tile_group, meta);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_moe_capacity_mask(const long long* idx, int n, int E, int cap, unsigned char* keep,
                                      cudaStream_t st) {
  const size_t smem = (size_t)PLAN_THREADS * E * sizeof(int);
  if (smem > 200 * 1024) return -1;
  static size_t attr_set = 0;
  if (smem > 48 * 1024 && smem > attr_set) {
    if (cudaFuncSetAttribute(moe_capacity_mask_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return -3;
    attr_set = smem;
  }
  moe_capacity_mask_kernel<<<1, PLAN_THREADS, smem, st>>>(idx, n, E, cap, keep);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// `counts` holds k + 1 rows of E ints, zeroed by the caller: row j = expert loads at the start of slot j.
extern "C" int kmoe_moe_balanced_assign(const float* probs, unsigned char* taken, int* counts, long long* sel, int T,
                                        int E, int k, int cap, cudaStream_t st) {
  for (int j = 0; j < k; ++j) {
    if (j > 0) cudaMemcpyAsync(counts + (size_t)(j + 1) * E, counts + (size_t)j * E, E * sizeof(int),
                               cudaMemcpyDeviceToDevice, st);
    // slot j reads row j and accumulates the loads after the slot into row j + 1 (which starts as a copy of row j)
    moe_balanced_slot_kernel<<<148 * 4, 256, 0, st>>>(probs, taken, counts + (size_t)j * E,
                                                      counts + (size_t)(j + 1) * E, sel + j, k, T, E, cap);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_moe_gather_rows(const void* src, const int* row_src, const float* assign_scale, const int* meta,
                                    void* dst, int max_rows, int d, int div, cudaStream_t st) {
  if (d % 8) return -1;
  moe_gather_rows_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)src, row_src, assign_scale, meta,
                                                  (__nv_bfloat16*)dst, max_rows, d, div);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_moe_combine(const void* Y, const int* pos, const float* w, void* out, int T, int k, int d,
                                cudaStream_t st) {
  if (d % 8) return -1;
  moe_combine_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)Y, pos, w, (__nv_bfloat16*)out, T, k, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_moe_combine_dw(const void* Y, const void* dout, const int* pos, float* dw, int n, int k, int d,
                                   cudaStream_t st) {
  if (d % 8) return -1;
  moe_combine_dw_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)Y, (const __nv_bfloat16*)dout, pos, dw, n, k,
                                                 d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
