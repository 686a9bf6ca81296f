// Collectives fused with compute, over NVLink peer pointers (symmetric memory): every rank
// maps every peer's buffers, and these kernels load from / store to the peers directly.
// No TMA multicast is used anywhere; loads are plain 16-byte peer loads.
//
//   barrier            flag exchange with release/acquire at system scope; the wait is bounded
//                      by a wall-clock limit and reports expiry through a status word.
//   reduce_scatter     own segment <- mean over ranks of the same segment of every rank's
//                      gradient buffer, fused with the squared-norm reduction needed for
//                      global-norm clipping.
//   adamw_allgather    AdamW on the owned range (clip coefficient read from device memory,
//                      fp32 moments) whose result is stored into every rank's parameter
//                      buffer - the update and the all-gather are one kernel.
//   allgather          copy of an owned range into every rank's buffer (used after Muon).
// Each of the three takes an optional NVLink-switch multicast address of the same buffer: the reduction
// then happens inside the switch (multimem.ld_reduce, one load instead of `world`) and the publication is
// one multimem.st instead of `world` stores, which cuts the bytes through each GPU's port by ~world.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int MAX_RANKS = 16;
struct PeerPtrs {
  void* p[MAX_RANKS];
};

__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

// NVLink-switch (NVLS) multicast: one address that stands for the same offset in every rank's buffer.
// ld_reduce returns the sum over all ranks, formed in the switch with fp32 accumulation; st writes to all ranks.
__device__ __forceinline__ uint4 multimem_ld_reduce_bf16x8(const void* mc_addr) {
  uint4 r;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(mc_addr)
               : "memory");
  return r;
}
__device__ __forceinline__ void multimem_st_16B(void* mc_addr, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc_addr), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// flags[r] on every rank is written by rank r.  One CTA; thread r handles peer r.
__global__ void p2p_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, unsigned long long timeout_ns,
                                   int* status) {
  const int r = threadIdx.x;
  if (r < world) {
    __threadfence_system();
    int* dst = reinterpret_cast<int*>(flags.p[r]) + rank;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(dst), "r"(epoch) : "memory");
    const int* src = reinterpret_cast<const int*>(flags.p[rank]) + r;
    const unsigned long long t0 = globaltimer_ns();
    int v;
    while (true) {
      asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(src) : "memory");
      if (v >= epoch) break;
      if (globaltimer_ns() - t0 > timeout_ns) {
        atomicExch(status, 100 + r);
        break;
      }
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void acc8(const uint4& r, float* a) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    a[2 * i] += f.x;
    a[2 * i + 1] += f.y;
  }
}

// out[i] = (1/world) * sum_r grads[r][off + i], i in [0, n); sq_out += sum out^2 (fp32 atomics per CTA)
// mc != null: the sum comes from one multicast load per 16 bytes instead of `world` peer loads.
// Each thread keeps RS_UNROLL independent 16-byte loads in flight (per peer), so that a small grid running
// beside the backward pass still covers the NVLink latency.
constexpr int RS_UNROLL = 4;
__global__ void p2p_reduce_scatter_kernel(PeerPtrs grads, int rank, int world, long long off, long long n,
                                          float* __restrict__ sq_out, const void* mc) {
  const long long nvec = n / 8;
  const float inv = 1.f / world;
  float sq = 0.f;
  __nv_bfloat16* own = reinterpret_cast<__nv_bfloat16*>(grads.p[rank]) + off;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; v0 < nvec; v0 += stride * RS_UNROLL) {
    float a[RS_UNROLL][8];
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) a[u][i] = 0.f;
    if (mc != nullptr) {
      uint4 x[RS_UNROLL];
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
        if (v0 + u * stride < nvec)
          x[u] = multimem_ld_reduce_bf16x8(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(mc) + off) +
                                           v0 + u * stride);
#pragma unroll
      for (int u = 0; u < RS_UNROLL; ++u)
        if (v0 + u * stride < nvec) acc8(x[u], a[u]);
    } else {
      for (int r = 0; r < world; ++r) {
        const int src = (rank + r) % world;     // stagger peers so ranks do not all hit the same one
        const uint4* sp = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[src]) + off);
        uint4 x[RS_UNROLL];
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u)
          if (v0 + u * stride < nvec) x[u] = sp[v0 + u * stride];
#pragma unroll
        for (int u = 0; u < RS_UNROLL; ++u)
          if (v0 + u * stride < nvec) acc8(x[u], a[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < RS_UNROLL; ++u) {
      if (v0 + u * stride >= nvec) continue;
      uint4 o;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        a[u][i] *= inv;
        sq += a[u][i] * a[u][i];
      }
      o.x = pack_bf16(a[u][0], a[u][1]); o.y = pack_bf16(a[u][2], a[u][3]);
      o.z = pack_bf16(a[u][4], a[u][5]); o.w = pack_bf16(a[u][6], a[u][7]);
      *(reinterpret_cast<uint4*>(own) + v0 + u * stride) = o;
    }
  }
  sq = warp_sum(sq);
  __shared__ float s[32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0 && sq_out != nullptr) atomicAdd(sq_out, t);
  }
}

struct AdamArgs {
  float lr, beta1, beta2, eps, wd, bc1, bc2;   // bc = 1 - beta^t
  const float* clip_coef;                      // device scalar multiplying the gradient (null = 1)
};

// AdamW on [off, off+n) of the owner's gradient/parameter segment; new parameters go to every rank.
__global__ void p2p_adamw_allgather_kernel(PeerPtrs params, const __nv_bfloat16* __restrict__ grad, float* __restrict__ m,
                                           float* __restrict__ v2, int rank, int world, long long off, long long n,
                                           AdamArgs h, void* mc) {
  const long long nvec = n / 8;
  const float cc = h.clip_coef ? *h.clip_coef : 1.f;
  const __nv_bfloat16* own = reinterpret_cast<const __nv_bfloat16*>(params.p[rank]) + off;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 pr = *(reinterpret_cast<const uint4*>(own) + i);
    const uint4 gr = *(reinterpret_cast<const uint4*>(grad + off) + i);
    const __nv_bfloat162* pp = reinterpret_cast<const __nv_bfloat162*>(&pr);
    const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&gr);
    float pv[8], gv[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float2 a = __bfloat1622float2(pp[j]), b = __bfloat1622float2(gp[j]);
      pv[2 * j] = a.x; pv[2 * j + 1] = a.y; gv[2 * j] = b.x * cc; gv[2 * j + 1] = b.y * cc;
    }
    float4 m0 = *reinterpret_cast<float4*>(m + i * 8), m1 = *reinterpret_cast<float4*>(m + i * 8 + 4);
    float4 s0 = *reinterpret_cast<float4*>(v2 + i * 8), s1 = *reinterpret_cast<float4*>(v2 + i * 8 + 4);
    float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
    float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      mv[j] = h.beta1 * mv[j] + (1.f - h.beta1) * gv[j];
      sv[j] = h.beta2 * sv[j] + (1.f - h.beta2) * gv[j] * gv[j];
      const float denom = sqrtf(sv[j] / h.bc2) + h.eps;
      pv[j] = pv[j] * (1.f - h.lr * h.wd) - h.lr * (mv[j] / h.bc1) / denom;
    }
    *reinterpret_cast<float4*>(m + i * 8) = make_float4(mv[0], mv[1], mv[2], mv[3]);
    *reinterpret_cast<float4*>(m + i * 8 + 4) = make_float4(mv[4], mv[5], mv[6], mv[7]);
    *reinterpret_cast<float4*>(v2 + i * 8) = make_float4(sv[0], sv[1], sv[2], sv[3]);
    *reinterpret_cast<float4*>(v2 + i * 8 + 4) = make_float4(sv[4], sv[5], sv[6], sv[7]);
    uint4 o;
    o.x = pack_bf16(pv[0], pv[1]); o.y = pack_bf16(pv[2], pv[3]); o.z = pack_bf16(pv[4], pv[5]); o.w = pack_bf16(pv[6], pv[7]);
    if (mc != nullptr) {
      multimem_st_16B(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(mc) + off) + i, o);
    } else {
      for (int r = 0; r < world; ++r) {
        const int dst = (rank + r) % world;
        *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[dst]) + off) + i) = o;
      }
    }
  }
}

// Copy n elements into [off, off+n) of every rank's buffer.  src == null: the source is this rank's own
// buffer at the same offset (which is then left alone); otherwise `src` (e.g. a parameter shard) is also
// stored into this rank's buffer.  AG_UNROLL loads are in flight per thread, so a small grid that runs
// beside compute kernels still fills the link.
constexpr int AG_UNROLL = 4;
__global__ void p2p_allgather_kernel(PeerPtrs bufs, int rank, int world, long long off, long long n, void* mc,
                                     const __nv_bfloat16* __restrict__ src) {
  const long long nvec = n / 8;
  const uint4* from = src != nullptr
                          ? reinterpret_cast<const uint4*>(src)
                          : reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[rank]) + off);
  const int first = src != nullptr ? 0 : 1;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i0 = blockIdx.x * (long long)blockDim.x + threadIdx.x; i0 < nvec; i0 += stride * AG_UNROLL) {
    uint4 x[AG_UNROLL];
#pragma unroll
    for (int u = 0; u < AG_UNROLL; ++u)
      if (i0 + u * stride < nvec) x[u] = from[i0 + u * stride];
#pragma unroll
    for (int u = 0; u < AG_UNROLL; ++u) {
      const long long i = i0 + u * stride;
      if (i >= nvec) continue;
      if (mc != nullptr) {                    // one store reaches every rank (this one included)
        multimem_st_16B(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(mc) + off) + i, x[u]);
        continue;
      }
      for (int r = first; r < world; ++r) {
        const int dst = (rank + r) % world;
        *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[dst]) + off) + i) = x[u];
      }
    }
  }
}

static PeerPtrs make_ptrs(const long long* ptrs, int world) {
  PeerPtrs p;
  for (int i = 0; i < MAX_RANKS; ++i) p.p[i] = i < world ? reinterpret_cast<void*>(ptrs[i]) : nullptr;
  return p;
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_p2p_barrier(const long long* flag_ptrs, int rank, int world, int epoch, double timeout_s,
                                int* status, cudaStream_t st) {
  if (world > MAX_RANKS) return -1;
  p2p_barrier_kernel<<<1, 32, 0, st>>>(make_ptrs(flag_ptrs, world), rank, world, epoch,
                                       (unsigned long long)(timeout_s * 1e9), status);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_p2p_reduce_scatter(const long long* grad_ptrs, int rank, int world, long long off, long long n,
                                       float* sq_out, long long mc_ptr, int max_blocks, cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8) return -1;
  if (n == 0) return 0;
  const int blocks = max_blocks > 0 ? max_blocks : 148 * 8;
  p2p_reduce_scatter_kernel<<<blocks, 256, 0, st>>>(make_ptrs(grad_ptrs, world), rank, world, off, n, sq_out,
                                                     reinterpret_cast<const void*>(mc_ptr));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_p2p_adamw_allgather(const long long* param_ptrs, const void* grad, float* m, float* v, int rank,
                                        int world, long long off, long long n, float lr, float beta1, float beta2,
                                        float eps, float wd, int step, const float* clip_coef, long long mc_ptr,
                                        cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8) return -1;
  AdamArgs h{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), clip_coef};
  p2p_adamw_allgather_kernel<<<148 * 8, 256, 0, st>>>(make_ptrs(param_ptrs, world), (const __nv_bfloat16*)grad, m, v,
                                                      rank, world, off, n, h, reinterpret_cast<void*>(mc_ptr));
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_p2p_allgather(const long long* buf_ptrs, int rank, int world, long long off, long long n,
                                  long long mc_ptr, const void* src, int max_blocks, cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8 || (reinterpret_cast<uintptr_t>(src) & 15)) return -1;
  if (n == 0) return 0;
  const int blocks = max_blocks > 0 ? max_blocks : 148 * 8;
  p2p_allgather_kernel<<<blocks, 256, 0, st>>>(make_ptrs(buf_ptrs, world), rank, world, off, n,
                                               reinterpret_cast<void*>(mc_ptr), (const __nv_bfloat16*)src);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// =====================================================================================
// Expert-parallel token exchange over peer pointers.
//
// Source side: the local plan (moe_route.cu) lays the assignments of ALL experts out in a padded
// expert-major order; `ep_dispatch` reads each assignment's row straight from the token matrix
// (the permute) and stores it into the owning rank's receive buffer (the all-to-all) in one pass:
//     recv[dest][(e_local * world + src) * cap + j]   <-  x[token of the j-th assignment to expert e]
// together with the per-(expert, source) counts and the source's row offsets.  Expert side:
// `ep_recv_plan` turns the counts into a padded expert-major layout, `ep_compact` gathers the slots
// into it, the grouped GEMMs run on that, and `ep_return` stores every result row back into the
// source rank's buffer at the position its local plan expects, so the weighted top-k un-permute
// is the ordinary local combine.  No host synchronisation, no NCCL.
namespace kmoe {

// one warp per padded source row
__global__ void ep_dispatch_kernel(const __nv_bfloat16* __restrict__ src, const int* __restrict__ row_src,
                                   const float* __restrict__ assign_scale, const int* __restrict__ offsets,
                                   const int* __restrict__ counts, PeerPtrs recv, PeerPtrs recv_meta, int rank,
                                   int world, int E, int n_local, long long cap, int d, int div, int max_rows) {
  const int vec = d / 8;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  // publish counts and offsets: meta[dest][(e_local * world + rank) * 2 + {0,1}]
  for (int e = blockIdx.x * blockDim.x + threadIdx.x; e < E; e += gridDim.x * blockDim.x) {
    int* m = reinterpret_cast<int*>(recv_meta.p[e / n_local]) + ((e % n_local) * world + rank) * 2;
    m[0] = min(counts[e], (int)cap);      // rows beyond the slot capacity are dropped
    m[1] = offsets[e];
  }
  const int live_rows = min(offsets[E], max_rows);
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < live_rows; row += warps) {
    const int a = row_src[row];
    if (a < 0) continue;                       // padding rows are not sent
    int e = 0;                                 // expert whose segment holds this row (E is small)
    while (e + 1 < E && offsets[e + 1] <= row) ++e;
    const int j = row - offsets[e];
    if (j >= cap) continue;
    const int dest = e / n_local;
    __nv_bfloat16* drow = reinterpret_cast<__nv_bfloat16*>(recv.p[dest]) +
                          (((long long)(e % n_local) * world + rank) * cap + j) * d;
    const uint4* srow = reinterpret_cast<const uint4*>(src + (size_t)(div > 0 ? a / div : row) * d);
    const float s = assign_scale ? assign_scale[a] : 1.f;
    // four 16-byte loads in flight per lane before the (possibly remote) stores
    for (int v0 = lane; v0 < vec; v0 += 128) {
      uint4 r[4];
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + 32 * u < vec) r[u] = srow[v0 + 32 * u];
      if (assign_scale) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r[u]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            float2 f = __bfloat1622float2(p[i]);
            p[i] = __floats2bfloat162_rn(f.x * s, f.y * s);
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u)
        if (v0 + 32 * u < vec) reinterpret_cast<uint4*>(drow)[v0 + 32 * u] = r[u];
    }
  }
}

// Single block.  meta_in: [n_local * world][2] = (count, source offset).  Outputs:
//   slot_dst [n_local*world]   first row of each (expert, source) slot in the compacted layout
//   offsets  [n_local+1]       padded expert offsets ; tile_group ; out_meta = {live tiles, live rows}
__global__ void ep_recv_plan_kernel(const int* __restrict__ meta_in, int n_local, int world, int max_rows,
                                    int* __restrict__ slot_dst, int* __restrict__ offsets,
                                    int* __restrict__ tile_group, int* __restrict__ out_meta) {
  if (threadIdx.x != 0) return;
  int run = 0, tiles = 0;
  for (int e = 0; e < n_local; ++e) {
    offsets[e] = run;
    int cnt = 0;
    for (int s = 0; s < world; ++s) {
      slot_dst[e * world + s] = run + cnt;
      cnt += meta_in[(e * world + s) * 2];
    }
    const int nt = (cnt + 127) / 128;
    for (int j = 0; j < nt && tiles + j < max_rows / 128; ++j) tile_group[tiles + j] = e;
    tiles += nt;
    run += nt * 128;
  }
  offsets[n_local] = run;
  for (int j = tiles; j < max_rows / 128; ++j) tile_group[j] = 0;
  out_meta[0] = min(tiles, max_rows / 128);
  out_meta[1] = min(run, max_rows);
}

// dir = 0: compact  (slots of the local receive buffer -> expert-major padded rows, padding zeroed)
// dir = 1: return   (expert-major rows -> the source rank's buffer at its own padded position)
__global__ void ep_move_kernel(const __nv_bfloat16* __restrict__ slots, __nv_bfloat16* __restrict__ packed,
                               const int* __restrict__ meta_in, const int* __restrict__ slot_dst,
                               const int* __restrict__ offsets, PeerPtrs ret, int rank, int n_local, int world,
                               long long cap, int d, int max_rows, int dir, long long* __restrict__ row_ptr_out) {
  const int vec = d / 8;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int live_rows = min(offsets[n_local], max_rows);
  const int nslots = n_local * world;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < live_rows; row += warps) {
    // find the slot containing this packed row
    int sl = -1, j = 0;
    for (int q = 0; q < nslots; ++q) {
      const int b0 = slot_dst[q], c = meta_in[q * 2];
      if (row >= b0 && row < b0 + c) { sl = q; j = row - b0; break; }
    }
    uint4* prow = reinterpret_cast<uint4*>(packed + (size_t)row * d);
    if (dir == 0 && row_ptr_out != nullptr && lane == 0) {
      long long addr = 0;
      if (sl >= 0)
        addr = reinterpret_cast<long long>(reinterpret_cast<__nv_bfloat16*>(ret.p[sl % world]) +
                                           (size_t)(meta_in[sl * 2 + 1] + j) * d);
      row_ptr_out[row] = addr;
    }
    if (dir == 0) {
      if (sl < 0) {
        for (int v = lane; v < vec; v += 32) prow[v] = make_uint4(0, 0, 0, 0);
      } else {
        const uint4* srow = reinterpret_cast<const uint4*>(slots + ((long long)sl * cap + j) * d);
        for (int v0 = lane; v0 < vec; v0 += 128) {
          uint4 r[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + 32 * u < vec) r[u] = srow[v0 + 32 * u];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (v0 + 32 * u < vec) prow[v0 + 32 * u] = r[u];
        }
      }
    } else if (sl >= 0) {
      const int src_rank = sl % world;
      const int src_off = meta_in[sl * 2 + 1];
      uint4* drow = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(ret.p[src_rank]) +
                                             (size_t)(src_off + j) * d);
      for (int v = lane; v < vec; v += 32) drow[v] = prow[v];
    }
  }
}

}  // namespace kmoe

extern "C" int kmoe_ep_dispatch(const void* src, const int* row_src, const float* assign_scale, const int* offsets,
                                const int* counts, const long long* recv_ptrs, const long long* meta_ptrs, int rank,
                                int world, int E, long long cap, int d, int div, int max_rows, cudaStream_t st) {
  if (world > MAX_RANKS || d % 8 || E % world) return -1;
  ep_dispatch_kernel<<<148 * 8, 256, 0, st>>>((const __nv_bfloat16*)src, row_src, assign_scale, offsets, counts,
                                              make_ptrs(recv_ptrs, world), make_ptrs(meta_ptrs, world), rank, world, E,
                                              E / world, cap, d, div, max_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_ep_recv_plan(const int* meta_in, int n_local, int world, int max_rows, int* slot_dst,
                                 int* offsets, int* tile_group, int* out_meta, cudaStream_t st) {
  ep_recv_plan_kernel<<<1, 32, 0, st>>>(meta_in, n_local, world, max_rows, slot_dst, offsets, tile_group, out_meta);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_ep_move(const void* slots, void* packed, const int* meta_in, const int* slot_dst,
                            const int* offsets, const long long* ret_ptrs, int rank, int n_local, int world,
                            long long cap, int d, int max_rows, int dir, long long* row_ptr_out, cudaStream_t st) {
  if (world > MAX_RANKS || d % 8) return -1;
  ep_move_kernel<<<148 * 4, 256, 0, st>>>((const __nv_bfloat16*)slots, (__nv_bfloat16*)packed, meta_in, slot_dst,
                                          offsets, make_ptrs(ret_ptrs, world), rank, n_local, world, cap, d, max_rows,
                                          dir, row_ptr_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
