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
#include <cuda_bf16.h>
#include <cuda_runtime.h>

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
__global__ void p2p_reduce_scatter_kernel(PeerPtrs grads, int rank, int world, long long off, long long n,
                                          float* __restrict__ sq_out) {
  const long long nvec = n / 8;
  const float inv = 1.f / world;
  float sq = 0.f;
  __nv_bfloat16* own = reinterpret_cast<__nv_bfloat16*>(grads.p[rank]) + off;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    float a[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (int r = 0; r < world; ++r) {
      const int src = (rank + r) % world;     // stagger peers so ranks do not all hit the same one
      const uint4 x = *(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(grads.p[src]) + off) + v);
      acc8(x, a);
    }
    uint4 o;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] *= inv;
      sq += a[i] * a[i];
    }
    o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]); o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
    *(reinterpret_cast<uint4*>(own) + v) = o;
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
                                           AdamArgs h) {
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
    for (int r = 0; r < world; ++r) {
      const int dst = (rank + r) % world;
      *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(params.p[dst]) + off) + i) = o;
    }
  }
}

// Copy [off, off+n) of this rank's buffer into every other rank's buffer.
__global__ void p2p_allgather_kernel(PeerPtrs bufs, int rank, int world, long long off, long long n) {
  const long long nvec = n / 8;
  const uint4* own = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(bufs.p[rank]) + off);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 x = own[i];
    for (int r = 1; r < world; ++r) {
      const int dst = (rank + r) % world;
      *(reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(bufs.p[dst]) + off) + i) = x;
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
                                       float* sq_out, cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8) return -1;
  p2p_reduce_scatter_kernel<<<148 * 8, 256, 0, st>>>(make_ptrs(grad_ptrs, world), rank, world, off, n, sq_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_p2p_adamw_allgather(const long long* param_ptrs, const void* grad, float* m, float* v, int rank,
                                        int world, long long off, long long n, float lr, float beta1, float beta2,
                                        float eps, float wd, int step, const float* clip_coef, cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8) return -1;
  AdamArgs h{lr, beta1, beta2, eps, wd, 1.f - powf(beta1, (float)step), 1.f - powf(beta2, (float)step), clip_coef};
  p2p_adamw_allgather_kernel<<<148 * 8, 256, 0, st>>>(make_ptrs(param_ptrs, world), (const __nv_bfloat16*)grad, m, v,
                                                      rank, world, off, n, h);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_p2p_allgather(const long long* buf_ptrs, int rank, int world, long long off, long long n,
                                  cudaStream_t st) {
  if (world > MAX_RANKS || n % 8 || off % 8) return -1;
  p2p_allgather_kernel<<<148 * 8, 256, 0, st>>>(make_ptrs(buf_ptrs, world), rank, world, off, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
