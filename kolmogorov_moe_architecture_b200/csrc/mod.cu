// Mixture-of-depths data movement: the router keeps k of S tokens per sequence (indices ascending); the kept
// rows are gathered, run through the FFN, weighted and added back onto the residual stream.
//   rows_gather       out[b, j, :] = src[b, idx[b, j], :]
//   rows_scatter      out[b, t, :] = src[b, j, :] if idx[b, j] == t else 0          (backward of the gather)
//   combine_fwd       out[b, t, :] = res[b, t, :] + (w[b, j] * proc[b, j, :] if idx[b, j] == t)
//   combine_bwd       dproc[b, j, :] = w[b, j] * dout[b, idx[b, j], :] ;  dw[b, j] = <dout[b, idx[b, j], :], proc[b, j, :]>
// One warp per row, 16-byte lanes; the inverse map token -> slot is a binary search in the sorted index row,
// so every output is written exactly once and nothing is zero-filled or accumulated afterwards.
// reference: moe_arch/model/layers.py:148-185 (gather, multiply, scatter_add_ into zeros, residual add).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

__device__ __forceinline__ int find_slot(const long long* __restrict__ row_idx, int k, int t) {
  int lo = 0, hi = k;                         // first position with idx >= t
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (row_idx[mid] < t) lo = mid + 1; else hi = mid;
  }
  return (lo < k && row_idx[lo] == t) ? lo : -1;
}

__global__ void rows_gather_kernel(const __nv_bfloat16* __restrict__ src, const long long* __restrict__ idx,
                                   __nv_bfloat16* __restrict__ out, int B, int S, int k, int d) {
  const int vec = d / 8, lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < (long long)B * k; r += warps) {
    const int b = (int)(r / k);
    const long long t = idx[r];
    const uint4* s = reinterpret_cast<const uint4*>(src + ((long long)b * S + t) * d);
    uint4* o = reinterpret_cast<uint4*>(out + r * d);
    for (int v = lane; v < vec; v += 32) o[v] = s[v];
  }
}

// out[b, t, :] = src[b, slot(t), :] for kept positions, zero elsewhere; with `coef` / `wvec` the rank-one term
// coef[b, t] * wvec[:] is added in the same pass (the gradient of a per-row dot product with wvec, i.e. of the
// mixture-of-depths scorer, which reads the same rows).
__global__ void rows_scatter_kernel(const __nv_bfloat16* __restrict__ src, const long long* __restrict__ idx,
                                    __nv_bfloat16* __restrict__ out, int B, int S, int k, int d,
                                    const __nv_bfloat16* __restrict__ coef = nullptr,
                                    const __nv_bfloat16* __restrict__ wvec = nullptr) {
  const int vec = d / 8, lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < (long long)B * S; r += warps) {
    const int b = (int)(r / S), t = (int)(r % S);
    const int j = find_slot(idx + (long long)b * k, k, t);
    uint4* o = reinterpret_cast<uint4*>(out + r * d);
    const uint4* s = j < 0 ? nullptr : reinterpret_cast<const uint4*>(src + ((long long)b * k + j) * d);
    if (coef == nullptr) {
      if (j < 0) {
        for (int v = lane; v < vec; v += 32) o[v] = make_uint4(0, 0, 0, 0);
      } else {
        for (int v = lane; v < vec; v += 32) o[v] = s[v];
      }
      continue;
    }
    const float c = __bfloat162float(coef[r]);
    for (int v = lane; v < vec; v += 32) {
      const uint4 wq = __ldg(reinterpret_cast<const uint4*>(wvec) + v);
      const uint4 sq = j < 0 ? make_uint4(0, 0, 0, 0) : s[v];
      const __nv_bfloat162* pw = reinterpret_cast<const __nv_bfloat162*>(&wq);
      const __nv_bfloat162* ps = reinterpret_cast<const __nv_bfloat162*>(&sq);
      uint4 oq;
      __nv_bfloat162* po = reinterpret_cast<__nv_bfloat162*>(&oq);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 fw = __bfloat1622float2(pw[i]), fs = __bfloat1622float2(ps[i]);
        po[i] = __floats2bfloat162_rn(fs.x + c * fw.x, fs.y + c * fw.y);
      }
      o[v] = oq;
    }
  }
}

__device__ __forceinline__ void unpack8f(const uint4& r, float* v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(p[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}

__global__ void mod_combine_fwd_kernel(const __nv_bfloat16* __restrict__ res, const __nv_bfloat16* __restrict__ proc,
                                       const float* __restrict__ w, const long long* __restrict__ idx,
                                       __nv_bfloat16* __restrict__ out, int B, int S, int k, int d) {
  const int vec = d / 8, lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < (long long)B * S; r += warps) {
    const int b = (int)(r / S), t = (int)(r % S);
    const int j = find_slot(idx + (long long)b * k, k, t);
    const uint4* rs = reinterpret_cast<const uint4*>(res + r * d);
    uint4* o = reinterpret_cast<uint4*>(out + r * d);
    if (j < 0) {
      for (int v = lane; v < vec; v += 32) o[v] = rs[v];
    } else {
      const float wj = w[(long long)b * k + j];
      const uint4* ps = reinterpret_cast<const uint4*>(proc + ((long long)b * k + j) * d);
      for (int v = lane; v < vec; v += 32) {
        float a[8], p[8];
        unpack8f(rs[v], a);
        unpack8f(ps[v], p);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          // the weighted row is rounded to bf16 before the add, as the unfused multiply produced a bf16 tensor
          a[i] += __bfloat162float(__float2bfloat16(wj * p[i]));
        }
        uint4 q;
        q.x = pack_bf16(a[0], a[1]); q.y = pack_bf16(a[2], a[3]); q.z = pack_bf16(a[4], a[5]); q.w = pack_bf16(a[6], a[7]);
        o[v] = q;
      }
    }
  }
}

__global__ void mod_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ proc,
                                       const float* __restrict__ w, const long long* __restrict__ idx,
                                       __nv_bfloat16* __restrict__ dproc, float* __restrict__ dw, int B, int S, int k,
                                       int d) {
  const int vec = d / 8, lane = threadIdx.x & 31;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long r = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < (long long)B * k; r += warps) {
    const int b = (int)(r / k);
    const long long t = idx[r];
    const float wj = w[r];
    const uint4* gs = reinterpret_cast<const uint4*>(dout + ((long long)b * S + t) * d);
    const uint4* ps = reinterpret_cast<const uint4*>(proc + r * d);
    uint4* o = reinterpret_cast<uint4*>(dproc + r * d);
    float dot = 0.f;
    for (int v = lane; v < vec; v += 32) {
      float g[8], p[8];
      unpack8f(gs[v], g);
      unpack8f(ps[v], p);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dot += g[i] * p[i];
        g[i] *= wj;
      }
      uint4 q;
      q.x = pack_bf16(g[0], g[1]); q.y = pack_bf16(g[2], g[3]); q.z = pack_bf16(g[4], g[5]); q.w = pack_bf16(g[6], g[7]);
      o[v] = q;
    }
    dot = warp_sum(dot);
    if (lane == 0) dw[r] = dot;
  }
}

static int grid_rows(long long rows) {
  const long long want = (rows + 7) / 8;           // 8 warps per 256-thread CTA
  return (int)(want < 148 * 16 ? (want > 0 ? want : 1) : 148 * 16);
}

// Binary cross-entropy of the selection predictor: the target of position (b, t) is 1 iff t is among the kept
// (ascending) indices of sequence b.  loss = mean over B * S of softplus(x) - x * target, and
// dlogits = (sigmoid(x) - target) / (B * S) for an upstream gradient of 1.  Blocks of 256 positions write partial
// sums, a second one-warp kernel adds them in a fixed order.
__global__ void __launch_bounds__(256)
mod_bce_kernel(const __nv_bfloat16* __restrict__ logits, const long long* __restrict__ idx,
               float* __restrict__ partial, __nv_bfloat16* __restrict__ dlogits, int B, int S, int k) {
  __shared__ float red[8];
  const long long n = (long long)B * S;
  const float inv = 1.f / (float)n;
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  float acc = 0.f;
  if (i < n) {
    const int b = (int)(i / S), t = (int)(i % S);
    const float x = __bfloat162float(logits[i]);
    const float tgt = find_slot(idx + (long long)b * k, k, t) >= 0 ? 1.f : 0.f;
    acc = fmaxf(x, 0.f) - x * tgt + log1pf(__expf(-fabsf(x)));
    dlogits[i] = __float2bfloat16((1.f / (1.f + __expf(-x)) - tgt) * inv);
  }
  acc = warp_sum(acc);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float tot = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) tot += red[w];
    partial[blockIdx.x] = tot;
  }
}
__global__ void mod_bce_sum_kernel(const float* __restrict__ partial, int nparts, float inv, float* __restrict__ loss) {
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 32) s += partial[i];
  s = warp_sum(s);
  if (threadIdx.x == 0) loss[0] = s * inv;
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_mod_bce_num_partials(int B, int S) { return (int)(((long long)B * S + 255) / 256); }

// partial: scratch of kmoe_mod_bce_num_partials(B, S) floats
extern "C" int kmoe_mod_bce(const void* logits, const long long* idx, float* partial, float* loss, void* dlogits, int B,
                            int S, int k, cudaStream_t st) {
  if (B * (long long)S == 0) return -1;
  const int g = kmoe_mod_bce_num_partials(B, S);
  mod_bce_kernel<<<g, 256, 0, st>>>((const __nv_bfloat16*)logits, idx, partial, (__nv_bfloat16*)dlogits, B, S, k);
  mod_bce_sum_kernel<<<1, 32, 0, st>>>(partial, g, 1.f / (float)((long long)B * S), loss);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rows_gather(const void* src, const long long* idx, void* out, int B, int S, int k, int d,
                                cudaStream_t st) {
  if (d % 8) return -1;
  if (B * (long long)k == 0) return 0;
  rows_gather_kernel<<<grid_rows((long long)B * k), 256, 0, st>>>((const __nv_bfloat16*)src, idx, (__nv_bfloat16*)out,
                                                                  B, S, k, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rows_scatter(const void* src, const long long* idx, void* out, int B, int S, int k, int d,
                                 cudaStream_t st) {
  if (d % 8) return -1;
  if (B * (long long)S == 0) return 0;
  rows_scatter_kernel<<<grid_rows((long long)B * S), 256, 0, st>>>((const __nv_bfloat16*)src, idx, (__nv_bfloat16*)out,
                                                                   B, S, k, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rows_scatter_rank1(const void* src, const long long* idx, const void* coef, const void* wvec,
                                       void* out, int B, int S, int k, int d, cudaStream_t st) {
  if (d % 8 || coef == nullptr || wvec == nullptr) return -1;
  if (B * (long long)S == 0) return 0;
  rows_scatter_kernel<<<grid_rows((long long)B * S), 256, 0, st>>>(
      (const __nv_bfloat16*)src, idx, (__nv_bfloat16*)out, B, S, k, d, (const __nv_bfloat16*)coef,
      (const __nv_bfloat16*)wvec);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_mod_combine_fwd(const void* res, const void* proc, const float* w, const long long* idx, void* out,
                                    int B, int S, int k, int d, cudaStream_t st) {
  if (d % 8) return -1;
  if (B * (long long)S == 0) return 0;
  mod_combine_fwd_kernel<<<grid_rows((long long)B * S), 256, 0, st>>>(
      (const __nv_bfloat16*)res, (const __nv_bfloat16*)proc, w, idx, (__nv_bfloat16*)out, B, S, k, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_mod_combine_bwd(const void* dout, const void* proc, const float* w, const long long* idx,
                                    void* dproc, float* dw, int B, int S, int k, int d, cudaStream_t st) {
  if (d % 8) return -1;
  if (B * (long long)k == 0) return 0;
  mod_combine_bwd_kernel<<<grid_rows((long long)B * k), 256, 0, st>>>(
      (const __nv_bfloat16*)dout, (const __nv_bfloat16*)proc, w, idx, (__nv_bfloat16*)dproc, dw, B, S, k, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
