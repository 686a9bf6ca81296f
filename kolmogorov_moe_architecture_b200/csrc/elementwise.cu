// Bandwidth-bound row kernels: RMSNorm fwd/bwd, rotate-half RoPE, SwiGLU fwd/bwd.
// bf16 in/out, fp32 math, 16-byte vector accesses.  One warp per row for the
// normalisation kernels (a 2048-wide row is 8 x uint4 per lane).
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <cstdlib>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

__device__ __forceinline__ void unpack8(const uint4& r, float* v) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(p[i]);
    v[2 * i] = f.x;
    v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 o;
  o.x = pack_bf16(v[0], v[1]);
  o.y = pack_bf16(v[2], v[3]);
  o.z = pack_bf16(v[4], v[5]);
  o.w = pack_bf16(v[6], v[7]);
  return o;
}

// ------------------------------------------------------------------- RMSNorm
// y = w * x * rsqrt(mean(x^2) + eps); optionally res_out = x (+ residual) is fused by the caller.
// With `addend` the normalised row is h = bf16(x + addend), which is also written to `sum_out` (the residual
// stream after the sequence mixer): residual add and pre-FFN norm in one pass.
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, int d,
                                   float eps, const __nv_bfloat16* __restrict__ addend,
                                   __nv_bfloat16* __restrict__ sum_out) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const __nv_bfloat16* xr = x + (size_t)row * d;
    if (addend != nullptr) {
      const __nv_bfloat16* ar = addend + (size_t)row * d;
      __nv_bfloat16* sr = sum_out + (size_t)row * d;
      for (int c = lane * 8; c < d; c += 256) {
        float v[8], a[8];
        unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
        unpack8(*reinterpret_cast<const uint4*>(ar + c), a);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += a[i];
        *reinterpret_cast<uint4*>(sr + c) = pack8(v);
      }
      __syncwarp();
      xr = sr;                                   // each lane re-reads the columns it wrote itself
    }
    float ss = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / d + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
    __nv_bfloat16* yr = y + (size_t)row * d;
    for (int c = lane * 8; c < d; c += 256) {
      float v[8], g[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
      unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * r * g[i];
      *reinterpret_cast<uint4*>(yr + c) = pack8(v);
    }
  }
}

// Register-resident variants for rows of NCH * 256 elements (NCH <= 8): a warp reads its row once (eight
// elements per lane and 256-column chunk), so x / dy are not read a second time for the output pass, and the
// backward also accumulates the weight gradient (column sums of dy * x * rstd over the rows a warp visits, then
// over the block through shared memory): one pass over x and dy instead of three.
template <int NCH>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows, float eps,
                        const __nv_bfloat16* __restrict__ addend, __nv_bfloat16* __restrict__ sum_out) {
  constexpr int D = NCH * 256;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint4 wq[NCH];
#pragma unroll
  for (int j = 0; j < NCH; ++j) wq[j] = __ldg(reinterpret_cast<const uint4*>(w + j * 256 + lane * 8));
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const size_t base = (size_t)row * D + lane * 8;
    uint4 xq[NCH];
#pragma unroll
    for (int j = 0; j < NCH; ++j) xq[j] = *reinterpret_cast<const uint4*>(x + base + j * 256);
    if (addend != nullptr) {
#pragma unroll
      for (int j = 0; j < NCH; ++j) {
        float v[8], a[8];
        unpack8(xq[j], v);
        unpack8(*reinterpret_cast<const uint4*>(addend + base + j * 256), a);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] += a[i];
        xq[j] = pack8(v);                          // the normalised row is the rounded sum, as stored
        *reinterpret_cast<uint4*>(sum_out + base + j * 256) = xq[j];
      }
    }
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float v[8];
      unpack8(xq[j], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += v[i] * v[i];
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / D + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float v[8], g[8];
      unpack8(xq[j], v);
      unpack8(wq[j], g);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = v[i] * r * g[i];
      *reinterpret_cast<uint4*>(y + base + j * 256) = pack8(v);
    }
  }
}

template <int NCH, bool WITH_DW>
__global__ void __launch_bounds__(256, WITH_DW ? 1 : 2)
rmsnorm_bwd_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ partial, int rows,
                        const __nv_bfloat16* __restrict__ dres) {
  constexpr int D = NCH * 256;
  __shared__ float sacc[D];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (WITH_DW) {
    for (int i = threadIdx.x; i < D; i += 256) sacc[i] = 0.f;
    __syncthreads();
  }
  const __nv_bfloat16* wl = w + lane * 8;          // re-read per row (first-level cache hits): saves 4 NCH registers
  float acc[WITH_DW ? NCH * 8 : 1];
#pragma unroll
  for (int i = 0; i < (WITH_DW ? NCH * 8 : 1); ++i) acc[i] = 0.f;
  for (int row = blockIdx.x * 8 + warp; row < rows; row += gridDim.x * 8) {
    const size_t base = (size_t)row * D + lane * 8;
    uint4 xq[NCH], gq[NCH];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      xq[j] = *reinterpret_cast<const uint4*>(x + base + j * 256);
      gq[j] = *reinterpret_cast<const uint4*>(dy + base + j * 256);
    }
    const float r = rstd[row];
    float dot = 0.f;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float xv[8], gv[8], wv[8];
      unpack8(xq[j], xv);
      unpack8(gq[j], gv);
      unpack8(__ldg(reinterpret_cast<const uint4*>(wl + j * 256)), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        dot += gv[i] * wv[i] * xv[i];
        if (WITH_DW) acc[j * 8 + i] += gv[i] * xv[i] * r;
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * r * r * r / D;
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
      float xv[8], gv[8], wv[8], o[8];
      unpack8(xq[j], xv);
      unpack8(gq[j], gv);
      unpack8(__ldg(reinterpret_cast<const uint4*>(wl + j * 256)), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = gv[i] * wv[i] * r - xv[i] * coef;
      if (dres != nullptr) {
        float rv[8];
        unpack8(*reinterpret_cast<const uint4*>(dres + base + j * 256), rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += rv[i];
      }
      *reinterpret_cast<uint4*>(dx + base + j * 256) = pack8(o);
    }
  }
  if (WITH_DW) {
#pragma unroll
    for (int j = 0; j < NCH; ++j)
#pragma unroll
      for (int i = 0; i < 8; ++i) atomicAdd(&sacc[j * 256 + lane * 8 + i], acc[j * 8 + i]);
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += 256) partial[(size_t)blockIdx.x * D + i] = sacc[i];
  }
}

// dx = rstd * (w dy) - x * rstd^3 * mean(w dy x).  One warp per row.
// `dres` (optional): gradient arriving through the residual branch that bypasses the norm; dx = norm term + dres.
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                   const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                                   __nv_bfloat16* __restrict__ dx, int rows, int d,
                                   const __nv_bfloat16* __restrict__ dres = nullptr) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const __nv_bfloat16* xr = x + (size_t)row * d;
    const __nv_bfloat16* gr = dy + (size_t)row * d;
    const float r = rstd[row];
    float dot = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
      float xv[8], gv[8], wv[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), xv);
      unpack8(*reinterpret_cast<const uint4*>(gr + c), gv);
      unpack8(*reinterpret_cast<const uint4*>(w + c), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) dot += gv[i] * wv[i] * xv[i];
    }
    dot = warp_sum(dot);
    const float coef = dot * r * r * r / d;
    __nv_bfloat16* dxr = dx + (size_t)row * d;
    for (int c = lane * 8; c < d; c += 256) {
      float xv[8], gv[8], wv[8], o[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), xv);
      unpack8(*reinterpret_cast<const uint4*>(gr + c), gv);
      unpack8(*reinterpret_cast<const uint4*>(w + c), wv);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = gv[i] * wv[i] * r - xv[i] * coef;
      if (dres != nullptr) {
        float rv[8];
        unpack8(*reinterpret_cast<const uint4*>(dres + (size_t)row * d + c), rv);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += rv[i];
      }
      *reinterpret_cast<uint4*>(dxr + c) = pack8(o);
    }
  }
}

// Column sums of dy * x * rstd over a slice of the rows: partial[blockIdx.y][c].
// Block = 32 column-vectors (256 columns) x 8 row lanes.
__global__ void rmsnorm_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                  const float* __restrict__ rstd, float* __restrict__ partial, int rows, int d) {
  __shared__ float red[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + tx * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < d) {
    for (int row = blockIdx.y * 8 + ty; row < rows; row += gridDim.y * 8) {
      float xv[8], gv[8];
      unpack8(*reinterpret_cast<const uint4*>(x + (size_t)row * d + c), xv);
      unpack8(*reinterpret_cast<const uint4*>(dy + (size_t)row * d + c), gv);
      const float r = rstd[row];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += gv[i] * xv[i] * r;
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[ty][tx * 8 + i] = acc[i];
  __syncthreads();
  const int col = threadIdx.x;  // 256 threads, one column each
  float s_ = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s_ += red[j][col];
  if (blockIdx.x * 256 + col < d) partial[(size_t)blockIdx.y * d + blockIdx.x * 256 + col] = s_;
}

// Sum of `nparts` rows of partial column sums.  A block owns 32 columns; its eight warps take every eighth row
// and the warp results are added in a fixed order.  Launch with colsum_grid(d) blocks of 256 threads.
__global__ void __launch_bounds__(256)
colsum_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out_bf16,
                       float* __restrict__ out_f32, int nparts, int d) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f;
  if (c < d) {
    int p = warp;
    for (; p + 8 < nparts; p += 16) {
      s0 += partial[(size_t)p * d + c];
      s1 += partial[(size_t)(p + 8) * d + c];
    }
    if (p < nparts) s0 += partial[(size_t)p * d + c];
  }
  red[warp][lane] = s0 + s1;
  __syncthreads();
  if (warp == 0 && c < d) {
    float s = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) s += red[w][lane];
    if (out_bf16 != nullptr) out_bf16[c] = __float2bfloat16(s);
    if (out_f32 != nullptr) out_f32[c] = s;
  }
}
static inline int colsum_grid(int d) { return (d + 31) / 32; }

// ------------------------------------------------- Linear with one output column
// y[row] = sum_c x[row, c] * w[c]   (the mixture-of-depths scorer and the last layer of its
// auxiliary predictor: nn.Linear(d, 1)).  One warp per row.
__global__ void rowdot_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                  __nv_bfloat16* __restrict__ y, int rows, int d) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const __nv_bfloat16* xr = x + (size_t)row * d;
    float s = 0.f;
    for (int c = lane * 8; c < d; c += 256) {
      float v[8], g[8];
      unpack8(*reinterpret_cast<const uint4*>(xr + c), v);
      unpack8(*reinterpret_cast<const uint4*>(w + c), g);
#pragma unroll
      for (int i = 0; i < 8; ++i) s += v[i] * g[i];
    }
    s = warp_sum(s);
    if (lane == 0) y[row] = __float2bfloat16(s);
  }
}

// dx[row, c] = dy[row] * w[c]
__global__ void rowdot_dx_kernel(const __nv_bfloat16* __restrict__ dy, const __nv_bfloat16* __restrict__ w,
                                 __nv_bfloat16* __restrict__ dx, int rows, int d) {
  const int warps_per_block = blockDim.x >> 5;
  const int lane = threadIdx.x & 31;
  for (int row = blockIdx.x * warps_per_block + (threadIdx.x >> 5); row < rows; row += gridDim.x * warps_per_block) {
    const float g = __bfloat162float(dy[row]);
    __nv_bfloat16* dxr = dx + (size_t)row * d;
    for (int c = lane * 8; c < d; c += 256) {
      float v[8];
      unpack8(*reinterpret_cast<const uint4*>(w + c), v);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] *= g;
      *reinterpret_cast<uint4*>(dxr + c) = pack8(v);
    }
  }
}

// partial[blockIdx.y][c] = sum over a slice of the rows of dy[row] * x[row, c]
__global__ void rowdot_dw_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                 float* __restrict__ partial, int rows, int d) {
  __shared__ float red[8][256];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 256 + tx * 8;
  float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
  if (c < d) {
    for (int row = blockIdx.y * 8 + ty; row < rows; row += gridDim.y * 8) {
      float xv[8];
      unpack8(*reinterpret_cast<const uint4*>(x + (size_t)row * d + c), xv);
      const float g = __bfloat162float(dy[row]);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += g * xv[i];
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) red[ty][tx * 8 + i] = acc[i];
  __syncthreads();
  const int col = threadIdx.x;
  float s_ = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) s_ += red[j][col];
  if (blockIdx.x * 256 + col < d) partial[(size_t)blockIdx.y * d + blockIdx.x * 256 + col] = s_;
}

// ---------------------------------------------------------------------- RoPE
// x: [B, S, H, D] bf16 ; cos/sin: fp32 [*, S, D] with batch stride cs_bstride (0 = shared).
// out = x * cos + rotate_half(x) * sin ; `sign` = -1 gives the transpose (the backward).
__global__ void rope_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ cs,
                            const float* __restrict__ sn, __nv_bfloat16* __restrict__ out, int B, int S, int H, int D,
                            long long cs_bstride, float sign) {
  const int half = D / 2;
  const int vec_per_head = half / 8;
  const long long total = (long long)B * S * H * vec_per_head;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(i % vec_per_head);
    long long t = i / vec_per_head;
    const int h = (int)(t % H);
    t /= H;
    const int s = (int)(t % S);
    const int b = (int)(t / S);
    const size_t base = (((size_t)b * S + s) * H + h) * D + v * 8;
    const size_t cbase = (size_t)b * cs_bstride + (size_t)s * D + v * 8;
    float x1[8], x2[8], o1[8], o2[8];
    unpack8(*reinterpret_cast<const uint4*>(x + base), x1);
    unpack8(*reinterpret_cast<const uint4*>(x + base + half), x2);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float c1 = cs[cbase + j], c2 = cs[cbase + half + j];
      const float s1 = sign * sn[cbase + j], s2 = sign * sn[cbase + half + j];
      // forward: o1 = x1 c1 - x2 s1 ; o2 = x2 c2 + x1 s2.  transpose: o1 = x1 c1 + x2 s2 ; o2 = x2 c2 - x1 s1
      if (sign > 0.f) {
        o1[j] = x1[j] * c1 - x2[j] * s1;
        o2[j] = x2[j] * c2 + x1[j] * s2;
      } else {
        o1[j] = x1[j] * c1 - x2[j] * s2;
        o2[j] = x2[j] * c2 + x1[j] * s1;
      }
    }
    *reinterpret_cast<uint4*>(out + base) = pack8(o1);
    *reinterpret_cast<uint4*>(out + base + half) = pack8(o2);
  }
}

// -------------------------------------------------------------------- SwiGLU
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                  __nv_bfloat16* __restrict__ h, long long rows, int cols, long long ldg,
                                  long long ldu, const int* __restrict__ live_rows) {
  const int vpr = cols / 8;
  if (live_rows != nullptr) rows = min(rows, (long long)*live_rows);   // rows past the live count hold no data
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float gv[8], uv[8];
    unpack8(*reinterpret_cast<const uint4*>(g + r * ldg + c), gv);
    unpack8(*reinterpret_cast<const uint4*>(u + r * ldu + c), uv);
#pragma unroll
    for (int j = 0; j < 8; ++j) gv[j] = silu_f(gv[j]) * uv[j];
    *reinterpret_cast<uint4*>(h + r * cols + c) = pack8(gv);
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ g, const __nv_bfloat16* __restrict__ u,
                                  const __nv_bfloat16* __restrict__ dh, __nv_bfloat16* __restrict__ dg,
                                  __nv_bfloat16* __restrict__ du, long long rows, int cols, long long ldg,
                                  long long ldu, long long ldo, const int* __restrict__ live_rows) {
  const int vpr = cols / 8;
  if (live_rows != nullptr) rows = min(rows, (long long)*live_rows);
  const long long total = rows * vpr;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
       i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vpr;
    const int c = (int)(i % vpr) * 8;
    float gv[8], uv[8], dv[8], og[8], ou[8];
    unpack8(*reinterpret_cast<const uint4*>(g + r * ldg + c), gv);
    unpack8(*reinterpret_cast<const uint4*>(u + r * ldu + c), uv);
    unpack8(*reinterpret_cast<const uint4*>(dh + r * cols + c), dv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float sg = 1.f / (1.f + __expf(-gv[j]));
      og[j] = dv[j] * uv[j] * sg * (1.f + gv[j] * (1.f - sg));
      ou[j] = dv[j] * gv[j] * sg;
    }
    *reinterpret_cast<uint4*>(dg + r * ldo + c) = pack8(og);
    *reinterpret_cast<uint4*>(du + r * ldo + c) = pack8(ou);
  }
}

static inline int grid_for(long long work, int block, int sms = 148) {
  long long g = (work + block - 1) / block;
  long long cap = (long long)sms * 16;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_add_rmsnorm_fwd(const void* x, const void* addend, const void* w, void* sum_out, void* y,
                                    float* rstd, int rows, int d, float eps, cudaStream_t st) {
  if (d % 8 || (addend != nullptr) != (sum_out != nullptr)) return -1;
  const int block = 256, wpb = block / 32;
  int grid = (rows + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  if (rows > 0 && (d == 256 || d == 512 || d == 1024 || d == 2048)) {
    const int g2 = grid > 148 * 4 ? 148 * 4 : grid;
#define KMOE_FWD_ROWS(NCH)                                                                                        \
  rmsnorm_fwd_rows_kernel<NCH><<<g2, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,              \
                                                   (__nv_bfloat16*)y, rstd, rows, eps,                            \
                                                   (const __nv_bfloat16*)addend, (__nv_bfloat16*)sum_out)
    if (d == 2048) KMOE_FWD_ROWS(8);
    else if (d == 1024) KMOE_FWD_ROWS(4);
    else if (d == 512) KMOE_FWD_ROWS(2);
    else KMOE_FWD_ROWS(1);
#undef KMOE_FWD_ROWS
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  rmsnorm_fwd_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y,
                                             rstd, rows, d, eps, (const __nv_bfloat16*)addend,
                                             (__nv_bfloat16*)sum_out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, int rows, int d, float eps,
                                cudaStream_t st) {
  return kmoe_add_rmsnorm_fwd(x, nullptr, w, nullptr, y, rstd, rows, d, eps, st);
}

// Rows of fp32 partial column sums a backward pass may write: one per CTA of the register-resident kernel (eight
// rows per CTA and sweep, at most two CTAs per SM).
extern "C" int kmoe_rmsnorm_bwd_num_partials(int rows) {
  int r = (rows + 7) / 8;
  return r > 296 ? 296 : (r < 1 ? 1 : r);
}

// `partial` is scratch of kmoe_rmsnorm_bwd_num_partials(rows) * d floats.
extern "C" int kmoe_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                void* dw_bf16, float* dw_f32, float* partial, int rows, int d, cudaStream_t st) {
  return kmoe_rmsnorm_bwd_res(x, w, dy, rstd, nullptr, dx, dw_bf16, dw_f32, partial, rows, d, st);
}

// dres (optional, bf16 [rows, d]): gradient of the residual branch, added to dx in the same pass.
extern "C" int kmoe_rmsnorm_bwd_res(const void* x, const void* w, const void* dy, const float* rstd, const void* dres,
                                    void* dx, void* dw_bf16, float* dw_f32, float* partial, int rows, int d,
                                    cudaStream_t st) {
  if (d % 8) return -1;
  const int block = 256, wpb = block / 32;
  int grid = (rows + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  static int rows_mode = -1;      // KMOE_NORM_ROWS: 0 = generic kernels, 1 = one fused pass, 2 = register-resident dx + separate dw
  if (rows_mode < 0) {
    const char* e = getenv("KMOE_NORM_ROWS");
    rows_mode = e != nullptr ? atoi(e) : 1;
  }
  if (rows_mode != 0 && rows > 0 && (d == 256 || d == 512 || d == 1024 || d == 2048)) {
    const int g2 = kmoe_rmsnorm_bwd_num_partials(rows);
    const bool fused = rows_mode == 1;
#define KMOE_BWD_ROWS(NCH)                                                                                        \
  do {                                                                                                            \
    if (fused)                                                                                                    \
      rmsnorm_bwd_rows_kernel<NCH, true><<<g2, 256, 0, st>>>(                                                     \
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx,   \
          partial, rows, (const __nv_bfloat16*)dres);                                                             \
    else                                                                                                          \
      rmsnorm_bwd_rows_kernel<NCH, false><<<grid > 148 * 4 ? 148 * 4 : grid, 256, 0, st>>>(                       \
          (const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx,   \
          partial, rows, (const __nv_bfloat16*)dres);                                                             \
  } while (0)
    if (d == 2048) KMOE_BWD_ROWS(8);
    else if (d == 1024) KMOE_BWD_ROWS(4);
    else if (d == 512) KMOE_BWD_ROWS(2);
    else KMOE_BWD_ROWS(1);
#undef KMOE_BWD_ROWS
    int parts = g2;
    if (!fused) {
      parts = g2 > 64 ? 64 : g2;
      rmsnorm_dw_kernel<<<dim3((d + 255) / 256, parts), 256, 0, st>>>((const __nv_bfloat16*)x,
                                                                      (const __nv_bfloat16*)dy, rstd, partial, rows, d);
    }
    colsum_partials_kernel<<<colsum_grid(d), 256, 0, st>>>(partial, (__nv_bfloat16*)dw_bf16, dw_f32, parts, d);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  rmsnorm_bwd_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                             (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, rows, d,
                                             (const __nv_bfloat16*)dres);
  const int parts = kmoe_rmsnorm_bwd_num_partials(rows);
  rmsnorm_dw_kernel<<<dim3((d + 255) / 256, parts), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                  rstd, partial, rows, d);
  colsum_partials_kernel<<<colsum_grid(d), 256, 0, st>>>(partial, (__nv_bfloat16*)dw_bf16, dw_f32, parts, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// out[i] = sum over p of partial[p][i] (fp32 partial results of a split reduction) as bf16; four values per thread.
__global__ void sum_partials_kernel(const float* __restrict__ partial, __nv_bfloat16* __restrict__ out, int nparts,
                                    long long n) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int p = 0; p < nparts; ++p) {
    const float4 v = *reinterpret_cast<const float4*>(partial + (size_t)p * n + i);
    s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
  }
  uint2 o;
  o.x = pack_bf16(s.x, s.y);
  o.y = pack_bf16(s.z, s.w);
  *reinterpret_cast<uint2*>(out + i) = o;
}

// Sum of squares of n bf16 values in fp32 (the gradient norm of a flat buffer): block partial sums, then one
// block adds them in a fixed order, so the result does not depend on scheduling.
constexpr int SUMSQ_BLOCKS = 148 * 8;
__global__ void __launch_bounds__(256)
sumsq_partial_kernel(const __nv_bfloat16* __restrict__ x, long long n, float* __restrict__ partial) {
  __shared__ float red[8];
  const long long nvec = n / 8;
  const uint4* xv = reinterpret_cast<const uint4*>(x);
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  for (; i + 3 * stride < nvec; i += 4 * stride) {          // four independent 16-byte loads in flight
    const uint4 a = __ldg(xv + i), b = __ldg(xv + i + stride), c = __ldg(xv + i + 2 * stride),
                d = __ldg(xv + i + 3 * stride);
    float v[8];
    unpack8(a, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s0 += v[k] * v[k];
    unpack8(b, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s1 += v[k] * v[k];
    unpack8(c, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s2 += v[k] * v[k];
    unpack8(d, v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s3 += v[k] * v[k];
  }
  for (; i < nvec; i += stride) {
    float v[8];
    unpack8(__ldg(xv + i), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) s0 += v[k] * v[k];
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * 8)) {   // tail of fewer than eight values
    const float t = __bfloat162float(x[nvec * 8 + threadIdx.x]);
    s1 += t * t;
  }
  float s = warp_sum((s0 + s1) + (s2 + s3));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}
__global__ void __launch_bounds__(256) sumsq_final_kernel(const float* __restrict__ partial, int nparts,
                                                          float* __restrict__ out) {
  __shared__ float red[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < nparts; i += 256) s += partial[i];
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) t += red[w];
    out[0] = t;
  }
}

extern "C" int kmoe_sumsq_num_partials(void) { return SUMSQ_BLOCKS; }

// x: n bf16 values, 16-byte aligned; partial: kmoe_sumsq_num_partials() floats of scratch; out: one float.
extern "C" int kmoe_sumsq_bf16(const void* x, long long n, float* partial, float* out, cudaStream_t st) {
  if (n < 0 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  sumsq_partial_kernel<<<SUMSQ_BLOCKS, 256, 0, st>>>((const __nv_bfloat16*)x, n, partial);
  sumsq_final_kernel<<<1, 256, 0, st>>>(partial, SUMSQ_BLOCKS, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dst = bf16(src * *scale): a gradient computed for an upstream gradient of 1, rescaled on its way into the flat
// gradient buffer.  16 bytes per thread and iteration.
__global__ void __launch_bounds__(256)
scale_copy_kernel(const __nv_bfloat16* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n,
                  const float* __restrict__ scale) {
  const float sc = *scale;
  const long long nvec = n / 8;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    float v[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(src) + i), v);
#pragma unroll
    for (int k = 0; k < 8; ++k) v[k] *= sc;
    reinterpret_cast<uint4*>(dst)[i] = pack8(v);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n - nvec * 8))
    dst[nvec * 8 + threadIdx.x] = __float2bfloat16(__bfloat162float(src[nvec * 8 + threadIdx.x]) * sc);
}

extern "C" int kmoe_scale_copy(const void* src, void* dst, long long n, const float* scale, cudaStream_t st) {
  if (n < 0 || ((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15)) return -1;
  if (n == 0) return 0;
  scale_copy_kernel<<<148 * 8, 256, 0, st>>>((const __nv_bfloat16*)src, (__nv_bfloat16*)dst, n, scale);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_sum_partials(const float* partial, void* out, int nparts, long long n, cudaStream_t st) {
  if (n % 4 || nparts < 1) return -1;
  sum_partials_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, st>>>(partial, (__nv_bfloat16*)out, nparts, n);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rowdot_fwd(const void* x, const void* w, void* y, int rows, int d, cudaStream_t st) {
  if (d % 8) return -1;
  const int block = 256, wpb = block / 32;
  int grid = (rows + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  rowdot_fwd_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w, (__nv_bfloat16*)y, rows, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// `partial` is scratch of kmoe_rmsnorm_bwd_num_partials(rows) * d floats; dw may be bf16 and/or fp32.
extern "C" int kmoe_rowdot_bwd(const void* x, const void* w, const void* dy, void* dx, void* dw_bf16, float* dw_f32,
                               float* partial, int rows, int d, cudaStream_t st) {
  if (d % 8) return -1;
  const int block = 256, wpb = block / 32;
  int grid = (rows + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  if (dx != nullptr)
    rowdot_dx_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)dy, (const __nv_bfloat16*)w, (__nv_bfloat16*)dx,
                                             rows, d);
  const int parts = kmoe_rmsnorm_bwd_num_partials(rows);
  rowdot_dw_kernel<<<dim3((d + 255) / 256, parts), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                 partial, rows, d);
  colsum_partials_kernel<<<colsum_grid(d), 256, 0, st>>>(partial, (__nv_bfloat16*)dw_bf16, dw_f32, parts, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_rope(const void* x, const float* cs, const float* sn, void* out, int B, int S, int H, int D,
                         long long cs_bstride, int transpose, cudaStream_t st) {
  if (D % 16) return -1;
  const long long total = (long long)B * S * H * (D / 16);
  rope_kernel<<<grid_for(total, 256), 256, 0, st>>>((const __nv_bfloat16*)x, cs, sn, (__nv_bfloat16*)out, B, S, H, D,
                                                    cs_bstride, transpose ? -1.f : 1.f);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_swiglu_fwd(const void* g, const void* u, void* h, long long rows, int cols, long long ldg,
                               long long ldu, const int* live_rows, cudaStream_t st) {
  if (cols % 8 || ldg % 8 || ldu % 8) return -1;
  swiglu_fwd_kernel<<<grid_for(rows * (cols / 8), 256), 256, 0, st>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)h, rows, cols, ldg, ldu, live_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_swiglu_bwd(const void* g, const void* u, const void* dh, void* dg, void* du, long long rows,
                               int cols, long long ldg, long long ldu, long long ldo, const int* live_rows,
                               cudaStream_t st) {
  if (cols % 8 || ldg % 8 || ldu % 8 || ldo % 8) return -1;
  swiglu_bwd_kernel<<<grid_for(rows * (cols / 8), 256), 256, 0, st>>>(
      (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (const __nv_bfloat16*)dh, (__nv_bfloat16*)dg,
      (__nv_bfloat16*)du, rows, cols, ldg, ldu, ldo, live_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// ------------------------------------------------- allocation-free RMSNorm backward
// See kmoe_noalloc.h.  The scratch lives in the device image; host code must not pass the
// symbol itself to a kernel (on the host it is only a stand-in), so its device address is
// looked up once per device and cached.
#include "kmoe_noalloc.h"

namespace kmoe {
constexpr int NOALLOC_PARTS = 64;
constexpr int NOALLOC_MAX_DEVICES = 64;
static __device__ __align__(256) float g_noalloc_scratch[NOALLOC_PARTS * KMOE_NOALLOC_MAX_D];
static float* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {nullptr};
}  // namespace kmoe

extern "C" int kmoe_rmsnorm_bwd_noalloc(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                                        float* dw_f32, int rows, int d, cudaStream_t st) {
  if (rows < 1 || d < 8 || d % 8 != 0 || d > KMOE_NOALLOC_MAX_D) return KMOE_NOALLOC_E_SIZE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= NOALLOC_MAX_DEVICES) return KMOE_NOALLOC_E_SYMBOL;
  if (g_noalloc_ptr[dev] == nullptr) {
    // first call on this device: resolve the array's device address (device `dev` is current)
    float* p = nullptr;
    if (cudaGetSymbolAddress((void**)&p, g_noalloc_scratch) != cudaSuccess || p == nullptr)
      return KMOE_NOALLOC_E_SYMBOL;
    g_noalloc_ptr[dev] = p;
  }
  float* partial = g_noalloc_ptr[dev];
  const int block = 256, wpb = block / 32;
  int grid = (rows + wpb - 1) / wpb;
  if (grid > 148 * 8) grid = 148 * 8;
  rmsnorm_bwd_kernel<<<grid, block, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)w,
                                             (const __nv_bfloat16*)dy, rstd, (__nv_bfloat16*)dx, rows, d);
  int parts = kmoe_rmsnorm_bwd_num_partials(rows);
  if (parts > NOALLOC_PARTS) parts = NOALLOC_PARTS;
  // every partial row that is summed below is fully written by rmsnorm_dw_kernel first, so nothing
  // left over from an earlier call is ever read and no clearing pass is needed
  rmsnorm_dw_kernel<<<dim3((d + 255) / 256, parts), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                  rstd, partial, rows, d);
  colsum_partials_kernel<<<colsum_grid(d), 256, 0, st>>>(partial, nullptr, dw_f32, parts, d);
  return cudaGetLastError() == cudaSuccess ? 0 : KMOE_NOALLOC_E_LAUNCH;
}

// ------------------------------------------------- Muon: momentum update and parameter update, one pass each
// (the orthogonalisation between them is the batched Newton-Schulz GEMM loop).  grid.y = matrix index.
namespace kmoe {

// gcoef (optional, device): the gradient is used as bf16(g * bf16(*gcoef)), i.e. as if the clip coefficient
// had been multiplied into the bf16 gradient in memory beforehand (both Muon kernels apply it the same way)
__device__ __forceinline__ float muon_gcoef(const float* gcoef) {
  return gcoef != nullptr ? __bfloat162float(__float2bfloat16(*gcoef)) : 1.f;
}

__global__ void muon_momentum_kernel(__nv_bfloat16* __restrict__ buf, const long long* __restrict__ grad_ptrs,
                                     float* __restrict__ sumsq, long long numel, float mu,
                                     const float* __restrict__ gcoef) {
  const float gc = muon_gcoef(gcoef);
  const int mi = blockIdx.y;
  __nv_bfloat16* b = buf + (long long)mi * numel;
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(grad_ptrs[mi]);
  const long long nvec = numel / 8;
  float sq = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    float bv[8], gv[8];
    unpack8(*(reinterpret_cast<const uint4*>(b) + i), bv);
    unpack8(*(reinterpret_cast<const uint4*>(g) + i), gv);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float gj = gcoef != nullptr ? __bfloat162float(__float2bfloat16(gv[j] * gc)) : gv[j];
      bv[j] = mu * bv[j] + gj;
    }
    const uint4 o = pack8(bv);
    *(reinterpret_cast<uint4*>(b) + i) = o;
    float rv[8];
    unpack8(o, rv);                      // the norm of what is stored (bf16-rounded), as the GEMMs will see it
#pragma unroll
    for (int j = 0; j < 8; ++j) sq += rv[j] * rv[j];
  }
  sq = warp_sum(sq);
  __shared__ float s[32];
  if ((threadIdx.x & 31) == 0) s[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? s[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) atomicAdd(&sumsq[mi], t);
  }
}

__global__ void muon_apply_kernel(__nv_bfloat16* __restrict__ buf, const __nv_bfloat16* __restrict__ ortho,
                                  const long long* __restrict__ grad_ptrs, const long long* __restrict__ param_ptrs,
                                  long long numel, float lr, float mu, float wd, int nesterov,
                                  const float* __restrict__ gcoef) {
  const float gc = muon_gcoef(gcoef);
  const int mi = blockIdx.y;
  __nv_bfloat16* b = buf + (long long)mi * numel;
  const __nv_bfloat16* o = ortho + (long long)mi * numel;
  const __nv_bfloat16* g = reinterpret_cast<const __nv_bfloat16*>(grad_ptrs[mi]);
  __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(param_ptrs[mi]);
  const long long nvec = numel / 8;
  const float decay = 1.f - lr * wd;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nvec;
       i += (long long)gridDim.x * blockDim.x) {
    const uint4 ov = *(reinterpret_cast<const uint4*>(o) + i);
    float of[8], gf[8], pf[8];
    unpack8(ov, of);
    unpack8(*(reinterpret_cast<const uint4*>(p) + i), pf);
    if (nesterov) {
      unpack8(*(reinterpret_cast<const uint4*>(g) + i), gf);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        // same rounding points as the unfused sequence: p*decay -> bf16, g + mu*o -> bf16, then the update
        const float pd = __bfloat162float(__float2bfloat16(pf[j] * decay));
        const float gj = gcoef != nullptr ? __bfloat162float(__float2bfloat16(gf[j] * gc)) : gf[j];
        const float up = __bfloat162float(__float2bfloat16(gj + mu * of[j]));
        pf[j] = pd - lr * up;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) pf[j] = __bfloat162float(__float2bfloat16(pf[j] * decay)) - lr * of[j];
    }
    *(reinterpret_cast<uint4*>(p) + i) = pack8(pf);
    *(reinterpret_cast<uint4*>(b) + i) = ov;
  }
}

}  // namespace kmoe

// ------------------------------------------------------------ int8 momentum (Muon8bit)
// Block-wise absmax int8: q = rint(x / s * 127), s = max(|x| over the block, 1e-8); one CTA per block.
// Elements past n (the padding of the last block) are written as 0.  Divisions are IEEE so that the
// result matches the same formula evaluated by PyTorch.
template <typename T>
__device__ __forceinline__ float q8_load(const T* p, long long i);
template <>
__device__ __forceinline__ float q8_load<float>(const float* p, long long i) { return p[i]; }
template <>
__device__ __forceinline__ float q8_load<__nv_bfloat16>(const __nv_bfloat16* p, long long i) { return __bfloat162float(p[i]); }
template <typename T>
__device__ __forceinline__ void q8_store(T* p, long long i, float v);
template <>
__device__ __forceinline__ void q8_store<float>(float* p, long long i, float v) { p[i] = v; }
template <>
__device__ __forceinline__ void q8_store<__nv_bfloat16>(__nv_bfloat16* p, long long i, float v) { p[i] = __float2bfloat16(v); }

template <typename T>
__global__ void q8_quant_kernel(const T* __restrict__ x, signed char* __restrict__ q, float* __restrict__ scales,
                                long long n, int block) {
  __shared__ float red[32];
  const long long base = (long long)blockIdx.x * block;
  float m = 0.f;
  for (int i = threadIdx.x; i < block; i += blockDim.x) {
    const long long j = base + i;
    if (j < n) m = fmaxf(m, fabsf(q8_load<T>(x, j)));
  }
  m = warp_max(m);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    v = warp_max(v);
    if (threadIdx.x == 0) red[0] = fmaxf(v, 1e-8f);
  }
  __syncthreads();
  const float s = red[0];
  if (threadIdx.x == 0) scales[blockIdx.x] = s;
  for (int i = threadIdx.x; i < block; i += blockDim.x) {
    const long long j = base + i;
    const float v = j < n ? q8_load<T>(x, j) : 0.f;
    q[j] = (signed char)__float2int_rn(__fmul_rn(__fdiv_rn(v, s), 127.f));
  }
}

// out = mu * dequant(q) + g   (the momentum update on the dequantised buffer), n elements
template <typename T>
__global__ void q8_momentum_kernel(const signed char* __restrict__ q, const float* __restrict__ scales,
                                   const T* __restrict__ g, T* __restrict__ out, long long n, int block, float mu) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    // the stored buffer is rounded to the parameter's type before the update, as the eager path does
    // q / 127 as PyTorch evaluates a division by a host scalar: a multiplication by its reciprocal
    float d = __fmul_rn(__fmul_rn((float)q[i], 1.0f / 127.0f), scales[i / block]);
    T tmp;
    q8_store<T>(&tmp, 0, d);
    d = q8_load<T>(&tmp, 0);
    q8_store<T>(&tmp, 0, __fmul_rn(d, mu));
    d = q8_load<T>(&tmp, 0);
    q8_store<T>(out, i, d + q8_load<T>(g, i));
  }
}

extern "C" int kmoe_q8_quant(const void* x, int is_bf16, signed char* q, float* scales, long long n, int block,
                             cudaStream_t st) {
  if (block < 32 || n <= 0) return -1;
  const long long nb = (n + block - 1) / block;
  if (is_bf16)
    q8_quant_kernel<__nv_bfloat16><<<(unsigned)nb, 256, 0, st>>>((const __nv_bfloat16*)x, q, scales, n, block);
  else
    q8_quant_kernel<float><<<(unsigned)nb, 256, 0, st>>>((const float*)x, q, scales, n, block);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_q8_momentum(const signed char* q, const float* scales, const void* g, int is_bf16, void* out,
                                long long n, int block, float mu, cudaStream_t st) {
  if (block < 32 || n <= 0) return -1;
  const int grid = grid_for(n, 256);
  if (is_bf16)
    q8_momentum_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(q, scales, (const __nv_bfloat16*)g, (__nv_bfloat16*)out, n,
                                                            block, mu);
  else
    q8_momentum_kernel<float><<<grid, 256, 0, st>>>(q, scales, (const float*)g, (float*)out, n, block, mu);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_muon_momentum(void* buf, const long long* grad_ptrs, float* sumsq, int n_mat, long long numel,
                                  float mu, const float* gcoef, cudaStream_t st) {
  if (numel % 8 || n_mat <= 0 || n_mat > 65535) return -1;
  const long long per = (numel / 8 + 255) / 256;
  const long long cap = 2368 / n_mat > 64 ? 2368 / n_mat : 64;      // ~16 CTAs per SM over all matrices
  dim3 grid((unsigned)(per < cap ? per : cap), n_mat);
  kmoe::muon_momentum_kernel<<<grid, 256, 0, st>>>((__nv_bfloat16*)buf, grad_ptrs, sumsq, numel, mu, gcoef);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_muon_apply(void* buf, const void* ortho, const long long* grad_ptrs, const long long* param_ptrs,
                               int n_mat, long long numel, float lr, float mu, float wd, int nesterov,
                               const float* gcoef, cudaStream_t st) {
  if (numel % 8 || n_mat <= 0 || n_mat > 65535) return -1;
  const long long per = (numel / 8 + 255) / 256;
  const long long cap = 2368 / n_mat > 64 ? 2368 / n_mat : 64;
  dim3 grid((unsigned)(per < cap ? per : cap), n_mat);
  kmoe::muon_apply_kernel<<<grid, 256, 0, st>>>((__nv_bfloat16*)buf, (const __nv_bfloat16*)ortho, grad_ptrs, param_ptrs,
                                                numel, lr, mu, wd, nesterov, gcoef);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
