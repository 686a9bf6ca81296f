// MXFP8 quantisation (OCP microscaling): e4m3 values with one e8m0 power-of-two scale per 32
// consecutive elements of the reduction dimension; scale = 2^(floor(log2(amax)) - 8).
//
// The block-scaled tensor-core instruction reads its scale factors from TMEM in a fixed arrangement:
// for a block of 128 operand rows and 4 consecutive 32-element groups (128 reduction elements) the
// 512 scale bytes sit at
//        (row % 32) * 16 + ((row % 128) / 32) * 4 + (k_group % 4)
// so that one 32-lane x 16-byte shared->tensor-memory copy delivers them.  The kernels here write the
// scales directly in that arrangement - chunk index (row / 128) * (K / 128) + k / 128, 512 bytes per
// chunk - so the GEMM moves each chunk with one bulk copy and never shuffles it.
//
//   quant_rows  : x (R, C) bf16, reduction along C     -> q (R, C)  e4m3, scales for rows R
//   quant_cols  : x (R, C) bf16, reduction along R     -> q (C, R)  e4m3 (transposed, so the reduction
//                 dimension is contiguous for the tensor core), scales for rows C
//   swiglu_quant: h = silu(g) * u, then quant_rows of h; h itself is never stored
// All take a leading batch (expert) dimension.  The reference's "FP8" experts clamp and multiply in
// bf16 (moe_arch/model/fp8_moe.py:247-266); there is no counterpart kernel.
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

__device__ __forceinline__ int mx_scale_exp(float amax) {
  // floor(log2(amax)) - 8 clamped to [-127, 127]; amax == 0 maps to the smallest scale
  const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 127;   // exact for normal floats
  return max(-127, min(127, e - 8));
}

__device__ __forceinline__ uint8_t to_e4m3(float v) {
  return (uint8_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}

__device__ __forceinline__ size_t sf_offset(long long row, long long kgroup32, long long k_chunks) {
  const long long chunk = (row >> 7) * k_chunks + (kgroup32 >> 2);
  return (size_t)chunk * 512 + (row & 31) * 16 + ((row & 127) >> 5) * 4 + (kgroup32 & 3);
}

// one thread per 32-element block; MODE 0: plain rows, MODE 1: silu(g) * u
template <int MODE>
__global__ void mx_quant_rows_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ x2,
                                     long long rows, int C, long long ld, uint8_t* __restrict__ q,
                                     uint8_t* __restrict__ sf, const int* __restrict__ live_rows) {
  const int blocks_per_row = C / 32;
  const long long nrows = live_rows ? min((long long)*live_rows, rows) : rows;
  const long long total = nrows * blocks_per_row;
  for (long long b = blockIdx.x * (long long)blockDim.x + threadIdx.x; b < total;
       b += (long long)gridDim.x * blockDim.x) {
    const long long r = b / blocks_per_row;
    const int kb = (int)(b - r * blocks_per_row);
    const uint4* src = reinterpret_cast<const uint4*>(x + r * ld + kb * 32);
    float v[32];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 w = src[i];
      const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(p[j]);
        v[i * 8 + 2 * j] = f.x;
        v[i * 8 + 2 * j + 1] = f.y;
      }
    }
    if (MODE == 1) {
      const uint4* src2 = reinterpret_cast<const uint4*>(x2 + r * ld + kb * 32);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint4 w = src2[i];
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&w);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __bfloat1622float2(p[j]);
          // the product is rounded to bf16 first so the values match an unfused SwiGLU followed by quantisation
          v[i * 8 + 2 * j] = __bfloat162float(__float2bfloat16(silu_f(v[i * 8 + 2 * j]) * f.x));
          v[i * 8 + 2 * j + 1] = __bfloat162float(__float2bfloat16(silu_f(v[i * 8 + 2 * j + 1]) * f.y));
        }
      }
    }
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) amax = fmaxf(amax, fabsf(v[i]));
    const int e = mx_scale_exp(amax);
    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);     // 2^-e, e in [-127,127] -> exponent field 0..254
    uint32_t out[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      out[i] = (uint32_t)to_e4m3(v[4 * i] * inv) | ((uint32_t)to_e4m3(v[4 * i + 1] * inv) << 8) |
               ((uint32_t)to_e4m3(v[4 * i + 2] * inv) << 16) | ((uint32_t)to_e4m3(v[4 * i + 3] * inv) << 24);
    }
    uint4* dst = reinterpret_cast<uint4*>(q + r * (long long)C + kb * 32);
    dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
    dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
    sf[sf_offset(r, kb, C / 128)] = (uint8_t)(e + 127);
  }
}

// x (G, R, C) -> q (G, C, R).  Block: 32 reduction rows x 128 columns; thread c owns column c of the tile.
__global__ void mx_quant_cols_kernel(const __nv_bfloat16* __restrict__ x, long long R, int C, long long ld,
                                     long long g_stride, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                     const int* __restrict__ live_rows) {
  __shared__ __nv_bfloat16 tile[32][128 + 8];
  const int g = blockIdx.z;
  const long long r0 = (long long)blockIdx.y * 32;
  const int c0 = blockIdx.x * 128;
  const long long nrows = live_rows ? min((long long)*live_rows, R) : R;
  if (r0 >= nrows) return;                               // rows past the live range are never read by the GEMM
  const __nv_bfloat16* xg = x + (long long)g * g_stride;
  // 32 rows x 128 cols = 512 vectors of 8; 128 threads load 4 each
  for (int v = threadIdx.x; v < 32 * 16; v += blockDim.x) {
    const int rr = v >> 4, cv = (v & 15) * 8;
    uint4 w = make_uint4(0, 0, 0, 0);
    if (r0 + rr < R && c0 + cv < C) w = *reinterpret_cast<const uint4*>(xg + (r0 + rr) * ld + c0 + cv);
    *reinterpret_cast<uint4*>(&tile[rr][cv]) = w;
  }
  __syncthreads();
  const int c = c0 + threadIdx.x;
  if (c >= C) return;
  float v[32];
  float amax = 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    v[i] = __bfloat162float(tile[i][threadIdx.x]);
    amax = fmaxf(amax, fabsf(v[i]));
  }
  const int e = mx_scale_exp(amax);
  const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
  uint32_t out[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[i] = (uint32_t)to_e4m3(v[4 * i] * inv) | ((uint32_t)to_e4m3(v[4 * i + 1] * inv) << 8) |
             ((uint32_t)to_e4m3(v[4 * i + 2] * inv) << 16) | ((uint32_t)to_e4m3(v[4 * i + 3] * inv) << 24);
  }
  const long long rows_out = (long long)gridDim.z * C;           // scale rows: (g, c) flattened
  (void)rows_out;
  uint4* dst = reinterpret_cast<uint4*>(q + ((long long)g * C + c) * R + r0);
  dst[0] = make_uint4(out[0], out[1], out[2], out[3]);
  dst[1] = make_uint4(out[4], out[5], out[6], out[7]);
  sf[sf_offset((long long)g * C + c, r0 >> 5, R / 128)] = (uint8_t)(e + 127);
}

}  // namespace kmoe

using namespace kmoe;

extern "C" long long kmoe_mx_sf_bytes(long long rows, long long K) {
  return ((rows + 127) / 128) * (K / 128) * 512;
}

extern "C" int kmoe_mx_quant_rows(const void* x, const void* x2, long long rows, int C, long long ld, void* q, void* sf,
                                  const int* live_rows, cudaStream_t st) {
  if (C % 128 != 0 || ld % 8 != 0) return -1;
  if (rows == 0) return 0;
  const long long total = rows * (C / 32);
  const long long want = (total + 255) / 256;
  const int grid = (int)(want < 148 * 16 ? want : 148 * 16);
  if (x2 == nullptr)
    mx_quant_rows_kernel<0><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, nullptr, rows, C, ld, (uint8_t*)q,
                                                  (uint8_t*)sf, live_rows);
  else
    mx_quant_rows_kernel<1><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)x2, rows, C, ld,
                                                  (uint8_t*)q, (uint8_t*)sf, live_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_mx_quant_cols(const void* x, int groups, long long R, int C, long long ld, long long g_stride,
                                  void* q, void* sf, const int* live_rows, cudaStream_t st) {
  // R is the reduction dimension of the output; the per-group output rows (C) must tile by 128 so that
  // groups do not share a scale chunk
  if (R % 128 != 0 || ld % 8 != 0 || C % 8 != 0 || (groups > 1 && C % 128 != 0)) return -1;
  if (R == 0 || C == 0) return 0;
  dim3 grid((C + 127) / 128, (unsigned)(R / 32), groups);
  if (grid.y > 65535 || grid.z > 65535) return -3;
  mx_quant_cols_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, R, C, ld, g_stride, (uint8_t*)q, (uint8_t*)sf,
                                             live_rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
