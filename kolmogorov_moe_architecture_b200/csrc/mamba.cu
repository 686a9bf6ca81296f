// Mamba kernels, channels-last: depthwise causal conv1d (+SiLU), forward and backward (the selective
// scan lives in scan.cu).  Activations are bf16 [B, S, C] (row strides allowed where a
// tensor is a column slice of a fused projection); the small per-channel parameters
// (conv taps, bias, A, D, dt bias) and the per-step B/C vectors are fp32.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------ conv1d
// y[b,t,c] = act(bias[c] + sum_j w[c,j] * x[b, t-(W-1)+j, c]),  W = 4
constexpr int CONV_T = 64;  // time steps per thread

__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int S, int C,
                                  long long ldx, int act, int bpg) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_T;
  const int pc = (b / bpg) * C + c;   // parameter row: batch entries [g*bpg, (g+1)*bpg) use parameter set g
  const float w0 = w[pc * 4 + 0], w1 = w[pc * 4 + 1], w2 = w[pc * 4 + 2], w3 = w[pc * 4 + 3];
  const float bs = bias ? bias[pc] : 0.f;
  const __nv_bfloat16* xb = x + (size_t)b * S * ldx + c;
  __nv_bfloat16* yb = y + (size_t)b * S * C + c;
  float x0 = t0 >= 3 ? bf2f(xb[(size_t)(t0 - 3) * ldx]) : 0.f;
  float x1 = t0 >= 2 ? bf2f(xb[(size_t)(t0 - 2) * ldx]) : 0.f;
  float x2 = t0 >= 1 ? bf2f(xb[(size_t)(t0 - 1) * ldx]) : 0.f;
  const int t1 = min(t0 + CONV_T, S);
#pragma unroll 4
  for (int t = t0; t < t1; ++t) {
    const float x3 = bf2f(xb[(size_t)t * ldx]);
    float v = bs + w0 * x0 + w1 * x1 + w2 * x2 + w3 * x3;
    if (act) v = silu_f(v);
    yb[(size_t)t * C] = __float2bfloat16(v);
    x0 = x1; x1 = x2; x2 = x3;
  }
}

// dx, and atomically accumulated dw [C,4], dbias [C] (fp32, zeroed by the caller).
__global__ void conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dx, float* __restrict__ dw, float* __restrict__ dbias,
                                  int S, int C, long long ldx, int act, int bpg) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_T;
  const int pc = (b / bpg) * C + c;
  const float w0 = w[pc * 4 + 0], w1 = w[pc * 4 + 1], w2 = w[pc * 4 + 2], w3 = w[pc * 4 + 3];
  const float bs = bias ? bias[pc] : 0.f;
  const __nv_bfloat16* xb = x + (size_t)b * S * ldx + c;
  const __nv_bfloat16* gb = dy + (size_t)b * S * C + c;
  __nv_bfloat16* dxb = dx + (size_t)b * S * C + c;
  float x0 = t0 >= 3 ? bf2f(xb[(size_t)(t0 - 3) * ldx]) : 0.f;
  float x1 = t0 >= 2 ? bf2f(xb[(size_t)(t0 - 2) * ldx]) : 0.f;
  float x2 = t0 >= 1 ? bf2f(xb[(size_t)(t0 - 1) * ldx]) : 0.f;
  float p0 = 0.f, p1 = 0.f, p2 = 0.f;  // dpre[t-3], dpre[t-2], dpre[t-1]
  float aw0 = 0.f, aw1 = 0.f, aw2 = 0.f, aw3 = 0.f, ab = 0.f;
  const int t_own_end = min(t0 + CONV_T, S);
  const int t_end = t0 + CONV_T + 3;  // dx[t] needs dpre up to t+3
  for (int t = t0; t < t_end; ++t) {
    float p3 = 0.f, x3 = 0.f;
    if (t < S) {
      x3 = bf2f(xb[(size_t)t * ldx]);
      const float pre = bs + w0 * x0 + w1 * x1 + w2 * x2 + w3 * x3;
      float g = bf2f(gb[(size_t)t * C]);
      if (act) {
        const float sg = sigmoid_f(pre);
        g *= sg * (1.f + pre * (1.f - sg));
      }
      p3 = g;
      if (t < t_own_end) {
        aw0 += g * x0; aw1 += g * x1; aw2 += g * x2; aw3 += g * x3; ab += g;
      }
    }
    const int td = t - 3;  // dx[td] = w0 dpre[td+3] + w1 dpre[td+2] + w2 dpre[td+1] + w3 dpre[td]
    if (td >= t0 && td < t_own_end) {
      float v = w0 * p3 + w1 * p2 + w2 * p1 + w3 * p0;
      dxb[(size_t)td * C] = __float2bfloat16(v);
    }
    x0 = x1; x1 = x2; x2 = x3;
    p0 = p1; p1 = p2; p2 = p3;
  }
  // the dpre window starts empty, which is exact: dx[td >= t0] never reads dpre[< t0]
  atomicAdd(&dw[pc * 4 + 0], aw0);
  atomicAdd(&dw[pc * 4 + 1], aw1);
  atomicAdd(&dw[pc * 4 + 2], aw2);
  atomicAdd(&dw[pc * 4 + 3], aw3);
  if (dbias) atomicAdd(&dbias[pc], ab);
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_conv1d_fwd(const void* x, const float* w, const float* bias, void* y, int B, int S, int C,
                               long long ldx, int act, int groups, cudaStream_t st) {
  if (groups < 1 || B % groups) return -1;
  dim3 grid((C + 127) / 128, (S + CONV_T - 1) / CONV_T, B);
  conv1d_fwd_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias, (__nv_bfloat16*)y, S, C, ldx, act,
                                          B / groups);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_conv1d_bwd(const void* x, const float* w, const float* bias, const void* dy, void* dx, float* dw,
                               float* dbias, int B, int S, int C, long long ldx, int act, int groups,
                               cudaStream_t st) {
  if (groups < 1 || B % groups) return -1;
  dim3 grid((C + 127) / 128, (S + CONV_T - 1) / CONV_T, B);
  conv1d_bwd_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias, (const __nv_bfloat16*)dy,
                                          (__nv_bfloat16*)dx, dw, dbias, S, C, ldx, act, B / groups);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
