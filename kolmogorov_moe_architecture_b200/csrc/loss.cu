// Cross-entropy over a bf16 logits tile with the gradient written in place.
//
// The LM-head + MTP loss is evaluated head by head and row-chunk by row-chunk:
// logits = H W^T (tcgen05 GEMM), then this kernel turns the chunk into
// d(loss)/d(logits) in place while producing the per-row losses, then two more
// GEMMs consume the gradient chunk.  The chunk is the only (rows, V) tensor that
// ever exists.  One CTA per row; fp32 online max / sum-exp; second pass hits L2.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int CE_THREADS = 256;

__device__ __forceinline__ void merge_ms(float& m, float& s, float m2, float s2) {
  if (m2 == -INFINITY) return;
  if (m == -INFINITY) {
    m = m2;
    s = s2;
    return;
  }
  const float mn = fmaxf(m, m2);
  s = s * __expf(m - mn) + s2 * __expf(m2 - mn);
  m = mn;
}

// logits [R, V] (ld), labels [R] int64 (already shifted / masked; ignore_index rows give zero loss and gradient)
// loss_rows [R] fp32 ; if write_grad: logits <- (softmax - onehot) * (*grad_scale)
__global__ void __launch_bounds__(CE_THREADS)
ce_fwd_bwd_kernel(__nv_bfloat16* __restrict__ logits, const long long* __restrict__ labels,
                  float* __restrict__ loss_rows, const float* __restrict__ grad_scale, int V, long long ld,
                  long long ignore_index, int write_grad) {
  __shared__ float sm[CE_THREADS / 32], ss[CE_THREADS / 32];
  __shared__ float s_max, s_sum;
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (size_t)row * ld;
  const long long label = labels[row];
  const bool ignored = (label == ignore_index) || label < 0 || label >= V;
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const int vec = V / 8;
  if (ignored) {
    if (tid == 0) loss_rows[row] = 0.f;
    if (write_grad) {
      for (int v = tid; v < vec; v += CE_THREADS) reinterpret_cast<uint4*>(lr)[v] = make_uint4(0, 0, 0, 0);
      for (int c = vec * 8 + tid; c < V; c += CE_THREADS) lr[c] = __float2bfloat16(0.f);
    }
    return;
  }
  float m = -INFINITY, s = 0.f;
  for (int v = tid; v < vec; v += CE_THREADS) {
    uint4 r = reinterpret_cast<const uint4*>(lr)[v];
    const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&r);
    float x[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(p[i]);
      x[2 * i] = f.x;
      x[2 * i + 1] = f.y;
    }
    float mx = x[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) mx = fmaxf(mx, x[i]);
    const float mn = fmaxf(m, mx);
    float acc = s * __expf(m - mn);
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += __expf(x[i] - mn);
    m = mn;
    s = acc;
  }
  for (int c = vec * 8 + tid; c < V; c += CE_THREADS) merge_ms(m, s, __bfloat162float(lr[c]), 1.f);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float m2 = __shfl_xor_sync(0xffffffffu, m, o), s2 = __shfl_xor_sync(0xffffffffu, s, o);
    merge_ms(m, s, m2, s2);
  }
  if (lane == 0) { sm[wid] = m; ss[wid] = s; }
  __syncthreads();
  if (tid == 0) {
    float M = sm[0], S = ss[0];
    for (int w = 1; w < CE_THREADS / 32; ++w) merge_ms(M, S, sm[w], ss[w]);
    s_max = M;
    s_sum = S;
    loss_rows[row] = (M + __logf(S)) - __bfloat162float(lr[label]);
  }
  __syncthreads();
  if (!write_grad) return;
  const float M = s_max, inv = 1.f / s_sum, gs = *grad_scale;
  for (int v = tid; v < vec; v += CE_THREADS) {
    uint4 r = reinterpret_cast<const uint4*>(lr)[v];
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&r);
    const int c0 = v * 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(p[i]);
      float g0 = __expf(f.x - M) * inv, g1 = __expf(f.y - M) * inv;
      if (c0 + 2 * i == label) g0 -= 1.f;
      if (c0 + 2 * i + 1 == label) g1 -= 1.f;
      p[i] = __floats2bfloat162_rn(g0 * gs, g1 * gs);
    }
    reinterpret_cast<uint4*>(lr)[v] = r;
  }
  for (int c = vec * 8 + tid; c < V; c += CE_THREADS) {
    float g = __expf(__bfloat162float(lr[c]) - M) * inv;
    if (c == label) g -= 1.f;
    lr[c] = __float2bfloat16(g * gs);
  }
}

}  // namespace kmoe

extern "C" int kmoe_ce_fwd_bwd(void* logits, const long long* labels, float* loss_rows, const float* grad_scale,
                               int R, int V, long long ld, long long ignore_index, int write_grad, cudaStream_t st) {
  if (ld % 8) return -1;
  if (R <= 0) return 0;
  kmoe::ce_fwd_bwd_kernel<<<R, kmoe::CE_THREADS, 0, st>>>((__nv_bfloat16*)logits, labels, loss_rows, grad_scale, V, ld,
                                                          ignore_index, write_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
