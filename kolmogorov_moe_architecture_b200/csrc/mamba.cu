// Mamba kernels, channels-last: depthwise causal conv1d (+SiLU) and the selective scan,
// forward and backward.  Activations are bf16 [B, S, C] (row strides allowed where a
// tensor is a column slice of a fused projection); the small per-channel parameters
// (conv taps, bias, A, D, dt bias) and the per-step B/C vectors are fp32.
//
// Scan mapping: one thread per channel holding the N (=16) states in registers;
// consecutive threads own consecutive channels so every per-step load is coalesced.
// The 16 state recurrences are independent, which gives the ILP that hides the
// fma/ex2 latency at the low occupancy this mapping has.  Forward stores the state at
// every CHUNK-th step; backward replays one chunk at a time from that checkpoint into
// shared memory and then walks it in reverse.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int SCAN_N = 16;      // state size
constexpr int SCAN_CHUNK = 16;  // checkpoint interval
constexpr int SCAN_THREADS = 64;

__device__ __forceinline__ float bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.f / (1.f + __expf(-x)); }

// ------------------------------------------------------------------ conv1d
// y[b,t,c] = act(bias[c] + sum_j w[c,j] * x[b, t-(W-1)+j, c]),  W = 4
constexpr int CONV_W = 4;
constexpr int CONV_T = 64;  // time steps per thread

__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, __nv_bfloat16* __restrict__ y, int S, int C,
                                  long long ldx, int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_T;
  const float w0 = w[c * 4 + 0], w1 = w[c * 4 + 1], w2 = w[c * 4 + 2], w3 = w[c * 4 + 3];
  const float bs = bias ? bias[c] : 0.f;
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
                                  int S, int C, long long ldx, int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * CONV_T;
  const float w0 = w[c * 4 + 0], w1 = w[c * 4 + 1], w2 = w[c * 4 + 2], w3 = w[c * 4 + 3];
  const float bs = bias ? bias[c] : 0.f;
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
  // dx for the first three steps of this chunk needs dpre of t0..t0+2 only through later taps; the loop
  // above starts its dpre window empty, which is exact because dx[td >= t0] never reads dpre[< t0].
  atomicAdd(&dw[c * 4 + 0], aw0);
  atomicAdd(&dw[c * 4 + 1], aw1);
  atomicAdd(&dw[c * 4 + 2], aw2);
  atomicAdd(&dw[c * 4 + 3], aw3);
  if (dbias) atomicAdd(&dbias[c], ab);
}

// ----------------------------------------------------------- selective scan
struct ScanArgs {
  const __nv_bfloat16* u;      // [B,S,C]
  const __nv_bfloat16* delta;  // [B,S,C]
  const __nv_bfloat16* z;      // [B,S,*] ld = ldz, may be null
  const float* A;              // [C,N]
  const float* Bm;             // [B,S,N]
  const float* Cm;             // [B,S,N]
  const float* D;              // [C] or null
  const float* dt_bias;        // [C] or null
  int S, C;
  long long ldz;
  int softplus;
};

__global__ void __launch_bounds__(SCAN_THREADS)
scan_fwd_kernel(ScanArgs a, __nv_bfloat16* __restrict__ out, float* __restrict__ ckpt /*[B, S/CHUNK, N, C]*/) {
  const int c = blockIdx.x * SCAN_THREADS + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= a.C) return;
  float An[SCAN_N], h[SCAN_N];
#pragma unroll
  for (int n = 0; n < SCAN_N; ++n) {
    An[n] = a.A[c * SCAN_N + n] * 1.4426950408889634f;  // exp(x) = 2^(x log2 e)
    h[n] = 0.f;
  }
  const float Dc = a.D ? a.D[c] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[c] : 0.f;
  const size_t base = (size_t)b * a.S * a.C + c;
  const __nv_bfloat16* up = a.u + base;
  const __nv_bfloat16* dp = a.delta + base;
  const __nv_bfloat16* zp = a.z ? a.z + (size_t)b * a.S * a.ldz + c : nullptr;
  const float* Bp = a.Bm + (size_t)b * a.S * SCAN_N;
  const float* Cp = a.Cm + (size_t)b * a.S * SCAN_N;
  __nv_bfloat16* op = out + base;
  const int nchunks = (a.S + SCAN_CHUNK - 1) / SCAN_CHUNK;
  for (int ch = 0; ch < nchunks; ++ch) {
    if (ckpt != nullptr) {
      float* ck = ckpt + (((size_t)b * nchunks + ch) * SCAN_N) * a.C + c;
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) ck[(size_t)n * a.C] = h[n];
    }
    const int t0 = ch * SCAN_CHUNK;
    float uu[SCAN_CHUNK], dd[SCAN_CHUNK], zz[SCAN_CHUNK];
#pragma unroll
    for (int i = 0; i < SCAN_CHUNK; ++i) {
      const int t = t0 + i;
      const bool ok = t < a.S;
      uu[i] = ok ? bf2f(up[(size_t)t * a.C]) : 0.f;
      dd[i] = ok ? bf2f(dp[(size_t)t * a.C]) : 0.f;
      zz[i] = (ok && zp) ? bf2f(zp[(size_t)t * a.ldz]) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < SCAN_CHUNK; ++i) {
      const int t = t0 + i;
      if (t >= a.S) break;
      float dt = dd[i] + bias;
      if (a.softplus) dt = softplus_f(dt);
      const float4* B4 = reinterpret_cast<const float4*>(Bp + (size_t)t * SCAN_N);
      const float4* C4 = reinterpret_cast<const float4*>(Cp + (size_t)t * SCAN_N);
      float Bv[SCAN_N], Cv[SCAN_N];
#pragma unroll
      for (int q = 0; q < SCAN_N / 4; ++q) {
        const float4 bq = __ldg(B4 + q), cq = __ldg(C4 + q);
        Bv[4 * q] = bq.x; Bv[4 * q + 1] = bq.y; Bv[4 * q + 2] = bq.z; Bv[4 * q + 3] = bq.w;
        Cv[4 * q] = cq.x; Cv[4 * q + 1] = cq.y; Cv[4 * q + 2] = cq.z; Cv[4 * q + 3] = cq.w;
      }
      const float dtu = dt * uu[i];
      float y = 0.f;
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) {
        h[n] = exp2f(dt * An[n]) * h[n] + dtu * Bv[n];
        y += Cv[n] * h[n];
      }
      y += Dc * uu[i];
      if (zp) y *= silu_f(zz[i]);
      op[(size_t)t * a.C] = __float2bfloat16(y);
    }
  }
}

// Sum `v[0..15]` across the 32 lanes; lane l (< 16) ends with the total of element l.
__device__ __forceinline__ float warp_reduce_scatter16(float (&v)[SCAN_N], int lane) {
  // step 1: lanes exchange halves of the 16 values with lane^16
  float r8[8];
  {
    const bool hi = lane & 16;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float send = hi ? v[i] : v[i + 8];
      const float keep = hi ? v[i + 8] : v[i];
      r8[i] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
    }
  }  // lanes with bit4=0 hold elements 0..7, bit4=1 hold 8..15
  float r4[4];
  {
    const bool hi = lane & 8;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float send = hi ? r8[i] : r8[i + 4];
      const float keep = hi ? r8[i + 4] : r8[i];
      r4[i] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
    }
  }
  float r2[2];
  {
    const bool hi = lane & 4;
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const float send = hi ? r4[i] : r4[i + 2];
      const float keep = hi ? r4[i + 2] : r4[i];
      r2[i] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
  }
  float r1;
  {
    const bool hi = lane & 2;
    const float send = hi ? r2[0] : r2[1];
    const float keep = hi ? r2[1] : r2[0];
    r1 = keep + __shfl_xor_sync(0xffffffffu, send, 2);
  }
  r1 += __shfl_xor_sync(0xffffffffu, r1, 1);
  // element index held by this lane: bit4 -> 8, bit3 -> 4, bit2 -> 2, bit1 -> 1
  return r1;
}
__device__ __forceinline__ int reduce_scatter16_index(int lane) {
  return ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
}

__global__ void __launch_bounds__(SCAN_THREADS)
scan_bwd_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ ckpt,
                __nv_bfloat16* __restrict__ du, __nv_bfloat16* __restrict__ ddelta, __nv_bfloat16* __restrict__ dz,
                long long lddz, float* __restrict__ dA, float* __restrict__ dB, float* __restrict__ dC,
                float* __restrict__ dD, float* __restrict__ dbias) {
  extern __shared__ float hs[];  // [SCAN_CHUNK + 1][SCAN_N][SCAN_THREADS]; slot 0 = state before the chunk
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int c = blockIdx.x * SCAN_THREADS + tid;
  const int b = blockIdx.y;
  const bool live = c < a.C;
  const int cc = live ? c : a.C - 1;
  float An[SCAN_N], g[SCAN_N], dAacc[SCAN_N];
#pragma unroll
  for (int n = 0; n < SCAN_N; ++n) {
    An[n] = a.A[cc * SCAN_N + n];
    g[n] = 0.f;
    dAacc[n] = 0.f;
  }
  const float Dc = a.D ? a.D[cc] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[cc] : 0.f;
  float dDacc = 0.f, dbacc = 0.f;
  const size_t base = (size_t)b * a.S * a.C + cc;
  const __nv_bfloat16* up = a.u + base;
  const __nv_bfloat16* dp = a.delta + base;
  const __nv_bfloat16* zp = a.z ? a.z + (size_t)b * a.S * a.ldz + cc : nullptr;
  const __nv_bfloat16* gp = dout + base;
  const float* Bp = a.Bm + (size_t)b * a.S * SCAN_N;
  const float* Cp = a.Cm + (size_t)b * a.S * SCAN_N;
  const int nchunks = (a.S + SCAN_CHUNK - 1) / SCAN_CHUNK;
#define HS(t, n) hs[((t) * SCAN_N + (n)) * SCAN_THREADS + tid]
  for (int ch = nchunks - 1; ch >= 0; --ch) {
    const int t0 = ch * SCAN_CHUNK;
    const int len = min(SCAN_CHUNK, a.S - t0);
    const float* ck = ckpt + (((size_t)b * nchunks + ch) * SCAN_N) * a.C + cc;
    float h[SCAN_N];
#pragma unroll
    for (int n = 0; n < SCAN_N; ++n) {
      h[n] = ck[(size_t)n * a.C];
      HS(0, n) = h[n];
    }
    float uu[SCAN_CHUNK], dt_[SCAN_CHUNK];
    // replay forward, keeping every state of the chunk
#pragma unroll
    for (int i = 0; i < SCAN_CHUNK; ++i) {
      if (i >= len) break;
      const int t = t0 + i;
      uu[i] = bf2f(up[(size_t)t * a.C]);
      float dt = bf2f(dp[(size_t)t * a.C]) + bias;
      if (a.softplus) dt = softplus_f(dt);
      dt_[i] = dt;
      const float4* B4 = reinterpret_cast<const float4*>(Bp + (size_t)t * SCAN_N);
      const float dtu = dt * uu[i];
#pragma unroll
      for (int q = 0; q < SCAN_N / 4; ++q) {
        const float4 bq = __ldg(B4 + q);
        const float bv[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = 4 * q + j;
          h[n] = __expf(dt * An[n]) * h[n] + dtu * bv[j];
          HS(i + 1, n) = h[n];
        }
      }
    }
    // reverse sweep
#pragma unroll
    for (int i = SCAN_CHUNK - 1; i >= 0; --i) {
      if (i >= len) continue;
      const int t = t0 + i;
      const float dt = dt_[i], u = uu[i];
      const float go = live ? bf2f(gp[(size_t)t * a.C]) : 0.f;
      const float4* B4 = reinterpret_cast<const float4*>(Bp + (size_t)t * SCAN_N);
      const float4* C4 = reinterpret_cast<const float4*>(Cp + (size_t)t * SCAN_N);
      float Bv[SCAN_N], Cv[SCAN_N];
#pragma unroll
      for (int q = 0; q < SCAN_N / 4; ++q) {
        const float4 bq = __ldg(B4 + q), cq = __ldg(C4 + q);
        Bv[4 * q] = bq.x; Bv[4 * q + 1] = bq.y; Bv[4 * q + 2] = bq.z; Bv[4 * q + 3] = bq.w;
        Cv[4 * q] = cq.x; Cv[4 * q + 1] = cq.y; Cv[4 * q + 2] = cq.z; Cv[4 * q + 3] = cq.w;
      }
      // y before gating (needed for dz)
      float ypre = Dc * u;
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) ypre += Cv[n] * HS(i + 1, n);
      float dy = go;
      if (zp) {
        const float zv = bf2f(zp[(size_t)t * a.ldz]);
        const float sg = sigmoid_f(zv);
        if (live) dz[(size_t)b * a.S * lddz + (size_t)t * lddz + cc] = __float2bfloat16(go * ypre * sg * (1.f + zv * (1.f - sg)));
        dy = go * zv * sg;
      }
      dDacc += dy * u;
      float du_v = dy * Dc;
      float ddt = 0.f;
      float dBv[SCAN_N], dCv[SCAN_N];
#pragma unroll
      for (int n = 0; n < SCAN_N; ++n) {
        const float hprev = HS(i, n);
        const float hcur = HS(i + 1, n);
        dCv[n] = dy * hcur;
        g[n] += Cv[n] * dy;                       // adjoint of h_t
        const float dA_t = __expf(dt * An[n]);
        const float gh = g[n] * hprev * dA_t;     // d/d(dt*A)
        ddt += gh * An[n] + g[n] * Bv[n] * u;
        dAacc[n] += gh * dt;
        dBv[n] = g[n] * dt * u;
        du_v += g[n] * dt * Bv[n];
        g[n] *= dA_t;                             // carry to step t-1
      }
      float dd = ddt;
      if (a.softplus) dd *= sigmoid_f(bf2f(dp[(size_t)t * a.C]) + bias);
      dbacc += dd;
      if (live) {
        du[base + (size_t)t * a.C] = __float2bfloat16(du_v);
        ddelta[base + (size_t)t * a.C] = __float2bfloat16(dd);
      }
      const float sB = warp_reduce_scatter16(dBv, lane);
      const float sC = warp_reduce_scatter16(dCv, lane);
      if ((lane & 1) == 0) {
        const int n = reduce_scatter16_index(lane);
        atomicAdd(&dB[((size_t)b * a.S + t) * SCAN_N + n], sB);
        atomicAdd(&dC[((size_t)b * a.S + t) * SCAN_N + n], sC);
      }
    }
  }
#undef HS
  if (live) {
#pragma unroll
    for (int n = 0; n < SCAN_N; ++n) atomicAdd(&dA[c * SCAN_N + n], dAacc[n]);
    if (dD) atomicAdd(&dD[c], dDacc);
    if (dbias) atomicAdd(&dbias[c], dbacc);
  }
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_conv1d_fwd(const void* x, const float* w, const float* bias, void* y, int B, int S, int C,
                               long long ldx, int act, cudaStream_t st) {
  dim3 grid((C + 127) / 128, (S + CONV_T - 1) / CONV_T, B);
  conv1d_fwd_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias, (__nv_bfloat16*)y, S, C, ldx, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_conv1d_bwd(const void* x, const float* w, const float* bias, const void* dy, void* dx, float* dw,
                               float* dbias, int B, int S, int C, long long ldx, int act, cudaStream_t st) {
  dim3 grid((C + 127) / 128, (S + CONV_T - 1) / CONV_T, B);
  conv1d_bwd_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias, (const __nv_bfloat16*)dy,
                                          (__nv_bfloat16*)dx, dw, dbias, S, C, ldx, act);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_scan_chunk(void) { return SCAN_CHUNK; }

extern "C" int kmoe_scan_fwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, void* out, float* ckpt, int B,
                             int S, int C, int N, long long ldz, int softplus, cudaStream_t st) {
  if (N != SCAN_N) return -1;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus};
  dim3 grid((C + SCAN_THREADS - 1) / SCAN_THREADS, B);
  scan_fwd_kernel<<<grid, SCAN_THREADS, 0, st>>>(a, (__nv_bfloat16*)out, ckpt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dA [C,N], dB/dC [B,S,N], dD [C], dbias [C] are fp32 and must be zeroed by the caller.
extern "C" int kmoe_scan_bwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, const void* dout,
                             const float* ckpt, void* du, void* ddelta, void* dz, long long lddz, float* dA, float* dB,
                             float* dC, float* dD, float* dbias, int B, int S, int C, int N, long long ldz,
                             int softplus, cudaStream_t st) {
  if (N != SCAN_N) return -1;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus};
  const int smem = (SCAN_CHUNK + 1) * SCAN_N * SCAN_THREADS * sizeof(float);
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    attr = true;
  }
  dim3 grid((C + SCAN_THREADS - 1) / SCAN_THREADS, B);
  scan_bwd_kernel<<<grid, SCAN_THREADS, smem, st>>>(a, (const __nv_bfloat16*)dout, ckpt, (__nv_bfloat16*)du,
                                                    (__nv_bfloat16*)ddelta, (__nv_bfloat16*)dz, lddz, dA, dB, dC, dD,
                                                    dbias);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
