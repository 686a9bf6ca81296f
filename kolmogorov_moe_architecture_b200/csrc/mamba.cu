// Mamba kernels, channels-last: depthwise causal conv1d (+SiLU) and the selective scan,
// forward and backward.  Activations are bf16 [B, S, C] (row strides allowed where a
// tensor is a column slice of a fused projection); the small per-channel parameters
// (conv taps, bias, A, D, dt bias) and the per-step B/C vectors are fp32.
//
// Scan: a CTA owns 32 channels, a thread one channel and 4 of the N (=16) states; inputs
// are staged through shared memory with double-buffered cp.async.  Forward stores the state
// at every CHUNK-th step; backward replays one chunk at a time from that checkpoint into
// shared memory and then walks it in reverse.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int SCAN_N = 16;      // state size
constexpr int SCAN_CHUNK = 16;  // checkpoint interval

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
  int bpg;                     // batch entries per parameter set: A, D, dt_bias (and their gradients) of
                               // batch entry b are rows (b / bpg) * C + c
};

// Thread mapping of both scan kernels: a CTA of 128 threads owns 32 consecutive channels;
// thread = (channel, group of 4 states).  Inputs are staged through shared memory with
// cp.async, double buffered, so the global-memory latency of tile k+1 hides behind the
// recurrence of tile k; all global traffic is in full 64-byte rows.
constexpr int SCAN_CH = 32;   // channels per CTA
constexpr int SCAN_SG = 4;    // states per thread
constexpr int FWD_T = 32;     // steps per forward stage

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int sz = valid ? 16 : 0;   // src-size 0 zero-fills the destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

struct __align__(16) FwdStage {
  __nv_bfloat16 u[FWD_T][SCAN_CH], dt[FWD_T][SCAN_CH], z[FWD_T][SCAN_CH];
  float B[FWD_T][SCAN_N], C[FWD_T][SCAN_N];
};

__global__ void __launch_bounds__(SCAN_CH * SCAN_SG)
scan_fwd_kernel(ScanArgs a, __nv_bfloat16* __restrict__ out, float* __restrict__ ckpt /*[B, S/CHUNK, N, C]*/) {
  __shared__ FwdStage st[2];
  __shared__ __align__(16) __nv_bfloat16 ytile[FWD_T][SCAN_CH];
  const int tid = threadIdx.x, ch = tid >> 2, sg = tid & 3;
  const int c0 = blockIdx.x * SCAN_CH, c = c0 + ch, b = blockIdx.y;
  const int pc = (b / a.bpg) * a.C + c;   // row of this channel's parameters
  const bool has_z = a.z != nullptr;
  float An[SCAN_SG], h[SCAN_SG];
#pragma unroll
  for (int j = 0; j < SCAN_SG; ++j) {
    An[j] = a.A[pc * SCAN_N + sg * SCAN_SG + j] * 1.4426950408889634f;
    h[j] = 0.f;
  }
  const float Dc = a.D ? a.D[pc] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[pc] : 0.f;
  const int nchunks = (a.S + SCAN_CHUNK - 1) / SCAN_CHUNK;
  const int ntiles = (a.S + FWD_T - 1) / FWD_T;
  const int lrow = tid >> 2, lpart = tid & 3;

  auto load_tile = [&](int s, int tile) {
    const int t = tile * FWD_T + lrow;
    const bool ok = t < a.S;
    const size_t tt = (size_t)b * a.S + (ok ? t : a.S - 1);
    cp_async16(&st[s].u[lrow][lpart * 8], a.u + tt * a.C + c0 + lpart * 8, ok);
    cp_async16(&st[s].dt[lrow][lpart * 8], a.delta + tt * a.C + c0 + lpart * 8, ok);
    if (has_z) cp_async16(&st[s].z[lrow][lpart * 8], a.z + tt * a.ldz + c0 + lpart * 8, ok);
    cp_async16(&st[s].B[lrow][lpart * 4], a.Bm + tt * SCAN_N + lpart * 4, ok);
    cp_async16(&st[s].C[lrow][lpart * 4], a.Cm + tt * SCAN_N + lpart * 4, ok);
  };

  load_tile(0, 0);
  cp_async_commit();
  for (int tile = 0; tile < ntiles; ++tile) {
    const int s = tile & 1;
    if (tile + 1 < ntiles) load_tile(s ^ 1, tile + 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll 4
    for (int i = 0; i < FWD_T; ++i) {
      const int t = tile * FWD_T + i;
      if (ckpt != nullptr && (i % SCAN_CHUNK) == 0 && t < a.S) {
        float* ck = ckpt + (((size_t)b * nchunks + t / SCAN_CHUNK) * SCAN_N + sg * SCAN_SG) * a.C + c;
#pragma unroll
        for (int j = 0; j < SCAN_SG; ++j) ck[(size_t)j * a.C] = h[j];
      }
      const float uu = bf2f(st[s].u[i][ch]);
      float dt = bf2f(st[s].dt[i][ch]) + bias;
      if (a.softplus) dt = softplus_f(dt);
      const float4 Bq = *reinterpret_cast<const float4*>(&st[s].B[i][sg * SCAN_SG]);
      const float4 Cq = *reinterpret_cast<const float4*>(&st[s].C[i][sg * SCAN_SG]);
      const float Bv[4] = {Bq.x, Bq.y, Bq.z, Bq.w}, Cv[4] = {Cq.x, Cq.y, Cq.z, Cq.w};
      const float dtu = dt * uu;
      float y = 0.f;
#pragma unroll
      for (int j = 0; j < SCAN_SG; ++j) {
        h[j] = exp2f(dt * An[j]) * h[j] + dtu * Bv[j];
        y += Cv[j] * h[j];
      }
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += Dc * uu;
      if (has_z) y *= silu_f(bf2f(st[s].z[i][ch]));
      if (sg == 0) ytile[i][ch] = __float2bfloat16(y);
    }
    __syncthreads();
    {
      const int t = tile * FWD_T + lrow;
      if (t < a.S)
        *reinterpret_cast<uint4*>(out + ((size_t)b * a.S + t) * a.C + c0 + lpart * 8) =
            *reinterpret_cast<const uint4*>(&ytile[lrow][lpart * 8]);
    }
  }
  cp_async_wait<0>();
}

struct __align__(16) BwdStage {
  __nv_bfloat16 u[SCAN_CHUNK][SCAN_CH], dt[SCAN_CHUNK][SCAN_CH], z[SCAN_CHUNK][SCAN_CH], go[SCAN_CHUNK][SCAN_CH];
  float B[SCAN_CHUNK][SCAN_N], C[SCAN_CHUNK][SCAN_N];
};

__global__ void __launch_bounds__(SCAN_CH * SCAN_SG)
scan_bwd_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ ckpt,
                __nv_bfloat16* __restrict__ du, __nv_bfloat16* __restrict__ ddelta, __nv_bfloat16* __restrict__ dz,
                long long lddz, float* __restrict__ dA, float* __restrict__ dB, float* __restrict__ dC,
                float* __restrict__ dD, float* __restrict__ dbias) {
  __shared__ BwdStage st[2];
  extern __shared__ float4 hs_raw[];  // [SCAN_CHUNK + 1][128]; slot 0 = state before the chunk
  float4 (*hs)[SCAN_CH * SCAN_SG] = reinterpret_cast<float4 (*)[SCAN_CH * SCAN_SG]>(hs_raw);
  __shared__ float dBs[SCAN_CHUNK][SCAN_N], dCs[SCAN_CHUNK][SCAN_N];
  __shared__ __align__(16) __nv_bfloat16 du_t[SCAN_CHUNK][SCAN_CH], dd_t[SCAN_CHUNK][SCAN_CH], dz_t[SCAN_CHUNK][SCAN_CH];
  const int tid = threadIdx.x, lane = tid & 31, ch = tid >> 2, sg = tid & 3;
  const int c0 = blockIdx.x * SCAN_CH, c = c0 + ch, b = blockIdx.y;
  const int pc = (b / a.bpg) * a.C + c;   // row of this channel's parameters and of their gradients
  const bool has_z = a.z != nullptr;
  float An[SCAN_SG], g[SCAN_SG], dAacc[SCAN_SG];
#pragma unroll
  for (int j = 0; j < SCAN_SG; ++j) {
    An[j] = a.A[pc * SCAN_N + sg * SCAN_SG + j];
    g[j] = 0.f;
    dAacc[j] = 0.f;
  }
  const float Dc = a.D ? a.D[pc] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[pc] : 0.f;
  float dDacc = 0.f, dbacc = 0.f;
  const int nchunks = (a.S + SCAN_CHUNK - 1) / SCAN_CHUNK;
  for (int i = tid; i < SCAN_CHUNK * SCAN_N; i += blockDim.x) {
    (&dBs[0][0])[i] = 0.f;
    (&dCs[0][0])[i] = 0.f;
  }

  // 6 arrays x 64 sixteen-byte pieces per stage; each thread copies three of them
  const int lrow = (tid & 63) >> 2, lpart = tid & 3, lhalf = tid >> 6;
  auto load_chunk = [&](int s, int chunk) {
    const int t = chunk * SCAN_CHUNK + lrow;
    const bool ok = t < a.S;
    const size_t tt = (size_t)b * a.S + (ok ? t : a.S - 1);
    if (lhalf == 0) {
      cp_async16(&st[s].u[lrow][lpart * 8], a.u + tt * a.C + c0 + lpart * 8, ok);
      cp_async16(&st[s].go[lrow][lpart * 8], dout + tt * a.C + c0 + lpart * 8, ok);
      cp_async16(&st[s].B[lrow][lpart * 4], a.Bm + tt * SCAN_N + lpart * 4, ok);
    } else {
      cp_async16(&st[s].dt[lrow][lpart * 8], a.delta + tt * a.C + c0 + lpart * 8, ok);
      if (has_z) cp_async16(&st[s].z[lrow][lpart * 8], a.z + tt * a.ldz + c0 + lpart * 8, ok);
      cp_async16(&st[s].C[lrow][lpart * 4], a.Cm + tt * SCAN_N + lpart * 4, ok);
    }
  };

  load_chunk(0, nchunks - 1);
  cp_async_commit();
  int s = 0;
  for (int chk = nchunks - 1; chk >= 0; --chk, s ^= 1) {
    if (chk > 0) load_chunk(s ^ 1, chk - 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const int t0 = chk * SCAN_CHUNK;
    const int len = min(SCAN_CHUNK, a.S - t0);
    float h[SCAN_SG];
    {
      const float* ck = ckpt + (((size_t)b * nchunks + chk) * SCAN_N + sg * SCAN_SG) * a.C + c;
#pragma unroll
      for (int j = 0; j < SCAN_SG; ++j) h[j] = ck[(size_t)j * a.C];
      hs[0][tid] = make_float4(h[0], h[1], h[2], h[3]);
    }
    float uu[SCAN_CHUNK], dtv[SCAN_CHUNK];
    // replay the chunk forward, keeping every state
#pragma unroll
    for (int i = 0; i < SCAN_CHUNK; ++i) {
      uu[i] = bf2f(st[s].u[i][ch]);
      float dt = bf2f(st[s].dt[i][ch]) + bias;
      if (a.softplus) dt = softplus_f(dt);
      dtv[i] = dt;
      const float4 Bq = *reinterpret_cast<const float4*>(&st[s].B[i][sg * SCAN_SG]);
      const float Bv[4] = {Bq.x, Bq.y, Bq.z, Bq.w};
      const float dtu = dt * uu[i];
#pragma unroll
      for (int j = 0; j < SCAN_SG; ++j) h[j] = __expf(dt * An[j]) * h[j] + dtu * Bv[j];
      hs[i + 1][tid] = make_float4(h[0], h[1], h[2], h[3]);
    }
    // reverse sweep
#pragma unroll
    for (int i = SCAN_CHUNK - 1; i >= 0; --i) {
      if (i >= len) continue;           // uniform across the CTA
      const float dt = dtv[i], u = uu[i];
      const float go = bf2f(st[s].go[i][ch]);
      const float4 Bq = *reinterpret_cast<const float4*>(&st[s].B[i][sg * SCAN_SG]);
      const float4 Cq = *reinterpret_cast<const float4*>(&st[s].C[i][sg * SCAN_SG]);
      const float Bv[4] = {Bq.x, Bq.y, Bq.z, Bq.w}, Cv[4] = {Cq.x, Cq.y, Cq.z, Cq.w};
      const float4 hc4 = hs[i + 1][tid], hp4 = hs[i][tid];
      const float hc[4] = {hc4.x, hc4.y, hc4.z, hc4.w}, hp[4] = {hp4.x, hp4.y, hp4.z, hp4.w};
      float dy = go, dzv = 0.f;
      if (has_z) {
        float yp = 0.f;
#pragma unroll
        for (int j = 0; j < SCAN_SG; ++j) yp += Cv[j] * hc[j];
        yp += __shfl_xor_sync(0xffffffffu, yp, 1);
        yp += __shfl_xor_sync(0xffffffffu, yp, 2);
        yp += Dc * u;
        const float zv = bf2f(st[s].z[i][ch]);
        const float sgm = sigmoid_f(zv);
        dzv = go * yp * sgm * (1.f + zv * (1.f - sgm));
        dy = go * zv * sgm;
      }
      float ddt = 0.f, du_p = 0.f;
      float dBv[SCAN_SG], dCv[SCAN_SG];
#pragma unroll
      for (int j = 0; j < SCAN_SG; ++j) {
        dCv[j] = dy * hc[j];
        g[j] += Cv[j] * dy;
        const float dA_t = __expf(dt * An[j]);
        const float gh = g[j] * hp[j] * dA_t;
        ddt += gh * An[j] + g[j] * Bv[j] * u;
        dAacc[j] += gh * dt;
        dBv[j] = g[j] * dt * u;
        du_p += g[j] * dt * Bv[j];
        g[j] *= dA_t;
      }
      ddt += __shfl_xor_sync(0xffffffffu, ddt, 1);
      ddt += __shfl_xor_sync(0xffffffffu, ddt, 2);
      du_p += __shfl_xor_sync(0xffffffffu, du_p, 1);
      du_p += __shfl_xor_sync(0xffffffffu, du_p, 2);
      float dd = ddt;
      if (a.softplus) dd *= sigmoid_f(bf2f(st[s].dt[i][ch]) + bias);
      if (sg == 0) {
        dDacc += dy * u;
        dbacc += dd;
        du_t[i][ch] = __float2bfloat16(du_p + dy * Dc);
        dd_t[i][ch] = __float2bfloat16(dd);
        dz_t[i][ch] = __float2bfloat16(dzv);
      }
      // sum dB, dC over the 8 channels of this warp (lanes with equal sg), then over warps in smem
#pragma unroll
      for (int j = 0; j < SCAN_SG; ++j) {
#pragma unroll
        for (int o = 4; o < 32; o <<= 1) {
          dBv[j] += __shfl_xor_sync(0xffffffffu, dBv[j], o);
          dCv[j] += __shfl_xor_sync(0xffffffffu, dCv[j], o);
        }
      }
      if (lane < 4) {
#pragma unroll
        for (int j = 0; j < SCAN_SG; ++j) {
          atomicAdd(&dBs[i][sg * SCAN_SG + j], dBv[j]);
          atomicAdd(&dCs[i][sg * SCAN_SG + j], dCv[j]);
        }
      }
    }
    __syncthreads();
    // flush the chunk: coalesced du / ddelta / dz rows, and the channel-summed dB / dC
    if (tid < 64) {
      const int t = t0 + lrow;
      if (t < a.S) {
        const size_t o = ((size_t)b * a.S + t) * a.C + c0 + lpart * 8;
        *reinterpret_cast<uint4*>(du + o) = *reinterpret_cast<const uint4*>(&du_t[lrow][lpart * 8]);
        *reinterpret_cast<uint4*>(ddelta + o) = *reinterpret_cast<const uint4*>(&dd_t[lrow][lpart * 8]);
        if (has_z)
          *reinterpret_cast<uint4*>(dz + ((size_t)b * a.S + t) * lddz + c0 + lpart * 8) =
              *reinterpret_cast<const uint4*>(&dz_t[lrow][lpart * 8]);
      }
    }
    for (int i = tid; i < SCAN_CHUNK * SCAN_N; i += blockDim.x) {
      const int row = i / SCAN_N;
      if (row < len) {
        const size_t o = ((size_t)b * a.S + t0 + row) * SCAN_N + (i % SCAN_N);
        atomicAdd(&dB[o], (&dBs[0][0])[i]);
        atomicAdd(&dC[o], (&dCs[0][0])[i]);
      }
      (&dBs[0][0])[i] = 0.f;
      (&dCs[0][0])[i] = 0.f;
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int j = 0; j < SCAN_SG; ++j) atomicAdd(&dA[pc * SCAN_N + sg * SCAN_SG + j], dAacc[j]);
  if (sg == 0) {
    if (dD) atomicAdd(&dD[pc], dDacc);
    if (dbias) atomicAdd(&dbias[pc], dbacc);
  }
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

extern "C" int kmoe_scan_chunk(void) { return SCAN_CHUNK; }

extern "C" int kmoe_scan_fwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, void* out, float* ckpt, int B,
                             int S, int C, int N, long long ldz, int softplus, int groups, cudaStream_t st) {
  if (N != SCAN_N || groups < 1 || B % groups) return -1;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus, B / groups};
  if (C % SCAN_CH || (z != nullptr && ldz % 8)) return -4;
  dim3 grid(C / SCAN_CH, B);
  scan_fwd_kernel<<<grid, SCAN_CH * SCAN_SG, 0, st>>>(a, (__nv_bfloat16*)out, ckpt);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dA [G,C,N], dB/dC [B,S,N], dD [G,C], dbias [G,C] (G = groups) are fp32 and must be zeroed by the caller.
extern "C" int kmoe_scan_bwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, const void* dout,
                             const float* ckpt, void* du, void* ddelta, void* dz, long long lddz, float* dA, float* dB,
                             float* dC, float* dD, float* dbias, int B, int S, int C, int N, long long ldz,
                             int softplus, int groups, cudaStream_t st) {
  if (N != SCAN_N || groups < 1 || B % groups) return -1;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus, B / groups};
  if (C % SCAN_CH || (z != nullptr && (ldz % 8 || lddz % 8))) return -4;
  dim3 grid(C / SCAN_CH, B);
  const int hs_bytes = (SCAN_CHUNK + 1) * SCAN_CH * SCAN_SG * sizeof(float4);
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, hs_bytes) != cudaSuccess)
      return -3;
    attr = true;
  }
  scan_bwd_kernel<<<grid, SCAN_CH * SCAN_SG, hs_bytes, st>>>(a, (const __nv_bfloat16*)dout, ckpt, (__nv_bfloat16*)du,
                                                     (__nv_bfloat16*)ddelta, (__nv_bfloat16*)dz, lddz, dA, dB, dC,
                                                     dD, dbias);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
