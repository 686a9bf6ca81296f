// Selective scan (Mamba), forward and backward, channels-last bf16 activations.
//
//   h_t[n] = exp(dt_t A[n]) h_{t-1}[n] + dt_t u_t B_t[n]        y_t = sum_n C_t[n] h_t[n] + D u_t   (* silu(z_t))
//
// Layout of the work: a thread owns one channel and keeps all N = 16 states in registers, so the per-step
// scalars (softplus, gates) are computed once per channel and the sums over states stay inside the thread;
// a CTA owns 128 consecutive channels, so every global access is a full 256-byte row.  The sequence is cut
// into P segments that run in parallel (the recurrence is linear, so a segment started from zero only lacks
// decay(segment) * state_before):
//   forward : pass 1 computes each segment's end state from zero and its sum of dt; pass 2 starts every segment
//             from the true state (a short serial combination of the earlier segments) and writes y plus a
//             state checkpoint every 8 steps.
//   backward: pass 1 runs dL/dh backwards through each segment from zero; pass 2 starts from the true incoming
//             value, replays 8 steps at a time from the checkpoint into shared memory and walks them in reverse.
// Inputs are staged through shared memory with double-buffered cp.async.  dB and dC are sums over channels:
// a warp transposes its 32 lanes x 32 values through shared memory (each lane then owns one value summed over
// the warp's channels), the four warps meet in a shared accumulator, CTAs in global atomics.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int SN = 16;        // states
constexpr int CK = 8;         // checkpoint interval = steps per staged tile
constexpr int STH = 128;      // channels (= threads) per CTA
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

__device__ __forceinline__ float s_bf2f(__nv_bfloat16 v) { return __bfloat162float(v); }
__device__ __forceinline__ float s_softplus(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float s_sigmoid(float x) { return 1.f / (1.f + __expf(-x)); }
__device__ __forceinline__ float s_ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void s_cp16(void* dst, const void* src, bool valid) {
  const uint32_t d = smem_u32(dst);
  const int sz = valid ? 16 : 0;   // src-size 0 zero-fills the destination
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void s_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N_>
__device__ __forceinline__ void s_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N_) : "memory"); }

struct ScanArgs {
  const __nv_bfloat16* u;      // [B,S,C]
  const __nv_bfloat16* delta;  // [B,S,C]
  const __nv_bfloat16* z;      // [B,S,*] ld = ldz, may be null
  const float* A;              // [G,C,N]
  const float* Bm;             // [B,S,N]
  const float* Cm;             // [B,S,N]
  const float* D;              // [G,C] or null
  const float* dt_bias;        // [G,C] or null
  int S, C;
  long long ldz;
  int softplus;
  int bpg;                     // batch entries per parameter set
  int P, seg_len;              // segments, steps per segment (multiple of CK)
};

// seg scratch: [B, P, SN + 1, C] floats; rows 0..SN-1 = end state of the segment started from zero, row SN = sum dt
__device__ __forceinline__ size_t seg_off(const ScanArgs& a, int b, int p, int row, int c) {
  return (((size_t)b * a.P + p) * (SN + 1) + row) * a.C + c;
}

struct __align__(16) FwdTile {
  __nv_bfloat16 u[CK][STH], dt[CK][STH], z[CK][STH];
  float B[CK][SN], C[CK][SN];
};

// MODE 0: end state from zero + sum of dt (segments 0 .. P-2).  MODE 1: outputs and checkpoints.
template <int MODE>
__global__ void __launch_bounds__(STH)
scan_fwd_kernel(ScanArgs a, __nv_bfloat16* __restrict__ out, float* __restrict__ ckpt, float* __restrict__ seg) {
  __shared__ FwdTile st[2];
  __shared__ __align__(16) __nv_bfloat16 ytile[CK][STH];
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * STH, c = c0 + tid, p = blockIdx.y, b = blockIdx.z;
  const bool cok = c < a.C;                            // the last CTA may own fewer than 128 channels
  const int pc = (b / a.bpg) * a.C + (cok ? c : 0);
  const bool has_z = a.z != nullptr;
  const int t_begin = p * a.seg_len, t_end = min(a.S, t_begin + a.seg_len);
  float An[SN], h[SN];
#pragma unroll
  for (int n = 0; n < SN; ++n) {
    An[n] = a.A[(size_t)pc * SN + n] * LOG2E;
    h[n] = 0.f;
  }
  const float Dc = a.D ? a.D[pc] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[pc] : 0.f;
  if (MODE == 1 && cok) {
    // state before this segment: fold the earlier segments' zero-started end states, oldest first
    for (int q = 0; q < p; ++q) {
      const float sdt = seg[seg_off(a, b, q, SN, c)];
#pragma unroll
      for (int n = 0; n < SN; ++n) h[n] = s_ex2(An[n] * sdt) * h[n] + seg[seg_off(a, b, q, n, c)];
    }
  }
  float sdt = 0.f;
  const int nchunks = (a.S + CK - 1) / CK;
  const int ntiles = (t_end - t_begin + CK - 1) / CK;
  const int lrow = tid >> 4, lpart = tid & 15;      // 8 rows x 16 sixteen-byte pieces of a bf16 row tile

  auto load_tile = [&](int s, int tile) {
    const int t = t_begin + tile * CK + lrow;
    const bool ok = t < t_end;
    const bool okc = ok && c0 + lpart * 8 < a.C;
    const size_t tt = (size_t)b * a.S + (ok ? t : a.S - 1);
    const int cc = okc ? c0 + lpart * 8 : 0;
    s_cp16(&st[s].u[lrow][lpart * 8], a.u + tt * a.C + cc, okc);
    s_cp16(&st[s].dt[lrow][lpart * 8], a.delta + tt * a.C + cc, okc);
    if (MODE == 1 && has_z) s_cp16(&st[s].z[lrow][lpart * 8], a.z + tt * a.ldz + cc, okc);
    if (lpart < 4) s_cp16(&st[s].B[lrow][lpart * 4], a.Bm + tt * SN + lpart * 4, ok);
    else if (MODE == 1 && lpart < 8) s_cp16(&st[s].C[lrow][(lpart - 4) * 4], a.Cm + tt * SN + (lpart - 4) * 4, ok);
  };

  load_tile(0, 0);
  s_commit();
  for (int tile = 0; tile < ntiles; ++tile) {
    const int s = tile & 1;
    if (tile + 1 < ntiles) load_tile(s ^ 1, tile + 1);
    s_commit();
    s_wait<1>();
    __syncthreads();
    const int t0 = t_begin + tile * CK;
    if (MODE == 1 && ckpt != nullptr && cok) {
      float* ck = ckpt + ((size_t)b * nchunks + t0 / CK) * SN * a.C + c;
#pragma unroll
      for (int n = 0; n < SN; ++n) ck[(size_t)n * a.C] = h[n];
    }
#pragma unroll
    for (int i = 0; i < CK; ++i) {
      if (t0 + i >= t_end) break;                     // uniform
      const float uu = s_bf2f(st[s].u[i][tid]);
      float dt = s_bf2f(st[s].dt[i][tid]) + bias;
      if (a.softplus) dt = s_softplus(dt);
      const float dtu = dt * uu;
      const float4* Bq = reinterpret_cast<const float4*>(&st[s].B[i][0]);
      const float4* Cq = reinterpret_cast<const float4*>(&st[s].C[i][0]);
      float ys[4] = {0.f, 0.f, 0.f, 0.f};                // four partial sums: no 16-long dependent chain
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const float4 bq = Bq[n4];
        const float bv[4] = {bq.x, bq.y, bq.z, bq.w};
        float cv[4] = {0.f, 0.f, 0.f, 0.f};
        if (MODE == 1) {
          const float4 cq = Cq[n4];
          cv[0] = cq.x; cv[1] = cq.y; cv[2] = cq.z; cv[3] = cq.w;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n4 * 4 + j;
          h[n] = s_ex2(dt * An[n]) * h[n] + dtu * bv[j];
          if (MODE == 1) ys[j] += cv[j] * h[n];
        }
      }
      if (MODE == 0) {
        sdt += dt;
      } else {
        float y = (ys[0] + ys[1]) + (ys[2] + ys[3]) + Dc * uu;
        if (has_z) {
          const float zv = s_bf2f(st[s].z[i][tid]);
          y *= zv * s_sigmoid(zv);
        }
        ytile[i][tid] = __float2bfloat16(y);
      }
    }
    if (MODE == 1) {
      __syncthreads();
      const int t = t0 + lrow;
      if (t < t_end && c0 + lpart * 8 < a.C)
        *reinterpret_cast<uint4*>(out + ((size_t)b * a.S + t) * a.C + c0 + lpart * 8) =
            *reinterpret_cast<const uint4*>(&ytile[lrow][lpart * 8]);
    }
    __syncthreads();
  }
  s_wait<0>();
  if (MODE == 0 && cok) {
#pragma unroll
    for (int n = 0; n < SN; ++n) seg[seg_off(a, b, p, n, c)] = h[n];
    seg[seg_off(a, b, p, SN, c)] = sdt;
  }
}

// ------------------------------------------------------------------ backward, pass 1
// dL/dh carried backwards through segment p (1 .. P-1) from zero: gseg[b][p][n][c] = what the segment hands to
// the step before its first one.
struct __align__(16) G1Tile {
  __nv_bfloat16 dt[CK][STH], z[CK][STH], go[CK][STH];
  float C[CK][SN];
};

__global__ void __launch_bounds__(STH)
scan_bwd_carry_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dout, float* __restrict__ gseg) {
  __shared__ G1Tile st[2];
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * STH, c = c0 + tid, p = blockIdx.y + 1, b = blockIdx.z;
  const bool cok = c < a.C;
  const int pc = (b / a.bpg) * a.C + (cok ? c : 0);
  const bool has_z = a.z != nullptr;
  const int t_begin = p * a.seg_len, t_end = min(a.S, t_begin + a.seg_len);
  float An[SN], g[SN];
#pragma unroll
  for (int n = 0; n < SN; ++n) {
    An[n] = a.A[(size_t)pc * SN + n] * LOG2E;
    g[n] = 0.f;
  }
  const float bias = a.dt_bias ? a.dt_bias[pc] : 0.f;
  const int ntiles = (t_end - t_begin + CK - 1) / CK;
  const int lrow = tid >> 4, lpart = tid & 15;
  auto load_tile = [&](int s, int tile) {
    const int t = t_begin + tile * CK + lrow;
    const bool ok = t < t_end;
    const size_t tt = (size_t)b * a.S + (ok ? t : a.S - 1);
    const bool okc = ok && c0 + lpart * 8 < a.C;
    const int cc = okc ? c0 + lpart * 8 : 0;
    s_cp16(&st[s].dt[lrow][lpart * 8], a.delta + tt * a.C + cc, okc);
    s_cp16(&st[s].go[lrow][lpart * 8], dout + tt * a.C + cc, okc);
    if (has_z) s_cp16(&st[s].z[lrow][lpart * 8], a.z + tt * a.ldz + cc, okc);
    if (lpart < 4) s_cp16(&st[s].C[lrow][lpart * 4], a.Cm + tt * SN + lpart * 4, ok);
  };
  load_tile(0, ntiles - 1);
  s_commit();
  int s = 0;
  for (int tile = ntiles - 1; tile >= 0; --tile, s ^= 1) {
    if (tile > 0) load_tile(s ^ 1, tile - 1);
    s_commit();
    s_wait<1>();
    __syncthreads();
    const int t0 = t_begin + tile * CK;
#pragma unroll
    for (int i = CK - 1; i >= 0; --i) {
      if (t0 + i >= t_end) continue;                  // uniform
      float dt = s_bf2f(st[s].dt[i][tid]) + bias;
      if (a.softplus) dt = s_softplus(dt);
      float dy = s_bf2f(st[s].go[i][tid]);
      if (has_z) {
        const float zv = s_bf2f(st[s].z[i][tid]);
        dy *= zv * s_sigmoid(zv);
      }
      const float4* Cq = reinterpret_cast<const float4*>(&st[s].C[i][0]);
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const float4 cq = Cq[n4];
        const float cv[4] = {cq.x, cq.y, cq.z, cq.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int n = n4 * 4 + j;
          g[n] = (g[n] + cv[j] * dy) * s_ex2(dt * An[n]);
        }
      }
    }
    __syncthreads();
  }
  s_wait<0>();
  if (cok) {
#pragma unroll
    for (int n = 0; n < SN; ++n) gseg[(((size_t)b * a.P + p) * SN + n) * a.C + c] = g[n];
  }
}

// ------------------------------------------------------------------ backward, pass 2
struct __align__(16) BwdTile {
  __nv_bfloat16 u[CK][STH], dt[CK][STH], z[CK][STH], go[CK][STH];
  float B[CK][SN], C[CK][SN];
};
constexpr int TPAD = 36;      // row pitch (floats) of the per-warp transposition buffer

struct BwdSmem {
  float4 hs[CK][4][STH];                       // state after step i of the chunk, [i][state quad][channel]
  BwdTile st[2];
  __nv_bfloat16 du_t[CK][STH], dd_t[CK][STH], dz_t[CK][STH];
  float tr[STH / 32][32][TPAD];                // per warp: lane x (dB[0..15], dC[0..15])
  float acc[CK][2 * SN];                       // channel sums of the CTA for the chunk
};

__global__ void __launch_bounds__(STH, 2)
scan_bwd_kernel(ScanArgs a, const __nv_bfloat16* __restrict__ dout, const float* __restrict__ ckpt,
                const float* __restrict__ seg, const float* __restrict__ gseg, __nv_bfloat16* __restrict__ du,
                __nv_bfloat16* __restrict__ ddelta, __nv_bfloat16* __restrict__ dz, long long lddz,
                float* __restrict__ dA, float* __restrict__ dB, float* __restrict__ dC, float* __restrict__ dD,
                float* __restrict__ dbias) {
  extern __shared__ __align__(16) uint8_t bwd_raw[];
  BwdSmem& sm = *reinterpret_cast<BwdSmem*>(bwd_raw);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int c0 = blockIdx.x * STH, c = c0 + tid, p = blockIdx.y, b = blockIdx.z;
  const bool cok = c < a.C;                            // idle lanes compute on zero-filled inputs and store nothing
  const int pc = (b / a.bpg) * a.C + (cok ? c : 0);
  const bool has_z = a.z != nullptr;
  const int t_begin = p * a.seg_len, t_end = min(a.S, t_begin + a.seg_len);
  float An[SN], g[SN], dAacc[SN];
#pragma unroll
  for (int n = 0; n < SN; ++n) {
    An[n] = a.A[(size_t)pc * SN + n] * LOG2E;
    g[n] = 0.f;
    dAacc[n] = 0.f;
  }
  // dL/dh flowing into the last step of this segment: fold the later segments' zero-started carries, last first
  for (int q = a.P - 1; q > p && cok; --q) {
    const float sdt = (q < a.P - 1) ? seg[seg_off(a, b, q, SN, c)] : 0.f;
#pragma unroll
    for (int n = 0; n < SN; ++n) {
      const float loc = gseg[(((size_t)b * a.P + q) * SN + n) * a.C + c];
      g[n] = (q < a.P - 1) ? loc + s_ex2(An[n] * sdt) * g[n] : loc;
    }
  }
  const float Dc = a.D ? a.D[pc] : 0.f;
  const float bias = a.dt_bias ? a.dt_bias[pc] : 0.f;
  float dDacc = 0.f, dbacc = 0.f;
  const int nchunks = (a.S + CK - 1) / CK;
  const int ntiles = (t_end - t_begin + CK - 1) / CK;
  const int lrow = tid >> 4, lpart = tid & 15;
  for (int i = tid; i < CK * 2 * SN; i += STH) (&sm.acc[0][0])[i] = 0.f;

  auto load_tile = [&](int s, int tile) {
    const int t = t_begin + tile * CK + lrow;
    const bool ok = t < t_end;
    const size_t tt = (size_t)b * a.S + (ok ? t : a.S - 1);
    const bool okc = ok && c0 + lpart * 8 < a.C;
    const int cc = okc ? c0 + lpart * 8 : 0;
    s_cp16(&sm.st[s].u[lrow][lpart * 8], a.u + tt * a.C + cc, okc);
    s_cp16(&sm.st[s].dt[lrow][lpart * 8], a.delta + tt * a.C + cc, okc);
    s_cp16(&sm.st[s].go[lrow][lpart * 8], dout + tt * a.C + cc, okc);
    if (has_z) s_cp16(&sm.st[s].z[lrow][lpart * 8], a.z + tt * a.ldz + cc, okc);
    if (lpart < 4) s_cp16(&sm.st[s].B[lrow][lpart * 4], a.Bm + tt * SN + lpart * 4, ok);
    else if (lpart < 8) s_cp16(&sm.st[s].C[lrow][(lpart - 4) * 4], a.Cm + tt * SN + (lpart - 4) * 4, ok);
  };
  auto load_ckpt = [&](int tile, float (&h0)[SN]) {
    const float* ck = ckpt + ((size_t)b * nchunks + (t_begin / CK + tile)) * SN * a.C + (cok ? c : 0);
#pragma unroll
    for (int n = 0; n < SN; ++n) h0[n] = cok ? ck[(size_t)n * a.C] : 0.f;
  };

  float h0[SN], h0n[SN];
  load_tile(0, ntiles - 1);
  s_commit();
  load_ckpt(ntiles - 1, h0);
  int s = 0;
  for (int tile = ntiles - 1; tile >= 0; --tile, s ^= 1) {
    if (tile > 0) {
      load_tile(s ^ 1, tile - 1);
      load_ckpt(tile - 1, h0n);                       // in flight while this chunk is processed
    }
    s_commit();
    s_wait<1>();
    __syncthreads();
    const int t0 = t_begin + tile * CK;
    const int len = min(CK, t_end - t0);
    float uu[CK], dtv[CK];
    {
      // replay the chunk forward, keeping every state
      float h[SN];
#pragma unroll
      for (int n = 0; n < SN; ++n) h[n] = h0[n];
#pragma unroll
      for (int i = 0; i < CK; ++i) {
        uu[i] = s_bf2f(sm.st[s].u[i][tid]);
        float dt = s_bf2f(sm.st[s].dt[i][tid]) + bias;
        if (a.softplus) dt = s_softplus(dt);
        dtv[i] = dt;
        const float dtu = dt * uu[i];
        const float4* Bq = reinterpret_cast<const float4*>(&sm.st[s].B[i][0]);
#pragma unroll
        for (int n4 = 0; n4 < 4; ++n4) {
          const float4 bq = Bq[n4];
          const float bv[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int n = n4 * 4 + j;
            h[n] = s_ex2(dt * An[n]) * h[n] + dtu * bv[j];
          }
          sm.hs[i][n4][tid] = make_float4(h[n4 * 4], h[n4 * 4 + 1], h[n4 * 4 + 2], h[n4 * 4 + 3]);
        }
      }
    }
    // reverse sweep; hc = state after step i, hp = state before it
    float hc[SN];
    {
      const int il = len - 1;
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const float4 v = sm.hs[il][n4][tid];
        hc[n4 * 4] = v.x; hc[n4 * 4 + 1] = v.y; hc[n4 * 4 + 2] = v.z; hc[n4 * 4 + 3] = v.w;
      }
    }
#pragma unroll
    for (int i = CK - 1; i >= 0; --i) {
      if (i >= len) continue;                          // uniform
      float hp[SN];
      if (i > 0) {
#pragma unroll
        for (int n4 = 0; n4 < 4; ++n4) {
          const float4 v = sm.hs[i - 1][n4][tid];
          hp[n4 * 4] = v.x; hp[n4 * 4 + 1] = v.y; hp[n4 * 4 + 2] = v.z; hp[n4 * 4 + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int n = 0; n < SN; ++n) hp[n] = h0[n];
      }
      const float dt = dtv[i], u = uu[i];
      const float go = s_bf2f(sm.st[s].go[i][tid]);
      const float4* Bq = reinterpret_cast<const float4*>(&sm.st[s].B[i][0]);
      const float4* Cq = reinterpret_cast<const float4*>(&sm.st[s].C[i][0]);
      float Bv[SN], Cv[SN];
#pragma unroll
      for (int n4 = 0; n4 < 4; ++n4) {
        const float4 bq = Bq[n4], cq = Cq[n4];
        Bv[n4 * 4] = bq.x; Bv[n4 * 4 + 1] = bq.y; Bv[n4 * 4 + 2] = bq.z; Bv[n4 * 4 + 3] = bq.w;
        Cv[n4 * 4] = cq.x; Cv[n4 * 4 + 1] = cq.y; Cv[n4 * 4 + 2] = cq.z; Cv[n4 * 4 + 3] = cq.w;
      }
      float dy = go, dzv = 0.f;
      if (has_z) {
        float yq[4] = {Dc * u, 0.f, 0.f, 0.f};
#pragma unroll
        for (int n = 0; n < SN; ++n) yq[n & 3] += Cv[n] * hc[n];
        const float yp = (yq[0] + yq[1]) + (yq[2] + yq[3]);
        const float zv = s_bf2f(sm.st[s].z[i][tid]);
        const float sgm = s_sigmoid(zv);
        dzv = go * yp * sgm * (1.f + zv * (1.f - sgm));
        dy = go * zv * sgm;
      }
      const float dtu = dt * u;
      float sAq[4] = {0.f, 0.f, 0.f, 0.f}, sBq[4] = {0.f, 0.f, 0.f, 0.f};   // partial sums over the states
      float vals[2 * SN];
#pragma unroll
      for (int n = 0; n < SN; ++n) {
        vals[SN + n] = dy * hc[n];                     // dC
        const float gn = g[n] + Cv[n] * dy;            // dL/dh_t
        const float an = s_ex2(dt * An[n]);
        const float gh = gn * hp[n] * an;
        sAq[n & 3] += gh * An[n];
        sBq[n & 3] += gn * Bv[n];
        dAacc[n] += gh * dt;
        vals[n] = gn * dtu;                            // dB
        g[n] = gn * an;                                // handed to step t-1
      }
      const float sA = (sAq[0] + sAq[1]) + (sAq[2] + sAq[3]);   // sum_n g h_prev a A2[n]
      const float sB = (sBq[0] + sBq[1]) + (sBq[2] + sBq[3]);   // sum_n g B[n]
      float dd = sA * LN2 + u * sB;
      if (a.softplus) dd *= s_sigmoid(s_bf2f(sm.st[s].dt[i][tid]) + bias);
      dDacc += dy * u;
      dbacc += dd;
      sm.du_t[i][tid] = __float2bfloat16(dt * sB + dy * Dc);
      sm.dd_t[i][tid] = __float2bfloat16(dd);
      sm.dz_t[i][tid] = __float2bfloat16(dzv);
      // sum dB / dC over the warp's 32 channels: transpose through shared memory, lane k sums value k
      {
        float* row = &sm.tr[warp][lane][0];
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4)
          *reinterpret_cast<float4*>(row + k4 * 4) =
              make_float4(vals[k4 * 4], vals[k4 * 4 + 1], vals[k4 * 4 + 2], vals[k4 * 4 + 3]);
        __syncwarp();
        float sq[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int r = 0; r < 32; ++r) sq[r & 3] += sm.tr[warp][r][lane];
        __syncwarp();
        atomicAdd(&sm.acc[i][lane], (sq[0] + sq[1]) + (sq[2] + sq[3]));
      }
#pragma unroll
      for (int n = 0; n < SN; ++n) hc[n] = hp[n];
    }
    __syncthreads();
    // flush the chunk: coalesced du / ddelta / dz rows and the channel-summed dB / dC
    {
      const int t = t0 + lrow;
      if (t < t_end && c0 + lpart * 8 < a.C) {
        const size_t o = ((size_t)b * a.S + t) * a.C + c0 + lpart * 8;
        *reinterpret_cast<uint4*>(du + o) = *reinterpret_cast<const uint4*>(&sm.du_t[lrow][lpart * 8]);
        *reinterpret_cast<uint4*>(ddelta + o) = *reinterpret_cast<const uint4*>(&sm.dd_t[lrow][lpart * 8]);
        if (has_z)
          *reinterpret_cast<uint4*>(dz + ((size_t)b * a.S + t) * lddz + c0 + lpart * 8) =
              *reinterpret_cast<const uint4*>(&sm.dz_t[lrow][lpart * 8]);
      }
    }
    for (int i = tid; i < CK * 2 * SN; i += STH) {
      const int row = i / (2 * SN), k = i % (2 * SN);
      if (row < len) {
        const size_t o = ((size_t)b * a.S + t0 + row) * SN + (k % SN);
        atomicAdd(k < SN ? &dB[o] : &dC[o], (&sm.acc[0][0])[i]);
      }
      (&sm.acc[0][0])[i] = 0.f;
    }
#pragma unroll
    for (int n = 0; n < SN; ++n) h0[n] = h0n[n];
    __syncthreads();
  }
  s_wait<0>();
  if (cok) {
#pragma unroll
    for (int n = 0; n < SN; ++n) atomicAdd(&dA[(size_t)pc * SN + n], dAacc[n]);
    if (dD) atomicAdd(&dD[pc], dDacc);
    if (dbias) atomicAdd(&dbias[pc], dbacc);
  }
}

// Segment count: the one that minimises (waves of two resident CTAs per SM) x (steps per segment), counting
// the extra pass over all but one segment; segments are multiples of the chunk and at least 64 steps long.
static void plan(int B, int S, int C, int* P, int* seg_len) {
  const long long per_seg = (long long)((C + STH - 1) / STH) * B;
  const long long slots = 148 * 2;
  long long best_cost = -1;
  int best_len = (S + CK - 1) / CK * CK;
  for (int want = 1; want <= 16; ++want) {
    int len = (S + want - 1) / want;
    if (len < 64) len = 64;
    len = (len + CK - 1) / CK * CK;
    const int p = (S + len - 1) / len;
    const long long waves = (per_seg * p + slots - 1) / slots;
    const long long cost = waves * len * (p > 1 ? 5 : 4);      // the carry pass costs about a quarter more
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      best_len = len;
    }
  }
  if (best_len < CK) best_len = CK;
  *seg_len = best_len;
  *P = (S + best_len - 1) / best_len;
  if (*P < 1) *P = 1;
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_scan_chunk(void) { return CK; }

extern "C" int kmoe_scan_segments(int B, int S, int C) {
  int P, len;
  plan(B, S, C, &P, &len);
  return P;
}

extern "C" int kmoe_scan_fwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, void* out, float* ckpt,
                             float* seg, int B, int S, int C, int N, long long ldz, int softplus, int groups,
                             cudaStream_t st) {
  if (N != SN || groups < 1 || B % groups) return -1;
  if (C % 8 || (z != nullptr && ldz % 8)) return -4;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus, B / groups, 1, 0};
  plan(B, S, C, &a.P, &a.seg_len);
  if (a.P > 1) {
    if (seg == nullptr) return -5;
    scan_fwd_kernel<0><<<dim3((C + STH - 1) / STH, a.P - 1, B), STH, 0, st>>>(a, nullptr, nullptr, seg);
  }
  scan_fwd_kernel<1><<<dim3((C + STH - 1) / STH, a.P, B), STH, 0, st>>>(a, (__nv_bfloat16*)out, ckpt, seg);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// dA [G,C,N], dB/dC [B,S,N], dD [G,C], dbias [G,C] (G = groups) are fp32 and must be zeroed by the caller.
// seg: the forward's segment scratch; gseg: scratch of B * P * N * C floats.
extern "C" int kmoe_scan_bwd(const void* u, const void* delta, const void* z, const float* A, const float* Bm,
                             const float* Cm, const float* D, const float* dt_bias, const void* dout,
                             const float* ckpt, const float* seg, float* gseg, void* du, void* ddelta, void* dz,
                             long long lddz, float* dA, float* dB, float* dC, float* dD, float* dbias, int B, int S,
                             int C, int N, long long ldz, int softplus, int groups, cudaStream_t st) {
  if (N != SN || groups < 1 || B % groups) return -1;
  if (C % 8 || (z != nullptr && (ldz % 8 || lddz % 8))) return -4;
  ScanArgs a{(const __nv_bfloat16*)u, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)z, A, Bm, Cm, D, dt_bias,
             S, C, ldz, softplus, B / groups, 1, 0};
  plan(B, S, C, &a.P, &a.seg_len);
  if (a.P > 1 && (seg == nullptr || gseg == nullptr)) return -5;
  const int smem = (int)sizeof(BwdSmem);
  static bool attr = false;
  if (!attr) {
    if (cudaFuncSetAttribute(scan_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return -3;
    attr = true;
  }
  if (a.P > 1)
    scan_bwd_carry_kernel<<<dim3((C + STH - 1) / STH, a.P - 1, B), STH, 0, st>>>(a, (const __nv_bfloat16*)dout, gseg);
  scan_bwd_kernel<<<dim3((C + STH - 1) / STH, a.P, B), STH, smem, st>>>(a, (const __nv_bfloat16*)dout, ckpt, seg, gseg,
                                                            (__nv_bfloat16*)du, (__nv_bfloat16*)ddelta,
                                                            (__nv_bfloat16*)dz, lddz, dA, dB, dC, dD, dbias);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
