// Routing decisions as single kernels (CUDA cores; the inputs are tiny next to the expert GEMMs, the
// point is one launch instead of a chain of softmax / top-k / sort / bincount launches, and no
// intermediate tensors).
//
//   route_topk      token-choice router tail: softmax over experts -> top-k -> renormalise, plus the
//                   load-balance and z-loss partial sums (sum of probabilities and assignment count
//                   per expert, sum of logsumexp^2).            reference: moe_arch/model/moe.py:441-460, 840-939
//   seq_topk        per-row top-k of a (rows, S) score matrix, one CTA per row, bitonic sort in shared
//                   memory.  mode 0 (mixture-of-depths): keep the k largest logits, emit their indices in
//                   ascending order and a softmax over the kept logits.  reference: moe_arch/model/mod.py:93-112
//                   mode 1 (expert choice): softmax over the whole row, keep the k largest probabilities
//                   in descending order, renormalise.          reference: moe_arch/model/moe.py:494-530
// Each has a backward kernel producing d(logits).
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math_constants.h>

#include "kmoe_api.h"
#include "ptx.cuh"

namespace kmoe {

constexpr int ROUTE_MAX_E = 128;
constexpr int ROUTE_MAX_K = 8;

// ---------------------------------------------------------------------------- token choice
// one thread per token; logits fp32 (T, E)
__global__ void route_topk_fwd_kernel(const float* __restrict__ logits, int T, int E, int k, float* __restrict__ w_out,
                                      long long* __restrict__ idx_out, float* __restrict__ lse_out,
                                      float* __restrict__ p_sum, float* __restrict__ counts,
                                      float* __restrict__ z_sum) {
  extern __shared__ float sm[];           // [2*E] per-CTA partials: sum p, counts
  float* s_p = sm;
  float* s_c = sm + E;
  for (int i = threadIdx.x; i < 2 * E; i += blockDim.x) sm[i] = 0.f;
  __syncthreads();
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  float z = 0.f;
  float my_p[ROUTE_MAX_E];
  int my_sel[ROUTE_MAX_K];
  if (t < T) {
    const float* row = logits + (size_t)t * E;
    float mx = -CUDART_INF_F;
    for (int e = 0; e < E; ++e) mx = fmaxf(mx, row[e]);
    float den = 0.f;
    for (int e = 0; e < E; ++e) den += __expf(row[e] - mx);
    const float lse = mx + __logf(den);
    lse_out[t] = lse;
    z = lse * lse;
    const float inv = 1.f / den;
    int sel[ROUTE_MAX_K];
    float pv[ROUTE_MAX_K];
    float s = 0.f;
    for (int j = 0; j < k; ++j) {
      float best = -CUDART_INF_F;
      int be = 0;
      for (int e = 0; e < E; ++e) {
        bool used = false;
        for (int l = 0; l < j; ++l) used |= (sel[l] == e);
        const float v = row[e];
        if (!used && v > best) { best = v; be = e; }   // first maximum wins ties, like a stable arg-max
      }
      sel[j] = be;
      pv[j] = __expf(best - mx) * inv;
      s += pv[j];
    }
    for (int j = 0; j < k; ++j) {
      w_out[(size_t)t * k + j] = pv[j] / s;
      idx_out[(size_t)t * k + j] = sel[j];
    }
    for (int j = 0; j < ROUTE_MAX_K; ++j) my_sel[j] = j < k ? sel[j] : -1;
    for (int e = 0; e < E; ++e) my_p[e] = __expf(row[e] - mx) * inv;
  }
  // per-expert sums: reduce inside the warp first, so shared memory sees one atomic per warp and expert
  // instead of one per token and expert
  for (int e = 0; e < E; ++e) {
    const float ps = warp_sum(t < T ? my_p[e] : 0.f);
    int hit = 0;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_K; ++j) hit += (t < T && my_sel[j] == e) ? 1 : 0;
    const float cs = warp_sum((float)hit);
    if ((threadIdx.x & 31) == 0) {
      if (ps != 0.f) atomicAdd(&s_p[e], ps);
      if (cs != 0.f) atomicAdd(&s_c[e], cs);
    }
  }
  z = warp_sum(z);
  if ((threadIdx.x & 31) == 0 && z != 0.f) atomicAdd(z_sum, z);
  __syncthreads();
  for (int i = threadIdx.x; i < E; i += blockDim.x) {
    if (s_p[i] != 0.f) atomicAdd(&p_sum[i], s_p[i]);
    if (s_c[i] != 0.f) atomicAdd(&counts[i], s_c[i]);
  }
}

// dlogits = softmax-backward of [renorm-backward(dw) at the selected experts + c_lb[e]] + c_z * 2 lse p
//   c_lb[e] = d_aux * w_lb * E * f_e / T   (the assignment fractions f_e are constants, as in the reference)
//   c_z     = d_aux * w_z / T
__global__ void route_topk_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ lse,
                                      const long long* __restrict__ idx, const float* __restrict__ w,
                                      const float* __restrict__ dw, const float* __restrict__ counts,
                                      const float* __restrict__ d_aux, float w_lb, float w_z, int T, int E, int k,
                                      float* __restrict__ dlogits) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float da = d_aux ? *d_aux : 0.f;
  const float* row = logits + (size_t)t * E;
  const float l = lse[t];
  float s = 0.f, dot_w = 0.f;
  for (int j = 0; j < k; ++j) {
    const int e = (int)idx[(size_t)t * k + j];
    s += __expf(row[e] - l);
    dot_w += (dw ? dw[(size_t)t * k + j] : 0.f) * w[(size_t)t * k + j];
  }
  const float lb_scale = da * w_lb * (float)E / ((float)T * (float)T * (float)k);
  float dp[ROUTE_MAX_E];
  for (int e = 0; e < E; ++e) dp[e] = lb_scale * counts[e];
  for (int j = 0; j < k; ++j) {
    const int e = (int)idx[(size_t)t * k + j];
    dp[e] += ((dw ? dw[(size_t)t * k + j] : 0.f) - dot_w) / s;
  }
  float pd = 0.f;
  for (int e = 0; e < E; ++e) pd += __expf(row[e] - l) * dp[e];
  const float cz = da * w_z * 2.f * l / (float)T;
  for (int e = 0; e < E; ++e) {
    const float p = __expf(row[e] - l);
    dlogits[(size_t)t * E + e] = p * (dp[e] - pd) + cz * p;
  }
}

// ---------------------------------------------------------------------------- per-row top-k
// One CTA per row.  keys: value descending, index ascending on ties.
__device__ __forceinline__ bool key_before(float va, int ia, float vb, int ib) {
  return va > vb || (va == vb && ia < ib);
}

__global__ void seq_topk_fwd_kernel(const float* __restrict__ scores, long long row_stride, long long col_stride,
                                    int rows_inner, long long outer_stride, int S, int S2, int k, int mode,
                                    long long* __restrict__ idx_out, float* __restrict__ w_out,
                                    float* __restrict__ stat_out) {
  extern __shared__ float sm[];
  float* val = sm;                                   // [S2]
  int* ind = reinterpret_cast<int*>(sm + S2);        // [S2]
  __shared__ float red[32];
  __shared__ float s_mx, s_den;
  const int r = blockIdx.x;
  const float* base = scores + (long long)(r / rows_inner) * outer_stride + (long long)(r % rows_inner) * row_stride;
  float mx = -CUDART_INF_F;
  for (int i = threadIdx.x; i < S2; i += blockDim.x) {
    const float v = i < S ? base[(long long)i * col_stride] : -CUDART_INF_F;
    val[i] = v;
    ind[i] = i < S ? i : 0x7fffffff;
    mx = fmaxf(mx, v);
  }
  if (mode == 1) {                                   // softmax statistics of the whole row
    mx = warp_max(mx);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x < 32) {
      float m = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : -CUDART_INF_F;
      m = warp_max(m);
      if (threadIdx.x == 0) s_mx = m;
    }
    __syncthreads();
    float den = 0.f;
    for (int i = threadIdx.x; i < S; i += blockDim.x) den += __expf(val[i] - s_mx);
    den = warp_sum(den);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = den;
    __syncthreads();
    if (threadIdx.x < 32) {
      float d = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      d = warp_sum(d);
      if (threadIdx.x == 0) s_den = d;
    }
  }
  __syncthreads();
  // bitonic sort, best key first
  for (int size = 2; size <= S2; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = threadIdx.x; i < (S2 >> 1); i += blockDim.x) {
        const int lo = 2 * i - (i & (stride - 1));
        const int hi = lo + stride;
        const bool up = (lo & size) == 0;
        const float va = val[lo], vb = val[hi];
        const int ia = ind[lo], ib = ind[hi];
        const bool a_first = key_before(va, ia, vb, ib);
        if (a_first != up) {
          val[lo] = vb; val[hi] = va;
          ind[lo] = ib; ind[hi] = ia;
        }
      }
      __syncthreads();
    }
  }
  if (mode == 1) {
    // top-k probabilities, descending; renormalised over the kept ones (+1e-9 as the reference)
    float part = 0.f;
    for (int i = threadIdx.x; i < k; i += blockDim.x) part += __expf(val[i] - s_mx) / s_den;
    part = warp_sum(part);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = part;
    __syncthreads();
    float tot = 0.f;
    for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
    for (int i = threadIdx.x; i < k; i += blockDim.x) {
      idx_out[(size_t)r * k + i] = ind[i];
      w_out[(size_t)r * k + i] = (__expf(val[i] - s_mx) / s_den) / (tot + 1e-9f);
    }
    if (threadIdx.x == 0) {
      stat_out[(size_t)r * 3 + 0] = s_mx;
      stat_out[(size_t)r * 3 + 1] = s_den;
      stat_out[(size_t)r * 3 + 2] = tot;
    }
    return;
  }
  // mode 0: the k-th key is the threshold; kept positions are emitted in ascending index order
  const float thr_v = val[k - 1];
  const int thr_i = ind[k - 1];
  const float top = val[0];
  __syncthreads();
  // flags over original positions, reusing `ind` as a prefix-sum array after reloading the scores
  for (int i = threadIdx.x; i < S2; i += blockDim.x) {
    const float v = i < S ? base[(long long)i * col_stride] : -CUDART_INF_F;
    val[i] = v;
    ind[i] = (i < S && !key_before(thr_v, thr_i, v, i)) ? 1 : 0;   // keep iff key(i) is not after the threshold
  }
  __syncthreads();
  // inclusive scan (Hillis-Steele over S2 entries, ping-pong avoided by chunked sequential-per-thread scan)
  __shared__ int chunk_sum[1024];
  const int per = (S2 + blockDim.x - 1) / blockDim.x;
  const int b0 = threadIdx.x * per;
  int acc = 0;
  for (int i = b0; i < min(b0 + per, S2); ++i) acc += ind[i];
  chunk_sum[threadIdx.x] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int i = 0; i < blockDim.x; ++i) { const int c = chunk_sum[i]; chunk_sum[i] = run; run += c; }
  }
  __syncthreads();
  float den = 0.f;
  int o = chunk_sum[threadIdx.x];
  for (int i = b0; i < min(b0 + per, S2); ++i) {
    if (ind[i]) {
      const float ex = __expf(val[i] - top);
      idx_out[(size_t)r * k + o] = i;
      w_out[(size_t)r * k + o] = ex;               // normalised below
      den += ex;
      ++o;
    }
  }
  den = warp_sum(den);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = den;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  __threadfence_block();
  __syncthreads();
  for (int i = threadIdx.x; i < k; i += blockDim.x) w_out[(size_t)r * k + i] /= tot;
}

// Mode 0 without a sort: the k-th best key of the row is found by a 4-pass radix selection over
// order-preserving 32-bit images of the scores (256-bin histograms in shared memory), then one block-wide
// prefix count places the kept positions in ascending order.  Same result as the sorting kernel above: keys
// compare by value descending and index ascending, so of the scores equal to the threshold the lowest
// positions are kept.  (The images order -0.0 below +0.0.)
__device__ __forceinline__ uint32_t score_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float key_score(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k ^ 0x80000000u) : ~k);
}

__global__ void __launch_bounds__(1024)
seq_topk_select_kernel(const float* __restrict__ scores, long long row_stride, long long col_stride, int rows_inner,
                       long long outer_stride, int S, int k, long long* __restrict__ idx_out,
                       float* __restrict__ w_out) {
  extern __shared__ uint32_t ukey[];                 // [S]
  __shared__ int hist[256];
  __shared__ int warp_tot[32];
  __shared__ float red[32];
  __shared__ uint32_t s_prefix, s_top;
  __shared__ int s_need;
  const int r = blockIdx.x, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  const float* base = scores + (long long)(r / rows_inner) * outer_stride + (long long)(r % rows_inner) * row_stride;
  uint32_t mxk = 0;
  for (int i = tid; i < S; i += 1024) {
    const uint32_t u = score_key(base[(long long)i * col_stride]);
    ukey[i] = u;
    mxk = max(mxk, u);
  }
  mxk = __reduce_max_sync(0xffffffffu, mxk);
  if (lane == 0) warp_tot[wid] = (int)mxk;
  if (tid == 0) { s_prefix = 0u; s_need = k; }
  __syncthreads();
  if (wid == 0) {
    const uint32_t m = __reduce_max_sync(0xffffffffu, (uint32_t)warp_tot[lane]);
    if (lane == 0) s_top = m;
  }
  for (int pass = 0; pass < 4; ++pass) {
    const int shift = 24 - 8 * pass;
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    const uint32_t prefix = s_prefix;
    const uint32_t mask = pass == 0 ? 0u : (0xffffffffu << (shift + 8));
    for (int i = tid; i < S; i += 1024) {
      const uint32_t u = ukey[i];
      if ((u & mask) == prefix) atomicAdd(&hist[(u >> shift) & 255u], 1);
    }
    __syncthreads();
    if (wid == 0) {
      // lane L owns bins 8L .. 8L+7; the wanted key lies in the bin where the count from the top reaches `need`
      int c[8], tot = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) { c[j] = hist[8 * lane + j]; tot += c[j]; }
      int suf = tot;                                 // sum over this and all higher lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_down_sync(0xffffffffu, suf, o);
        if (lane + o < 32) suf += t;
      }
      const int need = s_need;
      int above = suf - tot;
      if (above < need && need <= suf) {
#pragma unroll
        for (int j = 7; j >= 0; --j) {
          if (above < need && above + c[j] >= need) {
            s_prefix = prefix | ((uint32_t)(8 * lane + j) << shift);
            s_need = need - above;
            above = need;                            // taken: no lower bin matches
          } else {
            above += c[j];
          }
        }
      }
    }
    __syncthreads();
  }
  const uint32_t thr = s_prefix;
  const int need = s_need;                           // how many of the scores equal to the threshold are kept
  // exclusive prefix counts (greater in the low half-word, equal in the high one) over contiguous chunks
  const int per = (S + 1023) / 1024;
  const int b0 = tid * per, b1 = min(b0 + per, S);
  int packed = 0;
  for (int i = b0; i < b1; ++i) {
    const uint32_t u = ukey[i];
    packed += (u > thr ? 1 : 0) + (u == thr ? 0x10000 : 0);
  }
  int inc = packed;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int t = __shfl_up_sync(0xffffffffu, inc, o);
    if (lane >= o) inc += t;
  }
  if (lane == 31) warp_tot[wid] = inc;
  __syncthreads();
  if (wid == 0) {
    const int w = warp_tot[lane];
    int winc = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int t = __shfl_up_sync(0xffffffffu, winc, o);
      if (lane >= o) winc += t;
    }
    warp_tot[lane] = winc - w;
  }
  __syncthreads();
  const int excl = warp_tot[wid] + inc - packed;
  int g = excl & 0xffff, e = excl >> 16;
  const float top = key_score(s_top);
  float den = 0.f;
  for (int i = b0; i < b1; ++i) {
    const uint32_t u = ukey[i];
    const bool eq = u == thr;
    if (u > thr || (eq && e < need)) {
      const int o = g + min(e, need);
      const float ex = __expf(key_score(u) - top);
      idx_out[(size_t)r * k + o] = i;
      w_out[(size_t)r * k + o] = ex;                 // normalised below
      den += ex;
    }
    g += (u > thr) ? 1 : 0;
    e += eq ? 1 : 0;
  }
  den = warp_sum(den);
  if (lane == 0) red[wid] = den;
  __threadfence_block();
  __syncthreads();
  float tot = 0.f;
#pragma unroll 8
  for (int i = 0; i < 32; ++i) tot += red[i];
  for (int i = tid; i < k; i += 1024) w_out[(size_t)r * k + i] /= tot;
}

// mode 0: dscore[idx_j] = w_j (dw_j - sum_l w_l dw_l), zero elsewhere.
// mode 1: p = softmax(row); w_j = p_j / (tot + eps); dp_j = (dw_j - sum_l dw_l w_l) / (tot + eps);
//         dscore_t = p_t (dp_t - sum_j p_j dp_j)   (dp = 0 for tokens that were not picked)
__global__ void seq_topk_bwd_kernel(const float* __restrict__ scores, long long row_stride, long long col_stride,
                                    int rows_inner, long long outer_stride, int S, int k, int mode,
                                    const long long* __restrict__ idx, const float* __restrict__ w,
                                    const float* __restrict__ dw, const float* __restrict__ stat,
                                    float* __restrict__ dscores) {
  extern __shared__ float sm[];                      // [S] dp per position (mode 1) / output staging
  __shared__ float red[32];
  const int r = blockIdx.x;
  const long long boff = (long long)(r / rows_inner) * outer_stride + (long long)(r % rows_inner) * row_stride;
  for (int i = threadIdx.x; i < S; i += blockDim.x) sm[i] = 0.f;
  float dot = 0.f;
  for (int j = threadIdx.x; j < k; j += blockDim.x) dot += w[(size_t)r * k + j] * dw[(size_t)r * k + j];
  dot = warp_sum(dot);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = dot;
  __syncthreads();
  float tot = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) tot += red[i];
  __syncthreads();
  if (mode == 0) {
    for (int j = threadIdx.x; j < k; j += blockDim.x) {
      const float wj = w[(size_t)r * k + j];
      sm[(int)idx[(size_t)r * k + j]] = wj * (dw[(size_t)r * k + j] - tot);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < S; i += blockDim.x) dscores[boff + (long long)i * col_stride] = sm[i];
    return;
  }
  const float mx = stat[(size_t)r * 3], den = stat[(size_t)r * 3 + 1], keep = stat[(size_t)r * 3 + 2] + 1e-9f;
  float pd = 0.f;
  for (int j = threadIdx.x; j < k; j += blockDim.x) {
    const int t = (int)idx[(size_t)r * k + j];
    const float dp = (dw[(size_t)r * k + j] - tot) / keep;
    sm[t] = dp;
    pd += (__expf(scores[boff + (long long)t * col_stride] - mx) / den) * dp;
  }
  pd = warp_sum(pd);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = pd;
  __syncthreads();
  float pdt = 0.f;
  for (int i = 0; i < (blockDim.x >> 5); ++i) pdt += red[i];
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    const float p = __expf(scores[boff + (long long)i * col_stride] - mx) / den;
    dscores[boff + (long long)i * col_stride] = p * (sm[i] - pdt);
  }
}

}  // namespace kmoe

using namespace kmoe;

extern "C" int kmoe_route_topk_fwd(const float* logits, int T, int E, int k, float* w, long long* idx, float* lse,
                                   float* p_sum, float* counts, float* z_sum, cudaStream_t st) {
  if (E > ROUTE_MAX_E || k > ROUTE_MAX_K || k > E) return -1;
  if (T == 0) return 0;
  route_topk_fwd_kernel<<<(T + 127) / 128, 128, 2 * E * sizeof(float), st>>>(logits, T, E, k, w, idx, lse, p_sum,
                                                                            counts, z_sum);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_route_topk_bwd(const float* logits, const float* lse, const long long* idx, const float* w,
                                   const float* dw, const float* counts, const float* d_aux, float w_lb, float w_z,
                                   int T, int E, int k, float* dlogits, cudaStream_t st) {
  if (E > ROUTE_MAX_E || k > ROUTE_MAX_K) return -1;
  if (T == 0) return 0;
  route_topk_bwd_kernel<<<(T + 127) / 128, 128, 0, st>>>(logits, lse, idx, w, dw, counts, d_aux, w_lb, w_z, T, E, k,
                                                          dlogits);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

static int next_pow2(int x) {
  int p = 1;
  while (p < x) p <<= 1;
  return p;
}

extern "C" int kmoe_seq_topk_fwd(const float* scores, long long row_stride, long long col_stride, int rows_inner,
                                 long long outer_stride, int rows, int S, int k, int mode, long long* idx, float* w,
                                 float* stat, cudaStream_t st) {
  const int S2 = next_pow2(S < 2 ? 2 : S);
  if (k < 1 || k > S || S2 > 16384) return -1;
  if (rows == 0) return 0;
  const size_t smem = (size_t)S2 * 8;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(seq_topk_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 8) != cudaSuccess)
      return -3;
    if (cudaFuncSetAttribute(seq_topk_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4) !=
        cudaSuccess)
      return -3;
    attr_set = true;
  }
  if (mode == 0) {      // kept positions in ascending order: selection instead of a sort
    seq_topk_select_kernel<<<rows, 1024, (size_t)S * 4, st>>>(scores, row_stride, col_stride, rows_inner,
                                                              outer_stride, S, k, idx, w);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
  }
  seq_topk_fwd_kernel<<<rows, 1024, smem, st>>>(scores, row_stride, col_stride, rows_inner, outer_stride, S, S2, k,
                                                mode, idx, w, stat);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

extern "C" int kmoe_seq_topk_bwd(const float* scores, long long row_stride, long long col_stride, int rows_inner,
                                 long long outer_stride, int rows, int S, int k, int mode, const long long* idx,
                                 const float* w, const float* dw, const float* stat, float* dscores, cudaStream_t st) {
  if (S > 16384) return -1;
  if (rows == 0) return 0;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(seq_topk_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * 4) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  seq_topk_bwd_kernel<<<rows, 512, (size_t)S * 4, st>>>(scores, row_stride, col_stride, rows_inner, outer_stride, S, k,
                                                        mode, idx, w, dw, stat, dscores);
  return cudaGetLastError() == cudaSuccess ? 0 : -2;
}
