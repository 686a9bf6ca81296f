// PyTorch operator registrations (namespace torch.ops.kmoe) over the C launch API in
// kmoe_api.h.  This is the only translation unit that includes torch headers.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include "kmoe_api.h"

namespace {

using at::Tensor;
using OptT = c10::optional<Tensor>;

inline cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
inline void check(int rc, const char* what) { TORCH_CHECK(rc == 0, "kmoe::", what, " failed with code ", rc); }
inline const void* ptr_or_null(const OptT& t) { return (t.has_value() && t->defined()) ? t->data_ptr() : nullptr; }
inline void need_bf16(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, n, " must be a CUDA bf16 tensor");
}
inline void need_f32(const Tensor& t, const char* n) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat && t.is_contiguous(), n,
              " must be a contiguous CUDA fp32 tensor");
}
// row stride of a (..., C) tensor whose last dim is dense and whose leading dims collapse to rows
inline long long row_stride(const Tensor& t) {
  TORCH_CHECK(t.stride(-1) == 1, "last dimension must be contiguous");
  long long ld = t.stride(-2);
  for (int i = t.dim() - 3; i >= 0; --i)
    TORCH_CHECK(t.size(i) == 1 || t.stride(i) == t.stride(i + 1) * t.size(i + 1), "leading dims must collapse");
  return ld;
}

// ------------------------------------------------------------------------ GEMM
void gemm(const Tensor& A, const Tensor& B, const OptT& B2, Tensor C, const OptT& D, const OptT& G, const OptT& U,
          int64_t mode, int64_t epilogue, int64_t M, int64_t N, int64_t K, int64_t groups, int64_t a_major,
          int64_t b_major, int64_t lda, int64_t ldb, int64_t ldc, int64_t ldd, int64_t a_gs, int64_t b_gs,
          int64_t c_gs, const OptT& tile_group, const OptT& num_m_tiles, const OptT& k_begin, const OptT& k_len,
          double alpha, double beta, const OptT& row_scale, const OptT& row_ptr, const OptT& alpha_dev,
          const OptT& beta_dev, bool sym_upper, double diag_add, int64_t k_split, const OptT& D2, double beta2,
          Tensor status) {
  c10::cuda::CUDAGuard guard(A.device());
  need_bf16(A, "A");
  need_bf16(B, "B");
  KmoeGemmDesc d{};
  d.D2 = ptr_or_null(D2);
  d.beta2 = (float)beta2;
  if (D2.has_value() && D2->defined())
    TORCH_CHECK(D2->scalar_type() == at::kBFloat16 && D.has_value() && D->defined() && D2->sizes() == D->sizes() &&
                D2->strides() == D->strides(), "D2 must be a bf16 tensor laid out like D");
  d.A = A.data_ptr(); d.B = B.data_ptr(); d.B2 = ptr_or_null(B2); d.C = C.data_ptr();
  d.D = ptr_or_null(D); d.G_out = const_cast<void*>(ptr_or_null(G)); d.U_out = const_cast<void*>(ptr_or_null(U));
  d.mode = (int)mode; d.epilogue = (int)epilogue; d.M = (int)M; d.N = (int)N; d.K = (int)K; d.groups = (int)groups;
  d.a_major = (int)a_major; d.b_major = (int)b_major;
  d.lda = lda; d.ldb = ldb; d.ldc = ldc; d.ldd = ldd; d.a_gstride = a_gs; d.b_gstride = b_gs; d.c_gstride = c_gs;
  d.tile_group = (const int*)ptr_or_null(tile_group); d.num_m_tiles = (const int*)ptr_or_null(num_m_tiles);
  d.k_begin = (const int*)ptr_or_null(k_begin); d.k_len = (const int*)ptr_or_null(k_len);
  d.out_f32 = C.scalar_type() == at::kFloat ? 1 : 0;
  TORCH_CHECK(d.out_f32 || C.scalar_type() == at::kBFloat16, "C must be bf16 or fp32");
  if (D.has_value() && D->defined()) TORCH_CHECK(D->scalar_type() == C.scalar_type(), "D must have C's dtype");
  d.alpha = (float)alpha; d.beta = (float)beta; d.row_scale = (const float*)ptr_or_null(row_scale);
  if (row_ptr.has_value() && row_ptr->defined()) {
    TORCH_CHECK(row_ptr->scalar_type() == at::kLong && row_ptr->is_contiguous() && row_ptr->numel() >= M &&
                epilogue == KMOE_EPI_STORE, "row_ptr: int64, one entry per output row, plain store epilogue");
    d.c_row_ptr = (const long long*)row_ptr->data_ptr<int64_t>();
  }
  d.sym_upper = sym_upper ? 1 : 0;
  d.diag_add = (float)diag_add;
  d.k_split = (int)k_split;
  const int64_t n_groups = mode == KMOE_GEMM_BATCHED ? groups : 1;
  if (alpha_dev.has_value() && alpha_dev->defined()) {
    need_f32(*alpha_dev, "alpha_dev");
    TORCH_CHECK(alpha_dev->numel() >= n_groups);
    d.alpha_dev = alpha_dev->data_ptr<float>();
  }
  if (beta_dev.has_value() && beta_dev->defined()) {
    need_f32(*beta_dev, "beta_dev");
    TORCH_CHECK(beta_dev->numel() >= n_groups);
    d.beta_dev = beta_dev->data_ptr<float>();
  }
  TORCH_CHECK(status.scalar_type() == at::kInt && status.is_cuda(), "status must be a CUDA int32 tensor");
  d.status = status.data_ptr<int>();
  d.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  check(kmoe_gemm(&d, cur_stream()), "gemm");
}

// ----------------------------------------------------------------- row kernels
std::tuple<Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  check(kmoe_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows, d, (float)eps,
                         cur_stream()), "rmsnorm_fwd");
  return {y, rstd};
}

std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(dy, "dy"); need_f32(rstd, "rstd");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous());
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty({d}, x.options().dtype(at::kFloat));
  Tensor partial = at::empty({kmoe_rmsnorm_bwd_num_partials(rows), d}, x.options().dtype(at::kFloat));
  check(kmoe_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr<float>(), dx.data_ptr(), nullptr,
                         dw.data_ptr<float>(), partial.data_ptr<float>(), rows, d, cur_stream()), "rmsnorm_bwd");
  return {dx, dw};
}

// (sum, y, rstd): sum = x + addend (or x itself when addend is absent), y = rmsnorm(sum)
std::tuple<Tensor, Tensor, Tensor> add_rmsnorm_fwd(const Tensor& x, const OptT& addend, const Tensor& w, double eps) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const bool has = addend.has_value() && addend->defined();
  if (has) { need_bf16(*addend, "addend"); TORCH_CHECK(addend->is_contiguous() && addend->sizes() == x.sizes()); }
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  Tensor y = at::empty_like(x);
  Tensor sum = has ? at::empty_like(x) : x;
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  check(kmoe_add_rmsnorm_fwd(x.data_ptr(), has ? addend->data_ptr() : nullptr, w.data_ptr(),
                             has ? sum.data_ptr() : nullptr, y.data_ptr(), rstd.data_ptr<float>(), rows, d, (float)eps,
                             cur_stream()), "add_rmsnorm_fwd");
  return {sum, y, rstd};
}

// rmsnorm backward with the residual-branch gradient folded in: dx = norm term + dres
std::tuple<Tensor, Tensor> rmsnorm_bwd_res(const Tensor& x, const Tensor& w, const Tensor& dy, const Tensor& rstd,
                                           const OptT& dres) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(dy, "dy"); need_f32(rstd, "rstd");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous());
  const bool has = dres.has_value() && dres->defined();
  if (has) { need_bf16(*dres, "dres"); TORCH_CHECK(dres->is_contiguous() && dres->sizes() == x.sizes()); }
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  Tensor dx = at::empty_like(x);
  Tensor dw = at::empty({d}, x.options().dtype(at::kFloat));
  Tensor partial = at::empty({kmoe_rmsnorm_bwd_num_partials(rows), d}, x.options().dtype(at::kFloat));
  check(kmoe_rmsnorm_bwd_res(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr<float>(),
                             has ? dres->data_ptr() : nullptr, dx.data_ptr(), nullptr, dw.data_ptr<float>(),
                             partial.data_ptr<float>(), rows, d, cur_stream()), "rmsnorm_bwd_res");
  return {dx, dw};
}

Tensor rowdot_fwd(const Tensor& x, const Tensor& w) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(w, "w");
  TORCH_CHECK(x.is_contiguous() && w.is_contiguous());
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  TORCH_CHECK(w.numel() == d, "w must hold one row of d weights");
  Tensor y = at::empty({rows}, x.options());
  check(kmoe_rowdot_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rows, d, cur_stream()), "rowdot_fwd");
  return y;
}

// dw goes to `dw_out` (bf16, d elements) when given, else a new tensor is returned
std::tuple<Tensor, Tensor> rowdot_bwd(const Tensor& x, const Tensor& w, const Tensor& dy, bool need_dx,
                                      const c10::optional<Tensor>& dw_out) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(w, "w"); need_bf16(dy, "dy");
  TORCH_CHECK(x.is_contiguous() && dy.is_contiguous() && w.is_contiguous());
  const int d = x.size(-1);
  const int rows = x.numel() / d;
  TORCH_CHECK(dy.numel() == rows);
  Tensor dx = need_dx ? at::empty_like(x) : Tensor();
  Tensor dw = (dw_out.has_value() && dw_out->defined()) ? *dw_out : at::empty({d}, x.options());
  need_bf16(dw, "dw");
  TORCH_CHECK(dw.is_contiguous() && dw.numel() == d);
  Tensor partial = at::empty({kmoe_rmsnorm_bwd_num_partials(rows), d}, x.options().dtype(at::kFloat));
  check(kmoe_rowdot_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), need_dx ? dx.data_ptr() : nullptr, dw.data_ptr(),
                        nullptr, partial.data_ptr<float>(), rows, d, cur_stream()), "rowdot_bwd");
  return {need_dx ? dx : at::empty({0}, x.options()), dw};
}

Tensor sumsq(const Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous(), "x must be contiguous");
  Tensor partial = at::empty({kmoe_sumsq_num_partials()}, x.options().dtype(at::kFloat));
  Tensor out = at::empty({1}, x.options().dtype(at::kFloat));
  check(kmoe_sumsq_bf16(x.data_ptr(), x.numel(), partial.data_ptr<float>(), out.data_ptr<float>(), cur_stream()),
        "sumsq");
  return out;
}

void scale_copy(const Tensor& src, Tensor dst, const Tensor& scale) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src"); need_bf16(dst, "dst"); need_f32(scale, "scale");
  TORCH_CHECK(src.is_contiguous() && dst.is_contiguous() && src.numel() == dst.numel() && scale.numel() >= 1);
  check(kmoe_scale_copy(src.data_ptr(), dst.data_ptr(), src.numel(), scale.data_ptr<float>(), cur_stream()),
        "scale_copy");
}

void sum_partials(const Tensor& partial, Tensor out) {
  c10::cuda::CUDAGuard guard(partial.device());
  need_f32(partial, "partial"); need_bf16(out, "out");
  TORCH_CHECK(partial.is_contiguous() && out.is_contiguous() && partial.dim() >= 2);
  const int64_t n = out.numel();
  TORCH_CHECK(partial.numel() == partial.size(0) * n && n % 4 == 0, "partial must be [parts, out.numel()]");
  check(kmoe_sum_partials(partial.data_ptr<float>(), out.data_ptr(), (int)partial.size(0), n, cur_stream()),
        "sum_partials");
}

Tensor rope(const Tensor& x, const Tensor& cs, const Tensor& sn, bool transpose) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_f32(cs, "cos"); need_f32(sn, "sin");
  TORCH_CHECK(x.dim() == 4 && x.is_contiguous(), "x must be contiguous [B,S,H,D]");
  const int B = x.size(0), S = x.size(1), H = x.size(2), D = x.size(3);
  long long bstride = 0;
  if (cs.dim() == 3 && cs.size(0) > 1) bstride = (long long)S * D;
  TORCH_CHECK(cs.size(-1) == D && cs.size(-2) == S, "cos/sin must be [S,D] or [B,S,D]");
  Tensor out = at::empty_like(x);
  check(kmoe_rope(x.data_ptr(), cs.data_ptr<float>(), sn.data_ptr<float>(), out.data_ptr(), B, S, H, D, bstride,
                  transpose ? 1 : 0, cur_stream()), "rope");
  return out;
}

Tensor swiglu_fwd(const Tensor& g, const Tensor& u, const OptT& live_rows) {
  c10::cuda::CUDAGuard guard(g.device());
  need_bf16(g, "gate"); need_bf16(u, "up");
  const int cols = g.size(-1);
  const long long rows = g.numel() / cols;
  Tensor g2 = g.dim() == 1 ? g.unsqueeze(0) : g, u2 = u.dim() == 1 ? u.unsqueeze(0) : u;
  Tensor h = at::empty(g.sizes(), g.options());
  check(kmoe_swiglu_fwd(g2.data_ptr(), u2.data_ptr(), h.data_ptr(), rows, cols, row_stride(g2), row_stride(u2),
                        (const int*)ptr_or_null(live_rows), cur_stream()), "swiglu_fwd");
  return h;
}

std::tuple<Tensor, Tensor> swiglu_bwd(const Tensor& g, const Tensor& u, const Tensor& dh, const OptT& live_rows) {
  c10::cuda::CUDAGuard guard(g.device());
  need_bf16(g, "gate"); need_bf16(u, "up"); need_bf16(dh, "dh");
  TORCH_CHECK(dh.is_contiguous());
  const int cols = g.size(-1);
  const long long rows = g.numel() / cols;
  Tensor g2 = g.dim() == 1 ? g.unsqueeze(0) : g, u2 = u.dim() == 1 ? u.unsqueeze(0) : u;
  Tensor dg = at::empty(g.sizes(), g.options()), du = at::empty(g.sizes(), g.options());
  check(kmoe_swiglu_bwd(g2.data_ptr(), u2.data_ptr(), dh.data_ptr(), dg.data_ptr(), du.data_ptr(), rows, cols,
                        row_stride(g2), row_stride(u2), cols, (const int*)ptr_or_null(live_rows), cur_stream()),
        "swiglu_bwd");
  return {dg, du};
}

// dG and dU side by side in one (rows, 2 * cols) buffer: the [dG | dU] operand of a split-reduction GEMM
Tensor swiglu_bwd_cat(const Tensor& g, const Tensor& u, const Tensor& dh, const OptT& live_rows) {
  c10::cuda::CUDAGuard guard(g.device());
  need_bf16(g, "gate"); need_bf16(u, "up"); need_bf16(dh, "dh");
  TORCH_CHECK(dh.is_contiguous() && g.dim() == 2);
  const int cols = g.size(-1);
  const long long rows = g.numel() / cols;
  Tensor out = at::empty({rows, 2 * (long long)cols}, g.options());
  char* base = reinterpret_cast<char*>(out.data_ptr());
  check(kmoe_swiglu_bwd(g.data_ptr(), u.data_ptr(), dh.data_ptr(), base, base + 2LL * cols, rows, cols, row_stride(g),
                        row_stride(u), 2LL * cols, (const int*)ptr_or_null(live_rows), cur_stream()),
        "swiglu_bwd_cat");
  return out;
}

// ------------------------------------------------------------------------ Mamba
Tensor conv1d_fwd(const Tensor& x, const Tensor& w, const OptT& bias, bool act) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_f32(w, "w");
  // w [C,4], or [G,C,4] with G parameter sets: batch entries [g*B/G, (g+1)*B/G) use set g (bias [G,C] then)
  TORCH_CHECK(x.dim() == 3 && (w.dim() == 2 || w.dim() == 3) && w.size(-1) == 4 && w.is_contiguous(),
              "x [B,S,C], w [C,4] or [G,C,4]");
  const int B = x.size(0), S = x.size(1), C = x.size(2);
  const int G = w.dim() == 3 ? (int)w.size(0) : 1;
  TORCH_CHECK(w.size(-2) == C && B % G == 0, "w does not match x");
  Tensor y = at::empty({B, S, C}, x.options());
  check(kmoe_conv1d_fwd(x.data_ptr(), w.data_ptr<float>(), (const float*)ptr_or_null(bias), y.data_ptr(), B, S, C,
                        row_stride(x), act ? 1 : 0, G, cur_stream()), "conv1d_fwd");
  return y;
}

std::tuple<Tensor, Tensor, Tensor> conv1d_bwd(const Tensor& x, const Tensor& w, const OptT& bias, const Tensor& dy,
                                              bool act) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x"); need_bf16(dy, "dy"); need_f32(w, "w");
  TORCH_CHECK(dy.is_contiguous());
  const int B = x.size(0), S = x.size(1), C = x.size(2);
  const int G = w.dim() == 3 ? (int)w.size(0) : 1;
  TORCH_CHECK(w.is_contiguous() && w.size(-2) == C && B % G == 0, "w does not match x");
  Tensor dx = at::empty({B, S, C}, x.options());
  Tensor dw = at::zeros_like(w);
  Tensor db = w.dim() == 3 ? at::zeros({G, C}, w.options()) : at::zeros({C}, w.options());
  check(kmoe_conv1d_bwd(x.data_ptr(), w.data_ptr<float>(), (const float*)ptr_or_null(bias), dy.data_ptr(),
                        dx.data_ptr(), dw.data_ptr<float>(), db.data_ptr<float>(), B, S, C, row_stride(x),
                        act ? 1 : 0, G, cur_stream()), "conv1d_bwd");
  return {dx, dw, db};
}

std::tuple<Tensor, Tensor, Tensor> scan_fwd(const Tensor& u, const Tensor& delta, const OptT& z, const Tensor& A,
                                            const Tensor& Bm, const Tensor& Cm, const OptT& D, const OptT& dt_bias,
                                            bool softplus, bool save) {
  c10::cuda::CUDAGuard guard(u.device());
  need_bf16(u, "u"); need_bf16(delta, "delta"); need_f32(A, "A"); need_f32(Bm, "B"); need_f32(Cm, "C");
  // A [C,N], or [G,C,N] with G parameter sets over the batch (D, dt_bias [G,C] then)
  TORCH_CHECK(u.is_contiguous() && delta.is_contiguous() && u.dim() == 3 && A.is_contiguous());
  const int B = u.size(0), S = u.size(1), C = u.size(2), N = A.size(-1);
  const int G = A.dim() == 3 ? (int)A.size(0) : 1;
  TORCH_CHECK(A.size(-2) == C && B % G == 0, "A does not match u");
  Tensor out = at::empty_like(u);
  const int nch = (S + kmoe_scan_chunk() - 1) / kmoe_scan_chunk();
  Tensor ckpt = save ? at::empty({B, nch, N, C}, A.options()) : at::empty({0}, A.options());
  const int P = kmoe_scan_segments(B, S, C);
  Tensor seg = P > 1 ? at::empty({B, P, N + 1, C}, A.options()) : at::empty({0}, A.options());
  const bool has_z = z.has_value() && z->defined();
  if (has_z) need_bf16(*z, "z");
  check(kmoe_scan_fwd(u.data_ptr(), delta.data_ptr(), has_z ? z->data_ptr() : nullptr, A.data_ptr<float>(),
                      Bm.data_ptr<float>(), Cm.data_ptr<float>(), (const float*)ptr_or_null(D),
                      (const float*)ptr_or_null(dt_bias), out.data_ptr(), save ? ckpt.data_ptr<float>() : nullptr,
                      P > 1 ? seg.data_ptr<float>() : nullptr, B, S, C, N, has_z ? row_stride(*z) : 0,
                      softplus ? 1 : 0, G, cur_stream()), "scan_fwd");
  return {out, ckpt, seg};
}

std::vector<Tensor> scan_bwd(const Tensor& u, const Tensor& delta, const OptT& z, const Tensor& A, const Tensor& Bm,
                             const Tensor& Cm, const OptT& D, const OptT& dt_bias, const Tensor& dout,
                             const Tensor& ckpt, const Tensor& seg, bool softplus) {
  c10::cuda::CUDAGuard guard(u.device());
  need_bf16(dout, "dout");
  TORCH_CHECK(dout.is_contiguous());
  const int B = u.size(0), S = u.size(1), C = u.size(2), N = A.size(-1);
  const int G = A.dim() == 3 ? (int)A.size(0) : 1;
  TORCH_CHECK(A.is_contiguous() && A.size(-2) == C && B % G == 0, "A does not match u");
  const bool has_z = z.has_value() && z->defined();
  Tensor du = at::empty_like(u), dd = at::empty_like(u);
  Tensor dz = has_z ? at::empty({B, S, C}, u.options()) : at::empty({0}, u.options());
  auto f32 = A.options();
  Tensor dA = at::zeros_like(A), dB = at::zeros({B, S, N}, f32), dC = at::zeros({B, S, N}, f32);
  Tensor dD = A.dim() == 3 ? at::zeros({G, C}, f32) : at::zeros({C}, f32);
  Tensor dbias = at::zeros_like(dD);
  const int P = kmoe_scan_segments(B, S, C);
  TORCH_CHECK(P == 1 || seg.numel() == (int64_t)B * P * (N + 1) * C, "segment scratch of the forward pass expected");
  Tensor gseg = P > 1 ? at::empty({B, P, N, C}, f32) : at::empty({0}, f32);
  check(kmoe_scan_bwd(u.data_ptr(), delta.data_ptr(), has_z ? z->data_ptr() : nullptr, A.data_ptr<float>(),
                      Bm.data_ptr<float>(), Cm.data_ptr<float>(), (const float*)ptr_or_null(D),
                      (const float*)ptr_or_null(dt_bias), dout.data_ptr(), ckpt.data_ptr<float>(),
                      P > 1 ? seg.data_ptr<float>() : nullptr, P > 1 ? gseg.data_ptr<float>() : nullptr, du.data_ptr(),
                      dd.data_ptr(), has_z ? dz.data_ptr() : nullptr, C, dA.data_ptr<float>(), dB.data_ptr<float>(),
                      dC.data_ptr<float>(), dD.data_ptr<float>(), dbias.data_ptr<float>(), B, S, C, N,
                      has_z ? row_stride(*z) : 0, softplus ? 1 : 0, G, cur_stream()), "scan_bwd");
  return {du, dd, dz, dA, dB, dC, dD, dbias};
}

// -------------------------------------------------------------------------- MoE
std::vector<Tensor> moe_plan(const Tensor& idx, const OptT& keep, int64_t E, int64_t expert_base) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous(), "idx must be contiguous int64");
  const int n = idx.numel();
  const int max_rows = kmoe_moe_max_rows(n, (int)E);
  auto i32 = idx.options().dtype(at::kInt);
  Tensor pos = at::empty({n}, i32), row_src = at::empty({max_rows}, i32), counts = at::empty({E}, i32);
  Tensor offsets = at::empty({E + 1}, i32), tile_group = at::empty({max_rows / 128}, i32), meta = at::empty({2}, i32);
  const unsigned char* kp = nullptr;
  Tensor k8;
  if (keep.has_value() && keep->defined()) {
    k8 = keep->to(at::kByte).contiguous();
    kp = k8.data_ptr<unsigned char>();
  }
  check(kmoe_moe_plan((const long long*)idx.data_ptr<int64_t>(), kp, n, (int)E, max_rows, (int)expert_base,
                      pos.data_ptr<int>(), row_src.data_ptr<int>(), counts.data_ptr<int>(), offsets.data_ptr<int>(),
                      tile_group.data_ptr<int>(), meta.data_ptr<int>(), cur_stream()), "moe_plan");
  return {pos, row_src, counts, offsets, tile_group, meta};
}

Tensor moe_capacity_mask(const Tensor& idx, int64_t E, int64_t cap) {
  c10::cuda::CUDAGuard guard(idx.device());
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous(), "idx must be contiguous int64");
  Tensor keep = at::empty(idx.sizes(), idx.options().dtype(at::kBool));
  if (idx.numel() > 0)
    check(kmoe_moe_capacity_mask((const long long*)idx.data_ptr<int64_t>(), (int)idx.numel(), (int)E, (int)cap,
                                 (unsigned char*)keep.data_ptr(), cur_stream()), "moe_capacity_mask");
  return keep;
}

// expert indices [T, k] of the balanced assignment (non-differentiable; weights are gathered by the caller)
Tensor moe_balanced_assign(const Tensor& probs, int64_t k, int64_t cap) {
  c10::cuda::CUDAGuard guard(probs.device());
  need_f32(probs, "probs");
  TORCH_CHECK(probs.dim() == 2);
  const int T = probs.size(0), E = probs.size(1);
  Tensor taken = at::zeros({T, E}, probs.options().dtype(at::kByte));
  Tensor counts = at::zeros({k + 1, E}, probs.options().dtype(at::kInt));
  Tensor sel = at::empty({T, k}, probs.options().dtype(at::kLong));
  if (T > 0)
    check(kmoe_moe_balanced_assign(probs.data_ptr<float>(), taken.data_ptr<unsigned char>(), counts.data_ptr<int>(),
                                   (long long*)sel.data_ptr<int64_t>(), T, E, (int)k, (int)cap, cur_stream()),
          "moe_balanced_assign");
  return sel;
}

Tensor moe_gather_rows(const Tensor& src, const Tensor& row_src, const OptT& assign_scale, const Tensor& meta,
                       int64_t div) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src");
  TORCH_CHECK(src.is_contiguous() && src.dim() == 2);
  const int max_rows = row_src.numel(), d = src.size(1);
  Tensor dst = at::empty({max_rows, d}, src.options());
  check(kmoe_moe_gather_rows(src.data_ptr(), row_src.data_ptr<int>(), (const float*)ptr_or_null(assign_scale),
                             meta.data_ptr<int>(), dst.data_ptr(), max_rows, d, (int)div, cur_stream()),
        "moe_gather_rows");
  return dst;
}

Tensor moe_combine(const Tensor& Y, const Tensor& pos, const OptT& w, int64_t T, int64_t k) {
  c10::cuda::CUDAGuard guard(Y.device());
  need_bf16(Y, "Y");
  TORCH_CHECK(Y.is_contiguous());
  const int d = Y.size(1);
  Tensor out = at::empty({T, d}, Y.options());
  check(kmoe_moe_combine(Y.data_ptr(), pos.data_ptr<int>(), (const float*)ptr_or_null(w), out.data_ptr(), (int)T,
                         (int)k, d, cur_stream()), "moe_combine");
  return out;
}

Tensor moe_combine_dw(const Tensor& Y, const Tensor& dout, const Tensor& pos, int64_t k) {
  c10::cuda::CUDAGuard guard(Y.device());
  need_bf16(Y, "Y"); need_bf16(dout, "dout");
  TORCH_CHECK(Y.is_contiguous() && dout.is_contiguous());
  const int n = pos.numel(), d = Y.size(1);
  Tensor dw = at::empty({n}, Y.options().dtype(at::kFloat));
  check(kmoe_moe_combine_dw(Y.data_ptr(), dout.data_ptr(), pos.data_ptr<int>(), dw.data_ptr<float>(), n, (int)k, d,
                            cur_stream()), "moe_combine_dw");
  return dw;
}

// -------------------------------------------------------------------- attention
static const int* doc_ptr(const OptT& doc_start, int64_t B, int64_t S) {
  if (!doc_start.has_value() || !doc_start->defined()) return nullptr;
  TORCH_CHECK(doc_start->is_cuda() && doc_start->scalar_type() == at::kInt && doc_start->is_contiguous() &&
              doc_start->numel() == B * S, "doc_start must be a contiguous (B, S) int32 CUDA tensor");
  return doc_start->data_ptr<int>();
}

std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, double scale,
                                    const OptT& doc_start, Tensor status) {
  c10::cuda::CUDAGuard guard(q.device());
  need_bf16(q, "q"); need_bf16(k, "k"); need_bf16(v, "v");
  TORCH_CHECK(q.is_contiguous() && k.is_contiguous() && v.is_contiguous() && q.dim() == 4);
  const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  Tensor out = at::empty_like(q);
  Tensor lse = at::empty({B, H, S}, q.options().dtype(at::kFloat));
  check(kmoe_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr<float>(), B, S, H, Hkv,
                      D, (float)scale, doc_ptr(doc_start, B, S), status.data_ptr<int>(), cur_stream()), "attn_fwd");
  return {out, lse};
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                                            const Tensor& d_o, const Tensor& lse, double scale, const OptT& doc_start,
                                            Tensor status) {
  c10::cuda::CUDAGuard guard(q.device());
  need_bf16(d_o, "do");
  TORCH_CHECK(d_o.is_contiguous() && o.is_contiguous());
  const int B = q.size(0), S = q.size(1), H = q.size(2), D = q.size(3), Hkv = k.size(2);
  Tensor dq = at::empty_like(q), dk = at::empty_like(k), dv = at::empty_like(v);
  Tensor delta = at::empty({B, H, S}, lse.options());
  check(kmoe_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr<float>(),
                      delta.data_ptr<float>(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), B, S, H, Hkv, D,
                      (float)scale, doc_ptr(doc_start, B, S), status.data_ptr<int>(), cur_stream()), "attn_bwd");
  return {dq, dk, dv};
}

// ------------------------------------------------------------------------- loss
Tensor ce_fwd_bwd(Tensor logits, const Tensor& labels, const Tensor& grad_scale, int64_t ignore_index,
                  bool write_grad) {
  c10::cuda::CUDAGuard guard(logits.device());
  need_bf16(logits, "logits"); need_f32(grad_scale, "grad_scale");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1);
  TORCH_CHECK(labels.scalar_type() == at::kLong && labels.is_contiguous() && labels.numel() == logits.size(0));
  Tensor loss_rows = at::empty({logits.size(0)}, logits.options().dtype(at::kFloat));
  check(kmoe_ce_fwd_bwd(logits.data_ptr(), (const long long*)labels.data_ptr<int64_t>(), loss_rows.data_ptr<float>(),
                        grad_scale.data_ptr<float>(), (int)logits.size(0), (int)logits.size(1), logits.stride(0),
                        ignore_index, write_grad ? 1 : 0, cur_stream()), "ce_fwd_bwd");
  return loss_rows;
}

// ------------------------------------------------------------- peer-to-peer collectives
void p2p_barrier(std::vector<int64_t> flag_ptrs, int64_t rank, int64_t world, int64_t epoch, double timeout_s,
                 Tensor status) {
  c10::cuda::CUDAGuard guard(status.device());
  check(kmoe_p2p_barrier((const long long*)flag_ptrs.data(), (int)rank, (int)world, (int)epoch, timeout_s,
                         status.data_ptr<int>(), cur_stream()), "p2p_barrier");
}

void p2p_reduce_scatter(std::vector<int64_t> grad_ptrs, int64_t rank, int64_t world, int64_t off, int64_t n,
                        const OptT& sq_out, int64_t mc_ptr, int64_t max_blocks) {
  check(kmoe_p2p_reduce_scatter((const long long*)grad_ptrs.data(), (int)rank, (int)world, off, n,
                                (float*)const_cast<void*>(ptr_or_null(sq_out)), mc_ptr, (int)max_blocks,
                                cur_stream()),
        "p2p_reduce_scatter");
}

void p2p_adamw_allgather(std::vector<int64_t> param_ptrs, const Tensor& grad, Tensor m, Tensor v, int64_t rank,
                         int64_t world, int64_t off, int64_t n, double lr, double beta1, double beta2, double eps,
                         double wd, int64_t step, const OptT& clip_coef, int64_t mc_ptr) {
  c10::cuda::CUDAGuard guard(grad.device());
  need_bf16(grad, "grad"); need_f32(m, "m"); need_f32(v, "v");
  TORCH_CHECK(m.numel() >= n && v.numel() >= n, "moment buffers too small");
  check(kmoe_p2p_adamw_allgather((const long long*)param_ptrs.data(), grad.data_ptr(), m.data_ptr<float>(),
                                 v.data_ptr<float>(), (int)rank, (int)world, off, n, (float)lr, (float)beta1,
                                 (float)beta2, (float)eps, (float)wd, (int)step, (const float*)ptr_or_null(clip_coef),
                                 mc_ptr, cur_stream()), "p2p_adamw_allgather");
}

void p2p_allgather(std::vector<int64_t> buf_ptrs, int64_t rank, int64_t world, int64_t off, int64_t n,
                   int64_t mc_ptr, const OptT& src, int64_t max_blocks) {
  if (src.has_value()) {
    need_bf16(*src, "src");
    TORCH_CHECK(src->is_contiguous() && src->numel() >= n, "src too small or not contiguous");
  }
  check(kmoe_p2p_allgather((const long long*)buf_ptrs.data(), (int)rank, (int)world, off, n, mc_ptr,
                           ptr_or_null(src), (int)max_blocks, cur_stream()),
        "p2p_allgather");
}

// ------------------------------------------------------------- mixture-of-depths rows
static void check_idx(const Tensor& idx) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous() && idx.dim() == 2,
              "idx must be a contiguous (B, k) int64 CUDA tensor");
}

Tensor rows_gather(const Tensor& src, const Tensor& idx) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src"); check_idx(idx);
  TORCH_CHECK(src.is_contiguous() && src.dim() == 3);
  const int B = src.size(0), S = src.size(1), d = src.size(2), k = idx.size(1);
  Tensor out = at::empty({B, k, d}, src.options());
  check(kmoe_rows_gather(src.data_ptr(), (const long long*)idx.data_ptr<int64_t>(), out.data_ptr(), B, S, k, d,
                         cur_stream()), "rows_gather");
  return out;
}

Tensor rows_scatter(const Tensor& src, const Tensor& idx, int64_t S) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src"); check_idx(idx);
  TORCH_CHECK(src.is_contiguous() && src.dim() == 3);
  const int B = src.size(0), k = src.size(1), d = src.size(2);
  Tensor out = at::empty({B, S, d}, src.options());
  check(kmoe_rows_scatter(src.data_ptr(), (const long long*)idx.data_ptr<int64_t>(), out.data_ptr(), B, (int)S, k, d,
                          cur_stream()), "rows_scatter");
  return out;
}

Tensor rows_scatter_rank1(const Tensor& src, const Tensor& idx, int64_t S, const Tensor& coef, const Tensor& wvec) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src"); need_bf16(coef, "coef"); need_bf16(wvec, "wvec"); check_idx(idx);
  TORCH_CHECK(src.is_contiguous() && src.dim() == 3 && coef.is_contiguous() && wvec.is_contiguous());
  const int B = src.size(0), k = src.size(1), d = src.size(2);
  TORCH_CHECK(coef.numel() == (int64_t)B * S && wvec.numel() == d, "coef must hold B * S values, wvec d values");
  Tensor out = at::empty({B, S, d}, src.options());
  check(kmoe_rows_scatter_rank1(src.data_ptr(), (const long long*)idx.data_ptr<int64_t>(), coef.data_ptr(),
                                wvec.data_ptr(), out.data_ptr(), B, (int)S, k, d, cur_stream()),
        "rows_scatter_rank1");
  return out;
}

std::tuple<Tensor, Tensor> mod_bce(const Tensor& logits, const Tensor& idx) {
  c10::cuda::CUDAGuard guard(logits.device());
  need_bf16(logits, "logits"); check_idx(idx);
  TORCH_CHECK(logits.is_contiguous() && logits.dim() == 2 && idx.size(0) == logits.size(0));
  Tensor loss = at::empty({1}, logits.options().dtype(at::kFloat));
  Tensor partial = at::empty({kmoe_mod_bce_num_partials((int)logits.size(0), (int)logits.size(1))},
                             logits.options().dtype(at::kFloat));
  Tensor dl = at::empty_like(logits);
  check(kmoe_mod_bce(logits.data_ptr(), (const long long*)idx.data_ptr<int64_t>(), partial.data_ptr<float>(),
                     loss.data_ptr<float>(), dl.data_ptr(), (int)logits.size(0), (int)logits.size(1),
                     (int)idx.size(1), cur_stream()),
        "mod_bce");
  return {loss, dl};
}

Tensor mod_combine_fwd(const Tensor& res, const Tensor& proc, const Tensor& w, const Tensor& idx) {
  c10::cuda::CUDAGuard guard(res.device());
  need_bf16(res, "res"); need_bf16(proc, "proc"); need_f32(w, "w"); check_idx(idx);
  TORCH_CHECK(res.is_contiguous() && proc.is_contiguous() && res.dim() == 3 && proc.dim() == 3);
  const int B = res.size(0), S = res.size(1), d = res.size(2), k = proc.size(1);
  Tensor out = at::empty_like(res);
  check(kmoe_mod_combine_fwd(res.data_ptr(), proc.data_ptr(), w.data_ptr<float>(),
                             (const long long*)idx.data_ptr<int64_t>(), out.data_ptr(), B, S, k, d, cur_stream()),
        "mod_combine_fwd");
  return out;
}

std::tuple<Tensor, Tensor> mod_combine_bwd(const Tensor& dout, const Tensor& proc, const Tensor& w, const Tensor& idx) {
  c10::cuda::CUDAGuard guard(dout.device());
  need_bf16(dout, "dout"); need_bf16(proc, "proc"); need_f32(w, "w"); check_idx(idx);
  TORCH_CHECK(dout.is_contiguous() && proc.is_contiguous());
  const int B = dout.size(0), S = dout.size(1), d = dout.size(2), k = proc.size(1);
  Tensor dproc = at::empty_like(proc);
  Tensor dw = at::empty({B, k}, w.options());
  check(kmoe_mod_combine_bwd(dout.data_ptr(), proc.data_ptr(), w.data_ptr<float>(),
                             (const long long*)idx.data_ptr<int64_t>(), dproc.data_ptr(), dw.data_ptr<float>(), B, S,
                             k, d, cur_stream()), "mod_combine_bwd");
  return {dproc, dw};
}

// ------------------------------------------------------------- Muon elementwise passes
void muon_momentum(Tensor buf, const Tensor& grad_ptrs, Tensor sumsq, double mu, const OptT& gcoef) {
  c10::cuda::CUDAGuard guard(buf.device());
  need_bf16(buf, "buf"); need_f32(sumsq, "sumsq");
  TORCH_CHECK(buf.is_contiguous() && buf.dim() == 3 && grad_ptrs.scalar_type() == at::kLong &&
              grad_ptrs.numel() == buf.size(0) && sumsq.numel() == buf.size(0));
  check(kmoe_muon_momentum(buf.data_ptr(), (const long long*)grad_ptrs.data_ptr<int64_t>(), sumsq.data_ptr<float>(),
                           (int)buf.size(0), buf.size(1) * buf.size(2), (float)mu, (const float*)ptr_or_null(gcoef),
                           cur_stream()), "muon_momentum");
}

void muon_apply(Tensor buf, const Tensor& ortho, const Tensor& grad_ptrs, const Tensor& param_ptrs, double lr,
                double mu, double wd, bool nesterov, const OptT& gcoef) {
  c10::cuda::CUDAGuard guard(buf.device());
  need_bf16(buf, "buf"); need_bf16(ortho, "ortho");
  TORCH_CHECK(buf.is_contiguous() && ortho.is_contiguous() && buf.sizes() == ortho.sizes() && buf.dim() == 3);
  TORCH_CHECK(grad_ptrs.numel() == buf.size(0) && param_ptrs.numel() == buf.size(0));
  check(kmoe_muon_apply(buf.data_ptr(), ortho.data_ptr(), (const long long*)grad_ptrs.data_ptr<int64_t>(),
                        (const long long*)param_ptrs.data_ptr<int64_t>(), (int)buf.size(0), buf.size(1) * buf.size(2),
                        (float)lr, (float)mu, (float)wd, nesterov ? 1 : 0, (const float*)ptr_or_null(gcoef),
                        cur_stream()), "muon_apply");
}

// int8 block-quantised momentum (Muon8bit): returns (q [blocks, block] int8, scales [blocks, 1] fp32)
std::tuple<Tensor, Tensor> q8_quant(const Tensor& x, int64_t block) {
  c10::cuda::CUDAGuard guard(x.device());
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && (x.scalar_type() == at::kFloat || x.scalar_type() == at::kBFloat16),
              "x must be a contiguous CUDA fp32 or bf16 tensor");
  const int64_t n = x.numel(), nb = (n + block - 1) / block;
  Tensor q = at::empty({nb, block}, x.options().dtype(at::kChar));
  Tensor sc = at::empty({nb, 1}, x.options().dtype(at::kFloat));
  check(kmoe_q8_quant(x.data_ptr(), x.scalar_type() == at::kBFloat16, (signed char*)q.data_ptr(), sc.data_ptr<float>(),
                      n, (int)block, cur_stream()), "q8_quant");
  return {q, sc};
}

// mu * dequant(q, scales) + g, shaped and typed like g
Tensor q8_momentum(const Tensor& q, const Tensor& scales, const Tensor& g, double mu) {
  c10::cuda::CUDAGuard guard(g.device());
  TORCH_CHECK(g.is_cuda() && g.is_contiguous() && (g.scalar_type() == at::kFloat || g.scalar_type() == at::kBFloat16));
  TORCH_CHECK(q.scalar_type() == at::kChar && q.is_contiguous() && q.dim() == 2 && q.numel() >= g.numel());
  need_f32(scales, "scales");
  TORCH_CHECK(scales.numel() == q.size(0));
  Tensor out = at::empty_like(g);
  check(kmoe_q8_momentum((const signed char*)q.data_ptr(), scales.data_ptr<float>(), g.data_ptr(),
                         g.scalar_type() == at::kBFloat16, out.data_ptr(), g.numel(), (int)q.size(1), (float)mu,
                         cur_stream()), "q8_momentum");
  return out;
}

// ------------------------------------------------------------- MXFP8
// x: (..., C) bf16 with collapsing leading dims -> (q e4m3 same shape, scale chunks uint8)
std::vector<Tensor> mx_quant_rows(const Tensor& x, const OptT& x2, const OptT& live_rows) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x");
  TORCH_CHECK(x.dim() >= 2);
  const long long ld = row_stride(x);
  const int64_t C = x.size(-1), rows = x.numel() / C;
  if (x2.has_value() && x2->defined()) {
    need_bf16(*x2, "x2");
    TORCH_CHECK(x2->sizes() == x.sizes() && row_stride(*x2) == ld, "x2 must match x");
  }
  Tensor q = at::empty(x.sizes(), x.options().dtype(at::kFloat8_e4m3fn));
  Tensor sf = at::zeros({kmoe_mx_sf_bytes(rows, C)}, x.options().dtype(at::kByte));
  check(kmoe_mx_quant_rows(x.data_ptr(), ptr_or_null(x2), rows, (int)C, ld, q.data_ptr(), sf.data_ptr(),
                           (const int*)ptr_or_null(live_rows), cur_stream()), "mx_quant_rows");
  return {q, sf};
}

// x: (R, C) or (G, R, C) bf16 contiguous -> (q e4m3 (G, C, R), scale chunks)
std::vector<Tensor> mx_quant_cols(const Tensor& x, const OptT& live_rows) {
  c10::cuda::CUDAGuard guard(x.device());
  need_bf16(x, "x");
  TORCH_CHECK(x.is_contiguous() && (x.dim() == 2 || x.dim() == 3));
  const int64_t G = x.dim() == 3 ? x.size(0) : 1, R = x.size(-2), C = x.size(-1);
  Tensor q = x.dim() == 3 ? at::empty({G, C, R}, x.options().dtype(at::kFloat8_e4m3fn))
                          : at::empty({C, R}, x.options().dtype(at::kFloat8_e4m3fn));
  Tensor sf = at::zeros({kmoe_mx_sf_bytes(G * C, R)}, x.options().dtype(at::kByte));
  check(kmoe_mx_quant_cols(x.data_ptr(), (int)G, R, (int)C, C, R * C, q.data_ptr(), sf.data_ptr(),
                           (const int*)ptr_or_null(live_rows), cur_stream()), "mx_quant_cols");
  return {q, sf};
}

void gemm_mxfp8(const Tensor& A, const Tensor& sfa, const Tensor& B, const Tensor& sfb, Tensor C, const OptT& D,
                int64_t mode, int64_t M, int64_t N, int64_t K, int64_t groups, bool a_grouped, bool b_grouped,
                int64_t ldc, int64_t ldd, int64_t c_gs, const OptT& tile_group, const OptT& num_m_tiles,
                const OptT& k_begin, const OptT& k_len, double alpha, double beta, Tensor status) {
  c10::cuda::CUDAGuard guard(A.device());
  TORCH_CHECK(A.scalar_type() == at::kFloat8_e4m3fn && B.scalar_type() == at::kFloat8_e4m3fn && A.is_contiguous() &&
              B.is_contiguous(), "A and B must be contiguous float8_e4m3fn tensors");
  TORCH_CHECK(sfa.scalar_type() == at::kByte && sfb.scalar_type() == at::kByte);
  TORCH_CHECK(sfa.numel() >= kmoe_mx_sf_bytes((a_grouped ? groups : 1) * M, K), "A scale buffer too small");
  TORCH_CHECK(sfb.numel() >= kmoe_mx_sf_bytes((b_grouped ? groups : 1) * N, K), "B scale buffer too small");
  KmoeMxGemmDesc d{};
  d.A = A.data_ptr(); d.B = B.data_ptr(); d.sfa = sfa.data_ptr(); d.sfb = sfb.data_ptr();
  d.C = C.data_ptr(); d.D = ptr_or_null(D);
  d.mode = (int)mode; d.M = (int)M; d.N = (int)N; d.K = (int)K; d.groups = (int)groups;
  d.a_grouped = a_grouped; d.b_grouped = b_grouped;
  d.ldc = ldc; d.ldd = ldd; d.c_gstride = c_gs;
  d.tile_group = (const int*)ptr_or_null(tile_group); d.num_m_tiles = (const int*)ptr_or_null(num_m_tiles);
  d.k_begin = (const int*)ptr_or_null(k_begin); d.k_len = (const int*)ptr_or_null(k_len);
  d.out_f32 = C.scalar_type() == at::kFloat ? 1 : 0;
  TORCH_CHECK(d.out_f32 || C.scalar_type() == at::kBFloat16, "C must be bf16 or fp32");
  if (D.has_value() && D->defined()) TORCH_CHECK(D->scalar_type() == C.scalar_type(), "D must have C's dtype");
  d.alpha = (float)alpha; d.beta = (float)beta;
  d.status = status.data_ptr<int>();
  d.num_sms = at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  check(kmoe_gemm_mxfp8(&d, cur_stream()), "gemm_mxfp8");
}

// ------------------------------------------------------------- routing decisions
std::vector<Tensor> route_topk_fwd(const Tensor& logits, int64_t k) {
  c10::cuda::CUDAGuard guard(logits.device());
  need_f32(logits, "logits");
  TORCH_CHECK(logits.dim() == 2 && logits.is_contiguous());
  const int64_t T = logits.size(0), E = logits.size(1);
  auto of = logits.options();
  Tensor w = at::empty({T, k}, of), idx = at::empty({T, k}, of.dtype(at::kLong)), lse = at::empty({T}, of);
  Tensor acc = at::zeros({2 * E + 1}, of);   // [0,E) sum of probabilities, [E,2E) counts, [2E] sum lse^2
  float* a = acc.data_ptr<float>();
  check(kmoe_route_topk_fwd(logits.data_ptr<float>(), (int)T, (int)E, (int)k, w.data_ptr<float>(),
                            (long long*)idx.data_ptr<int64_t>(), lse.data_ptr<float>(), a, a + E, a + 2 * E,
                            cur_stream()), "route_topk_fwd");
  return {w, idx, lse, acc};
}

Tensor route_topk_bwd(const Tensor& logits, const Tensor& lse, const Tensor& idx, const Tensor& w, const OptT& dw,
                      const Tensor& acc, const OptT& d_aux, double w_lb, double w_z) {
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1), k = idx.size(1);
  Tensor dl = at::empty_like(logits);
  check(kmoe_route_topk_bwd(logits.data_ptr<float>(), lse.data_ptr<float>(), (const long long*)idx.data_ptr<int64_t>(),
                            w.data_ptr<float>(), (const float*)ptr_or_null(dw), acc.data_ptr<float>() + E,
                            (const float*)ptr_or_null(d_aux), (float)w_lb, (float)w_z, (int)T, (int)E, (int)k,
                            dl.data_ptr<float>(), cur_stream()), "route_topk_bwd");
  return dl;
}

// scores: contiguous fp32; (rows, S) when rows_inner == rows, or (outer, S, rows_inner) for column-wise rows
std::vector<Tensor> seq_topk_fwd(const Tensor& scores, int64_t row_stride, int64_t col_stride, int64_t rows_inner,
                                 int64_t outer_stride, int64_t rows, int64_t S, int64_t k, int64_t mode) {
  c10::cuda::CUDAGuard guard(scores.device());
  need_f32(scores, "scores");
  TORCH_CHECK(scores.is_contiguous());
  auto of = scores.options();
  Tensor idx = at::empty({rows, k}, of.dtype(at::kLong)), w = at::empty({rows, k}, of), stat = at::empty({rows, 3}, of);
  check(kmoe_seq_topk_fwd(scores.data_ptr<float>(), row_stride, col_stride, (int)rows_inner, outer_stride, (int)rows,
                          (int)S, (int)k, (int)mode, (long long*)idx.data_ptr<int64_t>(), w.data_ptr<float>(),
                          stat.data_ptr<float>(), cur_stream()), "seq_topk_fwd");
  return {idx, w, stat};
}

Tensor seq_topk_bwd(const Tensor& scores, int64_t row_stride, int64_t col_stride, int64_t rows_inner,
                    int64_t outer_stride, int64_t rows, int64_t S, int64_t k, int64_t mode, const Tensor& idx,
                    const Tensor& w, const Tensor& dw, const Tensor& stat) {
  c10::cuda::CUDAGuard guard(scores.device());
  need_f32(dw, "dw");
  TORCH_CHECK(dw.is_contiguous());
  Tensor ds = at::empty_like(scores);
  check(kmoe_seq_topk_bwd(scores.data_ptr<float>(), row_stride, col_stride, (int)rows_inner, outer_stride, (int)rows,
                          (int)S, (int)k, (int)mode, (const long long*)idx.data_ptr<int64_t>(), w.data_ptr<float>(),
                          dw.data_ptr<float>(), stat.data_ptr<float>(), ds.data_ptr<float>(), cur_stream()),
        "seq_topk_bwd");
  return ds;
}

// ------------------------------------------------------------- expert-parallel exchange
void ep_dispatch(const Tensor& src, const Tensor& row_src, const OptT& assign_scale, const Tensor& offsets,
                 const Tensor& counts, std::vector<int64_t> recv_ptrs, std::vector<int64_t> meta_ptrs, int64_t rank,
                 int64_t world, int64_t E, int64_t cap, int64_t div) {
  c10::cuda::CUDAGuard guard(src.device());
  need_bf16(src, "src");
  TORCH_CHECK(src.dim() == 2 && src.is_contiguous());
  check(kmoe_ep_dispatch(src.data_ptr(), row_src.data_ptr<int>(), (const float*)ptr_or_null(assign_scale),
                         offsets.data_ptr<int>(), counts.data_ptr<int>(), (const long long*)recv_ptrs.data(),
                         (const long long*)meta_ptrs.data(), (int)rank, (int)world, (int)E, cap, (int)src.size(1),
                         (int)div, (int)row_src.numel(), cur_stream()), "ep_dispatch");
}

std::vector<Tensor> ep_recv_plan(const Tensor& meta_in, int64_t n_local, int64_t world, int64_t max_rows) {
  c10::cuda::CUDAGuard guard(meta_in.device());
  auto o = meta_in.options().dtype(at::kInt);
  Tensor slot_dst = at::empty({n_local * world}, o), offsets = at::empty({n_local + 1}, o);
  Tensor tile_group = at::empty({max_rows / 128}, o), out_meta = at::empty({2}, o);
  check(kmoe_ep_recv_plan(meta_in.data_ptr<int>(), (int)n_local, (int)world, (int)max_rows, slot_dst.data_ptr<int>(),
                          offsets.data_ptr<int>(), tile_group.data_ptr<int>(), out_meta.data_ptr<int>(),
                          cur_stream()), "ep_recv_plan");
  return {slot_dst, offsets, tile_group, out_meta};
}

void ep_move(const Tensor& slots, Tensor packed, const Tensor& meta_in, const Tensor& slot_dst, const Tensor& offsets,
             std::vector<int64_t> ret_ptrs, int64_t rank, int64_t n_local, int64_t world, int64_t cap, int64_t dir,
             const OptT& row_ptr_out) {
  c10::cuda::CUDAGuard guard(packed.device());
  need_bf16(packed, "packed");
  TORCH_CHECK(packed.dim() == 2 && packed.is_contiguous());
  check(kmoe_ep_move(slots.data_ptr(), packed.data_ptr(), meta_in.data_ptr<int>(), slot_dst.data_ptr<int>(),
                     offsets.data_ptr<int>(), (const long long*)ret_ptrs.data(), (int)rank, (int)n_local, (int)world,
                     cap, (int)packed.size(1), (int)packed.size(0), (int)dir,
                     (long long*)const_cast<void*>(ptr_or_null(row_ptr_out)), cur_stream()), "ep_move");
}

}  // namespace

// error-path self test: raises the same way a failed kernel entry point does (no device needed)
void raise_check(int64_t code) { check((int)code, "self_test"); }

TORCH_LIBRARY(kmoe, m) {
  m.def("raise_check", &raise_check);
  m.def("gemm", &gemm);
  m.def("rmsnorm_fwd", &rmsnorm_fwd);
  m.def("rmsnorm_bwd", &rmsnorm_bwd);
  m.def("add_rmsnorm_fwd", &add_rmsnorm_fwd);
  m.def("rmsnorm_bwd_res", &rmsnorm_bwd_res);
  m.def("rope", &rope);
  m.def("rowdot_fwd", &rowdot_fwd);
  m.def("rowdot_bwd", &rowdot_bwd);
  m.def("sum_partials", &sum_partials);
  m.def("sumsq", &sumsq);
  m.def("scale_copy", &scale_copy);
  m.def("swiglu_fwd", &swiglu_fwd);
  m.def("swiglu_bwd", &swiglu_bwd);
  m.def("swiglu_bwd_cat", &swiglu_bwd_cat);
  m.def("conv1d_fwd", &conv1d_fwd);
  m.def("conv1d_bwd", &conv1d_bwd);
  m.def("scan_fwd", &scan_fwd);
  m.def("scan_bwd", &scan_bwd);
  m.def("moe_plan", &moe_plan);
  m.def("moe_capacity_mask", &moe_capacity_mask);
  m.def("moe_balanced_assign", &moe_balanced_assign);
  m.def("moe_gather_rows", &moe_gather_rows);
  m.def("moe_combine", &moe_combine);
  m.def("moe_combine_dw", &moe_combine_dw);
  m.def("ce_fwd_bwd", &ce_fwd_bwd);
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd);
  m.def("p2p_barrier", &p2p_barrier);
  m.def("p2p_reduce_scatter", &p2p_reduce_scatter);
  m.def("p2p_adamw_allgather", &p2p_adamw_allgather);
  m.def("p2p_allgather", &p2p_allgather);
  m.def("rows_gather", &rows_gather);
  m.def("rows_scatter", &rows_scatter);
  m.def("rows_scatter_rank1", &rows_scatter_rank1);
  m.def("mod_bce", &mod_bce);
  m.def("mod_combine_fwd", &mod_combine_fwd);
  m.def("mod_combine_bwd", &mod_combine_bwd);
  m.def("muon_momentum", &muon_momentum);
  m.def("muon_apply", &muon_apply);
  m.def("q8_quant", &q8_quant);
  m.def("q8_momentum", &q8_momentum);
  m.def("mx_quant_rows", &mx_quant_rows);
  m.def("mx_quant_cols", &mx_quant_cols);
  m.def("gemm_mxfp8", &gemm_mxfp8);
  m.def("route_topk_fwd", &route_topk_fwd);
  m.def("route_topk_bwd", &route_topk_bwd);
  m.def("seq_topk_fwd", &seq_topk_fwd);
  m.def("seq_topk_bwd", &seq_topk_bwd);
  m.def("ep_dispatch", &ep_dispatch);
  m.def("ep_recv_plan", &ep_recv_plan);
  m.def("ep_move", &ep_move);
}
