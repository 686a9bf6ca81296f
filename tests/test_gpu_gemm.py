"""tcgen05 GEMM against an fp32 PyTorch reference: operand majors, tile edges, grouped and
batched (ragged-K) schedules, the SwiGLU and axpby epilogues."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    from kolmogorov_moe_architecture_b200.ops import cuda_ops
    return cuda_ops


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def _close(out, ref, tol=2e-2):
    err = (out.float() - ref).abs().max().item()
    den = ref.abs().max().item() + 1e-6
    assert err / den < tol, f"rel err {err / den:.4g} (abs {err:.4g})"


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (300, 264, 200), (4096, 2048, 2048),
                                    (1000, 50304 // 8, 512)])
def test_mm_nt(M, N, K):
    c = _ops()
    a, b = _rand(M, K), _rand(N, K)
    out = c.mm_nt(a, b)
    c.check_status()
    _close(out, a.float() @ b.float().t())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (512, 2816, 2048), (130, 192, 72)])
def test_mm_nn(M, N, K):
    c = _ops()
    a, b = _rand(M, K), _rand(K, N)
    out = c.mm_nn(a, b)
    c.check_status()
    _close(out, a.float() @ b.float())


@pytest.mark.parametrize("M,N,K", [(256, 256, 128), (2048, 2816, 1024), (192, 320, 200)])
def test_mm_tn(M, N, K):
    c = _ops()
    a, b = _rand(K, M), _rand(K, N)
    out = c.mm_tn(a, b)
    c.check_status()
    _close(out, a.float().t() @ b.float())


def test_axpby_fp32_out():
    c = _ops()
    a, b = _rand(256, 128), _rand(384, 128)
    d = torch.randn(256, 384, device="cuda")
    out = c.mm_nt(a, b, out_dtype=torch.float32, D=d, alpha=-0.5, beta=1.5)
    c.check_status()
    _close(out, -0.5 * (a.float() @ b.float().t()) + 1.5 * d, tol=1e-2)


def test_batched_and_ragged_k():
    c = _ops()
    g, m, n, k = 3, 128, 192, 256
    A, B = _rand(g, m, k), _rand(g, n, k)
    C = torch.empty(g, m, n, dtype=torch.bfloat16, device="cuda")
    c.gemm(A, B, C, mode=c.BATCHED, groups=g, M=m, N=n, Kd=k, lda=k, ldb=k, ldc=n,
           a_gs=m * k, b_gs=n * k, c_gs=m * n)
    c.check_status()
    _close(C, torch.bmm(A.float(), B.float().transpose(1, 2)))
    # ragged reduction ranges over a shared [rows, *] buffer; one empty group
    rows = 640
    X, Y = _rand(rows, 128), _rand(rows, 192)
    kb = torch.tensor([0, 128, 128, 384], dtype=torch.int32, device="cuda")
    kl = torch.tensor([128, 0, 256, 256], dtype=torch.int32, device="cuda")
    out = torch.full((4, 128, 192), 7.0, dtype=torch.bfloat16, device="cuda")
    c.gemm(X, Y, out, mode=c.BATCHED, groups=4, a_major=c.MAJ_MN, b_major=c.MAJ_MN, M=128, N=192, Kd=rows,
           lda=128, ldb=192, ldc=192, c_gs=128 * 192, k_begin=kb, k_len=kl)
    c.check_status()
    for i, (s, l) in enumerate([(0, 128), (128, 0), (128, 256), (384, 256)]):
        ref = X[s:s + l].float().t() @ Y[s:s + l].float()
        _close(out[i], ref) if l else None
        if l == 0:
            assert out[i].abs().max().item() == 0.0


def test_grouped_m_swiglu():
    c = _ops()
    E, d, f = 4, 256, 384
    tiles = torch.tensor([0, 0, 2, 3, 3, 0, 0, 0], dtype=torch.int32, device="cuda")
    live = torch.tensor([5], dtype=torch.int32, device="cuda")
    rows = 8 * 128
    X = _rand(rows, d, scale=0.5)
    w1, w2 = _rand(E, d, f, scale=0.1), _rand(E, d, f, scale=0.1)
    H = torch.zeros(rows, f, dtype=torch.bfloat16, device="cuda")
    G, U = torch.zeros_like(H), torch.zeros_like(H)
    c.gemm(X, w1, H, B2=w2, G=G, U=U, mode=c.GROUPED_M, epi=c.EPI_SWIGLU, M=rows, N=f, Kd=d, groups=E,
           b_major=c.MAJ_MN, lda=d, ldb=f, ldc=f, b_gs=d * f, tile_group=tiles, num_m_tiles=live)
    c.check_status()
    for t in range(5):
        e = int(tiles[t])
        xs = X[t * 128:(t + 1) * 128].float()
        g, u = xs @ w1[e].float(), xs @ w2[e].float()
        _close(G[t * 128:(t + 1) * 128], g)
        _close(U[t * 128:(t + 1) * 128], u)
        _close(H[t * 128:(t + 1) * 128], torch.nn.functional.silu(g) * u, tol=3e-2)
    assert H[5 * 128:].abs().max().item() == 0.0   # tiles past the live count are untouched


@pytest.mark.parametrize("b,m,n", [(3, 512, 320), (1, 2048, 1024), (2, 192, 192)])
def test_symmetric_gram_skips_and_mirrors(b, m, n):
    """A A^T with ``sym_upper``: tiles below the diagonal are mirrored, the result equals the full product."""
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    torch.manual_seed(2)
    a = (torch.randn(b, m, n, device="cuda") * 0.1).to(torch.bfloat16)
    full = torch.empty(b, m, m, dtype=torch.bfloat16, device="cuda")
    sym = torch.full((b, m, m), 7.0, dtype=torch.bfloat16, device="cuda")
    kw = dict(mode=c.BATCHED, groups=b, M=m, N=m, Kd=n, lda=n, ldb=n, ldc=m, a_gs=m * n, b_gs=m * n, c_gs=m * m)
    c.gemm(a, a, full, **kw)
    c.gemm(a, a, sym, sym_upper=True, **kw)
    c.check_status()
    ref = a.float() @ a.float().transpose(1, 2)
    assert (full.float() - ref).abs().max().item() < 2e-2 * ref.abs().max().item()
    assert torch.equal(torch.triu(sym), torch.triu(full))
    assert torch.equal(sym, sym.transpose(1, 2))


@pytest.mark.parametrize("b,m,n", [(2, 512, 320), (1, 2048, 512), (3, 128, 192)])
def test_symmetric_gram_with_scaled_identity(b, m, n):
    """``alpha * A A^T + diag_add * I`` (the ``1.5 I - 0.5 X X^T`` factor of a Newton-Schulz step) with and
    without the symmetric shortcut, against fp32."""
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    torch.manual_seed(3)
    a = (torch.randn(b, m, n, device="cuda") * 0.05).to(torch.bfloat16)
    ref = -0.5 * (a.float() @ a.float().transpose(1, 2)) + 1.5 * torch.eye(m, device="cuda")
    kw = dict(mode=c.BATCHED, groups=b, M=m, N=m, Kd=n, lda=n, ldb=n, ldc=m, a_gs=m * n, b_gs=m * n, c_gs=m * m,
              alpha=-0.5, diag_add=1.5)
    for sym in (False, True):
        out = torch.full((b, m, m), 7.0, dtype=torch.bfloat16, device="cuda")
        c.gemm(a, a, out, sym_upper=sym, **kw)
        c.check_status()
        _close(out, ref, tol=1e-2)
        if sym:
            assert torch.equal(out, out.transpose(1, 2))
