"""The allocation-free RMSNorm-backward entry point, called through its exported C symbol.

Some hosts cannot allocate device memory once they are running (a serving loop that bans
cudaMalloc because it synchronises the device, a process whose memory was all handed out
at start-up, a runtime that owns every buffer and lends this library only raw pointers).
For them the library exports ``kmoe_rmsnorm_bwd_noalloc``, which keeps its scratch in a
fixed array inside the library instead of taking a scratch pointer.  This test calls that
symbol with ctypes on caller-owned buffers, twice in a row with different sizes (the calls
share the scratch array, so the second must not be disturbed by what the first left
there), and compares each result with the regular operator.  It also checks that a size
beyond the stated maximum is refused.  The file name sorts last so a run that stops at the
first failure has already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from kolmogorov_moe_architecture_b200.ops import loader
    loader.require_ext()
    lib = ctypes.CDLL(loader.EXT_PATH)
    fn = lib.kmoe_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def _case(fn, rows, d, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
    w = (1.0 + 0.1 * torch.randn(d, device="cuda", generator=g)).to(torch.bfloat16)
    dy = torch.randn(rows, d, device="cuda", generator=g).to(torch.bfloat16)
    _, rstd = torch.ops.kmoe.rmsnorm_fwd(x, w, 1e-5)
    dx_ref, dw_ref = torch.ops.kmoe.rmsnorm_bwd(x, w, dy, rstd)
    dx = torch.empty_like(x)
    dw = torch.empty(d, dtype=torch.float32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), rows, d, stream)
    assert rc == 0, f"kmoe_rmsnorm_bwd_noalloc returned {rc}"
    torch.cuda.synchronize()
    rel = lambda a, b: ((a.float() - b.float()).abs().max() / (b.float().abs().max() + 1e-6)).item()
    assert rel(dx, dx_ref) < 2e-2
    assert rel(dw, dw_ref) < 2e-2
    # and against the definition itself, evaluated in fp32 by autograd
    xr, wr = x.float().requires_grad_(True), w.float().requires_grad_(True)
    (xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr).backward(dy.float())
    assert rel(dx, xr.grad) < 2e-2
    assert rel(dw, wr.grad) < 2e-2


def test_noalloc_matches_regular_entry_point_on_two_calls():
    fn = _lib()
    _case(fn, 4096, 2048, seed=1)      # fills 64 partial rows of width 2048
    _case(fn, 300, 512, seed=2)        # smaller call right after: reuses the same scratch
    _case(fn, 4096, 2048, seed=3)


def test_noalloc_at_the_size_limit_and_with_a_ragged_column_tail():
    fn = _lib()
    _case(fn, 520, 8192, seed=4)       # d at the stated maximum: every float of the 2 MiB scratch array is used
    _case(fn, 64, 520, seed=5)         # d not a multiple of 256: the last column block is partly empty


def test_noalloc_rejects_sizes_beyond_the_maximum():
    fn = _lib()
    x = torch.zeros(8, device="cuda")
    for rows, d in [(16, 8192 + 8), (16, 100), (0, 512)]:
        rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), rows, d, None)
        assert rc == -1
