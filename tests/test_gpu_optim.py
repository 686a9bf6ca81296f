"""Fused AdamW (clip coefficient on device, fp32 moments) against torch.optim.AdamW, and the
sharded-data-parallel step on one GPU against the plain optimizer path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _tiny(dtype=torch.bfloat16):
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    cfg = AdvancedMoEConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                            d_ff_expert=128, n_experts=4, moe_layers=(1,), mamba_layers=(1,), max_seq_len=64,
                            n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), mamba_moe_mode="moe_ffn", dropout=0.0,
                            attention_dropout=0.0, residual_dropout=0.0)
    torch.manual_seed(0)
    return cfg, MoETransformer(cfg, verbose=False).cuda().to(dtype)


def test_fused_adamw_kernel_matches_torch():
    from kolmogorov_moe_architecture_b200.ops import cuda_ops  # noqa: F401  (loads the extension)
    n = 4096 + 128
    torch.manual_seed(1)
    p0 = (0.1 * torch.randn(n, device="cuda")).to(torch.bfloat16)
    ref_p = p0.float().clone().requires_grad_(True)
    opt = torch.optim.AdamW([ref_p], lr=1e-2, betas=(0.9, 0.95), weight_decay=0.1, eps=1e-8)
    flat_p, flat_g = p0.clone(), torch.zeros_like(p0)
    m = torch.zeros(n, device="cuda")
    v = torch.zeros(n, device="cuda")
    coef = torch.tensor([0.5], device="cuda")
    for step in range(1, 4):
        g = torch.randn(n, device="cuda").to(torch.bfloat16)
        flat_g.copy_(g)
        torch.ops.kmoe.p2p_adamw_allgather([flat_p.data_ptr()], flat_g, m, v, 0, 1, 0, n, 1e-2, 0.9, 0.95, 1e-8, 0.1,
                                           step, coef, 0)
        ref_p.grad = g.float() * 0.5
        opt.step()
    err = (flat_p.float() - ref_p.detach()).abs().max().item()
    assert err < 5e-3, err          # bf16 parameter rounding (ulp 1e-3 at 0.25) over three steps


def test_sharded_pool_single_gpu_trains():
    from kolmogorov_moe_architecture_b200.ops import cuda_ops
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg, model = _tiny()
    dp = ShardedDataParallel(model, optimizer_kind="muon", lr=2e-3, adamw_lr=2e-3)
    assert dp.fused is not None and dp.muon is not None
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, dp=dp)
    ids = torch.randint(0, cfg.vocab_size, (2, 64), device="cuda")
    losses = [eng.step(ids).loss_value() for _ in range(6)]
    cuda_ops.check_status()
    assert losses[-1] < losses[0], losses
    assert all(torch.isfinite(p).all() for p in model.parameters())


def test_muon_fused_kernels_match_unfused(monkeypatch):
    """Momentum / normalisation-in-GEMM / parameter-update kernels against the sequence of torch ops
    they replace (same optimizer class, fused path switched off), over 2-D and stacked 3-D parameters."""
    from kolmogorov_moe_architecture_b200.ops import cuda_ops  # noqa: F401  (loads the extension)
    from kolmogorov_moe_architecture_b200.training.muon_optimizer import Muon

    def run(fused: bool):
        monkeypatch.setenv("KMOE_MUON_FUSED", "1" if fused else "0")
        torch.manual_seed(0)
        ps = [torch.nn.Parameter((torch.randn(256, 512, device="cuda") * 0.05).bfloat16()),
              torch.nn.Parameter((torch.randn(512, 128, device="cuda") * 0.05).bfloat16()),
              torch.nn.Parameter((torch.randn(3, 256, 512, device="cuda") * 0.05).bfloat16()),
              torch.nn.Parameter((torch.randn(256, 512, device="cuda") * 0.05).bfloat16())]
        opt = Muon(ps, lr=2e-2, momentum=0.9, weight_decay=0.1)
        g = torch.Generator(device="cuda").manual_seed(1)
        for _ in range(3):
            for p in ps:
                p.grad = (torch.randn(p.shape, device="cuda", generator=g) * 0.1).bfloat16()
            opt.step()
        bufs = [opt.state[p]["momentum_buffer"].float().clone() for p in ps]
        return [p.detach().float().clone() for p in ps], bufs

    pf, bf_ = run(True)
    pu, bu = run(False)
    for a, b in zip(pf, pu):
        assert (a - b).abs().max().item() < 4e-3 * max(b.abs().max().item(), 1e-3) + 2e-4
    for a, b in zip(bf_, bu):
        assert (a - b).norm().item() < 3e-2 * b.norm().item()


def test_barrier_wait_runs_out_and_reports_status():
    """Failure detection on the device without faulting it: a flag barrier whose peer never arrives gives up
    after its wall-clock limit, records a status code that the host turns into an exception, and leaves the
    context usable."""
    import time
    from kolmogorov_moe_architecture_b200.ops import cuda_ops
    cuda_ops.check_status()
    mine = torch.zeros(64, dtype=torch.int32, device="cuda")      # this rank's flag words
    absent = torch.zeros(64, dtype=torch.int32, device="cuda")    # stands in for a peer that never writes
    status = cuda_ops.status_tensor(torch.device("cuda"))
    t0 = time.time()
    torch.ops.kmoe.p2p_barrier([mine.data_ptr(), absent.data_ptr()], 0, 2, 1, 0.05, status)
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0
    assert int(absent[0]) == 1                                    # the arrival was published to the "peer"
    with pytest.raises(RuntimeError, match="wait-timeout status 101"):
        cuda_ops.check_status()
    cuda_ops.check_status()                                       # cleared by the report
    x = torch.ones(1024, device="cuda")
    assert float((x * 2).sum()) == 2048.0                         # the context still works


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,block", [(5000, 2048), (4096, 2048), (100, 64)])
def test_int8_momentum_kernels_equal_the_formulas(dtype, n, block):
    """Block-wise absmax int8 quantisation of the Muon8bit momentum and the fused dequantise-decay-add pass
    against the same formulas in plain PyTorch: identical int8 codes, scales and updated buffer."""
    torch.manual_seed(0)
    x = (torch.randn(n, device="cuda") * 3).to(dtype)
    q, sc = torch.ops.kmoe.q8_quant(x, block)
    flat = torch.nn.functional.pad(x.flatten(), (0, (-n) % block)).view(-1, block)
    sc_ref = flat.abs().amax(dim=1, keepdim=True).clamp(min=1e-8).float()
    q_ref = (flat.float() / sc_ref * 127).round().to(torch.int8)
    assert torch.equal(sc, sc_ref) and torch.equal(q, q_ref)
    g = torch.randn(n, device="cuda").to(dtype)
    out = torch.ops.kmoe.q8_momentum(q, sc, g, 0.95)
    ref = ((q_ref.float() / 127) * sc_ref).flatten()[:n].to(dtype)
    ref.mul_(0.95).add_(g)
    assert torch.equal(out, ref)


def test_muon8bit_step_on_kernels_matches_eager_path(monkeypatch):
    from kolmogorov_moe_architecture_b200.training import muon_optimizer as mo
    torch.manual_seed(1)
    shapes = [(128, 192), (64,), (3, 64, 128)]
    res = {}
    for kernels in (True, False):
        ps = [torch.nn.Parameter((torch.randn(*s, device="cuda", generator=None) * 0.1).bfloat16()) for s in shapes]
        torch.manual_seed(1)
        for p in ps:
            p.data.copy_((torch.randn_like(p, dtype=torch.float32) * 0.1).bfloat16())
        if not kernels:
            monkeypatch.setattr(mo.Muon8bit, "_on_kernels", staticmethod(lambda t: False))
        opt = mo.Muon8bit(ps, lr=1e-2, block_size=256)
        for step in range(3):
            torch.manual_seed(10 + step)
            for p in ps:
                p.grad = torch.randn_like(p, dtype=torch.float32).bfloat16()
            opt.step()
        res[kernels] = [p.detach().float().clone() for p in ps]
    for a, b in zip(res[True], res[False]):
        assert torch.allclose(a, b, atol=1e-3, rtol=0), (a - b).abs().max()


@pytest.mark.gpu
@pytest.mark.parametrize("n", [7, 8, 4099, 3 * 2**20 + 5])
def test_sum_of_squares_kernel(n):
    """fp32 sum of squares of a bf16 buffer (the gradient norm of the flat buffer) against PyTorch in fp64; the
    same call twice gives identical bits (fixed summation order)."""
    import kolmogorov_moe_architecture_b200.ops.cuda_ops  # noqa: F401  (loads the extension)
    torch.manual_seed(n)
    x = (torch.randn(n, device="cuda") * 3).to(torch.bfloat16)
    a, b = torch.ops.kmoe.sumsq(x), torch.ops.kmoe.sumsq(x)
    ref = x.double().pow(2).sum()
    assert torch.equal(a, b)
    assert abs(a.item() - ref.item()) <= 1e-5 * ref.item()
