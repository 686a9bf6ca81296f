"""Expert-parallel dispatch/combine on CPU ranks (gloo): forward and every gradient against
a single-process oracle that holds all experts."""
import torch

from dist_utils import run_ranks


def _cfg(impl):
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    return AdvancedMoEConfig(vocab_size=64, d_model=32, n_layers=1, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                             d_ff_expert=48, n_experts=4, moe_top_k=2, moe_layers=(0,), mamba_layers=(),
                             moe_implementation=impl, dtype="float32", device="cpu", max_seq_len=16,
                             n_pred_tokens=1, aux_loss_weights=(1.0,))


def _oracle(world, drop):
    from kolmogorov_moe_architecture_b200.models.sparse_moe import ExpertParallelMoE
    torch.manual_seed(3)
    cfg = _cfg("expert_parallel")
    cfg.moe_drop_tokens = drop
    cfg.moe_capacity_factor = 0.6 if drop else 1.25
    layer = ExpertParallelMoE(cfg, 0)            # no process group: all experts local
    layer.train()
    xs = torch.randn(world, 2, 8, 32)
    gs = torch.randn(world, 2, 8, 32)
    outs, gx = [], []
    for r in range(world):
        x = xs[r].clone().requires_grad_(True)
        o = layer(x)
        (o * gs[r]).sum().backward()
        outs.append(o.detach())
        gx.append(x.grad)
    grads = {n: p.grad.clone() for n, p in layer.named_parameters()}
    return layer.state_dict(), xs, gs, outs, gx, grads


def _worker(rank, world, drop, state, xs, gs, outs, gx, grads):
    from kolmogorov_moe_architecture_b200.models.sparse_moe import ExpertParallelMoE
    cfg = _cfg("expert_parallel")
    cfg.moe_drop_tokens = drop
    cfg.moe_capacity_factor = 0.6 if drop else 1.25
    layer = ExpertParallelMoE(cfg, 0)
    n_local = layer.n_local_experts
    sl = slice(rank * n_local, (rank + 1) * n_local)
    with torch.no_grad():
        layer.router.weight.copy_(state["router.weight"])
        for k in ("w1", "w2", "w3"):
            getattr(layer.local_experts, k).copy_(state[f"local_experts.{k}"][sl])
    layer.train()
    x = xs[rank].clone().requires_grad_(True)
    o = layer(x)
    (o * gs[rank]).sum().backward()
    assert torch.allclose(o, outs[rank], atol=1e-5), (o - outs[rank]).abs().max()
    assert torch.allclose(x.grad, gx[rank], atol=1e-5)
    for k in ("w1", "w2", "w3"):
        got = getattr(layer.local_experts, k).grad
        assert torch.allclose(got, grads[f"local_experts.{k}"][sl], atol=1e-5), k
    # router gradient: each rank holds the part from its own tokens; the sum is the oracle's
    import torch.distributed as dist
    rg = layer.router.weight.grad.clone()
    dist.all_reduce(rg)
    assert torch.allclose(rg, grads["router.weight"], atol=1e-5)


def test_expert_parallel_matches_oracle_2ranks():
    run_ranks(_worker, 2, False, *_oracle(2, False))


def test_expert_parallel_with_token_drop_4ranks():
    run_ranks(_worker, 4, True, *_oracle(4, True))
