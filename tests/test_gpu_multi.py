"""Multi-GPU checks (run only where at least 2 GPUs are visible): the peer-to-peer transport
of the sharded data-parallel step against the NCCL transport, as child processes."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KMOE_ROOT"])
from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
from kolmogorov_moe_architecture_b200.ops import cuda_ops
from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
rank = int(os.environ["RANK"]); torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
cfg = AdvancedMoEConfig(vocab_size=512, d_model=128, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                        d_ff_expert=128, n_experts=4, moe_layers=(1,), mamba_layers=(1,), max_seq_len=64,
                        n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), mamba_moe_mode="moe_ffn", dropout=0.0,
                        attention_dropout=0.0, residual_dropout=0.0)
out = {}
for transport in ("nccl", "p2p"):
    torch.manual_seed(0)
    model = MoETransformer(cfg, verbose=False).cuda().to(torch.bfloat16)
    dp = ShardedDataParallel(model, optimizer_kind="muon", lr=2e-3, adamw_lr=2e-3, transport=transport)
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, dp=dp)
    g = torch.Generator().manual_seed(5 + rank)
    for s in range(3):
        eng.step(torch.randint(0, 512, (2, 64), generator=g).cuda())
    cuda_ops.check_status()
    out[transport] = torch.cat([p.detach().float().flatten() for p in model.parameters()])
err = (out["nccl"] - out["p2p"]).abs().max().item()
ref = out["nccl"].abs().max().item()
# replicas must agree bit for bit after the all-gather
mine = out["p2p"].clone(); other = mine.clone(); dist.broadcast(other, 0)
assert torch.equal(mine, other), "ranks diverged"
assert err < 2e-2 * ref, (err, ref)
want_mc = os.environ.get("KMOE_EXPECT_MULTIMEM") == "1"
if want_mc:
    assert dp.p2p.grad_mc != 0 and dp.p2p.param_mc != 0, "no multicast address on this fabric"
else:
    assert dp.p2p.grad_mc == 0
if rank == 0: print("MULTI_OK", err, "multimem" if want_mc else "peer")
dist.destroy_process_group()
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
@pytest.mark.parametrize("multimem,overlap", [(False, False), (True, False), (False, True)])
def test_p2p_transport_matches_nccl_2gpus(tmp_path, multimem, overlap):
    """Plain peer loads/stores, the NVLink-switch path (multimem.ld_reduce / multimem.st), and the
    reduce-scatter issued in groups on a side stream while the backward pass is still running."""
    f = tmp_path / "worker.py"
    f.write_text(WORKER)
    env = dict(os.environ, KMOE_ROOT=ROOT, KMOE_STRICT="1", KMOE_RS_OVERLAP="1" if overlap else "0",
               KMOE_RS_CHUNKS="3")
    if multimem:
        env.pop("NCCL_NVLS_ENABLE", None)
        env.update(KMOE_MULTIMEM="1", KMOE_EXPECT_MULTIMEM="1")
    else:
        env.update(NCCL_NVLS_ENABLE="0")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29581", str(f)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "MULTI_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


EP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KMOE_ROOT"])
from kolmogorov_moe_architecture_b200.ops import cuda_ops, eager
from kolmogorov_moe_architecture_b200.parallel import ep, ep_p2p
from kolmogorov_moe_architecture_b200 import ops
rank = int(os.environ["RANK"]); ws = int(os.environ["WORLD_SIZE"]); torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
E, d, f, k, T = 8, 256, 384, 2, 1000
nl = E // ws
g = torch.Generator().manual_seed(1)
W1 = (torch.randn(E, d, f, generator=g) * 0.05); W2 = (torch.randn(E, d, f, generator=g) * 0.05)
W3 = (torch.randn(E, f, d, generator=g) * 0.05)
g2 = torch.Generator().manual_seed(10 + rank)
x0 = torch.randn(T, d, generator=g2); logits = torch.randn(T, E, generator=g2)
logits[:, 3] += 1.5                                   # skewed load
wts0, idx = torch.softmax(logits, -1).topk(k, dim=-1)
dout = torch.randn(T, d, generator=g2).cuda().bfloat16()
idx = idx.cuda()
cap = T * k // E                                      # capacity factor 1.0: the skewed expert really drops
keep = ops.capacity_keep_mask(idx, E, cap)
assert int((~keep).sum()) > 0
res = {}
for mode in ("fused", "a2a", "fused_mx", "a2a_mx", "oracle"):
    dt = "mxfp8" if mode.endswith("_mx") else "bf16"
    x = x0.cuda().bfloat16().requires_grad_(True)
    wts = wts0.cuda().bfloat16().requires_grad_(True)
    sl = slice(rank * nl, (rank + 1) * nl)
    if mode == "oracle":
        ws_ = [w.cuda().float().requires_grad_(True) for w in (W1, W2, W3)]
        out = eager.grouped_swiglu(x.float(), ws_[0], ws_[1], ws_[2], idx, wts.float(), keep)
        out.backward(dout.float())
        grads = [w.grad[sl] for w in ws_]
        # expert weight gradients sum over the ranks' tokens
        full = [w.grad.clone() for w in ws_]
        for t in full: dist.all_reduce(t)
        grads = [t[sl] for t in full]
    else:
        ws_ = [w[sl].cuda().bfloat16().contiguous().requires_grad_(True) for w in (W1, W2, W3)]
        if mode.startswith("fused"):
            for rep in range(2):                      # twice: buffers and epochs are reused across layers
                for t in [x, wts] + ws_: t.grad = None
                out = ep_p2p.expert_parallel_ffn_fused(x, idx, wts, ws_[0], ws_[1], ws_[2], E, None, keep,
                                                       slot_cap=cap if rep == 1 else None,   # capacity-sized slots
                                                       moe_dtype=dt)
                out.backward(dout)
        else:
            fn = lambda xx, ii, ww, kk: ops.grouped_swiglu(xx, ws_[0], ws_[1], ws_[2], ii, ww, kk, dt)
            out = ep.expert_parallel_ffn(x, idx, wts, fn, E, None, keep=keep)
            out.backward(dout)
        grads = [w.grad for w in ws_]
    cuda_ops.check_status()
    res[mode] = [out.detach().float(), x.grad.float(), wts.grad.float()] + [t.float() for t in grads]
names = ["out", "dx", "dw", "dW1", "dW2", "dW3"]
for mode in ("fused", "a2a"):
    for n, a, b in zip(names, res[mode], res["oracle"]):
        err = (a - b).abs().max().item(); ref = b.abs().max().item()
        assert err <= 3e-2 * ref + 1e-3, (mode, n, err, ref)
# block-scaled fp8 experts: both transports quantise the same rows at the same points (the layer output
# agrees closely; weight gradients quantise along the row order, which differs), and stay near the fp32 oracle
for n, a, b, c in zip(names, res["fused_mx"], res["a2a_mx"], res["oracle"]):
    ref = c.abs().max().item()
    e_t = (a - b).abs().max().item(); e_o = (a - c).abs().max().item()
    assert e_t <= (1e-2 if n == "out" else 6e-2) * ref + 1e-3, ("mx transports", n, e_t, ref)
    assert e_o <= 0.15 * ref + 1e-3, ("mx oracle", n, e_o, ref)
if rank == 0: print("EP_OK")
dist.barrier()
ep_p2p.release_buffers()
dist.destroy_process_group()
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_expert_parallel_fused_exchange_2gpus(tmp_path):
    """Peer-pointer dispatch/return kernels and the all_to_all transport against the fp32 oracle
    evaluated with every expert on one rank (outputs, input/routing-weight/expert-weight gradients)."""
    f = tmp_path / "ep_worker.py"
    f.write_text(EP_WORKER)
    env = dict(os.environ, KMOE_ROOT=ROOT, NCCL_NVLS_ENABLE="0", KMOE_STRICT="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29583", str(f)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "EP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


FSDP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KMOE_ROOT"])
from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
from kolmogorov_moe_architecture_b200.ops import cuda_ops
from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
rank = int(os.environ["RANK"]); torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
cfg = AdvancedMoEConfig(vocab_size=512, d_model=128, n_layers=4, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                        d_ff_expert=128, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=64,
                        n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), mamba_moe_mode="moe_ffn", dropout=0.0,
                        attention_dropout=0.0, residual_dropout=0.0)
out, losses = {}, {}
variants = {"replicated": None, "nccl": dict(transport="nccl", overlap=False),
            "nccl-overlap": dict(transport="nccl", overlap=True), "p2p-overlap": dict(transport="p2p", overlap=True)}
for kind, kw in variants.items():
    torch.manual_seed(0)
    model = MoETransformer(cfg, verbose=False).cuda().to(torch.bfloat16)
    n_full = sum(p.numel() for p in model.parameters())
    if kw is None:
        dp = ShardedDataParallel(model, optimizer_kind="adamw", adamw_lr=2e-3, transport="nccl")
    else:
        dp = FullyShardedDataParallel(model, lr=2e-3, **kw)
        assert dp.transport == kw["transport"] and dp.overlap == kw["overlap"]
        assert all(p.numel() == 0 for p in model.parameters())
        assert dp.param_bytes_per_rank() <= 0.55 * n_full * 2
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, dp=dp)
    g = torch.Generator().manual_seed(5 + rank)
    ls = []
    for s in range(3):
        ls.append(eng.step(torch.randint(0, 512, (2, 64), generator=g).cuda()).loss_value())
    cuda_ops.check_status()
    losses[kind] = ls
    if kw is None:
        out[kind] = {n: p.detach().float().clone() for n, p in model.named_parameters()}
    else:
        out[kind] = {n: t.float().cuda() for n, t in dp.full_state_dict().items()}
        assert dp.early_gathers == (3 * (2 * (len(dp.units) - 1) + 1) if kw["overlap"] else 0)
ref = max(t.abs().max().item() for t in out["replicated"].values())
err = 0.0
for kind in variants:
    if kind == "replicated":
        continue
    e = max((out["replicated"][n] - out[kind][n]).abs().max().item() for n in out["replicated"])
    assert max(abs(a - b) for a, b in zip(losses["replicated"], losses[kind])) < 5e-2, (kind, losses)
    assert e < 3e-2 * ref, (kind, e, ref)
    err = max(err, e)
# the variants of the sharded plan do the same arithmetic: a race on a buffer would show up here
for kind in ("nccl-overlap", "p2p-overlap"):
    d = max((out["nccl"][n] - out[kind][n]).abs().max().item() for n in out["nccl"])
    assert d < 5e-3 * ref, (kind, d, ref)
if rank == 0: print("FSDP_OK", err, losses)
dist.destroy_process_group()
'''


@pytest.mark.skipif(not torch.cuda.is_available() or torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_param_sharded_plan_matches_replicated_2gpus(tmp_path):
    """ZeRO-3 style plan (parameters gathered per block into two rotating buffers) against the replicated plan:
    library collectives, the same with gathers and reduce-scatters on side streams, and the peer-memory transport."""
    f = tmp_path / "fsdp_worker.py"
    f.write_text(FSDP_WORKER)
    env = dict(os.environ, KMOE_ROOT=ROOT, NCCL_NVLS_ENABLE="0", KMOE_STRICT="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", "29585", str(f)],
                       env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "FSDP_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]


DEFAULT_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KMOE_ROOT"])
from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
from kolmogorov_moe_architecture_b200.ops import cuda_ops
from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
rank = int(os.environ["RANK"]); ws = int(os.environ["WORLD_SIZE"]); torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
cfg = AdvancedMoEConfig(vocab_size=512, d_model=128, n_layers=4, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                        d_ff_expert=128, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=64,
                        n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), mamba_moe_mode="moe_ffn", dropout=0.0,
                        attention_dropout=0.0, residual_dropout=0.0)
out, used = {}, {}
for transport in ("nccl", None):                      # None = what the benchmark runs: the library's own default
    torch.manual_seed(0)
    model = MoETransformer(cfg, verbose=False).cuda().to(torch.bfloat16)
    dp = ShardedDataParallel(model, optimizer_kind="muon", lr=2e-3, adamw_lr=2e-3, transport=transport)
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, dp=dp)
    g = torch.Generator().manual_seed(5 + rank)
    for s in range(3):
        eng.step(torch.randint(0, 512, (2, 64), generator=g).cuda())
    cuda_ops.check_status()
    out[transport] = torch.cat([p.detach().float().flatten() for p in model.parameters()])
    used[transport] = (dp.transport, bool(getattr(dp, "_chunks", None)),
                       int(dp.p2p.grad_mc != 0) if dp.transport == "p2p" else 0)
err = (out["nccl"] - out[None]).abs().max().item()
ref = out["nccl"].abs().max().item()
mine = out[None].clone(); other = mine.clone(); dist.broadcast(other, 0)
assert torch.equal(mine, other), "ranks diverged"
assert err < 2e-2 * ref, (err, ref)
if rank == 0: print("DEFAULT_OK", ws, err, used[None])
dist.destroy_process_group()
'''


@pytest.mark.parametrize("n", [4, 8])
def test_default_transport_matches_nccl_at_bench_rank_counts(tmp_path, n):
    """The configuration the benchmark runs at 4 and 8 GPUs - no environment switches, so from 4 ranks the
    switch's in-fabric reduction and the reduce-scatter overlapped with the backward pass - against the NCCL
    transport: parameters after three steps agree, replicas are bit-identical."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    f = tmp_path / "default_worker.py"
    f.write_text(DEFAULT_WORKER)
    env = dict(os.environ, KMOE_ROOT=ROOT, KMOE_STRICT="1")
    for k in ("KMOE_RS_OVERLAP", "KMOE_RS_CHUNKS", "KMOE_MULTIMEM", "NCCL_NVLS_ENABLE"):
        env.pop(k, None)
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
                        "--master-addr", "127.0.0.1", "--master-port", "29587", str(f)],
                       env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0 and "DEFAULT_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
    line = [l for l in r.stdout.splitlines() if l.startswith("DEFAULT_OK")][0]
    assert "'p2p', True, 1" in line, f"expected the peer transport with overlap and the multicast address: {line}"


CURVE_WORKER = r'''
import json, os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["KMOE_ROOT"])
from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
from kolmogorov_moe_architecture_b200.ops import cuda_ops
from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
rank = int(os.environ["RANK"]); ws = int(os.environ["WORLD_SIZE"]); torch.cuda.set_device(rank)
n = int(os.environ["KMOE_GLOBAL_RANKS"])              # the global batch is n micro-batches of 2 sequences
if ws > 1:
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
cfg = AdvancedMoEConfig(vocab_size=512, d_model=128, n_layers=4, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                        d_ff_expert=128, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=64,
                        n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), mamba_moe_mode="moe_ffn", dropout=0.0,
                        attention_dropout=0.0, residual_dropout=0.0)
torch.manual_seed(0)
model = MoETransformer(cfg, verbose=False).cuda().to(torch.bfloat16)
dp = ShardedDataParallel(model, optimizer_kind="muon", lr=2e-3, adamw_lr=2e-3)
eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, grad_accum=(n if ws == 1 else 1), dp=dp)
g = torch.Generator().manual_seed(11)
losses = []
for s in range(5):
    batch = torch.randint(0, 512, (2 * n, 64), generator=g)      # the same global batch in both runs
    mine = batch if ws == 1 else batch[2 * rank: 2 * rank + 2]
    l = eng.step(mine.cuda()).loss.detach().float().reshape(1)
    if ws > 1:
        dist.all_reduce(l); l /= ws
    losses.append(float(l.item()))
cuda_ops.check_status()
if rank == 0: print("CURVE", json.dumps(losses))
if ws > 1: dist.destroy_process_group()
'''


@pytest.mark.parametrize("n", [2, 4, 8])
def test_loss_curve_one_gpu_equals_n_gpus(tmp_path, n):
    """The same global batch, once as n accumulated micro-batches on one GPU and once as one micro-batch on
    each of n GPUs: the loss curves agree step by step."""
    import json
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} GPUs")
    f = tmp_path / "curve_worker.py"
    f.write_text(CURVE_WORKER)
    env = dict(os.environ, KMOE_ROOT=ROOT, KMOE_STRICT="1", KMOE_GLOBAL_RANKS=str(n))
    curves = {}
    for ranks in (1, n):
        r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={ranks}",
                            "--master-addr", "127.0.0.1", "--master-port", str(29589 + ranks), str(f)],
                           env=env, capture_output=True, text=True, timeout=900)
        assert r.returncode == 0 and "CURVE" in r.stdout, r.stdout[-2000:] + r.stderr[-3000:]
        curves[ranks] = json.loads([l for l in r.stdout.splitlines() if l.startswith("CURVE")][0][6:])
    for a, b in zip(curves[1], curves[n]):
        assert abs(a - b) < 2e-2 * abs(a), (curves[1], curves[n])
