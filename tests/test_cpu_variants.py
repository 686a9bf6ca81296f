"""Alternative MoE layer classes, the native-kernel call interface, and the small utilities (metric sink,
phase timer, roofline reporter, tokenizer wrapper) on CPU."""
import json
import os

import pytest
import torch
import torch.nn.functional as F

import kolmogorov_moe_architecture_b200 as kmoe
from kolmogorov_moe_architecture_b200.ops import eager


def _route(T, E, k, seed=0):
    g = torch.Generator().manual_seed(seed)
    w, idx = torch.softmax(torch.randn(T, E, generator=g), -1).topk(k, dim=-1)
    return idx, w / w.sum(-1, keepdim=True)


def test_alternative_expert_classes_compute_the_same_function():
    """OptimizedGroupedExperts and the benchmark classes of triton_moe are the one grouped path under
    other names: same weights -> same output as the eager definition."""
    from kolmogorov_moe_architecture_b200.models.fused_moe import FusedSparseMoE, OptimizedGroupedExperts
    from kolmogorov_moe_architecture_b200.models.triton_moe import (BatchedMoE, BatchedMoEOptimized,
                                                                    TritonGroupedExperts, TritonGroupedExpertsFused,
                                                                    sort_tokens_by_expert)
    torch.manual_seed(0)
    T, d, f, E, k = 24, 16, 32, 4, 2
    x = torch.randn(T, d)
    idx, w = _route(T, E, k)
    for cls in (OptimizedGroupedExperts, TritonGroupedExperts, TritonGroupedExpertsFused, BatchedMoE, BatchedMoEOptimized):
        m = cls(E, d, f)
        want = eager.grouped_swiglu(x, m.w1, m.w2, m.w3, idx, w)
        assert torch.allclose(m(x, idx, w), want, atol=1e-5), cls.__name__
    tok, ids, order, starts, ends = sort_tokens_by_expert(idx, E)
    flat = idx.reshape(-1)
    assert torch.equal(ids, flat[order]) and torch.equal(ids, ids.sort().values)      # expert ids ascending
    assert torch.equal(tok, order // k) and int(ends[-1]) == T * k
    assert all(bool((ids[s:e] == i).all()) for i, (s, e) in enumerate(zip(starts.tolist(), ends.tolist())))
    layer = FusedSparseMoE(d, f, E, top_k=k)
    y = layer(torch.randn(2, 6, d))
    assert y.shape == (2, 6, d) and torch.isfinite(y).all()
    y.sum().backward()
    assert all(p.grad is not None for p in layer.parameters())


def test_fp8_layers_follow_the_mx_number_format_on_cpu():
    """FP8Linear / FP8GroupedExperts / FP8MoELayer: on CPU the block-scaled format is emulated, so the result
    is the exact-arithmetic result of the quantised operands and stays near the bf16 layer."""
    from kolmogorov_moe_architecture_b200.models.fp8_moe import (FP8GroupedExperts, FP8Linear, FP8MoELayer,
                                                                 is_fp8_available)
    from kolmogorov_moe_architecture_b200.ops.mxfp8 import fake_quant_mx
    assert is_fp8_available() in (True, False)
    torch.manual_seed(0)
    lin = FP8Linear(64, 32).float()
    x = torch.randn(5, 64)
    want = fake_quant_mx(x) @ fake_quant_mx(lin.weight).t()
    got = lin(x)
    assert torch.allclose(got, want, atol=1e-4, rtol=1e-4)
    assert (got - x @ lin.weight.t()).abs().max() < 0.1 * (x @ lin.weight.t()).abs().max()
    assert {"input_scale", "weight_scale", "input_amax_history"} <= set(lin.state_dict())     # reference's buffer names
    ex = FP8GroupedExperts(4, 64, 64).float()
    idx, w = _route(12, 4, 2)
    xe = torch.randn(12, 64)
    ref = eager.grouped_swiglu(xe, ex.w1, ex.w2, ex.w3, idx, w)
    out = ex(xe, idx, w)
    assert (out - ref).abs().max() < 0.15 * ref.abs().max() + 1e-3
    layer = FP8MoELayer(64, 64, 4, top_k=2).float().train()
    y = layer(torch.randn(2, 8, 64))
    assert y.shape == (2, 8, 64) and float(layer.aux_loss) > 0


def test_native_kernel_interface_on_sorted_rows():
    """``grouped_swiglu_forward`` / ``grouped_swiglu_with_grad`` / ``GroupedSwiGLUFunction`` on expert-sorted
    rows with segment bounds (the calling convention of the reference's extension)."""
    from kolmogorov_moe_architecture_b200 import kernels as K
    torch.manual_seed(0)
    E, d, f = 3, 8, 16
    counts = [5, 0, 7]
    ids = torch.cat([torch.full((c,), e) for e, c in enumerate(counts)])
    ends = torch.tensor(counts).cumsum(0)
    starts = ends - torch.tensor(counts)
    x = torch.randn(sum(counts), d, requires_grad=True)
    W = [torch.randn(E, d, f, requires_grad=True), torch.randn(E, d, f, requires_grad=True),
         torch.randn(E, f, d, requires_grad=True)]
    want = torch.cat([(F.silu(x[s:t] @ W[0][e]) * (x[s:t] @ W[1][e])) @ W[2][e]
                      for e, (s, t) in enumerate(zip(starts.tolist(), ends.tolist()))])
    got = K.grouped_swiglu_forward(x.detach(), W[0].detach(), W[1].detach(), W[2].detach(), ids, starts, ends)
    assert torch.allclose(got, want, atol=1e-5)
    out = K.GroupedSwiGLUFunction.apply(x, *W, ids, starts, ends)
    assert torch.allclose(out, want, atol=1e-5)
    g_ref = torch.autograd.grad(want.sum(), [x] + W, retain_graph=True)
    g_got = torch.autograd.grad(out.sum(), [x] + W)
    assert all(torch.allclose(a, b, atol=1e-4) for a, b in zip(g_got, g_ref))
    assert K.is_kernel_available() in (True, False)
    import moe_arch.kernels as shim                        # the reference's import path resolves to the same module
    assert shim.grouped_swiglu_forward is K.grouped_swiglu_forward


def test_metric_logger_phase_timer_and_roofline(tmp_path):
    from kolmogorov_moe_architecture_b200.utils.logging import MetricLogger
    from kolmogorov_moe_architecture_b200.utils.profiling import PhaseTimer, measured_peaks, nvtx_range, roofline
    path = str(tmp_path / "m" / "metrics.jsonl")
    lg = MetricLogger(path)
    lg.log({"loss": torch.tensor(1.5), "lr": 1e-3, "router/avg_entropy": 0.9}, step=7)
    lg.close()
    MetricLogger(path, rank=1).log({"loss": 0.0}, step=8)          # other ranks write nothing
    rows = [json.loads(l) for l in open(path)]
    assert len(rows) == 1 and rows[0]["step"] == 7 and rows[0]["loss"] == 1.5 and "time" in rows[0]
    t = PhaseTimer(enabled=True, device=torch.device("cpu"))
    for _ in range(3):
        with t.phase("fwd"):
            sum(range(1000))
        with t.phase("bwd"), nvtx_range("bwd"):
            sum(range(1000))
    s = t.summary()
    assert set(s) >= {"fwd", "bwd"} and all(v >= 0 for v in s.values())
    off = PhaseTimer(enabled=False)
    with off.phase("x"):
        pass
    assert off.summary() == {}
    pk = measured_peaks()
    assert pk["kind"] in ("measured", "fallback") and pk["hbm_bytes_s"] > 1e12
    r = roofline(1e-3, flops=pk["bf16_flops"] * 0.5e-3, hbm_bytes=pk["hbm_bytes_s"] * 0.25e-3)
    assert abs(r["achieved_fraction"] - 0.5) < 1e-6                  # compute is the binding limit here
    r = roofline(1e-3, nvlink_bytes=770e9 * 0.8e-3)
    assert abs(r["achieved_fraction"] - 0.8) < 1e-6


def test_tokenizer_wrapper_with_the_offline_byte_tokenizer(monkeypatch):
    """No tokenizer files are reachable here: the wrapper falls back to the byte tokenizer and keeps the
    Hugging Face calling convention (pad = its own id, batches padded to the longest row)."""
    from kolmogorov_moe_architecture_b200.data import ByteTokenizer, TokenizerWrapper
    monkeypatch.setenv("HF_HUB_OFFLINE", "1")
    w = TokenizerWrapper("no-such-tokenizer-anywhere", verbose=False)
    assert isinstance(w.tokenizer, ByteTokenizer) and w.vocab_size == 258 and w.pad_token_id == 257
    one = w.encode("héllo wörld")
    assert one["input_ids"][-1] == w.eos_token_id and w.decode(one["input_ids"]) == "héllo wörld"
    batch = w.encode(["ab", "abcdef"], padding=True, return_tensors="pt")
    assert batch["input_ids"].shape == (2, 7) and batch["attention_mask"][0].tolist() == [1, 1, 1, 0, 0, 0, 0]
    assert w.batch_decode(batch["input_ids"]) == ["ab", "abcdef"]
    with pytest.raises(Exception):
        TokenizerWrapper("no-such-tokenizer-anywhere", allow_byte_fallback=False, verbose=False)


def _tiny_model():
    cfg = kmoe.get_tiny_debug_config(vocab_size=128, d_model=32, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                                     d_ff_expert=32, max_seq_len=16, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5))
    torch.manual_seed(0)
    return kmoe.MoETransformer(cfg, verbose=False), cfg


def test_library_trainer_loop_eval_and_format_a_checkpoints(tmp_path):
    """``Trainer``: accumulation keyed on the micro-step counter, metric names of the reference, evaluation,
    ``checkpoint_step_{N}.pt`` / ``checkpoint_final.pt`` and resume of the counters."""
    from kolmogorov_moe_architecture_b200.training.lr_schedule import CosineScheduleWithWarmup
    from kolmogorov_moe_architecture_b200.training.trainer import Trainer
    model, cfg = _tiny_model()
    g = torch.Generator().manual_seed(1)
    data = [{"input_ids": (t := torch.randint(0, 128, (2, 16), generator=g)), "labels": t} for _ in range(5)]
    opt = torch.optim.AdamW(model.parameters(), lr=1e-3)
    sched = CosineScheduleWithWarmup(opt, 2, 20, 1e-3, 1e-4, 0.0)
    jl = str(tmp_path / "log.jsonl")
    tr = Trainer(model, opt, sched, data, data[:2], {"run_name": "t"}, device="cpu", use_amp=False,
                 gradient_accumulation_steps=2, checkpoint_dir=str(tmp_path / "ck"), log_interval=1, eval_interval=3,
                 save_interval=3, jsonl_path=jl, verbose=False)    # updates fall on odd micro-steps (1, 3, 5, ...)
    tr.train(max_steps=9)
    names = sorted(os.listdir(tmp_path / "ck"))
    assert "checkpoint_final.pt" in names and any(n.startswith("checkpoint_step_") for n in names)
    rows = [json.loads(l) for l in open(jl)]
    train_rows = [r for r in rows if "loss" in r and "eval_loss" not in r]
    assert train_rows and {"lm_loss", "aux_loss", "lr", "grad_norm", "tokens_seen", "tokens_per_sec"} <= set(train_rows[0])
    assert any(k.startswith("mt_") for k in train_rows[0])
    assert any("eval_ppl" in r for r in rows)
    assert tr.epoch >= 1                                           # five batches, nine micro-steps: the loader wrapped
    ev = tr.evaluate(num_batches=2)
    assert ev["eval_ppl"] > 1.0
    model2, _ = _tiny_model()
    opt2 = torch.optim.AdamW(model2.parameters(), lr=1e-3)
    tr2 = Trainer(model2, opt2, CosineScheduleWithWarmup(opt2, 2, 20, 1e-3, 1e-4, 0.0), data, None, {}, device="cpu",
                  use_amp=False, checkpoint_dir=str(tmp_path / "ck2"), verbose=False)
    tr2.load_checkpoint(str(tmp_path / "ck" / "checkpoint_final.pt"))
    assert (tr2.global_step, tr2.tokens_seen) == (tr.global_step, tr.tokens_seen)
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), model2.state_dict().values()))


def test_hf_wrapper_signature_and_prefixed_checkpoint_keys(tmp_path):
    from kolmogorov_moe_architecture_b200.training import checkpoint as ck
    from kolmogorov_moe_architecture_b200.training.hf import MoEModelWrapper, make_hf_classes
    model, cfg = _tiny_model()
    w = MoEModelWrapper(model)
    ids = torch.randint(0, 128, (2, 16))
    out = w(input_ids=ids, labels=ids)
    assert set(out) == {"loss"} and out["loss"].requires_grad            # no logits materialised with labels
    out = w(input_ids=ids)
    assert out["logits"].shape == (2, 16, 128)
    assert all(k.startswith("model.") for k in w.state_dict())
    path = str(tmp_path / "pytorch_model.bin")
    torch.save(w.state_dict(), path)
    fresh, _ = _tiny_model()
    with torch.no_grad():
        for p in fresh.parameters():
            p.add_(1.0)
    ck.load_model_state(fresh, path)                                      # the prefix is stripped on load
    assert all(torch.equal(a, b) for a, b in zip(model.state_dict().values(), fresh.state_dict().values()))
    MoETrainer, Callback = make_hf_classes()
    logs = {"loss": 8.0}
    Callback(4).on_log(None, None, None, logs=logs)
    assert logs["true_loss"] == 2.0 and logs["accumulated_loss"] == 8.0
    assert hasattr(MoETrainer, "create_optimizer") and hasattr(MoETrainer, "compute_loss")


def test_block_annotations_open_a_range_per_block_and_direction():
    from kolmogorov_moe_architecture_b200.utils.profiling import annotate_blocks
    model, cfg = _tiny_model()
    ann = annotate_blocks(model)
    ids = torch.randint(0, 128, (2, 16))
    model.train()
    model(ids, labels=ids, return_logits=False)["loss"].backward()
    L = len(model.layers)
    assert ann.events == {"forward": 3 * L, "backward": L}       # block + mixer + FFN forward, block backward
    ann.remove()
    model(ids, labels=ids, return_logits=False)["loss"].backward()
    assert ann.events == {"forward": 3 * L, "backward": L}


def test_module_level_benchmarks_and_single_modules_of_the_reference_api():
    """``moe_arch.model.*`` exposes, beside the layer classes, one benchmark function per variant module, the
    ``MoDLayer`` wrapper and the single ``Expert``; ``moe_arch.kernels`` has its benchmark harness and build
    helpers.  All of them run on the CPU at small sizes."""
    import torch
    from moe_arch.kernels.benchmark import benchmark, create_test_data, verify_correctness
    from moe_arch.kernels.setup import get_cuda_arch_flags, get_gpu_arch
    from moe_arch.model.config import AdvancedMoEConfig
    from moe_arch.model.fp8_moe import benchmark_fp8_vs_bf16
    from moe_arch.model.fused_moe import benchmark_fused_vs_original
    from moe_arch.model.mod import MoDLayer
    from moe_arch.model.moe import Expert
    from moe_arch.model.sparse_moe import benchmark_sparse_vs_batched
    from moe_arch.model.triton_moe import benchmark_moe_implementations
    kw = dict(n_experts=4, d_model=32, d_ff=64, n_tokens=48, top_k=2, n_iters=1, device="cpu")
    t = benchmark_sparse_vs_batched(**kw)
    assert t["max_diff"] < 1e-5 and t["sparse"] > 0 and t["batched"] > 0
    t = benchmark_moe_implementations(**kw)
    assert t["max_diff"] < 1e-5 and {"BatchedMoE", "TritonGroupedExpertsFused"} <= set(t)
    t = benchmark_fused_vs_original(d_model=64, d_ff=64, n_experts=4, top_k=2, batch=2, seq_len=8, n_iters=1, device="cpu")
    assert set(t) == {"MoELayer", "FusedSparseMoE"}
    assert benchmark_fp8_vs_bf16(device="cpu") is None            # block-scaled fp8 exists on the GPU only
    data = create_test_data(4, 32, 64, 40, 2, device="cpu")
    assert data[0].shape == (80, 32) and bool((data[4][1:] >= data[4][:-1]).all()) and int(data[6][-1]) == 80
    assert verify_correctness(*data) and benchmark(*data, n_warmup=1, n_iters=1)["pytorch_ms"] > 0
    assert get_cuda_arch_flags() == ["-gencode", "arch=compute_100a,code=sm_100a"] and get_gpu_arch() is None
    # MoDLayer: kept positions get x + w * layer(x), the others pass unchanged; evaluation runs every position
    cfg = AdvancedMoEConfig(vocab_size=100, d_model=32, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                            d_ff_expert=32, n_experts=4, moe_layers=(1,), mamba_layers=(), max_seq_len=16,
                            mod_capacity_factor=0.5, dropout=0.0, device="cpu", dtype="float32")
    torch.manual_seed(0)
    layer = MoDLayer(cfg, torch.nn.Linear(32, 32))
    x = torch.randn(2, 16, 32)
    layer.train()
    y = layer(x)
    idx, w, _, _ = layer.router(x)
    changed = (y != x).any(-1)
    assert changed.sum(1).tolist() == [8, 8] and torch.equal(changed.nonzero()[:, 1].view(2, 8), idx)
    want = x[0, idx[0]] + w[0, :, None] * layer.layer(x[0, idx[0]])
    assert torch.allclose(y[0, idx[0]], want, atol=1e-6) and torch.is_tensor(layer.aux_loss)
    layer.eval()
    assert torch.allclose(layer(x), x + layer.layer(x)) and layer.aux_loss == 0.0
    e = Expert(cfg)
    assert e(torch.randn(5, 32)).shape == (5, 32) and {n for n, _ in e.named_parameters()} == {
        "expert_ffn.ffn.w1.weight", "expert_ffn.ffn.w2.weight", "expert_ffn.ffn.w3.weight"}


def test_grouped_swiglu_function_matches_the_differentiable_path():
    import torch
    from moe_arch.kernels import GroupedSwiGLUFunction, grouped_swiglu_with_grad
    from moe_arch.kernels.benchmark import create_test_data
    x, w1, w2, w3, ids, s0, s1 = create_test_data(3, 16, 32, 20, 2, device="cpu")
    a = [t.clone().requires_grad_(True) for t in (x, w1, w2, w3)]
    b = [t.clone().requires_grad_(True) for t in (x, w1, w2, w3)]
    ya = GroupedSwiGLUFunction.apply(*a, ids, s0, s1)
    yb = grouped_swiglu_with_grad(*b, ids)
    g = torch.randn_like(ya)
    ya.backward(g)
    yb.backward(g)
    assert torch.allclose(ya, yb, atol=1e-6)
    assert all(torch.allclose(p.grad, q.grad, atol=1e-6) for p, q in zip(a, b))
    frozen = GroupedSwiGLUFunction.apply(x.clone().requires_grad_(True), w1, w2, w3, ids)      # weights without gradients
    frozen.sum().backward()


def test_keyword_names_of_the_reference_are_accepted():
    import torch
    from moe_arch.model.ffn import ExpertFFN
    from moe_arch.model.triton_moe import sort_tokens_by_expert
    e = ExpertFFN(d_model=16, d_ff_expert=32)
    assert e(torch.randn(3, 16)).shape == (3, 16)
    idx = torch.tensor([[2, 0], [1, 2], [0, 1]])
    w = torch.tensor([[0.6, 0.4], [0.7, 0.3], [0.5, 0.5]])
    tok, ids, sw, s0, s1 = sort_tokens_by_expert(expert_indices=idx, expert_weights=w, n_experts=3)
    assert ids.tolist() == [0, 0, 1, 1, 2, 2] and tok.tolist() == [0, 2, 1, 2, 0, 1]
    assert torch.allclose(sw, torch.tensor([0.4, 0.5, 0.7, 0.5, 0.6, 0.3])) and s0.tolist() == [0, 2, 4] and s1.tolist() == [2, 4, 6]
    _, _, order, _, _ = sort_tokens_by_expert(idx, 3)
    assert torch.equal(w.reshape(-1)[order], sw)
