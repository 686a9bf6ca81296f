"""Reference arm of the benchmark: the unmodified reference package installed under
``baseline/_ref`` (``pip install --target baseline/_ref``; its root-level training scripts are
copied beside it in ``baseline/_ref/ref_scripts``), driven through its own public API:

* 1 GPU  - the single-GPU regime of the reference's ``train.py``: ``MoETransformer(config)``
  cast to bf16, ``get_muon_optimizer`` (Muon on 2-D weight matrices, AdamW on the rest),
  ``clip_grad_norm_``, ``optimizer.step()``.
* N GPUs - the regime of the reference's ``train_distributed.py``: the same model wrapped by
  its own ``wrap_model_with_fsdp`` (FULL_SHARD, bf16, activation checkpointing), same optimizer.

``--mamba-moe-mode`` selects what a layer listed in both ``moe_layers`` and ``mamba_layers``
becomes.  ``routing_mamba`` is the stock reference (RoutingMamba + dense FFN,
moe_arch/model/layers.py:58-82).  ``moe_ffn`` (the default of ``bench.py``, the layer the
benchmark names: Mamba mixer + MoE FFN) cannot be expressed by the reference's config, so
those layers are built by ``MambaMoEBlock`` below: a subclass of the reference's
``TransformerBlock`` that composes the reference's own unmodified ``MambaBlock`` and
``MoELayer`` and inherits its ``forward`` untouched.  Both arms then hold the same
parameter count (``params_b``).

Nothing from this repository's package is imported here.  The same JSON line as the other
arm is printed, with ``"impl": "reference"``; if the reference cannot be imported or run,
``{"impl": "reference", "unavailable": "<reason>"}`` is printed instead and the exit code is 0.
"""
from __future__ import annotations

import json
import os
import sys
import traceback

import torch

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
METRIC = "train_tokens_per_sec_5b_hybrid_moe"


def _unavailable(why: str):
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps({"impl": "reference", "unavailable": why.replace("\n", " ")[:300]}), flush=True)


def _import_reference():
    for k in [k for k in sys.modules if k == "moe_arch" or k.startswith("moe_arch.")]:
        del sys.modules[k]
    sys.path.insert(0, os.path.join(REF, "ref_scripts"))
    sys.path.insert(0, REF)
    from moe_arch.model.config import AdvancedMoEConfig
    from moe_arch.model.transformer import MoETransformer
    from moe_arch.training.muon_optimizer import get_muon_optimizer
    import moe_arch
    assert os.path.abspath(moe_arch.__file__).startswith(REF), "wrong moe_arch on the path"
    return AdvancedMoEConfig, MoETransformer, get_muon_optimizer


def _mamba_moe_block_factory():
    """``TransformerBlock`` factory for ``--mamba-moe-mode moe_ffn``.

    A layer in both lists is first built by the reference's own constructor as a Mamba layer
    without MoE (``MambaBlock`` + dense FFN), then its FFN is replaced by the reference's
    ``MoELayer`` and ``use_moe`` is switched on, which is all the inherited ``forward``
    (moe_arch/model/layers.py:96-207) needs to run the mixer, the MoD routing and the MoE
    auxiliary loss.  Every other layer is the stock block."""
    import dataclasses
    from moe_arch.model.layers import TransformerBlock
    from moe_arch.model.moe import MoELayer
    from moe_arch.model.mamba import MambaBlock

    class MambaMoEBlock(TransformerBlock):
        def __init__(self, config, layer_idx):
            plain = dataclasses.replace(
                config, moe_layers=tuple(i for i in config.moe_layers if i != layer_idx))
            super().__init__(plain, layer_idx)
            assert isinstance(self.seq_layer, MambaBlock)
            self.config = config
            self.use_moe = True
            self.ffn = MoELayer(config, layer_idx)

    def make(config, layer_idx):
        both = config.mamba_enabled and layer_idx in config.mamba_layers and layer_idx in config.moe_layers
        return (MambaMoEBlock if both else TransformerBlock)(config, layer_idx)

    return make, TransformerBlock


def _build_model(MoETransformer, cfg, mode: str):
    """Stock ``MoETransformer(cfg)``; for ``moe_ffn`` the name ``TransformerBlock`` that its
    constructor looks up (moe_arch/model/transformer.py:56-59) is pointed at the factory
    above for the duration of the call.  No reference file is edited."""
    if mode == "routing_mamba":
        return MoETransformer(cfg)
    import moe_arch.model.transformer as ref_tf
    make, stock = _mamba_moe_block_factory()
    ref_tf.TransformerBlock = make
    try:
        return MoETransformer(cfg)
    finally:
        ref_tf.TransformerBlock = stock


def run_reference(args):
    if not os.path.isdir(os.path.join(REF, "moe_arch")):
        return _unavailable("baseline/_ref/moe_arch is missing (reference not installed)")
    try:
        _run(args)
    except Exception as e:  # the arm must exit 0 and say why
        traceback.print_exc(file=sys.stderr)
        _unavailable(f"{type(e).__name__}: {e}")


def _run(args):
    from bench import ClockSampler, barrier, dist_setup, max_over_ranks, metric_name, workload_config
    AdvancedMoEConfig, MoETransformer, get_muon_optimizer = _import_reference()
    world, rank, local = dist_setup(args)
    dev = torch.device("cuda", local)
    L = args.layers
    cfg = AdvancedMoEConfig(
        vocab_size=50304, n_layers=L, max_seq_len=args.seq_len,
        moe_layers=tuple(i for i in range(L) if i % 4 in (1, 2)),
        mamba_layers=tuple(i for i in range(L) if i % 4 == 1),
        dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)
    mode = getattr(args, "mamba_moe_mode", "moe_ffn")
    torch.manual_seed(0)
    if rank != 0:
        sys.stdout = open(os.devnull, "w")
    ckpt = world > 1
    if world == 1:
        model = _build_model(MoETransformer, cfg, mode).to(dev).to(torch.bfloat16)
        model.train()
        regime = "train.py single-GPU regime: bf16 weights, no activation checkpointing"
    else:
        from train_distributed import wrap_model_with_fsdp
        with torch.device(dev):
            model = _build_model(MoETransformer, cfg, mode)
        n_params_unwrapped = sum(p.numel() for p in model.parameters())
        model = wrap_model_with_fsdp(model, rank, use_bf16=True, cpu_offload=False, activation_checkpointing=True)
        model.train()
        regime = "train_distributed.py regime: FSDP FULL_SHARD bf16 + activation checkpointing"
    n_params = n_params_unwrapped if ckpt else sum(p.numel() for p in model.parameters())
    os.environ.setdefault("WORLD_SIZE", str(world))
    optimizer = get_muon_optimizer(model, lr=1e-3)
    sys.stdout = sys.__stdout__

    B, S = args.micro_batch, args.seq_len
    g = torch.Generator().manual_seed(1234 + rank)
    host = [torch.randint(0, cfg.vocab_size, (B, S), generator=g).pin_memory() for _ in range(4)]
    devb = [h.to(dev) for h in host]

    def step(ids):
        out = model(ids, labels=ids, return_logits=False)
        out["loss"].backward()
        if world == 1:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        else:
            model.clip_grad_norm_(1.0)
        optimizer.step()
        optimizer.zero_grad(set_to_none=True)
        return out["loss"]

    for i in range(args.warmup):
        step(devb[i % 4])
    barrier(world)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        step(devb[i % 4])
    e1.record()
    barrier(world)
    ms = max_over_ranks(e0.elapsed_time(e1), world)
    clocks = sampler.stop() if rank == 0 else {}
    tokens = B * S * world * args.steps
    barrier(world)
    e0.record()
    last = 0.0
    for i in range(args.steps):
        last = float(step(host[i % 4].to(dev, non_blocking=True)).item())
    e1.record()
    barrier(world)
    ms2 = max_over_ranks(e0.elapsed_time(e1), world)
    if rank == 0:
        mamba = "mamba_ssm" if _has_mamba_ssm() else "SimpleSSM fallback (mamba_ssm not installed)"
        print(json.dumps({
            "metric": metric_name(args), "value": tokens / (ms / 1e3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "impl": "reference", "clocks": clocks,
            "e2e": {"value": tokens / (ms2 / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": B * S * 8,
                    "d2h_bytes_per_step": 4, "ms_per_step": ms2 / args.steps, "last_loss": last},
            "config": workload_config(args, world, L == 32 and B == 4 and S == 2048),
            "detail": {"params_b": round(n_params / 1e9, 3),
                       "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2**30, 1),
                       "model": ("reference MoETransformer; Mamba+MoE layers = the reference's own MambaBlock + "
                                 "MoELayer composed by a harness-side TransformerBlock subclass"
                                 if mode == "moe_ffn" else
                                 "stock reference MoETransformer (a layer in both moe_layers and mamba_layers "
                                 "is RoutingMamba + dense FFN)"),
                       "regime": regime, "mamba": mamba,
                       "optimizer": "get_muon_optimizer (Muon8bit + AdamW)"}}), flush=True)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


def _has_mamba_ssm() -> bool:
    try:
        import mamba_ssm  # noqa: F401
        return True
    except Exception:
        return False
