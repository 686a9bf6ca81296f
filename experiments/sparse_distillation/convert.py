"""Swap the dense FFNs of a model for trained MoE layers (counterpart of the reference's
``Experiments/sparse_distillation/convert.py``)."""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn

from .distill import MoEDistillationLayer
from .hooks import find_ffn_modules


def _set_submodule(root: nn.Module, path: str, new: nn.Module) -> None:
    parts = path.split(".")
    parent = root
    for p in parts[:-1]:
        parent = getattr(parent, p) if not p.isdigit() else parent[int(p)]
    if parts[-1].isdigit():
        parent[int(parts[-1])] = new
    else:
        setattr(parent, parts[-1], new)


def replace_ffn_with_moe(model: nn.Module, moe_layers, layer_indices=None, ffn_name_pattern: Optional[str] = None,
                         inplace: bool = True) -> nn.Module:
    """Put ``moe_layers[str(i)]`` (a dict or ``nn.ModuleDict`` keyed by layer index) in the place of the i-th
    feed-forward block.  ``layer_indices`` restricts the replacement to those layers; ``ffn_name_pattern`` names the
    attribute of the blocks (``"mlp"``, ``"ffn"``, ...) when the default name rule should not decide;
    ``inplace=False`` works on a deep copy (reference: convert.py:18-77, which copies by default; here the default
    is in place, because the copy of a multi-billion-parameter model is rarely wanted)."""
    if not inplace:
        import copy
        model = copy.deepcopy(model)
    names = (ffn_name_pattern,) if ffn_name_pattern else None
    found = find_ffn_modules(model, names=names) if names else find_ffn_modules(model)
    wanted = None if layer_indices is None else {int(i) for i in layer_indices}
    for i, (name, _) in enumerate(found):
        if str(i) in moe_layers and (wanted is None or i in wanted):
            _set_submodule(model, name, moe_layers[str(i)])
    return model


class SparseModelWrapper(nn.Module):
    """The converted model plus helpers: routing statistics of the last forward and parameter counts."""

    def __init__(self, model: nn.Module = None, moe_paths: Dict[int, str] = None, base_model: nn.Module = None,
                 moe_layers=None, layer_indices=None):
        """``SparseModelWrapper(model, {layer: path of its MoE module})``, or in the reference's form
        ``SparseModelWrapper(base_model, moe_layers, layer_indices)`` with the MoE layers already in the model: the
        paths are then found by identity."""
        super().__init__()
        model = base_model if model is None else model
        if moe_paths is not None and not all(isinstance(v, str) for v in dict(moe_paths).values()):
            moe_layers, moe_paths = moe_paths, None            # second positional was the reference's moe_layers
        if moe_paths is None:
            where = {id(m): n for n, m in model.named_modules()}
            items = moe_layers.items() if moe_layers is not None else []
            moe_paths = {int(k): where[id(m)] for k, m in items if id(m) in where
                         and (layer_indices is None or int(k) in {int(i) for i in layer_indices})}
        self.model, self.moe_paths = model, dict(moe_paths)

    def forward(self, *a, **kw):
        return self.model(*a, **kw)

    def moe_modules(self):
        mods = dict(self.model.named_modules())
        return {i: mods[p] for i, p in self.moe_paths.items()}

    def routing_stats(self) -> Dict[int, Dict[str, float]]:
        out = {}
        for i, m in self.moe_modules().items():
            c = getattr(m, "_last_expert_counts", None)
            if c is not None:
                u = c.float() / c.sum().clamp(min=1)
                out[i] = {"max_usage": float(u.max()), "dead": int((u == 0).sum()),
                          "entropy": float(-(u * torch.log(u + 1e-10)).sum() / torch.log(torch.tensor(float(len(u)))))}
        return out

    # the reference's view of the same object (Experiments/sparse_distillation/convert.py:80-143)
    @property
    def base_model(self) -> nn.Module:
        return self.model

    @property
    def moe_layers(self) -> nn.ModuleDict:
        """The MoE layers keyed by layer index (a view: the modules live inside ``model``)."""
        return nn.ModuleDict({str(i): m for i, m in self.moe_modules().items()})

    @property
    def n_experts(self) -> int:
        """Experts per layer (of the first MoE layer; layers may differ under a per-layer configuration)."""
        return next(iter(self.moe_modules().values())).n_experts

    def get_active_parameters(self, top_k: Optional[int] = None) -> int:
        """Parameters a token touches: everything outside the experts, plus ``top_k`` of each layer's experts
        (each layer's own ``top_k`` when none is given)."""
        total = sum(p.numel() for p in self.model.parameters())
        idle = 0.0
        for m in self.moe_modules().values():
            k = min(top_k if top_k is not None else m.top_k, m.n_experts)
            idle += sum(p.numel() for p in m.experts.parameters()) * (1.0 - k / m.n_experts)
        return int(total - idle)

    def count_parameters(self) -> Dict[str, int]:
        total = sum(p.numel() for p in self.model.parameters())
        expert = sum(p.numel() for m in self.moe_modules().values() for p in m.experts.parameters())
        frac = next(iter(self.moe_modules().values())).top_k / next(iter(self.moe_modules().values())).n_experts \
            if self.moe_paths else 1.0
        return {"total": total, "expert": expert, "active": int(total - expert * (1 - frac))}


def infer_layer_dims(state: Dict[str, torch.Tensor]):
    """(n_experts, d_model, d_ff) from a saved MoE layer's ``experts.w1`` shape."""
    w1 = state["experts.w1"]
    return w1.shape[0], w1.shape[1], w1.shape[2]


def convert_to_sparse(model: nn.Module = None, distilled_path: Optional[str] = None, trainer=None,
                      random_init: bool = False, layer_config_path: Optional[str] = None,
                      device=None, dense_model: nn.Module = None,
                      distillation_checkpoint: Optional[str] = None) -> SparseModelWrapper:
    """Build the sparse model from a ``SparseDistillationTrainer`` or from its ``save()`` file.
    ``random_init=True`` keeps the architecture but re-initialises the experts (a control).
    ``layer_config_path``: the per-layer file of ``generate_config``; expert counts and widths always come from
    the saved weights' shapes, the file supplies each layer's ``top_k`` (and must agree with the shapes).
    ``device``: where the model goes first (default: where it is)."""
    model = dense_model if model is None else model                      # the reference's keyword names
    distilled_path = distillation_checkpoint if distilled_path is None else distilled_path
    if device is not None:
        model.to(device)
    per_layer = {}
    if layer_config_path:
        import json
        per_layer = json.load(open(layer_config_path))
        per_layer = per_layer.get("layers", per_layer)
    if trainer is not None:
        layers = {k: v for k, v in trainer.get_moe_layers().items()}
    else:
        from .distill import checkpoint_config, checkpoint_layers, load_layer_state
        ck = torch.load(distilled_path, map_location="cpu", weights_only=False)
        cfg = checkpoint_config(ck)
        if any(k.startswith("router.mlp.") for sd in checkpoint_layers(ck).values() for k in sd) and not cfg.router_mlp:
            import dataclasses
            cfg = dataclasses.replace(cfg, router_mlp=True)
        layers = {}
        for k, sd in checkpoint_layers(ck).items():
            E, d, f = infer_layer_dims(sd)
            top_k = ck.get("dims", {}).get(k, (d, f, E, cfg.moe_top_k))[3]
            lc = per_layer.get(str(k), {})
            if lc:
                if int(lc.get("n_experts", E)) != E or int(lc.get("d_ff_expert", f)) != f:
                    raise ValueError(f"layer {k}: the layer configuration says {lc.get('n_experts')} experts of width "
                                     f"{lc.get('d_ff_expert')}, the checkpoint holds {E} of width {f}")
                top_k = int(lc.get("top_k", top_k))
            layer = MoEDistillationLayer(d, f, cfg, n_experts=E, top_k=top_k)
            load_layer_state(layer, sd)
            layers[k] = layer
    if random_init:
        for layer in layers.values():
            for p in layer.experts.parameters():
                nn.init.normal_(p, std=0.02)
    paths = {i: name for i, (name, _) in enumerate(find_ffn_modules(model)) if str(i) in layers}
    p0 = next(model.parameters())
    for layer in layers.values():
        layer.to(p0.device).to(p0.dtype)
    replace_ffn_with_moe(model, layers)
    return SparseModelWrapper(model, paths)
