"""Forward hooks that capture the input and output of every feed-forward block of an arbitrary
transformer (counterpart of the reference's ``Experiments/sparse_distillation/hooks.py``).

FFN modules are discovered by name: the last path component is one of ``mlp``, ``ffn``,
``feed_forward``, ``ff`` (HF LLaMA/GPT-style models and this framework's blocks all match).

Layers are numbered in the order they are found, 0 .. n-1.  The reference numbers a layer by the first number in
its module path (``model.layers.5.mlp`` -> 5, hooks.py:98-106); the two agree whenever every block of the model has
a feed-forward module, which is what its checkpoints' layer keys assume.  With a ``layer_filter`` that keeps only
some blocks the numbers differ: here the kept layers are renumbered.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

FFN_NAMES = ("mlp", "ffn", "feed_forward", "ff")


@dataclass
class FFNActivation:
    """Input and output of one FFN layer for the last forward pass, (batch, seq, d_model) each."""
    layer_idx: int
    input: torch.Tensor
    output: torch.Tensor


def find_ffn_modules(model: nn.Module, names=FFN_NAMES,
                     layer_filter: Optional[Callable[[str, nn.Module], bool]] = None) -> List[Tuple[str, nn.Module]]:
    """(path, module) of every feed-forward block, outermost match only.  ``layer_filter(name, module)`` replaces
    the name rule when given."""
    found = []
    for name, mod in model.named_modules():
        leaf = name.split(".")[-1].lower()
        hit = layer_filter(name, mod) if layer_filter is not None else leaf in names
        if name and hit and not any(name.startswith(p + ".") for p, _ in found):
            found.append((name, mod))
    return found


class FFNActivationCache:
    """``with FFNActivationCache(model) as cache: model(x)`` then ``cache.inputs[i]`` / ``cache.outputs[i]``
    hold the (detached) activations of FFN layer i for the last forward."""

    def __init__(self, model: nn.Module, layers: Optional[List[int]] = None, detach: bool = True, to_cpu: bool = False,
                 layer_filter: Optional[Callable[[str, nn.Module], bool]] = None):
        self.model, self.detach, self.to_cpu = model, detach, to_cpu
        self.ffn = find_ffn_modules(model, layer_filter=layer_filter)
        self.layers = list(range(len(self.ffn))) if layers is None else layers
        self.inputs: Dict[int, torch.Tensor] = {}
        self.outputs: Dict[int, torch.Tensor] = {}
        self._handles = []

    @property
    def n_layers(self) -> int:
        return len(self.ffn)

    def _keep(self, t):
        if isinstance(t, tuple):
            t = t[0]
        if self.detach:
            t = t.detach()
        return t.cpu() if self.to_cpu else t

    def register(self):
        for i in self.layers:
            def hook(mod, inp, out, i=i):
                self.inputs[i] = self._keep(inp[0])
                self.outputs[i] = self._keep(out)
            self._handles.append(self.ffn[i][1].register_forward_hook(hook))
        return self

    def remove(self):
        for h in self._handles:
            h.remove()
        self._handles = []

    def clear(self):
        self.inputs.clear()
        self.outputs.clear()

    # the reference's names for the same operations (Experiments/sparse_distillation/hooks.py:108-158)
    @property
    def layer_indices(self) -> List[int]:
        return list(self.layers)

    def register_hooks(self):
        return self.register()

    def remove_hooks(self):
        self.remove()

    def get_activations(self) -> Dict[int, FFNActivation]:
        return {i: FFNActivation(i, self.inputs[i], self.outputs[i]) for i in sorted(self.inputs) if i in self.outputs}

    def get_layer_activation(self, layer_idx: int) -> Optional[FFNActivation]:
        return self.get_activations().get(layer_idx)

    __enter__ = register

    def __exit__(self, *exc):
        self.remove()
        return False


class StreamingFFNExtractor:
    """Activations without keeping them around, in two forms.

    Pull (the reference's form, hooks.py:171-243): ``StreamingFFNExtractor(model).extract(input_ids)`` runs one
    forward pass of the (evaluation-mode) model and returns ``{layer: FFNActivation}`` for that batch only.

    Push: ``with StreamingFFNExtractor(model, fn): model(x)`` calls ``fn(layer, ffn_input, ffn_output)`` as each
    layer runs, so only one layer's tensors are alive at a time."""

    def __init__(self, model: nn.Module, fn: Optional[Callable[[int, torch.Tensor, torch.Tensor], None]] = None,
                 **cache_kwargs):
        self.model, self.fn = model, fn
        self._handles = []
        if fn is None:
            self.cache = FFNActivationCache(model, **cache_kwargs)
            self.cache.register_hooks()
            self.ffn = self.cache.ffn
            model.eval()
        else:
            self.cache = None
            self.ffn = find_ffn_modules(model, layer_filter=cache_kwargs.get("layer_filter"))

    @torch.no_grad()
    def extract(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                **kwargs) -> Dict[int, FFNActivation]:
        assert self.cache is not None, "extract() belongs to the form without a callback"
        self.cache.clear()
        if attention_mask is not None:
            kwargs["attention_mask"] = attention_mask
        self.model(input_ids, **kwargs)
        return self.cache.get_activations()

    @property
    def n_layers(self) -> int:
        return len(self.ffn)

    @property
    def layer_indices(self) -> List[int]:
        return self.cache.layer_indices if self.cache is not None else list(range(len(self.ffn)))

    def close(self) -> None:
        if self.cache is not None:
            self.cache.remove_hooks()
        for h in self._handles:
            h.remove()
        self._handles = []

    def __enter__(self):
        if self.fn is not None:
            for i, (_, mod) in enumerate(self.ffn):
                self._handles.append(mod.register_forward_hook(
                    lambda m, inp, out, i=i: self.fn(i, inp[0].detach(),
                                                     (out[0] if isinstance(out, tuple) else out).detach())))
        return self

    def __exit__(self, *exc):
        self.close()
        return False

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
