"""Forward hooks that capture the input and output of every feed-forward block of an arbitrary
transformer (counterpart of the reference's ``Experiments/sparse_distillation/hooks.py``).

FFN modules are discovered by name: the last path component is one of ``mlp``, ``ffn``,
``feed_forward``, ``ff`` (HF LLaMA/GPT-style models and this framework's blocks all match).
"""
from __future__ import annotations

from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.nn as nn

FFN_NAMES = ("mlp", "ffn", "feed_forward", "ff")


def find_ffn_modules(model: nn.Module, names=FFN_NAMES) -> List[Tuple[str, nn.Module]]:
    found = []
    for name, mod in model.named_modules():
        leaf = name.split(".")[-1].lower()
        if leaf in names and not any(name.startswith(p + ".") for p, _ in found):
            found.append((name, mod))
    return found


class FFNActivationCache:
    """``with FFNActivationCache(model) as cache: model(x)`` then ``cache.inputs[i]`` / ``cache.outputs[i]``
    hold the (detached) activations of FFN layer i for the last forward."""

    def __init__(self, model: nn.Module, layers: Optional[List[int]] = None, detach: bool = True, to_cpu: bool = False):
        self.model, self.detach, self.to_cpu = model, detach, to_cpu
        self.ffn = find_ffn_modules(model)
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

    __enter__ = register

    def __exit__(self, *exc):
        self.remove()
        return False


class StreamingFFNExtractor:
    """Calls ``fn(layer_idx, ffn_input, ffn_output)`` during the forward pass instead of storing
    activations, so only one layer's tensors are alive at a time."""

    def __init__(self, model: nn.Module, fn: Callable[[int, torch.Tensor, torch.Tensor], None]):
        self.ffn = find_ffn_modules(model)
        self.fn = fn
        self._handles = []

    def __enter__(self):
        for i, (_, mod) in enumerate(self.ffn):
            self._handles.append(mod.register_forward_hook(
                lambda m, inp, out, i=i: self.fn(i, inp[0].detach(), (out[0] if isinstance(out, tuple) else out).detach())))
        return self

    def __exit__(self, *exc):
        for h in self._handles:
            h.remove()
        return False
