"""Opt-in validation of data-dependent kernel inputs (``KMOE_CHECK_INPUTS=1``).

The kernels index memory with values that come from data: expert ids pick a weight matrix and a histogram bin,
labels pick a logit, mixture-of-depths and expert-choice indices pick token rows, packed-document starts bound the
keys a query may see.  The kernels trust those values (a test per element would cost a host read or a device-side
error path on every launch).  With ``KMOE_CHECK_INPUTS=1`` every dispatch function in :mod:`..ops` validates them
first, on whatever device they live, and raises ``IndexError`` / ``ValueError`` naming the first offending element
instead of launching.  Each check costs a device-to-host read, so the mode is for debugging a new data pipeline or
router, not for training runs.  It is the host-side counterpart of a bounds-checking kernel build: nothing on the
device ever traps.
"""
from __future__ import annotations

import os

import torch


def enabled() -> bool:
    return os.environ.get("KMOE_CHECK_INPUTS", "0") == "1"


def _first(mask: torch.Tensor):
    """Index tuple of the first True element of ``mask``."""
    flat = int(torch.nonzero(mask.reshape(-1))[0])
    out = []
    for n in reversed(mask.shape):
        out.append(flat % n)
        flat //= n
    return tuple(reversed(out))


def _integral(t: torch.Tensor, what: str) -> None:
    if t.is_floating_point() or t.is_complex() or t.dtype == torch.bool:
        raise ValueError(f"{what}: expected an integer tensor, got {t.dtype}")


def index_range(idx: torch.Tensor, upper: int, what: str, lower: int = 0) -> None:
    """Every element of ``idx`` lies in [lower, upper)."""
    _integral(idx, what)
    if idx.numel() == 0:
        return
    bad = (idx < lower) | (idx >= upper)
    if bool(bad.any()):
        at = _first(bad)
        raise IndexError(f"{what}: value {int(idx[at])} at position {at} is outside [{lower}, {upper})")


def expert_indices(idx: torch.Tensor, n_experts: int, top_k_distinct: bool = True) -> None:
    """Token-choice assignments (T, k): ids in [0, E) and, per token, distinct (the slot sizing of the
    expert-parallel exchange and the capacity of a (expert, source) pair rely on it)."""
    index_range(idx, n_experts, "expert index")
    if top_k_distinct and idx.dim() == 2 and idx.shape[1] > 1 and idx.numel() > 0:
        s, _ = torch.sort(idx, dim=1)
        dup = s[:, 1:] == s[:, :-1]
        if bool(dup.any()):
            at = _first(dup)
            raise ValueError(f"expert index: token {at[0]} is assigned to expert {int(s[at[0], at[1]])} twice")


def routing_weights(w: torch.Tensor, what: str = "routing weights") -> None:
    if w.numel() and not bool(torch.isfinite(w).all()):
        at = _first(~torch.isfinite(w))
        raise ValueError(f"{what}: non-finite value at position {at}")


def labels(lab: torch.Tensor, vocab: int, ignore_index: int = -100) -> None:
    """Targets of the cross-entropy: the ignore value or a class in [0, vocab)."""
    _integral(lab, "labels")
    if lab.numel() == 0:
        return
    bad = ((lab < 0) | (lab >= vocab)) & (lab != ignore_index)
    if bool(bad.any()):
        at = _first(bad)
        raise IndexError(f"labels: value {int(lab[at])} at position {at} is neither {ignore_index} nor in [0, {vocab})")


def kept_rows(idx: torch.Tensor, n_rows: int, what: str = "kept positions", ascending: bool = True) -> None:
    """Per-sequence row selections (B, k): in range, and strictly ascending (hence distinct) where the kernels
    rely on it (the mixture-of-depths gather / scatter writes each kept row once)."""
    index_range(idx, n_rows, what)
    if ascending and idx.dim() >= 2 and idx.shape[-1] > 1 and idx.numel() > 0:
        bad = idx[..., 1:] <= idx[..., :-1]
        if bool(bad.any()):
            at = _first(bad)
            raise ValueError(f"{what}: not strictly ascending at position {at} "
                             f"({int(idx[at])} is followed by {int(idx[at[:-1] + (at[-1] + 1,)])})")


def distinct_rows(idx: torch.Tensor, n_rows: int, what: str) -> None:
    """Selections (..., C) whose last dimension must not repeat a row (expert-choice: an expert takes a token once)."""
    index_range(idx, n_rows, what)
    if idx.shape[-1] > 1 and idx.numel() > 0:
        s, _ = torch.sort(idx, dim=-1)
        dup = s[..., 1:] == s[..., :-1]
        if bool(dup.any()):
            at = _first(dup)
            raise ValueError(f"{what}: row {int(s[at])} is selected twice in group {at[:-1]}")


def doc_start(ds: torch.Tensor) -> None:
    """Packed-document starts (B, S): ``ds[b, i]`` is the first position of the document that holds position i, so
    0 <= ds[b, i] <= i, and it never decreases along the sequence (the kernels skip whole key blocks on that)."""
    _integral(ds, "doc_start")
    if ds.numel() == 0:
        return
    if ds.dim() != 2:
        raise ValueError(f"doc_start: expected (batch, seq), got shape {tuple(ds.shape)}")
    pos = torch.arange(ds.shape[1], device=ds.device).expand_as(ds)
    bad = (ds < 0) | (ds > pos)
    if bool(bad.any()):
        at = _first(bad)
        raise IndexError(f"doc_start: value {int(ds[at])} at position {at} is outside [0, {at[1]}]")
    dec = ds[:, 1:] < ds[:, :-1]
    if bool(dec.any()):
        at = _first(dec)
        raise ValueError(f"doc_start: decreases after position {at} ({int(ds[at])} -> {int(ds[at[0], at[1] + 1])})")


def keep_mask(keep, idx: torch.Tensor) -> None:
    if keep is None:
        return
    if keep.numel() != idx.numel():
        raise ValueError(f"keep mask has {keep.numel()} elements for {idx.numel()} assignments")
