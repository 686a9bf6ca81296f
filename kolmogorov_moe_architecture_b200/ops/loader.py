"""Locate and load the in-tree CUDA extension (``_C.so`` beside the package).

The library registers its operators under ``torch.ops.kmoe`` when loaded.  It
is built by ``build_ext.py`` at the repository root (``python build_ext.py``).
"""
from __future__ import annotations

import os
import threading

import torch

_LOCK = threading.Lock()
_STATE = {"tried": False, "ok": False, "err": None}

PKG_DIR = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
EXT_PATH = os.path.join(PKG_DIR, "_C.so")


def load_ext() -> bool:
    with _LOCK:
        if _STATE["tried"]:
            return _STATE["ok"]
        _STATE["tried"] = True
        if not os.path.exists(EXT_PATH):
            _STATE["err"] = f"{EXT_PATH} not found (run `python build_ext.py`)"
            return False
        try:
            torch.ops.load_library(EXT_PATH)
            _STATE["ok"] = True
        except Exception as e:  # pragma: no cover - depends on the toolchain
            _STATE["err"] = repr(e)
        return _STATE["ok"]


def ext_available() -> bool:
    return load_ext()


def require_ext() -> None:
    if not load_ext():
        raise RuntimeError(
            "the kmoe CUDA extension is required for CUDA tensors but could not be loaded: "
            f"{_STATE['err']}")
