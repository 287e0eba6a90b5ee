"""Loader and thin Python surface of the in-tree sm_100a extension (``ops/csrc``).

The shared object is built by ``ops/build.py`` (nvcc, ``-gencode arch=compute_100a,code=sm_100a``)
next to this file so it ships with the source tree.  On a machine with a CUDA device a missing or
unloadable extension is an error, never a silent fallback.
"""
from __future__ import annotations

import glob
import os
from typing import Optional

import torch

_EXT = None
_TRIED = False
_LAUNCHES = 0          # kernels of this library launched since the last reset (host-side count)
_HERE = os.path.dirname(os.path.abspath(__file__))


def so_path() -> Optional[str]:
    hits = sorted(glob.glob(os.path.join(_HERE, "_loom_b200*.so")))
    return hits[0] if hits else None


def load(required: bool = False):
    global _EXT, _TRIED
    if _EXT is not None:
        return _EXT
    if _TRIED and not required:
        return None
    _TRIED = True
    path = so_path()
    if path is None:
        if required:
            raise RuntimeError("native extension _loom_b200 is not built; run `python -m "
                               "loomformer_paraplex_b200.ops.build`")
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("_loom_b200", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    _EXT = mod
    return mod


def available() -> bool:
    """True when CUDA is present and the extension is loaded (raises if CUDA is present but the
    extension is missing, so GPU runs cannot silently use PyTorch fallbacks)."""
    if not torch.cuda.is_available():
        return False
    return load(required=True) is not None


def ext():
    return load(required=True)


def count(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launches() -> int:
    return _LAUNCHES


def reset_launches() -> None:
    global _LAUNCHES
    _LAUNCHES = 0


def optimizer_step(opt) -> None:
    from . import kernels
    kernels.optimizer_step(opt)
