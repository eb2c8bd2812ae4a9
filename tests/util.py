"""Shared helpers of the tests: synthetic weight files and engine pairs (product, oracle)."""
from __future__ import annotations

import functools
import os
import tempfile
from pathlib import Path

import numpy as np

from silicon_violetto_b200 import synth

_TMP = Path(tempfile.mkdtemp(prefix="vlt_tests_"))

# A decoder smaller than the benchmark's plumbing configuration, for cases the CPU oracle must finish in a blink.
MICRO = dict(n_layers=2, d=256, n_heads=4, n_kv=2, hd=64, ffn=512, vocab=512, eps=1e-5, theta=500000.0, page=16)
MICRO4 = dict(n_layers=1, d=256, n_heads=8, n_kv=2, hd=64, ffn=256, vocab=256, eps=1e-5, theta=500000.0, page=16)  # 4 query heads per kv head


@functools.lru_cache(maxsize=None)
def weights(name: str, int8_group=None, seed: int = 0) -> Path:
    cfg = {"micro": MICRO, "micro4": MICRO4}.get(name, name)
    tag = name if isinstance(name, str) else "custom"
    path = _TMP / f"{tag}_{int8_group}_{seed}.vlt"
    if not path.exists():
        synth.write_target(path, cfg, seed=seed, int8_group=int8_group)
    return path


def cuda_available() -> bool:
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


@functools.lru_cache(maxsize=None)
def _custom(tag: str, items: tuple, int8_group=None, seed: int = 0) -> Path:
    path = _TMP / f"{tag}_{int8_group}_{seed}.vlt"
    if not path.exists():
        synth.write_target(path, dict(items), seed=seed, int8_group=int8_group)
    return path


def weights_custom(tag: str, cfg: dict, int8_group=None, seed: int = 0) -> Path:
    return _custom(tag, tuple(sorted(cfg.items())), int8_group, seed)
