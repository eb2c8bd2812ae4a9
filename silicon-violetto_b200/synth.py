"""Random-init weight files for the benchmark configurations (no checkpoint or dataset is
needed: the decode step's speed and its parity against the oracle depend on shapes only).

A target file holds what the reference's converter writes (tools/convert.py:64-114), with
a plain decoder's tensor set: `embed` (bf16), optional int8 `head` (+ `head.scale`),
`L%02d.qkv|o|gate_up|down` (bf16, or int8 + `.scale`), `rope_freq` (f32) and a `meta`
descriptor (f32, as the reference's drafter file carries one: tools/spec/export.py:53).
gate_up rows are interleaved gate_0, up_0, gate_1, ... (tools/convert.py:102). RMSNorm gains
are folded into the following matrix's columns, as the reference folds its drafter's output
gain (tools/spec/export.py:50); at random init they are 1.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from . import vlt

CONFIGS = {
    # Benchmark configuration 0: the plumbing check.
    "tiny": dict(n_layers=2, d=256, n_heads=4, n_kv=2, hd=64, ffn=1024, vocab=4096, eps=1e-5, theta=500000.0, page=16),
    # Benchmark configurations 2 to 4: the 1B target.
    "1b": dict(n_layers=16, d=2048, n_heads=32, n_kv=8, hd=64, ffn=8192, vocab=128256, eps=1e-5, theta=500000.0, page=16),
}
META_VERSION = 1.0
PRESET_LLAMA = 0.0
DRAFTER_KIND_CHAIN = 1.0


def meta_tensor(c: dict) -> np.ndarray:
    return np.array([META_VERSION, PRESET_LLAMA, c["n_layers"], c["d"], c["n_heads"], c["n_kv"], c["hd"], c["ffn"], c["vocab"],
                     c.get("vocab_real", c["vocab"]), c["eps"], c["page"], c["theta"], 1.0 / np.sqrt(c["hd"])], dtype=np.float32)


def rope_freq(c: dict) -> np.ndarray:
    i = np.arange(c["hd"] // 2, dtype=np.float64)
    return (c["theta"] ** (-2.0 * i / c["hd"])).astype(np.float32)


def _randn(gen: torch.Generator, m: int, k: int, std: float) -> np.ndarray:
    """N(0, std^2) rounded to bf16 (a checkpoint's weights are bf16), as fp32."""
    return (torch.randn(m, k, generator=gen) * std).to(torch.bfloat16).float().numpy()


def _put(out: dict, name: str, w: np.ndarray, group: int | None) -> None:
    if group is None:
        out[name] = vlt.Bf16.from_f32(w)
        return
    g = w.shape[1] if group == 0 else group  # 0: one scale per output row
    qs, ss = [], []
    for r0 in range(0, w.shape[0], 8192):
        q, s = vlt.quantize(w[r0:r0 + 8192], g)
        qs.append(q)
        ss.append(s.bits)
    out[name + ".scale"] = vlt.Bf16(np.concatenate(ss))
    out[name] = np.concatenate(qs)


def write_target(path, config: str | dict, seed: int = 0, int8_group: int | None = None, std: float = 0.02) -> dict:
    """int8_group: None keeps bf16; 0 quantises with one scale per output row; n with groups of n."""
    c = CONFIGS[config] if isinstance(config, str) else config
    gen = torch.Generator().manual_seed(seed)
    d, qkv_w = c["d"], (c["n_heads"] + 2 * c["n_kv"]) * c["hd"]
    out: dict = {"meta": meta_tensor(c), "rope_freq": rope_freq(c)}
    embed = _randn(gen, c["vocab"], d, std)
    out["embed"] = vlt.Bf16.from_f32(embed)
    if int8_group is not None:
        _put(out, "head", embed, int8_group)  # tied: the head is the quantised embedding
    del embed
    for i in range(c["n_layers"]):
        L = f"L{i:02d}."
        _put(out, L + "qkv", _randn(gen, qkv_w, d, std), int8_group)
        _put(out, L + "o", _randn(gen, d, c["n_heads"] * c["hd"], std), int8_group)
        _put(out, L + "gate_up", _randn(gen, 2 * c["ffn"], d, std), int8_group)
        _put(out, L + "down", _randn(gen, d, c["ffn"], std), int8_group)
    vlt.write(path, out)
    return c


def write_drafter(path, config: str | dict, seed: int = 100, int8_group: int | None = None, draft_vocab: int | None = None, std: float = 0.02,
                  window: int = 0) -> None:
    """The chain drafter: fc [d][2d] over (tapped hidden ; token embedding), one decoder layer
    `D00.*`, a head over a draft vocabulary of `draft_vocab` ids (`vocab`, ascending target
    ids stored as f32 like the reference's drafter file, tools/spec/export.py:51). With `window`,
    a draft pass attends to the last `window` keys of its context (down to a page boundary), as the
    reference's drafter layers attend to 1024 positions (tools/spec/drafter.py:17); the descriptor
    then has a fifth field."""
    c = CONFIGS[config] if isinstance(config, str) else config
    gen = torch.Generator().manual_seed(seed)
    d, qkv_w = c["d"], (c["n_heads"] + 2 * c["n_kv"]) * c["hd"]
    v = draft_vocab or c["vocab"]
    out: dict = {"meta": np.array([META_VERSION, DRAFTER_KIND_CHAIN, 1, v] + ([window] if window else []), dtype=np.float32)}
    _put(out, "fc", _randn(gen, d, 2 * d, std), int8_group)
    _put(out, "D00.qkv", _randn(gen, qkv_w, d, std), int8_group)
    _put(out, "D00.o", _randn(gen, d, c["n_heads"] * c["hd"], std), int8_group)
    _put(out, "D00.gate_up", _randn(gen, 2 * c["ffn"], d, std), int8_group)
    _put(out, "D00.down", _randn(gen, d, c["ffn"], std), int8_group)
    _put(out, "head", _randn(gen, v, d, std), int8_group)
    ids = np.sort(torch.randperm(c["vocab"], generator=gen)[:v].numpy()) if v < c["vocab"] else np.arange(v)
    out["vocab"] = ids.astype(np.float32)
    vlt.write(path, out)


def lcg_ids(n: int, seed: int, vocab: int) -> np.ndarray:
    """Deterministic pseudo-random token ids: the reference benchmark's generator
    (cli/src/bench.rs:47-56; a 64-bit LCG, `(x >> 33) % vocab`)."""
    mask = (1 << 64) - 1
    a, c = 6364136223846793005, 1442695040888963407
    x = (seed * a + c) & mask
    out = np.empty(n, np.uint32)
    for i in range(n):
        x = (x * a + c) & mask
        out[i] = (x >> 33) % vocab
    return out
