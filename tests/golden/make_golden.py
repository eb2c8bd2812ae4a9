"""Generates the golden fixtures of this directory from the reference's own Python tooling.

Run where the reference checkout is available (it is not at test time):

    python tests/golden/make_golden.py /path/to/silicon-violetto

What it records, each produced by unmodified reference code:
  quantize.npz    tools/convert.py `quantize` on seeded matrices (inputs and outputs)
  ref_small.vlt   a weight file written by tools/convert.py `write`
  ref_small.npz   the tensors that went into it, and what `read` gives back
  draft_tree.npz  tools/spec/check_engine.py `draft_tree` (its restatement of the draft_top
                  and draft_tree kernels) on seeded block logits
  rope.npz        tools/spec/drafter.py `rope_tables` / `rope` on a seeded tensor
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def bits(t: torch.Tensor) -> np.ndarray:
    """bf16 tensors as uint16 bit patterns, others as they are."""
    if t.dtype == torch.bfloat16:
        return t.contiguous().view(torch.uint16).numpy().copy()
    return t.contiguous().numpy().copy()


def main(ref: Path) -> None:
    sys.path.insert(0, str(ref / "tools"))
    sys.path.insert(0, str(ref / "tools" / "spec"))
    import check_engine
    import convert
    import drafter

    # --- quantize
    g = torch.Generator().manual_seed(0)
    out = {}
    cases = [(4, 64, 8), (3, 256, 64), (2, 512, 256), (5, 128, 128), (6, 2048, 2048)]
    for i, (m, k, group) in enumerate(cases):
        w = torch.randn(m, k, generator=g) * 0.02
        if i == 0:
            w[1] = 0.0  # an all-zero row: scale 0, q 0
            w[2, :8] = torch.tensor([0.5, -0.5, 1.5, -1.5, 2.5, 127.0, -127.0, 63.5]) * (1.0 / 127)  # ties and the clamp
        if i == 1:
            w = w.to(torch.bfloat16).float()  # bf16-representable inputs, as a converted checkpoint's
        q, s = convert.quantize(w, group)
        out[f"w{i}"], out[f"q{i}"], out[f"s{i}"] = w.numpy(), q.numpy(), bits(s)
        out[f"group{i}"] = np.int64(group)
        out[f"dq{i}"] = convert.dequantize(q, s).numpy()
    np.savez_compressed(HERE / "quantize.npz", **out)

    # --- a weight file
    g = torch.Generator().manual_seed(1)
    w = torch.randn(8, 64, generator=g) * 0.02
    q, s = convert.quantize(w, 16)
    tensors = {
        "meta": torch.tensor([1.0, 0.0, 2.0, 3.5], dtype=torch.float32),
        "embed": (torch.randn(16, 8, generator=g)).to(torch.bfloat16),
        "L00.qkv.scale": s,
        "L00.qkv": q,
        "four_d": torch.arange(2 * 3 * 4 * 5, dtype=torch.float32).reshape(2, 3, 4, 5),
        "a_name_that_is_sixty_three_bytes_long_______________________end": torch.tensor([7.0]),
    }
    convert.write(HERE / "ref_small.vlt", tensors)
    back = convert.read(HERE / "ref_small.vlt")
    rec = {}
    for i, (name, t) in enumerate(tensors.items()):
        rec[f"name{i}"] = np.array(name)
        rec[f"in{i}"] = bits(t)
        rec[f"back{i}"] = bits(back[name])
        rec[f"dtype{i}"] = np.int64(convert.DTYPES[t.dtype])
    np.savez_compressed(HERE / "ref_small.npz", **rec)

    # --- draft tree
    g = torch.Generator().manual_seed(2)
    rec = {}
    for c, (rows, nv) in enumerate([(5, 64), (8, 96), (2, 32), (3, 48)]):
        logits = torch.randn(rows, nv, generator=g) * 3.0
        vocab = torch.randperm(1000, generator=g)[:nv]
        tree = check_engine.draft_tree(logits, vocab)
        rec[f"logits{c}"] = logits.numpy()
        rec[f"vocab{c}"] = vocab.numpy().astype(np.uint32)
        rec[f"tree{c}"] = np.array(tree, dtype=np.int64).reshape(-1, 4)
    rec["temp"] = np.float32(check_engine.TEMP)
    rec["cands"] = np.int64(check_engine.CANDS)
    np.savez_compressed(HERE / "draft_tree.npz", **rec)

    # --- rope
    g = torch.Generator().manual_seed(3)
    freq = convert.rope_frequency()
    pos = torch.tensor([0, 1, 7, 100, 4097, 65535])
    cos, sin = drafter.rope_tables(pos)
    x = torch.randn(len(pos), 2, drafter.D, generator=g)
    y = drafter.rope(x, cos[:, None, :], sin[:, None, :])
    np.savez_compressed(HERE / "rope.npz", freq=freq.numpy(), pos=pos.numpy(), cos=cos.float().numpy(), sin=sin.float().numpy(), x=x.numpy(), y=y.float().numpy())


if __name__ == "__main__":
    main(Path(sys.argv[1]))
