"""Golden outputs of the reference's block drafter (tools/spec/drafter.py) for tests/test_block_drafter_*.py.

Run where the reference checkout is available (it is not at test time):

    python tests/golden/make_block_drafter_golden.py /path/to/silicon-violetto

The weights are `synth.block_drafter_state(0)` (numpy-seeded, bf16-exact, the recipe of check_engine.py's
`random_drafter`) loaded into the unmodified `Drafter`; the inputs are `synth.block_case_inputs`. Recorded per case, all
from reference code: `model(ctx, [0], bonus, [[P]], rows)[0, 0]` (the final normed hidden states times the output gain),
`model.head` of it at 512 fixed columns, each row's four best draft-vocabulary indices, and check_engine.py's
`draft_tree` of the logits. Also the SHA-256 of the file tools/spec/export.py writes for these weights (--bf16 and
int8), which `synth.write_block_drafter` must reproduce byte for byte.
"""
from __future__ import annotations

import hashlib
import subprocess
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parents[1]
CASES = [(11, 37, 8), (12, 1100, 5), (13, 1, 2), (14, 300, 8)]  # (input seed, context positions, block rows)
COLS = np.arange(512) * 32 + 5


def main(ref: Path) -> None:
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import conftest  # noqa: F401  (registers the package)
    from silicon_violetto_b200 import synth
    sys.path.insert(0, str(ref / "tools"))
    sys.path.insert(0, str(ref / "tools" / "spec"))
    import check_engine
    import drafter

    sd = synth.block_drafter_state(0)
    state = {k: torch.from_numpy(np.ascontiguousarray(v)) for k, v in sd.items() if k != "_meta"}
    model = drafter.Drafter(state["vocab"])
    model.load_state_dict(state)
    model.eval()
    out = {"cases": np.array(CASES, np.int64), "cols": COLS}
    with torch.no_grad():
        for i, (seed, n_ctx, rows) in enumerate(CASES):
            feat, emb = synth.block_case_inputs(seed, n_ctx)
            ctx = model.context(torch.from_numpy(feat).bfloat16()[None])
            bonus = drafter.rms(torch.from_numpy(emb)[None, None])
            final = model(ctx, torch.tensor([0]), bonus, torch.tensor([[n_ctx]]), rows)[0, 0]
            logits = model.head(final)
            out[f"final{i}"] = final.numpy()
            out[f"logits{i}"] = logits[:, COLS].numpy()
            out[f"top{i}"] = logits.topk(4, -1).indices.numpy()
            out[f"max{i}"] = np.float32(logits.abs().max().item())
            out[f"tree{i}"] = np.array(check_engine.draft_tree(logits, model.vocab), np.int64)
    with tempfile.TemporaryDirectory() as tmp:
        pt = Path(tmp) / "d.pt"
        torch.save({"state": model.state_dict()}, pt)
        for flag, key in ((["--bf16"], "sha_bf16"), ([], "sha_int8")):
            dst = Path(tmp) / "d.vlt"
            subprocess.run([sys.executable, str(ref / "tools" / "spec" / "export.py"), "--model", str(pt), "--out", str(dst), *flag], check=True)
            out[key] = np.frombuffer(hashlib.sha256(dst.read_bytes()).digest(), np.uint8)
    np.savez_compressed(HERE / "block_drafter.npz", **out)
    print({k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    main(Path(sys.argv[1]))
