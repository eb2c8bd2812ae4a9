"""The oracle's block drafter against the reference's own Python model (tools/spec/drafter.py): fixtures made by
tests/golden/make_block_drafter_golden.py from the unmodified module, on numpy-seeded weights and inputs that this test
regenerates. What the reference's own check compares (tools/spec/check_engine.py:96-107): the block's logits, by their
largest error over the largest logit, and the draft tree rows."""
import hashlib

import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import synth, vlt

GOLD = np.load(__import__("pathlib").Path(__file__).parent / "golden" / "block_drafter.npz")
EPS, SCALE, TEMP = 2.0 ** -23, 0.1, 0.6  # tools/spec/drafter.py:13-14,18
FREQ = (1.0 / 1024) ** np.linspace(0, 1, 32, dtype=np.float32)  # drafter.py:27-28


@pytest.fixture(scope="module")
def drafter(tmp_path_factory):
    sd = synth.block_drafter_state(0)
    path = tmp_path_factory.mktemp("block") / "drafter.vlt"
    synth.write_block_drafter(path, sd)
    return sd, path


def test_writer_reproduces_the_reference_exporter_byte_for_byte(drafter, tmp_path):
    sd, path = drafter
    assert np.array_equal(np.frombuffer(hashlib.sha256(path.read_bytes()).digest(), np.uint8), GOLD["sha_bf16"])
    q = tmp_path / "int8.vlt"
    synth.write_block_drafter(q, sd, int8=True)
    assert np.array_equal(np.frombuffer(hashlib.sha256(q.read_bytes()).digest(), np.uint8), GOLD["sha_int8"])


def tree_rows(feed, tree, rows):
    """(token, parent, depth, sees) of rows 1.., as check_engine.py:104 reads the engine's feed and tree."""
    return [(int(feed[i]), (int(tree[i]) >> 8) & 0xFF, int(tree[i]) & 0xFF, int(tree[i]) >> 16) for i in range(1, rows)]


@pytest.mark.parametrize("case", range(len(GOLD["cases"])))
def test_block_logits_and_tree_follow_the_python_model(drafter, case):
    sd, path = drafter
    seed, n_ctx, rows = (int(x) for x in GOLD["cases"][case])
    feat, emb = synth.block_case_inputs(seed, n_ctx)
    d = oracle.BlockDrafter(path, EPS, SCALE, FREQ, max_seqs=1, max_chunk=n_ctx + 16)
    assert (d.n_layers, d.n_taps, d.block, d.window, d.v, d.hidden, d.ffn) == (2, 2, 8, 1024, 16384, 1280, 3328)
    meta = np.stack([np.zeros(n_ctx, np.uint32), np.arange(n_ctx, dtype=np.uint32)], axis=1)
    d.context(feat.transpose(1, 0, 2), meta)
    d.run([0], [rows], [n_ctx], vlt.to_bf16(emb)[None])
    logits = d.array("logits").reshape(rows, d.v)
    final = d.array("hfin").reshape(rows, d.hidden) * sd["out_gain"][None]
    # The oracle rounds matmul inputs to bf16 (2^-9 relative per element, averaging out over 1280 to 3328 terms); the
    # reference's own check prints this same ratio for its engine.
    err = float(np.abs(logits[:, GOLD["cols"]] - GOLD[f"logits{case}"]).max() / GOLD[f"max{case}"])
    assert err <= 1e-2, f"logits error {err} of the largest logit"
    ferr = float(np.abs(final - GOLD[f"final{case}"]).max() / np.abs(GOLD[f"final{case}"]).max())
    assert ferr <= 1e-2, f"final hidden states: {ferr}"
    # Trees: where the Python model's candidates are not near-ties, the same rows.
    ncand = min(4, rows - 1)
    tin = np.stack([np.zeros(rows, np.uint32), np.arange(rows, dtype=np.uint32)], axis=1).reshape(-1)
    cand, cand_q = oracle.draft_top(logits, d.array("vocab"), tin, 1.0 / TEMP, ncand)
    feed, tree = np.zeros(16, np.uint32), np.zeros(16, np.uint32)
    oracle.draft_tree([0, rows], tin, cand, cand_q, ncand, feed, tree)
    want = [tuple(int(x) for x in r) for r in GOLD[f"tree{case}"]]
    got = tree_rows(feed, tree, rows)
    same = sum(a == b for a, b in zip(got, want))
    assert same >= len(want) - 1, f"tree rows {got} vs {want}"
    d.close()
