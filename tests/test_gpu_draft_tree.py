"""The reference drafter's candidate kernels on the GPU (`draft_top`, `draft_tree`): against the golden
vectors produced by the reference's own Python (`tools/spec/check_engine.py draft_tree`, see
tests/golden/make_golden.py) -- the one place where a CUDA kernel's parity is pinned to the reference
itself -- and bit for bit against the oracle on random logits, several blocks and slots at once."""
from pathlib import Path

import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E
from tests import util

pytestmark = pytest.mark.gpu
GOLDEN = Path(__file__).resolve().parent / "golden"


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.fixture(scope="module")
def eng():
    return E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=4, max_step_tokens=64, max_chunk=16, global_kv_tokens=256, max_seq_len=64, max_head_rows=16))


def test_draft_tree_matches_the_reference_vectors(eng):
    z = np.load(GOLDEN / "draft_tree.npz")
    temp, ncand = float(z["temp"]), int(z["cands"])
    c = 0
    while f"logits{c}" in z:
        logits, vocab, want = z[f"logits{c}"], z[f"vocab{c}"], z[f"tree{c}"]
        rows = logits.shape[0]
        _, _, feed, tree = eng.draft_trees(logits, vocab, [0, rows], [c % 4], 1.0 / temp, ncand)
        feed, tree = feed[c % 4], tree[c % 4]
        for n, (tok, parent, depth, sees) in enumerate(want, start=1):
            assert feed[n] == tok, (c, n)
            assert tree[n] == (depth | parent << 8 | sees << 16), (c, n)
        for n in range(len(want) + 1, 16):
            assert tree[n] == oracle.dead_node(n)
        c += 1
    assert c == 4


@pytest.mark.parametrize("nv,ncand,temp", [(1000, 4, 1.0), (16384, 3, 0.7), (257, 1, 2.0)])
def test_draft_top_and_tree_are_bit_exact_against_the_oracle(eng, nv, ncand, temp):
    rng = np.random.default_rng(nv)
    blocks = [(0, 8), (8, 5), (13, 2), (15, 7)]  # (first row, rows) of four slots
    rows = 22
    logits = (rng.standard_normal((rows, nv)) * 2.5).astype(np.float32)
    logits[3, 10] = logits[3, 900 % nv] = logits[3].max() + 1.0  # an exact tie for the best entry: the lowest index wins
    ids = np.sort(rng.choice(200000, nv, replace=False)).astype(np.uint32)
    tin = np.zeros(2 * rows, np.uint32)
    for s, (first, n) in enumerate(blocks):
        tin[2 * first:2 * (first + n):2] = s
        tin[2 * first + 1:2 * (first + n) + 1:2] = np.arange(n)
    cand_o, q_o = oracle.draft_top(logits, ids, tin, 1.0 / temp, ncand)
    feed_o, tree_o = np.zeros(4 * 16, np.uint32), np.zeros(4 * 16, np.uint32)
    oracle.draft_tree(np.array(blocks, np.uint32).reshape(-1), tin, cand_o, q_o, ncand, feed_o, tree_o)
    cand, q, feed, tree = eng.draft_trees(logits, ids, np.array(blocks, np.uint32).reshape(-1), [0, 1, 2, 3], 1.0 / temp, ncand, tin=tin)
    assert np.array_equal(cand[:, :ncand], np.asarray(cand_o).reshape(rows, 4)[:, :ncand])
    assert np.array_equal(q[:, :ncand].view(np.uint32), np.asarray(q_o, np.float32).reshape(rows, 4)[:, :ncand].view(np.uint32))  # the same bits
    assert cand[3, 0] == ids[min(10, 900 % nv)] and (cand[0] == 0).all()  # row 0 of a block is skipped
    for s, (first, n) in enumerate(blocks):
        assert np.array_equal(feed[s][1:n], feed_o.reshape(4, 16)[s][1:n]), s
        assert np.array_equal(tree[s][1:], tree_o.reshape(4, 16)[s][1:]), s
