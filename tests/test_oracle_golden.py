"""The oracle and the product's numpy weight-file code against fixtures produced by the
reference's own Python tooling (tests/golden/make_golden.py)."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import vlt


def test_quantize_matches_reference(golden):
    z = np.load(golden / "quantize.npz")
    for i in range(5):
        w, group = z[f"w{i}"], int(z[f"group{i}"])
        q, s = oracle.quantize(w, group)
        assert np.array_equal(q, z[f"q{i}"]), f"case {i}: oracle q"
        assert np.array_equal(s, z[f"s{i}"]), f"case {i}: oracle scales"
        q2, s2 = vlt.quantize(w, group)
        assert np.array_equal(q2, z[f"q{i}"]), f"case {i}: numpy q"
        assert np.array_equal(s2.bits, z[f"s{i}"]), f"case {i}: numpy scales"
        assert np.array_equal(vlt.dequantize(q2, s2), z[f"dq{i}"]), f"case {i}: dequantize"


def test_quantize_edge_cases(golden):
    z = np.load(golden / "quantize.npz")
    q, s = z["q0"], z["s0"]
    assert not q[1].any() and not s[1].any()  # an all-zero row
    assert q.min() >= -127 and q.max() <= 127


def _fixture_tensors(golden):
    z = np.load(golden / "ref_small.npz")
    i = 0
    while f"name{i}" in z:
        yield str(z[f"name{i}"]), int(z[f"dtype{i}"]), z[f"in{i}"], z[f"back{i}"]
        i += 1


def test_vlt_read_matches_reference(golden):
    got = oracle.vlt_read(golden / "ref_small.vlt")
    mine = vlt.read(golden / "ref_small.vlt")
    names = []
    for name, dtype, arr, back in _fixture_tensors(golden):
        names.append(name)
        assert np.array_equal(arr, back)
        code, data, offset = got[name]
        assert code == dtype and data.shape == arr.shape and np.array_equal(data, arr)
        assert offset % 256 == 0
        m = mine[name]
        assert np.array_equal(m.bits if isinstance(m, vlt.Bf16) else m, arr)
    assert list(got) == names == list(mine)  # file order kept


def test_vlt_write_is_byte_identical(golden, tmp_path):
    ref = (golden / "ref_small.vlt").read_bytes()
    tensors = {}
    for name, dtype, arr, _ in _fixture_tensors(golden):
        tensors[name] = vlt.Bf16(arr) if dtype == vlt.BF16 else arr
    vlt.write(tmp_path / "a.vlt", tensors)
    assert (tmp_path / "a.vlt").read_bytes() == ref
    oracle.vlt_write(tmp_path / "b.vlt", {n: (d, a) for n, d, a, _ in _fixture_tensors(golden)})
    assert (tmp_path / "b.vlt").read_bytes() == ref


def test_vlt_rejects_bad_files(tmp_path):
    p = tmp_path / "bad.vlt"
    p.write_bytes(b"NOTAVLT!" + bytes(64))
    with pytest.raises(RuntimeError, match="not a version-1"):
        oracle.vlt_read(p)
    with pytest.raises(ValueError):
        vlt.read(p)
    with pytest.raises(RuntimeError, match="cannot open"):
        oracle.vlt_read(tmp_path / "missing.vlt")


def test_rope_matches_reference(golden):
    z = np.load(golden / "rope.npz")
    pos, freq, x, y = z["pos"], z["freq"], z["x"], z["y"]
    rows = x.reshape(-1, x.shape[-1])[:, :64]
    got, cs = oracle.rope(rows, np.repeat(pos, x.shape[1]), freq)
    # cos/sin come from libm here and from torch there: the same but for an occasional last
    # bit before the bf16 rounding, so allow one bf16 step on the table and its effect on y.
    cs = cs.reshape(len(pos), x.shape[1], 32, 2)[:, 0]
    assert np.abs(cs[..., 0] - z["cos"]).max() <= 2.0 ** -8
    assert np.abs(cs[..., 1] - z["sin"]).max() <= 2.0 ** -8
    assert (cs[..., 0] == z["cos"]).mean() > 0.98 and (cs[..., 1] == z["sin"]).mean() > 0.98
    want = y.reshape(-1, y.shape[-1])[:, :64]
    np.testing.assert_allclose(got, want, atol=4e-2, rtol=0)
    same_table = np.repeat((cs[..., 0] == z["cos"]).all(-1) & (cs[..., 1] == z["sin"]).all(-1), x.shape[1])
    np.testing.assert_allclose(got[same_table], want[same_table], atol=1e-6, rtol=1e-6)


def test_draft_tree_matches_reference(golden):
    z = np.load(golden / "draft_tree.npz")
    temp, ncand = float(z["temp"]), int(z["cands"])
    c = 0
    while f"logits{c}" in z:
        logits, vocab, want = z[f"logits{c}"], z[f"vocab{c}"], z[f"tree{c}"]
        rows = logits.shape[0]
        tin = np.stack([np.zeros(rows, np.uint32), np.arange(rows, dtype=np.uint32)], 1).reshape(-1)
        cand, cand_q = oracle.draft_top(logits, vocab, tin, 1.0 / temp, ncand)
        feed = np.zeros(oracle.FEED_W, np.uint32)
        tree = np.zeros(oracle.FEED_W, np.uint32)
        oracle.draft_tree(np.array([0, rows], np.uint32), tin, cand, cand_q, ncand, feed, tree)
        for n, (tok, parent, depth, sees) in enumerate(want, start=1):
            assert feed[n] == tok, (c, n)
            assert tree[n] == (depth | parent << 8 | sees << 16), (c, n)
        for n in range(len(want) + 1, oracle.FEED_W):
            assert tree[n] == oracle.dead_node(n)
        c += 1
    assert c == 4
