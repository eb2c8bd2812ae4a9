"""The oracle's restatement of the reference's own architecture (oracle/limite.hpp, limite_forward.hpp) on CPU. Nothing
pins it from outside (the reference's target has no Python definition in its tree), so these are the properties it must
have by construction; the CUDA path is then held to it in tests/test_gpu_limite.py."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import synth, vlt

LAST, ALL, NONE, FEED_ROW = oracle.ROWS_LAST, oracle.ROWS_ALL, oracle.ROWS_NONE, oracle.FEED_ROW
KW = dict(max_seqs=2, max_step_tokens=64, max_chunk=32, kv_tokens=128 * 12, max_seq_len=1400, max_head_rows=64)


@pytest.fixture(scope="module")
def model(tmp_path_factory):
    path = tmp_path_factory.mktemp("limite") / "limite.vlt"
    desc = synth.write_limite(path, n_layers=48, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630, seed=1)
    return path, desc


def test_descriptor_comes_from_the_files_shapes(model):
    path, desc = model
    o = oracle.Engine(path, **KW)
    assert o.desc == dict(n_layers=48, d=256, n_heads=2, n_kv=1, hd=128, ffn=512, vocab=640, vocab_real=630, page=128)
    names = set(vlt.read(path))
    assert "meta" not in names and {"embed", "value_embed", "rope_freq", "mudd.dense1", "mudd.mix", "L00.scalars", "L01.ve_gate", "L47.xsa"} <= names
    assert "L00.ve_gate" not in names and "L04.ve_gate" in names  # layers with i % 3 == 1 (tools/convert.py:13)


def test_logits_are_capped_and_do_not_depend_on_how_the_prompt_was_chunked(model):
    path, _ = model
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 630, 45).astype(np.uint32)
    a, b = oracle.Engine(path, **KW), oracle.Engine(path, **KW)
    sa, sb = a.new_seq(), b.new_seq()
    a.step([(sa, prompt[:32], ALL, False)])
    rows = [a.array("logits").reshape(32, -1).copy()]
    a.step([(sa, prompt[32:], ALL, False)])
    rows.append(a.array("logits").reshape(13, -1).copy())
    whole = np.concatenate(rows)
    assert whole[:, :630].min() > 0 and whole[:, :630].max() < 23 and np.isneginf(whole[:, 630:]).all()  # kernels.metal:196-199
    one = []
    for t in prompt:
        b.step([(sb, [t], ALL, False)])
        one.append(b.array("logits").reshape(1, -1)[0].copy())
    # The same arithmetic on the same inputs, whatever the step's layout: bit for bit.
    assert np.array_equal(np.stack(one)[:, :630], whole[:, :630])
    assert np.array_equal(a.array("limite_k_local"), b.array("limite_k_local")) and np.array_equal(a.array("k_cache"), b.array("k_cache"))


def test_local_layers_forget_what_is_behind_their_window_and_global_ones_do_not(model):
    """1 100 positions, then one more token: the ring of a local layer holds window + max_chunk positions and a query
    reads the last 1 024 of them; position 0's key is still in a global layer's pages."""
    path, _ = model
    o = oracle.Engine(path, **KW)
    s = o.new_seq()
    rng = np.random.default_rng(3)
    toks = rng.integers(0, 630, 1100).astype(np.uint32)
    for i in range(0, 1100, 32):
        o.step([(s, toks[i:i + 32], NONE, False)])
    assert o.seq_len(s) == 1100
    ring = 1024 + 32
    k_local = o.array("limite_k_local").reshape(36, 2, 1, ring, 128)  # [local layer][slot][kv head][ring][128]
    assert np.any(k_local[0, 0, 0, 1099 % ring]) and np.any(k_local[0, 0, 0, (1099 - 1055) % ring])
    pages = o.array("page_table")[:9]
    assert list(pages) == list(range(9))  # 1 100 positions in pages of 128, popped 0, 1, 2, ...
    o.step([(s, [7], LAST, False)])
    assert o.seq_len(s) == 1101 and 0 <= int(o.array("feed")[0]) < 630
