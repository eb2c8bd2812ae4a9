"""Chunked prefill: prompt chunks of hundreds of rows through the tensor-core GEMM in blocks of 256 tokens and the chunk
attention kernel (rows as the MMA's M side, keys read once per 64 rows), against the oracle: logits, the K/V the chunks
leave in the cache, and every integer of the step state. Steps that mix a prompt chunk with decode and verify runs of
other sequences (continuous batching) take the same kernel."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth, vlt
from tests import util
from tests.test_gpu_bench_shapes import ONE_LAYER_1B, _agree_at_scale, _same_but_feed
from tests.test_gpu_parity import TOL, same_state

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def _caches_agree(prod, orc, tol=2e-2):
    for name in ("k_cache", "v_cache"):
        got = vlt.from_bf16(prod.debug_read(name).view(np.uint16))
        want = vlt.from_bf16(orc.array(name))
        assert got.shape == want.shape, name
        err = float(np.abs(got - want).max())
        assert err <= tol, f"{name}: max-abs {err}"


@pytest.mark.parametrize("name,int8_group", [("micro", None), ("micro4", 0), ("micro", 64)])
def test_prompt_chunks_match_the_oracle(name, int8_group):
    w = util.weights(name, int8_group)
    kw = dict(max_seqs=3, max_step_tokens=320, max_chunk=300, max_seq_len=640, max_head_rows=64)
    prod = E.Engine(w, E.EngineConfig(global_kv_tokens=3 * 640, **kw))
    orc = oracle.Engine(w, kv_tokens=3 * 640, **kw)
    seqs = [prod.new_seq() for _ in range(3)]
    assert [orc.new_seq() for _ in range(3)] == seqs
    vocab = prod.desc.vocab
    rng = np.random.default_rng(12)
    tol = TOL[int8_group]
    prompt = rng.integers(0, vocab, 600).astype(np.uint32)

    def step(runs, n_runs, n):
        out = prod.debug_step(runs, E.StepOptions(read_logits=True))
        orc.step(runs)
        want = orc.array("logits").reshape(-1, vocab)
        err = float(np.abs(out.logits - want).max()) if want.size else 0.0
        assert err <= tol, f"logits max-abs error {err}"
        same_state(prod, orc, n_runs, n)
        return err

    # A 300-row chunk (two GEMM blocks: 256 + 44 tokens; five chunk tiles), every 37th-ish row through the head via a second run.
    e1 = step([(seqs[0], prompt[:300], E.Rows.LAST, False), (seqs[1], prompt[300:317], E.Rows.ALL, False)], 2, 317)
    # Then a step that mixes: the next chunk of sequence 0 (attends 300 cached keys + itself), a one-token decode run of
    # sequence 1, and a verify run of sequence 2 over a small draft tree after its own short prefill.
    step([(seqs[2], prompt[400:409], E.Rows.LAST, False)], 1, 9)
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    tree = [oracle.chain_node(0), node(1, 0, 0b0011), node(1, 0, 0b0101), node(2, 2, 0b1101)]
    feed = [int(orc.array("feed")[seqs[2] * 16])] + [int(x) for x in rng.integers(0, vocab, 3)]
    for e, wr in ((prod, prod.debug_write), (orc, orc.write)):
        wr("feed", seqs[2] * 16, feed)
        wr("tree", seqs[2] * 16, tree)
    e2 = step([(seqs[0], prompt[300:480], E.Rows.LAST, False), (seqs[1], [E.FEED_ROW], E.Rows.LAST, False),
               (seqs[2], [E.FEED_ROW + i for i in range(4)], E.Rows.LAST, True)], 3, 185)
    _caches_agree(prod, orc)
    print(f"{name} int8_group={int8_group}: logits error {e1:.2e} (300-row chunk) {e2:.2e} (chunk + decode + verify)")
    prod.close()


def test_a_computed_context_at_the_1b_dimensions_matches_the_oracle(tmp_path):
    """One layer at d 2048 / 32 q, 8 kv heads / FFN 8192 / 128 256 ids (int8): an 8192-token context computed in sixteen
    chunks of 512 (two GEMM blocks and eight chunk tiles a step), then a verify-shaped step of 5 rows over it -- the
    benchmark's context length with K/V that were computed, not filled."""
    path = tmp_path / "one_layer_1b.vlt"
    synth.write_target(path, ONE_LAYER_1B, seed=0, int8_group=0)
    kw = dict(max_seqs=2, max_step_tokens=512, max_chunk=512, max_seq_len=8256, max_head_rows=16)
    prod = E.Engine(path, E.EngineConfig(global_kv_tokens=2 * 8256, **kw))
    orc = oracle.Engine(path, kv_tokens=2 * 8256, **kw)
    a = prod.new_seq()
    assert orc.new_seq() == a
    vocab = prod.desc.vocab
    rng = np.random.default_rng(2)
    prompt = rng.integers(0, vocab, 8192).astype(np.uint32)
    errs = []
    for lo in range(0, 8192, 512):
        errs.append(_agree_at_scale(prod, orc, [(a, prompt[lo:lo + 512], E.Rows.LAST, False)], TOL[0]))
        _same_but_feed(prod, orc, 1, 512)
    k_got = vlt.from_bf16(prod.debug_read("k_cache").view(np.uint16))
    assert float(np.abs(k_got - vlt.from_bf16(orc.array("k_cache"))).max()) <= 5e-2
    errs.append(_agree_at_scale(prod, orc, [(a, rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False)], TOL[0]))
    print("1B dims, computed 8192-token context: logits error per step", [f"{e[0]:.2e}" for e in errs])
    prod.close()
