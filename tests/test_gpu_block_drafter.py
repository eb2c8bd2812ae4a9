"""The reference's block drafter on the GPU (k_block.cu, Engine::encode_block_drafter) against the oracle's
(oracle/block_drafter.hpp, itself held to the reference's Python model by tests/test_block_drafter_oracle.py): a target
with the reference's conventions (hidden 1280, epsilon 2^-23, attention scale 0.1, its RoPE frequencies) and a drafter of
the reference's shapes (2 layers, 10 query / 2 kv heads of 128, FFN 3328, four convolutions a layer, window 1024) over
a reduced draft vocabulary."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth, vlt
from tests.test_gpu_parity import STATE, same_state

pytestmark = pytest.mark.gpu
TARGET = dict(n_layers=2, d=1280, n_heads=20, n_kv=5, hd=64, ffn=2560, vocab=4096, eps=2.0 ** -23, theta=10000.0, page=16, attn_scale=0.1,
              rope_freq=(1.0 / 1024) ** np.linspace(0, 1, 32, dtype=np.float32))
DRAFT_V = 2048


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.fixture(scope="module")
def files(tmp_path_factory):
    d = tmp_path_factory.mktemp("blockdrafter")
    synth.write_target(d / "target.vlt", TARGET, seed=3)
    paths = {}
    for window in (1024, 48):
        sd = synth.block_drafter_state(1, hidden=1280, ffn=3328, layers=2, taps=(0, 1), draft_vocab=DRAFT_V, target_vocab=TARGET["vocab"])
        sd["out_gain"] = sd["out_gain"] * 16  # logits up to 10 instead of 0.6: a row's best candidates are then no near-ties
        paths[window] = d / f"drafter_w{window}.vlt"
        # (the exporter's default is int8 in groups of 64, the head in groups of 8: the window-48 file is written that way)
        synth.write_block_drafter(paths[window], sd, window=window, int8=window == 48)
    return d / "target.vlt", paths


def _pair(target, drafter, rows, **kw):
    cfg = dict(max_seqs=4, max_step_tokens=96, max_chunk=64, global_kv_tokens=16 * 64, max_seq_len=256, max_head_rows=32)
    cfg.update(kw)
    prod = E.Engine(target, E.EngineConfig(**cfg))
    orc = oracle.Engine(target, max_seqs=cfg["max_seqs"], max_step_tokens=cfg["max_step_tokens"], max_chunk=cfg["max_chunk"], kv_tokens=cfg["global_kv_tokens"],
                        max_seq_len=cfg["max_seq_len"], max_head_rows=cfg["max_head_rows"])
    prod.load_drafter(drafter)
    orc.load_drafter(drafter)
    assert prod.has_drafter()
    prod.set_draft_rows(rows)
    return prod, orc


def _bf16_err(a_bits, b_bits):
    """The largest difference of two arrays of bf16 bit patterns, as a share of the second one's largest value."""
    a = (a_bits.astype(np.uint32) << 16).view(np.float32)
    b = (b_bits.astype(np.uint32) << 16).view(np.float32)
    return float(np.abs(a - b).max() / np.abs(b).max())


def _step(prod, orc, runs, rows, n_blocks):
    """One step with a block of `rows` rows per run that has head rows. The block's logits within 1e-2 of their largest
    (what the reference's own check measures, tools/spec/check_engine.py:101); the trees must be what the reference's
    candidate kernels make of the product's own logits (those kernels are pinned bit for bit elsewhere), and equal the
    oracle's wherever both saw the same candidates; then the product is put on the oracle's drafts."""
    prod.debug_step(runs, E.StepOptions())
    orc.step(runs, draft_rows=rows)
    nr, n = len(runs), sum(len(r[1]) for r in runs)
    same_state(prod, orc, nr, n, names=[x for x in STATE if x not in ("feed", "tree")])
    want = orc.array("block_logits").reshape(-1, DRAFT_V)
    got = prod.debug_read("block_logits").view(np.float32).reshape(-1, DRAFT_V)
    assert want.shape == got.shape == (n_blocks * rows, DRAFT_V)
    err = float(np.abs(got - want).max() / np.abs(want).max())
    assert err <= 1e-2, f"block logits: {err} of the largest"
    hw, hg = orc.array("block_hfin"), prod.debug_read("block_hfin").view(np.float32)
    assert float(np.abs(hg - hw).max() / np.abs(hw).max()) <= 1e-2
    cw, cg = orc.array("block_ctx_ring"), prod.debug_read("block_ctx_ring").view(np.float32)
    assert float(np.abs(cg - cw).max() / np.abs(cw).max()) <= 1e-2
    # The rings hold the context's K/V and the blocks' own (layer 1's after a whole layer): one bf16 step at the largest
    # value is 2^-8 of it, and a block row's second-layer key inherits the first layer's differences.
    for name in ("block_k_ring", "block_v_ring"):
        e = _bf16_err(prod.debug_read(name).view(np.uint16), orc.array(name))
        assert e <= 2e-2, f"{name}: {e} of the largest"
    feed_p, tree_p = prod.debug_read("feed").reshape(-1, 16), prod.debug_read("tree").reshape(-1, 16)
    feed_o, tree_o = orc.array("feed").reshape(-1, 16), orc.array("tree").reshape(-1, 16)
    slots = [r[0] for r in runs if r[2] != E.Rows.NONE]
    ids = vlt.read(prod._drafter_path)["vocab"].astype(np.uint32)
    ncand = min(4, rows - 1)
    for b, slot in enumerate(slots):
        tin = np.stack([np.full(rows, slot, np.uint32), np.arange(rows, dtype=np.uint32)], axis=1).reshape(-1)
        cand, cand_q = oracle.draft_top(got[b * rows:(b + 1) * rows], ids, tin, 1.0 / 0.6, ncand)
        feed, tree = feed_p.copy().reshape(-1), tree_p.copy().reshape(-1)
        feed[slot * 16 + 1:slot * 16 + 16] = 0
        tree[slot * 16 + 1:slot * 16 + 16] = 0
        oracle.draft_tree([0, rows], tin, cand, cand_q, ncand, feed, tree)
        assert np.array_equal(feed.reshape(-1, 16)[slot][:rows], feed_p[slot][:rows]), f"slot {slot}: tree tokens from the product's logits"
        assert np.array_equal(tree.reshape(-1, 16)[slot][1:rows], tree_p[slot][1:rows]), f"slot {slot}: tree nodes from the product's logits"
        assert feed_p[slot][0] == feed_o[slot][0]
    agree = sum(np.array_equal(feed_p[s][:rows], feed_o[s][:rows]) and np.array_equal(tree_p[s][1:rows], tree_o[s][1:rows]) for s in slots)
    prod.debug_write("feed", 0, feed_o.reshape(-1))
    prod.debug_write("tree", 0, tree_o.reshape(-1))
    return agree, len(slots)


@pytest.mark.parametrize("window,rows", [(1024, 8), (48, 5)])
def test_block_drafter_matches_the_oracle(files, window, rows):
    target, drafters = files
    _run_case(target, drafters[window], rows)


def test_block_drafter_of_another_width(tmp_path):
    """Hidden 768: 6 query heads over the drafter's 2 kv heads (3 a kv head: 24 of the attention's 48 columns at 8 rows a
    block), projections of 6 and 8 row tiles, 96 correction rows in the file's 192."""
    target = dict(TARGET, d=768, n_heads=12, n_kv=3, ffn=1536)
    synth.write_target(tmp_path / "target.vlt", target, seed=4)
    sd = synth.block_drafter_state(2, hidden=768, ffn=1024, layers=2, taps=(0, 1), draft_vocab=DRAFT_V, target_vocab=target["vocab"])
    sd["out_gain"] = sd["out_gain"] * 16
    synth.write_block_drafter(tmp_path / "drafter.vlt", sd, window=1024)
    # (a narrower random drafter has more near-ties among its candidates: 5 of its 11 trees equal the oracle's, where every
    # step's exact checks -- logits, rings, the tree of the product's own logits -- hold)
    _run_case(tmp_path / "target.vlt", tmp_path / "drafter.vlt", 8, min_share=1 / 3)


def _run_case(target, drafter, rows, min_share=0.5):
    prod, orc = _pair(target, drafter, rows)
    prod._drafter_path = drafter
    rng = np.random.default_rng(31)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    pa, pb = rng.integers(0, 4096, 21).astype(np.uint32), rng.integers(0, 4096, 60).astype(np.uint32)
    agree = total = 0
    # Prefill: a in one chunk (a block at once), b in two (its context crosses the steps, no block for the first).
    g, t = _step(prod, orc, [(a, pa, E.Rows.LAST, False), (b, pb[:32], E.Rows.NONE, False)], rows, 1)
    agree, total = agree + g, total + t
    verify = lambda seqs: [(s, [E.FEED_ROW + i for i in range(rows)], E.Rows.LAST, True) for s in seqs]
    g, t = _step(prod, orc, [(b, pb[32:], E.Rows.LAST, False)] + verify([a]), rows, 2)
    agree, total = agree + g, total + t
    for _ in range(4):
        g, t = _step(prod, orc, verify([a, b]), rows, 2)
        agree, total = agree + g, total + t
        for s, e in zip((a, b), orc.array("emitted")[:2]):
            prod.settle(s, rows - int(e))
            orc.settle(s, rows - int(e))
        assert prod.seq_len(a) == orc.seq_len(a) and prod.seq_len(b) == orc.seq_len(b)
    # A tree is grown best-first by products of candidate probabilities; probabilities that differ by a percent (logits within
    # the tolerance) swap neighbours a percent apart, which a random drafter has in every other block. What must hold
    # exactly is asserted per step: the product's tree is the reference kernels' tree of the product's own logits.
    assert agree >= min_share * total, f"only {agree} of {total} trees equal the oracle's"
    prod.close()


def test_generator_with_the_block_drafter_decodes_like_plain_decoding(files):
    """Draft trees of a random drafter are rarely right; whatever they are, the tokens must be the plain decoding's
    (greedy): tree verification, the accepted path and the cache compaction behind a drafter that draws trees."""
    from tests.test_gpu_bench_shapes import _compare_stream, _plain_decode
    target, drafters = files
    rng = np.random.default_rng(6)
    prompts = [rng.integers(0, 4096, n).astype(np.uint32) for n in (11, 40, 17)]
    max_tokens = [24, 16, 12]
    want = [_plain_decode(target, p, mt) for p, mt in zip(prompts, max_tokens)]
    eng = E.Engine(target, E.EngineConfig(max_seqs=3, max_step_tokens=64, max_chunk=32, global_kv_tokens=16 * 24, max_seq_len=128, max_head_rows=24),
                   E.Tuning(spec_policy_off=True))
    eng.load_drafter(drafters[1024])
    with eng.generator() as g:
        ids = [g.submit(E.Request(list(p), mt, draft=[E.Draft.MODEL, E.Draft.MODEL, E.Draft.NONE][i], rows=[8, 4, 1][i])) for i, (p, mt) in enumerate(zip(prompts, max_tokens))]
        got = {i: [] for i in ids}
        for _ in range(400):
            if g.is_idle():
                break
            for ev in g.step():
                if ev.kind == "token":
                    got[ev.req].append(ev.value)
        assert g.is_idle()
    for i, rid in enumerate(ids):
        toks, margins = want[i]
        assert _compare_stream(got[rid], toks, margins) >= 4, f"request {i}"
        assert len(got[rid]) == max_tokens[i]
    assert len(eng.debug_read("free_pages")) == 24
    eng.close()
