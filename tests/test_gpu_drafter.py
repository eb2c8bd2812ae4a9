"""The chain drafter (Draft::Model) against the oracle: its logits within tolerance, the drafts it
writes to feed / tree, the carried taps and every integer of the step state bit for bit; and a
generator run whose tokens must be the plain decoding's whatever the drafter proposes."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth, vlt
from tests import util
from tests.test_gpu_parity import STATE, same_state

pytestmark = pytest.mark.gpu
ROWS = 5
DRAFT_V = 128


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.fixture(scope="module", params=[0, 16], ids=["full", "window16"])
def drafter_file(request, tmp_path_factory):
    """The chain drafter over the whole context, and with a window of one page (the steps below reach 50 positions:
    the passes start at key 0, 16 or 32)."""
    path = tmp_path_factory.mktemp("drafter") / "micro_drafter.vlt"
    synth.write_drafter(path, util.MICRO, seed=100, draft_vocab=DRAFT_V, window=request.param)
    return path


def _pair(drafter_file, **kw):
    cfg = dict(max_seqs=4, max_step_tokens=64, max_chunk=16, global_kv_tokens=16 * 64, max_seq_len=256, max_head_rows=32)
    cfg.update(kw)
    w = util.weights("micro")
    prod = E.Engine(w, E.EngineConfig(**cfg))
    orc = oracle.Engine(w, max_seqs=cfg["max_seqs"], max_step_tokens=cfg["max_step_tokens"], max_chunk=cfg["max_chunk"], kv_tokens=cfg["global_kv_tokens"],
                        max_seq_len=cfg["max_seq_len"], max_head_rows=cfg["max_head_rows"])
    prod.load_drafter(drafter_file)
    orc.load_drafter(drafter_file)
    assert prod.has_drafter()
    prod.set_draft_rows(ROWS)
    return prod, orc, cfg


def _step(prod, orc, runs, cfg, ids):
    """One step on both engines with the drafter. Integer state must agree bit for bit; the drafter's logits
    within the bf16 tolerance; a draft may differ from the oracle's only where the oracle's own margin between
    the two candidates is inside that tolerance (an argmax near-tie) -- the product's feed is then set to the
    oracle's so that the engines stay in step, and that run's later passes are not compared."""
    tol = 2e-2
    prod.debug_step(runs, E.StepOptions())
    orc.step(runs, draft_rows=ROWS)
    nr, n = len(runs), sum(len(r[1]) for r in runs)
    same_state(prod, orc, nr, n, names=[x for x in STATE if x != "feed"])
    want = orc.array("draft_logits").reshape(ROWS - 1, nr, DRAFT_V)
    got = prod.debug_read("draft_logits").view(np.float32).reshape(E.VERIFY_T - 1, cfg["max_seqs"], DRAFT_V)[:ROWS - 1, :nr]
    live = np.abs(want).max(axis=2) > 0  # rows of runs that did not draft stay zero in the oracle
    feed_p, feed_o = prod.debug_read("feed").reshape(-1, 16), orc.array("feed").reshape(-1, 16)
    index_of = {int(t): j for j, t in enumerate(ids)}
    diverged = False
    for r, run in enumerate(runs):
        slot = run[0]
        assert feed_p[slot][0] == feed_o[slot][0]
        for i in range(1, ROWS):
            if not live[i - 1, r]:
                assert feed_p[slot][i] == feed_o[slot][i]
                continue
            err = float(np.abs(got[i - 1, r] - want[i - 1, r]).max())
            assert err <= tol, f"draft logits max-abs error {err} (pass {i}, run {r})"
            if feed_p[slot][i] != feed_o[slot][i]:
                margin = want[i - 1, r][index_of[int(feed_o[slot][i])]] - want[i - 1, r][index_of[int(feed_p[slot][i])]]
                assert 0 <= margin <= 2 * tol, f"draft {feed_p[slot][i]} vs {feed_o[slot][i]} with margin {margin} (pass {i}, run {r})"
                prod.debug_write("feed", slot * 16, feed_o[slot])
                diverged = True
                break
    carry_p = prod.debug_read("carry").view(np.float32)
    assert float(np.abs(carry_p - orc.array("carry")[:len(carry_p)]).max()) <= tol
    if not diverged:
        kp = prod.debug_read("draft_k_cache").view(np.uint16).astype(np.uint32) << 16
        ko = orc.array("draft_k_cache").astype(np.uint32) << 16
        kerr = float(np.abs(kp.view(np.float32) - ko.view(np.float32)[:len(kp)]).max())
        assert kerr <= tol, f"drafter K cache max-abs error {kerr}"
    return live


def test_chain_drafter_matches_the_oracle(drafter_file):
    prod, orc, cfg = _pair(drafter_file)
    ids = vlt.read(drafter_file)["vocab"].astype(np.uint32)
    rng = np.random.default_rng(21)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    pa, pb = rng.integers(0, 512, 13).astype(np.uint32), rng.integers(0, 512, 23).astype(np.uint32)
    # The plain continuation of sequence a, to make some of its drafts right later on.
    o2 = oracle.Engine(util.weights("micro"), max_seqs=1, max_step_tokens=64, max_chunk=40, kv_tokens=256, max_seq_len=256, max_head_rows=8)
    q = o2.new_seq()
    o2.step([(q, pa, E.Rows.LAST, False)])
    cont = []
    for _ in range(12):
        cont.append(int(o2.array("feed")[0]))
        o2.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
    # Prefill: a in one chunk (drafts at once), b in two (the carried tap crosses the steps).
    live = _step(prod, orc, [(a, pa, E.Rows.LAST, False), (b, pb[:16], E.Rows.NONE, False)], cfg, ids)
    assert live[:, 0].all() and not live[:, 1].any()
    runs = lambda seqs: [(s, [E.FEED_ROW + i for i in range(ROWS)], E.Rows.LAST, True) for s in seqs]
    _step(prod, orc, [(b, pb[16:], E.Rows.LAST, False)] + runs([a]), cfg, ids)
    emitted_a = 1
    for it in range(4):
        if it == 1:
            # Two right drafts for a: the next verify step accepts three rows and the catch-up covers all of them.
            fix = np.array(cont[emitted_a:emitted_a + 2], np.uint32)
            prod.debug_write("feed", a * 16 + 1, fix)
            orc.write("feed", a * 16 + 1, fix)
        _step(prod, orc, runs([a, b]), cfg, ids)
        em = orc.array("emitted")[:2]
        if it == 1:
            assert em[0] == 3
        emitted_a += int(em[0])
        for s, e in zip((a, b), em):
            prod.settle(s, ROWS - int(e))
            orc.settle(s, ROWS - int(e))
        assert prod.seq_len(a) == orc.seq_len(a) and prod.seq_len(b) == orc.seq_len(b)


def test_windowed_drafter_over_a_long_context_and_two_key_splits(tmp_path):
    """A window of 64 keys at 150 to 190 positions, the kernel's key split forced to 64 keys per block: the draft passes
    run two splits from the window's page-aligned start. The oracle's draft logits must differ from a full-context
    drafter's (the window is in effect) and the product must follow the windowed ones."""
    ids = None
    logits = {}
    for window in (64, 0):
        path = tmp_path / f"d{window}.vlt"
        synth.write_drafter(path, util.MICRO, seed=100, draft_vocab=DRAFT_V, window=window)
        ids = vlt.read(path)["vocab"].astype(np.uint32)
        cfg = dict(max_seqs=2, max_step_tokens=256, max_chunk=256, global_kv_tokens=16 * 40, max_seq_len=256, max_head_rows=16)
        w = util.weights("micro")
        prod = E.Engine(w, E.EngineConfig(**cfg), E.Tuning(attn_keys_per_cta=64))
        orc = oracle.Engine(w, max_seqs=2, max_step_tokens=256, max_chunk=256, kv_tokens=16 * 40, max_seq_len=256, max_head_rows=16)
        prod.load_drafter(path)
        orc.load_drafter(path)
        prod.set_draft_rows(ROWS)
        rng = np.random.default_rng(77)
        a, b = prod.new_seq(), prod.new_seq()
        assert (orc.new_seq(), orc.new_seq()) == (a, b)
        _step(prod, orc, [(a, rng.integers(0, 512, 150).astype(np.uint32), E.Rows.LAST, False), (b, rng.integers(0, 512, 71).astype(np.uint32), E.Rows.LAST, False)], cfg, ids)
        for _ in range(3):
            _step(prod, orc, [(s, [E.FEED_ROW + i for i in range(ROWS)], E.Rows.LAST, True) for s in (a, b)], cfg, ids)
            for s, e in zip((a, b), orc.array("emitted")[:2]):
                prod.settle(s, ROWS - int(e))
                orc.settle(s, ROWS - int(e))
        logits[window] = orc.array("draft_logits").copy()
    assert np.abs(logits[64] - logits[0]).max() > 1e-3


def test_generator_with_the_model_drafter_decodes_like_plain_decoding(drafter_file):
    w = util.weights("micro")
    rng = np.random.default_rng(5)
    prompts = [rng.integers(0, 512, n).astype(np.uint32) for n in (9, 21, 14)]
    max_tokens = [10, 14, 8]
    want = []
    for p, mt in zip(prompts, max_tokens):
        o = oracle.Engine(w, max_seqs=1, max_step_tokens=64, max_chunk=64, kv_tokens=256, max_seq_len=256, max_head_rows=8)
        q = o.new_seq()
        o.step([(q, p, E.Rows.LAST, False)])
        out = [int(o.array("feed")[0])]
        while len(out) < mt:
            o.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
            out.append(int(o.array("feed")[0]))
        want.append(out)
    eng = E.Engine(w, E.EngineConfig(max_seqs=3, max_step_tokens=48, max_chunk=16, global_kv_tokens=16 * 24, max_seq_len=128, max_head_rows=24),
                   E.Tuning(spec_policy_off=True))
    eng.load_drafter(drafter_file)
    with eng.generator() as g:
        ids = [g.submit(E.Request(list(p), mt, draft=[E.Draft.MODEL, E.Draft.MODEL, E.Draft.NONE][i], rows=[5, 3, 1][i])) for i, (p, mt) in enumerate(zip(prompts, max_tokens))]
        got = {i: [] for i in ids}
        for _ in range(400):
            if g.is_idle():
                break
            for ev in g.step():
                if ev.kind == "token":
                    got[ev.req].append(ev.value)
        assert g.is_idle()
    for i, rid in enumerate(ids):
        assert got[rid] == want[i], f"request {i}"
    assert len(eng.debug_read("free_pages")) == 24
