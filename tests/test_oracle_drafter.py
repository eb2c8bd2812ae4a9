"""The oracle's chain drafter on CPU: what it must satisfy by construction. The drafter is an extension
of the benchmark configurations (the reference's drafter is a different model), so nothing pins it from
outside; these are the properties the CUDA path is then held to through the oracle."""
import numpy as np

import oracle
from silicon_violetto_b200 import synth
from tests import util

ROWS = 5
FEED_ROW, LAST = oracle.FEED_ROW, oracle.ROWS_LAST


def _engine(tmp_path):
    d = tmp_path / "drafter.vlt"
    if not d.exists():
        synth.write_drafter(d, util.MICRO, seed=100, draft_vocab=128)
    e = oracle.Engine(util.weights("micro"), max_seqs=2, max_step_tokens=64, max_chunk=32, kv_tokens=512, max_seq_len=256, max_head_rows=16)
    e.load_drafter(d)
    return e


def _committed(e, name, n_pos):
    """Rows of a one-layer pool [page][kv head][16][64] for positions 0..n_pos of slot 0 (pages 0, 1, ... in order)."""
    pool = e.array(name).reshape(-1, util.MICRO["n_kv"], 16, 64)
    return np.stack([pool[p // 16, :, p % 16] for p in range(n_pos)])


def test_drafter_cache_of_committed_positions_does_not_depend_on_how_they_were_verified(tmp_path):
    prompt = np.random.default_rng(4).integers(0, 512, 19).astype(np.uint32)
    # A: verify steps of 5 rows with the drafter's own (mostly wrong) drafts; B: one row at a time.
    a, b = _engine(tmp_path), _engine(tmp_path)
    sa, sb = a.new_seq(), b.new_seq()
    a.step([(sa, prompt, LAST, False)], draft_rows=ROWS)
    b.step([(sb, prompt, LAST, False)], draft_rows=1)
    toks_a, toks_b = [int(a.array("feed")[0])], [int(b.array("feed")[0])]
    for _ in range(6):
        a.step([(sa, [FEED_ROW + i for i in range(ROWS)], LAST, True)], draft_rows=ROWS)
        em = int(a.array("emitted")[0])
        a.settle(sa, ROWS - em)
        toks_a.append(int(a.array("feed")[0]))
    while b.seq_len(sb) < a.seq_len(sa):
        b.step([(sb, [FEED_ROW], LAST, False)], draft_rows=1)
        toks_b.append(int(b.array("feed")[0]))
    n = a.seq_len(sa)
    assert n == b.seq_len(sb) and n >= len(prompt) + 6
    for name in ("draft_k_cache", "draft_v_cache", "k_cache", "v_cache"):
        ka, kb = _committed(a, name, n), _committed(b, name, n)
        assert np.array_equal(ka, kb), name  # the same arithmetic on the same inputs: bit for bit
    assert np.array_equal(a.array("carry")[:util.MICRO["d"]], b.array("carry")[:util.MICRO["d"]])


def test_drafts_are_chain_nodes_from_the_draft_vocabulary_and_rows_of_one_draft_nothing(tmp_path):
    e = _engine(tmp_path)
    s = e.new_seq()
    prompt = np.arange(40, 51, dtype=np.uint32)
    before = e.array("feed").copy()
    e.step([(s, prompt, LAST, False)], draft_rows=1)  # catch-up only
    after = e.array("feed")
    assert np.array_equal(before[1:16], after[1:16])
    e.step([(s, [FEED_ROW], LAST, False)], draft_rows=ROWS)
    from silicon_violetto_b200 import vlt
    ids = set(vlt.read(tmp_path / "drafter.vlt")["vocab"].astype(np.uint32).tolist())
    feed, tree = e.array("feed")[:16], e.array("tree")[:16]
    for i in range(1, ROWS):
        assert int(feed[i]) in ids
        assert tree[i] == (i | ((i - 1) << 8) | (((2 << i) - 1) << 16))  # depth i, parent i - 1, sees rows 0..i
    # Reserving for the draft passes: 8 positions past the step (bounded by max_seq_len).
    assert len(e.array("free_pages")) == 512 // 16 - -(-(e.seq_len(s) + 8) // 16)


def test_a_window_that_covers_the_context_changes_nothing_and_a_shorter_one_starts_on_a_page(tmp_path):
    """meta[4] = window: a pass at position p sees keys from 16 * ((p + 1 - window) // 16) on. With the window past the
    context the draft logits are the full drafter's bit for bit; with a shorter one they equal those of a drafter whose
    cache below the window's start has been overwritten (nothing below it is read)."""
    from silicon_violetto_b200 import vlt
    prompt = np.random.default_rng(9).integers(0, 512, 45).astype(np.uint32)

    def run(window, scribble=False):
        d = tmp_path / f"w{window}.vlt"
        synth.write_drafter(d, util.MICRO, seed=100, draft_vocab=128, window=window)
        assert len(vlt.read(d)["meta"]) == (5 if window else 4)
        e = oracle.Engine(util.weights("micro"), max_seqs=1, max_step_tokens=64, max_chunk=64, kv_tokens=256, max_seq_len=256, max_head_rows=16)
        e.load_drafter(d)
        s = e.new_seq()
        e.step([(s, prompt, LAST, False)], draft_rows=1)
        if scribble:  # positions 0..15 (page 0 of the slot) of the drafter's cache
            junk = np.full(util.MICRO["n_kv"] * 16 * 64, 0x4120, np.uint16)  # bf16 10.0
            page = int(e.array("page_table")[0])
            e.write("draft_k_cache", page * len(junk), junk)
            e.write("draft_v_cache", page * len(junk), junk)
        e.step([(s, [FEED_ROW], LAST, False)], draft_rows=ROWS)
        return e.array("draft_logits").copy()

    full = run(0)
    assert np.array_equal(run(200), full)
    short = run(20)  # passes at positions 45..48: keys from 16 on ((46 - 20) // 16 * 16 .. (49 - 20) // 16 * 16)
    assert not np.array_equal(short, full)
    assert np.array_equal(run(20, scribble=True), short)
    assert not np.array_equal(run(0, scribble=True), full)
