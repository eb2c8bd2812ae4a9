"""CPU-side checks of the product library: it loads, exports every declared symbol, fails
loudly without a GPU, and its planner and page allocator agree with the oracle bit for bit."""
import re
from pathlib import Path

import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E
from tests import util

ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def test_every_declared_symbol_is_exported():
    header = (ROOT / "include" / "violetto.h").read_text()
    names = re.findall(r"\b(vlt_[a-z0-9_]+)\s*\(", header)
    assert len(set(names)) >= 30
    lib = E.lib()
    for n in set(names):
        assert hasattr(lib, n), f"{n} is declared in include/violetto.h but not exported"


def test_header_cites_the_reference_for_every_entry_point():
    header = (ROOT / "include" / "violetto.h").read_text()
    assert header.count(".rs:") >= 25


@pytest.mark.skipif(util.cuda_available(), reason="checks the no-GPU failure mode")
def test_engine_without_a_gpu_fails_loudly():
    with pytest.raises(E.EngineError, match="no usable CUDA device.*no CPU path"):
        E.Engine(util.weights("micro"))


def test_host_only_engine_refuses_to_run():
    eng = E.Engine(util.weights("micro"), E.EngineConfig(host_only=True, max_seq_len=256, global_kv_tokens=256))
    s = eng.new_seq()
    with pytest.raises(E.EngineError, match="host-only"):
        eng.step([E.Run(s, [1, 2, 3])])
    assert eng.device_name().startswith("host")


def test_bad_weight_files_are_rejected(tmp_path):
    p = tmp_path / "x.vlt"
    p.write_bytes(b"nope" * 100)
    with pytest.raises(E.EngineError, match="not a version-1 violetto weight file"):
        E.Engine(p, E.EngineConfig(host_only=True))
    with pytest.raises(E.EngineError, match="cannot open"):
        E.Engine(tmp_path / "missing.vlt", E.EngineConfig(host_only=True))


def _pair(**kw):
    cfg = dict(max_seqs=4, max_step_tokens=64, max_chunk=24, global_kv_tokens=16 * 40, max_seq_len=400, max_head_rows=32)
    cfg.update(kw)
    w = util.weights("micro")
    prod = E.Engine(w, E.EngineConfig(host_only=True, **cfg))
    orc = oracle.Engine(w, max_seqs=cfg["max_seqs"], max_step_tokens=cfg["max_step_tokens"], max_chunk=cfg["max_chunk"], kv_tokens=cfg["global_kv_tokens"],
                        max_seq_len=cfg["max_seq_len"], max_head_rows=cfg["max_head_rows"])
    return prod, orc


PLAN_ARRAYS = ["tokens", "tin", "vis", "head_rows", "hidden_rows", "sample_rows", "runs", "tiles", "page_table", "free_pages", "lens"]


def _same_plan(prod, orc, n_head, n_runs):
    for name in PLAN_ARRAYS:
        a, b = prod.debug_read(name), orc.array(name)
        if name in ("head_rows", "hidden_rows", "sample_rows", "runs", "tiles"):
            assert len(a) >= len(b)
            a = a[:len(b)]  # the product returns the whole fixed-size array
        assert np.array_equal(a, b), name


def test_plan_and_page_allocator_match_the_oracle():
    prod, orc = _pair()
    rng = np.random.default_rng(0)
    seqs = []
    for step in range(40):
        # Sequences come and go; runs mix prompt chunks, one-token decodes and verify runs of GPU-fed rows.
        if len(seqs) < 4 and rng.random() < 0.5:
            a, b = prod.new_seq(), orc.new_seq()
            assert a == b
            t, p, sd = float(rng.choice([0.0, 0.6])), float(rng.choice([1.0, 0.95])), int(rng.integers(1 << 40))
            prod.set_sampling(a, E.Sampling(t, p, sd))
            orc.set_sampling(b, t, p, sd)
            seqs.append(a)
        if seqs and rng.random() < 0.15:
            s = seqs.pop(int(rng.integers(len(seqs))))
            prod.free_seq(s)
            orc.free_seq(s)
        if not seqs:
            continue
        runs = []
        for s in seqs:
            if rng.random() < 0.3:
                continue
            kind = rng.integers(3)
            if kind == 0:
                toks, head, verify = list(rng.integers(0, 512, int(rng.integers(1, 20)))), int(rng.integers(3)), False
            elif kind == 1:
                toks, head, verify = [E.FEED_ROW], E.Rows.LAST, False
            else:
                toks, head, verify = [E.FEED_ROW + i for i in range(int(rng.integers(2, 9)))], E.Rows.LAST, True
            if prod.seq_len(s) + len(toks) > 390:
                continue
            runs.append((s, toks, head, verify))
        if not runs or sum(len(r[1]) for r in runs) > 64:
            continue
        hidden = int(rng.integers(3))
        try:
            orc.step(runs, hidden=hidden, plan_only=True)
            err = None
        except RuntimeError as e:
            err = str(e)
        if err is None:
            prod.debug_plan(runs, hidden)
            n_head = sum(len(r[1]) if r[3] or r[2] == 2 else (1 if r[2] == 1 else 0) for r in runs)
            _same_plan(prod, orc, n_head, len(runs))
            for s in seqs:
                assert prod.seq_len(s) == orc.seq_len(s)
            # The collect step's correction of verify runs.
            for s, toks, _, verify in runs:
                if verify and rng.random() < 0.7:
                    unused = int(rng.integers(0, len(toks)))
                    prod.settle(s, unused)
                    orc.settle(s, unused)
        else:
            with pytest.raises(E.EngineError) as got:
                prod.debug_plan(runs, hidden)
            assert str(got.value) == err


def test_plan_errors_match_the_oracle_and_the_reference_messages():
    prod, orc = _pair()
    a, b = prod.new_seq(), orc.new_seq()
    cases = [
        ([], "step has 0 tokens (max 64)"),
        ([(a, list(range(25)), 1, False)], "25 tokens for one sequence in a step (max_chunk 24)"),
        ([(a, [E.FEED_ROW + 16], 1, False)], "only 16 GPU-fed tokens per slot"),
        ([(a, [1], 1, False), (a, [2], 1, False)], "a sequence appears twice in one step"),
        ([(3, [1], 1, False)], "unknown sequence"),
    ]
    for runs, msg in cases:
        with pytest.raises(E.EngineError, match=re.escape(msg)):
            prod.debug_plan(runs)
        with pytest.raises(RuntimeError, match=re.escape(msg)):
            orc.step(runs, plan_only=True)
    # Too many head rows.
    with pytest.raises(E.EngineError, match=r"head rows \(max 32\)"):
        s2 = prod.new_seq()
        prod.debug_plan([(a, list(range(20)), 2, False), (s2, list(range(20)), 2, False)])


def test_pool_exhaustion_and_sequence_limit():
    prod, orc = _pair(global_kv_tokens=64, max_seq_len=100)
    a, b = prod.new_seq(), orc.new_seq()
    prod.bench_fill(a, 60)
    orc.bench_fill(b, 60)
    for e, exc in ((prod, E.EngineError), (orc, RuntimeError)):
        with pytest.raises(exc, match="global KV pool exhausted"):
            (e.debug_plan if e is prod else lambda r: e.step(r, plan_only=True))([(a, list(range(10)), 1, False)])
    prod2, orc2 = _pair(global_kv_tokens=640, max_seq_len=100)
    a, b = prod2.new_seq(), orc2.new_seq()
    prod2.bench_fill(a, 95)
    orc2.bench_fill(b, 95)
    with pytest.raises(E.EngineError, match=r"sequence would reach 105 tokens \(max 100\)"):
        prod2.debug_plan([(a, list(range(10)), 1, False)])
    with pytest.raises(RuntimeError, match=r"sequence would reach 105 tokens \(max 100\)"):
        orc2.step([(b, list(range(10)), 1, False)], plan_only=True)


def test_pages_come_back_in_their_original_order():
    prod, orc = _pair()
    a = prod.new_seq()
    prod.bench_fill(a, 50)  # pages 0..3
    b = prod.new_seq()
    prod.bench_fill(b, 20)  # pages 4, 5
    pt = prod.debug_read("page_table").reshape(4, -1)
    assert list(pt[a][:4]) == [0, 1, 2, 3] and list(pt[b][:2]) == [4, 5]
    prod.free_seq(a)
    c = prod.new_seq()
    assert c == a
    prod.bench_fill(c, 40)
    assert list(prod.debug_read("page_table").reshape(4, -1)[c][:3]) == [0, 1, 2]  # kv.rs:60-62
    assert prod.debug_read("lens")[c] == 40


def test_sampling_is_checked():
    prod, _ = _pair()
    s = prod.new_seq()
    for bad in (E.Sampling(-1.0, 1.0, 0), E.Sampling(0.5, 0.0, 0), E.Sampling(0.5, 1.5, 0), E.Sampling(float("nan"), 1.0, 0)):
        with pytest.raises(E.EngineError, match="needs a temperature of 0 or a normal positive one"):
            prod.set_sampling(s, bad)
    prod.set_sampling(s, E.Sampling(0.6, 0.95, 7))


def test_inputs_that_would_overrun_device_arrays_are_refused_on_the_host():
    """A verify run longer than one attention tile, more stop tokens than a slot's state holds, a slot past the
    table: refused before any kernel could index out of its arrays."""
    eng = E.Engine(util.weights("micro"), E.EngineConfig(host_only=True, max_seqs=2, max_step_tokens=64, max_chunk=32, max_seq_len=256, global_kv_tokens=256))
    s = eng.new_seq()
    with pytest.raises(E.EngineError, match="a verify run takes at most 8 rows"):
        eng.debug_plan([(s, [E.FEED_ROW + i for i in range(9)], E.Rows.LAST, True)])
    eng.debug_plan([(s, list(range(9)), E.Rows.LAST, False)])  # a plain run of the same length is fine
    with pytest.raises(E.EngineError, match="9 stop tokens"):
        eng.set_gen(s, 5, stop=list(range(9)))
    with pytest.raises(E.EngineError, match="slot out of range"):
        eng.set_gen(7, 5)
    eng.set_gen(s, 5, stop=list(range(8)))


def test_a_failed_page_reservation_changes_nothing():
    """A step that does not fit the pool fails as a whole: the pages it had taken go back, in order."""
    eng = E.Engine(util.weights("micro"), E.EngineConfig(host_only=True, max_seqs=2, max_step_tokens=64, max_chunk=64, max_seq_len=256, global_kv_tokens=48))
    s = eng.new_seq()
    before = eng.debug_read("free_pages").copy()
    with pytest.raises(E.EngineError, match="global KV pool exhausted"):
        eng.debug_plan([(s, list(range(50)), E.Rows.LAST, False)])
    assert np.array_equal(eng.debug_read("free_pages"), before)


def test_admission_budgets_the_drafters_reach(tmp_path):
    """With a drafter loaded a step reserves pages 8 positions past itself; submit() budgets the pool for that reach,
    so a request the pool holds only without the margin is refused up front instead of failing inside a step."""
    from silicon_violetto_b200 import synth
    d = tmp_path / "drafter.vlt"
    synth.write_drafter(d, util.MICRO, seed=100, draft_vocab=64)
    # 20 prompt tokens + 13 new ones reach 32 positions: exactly two pages.
    cfg = E.EngineConfig(host_only=True, max_seqs=2, max_step_tokens=64, max_chunk=32, max_seq_len=256, global_kv_tokens=32, max_head_rows=8)
    plain = E.Engine(util.weights("micro"), cfg)
    with plain.generator() as g:
        g.submit(E.Request(list(range(20)), 13))
    drafted = E.Engine(util.weights("micro"), cfg)
    drafted.load_drafter(d)
    assert drafted.has_drafter()
    with drafted.generator() as g:
        with pytest.raises(E.EngineError, match="doesn't fit max_seq_len or the KV pool"):
            g.submit(E.Request(list(range(20)), 13))
        g.submit(E.Request(list(range(20)), 5))  # reaches 24 + 8 = 32 positions: fits
