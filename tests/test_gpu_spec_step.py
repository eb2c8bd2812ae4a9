"""The rejection-sampling rule inside the engine's step (vlt_set_acceptance(VLT_ACCEPT_REJECTION)): the chain drafter
draws its drafts from softmax(q / T) and keeps the q rows, the next verify step accepts draft i with probability
min(1, P / Q), replaces the first rejected one by a draw from max(0, P - Q), and commits through `accept`'s state.

The rule has no counterpart in the reference; the oracle defines it (oracle/sampling.hpp: spec_step_run). Given
identical logits and draws every integer of the step must be the oracle's: the product's step is fed the oracle's
target and draft logits (vlt_debug_force_logits), so that the decision kernels see the same bits, and its own logits
are compared with the oracle's within the bf16 tolerance beforehand."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth
from tests import util
from tests.test_gpu_parity import STATE, same_state

pytestmark = pytest.mark.gpu
ROWS = 5
DRAFT_V = 96


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.fixture(scope="module")
def drafter_file(tmp_path_factory):
    path = tmp_path_factory.mktemp("drafter") / "micro_drafter.vlt"
    synth.write_drafter(path, util.MICRO, seed=100, draft_vocab=DRAFT_V)
    return path


def _pair(drafter_file):
    cfg = dict(max_seqs=4, max_step_tokens=64, max_chunk=24, global_kv_tokens=16 * 64, max_seq_len=256, max_head_rows=32)
    w = util.weights("micro")
    prod = E.Engine(w, E.EngineConfig(**cfg))
    okw = dict(cfg)
    okw["kv_tokens"] = okw.pop("global_kv_tokens")
    orc = oracle.Engine(w, **okw)
    for e in (prod, orc):
        e.load_drafter(drafter_file)
        e.set_acceptance(1)
    prod.set_draft_rows(ROWS)
    return prod, orc


def _step(prod, orc, runs):
    """The oracle's step first; then the product's, its tail fed the oracle's logits. Everything integer must agree."""
    orc.step(runs, draft_rows=ROWS)
    nr, n = len(runs), sum(len(r[1]) for r in runs)
    prod.force_logits(orc.array("logits"), orc.array("draft_logits"))
    prod.debug_step(runs, E.StepOptions())
    same_state(prod, orc, nr, n)
    assert np.array_equal(prod.debug_read("q_rows"), orc.array("q_rows")), "q_rows"
    e = orc.array("emitted")[:nr]
    got, want = prod.debug_read("out_ids"), orc.array("out_ids")
    ru = orc.array("runs").reshape(-1, 6)
    for r in range(nr):
        h0 = ru[r][3]
        assert np.array_equal(got[h0:h0 + e[r]], want[h0:h0 + e[r]]), f"emitted tokens of run {r}"
    return e


def test_rejection_rule_in_the_step_is_bit_exact_given_the_oracles_logits(drafter_file):
    prod, orc = _pair(drafter_file)
    rng = np.random.default_rng(8)
    seqs = [prod.new_seq() for _ in range(4)]
    assert [orc.new_seq() for _ in range(4)] == seqs
    # Three sampling sequences (the rule applies), one of them hot enough that drafts pass often, and a greedy one plus a
    # top-p one (the rule does not fit: the reference's sample-then-match decides them in the same step).
    samplings = [(0.8, 1.0, 11), (3.0, 1.0, 12), (0.0, 1.0, 13), (0.7, 0.9, 14)]
    for s, (t, tp, seed) in zip(seqs, samplings):
        prod.set_sampling(s, E.Sampling(t, tp, seed))
        orc.set_sampling(s, t, tp, seed)
    prompts = [rng.integers(0, 512, n).astype(np.uint32) for n in (9, 17, 5, 12)]
    _step(prod, orc, [(s, p, E.Rows.LAST, False) for s, p in zip(seqs, prompts)])
    assert list(orc.array("q_rows")) == [ROWS - 1, ROWS - 1, 0, 0]
    accepted = np.zeros(4, int)
    verify = lambda ss: [(s, [E.FEED_ROW + i for i in range(ROWS)], E.Rows.LAST, True) for s in ss]
    for it in range(10):
        e = _step(prod, orc, verify(seqs))
        accepted += e
        for s, k in zip(seqs, e):
            prod.settle(s, ROWS - int(k))
            orc.settle(s, ROWS - int(k))
        assert all(prod.seq_len(s) == orc.seq_len(s) for s in seqs)
    print("tokens emitted over 10 verify steps per sequence:", accepted)
    assert accepted[1] > 10  # the hot sequence's drafts (its own distribution is nearly the target's at T = 3: both flat) pass often
    # A shorter verify run than the kept rows, and a run with no kept rows after a step without the drafter.
    prod.set_draft_rows(0)
    orc.step(verify(seqs[:2]), draft_rows=0)
    prod.force_logits(orc.array("logits"))
    prod.debug_step(verify(seqs[:2]), E.StepOptions())
    same_state(prod, orc, 2, 2 * ROWS)
    assert list(orc.array("q_rows")[:2]) == [0, 0]


def test_generator_under_the_rejection_rule_runs_and_frees_everything(drafter_file):
    """End to end through the generator: sampling requests with Draft::Model under the rule finish with their token
    budgets, the same seeds give the same tokens again, and all pages come back."""
    w = util.weights("micro")
    outs = []
    for _ in range(2):
        eng = E.Engine(w, E.EngineConfig(max_seqs=3, max_step_tokens=48, max_chunk=16, global_kv_tokens=16 * 30, max_seq_len=160, max_head_rows=24), E.Tuning(spec_policy_off=True))
        eng.load_drafter(drafter_file)
        eng.set_acceptance(1)
        rng = np.random.default_rng(3)
        got = {}
        with eng.generator() as g:
            ids = [g.submit(E.Request(list(rng.integers(0, 512, n)), mt, sampling=E.Sampling(t, 1.0, 40 + i), draft=E.Draft.MODEL, rows=5))
                   for i, (n, mt, t) in enumerate([(9, 30, 0.8), (21, 24, 2.0), (14, 17, 0.0)])]
            got = {i: [] for i in ids}
            for _ in range(400):
                if g.is_idle():
                    break
                for ev in g.step():
                    if ev.kind == "token":
                        got[ev.req].append(ev.value)
            assert g.is_idle()
        assert [len(got[i]) for i in ids] == [30, 24, 17]
        assert len(eng.debug_read("free_pages")) == 30
        outs.append(got)
        eng.close()
    assert outs[0] == outs[1]
