"""The rejection-sampling acceptance kernel against the oracle: accepted lengths, replacement / bonus
tokens and rollback offsets, bit for bit (the benchmark's single-kernel configuration: 32 streams, k = 4,
vocabulary 128256, bf16 logits drawn N(0, 3^2), temperature 1)."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, vlt
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def _case(streams, k, vocab, seed, temperature, peaked=0.0):
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal((streams, k + 1, vocab)) * 3.0).astype(np.float32)
    q = (rng.standard_normal((streams, k, vocab)) * 3.0).astype(np.float32)
    if peaked:
        # Correlated draft and target rows, so that several drafts get accepted.
        q = (p[:, :k] * peaked + q * (1.0 - peaked)).astype(np.float32)
    pb, qb = vlt.to_bf16(p), vlt.to_bf16(q)
    seeds = (np.arange(streams, dtype=np.uint64) * np.uint64(7919) + np.uint64(2))
    pos0 = rng.integers(1, 9000, streams).astype(np.uint32)
    drafts = oracle.draw_drafts(qb, temperature, seeds + np.uint64(1), pos0)  # drafts drawn from q (seed 1), uniforms from seed 2
    return pb, qb, drafts, seeds, pos0


@pytest.mark.parametrize("vocab_cfg,streams,k,temperature,peaked", [("wide", 32, 4, 1.0, 0.0), ("wide", 8, 4, 0.6, 0.9), ("micro", 16, 7, 1.0, 0.8), ("micro", 5, 1, 2.5, 0.5)])
def test_spec_accept_is_bit_exact(vocab_cfg, streams, k, temperature, peaked):
    w = util.weights_custom("wide", dict(util.MICRO, n_layers=1, vocab=128256)) if vocab_cfg == "wide" else util.weights("micro")
    eng = E.Engine(w, E.EngineConfig(max_seqs=2, max_step_tokens=16, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=8))
    pb, qb, drafts, seeds, pos0 = _case(streams, k, eng.desc.vocab, 5, temperature, peaked)
    want = oracle.spec_accept(pb, qb, drafts, temperature, seeds, pos0)
    acc, tok, rb, secs = eng.spec_accept(pb, qb, drafts, temperature, seeds, pos0, reps=3)
    assert np.array_equal(acc, want[0])
    assert np.array_equal(tok, want[1])
    assert np.array_equal(rb, want[2]) and np.array_equal(rb, k - acc)
    if peaked:
        assert acc.max() >= 1  # some drafts were accepted
    print(f"{vocab_cfg} S={streams} k={k}: accepted {acc.tolist()}, kernels {secs * 1e6:.1f} us")


def test_spec_accept_identical_distributions_accept_everything():
    eng = E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=2, max_step_tokens=16, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=8))
    pb, qb, drafts, seeds, pos0 = _case(6, 4, eng.desc.vocab, 9, 1.0)
    pb[:, :4] = qb  # q == p: min(1, p/q) = 1 > u always
    acc, tok, rb, _ = eng.spec_accept(pb, qb, drafts, 1.0, seeds, pos0)
    assert (acc == 4).all() and (rb == 0).all()
    want = oracle.spec_accept(pb, qb, drafts, 1.0, seeds, pos0)
    assert np.array_equal(tok, want[1])


def test_spec_accept_rejects_bad_arguments():
    eng = E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=2, max_step_tokens=16, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=8))
    pb, qb, drafts, seeds, pos0 = _case(2, 2, eng.desc.vocab, 1, 1.0)
    with pytest.raises(E.EngineError, match="temperature"):
        eng.spec_accept(pb, qb, drafts, 0.0, seeds, pos0)
    bad = drafts.copy()
    bad[0, 0] = 9999
    with pytest.raises(E.EngineError, match="out of range"):
        eng.spec_accept(pb, qb, bad, 1.0, seeds, pos0)
