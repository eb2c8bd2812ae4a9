"""How a kernel's bounded wait running out is reported, and a randomized sweep of model shapes against the oracle."""
import numpy as np
import pytest
from hypothesis import HealthCheck, given, settings, strategies as st

import oracle
from silicon_violetto_b200 import build, engine as E, synth
from tests import util
from tests.test_gpu_parity import TOL

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def test_a_wait_that_runs_out_is_reported_and_the_engine_carries_on():
    """Every mbarrier wait in the kernels gives up after a bounded number of polls, sets the device error word and lets its
    kernel return. A debug kernel makes exactly that happen (it waits for an arrival nobody makes, 1024 polls): the step
    collected next must fail with the report, synchronously and through the generator, and later steps must be untouched."""
    w = util.weights("micro")
    kw = dict(max_seqs=2, max_step_tokens=32, max_chunk=16, max_seq_len=128, max_head_rows=16)
    eng = E.Engine(w, E.EngineConfig(global_kv_tokens=256, **kw))
    orc = oracle.Engine(w, kv_tokens=256, **kw)
    a, b = eng.new_seq(), orc.new_seq()
    toks = np.arange(1, 11, dtype=np.uint32)
    eng.debug_stalled_wait()
    with pytest.raises(E.EngineError, match="bounded wait ran out.*flag 7"):
        eng.step([E.Run(a, toks[:4])])
    orc.step([(b, toks[:4], E.Rows.LAST, False)])  # the step itself ran: both sequences hold 4 positions
    out = eng.debug_step([(a, toks[4:], E.Rows.ALL, False)], E.StepOptions(read_logits=True))
    orc.step([(b, toks[4:], E.Rows.ALL, False)])
    assert float(np.abs(out.logits - orc.array("logits").reshape(out.logits.shape)).max()) <= 2e-2
    with eng.generator() as g:
        rid = g.submit(E.Request(list(range(1, 9)), 6))
        g.step()
        eng.debug_stalled_wait()
        with pytest.raises(E.EngineError, match="bounded wait ran out"):
            for _ in range(4):
                g.step()
    with eng.generator() as g:  # a new generator on the same engine decodes as if nothing had happened
        g.submit(E.Request(list(range(1, 9)), 6))
        got = []
        while not g.is_idle():
            got += [e.value for e in g.step() if e.kind == "token"]
    assert len(got) == 6


SHAPES = st.fixed_dictionaries(dict(
    d=st.sampled_from([256, 512]), heads=st.sampled_from([(1, 4), (2, 2), (4, 1), (2, 4), (4, 2)]),  # (kv heads, query heads per kv head): the loader wants 256-multiples
    ffn=st.sampled_from([256, 512, 768, 1024]), vocab=st.sampled_from([128, 500, 1024, 1536]), n_layers=st.integers(1, 2),
    int8_group=st.sampled_from([None, 0, 64, 128]), counts=st.lists(st.integers(1, 12), min_size=1, max_size=4),
    keys_per_block=st.sampled_from([0, 64, 128]), prefill=st.integers(0, 300), seed=st.integers(0, 1000)))


@settings(max_examples=16, deadline=None, derandomize=True, suppress_health_check=list(HealthCheck))
@given(SHAPES)
def test_random_shapes_match_the_oracle(tmp_path_factory, c):
    """Random decoders (width, heads per kv head, FFN, vocabulary -- also sizes no tile divides --, bf16 / int8 per row / int8
    in groups of 64 or 128), random step shapes (1 to 48 tokens over 1 to 4 sequences: the streamed matmul, its 8-token
    blocks, the tensor-core GEMM with and without split k), over a filled context of 0 to 300 positions with random key splits."""
    cfg = dict(n_layers=c["n_layers"], d=c["d"], n_heads=c["heads"][0] * c["heads"][1], n_kv=c["heads"][0], hd=64, ffn=c["ffn"], vocab=c["vocab"], eps=1e-5, theta=500000.0, page=16)
    if c["int8_group"] and (c["d"] % c["int8_group"] or c["ffn"] % c["int8_group"] or (cfg["n_heads"] * 64) % c["int8_group"]):
        c = dict(c, int8_group=0)
    w = tmp_path_factory.mktemp("fuzz") / "m.vlt"
    synth.write_target(w, cfg, seed=c["seed"], int8_group=c["int8_group"])
    n = sum(c["counts"])
    kw = dict(max_seqs=4, max_step_tokens=64, max_chunk=16, max_seq_len=400, max_head_rows=64)
    prod = E.Engine(w, E.EngineConfig(global_kv_tokens=4 * 416, **kw), E.Tuning(attn_keys_per_cta=c["keys_per_block"]))
    orc = oracle.Engine(w, kv_tokens=4 * 416, **kw)
    rng = np.random.default_rng(c["seed"])
    seqs = [prod.new_seq() for _ in c["counts"]]
    assert [orc.new_seq() for _ in c["counts"]] == seqs
    for i, s in enumerate(seqs):
        fill = int(rng.integers(0, c["prefill"] + 1))
        if fill:
            prod.bench_fill(s, fill, seed=1 + i)
            orc.bench_fill(s, fill, seed=1 + i)
    tol = TOL[0] if c["int8_group"] is not None else TOL[None]
    for step in range(2):
        runs = [(s, rng.integers(0, c["vocab"], k).astype(np.uint32), E.Rows.ALL, False) for s, k in zip(seqs, c["counts"])]
        out = prod.debug_step(runs, E.StepOptions(read_logits=True))
        orc.step(runs)
        want = orc.array("logits").reshape(n, -1)
        scale = max(1.0, float(np.abs(want).max()))
        err = float(np.abs(out.logits - want).max()) / scale
        assert err <= tol, (c, step, err)
        for name in ("lens", "page_table", "free_pages", "meta"):
            assert np.array_equal(prod.debug_read(name)[:len(orc.array(name))], orc.array(name)), (c, name)
        prod.debug_write("feed", 0, orc.array("feed")[:64])
    prod.close()
