"""vlt_step_capture (the reference's own parity entry point, engine/src/engine.rs:318-355) and vlt_set_taps with a list of
layers (engine.rs:381-389): every layer's intermediates and the tapped layers' outputs against the oracle's."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, vlt
from tests import util

pytestmark = pytest.mark.gpu
FIELDS = ["resid_in", "attn_in", "qkv", "sdpa_out", "attn_out", "mlp_in", "mlp_out"]


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.mark.parametrize("int8_group,counts", [(None, (5, 3)), (0, (5, 3)), (None, (12, 8)), (0, (12, 8))])
def test_layer_captures_and_taps_match_the_oracle(int8_group, counts):
    """Two sequences; steps of 8 tokens (the streamed matmul) and of 20 (the tensor-core GEMM), after a prefill."""
    w = util.weights("micro", int8_group)
    kw = dict(max_seqs=2, max_step_tokens=32, max_chunk=16, max_seq_len=128, max_head_rows=32)
    prod = E.Engine(w, E.EngineConfig(global_kv_tokens=256, **kw))
    orc = oracle.Engine(w, kv_tokens=256, **kw)
    orc.set_capture(True)
    for e in (prod, orc):
        e.set_taps([1, 0])
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    rng = np.random.default_rng(6)
    tol = 5e-2 if int8_group is not None else 2e-2
    for step in range(2):
        runs = [(s, rng.integers(0, 512, c).astype(np.uint32)) for s, c in zip((a, b), counts)]
        out, layers = prod.step_capture([E.Run(s, t) for s, t in runs], E.StepOptions(head=E.Rows.ALL, read_logits=True, read_taps=True))
        orc.step([(s, t, E.Rows.ALL, False) for s, t in runs])
        n = sum(counts)
        assert [l["layer"] for l in layers] == [0, 1]
        worst = {}
        for l in layers:
            for f in FIELDS:
                want = orc.array("cap_" + f).reshape(2, n, -1)[l["layer"]]
                assert l[f].shape == want.shape, f
                scale = max(1.0, float(np.abs(want).max()))
                worst[f] = max(worst.get(f, 0.0), float(np.abs(l[f] - want).max()) / scale)
        assert max(worst.values()) <= tol, worst
        want_logits = orc.array("logits").reshape(n, -1)
        assert float(np.abs(out.logits - want_logits).max()) <= tol
        taps = vlt.from_bf16(out.taps)
        want_taps = orc.array("taps_all").reshape(2, n, -1)
        assert taps.shape == want_taps.shape
        assert float(np.abs(taps - want_taps).max()) <= tol
        assert np.array_equal(want_taps[0], orc.array("taps").reshape(n, -1))  # tap 0 is layer 1, the last one
        for name in ("lens", "page_table", "free_pages"):
            assert np.array_equal(prod.debug_read(name)[:len(orc.array(name))], orc.array(name)), name
        # keep both engines on the oracle's tokens
        prod.debug_write("feed", 0, orc.array("feed")[:32])
        print(f"int8_group={int8_group} step {step}: worst relative error per field", {k: f"{v:.1e}" for k, v in worst.items()})


def test_capture_is_refused_while_a_generator_has_a_step_in_flight():
    eng = E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=2, max_step_tokens=32, max_chunk=16, global_kv_tokens=256, max_seq_len=128, max_head_rows=8))
    s = eng.new_seq()
    with eng.generator() as g:
        g.submit(E.Request(list(range(1, 9)), 4))
        g.step()
        with pytest.raises(E.EngineError, match="step in flight"):
            eng.step_capture([E.Run(s, [1, 2])])
        with pytest.raises(E.EngineError, match="step in flight"):
            eng.step([E.Run(s, [1, 2])])
        while not g.is_idle():
            g.step()
    eng.step([E.Run(s, [1, 2])])
    with pytest.raises(E.EngineError, match="taps: layer 7"):
        eng.set_taps([7])
