"""The reference's own architecture on the GPU (k_limite.cu, Engine::encode_forward_limite) against the oracle's
restatement of it (oracle/limite.hpp, limite_forward.hpp): synthetic files of tools/convert.py's tensor set. Local rings
and the global pool, q/k norm, RoPE on local layers only, value embeddings, attention gates, XSA, matrix scales and
residual lambdas, both MUDD sites, the capped head with masked padding ids; prompt chunks, decoding, tree verification
with cache compaction; integer state bit for bit."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth
from tests.test_gpu_parity import STATE, same_state

pytestmark = pytest.mark.gpu
MODELS = {
    "26 layers, hidden 256": dict(n_layers=26, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630),
    "48 layers, hidden 256, int8": dict(n_layers=48, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630, int8_group=64),
    "5 layers, the reference's widths": dict(n_layers=5, hidden=1280, n_kv=2, ffn=3328, vocab=1024),
}


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


@pytest.fixture(scope="module", params=list(MODELS), ids=list(MODELS))
def model(request, tmp_path_factory):
    path = tmp_path_factory.mktemp("limite") / "limite.vlt"
    desc = synth.write_limite(path, seed=5, **MODELS[request.param])
    return path, desc


def _pair(path, tuning=None, **kw):
    cfg = dict(max_seqs=3, max_step_tokens=64, max_chunk=32, global_kv_tokens=128 * 8, max_seq_len=512, max_head_rows=32)
    cfg.update(kw)
    prod = E.Engine(path, E.EngineConfig(**cfg), tuning or E.Tuning())
    orc = oracle.Engine(path, max_seqs=cfg["max_seqs"], max_step_tokens=cfg["max_step_tokens"], max_chunk=cfg["max_chunk"], kv_tokens=cfg["global_kv_tokens"],
                        max_seq_len=cfg["max_seq_len"], max_head_rows=cfg["max_head_rows"])
    return prod, orc


def _bf16(bits):
    return (np.asarray(bits).astype(np.uint32) << 16).view(np.float32)


def _step(prod, orc, runs, vocab_real, replay=None):
    """One step on both engines. The logits are capped to (0, 23): 5e-2 absolute (int8: 1e-1); a sampled or greedy token may
    differ from the oracle's only at a near-tie of its two best logits, and the product is then put on the oracle's token."""
    out = prod.debug_step(runs, E.StepOptions(read_logits=True), replay=replay)
    orc.step(runs, replay=replay)
    nr, n = len(runs), sum(len(r[1]) for r in runs)
    want = orc.array("logits").reshape(-1, prod.desc.vocab)
    assert out.logits.shape == want.shape
    assert np.isneginf(out.logits[:, vocab_real:]).all() and np.isneginf(want[:, vocab_real:]).all()
    err = float(np.abs(out.logits[:, :vocab_real] - want[:, :vocab_real]).max()) if want.size else 0.0
    assert err <= 1e-1, f"logits max-abs error {err}"
    assert not want.size or (want[:, :vocab_real].min() > 0 and want[:, :vocab_real].max() < 23)
    same_state(prod, orc, nr, n, names=[x for x in STATE if x != "feed"])
    top2 = np.sort(want[:, :vocab_real], axis=1)[:, -2:]
    clear = top2[:, 1] - top2[:, 0] > 2 * max(err, 1e-3)
    assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear])
    prod.debug_write("feed", 0, orc.array("feed"))
    for name in ("limite_k_local", "limite_v_local", "k_cache", "v_cache"):
        got, exp = _bf16(prod.debug_read(name).view(np.uint16)), _bf16(orc.array(name))
        e = float(np.abs(got - exp[:len(got)]).max() / max(np.abs(exp).max(), 1e-6))
        assert e <= 3e-2, f"{name}: {e} of the largest"
    return err


@pytest.mark.parametrize("keys_per_block", [0, 64], ids=["the library's key splits", "splits of 64 keys"])
def test_limite_forward_matches_the_oracle(model, keys_per_block):
    """keys_per_block (VltTuning.attn_keys_per_cta) = 64: a row's keys in many splits whatever the context (the partials and
    merge_kernel path as a long context takes it)."""
    path, desc = model
    if keys_per_block and desc["n_layers"] != 26:
        pytest.skip("the override's path is covered on one model")
    prod, orc = _pair(path, E.Tuning(attn_keys_per_cta=keys_per_block))
    assert (prod.desc.n_layers, prod.desc.d_model, prod.desc.head_dim, prod.desc.page_size) == (desc["n_layers"], desc["d"], 128, 128)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(17)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    pa, pb = rng.integers(0, vr, 21).astype(np.uint32), rng.integers(0, vr, 40).astype(np.uint32)
    errs = [_step(prod, orc, [(a, pa, E.Rows.LAST, False), (b, pb[:30], E.Rows.NONE, False)], vr)]
    errs.append(_step(prod, orc, [(b, pb[30:], E.Rows.ALL, False), (a, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    # Draft trees written by hand: a chain of wrong drafts for a; for b a tree whose second branch is b's own continuation
    # (taken from a plain decoding of the same prompt), so that the accepted path 0 -> 2 -> 3 is not a prefix of the rows
    # and the caches, rings and pages alike, are compacted.
    o2 = oracle.Engine(path, max_seqs=1, max_step_tokens=64, max_chunk=32, kv_tokens=128 * 8, max_seq_len=512, max_head_rows=32)
    q = o2.new_seq()
    o2.step([(q, pb[:30], E.Rows.NONE, False)])
    o2.step([(q, pb[30:], E.Rows.LAST, False)])
    cont = []
    for _ in range(3):
        cont.append(int(o2.array("feed")[0]))
        o2.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
    feed = orc.array("feed").reshape(-1, 16).copy()
    tree = orc.array("tree").reshape(-1, 16).copy()
    assert feed[b][0] == cont[0]
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    wrong = lambda t: (t + 1) % vr
    feed[a][1:4] = rng.integers(0, vr, 3)
    tree[a][1:4] = [node(1, 0, 0b0011), node(2, 1, 0b0111), node(3, 2, 0b1111)]
    feed[b][1:5] = [wrong(cont[1]), cont[1], cont[2], wrong(cont[2])]
    tree[b][1:5] = [node(1, 0, 0b00011), node(1, 0, 0b00101), node(2, 2, 0b01101), node(2, 1, 0b10011)]
    for eng, w in ((prod, prod.debug_write), (orc, orc.write)):
        w("feed", 0, feed.reshape(-1))
        w("tree", 0, tree.reshape(-1))
    runs = [(a, [E.FEED_ROW + i for i in range(4)], E.Rows.LAST, True), (b, [E.FEED_ROW + i for i in range(5)], E.Rows.LAST, True)]
    errs.append(_step(prod, orc, runs, vr))
    assert list(orc.array("path").reshape(-1, 16)[1][:3]) == [0, 2, 3] and orc.array("emitted")[1] == 3
    for s, e, rows in zip((a, b), orc.array("emitted")[:2], (4, 5)):
        prod.settle(s, rows - int(e))
        orc.settle(s, rows - int(e))
    assert prod.seq_len(a) == orc.seq_len(a) and prod.seq_len(b) == orc.seq_len(b)
    for _ in range(3):
        errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    print(f"limite {desc['n_layers']} layers d {desc['d']}: logits max-abs errors {['%.1e' % e for e in errs]}")
    prod.close()


def test_generator_on_the_reference_architecture_with_its_block_drafter(tmp_path):
    """The reference's own pairing: a target of its architecture (5 layers at its widths here) and its block drafter
    reading two of the target's layers, through the generator, beside a request behind the replay drafter and a plain
    one. Greedy: whatever is drafted, the tokens are those of the oracle's one-token-at-a-time decoding."""
    from tests.test_gpu_bench_shapes import _compare_stream
    target = tmp_path / "limite.vlt"
    synth.write_limite(target, n_layers=5, hidden=1280, n_kv=2, ffn=3328, vocab=1024, seed=8)
    sd = synth.block_drafter_state(2, hidden=1280, ffn=3328, layers=2, taps=(1, 3), draft_vocab=512, target_vocab=1024)
    drafter = tmp_path / "drafter.vlt"
    synth.write_block_drafter(drafter, sd)
    rng = np.random.default_rng(12)
    prompts = [rng.integers(0, 1024, n).astype(np.uint32) for n in (19, 33, 9)]
    max_tokens = [20, 14, 10]
    want = []
    for p, mt in zip(prompts, max_tokens):
        o = oracle.Engine(target, max_seqs=1, max_step_tokens=64, max_chunk=32, kv_tokens=128 * 4, max_seq_len=256, max_head_rows=8)
        q = o.new_seq()
        o.step([(q, p[:32], E.Rows.LAST if len(p) <= 32 else E.Rows.NONE, False)])
        if len(p) > 32:
            o.step([(q, p[32:], E.Rows.LAST, False)])
        toks, margins = [], []
        for i in range(mt):
            lg = np.sort(o.array("logits"))
            toks.append(int(o.array("feed")[0]))
            margins.append(float(lg[-1] - lg[-2]))
            if i + 1 < mt:
                o.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
        want.append((toks, margins))
    eng = E.Engine(target, E.EngineConfig(max_seqs=3, max_step_tokens=64, max_chunk=32, global_kv_tokens=128 * 6, max_seq_len=256, max_head_rows=24),
                   E.Tuning(spec_policy_off=True))
    eng.load_drafter(drafter)
    with eng.generator() as g:
        g.set_replay_mistakes(0.3, 4)
        reqs = [E.Request(list(prompts[0]), max_tokens[0], draft=E.Draft.MODEL, rows=8),
                E.Request(list(prompts[1]), max_tokens[1], draft=E.Draft.REPLAY, rows=5, trace=list(prompts[1]) + want[1][0]),
                E.Request(list(prompts[2]), max_tokens[2])]
        ids = [g.submit(r) for r in reqs]
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
    assert len(eng.debug_read("free_pages")) == 6
    eng.close()


def test_limite_rings_wrap_and_windows_slide(tmp_path):
    """A context longer than a local layer's ring (1024 + max_chunk positions): prompt chunks until the rings have wrapped
    and the windows no longer start at 0, then decoding steps of a second stream beside the long one (key splits of very
    different lengths in one launch), a chain of wrong drafts on the long stream with its compaction, and more decoding."""
    path = tmp_path / "limite_long.vlt"
    desc = synth.write_limite(path, seed=6, n_layers=5, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630)
    prod, orc = _pair(path, max_seqs=2, max_seq_len=1400, global_kv_tokens=128 * 14)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(23)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    prompt = rng.integers(0, vr, 1190).astype(np.uint32)
    errs = []
    for at in range(0, len(prompt), 32):
        last = at + 32 >= len(prompt)
        errs.append(_step(prod, orc, [(a, prompt[at:at + 32], E.Rows.LAST if last else E.Rows.NONE, False)], vr))
    assert prod.seq_len(a) == orc.seq_len(a) == 1190
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, rng.integers(0, vr, 9).astype(np.uint32), E.Rows.LAST, False)], vr))
    feed = orc.array("feed").reshape(-1, 16).copy()
    tree = orc.array("tree").reshape(-1, 16).copy()
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    feed[a][1:4] = rng.integers(0, vr, 3)
    tree[a][1:4] = [node(1, 0, 0b0011), node(2, 1, 0b0111), node(3, 2, 0b1111)]
    for w in (prod.debug_write, orc.write):
        w("feed", 0, feed.reshape(-1))
        w("tree", 0, tree.reshape(-1))
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW + i for i in range(4)], E.Rows.LAST, True), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    e = int(orc.array("emitted")[0])
    prod.settle(a, 4 - e)
    orc.settle(a, 4 - e)
    assert prod.seq_len(a) == orc.seq_len(a)
    for _ in range(3):
        errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    print(f"limite past the ring: logits max-abs errors, largest {max(errs):.1e}, last {errs[-1]:.1e}")
    prod.close()


def test_limite_many_streams_merge_their_key_splits_in_a_cluster(tmp_path):
    """Fifty streams decoding a token each, one of them over a context of 300 tokens: with that many rows and so few keys
    a row's key splits are one thread-block cluster that merges them in its first block's shared memory and finishes
    the attention itself (the short streams' later splits are empty)."""
    path = tmp_path / "limite_many.vlt"
    desc = synth.write_limite(path, seed=7, n_layers=5, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630)
    prod, orc = _pair(path, max_seqs=50, max_seq_len=512, global_kv_tokens=128 * 56, max_head_rows=64)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(29)
    seqs = [prod.new_seq() for _ in range(50)]
    assert [orc.new_seq() for _ in range(50)] == seqs
    prompt = rng.integers(0, vr, 300).astype(np.uint32)
    for at in range(0, 288, 32):
        _step(prod, orc, [(seqs[0], prompt[at:at + 32], E.Rows.NONE, False)], vr)
    first = [(seqs[0], prompt[288:], E.Rows.LAST, False)] + [(s, rng.integers(0, vr, 1).astype(np.uint32), E.Rows.LAST, False) for s in seqs[1:]]
    errs = [_step(prod, orc, first, vr)]
    for _ in range(3):
        errs.append(_step(prod, orc, [(s, [E.FEED_ROW], E.Rows.LAST, False) for s in seqs], vr))
    assert prod.seq_len(seqs[0]) == orc.seq_len(seqs[0]) == 303
    print(f"limite, 50 streams: logits max-abs errors {['%.1e' % e for e in errs]}")
    prod.close()


@pytest.mark.parametrize("hidden,n_kv", [(768, 6), (768, 2), (1024, 2), (768, 1), (896, 1), (1024, 1)],
                         ids=["1 query head a kv head", "3", "4", "6", "7", "8"])
def test_limite_attention_for_every_head_grouping(tmp_path, hidden, n_kv):
    """The attention kernels pack a kv head's query heads into the MMAs' columns: every grouping from 1 to 8 heads a kv
    head (6 fills the rows kernel's 48 columns with a tile of 8 rows; 7 and 8 keep a row per block) through a prompt chunk
    of 32 rows, decoding, a verified chain of 8 rows with its compaction, and decoding again, on 4 layers (three local,
    one global)."""
    path = tmp_path / "limite_g.vlt"
    desc = synth.write_limite(path, seed=11, n_layers=4, hidden=hidden, n_kv=n_kv, ffn=512, vocab=640, vocab_real=630)
    prod, orc = _pair(path, max_seqs=2)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(37)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    errs = [_step(prod, orc, [(a, rng.integers(0, vr, 32).astype(np.uint32), E.Rows.LAST, False), (b, rng.integers(0, vr, 5).astype(np.uint32), E.Rows.LAST, False)], vr)]
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    feed = orc.array("feed").reshape(-1, 16).copy()
    tree = orc.array("tree").reshape(-1, 16).copy()
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    feed[a][1:8] = rng.integers(0, vr, 7)
    tree[a][1:8] = [node(i, i - 1, (1 << (i + 1)) - 1) for i in range(1, 8)]
    for w in (prod.debug_write, orc.write):
        w("feed", 0, feed.reshape(-1))
        w("tree", 0, tree.reshape(-1))
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW + i for i in range(8)], E.Rows.LAST, True), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    e = int(orc.array("emitted")[0])
    prod.settle(a, 8 - e)
    orc.settle(a, 8 - e)
    assert prod.seq_len(a) == orc.seq_len(a)
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    print(f"limite hidden {hidden}, {n_kv} kv heads: logits max-abs errors {['%.1e' % x for x in errs]}")
    prod.close()


@pytest.mark.parametrize("group", [16, 32, 128, 256])
def test_limite_int8_scale_groups_through_the_gemm(tmp_path, group):
    """int8 projections with scale groups along k other than the converter's default 64 (the head stays at 8): steps of 40
    and 12 rows take the tensor-core GEMM, whose converter warps put the groups' scales onto the weights -- groups within
    a k block of 64 and groups that span two and four of them -- then decoding on the streamed kernel."""
    path = tmp_path / "limite_q.vlt"
    desc = synth.write_limite(path, seed=13, n_layers=4, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630, int8_group=group)
    prod, orc = _pair(path, max_seqs=2)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(41)
    a, b = prod.new_seq(), prod.new_seq()
    assert (orc.new_seq(), orc.new_seq()) == (a, b)
    errs = [_step(prod, orc, [(a, rng.integers(0, vr, 30).astype(np.uint32), E.Rows.LAST, False), (b, rng.integers(0, vr, 10).astype(np.uint32), E.Rows.ALL, False)], vr)]
    errs.append(_step(prod, orc, [(a, rng.integers(0, vr, 11).astype(np.uint32), E.Rows.ALL, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    errs.append(_step(prod, orc, [(a, [E.FEED_ROW], E.Rows.LAST, False), (b, [E.FEED_ROW], E.Rows.LAST, False)], vr))
    print(f"limite int8 in groups of {group}: logits max-abs errors {['%.1e' % x for x in errs]}")
    assert max(errs) <= 2e-2
    prod.close()


def test_limite_step_longer_than_a_gemm_launch(tmp_path):
    """Ten streams' prompt chunks of 32 rows in one step of 320 tokens: the GEMMs run in blocks of 256 and 64 tokens (the
    bf16 inputs and sums of squares a layer's last projection leaves for the next are indexed by the step's token, not
    the block's), the attention in 40 tiles of 8 rows; then all ten decode."""
    path = tmp_path / "limite_wide.vlt"
    desc = synth.write_limite(path, seed=15, n_layers=5, hidden=256, n_kv=1, ffn=512, vocab=640, vocab_real=630)
    prod, orc = _pair(path, max_seqs=10, max_step_tokens=320, global_kv_tokens=128 * 12, max_head_rows=32)
    vr = desc["vocab_real"]
    rng = np.random.default_rng(43)
    seqs = [prod.new_seq() for _ in range(10)]
    assert [orc.new_seq() for _ in range(10)] == seqs
    errs = [_step(prod, orc, [(s, rng.integers(0, vr, 32).astype(np.uint32), E.Rows.LAST, False) for s in seqs], vr)]
    for _ in range(2):
        errs.append(_step(prod, orc, [(s, [E.FEED_ROW], E.Rows.LAST, False) for s in seqs], vr))
    print(f"limite, a step of 320 tokens: logits max-abs errors {['%.1e' % x for x in errs]}")
    assert max(errs) <= 2e-2
    prod.close()
