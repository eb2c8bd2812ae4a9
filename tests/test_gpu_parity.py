"""GPU parity: the CUDA path through the C ABI against the CPU oracle on the same seeded inputs.

Tolerances (from the task's statement): logits within 2e-2 max-abs with bf16 weights and 5e-2
with int8; everything integer -- sampled tokens given identical logits, acceptance, emitted
counts, page tables, per-slot state -- bit for bit.
"""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E
from tests import util

pytestmark = pytest.mark.gpu
TOL = {None: 2e-2, 0: 5e-2, 64: 5e-2}
STATE = ["lens", "feed", "tree", "gen", "path_len", "emitted", "page_table", "free_pages"]


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def pair(name="micro", int8_group=None, tuning=None, **kw):
    cfg = dict(max_seqs=4, max_step_tokens=64, max_chunk=32, global_kv_tokens=16 * 64, max_seq_len=512, max_head_rows=32)
    cfg.update(kw)
    w = util.weights(name, int8_group)
    prod = E.Engine(w, E.EngineConfig(**cfg), tuning)
    orc = oracle.Engine(w, max_seqs=cfg["max_seqs"], max_step_tokens=cfg["max_step_tokens"], max_chunk=cfg["max_chunk"], kv_tokens=cfg["global_kv_tokens"],
                        max_seq_len=cfg["max_seq_len"], max_head_rows=cfg["max_head_rows"])
    return prod, orc


def same_state(prod, orc, n_runs, n_tokens, names=STATE):
    for name in names:
        a, b = prod.debug_read(name), orc.array(name)
        if name == "emitted":
            a = a[:n_runs]
        assert np.array_equal(a[:len(b)], b), name
    assert np.array_equal(prod.debug_read("on_path")[:n_tokens], orc.array("on_path")[:n_tokens]), "on_path"
    assert np.array_equal(prod.debug_read("meta")[:2 * n_tokens], orc.array("meta")[:2 * n_tokens]), "meta"
    assert np.array_equal(prod.debug_read("tokens")[:n_tokens], orc.array("tokens")[:n_tokens]), "tokens"
    assert np.array_equal(prod.debug_read("vis")[:n_tokens], orc.array("vis")[:n_tokens]), "vis"
    k = orc.array("path_len")
    pa, pb = prod.debug_read("path").reshape(-1, 16), orc.array("path").reshape(-1, 16)
    for r in range(n_runs):
        assert np.array_equal(pa[r][:k[r]], pb[r][:k[r]]), "path"


def both_step(prod, orc, runs, tol, replay=None, check_ids=True):
    out = prod.debug_step(runs, E.StepOptions(read_logits=True), replay=replay)
    if replay:
        orc.set_replay(*replay)
    orc.step(runs, replay=bool(replay))
    v = prod.desc.vocab
    want = orc.array("logits").reshape(-1, v)
    got = out.logits
    assert got.shape == want.shape
    err = float(np.abs(got - want).max()) if got.size else 0.0
    assert err <= tol, f"logits max-abs error {err}"
    return out, want, err


@pytest.mark.parametrize("int8_group", [None, 0, 64])
@pytest.mark.parametrize("name", ["micro", "micro4"])
def test_forward_logits_match_the_oracle(name, int8_group):
    """Prefill in chunks (several attention tiles and pages), then one-token steps, greedy."""
    prod, orc = pair(name, int8_group)
    rng = np.random.default_rng(1)
    a, b = prod.new_seq(), orc.new_seq()
    vocab = prod.desc.vocab
    toks = rng.integers(0, vocab, 70).astype(np.uint32)
    worst = 0.0
    for lo, hi in ((0, 30), (30, 37), (37, 38), (38, 70)):
        out, want, err = both_step(prod, orc, [(a, toks[lo:hi], E.Rows.ALL, False)], TOL[int8_group])
        worst = max(worst, err)
        # Greedy tokens agree wherever the oracle's top-2 margin exceeds 1e-2.
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = top2[:, 1] - top2[:, 0] > 1e-2
        assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear])
        assert clear.mean() > 0.5
        # Keep both sides on the same path: the next input is what the oracle chose.
        prod.debug_write("feed", a * 16, orc.array("feed")[a * 16:a * 16 + 1])
        for name_ in ("lens", "page_table", "free_pages", "meta"):
            assert np.array_equal(prod.debug_read(name_)[:len(orc.array(name_))], orc.array(name_)), name_
    print(f"{name} int8_group={int8_group}: worst logits error {worst:.2e}")


@pytest.mark.parametrize("int8_group", [None, 0])
def test_full_width_steps_match_the_oracle(int8_group):
    """The benchmark's step shapes through the tensor-core GEMM: 32 sequences x 8 tokens = 256 tokens in one step
    (the GEMM's widest N), then verify-shaped steps of 32 x 5 = 160 rows with every row through the head."""
    prod, orc = pair("micro", int8_group, max_seqs=32, max_step_tokens=256, max_chunk=16, global_kv_tokens=32 * 64, max_seq_len=64, max_head_rows=160)
    rng = np.random.default_rng(23)
    seqs = [prod.new_seq() for _ in range(32)]
    assert [orc.new_seq() for _ in range(32)] == seqs
    vocab = prod.desc.vocab
    prompts = [rng.integers(0, vocab, 8).astype(np.uint32) for _ in seqs]
    both_step(prod, orc, [(s, p, E.Rows.NONE if i % 4 else E.Rows.LAST, False) for i, (s, p) in enumerate(zip(seqs, prompts))], TOL[int8_group])
    same_state(prod, orc, 32, 256)
    for step in range(2):
        runs = [(s, rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False) for s in seqs]
        out, want, err = both_step(prod, orc, runs, TOL[int8_group])
        assert want.shape[0] == 160
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = top2[:, 1] - top2[:, 0] > 1e-2
        assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear]) and clear.mean() > 0.5
        for name_ in ("lens", "page_table", "free_pages", "meta"):
            assert np.array_equal(prod.debug_read(name_)[:len(orc.array(name_))], orc.array(name_)), name_
        print(f"160-row step, int8_group={int8_group}: logits error {err:.2e}")


@pytest.mark.parametrize("int8_group", [None, 0])
def test_wide_matrices_take_the_unsplit_gemm_path(int8_group):
    """gate_up with 80 and a head with 96 tiles of 128 rows: more than half the SMs, so the GEMM keeps a tile's
    whole k in one block and its epilogue goes straight from tensor memory to global memory (SwiGLU and head);
    the narrow matrices of the same model still split k over clusters."""
    cfg = dict(util.MICRO, n_layers=1, ffn=5120, vocab=12288)
    w = util.weights_custom("wide_ffn", cfg, int8_group)
    kw = dict(max_seqs=8, max_step_tokens=64, max_chunk=16, max_seq_len=64, max_head_rows=64)
    prod = E.Engine(w, E.EngineConfig(global_kv_tokens=8 * 64, **kw))
    orc = oracle.Engine(w, kv_tokens=8 * 64, **kw)
    rng = np.random.default_rng(29)
    seqs = [prod.new_seq() for _ in range(8)]
    assert [orc.new_seq() for _ in range(8)] == seqs
    for count in (8, 5, 3):  # 64, 40 and 24 tokens a step, every row through the head
        runs = [(s, rng.integers(0, cfg["vocab"], count).astype(np.uint32), E.Rows.ALL, False) for s in seqs]
        out, want, err = both_step(prod, orc, runs, TOL[int8_group])
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = top2[:, 1] - top2[:, 0] > 1e-2
        assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear]) and clear.mean() > 0.5
        print(f"{8 * count}-token step over wide matrices, int8_group={int8_group}: logits error {err:.2e}")


@pytest.mark.parametrize("std", [0.0005, 4.0])
def test_small_steps_with_activations_far_from_one_match_the_oracle(std, tmp_path):
    """int8 weights in steps of at most 8 tokens are multiplied as fp16, the activations scaled per token by a power of
    two when their largest magnitude leaves [2^-6, 2^15): weights 40 times smaller than usual (attention output and
    SwiGLU products far below 2^-6) and 200 times larger (a residual stream beyond fp16's range) take that path."""
    from silicon_violetto_b200 import synth
    w = tmp_path / f"micro_std{std}.vlt"
    synth.write_target(w, util.MICRO, seed=3, int8_group=0, std=std)
    kw = dict(max_seqs=2, max_step_tokens=16, max_chunk=8, max_seq_len=64, max_head_rows=16)
    prod = E.Engine(w, E.EngineConfig(global_kv_tokens=2 * 64, **kw))
    orc = oracle.Engine(w, kv_tokens=2 * 64, **kw)
    rng = np.random.default_rng(31)
    a, b = prod.new_seq(), orc.new_seq()
    assert a == b
    for count in (5, 1, 8, 1):
        runs = [(a, rng.integers(0, 512, count).astype(np.uint32), E.Rows.ALL, False)]
        out = prod.debug_step(runs, E.StepOptions(read_logits=True))
        orc.step(runs)
        want = orc.array("logits").reshape(-1, 512)
        scale = max(1.0, float(np.abs(want).max()))
        err = float(np.abs(out.logits - want).max()) / scale
        assert np.isfinite(out.logits).all() and err < TOL[0], (std, count, err, scale)
    prod.close()


def test_kv_cache_matches_the_oracle_after_prefill():
    prod, orc = pair("micro")
    a, b = prod.new_seq(), orc.new_seq()
    toks = np.arange(30, dtype=np.uint32) * 7 % 512
    both_step(prod, orc, [(a, toks, E.Rows.LAST, False)], 2e-2)
    # Layer 0's K and V depend only on the embedding and one matmul: near bit-equal.
    # (The cache itself is read back through a second engine step's logits in other tests;
    # here the page table and lengths say where it went.)
    assert prod.debug_read("lens")[a] == 30 and orc.array("lens")[b] == 30
    assert np.array_equal(prod.debug_read("page_table")[:2], np.array([0, 1], np.uint32))


@pytest.mark.parametrize("keys_per_block", [640, 128])
def test_two_attention_kernels_agree_at_long_context(keys_per_block):
    """The tensor-core attention against the scalar one, 3000 cached keys with filled values, 5 key splits and 24."""
    w = util.weights("micro4", 0)
    cfg = E.EngineConfig(max_seqs=3, max_step_tokens=32, max_chunk=8, global_kv_tokens=3 * 3200, max_seq_len=3200, max_head_rows=24)
    outs = []
    for plain in (False, True):
        eng = E.Engine(w, cfg, E.Tuning(plain_attention=plain, attn_keys_per_cta=keys_per_block))
        seqs = [eng.new_seq() for _ in range(3)]
        for i, s in enumerate(seqs):
            eng.bench_fill(s, [3000, 17, 1234][i], seed=5 + i)
        runs = [(s, [3 + i, 9, 100 + i, 7, 200][: [5, 3, 8 - 3][i]], E.Rows.ALL, False) for i, s in enumerate(seqs)]
        outs.append(eng.debug_step(runs, E.StepOptions(read_logits=True)).logits)
        eng.close()
    err = float(np.abs(outs[0] - outs[1]).max())
    assert err < 2e-2, err


def test_verify_runs_with_the_replay_drafter_match_the_oracle():
    """Chain verification: the replay drafter's drafts (some wrong), accept, lens, feed, emitted."""
    prod, orc = pair("micro", None)
    rng = np.random.default_rng(3)
    a, b = prod.new_seq(), orc.new_seq()
    prompt = rng.integers(0, 512, 20).astype(np.uint32)
    # The recorded continuation: the oracle's own greedy decode, so that right drafts exist.
    o2 = oracle.Engine(util.weights("micro"), max_seqs=1, max_step_tokens=64, max_chunk=40, kv_tokens=256, max_seq_len=256, max_head_rows=8)
    q = o2.new_seq()
    o2.step([(q, prompt, E.Rows.LAST, False)])
    cont = []
    for _ in range(24):
        cont.append(int(o2.array("feed")[0]))
        o2.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
    trace = np.concatenate([prompt, np.array(cont, np.uint32)])
    assert a == b
    for e in (prod, orc):
        e.set_trace(a, trace)
        e.set_gen(a, 20, stop=[])
    both_step(prod, orc, [(a, prompt, E.Rows.LAST, False)], 2e-2, replay=(0.3, 7))
    same_state(prod, orc, 1, len(prompt))
    total = 0
    for step in range(8):
        rows = [5, 8, 2, 5, 3, 8, 5, 5][step]
        runs = [(a, [E.FEED_ROW + i for i in range(rows)], E.Rows.LAST, True)]
        both_step(prod, orc, runs, 2e-2, replay=(0.3, 7))
        same_state(prod, orc, 1, rows)
        e = int(orc.array("emitted")[0])
        total += e
        for eng in (prod, orc):
            eng.settle(a, rows - e)
        assert prod.seq_len(a) == orc.seq_len(b)
        if orc.array("gen")[a * 12 + 1]:
            break
    assert total >= 10  # several multi-token acceptances happened


def test_draft_trees_accept_and_compact_like_the_oracle():
    """A hand-built draft tree per slot: the accepted path is not a prefix of the rows, so kv_compact moves K/V."""
    prod, orc = pair("micro", None, max_seqs=2)
    rng = np.random.default_rng(4)
    seqs = [prod.new_seq(), prod.new_seq()]
    assert seqs == [orc.new_seq(), orc.new_seq()]
    prompts = [rng.integers(0, 512, 18).astype(np.uint32), rng.integers(0, 512, 31).astype(np.uint32)]
    both_step(prod, orc, [(s, p, E.Rows.LAST, False) for s, p in zip(seqs, prompts)], 2e-2)
    same_state(prod, orc, 2, 49)
    # What plain decoding emits next, from a scratch oracle run.
    greedy = {}
    for s, p in zip(seqs, prompts):
        o2 = oracle.Engine(util.weights("micro"), max_seqs=1, max_step_tokens=64, max_chunk=40, kv_tokens=256, max_seq_len=256, max_head_rows=8)
        q = o2.new_seq()
        o2.step([(q, p, E.Rows.LAST, False)])
        out = []
        for _ in range(4):
            out.append(int(o2.array("feed")[0]))
            o2.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
        greedy[s] = out
    # Tree rows: 0 root; 1 wrong child of 0; 2 right child of 0; 3 child of 1; 4 right child of 2; 5 wrong child of 4.
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    for s in seqs:
        g = greedy[s]
        feed = [g[0], (g[1] + 1) % 512, g[1], g[2], g[2], (g[3] + 5) % 512]
        tree = [oracle.chain_node(0), node(1, 0, 0b000011), node(1, 0, 0b000101), node(2, 1, 0b001011), node(2, 2, 0b010101), node(3, 4, 0b110101)]
        for e in (prod, orc):
            (e.debug_write if e is prod else e.write)("feed", s * 16, feed)
            (e.debug_write if e is prod else e.write)("tree", s * 16, tree)
    runs = [(s, [E.FEED_ROW + i for i in range(6)], E.Rows.LAST, True) for s in seqs]
    both_step(prod, orc, runs, 2e-2)
    same_state(prod, orc, 2, 12)
    assert list(orc.array("path_len")[:2]) == [3, 3]
    assert list(orc.array("path")[:3]) == [0, 2, 4]
    for s in seqs:
        for e in (prod, orc):
            e.settle(s, 6 - 3)
    # The compacted K/V must now serve a plain step: logits agree again.
    both_step(prod, orc, [(s, [E.FEED_ROW], E.Rows.LAST, False) for s in seqs], 2e-2)
    same_state(prod, orc, 2, 2)


def _rows(n, rng, temps, top_ps):
    return [(E.Sampling(float(rng.choice(temps)), float(rng.choice(top_ps)), int(rng.integers(1 << 62))), int(rng.integers(1, 1 << 20))) for _ in range(n)]


def _oracle_rows(rows):
    r = np.zeros(len(rows), oracle.SAMPLE_ROW)
    for i, (s, pos) in enumerate(rows):
        r[i] = (s.seed & 0xFFFFFFFF, s.seed >> 32, pos, s.temperature, s.top_p, oracle.NO_TOK)
    return r


@pytest.mark.parametrize("vocab_cfg", ["micro", "wide"])
def test_sampler_is_bit_exact(vocab_cfg):
    """Engine::sample_logits on caller-supplied logits: every drawn token equals the oracle's."""
    if vocab_cfg == "wide":
        cfg = dict(util.MICRO, n_layers=1, vocab=128256)
        w = util.weights_custom("wide", cfg)
    else:
        w = util.weights("micro")
    eng = E.Engine(w, E.EngineConfig(max_seqs=2, max_step_tokens=40, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=40))
    v = eng.desc.vocab
    rng = np.random.default_rng(9)
    n = 40
    logits = (rng.standard_normal((n, v)) * 3.0).astype(np.float32)
    logits[0, :] = 1.0  # all tied: the lowest id at temperature 0
    logits[1, 5::7] = logits[1].max() + 1.0  # many tied maxima
    logits[2] = np.round(logits[2])  # many equal values
    logits[3, 100] = 60.0  # one dominant token: everything else underflows at low temperature
    logits[4] = -1e30
    logits[4, v - 1] = 0.0
    rows = _rows(n, rng, [0.0, 0.6, 1.0, 0.05, 3.0], [1.0, 0.95, 0.5, 0.05])
    rows[0] = (E.Sampling(0.0, 1.0, 0), 3)
    got = eng.sample_logits(logits, rows)
    want = oracle.sample(logits, _oracle_rows(rows))
    assert np.array_equal(got, want)
    assert got[0] == 0 and got[4] == v - 1
    # The draw is a function of (seed, position) alone: the same rows again give the same tokens,
    # and a different position gives different draws.
    assert np.array_equal(eng.sample_logits(None, rows), got)
    hot = [(E.Sampling(1.0, 1.0, 11), p) for p in range(1, n + 1)]
    d1 = eng.sample_logits(logits, hot)
    assert np.array_equal(d1, oracle.sample(logits, _oracle_rows(hot)))
    assert len(set(d1.tolist())) > n // 2


def test_sampler_with_many_rows_takes_the_one_block_form_and_stays_bit_exact():
    """More than 96 rows go through the one-block-per-row kernel, fewer through the cluster of 8 blocks per row: same tokens."""
    eng = E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=2, max_step_tokens=128, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=128))
    v = eng.desc.vocab
    rng = np.random.default_rng(17)
    n = 128
    logits = (rng.standard_normal((n, v)) * 3.0).astype(np.float32)
    rows = _rows(n, rng, [0.0, 0.6, 1.0, 3.0], [1.0, 0.95, 0.5, 0.05])
    many = eng.sample_logits(logits, rows)
    assert np.array_equal(many, oracle.sample(logits, _oracle_rows(rows)))
    few = np.concatenate([eng.sample_logits(logits[i:i + 64], rows[i:i + 64]) for i in (0, 64)])
    assert np.array_equal(few, many)


def test_generator_reproduces_plain_decoding():
    """Continuous batching with replay drafts, greedy: every request's tokens are what the oracle
    decodes one token at a time (the reference's own check, cli/src/bench_spec.rs:133-139)."""
    w = util.weights("micro")
    rng = np.random.default_rng(11)
    prompts = [rng.integers(0, 512, n).astype(np.uint32) for n in (5, 23, 40, 9, 31)]
    max_tokens = [12, 20, 7, 16, 10]
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
    # Margins: a near-tie in the oracle's logits could legitimately flip on the GPU; the seeds above have none.
    eng = E.Engine(w, E.EngineConfig(max_seqs=3, max_step_tokens=48, max_chunk=16, global_kv_tokens=16 * 24, max_seq_len=128, max_head_rows=24),
                   E.Tuning(spec_policy_off=True))
    for rate in (0.0, 0.3):
        with eng.generator() as g:
            g.set_replay_mistakes(rate, 5)
            ids = []
            for i, (p, mt) in enumerate(zip(prompts, max_tokens)):
                kind = [E.Draft.REPLAY, E.Draft.NONE, E.Draft.REPLAY, E.Draft.REPLAY, E.Draft.NONE][i]
                rows = [5, 1, 8, 3, 1][i]
                ids.append(g.submit(E.Request(list(p), mt, draft=kind, rows=rows, trace=list(p) + want[i])))
            got = {i: [] for i in ids}
            done = {}
            for _ in range(400):
                if g.is_idle():
                    break
                for ev in g.step():
                    if ev.kind == "token":
                        got[ev.req].append(ev.value)
                    else:
                        done[ev.req] = ev.value
            assert g.is_idle()
            stats = g.take_stats()
        for i, rid in enumerate(ids):
            assert got[rid] == want[i], f"request {i} at mistake rate {rate}"
            assert done[rid] == E.Finish.LENGTH
        assert sum(s["emitted"] for s in stats) == sum(max_tokens)
        if rate == 0.0:
            # Perfect drafts: the drafted requests take far fewer steps than tokens.
            assert len(stats) < sum(max_tokens)
    # Everything was freed: all pages are back.
    assert len(eng.debug_read("free_pages")) == 24


def test_generator_stop_tokens_and_cancel():
    w = util.weights("micro")
    eng = E.Engine(w, E.EngineConfig(max_seqs=2, max_step_tokens=32, max_chunk=16, global_kv_tokens=16 * 16, max_seq_len=128, max_head_rows=8))
    p = list(range(1, 12))
    with eng.generator() as g:
        rid = g.submit(E.Request(p, 10))
        toks = []
        while not g.is_idle():
            toks += [e.value for e in g.step() if e.kind == "token"]
    assert len(toks) == 10
    stop = toks[3]
    first = toks.index(stop)
    with eng.generator() as g:
        rid = g.submit(E.Request(p, 10, stop=[stop]))
        rid2 = g.submit(E.Request(p, 50))
        g.cancel(rid2)
        evs = []
        while not g.is_idle():
            evs += g.step()
    assert [e.value for e in evs if e.kind == "token"] == toks[:first + 1]
    assert [e for e in evs if e.kind == "done"][0].value == E.Finish.STOP
    assert all(e.req == rid for e in evs)
    with eng.generator() as g:
        for bad, msg in ((E.Request([], 5), "empty prompt"), (E.Request(p, 0), "max_tokens is 0"), (E.Request([9999], 5), "token id out of range"),
                         (E.Request(p, 5, stop=list(range(9))), "9 stop tokens"), (E.Request(p, 5, draft=E.Draft.MODEL, rows=4), "needs a loaded drafter"),
                         (E.Request(p, 500), "doesn't fit max_seq_len or the KV pool")):
            with pytest.raises(E.EngineError, match=msg):
                g.submit(bad)
