"""GPU parity at the shapes the benchmark runs, against the CPU oracle through the C ABI.

  - the tensor-core attention with its key splits and both split-merge kernels over long filled contexts
    (the oracle fills the same hashed K/V for the same seed), chain and tree masks, 2 and 4 query heads
    per kv head, lengths 17 / 1234 / 8192 in one step;
  - one decoder layer at the 1B model's dimensions (d 2048, 32 q / 8 kv heads, FFN 8192, 128 256 ids),
    bf16 and int8 per row, at 5 tokens (the streamed matmul, four k slices on `down`), 160 and 256 tokens
    (the tcgen05 GEMM: 32 and 128 k blocks, rings wrapping, the head's seven waves);
  - the plumbing configuration as the benchmark states it (2 layers, d 256, FFN 1024, 4096 ids, a 64-token
    prompt, greedy, four drafts a step) through the generator with the chain drafter and with the replay
    drafter: the token stream is the oracle's plain decoding.

Tolerances: logits within 2e-2 (bf16 weights) / 5e-2 (int8) max-abs -- at the 1B dimensions, where logits reach +-5,
that or one bf16 unit in the last place of the largest logit (see _agree_at_scale); greedy tokens equal wherever the
oracle's top-2 margin exceeds 1e-2; integer state bit for bit.
"""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, synth
from tests import util
from tests.test_gpu_parity import STATE, TOL, same_state

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def _pair(w, tuning=None, **kw):
    prod = E.Engine(w, E.EngineConfig(**kw), tuning)
    okw = dict(kw)
    okw["kv_tokens"] = okw.pop("global_kv_tokens")
    return prod, oracle.Engine(w, **okw)


def _logits_agree(prod, orc, runs, tol, check_ids=True):
    out = prod.debug_step(runs, E.StepOptions(read_logits=True))
    orc.step(runs)
    want = orc.array("logits").reshape(-1, prod.desc.vocab)
    assert out.logits.shape == want.shape
    assert np.isfinite(out.logits[:, :prod.desc.vocab_real]).all()
    err = float(np.abs(out.logits - want).max())
    assert err <= tol, f"logits max-abs error {err}"
    if check_ids:
        top2 = np.sort(want, axis=1)[:, -2:]
        clear = top2[:, 1] - top2[:, 0] > 1e-2
        assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear])
    return err


# ---------------------------------------------------------------- attention over long filled contexts
# (context of the longest sequence, keys one attention block takes, the split count that must result)
SPLITS = [(3000, 1503, 2), (3000, 602, 5), (3000, 126, 24), (8192, 4100, 2), (8192, 1640, 5), (8192, 342, 22), (8192, 191, 43)]


@pytest.mark.parametrize("name,int8_group", [("micro4", 0), ("micro", None)])
@pytest.mark.parametrize("ctx,keys_per_block,splits", SPLITS)
def test_split_attention_matches_the_oracle_over_filled_contexts(name, int8_group, ctx, keys_per_block, splits):
    """Three sequences of 17, 1234 and `ctx` filled positions in one step: first plain runs of 5, 3 and 5
    tokens (causal masks), then verify runs over a draft tree whose accepted path is not a prefix."""
    w = util.weights(name, int8_group)
    kw = dict(max_seqs=3, max_step_tokens=64, max_chunk=8, global_kv_tokens=ctx + 17 + 1234 + 3 * 64, max_seq_len=ctx + 64, max_head_rows=24)
    prod, orc = _pair(w, E.Tuning(attn_keys_per_cta=keys_per_block), **kw)
    seqs = [prod.new_seq() for _ in range(3)]
    assert [orc.new_seq() for _ in range(3)] == seqs
    for i, (s, n) in enumerate(zip(seqs, (ctx, 17, 1234))):
        prod.bench_fill(s, n, seed=5 + i)
        orc.bench_fill(s, n, seed=5 + i)
    vocab = prod.desc.vocab
    rng = np.random.default_rng(ctx + keys_per_block)
    tol = TOL[int8_group]
    runs = [(s, rng.integers(0, vocab, c).astype(np.uint32), E.Rows.ALL, False) for s, c in zip(seqs, (5, 3, 5))]
    err = _logits_agree(prod, orc, runs, tol)
    assert list(prod.debug_read("attn_split")) [1] == splits
    same_state(prod, orc, 3, 13)
    # A draft tree per slot (rows: 0 root; 1, 2 children of 0; 3 child of 1; 4 child of 2; 5 child of 4), tokens arbitrary:
    # whatever path is accepted, the masks and the compaction that follows must be the oracle's.
    node = lambda depth, parent, sees: depth | parent << 8 | sees << 16
    tree = [oracle.chain_node(0), node(1, 0, 0b000011), node(1, 0, 0b000101), node(2, 1, 0b001011), node(2, 2, 0b010101), node(3, 4, 0b110101)]
    for s in seqs:
        first = int(orc.array("feed")[s * 16])
        feed = [first] + [int(x) for x in rng.integers(0, vocab, 5)]
        # Make rows 2 and 4 right where that is known: the token the target drew on row 0 is only known after the step,
        # so the accepted path is usually just the root; the tree mask itself is exercised either way.
        prod.debug_write("feed", s * 16, feed)
        orc.write("feed", s * 16, feed)
        prod.debug_write("tree", s * 16, tree)
        orc.write("tree", s * 16, tree)
    vruns = [(s, [E.FEED_ROW + i for i in range(6)], E.Rows.LAST, True) for s in seqs]
    err2 = _logits_agree(prod, orc, vruns, tol)
    same_state(prod, orc, 3, 18)
    print(f"{name} ctx {ctx}, {splits} splits: logits error {err:.2e} (chain) {err2:.2e} (tree)")
    prod.close()


def test_split_merge_with_four_heads_a_block_matches_the_oracle():
    """256 tokens x 8 heads: the split merge takes its four-heads-per-block form (as at 160 tokens x 32 heads),
    here over 32 sequences of 300 to 1200 filled positions and about five key splits."""
    w = util.weights("micro4", 0)
    kw = dict(max_seqs=32, max_step_tokens=256, max_chunk=8, global_kv_tokens=32 * 1280, max_seq_len=1280, max_head_rows=64)
    prod, orc = _pair(w, E.Tuning(attn_keys_per_cta=256), **kw)
    seqs = [prod.new_seq() for _ in range(32)]
    assert [orc.new_seq() for _ in range(32)] == seqs
    rng = np.random.default_rng(77)
    for i, s in enumerate(seqs):
        n = int(rng.integers(300, 1200))
        prod.bench_fill(s, n, seed=100 + i)
        orc.bench_fill(s, n, seed=100 + i)
    runs = [(s, rng.integers(0, 256, 8).astype(np.uint32), E.Rows.LAST if i % 2 else E.Rows.ALL if i < 4 else E.Rows.NONE, False) for i, s in enumerate(seqs)]
    err = _logits_agree(prod, orc, runs, TOL[0])
    sp = prod.debug_read("attn_split")
    assert 2 <= sp[1] <= 8
    same_state(prod, orc, 32, 256)
    print(f"256 tokens x 8 heads, {sp[1]} splits: logits error {err:.2e}")


# ---------------------------------------------------------------- one layer at the 1B model's dimensions
ONE_LAYER_1B = dict(synth.CONFIGS["1b"], n_layers=1)


@pytest.fixture(scope="module", params=[None, 0], ids=["bf16", "int8"])
def one_layer_1b(request, tmp_path_factory):
    path = tmp_path_factory.mktemp("w1b") / f"one_layer_1b_{request.param}.vlt"
    synth.write_target(path, ONE_LAYER_1B, seed=0, int8_group=request.param)
    yield path, request.param
    path.unlink()


def _bf16_ulp(x: float) -> float:
    """The spacing of bf16 values (8 significant bits) at magnitude x."""
    return float(2.0 ** (np.floor(np.log2(x)) - 7))


def _agree_at_scale(prod, orc, runs, tol):
    """At d 2048 and 128 256 ids the random-init model's logits have a standard deviation of 0.9 and reach +-5, where one
    unit in the last place of a bf16 value is 0.031. Two correct pipelines that round activations to bf16 between matmuls
    (the benchmark's convention) and add in different orders differ by about that much in their largest logits: a sum that
    moves by 1e-7 now and then rounds an activation the other way, and each of a layer's three rounding points (attention
    output, residual stream, SwiGLU output) turns a relative difference d into sqrt(d x ulp) -- measured here with
    vlt_step_capture: 1e-7 at the attention's output, 2e-4 after the o projection, 2e-3 after the MLP, whatever the
    attention kernel. So the bound is the stated tolerance or one bf16 unit at the largest logit, whichever is more, and
    the root-mean-square error must stay below 2^-7 of the logits' own (bf16's relative spacing at its widest; 0.4 to
    0.5 % is what these steps show)."""
    out = prod.debug_step(runs, E.StepOptions(read_logits=True))
    orc.step(runs)
    want = orc.array("logits").reshape(-1, prod.desc.vocab)
    assert out.logits.shape == want.shape and np.isfinite(out.logits).all()
    d = out.logits - want
    err, bound = float(np.abs(d).max()), max(tol, _bf16_ulp(float(np.abs(want).max())))
    rms = float(np.sqrt((d * d).mean()) / np.sqrt((want * want).mean()))
    assert err <= bound, f"logits max-abs error {err} (bound {bound})"
    assert rms <= 2.0 ** -7, f"logits rms error {rms} of their rms"
    top2 = np.sort(want, axis=1)[:, -2:]
    clear = top2[:, 1] - top2[:, 0] > max(1e-2, bound)
    assert np.array_equal(out.ids[clear], orc.array("out_ids")[clear])
    return err, rms


def _same_but_feed(prod, orc, n_runs, n_tokens):
    """Every integer of the step's state but `feed`, whose first entry per slot is a greedy token: that one is compared
    where the oracle's margin is clear (inside _agree_at_scale), and the product is put on the oracle's token for the next step."""
    same_state(prod, orc, n_runs, n_tokens, names=[x for x in STATE if x != "feed"])
    prod.debug_write("feed", 0, orc.array("feed"))


@pytest.mark.parametrize("filled", [True, False], ids=["filled-contexts", "empty-sequences"])
def test_one_layer_at_the_1b_dimensions_matches_the_oracle(one_layer_1b, filled):
    """32 sequences, with 600 to 900 filled positions each (a short version of the benchmark's contexts; several key
    splits) or empty (every row attends to at most 14 keys, where the bf16 rounding of the attention's probabilities in the
    tensor-core P.V -- fp32 in the reference and in the oracle -- weighs most): 256 tokens in a step, then 160 with every
    row through the head (the benchmark's verify step), then 5 tokens and 1 token of single sequences (the streamed
    matmul, four k slices on `down`)."""
    path, int8_group = one_layer_1b
    tol = TOL[int8_group]
    kw = dict(max_seqs=32, max_step_tokens=256, max_chunk=8, global_kv_tokens=32 * 960, max_seq_len=960, max_head_rows=160)
    prod, orc = _pair(path, **kw)
    seqs = [prod.new_seq() for _ in range(32)]
    assert [orc.new_seq() for _ in range(32)] == seqs
    vocab = prod.desc.vocab
    rng = np.random.default_rng(41)
    if filled:
        for i, s in enumerate(seqs):
            n = int(rng.integers(600, 900))
            prod.bench_fill(s, n, seed=300 + i)
            orc.bench_fill(s, n, seed=300 + i)
    runs = [(s, rng.integers(0, vocab, 8).astype(np.uint32), E.Rows.LAST if i % 4 == 0 else E.Rows.NONE, False) for i, s in enumerate(seqs)]
    e256 = _agree_at_scale(prod, orc, runs, tol)
    _same_but_feed(prod, orc, 32, 256)
    runs = [(s, rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False) for s in seqs]
    e160 = _agree_at_scale(prod, orc, runs, tol)
    assert orc.array("logits").size == 160 * vocab
    _same_but_feed(prod, orc, 32, 160)
    e5 = _agree_at_scale(prod, orc, [(seqs[3], rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False)], tol)
    e1 = _agree_at_scale(prod, orc, [(seqs[7], rng.integers(0, vocab, 1).astype(np.uint32), E.Rows.ALL, False)], tol)
    _same_but_feed(prod, orc, 1, 1)
    fmt = lambda e: f"{e[0]:.2e} max / {e[1]:.1e} rms"
    print(f"1B dims, int8_group={int8_group}, {'filled contexts' if filled else 'empty sequences'}: logits error {fmt(e256)} (256 tokens), {fmt(e160)} (160), {fmt(e5)} (5), {fmt(e1)} (1)")
    prod.close()


def test_head_gemm_in_paired_blocks_gives_the_one_block_per_sm_logits_bit_for_bit(one_layer_1b):
    """The head over 128 256 ids is 1002 tiles: by default two half-size blocks share an SM (one's fill and epilogue under
    the other's main loop). A tile's arithmetic and its order are the same either way, so the logits must be the same bits
    as with one block per SM (gemm_unpaired), at 160 rows and at 40."""
    path, int8_group = one_layer_1b
    if int8_group is None:
        pytest.skip("bf16 weights have no converter warps to halve: one block per SM always")
    kw = dict(max_seqs=32, max_step_tokens=160, max_chunk=8, global_kv_tokens=32 * 64, max_seq_len=64, max_head_rows=160)
    got = []
    for unpaired in (False, True):
        eng = E.Engine(path, E.EngineConfig(**kw), E.Tuning(gemm_unpaired=unpaired))
        seqs = [eng.new_seq() for _ in range(32)]
        rng = np.random.default_rng(8)
        vocab = eng.desc.vocab
        a = eng.debug_step([(s, rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False) for s in seqs], E.StepOptions(read_logits=True))
        b = eng.debug_step([(s, rng.integers(0, vocab, 5).astype(np.uint32), E.Rows.ALL, False) for s in seqs[:8]], E.StepOptions(read_logits=True))
        got.append((a.logits.copy(), b.logits.copy(), a.ids.copy(), b.ids.copy()))
        eng.close()
    assert got[0][0].shape == (160, 128256) and got[0][1].shape == (40, 128256)
    for x, y in zip(got[0], got[1]):
        assert np.array_equal(x.view(np.uint32), y.view(np.uint32))


# ---------------------------------------------------------------- the plumbing configuration as stated
def _plain_decode(w, prompt, n_tokens):
    """The oracle's one-token-at-a-time greedy decoding with each token's top-2 logit margin."""
    o = oracle.Engine(w, max_seqs=1, max_step_tokens=64, max_chunk=64, kv_tokens=1024, max_seq_len=1024, max_head_rows=8)
    q = o.new_seq()
    o.step([(q, prompt, E.Rows.LAST, False)])
    toks, margins = [], []
    for i in range(n_tokens):
        lg = np.sort(o.array("logits"))
        toks.append(int(o.array("feed")[0]))
        margins.append(float(lg[-1] - lg[-2]))
        if i + 1 < n_tokens:
            o.step([(q, [E.FEED_ROW], E.Rows.LAST, False)])
    return toks, margins


def _compare_stream(got, want, margins):
    """Equal up to the first token the oracle itself chose by less than 1e-2 (either choice is right there, and the
    streams may part ways after it). Returns how many tokens were compared."""
    for i, (g, w_) in enumerate(zip(got, want)):
        if g != w_:
            assert margins[i] <= 1e-2, f"token {i}: {g} vs {w_} with a top-2 margin of {margins[i]}"
            return i
    return min(len(got), len(want))


@pytest.mark.parametrize("draft", ["model", "replay"])
def test_plumbing_configuration_decodes_the_oracles_stream(draft, tmp_path):
    """2 layers, d 256, 4 q / 2 kv heads, FFN 1024, 4096 ids, bf16; a 64-token prompt of uniform random ids, greedy,
    k = 4 drafts a step (5 rows), 16-token pages; 128 decode steps' worth of tokens."""
    w = tmp_path / "tiny.vlt"
    synth.write_target(w, "tiny", seed=0)
    rng = np.random.default_rng(0)
    prompt = rng.integers(0, 4096, 64).astype(np.uint32)
    n_tokens = 128 if draft == "model" else 352  # 128 steps at one token a step (random-init drafts) / about 2.75 a step
    want, margins = _plain_decode(w, prompt, n_tokens)
    eng = E.Engine(w, E.EngineConfig(max_seqs=1, max_step_tokens=64, max_chunk=64, global_kv_tokens=1024, max_seq_len=1024, max_head_rows=8), E.Tuning(spec_policy_off=True))
    if draft == "model":
        d = tmp_path / "tiny_drafter.vlt"
        synth.write_drafter(d, "tiny", seed=100, draft_vocab=1024)
        eng.load_drafter(d)
        req = E.Request(list(prompt), n_tokens, draft=E.Draft.MODEL, rows=5)
    else:
        req = E.Request(list(prompt), n_tokens, draft=E.Draft.REPLAY, rows=5, trace=list(prompt) + want)
    got = []
    with eng.generator() as g:
        g.set_replay_mistakes(0.3, 9)
        g.submit(req)
        for _ in range(2000):
            if g.is_idle():
                break
            got += [ev.value for ev in g.step() if ev.kind == "token"]
        assert g.is_idle()
        stats = g.take_stats()
    assert len(got) == n_tokens
    compared = _compare_stream(got, want, margins)
    assert compared >= 64, f"only {compared} tokens before a near-tie"
    steps = sum(1 for s in stats if s["decode"])
    print(f"plumbing configuration, {draft} drafter: {compared} of {n_tokens} tokens compared, {steps} decode steps, {n_tokens / max(steps, 1):.2f} tokens a step")
    if draft == "replay" and compared == n_tokens:
        assert steps < n_tokens // 2  # drafts were accepted
