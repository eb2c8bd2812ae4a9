"""Random-init weight files for the benchmark configurations (no checkpoint or dataset is
needed: the decode step's speed and its parity against the oracle depend on shapes only).

A target file holds what the reference's converter writes (tools/convert.py:64-114), with
a plain decoder's tensor set: `embed` (bf16), optional int8 `head` (+ `head.scale`),
`L%02d.qkv|o|gate_up|down` (bf16, or int8 + `.scale`), `rope_freq` (f32) and a `meta`
descriptor (f32, as the reference's drafter file carries one: tools/spec/export.py:53).
gate_up rows are interleaved gate_0, up_0, gate_1, ... (tools/convert.py:102). RMSNorm gains
are folded into the following matrix's columns, as the reference folds its drafter's output
gain (tools/spec/export.py:50); at random init they are 1.
"""
from __future__ import annotations

from pathlib import Path

import numpy as np
import torch

from . import vlt

CONFIGS = {
    # Benchmark configuration 0: the plumbing check.
    "tiny": dict(n_layers=2, d=256, n_heads=4, n_kv=2, hd=64, ffn=1024, vocab=4096, eps=1e-5, theta=500000.0, page=16),
    # Benchmark configurations 2 to 4: the 1B target.
    "1b": dict(n_layers=16, d=2048, n_heads=32, n_kv=8, hd=64, ffn=8192, vocab=128256, eps=1e-5, theta=500000.0, page=16),
}
META_VERSION = 1.0
PRESET_LLAMA = 0.0
DRAFTER_KIND_CHAIN = 1.0


def meta_tensor(c: dict) -> np.ndarray:
    return np.array([META_VERSION, PRESET_LLAMA, c["n_layers"], c["d"], c["n_heads"], c["n_kv"], c["hd"], c["ffn"], c["vocab"],
                     c.get("vocab_real", c["vocab"]), c["eps"], c["page"], c["theta"], c.get("attn_scale", 1.0 / np.sqrt(c["hd"]))], dtype=np.float32)


def rope_freq(c: dict) -> np.ndarray:
    if "rope_freq" in c:  # given outright (the reference's target: (1 / 1024) ^ linspace(0, 1, 32), tools/spec/drafter.py:27)
        return np.asarray(c["rope_freq"], np.float32)
    i = np.arange(c["hd"] // 2, dtype=np.float64)
    return (c["theta"] ** (-2.0 * i / c["hd"])).astype(np.float32)


def _randn(gen: torch.Generator, m: int, k: int, std: float) -> np.ndarray:
    """N(0, std^2) rounded to bf16 (a checkpoint's weights are bf16), as fp32."""
    return (torch.randn(m, k, generator=gen) * std).to(torch.bfloat16).float().numpy()


def _put(out: dict, name: str, w: np.ndarray, group: int | None) -> None:
    if group is None:
        out[name] = vlt.Bf16.from_f32(w)
        return
    g = w.shape[1] if group == 0 else group  # 0: one scale per output row
    qs, ss = [], []
    for r0 in range(0, w.shape[0], 8192):
        q, s = vlt.quantize(w[r0:r0 + 8192], g)
        qs.append(q)
        ss.append(s.bits)
    out[name + ".scale"] = vlt.Bf16(np.concatenate(ss))
    out[name] = np.concatenate(qs)


def write_target(path, config: str | dict, seed: int = 0, int8_group: int | None = None, std: float = 0.02) -> dict:
    """int8_group: None keeps bf16; 0 quantises with one scale per output row; n with groups of n."""
    c = CONFIGS[config] if isinstance(config, str) else config
    gen = torch.Generator().manual_seed(seed)
    d, qkv_w = c["d"], (c["n_heads"] + 2 * c["n_kv"]) * c["hd"]
    out: dict = {"meta": meta_tensor(c), "rope_freq": rope_freq(c)}
    embed = _randn(gen, c["vocab"], d, std)
    out["embed"] = vlt.Bf16.from_f32(embed)
    if int8_group is not None:
        _put(out, "head", embed, int8_group)  # tied: the head is the quantised embedding
    del embed
    for i in range(c["n_layers"]):
        L = f"L{i:02d}."
        _put(out, L + "qkv", _randn(gen, qkv_w, d, std), int8_group)
        _put(out, L + "o", _randn(gen, d, c["n_heads"] * c["hd"], std), int8_group)
        _put(out, L + "gate_up", _randn(gen, 2 * c["ffn"], d, std), int8_group)
        _put(out, L + "down", _randn(gen, d, c["ffn"], std), int8_group)
    vlt.write(path, out)
    return c


def write_drafter(path, config: str | dict, seed: int = 100, int8_group: int | None = None, draft_vocab: int | None = None, std: float = 0.02,
                  window: int = 0) -> None:
    """The chain drafter: fc [d][2d] over (tapped hidden ; token embedding), one decoder layer
    `D00.*`, a head over a draft vocabulary of `draft_vocab` ids (`vocab`, ascending target
    ids stored as f32 like the reference's drafter file, tools/spec/export.py:51). With `window`,
    a draft pass attends to the last `window` keys of its context (down to a page boundary), as the
    reference's drafter layers attend to 1024 positions (tools/spec/drafter.py:17); the descriptor
    then has a fifth field."""
    c = CONFIGS[config] if isinstance(config, str) else config
    gen = torch.Generator().manual_seed(seed)
    d, qkv_w = c["d"], (c["n_heads"] + 2 * c["n_kv"]) * c["hd"]
    v = draft_vocab or c["vocab"]
    out: dict = {"meta": np.array([META_VERSION, DRAFTER_KIND_CHAIN, 1, v] + ([window] if window else []), dtype=np.float32)}
    _put(out, "fc", _randn(gen, d, 2 * d, std), int8_group)
    _put(out, "D00.qkv", _randn(gen, qkv_w, d, std), int8_group)
    _put(out, "D00.o", _randn(gen, d, c["n_heads"] * c["hd"], std), int8_group)
    _put(out, "D00.gate_up", _randn(gen, 2 * c["ffn"], d, std), int8_group)
    _put(out, "D00.down", _randn(gen, d, c["ffn"], std), int8_group)
    _put(out, "head", _randn(gen, v, d, std), int8_group)
    ids = np.sort(torch.randperm(c["vocab"], generator=gen)[:v].numpy()) if v < c["vocab"] else np.arange(v)
    out["vocab"] = ids.astype(np.float32)
    vlt.write(path, out)


def lcg_ids(n: int, seed: int, vocab: int) -> np.ndarray:
    """Deterministic pseudo-random token ids: the reference benchmark's generator
    (cli/src/bench.rs:47-56; a 64-bit LCG, `(x >> 33) % vocab`)."""
    mask = (1 << 64) - 1
    a, c = 6364136223846793005, 1442695040888963407
    x = (seed * a + c) & mask
    out = np.empty(n, np.uint32)
    for i in range(n):
        x = (x * a + c) & mask
        out[i] = (x >> 33) % vocab
    return out


# ------------------------------------------------------------------ the reference's block drafter
# tools/spec/drafter.py's model (fc over the tapped layers, inject, a mask embedding, layers with four two-tap
# convolutions each, a head over a draft vocabulary) as the file tools/spec/export.py writes. The reference fixes the
# shapes to its target's local layers (hidden 1280, 10 query / 2 kv heads of 128, FFN 3328); here the hidden width is
# a parameter (it has to be the target's), heads stay 128 wide with 2 kv heads.
BLOCK_HEAD_DIM, BLOCK_KV_HEADS, CONV_GROUP, CONV_ROWS = 128, 2, 16, 192


def block_drafter_state(seed: int = 0, hidden: int = 1280, ffn: int = 3328, layers: int = 2, taps=(35, 47), draft_vocab: int = 16384,
                        target_vocab: int = 151667) -> dict:
    """A random drafter with nothing at its initial zero or identity, in values bf16 keeps exactly (the recipe of
    tools/spec/check_engine.py:47-62 `random_drafter`, from numpy's generator), keyed like the reference module's
    state_dict so that the same arrays load into tools/spec/drafter.py `Drafter`."""
    rng = np.random.default_rng(seed)
    nq = hidden // BLOCK_HEAD_DIM

    def lin(m, k, std=None):  # nn.Linear's default range, halved, bf16-exact
        bound = 1.0 / np.sqrt(k)
        w = rng.uniform(-bound, bound, (m, k)) if std is None else rng.normal(0.0, std, (m, k))
        return vlt.from_bf16(vlt.to_bf16((0.5 * w).astype(np.float32)))

    def vec(x):
        return vlt.from_bf16(vlt.to_bf16((0.5 * np.asarray(x)).astype(np.float32)))

    sd = {"fc.weight": lin(hidden, len(taps) * hidden), "inject.weight": lin(hidden, hidden, 0.05), "mask_emb": vec(rng.normal(0.0, 0.02, hidden))}
    for i in range(layers):
        p = f"layers.{i}."
        for c in range(4):
            base = np.stack([np.ones(hidden), np.zeros(hidden)]) + rng.normal(0.0, 0.3, (2, hidden))
            sd[f"{p}convs.{c}.base"] = vec(base)
            sd[f"{p}convs.{c}.corr.weight"] = lin(2 * hidden // CONV_GROUP, hidden, 0.05)
        sd[p + "wq.weight"] = lin(nq * BLOCK_HEAD_DIM, hidden)
        sd[p + "wk.weight"] = lin(BLOCK_KV_HEADS * BLOCK_HEAD_DIM, hidden)
        sd[p + "wv.weight"] = lin(BLOCK_KV_HEADS * BLOCK_HEAD_DIM, hidden)
        sd[p + "wo.weight"] = lin(hidden, nq * BLOCK_HEAD_DIM)
        sd[p + "wgu.weight"] = lin(2 * ffn, hidden)
        sd[p + "wd.weight"] = lin(hidden, ffn)
    sd["head.weight"] = lin(draft_vocab, hidden)
    sd["out_gain"] = vec(rng.uniform(0.5, 1.5, hidden))
    sd["vocab"] = np.sort(rng.permutation(target_vocab)[:draft_vocab]).astype(np.int64)
    sd["_meta"] = dict(layers=layers, taps=tuple(taps), hidden=hidden, ffn=ffn)
    return sd


def write_block_drafter(path, sd: dict, int8: bool = False, block: int = 8, window: int = 1024) -> None:
    """tools/spec/export.py:17-55: fc split per tap, the layers' q | k | v stacked, every layer's k | v rows again as
    `kv_all` (the context goes through all of them at once), the convolutions' corrections padded to 192 rows, the
    output gain folded into the head's columns, `vocab` and `meta` as f32; matrices bf16, or int8 in groups of 64 (the
    head: 8)."""
    m = sd["_meta"]
    hidden, layers, taps = m["hidden"], m["layers"], m["taps"]
    out: dict = {}

    def matrix(name, w, group=64):
        _put(out, name, np.ascontiguousarray(w, np.float32), group if int8 else None)

    for k in range(len(taps)):
        matrix(f"fc.{k}", sd["fc.weight"][:, k * hidden:(k + 1) * hidden])
    out["mask_emb"] = np.ascontiguousarray(sd["mask_emb"], np.float32)
    matrix("inject", sd["inject.weight"])
    for i in range(layers):
        p = f"layers.{i}."
        matrix(f"D{i:02d}.qkv", np.concatenate([sd[p + "wq.weight"], sd[p + "wk.weight"], sd[p + "wv.weight"]]))
        matrix(f"D{i:02d}.o", sd[p + "wo.weight"])
        matrix(f"D{i:02d}.gate_up", sd[p + "wgu.weight"])
        matrix(f"D{i:02d}.down", sd[p + "wd.weight"])
        for c in range(4):
            out[f"D{i:02d}.conv{c}.base"] = np.ascontiguousarray(sd[f"{p}convs.{c}.base"], np.float32)
            corr = sd[f"{p}convs.{c}.corr.weight"]
            matrix(f"D{i:02d}.conv{c}.corr", np.concatenate([corr, np.zeros((CONV_ROWS - len(corr), hidden), np.float32)]))
    matrix("kv_all", np.concatenate([sd[f"layers.{i}.{w}.weight"] for i in range(layers) for w in ("wk", "wv")]))
    matrix("head", sd["head.weight"] * sd["out_gain"][None], 8)
    out["vocab"] = sd["vocab"].astype(np.float32)
    out["meta"] = np.array([layers, len(taps), block, window, len(sd["vocab"]), *taps], dtype=np.float32)
    vlt.write(path, out)


def block_case_inputs(seed: int, n_ctx: int, hidden: int = 1280, n_taps: int = 2):
    """Seeded inputs of one block-drafter case: the tapped features of `n_ctx` context positions
    ([n_ctx][n_taps][hidden], rms-normed and rounded to bf16 as the target's taps are) and the bonus token's
    embedding row ([hidden], bf16 values)."""
    rng = np.random.default_rng(seed)
    f = rng.normal(0.0, 1.0, (n_ctx, n_taps, hidden)).astype(np.float32)
    f = f / np.sqrt((f * f).mean(axis=-1, keepdims=True) + np.float32(2.0 ** -23))
    feat = vlt.from_bf16(vlt.to_bf16(f.astype(np.float32)))
    emb = vlt.from_bf16(vlt.to_bf16(rng.normal(0.0, 0.02, hidden).astype(np.float32)))
    return feat, emb


# ------------------------------------------------------------------ the reference's own architecture ("Limite")
def write_limite(path, n_layers: int = 48, hidden: int = 1280, n_kv: int = 2, ffn: int = 3328, vocab: int = 4096, vocab_real: int | None = None,
                 seed: int = 0, int8_group: int | None = None, std: float = 0.02) -> dict:
    """A random-init weight file with the tensor set tools/convert.py:64-114 writes for the reference's own model (no
    `meta`: the reference hard-codes the architecture, engine/src/model.rs:6-20): `embed`, `value_embed`, `rope_freq`
    (32 frequencies, (1 / 1024) ^ linspace(0, 1, 32)), `mudd.dense1`, `mudd.mix`, and per layer the four projections
    (gate_up interleaved) with `attn_gate`, `xsa` (tanh applied), `scalars` (qkv_scale, o_scale, the four residual
    lambdas, two zeros) and, on layers with i % 3 == 1, `ve_gate`. Heads are 128 wide, hidden / 128 of them; the
    reference's shapes are the defaults. `limite_vocab_real` (not in the reference's files, whose padding starts at
    151 667) names the first padding id of a smaller vocabulary."""
    gen = torch.Generator().manual_seed(seed)
    rng = np.random.default_rng(seed)
    d_head = 128
    nq = hidden // d_head
    qkv_w = (nq + 2 * n_kv) * d_head
    out: dict = {}
    embed = _randn(gen, vocab, hidden, std)
    out["embed"] = vlt.Bf16.from_f32(embed)
    out["value_embed"] = vlt.Bf16.from_f32(_randn(gen, vocab, n_kv * d_head, 0.5))
    out["rope_freq"] = ((1.0 / 1024.0) ** np.linspace(0, 1, 32, dtype=np.float32)).astype(np.float32)
    out["mudd.dense1"] = rng.normal(0.0, 0.05, (32, hidden)).astype(np.float32)
    mix = rng.normal(0.0, 0.3, (2, 2, 3, 33)).astype(np.float32)
    mix[:, :, :, 32] = np.array([0.1, 0.2, 0.9], np.float32) + rng.normal(0.0, 0.05, (2, 2, 3)).astype(np.float32)
    out["mudd.mix"] = mix
    for i in range(n_layers):
        L = f"L{i:02d}."
        _put(out, L + "qkv", _randn(gen, qkv_w, hidden, std), int8_group)
        _put(out, L + "o", _randn(gen, hidden, hidden, std), int8_group)
        _put(out, L + "gate_up", _randn(gen, 2 * ffn, hidden, std), int8_group)
        _put(out, L + "down", _randn(gen, hidden, ffn, std), int8_group)
        out[L + "attn_gate"] = rng.normal(0.0, 0.1, (nq, d_head)).astype(np.float32)
        if i % 3 == 1:
            out[L + "ve_gate"] = rng.normal(0.0, 0.3, (n_kv, 12)).astype(np.float32)
        out[L + "xsa"] = np.tanh(rng.normal(0.0, 0.5, nq)).astype(np.float32)
        out[L + "scalars"] = np.concatenate([rng.uniform(0.8, 1.2, 6), [0.0, 0.0]]).astype(np.float32)
    if int8_group is not None:
        _put(out, "head", embed, 8 if int8_group else 0)
    if vocab_real is not None:
        out["limite_vocab_real"] = np.array([vocab_real], np.float32)
    vlt.write(path, out)
    return dict(n_layers=n_layers, d=hidden, n_heads=nq, n_kv=n_kv, hd=d_head, ffn=ffn, vocab=vocab, vocab_real=vocab_real or vocab)
