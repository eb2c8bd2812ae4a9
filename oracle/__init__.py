"""ctypes binding of the CPU oracle (oracle/_ref/liboracle.so).

Test infrastructure only: the tests, the smoke check and the benchmark's CPU-baseline leg
import this; nothing in the product package does. Parity status of the oracle: unpinned
(see oracle/bits.hpp) except for the weight file layout and the int8 quantiser, which are
pinned by tests/golden against the reference's tools/convert.py.
"""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "_ref" / "liboracle.so"

FEED_ROW = 0xFFFF0000
FEED_W = 16
NO_TOK = 0xFFFFFFFF
ROWS_NONE, ROWS_LAST, ROWS_ALL = 0, 1, 2

SAMPLE_ROW = np.dtype([("seed_lo", "<u4"), ("seed_hi", "<u4"), ("pos", "<u4"), ("temperature", "<f4"), ("top_p", "<f4"), ("tok", "<u4")])
RUN_IN = np.dtype([("slot", "<u4"), ("first", "<u4"), ("count", "<u4"), ("head0", "<u4"), ("nhead", "<u4"), ("verify", "<u4")])
GEN_STATE = np.dtype([("remaining", "<u4"), ("done", "<u4"), ("nstop", "<u4"), ("pad", "<u4"), ("stop", "<u4", (8,))])


def build() -> Path:
    """Compiles the oracle with its Makefile (g++, OpenMP)."""
    subprocess.run(["make", "-s", "-C", str(HERE)], check=True)
    return LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            build()
        _lib = C.CDLL(str(LIB_PATH))
        _lib.orc_last_error.restype = C.c_char_p
        _lib.orc_uniform01.restype = C.c_float
        _lib.orc_chain_node.restype = C.c_uint32
        _lib.orc_dead_node.restype = C.c_uint32
        _lib.orc_vlt_load.restype = C.c_void_p
        _lib.orc_vlt_tensor.restype = C.c_void_p
        _lib.orc_vlt_count.restype = C.c_uint32
        _lib.orc_engine_new.restype = C.c_void_p
        _lib.orc_seq_len.restype = C.c_uint32
        _lib.orc_array.restype = C.c_uint64
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def _err() -> str:
    return lib().orc_last_error().decode()


def philox(counter, key) -> np.ndarray:
    c = np.asarray(counter, dtype=np.uint32)
    k = np.asarray(key, dtype=np.uint32)
    out = np.zeros(4, np.uint32)
    lib().orc_philox(_p(c), _p(k), _p(out))
    return out


def uniform01(seed: int, pos: int, rnd: int) -> float:
    return float(lib().orc_uniform01(C.c_uint32(seed & 0xFFFFFFFF), C.c_uint32(seed >> 32), C.c_uint32(pos), C.c_uint32(rnd)))


def exp2(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty_like(x)
    lib().orc_exp2(_p(x), _p(y), C.c_uint64(x.size))
    return y


def to_bf16(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    y = np.empty(x.shape, np.uint16)
    lib().orc_to_bf16(_p(x), _p(y), C.c_uint64(x.size))
    return y


def rope(x: np.ndarray, pos, freq):
    """x [rows][hd] -> (rotated, cos/sin table [rows][hd/2][2])."""
    x = np.ascontiguousarray(x, np.float32)
    rows, hd = x.shape
    pos = np.ascontiguousarray(pos, np.uint32)
    freq = np.ascontiguousarray(freq, np.float32)
    y = np.empty_like(x)
    cs = np.empty((rows, hd // 2, 2), np.float32)
    lib().orc_rope(_p(x), C.c_uint32(rows), C.c_uint32(hd), _p(pos), _p(freq), _p(y), _p(cs))
    return y, cs


def chain_node(row: int) -> int:
    return int(lib().orc_chain_node(C.c_uint32(row)))


def dead_node(row: int) -> int:
    return int(lib().orc_dead_node(C.c_uint32(row)))


def quantize(w: np.ndarray, group: int):
    w = np.ascontiguousarray(w, np.float32)
    m, k = w.shape
    q = np.empty((m, k), np.int8)
    s = np.empty((m, k // group), np.uint16)
    lib().orc_quantize(_p(w), C.c_uint32(m), C.c_uint32(k), C.c_uint32(group), _p(q), _p(s))
    return q, s


_NP_DTYPES = {0: np.float32, 1: np.uint16, 2: np.int8}


def vlt_read(path) -> dict[str, tuple[int, np.ndarray]]:
    """name -> (dtype code, array); bf16 tensors come back as uint16 bit patterns."""
    h = lib().orc_vlt_load(str(path).encode())
    if not h:
        raise RuntimeError(_err())
    h = C.c_void_p(h)
    out = {}
    try:
        for i in range(lib().orc_vlt_count(h)):
            name = C.create_string_buffer(64)
            dtype, ndim = C.c_uint32(), C.c_uint32()
            shape = (C.c_uint32 * 4)()
            off, nb = C.c_uint64(), C.c_uint64()
            ptr = lib().orc_vlt_tensor(h, C.c_uint32(i), name, C.byref(dtype), C.byref(ndim), shape, C.byref(off), C.byref(nb))
            raw = C.string_at(ptr, nb.value)
            arr = np.frombuffer(raw, dtype=_NP_DTYPES[dtype.value]).reshape([shape[j] for j in range(ndim.value)]).copy()
            out[name.value.decode()] = (dtype.value, arr, off.value)
    finally:
        lib().orc_vlt_free(h)
    return out


def vlt_write(path, tensors: dict[str, tuple[int, np.ndarray]]) -> None:
    n = len(tensors)
    names = (C.c_char_p * n)(*[k.encode() for k in tensors])
    arrs = [np.ascontiguousarray(a) for _, a in tensors.values()]
    dtypes = (C.c_uint32 * n)(*[d for d, _ in tensors.values()])
    ndims = (C.c_uint32 * n)(*[a.ndim for a in arrs])
    shapes = (C.c_uint32 * (4 * n))()
    for i, a in enumerate(arrs):
        for j, s in enumerate(a.shape):
            shapes[4 * i + j] = s
    ptrs = (C.c_void_p * n)(*[a.ctypes.data for a in arrs])
    nbytes = (C.c_uint64 * n)(*[a.nbytes for a in arrs])
    if lib().orc_vlt_write(str(path).encode(), C.c_uint32(n), names, dtypes, ndims, shapes, ptrs, nbytes):
        raise RuntimeError(_err())


def sample(logits: np.ndarray, rows: np.ndarray, meta: np.ndarray | None = None) -> np.ndarray:
    logits = np.ascontiguousarray(logits, np.float32)
    rows = np.ascontiguousarray(rows, SAMPLE_ROW)
    n, vocab = logits.shape
    out = np.zeros(n, np.uint32)
    m = np.ascontiguousarray(meta, np.uint32) if meta is not None else np.zeros(2, np.uint32)
    lib().orc_sample(_p(logits), C.c_uint32(vocab), _p(rows), C.c_uint32(n), _p(m), _p(out))
    return out


def accept(runs, tokens, out, lens, feed, gen, tree):
    """Runs `accept` in place on out/lens/feed/gen; returns (emitted, path, path_len, on_path)."""
    runs = np.ascontiguousarray(runs, RUN_IN)
    n = len(runs)
    emitted = np.zeros(n, np.uint32)
    path = np.zeros(n * FEED_W, np.uint32)
    path_len = np.zeros(n, np.uint32)
    on_path = np.zeros(len(tokens), np.uint32)
    lib().orc_accept(_p(runs), C.c_uint32(n), _p(tokens), _p(out), _p(lens), _p(feed), _p(gen), _p(emitted), _p(tree), _p(path), _p(path_len), _p(on_path))
    return emitted, path, path_len, on_path


def replay_draft(runs, lens, feed, trace, trace_len, stride, seed, rate, vocab, tree):
    runs = np.ascontiguousarray(runs, RUN_IN)
    lib().orc_replay_draft(_p(runs), C.c_uint32(len(runs)), _p(lens), _p(feed), _p(trace), _p(trace_len), C.c_uint32(stride), C.c_uint32(seed),
                           C.c_float(rate), C.c_uint32(vocab), _p(tree))


def draft_top(logits, vocab_ids, tin, inv_t, ncand):
    logits = np.ascontiguousarray(logits, np.float32)
    n, nv = logits.shape
    cand = np.zeros((n, 4), np.uint32)
    cand_q = np.zeros((n, 4), np.float32)
    vid = np.ascontiguousarray(vocab_ids, np.uint32)
    tin = np.ascontiguousarray(tin, np.uint32)
    lib().orc_draft_top(_p(logits), C.c_uint32(n), C.c_uint32(nv), _p(vid), _p(tin), C.c_float(inv_t), C.c_uint32(ncand), _p(cand), _p(cand_q))
    return cand, cand_q


def draft_tree(blocks, tin, cand, cand_q, ncand, feed, tree):
    blocks = np.ascontiguousarray(blocks, np.uint32)
    tin = np.ascontiguousarray(tin, np.uint32)
    lib().orc_draft_tree(_p(blocks), C.c_uint32(len(blocks) // 2), _p(tin), _p(np.ascontiguousarray(cand, np.uint32)), _p(np.ascontiguousarray(cand_q, np.float32)),
                         C.c_uint32(ncand), _p(feed), _p(tree))


def spec_accept(p, q, drafts, temperature, seeds, pos0):
    """p [S][k+1][V], q [S][k][V] bf16 bit patterns (uint16); returns accepted, token, rollback."""
    p = np.ascontiguousarray(p, np.uint16)
    q = np.ascontiguousarray(q, np.uint16)
    s, k, v = q.shape
    drafts = np.ascontiguousarray(drafts, np.uint32)
    seeds = np.ascontiguousarray(seeds, np.uint64)
    pos0 = np.ascontiguousarray(pos0, np.uint32)
    acc, tok, rb = (np.zeros(s, np.uint32) for _ in range(3))
    lib().orc_spec_accept(_p(p), _p(q), _p(drafts), C.c_uint32(s), C.c_uint32(k), C.c_uint32(v), C.c_float(temperature), _p(seeds), _p(pos0), _p(acc), _p(tok), _p(rb))
    return acc, tok, rb


def draw_drafts(q, temperature, seeds, pos0):
    q = np.ascontiguousarray(q, np.uint16)
    s, k, v = q.shape
    seeds = np.ascontiguousarray(seeds, np.uint64)
    pos0 = np.ascontiguousarray(pos0, np.uint32)
    out = np.zeros((s, k), np.uint32)
    lib().orc_draw_drafts(_p(q), C.c_uint32(s), C.c_uint32(k), C.c_uint32(v), C.c_float(temperature), _p(seeds), _p(pos0), _p(out))
    return out


def set_threads(n: int) -> int:
    """OpenMP threads the oracle uses from now on; returns the number in effect."""
    lib().orc_set_threads(C.c_int(int(n)))
    return int(lib().orc_max_threads())


class OrcConfig(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("max_seqs", "max_step_tokens", "max_chunk", "kv_tokens", "max_seq_len", "max_head_rows")]


class Engine:
    """The oracle's engine: same calls as the product's, on host memory."""

    def __init__(self, path, max_seqs=8, max_step_tokens=512, max_chunk=512, kv_tokens=65536, max_seq_len=131072, max_head_rows=64):
        cfg = OrcConfig(max_seqs, max_step_tokens, max_chunk, kv_tokens, max_seq_len, max_head_rows)
        h = lib().orc_engine_new(str(path).encode(), C.byref(cfg))
        if not h:
            raise RuntimeError(_err())
        self.h = C.c_void_p(h)
        d = (C.c_uint32 * 12)()
        lib().orc_model_desc(self.h, d)
        names = ("n_layers", "d", "n_heads", "n_kv", "hd", "ffn", "vocab", "vocab_real", "page")
        self.desc = {n: int(d[i]) for i, n in enumerate(names)}
        self.n_pages = int(d[11])

    def close(self):
        if self.h:
            lib().orc_engine_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def new_seq(self) -> int:
        i = C.c_uint32()
        if lib().orc_seq_new(self.h, C.byref(i)):
            raise RuntimeError(_err())
        return i.value

    def free_seq(self, s: int):
        lib().orc_seq_free(self.h, C.c_uint32(s))

    def seq_len(self, s: int) -> int:
        return int(lib().orc_seq_len(self.h, C.c_uint32(s)))

    def settle(self, s: int, unused: int):
        lib().orc_seq_settle(self.h, C.c_uint32(s), C.c_uint32(unused))

    def set_sampling(self, s: int, temperature=0.0, top_p=1.0, seed=0):
        if lib().orc_seq_set_sampling(self.h, C.c_uint32(s), C.c_float(temperature), C.c_float(top_p), C.c_uint64(seed)):
            raise RuntimeError(_err())

    def bench_fill(self, s: int, n: int, seed: int = 0):
        """Advances a sequence without computing it; seed != 0 fills the new positions' K/V with the hashed values
        the CUDA engine's bench_fill writes for the same seed."""
        if lib().orc_bench_fill(self.h, C.c_uint32(s), C.c_uint32(n), C.c_uint32(seed)):
            raise RuntimeError(_err())

    def set_gen(self, slot: int, remaining: int, stop=()):
        st = np.asarray(list(stop), np.uint32)
        lib().orc_set_gen(self.h, C.c_uint32(slot), C.c_uint32(remaining), _p(st), C.c_uint32(len(st)))

    def set_trace(self, slot: int, trace):
        t = np.ascontiguousarray(trace, np.uint32)
        lib().orc_set_trace(self.h, C.c_uint32(slot), _p(t), C.c_uint32(len(t)))

    def set_replay(self, rate: float, seed: int):
        lib().orc_set_replay(self.h, C.c_float(rate), C.c_uint32(seed))

    def set_capture(self, on: bool):
        """Keep every layer's intermediates of the next steps (arrays cap_resid_in, cap_attn_in, cap_qkv, cap_sdpa_out,
        cap_attn_out, cap_mlp_in, cap_mlp_out: [layer][n][width])."""
        lib().orc_set_capture(self.h, C.c_uint32(int(on)))

    def set_taps(self, layers):
        a = np.ascontiguousarray(list(layers), np.uint32)
        lib().orc_set_taps(self.h, _p(a), C.c_uint32(a.size))

    def set_acceptance(self, rule: int):
        """0: the reference's sample-then-match; 1: rejection sampling where a run's drafts came with their q rows."""
        lib().orc_set_acceptance(self.h, C.c_uint32(rule))

    def load_drafter(self, path):
        if lib().orc_load_drafter(self.h, str(path).encode()):
            raise RuntimeError(_err())

    def step(self, runs, hidden=ROWS_NONE, plan_only=False, replay=False, draft_rows=0):
        """runs: list of (seq, tokens, head Rows, verify bool). draft_rows: the chain drafter proposes for that many rows."""
        seq = np.asarray([r[0] for r in runs], np.uint32)
        count = np.asarray([len(r[1]) for r in runs], np.uint32)
        heads = np.asarray([r[2] for r in runs], np.uint32)
        verify = np.asarray([1 if r[3] else 0 for r in runs], np.uint32)
        toks = np.concatenate([np.asarray(r[1], np.uint32) for r in runs]) if runs else np.zeros(0, np.uint32)
        mode = (1 if plan_only else 0) | (2 if replay else 0) | (int(draft_rows) << 8)
        if lib().orc_step(self.h, C.c_uint32(len(runs)), _p(seq), _p(count), _p(verify), _p(heads), _p(toks), C.c_uint32(hidden), C.c_uint32(mode)):
            raise RuntimeError(_err())

    def write(self, name: str, index: int, data):
        d = np.ascontiguousarray(data, np.uint32)
        if lib().orc_array_write(self.h, name.encode(), C.c_uint64(index), _p(d), C.c_uint64(d.size)):
            raise RuntimeError(_err())

    _F32 = ("logits", "hidden_out", "taps", "draft_logits", "carry", "q_keep", "taps_all", "cap_resid_in", "cap_attn_in", "cap_qkv", "cap_sdpa_out", "cap_attn_out",
            "cap_mlp_in", "cap_mlp_out", "block_logits", "block_hfin", "block_ctx_ring")
    _U16 = ("k_cache", "v_cache", "draft_k_cache", "draft_v_cache", "block_k_ring", "block_v_ring", "limite_k_local", "limite_v_local")

    def array(self, name: str) -> np.ndarray:
        ptr = C.c_void_p()
        n = lib().orc_array(self.h, name.encode(), C.byref(ptr))
        if not ptr.value:
            return np.zeros(0, np.uint32)
        dt = np.float32 if name in self._F32 else np.uint16 if name in self._U16 else np.uint32
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(n * np.dtype(dt).itemsize,)).view(dt).copy()


class BlockDrafter:
    """block_drafter.hpp stand-alone: the reference's block drafter (tools/spec/drafter.py as engine/src/engine/drafter.rs
    runs it) on features and blocks the caller supplies."""
    _U16 = ("k_ring", "v_ring")
    _U32 = ("vocab",)

    def __init__(self, path, eps: float, scale: float, rope_freq, max_seqs: int = 1, max_chunk: int = 64):
        f = lib()
        f.orc_block_new.restype = C.c_void_p
        f.orc_block_array.restype = C.c_uint64
        freq = np.ascontiguousarray(rope_freq, np.float32)
        assert freq.size == 32
        self.h = C.c_void_p(f.orc_block_new(str(path).encode(), C.c_float(eps), C.c_float(scale), _p(freq), C.c_uint32(max_seqs), C.c_uint32(max_chunk)))
        if not self.h.value:
            raise RuntimeError(_err())
        d = np.zeros(8, np.uint32)
        f.orc_block_desc(self.h, _p(d))
        self.n_layers, self.n_taps, self.block, self.window, self.v, self.hidden, self.ffn, self.ring = (int(x) for x in d)

    def close(self):
        if self.h.value:
            lib().orc_block_free(self.h)
            self.h = C.c_void_p()

    def context(self, taps, meta, on_path=None):
        """taps [n_taps][n][hidden] fp32 holding bf16 values; meta [n][2] (slot, position)."""
        taps = np.ascontiguousarray(taps, np.float32)
        meta = np.ascontiguousarray(meta, np.uint32)
        n = taps.shape[1]
        op = None if on_path is None else np.ascontiguousarray(on_path, np.uint32)
        if lib().orc_block_context(self.h, C.c_uint32(n), _p(taps), _p(meta), None if op is None else _p(op)):
            raise RuntimeError(_err())

    def run(self, slots, rows, p0, bonus_rows):
        """Blocks (slot, rows, the bonus token's position) with the bonus tokens' embedding rows [blocks][hidden] as bf16 bits."""
        slots, rows, p0 = (np.ascontiguousarray(x, np.uint32) for x in (slots, rows, p0))
        bonus = np.ascontiguousarray(bonus_rows, np.uint16)
        if lib().orc_block_run(self.h, C.c_uint32(len(slots)), _p(slots), _p(rows), _p(p0), _p(bonus)):
            raise RuntimeError(_err())

    def array(self, name: str) -> np.ndarray:
        ptr = C.c_void_p()
        n = lib().orc_block_array(self.h, name.encode(), C.byref(ptr))
        if not ptr.value:
            return np.zeros(0, np.float32)
        dt = np.uint16 if name in self._U16 else np.uint32 if name in self._U32 else np.float32
        return np.ctypeslib.as_array(C.cast(ptr, C.POINTER(C.c_uint8)), shape=(n * np.dtype(dt).itemsize,)).view(dt).copy()
