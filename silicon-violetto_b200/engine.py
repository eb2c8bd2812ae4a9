"""ctypes mirror of the reference's public API (`violetto::{Engine, Generator, ...}`,
engine/src/lib.rs:6-10) over libvioletto_b200.so's C ABI (include/violetto.h).

Names, argument meaning and error behaviour follow the reference: a failing call raises
`EngineError` with the message the Rust API would return in `Err(String)`. There is no CPU
path: the library must be built (`build.build()`) and, except for host-only planning
engines, a CUDA device must be present.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
LIB_PATH = HERE / "libvioletto_b200.so"

FEED_ROW = 0xFFFF0000
FEED_W = 16
NO_TOK = 0xFFFFFFFF
VERIFY_T = 8
FLAG_HOST_ONLY = 1


class EngineError(RuntimeError):
    pass


class Rows:
    NONE, LAST, ALL = 0, 1, 2


class _Config(C.Structure):
    _fields_ = [("max_seqs", C.c_uint32), ("max_step_tokens", C.c_uint32), ("max_chunk", C.c_uint32), ("global_kv_tokens", C.c_uint32),
                ("max_seq_len", C.c_uint32), ("max_head_rows", C.c_uint32), ("device_ordinal", C.c_int32), ("flags", C.c_uint32)]


class _Tuning(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("spec_tokens", "spec_tokens_short", "spec_kv", "spec_rows_long", "spec_policy_off", "sm_count",
                                          "attn_keys_per_cta", "gemm_min_rows", "plain_attention", "gemm_unpaired")]


class _Sampling(C.Structure):
    _fields_ = [("temperature", C.c_float), ("top_p", C.c_float), ("seed", C.c_uint64)]


class _Run(C.Structure):
    _fields_ = [("seq", C.c_uint32), ("tokens", C.POINTER(C.c_uint32)), ("n_tokens", C.c_uint32)]


class _StepOptions(C.Structure):
    _fields_ = [("head", C.c_uint32), ("hidden", C.c_uint32), ("read_logits", C.c_uint32), ("read_taps", C.c_uint32)]


class _StepOutput(C.Structure):
    _fields_ = [("ids", C.POINTER(C.c_uint32)), ("ids_cap", C.c_uint32), ("n_ids", C.c_uint32), ("logits", C.POINTER(C.c_float)), ("logits_cap", C.c_uint64),
                ("hidden", C.POINTER(C.c_float)), ("hidden_cap", C.c_uint64), ("n_hidden", C.c_uint32), ("taps", C.POINTER(C.c_uint16)),
                ("taps_cap", C.c_uint64), ("gpu_seconds", C.c_double), ("n_taps", C.c_uint32)]


class _LayerCapture(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("layer", "n", "d_model", "qkv_width", "attn_width")] + \
               [(n, C.POINTER(C.c_float)) for n in ("resid_in", "attn_in", "qkv", "sdpa_out", "attn_out", "mlp_in", "mlp_out", "resid_base")]


_CAPTURE_FN = C.CFUNCTYPE(None, C.POINTER(_LayerCapture), C.c_void_p)


class _ModelDesc(C.Structure):
    _fields_ = [(n, C.c_uint32) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "ffn", "vocab", "vocab_real", "page_size")] + \
               [("rms_eps", C.c_float), ("attn_scale", C.c_float), ("int8", C.c_uint32)]


class _Request(C.Structure):
    _fields_ = [("prompt_kind", C.c_uint32), ("prompt_tokens", C.POINTER(C.c_uint32)), ("n_prompt", C.c_uint32), ("resume_seq", C.c_uint32),
                ("resume_token", C.c_uint32), ("max_tokens", C.c_uint32), ("stop", C.POINTER(C.c_uint32)), ("n_stop", C.c_uint32),
                ("sampling", _Sampling), ("draft_kind", C.c_uint32), ("draft_rows", C.c_uint32), ("trace", C.POINTER(C.c_uint32)), ("n_trace", C.c_uint32)]


class _Event(C.Structure):
    _fields_ = [("kind", C.c_uint32), ("req", C.c_uint32), ("value", C.c_uint32)]


class _StepStats(C.Structure):
    _fields_ = [("tokens", C.c_uint32), ("decode", C.c_uint32), ("emitted", C.c_uint32), ("gpu_seconds", C.c_double), ("encode_seconds", C.c_double)]


_lib = None


def lib() -> C.CDLL:
    """The product library. Fails loudly if it has not been built: there is no fallback."""
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise EngineError(f"{LIB_PATH} is missing: build it with silicon_violetto_b200.build.build() (nvcc, sm_100a)")
        _lib = C.CDLL(str(LIB_PATH))
        _lib.vlt_last_error.restype = C.c_char_p
        _lib.vlt_seq_len.restype = C.c_uint32
    return _lib


def _check(rc: int) -> None:
    if rc != 0:
        raise EngineError(lib().vlt_last_error().decode())


def _u32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.uint32)


def _ptr(a: np.ndarray, t=C.c_uint32):
    return a.ctypes.data_as(C.POINTER(t))


@dataclass
class EngineConfig:
    """engine/src/engine.rs:31-57."""
    max_seqs: int = 8
    max_step_tokens: int = 512
    max_chunk: int = 512
    global_kv_tokens: int = 65536
    max_seq_len: int = 131072
    max_head_rows: int = 64
    device_ordinal: int = 0
    host_only: bool = False


@dataclass
class Tuning:
    """engine/src/engine.rs:59-95 (rows policy) plus the B200 knobs; 0 means the default."""
    spec_tokens: int = 0
    spec_tokens_short: int = 0
    spec_kv: int = 0
    spec_rows_long: int = 0
    spec_policy_off: bool = False
    sm_count: int = 0
    attn_keys_per_cta: int = 0
    gemm_min_rows: int = 0
    plain_attention: bool = False
    gemm_unpaired: bool = False


@dataclass
class Sampling:
    """engine/src/engine.rs:100-138."""
    temperature: float = 0.0
    top_p: float = 1.0
    seed: int = 0

    def c(self) -> _Sampling:
        return _Sampling(self.temperature, self.top_p, self.seed)


GREEDY = Sampling()


@dataclass
class Run:
    seq: int
    tokens: list


@dataclass
class StepOptions:
    head: int = Rows.LAST
    hidden: int = Rows.NONE
    read_logits: bool = False
    read_taps: bool = False


@dataclass
class StepOutput:
    ids: np.ndarray
    logits: np.ndarray
    hidden: np.ndarray
    taps: np.ndarray
    gpu_seconds: float


class Engine:
    """engine/src/engine.rs `Engine`."""

    def __init__(self, weights, cfg: EngineConfig | None = None, tuning: Tuning | None = None):
        cfg = cfg or EngineConfig()
        t = tuning or Tuning()
        c = _Config(cfg.max_seqs, cfg.max_step_tokens, cfg.max_chunk, cfg.global_kv_tokens, cfg.max_seq_len, cfg.max_head_rows, cfg.device_ordinal,
                    FLAG_HOST_ONLY if cfg.host_only else 0)
        ct = _Tuning(t.spec_tokens, t.spec_tokens_short, t.spec_kv, t.spec_rows_long, int(t.spec_policy_off), t.sm_count, t.attn_keys_per_cta,
                     t.gemm_min_rows, int(t.plain_attention), int(t.gemm_unpaired))
        self.h = C.c_void_p()
        self.cfg = cfg
        _check(lib().vlt_engine_new(str(weights).encode(), C.byref(c), C.byref(ct), C.byref(self.h)))
        d = _ModelDesc()
        _check(lib().vlt_model_desc(self.h, C.byref(d)))
        self.desc = d

    def close(self) -> None:
        if getattr(self, "h", None):
            lib().vlt_engine_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:  # at interpreter shutdown the module's globals may already be gone
            pass

    def device_name(self) -> str:
        buf = C.create_string_buffer(256)
        _check(lib().vlt_device_name(self.h, buf, C.c_size_t(256)))
        return buf.value.decode()

    def new_seq(self) -> int:
        s = C.c_uint32()
        _check(lib().vlt_seq_new(self.h, C.byref(s)))
        return s.value

    def free_seq(self, seq: int) -> None:
        lib().vlt_seq_free(self.h, C.c_uint32(seq))

    def seq_len(self, seq: int) -> int:
        return int(lib().vlt_seq_len(self.h, C.c_uint32(seq)))

    def set_sampling(self, seq: int, s: Sampling) -> None:
        cs = s.c()
        _check(lib().vlt_seq_set_sampling(self.h, C.c_uint32(seq), C.byref(cs)))

    def set_taps(self, layers) -> None:
        """engine.rs:381-389: tap these layers' outputs from the next step on (StepOptions.read_taps)."""
        a = _u32(list(layers))
        _check(lib().vlt_set_taps(self.h, _ptr(a), C.c_uint32(a.size)))
        self._taps = [int(x) for x in a]

    def set_acceptance(self, rule: int) -> None:
        """0: the reference's sample-then-match `accept`; 1: rejection sampling for runs whose drafts the chain drafter drew."""
        _check(lib().vlt_set_acceptance(self.h, C.c_uint32(rule)))

    def load_drafter(self, path) -> None:
        _check(lib().vlt_load_drafter(self.h, str(path).encode()))

    def set_draft_rows(self, rows: int) -> None:
        """debug_step then runs the loaded drafter for `rows` rows (rows - 1 drafts) after each step; 0: not."""
        lib().vlt_debug_set_draft_rows(self.h, C.c_uint32(rows))

    def debug_stalled_wait(self) -> None:
        """Queues a kernel whose bounded wait runs out on purpose: the next collected step raises, the engine carries on."""
        _check(lib().vlt_debug_stalled_wait(self.h))

    def force_logits(self, logits=None, draft_logits=None) -> None:
        """The next debug_step's sampler / acceptance / drafter pick read these instead of the logits it computed."""
        a = None if logits is None else np.ascontiguousarray(logits, np.float32)
        b = None if draft_logits is None else np.ascontiguousarray(draft_logits, np.float32)
        _check(lib().vlt_debug_force_logits(self.h, None if a is None else _ptr(a, C.c_float), C.c_uint64(0 if a is None else a.size),
                                            None if b is None else _ptr(b, C.c_float), C.c_uint64(0 if b is None else b.size)))

    def has_drafter(self) -> bool:
        return bool(lib().vlt_has_drafter(self.h))

    def _runs(self, runs):
        keep = [_u32(r.tokens if isinstance(r, Run) else r[1]) for r in runs]
        arr = (_Run * len(runs))()
        for i, r in enumerate(runs):
            arr[i] = _Run(r.seq if isinstance(r, Run) else r[0], _ptr(keep[i]), len(keep[i]))
        return arr, keep

    def _out(self, n_tokens: int, opts: StepOptions):
        d = self.desc
        rows = self.cfg.max_head_rows
        ids = np.zeros(rows, np.uint32)
        logits = np.zeros(rows * d.vocab if opts.read_logits else 0, np.float32)
        hidden = np.zeros(n_tokens * d.d_model if opts.hidden != Rows.NONE else 0, np.float32)
        n_taps = len(getattr(self, "_taps", [])) + 1  # (+1: a loaded drafter keeps the last layer tapped)
        taps = np.zeros(n_taps * n_tokens * d.d_model if opts.read_taps else 0, np.uint16)
        out = _StepOutput(_ptr(ids), rows, 0, _ptr(logits, C.c_float), logits.size, _ptr(hidden, C.c_float), hidden.size, 0, _ptr(taps, C.c_uint16), taps.size, 0.0, 0)
        return out, (ids, logits, hidden, taps)

    def _result(self, out, bufs, n_tokens, opts) -> StepOutput:
        ids, logits, hidden, taps = bufs
        d = self.desc
        return StepOutput(ids[:out.n_ids].copy(), logits[:out.n_ids * d.vocab].reshape(-1, d.vocab) if opts.read_logits else logits,
                          hidden[:out.n_hidden * d.d_model].reshape(-1, d.d_model), taps[:out.n_taps * n_tokens * d.d_model].reshape(out.n_taps, n_tokens, d.d_model) if taps.size else taps, out.gpu_seconds)

    def step(self, runs, opts: StepOptions | None = None) -> StepOutput:
        """engine.rs:310-314: one synchronous step of CPU-fed runs."""
        opts = opts or StepOptions()
        arr, keep = self._runs(runs)
        n = sum(len(k) for k in keep)
        co = _StepOptions(opts.head, opts.hidden, int(opts.read_logits), int(opts.read_taps))
        out, bufs = self._out(n, opts)
        _check(lib().vlt_step(self.h, arr, C.c_uint32(len(runs)), C.byref(co), C.byref(out)))
        return self._result(out, bufs, n, opts)

    def step_capture(self, runs, opts: StepOptions | None = None):
        """engine.rs:318-355: a step that hands every layer's intermediates back. Returns (StepOutput, [layer dicts]) with
        each dict's arrays shaped [n][width]."""
        opts = opts or StepOptions()
        arr, keep = self._runs(runs)
        n = sum(len(k) for k in keep)
        co = _StepOptions(opts.head, opts.hidden, int(opts.read_logits), int(opts.read_taps))
        out, bufs = self._out(n, opts)
        layers = []

        def take(pc, _user):
            c = pc.contents
            widths = dict(resid_in=c.d_model, attn_in=c.d_model, qkv=c.qkv_width, sdpa_out=c.attn_width, attn_out=c.d_model, mlp_in=c.d_model, mlp_out=c.d_model)
            layers.append({"layer": c.layer, **{k: np.ctypeslib.as_array(getattr(c, k), shape=(c.n, w)).copy() for k, w in widths.items()}})

        cb = _CAPTURE_FN(take)
        _check(lib().vlt_step_capture(self.h, arr, C.c_uint32(len(runs)), C.byref(co), cb, None, C.byref(out)))
        return self._result(out, bufs, n, opts), layers

    def bench_fill(self, seq: int, n: int, seed: int = 0) -> None:
        _check(lib().vlt_bench_fill(self.h, C.c_uint32(seq), C.c_uint32(n), C.c_uint32(seed)))

    def sample_logits(self, logits, rows) -> np.ndarray:
        """hooks.rs:41-54: rows is a list of (Sampling, position of the drawn token)."""
        n = len(rows)
        cs = (_Sampling * n)(*[s.c() for s, _ in rows])
        pos = _u32([p for _, p in rows])
        out = np.zeros(n, np.uint32)
        lp = None
        if logits is not None:
            logits = np.ascontiguousarray(logits, np.float32)
            if logits.size != n * self.desc.vocab:
                raise EngineError(f"{n} rows of logits need {n * self.desc.vocab} values")
            lp = _ptr(logits, C.c_float)
        _check(lib().vlt_sample_logits(self.h, lp, cs, _ptr(pos), C.c_uint32(n), _ptr(out)))
        return out

    def spec_accept(self, p, q, drafts, temperature: float, seeds, pos0, reps: int = 1):
        """Rejection-sampling acceptance on bf16 logits (uint16 bit patterns): p [S][k+1][V], q [S][k][V],
        drafts [S][k]. Returns (accepted, token, rollback, kernel seconds)."""
        p = np.ascontiguousarray(p, np.uint16)
        q = np.ascontiguousarray(q, np.uint16)
        s, k, v = q.shape
        if p.shape != (s, k + 1, v) or v != self.desc.vocab:
            raise EngineError(f"spec_accept: p {p.shape} / q {q.shape} do not fit k+1 / k rows of vocab {self.desc.vocab}")
        drafts = _u32(drafts).reshape(s, k)
        seeds = np.ascontiguousarray(seeds, np.uint64)
        pos0 = _u32(pos0)
        acc, tok, rb = (np.zeros(s, np.uint32) for _ in range(3))
        secs = C.c_double()
        _check(lib().vlt_spec_accept(self.h, _ptr(p, C.c_uint16), _ptr(q, C.c_uint16), _ptr(drafts), C.c_uint32(s), C.c_uint32(k), C.c_float(temperature),
                                     _ptr(seeds, C.c_uint64), _ptr(pos0), C.c_uint32(reps), _ptr(acc), _ptr(tok), _ptr(rb), C.byref(secs)))
        return acc, tok, rb, secs.value

    def draft_trees(self, logits, vocab_ids, blocks, slots, inv_t: float, ncand: int, tin=None):
        """draft_top + draft_tree on draft logits [rows][nv]; blocks: (first row, rows) pairs, one slot each.
        Returns (cand [rows][4], cand_q [rows][4], feed [max_seqs][16], tree [max_seqs][16])."""
        logits = np.ascontiguousarray(logits, np.float32)
        rows, nv = logits.shape
        ids = None if vocab_ids is None else _u32(vocab_ids)
        blocks, slots = _u32(blocks), _u32(slots)
        tin = None if tin is None else _u32(tin)
        cand, cand_q = np.zeros((rows, 4), np.uint32), np.zeros((rows, 4), np.float32)
        feed, tree = np.zeros((self.cfg.max_seqs, 16), np.uint32), np.zeros((self.cfg.max_seqs, 16), np.uint32)
        _check(lib().vlt_draft_trees(self.h, _ptr(logits, C.c_float), C.c_uint32(rows), C.c_uint32(nv), None if ids is None else _ptr(ids), None if tin is None else _ptr(tin),
                                     _ptr(blocks),                                     _ptr(slots), C.c_uint32(len(slots)), C.c_float(inv_t), C.c_uint32(ncand), _ptr(cand), _ptr(cand_q, C.c_float), _ptr(feed),
                                     _ptr(tree)))
        return cand, cand_q, feed, tree

    def set_profile_skip(self, mask: int) -> None:
        lib().vlt_set_profile_skip(self.h, C.c_uint32(mask))

    def bench_matmul(self, kind: str, n: int, variant: int = 0, reps: int = 5):
        secs, nbytes = C.c_double(), C.c_uint64()
        _check(lib().vlt_bench_matmul(self.h, kind.encode(), C.c_uint32(n), C.c_uint32(variant), C.c_uint32(reps), C.byref(secs), C.byref(nbytes)))
        return secs.value, nbytes.value

    def generator(self) -> "Generator":
        return Generator(self)

    # ---- inspection (parity tests)
    def debug_read(self, name: str) -> np.ndarray:
        cap = 1 << 16
        while True:
            buf = np.zeros(cap, np.uint32)
            n = C.c_uint64()
            rc = lib().vlt_debug_read(self.h, name.encode(), _ptr(buf), C.c_uint64(cap), C.byref(n))
            if rc != 0 and n.value > cap:
                cap = int(n.value)
                continue
            _check(rc)
            return buf[:n.value].copy()

    def debug_write(self, name: str, index: int, data) -> None:
        d = _u32(data)
        _check(lib().vlt_debug_write(self.h, name.encode(), C.c_uint64(index), _ptr(d), C.c_uint64(d.size)))

    def debug_plan(self, runs, hidden: int = Rows.NONE) -> None:
        """runs: (seq, tokens, head Rows, verify)."""
        arr, keep = self._runs([(r[0], r[1]) for r in runs])
        heads = _u32([r[2] for r in runs])
        verify = _u32([1 if r[3] else 0 for r in runs])
        _check(lib().vlt_debug_plan(self.h, arr, _ptr(verify), _ptr(heads), C.c_uint32(len(runs)), C.c_uint32(hidden)))

    def debug_step(self, runs, opts: StepOptions | None = None, replay=None) -> StepOutput:
        """runs: (seq, tokens, head Rows, verify); replay: None or (mistake rate, seed)."""
        opts = opts or StepOptions()
        arr, keep = self._runs([(r[0], r[1]) for r in runs])
        n = sum(len(k) for k in keep)
        heads = _u32([r[2] for r in runs])
        verify = _u32([1 if r[3] else 0 for r in runs])
        co = _StepOptions(0, opts.hidden, int(opts.read_logits), int(opts.read_taps))
        out, bufs = self._out(n, opts)
        rate, seed = replay if replay else (0.0, 0)
        _check(lib().vlt_debug_step(self.h, arr, _ptr(verify), _ptr(heads), C.c_uint32(len(runs)), C.byref(co), C.c_uint32(1 if replay else 0),
                                    C.c_float(rate), C.c_uint32(seed), C.byref(out)))
        return self._result(out, bufs, n, opts)

    def settle(self, seq: int, unused: int) -> None:
        lib().vlt_debug_settle(self.h, C.c_uint32(seq), C.c_uint32(unused))

    def set_gen(self, slot: int, remaining: int, stop=()) -> None:
        st = _u32(list(stop))
        _check(lib().vlt_debug_set_gen(self.h, C.c_uint32(slot), C.c_uint32(remaining), _ptr(st), C.c_uint32(st.size)))

    def set_trace(self, slot: int, trace) -> None:
        t = _u32(trace)
        _check(lib().vlt_debug_set_trace(self.h, C.c_uint32(slot), _ptr(t), C.c_uint32(t.size)))

    # ---- measurement
    def mark(self, which: int) -> None:
        _check(lib().vlt_debug_mark(self.h, C.c_uint32(which)))

    def mark_elapsed_ms(self) -> float:
        ms = C.c_double()
        _check(lib().vlt_debug_mark_elapsed_ms(self.h, C.byref(ms)))
        return ms.value

    @staticmethod
    def launches() -> int:
        f = lib().vlt_debug_launches
        f.restype = C.c_uint64
        return int(f())

    def set_profile(self, on: bool) -> None:
        _check(lib().vlt_debug_profile(self.h, C.c_uint32(int(on))))

    def profile_read(self) -> dict:
        ms = (C.c_double * 5)()
        n = (C.c_uint32 * 5)()
        _check(lib().vlt_debug_profile_read(self.h, ms, n))
        names = ("matmul", "attention", "small", "tail", "drafter")
        return {k: dict(ms=ms[i], launches=int(n[i])) for i, k in enumerate(names)}

    def step_bytes(self):
        a, b = C.c_uint64(), C.c_uint64()
        _check(lib().vlt_debug_step_bytes(self.h, C.byref(a), C.byref(b)))
        return a.value, b.value


def spec_accept_static(p_dev: int, q_dev: int, drafts_dev: int, streams: int, k: int, vocab: int, temperature: float, seeds_dev: int, pos0_dev: int,
                       accepted_dev: int, token_dev: int, rollback_dev: int, cuda_stream: int = 0) -> None:
    """vlt_spec_accept_static: the acceptance step on device pointers (integers) of the current device,
    with static scratch -- nothing is allocated. Queues the kernels on `cuda_stream` and returns."""
    fn = lib().vlt_spec_accept_static
    fn.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_uint32, C.c_uint32, C.c_uint32, C.c_float, C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,
                   C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    _check(fn(p_dev, q_dev, drafts_dev, streams, k, vocab, temperature, seeds_dev, pos0_dev, accepted_dev, token_dev, rollback_dev, cuda_stream or None))


def spec_accept_static_max_rows() -> int:
    fn = lib().vlt_spec_accept_static_max_rows
    fn.restype = C.c_uint32
    return int(fn())


class Draft:
    """engine/src/engine/generate.rs:24-42."""
    NONE, REPLAY, MODEL = 0, 1, 2


class Finish:
    STOP, LENGTH, FAILED = 0, 1, 2


@dataclass
class Request:
    """engine/src/engine/generate.rs:12-21; prompt is a token list, or ("resume", seq, token)."""
    prompt: object
    max_tokens: int
    stop: list = field(default_factory=list)
    sampling: Sampling = field(default_factory=Sampling)
    draft: int = Draft.NONE
    rows: int = 1
    trace: list = field(default_factory=list)


@dataclass
class Event:
    kind: str  # "token" or "done"
    req: int
    value: int


class Generator:
    """engine/src/engine/generate.rs `Generator`."""

    def __init__(self, engine: Engine):
        self.engine = engine
        self.h = C.c_void_p()
        _check(lib().vlt_generator_new(engine.h, C.byref(self.h)))

    def close(self) -> None:
        if getattr(self, "h", None):
            lib().vlt_generator_free(self.h)
            self.h = None

    def __del__(self):
        self.close()

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def submit(self, req: Request) -> int:
        r = _Request()
        keep = []
        if isinstance(req.prompt, tuple) and req.prompt and req.prompt[0] == "resume":
            r.prompt_kind, r.resume_seq, r.resume_token = 1, req.prompt[1], req.prompt[2]
        else:
            p = _u32(req.prompt)
            keep.append(p)
            r.prompt_kind, r.prompt_tokens, r.n_prompt = 0, _ptr(p), p.size
        st, tr = _u32(req.stop), _u32(req.trace)
        keep += [st, tr]
        r.max_tokens, r.stop, r.n_stop = req.max_tokens, _ptr(st), st.size
        r.sampling = req.sampling.c()
        r.draft_kind, r.draft_rows, r.trace, r.n_trace = req.draft, req.rows, _ptr(tr), tr.size
        rid = C.c_uint32()
        _check(lib().vlt_generator_submit(self.h, C.byref(r), C.byref(rid)))
        return rid.value

    def cancel(self, req: int) -> None:
        lib().vlt_generator_cancel(self.h, C.c_uint32(req))

    def step(self) -> list:
        cap = 4096
        ev = (_Event * cap)()
        n = C.c_uint32()
        _check(lib().vlt_generator_step(self.h, ev, C.c_uint32(cap), C.byref(n)))
        return [Event("token" if ev[i].kind == 0 else "done", ev[i].req, ev[i].value) for i in range(n.value)]

    def is_idle(self) -> bool:
        return bool(lib().vlt_generator_is_idle(self.h))

    def counts(self):
        q, r = C.c_uint32(), C.c_uint32()
        lib().vlt_generator_counts(self.h, C.byref(q), C.byref(r))
        return q.value, r.value

    def take_stats(self) -> list:
        out = []
        while True:
            buf = (_StepStats * 1024)()
            n = C.c_uint32()
            _check(lib().vlt_generator_stats(self.h, buf, C.c_uint32(1024), C.byref(n)))
            out += [dict(tokens=b.tokens, decode=bool(b.decode), emitted=b.emitted, gpu_seconds=b.gpu_seconds, encode_seconds=b.encode_seconds) for b in buf[:n.value]]
            if n.value < 1024:
                return out

    def set_hold(self, hold: bool) -> None:
        lib().vlt_generator_set_hold(self.h, C.c_uint32(int(hold)))

    def set_replay_mistakes(self, rate: float, seed: int) -> None:
        lib().vlt_generator_set_replay_mistakes(self.h, C.c_float(rate), C.c_uint32(seed))


class _ReplicaOps(C.Structure):
    _fields_ = [("ctx", C.c_void_p),
                ("submit", C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(_Request), C.POINTER(C.c_uint32))),
                ("step", C.CFUNCTYPE(C.c_int, C.c_void_p, C.POINTER(_Event), C.c_uint32, C.POINTER(C.c_uint32))),
                ("cancel", C.CFUNCTYPE(None, C.c_void_p, C.c_uint32)),
                ("is_idle", C.CFUNCTYPE(C.c_int, C.c_void_p)),
                ("counts", C.CFUNCTYPE(None, C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)))]


class Router:
    """Streams sharded over replicas, a failed replica's streams re-queued on the others (vlt_router_*). `replicas` are
    Generators of this module, or objects with the same submit / step / cancel / is_idle / counts methods (stand-ins on
    the host: their step may raise to play a failed replica)."""

    def __init__(self, replicas):
        self.replicas = list(replicas)
        self._keep = []
        ops = (_ReplicaOps * len(self.replicas))()
        for i, r in enumerate(self.replicas):
            if isinstance(r, Generator):
                lib().vlt_replica_of_generator(r.h, C.byref(ops[i]))
            else:
                ops[i] = self._wrap(r)
        self.h = C.c_void_p()
        _check(lib().vlt_router_new(ops, C.c_uint32(len(self.replicas)), C.byref(self.h)))

    def _wrap(self, rep) -> _ReplicaOps:
        F = dict(_ReplicaOps._fields_)

        def submit(_ctx, preq, pid):
            q = preq.contents
            try:
                req = Request([q.prompt_tokens[i] for i in range(q.n_prompt)], q.max_tokens, [q.stop[i] for i in range(q.n_stop)],
                              Sampling(q.sampling.temperature, q.sampling.top_p, q.sampling.seed), q.draft_kind, q.draft_rows, [q.trace[i] for i in range(q.n_trace)])
                pid[0] = rep.submit(req)
                return 0
            except Exception:
                return 1

        def step(_ctx, pev, cap, pn):
            try:
                evs = rep.step()
            except Exception:
                return 1
            for i, e in enumerate(evs[:cap]):
                pev[i] = _Event(0 if e.kind == "token" else 1, e.req, e.value)
            pn[0] = min(len(evs), cap)
            return 0

        def cancel(_ctx, rid):
            rep.cancel(rid)

        def is_idle(_ctx):
            return int(rep.is_idle())

        def counts(_ctx, pq, pr):
            pq[0], pr[0] = rep.counts()

        fns = [F["submit"](submit), F["step"](step), F["cancel"](cancel), F["is_idle"](is_idle), F["counts"](counts)]
        self._keep.append(fns)
        return _ReplicaOps(None, *fns)

    def close(self) -> None:
        if getattr(self, "h", None):
            lib().vlt_router_free(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def submit(self, req: Request) -> int:
        r = _Request()
        p, st, tr = _u32(req.prompt), _u32(req.stop), _u32(req.trace)
        r.prompt_kind, r.prompt_tokens, r.n_prompt = 0, _ptr(p), p.size
        r.max_tokens, r.stop, r.n_stop = req.max_tokens, _ptr(st), st.size
        r.sampling = req.sampling.c()
        r.draft_kind, r.draft_rows, r.trace, r.n_trace = req.draft, req.rows, _ptr(tr), tr.size
        rid = C.c_uint32()
        _check(lib().vlt_router_submit(self.h, C.byref(r), C.byref(rid)))
        return rid.value

    def cancel(self, req: int) -> None:
        lib().vlt_router_cancel(self.h, C.c_uint32(req))

    def step(self) -> list:
        cap = 8192
        ev = (_Event * cap)()
        n = C.c_uint32()
        _check(lib().vlt_router_step(self.h, ev, C.c_uint32(cap), C.byref(n)))
        return [Event("token" if ev[i].kind == 0 else "done", ev[i].req, ev[i].value) for i in range(n.value)]

    def is_idle(self) -> bool:
        return bool(lib().vlt_router_is_idle(self.h))

    def alive(self) -> int:
        f = lib().vlt_router_alive
        f.restype = C.c_uint32
        return int(f(self.h))

    def replica_of(self, req: int) -> int:
        f = lib().vlt_router_replica_of
        f.restype = C.c_uint32
        return int(f(self.h, C.c_uint32(req)))
