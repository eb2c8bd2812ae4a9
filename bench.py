"""Decode tokens/s of the speculative-decoding step: the 1B int8 target at 8k context.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--streams S] [--ctx C] [--impl reference]

One rank per GPU (torchrun for N > 1): each rank is an independent replica with its own
streams -- no collective on the data path; ranks only meet at the timing barriers. A "step"
is one decode step of every stream on the rank: the chain drafter's catch-up and k = 4 draft passes,
k + 1 rows per stream through the int8 target, acceptance at T = 0.6 (rejection sampling against the
drafter's distribution) and KV commit. Further passes in the same JSON line: the target alone behind the
replay drafter, 1 and 8 streams, bf16 at one stream, the 64k context, the acceptance kernel alone, a drafter without
its attention window, prefill, the reference's own architecture at its shapes (plain decoding), and the CPU
restatement's sample. Prints one JSON line.
"""
from __future__ import annotations

import argparse
import copy
import importlib.util
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
CACHE = Path(os.environ.get("VLT_BENCH_CACHE", "/tmp/vlt_bench"))


def _package():
    name = "silicon_violetto_b200"
    if name not in sys.modules:
        pkg_dir = ROOT / "silicon-violetto_b200"
        spec = importlib.util.spec_from_file_location(name, pkg_dir / "__init__.py", submodule_search_locations=[str(pkg_dir)])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    if str(ROOT) not in sys.path:
        sys.path.insert(0, str(ROOT))


def model_file(config: str, int8: bool, rank: int, layers: int = 0) -> Path:
    """The random-init weight file (seed 0, N(0, 0.02^2), int8 per output row), written once per box.
    `layers` > 0 cuts the model to that many layers (a profiling-size case of the same shapes)."""
    from silicon_violetto_b200 import synth
    CACHE.mkdir(parents=True, exist_ok=True)
    path = CACHE / f"{config}{f'_L{layers}' if layers else ''}_{'int8row' if int8 else 'bf16'}.vlt"
    done = path.with_suffix(".ok")
    if rank == 0 and not done.exists():
        c = dict(synth.CONFIGS[config], n_layers=layers) if layers else config
        synth.write_target(path, c, seed=0, int8_group=0 if int8 else None)
        done.write_text("ok")
    while not done.exists():
        time.sleep(0.5)
    return path


class Clocks:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device: int):
        self.device, self.rows, self.proc = device, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(self.device)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            self.thread.join(timeout=2)

    def summary(self) -> dict:
        sm = [float(r[1]) for r in self.rows if len(r) >= 9 and r[1].replace(".", "").isdigit()]
        mx = [float(r[2]) for r in self.rows if len(r) >= 9 and r[2].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = sorted({n for r in self.rows if len(r) >= 9 for n, v in zip(names, r[5:9]) if v == "Active"})
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons, "samples": len(sm)}


ROWS = 5           # k = 4 drafts + the bonus row
ATTN_TRAFFIC_RATIO = 542.4 / 537.6  # DRAM traffic / algorithmic bytes of the attention launch, from its ncu capture
KV_BYTES_PER_TOKEN_LAYER = 8 * 64 * 2 * 2  # 8 kv heads x 64 dims x bf16 x (K, V)
WEIGHT_PARAMS = 16 * (3072 * 2048 + 2048 * 2048 + 16384 * 2048 + 2048 * 8192) + 128256 * 2048


def drafter_file(rank: int, window: int) -> Path:
    """The chain drafter of the 1B target (fc, one layer, a head over 16384 draft ids), int8 per row, random-init; its
    draft passes attend to the last `window` positions (0: all), as the reference's drafter layers attend to 1024
    (tools/spec/drafter.py:17)."""
    from silicon_violetto_b200 import synth
    path = CACHE / f"1b_drafter_int8row_w{window}.vlt"
    done = path.with_suffix(".ok")
    if rank == 0 and not done.exists():
        synth.write_drafter(path, "1b", seed=100, int8_group=0, draft_vocab=16384, window=window)
        done.write_text("ok")
    while not done.exists():
        time.sleep(0.5)
    return path


def make_engine(E, path, streams, ctx, steps_total, device, attn_keys=0):
    room = ROWS * (steps_total + 8) + 64
    cfg = E.EngineConfig(max_seqs=streams, max_step_tokens=max(streams * ROWS, 64), max_chunk=16, global_kv_tokens=streams * (ctx + room + 16),
                         max_seq_len=ctx + room, max_head_rows=max(streams * ROWS, 8), device_ordinal=device)
    return E.Engine(path, cfg, E.Tuning(spec_policy_off=True, attn_keys_per_cta=attn_keys)), room


def fill(eng, streams, ctx, rank):
    seqs = [eng.new_seq() for _ in range(streams)]
    for j, s in enumerate(seqs):
        eng.bench_fill(s, ctx, seed=stream_seeds(rank, j)[0])
    return seqs


def record_plain(E, eng, streams, ctx, n_tokens, rank, sampling):
    """Plain decoding (one row per stream and step) from the filled context: the tokens the replay drafter will draft."""
    seqs = fill(eng, streams, ctx, rank)
    out = [[] for _ in seqs]
    with eng.generator() as g:
        for j, s in enumerate(seqs):
            g.submit(E.Request(("resume", s, 100 + j), n_tokens, sampling=sampling(j)))
        while not g.is_idle():
            for ev in g.step():
                if ev.kind == "token":
                    out[ev.req].append(ev.value)
        g.take_stats()
    return out


def run_replica(args, rank, world, barrier, device, eng, mistakes, model_drafter=False):
    """One timed pass: `warmup` + `steps` verify steps of every stream, drafts from the replay drafter
    (or, with `model_drafter`, from the loaded chain drafter)."""
    from silicon_violetto_b200 import engine as E
    total_steps = args.warmup + args.steps + 6
    sampling = lambda j: E.Sampling(args.temperature, args.top_p, stream_seeds(rank, j)[1])
    n_rec = ROWS * total_steps + 8
    recorded = record_plain(E, eng, args.streams, args.ctx, n_rec, rank, sampling) if mistakes < 1.0 and not model_drafter else [[0] * n_rec] * args.streams
    seqs = fill(eng, args.streams, args.ctx, rank)
    g = eng.generator()
    g.set_replay_mistakes(mistakes, 1)
    for j, s in enumerate(seqs):
        if model_drafter:
            g.submit(E.Request(("resume", s, 100 + j), n_rec - 2, sampling=sampling(j), draft=E.Draft.MODEL, rows=ROWS))
            continue
        trace = [0] * args.ctx + [100 + j] + recorded[j]
        g.submit(E.Request(("resume", s, 100 + j), n_rec - 2, sampling=sampling(j), draft=E.Draft.REPLAY, rows=ROWS, trace=trace))
    with Clocks(device) as clocks:  # nvidia-smi needs a moment to start: it samples from the warm-up on
        for _ in range(args.warmup):
            g.step()
        barrier()
        launches0 = E.Engine.launches()
        eng.mark(0)
        t0 = time.perf_counter()
        for _ in range(args.steps):
            g.step()
        eng.mark(1)
        g.step()  # collects the last timed step (and queues one more, outside both timings)
        wall = time.perf_counter() - t0
        dev_ms = eng.mark_elapsed_ms()
    launches = E.Engine.launches() - launches0
    barrier()
    stats = g.take_stats()
    timed = stats[args.warmup:args.warmup + args.steps]
    emitted = sum(s["emitted"] for s in timed)
    # A profiling pass: GPU time of each kernel group, from events around the group's launches.
    eng.set_profile(True)
    prof_steps = 3
    for _ in range(prof_steps):
        g.step()
    prof = eng.profile_read()
    eng.set_profile(False)
    mean_len = float(np.mean([eng.seq_len(s) for s in seqs]))
    h2d, d2h = eng.step_bytes()
    g.close()
    return dict(dev_ms=dev_ms, wall=wall, emitted=emitted, launches=launches * args.steps // (args.steps + 1), prof=prof, prof_steps=prof_steps,
                mean_len=mean_len, h2d=h2d, d2h=d2h, clocks=clocks.summary(), tokens_per_step=[s["tokens"] for s in timed])


def cpu_reference(args, streams, steps, warmup=1):
    """The CPU restatement of the path (the oracle) timed on this machine's cores, on a bounded
    sample of the workload: `streams` streams at the full context, `steps` verify steps of 5 rows."""
    _package()
    import oracle
    threads = oracle.set_threads(os.cpu_count() or 1)  # torchrun sets OMP_NUM_THREADS=1 for its workers: take the machine's cores anyway
    path = model_file("1b", not args.bf16, 0)
    room = ROWS * (steps + warmup + 2) + 32
    eng = oracle.Engine(path, max_seqs=streams, max_step_tokens=streams * ROWS, max_chunk=16, kv_tokens=streams * (args.ctx + room + 16),
                        max_seq_len=args.ctx + room, max_head_rows=streams * ROWS)
    seqs = [eng.new_seq() for _ in range(streams)]
    for j, s in enumerate(seqs):
        eng.set_sampling(s, args.temperature, 0.95, 1 + j)  # (the reference's sample-then-match acceptance: the target's verify step alone)
        eng.bench_fill(s, args.ctx)
        eng.write("feed", s * 16, [100 + j, 1, 2, 3, 4])
    runs = [(s, [oracle.FEED_ROW + i for i in range(ROWS)], oracle.ROWS_LAST, True) for s in seqs]
    times, emitted = [], []
    for i in range(steps + warmup):
        t0 = time.perf_counter()
        eng.step(runs)
        dt = time.perf_counter() - t0
        em = eng.array("emitted")[:streams]
        for j, s in enumerate(seqs):  # what `collect` does: give back the rows that were not accepted
            eng.settle(s, ROWS - int(em[j]))
        if i >= warmup:
            times.append(dt)
            emitted.append(int(em.sum()))
    return float(np.median(times)), threads, float(np.mean(emitted))


def reduce_over_ranks(dev_ms, wall_s, emitted, launches, world, device):
    """What the replicas share after the timed region: the slowest rank's times (MAX) and the whole job's
    emitted tokens and kernel launches (SUM). The only collective of the bench; none on the data path."""
    import torch
    import torch.distributed as dist
    vals = torch.tensor([dev_ms, wall_s], dtype=torch.float64, device=device)
    sums = torch.tensor([float(emitted), float(launches)], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(vals, op=dist.ReduceOp.MAX)
        dist.all_reduce(sums, op=dist.ReduceOp.SUM)
    return vals.tolist(), sums.tolist()


def stream_seeds(rank: int, stream: int):
    """(context seed, sampling seed) of stream `stream` on replica `rank`: distinct over the whole job.
    Rank 0 keeps the reference's 7 + j (cli/src/bench.rs:165)."""
    return 1000 * rank + 7 + stream, 1 + 1000 * rank + stream


def spec_accept_figure(E, eng, hbm_peak):
    """BASELINE configuration 1: the stand-alone acceptance step on 32 streams x (5 target + 4 draft) rows of bf16
    logits N(0, 3^2) over 128 256 ids at temperature 1; drafts drawn from softmax(q) (numpy, seed 1), uniforms keyed by
    seed 2. Algorithmic bytes: p and q read once."""
    rng = np.random.default_rng(0)
    streams, k, v = 32, 4, eng.desc.vocab
    from silicon_violetto_b200 import vlt
    p = vlt.to_bf16((rng.standard_normal((streams, k + 1, v)) * 3.0).astype(np.float32))
    q = vlt.to_bf16((rng.standard_normal((streams, k, v)) * 3.0).astype(np.float32))
    qf = vlt.from_bf16(q).astype(np.float64)
    pr = np.exp(qf - qf.max(axis=2, keepdims=True))
    pr /= pr.sum(axis=2, keepdims=True)
    r1 = np.random.default_rng(1)
    drafts = np.array([[r1.choice(v, p=pr[s_, i]) for i in range(k)] for s_ in range(streams)], np.uint32)
    seeds = np.arange(streams, dtype=np.uint64) + np.uint64(2)
    pos0 = np.full(streams, 8192, np.uint32)
    acc, tok, rb, secs = eng.spec_accept(p, q, drafts, 1.0, seeds, pos0, reps=10)
    nbytes = p.nbytes + q.nbytes
    return {"workload": "32 streams, k=4, 128256 ids, bf16 logits N(0, 3^2), T=1", "us": secs * 1e6, "algorithmic_bytes": nbytes, "achieved_gbs": nbytes / secs / 1e9,
            "frac_of_hbm_peak": nbytes / secs / 1e9 / hbm_peak, "mean_accepted": float(acc.mean())}


def limite_figure(E, local, ctx, steps=30, stream_counts=(1, 8, 32), keys_per_block=0, drafter=False, int8=False):
    """The reference's own architecture at its shapes (48 layers, hidden 1280, 10 query / 2 kv heads of 128, FFN 3328,
    151 680 ids, bf16, random-init): decoding one token a step
    at 1, 8 and 32 streams over contexts advanced without computing them. With `drafter`, the reference's pairing: its
    block drafter (tools/spec/drafter.py's shapes: 2 layers reading target layers 35 and 47, blocks of 8, window 1024, 16 384
    draft ids; random-init, so next to nothing it drafts is accepted) drafts a tree of up to 8 rows per stream and step and
    the target verifies it. Not BASELINE's metric: figures for the record."""
    from silicon_violetto_b200 import synth
    CACHE.mkdir(parents=True, exist_ok=True)
    # int8: the reference converter's default format (tools/convert.py:20): scale groups of 64, of 8 for the head.
    kind = "int8" if int8 else "bf16"
    path = CACHE / f"limite_48x1280_{kind}.vlt"
    done = path.with_suffix(".ok")
    if not done.exists():
        synth.write_limite(path, n_layers=48, hidden=1280, n_kv=2, ffn=3328, vocab=151680, seed=0, int8_group=64 if int8 else None)
        done.write_text("ok")
    dpath = CACHE / f"block_drafter_1280_{kind}.vlt"
    if drafter and not dpath.with_suffix(".ok").exists():
        synth.write_block_drafter(dpath, synth.block_drafter_state(1), int8=int8)
        dpath.with_suffix(".ok").write_text("ok")
    what = "the block drafter's tree of up to 8 rows verified per stream and step" if drafter else "one token per stream and step"
    out = {"workload": f"reference architecture 48 x 1280, {'int8 in groups of 64 (head: 8)' if int8 else 'bf16'}, ctx {ctx}, {what}"}
    for n_s in stream_counts:
        cfg = E.EngineConfig(max_seqs=n_s, max_step_tokens=max(64, 8 * n_s), max_chunk=32, global_kv_tokens=n_s * (ctx + 512), max_seq_len=ctx + 512, max_head_rows=8 * n_s,
                             device_ordinal=local)
        eng = E.Engine(path, cfg, E.Tuning(spec_policy_off=True, attn_keys_per_cta=keys_per_block))
        if drafter:
            eng.load_drafter(dpath)
        seqs = [eng.new_seq() for _ in range(n_s)]
        for s_ in seqs:
            eng.bench_fill(s_, ctx)
        with eng.generator() as g:
            for j, s_ in enumerate(seqs):
                g.submit(E.Request(("resume", s_, 100 + j), 8 * (steps + 16), sampling=E.Sampling(0.6, 0.95, 1 + j), draft=E.Draft.MODEL if drafter else E.Draft.NONE, rows=8 if drafter else 1))
            warm = 4
            for _ in range(warm):
                g.step()
            eng.mark(0)
            for _ in range(steps):
                g.step()
            eng.mark(1)
            g.step()
            ms = eng.mark_elapsed_ms() / steps
            timed = g.take_stats()[warm:warm + steps]
        eng.close()
        emitted = sum(s_["emitted"] for s_ in timed)
        out[f"streams_{n_s}"] = {"ms_per_step": ms, "tokens_per_s": emitted / (ms * steps * 1e-3), "mean_accepted_len": emitted / (steps * n_s),
                                 "rows_per_step": float(np.mean([s_["tokens"] for s_ in timed]))}
    return out


def prefill_figure(E, path, ctx, local, chunk=512):
    """A `ctx`-token prompt of the reference's LCG ids computed in chunks of `chunk` tokens through the generator (the
    tensor-core GEMM in blocks of 256 tokens, the chunk attention kernel), one stream; device time from the first chunk's
    start to the last one's end."""
    from silicon_violetto_b200 import synth
    cfg = E.EngineConfig(max_seqs=1, max_step_tokens=chunk, max_chunk=chunk, global_kv_tokens=ctx + 64, max_seq_len=ctx + 64, max_head_rows=8, device_ordinal=local)
    eng = E.Engine(path, cfg, E.Tuning(spec_policy_off=True))
    prompt = synth.lcg_ids(ctx, 2 + ctx, eng.desc.vocab)  # cli/src/bench.rs:136
    best = None
    for _ in range(2):  # the first pass warms up (tensor maps, instruction caches)
        with eng.generator() as g:
            g.submit(E.Request(list(prompt), 1))
            eng.mark(0)
            while not g.is_idle():
                g.step()
            eng.mark(1)
            ms = eng.mark_elapsed_ms()
            steps = g.take_stats()
        best = ms if best is None else min(best, ms)
    eng.close()
    return {"workload": f"1 stream, {ctx}-token prompt in chunks of {chunk}", "value": ctx / (best * 1e-3), "unit": "prompt tokens/s", "ms": best, "steps": len(steps)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--streams", type=int, default=32, help="streams per GPU")
    ap.add_argument("--ctx", type=int, default=8192)
    ap.add_argument("--temperature", type=float, default=0.6)
    ap.add_argument("--top-p", type=float, default=1.0, help="1: the rejection-sampling acceptance decides the drafted runs (BASELINE configurations 3 and 4); below 1 the reference's sample-then-match does")
    ap.add_argument("--mistakes", type=float, default=1.0, help="share of positions drafted wrong in the replay-drafter passes' first one (1: every draft wrong, what a random-init drafter gives)")
    ap.add_argument("--replay-mistakes", type=float, default=0.3, help="a second pass with the replay drafter at this mistake rate (cli/src/bench_spec.rs:26-28); 1: skip")
    ap.add_argument("--bf16", action="store_true", help="bf16 weights instead of int8 (no drafter pass)")
    ap.add_argument("--cpu-streams", type=int, default=8, help="streams of the CPU sample")
    ap.add_argument("--cpu-steps", type=int, default=10, help="timed verify steps of the CPU sample (the reference arm takes --steps, at most 20)")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--also-streams", default="1,8", help="comma list: extra passes at these stream counts on rank 0's engine (the headline metric is quoted at 1, 8 and 32 streams); empty: none")
    ap.add_argument("--drafter-window", type=int, default=1024, help="the chain drafter's attention window in positions (the reference's drafter: 1024); 0: the whole context")
    ap.add_argument("--no-model-drafter", action="store_true", help="the headline pass without the chain drafter (replay drafter, every draft wrong)")
    ap.add_argument("--no-extras", action="store_true", help="only the headline pass (no replay, stream-count, bf16, long-context or acceptance-kernel passes)")
    ap.add_argument("--long-ctx", type=int, default=65536, help="context of the long-context pass every rank runs after the headline one (BASELINE configuration 4); 0: skip")
    ap.add_argument("--long-steps", type=int, default=20)
    ap.add_argument("--attn-keys", type=int, default=0, help="keys per attention block (0: the engine's own choice)")
    ap.add_argument("--layers", type=int, default=0, help="cut the model to this many layers: a profiler-size case, not a bench value")
    ap.add_argument("--no-limite", action="store_true", help="skip the reference-architecture pass of the extras (it writes a 2 GB file first)")
    ap.add_argument("--limite-streams", default="1,8,32", help="stream counts of --only limite")
    ap.add_argument("--limite-drafter", action="store_true", help="--only limite: with the reference's block drafter loaded (tree drafts of up to 8 rows)")
    ap.add_argument("--limite-int8", action="store_true", help="--only limite: int8 weights in the reference converter's default groups (64; the head 8)")
    ap.add_argument("--limite-keys", type=int, default=0, help="--only limite: keys per attention block (VltTuning.attn_keys_per_cta); 0 = the library's choice")
    ap.add_argument("--only", default="", help="'prefill', 'acceptance' or 'limite' (the reference's own architecture at its shapes, decoding): run that one pass alone and print its figure (not the bench line)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    rank, world, local = int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))
    peaks = {}
    if (ROOT / "MEASURED_PEAKS.json").exists():
        peaks = json.loads((ROOT / "MEASURED_PEAKS.json").read_text())
    hbm_peak, peak_src = (peaks["hbm_gbs"], "measured") if "hbm_gbs" in peaks else (6650.0, "fallback")
    with_drafter = not (args.no_model_drafter or args.bf16)
    workload = (f"1B llama-style target{' + chain drafter' if with_drafter else ''}, {'bf16' if args.bf16 else 'int8 per-row'} weights, {args.streams} streams/GPU, ctx {args.ctx}, "
                f"k=4 (5 rows), T={args.temperature} top-p {args.top_p}")
    if args.layers:
        workload += f" -- CUT TO {args.layers} LAYERS (profiler-size case)"

    if args.impl == "reference":
        # The reference has no CPU implementation of this path (its arithmetic is Metal shaders); what runs here is the C++
        # restatement of that shader math on this machine's cores, on the main arm's stream count, a bounded number of steps.
        if rank != 0:
            return
        ref_steps = max(1, min(args.steps, 20))
        t_step, cores, em = cpu_reference(args, args.streams, ref_steps, warmup=1)
        v = em / t_step
        print(json.dumps({"impl": "reference", "metric": "decode tokens/s at 8k context", "value": v, "unit": "tokens/s",
                          "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak",
                          "vs_baseline": None, "dtype": "bf16 activations, int8 weights" if not args.bf16 else "bf16", "data": "synthetic",
                          "config": {"workload": workload, "streams_timed": args.streams, "steps_timed": ref_steps, "drafter": "every draft wrong (the target's verify step alone)",
                                     "mean_accepted_len": em / args.streams},
                          "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": "port",
                                           "sample": f"{args.streams} streams x {ref_steps} verify steps of 5 rows at ctx {args.ctx}; the reference has no CPU path, this is the C++ restatement of its shader math"},
                          "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}))
        return

    import torch
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
        torch.cuda.set_device(local)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(local)

    solo = lambda: torch.cuda.synchronize(local)
    _package()
    from silicon_violetto_b200 import engine as E
    path = model_file("1b", not args.bf16, rank, args.layers)
    if args.only:
        if args.only == "prefill":
            print(json.dumps(prefill_figure(E, path, args.ctx, local)))
        elif args.only == "acceptance":
            e1, _ = make_engine(E, path, 2, 64, 8, local)
            print(json.dumps(spec_accept_figure(E, e1, hbm_peak)))
        elif args.only == "limite":
            print(json.dumps(limite_figure(E, local, args.ctx, min(args.steps, 30), [int(x) for x in args.limite_streams.split(",")], args.limite_keys, args.limite_drafter, args.limite_int8)))
        else:
            raise SystemExit(f"--only {args.only}: 'prefill', 'acceptance' or 'limite'")
        return
    total = args.warmup + args.steps + 6
    # The headline pass, on every rank: the int8 target with the chain drafter loaded (1 layer + fc + a head over 16 384 draft
    # ids, random-init), drafts drawn from its distribution, the rejection-sampling rule deciding them in the step.
    eng, _ = make_engine(E, path, args.streams, args.ctx, total, local, args.attn_keys)
    if with_drafter:
        eng.load_drafter(drafter_file(rank, args.drafter_window))
        eng.set_acceptance(1 if args.top_p >= 1.0 else 0)
    r = run_replica(args, rank, world, barrier, local, eng, args.mistakes, model_drafter=with_drafter)
    vals, sums = reduce_over_ranks(r["dev_ms"], r["wall"], r["emitted"], r["launches"], world, f"cuda:{local}")
    eng.close()
    # The long-context pass (BASELINE configuration 4's share of one GPU), on every rank as well.
    long_pass = None
    if args.long_ctx and not args.no_extras and not args.layers:
        a4 = copy.copy(args)
        a4.ctx, a4.steps = args.long_ctx, args.long_steps
        e4, _ = make_engine(E, path, args.streams, a4.ctx, a4.warmup + a4.steps + 6, local, args.attn_keys)
        if with_drafter:
            e4.load_drafter(drafter_file(rank, args.drafter_window))
            e4.set_acceptance(1 if args.top_p >= 1.0 else 0)
        r4 = run_replica(a4, rank, world, barrier, local, e4, 1.0, model_drafter=with_drafter)
        v4, s4 = reduce_over_ranks(r4["dev_ms"], r4["wall"], r4["emitted"], r4["launches"], world, f"cuda:{local}")
        e4.close()
        kv4 = args.streams * (r4["mean_len"] + ROWS) * KV_BYTES_PER_TOKEN_LAYER * 16
        long_pass = {"workload": f"{args.streams} streams/GPU at ctx {a4.ctx}, {a4.steps} steps", "value": s4[0] / (v4[0] * 1e-3), "unit": "tokens/s (all ranks)",
                     "ms_per_step": v4[0] / a4.steps, "e2e": s4[0] / v4[1], "mean_accepted_len": s4[0] / (a4.steps * args.streams * world),
                     "step_frac": (WEIGHT_PARAMS + kv4) / (v4[0] * 1e-3 / a4.steps) / 1e9 / hbm_peak,
                     "kernel_groups_ms_per_step": {k: v["ms"] / r4["prof_steps"] for k, v in r4["prof"].items()}}
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    dev_s, wall_s = vals[0] * 1e-3, vals[1]
    emitted = sums[0]
    steps = args.steps
    tau = emitted / (steps * args.streams * world)
    # Roofline of the dominant kernel (the paged attention at 32 streams): algorithmic bytes of one
    # launch = every stream's cached and new K/V rows of one layer, read once.
    att = r["prof"]["attention"]
    att_ms = att["ms"] / max(att["launches"], 1)
    att_bytes = args.streams * (r["mean_len"] + ROWS) * KV_BYTES_PER_TOKEN_LAYER
    achieved = att_bytes / (att_ms * 1e-3) / 1e9 if att_ms > 0 else 0.0
    step_bytes = WEIGHT_PARAMS * (2 if args.bf16 else 1) + args.streams * (r["mean_len"] + ROWS) * KV_BYTES_PER_TOKEN_LAYER * (args.layers or 16)
    drafter_note = (f"chain drafter (1 layer + fc + head over 16384 draft ids, int8, attention window {args.drafter_window or 'none'}, random-init: its drafts are practically never accepted), drafts drawn from its own "
                    "distribution, rejection-sampling acceptance in the step" if with_drafter else f"replay drafter, {args.mistakes:.2f} of positions drafted wrong")
    out = {
        "metric": "decode tokens/s at 8k context", "value": emitted / dev_s, "unit": "tokens/s", "n_gpus": world, "steps": steps, "warmup": args.warmup,
        "ms_per_step": dev_s * 1e3 / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16" if args.bf16 else "bf16 activations x int8 weights, fp32 accumulate", "data": "synthetic",
        "config": {"workload": workload, "drafter": drafter_note, "mean_accepted_len": tau,
                   "kv": "filled without computing it (timing does not depend on KV values)", "l2": "per-step traffic (weights 1.2 GB + KV) exceeds the 126 MB L2",
                   "parallelism": f"{world} replica(s), streams sharded, no collective"},
        "e2e": {"value": emitted / wall_s, "unit": "tokens/s", "h2d_bytes_per_step": r["h2d"], "d2h_bytes_per_step": r["d2h"]},
        "gpu_launches": int(sums[1]),
        "clocks": r["clocks"],
        "roofline": {"bound": "hbm", "kernel": "attn_mma_kernel", "achieved": achieved, "peak": hbm_peak, "unit": "GB/s", "frac": achieved / hbm_peak, "peak_source": peak_src,
                     # dram__bytes_read + dram__bytes_write of one launch of this very shape under ncu: 1.009 x the algorithmic
                     # bytes (profiles/attn_mma_kernel_32streams_8k.md); scaled to this run's key count.
                     "traffic": att_bytes * ATTN_TRAFFIC_RATIO, "traffic_source": "ncu capture of the same launch shape, scaled by keys",
                     # the target's verify step alone (weights + K/V once) against the whole step's time, drafter included
                     "step_frac": step_bytes / (dev_s / steps) / 1e9 / hbm_peak},
        "kernel_groups_ms_per_step": {k: v["ms"] / r["prof_steps"] for k, v in r["prof"].items()},
    }
    if long_pass is not None:
        out["long_context_pass"] = long_pass
    if not args.no_extras and not args.layers:
        # The target's verify step alone, drafts from the replay drafter: every one wrong, then at the reference's mistake rate.
        a0 = copy.copy(args)
        a0.top_p = 0.95
        e0, _ = make_engine(E, path, args.streams, args.ctx, total, local, args.attn_keys)
        r0 = run_replica(a0, rank, 1, solo, local, e0, 1.0)
        p0 = r0["prof"]
        out["replay_pass_all_wrong"] = {"value": r0["emitted"] / (r0["dev_ms"] * 1e-3), "unit": "tokens/s (this rank)", "ms_per_step": r0["dev_ms"] / steps, "e2e": r0["emitted"] / r0["wall"],
                                        "mean_accepted_len": r0["emitted"] / (steps * args.streams), "sampling": "T as above, top-p 0.95 (the reference's sample-then-match acceptance)",
                                        "step_frac": step_bytes / (r0["dev_ms"] * 1e-3 / steps) / 1e9 / hbm_peak,
                                        "verify_attention_frac": step_bytes / ((p0["matmul"]["ms"] + p0["attention"]["ms"]) / r0["prof_steps"] * 1e-3) / 1e9 / hbm_peak,
                                        "kernel_groups_ms_per_step": {k: v["ms"] / r0["prof_steps"] for k, v in p0.items()}}
        if args.replay_mistakes < 1.0:
            extra = run_replica(a0, rank, 1, solo, local, e0, args.replay_mistakes)
            out["replay_pass"] = {"mistakes": args.replay_mistakes, "value": extra["emitted"] / (extra["dev_ms"] * 1e-3), "unit": "tokens/s (this rank)",
                                  "mean_accepted_len": extra["emitted"] / (steps * args.streams), "ms_per_step": extra["dev_ms"] / steps,
                                  # Chains that stop at the first wrong draft accept 1 + 0.7 + 0.7^2 + ... = 2.77 of 5 rows at 0.30. The drafts
                                  # replay a recording of one-row decoding; a stream whose sampled token once differs from it (sums in another
                                  # order, a random-init model's flat distributions: a near-tie of the draw) drafts wrong from then on.
                                  "note": "expected 2.77 at 0.30 mistakes; streams that leave their recorded continuation (sampling near-ties) draft wrong afterwards"}
        out["acceptance_kernel"] = spec_accept_figure(E, e0, hbm_peak)
        e0.close()
        if with_drafter and args.drafter_window:
            # The headline pass again with a chain drafter that attends to its whole context (four more reads of a layer's K/V a step).
            e5, _ = make_engine(E, path, args.streams, args.ctx, total, local, args.attn_keys)
            e5.load_drafter(drafter_file(0, 0))
            e5.set_acceptance(1 if args.top_p >= 1.0 else 0)
            r5 = run_replica(args, rank, 1, solo, local, e5, 1.0, model_drafter=True)
            e5.close()
            out["full_context_drafter_pass"] = {"value": r5["emitted"] / (r5["dev_ms"] * 1e-3), "unit": "tokens/s (this rank)", "ms_per_step": r5["dev_ms"] / steps,
                                                "mean_accepted_len": r5["emitted"] / (steps * args.streams),
                                                "kernel_groups_ms_per_step": {k: v["ms"] / r5["prof_steps"] for k, v in r5["prof"].items()}}
        out["prefill_pass"] = prefill_figure(E, path, args.ctx, local)
        for n_s in [int(x) for x in args.also_streams.split(",") if x.strip()]:
            if n_s >= args.streams:
                continue
            a2 = copy.copy(a0)
            a2.streams = n_s
            e2, _ = make_engine(E, path, n_s, args.ctx, total, local, args.attn_keys)
            r2 = run_replica(a2, rank, 1, solo, local, e2, args.replay_mistakes)
            r1 = run_replica(a2, rank, 1, solo, local, e2, 1.0)
            e2.close()
            entry = {"value": r1["emitted"] / (r1["dev_ms"] * 1e-3), "unit": "tokens/s (this rank)", "ms_per_step": r1["dev_ms"] / steps,
                     "e2e": r1["emitted"] / r1["wall"], "mean_accepted_len": r1["emitted"] / (steps * n_s),
                     "replay_pass": {"mistakes": args.replay_mistakes, "value": r2["emitted"] / (r2["dev_ms"] * 1e-3),
                                     "mean_accepted_len": r2["emitted"] / (steps * n_s), "ms_per_step": r2["dev_ms"] / steps},
                     "kernel_groups_ms_per_step": {k: v["ms"] / r1["prof_steps"] for k, v in r1["prof"].items()}}
            if with_drafter:
                a3 = copy.copy(args)
                a3.streams = n_s
                e3, _ = make_engine(E, path, n_s, args.ctx, total, local, args.attn_keys)
                e3.load_drafter(drafter_file(0, args.drafter_window))
                e3.set_acceptance(1 if args.top_p >= 1.0 else 0)
                r3 = run_replica(a3, rank, 1, solo, local, e3, 1.0, model_drafter=True)
                e3.close()
                entry["with_chain_drafter"] = {"value": r3["emitted"] / (r3["dev_ms"] * 1e-3), "ms_per_step": r3["dev_ms"] / steps, "mean_accepted_len": r3["emitted"] / (steps * n_s)}
            out[f"streams_{n_s}"] = entry
        if not args.bf16:
            # BASELINE configuration 2: the same target in bf16, one stream.
            ab = copy.copy(a0)
            ab.streams, ab.bf16 = 1, True
            eb, _ = make_engine(E, model_file("1b", False, 0), 1, args.ctx, total, local, args.attn_keys)
            rb = run_replica(ab, rank, 1, solo, local, eb, 1.0)
            eb.close()
            out["bf16_streams_1"] = {"value": rb["emitted"] / (rb["dev_ms"] * 1e-3), "unit": "tokens/s (this rank)", "ms_per_step": rb["dev_ms"] / steps, "e2e": rb["emitted"] / rb["wall"],
                                     "mean_accepted_len": rb["emitted"] / steps}
        if not args.no_limite:
            # Not BASELINE's metric: the reference's own architecture at its shapes through this library, plain decoding. It
            # needs a 2 GB random-init file written first; whatever goes wrong there is reported, not raised.
            try:
                out["reference_architecture_pass"] = limite_figure(E, local, args.ctx)
            except Exception as e:  # noqa: BLE001
                out["reference_architecture_pass"] = {"error": str(e)[:300]}
            try:  # the same target behind the reference's block drafter: trees of 8 rows drafted and verified
                out["reference_pairing_pass"] = limite_figure(E, local, args.ctx, stream_counts=(1, 32), drafter=True)
            except Exception as e:  # noqa: BLE001
                out["reference_pairing_pass"] = {"error": str(e)[:300]}
    if world == 1 and not args.no_cpu:
        t_step, cores, em = cpu_reference(args, args.cpu_streams, args.cpu_steps)
        out["cpu_baseline"] = {"value": em / t_step, "unit": "tokens/s", "cores": cores, "kind": "port",
                               "sample": f"{args.cpu_streams} streams x {args.cpu_steps} verify steps of 5 rows at ctx {args.ctx} ({t_step:.2f} s/step), every draft wrong"}
        t1, _, em1 = cpu_reference(args, 1, args.cpu_steps)
        out["cpu_baseline"]["one_stream"] = {"value": em1 / t1, "unit": "tokens/s", "sample": f"1 stream x {args.cpu_steps} verify steps of 5 rows at ctx {args.ctx} ({t1:.2f} s/step)"}
    print(json.dumps(out))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
