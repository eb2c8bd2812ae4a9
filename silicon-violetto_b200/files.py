"""The reference CLI's file formats (cli/src/files.rs, cli/src/generate.rs), so that request files and outputs move
between the two engines unchanged.

  request file   one request per non-blank line: `name opts id id id ...`; `opts` is `-` or comma-separated
                 key=value pairs among seed, max_tokens, temperature, top_p (cli/src/files.rs:28-53, cli/src/generate.rs:51-73)
  output file    one JSON object per line: {"name", "finish": "stop" | "length", "prompt_tokens", "tokens": [ids]}
                 (cli/src/generate.rs:127), read back as name -> tokens for --resume and --replay (cli/src/files.rs:56-72)

`generate` is the batch driver of cli/src/generate.rs:75-164 on this package's Engine / Generator.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field
from pathlib import Path

from . import engine as E

OPTION_KEYS = ("seed", "max_tokens", "temperature", "top_p")


class FormatError(ValueError):
    pass


@dataclass
class RequestLine:
    """cli/src/files.rs:31-36."""
    name: str
    opts: str
    prompt: list


def _number(at: str, what: str, text: str, kind):
    try:
        v = kind(text)
    except ValueError:
        raise FormatError(f"{at}: bad {what} {text}") from None
    if kind is int and v < 0:
        raise FormatError(f"{at}: bad {what} {text}")
    return v


def read_requests(path) -> list:
    """cli/src/files.rs:38-49 `requests`."""
    out = []
    for i, line in enumerate(Path(path).read_text().splitlines()):
        fields = line.split()
        if not fields:
            continue
        at = f"{path}:{i + 1}"
        if len(fields) < 2:
            raise FormatError(f"{at}: no options (`-` for none)")
        out.append(RequestLine(fields[0], fields[1], [_number(at, "token id", x, int) for x in fields[2:]]))
    return out


def write_requests(path, lines) -> None:
    Path(path).write_text("".join(f"{r.name} {r.opts} {' '.join(str(t) for t in r.prompt)}".rstrip() + "\n" for r in lines))


def parse_options(line: RequestLine, sampling: E.Sampling, max_tokens: int):
    """cli/src/generate.rs:55-67: the line's options over the command line's defaults -> (Sampling, max_tokens)."""
    s = E.Sampling(sampling.temperature, sampling.top_p, sampling.seed)
    for kv in line.opts.split(","):
        if kv == "-":
            continue
        if "=" not in kv:
            raise FormatError(f"{line.name}: option {kv} isn't key=value")
        k, v = kv.split("=", 1)
        if k == "seed":
            s.seed = _number(line.name, k, v, int)
        elif k == "max_tokens":
            max_tokens = _number(line.name, k, v, int)
        elif k == "temperature":
            s.temperature = _number(line.name, k, v, float)
        elif k == "top_p":
            s.top_p = _number(line.name, k, v, float)
        else:
            raise FormatError(f"{line.name}: unknown option {k}")
    return s, max_tokens


def output_line(name: str, finish: int, prompt_tokens: int, tokens) -> str:
    """cli/src/generate.rs:127."""
    return json.dumps({"name": name, "finish": "stop" if finish == E.Finish.STOP else "length", "prompt_tokens": prompt_tokens, "tokens": [int(t) for t in tokens]})


def read_outputs(path) -> dict:
    """cli/src/files.rs:56-72 `outputs`: name -> tokens."""
    out = {}
    for i, line in enumerate(Path(path).read_text().splitlines()):
        if not line.strip():
            continue
        bad = lambda what: FormatError(f"{path}:{i + 1}: {what}")
        try:
            v = json.loads(line)
        except json.JSONDecodeError as e:
            raise bad(str(e)) from None
        if not isinstance(v, dict) or not isinstance(v.get("name"), str):
            raise bad("no name")
        if not isinstance(v.get("tokens"), list):
            raise bad("no tokens")
        if not all(isinstance(t, int) and not isinstance(t, bool) and t >= 0 for t in v["tokens"]):
            raise bad("tokens aren't ids")
        out[v["name"]] = v["tokens"]
    return out


@dataclass
class GenerateArgs:
    """The options of cli/src/generate.rs:12-49 that shape the run."""
    requests: Path
    out: Path
    resume: bool = False
    max_seqs: int = 16
    max_tokens: int = 32768
    stop: list = field(default_factory=lambda: [151643, 151645])
    chunk: int = 512
    kv_tokens: int | None = None
    replay: Path | None = None
    replay_mistakes: float = 0.0
    drafter: Path | None = None
    spec_rows: int = 8
    temperature: float = 0.6
    top_p: float = 0.95
    seed: int = 0


def generate(weights, a: GenerateArgs, tuning: E.Tuning | None = None) -> dict:
    """cli/src/generate.rs:75-164: every request of the file through one generator, a JSON line per finished request;
    with `resume` the requests already in the output are kept and skipped. Returns counts for the caller's report."""
    lines = read_requests(a.requests)
    reqs = []
    for i, line in enumerate(lines):
        sampling, max_tokens = parse_options(line, E.Sampling(a.temperature, a.top_p, a.seed + i), a.max_tokens)  # SamplingArgs::with(0.6, i), cli/src/main.rs
        draft, rows, trace = (E.Draft.MODEL, a.spec_rows, []) if a.drafter else (E.Draft.NONE, 1, [])
        reqs.append((line.name, E.Request(list(line.prompt), max_tokens, list(a.stop), sampling, draft, rows, trace)))
    if a.replay:
        outs = read_outputs(a.replay)
        for name, r in reqs:
            if name in outs:
                r.draft, r.rows, r.trace = E.Draft.REPLAY, a.spec_rows, list(r.prompt) + list(outs[name])
    max_seqs = max(1, min(a.max_seqs, len(reqs)))
    longest = max((len(r.prompt) + r.max_tokens for _, r in reqs), default=1)
    drafts = bool(a.replay or a.drafter)
    cfg = E.EngineConfig(max_seqs=max_seqs, max_step_tokens=max(a.chunk, max_seqs), max_chunk=a.chunk,
                         global_kv_tokens=a.kv_tokens or max_seqs * (-(-longest // 128) * 128 + (16 if a.drafter else 0)), max_seq_len=longest,
                         max_head_rows=max_seqs * (a.spec_rows if drafts else 1))
    eng = E.Engine(weights, cfg, tuning)
    if a.drafter:
        eng.load_drafter(a.drafter)
    finished = read_outputs(a.out) if a.resume and Path(a.out).exists() else {}
    names, prompts, generated, done = [], [], 0, 0
    with open(a.out, "a" if finished else "w") as out, eng.generator() as g:
        g.set_replay_mistakes(a.replay_mistakes, 1)
        for name, r in reqs:
            if name in finished:
                continue
            prompts.append(len(r.prompt))
            try:
                g.submit(r)
            except E.EngineError as e:
                raise E.EngineError(f"{name}: {e}") from None
            names.append(name)
        tokens = [[] for _ in names]
        while not g.is_idle():
            for ev in g.step():
                if ev.kind == "token":
                    tokens[ev.req].append(ev.value)
                    generated += 1
                else:
                    out.write(output_line(names[ev.req], ev.value, prompts[ev.req], tokens[ev.req]) + "\n")
                    out.flush()
                    tokens[ev.req] = []
                    done += 1
        stats = g.take_stats()
    eng.close()
    return dict(requests=len(reqs), skipped=len(finished), done=done, generated=generated, steps=len(stats))
