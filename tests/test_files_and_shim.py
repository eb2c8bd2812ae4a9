"""The reference CLI's file formats (request files, JSONL outputs) round-trip, with its error messages; and the Rust shim
shipped as source declares exactly the C functions and struct fields of include/violetto.h that it uses."""
import json
import re
from pathlib import Path

import pytest

from silicon_violetto_b200 import engine as E, files

ROOT = Path(__file__).resolve().parents[1]


def test_request_files_round_trip(tmp_path):
    p = tmp_path / "reqs.txt"
    p.write_text("alpha - 1 2 3\n\n  beta seed=7,max_tokens=12,temperature=0.25,top_p=0.5   40 41\ngamma max_tokens=3\n")
    lines = files.read_requests(p)
    assert [(l.name, l.opts, l.prompt) for l in lines] == [("alpha", "-", [1, 2, 3]), ("beta", "seed=7,max_tokens=12,temperature=0.25,top_p=0.5", [40, 41]), ("gamma", "max_tokens=3", [])]
    s, mt = files.parse_options(lines[0], E.Sampling(0.6, 0.95, 5), 100)
    assert (s.temperature, s.top_p, s.seed, mt) == (0.6, 0.95, 5, 100)
    s, mt = files.parse_options(lines[1], E.Sampling(0.6, 0.95, 5), 100)
    assert (s.temperature, s.top_p, s.seed, mt) == (0.25, 0.5, 7, 12)
    files.write_requests(tmp_path / "again.txt", lines)
    assert [(l.name, l.opts, l.prompt) for l in files.read_requests(tmp_path / "again.txt")] == [(l.name, l.opts, l.prompt) for l in lines]


def test_request_file_errors_carry_the_references_wording(tmp_path):
    p = tmp_path / "bad.txt"
    p.write_text("ok - 1\nlonely\n")
    with pytest.raises(files.FormatError, match=r"bad.txt:2: no options \(`-` for none\)"):
        files.read_requests(p)
    p.write_text("x - 1 two 3\n")
    with pytest.raises(files.FormatError, match=r"bad.txt:1: bad token id two"):
        files.read_requests(p)
    for opts, msg in (("seed", "r: option seed isn't key=value"), ("speed=3", "r: unknown option speed"), ("top_p=high", "r: bad top_p high")):
        with pytest.raises(files.FormatError, match=msg):
            files.parse_options(files.RequestLine("r", opts, [1]), E.GREEDY, 10)


def test_outputs_round_trip(tmp_path):
    p = tmp_path / "out.jsonl"
    p.write_text(files.output_line("a", E.Finish.STOP, 3, [5, 6, 7]) + "\n\n" + files.output_line("b", E.Finish.LENGTH, 1, []) + "\n")
    first = json.loads(p.read_text().splitlines()[0])
    assert first == {"name": "a", "finish": "stop", "prompt_tokens": 3, "tokens": [5, 6, 7]}
    assert files.read_outputs(p) == {"a": [5, 6, 7], "b": []}
    for text, msg in (('{"tokens": [1]}', "no name"), ('{"name": "x"}', "no tokens"), ('{"name": "x", "tokens": [1, "2"]}', "tokens aren't ids"), ("{", r"out.jsonl:1: ")):
        p.write_text(text + "\n")
        with pytest.raises(files.FormatError, match=msg):
            files.read_outputs(p)


def _c_struct_fields(header: str, name: str):
    end = header.index("} " + name + ";")
    body = header[header.rindex("typedef struct {", 0, end) + len("typedef struct {"):end]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    fields = []
    for decl in body.split(";"):
        decl = decl.strip()
        if not decl:
            continue
        fn = re.match(r".*\(\*(\w+)\)\(", decl)  # a function pointer
        if fn:
            fields.append(fn.group(1))
            continue
        names = re.sub(r"^(const\s+)?\w+\s*\**", "", decl, count=1)
        fields += [re.sub(r"[\*\s]|\[.*\]", "", n) for n in names.split(",")]
    return fields


def test_rust_shim_declares_what_the_header_declares():
    header = (ROOT / "include" / "violetto.h").read_text()
    ffi = (ROOT / "silicon-violetto_b200" / "shim" / "engine-b200" / "src" / "ffi.rs").read_text()
    c_fns = set(re.findall(r"\b(vlt_[a-z0-9_]+)\s*\(", header))
    rust_fns = set(re.findall(r"pub fn (vlt_[a-z0-9_]+)\(", ffi))
    assert rust_fns and rust_fns <= c_fns, rust_fns - c_fns
    assert {"vlt_engine_new", "vlt_step", "vlt_step_capture", "vlt_generator_step", "vlt_router_step"} <= rust_fns
    for name in ("VltEngineConfig", "VltTuning", "VltSampling", "VltRun", "VltStepOptions", "VltStepOutput", "VltModelDesc", "VltLayerCapture", "VltRequest", "VltEvent",
                 "VltStepStats", "VltReplicaOps"):
        body = re.search(r"pub struct " + name + r" \{(.*?)\n\}", ffi, re.S).group(1)
        rust_fields = re.findall(r"pub (\w+):", body)
        assert rust_fields == _c_struct_fields(header, name), name
    lib = (ROOT / "silicon-violetto_b200" / "shim" / "engine-b200" / "src" / "lib.rs").read_text()
    for item in ("pub struct Engine", "pub struct Generator", "pub struct EngineConfig", "pub struct Tuning", "pub struct Sampling", "pub struct SeqId", "pub enum Rows",
                 "pub struct Run", "pub struct StepOptions", "pub struct StepOutput", "pub struct LayerCapture", "pub struct Request", "pub enum Draft", "pub enum Prompt",
                 "pub struct ReqId", "pub enum Finish", "pub enum Event", "pub struct StepStats", "pub mod skip"):
        assert item in lib, item  # the names engine/src/lib.rs:6-10 re-exports
