"""The batch driver over the reference CLI's file formats (cli/src/generate.rs): a request file in, one JSON line per
request out, --resume keeps what is there, --replay drafts an earlier output's tokens and reproduces them."""
import json

import pytest

from silicon_violetto_b200 import build, engine as E, files
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def test_generate_writes_resumes_and_replays(tmp_path):
    w = util.weights("micro")
    reqs = tmp_path / "reqs.txt"
    files.write_requests(reqs, [files.RequestLine("a", "temperature=0,max_tokens=9", [3, 1, 4, 1, 5]), files.RequestLine("b", "temperature=0", [9, 2, 6, 5, 3, 5, 8, 9, 7]),
                               files.RequestLine("c", "seed=3,temperature=0.8,top_p=1,max_tokens=6", [2, 7, 1, 8])])
    out = tmp_path / "out.jsonl"
    args = files.GenerateArgs(requests=reqs, out=out, max_seqs=2, max_tokens=12, stop=[511], chunk=8)
    r = files.generate(w, args)
    assert (r["requests"], r["done"], r["skipped"]) == (3, 3, 0)
    first = files.read_outputs(out)
    lines = [json.loads(l) for l in out.read_text().splitlines()]
    assert {l["name"]: (l["prompt_tokens"], len(l["tokens"])) for l in lines} == {"a": (5, 9), "b": (9, 12), "c": (4, 6)}
    assert all(l["finish"] == "length" for l in lines)
    # --resume: drop one line, run again: only that request is generated, and (same seeds, same positions) with the same tokens.
    out.write_text("".join(l + "\n" for l in out.read_text().splitlines() if json.loads(l)["name"] != "b"))
    args.resume = True
    r = files.generate(w, args)
    assert (r["done"], r["skipped"]) == (1, 2)
    assert files.read_outputs(out) == first
    # --replay: the earlier output as drafts, no mistakes: the same tokens in fewer steps.
    out2 = tmp_path / "out2.jsonl"
    r2 = files.generate(w, files.GenerateArgs(requests=reqs, out=out2, max_seqs=2, max_tokens=12, stop=[511], chunk=8, replay=out, spec_rows=5))
    second = files.read_outputs(out2)
    assert second["a"] == first["a"] and second["b"] == first["b"]  # the greedy ones; "c" samples and follows its draws
    assert r2["steps"] < r["steps"] + 30
