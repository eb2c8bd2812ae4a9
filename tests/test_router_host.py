"""The replica router on the host: streams dealt to the least-loaded replica, a failed replica's streams continued on the
others from the tokens they had emitted. The replicas here are stand-ins that behave like a Generator and emit, per
request, a token that is a function of the prompt and the position alone -- as an engine's draws are keyed by seed and
position -- so a moved request must end up with exactly the tokens it would have had."""
import pytest

from silicon_violetto_b200 import build, engine as E


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def token_at(prompt0: int, pos: int) -> int:
    return (prompt0 * 7919 + pos * 104729) % 50000


class FakeReplica:
    """One token per running request and step (a request's first step consumes its prompt), at most `slots` running."""

    def __init__(self, slots=4, fail_at=None, refuse_longer_than=None):
        self.slots, self.fail_at, self.refuse = slots, fail_at, refuse_longer_than
        self.queue, self.running, self.steps, self.next_id = [], [], 0, 0

    def submit(self, req):
        if self.refuse is not None and len(req.prompt) + req.max_tokens > self.refuse:
            raise RuntimeError("does not fit")
        self.queue.append(dict(id=self.next_id, key=req.prompt[0], pos=len(req.prompt), left=req.max_tokens, stop=set(req.stop), cancelled=False))
        self.next_id += 1
        return self.next_id - 1

    def step(self):
        self.steps += 1
        if self.fail_at is not None and self.steps >= self.fail_at:
            raise RuntimeError("device lost")
        while self.queue and len(self.running) < self.slots:
            self.running.append(self.queue.pop(0))
        out = []
        for r in self.running:
            tok = token_at(r["key"], r["pos"])
            r["pos"] += 1
            r["left"] -= 1
            out.append(E.Event("token", r["id"], tok))
            if tok in r["stop"] or r["left"] == 0 or r["cancelled"]:
                out.append(E.Event("done", r["id"], E.Finish.STOP if tok in r["stop"] else E.Finish.LENGTH))
                r["left"] = 0
        self.running = [r for r in self.running if r["left"] > 0]
        return out

    def cancel(self, rid):
        for r in self.queue + self.running:
            if r["id"] == rid:
                r["cancelled"] = True

    def is_idle(self):
        return not self.queue and not self.running

    def counts(self):
        return len(self.queue), len(self.running)


def drain(router, limit=1000):
    toks, done = {}, {}
    for _ in range(limit):
        if router.is_idle():
            break
        for ev in router.step():
            if ev.kind == "token":
                toks.setdefault(ev.req, []).append(ev.value)
            else:
                done[ev.req] = ev.value
    assert router.is_idle()
    return toks, done


def test_streams_are_dealt_out_evenly_and_finish():
    reps = [FakeReplica(), FakeReplica(), FakeReplica()]
    router = E.Router(reps)
    ids = [router.submit(E.Request([100 + i, 5, 6], 10 + i)) for i in range(9)]
    assert [router.replica_of(i) for i in ids] == [0, 1, 2, 0, 1, 2, 0, 1, 2]
    toks, done = drain(router)
    for i, rid in enumerate(ids):
        assert toks[rid] == [token_at(100 + i, 3 + p) for p in range(10 + i)]
        assert done[rid] == E.Finish.LENGTH
    assert router.alive() == 3


def test_a_failed_replicas_streams_continue_elsewhere_with_the_same_tokens():
    reps = [FakeReplica(slots=2), FakeReplica(slots=2, fail_at=6), FakeReplica(slots=2)]
    router = E.Router(reps)
    ids = [router.submit(E.Request([200 + i, 1], 20, stop=[token_at(200 + i, 17)] if i == 4 else [])) for i in range(9)]
    on_failed = [rid for rid in ids if router.replica_of(rid) == 1]
    assert len(on_failed) == 3
    toks, done = drain(router)
    assert router.alive() == 2
    for i, rid in enumerate(ids):
        want = [token_at(200 + i, 2 + p) for p in range(20)]
        if i == 4:
            want = want[:16]  # stops at its stop token (position 17), which it emits
        assert toks[rid] == want, f"request {i}"
        assert done[rid] == (E.Finish.STOP if i == 4 else E.Finish.LENGTH)
    assert reps[1].steps == 6  # the failed replica is not called again


def test_requests_nobody_can_take_end_as_failed_and_the_last_failure_stops_the_router():
    small = FakeReplica(refuse_longer_than=12)
    big = FakeReplica(fail_at=3)
    router = E.Router([big, small])
    a = router.submit(E.Request([300], 30))      # only `big` can hold it
    b = router.submit(E.Request([301], 5))       # goes to `small` (fewest requests)
    assert (router.replica_of(a), router.replica_of(b)) == (0, 1)
    toks, done = drain(router)
    assert done[a] == E.Finish.FAILED and len(toks[a]) == 2  # two steps' tokens before the failure, then nowhere to go
    assert done[b] == E.Finish.LENGTH and toks[b] == [token_at(301, 1 + p) for p in range(5)]
    only = E.Router([FakeReplica(fail_at=2)])
    c = only.submit(E.Request([1, 2], 9))
    only.step()
    assert [(e.kind, e.req, e.value) for e in only.step()] == [("done", c, E.Finish.FAILED)]
    assert only.is_idle() and only.alive() == 0
    with pytest.raises(E.EngineError, match="no replica is alive.*device lost|no replica is alive"):
        only.submit(E.Request([1, 2], 9))
    with pytest.raises(E.EngineError, match="token prompts only"):
        r = E._Request()
        r.prompt_kind = 1
        E._check(E.lib().vlt_router_submit(only.h, E.C.byref(r), E.C.byref(E.C.c_uint32())))
