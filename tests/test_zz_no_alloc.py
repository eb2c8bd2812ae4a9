"""vlt_spec_accept_static (the acceptance step with static scratch, nothing allocated) against
vlt_spec_accept and the CPU oracle on the same inputs, several calls in a row, on the default stream
and on a stream of the caller's; and the property in its name: the device's free memory does not
move across a call. Collected last on purpose: it must pass alone and after every other test has
used the device."""
import numpy as np
import pytest

import oracle
from silicon_violetto_b200 import build, engine as E, vlt
from tests import util

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def built():
    build.build()


def _case(streams, k, vocab, seed, temperature):
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal((streams, k + 1, vocab)) * 3.0).astype(np.float32)
    q = (p[:, :k] * 0.8 + rng.standard_normal((streams, k, vocab)) * 0.6).astype(np.float32)  # close to p: some drafts pass
    pb, qb = vlt.to_bf16(p), vlt.to_bf16(q)
    seeds = np.arange(streams, dtype=np.uint64) * np.uint64(104729) + np.uint64(seed)
    pos0 = rng.integers(1, 9000, streams).astype(np.uint32)
    drafts = oracle.draw_drafts(qb, temperature, seeds + np.uint64(1), pos0)
    return pb, qb, drafts, seeds, pos0


def _static(torch, pb, qb, drafts, temperature, seeds, pos0, stream=None, check_free=False):
    dev = torch.device("cuda:0")
    s, k, v = qb.shape
    t = lambda a, dt: torch.from_numpy(np.ascontiguousarray(a).view(dt)).to(dev)
    p_d, q_d = t(pb, np.int16), t(qb, np.int16)
    d_d, s_d, o_d = t(drafts.astype(np.uint32), np.int32), t(seeds, np.int64), t(pos0, np.int32)
    out = torch.full((3, s), -1, dtype=torch.int32, device=dev)
    stream = stream or torch.cuda.current_stream(dev)
    torch.cuda.synchronize(dev)  # the inputs are in place whatever stream the call uses
    free_before = torch.cuda.mem_get_info(dev)[0]
    E.spec_accept_static(p_d.data_ptr(), q_d.data_ptr(), d_d.data_ptr(), s, k, v, temperature, s_d.data_ptr(), o_d.data_ptr(), out[0].data_ptr(),
                         out[1].data_ptr(), out[2].data_ptr(), stream.cuda_stream)
    stream.synchronize()
    if check_free:  # cudaMemGetInfo: what the driver has handed out on the device, to anyone
        assert torch.cuda.mem_get_info(dev)[0] == free_before
    return out.cpu().numpy().view(np.uint32)


def test_static_scratch_variant_matches_the_allocating_one_twice_in_a_row():
    import torch
    torch.cuda.set_device(0)
    eng = E.Engine(util.weights("micro"), E.EngineConfig(max_seqs=2, max_step_tokens=16, max_chunk=8, global_kv_tokens=64, max_seq_len=64, max_head_rows=8))
    vocab = eng.desc.vocab
    some_accepted = False
    side = torch.cuda.Stream(device="cuda:0")  # a caller's own stream, not the default one
    # A large call, a small one over the same arrays, the first again (on the caller's stream), the small one again.
    for n, (streams, k, seed, temperature) in enumerate([(16, 7, 3, 1.0), (5, 1, 11, 0.6), (16, 7, 3, 1.0), (5, 1, 11, 0.6)]):
        pb, qb, drafts, seeds, pos0 = _case(streams, k, vocab, seed, temperature)
        acc, tok, rb, _ = eng.spec_accept(pb, qb, drafts, temperature, seeds, pos0)
        # The first call on a device is set-up (it looks up the arrays' addresses); from the second on nothing may move.
        got = _static(torch, pb, qb, drafts, temperature, seeds, pos0, stream=side if n >= 2 else None, check_free=n >= 1)
        assert np.array_equal(got[0], acc) and np.array_equal(got[1], tok) and np.array_equal(got[2], rb)
        want = oracle.spec_accept(pb, qb, drafts, temperature, seeds, pos0)
        assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1]) and np.array_equal(got[2], want[2])
        some_accepted |= bool(acc.max() >= 1)
    assert some_accepted


def test_static_scratch_variant_refuses_more_rows_than_it_holds():
    import torch
    torch.cuda.set_device(0)
    assert E.spec_accept_static_max_rows() == 2048
    x = torch.zeros(16, dtype=torch.int64, device="cuda:0")
    a = x.data_ptr()
    with pytest.raises(E.EngineError, match="2048 rows"):
        E.spec_accept_static(a, a, a, 200, 7, 256, 1.0, a, a, a, a, a)  # 200 * 15 rows: refused before anything is launched
    with pytest.raises(E.EngineError, match="temperature"):
        E.spec_accept_static(a, a, a, 2, 2, 256, 0.0, a, a, a, a, a)
