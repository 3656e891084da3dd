"""A device-side wait that runs out, on ONE GPU and without faulting it: two ranks of a
world share device 0, only rank 0 launches its collective, and the poll limit is a few
thousand.  Nothing ever sets the flags rank 0 waits for, so its kernel gives up after the
limit, records HB_ERR_TIMEOUT in the world's status word and returns (the reference's
counterpart is the Err that nccl_all_reduce propagates, src/parallel/comm.rs:113-143).
Only one kernel is ever in flight, so nothing waits for a launch that cannot run."""
import numpy as np
import pytest
import torch

from oracle import kernels_ref as K

pytestmark = pytest.mark.gpu


@pytest.fixture()
def lonely_world(hb, cuda):
    ws = hb.TpWorld.new_local(2, device_ids=[0, 0], staging_bytes=8 << 20)
    for w in ws:
        w.set_wait_limit(3000)
    yield ws
    for w in ws:
        w.close()


@pytest.mark.parametrize("algo", ["one_shot", "two_shot"])
def test_exchange_norm_kernel_gives_up(hb, cuda, lonely_world, algo):
    w0 = lonely_world[0]
    code = {"one_shot": hb.ALGO_ONE_SHOT, "two_shot": hb.ALGO_TWO_SHOT}[algo]
    M, N = 8, 4096
    part = torch.ones(M, N, device=cuda, dtype=torch.bfloat16)
    resid = torch.ones(M, N, device=cuda, dtype=torch.bfloat16)
    nw = torch.ones(N, device=cuda, dtype=torch.bfloat16)
    assert w0.status() == 0
    w0.all_reduce_add_rms_norm(part, resid, nw, 1e-5, code)   # the peer never calls
    torch.cuda.synchronize()                                  # returns: the wait was bounded
    assert w0.status() == hb.ERR_TIMEOUT
    assert "wait" in hb.last_error()
    assert w0.status() == 0                                   # reading the status cleared it


def test_all_reduce_kernel_gives_up(hb, cuda, lonely_world):
    w0 = lonely_world[0]
    buf = torch.ones(64 * 1024, device=cuda, dtype=torch.float32)
    w0.all_reduce(buf, hb.ALGO_TWO_SHOT)
    torch.cuda.synchronize()
    assert w0.status() == hb.ERR_TIMEOUT
    # a second collective on the broken world reports for itself (its peer is still absent)
    w0.all_reduce(buf, hb.ALGO_ONE_SHOT)
    torch.cuda.synchronize()
    assert w0.status() == hb.ERR_TIMEOUT


def test_context_is_usable_after_a_timeout(hb, cuda, lonely_world):
    """The kernel returned an error status instead of trapping: the CUDA context lives on and
    the next kernels give right answers."""
    w0 = lonely_world[0]
    buf = torch.ones(4096, device=cuda, dtype=torch.float32)
    w0.all_reduce(buf)
    torch.cuda.synchronize()
    assert w0.status() == hb.ERR_TIMEOUT
    rng = np.random.default_rng(0)
    x = rng.standard_normal((4, 1024)).astype(np.float32)
    wgt = rng.standard_normal(1024).astype(np.float32)
    got = hb.kernels.rms_norm.apply(torch.from_numpy(x).to(cuda), torch.from_numpy(wgt).to(cuda), 1e-5)
    want = K.rms_norm_kernel(x, wgt, 1e-5, "f32")
    assert float(np.max(np.abs(got.cpu().numpy() - want))) <= 1e-3 * float(np.max(np.abs(want)))
    # a single-rank world is a passthrough and reports no error
    solo = hb.TpWorld.new_local(1)
    solo[0].all_reduce(buf)
    assert solo[0].status() == 0
    solo[0].close()
