"""The error path of the chunked kernels, exercised without faulting the GPU.

Every in-kernel wait has a time limit; a wait that runs out makes the kernel record a code, drain what it has in
flight, free its tensor memory and return.  The host-side hook wkv6_debug_inject shortens the limit and makes the
forward skip the request for one chunk's input tiles, so that the wait for them runs out with no copy outstanding.
Nothing traps or hangs: the kernel returns normally and the context stays usable, which is what this test checks.
"""
import pytest
import torch

from oracle import wkv6_oracle as O

pytestmark = pytest.mark.gpu
N = 64


def _inputs(B, T, H, seed):
    d = O.make_inputs(B, T, H, N, seed=seed)
    t = {n: torch.tensor(d[n]).to(torch.bfloat16).cuda() for n in ("r", "k", "v", "w", "gy")}
    return t, torch.tensor(d["u"]).cuda()


@pytest.mark.parametrize("skip_chunk", [0, 2])
def test_wait_runs_out_and_the_context_survives(skip_chunk):
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200._lib import check, lib
    t, u = _inputs(1, 256, 2, 71)
    run = lambda: pkg.forward_raw(t["r"], t["k"], t["v"], t["w"], u, N, want_state=True, want_ckpt=True,
                                  variant=pkg.VARIANT_CHUNK)
    y0, s0, _ = run()
    torch.cuda.synchronize()
    assert lib.wkv6_device_status() == 0
    try:
        check(lib.wkv6_debug_inject(skip_chunk, 20))       # 20 ms limit; chunk `skip_chunk` is never requested
        run()
        torch.cuda.synchronize()                            # the kernel returns by itself
        assert lib.wkv6_device_status() == 1                # code of the wait for the input tiles
        assert lib.wkv6_device_status() == 0                # reading cleared the word
    finally:
        check(lib.wkv6_debug_inject(-1, 0))
    # normal operation again, bit-identical to the clean run, forward and backward
    y1, s1, ck = run()
    grads = pkg.backward_raw(t["r"], t["k"], t["v"], t["w"], u, t["gy"], N, ckpt=ck, variant=pkg.VARIANT_CHUNK)
    torch.cuda.synchronize()
    assert lib.wkv6_device_status() == 0
    assert torch.equal(y0, y1) and torch.equal(s0, s1)
    assert all(torch.isfinite(g.float()).all() for g in grads)
