"""The host-buffer call (batch rows, and head groups of the first and last row, streamed through the GPU on several
streams) gives exactly the results of the one-piece device call."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_host_pipeline_matches_device_call():
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200.host import fwd_bwd_host
    B, T, H, N = 5, 320, 2, 64
    g = torch.Generator().manual_seed(0)
    mk = lambda s: (torch.randn(B, T, H * N, generator=g) * s).to(torch.bfloat16).pin_memory()
    r, k, v, gy = mk(0.125), mk(0.125), mk(0.125), mk(1.0)
    w = (torch.rand(B, T, H * N, generator=g) * 7 - 6).to(torch.bfloat16).pin_memory()
    u = torch.randn(H, N, generator=g) * 0.1
    for rows in (1, 2):
        out, gu = fwd_bwd_host(r, k, v, w, u, gy, N, rows_per_slice=rows, slots=3)
        d = {n: x.cuda() for n, x in (("r", r), ("k", k), ("v", v), ("w", w), ("gy", gy))}
        y, _, ck = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], u.cuda(), N, want_ckpt=True)
        gr, gk, gv, gw, gub = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], u.cuda(), d["gy"], N, ckpt=ck)
        for name, want in (("y", y), ("gr", gr), ("gk", gk), ("gv", gv), ("gw", gw)):
            assert torch.equal(out[name], want.cpu()), name
        assert torch.allclose(gu, gub.sum(0).cpu(), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("B", [1, 2, 4])
def test_host_pipeline_head_groups(B):
    """The first and the last row travel as two head groups each (pitched copies)."""
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200.host import HostPipeline
    T, H, N = 192, 8, 64
    g = torch.Generator().manual_seed(B)
    mk = lambda s: (torch.randn(B, T, H * N, generator=g) * s).to(torch.bfloat16).pin_memory()
    r, k, v, gy = mk(0.125), mk(0.125), mk(0.125), mk(1.0)
    w = (torch.rand(B, T, H * N, generator=g) * 7 - 6).to(torch.bfloat16).pin_memory()
    u = torch.randn(H, N, generator=g) * 0.1
    pipe = HostPipeline(T, H, N)
    sl = pipe.slices(B)
    assert len(sl) == (2 if B == 1 else B + 2) and sl[0] == (0, 1, 0, 4) and sl[-1] == (B - 1, B, 4, 8)
    cover = torch.zeros(B, H, dtype=torch.int32)
    for b0, b1, h0, h1 in sl:
        cover[b0:b1, h0:h1] += 1
    assert (cover == 1).all()
    out, gu = pipe.fwd_bwd(r, k, v, w, u, gy)
    out2, gu2 = HostPipeline(T, H, N, ramp=False).fwd_bwd(r, k, v, w, u, gy)
    d = {n: x.cuda() for n, x in (("r", r), ("k", k), ("v", v), ("w", w), ("gy", gy))}
    y, _, ck = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], u.cuda(), N, want_ckpt=True)
    gr, gk, gv, gw, gub = pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], u.cuda(), d["gy"], N, ckpt=ck)
    for name, want in (("y", y), ("gr", gr), ("gk", gk), ("gv", gv), ("gw", gw)):
        assert torch.equal(out[name], want.cpu()), name
        assert torch.equal(out2[name], want.cpu()), name
    assert torch.allclose(gu, gub.sum(0).cpu(), rtol=1e-5, atol=1e-6)
    assert torch.allclose(gu2, gub.sum(0).cpu(), rtol=1e-5, atol=1e-6)


def test_calls_in_flight():
    """submit / wait with several calls in flight (different inputs and different u per call, separate output tensors per
    call, more calls than the pipeline keeps in flight): every call delivers exactly what the same call made alone delivers."""
    from star_rwkv6_b200.host import HostPipeline
    B, T, H, N = 3, 128, 4, 64
    g = torch.Generator().manual_seed(7)
    mk = lambda s: (torch.randn(B, T, H * N, generator=g) * s).to(torch.bfloat16).pin_memory()
    calls = []
    for i in range(5):
        calls.append(dict(r=mk(0.125), k=mk(0.125), v=mk(0.125), gy=mk(1.0),
                          w=(torch.rand(B, T, H * N, generator=g) * 7 - 6).to(torch.bfloat16).pin_memory(),
                          u=torch.randn(H, N, generator=g) * 0.1))
    pipe = HostPipeline(T, H, N, slots=3)
    alone = [pipe.fwd_bwd(c["r"], c["k"], c["v"], c["w"], c["u"], c["gy"]) for c in calls]
    tickets = [pipe.submit(c["r"], c["k"], c["v"], c["w"], c["u"], c["gy"]) for c in calls]   # all five queued, then collected
    for i, t in enumerate(tickets):
        out, gu = pipe.wait(t)
        for name in ("y", "gr", "gk", "gv", "gw"):
            assert torch.equal(out[name], alone[i][0][name]), (i, name)
        assert torch.equal(gu, alone[i][1]), i
