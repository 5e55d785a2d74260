"""Where a chunk's time goes inside the chunked kernels: a developer's aid, not part of the operator.

``python star_rwkv6_b200/phase_timing.py build <lib.so>`` compiles an instrumented copy of the library (``-DWKV6_TIMING``:
lane 0 of every warp of CTA 0 stamps ``clock64()`` at the phase boundaries of every chunk, and the fast backward records
``%globaltimer`` at entry and exit and ``%smid`` of every CTA); ``python star_rwkv6_b200/phase_timing.py run <lib.so> [B]``
runs one forward + backward at B x T4096 x H32 x N64 (bf16, the benchmark distributions; B = 8 by default) on that build
and prints (1) per kernel the median time of every stamp relative to the start of its chunk, per warp, and (2) for the fast
backward how the CTAs were spread over the SMs and how long the paired and the single ones ran.  The numbers quoted in
``profiles/chunk_kernels_*.md`` come from these two commands.
"""
import ctypes
import os
import sys


def run(lib_path: str, B: int = 8):
    os.environ["WKV6_B200_LIB"] = lib_path
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    import numpy as np
    import torch
    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib
    T, H, N = 4096, 32, 64
    g = torch.Generator().manual_seed(0)
    mk = lambda s=1.0: (torch.randn(B, T, H * N, generator=g) * s).to(torch.bfloat16).cuda()
    r, k, v, gy = mk(0.125), mk(0.125), mk(0.125), mk()
    w = (torch.rand(B, T, H * N, generator=g) * 7 - 6).to(torch.bfloat16).cuda()
    u = (torch.randn(H, N, generator=g) * 0.1).cuda()
    L = ctypes.CDLL(lib_path)   # the two readers exist in instrumented builds only
    np.set_printoptions(linewidth=200)

    def dump(name, first, last):
        buf = (ctypes.c_longlong * (64 * 16 * 8))()
        L.wkv6_debug_timing(buf)
        a = np.array(buf[:]).reshape(64, 16, 8).astype(np.float64)
        per = a[1:, first, 0] - a[:-1, first, 0]
        print(f"{name}: cycles per chunk of CTA 0 (median over chunks 4..59): {np.median(per[4:60]):.0f}")
        rel = a - a[:, first:first + 1, 0:1]
        med = np.median(rel[4:60], axis=0)
        print("  stamp time relative to the chunk's first stamp; rows = stamp, columns = warp 0..7")
        for ph in range(first, last + 1):
            print("   ", ph, np.round(med[ph]).astype(int))

    for _ in range(3):
        y, _, ck = pkg.forward_raw(r, k, v, w, u, N, want_ckpt=True)
    torch.cuda.synchronize()
    dump("chunk_fwd_kernel", 2, 9)
    for _ in range(3):
        pkg.backward_raw(r, k, v, w, u, gy, N, ckpt=ck)
    torch.cuda.synchronize()
    dump("chunk_bwd_wide_kernel", 0, 11)

    buf = (ctypes.c_longlong * (1024 * 8))()
    L.wkv6_debug_cta_times(buf)
    a = np.array(buf[:]).reshape(1024, 8)[:min(B * H, 1024)].astype(np.float64)
    # the fast backward stamps %globaltimer at entry (0) and exit (7); the forward leaves its own stamps in 0..7 first, the
    # backward overwrites them
    smb = (ctypes.c_int * 1024)()
    L.wkv6_debug_cta_sm(smb)
    sm = np.array(smb[:])[:a.shape[0]]
    cnt = np.bincount(sm, minlength=sm.max() + 1)
    paired = cnt[sm] == 2
    t0 = a[:, 0].min()
    dur = (a[:, 7] - a[:, 0]) / 1e3
    print(f"fast backward: first entry to last exit {(a[:, 7].max() - t0) / 1e3:.1f} us; entries spread over "
          f"{(a[:, 0].max() - t0) / 1e3:.2f} us; SMs with two CTAs {(cnt == 2).sum()}, with one {(cnt == 1).sum()}")
    for name, sel in (("CTAs that share their SM", paired), ("CTAs alone on their SM", ~paired)):
        if sel.any():
            print(f"  {name}: duration min / median / max {dur[sel].min():.1f} / {np.median(dur[sel]):.1f} / {dur[sel].max():.1f} us")


if __name__ == "__main__":
    if len(sys.argv) >= 3 and sys.argv[1] == "build":
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        import build as _build
        print(_build.build_variant(os.path.abspath(sys.argv[2]), ["-DWKV6_TIMING"]))
    elif len(sys.argv) >= 3 and sys.argv[1] == "run":
        run(os.path.abspath(sys.argv[2]), int(sys.argv[3]) if len(sys.argv) > 3 else 8)
    else:
        print(__doc__)
