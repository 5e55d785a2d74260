#!/usr/bin/env python
"""Benchmark of the WKV6 hot path: forward + backward at B8 T4096 H32 N64 bf16 (fp32 u, fp32 state).

    python bench.py --gpus N --steps K --warmup W            # this library
    python bench.py --impl reference --gpus N --steps K ...  # the reference algorithm on the host cores

One "step" is one forward plus one backward of the operator over one batch of seeded synthetic inputs
(r,k,v ~ N(0,1)/sqrt(N), w ~ U(-6,1), u ~ N(0,0.1), gy ~ N(0,1)).  With N GPUs the one workload is split over the
ranks by (batch, head) pairs, which are independent, so there is no data-path collective (``--scaling strong``, the
default); every rank first checks its shard against the unsplit kernels on the same data and the verdict is part of
the JSON line (``shard_check``), and a short run of the long-sequence workload (B1 T131072 H32, T sharded over the
ranks, states carried rank to rank) is reported under ``long_sequence``.  ``--scaling weak`` instead runs the full
workload on every rank.

Rank 0 prints one JSON line.  ``value`` is device-resident throughput (CUDA events, max over ranks);
``e2e`` is the same step driven through ``RWKVKernelOperator`` from pinned host buffers with the host<->device
copies inside the timed region; ``roofline`` relates the dominant kernel to the measured HBM copy bandwidth;
``cpu_baseline`` is the C restatement of the reference algorithm timed on the host cores on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

METRIC = "wkv6_fwd_bwd_mtokens_per_s"
UNIT = "Mtokens/s"
FALLBACK_HBM_GBS = 6650.0


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--variant", default="auto", choices=["auto", "seq", "chunk"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--B", type=int, default=8)
    ap.add_argument("--T", type=int, default=4096)
    ap.add_argument("--fast-channel", type=float, default=None,
                    help="not the benchmark distribution: channel 5 of every head gets this constant w (1.0 = 250 bits of decay "
                         "per chunk, which sends every sequence to the per-block reference points and the general backward)")
    ap.add_argument("--H", type=int, default=32)
    ap.add_argument("--N", type=int, default=64)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f32"])
    ap.add_argument("--segments", type=int, default=0,
                    help="cut every local sequence into this many segments along T (summaries + scan + seeded kernels); "
                         "0 = automatic: 1 when a rank has at least 256 (batch, head) sequences, else enough to reach 256")
    ap.add_argument("--tshard", action="store_true",
                    help="shard T over the ranks (long sequences): states are carried rank to rank; implies weak=False")
    ap.add_argument("--workload", default="train", choices=["train", "decode", "gn_gate", "shift_mix", "channel_mix_act", "lm_loss", "train_step", "inference"],
                    help="train: the headline metric (fwd+bwd).  decode: single-token state updates of an inference step "
                         "(B16 H64 N64, one fp32 state per layer, --layers of them, replayed from a CUDA graph).  gn_gate: the "
                         "fused per-head GroupNorm + gate after the WKV op, forward + backward, at the B, T, H of config 1.  shift_mix: the "
                         "five token-shift interpolations in front of the projections, forward + backward, same shape.  train_step: one "
                         "optimizer step of the 1.6B-shape RWKV-6 model (24 layers, d 2048, ffn 7168, vocab 65536, B8 T4096 per "
                         "GPU, bf16, AdamW, data parallel with NCCL gradient all-reduce when launched on several GPUs)")
    ap.add_argument("--no-checkpoint", action="store_true", help="train_step: keep all activations instead of recomputing blocks")
    ap.add_argument("--framework-loss", action="store_true",
                    help="train_step: torch's cross_entropy on an fp32 copy of the logits instead of the fused loss kernel")
    ap.add_argument("--decode-steps", type=int, default=256, help="inference: greedy decode steps after the prefill")
    ap.add_argument("--layers", type=int, default=32)
    ap.add_argument("--no-graph", action="store_true",
                    help="launch every step from Python instead of replaying CUDA graphs (one graph per kernel group and input set)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip timing the reference's own CUDA kernels (one-GPU runs)")
    ap.add_argument("--no-long-sequence", action="store_true", help="skip the T-sharded long-sequence leg of multi-GPU runs")
    ap.add_argument("--long-T", type=int, default=131072, help="sequence length of the long-sequence leg")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample-heads", type=int, default=0, help="(b,h) pairs in the CPU sample; 0 = auto")
    return ap.parse_args()


def workload_name(a):
    extra = f", channel 5 of every head at w = {a.fast_channel}" if getattr(a, "fast_channel", None) is not None else ""
    return f"wkv6 fwd+bwd B{a.B} T{a.T} H{a.H} N{a.N} {a.dtype}{extra}"


# ---- CPU baseline / reference arm -----------------------------------------------------------------

def cpu_fwd_bwd(a, pairs, reps):
    """Time the C restatement (fp32, all host threads) on `pairs` (b,h) sequences of full length T."""
    from oracle import c_oracle
    from oracle.wkv6_oracle import make_inputs
    d = make_inputs(1, a.T, pairs, a.N, seed=1)
    times = []
    for _ in range(reps):
        t0 = time.perf_counter()
        c_oracle.fwd(d["r"], d["k"], d["v"], d["w"], d["u"], a.N, dtype=np.float32)
        c_oracle.bwd(d["r"], d["k"], d["v"], d["w"], d["u"], d["gy"], a.N, dtype=np.float32)
        times.append(time.perf_counter() - t0)
    return times, c_oracle.threads()


def pick_sample(a, budget_s):
    """Number of (b,h) sequences per CPU step: the whole workload if it fits the time budget, else a
    multiple of the thread count that does."""
    from oracle import c_oracle
    threads = c_oracle.use_all_cores()  # torchrun sets OMP_NUM_THREADS=1 for its workers
    if a.cpu_sample_heads:
        return a.cpu_sample_heads, threads
    probe = max(threads, 8)
    t_probe, _ = cpu_fwd_bwd(a, probe, 2)
    per_pair = min(t_probe) / probe
    total = a.B * a.H
    if per_pair * total <= budget_s:
        return total, threads
    pairs = max(threads, int(budget_s / per_pair) // threads * threads)
    return min(pairs, total), threads


def sample_text(a, pairs):
    whole = "the whole workload: " if pairs == a.B * a.H else ""
    return (f"{whole}{pairs} of {a.B * a.H} (batch,head) sequences at full T={a.T}, fp32; "
            "C restatement of the reference loop, OpenMP over sequences")


def cpu_baseline(a):
    """Tokens/s on the host cores.  A token is one time step of all H heads, so P sequences of length T are
    P*T/H tokens."""
    pairs, threads = pick_sample(a, budget_s=4.0)
    times, _ = cpu_fwd_bwd(a, pairs, 3)
    best = min(times)
    tokens = pairs * a.T / a.H
    return {"value": tokens / best / 1e6, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": sample_text(a, pairs) + ", best of 3", "seconds_per_sample": best}


def run_reference(a):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # the sample per step is sized so that warm-up + steps take about two and a half minutes at most
    pairs, threads = pick_sample(a, budget_s=min(3.0, 150.0 / max(1, a.warmup + a.steps)))
    times, _ = cpu_fwd_bwd(a, pairs, a.warmup + a.steps)
    timed = times[a.warmup:]
    tokens = pairs * a.T / a.H
    total = sum(timed)
    val = tokens * len(timed) / total / 1e6
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": a.gpus, "steps": a.steps,
        "warmup": a.warmup, "ms_per_step": 1e3 * total / len(timed), "higher_is_better": True,
        "scaling": a.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_name(a)},
        "setup": {"note": "reference algorithm on the host cores only"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": sample_text(a, pairs) + " per step"},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ---- clocks ---------------------------------------------------------------------------------------

class ClockSampler:
    """SM clock and throttle reasons sampled while the steps run.  Preferred: NVML inside this process, from a thread
    (a query costs microseconds and leaves the GPU alone).  Fallback: an ``nvidia-smi -lms 200`` child process, whose
    start-up and queries were measured to slow the timed steps by 4-5 % and occasionally much more."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index = index
        self.f = None
        self.p = None
        self.thread = None
        self.samples = []  # (sm MHz, max MHz, reason bit mask)

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.index).uuid)
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            mx = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            self._stop = threading.Event()

            def loop():
                while True:
                    try:
                        self.samples.append((nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM), mx,
                                             nv.nvmlDeviceGetCurrentClocksEventReasons(h)))
                    except Exception:
                        pass
                    if self._stop.wait(0.1):
                        return

            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
            self.p = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}",
                                       "--format=csv,noheader,nounits", "-lms", "200"],
                                      stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            if self.samples:
                mask = 0
                for _, _, m in self.samples:
                    mask |= int(m)
                out.update(sm_mhz=float(statistics.median(x[0] for x in self.samples)), sm_max_mhz=float(self.samples[0][1]),
                           reasons=sorted(n for bit, n in self.REASONS.items() if mask & bit), samples=len(self.samples),
                           source="nvml")
            return out
        if self.p is None:
            return out
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.f.read().splitlines():
            c = [x.strip() for x in ln.split(",")]
            if len(c) < 9:
                continue
            try:
                sm.append(float(c[1])); mx.append(float(c[2]))
            except ValueError:
                continue
            for nm, val in zip(names, c[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(nm)
        self.f.close()
        os.unlink(self.f.name)
        if sm:
            out.update(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))
        return out


# ---- GPU arm --------------------------------------------------------------------------------------

def _scaled_err(a, b):
    import torch
    den = float(b.float().abs().max())
    return float((a.float() - b.float()).abs().max()) / (den if den > 0 else 1.0)


FAST_CHANNEL_W = None   # --fast-channel: one channel per head gets this constant w (a decay spectrum with a fast channel)


def _device_inputs(torch, dev, B, T, C, H, N, xdt, seed):
    """One seeded input set, generated on the device (the same values on every rank for the same seed)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    mk = lambda s: (torch.randn(B, T, C, generator=g, device=dev) * s).to(xdt)
    w = torch.rand(B, T, C, generator=g, device=dev) * 7.0 - 6.0
    if FAST_CHANNEL_W is not None:
        w.view(B, T, H, N)[..., 5] = FAST_CHANNEL_W
    d = {"r": mk(N ** -0.5), "k": mk(N ** -0.5), "v": mk(N ** -0.5), "w": w.to(xdt), "gy": mk(1.0)}
    u = torch.randn(H, N, generator=g, device=dev) * 0.1
    return d, u


def run_b200(a):
    import torch
    import torch.distributed as dist
    global FAST_CHANNEL_W
    FAST_CHANNEL_W = a.fast_channel

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != a.gpus and world > 1:
        raise SystemExit(f"--gpus {a.gpus} but WORLD_SIZE={world}")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)

    import star_rwkv6_b200 as pkg
    from star_rwkv6_b200 import _lib, segments as seg, sharding
    from star_rwkv6_b200.rwkv_kernel.torch_rwkv_kernel import RWKVKernelOperator

    N = a.N
    xdt = torch.bfloat16 if a.dtype == "bf16" else torch.float32
    variant = _lib.VARIANTS[a.variant]
    strong = a.scaling == "strong" and world > 1 and not a.tshard
    plan = sharding.make_plan(a.B, a.H, world) if strong else None
    B, T, H = a.B, a.T, a.H
    if a.tshard and world > 1:
        assert T % world == 0
        T = T // world                                            # each rank holds a contiguous T range
    elif strong:
        B, H = plan.local_shape()
    C = H * N
    chunk_ok = a.dtype == "bf16" and N == 64 and a.variant != "seq"
    if a.segments == 0:
        a.segments = seg.auto_segments(B, T, H) if chunk_ok else 1

    # Seeded synthetic inputs, generated on the device; two rotating sets so that consecutive steps do not reuse cache
    # lines.  A split run generates the whole workload on every rank (same seed, same values) and keeps its shard.
    nsets = 2
    devs, globals0 = [], None
    for sidx in range(nsets):
        if strong:
            gd, gu_ = _device_inputs(torch, dev, a.B, a.T, a.H * N, a.H, N, xdt, 1234 + sidx)
            devs.append({n: x.contiguous() for n, x in zip(("r", "k", "v", "w", "gy"),
                                                          sharding.shard(plan, rank, N, *(gd[n] for n in ("r", "k", "v", "w", "gy"))))})
            if sidx == 0:   # one u for every input set
                u = sharding.shard_u(plan, rank, gu_).contiguous()
                globals0 = (gd, gu_)
            del gd
        else:
            d, u_ = _device_inputs(torch, dev, B, T, C, H, N, xdt, 1234 + sidx)  # T-sharded runs: every rank its own range
            devs.append(d)
            if sidx == 0:
                u = u_
    host = [{n: t.cpu().pin_memory() for n, t in d.items()} for d in devs]
    u_host = u.cpu().pin_memory()

    resolved = pkg.ops.resolve_variant(devs[0]["r"], u, N, variant)
    vname = {1: "seq", 2: "chunk"}[resolved]
    launches_per_step = {"seq": 4, "chunk": 3}[vname]  # chunk: forward, fast backward, general backward (exits at once when nothing is flagged)
    segmented = a.segments > 1 or (a.tshard and world > 1)
    collective = a.tshard and world > 1
    if segmented:
        assert vname == "chunk", "sequence splitting uses the chunked kernels"
        be = seg.LibraryBackend(N, reuse_buffers=not collective)
        grp = dist.group.WORLD if collective else None
        launches_per_step = 8  # forward: summary, scan, kernel; backward: summary, scan, fast + general kernel, gu row sum

        def step(d):
            y, _, ctx = seg.segmented_forward(be, d["r"], d["k"], d["v"], d["w"], u, a.segments, want_ckpt=True, group=grp,
                                              need_last=False)  # the step returns y and the gradients, not the final state
            return y, ctx

        def step_bwd(d, ctx):
            return seg.segmented_backward(be, ctx, d["r"], d["k"], d["v"], d["w"], u, d["gy"])
    else:
        def step(d):
            y, _, ckpt = pkg.forward_raw(d["r"], d["k"], d["v"], d["w"], u, N, want_ckpt=True, variant=variant)
            return y, ckpt

        def step_bwd(d, ckpt):
            return pkg.backward_raw(d["r"], d["k"], d["v"], d["w"], u, d["gy"], N, ckpt=ckpt, variant=variant)

    # ---- a split run first proves its split: the shard's results against the unsplit kernels on the whole workload
    shard_check = None
    if strong:
        gd, gu_ = globals0
        yg, _, ckg = pkg.forward_raw(gd["r"], gd["k"], gd["v"], gd["w"], gu_, N, want_ckpt=True, variant=variant)
        gg = pkg.backward_raw(gd["r"], gd["k"], gd["v"], gd["w"], gu_, gd["gy"], N, ckpt=ckg, variant=variant)
        bs, cs = plan.batch_slice(rank), plan.channel_slice(rank, N)
        want = [yg[bs, :, cs]] + [x[bs, :, cs] for x in gg[:4]]
        gu_ref = gg[4][bs].sum(0)[plan.head_slice(rank)]
        d0 = devs[0]
        # (1) the shard through the same kernels, one piece per sequence: bit for bit the slice of the whole run
        y1, _, ck1 = pkg.forward_raw(d0["r"], d0["k"], d0["v"], d0["w"], u, N, want_ckpt=True, variant=variant)
        g1 = pkg.backward_raw(d0["r"], d0["k"], d0["v"], d0["w"], u, d0["gy"], N, ckpt=ck1, variant=variant)
        bit_equal = all(torch.equal(x, y_) for x, y_ in zip([y1, *g1[:4]], want)) and torch.equal(g1[4].sum(0), gu_ref)
        # (2) the step that is timed (its sequences cut into segments when the shard alone cannot fill the GPU)
        ys, ck = step(d0)
        gs = step_bwd(d0, ck)
        torch.cuda.synchronize()
        gu_got = gs[4] if gs[4].dim() == 2 else gs[4].sum(0)
        worst = max([_scaled_err(x, y_) for x, y_ in zip([ys, *gs[:4]], want)] + [_scaled_err(gu_got, gu_ref)])
        status = _lib.lib.wkv6_device_status()
        flags = torch.tensor([1.0 if bit_equal else 0.0, 1.0 if (worst <= 1e-2 and status == 0) else 0.0, -worst], device=dev,
                             dtype=torch.float64)
        dist.all_reduce(flags, op=dist.ReduceOp.MIN)
        shard_check = {"bxh_bit_equal": bool(flags[0].item() == 1.0),
                       "timed_step_within_1e-2_of_unsplit": bool(flags[1].item() == 1.0), "max_scaled_err": -flags[2].item(),
                       "against": "forward + backward of the whole workload through the unsplit kernels on every rank, "
                                  "compared on the rank's (batch, head) shard: y, gr, gk, gv, gw, gu",
                       "segments_per_sequence_in_timed_step": a.segments}
        del gd, gu_, yg, ckg, gg, ys, ck, gs, globals0, want, y1, ck1, g1
        torch.cuda.empty_cache()

    # clocks are sampled from the warm-up on: the timed region itself can be shorter than one sampling period
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for i in range(max(3, a.warmup)):  # never fewer than three warm-up steps
        d = devs[i % nsets]
        y, ck = step(d)
        step_bwd(d, ck)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # The timed steps replay CUDA graphs (forward and backward captured separately per input set, so that the events
    # between them stay outside the graphs): a step then costs the host three event records and two replays, and a
    # busy host cannot stretch the measured kernels.  Runs with a collective inside the step (T sharded over ranks)
    # stay eager.
    graphs = None
    if not a.no_graph and not collective:
        graphs = []
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for d in devs:
                if segmented:
                    be = seg.LibraryBackend(N, reuse_buffers=True)   # one buffer set per captured input set
                gf = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gf, stream=side):
                    y, ck = step(d)
                gb = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gb, pool=gf.pool(), stream=side):
                    grads = step_bwd(d, ck)
                graphs.append((gf, gb, (y, ck, grads)))
        torch.cuda.current_stream().wait_stream(side)
        for i in range(4):
            graphs[i % nsets][0].replay(); graphs[i % nsets][1].replay()
        torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(a.steps)]
    e_start, e_stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e_start.record()
    for i in range(a.steps):
        ev[i][0].record()
        if graphs is not None:
            graphs[i % nsets][0].replay()
            ev[i][1].record()
            graphs[i % nsets][1].replay()
        else:
            d = devs[i % nsets]
            y, ck = step(d)
            ev[i][1].record()
            grads = step_bwd(d, ck)
        ev[i][2].record()
    e_stop.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = e_start.elapsed_time(e_stop)
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    if world > 1:
        t = torch.tensor([total_ms, fwd_ms, bwd_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, fwd_ms, bwd_ms = t.tolist()
    ms_per_step = total_ms / a.steps
    tokens_per_step_global = B * T * world  # weak scaling: every rank processes B*T tokens of H heads
    if (strong or a.tshard) and world > 1:
        tokens_per_step_global = a.B * a.T
    value = tokens_per_step_global / (ms_per_step * 1e-3) / 1e6
    device_status = _lib.lib.wkv6_device_status()

    # e2e: through the operator, host buffers, copies inside the timed region
    e2e = None
    if not a.no_e2e and not collective:
        op = RWKVKernelOperator(N, T, variant=a.variant)
        ydt = xdt
        out_host = {n: torch.empty(B, T, C, dtype=ydt).pin_memory() for n in ("y", "gr", "gk", "gv", "gw")}
        gu_host = torch.empty(H, N, dtype=torch.float32).pin_memory()

        def e2e_step(hs):
            t = {n: hs[n].to(dev, non_blocking=True) for n in ("r", "k", "v", "w", "gy")}
            ud = u_host.to(dev, non_blocking=True).requires_grad_(True)
            for n in ("r", "k", "v", "w"):
                t[n].requires_grad_(True)
            y, _ = op(t["r"], t["k"], t["v"], t["w"], ud)
            y.backward(t["gy"])
            out_host["y"].copy_(y.detach(), non_blocking=True)
            out_host["gr"].copy_(t["r"].grad, non_blocking=True)
            out_host["gk"].copy_(t["k"].grad, non_blocking=True)
            out_host["gv"].copy_(t["v"].grad, non_blocking=True)
            out_host["gw"].copy_(t["w"].grad, non_blocking=True)
            gu_host.copy_(ud.grad, non_blocking=True)

        from star_rwkv6_b200.host import HostPipeline
        pipe = HostPipeline(T, H, N, dtype=xdt, device=dev, rows_per_slice=1, slots=6, variant=variant)

        def host_step(hs):  # the package's host-buffer call: batch rows streamed through the GPU, copies overlapped
            pipe.fwd_bwd(hs["r"], hs["k"], hs["v"], hs["w"], u_host, hs["gy"], out=out_host)

        out_host2 = {n: torch.empty(B, T, C, dtype=ydt).pin_memory() for n in ("y", "gr", "gk", "gv", "gw")}

        def timed_two_in_flight():
            """The same calls as a loop keeps them: step i + 1 is submitted before step i is waited for (its own output
            tensors per step in flight), so the copies back of one step run beside the copies in of the next.  Every
            step's copies in and out lie inside the timed region; the time per step is the total over the steps."""
            n = max(3, min(a.steps, 10))
            outs = (out_host, out_host2)
            for i in range(2):
                pipe.fwd_bwd(host[i % nsets]["r"], host[i % nsets]["k"], host[i % nsets]["v"], host[i % nsets]["w"], u_host,
                             host[i % nsets]["gy"], out=outs[i & 1])
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            prev = None
            for i in range(n):
                hs = host[i % nsets]
                t = pipe.submit(hs["r"], hs["k"], hs["v"], hs["w"], u_host, hs["gy"], out=outs[i & 1])
                if prev is not None:
                    pipe.wait(prev)
                prev = t
            pipe.wait(prev)
            s1.record()
            barrier()
            ms = s0.elapsed_time(s1) / n
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
            return ms, n

        def timed(fn):
            n = max(3, min(a.steps, 10))
            for i in range(2):
                fn(host[i % nsets])
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for i in range(n):
                fn(host[i % nsets])
            s1.record()
            barrier()
            ms = s0.elapsed_time(s1) / n
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = t.item()
            return ms, n

        op_ms, n_e2e = timed(e2e_step)
        call_ms, _ = timed(host_step)
        pipe.ramp = False   # with the next step's fill beside this step's drain, whole rows (plain copies) are faster than head groups
        e2e_ms, _ = timed_two_in_flight()
        esz = 2 if a.dtype == "bf16" else 4
        e2e = {"value": tokens_per_step_global / (e2e_ms * 1e-3) / 1e6, "unit": UNIT,
               "h2d_bytes_per_step": 5 * B * T * C * esz + H * N * 4,
               "d2h_bytes_per_step": 5 * B * T * C * esz + H * N * 4,
               "bytes_are": "per rank",
               "ms_per_step": e2e_ms, "steps": n_e2e,
               "api": "star_rwkv6_b200.host.HostPipeline.submit / wait on pinned host tensors (batch rows streamed, both copy "
                      "directions and the kernels overlapped; step i + 1 submitted before step i is waited for, separate output "
                      "tensors per step in flight)",
               "one_call_at_a_time": {"value": tokens_per_step_global / (call_ms * 1e-3) / 1e6, "ms_per_step": call_ms,
                                      "api": "HostPipeline.fwd_bwd, which returns when its results are in host memory"},
               "operator_on_device_copies": {"value": tokens_per_step_global / (op_ms * 1e-3) / 1e6, "ms_per_step": op_ms,
                                             "api": "copy everything in, RWKVKernelOperator.__call__ + backward, copy everything out"}}
        del pipe, out_host, out_host2

    # ---- one GPU: the reference's own CUDA kernels on the first input set, beside this library's results for it
    ref_cuda_res = None
    if world == 1 and not segmented and vname == "chunk" and not a.no_reference_cuda:
        yo, cko = step(devs[0])
        ref_cuda_res = reference_cuda_leg(a, torch, pkg, devs[0], u, N, (yo, step_bwd(devs[0], cko)))
        del yo, cko

    # ---- multi-GPU runs add a short leg of the long-sequence workload, T sharded over the ranks
    long_seq = None
    launch_mode = "CUDA graph replays (forward, backward)" if graphs is not None else "eager launches"
    if world > 1 and not a.no_long_sequence and not a.tshard and chunk_ok:
        del devs, host, graphs, y, ck, grads
        torch.cuda.empty_cache()
        long_seq = long_sequence_leg(a, torch, dist, pkg, seg, dev, rank, world, N)

    if rank == 0:
        peak, peak_src = measured_peak()
        esz = 2 if a.dtype == "bf16" else 4
        elems = B * T * C          # per rank
        bwd_bytes, fwd_bytes = 9 * esz * elems, 5 * esz * elems
        # dram__bytes_read.sum + dram__bytes_write.sum of one backward launch: per (token, channel) figure of the ncu
        # capture whose summary sits beside it (traffic grows in proportion to the (batch, head) sequences)
        traffic = None
        per_elem = profiled_traffic_per_element()
        if per_elem is not None and vname == "chunk" and a.dtype == "bf16" and not segmented:
            traffic = per_elem * elems
        achieved = bwd_bytes / (bwd_ms * 1e-3) / 1e9
        roofline = {
            "bound": "hbm", "kernel": f"{vname} backward", "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": traffic, "peak_source": peak_src,
            "algorithmic_bytes_per_launch": bwd_bytes, "avg_ms": bwd_ms, "figures_are": "per GPU",
            "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                        "algorithmic_bytes_per_launch": fwd_bytes, "avg_ms": fwd_ms},
            "step": {"achieved": (fwd_bytes + bwd_bytes) / (ms_per_step * 1e-3) / 1e9,
                     "frac": (fwd_bytes + bwd_bytes) / (ms_per_step * 1e-3) / 1e9 / peak},
        }
        cpu = None if (a.no_cpu_baseline or world > 1) else cpu_baseline(a)  # a one-GPU figure
        if collective:
            par = f"T sharded over {world} ranks, states carried by all-gather + scan"
        elif strong:
            par = (f"one workload split over {world} ranks by (batch, head): {plan.batch_parts} batch x {plan.head_parts} head "
                   "parts, no collective")
        else:
            par = f"{world} independent ranks, each the whole workload, no collective"
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": a.steps, "warmup": max(3, a.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong" if (a.tshard or strong or world == 1 and a.scaling == "strong") else "weak", "vs_baseline": None,
            "dtype": "bf16" if a.dtype == "bf16" else "f32", "data": "synthetic",
            "config": {"workload": workload_name(a),
                       "l2": f"two rotating input sets; a step touches {(5 + 5 + 1) * elems * esz / 1e6:.0f} MB per GPU (5 inputs, 5 outputs, "
                             "checkpoints), more than the 126 MB L2, and the next step uses the other set"},
            "setup": {"per_gpu": f"B{B} T{T} H{H} N{N}", "variant": vname,
                       "u_dtype": "f32", "state": "f32",
                       "segments_per_sequence": a.segments,
                       "launch": launch_mode,
                       "parallelism": par},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "clocks": clocks,
            "gpu_launches": launches_per_step * a.steps, "device_status": device_status,
        }
        if ref_cuda_res is not None:
            line["reference_cuda"] = ref_cuda_res
        if shard_check is not None:
            line["shard_check"] = shard_check
        if long_seq is not None:
            line["long_sequence"] = long_seq
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def reference_cuda_leg(a, torch, pkg, d, u, N, ours):
    """The reference's own CUDA kernels (rwkv_kernels.cu compiled unchanged for sm_100a into oracle/_ref/, see
    oracle/build_ref_cuda.py) on the same inputs on this GPU: a reported baseline beside the host-core one."""
    from oracle import ref_cuda
    if not ref_cuda.available():
        return {"unavailable": "oracle/_ref/libref_wkv6_cuda.so has not been built (it is compiled where the reference tree is at hand)"}
    B, T, C = d["r"].shape
    if N != ref_cuda.HEAD_SIZE or T > ref_cuda.MAX_T or T < 3 or a.dtype != "bf16":
        return {"unavailable": f"the reference kernels are compiled for head size {ref_cuda.HEAD_SIZE}, T <= {ref_cuda.MAX_T}"}
    ub = u.to(d["r"].dtype)                               # the reference takes u in the dtype of r, k, v, w
    y = torch.empty_like(d["r"])
    g = [torch.empty_like(d["r"]) for _ in range(4)]
    gu = torch.empty((B, C), dtype=d["r"].dtype, device=d["r"].device)
    st = torch.cuda.current_stream().cuda_stream

    def step():
        ref_cuda.forward(d["r"], d["k"], d["v"], d["w"], ub, y, st)
        ref_cuda.backward(d["r"], d["k"], d["v"], d["w"], ub, d["gy"], *g, gu, st)

    step()
    torch.cuda.synchronize()
    if ref_cuda.lib().ref_wkv6_last_cuda_error() != 0:
        return {"unavailable": "the reference kernels reported a CUDA error on their first launch"}
    for _ in range(2):
        step()
    steps = 5
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    e[0].record()
    for _ in range(steps):
        ref_cuda.forward(d["r"], d["k"], d["v"], d["w"], ub, y, st)
    e[1].record()
    for _ in range(steps):
        ref_cuda.backward(d["r"], d["k"], d["v"], d["w"], ub, d["gy"], *g, gu, st)
    e[2].record()
    torch.cuda.synchronize()
    fwd_ms, bwd_ms = e[0].elapsed_time(e[1]) / steps, e[1].elapsed_time(e[2]) / steps
    yo, go = ours
    agree = max([_scaled_err(y, yo)] + [_scaled_err(x, x0) for x, x0 in zip(g, go[:4])]
                + [_scaled_err(gu.view(go[4].shape), go[4])])
    peak, _ = measured_peak()
    ms = fwd_ms + bwd_ms
    return {"value": B * T / (ms * 1e-3) / 1e6, "unit": UNIT, "ms_per_step": ms, "forward_ms": fwd_ms, "backward_ms": bwd_ms,
            "steps": steps, "warmup": 3, "roofline_step_frac": 28.0 * B * T * C / (ms * 1e-3) / 1e9 / peak,
            "kernels": "rwkv_kernel/jax_kernel/rwkv_kernels.cu of the reference, unchanged, nvcc -O3 -DNDEBUG for sm_100a, "
                       "_N_=64 _T_=4096; forward 1 launch, backward 4 launches",
            "max_scaled_difference_to_this_library": agree}


def long_sequence_leg(a, torch, dist, pkg, seg, dev, rank, world, N):
    """B1 T131072 H32 bf16, T sharded over the ranks: per-head states carried rank to rank (all-gather of the segment
    summaries over NCCL + scan), checked on every rank against the unsplit kernels run over the whole sequence."""
    from star_rwkv6_b200 import _lib
    B, T, H = 1, a.long_T, 32
    C = H * N
    Tl = T // world
    gd, u = _device_inputs(torch, dev, B, T, C, H, N, torch.bfloat16, 4321)
    sl = slice(rank * Tl, (rank + 1) * Tl)
    loc = {n: x[:, sl].contiguous() for n, x in gd.items()}
    G = seg.auto_segments(B, Tl, H)
    be = seg.LibraryBackend(N)
    grp = dist.group.WORLD

    def step():
        y, _, ctx = seg.segmented_forward(be, loc["r"], loc["k"], loc["v"], loc["w"], u, G, want_ckpt=True, group=grp)
        return y, seg.segmented_backward(be, ctx, loc["r"], loc["k"], loc["v"], loc["w"], u, loc["gy"])

    y, g = step()
    # the single-GPU result: the same sequence in one piece on this rank (cut into segments inside the GPU only)
    G1 = seg.auto_segments(B, T, H)
    y1, _, ctx1 = seg.segmented_forward(be, gd["r"], gd["k"], gd["v"], gd["w"], u, G1, want_ckpt=True)
    g1 = seg.segmented_backward(be, ctx1, gd["r"], gd["k"], gd["v"], gd["w"], u, gd["gy"])
    torch.cuda.synchronize()
    errs = [_scaled_err(y, y1[:, sl])] + [_scaled_err(x, x1[:, sl]) for x, x1 in zip(g[:4], g1[:4])] + [_scaled_err(g[4], g1[4])]
    status = _lib.lib.wkv6_device_status()
    flags = torch.tensor([1.0 if (max(errs) <= 1e-2 and status == 0) else 0.0, -max(errs)], device=dev, dtype=torch.float64)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    del y1, ctx1, g1, gd
    torch.cuda.empty_cache()
    for _ in range(3):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    # one CUDA graph per step, the NCCL all-gathers of the summaries inside it (eager launches when capture is refused)
    run, launch = step, "eager launches, NCCL all-gather of the summaries inside every step"
    if not a.no_graph:
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=side):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            graph.replay()
            torch.cuda.synchronize()
            run, launch = graph.replay, "one CUDA graph replay per step, the NCCL all-gathers of the summaries captured in it"
        except Exception as exc:  # noqa: BLE001
            launch += f" (graph capture refused: {type(exc).__name__})"
            torch.cuda.synchronize()
    ok = torch.tensor([1.0 if run is not step else 0.0], device=dev)
    dist.all_reduce(ok, op=dist.ReduceOp.MIN)      # every rank must take the same path: collectives pair up across ranks
    if ok.item() == 0.0:
        run = step
    dist.barrier()
    torch.cuda.synchronize()
    steps = 10
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        run()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / steps], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    peak, _ = measured_peak()
    return {"workload": f"wkv6 fwd+bwd B{B} T{T} H{H} N{N} bf16, T sharded over {world} ranks, {G} segments per rank",
            "ms_per_step": ms, "value": B * T / (ms * 1e-3) / 1e6, "unit": UNIT, "steps": steps, "warmup": 3,
            "roofline_step_frac": 28.0 * B * Tl * C / (ms * 1e-3) / 1e9 / peak,
            "launch": launch,
            "matches_single_gpu": bool(flags[0].item() == 1.0), "max_scaled_err_vs_single_gpu": -flags[1].item(),
            "against": "the same sequence through the kernels of one GPU (every rank runs it whole), all of y, gr, gk, gv, gw, gu"}


def profiled_traffic_per_element():
    """DRAM bytes per (token, channel) of one launch of the chunked backward, from the figure stored beside the ncu
    summary it was captured for (profiles/chunk_backward_dram_bytes.json); None when that file is absent."""
    path = os.path.join(ROOT, "profiles", "chunk_backward_dram_bytes.json")
    try:
        return float(json.load(open(path))["dram_bytes_per_token_channel"])
    except (OSError, KeyError, ValueError):
        return None


def measured_peak():
    """HBM copy bandwidth measured on this pool (GB/s), or the stated fallback."""
    peaks_path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(peaks_path):
        return float(json.load(open(peaks_path))["hbm_gbs"]), "measured"
    return FALLBACK_HBM_GBS, "fallback"


def run_decode(a):
    """One step = one new token for every sequence: the WKV state update of every layer (T = 1).  The fp32 states
    [layers][B,H,64,64] are read once and written once per step; everything else is a few KB."""
    import torch
    import star_rwkv6_b200 as pkg
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, H, N, L = (16 if a.B == 8 else a.B), (64 if a.H == 32 else a.H), 64, a.layers
    C = H * N
    g = torch.Generator().manual_seed(0)
    mk = lambda s=1.0: (torch.randn(B, 1, C, generator=g) * s).to(torch.bfloat16).to(dev)
    ins = [dict(r=mk(0.125), k=mk(0.125), v=mk(0.125), w=(torch.rand(B, 1, C, generator=g) * 7 - 6).to(torch.bfloat16).to(dev))
           for _ in range(L)]
    u = (torch.randn(H, N, generator=g) * 0.1).to(dev)
    states = [(torch.randn(B, H, N, N, generator=g) * 0.1).to(dev) for _ in range(L)]

    def one_step():
        for d, st in zip(ins, states):
            pkg.ops.wkv6_decode(d["r"], d["k"], d["v"], d["w"], u, N, state=st, out_state=st)

    for _ in range(3):
        one_step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        one_step()
    sampler = ClockSampler(0)
    sampler.start()
    for _ in range(max(3, a.warmup)):
        graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(a.steps):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    state_bytes = 2 * L * B * H * N * N * 4
    peak, peak_src = measured_peak()
    achieved = state_bytes / (ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "wkv6_decode_tokens_per_s", "value": B / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"wkv6 decode step B{B} H{H} N{N} x {L} layers, bf16 activations, fp32 states",
                   "l2": f"states of all layers {state_bytes // 2 / 1e6:.0f} MB, larger than the 126 MB L2",
                   "launch": "one CUDA-graph replay per step"},
        "roofline": {"bound": "hbm", "kernel": "decode_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                     "frac": achieved / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": state_bytes // L, "avg_ms": ms / L},
        "clocks": clocks, "gpu_launches": L * a.steps,
    }), flush=True)


def run_gn_gate(a):
    """One step = forward + backward of the fused GroupNorm * gate stage on [B*T, H*N] bf16 tensors."""
    import torch
    from star_rwkv6_b200 import group_norm as M
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rows, H, N = a.B * a.T, a.H, a.N
    C = H * N
    g = torch.Generator().manual_seed(0)
    sets = []
    for _ in range(2):  # two rotating sets of 3 x 134 MB: larger than L2
        sets.append(dict(y=(torch.randn(rows, C, generator=g) * 0.03).to(torch.bfloat16).to(dev),
                         g=torch.nn.functional.silu(torch.randn(rows, C, generator=g)).to(torch.bfloat16).to(dev),
                         gout=torch.randn(rows, C, generator=g).to(torch.bfloat16).to(dev)))
    scale = (1 + 0.1 * torch.randn(H, N, generator=g)).to(dev)
    offset = (0.1 * torch.randn(H, N, generator=g)).to(dev)

    def step(d):
        out = M.groupnorm_gate_forward_raw(d["y"], d["g"], scale, offset)
        return out, M.groupnorm_gate_backward_raw(d["y"], d["g"], scale, offset, d["gout"])

    sampler = ClockSampler(0)
    sampler.start()
    for i in range(max(3, a.warmup)):
        step(sets[i % 2])
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(a.steps)]
    for i in range(a.steps):
        d = sets[i % 2]
        ev[i][0].record()
        out = M.groupnorm_gate_forward_raw(d["y"], d["g"], scale, offset)
        ev[i][1].record()
        M.groupnorm_gate_backward_raw(d["y"], d["g"], scale, offset, d["gout"])
        ev[i][2].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    ms = ev[0][0].elapsed_time(ev[-1][2]) / a.steps
    elems = rows * C
    fwd_bytes, bwd_bytes = 6 * elems, 10 * elems
    peak, peak_src = measured_peak()
    print(json.dumps({
        "metric": "gn_gate_fwd_bwd_mtokens_per_s", "value": rows / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"per-head GroupNorm * gate, fwd+bwd, rows {rows} H{H} N{N} bf16",
                   "l2": "two rotating input sets of 403 MB each, larger than the 126 MB L2"},
        "roofline": {"bound": "hbm", "kernel": "gn_gate_bwd_kernel", "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": bwd_bytes, "avg_ms": bwd_ms,
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes_per_launch": fwd_bytes, "avg_ms": fwd_ms}},
        "clocks": clocks, "gpu_launches": 3 * a.steps,
    }), flush=True)


def run_shift_mix(a):
    """One step = forward + backward of the five data-dependent token-shift interpolations on [B,T,C] bf16."""
    import torch
    from star_rwkv6_b200 import time_mix_inputs as M
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    B, T, C = a.B, a.T, a.H * a.N
    g = torch.Generator().manual_seed(0)
    sets = []
    for _ in range(2):  # two rotating sets (x 134 MB, m and gout 671 MB each): far larger than L2
        sets.append(dict(x=torch.randn(B, T, C, generator=g).to(torch.bfloat16).to(dev),
                         m=torch.randn(5, B, T, C, generator=g).to(torch.bfloat16).to(dev),
                         gout=torch.randn(5, B, T, C, generator=g).to(torch.bfloat16).to(dev)))
    sampler = ClockSampler(0)
    sampler.start()
    for i in range(max(3, a.warmup)):
        d = sets[i % 2]
        M._shift_mix_fwd(d["x"], d["m"], False); M._shift_mix_bwd(d["x"], d["m"], d["gout"], False)
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(a.steps)]
    for i in range(a.steps):
        d = sets[i % 2]
        ev[i][0].record()
        M._shift_mix_fwd(d["x"], d["m"], False)
        ev[i][1].record()
        M._shift_mix_bwd(d["x"], d["m"], d["gout"], False)
        ev[i][2].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    ms = ev[0][0].elapsed_time(ev[-1][2]) / a.steps
    elems = B * T * C
    fwd_bytes, bwd_bytes = 22 * elems, 34 * elems  # x + 5 m in, 5 out  |  x + 5 m + 5 gout in, gx + 5 gm out
    peak, peak_src = measured_peak()
    print(json.dumps({
        "metric": "shift_mix5_fwd_bwd_mtokens_per_s", "value": B * T / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"five token-shift interpolations, fwd+bwd, B{B} T{T} C{C} bf16",
                   "l2": "two rotating input sets of 1.5 GB each, larger than the 126 MB L2"},
        "roofline": {"bound": "hbm", "kernel": "shift_mix_bwd_kernel", "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": bwd_bytes, "avg_ms": bwd_ms,
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes_per_launch": fwd_bytes, "avg_ms": fwd_ms}},
        "clocks": clocks, "gpu_launches": 2 * a.steps,
    }), flush=True)


def run_channel_mix_act(a):
    """One step = forward + backward of the two channel-mix activations at the training shape: relu_sq on
    [B*T, 7168] (ffn width of the 1.6B shape, scaled with H*N) and sigmoid_mul on [B*T, H*N], bf16."""
    import ctypes
    import torch
    from star_rwkv6_b200._lib import check, lib
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rows, D = a.B * a.T, a.H * a.N
    FF = 7168 * D // 2048
    g = torch.Generator(device=dev).manual_seed(0)
    mk = lambda n, s=1.0: (torch.randn(rows, n, generator=g, device=dev) * s).to(torch.bfloat16)
    sets = [dict(x=mk(FF, 2.0), gk=mk(FF), r=mk(D, 3.0), kv=mk(D), go=mk(D)) for _ in range(2)]   # 1.1 GB per set
    outs = dict(k=torch.empty(rows, FF, dtype=torch.bfloat16, device=dev), gx=torch.empty(rows, FF, dtype=torch.bfloat16, device=dev),
                o=torch.empty(rows, D, dtype=torch.bfloat16, device=dev), gr=torch.empty(rows, D, dtype=torch.bfloat16, device=dev),
                gkv=torch.empty(rows, D, dtype=torch.bfloat16, device=dev))
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    p = lambda t: ctypes.c_void_p(t.data_ptr())

    def fwd(d):
        check(lib.wkv6_relu_sq_forward(rows * FF, 0, p(d["x"]), p(outs["k"]), st))
        check(lib.wkv6_sigmoid_mul_forward(rows * D, 0, p(d["r"]), p(d["kv"]), p(outs["o"]), st))

    def bwd(d):
        check(lib.wkv6_relu_sq_backward(rows * FF, 0, p(d["x"]), p(d["gk"]), p(outs["gx"]), st))
        check(lib.wkv6_sigmoid_mul_backward(rows * D, 0, p(d["r"]), p(d["kv"]), p(d["go"]), p(outs["gr"]), p(outs["gkv"]), st))

    sampler = ClockSampler(0)
    sampler.start()
    for i in range(max(3, a.warmup)):
        fwd(sets[i % 2]); bwd(sets[i % 2])
    torch.cuda.synchronize()
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(a.steps)]
    for i in range(a.steps):
        ev[i][0].record(); fwd(sets[i % 2]); ev[i][1].record(); bwd(sets[i % 2]); ev[i][2].record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    fwd_ms = statistics.mean(e[0].elapsed_time(e[1]) for e in ev)
    bwd_ms = statistics.mean(e[1].elapsed_time(e[2]) for e in ev)
    ms = ev[0][0].elapsed_time(ev[-1][2]) / a.steps
    fwd_bytes = 2 * (2 * rows * FF + 3 * rows * D)
    bwd_bytes = 2 * (3 * rows * FF + 5 * rows * D)
    peak, peak_src = measured_peak()
    print(json.dumps({
        "metric": "channel_mix_act_fwd_bwd_mtokens_per_s", "value": rows / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "n_gpus": 1,
        "steps": a.steps, "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"channel-mix activations fwd+bwd: relu_sq on [{rows}, {FF}], sigmoid_mul on [{rows}, {D}], bf16",
                   "l2": "two rotating input sets of 1.1 GB each, larger than the 126 MB L2"},
        "roofline": {"bound": "hbm", "kernel": "channel_mix_elementwise_kernel (backward pair)", "achieved": bwd_bytes / (bwd_ms * 1e-3) / 1e9,
                     "peak": peak, "unit": "GB/s", "frac": bwd_bytes / (bwd_ms * 1e-3) / 1e9 / peak, "traffic": None,
                     "peak_source": peak_src, "algorithmic_bytes_per_launch": bwd_bytes, "avg_ms": bwd_ms,
                     "forward": {"achieved": fwd_bytes / (fwd_ms * 1e-3) / 1e9, "frac": fwd_bytes / (fwd_ms * 1e-3) / 1e9 / peak,
                                 "algorithmic_bytes_per_launch": fwd_bytes, "avg_ms": fwd_ms}},
        "clocks": clocks, "gpu_launches": 4 * a.steps,
    }), flush=True)


def run_lm_loss(a):
    """One step = the fused language-model loss (softmax cross-entropy + logit gradient, one kernel) over 8192 x 65536
    bf16 logits; two rotating buffers of 1.07 GB each, larger than the 126 MB L2."""
    import ctypes
    import torch
    from star_rwkv6_b200._lib import check, lib
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    rows, V = 8192, 65536
    g = torch.Generator(device=dev).manual_seed(0)
    bufs = [(torch.randn(rows, V, generator=g, device=dev) * 3).to(torch.bfloat16) for _ in range(2)]
    fresh = [b.clone() for b in bufs]
    targets = torch.randint(0, V, (rows,), generator=g, device=dev)
    loss = torch.empty(rows, dtype=torch.float32, device=dev)
    st = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)

    def step(i):
        check(lib.wkv6_softmax_xent_bf16(rows, V, bufs[i % 2].data_ptr(), targets.data_ptr(), 1.0 / rows, loss.data_ptr(), st))

    sampler = ClockSampler(0)
    sampler.start()
    for i in range(max(3, a.warmup)):
        step(i)
    for b, f in zip(bufs, fresh):
        b.copy_(f)          # real logits again (a step leaves gradients in its buffer)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        step(i)
    e1.record()
    torch.cuda.synchronize()
    clocks = sampler.stop()
    ms = e0.elapsed_time(e1) / a.steps
    peak, peak_src = measured_peak()
    nbytes = 2 * rows * V * 2
    print(json.dumps({
        "metric": "lm_loss_mtokens_per_s", "value": rows / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "n_gpus": 1, "steps": a.steps,
        "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"softmax cross-entropy + logit gradient, {rows} x {V} bf16 logits",
                   "l2": "two rotating buffers of 1.07 GB each, larger than the 126 MB L2"},
        "roofline": {"bound": "hbm", "kernel": "softmax_xent_kernel", "achieved": nbytes / (ms * 1e-3) / 1e9, "peak": peak,
                     "unit": "GB/s", "frac": nbytes / (ms * 1e-3) / 1e9 / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": nbytes, "avg_ms": ms},
        "clocks": clocks, "gpu_launches": a.steps,
    }), flush=True)


def run_train_step(a):
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    from star_rwkv6_b200.loss import lm_loss
    from star_rwkv6_b200.model import RWKV6
    L = 24 if a.layers == 32 else a.layers
    D, V, FF, B, T = a.H * a.N, 65536, 7168 * (a.H * a.N) // 2048, a.B, a.T
    torch.manual_seed(0)
    model = RWKV6(L, V, D, head_size=a.N, decomposer_size=32, expand_size=FF, decay_rank=64).to(dev).to_bf16_()
    nparams = sum(p.numel() for p in model.parameters())
    net = model
    if world > 1:
        net = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local], gradient_as_bucket_view=True)
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4, fused=True)
    g = torch.Generator().manual_seed(1 + rank)
    host = [torch.randint(0, V, (B, T + 1), generator=g).pin_memory() for _ in range(2)]
    ckpt = not a.no_checkpoint

    def step(i):
        tok = host[i % 2].to(dev, non_blocking=True)              # the step's input comes from pinned host memory
        logits = net(tok[:, :-1], checkpoint_blocks=ckpt)
        if a.framework_loss:
            loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, V), tok[:, 1:].reshape(-1))
        else:   # loss and logit gradient in one pass over the bf16 logits (same fp32 softmax arithmetic)
            loss = lm_loss(logits, tok[:, 1:])
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()
    for i in range(max(3, a.warmup)):
        step(i)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(a.steps):
        loss = step(i)
    last = float(loss.detach().cpu())                              # device-to-host read of the step's result
    e1.record()
    barrier()
    clocks = sampler.stop() if sampler else None
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    if rank == 0:
        ms = total_ms / a.steps
        tokens = B * T * world
        flops = 6.0 * nparams * B * T                                # model FLOPs per GPU and step (recomputation not counted)
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json"))) if os.path.exists(os.path.join(ROOT, "MEASURED_PEAKS.json")) else {}
        peak = float(peaks.get("bf16_tflops_sustained", 1400.0))
        ach = flops / (ms * 1e-3) / 1e12
        val = tokens / (ms * 1e-3)
        print(json.dumps({
            "metric": "rwkv6_train_tokens_per_s", "value": val, "unit": "tokens/s", "n_gpus": world, "steps": a.steps,
            "warmup": max(3, a.warmup), "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"RWKV-6 training step: {L} layers, d_model {D}, ffn {FF}, vocab {V}, B{B} T{T} per GPU, AdamW",
                       "parameters": nparams, "block_recomputation": ckpt, "last_loss": last,
                       "loss": "framework cross_entropy on fp32 logits" if a.framework_loss else "fused softmax cross-entropy + logit gradient on bf16 logits",
                       "parallelism": f"dp{world}" + (" (DDP, NCCL bucketed all-reduce overlapped with the backward)" if world > 1 else "")},
            "roofline": {"bound": "tensor", "kernel": "whole step (library GEMMs dominate)", "achieved": ach, "peak": peak,
                         "unit": "TFLOP/s", "frac": ach / peak, "traffic": None,
                         "peak_source": "measured (sustained)" if peaks else "fallback"},
            "e2e": {"value": val, "unit": "tokens/s", "h2d_bytes_per_step": B * (T + 1) * 8, "d2h_bytes_per_step": 4,
                    "note": "the timed steps already start from pinned host token ids; the loss is read back once at the end"},
            "clocks": clocks, "gpu_launches": None,
        }), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_inference(a):
    """The 7B-shape inference workload: (32 layers, d_model 4096, 64 heads of 64, ffn 14336, vocab
    65536, bf16, random init), prefill of B16 x T4096 random token ids, then greedy decode steps replayed from one CUDA
    graph, each carrying the per-layer [B,H,64,64] fp32 WKV states (updated in place by the decode kernel).
    With N GPUs the batch is sharded (B/N sequences per rank, weights replicated, no collective on the data path)."""
    import torch
    import torch.distributed as dist
    from star_rwkv6_b200.model import RWKV6
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    L = a.layers
    B_global = 16 if a.B == 8 else a.B
    assert B_global % world == 0, "the batch must divide over the ranks"
    B = B_global // world
    H = 64 if a.H == 32 else a.H
    D, V, T = H * a.N, 65536, a.T
    FF = 14336 * D // 4096
    torch.manual_seed(0)
    with torch.device(dev):
        model = RWKV6(L, V, D, head_size=a.N, decomposer_size=32, expand_size=FF, decay_rank=64)
    model = model.to_bf16_().eval()
    nparams = sum(p.numel() for p in model.parameters())
    g = torch.Generator().manual_seed(1)
    prompt = torch.randint(0, V, (B_global, T), generator=g)[rank * B:(rank + 1) * B].contiguous().pin_memory()
    sampler = ClockSampler(local) if rank == 0 else None
    if sampler:
        sampler.start()

    def max_over_ranks(ms):
        if world == 1:
            return ms
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    pre_ms = []
    for _ in range(3):  # the first pass also warms cuBLAS up; the best of the later two is reported
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        logits, states = model.prefill(prompt.to(dev, non_blocking=True))
        e1.record()
        torch.cuda.synchronize()
        pre_ms.append(e0.elapsed_time(e1))
    prefill_ms = max_over_ranks(min(pre_ms[1:]))
    tok0 = logits.argmax(-1)                                         # [B,1] first generated token

    def timed_decode(fused):
        """Greedy decode from the prefill state: one CUDA-graph replay per token step."""
        tok = tok0.clone()
        st = [((xa.clone(), S.clone()), xf.clone()) for (xa, S), xf in states]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):                                 # warm the decode path outside the capture
            for _ in range(2):
                tok.copy_(model.decode(tok, st, fused=fused).argmax(-1))
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            tok.copy_(model.decode(tok, st, fused=fused).argmax(-1))
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.decode_steps):
            graph.replay()
        e1.record()
        torch.cuda.synchronize()
        return max_over_ranks(e0.elapsed_time(e1) / a.decode_steps), tok

    plain_ms, _ = timed_decode(False)
    dec_ms, tok = timed_decode(True)
    last = tok.cpu()                                                  # the generated token ids come back to the host
    clocks = sampler.stop() if sampler else None
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak, peak_src = measured_peak()
    weight_bytes = 2 * (nparams - V * D)                             # every weight but the embedding table is read per step
    state_bytes = 2 * L * B * H * a.N * a.N * 4
    ach = (weight_bytes + state_bytes) / (dec_ms * 1e-3) / 1e9
    print(json.dumps({
        "metric": "rwkv6_decode_tokens_per_s", "value": B_global / (dec_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
        "steps": a.decode_steps, "warmup": 3, "ms_per_step": dec_ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"RWKV-6 inference: {L} layers, d_model {D}, ffn {FF}, vocab {V}, B{B_global}, prefill T{T} then greedy decode",
                   "parallelism": f"batch sharded over {world} GPU(s), {B} sequences each, weights replicated, no collective",
                   "parameters": nparams, "decode": "one CUDA-graph replay per token step, WKV states fp32 in HBM, updated in place; element-wise "
                             "stages of every block fused, r/k/v/g as one batched product (15 launches per block)",
                   "decode_ms_with_framework_elementwise_ops": plain_ms,
                   "prefill_ms": prefill_ms, "prefill_tokens_per_s": B_global * T / (prefill_ms * 1e-3),
                   "prefill_model_tflops_per_gpu": 2.0 * nparams * B * T / (prefill_ms * 1e-3) / 1e12},
        "roofline": {"bound": "hbm", "kernel": "decode step on one GPU (weights + its WKV states streamed once)", "achieved": ach, "peak": peak,
                     "unit": "GB/s", "frac": ach / peak, "traffic": None, "peak_source": peak_src,
                     "algorithmic_bytes_per_launch": weight_bytes + state_bytes, "avg_ms": dec_ms},
        "e2e": {"value": B_global / (dec_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": B_global * 8,
                "note": "token ids stay on the device between steps and are read back once at the end"},
        "clocks": clocks, "gpu_launches": None, "last_tokens": last.flatten().tolist()[:4],
    }), flush=True)


def main():
    a = parse()
    if a.impl == "reference":
        run_reference(a)
    elif a.workload == "decode":
        run_decode(a)
    elif a.workload == "gn_gate":
        run_gn_gate(a)
    elif a.workload == "shift_mix":
        run_shift_mix(a)
    elif a.workload == "channel_mix_act":
        run_channel_mix_act(a)
    elif a.workload == "lm_loss":
        run_lm_loss(a)
    elif a.workload == "train_step":
        run_train_step(a)
    elif a.workload == "inference":
        run_inference(a)
    else:
        run_b200(a)


if __name__ == "__main__":
    main()
