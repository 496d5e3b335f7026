#!/usr/bin/env python
"""WKV forward+backward throughput on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the op over the v6 7B-shape workload: bf16 r,k,v,w,gy of
shape [B=4, T=16384, C=4096] (H=64 heads of 64), processed as 4 BPTT segments of
4096 tokens -- forward over all segments with the fp32 state carried, then
backward over them in reverse with the state gradient carried.  Synthetic
inputs: r,k,v,gy ~ N(0,1), x ~ N(-0.6,0.5) (decay exp(-exp(x))), u ~ U(-1,1).

With N GPUs the workload's 64 heads are split over the ranks (64/N heads of all 4
batch rows each): strong scaling, value = tokens / max-over-ranks time.  No
collective runs on the data path (NCCL only carries the barrier and the
max-over-ranks time).  ``--scaling weak`` makes every rank run the whole workload
instead.  Prints ONE JSON line (rank 0).

``--impl reference`` times the reference's own CPU implementation of the path on
the host cores, on a bounded sample of the same workload: the project's
``rwkv_inner`` itself where its checkout is present, else the restatement of it in
oracle/wkv_chunked_port.py.

Side modes (one GPU, a JSON line each, not the headline): ``--config 1|2`` the v4
fp32 and v5 bf16 workloads, ``--config 4`` one GPU's 5-head slice of the
1M-token stream, ``--ref-kernels`` the project's own CUDA kernels (compiled
unchanged for sm_100a into oracle/_ref/) on the shapes they are valid for.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402

WORKLOAD = dict(name="rwkv6_7b_wkv_fwd_bwd", variant="v6", B=4, T=16384, seg=4096, C=4096, H=64,
                N=64)
METRIC = "wkv_fwd_bwd_tokens_per_s"
# bytes each tensor element is touched, once: fwd r,k,v,w -> y ; bwd r,k,v,w,gy -> gr,gk,gv,gw
FWD_ELEMS, BWD_ELEMS = 5, 9
# DRAM bytes per head-token of the backward launch group, from the ncu captures of the B=1,
# T=4096, H=64 case: (102.3 + 15.1 MB dS scan) + (236.0 + 101.9 MB per-chunk kernel) over
# 64 * 4096 head-tokens.  Traffic grows in proportion to head-tokens.
NCU_BWD_DRAM_BYTES_PER_HEAD_TOKEN = (102.27e6 + 15.10e6 + 236.01e6 + 101.88e6) / (64 * 4096)


def peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


_NVML_CHILD = r"""
import sys, time
import pynvml as N
N.nvmlInit()
h = N.nvmlDeviceGetHandleByIndex(int(sys.argv[1]))
mx = N.nvmlDeviceGetMaxClockInfo(h, N.NVML_CLOCK_SM)
bits = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
print("ready", flush=True)
while True:
    sm = N.nvmlDeviceGetClockInfo(h, N.NVML_CLOCK_SM)
    try:
        r = N.nvmlDeviceGetCurrentClocksEventReasons(h)
    except Exception:
        r = N.nvmlDeviceGetCurrentClocksThrottleReasons(h)
    print("%.6f,%d,%d,%s" % (time.time(), sm, mx, "|".join(k for k, b in bits.items() if r & b)), flush=True)
    time.sleep(0.003)
"""


class NvmlSampler:
    """Reads (never sets) the SM clock and the clock-event reasons through NVML every ~3 ms from a
    child process, so that even a timed region of tens of milliseconds gets its own samples; only
    the samples whose time stamp falls inside [mark_start, mark_end] are reported."""

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []
        self.t0 = self.t1 = None

    def start(self):
        try:
            phys = os.environ.get("CUDA_VISIBLE_DEVICES", "")
            idx = int(phys.split(",")[self.index]) if phys and phys.split(",")[self.index].isdigit() else self.index
            self.proc = subprocess.Popen([sys.executable, "-c", _NVML_CHILD, str(idx)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            if self.proc.stdout.readline().strip() != "ready":
                raise RuntimeError("nvml child not ready")
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            if self.proc is not None:
                self.proc.kill()
            self.proc = None
        return self.proc is not None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def mark_start(self):
        self.t0 = time.time()

    def mark_end(self):
        self.t1 = time.time()

    def stop(self) -> dict:
        time.sleep(0.01)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for line in list(self.lines):
            f = line.strip().split(",")
            if len(f) < 4:
                continue
            ts = float(f[0])
            if self.t0 is not None and not (self.t0 <= ts <= (self.t1 or ts)):
                continue
            sm.append(float(f[1])); mx.append(float(f[2]))
            reasons.update(x for x in f[3].split("|") if x)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no_samples"], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm), "source": "nvml, ~3 ms period, samples inside the timed region only"}


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs
    (the fallback when NVML cannot be read from Python)."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-i", str(self.index), "-lms", "100"], stdout=subprocess.PIPE,
                stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line)

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 6:
                continue
            try:
                sm.append(float(f[0])); mx.append(float(f[1]))
            except ValueError:
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no_samples"]}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                "samples": len(sm)}


def make_inputs(wl, device, pinned_host=False):
    """Seeded synthetic inputs of the workload's shapes and distributions (bf16)."""
    B, T, C, H, N = wl["B"], wl["T"], wl["C"], wl["H"], wl["N"]
    g = torch.Generator(device="cpu").manual_seed(0)
    host = {}
    for name in ("r", "k", "v", "gy"):
        host[name] = torch.randn((B, T, C), generator=g, dtype=torch.float32).to(torch.bfloat16)
    host["w"] = (torch.randn((B, T, C), generator=g) * 0.5 - 0.6).to(torch.bfloat16)
    host["u"] = (torch.rand((H, N), generator=g) * 2 - 1).to(torch.bfloat16)
    if pinned_host:
        host = {n: t.pin_memory() for n, t in host.items()}
    dev = {n: t.to(device, non_blocking=True) for n, t in host.items()}
    return host, dev


class Runner:
    """Device-resident step.  Every call of the step is prepared once (outputs, workspaces and
    the forward-to-backward hand-over allocated up front), so a step is 2 x segments crossings of
    the C ABI and nothing else on the host; events around every forward and backward call."""

    def __init__(self, wl, seg_tensors, u, device):
        import ctypes
        import rwkv_infctx_trainer_b200 as W
        from rwkv_infctx_trainer_b200 import wkv56
        self.W, self.wkv56, self.wl, self.device = W, wkv56, wl, device
        B, H, N = wl["B"], wl["H"], wl["N"]
        n = len(seg_tensors["r"])
        states = [torch.zeros((B, H, N, N), device=device) for _ in range(n + 1)]
        gstates = [torch.empty((B, H, N, N), device=device) for _ in range(n + 1)]
        self.fwd, self.bwd = [], []
        for i in range(n):
            t = {m: seg_tensors[m][i] for m in ("r", "k", "v", "w", "gy")}
            f = wkv56.prepare_forward("wkv6", t["r"], t["k"], t["v"], t["w"], u, states[i], w_kind=W.WKV_W_RAW,
                                      state_out=states[i + 1])
            b = wkv56.prepare_backward("wkv6", t["r"], t["k"], t["v"], t["w"], u, states[i], t["gy"],
                                       None if i == n - 1 else gstates[i + 1], w_kind=W.WKV_W_RAW,
                                       ckpt=f.ckpt, gstate_in=gstates[i])
            self.fwd.append(f); self.bwd.append(b)
        self.bwd_events, self.fwd_events = [], []
        self.launches = 0
        # kernels per call: k_chunk_fwd ; k_chunk_dscan, k_chunk_bwd, k_chunk_bwd_steep, k_reduce_partials
        # -- and, when the library cuts the chains into time groups (few chains per GPU), a summary pass
        # and a group scan more for the forward and for the dS scan
        a = wkv56._args("wkv6", B, wl["seg"], H, torch.bfloat16, W.WKV_W_RAW, W.WKV_STATE_KV, W.WKV_PATH_AUTO)
        split = W._lib.load().wkv6_forward_workspace(ctypes.byref(a)) > 256
        self.fwd_launches, self.bwd_launches = (3, 6) if split else (1, 4)

    def step(self, record=False):
        for f in self.fwd:
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            f.run()
            if record:
                e1.record()
                self.fwd_events.append((e0, e1))
            self.launches += self.fwd_launches
        for b in reversed(self.bwd):
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            b.run()
            if record:
                e1.record()
                self.bwd_events.append((e0, e1))
            self.launches += self.bwd_launches

    def status(self) -> int:
        """OR of the status words of every call (0 = no device-side wait ran out)"""
        code = 0
        for c in self.fwd + self.bwd:
            code |= c.status()
        return code


def contiguous_segments(t, bounds):
    return [t[:, a:b].contiguous() for a, b in bounds]


def run_ours(args):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU path for the product arm)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    wl = dict(WORKLOAD)
    if args.small:
        wl.update(name=wl["name"] + "_small", B=1, T=4096)
    if args.medium:
        wl.update(name=wl["name"] + "_medium", T=4096)
    if args.heads:
        wl.update(name=wl["name"] + f"_{args.heads}heads", H=args.heads, C=args.heads * wl["N"])
    H_total = wl["H"]
    if args.scaling is None:
        args.scaling = "strong"
    if args.scaling == "strong" and world > 1:
        from rwkv_infctx_trainer_b200.sharding import shard_units
        sh = shard_units(wl["B"], wl["H"], world, rank)
        if sh.b1 - sh.b0 != wl["B"] or wl["H"] % world:
            raise SystemExit("--scaling strong needs the head count to be divisible by the GPU count")
        wl.update(H=sh.h1 - sh.h0, C=(sh.h1 - sh.h0) * wl["N"])   # this rank's heads (same distributions)
    B, T, C, H = wl["B"], wl["T"], wl["C"], wl["H"]
    host, dev = make_inputs(wl, device, pinned_host=True)
    # the op takes contiguous [B,T_seg,C] tensors: lay the segments out once, outside the timing
    bounds = [(t0, min(T, t0 + wl["seg"])) for t0 in range(0, T, wl["seg"])]
    segd = {n: contiguous_segments(dev[n], bounds) for n in ("r", "k", "v", "w", "gy")}

    runner = Runner(wl, segd, dev["u"], device)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        runner.step()
    barrier()
    runner.launches = 0
    sampler = None
    if rank == 0:
        sampler = NvmlSampler(local)
        if not sampler.start():
            sampler = ClockSampler(local)
            sampler.start()
        barrier_free_sleep = 0.05      # let the first samples arrive before the clock starts
        time.sleep(barrier_free_sleep)
    barrier()
    if rank == 0 and isinstance(sampler, NvmlSampler):
        sampler.mark_start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for i in range(args.steps):
        runner.step(record=i < 32)      # per-launch events on the first steps only
    t_end.record()
    barrier()
    if rank == 0 and isinstance(sampler, NvmlSampler):
        sampler.mark_end()
    clocks = sampler.stop() if rank == 0 else None
    ms = t_start.elapsed_time(t_end)
    if runner.status() != 0:
        raise SystemExit("a device-side wait ran out during the timed region: the results are invalid")
    launches = runner.launches
    bwd_ms = [a.elapsed_time(b) for a, b in runner.bwd_events]
    fwd_ms = [a.elapsed_time(b) for a, b in runner.fwd_events]

    # ---- end to end through the public autograd op, host buffers in pinned memory
    import rwkv_infctx_trainer_b200 as W
    hseg = {n: [s.contiguous().pin_memory() for s in contiguous_segments(host[n], bounds)]
            for n in ("r", "k", "v", "w", "gy")}
    out_host = {n: [torch.empty_like(s).pin_memory() for s in hseg["r"]]
                for n in ("y", "gr", "gk", "gv", "gw")}
    u_dev = dev["u"]

    # Software pipeline over steps: while step s computes, the inputs of step s+1 are copied
    # in on one side stream and the results of step s-1 are copied out on another (PCIe is
    # full duplex).  Every step's host->device and device->host copies are inside the timed
    # region; the ops are called through the public autograd Function.
    in_s, out_s = torch.cuda.Stream(device), torch.cuda.Stream(device)
    names_in, names_g = ("r", "k", "v", "w", "gy"), ("gr", "gk", "gv", "gw")

    def prefetch():
        cur = torch.cuda.current_stream(device)
        bufs, evs = [], []
        with torch.cuda.stream(in_s):
            for i in range(len(bounds)):
                seg = {n: hseg[n][i].to(device, non_blocking=True) for n in names_in}
                for t in seg.values():
                    t.record_stream(cur)
                ev = torch.cuda.Event()
                ev.record(in_s)
                bufs.append(seg)
                evs.append(ev)
        return bufs, evs

    def compute_and_drain(bufs, evs):
        cur = torch.cuda.current_stream(device)
        leaves, ys = [], []
        state = torch.zeros((B, H, 64, 64), device=device)
        for i, (t0, t1) in enumerate(bounds):
            cur.wait_event(evs[i])
            r, k, v, w = (bufs[i][n].requires_grad_(True) for n in ("r", "k", "v", "w"))
            y, state = W.WKV6.apply(B, t1 - t0, C, H, r, k, v, w, u_dev, state)
            leaves.append((r, k, v, w)); ys.append(y)
            ev = torch.cuda.Event(); ev.record(cur)
            with torch.cuda.stream(out_s):
                out_s.wait_event(ev)
                out_host["y"][i].copy_(y.detach(), non_blocking=True)
                y.record_stream(out_s)
        torch.autograd.backward(ys, [bufs[i]["gy"] for i in range(len(bounds))])
        ev = torch.cuda.Event(); ev.record(cur)
        with torch.cuda.stream(out_s):
            out_s.wait_event(ev)
            for i, tensors in enumerate(leaves):
                for n, t in zip(names_g, tensors):
                    out_host[n][i].copy_(t.grad, non_blocking=True)
                    t.grad.record_stream(out_s)

    def e2e_run(nsteps):
        nxt = prefetch()
        for sidx in range(nsteps):
            cur_in = nxt
            if sidx + 1 < nsteps:
                nxt = prefetch()
            compute_and_drain(*cur_in)
        out_s.synchronize()
        torch.cuda.current_stream(device).synchronize()

    h2d = sum(s.numel() * s.element_size() for n in hseg for s in hseg[n])
    d2h = sum(s.numel() * s.element_size() for n in out_host for s in out_host[n])
    # (enough steps that the un-overlapped first copy in and last copy out are a small part of the region)
    e2e_steps = max(1, min(args.steps, 24))
    if args.skip_e2e:
        e2e_s = float("nan")
    else:
        e2e_run(1)
        barrier()
        t0 = time.perf_counter()
        e2e_run(e2e_steps)
        barrier()
        e2e_s = time.perf_counter() - t0

    times = torch.tensor([ms, e2e_s * 1e3], device=device, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(times[0]), float(times[1])
    tokens = B * T
    job = world if args.scaling == "weak" else 1       # strong: the ranks share one workload
    value = job * tokens * args.steps / (ms * 1e-3)
    e2e_value = job * tokens * e2e_steps / (e2e_ms * 1e-3)

    if rank == 0:
        hbm, which = peaks()
        seg_tokens = wl["seg"]
        bwd_bytes = BWD_ELEMS * 2 * B * seg_tokens * C + 3 * B * H * 64 * 64 * 4
        avg_bwd_ms = sum(bwd_ms) / len(bwd_ms)
        achieved = bwd_bytes / (avg_bwd_ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": wl["name"], "variant": "v6", "B_per_gpu": B, "T": T,
                       "bptt_segment": wl["seg"], "C_per_gpu": C, "H_per_gpu": H, "H": H_total,
                       "head_size": 64,
                       "state": "fp32 carried across segments, gradient carried back",
                       "sharding": (f"{world} x (batch x head) replicas of the workload" if args.scaling == "weak"
                                    else f"heads split {H} per GPU over {world} GPUs") + ", no collective on the data path",
                       "l2": f"inputs ({5 * 2 * B * T * C / 1e9:.2f} GB per GPU) larger than L2, no flush"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "how": "WKV6.apply + autograd; pinned host buffers; copies of step s+1 (in) and "
                           "s-1 (out) overlap the compute of step s on side streams"},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm",
                         "kernel": "wkv6 backward of one BPTT segment: k_chunk_dscan + k_chunk_bwd "
                                   "(+ k_chunk_bwd_steep, k_reduce_partials), timed as one launch group",
                         "achieved": achieved, "peak": hbm, "unit": "GB/s",
                         "frac": achieved / hbm, "peak_source": which + " HBM copy bandwidth",
                         "algorithmic_bytes_per_launch": bwd_bytes,
                         "avg_launch_ms": avg_bwd_ms,
                         "traffic": NCU_BWD_DRAM_BYTES_PER_HEAD_TOKEN * B * seg_tokens * H,
                         "traffic_source": "ncu dram__bytes_read+write of both kernels on the "
                                           "B=1 small case, scaled by head-tokens"},
            "forward_launch": {"avg_launch_ms": sum(fwd_ms) / len(fwd_ms),
                               "achieved_gbs": (FWD_ELEMS * 2 * B * seg_tokens * C
                                                + 2 * B * H * 64 * 64 * 4)
                               / (sum(fwd_ms) / len(fwd_ms) * 1e-3) / 1e9},
            "whole_step_roofline_frac": (
                (FWD_ELEMS + BWD_ELEMS) * 2 * B * T * C / (ms / args.steps * 1e-3) / 1e9 / hbm),
        }
        if world == 1 and not args.skip_cpu:
            line["cpu_baseline"] = cpu_baseline(steps=8, warmup=1)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def cpu_sample():
    """Bounded sample of the workload for the CPU arm: one batch row, 8 of the 64 heads, the full
    16384 tokens as 4 BPTT segments of 4096 with state carried, forward + backward."""
    wl = dict(WORKLOAD)
    Bs, Hs, T, N = 1, 8, wl["T"], wl["N"]
    g = torch.Generator().manual_seed(0)
    C = Hs * N
    t = {n: torch.randn((Bs, T, C), generator=g) for n in ("r", "k", "v", "gy")}
    t["x"] = torch.randn((Bs, T, C), generator=g) * 0.5 - 0.6
    t["u"] = torch.rand((Hs, N), generator=g) * 2 - 1
    t["s"] = torch.zeros((Bs, Hs, N, N))
    desc = (f"B=1, {Hs} of {wl['H']} heads, T={T} as {T // wl['seg']} segments of {wl['seg']}, "
            "fp32 I/O, fwd+bwd with state carried")
    return t, Bs * T * Hs, desc


def reference_rwkv_inner():
    """The project's own rwkv_inner (RWKV-v6/src/module/rwkv_inner.py), imported from its checkout
    with the trainer-only packages stubbed (tests/golden/make_golden.py does the same to make the
    fixtures), or None where the checkout is not present."""
    root = os.environ.get("WKV_REFERENCE_ROOT", "/root/reference")
    if not os.path.isdir(os.path.join(root, "RWKV-v6", "src", "module")):
        return None
    try:
        sys.path.insert(0, os.path.join(ROOT, "tests", "golden"))
        import make_golden
        return make_golden.load_rwkv_inner("RWKV-v6")
    except Exception:
        return None


def cpu_baseline(steps: int, warmup: int) -> dict:
    from oracle import wkv_chunked_port as P
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t, head_tokens, desc = cpu_sample()
    inner = reference_rwkv_inner()
    if inner is None:
        kind = "port"
        run = lambda: P.run_chain("v6", t["r"], t["k"], t["v"], t["x"], t["u"], t["s"], t["gy"],
                                  WORKLOAD["seg"])
    else:
        kind = "reference"
        Hs, N = t["u"].shape

        def run():
            # the trainer's calling pattern (RWKV-v6/src/module/TimeMix.py:283-295): segments with the
            # state carried, one backward over the chain
            leaves = [t[n].clone().requires_grad_(True) for n in ("r", "k", "v", "x", "u", "s")]
            r, k, v, x, u, state = leaves
            w = torch.exp(-torch.exp(x))
            B, T, C = r.shape
            ys = []
            for t0 in range(0, T, WORKLOAD["seg"]):
                t1 = min(T, t0 + WORKLOAD["seg"])
                sl = lambda a: a[:, t0:t1].reshape(B, t1 - t0, Hs, N).transpose(1, 2)
                o, state = inner(sl(r), sl(k), sl(v), sl(w), u.view(1, Hs, 1, N), state, 128, 64)
                ys.append(o.transpose(1, 2).reshape(B, t1 - t0, C))
            torch.autograd.grad((torch.cat(ys, 1) * t["gy"]).sum(), leaves)
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    # tokens/s of the full-width op (all H heads) at this head-token rate
    return {"value": head_tokens / dt / WORKLOAD["H"], "unit": "tokens/s", "cores": cores,
            "kind": kind, "sample": desc, "head_tokens_per_s": head_tokens / dt,
            "s_per_sample": dt}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    world = int(os.environ.get("WORLD_SIZE", "1"))
    b = cpu_baseline(steps=args.steps, warmup=args.warmup)
    wl = WORKLOAD
    line = {
        "impl": "reference", "metric": METRIC, "value": b["value"], "unit": "tokens/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": b["s_per_sample"] * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl["name"], "variant": "v6", "B_per_gpu": wl["B"], "T": wl["T"],
                   "bptt_segment": wl["seg"], "C": wl["C"], "H": wl["H"], "head_size": 64,
                   "note": "reference's pure-PyTorch chunked WKV (RWKV_NO_CUDA=1 path) on host "
                           "cores; each step is the bounded sample named in cpu_baseline"},
        "cpu_baseline": b,
        "e2e": {"value": b["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0,
                "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def run_side_config(args):
    """Configs 1 (v4, fp32 I/O) and 2 (v5, bf16) of the benchmark list: forward over the BPTT
    segments with state carried, backward in reverse with the state gradient carried.  Not the
    headline line -- prints a JSON line of its own with ``"config_index"``."""
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56, _lib as L
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(0)
    hbm, which = peaks()
    small = 2 if args.small else 8          # --small: two batch rows (profiling aid)
    if args.config == 1:
        B, T, seg, C = small, 4096, 2048, 2048
        dt = {"fp32": torch.float32, "bf16": torch.bfloat16}[args.dtype]
        k, v, gy = (torch.randn((B, T, C), generator=g).to(dt).to(device) for _ in range(3))
        w = (-torch.exp(torch.rand(C, generator=g) * 6 - 5)).to(device)
        u = (torch.rand(C, generator=g) * 2 - 1).to(dt).to(device)
        segs = [(a, a + seg) for a in range(0, T, seg)]
        kk = [k[:, a:b].contiguous() for a, b in segs]
        vv = [v[:, a:b].contiguous() for a, b in segs]
        gg = [gy[:, a:b].contiguous() for a, b in segs]
        lib, code = L.load(), L.DTYPE_CODE[dt]
        st = torch.cuda.current_stream().cuda_stream
        nws = lib.wkv4_backward_workspace(B, seg, C)
        ws = torch.empty(nws, dtype=torch.uint8, device=device)
        nwf = lib.wkv4_forward_workspace(B, seg, C)
        wsf = torch.empty(max(nwf, 16), dtype=torch.uint8, device=device)
        ys = [torch.empty_like(x) for x in kk]
        gk = [torch.empty_like(x) for x in kk]
        gv = [torch.empty_like(x) for x in kk]
        gw = torch.empty((B, C), device=device); gu = torch.empty((B, C), device=device)
        states = [torch.zeros((B, C, 3), device=device) for _ in range(len(segs) + 1)]
        states[0][..., 2] = -1e38
        gst = [torch.empty((B, C, 3), device=device) for _ in range(len(segs) + 1)]
        nck = lib.wkv4_state_ckpt_bytes(B, seg, C)      # piece-start states handed from forward to backward
        cks = [torch.empty(max(nck, 16), dtype=torch.uint8, device=device) for _ in segs]

        def step():
            for i in range(len(segs)):
                L.check(lib.wkv4_forward_ckpt(B, seg, C, code, w.data_ptr(), u.data_ptr(), kk[i].data_ptr(),
                                              vv[i].data_ptr(), states[i].data_ptr(), ys[i].data_ptr(),
                                              states[i + 1].data_ptr(), wsf.data_ptr(), nwf, cks[i].data_ptr(), nck,
                                              st), "wkv4_forward")
            for i in reversed(range(len(segs))):
                gin = None if i == len(segs) - 1 else gst[i + 1].data_ptr()
                L.check(lib.wkv4_backward_ckpt(B, seg, C, code, w.data_ptr(), u.data_ptr(), kk[i].data_ptr(),
                                               vv[i].data_ptr(), states[i].data_ptr(), gg[i].data_ptr(), gin,
                                               gw.data_ptr(), gu.data_ptr(), gk[i].data_ptr(), gv[i].data_ptr(),
                                               gst[i].data_ptr(), ws.data_ptr(), nws, cks[i].data_ptr(), nck, st),
                        "wkv4_backward")
        bytes_step = 8 * k.element_size() * B * T * C
        name = "rwkv4_wkv_fwd_bwd_" + args.dtype
    else:
        B, T, seg, C, H = small, 4096, 2048, 2048, 32
        dt = torch.bfloat16
        r, k, v, gy = (torch.randn((B, T, C), generator=g).to(dt).to(device) for _ in range(4))
        w = (torch.rand((H, 64), generator=g) * 5 - 6).to(device)
        u = (torch.rand((H, 64), generator=g) * 2 - 1).to(dt).to(device)
        segs = [(a, a + seg) for a in range(0, T, seg)]
        cs = lambda t: [t[:, a:b].contiguous() for a, b in segs]
        rr, kk, vv, gg = cs(r), cs(k), cs(v), cs(gy)
        # every call prepared once (buffers allocated up front): a step is 4 crossings of the C ABI
        n = len(segs)
        states = [torch.zeros((B, H, 64, 64), device=device) for _ in range(n + 1)]
        gstates = [torch.empty((B, H, 64, 64), device=device) for _ in range(n)]
        fwd, bwd = [], []
        for i in range(n):
            f = wkv56.prepare_forward("wkv5", rr[i], kk[i], vv[i], w, u, states[i], w_kind=W.WKV_W_RAW,
                                      state_out=states[i + 1])
            bk = wkv56.prepare_backward("wkv5", rr[i], kk[i], vv[i], w, u, states[i], gg[i],
                                        None if i == n - 1 else gstates[i + 1], w_kind=W.WKV_W_RAW,
                                        ckpt=f.ckpt, gstate_in=gstates[i])
            fwd.append(f); bwd.append(bk)

        def step():
            for f in fwd:
                f.run()
            for bk in reversed(bwd):
                bk.run()
        bytes_step = 11 * 2 * B * T * C
        name = "rwkv5_1b5_wkv_fwd_bwd_bf16"
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    if args.config == 2 and any(c.status() for c in fwd + bwd):
        raise RuntimeError("a device-side wait ran out during the run")
    print(json.dumps({"config_index": args.config, "workload": name, "metric": METRIC,
                      "value": B * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                      "algorithmic_bytes_per_step": bytes_step,
                      "roofline_frac": bytes_step / (ms * 1e-3) / 1e9 / hbm, "peak_source": which,
                      "steps": args.steps, "warmup": args.warmup}), flush=True)


def _time_steps(step, steps, warmup):
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / steps


def run_stream_config(args):
    """One GPU's share of the long-context stream: v6 3B shape (C=2560, 40 heads) with the heads
    split over 8 GPUs -> 5 heads per GPU, B=1, segments of 4096 tokens with the state carried,
    forward plus truncated backward per segment (no state gradient across segments).  Five chains
    cannot fill 148 SMs by themselves: the library cuts every segment's chain into time groups."""
    import rwkv_infctx_trainer_b200 as W
    from rwkv_infctx_trainer_b200 import wkv56
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    hbm, which = peaks()
    B, H, seg, nseg = 1, 5, 4096, args.segments
    C, T = H * 64, seg * args.segments
    g = torch.Generator(device="cuda").manual_seed(0)
    mk = lambda: torch.randn((nseg, B, seg, C), generator=g, device=device).to(torch.bfloat16)
    r, k, v, gy = mk(), mk(), mk(), mk()
    w = (torch.randn((nseg, B, seg, C), generator=g, device=device) * 0.5 - 0.6).to(torch.bfloat16)
    u = (torch.rand((H, 64), generator=g, device=device) * 2 - 1).to(torch.bfloat16)
    s0 = torch.zeros((B, H, 64, 64), device=device)

    def make_step(groups):
        # every call prepared once: a step is 2 * nseg crossings of the C ABI
        states = [s0] + [torch.empty_like(s0) for _ in range(nseg)]
        calls = []
        for i in range(nseg):
            f = wkv56.prepare_forward("wkv6", r[i], k[i], v[i], w[i], u, states[i], w_kind=W.WKV_W_RAW,
                                      state_out=states[i + 1], time_groups=groups)
            b = wkv56.prepare_backward("wkv6", r[i], k[i], v[i], w[i], u, states[i], gy[i], None,
                                       w_kind=W.WKV_W_RAW, ckpt=f.ckpt, want_gstate=False, time_groups=groups)
            calls += [f, b]

        def step():
            for c in calls:
                c.run()
        return step

    steps, warmup = max(1, min(args.steps, 5)), max(1, min(args.warmup, 2))
    ms = _time_steps(make_step(0), steps, warmup)
    ms_uncut = _time_steps(make_step(1), 1, 1)
    bytes_step = (FWD_ELEMS + BWD_ELEMS) * 2 * B * T * C
    print(json.dumps({"config_index": 4, "workload": "rwkv6_3b_stream_5_heads_of_40", "metric": METRIC,
                      "value": B * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                      "segments": nseg, "us_per_segment": ms * 1e3 / nseg,
                      "value_chains_uncut": B * T / (ms_uncut * 1e-3),
                      "us_per_segment_chains_uncut": ms_uncut * 1e3 / nseg,
                      "algorithmic_bytes_per_step": bytes_step,
                      "roofline_frac": bytes_step / (ms * 1e-3) / 1e9 / hbm, "peak_source": which,
                      "note": "5 (batch x head) chains per GPU: launch- and latency-bound, not HBM-bound",
                      "steps": steps, "warmup": warmup}), flush=True)


def run_ref_kernels(args):
    """The RWKV-infctx-trainer project's own CUDA kernels, compiled unchanged for sm_100a
    (oracle/_ref/, test infrastructure), timed with CUDA events on the shapes and inputs they are
    valid for: v4 (wkv_cuda_bf16.cu:160-172) on the v4 workload at bf16; v5 (wkv5_cuda.cu:348-383)
    on the v5 workload with a zero state; v6 (wkv6state_cuda_v1.cu:295-308) on one batch row of
    the v6 workload.  Forward + backward of every BPTT segment; prints one JSON line per variant."""
    import ctypes
    from oracle import build as OB
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    hbm, which = peaks()
    P = lambda t: ctypes.c_void_p(t.data_ptr())
    g = torch.Generator(device="cuda").manual_seed(0)
    BF = torch.bfloat16
    steps, warmup = max(1, min(args.steps, 10)), max(1, min(args.warmup, 3))

    def lib(name):
        path = os.path.join(OB.REF_DIR, name)
        return ctypes.CDLL(path) if os.path.exists(path) else None

    def report(name, cite, B, T, C, elems, ms, note):
        nbytes = elems * 2 * B * T * C
        print(json.dumps({"ref_kernel": name, "source": cite, "metric": METRIC, "value": B * T / (ms * 1e-3),
                          "unit": "tokens/s", "ms_per_step": ms, "B": B, "T": T, "C": C,
                          "algorithmic_gbs": nbytes / (ms * 1e-3) / 1e9,
                          "roofline_frac": nbytes / (ms * 1e-3) / 1e9 / hbm, "peak_source": which,
                          "note": note, "steps": steps, "warmup": warmup}), flush=True)

    rn = lambda *s: torch.randn(s, generator=g, device=device).to(BF)
    # ---- v4: B=8, T=4096 as 2 x 2048, C=2048, bf16 (the only dtype the project's kernel has)
    L4 = lib("libref_wkv4.so")
    if L4 is not None:
        B, T, seg, C = 8, 4096, 2048, 2048
        k, v, gy = [[rn(B, seg, C) for _ in range(T // seg)] for _ in range(3)]
        w = -torch.exp(torch.rand(C, generator=g, device=device) * 6 - 5)
        u = (torch.rand(C, generator=g, device=device) * 2 - 1).to(BF)
        st = [torch.zeros((B, C, 3), device=device) for _ in range(T // seg + 1)]
        st[0][..., 2] = -1e38
        gst = [torch.empty((B, C, 3), device=device) for _ in range(T // seg + 1)]
        y, gk, gv = rn(B, seg, C), rn(B, seg, C), rn(B, seg, C)
        gw, gu = rn(B, C), rn(B, C)

        def step4():
            n = T // seg
            for i in range(n):
                L4.ref_wkv4_forward(B, seg, C, P(w), P(u), P(k[i]), P(v[i]), P(st[i]), P(y), P(st[i + 1]))
            for i in reversed(range(n)):
                gin = None if i == n - 1 else P(gst[i + 1])
                L4.ref_wkv4_backward(B, seg, C, P(w), P(u), P(k[i]), P(v[i]), P(st[i]), P(gy[i]), gin,
                                     P(gw), P(gu), P(gk), P(gv), P(gst[i]))
        report("v4", "RWKV-v4neo/cuda/wkv_cuda_bf16.cu:160-172", B, T, C, 8, _time_steps(step4, steps, warmup),
               "bf16 I/O; state and its gradient carried over 2 segments of 2048")
    # ---- v5: B=8, T=4096 as 2 x 2048, H=32; zero state (its backward ignores the state)
    L5 = lib("libref_wkv5.so")
    if L5 is not None:
        B, T, seg, H = 8, 4096, 2048, 32
        C = H * 64
        r, k, v, gy = [[rn(B, seg, C) for _ in range(T // seg)] for _ in range(4)]
        x = torch.rand((H, 64), generator=g, device=device) * 5 - 6
        ew = -torch.exp(x)
        eew = torch.exp(ew)
        u = (torch.rand((H, 64), generator=g, device=device) * 2 - 1).to(BF)
        zero = torch.zeros((B, H, 64, 64), device=device)
        y, gr, gk, gv = rn(B, seg, C), rn(B, seg, C), rn(B, seg, C), rn(B, seg, C)
        gw, gu = rn(B, C), rn(B, C)

        def step5():
            for i in range(T // seg):
                zero.zero_()
                L5.ref_wkv5_forward(1, B, seg, C, H, P(zero), P(r[i]), P(k[i]), P(v[i]), P(eew), P(u), P(y))
            zero.zero_()
            for i in reversed(range(T // seg)):
                L5.ref_wkv5_backward(1, B, seg, C, H, P(zero), P(r[i]), P(k[i]), P(v[i]), P(eew), P(ew), P(u),
                                     P(gy[i]), P(gr), P(gk), P(gv), P(gw), P(gu))
        report("v5", "RWKV-v5/src/module/cuda/wkv5_cuda.cu:348-383", B, T, C, 11, _time_steps(step5, steps, warmup),
               "bf16; every segment from a zero state (the kernel indexes its state without the batch "
               "row and its backward ignores it)")
    # ---- v6: one batch row of the 7B-shape workload, T=16384 as 4 x 4096, H=64
    L6 = lib("libref_wkv6state.so")
    if L6 is not None:
        B, T, seg, H = 1, 16384, 4096, 64
        C = H * 64
        r, k, v, gy = [[rn(B, seg, C) for _ in range(T // seg)] for _ in range(4)]
        ew = [(-torch.exp((torch.randn((B, seg, C), generator=g, device=device) * 0.5 - 0.6).to(BF).float()))
              for _ in range(T // seg)]
        u = (torch.rand((H, 64), generator=g, device=device) * 2 - 1).to(BF)
        s = [torch.zeros((B, H, 64, 64), device=device, dtype=BF) for _ in range(T // seg + 1)]
        y, gr, gk, gv, gw = rn(B, seg, C), rn(B, seg, C), rn(B, seg, C), rn(B, seg, C), rn(B, seg, C)
        gu, gs = rn(B, C), rn(B, H, 64, 64)

        def step6():
            n = T // seg
            for i in range(n):
                s[i + 1].copy_(s[i])
                L6.ref_wkv6_forward(B, seg, C, H, P(r[i]), P(k[i]), P(v[i]), P(ew[i]), P(u), P(s[i + 1]), P(y))
            for i in reversed(range(n)):
                L6.ref_wkv6_backward(B, seg, C, H, P(r[i]), P(k[i]), P(v[i]), P(ew[i]), P(u), P(s[i]), P(gy[i]),
                                     P(gr), P(gk), P(gv), P(gw), P(gu), P(gs))
        report("v6", "RWKV-v6/src/module/cuda/wkv6state_cuda_v1.cu:295-308", B, T, C, 14,
               _time_steps(step6, steps, warmup),
               "bf16, B=1 (the kernel indexes its state without the batch row): one of the workload's "
               "4 batch rows; state carried forward, its gradient output not chained (the kernel takes none)")
    if L4 is None and L5 is None and L6 is None:
        print(json.dumps({"ref_kernels": "unavailable", "why": "oracle/_ref/*.so not prebuilt"}), flush=True)


def run_neighbours(args):
    """The fused elementwise neighbours of the op (group-norm * gate, token-shift mixes) on one
    4096-token segment of the v6 7B-shape workload, forward and backward, next to the PyTorch
    expressions the trainer runs (RWKV-v6/src/module/TimeMix.py:262-273, 296-298) on the same GPU."""
    import torch.nn.functional as F
    import rwkv_infctx_trainer_b200 as W
    device = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    hbm, which = peaks()
    B, T, H = 4, 4096, 64
    C = H * 64
    g = torch.Generator(device="cuda").manual_seed(0)
    bf = torch.bfloat16
    rn = lambda *s: torch.randn(s, generator=g, device=device).to(bf)
    steps, warmup = max(3, min(args.steps, 20)), max(3, min(args.warmup, 5))
    eps = 64e-5
    y, gt, gout = rn(B, T, C).requires_grad_(True), rn(B, T, C).requires_grad_(True), rn(B, T, C)
    wt = torch.ones(C, device=device, dtype=bf).requires_grad_(True)
    bs = torch.zeros(C, device=device, dtype=bf).requires_grad_(True)
    x, sh = rn(B, T, C).requires_grad_(True), rn(B, C).requires_grad_(True)
    maa = torch.rand((5, C), generator=g, device=device).to(bf).requires_grad_(True)
    m = (rn(5, B, T, C) * 0.3).detach().requires_grad_(True)
    gout5 = rn(5, B, T, C)

    def fb(fn, grad):
        def step():
            fn().backward(grad)
        return step

    def eager_lnx():
        return F.group_norm(y.view(-1, C), H, wt, bs, eps).view(B, T, C) * gt

    def eager_mix():
        dx = torch.cat((sh.unsqueeze(1), x[:, :-1]), 1) - x
        return x.unsqueeze(0) + dx.unsqueeze(0) * (maa.view(5, 1, 1, C) + m)

    n = B * T * C * 2
    rows = [("lnx_gate", fb(lambda: W.lnx_gate(y, gt, wt, bs, eps, H), gout), fb(eager_lnx, gout), 8 * n),
            ("ddlerp5", fb(lambda: W.ddlerp(x, sh, maa, m), gout5), fb(eager_mix, gout5), (1 + 5 + 5 + 1 + 5 + 5 + 1) * n)]
    for name, ours, eager, nbytes in rows:
        ms_o, ms_e = _time_steps(ours, steps, warmup), _time_steps(eager, steps, warmup)
        print(json.dumps({"fused_neighbour": name, "shape": [B, T, C], "ms_fwd_bwd": ms_o,
                          "algorithmic_gbs": nbytes / (ms_o * 1e-3) / 1e9,
                          "roofline_frac": nbytes / (ms_o * 1e-3) / 1e9 / hbm, "peak_source": which,
                          "pytorch_eager_ms_fwd_bwd": ms_e, "speedup_vs_eager": ms_e / ms_o,
                          "steps": steps, "warmup": warmup}), flush=True)
    del y, gt, gout, x, sh, maa, m, gout5, rows
    torch.cuda.empty_cache()

    # the whole v6 time-mix block, forward + backward of one segment: the library's block next to
    # the same block with the mixes and the norm-gate written as PyTorch expressions (both use
    # the library's WKV op and cuBLAS projections)
    class EagerNeighbours(W.RWKV_TimeMix6_0):
        def forward(self, x, last_state):
            shift, wkv_state = last_state
            Bx, Tx, Cx = x.shape
            dx = torch.cat((shift.unsqueeze(1), x[:, :-1]), 1) - x
            xxx = torch.tanh((x + dx * self.time_maa_x) @ self.time_maa_w1).view(Bx * Tx, 5, -1).transpose(0, 1)
            mw, mk, mv, mr, mg = torch.bmm(xxx, self.time_maa_w2).view(5, Bx, Tx, Cx).unbind(0)
            xw, xk, xv = x + dx * (self.time_maa_w + mw), x + dx * (self.time_maa_k + mk), x + dx * (self.time_maa_v + mv)
            xr, xg = x + dx * (self.time_maa_r + mr), x + dx * (self.time_maa_g + mg)
            r, k, v, gg = self.receptance(xr), self.key(xk), self.value(xv), F.silu(self.gate(xg))
            w = self.time_decay + torch.tanh(xw @ self.time_decay_w1) @ self.time_decay_w2
            yy, wkv_state = W.WKV6.apply(Bx, Tx, Cx, self.n_head, r, k, v, w, self.time_faaaa, wkv_state)
            yy = self.ln_x(yy.view(-1, Cx)).view(Bx, Tx, Cx)
            return self.output(yy * gg), (x[:, -1], wkv_state)

    torch.manual_seed(0)
    blocks = {}
    for name, cls in (("fused", W.RWKV_TimeMix6_0), ("pytorch_expressions", EagerNeighbours)):
        blk = cls(1, 4, C, H, 64, C)
        with torch.no_grad():     # (the default initialisation leaves the low-rank maps at zero)
            blk.time_maa_w2.normal_(0, 0.02); blk.time_decay_w2.normal_(0, 0.02)
        blocks[name] = blk.to(device=device, dtype=bf)
    xb = rn(B, T, C).requires_grad_(True)
    state = (rn(B, C), torch.zeros((B, H, 64, 64), device=device))
    gob = rn(B, T, C)
    res = {name: _time_steps(fb(lambda blk=blk: blk(xb, state)[0], gob), steps, warmup) for name, blk in blocks.items()}
    print(json.dumps({"time_mix_block": "RWKV_TimeMix6_0", "shape": [B, T, C], "ms_fwd_bwd": res["fused"],
                      "ms_fwd_bwd_with_pytorch_expressions": res["pytorch_expressions"],
                      "speedup": res["pytorch_expressions"] / res["fused"],
                      "tokens_per_s": B * T / (res["fused"] * 1e-3), "steps": steps, "warmup": warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=500,
                    help="timed steps (the default makes the timed region about 2 s)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="strong (default): the workload's heads are split across the GPUs (needs H "
                         "divisible by N); weak: every GPU runs the whole workload")
    ap.add_argument("--config", type=int, default=3, choices=[1, 2, 3, 4],
                    help="3 (default): the headline v6 7B-shape workload; 1: v4 fp32 B=8 T=4096 C=2048; "
                         "2: v5 bf16 1.5B shape; 4: one GPU's 5-head slice of the v6 1M-token stream "
                         "(side measurements, one GPU)")
    ap.add_argument("--ref-kernels", action="store_true",
                    help="side measurement: the project's own CUDA kernels (oracle/_ref/, compiled "
                         "unchanged for sm_100a) on the shapes they are valid for")
    ap.add_argument("--neighbours", action="store_true",
                    help="side measurement: the fused group-norm*gate and token-shift-mix kernels next to "
                         "the PyTorch expressions, one 4096-token segment of the v6 7B shape")
    ap.add_argument("--segments", type=int, default=256, help="--config 4: BPTT segments of 4096 tokens")
    ap.add_argument("--small", action="store_true",
                    help="profiling aid: one batch row, one 4096-token segment (170 MB of inputs, "
                         "still larger than L2) instead of the benchmark workload")
    ap.add_argument("--medium", action="store_true",
                    help="profiling aid: the benchmark's batch and heads but a single 4096-token segment "
                         "(under 2 GB on the device) -- the grid sizes of the benchmark's launches")
    ap.add_argument("--dtype", default="fp32", choices=["fp32", "bf16"],
                    help="--config 1 only: I/O dtype of the v4 workload (the benchmark names fp32; the "
                         "project's own v4 kernel is bf16 only)")
    ap.add_argument("--heads", type=int, default=0,
                    help="profiling aid: this many heads instead of 64 (8 = what one of 8 GPUs gets)")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling aid: no end-to-end leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling aid: no CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.ref_kernels:
        run_ref_kernels(args)
    elif args.neighbours:
        run_neighbours(args)
    elif args.config == 4:
        run_stream_config(args)
    elif args.config != 3:
        run_side_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
