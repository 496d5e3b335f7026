#!/usr/bin/env python
"""WKV forward+backward throughput on B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One step = one pass of the op over the v6 7B-shape workload: bf16 r,k,v,w,gy of
shape [B=4, T=16384, C=4096] (H=64 heads of 64), processed as 4 BPTT segments of
4096 tokens -- forward over all segments with the fp32 state carried, then
backward over them in reverse with the state gradient carried.  Synthetic
inputs: r,k,v,gy ~ N(0,1), x ~ N(-0.6,0.5) (decay exp(-exp(x))), u ~ U(-1,1).

With N GPUs every rank runs the same workload on its own (batch x head) units:
no collective on the data path, weak scaling, value = N * tokens / max-over-ranks
time.  Prints ONE JSON line (rank 0).

``--impl reference`` times the reference's own CPU implementation of the path
(the chunked pure-PyTorch algorithm, oracle/wkv_chunked_port.py) on the host
cores, on a bounded sample of the same workload.
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


class ClockSampler:
    """nvidia-smi sampling of SM clock and throttle reasons while the timed region runs."""

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
    """Device-resident step: raw op calls (package wrappers over the C ABI), preallocated
    outputs are created by the wrappers; events around every backward launch."""

    def __init__(self, wl, dev_inputs, device):
        import rwkv_infctx_trainer_b200 as W
        from rwkv_infctx_trainer_b200 import wkv56
        self.W, self.wkv56, self.wl, self.d, self.device = W, wkv56, wl, dev_inputs, device
        self.bounds = [(t0, min(wl["T"], t0 + wl["seg"])) for t0 in range(0, wl["T"], wl["seg"])]
        B, H, N = wl["B"], wl["H"], wl["N"]
        self.state0 = torch.zeros((B, H, N, N), device=device)
        self.bwd_events = []
        self.fwd_events = []
        self.launches = 0

    def seg(self, name, t0, t1):
        return self.d[name][:, t0:t1]

    def step(self, record=False):
        W, d = self.W, self.d
        states = [self.state0]
        ckpts = []
        for t0, t1 in self.bounds:
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            y, s, ck = self.wkv56.forward("wkv6", self.seg("r", t0, t1), self.seg("k", t0, t1),
                                          self.seg("v", t0, t1), self.seg("w", t0, t1), d["u"],
                                          states[-1], w_kind=W.WKV_W_RAW, save_ckpt=True)
            ckpts.append(ck)
            if record:
                e1.record()
                self.fwd_events.append((e0, e1))
            states.append(s)
            self.launches += 1          # k_chunk_fwd
        gs = None
        out = None
        for (t0, t1), s_in, ck in reversed(list(zip(self.bounds, states[:-1], ckpts))):
            if record:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            out = self.wkv56.backward("wkv6", self.seg("r", t0, t1), self.seg("k", t0, t1),
                                      self.seg("v", t0, t1), self.seg("w", t0, t1), d["u"], s_in,
                                      self.seg("gy", t0, t1), gs, w_kind=W.WKV_W_RAW, ckpt=ck)
            if record:
                e1.record()
                self.bwd_events.append((e0, e1))
            gs = out[5]
            self.launches += 3          # k_chunk_dscan, k_chunk_bwd, k_reduce_partials
        return out


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
    H_total = wl["H"]
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

    class SegRunner(Runner):
        def seg(self, name, t0, t1):
            return segd[name][t0 // wl["seg"]]

    runner = SegRunner(wl, dev, device)
    torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        runner.step()
    barrier()
    runner.launches = 0
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    t_start, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_start.record()
    for _ in range(args.steps):
        runner.step(record=True)
    t_end.record()
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    ms = t_start.elapsed_time(t_end)
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
    e2e_steps = max(1, min(args.steps, 6))
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
                       "l2": "inputs (2.7 GB per GPU) larger than L2, no flush"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "tokens/s", "h2d_bytes_per_step": h2d,
                    "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "how": "WKV6.apply + autograd; pinned host buffers; copies of step s+1 (in) and "
                           "s-1 (out) overlap the compute of step s on side streams"},
            "gpu_launches": launches,
            "roofline": {"bound": "hbm",
                         "kernel": "wkv6 backward of one BPTT segment: k_chunk_dscan + k_chunk_bwd "
                                   "(+ k_reduce_partials), timed as one launch group",
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


def cpu_baseline(steps: int, warmup: int) -> dict:
    from oracle import wkv_chunked_port as P
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    t, head_tokens, desc = cpu_sample()
    run = lambda: P.run_chain("v6", t["r"], t["k"], t["v"], t["x"], t["u"], t["s"], t["gy"],
                              WORKLOAD["seg"])
    for _ in range(warmup):
        run()
    t0 = time.perf_counter()
    for _ in range(steps):
        run()
    dt = (time.perf_counter() - t0) / steps
    # tokens/s of the full-width op (all H heads) at this head-token rate
    return {"value": head_tokens / dt / WORKLOAD["H"], "unit": "tokens/s", "cores": cores,
            "kind": "port", "sample": desc, "head_tokens_per_s": head_tokens / dt,
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
    if args.config == 1:
        B, T, seg, C, dt = 8, 4096, 2048, 2048, torch.float32
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

        def step():
            for i in range(len(segs)):
                L.check(lib.wkv4_forward(B, seg, C, code, w.data_ptr(), u.data_ptr(), kk[i].data_ptr(),
                                         vv[i].data_ptr(), states[i].data_ptr(), ys[i].data_ptr(),
                                         states[i + 1].data_ptr(), wsf.data_ptr(), nwf, st), "wkv4_forward")
            for i in reversed(range(len(segs))):
                gin = None if i == len(segs) - 1 else gst[i + 1].data_ptr()
                L.check(lib.wkv4_backward(B, seg, C, code, w.data_ptr(), u.data_ptr(), kk[i].data_ptr(),
                                          vv[i].data_ptr(), states[i].data_ptr(), gg[i].data_ptr(), gin,
                                          gw.data_ptr(), gu.data_ptr(), gk[i].data_ptr(), gv[i].data_ptr(),
                                          gst[i].data_ptr(), ws.data_ptr(), nws, st), "wkv4_backward")
        bytes_step = 8 * 4 * B * T * C
        name = "rwkv4_wkv_fwd_bwd_fp32"
    else:
        B, T, seg, C, H = 8, 4096, 2048, 2048, 32
        dt = torch.bfloat16
        r, k, v, gy = (torch.randn((B, T, C), generator=g).to(dt).to(device) for _ in range(4))
        w = (torch.rand((H, 64), generator=g) * 5 - 6).to(device)
        u = (torch.rand((H, 64), generator=g) * 2 - 1).to(dt).to(device)
        segs = [(a, a + seg) for a in range(0, T, seg)]
        cs = lambda t: [t[:, a:b].contiguous() for a, b in segs]
        rr, kk, vv, gg = cs(r), cs(k), cs(v), cs(gy)
        s0 = torch.zeros((B, H, 64, 64), device=device)

        def step():
            states, cks = [s0], []
            for i in range(len(segs)):
                y, s, ck = wkv56.forward("wkv5", rr[i], kk[i], vv[i], w, u, states[-1], w_kind=W.WKV_W_RAW,
                                         save_ckpt=True)
                states.append(s); cks.append(ck)
            gs = None
            for i in reversed(range(len(segs))):
                out = wkv56.backward("wkv5", rr[i], kk[i], vv[i], w, u, states[i], gg[i], gs,
                                     w_kind=W.WKV_W_RAW, ckpt=cks[i])
                gs = out[5]
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
    print(json.dumps({"config_index": args.config, "workload": name, "metric": METRIC,
                      "value": B * T / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms,
                      "algorithmic_bytes_per_step": bytes_step,
                      "roofline_frac": bytes_step / (ms * 1e-3) / 1e9 / hbm, "peak_source": which,
                      "steps": args.steps, "warmup": args.warmup}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"],
                    help="weak: every GPU runs the whole workload; strong: the workload's heads "
                         "are split across the GPUs (needs H divisible by N)")
    ap.add_argument("--config", type=int, default=3, choices=[1, 2, 3],
                    help="3 (default): the headline v6 7B-shape workload; 1: v4 fp32 B=8 T=4096 C=2048; "
                         "2: v5 bf16 1.5B shape (side measurements, one GPU)")
    ap.add_argument("--small", action="store_true",
                    help="profiling aid: one batch row, one 4096-token segment (170 MB of inputs, "
                         "still larger than L2) instead of the benchmark workload")
    ap.add_argument("--medium", action="store_true",
                    help="profiling aid: the benchmark's batch and heads but a single 4096-token segment "
                         "(under 2 GB on the device) -- the grid sizes of the benchmark's launches")
    ap.add_argument("--skip-e2e", action="store_true", help="profiling aid: no end-to-end leg")
    ap.add_argument("--skip-cpu", action="store_true", help="profiling aid: no CPU baseline leg")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.config != 3:
        run_side_config(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
