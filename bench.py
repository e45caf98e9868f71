#!/usr/bin/env python
"""Benchmark of the sparse entmax attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c4|c5|small] [--path auto|simt|tcgen05]

One step = one forward + backward of causal entmax-1.5 `adasplash_v2` over one
batch of seeded synthetic inputs.  The default workload is the configuration
the headline metric is quoted on (B=4, Hq=Hkv=32, N=8192, D=128, bf16, inputs
N(0,1)*1.5, niter=1).  With N > 1 GPUs (one process per GPU under torchrun)
every rank runs its own copy of the batch -- the (batch x kv-head) shards are
independent, so there is no collective on the data path -- and the reported
value is the work of all ranks divided by the slowest rank's time.

Prints ONE JSON line (rank 0).  `--impl reference` times the reference's CPU
dense entmax attention (the oracle's restatement of `slow_entmax_attention`)
on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

METRIC = "adasplash_v2 fwd+bwd dense-equivalent TFLOP/s (causal entmax-1.5, bf16)"

WORKLOADS = {
    # name: B, Hq, Hkv, N, D, input scale, varlen?
    "c3": dict(B=4, Hq=32, Hkv=32, N=8192, D=128, scale=1.5, varlen=False,
               label="adasplash_v2 causal alpha=1.5 bf16 B=4 Hq=Hkv=32 N=8192 D=128 niter=1"),
    "c4": dict(B=8, Hq=32, Hkv=8, N=16384, D=128, scale=1.0, varlen=True,
               label="adasplash_v2 GQA+varlen bf16 B=8 Hq=32 Hkv=8 N=16384 D=128 niter=1"),
    "c5": dict(B=2, Hq=64, Hkv=8, N=65536, D=128, scale=1.5, varlen=False,
               label="adasplash_v2 long context bf16 B=2 Hq=64 Hkv=8 N=65536 D=128 niter=1"),
    "mid": dict(B=2, Hq=16, Hkv=16, N=8192, D=128, scale=1.5, varlen=False,
                label="adasplash_v2 bf16 B=2 Hq=Hkv=16 N=8192 D=128 niter=1 (ncu capture case, 268 MB of inputs)"),
    "small": dict(B=1, Hq=8, Hkv=8, N=2048, D=128, scale=1.5, varlen=False,
                  label="adasplash_v2 bf16 B=1 Hq=Hkv=8 N=2048 D=128 niter=1 (profiling case)"),
}
SEED_BASE = 20260

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of a kernel, from the
# ncu captures summarised under profiles/ (None = not captured for that workload)
NCU_DRAM_BYTES_PER_LAUNCH = {
    # headline workload: captured on the 32-head "mid" case (profiles/*_bf16_d128_mid.txt) and
    # scaled by 4 to the 128 heads of C3 (traffic is per head: every head streams its own q/k/v)
    ("c3", "solve"): 4 * (225.10e6 + 10.92e6),
    ("c3", "fwd"): 4 * (202.50e6 + 103.72e6),
    ("c3", "bwd_dq"): 4 * (270.74e6 + 52.86e6),
    ("c3", "bwd_dkv"): 4 * (270.71e6 + 108.38e6),
    ("mid", "solve"): 225.10e6 + 10.92e6,
    ("mid", "fwd"): 202.50e6 + 103.72e6,
    ("mid", "bwd_dq"): 270.74e6 + 52.86e6,
    ("mid", "bwd_dkv"): 270.71e6 + 108.38e6,
    # profiles/entmax_fwd_f32_16384x4096.txt
    ("c2", "entmax_fwd"): 268.49e6 + 219.89e6,
}


def dense_equiv_flops(w, lens):
    """FlashAttention convention, causal: 7 * Hq * D * sum_b L_b^2 for fwd+bwd."""
    return 7.0 * w["Hq"] * w["D"] * float(sum(l * l for l in lens))


def max_over_ranks(ms, world, device):
    """Slowest rank's elapsed time (the only communication of a multi-GPU run, outside
    the timed region; works on the nccl and the gloo backend alike)."""
    if world <= 1:
        return float(ms)
    import torch.distributed as dist
    t = torch.tensor([float(ms)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def aggregate_tflops(world, flops_per_rank, ms_step):
    """Whole-job throughput: every rank processed `flops_per_rank` per step in the
    slowest rank's time."""
    return world * flops_per_rank / (ms_step * 1e-3) / 1e12


def make_inputs(w, rank, pinned=True):
    """Seeded synthetic q,k,v,dO on the host (bf16), per-rank seed."""
    g = torch.Generator().manual_seed((SEED_BASE + 2) * 1000 + rank)
    B, Hq, Hkv, N, D = w["B"], w["Hq"], w["Hkv"], w["N"], w["D"]

    def mk(shape, scale):
        t = torch.empty(shape, dtype=torch.bfloat16, pin_memory=pinned)
        # generate head by head to bound the fp32 temporary
        for b in range(shape[0]):
            t[b] = (torch.randn(shape[1:], generator=g) * scale).to(torch.bfloat16)
        return t
    q = mk((B, Hq, N, D), w["scale"])
    k = mk((B, Hkv, N, D), w["scale"])
    v = mk((B, Hkv, N, D), w["scale"])
    do = mk((B, Hq, N, D), 1.0)
    lens = [N] * B
    varlen = None
    if w["varlen"]:
        varlen = torch.randint(N // 4, N + 1, (B,), generator=g, dtype=torch.int32)
        lens = [int(x) for x in varlen]
        rows = torch.arange(N)[None, None, :, None] < varlen[:, None, None, None]
        do.mul_(rows)
    return q, k, v, do, varlen, lens


class ClockSampler:
    """Samples SM clock, power and throttle reasons while the timed region runs.

    Reads through NVML from a thread of this process every few milliseconds (a timed region of
    a few steps lasts tens of milliseconds, too short for `nvidia-smi -lms`); if NVML cannot be
    loaded it falls back to an `nvidia-smi` child.  Only reads: no setting is touched.
    `sm_mhz` is the median clock of the samples taken under load, i.e. whose power draw is at
    least half of the highest draw seen.
    """
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown",
                   0x40: "hw_thermal_slowdown"}

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []       # (sm_mhz, watts)
        self.reasons = set()
        self.max_mhz = None
        self._stop = False

    def _nvml_loop(self, nv, handle):
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                watts = nv.nvmlDeviceGetPowerUsage(handle) / 1000.0
                bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((float(mhz), watts))
                for bit, name in self.REASON_BITS.items():
                    if bits & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.003)

    def start(self):
        try:
            import pynvml as nv
            import threading
            nv.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(torch.cuda.current_device()).uuid)
                handle = nv.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
        elif self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except Exception:
                self.proc.kill()
            try:
                for line in open(self.path):
                    f = [x.strip() for x in line.split(",")]
                    if len(f) < 9:
                        continue
                    try:
                        self.samples.append((float(f[1]), float(f[3])))
                        self.max_mhz = float(f[2])
                    except ValueError:
                        continue
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown",
                                          "sw_power_cap"), f[5:9]):
                        if val.lower() == "active":
                            self.reasons.add(name)
                os.unlink(self.path)
            except Exception:
                pass
        else:
            return out
        if self.samples:
            top = max(w for _, w in self.samples)
            load = sorted(m for m, w in self.samples if w >= 0.5 * top) or sorted(m for m, _ in self.samples)
            out["sm_mhz"] = load[len(load) // 2]
            out["sm_max_mhz"] = self.max_mhz
            out["samples"] = len(self.samples)
            out["samples_under_load"] = len(load)
            out["max_watts"] = round(top, 1)
        out["reasons"] = sorted(self.reasons)
        return out


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"],
                "hbm_gbs": p["hbm_gbs"], "source": "measured"}
    return {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0,
            "source": "fallback"}


def executed_tile_flops(bmask, w, lens, niter, sweeps):
    """FLOPs of the 64x64xD tile products the kernels issue: `sweeps` dense causal
    QK^T passes of the solver plus 3 (forward) + 3 + 4 (backward) products per
    active tile.  Returns (total, solver, active_tiles, causal_tiles)."""
    g = 2.0 * 64 * 64 * w["D"]
    causal_tiles = 0
    for l in lens:
        nb = (l + 63) // 64
        causal_tiles += nb * (nb + 1) // 2
    causal_tiles *= w["Hq"]
    words = bmask.view(torch.int32).flatten()
    active = 0
    # popcount on the device, chunked
    x = words.to(torch.int64) & 0xFFFFFFFF
    for s in range(32):
        active += int(((x >> s) & 1).sum().item())
    solver = sweeps * causal_tiles * g
    return solver + 10.0 * active * g, solver, active, causal_tiles


def run_ours(args):
    import adasplash_b200 as adasplash
    from adasplash_b200 import _lib, attention as att
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # the shards are independent: the only inter-rank traffic is the barrier and the
        # max-reduction of the elapsed time, both host-side (gloo); NCCL is not needed
        dist.init_process_group("gloo")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.path:
        _lib.set_kernel_path(args.path)
    w = WORKLOADS[args.workload]
    niter = 1
    hq, hk, hv, hdo, varlen, lens = make_inputs(w, rank)
    vl_dev = None if varlen is None else varlen.to(dev)
    q, k, v, do = (t.to(dev, non_blocking=True) for t in (hq, hk, hv, hdo))
    torch.cuda.synchronize()

    def step_device():
        qq, kk, vv = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        out = adasplash.adasplash_v2(qq, kk, vv, niter=niter, varlen=vl_dev)
        grads = torch.autograd.grad(out, (qq, kk, vv), do)
        return out, grads

    host_out = [torch.empty_like(t, pin_memory=True) for t in (hq, hq, hk, hv)]

    # End to end: the batch items are independent, so the public call is issued per batch
    # item on its own stream and the H2D copy of item b+1, the kernels of item b and the D2H
    # copy of item b-1 overlap (three streams, ordered by events; everything is joined back
    # into the current stream, which the timing events are recorded on).
    s_in, s_run, s_out = (torch.cuda.Stream(device=dev) for _ in range(3))
    B_items = w["B"]

    def step_e2e():
        cur = torch.cuda.current_stream()
        for st in (s_in, s_run, s_out):
            st.wait_stream(cur)
        for bi in range(B_items):
            with torch.cuda.stream(s_in):
                qq, kk, vv, dd = (t[bi:bi + 1].to(dev, non_blocking=True) for t in (hq, hk, hv, hdo))
                vl = None if vl_dev is None else vl_dev[bi:bi + 1]
            s_run.wait_stream(s_in)
            with torch.cuda.stream(s_run):
                for t in (qq, kk, vv, dd):
                    t.record_stream(s_run)
                qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
                out = adasplash.adasplash_v2(qq, kk, vv, niter=niter, varlen=vl)
                grads = torch.autograd.grad(out, (qq, kk, vv), dd)
            s_out.wait_stream(s_run)
            with torch.cuda.stream(s_out):
                for h, d in zip(host_out, (out.detach(),) + tuple(grads)):
                    d.record_stream(s_out)
                    h[bi:bi + 1].copy_(d, non_blocking=True)
        for st in (s_in, s_run, s_out):
            cur.wait_stream(st)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps, warm):
        for _ in range(warm):
            fn()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_count()
        a.record()
        for _ in range(steps):
            fn()
        b.record()
        barrier()
        ms = a.elapsed_time(b)
        launches = _lib.launch_count() - l0
        ms = max_over_ranks(ms, world, torch.device("cpu"))
        return ms / steps, launches

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    ms_step, launches = timed(step_device, args.steps, args.warmup)
    clocks = sampler.stop() if rank == 0 else None
    ms_e2e, _ = timed(step_e2e, max(2, min(args.steps, 5)), 1)

    flops = dense_equiv_flops(w, lens)
    value = aggregate_tflops(world, flops, ms_step)
    e2e_value = aggregate_tflops(world, flops, ms_e2e)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # per-kernel timing through the C ABI (rank 0) for the roofline: CUDA events on the
    # launching stream around `reps` back-to-back launches of one kernel
    roof = None
    extra = {}
    if rank == 0:
        pk = peaks()
        out = adasplash.adasplash_v2(q.requires_grad_(True), k, v, niter=niter, varlen=vl_dev)
        saved = out.grad_fn.saved_tensors
        out2, taus, bmask = saved[3], saved[4], saved[5]
        del out
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        reps = 5
        stream = torch.cuda.current_stream()

        def ev(fn):
            fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record(stream)
            for _ in range(reps):
                fn()
            b.record(stream)
            torch.cuda.synchronize()
            return a.elapsed_time(b) / reps
        kernel_ms = {"solve": ev(lambda: att.solve(qd, kd, niter, vl_dev)),
                     "fwd": ev(lambda: att.forward_raw(qd, kd, vd, taus, bmask, vl_dev))}
        bufs = att.backward_raw(qd, kd, vd, do, out2, taus, bmask, vl_dev, niter)
        for name, mask in (("bwd_delta", 1), ("bwd_transpose", 2), ("bwd_dq", 4), ("bwd_dkv", 8)):
            kernel_ms[name] = ev(lambda: att.backward_raw(qd, kd, vd, do, out2, taus, bmask, vl_dev,
                                                          niter, stages=mask, buffers=bufs))
        # The solver computes S twice (row maxima, then the candidate lists); the remaining steps
        # of the reference's (3 + niter) sweeps run on the lists.  A CTA whose candidate pool
        # overflows sweeps S (3 + niter) times: its extra products are not counted here.
        sweeps = 2
        total_f, solver_f, active, causal_tiles = executed_tile_flops(bmask, w, lens, niter, sweeps)
        g = 2.0 * 64 * 64 * w["D"]
        kernel_flops = {"solve": solver_f, "fwd": 3.0 * active * g, "bwd_dq": 3.0 * active * g,
                        "bwd_dkv": 4.0 * active * g}
        dom = max(kernel_flops, key=lambda s: kernel_ms[s])
        achieved = kernel_flops[dom] / (kernel_ms[dom] * 1e-3) / 1e12
        peak = pk["bf16_tflops_sustained"]
        roof = {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 2), "peak": peak,
                "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((args.workload, dom)),
                "peak_source": pk["source"] + " (sustained cuBLAS bf16; the kernel runs inside a long step)",
                "algorithmic_flops_per_launch": kernel_flops[dom],
                "ms_per_launch": round(kernel_ms[dom], 3)}
        rows_total = float(w["B"] * w["Hq"] * w["N"])
        delta_bytes = rows_total * (2 * w["D"] * 2 + 4)
        extra = {
            "kernel_ms": {k2: round(v2, 3) for k2, v2 in kernel_ms.items()},
            "kernel_tflops": {k2: round(kernel_flops[k2] / (kernel_ms[k2] * 1e-3) / 1e12, 1)
                              for k2 in kernel_flops},
            "kernel_frac_of_peak": {k2: round(kernel_flops[k2] / (kernel_ms[k2] * 1e-3) / 1e12 / peak, 3)
                                    for k2 in kernel_flops},
            "bwd_delta_hbm_gbs": round(delta_bytes / (kernel_ms["bwd_delta"] * 1e-3) / 1e9, 1),
            "bwd_delta_frac_of_hbm_peak": round(delta_bytes / (kernel_ms["bwd_delta"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
            "executed_tile_tflops": round(total_f / (ms_step * 1e-3) / 1e12, 2),
            "executed_tile_frac_of_peak": round(total_f / (ms_step * 1e-3) / 1e12 / peak, 4),
            "block_sparsity": round(1.0 - active / max(1, causal_tiles), 4),
            "resolved_path": {1: "simt", 2: "tcgen05"}.get(
                _lib.load().adasplash2_resolved_path(__import__("ctypes").byref(
                    att.make_shape(q, k, niter, vl_dev))), "?"),
        }
    cpu = cpu_baseline(rank, world) if rank == 0 else None
    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 3), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 3),
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": {"workload": w["label"], "per_gpu_batch": w["B"], "shards_per_gpu": w["B"] * w["Hkv"],
                       "parallelism": f"{world} x independent (batch x kv-head) shards, no collective",
                       "l2": "inputs (>= 1 GiB per step) exceed the 126 MB L2"},
            "e2e": {"value": round(e2e_value, 3), "unit": "TFLOP/s", "ms_per_step": round(ms_e2e, 3),
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roof,
            "cpu_baseline": cpu,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


ROWWISE_METRIC = "triton_entmax fwd+bwd algorithmic GB/s (x 16384x4096 fp32, alpha=1.5, n_iter=2, histogram)"


def run_rowwise(args):
    """Secondary workload: row-wise entmax on a 16384 x 4096 fp32 matrix = N(0,1)*4
    (HBM-bound).  One step = forward + backward for alpha = 1.5; alpha = 2.0 and
    1.333 are timed beside it.  Algorithmic bytes: 8 per element forward (read x,
    write y), 12 backward (read y, dy, write dx)."""
    import adasplash_b200 as adasplash
    from adasplash_b200 import _lib
    from oracle import entmax_oracle as O
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    rows, cols = 16384, 4096
    g = torch.Generator().manual_seed(SEED_BASE + 1)
    hx = torch.empty(rows, cols, pin_memory=True)
    hdy = torch.empty(rows, cols, pin_memory=True)
    for r0 in range(0, rows, 2048):
        hx[r0:r0 + 2048] = torch.randn(2048, cols, generator=g) * 4
        hdy[r0:r0 + 2048] = torch.randn(2048, cols, generator=g)
    x = hx.to(dev).requires_grad_(True)
    dy = hdy.to(dev)
    hdx = torch.empty(rows, cols, pin_memory=True)
    stream = torch.cuda.current_stream()

    def ev(fn, reps):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        l0 = _lib.launch_count()
        a.record(stream)
        for _ in range(reps):
            fn()
        b.record(stream)
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps, _lib.launch_count() - l0
    fb = 8.0 * rows * cols
    bb = 12.0 * rows * cols
    per_alpha = {}
    for tag, kw in (("alpha1.5", dict(alpha=1.5, n_iter=2, use_histogram=True)), ("alpha2.0", dict(alpha=2.0)),
                    ("alpha1.333", dict(alpha=1.333, use_histogram=False))):
        y = adasplash.triton_entmax(x, **kw)
        f_ms, _ = ev(lambda: adasplash.triton_entmax(x.detach(), **kw), args.steps)
        b_ms, _ = ev(lambda: torch.autograd.grad(y, x, dy, retain_graph=True), args.steps)
        per_alpha[tag] = {"fwd_ms": round(f_ms, 4), "bwd_ms": round(b_ms, 4),
                          "fwd_gbs": round(fb / f_ms / 1e6, 1), "bwd_gbs": round(bb / b_ms / 1e6, 1)}
        del y
    sampler = ClockSampler(dev.index)
    sampler.start()

    def step():
        yy = adasplash.triton_entmax(x, alpha=1.5, n_iter=2, use_histogram=True)
        torch.autograd.grad(yy, x, dy)
    ms, launches = ev(step, max(args.steps, 20))
    clocks = sampler.stop()

    def step_e2e():
        xx = hx.to(dev, non_blocking=True).requires_grad_(True)
        dd = hdy.to(dev, non_blocking=True)
        yy = adasplash.triton_entmax(xx, alpha=1.5, n_iter=2, use_histogram=True)
        (dx,) = torch.autograd.grad(yy, xx, dd)
        hdx.copy_(dx, non_blocking=True)
    ms_e2e, _ = ev(step_e2e, 5)
    pk = peaks()
    f = per_alpha["alpha1.5"]
    # CPU baseline: the oracle's restatement of the reference kernel on a 1024-row slice
    torch.set_num_threads(os.cpu_count() or 1)
    xs, dys = hx[:1024].clone(), hdy[:1024].clone()
    t0 = time.perf_counter()
    ys = O.rowwise_entmax_v2(xs, 1.5, 2, True)
    O.rowwise_entmax_backward(ys, dys, 1.5)
    tc = time.perf_counter() - t0
    line = {
        "metric": ROWWISE_METRIC, "value": round((fb + bb) / ms / 1e6, 1), "unit": "GB/s", "n_gpus": 1,
        "steps": max(args.steps, 20), "warmup": max(3, args.warmup), "ms_per_step": round(ms, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "row-wise entmax, x 16384x4096 fp32 = N(0,1)*4, dY N(0,1); forward + backward",
                   "l2": "x, y, dy, dx are 256 MiB each (> 126 MB L2)"},
        "e2e": {"value": round((fb + bb) / ms_e2e / 1e6, 1), "unit": "GB/s", "ms_per_step": round(ms_e2e, 3),
                "h2d_bytes_per_step": 2 * rows * cols * 4, "d2h_bytes_per_step": rows * cols * 4},
        "gpu_launches": int(launches), "clocks": clocks,
        "roofline": {"bound": "hbm", "kernel": "entmax_fwd_reg_kernel<float,128,8>", "achieved": f["fwd_gbs"],
                     "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(f["fwd_gbs"] / pk["hbm_gbs"], 4),
                     "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(("c2", "entmax_fwd")),
                     "peak_source": pk["source"] + " (STREAM-style copy)",
                     "algorithmic_bytes_per_launch": fb, "ms_per_launch": f["fwd_ms"]},
        "cpu_baseline": {"value": round(20.0 * 1024 * cols / tc / 1e9, 3), "unit": "GB/s", "cores": os.cpu_count(),
                         "kind": "port", "sample": "oracle restatement of the reference kernel, fwd+bwd, 1024x4096 slice",
                         "seconds": round(tc, 2)},
        "per_alpha": per_alpha,
    }
    print(json.dumps(line), flush=True)


def _cpu_sample(steps=1):
    """Bounded CPU sample: dense causal entmax-1.5 attention fwd+bwd, B=1, H=8,
    N=4096, D=128, fp32, all host threads."""
    from oracle import entmax_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    H, N, D = 8, 4096, 128
    g = torch.Generator().manual_seed(SEED_BASE)
    q, k, v, do = (torch.randn(1, H, N, D, generator=g) * s for s in (1.5, 1.5, 1.5, 1.0))
    O.cpu_dense_entmax15_attention(q[:, :1, :512], k[:, :1, :512], v[:, :1, :512], do[:, :1, :512])
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        O.cpu_dense_entmax15_attention(q, k, v, do)
        ts.append(time.perf_counter() - t0)
    flops = 7.0 * H * D * N * N
    return ts, flops, f"dense causal entmax-1.5 attention fwd+bwd, B=1 H=8 N={N} D={D} fp32, tau by 30-step bisection"


def cpu_baseline(rank, world):
    if world != 1:
        return None
    ts, flops, what = _cpu_sample(1)
    t = min(ts)
    return {"value": round(flops / t / 1e12, 5), "unit": "TFLOP/s", "cores": os.cpu_count(),
            "kind": "port", "sample": what, "seconds": round(t, 2)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    for _ in range(max(0, min(args.warmup, 1))):
        _cpu_sample(1)
    ts, flops, what = _cpu_sample(max(1, min(args.steps, 3)))
    t = sum(ts) / len(ts)
    val = round(flops / t / 1e12, 5)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": len(ts), "warmup": min(args.warmup, 1),
        "ms_per_step": round(t * 1e3, 1), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": WORKLOADS.get(args.workload, WORKLOADS["c3"])["label"], "sample": what},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": os.cpu_count(), "kind": "port",
                         "sample": what},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c2"])
    ap.add_argument("--path", default=None, choices=["auto", "simt", "tcgen05"])
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c2":
        run_rowwise(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
