#!/usr/bin/env python
"""Benchmark of the sparse entmax attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
                    [--workload c3|c4|c5|mid|small|c2|v1] [--path auto|simt|tcgen05]
                    [--sections LIST|none]

One step = one forward + backward of causal entmax-1.5 `adasplash_v2` over one
batch of seeded synthetic inputs.  The default workload is the configuration
the headline metric is quoted on (B=4, Hq=Hkv=32, N=8192, D=128, bf16, inputs
N(0,1)*1.5, niter=1).  With N > 1 GPUs (one process per GPU under torchrun)
every rank runs its own copy of that batch -- the (batch x kv-head) shards are
independent, so there is no collective on the data path -- and the headline
value is the work of all ranks divided by the slowest rank's time (weak scaling).

Prints ONE JSON line (rank 0).  Beside the headline it carries sub-records
(`--sections`, default all that apply):

  fwd_only   forward-only time and throughput of the headline workload
  c2         row-wise entmax 16384 x 4096 fp32: three alphas, forward / backward GB/s
  c4, c5     the GQA + varlen and the long-context configurations (3 steps each)
  sharded    strong scaling of the long-context configuration: its 16 (batch x kv-head)
             shards split over the ranks (adasplash_b200/sharding.py), per-rank times, and
             the same job on rank 0 alone in the same run
  triton     the reference's own Triton kernels (unmodified, from baseline/_ref) timed on the
             same device tensors as the headline workload (1 GPU only; first call compiles)
  latency    host-side latency of a small call (N = 256)

`--impl reference` times the reference's CPU dense entmax attention (the oracle's
restatement of `slow_entmax_attention`) on the host cores instead.
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
NOMINAL_BF16_TFLOPS = 2250.0   # dense bf16 tensor-core peak of a B200 as NVIDIA states it
ALL_SECTIONS = ("fwd_only", "c2", "c4", "c5", "sharded", "triton", "latency")

# dram__bytes_read.sum + dram__bytes_write.sum of one launch of a kernel, from the
# ncu captures summarised under profiles/ (None = not captured for that workload)
NCU_DRAM_BYTES_PER_LAUNCH = {
    # headline workload: captured on the 32-head "mid" case (profiles/*_bf16_d128_mid.txt) and
    # scaled by 4 to the 128 heads of C3 (traffic is per head: every head streams its own q/k/v)
    ("c3", "solve"): 4 * (225.10e6 + 10.92e6),
    ("c3", "solve_with_export"): 4 * (226.04e6 + 18.88e6),   # profiles/solve_export_bf16_d128_mid.txt
    ("mid", "solve_with_export"): 226.04e6 + 18.88e6,
    ("c3", "fwd"): 4 * (202.50e6 + 103.72e6),
    ("c3", "bwd_dq"): 4 * (270.74e6 + 52.86e6),
    ("c3", "bwd_dkv"): 4 * (270.71e6 + 108.38e6),
    ("mid", "solve"): 225.10e6 + 10.92e6,
    ("mid", "fwd"): 202.50e6 + 103.72e6,
    ("mid", "bwd_dq"): 270.74e6 + 52.86e6,
    ("mid", "bwd_dkv"): 270.71e6 + 108.38e6,
    # profiles/entmax_fwd_f32_16384x4096.txt
    ("c2", "entmax_fwd"): 268.54e6 + 213.76e6,
}


def dense_equiv_flops(w, lens, fwd_only=False):
    """FlashAttention convention, causal: 7 * Hq * D * sum_b L_b^2 for fwd+bwd, 2 * ... forward."""
    return (2.0 if fwd_only else 7.0) * w["Hq"] * w["D"] * float(sum(l * l for l in lens))


def max_over_ranks(ms, world, device):
    """Slowest rank's elapsed time (the only communication of a multi-GPU run, outside
    the timed region; works on the nccl and the gloo backend alike)."""
    if world <= 1:
        return float(ms)
    import torch.distributed as dist
    t = torch.tensor([float(ms)], device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_over_ranks(ms, world):
    """Every rank's elapsed time, in rank order (host-side, gloo)."""
    if world <= 1:
        return [float(ms)]
    import torch.distributed as dist
    out = [torch.zeros(1, dtype=torch.float64) for _ in range(world)]
    dist.all_gather(out, torch.tensor([float(ms)], dtype=torch.float64))
    return [float(x.item()) for x in out]


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


def make_inputs_device(w, seed, dev):
    """The same distributions drawn on the device (sub-records: no host copy of gigabytes)."""
    g = torch.Generator(device=dev).manual_seed(seed)
    B, Hq, Hkv, N, D = w["B"], w["Hq"], w["Hkv"], w["N"], w["D"]

    def mk(shape, scale):
        t = torch.empty(shape, dtype=torch.bfloat16, device=dev)
        for b in range(shape[0]):
            t[b] = (torch.randn(shape[1:], generator=g, device=dev) * scale).to(torch.bfloat16)
        return t
    q, k, v, do = mk((B, Hq, N, D), w["scale"]), mk((B, Hkv, N, D), w["scale"]), mk((B, Hkv, N, D), w["scale"]), \
        mk((B, Hq, N, D), 1.0)
    lens, varlen = [N] * B, None
    if w["varlen"]:
        gc = torch.Generator().manual_seed(seed)
        vl = torch.randint(N // 4, N + 1, (B,), generator=gc, dtype=torch.int32)
        lens = [int(x) for x in vl]
        varlen = vl.to(dev)
        do.mul_(torch.arange(N, device=dev)[None, None, :, None] < varlen[:, None, None, None])
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
            return self
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
        return self

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


def spread_cpu_affinity(rank, world):
    """Give each rank of a multi-process run its own slice of the CPUs this process may use, so
    that the ranks' copy and launch threads do not share cores.  (On this pool's boxes NVML and
    `nvidia-smi topo` report the same CPU set and NUMA node for all eight GPUs, so there is no
    per-GPU locality to honour.)  Returns the CPUs chosen, or None if left alone."""
    if world <= 1 or not hasattr(os, "sched_getaffinity"):
        return None
    try:
        cpus = sorted(os.sched_getaffinity(0))
        per = len(cpus) // world
        if per < 2:
            return None
        mine = cpus[rank * per:(rank + 1) * per]
        os.sched_setaffinity(0, mine)
        return mine
    except Exception:
        return None


def tile_counts(bmask, lens, Hq):
    """Counts over a block mask (B, Hq, rows_padded, n_words), on the device.

    active     64x64 tiles whose bit is set -- the tiles the reference computes
    causal     64x64 tiles of the causal (and length-limited) triangle
    visits_q   128x128 (query tile, key tile) pairs with any of their four bits set: what the
               forward and dQ kernels issue, in units of 64x64 tiles = 4 per visit
    visits_kv  (128-key tile, 64-query block) pairs with any of their two bits set: what the
               dK/dV kernel issues, = 2 per visit
    """
    B, H, rows, words = bmask.shape
    nbp = words * 32
    shifts = torch.arange(32, device=bmask.device, dtype=torch.int32)
    active = visits_q = visits_kv = 0
    for b in range(B):  # one batch item at a time bounds the unpacked copy
        bits = ((bmask[b].unsqueeze(-1) >> shifts) & 1).bool().reshape(H, rows, nbp)
        r2, c2 = rows // 2 * 2, nbp // 2 * 2
        active += int(bits.sum().item())
        visits_q += int(bits[:, :r2, :c2].reshape(H, r2 // 2, 2, c2 // 2, 2).any(4).any(2).sum().item())
        visits_kv += int(bits[:, :, :c2].reshape(H, rows, c2 // 2, 2).any(3).sum().item())
    causal = 0
    for l in lens:
        nb = (l + 63) // 64
        causal += nb * (nb + 1) // 2
    return {"active": active, "causal": causal * Hq, "issued_q": 4 * visits_q, "issued_kv": 2 * visits_kv}


def timed_steps(fn, steps, warm, barrier=None):
    """CUDA-event time per step of `fn` on the current stream after `warm` untimed steps."""
    for _ in range(warm):
        fn()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / steps


def kernel_times(att, q, k, v, do, out2, taus, bmask, varlen, niter, reps):
    """Per-kernel CUDA-event times of the tile kernels through the C ABI, run on every head (no
    support buffer): `reps` back-to-back launches of one kernel."""
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
    ms = {"solve": ev(lambda: att.solve(q, k, niter, varlen)),
          "fwd": ev(lambda: att.forward_raw(q, k, v, taus, bmask, varlen))}
    bufs = att.backward_raw(q, k, v, do, out2, taus, bmask, varlen, niter)
    for name, mask in (("bwd_delta", 1), ("bwd_transpose", 2), ("bwd_dq", 4), ("bwd_dkv", 8)):
        ms[name] = ev(lambda: att.backward_raw(q, k, v, do, out2, taus, bmask, varlen, niter,
                                               stages=mask, buffers=bufs))
    return ms


def route_record(att, q, k, v, do, varlen, niter, reps):
    """Which route the heads take when the solver may export the rows' supports, and the times
    of the three calls of a step on that route (CUDA events, `reps` back-to-back calls each):
    solver + export; forward (gather kernel for the sparse heads, tile kernel for the others);
    backward (row and key gather kernels, tile kernels for the others)."""
    shape = att.make_shape(q, k, niter, varlen)
    sup = att.support_buffer(shape, q.device)
    B, Hq, N, _ = q.shape
    Hkv = k.shape[1]
    if sup is None:
        return {"kv_heads": B * Hkv, "kv_heads_on_gather_kernels": 0, "note": "no gather route for this shape"}
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
    ms = {"solve_with_export": ev(lambda: att.solve(q, k, niter, varlen, support=sup))}
    taus, bmask = att.solve(q, k, niter, varlen, support=sup)
    torch.cuda.synchronize()
    entries = int(sup[:4].view(torch.int32).item())
    why = sup[16:32].view(torch.int32).tolist()
    dense = sup[256:256 + 4 * B * Hkv].view(torch.int32)
    sparse_heads = int((dense == 0).sum().item())
    ms["fwd"] = ev(lambda: att.forward_raw(q, k, v, taus, bmask, varlen, support=sup))
    out, out2 = att.forward_raw(q, k, v, taus, bmask, varlen, support=sup)
    ms["bwd"] = ev(lambda: att.backward_raw(q, k, v, do, out2, taus, bmask, varlen, niter, support=sup))
    rows = sum(int(x) for x in (varlen.tolist() if varlen is not None else [N] * B)) * Hq
    return {"kv_heads": B * Hkv, "kv_heads_on_gather_kernels": sparse_heads,
            "support_entries_per_row": round(entries / max(1, rows), 2),
            # solver CTAs (256 rows each) that could not export, by reason
            "ctas_without_export": {"pool_overflow": why[0], "rows_too_dense": why[2], "entry_array_full": why[3]},
            "call_ms": {n: round(x, 3) for n, x in ms.items()}}


def attention_record(w, q, k, v, do, varlen, lens, niter, steps, kernel_reps, gpu_index):
    """fwd+bwd and forward-only times of the public call on device-resident tensors, per-kernel
    times, measured block sparsity and issued vs useful tile products; with its own clock record."""
    import adasplash_b200 as adasplash
    from adasplash_b200 import attention as att

    def step():
        qq, kk, vv = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        out = adasplash.adasplash_v2(qq, kk, vv, niter=niter, varlen=varlen)
        torch.autograd.grad(out, (qq, kk, vv), do)

    def fwd():
        adasplash.adasplash_v2(q.detach(), k.detach(), v.detach(), niter=niter, varlen=varlen)
    sampler = ClockSampler(gpu_index).start()
    ms = timed_steps(step, steps, 1)
    ms_fwd = timed_steps(fwd, steps, 1)
    clocks = sampler.stop()
    out = adasplash.adasplash_v2(q.detach().requires_grad_(True), k.detach(), v.detach(), niter=niter, varlen=varlen)
    saved = out.grad_fn.saved_tensors
    out2, taus, bmask = saved[3], saved[4], saved[5]
    del out
    qd, kd, vd = q.detach(), k.detach(), v.detach()
    kms = kernel_times(att, qd, kd, vd, do, out2, taus, bmask, varlen, niter, kernel_reps)
    route = route_record(att, qd, kd, vd, do, varlen, niter, kernel_reps)
    tc = tile_counts(bmask, lens, w["Hq"])
    g = 2.0 * 64 * 64 * w["D"]
    pk = peaks()
    kflops = {"solve": 2.0 * tc["causal"] * g, "fwd": 3.0 * tc["active"] * g, "bwd_dq": 3.0 * tc["active"] * g,
              "bwd_dkv": 4.0 * tc["active"] * g}
    dom = max(kflops, key=lambda s: kms[s])
    useful = 10.0 * tc["active"]
    issued = 6.0 * tc["issued_q"] + 4.0 * tc["issued_kv"]
    flops = dense_equiv_flops(w, lens)
    return {
        "workload": w["label"], "steps": steps, "ms_per_step": round(ms, 3), "fwd_ms": round(ms_fwd, 3),
        "tflops_dense_equiv": round(flops / ms / 1e9, 1),
        "fwd_tflops_dense_equiv": round(dense_equiv_flops(w, lens, True) / ms_fwd / 1e9, 1),
        "block_sparsity": round(1.0 - tc["active"] / max(1, tc["causal"]), 4),
        "route": route,
        "tile_kernel_ms": {n: round(x, 3) for n, x in kms.items()},
        "dominant_tile_kernel": dom,
        "dominant_tile_kernel_tflops": round(kflops[dom] / kms[dom] / 1e9, 1),
        "dominant_tile_kernel_frac_of_burst_peak": round(kflops[dom] / kms[dom] / 1e9 / pk["bf16_tflops"], 3),
        # tile products at the kernels' own granularity (128x128 forward / dQ, 128 keys x 64 queries
        # dK/dV; a visited tile computes all of its 64x64 sub-tiles) over those whose bit is set
        "issued_over_useful_tile_products": round(issued / max(1.0, useful), 3),
        # the tile products the block mask stands for (what the reference executes): over the sum of
        # the tile kernels' times (the tile route), and over the time of the step as run, where
        # heads on the gather route replace those products by a few pairs per row (an equivalent,
        # not tensor work)
        "tile_route_executed_tile_tflops": round((kflops["solve"] + useful * g) / sum(kms.values()) / 1e9, 1),
        "step_block_mask_equivalent_tflops": round((kflops["solve"] + useful * g) / ms / 1e9, 1),
        "lens": lens if w["varlen"] else None,
        "clocks": clocks,
    }, (out2, taus, bmask, kms, tc)


def rowwise_measure(dev, steps, warm):
    """Row-wise entmax on 16384 x 4096 fp32 = N(0,1)*4: forward / backward times of the three
    alphas of the configuration, algorithmic GB/s (8 bytes per element forward, 12 backward)."""
    import adasplash_b200 as adasplash
    rows, cols = 16384, 4096
    g = torch.Generator(device=dev).manual_seed(SEED_BASE + 1)
    x = (torch.randn(rows, cols, generator=g, device=dev) * 4).requires_grad_(True)
    dy = torch.randn(rows, cols, generator=g, device=dev)
    fb, bb = 8.0 * rows * cols, 12.0 * rows * cols
    pk = peaks()
    per_alpha = {}
    for tag, kw in (("alpha1.5", dict(alpha=1.5, n_iter=2, use_histogram=True)), ("alpha2.0", dict(alpha=2.0)),
                    ("alpha1.333", dict(alpha=1.333, use_histogram=False))):
        y = adasplash.triton_entmax(x, **kw)
        f_ms = timed_steps(lambda: adasplash.triton_entmax(x.detach(), **kw), steps, warm)
        b_ms = timed_steps(lambda: torch.autograd.grad(y, x, dy, retain_graph=True), steps, warm)
        per_alpha[tag] = {"fwd_ms": round(f_ms, 4), "bwd_ms": round(b_ms, 4),
                          "fwd_gbs": round(fb / f_ms / 1e6, 1), "bwd_gbs": round(bb / b_ms / 1e6, 1),
                          "fwd_frac_of_hbm_peak": round(fb / f_ms / 1e6 / pk["hbm_gbs"], 3),
                          "bwd_frac_of_hbm_peak": round(bb / b_ms / 1e6 / pk["hbm_gbs"], 3)}
        del y
    return per_alpha, x, dy


def triton_reference_record(q, k, v, do, niter, ours_step):
    """The reference's unmodified Triton kernels (installed under baseline/_ref) on the same
    device tensors: median of 10 forward and forward+backward calls after the compiling first
    call, and this library timed the same way right before."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "adasplash")):
        return "unavailable: baseline/_ref/adasplash is not installed"
    try:
        import triton
        sys.path.insert(0, ref_dir)
        import adasplash as ref
        assert os.path.abspath(ref.__file__).startswith(os.path.abspath(ref_dir)), ref.__file__
    except Exception as e:  # noqa: BLE001
        return f"unavailable: {type(e).__name__}: {e}"

    def median_ms(fn, reps=10):
        ts = []
        for _ in range(reps):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            fn()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b))
        ts.sort()
        return ts[len(ts) // 2]
    try:
        for _ in range(2):
            ours_step()
        ours_ms = median_ms(ours_step)
        qq, kk, vv = (t.detach().clone().requires_grad_(True) for t in (q, k, v))

        def ref_fwd():
            return ref.adasplash_v2(qq, kk, vv, niter=niter)

        def ref_step():
            torch.autograd.grad(ref_fwd(), (qq, kk, vv), do)
        t0 = time.time()
        ref_step()
        torch.cuda.synchronize()
        first = time.time() - t0
        ref_step()
        fwd_ms = median_ms(ref_fwd)
        fb_ms = median_ms(ref_step)
        return {"fwd_ms": round(fwd_ms, 3), "fwdbwd_ms": round(fb_ms, 3), "ours_fwdbwd_ms": round(ours_ms, 3),
                "speedup_fwdbwd": round(fb_ms / ours_ms, 3), "triton": triton.__version__,
                "first_call_s": round(first, 1), "protocol": "median of 10 calls, CUDA events, same device tensors"}
    except Exception as e:  # noqa: BLE001
        return f"unavailable: {type(e).__name__}: {e}"


def sharded_record(world, rank, dev, gpu_index, steps, barrier):
    """Strong scaling of the long-context configuration: its B * Hkv = 16 shards are split over
    the ranks, every rank draws its shards on its own GPU from the shards' seeds and runs
    forward + backward on them; the job's time is the slowest rank's.  With more than one rank,
    rank 0 then runs all 16 shards alone for the 1-GPU time of the same run."""
    import adasplash_b200 as adasplash
    from adasplash_b200 import sharding as sh
    w = WORKLOADS["c5"]
    G = w["Hq"] // w["Hkv"]
    shards = sh.enumerate_shards(w["B"], w["Hkv"], w["N"])
    parts = sh.assign(shards, world)

    def run(my, sync):
        q, k, v, do, varlen = sh.make_rank_batch(my, G, w["N"], w["D"], SEED_BASE + 4, w["scale"], torch.bfloat16, dev)

        def step():
            qq, kk, vv = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
            out = adasplash.adasplash_v2(qq, kk, vv, niter=1, varlen=varlen)
            torch.autograd.grad(out, (qq, kk, vv), do)
        ms = timed_steps(step, steps, 1, sync)
        out = adasplash.adasplash_v2(q.detach().requires_grad_(True), k.detach(), v.detach(), niter=1, varlen=varlen)
        bm = out.grad_fn.saved_tensors[5]
        tc = tile_counts(bm, [w["N"]] * len(my), G)
        return ms, 1.0 - tc["active"] / max(1, tc["causal"])
    sampler = ClockSampler(gpu_index).start() if rank == 0 else None
    ms_mine, sparsity = run(parts[rank], barrier)
    clocks = sampler.stop() if sampler else None
    per_rank = gather_over_ranks(ms_mine, world)
    per_rank_sparsity = gather_over_ranks(sparsity, world)
    ms = max(per_rank)
    flops = dense_equiv_flops(w, [w["N"]] * w["B"])
    rec = {"workload": w["label"], "shards": len(shards), "shards_per_rank": [len(p) for p in parts],
           "assignment": "round-robin over shard id (equal lengths)", "steps": steps,
           "ms_per_step": round(ms, 2), "per_rank_ms": [round(x, 2) for x in per_rank],
           "per_rank_block_sparsity": [round(x, 4) for x in per_rank_sparsity],
           "tflops_dense_equiv": round(flops / ms / 1e9, 1), "scaling": "strong", "clocks": clocks}
    torch.cuda.empty_cache()
    if world > 1:
        ms1 = 0.0
        if rank == 0:
            ms1, _ = run(shards, None)   # the other ranks wait at the barrier below
        barrier()
        rec["ms_per_step_1gpu_same_run"] = round(ms1, 2)
        rec["speedup_vs_1gpu"] = round(ms1 / ms, 3) if rank == 0 else None
        rec["limiter"] = ("slowest rank's data-dependent sparse work (per_rank_ms), no communication"
                          if rank == 0 else None)
    else:
        rec["speedup_vs_1gpu"] = 1.0
    return rec


def small_call_latency(dev):
    """Host + device time of one small forward+backward call (B=1, H=2, N=256, D=64, bf16):
    what the per-call set-up (tensor maps, attribute calls, allocations) costs."""
    import adasplash_b200 as adasplash
    g = torch.Generator(device=dev).manual_seed(7)
    q, k, v, do = ((torch.randn(1, 2, 256, 64, generator=g, device=dev)).bfloat16() for _ in range(4))

    def step():
        qq, kk, vv = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        out = adasplash.adasplash_v2(qq, kk, vv, niter=1)
        torch.autograd.grad(out, (qq, kk, vv), do)
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 200
    for _ in range(n):
        step()
    torch.cuda.synchronize()
    return round((time.perf_counter() - t0) / n * 1e6, 1)


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
    cpus = spread_cpu_affinity(rank, world)   # before the pinned buffers are allocated
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if args.path:
        _lib.set_kernel_path(args.path)
    sections = set(ALL_SECTIONS if args.sections == "all" else
                   [] if args.sections == "none" else args.sections.split(","))
    if args.workload != "c3":
        sections &= {"fwd_only", "latency"}
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

    def step_e2e(compute=True):
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
                if compute:
                    qq.requires_grad_(True); kk.requires_grad_(True); vv.requires_grad_(True)
                    out = adasplash.adasplash_v2(qq, kk, vv, niter=niter, varlen=vl)
                    res = (out.detach(),) + tuple(torch.autograd.grad(out, (qq, kk, vv), dd))
                else:
                    res = (qq, dd, kk, vv)   # the same bytes back, no kernels: the copy ceiling
            s_out.wait_stream(s_run)
            with torch.cuda.stream(s_out):
                for h, d in zip(host_out, res):
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
    e2e_steps = max(2, min(args.steps, 5))
    ms_e2e, _ = timed(step_e2e, e2e_steps, 1)
    ms_copy, _ = timed(lambda: step_e2e(False), e2e_steps, 1)

    flops = dense_equiv_flops(w, lens)
    value = aggregate_tflops(world, flops, ms_step)
    e2e_value = aggregate_tflops(world, flops, ms_e2e)
    h2d = sum(t.numel() * t.element_size() for t in (hq, hk, hv, hdo))
    d2h = sum(t.numel() * t.element_size() for t in host_out)

    # per-kernel timing through the C ABI (rank 0) for the roofline: CUDA events on the
    # launching stream around `reps` back-to-back launches of one kernel
    roof = None
    extra = {}
    sub = {}
    if rank == 0:
        pk = peaks()
        out = adasplash.adasplash_v2(q.requires_grad_(True), k, v, niter=niter, varlen=vl_dev)
        saved = out.grad_fn.saved_tensors
        out2, taus, bmask = saved[3], saved[4], saved[5]
        del out
        qd, kd, vd = q.detach(), k.detach(), v.detach()
        kernel_ms = kernel_times(att, qd, kd, vd, do, out2, taus, bmask, vl_dev, niter, reps=10)
        # The solver computes S twice (row maxima, then the candidate lists); the remaining steps
        # of the reference's (3 + niter) sweeps run on the lists.
        tc = tile_counts(bmask, lens, w["Hq"])
        g = 2.0 * 64 * 64 * w["D"]
        solver_f = 2.0 * tc["causal"] * g
        total_f = solver_f + 10.0 * tc["active"] * g
        kernel_flops = {"solve": solver_f, "fwd": 3.0 * tc["active"] * g, "bwd_dq": 3.0 * tc["active"] * g,
                        "bwd_dkv": 4.0 * tc["active"] * g}
        # The step as run: heads whose supports the solver exported go through the gather kernels
        # (no tensor work beyond the solver's), the others through the tile kernels.
        route = route_record(att, qd, kd, vd, do, vl_dev, niter, reps=10)
        all_gather = route.get("kv_heads_on_gather_kernels", 0) == route["kv_heads"]
        if all_gather:
            dom = "solve"
            dom_ms = route["call_ms"]["solve_with_export"]
        else:
            dom = max(kernel_flops, key=lambda s: kernel_ms[s])
            dom_ms = kernel_ms[dom]
        achieved = kernel_flops[dom] / (dom_ms * 1e-3) / 1e12
        # a kernel timed alone in a region of tens of milliseconds runs at burst clocks: the burst
        # cuBLAS figure is the denominator; the sustained and the nominal ones are given beside it
        peak = pk["bf16_tflops"]
        roof = {"bound": "tensor", "kernel": dom, "achieved": round(achieved, 2), "peak": peak,
                "unit": "TFLOP/s", "frac": round(achieved / peak, 4),
                "frac_sustained": round(achieved / pk["bf16_tflops_sustained"], 4),
                "frac_nominal": round(achieved / NOMINAL_BF16_TFLOPS, 4),
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get((args.workload, "solve_with_export" if all_gather else dom)),
                "peak_source": pk["source"] + " (burst cuBLAS bf16: the kernel is timed alone, 10 launches back to back; "
                "frac_sustained = against the seconds-long cuBLAS loop, frac_nominal = against 2250 TFLOP/s)",
                "algorithmic_flops_per_launch": kernel_flops[dom],
                "ms_per_launch": round(dom_ms, 3),
                "note": ("every kv head runs on the gather kernels: the solver (with the support export) is the "
                         "only tensor-core kernel of the step and its longest" if all_gather else
                         "longest tile kernel (run on every head)")}
        rows_total = float(w["B"] * w["Hq"] * w["N"])
        delta_bytes = rows_total * (2 * w["D"] * 2 + 4)
        step_tflops = total_f / (ms_step * 1e-3) / 1e12

        def fracs(x):
            return {"of_burst": round(x / pk["bf16_tflops"], 3), "of_sustained": round(x / pk["bf16_tflops_sustained"], 3),
                    "of_nominal": round(x / NOMINAL_BF16_TFLOPS, 3)}
        extra = {
            "route": route,
            # the tile kernels timed on every head (no support buffer): the route of heads that are
            # too dense for the solver's lists, and of callers that pass no buffer
            "tile_kernel_ms": {k2: round(v2, 3) for k2, v2 in kernel_ms.items()},
            "tile_kernel_tflops": {k2: round(kernel_flops[k2] / (kernel_ms[k2] * 1e-3) / 1e12, 1)
                                   for k2 in kernel_flops},
            "tile_kernel_frac_of_burst_peak": {k2: round(kernel_flops[k2] / (kernel_ms[k2] * 1e-3) / 1e12 / peak, 3)
                                               for k2 in kernel_flops},
            "tile_route_step_ms": round(sum(kernel_ms.values()), 3),
            "bwd_delta_hbm_gbs": round(delta_bytes / (kernel_ms["bwd_delta"] * 1e-3) / 1e9, 1),
            "bwd_delta_frac_of_hbm_peak": round(delta_bytes / (kernel_ms["bwd_delta"] * 1e-3) / 1e9 / pk["hbm_gbs"], 3),
            "solver_hbm_gbs": round((h2d / 2 + 4 * rows_total) / (kernel_ms["solve"] * 1e-3) / 1e9, 1),
            # the tile products the block mask stands for (what the reference executes): over the sum
            # of the tile kernels' times -- the executed-tile throughput of the tile route -- and over
            # the time of the step as run, where heads on the gather route replace those products by
            # a few pairs per row (an equivalent: it says how much work was avoided, not what the
            # tensor pipe did)
            "tile_route_executed_tile_tflops": round(total_f / (sum(kernel_ms.values()) * 1e-3) / 1e12, 2),
            "tile_route_executed_tile_frac_of_peak": fracs(total_f / (sum(kernel_ms.values()) * 1e-3) / 1e12),
            "step_block_mask_equivalent_tflops": round(step_tflops, 2),
            "issued_over_useful_tile_products": round(
                (6.0 * tc["issued_q"] + 4.0 * tc["issued_kv"]) / max(1.0, 10.0 * tc["active"]), 3),
            "block_sparsity": round(1.0 - tc["active"] / max(1, tc["causal"]), 4),
            "resolved_path": {1: "simt", 2: "tcgen05"}.get(
                _lib.load().adasplash2_resolved_path(__import__("ctypes").byref(
                    att.make_shape(q, k, niter, vl_dev))), "?"),
        }
        del out2, taus, bmask
        if "fwd_only" in sections:
            s2 = ClockSampler(local).start()
            f_ms = timed_steps(lambda: adasplash.adasplash_v2(qd, kd, vd, niter=niter, varlen=vl_dev),
                               max(5, args.steps), 2)
            sub["fwd_only"] = {"ms": round(f_ms, 3),
                               "tflops_dense_equiv": round(dense_equiv_flops(w, lens, True) / f_ms / 1e9, 1),
                               "clocks": s2.stop()}
        if "latency" in sections:
            sub["small_call_latency_us"] = {"fwd_bwd_B1_H2_N256_D64_bf16": small_call_latency(dev)}
    cpu = cpu_baseline(rank, world) if rank == 0 else None
    triton_rec = None
    if rank == 0 and world == 1 and "triton" in sections:
        triton_rec = triton_reference_record(q.detach(), k.detach(), v.detach(), do, niter, step_device)
    # the sub-records need the memory of the headline tensors
    del q, k, v, do, hq, hk, hv, hdo, host_out
    torch.cuda.empty_cache()
    if rank == 0 and world == 1:
        if "c2" in sections:
            s2 = ClockSampler(local).start()
            per_alpha, x, dy = rowwise_measure(dev, max(10, args.steps), 3)
            sub["c2"] = {"workload": "row-wise entmax 16384x4096 fp32 = N(0,1)*4, dY N(0,1)", "per_alpha": per_alpha,
                         "hbm_peak_gbs": peaks()["hbm_gbs"], "clocks": s2.stop()}
            del x, dy
            torch.cuda.empty_cache()
        if "c4" in sections:
            w4 = WORKLOADS["c4"]
            ins = make_inputs_device(w4, SEED_BASE + 3, dev)
            sub["c4"], keep = attention_record(w4, *ins, niter=1, steps=3, kernel_reps=2, gpu_index=local)
            del ins, keep
            torch.cuda.empty_cache()
    if "sharded" in sections or ("c5" in sections and world == 1):
        rec = sharded_record(world, rank, dev, local, 3, barrier)
        if rank == 0:
            sub["sharded"] = {"c5": rec}
    if rank == 0 and world == 1 and "c5" in sections:
        w5 = WORKLOADS["c5"]
        # one kv head of each batch item with its 8 query heads: the per-kernel split and the
        # issued / useful tile products of the long-context configuration
        w5s = dict(w5, B=2, Hq=8, Hkv=1, label=w5["label"] + " [2 of its 16 shards]")
        ins = make_inputs_device(w5s, SEED_BASE + 4, dev)
        sub["c5"], keep = attention_record(w5s, *ins, niter=1, steps=3, kernel_reps=2, gpu_index=local)
        sub["c5"]["full_config"] = {k2: sub["sharded"]["c5"][k2] for k2 in ("ms_per_step", "tflops_dense_equiv")}
        del ins, keep
        torch.cuda.empty_cache()
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
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    # the same copies on the same three streams with no kernel between them
                    "copy_only_ms": round(ms_copy, 3), "copy_frac": round(ms_copy / ms_e2e, 3),
                    "copy_gbs_per_gpu": round((h2d + d2h) / ms_copy / 1e6, 1),
                    "cpus_of_rank0": None if cpus is None else f"{cpus[0]}-{cpus[-1]}"},
            "gpu_launches": int(launches),
            "clocks": clocks,
            "roofline": roof,
            "cpu_baseline": cpu,
        }
        line.update(extra)
        line.update(sub)
        if triton_rec is not None:
            line["triton_reference"] = triton_rec
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


V1_METRIC = "adasplash (alpha=2, full attention) fwd+bwd dense-equivalent TFLOP/s, bf16"


def run_v1(args):
    """Secondary workload: the first-generation semantics on the tensor-core kernels --
    `adasplash(q, k, v, alpha=2.0, is_causal=False)` (sparsemax, full attention, niter = 10),
    B=4, H=32, N=8192, D=64, bf16, inputs N(0,1) -- beside the same call on the CUDA-core
    kernels (one step: they take seconds).  Dense-equivalent FLOPs: 14 * H * D * N^2 per batch item."""
    import adasplash_b200 as adasplash
    from adasplash_b200 import _lib
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, H, N, D = 4, 32, 8192, 64
    g = torch.Generator(device=dev).manual_seed(SEED_BASE + 5)
    q, k, v, do = ((torch.randn(B, H, N, D, generator=g, device=dev)).bfloat16() for _ in range(4))

    def step():
        qq, kk, vv = q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        out = adasplash.adasplash(qq, kk, vv, alpha=2.0, is_causal=False)
        torch.autograd.grad(out, (qq, kk, vv), do)
    sampler = ClockSampler(dev.index).start()
    l0 = _lib.launch_count()
    ms = timed_steps(step, args.steps, max(3, args.warmup))
    launches = _lib.launch_count() - l0
    clocks = sampler.stop()
    _lib.set_kernel_path("simt")
    ms_simt = timed_steps(step, 1, 1)
    _lib.set_kernel_path(None)
    flops = 14.0 * B * H * D * float(N) * N
    line = {
        "metric": V1_METRIC, "value": round(flops / ms / 1e9, 1), "unit": "TFLOP/s", "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": round(ms, 3), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "adasplash alpha=2.0 is_causal=False niter=10, bf16 B=4 H=32 N=8192 D=64",
                   "l2": "q, k, v, dO are 134 MB each (> 126 MB L2)"},
        "gpu_launches": int(launches), "clocks": clocks,
        "cuda_core_kernels_ms_per_step": round(ms_simt, 1),
        "tensor_core_over_cuda_core": round(ms_simt / ms, 1),
    }
    print(json.dumps(line), flush=True)


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
        "roofline": {"bound": "hbm", "kernel": "entmax_fwd_pipe_kernel<float,128,8>", "achieved": f["fwd_gbs"],
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
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS) + ["c2", "v1"])
    ap.add_argument("--path", default=None, choices=["auto", "simt", "tcgen05"])
    ap.add_argument("--sections", default="all",
                    help="'all', 'none' or a comma list of: " + ",".join(ALL_SECTIONS))
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "c2":
        run_rowwise(args)
    elif args.workload == "v1":
        run_v1(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
