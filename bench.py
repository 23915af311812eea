#!/usr/bin/env python
"""Benchmark of the INT8 SageAttention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C3] [--impl reference]

One "step" is one pass of the hot path (Q/K quantisation, with the K mean when smooth_k, + fp16 copy
of V; fused attention) over one batch of synthetic input of the named workload.  One JSON line is printed:

* ``value``     - attention TOPS, 4*B*Hq*Sq*Skv*D / t (benchmark_attn/benchmark_attn.py:40-47 of the
                  reference), timed through ``sageattn()`` on inputs resident in HBM, aggregated over
                  all ranks (time = max over ranks).
* ``roofline``  - the fused attention kernel against the tensor-core roofline (executed flops, burst
                  peak), from a second loop that calls the operators with events around each kernel;
                  ``roofline_prep`` gives the HBM-bound preparation kernel.
* ``e2e``       - the same metric through ``sageattn_host()`` with HOST (pinned) q, k, v and a host
                  output: the copies in both directions are inside the timed region; ``copy_floor_ms``
                  is the same bytes copied with no compute.
* ``allgather`` - N > 1: the step with the final all-gather of the outputs: NCCL after the step (serial),
                  NCCL on a side stream under the next step (overlapped), and written by the attention
                  kernel itself into every rank's copy over NVLink (fused).
* ``configs``   - N = 1: step time / TOPS / roofline fraction of the other benchmark configurations.
* ``cpu_baseline`` - the CPU oracle (a port of the reference's arithmetic) on the host cores, on a
                  bounded sample of the same workload.
* ``--impl reference`` - times that CPU oracle only (the reference has no CPU or NVIDIA
                  implementation of its own); rank 0 alone runs it.
With N > 1 the workload's (batch, kv-head) units are sharded over the ranks (strong scaling: every
rank generates and holds only its own units, no collective on the data path); ``--scaling weak``
runs the whole workload on every rank instead.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: B, Hq, Hkv, S, D, dtype, layout, causal, smooth_k, note
    "C1": dict(B=1, Hq=2, Hkv=2, S=1024, D=64, dtype="fp16", layout="HND", causal=False, smooth_k=False),
    "C2": dict(B=1, Hq=10, Hkv=10, S=4096, D=64, dtype="fp16", layout="NHD", causal=False, smooth_k=False),
    "C3": dict(B=2, Hq=32, Hkv=32, S=8192, D=128, dtype="bf16", layout="HND", causal=True, smooth_k=True),
    "C4": dict(B=4, Hq=32, Hkv=8, S=4096, D=128, dtype="bf16", layout="HND", causal=True, smooth_k=False),
    "C5": dict(B=1, Hq=24, Hkv=24, S=32768, D=128, dtype="fp16", layout="NHD", causal=False, smooth_k=False),
}
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
METRIC = "attention TOPS (4*B*H*S^2*D/t)"
DTYPE_NOTE = "int8 x int8 -> int32 (QK^T), fp16 x fp16 -> fp32 (PV), fp32 softmax"
# dram__bytes_read.sum + dram__bytes_write.sum of one sage_attn_kernel launch, from an ncu capture of
# this workload (ncu --set full -k regex:sage_ on `bench.py --steps 1 --warmup 3`)
ATTN_TRAFFIC_BYTES = {"C3": 379.3e6}


def nominal_ops(w, B=None):
    B = w["B"] if B is None else B
    return 4.0 * B * w["Hq"] * w["S"] * w["S"] * w["D"]


def executed_ops(w, B=None):
    B = w["B"] if B is None else B
    pairs = w["S"] * (w["S"] + 1) / 2 if w["causal"] else w["S"] * w["S"]
    return 4.0 * B * w["Hq"] * w["D"] * pairs


def make_inputs(w, name, seed_offset=0, heads=None, batch=None):
    """Seeded synthetic q, k, v of the workload's shape and value distribution (CPU generator)."""
    B = w["B"] if batch is None else batch
    Hq, Hkv = (w["Hq"], w["Hkv"]) if heads is None else heads
    S, D, dt = w["S"], w["D"], DTYPES[w["dtype"]]
    shape = (lambda h: (B, h, S, D)) if w["layout"] == "HND" else (lambda h: (B, S, h, D))

    def rn(shp, seed):
        g = torch.Generator(device="cpu").manual_seed(seed + seed_offset)
        return torch.randn(shp, generator=g, dtype=torch.float32)

    q, k, v = rn(shape(Hq), 0), rn(shape(Hkv), 1), rn(shape(Hkv), 2)
    g3 = torch.Generator(device="cpu").manual_seed(3 + seed_offset)
    if name == "C3":      # per-channel DC offset U(-4, 4) on K, shared across tokens
        off_shape = (1, Hkv, 1, D) if w["layout"] == "HND" else (1, 1, Hkv, D)
        k = k + (torch.rand(off_shape, generator=g3) * 8.0 - 4.0)
    if name == "C4":      # 1 % of q / k entries scaled x20
        q = torch.where(torch.rand(q.shape, generator=g3) < 0.01, q * 20.0, q)
        k = torch.where(torch.rand(k.shape, generator=g3) < 0.01, k * 20.0, k)
    return q.to(dt), k.to(dt), v.to(dt)


class ClockSampler:
    """Samples SM clock and throttle reasons of one GPU while a timed region runs."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            "hw_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
            "hw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
            "sw_thermal_slowdown": getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
            "sw_power_cap": getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4),
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if mask & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self.nv is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"],
                "bf16_tflops_sustained": p.get("bf16_tflops_sustained", p["bf16_tflops"]), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def cpu_oracle_run(w, name, steps, warmup):
    """Times the CPU oracle on a bounded sample: one (batch, kv-head) unit of the workload with
    its full sequence length.  Returns (TOPS of the sample, description, threads)."""
    from oracle import sage_oracle as so
    # torchrun pins OMP_NUM_THREADS=1; the CPU arm is meant to use every core this process may use
    try:
        torch.set_num_threads(max(1, len(os.sched_getaffinity(0))))
    except (AttributeError, RuntimeError):
        pass
    rep = w["Hq"] // w["Hkv"]
    S = w["S"]
    rows = S
    q, k, v = make_inputs(w, name, heads=(rep, 1), batch=1)
    times = []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        so.sageattn_emulated(q, k, v, tensor_layout=w["layout"], is_causal=w["causal"], smooth_k=w["smooth_k"])
        if i >= warmup:
            times.append(time.perf_counter() - t0)
    t = statistics.median(times)
    ops = 4.0 * rep * rows * S * w["D"]
    sample = (f"1 of {w['B'] * w['Hkv']} (batch, kv-head) units of {name} ({rep} query head(s), S={S}, D={w['D']}), "
              f"median of {steps} run(s) after {warmup} warm-up")
    cpu_oracle_run.last_ms = t * 1e3
    return ops / t / 1e12, sample, torch.get_num_threads()


def run_reference(args, w, name, rank):
    """The reference arm: the CPU oracle (a port of the reference's arithmetic; the reference has no
    CPU or NVIDIA implementation of its own) on the host cores, ``--warmup`` + ``--steps`` runs of a
    bounded sample (one (batch, kv-head) unit) of the workload."""
    if rank != 0:
        return
    steps, warmup = max(1, args.steps), max(0, args.warmup)
    tops, sample, threads = cpu_oracle_run(w, name, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": cpu_oracle_run.last_ms, "higher_is_better": True,
        "scaling": "strong",
        "vs_baseline": None, "dtype": DTYPE_NOTE, "data": "synthetic",
        "config": {"workload": workload_string(name, w)},
        "cpu_baseline": {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": tops, "unit": "TOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "the reference has no CPU or NVIDIA implementation; this is the CPU oracle (a PyTorch port of its "
                "arithmetic) on the host cores",
    }
    print(json.dumps(line), flush=True)


def workload_string(name, w):
    return (f"{name}: B={w['B']} Hq={w['Hq']} Hkv={w['Hkv']} S={w['S']} D={w['D']} {w['dtype']} {w['layout']} "
            f"{'causal' if w['causal'] else 'non-causal'} smooth_k={w['smooth_k']}")


def bind_near_gpu(index):
    """Run this process on the CPU cores NVML lists as local to GPU ``index`` (when it says so), so
    that pinned host buffers allocated afterwards are first touched on that socket.  Only this
    process's own CPU affinity changes; nothing on the GPU or the host is reconfigured."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(index)
        n_words = (os.cpu_count() + 63) // 64
        words = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (int(wd) >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class Problem:
    """One rank's share of a workload: ``units`` (batch, kv-head) units laid out as a batch of
    single-kv-head problems (identical work and memory traffic to a [B, H] slab), resident in HBM."""

    def __init__(self, w, name, units, full, seed_offset, dev, ops, lib):
        self.w, self.name, self.dev, self.ops = w, name, dev, ops
        rep = w["Hq"] // w["Hkv"]
        if full:
            self.host = make_inputs(w, name, seed_offset=seed_offset)
            self.Bl, self.Hql, self.Hkvl = w["B"], w["Hq"], w["Hkv"]
        else:
            self.host = make_inputs(w, name, seed_offset=seed_offset, heads=(rep, 1), batch=units)
            self.Bl, self.Hql, self.Hkvl = units, rep, 1
        self.units = units
        self.nominal = 4.0 * self.Bl * self.Hql * w["S"] * w["S"] * w["D"]
        self.executed = self.nominal * (executed_ops(w) / nominal_ops(w))
        self.layout_code = 1 if w["layout"] == "HND" else 0
        self.sm_scale = w["D"] ** -0.5
        self.q, self.k, self.v = (t.to(dev) for t in self.host)
        self.o = torch.empty_like(self.q)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.empty_mean = torch.empty(0, device=dev, dtype=self.q.dtype)
        self.attn_events, self.prep_events = [], []
        # the same choice sageattn() makes: one preparation launch for few heads, K mean + preparation otherwise
        self.fused_prep = bool(w["smooth_k"] and lib.sage_prep_smooth_preferred(self.Bl, self.Hkvl))
        self.launches_per_step = 2 + (1 if (w["smooth_k"] and not self.fused_prep) else 0)
        # a problem that fills the GPU unevenly runs on persistent CTAs and adds the merge kernel
        if lib.sage_attn_workspace_bytes(self.Bl, self.Hql, w["S"], w["S"], w["D"], int(w["causal"])) > 0:
            self.launches_per_step += 1

    @staticmethod
    def _ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def step_ops(self, record=False, o=None, peers=None):
        """The hot path as its operators, optionally with CUDA events around each kernel.  ``peers``:
        addresses of further copies of ``o`` (other GPUs' memory) that the attention kernel writes too."""
        w, ops = self.w, self.ops
        o = self.o if o is None else o
        bf16 = self.q.dtype == torch.bfloat16
        p0 = self._ev() if record else None
        if w["smooth_k"] and self.fused_prep:       # few heads: K mean and quantisation in one launch
            parts = ops.prep_smooth_qkv(self.q, self.k, self.v if bf16 else None, self.layout_code, self.sm_scale)
            q8, qs, k8, ks = parts[:4]
            v16, vl = (parts[5], 1) if bf16 else (self.v, self.layout_code)
        else:
            k_mean = ops.mean_seq(self.k, self.layout_code) if w["smooth_k"] else self.empty_mean
            if bf16:
                q8, qs, k8, ks, v16 = ops.prep_qkv(self.q, self.k, self.v, k_mean, self.layout_code, self.sm_scale)
                vl = 1
            else:
                q8, qs, k8, ks = ops.quant_qk_int8(self.q, self.k, k_mean, self.layout_code, self.sm_scale)
                v16, vl = self.v, self.layout_code
        if record:
            e0 = self._ev()
            self.prep_events.append((p0, e0))
        ops.qk_int8_sv_f16_attn(q8, k8, v16, o, qs, ks, self.layout_code, int(w["causal"]), self.sm_scale,
                                value_layout=vl, status=self.status, peer_ptrs=peers)
        if record:
            self.attn_events.append((e0, self._ev()))
        return o

    def step_public(self):
        """The same step through the public call."""
        from sageattention_rdna3_b200 import sageattn
        w = self.w
        return sageattn(self.q, self.k, self.v, tensor_layout=w["layout"], is_causal=w["causal"],
                        smooth_k=w["smooth_k"], kernel="int8")

    def kernel_ms(self):
        avg = lambda evs: sum(a.elapsed_time(b) for a, b in evs) / max(len(evs), 1)
        return avg(self.attn_events), avg(self.prep_events)

    def hbm_bytes(self):
        """Algorithmic bytes of the preparation launch on this rank (with smooth_k it includes the mean)."""
        w, e = self.w, self.q.element_size()
        nq, nk = self.q.numel(), self.k.numel()
        n_scales = self.Bl * self.Hql * ((w["S"] + 31) // 32) + self.Bl * self.Hkvl * ((w["S"] + 15) // 16)
        prep = nq * e + nk * e + nq + nk + 4 * n_scales + (nk * (e + 2) if self.q.dtype == torch.bfloat16 else 0)
        if w["smooth_k"]:
            prep += self.Bl * self.Hkvl * w["D"] * e
        return prep


def timed(fn, steps, barrier):
    """ms per call of ``fn`` over ``steps`` calls: CUDA events on the launching stream, a barrier and
    a device synchronize on both sides."""
    barrier()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for i in range(steps):
        fn(i)
    t1.record()
    barrier()
    return t0.elapsed_time(t1) / steps


def measure_gather(prob, steps, warmup, barrier, world, dist, sizes):
    """The optional final all-gather of the outputs (NCCL over NVLink), two ways: serial (each step
    computes, then gathers, on one stream) and overlapped (the gather of step i runs on a side
    stream while step i+1 computes into the other of two output buffers).  Returns ms per step of
    both, the gather alone, and the bytes every rank receives."""
    dev, w = prob.dev, prob.w
    n_max = max(sizes)
    padded = len(set(sizes)) > 1
    unit_shape = tuple(prob.o.shape[1:])
    outs = [torch.empty((n_max,) + unit_shape, dtype=prob.o.dtype, device=dev) for _ in range(2)]
    fulls = [torch.empty((world * n_max,) + unit_shape, dtype=prob.o.dtype, device=dev) for _ in range(2)]
    views = [o[:prob.units] if prob.units > 0 else o[:0] for o in outs]

    def finish(full):
        # NHD: a rank's units are [n, S, heads, D] slabs; the caller's [B, S, H, D] needs one local permute
        if w["layout"] == "NHD":
            return full.permute(1, 0, 2, 3).contiguous()
        return full

    def serial(i):
        if prob.units > 0:
            prob.step_ops(o=views[0])
        dist.all_gather_into_tensor(fulls[0], outs[0])
        finish(fulls[0])

    side = torch.cuda.Stream(device=dev)
    gathered = [None, None]

    def overlapped(i):
        b = i & 1
        cur = torch.cuda.current_stream(dev)
        if gathered[b] is not None:
            cur.wait_event(gathered[b])           # the gather of step i-2 has read this buffer
        if prob.units > 0:
            prob.step_ops(o=views[b])
        computed = torch.cuda.Event()
        computed.record(cur)
        with torch.cuda.stream(side):
            side.wait_event(computed)
            dist.all_gather_into_tensor(fulls[b], outs[b])
            finish(fulls[b])
            e = torch.cuda.Event()
            e.record(side)
            gathered[b] = e

    def drain(_=None):
        torch.cuda.current_stream(dev).wait_stream(side)

    def alone(i):
        dist.all_gather_into_tensor(fulls[0], outs[0])
        finish(fulls[0])

    res = {}
    for key, fn in (("serial_ms", serial), ("gather_alone_ms", alone)):
        for i in range(warmup):
            fn(i)
        res[key] = timed(fn, steps, barrier)
    for i in range(warmup):
        overlapped(i)
    drain()

    def overlapped_all(i):
        overlapped(i)
        if i == steps - 1:
            drain()

    res["overlapped_ms"] = timed(overlapped_all, steps, barrier)

    elem = prob.o.element_size()
    per_unit = elem
    for d in unit_shape:
        per_unit *= d
    res["recv_bytes_per_rank"] = per_unit * (sum(sizes) - prob.units)
    res["padded"] = padded
    return res


def measure_fused_gather(prob, steps, warmup, barrier, dist, sizes):
    """The gather inside the attention launch: the epilogue writes every finished tile into all ranks'
    copies of the output (mapped peer memory, ordinary stores); a one-element all-reduce follows.
    Two sets of buffers, used alternately, so that no rank writes into a copy that another rank may
    still be reading from the step before.  Returns ms per step, or a string that says why the
    buffers could not be set up (the same on every rank)."""
    from sageattention_rdna3_b200.peer_gather import PeerOutput
    dev, w = prob.dev, prob.w
    unit_shape = tuple(prob.o.shape[1:])
    try:
        peer_sets = [PeerOutput(sizes, unit_shape, prob.o.dtype, dev) for _ in range(2)]
    except RuntimeError as e:
        return str(e)

    def fused(i):
        po = peer_sets[i & 1]
        if prob.units > 0:
            prob.step_ops(o=po.local_slab(), peers=po.scatter_addresses())
        po.sync()
        if w["layout"] == "NHD":
            po.full.permute(1, 0, 2, 3).contiguous()

    for i in range(warmup):
        fused(i)
    ms = timed(fused, steps, barrier)
    for po in peer_sets:
        po.close()
    return ms


def measure_e2e(prob, steps, barrier):
    """End to end through ``sageattn_host()``: pinned host q, k, v in, pinned host output back, every
    step.  Also times the bare copies of the same bytes (host->device on one stream, device->host on
    another, no compute): the floor this box's host link puts under the call."""
    from sageattention_rdna3_b200 import sageattn_host
    w, dev = prob.w, prob.dev
    qp, kp, vp = (t.pin_memory() for t in prob.host)
    o_host = torch.empty(qp.shape, dtype=qp.dtype).pin_memory()
    layout = w["layout"]

    def step(_):
        sageattn_host(qp, kp, vp, out=o_host, tensor_layout=layout, is_causal=w["causal"], smooth_k=w["smooth_k"],
                      device=dev, kernel="int8")

    for i in range(3):
        step(i)
    ms = timed(step, steps, barrier)

    s_in, s_out = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
    qd, kd, vd = (torch.empty_like(t, device=dev) for t in (qp, kp, vp))

    def copies(_):
        cur = torch.cuda.current_stream(dev)
        s_in.wait_stream(cur)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_in):
            qd.copy_(qp, non_blocking=True)
            kd.copy_(kp, non_blocking=True)
            vd.copy_(vp, non_blocking=True)
        with torch.cuda.stream(s_out):
            o_host.copy_(prob.o, non_blocking=True)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)

    for i in range(2):
        copies(i)
    floor = timed(copies, steps, barrier)
    h2d = sum(t.numel() * t.element_size() for t in (qp, kp, vp))
    d2h = o_host.numel() * o_host.element_size()
    return {"ms": ms, "copy_floor_ms": floor, "h2d": h2d, "d2h": d2h}


def roofline_records(prob, attn_ms, prep_ms, peaks, capped):
    """Roofline objects of the three kernels from their event-timed launches on this rank."""
    w = prob.w
    # Half of the executed operations are int8 (QK^T, taken as 2x the bf16 rate), half fp16 (PV):
    # time = F/2/(2P) + F/2/P, a blended peak of P/0.75 with P the measured cuBLAS bf16 rate.  The
    # fraction is quoted on the burst figure (an event-timed kernel); the sustained one is beside it.
    peak_burst = peaks["bf16_tflops"] / 0.75
    peak_sustained = peaks["bf16_tflops_sustained"] / 0.75
    achieved = (prob.executed / (attn_ms / 1e3)) / 1e12
    total_units = w["B"] * w["Hkv"]
    traffic = ATTN_TRAFFIC_BYTES.get(prob.name)
    if traffic is not None:
        traffic = traffic * prob.units / total_units      # DRAM bytes grow in proportion to the units
    out = {"roofline": {
        "bound": "tensor", "kernel": "sage_attn_kernel", "achieved": achieved, "peak": peak_burst, "unit": "TFLOP/s",
        "frac": achieved / peak_burst, "traffic": traffic, "ms_per_launch": attn_ms,
        "frac_of_sustained_peak": achieved / peak_sustained, "power_capped_during_run": capped,
        "peak_source": f"{peaks['source']}: cuBLAS bf16 {peaks['bf16_tflops']} TFLOP/s (burst), int8 taken as 2x; "
                       "executed flops, half int8 half fp16"}}
    prep_bytes = prob.hbm_bytes()
    kernel = "sage_prep_kernel" if not w["smooth_k"] else \
        ("sage_prep_smooth_kernel" if prob.fused_prep else "sage_kmean_kernel + sage_prep_kernel (K is read twice)")
    out["roofline_prep"] = {"bound": "hbm", "kernel": kernel,
                            "achieved": prep_bytes / (prep_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                            "frac": prep_bytes / (prep_ms / 1e3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": prep_ms,
                            "bytes": prep_bytes}
    return out


def run_extra_config(name, dev, ops, lib, peaks, steps=10, warmup=3):
    """One of the other benchmark configurations on one GPU: step time, TOPS and the attention
    kernel's roofline fraction, from the operator loop with events."""
    w = dict(WORKLOADS[name])
    prob = Problem(w, name, w["B"] * w["Hkv"], True, 0, dev, ops, lib)
    for _ in range(warmup):
        prob.step_ops()
    ms = timed(lambda i: prob.step_ops(record=True), steps, torch.cuda.synchronize)
    attn_ms, prep_ms = prob.kernel_ms()
    achieved = prob.executed / (attn_ms / 1e3) / 1e12
    return {"workload": workload_string(name, w), "ms_per_step": ms, "tops": prob.nominal / (ms / 1e3) / 1e12,
            "attn_ms": attn_ms, "prep_ms": prep_ms, "attn_executed_tflops": achieved,
            "attn_frac_of_burst_peak": achieved / (peaks["bf16_tflops"] / 0.75), "steps": steps}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="C3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scaling", default="strong", choices=["strong", "weak"],
                    help="N > 1: 'strong' shards the workload's (batch, kv-head) units over the ranks (default); "
                         "'weak' runs the whole workload on every rank (independent replicas)")
    ap.add_argument("--units", type=int, default=0,
                    help="N = 1 only: run this many (batch, kv-head) units of the workload instead of all of them - a "
                         "trimmed case for profiler captures, not a benchmark result")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-gather", action="store_true")
    ap.add_argument("--no-extra-configs", action="store_true")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    name = args.workload
    w = dict(WORKLOADS[name])

    if args.impl == "reference":
        run_reference(args, w, name, rank)
        return
    args.warmup = max(args.warmup, 3)

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (NVIDIA B200); there is no CPU path")
    cores_near_gpu = bind_near_gpu(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from sageattention_rdna3_b200 import _native, check_status
    from sageattention_rdna3_b200.shard import plan_shards
    ops = _native.load_ops()
    lib = _native.load_abi()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- this rank's share of the work: its own units only, generated here
    total_units = w["B"] * w["Hkv"]
    strong = args.scaling == "strong"
    sizes = [s.n_units for s in plan_shards(w["B"], w["Hq"], w["Hkv"], world)] if strong else [total_units] * world
    if args.units > 0 and world == 1:
        sizes = [min(args.units, total_units)]
    units = sizes[rank]
    prob = Problem(w, name, units, full=(units == total_units), seed_offset=100 * rank, dev=dev, ops=ops, lib=lib)

    sampler = ClockSampler(local_rank)
    gather = e2e = None
    with sampler:
        # (1) the step as its operators with events around every kernel: the rooflines
        for _ in range(args.warmup):
            prob.step_ops()
        ms_ops = timed(lambda i: prob.step_ops(record=True), args.steps, barrier)
        attn_ms, prep_ms = prob.kernel_ms()
        time.sleep(0.3)         # the phases are measured apart: a 1 kW part is power capped within ~100 ms of load
        # (2) the same step through the public call: this is `value`
        for _ in range(args.warmup):
            prob.step_public()
        ms_public = timed(lambda i: prob.step_public(), args.steps, barrier)
        time.sleep(0.3)
        # (3) with the final all-gather of the outputs
        if world > 1 and strong and not args.no_gather:
            gather = measure_gather(prob, args.steps, args.warmup, barrier, world, dist, sizes)
        # (4) end to end with host buffers
        if not args.no_e2e:
            e2e = measure_e2e(prob, max(3, min(args.steps, 20)), barrier)
    check_status(dev)

    def over_ranks(values, op):
        t = torch.tensor(values, dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=op)
        return [float(x) for x in t.tolist()]

    MAX, SUM = dist.ReduceOp.MAX, dist.ReduceOp.SUM
    g = gather or {}
    ms_public, ms_ops, attn_ms_max, ser_ms, ovl_ms, alone_ms, e2e_ms, floor_ms = over_ranks(
        [ms_public, ms_ops, attn_ms, g.get("serial_ms", 0.0), g.get("overlapped_ms", 0.0), g.get("gather_alone_ms", 0.0),
         e2e["ms"] if e2e else 0.0, e2e["copy_floor_ms"] if e2e else 0.0], MAX)
    total_nominal, total_executed, h2d_total, d2h_total = over_ranks(
        [prob.nominal, prob.executed, e2e["h2d"] if e2e else 0.0, e2e["d2h"] if e2e else 0.0], SUM)

    line = None
    if rank == 0:
        peaks = measured_peaks()
        clocks = sampler.summary()
        capped = "sw_power_cap" in clocks["reasons"]
        tops = lambda ms: total_nominal / (ms / 1e3) / 1e12
        in_bytes = 3 * prob.q.numel() * prob.q.element_size() if prob.units else 0
        line = {
            "metric": METRIC, "value": tops(ms_public), "unit": "TOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_public, "higher_is_better": True,
            "scaling": args.scaling if world > 1 else "strong", "vs_baseline": None, "dtype": DTYPE_NOTE,
            "data": "synthetic",
            "config": {"workload": workload_string(name, w) +
                       (f" (TRIMMED to {units} of {total_units} units)" if units != total_units and world == 1 else "")},
            "per_gpu": {"units": sizes, "shape": f"B={prob.Bl} Hq={prob.Hql} Hkv={prob.Hkvl}",
                        "l2": "inputs larger than L2, no flush" if in_bytes > 126e6 else "inputs fit in L2, no flush"},
            "timed_call": "sageattn(q, k, v, kernel='int8') on HBM-resident inputs, max over ranks",
            "executed_tops": total_executed / (ms_public / 1e3) / 1e12,
            "operator_loop": {"ms_per_step": ms_ops, "value": tops(ms_ops),
                              "note": "the same step as its two operators (preparation, attention) with events "
                                      "around each kernel; the rooflines come from it"},
            "gpu_launches": prob.launches_per_step * args.steps,
            "clocks": clocks,
        }
        line.update(roofline_records(prob, attn_ms, prep_ms, peaks, capped))
        if gather:
            recv = gather["recv_bytes_per_rank"]
            line["allgather"] = {
                "collective": "NCCL all_gather_into_tensor of O" + (" + local permute (NHD)" if w["layout"] == "NHD" else ""),
                "recv_bytes_per_rank": recv, "nvlink_floor_ms": recv / 770e9 * 1e3,
                "gather_alone_ms": alone_ms,
                "serial": {"ms_per_step": ser_ms, "value": tops(ser_ms)},
                "overlapped": {"ms_per_step": ovl_ms, "value": tops(ovl_ms),
                               "how": "gather of step i on a side stream while step i+1 computes (two output buffers)"},
            }
        if e2e:
            line["e2e"] = {"value": tops(e2e_ms), "unit": "TOPS", "h2d_bytes_per_step": int(h2d_total),
                           "d2h_bytes_per_step": int(d2h_total), "ms_per_step": e2e_ms, "copy_floor_ms": floor_ms,
                           "of_copy_floor": floor_ms / e2e_ms if e2e_ms > 0 else None,
                           "host_cores_bound_near_gpu": cores_near_gpu,
                           "call": "sageattn_host(): pinned host q, k, v in, pinned host output back, every step; "
                                   "copy_floor_ms = the same bytes copied with no compute, all ranks at once"}
        if world == 1 and not args.no_extra_configs:
            del prob
            torch.cuda.empty_cache()
            line["configs"] = {n: run_extra_config(n, dev, ops, lib, peaks) for n in ("C2", "C4", "C5") if n != name}
        if world == 1 and not args.no_cpu_baseline:
            c_tops, sample, threads = cpu_oracle_run(w, name, 2, 1)
            line["cpu_baseline"] = {"value": c_tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample}
    # (5) N > 1: the gather done by the attention kernel itself.  It comes after everything else is
    # measured and reduced, under a watchdog: it maps other processes' memory, and whatever happens in
    # it, the line above is printed.
    if gather is not None:
        finished = threading.Event()

        def watchdog():
            if not finished.wait(180.0):
                if rank == 0:
                    line["allgather"]["fused"] = {"unavailable": "did not finish within 180 s"}
                    print(json.dumps(line), flush=True)
                os._exit(0)

        threading.Thread(target=watchdog, daemon=True).start()
        try:
            fused = measure_fused_gather(prob, args.steps, args.warmup, barrier, dist, sizes)
        except Exception as e:          # noqa: BLE001 - reported in the line
            fused = f"{type(e).__name__}: {e}"
        ok = isinstance(fused, float)
        all_ok, worst = over_ranks([1.0 if ok else 0.0], dist.ReduceOp.MIN)[0], over_ranks([fused if ok else 0.0], MAX)[0]
        finished.set()
        if rank == 0:
            if all_ok > 0.5:
                line["allgather"]["fused"] = {
                    "ms_per_step": worst, "value": total_nominal / (worst / 1e3) / 1e12,
                    "how": "no gather collective: the attention kernel's epilogue writes every finished tile into all "
                           "ranks' copies of the output (mapped peer memory, ordinary stores over NVLink), then a "
                           "one-element all-reduce; one stream, two sets of buffers used alternately"}
            else:
                line["allgather"]["fused"] = {"unavailable": fused if not ok else "failed on another rank"}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
