#!/usr/bin/env python
"""Benchmark of the INT8 SageAttention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload C3] [--impl reference]

One "step" is one pass of the hot path (K mean when smooth_k, Q/K quantisation + fp16 copy of V,
fused attention) over one batch of synthetic input of the named workload.  One JSON line is printed:

* ``value``     - attention TOPS, 4*B*Hq*Sq*Skv*D / t (benchmark_attn/benchmark_attn.py:40-47 of the
                  reference), inputs resident in HBM, aggregated over all ranks.
* ``e2e``       - the same metric through the public ``sageattn_host()`` call with HOST (pinned) q, k,
                  v and a host output: the host->device copies and the device->host copy of the
                  output are inside the timed region (pipelined over streams by that call).
* ``roofline``  - the fused attention kernel against the tensor-core roofline (executed flops).
* ``cpu_baseline`` - the CPU oracle (a port of the reference's arithmetic) on the host cores, on a
                  bounded sample of the same workload.
* ``--impl reference`` - times that CPU oracle only (the reference has no CPU or NVIDIA
                  implementation of its own); rank 0 alone runs it.
With N > 1 every rank runs the full workload on its own GPU (weak scaling: the global batch is
N times the workload's); ``--scaling strong`` shards the workload's (batch, kv-head) units instead.
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
    if rank != 0:
        return
    steps = max(1, min(args.steps, 3))
    warmup = 1 if args.warmup > 0 else 0
    tops, sample, threads = cpu_oracle_run(w, name, steps, warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": tops, "unit": "TOPS", "n_gpus": args.gpus,
        "steps": steps, "warmup": warmup, "ms_per_step": cpu_oracle_run.last_ms, "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None, "dtype": "int8 x int8 -> int32 (QK^T), fp16 x fp16 -> fp32 (PV)", "data": "synthetic",
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--workload", default="C3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--scaling", default="weak", choices=["weak", "strong"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    name = args.workload
    w = dict(WORKLOADS[name])

    if args.impl == "reference":
        run_reference(args, w, name, rank)
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (NVIDIA B200); there is no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    from sageattention_rdna3_b200 import _native, check_status, sageattn_host
    from sageattention_rdna3_b200.shard import plan_shards
    ops = _native.load_ops()

    # ---- this rank's share of the work
    if args.scaling == "strong" and world > 1:
        shard = plan_shards(w["B"], w["Hq"], w["Hkv"], world)[rank]
        local_units = shard.n_units
    else:
        local_units = w["B"] * w["Hkv"]
    rep = w["Hq"] // w["Hkv"]
    # A rank's units are laid out as a batch of single-kv-head problems: identical work and
    # memory traffic to a [B, H] slab, and it lets any number of units be expressed.
    if local_units == w["B"] * w["Hkv"]:
        q_h, k_h, v_h = make_inputs(w, name, seed_offset=100 * rank if args.scaling == "weak" else 0)
        Bl, Hql, Hkvl = w["B"], w["Hq"], w["Hkv"]
    else:
        q_h, k_h, v_h = make_inputs(w, name, seed_offset=100 * rank, heads=(rep, 1), batch=local_units)
        Bl, Hql, Hkvl = local_units, rep, 1
    local_nominal = 4.0 * Bl * Hql * w["S"] * w["S"] * w["D"]
    local_executed = local_nominal * (executed_ops(w) / nominal_ops(w))
    layout_code = 1 if w["layout"] == "HND" else 0
    sm_scale = w["D"] ** -0.5
    q, k, v = q_h.to(dev), k_h.to(dev), v_h.to(dev)
    o = torch.empty_like(q)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    empty_mean = torch.empty(0, device=dev, dtype=q.dtype)

    attn_events, prep_events, mean_events = [], [], []

    def ev():
        e = torch.cuda.Event(enable_timing=True)
        e.record()
        return e

    def step(record):
        m0 = ev() if record else None
        k_mean = ops.mean_seq(k, layout_code) if w["smooth_k"] else empty_mean
        p0 = ev() if record else None
        if q.dtype == torch.bfloat16:
            q8, qs, k8, ks, v16 = ops.prep_qkv(q, k, v, k_mean, layout_code, sm_scale)
            vl = 1
        else:
            q8, qs, k8, ks = ops.quant_qk_int8(q, k, k_mean, layout_code, sm_scale)
            v16, vl = v, layout_code
        if record:
            e0 = ev()
            mean_events.append((m0, p0))
            prep_events.append((p0, e0))
        ops.qk_int8_sv_f16_attn(q8, k8, v16, o, qs, ks, layout_code, vl, int(w["causal"]), sm_scale, None, status)
        if record:
            attn_events.append((e0, ev()))

    launches_per_step = 2 + (1 if w["smooth_k"] else 0)
    # a problem that fills the GPU unevenly runs on persistent CTAs and adds the merge kernel
    lib = _native.load_abi()
    if lib.sage_attn_workspace_bytes(Bl, Hql, w["S"], w["S"], w["D"], int(w["causal"])) > 0:
        launches_per_step += 1

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    sampler = ClockSampler(local_rank)
    with sampler:
        for _ in range(args.warmup):
            step(False)
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            step(True)
        t1.record()
        barrier()
        ms_total = t0.elapsed_time(t1)
        attn_ms = sum(a.elapsed_time(b) for a, b in attn_events) / len(attn_events)
        prep_ms = sum(a.elapsed_time(b) for a, b in prep_events) / len(prep_events)
        mean_ms = sum(a.elapsed_time(b) for a, b in mean_events) / len(mean_events)

        # ---- end to end through sageattn(): host (pinned) inputs in, host output back, every step
        e2e = None
        if not args.no_e2e:
            qp, kp, vp = q_h.pin_memory(), k_h.pin_memory(), v_h.pin_memory()
            o_host = torch.empty(q_h.shape, dtype=q_h.dtype).pin_memory()
            e2e_steps = max(3, min(args.steps, 20))

            def e2e_step():
                sageattn_host(qp, kp, vp, out=o_host, tensor_layout=w["layout"], is_causal=w["causal"],
                              smooth_k=w["smooth_k"], device=dev)

            for _ in range(3):
                e2e_step()
            barrier()
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            for _ in range(e2e_steps):
                e2e_step()
            s1.record()
            barrier()
            e2e_ms = s0.elapsed_time(s1) / e2e_steps
            e2e = (e2e_ms, q_h.numel() * q_h.element_size() + 2 * k_h.numel() * k_h.element_size(),
                   o_host.numel() * o_host.element_size())
    check_status(dev)

    ms_step = ms_total / args.steps
    stats = torch.tensor([ms_step, attn_ms, e2e[0] if e2e else 0.0], dtype=torch.float64, device=dev)
    units = torch.tensor([local_nominal, local_executed], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    ms_step, attn_ms_max, e2e_ms = (float(x) for x in stats.tolist())
    total_nominal, total_executed = (float(x) for x in units.tolist())

    if rank == 0:
        peaks = measured_peaks()
        clocks = sampler.summary()
        # Half of the executed operations are int8 (QK^T, taken as 2x the bf16 rate), half fp16
        # (PV): time = F/2/(2P) + F/2/P, i.e. a blended peak of P/0.75.  P is the measured cuBLAS
        # bf16 rate: the sustained (power-capped) figure when this run itself was power capped
        # (the kernel is timed inside a long back-to-back loop), the burst figure otherwise.
        capped = "sw_power_cap" in clocks["reasons"]
        peak_burst = peaks["bf16_tflops"] / 0.75
        peak_sustained = peaks["bf16_tflops_sustained"] / 0.75
        blended_peak = peak_sustained if capped else peak_burst
        achieved = (local_executed / (attn_ms / 1e3)) / 1e12
        # algorithmic bytes of the HBM-bound kernels on this rank
        e = q.element_size()
        nq, nk = q.numel(), k.numel()
        n_scales = Bl * Hql * ((w["S"] + 31) // 32) + Bl * Hkvl * ((w["S"] + 15) // 16)
        prep_bytes = nq * e + nk * e + nq + nk + 4 * n_scales + (nk * (e + 2) if q.dtype == torch.bfloat16 else 0)
        mean_bytes = nk * e + Bl * Hkvl * w["D"] * e
        line = {
            "metric": METRIC, "value": total_nominal / (ms_step / 1e3) / 1e12, "unit": "TOPS",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "int8 x int8 -> int32 (QK^T), fp16 x fp16 -> fp32 (PV), fp32 softmax", "data": "synthetic",
            "config": {"workload": workload_string(name, w), "per_gpu": f"B={Bl} Hq={Hql} Hkv={Hkvl}",
                       "l2": "inputs larger than L2, no flush" if q.numel() * 2 * 3 > 126e6 else "inputs fit in L2, no flush",
                       "executed_tops": total_executed / (ms_step / 1e3) / 1e12},
            "roofline": {"bound": "tensor", "kernel": "sage_attn_kernel", "achieved": achieved, "peak": blended_peak,
                         "unit": "TFLOP/s", "frac": achieved / blended_peak, "traffic": ATTN_TRAFFIC_BYTES.get(name),
                         "ms_per_launch": attn_ms,
                         "frac_of_burst_peak": achieved / peak_burst, "frac_of_sustained_peak": achieved / peak_sustained,
                         "peak_source": f"{peaks['source']}: cuBLAS bf16 {peaks['bf16_tflops_sustained'] if capped else peaks['bf16_tflops']} "
                                        f"TFLOP/s ({'sustained, this run was power capped' if capped else 'burst'}), "
                                        "int8 taken as 2x; executed flops, half int8 half fp16"},
            "roofline_prep": {"bound": "hbm", "kernel": "sage_prep_kernel", "achieved": prep_bytes / (prep_ms / 1e3) / 1e9,
                              "peak": peaks["hbm_gbs"], "unit": "GB/s",
                              "frac": prep_bytes / (prep_ms / 1e3) / 1e9 / peaks["hbm_gbs"], "ms_per_launch": prep_ms,
                              "bytes": prep_bytes},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if w["smooth_k"]:
            line["roofline_kmean"] = {"bound": "hbm", "kernel": "sage_kmean_kernel",
                                      "achieved": mean_bytes / (mean_ms / 1e3) / 1e9, "peak": peaks["hbm_gbs"],
                                      "unit": "GB/s", "frac": mean_bytes / (mean_ms / 1e3) / 1e9 / peaks["hbm_gbs"],
                                      "ms_per_launch": mean_ms, "bytes": mean_bytes}
        if e2e:
            line["e2e"] = {"value": total_nominal / (e2e_ms / 1e3) / 1e12, "unit": "TOPS",
                           "h2d_bytes_per_step": e2e[1], "d2h_bytes_per_step": e2e[2], "ms_per_step": e2e_ms}
        if not args.no_cpu_baseline and world == 1:
            tops, sample, threads = cpu_oracle_run(w, name, 2, 1)
            line["cpu_baseline"] = {"value": tops, "unit": "TOPS", "cores": threads, "kind": "port", "sample": sample}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
