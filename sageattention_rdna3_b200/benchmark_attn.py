"""The reference's attention benchmark on a B200: same shapes, metric and protocol as
``benchmark_attn/benchmark_attn.py`` of LuXuxue/sageattention-rdna3, run as

    python -m sageattention_rdna3_b200.benchmark_attn [--markdown out.md] [--only SDXL01,Anima01]

Protocol (``benchmark_attn.py:84-131,210-221,271``): NHD layout, non-causal, q, k, v ~ N(0,1);
CUDA events, 10 warm-up + 50 timed iterations per round, round-robin over the implementations,
median over 3 rounds; TFLOPS = 4*b*h_q*sq*sk*d / t (``:40-47``); accuracy against fp32 attention,
OK iff max-err <= 0.05 (``:50-81,216,317``).

Columns: ``sageattn`` as a caller gets it (the kernel the dispatch picks), the INT8 path and the
un-quantised kernel forced, and torch's fp16 / bf16 ``scaled_dot_product_attention`` on the same
GPU for context.
"""
from __future__ import annotations

import argparse
import statistics
import sys

import torch
import torch.nn.functional as F

# name, b, h_q, h_kv, sq, sk, d, dtype: the shape list of benchmark_attn.py:141-186 (SDXL UNet and
# VAE attention in fp16, Anima DiT and VAE attention in bf16), plus the GQA pair it keeps commented out.
CASES = [
    ("SDXL01", 1, 10, 10, 4096, 4096, 64, "fp16"), ("SDXL02", 1, 10, 10, 4096, 77, 64, "fp16"),
    ("SDXL03", 1, 10, 10, 4096, 154, 64, "fp16"), ("SDXL04", 1, 20, 20, 1024, 1024, 64, "fp16"),
    ("SDXL05", 1, 20, 20, 1024, 77, 64, "fp16"), ("SDXL06", 1, 20, 20, 1024, 154, 64, "fp16"),
    ("SDXLVAE01", 1, 4, 4, 16384, 16384, 128, "fp16"), ("SDXL07", 1, 10, 10, 6144, 6144, 64, "fp16"),
    ("SDXL08", 1, 10, 10, 6144, 77, 64, "fp16"), ("SDXL09", 1, 10, 10, 6144, 154, 64, "fp16"),
    ("SDXL10", 1, 20, 20, 1536, 1536, 64, "fp16"), ("SDXL11", 1, 20, 20, 1536, 77, 64, "fp16"),
    ("SDXL12", 1, 20, 20, 1536, 154, 64, "fp16"), ("SDXLVAE02", 1, 4, 4, 24576, 24576, 128, "fp16"),
    ("SDXL13", 1, 10, 10, 9216, 9216, 64, "fp16"), ("SDXL14", 1, 10, 10, 9216, 77, 64, "fp16"),
    ("SDXL15", 1, 10, 10, 9216, 154, 64, "fp16"), ("SDXL16", 1, 20, 20, 2304, 2304, 64, "fp16"),
    ("SDXL17", 1, 20, 20, 2304, 77, 64, "fp16"), ("SDXL18", 1, 20, 20, 2304, 154, 64, "fp16"),
    ("Anima01", 1, 16, 16, 4096, 4096, 128, "bf16"), ("Anima02", 1, 16, 16, 4096, 512, 128, "bf16"),
    ("AnimaVAE01", 1, 3, 3, 16384, 16384, 128, "bf16"), ("Anima03", 1, 16, 16, 6144, 6144, 128, "bf16"),
    ("Anima04", 1, 16, 16, 6144, 512, 128, "bf16"), ("AnimaVAE02", 1, 3, 3, 24576, 24576, 128, "bf16"),
    ("Anima05", 1, 16, 16, 9216, 9216, 128, "bf16"), ("Anima06", 1, 16, 16, 9216, 512, 128, "bf16"),
    ("Krea01", 1, 48, 12, 4213, 4213, 128, "bf16"), ("Krea02", 1, 48, 12, 117, 117, 128, "bf16"),
]
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}
WARMUP, ITERS, ROUNDS = 10, 50, 3


def attention_fp32(q, k, v):
    """fp32 softmax(q k^T / sqrt(d)) v in NHD, one query head at a time (the scores of the largest
    case are 2.4 GB per head)."""
    B, Sq, Hq, D = q.shape
    rep = Hq // k.shape[2]
    out = torch.empty(B, Sq, Hq, D, dtype=torch.float32, device=q.device)
    for h in range(Hq):
        qh = q[:, :, h].float()
        kh, vh = k[:, :, h // rep].float(), v[:, :, h // rep].float()
        s = torch.matmul(qh, kh.transpose(1, 2)) * (D ** -0.5)
        out[:, :, h] = torch.matmul(torch.softmax(s, dim=-1), vh)
    return out


def time_round_robin(fns):
    """Median over ROUNDS of the mean time (ms) of ITERS back-to-back calls, implementations interleaved."""
    results = [[] for _ in fns]
    for fn in fns:
        for _ in range(WARMUP):
            fn()
    torch.cuda.synchronize()
    for _ in range(ROUNDS):
        for i, fn in enumerate(fns):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            for _ in range(ITERS):
                fn()
            end.record()
            torch.cuda.synchronize()
            results[i].append(start.elapsed_time(end) / ITERS)
    return [statistics.median(r) for r in results]


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--markdown", default=None, help="also write the table to this file")
    ap.add_argument("--only", default=None, help="comma-separated case names")
    args = ap.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("benchmark_attn needs a CUDA device (NVIDIA B200)")
    from . import check_status, sageattn
    from .core import use_direct_kernel
    dev = torch.device("cuda", torch.cuda.current_device())
    only = set(args.only.split(",")) if args.only else None

    header = ("| case | b h_q h_kv sq sk d dtype | kernel | sageattn ms | TFLOPS | INT8 path ms | un-quantised ms | "
              "torch SDPA ms | max-err | cos | |")
    lines = [header, "|---|---|---|---:|---:|---:|---:|---:|---:|---:|---|"]
    print(f"device: {torch.cuda.get_device_name(dev)}; layout NHD, non-causal; {WARMUP} warm-up + {ITERS} iterations, "
          f"median of {ROUNDS} rounds")
    print(header)
    for name, b, hq, hkv, sq, sk, d, dt in CASES:
        if only and name not in only:
            continue
        dtype = DTYPES[dt]
        g = torch.Generator(device="cpu").manual_seed(0)
        q = torch.randn(b, sq, hq, d, generator=g).to(dtype).to(dev)
        k = torch.randn(b, sk, hkv, d, generator=g).to(dtype).to(dev)
        v = torch.randn(b, sk, hkv, d, generator=g).to(dtype).to(dev)
        picked = "un-quantised" if use_direct_kernel(d, "NHD", False, sq, sk) else "INT8"
        o = sageattn(q, k, v, tensor_layout="NHD")
        check_status(dev)
        ref = attention_fp32(q, k, v)
        diff = (o.float() - ref).abs()
        max_err = float(diff.max())
        cos = float(F.cosine_similarity(o.float().flatten(), ref.flatten(), dim=0))
        del ref, diff
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)      # [B,H,S,D] views for torch

        def sdpa():
            return F.scaled_dot_product_attention(qt, kt, vt, enable_gqa=(hq != hkv))

        t_auto, t_int8, t_direct, t_sdpa = time_round_robin([
            lambda: sageattn(q, k, v, tensor_layout="NHD"),
            lambda: sageattn(q, k, v, tensor_layout="NHD", kernel="int8"),
            lambda: sageattn(q, k, v, tensor_layout="NHD", kernel="direct"),
            sdpa,
        ])
        tflops = 4.0 * b * hq * sq * sk * d / (t_auto * 1e-3) / 1e12
        row = (f"| {name} | {b} {hq} {hkv} {sq} {sk} {d} {dt} | {picked} | {t_auto:.4f} | {tflops:.1f} | {t_int8:.4f} | "
               f"{t_direct:.4f} | {t_sdpa:.4f} | {max_err:.6f} | {cos:.6f} | {'OK' if max_err <= 0.05 else 'FAIL'} |")
        print(row, flush=True)
        lines.append(row)
    if args.markdown:
        with open(args.markdown, "w") as f:
            f.write("\n".join(lines) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
