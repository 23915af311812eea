"""Regenerates the golden fixtures in this folder from the CPU oracle:

    python tests/golden/make_golden.py

The reference project ships no golden vectors and cannot be built or imported without a ROCm GPU,
so these files pin the ORACLE (oracle/sage_oracle.py) against drift and give the GPU tests a
machine-independent target; they are not outputs of the reference itself.  Inputs are not stored:
every case regenerates them from its seeds with ``cases.make_case`` (CPU generator, so the bits are
the same everywhere).  Stored per case: int8 Q/K, fp32 scales, the K mean, a checksum of the int32
Q.K^T products, and the fp16/bf16 output (as raw 16-bit words).
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

from cases import CASES, make_case  # noqa: E402
from oracle import sage_oracle as so  # noqa: E402


def s_checksum(s_int: torch.Tensor) -> np.ndarray:
    """Position-weighted 64-bit checksum of the int32 score matrix."""
    s = s_int.to(torch.int64).flatten()
    w = (torch.arange(s.numel(), dtype=torch.int64) % 65521) + 1
    return np.array([int(s.sum()), int((s * w).sum()), int(s.abs().max())], dtype=np.int64)


def main():
    torch.set_num_threads(1)      # oracle results do not depend on this; keep the run reproducible
    for name, spec in CASES.items():
        q, k, v = make_case(spec)
        o, parts = so.sageattn_emulated(q, k, v, tensor_layout=spec["layout"], is_causal=spec["causal"],
                                        sm_scale=spec.get("sm_scale"), smooth_k=spec["smooth_k"], return_parts=True)
        s_int = so.qk_int32(parts["q_i8"], parts["k_i8"])
        out = {
            "q_i8": parts["q_i8"].numpy(), "k_i8": parts["k_i8"].numpy(),
            "q_scale": parts["q_scale"].numpy(), "k_scale": parts["k_scale"].numpy(),
            "s_checksum": s_checksum(s_int),
            "o_bits": o.contiguous().view(torch.int16).numpy(),
        }
        if parts["k_mean"] is not None:
            out["k_mean_bits"] = parts["k_mean"].contiguous().view(torch.int16).numpy()
        path = os.path.join(HERE, f"{name}.npz")
        np.savez_compressed(path, **out)
        print(f"{name}: {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
