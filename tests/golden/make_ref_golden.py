"""Golden vectors produced by the REFERENCE ITSELF: its Triton back-end
(``sageattention/triton_backend.py``: ``per_block_int8`` ``:248-298``, ``sageattn`` ``:488-530``)
run unmodified on an NVIDIA GPU, on seeded inputs.

    python oracle/make_ref.py                       # where the reference checkout is
    python tests/golden/make_ref_golden.py OUTDIR   # on a machine with a GPU and Triton

writes ``OUTDIR/ref_triton_<case>.npz``; the files committed next to this script were made that way
on a B200 (Triton 3.6, the reference's own autotune over its non-AMD configuration list).  Inputs
are not stored: ``ref_cases.make_ref_case`` regenerates them from CPU seeds.  Stored per case: the
reference's int8 Q / K and fp32 scales, the K mean it subtracted (torch ``k.mean``), and its
attention output as raw 16-bit words.

These files pin the CPU oracle and the CUDA kernels to outputs of the reference, not to a reading
of its source.  What may differ, and by how much, is stated in ``tests/test_reference_pin.py``.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from ref_cases import REF_CASES, make_ref_case  # noqa: E402
from oracle.make_ref import load_ref_triton  # noqa: E402


def main(outdir: str) -> None:
    os.makedirs(outdir, exist_ok=True)
    ref = load_ref_triton()
    dev = torch.device("cuda", 0)
    for name, spec in REF_CASES.items():
        q, k, v = (t.to(dev) for t in make_ref_case(spec))
        layout, smooth = spec["layout"], spec["smooth_k"]
        seq_dim = 1 if layout == "NHD" else 2
        sm_scale = spec.get("sm_scale") or spec["D"] ** -0.5
        km = k.mean(dim=seq_dim, keepdim=False) if smooth else None          # triton_backend.py:523-525
        q8, qs, k8, ks = ref.per_block_int8(q, k, km, BLKQ=128, BLKK=64, sm_scale=sm_scale, tensor_layout=layout)
        o = ref.sageattn(q, k, v, tensor_layout=layout, is_causal=spec["causal"], sm_scale=spec.get("sm_scale"),
                         smooth_k=smooth)
        torch.cuda.synchronize()
        out = {
            "q_i8": q8.cpu().numpy(), "k_i8": k8.cpu().numpy(),
            "q_scale": qs.squeeze(-1).cpu().numpy(), "k_scale": ks.squeeze(-1).cpu().numpy(),
            "o_bits": o.contiguous().view(torch.int16).cpu().numpy(),
        }
        if km is not None:
            out["k_mean_bits"] = km.contiguous().view(torch.int16).cpu().numpy()
        path = os.path.join(outdir, f"ref_triton_{name}.npz")
        np.savez_compressed(path, **out)
        print(f"{name}: {os.path.getsize(path)} bytes", flush=True)


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "_new"))
