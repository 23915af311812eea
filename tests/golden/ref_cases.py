"""Seeded cases for the golden vectors made by the reference's own Triton back-end
(``make_ref_golden.py``).  kv lengths are above 512, so the reference takes its INT8 branch
(``sageattention/triton_backend.py:513-521``).  The cases share two autotune keys
(qo_len, kv_len, H, head_dim, kv groups; ``triton_backend.py:157-160``) to keep the generation short.
"""
import torch

DT = {"fp16": torch.float16, "bf16": torch.bfloat16}

REF_CASES = {
    # B=1 H=2 S=1024 D=64 fp16 HND non-causal: the CPU-runnable configuration of the benchmark list
    "c1_fp16_hnd": dict(B=1, Hq=2, Hkv=2, S=1024, D=64, dtype="fp16", layout="HND", causal=False, smooth_k=False,
                        k_offset=0.0),
    "d64_bf16_hnd_causal": dict(B=1, Hq=2, Hkv=2, S=1024, D=64, dtype="bf16", layout="HND", causal=True,
                                smooth_k=False, k_offset=0.0),
    "d64_fp16_nhd_smooth": dict(B=1, Hq=2, Hkv=2, S=1024, D=64, dtype="fp16", layout="NHD", causal=False,
                                smooth_k=True, k_offset=3.0),
    # ragged length (600 = 4 * 128 + 88), GQA 4:2, head_dim 128
    "d128_fp16_nhd_gqa_ragged": dict(B=1, Hq=4, Hkv=2, S=600, D=128, dtype="fp16", layout="NHD", causal=False,
                                     smooth_k=False, k_offset=0.0),
    "d128_bf16_hnd_gqa_causal_smooth": dict(B=1, Hq=4, Hkv=2, S=600, D=128, dtype="bf16", layout="HND", causal=True,
                                            smooth_k=True, k_offset=3.0),
}


def make_ref_case(spec):
    """q, k, v ~ N(0,1) from CPU generators seeded 10, 11, 12 (K gets ``k_offset`` added in fp32)."""
    B, Hq, Hkv, S, D = (spec[x] for x in ("B", "Hq", "Hkv", "S", "D"))
    dt = DT[spec["dtype"]]
    shape = (lambda h: (B, h, S, D)) if spec["layout"] == "HND" else (lambda h: (B, S, h, D))

    def rn(shp, seed):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(shp, generator=g, dtype=torch.float32)

    q = rn(shape(Hq), 10).to(dt)
    k = (rn(shape(Hkv), 11) + spec["k_offset"]).to(dt)
    v = rn(shape(Hkv), 12).to(dt)
    return q, k, v
