"""Seeded small cases shared by the golden-fixture generator and the tests."""
import torch

DT = {"fp16": torch.float16, "bf16": torch.bfloat16}

# B, Hq, Hkv, Sq, Skv, D, dtype, layout, causal, smooth_k, k_offset (DC offset added to K)
CASES = {
    "c1_small_fp16_hnd": dict(B=1, Hq=2, Hkv=2, Sq=128, Skv=128, D=64, dtype="fp16", layout="HND", causal=False,
                              smooth_k=False, k_offset=0.0),
    "ragged_bf16_nhd_causal_smooth": dict(B=1, Hq=2, Hkv=1, Sq=100, Skv=100, D=128, dtype="bf16", layout="NHD",
                                          causal=True, smooth_k=True, k_offset=3.0),
    "cross_fp16_hnd_scale": dict(B=1, Hq=2, Hkv=2, Sq=65, Skv=200, D=64, dtype="fp16", layout="HND", causal=False,
                                 smooth_k=False, k_offset=0.0, sm_scale=0.5),
    "gqa_bf16_hnd_causal": dict(B=1, Hq=4, Hkv=2, Sq=96, Skv=96, D=128, dtype="bf16", layout="HND", causal=True,
                                smooth_k=False, k_offset=0.0),
}


def make_case(spec, device="cpu"):
    """q, k, v ~ N(0,1) from CPU generators seeded 0, 1, 2 (K gets ``k_offset`` added in fp32)."""
    B, Hq, Hkv, Sq, Skv, D = (spec[x] for x in ("B", "Hq", "Hkv", "Sq", "Skv", "D"))
    dt = DT[spec["dtype"]]
    shape = (lambda h, s: (B, h, s, D)) if spec["layout"] == "HND" else (lambda h, s: (B, s, h, D))

    def rn(shp, seed):
        g = torch.Generator(device="cpu").manual_seed(seed)
        return torch.randn(shp, generator=g, dtype=torch.float32)

    q = rn(shape(Hq, Sq), 0).to(dt)
    k = (rn(shape(Hkv, Skv), 1) + spec["k_offset"]).to(dt)
    v = rn(shape(Hkv, Skv), 2).to(dt)
    return q.to(device), k.to(device), v.to(device)
