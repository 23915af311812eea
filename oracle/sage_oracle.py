"""CPU oracle for the INT8 SageAttention path of LuXuxue/sageattention-rdna3.

TEST INFRASTRUCTURE ONLY.  This module restates, in plain PyTorch on CPU tensors, the
arithmetic of the reference's native quantised-attention path.  It is the checker used by the
test-suite, by the smoke check and by the CPU-baseline leg of the benchmark.  It is never part of
the product path: the shipped ``sageattn`` runs CUDA kernels only and raises if they are missing.

Pin status.  The reference ships no golden vectors and neither of its back-ends can be built or
imported without a ROCm GPU (HIP-only sources, AMD inline assembly), so bit-level parity of the
int8 values / scales / int32 products is *unpinned in the reference*: it is defined by this
restatement of the reference source.  What the reference does pin, and what this oracle is checked
against, are its tolerance gates versus fp32 SDPA (``test_sageattn_rdna3.py:39-53,273-276``,
``benchmark_attn/benchmark_attn.py:216,317``) and its published accuracy figures
(cosine 0.99992-0.99993, max-err 0.0033 at B1 H10 S4096 D64 fp16;
``benchmark_attn/benchmark_attn-result-native.txt:4,64``).

Every function cites the reference lines it follows (paths are relative to the reference tree).
All fp32 arithmetic below is done as separate IEEE operations (torch CPU never contracts a
multiply and an add into an FMA), which is what "bit-exact" is defined against.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import numpy as np
import torch

# csrc/attn_gfx11.cu:34  constexpr float kLog2e = 1.4426950408889634f;
LOG2E_F32 = float(np.float32(1.4426950408889634))
# csrc/attn_gfx11.cu:46-47  scale granularity of Q and K
MIN_BLK_Q = 32
MIN_BLK_K = 16
# csrc/attn_gfx11.cu:499,628-631  mask value and initial running max
NEG_BIG = float(np.float32(-3.4028234663852886e38) * np.float32(0.5))
# csrc/attn_gfx11.cu:121-136  the mean kernel keeps one partial sum per thread, 256 threads
MEAN_LANES = 256


def to_hnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    """View a [B,S,H,D] (NHD) or [B,H,S,D] (HND) tensor as [B,H,S,D] (core.py:97,105-110)."""
    if tensor_layout == "HND":
        return x
    if tensor_layout == "NHD":
        return x.permute(0, 2, 1, 3)
    raise ValueError(f"unknown tensor_layout {tensor_layout!r}")


def sm_scale_log2e(sm_scale: float) -> torch.Tensor:
    """fp32 ``float(sm_scale) * kLog2e`` (csrc/attn_gfx11.cu:1995)."""
    return torch.tensor(sm_scale, dtype=torch.float32) * torch.tensor(LOG2E_F32, dtype=torch.float32)


def mean_seq(k_hnd: torch.Tensor) -> torch.Tensor:
    """Per-(b,h,d) mean of K over the sequence, in the reference's summation order.

    csrc/attn_gfx11.cu:94-145: thread ``t`` of 256 adds rows ``t, t+256, ...`` in fp32
    (``:121-127``); the 256 partials are then added serially from 0 to 255 (``:131-135``); the
    sum is divided by ``float(seq_len)`` and rounded to the input dtype (``:136-143``).
    Returns ``[B, H, D]`` in ``k_hnd.dtype``.
    """
    B, H, S, D = k_hnd.shape
    kf = k_hnd.to(torch.float32)
    n_iter = (S + MEAN_LANES - 1) // MEAN_LANES
    pad = n_iter * MEAN_LANES - S
    if pad:
        kf = torch.cat([kf, kf.new_zeros(B, H, pad, D)], dim=2)
    kf = kf.reshape(B, H, n_iter, MEAN_LANES, D)
    partial = torch.zeros(B, H, MEAN_LANES, D, dtype=torch.float32)
    for i in range(n_iter):          # rows t + 256*i, one fp32 add each
        partial = partial + kf[:, :, i]
    total = torch.zeros(B, H, D, dtype=torch.float32)
    for t in range(MEAN_LANES):      # serial sum of the 256 partials
        total = total + partial[:, :, t]
    mean = total / torch.tensor(float(S), dtype=torch.float32)
    return mean.to(k_hnd.dtype)


def _quant_groups(xf: torch.Tensor, group: int, s: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """Quantise fp32 ``xf [B,H,S,D]`` per ``group`` rows.  csrc/attn_gfx11.cu:85-92,189-318."""
    B, H, S, D = xf.shape
    n_groups = (S + group - 1) // group
    pad = n_groups * group - S
    # pass 1 (:189-237): amax over existing rows of fabsf(v * pass1_scale), floor 1e-7
    mag = (xf * s).abs()
    if pad:
        mag = torch.cat([mag, mag.new_zeros(B, H, pad, D)], dim=2)
    amax = mag.reshape(B, H, n_groups, group * D).amax(dim=-1)
    amax = torch.maximum(amax, torch.tensor(1e-7, dtype=torch.float32))
    scale = amax / torch.tensor(127.0, dtype=torch.float32)            # :244-245
    inv = torch.tensor(127.0, dtype=torch.float32) / amax              # :252
    iscale = inv * s                                                   # :296
    iscale_rows = iscale.repeat_interleave(group, dim=2)[:, :, :S]
    y = xf * iscale_rows[..., None]                                    # :297-312
    y = y + torch.where(y >= 0, 0.5, -0.5).to(torch.float32)           # :86
    q = torch.trunc(y).clamp_(-128, 127).to(torch.int8)                # :88-91 (convert toward zero, clamp)
    return q.contiguous(), scale.contiguous()


def quant_qk_int8(q_hnd: torch.Tensor, k_hnd: torch.Tensor, k_mean: Optional[torch.Tensor],
                  sm_scale: float):
    """Per-block INT8 quantisation of Q (32-row groups) and K (16-row groups).

    csrc/attn_gfx11.cu:1974-2067 (host) and :147-321 (device).  Q carries ``sm_scale*log2e``;
    K optionally has ``k_mean [B,Hkv,D]`` (input dtype) subtracted in fp32 first (:209-219).
    Returns ``q_i8 [B,Hq,Sq,D]``, ``q_scale [B,Hq,ceil(Sq/32)]``, ``k_i8``, ``k_scale``.
    """
    s = sm_scale_log2e(sm_scale)
    one = torch.tensor(1.0, dtype=torch.float32)
    q_i8, q_scale = _quant_groups(q_hnd.to(torch.float32), MIN_BLK_Q, s)
    kf = k_hnd.to(torch.float32)
    if k_mean is not None and k_mean.numel() > 0:
        kf = kf - k_mean.to(torch.float32)[:, :, None, :]
    k_i8, k_scale = _quant_groups(kf, MIN_BLK_K, one)
    return q_i8, q_scale, k_i8, k_scale


def v_to_f16(v_hnd: torch.Tensor) -> torch.Tensor:
    """V is always fp16 for P.V; bf16 is converted round-to-nearest (csrc/attn_gfx11.cu:377-381)."""
    return v_hnd.to(torch.float16)


def qk_int32(q_i8: torch.Tensor, k_i8: torch.Tensor) -> torch.Tensor:
    """Exact int32 ``Q_i8 . K_i8^T`` per (b, hq) with GQA mapping ``hkv = hq // (Hq/Hkv)``.

    csrc/attn_gfx11.cu:464,608-616.  Every partial sum is below 2**24 in magnitude
    (128 * 127 * 128 = 2 080 768), so an fp32 GEMM of the int8 values is exact.
    """
    B, Hq, Sq, D = q_i8.shape
    Hkv = k_i8.shape[1]
    rep = Hq // Hkv
    kf = k_i8.to(torch.float32).repeat_interleave(rep, dim=1)
    s = torch.matmul(q_i8.to(torch.float32), kf.transpose(-1, -2))
    return s.to(torch.int32)


def attention(q_i8: torch.Tensor, k_i8: torch.Tensor, v16_hnd: torch.Tensor,
              q_scale: torch.Tensor, k_scale: torch.Tensor, is_causal: bool,
              out_dtype: torch.dtype, block_n: int = 64, return_lse: bool = False):
    """Fused INT8 attention, blockwise online softmax in base 2.  Returns ``[B,Hq,Sq,D]``
    (and, with ``return_lse``, ``(m + log2 l) * ln 2`` per row, ``[B,Hq,Sq]`` fp32: the reference
    keeps m and l (:499-500) but does not write them out, sageattention/core.py:203-211).

    csrc/attn_gfx11.cu:487-502 (state), :608-633 (scores, masks), :657-689 (softmax),
    :699-713 with csrc/mma_gfx11.h:97-106 (P rounded to fp16, fp32 accumulate), :769-786 (epilogue).
    ``block_n`` is the KV tile of the reference's default D=128 kernel (:2260-2261); it only fixes
    the order of fp32 additions and the points at which P is rounded.
    """
    B, Hq, Sq, D = q_i8.shape
    Hkv, Skv = k_i8.shape[1], k_i8.shape[2]
    rep = Hq // Hkv
    S_int = qk_int32(q_i8, k_i8).to(torch.float32)                              # exact
    qs = q_scale.repeat_interleave(MIN_BLK_Q, dim=2)[:, :, :Sq]                 # row // 32
    ks = k_scale.repeat_interleave(MIN_BLK_K, dim=2)[:, :, :Skv]                # col // 16
    ks = ks.repeat_interleave(rep, dim=1)
    score_scale = qs[..., :, None] * ks[..., None, :]                           # :621
    s = S_int * score_scale                                                     # :627
    if is_causal:
        row = torch.arange(Sq)[:, None]
        col = torch.arange(Skv)[None, :]
        s = torch.where(col > row, torch.tensor(NEG_BIG), s)                    # :628-630
    vf = v16_hnd.to(torch.float16).to(torch.float32).repeat_interleave(rep, dim=1)
    return _online_softmax_pv(s, vf, out_dtype, block_n, return_lse)


def _online_softmax_pv(s: torch.Tensor, vf: torch.Tensor, out_dtype: torch.dtype, block_n: int, return_lse: bool):
    """Blockwise base-2 online softmax of masked fp32 scores ``s`` ``[B,Hq,Sq,Skv]`` and P.V with P
    rounded to fp16 (csrc/attn_gfx11.cu:499-500, :657-689, :699-713, :769-786; the un-quantised
    kernel does the same at :1552-1553, :1689-1745, :1790-1793)."""
    B, Hq, Sq, Skv = s.shape
    D = vf.shape[-1]
    m = torch.full((B, Hq, Sq), NEG_BIG, dtype=torch.float32)                   # :499
    l = torch.zeros(B, Hq, Sq, dtype=torch.float32)                             # :500
    acc = torch.zeros(B, Hq, Sq, D, dtype=torch.float32)
    for n0 in range(0, Skv, block_n):
        st = s[..., n0:n0 + block_n]
        gm = torch.maximum(m, st.amax(dim=-1))                                  # :657-666
        alpha = torch.where(l == 0, torch.zeros_like(l), torch.exp2(m - gm))    # :667
        m = gm
        l = l * alpha                                                           # :669
        acc = acc * alpha[..., None]                                            # :671
        p = torch.exp2(st - gm[..., None])                                      # :676
        l = l + p.sum(dim=-1)                                                   # :681-689 (un-rounded p)
        p16 = p.to(torch.float16).to(torch.float32)                             # mma_gfx11.h:102-103
        acc = acc + torch.matmul(p16, vf[..., n0:n0 + block_n, :])              # :711
    inv_l = torch.where(l > 0, 1.0 / l, torch.zeros_like(l))                    # :771
    o = (acc * inv_l[..., None]).to(out_dtype)                                  # :783-786
    if return_lse:
        lse = torch.where(l > 0, (m + torch.log2(l)) * math.log(2.0), torch.full_like(l, float("-inf")))
        return o, lse
    return o


def direct_attn_emulated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                         is_causal: bool = False, sm_scale: Optional[float] = None, block_n: int = 64,
                         return_lse: bool = False):
    """The reference's un-quantised branch (sageattention/core.py:141-163: v_transpose with the
    bf16 -> fp16 conversion, then fp16_attn_t / bf16_attn_t; kernel csrc/attn_gfx11.cu:1468-1846).

    Scores are fp32-accumulated products of the fp16 / bf16 inputs (:1662-1671), multiplied by
    ``fl32(sm_scale * log2e)`` in fp32 (:1679), masked with ``-FLT_MAX/2`` for ``col > row`` and
    ``col >= kv_len`` (:1680-1683); the rest is the same online softmax and fp16 P.V.  fp32 inputs
    are computed in fp16 (core.py:78-83).  The accumulation order of a dot product inside the matrix
    unit is not defined, so this path is compared by tolerance only.
    """
    in_dtype = q.dtype
    if in_dtype == torch.float32:
        q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
    D = q.shape[-1]
    if sm_scale is None:
        sm_scale = D ** -0.5
    qh, kh, vh = to_hnd(q, tensor_layout), to_hnd(k, tensor_layout), to_hnd(v, tensor_layout)
    rep = qh.shape[1] // kh.shape[1]
    Sq, Skv = qh.shape[2], kh.shape[2]
    c = (torch.tensor(float(sm_scale), dtype=torch.float32) * torch.tensor(LOG2E_F32, dtype=torch.float32))
    kf = kh.to(torch.float32).repeat_interleave(rep, dim=1)
    s = torch.matmul(qh.to(torch.float32), kf.transpose(-1, -2)) * c
    if is_causal:
        row = torch.arange(Sq)[:, None]
        col = torch.arange(Skv)[None, :]
        s = torch.where(col > row, torch.tensor(NEG_BIG), s)
    vf = v_to_f16(vh).to(torch.float32).repeat_interleave(rep, dim=1)
    out = _online_softmax_pv(s, vf, q.dtype, block_n, return_lse)
    o, lse = out if return_lse else (out, None)
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3).contiguous()
    if in_dtype == torch.float32:
        o = o.to(torch.float32)
    return (o, lse) if return_lse else o


def sageattn_emulated(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
                      is_causal: bool = False, sm_scale: Optional[float] = None,
                      smooth_k: bool = False, return_parts: bool = False, return_lse: bool = False):
    """End-to-end emulation of ``sageattn``'s INT8 branch (sageattention/core.py:40-213).

    fp32 inputs are computed in fp16 and returned in fp32 (core.py:78-83,200-201).  With
    ``return_lse`` the result is ``(o, lse)`` (or ``(o, lse, parts)``), lse ``[B,Hq,Sq]`` referring
    to the caller's keys: ``sm_scale * q . mean`` is added back when the mean was subtracted.
    """
    in_dtype = q.dtype
    if in_dtype == torch.float32:
        q, k, v = q.to(torch.float16), k.to(torch.float16), v.to(torch.float16)
    D = q.shape[-1]
    if sm_scale is None:
        sm_scale = D ** -0.5                                                    # core.py:65-66
    qh, kh, vh = to_hnd(q, tensor_layout), to_hnd(k, tensor_layout), to_hnd(v, tensor_layout)
    k_mean = mean_seq(kh) if smooth_k else None                                 # core.py:186-190
    q_i8, q_scale, k_i8, k_scale = quant_qk_int8(qh, kh, k_mean, sm_scale)
    o, lse = attention(q_i8, k_i8, v_to_f16(vh), q_scale, k_scale, is_causal, q.dtype, return_lse=True)
    if smooth_k:
        rep = qh.shape[1] // kh.shape[1]
        km = k_mean.to(torch.float32).repeat_interleave(rep, dim=1)
        lse = lse + torch.einsum("bhsd,bhd->bhs", qh.to(torch.float32), km) * sm_scale
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3).contiguous()
    if in_dtype == torch.float32:
        o = o.to(torch.float32)
    out = (o, lse) if return_lse else (o,)
    if return_parts:
        out = out + (dict(q_i8=q_i8, q_scale=q_scale, k_i8=k_i8, k_scale=k_scale, k_mean=k_mean),)
    return out if len(out) > 1 else out[0]


def sdpa_fp32(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, tensor_layout: str = "HND",
              is_causal: bool = False, sm_scale: Optional[float] = None, return_lse: bool = False):
    """The reference's own oracle: fp32 scaled-dot-product attention
    (test_sageattn_rdna3.py:20-24, benchmark_attn/benchmark_attn.py:50-66), with GQA heads
    repeated.  Causal masking is top-left aligned (``col > row``), as in the kernels.
    """
    qh, kh, vh = (to_hnd(t, tensor_layout).to(torch.float32) for t in (q, k, v))
    rep = qh.shape[1] // kh.shape[1]
    if rep > 1:
        kh, vh = kh.repeat_interleave(rep, dim=1), vh.repeat_interleave(rep, dim=1)
    if sm_scale is None:
        sm_scale = qh.shape[-1] ** -0.5
    s = torch.matmul(qh, kh.transpose(-1, -2)) * sm_scale
    if is_causal:
        Sq, Skv = qh.shape[2], kh.shape[2]
        mask = torch.arange(Skv)[None, :] > torch.arange(Sq)[:, None]
        s = s.masked_fill(mask, float("-inf"))
    o = torch.matmul(torch.softmax(s, dim=-1), vh)
    if tensor_layout == "NHD":
        o = o.permute(0, 2, 1, 3).contiguous()
    if return_lse:
        return o, torch.logsumexp(s, dim=-1)                                    # [B,Hq,Sq]
    return o


def fold_partial(o_acc: torch.Tensor, lse_acc: torch.Tensor, o_j: torch.Tensor, lse_j: torch.Tensor,
                 tensor_layout: str, first: bool) -> None:
    """Checker for the fold of partial attention results (sage_fold_attn_partial), in place on fp32
    accumulators: lse' = logaddexp(lse, lse_j); o' = o * exp(lse - lse') + o_j * exp(lse_j - lse').
    The reference has no counterpart; its ``return_lse`` is a placeholder (sageattention/core.py:203-211)."""
    o_j = o_j.float()
    if first:
        o_acc.copy_(o_j)
        lse_acc.copy_(lse_j)
        return
    new = torch.logaddexp(lse_acc, lse_j)
    # a row that has seen no key on either side has -inf twice: exp(nan) -> weight 0
    w_old = torch.nan_to_num(torch.exp(lse_acc - new), nan=0.0)
    w_new = torch.nan_to_num(torch.exp(lse_j - new), nan=0.0)
    if tensor_layout == "HND":
        w_old, w_new = w_old[..., None], w_new[..., None]                       # [B,H,S,1]
    else:
        w_old, w_new = w_old.transpose(1, 2)[..., None], w_new.transpose(1, 2)[..., None]   # [B,S,H,1]
    o_acc.copy_(o_acc * w_old + o_j * w_new)
    lse_acc.copy_(new)


def accuracy(a: torch.Tensor, b: torch.Tensor) -> dict:
    """Cosine similarity, relative L1, max-abs error (benchmark_attn/benchmark_attn.py:69-81)."""
    a64, b64 = a.detach().double().flatten().cpu(), b.detach().double().flatten().cpu()
    cos = float(torch.dot(a64, b64) / (a64.norm() * b64.norm()).clamp_min(1e-300))
    rel_l1 = float((a64 - b64).abs().sum() / b64.abs().sum().clamp_min(1e-300))
    return {"cos": cos, "rel_l1": rel_l1, "max_abs": float((a64 - b64).abs().max())}
