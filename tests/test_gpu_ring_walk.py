"""The multi-rank paths walked on ONE GPU, rank by rank, with the real kernels: the ring of the
sequence-parallel path (attention with log-sum-exp + the fold kernel, contiguous and zig-zag shards)
and the unit slicing of the head-sharded path.  No process group: the same kernels, the same
schedule, the same fold as the distributed calls, with the exchange replaced by indexing."""
import os
import sys

import pytest
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import helpers as H  # noqa: E402
from oracle import sage_oracle as so  # noqa: E402

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from sageattention_rdna3_b200 import _native
    _native.load_ops()
    return torch.device("cuda", 0)


@pytest.mark.parametrize("dtype,layout,D", [(torch.float16, "HND", 128), (torch.bfloat16, "NHD", 64)])
def test_fold_kernel_matches_the_checker(dev, dtype, layout, D):
    """sage_fold_attn_partial (through the operator) against oracle.fold_partial: three folds, the
    second and third into a row slice of the accumulators, with rows that have seen no key."""
    from sageattention_rdna3_b200.context_parallel import fold_partial_cuda
    B, Hh, S = 2, 3, 200
    shp = (B, Hh, S, D) if layout == "HND" else (B, S, Hh, D)
    s_dim = 2 if layout == "HND" else 1
    g = torch.Generator(device="cpu").manual_seed(5)
    acc_o, acc_l = torch.full(shp, float("nan")), torch.full((B, Hh, S), float("nan"))
    dev_o, dev_l = acc_o.to(dev), acc_l.to(dev)
    for i, rows in enumerate((slice(0, S), slice(40, S), slice(40, 160))):
        n = rows.stop - rows.start
        pshape = list(shp)
        pshape[s_dim] = n
        o_j = torch.randn(pshape, generator=g).to(dtype)
        lse_j = torch.randn((B, Hh, n), generator=g) * 3.0
        lse_j[0, 0, : n // 4] = float("-inf")               # rows without visible keys in this partial ...
        if layout == "HND":                                 # ... for which the attention kernels write zeros
            o_j[0, 0, : n // 4] = 0
        else:
            o_j[0, : n // 4, 0] = 0
        sel = [slice(None)] * 4
        sel[s_dim] = rows
        so.fold_partial(acc_o[tuple(sel)], acc_l[:, :, rows], o_j, lse_j, layout, i == 0)
        fold_partial_cuda(dev_o[tuple(sel)], dev_l[:, :, rows], o_j.to(dev), lse_j.to(dev), layout, i == 0)
    torch.cuda.synchronize()
    assert torch.allclose(dev_o.cpu(), acc_o, atol=1e-5, rtol=1e-5, equal_nan=True)
    assert torch.allclose(dev_l.cpu(), acc_l, atol=1e-5, rtol=1e-6, equal_nan=True)


@pytest.mark.parametrize("world,zigzag,causal,layout,dtype", [
    (4, True, True, "HND", torch.bfloat16),
    (2, False, True, "NHD", torch.float16),
    (3, False, False, "HND", torch.float16),
])
def test_ring_walk_on_one_gpu(dev, world, zigzag, causal, layout, dtype):
    from sageattention_rdna3_b200 import check_status
    from sageattention_rdna3_b200.context_parallel import sageattn_context_parallel, zigzag_shard, zigzag_unshard
    B, Hq, Hkv, D = 1, 4, 2, 128
    S = 256 * world * (2 if zigzag else 1)
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    s_dim = 2 if layout == "HND" else 1
    q, k, v = H.randn(shp(Hq), 0, dtype), H.randn(shp(Hkv), 1, dtype, offset=0.5), H.randn(shp(Hkv), 2, dtype)
    cut = (lambda t, r: zigzag_shard(t, r, world, s_dim).contiguous()) if zigzag else \
        (lambda t, r: t.chunk(world, dim=s_dim)[r].contiguous())
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    shards = [(cut(kd, r), cut(vd, r)) for r in range(world)]
    outs = [sageattn_context_parallel(cut(qd, r), *shards[r], tensor_layout=layout, is_causal=causal, smooth_k=True,
                                      zigzag=zigzag, all_shards=shards, rank=r, kernel="int8") for r in range(world)]
    check_status(dev)
    got = (zigzag_unshard(outs, s_dim) if zigzag else torch.cat(outs, dim=s_dim)).cpu()
    assert torch.isfinite(got.float()).all()
    # every shard is quantised on its own: the bar is the accuracy of the INT8 path against fp32
    acc = so.accuracy(got.float(), so.sdpa_fp32(q, k, v, tensor_layout=layout, is_causal=causal))
    assert acc["cos"] > 0.9995 and acc["max_abs"] < 0.05, acc
    # and the whole sequence on one GPU gives the same to the same accuracy
    from sageattention_rdna3_b200 import sageattn
    whole = sageattn(qd, kd, vd, tensor_layout=layout, is_causal=causal, smooth_k=True, kernel="int8").cpu()
    acc2 = so.accuracy(got.float(), whole.float())
    assert acc2["cos"] > 0.9995, acc2


@pytest.mark.parametrize("layout,world", [("HND", 4), ("NHD", 3)])
def test_unit_slicing_walked_on_one_gpu_is_bit_identical(dev, layout, world):
    """Head sharding: every rank's units computed one after the other on this GPU and put back
    together equal the unsharded call bit for bit (units are independent problems)."""
    from sageattention_rdna3_b200 import check_status, sageattn
    from sageattention_rdna3_b200.shard import from_units, plan_shards, shard_inputs
    B, Hq, Hkv, S, D = 2, 8, 4, 1536, 128
    shp = (lambda h: (B, h, S, D)) if layout == "HND" else (lambda h: (B, S, h, D))
    q, k, v = (H.randn(shp(h), i, torch.bfloat16).to(dev) for i, h in enumerate((Hq, Hkv, Hkv)))
    kw = dict(is_causal=True, smooth_k=True, kernel="int8")
    H.set_streamk(0)                      # the same launch schedule for every slice and the whole
    try:
        whole = sageattn(q, k, v, tensor_layout=layout, **kw)
        parts = []
        for shard in plan_shards(B, Hq, Hkv, world):
            ql, kl, vl = shard_inputs(q, k, v, layout, shard)
            assert ql.size(0) == shard.n_units
            parts.append(sageattn(ql, kl, vl, tensor_layout="HND", **kw) if shard.n_units else ql.new_empty(ql.shape))
        check_status(dev)
    finally:
        H.set_streamk(-1)
    got = from_units(torch.cat(parts, dim=0), B, Hq, layout)
    assert torch.equal(got, whole)


@pytest.mark.parametrize("kernel", ["int8", "direct"])
@pytest.mark.parametrize("causal,dtype,S,D,n_copies", [(True, torch.bfloat16, 700, 128, 3), (False, torch.float16, 333, 64, 3),
                                                        (True, torch.bfloat16, 700, 128, 12)])
def test_scatter_entry_point_writes_every_copy(dev, causal, dtype, S, D, n_copies, kernel):
    """sage_qk_int8_sv_f16_attn_scatter / sage_direct_attn_scatter on one GPU: the further copies are ordinary local buffers here
    (on several GPUs they are mapped peer memory); each must equal the primary output bit for bit
    (sequence lengths that end inside a tile)."""
    from sageattention_rdna3_b200 import _native, check_status, sageattn
    B, Hq, Hkv = 2, 4, 2
    q = H.randn((B, Hq, S, D), 0, dtype).to(dev)
    k = H.randn((B, Hkv, S, D), 1, dtype, offset=0.5).to(dev)
    v = H.randn((B, Hkv, S, D), 2, dtype).to(dev)
    want = sageattn(q, k, v, is_causal=causal, smooth_k=True, kernel=kernel)
    out = torch.empty_like(q)
    # (with 12 copies the transfer is estimated to outlast the computation by a factor in the band in
    # which the launcher starts the causal items lightest first: the results do not depend on the order)
    dense = [torch.full_like(q, float("nan")) for _ in range(n_copies)]
    got = sageattn(q, k, v, is_causal=causal, smooth_k=True, kernel=kernel, out=out,
                   scatter_to=[d.data_ptr() for d in dense])
    check_status(dev)
    assert got.data_ptr() == out.data_ptr() and torch.equal(out, want)
    for i, d in enumerate(dense):
        assert torch.equal(d, want), f"copy {i}"
    lib = _native.load_abi()
    assert lib.sage_qk_int8_sv_f16_attn_scatter(None, None, None, None, 0, 0, 0, None, None, 1, 1, 1, 1, 1, 1, 64, 0, None,
                                                None, 16, None, None) != 0     # more peers than the kernel takes
