"""tcgen05 forward kernel: parity with the CPU oracle on small cases and with
the generic CUDA-core kernel (same device, same inputs) on long sequences."""
import math

import numpy as np
import pytest
import torch

from oracle import dkernel_oracle as O
from helpers import assert_out_close, assert_lse_close, seeded_qkv

pytestmark = pytest.mark.gpu


def _module(Hq, max_seq, pk, **kw):
    from dkernel_b200 import LocalStrideSparseAttention
    pk = dict(pk)
    return LocalStrideSparseAttention.__wrapped__(Hq, max_seq, pk.pop("block_size"), pk.pop("local_blocks"),
                                                  pk.pop("vert_stride"), **pk, **kw)


def _wait_status_clean():
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0, "a device-side wait gave up"


CASES = [
    # B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pattern kwargs
    (1, 2, 2, 128, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    (2, 4, 4, 512, 512, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=4)),
    (1, 8, 2, 1024, 1024, torch.bfloat16, 2, dict(block_size=64, local_blocks=3, vert_stride=4, num_kv_heads=2)),
    (1, 2, 2, 200, 200, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    (1, 3, 3, 1028, 1028, torch.bfloat16, 1, dict(block_size=64, local_blocks=4, vert_stride=4)),
    (1, 4, 2, 15, 15, torch.float16, 2, dict(block_size=64, local_blocks=4, vert_stride=4, num_kv_heads=2)),
    (1, 2, 2, 256, 256, torch.bfloat16, 2, dict(block_size=64, local_blocks=1, vert_stride=3, causal=False)),
    (1, 2, 2, 256, 640, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=3)),
    (1, 6, 2, 448, 448, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=4, num_kv_heads=2)),
    (1, 4, 4, 512, 512, torch.bfloat16, 1, dict(block_size=64, local_blocks=8, vert_stride=1)),
    # coarser pattern blocks are refined to 64-token blocks for the tensor-core kernels
    (1, 4, 2, 1024, 1024, torch.bfloat16, 1, dict(block_size=128, local_blocks=2, vert_stride=3, num_kv_heads=2)),
    (2, 2, 2, 700, 700, torch.float16, 2, dict(block_size=128, local_blocks=1, vert_stride=2)),
]


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,dtype,seq_dim,pk", CASES)
def test_sm100_forward_vs_oracle(B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pk, D):
    causal = pk.get("causal", True)
    bs = pk["block_size"]
    shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
    q, k, v = seeded_qkv(20, shape(Hq, Sq), shape(Hkv, Sk), dtype)
    bm = O.block_mask(Hq, Sk, **pk)
    # q rows are tile rows of the pattern; with Sq < Sk the causal offset is Sk - Sq
    ref, ref_lse = O.block_sparse_attention(q, k, v, bm, bs, None, seq_dim=seq_dim, causal=causal)
    mod = _module(Hq, Sk, pk, seq_dim=seq_dim, impl="sm100")
    with torch.no_grad():
        out, lse = mod(q.cuda(), k.cuda(), v.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


@pytest.mark.parametrize("B,Hq,Hkv,S,pk", [
    (1, 8, 2, 4096, dict(block_size=64, local_blocks=16, vert_stride=8, num_kv_heads=2)),
    (1, 4, 4, 4096, dict(block_size=64, local_blocks=32, vert_stride=8)),
    (2, 2, 2, 8192, dict(block_size=64, local_blocks=4, vert_stride=16)),
    # several tiles per persistent CTA (1024 tiles for 296 CTAs)
    (4, 16, 16, 2048, dict(block_size=64, local_blocks=2, vert_stride=4)),
])
def test_sm100_matches_generic_on_long_sequences(B, Hq, Hkv, S, pk):
    q, k, v = seeded_qkv(1, (B, S, Hq, 128), (B, S, Hkv, 128), torch.bfloat16, device="cuda")
    fast = _module(Hq, S, pk, seq_dim=1, impl="sm100")
    slow = _module(Hq, S, pk, seq_dim=1, impl="generic")
    with torch.no_grad():
        o1, l1 = fast(q, k, v, return_lse=True)
        o2, l2 = slow(q, k, v, return_lse=True)
    _wait_status_clean()
    assert_out_close(o1, o2, max_abs=2e-2, mean_abs=1e-3)
    assert_lse_close(l1, l2)
    # deterministic: a second launch gives the same bits
    with torch.no_grad():
        o3 = fast(q, k, v)
    assert torch.equal(o1, o3)


def test_sm100_shared_pattern_pairs_heads_over_many_tiles():
    """One pattern for all heads + GQA: a tile is two q heads of a kv group (1536 tiles for 296
    persistent CTAs); checked against the generic kernel on the same device."""
    from dkernel_b200 import SparseAttention
    B, Hq, Hkv, S, bs = 3, 16, 4, 4096, 64
    pat = torch.from_numpy(O.block_mask(1, S, block_size=bs, local_blocks=3, vert_stride=8)).bool()
    q, k, v = seeded_qkv(3, (B, S, Hq, 128), (B, S, Hkv, 128), torch.bfloat16, device="cuda")
    fast = SparseAttention(bs, pat.cuda(), seq_dim=1, impl="sm100")
    slow = SparseAttention(bs, pat.cuda(), seq_dim=1, impl="generic")
    with torch.no_grad():
        o1, l1 = fast(q, k, v, return_lse=True)
        o2, l2 = slow(q, k, v, return_lse=True)
    _wait_status_clean()
    assert_out_close(o1, o2, max_abs=2e-2, mean_abs=1e-3)
    assert_lse_close(l1, l2)


@pytest.mark.parametrize("D", [128, 64])
def test_sm100_varlen_and_padded_routes(D):
    from dkernel_b200 import SparseAttention
    Hq, Hkv, bs, nb = 4, 4, 64, 16
    g = torch.Generator().manual_seed(0)
    pat = torch.rand(Hq, nb, nb, generator=g) < 0.3
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    lens = [512, 100, 333, 64, 1, 700]
    T = sum(lens)
    q, k, v = seeded_qkv(5, (T, Hq, D), (T, Hkv, D), torch.bfloat16)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    ref, ref_lse = O.varlen_attention(q.float(), k.float(), v.float(), cu, pat.numpy().astype(np.uint8), bs)
    with pytest.warns(UserWarning):
        mod = SparseAttention(bs, pat.cuda(), impl="sm100")
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), cu_seqlen_k=cu.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    # left-padded prefill, GQA (head-pair tiles)
    B, S, Hq, Hkv = 3, 512, 8, 2
    pk = dict(block_size=64, local_blocks=2, vert_stride=4, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(6, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    lens = torch.tensor([512, 77, 300])
    left = S - lens
    bm = O.block_mask(Hq, S, **pk)
    ref, ref_lse = O.padded_attention(q.float(), k.float(), v.float(), bm, 64, left_paddings=left, seq_dim=1)
    mod = _module(Hq, S, pk, seq_dim=1, impl="sm100")
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), left_paddings=left.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


def test_sm100_tile_counter_gives_the_same_bits(monkeypatch):
    """Tiles drawn from a counter (dynamic order, any CTA may take any tile) against the fixed
    assignment: outputs and LSE must agree bit for bit on the dense-grid, padded and packed routes,
    including tiles that attend nothing, and repeated launches must each start from a zeroed counter."""
    import dkernel_b200.ops as ops
    from dkernel_b200 import SparseAttention
    D = 128
    runs = {}
    for mode, threshold in (("fixed", 10 ** 12), ("counter", 0)):
        monkeypatch.setattr(ops, "_DYNAMIC_TILES_FROM", threshold)
        res = []
        # dense grid, more tiles than CTAs (2 * 8 * 32 = 512 tiles of 128 rows on 296 CTAs)
        B, S, Hq, Hkv = 2, 4096, 8, 2
        pk = dict(block_size=64, local_blocks=3, vert_stride=5, num_kv_heads=Hkv)
        q, k, v = seeded_qkv(31, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16)
        mod = _module(Hq, S, pk, seq_dim=1, impl="sm100")
        with torch.no_grad():
            for _ in range(3):
                res.append(mod(q.cuda(), k.cuda(), v.cuda(), return_lse=True))
            lens = torch.tensor([4096, 130])
            res.append(mod(q.cuda(), k.cuda(), v.cuda(), left_paddings=(S - lens).cuda(), return_lse=True))
        # packed batch with a user pattern whose first rows of some heads attend nothing
        Hq2, nb = 4, 16
        g = torch.Generator().manual_seed(3)
        pat = torch.rand(Hq2, nb, nb, generator=g) < 0.3
        pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
        pat[:, -1, -1] = True
        lens = [512, 100, 333, 64, 1, 700, 1024]
        cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
        q2, k2, v2 = seeded_qkv(32, (sum(lens), Hq2, D), (sum(lens), Hq2, D), torch.bfloat16)
        with pytest.warns(UserWarning):
            mod2 = SparseAttention(64, pat.cuda(), impl="sm100")
        with torch.no_grad():
            res.append(mod2(q2.cuda(), k2.cuda(), v2.cuda(), cu_seqlen_k=cu.cuda(), return_lse=True))
        torch.cuda.synchronize()
        _wait_status_clean()
        runs[mode] = res
    for (o1, l1), (o2, l2) in zip(runs["fixed"], runs["counter"]):
        assert torch.equal(o1, o2)
        assert torch.equal(torch.nan_to_num(l1, neginf=-1e30), torch.nan_to_num(l2, neginf=-1e30))
    # and the counter route against the oracle on the packed case
    ref, ref_lse = O.varlen_attention(q2.float(), k2.float(), v2.float(), cu, pat.numpy().astype(np.uint8), 64)
    assert_out_close(runs["counter"][-1][0], ref)
    assert_lse_close(runs["counter"][-1][1], ref_lse)


BWD_CASES = [
    # B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pattern kwargs
    (1, 2, 2, 128, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    (1, 2, 2, 512, 512, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=4)),
    (2, 4, 2, 320, 320, torch.bfloat16, 2, dict(block_size=64, local_blocks=2, vert_stride=3, num_kv_heads=2)),
    (1, 3, 3, 200, 200, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    (1, 2, 2, 256, 256, torch.bfloat16, 2, dict(block_size=64, local_blocks=1, vert_stride=3, causal=False)),
    (1, 2, 2, 256, 640, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=3)),
    (1, 6, 2, 448, 448, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=4, num_kv_heads=2)),
    (1, 8, 1, 192, 192, torch.bfloat16, 1, dict(block_size=64, local_blocks=1, vert_stride=2, num_kv_heads=1)),
    (1, 4, 2, 512, 512, torch.bfloat16, 1, dict(block_size=128, local_blocks=1, vert_stride=2, num_kv_heads=2)),
]


@pytest.mark.parametrize("route", ["ds_handover", "recompute"])
@pytest.mark.parametrize("D", [48, 96, 80])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,dtype,seq_dim,pk", [BWD_CASES[1], BWD_CASES[2], BWD_CASES[3], BWD_CASES[5]])
def test_sm100_backward_other_head_dims(B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pk, D, route, monkeypatch):
    """Head dims between the kernels' two widths (64, 128): the tensor maps carry the real head dim,
    the columns up to the width come back as zeros and only the real columns of dQ/dK/dV are stored."""
    test_sm100_backward_vs_oracle(B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pk, D, route, monkeypatch)


@pytest.mark.parametrize("route", ["ds_handover", "recompute"])
@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,dtype,seq_dim,pk", BWD_CASES)
def test_sm100_backward_vs_oracle(B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pk, D, route, monkeypatch):
    """Both routes of the tensor-core backward: dQ from the dS tiles the dK/dV kernel hands over
    (the default when the scratch is affordable) and dQ with S and dP recomputed."""
    from helpers import assert_grad_close
    import dkernel_b200.ops as ops
    if route == "recompute":
        monkeypatch.setattr(ops, "_DS_WS_MAX_BYTES", 0)
    causal = pk.get("causal", True)
    bs = pk["block_size"]
    shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
    q, k, v, do = seeded_qkv(21, shape(Hq, Sq), shape(Hkv, Sk), dtype, with_do=True)
    bm = O.block_mask(Hq, Sk, **pk)
    qf, kf, vf = (t.detach().clone().float().requires_grad_() for t in (q, k, v))
    # oracle: q tile rows of the pattern, causal offset Sk - Sq
    dense = torch.from_numpy(bm[:, :(Sq + bs - 1) // bs]).repeat_interleave(bs, 1).repeat_interleave(bs, 2)
    dense = dense[:, :Sq, :Sk].bool()
    if causal:
        dense = dense & (torch.arange(Sq)[:, None] + (Sk - Sq) >= torch.arange(Sk)[None, :])
    ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense[None].to(torch.uint8), None, seq_dim=seq_dim,
                                            return_lse=True)
    w = torch.randn(ref_lse.shape, generator=torch.Generator().manual_seed(2))
    ((ref * do.float()).sum() + (ref_lse * w).sum()).backward()
    mod = _module(Hq, Sk, pk, seq_dim=seq_dim, impl="sm100", bwd_impl="sm100")
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out, lse = mod(qg, kg, vg, return_lse=True)
    ((out.float() * do.cuda().float()).sum() + (lse * w.cuda()).sum()).backward()
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_grad_close(qg.grad, qf.grad, "dq")
    assert_grad_close(kg.grad, kf.grad, "dk")
    assert_grad_close(vg.grad, vf.grad, "dv")


@pytest.mark.parametrize("D", [128, 64])
@pytest.mark.parametrize("B,Hq,Hkv,S,pk", [
    (1, 4, 4, 2048, dict(block_size=64, local_blocks=8, vert_stride=8)),
    (1, 8, 2, 2048, dict(block_size=64, local_blocks=4, vert_stride=4, num_kv_heads=2)),
    (2, 2, 2, 4096, dict(block_size=64, local_blocks=32, vert_stride=8)),
])
def test_sm100_backward_matches_generic_on_long_sequences(B, Hq, Hkv, S, pk, D):
    from helpers import assert_grad_close
    q, k, v, do = seeded_qkv(3, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16, device="cuda", with_do=True)
    grads = {}
    for name in ("sm100", "generic"):
        mod = _module(Hq, S, pk, seq_dim=1, impl=name, bwd_impl=name)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        out = mod(qg, kg, vg)
        out.backward(do)
        grads[name] = (qg.grad, kg.grad, vg.grad)
    _wait_status_clean()
    for a, b_, n in zip(grads["sm100"], grads["generic"], ("dq", "dk", "dv")):
        assert_grad_close(a, b_, n, 2e-2)
    # atomics-free: a second run reproduces the same bits
    mod = _module(Hq, S, pk, seq_dim=1, impl="sm100", bwd_impl="sm100")
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    mod(qg, kg, vg).backward(do)
    for a, b_ in zip(grads["sm100"], (qg.grad, kg.grad, vg.grad)):
        assert torch.equal(a, b_)
    # the route that recomputes S and dP for dQ: dK and dV are the same bits, dQ agrees
    import dkernel_b200.ops as ops
    saved = ops._DS_WS_MAX_BYTES
    try:
        ops._DS_WS_MAX_BYTES = 0
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        mod(qg, kg, vg).backward(do)
    finally:
        ops._DS_WS_MAX_BYTES = saved
    _wait_status_clean()
    assert torch.equal(kg.grad, grads["sm100"][1]) and torch.equal(vg.grad, grads["sm100"][2])
    assert_grad_close(qg.grad, grads["sm100"][0], "dq (recompute route)", 2e-2)


def test_sm100_head_dim_64_matches_generic_over_many_tiles():
    """Head dim 64 on the tensor-core forward: several tiles per persistent CTA, GQA head pairs
    and per-head patterns (row pairs), against the CUDA-core kernel on the same device."""
    for Hq, Hkv, pk in ((16, 4, dict(block_size=64, local_blocks=4, vert_stride=4, num_kv_heads=4)),
                        (8, 8, dict(block_size=64, local_blocks=8, vert_stride=8))):
        B, S, D = 2, 4096, 64
        q, k, v = seeded_qkv(11, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16, device="cuda")
        fast = _module(Hq, S, pk, seq_dim=1, impl="sm100")
        slow = _module(Hq, S, pk, seq_dim=1, impl="generic")
        with torch.no_grad():
            o1, l1 = fast(q, k, v, return_lse=True)
            o2, l2 = slow(q, k, v, return_lse=True)
            o3 = fast(q, k, v)
        _wait_status_clean()
        assert_out_close(o1, o2, max_abs=2e-2, mean_abs=1e-3)
        assert_lse_close(l1, l2)
        assert torch.equal(o1, o3)


@pytest.mark.parametrize("D", [128, 64])
def test_sm100_padding_may_hold_nan_or_inf(D):
    """Whatever sits in the padding of K/V (a torch.empty cache, NaN, Inf) must not reach the
    output: right padding (seqlens), left + right padding, and the tail behind a packed batch
    whose last block crosses the end of the buffer's last sequence."""
    from dkernel_b200 import SparseAttention
    B, S, Hq, Hkv, bs = 3, 512, 4, 2, 64
    pk = dict(block_size=bs, local_blocks=2, vert_stride=4, num_kv_heads=Hkv)
    bm = O.block_mask(Hq, S, **pk)
    mod = _module(Hq, S, pk, seq_dim=1, impl="sm100")
    q, k, v = seeded_qkv(31, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    for left, lens in ((torch.tensor([0, 0, 0]), torch.tensor([500, 77, 301])),
                       (torch.tensor([5, 100, 64]), torch.tensor([480, 33, 300]))):
        kk, vv, qq = k.clone(), v.clone(), q.clone()
        for b in range(B):
            lo, hi = int(left[b]), int(left[b] + lens[b])
            for t, bad in ((kk, float("nan")), (vv, float("inf")), (qq, float("nan"))):
                t[b, :lo] = bad
                t[b, hi:] = bad
        ref, ref_lse = O.padded_attention(q.float(), k.float(), v.float(), bm, bs, left_paddings=left,
                                          seqlens=lens, seq_dim=1)
        out, lse = mod(qq.cuda(), kk.cuda(), vv.cuda(), left_paddings=left.cuda(), seqlens=lens.cuda(),
                       return_lse=True)
        _wait_status_clean()
        assert torch.isfinite(out.float()).all()
        assert_out_close(out, ref)
        assert_lse_close(lse, ref_lse)
    # packed batch inside a larger buffer whose tail is NaN: the last sequence's last block crosses
    # the end of the real tokens
    lens = [130, 70, 257]
    T = sum(lens)
    H = 4
    nb = 8
    g = torch.Generator().manual_seed(3)
    pat = torch.rand(H, nb, nb, generator=g) < 0.4
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    q, k, v = seeded_qkv(32, (T, H, D), (T, H, D), torch.bfloat16)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    ref, ref_lse = O.varlen_attention(q.float(), k.float(), v.float(), cu, pat.numpy().astype(np.uint8), bs)
    big = [torch.full((T + 100, H, D), float("nan"), dtype=torch.bfloat16) for _ in range(3)]
    for dst, src in zip(big, (q, k, v)):
        dst[:T] = src
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        modv = SparseAttention(bs, pat.cuda(), impl="sm100")
    qg, kg, vg = (t.cuda()[:T] for t in big)
    out, lse = modv(qg, kg, vg, cu_seqlen_k=cu.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


@pytest.mark.parametrize("D", [48, 96, 160, 192, 256])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,dtype,seq_dim,pk", [CASES[1], CASES[2], CASES[4], CASES[7]])
def test_sm100_forward_other_head_dims(B, Hq, Hkv, Sq, Sk, dtype, seq_dim, pk, D):
    """The reference's head-dim matrix (tests/test_sparse_attn.py: 48 .. 256) on the tensor-core
    forward: a head narrower than the kernel's 64 / 128 / 256 columns is padded with zeros by the
    TMA loads and only its real columns are stored."""
    bs = pk["block_size"]
    shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
    q, k, v = seeded_qkv(23, shape(Hq, Sq), shape(Hkv, Sk), dtype)
    bm = O.block_mask(Hq, Sk, **pk)
    ref, ref_lse = O.block_sparse_attention(q, k, v, bm, bs, None, seq_dim=seq_dim, causal=pk.get("causal", True))
    mod = _module(Hq, Sk, pk, seq_dim=seq_dim, impl="sm100")
    with torch.no_grad():
        out, lse = mod(q.cuda(), k.cuda(), v.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


FINE_CASES = [
    # B, Hq, Hkv, Sq, Sk, D, dtype, seq_dim, pattern kwargs
    (1, 2, 2, 512, 512, 128, torch.bfloat16, 1, dict(block_size=16, local_blocks=4, vert_stride=4)),
    (2, 4, 2, 320, 320, 64, torch.float16, 2, dict(block_size=32, local_blocks=2, vert_stride=3, num_kv_heads=2)),
    (1, 3, 3, 1000, 1000, 128, torch.bfloat16, 1, dict(block_size=32, local_blocks=5, vert_stride=7)),
    (1, 2, 2, 256, 640, 96, torch.bfloat16, 1, dict(block_size=16, local_blocks=3, vert_stride=5)),
    (1, 2, 2, 256, 256, 128, torch.bfloat16, 2, dict(block_size=16, local_blocks=2, vert_stride=3, causal=False)),
    (1, 4, 4, 77, 77, 64, torch.float16, 1, dict(block_size=16, local_blocks=2, vert_stride=2)),
]


@pytest.mark.parametrize("bwd", ["sm100", "generic"])
@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,D,dtype,seq_dim,pk", FINE_CASES)
def test_sm100_forward_with_16_and_32_token_blocks(B, Hq, Hkv, Sq, Sk, D, dtype, seq_dim, pk, bwd):
    """Patterns with blocks finer than the kernel's 64-token tiles: the layout is coarsened to
    64 x 64 blocks on the host side and the kernels mask with one bit per sub-block; forward on the
    tensor cores (impl="sm100" would raise otherwise); backward on the tensor cores too (the dK/dV
    kernel applies the masks and hands masked dS tiles to the dQ kernel; bwd_impl="sm100" would raise
    otherwise), or on the CUDA-core kernels from the pattern's own layout."""
    from helpers import assert_grad_close
    from dkernel_b200 import _lib
    bs = pk["block_size"]
    causal = pk.get("causal", True)
    shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
    q, k, v, do = seeded_qkv(27, shape(Hq, Sq), shape(Hkv, Sk), dtype, with_do=True)
    bm = O.block_mask(Hq, Sk, **pk)
    qf, kf, vf = (t.detach().clone().float().requires_grad_() for t in (q, k, v))
    nq = (Sq + bs - 1) // bs
    dense = torch.from_numpy(bm[:, :nq]).repeat_interleave(bs, 1).repeat_interleave(bs, 2)[:, :Sq, :Sk].bool()
    if causal:
        dense = dense & (torch.arange(Sq)[:, None] + (Sk - Sq) >= torch.arange(Sk)[None, :])
    ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense[None].to(torch.uint8), None, seq_dim=seq_dim,
                                            return_lse=True)
    ref.backward(do.float())
    mod = _module(Hq, Sk, pk, seq_dim=seq_dim, impl="sm100", bwd_impl=bwd)
    assert mod._plan().for_kernels(q.cuda()).fine_block == bs
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out, lse = mod(qg, kg, vg, return_lse=True)
    out.backward(do.cuda())
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    assert_grad_close(qg.grad, qf.grad, "dq")
    assert_grad_close(kg.grad, kf.grad, "dk")
    assert_grad_close(vg.grad, vf.grad, "dv")


def test_sm100_fine_block_user_pattern_varlen_and_padded():
    """A Bernoulli pattern of 16-token blocks on the packed and padded routes of the tensor-core forward."""
    from dkernel_b200 import SparseAttention
    H, D, bs, nb = 4, 128, 16, 64
    g = torch.Generator().manual_seed(4)
    pat = torch.rand(H, nb, nb, generator=g) < 0.25
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        mod = SparseAttention(bs, pat.cuda(), impl="sm100")
    lens = [512, 100, 333, 64, 1, 700]
    T = sum(lens)
    q, k, v = seeded_qkv(5, (T, H, D), (T, H, D), torch.bfloat16)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    ref, ref_lse = O.varlen_attention(q.float(), k.float(), v.float(), cu, pat.numpy().astype(np.uint8), bs)
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), cu_seqlen_k=cu.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    B, S = 3, 1024
    q, k, v = seeded_qkv(6, (B, S, H, D), (B, S, H, D), torch.bfloat16)
    lens_t, left = torch.tensor([1000, 77, 300]), torch.tensor([24, 900, 0])
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        mod2 = SparseAttention(bs, pat.cuda(), seq_dim=1, impl="sm100")
    ref, ref_lse = O.padded_attention(q.float(), k.float(), v.float(), pat.numpy().astype(np.uint8), bs,
                                      left_paddings=left, seqlens=lens_t, seq_dim=1)
    out, lse = mod2(q.cuda(), k.cuda(), v.cuda(), left_paddings=left.cuda(), seqlens=lens_t.cuda(), return_lse=True)
    _wait_status_clean()
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


def test_sm100_random_sweep_against_cuda_core_kernels():
    """Seeded random sweep over shapes and patterns (head dims, GQA ratios, block sizes 16-128, odd
    lengths, Sq < Sk, causal or not, both layouts, both 16-bit types): forward, LSE and all three
    gradients of the tensor-core kernels against the CUDA-core kernels on the same inputs."""
    from helpers import assert_grad_close
    rng = np.random.default_rng(2024)
    ran = 0
    for trial in range(24):
        D = int(rng.choice([48, 64, 96, 128]))
        Hkv = int(rng.choice([1, 2, 3]))
        G = int(rng.choice([1, 2, 4]))
        Hq = Hkv * G
        bs = int(rng.choice([16, 32, 64, 128]))
        Sk = int(rng.integers(1, 1500))
        Sq = Sk if rng.random() < 0.7 else int(rng.integers(1, Sk + 1))
        causal = bool(rng.random() < 0.8)
        seq_dim = int(rng.choice([1, 2]))
        dtype = torch.bfloat16 if rng.random() < 0.6 else torch.float16
        B = int(rng.choice([1, 2]))
        pk = dict(block_size=bs, local_blocks=int(rng.integers(1, 6)), vert_stride=int(rng.integers(1, 7)),
                  num_kv_heads=Hkv, causal=causal)
        if Hkv == 1 and rng.random() < 0.5:
            pk["homo_head"] = True      # one pattern for all heads (the generator wants num_kv_heads = 1 with it)
        max_seq = (Sk + bs - 1) // bs * bs
        shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
        q, k, v, do = seeded_qkv(100 + trial, shape(Hq, Sq), shape(Hkv, Sk), dtype, device="cuda", with_do=True)
        res = {}
        for name in ("sm100", "generic"):
            mod = _module(Hq, max_seq, pk, seq_dim=seq_dim, impl=name, bwd_impl=name)
            qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
            out, lse = mod(qg, kg, vg, return_lse=True)
            out.backward(do)
            res[name] = (out, lse, qg.grad, kg.grad, vg.grad)
        _wait_status_clean()
        what = f"trial {trial}: D={D} Hq={Hq} Hkv={Hkv} bs={bs} Sq={Sq} Sk={Sk} causal={causal} seq_dim={seq_dim} {dtype}"
        a, b_ = res["sm100"], res["generic"]
        assert (a[0].float() - b_[0].float()).abs().max().item() <= 2e-2, what
        fin = torch.isfinite(b_[1])
        assert torch.equal(torch.isfinite(a[1]), fin), what
        assert (a[1][fin] - b_[1][fin]).abs().max().item() <= 1e-3 if fin.any() else True, what
        for x, y, n in zip(a[2:], b_[2:], ("dq", "dk", "dv")):
            assert_grad_close(x, y, f"{n} ({what})", 3e-2)
        ran += 1
    assert ran == 24
