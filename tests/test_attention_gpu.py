"""CUDA attention path (through the module API -> C ABI) vs the CPU oracle."""
import math

import numpy as np
import pytest
import torch

from oracle import dkernel_oracle as O
from helpers import (assert_out_close, assert_lse_close, assert_grad_close, seeded_qkv)

pytestmark = pytest.mark.gpu


def _mask(mod_kwargs, Hq, S):
    return O.block_mask(Hq, S, **mod_kwargs)


def _module(Hq, max_seq, pk, **kw):
    from dkernel_b200 import LocalStrideSparseAttention
    pk = dict(pk)
    bs = pk.pop("block_size")
    lb = pk.pop("local_blocks")
    vs = pk.pop("vert_stride")
    return LocalStrideSparseAttention.__wrapped__(Hq, max_seq, bs, lb, vs, **pk, **kw)


FWD_CASES = [
    # B, Hq, Hkv, Sq, Sk, D, dtype, seq_dim, pattern kwargs, impl
    (2, 4, 4, 256, 256, 64, torch.float32, 2, dict(block_size=64, local_blocks=2, vert_stride=2), "generic"),
    (1, 4, 2, 320, 320, 32, torch.float32, 1, dict(block_size=32, local_blocks=2, vert_stride=3, num_kv_heads=2), "generic"),
    (1, 2, 2, 200, 200, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=2), "generic"),
    (1, 2, 2, 256, 256, 64, torch.float32, 2, dict(block_size=64, local_blocks=1, vert_stride=3, causal=False), "generic"),
    (1, 3, 3, 15, 15, 64, torch.float16, 2, dict(block_size=64, local_blocks=4, vert_stride=4), "generic"),
    (1, 2, 2, 1028, 1028, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=4, vert_stride=4), "generic"),
    (1, 2, 2, 512, 512, 48, torch.float16, 2, dict(block_size=16, local_blocks=4, vert_stride=4), "generic"),
    (1, 2, 2, 512, 512, 160, torch.bfloat16, 2, dict(block_size=128, local_blocks=2, vert_stride=2), "generic"),
    (1, 2, 2, 384, 384, 256, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=3), "generic"),
    (2, 8, 2, 512, 512, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=4, num_kv_heads=2), "generic"),
    (1, 4, 4, 448, 448, 64, torch.bfloat16, 2, dict(block_size=64, local_blocks=2, vert_stride=4, num_dense_heads=1), "generic"),
    (1, 4, 4, 512, 512, 64, torch.float16, 1, dict(block_size=64, local_blocks=3, vert_stride=4, homo_head=True), "generic"),
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Sk,D,dtype,seq_dim,pk,impl", FWD_CASES)
def test_forward_and_backward_vs_oracle(B, Hq, Hkv, Sq, Sk, D, dtype, seq_dim, pk, impl):
    causal = pk.get("causal", True)
    bs = pk["block_size"]
    shape = (lambda h, s: (B, h, s, D)) if seq_dim == 2 else (lambda h, s: (B, s, h, D))
    q, k, v, do = seeded_qkv(20, shape(Hq, Sq), shape(Hkv, Sk), dtype, with_do=True)
    k = k[..., :]  # same generator stream: k and v share a shape
    bm = O.block_mask(Hq, Sk, **pk)
    scale = 1.0 / math.sqrt(D)
    # oracle in fp32 with autograd
    qf, kf, vf = (t.detach().clone().float().requires_grad_() for t in (q, k, v))
    dense = O.token_mask(bm, bs, Sq, Sk, causal=causal)
    ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense, scale, seq_dim=seq_dim, return_lse=True)
    ref.backward(do.float())

    mod = _module(Hq, Sk, pk, seq_dim=seq_dim, impl=impl)
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out, lse = mod(qg, kg, vg, sm_scale=scale, return_lse=True)
    assert out.shape == q.shape and out.dtype == dtype
    assert lse.shape == (B, Hq, Sq) and lse.dtype == torch.float32
    tight = dtype == torch.float32
    assert_out_close(out, ref, max_abs=2e-4 if tight else 2e-2, mean_abs=2e-5 if tight else 2e-3)
    assert_lse_close(lse, ref_lse, tol=1e-4 if tight else 1e-3)
    out.backward(do.cuda())
    tol = 1e-4 if tight else 5e-2
    assert_grad_close(qg.grad, qf.grad, "dq", tol)
    assert_grad_close(kg.grad, kf.grad, "dk", tol)
    assert_grad_close(vg.grad, vf.grad, "dv", tol)


def test_golden_fixture_forward():
    """Committed outputs of the reference's own oracle (tests/golden/attention.npz)."""
    from test_oracle import ATTN, ATTN_CASES, golden_attention_inputs
    for name, (B, Hq, Hkv, S, D, dt, seq_dim, pk) in ATTN_CASES.items():
        q, k, v, do = golden_attention_inputs(name)
        mod = _module(Hq, S, pk, seq_dim=seq_dim)
        qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
        out = mod(qg, kg, vg, sm_scale=0.0078125 * 8)
        out.backward(do.cuda())
        tight = dt == torch.float32
        assert_out_close(out, torch.from_numpy(ATTN[f"{name}/out"]), what=name,
                         max_abs=2e-4 if tight else 2e-2, mean_abs=2e-5 if tight else 2e-3)
        for g, key in ((qg.grad, "dq"), (kg.grad, "dk"), (vg.grad, "dv")):
            assert_grad_close(g, torch.from_numpy(ATTN[f"{name}/{key}"]), f"{name}/{key}",
                              1e-4 if tight else 5e-2)


def test_dlse_gradient_and_lse_only_loss():
    """Gradient flowing through the LSE output (used by KV-partition merging)."""
    B, H, S, D, bs = 1, 2, 192, 64, 64
    pk = dict(block_size=bs, local_blocks=2, vert_stride=2)
    q, k, v, do = seeded_qkv(3, (B, H, S, D), (B, H, S, D), torch.float32, with_do=True)
    bm = O.block_mask(H, S, **pk)
    dense = O.token_mask(bm, bs, S, S)
    w = torch.randn(B, H, S, generator=torch.Generator().manual_seed(5))
    qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
    ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense, None, seq_dim=2, return_lse=True)
    ((ref * do).sum() + (ref_lse * w).sum()).backward()
    mod = _module(H, S, pk, seq_dim=2)
    qg, kg, vg = (t.cuda().requires_grad_() for t in (q, k, v))
    out, lse = mod(qg, kg, vg, return_lse=True)
    ((out * do.cuda()).sum() + (lse * w.cuda()).sum()).backward()
    assert_grad_close(qg.grad, qf.grad, "dq", 1e-4)
    assert_grad_close(kg.grad, kf.grad, "dk", 1e-4)
    assert_grad_close(vg.grad, vf.grad, "dv", 1e-4)


def test_views_packing_and_out_kwarg():
    """Non-contiguous views (reference tests/test_sparse_attn.py:188-198) and packed
    qkv / kv gradients (:216-220)."""
    B, H, S, D, bs = 1, 2, 256, 64, 64
    pk = dict(block_size=bs, local_blocks=2, vert_stride=2)
    g = torch.Generator().manual_seed(7)
    big = [torch.randn(B, S + 37, H + 3, D, generator=g).to(torch.float16) for _ in range(3)]
    q, k, v = (t[:, :S, :H] for t in big)
    do = torch.randn(B, S, H, D, generator=g).to(torch.float16)
    bm = O.block_mask(H, S, **pk)
    dense = O.token_mask(bm, bs, S, S)
    qf, kf, vf = (t.detach().clone().float().requires_grad_() for t in (q, k, v))
    ref = O.masked_dense_attention(qf, kf, vf, dense, None, seq_dim=1)
    ref.backward(do.float())
    mod = _module(H, S, pk, seq_dim=1)
    bigg = [t.cuda() for t in big]
    qg, kg, vg = (t[:, :S, :H].requires_grad_() for t in bigg)
    out = mod(qg, kg, vg)
    assert_out_close(out, ref)
    # packed qkv along the head axis
    qkv = torch.cat([q, k, v], dim=2).cuda().requires_grad_()
    split = lambda x: x.chunk(3, dim=2)
    out2 = mod(qkv, split_qkv=split)
    assert_out_close(out2, ref)
    out2.backward(do.cuda())
    dq, dk, dv = split(qkv.grad)
    assert_grad_close(dq, qf.grad, "dq")
    assert_grad_close(dk, kf.grad, "dk")
    assert_grad_close(dv, vf.grad, "dv")
    # packed kv
    kv = torch.cat([k, v], dim=2).cuda().requires_grad_()
    q2 = q.cuda().requires_grad_()
    out3 = mod(q2, kv, split_qkv=lambda x: x.chunk(2, dim=2))
    out3.backward(do.cuda())
    assert_grad_close(q2.grad, qf.grad, "dq")
    assert_grad_close(kv.grad.chunk(2, dim=2)[0], kf.grad, "dk")
    # explicit output tensor, inference
    from dkernel_b200 import SparseAttention
    dst = torch.empty(B, S, H, D, dtype=torch.float16, device="cuda")
    mod2 = SparseAttention(bs, torch.from_numpy(bm).cuda(), seq_dim=1, out=dst)
    with torch.no_grad():
        r = mod2(q.cuda(), k.cuda(), v.cuda())
    assert r.data_ptr() == dst.data_ptr()
    assert_out_close(dst, ref)


def test_errors_are_python_exceptions():
    from dkernel_b200 import SparseAttention, LocalStrideSparseAttention
    pat = torch.ones(4, 4, dtype=torch.uint8, device="cuda").tril()
    with pytest.raises(AssertionError):
        SparseAttention(48, pat)                       # not a power of two
    with pytest.raises(AssertionError):
        SparseAttention(8, pat)                        # below 16
    with pytest.raises(AssertionError):
        LocalStrideSparseAttention.__wrapped__(4, 256, 64, 0, 4)   # no local block with stride > 1
    mod = SparseAttention(64, pat, seq_dim=1)
    q = torch.randn(1, 512, 2, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError):
        mod(q, q, q)                                   # longer than max_seqlen = 256
    mod3 = SparseAttention(64, torch.ones(3, 4, 4, dtype=torch.uint8, device="cuda").tril(), seq_dim=1)
    q = torch.randn(1, 128, 2, 64, device="cuda", dtype=torch.float16)
    with pytest.raises(AssertionError):
        mod3(q, q, q)                                  # 3 pattern heads vs 2 heads
    with pytest.raises(RuntimeError):
        mod(q.cpu(), q.cpu(), q.cpu())                 # no CPU path
    with pytest.raises(AssertionError):
        mod(q, q)                                      # packed kv without split_qkv
    # padded inputs have no backward
    qg = q.clone().requires_grad_()
    o = mod(qg, q, q, left_paddings=torch.tensor([3], device="cuda"))
    with pytest.raises(AssertionError):
        o.sum().backward()


def test_bounded_wait_gives_up_and_service_resumes():
    """A device-side wait whose barrier nothing ever arrives at (1 ms limit) must give up, record
    its code, make later launches no-ops, raise on the host without a sync, and be clearable."""
    import ctypes as C
    from dkernel_b200 import LocalStrideSparseAttention, _lib
    lib = _lib.lib()
    mod = LocalStrideSparseAttention.__wrapped__(2, 256, 64, 2, 2, seq_dim=1)
    q, k, v = seeded_qkv(40, (1, 256, 2, 128), (1, 256, 2, 128), torch.bfloat16, device="cuda")
    with torch.no_grad():
        good = mod(q, k, v)
    assert _lib.wait_status() == 0
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.bsa_selftest_wait_timeout(1000, stream) == 0
    torch.cuda.synchronize()
    # the mirror word already tells the host, and the next checked call raises
    assert C.c_int32.from_address(_lib._mirror_addr).value == 900
    with pytest.raises(_lib.BsaError, match="900"):
        with torch.no_grad():
            mod(q, k, v)
    assert _lib.wait_status(reset=False) == 900
    # kernels are no-ops while the status is set: the output buffer keeps its contents
    from dkernel_b200.ops import _fwd_params
    o = torch.full_like(q, 7.0)
    p = _fwd_params(q, k, v, o, None, 1, mod._plan(), 0.1, True, _lib.ROWS_BY_TILE)
    assert lib.bsa_fwd(C.byref(p), stream) == 0
    torch.cuda.synchronize()
    assert (o == 7.0).all()
    # clearing restores service
    assert _lib.wait_status() == 900
    assert _lib.wait_status() == 0
    assert C.c_int32.from_address(_lib._mirror_addr).value == 0
    with torch.no_grad():
        again = mod(q, k, v)
    assert torch.equal(good, again)
    assert _lib.wait_status() == 0
