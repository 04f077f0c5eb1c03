"""Parity at the full sizes of the benchmark configurations (the CPU oracle cannot finish
them), through properties that do not depend on the size, plus oracle checks on sampled rows.

* K = 0 makes every logit 0: LSE = log(number of attended keys) for every row, and with V equal
  to one vector per kv head the output is exactly that vector (a convex combination).
* A handful of (batch, head, row) samples are recomputed on the CPU in fp32 from the oracle's
  block mask.
* Config 3 (training) and config 5 (packed varlen): one (batch, head) pair, resp. two short
  sequences x two heads, are recomputed by the CPU oracle (masked-dense attention with autograd /
  per-sequence evaluator) at the full sequence length and compared with the tensor-core results;
  the tensor-core kernels are also compared with the CUDA-core kernels on the whole problem.
"""
import math

import numpy as np
import pytest
import torch

from oracle import dkernel_oracle as O
from helpers import GRAD_REL_NORM, assert_lse_close, assert_out_close

pytestmark = pytest.mark.gpu


def _module(Hq, max_seq, **kw):
    from dkernel_b200 import LocalStrideSparseAttention
    return LocalStrideSparseAttention.__wrapped__(Hq, max_seq, 64, **kw)


def _attended_key_counts(bm, S, bs):
    """(H, S) number of keys each query position attends (causal, square)."""
    nb = S // bs
    H = bm.shape[0]
    tri = np.tril(bm[:, :nb, :nb].astype(np.int64), -1)          # whole blocks below the diagonal
    full = tri.sum(-1) * bs                                      # (H, nb)
    diag = bm[:, np.arange(nb), np.arange(nb)].astype(np.int64)  # (H, nb)
    within = np.arange(bs)[None, None, :] + 1                    # keys of the diagonal block
    return (full[:, :, None] + diag[:, :, None] * within).reshape(H, S)


def _sampled_rows_oracle(q, k, v, bm, bs, samples, scale):
    """fp32 attention for sampled (b, h, i) rows from (B,S,H,D) tensors on the CPU."""
    G = q.size(2) // k.size(2)
    outs, lses = [], []
    for b, h, i in samples:
        row = bm[h, i // bs, : i // bs + 1]
        cols = np.nonzero(row)[0]
        pos = np.concatenate([np.arange(c * bs, min((c + 1) * bs, i + 1)) for c in cols])
        kk = k[b, pos, h // G].float().cpu()
        vv = v[b, pos, h // G].float().cpu()
        s = (kk @ q[b, i, h].float().cpu()) * scale
        lse = torch.logsumexp(s, 0)
        outs.append(torch.softmax(s, 0) @ vv)
        lses.append(lse)
    return torch.stack(outs), torch.stack(lses)


def test_config2_prefill_full_size():
    B, S, Hq, Hkv, D, bs = 4, 8192, 32, 8, 128, 64
    mod = _module(Hq, S, local_blocks=16, vert_stride=8, num_kv_heads=Hkv, seq_dim=1)
    bm = O.block_mask(Hq, S, block_size=bs, local_blocks=16, vert_stride=8, num_kv_heads=Hkv)
    scale = 1.0 / math.sqrt(D)
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((B, S, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    # property: K = 0, V = one vector per (batch, kv head)
    k0 = torch.zeros((B, S, Hkv, D), dtype=torch.bfloat16, device="cuda")
    vec = torch.randn((B, 1, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        out, lse = mod(q, k0, vec.expand(B, S, Hkv, D).contiguous(), sm_scale=scale, return_lse=True)
    want = vec.repeat_interleave(Hq // Hkv, dim=2).expand(B, S, Hq, D).float()
    assert (out.float() - want).abs().max().item() <= 1e-2
    counts = torch.from_numpy(_attended_key_counts(bm, S, bs)).float().log()      # (Hq, S)
    assert (lse.cpu() - counts[None]).abs().max().item() <= 1e-3
    # sampled rows against the fp32 oracle arithmetic
    k = torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        out, lse = mod(q, k, v, sm_scale=scale, return_lse=True)
    samples = [(0, 0, 0), (0, 5, 63), (1, 7, 64), (1, 12, 1000), (2, 19, 4095), (3, 31, 8191),
               (3, 16, 8128), (2, 3, 6200)]
    ref_o, ref_l = _sampled_rows_oracle(q, k, v, bm, bs, samples, scale)
    got_o = torch.stack([out[b, i, h].float().cpu() for b, h, i in samples])
    got_l = torch.stack([lse[b, h, i].cpu() for b, h, i in samples])
    assert_out_close(got_o, ref_o)
    assert_lse_close(got_l, ref_l)
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0


def test_config3_training_full_size_matches_cuda_core_kernels():
    B, S, H, D, bs = 2, 8192, 32, 128, 64
    kw = dict(local_blocks=32, vert_stride=8, seq_dim=1)
    fast = _module(H, S, impl="sm100", bwd_impl="sm100", **kw)
    slow = _module(H, S, impl="generic", bwd_impl="generic", **kw)
    g = torch.Generator(device="cuda").manual_seed(6)
    q, k, v, do = (torch.randn((B, S, H, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(4))
    grads = []
    for mod in (fast, slow):
        qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))
        out = mod(qq, kk, vv)
        out.backward(do)
        grads.append((out.detach(), qq.grad, kk.grad, vv.grad))
    assert_out_close(grads[0][0], grads[1][0], max_abs=2e-2, mean_abs=1e-3)
    for a, b_, name in zip(grads[0][1:], grads[1][1:], ("dq", "dk", "dv")):
        rel = (a.float() - b_.float()).norm() / b_.float().norm()
        assert rel.item() <= GRAD_REL_NORM, f"{name}: relative norm {rel.item():.3e}"
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0
    # One (batch, head) pair against the CPU oracle with autograd at the full length.  Here every
    # q head has its own kv head, so the pair's dK and dV depend on no other head.
    bm = O.block_mask(H, S, block_size=bs, local_blocks=32, vert_stride=8)
    for b, h in ((1, 13),):
        dense = O.token_mask(bm[h:h + 1], bs, S, S)
        qf, kf, vf = (t[b:b + 1, :, h:h + 1].float().cpu().requires_grad_() for t in (q, k, v))
        ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense, None, seq_dim=1, return_lse=True)
        ref.backward(do[b:b + 1, :, h:h + 1].float().cpu())
        out, dq, dk, dv = grads[0]
        assert_out_close(out[b:b + 1, :, h:h + 1], ref)
        for got, want, name in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
            g_ = got[b:b + 1, :, h:h + 1].float().cpu()
            rel = (g_ - want).norm() / want.norm()
            assert rel.item() <= GRAD_REL_NORM, f"{name} vs oracle: relative norm {rel.item():.3e}"
        with torch.no_grad():
            _, lse = fast(q[b:b + 1], k[b:b + 1], v[b:b + 1], return_lse=True)
        assert_lse_close(lse[:, h:h + 1], ref_lse.detach())


def test_config4_decode_full_size():
    B, S, Hq, Hkv, D, bs = 64, 8192, 32, 8, 128, 64
    mod = _module(Hq, S, local_blocks=16, vert_stride=8, num_kv_heads=Hkv, seq_dim=1)
    bm = O.block_mask(Hq, S, block_size=bs, local_blocks=16, vert_stride=8, num_kv_heads=Hkv)
    scale = 1.0 / math.sqrt(D)
    gc = torch.Generator().manual_seed(0)
    lens = torch.randint(1024, 8193, (B,), generator=gc)
    left = (S - lens).to(torch.int32).cuda()
    g = torch.Generator(device="cuda").manual_seed(7)
    q = torch.randn((B, 1, Hq, D), generator=g, device="cuda").to(torch.bfloat16)
    # property: K = 0 -> LSE = log(attended real tokens); V = one vector per (batch, kv head)
    k0 = torch.zeros((B, S, Hkv, D), dtype=torch.bfloat16, device="cuda")
    vec = torch.randn((B, 1, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        out, lse = mod(q, k0, vec.expand(B, S, Hkv, D).contiguous(), sm_scale=scale, left_paddings=left,
                       return_lse=True)
    want = vec.repeat_interleave(Hq // Hkv, dim=2).float()
    assert (out.float() - want).abs().max().item() <= 1e-2
    counts = torch.empty((B, Hq))
    for b, L in enumerate(lens.tolist()):
        row = (L - 1) // bs
        for h in range(Hq):
            cols = np.nonzero(bm[h, row, : row + 1])[0]
            counts[b, h] = float(np.minimum((cols + 1) * bs, L).sum() - (cols * bs).sum())
    assert (lse.reshape(B, Hq).cpu() - counts.log()).abs().max().item() <= 1e-3
    # four sequences against the oracle
    k = torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((B, S, Hkv, D), generator=g, device="cuda").to(torch.bfloat16)
    with torch.no_grad():
        out, lse = mod(q, k, v, sm_scale=scale, left_paddings=left, return_lse=True)
    idx = [0, 17, 40, 63]
    ref, ref_lse = O.decode_attention(q[idx].float().cpu(), k[idx].float().cpu(), v[idx].float().cpu(), bm, bs,
                                      sm_scale=scale, left_paddings=(S - lens)[idx])
    assert_out_close(out[idx], ref)
    assert_lse_close(lse[idx].reshape(len(idx), Hq, 1), ref_lse)
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0


def test_config5_varlen_full_size_matches_cuda_core_kernels():
    import warnings
    from dkernel_b200 import SparseAttention
    H, D, bs, nb = 32, 128, 64, 256
    gc = torch.Generator().manual_seed(0)
    pat = torch.rand((H, nb, nb), generator=gc) < 0.2
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    lens = torch.randint(512, 4097, (16,), generator=gc)
    T = int(lens.sum())
    cu = torch.cat([torch.zeros(1, dtype=torch.int64), lens.cumsum(0)]).to(torch.int32).cuda()
    g = torch.Generator(device="cuda").manual_seed(8)
    q, k, v = (torch.randn((T, H, D), generator=g, device="cuda").to(torch.bfloat16) for _ in range(3))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        fast = SparseAttention(bs, pat.cuda(), impl="sm100")
        slow = SparseAttention(bs, pat.cuda(), impl="generic")
    with torch.no_grad():
        o1, l1 = fast(q, k, v, cu_seqlen_k=cu, return_lse=True)
        o2 = slow(q, k, v, cu_seqlen_k=cu)
    assert_out_close(o1, o2, max_abs=2e-2, mean_abs=1e-3)
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0
    # the two shortest sequences x two heads against the CPU oracle's per-sequence evaluator
    cu_h = cu.cpu().tolist()
    heads = [3, 30]
    for sidx in torch.argsort(lens)[:2].tolist():
        a, b_ = cu_h[sidx], cu_h[sidx + 1]
        sub = lambda t: t[a:b_][:, heads].float().cpu()
        ref, ref_lse = O.varlen_attention(sub(q), sub(k), sub(v), [0, b_ - a], pat[heads].numpy(), bs)
        assert_out_close(o1[a:b_][:, heads], ref)
        assert_lse_close(l1[heads][:, a:b_], ref_lse)
