"""The CPU oracle against the golden vectors produced by the reference."""
import math

import numpy as np
import pytest
import torch

from oracle import dkernel_oracle as O
from helpers import GOLDEN, load_patterns, pattern_kwargs, seeded_qkv

P, META = load_patterns()
CASES = [n for n in META if not n.startswith("mod_") and n != "bernoulli"]


def test_reference_known_answer_masks():
    # the two literal matrices of the reference's tests/test_utils.py:24-34,55-64
    causal = np.array([[1, 0, 0, 0, 0, 0, 0, 0], [1, 1, 0, 0, 0, 0, 0, 0], [1, 1, 1, 0, 0, 0, 0, 0],
                       [1, 0, 1, 1, 0, 0, 0, 0], [1, 0, 0, 1, 1, 0, 0, 0], [1, 0, 0, 1, 1, 1, 0, 0],
                       [1, 0, 0, 1, 0, 1, 1, 0], [1, 0, 0, 1, 0, 0, 1, 1]], dtype=np.uint8)
    bidir = np.array([[1, 1, 0, 0, 1, 0, 0, 1], [1, 1, 1, 0, 0, 1, 0, 0], [0, 1, 1, 1, 0, 0, 1, 0],
                      [0, 0, 1, 1, 1, 0, 0, 1], [1, 0, 0, 1, 1, 1, 0, 0], [0, 1, 0, 0, 1, 1, 1, 0],
                      [0, 0, 1, 0, 0, 1, 1, 1], [1, 0, 0, 1, 0, 0, 1, 1]], dtype=np.uint8)
    kw = dict(num_heads=2, seqlen=16, block_size=2, local_blocks=2, vert_stride=3, homo_head=True)
    assert (O.block_mask(causal=True, **kw)[0] == causal).all()
    assert (O.block_mask(causal=False, **kw)[0] == bidir).all()
    assert (P["kat_causal/mask"][0] == causal).all() and (P["kat_bidir/mask"][0] == bidir).all()


@pytest.mark.parametrize("name", CASES)
def test_block_mask_and_layouts(name):
    bm = O.block_mask(**pattern_kwargs(META[name]))
    g = P[f"{name}/mask"]
    assert bm.shape == g.shape and (bm == g).all()
    crow, col = O.dense_to_crow_col(bm)
    ccol, row = O.dense_to_ccol_row(bm)
    for a, key in ((crow, "crow"), (col, "col"), (ccol, "ccol"), (row, "row")):
        ref = P[f"{name}/{key}"]
        assert a.dtype == ref.dtype == np.int32
        assert a.shape == ref.shape and (a == ref).all(), f"{name}/{key}"
    if META[name]["kv_cache_efficient"] is not None:
        bs = META[name]["block_size"]
        assert O.is_kv_cache_efficient(bm, bs, bs) == META[name]["kv_cache_efficient"]
    back = O.crow_col_to_dense(crow, col, n_cols=bm.shape[-1])
    assert (back == bm).all()


def test_bernoulli_pattern_layouts():
    bm = P["bernoulli/mask"]
    crow, col = O.dense_to_crow_col(bm)
    ccol, row = O.dense_to_ccol_row(bm)
    assert (crow == P["bernoulli/crow"]).all() and (col == P["bernoulli/col"]).all()
    assert (ccol == P["bernoulli/ccol"]).all() and (row == P["bernoulli/row"]).all()
    assert O.is_kv_cache_efficient(bm, 64, 64) == META["bernoulli"]["kv_cache_efficient"]


def test_merge_split_layouts():
    seen = 0
    for key in P.files:
        if "/ms_" in key and key.endswith("/crow"):
            name, ms, _ = key.split("/")
            _, bm_, bn_ = ms.split("_")
            crow, col = O.merge_split_fwd_kernel_blocks(META[name]["block_size"], P[f"{name}/mask"],
                                                        int(bm_), int(bn_))
            assert (crow == P[key]).all()
            ref_col = P[key[:-4] + "col"]
            assert col.shape == ref_col.shape and (col == ref_col).all()
            seen += 1
    assert seen == 6


ATTN = np.load(f"{GOLDEN}/attention.npz")
ATTN_CASES = {
    # name: B, Hq, Hkv, S, D, dtype, seq_dim, pattern kwargs (same recipe as make_golden.py)
    "small_f32": (1, 2, 2, 256, 64, torch.float32, 2, dict(block_size=64, local_blocks=2, vert_stride=2)),
    "gqa_f32": (1, 4, 2, 160, 32, torch.float32, 1, dict(block_size=32, local_blocks=2, vert_stride=3,
                                                         num_kv_heads=2)),
    "ragged_bf16": (1, 2, 2, 200, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    "bidir_f32": (1, 2, 2, 192, 64, torch.float32, 2, dict(block_size=64, local_blocks=1, vert_stride=3,
                                                          causal=False)),
}


def golden_attention_inputs(name):
    B, Hq, Hkv, S, D, dt, seq_dim, pk = ATTN_CASES[name]
    torch.manual_seed(20)
    shp = (lambda h: (B, h, S, D)) if seq_dim == 2 else (lambda h: (B, S, h, D))
    q = torch.randn(shp(Hq)).to(dt)
    k = torch.randn(shp(Hkv)).to(dt)
    v = torch.randn(shp(Hkv)).to(dt)
    do = torch.randn(shp(Hq)).to(dt)
    s = sum(t.double().sum().item() for t in (q, k, v, do))
    assert abs(s - float(ATTN[f"{name}/input_sum"])) < 1e-6, "torch RNG stream differs from the golden run"
    return q, k, v, do


@pytest.mark.parametrize("name", list(ATTN_CASES))
def test_masked_dense_attention_matches_reference_oracle(name):
    B, Hq, Hkv, S, D, dt, seq_dim, pk = ATTN_CASES[name]
    q, k, v, do = golden_attention_inputs(name)
    q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
    causal = pk.get("causal", True)
    bm = O.block_mask(Hq, S, **pk)
    assert (bm == ATTN[f"{name}/mask"]).all()
    dense = O.token_mask(bm, pk["block_size"], S, S, causal=causal)
    out = O.masked_dense_attention(q, k, v, dense, 0.0078125 * 8, seq_dim=seq_dim)
    out.backward(do)
    tol = 1e-5 if dt == torch.float32 else 2e-2
    for got, key in ((out, "out"), (q.grad, "dq"), (k.grad, "dk"), (v.grad, "dv")):
        ref = torch.from_numpy(ATTN[f"{name}/{key}"])
        assert (got.detach().float() - ref).abs().max().item() <= tol, f"{name}/{key}"
    # the per-head fp32 evaluator agrees with the masked-dense path
    o2, lse2 = O.block_sparse_attention(q.detach(), k.detach(), v.detach(), bm, pk["block_size"],
                                        0.0078125 * 8, seq_dim=seq_dim, causal=causal)
    assert (o2 - torch.from_numpy(ATTN[f"{name}/out"])).abs().max().item() <= (1e-5 if dt == torch.float32 else 2e-2)
    _, lse = O.masked_dense_attention(q.detach(), k.detach(), v.detach(), dense, 0.0078125 * 8,
                                      seq_dim=seq_dim, return_lse=True)
    # (the masked-dense path forms bf16 logits in bf16, like the reference's oracle)
    assert (lse - lse2).abs().max().item() < (1e-4 if dt == torch.float32 else 1e-2)


def test_config1_sample():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1024, 8, 64) for _ in range(3))
    bm = O.block_mask(8, 1024, 64, 4, 4)
    assert (bm == ATTN["c1/mask"]).all()
    assert int(bm.sum()) == 620
    dense = O.token_mask(bm, 64, 1024, 1024)
    out = O.masked_dense_attention(q, k, v, dense, 0.125, seq_dim=1)
    assert np.abs(out.numpy()[0, ::37, :, ::5] - ATTN["c1/out_sample"]).max() < 1e-5
    assert abs(out.double().sum().item() - float(ATTN["c1/out_sum"])) < 1e-2
    assert abs(out.double().abs().sum().item() - float(ATTN["c1/out_abs_sum"])) < 1e-1


def test_combine_attn_partitions():
    C = np.load(f"{GOLDEN}/combine.npz")
    parts = [(torch.from_numpy(C[f"o{i}"]), torch.from_numpy(C[f"lse{i}"])) for i in range(3)]
    res, lse = O.combine_attn_partitions(*parts)
    assert (res - torch.from_numpy(C["combined"])).abs().max().item() < 1e-6
    ref_lse = torch.logsumexp(torch.stack([p[1] for p in parts]), dim=0)
    assert (lse - ref_lse).abs().max().item() < 1e-5
    # hdim=2 layout gives the transposed result
    parts2 = [(o.transpose(1, 2).contiguous(), l) for o, l in parts]
    res2, _ = O.combine_attn_partitions(*parts2, hdim=2)
    assert (res2.transpose(1, 2) - res).abs().max().item() < 1e-6


def test_padded_varlen_decode_are_consistent():
    """The padded / packed / decode restatements agree with plain per-sequence attention."""
    torch.manual_seed(1)
    B, Hq, Hkv, S, D, bs = 3, 4, 2, 256, 32, 32
    bm = O.block_mask(Hq, S, bs, 2, 3, num_kv_heads=Hkv)
    lens = [256, 100, 33]
    q = torch.randn(B, S, Hq, D)
    k = torch.randn(B, S, Hkv, D)
    v = torch.randn(B, S, Hkv, D)
    left = [S - l for l in lens]
    out, lse = O.padded_attention(q, k, v, bm, bs, left_paddings=left, seq_dim=1)
    qs = torch.cat([q[b, left[b]:] for b in range(B)])
    ks = torch.cat([k[b, left[b]:] for b in range(B)])
    vs = torch.cat([v[b, left[b]:] for b in range(B)])
    cu = [0, 256, 356, 389]
    o2, lse2 = O.varlen_attention(qs, ks, vs, cu, bm, bs)
    for b in range(B):
        assert (out[b, left[b]:] - o2[cu[b]:cu[b + 1]]).abs().max() < 1e-5
        assert out[b, :left[b]].abs().max() == 0 if left[b] else True
        ref, _ = O.block_sparse_attention(q[b:b + 1, left[b]:], k[b:b + 1, left[b]:], v[b:b + 1, left[b]:],
                                          bm, bs, seq_dim=1)
        assert (ref[0] - o2[cu[b]:cu[b + 1]]).abs().max() < 1e-5
    # decode = last row of the prefill
    qd = torch.stack([q[b, S - 1:S] for b in range(B)])
    od, lsed = O.decode_attention(qd, k, v, bm, bs, left_paddings=left)
    for b in range(B):
        assert (od[b, 0] - out[b, S - 1]).abs().max() < 1e-5
        assert (lsed[b, :, 0] - lse[b, :, S - 1]).abs().max() < 1e-4
    # KV shards merge back to the whole
    parts = []
    for lo, hi in ((0, 3), (3, 8)):
        o_, l_ = O.decode_attention(qd, k, v, bm, bs, left_paddings=left, kv_block_range=(lo, hi))
        parts.append((o_.transpose(1, 2), l_))
    merged, mlse = O.combine_attn_partitions(*parts)
    assert (merged.transpose(1, 2) - od).abs().max() < 1e-5
    assert (mlse - lsed).abs().max() < 1e-4
