"""Padded, packed (varlen) and decode routes vs the CPU oracle."""
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


@pytest.mark.parametrize("B,Hq,Hkv,S,D,dtype,seq_dim,pk,right", [
    (3, 4, 2, 320, 64, torch.float16, 1, dict(block_size=64, local_blocks=2, vert_stride=3, num_kv_heads=2), False),
    (2, 2, 2, 512, 128, torch.bfloat16, 2, dict(block_size=64, local_blocks=2, vert_stride=4, homo_head=True), False),
    (3, 2, 2, 300, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=3, vert_stride=2), True),
    (2, 2, 2, 256, 32, torch.float32, 1, dict(block_size=16, local_blocks=4, vert_stride=4), False),
])
def test_padded_prefill(B, Hq, Hkv, S, D, dtype, seq_dim, pk, right):
    bs = pk["block_size"]
    shape = (lambda h: (B, h, S, D)) if seq_dim == 2 else (lambda h: (B, S, h, D))
    q, k, v = seeded_qkv(11, shape(Hq), shape(Hkv), dtype)
    lens = torch.randint(1, S, (B,), generator=torch.Generator().manual_seed(2))
    lens[0] = S
    bm = O.block_mask(Hq, S, **pk)
    mod = _module(Hq, S, pk, seq_dim=seq_dim)
    if right:
        ref, ref_lse = O.padded_attention(q.float(), k.float(), v.float(), bm, bs, seqlens=lens, seq_dim=seq_dim)
        out, lse = mod(q.cuda(), k.cuda(), v.cuda(), seqlens=lens.cuda(), return_lse=True)
    else:
        left = S - lens
        ref, ref_lse = O.padded_attention(q.float(), k.float(), v.float(), bm, bs, left_paddings=left,
                                          seq_dim=seq_dim)
        out, lse = mod(q.cuda(), k.cuda(), v.cuda(), left_paddings=left.cuda(), return_lse=True)
    tight = dtype == torch.float32
    assert_out_close(out, ref, max_abs=2e-4 if tight else 2e-2, mean_abs=2e-5 if tight else 2e-3)
    assert_lse_close(lse, ref_lse, tol=1e-4 if tight else 1e-3)


@pytest.mark.parametrize("Hq,Hkv,D,dtype,bs,lens", [
    (4, 4, 128, torch.bfloat16, 64, [512, 100, 333, 64, 1]),
    (4, 2, 64, torch.float16, 32, [200, 31, 256]),
    (2, 2, 128, torch.bfloat16, 64, [700]),
])
def test_varlen_prefill_user_pattern(Hq, Hkv, D, dtype, bs, lens):
    """Packed sequences with a random lower-triangular user pattern (config-5 style)."""
    from dkernel_b200 import SparseAttention
    nb = 16
    g = torch.Generator().manual_seed(0)
    pat = torch.rand(Hq, nb, nb, generator=g) < 0.3
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    T = sum(lens)
    q, k, v = seeded_qkv(5, (T, Hq, D), (T, Hkv, D), dtype)
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32)
    ref, ref_lse = O.varlen_attention(q.float(), k.float(), v.float(), cu, pat.numpy().astype(np.uint8), bs)
    with pytest.warns(UserWarning):
        mod = SparseAttention(bs, pat.cuda())
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), cu_seqlen_k=cu.cuda(), return_lse=True)
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


@pytest.mark.parametrize("impl", ["sm100", "generic"])
def test_varlen_batched_chunked_prefill(impl):
    """A packed batch that mixes whole prompts, decode tokens and prompt chunks whose earlier
    part is already in the KV cache (q_len not in {1, k_len}; the chunk starts on a block
    boundary).  The reference's kernel computes this case (pattern row from past_len + q
    offset, dkernel/ops/sparse_attn_inference.py:507-514) but its host code refuses it
    (:211-212); here the host does not look at the lengths, so it is served."""
    from dkernel_b200 import SparseAttention
    Hq, Hkv, D, bs, nb = 8, 2, 128, 64, 16
    g = torch.Generator().manual_seed(3)
    pat = torch.rand(Hq, nb, nb, generator=g) < 0.35
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    q_lens = [64, 1, 130, 72, 300]
    k_lens = [192, 300, 130, 200, 940]          # pasts 128, 299, 0, 128, 640
    cu_q = torch.tensor([0] + list(np.cumsum(q_lens)), dtype=torch.int32)
    cu_k = torch.tensor([0] + list(np.cumsum(k_lens)), dtype=torch.int32)
    q, k, v = seeded_qkv(31, (sum(q_lens), Hq, D), (sum(k_lens), Hkv, D), torch.bfloat16)
    ref, ref_lse = O.varlen_attention(q.float(), k.float(), v.float(), cu_k, pat.numpy().astype(np.uint8), bs,
                                      cu_seqlens_q=cu_q)
    with pytest.warns(UserWarning):
        mod = SparseAttention(bs, pat.cuda(), impl=impl)
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), cu_seqlen_k=cu_k.cuda(), cu_seqlen_q=cu_q.cuda(),
                   return_lse=True)
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)


@pytest.mark.parametrize("B,Hq,Hkv,S,D,dtype,seq_dim,pk,bps", [
    (5, 8, 2, 1024, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=4, vert_stride=4, num_kv_heads=2), 0),
    (3, 4, 4, 640, 64, torch.float16, 2, dict(block_size=64, local_blocks=2, vert_stride=3), 2),
    (2, 4, 1, 1024, 128, torch.bfloat16, 1, dict(block_size=128, local_blocks=2, vert_stride=2, num_kv_heads=1), 1),
    (2, 2, 2, 256, 32, torch.float32, 1, dict(block_size=32, local_blocks=2, vert_stride=2), 0),   # generic route
])
def test_left_padded_decode(B, Hq, Hkv, S, D, dtype, seq_dim, pk, bps):
    bs = pk["block_size"]
    kshape = (B, Hkv, S, D) if seq_dim == 2 else (B, S, Hkv, D)
    qshape = (B, Hq, 1, D) if seq_dim == 2 else (B, 1, Hq, D)
    q, k, v = seeded_qkv(13, qshape, kshape, dtype)
    lens = torch.randint(1, S + 1, (B,), generator=torch.Generator().manual_seed(4))
    lens[0] = S
    lens[-1] = 1
    left = S - lens
    bm = O.block_mask(Hq, S, **pk)
    q1 = q if seq_dim == 1 else q.transpose(1, 2)
    k1, v1 = (k, v) if seq_dim == 1 else (k.transpose(1, 2), v.transpose(1, 2))
    ref, ref_lse = O.decode_attention(q1.float(), k1.float(), v1.float(), bm, bs, left_paddings=left)
    if seq_dim == 2:
        ref = ref.transpose(1, 2)
    mod = _module(Hq, S, pk, seq_dim=seq_dim)
    if bps:
        from dkernel_b200.ops import decode
        out, lse = decode(q.cuda(), k.cuda(), v.cuda(), mod._plan(), 1 / math.sqrt(D), seq_dim=seq_dim,
                          k_start=left.to(torch.int32).cuda(),
                          k_end=torch.full((B,), S, dtype=torch.int32).cuda(), blocks_per_split=bps)
        lse = lse.unsqueeze(-1)
    else:
        out, lse = mod(q.cuda(), k.cuda(), v.cuda(), left_paddings=left.cuda(), return_lse=True)
    tight = dtype == torch.float32
    assert_out_close(out, ref, max_abs=2e-4 if tight else 2e-2, mean_abs=2e-5 if tight else 2e-3)
    assert_lse_close(lse, ref_lse, tol=1e-4 if tight else 1e-3)


def test_unpadded_and_packed_decode():
    B, Hq, Hkv, S, D, bs = 2, 4, 2, 64 * 5 + 12, 128, 64
    pk = dict(block_size=bs, local_blocks=2, vert_stride=3, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(17, (B, 1, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    bm = O.block_mask(Hq, 1024, **pk)
    ref, ref_lse = O.decode_attention(q.float(), k.float(), v.float(), bm, bs)
    mod = _module(Hq, 1024, pk, seq_dim=1)
    out, lse = mod(q.cuda(), k.cuda(), v.cuda(), return_lse=True)
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    # packed: q (B, Hq, D), k/v (sum lens, Hkv, D)
    lens = [S, 77]
    kp = torch.cat([k[0, :lens[0]], k[1, :lens[1]]])
    vp = torch.cat([v[0, :lens[0]], v[1, :lens[1]]])
    cu = torch.tensor([0, lens[0], lens[0] + lens[1]], dtype=torch.int32)
    refp, _ = O.varlen_attention(q[:, 0].float(), kp.float(), vp.float(), cu, bm, bs)
    outp = mod(q[:, 0].cuda(), kp.cuda(), vp.cuda(), cu_seqlen_k=cu.cuda())
    assert_out_close(outp, refp)


def test_kv_sharded_decode_merges_to_whole():
    """KV shards by position range + combine_attn_partitions == un-sharded decode."""
    from dkernel_b200.ops import decode
    from dkernel_b200 import combine_attn_partitions
    B, Hq, Hkv, S, D, bs = 4, 8, 2, 1024, 128, 64
    pk = dict(block_size=bs, local_blocks=4, vert_stride=4, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(19, (B, 1, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    lens = torch.tensor([1024, 700, 65, 300])
    left = S - lens
    bm = O.block_mask(Hq, S, **pk)
    ref, ref_lse = O.decode_attention(q.float(), k.float(), v.float(), bm, bs, left_paddings=left)
    mod = _module(Hq, S, pk, seq_dim=1)
    G = 2
    parts = []
    for r in range(G):
        # rank r holds, for every sequence, positions [lo, hi) (block aligned), left-packed locally
        nblk = (lens + bs - 1) // bs
        lo = (nblk * r // G) * bs
        hi = torch.minimum((nblk * (r + 1) // G) * bs, lens)
        n = (hi - lo).clamp_min(0)
        cap = int(n.max().item())
        ks = torch.zeros(B, max(cap, 1), Hkv, D, dtype=k.dtype)
        vs = torch.zeros_like(ks)
        for b in range(B):
            s0 = int(left[b] + lo[b])
            ks[b, :int(n[b])] = k[b, s0:s0 + int(n[b])]
            vs[b, :int(n[b])] = v[b, s0:s0 + int(n[b])]
        o, l = decode(q.cuda(), ks.cuda(), vs.cuda(), mod._plan(), 1 / math.sqrt(D), seq_dim=1,
                      k_start=torch.zeros(B, dtype=torch.int32).cuda(), k_end=n.to(torch.int32).cuda(),
                      k_pos0=lo.to(torch.int32).cuda(), k_total=lens.to(torch.int32).cuda())
        parts.append((o, l.unsqueeze(-1)))
    merged, mlse = combine_attn_partitions(*parts, hdim=2, return_lse=True)
    assert_out_close(merged, ref)
    assert_lse_close(mlse, ref_lse)


@pytest.mark.parametrize("W", [2, 4, 8])
def test_block_cyclic_kv_shards_merge_to_whole(W):
    """Block-cyclic KV shards (block j of a sequence on rank j % W) decoded one rank after the
    other on this GPU + combine_attn_partitions == un-sharded decode; ranks without any attended
    block give O = 0, LSE = -inf."""
    from dkernel_b200.ops import decode
    from dkernel_b200.dist import kv_shard_cyclic_blocks, pack_kv_shard_cyclic
    from dkernel_b200 import combine_attn_partitions
    B, Hq, Hkv, S, D, bs = 5, 8, 2, 2048, 128, 64
    pk = dict(block_size=bs, local_blocks=6, vert_stride=4, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(29, (B, 1, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    lens = torch.tensor([2048, 700, 65, 1, 1300])
    left = S - lens
    bm = O.block_mask(Hq, S, **pk)
    ref, ref_lse = O.decode_attention(q.float(), k.float(), v.float(), bm, bs, left_paddings=left)
    mod = _module(Hq, S, pk, seq_dim=1)
    parts, stored = [], torch.zeros_like(lens)
    for r in range(W):
        ks, vs, n = pack_kv_shard_cyclic(k, v, left, lens, r, W, bs)
        assert torch.equal(n, kv_shard_cyclic_blocks(lens, r, W, bs))
        stored += n
        o, l = decode(q.cuda(), ks.cuda(), vs.cuda(), mod._plan(), 1 / math.sqrt(D), seq_dim=1,
                      k_end=n.to(torch.int32).cuda(), k_total=lens.to(torch.int32).cuda(), k_blk=(W, r))
        parts.append((o, l.unsqueeze(-1)))
    assert torch.equal(stored, lens)                       # every token lives on exactly one rank
    merged, mlse = combine_attn_partitions(*parts, hdim=2, return_lse=True)
    assert_out_close(merged, ref)
    assert_lse_close(mlse, ref_lse)
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0


@pytest.mark.parametrize("D,dtype", [(128, torch.bfloat16), (64, torch.bfloat16), (128, torch.float16)])
def test_decode_reads_an_e4m3_kv_cache(D, dtype):
    """K/V stored as float8_e4m3fn with per-tensor scales: the decode kernel converts the stored
    bytes exactly, so the result must equal the oracle on the de-quantised cache -- left padding,
    right padding, the split-KV path (long rows) and a packed batch."""
    from dkernel_b200 import SparseAttention
    B, Hq, Hkv, S, bs = 5, 8, 2, 2048, 64
    pk = dict(block_size=bs, local_blocks=6, vert_stride=4, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(61, (B, 1, Hq, D), (B, S, Hkv, D), dtype)
    ks, vs = float(k.float().abs().max()) / 448.0, float(v.float().abs().max()) / 448.0
    k8 = (k.float() / ks).to(torch.float8_e4m3fn)
    v8 = (v.float() / vs).to(torch.float8_e4m3fn)
    kd, vd = k8.float() * ks, v8.float() * vs                  # what the cache stands for
    bm = O.block_mask(Hq, S, **pk)
    mod = _module(Hq, S, pk, seq_dim=1)
    lens = torch.tensor([2048, 700, 65, 1, 1300])
    left = S - lens
    ref, ref_lse = O.decode_attention(q.float(), kd, vd, bm, bs, left_paddings=left)
    with torch.no_grad():
        out, lse = mod(q.cuda(), k8.cuda(), v8.cuda(), left_paddings=left.cuda(), return_lse=True,
                       kv_scales=(ks, vs))
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    # right padding: whatever follows the sequence in the cache is ignored (0xff bytes are NaN in e4m3)
    k8r, v8r = k8.clone(), v8.clone()
    for b in range(B):
        k8r[b, int(lens[b]):].view(torch.uint8).fill_(0xff)
        v8r[b, int(lens[b]):].view(torch.uint8).fill_(0xff)
    ref, ref_lse = O.decode_attention(q.float(), kd, vd, bm, bs, seqlens=lens)
    with torch.no_grad():
        out, lse = mod(q.cuda(), k8r.cuda(), v8r.cuda(), seqlens=lens.cuda(), return_lse=True, kv_scales=(ks, vs))
    assert_out_close(out, ref)
    assert_lse_close(lse, ref_lse)
    # packed batch, one query token per sequence
    lens2 = [300, 64, 1, 999]
    cu = torch.tensor([0] + list(np.cumsum(lens2)), dtype=torch.int32)
    T = int(cu[-1])
    kp, vp = seeded_qkv(62, (T, Hkv, D), (T, Hkv, D), dtype)[:2]
    kp8, vp8 = (kp.float() / ks).to(torch.float8_e4m3fn), (vp.float() / vs).to(torch.float8_e4m3fn)
    qp = q[:4, 0]
    refp, _ = O.varlen_attention(qp.float(), kp8.float() * ks, vp8.float() * vs, cu, bm, bs)
    with torch.no_grad():
        outp = mod(qp.cuda(), kp8.cuda(), vp8.cuda(), cu_seqlen_k=cu.cuda(), kv_scales=(ks, vs))
    assert_out_close(outp, refp)
    # an 8-bit cache without scales, or on a prefill call, is refused before any launch
    with pytest.raises(AssertionError):
        mod(q.cuda(), k8.cuda(), v8.cuda(), left_paddings=left.cuda())
    with pytest.raises(AssertionError):
        mod(q.expand(B, 1, Hq, D).repeat(1, S, 1, 1).cuda(), k8.cuda(), v8.cuda(), kv_scales=(ks, vs))
    from dkernel_b200 import _lib
    assert _lib.wait_status() == 0


def test_sharded_decode_single_rank_group(tmp_path):
    """sharded_decode end to end (packed (O, LSE) rows -> all-gather -> fused merge) with a
    one-rank NCCL group: the whole sequence is the only shard."""
    import torch.distributed as dist
    from dkernel_b200.dist import sharded_decode
    B, Hq, Hkv, S, D, bs = 3, 8, 2, 1024, 128, 64
    pk = dict(block_size=bs, local_blocks=4, vert_stride=4, num_kv_heads=Hkv)
    q, k, v = seeded_qkv(23, (B, 1, Hq, D), (B, S, Hkv, D), torch.bfloat16)
    lens = torch.tensor([1024, 513, 64])
    bm = O.block_mask(Hq, S, **pk)
    # left-aligned storage: sequence b occupies rows [0, lens[b])
    ref, ref_lse = O.decode_attention(q.float(), k.float(), v.float(), bm, bs, seqlens=lens)
    mod = _module(Hq, S, pk, seq_dim=1)
    store = dist.FileStore(str(tmp_path / "pg"), 1)
    dist.init_process_group("nccl", store=store, rank=0, world_size=1)
    try:
        out, lse = sharded_decode(mod, q.cuda(), k.cuda(), v.cuda(), lens.to(torch.int32).cuda(),
                                  torch.zeros(B, dtype=torch.int32).cuda(), lens.to(torch.int32).cuda(),
                                  1 / math.sqrt(D))
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()
    assert_out_close(out, ref)
    assert_lse_close(lse.unsqueeze(-1), ref_lse)


def test_combine_attn_partitions_matches_reference_fixture(golden_dir):
    from dkernel_b200 import combine_attn_partitions
    C = np.load(f"{golden_dir}/combine.npz")
    parts = [(torch.from_numpy(C[f"o{i}"]).cuda(), torch.from_numpy(C[f"lse{i}"]).cuda()) for i in range(3)]
    res = combine_attn_partitions(*parts)
    assert (res.cpu() - torch.from_numpy(C["combined"])).abs().max().item() < 1e-5
    # hdim = 2 (outputs laid out (B, S, H, D))
    parts2 = [(o.transpose(1, 2).contiguous(), l) for o, l in parts]
    res2 = combine_attn_partitions(*parts2, hdim=2)
    assert (res2.transpose(1, 2).cpu() - torch.from_numpy(C["combined"])).abs().max().item() < 1e-5
    # -inf partitions contribute nothing and do not create NaN
    o0, l0 = parts[0]
    dead = (torch.full_like(o0, float("nan")).nan_to_num(0.0), torch.full_like(l0, float("-inf")))
    res3, lse3 = combine_attn_partitions(parts[0], dead, return_lse=True)
    assert (res3 - o0).abs().max().item() < 1e-6 and (lse3 - l0).abs().max().item() < 1e-6
    # differentiable route gives the same numbers and gradients reach the LSEs
    pg = [(o.clone().requires_grad_(), l.clone().requires_grad_()) for o, l in parts]
    r = combine_attn_partitions(*pg)
    assert (r.detach().cpu() - torch.from_numpy(C["combined"])).abs().max().item() < 1e-5
    r.sum().backward()
    assert pg[0][1].grad is not None and torch.isfinite(pg[0][1].grad).all()


def test_seq_partition_equivalence():
    """Chunked q x kv attention merged by LSE equals the un-partitioned result
    (the reference's tests/test_seq_partition.py, 'ring' and 'one-kv' modes), forward
    and backward."""
    from dkernel_b200 import SparseAttention, get_sparse_attn_mask, combine_attn_partitions
    b, h, S, d, bs, nparts = 1, 3, 1024, 64, 64, 4
    dtype = torch.bfloat16
    for mode in ("ring", "one-kv"):
        q, k, v, do = seeded_qkv(20, (b, h, S, d), (b, h, S, d), dtype, device="cuda", with_do=True)
        q.requires_grad_(), k.requires_grad_(), v.requires_grad_()
        chunk = S // nparts
        outs = []
        for qc in range(nparts):
            end_kv = (qc + 1) * chunk
            ranges = [(i * chunk, (i + 1) * chunk) for i in range(qc + 1)] if mode == "ring" else [(0, end_kv)]
            parts, masks = [], []
            for (ks, ke) in ranges:
                _, bmask, _ = get_sparse_attn_mask(h, chunk, bs, 4, 4, dtype=torch.uint8,
                                                   q_start_position=qc * chunk, kv_start_position=ks,
                                                   kv_seqlen=ke - ks)
                masks.append(bmask)
                layer = SparseAttention(bs, bmask, seq_dim=2, causal=(ke == end_kv))
                parts.append(layer(q[:, :, qc * chunk:end_kv], k[:, :, ks:ke], v[:, :, ks:ke], return_lse=True))
            outs.append(parts[0][0] if len(parts) == 1 else combine_attn_partitions(*parts, hdim=1))
            _, full, _ = get_sparse_attn_mask(h, S, bs, 4, 4, dtype=torch.uint8)
            cat = torch.cat(masks, dim=-1)
            assert (cat == full[:, qc * (chunk // bs):(qc + 1) * (chunk // bs), :cat.size(-1)]).all()
        out = torch.cat(outs, dim=2)
        out.backward(do)
        grads = [t.grad.clone() for t in (q, k, v)]
        for t in (q, k, v):
            t.grad = None
        _, full, _ = get_sparse_attn_mask(h, S, bs, 4, 4, dtype=torch.uint8)
        ref_layer = SparseAttention(bs, full, seq_dim=2)
        ref = ref_layer(q, k, v)
        ref.backward(do)
        assert torch.allclose(out, ref, rtol=1e-2, atol=1e-2), mode
        for g, t, n in zip(grads, (q, k, v), "qkv"):
            assert torch.allclose(g, t.grad, rtol=1e-2, atol=2e-2), f"{mode} d{n}: {(g - t.grad).abs().max()}"
            t.grad = None
