"""Multi-rank host logic on CPU (gloo, world_size 2): head sharding, KV-sequence
sharding with the one-message gather of packed decode partials, and the ring
schedule of context-parallel attention (forward and backward).  The per-rank
compute is done by the CPU oracle here (the GPU tests cover the kernels); what is
checked is that partitioning + exchange + merge reproduce the un-partitioned result."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import dkernel_oracle as O


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dkernel_b200.dist import (head_shard, kv_shard_ranges, pack_kv_shard, packed_partial_views,
                                       partial_row_bytes, gather_packed_partials, split_gathered_partials)
        torch.manual_seed(0)                      # identical inputs on every rank
        B, Hq, Hkv, S, D, bs = 3, 4, 2, 512, 32, 64
        q = torch.randn(B, 1, Hq, D)
        k = torch.randn(B, S, Hkv, D)
        v = torch.randn(B, S, Hkv, D)
        lens = torch.tensor([512, 130, 64])
        left = S - lens
        bm = O.block_mask(Hq, S, bs, 2, 3, num_kv_heads=Hkv)
        ref, ref_lse = O.decode_attention(q, k, v, bm, bs, left_paddings=left)

        # ---- KV-sequence sharding: rank-local partial, one all-gather, merge
        lo, hi = kv_shard_ranges(lens, rank, world, bs)
        ks, vs, n = pack_kv_shard(k, v, left, lo, hi)
        part_o = torch.zeros(B, 1, Hq, D)
        part_l = torch.full((B, Hq, 1), float("-inf"))
        for b in range(B):
            if n[b] == 0:
                continue
            # the shard holds positions [lo, hi): evaluate with the block range restriction
            o_b, l_b = O.decode_attention(q[b:b + 1], k[b:b + 1], v[b:b + 1], bm, bs,
                                          left_paddings=left[b:b + 1],
                                          kv_block_range=(int(lo[b]) // bs, (int(hi[b]) + bs - 1) // bs))
            part_o[b], part_l[b] = o_b[0], l_b[0]
            # and the packed shard really is that slice of the sequence
            s0 = int(left[b] + lo[b])
            assert torch.equal(ks[b, :int(n[b])], k[b, s0:s0 + int(n[b])])
        # the byte packing sharded_decode uses: 16-bit outputs and the fp32 LSE of a row side by
        # side, written through strided views, one message, read back through strided views
        packed = torch.zeros((B * Hq, partial_row_bytes(D)), dtype=torch.uint8)
        o_view, lse_view = packed_partial_views(packed, D, torch.bfloat16)
        assert o_view.shape == (B * Hq, D) and o_view.stride() == (D + 2, 1) and lse_view.stride() == ((2 * D + 4) // 4,)
        o_view.copy_(part_o.reshape(B * Hq, D))
        lse_view.copy_(part_l.reshape(B * Hq))
        gathered = gather_packed_partials(packed)
        o_parts, l_parts = split_gathered_partials(gathered, world, D, torch.bfloat16)
        assert o_parts.shape == (world, B * Hq, D) and l_parts.shape == (world, B * Hq)
        assert torch.equal(o_parts[rank], part_o.reshape(B * Hq, D).to(torch.bfloat16))
        assert torch.equal(l_parts[rank], part_l.reshape(B * Hq))
        parts = [(o_parts[r].float().reshape(B, 1, Hq, D).transpose(1, 2), l_parts[r].reshape(B, Hq, 1))
                 for r in range(world)]
        merged, mlse = O.combine_attn_partitions(*parts)
        assert (merged.transpose(1, 2) - ref).abs().max() < 2e-2       # partials rounded to bf16
        assert (mlse - ref_lse).abs().max() < 1e-4

        # ---- head sharding: rank-local heads, no collective; concatenation == whole
        (h0, h1), (kv0, kv1) = head_shard(Hq, Hkv, rank, world)
        qs = torch.randn(1, 256, Hq, D)
        kk = torch.randn(1, 256, Hkv, D)
        vv = torch.randn(1, 256, Hkv, D)
        bm2 = O.block_mask(Hq, 256, bs, 2, 3, num_kv_heads=Hkv)
        full, _ = O.block_sparse_attention(qs, kk, vv, bm2, bs, seq_dim=1)
        mine, _ = O.block_sparse_attention(qs[:, :, h0:h1], kk[:, :, kv0:kv1], vv[:, :, kv0:kv1],
                                           bm2[h0:h1], bs, seq_dim=1)
        assert (mine - full[:, :, h0:h1]).abs().max() < 1e-5
        gathered = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(gathered, mine.contiguous())       # test-side check only
        assert (torch.cat(gathered, dim=2) - full).abs().max() < 1e-5
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


def test_two_ranks_gloo():
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {0: "ok", 1: "ok"}


def _ring_worker(rank, world, port, ret, zigzag=False):
    """Ring attention schedule (K/V chunks round the ring, LSE merge, dK/dV contributions sent to
    the chunk's owner) with the oracle as the per-chunk compute; compared with full-sequence autograd.
    zigzag: every rank owns two pieces of the sequence (r and 2 * world - 1 - r) and no step is skipped."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from dkernel_b200.dist import (chunk_bounds, ring_backward, ring_forward, ring_steps, zigzag_bounds,
                                       zigzag_shard)
        torch.manual_seed(1)
        B, H, S, D, bs = 2, 2, 512, 16, 64
        scale = 1.0 / D ** 0.5
        q, k, v, do = (torch.randn(B, S, H, D) for _ in range(4))
        dl = torch.randn(B, H, S)
        bm = O.block_mask(H, S, bs, 2, 3)
        dense = O.token_mask(bm, bs, S, S).bool()                   # (H, S, S), causal
        if zigzag:
            pieces = zigzag_bounds(S, world, bs)
            assert sorted(x for p in pieces for x in p) == [(i * S // (2 * world), (i + 1) * S // (2 * world))
                                                            for i in range(2 * world)]
        else:
            pieces = [[b] for b in chunk_bounds(S, world, bs)]
            assert [s for _, s, a in ring_steps(rank, world) if a] == list(range(rank, -1, -1))
        idx = [torch.cat([torch.arange(a, b) for a, b in p]) for p in pieces]     # positions of every rank

        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        ref, ref_lse = O.masked_dense_attention(qf, kf, vf, dense.to(torch.uint8), scale, seq_dim=1,
                                                return_lse=True)
        ((ref * do).sum() + (ref_lse * dl).sum()).backward()

        def pair_mask(r, s):
            return dense[:, idx[r]][:, :, idx[s]]

        def fwd_chunk(qc, kc, vc, r, s):
            return O.masked_dense_attention(qc, kc, vc, pair_mask(r, s).to(torch.uint8), scale, seq_dim=1,
                                            return_lse=True)

        def merge(parts):
            if len(parts) == 1:
                return parts[0]
            o, l = O.combine_attn_partitions(*[(o.transpose(1, 2), l) for o, l in parts])
            return o.transpose(1, 2), l

        def bwd_chunk(qc, kc, vc, o, lse, dout, dlse, r, s):
            # gradients of one chunk pair from the merged output and LSE
            sc = torch.einsum("bmhd,bnhd->bhmn", qc, kc) * scale
            sc = sc.masked_fill(~pair_mask(r, s)[None], float("-inf"))
            p = torch.exp(sc - lse[..., None])
            dp = torch.einsum("bmhd,bnhd->bhmn", dout, vc)
            delta = (dout * o).sum(-1).transpose(1, 2) - (dlse if dlse is not None else 0)
            ds = p * (dp - delta[..., None])
            return (torch.einsum("bhmn,bnhd->bmhd", ds, kc) * scale,
                    torch.einsum("bhmn,bmhd->bnhd", ds, qc) * scale,
                    torch.einsum("bhmn,bmhd->bnhd", p, dout))

        mine = idx[rank]
        ql, kl, vl = q[:, mine].contiguous(), k[:, mine].contiguous(), v[:, mine].contiguous()
        if zigzag:
            assert torch.equal(ql, zigzag_shard(q, rank, world, bs, seq_dim=1))
        skip = not zigzag      # contiguous chunks: kv chunks after the own one are skipped
        out, lse = ring_forward(ql, kl, vl, fwd_chunk, merge, causal=skip)
        assert (out - ref[:, mine].detach()).abs().max() < 1e-5
        assert (lse - ref_lse[:, :, mine].detach()).abs().max() < 1e-5
        dq, dk, dv = ring_backward(ql, kl, vl, out, lse, do[:, mine].contiguous(), dl[:, :, mine].contiguous(),
                                   bwd_chunk, causal=skip)
        for got, want, name in ((dq, qf.grad, "dq"), (dk, kf.grad, "dk"), (dv, vf.grad, "dv")):
            err = (got - want[:, mine]).abs().max().item()
            assert err < 1e-4, f"{name}: {err}"
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("zigzag", [False, True])
@pytest.mark.parametrize("world", [2, 4])
def test_ring_attention_schedule_gloo(world, zigzag):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_ring_worker, args=(world, _free_port(), ret, zigzag), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}


def test_planning_functions():
    from dkernel_b200.dist import head_shard, kv_shard_ranges
    # head shards tile the head range and keep kv groups whole
    for hq, hkv, w in ((32, 8, 1), (32, 8, 2), (32, 8, 4), (32, 8, 8), (32, 32, 8), (8, 2, 2)):
        seen_q, seen_kv = [], []
        for r in range(w):
            (a, b), (c, d) = head_shard(hq, hkv, r, w)
            assert (b - a) == (d - c) * (hq // hkv) and a == c * (hq // hkv)
            seen_q += list(range(a, b))
            seen_kv += list(range(c, d))
        assert seen_q == list(range(hq)) and seen_kv == list(range(hkv))
    with pytest.raises(AssertionError):
        head_shard(32, 8, 0, 3)
    # kv shards: disjoint, block aligned, cover [0, len)
    lens = torch.tensor([1, 63, 64, 65, 1024, 5263, 8192])
    for w in (1, 2, 4, 8):
        cover = torch.zeros_like(lens)
        prev_hi = torch.zeros_like(lens)
        for r in range(w):
            lo, hi = kv_shard_ranges(lens, r, w, 64)
            assert (lo % 64 == 0).all() and (hi >= lo).all() and (hi <= lens).all()
            assert (lo == prev_hi).all() or ((hi - lo)[lo != prev_hi] == 0).all()
            prev_hi = torch.where(hi > lo, hi, prev_hi)
            cover += hi - lo
        assert (cover == lens).all()
        # balance: no rank holds more than one block above the ideal share
        for r in range(w):
            lo, hi = kv_shard_ranges(lens, r, w, 64)
            assert ((hi - lo) <= (lens + w - 1) // w + 64).all()


def test_host_logic_without_gpu():
    """Package import, pack-mode splitting and the no-CPU-path errors."""
    import dkernel_b200
    from dkernel_b200.ops import get_qkv_and_pack_mode, _pick_heads_per_cta
    from dkernel_b200.utils import multiple_of, zero_stride, cdiv
    assert multiple_of(1000, 64) == 1024 and multiple_of(1024, 64) == 1024 and cdiv(65, 64) == 2
    x = torch.zeros(1, 4, 5)
    assert zero_stride(x).stride(0) == 0
    q = torch.randn(2, 8, 6, 4)
    (a, b, c), (shape, mode, fn) = get_qkv_and_pack_mode(q, None, None, split_qkv=lambda t: t.chunk(3, dim=2))
    assert mode == "packed_qkv" and shape == q.shape and a.shape == (2, 8, 2, 4)
    (a, b, c), (shape, mode, fn) = get_qkv_and_pack_mode(q, q, None, split_qkv=lambda t: t.chunk(2, dim=2))
    assert mode == "packed_kv" and b.shape == (2, 8, 3, 4)
    with pytest.raises(AssertionError):
        get_qkv_and_pack_mode(q, None, None)
    assert [_pick_heads_per_cta(g) for g in (1, 2, 4, 7, 16, 32, 24)] == [1, 2, 4, 7, 16, 16, 12]
    if not torch.cuda.is_available():
        with pytest.raises(RuntimeError, match="no CPU path"):
            dkernel_b200.get_sparse_attn_mask(2, 128)
        with pytest.raises(RuntimeError, match="no CPU path|CUDA"):
            dkernel_b200.SparseAttention(64, torch.ones(2, 2))


def test_kv_block_pairing_table_for_the_dkdv_kernel():
    """Host-side planning: the pairing of kv blocks handed to the tensor-core dK/dV kernel covers
    every block once, shortens the unions for a local + vertical-stride pattern and is not
    produced where pairing neighbours is as good."""
    import numpy as np
    from oracle import dkernel_oracle as O
    from dkernel_b200.ops import _Plan
    H, S, bs = 4, 4096, 64
    bm = np.tril(np.ones((S // bs, S // bs), bool))[None] & O.block_mask(H, S, block_size=bs, local_blocks=8,
                                                                         vert_stride=8).astype(bool)
    as_i32 = lambda arrs: [torch.from_numpy(np.ascontiguousarray(a)).int() for a in arrs]
    plan = _Plan(*as_i32(O.dense_to_crow_col(bm)), *as_i32(O.dense_to_ccol_row(bm)), bs, 0)
    pairs = plan.kv_pairs(H, H, S // bs)
    assert pairs is not None and pairs.shape == (H, S // bs // 2, 2) and pairs.dtype == torch.int32
    for h in range(H):
        assert sorted(pairs[h].flatten().tolist()) == list(range(S // bs))
        union = sum(int((bm[h, :, a] | bm[h, :, b]).sum()) for a, b in pairs[h].tolist())
        adjacent = sum(int((bm[h, :, c] | bm[h, :, c + 1]).sum()) for c in range(0, S // bs, 2))
        assert union < 0.97 * adjacent
    assert plan.kv_pairs(H, H, S // bs) is pairs                       # cached
    # fewer key blocks than the pattern has: only those are paired, odd count leaves one alone
    p5 = plan.kv_pairs(H, H, 31)
    assert p5 is None or (p5.shape[1] == 16 and sorted(x for x in p5[0].flatten().tolist() if x >= 0) == list(range(31)))
    # a dense causal pattern gains nothing: neighbours stay paired
    dense = np.tril(np.ones((16, 16), bool))[None]
    plan2 = _Plan(*as_i32(O.dense_to_crow_col(dense)), *as_i32(O.dense_to_ccol_row(dense)), bs, 0)
    assert plan2.kv_pairs(1, 1, 16) is None
