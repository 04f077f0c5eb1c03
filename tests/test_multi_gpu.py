"""Multi-GPU paths on real devices (2 and 4 ranks, one process per GPU, NCCL for the plumbing):

* KV-sharded decode: both exchange routes (the peer-store kernel ``ShardedDecoder`` and the NCCL
  all-gather ``sharded_decode``) against the single-GPU decode of the un-sharded cache and
  against the CPU oracle, over several steps and under CUDA-graph replay.
* Context-parallel (ring) attention: forward and backward against the single-GPU module on the
  whole sequence.

Skipped on a machine with fewer GPUs than ranks (the gloo tests cover the host logic there).
"""
import math
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    # a short collective timeout: if one rank fails an assertion and leaves, the others stop after
    # three minutes instead of the default ten
    import datetime
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev,
                            timeout=datetime.timedelta(seconds=180))
    try:
        from oracle import dkernel_oracle as O
        from dkernel_b200 import LocalStrideSparseAttention, _lib
        from dkernel_b200.dist import (ContextParallelSparseAttention, ShardedDecoder, kv_shard_ranges,
                                       pack_kv_shard, pack_kv_shard_cyclic, sharded_decode, zigzag_bounds)
        # ---------------------------------------------------------------- KV-sharded decode
        B, S, Hq, Hkv, D, bs = 5, 2048, 8, 2, 128, 64
        attn = LocalStrideSparseAttention.__wrapped__(Hq, S, bs, 4, 4, num_kv_heads=Hkv, seq_dim=1)
        bm = O.block_mask(Hq, S, bs, 4, 4, num_kv_heads=Hkv)
        scale = 1.0 / math.sqrt(D)
        dec = ShardedDecoder(attn, B, Hq, D, torch.bfloat16, dev)
        for step in range(3):
            g = torch.Generator().manual_seed(50 + step)            # the same data on every rank
            q = torch.randn((B, 1, Hq, D), generator=g).to(torch.bfloat16)
            k = torch.randn((B, S, Hkv, D), generator=g).to(torch.bfloat16)
            v = torch.randn((B, S, Hkv, D), generator=g).to(torch.bfloat16)
            lens = torch.randint(1, S + 1, (B,), generator=g)
            lens[step] = S
            left = S - lens
            ref, ref_lse = O.decode_attention(q.float(), k.float(), v.float(), bm, bs, left_paddings=left)
            with torch.no_grad():
                one, one_lse = attn(q.to(dev), k.to(dev), v.to(dev), left_paddings=left.to(dev), return_lse=True)
            lo, hi = kv_shard_ranges(lens, rank, world, bs)
            ks, vs, n = pack_kv_shard(k, v, left, lo, hi)
            args = (q.to(dev), ks.to(dev), vs.to(dev), n.int().to(dev), lo.int().to(dev), lens.int().to(dev), scale)
            out_x, lse_x = dec.step(*args)
            out_n, lse_n = sharded_decode(attn, *args)
            torch.cuda.synchronize()
            assert _lib.wait_status() == 0, "a bounded wait gave up"
            for out, lse, name in ((out_x, lse_x, "peer-store"), (out_n, lse_n, "all-gather")):
                assert (out.float().cpu() - ref).abs().max().item() <= 2e-2, f"{name} step {step}: output"
                assert (lse.cpu().unsqueeze(-1) - ref_lse).abs().max().item() <= 1e-3, f"{name} step {step}: lse"
                assert (out.float() - one.float()).abs().max().item() <= 2e-2
            assert torch.equal(out_x, out_n) or (out_x.float() - out_n.float()).abs().max().item() <= 4e-3
            # block-cyclic shards (block j of a sequence on rank j % world)
            kc, vc, nc = pack_kv_shard_cyclic(k, v, left, lens, rank, world, bs)
            cargs = (q.to(dev), kc.to(dev), vc.to(dev), nc.int().to(dev), None, lens.int().to(dev), scale)
            out_c, lse_c = dec.step(*cargs, cyclic=True)
            out_cn, lse_cn = sharded_decode(attn, *cargs, cyclic=True)
            torch.cuda.synchronize()
            assert _lib.wait_status() == 0
            for out, lse, name in ((out_c, lse_c, "cyclic peer-store"), (out_cn, lse_cn, "cyclic all-gather")):
                assert (out.float().cpu() - ref).abs().max().item() <= 2e-2, f"{name} step {step}: output"
                assert (lse.cpu().unsqueeze(-1) - ref_lse).abs().max().item() <= 1e-3, f"{name} step {step}: lse"
        # graph replay of the peer-store route: the step counter lives in the exchange buffer
        out_g = torch.empty_like(out_x)
        lse_g = torch.empty_like(lse_x)
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            dec.step(*args, out=out_g, lse=lse_g)
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                dec.step(*args, out=out_g, lse=lse_g)
        for _ in range(3):
            out_g.zero_()
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out_g, out_x) and torch.equal(lse_g, lse_x)
        assert _lib.wait_status() == 0

        # ---------------------------------------------------------------- ring attention
        B, S, H, Hkv, D = 1, 2048, 4, 2, 128
        g = torch.Generator().manual_seed(77)
        q, k, v, do = (torch.randn((B, S, hh, D), generator=g).to(torch.bfloat16).to(dev)
                       for hh in (H, Hkv, Hkv, H))
        full = LocalStrideSparseAttention.__wrapped__(H, S, bs, 4, 4, num_kv_heads=Hkv, seq_dim=1)
        qf, kf, vf = (t.clone().requires_grad_() for t in (q, k, v))
        ref, ref_lse = full(qf, kf, vf, return_lse=True)
        ref.backward(do)
        # contiguous chunks, and the zig-zag split (two pieces per rank, balanced under the causal mask)
        for zigzag in (False, True):
            cp = ContextParallelSparseAttention(H, S, bs, 4, 4, num_kv_heads=Hkv, seq_dim=1, zigzag=zigzag)
            pieces = zigzag_bounds(S, world, bs)[rank] if zigzag else [cp.bounds[rank]]
            mine = torch.cat([torch.arange(a, b_) for a, b_ in pieces]).to(dev)
            ql, kl, vl = (t[:, mine].clone().requires_grad_() for t in (q, k, v))
            out, lse = cp(ql, kl, vl, return_lse=True)
            out.backward(do[:, mine])
            torch.cuda.synchronize()
            assert _lib.wait_status() == 0
            assert (out.float() - ref[:, mine].float()).abs().max().item() <= 2e-2, f"zigzag={zigzag}"
            assert (lse - ref_lse[:, :, mine]).abs().max().item() <= 1e-3, f"zigzag={zigzag}"
            for got, want, name in ((ql.grad, qf.grad, "dq"), (kl.grad, kf.grad, "dk"), (vl.grad, vf.grad, "dv")):
                w = want[:, mine].float()
                rel = ((got.float() - w).norm() / w.norm()).item()
                assert rel <= 5e-2, f"ring {name} (zigzag={zigzag}): relative norm error {rel:.3e}"
            with torch.no_grad():
                out2 = cp(ql, kl, vl)
            assert (out2.float() - out.float()).abs().max().item() <= 1e-6
        ret[rank] = "ok"
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_sharded_decode_and_ring_attention_on_several_gpus(world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    assert dict(ret) == {r: "ok" for r in range(world)}
