"""Single-node multi-GPU partitioning (one process per GPU, torch.distributed).

Two schemes, matching what the attention path allows:

* **Head sharding** -- heads are independent, so a rank owns a contiguous range of
  q heads (whole kv groups) and builds its module with ``active_head_range``
  (dkernel/interface.py:293-298).  No collective is involved.
* **KV-sequence sharding for decode** -- every rank holds a block-aligned slice
  of each sequence's keys/values, computes a partial (O, LSE) with the decode
  kernel and the partials are merged after ONE all-gather (NCCL over NVLink on
  GPUs) with the semantics of ``combine_attn_partitions``
  (dkernel/interface.py:319-324).

The planning functions are pure Python / CPU torch so that they can be tested
with the gloo backend; only ``sharded_decode`` touches the GPU.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


def head_shard(num_heads: int, num_kv_heads: Optional[int], rank: int, world: int
               ) -> Tuple[Tuple[int, int], Tuple[int, int]]:
    """((q_head_start, q_head_end), (kv_head_start, kv_head_end)) of ``rank``.
    Whole kv groups stay on one rank, so ``world`` must divide the kv head count."""
    num_kv_heads = num_kv_heads or num_heads
    assert num_heads % num_kv_heads == 0
    assert num_kv_heads % world == 0, \
        f"{num_kv_heads} kv heads cannot be split over {world} ranks without breaking a group"
    g = num_heads // num_kv_heads
    per = num_kv_heads // world
    kv0, kv1 = rank * per, (rank + 1) * per
    return (kv0 * g, kv1 * g), (kv0, kv1)


def kv_shard_ranges(lens: Tensor, rank: int, world: int, block_size: int) -> Tuple[Tensor, Tensor]:
    """Position range [lo, hi) of every sequence owned by ``rank``: the blocks of
    each sequence are dealt out proportionally, so all ranks hold about 1/world
    of *every* sequence (a split of the left-padded storage instead would put
    short sequences entirely on the last rank).  ``lens``: (B,) integer tensor.
    Boundaries are multiples of ``block_size``; hi is clipped to the length."""
    lens = lens.to(torch.int64)
    nblk = (lens + block_size - 1) // block_size
    lo = (nblk * rank // world) * block_size
    hi = torch.minimum((nblk * (rank + 1) // world) * block_size, lens)
    hi = torch.maximum(hi, lo)
    return lo, hi


def pack_kv_shard(k: Tensor, v: Tensor, left_paddings: Tensor, lo: Tensor, hi: Tensor,
                  capacity: Optional[int] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """Cut the shard [lo, hi) of every sequence out of left-padded (B,S,Hkv,D)
    K/V buffers into left-aligned (B,capacity,Hkv,D) buffers.  Returns
    (k_shard, v_shard, n) with n = hi - lo.  Host-side data preparation for tests
    and benchmarks (a serving system would write its shard in place)."""
    B = k.size(0)
    n = (hi - lo).clamp_min(0)
    cap = capacity if capacity is not None else max(int(n.max().item()), 1)
    ks = k.new_zeros((B, cap) + tuple(k.shape[2:]))
    vs = v.new_zeros((B, cap) + tuple(v.shape[2:]))
    for b in range(B):
        s0 = int(left_paddings[b].item() + lo[b].item())
        nb = int(n[b].item())
        ks[b, :nb] = k[b, s0:s0 + nb]
        vs[b, :nb] = v[b, s0:s0 + nb]
    return ks, vs, n


def gather_partials(o: Tensor, lse: Tensor, group=None) -> Tuple[Tensor, Tensor]:
    """All-gather one rank's partial (o: (rows, D) any float dtype, lse: (rows,)
    fp32) into (world, rows, D) / (world, rows).  O and LSE travel in ONE message:
    they are packed into a single fp32 buffer (rows, D+1) so that a decode step
    costs one collective."""
    world = dist.get_world_size(group)
    rows, D = o.shape
    packed = torch.empty((rows, D + 1), dtype=torch.float32, device=o.device)
    packed[:, :D] = o
    packed[:, D] = lse
    out = torch.empty((world * rows, D + 1), dtype=torch.float32, device=o.device)
    dist.all_gather_into_tensor(out, packed, group=group)
    out = out.view(world, rows, D + 1)
    return out[:, :, :D], out[:, :, D]


def merge_gathered(o_parts: Tensor, lse_parts: Tensor, out_dtype: torch.dtype
                   ) -> Tuple[Tensor, Tensor]:
    """Merge gathered partials ((P, rows, D) fp32 strided views and (P, rows)) with
    the fused CUDA kernel (bsa_merge_partials).  Returns (o (rows, D) in
    ``out_dtype``, lse (rows,))."""
    import ctypes as C  # noqa: F401
    from . import _lib
    P, rows, D = o_parts.shape
    _lib.require_cuda(o_parts, "gathered partials")
    assert o_parts.dtype == torch.float32 and o_parts.stride(2) == 1
    lse_c = lse_parts.contiguous()
    res32 = torch.empty((rows, D), dtype=torch.float32, device=o_parts.device)
    lse = torch.empty((rows,), dtype=torch.float32, device=o_parts.device)
    with torch.cuda.device(o_parts.device):
        _lib.check(_lib.lib().bsa_merge_partials(
            _lib.ptr(o_parts), _lib.ptr(lse_c), P, rows, D, o_parts.stride(0), o_parts.stride(1),
            lse_c.stride(0), 1, _lib.ptr(res32), D, _lib.ptr(lse), _lib.BSA_F32,
            _lib.stream_of(o_parts)), "bsa_merge_partials")
    return res32.to(out_dtype), lse


def _as_i32(t: Optional[Tensor], device) -> Optional[Tensor]:
    if t is None:
        return None
    return t.to(device=device, dtype=torch.int32).contiguous()   # no-op for int32 device tensors


def sharded_decode(attn, q: Tensor, k_shard: Tensor, v_shard: Tensor, n_local: Tensor,
                   pos0: Tensor, total_len: Tensor, sm_scale: Optional[float] = None,
                   group=None) -> Tuple[Tensor, Tensor]:
    """One decode step with the KV sequence sharded over the ranks of ``group``.

    attn: a SparseAttention module (its pattern covers the full sequence).
    q: (B,1,Hq,D) replicated on every rank.  k_shard/v_shard: (B,cap,Hkv,D) this
    rank's left-aligned slice; n_local (B,) stored tokens; pos0 (B,) position of the
    first stored token (multiple of the block size); total_len (B,) full lengths
    (int32 device tensors are used as they are).
    Returns the merged (out (B,1,Hq,D), lse (B,Hq)) on every rank.

    Per step: the decode kernel (+ its split merge) writes this rank's partial O (input
    dtype) and LSE (fp32) side by side into one byte buffer of (B*Hq) rows of 2*D+4 bytes,
    ONE all-gather moves it, and the fused merge kernel reads the gathered rows in place."""
    import math
    from . import _lib
    from .ops import decode
    B, _, Hq, D = q.shape
    rows, row_bytes = B * Hq, 2 * D + 4
    assert q.element_size() == 2, "sharded decode packs 16-bit partial outputs"
    scale = sm_scale or 1.0 / math.sqrt(D)
    world = dist.get_world_size(group)
    packed = torch.empty((rows, row_bytes), dtype=torch.uint8, device=q.device)
    o_view = packed[:, :2 * D].view(q.dtype)                 # (rows, D), row stride D + 2 elements
    lse_view = packed[:, 2 * D:].view(torch.float32)[:, 0]   # (rows,), row stride (2*D+4)/4 floats
    decode(q, k_shard, v_shard, attn._plan(), scale, seq_dim=1, k_start=None,
           k_end=_as_i32(n_local, q.device), k_pos0=_as_i32(pos0, q.device),
           k_total=_as_i32(total_len, q.device), out=o_view, lse_out=lse_view)
    gathered = torch.empty((world * rows, row_bytes), dtype=torch.uint8, device=q.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    merged = torch.empty((B, 1, Hq, D), dtype=q.dtype, device=q.device)
    mlse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    elems, floats = row_bytes // 2, row_bytes // 4
    lse_parts = gathered.view(torch.float32)      # (world*rows, floats); the LSE is the last float of a row
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().bsa_merge_partials(
            _lib.ptr(gathered), lse_parts.data_ptr() + 2 * D, world, rows, D, rows * elems, elems,
            rows * floats, floats, _lib.ptr(merged), D, _lib.ptr(mlse), _lib.dtype_code(q.dtype),
            _lib.stream_of(q)), "bsa_merge_partials")
    return merged, mlse
