"""Single-node multi-GPU partitioning (one process per GPU, torch.distributed).

Three schemes, matching what the attention path allows:

* **Head sharding** -- heads are independent, so a rank owns a contiguous range of
  q heads (whole kv groups) and builds its module with ``active_head_range``
  (dkernel/interface.py:293-298).  No collective is involved.
* **KV-sequence sharding for decode** -- every rank holds a block-aligned slice
  of each sequence's keys/values, computes a partial (O, LSE) with the decode
  kernel, and the partials are merged with the semantics of
  ``combine_attn_partitions`` (dkernel/interface.py:319-324).  Two exchange
  routes: ``ShardedDecoder`` (one fused kernel per rank that stores the partial
  rows straight into every peer's buffer over NVLink and merges as soon as the
  peers' rows have landed; no collective library on the data path) and
  ``sharded_decode`` (one NCCL all-gather + the fused merge kernel).
* **Context-parallel (ring) prefill / training** -- the sequence is cut into one
  chunk per rank; K/V chunks travel round the ring while every rank attends its
  q chunk to the chunk it currently holds, partial results are merged by LSE, and in
  the backward pass each rank sends its dK/dV contribution for a chunk straight to the
  chunk's owner.  This is the multi-GPU form of what the
  reference simulates on one GPU in tests/test_seq_partition.py:83-139.

The planning functions and the ring schedule are pure Python / torch so that they
run under the gloo backend on CPU; only the compute callbacks touch the GPU.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Callable, Dict, List, Optional, Tuple

import torch
import torch.distributed as dist
from torch import Tensor


# --------------------------------------------------------------------------- head sharding
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


# --------------------------------------------------------------------------- KV-sharded decode
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


def kv_shard_cyclic_blocks(lens: Tensor, rank: int, world: int, block_size: int) -> Tensor:
    """Stored tokens per sequence of ``rank`` under block-cyclic sharding: block j of a sequence
    (positions re-based to its first token) lives on rank j % world, as local block j // world.
    A window of consecutive blocks -- the bulk of a local-stride row -- then spreads evenly over
    the ranks, where a split into contiguous position ranges leaves it all on the last one."""
    lens = lens.to(torch.int64)
    nblk = (lens + block_size - 1) // block_size
    mine = (nblk - rank + world - 1) // world                 # blocks j < nblk with j % world == rank
    mine = mine.clamp_min(0)
    last_is_mine = (nblk > 0) & ((nblk - 1) % world == rank)
    tail = lens - (nblk - 1) * block_size                     # tokens of the last block
    return torch.where(last_is_mine, (mine - 1) * block_size + tail, mine * block_size)


def pack_kv_shard_cyclic(k: Tensor, v: Tensor, left_paddings: Tensor, lens: Tensor, rank: int, world: int,
                         block_size: int, capacity: Optional[int] = None) -> Tuple[Tensor, Tensor, Tensor]:
    """Cut the block-cyclic shard of ``rank`` out of left-padded (B,S,Hkv,D) K/V buffers into
    left-aligned (B,capacity,Hkv,D) buffers.  Returns (k_shard, v_shard, n) with n the stored
    tokens per sequence.  Host-side data preparation for tests and benchmarks (a serving system
    appends block j of a sequence to rank j % world directly)."""
    B, S = k.size(0), k.size(1)
    n = kv_shard_cyclic_blocks(lens, rank, world, block_size)
    cap = capacity if capacity is not None else max(int(n.max().item()), 1)
    ks = k.new_zeros((B, cap) + tuple(k.shape[2:]))
    vs = v.new_zeros((B, cap) + tuple(v.shape[2:]))
    for b in range(B):
        L, left = int(lens[b]), int(left_paddings[b])
        pos = torch.arange(L, device=k.device)
        sel = pos[(pos // block_size) % world == rank] + left
        ks[b, :sel.numel()] = k[b, sel]
        vs[b, :sel.numel()] = v[b, sel]
    return ks, vs, n


def partial_row_bytes(d: int, elem_size: int = 2) -> int:
    """Bytes of one packed partial row: d 16-bit outputs followed by the fp32 LSE."""
    return d * elem_size + 4


def packed_partial_views(packed: Tensor, d: int, dtype: torch.dtype) -> Tuple[Tensor, Tensor]:
    """Views into a (rows, partial_row_bytes) uint8 buffer: the (rows, d) outputs in ``dtype``
    (row stride d + 2 elements) and the (rows,) fp32 LSE column.  The decode kernel writes its
    results straight through these views, so that ONE message carries both."""
    assert packed.dtype == torch.uint8 and packed.dim() == 2 and packed.size(1) == partial_row_bytes(d)
    o_view = packed[:, :2 * d].view(dtype)
    lse_view = packed[:, 2 * d:].view(torch.float32)[:, 0]
    return o_view, lse_view


def gather_packed_partials(packed: Tensor, group=None) -> Tensor:
    """All-gather of every rank's packed partial rows: (world * rows, row_bytes) uint8, rank-major."""
    world = dist.get_world_size(group)
    gathered = torch.empty((world * packed.size(0), packed.size(1)), dtype=torch.uint8, device=packed.device)
    dist.all_gather_into_tensor(gathered, packed, group=group)
    return gathered


def split_gathered_partials(gathered: Tensor, world: int, d: int, dtype: torch.dtype
                            ) -> Tuple[Tensor, Tensor]:
    """(o_parts (world, rows, d) in ``dtype``, lse_parts (world, rows) fp32) as strided views of a
    gathered packed buffer (no copy)."""
    rows = gathered.size(0) // world
    o, lse = packed_partial_views(gathered, d, dtype)
    return o.unflatten(0, (world, rows)), lse.unflatten(0, (world, rows))


def sharded_decode(attn, q: Tensor, k_shard: Tensor, v_shard: Tensor, n_local: Tensor,
                   pos0: Optional[Tensor], total_len: Tensor, sm_scale: Optional[float] = None,
                   group=None, cyclic: bool = False) -> Tuple[Tensor, Tensor]:
    """One decode step with the KV sequence sharded over the ranks of ``group``, exchanged by
    ONE NCCL all-gather (the portable route; ``ShardedDecoder`` is the faster one).

    attn: a SparseAttention module (its pattern covers the full sequence).
    q: (B,1,Hq,D) replicated on every rank.  k_shard/v_shard: (B,cap,Hkv,D) this
    rank's left-aligned slice; n_local (B,) stored tokens; pos0 (B,) position of the
    first stored token (multiple of the block size); total_len (B,) full lengths
    (int32 device tensors are used as they are).  With ``cyclic=True`` the shard is block-cyclic
    (``pack_kv_shard_cyclic``) and pos0 is ignored.
    Returns the merged (out (B,1,Hq,D), lse (B,Hq)) on every rank.

    Per step: the decode kernel (+ its split merge) writes this rank's partial O (input
    dtype) and LSE (fp32) side by side into one byte buffer of (B*Hq) rows of 2*D+4 bytes,
    one all-gather moves it, and the fused merge kernel reads the gathered rows in place."""
    from . import _lib
    from .ops import decode
    B, _, Hq, D = q.shape
    rows, row_bytes = B * Hq, partial_row_bytes(D)
    assert q.element_size() == 2, "sharded decode packs 16-bit partial outputs"
    scale = sm_scale or 1.0 / math.sqrt(D)
    world = dist.get_world_size(group)
    packed = torch.empty((rows, row_bytes), dtype=torch.uint8, device=q.device)
    o_view, lse_view = packed_partial_views(packed, D, q.dtype)
    decode(q, k_shard, v_shard, attn._plan(), scale, seq_dim=1, k_start=None,
           k_end=_as_i32(n_local, q.device), k_pos0=None if cyclic else _as_i32(pos0, q.device),
           k_total=_as_i32(total_len, q.device), out=o_view, lse_out=lse_view,
           k_blk=(world, dist.get_rank(group)) if cyclic else None)
    gathered = gather_packed_partials(packed, group)
    merged = torch.empty((B, 1, Hq, D), dtype=q.dtype, device=q.device)
    mlse = torch.empty((B, Hq), dtype=torch.float32, device=q.device)
    elems, floats = row_bytes // 2, row_bytes // 4
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().bsa_merge_partials(
            _lib.ptr(gathered), gathered.data_ptr() + 2 * D, world, rows, D, rows * elems, elems,
            rows * floats, floats, _lib.ptr(merged), D, _lib.ptr(mlse), _lib.dtype_code(q.dtype),
            _lib.stream_of(q)), "bsa_merge_partials")
    return merged, mlse


def _as_i32(t: Optional[Tensor], device) -> Optional[Tensor]:
    if t is None:
        return None
    return t.to(device=device, dtype=torch.int32).contiguous()   # no-op for int32 device tensors


class ShardedDecoder:
    """KV-sharded decode whose exchange step is the library's own kernel over peer memory.

    Construction (collective over ``group``, once): every rank allocates an exchange buffer in
    torch's symmetric memory and maps the buffers of all ranks of the node.  A step is then
    two launches on the caller's stream and no host synchronisation: the decode kernel leaves this
    rank's split-KV partials in its workspace, and ``bsa_xchg_merge`` (launched as its programmatic
    dependent) merges the splits, stores the rank's (O, LSE) rows into every rank's exchange buffer
    over NVLink, waits (bounded) for the peers' rows to land in the local buffer and merges them.  All ranks must call
    ``step`` the same number of times.  The call can be captured in a CUDA graph and replayed."""

    def __init__(self, attn, batch: int, num_heads: int, head_dim: int, dtype: torch.dtype,
                 device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        from . import _lib
        assert dtype in (torch.float16, torch.bfloat16), "sharded decode exchanges 16-bit partial outputs"
        self.attn, self.group = attn, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.B, self.Hq, self.D, self.dtype = batch, num_heads, head_dim, dtype
        self.rows = batch * num_heads
        nbytes = _lib.lib().bsa_xchg_buffer_bytes(self.world, self.rows, head_dim)
        assert nbytes > 0, "unsupported exchange geometry (at most 8 ranks, head dim a multiple of 8)"
        self.xbuf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.xbuf.zero_()
        torch.cuda.synchronize(device)
        grp = group if group is not None else dist.group.WORLD
        self.handle = symm_mem.rendezvous(self.xbuf, grp)
        self.peer_ptrs = [int(p) for p in self.handle.buffer_ptrs]
        assert len(self.peer_ptrs) == self.world and self.peer_ptrs[self.rank] == self.xbuf.data_ptr()
        dist.barrier(group)      # every buffer is zeroed before anyone's first push can arrive

    def step(self, q: Tensor, k_shard: Tensor, v_shard: Tensor, n_local: Tensor, pos0: Optional[Tensor],
             total_len: Tensor, sm_scale: Optional[float] = None,
             out: Optional[Tensor] = None, lse: Optional[Tensor] = None, cyclic: bool = False
             ) -> Tuple[Tensor, Tensor]:
        """Arguments as for ``sharded_decode``; returns the merged (out (B,1,Hq,D), lse (B,Hq))."""
        from . import _lib
        from .ops import decode
        B, _, Hq, D = q.shape
        assert (B, Hq, D) == (self.B, self.Hq, self.D) and q.dtype == self.dtype
        scale = sm_scale or 1.0 / math.sqrt(D)
        part_o, part_lse = decode(q, k_shard, v_shard, self.attn._plan(), scale, seq_dim=1, k_start=None,
                                  k_end=_as_i32(n_local, q.device),
                                  k_pos0=None if cyclic else _as_i32(pos0, q.device),
                                  k_total=_as_i32(total_len, q.device),
                                  k_blk=(self.world, self.rank) if cyclic else None, partials_only=True)
        merged = out if out is not None else torch.empty((B, 1, Hq, D), dtype=q.dtype, device=q.device)
        mlse = lse if lse is not None else torch.empty((B, Hq), dtype=torch.float32, device=q.device)
        assert merged.is_contiguous() and mlse.is_contiguous()
        p = _lib.XchgParams()
        p.part_o, p.part_lse, p.nsplit = _lib.ptr(part_o), _lib.ptr(part_lse), part_o.size(1)
        p.out, p.out_lse = _lib.ptr(merged), _lib.ptr(mlse)
        for w in range(self.world):
            p.xbuf[w] = self.peer_ptrs[w]
        p.rows, p.world, p.rank, p.d = self.rows, self.world, self.rank, D
        p.dtype = _lib.dtype_code(q.dtype)
        with torch.cuda.device(q.device):
            _lib.check(_lib.lib().bsa_xchg_merge(C.byref(p), _lib.stream_of(q)), "bsa_xchg_merge")
        return merged, mlse


# --------------------------------------------------------------------------- context parallelism
def chunk_bounds(seq_len: int, world: int, block_size: int) -> List[Tuple[int, int]]:
    """Contiguous position ranges, one per rank: equal chunks, multiples of the block size."""
    assert seq_len % world == 0 and (seq_len // world) % block_size == 0, \
        f"sequence length {seq_len} must split into {world} chunks that are multiples of {block_size}"
    c = seq_len // world
    return [(r * c, (r + 1) * c) for r in range(world)]


def zigzag_bounds(seq_len: int, world: int, block_size: int) -> List[List[Tuple[int, int]]]:
    """Two position ranges per rank: the sequence is cut into 2 * world equal pieces and rank r owns
    pieces r and 2 * world - 1 - r (its local tensors are the two pieces back to back).  Under a
    causal mask every rank then has the same share of the work, which contiguous chunks do not
    give (there the last rank attends everything and the first only itself)."""
    assert seq_len % (2 * world) == 0 and (seq_len // (2 * world)) % block_size == 0, \
        f"sequence length {seq_len} must split into {2 * world} pieces that are multiples of {block_size}"
    c = seq_len // (2 * world)
    return [[(r * c, (r + 1) * c), ((2 * world - 1 - r) * c, (2 * world - r) * c)] for r in range(world)]


def zigzag_shard(x: Tensor, rank: int, world: int, block_size: int, seq_dim: int = 1) -> Tensor:
    """This rank's part of a whole-sequence tensor under the zig-zag split (for tests and loaders)."""
    (a0, a1), (b0, b1) = zigzag_bounds(x.size(seq_dim), world, block_size)[rank]
    return torch.cat([x.narrow(seq_dim, a0, a1 - a0), x.narrow(seq_dim, b0, b1 - b0)], seq_dim).contiguous()


def ring_steps(rank: int, world: int, causal: bool = True) -> List[Tuple[int, int, bool]]:
    """The ring schedule of one rank: [(step, kv_chunk, active)].  At step t the rank holds kv
    chunk (rank - t) mod world (its own at t = 0; chunks arrive from the previous rank); with a
    causal mask over contiguous chunks only chunks at or before the rank's own q chunk are computed
    (pass causal=False for the zig-zag split, where every pair of ranks has visible pieces)."""
    return [(t, (rank - t) % world, (not causal) or ((rank - t) % world) <= rank) for t in range(world)]


def _ring_exchange(send: Tensor, recv: Tensor, group) -> list:
    """Post "send to the next rank, receive from the previous one"; returns the requests."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    nxt = dist.get_global_rank(group, (rank + 1) % world) if group is not None else (rank + 1) % world
    prv = dist.get_global_rank(group, (rank - 1) % world) if group is not None else (rank - 1) % world
    ops = [dist.P2POp(dist.isend, send, nxt, group), dist.P2POp(dist.irecv, recv, prv, group)]
    return dist.batch_isend_irecv(ops)


def ring_forward(q: Tensor, k: Tensor, v: Tensor, forward_chunk: Callable, merge: Callable,
                 group=None, causal: bool = True):
    """Forward pass of ring attention for this rank's q chunk.

    forward_chunk(q, k_s, v_s, r, s) -> (o, lse) attends q (chunk r) to kv chunk s;
    merge(list of (o, lse)) -> (out, lse) combines the partial results.
    The K/V chunk for the next step is received while the current one is computed."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    kv = torch.stack([k, v]).contiguous()
    parts = []
    for t, s, active in ring_steps(rank, world, causal):
        reqs, nxt = [], None
        if t < world - 1:
            nxt = torch.empty_like(kv)
            reqs = _ring_exchange(kv, nxt, group)
        if active:
            parts.append(forward_chunk(q, kv[0], kv[1], rank, s))
        for r_ in reqs:
            r_.wait()
        if nxt is not None:
            kv = nxt
    return merge(parts)


def ring_backward(q: Tensor, k: Tensor, v: Tensor, o: Tensor, lse: Tensor, do: Tensor,
                  dlse: Optional[Tensor], backward_chunk: Callable, group=None, causal: bool = True):
    """Backward pass of ring attention.  backward_chunk(q, k_s, v_s, o, lse, do, dlse, r, s) ->
    (dq, dk_s, dv_s) evaluates the gradients of the (r, s) chunk pair from the MERGED output and
    LSE of the forward pass (the probabilities exp(S - lse) are then already globally normalised,
    so the pair's contributions simply add up).  dQ accumulates locally in fp32.  The K/V chunks
    travel round the ring as in the forward pass; the dK/dV contribution a rank computes for
    another rank's chunk is sent straight to that rank (one message per chunk pair, in the
    gradients' own dtype) while the next pair is computed; the owner adds the messages to its fp32
    accumulator in step order, so the result does not depend on timing."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    peer = (lambda r_: dist.get_global_rank(group, r_)) if group is not None else (lambda r_: r_)
    kv = torch.stack([k, v]).contiguous()
    dkv = torch.zeros(kv.shape, dtype=torch.float32, device=kv.device)
    dq = torch.zeros(q.shape, dtype=torch.float32, device=q.device)
    pending = None      # (requests, received contribution, sent tensor) of the previous step's messages

    def settle(p):
        # the previous step's dK/dV messages travelled while this step's pair was computed
        if p is None:
            return
        for r_ in p[0]:
            r_.wait()
        if p[1] is not None:
            dkv.add_(p[1])

    for t, s, active in ring_steps(rank, world, causal):
        reqs, nxt = [], None
        if t < world - 1:
            nxt = torch.empty_like(kv)
            reqs = _ring_exchange(kv, nxt, group)
        part = None
        if active:
            dq_p, dk_p, dv_p = backward_chunk(q, kv[0], kv[1], o, lse, do, dlse, rank, s)
            dq += dq_p
            if t == 0:
                dkv[0] += dk_p
                dkv[1] += dv_p
            else:
                part = torch.stack([dk_p, dv_p])
        settle(pending)
        # this step's chunk belongs to rank s; the rank that holds MY chunk now is (rank + t) % world
        src = (rank + t) % world
        src_active = t > 0 and ((not causal) or rank <= src)     # does it compute a pair with my chunk?
        ops, got = [], None
        if part is not None:
            ops.append(dist.P2POp(dist.isend, part, peer(s), group))
        if src_active:
            got = torch.empty((2,) + tuple(k.shape), dtype=k.dtype, device=k.device)
            ops.append(dist.P2POp(dist.irecv, got, peer(src), group))
        pending = (dist.batch_isend_irecv(ops) if ops else [], got, part)
        for r_ in reqs:
            r_.wait()
        if nxt is not None:
            kv = nxt
    settle(pending)
    return dq.to(q.dtype), dkv[0].to(k.dtype), dkv[1].to(v.dtype)


class _RingAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, owner):
        out, lse = ring_forward(q, k, v, owner._forward_chunk, owner._merge, owner.group, owner.skip_later_chunks)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.owner = owner
        return out, lse

    @staticmethod
    def backward(ctx, do, dlse):
        q, k, v, out, lse = ctx.saved_tensors
        owner = ctx.owner
        if dlse is not None and not bool((dlse != 0).any()):
            dlse = None
        dq, dk, dv = ring_backward(q, k, v, out, lse, do.contiguous(), dlse, owner._backward_chunk,
                                   owner.group, owner.skip_later_chunks)
        return dq, dk, dv, None


class ContextParallelSparseAttention(torch.nn.Module):
    """Local-stride block-sparse attention over a sequence that is split across the ranks of a
    process group (one contiguous chunk of q, k and v per rank, or with ``zigzag=True`` the two
    pieces of ``zigzag_bounds`` back to back, which balances a causal mask), forward and backward.

    Rank r attends its q chunk to kv chunk s through a ``SparseAttention`` built on the block mask
    of that chunk pair (``get_sparse_attn_mask`` with ``q_start_position`` / ``kv_start_position``,
    dkernel/utils.py:161-169,185-191), causal only on the diagonal pair; the K/V chunks travel
    round the ring over NCCL send/recv while the previous pair is computed, partial results are
    merged by LSE, and the backward pass sends every dK/dV contribution to the owner of its chunk.

    forward(q, k, v, sm_scale=None, return_lse=False): tensors are this rank's chunk,
    (B, S/world, H, D) for ``seq_dim=1`` or (B, H, S/world, D) for ``seq_dim=2``."""

    def __init__(self, num_heads: int, seq_len: int, block_size: int, local_blocks: int,
                 vert_stride: int, *, num_kv_heads: Optional[int] = None, homo_head: bool = False,
                 head_sliding_offset: int = 0, seq_dim: int = 1, causal: bool = True, group=None,
                 zigzag: bool = False, **kwargs):
        super().__init__()
        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.zigzag = bool(zigzag) and causal
        # per rank: one position range, or two with the zig-zag split
        self.pieces = (zigzag_bounds(seq_len, self.world, block_size) if self.zigzag
                       else [[b] for b in chunk_bounds(seq_len, self.world, block_size)])
        self.bounds = [p[0] for p in self.pieces] if not self.zigzag else None
        self.mask_args = dict(num_heads=num_heads, block_size=block_size, local_blocks=local_blocks,
                              vert_stride=vert_stride, homo_head=homo_head, num_kv_heads=num_kv_heads,
                              head_sliding_offset=head_sliding_offset, causal=causal)
        self.block_size, self.seq_dim, self.causal, self.kwargs = block_size, seq_dim, causal, kwargs
        self._chunks: Dict[int, object] = {}
        self._scale = None
        # contiguous chunks under a causal mask: kv chunks after the own q chunk are skipped
        self.skip_later_chunks = causal and not self.zigzag

    def _module(self, s: int):
        """SparseAttention of the (own q chunk, kv chunk s) pair, built on first use."""
        if s not in self._chunks:
            from .interface import SparseAttention
            from .utils import get_sparse_attn_mask
            a = self.mask_args

            def piece_mask(qr, kr):
                (q0, q1), (k0, k1) = qr, kr
                return get_sparse_attn_mask(a["num_heads"], q1 - q0, a["block_size"], a["local_blocks"],
                                            a["vert_stride"], homo_head=a["homo_head"], dtype=torch.uint8,
                                            num_kv_heads=a["num_kv_heads"],
                                            head_sliding_offset=a["head_sliding_offset"], causal=a["causal"],
                                            q_start_position=q0, kv_start_position=k0, kv_seqlen=k1 - k0)[1]
            # Block mask of (own pieces) x (pieces of rank s), stitched from the pieces' masks.  A kv
            # piece that lies after a q piece is invisible under a causal mask.  Own pair: the
            # pieces are in position order locally, so the kernel's own causal test on local
            # indices is the right one (the diagonal pieces get it, the later-q / earlier-kv piece
            # passes it whole, the earlier-q / later-kv piece fails it whole); other pairs have no
            # diagonal piece and run without it.
            rows = []
            for qr in self.pieces[self.rank]:
                row = []
                for kr in self.pieces[s]:
                    m = piece_mask(qr, kr)
                    if self.causal and kr[0] > qr[0]:
                        m = torch.zeros_like(m)
                    row.append(m)
                rows.append(torch.cat(row, -1))
            bmask = torch.cat(rows, -2).contiguous()
            self._chunks[s] = SparseAttention(self.block_size, bmask, seq_dim=self.seq_dim,
                                              causal=self.causal and s == self.rank, **self.kwargs)
        return self._chunks[s]

    def _forward_chunk(self, q, k, v, r, s):
        from . import ops
        mod = self._module(s)
        impl = ops._IMPL_NAMES[mod.kwargs.get("impl", None)]
        return ops._train_forward(None, q, k, v, self._scale, mod._plan(), self.seq_dim,
                                  mod.kwargs["causal"], None, impl, need_lse=True, inference=True)

    def _backward_chunk(self, q, k, v, o, lse, do, dlse, r, s):
        from types import SimpleNamespace
        from . import ops
        mod = self._module(s)
        name = mod.kwargs.get("bwd_impl", "generic" if mod.kwargs.get("impl") == "generic" else None)
        ctx = SimpleNamespace(saved_tensors=(q, k, v, o, lse), sm_scale=self._scale, seq_dim=self.seq_dim,
                              causal=mod.kwargs["causal"], plan=mod._plan(), bwd_impl=ops._IMPL_NAMES[name])
        return ops._backward(ctx, do, dlse)

    def _merge(self, parts):
        from .interface import combine_attn_partitions
        if len(parts) == 1:
            return parts[0]
        return combine_attn_partitions(*parts, hdim=3 - self.seq_dim, return_lse=True)

    def forward(self, q: Tensor, k: Tensor, v: Tensor, sm_scale: Optional[float] = None,
                return_lse: bool = False):
        from . import ops
        ops._check_inputs(q, k, v)
        self._scale = sm_scale or 1.0 / math.sqrt(float(q.size(-1)))
        q, k, v = (ops._tma_friendly(t.contiguous()) for t in (q, k, v))
        if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad):
            out, lse = _RingAttention.apply(q, k, v, self)
        else:
            out, lse = ring_forward(q, k, v, self._forward_chunk, self._merge, self.group, self.skip_later_chunks)
        return (out, lse) if return_lse else out


__all__ = ["head_shard", "kv_shard_ranges", "pack_kv_shard", "kv_shard_cyclic_blocks", "pack_kv_shard_cyclic",
           "sharded_decode", "ShardedDecoder",
           "chunk_bounds", "zigzag_bounds", "zigzag_shard", "ring_steps", "ring_forward", "ring_backward",
           "ContextParallelSparseAttention"]
