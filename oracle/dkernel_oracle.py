"""CPU oracle for the block-sparse attention path of linxihui/dkernel.

TEST INFRASTRUCTURE ONLY.  This file restates, on the CPU, the algorithms of
the reference package so that the CUDA path can be checked against them.  It
must never be imported by the product package; only the tests, the smoke
check and the CPU-baseline leg of the benchmark use it.

Parity status: PINNED.  ``tests/golden/`` holds vectors produced by the
reference's own code (imported from a read-only checkout by
``tests/golden/make_golden.py``): the two literal block masks of the
reference's ``tests/test_utils.py:24-34,55-64``, masks and CSR/CSC layouts for
a sweep of pattern parameters, and masked-dense attention outputs of the
reference's test oracle.  ``tests/test_oracle.py`` checks every function here
against those vectors.

Each function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import math
from typing import Optional, Sequence, Tuple, Union

import numpy as np
import torch

__all__ = [
    "cdiv", "multiple_of", "block_mask", "to_csr", "dense_to_crow_col",
    "dense_to_ccol_row", "crow_col_to_dense", "merge_split_fwd_kernel_blocks",
    "is_kv_cache_efficient", "token_mask", "masked_dense_attention",
    "block_sparse_attention", "padded_attention", "varlen_attention",
    "decode_attention", "combine_attn_partitions", "attended_tiles",
]


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def multiple_of(x: int, y: int) -> int:
    """dkernel/utils.py:323-324."""
    return ((x + y - 1) // y) * y


# ---------------------------------------------------------------------------
# Pattern generation (dkernel/utils.py:105-229)
# ---------------------------------------------------------------------------
def block_mask(num_heads: int,
               seqlen: int,
               block_size: int = 64,
               local_blocks: Union[int, Tuple[int, int]] = 4,
               vert_stride: int = 4,
               homo_head: bool = False,
               num_kv_heads: Optional[int] = None,
               past_len: Optional[int] = None,
               head_sliding_step: Optional[int] = None,
               head_sliding_offset: int = 0,
               num_dense_heads: int = 0,
               kv_seqlen: Optional[int] = None,
               q_start_position: Optional[int] = None,
               kv_start_position: Optional[int] = None,
               vert_position_type: Optional[str] = None,
               causal: bool = True) -> np.ndarray:
    """Block mask (H or 1, q_blocks - trimmed, kv_blocks) as uint8.

    Restates ``get_sparse_attn_mask`` (dkernel/utils.py:143-220): the local
    band ``(q-k < left) & (k-q < right)`` OR-ed with the vertical stripes
    ``(kv_start_block + j + h*step + offset) % vert_stride == 0`` for absolute
    positions (utils.py:187-194), or the relative variant (utils.py:196-210),
    AND-ed with ``q >= k`` when causal (utils.py:213-215), rows before
    ``cdiv(past_len, block_size)`` dropped (utils.py:219-220).
    """
    past_len = past_len or 0
    kv_seqlen = kv_seqlen or seqlen
    if homo_head:
        num_heads = 1
        assert num_dense_heads == 0
    if vert_position_type is None:
        vert_position_type = "absolute" if causal else "relative"
    assert vert_position_type in ("absolute", "relative")
    num_kv_heads = num_kv_heads or num_heads
    num_sparse_heads = num_kv_heads - num_dense_heads
    num_q_per_kv = num_heads // num_kv_heads

    q_start_block = 0
    kv_start_block = 0
    if q_start_position is not None:
        assert q_start_position % block_size == 0
        q_start_block = q_start_position // block_size
        assert past_len in (0, None)
    if kv_start_position is not None:
        assert kv_start_position % block_size == 0
        kv_start_block = kv_start_position // block_size

    if causal:
        assert local_blocks >= 1
        local = (local_blocks, 1)
    else:
        if isinstance(local_blocks, int):
            assert local_blocks >= 0
            local = (local_blocks, local_blocks)
        else:
            assert isinstance(local_blocks, tuple) and len(local_blocks) == 2
            assert all(x > 0 for x in local_blocks)
            local = local_blocks

    blocks = cdiv(seqlen, block_size)
    kv_blocks = cdiv(kv_seqlen, block_size)
    q_pos = q_start_block + np.arange(blocks, dtype=np.int64)[None, :, None]
    k_pos = kv_start_block + np.arange(kv_blocks, dtype=np.int64)[None, None]
    if head_sliding_step is None:
        head_sliding_step = max(1, int(vert_stride / num_heads))
    if vert_position_type == "absolute":
        rows = []
        for h in range(num_kv_heads):
            for _ in range(num_q_per_kv):
                if h < num_sparse_heads:
                    rows.append((kv_start_block + np.arange(kv_blocks) + h * head_sliding_step
                                 + head_sliding_offset) % vert_stride == 0)
                else:
                    rows.append(np.ones(kv_blocks, dtype=bool))
        vert = np.stack(rows)[:, None, :]
        local_mask = ((q_pos - k_pos) < local[0]) & ((k_pos - q_pos) < local[1])
        mask = vert | local_mask
    else:
        left = (q_pos - k_pos) - local[0] + 1
        left = left * (left > 0)
        right = (k_pos - q_pos) - local[1] + 1
        right = right * (right > 0)
        if num_sparse_heads == num_kv_heads:
            mask = (left + right) % vert_stride == 0
        elif num_sparse_heads == 0:
            mask = np.ones_like(left, dtype=bool)
        else:
            rows = []
            for h in range(num_kv_heads):
                for _ in range(num_q_per_kv):
                    if h < num_sparse_heads:
                        rows.append((left + right)[0] % vert_stride == 0)
                    else:
                        rows.append(np.ones((blocks, kv_blocks), dtype=bool))
            mask = np.concatenate(rows, axis=0)
            # the reference vstack-s 2-D masks: result is (H*blocks, kv_blocks)
    if causal:
        mask = (q_pos >= k_pos) & mask
    mask = np.ascontiguousarray(mask).astype(np.uint8)
    trim = cdiv(past_len, block_size)
    return mask[:, trim:]


# ---------------------------------------------------------------------------
# CSR / CSC (dkernel/utils.py:19-65, 68-102)
# ---------------------------------------------------------------------------
def to_csr(mat: np.ndarray) -> Tuple[np.ndarray, np.ndarray, np.ndarray]:
    """dkernel/utils.py:19-24: (indptr, indices, data) of a 2-D matrix."""
    nz = mat != 0
    counts = nz.astype(np.int32).sum(-1)
    _, col_idx = np.where(nz)
    crow = np.cumsum(np.concatenate([[0], counts]))
    return crow.astype(np.int32), col_idx.astype(np.int32), mat[nz]


def dense_to_crow_col(x: np.ndarray, include_values: bool = False
                      ) -> Tuple[np.ndarray, np.ndarray]:
    """dkernel/utils.py:27-65: per-head CSR, column lists padded with -1 to the
    longest head; with ``include_values`` col becomes (..., nnz, 2) = (col, value)
    and the value padding is 0."""
    x = np.asarray(x)
    dim = x.ndim
    assert dim in (2, 3)
    if dim == 2:
        x = x[None]
    per_head = [to_csr(xi.astype(np.int32)) for xi in x]
    crows = np.stack([p[0] for p in per_head]).astype(np.int32)
    max_cols = max(len(p[1]) for p in per_head)
    cols = np.full((len(per_head), max_cols), -1, dtype=np.int32)
    for i, p in enumerate(per_head):
        cols[i, :len(p[1])] = p[1]
    if include_values:
        vals = np.zeros((len(per_head), max_cols), dtype=np.int32)
        for i, p in enumerate(per_head):
            vals[i, :len(p[2])] = p[2]
        cols = np.stack([cols, vals], axis=-1)
    if dim == 2:
        return crows[0], cols[0]
    return crows, cols


def dense_to_ccol_row(x: np.ndarray, **kw) -> Tuple[np.ndarray, np.ndarray]:
    """dkernel/utils.py:91-95: CSC = CSR of the transposed pattern."""
    return dense_to_crow_col(np.swapaxes(np.asarray(x), -2, -1), **kw)


def crow_col_to_dense(crows: np.ndarray, cols: np.ndarray, n_cols: Optional[int] = None) -> np.ndarray:
    """Inverse of ``dense_to_crow_col`` (dkernel/utils.py:68-88)."""
    crows = np.asarray(crows)
    cols = np.asarray(cols)
    if crows.ndim == 1:
        crows, cols = crows[None], cols[None]
    H, M = crows.shape[0], crows.shape[1] - 1
    N = n_cols if n_cols is not None else int(cols.max()) + 1
    out = np.zeros((H, M, N), dtype=np.int32)
    for h in range(H):
        for m in range(M):
            s, e = crows[h, m], crows[h, m + 1]
            if cols.ndim == 2:
                out[h, m, cols[h, s:e]] = 1
            else:
                out[h, m, cols[h, s:e, 0]] = cols[h, s:e, 1]
    return out


def merge_split_fwd_kernel_blocks(block_size: int, pattern: np.ndarray,
                                  block_m: int, block_n: int
                                  ) -> Tuple[np.ndarray, np.ndarray]:
    """dkernel/utils.py:262-310.  Identity (plain CSR) when the kernel tile
    equals the sparse block; otherwise split by a Kronecker product and re-apply
    the block-causal mask (:287-297), and, when block_m > block_size, merge
    m-blocks storing (index of last attending sub-row + 1) * block_size beside
    each column (:299-308)."""
    pattern = np.asarray(pattern)
    if block_size == block_m and block_size == block_n:
        return dense_to_crow_col(pattern)
    assert (block_m % block_size == 0) or (block_size % block_n == 0)
    assert block_size % block_n == 0
    block_m_mult = block_size // block_m if block_size > block_m else 1
    kron = np.ones((block_m_mult, block_size // block_n), dtype=pattern.dtype)
    if kron.size > 1:
        _bm = block_size // kron.shape[0]
        _bn = block_size // kron.shape[1]
        pattern = np.kron(pattern, kron)
        cm = (np.arange(1, pattern.shape[1] + 1)[:, None] * _bm
              > np.arange(0, pattern.shape[2])[None, :] * _bn)
        pattern = pattern * cm.astype(pattern.dtype)
    if block_size < block_m:
        H, M, N = pattern.shape
        m_mult = block_m // block_size
        assert M % m_mult == 0
        p = pattern.astype(np.int32).reshape(H, M // m_mult, m_mult, N)
        p = (np.cumsum(p[:, :, ::-1, :], axis=2) > 0).sum(2)
        p = p * block_size
        return dense_to_crow_col(p, include_values=True)
    return dense_to_crow_col(pattern)


def is_kv_cache_efficient(pattern: np.ndarray, block_m: int, block_n: int) -> bool:
    """dkernel/utils.py:232-245."""
    p = np.asarray(pattern).astype(np.int8)
    non_diag = (np.arange(0, p.shape[1])[:, None] * block_m
                >= np.arange(1, p.shape[2] + 1)[None, :] * block_n)
    return bool((((p[:, 1:] - p[:, :-1]) <= 0) | (~non_diag[1:])).all())


# ---------------------------------------------------------------------------
# Masked-dense attention (tests/test_sparse_attn.py:486-537 of the reference)
# ---------------------------------------------------------------------------
def token_mask(bmask: np.ndarray, block_size: int, seqlen: int, kv_seqlen: int,
               causal: bool = True, past_len: int = 0) -> torch.Tensor:
    """Token-level mask from an *untrimmed* block mask (dkernel/utils.py:222-227):
    kron(block, ones) cropped to (seqlen, kv_seqlen), times tril when causal,
    rows before past_len dropped."""
    bm = torch.from_numpy(np.asarray(bmask).astype(np.uint8))
    dense = torch.kron(bm, bm.new_ones((block_size, block_size)))[..., :seqlen, :kv_seqlen]
    if causal:
        tri = torch.tril(torch.ones(seqlen, kv_seqlen, dtype=dense.dtype))[past_len:]
        dense = dense[..., past_len:, :] * tri[None]
    return dense


def masked_dense_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           attn_mask: Optional[torch.Tensor], sm_scale: Optional[float] = None,
                           seq_dim: int = 2, return_lse: bool = False):
    """The reference's ``torch_attention`` with the dense-mask branch
    (tests/test_sparse_attn.py:523-533): einsum logits in the input dtype, cast
    to fp32, scale, ``masked_fill(-inf)``, softmax, PV in the value dtype.
    q: (B,H,Sq,D) for seq_dim=2 or (B,Sq,H,D) for seq_dim=1; K/V with fewer heads
    are repeated along the head axis (dkernel/utils.py:193,
    dkernel/ops/sparse_attn_inference.py:488).  Rows with no attended key give 0
    (and LSE=-inf) instead of NaN.  LSE = logsumexp of the scaled masked logits."""
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(float(q.size(-1)))
    if seq_dim == 1:
        q, k, v = [x.transpose(1, 2) for x in (q, k, v)]
    if k.size(1) != q.size(1):
        rep = q.size(1) // k.size(1)
        k = k.repeat_interleave(rep, dim=1)
        v = v.repeat_interleave(rep, dim=1)
    attn = torch.einsum("bhmd,bhnd->bhmn", q, k).float() * sm_scale
    if attn_mask is not None:
        attn = attn.masked_fill((1 - attn_mask.to(torch.int32)).bool(), float("-inf"))
    lse = torch.logsumexp(attn, dim=-1)
    p = torch.exp(attn - torch.where(torch.isinf(lse), torch.zeros_like(lse), lse)[..., None])
    out = torch.einsum("bhmn,bhnd->bhmd", p.type_as(v), v)
    if seq_dim == 1:
        out = out.transpose(1, 2)
    if return_lse:
        return out, lse
    return out


def block_sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor,
                           bmask: np.ndarray, block_size: int,
                           sm_scale: Optional[float] = None, seq_dim: int = 1,
                           causal: bool = True, heads: Optional[Sequence[int]] = None,
                           batches: Optional[Sequence[int]] = None):
    """Masked-dense attention evaluated one (batch, head) at a time in fp32, so
    that long sequences fit in memory.  ``bmask`` is (Hpat, Mblk, Nblk) with
    Hpat in {1, Hkv, Hq}; q rows are q-tile rows of the pattern (no offset) and
    the causal offset is ``Sk - Sq`` (dkernel/ops/sparse_attn_fwd.py:517).
    Returns (out fp32 shaped like q restricted to the chosen batches/heads on the
    (B,H,S,D) layout, lse (B,H,Sq)).  Only the selected ``heads``/``batches`` are
    evaluated (others are left at zero)."""
    if seq_dim == 1:
        q, k, v = [x.transpose(1, 2) for x in (q, k, v)]
    B, Hq, Sq, D = q.shape
    Hkv, Sk = k.size(1), k.size(2)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(float(D))
    bmask = np.asarray(bmask)
    Hp = bmask.shape[0]
    out = torch.zeros((B, Hq, Sq, D), dtype=torch.float32)
    lse = torch.full((B, Hq, Sq), float("-inf"), dtype=torch.float32)
    past = Sk - Sq if causal else 0
    for h in (heads if heads is not None else range(Hq)):
        hp = 0 if Hp == 1 else (h if Hp == Hq else h // (Hq // Hkv))
        hk = h // (Hq // Hkv)
        bm = torch.from_numpy(bmask[hp].astype(np.uint8))
        dense = torch.kron(bm, bm.new_ones((block_size, block_size)))[:Sq, :Sk].bool()
        if causal:
            dense = dense & (torch.arange(Sq)[:, None] + past >= torch.arange(Sk)[None, :])
        for b in (batches if batches is not None else range(B)):
            a = (q[b, h].float() @ k[b, hk].float().T) * sm_scale
            a = a.masked_fill(~dense, float("-inf"))
            l = torch.logsumexp(a, dim=-1)
            p = torch.exp(a - torch.where(torch.isinf(l), torch.zeros_like(l), l)[:, None])
            out[b, h] = p @ v[b, hk].float()
            lse[b, h] = l
    if seq_dim == 1:
        out = out.transpose(1, 2)
    return out, lse


def _seq_attention(q, k, v, bmask, block_size, sm_scale, causal=True):
    """One sequence, (Hq, Lq, D) x (Hkv, Lk, D), positions re-based to 0, q rows
    placed at the END of the kv positions (past_len = Lk - Lq), pattern row =
    position // block_size (dkernel/ops/sparse_attn_inference.py:503-514)."""
    Hq, Lq, D = q.shape
    Hkv, Lk, _ = k.shape
    Hp = bmask.shape[0]
    past = Lk - Lq
    out = torch.zeros((Hq, Lq, D), dtype=torch.float32)
    lse = torch.full((Hq, Lq), float("-inf"), dtype=torch.float32)
    qpos = past + torch.arange(Lq)
    kpos = torch.arange(Lk)
    for h in range(Hq):
        hp = 0 if Hp == 1 else (h if Hp == Hq else h // (Hq // Hkv))
        hk = h // (Hq // Hkv)
        bm = torch.from_numpy(np.asarray(bmask[hp]).astype(np.uint8)).bool()
        allowed = bm[(qpos // block_size)[:, None], (kpos // block_size)[None, :]]
        if causal:
            allowed = allowed & (qpos[:, None] >= kpos[None, :])
        a = (q[h].float() @ k[hk].float().T) * sm_scale
        a = a.masked_fill(~allowed, float("-inf"))
        l = torch.logsumexp(a, dim=-1)
        p = torch.exp(a - torch.where(torch.isinf(l), torch.zeros_like(l), l)[:, None])
        out[h] = p @ v[hk].float()
        lse[h] = l
    return out, lse


def padded_attention(q, k, v, bmask, block_size, sm_scale=None, left_paddings=None,
                     seqlens=None, seq_dim=1, causal=True):
    """Semantics of ``padded_sparse_attn`` (dkernel/ops/sparse_attn_inference.py:10-147):
    sequence b occupies storage [left_b, left_b + len_b) of K/V; q is either one
    token (decode, stored at index 0) or laid out like K.  Pad rows of the output
    are zero (:67).  Returns (out fp32 shaped like q, lse (B,Hq,Sq), -inf on pads)."""
    if seq_dim == 1:
        q, k, v = [x.transpose(1, 2) for x in (q, k, v)]
    B, Hq, Sq, D = q.shape
    Sk = k.size(2)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(float(D))
    out = torch.zeros((B, Hq, Sq, D), dtype=torch.float32)
    lse = torch.full((B, Hq, Sq), float("-inf"), dtype=torch.float32)
    for b in range(B):
        ks = int(left_paddings[b]) if left_paddings is not None else 0
        ke = ks + int(seqlens[b]) if seqlens is not None else Sk
        if Sq == 1:
            qs, qe = 0, 1
        else:
            qs, qe = ks, ke
        if ke <= ks:
            continue
        o, l = _seq_attention(q[b, :, qs:qe], k[b, :, ks:ke], v[b, :, ks:ke], bmask,
                              block_size, sm_scale, causal)
        out[b, :, qs:qe] = o
        lse[b, :, qs:qe] = l
    if seq_dim == 1:
        out = out.transpose(1, 2)
    return out, lse


def varlen_attention(q, k, v, cu_seqlens_k, bmask, block_size, sm_scale=None,
                     cu_seqlens_q=None, causal=True):
    """Semantics of ``varlen_sparse_attn`` (dkernel/ops/sparse_attn_inference.py:150-287):
    q (Tq,Hq,D), k/v (Tk,Hkv,D); per sequence q_len in {1, k_len}.
    Returns (out fp32 (Tq,Hq,D), lse (Hq,Tq))."""
    cu_k = [int(x) for x in cu_seqlens_k]
    nb = len(cu_k) - 1
    if cu_seqlens_q is None:
        if q.size(0) == nb:
            cu_q = list(range(nb + 1))
        elif q.size(0) == k.size(0):
            cu_q = cu_k
        else:
            raise ValueError("cu_seqlens_q must be specified")
    else:
        cu_q = [int(x) for x in cu_seqlens_q]
    D = q.size(-1)
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(float(D))
    out = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.full((q.size(1), q.size(0)), float("-inf"), dtype=torch.float32)
    for b in range(nb):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe <= qs:
            continue
        o, l = _seq_attention(q[qs:qe].transpose(0, 1), k[ks:ke].transpose(0, 1),
                              v[ks:ke].transpose(0, 1), bmask, block_size, sm_scale, causal)
        out[qs:qe] = o.transpose(0, 1)
        lse[:, qs:qe] = l
    return out, lse


def decode_attention(q, k, v, bmask, block_size, sm_scale=None, left_paddings=None,
                     seqlens=None, kv_block_range=None):
    """One query token per sequence against a (B,Sk,Hkv,D) left/right padded KV
    buffer: the pattern row is (len_b - 1) // block_size
    (dkernel/ops/sparse_attn_inference.py:507-514), every real token of an
    attended block is visible.  ``kv_block_range=(lo, hi)`` restricts the
    attended blocks to [lo, hi) positions-blocks (a KV shard).  q: (B,1,Hq,D).
    Returns (out fp32 (B,1,Hq,D), lse (B,Hq,1))."""
    B, _, Hq, D = q.shape
    Sk, Hkv = k.size(1), k.size(2)
    Hp = bmask.shape[0]
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(float(D))
    out = torch.zeros((B, 1, Hq, D), dtype=torch.float32)
    lse = torch.full((B, Hq, 1), float("-inf"), dtype=torch.float32)
    for b in range(B):
        ks = int(left_paddings[b]) if left_paddings is not None else 0
        L = int(seqlens[b]) if seqlens is not None else Sk - ks
        if L <= 0:
            continue
        row = (L - 1) // block_size
        kpos = torch.arange(L)
        for h in range(Hq):
            hp = 0 if Hp == 1 else (h if Hp == Hq else h // (Hq // Hkv))
            hk = h // (Hq // Hkv)
            bm = torch.from_numpy(np.asarray(bmask[hp, row]).astype(np.uint8)).bool()
            allowed = bm[kpos // block_size]
            if kv_block_range is not None:
                lo, hi = kv_block_range
                allowed = allowed & (kpos // block_size >= lo) & (kpos // block_size < hi)
            a = (k[b, ks:ks + L, hk].float() @ q[b, 0, h].float()) * sm_scale
            a = a.masked_fill(~allowed, float("-inf"))
            l = torch.logsumexp(a, dim=-1)
            if torch.isinf(l):
                continue
            p = torch.exp(a - l)
            out[b, 0, h] = p @ v[b, ks:ks + L, hk].float()
            lse[b, h, 0] = l
    return out, lse


def combine_attn_partitions(*parts, hdim: int = 1):
    """dkernel/interface.py:303-324: weights = softmax over partitions of the LSEs,
    output = sum_p o_p * w_p in fp32, cast back.  ``hdim`` selects the head axis
    of the outputs (the reference ignores it and only works for hdim=1): outputs
    (B,H,S,D) for hdim=1 or (B,S,H,D) for hdim=2; LSE always (B,H,S).
    Partitions whose LSE is -inf everywhere for a row contribute nothing; a row
    with all partitions at -inf gives 0."""
    assert len(parts) >= 2 and len(parts[0]) == 2
    outs, lses = zip(*parts)
    w = torch.stack([l.float() for l in lses], dim=0)
    mx = w.max(dim=0, keepdim=True).values
    mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    e = torch.exp(w - mx)
    den = e.sum(0, keepdim=True)
    w = e / torch.where(den == 0, torch.ones_like(den), den)
    o = torch.stack([x.float() for x in outs], dim=0)
    if hdim == 2:
        w = w.transpose(2, 3)
    res = (o * w.unsqueeze(-1)).sum(0)
    lse = (mx + torch.log(den)).squeeze(0)
    return res.to(outs[0].dtype), lse


def attended_tiles(bmask: np.ndarray, n_q_blocks: int, n_kv_blocks: int) -> int:
    """Number of attended blocks in the top-left (n_q_blocks, n_kv_blocks) corner,
    summed over heads: the unit the throughput metric counts FLOPs on."""
    return int(np.asarray(bmask)[:, :n_q_blocks, :n_kv_blocks].astype(np.int64).sum())
