"""Module API: drop-in counterparts of dkernel/interface.py.

``SparseAttention`` (user pattern), ``LocalStrideSparseAttention`` (local band +
vertical stripes, ``lru_cache``-d like the reference) and
``combine_attn_partitions``.  Constructor and ``forward`` signatures, registered
buffers, attributes and error behaviour follow the reference; the layouts are
built on the device and the kernels are hand-written sm_100a CUDA behind a C ABI.
"""
from __future__ import annotations

import copy
import ctypes as C
import math
import warnings
from functools import lru_cache
from typing import Optional, Tuple

import torch
from torch import Tensor

from . import _lib
from .ops import _Plan, _sparse_attention
from .utils import (dense_to_ccol_row, dense_to_crow_col, get_sparse_attn_mask, is_kv_cache_efficient,
                    merge_split_fwd_kernel_blocks, multiple_of, verify_sparse_pattern, zero_stride)


class SparseAttention(torch.nn.Module):
    """Block-sparse attention with a user-defined block pattern
    (dkernel/interface.py:18-215).

    Arguments
    =========
    block_size: sparse block size, a power of 2, at least 16.
    sparse_pattern: 2-D or 3-D (per head) boolean/uint8 tensor on a CUDA device; 1 = attended.
    causal: default True.
    seq_dim: None/1 -> inputs are (batch, seq, heads, dim); 2 -> (batch, heads, seq, dim).
        Ignored for packed variable-length inputs.
    block_m, block_n: kernel tile sizes of the reference.  They are validated and
        only determine the *published* ``layout_csr_*`` buffers (which stay
        bit-identical to the reference's); the kernels here choose their own tiles
        and read the block-level layout.
    kwargs: "out" (output tensor), "inference" (force/forbid saving state for
        backward), "d_splits" (accepted, ignored: the head dimension is not split),
        "impl" ("auto" | "generic" | "sm100": kernel family, for tests).

    forward(q, k, v, sm_scale, *, cu_seqlen_k, cu_seqlen_q, left_paddings, seqlens,
            return_lse, split_qkv): see the reference docstring; the padded and
    variable-length routes also honour ``return_lse`` here.
    """

    def __init__(self,
                 block_size: int,
                 sparse_pattern: Tensor,
                 *,
                 causal: bool = True,
                 seq_dim: Optional[int] = None,
                 block_m: Optional[int] = None,
                 block_n: Optional[int] = None,
                 **kwargs):
        super().__init__()

        def _check_block_size(block_size, name):
            if block_size is not None:
                assert block_size >= 16 and math.log2(block_size) % 1 == 0, \
                    f"{name} must be power of 2 and at least 16, but {block_size} is given."

        _check_block_size(block_size, "block_size")
        _check_block_size(block_m, "block_m")
        _check_block_size(block_n, "block_n")
        assert block_size >= 16 and math.log2(block_size) % 1 == 0, \
            f"block_size must be power of 2 and at least 16, but {block_size} is given."
        assert block_size <= 128, f"block_size above 128 is not supported, got {block_size}"

        if block_m is None:
            block_m = max(block_size, 64) if causal else block_size
        if block_n is None:
            block_n = block_size

        _lib.require_cuda(sparse_pattern, "sparse_pattern")
        sparse_pattern = sparse_pattern.to(torch.uint8)
        if sparse_pattern.dim() == 2:
            sparse_pattern = zero_stride(sparse_pattern[None])
        verify_sparse_pattern(sparse_pattern)
        if causal and not is_kv_cache_efficient(sparse_pattern, block_size, block_size):
            warnings.warn("The provided sparse_pattern is not efficient for KV cache, "
                          "i.e., KV cache needed for later tokens are not used in "
                          "earlier tokens. This may result in unexpected larger KV cache.")

        self.block_size = block_size
        self.block_m = block_m
        self.block_n = block_n
        self.seq_dim = seq_dim
        self.max_seqlen = max(sparse_pattern.shape[1:]) * block_size
        self.kwargs = copy.copy(kwargs)
        self.kwargs["max_seqlen"] = self.max_seqlen
        self.kwargs["causal"] = causal

        if not causal:
            assert self.block_m <= block_size
            assert self.block_n <= block_size

        # published layouts, identical to the reference's (dkernel/interface.py:118-147)
        layout_csr = list(merge_split_fwd_kernel_blocks(block_size, sparse_pattern, self.block_m,
                                                        self.block_n))
        self.block_m2, self.block_n2 = self.block_size, self.block_size
        layout_csc = list(dense_to_ccol_row(sparse_pattern, include_values=False))
        # block-level CSR read by the kernels
        if self.block_m == block_size and self.block_n == block_size:
            blk_csr = layout_csr
        else:
            blk_csr = list(dense_to_crow_col(sparse_pattern))

        def _norm(layout):
            if layout[0].dim() == 1:
                layout = [x[None] for x in layout]
            if layout[0].size(0) == 1:
                layout = [zero_stride(x) for x in layout]
            return [x.to(torch.int32) for x in layout]

        layout_csr, layout_csc, blk_csr = _norm(layout_csr), _norm(layout_csc), _norm(blk_csr)
        self.register_buffer("layout_csr_crow", layout_csr[0], persistent=False)
        self.register_buffer("layout_csr_col", layout_csr[1], persistent=False)
        self.register_buffer("layout_csc_ccol", layout_csc[0], persistent=False)
        self.register_buffer("layout_csc_row", layout_csc[1], persistent=False)
        self.register_buffer("_blk_crow", blk_csr[0], persistent=False)
        self.register_buffer("_blk_col", blk_csr[1], persistent=False)
        cr = blk_csr[0]
        self._max_row_nnz = int((cr[:, 1:] - cr[:, :-1]).max().item()) if cr.size(1) > 1 else 0
        self._plan_cache = None

    def _plan(self) -> _Plan:
        p = self._plan_cache
        if p is None or p.crow.data_ptr() != self._blk_crow.data_ptr() or p.crow.device != self._blk_crow.device:
            p = _Plan(self._blk_crow, self._blk_col, self.layout_csc_ccol, self.layout_csc_row,
                      self.block_size, self._max_row_nnz)
            self._plan_cache = p
        return p

    def forward(self,
                q: Tensor,
                k: Optional[Tensor] = None,
                v: Optional[Tensor] = None,
                sm_scale: Optional[float] = None,
                *,
                cu_seqlen_k: Optional[Tensor] = None,
                cu_seqlen_q: Optional[Tensor] = None,
                left_paddings: Optional[Tensor] = None,
                seqlens: Optional[Tensor] = None,
                return_lse: bool = False,
                split_qkv: Optional[callable] = None,
                kv_scales: Optional[Tuple[float, float]] = None,
                ) -> Tensor:
        """As the reference's forward.  One extension (its README lists it as future work): a decode
        call (one query token per sequence) may pass ``k`` and ``v`` as ``torch.float8_e4m3fn``
        tensors together with ``kv_scales = (k_scale, v_scale)``; they stand for ``k * k_scale``
        and ``v * v_scale``, and the kernel reads half the bytes."""
        inf_kwargs = {"cu_seqlen_k": cu_seqlen_k,
                      "cu_seqlen_q": cu_seqlen_q,
                      "left_paddings": left_paddings,
                      "seqlens": seqlens,
                      "kv_scales": kv_scales}
        kwargs = copy.copy(self.kwargs)
        kwargs["return_lse"] = return_lse
        kwargs["split_qkv"] = split_qkv
        kwargs["_plan"] = self._plan()
        output, lse = _sparse_attention.apply(
            q, k, v, sm_scale,
            (self.layout_csr_crow, self.layout_csr_col, self.block_m, self.block_n),
            (self.layout_csc_ccol, self.layout_csc_row, self.block_m2, self.block_n2),
            self.seq_dim, inf_kwargs, kwargs)
        if return_lse:
            return output, lse
        return output


@lru_cache(maxsize=8)
class LocalStrideSparseAttention(SparseAttention):
    """Local band + vertical stripes (dkernel/interface.py:218-300).

    num_heads: q heads; max_seq_len: longest supported sequence; block_size;
    local_blocks: width of the band in blocks (including the diagonal);
    vert_stride: one attended block column per ``vert_stride``;
    homo_head: same stripes for all heads; num_dense_heads: last heads dense;
    num_kv_heads: kv heads (the pattern is shared inside a group);
    active_head_range: (start, end) q heads of this rank, for head parallelism;
    head_sliding_offset: head whose stripes start at block 0.
    As in the reference, equal (hashable) arguments return the same instance.
    """

    def __init__(self,
                 num_heads: int,
                 max_seq_len: int,
                 block_size: int,
                 local_blocks: int,
                 vert_stride: int,
                 *,
                 homo_head: bool = False,
                 num_dense_heads: int = 0,
                 num_kv_heads: Optional[int] = None,
                 active_head_range: Optional[Tuple[int, int]] = None,
                 head_sliding_offset: int = 0,
                 block_m: Optional[int] = None,
                 block_n: Optional[int] = None,
                 causal: bool = True,
                 **kwargs):
        assert vert_stride >= 1, \
            "Vertical stride should be position integer. Value 1 will collapse to dense attention."
        if vert_stride > 1:
            assert local_blocks >= 1, "Token in the first block will attend to nothing in some blocks."
        self.max_seq_len = multiple_of(max_seq_len, max([block_size, block_m or 1, block_n or 1, 64]))
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.local_blocks = local_blocks
        self.vert_stride = vert_stride
        self.homo_head = homo_head
        self.num_dense_heads = num_dense_heads
        sparse_pattern = get_sparse_attn_mask(num_heads, self.max_seq_len,
                                              block_size=block_size,
                                              local_blocks=local_blocks,
                                              vert_stride=vert_stride,
                                              homo_head=homo_head,
                                              dtype=torch.uint8,
                                              num_kv_heads=num_kv_heads,
                                              head_sliding_offset=head_sliding_offset,
                                              num_dense_heads=num_dense_heads,
                                              causal=causal)[1]
        if (not homo_head) and (active_head_range is not None):
            assert isinstance(active_head_range, tuple)
            assert len(active_head_range) == 2, \
                '"active_head_range" should be a tuple of start/end index of the heads.'
            h_start, h_end = active_head_range
            sparse_pattern = sparse_pattern[h_start:h_end]
        super().__init__(block_size, sparse_pattern, block_m=block_m, block_n=block_n, causal=causal,
                         **kwargs)


def combine_attn_partitions(*x: Tuple[Tensor, Tensor], hdim: int = 1, return_lse: bool = False):
    """Merge attention results computed over disjoint key/value partitions
    (dkernel/interface.py:303-324): ``out = sum_p o_p * softmax_p(lse_p)``.

    Each element of ``x`` is ``(output, lse)`` with lse fp32 (batch, heads, seq);
    outputs are (batch, heads, seq, dim) for ``hdim=1`` or (batch, seq, heads, dim)
    for ``hdim=2`` (the reference ignores ``hdim`` and fails on the second layout).
    Without gradients one fused kernel does the merge; when a gradient is required
    the same formula is evaluated with differentiable torch ops so that it reaches
    both the outputs and the LSEs."""
    assert len(x) >= 2 and len(x[0]) == 2
    outputs, weights = list(zip(*x))
    o0 = outputs[0]
    _lib.require_cuda(o0, "partition output")
    needs_grad = torch.is_grad_enabled() and any(t.requires_grad for t in outputs + weights)
    if needs_grad:
        w = torch.stack(weights, dim=0).float()
        mx = w.max(dim=0, keepdim=True).values
        mx = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx).detach()
        e = torch.exp(w - mx)
        den = e.sum(0, keepdim=True)
        lse = (mx + torch.log(den)).squeeze(0)
        w = e / torch.where(den == 0, torch.ones_like(den), den)
        if hdim == 2:
            w = w.transpose(2, 3)
        o = torch.stack(outputs, dim=0)
        output = (o * w.unsqueeze(-1)).sum(0).type_as(o)
        return (output, lse) if return_lse else output
    P = len(outputs)
    B, H, S = weights[0].shape
    D = o0.size(-1)
    if hdim == 2:       # rows must be ordered like the LSE: (batch, head, seq)
        outs = [o.transpose(1, 2) for o in outputs]
    else:
        outs = list(outputs)
    o_parts = torch.stack([o.reshape(B * H * S, D) for o in outs], dim=0).contiguous()
    l_parts = torch.stack([w.to(torch.float32).reshape(B * H * S) for w in weights], dim=0).contiguous()
    res = torch.empty((B * H * S, D), dtype=o0.dtype, device=o0.device)
    lse = torch.empty((B * H * S,), dtype=torch.float32, device=o0.device)
    rows = B * H * S
    with torch.cuda.device(o0.device):
        _lib.check(_lib.lib().bsa_merge_partials(
            _lib.ptr(o_parts), _lib.ptr(l_parts), P, rows, D, rows * D, D, rows, 1, _lib.ptr(res), D,
            _lib.ptr(lse), _lib.dtype_code(o0.dtype), _lib.stream_of(o0)), "bsa_merge_partials")
    res = res.view(B, H, S, D)
    if hdim == 2:
        res = res.transpose(1, 2)
    return (res, lse.view(B, H, S)) if return_lse else res


__all__ = [
    "SparseAttention",
    "LocalStrideSparseAttention",
    "combine_attn_partitions",
]
