"""Sparse-pattern helpers: the device-side counterpart of dkernel/utils.py.

Same names, arguments and results as the reference module, but the block mask
and the CSR/CSC layouts are produced by CUDA kernels of libbsa_b200.so instead
of a GPU -> CPU -> numpy -> GPU round trip (dkernel/utils.py:47-49,65).
Everything here needs a CUDA device; there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Tuple, Union

import torch
from torch import Tensor

from . import _lib


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def multiple_of(x: int, y: int) -> int:
    """dkernel/utils.py:323-324."""
    return ((x + y - 1) // y) * y


def zero_stride(x: Tensor, dim: int = 0) -> Tensor:
    """View of ``x`` whose stride along the size-1 dimension ``dim`` is 0
    (dkernel/utils.py:313-320)."""
    assert x.size(dim) <= 1, f"Cannot set stride at {dim=} to 0 as the size is {x.size(dim)}."
    strides = list(x.stride())
    strides[dim] = 0
    return x.as_strided(x.shape, tuple(strides))


def _device(device=None) -> torch.device:
    if not torch.cuda.is_available():
        raise RuntimeError("dkernel_b200 builds sparse layouts on a CUDA device; none is available "
                           "(there is no CPU path).")
    if device is None:
        return torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError(f"layouts are built on CUDA devices, got {device}")
    return device


def _as_u8_mask(x: Tensor) -> Tensor:
    if x.dtype == torch.uint8:
        return x
    if x.dtype == torch.bool:
        return x.to(torch.uint8)
    return (x != 0).to(torch.uint8)


def dense_to_crow_col(x: Tensor, include_values: bool = False) -> Tuple[Tensor, Tensor]:
    """2-D/3-D pattern -> (crow, col) int32 on the pattern's device, col padded
    with -1 to the longest head; with ``include_values`` col is (..., nnz, 2) =
    (column, value).  Bit-exact with dkernel/utils.py:27-65."""
    _lib.require_cuda(x, "sparse pattern")
    dim = x.dim()
    assert dim in (2, 3)
    if dim == 2:
        x = x[None]
    H, M, N = x.shape
    if include_values:
        assert x.dtype in (torch.bool, torch.uint8, torch.int8, torch.int32, torch.int64), f"> {x.dtype}"
        assert int(x.max().item()) <= 255 if x.numel() else True, "values above 255 are not supported"
        m8 = x.to(torch.uint8)
    else:
        m8 = _as_u8_mask(x)
    lib = _lib.lib()
    with torch.cuda.device(x.device):
        st = _lib.stream_of(x)
        crow = torch.empty((H, M + 1), dtype=torch.int32, device=x.device)
        nnz = torch.empty((H,), dtype=torch.int32, device=x.device)
        _lib.check(lib.bsa_csr_row_ptr(_lib.ptr(m8), H, M, N, m8.stride(0), m8.stride(1), m8.stride(2),
                                       _lib.ptr(crow), _lib.ptr(nnz), st), "bsa_csr_row_ptr")
        width = int(nnz.max().item()) if H > 0 else 0   # allocation size: one sync, constructor only
        shape = (H, width, 2) if include_values else (H, width)
        col = torch.empty(shape, dtype=torch.int32, device=x.device)
        _lib.check(lib.bsa_csr_fill_cols(_lib.ptr(m8), H, M, N, m8.stride(0), m8.stride(1),
                                         m8.stride(2), _lib.ptr(crow), _lib.ptr(col), width,
                                         1 if include_values else 0, st), "bsa_csr_fill_cols")
    if dim == 2:
        return crow[0], col[0]
    return crow, col


def dense_to_ccol_row(x: Tensor, **kwargs) -> Tuple[Tensor, Tensor]:
    """CSC = CSR of the transposed pattern (dkernel/utils.py:91-95); the kernels
    read the transposed view through its strides, nothing is copied."""
    return dense_to_crow_col(x.transpose(-2, -1), **kwargs)


def crow_col_to_dense(crows: Tensor, cols: Tensor, dtype: torch.dtype = torch.float16) -> Tensor:
    """Inverse of :func:`dense_to_crow_col` (dkernel/utils.py:68-88); a test-side
    helper, evaluated with torch indexing on the tensors' device."""
    dim = crows.dim()
    if dim == 1:
        crows, cols = crows[None], cols[None]
    H, M = crows.size(0), crows.size(1) - 1
    has_val = cols.dim() == 3
    idx = cols[..., 0] if has_val else cols
    N = int(idx.max().item()) + 1
    x = torch.zeros((H, M, N), dtype=dtype, device=crows.device)
    width = idx.size(1)
    pos = torch.arange(width, device=crows.device)
    for h in range(H):
        n = int(crows[h, -1].item())
        rows = torch.searchsorted(crows[h].contiguous(), pos[:n].to(crows.dtype), right=True) - 1
        vals = cols[h, :n, 1].to(dtype) if has_val else torch.ones(n, dtype=dtype, device=crows.device)
        x[h, rows.long(), idx[h, :n].long()] = vals
    return x[0] if dim == 1 else x


def ccol_row_to_dense(ccol: Tensor, rows: Tensor, dtype: torch.dtype = torch.float16) -> Tensor:
    """dkernel/utils.py:98-102."""
    return crow_col_to_dense(ccol, rows, dtype).permute(0, 2, 1).contiguous()


def get_sparse_attn_mask(num_heads: int,
                         seqlen: int,
                         block_size: int = 64,
                         local_blocks: Union[int, Tuple[int, int]] = 4,
                         vert_stride: int = 4,
                         homo_head: bool = False,
                         num_kv_heads: Optional[int] = None,
                         past_len: Optional[int] = None,
                         dtype: torch.dtype = torch.bfloat16,
                         device=None,
                         return_dense: bool = False,
                         head_sliding_step: Optional[int] = None,
                         head_sliding_offset: int = 0,
                         num_dense_heads: int = 0,
                         kv_seqlen: Optional[int] = None,
                         q_start_position: Optional[int] = None,
                         kv_start_position: Optional[int] = None,
                         vert_position_type: Optional[str] = None,
                         causal: bool = True):
    """Local + vertical-stride block pattern, as dkernel/utils.py:105-229.

    Returns ``((crow, col), block_mask, dense_mask | None)`` on the current CUDA
    device (the reference also ignores ``device`` and uses the current one,
    dkernel/utils.py:143).  The mask is evaluated analytically by a CUDA kernel,
    one thread per block; the CSR comes from :func:`dense_to_crow_col`.

    One deliberate difference: with ``causal=False``, relative vertical positions
    and ``0 < num_dense_heads < num_kv_heads`` the reference stacks 2-D masks into
    a (H*blocks, kv_blocks) matrix (dkernel/utils.py:205-210), which no caller can
    use; here that case yields the intended (H, blocks, kv_blocks) mask.
    """
    dev = _device(None)
    past_len = past_len or 0
    kv_seqlen = kv_seqlen or seqlen
    if homo_head:
        num_heads = 1
        assert num_dense_heads == 0, "Cannot have dense head if stride pattern for heads is homogeneous."
    if vert_position_type is None:
        vert_position_type = "absolute" if causal else "relative"
    else:
        assert vert_position_type in ("absolute", "relative")
    num_kv_heads = num_kv_heads or num_heads
    assert num_heads % num_kv_heads == 0
    q_start_block = 0
    kv_start_block = 0
    if q_start_position is not None:
        assert q_start_position % block_size == 0, "Sequence chunking must be at the block boundary"
        q_start_block = q_start_position // block_size
        assert past_len in [0, None], "Cannot specify both past_len and q_start_position"
    if kv_start_position is not None:
        assert kv_start_position % block_size == 0, "Sequence chunking must be at the block boundary"
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
    if head_sliding_step is None:
        head_sliding_step = max(1, int(vert_stride / num_heads))

    blocks = cdiv(seqlen, block_size)
    kv_blocks = cdiv(kv_seqlen, block_size)
    trim = cdiv(past_len, block_size)
    p = _lib.LocalStrideParams(
        num_heads=num_heads, num_kv_heads=num_kv_heads, num_dense_heads=num_dense_heads,
        q_blocks=blocks, kv_blocks=kv_blocks, q_start_block=q_start_block,
        kv_start_block=kv_start_block, trim_q_blocks=trim, local_left=local[0], local_right=local[1],
        vert_stride=vert_stride, head_sliding_step=head_sliding_step,
        head_sliding_offset=head_sliding_offset, causal=1 if causal else 0,
        absolute_vert=1 if vert_position_type == "absolute" else 0)
    if vert_position_type == "relative" and num_dense_heads in (0, num_kv_heads):
        # every head has the same relative pattern: the reference returns one head
        # (broadcast of (1, M, 1) against (1, 1, N), dkernel/utils.py:196-204)
        p.num_heads = p.num_kv_heads = 1
        p.num_dense_heads = 1 if num_dense_heads else 0
        num_heads = 1
    with torch.cuda.device(dev):
        mask8 = torch.empty((num_heads, max(blocks - trim, 0), kv_blocks), dtype=torch.uint8, device=dev)
        _lib.check(_lib.lib().bsa_local_stride_mask(C.byref(p), _lib.ptr(mask8), _lib.stream_of(mask8)),
                   "bsa_local_stride_mask")
        csr = dense_to_crow_col(mask8)
        trimmed = mask8.to(dtype)
        mask_dense = None
        if return_dense:
            # token-level mask of the untrimmed pattern (dkernel/utils.py:222-227); test aid only
            if trim:
                q = LocalStrideParams_copy(p, trim_q_blocks=0)
                full8 = torch.empty((num_heads, blocks, kv_blocks), dtype=torch.uint8, device=dev)
                _lib.check(_lib.lib().bsa_local_stride_mask(C.byref(q), _lib.ptr(full8),
                                                            _lib.stream_of(full8)), "bsa_local_stride_mask")
            else:
                full8 = mask8
            full = full8.to(dtype)
            mask_dense = torch.kron(full, full.new_ones((block_size, block_size)))[..., :seqlen, :kv_seqlen]
            if causal:
                causal_mask = torch.tril(torch.ones(seqlen, kv_seqlen, device=dev)).type_as(mask_dense)[past_len:]
                mask_dense = mask_dense[..., past_len:, :] * causal_mask[None]
    return csr, trimmed, mask_dense


def LocalStrideParams_copy(p, **changes):
    q = _lib.LocalStrideParams()
    C.memmove(C.byref(q), C.byref(p), C.sizeof(q))
    for k, v in changes.items():
        setattr(q, k, v)
    return q


def is_kv_cache_efficient(sparse_pattern: Tensor, block_m: int, block_n: int) -> bool:
    """True when the non-local blocks used by later rows are also used by earlier
    rows (dkernel/utils.py:232-245)."""
    sp = sparse_pattern.to(torch.int8)
    dev = sp.device
    non_diag = (torch.arange(0, sp.size(1), device=dev)[:, None] * block_m
                >= torch.arange(1, sp.size(2) + 1, device=dev) * block_n)
    return bool((((sp[:, 1:] - sp[:, :-1]) <= 0) | (~non_diag[1:])).all().item())


def verify_sparse_pattern(sparse_pattern: Tensor) -> None:
    """dkernel/utils.py:248-252."""
    assert sparse_pattern.dim() in (2, 3)


def is_causal(sparse_pattern: Tensor) -> bool:
    """dkernel/utils.py:255-259."""
    sp = sparse_pattern.to(torch.int8)
    assert sp.size(-2) == sp.size(-1)
    sp = sp * (1 - torch.tril(torch.ones_like(sp[0])))
    return not bool(sp.any().item())


def merge_split_fwd_kernel_blocks(block_size: int, sparse_pattern: Tensor, block_m: int,
                                  block_n: int) -> Tuple[Tensor, Tensor]:
    """Layout in (block_m, block_n) kernel tiles, as dkernel/utils.py:262-310: plain
    CSR when the tile equals the sparse block, otherwise blocks are split by a
    Kronecker product (block-causal mask re-applied) and, when block_m is larger
    than the sparse block, m-blocks are merged with the value
    ``(index of last attending sub-row + 1) * block_size`` stored beside each column."""
    if block_size == block_m and block_size == block_n:
        return dense_to_crow_col(sparse_pattern)
    assert (block_m % block_size == 0) or (block_size % block_n == 0), \
        "block_m must be mutliple or a factor of sparse block size for merging on Q blocks"
    assert block_size % block_n == 0, \
        "block_n must be a factor of sparse block size for splitting on K blocks"
    dev = sparse_pattern.device
    block_m_mult = block_size // block_m if block_size > block_m else 1
    kron_factor = sparse_pattern.new_ones((block_m_mult, block_size // block_n))
    if kron_factor.numel() > 1:
        _bm = block_size // kron_factor.size(0)
        _bn = block_size // kron_factor.size(1)
        sparse_pattern = torch.kron(sparse_pattern, kron_factor)
        causal_mask = (torch.arange(1, sparse_pattern.size(1) + 1, device=dev)[:, None] * _bm
                       > torch.arange(0, sparse_pattern.size(2), device=dev) * _bn)
        sparse_pattern = sparse_pattern * causal_mask.type_as(sparse_pattern)
    if block_size < block_m:
        H, M, N = sparse_pattern.shape
        m_mult = block_m // block_size
        assert M % m_mult == 0, f"> {M=}, {m_mult=}"
        sp = (sparse_pattern.to(torch.int32).reshape(H, M // m_mult, m_mult, N).flip([2]).cumsum(2) > 0).sum(2)
        sp = (sp * block_size).to(torch.int32)
        return dense_to_crow_col(sp, include_values=True)
    return dense_to_crow_col(sparse_pattern)


def get_q_block_ids(past_len: int, q_len: int, block_size: int):
    """dkernel/utils.py:334-337."""
    return range(past_len // block_size, cdiv(past_len + q_len, block_size))
