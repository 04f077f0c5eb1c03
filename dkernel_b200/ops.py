"""Autograd dispatcher: the counterpart of dkernel/ops/__init__.py.

``_sparse_attention.apply`` keeps the reference's argument list
(dkernel/ops/__init__.py:12-23) and routing: 3-D inputs -> packed variable-length
batch, ``left_paddings``/``seqlens`` -> padded batch, otherwise the training
forward, whose backward is available.  Every route ends in one C-ABI call
(``bsa_fwd``, ``bsa_decode`` or ``bsa_bwd``) on the current CUDA stream; nothing
synchronises with the host.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Dict, Optional, Tuple, Union

import torch
from torch import Tensor

from . import _lib


# --------------------------------------------------------------------------- helpers
def _last_dim_contig(t: Tensor) -> Tensor:
    return t if t.stride(-1) == 1 else t.contiguous()


def _tma_friendly(t: Tensor) -> Tensor:
    """Tensor-map requirements of the tcgen05 / decode kernels: 16-byte aligned
    base and strides that are multiples of 16 bytes.  Anything else is copied."""
    t = _last_dim_contig(t)
    if t.element_size() > 2:
        return t
    per16 = 16 // t.element_size()
    ok = t.data_ptr() % 16 == 0 and all(s % per16 == 0 for s in t.stride()[:-1])
    return t if ok else t.contiguous()


def _strides_bsh(t: Tensor, seq_dim: Optional[int]) -> Tuple[int, int, int]:
    """(batch, seq, head) element strides of a 4-D (seq_dim 1 or 2) or packed 3-D tensor."""
    if t.dim() == 3:
        return 0, t.stride(0), t.stride(1)
    hdim = 3 - seq_dim
    return t.stride(0), t.stride(seq_dim), t.stride(hdim)


class _Plan:
    """Kernel-side view of a module's layouts: block-level CSR/CSC and what the
    launchers need to know without touching the device."""

    def __init__(self, crow: Tensor, col: Tensor, ccol: Tensor, row: Tensor, block_size: int,
                 max_row_nnz: int, col_bits: Optional[Tensor] = None, fine_block: int = 0):
        self.crow, self.col, self.ccol, self.row = crow, col, ccol, row
        self.block_size = block_size
        self.max_row_nnz = max_row_nnz
        # a pattern with 16/32-token blocks coarsened to 64-token blocks: per entry of col one bit
        # per (sub-row, sub-column) pair of the block; only the tensor-core forward reads this form
        self.col_bits, self.fine_block = col_bits, fine_block
        self._coarse: Optional["_Plan"] = None
        self._group_shared: Dict[int, bool] = {}
        self._kv_pairs: Dict[Tuple[int, int, int], Optional[Tensor]] = {}
        self._fine: Optional["_Plan"] = None
        self._cyclic_nnz: Dict[Tuple[int, int], int] = {}
        self._max_head_nnz: Optional[int] = None
        self._csc_csr: Optional[Tensor] = None

    def max_row_nnz_cyclic(self, mod: int, rem: int) -> int:
        """Longest pattern row when only the blocks congruent to ``rem`` modulo ``mod`` count
        (what one rank of a block-cyclic KV shard sees): bounds the decode split count."""
        key = (mod, rem)
        if key not in self._cyclic_nnz:
            from .utils import crow_col_to_dense
            dense = crow_col_to_dense(self.crow, self.col, torch.int32)
            self._cyclic_nnz[key] = int(dense[:, :, rem::mod].sum(-1).max().item()) if dense.numel() else 0
        return self._cyclic_nnz[key]

    def for_kernels(self, q: Tensor, backward: bool = False) -> "_Plan":
        """The layouts the prefill / backward kernels should read.  The tensor-core kernels work
        on 64 x 64 blocks; a pattern with blocks of 128, 256, ... tokens is the same attention
        as its refinement to 64-token blocks (every block becomes a square of sub-blocks; the
        kernels mask the diagonal per element anyway), so such patterns get refined layouts
        instead of falling back to the CUDA-core kernels.  A pattern with 16- or 32-token blocks
        is coarsened to 64-token blocks with a bit mask per block (forward only)."""
        bs = self.block_size
        if bs in (16, 32) and not backward and q.dtype in (torch.float16, torch.bfloat16) \
                and q.size(-1) % 8 == 0 and q.size(-1) <= 128:
            return self._coarsened()
        if not (bs > 64 and bs % 64 == 0 and q.dtype in (torch.float16, torch.bfloat16)
                and q.size(-1) % 8 == 0 and q.size(-1) <= 256):
            return self
        if self._fine is None:
            from .utils import crow_col_to_dense, dense_to_crow_col, dense_to_ccol_row, zero_stride
            f = bs // 64
            n_cols = self.ccol.size(1) - 1
            dense = crow_col_to_dense(self.crow, self.col, torch.uint8)
            if dense.size(2) < n_cols:
                dense = torch.nn.functional.pad(dense, (0, n_cols - dense.size(2)))
            dense = dense.repeat_interleave(f, 1).repeat_interleave(f, 2).contiguous()
            lay = list(dense_to_crow_col(dense)) + list(dense_to_ccol_row(dense, include_values=False))
            lay = [x.to(torch.int32) for x in lay]
            if lay[0].size(0) == 1:
                lay = [zero_stride(x) for x in lay]
            self._fine = _Plan(lay[0], lay[1], lay[2], lay[3], 64, self.max_row_nnz * f)
        return self._fine

    def _coarsened(self) -> "_Plan":
        if self._coarse is None:
            from .utils import crow_col_to_dense, dense_to_crow_col, dense_to_ccol_row, zero_stride
            bs = self.block_size
            f = 64 // bs
            dense = crow_col_to_dense(self.crow, self.col, torch.uint8)          # (H, M, N')
            n_cols = max(self.ccol.size(1) - 1, dense.size(2))
            H, M = dense.size(0), dense.size(1)
            Mp, Np = (M + f - 1) // f * f, (n_cols + f - 1) // f * f
            dense = torch.nn.functional.pad(dense, (0, Np - dense.size(2), 0, Mp - M))
            sub = dense.view(H, Mp // f, f, Np // f, f).permute(0, 1, 3, 2, 4).reshape(H, Mp // f, Np // f, f * f)
            weights = (1 << torch.arange(f * f, device=dense.device, dtype=torch.int32))
            bits_dense = (sub.to(torch.int32) * weights).sum(-1).to(torch.int32)      # (H, Mc, Nc)
            coarse = (bits_dense != 0).to(torch.uint8).contiguous()
            lay = [x.to(torch.int32) for x in
                   list(dense_to_crow_col(coarse)) + list(dense_to_ccol_row(coarse, include_values=False))]
            crow_c, col_c = lay[0], lay[1]
            width = col_c.size(1)
            pos = torch.arange(width, device=dense.device, dtype=crow_c.dtype)[None].expand(H, -1).contiguous()
            rows = torch.searchsorted(crow_c[:, 1:].contiguous(), pos, right=True).clamp_(max=coarse.size(1) - 1)
            hidx = torch.arange(H, device=dense.device)[:, None].expand(-1, width)
            col_bits = (bits_dense[hidx, rows, col_c.clamp_min(0).long()] * (col_c >= 0)).to(torch.int32).contiguous()
            max_nnz = int((crow_c[:, 1:] - crow_c[:, :-1]).max().item()) if crow_c.size(1) > 1 else 0
            if H == 1:
                lay = [zero_stride(x) for x in lay]
                col_bits = zero_stride(col_bits)
            self._coarse = _Plan(lay[0], lay[1], lay[2], lay[3], 64, max_nnz, col_bits=col_bits, fine_block=bs)
        return self._coarse

    def max_head_nnz(self) -> int:
        """Attended blocks of the pattern head that has the most."""
        if self._max_head_nnz is None:
            self._max_head_nnz = int(self.crow[:, -1].max().item()) if self.crow.numel() else 0
        return self._max_head_nnz

    def csc_to_csr(self) -> Tensor:
        """int32, shape and head stride of ``row``: for every CSC entry the position of the same
        block in ``col`` (the CSR); -1 in the padding."""
        if self._csc_csr is None:
            crow, col, ccol, row = self.crow, self.col, self.ccol, self.row
            dev = crow.device
            H, R, Cn = crow.size(0), crow.size(1) - 1, ccol.size(1) - 1
            hh = torch.arange(H, device=dev)[:, None]
            # CSR position of every (head, row, column)
            i = torch.arange(col.size(1), device=dev, dtype=torch.int64)[None].expand(H, -1)
            rows_of = torch.searchsorted(crow[:, 1:].contiguous().long(), i.contiguous(), right=True).clamp_(max=max(R - 1, 0))
            ok = (i < crow[:, -1:].long()) & (col >= 0) & (col < Cn)
            where = torch.full((H, max(R, 1), max(Cn, 1)), -1, dtype=torch.int32, device=dev)
            hsel = hh.expand(-1, col.size(1))[ok]
            where[hsel, rows_of[ok], col.long()[ok]] = i[ok].to(torch.int32)
            # ... looked up in CSC order
            j = torch.arange(row.size(1), device=dev, dtype=torch.int64)[None].expand(H, -1)
            cols_of = torch.searchsorted(ccol[:, 1:].contiguous().long(), j.contiguous(), right=True).clamp_(max=max(Cn - 1, 0))
            okc = (j < ccol[:, -1:].long()) & (row >= 0) & (row < R)
            out = torch.full(tuple(row.shape), -1, dtype=torch.int32, device=dev)
            hselc = hh.expand(-1, row.size(1))[okc]
            out[okc] = where[hselc, row.long()[okc], cols_of[okc]]
            assert H == 1 or row.size(1) <= 1 or out.stride(0) == row.stride(0), \
                "the CSC row array is expected to be dense"
            self._csc_csr = out
        return self._csc_csr

    def heads_shared_in_group(self, hq: int, hkv: int) -> bool:
        """True when all q heads of a kv group use the same pattern rows (then the
        decode kernel stacks them into one tensor-core tile)."""
        hp = self.crow.size(0)
        if hp == 1 or hp == hkv or hq == hkv:
            return True
        if hkv not in self._group_shared:
            g = hq // hkv
            cr = self.crow.reshape(hkv, g, -1)
            cc = self.col.reshape(hkv, g, -1)
            same = bool((cr == cr[:, :1]).all().item()) and bool((cc == cc[:, :1]).all().item())
            self._group_shared[hkv] = same
        return self._group_shared[hkv]


    def kv_pairs(self, hq: int, hkv: int, n_kv_blocks: int) -> Optional[Tensor]:
        """Pairing of kv blocks for the tensor-core dK/dV kernel, which computes two kv blocks
        (128 rows) per tile and walks the union of their CSC columns: int32 (1 or hkv,
        ceil(n/2), 2), -1 = no partner, or None when pairing neighbours is at least as good.

        Candidate: blocks ordered by how many q blocks attend them (ties in index order),
        neighbours in that order paired.  For a local + vertical-stride pattern this puts
        vertical columns (attended by every later row) with vertical columns, where a
        neighbour pair would pad a short local column up to a long vertical one.  The
        candidate is kept only if it shrinks the total length of the unions."""
        key = (hq, hkv, n_kv_blocks)
        if key in self._kv_pairs:
            return self._kv_pairs[key]
        from .utils import ccol_row_to_dense
        hp = self.ccol.size(0)
        n = min(n_kv_blocks, self.ccol.size(1) - 1)
        result = None
        if n >= 4 and (hp == 1 or hp == hkv or hp == hq):
            dense = ccol_row_to_dense(self.ccol, self.row, torch.float32)[:, :, :n]   # (hp, M, N)
            if dense.size(2) < n:
                dense = torch.nn.functional.pad(dense, (0, n - dense.size(2)))
            if hp == hq and hq != hkv:
                # the CTA of a kv head walks all q heads of its group: stack their rows
                m = dense.reshape(hkv, (hq // hkv) * dense.size(1), n)
            else:
                m = dense
            count = m.sum(1)                                               # (heads, n)
            order = torch.argsort(count, dim=1, stable=True)
            if n % 2:
                order = torch.cat([order, order.new_full((order.size(0), 1), -1)], 1)
            cand = order.reshape(order.size(0), -1, 2)
            a_idx, b_idx = cand[..., 0], cand[..., 1].clamp_min(0)
            has_b = (cand[..., 1] >= 0).float()
            ma = torch.gather(m, 2, a_idx[:, None, :].expand(-1, m.size(1), -1))
            mb = torch.gather(m, 2, b_idx[:, None, :].expand(-1, m.size(1), -1)) * has_b[:, None, :]
            cost_cand = torch.maximum(ma, mb).sum().item()
            even, odd = m[:, :, 0::2], m[:, :, 1::2]
            if odd.size(2) < even.size(2):
                odd = torch.nn.functional.pad(odd, (0, 1))
            cost_adj = torch.maximum(even, odd).sum().item()
            if cost_cand < 0.97 * cost_adj:
                result = cand.to(torch.int32).contiguous()
        self._kv_pairs[key] = result
        return result


def _fill_layout(p, plan: _Plan) -> None:
    p.crow, p.col = _lib.ptr(plan.crow), _lib.ptr(plan.col)
    p.crow_sh = plan.crow.stride(0) if plan.crow.size(0) > 1 else 0
    p.col_sh = plan.col.stride(0) if plan.col.size(0) > 1 else 0
    p.h_pat = plan.crow.size(0)
    p.n_rows = plan.crow.size(1) - 1
    p.block_size = plan.block_size
    if hasattr(p, "fine_block"):
        cb = getattr(plan, "col_bits", None)
        p.col_bits = _lib.ptr(cb)
        p.col_bits_sh = cb.stride(0) if cb is not None and cb.size(0) > 1 else 0
        p.fine_block = plan.fine_block if cb is not None else 0


def _fwd_params(q, k, v, o, lse, seq_dim, plan: _Plan, sm_scale, causal, row_mode,
                q_start=None, q_end=None, k_start=None, k_end=None, total_q=0, impl=0, kernel_plan=True):
    p = _lib.FwdParams()
    own_plan = plan
    if impl != _lib.IMPL_GENERIC and kernel_plan:
        plan = plan.for_kernels(q)
    p.q, p.k, p.v, p.o, p.lse = _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse)
    p.q_sb, p.q_ss, p.q_sh = _strides_bsh(q, seq_dim)
    p.k_sb, p.k_ss, p.k_sh = _strides_bsh(k, seq_dim)
    p.v_sb, p.v_ss, p.v_sh = _strides_bsh(v, seq_dim)
    p.o_sb, p.o_ss, p.o_sh = _strides_bsh(o, seq_dim)
    if q.dim() == 3:
        p.batch = q_start.numel()
        p.hq, p.hkv, p.d = q.size(1), k.size(1), q.size(2)
        p.sq, p.sk = q.size(0), k.size(0)
        if lse is not None:          # (Hq, total tokens)
            p.lse_sb, p.lse_sh = 0, lse.stride(0)
    else:
        hdim = 3 - seq_dim
        p.batch, p.hq, p.hkv, p.d = q.size(0), q.size(hdim), k.size(hdim), q.size(3)
        p.sq, p.sk = q.size(seq_dim), k.size(seq_dim)
        if lse is not None:          # (B, Hq, Sq)
            p.lse_sb, p.lse_sh = lse.stride(0), lse.stride(1)
    p.total_q = total_q
    p.q_start, p.q_end = _lib.ptr(q_start), _lib.ptr(q_end)
    p.k_start, p.k_end = _lib.ptr(k_start), _lib.ptr(k_end)
    _fill_layout(p, plan)
    p.causal = 1 if causal else 0
    p.row_mode = row_mode
    p.dtype = _lib.dtype_code(q.dtype)
    p.impl = impl
    p.sm_scale = float(sm_scale)
    if plan.fine_block and impl == _lib.IMPL_AUTO and _lib.lib().bsa_fwd_why_not_sm100(C.byref(p)):
        # the coarsened form is only read by the tensor-core kernel: hand the pattern's own layout on
        _fill_layout(p, own_plan)
    return p


_warned_fallback = set()
_DYNAMIC_TILES_FROM = 1024     # 128-row tiles from which a forward launch gets a tile counter
_DS_WS_MAX_BYTES = 8 << 30     # largest dS scratch the backward allocates by itself


def _launch_fwd(p, q: Tensor) -> None:
    """bsa_fwd on q's device and stream.  A call whose shape the tensor-core kernel handles but
    which would still run on the CUDA-core kernel (an unaligned output view, for instance) is
    reported once per reason: that path is tens of times slower."""
    lib = _lib.lib()
    counter = None
    if (p.impl != _lib.IMPL_GENERIC and p.dtype != _lib.BSA_F32 and p.d % 8 == 0 and p.d <= 256
            and p.block_size == 64):
        why = lib.bsa_fwd_why_not_sm100(C.byref(p))
        if why and p.impl == _lib.IMPL_AUTO and why not in _warned_fallback:
            _warned_fallback.add(why)
            import warnings
            warnings.warn("dkernel_b200: this attention call runs on the CUDA-core fallback kernel, "
                          f"not on the tensor cores: {why.decode()}", RuntimeWarning, stacklevel=3)
        rows = p.total_q if p.total_q > 0 else p.batch * p.sq
        if not why and rows * p.hq >= _DYNAMIC_TILES_FROM * 128:
            # more tiles than a few rounds of the persistent grid: let the CTAs draw them from a
            # counter (zeroed on this stream; a memset node under graph capture)
            counter = torch.zeros(1, dtype=torch.int32, device=q.device)
            p.tile_counter = _lib.ptr(counter)
    with torch.cuda.device(q.device):
        _lib.check(lib.bsa_fwd(C.byref(p), _lib.stream_of(q)), "bsa_fwd")


_FP8 = getattr(torch, "float8_e4m3fn", None)


def _check_inputs(q: Tensor, k: Tensor, v: Tensor) -> None:
    for n, t in (("q", q), ("k", k), ("v", v)):
        _lib.require_cuda(t, n)
    if _FP8 is not None and k.dtype == _FP8 and v.dtype == _FP8:
        assert q.dtype in (torch.float16, torch.bfloat16), "an e4m3 K/V cache needs f16/bf16 queries"
    else:
        assert q.dtype == k.dtype == v.dtype, f"q/k/v dtypes differ: {q.dtype}, {k.dtype}, {v.dtype}"
    assert q.device == k.device == v.device
    _lib.dtype_code(q.dtype)


_IMPL_NAMES = {None: _lib.IMPL_AUTO, "auto": _lib.IMPL_AUTO, "generic": _lib.IMPL_GENERIC,
               "sm100": _lib.IMPL_SM100}


def _fp8_kv_scales(q: Tensor, k: Tensor, kv_scales) -> Optional[Tuple[float, float]]:
    """The (k_scale, v_scale) of an e4m3 K/V cache, or None for K/V of q's type.  Only the decode
    kernel reads 8-bit K/V: a single query token per sequence on 64/128-wide heads."""
    if _FP8 is None or k.dtype != _FP8:
        assert kv_scales is None, "kv_scales only applies to float8_e4m3fn K/V"
        return None
    assert kv_scales is not None and len(kv_scales) == 2, \
        "float8_e4m3fn K/V need kv_scales=(k_scale, v_scale)"
    return float(kv_scales[0]), float(kv_scales[1])


def _decode_eligible(q: Tensor, plan: _Plan, impl: int) -> bool:
    return (impl != _lib.IMPL_GENERIC and q.dtype in (torch.float16, torch.bfloat16)
            and q.size(-1) in (64, 128) and plan.block_size in (64, 128))


def _pick_heads_per_cta(g: int) -> int:
    for c in range(min(g, 16), 0, -1):
        if g % c == 0:
            return c
    return 1


def decode(q: Tensor, k: Tensor, v: Tensor, plan: _Plan, sm_scale: float, *, seq_dim: Optional[int],
           k_start: Optional[Tensor] = None, k_end: Optional[Tensor] = None,
           k_pos0: Optional[Tensor] = None, k_total: Optional[Tensor] = None,
           out: Optional[Tensor] = None, blocks_per_split: int = 0,
           workspace: Optional[Tensor] = None, lse_out: Optional[Tensor] = None,
           k_blk: Optional[Tuple[int, int]] = None, partials_only: bool = False,
           kv_scales: Optional[Tuple[float, float]] = None) -> Tuple[Tensor, Tensor]:
    """One query token per sequence (split-KV decode kernel).

    q: (B,1,Hq,D)/(B,Hq,1,D) or packed (B,Hq,D); k, v: 4-D with the module's
    seq_dim, or packed (T,Hkv,D) with ``k_start``/``k_end`` = cu_seqlens slices.
    ``k_pos0``/``k_total`` describe a contiguous KV shard, ``k_blk = (W, r)`` with ``k_total`` a
    block-cyclic one (see include/bsa.h).
    Returns (out shaped like q, lse fp32 (B,Hq)); with ``partials_only`` the split-KV partials
    stay unmerged and (o_parts fp32 (B*Hq, splits, D), lse_parts fp32 (B*Hq, splits)) are returned
    (views of one workspace tensor) for a consumer that merges them itself."""
    lib = _lib.lib()
    q = _last_dim_contig(q)     # before the strides are read: a copy has its own
    if q.dim() == 4:
        B = q.size(0)
        hdim = 3 - seq_dim
        hq, d = q.size(hdim), q.size(3)
        q_sb, q_sh = q.stride(0), q.stride(hdim)
    else:
        B, hq, d = q.shape
        q_sb, q_sh = q.stride(0), q.stride(1)
    if partials_only:
        o, o_sh, lse, lse_sh = None, d, None, 1
    elif out is not None and out.dim() == 2:
        # rows = (batch, head) with a row stride, e.g. packed next to the LSE for one all-gather
        assert out.shape == (B * hq, d) and out.stride(1) == 1 and out.dtype == q.dtype
        o, o_sh = out, out.stride(0)
    else:
        o = out if out is not None else torch.empty(q.shape, dtype=q.dtype, device=q.device)
        assert o.is_contiguous(), "decode output must be contiguous"
        o_sh = d
    if partials_only:
        pass
    elif lse_out is not None:
        assert lse_out.dtype == torch.float32 and lse_out.numel() == B * hq and lse_out.dim() == 1
        lse, lse_sh = lse_out, lse_out.stride(0)
    else:
        lse, lse_sh = torch.empty((B, hq), dtype=torch.float32, device=q.device), 1
    p = _lib.DecodeParams()
    k = _tma_friendly(k)
    v = _tma_friendly(v)
    p.q, p.k, p.v, p.o, p.lse = _lib.ptr(q), _lib.ptr(k), _lib.ptr(v), _lib.ptr(o), _lib.ptr(lse)
    p.q_sb, p.q_sh = q_sb, q_sh
    p.k_sb, p.k_ss, p.k_sh = _strides_bsh(k, seq_dim)
    p.v_sb, p.v_ss, p.v_sh = _strides_bsh(v, seq_dim)
    p.o_sb, p.o_sh = hq * o_sh, o_sh
    p.lse_sb, p.lse_sh = hq * lse_sh, lse_sh
    if k.dim() == 3:
        hkv, sk = k.size(1), k.size(0)
    else:
        hkv, sk = k.size(3 - seq_dim), k.size(seq_dim)
    p.batch, p.hq, p.hkv, p.d, p.sk = B, hq, hkv, d, sk
    p.k_start, p.k_end = _lib.ptr(k_start), _lib.ptr(k_end)
    p.k_pos0, p.k_total = _lib.ptr(k_pos0), _lib.ptr(k_total)
    _fill_layout(p, plan)
    g = hq // hkv
    p.heads_per_cta = _pick_heads_per_cta(g) if plan.heads_shared_in_group(hq, hkv) else 1
    p.blocks_per_split = blocks_per_split if blocks_per_split > 0 else 0   # 0: the library picks
    p.max_row_nnz = plan.max_row_nnz
    if k_blk is not None and k_blk[0] > 1:
        p.k_blk_mod, p.k_blk_rem = k_blk
        p.max_row_nnz = plan.max_row_nnz_cyclic(*k_blk)
    p.dtype = _lib.dtype_code(q.dtype)
    p.sm_scale = float(sm_scale)
    if kv_scales is not None:       # e4m3 K/V cache
        assert k.dtype == _FP8 and v.dtype == _FP8
        p.kv_dtype, p.k_scale, p.v_scale = _lib.BSA_F8E4M3, float(kv_scales[0]), float(kv_scales[1])
    need = lib.bsa_decode_workspace_bytes(C.byref(p))
    ws = None
    if need:
        if workspace is not None and workspace.numel() * workspace.element_size() >= need:
            ws = workspace
        else:
            ws = torch.empty((need + 3) // 4, dtype=torch.float32, device=q.device)
    p.ws = _lib.ptr(ws)
    with torch.cuda.device(q.device):
        _lib.check(lib.bsa_decode(C.byref(p), _lib.stream_of(q)), "bsa_decode")
    if partials_only:
        rows = B * hq
        nsplit = need // (4 * rows * (d + 1))
        flat = ws.view(-1)
        return (flat[:rows * nsplit * d].view(rows, nsplit, d),
                flat[rows * nsplit * d:rows * nsplit * (d + 1)].view(rows, nsplit))
    return o, lse


# --------------------------------------------------------------------------- routes
def _varlen(q, k, v, cu_seqlens_k, cu_seqlens_q, sm_scale, plan, causal, out, impl, return_lse,
            kv_scales=None):
    """Packed variable-length batch (dkernel/ops/sparse_attn_inference.py:150-287).
    Unlike the reference nothing is copied to the host: the kernels read the
    cu_seqlens on the device and enumerate q tiles themselves."""
    assert q.dim() == k.dim() == v.dim() == 3
    assert q.size(1) % k.size(1) == 0
    assert q.size(2) == k.size(2)
    assert k.shape == v.shape
    assert cu_seqlens_k.dim() == 1
    batch = cu_seqlens_k.size(0) - 1
    cu_k = cu_seqlens_k.to(device=q.device, dtype=torch.int32).contiguous()
    decoding = False
    if cu_seqlens_q is None:
        if q.size(0) == batch and q.size(0) != k.size(0):
            decoding = True
        elif q.size(0) == k.size(0):
            cu_q = cu_k
        else:
            raise ValueError("cu_seqlens_q must be specified if it mix of prefilling and decoding.")
    else:
        assert cu_seqlens_k.size(0) == cu_seqlens_q.size(0)
        cu_q = cu_seqlens_q.to(device=q.device, dtype=torch.int32).contiguous()
    fp8 = _fp8_kv_scales(q, k, kv_scales)
    if decoding and _decode_eligible(q, plan, impl):
        o, lse = decode(q, k, v, plan, sm_scale, seq_dim=None, k_start=cu_k[:-1], k_end=cu_k[1:],
                        out=out, kv_scales=fp8)
        return o, (lse.transpose(0, 1) if return_lse else None)
    assert fp8 is None, "an e4m3 K/V cache is only read by the decode kernel (one query token per sequence)"
    if decoding:
        cu_q = torch.arange(0, batch + 1, dtype=torch.int32, device=q.device)
    q, k, v = _tma_friendly(q), _tma_friendly(k), _tma_friendly(v)
    o = out if out is not None else torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.full((q.size(1), q.size(0)), float("-inf"), dtype=torch.float32, device=q.device) \
        if return_lse else None
    p = _fwd_params(q, k, v, o, lse, None, plan, sm_scale, causal, _lib.ROWS_BY_POSITION,
                    cu_q[:-1], cu_q[1:], cu_k[:-1], cu_k[1:], total_q=q.size(0), impl=impl)
    _launch_fwd(p, q)
    return o, lse


def _padded(q, k, v, sm_scale, plan, left_paddings, seqlens, seq_dim, max_seqlen, causal, out,
            impl, return_lse, kv_scales=None):
    """Left/right padded batch (dkernel/ops/sparse_attn_inference.py:10-147): pad
    rows of the output are zero, positions are re-based to the first real token."""
    assert seq_dim in (1, 2)
    hdim = 3 - seq_dim
    batches = q.size(0)
    q_len, k_len = q.size(seq_dim), k.size(seq_dim)
    assert q.dim() == k.dim() == v.dim() == 4
    assert q.size(hdim) % k.size(hdim) == 0
    assert q.size(0) == k.size(0) and q.size(3) == k.size(3)
    assert k.shape == v.shape
    assert q_len == 1 or q_len == k_len, \
        (f"q length can only 1 for decoding or the same as k length for prefilling, "
         f"but got {q_len=}, {k_len=}.")
    if max_seqlen:
        assert k_len <= max_seqlen, f"k has seqlen {k_len} while max sequence length is set to {max_seqlen}."
    dev = q.device
    if left_paddings is not None:
        assert left_paddings.shape == (batches,)
        k_starts = left_paddings.to(dev, dtype=torch.int32).contiguous()
    else:
        k_starts = torch.zeros((batches,), dtype=torch.int32, device=dev)
    if seqlens is not None:
        k_ends = k_starts + seqlens.to(dev, dtype=torch.int32)
    else:
        k_ends = None   # every sequence ends at k_len
    fp8 = _fp8_kv_scales(q, k, kv_scales)
    if q_len == 1 and _decode_eligible(q, plan, impl):
        o, lse = decode(q, k, v, plan, sm_scale, seq_dim=seq_dim, k_start=k_starts, k_end=k_ends, out=out,
                        kv_scales=fp8)
        return o, (lse.unsqueeze(-1) if return_lse else None)
    assert fp8 is None, "an e4m3 K/V cache is only read by the decode kernel (one query token per sequence)"
    if k_ends is None:
        k_ends = torch.full_like(k_starts, k_len)
    if q_len == 1:
        q_starts = torch.zeros_like(k_starts)
        q_ends = q_starts + 1
    else:
        q_starts, q_ends = k_starts, k_ends
    q, k, v = _tma_friendly(q), _tma_friendly(k), _tma_friendly(v)
    o = out if out is not None else torch.zeros(q.shape, dtype=q.dtype, device=dev)
    lse = torch.full((batches, q.size(hdim), q_len), float("-inf"), dtype=torch.float32, device=dev) \
        if return_lse else None
    p = _fwd_params(q, k, v, o, lse, seq_dim, plan, sm_scale, causal, _lib.ROWS_BY_POSITION,
                    q_starts, q_ends, k_starts, k_ends, impl=impl)
    _launch_fwd(p, q)
    return o, lse


def _train_forward(ctx, q, k, v, sm_scale, plan, seq_dim, causal, out, impl, need_lse, inference,
                   kv_scales=None):
    """Un-padded forward (dkernel/ops/sparse_attn_fwd.py:383-567).  Pattern rows are
    q tile indices; a single query token uses the row of the last key block
    (:435-440)."""
    assert seq_dim in (1, 2)
    hdim = 3 - seq_dim
    assert q.shape[-1] == k.shape[-1] == v.shape[-1]
    assert k.shape[seq_dim] == v.shape[seq_dim]
    qlen, klen = q.size(seq_dim), k.size(seq_dim)
    hq, hkv = q.size(hdim), k.size(hdim)
    assert hq % hkv == 0
    dev = q.device
    fp8 = _fp8_kv_scales(q, k, kv_scales)
    if qlen == 1 and klen > 1 and inference and _decode_eligible(q, plan, impl):
        o, lse = decode(q, k, v, plan, sm_scale, seq_dim=seq_dim, out=out, kv_scales=fp8)
        return o, lse.unsqueeze(-1)
    assert fp8 is None, "an e4m3 K/V cache is only read by the decode kernel (one query token per sequence)"
    # A single query token against a longer key sequence takes its pattern row from the key
    # position; the backward kernels index rows by q tile, so that case has no backward.
    assert inference or qlen > 1 or klen == 1, \
        "a single query token against a longer key sequence is an inference-only call (inference=True)"
    row_mode = _lib.ROWS_BY_POSITION if qlen == 1 else _lib.ROWS_BY_TILE
    q, k, v = _tma_friendly(q), _tma_friendly(k), _tma_friendly(v)
    o = out if out is not None else torch.empty(q.shape, dtype=q.dtype, device=dev)
    lse = torch.empty((q.size(0), hq, qlen), dtype=torch.float32, device=dev) if need_lse else None
    p = _fwd_params(q, k, v, o, lse, seq_dim, plan, sm_scale, causal, row_mode, impl=impl)
    _launch_fwd(p, q)
    if ctx is not None and not inference:
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.sm_scale, ctx.seq_dim, ctx.causal, ctx.plan = sm_scale, seq_dim, causal, plan
    return o, lse


def _backward(ctx, do: Tensor, dlse: Optional[Tensor], dq=None, dk=None, dv=None):
    """dQ / dK / dV of the un-padded forward (dkernel/ops/sparse_attn_bwd.py:724-852)."""
    q, k, v, o, lse = ctx.saved_tensors
    seq_dim, plan = ctx.seq_dim, ctx.plan
    if ctx.bwd_impl != _lib.IMPL_GENERIC:
        plan = plan.for_kernels(q, backward=True)
        if (plan.block_size in (16, 32) and q.dtype in (torch.float16, torch.bfloat16)
                and q.size(-1) % 8 == 0 and q.size(-1) <= 128):
            # 16/32-token blocks: the tensor-core kernels take the pattern coarsened to 64-token blocks
            # with a bit mask per block, which needs the dS hand-over (the dQ kernel then reads dS
            # tiles that are already masked); without room for its scratch the generic kernels serve it
            coarse = plan._coarsened()
            if 0 < q.size(0) * q.size(3 - seq_dim) * coarse.max_head_nnz() * 8192 <= _DS_WS_MAX_BYTES:
                plan = coarse
    do = _tma_friendly(do)
    if dq is None:
        dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    if dk is None:
        dk = torch.empty_like(k, memory_format=torch.contiguous_format)
    if dv is None:
        dv = torch.empty_like(v, memory_format=torch.contiguous_format)
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert t.stride(-1) == 1, f"{n} must be contiguous in the head dimension"
    bp = _lib.BwdParams()
    bp.f = _fwd_params(q, k, v, o, lse, seq_dim, plan, ctx.sm_scale, ctx.causal, _lib.ROWS_BY_TILE,
                       impl=ctx.bwd_impl, kernel_plan=False)
    bp.d_o = _lib.ptr(do)
    bp.do_sb, bp.do_ss, bp.do_sh = _strides_bsh(do, seq_dim)
    if dlse is not None:
        dlse = dlse.to(torch.float32).contiguous()     # (B, Hq, Sq), same strides as lse
        assert dlse.shape == lse.shape
    bp.d_lse = _lib.ptr(dlse)
    bp.dq, bp.dk, bp.dv = _lib.ptr(dq), _lib.ptr(dk), _lib.ptr(dv)
    bp.dq_sb, bp.dq_ss, bp.dq_sh = _strides_bsh(dq, seq_dim)
    bp.dk_sb, bp.dk_ss, bp.dk_sh = _strides_bsh(dk, seq_dim)
    bp.dv_sb, bp.dv_ss, bp.dv_sh = _strides_bsh(dv, seq_dim)
    bp.ccol, bp.row = _lib.ptr(plan.ccol), _lib.ptr(plan.row)
    bp.ccol_sh = plan.ccol.stride(0) if plan.ccol.size(0) > 1 else 0
    bp.row_sh = plan.row.stride(0) if plan.row.size(0) > 1 else 0
    bp.n_cols = plan.ccol.size(1) - 1
    hdim = 3 - seq_dim
    pairs = plan.kv_pairs(q.size(hdim), k.size(hdim), (k.size(seq_dim) + plan.block_size - 1) // plan.block_size)
    if pairs is not None:
        bp.kv_pairs = _lib.ptr(pairs)
        bp.kv_pairs_sh = pairs.stride(0) if pairs.size(0) > 1 else 0
        bp.n_pairs = pairs.size(1)
    sq_pad = (q.size(seq_dim) + 63) // 64 * 64
    delta = torch.empty((2, q.size(0), q.size(3 - seq_dim), sq_pad), dtype=torch.float32, device=q.device)
    bp.delta = _lib.ptr(delta)
    ds_ws = None
    if (ctx.bwd_impl != _lib.IMPL_GENERIC and plan.block_size == 64 and q.size(3) % 8 == 0 and q.size(3) <= 128
            and q.dtype in (torch.float16, torch.bfloat16)):
        # dS hand-over between the two tensor-core backward kernels (five products per block instead
        # of seven) when its scratch, one 8 KB tile per attended block and (batch, head), is affordable
        tiles = plan.max_head_nnz()
        need = q.size(0) * q.size(hdim) * tiles * 8192
        if 0 < need <= _DS_WS_MAX_BYTES:
            ds_ws = torch.empty(need, dtype=torch.uint8, device=q.device)
            bp.ds_ws = _lib.ptr(ds_ws)
            bp.ds_tiles_per_head = tiles
            bp.csc_csr = _lib.ptr(plan.csc_to_csr())
    with torch.cuda.device(q.device):
        _lib.check(_lib.lib().bsa_bwd(C.byref(bp), _lib.stream_of(q)), "bsa_bwd")
    return dq, dk, dv


# --------------------------------------------------------------------------- autograd
class _sparse_attention(torch.autograd.Function):

    @staticmethod
    def forward(ctx,
                q: Tensor,
                k: Optional[Tensor],
                v: Optional[Tensor],
                sm_scale: float,
                layout_csr: Tuple[Tensor, Tensor, int, int],
                layout_csc: Tuple[Tensor, Tensor, int, int],
                seq_dim: Optional[int],
                inf_kwargs: Dict,
                kwargs: Dict):
        (q, k, v), (packed_shape, packed_mode, split_qkv) = \
            get_qkv_and_pack_mode(q, k, v, split_qkv=kwargs.get("split_qkv", None))
        ctx.packed_shape, ctx.packed_mode, ctx.split_qkv = packed_shape, packed_mode, split_qkv
        _check_inputs(q, k, v)

        plan: _Plan = kwargs["_plan"]
        seq_dim = 1 if seq_dim is None else seq_dim
        max_seqlen = kwargs.get("max_seqlen", None)
        causal = kwargs.get("causal", True)
        return_lse = kwargs.get("return_lse", False)
        out = kwargs.get("out", None)
        impl = _IMPL_NAMES[kwargs.get("impl", None)]
        ctx.bwd_impl = _IMPL_NAMES[kwargs.get("bwd_impl", "generic" if kwargs.get("impl") == "generic"
                                              else None)]

        hdim = 3 - (seq_dim or 1) if q.dim() == 4 else 1
        n_pat = layout_csr[0].size(0)
        assert n_pat in [1, k.size(hdim), q.size(hdim)], \
            (f"Input (q, k) have ({q.size(hdim)}, {k.size(hdim)}) heads"
             f"but the number of heads in the sparse pattern is {n_pat}")
        sm_scale = sm_scale or 1. / math.sqrt(float(q.size(-1)))
        assert q.dim() in (3, 4)

        needs_grad = q.requires_grad or k.requires_grad or v.requires_grad
        if q.dim() == 3:
            assert inf_kwargs.get("cu_seqlen_k", None) is not None
            ctx.support_backward = False
            ctx.message = "Currently does not suppoort variable length inputs. WIP."
            output, lse = _varlen(q, k, v, inf_kwargs["cu_seqlen_k"], inf_kwargs.get("cu_seqlen_q", None),
                                  sm_scale, plan, causal, out, impl, return_lse,
                                  kv_scales=inf_kwargs.get("kv_scales"))
        else:
            assert k.size(seq_dim) <= max_seqlen, \
                (f"Input length {k.size(seq_dim)} is larger "
                 f"than the maximum length allowed ({max_seqlen})")
            left_paddings = inf_kwargs.get("left_paddings", None)
            seqlens = inf_kwargs.get("seqlens", None)
            if (left_paddings is not None) or (seqlens is not None):
                ctx.support_backward = False
                ctx.message = "Currently does not support paddings in inputs. WIP."
                output, lse = _padded(q, k, v, sm_scale, plan, left_paddings, seqlens, seq_dim,
                                      max_seqlen, causal, out, impl, return_lse,
                                      kv_scales=inf_kwargs.get("kv_scales"))
            else:
                inference = kwargs.get("inference", None)
                if inference is None:
                    inference = not needs_grad
                # an inference call saves nothing for backward
                ctx.support_backward = not inference
                ctx.message = "the forward pass ran with inference=True: nothing was saved for backward"
                output, lse = _train_forward(ctx, q, k, v, sm_scale, plan, seq_dim, causal, out, impl,
                                             need_lse=return_lse or not inference, inference=inference,
                                             kv_scales=inf_kwargs.get("kv_scales"))
        if not return_lse:
            lse = None
        if lse is not None and not ctx.support_backward:
            ctx.mark_non_differentiable(lse)
        return output, lse

    @staticmethod
    def backward(ctx, do: Tensor, dlse: Optional[Tensor]) -> Tuple[Union[Tensor, None], ...]:
        assert ctx.support_backward, ctx.message
        q, k = ctx.saved_tensors[:2]
        dq, dk, dv = None, None, None
        if ctx.packed_mode == 'packed_qkv':
            dqkv = q.new_empty(ctx.packed_shape)
            dq, dk, dv = ctx.split_qkv(dqkv)
        elif ctx.packed_mode == 'packed_kv':
            dkv = k.new_empty(ctx.packed_shape)
            dk, dv = ctx.split_qkv(dkv)
        dq, dk, dv = _backward(ctx, do, dlse, dq=dq, dk=dk, dv=dv)
        if ctx.packed_mode == 'packed_qkv':
            grads = (dqkv, None, None)
        elif ctx.packed_mode == 'packed_kv':
            grads = (dq, dkv, None)
        else:
            grads = (dq, dk, dv)
        return grads + (None,) * 6


def get_qkv_and_pack_mode(q: Tensor, k: Optional[Tensor], v: Optional[Tensor],
                          split_qkv: Optional[callable] = None):
    """dkernel/ops/__init__.py:128-149: unpack a packed qkv (k, v None) or a packed
    kv (v None) through the user's ``split_qkv`` callable."""
    qkv_pack_mode = 'split_qkv'
    packed_shape = None
    if v is None:
        assert split_qkv is not None, "Callable `split_qkv` must be specified if qkv or kv are packed."
        if k is None:
            packed_shape = q.shape
            q, k, v = split_qkv(q)
            qkv_pack_mode = 'packed_qkv'
        else:
            packed_shape = k.shape
            k, v = split_qkv(k)
            qkv_pack_mode = 'packed_kv'
    return (q, k, v), (packed_shape, qkv_pack_mode, split_qkv)


__all__ = ["_sparse_attention", "get_qkv_and_pack_mode", "decode"]
