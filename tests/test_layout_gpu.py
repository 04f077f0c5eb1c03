"""Device-side layout builder vs the golden vectors of the reference (bit-exact)."""
import numpy as np
import pytest
import torch

from helpers import load_patterns, pattern_kwargs

pytestmark = pytest.mark.gpu
P, META = load_patterns()
CASES = [n for n in META if not n.startswith("mod_") and n != "bernoulli"]


def _np(t):
    return t.detach().cpu().numpy()


@pytest.mark.parametrize("name", CASES)
def test_mask_csr_csc_bit_exact(name):
    from dkernel_b200.utils import get_sparse_attn_mask, dense_to_ccol_row, crow_col_to_dense
    (crow, col), bm, _ = get_sparse_attn_mask(dtype=torch.uint8, **pattern_kwargs(META[name]))
    assert bm.is_cuda and crow.is_cuda and col.is_cuda
    assert crow.dtype == torch.int32 and col.dtype == torch.int32
    g = P[f"{name}/mask"]
    assert tuple(bm.shape) == g.shape and (_np(bm) == g).all()
    assert _np(crow).shape == P[f"{name}/crow"].shape and (_np(crow) == P[f"{name}/crow"]).all()
    assert _np(col).shape == P[f"{name}/col"].shape and (_np(col) == P[f"{name}/col"]).all()
    ccol, row = dense_to_ccol_row(bm)
    assert (_np(ccol) == P[f"{name}/ccol"]).all()
    assert _np(row).shape == P[f"{name}/row"].shape and (_np(row) == P[f"{name}/row"]).all()
    back = crow_col_to_dense(crow, col, dtype=torch.uint8)
    n = back.size(-1)
    assert (_np(back) == g[..., :n]).all() and not g[..., n:].any()


def test_user_pattern_and_merge_split():
    from dkernel_b200.utils import (dense_to_crow_col, dense_to_ccol_row, merge_split_fwd_kernel_blocks,
                                    is_kv_cache_efficient)
    pat = torch.from_numpy(P["bernoulli/mask"]).cuda()
    crow, col = dense_to_crow_col(pat)
    ccol, row = dense_to_ccol_row(pat)
    assert (_np(crow) == P["bernoulli/crow"]).all() and (_np(col) == P["bernoulli/col"]).all()
    assert (_np(ccol) == P["bernoulli/ccol"]).all() and (_np(row) == P["bernoulli/row"]).all()
    assert is_kv_cache_efficient(pat, 64, 64) == META["bernoulli"]["kv_cache_efficient"]
    # 2-D pattern
    c2, l2 = dense_to_crow_col(pat[1])
    n1 = int(P["bernoulli/crow"][1, -1])
    assert (_np(c2) == P["bernoulli/crow"][1]).all() and (_np(l2) == P["bernoulli/col"][1, :n1]).all()
    seen = 0
    for key in P.files:
        if "/ms_" in key and key.endswith("/crow"):
            name, ms, _ = key.split("/")
            _, bm_, bn_ = ms.split("_")
            pat = torch.from_numpy(P[f"{name}/mask"]).cuda()
            crow, col = merge_split_fwd_kernel_blocks(META[name]["block_size"], pat, int(bm_), int(bn_))
            ref_col = P[key[:-4] + "col"]
            assert (_np(crow) == P[key]).all(), key
            assert _np(col).shape == ref_col.shape and (_np(col) == ref_col).all(), key
            seen += 1
    assert seen == 6


@pytest.mark.parametrize("name", ["mod_c2_shard", "mod_small", "mod_homo"])
def test_module_buffers_match_reference(name):
    from dkernel_b200 import LocalStrideSparseAttention
    m = META[name]
    kw = {k: (tuple(v) if isinstance(v, list) else v) for k, v in m["kwargs"].items()}
    mod = LocalStrideSparseAttention(*m["args"], **kw)
    assert mod.max_seqlen == m["max_seqlen"] and mod.block_m == m["block_m"] and mod.block_n == m["block_n"]
    for b in ("layout_csr_crow", "layout_csr_col", "layout_csc_ccol", "layout_csc_row"):
        t = getattr(mod, b)
        ref = P[f"{name}/{b}"]
        assert t.dtype == torch.int32
        assert tuple(t.shape) == ref.shape and (_np(t) == ref).all(), b
    if name == "mod_homo":
        assert mod.layout_csr_crow.stride(0) == 0
    assert len(mod.state_dict()) == 0          # buffers are non-persistent, as in the reference
    # lru_cache on the class: equal arguments -> the same instance
    assert LocalStrideSparseAttention(*m["args"], **kw) is mod


def test_empty_and_degenerate_patterns():
    from dkernel_b200.utils import dense_to_crow_col
    z = torch.zeros((2, 4, 4), dtype=torch.uint8, device="cuda")
    crow, col = dense_to_crow_col(z)
    assert (crow == 0).all() and col.shape == (2, 0)
    z[1, 3, 2] = 1
    crow, col = dense_to_crow_col(z)
    assert col.shape == (2, 1) and col[0, 0].item() == -1 and col[1, 0].item() == 2
    assert crow[1].tolist() == [0, 0, 0, 0, 1]
    big = (torch.rand((3, 300, 2100), device="cuda") < 0.3).to(torch.uint8)   # rows longer than a block scan
    crow, col = dense_to_crow_col(big)
    ref = big.sum(-1).cumsum(-1).to(torch.int32)
    assert (crow[:, 1:] == ref).all()
    h, r = 2, 123
    nz = torch.nonzero(big[h, r]).flatten().to(torch.int32)
    assert (col[h, crow[h, r]:crow[h, r + 1]] == nz).all()
