"""Host-side layout bookkeeping of the kernels' plan, on CPU tensors built with the oracle's layouts."""
import numpy as np
import torch

from oracle import dkernel_oracle as O


def _plan(mask: np.ndarray):
    from dkernel_b200.ops import _Plan
    crow, col = O.dense_to_crow_col(mask)
    ccol, row = O.dense_to_ccol_row(mask)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(torch.int32)
    nnz = int((crow[:, 1:] - crow[:, :-1]).max())
    return _Plan(t(crow), t(col), t(ccol), t(row), 64, nnz)


def test_csc_to_csr_names_the_same_block():
    rng = np.random.default_rng(0)
    for H, R, Cn, dens in ((1, 5, 5, 0.5), (3, 16, 16, 0.3), (2, 7, 12, 0.6), (2, 9, 4, 0.0)):
        mask = (rng.random((H, R, Cn)) < dens).astype(np.uint8)
        if dens > 0:
            mask[:, 0, 0] = 1
        plan = _plan(mask)
        m = plan.csc_to_csr()
        assert m.shape == plan.row.shape and m.dtype == torch.int32
        crow, col, ccol, row = (x.numpy() for x in (plan.crow, plan.col, plan.ccol, plan.row))
        for h in range(H):
            for c in range(Cn):
                for j in range(ccol[h, c], ccol[h, c + 1]):
                    r = row[h, j]
                    i = int(m[h, j])
                    assert crow[h, r] <= i < crow[h, r + 1] and col[h, i] == c
            assert (m[h, ccol[h, Cn]:] == -1).all()
        assert plan.max_head_nnz() == int(mask.reshape(H, -1).sum(1).max())
