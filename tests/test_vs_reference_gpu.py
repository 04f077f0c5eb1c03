"""This repository's CUDA kernels against the UNMODIFIED reference running its own Triton kernels on
the same GPU (installed under baseline/_ref by `pip install --no-deps --target baseline/_ref`).
The CPU oracle cannot be checked against reference OUTPUTS on the padded / variable-length / decode
routes (the reference evaluates those only with Triton); these tests do that where a GPU and the
install are present, and are skipped otherwise.  Test side only: the product never imports it."""
import math
import os
import sys

import numpy as np
import pytest
import torch

from helpers import assert_out_close, seeded_qkv

pytestmark = pytest.mark.gpu

REF_DIR = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "baseline", "_ref")


@pytest.fixture(scope="module")
def ref():
    if not os.path.isdir(os.path.join(REF_DIR, "dkernel")):
        pytest.skip("baseline/_ref (the reference package) is not installed")
    try:
        import triton  # noqa: F401
    except Exception as e:  # pragma: no cover
        pytest.skip(f"triton is not importable: {e}")
    sys.path.insert(0, REF_DIR)
    try:
        import dkernel
    finally:
        sys.path.remove(REF_DIR)
    return dkernel


def _both(ref, Hq, Hkv, S, pk):
    from dkernel_b200 import LocalStrideSparseAttention
    mine = LocalStrideSparseAttention.__wrapped__(Hq, S, pk["block_size"], pk["local_blocks"], pk["vert_stride"],
                                                  num_kv_heads=Hkv, seq_dim=1)
    theirs = ref.LocalStrideSparseAttention.__wrapped__(Hq, S, pk["block_size"], pk["local_blocks"],
                                                        pk["vert_stride"], num_kv_heads=Hkv, seq_dim=1)
    # the published layouts are bit-identical
    for name in ("layout_csr_crow", "layout_csr_col", "layout_csc_ccol", "layout_csc_row"):
        assert torch.equal(getattr(mine, name).cpu(), getattr(theirs, name).cpu()), name
    return mine, theirs.cuda()


def _run_ref(fn):
    try:
        out = fn()
        torch.cuda.synchronize()
        return out
    except AssertionError:
        raise
    except Exception as e:      # a Triton / API incompatibility of the reference is not this repository's failure
        pytest.skip(f"the reference did not run here: {type(e).__name__}: {str(e)[:200]}")


def test_unpadded_forward_matches_reference_kernels(ref):
    B, S, Hq, Hkv, D = 2, 1024, 8, 2, 128
    pk = dict(block_size=64, local_blocks=4, vert_stride=4)
    mine, theirs = _both(ref, Hq, Hkv, S, pk)
    q, k, v = seeded_qkv(71, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16, device="cuda")
    kr, vr = k.repeat_interleave(Hq // Hkv, 2), v.repeat_interleave(Hq // Hkv, 2)   # its training-path kernel has no GQA
    with torch.no_grad():
        want = _run_ref(lambda: theirs(q, kr, vr))
        got = mine(q, k, v)
    assert_out_close(got, want, max_abs=2e-2, mean_abs=1e-3)


def test_padded_and_decode_routes_match_reference_kernels(ref):
    B, S, Hq, Hkv, D = 3, 1024, 8, 2, 128
    pk = dict(block_size=64, local_blocks=4, vert_stride=4)
    mine, theirs = _both(ref, Hq, Hkv, S, pk)
    q, k, v = seeded_qkv(72, (B, S, Hq, D), (B, S, Hkv, D), torch.bfloat16, device="cuda")
    lens = torch.tensor([1024, 300, 77])
    left = (S - lens).cuda()
    with torch.no_grad():
        want = _run_ref(lambda: theirs(q, k, v, left_paddings=left))
        got = mine(q, k, v, left_paddings=left)
    for b in range(B):      # the reference leaves pad rows unspecified in places; compare the real rows
        lo = int(left[b])
        assert_out_close(got[b, lo:], want[b, lo:], max_abs=2e-2, mean_abs=1e-3)
    # decode: one query token per sequence against the left-padded cache
    qd = q[:, -1:].contiguous()
    with torch.no_grad():
        want = _run_ref(lambda: theirs(qd, k, v, left_paddings=left))
        got = mine(qd, k, v, left_paddings=left)
    assert_out_close(got, want, max_abs=2e-2, mean_abs=1e-3)


def test_varlen_route_matches_reference_kernels(ref):
    Hq, Hkv, D = 8, 2, 128
    pk = dict(block_size=64, local_blocks=4, vert_stride=4)
    mine, theirs = _both(ref, Hq, Hkv, 1024, pk)
    lens = [512, 100, 333, 64]
    T = sum(lens)
    q, k, v = seeded_qkv(73, (T, Hq, D), (T, Hkv, D), torch.bfloat16, device="cuda")
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32, device="cuda")
    with torch.no_grad():
        want = _run_ref(lambda: theirs(q, k, v, cu_seqlen_k=cu))
        got = mine(q, k, v, cu_seqlen_k=cu)
    assert_out_close(got, want, max_abs=2e-2, mean_abs=1e-3)
