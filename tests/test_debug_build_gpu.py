"""The bounds-checking build (``-DBSA_DEBUG_BOUNDS``, ``libbsa_b200_debug.so``): the kernels check their
index invariants where the indices are formed and record a violation in the wait-status block instead of
faulting.  Here the same small workloads run through the release and the checking library in child
processes: no check may fire, and the outputs must be the same bits."""
import hashlib
import json
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import hashlib, json, sys
import numpy as np, torch
sys.path.insert(0, %(root)r)
import dkernel_b200.ops as ops
from dkernel_b200 import LocalStrideSparseAttention, SparseAttention, _lib

def digest(*ts):
    h = hashlib.md5()
    for t in ts:
        h.update(torch.nan_to_num(t.detach().float(), neginf=-1e30).cpu().numpy().tobytes())
    return h.hexdigest()

out = {}
g = torch.Generator().manual_seed(5)
def rnd(*shape, dtype=torch.bfloat16):
    return torch.randn(shape, generator=g).to(dtype).cuda()

# dense grid forward + both backward routes, GQA head pairs and per-head patterns, odd lengths
for name, (B, S, Hq, Hkv, D, kw) in {
    "gqa": (2, 1088, 8, 2, 128, dict(num_kv_heads=2)),
    "mha64": (1, 777, 4, 4, 64, dict()),
}.items():
    mod = LocalStrideSparseAttention.__wrapped__(Hq, 2048, 64, 3, 4, seq_dim=1, impl="sm100", bwd_impl="sm100", **kw)
    for route, cap in (("handover", ops._DS_WS_MAX_BYTES), ("recompute", 0)):
        ops._DS_WS_MAX_BYTES, saved = cap, ops._DS_WS_MAX_BYTES
        q, k, v = rnd(B, S, Hq, D).requires_grad_(), rnd(B, S, Hkv, D).requires_grad_(), rnd(B, S, Hkv, D).requires_grad_()
        o, lse = mod(q, k, v, return_lse=True)
        o.backward(rnd(B, S, Hq, D))
        out[f"{name}_{route}"] = digest(o, lse, q.grad, k.grad, v.grad)
        ops._DS_WS_MAX_BYTES = saved
# many tiles per persistent CTA, tiles drawn from the counter
ops._DYNAMIC_TILES_FROM = 0
mod = LocalStrideSparseAttention.__wrapped__(8, 4096, 64, 4, 8, num_kv_heads=2, seq_dim=1, impl="sm100")
with torch.no_grad():
    o, lse = mod(rnd(2, 4096, 8, 128), rnd(2, 4096, 2, 128), rnd(2, 4096, 2, 128), return_lse=True)
    out["many_tiles"] = digest(o, lse)
    # left-padded batch and decode on the same module
    lens = torch.tensor([4096, 300])
    o, lse = mod(rnd(2, 4096, 8, 128), rnd(2, 4096, 2, 128), rnd(2, 4096, 2, 128),
                 left_paddings=(4096 - lens).cuda(), return_lse=True)
    out["padded"] = digest(o, lse)
    o, lse = mod(rnd(2, 1, 8, 128), rnd(2, 4096, 2, 128), rnd(2, 4096, 2, 128),
                 left_paddings=(4096 - lens).cuda(), return_lse=True)
    out["decode"] = digest(o, lse)
    # packed batch, user pattern with 32-token blocks (coarsened tiles with bit masks)
    nb = 32
    pat = torch.rand(4, nb, nb, generator=g) < 0.3
    pat |= torch.eye(nb, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(nb, nb, dtype=torch.bool))[None]
    lens = [512, 100, 333, 64, 1, 700]
    cu = torch.tensor([0] + list(np.cumsum(lens)), dtype=torch.int32).cuda()
    import warnings
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        m2 = SparseAttention(32, pat.cuda(), impl="sm100")
    T = sum(lens)
    o, lse = m2(rnd(T, 4, 128), rnd(T, 4, 128), rnd(T, 4, 128), cu_seqlen_k=cu, return_lse=True)
    out["packed_fine"] = digest(o, lse)
torch.cuda.synchronize()
out["wait_status"] = _lib.wait_status()
print("RESULT " + json.dumps(out))
"""


def _run(lib):
    env = dict(os.environ)
    env.pop("BSA_B200_LIB", None)
    if lib:
        env["BSA_B200_LIB"] = lib
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], env=env, capture_output=True, text=True,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-3000:]
    line = [x for x in r.stdout.splitlines() if x.startswith("RESULT ")][-1]
    return json.loads(line[len("RESULT "):])


def test_checking_build_fires_no_check_and_gives_the_same_bits():
    from dkernel_b200 import _build
    debug_lib = _build.LIB_DEBUG
    if not os.path.exists(debug_lib):
        _build.build(debug=True)
    release = _run(None)
    checked = _run(debug_lib)
    assert release["wait_status"] == 0
    assert checked["wait_status"] == 0, f"bounds check {checked['wait_status']} fired"
    assert release == checked
