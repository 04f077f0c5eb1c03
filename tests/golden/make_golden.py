"""Generate the golden vectors under tests/golden/ from the reference package.

Run once, where a read-only checkout of the reference (linxihui/dkernel) is available; its
path comes from the command line or from the environment variable DKERNEL_REF:

    python tests/golden/make_golden.py <path to the dkernel checkout>

It imports the reference's own ``dkernel.utils`` / ``dkernel.interface`` and the
``torch_attention`` oracle of its test-suite on the CPU (the Triton kernels are
never launched), runs the reference's two known-answer tests, and stores

  * patterns.npz   block masks, CSR and CSC layouts (and merged/split layouts)
                   for a sweep of pattern parameters,
  * attention.npz  masked-dense attention outputs / LSE / gradients of the
                   reference oracle on small seeded inputs, and a strided
                   sample of BASELINE config 1 (B1,S1024,H8,D64 fp32),
  * combine.npz    ``combine_attn_partitions`` outputs.

The tests only read the .npz files; the reference checkout is not needed to run
them.
"""
import importlib.metadata as md
import json
import os
import sys

import numpy as np
import torch

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("DKERNEL_REF")
if not REF or not os.path.isdir(os.path.join(REF, "dkernel")):
    raise SystemExit("usage: make_golden.py <path to the dkernel checkout>   (or set DKERNEL_REF)")
HERE = os.path.dirname(os.path.abspath(__file__))

_orig_version = md.version
md.version = lambda n: "0.0.2" if n == "dkernel" else _orig_version(n)
sys.path.insert(0, REF)
sys.path.insert(0, os.path.join(REF, "tests"))

from dkernel.utils import (get_sparse_attn_mask, dense_to_crow_col, dense_to_ccol_row,  # noqa: E402
                           merge_split_fwd_kernel_blocks, is_kv_cache_efficient)
from dkernel.interface import (LocalStrideSparseAttention, SparseAttention,  # noqa: E402
                               combine_attn_partitions)
import test_sparse_attn as ref_tests  # noqa: E402
import test_utils as ref_kat  # noqa: E402


def np_(x):
    return x.detach().cpu().numpy() if isinstance(x, torch.Tensor) else np.asarray(x)


PATTERN_CASES = [
    # name, kwargs for get_sparse_attn_mask
    ("kat_causal", dict(num_heads=2, seqlen=16, block_size=2, local_blocks=2, vert_stride=3,
                        causal=True, homo_head=True)),
    ("kat_bidir", dict(num_heads=2, seqlen=16, block_size=2, local_blocks=2, vert_stride=3,
                       causal=False, homo_head=True)),
    ("c1", dict(num_heads=8, seqlen=1024, block_size=64, local_blocks=4, vert_stride=4)),
    ("c2", dict(num_heads=32, seqlen=8192, block_size=64, local_blocks=16, vert_stride=8,
                num_kv_heads=8)),
    ("c3", dict(num_heads=32, seqlen=8192, block_size=64, local_blocks=32, vert_stride=8)),
    ("homo", dict(num_heads=4, seqlen=2048, block_size=64, local_blocks=4, vert_stride=4,
                  homo_head=True)),
    ("dense_heads", dict(num_heads=8, seqlen=1024, block_size=64, local_blocks=2, vert_stride=8,
                         num_dense_heads=2)),
    ("gqa_dense", dict(num_heads=8, seqlen=1024, block_size=32, local_blocks=3, vert_stride=5,
                       num_kv_heads=4, num_dense_heads=1)),
    ("slide3", dict(num_heads=6, seqlen=1536, block_size=64, local_blocks=4, vert_stride=8,
                    head_sliding_offset=3)),
    ("few_heads", dict(num_heads=2, seqlen=2048, block_size=64, local_blocks=1, vert_stride=8)),
    ("ragged", dict(num_heads=3, seqlen=1000, block_size=64, local_blocks=10, vert_stride=3)),
    ("past", dict(num_heads=4, seqlen=2048, block_size=64, local_blocks=4, vert_stride=4,
                  past_len=64 * 21 + 12)),
    ("bs16", dict(num_heads=4, seqlen=512, block_size=16, local_blocks=4, vert_stride=4)),
    ("bs128", dict(num_heads=4, seqlen=4096, block_size=128, local_blocks=2, vert_stride=4)),
    ("bidir", dict(num_heads=4, seqlen=1024, block_size=64, local_blocks=3, vert_stride=5,
                   causal=False)),
    ("bidir_lr", dict(num_heads=4, seqlen=1024, block_size=64, local_blocks=(2, 4), vert_stride=4,
                      causal=False)),
    ("bidir_huge_stride", dict(num_heads=2, seqlen=1024, block_size=64, local_blocks=4,
                               vert_stride=10000, causal=False)),
    ("chunk", dict(num_heads=3, seqlen=512, block_size=64, local_blocks=4, vert_stride=4,
                   q_start_position=1024, kv_start_position=512, kv_seqlen=512)),
    ("chunk_diag", dict(num_heads=3, seqlen=512, block_size=32, local_blocks=4, vert_stride=4,
                        q_start_position=1024, kv_start_position=1024, kv_seqlen=512)),
    ("dense_pattern", dict(num_heads=2, seqlen=512, block_size=64, local_blocks=8, vert_stride=1)),
]


def make_patterns():
    out = {}
    meta = {}
    for name, kw in PATTERN_CASES:
        (crow, col), bm, _ = get_sparse_attn_mask(dtype=torch.uint8, **kw)
        ccol, row = dense_to_ccol_row(bm)
        out[f"{name}/mask"] = np_(bm).astype(np.uint8)
        out[f"{name}/crow"] = np_(crow)
        out[f"{name}/col"] = np_(col)
        out[f"{name}/ccol"] = np_(ccol)
        out[f"{name}/row"] = np_(row)
        meta[name] = {k: (list(v) if isinstance(v, tuple) else v) for k, v in kw.items()}
        meta[name]["kv_cache_efficient"] = bool(
            is_kv_cache_efficient(bm, kw["block_size"], kw["block_size"])) \
            if bm.size(1) == bm.size(2) else None
    # merged / split kernel-tile layouts (dkernel/utils.py:262-310)
    for name, bs, bm_, bn_ in [("bs16", 16, 64, 16), ("bs16", 16, 128, 16), ("bs128", 128, 64, 64),
                               ("bs128", 128, 128, 32), ("c1", 64, 64, 32), ("c1", 64, 128, 64)]:
        pat = torch.from_numpy(out[f"{name}/mask"])
        crow, col = merge_split_fwd_kernel_blocks(bs, pat, bm_, bn_)
        out[f"{name}/ms_{bm_}_{bn_}/crow"] = np_(crow)
        out[f"{name}/ms_{bm_}_{bn_}/col"] = np_(col)
    # a random user pattern (BASELINE config 5 style, small)
    g = torch.Generator().manual_seed(0)
    pat = (torch.rand(4, 32, 32, generator=g) < 0.2)
    pat |= torch.eye(32, dtype=torch.bool)[None]
    pat &= torch.tril(torch.ones(32, 32, dtype=torch.bool))[None]
    crow, col = dense_to_crow_col(pat.to(torch.uint8))
    ccol, row = dense_to_ccol_row(pat.to(torch.uint8))
    out["bernoulli/mask"] = np_(pat).astype(np.uint8)
    out["bernoulli/crow"], out["bernoulli/col"] = np_(crow), np_(col)
    out["bernoulli/ccol"], out["bernoulli/row"] = np_(ccol), np_(row)
    meta["bernoulli"] = {"kv_cache_efficient": bool(is_kv_cache_efficient(pat.to(torch.uint8), 64, 64))}
    # module buffers incl. active_head_range slicing (dkernel/interface.py:293-298)
    for name, args, kw in [
        ("mod_c2_shard", (32, 8192, 64, 16, 8), dict(num_kv_heads=8, active_head_range=(8, 16))),
        ("mod_small", (8, 1000, 64, 4, 4), dict()),
        ("mod_homo", (8, 1024, 64, 4, 4), dict(homo_head=True)),
    ]:
        m = LocalStrideSparseAttention.__wrapped__(*args, **kw)
        for b in ("layout_csr_crow", "layout_csr_col", "layout_csc_ccol", "layout_csc_row"):
            out[f"{name}/{b}"] = np_(getattr(m, b))
        meta[name] = {"args": list(args), "kwargs": {k: (list(v) if isinstance(v, tuple) else v)
                                                       for k, v in kw.items()},
                      "max_seqlen": m.max_seqlen, "block_m": m.block_m, "block_n": m.block_n}
    np.savez_compressed(os.path.join(HERE, "patterns.npz"), **out)
    with open(os.path.join(HERE, "patterns_meta.json"), "w") as f:
        json.dump(meta, f, indent=1, sort_keys=True)


ATTN_CASES = [
    # name, B, Hq, Hkv, S, D, dtype, seq_dim, pattern kwargs
    ("small_f32", 1, 2, 2, 256, 64, torch.float32, 2, dict(block_size=64, local_blocks=2, vert_stride=2)),
    ("gqa_f32", 1, 4, 2, 160, 32, torch.float32, 1, dict(block_size=32, local_blocks=2, vert_stride=3,
                                                          num_kv_heads=2)),
    ("ragged_bf16", 1, 2, 2, 200, 128, torch.bfloat16, 1, dict(block_size=64, local_blocks=2, vert_stride=2)),
    ("bidir_f32", 1, 2, 2, 192, 64, torch.float32, 2, dict(block_size=64, local_blocks=1, vert_stride=3,
                                                           causal=False)),
]


def make_attention():
    out = {}
    for name, B, Hq, Hkv, S, D, dt, seq_dim, pk in ATTN_CASES:
        torch.manual_seed(20)
        shp = (lambda h: (B, h, S, D)) if seq_dim == 2 else (lambda h: (B, S, h, D))
        q = torch.randn(shp(Hq)).to(dt).requires_grad_()
        k = torch.randn(shp(Hkv)).to(dt).requires_grad_()
        v = torch.randn(shp(Hkv)).to(dt).requires_grad_()
        do = torch.randn(shp(Hq)).to(dt)
        causal = pk.get("causal", True)
        _, bm, dense = get_sparse_attn_mask(Hq, S, return_dense=True, dtype=torch.uint8, **pk)
        hd = 1 if seq_dim == 2 else 2
        kk = k.repeat_interleave(Hq // Hkv, dim=hd)
        vv = v.repeat_interleave(Hq // Hkv, dim=hd)
        o = ref_tests.torch_attention(q, kk, vv, dense, 0.0078125 * 8, seq_dim=seq_dim, causal=causal)
        o.backward(do)
        # inputs are regenerated from the seed by the tests (seeded_inputs below
        # is the recipe); their checksum guards against RNG drift
        out[f"{name}/input_sum"] = np.float64(sum(t.detach().double().sum().item() for t in (q, k, v, do)))
        for n, t in (("out", o), ("dq", q.grad), ("dk", k.grad), ("dv", v.grad)):
            out[f"{name}/{n}"] = np_(t.detach().float())
        out[f"{name}/mask"] = np_(bm).astype(np.uint8)
        out[f"{name}/sm_scale"] = np.float32(0.0078125 * 8)
    # BASELINE config 1: seed 0, fp32, B1 S1024 H8 D64, seq_dim 1, scale 1/8
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 1024, 8, 64) for _ in range(3))
    _, bm, dense = get_sparse_attn_mask(8, 1024, 64, 4, 4, return_dense=True, dtype=torch.uint8)
    o = ref_tests.torch_attention(q, k, v, dense, 0.125, seq_dim=1)
    out["c1/out_sample"] = np_(o)[0, ::37, :, ::5].copy()
    out["c1/out_abs_sum"] = np.float64(o.double().abs().sum().item())
    out["c1/out_sum"] = np.float64(o.double().sum().item())
    out["c1/mask"] = np_(bm).astype(np.uint8)
    np.savez_compressed(os.path.join(HERE, "attention.npz"), **out)


def make_combine():
    out = {}
    torch.manual_seed(3)
    parts = [(torch.randn(2, 3, 17, 16), torch.randn(2, 3, 17) * 3) for _ in range(3)]
    res = combine_attn_partitions(*parts)
    for i, (o, l) in enumerate(parts):
        out[f"o{i}"], out[f"lse{i}"] = np_(o), np_(l)
    out["combined"] = np_(res)
    np.savez_compressed(os.path.join(HERE, "combine.npz"), **out)


if __name__ == "__main__":
    # the reference's own known-answer tests must pass on this machine first
    ref_kat.test_get_sparse_attn_mask_causal()
    ref_kat.test_get_sparse_attn_mask_bidirectional()
    make_patterns()
    make_attention()
    make_combine()
    print("golden vectors written to", HERE)
