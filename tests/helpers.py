"""Shared test utilities: seeded inputs, tolerances of the parity bar."""
import json
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# parity bar: bf16/fp16 outputs vs the fp32 oracle
OUT_MAX_ABS = 2e-2
OUT_MEAN_ABS = 2e-3
LSE_ABS = 1e-3
GRAD_REL_NORM = 5e-2


def load_patterns():
    return np.load(os.path.join(GOLDEN, "patterns.npz")), json.load(
        open(os.path.join(GOLDEN, "patterns_meta.json")))


def pattern_kwargs(meta_entry):
    kw = {k: v for k, v in meta_entry.items() if k != "kv_cache_efficient"}
    if isinstance(kw.get("local_blocks"), list):
        kw["local_blocks"] = tuple(kw["local_blocks"])
    return kw


def seeded_qkv(seed, shape_q, shape_kv, dtype, device="cpu", with_do=False):
    """N(0,1) inputs generated on the CPU (so that oracle and GPU see the same
    bits), rounded to ``dtype``."""
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(shape_q, generator=g).to(dtype)
    k = torch.randn(shape_kv, generator=g).to(dtype)
    v = torch.randn(shape_kv, generator=g).to(dtype)
    outs = [q, k, v]
    if with_do:
        outs.append(torch.randn(shape_q, generator=g).to(dtype))
    return [t.to(device) for t in outs]


def assert_out_close(out, ref, what="out", max_abs=OUT_MAX_ABS, mean_abs=OUT_MEAN_ABS):
    out = out.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(out).all(), f"{what}: non-finite values"
    d = (out - ref).abs()
    assert d.max().item() <= max_abs, f"{what}: max abs diff {d.max().item():.3e} > {max_abs}"
    assert d.mean().item() <= mean_abs, f"{what}: mean abs diff {d.mean().item():.3e} > {mean_abs}"


def assert_lse_close(lse, ref, tol=LSE_ABS):
    lse = lse.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert lse.shape == ref.shape, f"lse: shape {tuple(lse.shape)} vs {tuple(ref.shape)}"
    inf_ref = torch.isinf(ref)
    assert (torch.isinf(lse) == inf_ref).all(), "lse: -inf pattern differs"
    d = (lse[~inf_ref] - ref[~inf_ref]).abs()
    if d.numel():
        assert d.max().item() <= tol, f"lse: max abs diff {d.max().item():.3e} > {tol}"


def assert_grad_close(g, ref, what, tol=GRAD_REL_NORM):
    g = g.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert g.shape == ref.shape
    assert torch.isfinite(g).all(), f"{what}: non-finite values"
    rel = (g - ref).norm() / ref.norm().clamp_min(1e-12)
    assert rel.item() <= tol, f"{what}: relative norm error {rel.item():.3e} > {tol}"
