"""Shared helpers of the parity tests: seeded inputs, oracle calls, tolerance checks."""
import os

import numpy as np
import torch

from oracle import attention_oracle as ao

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")

# Tolerances of the operator against the fp32 oracle evaluated on the same 16-bit-rounded inputs.
ATOL, RTOL = 2e-2, 1e-2
LSE_TOL = 1e-3


def load_golden(name):
    d = dict(np.load(os.path.join(GOLDEN, name + ".npz")))
    B, H, T, D = (int(x) for x in d["shape"])
    g = torch.Generator().manual_seed(int(d["seed"]))
    q, k, v, do = (torch.randn((B, H, T, D), generator=g) for _ in range(4))
    sums = np.array([float(x.double().sum()) for x in (q, k, v, do)])
    assert np.allclose(sums, d["input_sums"], rtol=0, atol=1e-6), "torch CPU generator differs from the fixture's"
    d.update(q=q, k=k, v=v, do=do)
    return d


def golden_mask(d):
    T = int(d["shape"][2])
    has_meta = "in_span" in d
    return ao.dense_mask(T, d.get("in_span"), d.get("span_id"), d.get("is_prefix"), d.get("lens"),
                         causal=bool(d["causal_fwd"]), B=int(d["shape"][0])), has_meta


def rand_inputs(B, H, T, D, dtype, seed, device="cpu", outlier_frac=0.0):
    g = torch.Generator().manual_seed(seed)
    ts = []
    for i in range(4):
        x = torch.randn((B, H, T, D), generator=g)
        if outlier_frac > 0 and i < 3:
            sel = torch.rand((B, H, T, D), generator=g) < outlier_frac
            x = torch.where(sel, torch.randn((B, H, T, D), generator=g) * 20.0, x)
        ts.append(x.to(dtype).to(device))
    return ts


def random_meta(seed, B, T, p_span=0.35, p_prefix=0.25, sid_range=(-1, 4)):
    """Non-canonical metadata: independent flags that may overlap, arbitrary small span ids."""
    rng = np.random.default_rng(seed)
    ins = rng.random((B, T)) < p_span
    pre = rng.random((B, T)) < p_prefix
    sid = rng.integers(sid_range[0], sid_range[1], size=(B, T)).astype(np.int64)
    return ins, sid, pre


def assert_close(name, got, ref, atol=ATOL, rtol=RTOL):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, f"{name}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{name}: non-finite values"
    err = (got - ref).abs()
    bound = atol + rtol * ref.abs()
    bad = err > bound
    if bad.any():
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{name}: {int(bad.sum())} of {bad.numel()} elements outside atol={atol} rtol={rtol}; "
            f"max err {float(err.max()):.4g}; first at {idx}: got {float(got[tuple(idx)]):.5g} ref {float(ref[tuple(idx)]):.5g}")


def assert_lse_close(got, ref, tol=LSE_TOL):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    inf_ref = torch.isinf(ref)
    assert torch.equal(torch.isinf(got) & (got < 0), inf_ref), "LSE: rows without keys must be -inf exactly where the oracle's are"
    err = (got[~inf_ref] - ref[~inf_ref]).abs()
    # base-2 LSE of bf16-rounded P sums: absolute tolerance relative to magnitude 1
    assert err.numel() == 0 or float(err.max()) <= tol * max(1.0, float(ref[~inf_ref].abs().max())), \
        f"LSE: max err {float(err.max()):.3g}"
