"""GPU parity of the span-mean head (kd_span_index, kd_span_mean through the C ABI) with the oracle
and with the fixture made by the reference's own code (model.py:258-296)."""
import os
import sys

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GDIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
sys.path.insert(0, GDIR)
from cocktail_inputs import CASES, cocktail_rows, embeddings  # noqa: E402
sys.path.pop(0)


def test_reference_fixture():
    from kerneldev_b200 import cocktail_scores, span_means
    z = np.load(os.path.join(GDIR, "cocktail_head.npz"))
    for name, (seed, B, T, D) in CASES.items():
        x, e = cocktail_rows(seed, B, T).to(DEV), embeddings(seed, B, T, D).to(DEV)
        h = span_means(e, x)
        np.testing.assert_allclose(h.cpu().numpy(), z[f"{name}_h_spans"], rtol=1e-5, atol=1e-6)
        np.testing.assert_allclose(cocktail_scores(e, x).cpu().numpy(), z[f"{name}_scores"], rtol=1e-4, atol=1e-4)


def test_span_index_is_exact():
    from kerneldev_b200 import span_index
    rng = np.random.default_rng(5)
    B, T = 5, 1000
    x = rng.integers(6, 100, size=(B, T))
    marks = rng.random((B, T)) < 0.1
    x[marks] = rng.integers(0, 6, size=int(marks.sum()))
    x[4] = 9                                            # no markers at all
    starts, ends, n_s, n_e, fm = (t.cpu().numpy() for t in span_index(torch.as_tensor(x, device=DEV)))
    for b in range(B):
        s = np.nonzero(x[b] == 3)[0]; e = np.nonzero(x[b] == 4)[0]; m = np.nonzero(x[b] == 2)[0]
        assert n_s[b] == len(s) and n_e[b] == len(e)
        assert np.array_equal(starts[b, :len(s)], s) and (starts[b, len(s):] == -1).all()
        assert np.array_equal(ends[b, :len(e)], e) and (ends[b, len(e):] == -1).all()
        assert fm[b] == (m[0] if len(m) else -1)


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2), (torch.float16, 2e-3)])
def test_forward_and_backward_against_oracle(dtype, tol):
    """h_spans, scores and the gradient with respect to x_embed (autograd through the oracle on CPU in
    fp32) for rows with overlapping pairs (an [ES] ahead of the first [SPAN]), empty pairs, rows
    without [MASK] and a strided embedding tensor."""
    from kerneldev_b200 import cocktail_scores
    seed, B, T, D = 21, 6, 257, 96
    x = cocktail_rows(seed, B, T, unbalanced=True)
    e32 = embeddings(seed, B, T, D)
    e_dev = torch.empty((B, T, D + 8), dtype=dtype, device=DEV)[:, :, :D]      # row stride D + 8
    e_dev.copy_(e32.to(dtype))
    e_dev.requires_grad_()
    e_ref = e_dev.detach().float().cpu().requires_grad_()
    scores = cocktail_scores(e_dev, x.to(DEV))
    want, _ = ao.cocktail_scores(e_ref, x)
    assert scores.shape == want.shape
    torch.testing.assert_close(scores.float().cpu(), want.detach(), rtol=tol, atol=tol * max(1.0, float(want.detach().abs().max())))
    g = torch.randn(want.shape, generator=torch.Generator().manual_seed(3))
    scores.backward(g.to(DEV, dtype))
    want.backward(g)
    torch.testing.assert_close(e_dev.grad.float().cpu(), e_ref.grad, rtol=tol, atol=tol * max(1.0, float(e_ref.grad.abs().max())))


def test_batch_without_spans_and_bad_inputs():
    from kerneldev_b200 import span_means
    x = torch.full((2, 40), 9, dtype=torch.int64, device=DEV)
    e = torch.randn((2, 40, 16), device=DEV)
    assert span_means(e, x).shape == (2, 0, 16)
    with pytest.raises(ValueError):
        span_means(e.double(), x)
    with pytest.raises(RuntimeError):
        span_means(e.cpu(), x)
