"""CPU tests: the oracle against the reference's own kernels (golden fixtures) and against
first principles (autograd of the dense math)."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import golden_mask, load_golden


@pytest.mark.parametrize("name", ["config0_lens", "config0_nolens", "random_meta_lens", "causal_plain"])
def test_oracle_matches_reference_kernels(name):
    d = load_golden(name)
    mask, _ = golden_mask(d)
    o, lse, dq, dk, dv = ao.attention_fwd_bwd(d["q"], d["k"], d["v"], d["do"], mask, float(d["scale"]))
    ref_lse = torch.from_numpy(d["lse"])
    # rows the reference leaves as NaN (beyond lens, or without a visible key) are -inf here
    valid = torch.isfinite(ref_lse)
    assert valid.float().mean() > 0.7
    assert torch.isinf(lse[~valid]).all()
    assert torch.allclose(lse[valid], ref_lse[valid], atol=2e-5, rtol=0)
    ref_o = torch.from_numpy(d["o"])
    assert torch.allclose(o[valid], ref_o[valid], atol=2e-5, rtol=1e-5)
    assert (ref_o[~valid] == 0).all() or not torch.isfinite(ref_o[~valid]).all()
    for nm, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        ref = torch.from_numpy(d[nm])
        assert torch.isfinite(ref).all()
        assert torch.allclose(got, ref, atol=3e-5, rtol=1e-4), f"{nm}: max err {float((got - ref).abs().max())}"


def test_mask_matches_reference_mask_dump():
    d = load_golden("random_meta_lens")
    B, _, T, _ = (int(x) for x in d["shape"])
    ref = np.unpackbits(d["mask"], axis=-1)[..., :T].astype(bool)
    mine = ao.dense_mask(T, d["in_span"], d["span_id"], d["is_prefix"], d["lens"], causal=False)
    assert mine.shape == ref.shape == (B, T, T)
    assert np.array_equal(mine, ref)


def test_config0_mask_counts():
    ins, sid, pre, lens = ao.config0_metadata()
    assert int(ao.dense_mask(256, ins, sid, pre, lens)[0].sum()) == 24112
    assert int(ao.dense_mask(256, ins, sid, pre, None)[0].sum()) == 27832


def test_mask_semantics_canonical_layout():
    ins, sid, pre, lens = ao.config0_metadata(B=1)
    m = ao.dense_mask(256, ins, sid, pre, lens)[0]
    assert m[:16, :16].all() and not m[:16, 16:].any()              # prefix sees prefix only
    assert m[100, :16].all() and m[100, 16:101].all() and not m[100, 101:].any()  # context: prefix + causal
    assert m[150, 16:144].all()                                      # span sees ALL context keys
    assert m[150, 144:156].all() and not m[150, 156:240].any()       # own span only
    assert not m[150, :16].any()                                     # span does not see the prefix
    assert m[240, :16].all() and m[240, 144:240].all() and not m[240, 16:144].any()  # MASKQ: prefix + spans
    assert not m[:, 240].any()                                       # nobody sees the MASKQ key
    assert not m[241:].any() and not m[:, 241:].any()                # beyond lens


def test_no_metadata_fallbacks():
    assert np.array_equal(ao.dense_mask(5, causal=True)[0], np.tril(np.ones((5, 5), bool)))
    assert ao.dense_mask(5, causal=False)[0].all()
    m = ao.dense_mask(5, causal=False, attention_mask_given=True)[0]   # rule path with all-context tokens
    assert np.array_equal(m, np.tril(np.ones((5, 5), bool)))
    m = ao.dense_mask(6, lens=np.array([4], np.int32), causal=False)[0]
    assert m[:4, :4].all() and not m[4:].any() and not m[:, 4:].any()


def test_tile_classes_exact_on_ragged_edge():
    mask = np.tril(np.ones((1, 200, 200), bool))
    cls = ao.tile_classes(mask)
    assert cls.tolist() == [[[ao.PARTIAL, ao.EMPTY], [ao.PARTIAL, ao.PARTIAL]]]
    mask = np.ones((1, 256, 256), bool)
    assert (ao.tile_classes(mask) == ao.FULL).all()


def test_backward_matches_autograd():
    torch.manual_seed(3)
    B, H, T, D = 2, 2, 64, 16
    ins, sid, pre = (np.random.default_rng(5).random((B, T)) < 0.3,
                     np.random.default_rng(6).integers(-1, 3, (B, T)),
                     np.random.default_rng(7).random((B, T)) < 0.3)
    mask = ao.dense_mask(T, ins, sid, pre, np.array([64, 50], np.int32))
    q, k, v, do = (torch.randn(B, H, T, D, dtype=torch.float64) for _ in range(4))
    qa, ka, va = (x.clone().requires_grad_() for x in (q, k, v))
    s = (qa @ ka.transpose(-1, -2)) * D ** -0.5
    s = s.masked_fill(~torch.as_tensor(mask)[:, None], float("-inf"))
    p = torch.softmax(s, -1)
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
    (p @ va).backward(do)
    o, lse, dq, dk, dv = ao.attention_fwd_bwd(q, k, v, do, mask)
    assert torch.allclose(dq.double(), qa.grad, atol=1e-4)
    assert torch.allclose(dk.double(), ka.grad, atol=1e-4)
    assert torch.allclose(dv.double(), va.grad, atol=1e-4)
    nat = torch.logsumexp(s, -1)
    ok = torch.isfinite(nat)
    assert torch.allclose(lse.double()[ok], nat[ok] * ao.LOG2E, atol=1e-4)


def test_generators_are_seeded_and_fit():
    a = ao.batch_metadata(0, 4, 4096, **ao.CONFIG_RANGES[2])
    b = ao.batch_metadata(0, 4, 4096, **ao.CONFIG_RANGES[2])
    for x, y in zip(a, b):
        assert np.array_equal(x, y)
    ins, sid, pre, lens = a
    for r in range(4):
        n = int(lens[r])
        assert n <= 4096 and sid[r, n - 1] == -1 and not ins[r, n:].any() and not pre[r, n:].any()
        assert 32 <= pre[r].sum() <= 256


def test_hadamard_is_orthogonal_and_preserves_scores():
    s = ao.generate_hadamard_signs(3, 64, seed=1)
    assert set(s.unique().tolist()) == {-1.0, 1.0}
    x = torch.randn(1, 3, 5, 64)
    y = torch.randn(1, 3, 5, 64)
    hx, hy = ao.hadamard_transform(x, s), ao.hadamard_transform(y, s)
    assert torch.allclose(hx @ hy.transpose(-1, -2), x @ y.transpose(-1, -2), atol=1e-4)
    assert torch.allclose(ao.hadamard_matrix(4), torch.tensor([[1., 1, 1, 1], [1, -1, 1, -1], [1, 1, -1, -1], [1, -1, -1, 1]]))


def test_package_generator_equals_oracle_generator():
    from kerneldev_b200 import synthetic
    for cfg, (B, T) in {2: (3, 4096), 3: (2, 8192), 4: (3, 2048)}.items():
        a = ao.batch_metadata(9, B, T, **ao.CONFIG_RANGES[cfg])
        b = synthetic.batch_metadata(9, B, T, **synthetic.CONFIG_RANGES[cfg])
        for x, y in zip(a, b):
            assert np.array_equal(x, y) and x.dtype == y.dtype


def test_metadata_from_tokens_matches_reference_fixture():
    """The token -> (in_span, span_id, is_prefix) restatement against outputs of the reference's own
    code (model.py:203-238, executed by tests/golden/make_golden_metadata.py): bit-exact, for canonical
    rows, rows without markers, unbalanced / nested markers and a batch that takes the reference's
    teacher-forcing branch."""
    import os
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "metadata_from_tokens.npz"))
    for name in "abcd":
        ins, sid, pre = ao.metadata_from_tokens(z[f"{name}_tokens"])
        assert np.array_equal(ins, z[f"{name}_in_span"]), name
        assert np.array_equal(sid, z[f"{name}_span_id"]), name
        assert np.array_equal(pre, z[f"{name}_is_prefix"]), name


def test_cocktail_head_matches_reference_fixture():
    """The span-mean head restatement against outputs of the reference's own code (model.py:258-296,
    executed by tests/golden/make_golden_cocktail.py) on the same seeded inputs."""
    import os
    import sys
    gdir = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, gdir)
    try:
        from cocktail_inputs import CASES, cocktail_rows, embeddings
    finally:
        sys.path.pop(0)
    z = np.load(os.path.join(gdir, "cocktail_head.npz"))
    for name, (seed, B, T, D) in CASES.items():
        x, e = cocktail_rows(seed, B, T), embeddings(seed, B, T, D)
        assert int(x.sum()) == int(z[f"{name}_tokens_sum"])      # the inputs are the generator's
        scores, h_spans = ao.cocktail_scores(e, x)
        assert tuple(h_spans.shape) == z[f"{name}_h_spans"].shape
        np.testing.assert_allclose(h_spans.numpy(), z[f"{name}_h_spans"], rtol=1e-6, atol=1e-6)
        np.testing.assert_allclose(scores.numpy(), z[f"{name}_scores"], rtol=1e-5, atol=1e-5)
