"""GPU parity of kd_metadata_from_tokens (through the C ABI) with the oracle and with the fixture made
by the reference's own code (model.py:203-238): bit-exact integer / boolean outputs."""
import os

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "metadata_from_tokens.npz")


def _run(tokens_np):
    from kerneldev_b200 import metadata_from_tokens
    x = torch.as_tensor(tokens_np, dtype=torch.int64, device=DEV)
    ins, sid, pre = metadata_from_tokens(x)
    assert ins.dtype == torch.bool and sid.dtype == torch.int64 and pre.dtype == torch.bool
    return ins.cpu().numpy(), sid.cpu().numpy(), pre.cpu().numpy()


def test_reference_fixture():
    z = np.load(GOLDEN)
    for name in "abcd":
        ins, sid, pre = _run(z[f"{name}_tokens"])
        assert np.array_equal(ins, z[f"{name}_in_span"]), name
        assert np.array_equal(sid, z[f"{name}_span_id"]), name
        assert np.array_equal(pre, z[f"{name}_is_prefix"]), name


@pytest.mark.parametrize("B,T", [(1, 1), (3, 255), (2, 256), (4, 257), (16, 4096), (2, 16384)])
def test_random_rows_against_oracle(B, T):
    rng = np.random.default_rng(B * 100003 + T)
    x = rng.integers(6, 300, size=(B, T))
    marks = rng.random((B, T)) < 0.08          # dense, unbalanced markers of every kind
    x[marks] = rng.integers(0, 6, size=int(marks.sum()))
    if B > 1:
        x[1] = np.where(x[1] < 6, 7, x[1])      # one row without any special token
    want = ao.metadata_from_tokens(x)
    got = _run(x)
    for g, w in zip(got, want):
        assert np.array_equal(g, w)


def test_strided_rows_and_operator_use():
    """Token rows taken from a wider buffer (row stride > T), and the outputs fed to the operator:
    same O as with the oracle's metadata."""
    from kerneldev_b200 import flash_attention, metadata_from_tokens
    from tests.helpers import rand_inputs
    B, T, H, D = 2, 384, 2, 64
    wide = np.full((B, T + 40), 9, np.int64)
    wide[:, 10] = 1                                               # [CLS]
    for b in range(B):
        for s0 in (100 + 7 * b, 200, 300):
            wide[b, s0] = 3; wide[b, s0 + 20] = 4                 # [SPAN] ... [ES]
        wide[b, 340] = 5                                          # [MASKQ]
    xw = torch.as_tensor(wide, device=DEV)
    x = xw[:, :T]
    assert x.stride(0) == T + 40
    ins, sid, pre = metadata_from_tokens(x)
    w_ins, w_sid, w_pre = ao.metadata_from_tokens(wide[:, :T])
    assert np.array_equal(ins.cpu().numpy(), w_ins) and np.array_equal(sid.cpu().numpy(), w_sid) and np.array_equal(pre.cpu().numpy(), w_pre)
    q, k, v, _ = (t.to(DEV) for t in rand_inputs(B, H, T, D, torch.bfloat16, seed=5))
    o1 = flash_attention(q, k, v, in_span=ins, span_id=sid, is_prefix=pre)
    o2 = flash_attention(q, k, v, in_span=torch.as_tensor(w_ins, device=DEV), span_id=torch.as_tensor(w_sid, device=DEV),
                         is_prefix=torch.as_tensor(w_pre, device=DEV))
    assert torch.equal(o1, o2)


def test_rejects_bad_inputs():
    from kerneldev_b200 import metadata_from_tokens
    with pytest.raises(ValueError):
        metadata_from_tokens(torch.zeros((2, 8), dtype=torch.int32, device=DEV))
    with pytest.raises(RuntimeError):
        metadata_from_tokens(torch.zeros((2, 8), dtype=torch.int64))
