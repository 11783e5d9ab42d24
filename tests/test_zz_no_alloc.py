"""GPU test of kd_attn_bwd_static, the backward entry point for hosts that may not allocate device
memory where they call it (its `delta` scratch is a fixed array inside the library).

Called through the C ABI with ctypes, twice in a row on different inputs, and compared with the
regular kd_attn_bwd on the same inputs. Collected last on purpose: a failure here must not keep
the other tests from running under `-x`.
"""
import ctypes

import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import assert_close, rand_inputs

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_both(seed, B=2, H=3, T=384, D=64, dtype=torch.bfloat16, ranges=None, phases=0):
    from kerneldev_b200 import _capi
    from kerneldev_b200.original_kernel import _forward, _kd_tensor, _params
    from kerneldev_b200.plan import AttentionPlan

    lib = _capi.load()
    ranges = ranges or dict(prefix=(8, 40), context=(64, 160), n_spans=(2, 6), span_len=(8, 40))
    ins, sid, pre, lens = ao.batch_metadata(seed, B, T, **ranges)
    dev = torch.device(DEV)
    t = lambda a, dt: torch.as_tensor(a, dtype=dt, device=dev)
    plan = AttentionPlan(B, T, dev, t(ins, torch.bool), t(sid, torch.int64), t(pre, torch.bool), t(lens, torch.int32), True, True)
    g = torch.Generator(device=dev).manual_seed(seed)
    q, k, v, do = (torch.randn((B, H, T, D), generator=g, device=dev, dtype=dtype) for _ in range(4))
    scale = D ** -0.5
    o, lse = _forward(q, k, v, plan, scale)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def call(entry, with_delta):
        dq, dk, dv = (torch.full_like(q, float("nan")) for _ in range(3))
        p = _params(q, k, v, o, lse, plan, scale)
        p.d_o = _kd_tensor(do)
        p.dq, p.dk, p.dv = _kd_tensor(dq), _kd_tensor(dk), _kd_tensor(dv)
        delta = torch.empty((B, H, T), dtype=torch.float32, device=dev) if with_delta else None
        p.delta = delta.data_ptr() if with_delta else None
        p.bwd_phases = phases
        _capi.check(entry(ctypes.byref(p), stream))
        torch.cuda.synchronize()
        plan.check_status()
        return dq, dk, dv

    ref = call(lib.kd_attn_bwd, True)
    got = call(lib.kd_attn_bwd_static, False)
    return ref, got


def test_static_scratch_backward_matches_regular_backward_twice():
    for seed in (101, 202):   # two calls in a row share the one scratch array
        ref, got = _run_both(seed)
        for name, r, g in zip(("dQ", "dK", "dV"), ref, got):
            assert torch.isfinite(g.float()).all(), f"{name}: non-finite values"
            assert_close(name, g, r.float())


def test_static_scratch_backward_fp16_head_dim_128():
    ref, got = _run_both(303, B=2, H=2, T=520, D=128, dtype=torch.float16, phases=3)
    for name, r, g in zip(("dQ", "dK", "dV"), ref, got):
        assert_close(name, g, r.float())


def test_static_scratch_backward_at_the_row_limit():
    """B*H*T = 1,048,576 rows fill the built-in scratch exactly and are accepted (BASELINE config 2's shape)."""
    ref, got = _run_both(404, B=16, H=16, T=4096, D=64, ranges=ao.CONFIG_RANGES[2])
    for r, g in zip(ref, got):
        assert torch.equal(r, g)


def test_static_scratch_backward_rejects_oversized_problems():
    from kerneldev_b200 import _capi
    lib = _capi.load()
    p = _capi.KdAttnParams()
    p.B, p.H, p.T, p.D = 64, 64, 4096, 64      # 16.8 M rows > 1,048,576
    p.dtype, p.sm_scale = _capi.KD_BF16, 0.125
    rc = lib.kd_attn_bwd_static(ctypes.byref(p), None)
    assert rc == -4
    assert b"exceed" in lib.kd_last_error()
    # just above the limit (2**20 + 1 has no factorisation with T <= 16384; this is 69 rows above)
    p.B, p.H, p.T = 1, 65, 16133
    assert p.B * p.H * p.T > 2 ** 20 and lib.kd_attn_bwd_static(ctypes.byref(p), None) == -4
    # a dK/dV-only pass would read another call's delta out of the shared scratch: rejected
    p.B, p.H, p.T, p.bwd_phases = 1, 1, 128, 2
    assert lib.kd_attn_bwd_static(ctypes.byref(p), None) == -1
    assert b"bwd_phases" in lib.kd_last_error()
