"""GPU parity tests of the plan kernels: token descriptors -> dense mask and 128x128 tile
classes must equal the oracle's bit for bit, for canonical and for arbitrary metadata."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as ao
from tests.helpers import random_meta

pytestmark = pytest.mark.gpu


def _plan(T, ins=None, sid=None, pre=None, lens=None, causal=True, rules=None, B=None):
    from kerneldev_b200.plan import AttentionPlan
    dev = torch.device("cuda:0")
    t = lambda a, dt: None if a is None else torch.as_tensor(a, dtype=dt, device=dev)
    if B is None:
        B = next(x.shape[0] for x in (ins, sid, pre, lens) if x is not None)
    if rules is None:
        rules = any(x is not None for x in (ins, sid, pre))
    return AttentionPlan(B, T, dev, t(ins, torch.bool), t(sid, torch.int64), t(pre, torch.bool),
                         t(lens, torch.int32), causal, rules)


def _check(plan, mask):
    got_mask = plan.dense_mask().cpu().numpy()
    assert np.array_equal(got_mask, mask), f"dense mask differs in {int((got_mask != mask).sum())} bits"
    cls = ao.tile_classes(mask)
    got = plan.tile_classes.cpu().numpy()
    assert np.array_equal(got, cls), f"tile classes differ at {np.argwhere(got != cls)[:5].tolist()}"
    stats = plan.stats.cpu().numpy()
    assert np.array_equal(stats[:, 0], (cls == ao.FULL).sum(axis=(1, 2)))
    assert np.array_equal(stats[:, 1], (cls == ao.PARTIAL).sum(axis=(1, 2)))
    # work lists: forward list of a pair = union of non-empty key tiles; backward list per key tile
    B, NT, _ = cls.shape
    fc, bc = plan.fwd_counts.cpu().numpy(), plan.bwd_counts.cpu().numpy()
    for b in range(B):
        for p in range((NT + 1) // 2):
            rows = cls[b, 2 * p:2 * p + 2]
            assert fc[b, p] == int((rows != ao.EMPTY).any(axis=0).sum())
        for kt in range(NT):
            assert bc[b, kt] == int((cls[b, :, kt] != ao.EMPTY).sum())
    assert plan.status() == 0


def test_config0_layout():
    ins, sid, pre, lens = ao.config0_metadata()
    _check(_plan(256, ins, sid, pre, lens), ao.dense_mask(256, ins, sid, pre, lens))
    _check(_plan(256, ins, sid, pre, None), ao.dense_mask(256, ins, sid, pre, None))


@pytest.mark.parametrize("seed,T", [(0, 128), (1, 200), (2, 384), (3, 513), (4, 1000)])
def test_random_noncanonical_metadata(seed, T):
    B = 3
    ins, sid, pre = random_meta(seed, B, T)
    lens = np.array([T, max(1, T - 37), max(1, T // 2 + 1)], np.int32)
    _check(_plan(T, ins, sid, pre, lens), ao.dense_mask(T, ins, sid, pre, lens))
    _check(_plan(T, ins, sid, pre, None), ao.dense_mask(T, ins, sid, pre, None))


def test_partial_metadata_and_attention_mask_only():
    T, B = 300, 2
    ins, sid, pre = random_meta(11, B, T)
    _check(_plan(T, ins, None, None), ao.dense_mask(T, ins, None, None))
    _check(_plan(T, None, sid, None), ao.dense_mask(T, None, sid, None))
    _check(_plan(T, None, None, pre), ao.dense_mask(T, None, None, pre))
    # attention_mask given, no metadata: rule path with all-context tokens
    _check(_plan(T, rules=True, B=B, causal=False), ao.dense_mask(T, causal=False, attention_mask_given=True, B=B))


@pytest.mark.parametrize("causal", [True, False])
def test_no_metadata(causal):
    lens = np.array([500, 129, 1], np.int32)
    _check(_plan(500, lens=lens, causal=causal), ao.dense_mask(500, lens=lens, causal=causal))
    _check(_plan(256, causal=causal, B=2), ao.dense_mask(256, causal=causal, B=2))


def test_blocky_spans_exercise_summary_fast_path():
    # whole tiles of one class: prefix tile, context tiles, span tiles with uniform / mixed ids
    T = 1024
    ins = np.zeros((1, T), bool); pre = np.zeros((1, T), bool); sid = np.zeros((1, T), np.int64)
    pre[0, :128] = True
    ins[0, 384:896] = True
    sid[0, 384:512] = 1; sid[0, 512:640] = 2; sid[0, 640:700] = 3; sid[0, 700:768] = 0; sid[0, 768:896] = 2
    sid[0, 896] = -1
    for lens in (None, np.array([897], np.int32)):
        _check(_plan(T, ins, sid, pre, lens), ao.dense_mask(T, ins, sid, pre, lens))


@pytest.mark.parametrize("cfg,B,T", [(2, 4, 4096), (3, 2, 8192), (4, 4, 2048)])
def test_baseline_config_generators(cfg, B, T):
    ins, sid, pre, lens = ao.batch_metadata(cfg, B, T, **ao.CONFIG_RANGES[cfg])
    plan = _plan(T, ins, sid, pre, lens)
    got = plan.tile_classes.cpu().numpy()
    dm = plan.dense_mask().cpu().numpy()
    for b in range(B):
        mask = ao.dense_mask(T, ins[b:b + 1], sid[b:b + 1], pre[b:b + 1], lens[b:b + 1])
        assert np.array_equal(dm[b:b + 1], mask)
        assert np.array_equal(got[b:b + 1], ao.tile_classes(mask))


def test_span_id_out_of_range_is_reported():
    T = 128
    sid = np.zeros((1, T), np.int64); sid[0, 5] = 1 << 30
    ins = np.zeros((1, T), bool); ins[0, 5] = True
    with pytest.raises(ValueError, match="span_id"):
        _plan(T, ins, sid, None)
