"""GPU test of the bounded waits: a wait that cannot be satisfied gives up by itself, the kernel unwinds and
reports it, the Python layer raises, and the next launch on the same device is correct.

The failure is made in the allowed form only. A TEST BUILD of the library (-DKD_TEST_DROP_LOAD, wait limit
20 ms instead of 0.4 s) lets the TMA producer of one CTA leave out one K tile load when the environment
variable KD_TEST_DROP_LOAD=1 is set at launch: no copy is issued and no bytes are expected, so nothing is in
flight for that stage. The first wait on the starved chain (the S issuer's for the tile, or a softmax warp's for
the scores) runs out after 20 ms, records
KD_STATUS_TIMEOUT | wait site in the plan's status word, raises the CTA's abort flag, and every role returns
through its normal exit (copies in flight drained with a bounded wait, TMEM freed). Nothing traps, faults or
spins without a limit. The test runs in a child process because the package binds one library per process.
"""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WAITTEST_FLAGS = ("-DKD_TEST_DROP_LOAD", "-DKD_WAIT_LIMIT_NS=20000000ull")

CHILD = r"""
import os, sys
sys.path.insert(0, %(root)r)
import numpy as np, torch
from kerneldev_b200 import _capi, flash_attention
from kerneldev_b200 import plan as plan_module
from oracle import attention_oracle as ao
assert "waittest" in str(_capi.LIB_PATH)
dev = torch.device("cuda:0")
B, H, T, D = 1, 2, 384, 64
g = torch.Generator().manual_seed(5)
q, k, v = (torch.randn((B, H, T, D), generator=g).to(torch.bfloat16).to(dev) for _ in range(3))

os.environ["KD_TEST_DROP_LOAD"] = "0"
flash_attention(q, k, v, causal=True)                  # warm-up: the first launch on a cold GPU loads the module and ramps the clocks
torch.cuda.synchronize()
assert next(iter(plan_module._CACHE.values())).status() == 0
os.environ["KD_TEST_DROP_LOAD"] = "1"
o_bad = flash_attention(q, k, v, causal=True)          # returns: the failure is on the device
torch.cuda.synchronize()                               # the kernel ended by itself
plan = next(iter(plan_module._CACHE.values()))        # the plan the call above built; get_plan() would already raise
raw = int(plan._status_host[0]) & 0xFFFFFFFF
# whichever wait on the starved chain ran out first: the S issuer's for the K tile (0x104) or a softmax warp's for the scores (0x107)
assert raw in (_capi.KD_STATUS_TIMEOUT | 0x104, _capi.KD_STATUS_TIMEOUT | 0x107), hex(raw)
os.environ["KD_TEST_DROP_LOAD"] = "0"
try:
    flash_attention(q, k, v, causal=True)              # the next call on the plan raises, without a sync of its own
    raise SystemExit("no exception")
except RuntimeError as e:
    assert "timed out" in str(e) and ("0x104" in str(e) or "0x107" in str(e)), str(e)
assert plan.status() == 0                              # reported once, then cleared on the device too
o = flash_attention(q, k, v, causal=True)              # and the device is still usable and correct
torch.cuda.synchronize()
ref, _ = ao.attention_forward(q.cpu(), k.cpu(), v.cpu(), ao.dense_mask(T, causal=True))
err = (o.float().cpu() - ref).abs()
assert bool((err <= 2e-2 + 1e-2 * ref.abs()).all()), float(err.max())
print("unwound and recovered")
"""


def test_wait_timeout_unwinds_reports_and_recovers():
    from kerneldev_b200.build import build
    lib = build(name="waittest", extra_flags=WAITTEST_FLAGS)
    env = dict(os.environ, KD_LIB_PATH=str(lib))
    env.pop("KD_CHECK_STATUS", None)     # the default, asynchronous reporting is what is under test
    r = subprocess.run([sys.executable, "-c", CHILD % {"root": ROOT}], env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "unwound and recovered" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
