"""CPU tests of the host side: the C ABI library loads and exports what include/kd_attention.h
declares, argument checks that run before any CUDA call, the bit-parallel mask rule, the
plan layout, and the operator's refusal to run without a CUDA device."""
import ctypes
import os
import re
import shutil
import subprocess

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from kerneldev_b200 import _capi
    lib = _capi.load()
    header = open(os.path.join(ROOT, "include", "kd_attention.h")).read()
    declared = set(re.findall(r"^(?:int|const char\*)\s+(kd_\w+)\s*\(", header, flags=re.M))
    assert declared, "no declarations found in the header"
    assert declared == set(_capi.EXPORTS)
    for name in declared:
        assert getattr(lib, name) is not None
    assert lib.kd_version() >= 1


def test_plan_layout_is_consistent():
    from kerneldev_b200 import _capi
    L = _capi.plan_layout(16, 4096)
    assert (L.NT, L.NP) == (32, 16)
    offs = [L.off_desc, L.off_summary, L.off_cls, L.off_fwd_cnt, L.off_fwd_list, L.off_bwd_cnt, L.off_bwd_list,
            L.off_tilebits, L.off_order, L.off_stats, L.off_status, L.total]
    assert offs == sorted(offs) and all(o % 256 == 0 for o in offs)
    assert L.off_summary - L.off_desc >= 16 * 32 * 128 * 4
    L = _capi.plan_layout(1, 200)
    assert (L.NT, L.NP) == (2, 1)
    with pytest.raises(_capi.KdError):
        _capi.plan_layout(1, 128 * 128 + 1)
    with pytest.raises(_capi.KdError):
        _capi.plan_layout(0, 128)


def test_entry_points_reject_bad_arguments_before_touching_cuda():
    from kerneldev_b200 import _capi
    lib = _capi.load()
    p = _capi.KdAttnParams()
    p.B, p.H, p.T, p.D = 1, 1, 128, 256         # unsupported head dim
    p.dtype, p.sm_scale = _capi.KD_BF16, 0.1
    assert lib.kd_attn_fwd(ctypes.byref(p), None) == -1
    assert b"head dim" in lib.kd_last_error()
    p.D, p.dtype = 64, 7                         # unsupported dtype
    assert lib.kd_attn_fwd(ctypes.byref(p), None) == -1
    p.dtype, p.sm_scale = _capi.KD_F16, -1.0     # bad scale
    assert lib.kd_attn_bwd(ctypes.byref(p), None) == -1
    assert b"sm_scale" in lib.kd_last_error()
    p.sm_scale = 0.1                             # no plan
    assert lib.kd_attn_fwd(ctypes.byref(p), None) == -1
    assert b"plan" in lib.kd_last_error()
    n = ctypes.c_size_t(0)
    assert lib.kd_workspace_bytes(2, 3, 5, 64, ctypes.byref(n)) == 0 and n.value == 2 * 3 * 5 * 4
    assert lib.kd_classify(None, None, None) == -1
    assert lib.kd_mask_dense(None, 1, 1, None, None) == -1


def test_operator_has_no_cpu_path():
    from kerneldev_b200 import flash_attention, hadamard_transform
    q = torch.randn(1, 1, 128, 64, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        flash_attention(q, q, q)
    with pytest.raises(ValueError):
        hadamard_transform(q)


def test_generate_hadamard_signs_matches_oracle_recipe():
    from kerneldev_b200 import generate_hadamard_signs
    from oracle import attention_oracle as ao
    s = generate_hadamard_signs(4, 64, seed=5, device="cpu")
    assert torch.equal(s, ao.generate_hadamard_signs(4, 64, seed=5))


@pytest.mark.skipif(shutil.which("nvcc") is None and not os.path.exists("/usr/local/cuda/bin/nvcc"), reason="needs nvcc to compile host code")
def test_bit_parallel_rule_equals_per_element_rule(tmp_path):
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    exe = tmp_path / "mask_rule_check"
    r = subprocess.run([nvcc, "-O1", "-o", str(exe), os.path.join(ROOT, "tests", "mask_rule_check.cu")], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    r = subprocess.run([str(exe)], capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "bad=0" in r.stdout


def _shard_worker(rank, world, port, out):
    import torch.distributed as dist
    from kerneldev_b200.sharding import shard_pairs
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    B, H = 5, 6
    lo, hi = shard_pairs(B, H, rank, world)
    mine = torch.zeros(B * H, dtype=torch.int32)
    mine[lo:hi] = 1
    dist.all_reduce(mine)
    counts = [torch.zeros(1, dtype=torch.int64) for _ in range(world)]
    dist.all_gather(counts, torch.tensor([hi - lo]))
    if rank == 0:
        out.put((mine.tolist(), [int(c) for c in counts]))
    dist.destroy_process_group()


def test_pair_sharding_covers_every_pair_once_world2():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 1000
    procs = [ctx.Process(target=_shard_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    cover, counts = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert cover == [1] * 30 and sum(counts) == 30 and max(counts) - min(counts) <= 1


def test_status_word_reporting_and_clearing_on_the_host():
    """Host half of the device status protocol: poll() reads the pinned mirror without touching the device
    tensor's stream, raises the right exception for each status bit and clears both copies, so that one
    event is reported once and a later launch on the same plan starts clean."""
    from kerneldev_b200 import _capi
    from kerneldev_b200.plan import AttentionPlan
    plan = object.__new__(AttentionPlan)          # no device: CPU tensors stand in for the two copies
    plan._status_dev = torch.zeros(1, dtype=torch.int32)
    plan._status_host = torch.zeros(1, dtype=torch.int32)
    plan.poll()                                    # clean: nothing happens
    plan._status_dev[0] = _capi.KD_STATUS_TIMEOUT | 0x104
    plan.poll()                                    # not mirrored yet: still silent
    plan.mirror_status()
    with pytest.raises(RuntimeError, match="wait site 0x104"):
        plan.poll()
    assert int(plan._status_dev[0]) == 0 and int(plan._status_host[0]) == 0
    plan.poll()
    plan._status_dev[0] = _capi.KD_STATUS_SPAN_RANGE
    with pytest.raises(ValueError, match="24 signed bits"):
        plan.check_status()
    assert int(plan._status_dev[0]) == 0
    plan._status_dev[0] = 5
    with pytest.raises(RuntimeError, match="0x00000005"):
        plan.check_status()


@pytest.mark.skipif(not os.environ.get("REFERENCE_DIR"), reason="needs a checkout of the reference project (REFERENCE_DIR)")
def test_reference_model_binds_the_dropin_operator():
    """With kerneldev_b200/dropin ahead of the reference checkout on sys.path, the reference's own model.py
    (`from original_kernel import flash_attention`, model.py:24) binds this package's operator."""
    code = (
        "import sys, functools\n"
        f"sys.path.insert(0, {os.environ['REFERENCE_DIR']!r})\n"
        f"sys.path.insert(0, {os.path.join(ROOT, 'kerneldev_b200', 'dropin')!r})\n"
        f"sys.path.insert(0, {ROOT!r})\n"
        "import model\n"
        "from kerneldev_b200.original_kernel import flash_attention as ours\n"
        "fa = model.flash_attention\n"
        "assert isinstance(fa, functools.partial) and fa.func is ours and fa.keywords == {'out_layout': 'input'}, fa\n"
        "import original_kernel\n"
        "assert original_kernel.__file__.startswith(" + repr(os.path.join(ROOT, 'kerneldev_b200', 'dropin')) + ")\n"
        "print('bound')\n")
    r = subprocess.run([os.sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "bound" in r.stdout, r.stdout + r.stderr
