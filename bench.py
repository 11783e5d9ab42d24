#!/usr/bin/env python
"""Benchmark of the attention hot path: hierarchical-mask flash attention forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2]

Workload (default): BASELINE config 2 -- bf16, B=16, H=16, L=4096, D=64, hierarchical mask with
per-sequence sections drawn from a seed (prefix U[32,256], context U[1024,2048], 4..32 spans of
16..128 tokens, one MASKQ, PAD) -- on every GPU ("weak" scaling: each rank owns one such batch;
the (batch, head) pairs are independent, so there is no collective on the data path).
One step = one forward + one backward over the batch.

The one JSON line printed by rank 0:
  value      effective TFLOP/s summed over all ranks, inputs resident in HBM. Effective FLOPs =
             14*D*H*128^2 * (number of non-EMPTY 128x128 mask tiles of the batch), i.e. 4D forward
             + 10D backward per unmasked pair, recomputation not counted.
  e2e        the same metric through flash_attention() + autograd with HOST (pinned) buffers: every
             step copies Q, K, V, dO host->device and O, dQ, dK, dV device->host.
  roofline   dominant kernel: algorithmic FLOPs per launch / its CUDA-event time, against the
             measured bf16 peak of MEASURED_PEAKS.json.
  cpu_baseline  the CPU oracle (dense-masked fp32 torch math) on a bounded sample, on the host cores.

--impl reference times the CPU restatement of the reference algorithm (oracle/) on the host cores
for the same workload, metric and unit; it is the only other place this file executes oracle/.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "Hier-mask flash-attn fwd+bwd effective TFLOP/s (sum over GPUs; per-GPU % of bf16 tensor peak alongside)"
UNIT = "TFLOP/s"

CONFIGS = {
    # name: (B, H, L, D, dtype, hierarchical, hadamard)
    1: dict(B=8, H=16, L=2048, D=128, dtype="bf16", hier=False, hadamard=False,
            name="config1: causal fwd+bwd bf16 B8 H16 L2048 D128"),
    2: dict(B=16, H=16, L=4096, D=64, dtype="bf16", hier=True, hadamard=False,
            name="config2: hierarchical-mask fwd+bwd bf16 B16 H16 L4096 D64"),
    3: dict(B=4, H=32, L=8192, D=128, dtype="fp16", hier=True, hadamard=True,
            name="config3: hierarchical-mask + Hadamard fwd+bwd fp16 B4 H32 L8192 D128"),
}
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}
# DRAM bytes (dram__bytes_read.sum + dram__bytes_write.sum) per launch and per batch row of config 2,
# from the ncu capture summarised in profiles/attention_kernels_config2_batch4.md (batch 4: 99.7,
# 136.2 and 159.3 MB); traffic grows in proportion to the number of (batch, head) pairs.
NCU_TRAFFIC_PER_BATCH_ROW = {"attn_fwd_kernel": 99.7e6 / 4, "attn_bwd_dq_kernel": 136.2e6 / 4,
                             "attn_bwd_dkdv_kernel": 159.3e6 / 4}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def make_metadata(cfg, seed):
    """Seeded synthetic metadata of the config's distribution (stands in for the reference's
    cocktail-party collate, data_builder.py:463-673). Returns numpy arrays or Nones."""
    from kerneldev_b200 import synthetic
    if not cfg["hier"]:
        return None, None, None, None
    key = 3 if cfg["L"] == 8192 else 2
    return synthetic.batch_metadata(seed, cfg["B"], cfg["L"], **synthetic.CONFIG_RANGES[key])


def effective_flops(cfg, nonempty_tiles):
    return 14.0 * cfg["D"] * cfg["H"] * 128.0 * 128.0 * nonempty_tiles


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled in the background during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100",
                 "-i", str(self.gpu_index)], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out.update(sm_mhz=float(np.median(sm)), sm_max_mhz=float(max(mx)), reasons=sorted(reasons), samples=len(sm))
        return out


# --------------------------------------------------------------------------------------------
# CPU oracle timing (cpu_baseline leg and --impl reference)
# --------------------------------------------------------------------------------------------
def time_cpu_oracle(cfg, seed, budget_s, max_heads=None):
    """Runs the oracle's dense-masked fp32 forward+backward head by head on batch row 0 until
    `budget_s` seconds are spent. Returns (effective TFLOP/s, description, seconds, heads)."""
    from oracle import attention_oracle as ao
    torch.set_num_threads(os.cpu_count() or 1)
    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    ins, sid, pre, lens = make_metadata(cfg, seed)
    g = torch.Generator().manual_seed(seed)
    heads, spent, flops = 0, 0.0, 0.0
    limit = max_heads or B * H
    for b in range(B):
        if cfg["hier"]:
            mask = ao.dense_mask(L, ins[b:b + 1], sid[b:b + 1], pre[b:b + 1], lens[b:b + 1])
        else:
            mask = ao.dense_mask(L, causal=True)
        tiles = int((ao.tile_classes(mask) != ao.EMPTY).sum())
        if b == 0:  # one untimed head to page in the BLAS threads
            q, k, v, do = (torch.randn((1, 1, L, D), generator=g) for _ in range(4))
            ao.attention_fwd_bwd(q, k, v, do, mask)
        for _ in range(H):
            q, k, v, do = (torch.randn((1, 1, L, D), generator=g) for _ in range(4))
            t0 = time.perf_counter()
            ao.attention_fwd_bwd(q, k, v, do, mask)
            spent += time.perf_counter() - t0
            heads += 1
            flops += 14.0 * D * 128.0 * 128.0 * tiles
            if heads >= limit or spent >= budget_s:
                break
        if heads >= limit or spent >= budget_s:
            break
    tflops = flops / spent / 1e12
    sample = (f"the first {heads} of {B * H} (batch, head) pairs of the workload, dense-masked fp32 torch math "
              f"(oracle/attention_oracle.py), {spent:.1f} s")
    return tflops, sample, spent, heads


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps, warmup = args.steps, args.warmup
    per_step = min(20.0, max(2.0, 120.0 / max(1, steps + warmup)))
    vals, secs = [], []
    sample = ""
    for i in range(warmup + steps):
        tf, sample, spent, heads = time_cpu_oracle(cfg, 1234, per_step)
        if i >= warmup:
            vals.append(tf); secs.append(spent / heads)
    value = float(np.mean(vals))
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": float(np.mean(secs) * 1e3 * cfg["B"] * cfg["H"]),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": cfg["name"], "sample": sample,
                   "note": "ms_per_step extrapolates the per-(batch, head) time of the sample to the whole batch"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# --------------------------------------------------------------------------------------------
# GPU arm
# --------------------------------------------------------------------------------------------
def run_ours(args, cfg):
    import torch.distributed as dist
    from kerneldev_b200 import flash_attention, generate_hadamard_signs
    from kerneldev_b200.original_kernel import _backward, _forward
    from kerneldev_b200.plan import get_plan

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA sm_100 device; there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    dtype = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float16
    seed = 1234 + rank                       # Q, K, V, dO differ per rank
    ins, sid, pre, lens = make_metadata(cfg, 1234)   # same section layout on every rank: equal work per GPU
    tt = lambda a, dt: None if a is None else torch.as_tensor(a, dtype=dt, device=dev)
    meta = dict(in_span=tt(ins, torch.bool), span_id=tt(sid, torch.int64), is_prefix=tt(pre, torch.bool),
                lens=tt(lens, torch.int32))
    g = torch.Generator(device=dev).manual_seed(seed)
    q, k, v, do = (torch.randn((B, H, L, D), generator=g, device=dev, dtype=dtype) for _ in range(4))
    signs = generate_hadamard_signs(H, D, seed=seed, device=dev) if cfg["hadamard"] else None
    sm_scale = D ** -0.5

    plan = get_plan(B, L, dev, meta["in_span"], meta["span_id"], meta["is_prefix"], meta["lens"], True, cfg["hier"])
    nonempty = plan.nonempty_tiles()
    f_eff = effective_flops(cfg, nonempty)
    f_dense = 14.0 * D * B * H * float(L) * L

    # ---- kernel-level step: inputs resident in HBM, raw C-ABI calls, buffers reused ----------
    bufs = (torch.empty_like(q), torch.empty_like(q), torch.empty_like(q),
            torch.empty((B, H, L), dtype=torch.float32, device=dev))
    if signs is not None:
        from kerneldev_b200 import hadamard_transform

    def step_resident():
        if signs is not None:
            qq, kk = hadamard_transform(q, signs), hadamard_transform(k, signs)
        else:
            qq, kk = q, k
        o, lse = _forward(qq, kk, v, plan, sm_scale)
        dq, dk, dv = _backward(qq, kk, v, o, lse, do, plan, sm_scale, 0, bufs)
        if signs is not None:
            from kerneldev_b200.original_kernel import _hadamard_call
            dq, dk = _hadamard_call(dq, signs, True), _hadamard_call(dk, signs, True)
        return o, lse

    launches_per_step = 4 + (4 if signs is not None else 0)   # forward, delta, dQ, dK/dV (+ Hadamard passes)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step_resident()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step_resident()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    plan.check_status()
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    feff_t = torch.tensor([f_eff], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.all_reduce(feff_t, op=dist.ReduceOp.SUM)
    ms_step = float(t.item()) / args.steps
    value = float(feff_t.item()) / (ms_step * 1e-3) / 1e12

    # ---- per-kernel times (rank 0's own kernels, CUDA events on the launching stream) --------
    def time_call(fn, iters):
        fn(); torch.cuda.synchronize()
        a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b_.record(); torch.cuda.synchronize()
        return a.elapsed_time(b_) / iters

    qq, kk = (hadamard_transform(q, signs), hadamard_transform(k, signs)) if signs is not None else (q, k)
    o, lse = _forward(qq, kk, v, plan, sm_scale)
    it = max(3, min(args.steps, 10))
    ms_fwd = time_call(lambda: _forward(qq, kk, v, plan, sm_scale), it)
    ms_dq = time_call(lambda: _backward(qq, kk, v, o, lse, do, plan, sm_scale, 1, bufs), it)
    ms_dkdv = time_call(lambda: _backward(qq, kk, v, o, lse, do, plan, sm_scale, 2, bufs), it)
    per_pair = D * H * 128.0 * 128.0 * nonempty
    kernels = {
        # name: (ms, algorithmic FLOPs per launch, executed MMA FLOPs per launch)
        "attn_fwd_kernel": (ms_fwd, 4 * per_pair, 4 * per_pair),
        "attn_bwd_dq_kernel": (ms_dq, 6 * per_pair, 6 * per_pair),        # S, dP, dQ
        "attn_bwd_dkdv_kernel": (ms_dkdv, 4 * per_pair, 8 * per_pair),    # dV, dK (+ recomputed S, dP)
    }
    dom = max(kernels, key=lambda n: kernels[n][0])
    peaks, peak_kind = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    peak_sus = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    dom_ms, dom_alg, dom_exec = kernels[dom]
    achieved = dom_alg / (dom_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
        "frac": achieved / peak_tf,
        "traffic": (NCU_TRAFFIC_PER_BATCH_ROW[dom] * B) if (args.config == 2) else None,
        "traffic_note": "bytes per launch: ncu capture at batch 4 scaled to this batch",
        "peak_kind": peak_kind + " burst (kernel timed alone)",
        "executed_tflops": dom_exec / (dom_ms * 1e-3) / 1e12,
        "kernels_ms": {n: kernels[n][0] for n in kernels},
        "kernels_algorithmic_tflops": {n: kernels[n][1] / (kernels[n][0] * 1e-3) / 1e12 for n in kernels},
    }

    # ---- end to end: public API with host buffers ----------------------------------------------
    hq, hk, hv, hdo = (x.cpu().pin_memory() for x in (q, k, v, do))
    ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
    h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hdo))
    d2h = sum(x.numel() * x.element_size() for x in (ho, hdq, hdk, hdv))

    from kerneldev_b200.host_io import HostPipeline
    pipe = HostPipeline(dev, chunks=args.e2e_chunks)

    def step_e2e():
        # public API on host buffers: chunks of the batch are copied in, run through flash_attention +
        # autograd and copied out on three streams, so PCIe transfers overlap the kernels
        pipe.run(hq, hk, hv, hdo, ho, hdq, hdk, hdv, causal=True, hadamard_signs=signs, **meta)

    e2e_steps = max(2, min(args.steps, 5))
    if args.kernels_only:
        ms_e2e, e2e_value = None, None
    else:
        for _ in range(2):
            step_e2e()
        barrier()
        ev0.record()
        for _ in range(e2e_steps):
            step_e2e()
        ev1.record()
        barrier()
        t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e = float(t.item()) / e2e_steps
        e2e_value = float(feff_t.item()) / (ms_e2e * 1e-3) / 1e12

    # the sampler covers the timed region and the per-kernel / end-to-end legs that follow it (all GPU load)
    clocks = sampler.stop() if rank == 0 else None
    if rank == 0:
        cpu = None
        if world == 1 and not args.no_cpu_baseline and not args.kernels_only:
            tf, sample, _, _ = time_cpu_oracle(cfg, 1234, 15.0)
            cpu = {"value": tf, "unit": UNIT, "cores": os.cpu_count() or 1, "kind": "port", "sample": sample}
        per_gpu = value / world
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": cfg["dtype"], "data": "synthetic",
            "config": {"workload": cfg["name"], "per_gpu_batch": B, "heads": H, "seq_len": L, "head_dim": D,
                       "sharding": "one config-shaped batch per GPU, (batch, head) pairs independent, no collective",
                       "l2": "inputs larger than L2 (Q, K, V, dO are %d MB each)" % (q.numel() * 2 // 2 ** 20),
                       "nonempty_tile_fraction": nonempty / float(B * plan.NT * plan.NT)},
            "per_gpu_tflops": per_gpu,
            "pct_of_bf16_peak": {"burst": 100 * per_gpu / peak_tf, "sustained": 100 * per_gpu / peak_sus, "peaks": peak_kind},
            "dense_equivalent_tflops": f_dense * world / (ms_step * 1e-3) / 1e12,
            "tokens_per_s": B * L * world / (ms_step * 1e-3),
            "e2e": None if e2e_value is None else {
                "value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                "ms_per_step": ms_e2e, "steps": e2e_steps},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "roofline": roofline,
            "cpu_baseline": cpu,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--config", type=int, default=2, choices=sorted(CONFIGS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--batch", type=int, default=0, help="override the per-GPU batch size (profiling on a small case)")
    ap.add_argument("--kernels-only", action="store_true", help="skip the end-to-end and CPU legs (profiling)")
    ap.add_argument("--e2e-chunks", type=int, default=8, help="batch chunks of the host-buffer pipeline in the end-to-end leg")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    cfg = dict(CONFIGS[args.config])
    if args.batch > 0:
        cfg["B"] = args.batch
        cfg["name"] += f" (batch overridden to {args.batch})"
    if args.impl == "reference":
        run_reference(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
