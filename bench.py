#!/usr/bin/env python
"""Benchmark of the attention hot path: hierarchical-mask flash attention forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config 2]

Workload (default): BASELINE config 2 -- bf16, B=16, H=16, L=4096, D=64, hierarchical mask with
per-sequence sections drawn from a seed (prefix U[32,256], context U[1024,2048], 4..32 spans of
16..128 tokens, one MASKQ, PAD). One step = one forward + one backward over the batch.

Scaling. The (batch, head) pairs of the operator are independent, so there is no collective on the data
path. The headline `value` is WEAK scaling: every rank owns one config-shaped batch. For N > 1 the line
also carries `strong`: ONE config-shaped batch split over the ranks by (batch, head) pairs
(kerneldev_b200.sharding.shard_pairs), aggregate = FLOPs of the whole batch / max time over ranks.

The one JSON line printed by rank 0:
  value      effective TFLOP/s summed over all ranks, inputs resident in HBM. Effective FLOPs =
             14*D*H*128^2 * (number of non-EMPTY 128x128 mask tiles of the batch): 4D forward + 10D
             backward per element of a non-empty tile (BASELINE.json's "unmasked-tile" count; PARTIAL
             tiles count in full, recomputation is not counted). `flops_exact_pairs` gives the same
             figure with 14*D*H * (allowed (query, key) pairs) instead.
  plan       time of the tile classifier (3 launches per new metadata batch) and `value_with_plan`, the
             headline figure when a new plan is built every step instead of being reused.
  e2e        the same metric through flash_attention() + autograd with HOST (pinned) buffers: every
             step copies Q, K, V, dO host->device and O, dQ, dK, dV device->host; `copy_ceiling_ms` is
             the time of those copies alone (no kernels) at this N.
  roofline   dominant kernel: algorithmic FLOPs per launch / its CUDA-event time, against the
             measured bf16 peak of MEASURED_PEAKS.json; `dq_accumulate` is the fused backward's dQ
             reduction traffic per launch and its rate.
  other_configs  short legs for BASELINE configs 1 and 3 (N = 1 only).
  cpu_baseline   the CPU oracle (dense-masked fp32 torch math) on a bounded sample, on the host cores.

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
TRAFFIC_FILE = os.path.join(ROOT, "profiles", "attention_kernels_traffic.json")


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return d, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


def load_traffic():
    """DRAM bytes per launch and per batch row of config 2 for each kernel, written next to the ncu summary
    they come from; traffic grows in proportion to the number of (batch, head) pairs."""
    try:
        with open(TRAFFIC_FILE) as f:
            return json.load(f)
    except Exception:
        return {}


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
              f"(oracle/attention_oracle.py; it executes all L x L pairs and is credited with the non-empty tiles only), {spent:.1f} s")
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
class Workload:
    """Resident inputs, plan and reusable buffers of one (possibly sharded) batch on one GPU."""

    def __init__(self, cfg, dev, seed, meta_np, rows=None, heads=None):
        from kerneldev_b200 import generate_hadamard_signs
        from kerneldev_b200.plan import get_plan
        self.cfg, self.dev = cfg, dev
        ins, sid, pre, lens = meta_np
        if rows is not None and ins is not None:
            ins, sid, pre, lens = (a[rows[0]:rows[1]] for a in (ins, sid, pre, lens))
        self.B = cfg["B"] if rows is None else rows[1] - rows[0]
        self.H = cfg["H"] if heads is None else heads[1] - heads[0]
        self.L, self.D = cfg["L"], cfg["D"]
        self.dtype = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float16
        tt = lambda a, dt: None if a is None else torch.as_tensor(a, dtype=dt, device=dev)
        self.meta = dict(in_span=tt(ins, torch.bool), span_id=tt(sid, torch.int64), is_prefix=tt(pre, torch.bool),
                         lens=tt(lens, torch.int32))
        g = torch.Generator(device=dev).manual_seed(seed)
        shape = (self.B, self.H, self.L, self.D)
        self.q, self.k, self.v, self.do = (torch.randn(shape, generator=g, device=dev, dtype=self.dtype) for _ in range(4))
        self.signs = None
        if cfg["hadamard"]:
            s = generate_hadamard_signs(cfg["H"], self.D, seed=seed, device=dev)
            self.signs = s if heads is None else s[heads[0]:heads[1]].contiguous()
        self.sm_scale = self.D ** -0.5
        self.hier = cfg["hier"]
        self.plan = self.new_plan()
        self.nonempty = self.plan.nonempty_tiles()
        self.f_eff = 14.0 * self.D * self.H * 128.0 * 128.0 * self.nonempty
        self.bufs = (torch.empty_like(self.q), torch.empty_like(self.q), torch.empty_like(self.q),
                     torch.empty((self.B, self.H, self.L), dtype=torch.float32, device=dev),
                     torch.empty(shape, dtype=torch.float32, device=dev) if self.D == 64 else None)
        self.fused = self.D == 64
        self.launches_per_step = 4 + (4 if self.signs is not None else 0)

    def new_plan(self, cached=True):
        from kerneldev_b200.plan import AttentionPlan, get_plan
        m = self.meta
        if cached:
            return get_plan(self.B, self.L, self.dev, m["in_span"], m["span_id"], m["is_prefix"], m["lens"], True, self.hier)
        return AttentionPlan(self.B, self.L, self.dev, m["in_span"], m["span_id"], m["is_prefix"], m["lens"], True, self.hier)

    def transformed(self):
        if self.signs is None:
            return self.q, self.k
        from kerneldev_b200 import hadamard_transform
        return hadamard_transform(self.q, self.signs), hadamard_transform(self.k, self.signs)

    def step(self, plan=None):
        """Forward + backward on resident inputs through the raw C-ABI calls, buffers reused."""
        from kerneldev_b200.original_kernel import _backward, _forward, _hadamard_call
        plan = plan or self.plan
        qq, kk = self.transformed()
        o, lse = _forward(qq, kk, self.v, plan, self.sm_scale)
        dq, dk, dv = _backward(qq, kk, self.v, o, lse, self.do, plan, self.sm_scale, 0, self.bufs)
        if self.signs is not None:
            dq, dk = _hadamard_call(dq, self.signs, True), _hadamard_call(dk, self.signs, True)
        return o, lse

    def allowed_pairs(self):
        """Exact number of allowed (query, key) pairs of the batch (one head), from the plan's dense mask."""
        total = 0
        from kerneldev_b200.plan import AttentionPlan
        m = self.meta
        for b in range(self.B):
            sl = lambda t: None if t is None else t[b:b + 1]
            p = AttentionPlan(1, self.L, self.dev, sl(m["in_span"]), sl(m["span_id"]), sl(m["is_prefix"]), sl(m["lens"]), True, self.hier)
            total += int(p.dense_mask().sum().item())
        return total


def time_call(fn, iters):
    fn(); torch.cuda.synchronize()
    a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b_.record(); torch.cuda.synchronize()
    return a.elapsed_time(b_) / iters


def kernel_times(w, iters):
    """CUDA-event times of the individual kernels of one step (inputs larger than L2 at the bench sizes)."""
    from kerneldev_b200.original_kernel import _backward, _forward
    qq, kk = w.transformed()
    o, lse = _forward(qq, kk, w.v, w.plan, w.sm_scale)
    per_pair = w.D * w.H * 128.0 * 128.0 * w.nonempty
    ms_fwd = time_call(lambda: _forward(qq, kk, w.v, w.plan, w.sm_scale), iters)
    bw = lambda ph: time_call(lambda: _backward(qq, kk, w.v, o, lse, w.do, w.plan, w.sm_scale, ph, w.bufs), iters)
    if w.fused:
        return {
            # name: (ms, algorithmic FLOPs per launch, executed MMA FLOPs per launch)
            "attn_fwd_kernel": (ms_fwd, 4 * per_pair, 4 * per_pair),
            "attn_bwd_delta_kernel": (bw(1), 0.0, 0.0),
            "attn_bwd_fused_kernel": (bw(2), 10 * per_pair, 10 * per_pair),   # S, dP, dV, dK, dQ (+ the dQ conversion kernel)
        }
    return {
        "attn_fwd_kernel": (ms_fwd, 4 * per_pair, 4 * per_pair),
        "attn_bwd_dq_kernel": (bw(1), 6 * per_pair, 6 * per_pair),        # delta; S, dP, dQ
        "attn_bwd_dkdv_kernel": (bw(2), 4 * per_pair, 8 * per_pair),      # dV, dK (+ recomputed S, dP)
    }


def timed_steps(fn, steps, barrier):
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(steps):
        fn()
    ev1.record()
    barrier()
    return ev0.elapsed_time(ev1)


def run_ours(args, cfg):
    import torch.distributed as dist
    from kerneldev_b200 import flash_attention  # noqa: F401  (loads the library; fails loudly when it is missing)
    from kerneldev_b200.sharding import shard_pairs

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA sm_100 device; there is no CPU path for the operator")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def sum_over_ranks(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.SUM)
        return float(t.item())

    B, H, L, D = cfg["B"], cfg["H"], cfg["L"], cfg["D"]
    meta_np = make_metadata(cfg, 1234)   # the same section layout on every rank: equal work per GPU
    w = Workload(cfg, dev, 1234 + rank, meta_np)   # Q, K, V, dO differ per rank
    f_dense = 14.0 * D * B * H * float(L) * L

    # ---- weak scaling, inputs resident in HBM ---------------------------------------------------
    for _ in range(args.warmup):
        w.step()
    sampler = ClockSampler(local_rank)
    barrier()
    if rank == 0:
        sampler.start()
    ms_total = timed_steps(w.step, args.steps, barrier)
    w.plan.check_status()
    ms_step = max_over_ranks(ms_total) / args.steps
    f_eff_all = sum_over_ranks(w.f_eff)
    value = f_eff_all / (ms_step * 1e-3) / 1e12

    # ---- the classifier: alone, and inside the step ("included" next to the "amortised" headline) ----
    ms_plan = time_call(lambda: w.new_plan(cached=False), max(3, min(args.steps, 10)))
    ms_with_plan = max_over_ranks(timed_steps(lambda: w.step(w.new_plan(cached=False)), args.steps, barrier)) / args.steps

    # ---- strong scaling: ONE config-shaped batch split over the ranks ---------------------------
    strong = None
    if world > 1:
        lo, hi = shard_pairs(B, H, rank, world)
        if lo % H == 0 and hi % H == 0:      # whole batch rows
            ws = Workload(cfg, dev, 4321, meta_np, rows=(lo // H, hi // H))
            split = f"{(hi - lo) // H} of {B} batch rows per GPU"
        else:                                # part of one row's heads; the row's metadata is replicated
            assert lo // H == (hi - 1) // H, "a rank's pairs must lie in one batch row"
            ws = Workload(cfg, dev, 4321, meta_np, rows=(lo // H, lo // H + 1), heads=(lo % H, (hi - 1) % H + 1))
            split = f"{hi - lo} of {H} heads of one batch row per GPU"
        for _ in range(args.warmup):
            ws.step()
        ms_s = max_over_ranks(timed_steps(ws.step, args.steps, barrier)) / args.steps
        ms_sp = max_over_ranks(timed_steps(lambda: ws.step(ws.new_plan(cached=False)), args.steps, barrier)) / args.steps
        f_s = sum_over_ranks(ws.f_eff)
        strong = {"workload": cfg["name"] + " (one batch over all GPUs)", "split": split, "ms_per_step": ms_s,
                  "value": f_s / (ms_s * 1e-3) / 1e12, "ms_per_step_with_plan": ms_sp,
                  "value_with_plan": f_s / (ms_sp * 1e-3) / 1e12, "unit": UNIT,
                  "note": "efficiency = value / (N x the N=1 value of the same line)"}
        del ws

    # ---- per-kernel times (rank 0's own kernels, CUDA events on the launching stream) -----------
    it = max(3, min(args.steps, 10))
    kernels = kernel_times(w, it)
    dom = max(kernels, key=lambda n: kernels[n][0])
    peaks, peak_kind = load_peaks()
    peak_tf = float(peaks.get("bf16_tflops", FALLBACK_PEAKS["bf16_tflops"]))
    peak_sus = float(peaks.get("bf16_tflops_sustained", FALLBACK_PEAKS["bf16_tflops_sustained"]))
    peak_hbm = float(peaks.get("hbm_gbs", FALLBACK_PEAKS["hbm_gbs"]))
    dom_ms, dom_alg, dom_exec = kernels[dom]
    achieved = dom_alg / (dom_ms * 1e-3) / 1e12
    traffic = load_traffic().get(dom)
    roofline = {
        "bound": "tensor", "kernel": dom, "achieved": achieved, "peak": peak_tf, "unit": "TFLOP/s",
        "frac": achieved / peak_tf,
        "traffic": (traffic["dram_bytes_per_batch_row"] * B) if (traffic and args.config == 2) else None,
        "traffic_note": "bytes per launch: ncu capture at a smaller batch scaled by batch rows (profiles/attention_kernels_traffic.json)",
        "peak_kind": peak_kind + " burst (kernel timed alone)",
        "executed_tflops": dom_exec / (dom_ms * 1e-3) / 1e12,
        "kernels_ms": {n: kernels[n][0] for n in kernels},
        "kernels_algorithmic_tflops": {n: kernels[n][1] / (kernels[n][0] * 1e-3) / 1e12 for n in kernels},
    }
    if w.fused:
        red_bytes = w.nonempty * w.H * 128.0 * w.D * 4.0     # one fp32 dQ tile per non-empty tile and head
        ms_f = kernels["attn_bwd_fused_kernel"][0]
        roofline["dq_accumulate"] = {
            "reduce_bytes_per_launch": red_bytes, "GBps": red_bytes / (ms_f * 1e-3) / 1e9,
            "hbm_peak_GBps": peak_hbm,
            "note": "fp32 bytes of the dQ tiles the TMA bulk reductions add into the scratch, over the fused kernel's time; the adds run in L2, "
                    "HBM sees the scratch once zeroed, once written back and once read by the conversion kernel"}

    # ---- end to end: public API with host buffers ------------------------------------------------
    e2e = None
    if not args.kernels_only:
        from kerneldev_b200.host_io import HostPipeline
        hq, hk, hv, hdo = (x.cpu().pin_memory() for x in (w.q, w.k, w.v, w.do))
        ho, hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(4))
        h2d = sum(x.numel() * x.element_size() for x in (hq, hk, hv, hdo))
        d2h = sum(x.numel() * x.element_size() for x in (ho, hdq, hdk, hdv))
        pipe = HostPipeline(dev, chunks=args.e2e_chunks)

        def step_e2e():
            # public API on host buffers: chunks of the batch are copied in, run through flash_attention +
            # autograd and copied out on three streams, so PCIe transfers overlap the kernels
            pipe.run(hq, hk, hv, hdo, ho, hdq, hdk, hdv, causal=True, hadamard_signs=w.signs, **w.meta)

        e2e_steps = max(2, min(args.steps, 5))
        for _ in range(2):
            step_e2e()
        ms_e2e = max_over_ranks(timed_steps(step_e2e, e2e_steps, barrier)) / e2e_steps
        # the copies alone, both directions at once, same bytes, no kernels: what the host link allows at this N
        s_in, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev)
        dst = [torch.empty_like(w.q) for _ in range(4)]

        def copies_only():
            cur = torch.cuda.current_stream(dev)
            s_in.wait_stream(cur); s_out.wait_stream(cur)
            with torch.cuda.stream(s_in):
                for d_, s_ in zip(dst, (hq, hk, hv, hdo)):
                    d_.copy_(s_, non_blocking=True)
            with torch.cuda.stream(s_out):
                for d_, s_ in zip((ho, hdq, hdk, hdv), w.bufs[:3] + (w.q,)):
                    d_.copy_(s_, non_blocking=True)
            cur.wait_stream(s_in); cur.wait_stream(s_out)

        copies_only()
        ms_copy = max_over_ranks(timed_steps(copies_only, e2e_steps, barrier)) / e2e_steps
        del dst
        e2e = {"value": f_eff_all / (ms_e2e * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "ms_per_step": ms_e2e, "steps": e2e_steps, "copy_ceiling_ms": ms_copy,
               "copy_ceiling_over_e2e": ms_copy / ms_e2e,
               "copy_GBps_per_gpu": (h2d + d2h) / (ms_copy * 1e-3) / 1e9}
        del hq, hk, hv, hdo, ho, hdq, hdk, hdv, pipe

    # the sampler covers the timed region and the per-kernel / end-to-end legs that follow it (all GPU load)
    clocks = sampler.stop() if rank == 0 else None

    # ---- the other BASELINE configurations, short legs (single GPU only) -------------------------
    other = None
    pairs_exact = None
    if rank == 0 and world == 1 and not args.kernels_only:
        pairs_exact = w.allowed_pairs()
        nonempty, frac = w.nonempty, w.nonempty / float(B * w.plan.NT * w.plan.NT)
        stats = w.plan.stats.sum(0).tolist()
        del w
        torch.cuda.empty_cache()
        other = []
        for cid in sorted(CONFIGS):
            if cid == args.config:
                continue
            c2 = dict(CONFIGS[cid])
            w2 = Workload(c2, dev, 1234, make_metadata(c2, 1234))
            for _ in range(3):
                w2.step()
            ms2 = timed_steps(w2.step, max(3, min(args.steps, 10)), barrier) / max(3, min(args.steps, 10))
            k2 = kernel_times(w2, 3)
            v2 = w2.f_eff / (ms2 * 1e-3) / 1e12
            other.append({"workload": c2["name"], "dtype": c2["dtype"], "ms_per_step": ms2, "value": v2, "unit": UNIT,
                          "pct_of_bf16_peak_burst": 100 * v2 / peak_tf, "kernels_ms": {n: k2[n][0] for n in k2},
                          "nonempty_tiles": w2.nonempty})
            del w2
            torch.cuda.empty_cache()
    else:
        nonempty, frac = w.nonempty, w.nonempty / float(B * w.plan.NT * w.plan.NT)
        stats = w.plan.stats.sum(0).tolist()

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
                       "l2": "inputs larger than L2 (Q, K, V, dO are %d MB each)" % (B * H * L * D * 2 // 2 ** 20),
                       "backward": "fused (dQ accumulated in fp32 with atomics)" if D == 64 else "two kernels (dQ, dK/dV)",
                       "nonempty_tile_fraction": frac, "full_tiles": stats[0], "partial_tiles": stats[1]},
            "per_gpu_tflops": per_gpu,
            "pct_of_bf16_peak": {"burst": 100 * per_gpu / peak_tf, "sustained": 100 * per_gpu / peak_sus, "peaks": peak_kind},
            "dense_equivalent_tflops": f_dense * world / (ms_step * 1e-3) / 1e12,
            "flops_exact_pairs": None if pairs_exact is None else {
                "allowed_pairs": pairs_exact, "share_of_nonempty_tile_area": pairs_exact / (nonempty * 16384.0),
                "tflops": 14.0 * D * H * pairs_exact / (ms_step * 1e-3) / 1e12},
            "tokens_per_s": B * L * world / (ms_step * 1e-3),
            "plan": {"classifier_ms": ms_plan, "ms_per_step_with_plan": ms_with_plan,
                     "value_with_plan": f_eff_all / (ms_with_plan * 1e-3) / 1e12,
                     "note": "headline reuses the plan (one per metadata batch, shared by heads and layers); value_with_plan builds it every step"},
            "strong": strong,
            "e2e": e2e,
            "gpu_launches": (4 + (4 if cfg["hadamard"] else 0)) * args.steps,
            "clocks": clocks,
            "roofline": roofline,
            "other_configs": other,
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
    ap.add_argument("--kernels-only", action="store_true", help="skip the end-to-end, other-config and CPU legs (profiling)")
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
