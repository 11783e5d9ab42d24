"""Mask metadata from token ids on the device.

``GPTModel.forward`` derives ``in_span``, ``span_id`` and ``is_prefix`` from the token ids when the
caller passes none of them (model.py:203-238): two cumulative sums and a Python loop over the batch
with one ``.nonzero()`` / ``.item()`` synchronisation per row. ``metadata_from_tokens`` produces the
same three tensors with one kernel launch and no synchronisation; they are what ``flash_attention``
takes, and the plan built from them is shared by all layers.
"""
from __future__ import annotations

import torch

from . import _capi

#: ids of the reference tokenizer's special tokens (data_builder.py:44-51)
SPECIAL_TOKENS = {"[PAD]": 0, "[CLS]": 1, "[MASK]": 2, "[SPAN]": 3, "[ES]": 4, "[MASKQ]": 5}


def metadata_from_tokens(tokens: torch.Tensor, special_tokens=None):
    """tokens: int64 (batch, time) on a CUDA device. Returns (in_span bool, span_id int64,
    is_prefix bool), each (batch, time), equal to model.py:211-238 for the same ids."""
    if tokens.dim() != 2 or tokens.dtype != torch.int64:
        raise ValueError("tokens must be an int64 tensor of shape (batch, time)")
    if not tokens.is_cuda:
        raise RuntimeError("metadata_from_tokens runs on CUDA devices only; there is no CPU path")
    st = SPECIAL_TOKENS if special_tokens is None else special_tokens
    if tokens.stride(1) != 1:
        tokens = tokens.contiguous()
    B, T = tokens.shape
    in_span = torch.empty((B, T), dtype=torch.bool, device=tokens.device)
    span_id = torch.empty((B, T), dtype=torch.int64, device=tokens.device)
    is_prefix = torch.empty((B, T), dtype=torch.bool, device=tokens.device)
    stream = torch.cuda.current_stream(tokens.device).cuda_stream
    with torch.cuda.device(tokens.device):
        _capi.check(_capi.load().kd_metadata_from_tokens(
            tokens.data_ptr(), tokens.stride(0) if B > 1 else max(T, 1), B, T, st["[SPAN]"], st["[ES]"], st["[CLS]"],
            st["[MASKQ]"], in_span.data_ptr(), span_id.data_ptr(), is_prefix.data_ptr(), stream))
    return in_span, span_id, is_prefix


def _bench():
    """python -m kerneldev_b200.metadata: times the kernel with CUDA events on token batches of the
    BASELINE config shapes and prints GB/s against the 18 bytes per token it moves; beside it the same
    formulas as written in model.py:211-238 (torch cumsum + a per-row host loop) on the same device."""
    import json
    import time

    dev = torch.device("cuda:0")
    st = SPECIAL_TOKENS
    out = []
    lib = _capi.load()
    for B, T in ((16, 4096), (4, 8192), (64, 16384), (512, 16384)):
        g = torch.Generator(device=dev).manual_seed(B * T)
        x = torch.randint(6, 300, (B, T), generator=g, device=dev)
        marks = torch.rand((B, T), generator=g, device=dev) < 0.02
        x = torch.where(marks, torch.randint(0, 6, (B, T), generator=g, device=dev), x)
        ins = torch.empty((B, T), dtype=torch.bool, device=dev)
        sid = torch.empty((B, T), dtype=torch.int64, device=dev)
        pre = torch.empty((B, T), dtype=torch.bool, device=dev)
        stream = torch.cuda.current_stream(dev).cuda_stream

        def call():   # the C ABI entry point on preallocated outputs
            _capi.check(lib.kd_metadata_from_tokens(x.data_ptr(), T, B, T, st["[SPAN]"], st["[ES]"], st["[CLS]"], st["[MASKQ]"],
                                                    ins.data_ptr(), sid.data_ptr(), pre.data_ptr(), stream))

        for _ in range(5):
            call()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n = 50
        a.record()
        for _ in range(n):
            call()
        b.record()
        torch.cuda.synchronize()
        us = a.elapsed_time(b) / n * 1e3

        def torch_formulation():
            in_span = (torch.cumsum((x == st["[SPAN]"]).int(), dim=1) - torch.cumsum((x == st["[ES]"]).int(), dim=1)) > 0
            span_id = torch.cumsum((x == st["[SPAN]"]).int(), dim=1)
            span_id[~in_span] = 0
            span_id[x == st["[MASKQ]"]] = -1
            is_prefix = torch.zeros((B, T), dtype=torch.bool, device=dev)
            for bi in range(B):
                pos = (x[bi] == st["[CLS]"]).nonzero(as_tuple=True)[0]
                if len(pos) > 0:
                    is_prefix[bi, : pos[0].item() + 1] = True
            return in_span, span_id, is_prefix

        if B > 64:
            out.append({"B": B, "T": T, "kernel_us": round(us, 2), "GBps": round(18.0 * B * T / us / 1e3, 1)})
            continue
        torch_formulation()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(5):
            torch_formulation()
        torch.cuda.synchronize()
        us_torch = (time.perf_counter() - t0) / 5 * 1e6
        out.append({"B": B, "T": T, "kernel_us": round(us, 2), "GBps": round(18.0 * B * T / us / 1e3, 1),
                    "torch_formulation_us": round(us_torch, 1)})
    print(json.dumps(out))


if __name__ == "__main__":
    _bench()
