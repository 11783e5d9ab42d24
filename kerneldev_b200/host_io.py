"""Forward + backward of the attention operator on HOST buffers.

The operator itself works on device tensors. A caller whose Q, K, V, dO live in (pinned) host memory
pays two PCIe transfers per step; because the sequences of a batch are independent, the batch can be
cut into chunks and the transfers of one chunk overlapped with the kernels of another:

    copy-in stream :  H2D(c+1)
    compute stream :           fwd+bwd(c)
    copy-out stream:                      D2H(c-1)

`attention_fwd_bwd_host` does that with the public `flash_attention` + autograd on each chunk.
"""
from __future__ import annotations

import torch

from .original_kernel import flash_attention


class HostPipeline:
    """Reusable staging buffers and streams for `attention_fwd_bwd_host` on one device."""

    def __init__(self, device, chunks: int = 4):
        self.device = torch.device(device)
        self.chunks = chunks
        self.s_in = torch.cuda.Stream(self.device)
        self.s_out = torch.cuda.Stream(self.device)
        self._stage = {}

    def _staging(self, shape, dtype):
        key = (tuple(shape), dtype)
        if key not in self._stage:
            # two sets of four input buffers: chunk c uses set c % 2
            self._stage[key] = [[torch.empty(shape, dtype=dtype, device=self.device) for _ in range(4)] for _ in range(2)]
        return self._stage[key]

    def run(self, hq, hk, hv, hdo, ho, hdq, hdk, hdv, lens=None, in_span=None, span_id=None, is_prefix=None,
            causal=True, sm_scale=None, hadamard_signs=None, deterministic=False):
        """hq, hk, hv, hdo: pinned host inputs (B,H,T,D); ho, hdq, hdk, hdv: pinned host outputs of the
        same shape. Metadata tensors are device tensors for the whole batch. Returns after enqueueing;
        synchronise the device (or the copy-out stream) before reading the outputs."""
        B = hq.shape[0]
        n = min(self.chunks, B)
        bounds = [(B * c) // n for c in range(n + 1)]
        cur = torch.cuda.current_stream(self.device)
        self.s_in.wait_stream(cur)
        self.s_out.wait_stream(cur)
        comp_done = []
        keep = []
        for c in range(n):
            lo, hi = bounds[c], bounds[c + 1]
            shape = (hi - lo,) + tuple(hq.shape[1:])
            bufs = self._staging(shape, hq.dtype)[c % 2]
            with torch.cuda.stream(self.s_in):
                if c >= 2:
                    self.s_in.wait_event(comp_done[c - 2])      # the staging set is free again
                for dst, src in zip(bufs, (hq, hk, hv, hdo)):
                    dst.copy_(src[lo:hi], non_blocking=True)
                in_done = torch.cuda.Event()
                in_done.record(self.s_in)
            cur.wait_event(in_done)
            q, k, v = (x.detach().requires_grad_() for x in bufs[:3])
            sl = lambda t: None if t is None else t[lo:hi]
            out = flash_attention(q, k, v, lens=sl(lens), sm_scale=sm_scale, causal=causal, in_span=sl(in_span),
                                  span_id=sl(span_id), is_prefix=sl(is_prefix), hadamard_signs=hadamard_signs,
                                  deterministic=deterministic)
            out.backward(bufs[3])
            ev = torch.cuda.Event()
            ev.record(cur)
            comp_done.append(ev)
            results = (out.detach(), q.grad, k.grad, v.grad)
            keep.append(results)
            with torch.cuda.stream(self.s_out):
                self.s_out.wait_event(ev)
                for src, dst in zip(results, (ho, hdq, hdk, hdv)):
                    src.record_stream(self.s_out)
                    dst[lo:hi].copy_(src, non_blocking=True)
        cur.wait_stream(self.s_out)
        cur.wait_stream(self.s_in)
        return keep


def attention_fwd_bwd_host(pipeline: HostPipeline, *args, **kwargs):
    return pipeline.run(*args, **kwargs)
