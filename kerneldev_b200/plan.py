"""Attention plans: the per-batch product of the tile classifier.

A plan holds the packed token descriptors, the class (EMPTY / FULL / PARTIAL) of every
128x128 tile of the mask and the work lists the kernels walk. It depends only on the
metadata (``in_span``, ``span_id``, ``is_prefix``, ``lens``, ``causal``), not on the head, so one
plan serves all heads and -- because ``model.GPTModel`` passes the same three metadata tensors
to every layer (model.py:243-244) -- all layers of a step. Plans are cached on the identity and
version of the metadata tensors (the cache keeps those tensors alive, so an address cannot be
reused while its plan is cached). Metadata rewritten in place through raw pointers -- by
kd_metadata_from_tokens into preallocated buffers, or through ``.data`` -- does not change a tensor's
version: call ``clear_plan_cache()`` after such a write.

Device status. Kernels report problems (a bounded wait that ran out, a span id out of range) in the
plan's status word. After every launch the word is copied to a pinned host mirror with an
asynchronous copy on the launching stream; the next call that uses the plan (or ``poll()``) looks at
the mirror without synchronising and raises, so a failed launch surfaces one call later at the
latest -- normally at the backward of the same step. ``KD_CHECK_STATUS=1`` makes every call
synchronise and check at once.
"""
from __future__ import annotations

import ctypes
import os
from collections import OrderedDict

import numpy as np
import torch

from . import _capi

_CACHE: "OrderedDict[tuple, AttentionPlan]" = OrderedDict()
_CACHE_SIZE = 64


def _tensor_key(t):
    if t is None:
        return None
    return (t.data_ptr(), t._version, tuple(t.shape), tuple(t.stride()), str(t.dtype))


_PINNED_WORDS = None
_PINNED_NEXT = 0


def _pinned_status_word() -> torch.Tensor:
    """One int32 of pinned host memory for a plan's status mirror. Pinning memory is a slow, device-wide
    call, so the words come from one pinned block handed out in rotation (1024 slots: a collision would
    need more than 1024 live plans, and could only make a reported failure show up on two of them)."""
    global _PINNED_WORDS, _PINNED_NEXT
    if _PINNED_WORDS is None:
        _PINNED_WORDS = torch.zeros(1024, dtype=torch.int32).pin_memory()
    w = _PINNED_WORDS[_PINNED_NEXT:_PINNED_NEXT + 1]
    _PINNED_NEXT = (_PINNED_NEXT + 1) % 1024
    w.zero_()
    return w


class AttentionPlan:
    """Device-resident plan for B sequences of T tokens (layout: kd_plan_layout in kd_attention.h)."""

    def __init__(self, B, T, device, in_span=None, span_id=None, is_prefix=None, lens=None,
                 causal=True, rules=False):
        self.B, self.T, self.device = B, T, device
        self.layout = _capi.plan_layout(B, T)
        self.NT, self.NP = self.layout.NT, self.layout.NP
        # torch's caching allocator returns 512-byte aligned blocks, which covers the 256 the ABI asks for
        self.buf = torch.empty(self.layout.total, dtype=torch.uint8, device=device)
        meta = _capi.KdMeta()
        meta.B, meta.T = B, T
        keep = []

        def prep(t, dtype, name):
            if t is None:
                return None, 0
            if t.shape != (B, T):
                raise ValueError(f"{name} must have shape (B, T) = ({B}, {T}), got {tuple(t.shape)}")
            if t.device != device:
                raise ValueError(f"{name} must live on {device}")
            if dtype is torch.bool and t.dtype is not torch.bool:
                raise ValueError(f"{name} must be a torch.bool tensor (the rule negates it logically)")
            if dtype is torch.int64 and t.dtype is not torch.int64:
                t = t.to(torch.int64)
            if t.stride(1) != 1:
                t = t.contiguous()
            keep.append(t)
            return t.data_ptr(), t.stride(0)

        meta.in_span, meta.in_span_stride_b = prep(in_span, torch.bool, "in_span")
        meta.span_id, meta.span_id_stride_b = prep(span_id, torch.int64, "span_id")
        meta.is_prefix, meta.is_prefix_stride_b = prep(is_prefix, torch.bool, "is_prefix")
        if lens is not None:
            if lens.dtype is not torch.int32 or lens.shape != (B,):
                raise ValueError("lens must be an int32 tensor of shape (B,)")
            lens = lens.contiguous()
            keep.append(lens)
            meta.lens = lens.data_ptr()
        meta.causal = 1 if causal else 0
        meta.rules = 1 if rules else 0
        # the caller's tensors and their converted copies stay alive while the plan is cached, so none of
        # the addresses in the cache key can be handed to another tensor
        self._keep = keep + [x for x in (in_span, span_id, is_prefix, lens) if x is not None]
        off = self.layout.off_status
        self._status_dev = self.buf[off:off + 4].view(torch.int32)
        self._status_host = _pinned_status_word()
        cur = torch.cuda.current_stream(device)
        with torch.cuda.device(device):
            _capi.check(_capi.load().kd_classify(ctypes.byref(meta), self.buf.data_ptr(), cur.cuda_stream))
        # a plan used later from another stream must wait for the classifier
        self._built_on = cur
        self._built = torch.cuda.Event()
        self._built.record(cur)
        self.mirror_status()
        if os.environ.get("KD_CHECK_STATUS") == "1":
            self.check_status()

    # ---- views into the plan buffer -------------------------------------------------------------
    def _view(self, off, nbytes, dtype, shape):
        return self.buf[off:off + nbytes].view(dtype).view(shape)

    @property
    def ptr(self) -> int:
        return self.buf.data_ptr()

    @property
    def desc(self) -> torch.Tensor:
        n = self.B * self.NT * _capi.KD_TILE
        return self._view(self.layout.off_desc, n * 4, torch.int32, (self.B, self.NT * _capi.KD_TILE))

    @property
    def tile_classes(self) -> torch.Tensor:
        """uint8 (B, NT, NT): class of tile [b][q_tile][k_tile]."""
        n = self.B * self.NT * self.NT
        return self._view(self.layout.off_cls, n, torch.uint8, (self.B, self.NT, self.NT))

    @property
    def stats(self) -> torch.Tensor:
        """int32 (B, 2): number of FULL and PARTIAL tiles per sequence."""
        return self._view(self.layout.off_stats, self.B * 8, torch.int32, (self.B, 2))

    @property
    def fwd_counts(self) -> torch.Tensor:
        return self._view(self.layout.off_fwd_cnt, self.B * self.NP * 4, torch.int32, (self.B, self.NP))

    @property
    def bwd_counts(self) -> torch.Tensor:
        return self._view(self.layout.off_bwd_cnt, self.B * self.NT * 4, torch.int32, (self.B, self.NT))

    def use_on_current_stream(self) -> None:
        """Orders the current stream after the classifier when the plan was built on another one."""
        cur = torch.cuda.current_stream(self.device)
        if cur != self._built_on:
            cur.wait_event(self._built)

    def status(self) -> int:
        """Reads the device status word (synchronises the current stream)."""
        return int(self._status_dev.item()) & 0xFFFFFFFF

    def mirror_status(self) -> None:
        """Enqueues a copy of the status word to the pinned host mirror behind the work just launched."""
        self._status_host.copy_(self._status_dev, non_blocking=True)

    def poll(self) -> None:
        """Raises if the host mirror holds a status a finished launch reported. Never synchronises."""
        s = int(self._status_host[0]) & 0xFFFFFFFF
        if s:
            self._report(s)

    def check_status(self) -> None:
        """Synchronises the current stream, reads the device status word and raises if it is set."""
        s = self.status()
        if s:
            self._report(s)

    def _report(self, s: int) -> None:
        # the word is cleared so that one event is reported once and later launches start clean
        self._status_dev.zero_()
        self._status_host.zero_()
        if s & _capi.KD_STATUS_SPAN_RANGE:
            raise ValueError("span_id values must fit in 24 signed bits (|span_id| < 2**23)")
        if s & _capi.KD_STATUS_TIMEOUT:
            raise RuntimeError(f"a device-side wait timed out (status 0x{s:08x}, wait site 0x{s & 0xFFFF:x}); "
                               "the results of that launch are invalid")
        raise RuntimeError(f"device status 0x{s:08x}")

    def dense_mask(self) -> torch.Tensor:
        """bool (B, T, T) mask materialised on the device from the descriptors."""
        out = torch.empty((self.B, self.T, self.T), dtype=torch.uint8, device=self.device)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        with torch.cuda.device(self.device):
            _capi.check(_capi.load().kd_mask_dense(self.ptr, self.B, self.T, out.data_ptr(), stream))
        return out.view(torch.bool)

    def nonempty_tiles(self) -> int:
        """Total number of non-EMPTY 128x128 tiles over the batch (one head)."""
        return int(self.stats.sum().item())


def get_plan(B, T, device, in_span=None, span_id=None, is_prefix=None, lens=None, causal=True,
             rules=False) -> AttentionPlan:
    """Returns a cached plan for this metadata, classifying on the device if it is new."""
    key = (B, T, str(device), _tensor_key(in_span), _tensor_key(span_id), _tensor_key(is_prefix),
           _tensor_key(lens), bool(causal), bool(rules))
    plan = _CACHE.get(key)
    if plan is not None:
        _CACHE.move_to_end(key)
        plan.use_on_current_stream()
        plan.poll()
        return plan
    plan = AttentionPlan(B, T, device, in_span, span_id, is_prefix, lens, causal, rules)
    _CACHE[key] = plan
    while len(_CACHE) > _CACHE_SIZE:
        _CACHE.popitem(last=False)
    return plan


def clear_plan_cache() -> None:
    _CACHE.clear()
