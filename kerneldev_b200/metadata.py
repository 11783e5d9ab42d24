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
