"""Cocktail-party head on the device (model.py:258-299).

After the last block the reference scores every span of a row against the row's [MASK] position:
``h_context[b]`` = the embedding at the first [MASK] token, ``h_spans[b, j]`` = the mean embedding of
the tokens between the j-th [SPAN] and the j-th [ES], ``scores = einsum('bd,bnd->bn')``. It finds the
markers with ``.nonzero()`` / ``torch.unique`` and fills ``h_spans`` in a Python double loop over rows
and spans (one small ``mean`` kernel and several host synchronisations per span).

``span_means`` does the marker ranking and the means with three kernels (one of them only in the
backward) and a single host read (the padded span count, which fixes the output shape as in the
reference); ``cocktail_scores`` is the whole block. Both are differentiable with respect to x_embed.
"""
from __future__ import annotations

import torch

from . import _capi
from .metadata import SPECIAL_TOKENS

_DT = {torch.float16: _capi.KD_F16, torch.bfloat16: _capi.KD_BF16, torch.float32: _capi.KD_F32}


def span_index(tokens: torch.Tensor, special_tokens=None):
    """(starts, ends, n_starts, n_ends, first_mask) of int64 token ids (batch, time) on a CUDA device:
    starts[b, r] / ends[b, r] = position of the r-th [SPAN] / [ES] of row b (-1 beyond the count)."""
    if tokens.dim() != 2 or tokens.dtype != torch.int64:
        raise ValueError("tokens must be an int64 tensor of shape (batch, time)")
    if not tokens.is_cuda:
        raise RuntimeError("span_index runs on CUDA devices only; there is no CPU path")
    st = SPECIAL_TOKENS if special_tokens is None else special_tokens
    if tokens.stride(1) != 1:
        tokens = tokens.contiguous()
    B, T = tokens.shape
    dev = tokens.device
    starts = torch.empty((B, T), dtype=torch.int32, device=dev)
    ends = torch.empty((B, T), dtype=torch.int32, device=dev)
    n_starts = torch.zeros((B,), dtype=torch.int32, device=dev)
    n_ends = torch.zeros((B,), dtype=torch.int32, device=dev)
    first_mask = torch.full((B,), -1, dtype=torch.int32, device=dev)
    with torch.cuda.device(dev):
        _capi.check(_capi.load().kd_span_index(
            tokens.data_ptr(), tokens.stride(0) if B > 1 else max(T, 1), B, T, st["[SPAN]"], st["[ES]"], st["[MASK]"],
            starts.data_ptr(), ends.data_ptr(), n_starts.data_ptr(), n_ends.data_ptr(), first_mask.data_ptr(),
            torch.cuda.current_stream(dev).cuda_stream))
    return starts, ends, n_starts, n_ends, first_mask


def _span_mean_call(backward, a, out, B, T, C, S, index):
    starts, ends, n_starts, n_ends = index
    with torch.cuda.device(a.device):
        _capi.check(_capi.load().kd_span_mean(
            1 if backward else 0, a.data_ptr(), a.stride(0), a.stride(1), out.data_ptr(), out.stride(0), out.stride(1),
            B, T, C, S, _DT[a.dtype], starts.data_ptr(), ends.data_ptr(), n_starts.data_ptr(), n_ends.data_ptr(),
            torch.cuda.current_stream(a.device).cuda_stream))


class _SpanMeanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, index, S):
        B, T, C = x.shape
        if x.stride(2) != 1:
            x = x.contiguous()
        h = torch.empty((B, S, C), dtype=x.dtype, device=x.device)
        _span_mean_call(False, x, h, B, T, C, S, index)
        ctx.index, ctx.shape, ctx.S = index, (B, T, C), S
        return h

    @staticmethod
    def backward(ctx, gh):
        B, T, C = ctx.shape
        gh = gh.contiguous()
        gx = torch.empty((B, T, C), dtype=gh.dtype, device=gh.device)
        _span_mean_call(True, gh, gx, B, T, C, ctx.S, ctx.index)
        return gx, None, None


def span_means(x_embed: torch.Tensor, tokens: torch.Tensor, special_tokens=None, index=None):
    """h_spans (batch, max_spans, dim) of model.py:280-293 for x_embed (batch, time, dim) in fp16 / bf16 /
    fp32 on a CUDA device; max_spans = the largest [SPAN] count of the batch (one host read)."""
    if x_embed.dim() != 3 or x_embed.dtype not in _DT:
        raise ValueError("x_embed must be (batch, time, dim) in float16, bfloat16 or float32")
    if not x_embed.is_cuda:
        raise RuntimeError("span_means runs on CUDA devices only; there is no CPU path")
    if index is None:
        index = span_index(tokens, special_tokens)
    S = int(index[2].max().item()) if index[2].numel() else 0
    if S == 0:
        return x_embed.new_zeros((x_embed.shape[0], 0, x_embed.shape[2]))
    return _SpanMeanFn.apply(x_embed, tuple(index[:4]), S)


def cocktail_scores(x_embed: torch.Tensor, tokens: torch.Tensor, special_tokens=None):
    """scores (batch, max_spans) of model.py:262-296: <embedding at the row's first [MASK], mean embedding
    of each of its spans>; rows without a [MASK] score 0."""
    index = span_index(tokens, special_tokens)
    h_spans = span_means(x_embed, tokens, special_tokens, index)
    first_mask = index[4].long()
    rows = torch.arange(x_embed.shape[0], device=x_embed.device)
    h_context = x_embed[rows, first_mask.clamp(min=0)] * (first_mask >= 0).unsqueeze(1).to(x_embed.dtype)
    return torch.einsum("bd,bnd->bn", h_context, h_spans)
