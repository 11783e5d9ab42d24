"""Host side of the attention operator: the call signature of the reference's
``original_kernel.flash_attention`` (original_kernel.py:2096-2168) in front of the hand-written
sm_100a kernels in libkd_attention.so.

``flash_attention`` is a drop-in for ``model.MultiHeadAttention`` (model.py:83-93): same
arguments, same return structure, O contiguous in the dtype of q (original_kernel.py:1801), LSE in base-2 units
(original_kernel.py:603-604), gradients for q, k and v only (the gradient of LSE is ignored,
as at original_kernel.py:1965-1992).

Differences from the reference, all deliberate:
  * the mask is the rule of original_kernel.py:480-517 for the forward AND the backward; the
    reference's backward loop bounds ignore the bidirectional sections when ``causal=True`` and
    metadata is given (original_kernel.py:1202-1204, :1368-1371);
  * a query row that sees no key gets O = 0, LSE = -inf and no gradient (the reference's default
    path produces NaN there, original_kernel.py:554-561);
  * CUDA sm_100 only, fp16 / bf16, head_dim a multiple of 16 up to 128 (the reference also takes 256 and
    fp32 tensors). There is no Triton, no autotuning and no
    CPU path: unsupported inputs raise.
``autotune``, ``prescale_qk`` and ``precision`` are accepted and ignored.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch

from . import _capi
from .plan import AttentionPlan, get_plan

_capi.load()  # fail at import time, loudly, when the CUDA library has not been built

__all__ = ["flash_attention", "generate_hadamard_signs", "hadamard_transform"]

_DTYPES = {torch.float16: _capi.KD_F16, torch.bfloat16: _capi.KD_BF16}

# Heads a CTA handles one after the other (kd_attn_params.heads_per_cta): 0 lets the library choose from
# the grid size. Small problems get 1 by themselves, so the tests of the multi-head path set this.
HEADS_PER_CTA = 0


def _kd_tensor(t: torch.Tensor) -> _capi.KdTensor:
    return _capi.KdTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def _usable(t: torch.Tensor) -> torch.Tensor:
    """Returns t itself when TMA can describe it (unit stride along D, 16-byte aligned rows),
    else one contiguous copy."""
    es = t.element_size()
    ok = (t.stride(3) == 1 and t.data_ptr() % 16 == 0
          and all((t.stride(i) * es) % 16 == 0 and t.stride(i) > 0 for i in range(3)))
    return t if ok else t.contiguous()


def _check_inputs(q, k, v):
    if q.dim() != 4:
        raise ValueError("q, k, v must be (batch, heads, time, head_dim)")
    if not (q.shape == k.shape == v.shape):
        raise ValueError(f"q, k, v must have the same shape, got {tuple(q.shape)}, {tuple(k.shape)}, {tuple(v.shape)}")
    if not q.is_cuda:
        raise RuntimeError("flash_attention runs on CUDA sm_100 devices only; there is no CPU path")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype float16, bfloat16 or float32")
    if q.shape[-1] % 16 != 0 or not 16 <= q.shape[-1] <= 128:
        raise ValueError(f"head_dim {q.shape[-1]} is not supported (a multiple of 16 from 16 to 128)")
    if not (k.device == q.device and v.device == q.device):
        raise ValueError("q, k, v must be on the same device")


def _params(q, k, v, o, lse, plan, sm_scale):
    B, H, T, D = q.shape
    p = _capi.KdAttnParams()
    p.B, p.H, p.T, p.D = B, H, T, D
    p.dtype = _DTYPES[q.dtype]
    p.sm_scale = sm_scale
    p.q, p.k, p.v, p.o = _kd_tensor(q), _kd_tensor(k), _kd_tensor(v), _kd_tensor(o)
    p.lse = lse.data_ptr()
    p.plan = plan.ptr
    p.heads_per_cta = HEADS_PER_CTA
    return p


def _after_launch(plan: AttentionPlan) -> None:
    """Device-side failures (a bounded wait that gave up) are written to the plan's status word. The word
    follows every launch to a pinned host mirror; ``plan.poll()`` at the next call raises from it without
    a synchronisation. KD_CHECK_STATUS=1 synchronises and checks after every launch instead."""
    plan.mirror_status()
    if os.environ.get("KD_CHECK_STATUS") == "1":
        plan.check_status()


def _forward(q, k, v, plan: AttentionPlan, sm_scale: float, like_input: bool = False):
    """One kd_attn_fwd call: returns (O, LSE) for inputs that passed _check_inputs. ``like_input``: O in the
    memory layout of q instead of contiguous."""
    q, k, v = _usable(q), _usable(k), _usable(v)
    B, H, T, D = q.shape
    # empty_like keeps the strides of a dense q, e.g. (B,T,H,D) memory seen as (B,H,T,D)
    o = torch.empty_like(q) if like_input else torch.empty((B, H, T, D), dtype=q.dtype, device=q.device)
    lse = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
    p = _params(q, k, v, o, lse, plan, sm_scale)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    plan.poll()
    with torch.cuda.device(q.device):
        _capi.check(_capi.load().kd_attn_fwd(ctypes.byref(p), stream))
    _after_launch(plan)
    return o, lse


def _backward(q, k, v, o, lse, d_o, plan: AttentionPlan, sm_scale: float, phases: int = 0, bufs=None,
              like_input: bool = False, deterministic: bool = False):
    """One kd_attn_bwd call: returns (dQ, dK, dV). ``phases`` selects a part of the backward (see
    kd_attn_params.bwd_phases); ``bufs`` = (dq, dk, dv, delta[, dq_acc]) reuses buffers.
    ``deterministic=False`` selects the fused backward where it exists (head_dim <= 64): one pass over the
    tiles instead of two, dQ accumulated with fp32 atomics in a (B,H,T,D) scratch."""
    q, k, v, d_o = _usable(q), _usable(k), _usable(v), _usable(d_o)
    B, H, T, D = q.shape
    if bufs is None:
        if like_input:   # each gradient in its input's layout
            dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        else:
            dq = torch.empty((B, H, T, D), dtype=q.dtype, device=q.device)
            dk = torch.empty_like(dq)
            dv = torch.empty_like(dq)
        delta = torch.empty((B, H, T), dtype=torch.float32, device=q.device)
        dq_acc = None
    else:
        dq, dk, dv, delta = bufs[:4]
        dq_acc = bufs[4] if len(bufs) > 4 else None
    fused = (not deterministic) and D <= 64
    if fused and dq_acc is None:   # rows as wide as the kernel's tile (kd_workspace_bytes_fused)
        dq_acc = torch.empty((B, H, T, 64), dtype=torch.float32, device=q.device)
    p = _params(q, k, v, o, lse, plan, sm_scale)
    p.d_o = _kd_tensor(d_o)
    p.dq, p.dk, p.dv = _kd_tensor(dq), _kd_tensor(dk), _kd_tensor(dv)
    p.delta = delta.data_ptr()
    p.bwd_phases = phases
    if fused:
        p.bwd_mode = _capi.KD_BWD_FUSED
        p.dq_acc = dq_acc.data_ptr()
    stream = torch.cuda.current_stream(q.device).cuda_stream
    plan.poll()
    with torch.cuda.device(q.device):
        _capi.check(_capi.load().kd_attn_bwd(ctypes.byref(p), stream))
    _after_launch(plan)
    return dq, dk, dv


class _FlashAttentionFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, plan, sm_scale, like_input=False, deterministic=False):
        o, lse = _forward(q, k, v, plan, sm_scale, like_input)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.plan = plan
        ctx.sm_scale = sm_scale
        ctx.like_input = like_input
        ctx.deterministic = deterministic
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, d_o, _d_lse):
        q, k, v, o, lse = ctx.saved_tensors
        dq, dk, dv = _backward(q, k, v, o, lse, d_o, ctx.plan, ctx.sm_scale, like_input=ctx.like_input,
                               deterministic=ctx.deterministic)
        return dq, dk, dv, None, None, None, None


def _hadamard_call(x: torch.Tensor, signs, inverse: bool) -> torch.Tensor:
    x = _usable(x)
    B, H, T, D = x.shape
    y = torch.empty((B, H, T, D), dtype=x.dtype, device=x.device)
    xs, ys = _kd_tensor(x), _kd_tensor(y)
    stream = torch.cuda.current_stream(x.device).cuda_stream
    with torch.cuda.device(x.device):
        _capi.check(_capi.load().kd_hadamard(ctypes.byref(xs), ctypes.byref(ys), B, H, T, D, _DTYPES[x.dtype],
                                             signs.data_ptr() if signs is not None else None,
                                             1 if inverse else 0, stream))
    return y


class _HadamardFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, signs):
        ctx.signs = signs
        return _hadamard_call(x, signs, inverse=False)

    @staticmethod
    def backward(ctx, dy):
        # y = x diag(s) W / sqrt(D) with W symmetric, so dx = dy W / sqrt(D) diag(s)
        return _hadamard_call(dy, ctx.signs, inverse=True), None


def generate_hadamard_signs(n_heads: int, head_dim: int, seed: int = 0, device="cuda") -> torch.Tensor:
    """(n_heads, head_dim) float32 tensor of +-1 drawn from a seeded CPU generator.

    The reference only names this utility (README.md:68-77); the recipe here is this package's own:
    ``torch.randint(0, 2, (n_heads, head_dim), generator=torch.Generator().manual_seed(seed)) * 2 - 1``.
    """
    g = torch.Generator(device="cpu").manual_seed(seed)
    s = torch.randint(0, 2, (n_heads, head_dim), generator=g, dtype=torch.int64) * 2 - 1
    return s.to(torch.float32).to(device)


def hadamard_transform(x: torch.Tensor, signs: torch.Tensor | None = None) -> torch.Tensor:
    """``WHT(x * signs[h]) / sqrt(D)`` over the last dimension of a (B, H, T, D) tensor, with the
    Walsh-Hadamard matrix in natural (Sylvester) order; differentiable."""
    if x.dim() != 4 or x.shape[-1] not in (16, 32, 64, 128) or x.dtype not in _DTYPES or not x.is_cuda:
        raise ValueError("hadamard_transform expects a CUDA (B, H, T, D) fp16/bf16 tensor with D in {16, 32, 64, 128}")
    if signs is not None:
        if signs.shape != (x.shape[1], x.shape[3]):
            raise ValueError("signs must have shape (heads, head_dim)")
        signs = signs.to(device=x.device, dtype=torch.float32).contiguous()
    return _HadamardFn.apply(x, signs)


def flash_attention(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    lens: torch.Tensor | None = None,
    sm_scale: float | None = None,
    causal: bool = True,
    autotune=False,
    return_lse=False,
    prescale_qk=False,
    precision="tf32",
    attention_mask: torch.Tensor | None = None,
    in_span: torch.Tensor | None = None,
    span_id: torch.Tensor | None = None,
    is_prefix: torch.Tensor | None = None,
    return_attention_mask: bool = False,
    hadamard_signs: torch.Tensor | None = None,
    out_layout: str = "contiguous",
    deterministic: bool = False,
):
    """Self-attention with the 4-section hierarchical mask; arguments and return value as the
    reference's ``flash_attention`` (original_kernel.py:2096-2168).

    q, k, v: (batch, heads, time, head_dim), any strides. lens: int32 (batch,) or None.
    in_span / is_prefix: bool (batch, time); span_id: int64 (batch, time) (1-based span ids, -1 at
    [MASKQ]). When any of attention_mask / in_span / span_id / is_prefix is given the mask is the
    rule of original_kernel.py:480-517 and ``causal`` is not part of it; otherwise the mask is
    ``i >= j`` (causal) or all-ones. ``attention_mask`` itself is never read (as in the reference).

    hadamard_signs (extension, default None): (heads, head_dim) +-1; Q and K are replaced by
    ``hadamard_transform(., signs)`` before the attention, which leaves Q K^T unchanged in exact
    arithmetic and spreads outliers over the head dimension.
    out_layout (extension): "contiguous" (default, as original_kernel.py:1801 and :1920-1922) or
    "input": O and the gradients take the memory layout of q, k, v. For the model's (B,H,T,D) views
    of (B,T,H,D) memory (model.py:76-78) the ``transpose(1, 2).contiguous()`` after the call
    (model.py:95) and its counterpart in the backward then copy nothing. The drop-in module uses it.
    deterministic (extension, default False): True forces the two-kernel backward, whose results are
    bit-identical from run to run; by default head_dim <= 64 takes the fused backward, which forms S and dP
    once per tile and adds dQ partials with fp32 atomics (dQ then varies in its last bits between runs).

    float32 q, k, v (the reference's default ``precision="tf32"`` path, original_kernel.py:2106): the tensors
    are rounded to float16 operands -- the 10-bit mantissa tf32 keeps -- the products accumulate in fp32 as
    everywhere, and O and the gradients come back as float32. Values must lie inside float16's range
    (|x| < 65504; tf32 keeps fp32's exponent). ``precision="ieee"`` with float32 tensors is not supported.

    Returns O, or (O, LSE) with return_lse, or (that, mask[B,H,T,T] bool) with return_attention_mask.
    """
    if q.dtype is torch.float32 and k.dtype is torch.float32 and v.dtype is torch.float32:
        if precision == "ieee":
            raise ValueError("float32 inputs with precision='ieee' are not supported: the tensor cores take 16-bit operands here "
                             "(precision='tf32' rounds the operands to tf32's 10-bit mantissa)")
        res = flash_attention(q.to(torch.float16), k.to(torch.float16), v.to(torch.float16), lens, sm_scale, causal, autotune,
                              return_lse, prescale_qk, precision, attention_mask, in_span, span_id, is_prefix,
                              return_attention_mask, hadamard_signs, out_layout, deterministic)
        widen = lambda x: x.to(torch.float32) if torch.is_tensor(x) and x.dtype is torch.float16 else x
        if return_attention_mask:
            first, mask = res
            first = tuple(widen(x) for x in first) if isinstance(first, tuple) else widen(first)
            return first, mask
        return tuple(widen(x) for x in res) if isinstance(res, tuple) else widen(res)
    _check_inputs(q, k, v)
    B, H, T, D = q.shape
    if sm_scale is None:
        sm_scale = D ** -0.5
    sm_scale = float(sm_scale)
    if not (sm_scale > 0.0 and math.isfinite(sm_scale)):
        raise ValueError("sm_scale must be positive and finite")
    rules = any(t is not None for t in (attention_mask, in_span, span_id, is_prefix))
    plan = get_plan(B, T, q.device, in_span, span_id, is_prefix, lens, causal, rules)

    if hadamard_signs is not None:
        q = hadamard_transform(q, hadamard_signs)
        k = hadamard_transform(k, hadamard_signs)

    if out_layout not in ("contiguous", "input"):
        raise ValueError("out_layout must be 'contiguous' or 'input'")
    o, lse = _FlashAttentionFn.apply(q, k, v, plan, sm_scale, out_layout == "input", bool(deterministic))

    if return_attention_mask:
        mask = plan.dense_mask().unsqueeze(1).expand(B, H, T, T)
        if return_lse:
            return (o, lse), mask
        return o, mask
    if return_lse:
        return o, lse
    return o
