"""CPU restatement of KernelDev's attention path.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline / reference legs
may import this module; nothing under ``kerneldev_b200/`` does.

What it restates (reference = Eupham/KernelDev, file:line inside that project):
  * dense_mask        -- the 4-section rule, original_kernel.py:332-347 (query predicates),
                         :460-510 (key predicates + rule), :512-517 (fallbacks + length mask)
  * attention_forward -- base-2 online-softmax math of _flash_attn_fwd: scores * sm_scale*log2(e)
                         (:415), exp2 (:554-563), LSE = m + log2(l) (:603-604); evaluated densely
  * attention_backward-- delta = rowsum(O*dO) (:695); dQ worker algebra (:1239-1335);
                         dK/dV worker algebra (:1425-1524)
  * section generators-- the canonical layout of data_builder.py:596-653
  * hadamard_*        -- NOT in the reference code (named only in README.md:68-77); defined here
                         and in kerneldev_b200.original_kernel identically.  Parity unpinned.

Pinning: tests/golden/*.npz hold outputs of the reference's own Triton kernels executed in
the Triton CPU interpreter (script: tests/golden/make_golden.py); tests/test_oracle.py checks
this restatement against them.  Rows without any visible key: O = 0, LSE = -inf, zero
gradients (the reference's default path yields NaN there; such rows are excluded from the
pinning comparison).
"""
from __future__ import annotations

import math

import numpy as np
import torch

LOG2E = 1.4426950408889634
TILE = 128
EMPTY, FULL, PARTIAL = 0, 1, 2


# ------------------------------------------------------------------------------------------
# mask
# ------------------------------------------------------------------------------------------
def dense_mask(T, in_span=None, span_id=None, is_prefix=None, lens=None, causal=True,
               attention_mask_given=False, B=None) -> np.ndarray:
    """bool (B, T, T): mask[b, i, j] = may query i attend to key j (original_kernel.py:480-517)."""
    metas = [m for m in (in_span, span_id, is_prefix) if m is not None]
    if B is None:
        B = int(metas[0].shape[0]) if metas else (int(len(lens)) if lens is not None else 1)
    to_np = lambda x: None if x is None else (x.detach().cpu().numpy() if torch.is_tensor(x) else np.asarray(x))
    in_span, span_id, is_prefix, lens = map(to_np, (in_span, span_id, is_prefix, lens))
    rules = attention_mask_given or bool(metas)
    idx = np.arange(T)
    ge = idx[:, None] >= idx[None, :]
    out = np.empty((B, T, T), dtype=bool)
    for b in range(B):
        if rules:
            ins = in_span[b].astype(bool) if in_span is not None else np.zeros(T, bool)
            pre = is_prefix[b].astype(bool) if is_prefix is not None else np.zeros(T, bool)
            sid = span_id[b].astype(np.int64) if span_id is not None else np.zeros(T, np.int64)
            mq = (sid == -1) if span_id is not None else np.zeros(T, bool)
            ctx = ~ins & ~pre & ~mq
            m = pre[:, None] & pre[None, :]                                   # prefix <-> prefix
            m |= ctx[:, None] & ctx[None, :] & ge                             # context causal
            m |= ctx[:, None] & pre[None, :]                                  # context -> prefix
            m |= ins[:, None] & ins[None, :] & (sid[:, None] == sid[None, :]) & (sid[:, None] > 0)
            m |= ins[:, None] & ctx[None, :]                                  # span -> all context
            m |= mq[:, None] & ins[None, :]                                   # MASKQ -> spans
            m |= mq[:, None] & pre[None, :]                                   # MASKQ -> prefix
        else:
            m = ge.copy() if causal else np.ones((T, T), bool)
        if lens is not None:
            n = min(int(lens[b]), T)
            m[n:, :] = False
            m[:, n:] = False
        out[b] = m
    return out


def tile_classes(mask: np.ndarray, tile: int = TILE) -> np.ndarray:
    """uint8 (B, NT, NT): EMPTY / FULL / PARTIAL of every tile x tile block; the part of an edge
    block that lies outside the (T, T) mask counts as masked."""
    B, T, _ = mask.shape
    NT = (T + tile - 1) // tile
    pad = NT * tile - T
    m = np.pad(mask, ((0, 0), (0, pad), (0, pad))) if pad else mask
    blocks = m.reshape(B, NT, tile, NT, tile)
    cnt = blocks.sum(axis=(2, 4))
    cls = np.full((B, NT, NT), PARTIAL, dtype=np.uint8)
    cls[cnt == 0] = EMPTY
    cls[cnt == tile * tile] = FULL
    return cls


# ------------------------------------------------------------------------------------------
# attention math (fp32, dense)
# ------------------------------------------------------------------------------------------
def attention_forward(q, k, v, mask, sm_scale=None):
    """q, k, v: (B, H, T, D) float tensors; mask: (B, T, T) bool. Returns O (fp32), LSE2 (fp32)."""
    q, k, v = q.float(), k.float(), v.float()
    D = q.shape[-1]
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    m = torch.as_tensor(mask, device=q.device)[:, None]
    s2 = (q @ k.transpose(-1, -2)) * (scale * LOG2E)             # base-2 scores (:415)
    s2 = s2.masked_fill(~m, float("-inf"))
    mx = s2.amax(dim=-1, keepdim=True)
    mx_safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    p = torch.exp2(s2 - mx_safe)
    l = p.sum(dim=-1, keepdim=True)
    o = (p @ v) / torch.where(l > 0, l, torch.ones_like(l))
    lse2 = (mx_safe + torch.log2(l)).squeeze(-1)                 # m + log2(l) (:603-604); -inf when l = 0
    lse2 = torch.where(l.squeeze(-1) > 0, lse2, torch.full_like(lse2, float("-inf")))
    o = torch.where(l > 0, o, torch.zeros_like(o))
    return o, lse2


def attention_backward(q, k, v, o, lse2, d_o, mask, sm_scale=None):
    """Closed-form gradients following the reference's two workers. Returns dQ, dK, dV (fp32)."""
    q, k, v, o, d_o = q.float(), k.float(), v.float(), o.float(), d_o.float()
    D = q.shape[-1]
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    m = torch.as_tensor(mask, device=q.device)[:, None]
    s2 = (q @ k.transpose(-1, -2)) * (scale * LOG2E)
    lse = torch.where(torch.isinf(lse2), torch.zeros_like(lse2), lse2)[..., None]
    p = torch.where(m, torch.exp2(s2 - lse), torch.zeros_like(s2))   # (:1273, :1459)
    delta = (o * d_o).sum(dim=-1, keepdim=True)                       # (:695)
    dv = p.transpose(-1, -2) @ d_o                                    # (:1519)
    dp = d_o @ v.transpose(-1, -2)                                    # (:1281, :1467)
    ds = p * (dp - delta)                                             # (:1331, :1517)
    dq = (ds @ k) * scale                                             # (:1333-1335)
    dk = (ds.transpose(-1, -2) @ q) * scale                           # (:1521-1524)
    return dq, dk, dv


def attention_fwd_bwd_operand_rounded(q, k, v, d_o, mask, dtype, sm_scale=None):
    """The same math with the roundings a 16-bit tensor-core implementation cannot avoid: P is rounded to
    `dtype` before P V and P^T dO (the reference forward does the same, original_kernel.py:565-566), O is
    rounded to `dtype` before delta = rowsum(O*dO) (delta is formed from the stored O, :695), and dS is
    rounded to `dtype` before dS K and dS^T Q (the reference rounds these operands to tf32 under its default
    precision, :1333, :1523). Accumulation stays fp32. Separates operand rounding from kernel error."""
    q, k, v, d_o = q.float(), k.float(), v.float(), d_o.float()
    D = q.shape[-1]
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    m = torch.as_tensor(mask, device=q.device)[:, None]
    rnd = lambda x: x.to(dtype).float()
    s2 = ((q @ k.transpose(-1, -2)) * (scale * LOG2E)).masked_fill(~m, float("-inf"))
    mx = s2.amax(dim=-1, keepdim=True)
    mx_safe = torch.where(torch.isinf(mx), torch.zeros_like(mx), mx)
    p = torch.exp2(s2 - mx_safe)
    l = p.sum(dim=-1, keepdim=True)
    live = l > 0
    o = torch.where(live, (rnd(p) @ v) / torch.where(live, l, torch.ones_like(l)), torch.zeros(1))
    lse2 = torch.where(live.squeeze(-1), (mx_safe + torch.log2(l)).squeeze(-1), torch.full_like(l.squeeze(-1), float("-inf")))
    lse = torch.where(torch.isinf(lse2), torch.zeros_like(lse2), lse2)[..., None]
    pn = torch.where(m, torch.exp2(s2 - lse), torch.zeros_like(s2))
    delta = (rnd(o) * d_o).sum(dim=-1, keepdim=True)
    dv = rnd(pn).transpose(-1, -2) @ d_o
    ds = rnd(pn * (d_o @ v.transpose(-1, -2) - delta))
    return o, lse2, (ds @ k) * scale, (ds.transpose(-1, -2) @ q) * scale, dv


def operand_rounding_bounds(q, k, v, d_o, mask, dtype, sm_scale=None):
    """First-order bounds on what rounding the second operand of each product to `dtype` can change:
    u*|P||V| for O, u*|P|^T|dO| for dV, scale*(u|dS| + P*u|O||dO|)|K| for dQ and its transpose with |Q| for dK
    (the second term is the rounding of the stored O that delta = rowsum(O*dO) is formed from), with u the
    unit roundoff of `dtype` (2^-11 for fp16, 2^-8 for bf16). With N(0,1) inputs these are far below the
    tolerances of the tests; with N(0,20) outliers in K and V single products |dS_ij K_jd| reach the
    hundreds and one rounding of dS_ij moves dQ by more than an absolute 2e-2. Returns (bO, bdQ, bdK, bdV)."""
    u = 2.0 ** -11 if dtype == torch.float16 else 2.0 ** -8
    q, k, v, d_o = q.float(), k.float(), v.float(), d_o.float()
    D = q.shape[-1]
    scale = (D ** -0.5) if sm_scale is None else sm_scale
    o, lse2 = attention_forward(q, k, v, mask, sm_scale)
    m = torch.as_tensor(mask, device=q.device)[:, None]
    s2 = (q @ k.transpose(-1, -2)) * (scale * LOG2E)
    lse = torch.where(torch.isinf(lse2), torch.zeros_like(lse2), lse2)[..., None]
    p = torch.where(m, torch.exp2(s2 - lse), torch.zeros_like(s2))
    ds = (p * (d_o @ v.transpose(-1, -2) - (o * d_o).sum(-1, keepdim=True))).abs()
    # delta = rowsum(O*dO) is formed from the stored 16-bit O: its error u*|O||dO| enters dS as P * d(delta)
    pd = p * (u * (o.abs() * d_o.abs()).sum(-1, keepdim=True))
    return (u * (p @ v.abs()), scale * ((u * ds + pd) @ k.abs()), scale * ((u * ds + pd).transpose(-1, -2) @ q.abs()),
            u * (p.transpose(-1, -2) @ d_o.abs()))


def attention_fwd_bwd(q, k, v, d_o, mask, sm_scale=None):
    o, lse2 = attention_forward(q, k, v, mask, sm_scale)
    dq, dk, dv = attention_backward(q, k, v, o, lse2, d_o, mask, sm_scale)
    return o, lse2, dq, dk, dv


# ------------------------------------------------------------------------------------------
# section generators (canonical layout of data_builder.py:596-653)
# ------------------------------------------------------------------------------------------
def sections_to_metadata(T, prefix_len, context_len, span_lens, with_maskq=True):
    """One sequence: [prefix ... CLS][context][SPAN .. ES]*n [MASKQ][PAD...]. Returns
    (in_span bool[T], span_id int64[T], is_prefix bool[T], n_real)."""
    in_span = np.zeros(T, bool)
    span_id = np.zeros(T, np.int64)
    is_prefix = np.zeros(T, bool)
    pos = 0
    is_prefix[:prefix_len] = True
    pos += prefix_len + context_len
    for sidx, sl in enumerate(span_lens, start=1):
        in_span[pos:pos + sl] = True
        span_id[pos:pos + sl] = sidx
        pos += sl
    if with_maskq:
        span_id[pos] = -1
        pos += 1
    assert pos <= T
    return in_span, span_id, is_prefix, pos


def config0_metadata(B=2, T=256):
    """BASELINE config 0: 16 prefix, 128 context, 8 spans of 12, MASKQ at 240, PAD to 256; lens 241."""
    ins, sid, pre, n = sections_to_metadata(T, 16, 128, [12] * 8)
    rep = lambda a: np.repeat(a[None], B, axis=0)
    return rep(ins), rep(sid), rep(pre), np.full(B, n, np.int32)


def random_sections(rng, T, prefix=(32, 256), context=(1024, 2048), n_spans=(4, 32), span_len=(16, 128)):
    """Seeded section lengths in the order prefix, context, span count, span lengths (all ranges
    inclusive); spans are appended while the sequence plus one MASKQ still fits in T."""
    p = int(rng.integers(prefix[0], prefix[1] + 1))
    c = int(rng.integers(context[0], context[1] + 1))
    ns = int(rng.integers(n_spans[0], n_spans[1] + 1))
    lens = [int(x) for x in rng.integers(span_len[0], span_len[1] + 1, size=ns)]
    p = min(p, T - 1)
    c = min(c, T - 1 - p)
    pos = p + c
    kept = []
    for sl in lens:
        if pos + sl + 1 <= T:
            kept.append(sl)
            pos += sl
    return p, c, kept


def batch_metadata(seed, B, T, **ranges):
    """(in_span, span_id, is_prefix, lens) numpy arrays for B seeded sequences; lens = MASKQ index + 1."""
    rng = np.random.default_rng(seed)
    ins = np.zeros((B, T), bool)
    sid = np.zeros((B, T), np.int64)
    pre = np.zeros((B, T), bool)
    lens = np.zeros(B, np.int32)
    for b in range(B):
        p, c, spans = random_sections(rng, T, **ranges)
        ins[b], sid[b], pre[b], lens[b] = sections_to_metadata(T, p, c, spans)
    return ins, sid, pre, lens


CONFIG_RANGES = {
    2: dict(prefix=(32, 256), context=(1024, 2048), n_spans=(4, 32), span_len=(16, 128)),
    3: dict(prefix=(32, 256), context=(2048, 4096), n_spans=(8, 64), span_len=(16, 128)),
    4: dict(prefix=(16, 128), context=(512, 1024), n_spans=(2, 16), span_len=(8, 64)),
}


# ------------------------------------------------------------------------------------------
# Hadamard incoherent processing (this build's definition; see module docstring)
# ------------------------------------------------------------------------------------------
def hadamard_matrix(n: int) -> torch.Tensor:
    h = torch.ones((1, 1))
    while h.shape[0] < n:
        h = torch.cat([torch.cat([h, h], 1), torch.cat([h, -h], 1)], 0)
    assert h.shape[0] == n, "n must be a power of two"
    return h


def generate_hadamard_signs(n_heads, head_dim, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randint(0, 2, (n_heads, head_dim), generator=g, dtype=torch.int64) * 2 - 1).float()


def hadamard_transform(x, signs=None):
    """x: (B, H, T, D). WHT(x * signs[h]) / sqrt(D), natural order, in fp32."""
    x = x.float()
    D = x.shape[-1]
    if signs is not None:
        x = x * signs[None, :, None, :].to(x.device)
    return (x @ hadamard_matrix(D).to(x.device)) / math.sqrt(D)


# ------------------------------------------------------------------------------------------
# metadata from token ids
# ------------------------------------------------------------------------------------------
SPECIAL_TOKENS = {"[PAD]": 0, "[CLS]": 1, "[MASK]": 2, "[SPAN]": 3, "[ES]": 4, "[MASKQ]": 5}   # data_builder.py:44-51


def metadata_from_tokens(tokens, special_tokens=None):
    """(in_span bool, span_id int64, is_prefix bool), each (B, T), from token ids (B, T): the fallback
    of GPTModel.forward (model.py:203-238). Both of its branches reduce to the same formulas: without
    [SPAN] / [ES] / [MASKQ] tokens the cumulative sums are zero (model.py:216-224 vs :231-237)."""
    st = SPECIAL_TOKENS if special_tokens is None else special_tokens
    x = tokens.detach().cpu().numpy() if torch.is_tensor(tokens) else np.asarray(tokens)
    c_span = np.cumsum(x == st["[SPAN]"], axis=1)
    c_es = np.cumsum(x == st["[ES]"], axis=1)
    in_span = (c_span - c_es) > 0                      # model.py:218
    span_id = np.where(in_span, c_span, 0).astype(np.int64)   # :219-220
    span_id[x == st["[MASKQ]"]] = -1                   # :223-224
    is_prefix = np.zeros(x.shape, dtype=bool)
    for b in range(x.shape[0]):                        # :227-231
        pos = np.nonzero(x[b] == st["[CLS]"])[0]
        if len(pos) > 0:
            is_prefix[b, : pos[0] + 1] = True
    return in_span, span_id, is_prefix


# ------------------------------------------------------------------------------------------
# cocktail-party head
# ------------------------------------------------------------------------------------------
def cocktail_scores(x_embed, tokens, special_tokens=None):
    """(scores (B, max_spans), h_spans (B, max_spans, D)) as model.py:262-296 computes them: the j-th [SPAN]
    of a row is paired with its j-th [ES] (zip stops at the shorter list, :288); a pair with
    st + 1 < ed contributes the mean of x_embed[b, st+1:ed], any other slot stays zero (:289-293);
    h_context is the embedding at the row's first [MASK] or zero (:265-273). Differentiable torch code
    on whatever device x_embed lives on (the tests run it on CPU)."""
    st_ = SPECIAL_TOKENS if special_tokens is None else special_tokens
    x = tokens.detach().cpu().numpy() if torch.is_tensor(tokens) else np.asarray(tokens)
    B, T = x.shape
    D = x_embed.shape[-1]
    max_spans = int((x == st_["[SPAN]"]).sum(1).max()) if B else 0
    h_context = x_embed.new_zeros((B, D))
    rows_spans = []
    for b in range(B):
        mpos = np.nonzero(x[b] == st_["[MASK]"])[0]
        if len(mpos) > 0:
            h_context = h_context.index_put((torch.tensor([b]),), x_embed[b, int(mpos[0])].unsqueeze(0))
        starts = np.nonzero(x[b] == st_["[SPAN]"])[0]
        ends = np.nonzero(x[b] == st_["[ES]"])[0]
        slots = [x_embed.new_zeros((D,)) for _ in range(max_spans)]
        for j, (s0, e0) in enumerate(zip(starts, ends)):
            if s0 + 1 < e0:
                slots[j] = x_embed[b, int(s0) + 1:int(e0)].mean(dim=0)
        rows_spans.append(torch.stack(slots) if max_spans else x_embed.new_zeros((0, D)))
    h_spans = torch.stack(rows_spans) if B else x_embed.new_zeros((0, max_spans, D))
    return torch.einsum("bd,bnd->bn", h_context, h_spans), h_spans

