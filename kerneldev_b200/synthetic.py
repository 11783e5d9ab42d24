"""Seeded synthetic metadata with the layout the reference's cocktail-party collate produces
(data_builder.py:596-653): ``[prefix .. CLS][context]([SPAN] tokens [ES])*n [MASKQ][PAD..]``.

``in_span`` / ``is_prefix`` are bool, ``span_id`` int64 with 1-based span ids and -1 at [MASKQ];
[PAD] carries all-zero metadata and is masked through ``lens`` (= MASKQ index + 1). Stands in for
the reference's datasets, which need network access.
"""
from __future__ import annotations

import numpy as np

# section-length ranges (inclusive) of the benchmark configurations
CONFIG_RANGES = {
    2: dict(prefix=(32, 256), context=(1024, 2048), n_spans=(4, 32), span_len=(16, 128)),
    3: dict(prefix=(32, 256), context=(2048, 4096), n_spans=(8, 64), span_len=(16, 128)),
    4: dict(prefix=(16, 128), context=(512, 1024), n_spans=(2, 16), span_len=(8, 64)),
}


def sequence_metadata(T, prefix_len, context_len, span_lens):
    in_span = np.zeros(T, bool)
    span_id = np.zeros(T, np.int64)
    is_prefix = np.zeros(T, bool)
    is_prefix[:prefix_len] = True
    pos = prefix_len + context_len
    for s, n in enumerate(span_lens, start=1):
        in_span[pos:pos + n] = True
        span_id[pos:pos + n] = s
        pos += n
    span_id[pos] = -1
    return in_span, span_id, is_prefix, pos + 1


def batch_metadata(seed, B, T, prefix, context, n_spans, span_len):
    """Draws, per sequence and in this order, prefix length, context length, span count and span
    lengths from ``numpy.random.default_rng(seed)``; spans are kept while the sequence plus one
    [MASKQ] still fits in T. Returns (in_span, span_id, is_prefix, lens) as numpy arrays."""
    rng = np.random.default_rng(seed)
    ins = np.zeros((B, T), bool)
    sid = np.zeros((B, T), np.int64)
    pre = np.zeros((B, T), bool)
    lens = np.zeros(B, np.int32)
    for b in range(B):
        p = int(rng.integers(prefix[0], prefix[1] + 1))
        c = int(rng.integers(context[0], context[1] + 1))
        ns = int(rng.integers(n_spans[0], n_spans[1] + 1))
        sl = [int(x) for x in rng.integers(span_len[0], span_len[1] + 1, size=ns)]
        p = min(p, T - 1)
        c = min(c, T - 1 - p)
        pos, kept = p + c, []
        for n in sl:
            if pos + n + 1 <= T:
                kept.append(n)
                pos += n
        ins[b], sid[b], pre[b], lens[b] = sequence_metadata(T, p, c, kept)
    return ins, sid, pre, lens
