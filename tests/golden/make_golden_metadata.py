"""Golden fixture for the token -> metadata step, produced by the REFERENCE's own code.

    REFERENCE_DIR=/path/to/KernelDev python tests/golden/make_golden_metadata.py

The fallback branch of ``GPTModel.forward`` (model.py:203-238) is read from the reference checkout at
generation time, dedented and executed on seeded token rows (nothing of it is stored here); the token
rows and its three outputs are saved to ``metadata_from_tokens.npz``.
"""
import os
import sys
import textwrap

import numpy as np
import torch

REF = os.environ["REFERENCE_DIR"]   # path of a checkout of the reference project
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REF)
from data_builder import SPECIAL_TOKENS  # noqa: E402  (the reference's table)


def reference_block():
    lines = open(os.path.join(REF, "model.py")).read().splitlines()
    start = next(i for i, l in enumerate(lines) if "Fallback: Generate metadata from tokens" in l) + 1
    end = next(i for i, l in enumerate(lines) if "Apply transformer blocks" in l)
    return textwrap.dedent("\n".join(lines[start:end]))


def run_reference(x):
    ns = {"torch": torch, "SPECIAL_TOKENS": SPECIAL_TOKENS, "x": x, "batch_size": x.shape[0], "seq_len": x.shape[1]}
    exec(reference_block(), ns)
    return ns["in_span"], ns["span_id"], ns["is_prefix"]


def token_rows(seed, B, T):
    """Canonical rows ([prefix][CLS] context ([SPAN] .. [ES])* [MASKQ] pad), rows without markers, rows with
    unbalanced / nested / repeated markers: the formulas are defined for all of them."""
    rng = np.random.default_rng(seed)
    x = rng.integers(6, 200, size=(B, T))
    for b in range(B):
        kind = b % 4
        if kind == 0:      # canonical
            cls = int(rng.integers(1, T // 4)); x[b, cls] = 1
            t = cls + int(rng.integers(5, T // 3))
            while t + 12 < T - 2 and rng.random() < 0.8:
                ln = int(rng.integers(3, 10)); x[b, t] = 3; x[b, t + ln] = 4; t += ln + int(rng.integers(1, 6))
            x[b, min(t + 1, T - 1)] = 5
        elif kind == 1:    # no markers at all
            pass
        elif kind == 2:    # random markers, unbalanced and nested, several [CLS] and [MASKQ]
            pos = rng.choice(T, size=T // 6, replace=False)
            x[b, pos] = rng.integers(0, 6, size=len(pos))
        else:              # [ES] before any [SPAN], [CLS] at position 0, trailing [SPAN] never closed
            x[b, 0] = 1; x[b, 3] = 4; x[b, T // 2] = 3; x[b, T - 1] = 5
    return torch.as_tensor(x, dtype=torch.int64)


if __name__ == "__main__":
    out = {}
    for name, (seed, B, T) in {"a": (1, 8, 97), "b": (2, 5, 1000), "c": (3, 4, 1), "d": (4, 3, 300)}.items():
        x = token_rows(seed, B, T) if T > 8 else torch.as_tensor([[1], [3], [5], [7]], dtype=torch.int64)
        if name == "d":   # no [SPAN] / [ES] / [MASKQ] anywhere: the reference takes its teacher-forcing branch
            x = torch.where((x == 3) | (x == 4) | (x == 5), torch.full_like(x, 9), x)
            x[1, 40] = 1
        ins, sid, pre = run_reference(x)
        out[f"{name}_tokens"] = x.numpy(); out[f"{name}_in_span"] = ins.numpy()
        out[f"{name}_span_id"] = sid.numpy(); out[f"{name}_is_prefix"] = pre.numpy()
    np.savez_compressed(os.path.join(HERE, "metadata_from_tokens.npz"), **out)
    print("wrote metadata_from_tokens.npz", {k: v.shape for k, v in out.items() if k.endswith("tokens")})
