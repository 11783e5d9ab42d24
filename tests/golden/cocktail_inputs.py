"""Seeded inputs of the cocktail-head fixture (shared by make_golden_cocktail.py and the tests)."""
import numpy as np
import torch


def cocktail_rows(seed, B, T, unbalanced=False):
    """Rows with [MASK] and several ([SPAN] .. [ES]) pairs, empty pairs, a row without [MASK]. With
    ``unbalanced``: also a row with an unclosed [SPAN] and a row with an [ES] ahead of its first [SPAN]
    (reversed / overlapping pairs). The fixture uses balanced rows only: when a row's [SPAN] and [ES]
    counts differ the reference selects the [ES] positions with the [SPAN] rows' mask (model.py:284-285),
    which shifts the pairs of the other rows or raises; pairing is per row here."""
    rng = np.random.default_rng(seed)
    x = rng.integers(6, 200, size=(B, T))
    for b in range(B):
        t = int(rng.integers(2, 8))
        if b != 1:
            x[b, t] = 2                       # [MASK]; row 1 has none
            x[b, t + 3] = 2                   # a second one: only the first counts
        t += 6
        n = int(rng.integers(1, 6))
        for j in range(n):
            ln = int(rng.integers(0, 9))      # ln = 0: [SPAN][ES] with nothing between
            if t + ln + 2 >= T:
                break
            x[b, t] = 3; x[b, t + ln + 1] = 4
            t += ln + 2 + int(rng.integers(0, 4))
        if unbalanced and b == 2 and t + 1 < T:
            x[b, t] = 3                       # unclosed [SPAN]
        if unbalanced and b == 3:
            x[b, 0] = 4                       # an [ES] before the first [SPAN]: pairs shift, some reversed
    return torch.as_tensor(x, dtype=torch.int64)


def embeddings(seed, B, T, D):
    g = torch.Generator().manual_seed(seed)
    return torch.randn((B, T, D), generator=g, dtype=torch.float32)


CASES = {"a": (11, 6, 96, 32), "b": (12, 4, 300, 64)}
