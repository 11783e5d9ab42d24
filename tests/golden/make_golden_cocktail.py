"""Golden fixture for the cocktail-party head, produced by the REFERENCE's own code.

    REFERENCE_DIR=/path/to/KernelDev python tests/golden/make_golden_cocktail.py

The block of ``GPTModel.forward`` between "Cocktail party processing" and the einsum (model.py:258-296)
is read from the reference checkout at generation time, dedented and executed on seeded token rows
and embeddings (nothing of it is stored here); inputs are regenerated from the seed by the tests,
the outputs ``scores`` and ``h_spans`` are saved to ``cocktail_head.npz``.
"""
import os
import sys
import textwrap

import numpy as np
import torch

REF = os.environ["REFERENCE_DIR"]   # path of a checkout of the reference project
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REF)
sys.path.insert(0, HERE)
from data_builder import SPECIAL_TOKENS  # noqa: E402  (the reference's table)


def reference_block():
    lines = open(os.path.join(REF, "model.py")).read().splitlines()
    start = next(i for i, l in enumerate(lines) if "Cocktail party processing (span-based reasoning)" in l) + 1
    end = next(i for i, l in enumerate(lines) if "scores = torch.einsum('bd,bnd->bn', h_context, h_spans)" in l) + 1
    body = textwrap.dedent("\n".join(lines[start:end]))
    # the block sits in a method and leaves it early when the batch has no [SPAN]; wrap it in a function
    return "def _block(x, x_embed):\n" + textwrap.indent(body, "    ") + "\n    return scores, h_spans\n"


from cocktail_inputs import CASES, cocktail_rows, embeddings  # noqa: E402  (seeded inputs, shared with the tests)

if __name__ == "__main__":
    ns = {"torch": torch, "SPECIAL_TOKENS": SPECIAL_TOKENS, "mask_token_id": SPECIAL_TOKENS["[MASK]"],
          "span_start_id": SPECIAL_TOKENS["[SPAN]"], "span_end_id": SPECIAL_TOKENS["[ES]"]}
    exec(reference_block(), ns)
    out = {}
    for name, (seed, B, T, D) in CASES.items():
        x, e = cocktail_rows(seed, B, T), embeddings(seed, B, T, D)
        scores, h_spans = ns["_block"](x, e)
        out[f"{name}_scores"] = scores.numpy(); out[f"{name}_h_spans"] = h_spans.numpy()
        out[f"{name}_tokens_sum"] = np.int64(x.sum().item())
    np.savez_compressed(os.path.join(HERE, "cocktail_head.npz"), **out)
    print("wrote cocktail_head.npz", {k: v.shape for k, v in out.items()})
