"""kerneldev_b200: KernelDev's hierarchical-mask flash attention as hand-written sm_100a CUDA.

Public surface (mirrors the reference's ``original_kernel`` module for the attention path):
  flash_attention, generate_hadamard_signs, hadamard_transform  -- the operator
  AttentionPlan, get_plan, clear_plan_cache                     -- tile classification of a batch
  metadata_from_tokens                                          -- in_span / span_id / is_prefix from token ids
  span_index, span_means, cocktail_scores                       -- the span-mean head of model.py:258-296

Names are resolved on first use, so that ``python -m kerneldev_b200.build`` can (re)build the
shared library before anything tries to load it. The first use of the operator loads
libkd_attention.so and fails loudly if it is missing or stale; there is no other compute path.
"""
_EXPORTS = {
    "flash_attention": "original_kernel", "generate_hadamard_signs": "original_kernel",
    "hadamard_transform": "original_kernel", "AttentionPlan": "plan", "get_plan": "plan",
    "clear_plan_cache": "plan", "metadata_from_tokens": "metadata",
    "span_means": "cocktail", "cocktail_scores": "cocktail", "span_index": "cocktail",
}

__all__ = sorted(_EXPORTS)


def __getattr__(name):
    if name in _EXPORTS:
        import importlib
        return getattr(importlib.import_module(f"{__name__}.{_EXPORTS[name]}"), name)
    raise AttributeError(f"module {__name__!r} has no attribute {name!r}")
