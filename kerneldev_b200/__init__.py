"""kerneldev_b200: KernelDev's hierarchical-mask flash attention as hand-written sm_100a CUDA.

Public surface (mirrors the reference's ``original_kernel`` module for the attention path):
  flash_attention, generate_hadamard_signs, hadamard_transform  -- the operator
  AttentionPlan, get_plan                                       -- tile classification of a batch
"""
from .original_kernel import flash_attention, generate_hadamard_signs, hadamard_transform
from .plan import AttentionPlan, clear_plan_cache, get_plan

__all__ = ["flash_attention", "generate_hadamard_signs", "hadamard_transform", "AttentionPlan",
           "get_plan", "clear_plan_cache"]
