"""Hugging Face ``transformers`` integration: ``cce_patch`` makes a causal-LM head compute its loss
with :func:`cut_cross_entropy.linear_cross_entropy` instead of materialising the logits."""

from .patch import cce_patch

__all__ = ["cce_patch"]
