"""Diagnostics: deciding whether two runs computed the same thing, and probing
the engine for what should not change its logits (how a prompt is cut)."""

from .equivalence import (COSINE_FLOOR, DECISIVE_DISAGREEMENT_TOLERANCE, DECISIVE_GAP, Agreement, LayerDivergence,
                          compare_logits, first_divergence, report)

__all__ = ["COSINE_FLOOR", "DECISIVE_GAP", "DECISIVE_DISAGREEMENT_TOLERANCE", "Agreement", "LayerDivergence",
           "compare_logits", "first_divergence", "report"]
