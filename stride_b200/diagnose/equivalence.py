"""Measures of agreement between two sets of logits (or hidden states) computed
from the same input.

Generated text is no measure: one near-tie that falls the other way changes
every token after it. What is compared is the logits themselves, position by
position, in float64: the worst cosine, the largest absolute difference, how
often the first-ranked token agrees, and, where it does not, how decisive the
reference run was about its choice. The rules and thresholds are those of the
reference's diagnostics (python/stride_worker/diagnose/equivalence.py:40-54 for
the constants, :73-97 for the verdict, :100-149 for the measures, :159-184 for
the first divergent layer); needs no GPU.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

# Lowest cosine at which two logit rows still count as the same computation
# (equivalence.py:40-44). Identical input must score above its floor, which is
# why the comparison runs in float64.
COSINE_FLOOR = {torch.float32: 0.9999999, torch.bfloat16: 0.9995, torch.float16: 0.9998}
_DEFAULT_FLOOR = 0.999            # a dtype that has no floor of its own (equivalence.py:74)
# A lead of the first over the second logit wider than this is a decision, not a coin flip (equivalence.py:49).
DECISIVE_GAP = 0.05
# Share of positions that may rank another token first at a decisive margin (equivalence.py:54).
DECISIVE_DISAGREEMENT_TOLERANCE = 0.01

_DTYPE_NAMES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def _dtype(dtype) -> torch.dtype:
    return _DTYPE_NAMES[dtype] if isinstance(dtype, str) else dtype


@dataclass(frozen=True)
class Agreement:
    positions: int
    cosine: float                       # worst row
    max_abs_diff: float
    argmax_match_rate: float
    top5_overlap: float
    worst_disagreement_gap: float       # widest reference margin among the positions whose first token differs
    decisive_disagreement_rate: float   # share of all positions that differ at a margin above DECISIVE_GAP
    finite: bool = True

    def verdict(self, dtype=torch.bfloat16) -> tuple[bool, str]:
        """(same computation?, why). Judged on the cosine floor of ``dtype`` and
        on decisive disagreements only: a first-ranked token that differs at a
        near-tie says nothing."""
        floor = COSINE_FLOOR.get(_dtype(dtype), _DEFAULT_FLOOR)
        if not self.finite:
            return False, "non-finite values in the compared logits"
        if self.cosine < floor:
            return False, f"cosine {self.cosine:.9f} lies below the floor {floor} for {dtype}: a different function, not rounding"
        if self.decisive_disagreement_rate > DECISIVE_DISAGREEMENT_TOLERANCE:
            return False, (f"{self.decisive_disagreement_rate:.1%} of the positions rank another token first although the "
                           f"reference leads by more than {DECISIVE_GAP}")
        return True, (f"equivalent: cosine {self.cosine:.9f}, first token agrees at {self.argmax_match_rate:.1%} of the "
                      f"positions, widest margin among the rest {self.worst_disagreement_gap:.4f}")


def compare_logits(candidate: torch.Tensor, reference: torch.Tensor) -> Agreement:
    """Compares two [positions, vocab] (or [vocab]) tensors; margins are taken
    from ``reference``."""
    if candidate.shape != reference.shape:
        raise ValueError(f"shapes differ: {tuple(candidate.shape)} and {tuple(reference.shape)}")
    c = candidate.detach().to("cpu", torch.float64).reshape(-1, candidate.shape[-1])
    r = reference.detach().to("cpu", torch.float64).reshape(-1, reference.shape[-1])
    n, vocab = r.shape
    finite = bool(torch.isfinite(c).all() and torch.isfinite(r).all())
    cosine = float(torch.nn.functional.cosine_similarity(c, r, dim=-1).min()) if n else 1.0
    max_abs = float((c - r).abs().max()) if n else 0.0
    differs = c.argmax(-1) != r.argmax(-1)
    k = min(5, vocab)
    top_c, top_r = c.topk(k, dim=-1).indices, r.topk(k, dim=-1).indices
    shared = (top_c.unsqueeze(-1) == top_r.unsqueeze(-2)).any(-1).sum(-1).to(torch.float64) / k
    worst_gap = decisive = 0.0
    if vocab >= 2 and bool(differs.any()):
        lead = r.topk(2, dim=-1).values
        margins = (lead[:, 0] - lead[:, 1])[differs]
        worst_gap = float(margins.max())
        decisive = float((margins > DECISIVE_GAP).sum()) / n
    return Agreement(positions=n, cosine=cosine, max_abs_diff=max_abs,
                     argmax_match_rate=float((~differs).to(torch.float64).mean()) if n else 1.0,
                     top5_overlap=float(shared.mean()) if n else 1.0, worst_disagreement_gap=worst_gap,
                     decisive_disagreement_rate=decisive, finite=finite)


@dataclass(frozen=True)
class LayerDivergence:
    layer: int
    cosine: float
    max_abs_diff: float


def first_divergence(candidate: list, reference: list, cosine_floor: float = 0.9999):
    """The first layer at which two captured runs (lists of [tokens, width]
    hidden states, one per layer run) stop agreeing, or None. Errors compound
    through a decoder, so the first layer below the floor is the one to read,
    not the last."""
    if len(candidate) != len(reference):
        raise ValueError(f"{len(candidate)} captured layers against {len(reference)}")
    for index, (x, y) in enumerate(zip(candidate, reference)):
        if x.shape != y.shape:
            return LayerDivergence(index, 0.0, float("inf"))
        a = x.detach().to("cpu", torch.float64).reshape(-1, x.shape[-1])
        b = y.detach().to("cpu", torch.float64).reshape(-1, y.shape[-1])
        cosine = float(torch.nn.functional.cosine_similarity(a, b, dim=-1).min())
        if not cosine >= cosine_floor:          # also catches NaN
            return LayerDivergence(index, cosine, float((a - b).abs().max()))
    return None


def report(name: str, agreement: Agreement, dtype) -> str:
    """One line for the verdict and one for the measures it rests on, e.g.

        chunk=16 [same] cosine 0.999999999 over 1 row | largest difference 1.2e-07 | first token agrees 100.0%, top-5 shared 100.0%
          differing rows: widest reference margin 0.0000, decisive 0.0% | equivalent: ...
    """
    same, why = agreement.verdict(dtype)
    a = agreement
    rows = "row" if a.positions == 1 else "rows"
    head = (f"{name} [{'same' if same else 'DIFFERENT'}] cosine {a.cosine:.9f} over {a.positions} {rows} | "
            f"largest difference {a.max_abs_diff:.1e} | first token agrees {a.argmax_match_rate:.1%}, "
            f"top-5 shared {a.top5_overlap:.1%}")
    tail = (f"  differing rows: widest reference margin {a.worst_disagreement_gap:.4f}, "
            f"decisive {a.decisive_disagreement_rate:.1%} | {why}")
    return head + "\n" + tail
