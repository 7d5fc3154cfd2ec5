"""Is a prompt cut into portions the same computation as the prompt whole?

Cutting changes nothing that the model should notice: the same tokens at the
same positions behind the same causal mask. A difference that shows at the
first boundary points at the mask, one that needs several boundaries at the
position arithmetic or at a page's edge. The probe drives the engine's own
trace replay (model, step function, cache manager and kernels), feeds one
prompt whole and then in portions of each given size, and compares the logits
of the last token (python/stride_worker/diagnose/prefill.py:21-107 is the
reference's probe; there the cache is zeroed between runs, here every run is a
request of its own whose pages go back to the pool and are used again).
"""

from __future__ import annotations

import torch

from .equivalence import Agreement, compare_logits


def seeded_prompt(vocab: int, count: int, seed: int) -> list:
    """Pseudo-token prompt: ids in [1, min(vocab, 30000)) from a seeded generator
    (python/stride_worker/diagnose/cli.py:36-41)."""
    high = max(2, min(vocab, 30000))
    return torch.randint(1, high, (count,), generator=torch.Generator().manual_seed(seed)).tolist()


class PrefillProbe:
    """Runs prompts through a ``TraceSession`` whole or in portions."""

    def __init__(self, session):
        self.session = session
        self._runs = 0
        self._step = 0

    def run_prompt(self, tokens, chunk_size: int | None = None, capture: bool = False):
        """Feeds ``tokens`` in portions of ``chunk_size`` (None: in one step) and
        returns (logits of the last token [1, vocab], hidden states captured in the
        last step or [])."""
        n = len(tokens)
        if n == 0:
            raise ValueError("nothing to prefill")
        if chunk_size is not None and chunk_size <= 0:
            raise ValueError("chunk_size must be positive")
        rid = f"probe-{self._runs}"
        self._runs += 1
        size = chunk_size or n
        model = self.session.model
        logits, states = None, []
        for at in range(0, n, size):
            part = list(tokens[at:at + size])
            last = at + len(part) >= n
            step = {"step": self._step, "entries": [{"id": rid, "tokens": part, "want": [len(part) - 1] if last else []}],
                    "end": [rid] if last else []}
            self._step += 1
            capturing = capture and last
            if capturing:                       # hidden states are collected by an eager step, never inside a captured graph
                graphs, self.session.runner.cuda_graphs = self.session.runner.cuda_graphs, False
                model.capture = []
            try:
                out = self.session.run_step(step)
            finally:
                if capturing:
                    states, model.capture = [s.cpu() for s in (model.capture or [])], None
                    self.session.runner.cuda_graphs = graphs
            if last:
                logits = out
        return logits, states

    def check(self, tokens, chunk_size: int) -> Agreement:
        whole, _ = self.run_prompt(tokens)
        cut, _ = self.run_prompt(tokens, chunk_size)
        return compare_logits(cut, whole)

    def sweep(self, tokens, chunk_sizes) -> dict:
        """chunk size -> Agreement of the cut run with the whole one."""
        whole, _ = self.run_prompt(tokens)
        return {size: compare_logits(self.run_prompt(tokens, size)[0], whole) for size in chunk_sizes}
