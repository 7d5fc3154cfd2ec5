"""Writes the golden logits that anchor the plain implementation on the
reference project's own model code.

The reference's ``StrideModel`` (python/stride_worker/model.py) imports and runs
on the CPU in float32 with an in-memory state dict. This script feeds it the
tiny configurations of ``tests/helpers.py`` with seeded weights, one token per
pass through its own paged cache with scattered page ids, so that logits at
every position come back, and stores them as ``<name>.npy`` beside this file.
``tests/test_plain.py`` then checks ``tests/plain_llama.py`` against the files.

Usage (from the repository root, with the reference checkout at hand):

    python tests/golden/make_golden.py /path/to/reference/python
"""

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from helpers import PAGE_SIZE, TINY, seeded_biases, seeded_state, seeded_tokens  # noqa: E402

# "A_bias": configuration A from a checkpoint that has q/k/v projection biases (the reference adds them when the
# tensors are there, python/stride_worker/model.py:159-169)
GOLDEN_SEED = {"A": 11, "B": 22, "C": 33, "A_bias": 44}
GOLDEN_TOKENS = {"A": 40, "B": 90, "C": 37, "A_bias": 40}


def main(reference_python: str) -> None:
    sys.path.insert(0, reference_python)
    from stride_worker.cache import PagedKVCache
    from stride_worker.model import StrideModel
    from stride_worker.protocol import SequenceWork

    for name in GOLDEN_SEED:
        cfg = TINY[name.split("_")[0]]
        state = seeded_state(cfg, GOLDEN_SEED[name])
        if name.endswith("_bias"):
            state.update(seeded_biases(cfg, GOLDEN_SEED[name] + 2))
        tokens = seeded_tokens(GOLDEN_TOKENS[name], cfg["vocab_size"], GOLDEN_SEED[name] + 1)
        model = StrideModel(dict(cfg), state, torch.device("cpu"), torch.float32)
        page = PAGE_SIZE[name.split("_")[0]]
        pages_needed = (len(tokens) + page - 1) // page
        cache = PagedKVCache(model.cache_spec(2 * pages_needed + 3, page))
        blocks = [2 * i + 1 for i in range(pages_needed)][::-1]
        rows = []
        for position, token in enumerate(tokens):
            _, logits, _ = model.forward(
                [SequenceWork(seq=0, tokens=[token], position=position, blocks=blocks, needs_logits=True)],
                cache)
            rows.append(logits[0].numpy())
        out = np.stack(rows).astype(np.float32)
        np.save(os.path.join(HERE, f"tiny_{name}.npy"), out)
        print(f"tiny_{name}: {out.shape}, max |logit| {np.abs(out).max():.4f}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to the reference's python/ folder>")
    main(sys.argv[1])
