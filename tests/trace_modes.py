"""Ways of cutting the same requests into trace steps. Each function returns a
list of steps in the format of bin/trace_run; ``expected_rows`` tells for each
step which (request, position) every row of its logits belongs to."""

from __future__ import annotations

import random


def whole(requests: dict, want_all: bool = True) -> list[dict]:
    """Each request alone, in one step."""
    steps = []
    for i, (rid, tokens) in enumerate(requests.items()):
        want = list(range(len(tokens))) if want_all else [len(tokens) - 1]
        steps.append({"step": i, "entries": [{"id": rid, "tokens": list(tokens), "want": want}], "end": [rid]})
    return steps


def tail_one_by_one(requests: dict, tail: int = 32) -> list[dict]:
    """Most of a request in one step, the last ``tail`` tokens one by one."""
    steps = []
    for rid, tokens in requests.items():
        head = max(1, len(tokens) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(tokens[:head]), "want": [head - 1]}], "end": []})
        for p in range(head, len(tokens)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [tokens[p]], "want": [0]}],
                          "end": [rid] if p == len(tokens) - 1 else []})
        if head == len(tokens):
            steps[-1]["end"] = [rid]
    return steps


def changing_portions(requests: dict, sizes=(2, 3, 5, 8, 13, 2, 21, 4)) -> list[dict]:
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    for rid, tokens in requests.items():
        at, k = 0, 0
        while at < len(tokens):
            n = min(sizes[k % len(sizes)], len(tokens) - at)
            k += 1
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": list(tokens[at:at + n]),
                                                            "want": sorted({0, n - 1})}],
                          "end": [rid] if at + n == len(tokens) else []})
            at += n
    return steps


def mixed(requests: dict, live_limit: int = 4, seed: int = 0, decode_tail: int = 6, skip_chance: float = 0.2) -> list[dict]:
    """Up to ``live_limit`` requests live at a time: portions of some beside single
    (decoded) tokens of others; a request may sit out a step; finished requests
    end at once, so their pages are given back and used again."""
    rng = random.Random(seed)
    cursor = {rid: 0 for rid in requests}
    pending, live, steps = list(requests), [], []
    while pending or live:
        while pending and len(live) < live_limit:
            live.append(pending.pop(0))
        entries, ends = [], []
        for rid in list(live):
            tokens = requests[rid]
            left = len(tokens) - cursor[rid]
            if len(live) > 1 and rng.random() < skip_chance and entries:
                continue
            n = 1 if left <= decode_tail else min(rng.choice([2, 3, 5, 7, 11, 16, 24]), left - decode_tail)
            entries.append({"id": rid, "tokens": list(tokens[cursor[rid]:cursor[rid] + n]), "want": sorted({0, n - 1})})
            cursor[rid] += n
            if cursor[rid] == len(tokens):
                ends.append(rid)
                live.remove(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ends})
    return steps


def decoding_together(requests: dict, decode_steps: int = 8, prompts_per_step: int = 4) -> list[dict]:
    """Every request live at once: the prompts (all but the last ``decode_steps`` tokens of each) go in a few at a
    time, then all requests bring one token a step for ``decode_steps`` steps, so that the decode-only steps have as
    many rows as there are requests."""
    steps, ids = [], list(requests)
    for at in range(0, len(ids), prompts_per_step):
        entries = []
        for rid in ids[at:at + prompts_per_step]:
            head = max(1, len(requests[rid]) - decode_steps)
            entries.append({"id": rid, "tokens": list(requests[rid][:head]), "want": [head - 1]})
        steps.append({"step": len(steps), "entries": entries, "end": []})
    for k in range(decode_steps, 0, -1):
        entries = [{"id": rid, "tokens": [t[len(t) - k]], "want": [0]} for rid, t in requests.items() if len(t) - k >= 1]
        steps.append({"step": len(steps), "entries": entries, "end": []})
    steps[-1]["end"] = ids
    return steps


def restrict_wants(steps: list[dict], keep: dict) -> list[dict]:
    """The same steps with logits wanted only at the positions ``keep[request]`` (a set): wide vocabularies make
    every row expensive to hold and to compare."""
    held: dict = {}
    for s in steps:
        for e in s["entries"]:
            base = held.get(e["id"], 0)
            e["want"] = [w for w in e["want"] if base + w in keep[e["id"]]]
            held[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            held.pop(rid, None)
    return steps


def expected_rows(steps: list[dict]) -> dict:
    """step number -> list of (request, position) in the order of the logits rows."""
    held: dict = {}
    out = {}
    for s in steps:
        rows = []
        for e in s["entries"]:
            base = held.get(e["id"], 0)
            rows += [(e["id"], base + w) for w in e["want"]]
            held[e["id"]] = base + len(e["tokens"])
        for rid in s["end"]:
            held.pop(rid, None)
        out[s["step"]] = rows
    return out


def peak_tokens(steps: list[dict], round_to: int = 64) -> int:
    """Most tokens that live requests hold at any time, each rounded up."""
    held: dict = {}
    peak = 0
    for s in steps:
        for e in s["entries"]:
            held[e["id"]] = held.get(e["id"], 0) + len(e["tokens"])
        peak = max(peak, sum(-(-n // round_to) * round_to for n in held.values()))
        for rid in s["end"]:
            held.pop(rid, None)
    return peak
