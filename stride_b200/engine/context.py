"""The index arrays of one step, as the kernels see them.

All arrays are int32 views of one device buffer that the host fills with a
single copy (layout: ``csrc/runtime/step_batch.hpp``). Arrays are padded to the
capacities of the layout: padded tokens carry ``seq_of_token == -1`` and a slot
of -1, padded sequences ``q_len == 0``.
"""

from __future__ import annotations

from dataclasses import dataclass, field

import torch


@dataclass
class StepContext:
    num_tokens: int                 # rows of the flat batch that the kernels run (padding included)
    num_seqs: int
    num_rows: int                   # logit rows wanted
    token_ids: torch.Tensor         # [token_cap]
    positions: torch.Tensor         # [token_cap] absolute position of each token in its request
    seq_of_token: torch.Tensor      # [token_cap] index of the token's sequence in this step, -1 for padding
    logit_rows: torch.Tensor        # [row_cap] flat-batch rows whose logits are wanted
    q_start: torch.Tensor           # [seq_cap] first flat-batch row of each sequence
    q_len: torch.Tensor             # [seq_cap] tokens of each sequence in this step
    ctx_len: torch.Tensor           # [seq_cap] position + q_len: keys the sequence holds after this step
    state_slot: torch.Tensor        # [seq_cap] per-request state slot
    slot_mapping: list              # per group [token_cap]: page * page_size + offset, -1 for padding
    block_table: list               # per group [seq_cap, table_width]
    max_q_len: int = 0
    max_ctx: int = 0
    decode_only: bool = False
    # Requests are laid out in the order given; the trailing run of single-token
    # requests (decodes) starts at flat row ``decode_tail_start`` and is made of
    # the sequences from ``decode_tail_seq`` on. Kernels specialised for decode
    # take that tail, kernels for portions take what comes before it.
    decode_tail_start: int = 0
    decode_tail_seq: int = 0
    # Upper bound of ctx_len that holds for as long as this context's launches
    # may be replayed (the longest context of the step, or of any step for a
    # captured graph).
    context_bound: int = 0
    # Host copy of the step's items for parts that loop in Python:
    # (request, first flat row, number of tokens, position of the first token, state slot)
    host_items: list = field(default_factory=list)


def make_context(dev: torch.Tensor, layout: dict, num_tokens: int, num_seqs: int, num_rows: int, **host) -> StepContext:
    tc, sc, rc, w = layout["token_cap"], layout["seq_cap"], layout["row_cap"], layout["table_width"]

    def view(name, n):
        return dev[layout[name]: layout[name] + n]

    return StepContext(
        num_tokens=num_tokens, num_seqs=num_seqs, num_rows=num_rows,
        token_ids=view("token_ids", tc), positions=view("positions", tc), seq_of_token=view("seq_of_token", tc),
        logit_rows=view("logit_rows", rc), q_start=view("q_start", sc), q_len=view("q_len", sc),
        ctx_len=view("ctx_len", sc), state_slot=view("state_slot", sc),
        slot_mapping=[dev[o: o + tc] for o in layout["slot_mapping"]],
        block_table=[dev[o: o + sc * w].view(sc, w) for o in layout["block_table"]],
        **host)
