"""Metadata of one RAGGED step: a flat batch in which every live sequence brings any number of new tokens (a prompt
portion) or one (a decode step), each after ``ctx`` tokens it already has in the cache / state.

The reference's per-step metadata (lite_llama/executor/attention_metadata.py:19-44) describes either a padded
prefill rectangle or a one-token-per-sequence decode batch; this is the same information per SEQUENCE instead, so
the two kinds of work share a step.  Everything the kernels read is int32 on the device and arrives in ONE
host-to-device copy.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Sequence

import torch


@dataclass
class RaggedBatch:
    tokens: int                       # total new tokens
    num_seqs: int
    seq_start: torch.Tensor           # [num_seqs + 1] offsets into the flat batch
    seq_ctx: torch.Tensor             # [num_seqs] tokens already cached
    seq_slot: torch.Tensor            # [num_seqs] request slot (row of the request table, recurrent-state slot)
    positions: torch.Tensor           # [tokens] position of every new token
    kv_rows: torch.Tensor             # [tokens] pool row every new token's K/V goes to
    portion_list: torch.Tensor        # sequences that bring more than one token
    single_list: torch.Tensor         # sequences that bring exactly one
    num_portions: int = 0
    num_singles: int = 0
    max_portion: int = 0              # longest portion (host int: sizes the tiled attention grid)
    max_single_ctx: int = 0           # longest context among the single-token sequences (sizes the key split)

    @classmethod
    def build(cls, lens: Sequence[int], ctxs: Sequence[int], slots: Sequence[int], kv_rows: torch.Tensor,
              device: str) -> "RaggedBatch":
        n = len(lens)
        starts = [0]
        for c in lens:
            starts.append(starts[-1] + c)
        total = starts[-1]
        pos: list[int] = []
        for c, ctx in zip(lens, ctxs):
            pos.extend(range(ctx, ctx + c))
        portions = [i for i, c in enumerate(lens) if c > 1]
        singles = [i for i, c in enumerate(lens) if c == 1]
        packed = starts + list(ctxs) + list(slots) + pos + portions + singles
        host = torch.tensor(packed, dtype=torch.int32)
        if device != "cpu":
            host = host.pin_memory() if torch.cuda.is_available() else host
        dev = host.to(device, non_blocking=True)
        cuts = [n + 1, n, n, total, len(portions), len(singles)]
        parts, at = [], 0
        for c in cuts:
            parts.append(dev[at:at + c])
            at += c
        return cls(tokens=total, num_seqs=n, seq_start=parts[0], seq_ctx=parts[1], seq_slot=parts[2],
                   positions=parts[3], kv_rows=kv_rows.to(torch.int32), portion_list=parts[4], single_list=parts[5],
                   num_portions=len(portions), num_singles=len(singles),
                   max_portion=max([lens[i] for i in portions], default=0),
                   max_single_ctx=max([ctxs[i] for i in singles], default=0))
