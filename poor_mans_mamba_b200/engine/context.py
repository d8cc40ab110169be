"""What a step hands to the parts: the flattened batch on the device and scratch memory."""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

import torch

from .workspace import Workspace

Tensor = torch.Tensor


class LengthBounds(list):
    """Stands for the tokens per sequence of a step that is recorded once and replayed for every cut
    of the same rounded shape: ``count`` sequences with ``total`` tokens, written as one long
    sequence and count - 1 sequences of one token.  Of all ways to cut ``total`` tokens into
    ``count`` sequences this one needs the most chunks (or tiles) of any size c: sum ceil(n_i / c)
    <= floor((total - count) / c) + count, reached here.  ``multi`` bounds the number of sequences
    of more than one token.  The true lengths are in ``cu_seqlens`` on the device and some of them
    may be zero (a cut with empty sequences needs no more blocks than one without: the bound
    floor((total - k) / c) + k does not fall as k grows); only parts that say
    `accepts_length_bounds` are ever given this."""

    def __init__(self, total: int, count: int):
        if count < 2 or total < count:
            raise ValueError("length bounds need at least two sequences and a token for each")
        super().__init__([total - (count - 1)] + [1] * (count - 1))
        self.multi = count


@dataclass
class StepContext:
    """One step's batch.  All index tensors are int32 on the device.

    tokens[T], positions[T] (absolute position of each token in its request), seq_of[T]
    (index of the token's sequence within the step), cu_seqlens[n_seq+1] (token offsets of
    the sequences), slots[n_seq] (fixed-state slot of each sequence), logit_rows[n_rows]
    (token rows whose logits are wanted).  ``decode_only``: every sequence brings exactly one
    token.  ``kv_len_bound``: an upper bound of position+1 over the step (host value, for
    launch decisions only).  ``new_lens`` / ``past_lens``: host copies per sequence (``new_lens``
    may be a LengthBounds instead, for models all of whose parts accept that).
    ``fetch_ahead``: while a layer runs, the matrices of the layer after it (set by the model;
    a layer that streams its weights once may ask the memory system for them early).
    ``unjoined_stream``: a side stream on which a layer left work running that nothing has waited
    for yet (a fetch-ahead beside its products); the model joins it before a layer that would not
    (`joins_side_stream`) and at the end of the step.
    """
    n_tokens: int
    n_seq: int
    tokens: Tensor
    positions: Tensor
    seq_of: Tensor
    cu_seqlens: Tensor
    slots: Tensor
    logit_rows: Tensor
    n_rows: int
    decode_only: bool
    kv_len_bound: int
    dtype: torch.dtype
    workspace: Workspace
    new_lens: List[int] = field(default_factory=list)
    past_lens: List[int] = field(default_factory=list)
    fetch_ahead: Optional[List[Tensor]] = None
    unjoined_stream: Optional["torch.cuda.Stream"] = None
