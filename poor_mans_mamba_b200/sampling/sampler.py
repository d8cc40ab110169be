"""Choosing the next token from logits on the device.

Greedy: the largest logit, the first index on ties (the reference's host loop,
src/runtime/worker.cpp:30-59).  Temperature: a draw from softmax(logits / T) by the
Gumbel-max rule with a counter-based generator keyed by (request seed, number of tokens
the request has generated), so a request's draws do not depend on batching, on preemption
or on how its prompt was cut.  Only the chosen ids come back to the host.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch

from ..kernels import ops as K


class Sampler:
    def __init__(self, device):
        self.device = torch.device(device)
        self._out: Optional[torch.Tensor] = None
        self._host: Optional[torch.Tensor] = None
        if self.device.type == "cuda":
            K.ensure_sample_scratch(self.device)

    def _buffers(self, n: int):
        if self._out is None or self._out.numel() < n:
            cap = max(64, n)
            self._out = torch.empty(cap, dtype=torch.int32, device=self.device)
            self._host = torch.empty(cap, dtype=torch.int32, pin_memory=self.device.type == "cuda")
        return self._out[:n], self._host[:n]

    def sample_device(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
                      seeds: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> torch.Tensor:
        """Token ids [n] int32 on the device (a buffer that the next call overwrites)."""
        n = logits.shape[0]
        out, _ = self._buffers(n)
        if temperatures is None or all(t <= 0 for t in temperatures):
            K.sample_rows(logits, None, None, None, out)
        else:
            temp = torch.tensor(list(temperatures), dtype=torch.float32).to(self.device, non_blocking=True)
            sd = torch.tensor([int(s) for s in seeds], dtype=torch.int64).to(self.device, non_blocking=True)
            st = torch.tensor([int(s) for s in steps], dtype=torch.int32).to(self.device, non_blocking=True)
            K.sample_rows(logits, temp, sd, st, out)
        return out

    def to_host(self, ids: torch.Tensor) -> List[int]:
        """Device token ids -> python ints through a pinned buffer (waits for the step)."""
        n = ids.numel()
        _, host = self._buffers(n)
        self._fetch(host, ids)
        return host.tolist()

    def _fetch(self, host: torch.Tensor, ids: torch.Tensor) -> None:
        """Blocking copy of the ids; the kernels' status words travel with them and a step in
        which a bounded wait gave up raises here instead of handing out its tokens."""
        K.status_snapshot(self.device)
        host.copy_(ids, non_blocking=False)
        K.check_status(self.device)

    def sample(self, logits: torch.Tensor, temperatures: Optional[Sequence[float]] = None,
               seeds: Optional[Sequence[int]] = None, steps: Optional[Sequence[int]] = None) -> List[int]:
        n = logits.shape[0]
        if n == 0:
            return []
        out = self.sample_device(logits, temperatures, seeds, steps)
        _, host = self._buffers(n)
        self._fetch(host, out)
        return host.tolist()
