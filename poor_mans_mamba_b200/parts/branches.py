"""Side streams for work that runs beside a layer's main chain of launches.

A layer forks a branch (the branch waits for what the main stream has issued so far), issues
launches on it and joins it again; in a step that is being recorded into a CUDA graph the
branch becomes a parallel path of the graph.  One stream per (device, purpose), made on first
use.  `on` switches the current stream without torch's stream context manager, whose
enter and exit cost the host 7 us a pair where two `set_stream` calls cost 1 (measured; a
36-layer prompt step forks three branches a layer).
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

_STREAMS: Dict[Tuple[torch.device, str], "torch.cuda.Stream"] = {}


def branch_stream(device: torch.device, purpose: str) -> "torch.cuda.Stream":
    key = (torch.device(device), purpose)
    st = _STREAMS.get(key)
    if st is None:
        st = torch.cuda.Stream(device=device)
        _STREAMS[key] = st
    return st


class on:
    """``with on(branch, back_to=main):`` launches issued inside go to ``branch``."""

    __slots__ = ("stream", "back_to")

    def __init__(self, stream: "torch.cuda.Stream", back_to: "torch.cuda.Stream"):
        self.stream, self.back_to = stream, back_to

    def __enter__(self) -> "torch.cuda.Stream":
        torch.cuda.set_stream(self.stream)
        return self.stream

    def __exit__(self, *exc) -> None:
        torch.cuda.set_stream(self.back_to)


def fork(main: "torch.cuda.Stream", branch: "torch.cuda.Stream") -> on:
    """The branch waits for everything issued on ``main`` so far; returns the context that issues on it."""
    branch.wait_stream(main)
    return on(branch, main)
