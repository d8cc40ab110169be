"""Decode steps as CUDA graphs.

A decode step (every sequence brings one token) is some hundreds of small kernels; issued
one by one the step is bound by launch latency, not by memory.  For each batch-size bucket
the whole step (embedding to sampled token id) is captured once into a CUDA graph over
buffers at fixed addresses; afterwards a step is one small host-to-device copy of the
step's indices, one graph launch and, if the caller wants the ids on the host, one
device-to-host copy.

Per bucket of b sequences the index buffer (int32) holds
  tokens[b] | positions[b] | slots[b] | temperature[b] (float bits) | steps[b] | seeds[2b] (int64) | block tables
and the constants seq_of = cu_seqlens = logit_rows = 0..b never change.  Rows beyond the
live sequences point at the spare slot and the spare page that no request owns.  The
split of the keys in attention is planned for a bound on the context: the smallest power of
two (from 1,024 on, capped at the longest context the engine allows) that holds every live
request, so a graph is captured per (batch-size bucket, context bucket) and short contexts do
not pay for empty key ranges.
"""
from __future__ import annotations

from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..kernels import ops as K
from .context import StepContext
from .workspace import Workspace, quiet_capture

Tensor = torch.Tensor


class _Bucket:
    def __init__(self, b: int, widths: List[int], device: torch.device):
        self.b = b
        self.widths = widths
        o = 0
        self.o_tok, o = o, o + b
        self.o_pos, o = o, o + b
        self.o_slot, o = o, o + b
        self.o_temp, o = o, o + b
        self.o_step, o = o, o + b
        o = (o + 1) // 2 * 2  # int64 alignment
        self.o_seed, o = o, o + 2 * b
        self.o_tabs = []
        for w in widths:
            self.o_tabs.append(o)
            o += b * w
        self.n_ints = o
        self.dev = torch.zeros(o, dtype=torch.int32, device=device)
        self.host = [torch.zeros(o, dtype=torch.int32, pin_memory=True) for _ in range(3)]
        self.events: List[Optional[torch.cuda.Event]] = [None, None, None]
        self.turn = 0
        self.arange = torch.arange(b + 1, dtype=torch.int32, device=device)
        self.sampled = torch.zeros(b, dtype=torch.int32, device=device)
        self.workspace = Workspace(device)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.kv_bound = 0  # the context bound the captured launches were planned for
        self.logits: Optional[Tensor] = None
        self.kernels_per_replay = 0


class GraphDecoder:
    def __init__(self, runner, max_seq_len: int, buckets: Optional[Sequence[int]] = None):
        self.runner = runner
        self.model = runner.model
        self.cache = runner.cache
        self.device = runner.device
        self.max_seq_len = int(max_seq_len)
        cap = self.cache.num_slots
        if buckets is None:
            buckets = [b for b in (1, 2, 4, 8, 16, 32, 64, 128, 256) if b < cap] + [cap]
        self.bucket_sizes = sorted(set(int(b) for b in buckets if b <= cap))
        self.groups = list(self.cache.groups.values())
        self.widths = [g.blocks_for(self.max_seq_len) for g in self.groups]
        self.buckets: Dict[Tuple[int, int], _Bucket] = {}
        self._last: Optional[_Bucket] = None  # the bucket of the last step: its sampled ids feed the next
        self._rows: Dict[Hashable, Tuple[List[np.ndarray], List[int], int]] = {}  # request -> its block-table rows (host copies)
        self.replays = 0
        self.kernels_replayed = 0
        K.ensure_sample_scratch(self.device, max(self.bucket_sizes))  # before any step is recorded

    # ------------------------------------------------------------------ capture
    _KV_BUCKET_MIN = 1024

    def kv_bucket(self, kv_len: int) -> int:
        """The context bound a step with ``kv_len`` keys in its longest request is planned for."""
        return min(self.max_seq_len, max(self._KV_BUCKET_MIN, 1 << (max(kv_len, 1) - 1).bit_length()))

    def kv_buckets(self) -> List[int]:
        out, b = [], self._KV_BUCKET_MIN
        while b < self.max_seq_len:
            out.append(b)
            b *= 2
        return out + [self.max_seq_len]

    def _context(self, bk: _Bucket) -> Tuple[StepContext, Dict]:
        b, d = bk.b, bk.dev
        tables = {g.key: d[o:o + b * w].view(b, w) for g, w, o in zip(self.groups, bk.widths, bk.o_tabs)}
        ctx = StepContext(
            n_tokens=b, n_seq=b, tokens=d[bk.o_tok:bk.o_tok + b], positions=d[bk.o_pos:bk.o_pos + b],
            seq_of=bk.arange[:b], cu_seqlens=bk.arange, slots=d[bk.o_slot:bk.o_slot + b],
            logit_rows=bk.arange[:b], n_rows=b, decode_only=True, kv_len_bound=bk.kv_bound,
            dtype=self.runner.dtype, workspace=bk.workspace, new_lens=[1] * b, past_lens=[0] * b)
        return ctx, tables

    def _run(self, bk: _Bucket) -> None:
        ctx, tables = self._context(bk)
        bk.workspace.reset()
        logits = self.model.forward(ctx, self.cache.layer_caches(tables))
        d, b = bk.dev, bk.b
        temps = d[bk.o_temp:bk.o_temp + b].view(torch.float32)
        seeds = d[bk.o_seed:bk.o_seed + 2 * b].view(torch.int64)
        steps = d[bk.o_step:bk.o_step + b]
        K.sample_rows(logits, temps, seeds, steps, bk.sampled)
        bk.logits = logits

    def _pad(self, bk: _Bucket, buf: np.ndarray, start: int) -> None:
        b = bk.b
        buf[bk.o_tok + start:bk.o_tok + b] = 0
        buf[bk.o_pos + start:bk.o_pos + b] = 0
        buf[bk.o_slot + start:bk.o_slot + b] = self.cache.spare_slot
        buf[bk.o_temp + start:bk.o_temp + b] = 0
        buf[bk.o_step + start:bk.o_step + b] = 0
        buf[bk.o_seed + 2 * start:bk.o_seed + 2 * b] = 0
        for g, w, o in zip(self.groups, bk.widths, bk.o_tabs):
            buf[o + start * w:o + b * w] = g.num_pages

    def bucket_for(self, n: int, kv_len: Optional[int] = None) -> Optional[_Bucket]:
        """The captured step for ``n`` sequences whose longest context (this step's token included)
        is ``kv_len`` (None: the longest the engine allows)."""
        kv = self.kv_bucket(self.max_seq_len if kv_len is None else kv_len)
        for size in self.bucket_sizes:
            if size >= n:
                if (size, kv) not in self.buckets:
                    self.buckets[(size, kv)] = self._capture(size, kv)
                return self.buckets[(size, kv)]
        return None

    def capture_all(self) -> None:
        """Capture every bucket now, so that no step pays for a capture while serving."""
        for size in self.bucket_sizes:
            for kv in self.kv_buckets():
                if (size, kv) not in self.buckets:
                    self.buckets[(size, kv)] = self._capture(size, kv)

    def _capture(self, b: int, kv_bound: int) -> _Bucket:
        bk = _Bucket(b, self.widths, self.device)
        bk.kv_bound = kv_bound
        host = bk.host[0].numpy()
        self._pad(bk, host, 0)
        bk.dev.copy_(bk.host[0])
        torch.cuda.synchronize(self.device)
        # warm-up on a side stream: sizes the workspace and lets the libraries set themselves up
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self._run(bk)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        bk.workspace.reset()   # merge chunks, then pin the addresses
        bk.workspace.freeze()
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count
        with quiet_capture(graph):
            self._run(bk)
        bk.kernels_per_replay = K.launch_count - before
        bk.graph = graph
        return bk

    # ------------------------------------------------------------------ per request bookkeeping
    def _table_rows(self, req: Hashable) -> List[np.ndarray]:
        entry = self._rows.get(req)
        admission = self.cache.admissions[req]
        if entry is None or entry[2] != admission:  # new, or given back and admitted again since
            entry = ([np.full(w, g.num_pages, dtype=np.int32) for g, w in zip(self.groups, self.widths)],
                     [-1] * len(self.groups), admission)
            self._rows[req] = entry
        rows, seen, _ = entry
        for j, (g, row) in enumerate(zip(self.groups, rows)):
            table = g.tables[req]
            if len(table) != seen[j] or g.window > 0:  # grown (or a window may have passed pages)
                arr = np.asarray(table, dtype=np.int32)
                arr[arr < 0] = g.num_pages
                row[:len(table)] = arr
                seen[j] = len(table)
        return rows

    def forget(self, req: Hashable) -> None:
        self._rows.pop(req, None)

    # ------------------------------------------------------------------ the step
    def decode(self, reqs: Sequence[Hashable], tokens: Optional[Sequence[int]],
               temperatures: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
               steps: Optional[Sequence[int]] = None) -> Optional[Tensor]:
        """One decode step for ``reqs`` (one token each).  ``tokens`` None: each request is fed
        the id sampled for the same row by the previous call (same requests, same order).
        Returns the sampled ids [n] int32 on the device, or None if no bucket fits."""
        n = len(reqs)
        cache = self.cache
        bk = self.bucket_for(n, max(cache.lengths[r] for r in reqs) + 1)
        if bk is None:
            return None
        for r in reqs:
            new_len = cache.lengths[r] + 1
            if new_len > self.max_seq_len:
                raise ValueError(f"request {r!r} would exceed max_seq_len {self.max_seq_len}")
            cache.grow(r, new_len)
        i = bk.turn
        bk.turn = (i + 1) % len(bk.host)
        if bk.events[i] is not None:
            bk.events[i].synchronize()
        buf = bk.host[i].numpy()
        b = bk.b
        if tokens is not None:
            buf[bk.o_tok:bk.o_tok + n] = np.asarray(tokens, dtype=np.int32)
        buf[bk.o_pos:bk.o_pos + n] = [cache.lengths[r] for r in reqs]
        buf[bk.o_slot:bk.o_slot + n] = [cache.slot(r) for r in reqs]
        if temperatures is not None and any(t > 0 for t in temperatures):
            buf[bk.o_temp:bk.o_temp + n] = np.asarray(temperatures, dtype=np.float32).view(np.int32)
            buf[bk.o_step:bk.o_step + n] = np.asarray(steps, dtype=np.int32)
            buf[bk.o_seed:bk.o_seed + 2 * n] = np.asarray(seeds, dtype=np.int64).view(np.int32)
        else:
            buf[bk.o_temp:bk.o_temp + n] = 0
        for s, r in enumerate(reqs):
            rows = self._table_rows(r)
            for w, o, row in zip(bk.widths, bk.o_tabs, rows):
                buf[o + s * w:o + (s + 1) * w] = row
        self._pad(bk, buf, n)
        if tokens is None:  # keep the device-side ids of the last step as this step's tokens
            if self._last is None or self._last.b < n:
                raise ValueError("no earlier step's ids to feed: give the tokens")
            bk.dev[bk.o_tok:bk.o_tok + n].copy_(self._last.sampled[:n])
            bk.dev[bk.o_pos:].copy_(bk.host[i][bk.o_pos:], non_blocking=True)
            self.h2d_bytes_last = 4 * (bk.n_ints - bk.o_pos)
        else:
            bk.dev.copy_(bk.host[i], non_blocking=True)
            self.h2d_bytes_last = 4 * bk.n_ints
        ev = torch.cuda.Event()
        ev.record()
        bk.events[i] = ev
        bk.graph.replay()
        self._last = bk
        self.replays += 1
        self.kernels_replayed += bk.kernels_per_replay
        for r in reqs:
            cache.advance(r, 1)
        return bk.sampled[:n]

    def last_logits(self, n: int) -> Tensor:
        """Logits [n, V] of the last replayed step (its first n rows)."""
        if self._last is None or self._last.b < n:
            raise ValueError("no step of that many sequences has been replayed")
        return self._last.logits[:n]
