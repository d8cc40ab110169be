"""The step function: one batch of (request, its next tokens) through the model.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere.  It
runs only the tokens it is given, as one flattened batch, on top of what earlier steps
left in the cache (keys/values in pages, conv windows and SSM states in slots), and
returns the logits at the wanted places as float32 [n_rows, vocab].  The reference has
no counterpart: its runner takes one whole prompt or one token of one request at a time
(include/runtime/runner/runner.h:13-23).

Host work per step: page bookkeeping, packing all index arrays into one pinned int32
buffer, one host-to-device copy.  Everything else is kernels on the current stream.
"""
from __future__ import annotations

import collections
import os
from dataclasses import dataclass, field
from typing import Dict, Hashable, List, Optional, Sequence, Tuple

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..cache.pages import OutOfPages
from ..kernels import ops as K
from .context import LengthBounds, StepContext
from .model import Model
from .workspace import Workspace, lean_capture

Tensor = torch.Tensor


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places (indices into
    ``tokens``) whose logits are wanted."""
    req: Hashable
    tokens: Sequence[int]
    want: Sequence[int] = field(default_factory=list)


# Prompt steps whose shape (token counts per request, wanted rows, key-length bucket) comes a second
# time are recorded into a CUDA graph and replayed from then on.  Two caches, so that a stream of
# short steps of ever new shapes cannot push out the shapes of chunked prefill: steps of at least
# _STEP_GRAPH_MIN_TOKENS tokens (their workspaces are large: at most _STEP_GRAPH_CAPACITY of them and
# _STEP_GRAPH_BYTES of workspace are kept), and shorter ones down to _STEP_GRAPH_SMALL_FROM tokens (a
# short prompt costs the host 10 ms of launches when it is not replayed, 36 layers of the 0.5B sizes).
_STEP_GRAPH_MIN_TOKENS = 256
_STEP_GRAPH_CAPACITY = 32
_STEP_GRAPH_BYTES = 8 << 30
_STEP_GRAPH_SMALL_FROM = 2
_STEP_GRAPH_SMALL_CAPACITY = 24
# Steps are recorded under a rounded shape (see ModelRunner._rounded_shape) where the model's
# parts allow it, so that a server's ever-changing cuts share recordings: a 36-layer prompt step costs
# the host 10 ms when issued launch by launch and the device 5.  PMM_ROUNDED_STEP_GRAPHS=0: exact
# shapes only.
_ROUNDED_STEP_GRAPHS = os.environ.get("PMM_ROUNDED_STEP_GRAPHS", "1") == "1"
_ROUND_TOKENS = 64


class _Staging:
    """A few pinned int32 host buffers used in rotation for the per-step index upload."""

    def __init__(self, device: torch.device, n_buffers: int = 3):
        self.device = device
        self.pinned = device.type == "cuda"
        self._host: List[Optional[Tensor]] = [None] * n_buffers
        self._events: List[Optional[torch.cuda.Event]] = [None] * n_buffers
        self._dev: Optional[Tensor] = None
        self._i = 0

    def upload(self, n: int, fill, dev: Optional[Tensor] = None) -> Tensor:
        """Calls fill(numpy int32 array of n) and returns the device copy (in ``dev`` if given)."""
        i = self._i
        self._i = (i + 1) % len(self._host)
        if self._host[i] is None or self._host[i].numel() < n:
            cap = max(1024, 1 << (n - 1).bit_length())
            self._host[i] = torch.empty(cap, dtype=torch.int32, pin_memory=self.pinned)
        elif self._events[i] is not None:
            self._events[i].synchronize()  # the copy that last read this buffer has finished
        if dev is None:
            if self._dev is None or self._dev.numel() < n:
                cap = max(1024, 1 << (n - 1).bit_length())
                self._dev = torch.empty(cap, dtype=torch.int32, device=self.device)
            dev = self._dev[:n]
        else:
            dev = dev[:n]
        host = self._host[i]
        fill(host.numpy()[:n])
        dev.copy_(host[:n], non_blocking=True)
        if self.pinned:
            ev = torch.cuda.Event()
            ev.record()
            self._events[i] = ev
        return dev


class ModelRunner:
    """Owns the cache manager and the per-request lengths; ``step`` is the step function."""

    def __init__(self, model: Model, cache: CacheManager):
        self.model = model
        self.cache = cache
        self.device = cache.device
        self.dtype = cache.dtype
        self.workspace = Workspace(self.device)
        self._staging = _Staging(self.device)
        self.steps_run = 0
        self.tokens_run = 0
        self.h2d_bytes = 0
        self.graphs = None
        self._sampler = None
        self._step_graphs: "collections.OrderedDict" = collections.OrderedDict()
        self._small_step_graphs: "collections.OrderedDict" = collections.OrderedDict()
        self._shape_seen: Dict[Tuple, int] = {}  # how often a shape without a recording was issued
        self._step_kernels_replayed = 0  # kernels inside the step graphs replayed so far
        self._accepts_bounds: Optional[bool] = None  # asked of the model when the first large step comes
        self._largest_rounded = 0
        self.token_budget: Optional[int] = None  # the scheduler's tokens per step, where there is one (see _rounded_shape)

    def enable_graphs(self, max_seq_len: int, buckets=None) -> None:
        """Serve decode-only steps from CUDA graphs (captured per batch-size bucket on first use).
        ``max_seq_len`` bounds the context of any request that decodes this way."""
        from .decode_graph import GraphDecoder
        self.graphs = GraphDecoder(self, max_seq_len, buckets)

    # ------------------------------------------------------------------ requests
    def start(self, req: Hashable) -> None:
        self.cache.admit(req)

    def finish(self, req: Hashable) -> None:
        self.cache.release(req)
        if self.graphs is not None:
            self.graphs.forget(req)

    def decode_tokens(self, reqs: Sequence[Hashable], tokens: Optional[Sequence[int]],
                      temperatures: Optional[Sequence[float]] = None, seeds: Optional[Sequence[int]] = None,
                      steps: Optional[Sequence[int]] = None) -> Tensor:
        """One decode step (one token per request) including sampling; returns the sampled ids
        [n] int32 on the device.  ``tokens`` None feeds every request the id sampled for it by
        the previous call (same requests, same order)."""
        if self.graphs is not None and all(
                self.cache.lengths[r] + 1 <= self.graphs.max_seq_len for r in reqs):
            out = self.graphs.decode(reqs, tokens, temperatures, seeds, steps)
            if out is not None:
                self.h2d_bytes += self.graphs.h2d_bytes_last
                self.steps_run += 1
                self.tokens_run += len(reqs)
                return out
        if self._sampler is None:
            from ..sampling import Sampler
            self._sampler = Sampler(self.device)
        if tokens is None:
            tokens = self._last_sampled.tolist()
        logits = self.step([StepEntry(r, [int(t)], [0]) for r, t in zip(reqs, tokens)])
        self._last_sampled = self._sampler.sample_device(logits, temperatures, seeds, steps)
        return self._last_sampled

    def _capture_step(self, total: int, fill, context) -> Optional[dict]:
        """Record the forward pass of one step shape into a CUDA graph over buffers of its own; None
        when the device has no memory left for them."""
        try:
            meta = torch.zeros(total, dtype=torch.int32, device=self.device)
            workspace = Workspace(self.device, initial_bytes=self.workspace.high_water + (8 << 20))
        except torch.cuda.OutOfMemoryError:
            return None  # no room for another recording: the caller issues the step launch by launch
        self._staging.upload(total, fill, dev=meta)
        workspace.freeze()
        ctx, tables = context(meta, workspace)
        graph = torch.cuda.CUDAGraph()
        before = K.launch_count
        with lean_capture(graph, self.device):
            logits = self.model.forward(ctx, self.cache.layer_caches(tables))
        return dict(graph=graph, meta=meta, workspace=workspace, logits=logits, kernels=K.launch_count - before)

    @staticmethod
    def _evict_step_graphs(shapes: "collections.OrderedDict", large: bool) -> None:
        """Least recently replayed recordings go when there are too many of them, or (large steps)
        when their workspaces together hold more than _STEP_GRAPH_BYTES; the newest two stay."""
        cap = _STEP_GRAPH_CAPACITY if large else _STEP_GRAPH_SMALL_CAPACITY
        while len(shapes) > 2 and (len(shapes) > cap or (
                large and sum(e["workspace"].capacity() for e in shapes.values()) > _STEP_GRAPH_BYTES)):
            shapes.popitem(last=False)

    def kernels_launched_since(self, launch_count_before: int) -> int:
        """Own kernels launched since ``launch_count_before`` (a value of kernels.ops.launch_count),
        graph replays counted by the kernels they hold."""
        n = K.launch_count - launch_count_before
        return n + self._kernels_replayed() - getattr(self, "_replayed_mark", 0)

    def _kernels_replayed(self) -> int:
        return self._step_kernels_replayed + (self.graphs.kernels_replayed if self.graphs else 0)

    def mark_launches(self) -> int:
        self._replayed_mark = self._kernels_replayed()
        return K.launch_count

    def check_kernels(self, wait: bool = False) -> None:
        """Raises KernelError if a kernel of an earlier step abandoned a bounded wait (its output
        rows are then incomplete).  Without ``wait`` it looks at the status copy that came to the
        host with the last step the host has waited for; with it, it waits for the device first."""
        K.check_status(self.device, wait=wait)

    def length(self, req: Hashable) -> int:
        return self.cache.lengths[req]

    def can_run(self, entries: Sequence[StepEntry]) -> bool:
        """Whether the cache has the pages (and slots) this batch needs."""
        reserved: Dict[Tuple, int] = {k: 0 for k in self.cache.groups}
        new_reqs = 0
        for e in entries:
            known = self.cache.has(e.req)
            new_reqs += 0 if known else 1
            new_len = self.cache.lengths.get(e.req, 0) + len(e.tokens)
            for k, g in self.cache.groups.items():
                reserved[k] += g.pages_to_grow(e.req, new_len) if known else g.blocks_for(new_len)
        return (new_reqs <= self.cache.free_slots
                and all(reserved[k] <= g.pool.n_free for k, g in self.cache.groups.items()))

    # ------------------------------------------------------------------ step shapes
    def _rounded_shape(self, new_lens: List[int], n_rows: int, kv_len: int):
        """For a step that is not decoding only, through a model whose parts accept lengths as
        bounds: (graph key, token counts of the padding sequences, rows, key-length bound) of the
        rounded shape it is replayed with, else None.  Short steps round up to
        _STEP_GRAPH_MIN_TOKENS tokens (the prompt kernels on the tensor cores start there): a step
        of 40 tokens then takes the device 2.3 ms instead of 1.9, against 10 ms of the host when it is
        issued launch by launch because its exact shape is new.

        The step is padded with sequences that belong to no request (tokens 0 from position 0, the
        spare state slot, block tables full of the spare page) up to a power of two of sequences
        (at least one padding sequence, which takes the padding tokens; further ones are empty) and
        a multiple of _ROUND_TOKENS tokens, its wanted rows with
        copies of the first up to the number of sequences (or a power of two above it).  The model
        sees the padded batch with `LengthBounds` in place of the tokens per sequence, so every
        launch has the shape the key gives it and the recording serves every cut of the real
        tokens; the real rows' results are what they are without the padding (rows and sequences do
        not mix)."""
        T, n_seq = sum(new_lens), len(new_lens)
        if T < _STEP_GRAPH_SMALL_FROM or max(new_lens) == 1 or not _ROUNDED_STEP_GRAPHS:
            return None
        if self._accepts_bounds is None:
            self._accepts_bounds = bool(self.model.accepts_length_bounds(self.cache.page_size))
        if not self._accepts_bounds:
            return None
        n_seq_b = 1 << n_seq.bit_length()          # the next power of two above n_seq
        n_pad = n_seq_b - n_seq
        T_b = max(_STEP_GRAPH_MIN_TOKENS, -(-T // _ROUND_TOKENS) * _ROUND_TOKENS)
        # Steps at the scheduler's token budget all round to one size.  The steps that end a burst of
        # prompts have any size: they are rounded four times as coarsely (up to 255 tokens of padding
        # against being issued launch by launch), so that few recordings serve them.  "At the budget":
        # within _ROUND_TOKENS of `token_budget` where the engine has set it, else no smaller than the
        # largest rounded step this runner has seen.
        if self.token_budget is not None:
            full = T + _ROUND_TOKENS >= self.token_budget
        else:
            self._largest_rounded = max(self._largest_rounded, T_b)
            full = T_b >= self._largest_rounded
        if not full:
            T_b = -(-T_b // (4 * _ROUND_TOKENS)) * (4 * _ROUND_TOKENS)
        # The padding tokens all go to the first padding sequence; the others are empty and cost
        # nothing.  (Padding sequences of one token each were measured first: every one is a read and
        # write of the spare slot's state, 2.6 MB a layer at the 1.5B-Deep sizes, and 60 of them made
        # a burst of the serve workload 10 % slower than no recording at all.)
        pad_lens = [T_b - T] + [0] * (n_pad - 1)
        kv_b = max(kv_len, 1 << (pad_lens[0] - 1).bit_length()) if pad_lens[0] > 0 else kv_len
        if kv_b > self.graphs.max_seq_len or T_b < n_seq_b:
            return None
        # wanted rows: none, or as many as sequences (a server wants at most one per sequence), or the
        # next power of two above that
        rows_b = max(n_seq_b, 1 << (n_rows - 1).bit_length()) if n_rows > 0 else 0
        return ("rounded", T_b, n_seq_b, rows_b, kv_b), pad_lens, rows_b, kv_b

    def _choose_form(self, shapes, exact_key, rounded_key):
        """(key, padded, record) for a step: the key it is replayed, recorded or counted under,
        whether it runs in the padded form of its rounded shape, and whether it is recorded now.
        ``shapes`` holds the recordings; `_note_issued` counts the steps issued launch by launch."""
        seen = self._shape_seen
        key, padded = exact_key, False
        if rounded_key is not None and exact_key not in shapes:
            came = seen.get(("came",) + exact_key, 0) + 1
            seen[("came",) + exact_key] = came
            if came < 3:
                key = rounded_key
                padded = key in shapes or seen.get(key, 0) >= 1
        if key is None or key in shapes:
            record = False
        elif key is exact_key:
            record = seen.get(key, 0) >= 1      # issued as it is at least once
        else:
            record = seen.get(key, 0) >= 2      # issued as it is and once more in its padded form
        return key, padded, record

    def _note_issued(self, key, exact_key, padded: bool) -> None:
        if key is None:
            return
        seen = self._shape_seen
        if len(seen) >= 8192:
            seen.clear()
        seen[key] = seen.get(key, 0) + 1
        if not padded and key is not exact_key:
            seen[exact_key] = seen.get(exact_key, 0) + 1  # the exact form has been issued, too

    def _layout(self, seqs, rows: List[int], groups, widths: List[int], kv_len: int, lens_for_parts):
        """One packed int32 upload for a batch of sequences (token ids, tokens already held, state
        slot, request or None for padding): tokens | positions | seq_of | cu | slots | rows | block
        tables.  Returns (number of ints, fill(host array), context(device array, workspace))."""
        cache = self.cache
        n_seq = len(seqs)
        lens = [len(q[0]) for q in seqs]
        T = sum(lens)
        n_rows = len(rows)
        o_tok, o_pos, o_seq = 0, T, 2 * T
        o_cu = 3 * T
        o_slot = o_cu + n_seq + 1
        o_rows = o_slot + n_seq
        o_tab = o_rows + n_rows
        tab_offsets = []
        total = o_tab
        for w in widths:
            tab_offsets.append(total)
            total += n_seq * w

        def fill(buf: np.ndarray) -> None:
            t0 = 0
            buf[o_cu] = 0
            for s, (toks, held, slot, _) in enumerate(seqs):
                n = lens[s]
                buf[o_tok + t0:o_tok + t0 + n] = toks
                buf[o_pos + t0:o_pos + t0 + n] = np.arange(held, held + n, dtype=np.int32)
                buf[o_seq + t0:o_seq + t0 + n] = s
                buf[o_cu + s + 1] = t0 + n
                buf[o_slot + s] = slot
                t0 += n
            buf[o_rows:o_rows + n_rows] = rows
            for g, w, off in zip(groups, widths, tab_offsets):
                tab = buf[off:off + n_seq * w].reshape(n_seq, w)
                tab[:] = g.num_pages  # the spare page: never owned, safe to touch
                for s, q in enumerate(seqs):
                    if q[3] is None:
                        continue
                    row = g.tables[q[3]]
                    arr = np.asarray(row, dtype=np.int32)
                    arr[arr < 0] = g.num_pages
                    tab[s, :len(row)] = arr

        def context(dev: Tensor, workspace: Workspace):
            tables = {g.key: dev[off:off + n_seq * w].view(n_seq, w) for g, w, off in zip(groups, widths, tab_offsets)}
            return StepContext(
                n_tokens=T, n_seq=n_seq,
                tokens=dev[o_tok:o_tok + T], positions=dev[o_pos:o_pos + T], seq_of=dev[o_seq:o_seq + T],
                cu_seqlens=dev[o_cu:o_cu + n_seq + 1], slots=dev[o_slot:o_slot + n_seq],
                logit_rows=dev[o_rows:o_rows + n_rows], n_rows=n_rows,
                decode_only=all(n == 1 for n in lens), kv_len_bound=kv_len,
                dtype=self.dtype, workspace=workspace, new_lens=lens_for_parts,
                past_lens=[q[1] for q in seqs]), tables

        return total, fill, context

    # ------------------------------------------------------------------ the step
    def step(self, entries: Sequence[StepEntry]) -> Tensor:
        """Run one batch; returns logits [n_rows, vocab] float32 in the order of the entries
        and of their ``want`` lists (a buffer that the next step overwrites).  Requests seen
        for the first time are admitted.  Raises OutOfPages before touching anything if the
        cache cannot hold the batch."""
        if not entries:
            raise ValueError("a step needs at least one entry")
        seen = set()
        token_arrays: List[np.ndarray] = []
        vocab = self.model.vocab_size
        for e in entries:
            if e.req in seen:
                raise ValueError(f"request {e.req!r} appears twice in one step")
            seen.add(e.req)
            if len(e.tokens) == 0:
                raise ValueError(f"request {e.req!r} brings no tokens")
            toks = np.asarray(e.tokens)
            if toks.dtype.kind not in "iu" or int(toks.min()) < 0 or int(toks.max()) >= vocab:
                raise ValueError("token id out of range")
            token_arrays.append(toks)
            for w in e.want:
                if not 0 <= int(w) < len(e.tokens):
                    raise ValueError(f"request {e.req!r}: wanted place {w} is outside its tokens")
        if not self.can_run(entries):
            raise OutOfPages("the cache cannot hold this batch")

        cache = self.cache
        for e in entries:
            if not cache.has(e.req):
                self.start(e.req)
            cache.grow(e.req, cache.lengths[e.req] + len(e.tokens))

        new_lens = [len(e.tokens) for e in entries]
        past = [cache.lengths[e.req] for e in entries]
        T = sum(new_lens)
        rows = [t0 + int(w) for e, t0 in zip(entries, np.cumsum([0] + new_lens[:-1]).tolist()) for w in e.want]
        n_rows = len(rows)
        groups = list(cache.groups.values())
        kv_len = max(p + n for p, n in zip(past, new_lens))
        seqs = [(token_arrays[s], past[s], cache.slot(e.req), e.req) for s, e in enumerate(entries)]
        # Steps of a shape that has been seen before are replayed from a CUDA graph (the host
        # issues hundreds of launches per step otherwise).  Such steps use block tables of a
        # fixed width and a key-length bound rounded up to a power of two, so that the launch
        # shapes depend on the key only.
        exact_key = None
        rounded = None
        if self.graphs is not None and kv_len <= self.graphs.max_seq_len and T >= _STEP_GRAPH_SMALL_FROM:
            kv_len = min(self.graphs.max_seq_len, 1 << (kv_len - 1).bit_length())
            widths = [g.blocks_for(self.graphs.max_seq_len) for g in groups]
            exact_key = (tuple(new_lens), n_rows, kv_len)
            rounded = self._rounded_shape(new_lens, n_rows, kv_len)
        else:
            widths = [max(len(g.tables[e.req]) for e in entries) for g in groups]

        # Which form the step takes: "exact" (the batch as it is) or "padded" (its rounded shape), and
        # under which key it is replayed, recorded or counted.  A shape is issued launch by launch
        # the first time and recorded the second time; a rounded shape is first issued once more in
        # its padded form (the recording must find every library product and scratch size already
        # seen) and recorded the third time.  An exact shape that keeps coming (a benchmark's, a
        # fixed chunk size) gets a recording of its own the third time: it saves the padding.
        large = rounded is not None or T >= _STEP_GRAPH_MIN_TOKENS  # rounded shapes have at least that many tokens
        shapes = self._step_graphs if large else self._small_step_graphs
        key, padded, record = self._choose_form(shapes, exact_key, rounded[0] if rounded is not None else None)
        if padded:
            _, pad_lens, rows_b, kv_b = rounded
            spare = cache.spare_slot
            seqs_g = seqs + [(np.zeros(n, dtype=np.int32), 0, spare, None) for n in pad_lens]
            rows_g = rows + rows[:1] * (rows_b - n_rows)
            lens_g = LengthBounds(T + sum(pad_lens), len(seqs_g))
            total, fill, context = self._layout(seqs_g, rows_g, groups, widths, kv_b, lens_g)
        else:
            total, fill, context = self._layout(seqs, rows, groups, widths, kv_len, new_lens)
        entry = shapes.get(key) if key is not None else None
        if record:
            entry = self._capture_step(total, fill, context)
            if entry is not None:
                shapes[key] = entry
                self._evict_step_graphs(shapes, large)
            else:
                for _ in range(len(shapes) // 2):  # make room; this shape may be recorded when it comes again
                    shapes.popitem(last=False)
        if entry is not None:
            shapes.move_to_end(key)
            self._staging.upload(total, fill, dev=entry["meta"])
            entry["graph"].replay()
            self._step_kernels_replayed += entry["kernels"]
            logits = entry["logits"][:n_rows]
        else:
            self._note_issued(key, exact_key, padded)
            dev = self._staging.upload(total, fill)
            self.workspace.reset()
            ctx, block_tables = context(dev, self.workspace)
            logits = self.model.forward(ctx, cache.layer_caches(block_tables))[:n_rows]
        self.h2d_bytes += 4 * total
        K.status_snapshot(self.device)  # read by check_kernels once the host has waited for this step

        for e, n in zip(entries, new_lens):
            cache.advance(e.req, n)
        self.steps_run += 1
        self.tokens_run += T
        return logits
