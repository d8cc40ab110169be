"""The Python entry point: ``Engine`` = model + cache + step function + scheduler + sampler.

    eng = Engine(model_dir, dtype="bfloat16", max_tokens=65536, max_seqs=64)
    outs = eng.generate([[1, 5, 9], [7, 7]], max_new_tokens=16)          # token ids in and out

or, in the manner of the reference's scheduler (submit / poll,
include/runtime/cluster_scheduler.h:111-142): ``rid = eng.submit(ids, params)``,
``eng.step()`` until ``eng.poll(rid).done``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Hashable, List, Optional, Sequence

import torch

from .cache import CacheManager
from .engine.load import load_model
from .engine.runner import ModelRunner, StepEntry
from .engine.scheduler import Request, SamplingParams, Scheduler, StepPlan
from .kernels import ops as K
from .sampling import Sampler


@dataclass
class Response:
    """A snapshot of a request (reference include/runtime/session.h:9-37: tokens, done, status)."""
    tokens: List[int]
    done: bool
    status: str
    preemptions: int = 0


class Engine:
    def __init__(self, model_dir: str, dtype: str = "bfloat16", device: str = "cuda:0",
                 max_tokens: int = 65536, max_seqs: int = 64, page_size: int = 64,
                 max_batched_tokens: int = 2048, max_seq_len: Optional[int] = None, cuda_graphs: bool = True,
                 warm_graphs: bool = False, run_ahead: bool = True):
        """``max_tokens``: capacity of the key/value cache in tokens (whole pages);
        ``max_seqs``: most requests alive at a time (= number of fixed-state slots);
        ``max_batched_tokens``: token budget of one step; ``max_seq_len``: longest context (prompt
        plus generated tokens) of one request, the reference's ``max_seq`` (src/main.cpp:112-129): a
        request that reaches it ends with what it has, status ``max_seq`` (there: KV overflow ->
        done with a partial result, src/runtime/cluster_scheduler.cpp:645-651); None: the whole pool;
        ``cuda_graphs``: capture decode-only steps into CUDA graphs (``warm_graphs``: all
        batch-size buckets at once here, else each at its first use); ``run_ahead``: launch a
        decode step before the previous one's ids have reached the host (see `step`)."""
        if not torch.cuda.is_available():
            raise RuntimeError("poor_mans_mamba_b200 runs on a CUDA device only; there is no CPU path")
        K.ensure_built()
        self.model, self.config = load_model(model_dir, dtype, device)
        self.device = self.model.device
        self.cache = CacheManager(self.model.state_specs(), page_size=page_size,
                                  num_pages=max(1, max_tokens // page_size), num_slots=max_seqs,
                                  dtype=self.model.dtype, device=self.device)
        self.runner = ModelRunner(self.model, self.cache)
        pool_tokens = max(1, max_tokens // page_size) * page_size
        max_seq_len = pool_tokens if max_seq_len is None else min(int(max_seq_len), pool_tokens)
        if max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        self.max_seq_len = max_seq_len
        if cuda_graphs:
            self.runner.enable_graphs(max_seq_len)
            if warm_graphs:
                with torch.cuda.device(self.device):
                    self.runner.graphs.capture_all()
        self.scheduler = Scheduler(self.cache, max_batched_tokens=max_batched_tokens, max_seqs=max_seqs,
                                   max_seq_len=max_seq_len, release=self.runner.finish)
        self.runner.token_budget = max_batched_tokens  # steps of about this size are rounded finely when recorded
        self.sampler = Sampler(self.device)
        self._next_id = 0
        self.run_ahead = run_ahead and cuda_graphs
        self._inflight = None   # (request ids, output slots, id fetch) of a launched decode step
        self._fetch_bufs = [None, None, None]
        self._fetch_turn = 0

    # ------------------------------------------------------------------ submit / step / poll
    def submit(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = params or SamplingParams(eos_id=self.model.spec.eos_token_id)
        vocab = self.model.vocab_size
        for t in prompt:
            if not 0 <= int(t) < vocab:
                raise ValueError("token id out of range")
        rid = self._next_id
        self._next_id += 1
        self.scheduler.add(rid, [int(t) for t in prompt], params)
        return rid

    def step(self) -> StepPlan:
        """Plan and run one step; returns the plan (empty when nothing could run).

        Decode-only steps through the CUDA-graph path run one step ahead of the host: the step
        is launched, its ids start their way to the host, and the call returns; the next call
        plans and launches the following step (fed with the ids still on the device) before it
        waits for the earlier ones.  A stop token is therefore seen one step late (the extra
        token is dropped); `poll` and the end of `generate` wait for everything in flight."""
        plan = self.scheduler.plan()
        if not plan.entries:
            if self._inflight is None:
                return plan
            self._resolve_inflight()
            plan = self.scheduler.plan()
            if not plan.entries:
                return plan
        pure = all(e.count == 1 and e.samples for e in plan.entries)
        ids = [e.req.id for e in plan.entries]
        ahead = (pure and self._inflight is not None and self._inflight[0] == ids and self._graph_decodable(ids))
        if self._inflight is not None and not ahead:
            # everything known first; a request that has just ended leaves the plan
            self._resolve_inflight()
            plan.entries = [e for e in plan.entries if not e.req.finished]
            if not plan.entries:
                return plan
            ids = [e.req.id for e in plan.entries]
        entries = []
        temps, seeds, steps = [], [], []
        for e in plan.entries:
            r = e.req
            n_prompt = len(r.prompt)
            toks = None
            if not ahead:
                if e.start >= n_prompt:
                    toks = r.output[e.start - n_prompt:e.start - n_prompt + e.count]
                else:
                    toks = r.tokens[e.start:e.start + e.count]
            entries.append((r.id, toks, [e.count - 1] if e.samples else []))
            if e.samples:
                temps.append(r.params.temperature)
                seeds.append(r.params.seed)
                steps.append(len(r.output))
        with torch.cuda.device(self.device):
            if pure and self._graph_decodable(ids):
                tokens = None if ahead else [t[0] for _, t, _ in entries]
                dev_ids = self.runner.decode_tokens(ids, tokens, temps, seeds, steps)
                fetch = self._fetch_async(dev_ids)
                slots = self.scheduler.advance(plan)
                if ahead:
                    self._resolve_inflight()  # the earlier step's ids; the GPU is busy with this one
                self._inflight = (ids, slots, fetch)
            elif pure:
                dev_ids = self.runner.decode_tokens(ids, [t[0] for _, t, _ in entries], temps, seeds, steps)
                self.scheduler.complete(plan, self.sampler.to_host(dev_ids))
            else:
                logits = self.runner.step([StepEntry(i, t, w) for i, t, w in entries])
                self.scheduler.complete(plan, self.sampler.sample(logits, temps, seeds, steps))
        return plan

    def _graph_decodable(self, ids) -> bool:
        g = self.runner.graphs
        return (self.run_ahead and g is not None and len(ids) <= g.bucket_sizes[-1]
                and all(self.cache.lengths[i] + 1 <= g.max_seq_len for i in ids))

    def _fetch_async(self, dev_ids: torch.Tensor):
        """Starts the copy of a step's ids into pinned memory; (buffer, count, event)."""
        n = dev_ids.numel()
        i = self._fetch_turn
        self._fetch_turn = (i + 1) % len(self._fetch_bufs)
        if self._fetch_bufs[i] is None or self._fetch_bufs[i].numel() < n:
            self._fetch_bufs[i] = torch.empty(max(n, 64), dtype=torch.int32, pin_memory=True)
        buf = self._fetch_bufs[i]
        buf[:n].copy_(dev_ids, non_blocking=True)
        K.status_snapshot(self.device)  # the kernels' status words come to the host with the ids
        ev = torch.cuda.Event()
        ev.record()
        return buf, n, ev

    def _resolve_inflight(self) -> None:
        if self._inflight is None:
            return
        _, slots, (buf, n, ev) = self._inflight
        self._inflight = None
        ev.synchronize()
        K.check_status(self.device)  # raises if a bounded wait inside a kernel of that step gave up
        self.scheduler.resolve(slots, buf[:n].tolist())

    def poll(self, rid: Hashable) -> Response:
        self._resolve_inflight()
        r = self.scheduler.requests[rid]
        return Response(list(r.output), r.finished, r.status, r.preemptions)

    def has_work(self) -> bool:
        return self.scheduler.has_work() or self._inflight is not None

    # ------------------------------------------------------------------ one-call generation
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0,
                 seed: int = 0, eos_token_id: Optional[int] = None) -> List[List[int]]:
        """Generated token ids for each prompt (the eos token, if hit, is the last one).
        ``eos_token_id`` None: the model's own; -1: never stop early."""
        eos = self.model.spec.eos_token_id if eos_token_id is None else eos_token_id
        ids = [self.submit(p, SamplingParams(max_new_tokens=max_new_tokens, eos_id=eos,
                                             temperature=temperature, seed=seed + i))
               for i, p in enumerate(prompts)]
        while self.has_work():
            self.step()
        return [self.poll(i).tokens for i in ids]
