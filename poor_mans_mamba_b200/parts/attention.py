"""Grouped-query attention over the paged key/value cache.

a_in = x * in_multiplier; Q, K, V projections (one stacked matrix); K * key_multiplier
before the position encoding; keys and values are written to the request's pages; every
token attends causally to keys lo..pos of its own request; o_proj; the out multiplier is
``out_scale`` (reference src/ops/cpu_backend.cpp:48-202, src/runtime/runner/
falconh1_runner.cpp:66-101).  Softmax scale is 1/sqrt(head_dim).  ``window`` > 0 limits
every token to the last ``window`` keys (and lets the cache manager give older pages back).
"""
from __future__ import annotations

import math
import os
from typing import Any, Dict, List, Optional

import torch

from ..kernels import ops as K
from .base import Mixer, ParamSpec, PartSpec, StateSpec, build_part, register_mixer

Tensor = torch.Tensor

# Key splits are sized so that a step launches about this many attention blocks.
_TARGET_BLOCKS = 592
_TC_BLOCKS = 148        # blocks the tcgen05 prompt kernel is planned for (one per SM)
_TC_FROM_TOKENS = 256   # shorter steps stay on the mma.sync kernel (few 128-row tiles)
_TC_ATTENTION = os.environ.get("PMM_TCGEN05_ATTENTION", "1") == "1"


class PagedAttention(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 position_encoding: Optional[Dict[str, Any]] = None, in_multiplier: float = 1.0,
                 out_multiplier: float = 1.0, key_multiplier: float = 1.0, window: int = 0,
                 shared_kv: bool = False):
        if num_heads % num_kv_heads:
            raise ValueError("query heads must be a multiple of key/value heads")
        K.check_head_dim(head_dim)
        self.hidden_size = int(hidden_size)
        self.num_heads, self.num_kv_heads, self.head_dim = int(num_heads), int(num_kv_heads), int(head_dim)
        self.q_dim = self.num_heads * self.head_dim
        self.kv_dim = self.num_kv_heads * self.head_dim
        self.in_multiplier = float(in_multiplier)
        self.key_multiplier = float(key_multiplier)
        self.out_scale = float(out_multiplier)
        self.window = int(window)
        # shared_kv: this layer projects queries only and reads the keys and values that the
        # layer owning its cache has written (the execution order pairs them up)
        self.shared_kv = bool(shared_kv)
        pe = position_encoding or {"kind": "none"}
        pe_params = {k: v for k, v in pe.items() if k != "kind"}
        self.position_encoding = build_part("position_encoding", PartSpec(pe["kind"], "", pe_params),
                                            head_dim=self.head_dim)
        self.w_in: Optional[Tensor] = None
        self.w_out: Optional[Tensor] = None

    # -- tensors and state
    def param_specs(self) -> List[ParamSpec]:
        d = self.hidden_size
        if self.shared_kv:
            return [ParamSpec("q_proj.weight", (self.q_dim, d)), ParamSpec("o_proj.weight", (d, self.q_dim))]
        return [ParamSpec("q_proj.weight", (self.q_dim, d)), ParamSpec("k_proj.weight", (self.kv_dim, d)),
                ParamSpec("v_proj.weight", (self.kv_dim, d)), ParamSpec("o_proj.weight", (d, self.q_dim))]

    def state_specs(self) -> List[StateSpec]:
        if self.shared_kv:
            return []
        return [StateSpec.paged("kv", planes=2, width=self.kv_dim, window=self.window)]

    def bind(self, params: Dict[str, Tensor]) -> None:
        if self.shared_kv:
            self.w_in = params["q_proj.weight"].contiguous()
        else:
            self.w_in = torch.cat([params["q_proj.weight"], params["k_proj.weight"], params["v_proj.weight"]],
                                  dim=0).contiguous()
        self.w_out = params["o_proj.weight"].contiguous()

    def finalize(self, dtype: torch.dtype, device: torch.device) -> None:
        self.position_encoding.finalize(dtype, device)
        # tickets of the key splits (zero between steps): the last block of a tile merges them
        self._split_counter = torch.zeros(4096, dtype=torch.int32, device=device) if device.type == "cuda" else None
        if self._split_counter is not None:
            K.watch_split_counter(self._split_counter)  # cleared if a launch is ever abandoned half-way

    # -- shared input projection
    def input_rows(self) -> int:
        return self.q_dim if self.shared_kv else self.q_dim + 2 * self.kv_dim

    def input_weight(self) -> Tensor:
        return self.w_in

    def adopt_input_weight(self, view: Tensor) -> None:
        self.w_in = view

    # -- the step
    def forward(self, x: Tensor, ctx, cache, out: Tensor) -> None:
        proj = ctx.workspace.alloc((x.shape[0], self.input_rows()), x.dtype)
        K.linear(x, self.w_in, proj)
        self.forward_projected(proj, ctx, cache, out)

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        K.linear(self.pre_output(proj, ctx, cache), self.w_out, out)

    def output_weight(self) -> Tensor:
        return self.w_out

    def pre_output(self, proj: Tensor, ctx, cache) -> Tensor:
        T = proj.shape[0]
        ws = ctx.workspace
        kv = cache.paged(f"{self.name}.kv")
        q = proj[:, :self.q_dim]
        s_in = self.in_multiplier
        pe = self.position_encoding
        fused = hasattr(pe, "inv_freq")  # rotary (or none): one kernel with the page write
        inv_freq = pe.inv_freq if fused else None
        scale = 1.0 / math.sqrt(float(self.head_dim))
        counter = getattr(self, "_split_counter", None)
        if (fused and ctx.decode_only and proj.dtype == torch.bfloat16 and counter is not None
                and K.flash_decode_supported(self.num_heads, self.num_kv_heads, self.head_dim)):
            n_splits, split_len = self.plan_splits(ctx.new_lens, ctx.kv_len_bound, proj.dtype)
            if n_splits <= 64 and counter.numel() >= T * self.num_kv_heads:
                # decode step: rotation, page write and attention in one launch
                scratch = None
                if n_splits > 1:
                    scratch = ws.alloc((K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits),),
                                       torch.float32)
                attn = ws.alloc((T, self.q_dim), proj.dtype)
                k = None if self.shared_kv else proj[:, self.q_dim:self.q_dim + self.kv_dim]
                v = None if self.shared_kv else proj[:, self.q_dim + self.kv_dim:]
                K.flash_decode_attention(q, k, v, s_in, s_in * self.key_multiplier, s_in, inv_freq, kv.pool,
                                         kv.block_table, ctx.positions, attn, self.num_heads, self.num_kv_heads,
                                         self.head_dim, scale, window=self.window, n_splits=n_splits,
                                         split_len=split_len, scratch=scratch, split_counter=counter)
                return attn
        q_rot = ws.alloc((T, self.q_dim), proj.dtype)
        if self.shared_kv:  # queries only; keys and values are the cache owner's
            K.qkv_rope_store(q, None, None, s_in, 0.0, 0.0, inv_freq, ctx.positions, ctx.seq_of, None, None,
                             q_rot, None, None, self.num_heads, 0, self.head_dim)
            if not fused:
                pe.apply(q_rot.view(T, self.num_heads, self.head_dim), None, ctx.positions)
        else:
            k = proj[:, self.q_dim:self.q_dim + self.kv_dim]
            v = proj[:, self.q_dim + self.kv_dim:]
            if fused:
                K.qkv_rope_store(q, k, v, s_in, s_in * self.key_multiplier, s_in, inv_freq, ctx.positions,
                                 ctx.seq_of, kv.block_table, kv.pool, q_rot, None, None, self.num_heads,
                                 self.num_kv_heads, self.head_dim)
            else:  # a position encoding defined elsewhere: scale, let it act, then store
                k_lin = ws.alloc((T, self.kv_dim), proj.dtype)
                v_lin = ws.alloc((T, self.kv_dim), proj.dtype)
                K.qkv_rope_store(q, k, v, s_in, s_in * self.key_multiplier, s_in, None, ctx.positions,
                                 ctx.seq_of, None, None, q_rot, k_lin, v_lin, self.num_heads,
                                 self.num_kv_heads, self.head_dim)
                pe.apply(q_rot.view(T, self.num_heads, self.head_dim),
                         k_lin.view(T, self.num_kv_heads, self.head_dim), ctx.positions)
                K.kv_store(k_lin, v_lin, ctx.positions, ctx.seq_of, kv.block_table, kv.pool)

        attn = ws.alloc((T, self.q_dim), proj.dtype)
        if (_TC_ATTENTION and proj.dtype == torch.bfloat16 and not ctx.decode_only and counter is not None
                and sum(ctx.new_lens) >= _TC_FROM_TOKENS
                and K.attention_tc_supported(self.num_heads, self.num_kv_heads, self.head_dim, kv.pool.shape[2])):
            # prompt portions: scores and P V on the fifth-generation tensor cores
            n_splits, split_len = self.plan_splits_tc(ctx.new_lens, ctx.kv_len_bound)
            per_tile = 128 // (self.num_heads // self.num_kv_heads)
            tiles = sum((n + per_tile - 1) // per_tile for n in ctx.new_lens)
            if n_splits <= 64 and counter.numel() >= tiles * self.num_kv_heads:
                scratch = None
                if n_splits > 1:
                    scratch = ws.alloc((K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits),),
                                       torch.float32)
                K.attention_tc(q_rot, kv.pool, kv.block_table, ctx.positions, ctx.cu_seqlens, ctx.new_lens, attn,
                               self.num_heads, self.num_kv_heads, self.head_dim, scale, window=self.window,
                               n_splits=n_splits, split_len=split_len, scratch=scratch, split_counter=counter)
                return attn
        n_splits, split_len = self.plan_splits(ctx.new_lens, ctx.kv_len_bound, proj.dtype)
        scratch = None
        if n_splits > 1:
            scratch = ws.alloc((K.attention_scratch_floats(T, self.num_heads, self.head_dim, n_splits),),
                               torch.float32)
        K.paged_attention(q_rot, kv.pool, kv.block_table, ctx.positions, ctx.seq_of, attn, self.num_heads,
                          self.num_kv_heads, self.head_dim, scale,
                          window=self.window, n_splits=n_splits, split_len=split_len, scratch=scratch,
                          cu_seqlens=ctx.cu_seqlens, new_lens=ctx.new_lens,
                          split_counter=counter)
        return attn

    def accepts_length_bounds(self, dtype: torch.dtype, page_size: int) -> bool:
        # the tcgen05 kernel finds its tile's sequence from the lengths on the device, and a block
        # beyond the last tile leaves; rotation and the page write go token by token
        return (_TC_ATTENTION and dtype == torch.bfloat16 and hasattr(self.position_encoding, "inv_freq")
                and getattr(self, "_split_counter", None) is not None
                and K.attention_tc_supported(self.num_heads, self.num_kv_heads, self.head_dim, page_size))

    def plan_splits_tc(self, new_lens, kv_len_bound: int):
        """Key ranges for the tcgen05 kernel (128 rows a block, two blocks an SM): one range when
        the row tiles alone give a block per SM, else enough ranges of at least 256 keys to get there."""
        per_tile = 128 // (self.num_heads // self.num_kv_heads)
        blocks = sum((n + per_tile - 1) // per_tile for n in new_lens) * self.num_kv_heads
        reach = min(kv_len_bound, self.window) if self.window > 0 else kv_len_bound
        want = min(_TC_BLOCKS // max(blocks, 1), (reach + 255) // 256)
        if want <= 1:
            return 1, 0
        split_len = ((kv_len_bound + want - 1) // want + 63) // 64 * 64
        n_splits = (kv_len_bound + split_len - 1) // split_len
        return (n_splits, split_len) if n_splits > 1 else (1, 0)

    def plan_splits(self, new_lens, kv_len_bound: int, dtype: torch.dtype):
        """How many key ranges every block's keys are cut into: enough blocks to fill the GPU
        when few tokens are in flight, one when the tokens alone do."""
        group = self.num_heads // self.num_kv_heads
        if dtype == torch.bfloat16 and K.flash_supported(self.num_heads, self.num_kv_heads, self.head_dim):
            rows = K.flash_tile_rows(self.num_heads, self.num_kv_heads, self.head_dim, new_lens)
            per_tile = rows // group
            blocks = sum((n + per_tile - 1) // per_tile for n in new_lens) * self.num_kv_heads
            min_len = 256 if rows == 16 else 64
            # about two blocks per SM: few warps per block, and causal tiles differ in length; a decode
            # block of head size 128 fills an SM's shared memory alone, so one block per SM there
            # (8 requests, 2 KV heads, 4,096 keys: 9 ranges 13.7 us, 17 ranges 21.3 us)
            target = _TARGET_BLOCKS // 4 if rows == 16 and self.head_dim > 64 else _TARGET_BLOCKS // 2
        else:
            blocks = sum(new_lens) * ((self.num_heads + 3) // 4)
            min_len = 128
            target = _TARGET_BLOCKS
        reach = min(kv_len_bound, self.window) if self.window > 0 else kv_len_bound
        if blocks >= target or reach <= min_len:
            return 1, 0
        if dtype == torch.bfloat16 and min_len == 256:
            # decode blocks all take the same time: as many as run at once and no more, or a second,
            # partly filled wave follows (at batch 64: 2 ranges 35 us, 3 ranges 48 us)
            want = min(max(1, target // blocks), (reach + min_len - 1) // min_len)
        else:
            want = min((target + blocks - 1) // blocks, (reach + min_len - 1) // min_len)
        if want <= 1:
            return 1, 0
        split_len = ((kv_len_bound + want - 1) // want + 63) // 64 * 64
        n_splits = (kv_len_bound + split_len - 1) // split_len
        return (n_splits, split_len) if n_splits > 1 else (1, 0)


register_mixer("paged_attention", PagedAttention)
