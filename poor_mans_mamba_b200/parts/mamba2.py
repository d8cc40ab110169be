"""Mamba2 (SSD) mixer with a per-request conv window and state.

u = x * in_multiplier; Pj = u W_in^T (+ in_proj.bias); columns [z:I][x:I][B:GN][C:GN][dt:H]
times the five chunk multipliers; causal depthwise conv + SiLU over [x,B,C]; the selective
state recurrence; gate (and optional grouped RMSNorm, before or after the gate); out_proj
(+ bias); the out multiplier is ``out_scale`` (reference src/ops/cpu_backend.cpp:306-492,
src/runtime/runner/falconh1_runner.cpp:50-64).

The scalar multipliers and the projection bias are folded into per-channel affine maps
that the conv, scan and gate kernels apply while reading the projection, so the
projection output is never split or rescaled in memory.

Per-request state (fixed size, float32): ``conv`` [K-1, conv_dim] (time-major, the last
K-1 conv inputs) and ``ssm`` [H, P, N].
"""
from __future__ import annotations

import os
import sys
from typing import Dict, List, Optional, Sequence

import torch

from ..kernels import ops as K
from . import branches
from .base import Mixer, ParamSpec, StateSpec, register_mixer

Tensor = torch.Tensor

# Steps whose longest portion has at least this many tokens use the chunked scan.
_CHUNKED_FROM = 8
# The chunked scan on the tcgen05 tensor cores (PMM_TCGEN05_SCAN=0: the mma.sync form, for the
# seven size pairs it is compiled for).
_TC_SCAN = os.environ.get("PMM_TCGEN05_SCAN", "1") == "1"
_NOTED = set()
def _note_serial(d_head: int, d_state: int) -> None:
    """Says once that prompts of this shape are scanned token by token."""
    if (d_head, d_state) not in _NOTED:
        _NOTED.add((d_head, d_state))
        print(f"[poor_mans_mamba_b200] note: the tensor-core scan takes head sizes that are multiples of 16 up to 128 "
              f"and state sizes that are multiples of 16 up to 256; with d_head={d_head}, d_state={d_state} prompt "
              f"portions run the token-serial scan", file=sys.stderr)


class Mamba2Mixer(Mixer):
    def __init__(self, hidden_size: int, n_heads: int, d_head: int, d_state: int, d_conv: int,
                 n_groups: int, chunk_size: int = 128, conv_bias: bool = True, proj_bias: bool = False,
                 gated_norm: bool = False, norm_before_gate: bool = False, norm_eps: float = 1e-5,
                 in_multiplier: float = 1.0, out_multiplier: float = 1.0,
                 chunk_multipliers: Sequence[float] = (1.0, 1.0, 1.0, 1.0, 1.0)):
        if n_heads % n_groups:
            raise ValueError("n_heads must be divisible by n_groups")
        if d_conv < 2:
            raise ValueError("d_conv must be at least 2")
        if d_state > 256:
            raise ValueError(f"the scan kernels take d_state up to 256, got {d_state}")
        if len(chunk_multipliers) != 5:
            raise ValueError("chunk_multipliers must have length 5 [z, x, B, C, dt]")
        self.hidden_size = int(hidden_size)
        self.n_heads, self.d_head, self.d_state = int(n_heads), int(d_head), int(d_state)
        self.d_conv, self.n_groups, self.chunk_size = int(d_conv), int(n_groups), int(chunk_size)
        self.d_ssm = self.n_heads * self.d_head
        self.conv_dim = self.d_ssm + 2 * self.n_groups * self.d_state
        self.proj_dim = self.d_ssm + self.conv_dim + self.n_heads
        self.conv_bias, self.proj_bias = bool(conv_bias), bool(proj_bias)
        self.gated_norm, self.norm_before_gate = bool(gated_norm), bool(norm_before_gate)
        self.norm_eps = float(norm_eps)
        self.in_multiplier = float(in_multiplier)
        self.out_scale = float(out_multiplier)
        self.chunk_multipliers = tuple(float(m) for m in chunk_multipliers)
        self.w_in: Optional[Tensor] = None

    # -- tensors and state
    def param_specs(self) -> List[ParamSpec]:
        h, c, k = self.n_heads, self.conv_dim, self.d_conv
        specs = [
            ParamSpec("in_proj.weight", (self.proj_dim, self.hidden_size)),
            ParamSpec("conv1d.weight", (c, k), kind="vector", alt_shapes=((c, 1, k),), stored_shape=(c, 1, k)),
            ParamSpec("A_log", (h,), kind="vector", init=("log_uniform", 1.0, 16.0)),
            ParamSpec("D", (h,), kind="vector", init=("ones",)),
            ParamSpec("dt_bias", (h,), kind="vector", init=("inv_softplus_log_uniform", 1e-3, 0.1)),
            ParamSpec("out_proj.weight", (self.hidden_size, self.d_ssm)),
        ]
        if self.conv_bias:
            specs.append(ParamSpec("conv1d.bias", (c,), kind="vector"))
        if self.proj_bias:
            specs.append(ParamSpec("in_proj.bias", (self.proj_dim,), kind="vector"))
            specs.append(ParamSpec("out_proj.bias", (self.hidden_size,), kind="vector"))
        if self.gated_norm:
            specs.append(ParamSpec("norm.weight", (self.d_ssm,), kind="vector", init=("ones",)))
        return specs

    def ignored_names(self) -> List[str]:
        """Tensors a checkpoint may carry for switched-off options; present or not, unused."""
        names = []
        if not self.conv_bias:
            names.append("conv1d.bias")
        if not self.gated_norm:
            names.append("norm.weight")
        return names

    def state_specs(self) -> List[StateSpec]:
        return [StateSpec.fixed("conv", (self.d_conv - 1, self.conv_dim), "float32"),
                StateSpec.fixed("ssm", (self.n_heads, self.d_head, self.d_state), "float32")]

    def bind(self, params: Dict[str, Tensor]) -> None:
        self.w_in = params["in_proj.weight"].contiguous()
        self.w_out = params["out_proj.weight"].contiguous()
        self.conv_w = params["conv1d.weight"].reshape(self.conv_dim, self.d_conv).contiguous()
        self.conv_w_t = self.conv_w.t().contiguous()  # tap-major copy for the vector kernel
        self.conv_b = params["conv1d.bias"].contiguous() if self.conv_bias else None
        self.a_log = params["A_log"].contiguous()
        self.d_skip = params["D"].contiguous()
        self.norm_w = params["norm.weight"].contiguous() if self.gated_norm else None
        self.out_b = params["out_proj.bias"].contiguous() if self.proj_bias else None
        in_b = params["in_proj.bias"] if self.proj_bias else None
        dt_bias = params["dt_bias"]

        mz, mx, mb, mc, mdt = self.chunk_multipliers
        s_in = self.in_multiplier
        i_dim, gn = self.d_ssm, self.n_groups * self.d_state
        seg = torch.cat([torch.full((i_dim,), mx), torch.full((gn,), mb), torch.full((gn,), mc)])
        seg = seg.to(device=dt_bias.device, dtype=torch.float32)
        self.conv_pre_scale = (seg * s_in).contiguous()
        self.z_scale = s_in * mz
        self.dt_scale = s_in * mdt
        if in_b is not None:
            self.conv_pre_bias = (in_b[i_dim:i_dim + self.conv_dim] * seg).contiguous()
            self.z_bias = (in_b[:i_dim] * mz).contiguous()
            self.dt_shift = (in_b[i_dim + self.conv_dim:] * mdt + dt_bias).contiguous()
        else:
            self.conv_pre_bias = None
            self.z_bias = None
            self.dt_shift = dt_bias.contiguous()

    # -- shared input projection
    def input_rows(self) -> int:
        return self.proj_dim

    def input_weight(self) -> Tensor:
        return self.w_in

    def adopt_input_weight(self, view: Tensor) -> None:
        self.w_in = view

    # -- the step
    def forward(self, x: Tensor, ctx, cache, out: Tensor) -> None:
        proj = ctx.workspace.alloc((x.shape[0], self.proj_dim), x.dtype)
        K.linear(x, self.w_in, proj)
        self.forward_projected(proj, ctx, cache, out)

    def forward_projected(self, proj: Tensor, ctx, cache, out: Tensor) -> None:
        K.linear(self.pre_output(proj, ctx, cache), self.w_out, out)
        if self.out_b is not None:
            K.add_row_bias_(out, self.out_b)

    def output_weight(self) -> Tensor:
        return self.w_out

    def output_bias(self) -> Optional[Tensor]:
        return self.out_b

    def accepts_length_bounds(self, dtype: torch.dtype, page_size: int) -> bool:
        # the tcgen05 scan's blocks find their chunk's sequence from the lengths on the device and
        # leave when there is none; the convolution and the lone tokens' scan go by token or sequence
        return _TC_SCAN and dtype == torch.bfloat16 and K.ssd_tc_supported(self.d_head, self.d_state)

    def pre_output(self, proj: Tensor, ctx, cache) -> Tensor:
        T = proj.shape[0]
        ws = ctx.workspace
        i_dim = self.d_ssm
        z = proj[:, :i_dim]
        xbc_raw = proj[:, i_dim:i_dim + self.conv_dim]
        dt = proj[:, i_dim + self.conv_dim:]
        window = cache.fixed(f"{self.name}.conv")
        state = cache.fixed(f"{self.name}.ssm")

        xbc = ws.alloc((T, self.conv_dim), proj.dtype)
        window_updating = None
        if ctx.decode_only:
            K.conv1d_decode(xbc_raw, self.conv_pre_scale, self.conv_pre_bias, self.conv_w, self.conv_b,
                            window, ctx.slots, xbc)
        else:
            K.conv1d_fwd(xbc_raw, self.conv_pre_scale, self.conv_pre_bias, self.conv_w, self.conv_b, window,
                         ctx.seq_of, ctx.cu_seqlens, ctx.slots, xbc, weight_t=self.conv_w_t)
            # The window is next read by the next step: its update leaves the scan's chain (a branch
            # of its own in a captured step, joined before this mixer returns).
            here = torch.cuda.current_stream(xbc.device)
            update = branches.branch_stream(xbc.device, "window")
            with branches.fork(here, update):
                K.conv1d_window_update(xbc_raw, self.conv_pre_scale, self.conv_pre_bias, window, ctx.cu_seqlens,
                                       ctx.slots, ctx.n_seq, self.d_conv)
            window_updating = (here, update)

        y = ws.alloc((T, i_dim), proj.dtype)
        # without a norm the gate y * silu(z) is the scan kernels' epilogue
        gate = (z, self.z_scale, self.z_bias) if self.norm_w is None else None
        chunked = not ctx.decode_only and proj.dtype == torch.bfloat16 and max(ctx.new_lens) >= _CHUNKED_FROM
        if chunked and _TC_SCAN and K.ssd_tc_supported(self.d_head, self.d_state):
            # prompt portions: chunks of 128 tokens on the tcgen05 tensor cores
            need = K.ssd_tc_scratch_floats(ctx.new_lens, self.n_heads, self.d_head, self.d_state)
            scratch = ws.alloc((need,), torch.float32)
            # in a mixed step the lone tokens (decoding requests) go through the token-serial kernel: a
            # 128-token chunk for one token is two tile-sized blocks of work for nothing
            lone = ctx.n_seq > 1 and any(n == 1 for n in ctx.new_lens)
            if lone:
                # The two scans touch different sequences (their states, their rows of y).  The lone
                # tokens' scan is a read and write of their states at the memory's rate, the chunked one
                # a chain of three tensor-core launches: they run side by side (parallel branches of a
                # captured step).
                side = branches.branch_stream(xbc.device, "lone")
                with branches.fork(here, side):
                    K.ssm_scan_seq(xbc, dt, self.dt_scale, self.dt_shift, self.a_log, self.d_skip, state,
                                   ctx.cu_seqlens, ctx.slots, ctx.n_seq, y, self.n_groups, gate=gate, only_single=True)
            K.ssm_scan_tc(xbc, dt, self.dt_scale, self.dt_shift, self.a_log, self.d_skip, state, ctx.cu_seqlens,
                          ctx.slots, ctx.new_lens, y, self.n_groups, scratch, gate=gate, skip_single=lone)
            if lone:
                here.wait_stream(side)
        elif chunked and K.ssd_supported(self.d_head, self.d_state):
            # the mma.sync form: chunks of 64 tokens
            need = K.ssd_scratch_floats(ctx.new_lens, self.n_heads, self.d_head, self.d_state, self.n_groups)
            scratch = ws.alloc((need,), torch.float32)
            K.ssm_scan_chunked(xbc, dt, self.dt_scale, self.dt_shift, self.a_log, self.d_skip, state,
                               ctx.cu_seqlens, ctx.slots, ctx.new_lens, y, self.n_groups, scratch, gate=gate)
        else:
            if chunked:
                _note_serial(self.d_head, self.d_state)
            K.ssm_scan_seq(xbc, dt, self.dt_scale, self.dt_shift, self.a_log, self.d_skip, state,
                           ctx.cu_seqlens, ctx.slots, ctx.n_seq, y, self.n_groups, gate=gate,
                           one_token=ctx.decode_only)
        if window_updating is not None:
            window_updating[0].wait_stream(window_updating[1])
        if gate is not None:
            return y
        gated = ws.alloc((T, i_dim), proj.dtype)
        K.gated_norm(y, z, self.z_scale, self.z_bias, self.norm_w, self.norm_eps, self.n_groups,
                     self.norm_before_gate, gated)
        return gated


register_mixer("mamba2", Mamba2Mixer)
