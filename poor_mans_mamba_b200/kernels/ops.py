"""Python face of the CUDA kernels: argument checks, then one C call per op on the
current CUDA stream.  Nothing here computes on the host and nothing falls back: a tensor
that is not on a CUDA device, a size a kernel cannot take, or a missing library raises.

Matrix products go to the library (cuBLAS through ``torch.mm``), as the reference sends
its linear layers to ``cublasSgemm`` (src/ops/gpu/linear.cu:3-21); in float32 the
reduced-precision matrix mode is switched off for the call.
"""
from __future__ import annotations

import ctypes
import os
import weakref
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from . import build as _build

Tensor = torch.Tensor

PMM_ERR_BAD_ARGUMENT = 1001


class KernelError(RuntimeError):
    """A kernel launch was refused or failed."""


_SIGNATURES = {
    "pmm_embed": [c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_add_rmsnorm": [c_void_p, c_void_p, c_float, c_void_p, c_float, c_void_p, c_float, c_void_p,
                        c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_scale_f32": [c_void_p, c_float, c_longlong, c_void_p],
    "pmm_cast_scale": [c_void_p, c_void_p, c_float, c_longlong, c_int, c_void_p],
    "pmm_conv1d_fwd": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                       c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_conv1d_window_update": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_conv1d_decode": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_ssm_scan_seq": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p,
                         c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                         c_int, c_void_p, c_longlong, c_float, c_void_p, c_int, c_int, c_void_p],
    "pmm_ssd_supported": [c_int, c_int],
    "pmm_ssd_chunked": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_void_p,
                        c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int,
                        c_int, c_int, c_int, c_int, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p],
    "pmm_ssd_tc_supported": [c_int, c_int],
    "pmm_ssd_tc": [c_void_p, c_int, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p,
                   c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                   c_longlong, c_float, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "pmm_gated_norm": [c_void_p, c_void_p, c_longlong, c_float, c_void_p, c_void_p, c_float, c_int,
                       c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_qkv_rope_store": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float,
                           c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p,
                           c_int, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                           c_void_p],
    "pmm_kv_store": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int,
                     c_int, c_int, c_void_p],
    "pmm_paged_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                            c_int, c_int, c_int, c_void_p],
    "pmm_flash_supported": [c_int, c_int, c_int],
    "pmm_flash_paged_attention": [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                  c_int, c_int, c_int, c_int, c_void_p, c_void_p],
    "pmm_l2_prefetch": [c_void_p, c_void_p, c_int, c_void_p],
    "pmm_attention_tc_supported": [c_int, c_int, c_int, c_int],
    "pmm_attention_tc": [c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                         c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                         c_void_p, c_void_p],
    "pmm_skinny_chain": [c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p],
    "pmm_flash_decode_attention": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float,
                                   c_float, c_float, c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p,
                                   c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int,
                                   c_int, c_void_p, c_void_p],
    "pmm_decode_attention_tma_supported": [c_int, c_int, c_int, c_int],
    "pmm_decode_attention_tma": [c_void_p, c_longlong, c_void_p, c_longlong, c_void_p, c_longlong, c_float, c_float,
                                 c_float, c_void_p, c_void_p, c_longlong, c_void_p, c_int, c_void_p, c_void_p, c_void_p,
                                 c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p,
                                 c_void_p, c_void_p],
    "pmm_flash_combine": [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p],
    "pmm_skinny_gemm": [c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_float, c_void_p, c_int,
                        c_float, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong, c_void_p,
                        c_int, c_void_p],
    "pmm_skinny_gemm_f32out": [c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong,
                               c_void_p],
    "pmm_skinny_tc_supported": [c_int, c_int, c_int, c_int, c_int, c_longlong, c_longlong, c_longlong],
    "pmm_skinny_tc": [c_int, c_int, c_int, c_void_p, c_longlong, c_void_p, c_int, c_float, c_void_p, c_longlong,
                      c_void_p, c_int, c_float, c_void_p, c_longlong, c_void_p, c_void_p, c_void_p],
    "pmm_tc_gemm_supported": [c_int, c_int, c_int, c_longlong, c_longlong],
    "pmm_tc_gemm": [c_int, c_void_p, c_longlong, c_void_p, c_void_p, c_longlong, c_int, c_int, c_int, c_float,
                    c_void_p, c_void_p],
    "pmm_silu_mul": [c_void_p, c_longlong, c_float, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_add_row_bias": [c_void_p, c_void_p, c_int, c_int, c_int, c_void_p],
    "pmm_sample_rows": [c_void_p, c_longlong, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                        c_void_p, c_void_p, c_void_p],
}

_FUNCS = {}
launch_count = 0  # kernels of this library launched since import (library GEMMs not counted)


def _fn(name: str):
    f = _FUNCS.get(name)
    if f is None:
        lib = _build.load()
        try:
            f = getattr(lib, name)
        except AttributeError as exc:
            raise KernelError(f"kernel library has no symbol {name}; rebuild it") from exc
        f.argtypes = _SIGNATURES[name]
        f.restype = c_int
        _FUNCS[name] = f
    return f


def _call(name: str, *args) -> None:
    global launch_count
    rc = _fn(name)(*args)
    launch_count += 1
    if rc != 0:
        if rc == PMM_ERR_BAD_ARGUMENT:
            raise KernelError(f"{name}: sizes or arguments outside what the kernel supports")
        raise KernelError(f"{name}: CUDA error {rc} at launch")


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Asked for at every launch: the raw getter takes 0.3 us where
    building a torch.cuda.Stream object takes 3 to 15."""
    if _RAW_STREAM is not None:
        return _RAW_STREAM(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: Tensor) -> int:
    if t.dtype == torch.float32:
        return 0
    if t.dtype == torch.bfloat16:
        return 1
    raise KernelError(f"storage type must be float32 or bfloat16, got {t.dtype}")


def _ptr(t: Optional[Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()



# ----------------------------------------------------------------------------- status of bounded waits
class _StatusWatch:
    """The status words of one device and their host copy.

    Kernels whose threads wait on one another (mbarrier waits of the tcgen05 kernels, the grid
    barrier of skinny_chain) bound every wait; a wait that gives up writes a code into a status
    word, the block abandons its tile and returns, and the output of that launch is incomplete.
    ``words[0]`` is shared by the tensor-core kernels, ``words[1]`` by the chain.  The engine
    copies the words to pinned memory with the results it fetches anyway (`snapshot`) and looks
    at the copy once the host has waited for that fetch (`check`)."""

    def __init__(self, device: torch.device):
        self.device = device
        self.words = torch.zeros(2, dtype=torch.int32, device=device)
        self.host = torch.zeros(2, dtype=torch.int32, pin_memory=True)
        self.counters: "weakref.WeakSet" = weakref.WeakSet()

    def snapshot(self) -> None:
        self.host.copy_(self.words, non_blocking=True)

    def check(self) -> None:
        tc, chain = int(self.host[0]), int(self.host[1])
        if tc == 0 and chain == 0:
            return
        # leave the device usable: clear the words and whatever a half-finished launch left behind
        self.words.zero_()
        self.host.zero_()
        for c in list(self.counters):
            c.zero_()
        raise KernelError(f"a bounded wait inside a kernel gave up on {self.device} (tensor-core kernels: code {tc}; "
                          f"grid-barrier chain: code {chain}): the step's results are incomplete and were discarded")


_WATCHES: Dict[torch.device, _StatusWatch] = {}


def _watch(device: torch.device) -> _StatusWatch:
    device = torch.device(device)
    if device.index is None and device.type == "cuda":
        device = torch.device("cuda", torch.cuda.current_device())
    w = _WATCHES.get(device)
    if w is None:
        w = _StatusWatch(device)
        _WATCHES[device] = w
    return w


def watch_split_counter(counter: Tensor) -> None:
    """Registers an attention split counter (zero between launches) to be cleared when a launch
    was abandoned half-way."""
    _watch(counter.device).counters.add(counter)


def status_snapshot(device) -> None:
    """Enqueue the copy of the device's status words to pinned memory on the current stream."""
    _watch(device).snapshot()


def check_status(device, wait: bool = False) -> None:
    """Raise KernelError if the last snapshot that has reached the host shows an abandoned wait.
    ``wait``: take a snapshot now and wait for the current stream first."""
    w = _watch(device)
    if wait:
        w.snapshot()
        torch.cuda.current_stream(w.device).synchronize()
    w.check()


def _cuda(*tensors: Optional[Tensor]) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise KernelError("kernels run on CUDA tensors only (no CPU path exists)")


def _rows_view(t: Tensor, what: str) -> int:
    """Row stride (elements) of a 2-D view whose rows are contiguous."""
    if not (t.dim() == 2 and t.stride(1) == 1):
        raise KernelError(f"{what}: need a 2-D view with unit column stride")
    return t.stride(0)


def _f32vec(t: Optional[Tensor], n: int, what: str) -> None:
    if t is not None:
        if not (t.dtype == torch.float32 and t.is_contiguous() and t.numel() == n):
            raise KernelError(f"{what}: need a contiguous float32 vector of {n}")


def _i32(t: Tensor, what: str) -> None:
    if not (t.dtype == torch.int32 and t.is_contiguous()):
        raise KernelError(f"{what}: need contiguous int32")


# ----------------------------------------------------------------------------- library GEMM
def padded_rows(n_rows: int) -> int:
    """The row count a library product of ``n_rows`` rows is issued with.  The library chooses a
    kernel per (M, N, K) and the first call with a new M costs about 1.4 ms on the host (measured:
    18 us once the shape is known); a server sees a new token count in almost every step.  Rounded
    up to a multiple of 64 (128 from 1,024 rows, 256 from 4,096) the shapes recur.  The extra rows
    are scratch: the step's arena reserves them behind every matrix it hands out."""
    if n_rows <= 64:
        return n_rows
    step = 64 if n_rows < 1024 else (128 if n_rows < 4096 else 256)
    return (n_rows + step - 1) // step * step


def _with_rows(t: Tensor, rows: int) -> Optional[Tensor]:
    """``t`` [T, n] seen with ``rows`` >= T rows of the same stride, if its storage reaches that far."""
    if t.dim() != 2 or t.stride(1) != 1:
        return None
    last = t.storage_offset() + (rows - 1) * t.stride(0) + t.shape[1]
    if last * t.element_size() > t.untyped_storage().nbytes():
        return None
    return t.as_strided((rows, t.shape[1]), t.stride())


def _mm(x: Tensor, weight: Tensor, out: Tensor, **kw) -> None:
    """The library product; with `padded_rows(T)` rows where ``out`` is a whole matrix of the step's
    arena (which marks it with the rows it keeps behind it) and x's storage reaches as far.  What
    the extra rows of x hold does not matter, rows being independent, and nothing reads the extra
    rows of out."""
    n = x.shape[0]
    if n > 64:
        rows = padded_rows(n)
        if rows != n and getattr(out, "_scratch_rows", 0) >= rows:
            # matrices of the arena carry the padded view with them; a slice of one is widened here
            xp = x._with_scratch_rows if getattr(x, "_scratch_rows", 0) == rows else _with_rows(x, rows)
            op = out._with_scratch_rows if out._scratch_rows == rows else _with_rows(out, rows)
            if xp is not None and op is not None:
                x, out = xp, op
    torch.mm(x, weight.t(), out=out, **kw)


def linear(x: Tensor, weight: Tensor, out: Tensor) -> Tensor:
    """out[T, N] = x[T, K] @ weight[N, K]^T through the GEMM library."""
    _cuda(x, weight, out)
    if not (x.dtype == weight.dtype):
        raise KernelError(f"linear: activation {x.dtype} vs weight {weight.dtype}")
    if x.dtype == torch.float32:
        prev = torch.backends.cuda.matmul.allow_tf32
        torch.backends.cuda.matmul.allow_tf32 = False
        try:
            _mm(x, weight, out)
        finally:
            torch.backends.cuda.matmul.allow_tf32 = prev
    else:
        _mm(x, weight, out)
    return out


_MM_F32_OUT: Optional[bool] = None


def mm_has_f32_out() -> bool:
    """Whether the GEMM library gives a float32 result from bfloat16 operands directly."""
    global _MM_F32_OUT
    if _MM_F32_OUT is None:
        try:
            a = torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda")
            torch.mm(a, a.t(), out_dtype=torch.float32)
            _MM_F32_OUT = True
        except (TypeError, RuntimeError):
            _MM_F32_OUT = False
    return _MM_F32_OUT


def linear_f32_out(x: Tensor, weight: Tensor, out: Tensor, scratch_low: Optional[Tensor], scale: float) -> None:
    """out (float32) = scale * (x @ weight^T) for bfloat16 operands.  The library is asked for
    a float32 result directly; a library build without that option gets a bfloat16 product
    that is widened (and scaled) by cast_scale."""
    _cuda(x, weight, out)
    if mm_has_f32_out():
        _mm(x, weight, out, out_dtype=torch.float32)
        if scale != 1.0:
            scale_f32_(out, scale)
    else:
        if not (scratch_low is not None):
            raise KernelError("linear_f32_out: needs a low-precision scratch buffer")
        torch.mm(x, weight.t(), out=scratch_low)
        cast_scale(out, scratch_low, scale)


# ----------------------------------------------------------------------------- own kernels
def embed(out: Tensor, table: Tensor, tokens: Tensor, mult: float) -> None:
    _cuda(out, table, tokens)
    T, D = out.shape
    if not (out.dtype == torch.float32 and out.is_contiguous()):
        raise KernelError("embed: out must be contiguous float32")
    if not (table.dim() == 2 and table.shape[1] == D and table.is_contiguous()):
        raise KernelError("embed: table must be [V, D]")
    _i32(tokens, "embed: tokens")
    if not (tokens.numel() == T):
        raise KernelError("embed: one token per output row")
    _call("pmm_embed", out.data_ptr(), table.data_ptr(), tokens.data_ptr(), float(mult), T, D,
          table.shape[0], _dt(table), _stream())


def add_rmsnorm(h: Tensor, branches: Sequence[Tuple[Tensor, float]], weight: Optional[Tensor],
                eps: float, out: Optional[Tensor], rows: Optional[Tensor] = None) -> None:
    """h <- (h + s0*b0) + s1*b1 (rows is None), then out = rmsnorm(h) * weight.
    With ``rows`` (int32 row indices) h is left as it is and out[r] comes from row rows[r]."""
    _cuda(h, weight, out, rows)
    if not (h.dtype == torch.float32 and h.dim() == 2 and h.is_contiguous()):
        raise KernelError("add_rmsnorm: the residual stream must be contiguous float32 [T, D]")
    T, D = h.shape
    if not (len(branches) <= 2):
        raise KernelError("add_rmsnorm: at most two branches")
    if not (D * 4 <= 200 * 1024):
        raise KernelError(f"add_rmsnorm: width {D} exceeds one block's shared memory")
    ptrs: List[Optional[int]] = [None, None]
    scales = [0.0, 0.0]
    dtype = None
    for i, (b, s) in enumerate(branches):
        _cuda(b)
        if not (b.shape == h.shape and b.is_contiguous()):
            raise KernelError("add_rmsnorm: branch must be contiguous [T, D]")
        ptrs[i], scales[i] = b.data_ptr(), float(s)
        dtype = _dt(b) if dtype is None else dtype
        if not (_dt(b) == dtype):
            raise KernelError("add_rmsnorm: branches of different storage types")
    R = T
    if rows is not None:
        _i32(rows, "add_rmsnorm: rows")
        R = rows.numel()
    if out is not None:
        if not (weight is not None):
            raise KernelError("add_rmsnorm: a norm needs its weight")
        _f32vec(weight, D, "add_rmsnorm: weight")
        if not (out.shape == (R, D) and out.is_contiguous()):
            raise KernelError("add_rmsnorm: out must be contiguous [rows, D]")
        if not (dtype is None or _dt(out) == dtype):
            raise KernelError("add_rmsnorm: out and branches differ in storage type")
        dtype = _dt(out)
    if dtype is None:
        return  # nothing to add and nothing to write
    _call("pmm_add_rmsnorm", h.data_ptr(), ptrs[0], scales[0], ptrs[1], scales[1], _ptr(weight),
          float(eps), _ptr(out), _ptr(rows), R, D, dtype, _stream())


def scale_f32_(x: Tensor, s: float) -> None:
    _cuda(x)
    if not (x.dtype == torch.float32 and x.is_contiguous()):
        raise KernelError("scale_f32_: contiguous float32 only")
    _call("pmm_scale_f32", x.data_ptr(), float(s), x.numel(), _stream())


def cast_scale(out: Tensor, src: Tensor, s: float) -> None:
    _cuda(out, src)
    if not (out.dtype == torch.float32 and out.is_contiguous() and src.is_contiguous()
            and out.numel() == src.numel()):
        raise KernelError("cast_scale: contiguous tensors of equal size, float32 out")
    _call("pmm_cast_scale", out.data_ptr(), src.data_ptr(), float(s), src.numel(), _dt(src), _stream())


def _conv_common(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], window: Tensor, K: int):
    C = x.shape[1]
    _f32vec(pre_scale, C, "conv1d: pre_scale")
    _f32vec(pre_bias, C, "conv1d: pre_bias")
    if not (window.dtype == torch.float32 and window.is_contiguous() and window.dim() == 3
            and tuple(window.shape[1:]) == (K - 1, C)):
        raise KernelError("conv1d: window must be float32 [slots, K-1, C]")
    return C


def conv1d_fwd(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], weight: Tensor,
               bias: Optional[Tensor], window: Tensor, seq_of: Tensor, cu: Tensor, slots: Tensor,
               out: Tensor, weight_t: Optional[Tensor] = None) -> None:
    """Causal depthwise conv + SiLU over all tokens of the step; reads the windows.
    ``weight_t`` is the tap-major copy [K, C] of ``weight`` [C, K]; with it bfloat16 inputs take
    the vector kernel."""
    _cuda(x, pre_scale, pre_bias, weight, bias, window, seq_of, cu, slots, out, weight_t)
    ld = _rows_view(x, "conv1d: x")
    T = x.shape[0]
    if not (weight.dtype == torch.float32 and weight.dim() == 2 and weight.is_contiguous()
            and weight.shape[0] == x.shape[1]):
        raise KernelError("conv1d: weight must be contiguous float32 [C, K]")
    K = weight.shape[1]
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    _f32vec(bias, C, "conv1d: bias")
    if not (out.shape == (T, C) and out.is_contiguous() and out.dtype == x.dtype):
        raise KernelError("conv1d: out must be [T, C]")
    if not (weight_t is None or (weight_t.dtype == torch.float32 and weight_t.is_contiguous()
            and weight_t.shape == (K, C))):
        raise KernelError("conv1d: weight_t must be contiguous float32 [K, C]")
    _call("pmm_conv1d_fwd", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias), weight.data_ptr(),
          _ptr(weight_t), _ptr(bias), window.data_ptr(), seq_of.data_ptr(), cu.data_ptr(), slots.data_ptr(),
          out.data_ptr(), T, C, K, _dt(x), _stream())


def conv1d_window_update(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], window: Tensor,
                         cu: Tensor, slots: Tensor, n_seq: int, K: int) -> None:
    """Leaves the last K-1 conv inputs of every sequence in its window."""
    _cuda(x, pre_scale, pre_bias, window, cu, slots)
    ld = _rows_view(x, "conv1d: x")
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    _call("pmm_conv1d_window_update", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias),
          window.data_ptr(), cu.data_ptr(), slots.data_ptr(), n_seq, C, K, _dt(x), _stream())


def conv1d_decode(x: Tensor, pre_scale: Tensor, pre_bias: Optional[Tensor], weight: Tensor,
                  bias: Optional[Tensor], window: Tensor, slots: Tensor, out: Tensor) -> None:
    """Conv + SiLU + window shift for a step in which every sequence brings one token."""
    _cuda(x, pre_scale, pre_bias, weight, bias, window, slots, out)
    ld = _rows_view(x, "conv1d: x")
    n_seq = x.shape[0]
    K = weight.shape[1]
    C = _conv_common(x, pre_scale, pre_bias, window, K)
    if not (weight.dtype == torch.float32 and weight.is_contiguous() and weight.shape[0] == C):
        raise KernelError("conv1d: weight must be contiguous float32 [C, K]")
    _f32vec(bias, C, "conv1d: bias")
    if not (out.shape == (n_seq, C) and out.is_contiguous() and out.dtype == x.dtype):
        raise KernelError("conv1d: out must be [T, C]")
    _call("pmm_conv1d_decode", x.data_ptr(), ld, pre_scale.data_ptr(), _ptr(pre_bias),
          weight.data_ptr(), _ptr(bias), window.data_ptr(), slots.data_ptr(), out.data_ptr(), n_seq, C,
          K, _dt(x), _stream())


def _gate_args(gate, out: Tensor, what: str):
    """(z pointer, row stride, scale, bias pointer) of an optional fused gate (z view, scale, bias)."""
    if gate is None:
        return None, 0, 0.0, None
    z, z_scale, z_bias = gate
    _cuda(z, z_bias)
    ld_z = _rows_view(z, f"{what}: z")
    if not (z.shape == out.shape and z.dtype == out.dtype):
        raise KernelError(f"{what}: z must match the output")
    _f32vec(z_bias, out.shape[1], f"{what}: z_bias")
    return z.data_ptr(), ld_z, float(z_scale), _ptr(z_bias)


def ssm_scan_seq(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor,
                 d_skip: Tensor, state: Tensor, cu: Tensor, slots: Tensor, n_seq: int, out: Tensor,
                 n_groups: int, gate=None, one_token: bool = False, only_single: bool = False) -> None:
    """Token-serial Mamba2 recurrence from the saved state; state[slots, H, P, N] is updated.
    ``gate`` = (z view [T, I], z_scale, z_bias or None): the output is y * silu(z*z_scale + z_bias).
    ``one_token``: sequence s brings exactly token s (a decode step); ``cu`` is then not read.
    ``only_single``: only the sequences that bring exactly one token are walked (the lone tokens of
    a mixed step, whose longer portions the chunked scan takes); the others are left alone."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (N <= 256):
        raise KernelError(f"ssm_scan: d_state {N} above 256 is not supported")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N):
        raise KernelError("ssm_scan: xbc must hold [x | B | C]")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype):
        raise KernelError("ssm_scan: out must be [T, H*P]")
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan")
    _call("pmm_ssm_scan_seq", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale),
          dt_shift.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(),
          slots.data_ptr(), out.data_ptr(), n_seq, H, P, N, n_groups, zp, ld_z, zs, zb, 2 if only_single else int(bool(one_token)),
          _dt(xbc), _stream())


SSD_CHUNK = 64  # tokens per chunk of the tensor-core scan


def ssd_supported(d_head: int, d_state: int) -> bool:
    """Whether the chunked tensor-core scan is compiled for this head size / state size."""
    return bool(_fn("pmm_ssd_supported")(d_head, d_state))


def ssd_chunks(new_lens: Sequence[int]) -> int:
    return sum((n + SSD_CHUNK - 1) // SSD_CHUNK for n in new_lens)


def ssd_scratch_floats(new_lens: Sequence[int], n_heads: int, d_head: int, d_state: int,
                       n_groups: Optional[int] = None) -> int:
    """Floats of scratch for the chunked scan: every chunk's local state (float), its decay, its
    start state (bfloat16, on a 16-byte boundary) and the 64 x 64 products C.B of every
    (chunk, group); without ``n_groups`` enough for one group per head."""
    chunks = ssd_chunks(new_lens)
    per_state = chunks * n_heads * d_head * d_state
    decays = (chunks * n_heads + 3) // 4 * 4
    starts = ((per_state + 1) // 2 + 3) // 4 * 4
    return per_state + decays + starts + chunks * (n_groups or n_heads) * 64 * 64


def ssm_scan_chunked(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor,
                     d_skip: Tensor, state: Tensor, cu: Tensor, slots: Tensor, new_lens: Sequence[int],
                     out: Tensor, n_groups: int, scratch: Tensor, gate=None) -> None:
    """The Mamba2 recurrence over prompt portions in chunks of 64 tokens on tensor cores
    (bfloat16 activations); same contract as ssm_scan_seq.  ``scratch``: float32, at least
    ssd_scratch_floats(...) elements."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out, scratch)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (xbc.dtype == torch.bfloat16 and ssd_supported(P, N)):
        raise KernelError(f"ssm_scan_chunked: needs bfloat16 and a compiled (d_head, d_state) pair, got {xbc.dtype} "
                          f"({P}, {N})")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N and ld_x % 8 == 0 and xbc.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan_chunked: xbc must hold [x | B | C] in rows that start on 16-byte boundaries")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype):
        raise KernelError("ssm_scan: out must be [T, H*P]")
    n_chunks = ssd_chunks(new_lens)
    need = ssd_scratch_floats(new_lens, H, P, N, n_groups)
    if not (scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need
            and scratch.data_ptr() % 16 == 0):
        raise KernelError(f"ssm_scan_chunked: needs {need} floats of 16-byte aligned scratch")
    chunk_state = scratch.data_ptr()
    chunk_decay = chunk_state + 4 * n_chunks * H * P * N
    start_state = chunk_decay + 4 * ((n_chunks * H + 3) // 4 * 4)
    chunk_cb = start_state + 4 * (((n_chunks * H * P * N + 1) // 2 + 3) // 4 * 4)
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan_chunked")
    if not (zp is None or (ld_z % 2 == 0 and zp % 4 == 0)):
        raise KernelError("ssm_scan_chunked: z rows must be 4-byte aligned")
    _call("pmm_ssd_chunked", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale),
          dt_shift.data_ptr(), a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(),
          slots.data_ptr(), out.data_ptr(), chunk_state, chunk_decay, start_state, chunk_cb, len(new_lens), n_chunks,
          H, P, N,
          n_groups, zp, ld_z, zs, zb, _stream())


SSD_TC_CHUNK = 128  # tokens per chunk of the tcgen05 scan


def ssd_tc_supported(d_head: int, d_state: int) -> bool:
    """Whether the tcgen05 scan takes this head size / state size (multiples of 16 up to 128 / 256)."""
    return bool(_fn("pmm_ssd_tc_supported")(d_head, d_state))


def ssd_tc_scratch_floats(new_lens: Sequence[int], n_heads: int, d_head: int, d_state: int) -> int:
    """Floats of scratch for the tcgen05 scan: every 128-token chunk's local state (float), its
    decay, delta and cs of its tokens per head, and its start state (bfloat16, on a 16-byte boundary)."""
    chunks = sum((n + SSD_TC_CHUNK - 1) // SSD_TC_CHUNK for n in new_lens)
    per_state = chunks * n_heads * d_head * d_state
    return (per_state + (chunks * n_heads + 3) // 4 * 4 + chunks * n_heads * 2 * SSD_TC_CHUNK
            + ((per_state + 1) // 2 + 3) // 4 * 4)


def ssm_scan_tc(xbc: Tensor, dt_raw: Tensor, dt_scale: float, dt_shift: Tensor, a_log: Tensor, d_skip: Tensor,
                state: Tensor, cu: Tensor, slots: Tensor, new_lens: Sequence[int], out: Tensor, n_groups: int,
                scratch: Tensor, gate=None, skip_single: bool = False) -> None:
    """The Mamba2 recurrence over prompt portions in chunks of 128 tokens on the tcgen05 tensor
    cores (bfloat16 activations); same contract as ssm_scan_seq.  ``scratch``: float32, at least
    ssd_tc_scratch_floats(...) elements.  ``skip_single``: sequences that bring exactly one token are
    left alone (their rows of ``out`` and their states): ssm_scan_seq(only_single=True) takes them."""
    _cuda(xbc, dt_raw, dt_shift, a_log, d_skip, state, cu, slots, out, scratch)
    if not (state.dtype == torch.float32 and state.dim() == 4 and state.is_contiguous()):
        raise KernelError("ssm_scan: state must be contiguous float32 [slots, H, P, N]")
    _, H, P, N = state.shape
    if not (xbc.dtype == torch.bfloat16 and ssd_tc_supported(P, N)):
        raise KernelError(f"ssm_scan_tc: needs bfloat16, a head size that is a multiple of 16 up to 128 and a state size that is a "
                          f"multiple of 16 up to 256, got {xbc.dtype} ({P}, {N})")
    ld_x = _rows_view(xbc, "ssm_scan: xbc")
    if not (xbc.shape[1] == H * P + 2 * n_groups * N and ld_x % 8 == 0 and xbc.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan_tc: xbc must hold [x | B | C] in rows that start on 16-byte boundaries")
    ld_dt = _rows_view(dt_raw, "ssm_scan: dt")
    if not (dt_raw.shape[1] == H and dt_raw.dtype == xbc.dtype):
        raise KernelError("ssm_scan: dt must be [T, H]")
    for v, nm in ((dt_shift, "dt_shift"), (a_log, "A_log"), (d_skip, "D")):
        _f32vec(v, H, f"ssm_scan: {nm}")
    if not (out.shape == (xbc.shape[0], H * P) and out.is_contiguous() and out.dtype == xbc.dtype
            and out.data_ptr() % 16 == 0):
        raise KernelError("ssm_scan: out must be [T, H*P] on a 16-byte boundary")
    n_chunks = sum((n + SSD_TC_CHUNK - 1) // SSD_TC_CHUNK for n in new_lens)
    need = ssd_tc_scratch_floats(new_lens, H, P, N)
    if not (scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need
            and scratch.data_ptr() % 16 == 0):
        raise KernelError(f"ssm_scan_tc: needs {need} floats of 16-byte aligned scratch")
    chunk_state = scratch.data_ptr()
    chunk_decay = chunk_state + 4 * n_chunks * H * P * N
    chunk_dt = chunk_decay + 4 * ((n_chunks * H + 3) // 4 * 4)
    start_state = chunk_dt + 4 * n_chunks * H * 2 * SSD_TC_CHUNK
    zp, ld_z, zs, zb = _gate_args(gate, out, "ssm_scan_tc")
    n_multi = getattr(new_lens, "multi", None)  # lengths given as bounds carry the bound with them
    if n_multi is None:
        n_multi = sum(1 for n in new_lens if n > 1)
    _call("pmm_ssd_tc", xbc.data_ptr(), ld_x, dt_raw.data_ptr(), ld_dt, float(dt_scale), dt_shift.data_ptr(),
          a_log.data_ptr(), d_skip.data_ptr(), state.data_ptr(), cu.data_ptr(), slots.data_ptr(), out.data_ptr(),
          chunk_state, chunk_decay, chunk_dt, start_state, len(new_lens), n_chunks, H, P, N, n_groups, zp, ld_z, zs, zb,
          int(bool(skip_single)), n_multi if skip_single else 0,
          _tc_status(xbc.device).data_ptr(), _stream())


def gated_norm(y: Tensor, z_raw: Tensor, z_scale: float, z_bias: Optional[Tensor],
               weight: Optional[Tensor], eps: float, n_groups: int, norm_before_gate: bool,
               out: Tensor) -> None:
    """out = y*silu(z), optionally RMS-normalised per group of channels (before or after the gate)."""
    _cuda(y, z_raw, z_bias, weight, out)
    T, I = y.shape
    if not (y.is_contiguous() and out.is_contiguous() and out.shape == y.shape and out.dtype == y.dtype):
        raise KernelError("gated_norm: y and out must be contiguous [T, I] of one type")
    ld_z = _rows_view(z_raw, "gated_norm: z")
    if not (z_raw.shape == y.shape and z_raw.dtype == y.dtype):
        raise KernelError("gated_norm: z must match y")
    _f32vec(z_bias, I, "gated_norm: z_bias")
    _f32vec(weight, I, "gated_norm: weight")
    groups = n_groups if weight is not None else 1
    if not (I % groups == 0):
        raise KernelError("gated_norm: width must be a multiple of the group count")
    _call("pmm_gated_norm", y.data_ptr(), z_raw.data_ptr(), ld_z, float(z_scale), _ptr(z_bias),
          _ptr(weight), float(eps), int(bool(norm_before_gate)), out.data_ptr(), T, I, groups, _dt(y),
          _stream())


def check_head_dim(head_dim: int) -> None:
    if not (head_dim % 16 == 0 and 16 <= head_dim <= 256):
        raise KernelError(f"attention kernels take head sizes 16..256 in steps of 16, got {head_dim}")


def qkv_rope_store(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], q_scale: float, k_scale: float,
                   v_scale: float, inv_freq: Optional[Tensor], positions: Tensor, seq_of: Tensor,
                   block_table: Optional[Tensor], pool: Optional[Tensor], q_out: Tensor,
                   k_out: Optional[Tensor], v_out: Optional[Tensor], n_q_heads: int, n_kv_heads: int,
                   head_dim: int) -> None:
    """Scales q/k/v, rotates q and k (when inv_freq is given) and stores k/v into the pages of
    ``pool`` [pages, 2, page_size, Hkv*Dh] through ``block_table`` [n_seq, max_blocks], or into
    k_out/v_out when no pool is given.  With k and v None (n_kv_heads 0) only q is prepared."""
    _cuda(q, k, v, inv_freq, positions, seq_of, block_table, pool, q_out, k_out, v_out)
    check_head_dim(head_dim)
    T = q.shape[0]
    ldq = _rows_view(q, "qkv: q")
    if not (q.shape[1] == n_q_heads * head_dim and q.dtype == q_out.dtype):
        raise KernelError("qkv: q width or type")
    if not (q_out.is_contiguous() and q_out.shape == (T, n_q_heads * head_dim)):
        raise KernelError("qkv: q_out must be [T, Hq*Dh]")
    _f32vec(inv_freq, head_dim // 2, "qkv: inv_freq")
    _i32(positions, "qkv: positions")
    _i32(seq_of, "qkv: seq_of")
    page_size, max_blocks, ldk, ldv = 0, 0, 0, 0
    if k is None or v is None:
        if not (k is None and v is None and n_kv_heads == 0):
            raise KernelError("qkv: queries only means no k, no v, no kv heads")
        pool = block_table = k_out = v_out = None
    else:
        ldk, ldv = _rows_view(k, "qkv: k"), _rows_view(v, "qkv: v")
        kv_dim = n_kv_heads * head_dim
        if not (k.shape[1] == kv_dim and v.shape[1] == kv_dim and q.dtype == k.dtype == v.dtype):
            raise KernelError("qkv: slice widths do not match the head counts")
        if pool is not None:
            if not (block_table is not None):
                raise KernelError("qkv: a pool needs a block table")
            _i32(block_table, "qkv: block_table")
            if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()
                    and pool.dtype == q.dtype):
                raise KernelError("qkv: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
            page_size, max_blocks = pool.shape[2], block_table.shape[1]
        else:
            if not (k_out is not None and v_out is not None and k_out.is_contiguous() and v_out.is_contiguous()
                    and k_out.shape == (T, kv_dim) and v_out.shape == (T, kv_dim)):
                raise KernelError("qkv: k_out/v_out must be [T, Hkv*Dh]")
    _call("pmm_qkv_rope_store", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale),
          float(k_scale), float(v_scale), _ptr(inv_freq), positions.data_ptr(), seq_of.data_ptr(),
          _ptr(block_table), max_blocks, _ptr(pool), page_size, q_out.data_ptr(), _ptr(k_out),
          _ptr(v_out), T, n_q_heads, n_kv_heads, head_dim, _dt(q), _stream())


def kv_store(k: Tensor, v: Tensor, positions: Tensor, seq_of: Tensor, block_table: Tensor,
             pool: Tensor) -> None:
    """Copies contiguous k/v rows [T, Hkv*Dh] into the pages of ``pool``."""
    _cuda(k, v, positions, seq_of, block_table, pool)
    T, kv_dim = k.shape
    if not (k.is_contiguous() and v.is_contiguous() and v.shape == k.shape and k.dtype == v.dtype == pool.dtype):
        raise KernelError("kv_store: k and v must be contiguous [T, Hkv*Dh] of the pool's type")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()):
        raise KernelError("kv_store: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "kv_store: block_table")
    _call("pmm_kv_store", k.data_ptr(), v.data_ptr(), positions.data_ptr(), seq_of.data_ptr(),
          block_table.data_ptr(), block_table.shape[1], pool.data_ptr(), pool.shape[2], T, kv_dim,
          _dt(k), _stream())


def attention_scratch_floats(T: int, n_q_heads: int, head_dim: int, n_splits: int) -> int:
    return T * n_q_heads * n_splits * (head_dim + 2) if n_splits > 1 else 0


def flash_supported(n_q_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernel takes this shape (bfloat16 caches only)."""
    return bool(_fn("pmm_flash_supported")(n_q_heads, n_kv_heads, head_dim))


def flash_tile_rows(n_q_heads: int, n_kv_heads: int, head_dim: int, new_lens: Sequence[int]) -> int:
    """Rows of (token, query head of a group) that one block of the tensor-core attention kernel
    takes: 16 when every sequence brings at most 16 of them (decode), 128 for long portions of
    head sizes up to 64 (each key/value fragment then feeds two row tiles), else 64."""
    group = n_q_heads // n_kv_heads
    if group <= 16 and max(new_lens) * group <= 16:
        return 16
    if head_dim <= 64 and sum(new_lens) * n_q_heads >= _FLASH_128_FROM_ROWS:
        return 128
    return 64


_FLASH_128_FROM_ROWS = 49152  # measured: 64 rows a block are faster at 16k rows, 128 at 64k


def paged_attention(q: Tensor, pool: Tensor, block_table: Tensor, positions: Tensor, seq_of: Tensor,
                    out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int, softmax_scale: float,
                    window: int = 0, n_splits: int = 1, split_len: int = 0,
                    scratch: Optional[Tensor] = None, cu_seqlens: Optional[Tensor] = None,
                    new_lens: Optional[Sequence[int]] = None, use_tensor_cores: bool = True,
                    split_counter: Optional[Tensor] = None, tile_rows: Optional[int] = None) -> None:
    """Causal attention of every token over keys lo..pos of its request in the paged cache.
    With ``cu_seqlens`` and ``new_lens`` (tokens per sequence, host values) a bfloat16 cache of a
    supported shape goes to the tensor-core kernel; everything else to the float kernel.
    ``split_counter`` (int32, zero between calls, at least tiles x kv heads entries) lets the
    tensor-core kernel merge its key splits itself instead of in a second launch.  ``tile_rows``
    (rows of (token, query head of a group) per block: 16, 64 or 128) defaults to flash_tile_rows."""
    _cuda(q, pool, block_table, positions, seq_of, out, scratch, cu_seqlens)
    check_head_dim(head_dim)
    T = q.shape[0]
    if not (q.is_contiguous() and out.is_contiguous() and q.shape == (T, n_q_heads * head_dim)
            and out.shape == q.shape and q.dtype == out.dtype == pool.dtype):
        raise KernelError("attention: q and out must be contiguous [T, Hq*Dh] of the pool's type")
    if not (n_q_heads % n_kv_heads == 0):
        raise KernelError("attention: query heads must be a multiple of key/value heads")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * head_dim
            and pool.is_contiguous()):
        raise KernelError("attention: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "attention: block_table")
    _i32(positions, "attention: positions")
    _i32(seq_of, "attention: seq_of")
    part_o = part_ml = None
    if n_splits > 1:
        need = attention_scratch_floats(T, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need):
            raise KernelError(f"attention: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 32 == 0):
            raise KernelError("attention: split_len must be a positive multiple of 32")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * T * n_q_heads * n_splits * head_dim
    flash = (use_tensor_cores and q.dtype == torch.bfloat16 and cu_seqlens is not None and new_lens is not None
             and flash_supported(n_q_heads, n_kv_heads, head_dim))
    if flash:
        _i32(cu_seqlens, "attention: cu_seqlens")
        group = n_q_heads // n_kv_heads
        if tile_rows is None:
            tile_rows = flash_tile_rows(n_q_heads, n_kv_heads, head_dim, new_lens)
        if not (tile_rows in (16, 64, 128) and group <= tile_rows and (tile_rows < 128 or head_dim <= 64)
                and (tile_rows > 16 or max(new_lens) * group <= 16)):
            raise KernelError(f"attention: {tile_rows} rows per block do not fit this shape")
        tokens_per_tile = tile_rows // group
        n_tiles = sum((n + tokens_per_tile - 1) // tokens_per_tile for n in new_lens)
        counter = None
        if (split_counter is not None and 1 < n_splits <= 64 and split_counter.numel() >= n_tiles * n_kv_heads):
            _cuda(split_counter)
            _i32(split_counter, "attention: split_counter")
            counter = split_counter.data_ptr()
        _call("pmm_flash_paged_attention", q.data_ptr(), pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), part_o,
              part_ml, float(softmax_scale), int(window), int(split_len), int(n_splits), pool.shape[2],
              len(new_lens), n_tiles, int(tile_rows), n_q_heads, n_kv_heads, head_dim, counter, _stream())
        if counter is not None:
            return
    else:
        _call("pmm_paged_attention", q.data_ptr(), pool.data_ptr(), block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), seq_of.data_ptr(), out.data_ptr(), part_o, part_ml,
              float(softmax_scale), int(window), int(split_len), int(n_splits), pool.shape[2], T, n_q_heads,
              n_kv_heads, head_dim, _dt(q), _stream())
    if n_splits > 1:
        _call("pmm_flash_combine", part_o, part_ml, out.data_ptr(), T * n_q_heads, int(n_splits), head_dim,
              _dt(out), _stream())


# Decode attention with TMA tile loads where the sizes allow (PMM_TMA_DECODE=0: cp.async gathers throughout).
_TMA_DECODE = os.environ.get("PMM_TMA_DECODE", "1") == "1"


def flash_decode_supported(n_q_heads: int, n_kv_heads: int, head_dim: int) -> bool:
    """Whether flash_decode_attention takes this head shape (bfloat16, at most 16 query heads a group)."""
    return flash_supported(n_q_heads, n_kv_heads, head_dim) and n_q_heads // n_kv_heads <= 16


def flash_decode_attention(q: Tensor, k: Optional[Tensor], v: Optional[Tensor], q_scale: float, k_scale: float,
                           v_scale: float, inv_freq: Optional[Tensor], pool: Tensor, block_table: Tensor,
                           positions: Tensor, out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                           softmax_scale: float, window: int = 0, n_splits: int = 1, split_len: int = 0,
                           scratch: Optional[Tensor] = None, split_counter: Optional[Tensor] = None) -> None:
    """A decode step's attention straight from the projections (token t is sequence t's one new
    token): scales and rotates queries and new keys, writes the new keys and values into their
    cache pages and attends over the cache, in one launch.  ``k``/``v`` None: the cache has them."""
    _cuda(q, k, v, inv_freq, pool, block_table, positions, out, scratch, split_counter)
    n_seq = q.shape[0]
    kv_dim = n_kv_heads * head_dim
    if not (q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and flash_decode_supported(n_q_heads, n_kv_heads, head_dim)):
        raise KernelError("decode attention: bfloat16 and a supported shape")
    ldq = _rows_view(q, "decode attention: q")
    if not (q.shape[1] == n_q_heads * head_dim and out.is_contiguous() and out.shape == (n_seq, n_q_heads * head_dim)):
        raise KernelError("decode attention: q/out must be [n_seq, Hq*Dh]")
    ldk = ldv = 0
    if k is not None or v is not None:
        if not (k is not None and v is not None and k.dtype == v.dtype == torch.bfloat16
                and k.shape == (n_seq, kv_dim) and v.shape == (n_seq, kv_dim)):
            raise KernelError("decode attention: k/v must be [n_seq, Hkv*Dh]")
        ldk, ldv = _rows_view(k, "decode attention: k"), _rows_view(v, "decode attention: v")
    _f32vec(inv_freq, head_dim // 2, "decode attention: inv_freq")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == kv_dim and pool.is_contiguous()):
        raise KernelError("decode attention: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    _i32(block_table, "decode attention: block_table")
    _i32(positions, "decode attention: positions")
    if not (block_table.shape[0] >= n_seq and positions.numel() >= n_seq):
        raise KernelError("decode attention: one table row and position per sequence")
    part_o = part_ml = counter = None
    if n_splits > 1:
        need = attention_scratch_floats(n_seq, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need):
            raise KernelError(f"decode attention: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 32 == 0 and n_splits <= 64):
            raise KernelError("decode attention: bad key split")
        if not (split_counter is not None and split_counter.numel() >= n_seq * n_kv_heads):
            raise KernelError("decode attention: split keys need a counter per (sequence, key/value head)")
        _i32(split_counter, "decode attention: split_counter")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * n_seq * n_q_heads * n_splits * head_dim
        counter = split_counter.data_ptr()
    if (_TMA_DECODE and (n_splits == 1 or split_len % 64 == 0)
            and _fn("pmm_decode_attention_tma_supported")(n_q_heads, n_kv_heads, head_dim, pool.shape[2])):
        # the copy engine brings the tiles (pages of a multiple of 64 positions, head sizes 64 and 128)
        _call("pmm_decode_attention_tma", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale), float(k_scale),
              float(v_scale), _ptr(inv_freq), pool.data_ptr(), pool.shape[0], block_table.data_ptr(),
              block_table.shape[1], positions.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale),
              int(window), int(split_len), int(n_splits), pool.shape[2], n_seq, n_q_heads, n_kv_heads, head_dim, counter,
              _tc_status(q.device).data_ptr(), _stream())
        return
    _call("pmm_flash_decode_attention", q.data_ptr(), ldq, _ptr(k), ldk, _ptr(v), ldv, float(q_scale), float(k_scale),
          float(v_scale), _ptr(inv_freq), pool.data_ptr(), block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale), int(window), int(split_len),
          int(n_splits), pool.shape[2], n_seq, n_q_heads, n_kv_heads, head_dim, counter, _stream())


SKINNY_MAX_TOKENS = 64  # the weight-streaming products take up to 64 tokens (where their shared memory fits)
SKINNY_NORM_MAX_TOKENS = 16  # every block redoes the norm of all rows: beyond this a norm launch of its own is cheaper
# from here on the tcgen05 form (skinny_tc_*) is the faster one inside a decode step (0.5B sizes, ms a step,
# mma.sync / tcgen05: 32 tokens 1.87 / 2.09, 40 tokens 2.35 / 2.26, 48 tokens 2.63 / 2.51); PMM_TC_SKINNY_FROM moves it
SKINNY_TC_FROM_TOKENS = int(os.environ.get("PMM_TC_SKINNY_FROM", "33"))
SKINNY_NORM_MAX_WIDTH = 1024  # ... and so it is for rows wider than a warp keeps in registers (they are read twice)


def _skinny_check(M: int, w: Tensor, K: int, what: str) -> None:
    if not (M <= 64):
        raise KernelError(f"{what}: at most 64 tokens")
    if not (w.dtype == torch.bfloat16 and w.dim() == 2 and w.is_contiguous() and w.shape[1] == K and K % 8 == 0):
        raise KernelError(f"{what}: weights must be contiguous bfloat16 [rows, K] with K a multiple of 8")


def skinny_fits(M: int, K: int) -> bool:
    """Whether M tokens x K columns of activations fit in shared memory beside the weight pipeline
    (the products that cannot split K keep the whole row block resident)."""
    mp = 8 if M <= 8 else 16 if M <= 16 else 32 if M <= 32 else 64
    kx = (K + 255) // 256 * 256
    stages = 3 if mp > 32 else 5
    return M <= 64 and stages * 32 * 264 * 2 + mp * (kx + 8) * 2 + 3 * 32 * mp * 4 + (kx + mp) * 4 <= 220 * 1024


def skinny_linear_norm(h: Tensor, norm_weight: Tensor, eps: float, weight: Tensor, out: Tensor) -> None:
    """out[M, N] = (rmsnorm(h) * norm_weight) @ weight^T for M <= 64 rows of the float32 stream."""
    _cuda(h, norm_weight, weight, out)
    M, K = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_linear_norm: h must be contiguous float32")
    _skinny_check(M, weight, K, "skinny_linear_norm")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear_norm: {M} tokens x {K} columns do not fit in shared memory")
    _f32vec(norm_weight, K, "skinny_linear_norm: norm weight")
    N = weight.shape[0]
    if not (out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear_norm: out [M, N] bfloat16")
    _call("pmm_skinny_gemm", 0, M, N, None, 0, h.data_ptr(), norm_weight.data_ptr(), float(eps), weight.data_ptr(), K,
          1.0, None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def _skinny_x(x: Tensor, M: int, K: int, what: str) -> None:
    if not (x.dtype == torch.bfloat16 and x.shape == (M, K) and x.stride(1) == 1 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0):
        raise KernelError(f"{what}: x must be bfloat16 [M, K] with 16-byte aligned rows")


def skinny_linear(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[M, N] = x @ weight^T for M <= 64 rows of bfloat16 activations (weights streamed once)."""
    _cuda(x, weight, out)
    M, K = x.shape
    _skinny_check(M, weight, K, "skinny_linear")
    _skinny_x(x, M, K, "skinny_linear")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear: {M} tokens x {K} columns do not fit in shared memory")
    N = weight.shape[0]
    if not (out.dtype == torch.bfloat16 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear: out [M, N] bfloat16")
    _call("pmm_skinny_gemm", 0, M, N, x.data_ptr(), x.stride(0), None, None, 0.0, weight.data_ptr(), K,
          1.0, None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_linear_f32(x: Tensor, weight: Tensor, out: Tensor, scale: float) -> None:
    """out[M, N] (float32) = scale * (x @ weight^T) for M <= 64 rows of bfloat16 activations: the
    output head of a step that asks for few rows of logits (the table is streamed once)."""
    _cuda(x, weight, out)
    M, K = x.shape
    _skinny_check(M, weight, K, "skinny_linear_f32")
    _skinny_x(x, M, K, "skinny_linear_f32")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_linear_f32: {M} tokens x {K} columns do not fit in shared memory")
    N = weight.shape[0]
    if not (out.dtype == torch.float32 and out.shape == (M, N) and out.stride(1) == 1):
        raise KernelError("skinny_linear_f32: out [M, N] float32")
    _call("pmm_skinny_gemm_f32out", M, N, x.data_ptr(), x.stride(0), weight.data_ptr(), K, float(scale),
          out.data_ptr(), out.stride(0), _stream())


def skinny_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[M, F] = silu(gate * gate_mult) * up with [gate | up] = x @ gate_up^T, x bfloat16."""
    _cuda(x, gate_up, out)
    M, K = x.shape
    _skinny_check(M, gate_up, K, "skinny_swiglu")
    _skinny_x(x, M, K, "skinny_swiglu")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_swiglu: {M} tokens x {K} columns do not fit in shared memory")
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and out.dtype == torch.bfloat16 and out.shape == (M, F) and out.is_contiguous()):
        raise KernelError("skinny_swiglu: out [M, F] bfloat16 for gate_up [2F, K]")
    _call("pmm_skinny_gemm", 1, M, F, x.data_ptr(), x.stride(0), None, None, 0.0, gate_up.data_ptr(), K,
          float(gate_mult), None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_swiglu_norm(h: Tensor, norm_weight: Tensor, eps: float, gate_up: Tensor, gate_mult: float,
                       out: Tensor) -> None:
    """out[M, F] = silu(gate * gate_mult) * up with [gate | up] = (rmsnorm(h) * norm_weight) @ gate_up^T."""
    _cuda(h, norm_weight, gate_up, out)
    M, K = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_swiglu_norm: h must be contiguous float32")
    _skinny_check(M, gate_up, K, "skinny_swiglu_norm")
    if not (skinny_fits(M, K)):
        raise KernelError(f"skinny_swiglu_norm: {M} tokens x {K} columns do not fit in shared memory")
    _f32vec(norm_weight, K, "skinny_swiglu_norm: norm weight")
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and out.dtype == torch.bfloat16 and out.shape == (M, F) and out.is_contiguous()):
        raise KernelError("skinny_swiglu_norm: out [M, F] bfloat16 for gate_up [2F, K]")
    _call("pmm_skinny_gemm", 1, M, F, None, 0, h.data_ptr(), norm_weight.data_ptr(), float(eps), gate_up.data_ptr(), K,
          float(gate_mult), None, 0, None, 0, 0.0, out.data_ptr(), out.stride(0), None, 1, _stream())


def skinny_residual(h: Tensor, products: Sequence[Tuple[Tensor, Tensor, float]]) -> None:
    """h[M, N] += sum_i scale_i * (x_i @ w_i^T) for one or two (x, w, scale); float32 atomics, the K
    ranges are split over blocks."""
    if not (1 <= len(products) <= 2):
        raise KernelError("skinny_residual: one or two products")
    M, N = h.shape
    _cuda(h)
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_residual: h must be contiguous float32")
    args = []
    k_max = 0
    for x, w, sc in products:
        _cuda(x, w)
        K = x.shape[1]
        if not (x.dtype == torch.bfloat16 and x.shape[0] == M and x.stride(1) == 1 and x.stride(0) % 8 == 0
                and x.data_ptr() % 16 == 0):
            raise KernelError("skinny_residual: x must be bfloat16 [M, K] with 16-byte aligned rows")
        _skinny_check(M, w, K, "skinny_residual")
        if not (w.shape[0] == N):
            raise KernelError("skinny_residual: weight rows must equal the stream width")
        args.append((x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)))
        k_max = max(k_max, K)
    chunks = (k_max + 255) // 256
    col_blocks = (N + 31) // 32 * len(products)
    k_split = max(1, min(chunks, (296 + col_blocks - 1) // col_blocks))
    while k_split < chunks and not skinny_fits(M, (chunks + k_split - 1) // k_split * 256):
        k_split += 1
    a0 = args[0]
    a1 = args[1] if len(args) > 1 else (None, 0, None, 0, 0.0)
    _call("pmm_skinny_gemm", 2, M, N, a0[0], a0[1], None, None, 0.0, a0[2], a0[3], a0[4], a1[0], a1[1], a1[2], a1[3],
          a1[4], None, 0, h.data_ptr(), k_split, _stream())


class _SkinnyPhase(ctypes.Structure):
    """One product of skinny_chain; mirrors PmmSkinnyPhase of csrc/skinny_gemm.cu."""
    _fields_ = [("mode", ctypes.c_int), ("N", ctypes.c_int), ("x0", ctypes.c_void_p), ("ldx0", ctypes.c_longlong),
                ("h_in", ctypes.c_void_p), ("norm_w", ctypes.c_void_p), ("eps", ctypes.c_float),
                ("w0", ctypes.c_void_p), ("K0", ctypes.c_int), ("scale0", ctypes.c_float),
                ("x1", ctypes.c_void_p), ("ldx1", ctypes.c_longlong), ("w1", ctypes.c_void_p), ("K1", ctypes.c_int),
                ("scale1", ctypes.c_float), ("y", ctypes.c_void_p), ("ldy", ctypes.c_longlong),
                ("h_out", ctypes.c_void_p)]


_CHAIN_STATE: Dict[torch.device, Tuple[Tensor, Tensor]] = {}
SKINNY_CHAIN_MAX = 4


def _chain_state(device: torch.device) -> Tuple[Tensor, Tensor]:
    st = _CHAIN_STATE.get(device)
    if st is None:
        st = (torch.zeros(1, dtype=torch.int64, device=device), _watch(device).words[1:2])
        _CHAIN_STATE[device] = st
    return st


def skinny_chain_status(device) -> int:
    """0, or 1 when a barrier wait of a skinny_chain launch on this device ever gave up (synchronises)."""
    return int(_watch(torch.device(device)).words[1].item())


def skinny_chain(h: Tensor, phases: Sequence[Tuple]) -> None:
    """Up to 4 weight-streaming products over the float32 stream ``h`` [M <= 16, D] in ONE launch,
    each reading what the one before it wrote (barriers over the grid in between, the next
    product's weights requested before each barrier).  Phases:
      ("residual", [(x, w, scale), ...])                      h += sum scale * x @ w^T      (1 or 2 products)
      ("swiglu", norm_weight, eps, gate_up, gate_mult, out)   out = silu(g * gate_mult) * u, [g|u] = norm(h) @ gate_up^T
      ("store", norm_weight, eps, weight, out)                out = norm(h) @ weight^T
    """
    _cuda(h)
    M, D = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous() and M <= 16):
        raise KernelError("skinny_chain: h must be contiguous float32 [<=16, D]")
    if not (1 <= len(phases) <= SKINNY_CHAIN_MAX):
        raise KernelError(f"skinny_chain: 1 to {SKINNY_CHAIN_MAX} phases")
    arr = (_SkinnyPhase * len(phases))()
    for ph, slot in zip(phases, arr):
        kind = ph[0]
        if kind == "residual":
            products = ph[1]
            if not (1 <= len(products) <= 2):
                raise KernelError("skinny_chain: one or two products per residual phase")
            slot.mode, slot.N, slot.h_out = 2, D, h.data_ptr()
            for i, (x, w, sc) in enumerate(products):
                _cuda(x, w)
                K = x.shape[1]
                if not (x.dtype == torch.bfloat16 and x.shape[0] == M and x.stride(1) == 1 and x.stride(0) % 8 == 0
                        and x.data_ptr() % 16 == 0):
                    raise KernelError("skinny_chain: x must be bfloat16 [M, K] with 16-byte aligned rows")
                _skinny_check(M, w, K, "skinny_chain")
                if not (w.shape[0] == D):
                    raise KernelError("skinny_chain: weight rows must equal the stream width")
                if i == 0:
                    slot.x0, slot.ldx0, slot.w0, slot.K0, slot.scale0 = x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)
                else:
                    slot.x1, slot.ldx1, slot.w1, slot.K1, slot.scale1 = x.data_ptr(), x.stride(0), w.data_ptr(), K, float(sc)
        elif kind in ("swiglu", "store"):
            norm_w, eps, w = ph[1], ph[2], ph[3]
            out = ph[-1]
            _cuda(norm_w, w, out)
            _skinny_check(M, w, D, "skinny_chain")
            if not (skinny_fits(M, D)):
                raise KernelError(f"skinny_chain: {M} tokens x {D} columns do not fit in shared memory")
            _f32vec(norm_w, D, "skinny_chain: norm weight")
            n_out = w.shape[0] // 2 if kind == "swiglu" else w.shape[0]
            if not (out.dtype == torch.bfloat16 and out.shape == (M, n_out) and out.stride(1) == 1
                    and (kind == "store" or w.shape[0] == 2 * n_out)):
                raise KernelError("skinny_chain: out must be bfloat16 [M, N]")
            slot.mode, slot.N = (1 if kind == "swiglu" else 0), n_out
            slot.h_in, slot.norm_w, slot.eps = h.data_ptr(), norm_w.data_ptr(), float(eps)
            slot.w0, slot.K0, slot.scale0 = w.data_ptr(), D, (float(ph[4]) if kind == "swiglu" else 1.0)
            slot.y, slot.ldy = out.data_ptr(), out.stride(0)
        else:
            raise KernelError(f"skinny_chain: unknown phase {kind!r}")
    counter, status = _chain_state(h.device)
    _call("pmm_skinny_chain", ctypes.cast(arr, ctypes.c_void_p), len(phases), M, counter.data_ptr(), status.data_ptr(),
          _stream())


def _tc_status(device: torch.device) -> Tensor:
    return _watch(device).words[0:1]


def tc_gemm_status(device) -> int:
    """0 unless a bounded wait inside a tensor-core kernel gave up (tc_gemm: 1 producer, 2 MMA
    issuer, 3 epilogue; attention_tc: 11..15; skinny_tc: 21..24; decode attention: 31..33).  Reading it waits for the device."""
    return int(_tc_status(torch.device(device)).item())


def _skinny_tc_operand(x: Tensor, w: Tensor) -> bool:
    return (x.is_cuda and x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.dim() == 2 and w.dim() == 2
            and x.stride(1) == 1 and w.is_contiguous() and x.shape[1] == w.shape[1] and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def skinny_tc_supported(kind: str, x: Tensor, weight: Tensor, out: Optional[Tensor] = None) -> bool:
    """Whether the tcgen05 weight-streaming product (1..64 tokens) takes these operands; kind is
    "store", "swiglu" (both keep all of K resident: at most 1,024 columns) or "residual"."""
    if not _skinny_tc_operand(x, weight):
        return False
    mode = {"store": 0, "swiglu": 1, "residual": 2}[kind]
    T, K = x.shape
    n = weight.shape[0] // 2 if kind == "swiglu" else weight.shape[0]
    ldy = 8
    if out is not None and kind != "residual":
        if out.dtype != torch.bfloat16 or out.stride(1) != 1 or out.data_ptr() % 16:
            return False
        ldy = out.stride(0)
    return bool(_fn("pmm_skinny_tc_supported")(mode, T, n, K, 0, x.stride(0), 0, ldy))


def skinny_tc_linear(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[T, N] (bfloat16) = x @ weight^T for up to 64 tokens on the tcgen05 tensor cores."""
    _cuda(x, weight, out)
    if not (skinny_tc_supported("store", x, weight, out) and out.shape == (x.shape[0], weight.shape[0])):
        raise KernelError("skinny_tc_linear: operands not supported (bfloat16, <= 64 tokens, K <= 1024 and a "
                          "multiple of 8, aligned rows)")
    T, K = x.shape
    _call("pmm_skinny_tc", 0, T, weight.shape[0], x.data_ptr(), x.stride(0), weight.data_ptr(), K, 1.0, None, 0, None, 0,
          0.0, out.data_ptr(), out.stride(0), None, _tc_status(x.device).data_ptr(), _stream())


def skinny_tc_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[T, F] = silu(gate * gate_mult) * up with [gate | up] = x @ gate_up^T (tcgen05, up to 64 tokens)."""
    _cuda(x, gate_up, out)
    F = gate_up.shape[0] // 2
    if not (gate_up.shape[0] == 2 * F and skinny_tc_supported("swiglu", x, gate_up, out) and out.shape == (x.shape[0], F)):
        raise KernelError("skinny_tc_swiglu: operands not supported (bfloat16, <= 64 tokens, K <= 1024 and a "
                          "multiple of 8, aligned rows)")
    T, K = x.shape
    _call("pmm_skinny_tc", 1, T, F, x.data_ptr(), x.stride(0), gate_up.data_ptr(), K, float(gate_mult), None, 0, None, 0,
          0.0, out.data_ptr(), out.stride(0), None, _tc_status(x.device).data_ptr(), _stream())


def skinny_tc_residual(h: Tensor, products: Sequence[Tuple[Tensor, Tensor, float]]) -> None:
    """h[T, N] += sum_i scale_i * (x_i @ w_i^T) for one or two products (tcgen05, up to 64 tokens;
    float32 atomics, K in slices of at most 1,024 columns)."""
    if not (1 <= len(products) <= 2):
        raise KernelError("skinny_tc_residual: one or two products")
    _cuda(h)
    T, N = h.shape
    if not (h.dtype == torch.float32 and h.is_contiguous()):
        raise KernelError("skinny_tc_residual: h must be contiguous float32")
    flat = []
    for x, w, sc in products:
        _cuda(x, w)
        if not (skinny_tc_supported("residual", x, w) and x.shape[0] == T and w.shape[0] == N):
            raise KernelError("skinny_tc_residual: operands not supported (bfloat16, <= 64 tokens, K a multiple of "
                              "8, aligned rows)")
        flat.append((x.data_ptr(), x.stride(0), w.data_ptr(), x.shape[1], float(sc)))
    a0 = flat[0]
    a1 = flat[1] if len(flat) > 1 else (None, 0, None, 0, 0.0)
    _call("pmm_skinny_tc", 2, T, N, a0[0], a0[1], a0[2], a0[3], a0[4], a1[0], a1[1], a1[2], a1[3], a1[4], None, 0,
          h.data_ptr(), _tc_status(h.device).data_ptr(), _stream())


def tc_gemm_supported(x: Tensor, weight: Tensor, n_out: int, swiglu: bool) -> bool:
    """Whether the tcgen05 product takes these operands (bfloat16, K a multiple of 64, output
    columns a multiple of 128 for SwiGLU or 256 otherwise, 16-byte aligned rows)."""
    if x.dtype != torch.bfloat16 or weight.dtype != torch.bfloat16 or not x.is_cuda:
        return False
    if x.dim() != 2 or x.stride(1) != 1 or not weight.is_contiguous() or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return False
    return bool(_fn("pmm_tc_gemm_supported")(1 if swiglu else 0, x.shape[1], n_out, x.stride(0), n_out))


def tc_gemm_swiglu(x: Tensor, gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[T, F] = silu((x Wg^T) * gate_mult) * (x Wu^T), gate_up = [Wg; Wu]: one tcgen05 kernel
    (TMA operands, accumulator in tensor memory, activation in the epilogue)."""
    _cuda(x, gate_up, out)
    T, K = x.shape
    F = gate_up.shape[0] // 2
    if not (gate_up.shape == (2 * F, K) and out.shape == (T, F) and out.is_contiguous() and out.dtype == torch.bfloat16):
        raise KernelError("tc_gemm_swiglu: out must be contiguous bfloat16 [T, F] for gate_up [2F, K]")
    if not (tc_gemm_supported(x, gate_up, F, True)):
        raise KernelError("tc_gemm_swiglu: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm", 1, x.data_ptr(), x.stride(0), gate_up.data_ptr(), out.data_ptr(), out.stride(0), T, K, F,
          float(gate_mult), _tc_status(x.device).data_ptr(), _stream())


def tc_gemm(x: Tensor, weight: Tensor, out: Tensor) -> None:
    """out[T, N] = x @ weight^T on tcgen05 (bfloat16 in and out, float accumulation)."""
    _cuda(x, weight, out)
    T, K = x.shape
    N = weight.shape[0]
    if not (weight.shape == (N, K) and out.shape == (T, N) and out.stride(1) == 1 and out.dtype == torch.bfloat16
            and out.stride(0) % 8 == 0 and out.data_ptr() % 16 == 0):
        raise KernelError("tc_gemm: out must be bfloat16 [T, N], rows 16-byte aligned")
    if not (tc_gemm_supported(x, weight, N, False)):
        raise KernelError("tc_gemm: sizes or alignment outside what the kernel takes")
    _call("pmm_tc_gemm", 0, x.data_ptr(), x.stride(0), weight.data_ptr(), out.data_ptr(), out.stride(0), T, K, N,
          1.0, _tc_status(x.device).data_ptr(), _stream())


def attention_tc_supported(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 attention for prompt portions takes this shape (bfloat16, head size 64,
    a group size that divides 128, pages of a multiple of 64 tokens)."""
    return bool(_fn("pmm_attention_tc_supported")(n_q_heads, n_kv_heads, head_dim, page_size))


def attention_tc(q: Tensor, pool: Tensor, block_table: Tensor, positions: Tensor, cu_seqlens: Tensor,
                 new_lens: Sequence[int], out: Tensor, n_q_heads: int, n_kv_heads: int, head_dim: int,
                 softmax_scale: float, window: int = 0, n_splits: int = 1, split_len: int = 0,
                 scratch: Optional[Tensor] = None, split_counter: Optional[Tensor] = None) -> None:
    """Causal attention of prompt portions over the paged cache on the fifth-generation tensor cores
    (TMA tiles straight from the pages, scores and P V in tensor memory, one thread per query row
    for the softmax).  Same contract as paged_attention with rotated queries and a cache that holds
    the step's keys already; 128 rows of (token, query head of a group) per block."""
    _cuda(q, pool, block_table, positions, cu_seqlens, out, scratch, split_counter)
    T = q.shape[0]
    if not (q.dtype == torch.bfloat16 and pool.dtype == torch.bfloat16 and out.dtype == torch.bfloat16
            and q.is_contiguous() and out.is_contiguous() and q.shape == (T, n_q_heads * head_dim) and out.shape == q.shape):
        raise KernelError("attention_tc: q and out must be contiguous bfloat16 [T, Hq*Dh]")
    if not (pool.dim() == 4 and pool.shape[1] == 2 and pool.shape[3] == n_kv_heads * head_dim and pool.is_contiguous()):
        raise KernelError("attention_tc: pool must be contiguous [pages, 2, page_size, Hkv*Dh]")
    if not (attention_tc_supported(n_q_heads, n_kv_heads, head_dim, pool.shape[2])):
        raise KernelError("attention_tc: head size 64 or 128, at most 64 query heads per key/value head and pages "
                          "of a multiple of 64 tokens")
    _i32(block_table, "attention_tc: block_table")
    _i32(positions, "attention_tc: positions")
    _i32(cu_seqlens, "attention_tc: cu_seqlens")
    per_tile = 128 // (n_q_heads // n_kv_heads)
    n_tiles = sum((n + per_tile - 1) // per_tile for n in new_lens)
    part_o = part_ml = counter = None
    if n_splits > 1:
        need = attention_scratch_floats(T, n_q_heads, head_dim, n_splits)
        if not (scratch is not None and scratch.dtype == torch.float32 and scratch.is_contiguous()
                and scratch.numel() >= need and scratch.data_ptr() % 16 == 0):
            raise KernelError(f"attention_tc: split keys need {need} floats of scratch")
        if not (split_len > 0 and split_len % 64 == 0 and n_splits <= 64):
            raise KernelError("attention_tc: split_len must be a multiple of 64")
        if not (split_counter is not None and split_counter.numel() >= n_tiles * n_kv_heads):
            raise KernelError("attention_tc: split keys need a counter per (row tile, key/value head)")
        _i32(split_counter, "attention_tc: split_counter")
        part_o = scratch.data_ptr()
        part_ml = part_o + 4 * T * n_q_heads * n_splits * head_dim
        counter = split_counter.data_ptr()
    _call("pmm_attention_tc", q.data_ptr(), pool.data_ptr(), pool.shape[0], block_table.data_ptr(), block_table.shape[1],
          positions.data_ptr(), cu_seqlens.data_ptr(), out.data_ptr(), part_o, part_ml, float(softmax_scale), int(window),
          int(split_len), int(n_splits), pool.shape[2], len(new_lens), n_tiles, n_q_heads, n_kv_heads, head_dim, counter,
          _tc_status(q.device).data_ptr(), _stream())


def silu_mul(gate_up: Tensor, gate_mult: float, out: Tensor) -> None:
    """out[t, f] = silu(gate_up[t, f] * gate_mult) * gate_up[t, F + f]."""
    _cuda(gate_up, out)
    ld = _rows_view(gate_up, "silu_mul: gate_up")
    T, F2 = gate_up.shape
    if not (F2 % 2 == 0 and out.shape == (T, F2 // 2) and out.is_contiguous() and out.dtype == gate_up.dtype):
        raise KernelError("silu_mul: out must be contiguous [T, F] for gate_up [T, 2F]")
    _call("pmm_silu_mul", gate_up.data_ptr(), ld, float(gate_mult), out.data_ptr(), T, F2 // 2,
          _dt(gate_up), _stream())


def add_row_bias_(x: Tensor, bias: Tensor) -> None:
    """x[t, :] += bias (float32 vector) for a contiguous [T, D] activation."""
    _cuda(x, bias)
    if not (x.dim() == 2 and x.is_contiguous()):
        raise KernelError("add_row_bias_: x must be contiguous [T, D]")
    _f32vec(bias, x.shape[1], "add_row_bias_: bias")
    _call("pmm_add_row_bias", x.data_ptr(), bias.data_ptr(), x.shape[0], x.shape[1], _dt(x), _stream())


_SAMPLE_SCRATCH: Dict[torch.device, Tuple[Tensor, Tensor]] = {}


def ensure_sample_scratch(device, rows: int = 4096) -> Tuple[Tensor, Tensor]:
    """A 64-bit slot and a ticket per row for the blocks that share a row of sample_rows: one pair of
    buffers per device, zero when made and left zero by every launch (launches that use them are
    expected on one stream at a time).  Call it before a step is recorded into a CUDA graph:
    memory cannot be taken for it while a recording is under way."""
    device = torch.device(device)
    have = _SAMPLE_SCRATCH.get(device)
    if have is None or have[0].numel() < rows:
        if not (not torch.cuda.is_current_stream_capturing()):
            raise KernelError("sample_rows: its scratch must exist before a CUDA graph is recorded "
                              "(ensure_sample_scratch)")
        n = max(4096, rows)
        have = (torch.zeros(n, dtype=torch.int64, device=device), torch.zeros(n, dtype=torch.int32, device=device))
        _SAMPLE_SCRATCH[device] = have
    return have


def sample_rows(logits: Tensor, temperature: Optional[Tensor], seeds: Optional[Tensor],
                steps: Optional[Tensor], out: Tensor) -> None:
    """out[r] = argmax (first index on ties) where temperature[r] <= 0, else a draw from
    softmax(logits[r] / temperature[r]) keyed by (seeds[r], steps[r])."""
    _cuda(logits, temperature, seeds, steps, out)
    ld = _rows_view(logits, "sample: logits")
    n, V = logits.shape
    if not (logits.dtype == torch.float32):
        raise KernelError("sample: logits must be float32")
    _i32(out, "sample: out")
    if not (out.numel() == n):
        raise KernelError("sample: one output per row")
    if temperature is not None:
        _f32vec(temperature, n, "sample: temperature")
        if not (seeds is not None and seeds.dtype == torch.int64 and seeds.numel() == n and seeds.is_contiguous()):
            raise KernelError("sample: seeds must be int64 [rows]")
        if not (steps is not None and steps.numel() == n):
            raise KernelError("sample: steps must be int32 [rows]")
        _i32(steps, "sample: steps")
    slots, tickets = ensure_sample_scratch(logits.device, n)
    _call("pmm_sample_rows", logits.data_ptr(), ld, _ptr(temperature), _ptr(seeds), _ptr(steps),
          out.data_ptr(), n, V, slots.data_ptr(), tickets.data_ptr(), _stream())


def l2_prefetch(tensors: Sequence[Tensor]) -> None:
    """Asks the memory system to bring these tensors (contiguous, at most 8 per call, further
    ones in further launches) into L2; nothing waits for it."""
    ts = [t for t in tensors if t is not None and t.numel() > 0]
    for i in range(0, len(ts), 8):
        part = ts[i:i + 8]
        _cuda(*part)
        for t in part:
            if not (t.is_contiguous() and t.data_ptr() % 16 == 0):
                raise KernelError("l2_prefetch: tensors must be contiguous and 16-byte aligned")
        ptrs = (ctypes.c_void_p * len(part))(*[t.data_ptr() for t in part])
        sizes = (ctypes.c_longlong * len(part))(*[t.numel() * t.element_size() for t in part])
        _call("pmm_l2_prefetch", ctypes.cast(ptrs, ctypes.c_void_p), ctypes.cast(sizes, ctypes.c_void_p), len(part),
              _stream())


def ensure_built() -> str:
    """Build (if needed) and load the library; returns its path."""
    _build.load()
    return _build.library_path()
