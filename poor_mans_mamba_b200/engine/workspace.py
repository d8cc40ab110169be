"""Per-step scratch memory: a bump arena over device buffers that are kept between steps.

Parts take temporaries with ``alloc`` and give them back in stack order with
``mark``/``release``; ``reset`` starts a new step.  The arena grows only when a step needs
more than any step before it (it then adds a chunk, and merges the chunks at the next
``reset``), so steady-state steps allocate nothing.
"""
from __future__ import annotations

import contextlib
import gc

from typing import List, Tuple

import torch

_ALIGN = 256
_ITEMSIZE = {torch.float32: 4, torch.bfloat16: 2, torch.float16: 2, torch.int32: 4, torch.int64: 8, torch.uint8: 1,
             torch.float64: 8, torch.int8: 1, torch.int16: 2, torch.bool: 1}


def _padded_rows(n_rows: int) -> int:
    from ..kernels.ops import padded_rows
    return padded_rows(n_rows)


class Workspace:
    def __init__(self, device: torch.device, initial_bytes: int = 0):
        self.device = torch.device(device)
        self._chunks: List[torch.Tensor] = []
        self._chunk = 0
        self._offset = 0
        self._frozen = False
        self._views = {}  # (chunk index, offset, shape, dtype) -> (tensor, bytes taken)
        self.high_water = 0
        if initial_bytes > 0:
            self._chunks.append(torch.empty(int(initial_bytes), dtype=torch.uint8, device=self.device))

    def freeze(self, frozen: bool = True) -> None:
        """While frozen the arena refuses to grow (addresses captured in a CUDA graph stay valid)."""
        self._frozen = frozen

    def capacity(self) -> int:
        return sum(c.numel() for c in self._chunks)

    def reset(self) -> None:
        if len(self._chunks) > 1 and not self._frozen:
            total = self.capacity()
            self._chunks = []
            self._views = {}
            self._chunks.append(torch.empty(total, dtype=torch.uint8, device=self.device))
        self._chunk = 0
        self._offset = 0

    def mark(self) -> Tuple[int, int]:
        return (self._chunk, self._offset)

    def release(self, mark: Tuple[int, int]) -> None:
        self._chunk, self._offset = mark

    def _used(self) -> int:
        return sum(c.numel() for c in self._chunks[:self._chunk]) + self._offset

    def alloc(self, shape, dtype: torch.dtype) -> torch.Tensor:
        """A tensor of ``shape``.  Behind a matrix of more than 64 rows the arena keeps scratch rows up
        to `kernels.ops.padded_rows`, so that a library product over it can be issued with a row
        count that recurs from step to step."""
        shape = tuple(shape)
        hit = self._views.get((self._chunk, self._offset, shape, dtype))
        if hit is not None:  # the same requests recur layer after layer and step after step
            view, size = hit
            self._offset += size
            if self._chunk == 0:
                if self._offset > self.high_water:
                    self.high_water = self._offset
            else:
                self.high_water = max(self.high_water, self._used())
            return view
        numel = 1
        for s in shape:
            numel *= s
        nbytes = numel * _ITEMSIZE[dtype]
        reserve, rows = nbytes, 0
        if len(shape) == 2 and shape[0] > 64:
            rows = _padded_rows(shape[0])
            reserve = rows * shape[1] * _ITEMSIZE[dtype]
        size = (max(reserve, 1) + _ALIGN - 1) // _ALIGN * _ALIGN
        while True:
            if self._chunk < len(self._chunks):
                chunk = self._chunks[self._chunk]
                off = self._offset
                if off + size <= chunk.numel():
                    view = chunk[off:off + nbytes].view(dtype).view(shape)
                    if rows > shape[0]:
                        # read by kernels.ops._mm: the matrix with its scratch rows (the storage is the chunk)
                        view._scratch_rows = rows
                        view._with_scratch_rows = chunk[off:off + reserve].view(dtype).view((rows, shape[1]))
                    self._views[(self._chunk, off, shape, dtype)] = (view, size)
                    self._offset = off + size
                    used = self._used()
                    if used > self.high_water:
                        self.high_water = used
                    return view
                self._chunk += 1
                self._offset = 0
                continue
            if self._frozen:
                raise RuntimeError("workspace is frozen and too small for this step")
            grow = max(size, self.capacity(), 1 << 20)
            self._chunks.append(torch.empty(grow, dtype=torch.uint8, device=self.device))


@contextlib.contextmanager
def quiet_capture(graph: "torch.cuda.CUDAGraph"):
    """``torch.cuda.graph(graph)`` with the garbage collector held back: a collection that runs in
    the middle of a capture may destroy CUDA graphs of objects that died earlier, and destroying a
    graph while a stream is capturing invalidates the capture."""
    gc.collect()
    was_enabled = gc.isenabled()
    gc.disable()
    try:
        with torch.cuda.graph(graph):
            yield
    finally:
        if was_enabled:
            gc.enable()


_CAPTURE_STREAMS = {}


@contextlib.contextmanager
def lean_capture(graph: "torch.cuda.CUDAGraph", device: torch.device):
    """Records what the body launches on the current stream into ``graph``, like `quiet_capture`, but
    without what ``torch.cuda.graph`` does on entry (a device synchronize, a full garbage collection
    and the return of all cached device memory to the driver: 40 ms and more, paid by a server
    whenever it records a new step shape between two steps).  The garbage collector is held back for
    the recording; the body runs on a stream kept for recordings (the legacy default stream cannot
    record), which first waits for the current one."""
    device = torch.device(device)
    stream = _CAPTURE_STREAMS.get(device)
    if stream is None:
        stream = _CAPTURE_STREAMS[device] = torch.cuda.Stream(device=device)
    current = torch.cuda.current_stream(device)
    stream.wait_stream(current)
    was_enabled = gc.isenabled()
    gc.disable()
    torch.cuda.set_stream(stream)
    try:
        graph.capture_begin()
        try:
            yield
        finally:
            graph.capture_end()
    finally:
        torch.cuda.set_stream(current)
        if was_enabled:
            gc.enable()
    current.wait_stream(stream)
