"""The attention entry point that allocates nothing, called through its exported C symbol.

Some callers cannot hand the library a workspace or let it allocate one when they need
attention computed: a host loop with a latency bound, a plug-in in a process whose memory is
fixed at start-up, a caller without a tensor library.  For them ``pmm_attention_noalloc`` keeps
the scratch of the key splits in a fixed device array inside the library.  This test calls it
twice in a row (the array keeps the first call's contents) and compares with the regular entry
point, which is given scratch by the caller; then it checks that an oversized call is refused
with a readable message and that nothing was allocated on the way.

The file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _setup(seed, contexts, Hq=8, Hkv=2, Dh=64, page=64):
    g = torch.Generator().manual_seed(seed)
    n_seq = len(contexts)
    n_pages = sum((c + page - 1) // page for c in contexts)
    pool = (torch.randn(n_pages + 1, 2, page, Hkv * Dh, generator=g)).to(torch.bfloat16).to(DEV)
    width = max((c + page - 1) // page for c in contexts)
    bt = torch.full((n_seq, width), n_pages, dtype=torch.int32)
    perm = torch.randperm(n_pages, generator=g).tolist()
    for s, c in enumerate(contexts):
        k = (c + page - 1) // page
        bt[s, :k] = torch.tensor([perm.pop() for _ in range(k)], dtype=torch.int32)
    q = torch.randn(n_seq, Hq * Dh, generator=g).to(torch.bfloat16).to(DEV)
    pos = torch.tensor([c - 1 for c in contexts], dtype=torch.int32, device=DEV)
    seq_of = torch.arange(n_seq, dtype=torch.int32, device=DEV)
    cu = torch.arange(n_seq + 1, dtype=torch.int32, device=DEV)
    return q, pool, bt.to(DEV), pos, seq_of, cu


def test_no_alloc_attention_matches_the_regular_entry_point():
    from poor_mans_mamba_b200.kernels import build, ops
    lib = build.load()
    fn = lib.pmm_attention_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    fn.restype = c_int
    err = lib.pmm_attention_noalloc_last_error
    err.restype = ctypes.c_char_p

    Hq, Hkv, Dh, page = 8, 2, 64, 64
    scale = 1.0 / math.sqrt(Dh)
    for call, (seed, contexts, n_splits) in enumerate([(1, [300, 129, 1000], 4), (2, [64, 777, 5, 1200], 7)]):
        q, pool, bt, pos, seq_of, cu = _setup(seed, contexts, Hq, Hkv, Dh, page)
        n = len(contexts)
        split_len = ((max(contexts) + n_splits - 1) // n_splits + 63) // 64 * 64
        ns = (max(contexts) + split_len - 1) // split_len
        ref = torch.empty_like(q)
        scratch = torch.empty(ops.attention_scratch_floats(n, Hq, Dh, ns), dtype=torch.float32, device=DEV)
        ops.paged_attention(q, pool, bt, pos, seq_of, ref, Hq, Hkv, Dh, scale, n_splits=ns, split_len=split_len,
                            scratch=scratch, cu_seqlens=cu, new_lens=[1] * n)
        out = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(q.data_ptr(), pool.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), cu.data_ptr(),
                out.data_ptr(), scale, 0, split_len, ns, page, n, n, n, 1, Hq, Hkv, Dh,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        assert torch.isfinite(out.float()).all()
        # the tolerance of the kernel tests for bfloat16 outputs; the two paths run the same kernels
        tol = 1.2e-2 * float(ref.float().abs().max())
        assert float((out.float() - ref.float()).abs().max()) <= tol, f"call {call}"

    # beyond the built-in array: refused, nothing launched, a sentence that says why
    q, pool, bt, pos, seq_of, cu = _setup(3, [4096] * 64, Hq, Hkv, Dh, page)
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), pool.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), cu.data_ptr(), out.data_ptr(),
            scale, 0, 64, 64, page, 64, 64, 64, 1, Hq, Hkv, Dh, torch.cuda.current_stream().cuda_stream)
    assert rc == 1002
    msg = err().decode()
    assert "scratch" in msg and str(64 * Hq * 64 * (Dh + 2)) in msg
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0
