"""The attention entry point that allocates nothing, called through its exported C symbol.

Some callers cannot hand the library a workspace or let it allocate one when they need
attention computed: a host loop with a latency bound, a plug-in in a process whose memory is
fixed at start-up, a caller without a tensor library.  For them ``pmm_attention_noalloc`` keeps
the scratch of the key splits in a fixed device array inside the library.  This test calls it
several times in a row (the array keeps the earlier calls' contents) and compares each result
with the regular entry point, which is given scratch by the caller, and with a softmax written
out in float32 over the keys gathered from the pages; one case has a window that lies wholly
behind some of the key splits.  The free device memory reported by the driver is read around
the later calls, so an allocation inside the library would show (the first call may load the
module).  Then calls the entry point must refuse are checked: each leaves a sentence and
launches nothing.

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


def _float32_reference(q, pool, bt, contexts, Hq, Hkv, Dh, page, window):
    """softmax(q k^T / sqrt(Dh)) v per sequence and head, in float32, keys gathered from the pages."""
    out = torch.empty(len(contexts), Hq * Dh, dtype=torch.float32)
    qf, poolf, btc = q.float().cpu(), pool.float().cpu(), bt.cpu()
    for s, c in enumerate(contexts):
        pages = btc[s, :(c + page - 1) // page].long()
        k = poolf[pages, 0].reshape(-1, Hkv, Dh)[:c]
        v = poolf[pages, 1].reshape(-1, Hkv, Dh)[:c]
        lo = max(0, c - window) if window > 0 else 0
        for h in range(Hq):
            g = h // (Hq // Hkv)
            sc = (k[lo:, g] @ qf[s, h * Dh:(h + 1) * Dh]) / math.sqrt(Dh)
            out[s, h * Dh:(h + 1) * Dh] = torch.softmax(sc, 0) @ v[lo:, g]
    return out


def _entry_point():
    from poor_mans_mamba_b200.kernels import build
    lib = build.load()
    fn = lib.pmm_attention_noalloc
    fn.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_float, c_int, c_int, c_int,
                   c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
    fn.restype = c_int
    err = lib.pmm_attention_noalloc_last_error
    err.restype = ctypes.c_char_p
    return fn, err


def test_no_alloc_attention_matches_the_regular_entry_point():
    from poor_mans_mamba_b200.kernels import ops
    fn, err = _entry_point()
    Hq, Hkv, Dh, page = 8, 2, 64, 64
    scale = 1.0 / math.sqrt(Dh)
    cases = [(1, [300, 129, 1000], 4, 0), (2, [64, 777, 5, 1200], 7, 0),
             (3, [900, 1100, 200], 6, 150)]   # window 150: of 6 ranges of 192 keys, the first ones lie wholly before it
    for call, (seed, contexts, n_splits, window) in enumerate(cases):
        q, pool, bt, pos, seq_of, cu = _setup(seed, contexts, Hq, Hkv, Dh, page)
        n = len(contexts)
        split_len = ((max(contexts) + n_splits - 1) // n_splits + 63) // 64 * 64
        ns = (max(contexts) + split_len - 1) // split_len
        assert ns > 1
        ref = torch.empty_like(q)
        scratch = torch.empty(ops.attention_scratch_floats(n, Hq, Dh, ns), dtype=torch.float32, device=DEV)
        ops.paged_attention(q, pool, bt, pos, seq_of, ref, Hq, Hkv, Dh, scale, window=window, n_splits=ns,
                            split_len=split_len, scratch=scratch, cu_seqlens=cu, new_lens=[1] * n)
        out = torch.full_like(q, float("nan"))
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = fn(q.data_ptr(), pool.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), cu.data_ptr(),
                out.data_ptr(), scale, window, split_len, ns, page, n, n, n, 1, Hq, Hkv, Dh,
                torch.cuda.current_stream().cuda_stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        if call > 0:  # the driver's own count of free memory: nothing was taken, by any allocator
            assert torch.cuda.mem_get_info()[0] == free_before
        assert torch.isfinite(out.float()).all()
        # the tolerance of the kernel tests for bfloat16 outputs
        exact = _float32_reference(q, pool, bt, contexts, Hq, Hkv, Dh, page, window)
        tol = 1.2e-2 * float(exact.abs().max())
        assert float((out.float().cpu() - exact).abs().max()) <= tol, f"call {call} against the float32 softmax"
        assert float((out.float() - ref.float()).abs().max()) <= tol, f"call {call} against the regular entry point"

    stream = torch.cuda.current_stream().cuda_stream
    # beyond the built-in array: refused, nothing launched, a sentence that says why
    q, pool, bt, pos, seq_of, cu = _setup(3, [4096] * 64, Hq, Hkv, Dh, page)
    out = torch.zeros_like(q)
    rc = fn(q.data_ptr(), pool.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), cu.data_ptr(), out.data_ptr(),
            scale, 0, 64, 64, page, 64, 64, 64, 1, Hq, Hkv, Dh, stream)
    assert rc == 1002
    msg = err().decode()
    assert "scratch" in msg and str(64 * Hq * 64 * (Dh + 2)) in msg
    # other refusals: each before any launch and each with its sentence
    q, pool, bt, pos, seq_of, cu = _setup(4, [200], Hq, Hkv, Dh, page)
    out = torch.zeros_like(q)

    def call(n_splits=2, split_len=128, sc=scale, rows16=1, hq=Hq, hkv=Hkv):
        return fn(q.data_ptr(), pool.data_ptr(), bt.data_ptr(), bt.shape[1], pos.data_ptr(), cu.data_ptr(),
                  out.data_ptr(), sc, 0, split_len, n_splits, page, 1, 1, 1, rows16, hq, hkv, Dh, stream)

    for kwargs, word in ((dict(n_splits=12289, split_len=64), "n_splits"), (dict(sc=0.0), "scale"),
                         (dict(hq=7), "head shape"), (dict(n_splits=2, split_len=0), "split_len"),
                         (dict(hq=64, hkv=2), "row tile"), (dict(n_splits=1, sc=-1.0), "scale")):
        assert call(**kwargs) == 1001, kwargs
        assert word in err().decode(), (kwargs, err().decode())
    torch.cuda.synchronize()
    assert float(out.float().abs().sum()) == 0.0
    assert call() == 0 and err().decode() == ""
    torch.cuda.synchronize()
