"""Each CUDA kernel alone against the plain formulas, at sizes other than the models' (GPU)."""
import math
import random

import pytest
import torch
import torch.nn.functional as F

from plain import falcon_h1_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def K():
    from poor_mans_mamba_b200.kernels import ops
    return ops


def tol(dtype, scale=1.0):
    return (2e-6 if dtype == torch.float32 else 1.2e-2) * scale


def close(got, ref, dtype, scale=None, what=""):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    scale = float(ref.abs().max()) if scale is None else scale
    err = float((got - ref).abs().max())
    assert err <= tol(dtype, max(scale, 1e-3)), f"{what}: err {err:.3e} scale {scale:.3e}"


def q(t, dtype):
    """Round a float64/32 tensor to the storage type (so kernel and reference see equal inputs)."""
    return t.to(dtype)


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(dtype):
    g = torch.Generator().manual_seed(1)
    table = q(torch.randn(101, 200, generator=g), dtype).to(DEV)
    toks = [100, 0, 57, 57, 3]
    out = torch.empty(5, 200, device=DEV)
    K().embed(out, table, i32(toks), 2.5)
    close(out, P.embedding(toks, table.double().cpu(), 2.5), torch.float32, what="embed")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [200, 1536, 13000])
def test_add_rmsnorm(dtype, D):
    g = torch.Generator().manual_seed(D)
    T = 7
    h0 = torch.randn(T, D, generator=g)
    a, b = q(torch.randn(T, D, generator=g), dtype), q(torch.randn(T, D, generator=g), dtype)
    w = torch.randn(D, generator=g)
    for branches in ([], [(a, 0.6)], [(a, 0.6), (b, -1.3)]):
        h = h0.clone().to(DEV)
        out = torch.empty(T, D, dtype=dtype, device=DEV)
        K().add_rmsnorm(h, [(t.to(DEV), s) for t, s in branches], w.to(DEV), 1e-3, out)
        hs = h0.double()
        for t, s in branches:
            hs = hs + s * t.double()
        close(h, hs, torch.float32, what="stream")
        close(out, P.rms_norm(hs, w.double(), 1e-3), dtype, what="norm")
    # selected rows leave the stream untouched
    h = h0.clone().to(DEV)
    rows = i32([6, 0, 3])
    out = torch.empty(3, D, dtype=dtype, device=DEV)
    K().add_rmsnorm(h, [(a.to(DEV), 0.6)], w.to(DEV), 1e-3, out, rows)
    assert torch.equal(h.cpu(), h0)
    close(out, P.rms_norm((h0.double() + 0.6 * a.double())[[6, 0, 3]], w.double(), 1e-3), dtype, what="rows")


def _batch(lens_steps):
    """lens_steps: per sequence a list of portion sizes.  Yields per step the flattened layout."""
    n_steps = max(len(p) for p in lens_steps)
    done = [0] * len(lens_steps)
    for s in range(n_steps):
        seqs = [(i, done[i], p[s]) for i, p in enumerate(lens_steps) if s < len(p)]
        yield seqs
        for i, a, n in seqs:
            done[i] += n


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,Kc,bias", [(200, 4, True), (33, 2, False), (130, 5, True), (64, 3, False)])
def test_conv1d_varlen_with_window(dtype, C, Kc, bias):
    g = torch.Generator().manual_seed(C)
    portions = [[5, 1, 1, 7], [1, 2, 9], [3, 1, 1, 1, 1]]
    lens = [sum(p) for p in portions]
    ld = C + 24  # the input is a column slice of a wider buffer
    xs = [q(torch.randn(n, C, generator=g), dtype) for n in lens]
    w = torch.randn(C, Kc, generator=g)
    cb = torch.randn(C, generator=g) if bias else None
    ps, pb = torch.rand(C, generator=g) + 0.5, (torch.randn(C, generator=g) if bias else None)
    refs = [P.causal_conv1d_silu(x.double() * ps.double() + (pb.double() if bias else 0), w.double(),
                                 cb.double() if bias else None) for x in xs]
    window = torch.zeros(4, Kc - 1, C, device=DEV)
    slots = [2, 0, 3]
    got = [torch.empty(n, C, dtype=dtype) for n in lens]
    dev = lambda t: None if t is None else t.to(DEV)
    for seqs in _batch(portions):
        T = sum(n for _, _, n in seqs)
        buf = torch.zeros(T, ld, dtype=dtype, device=DEV)
        x = buf[:, 8:8 + C]
        seq_of, cu, t0 = [], [0], 0
        for j, (i, a, n) in enumerate(seqs):
            x[t0:t0 + n] = xs[i][a:a + n].to(DEV)
            seq_of += [j] * n
            t0 += n
            cu.append(t0)
        out = torch.empty(T, C, dtype=dtype, device=DEV)
        sl = i32([slots[i] for i, _, _ in seqs])
        if all(n == 1 for _, _, n in seqs):
            K().conv1d_decode(x, dev(ps), dev(pb), dev(w), dev(cb), window, sl, out)
        else:
            K().conv1d_fwd(x, dev(ps), dev(pb), dev(w), dev(cb), window, i32(seq_of), i32(cu), sl, out,
                           weight_t=dev(w).t().contiguous())
            K().conv1d_window_update(x, dev(ps), dev(pb), window, i32(cu), sl, len(seqs), Kc)
        t0 = 0
        for i, a, n in seqs:
            got[i][a:a + n] = out[t0:t0 + n].cpu()
            t0 += n
    for i in range(3):
        close(got[i], refs[i], dtype, what=f"conv seq {i}")
    assert float(window[1].abs().sum()) == 0.0  # a slot nobody used


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,Pd,N,G", [(6, 20, 24, 3), (4, 64, 128, 1), (2, 40, 256, 2), (3, 16, 8, 1)])
def test_ssm_scan_continues_from_saved_state(dtype, H, Pd, N, G):
    g = torch.Generator().manual_seed(H * N)
    portions = [[6, 1, 1, 9], [1, 30]]
    lens = [sum(p) for p in portions]
    I, conv_dim = H * Pd, H * Pd + 2 * G * N
    xbcs = [q(torch.randn(n, conv_dim, generator=g), dtype) for n in lens]
    dts = [q(torch.randn(n, H, generator=g), dtype) for n in lens]
    a_log, d_skip, shift = torch.rand(H, generator=g) * 2, torch.randn(H, generator=g), torch.randn(H, generator=g)
    refs = [P.ssm_recurrence(x[:, :I].double().view(-1, H, Pd), x[:, I:I + G * N].double().view(-1, G, N),
                             x[:, I + G * N:].double().view(-1, G, N), dt.double() * 0.7, a_log.double(),
                             d_skip.double(), shift.double()).reshape(-1, I) for x, dt in zip(xbcs, dts)]
    state = torch.zeros(3, H, Pd, N, device=DEV)
    slots = [2, 0]
    got = [torch.empty(n, I, dtype=dtype) for n in lens]
    for seqs in _batch(portions):
        T = sum(n for _, _, n in seqs)
        xbc = torch.cat([xbcs[i][a:a + n] for i, a, n in seqs]).to(DEV)
        dtbuf = torch.zeros(T, H + 5, dtype=dtype, device=DEV)
        dtbuf[:, 5:] = torch.cat([dts[i][a:a + n] for i, a, n in seqs]).to(DEV)
        cu = [0]
        for _, _, n in seqs:
            cu.append(cu[-1] + n)
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        K().ssm_scan_seq(xbc, dtbuf[:, 5:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, i32(cu),
                         i32([slots[i] for i, _, _ in seqs]), len(seqs), out, G)
        t0 = 0
        for i, a, n in seqs:
            got[i][a:a + n] = out[t0:t0 + n].cpu()
            t0 += n
    for i in range(2):
        close(got[i], refs[i], dtype, what=f"scan seq {i}")
    assert float(state[1].abs().sum()) == 0.0 and float(state[2].abs().sum()) > 0


@pytest.mark.parametrize("H,Pd,N,G", [(6, 16, 16, 3), (4, 32, 32, 2), (2, 64, 64, 1), (4, 64, 128, 1), (2, 64, 256, 2),
                                      (2, 128, 128, 1), (2, 128, 256, 1)])
def test_ssd_chunked_scan(H, Pd, N, G):
    """The tensor-core scan over portions that start from a saved state, end inside a chunk, span
    several chunks, and share a step with single tokens; state checked against the serial kernel."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(H * N + Pd)
    portions = [[70, 1, 64, 9], [3, 130, 1], [64, 8, 128]]
    lens = [sum(p) for p in portions]
    I, conv_dim = H * Pd, H * Pd + 2 * G * N
    xbcs = [q(torch.randn(n, conv_dim, generator=g), dtype) for n in lens]
    dts = [q(torch.randn(n, H, generator=g), dtype) for n in lens]
    a_log, d_skip, shift = torch.rand(H, generator=g) * 2, torch.randn(H, generator=g), torch.randn(H, generator=g) - 1.0
    refs = [P.ssm_recurrence(x[:, :I].double().view(-1, H, Pd), x[:, I:I + G * N].double().view(-1, G, N),
                             x[:, I + G * N:].double().view(-1, G, N), dt.double() * 0.7, a_log.double(),
                             d_skip.double(), shift.double()).reshape(-1, I) for x, dt in zip(xbcs, dts)]
    state = torch.zeros(4, H, Pd, N, device=DEV)
    state_seq = torch.zeros(4, H, Pd, N, device=DEV)
    slots = [2, 0, 3]
    got = [torch.empty(n, I, dtype=dtype) for n in lens]
    for seqs in _batch(portions):
        T = sum(n for _, _, n in seqs)
        xbc = torch.cat([xbcs[i][a:a + n] for i, a, n in seqs]).to(DEV)
        dtbuf = torch.zeros(T, H + 8, dtype=dtype, device=DEV)
        dtbuf[:, 8:] = torch.cat([dts[i][a:a + n] for i, a, n in seqs]).to(DEV)
        cu = [0]
        for _, _, n in seqs:
            cu.append(cu[-1] + n)
        new_lens = [n for _, _, n in seqs]
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        out_seq = torch.empty(T, I, dtype=dtype, device=DEV)
        sl = i32([slots[i] for i, _, _ in seqs])
        scratch = torch.full((K().ssd_scratch_floats(new_lens, H, Pd, N),), float("nan"), device=DEV)
        K().ssm_scan_chunked(xbc, dtbuf[:, 8:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, i32(cu), sl,
                             new_lens, out, G, scratch)
        K().ssm_scan_seq(xbc, dtbuf[:, 8:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state_seq, i32(cu), sl,
                         len(seqs), out_seq, G)
        t0 = 0
        for i, a, n in seqs:
            got[i][a:a + n] = out[t0:t0 + n].cpu()
            t0 += n
    for i in range(3):
        close(got[i], refs[i], dtype, what=f"chunked scan seq {i}")
    close(state, state_seq, dtype, what="final states of the chunked and the serial scan")
    assert float(state[1].abs().sum()) == 0.0


@pytest.mark.parametrize("H,Pd,N,G,gated", [(6, 16, 16, 3, False), (4, 32, 48, 2, True), (3, 64, 64, 1, False),
                                            (24, 64, 128, 1, True), (5, 64, 256, 1, False), (2, 128, 128, 2, True),
                                            (2, 128, 256, 1, False), (3, 48, 80, 1, True), (2, 96, 112, 2, False)])
def test_ssd_tcgen05_scan(H, Pd, N, G, gated):
    """The tcgen05 scan over portions that start from a saved state, end inside a chunk, span several
    128-token chunks and share a step with single tokens, at head and state sizes the engine's
    models do not use (any multiples of 16); outputs against the plain recurrence, final states
    against the serial kernel; with and without the fused gate."""
    dtype = torch.bfloat16
    g = torch.Generator().manual_seed(H * N + Pd)
    portions = [[150, 1, 128, 9], [3, 260, 1], [128, 8, 130]]
    lens = [sum(p) for p in portions]
    I, conv_dim = H * Pd, H * Pd + 2 * G * N
    xbcs = [q(torch.randn(n, conv_dim, generator=g), dtype) for n in lens]
    dts = [q(torch.randn(n, H, generator=g), dtype) for n in lens]
    zs = [q(torch.randn(n, I, generator=g), dtype) for n in lens]
    zb = torch.randn(I, generator=g)
    a_log, d_skip, shift = torch.rand(H, generator=g) * 2, torch.randn(H, generator=g), torch.randn(H, generator=g) - 1.0
    refs = []
    for x, dt, z in zip(xbcs, dts, zs):
        yy = P.ssm_recurrence(x[:, :I].double().view(-1, H, Pd), x[:, I:I + G * N].double().view(-1, G, N),
                              x[:, I + G * N:].double().view(-1, G, N), dt.double() * 0.7, a_log.double(),
                              d_skip.double(), shift.double()).reshape(-1, I)
        refs.append(yy * P.silu(z.double() * 1.3 + zb.double()) if gated else yy)
    state = torch.zeros(4, H, Pd, N, device=DEV)
    state_seq = torch.zeros(4, H, Pd, N, device=DEV)
    slots = [2, 0, 3]
    got = [torch.empty(n, I, dtype=dtype) for n in lens]
    for seqs in _batch(portions):
        T = sum(n for _, _, n in seqs)
        xbc = torch.cat([xbcs[i][a:a + n] for i, a, n in seqs]).to(DEV)
        dtbuf = torch.zeros(T, H + 8, dtype=dtype, device=DEV)
        dtbuf[:, 8:] = torch.cat([dts[i][a:a + n] for i, a, n in seqs]).to(DEV)
        zbuf = torch.cat([zs[i][a:a + n] for i, a, n in seqs]).to(DEV)
        cu = [0]
        for _, _, n in seqs:
            cu.append(cu[-1] + n)
        new_lens = [n for _, _, n in seqs]
        out = torch.empty(T, I, dtype=dtype, device=DEV)
        out_seq = torch.empty(T, I, dtype=dtype, device=DEV)
        sl = i32([slots[i] for i, _, _ in seqs])
        gate = (zbuf, 1.3, zb.to(DEV)) if gated else None
        scratch = torch.full((K().ssd_tc_scratch_floats(new_lens, H, Pd, N),), float("nan"), device=DEV)
        lone = H % 2 == 0 and 1 in new_lens   # half the cases: lone tokens through the token-serial kernel
        K().ssm_scan_tc(xbc, dtbuf[:, 8:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, i32(cu), sl,
                        new_lens, out, G, scratch, gate=gate, skip_single=lone)
        if lone:
            K().ssm_scan_seq(xbc, dtbuf[:, 8:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state, i32(cu), sl,
                             len(seqs), out, G, gate=gate, only_single=True)
        K().ssm_scan_seq(xbc, dtbuf[:, 8:], 0.7, shift.to(DEV), a_log.to(DEV), d_skip.to(DEV), state_seq, i32(cu), sl,
                         len(seqs), out_seq, G, gate=gate)
        t0 = 0
        for i, a, n in seqs:
            got[i][a:a + n] = out[t0:t0 + n].cpu()
            t0 += n
    assert K().tc_gemm_status(DEV) == 0
    for i in range(3):
        close(got[i], refs[i], dtype, what=f"tcgen05 scan seq {i}")
    close(state, state_seq, dtype, what="final states of the tcgen05 and the serial scan")
    assert float(state[1].abs().sum()) == 0.0


def test_ssd_tcgen05_scan_refuses_other_sizes():
    assert not K().ssd_tc_supported(20, 24) and not K().ssd_tc_supported(64, 272) and not K().ssd_tc_supported(144, 64)
    assert K().ssd_tc_supported(112, 16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("mode", ["gate", "gate_then_norm", "norm_then_gate"])
def test_gated_norm(dtype, mode):
    g = torch.Generator().manual_seed(7)
    T, I, G = 5, 240, 3
    y, z = q(torch.randn(T, I, generator=g), dtype), q(torch.randn(T, I + 16, generator=g), dtype)
    zb, w = torch.randn(I, generator=g), torch.randn(I, generator=g)
    zz = z[:, 16:].double() * 1.3 + zb.double()
    ref = P.gate_and_norm(y.double(), zz, None if mode == "gate" else w.double(), 1e-4, G, mode == "norm_then_gate")
    out = torch.empty(T, I, dtype=dtype, device=DEV)
    K().gated_norm(y.to(DEV), z.to(DEV)[:, 16:], 1.3, zb.to(DEV), None if mode == "gate" else w.to(DEV), 1e-4, G,
                   mode == "norm_then_gate", out)
    close(out, ref, dtype, what=mode)


def _attention_case(dtype, Hq, Hkv, Dh, page_size, lens_steps, window=0, planted=True, n_splits=1, theta=1e4, seed=0,
                    tensor_cores=True, fused_merge=False, fused_decode=False, tc=False):
    """Runs qkv_rope_store + paged_attention over a script of portions with scattered pages and
    compares with the plain rope + causal attention on the whole sequences.  ``fused_decode``:
    steps in which every sequence brings one token go through flash_decode_attention instead
    (rotation, page write and attention in one launch).  ``tc``: the tcgen05 kernel for every step."""
    g = torch.Generator().manual_seed(seed)
    ops = K()
    lens = [sum(p) for p in lens_steps]
    qd, kvd = Hq * Dh, Hkv * Dh
    qs = [torch.randn(n, qd, generator=g) for n in lens]
    ks = [torch.randn(n, kvd, generator=g) for n in lens]
    vs = [torch.randn(n, kvd, generator=g) for n in lens]
    if planted:
        # one far key must win: the last query of every sequence is parallel to key 1
        # (rotation undone below by giving them the same position-independent direction is
        # impossible, so the score is made large through the norm instead)
        for x_q, x_k in zip(qs, ks):
            if x_k.shape[0] > 2:
                x_k[1] *= 4.0
                x_q[-1] *= 3.0
    qs, ks, vs = [q(t, dtype) for t in qs], [q(t, dtype) for t in ks], [q(t, dtype) for t in vs]
    q_scale, k_scale, v_scale = 0.8, 0.56, 0.8
    inv_freq = (1.0 / torch.pow(torch.tensor(theta, dtype=torch.float32),
                                (2.0 * torch.arange(Dh // 2, dtype=torch.float32)) / float(Dh)))
    refs = []
    for x_q, x_k, x_v in zip(qs, ks, vs):
        n = x_q.shape[0]
        pos = torch.arange(n)
        rq = P.rope_rotate_half(x_q.double().view(n, Hq, Dh) * q_scale, pos, Dh, theta)
        rk = P.rope_rotate_half(x_k.double().view(n, Hkv, Dh) * k_scale, pos, Dh, theta)
        rv = x_v.double().view(n, Hkv, Dh) * v_scale
        if dtype == torch.bfloat16:  # the cache holds rounded keys and values
            rq, rk, rv = rq.to(dtype).double(), rk.to(dtype).double(), rv.to(dtype).double()
        if window:
            out = torch.zeros(n, Hq, Dh, dtype=torch.float64)
            for t in range(n):
                lo = max(0, t - window + 1)
                o = P.causal_attention(torch.cat([rq[lo:t + 1]]), rk[lo:t + 1], rv[lo:t + 1], Hq // Hkv)
                out[t] = o[-1]
            refs.append(out.reshape(n, qd))
        else:
            refs.append(P.causal_attention(rq, rk, rv, Hq // Hkv).reshape(n, qd))
    n_pages = sum((n + page_size - 1) // page_size for n in lens) + 3
    order = list(range(n_pages))
    random.Random(seed).shuffle(order)
    pool = torch.zeros(n_pages + 1, 2, page_size, kvd, dtype=dtype, device=DEV)
    pool[n_pages].fill_(float("nan"))  # the spare page must never be read for a real key
    tables = [[] for _ in lens]
    got = [torch.empty(n, qd, dtype=dtype) for n in lens]
    counter = torch.zeros(1024, dtype=torch.int32, device=DEV)
    for seqs in _batch(lens_steps):
        T = sum(n for _, _, n in seqs)
        for i, a, n in seqs:
            while len(tables[i]) * page_size < a + n:
                tables[i].append(order.pop())
        width = max(len(tables[i]) for i, _, _ in seqs) + 1
        bt = torch.full((len(seqs), width), n_pages, dtype=torch.int32)
        for j, (i, _, _) in enumerate(seqs):
            bt[j, :len(tables[i])] = torch.tensor(tables[i], dtype=torch.int32)
        buf = torch.zeros(T, qd + 2 * kvd + 8, dtype=dtype, device=DEV)
        pos, seq_of, t0 = [], [], 0
        for j, (i, a, n) in enumerate(seqs):
            buf[t0:t0 + n, 8:8 + qd] = qs[i][a:a + n].to(DEV)
            buf[t0:t0 + n, 8 + qd:8 + qd + kvd] = ks[i][a:a + n].to(DEV)
            buf[t0:t0 + n, 8 + qd + kvd:] = vs[i][a:a + n].to(DEV)
            pos += list(range(a, a + n))
            seq_of += [j] * n
            t0 += n
        q_rot = torch.empty(T, qd, dtype=dtype, device=DEV)
        out = torch.empty(T, qd, dtype=dtype, device=DEV)
        if fused_decode and all(n == 1 for _, _, n in seqs):
            split_len, scratch, ns = 0, None, 1
            if n_splits > 1:
                split_len = ((max(pos) + 1 + n_splits - 1) // n_splits + 63) // 64 * 64
                ns = (max(pos) + 1 + split_len - 1) // split_len
                scratch = torch.full((ops.attention_scratch_floats(T, Hq, Dh, ns),), float("nan"), device=DEV)
            ops.flash_decode_attention(buf[:, 8:8 + qd], buf[:, 8 + qd:8 + qd + kvd], buf[:, 8 + qd + kvd:], q_scale,
                                       k_scale, v_scale, inv_freq.to(DEV), pool, bt.to(DEV), i32(pos), out, Hq, Hkv, Dh,
                                       1.0 / math.sqrt(Dh), window=window, n_splits=ns, split_len=split_len,
                                       scratch=scratch, split_counter=counter)
            t0 = 0
            for i, a, n in seqs:
                got[i][a:a + n] = out[t0:t0 + n].cpu()
                t0 += n
            continue
        ops.qkv_rope_store(buf[:, 8:8 + qd], buf[:, 8 + qd:8 + qd + kvd], buf[:, 8 + qd + kvd:], q_scale, k_scale,
                           v_scale, inv_freq.to(DEV), i32(pos), i32(seq_of), bt.to(DEV), pool, q_rot, None, None,
                           Hq, Hkv, Dh)
        split_len, scratch = 0, None
        if n_splits > 1:
            split_len = ((max(pos) + 1 + n_splits - 1) // n_splits + 31) // 32 * 32
            ns = (max(pos) + 1 + split_len - 1) // split_len
            scratch = torch.full((ops.attention_scratch_floats(T, Hq, Dh, ns),), float("nan"), device=DEV)
        else:
            ns = 1
        cu = [0]
        for _, _, n in seqs:
            cu.append(cu[-1] + n)
        if tc:
            if ns > 1:
                split_len = (split_len + 63) // 64 * 64
                ns = (max(pos) + 1 + split_len - 1) // split_len
            ops.attention_tc(q_rot, pool, bt.to(DEV), i32(pos), i32(cu), [n for _, _, n in seqs], out, Hq, Hkv, Dh,
                             1.0 / math.sqrt(Dh), window=window, n_splits=ns, split_len=split_len if ns > 1 else 0,
                             scratch=scratch, split_counter=counter)
            t0 = 0
            for i, a, n in seqs:
                got[i][a:a + n] = out[t0:t0 + n].cpu()
                t0 += n
            continue
        ops.paged_attention(q_rot, pool, bt.to(DEV), i32(pos), i32(seq_of), out, Hq, Hkv, Dh, 1.0 / math.sqrt(Dh),
                            window=window, n_splits=ns, split_len=split_len, scratch=scratch, cu_seqlens=i32(cu),
                            new_lens=[n for _, _, n in seqs], use_tensor_cores=tensor_cores,
                            split_counter=counter if fused_merge else None)
        t0 = 0
        for i, a, n in seqs:
            got[i][a:a + n] = out[t0:t0 + n].cpu()
            t0 += n
    for i in range(len(lens)):
        close(got[i], refs[i], dtype, what=f"attention seq {i} (len {lens[i]})")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tensor_cores", [True, False])
@pytest.mark.parametrize("Hq,Hkv,Dh,page", [(6, 3, 48, 16), (8, 2, 64, 64), (5, 1, 128, 32), (2, 2, 16, 16), (9, 3, 256, 16),
                                            (6, 2, 64, 16), (12, 2, 128, 64), (40, 2, 32, 32)])
def test_paged_attention_prefill_and_decode(dtype, tensor_cores, Hq, Hkv, Dh, page):
    """Head groups of 1..20 (also 3 and 6, which do not divide a row tile), head sizes on and off
    the tensor-core kernel's list, portions around page edges, single tokens."""
    steps = [[page + 1, 1, 1, page - 2, 1], [3, 2 * page, 1, 1], [1, 1, 1, 1, 1], [70, 1, 90]]
    _attention_case(dtype, Hq, Hkv, Dh, page, steps, seed=Hq, tensor_cores=tensor_cores)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_paged_attention_split_keys(dtype, tensor_cores):
    steps = [[300, 1, 1], [17, 1, 1], [129, 1, 1]]
    _attention_case(dtype, 8, 2, 64, 16, steps, n_splits=4, seed=5, tensor_cores=tensor_cores)
    _attention_case(dtype, 3, 1, 80, 32, steps, n_splits=7, seed=6, tensor_cores=tensor_cores)
    _attention_case(dtype, 6, 2, 128, 64, steps, n_splits=5, seed=7, tensor_cores=tensor_cores)
    if tensor_cores:  # the last block of every tile merges the splits (counter returns to zero each step)
        _attention_case(dtype, 8, 2, 64, 64, steps, n_splits=4, seed=5, fused_merge=True)
        _attention_case(dtype, 6, 2, 128, 16, steps, n_splits=9, seed=8, fused_merge=True)
        _attention_case(dtype, 4, 2, 32, 16, [[40, 1, 1, 30], [5, 1, 60]], window=24, n_splits=3, seed=9, fused_merge=True)


@pytest.mark.parametrize("tma", [True, False])
@pytest.mark.parametrize("Hq,Hkv,Dh,page", [(8, 2, 64, 64), (6, 2, 128, 16), (4, 4, 32, 32), (16, 1, 16, 16), (12, 2, 128, 64),
                                            (3, 1, 64, 128), (16, 1, 128, 64)])
def test_flash_decode_attention_from_projections(Hq, Hkv, Dh, page, tma, monkeypatch):
    """Decode steps that rotate, store and attend in one launch: after prompts of several lengths
    (page edges, tile edges), one key range and several, more tiles in one block than its ring
    holds (the new key's tile then comes in a later round), and a window.  Both forms: tiles
    brought by the copy engine (pages of a multiple of 64 positions, head sizes 64 and 128) and
    gathered with cp.async."""
    ops = K()
    monkeypatch.setattr(ops, "_TMA_DECODE", tma)
    calls = []
    original = ops._call
    monkeypatch.setattr(ops, "_call", lambda name, *a: (calls.append(name), original(name, *a))[1])
    steps = [[page + 1] + [1] * 6, [63] + [1] * 6, [300] + [1] * 6, [1] * 7, [700] + [1] * 3]
    _attention_case(torch.bfloat16, Hq, Hkv, Dh, page, steps, seed=Hq, fused_decode=True)
    _attention_case(torch.bfloat16, Hq, Hkv, Dh, page, steps, seed=Hq + 1, n_splits=3, fused_decode=True)
    _attention_case(torch.bfloat16, Hq, Hkv, Dh, page, steps, seed=Hq + 2, window=40, n_splits=2, fused_decode=True)
    _attention_case(torch.bfloat16, Hq, Hkv, Dh, page, steps, seed=Hq + 3, window=70, fused_decode=True)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    by_copy_engine = tma and page % 64 == 0 and Dh in (64, 128)
    assert ("pmm_decode_attention_tma" in calls) == by_copy_engine
    assert ("pmm_flash_decode_attention" in calls) == (not by_copy_engine)


@pytest.mark.parametrize("n_splits", [1, 5, 40])
def test_decode_attention_over_a_long_context(n_splits):
    """One decoded token over 33,100 cached positions in pages scattered over the pool: one key
    range (more block-table entries than the kernel keeps in shared memory), a cluster of five, and
    forty ranges (too many for a cluster: merged through global memory and the counter); a planted
    far key that takes the whole softmax, then random keys."""
    ops = K()
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(n_splits)
    Hq, Hkv, Dh, page, ctx = 8, 2, 64, 64, 33100
    G, kvd, qd = Hq // Hkv, Hkv * Dh, Hq * Dh
    n_blocks = (ctx + page) // page + 1
    pool = (torch.randn(n_blocks + 3, 2, page, kvd, generator=g) * 0.5).to(bf).to(DEV)
    table = torch.randperm(n_blocks + 3, generator=g)[:n_blocks].int()
    bt = table.view(1, -1).contiguous().to(DEV)
    pos = torch.tensor([ctx - 1], dtype=torch.int32, device=DEV)
    for planted in (True, False):
        proj = (torch.randn(1, qd + 2 * kvd, generator=g) * 0.5).to(bf).to(DEV)
        if planted:  # key 7 of the context equals 16 x the first query head's query: that score stands out
            pg, off = int(table[7 // page]), 7 % page
            pool[pg, 0, off, :Dh] = (proj[0, :Dh].float() * 16).to(bf)
        out = torch.empty(1, qd, dtype=bf, device=DEV)
        split_len = ((ctx + n_splits - 1) // n_splits + 63) // 64 * 64 if n_splits > 1 else 0
        ns = (ctx + split_len - 1) // split_len if n_splits > 1 else 1
        scratch = torch.empty(ops.attention_scratch_floats(1, Hq, Dh, ns), device=DEV) if ns > 1 else None
        counter = torch.zeros(Hkv, dtype=torch.int32, device=DEV)
        before = pool.clone()
        ops.flash_decode_attention(proj[:, :qd], proj[:, qd:qd + kvd], proj[:, qd + kvd:], 1.0, 1.0, 1.0, None, pool, bt, pos, out,
                                   Hq, Hkv, Dh, Dh ** -0.5, n_splits=ns, split_len=split_len, scratch=scratch,
                                   split_counter=counter)
        torch.cuda.synchronize()
        assert ops.tc_gemm_status(DEV) == 0 and int(counter.abs().sum()) == 0
        # the new token's key and value went into its page, nothing else changed
        pg, off = int(table[(ctx - 1) // page]), (ctx - 1) % page
        assert torch.equal(pool[pg, 0, off], proj[0, qd:qd + kvd]) and torch.equal(pool[pg, 1, off], proj[0, qd + kvd:])
        before[pg, :, off] = pool[pg, :, off]
        assert torch.equal(before, pool)
        # plain attention of the one token over the gathered context
        idx = table[: (ctx + page - 1) // page].long()
        kv = pool[idx.to(DEV)].double().cpu()                                    # [blocks, 2, page, kvd]
        keys = kv[:, 0].reshape(-1, Hkv, Dh)[:ctx]
        vals = kv[:, 1].reshape(-1, Hkv, Dh)[:ctx]
        q = proj[0, :qd].double().cpu().view(Hq, Dh)
        ref = torch.empty(Hq, Dh, dtype=torch.float64)
        for h in range(Hq):
            sc = (keys[:, h // G] @ q[h]) * Dh ** -0.5
            ref[h] = torch.softmax(sc, 0) @ vals[:, h // G]
        close(out.view(Hq, Dh), ref, bf, what=f"long-context decode attention, {ns} ranges, planted={planted}")
        if planted:
            assert float((out.view(Hq, Dh)[0].double().cpu() - vals[7, 0]).abs().max()) < 0.02


@pytest.mark.parametrize("Hq,Hkv,page,Dh", [(8, 2, 64, 64), (4, 4, 128, 64), (16, 1, 64, 64), (16, 2, 64, 64),
                                            (8, 2, 64, 128), (4, 1, 128, 128), (2, 2, 64, 128), (6, 2, 64, 128),
                                            (12, 2, 64, 128), (3, 1, 64, 64)])
def test_tcgen05_attention_over_the_paged_cache(Hq, Hkv, page, Dh):
    """The tcgen05 / TMA / tensor-memory attention for prompt portions: portions that start and end
    off the 128-key tiles and the 64-key boxes, portions over a long cached prefix, single tokens,
    several sequences in a step, key splits merged by the last block, and a window."""
    bf = torch.bfloat16
    steps = [[page + 1, 1, 200, page - 2, 1], [3, 2 * page, 1, 130], [1, 1, 1, 1], [70, 1, 333]]
    _attention_case(bf, Hq, Hkv, Dh, page, steps, seed=Hq, tc=True)
    _attention_case(bf, Hq, Hkv, Dh, page, steps, seed=Hq + 1, n_splits=3, tc=True)
    _attention_case(bf, Hq, Hkv, Dh, page, steps, seed=Hq + 2, window=100, tc=True)
    _attention_case(bf, Hq, Hkv, Dh, page, steps, seed=Hq + 3, window=150, n_splits=2, tc=True)
    assert K().tc_gemm_status(DEV) == 0
    assert not K().attention_tc_supported(Hq, Hkv, 96, page) and not K().attention_tc_supported(130, 2, 64, page)
    assert not K().attention_tc_supported(Hq, Hkv, Dh, 16)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tensor_cores", [True, False])
def test_paged_attention_window(dtype, tensor_cores):
    steps = [[40, 1, 1, 30], [5, 1, 60]]
    _attention_case(dtype, 4, 2, 32, 16, steps, window=24, seed=9, tensor_cores=tensor_cores)
    _attention_case(dtype, 4, 2, 32, 16, steps, window=24, n_splits=3, seed=9, tensor_cores=tensor_cores)
    _attention_case(dtype, 8, 2, 64, 64, [[200, 1, 1, 1]], window=70, n_splits=2, seed=10, tensor_cores=tensor_cores)


@pytest.mark.parametrize("dtype", DTYPES)
def test_silu_mul_bias_and_scale(dtype):
    g = torch.Generator().manual_seed(3)
    T, Fd = 4, 1100
    gu = q(torch.randn(T, 2 * Fd, generator=g), dtype)
    out = torch.empty(T, Fd, dtype=dtype, device=DEV)
    K().silu_mul(gu.to(DEV), 1.5, out)
    close(out, P.silu(gu[:, :Fd].double() * 1.5) * gu[:, Fd:].double(), dtype, what="silu_mul")
    x, b = q(torch.randn(T, 77, generator=g), dtype), torch.randn(77, generator=g)
    xd = x.to(DEV)
    K().add_row_bias_(xd, b.to(DEV))
    close(xd, x.double() + b.double(), dtype, what="row bias")
    f = torch.randn(1000, generator=g)
    fd = f.to(DEV)
    K().scale_f32_(fd, 0.3)
    close(fd, f.double() * 0.3, torch.float32)
    o = torch.empty(T, 77, device=DEV)
    K().cast_scale(o, x.to(DEV), 0.3)
    close(o, x.double() * 0.3, torch.float32)


def test_library_linear_in_true_float32():
    g = torch.Generator().manual_seed(4)
    x, w = torch.randn(33, 1000, generator=g), torch.randn(70, 1000, generator=g)
    out = torch.empty(33, 70, device=DEV)
    K().linear(x.to(DEV), w.to(DEV), out)
    err = float((out.double().cpu() - x.double() @ w.double().t()).abs().max())
    assert err < 2e-4, err  # a reduced-precision (tf32) product would be off by ~3e-2 here
    lo = torch.empty(33, 70, device=DEV)
    K().linear_f32_out(x.bfloat16().to(DEV), w.bfloat16().to(DEV), lo, torch.empty(33, 70, dtype=torch.bfloat16, device=DEV), 0.5)
    ref = 0.5 * (x.bfloat16().double() @ w.bfloat16().double().t())
    assert float((lo.double().cpu() - ref).abs().max()) < 0.3


@pytest.mark.parametrize("dtype", DTYPES)
def test_library_linear_with_padded_rows(dtype):
    """A product over whole matrices of the step's arena is issued with the row count rounded up
    (the arena keeps scratch rows behind them): the result is that of the exact product, rows that
    another tensor holds stay as they were, and a slice of rows is never padded."""
    from poor_mans_mamba_b200.engine import Workspace
    ops = K()
    g = torch.Generator().manual_seed(9)
    T, Kd, N = 100, 96, 72
    assert ops.padded_rows(T) == 128 and ops.padded_rows(64) == 64 and ops.padded_rows(1025) == 1152
    ws = Workspace(DEV, 1 << 22)
    x = ws.alloc((T, Kd), dtype)
    out = ws.alloc((T, N), dtype)
    after = ws.alloc((4, N), dtype)
    assert after.data_ptr() - out.data_ptr() >= 128 * N * out.element_size()
    xs, w = q(torch.randn(T, Kd, generator=g), dtype), q(torch.randn(N, Kd, generator=g), dtype).to(DEV)
    x.copy_(xs)
    after.fill_(7.0)
    ops.linear(x, w, out)
    close(out, xs.double() @ w.double().cpu().t(), dtype, what="padded product")
    assert bool((after == 7.0).all())
    # rows 10..90 of the same buffers: the rows behind belong to the tensor itself and must stay
    out.fill_(3.0)
    ops.linear(x[10:90], w, out[10:90])
    assert bool((out[:10] == 3.0).all()) and bool((out[90:] == 3.0).all())
    close(out[10:90], xs[10:90].double() @ w.double().cpu().t(), dtype, what="row slice")


def test_sampling_greedy_ties_and_temperature():
    ops = K()
    V = 1000
    logits = torch.zeros(4, V)
    logits[0, 5] = logits[0, 900] = 3.0     # tie: the first index wins
    logits[1, 999] = 1.0
    logits[2] = -1.0                         # all equal: index 0
    logits[3, 17] = float("inf")
    out = torch.empty(4, dtype=torch.int32, device=DEV)
    ops.sample_rows(logits.to(DEV), None, None, None, out)
    assert out.tolist() == [5, 999, 0, 17]
    # temperature: draws follow softmax(logits / T); same (seed, step) -> same draw
    V, n = 8, 4000
    base = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 1.5, -3.0, 0.0])
    rows = base.repeat(n, 1).to(DEV)
    temps = torch.full((n,), 0.7, device=DEV)
    seeds = torch.full((n,), 1234, dtype=torch.int64, device=DEV)
    steps = torch.arange(n, dtype=torch.int32, device=DEV)
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample_rows(rows, temps, seeds, steps, out)
    freq = torch.bincount(out.cpu().long(), minlength=V).double() / n
    want = torch.softmax(base.double() / 0.7, 0)
    assert float((freq - want).abs().max()) < 0.03, (freq, want)
    out2 = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample_rows(rows, temps, seeds, steps, out2)
    assert torch.equal(out, out2)
    ops.sample_rows(rows, temps, seeds + 1, steps, out2)
    assert not torch.equal(out, out2)
    temps[:] = 0.0  # temperature 0 inside a sampled batch is greedy
    ops.sample_rows(rows, temps, seeds, steps, out2)
    assert set(out2.tolist()) == {0}


@pytest.mark.parametrize("V", [4096, 4097, 32784, 130049])
def test_sampling_over_a_vocabulary_shared_by_several_blocks(V):
    """A row wider than one block's span is reduced by several blocks: greedy ties across spans
    (the first index wins), negative rows, repeated launches (slots and tickets are left clean), and
    temperature draws that equal those of the whole-row rule, argmax(logits / T + g_i)."""
    ops = K()
    g = torch.Generator().manual_seed(V)
    logits = torch.randn(6, V, generator=g)
    logits[0, 3] = logits[0, V - 1] = 9.0          # tie between the first and the last span
    logits[1] = -5.0                                # all equal and negative: index 0
    logits[2, V - 2] = 11.0
    logits[3, min(4096, V - 1)] = 12.0              # first entry of the second span (or the last)
    dev = logits.to(DEV)
    out = torch.empty(6, dtype=torch.int32, device=DEV)
    for _ in range(3):
        ops.sample_rows(dev, None, None, None, out)
        want = logits.argmax(dim=1).tolist()
        want[0], want[1] = 3, 0
        assert out.tolist() == want
    temps = torch.tensor([0.8, 1.3, 0.0, 0.5, 2.0, 1.0], device=DEV)
    seeds = torch.arange(6, dtype=torch.int64, device=DEV) + 77
    steps = torch.arange(6, dtype=torch.int32, device=DEV)
    a = torch.empty(6, dtype=torch.int32, device=DEV)
    b = torch.empty(6, dtype=torch.int32, device=DEV)
    ops.sample_rows(dev, temps, seeds, steps, a)
    ops.sample_rows(dev, temps, seeds, steps, b)
    assert torch.equal(a, b) and int(a[2]) == V - 2   # same keys -> same draws; T = 0 is greedy
    # one row at a time (another grid, same per-entry noise) draws the same tokens
    for r in range(6):
        one = torch.empty(1, dtype=torch.int32, device=DEV)
        ops.sample_rows(dev[r:r + 1], temps[r:r + 1], seeds[r:r + 1], steps[r:r + 1], one)
        assert int(one) == int(a[r])


def test_unsupported_sizes_are_refused():
    from poor_mans_mamba_b200.kernels.ops import KernelError
    from poor_mans_mamba_b200.parts.attention import PagedAttention
    from poor_mans_mamba_b200.parts.mamba2 import Mamba2Mixer
    with pytest.raises(KernelError, match="steps of 16"):
        PagedAttention(64, 4, 2, 24)
    with pytest.raises(KernelError, match="steps of 16"):
        PagedAttention(64, 4, 2, 512)
    with pytest.raises(ValueError, match="d_state"):
        Mamba2Mixer(64, 4, 16, 512, 4, 1)
    with pytest.raises(KernelError, match="CUDA tensors only"):
        K().silu_mul(torch.zeros(2, 4), 1.0, torch.zeros(2, 2))
    with pytest.raises(KernelError, match="float32 or bfloat16"):
        K().silu_mul(torch.zeros(2, 4, dtype=torch.float16, device=DEV), 1.0,
                     torch.zeros(2, 2, dtype=torch.float16, device=DEV))


@pytest.mark.parametrize("M,D,F,I2", [(8, 1024, 2048, 512), (1, 96, 160, 64), (16, 520, 264, 1544), (5, 1280, 3072, 768)])
def test_skinny_chain_matches_separate_products(M, D, F, I2):
    """Mixer output projections into the stream, norm + gate/up + SwiGLU, down projection into
    the stream and the next norm + projection, as one launch with grid barriers, against float64."""
    g = torch.Generator().manual_seed(M * D)
    bf = torch.bfloat16
    r = lambda *sh: torch.randn(*sh, generator=g)
    h0 = r(M, D)
    y1, y2 = (r(M, 768) * 0.5).to(bf), (r(M, I2) * 0.5).to(bf)
    w1, w2 = (r(D, 768) * 0.05).to(bf), (r(D, I2) * 0.05).to(bf)
    nw1, nw2 = torch.rand(D, generator=g) + 0.5, torch.rand(D, generator=g) + 0.5
    gu, down = (r(2 * F, D) * 0.05).to(bf), (r(D, F) * 0.05).to(bf)
    w_next = (r(200, D) * 0.05).to(bf)
    eps = 1e-5

    def norm(x, w):
        return x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * w.double()

    h_mid = h0.double() + 0.9 * (y1.double() @ w1.double().T) + 1.1 * (y2.double() @ w2.double().T)
    gate_up = norm(h_mid, nw1).to(bf).double() @ gu.double().T
    act = torch.nn.functional.silu(gate_up[:, :F] * 1.3) * gate_up[:, F:]

    hd = h0.to(DEV).contiguous()
    act_d = torch.empty(M, F, dtype=bf, device=DEV)
    nxt_d = torch.empty(M, 200, dtype=bf, device=DEV)
    dev = lambda t: t.to(DEV)

    def check(what):
        torch.cuda.synchronize()
        assert K().skinny_chain_status(DEV) == 0
        close(act_d, act, bf, what=f"{what}: activation")
        # the stream and the next projection, from the activation the kernel itself rounded
        h_end = h_mid + 0.7 * (act_d.double().cpu() @ down.double().T)
        close(hd, h_end, torch.float32, scale=30.0, what=f"{what}: stream")
        return h_end

    for rep in range(2):  # twice: the barrier counter carries over from launch to launch
        hd.copy_(h0)
        K().skinny_chain(hd, [("residual", [(dev(y1), dev(w1), 0.9), (dev(y2), dev(w2), 1.1)]),
                              ("swiglu", dev(nw1), eps, dev(gu), 1.3, act_d),
                              ("residual", [(act_d, dev(down), 0.7)]),
                              ("store", dev(nw2), eps, dev(w_next), nxt_d)])
        h_end = check(f"run {rep}")
        close(nxt_d, norm(h_end, nw2).to(bf).double() @ w_next.double().T, bf, what="next projection")
    # chains of one and of two phases leave the counter consistent for the next launch
    hd.copy_(h0)
    K().skinny_chain(hd, [("residual", [(dev(y1), dev(w1), 0.9), (dev(y2), dev(w2), 1.1)])])
    K().skinny_chain(hd, [("swiglu", dev(nw1), eps, dev(gu), 1.3, act_d), ("residual", [(act_d, dev(down), 0.7)])])
    check("two shorter chains")


@pytest.mark.parametrize("M", [1, 7, 16, 17, 40, 64])
@pytest.mark.parametrize("N,Kd", [(50, 96), (1024, 1000), (4120, 1024), (200, 2048), (9002, 3072), (20010, 520)])
def test_skinny_gemm_modes(M, N, Kd):
    """The weight-streaming product for few tokens: norm prologue + store, norm + SwiGLU, and
    residual accumulation of one and two products, at widths on and off the chunk size, and with
    more row tiles than blocks are resident (a block then walks several tiles)."""
    g = torch.Generator().manual_seed(M * 131 + N + Kd)
    ops = K()
    bf = torch.bfloat16
    h = torch.randn(M, Kd, generator=g)
    nw = torch.rand(Kd, generator=g) + 0.5
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(bf)
    x64 = P.rms_norm(h.double(), nw.double(), 1e-5).to(bf).double()  # the kernel rounds the normed row
    # STORE with the norm prologue, into a column slice of a wider buffer
    buf = torch.zeros(M, N + 16, dtype=bf, device=DEV)
    if not ops.skinny_fits(M, Kd):
        with pytest.raises(ops.KernelError, match="do not fit"):
            ops.skinny_linear_norm(h.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), buf[:, 8:8 + N])
    else:
        ops.skinny_linear_norm(h.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), buf[:, 8:8 + N])
        close(buf[:, 8:8 + N], x64 @ w.double().t(), bf, what="skinny store")
        assert float(buf[:, :8].abs().sum()) == 0 and float(buf[:, 8 + N:].abs().sum()) == 0
    # SWIGLU
    if N % 2 == 0 and ops.skinny_fits(M, Kd):
        F = N // 2
        act = torch.empty(M, F, dtype=bf, device=DEV)
        ops.skinny_swiglu_norm(h.to(DEV), nw.to(DEV), 1e-5, w.to(DEV), 1.5, act)
        gu = x64 @ w.double().t()
        close(act, P.silu(gu[:, :F] * 1.5) * gu[:, F:], bf, what="skinny swiglu")
    # RESIDUAL: one product, then two with different inner sizes and scales
    K2 = 64
    xa = (torch.randn(M, Kd, generator=g)).to(bf)
    xb = (torch.randn(M, K2, generator=g)).to(bf)
    wa = (torch.randn(N, Kd, generator=g) * 0.05).to(bf)
    wb = (torch.randn(N, K2, generator=g) * 0.05).to(bf)
    hres = torch.randn(M, N, generator=g)
    hd = hres.clone().to(DEV)
    ops.skinny_residual(hd, [(xa.to(DEV), wa.to(DEV), 0.6)])
    ref1 = hres.double() + 0.6 * (xa.double() @ wa.double().t())
    close(hd, ref1, torch.float32, scale=30.0, what="skinny residual one product")
    ops.skinny_residual(hd, [(xa.to(DEV), wa.to(DEV), -0.3), (xb.to(DEV), wb.to(DEV), 1.1)])
    ref2 = ref1 - 0.3 * (xa.double() @ wa.double().t()) + 1.1 * (xb.double() @ wb.double().t())
    close(hd, ref2, torch.float32, scale=30.0, what="skinny residual two products")


@pytest.mark.parametrize("M,N,Kd", [(1, 301, 64), (8, 32784, 1024), (33, 13001, 768), (64, 5000, 1024), (16, 5000, 3072)])
def test_skinny_product_with_float32_output_for_the_head(M, N, Kd):
    """scale * (x W^T) as float32 rows (the output head of steps that want few rows of logits),
    written into rows of a wider buffer; vocabularies that are no multiple of the 32-row tile."""
    g = torch.Generator().manual_seed(M + N + Kd)
    ops = K()
    bf = torch.bfloat16
    x = torch.randn(M, Kd, generator=g).to(bf)
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(bf)
    out = torch.full((M, N + 3), float("nan"), device=DEV)
    ops.skinny_linear_f32(x.to(DEV), w.to(DEV), out[:, :N], 0.7)
    close(out[:, :N], 0.7 * (x.double() @ w.double().t()), torch.float32, scale=30.0, what="skinny float32 head")
    assert bool(torch.isnan(out[:, N:]).all())


@pytest.mark.parametrize("T", [1, 17, 40, 64])
@pytest.mark.parametrize("N,Kd", [(50, 96), (1024, 1000), (4120, 1024), (6000, 512), (304, 72)])
def test_tcgen05_weight_streaming_product(T, N, Kd):
    """The tcgen05 form of the weight-streaming product (17..64 tokens; fewer work too): store,
    SwiGLU, and residual accumulation of one and two products with K in slices, at sizes on and
    off the boxes of 64 columns and tiles of 32 rows, with more row tiles than blocks (a block then
    walks several tiles through both accumulators), into column slices of wider buffers."""
    g = torch.Generator().manual_seed(T * 131 + N + Kd)
    ops = K()
    bf = torch.bfloat16
    xw = torch.randn(T, Kd + 8, generator=g).to(bf).to(DEV)
    x = xw[:, :Kd]                                       # rows with a stride of their own
    w = (torch.randn(N, Kd, generator=g) * 0.05).to(bf).to(DEV)
    ref = x.double().cpu() @ w.double().cpu().t()
    buf = torch.zeros(T, (N + 16 + 7) // 8 * 8, dtype=bf, device=DEV)  # rows of 16-byte multiples
    assert ops.skinny_tc_supported("store", x, w, buf[:, 8:8 + N])
    ops.skinny_tc_linear(x, w, buf[:, 8:8 + N])
    close(buf[:, 8:8 + N], ref, bf, what="tcgen05 skinny store")
    assert float(buf[:, :8].abs().sum()) == 0 and float(buf[:, 8 + N:].abs().sum()) == 0
    if N % 16 == 0:  # (rows of the output are 16-byte multiples)
        F = N // 2
        act = torch.full((T, F), float("nan"), dtype=bf, device=DEV)
        ops.skinny_tc_swiglu(x, w, 1.5, act)
        close(act, P.silu(ref[:, :F] * 1.5) * ref[:, F:], bf, what="tcgen05 skinny swiglu")
    # residual: one product whose K needs three slices, then two products of different inner sizes
    K1, K2 = 2304, 136
    xa = torch.randn(T, K1, generator=g).to(bf).to(DEV)
    xb = torch.randn(T, K2, generator=g).to(bf).to(DEV)
    wa = (torch.randn(N, K1, generator=g) * 0.05).to(bf).to(DEV)
    wb = (torch.randn(N, K2, generator=g) * 0.05).to(bf).to(DEV)
    hres = torch.randn(T, N, generator=g)
    hd = hres.clone().to(DEV)
    ops.skinny_tc_residual(hd, [(xa, wa, 0.6)])
    ref1 = hres.double() + 0.6 * (xa.double().cpu() @ wa.double().cpu().t())
    close(hd, ref1, torch.float32, scale=60.0, what="tcgen05 skinny residual one product")
    ops.skinny_tc_residual(hd, [(xa, wa, -0.3), (xb, wb, 1.1)])
    ref2 = ref1 - 0.3 * (xa.double().cpu() @ wa.double().cpu().t()) + 1.1 * (xb.double().cpu() @ wb.double().cpu().t())
    close(hd, ref2, torch.float32, scale=60.0, what="tcgen05 skinny residual two products")
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    # refusals: too many tokens, K not resident for a store
    assert not ops.skinny_tc_supported("store", torch.zeros(65, Kd, dtype=bf, device=DEV), w)
    assert not ops.skinny_tc_supported("store", xa, wa) and ops.skinny_tc_supported("residual", xa, wa)


@pytest.mark.parametrize("T,Kd,F", [(200, 128, 128), (128, 64, 256), (2048, 1024, 2048), (333, 1024, 384), (700, 3072, 640)])
def test_tcgen05_gemm_swiglu_and_plain(T, Kd, F):
    """The tcgen05 / TMA / tensor-memory product: SwiGLU epilogue and plain store, token counts
    that are no multiple of the 256-row tile (and below its half), several K stages (more than
    the pipeline is deep), and a refusal of feature counts off the tile."""
    g = torch.Generator().manual_seed(T + Kd + F)
    ops = K()
    bf = torch.bfloat16
    x = (torch.randn(T, Kd, generator=g)).to(bf)
    w = (torch.randn(2 * F, Kd, generator=g) * 0.05).to(bf)
    assert ops.tc_gemm_supported(x.to(DEV), w.to(DEV), F, True)
    act = torch.full((T, F), float("nan"), dtype=bf, device=DEV)
    ops.tc_gemm_swiglu(x.to(DEV), w.to(DEV), 1.5, act)
    torch.cuda.synchronize()
    assert ops.tc_gemm_status(DEV) == 0
    gu = x.double() @ w.double().t()
    close(act, P.silu(gu[:, :F] * 1.5) * gu[:, F:], bf, what="tcgen05 swiglu")
    assert not ops.tc_gemm_supported(x.to(DEV), w.to(DEV)[:2 * (F - 64)], F - 64, True)  # F no multiple of 128
    if (2 * F) % 256 == 0:
        y = torch.full((T, 2 * F), float("nan"), dtype=bf, device=DEV)
        ops.tc_gemm(x.to(DEV), w.to(DEV), y)
        torch.cuda.synchronize()
        assert ops.tc_gemm_status(DEV) == 0
        close(y, gu, bf, what="tcgen05 plain")
    assert not ops.tc_gemm_supported(x.to(DEV)[:, :Kd - 8], w.to(DEV), F, True)  # K no multiple of 64
