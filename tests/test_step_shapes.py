"""Rounded step shapes (no GPU): the bounds that stand for the tokens per sequence, the rounding
rule, and the packed index buffer of a padded batch."""
import itertools
import types

import numpy as np
import pytest
import torch

from poor_mans_mamba_b200.cache import CacheManager
from poor_mans_mamba_b200.engine import runner as runner_mod
from poor_mans_mamba_b200.engine.context import LengthBounds
from poor_mans_mamba_b200.engine.runner import ModelRunner
from poor_mans_mamba_b200.parts.base import StateSpec


def compositions(total, count):
    """Every way to write ``total`` as ``count`` positive integers, in order."""
    for cuts in itertools.combinations(range(1, total), count - 1):
        yield [b - a for a, b in zip((0,) + cuts, cuts + (total,))]


@pytest.mark.parametrize("total,count", [(9, 2), (13, 3), (17, 4), (12, 5)])
def test_length_bounds_need_the_most_blocks_of_any_cut(total, count):
    bounds = LengthBounds(total, count)
    assert len(bounds) == count and sum(bounds) == total and bounds.multi == count
    for c in (1, 2, 3, 4, 5, 8, 16):
        most = sum(-(-n // c) for n in bounds)
        reached = False
        for cut in compositions(total, count):
            need = sum(-(-n // c) for n in cut)
            assert need <= most, (cut, c)
            reached = reached or need == most
        assert reached  # the bound is the largest need, not merely above it
        for fewer in range(1, count):  # cuts in which count - fewer sequences are empty
            assert all(sum(-(-n // c) for n in cut) <= most for cut in compositions(total, fewer))
    for cut in compositions(total, count):
        assert sum(1 for n in cut if n > 1) <= bounds.multi
    assert any(n == 1 for n in bounds) and max(bounds) >= 2


def test_length_bounds_refuse_what_no_batch_can_be():
    with pytest.raises(ValueError):
        LengthBounds(10, 1)
    with pytest.raises(ValueError):
        LengthBounds(3, 4)


def make_runner(accepts=True, max_seq_len=4096, page_size=4):
    specs = {0: [("attn.kv", StateSpec.paged("kv", 2, 8)), ("ssm.state", StateSpec.fixed("state", (2, 3), "float32"))]}
    cache = CacheManager(specs, page_size=page_size, num_pages=64, num_slots=6, dtype=torch.float32, device="cpu")
    r = ModelRunner.__new__(ModelRunner)
    r.cache, r.device, r.dtype = cache, cache.device, cache.dtype
    r.model = types.SimpleNamespace(accepts_length_bounds=lambda page: accepts, vocab_size=100)
    r.graphs = types.SimpleNamespace(max_seq_len=max_seq_len)
    r._accepts_bounds = None
    r._largest_rounded = 0
    r.token_budget = None
    return r


def test_rounding_rule():
    r = make_runner()
    key, pads, _, kv_b = r._rounded_shape([100, 100], 2, 128)      # short steps round up to 256 tokens
    assert key == ("rounded", 256, 4, 4, 128) and pads == [56, 0] and kv_b == 128
    assert r._rounded_shape([2], 1, 64)[0] == ("rounded", 256, 2, 2, 256) and r._rounded_shape([2], 1, 64)[1] == [254]
    assert r._rounded_shape([200, 100], 9, 256)[0] == ("rounded", 320, 4, 16, 256)   # more rows than sequences
    assert r._rounded_shape([1] * 300, 300, 512) is None          # decoding only
    key, pads, rows_b, kv_b = r._rounded_shape([2048], 1, 2048)
    assert key == ("rounded", 2048, 2, 2, 2048) and pads == [0] and rows_b == 2 and kv_b == 2048
    key, pads, rows_b, kv_b = r._rounded_shape([1000, 700, 300, 1, 1], 5, 1024)
    # five sequences: three padding sequences make eight, the first holds the 46 tokens up to 2,048
    assert key == ("rounded", 2048, 8, 8, 1024) and pads == [46, 0, 0]
    # below the largest size seen (2,048) sizes go in steps of 256
    key, pads, _, _ = r._rounded_shape([300, 27], 0, 512)
    assert key == ("rounded", 512, 4, 0, 512) and pads == [185, 0]
    key, pads, _, kv_b = r._rounded_shape([257], 1, 512)
    assert key[1] == 512 and pads == [255] and kv_b == 512
    for lens in ([256], [255, 1], [64] * 4, [1000, 3, 3, 3, 3, 3, 3, 3], [2047, 1]):
        key, pads, _, _ = r._rounded_shape(list(lens), 1, 4096)
        n_seq_b = key[2]
        assert n_seq_b & (n_seq_b - 1) == 0 and n_seq_b > len(lens) and len(pads) == n_seq_b - len(lens)
        assert pads[0] >= 0 and not any(pads[1:]) and key[1] == sum(lens) + sum(pads) and key[1] % 64 == 0
    # a padding sequence longer than the context the graphs are made for: not rounded
    assert make_runner(max_seq_len=32)._rounded_shape([30] * 9, 1, 32) is None      # 50 padding tokens in a row
    assert make_runner()._rounded_shape([2] + [1] * 300, 1, 64) is None             # more sequences than tokens after rounding
    assert make_runner(max_seq_len=64)._rounded_shape([30] * 9, 1, 32) is not None
    assert make_runner(accepts=False)._rounded_shape([2048], 1, 2048) is None


def test_rounding_can_be_switched_off(monkeypatch):
    monkeypatch.setattr(runner_mod, "_ROUNDED_STEP_GRAPHS", False)
    assert make_runner()._rounded_shape([2048], 1, 2048) is None


def test_packed_indices_of_a_padded_batch():
    r = make_runner()
    c = r.cache
    for req, n in (("a", 6), ("b", 3)):
        c.admit(req)
        c.grow(req, n)
    c.advance("a", 2)   # "a" already holds two tokens
    group = next(iter(c.groups.values()))
    spare_page, spare_slot = group.num_pages, c.spare_slot
    seqs = [(np.array([5, 6, 7, 8]), 2, c.slot("a"), "a"), (np.array([9, 10, 11]), 0, c.slot("b"), "b"),
            (np.zeros(5, dtype=np.int32), 0, spare_slot, None), (np.zeros(0, dtype=np.int32), 0, spare_slot, None)]
    rows = [3, 6, 3, 3]
    total, fill, context = r._layout(seqs, rows, [group], [5], 16, LengthBounds(12, 4))
    buf = np.full(total, -7, dtype=np.int32)
    fill(buf)
    T = 12
    assert buf[:T].tolist() == [5, 6, 7, 8, 9, 10, 11, 0, 0, 0, 0, 0]
    assert buf[T:2 * T].tolist() == [2, 3, 4, 5, 0, 1, 2, 0, 1, 2, 3, 4]           # positions
    assert buf[2 * T:3 * T].tolist() == [0] * 4 + [1] * 3 + [2] * 5                  # sequence of each token
    assert buf[3 * T:3 * T + 5].tolist() == [0, 4, 7, 12, 12]                         # token offsets: the last is empty
    assert buf[3 * T + 5:3 * T + 9].tolist() == [c.slot("a"), c.slot("b"), spare_slot, spare_slot]
    assert buf[3 * T + 9:3 * T + 13].tolist() == rows
    tab = buf[3 * T + 13:].reshape(4, 5)
    assert tab[0, :2].tolist() == c.block_table("a", group.key) and tab[1, :1].tolist() == c.block_table("b", group.key)
    assert (tab[0, 2:] == spare_page).all() and (tab[1, 1:] == spare_page).all() and (tab[2:] == spare_page).all()
    assert total == 3 * T + 13 + 20 and not (buf == -7).any()
    ctx, tables = context(torch.from_numpy(buf), workspace=None)
    assert ctx.n_tokens == 12 and ctx.n_seq == 4 and ctx.n_rows == 4 and not ctx.decode_only
    assert list(ctx.new_lens) == [9, 1, 1, 1] and ctx.new_lens.multi == 4 and ctx.past_lens == [2, 0, 0, 0]
    assert tables[group.key].shape == (4, 5) and ctx.kv_len_bound == 16


def comings(r, shapes, exact_key, rounded_key):
    """What the runner does with a step: 'replay', 'record' (then replay) or 'issue' (launch by launch),
    and in which form; keeps the runner's counters and ``shapes`` as the runner would."""
    key, padded, record = r._choose_form(shapes, exact_key, rounded_key)
    form = "padded" if padded else "exact"
    if key is not None and key in shapes:
        return "replay", form, key
    if record:
        shapes[key] = {"graph": object()}
        return "record", form, key
    r._note_issued(key, exact_key, padded)
    return "issue", form, key


def test_which_form_a_step_takes_as_shapes_recur():
    r = make_runner()
    r._shape_seen = {}
    R = ("rounded", 512, 4, 4, 256)
    shapes = {}
    cuts = [((200 + i, 150 - i, 100), 3, 256) for i in range(6)]
    # ever new cuts of one rounded shape: as it is, then padded, then recorded, then replayed
    got = [comings(r, shapes, e, R)[:2] for e in cuts]
    assert got == [("issue", "exact"), ("issue", "padded"), ("record", "padded")] + [("replay", "padded")] * 3
    # one cut that keeps coming while the rounded recording exists: replayed padded twice, then
    # issued once as it is, then recorded as it is and replayed from its own recording
    same = ((180, 170, 100), 3, 256)
    got = [comings(r, shapes, same, R) for _ in range(6)]
    assert [g[:2] for g in got] == [("replay", "padded")] * 2 + [("issue", "exact"), ("record", "exact"),
                                                                 ("replay", "exact"), ("replay", "exact")]
    assert got[-1][2] == same and set(shapes) == {R, same}
    # a shape that nothing rounds (a short step, or parts that want the true lengths): second time recorded
    short = ((20, 20), 2, 64)
    assert [comings(r, shapes, short, None)[0] for _ in range(3)] == ["issue", "record", "replay"]
    # one exact shape from the start (a benchmark): exact, padded, then its own recording
    r2, shapes2 = make_runner(), {}
    r2._shape_seen = {}
    bench = ((2048,), 1, 2048)
    R2 = ("rounded", 2112, 2, 1, 2048)
    got = [comings(r2, shapes2, bench, R2)[:2] for _ in range(4)]
    assert got == [("issue", "exact"), ("issue", "padded"), ("record", "exact"), ("replay", "exact")]
    # no graphs at all (key None): always issued
    assert comings(r2, shapes2, None, None) == ("issue", "exact", None)


def test_rounding_at_the_schedulers_budget():
    """With the scheduler's token budget known, steps within 64 tokens of it round to multiples of
    64 and all others to multiples of 256, whatever came before."""
    r = make_runner()
    r.token_budget = 2048
    assert r._rounded_shape([8000, 192], 1, 4096)[0][1] == 8192        # a step far above the budget changes nothing below
    assert r._rounded_shape([1500, 540, 1, 1, 1, 1, 1, 1], 8, 2048)[0][:3] == ("rounded", 2048, 16)
    assert r._rounded_shape([1990], 1, 2048)[0][1] == 2048
    assert r._rounded_shape([1900, 1], 1, 2048)[0][1] == 2048          # 1,901 -> 1,920 -> 2,048
    assert r._rounded_shape([1000, 1], 1, 1024)[0][1] == 1024
    assert r._rounded_shape([1000, 30], 1, 1024)[0][1] == 1280
    assert r._rounded_shape([40, 1], 1, 64)[0][1] == 256
