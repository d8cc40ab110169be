"""How the attention part cuts the keys of a step into ranges (host-side decisions, no GPU):
enough blocks to fill the GPU when few tokens are in flight, one range when the tokens alone do,
ranges that are multiples of 64 keys and cover the whole context."""
import pytest
import torch


def _attention(hidden, heads, kv_heads, head_dim):
    from poor_mans_mamba_b200.parts.attention import PagedAttention
    return PagedAttention(hidden, heads, kv_heads, head_dim)


@pytest.mark.parametrize("batch,bound", [(1, 4160), (8, 4160), (64, 4160), (8, 320), (8, 32832), (3, 100)])
@pytest.mark.parametrize("shape", [(1024, 8, 2, 64), (3072, 12, 2, 128), (96, 3, 1, 32)])
def test_decode_ranges_cover_the_context(shape, batch, bound):
    a = _attention(*shape)
    n, length = a.plan_splits([1] * batch, bound, torch.bfloat16)
    assert 1 <= n <= 64
    if n == 1:
        assert length == 0
    else:
        assert length % 64 == 0 and n * length >= bound and (n - 1) * length < bound


def test_decode_ranges_follow_what_an_sm_holds():
    """Head size 64: about two blocks per SM; head size 128 (a block fills an SM's shared memory):
    one.  Many requests need fewer ranges than few."""
    small, large = _attention(1024, 8, 2, 64), _attention(3072, 12, 2, 128)
    n64, _ = small.plan_splits([1] * 8, 4160, torch.bfloat16)
    n128, _ = large.plan_splits([1] * 8, 4160, torch.bfloat16)
    assert 148 < n64 * 8 * 2 <= 2 * 148 and n128 * 8 * 2 <= 148 < 2 * n128 * 8 * 2
    assert small.plan_splits([1] * 64, 4160, torch.bfloat16)[0] < n64
    assert small.plan_splits([1] * 8, 200, torch.bfloat16) == (1, 0)   # nothing to cut below 256 keys


def test_prompt_ranges():
    a = _attention(1024, 8, 2, 64)
    assert a.plan_splits_tc([2048], 2048) == (1, 0)                 # 128 row tiles: a block per SM already
    n, length = a.plan_splits_tc([256], 8192)                         # few rows, long context: cut the keys
    assert n > 1 and length % 64 == 0 and n * length >= 8192
    assert a.plan_splits([8192], 8192, torch.bfloat16) == (1, 0)
