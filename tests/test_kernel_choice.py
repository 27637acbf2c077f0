"""Host-side rules that pick a kernel variant or a launch shape (no GPU needed)."""
import pytest

from hfee_b200.kernels import ops


@pytest.mark.parametrize("sms", [148, 132, 20])
@pytest.mark.parametrize("kv_heads", [1, 2, 8, 5])
def test_key_splits_stay_within_what_the_kernels_take(kv_heads, sms):
    for requests in (1, 2, 3, 8, 9, 12, 16, 64, 500):
        last = None
        for context in (1, 63, 128, 255, 256, 2048, 8192, 1 << 17):
            s = ops.attention_splits(requests, kv_heads, context, sms)
            assert 1 <= s <= ops.MAX_SPLITS
            # a split holds at least two key blocks of 64, and short contexts are not split at all
            assert s == 1 or s * 128 <= context
            # a longer context never gets fewer splits
            assert last is None or s >= last
            last = s


@pytest.mark.parametrize("sms", [148, 132])
def test_key_splits_fill_the_gpu_about_once(sms):
    # batch 8 with 8 kv heads and a long context: about four CTAs per SM in all, whatever the number of SMs
    s = ops.attention_splits(8, 8, 32768, sms)
    assert 3 * sms < s * 64 <= 4 * sms
    # a batch that fills the GPU by itself is still split in four
    assert ops.attention_splits(64, 8, 2048, sms) == 4
    # few (request, kv head) pairs: about two CTAs per SM (those grids run the kernel variant of which an SM holds one)
    for r in (3, 4, 6):
        s = ops.attention_splits(r, 8, 32768, sms)
        assert sms < s * r * 8 <= 2 * sms
    # within either rule more requests never get more splits each
    few = [ops.attention_splits(r, 8, 1 << 16, sms) for r in range(1, ops.FEW_PAIRS // 8 + 1)]
    many = [ops.attention_splits(r, 8, 1 << 16, sms) for r in range(ops.FEW_PAIRS // 8 + 1, 80)]
    assert all(a >= b for a, b in zip(few, few[1:])) and all(a >= b for a, b in zip(many, many[1:]))
