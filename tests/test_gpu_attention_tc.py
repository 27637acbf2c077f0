"""The tcgen05 prefill attention alone against the float64 reference over a paged cache with
shuffled pages and large stale values: groups that do and do not divide the tile, contexts that
end inside a page, windows, several requests, portions that continue a context."""
import math

import pytest
import torch

from test_gpu_attention import Batch, _err

pytestmark = pytest.mark.gpu

CASES = [  # heads, kv, page, before, new
    (4, 1, 64, [0], [128]),
    (4, 1, 64, [0], [37]),
    (32, 8, 64, [0], [300]),
    (32, 8, 64, [200, 0, 63], [130, 64, 5]),
    (8, 8, 128, [0, 500], [260, 40]),
    (6, 2, 64, [100], [129]),          # 3 query heads per kv head: 42 tokens x 3 = 126 rows per tile
    (5, 1, 64, [0, 7], [70, 33]),
    (64, 1, 256, [0], [17]),           # two tokens per tile
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("window", [0, 150])
def test_attention_tc(case, window):
    from hfee_b200.kernels import ops
    heads, kv, page, before, new = case
    hd = 64
    assert ops.attention_tc_supports(heads, kv, hd, page)
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, new, seed=sum(new) + heads)
    scale = 1 / math.sqrt(hd)
    out = torch.full_like(b.q, float("nan"))
    ops.attention_tc(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r,
                     b.max_new, heads, kv, hd, scale, window)
    ops.check_status()
    assert not torch.isnan(out.float()).any()
    assert _err(out, b.reference(scale, window)) < 1e-2


def test_refuses_other_head_sizes():
    from hfee_b200.kernels import ops
    assert not ops.attention_tc_supports(8, 2, 128, 64)
    assert not ops.attention_tc_supports(8, 2, 64, 16)
    assert not ops.attention_tc_supports(8, 3, 64, 64)
