"""The tcgen05 prefill attention alone against the float64 reference over a paged cache with
shuffled pages and large stale values: head sizes 64 and 128, groups that do and do not divide
the tile, contexts that end inside a page, windows, several requests, portions that continue a
context; scores that grow block after block (the kept row maximum has to move); pages whose
unused rows hold NaN."""
import math

import pytest
import torch

from test_gpu_attention import Batch, _err

pytestmark = pytest.mark.gpu

CASES = [  # heads, kv, hd, page, before, new
    (4, 1, 64, 64, [0], [128]),
    (4, 1, 64, 64, [0], [37]),
    (32, 8, 64, 64, [0], [300]),
    (32, 8, 64, 64, [200, 0, 63], [130, 64, 5]),
    (8, 8, 64, 128, [0, 500], [260, 40]),
    (6, 2, 64, 64, [100], [129]),          # 3 query heads per kv head: 42 tokens x 3 = 126 rows per tile
    (5, 1, 64, 64, [0, 7], [70, 33]),
    (64, 1, 64, 256, [0], [17]),           # two tokens per tile
    (32, 8, 128, 64, [0], [300]),          # the 8B shape's heads
    (8, 2, 128, 64, [200, 0, 63], [130, 64, 5]),
    (5, 5, 128, 64, [0, 300], [520, 129]),  # one query head per kv head (the 13B shape's grouping): 128 tokens per tile
    (6, 2, 128, 128, [100], [129]),
    (3, 1, 128, 256, [0, 7], [70, 33]),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("window", [0, 150])
def test_attention_tc(case, window):
    from hfee_b200.kernels import ops
    heads, kv, hd, page, before, new = case
    assert ops.attention_tc_supports(heads, kv, hd, page)
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, new, seed=sum(new) + heads)
    scale = 1 / math.sqrt(hd)
    out = torch.full_like(b.q, float("nan"))
    ops.attention_tc(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r,
                     b.max_new, heads, kv, hd, scale, window)
    ops.check_status()
    assert not torch.isnan(out.float()).any()
    assert _err(out, b.reference(scale, window)) < 1e-2


@pytest.mark.parametrize("hd", [64, 128])
def test_scores_that_grow_with_the_position(hd):
    """Keys are scaled up with their position, so every key block raises the row maxima by far more
    than the kernel tolerates without moving them: the outputs kept in tensor memory have to be
    rescaled block after block, and the last keys decide the result."""
    from hfee_b200.kernels import ops
    heads, kv, page = 8, 2, 64
    b = Batch(torch.bfloat16, heads, kv, hd, page, [100], [700], seed=11)
    pos = torch.arange(800, dtype=torch.float32)
    grow = (1 + pos / 40).reshape(-1, 1, 1)
    b.k[0] = (b.k[0].float().abs() * grow).to(torch.bfloat16)          # all scores of a positive query grow
    b.q = b.q.float().abs().to(torch.bfloat16)
    for p in range(800):
        b.kp[int(b.table[0, p // page]), :, p % page] = b.k[0][p].to(b.kp.device)
    scale = 1 / math.sqrt(hd)
    out = torch.full_like(b.q, float("nan"))
    ops.attention_tc(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r,
                     b.max_new, heads, kv, hd, scale, 0)
    ops.check_status()
    assert _err(out, b.reference(scale, 0)) < 1e-2


@pytest.mark.parametrize("hd", [64, 128])
@pytest.mark.parametrize("new", [5, 70, 200])
def test_nan_left_in_a_page_by_an_earlier_owner(hd, new):
    """Every row of every page that the requests do not hold (behind their last position, and in
    pages of nobody) is NaN: a kernel that lets a masked row reach an MMA shows it."""
    from hfee_b200.kernels import ops
    heads, kv, page = 8, 2, 64
    before = [130, 0]
    news = [new, new + 3]
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, news, seed=new)
    b.kp[:] = float("nan")
    b.vp[:] = float("nan")
    for i in range(b.r):
        for p in range(before[i] + news[i]):
            pg = int(b.table[i, p // page])
            b.kp[pg, :, p % page] = b.k[i][p].to(b.kp.device)
            b.vp[pg, :, p % page] = b.v[i][p].to(b.vp.device)
    scale = 1 / math.sqrt(hd)
    out = torch.full_like(b.q, float("nan"))
    ops.attention_tc(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r,
                     b.max_new, heads, kv, hd, scale, 0)
    ops.check_status()
    assert not torch.isnan(out.float()).any()
    assert _err(out, b.reference(scale, 0)) < 1e-2


def test_refuses_other_shapes():
    from hfee_b200.kernels import ops
    assert ops.attention_tc_supports(32, 8, 128, 64)
    assert ops.attention_tc_supports(40, 40, 128, 64)
    assert not ops.attention_tc_supports(8, 2, 96, 64)
    assert not ops.attention_tc_supports(8, 2, 64, 16)
    assert not ops.attention_tc_supports(8, 3, 64, 64)
