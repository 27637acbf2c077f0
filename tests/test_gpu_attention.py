"""The attention kernels alone against a plain float64 reference over a paged cache
with shuffled pages: head sizes from 16 to 256, any number of heads and groups,
windows, mixed batches, split keys; and inputs built so that a single far key, a
window's edge or a page's edge decides the result."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


class Batch:
    """A paged cache filled with random keys/values and a step over it."""

    def __init__(self, dtype, heads, kv, hd, page, before, new, seed=0, q_scale=1.0):
        g = torch.Generator().manual_seed(seed)
        self.heads, self.kv, self.hd, self.page = heads, kv, hd, page
        r = len(before)
        total = [b + n for b, n in zip(before, new)]
        max_pages = max(-(-t // page) for t in total) + 1
        n_pages = r * max_pages + 3
        perm = torch.randperm(n_pages, generator=g)[:r * max_pages].reshape(r, max_pages)
        self.table = perm.to(torch.int32).to(DEV)
        # stale content everywhere (large values): only positions < total may be read
        self.kp = (torch.randn(n_pages, kv, page, hd, generator=g) * 50).to(dtype).to(DEV)
        self.vp = (torch.randn(n_pages, kv, page, hd, generator=g) * 50).to(dtype).to(DEV)
        self.k = [torch.randn(t, kv, hd, generator=g).to(dtype) for t in total]
        self.v = [torch.randn(t, kv, hd, generator=g).to(dtype) for t in total]
        for i in range(r):
            for first in range(0, total[i], page):                 # a page at a time
                pg, m = int(perm[i, first // page]), min(page, total[i] - first)
                self.kp[pg, :, :m] = self.k[i][first:first + m].transpose(0, 1).to(DEV)
                self.vp[pg, :, :m] = self.v[i][first:first + m].transpose(0, 1).to(DEV)
        n = sum(new)
        self.q = (torch.randn(n, heads * hd, generator=g) * q_scale).to(dtype).to(DEV)
        cu = np.concatenate([[0], np.cumsum(new)])
        self.n, self.r, self.before, self.new = n, r, before, new
        self.max_new, self.max_context = max(new), max(total)
        i32 = lambda x: torch.tensor(np.asarray(x), dtype=torch.int32, device=DEV)
        self.cu_tokens, self.slots, self.context_before = i32(cu), i32(np.arange(r)), i32(before)
        self.positions = i32(np.concatenate([np.arange(b, b + k) for b, k in zip(before, new)]))
        self.slot_of_token = i32(np.concatenate([np.full(k, i) for i, k in enumerate(new)]))
        self.attention_splits = None

    def reference(self, scale, window=0):
        out = torch.zeros(self.n, self.heads, self.hd, dtype=torch.float64)
        q = self.q.double().cpu().reshape(self.n, self.heads, self.hd)
        group = self.heads // self.kv
        at = 0
        for i in range(self.r):
            k, v = self.k[i].double(), self.v[i].double()
            for t in range(self.new[i]):
                pos = self.before[i] + t
                lo = max(0, pos + 1 - window) if window else 0
                for h in range(self.heads):
                    s = (k[lo:pos + 1, h // group] @ q[at, h]) * scale
                    p = torch.softmax(s, 0)
                    out[at, h] = p @ v[lo:pos + 1, h // group]
                at += 1
        return out.reshape(self.n, -1)


def _err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / ref.abs().max())


CASES = [  # heads, kv, hd, page, before, new
    (4, 2, 16, 16, [0, 3, 40], [5, 1, 17]),
    (3, 1, 32, 16, [0, 100, 7, 63], [33, 1, 1, 2]),
    (8, 8, 64, 64, [0, 64, 200], [64, 1, 9]),
    (32, 8, 64, 64, [300, 511], [1, 1]),
    (6, 2, 128, 32, [5, 0], [20, 70]),
    (5, 5, 48, 16, [17], [30]),
    (2, 1, 256, 16, [10, 0], [1, 19]),
    (14, 2, 80, 32, [90], [3]),
]


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("window", [0, 24])
def test_attention_simt_float32(case, window):
    from hfee_b200.kernels import ops
    heads, kv, hd, page, before, new = case
    b = Batch(torch.float32, heads, kv, hd, page, before, new)
    out = torch.empty_like(b.q)
    scale = 1 / math.sqrt(hd)
    ops.attention_simt(b.q, b.kp, b.vp, b.table, page, b.positions, b.slot_of_token, out, heads, kv, hd, scale, window)
    assert _err(out, b.reference(scale, window)) < 2e-5


@pytest.mark.parametrize("case", CASES)
@pytest.mark.parametrize("window", [0, 24])
def test_attention_bfloat16_both_kernels(case, window):
    from hfee_b200.kernels import ops
    heads, kv, hd, page, before, new = case
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, new)
    scale = 1 / math.sqrt(hd)
    ref = b.reference(scale, window)
    out = torch.empty_like(b.q)
    ops.attention_simt(b.q, b.kp, b.vp, b.table, page, b.positions, b.slot_of_token, out, heads, kv, hd, scale, window)
    assert _err(out, ref) < 1e-2
    out2 = torch.full_like(b.q, float("nan"))
    ops.paged_attention(b.q, b.kp, b.vp, b.table, page, b.positions, b.slot_of_token, out2, heads, kv, hd, scale,
                        window, step=b)
    assert _err(out2, ref) < 1e-2


@pytest.mark.parametrize("heads,kv,hd,page", [(32, 8, 64, 64), (4, 1, 128, 16), (3, 3, 32, 16), (16, 1, 16, 32)])
@pytest.mark.parametrize("splits", [2, 5, 32])
def test_attention_split_keys(heads, kv, hd, page, splits):
    """Decode step with the keys of each request divided among CTAs, contexts from 1 to 1500."""
    from hfee_b200.kernels import ops
    before = [0, 63, 64, 1499, 700, 255]
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, [1] * len(before), seed=3)
    scale = 1 / math.sqrt(hd)
    scratch = torch.full((b.n * heads * splits * (hd + 2),), float("nan"), dtype=torch.float32, device=DEV)
    out = torch.full_like(b.q, float("nan"))
    ops.attention_mma(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r, 1,
                      heads, kv, hd, scale, 0, splits, scratch)
    assert _err(out, b.reference(scale)) < 1e-2


@pytest.mark.parametrize("batch", [1, 8, 64])
@pytest.mark.parametrize("heads,kv,hd", [(32, 8, 64), (8, 2, 128)])
def test_decode_at_the_contexts_and_splits_of_the_benchmark(batch, heads, kv, hd):
    """Decode steps at the context lengths the benchmark and long generations reach (a page's and a
    block's edge at 2,048 and 4,096; 8,191) with the number of key splits the dispatcher picks for
    batches of 1, 8 and 64, through the fused rotary kernel and through the plain one."""
    from hfee_b200.kernels import ops
    page = 64
    contexts = [2047, 2048, 4095, 4096, 8191]
    shown = min(batch, len(contexts))            # requests whose rows are checked; the dispatcher plans for `batch`
    before = contexts[:shown]
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, [1] * shown, seed=batch + hd)
    scale = 1 / math.sqrt(hd)
    ref = b.reference(scale)
    for planned in (max(before) + 1, 8192):     # planned for the longest context now, or for the engine's limit
        splits = ops.attention_splits(batch, kv, planned)
        assert 1 <= splits <= ops.MAX_SPLITS
        scratch = torch.full((b.n * heads * splits * (hd + 2),), float("nan"), dtype=torch.float32, device=DEV)
        out = torch.full_like(b.q, float("nan"))
        ops.attention_mma(b.q, b.kp, b.vp, b.table, page, b.cu_tokens, b.slots, b.context_before, out, b.n, b.r, 1,
                          heads, kv, hd, scale, 0, splits, scratch)
        assert _err(out, ref) < 1e-2, (splits, planned)
        # the fused kernel: no rotation (rope_dim 0), so its queries are the rows above and the new key and
        # value are the ones already in the cache; it rewrites them in place
        qkv = torch.cat([b.q, torch.stack([b.k[i][-1].reshape(-1) for i in range(b.r)]).to(DEV),
                         torch.stack([b.v[i][-1].reshape(-1) for i in range(b.r)]).to(DEV)], dim=1).contiguous()
        b.attention_splits = splits
        got = torch.full_like(b.q, float("nan"))
        kp, vp = b.kp.clone(), b.vp.clone()
        ops.paged_attention_rope(qkv, None, 0, False, True, kp, vp, b.table, page, got, heads, kv, hd, scale, 0, b,
                                 scratch if splits > 1 else None)
        assert torch.equal(got, out) and torch.equal(kp, b.kp) and torch.equal(vp, b.vp)
    b.attention_splits = None


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_one_far_key_decides(dtype):
    """Among 900 keys one early key (position 3, first page) matches the query exactly and is
    scaled up: the output must be that key's value, so a kernel that skips or misplaces a far
    page shows."""
    from hfee_b200.kernels import ops
    heads, kv, hd, page = 4, 2, 64, 16
    b = Batch(dtype, heads, kv, hd, page, [899], [1], seed=5, q_scale=0.05)
    q = b.q.reshape(1, heads, hd)
    for h in range(heads):
        key = (q[0, h].float() / q[0, h].float().norm() * 60).to(dtype)       # score ~ 60*|q|*sqrt... dominates
        pg = int(b.table[0, 3 // page])
        b.kp[pg, h // 2, 3 % page] = key
        b.k[0][3, h // 2] = key.cpu()
    b.q = (q * 40).reshape(1, -1).contiguous()
    scale = 1 / math.sqrt(hd)
    ref = b.reference(scale)
    out = torch.empty_like(b.q)
    ops.paged_attention(b.q, b.kp, b.vp, b.table, page, b.positions, b.slot_of_token, out, heads, kv, hd, scale, 0,
                        step=b if dtype == torch.bfloat16 else None)
    # kv head 1 is shared by heads 2 and 3, whose planted keys overwrite each other: check heads 1 and 3
    for h in (1, 3):
        want = b.v[0][3, h // 2].double()
        got = out.double().cpu().reshape(heads, hd)[h]
        assert float((got - want).abs().max()) < (1e-3 if dtype == torch.float32 else 3e-2)
    assert _err(out, ref) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_edge_decides(dtype):
    """The key just outside the window would dominate if it were read; the key just inside must be."""
    from hfee_b200.kernels import ops
    heads, kv, hd, page, window = 2, 1, 32, 16, 40
    pos = 200
    b = Batch(dtype, heads, kv, hd, page, [pos], [1], seed=6, q_scale=0.05)
    q = b.q.reshape(heads, hd).float()
    outside, inside = pos - window, pos - window + 1
    for p_, gain in ((outside, 80.0), (inside, 40.0)):
        key = (q[0] / q[0].norm() * gain).to(dtype)
        b.kp[int(b.table[0, p_ // page]), 0, p_ % page] = key
        b.k[0][p_, 0] = key.cpu()
    b.q = (b.q * 40).contiguous()
    scale = 1 / math.sqrt(hd)
    out = torch.empty_like(b.q)
    ops.paged_attention(b.q, b.kp, b.vp, b.table, page, b.positions, b.slot_of_token, out, heads, kv, hd, scale,
                        window, step=b if dtype == torch.bfloat16 else None)
    got = out.double().cpu().reshape(heads, hd)[0]
    assert float((got - b.v[0][inside, 0].double()).abs().max()) < (1e-3 if dtype == torch.float32 else 3e-2)
    assert _err(out, b.reference(scale, window)) < (2e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("heads,kv,hd,page,rope_dim,interleaved", [
    (32, 8, 64, 64, 64, False), (4, 1, 128, 16, 64, False), (3, 3, 32, 16, 32, True), (16, 1, 16, 32, 16, False),
    (6, 2, 80, 32, 32, True), (8, 2, 64, 64, 0, False)])
@pytest.mark.parametrize("splits", [1, 3])
@pytest.mark.parametrize("window", [0, 40])
def test_decode_attention_with_fused_rotary(heads, kv, hd, page, rope_dim, interleaved, splits, window):
    """One kernel for rotary + cache write + attention of a decode step gives what the rotary kernel
    followed by the attention kernel gives, and leaves the same keys and values in the cache; the new
    token sits at a page's first and last row, at a block's edge and in the middle."""
    from hfee_b200.kernels import ops
    before = [0, 63, 64, 1499, 700, 255, 127, 128]
    b = Batch(torch.bfloat16, heads, kv, hd, page, before, [1] * len(before), seed=11)
    g = torch.Generator().manual_seed(12)
    qkv = torch.randn(b.n, (heads + 2 * kv) * hd, generator=g).to(torch.bfloat16).to(DEV)
    cs = None
    if rope_dim:
        ang = torch.rand(b.n, rope_dim // 2, generator=g, dtype=torch.float64) * 6.28
        cs = torch.stack([torch.cos(ang), torch.sin(ang)], -1).float().contiguous().to(DEV)
    scale = 1 / math.sqrt(hd)
    # two copies of the cache: the new positions hold stale values in both before the step
    kp1, vp1, kp2, vp2 = b.kp.clone(), b.vp.clone(), b.kp.clone(), b.vp.clone()
    q = torch.empty(b.n, heads * hd, dtype=torch.bfloat16, device=DEV)
    ops.rope_cache_write(qkv, cs, b.positions, b.slot_of_token, q, kp1, vp1, b.table, page, heads, kv, hd, rope_dim, interleaved)
    scratch = torch.empty(b.n * heads * max(splits, 1) * (hd + 2), dtype=torch.float32, device=DEV)
    want = torch.full((b.n, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.attention_mma(q, kp1, vp1, b.table, page, b.cu_tokens, b.slots, b.context_before, want, b.n, b.r, 1, heads, kv, hd,
                      scale, window, splits, scratch)
    b.attention_splits = splits
    got = torch.full_like(want, float("nan"))
    assert ops.decode_rope_fusable(b, torch.bfloat16, heads, kv, hd, rope_dim, qkv, scratch)
    ops.paged_attention_rope(qkv, cs, rope_dim, interleaved, True, kp2, vp2, b.table, page, got, heads, kv, hd, scale,
                             window, b, scratch if splits > 1 else None)
    torch.cuda.synchronize()
    assert torch.equal(kp1, kp2) and torch.equal(vp1, vp2)
    assert torch.equal(got, want)
    # a run that only reads the cache (another run wrote the new key): queries rotated, cache untouched
    got2 = torch.full_like(want, float("nan"))
    kp3, vp3 = kp1.clone(), vp1.clone()
    ops.paged_attention_rope(qkv[:, :heads * hd], cs, rope_dim, interleaved, False, kp3, vp3, b.table, page, got2, heads,
                             kv, hd, scale, window, b, scratch if splits > 1 else None)
    assert torch.equal(got2, want) and torch.equal(kp3, kp1) and torch.equal(vp3, vp1)
