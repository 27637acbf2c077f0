"""Each CUDA kernel alone against a plain float32/float64 torch reference, at sizes
other than the engine's (odd widths, tails, head sizes from 16 to 256)."""
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from hfee_b200.kernels import ops as o
    o.library()
    return o


def _close(got, ref, tol):
    got, ref = got.double().cpu(), ref.double().cpu()
    err = float((got - ref).abs().max() / (ref.abs().max() + 1e-30))
    assert err < tol, f"relative error {err:.3g} >= {tol}"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,vocab", [(1, 7, 11), (33, 100, 57), (5, 2048, 300)])
def test_embed(ops, dtype, n, width, vocab):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(vocab, width, generator=g).to(dtype).to(DEV)
    tokens = torch.randint(0, vocab, (n,), generator=g, dtype=torch.int32).to(DEV)
    out = torch.empty(n, width, dtype=torch.float32, device=DEV)
    ops.embed(table, tokens, out)
    assert torch.equal(out, table[tokens.long()].float())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,width,eps", [(1, 1, 1e-5), (3, 97, 1e-6), (17, 2048, 1e-5), (4, 5000, 1e-3),
                                         (300, 2048, 1e-5), (259, 1004, 1e-6), (1000, 4096, 1e-5), (257, 5120, 1e-5)])
def test_rmsnorm(ops, out_dtype, n, width, eps):
    """From 256 rows on the bfloat16 output takes the warp-per-row kernel (rows of up to 4,096 values)."""
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(n + 2, width, generator=g) * 3).to(DEV)
    w = (1 + 0.1 * torch.randn(width, generator=g)).to(DEV)
    rows = torch.tensor([(i * 2 + 1) % (n + 2) for i in range(n)], dtype=torch.int32, device=DEV)
    for idx in (None, rows):
        out = torch.empty(n, width, dtype=out_dtype, device=DEV)
        ops.rmsnorm(x, w, out, eps, rows=idx)
        src = (x[:n] if idx is None else x[idx.long()]).double()
        ref = src / torch.sqrt((src * src).mean(1, keepdim=True) + eps) * w.double()
        _close(out, ref, 1e-5 if out_dtype == torch.float32 else 6e-3)
    src = x[:n].double()
    for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 6e-3)):
        out = torch.empty(n, width, dtype=dt, device=DEV)
        ops.rmsnorm(x, w, out, eps, add_unit=True)
        _close(out, src / torch.sqrt((src * src).mean(1, keepdim=True) + eps) * (1 + w.double()), tol)


def test_rope_table_far_positions(ops):
    """float64 angles: a position of 100000 keeps cos/sin right to float32 rounding."""
    pos = torch.tensor([0, 1, 63, 64, 4097, 100000, 131071], dtype=torch.int32, device=DEV)
    inv = torch.tensor([1.0 / (500000.0 ** (2 * i / 64)) for i in range(32)], dtype=torch.float64, device=DEV)
    out = torch.empty(len(pos), 32, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(pos, inv, out)
    ang = pos.double()[:, None] * inv[None, :]
    assert float((out[..., 0].double() - ang.cos()).abs().max()) < 1e-7
    assert float((out[..., 1].double() - ang.sin()).abs().max()) < 1e-7


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv,hd,rope_dim,inter", [(4, 2, 16, 16, False), (3, 1, 32, 32, True),
                                                         (2, 2, 48, 16, False), (5, 5, 64, 32, True),
                                                         (2, 1, 24, 8, False), (3, 1, 20, 12, True),   # not 16-byte pieces
                                                         (32, 8, 64, 64, False), (8, 2, 128, 64, False)])
def test_rope_cache_write(ops, dtype, heads, kv, hd, rope_dim, inter):
    g = torch.Generator().manual_seed(2)
    n, page, max_pages, slots = 23, 16, 4, 3
    qkv = torch.randn(n, (heads + 2 * kv) * hd, generator=g).to(dtype).to(DEV)
    slot = torch.randint(0, slots, (n,), generator=g, dtype=torch.int32)
    pos = torch.zeros(n, dtype=torch.int32)
    seen = {}
    for i in range(n):                       # distinct (slot, position) pairs
        s = int(slot[i]); seen[s] = seen.get(s, 5) + 1; pos[i] = seen[s] * 2
    table = torch.randperm(slots * max_pages, generator=g).reshape(slots, max_pages).to(torch.int32).to(DEV)
    kp = torch.zeros(slots * max_pages, kv, page, hd, dtype=dtype, device=DEV)
    vp = torch.zeros_like(kp)
    q = torch.empty(n, heads * hd, dtype=dtype, device=DEV)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * i / rope_dim)) for i in range(rope_dim // 2)], dtype=torch.float64, device=DEV)
    cs = torch.empty(n, rope_dim // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(pos.to(DEV), inv, cs)
    ops.rope_cache_write(qkv, cs, pos.to(DEV), slot.to(DEV), q, kp, vp, table, page, heads, kv, hd, rope_dim, inter)

    x = qkv.double().cpu().reshape(n, heads + 2 * kv, hd)
    ang = pos.double()[:, None] * inv.cpu()[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    rot = x[:, :heads + kv].clone()
    half = rope_dim // 2
    if inter:
        a, b = x[:, :heads + kv, 0:rope_dim:2], x[:, :heads + kv, 1:rope_dim:2]
        rot[..., 0:rope_dim:2], rot[..., 1:rope_dim:2] = a * c - b * s, a * s + b * c
    else:
        a, b = x[:, :heads + kv, :half], x[:, :heads + kv, half:rope_dim]
        rot[..., :half], rot[..., half:rope_dim] = a * c - b * s, a * s + b * c
    tol = 1e-6 if dtype == torch.float32 else 6e-3
    _close(q, rot[:, :heads].reshape(n, -1), tol)
    for i in range(n):
        pg = int(table[int(slot[i]), int(pos[i]) // page])
        _close(kp[pg, :, int(pos[i]) % page], rot[i, heads:], tol)
        assert torch.equal(vp[pg, :, int(pos[i]) % page].cpu().double(), x[i, heads + kv:])
    written = sum(1 for _ in range(n))
    assert int((kp.float().abs().sum(-1) > 0).sum()) == written * kv       # nothing else was touched


@pytest.mark.parametrize("heads,kv,hd,inter,n,k,page", [(4, 2, 64, False, 200, 256, 16), (3, 1, 128, False, 130, 192, 64),
                                                       (5, 5, 64, True, 129, 64, 16), (2, 1, 128, True, 300, 320, 32),
                                                       (32, 8, 64, False, 2048, 2048, 64), (6, 2, 64, False, 1100, 520, 64),
                                                       # enough tiles of 256 x 256 for the pairs of CTAs to take over
                                                       (32, 8, 128, False, 2048, 256, 64), (40, 40, 128, True, 600, 192, 64),
                                                       (48, 16, 64, False, 1500, 128, 32),
                                                       # 224 single-CTA tiles of three heads (192 columns) in two rounds
                                                       (32, 8, 64, False, 1792, 128, 64)])
@pytest.mark.parametrize("with_cache", [True, False])
def test_qkv_product_with_rotation_and_cache_write_in_its_epilogue(ops, heads, kv, hd, inter, n, k, page, with_cache):
    """Token rows that do not fill the last tile of 128, head counts that do not fill the last tile of
    256 columns, several requests whose tokens lie on pages in shuffled order; with the pools, and for a
    run that only needs the queries."""
    g = torch.Generator().manual_seed(23)
    slots = 3
    per = -(-n // slots)
    max_pages = -(-(per + 7) // page) + 1
    cols = (heads + 2 * kv) * hd if with_cache else heads * hd
    a = (torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    w = (torch.randn(cols, k, generator=g) * (1.0 / k ** 0.5)).to(torch.bfloat16).to(DEV)
    slot = (torch.arange(n) % slots).to(torch.int32)
    pos = (torch.arange(n) // slots + 7).to(torch.int32)          # distinct (slot, position) pairs, page edges inside
    table = torch.randperm(slots * max_pages, generator=g).reshape(slots, max_pages).to(torch.int32).to(DEV)
    kp = torch.full((slots * max_pages, kv, page, hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    vp = torch.full_like(kp, float("nan"))
    q = torch.full((n, heads * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
    inv = torch.tensor([1.0 / (10000.0 ** (2 * i / hd)) for i in range(hd // 2)], dtype=torch.float64, device=DEV)
    cs = torch.empty(n, hd // 2, 2, dtype=torch.float32, device=DEV)
    ops.rope_table(pos.to(DEV), inv, cs)
    assert ops.qkv_rope_fusable(torch.bfloat16, n, w, hd, hd, cs, q)
    ops.linear_rope_cache(a, w, cs, pos.to(DEV), slot.to(DEV), q, kp if with_cache else None, vp if with_cache else None,
                          table, page, heads, kv, hd, inter)
    ops.check_status()

    x = (a.double() @ w.double().t()).cpu().reshape(n, -1, hd)
    rotated = heads + kv if with_cache else heads
    ang = pos.double()[:, None] * inv.cpu()[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    rot = x[:, :rotated].clone()
    if inter:
        u, v = x[:, :rotated, 0::2], x[:, :rotated, 1::2]
        rot[..., 0::2], rot[..., 1::2] = u * c - v * s, u * s + v * c
    else:
        u, v = x[:, :rotated, :hd // 2], x[:, :rotated, hd // 2:]
        rot[..., :hd // 2], rot[..., hd // 2:] = u * c - v * s, u * s + v * c
    _close(q, rot[:, :heads].reshape(n, -1), 6e-3)
    if not with_cache:
        assert bool(torch.isnan(kp.float()).all())
        return
    pages = table.cpu()[slot.long(), (pos // page).long()].long()
    in_page = (pos % page).long()
    _close(kp[pages.to(DEV), :, in_page.to(DEV)], rot[:, heads:], 6e-3)
    _close(vp[pages.to(DEV), :, in_page.to(DEV)], x[:, heads + kv:], 6e-3)
    # nothing else was touched
    assert int((~torch.isnan(kp.float()).any(-1)).sum()) == n * kv and int((~torch.isnan(vp.float()).any(-1)).sum()) == n * kv


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,inter,granule", [(3, 172, None), (7, 172, 4), (2, 8192, 4), (1, 5, None)])
def test_swiglu(ops, dtype, n, inter, granule):
    g = torch.Generator().manual_seed(3)
    gu = (torch.randn(n, 2 * inter, generator=g) * 2).to(dtype).to(DEV)
    out = torch.empty(n, inter, dtype=dtype, device=DEV)
    ops.swiglu(gu, out, granule)
    gr = granule or inter
    x = gu.double().reshape(n, inter // gr, 2, gr)
    gate, up = x[:, :, 0].reshape(n, inter), x[:, :, 1].reshape(n, inter)
    _close(out, gate / (1 + torch.exp(-gate)) * up, 1e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (5, 7, 3), (64, 64, 16), (65, 130, 100), (33, 256, 172), (200, 96, 513)])
def test_gemm_simt(ops, dtype, m, n, k):
    g = torch.Generator().manual_seed(4)
    a = torch.randn(m, k, generator=g).to(dtype).to(DEV)
    w = torch.randn(n, k, generator=g).to(dtype).to(DEV)
    ref = a.double() @ w.double().t()
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemm_simt(a, w, out)
    _close(out, ref, 1e-5)
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_simt(a, w, acc, accumulate=True)
    _close(acc, base.double() + ref, 1e-5)
    if dtype == torch.bfloat16:
        outb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
        ops.gemm_simt(a, w, outb)
        _close(outb, ref, 6e-3)


def test_gemm_simt_rows_do_not_depend_on_batch(ops):
    g = torch.Generator().manual_seed(5)
    a = torch.randn(70, 333, generator=g).to(DEV)
    w = torch.randn(129, 333, generator=g).to(DEV)
    full = torch.empty(70, 129, device=DEV)
    ops.gemm_simt(a, w, full)
    one = torch.empty(1, 129, device=DEV)
    ops.gemm_simt(a[41:42], w, one)
    assert torch.equal(one[0], full[41])


@pytest.mark.parametrize("m", [1, 2, 8, 9, 12, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(8, 8), (24, 40), (100, 96), (2048, 2048), (257, 1000), (264, 4104), (20004, 520)])
def test_gemm_stream(ops, m, n, k):
    g = torch.Generator().manual_seed(6)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    ref = a.double() @ w.double().t()
    out = torch.empty(m, n, dtype=torch.float32, device=DEV)
    ops.gemm_stream(a, w, out)
    _close(out, ref, 1e-5)
    outb = torch.empty(m, n, dtype=torch.bfloat16, device=DEV)
    ops.gemm_stream(a, w, outb)
    _close(outb, ref, 6e-3)
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_stream(a, w, acc, ops.EPI_ACCUM)
    _close(acc, base.double() + ref, 1e-5)


@pytest.mark.parametrize("m", [1, 8, 16, 64])
def test_the_head_of_the_benchmark_model(ops, m):
    """The product the benchmark's logits come from: 128,256 rows of 2,048 for 1, 8, 16 and 64 tokens,
    through whatever kernel ``ops.linear`` picks for that many tokens (16,032 row tiles of 8)."""
    g = torch.Generator().manual_seed(60 + m)
    a = torch.randn(m, 2048, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(128256, 2048, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    ref = a.double() @ w.double().t()
    out = torch.full((m, 128256), float("nan"), dtype=torch.float32, device=DEV)
    ops.linear(a, w, out)
    ops.check_status()
    _close(out, ref, 1e-5)
    direct = torch.full((m, 128256), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_stream(a, w, direct)                  # the streaming kernel itself takes up to 64 tokens
    _close(direct, ref, 1e-5)


@pytest.mark.parametrize("m", [1, 8, 9, 16, 20, 64])
@pytest.mark.parametrize("inner,k", [(4, 8), (172, 64), (1000, 96), (8192, 256), (1028, 2048), (10004, 4104)])
def test_gemm_stream_swiglu(ops, m, inner, k):
    g = torch.Generator().manual_seed(7)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inner, k, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([gate.reshape(inner // 4, 4, k), up.reshape(inner // 4, 4, k)], 1).reshape(2 * inner, k).contiguous().to(DEV)
    out = torch.empty(m, inner, dtype=torch.bfloat16, device=DEV)
    scratch = torch.empty(m, 2 * inner, dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(a, w, out, 4, scratch)
    gd, ud = a.double().cpu() @ gate.double().t(), a.double().cpu() @ up.double().t()
    _close(out, gd / (1 + torch.exp(-gd)) * ud, 6e-3)


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k", [(1, 64), (9, 192), (100, 576), (2048, 2048), (3072, 2048), (257, 4096), (2048, 8192),
                                 (5000, 4160), (20004, 512)])
def test_gemm_ring(ops, m, n, k):
    """Fewer rows than SMs, rows that do not divide among the SMs, a K that is no multiple of a
    stage (512), tokens that stay in shared memory (K <= 4096) and tokens that stream (above)."""
    g = torch.Generator().manual_seed(16)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    ref = a.double() @ w.double().t()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_ring(a, w, out)
    ops.check_status()
    _close(out, ref, 1e-5)
    outb = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_ring(a, w, outb)
    _close(outb, ref, 6e-3)
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_ring(a, w, acc, ops.EPI_ACCUM)
    ops.check_status()
    _close(acc, base.double() + ref, 1e-5)


@pytest.mark.parametrize("m", [1, 5, 8])
@pytest.mark.parametrize("inner,k", [(4, 64), (172, 64), (1000, 192), (8192, 2048), (1028, 4096), (10004, 4160), (300, 8192)])
def test_gemm_ring_swiglu(ops, m, inner, k):
    g = torch.Generator().manual_seed(17)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inner, k, generator=g) * 0.2).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) * 0.2).to(torch.bfloat16)
    w = torch.stack([gate.reshape(inner // 4, 4, k), up.reshape(inner // 4, 4, k)], 1).reshape(2 * inner, k).contiguous().to(DEV)
    gd, ud = a.double().cpu() @ gate.double().t(), a.double().cpu() @ up.double().t()
    ref = gd / (1 + torch.exp(-gd)) * ud
    out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_ring(a, w, out, ops.EPI_SWIGLU)
    ops.check_status()
    _close(out, ref, 6e-3)
    out32 = torch.full((m, inner), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_ring(a, w, out32, ops.EPI_SWIGLU)
    _close(out32, ref, 2e-5)


def test_gemm_ring_refuses_what_it_cannot_do(ops):
    from hfee_b200.kernels import KernelLibraryError
    assert not ops.ring_takes(9, 64, 64, ops.EPI_STORE)            # more than 8 tokens
    assert not ops.ring_takes(2, 64, 96, ops.EPI_STORE)            # K is no multiple of 64
    assert not ops.ring_takes(2, 12, 64, ops.EPI_SWIGLU)           # SwiGLU wants groups of 8 rows
    assert ops.ring_takes(8, 12, 64, ops.EPI_STORE)
    a = torch.zeros(2, 96, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 96, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelLibraryError, match="multiple of 64"):
        ops.gemm_ring(a, w, torch.empty(2, 8, dtype=torch.float32, device=DEV))


def test_gemm_stream_refuses_unaligned(ops):
    from hfee_b200.kernels import KernelLibraryError
    a = torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 12, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelLibraryError, match="multiple of 8"):
        ops.gemm_stream(a, w, torch.empty(2, 8, dtype=torch.float32, device=DEV))
    # the dispatcher falls back to the CUDA-core kernel instead
    out = torch.empty(2, 8, dtype=torch.float32, device=DEV)
    ops.linear(a, w, out)
    assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("m,v", [(1, 5), (3, 257), (4, 128256), (2, 1000)])
def test_sample_greedy_and_temperature(ops, m, v):
    g = torch.Generator().manual_seed(8)
    logits = torch.randn(m, v, generator=g).to(DEV)
    logits[0, v // 2] = logits[0, v - 1] = 9.0          # a tie: the first maximum wins
    out = torch.zeros(m, dtype=torch.int32, device=DEV)
    ops.sample(logits, out)
    assert out.tolist() == [int(torch.argmax(logits[i].cpu())) for i in range(m)]
    assert out[0] == v // 2
    out2 = torch.full((m,), -1, dtype=torch.int32, device=DEV)
    ops.argmax(logits, out2, torch.empty(m * ops.ARGMAX_CHUNKS * 2, dtype=torch.float32, device=DEV))
    assert torch.equal(out, out2)
    temp = torch.full((m,), 0.7, dtype=torch.float32, device=DEV)
    for u in (0.0, 0.25, 0.5, 0.999999):
        un = torch.full((m,), u, dtype=torch.float64, device=DEV)
        ops.sample(logits, out, temp, un)
        # the kernel's fixed order: chunks of 2,048 ids; in a chunk the ids t, t + 256, ... for t = 0..255
        order = torch.tensor([c for b in range(0, v, 2048) for t in range(256) for c in range(b + t, min(b + 2048, v), 256)])
        assert sorted(order.tolist()) == list(range(v))
        for i in range(m):
            p = torch.exp((logits[i].double().cpu() - logits[i].double().max().cpu()) / 0.7)[order]
            cum = torch.cumsum(p, 0)
            at = int(torch.searchsorted(cum, u * float(cum[-1])).clamp(max=v - 1))
            want = int(order[at])
            got = int(out[i])
            where = int((order == got).nonzero()[0])
            # equal up to rounding of the running sum at the boundary
            assert got == want or abs(float(cum[where] - cum[at])) / float(cum[-1]) < 1e-9


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("n,k", [(24, 40), (96, 2048), (3072, 2048), (5000, 1000)])
def test_gemm_stream_with_fused_norm(ops, m, n, k):
    """The norm fused in front of the product equals norm kernel + product kernel (same bf16
    rounding of the normed rows), with and without a row gather, for every epilogue."""
    g = torch.Generator().manual_seed(9)
    x = (torch.randn(m + 3, k, generator=g) * 2).to(DEV)
    nw = (1 + 0.1 * torch.randn(k, generator=g)).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.1).to(torch.bfloat16).to(DEV)
    rows = torch.tensor([(3 * i + 1) % (m + 3) for i in range(m)], dtype=torch.int32, device=DEV)
    for idx in (None, rows):
        src = x if idx is not None else x[:m].contiguous()
        xn = torch.empty(m, k, dtype=torch.bfloat16, device=DEV)
        ops.rmsnorm(src, nw, xn, 1e-5, rows=idx)
        want = torch.empty(m, n, dtype=torch.float32, device=DEV)
        ops.gemm_stream(xn, w, want)
        got = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_stream_norm(src, nw, 1e-5, w, got, ops.EPI_STORE, idx)
        # differences come only from rows whose bf16 rounding flips on a last-bit change of 1/rms
        _close(got, want, 2e-3)
        s = (src if idx is None else src[idx.long()]).double()
        ref = (s / torch.sqrt((s * s).mean(1, keepdim=True) + 1e-5) * nw.double()) @ w.double().t()
        _close(got, ref, 6e-3)
    if n % 8 == 0:
        out = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_stream_norm(x[:m].contiguous(), nw, 1e-5, w, out, ops.EPI_SWIGLU)
        s = x[:m].double()
        y = ((s / torch.sqrt((s * s).mean(1, keepdim=True) + 1e-5) * nw.double()).to(torch.bfloat16).double()) @ w.double().t()
        y = y.reshape(m, n // 8, 2, 4)
        gate, up = y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)
        _close(out, gate / (1 + torch.exp(-gate)) * up, 6e-3)
