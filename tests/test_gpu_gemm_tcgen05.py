"""The tcgen05/TMA GEMM alone against a float64 reference: full tiles, ragged edges in
every dimension, K tails, both tile widths and every epilogue."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _err(got, ref):
    return float((got.double().cpu() - ref).abs().max() / (ref.abs().max() + 1e-30))


def _f32_tol(k):
    """Float32 accumulation in the tensor core rounds the running sum once per MMA (K = 16), and
    it truncates, so errors add up instead of averaging out: K/16 steps of one float32 ulp
    (2^-23 of the running sum) each, plus the rounding of the stored result."""
    return 2e-6 + (k / 16) * 2.0 ** -23


SHAPES = [(128, 128, 64), (128, 256, 128), (256, 128, 512), (65, 8, 8), (200, 300, 96), (129, 257, 72),
          (1000, 96, 2048), (2048, 3072, 2048), (333, 1000, 8192)]


@pytest.mark.parametrize("block_n", [128, 192, 256])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_store_and_accumulate(m, n, k, block_n):
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    ref = a.double().cpu() @ w.double().cpu().t()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(a, w, out, ops.EPI_STORE, block_n)
    ops.check_status()
    assert _err(out, ref) < _f32_tol(k)
    outb = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(a, w, outb, ops.EPI_STORE, block_n)
    assert _err(outb, ref) < 6e-3
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_tcgen05(a, w, acc, ops.EPI_ACCUM, block_n)
    ops.check_status()
    assert _err(acc, base.double().cpu() + ref) < _f32_tol(k)


@pytest.mark.parametrize("block_n", [128, 192, 256])
@pytest.mark.parametrize("m,inner,k", [(128, 64, 64), (300, 172, 96), (2048, 8192, 2048), (70, 1000, 264), (200, 1000, 4096)])
def test_swiglu_epilogue(m, inner, k, block_n):
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(inner)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inner, k, generator=g) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) * 0.1).to(torch.bfloat16)
    w = torch.stack([gate.reshape(inner // 4, 4, k), up.reshape(inner // 4, 4, k)], 1).reshape(2 * inner, k).contiguous().to(DEV)
    out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(a, w, out, ops.EPI_SWIGLU, block_n)
    ops.check_status()
    gd, ud = a.double().cpu() @ gate.double().t(), a.double().cpu() @ up.double().t()
    assert _err(out, gd / (1 + torch.exp(-gd)) * ud) < 6e-3


PAIR_SHAPES = [(256, 256, 64), (128, 256, 128), (65, 8, 8), (200, 300, 96), (257, 513, 72), (1000, 96, 2048),
               (2048, 2048, 2048), (333, 1000, 8192), (2048 + 128, 4096, 520)]


@pytest.mark.parametrize("m,n,k", PAIR_SHAPES)
def test_pairs_of_ctas_store_and_accumulate(m, n, k):
    """Two CTAs on a tile of 256 x 256: whole tiles, a pair whose second CTA has no rows (128, 65), rows
    and columns that end inside a tile, a K that is no multiple of 64, more tiles than pairs of SMs."""
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(m * 5 + n * 3 + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    ref = a.double().cpu() @ w.double().cpu().t()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05_pair(a, w, out, ops.EPI_STORE)
    ops.check_status()
    assert _err(out, ref) < _f32_tol(k)
    outb = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05_pair(a, w, outb, ops.EPI_STORE)
    assert _err(outb, ref) < 6e-3
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_tcgen05_pair(a, w, acc, ops.EPI_ACCUM)
    ops.check_status()
    assert _err(acc, base.double().cpu() + ref) < _f32_tol(k)
    # a start and a pitch the bulk reduction cannot take: the plain read-add-write epilogue
    view = torch.zeros(m, n + 3, dtype=torch.float32, device=DEV)[:, 1:n + 1]
    view.copy_(base)
    ops.gemm_tcgen05_pair(a, w, view, ops.EPI_ACCUM)
    ops.check_status()
    assert _err(view, base.double().cpu() + ref) < _f32_tol(k)


@pytest.mark.parametrize("m,inner,k", [(256, 128, 64), (300, 172, 96), (2048, 8192, 2048), (70, 1000, 264), (520, 1000, 4096)])
def test_pairs_of_ctas_swiglu(m, inner, k):
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(inner + 1)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    gate = (torch.randn(inner, k, generator=g) * 0.1).to(torch.bfloat16)
    up = (torch.randn(inner, k, generator=g) * 0.1).to(torch.bfloat16)
    w = torch.stack([gate.reshape(inner // 4, 4, k), up.reshape(inner // 4, 4, k)], 1).reshape(2 * inner, k).contiguous().to(DEV)
    out = torch.full((m, inner), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05_pair(a, w, out, ops.EPI_SWIGLU)
    ops.check_status()
    gd, ud = a.double().cpu() @ gate.double().t(), a.double().cpu() @ up.double().t()
    assert _err(out, gd / (1 + torch.exp(-gd)) * ud) < 6e-3


def test_the_dispatcher_takes_pairs_for_the_large_products_of_a_prompt(monkeypatch):
    """A large accumulating product of a 2,048-token prompt goes to the pair kernel and gives what the
    single-CTA kernel gives."""
    from hfee_b200.kernels import ops
    calls = []
    real = ops.gemm_tcgen05_pair
    monkeypatch.setattr(ops, "gemm_tcgen05_pair", lambda *a, **k: (calls.append(1), real(*a, **k))[1])
    g = torch.Generator().manual_seed(3)
    a = (torch.randn(2048, 1024, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    w = (torch.randn(4096, 1024, generator=g) * 0.05).to(torch.bfloat16).to(DEV)
    base = torch.randn(2048, 4096, generator=g).to(DEV)
    got, ref = base.clone(), base.clone()
    ops.gemm_tcgen05(a, w, got, ops.EPI_ACCUM)
    assert calls == [1]
    ops.gemm_tcgen05(a, w, ref, ops.EPI_ACCUM, block_n=256)
    ops.check_status()
    assert _err(got, ref.double().cpu()) < 1e-6


@pytest.mark.parametrize("m,n,k", [(512, 2048, 8192), (256, 2048, 8192), (333, 1000, 8192), (130, 300, 4104), (1000, 500, 6000)])
def test_split_by_k_blocks_matches_whole_tiles(m, n, k):
    """Shapes with tiles for less than half of the SMs and a long K are split by K blocks among the
    CTAs (partial tiles through a workspace, added in CTA order): same result as whole tiles up to the rounding of
    the partial sums, the same bits from launch to launch, and the flags are left clear."""
    from hfee_b200.kernels import ops
    lib = ops.library()
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(n, k, generator=g).to(torch.bfloat16).to(DEV)
    ref = a.double().cpu() @ w.double().cpu().t()
    ws, flags = ops._stream_k_workspace()
    assert lib.hfee_gemm_tcgen05_stream_k(m, n, k, 256, ws.numel()) > 0      # these shapes are split
    whole = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(a, w, whole, ops.EPI_STORE, 256, stream_k=False)
    outs = []
    for _ in range(3):
        out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
        ops.gemm_tcgen05(a, w, out, ops.EPI_STORE, 256, stream_k=True)
        ops.check_status()
        assert int(flags.abs().sum()) == 0
        outs.append(out)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    assert _err(outs[0], ref) < _f32_tol(k) and _err(whole, ref) < _f32_tol(k)
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_tcgen05(a, w, acc, ops.EPI_ACCUM, 256, stream_k=True)
    ops.check_status()
    assert _err(acc, base.double().cpu() + ref) < _f32_tol(k)


def test_strided_operands():
    """Views with a leading dimension larger than K (a slice of a wider buffer)."""
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(5)
    big_a = torch.randn(150, 256, generator=g).to(torch.bfloat16).to(DEV)
    big_w = torch.randn(90, 512, generator=g).to(torch.bfloat16).to(DEV)
    a, w = big_a[:, :128], big_w[:, 256:384]
    out = torch.empty(150, 90, dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(a, w, out)
    ops.check_status()
    assert _err(out, a.double().cpu() @ w.double().cpu().t()) < _f32_tol(128)


@pytest.mark.parametrize("m", [1, 8, 16, 17, 32, 33, 64])
@pytest.mark.parametrize("n,k", [(8, 8), (100, 96), (257, 1000), (2048, 2048), (3072, 2048), (2048, 8192), (16384, 2048)])
def test_skinny_swapped_operands_every_epilogue(m, n, k):
    """The few-token tcgen05 product (weights on the MMA's 128-row side, K split among CTAs and
    added in split order): direct and split paths, ragged edges, every epilogue."""
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16).to(DEV)
    w = (torch.randn(n, k, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    ref = a.double().cpu() @ w.double().cpu().t()
    out = torch.full((m, n), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_skinny(a, w, out)
    ops.check_status()
    assert _err(out, ref) < _f32_tol(k)
    outb = torch.full((m, n), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_skinny(a, w, outb)
    assert _err(outb, ref) < 6e-3
    base = torch.randn(m, n, generator=g).to(DEV)
    acc = base.clone()
    ops.gemm_skinny(a, w, acc, ops.EPI_ACCUM)
    ops.check_status()
    assert _err(acc, base.double().cpu() + ref) < _f32_tol(k)
    if n % 8 == 0:
        y = (ref * 0.1).reshape(m, n // 8, 2, 4)
        gate, up = y[:, :, 0].reshape(m, -1), y[:, :, 1].reshape(m, -1)
        w2 = (w.float() * 0.1).to(torch.bfloat16)
        y2 = (a.double().cpu() @ w2.double().cpu().t()).reshape(m, n // 8, 2, 4)
        gate, up = y2[:, :, 0].reshape(m, -1), y2[:, :, 1].reshape(m, -1)
        outs = torch.full((m, n // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
        ops.gemm_skinny(a, w2, outs, ops.EPI_SWIGLU)
        ops.check_status()
        assert _err(outs, gate / (1 + torch.exp(-gate)) * up) < 6e-3


def test_skinny_rows_do_not_depend_on_the_batch():
    from hfee_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    a = torch.randn(40, 2048, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(3072, 2048, generator=g).to(torch.bfloat16).to(DEV)
    full = torch.empty(40, 3072, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(a, w, full)
    one = torch.empty(1, 3072, dtype=torch.float32, device=DEV)
    ops.gemm_skinny(a[23:24], w, one)
    assert torch.equal(one[0], full[23])
