"""The fused tail of a layer for decode steps of at most 8 tokens (output projection, norm, gated
feed-forward in one persistent kernel) alone against a float64 reference: widths that are no power
of two, fewer rows than CTAs, 1 to 8 tokens, strided inputs, several launches in a row (the kernel
leaves its barrier words ready for the next one), and the same result as the separate kernels."""
import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _case(m, d, q, i, seed, std=0.05):
    g = torch.Generator().manual_seed(seed)
    bf = lambda *shape, s=1.0: (torch.randn(*shape, generator=g) * s).to(torch.bfloat16).to(DEV)
    att, w_o = bf(m, q), bf(d, q, s=std)
    gate, up, down = bf(i, d, s=std), bf(i, d, s=std), bf(d, i, s=std)
    residual = torch.randn(m, d, generator=g).to(DEV)
    norm_w = (1 + 0.1 * torch.randn(d, generator=g)).to(DEV)
    w_gu = torch.stack([gate.reshape(i // 4, 4, d), up.reshape(i // 4, 4, d)], dim=1).reshape(2 * i, d).contiguous()
    return att, w_o, gate, up, down, w_gu, residual, norm_w


def _reference(att, w_o, gate, up, down, residual, norm_w, eps, add_unit, rounded=True):
    """float64.  ``rounded``: with the two roundings to bfloat16 the kernel makes, where it makes them:
    x * w_norm before the gate/up product (the row's scale 1/sqrt(mean x^2 + eps) is applied to the
    sums behind it), and h before the down projection."""
    r = (lambda t: t.to(torch.bfloat16).double()) if rounded else (lambda t: t)
    x = residual.double() + att.double() @ w_o.double().t()
    w = norm_w.double() + (1.0 if add_unit else 0.0)
    scale = torch.rsqrt((x * x).mean(dim=1, keepdim=True) + eps)
    y = r(x * w)
    g, u = (y @ gate.double().t()) * scale, (y @ up.double().t()) * scale
    return x + r(g / (1 + torch.exp(-g)) * u) @ down.double().t()


def _err(got, ref):
    return float((got.double() - ref).abs().max() / ref.abs().max())


@pytest.mark.parametrize("m", [1, 3, 8])
@pytest.mark.parametrize("d,q,i", [(2048, 2048, 8192), (64, 128, 192), (4096, 4096, 14336), (1088, 576, 2880), (5120, 5120, 13824)])
@pytest.mark.parametrize("add_unit", [False, True])
def test_decode_tail(m, d, q, i, add_unit):
    from hfee_b200.kernels import ops
    assert ops.decode_tail_takes(m, d, q, i, torch.bfloat16)
    att, w_o, gate, up, down, w_gu, residual, norm_w = _case(m, d, q, i, seed=m + d)
    ref = _reference(att, w_o, gate, up, down, residual, norm_w, 1e-5, add_unit)
    out = residual.clone()
    hidden = torch.full((m, i), float("nan"), dtype=torch.bfloat16, device=DEV)
    for _ in range(3):                        # the barrier words are left ready for the next launch
        out.copy_(residual)
        ops.decode_tail(att, w_o, out, norm_w, 1e-5, add_unit, w_gu, down, hidden)
    ops.check_status()
    assert not torch.isnan(out).any() and not torch.isnan(hidden.float()).any()
    assert _err(out, ref) < 2e-3


def test_decode_tail_is_as_close_to_the_exact_result_as_the_separate_kernels():
    """The same step through the output projection, the norm kernel, the gate/up product with its
    SwiGLU epilogue and the down projection.  Both round two intermediate results to bfloat16 (the
    separate kernels the normed row, the fused one x * w_norm; both h), so they differ from each other by
    two such roundings and each from the exact float64 result by one."""
    from hfee_b200.kernels import ops
    m, d, q, i = 8, 2048, 2048, 8192
    att, w_o, gate, up, down, w_gu, residual, norm_w = _case(m, d, q, i, seed=77)
    a = residual.clone()
    ops.linear(att, w_o, a, accumulate=True)
    xn = torch.empty(m, d, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm(a, norm_w, xn, 1e-5)
    h = torch.empty(m, i, dtype=torch.bfloat16, device=DEV)
    ops.linear_swiglu(xn, w_gu, h, 4, torch.empty(m, 2 * i, dtype=torch.bfloat16, device=DEV))
    ops.linear(h, down, a, accumulate=True)
    b = residual.clone()
    ops.decode_tail(att, w_o, b, norm_w, 1e-5, False, w_gu, down, torch.empty(m, i, dtype=torch.bfloat16, device=DEV))
    ops.check_status()
    exact = _reference(att, w_o, gate, up, down, residual, norm_w, 1e-5, False, rounded=False)
    err_separate, err_fused = _err(a, exact), _err(b, exact)
    assert err_separate < 5e-3 and err_fused < 5e-3 and err_fused < 1.3 * err_separate


def test_strided_rows_and_what_it_refuses():
    from hfee_b200.kernels import ops
    m, d, q, i = 5, 256, 192, 512
    att, w_o, gate, up, down, w_gu, residual, norm_w = _case(m, d, q, i, seed=5)
    wide = torch.zeros(m, q + 64, dtype=torch.bfloat16, device=DEV)
    wide[:, :q] = att
    hidden = torch.zeros(8, i + 32, dtype=torch.bfloat16, device=DEV)
    out = residual.clone()
    ops.decode_tail(wide[:, :q], w_o, out, norm_w, 1e-6, False, w_gu, down, hidden[:, :i])
    ops.check_status()
    assert _err(out, _reference(att, w_o, gate, up, down, residual, norm_w, 1e-6, False)) < 3e-3
    assert not ops.decode_tail_takes(9, d, q, i, torch.bfloat16)            # more tokens than the MMA's 8 columns
    assert not ops.decode_tail_takes(4, d, q + 16, i, torch.bfloat16)       # a width that is no multiple of 64
    assert not ops.decode_tail_takes(4, d, q, i, torch.float32)
