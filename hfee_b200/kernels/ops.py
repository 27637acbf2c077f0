"""Python face of the sm_100a kernel library: one function per kernel, taking torch
tensors (used only as typed device buffers) and launching on torch's current CUDA
stream.  There is no other implementation behind these functions: without a
CUDA device of compute capability 10.x and the built library they raise.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import build as _build


class KernelLibraryError(RuntimeError):
    """The CUDA kernel library is missing, cannot be loaded or refused a call."""


_LIB: Optional[ctypes.CDLL] = None
_DT = {torch.float32: 0, torch.bfloat16: 1}

_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_longlong
_F = ctypes.c_float

_SIGNATURES = {
    "hfee_embed": [_P, _I, _P, _P, _I, _I, _I, _P],
    "hfee_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "hfee_rope_table": [_P, _P, _P, _I, _I, _P],
    "hfee_rope_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "hfee_swiglu": [_P, _I, _P, _I, _I, _I, _I, _P],
    "hfee_gemm_simt": [_P, _L, _P, _L, _I, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_attention_simt": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "hfee_sample": [_P, _L, _I, _I, _P, _P, _P, _P],
}


def library() -> ctypes.CDLL:
    """Load (building first if needed) the kernel library; raises if impossible."""
    global _LIB
    if _LIB is not None:
        return _LIB
    if not torch.cuda.is_available():
        raise KernelLibraryError("no CUDA device: hfee_b200 runs on sm_100a GPUs only and has no CPU path")
    try:
        path = _build.build()
        lib = ctypes.CDLL(path)
    except (OSError, _build.KernelBuildError) as e:
        raise KernelLibraryError(f"cannot load the sm_100a kernel library: {e}") from e
    lib.hfee_last_error.restype = ctypes.c_char_p
    lib.hfee_device_is_sm100.restype = _I
    for name, sig in _SIGNATURES.items():
        try:
            fn = getattr(lib, name)
        except AttributeError as e:
            raise KernelLibraryError(f"{path} lacks the symbol {name}") from e
        fn.argtypes = sig
        fn.restype = _I
    if not lib.hfee_device_is_sm100():
        major, minor = torch.cuda.get_device_capability()
        raise KernelLibraryError(f"the kernels are built for sm_100a only; this device is sm_{major}{minor}")
    _LIB = lib
    return lib


def loaded_library_path() -> Optional[str]:
    return _LIB._name if _LIB is not None else None


def _check(code: int, lib: ctypes.CDLL) -> None:
    if code != 0:
        raise KernelLibraryError(lib.hfee_last_error().decode() or f"kernel call failed with code {code}")


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelLibraryError(f"unsupported dtype {t.dtype}: kernels take float32 and bfloat16") from None


def _rows(t: torch.Tensor, what: str) -> int:
    """Leading dimension (in elements) of a 2-D tensor whose rows are contiguous."""
    if t.dim() != 2 or (t.shape[1] > 1 and t.stride(1) != 1):
        raise KernelLibraryError(f"{what}: expected a 2-D tensor with contiguous rows, got shape "
                                 f"{tuple(t.shape)} strides {t.stride()}")
    return t.stride(0) if t.shape[0] > 1 else max(t.stride(0), t.shape[1])


def _i32(t: Optional[torch.Tensor], what: str) -> None:
    if t is not None and (t.dtype != torch.int32 or not t.is_contiguous() or not t.is_cuda):
        raise KernelLibraryError(f"{what}: expected a contiguous int32 CUDA tensor")


# ----------------------------------------------------------------------------
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor) -> None:
    """out[i,:] = table[tokens[i],:] widened to float32."""
    lib = library()
    _i32(tokens, "embed tokens")
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    n, width = out.shape
    _check(lib.hfee_embed(table.data_ptr(), _dt(table), tokens.data_ptr(), out.data_ptr(), n, width,
                          table.shape[0], _stream()), lib)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None, add_unit: bool = False) -> None:
    """out[r,:] = x[rows[r] or r,:] * rsqrt(mean(x^2)+eps) * weight (float32 math)."""
    lib = library()
    _i32(rows, "rmsnorm rows")
    assert x.dtype == torch.float32 and x.is_contiguous() and out.is_contiguous()
    assert weight.dtype == torch.float32 and weight.numel() == x.shape[1]
    n, width = out.shape
    _check(lib.hfee_rmsnorm(x.data_ptr(), weight.data_ptr(), _ptr(rows), out.data_ptr(), _dt(out), n, width,
                            float(eps), int(add_unit), _stream()), lib)


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, out: torch.Tensor) -> None:
    """out[i, j] = (cos, sin)(positions[i] * inv_freq[j]), computed in float64."""
    lib = library()
    _i32(positions, "rope positions")
    assert inv_freq.dtype == torch.float64 and out.dtype == torch.float32 and out.is_contiguous()
    n, half = positions.numel(), inv_freq.numel()
    assert out.numel() == n * half * 2
    _check(lib.hfee_rope_table(positions.data_ptr(), inv_freq.data_ptr(), out.data_ptr(), n, half, _stream()), lib)


def rope_cache_write(qkv: torch.Tensor, cs: Optional[torch.Tensor], positions: torch.Tensor,
                     slot_of_token: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                     v_pool: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int,
                     heads: int, kv_heads: int, head_dim: int, rope_dim: int, interleaved: bool) -> None:
    """Rotate q into ``q_out`` and k into its cache page, copy v to its page.
    ``qkv`` rows are [q heads | k heads | v heads]; pools are [pages, kv_heads, page_size, head_dim]."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = qkv.shape[0]
    want = (heads + 2 * kv_heads) * head_dim if k_pool is not None else heads * head_dim
    assert qkv.shape[1] == want and q_out.dtype == qkv.dtype
    if k_pool is not None:
        assert k_pool.dtype == qkv.dtype and v_pool.dtype == qkv.dtype
        assert k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim), (k_pool.shape, kv_heads, page_size, head_dim)
    _check(lib.hfee_rope_cache_write(qkv.data_ptr(), _rows(qkv, "qkv"), _ptr(cs), positions.data_ptr(),
                                     slot_of_token.data_ptr(), q_out.data_ptr(), _rows(q_out, "q_out"),
                                     _ptr(k_pool), _ptr(v_pool), block_table.data_ptr(), block_table.shape[1],
                                     page_size, n, heads, kv_heads, head_dim, rope_dim, int(interleaved),
                                     _dt(qkv), _stream()), lib)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[i, c] = silu(gate_up[i, c]) * gate_up[i, I + c] with I = out.shape[1]."""
    lib = library()
    n, inter = out.shape
    assert gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype
    _check(lib.hfee_swiglu(gate_up.data_ptr(), _rows(gate_up, "gate_up"), out.data_ptr(), _rows(out, "swiglu out"),
                           n, inter, _dt(out), _stream()), lib)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T on the CUDA cores with float32 accumulation, k in order."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n) and a.dtype == w.dtype
    _check(lib.hfee_gemm_simt(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), _dt(a),
                              out.data_ptr(), _rows(out, "gemm out"), _dt(out), int(accumulate), m, n, k,
                              _stream()), lib)


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T, choosing the kernel for the dtype and the shape."""
    gemm_simt(a, w, out, accumulate)


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, block_table: torch.Tensor,
                   page_size: int, positions: torch.Tensor, slot_of_token: torch.Tensor, out: torch.Tensor,
                   heads: int, kv_heads: int, head_dim: int, scale: float, window: int = 0) -> None:
    """Causal GQA over the paged cache, one warp per (token, head), float32 math."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n = q.shape[0]
    assert q.shape[1] == heads * head_dim and out.shape == q.shape and q.dtype == k_pool.dtype == out.dtype
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_attention_simt(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                   block_table.data_ptr(), block_table.shape[1], page_size, positions.data_ptr(),
                                   slot_of_token.data_ptr(), out.data_ptr(), _rows(out, "attention out"), n, heads,
                                   kv_heads, head_dim, float(scale), int(window or 0), _dt(q), _stream()), lib)


def paged_attention(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                    head_dim, scale, window=0, step=None) -> None:
    """Attention over the cache, choosing the kernel for the dtype and the batch."""
    attention_simt(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                   head_dim, scale, window)


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or no temperatures are given),
    else a draw from softmax(logits[r] / temperature[r]) using uniform[r] in [0, 1)."""
    lib = library()
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.is_contiguous()
    m, v = logits.shape
    if temperature is not None:
        assert temperature.dtype == torch.float32 and uniform.dtype == torch.float64
    _check(lib.hfee_sample(logits.data_ptr(), _rows(logits, "logits"), m, v, _ptr(temperature), _ptr(uniform),
                           out.data_ptr(), _stream()), lib)
