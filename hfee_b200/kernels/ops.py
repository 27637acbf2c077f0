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
    "hfee_embed": [_P, _I, _P, _P, _P, _P, _I, _I, _I, _P],
    "hfee_rmsnorm": [_P, _P, _P, _P, _I, _I, _I, _F, _I, _P],
    "hfee_rope_table": [_P, _P, _P, _I, _I, _P],
    "hfee_rope_cache_write": [_P, _I, _P, _P, _P, _P, _I, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _I, _P],
    "hfee_swiglu": [_P, _I, _P, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_stream": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_stream_norm": [_P, _L, _P, _P, _F, _I, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_gemm_tcgen05": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _I, _P, _P, _L, _P, _P],
    "hfee_gemm_tcgen05_stream_k": [_I, _I, _I, _I, _L],
    "hfee_gemm_tcgen05_pair": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_tcgen05_rope": [_P, _L, _P, _L, _I, _I, _I, _P, _P, _P, _P, _L, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_tcgen05_rope_supports": [_I, _I],
    "hfee_gemm_skinny": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _L, _P, _P],
    "hfee_gemm_skinny_splits": [_I, _I, _I, _L],
    "hfee_gemm_ring": [_P, _L, _P, _L, _P, _L, _I, _I, _I, _I, _I, _P, _P],
    "hfee_gemm_ring_supports": [_I, _I, _I, _I],
    "hfee_attention_tc": [_P, _I, _P, _P, _I, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P, _P],
    "hfee_attention_tc_supports": [_I, _I, _I, _I],
    "hfee_attention_mma": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "hfee_attention_mma_rope": [_P, _I, _P, _I, _I, _I, _P, _P, _P, _I, _I, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P],
    "hfee_gemm_simt": [_P, _L, _P, _L, _I, _P, _L, _I, _I, _I, _I, _I, _P],
    "hfee_attention_simt": [_P, _I, _P, _P, _P, _I, _I, _P, _P, _P, _I, _I, _I, _I, _I, _F, _I, _I, _P],
    "hfee_sample": [_P, _L, _I, _I, _P, _P, _P, _L, _P, _P, _P, _P],
    "hfee_argmax": [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P],
    "hfee_sample_chain": [_P, _L, _I, _I, _P, _P, _P, _I, _P, _I, _P, _L, _P, _P, _P],
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
    lib.hfee_sm_count.restype = _I
    lib.hfee_set_carveout.restype = _I
    lib.hfee_set_carveout.argtypes = [_I]
    lib.hfee_gemm_skinny_splits.restype = _I
    lib.hfee_attention_tc_supports.restype = _I
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


def set_carveout(percent: Optional[int]) -> Optional[int]:
    """The split between shared memory and L1 that the launches that follow ask for: percent of the
    SM's shared-memory maximum, or None for the driver's choice per kernel.  Returns the setting before.
    A chain of short kernels runs fastest when all of them ask for the same split."""
    before = library().hfee_set_carveout(-1 if percent is None else int(percent))
    return None if before < 0 else before


def sm_count() -> int:
    """Streaming multiprocessors of the current device, as the kernels' launchers see them."""
    global _SMS
    if _SMS is None:
        n = library().hfee_sm_count()
        if n <= 0:
            raise KernelLibraryError("cannot ask the device for its number of SMs")
        _SMS = n
    return _SMS


_SMS: Optional[int] = None


def loaded_library_path() -> Optional[str]:
    return _LIB._name if _LIB is not None else None


_LAUNCHES = 0

# Measuring what a class of kernels costs inside a step: the parts name the class of their next
# launches with tag(); leave_out(classes) makes every launch of those classes a no-op (the results
# are then wrong, the timing of the rest is not), and the difference of the step time with and
# without a class is what it costs in place, overlap with its neighbours included.
_TAG = ""
_LEFT_OUT: frozenset = frozenset()


def tag(name: str) -> str:
    """Name the class of the launches that follow; returns the class named before."""
    global _TAG
    before, _TAG = _TAG, name
    return before


def leave_out(classes=()) -> None:
    global _LEFT_OUT
    _LEFT_OUT = frozenset(classes)


def _measurable(fn):
    import functools

    @functools.wraps(fn)
    def call(*args, **kwargs):
        if _LEFT_OUT and _TAG in _LEFT_OUT:
            # a product left out still lets the norm in front of it run, unless the kernel would have
            # computed that norm itself
            if args and not isinstance(args[0], torch.Tensor) and hasattr(args[0], "tensor") and not _norm_fusable(args[0], args[1]):
                args[0].tensor()
            return None
        return fn(*args, **kwargs)
    return call


def launch_count() -> int:
    """Kernels launched through this module so far (a graph replay counts its kernels)."""
    return _LAUNCHES


def count_launches(n: int) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def _check(code: int, lib: ctypes.CDLL) -> None:
    global _LAUNCHES
    _LAUNCHES += 1
    if code != 0:
        raise KernelLibraryError(lib.hfee_last_error().decode() or f"kernel call failed with code {code}")


_STREAM_HELD: Optional[int] = None


def _stream() -> int:
    return _STREAM_HELD if _STREAM_HELD is not None else torch.cuda.current_stream().cuda_stream


class stream_held:
    """``with ops.stream_held():`` every launch inside goes to the stream that is current at entry,
    asked of torch once instead of once per launch (a third of the host's time for a prompt pass of a
    16-layer model went into that question).  Nothing inside may change the current stream."""

    def __enter__(self):
        global _STREAM_HELD
        self.before = _STREAM_HELD
        _STREAM_HELD = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _STREAM_HELD
        _STREAM_HELD = self.before
        return False


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
def embed(table: torch.Tensor, tokens: torch.Tensor, out: torch.Tensor, slot_of_token: Optional[torch.Tensor] = None,
          feedback: Optional[torch.Tensor] = None) -> None:
    """out[i,:] = table[tokens[i],:] widened to float32.  With ``feedback`` (int32 per request slot)
    a negative token id stands for ``feedback[slot_of_token[i]]``: the token last sampled on the
    device for that request."""
    lib = library()
    _i32(tokens, "embed tokens"); _i32(slot_of_token, "slot_of_token"); _i32(feedback, "feedback")
    assert out.dtype == torch.float32 and out.is_contiguous() and table.is_contiguous()
    assert feedback is None or slot_of_token is not None
    n, width = out.shape
    _check(lib.hfee_embed(table.data_ptr(), _dt(table), tokens.data_ptr(), _ptr(slot_of_token), _ptr(feedback),
                          out.data_ptr(), n, width, table.shape[0], _stream()), lib)


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


# Prompt portions: rotation and cache write in the epilogue of the q/k/v product instead of a pass of
# their own over the projection (prompt of 2,048 tokens, benchmark model: 11 us per layer less).
FUSE_ROPE_INTO_QKV = True
QKV_ROPE_MIN_TOKENS = 65         # from here on linear() takes the large-tile tcgen05 kernel anyway


def qkv_rope_fusable(a_dtype: torch.dtype, n: int, w: torch.Tensor, head_dim: int, rope_dim: int,
                     cs: Optional[torch.Tensor], q_out: torch.Tensor) -> bool:
    """True when :func:`linear_rope_cache` takes this step."""
    return (FUSE_ROPE_INTO_QKV and USE_TCGEN05 and a_dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and n >= QKV_ROPE_MIN_TOKENS and head_dim in (64, 128) and (cs is None or rope_dim == head_dim)
            and w.shape[1] % 8 == 0 and _rows(w, "w") % 8 == 0 and w.data_ptr() % 16 == 0
            and _rows(q_out, "q_out") % 8 == 0 and q_out.data_ptr() % 16 == 0)


def linear_rope_cache(a: torch.Tensor, w: torch.Tensor, cs: Optional[torch.Tensor], positions: torch.Tensor,
                      slot_of_token: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                      v_pool: Optional[torch.Tensor], block_table: torch.Tensor, page_size: int, heads: int,
                      kv_heads: int, head_dim: int, interleaved: bool) -> None:
    """``a @ w.T`` with rows of ``w`` = [q heads | k heads | v heads] ([q heads] when the pools are
    None), rotated by ``cs`` ([n, head_dim/2, 2] cosines and sines) in the product's epilogue: queries
    to ``q_out``, keys and values to the cache pages of (slot, position).  Nothing else is stored."""
    lib = library()
    _i32(positions, "positions"); _i32(slot_of_token, "slot_of_token"); _i32(block_table, "block_table")
    n, k = a.shape
    want = (heads + 2 * kv_heads) * head_dim if k_pool is not None else heads * head_dim
    assert w.shape == (want, k) and a.dtype == w.dtype == q_out.dtype == torch.bfloat16
    assert a.data_ptr() % 16 == 0 and _rows(a, "a") % 8 == 0 and q_out.shape[0] == n
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == n * head_dim)
    if k_pool is not None:
        assert k_pool.dtype == v_pool.dtype == torch.bfloat16 and k_pool.is_contiguous() and v_pool.is_contiguous()
        assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_gemm_tcgen05_rope(a.data_ptr(), _rows(a, "a"), w.data_ptr(), _rows(w, "w"), n, want, k, _ptr(cs),
                                      positions.data_ptr(), slot_of_token.data_ptr(), q_out.data_ptr(),
                                      _rows(q_out, "q_out"), _ptr(k_pool), _ptr(v_pool), block_table.data_ptr(),
                                      block_table.shape[1], page_size, heads, kv_heads, head_dim, int(interleaved),
                                      _status().data_ptr(), _stream()), lib)


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, granule: Optional[int] = None) -> None:
    """out[i, c] = silu(gate) * up.  Columns of ``gate_up`` come in groups of ``granule`` gate
    columns followed by ``granule`` up columns (default: all gate columns, then all up columns)."""
    lib = library()
    n, inter = out.shape
    assert gate_up.shape[1] == 2 * inter and gate_up.dtype == out.dtype
    _check(lib.hfee_swiglu(gate_up.data_ptr(), _rows(gate_up, "gate_up"), out.data_ptr(), _rows(out, "swiglu out"),
                           n, inter, int(granule or inter), _dt(out), _stream()), lib)


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T on the CUDA cores with float32 accumulation, k in order."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and tuple(out.shape) == (m, n) and a.dtype == w.dtype
    _check(lib.hfee_gemm_simt(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), _dt(a),
                              out.data_ptr(), _rows(out, "gemm out"), _dt(out), int(accumulate), m, n, k,
                              _stream()), lib)


STREAM_MAX_TOKENS = 64
USE_TCGEN05 = True
EPI_STORE, EPI_ACCUM, EPI_SWIGLU = 0, 1, 2


def _streamable(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[0] <= STREAM_MAX_TOKENS and a.shape[1] % 8 == 0
            and _rows(a, "a") % 8 == 0 and _rows(w, "w") % 8 == 0
            and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_stream(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 64 rows of ``a`` (bfloat16), streaming ``w`` once through
    mma.sync tiles.  ``epilogue``: store, accumulate into float32 ``out``, or SwiGLU over rows
    of ``w`` interleaved as [4 gate | 4 up] (then ``out`` is [m, n/2])."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    _check(lib.hfee_gemm_stream(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _stream()), lib)


_STATUS: Optional[torch.Tensor] = None


def gemm_ring(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 8 rows of ``a`` (bfloat16, width a multiple of 64): one CTA per SM
    streams its share of the rows of ``w`` through a ring of TMA boxes.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    _check(lib.hfee_gemm_ring(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                              _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _status().data_ptr(), _stream()), lib)


_RING_TAKES: dict = {}


def ring_takes(m: int, n: int, k: int, epilogue: int) -> bool:
    key = (m, n, k, epilogue)
    if key not in _RING_TAKES:
        _RING_TAKES[key] = bool(library().hfee_gemm_ring_supports(*key))
    return _RING_TAKES[key]


def _status() -> torch.Tensor:
    global _STATUS
    if _STATUS is None:
        _STATUS = torch.zeros(1, dtype=torch.int32, device="cuda")
    return _STATUS


def check_status() -> None:
    """Raise if a kernel gave up a bounded wait since the last check (synchronises)."""
    if _STATUS is not None and int(_STATUS.item()) != 0:
        _STATUS.zero_()
        raise KernelLibraryError("a tcgen05 kernel gave up waiting on a barrier; its output is invalid")


def _tensor_core_ok(a: torch.Tensor, w: torch.Tensor) -> bool:
    return (a.dtype == torch.bfloat16 and a.shape[1] % 8 == 0 and _rows(a, "a") % 8 == 0
            and _rows(w, "w") % 8 == 0 and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0)


def gemm_tcgen05(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE,
                 block_n: Optional[int] = None, stream_k: Optional[bool] = None) -> None:
    """out (+)= a @ w.T with tcgen05.mma tiles of 128 x block_n fed by TMA (bfloat16 in, float32
    accumulation in tensor memory).  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    tiles_256 = 0
    if block_n is None:
        # wide tiles need a third less shared-memory feed per flop (a 128-wide tile's feed rate is at
        # the L2 -> shared-memory limit); narrow ones fill the SMs when there are few tiles.  Measured
        # at M = N = 2048 (128 wide tiles on 148 SMs): K = 8192 takes 61 us wide, 95 us narrow.
        tiles_256 = -(-m // 128) * -(-n // 256)
        block_n = 256 if tiles_256 >= 96 else 128
        # 192 wide where that saves a round of tiles: 16 x 12 tiles of 256 are two rounds on 148 SMs
        # with the second a third full, 16 x 16 tiles of 192 are two rounds of three quarters the work
        if block_n == 256 and n % 192 == 0:
            rounds = lambda bn: -(-(-(-m // 128) * -(-n // bn)) // sm_count())
            if rounds(192) * 192 * 1.05 < rounds(256) * 256:
                block_n = 192
    if USE_PAIRS and block_n == 256 and m > 128 and tiles_256 >= 96 and (epilogue != EPI_STORE or n * k >= PAIR_STORE_MIN):
        gemm_tcgen05_pair(a, w, out, epilogue)
        return
    if stream_k is None:
        stream_k = USE_STREAM_K
    ws, flags = _stream_k_workspace() if stream_k else (None, None)
    _check(lib.hfee_gemm_tcgen05(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                 _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, block_n,
                                 _status().data_ptr(), _ptr(ws), ws.numel() if ws is not None else 0, _ptr(flags),
                                 _stream()), lib)


# Two CTAs on a tile of 256 x 256 (cta_group::2) where the single-CTA kernel would take tiles of
# 128 x 256: measured at 2,048 tokens, gate/up of the benchmark model 102 -> 90 us (1,527 TFLOP/s), down
# projection 57 -> 50 us, output projection 16.6 -> 17.0 us.
USE_PAIRS = True
PAIR_STORE_MIN = 1 << 62        # plain stores: the single-CTA kernel until measured otherwise


def gemm_tcgen05_pair(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """:func:`gemm_tcgen05` with two CTAs on each tile of 256 x 256 (``cta_group::2``): each CTA loads
    its own 128 rows of ``a`` and half of the tile's rows of ``w``.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    _check(lib.hfee_gemm_tcgen05_pair(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                      _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _status().data_ptr(),
                                      _stream()), lib)


USE_STREAM_K = True
_STREAM_K_WS = None


def _stream_k_workspace():
    """One float32 tile of 128 x 256 per SM for the partial tiles of products split by K blocks, and
    two flag words per SM (zero at the start; every launch leaves them zero).  Made once, 19 MiB."""
    global _STREAM_K_WS
    if _STREAM_K_WS is None:
        _STREAM_K_WS = (torch.empty(sm_count() * 128 * 256, dtype=torch.float32, device="cuda"),
                        torch.zeros(2 * sm_count(), dtype=torch.int32, device="cuda"))
    return _STREAM_K_WS


def gemm_stream_norm(x: torch.Tensor, norm_weight: torch.Tensor, eps: float, w: torch.Tensor, out: torch.Tensor,
                     epilogue: int = EPI_STORE, rows: Optional[torch.Tensor] = None, add_unit: bool = False) -> None:
    """:func:`gemm_stream` with the RMS norm fused in front: the token operand is
    bf16(x[rows] * rsqrt(mean(x^2) + eps) * norm_weight) made on the fly from float32 rows.  At most
    8 rows and a width of at most 2,048 (the kernel that keeps the tokens in registers)."""
    lib = library()
    _i32(rows, "rows")
    k = x.shape[1]
    m = rows.numel() if rows is not None else x.shape[0]
    n = w.shape[0]
    assert x.dtype == torch.float32 and norm_weight.dtype == torch.float32 and norm_weight.numel() == k
    assert w.shape[1] == k and w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    _check(lib.hfee_gemm_stream_norm(x.data_ptr(), _rows(x, "x"), _ptr(rows), norm_weight.data_ptr(), float(eps),
                                     int(add_unit), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                     _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, _stream()), lib)


# Norming inside the streaming GEMM saves a launch, but every CTA then reads the float32 rows (twice
# the bytes of the normed bfloat16 rows, the same addresses from every SM at the same moment).
# Measured on B200 in the model: batch 1 gains (0.765 -> 0.737 ms per decode step), batch 8 loses
# (0.88 -> 0.92 ms); the break-even lies near three tokens.
FUSE_NORM_MAX_TOKENS = 2
FUSE_NORM_MAX_WIDTH = 2048      # one pass of the kernel that keeps the tokens in registers


def _norm_fusable(inp, w: torch.Tensor) -> bool:
    """True when ``inp`` (a lazily normed input, see parts/norm.py) can be normed inside the streaming GEMM."""
    if inp.n > FUSE_NORM_MAX_TOKENS:
        return False
    p = inp.fused_params()
    x = inp.source
    return (p is not None and inp.out_dtype == torch.bfloat16 and w.dtype == torch.bfloat16
            and inp.n <= 8 and x.shape[1] % 8 == 0 and x.shape[1] <= FUSE_NORM_MAX_WIDTH and _rows(x, "x") % 4 == 0
            and _rows(w, "w") % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0
            and p[0].data_ptr() % 16 == 0)


def linear_normed(inp, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= norm(x) @ w.T where ``inp`` is a lazily normed input: the norm runs inside the
    product when a kernel that can do so fits, else ``inp`` is materialised first."""
    if isinstance(inp, torch.Tensor):
        linear(inp, w, out, accumulate)
    elif _norm_fusable(inp, w):
        weight, eps, add_unit = inp.fused_params()
        gemm_stream_norm(inp.source, weight, eps, w, out, EPI_ACCUM if accumulate else EPI_STORE, inp.rows, add_unit)
    else:
        linear(inp.tensor(), w, out, accumulate)


def linear_swiglu_normed(inp, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int, scratch: torch.Tensor) -> None:
    """:func:`linear_swiglu` on a lazily normed input."""
    if isinstance(inp, torch.Tensor):
        linear_swiglu(inp, w_gate_up, out, granule, scratch)
    elif granule == SWIGLU_GRANULE and w_gate_up.shape[0] % 8 == 0 and _norm_fusable(inp, w_gate_up):
        weight, eps, add_unit = inp.fused_params()
        gemm_stream_norm(inp.source, weight, eps, w_gate_up, out, EPI_SWIGLU, inp.rows, add_unit)
    else:
        linear_swiglu(inp.tensor(), w_gate_up, out, granule, scratch)


_SKINNY_WS: Optional[torch.Tensor] = None
SKINNY_WS_FLOATS = 4 << 20


def _skinny_workspace() -> torch.Tensor:
    """Float32 workspace for the partial tiles of K-split skinny products (made once, 16 MiB)."""
    global _SKINNY_WS
    if _SKINNY_WS is None:
        _SKINNY_WS = torch.empty(SKINNY_WS_FLOATS, dtype=torch.float32, device="cuda")
    return _SKINNY_WS


def gemm_skinny(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int = EPI_STORE) -> None:
    """out (+)= a @ w.T for at most 64 rows of ``a`` on tcgen05 with the operands swapped (weight
    rows on the 128-row side of the MMA) and K split among CTAs when weight tiles are few; TMA
    streams the weights through a deep shared-memory ring.  Epilogues as in :func:`gemm_stream`."""
    lib = library()
    m, k = a.shape
    n = w.shape[0]
    assert w.shape[1] == k and a.dtype == w.dtype == torch.bfloat16
    assert tuple(out.shape) == (m, n // 2 if epilogue == EPI_SWIGLU else n)
    ws = _skinny_workspace()
    _check(lib.hfee_gemm_skinny(a.data_ptr(), _rows(a, "gemm a"), w.data_ptr(), _rows(w, "gemm w"), out.data_ptr(),
                                _rows(out, "gemm out"), _dt(out), epilogue, m, n, k, ws.data_ptr(), ws.numel(),
                                _status().data_ptr(), _stream()), lib)
    if lib.hfee_gemm_skinny_splits(m, n, k, ws.numel()) > 1:
        count_launches(1)


# The ring kernel (one CTA per SM, TMA boxes) against the register-streaming one, decode step of the
# benchmark model at batch 8: accumulating products (output and down projection) through the ring
# 0.873 -> 0.855 ms; all products through it 0.887 ms (gate/up and qkv, whose CTAs own several row
# tiles, are slower there); for one or two tokens the register kernel wins everywhere.
RING_MIN_TOKENS, RING_MAX_TOKENS = 3, 8
RING_EPILOGUES = (EPI_ACCUM,)
STREAM_BEST_TOKENS = 16      # up to here the register-streaming kernels win; above, the skinny tcgen05 kernel


def _small_gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, epilogue: int) -> None:
    m, n = a.shape[0], w.shape[0]
    if _ring_rule(m, n, a.shape[1], epilogue):
        gemm_ring(a, w, out, epilogue)
    elif m <= STREAM_BEST_TOKENS or not USE_TCGEN05:
        gemm_stream(a, w, out, epilogue)
    elif m > 32 and 64 * 128 <= n <= 256 * 128 and a.shape[1] <= 4096 and _tensor_core_ok(a, w) and (
            epilogue != EPI_SWIGLU or out.dtype == torch.bfloat16):
        # 64-256 narrow tiles of the large-tile kernel fill the SMs about once, and their epilogues are cheaper than the
        # swapped one: measured at 64 tokens, N = 16,384, K = 2,048: 16.3 us against 18.9 us
        gemm_tcgen05(a, w, out, epilogue)
    else:
        gemm_skinny(a, w, out, epilogue)


def _ring_rule(m: int, n: int, k: int, epilogue: int) -> bool:
    return (epilogue in RING_EPILOGUES and RING_MIN_TOKENS <= m <= RING_MAX_TOKENS and USE_TCGEN05
            and n <= 16 * sm_count() and ring_takes(m, n, k, epilogue))


def linear(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, accumulate: bool = False) -> None:
    """out (+)= a @ w.T, choosing the kernel for the dtype and the shape."""
    if _streamable(a, w):
        _small_gemm(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
    elif USE_TCGEN05 and _tensor_core_ok(a, w):
        gemm_tcgen05(a, w, out, EPI_ACCUM if accumulate else EPI_STORE)
    else:
        gemm_simt(a, w, out, accumulate)


SWIGLU_GRANULE = 4


def linear_swiglu(a: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor, granule: int,
                  scratch: torch.Tensor) -> None:
    """out = silu(a @ w_gate^T) * (a @ w_up^T) where ``w_gate_up`` holds the rows of both in groups
    of ``granule`` gate rows followed by ``granule`` up rows; ``scratch`` [m, 2*inner] holds the
    projection when it is not fused."""
    fusable = granule == SWIGLU_GRANULE and w_gate_up.shape[0] % 8 == 0
    if fusable and _streamable(a, w_gate_up):
        _small_gemm(a, w_gate_up, out, EPI_SWIGLU)
    elif fusable and USE_TCGEN05 and _tensor_core_ok(a, w_gate_up) and out.dtype == torch.bfloat16:
        gemm_tcgen05(a, w_gate_up, out, EPI_SWIGLU)
    else:
        linear(a, w_gate_up, scratch)
        swiglu(scratch, out, granule)


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


MAX_SPLITS = 32


def attention_splits(requests: int, kv_heads: int, max_context: int, sms: Optional[int] = None) -> int:
    """How many CTAs share the keys of one (request, kv head) in a decode step: about four CTAs
    per SM in all (measured alone at batch 8: 9 splits against 6 take 10.3 / 27.2 / 90.8 us against
    11.3 / 30.9 / 99.6 us at 2,048 / 8,192 / 32,768 keys; batch 12 at 8,192 keys: 6 against 4 take
    37.5 against 42.6 us), and at least four even when the batch alone would fill the GPU (shorter
    CTAs balance better and keep more loads in flight: at 2,048 keys, batch 32: 41.8 us unsplit,
    33.4 us with four), but at least two key blocks of 64 each.  With few (request, kv head) pairs,
    two CTAs per SM: those grids take the kernel variant with four key blocks in flight per CTA, of
    which the step's shared-memory carve-out holds one per SM (decode step of the benchmark model at
    batch 2 / 3 / 4 / 5 / 6: 0.742 / 0.777 / 0.786 / 0.802 / 0.817 ms against 0.755 / 0.798 / 0.809 /
    0.812 / 0.823 with four per SM; at batch 8: 0.857 against 0.838)."""
    pairs = max(1, requests * kv_heads)
    per_sm = 2 if pairs <= FEW_PAIRS else 4
    want = max(4, per_sm * (sms or sm_count()) // pairs)
    return max(1, min(MAX_SPLITS, want, max_context // 128))


FEW_PAIRS = 48


def attention_mma(q, k_pool, v_pool, block_table, page_size, cu_tokens, slots, context_before, out, n_tokens,
                  requests, max_new, heads, kv_heads, head_dim, scale, window=0, num_splits=1, scratch=None) -> None:
    """Flash attention over the paged cache on mma.sync tensor cores (bfloat16)."""
    lib = library()
    for t, what in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (slots, "slots"),
                    (context_before, "context_before")):
        _i32(t, what)
    assert q.dtype == k_pool.dtype == out.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    if num_splits > 1:
        need = n_tokens * heads * num_splits * (head_dim + 2)
        assert scratch is not None and scratch.dtype == torch.float32 and scratch.numel() >= need
    _check(lib.hfee_attention_mma(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(),
                                  block_table.data_ptr(), block_table.shape[1], page_size, cu_tokens.data_ptr(),
                                  slots.data_ptr(), context_before.data_ptr(), out.data_ptr(),
                                  _rows(out, "attention out"), n_tokens, requests, max_new, heads, kv_heads,
                                  head_dim, float(scale), int(window or 0), num_splits, _ptr(scratch), _stream()), lib)
    if num_splits > 1:
        count_launches(1)


USE_TC_ATTENTION = True


def attention_tc(q, k_pool, v_pool, block_table, page_size, cu_tokens, slots, context_before, out, n_tokens,
                 requests, max_new, heads, kv_heads, head_dim, scale, window=0) -> None:
    """Flash attention for prompt portions on tcgen05 (S, P and O in tensor memory, TMA-fed pages, one
    softmax thread per query row).  bfloat16, head size 64 or 128, pages of at least 64 tokens."""
    lib = library()
    for t, what in ((block_table, "block_table"), (cu_tokens, "cu_tokens"), (slots, "slots"),
                    (context_before, "context_before")):
        _i32(t, what)
    assert q.dtype == k_pool.dtype == out.dtype == torch.bfloat16
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    _check(lib.hfee_attention_tc(q.data_ptr(), _rows(q, "q"), k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0],
                                 block_table.data_ptr(), block_table.shape[1], page_size, cu_tokens.data_ptr(),
                                 slots.data_ptr(), context_before.data_ptr(), out.data_ptr(),
                                 _rows(out, "attention out"), n_tokens, requests, max_new, heads, kv_heads, head_dim,
                                 float(scale), int(window or 0), _status().data_ptr(), _stream()), lib)


_TC_TAKES: dict = {}


def attention_tc_supports(heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    key = (heads, kv_heads, head_dim, page_size)
    if key not in _TC_TAKES:
        _TC_TAKES[key] = bool(library().hfee_attention_tc_supports(*key))
    return _TC_TAKES[key]


def paged_attention(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                    head_dim, scale, window=0, step=None, scratch=None) -> None:
    """Attention over the cache, choosing the kernel for the dtype and the batch.  ``step`` gives
    the per-request layout (cu_tokens, slots, context_before, max_new, max_context) that the
    tensor-core kernel needs; without it, or in float32, the CUDA-core kernel runs."""
    group = heads // kv_heads
    if (step is not None and q.dtype == torch.bfloat16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and group <= 64 and _rows(q, "q") % 8 == 0):
        if (USE_TC_ATTENTION and step.max_new * group > 16 and _rows(out, "out") % 8 == 0
                and attention_tc_supports(heads, kv_heads, head_dim, page_size)):
            attention_tc(q, k_pool, v_pool, block_table, page_size, step.cu_tokens, step.slots, step.context_before,
                         out, step.n, step.r, step.max_new, heads, kv_heads, head_dim, scale, window)
            return
        splits = 1
        if step.max_new * group <= 16 and scratch is not None:
            splits = getattr(step, "attention_splits", None) or attention_splits(
                step.r, kv_heads, getattr(step, "planning_context", step.max_context))
            if step.n * heads * splits * (head_dim + 2) > scratch.numel():
                splits = 1
        attention_mma(q, k_pool, v_pool, block_table, page_size, step.cu_tokens, step.slots, step.context_before,
                      out, step.n, step.r, step.max_new, heads, kv_heads, head_dim, scale, window, splits, scratch)
    else:
        attention_simt(q, k_pool, v_pool, block_table, page_size, positions, slot_of_token, out, heads, kv_heads,
                       head_dim, scale, window)


# A decode step of one token per request can do the rotary kernel's work inside the attention
# kernel (one launch less per layer).
FUSE_ROPE_INTO_DECODE_ATTENTION = True


def decode_rope_fusable(step, dtype: torch.dtype, heads: int, kv_heads: int, head_dim: int, rope_dim: int,
                        qkv: torch.Tensor, scratch: Optional[torch.Tensor]) -> bool:
    """True when :func:`paged_attention_rope` takes this step: bfloat16, one new token per request,
    a group that fits the 16-row decode tile, rotary pieces of whole 16-byte units."""
    group = heads // kv_heads
    return (FUSE_ROPE_INTO_DECODE_ATTENTION and step is not None and dtype == torch.bfloat16
            and getattr(step, "max_new", 0) == 1 and group <= 16 and head_dim % 16 == 0 and 16 <= head_dim <= 256
            and rope_dim % 16 == 0 and _rows(qkv, "qkv") % 8 == 0 and qkv.data_ptr() % 16 == 0)


def paged_attention_rope(qkv, cs, rope_dim, interleaved, write_cache, k_pool, v_pool, block_table, page_size, out,
                         heads, kv_heads, head_dim, scale, window, step, scratch) -> None:
    """Rotary + cache write + attention of a decode step in one kernel (plus the combine kernel when
    the keys are split): ``qkv`` rows are [q heads | k heads | v heads] ([q heads] when
    ``write_cache`` is false), ``cs`` the (cos, sin) table of the step or None."""
    lib = library()
    for t, what in ((block_table, "block_table"), (step.cu_tokens, "cu_tokens"), (step.slots, "slots"),
                    (step.context_before, "context_before")):
        _i32(t, what)
    assert qkv.dtype == k_pool.dtype == out.dtype == torch.bfloat16 and step.n == step.r
    assert k_pool.is_contiguous() and v_pool.is_contiguous()
    assert tuple(k_pool.shape[1:]) == (kv_heads, page_size, head_dim)
    assert cs is None or (cs.dtype == torch.float32 and cs.is_contiguous() and cs.numel() == step.n * rope_dim)
    splits = 1
    if scratch is not None:
        splits = getattr(step, "attention_splits", None) or attention_splits(
            step.r, kv_heads, getattr(step, "planning_context", step.max_context))
        if step.n * heads * splits * (head_dim + 2) > scratch.numel():
            splits = 1
    _check(lib.hfee_attention_mma_rope(qkv.data_ptr(), _rows(qkv, "qkv"), _ptr(cs), rope_dim, int(interleaved),
                                       int(write_cache), k_pool.data_ptr(), v_pool.data_ptr(), block_table.data_ptr(),
                                       block_table.shape[1], page_size, step.cu_tokens.data_ptr(), step.slots.data_ptr(),
                                       step.context_before.data_ptr(), out.data_ptr(), _rows(out, "attention out"),
                                       step.n, step.r, heads, kv_heads, head_dim, float(scale), int(window or 0), splits,
                                       _ptr(scratch) if splits > 1 else None, _stream()), lib)
    if splits > 1:
        count_launches(1)


def sample(logits: torch.Tensor, out: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           uniform: Optional[torch.Tensor] = None, slots: Optional[torch.Tensor] = None,
           feedback: Optional[torch.Tensor] = None) -> None:
    """out[r] = argmax(logits[r]) where temperature[r] <= 0 (or no temperatures are given),
    else a draw from softmax(logits[r] / temperature[r]) using uniform[r] in [0, 1): the inverse CDF
    over the tokens in the fixed order of the kernel (chunks of 2,048 ids; in a chunk the ids
    t, t + 256, ... of t = 0..255 in turn).  With ``slots`` and ``feedback`` the choice is also stored
    in ``feedback[slots[r]]``."""
    lib = library()
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.is_contiguous()
    _i32(slots, "slots"); _i32(feedback, "feedback")
    assert (slots is None) == (feedback is None)
    m, v = logits.shape
    if temperature is not None:
        assert temperature.dtype == torch.float32 and uniform.dtype == torch.float64
    global _SAMPLE_SCRATCH
    need = m * -(-v // CHAIN_CHUNK) * 2
    if _SAMPLE_SCRATCH is None or _SAMPLE_SCRATCH.numel() < need:
        _SAMPLE_SCRATCH = torch.empty(max(need, 64 * 64 * 2), dtype=torch.float64, device=logits.device)
    _check(lib.hfee_sample(logits.data_ptr(), _rows(logits, "logits"), m, v, _ptr(temperature), _ptr(uniform),
                           _SAMPLE_SCRATCH.data_ptr(), _SAMPLE_SCRATCH.numel(), out.data_ptr(), _ptr(slots),
                           _ptr(feedback), _stream()), lib)
    count_launches(1)


_SAMPLE_SCRATCH: Optional[torch.Tensor] = None


CHAIN_MAX_K = 64            # largest top-k the device chain takes
CHAIN_HISTORY = 256         # tokens of recent history kept per request slot for the repeat penalty
CHAIN_CHUNK = 2048
CHAIN_MAX_VOCAB = 128 * CHAIN_CHUNK     # the chain kernels look at no more chunks than this; larger vocabularies take the host chain


def chain_scratch_floats(rows: int, vocab: int) -> int:
    return rows * -(-vocab // CHAIN_CHUNK) * CHAIN_MAX_K * 2


def sample_chain(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor,
                 slots: Optional[torch.Tensor] = None, feedback: Optional[torch.Tensor] = None,
                 history: Optional[torch.Tensor] = None, history_len: Optional[torch.Tensor] = None,
                 penalise: bool = False) -> None:
    """The reference's sampling chain on the device: repeat penalty over the request's recent tokens
    (``history`` [slots, cap] rings with ``history_len`` [slots] tokens appended so far), the top-k
    logits (1 <= k <= CHAIN_MAX_K; greedy rows are k = 1), float64 probabilities, top-p and min-p
    cuts, the draw.  ``params`` [m, 8] float64 per row: temperature, top_k, top_p, min_p, repeat
    penalty, repeat_last_n, uniform number, unused.  ``logits`` is changed in place where a row
    penalises; the choice is appended to the request's ring and stored in ``feedback[slots[r]]``."""
    lib = library()
    m, v = logits.shape
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and out.is_contiguous()
    assert params.dtype == torch.float64 and params.is_contiguous() and tuple(params.shape) == (m, 8)
    assert scratch.dtype == torch.float32 and scratch.numel() >= chain_scratch_floats(m, v)
    _i32(slots, "slots"); _i32(feedback, "feedback"); _i32(history, "history"); _i32(history_len, "history_len")
    cap = history.shape[1] if history is not None else 0
    _check(lib.hfee_sample_chain(logits.data_ptr(), _rows(logits, "logits"), m, v, params.data_ptr(), _ptr(slots),
                                 _ptr(history), cap, _ptr(history_len), int(penalise), scratch.data_ptr(),
                                 scratch.numel(), out.data_ptr(), _ptr(feedback), _stream()), lib)
    count_launches(2 if penalise else 1)


ARGMAX_CHUNKS = 64


def argmax(logits: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor, slots: Optional[torch.Tensor] = None,
           feedback: Optional[torch.Tensor] = None) -> None:
    """out[r] = index of the first maximum of logits[r]; ``scratch`` holds rows * ARGMAX_CHUNKS * 2
    floats.  With ``slots`` and ``feedback`` the choice is also stored in ``feedback[slots[r]]``."""
    lib = library()
    assert logits.dtype == torch.float32 and out.dtype == torch.int32 and scratch.dtype == torch.float32
    _i32(slots, "slots"); _i32(feedback, "feedback")
    assert (slots is None) == (feedback is None)
    m, v = logits.shape
    assert scratch.numel() >= m * ARGMAX_CHUNKS * 2
    _check(lib.hfee_argmax(logits.data_ptr(), _rows(logits, "logits"), m, v, ARGMAX_CHUNKS, scratch.data_ptr(),
                           out.data_ptr(), _ptr(slots), _ptr(feedback), _stream()), lib)
    count_launches(1)


# the entry points the parts and the sampler launch through can be left out by class (see tag())
for _name in ("embed", "rmsnorm", "rope_table", "rope_cache_write", "swiglu", "linear", "linear_normed", "linear_swiglu", "linear_rope_cache",
              "linear_swiglu_normed", "paged_attention", "paged_attention_rope", "sample", "argmax", "sample_chain"):
    globals()[_name] = _measurable(globals()[_name])
del _name
