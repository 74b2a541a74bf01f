"""Python face of the CUDA kernel library (csrc/): loads the shared library through
ctypes and wraps each entry point in a function that takes torch tensors.

There is no fallback: if the library cannot be built or loaded, or a kernel refuses
its sizes, an exception says so.  Every wrapper launches on torch's current stream,
so calls are captured by a CUDA graph like any torch operation.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Optional

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
OUT_SAME, OUT_F32, OUT_ADD_F32, OUT_SWIGLU = 0, 1, 2, 3

_DT = {torch.float32: F32, torch.bfloat16: BF16}


class KernelError(RuntimeError):
    pass


_lib = None
_lock = threading.Lock()
launch_count = 0   # kernels launched through this module (bench.py reports it)

_c_int, _c_float, _c_void_p, _c_ll = ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_longlong

_SIGNATURES = {
    "rl_embedding": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_rmsnorm": [_c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_int, _c_float, _c_void_p],
    "rl_swiglu": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p],
    "rl_convert": [_c_void_p, _c_int, _c_void_p, _c_int, _c_ll, _c_void_p],
    "rl_random_fill": [_c_void_p, _c_int, _c_ll, ctypes.c_ulonglong, _c_float, _c_float, _c_void_p],
    "rl_gemm_simt": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int,
                     _c_int, _c_int, _c_void_p],
    "rl_rope_kv_write": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p,
                         _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_simt": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p,
                          _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int,
                          _c_void_p],
    "rl_repeat_penalty": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_int, _c_float, _c_void_p],
    "rl_argmax": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_sample_temperature": [_c_void_p, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "rl_sample_candidates": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_int,
                             _c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_decode": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                            _c_int, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_int, _c_void_p],
    "rl_attention_decode_plan": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_attention_decode_order": [_c_void_p, _c_void_p, _c_int, _c_int, _c_void_p, _c_void_p],
    "rl_attention_decode_places": [_c_int],
    "rl_attention_decode_ring_bytes": [_c_int],
    "rl_attention_decode_supported": [_c_int, _c_int, _c_int],
    "rl_attention_prefill": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p, _c_void_p,
                             _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float, _c_int, _c_void_p],
    "rl_attention_prefill_supported": [_c_int, _c_int, _c_int],
    "rl_attention_prefill_tc": [_c_void_p, _c_int, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int, _c_void_p, _c_void_p,
                                _c_void_p, _c_int, _c_int, _c_int, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_float,
                                _c_int, _c_void_p, _c_void_p, _c_void_p],
    "rl_attention_prefill_tc_supported": [_c_int, _c_int, _c_int],
    "rl_gemm_tc_supported": [_c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int],
    "rl_gemm_tc": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int,
                   _c_void_p, _c_int, _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_void_p],
    "rl_gemm_tc_splits": [_c_int, _c_int, _c_int],
    "rl_gemm_tc_qkv_rope_supported": [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int],
    "rl_gemm_tc_qkv_rope": [_c_void_p, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_int, _c_int, _c_int, _c_void_p,
                            _c_void_p, _c_int, _c_float, _c_void_p, _c_void_p, _c_void_p, _c_int, _c_void_p, _c_int,
                            _c_int, _c_int, _c_int, _c_void_p, _c_void_p, _c_void_p],
}


def library() -> ctypes.CDLL:
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        with _lock:
            if _lib is None:
                path = _build.build()
                try:
                    lib = ctypes.CDLL(path)
                except OSError as e:
                    raise KernelError(f"cannot load the kernel library {path}: {e}") from e
                lib.rl_last_error.restype = ctypes.c_char_p
                lib.rl_last_error.argtypes = []
                for name, args in _SIGNATURES.items():
                    fn = getattr(lib, name, None)
                    if fn is None:
                        raise KernelError(f"kernel library {path} lacks the entry point {name}")
                    fn.restype = _c_int
                    fn.argtypes = args
                if lib.rl_page_size() != PAGE_SIZE:
                    raise KernelError(f"the kernel library was built for pages of {lib.rl_page_size()} "
                                      f"tokens, the package expects {PAGE_SIZE}")
                _lib = lib
    return _lib


def library_file() -> str:
    library()
    return _build.library_path()


def _check(code: int, name: str) -> None:
    if code != 0:
        msg = library().rl_last_error().decode("utf-8", "replace")
        raise KernelError(f"{name} failed ({code}): {msg}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle (asked for on every
    launch: during graph capture it is the capturing stream)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _dt(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise KernelError(f"dtype {t.dtype} is not handled by the kernels (float32 and bfloat16 are)") from None


def _need(t: torch.Tensor, name: str, dtype=None, contiguous: bool = True) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} is on {t.device}; the kernels run on CUDA tensors only (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} has dtype {t.dtype}, expected {dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


# ----------------------------------------------------------------------------- wrappers
def embedding(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor, err_flag: torch.Tensor) -> None:
    """out[m, :] = table[ids[m], :] as float32.  err_flag (int32[1]) is set to 1 on a bad id."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    _need(err_flag, "err_flag", torch.int32)
    V, d = table.shape
    M = ids.numel()
    assert out.shape == (M, d)
    _check(library().rl_embedding(table.data_ptr(), _dt(table), ids.data_ptr(), out.data_ptr(), M, d, V,
                                  err_flag.data_ptr(), _stream()), "rl_embedding")
    _count()


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor, eps: float,
            rows: Optional[torch.Tensor] = None) -> None:
    """out[r] = rms_norm(x[rows[r]] if rows is given else x[r]) * weight."""
    _need(x, "x", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    d = x.shape[-1]
    n = out.shape[0]
    if rows is not None:
        _need(rows, "rows", torch.int32)
        assert rows.numel() == n
    else:
        assert x.shape[0] == n
    assert weight.numel() == d and out.shape[-1] == d
    _check(library().rl_rmsnorm(x.data_ptr(), weight.data_ptr(), out.data_ptr(), _dt(out), _ptr(rows), n, d,
                                float(eps), _stream()), "rl_rmsnorm")
    _count()


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up.  gate_up: [M, 2I] holding the gate in columns [0, I) and up
    in [I, 2I), or, interleaved, gate_i in column 2i and up_i in column 2i + 1."""
    _need(gate_up, "gate_up"); _need(out, "out", gate_up.dtype)
    M, two_i = gate_up.shape
    assert two_i % 2 == 0 and out.shape == (M, two_i // 2)
    _check(library().rl_swiglu(gate_up.data_ptr(), out.data_ptr(), _dt(out), M, two_i // 2, int(interleaved), _stream()),
           "rl_swiglu")
    _count()


def convert(src: torch.Tensor, dst: torch.Tensor) -> None:
    _need(src, "src"); _need(dst, "dst")
    assert src.numel() == dst.numel()
    _check(library().rl_convert(src.data_ptr(), _dt(src), dst.data_ptr(), _dt(dst), src.numel(), _stream()), "rl_convert")
    _count()


def random_fill(out: torch.Tensor, seed: int, mean: float, std: float) -> None:
    """out[i] = mean + std * z_i with z_i the library's reproducible near-normal number i of
    ``seed`` (csrc/random_fill.cu): the same values as ``weights.random_init.normal_values``
    computes on the host, bit for bit."""
    _need(out, "out")
    _check(library().rl_random_fill(out.data_ptr(), _dt(out), out.numel(), int(seed) & ((1 << 64) - 1), float(mean), float(std),
                                    _stream()), "rl_random_fill")
    _count()


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, out_mode: int,
              bias: Optional[torch.Tensor] = None) -> None:
    """out = a @ w.T (+ bias) on the CUDA cores.  a: [M, K] (rows may be strided),
    w: [N, K] contiguous, same dtype.  out_mode: OUT_SAME / OUT_F32 / OUT_ADD_F32."""
    _need(a, "a", contiguous=False); _need(w, "w", a.dtype); _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and out.stride(1) == 1
    if out_mode == OUT_SAME:
        assert out.dtype == a.dtype
    else:
        assert out.dtype == torch.float32
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == N
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else N
    _check(library().rl_gemm_simt(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), _dt(a), out_mode,
                                  M, N, K, lda, ldo, _stream()), "rl_gemm_simt")
    _count()


def rope_kv_write(qkv: torch.Tensor, positions: torch.Tensor, slot_of_token: torch.Tensor,
                  page_table: torch.Tensor, inv_freq: torch.Tensor, num_heads: int, num_kv_heads: int,
                  head_dim: int, rotary_dim: int, interleaved: bool,
                  k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor], value_dim: Optional[int] = None) -> None:
    """Rotates the query and key heads of qkv ([M, H*hd + G*hd + G*vd]) in place and writes keys
    and values at their tokens' places of the paged pools.  ``value_dim`` (default: head_dim)
    is the width of a value head."""
    vd = head_dim if value_dim is None else value_dim
    _need(qkv, "qkv"); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32)
    M = qkv.shape[0]
    if k_pool is not None:
        _need(k_pool, "k_pool", qkv.dtype); _need(v_pool, "v_pool", qkv.dtype)
        _need(slot_of_token, "slot_of_token", torch.int32); _need(page_table, "page_table", torch.int32)
        assert k_pool.shape[1:] == (num_kv_heads, page_size(), head_dim), k_pool.shape
        assert v_pool.shape[1:] == (num_kv_heads, page_size(), vd), v_pool.shape
        max_pages = page_table.shape[1]
    else:
        max_pages = 0
    assert inv_freq.numel() >= rotary_dim // 2
    _check(library().rl_rope_kv_write(
        qkv.data_ptr(), _dt(qkv), qkv.stride(0), positions.data_ptr(), _ptr(slot_of_token), _ptr(page_table),
        max_pages, inv_freq.data_ptr(), M, num_heads, num_kv_heads, head_dim, vd, rotary_dim, int(interleaved),
        _ptr(k_pool), _ptr(v_pool), _stream()), "rl_rope_kv_write")
    _count()


def attention_simt(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                   slot_of_token: torch.Tensor, positions: torch.Tensor, out: torch.Tensor,
                   num_heads: int, num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                   value_dim: Optional[int] = None) -> None:
    """q: [M, >= H*hd] (a view into the qkv buffer is fine), out: [M, H*vd] where vd is
    ``value_dim`` (default: head_dim), the width of a value head."""
    vd = head_dim if value_dim is None else value_dim
    _need(q, "q", contiguous=False); _need(k_pool, "k_pool", q.dtype); _need(v_pool, "v_pool", q.dtype)
    _need(out, "out", q.dtype); _need(page_table, "page_table", torch.int32)
    _need(slot_of_token, "slot_of_token", torch.int32); _need(positions, "positions", torch.int32)
    M = q.shape[0]
    assert q.stride(1) == 1
    ldq = q.stride(0) if M > 1 else num_heads * head_dim
    _check(library().rl_attention_simt(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), _dt(q), page_table.data_ptr(),
        page_table.shape[1], slot_of_token.data_ptr(), positions.data_ptr(), out.data_ptr(), out.stride(0),
        M, num_heads, num_kv_heads, head_dim, vd, float(scale), int(window), _stream()), "rl_attention_simt")
    _count()


def repeat_penalty(logits: torch.Tensor, recent: torch.Tensor, recent_len: torch.Tensor, penalty: float) -> None:
    _need(logits, "logits", torch.float32); _need(recent, "recent", torch.int32)
    _need(recent_len, "recent_len", torch.int32)
    rows, vocab = logits.shape
    assert recent.shape[0] == rows and recent_len.numel() == rows
    _check(library().rl_repeat_penalty(logits.data_ptr(), rows, vocab, recent.data_ptr(), recent_len.data_ptr(),
                                       recent.shape[1], float(penalty), _stream()), "rl_repeat_penalty")
    _count()


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    rows, vocab = logits.shape
    assert out.numel() == rows
    _check(library().rl_argmax(logits.data_ptr(), rows, vocab, out.data_ptr(), _stream()), "rl_argmax")
    _count()


def sample_temperature(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                       out: torch.Tensor, min_p: Optional[torch.Tensor] = None) -> None:
    _need(logits, "logits", torch.float32); _need(temperature, "temperature", torch.float32)
    _need(uniform, "uniform", torch.float32); _need(out, "out", torch.int32)
    rows, vocab = logits.shape
    assert temperature.numel() == rows and uniform.numel() == rows and out.numel() == rows
    if min_p is not None:
        _need(min_p, "min_p", torch.float32)
    _check(library().rl_sample_temperature(logits.data_ptr(), rows, vocab, temperature.data_ptr(),
                                           uniform.data_ptr(), _ptr(min_p), out.data_ptr(), _stream()),
           "rl_sample_temperature")
    _count()


PAGE_SIZE = 64


def page_size() -> int:
    """Tokens per cache page.  A constant on the Python side so that host-side code
    (allocators, their tests) runs without a GPU; checked against the value the
    kernels were compiled with when the library is loaded."""
    return PAGE_SIZE


# ----------------------------------------------------------------------------- tensor-core GEMM
_tc_err = {}


def _tc_error_word(device: torch.device) -> torch.Tensor:
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _tc_err:
        _tc_err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _tc_err[key]


def gemm_tc_splits(M: int, N: int, K: int) -> int:
    """Parts (cluster size) the kernel cuts the K range into for these shapes."""
    return int(library().rl_gemm_tc_splits(M, N, K))


def check_device_errors() -> None:
    """Raise if a kernel recorded an error on the device (a bounded wait that ran
    out).  Synchronizes; call it where the host waits for results anyway."""
    for key, t in _tc_err.items():
        code = int(t.item())
        if code != 0:
            t.zero_()
            raise KernelError(f"a tensor-core kernel on cuda:{key} gave up waiting (code {code}; matrix product: "
                              "1 = for a free stage, 2 = for a TMA load, 3 = for the accumulator, 4 = for a free "
                              "accumulator; prefill attention: 11 = producer, 12/13 = MMA issuer, 14 = softmax)")


def gemm_tc_supported(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> bool:
    """Whether the tensor-core kernel takes these operands (else the caller uses
    the CUDA-core kernel, which takes every shape): bf16, K and the row stride of
    ``a`` multiples of 8 elements, bases 16-byte aligned."""
    if a.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or not w.is_contiguous() or a.stride(1) != 1:
        return False
    M, K = a.shape
    lda = a.stride(0) if M > 1 else K
    return bool(library().rl_gemm_tc_supported(a.data_ptr(), w.data_ptr(), M, w.shape[0], K, lda))


def norm_pieces(num_columns: int) -> int:
    """How many partial sums of squares a row the matrix product writes for ``num_columns``
    output columns when it prepares the next norm (4 per tile of 128 columns)."""
    return 4 * (-(-num_columns // 128))


def gemm_tc(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, out_mode: int,
            bias: Optional[torch.Tensor] = None, force_splits: int = 0,
            row_sumsq: Optional[torch.Tensor] = None, row_eps: float = 0.0,
            norm_weight: Optional[torch.Tensor] = None, norm_out: Optional[torch.Tensor] = None,
            norm_sumsq: Optional[torch.Tensor] = None) -> None:
    """out = a @ w.T (+ bias) on the tensor cores (tcgen05).  a: [M, K] bf16, w: [N, K] bf16;
    out: bf16 (OUT_SAME) or float32 (OUT_F32 store, OUT_ADD_F32 add), or, with OUT_SWIGLU,
    bf16 [M, N/2] = silu(even columns) * odd columns of the product.  force_splits: 0 = the
    kernel's own choice of K parts; 1 to 8 = as given.

    An RMSNorm around the product can ride along.  ``row_sumsq`` [M, pieces] float32 with
    ``row_eps``: ``a`` holds ``x * norm weight`` and row m of the product is multiplied by
    ``rsqrt(sum(row_sumsq[m]) / K + row_eps)``.  ``norm_weight`` [N], ``norm_out`` [M, N]
    bf16, ``norm_sumsq`` [M, norm_pieces(N)] float32 (OUT_ADD_F32 only): also
    ``norm_out = out * norm_weight`` and the sums of squares of ``out``'s rows, in pieces."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16); _need(out, "out", contiguous=False)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.stride(1) == 1
    if out_mode == OUT_SWIGLU:      # rows of w are (gate_0, up_0, gate_1, ...): out = silu(gate) * up, [M, N/2]
        assert N % 2 == 0 and out.shape == (M, N // 2) and out.dtype == torch.bfloat16
    else:
        assert out.shape == (M, N)
        assert out.dtype == (torch.bfloat16 if out_mode == OUT_SAME else torch.float32)
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == N
    pieces = 0
    if row_sumsq is not None:
        _need(row_sumsq, "row_sumsq", torch.float32)
        assert row_sumsq.dim() == 2 and row_sumsq.shape[0] == M
        pieces = row_sumsq.shape[1]
    if norm_weight is not None:
        _need(norm_weight, "norm_weight", torch.float32); _need(norm_out, "norm_out", torch.bfloat16)
        _need(norm_sumsq, "norm_sumsq", torch.float32)
        assert out_mode == OUT_ADD_F32 and norm_weight.numel() == N and norm_out.shape == (M, N)
        assert norm_sumsq.shape == (M, norm_pieces(N))
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else out.shape[1]
    _check(library().rl_gemm_tc(a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), out_mode, M, N, K, lda, ldo,
                                _tc_error_word(a.device).data_ptr(), int(force_splits),
                                _ptr(row_sumsq), pieces, float(row_eps),
                                _ptr(norm_weight), _ptr(norm_out), N, _ptr(norm_sumsq), _stream()), "rl_gemm_tc")
    _count()


def gemm_tc_qkv_rope_supported(a: torch.Tensor, w: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int,
                               rotary_dim: int) -> bool:
    """Whether the QKV product of these operands can carry the rotary encoding and the cache
    write in its epilogue (head size 128 or 64 rotated whole, up to 64 tokens, a product that
    is split over K)."""
    if not gemm_tc_supported(a, w, None) or w.shape[0] != (num_heads + 2 * num_kv_heads) * head_dim:
        return False
    return bool(library().rl_gemm_tc_qkv_rope_supported(a.shape[0], num_heads, num_kv_heads, head_dim, rotary_dim, a.shape[1]))


def gemm_tc_qkv_rope(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor],
                     positions: torch.Tensor, slot_of_token: torch.Tensor, page_table: torch.Tensor,
                     inv_freq: torch.Tensor, interleaved: bool, num_heads: int, num_kv_heads: int,
                     k_pool: Optional[torch.Tensor], v_pool: Optional[torch.Tensor],
                     row_sumsq: Optional[torch.Tensor] = None, row_eps: float = 0.0) -> None:
    """qkv = a @ w.T (+ bias) with rotary encoding of the query and key heads and the write of
    keys and values into the paged cache, all in the product's epilogue.  Of ``out``
    [M, (H + 2G) * head_dim] bf16 only the query heads are written; keys and values go to the
    pools (``None``: nowhere).  The head size (128 or 64) follows from ``w``'s rows.
    ``row_sumsq`` / ``row_eps``: as in ``gemm_tc``."""
    _need(a, "a", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16); _need(out, "out", torch.bfloat16, contiguous=False)
    _need(positions, "positions", torch.int32); _need(slot_of_token, "slot_of_token", torch.int32)
    _need(page_table, "page_table", torch.int32); _need(inv_freq, "inv_freq", torch.float32)
    M, K = a.shape
    hd = w.shape[0] // (num_heads + 2 * num_kv_heads)
    assert hd in (64, 128) and w.shape == ((num_heads + 2 * num_kv_heads) * hd, K)
    assert out.shape == (M, w.shape[0]) and out.stride(1) == 1
    assert positions.numel() == M and slot_of_token.numel() == M and inv_freq.numel() == hd // 2
    if bias is not None:
        _need(bias, "bias", torch.float32)
        assert bias.numel() == w.shape[0]
    if k_pool is not None:
        _need(k_pool, "k_pool", torch.bfloat16); _need(v_pool, "v_pool", torch.bfloat16)
        assert k_pool.shape[1:] == (num_kv_heads, PAGE_SIZE, hd) and v_pool.shape == k_pool.shape
    pieces = 0
    if row_sumsq is not None:
        _need(row_sumsq, "row_sumsq", torch.float32)
        assert row_sumsq.dim() == 2 and row_sumsq.shape[0] == M
        pieces = row_sumsq.shape[1]
    lda = a.stride(0) if M > 1 else K
    ldo = out.stride(0) if M > 1 else out.shape[1]
    _check(library().rl_gemm_tc_qkv_rope(
        a.data_ptr(), w.data_ptr(), _ptr(bias), out.data_ptr(), M, K, lda, ldo, _tc_error_word(a.device).data_ptr(),
        _ptr(row_sumsq), pieces, float(row_eps), positions.data_ptr(), slot_of_token.data_ptr(), page_table.data_ptr(),
        page_table.shape[1], inv_freq.data_ptr(), 1 if interleaved else 0, num_heads, num_kv_heads, hd,
        _ptr(k_pool), _ptr(v_pool), _stream()), "rl_gemm_tc_qkv_rope")
    _count()


# ----------------------------------------------------------------------------- decode attention
_num_sms = {}


def num_sms() -> int:
    """SMs of the current device, asked from the device once."""
    dev = torch.cuda.current_device() if torch.cuda.is_available() else -1
    if dev not in _num_sms:
        lib = library()
        lib.rl_sm_count.restype = _c_int
        lib.rl_sm_count.argtypes = []
        _num_sms[dev] = int(lib.rl_sm_count())
    return _num_sms[dev]


def attention_decode_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_decode_supported(num_heads, num_kv_heads, head_dim))


# One sequence alone: up to this many cached tokens its eight chunks run as one cluster that
# combines through shared memory (one kernel; 6.0 us against 7.9 us at 1,024 tokens, equal at
# 4,096); beyond, sixteen chunks and the combining kernel (32,768 tokens: 30 us against 52 us;
# 131,072: 95 us against 198 us - 64 CTAs cannot keep the memory busy).  A captured step keeps
# its grid, so the step carries on which side of this it lies (``StepState.long_context``).
LONG_CONTEXT = 6144


def decode_splits(num_seqs: int, num_kv_heads: int) -> int:
    """Splits of the context per (sequence, KV head): enough CTAs for about one and a
    half per SM, at most 8 for a batch and 16 for one sequence (measured best at 1 to 64
    sequences of 800 and 4,096 tokens), and at least 2 for a batch, so that its chunks are
    dealt by length: beside short sequences a long one is then cut in pieces (64 sequences of
    256 to 8,700 tokens: 115 us as one chunk each, 95 us dealt), and a sequence that remains
    one chunk costs nothing more for it.  Depends on the batch's size only, so that a
    captured step keeps its grid."""
    most = 16 if num_seqs == 1 else 8
    least = 1 if num_seqs == 1 else 2
    return max(least, min(most, -(-3 * num_sms() // (2 * num_seqs * num_kv_heads))))


# Several sequences: how far the longest lies above the mean of all decides whether equal chunks a
# sequence (a cluster, one kernel) or chunks dealt by length (and a second kernel that combines
# them) serve them better; a captured step keeps its launches, so the step carries the class
# (``StepState.length_spread``): 0 = within EVEN_SPREAD tokens, 1 = within NEAR_SPREAD, 2 = within
# FAR_SPREAD and the longest no more than one in LONGEST_SHARE of all tokens (63 sequences of 100
# tokens beside one of 4,000, whole: 50 us, dealt: 24 us), 3 = the rest.
EVEN_SPREAD = 16
NEAR_SPREAD = 768
FAR_SPREAD = 4096
LONGEST_SHARE = 20


def length_spread(kv_lens: Sequence[int]) -> int:
    """The class of a batch's lengths (see above); one sequence is class 0."""
    n = len(kv_lens)
    over = max(kv_lens) * n - sum(kv_lens)        # (longest - mean) * n, in integers
    if over <= NEAR_SPREAD * n:
        return 0 if over <= EVEN_SPREAD * n else 1
    return 2 if over <= FAR_SPREAD * n and max(kv_lens) * LONGEST_SHARE <= sum(kv_lens) else 3


def decode_places(head_dim: int) -> int:
    """CTAs of the decode kernel the GPU holds at once at this head size (296 at 128, 444 at 64)."""
    n = int(library().rl_attention_decode_places(int(head_dim)))
    if n <= 0:
        _check(n or -1, "rl_attention_decode_places")
    return n


def decode_order_wanted(num_seqs: int, num_kv_heads: int, head_dim: int) -> bool:
    """Whole sequences that are more CTAs than the GPU holds at once (and keep 30 MB in flight
    among them) start in the order of their lengths, the longest first.  Sequences of 128 to 2,047
    tokens, in order against dealt chunks: head size 128, 40 sequences 36.4 / 38.6 us, 48: 39.1 /
    43.2, 56: 40.7 / 48.8, 64: 43.0 / 54.3 (6.45 TB/s; 53 us sorted but KV head by KV head, 52.7
    unsorted); head size 64, 96: 38.4 / 40.5, 128: 42.0 / 50.2, but 64 (24 MB in flight): 31.7 /
    30.4.  The order kernel takes up to 1,024 sequences."""
    ctas = num_seqs * num_kv_heads
    ring = int(library().rl_attention_decode_ring_bytes(int(head_dim)))
    return ctas > decode_places(head_dim) and ctas * ring >= 30_000_000 and num_seqs <= 1024


def decode_cluster_size(num_seqs: int, num_kv_heads: int, head_dim: int, long_context: bool, spread: int) -> int:
    """How the decode attention cuts the sequences of a step: 8, 4 or 2 = so many equal chunks a
    sequence as one cluster; 1 = every sequence whole in one CTA a KV head; 0 = chunks dealt by
    length and a combining kernel.  One sequence alone: eight chunks up to the long-context mark.
    Whole sequences in order (``decode_order_wanted``) serve every batch up to class 2.  Else,
    lengths that are equal (class 0) or near (class 1): where two chunks a sequence no longer fit
    the GPU at once, every sequence whole if that keeps 15 MB in flight (head size 64, 4,096
    tokens a sequence, whole against dealt: 32 sequences 59 / 49 us, 40: 61 / 73); else the largest
    power of two within ``decode_splits`` - for class 1 only if nothing is lost to the rounding.
    Whole decode steps of the 8B shape, 1,024 tokens a sequence, against dealt chunks: 2 sequences
    2.91 / 2.95 ms, 6: 3.04 / 3.12, 8: 3.10 / 3.18, 16: 3.30 / 3.38, 20: 3.57 / 3.84, 32: 3.81 / 4.05,
    64: 4.93 / 5.23; lengths 1,024 +- 30 %: 8: 3.13 / 3.19, 16: 3.36 / 3.42, 32: 3.84 / 4.06, 64: 5.05 /
    5.20, but 4 sequences (7 splits rounded to 4): 3.07 / 3.04, so those stay dealt; with the
    longest 80 % above the mean the two are about even, and beyond, the longest sequence's few
    CTAs would finish last.  (A cluster of two at 20 sequences, 320 CTAs for 296 places: 17.7 us
    against 10.9 us whole at 512 tokens.)"""
    splits = decode_splits(num_seqs, num_kv_heads)
    if num_seqs == 1:
        return 8 if splits >= 8 and not long_context else 0
    if splits < 2:
        return 0
    if decode_order_wanted(num_seqs, num_kv_heads, head_dim):
        return 1 if spread <= 2 else 0
    if spread > 1:
        return 0
    places, ctas = decode_places(head_dim), num_seqs * num_kv_heads
    if ctas * 2 > places:
        return 1 if ctas * int(library().rl_attention_decode_ring_bytes(int(head_dim))) >= 15_000_000 else 0
    size = 8 if splits >= 8 else 4 if splits >= 4 else 2
    if spread == 1 and size != splits:
        return 0
    return size if ctas * size <= places else 0


def decode_order(seq_slots: torch.Tensor, kv_lens: torch.Tensor, window: int) -> torch.Tensor:
    """A plan of whole sequences, the longest first (inside ``window`` if it is not 0), made on the
    device: for ``attention_decode`` with one split.  At most 1,024 sequences."""
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = seq_slots.numel()
    assert kv_lens.numel() == B
    plan = torch.empty(6 * B, dtype=torch.int32, device=seq_slots.device)     # rl_attention_decode_order_ints
    _check(library().rl_attention_decode_order(seq_slots.data_ptr(), kv_lens.data_ptr(), B, int(window), plan.data_ptr(), _stream()),
           "rl_attention_decode_order")
    _count(1)
    return plan


def decode_scratch_floats(num_seqs: int, num_heads: int, head_dim: int, num_splits: int) -> int:
    if num_splits <= 1:
        return 0
    return num_seqs * num_heads * num_splits * (head_dim + 2)


def decode_plan(seq_slots: torch.Tensor, kv_lens: torch.Tensor, window: int, num_splits: int) -> Optional[torch.Tensor]:
    """Deals ``B * num_splits`` chunks to the sequences by their lengths, on the device.
    The plan serves every ``attention_decode`` call of the step with the same window and
    splits (``None`` with one split: every sequence is one chunk)."""
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = seq_slots.numel()
    if num_splits <= 1 or B == 0:
        return None
    plan = torch.empty(4 * B * num_splits + 2 * B, dtype=torch.int32, device=seq_slots.device)
    _check(library().rl_attention_decode_plan(seq_slots.data_ptr(), kv_lens.data_ptr(), B, int(window), int(num_splits),
                                              plan.data_ptr(), _stream()), "rl_attention_decode_plan")
    _count(1)
    return plan


def attention_decode(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                     seq_slots: torch.Tensor, kv_lens: torch.Tensor, out: torch.Tensor, num_heads: int,
                     num_kv_heads: int, head_dim: int, scale: float, window: int = 0,
                     num_splits: Optional[int] = None, scratch: Optional[torch.Tensor] = None,
                     plan: Optional[torch.Tensor] = None, cluster: bool = False) -> None:
    """One token per sequence over the bf16 cache, split over the context (tensor cores).
    q: [B, >= H*hd] bf16 (a view into the qkv buffer is fine); out: [B, H*hd] bf16.
    ``num_splits``: chunks per sequence; with a ``plan`` (from ``decode_plan`` with the
    same sequences, window and splits) that many on average, dealt to the sequences by
    length; with one split a ``plan`` from ``decode_order`` starts the longest sequences first.
    ``cluster`` (2, 4 or 8 splits, no plan): the chunks of a sequence run as a
    thread-block cluster and combine through shared memory - no scratch, one kernel."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(seq_slots, "seq_slots", torch.int32)
    _need(kv_lens, "kv_lens", torch.int32)
    B = q.shape[0]
    assert seq_slots.numel() == B and kv_lens.numel() == B and q.stride(1) == 1
    if num_splits is None:
        num_splits = decode_splits(B, num_kv_heads)
    if cluster:
        assert plan is None and scratch is None and num_splits in (2, 4, 8)
    need = 0 if cluster else decode_scratch_floats(B, num_heads, head_dim, num_splits)
    if num_splits > 1 and scratch is None and not cluster:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
        assert scratch.numel() >= need
    if plan is not None:
        _need(plan, "plan", torch.int32)
        assert plan.numel() >= 4 * B * num_splits + 2 * B
    ldq = q.stride(0) if B > 1 else max(q.stride(0), num_heads * head_dim)
    _check(library().rl_attention_decode(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        seq_slots.data_ptr(), kv_lens.data_ptr(), out.data_ptr(), out.stride(0), _ptr(scratch), _ptr(plan), B,
        num_heads, num_kv_heads, head_dim, float(scale), int(window), int(num_splits), _stream()), "rl_attention_decode")
    _count(2 if num_splits > 1 and not cluster else 1)


# ----------------------------------------------------------------------------- prefill attention
PREFILL_QTILE = 64


def attention_prefill_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_prefill_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                      cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, kv_lens: torch.Tensor, q_lens,
                      out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                      window: int = 0) -> None:
    """Causal attention of packed query tokens over the bf16 cache (tensor cores).
    q: [M, >= H*hd] bf16; cu_seqlens [B+1], seq_slots [B], kv_lens [B] on the device;
    q_lens: host list of tokens per sequence; out: [M, H*hd] bf16."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = len(q_lens)
    assert cu_seqlens.numel() == B + 1 and seq_slots.numel() == B and kv_lens.numel() == B
    assert q.shape[0] == sum(q_lens) and q.stride(1) == 1
    tiles = sum(-(-n // PREFILL_QTILE) for n in q_lens)
    ldq = q.stride(0) if q.shape[0] > 1 else max(q.stride(0), num_heads * head_dim)
    _check(library().rl_attention_prefill(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), page_table.data_ptr(), page_table.shape[1],
        cu_seqlens.data_ptr(), seq_slots.data_ptr(), kv_lens.data_ptr(), B, tiles, out.data_ptr(), out.stride(0),
        num_heads, num_kv_heads, head_dim, float(scale), int(window), _stream()), "rl_attention_prefill")
    _count()


PREFILL_TC_QTILE = 128


def prefill_tile_order(q_lens, kv_lens, device) -> torch.Tensor:
    """For the tcgen05 prefill attention: the step's 128-query tiles as (sequence, tile of the
    sequence) pairs by falling number of keys (a tile attends to its sequence's cached prefix and
    to the step's tokens up to its own last one), int32 [tiles, 2] on the device.  Made once a
    step from the host's copies of the lengths and used by every layer."""
    items = []
    for b, (nq, nkv) in enumerate(zip(q_lens, kv_lens)):
        first = nkv - nq
        for t in range(-(-nq // PREFILL_TC_QTILE)):
            items.append((-(first + min(nq, (t + 1) * PREFILL_TC_QTILE)), b, t))
    items.sort()
    return torch.tensor([[b, t] for _, b, t in items], dtype=torch.int32).to(device, non_blocking=True)


def attention_prefill_tc_supported(dtype: torch.dtype, num_heads: int, num_kv_heads: int, head_dim: int) -> bool:
    return dtype == torch.bfloat16 and bool(library().rl_attention_prefill_tc_supported(num_heads, num_kv_heads, head_dim))


def attention_prefill_tc(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
                         cu_seqlens: torch.Tensor, seq_slots: torch.Tensor, kv_lens: torch.Tensor, q_lens,
                         out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                         window: int = 0, tile_order: Optional[torch.Tensor] = None) -> None:
    """The same as ``attention_prefill`` on tcgen05 tensor cores (head size 64 or 128).  The cache
    pools must hold finite values everywhere (the cache zero-fills them when it allocates them).
    ``tile_order``: what ``prefill_tile_order`` made for this step (the blocks then start heaviest first)."""
    _need(q, "q", torch.bfloat16, contiguous=False); _need(k_pool, "k_pool", torch.bfloat16)
    _need(v_pool, "v_pool", torch.bfloat16); _need(out, "out", torch.bfloat16)
    _need(page_table, "page_table", torch.int32); _need(cu_seqlens, "cu_seqlens", torch.int32)
    _need(seq_slots, "seq_slots", torch.int32); _need(kv_lens, "kv_lens", torch.int32)
    B = len(q_lens)
    assert cu_seqlens.numel() == B + 1 and seq_slots.numel() == B and kv_lens.numel() == B
    assert q.shape[0] == sum(q_lens) and q.stride(1) == 1
    tiles = sum(-(-n // PREFILL_TC_QTILE) for n in q_lens)
    if tile_order is not None:
        _need(tile_order, "tile_order", torch.int32)
        assert tile_order.numel() == 2 * tiles
    ldq = q.stride(0) if q.shape[0] > 1 else max(q.stride(0), num_heads * head_dim)
    _check(library().rl_attention_prefill_tc(
        q.data_ptr(), ldq, k_pool.data_ptr(), v_pool.data_ptr(), k_pool.shape[0], page_table.data_ptr(),
        page_table.shape[1], cu_seqlens.data_ptr(), seq_slots.data_ptr(), kv_lens.data_ptr(), B, tiles, q.shape[0],
        out.data_ptr(), out.stride(0), num_heads, num_kv_heads, head_dim, float(scale), int(window),
        _tc_error_word(q.device).data_ptr(), _ptr(tile_order), _stream()), "rl_attention_prefill_tc")
    _count()


# ----------------------------------------------------------------------------- attention dispatch
def attention(q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor, page_table: torch.Tensor,
              step, out: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
              window: int = 0, value_dim: Optional[int] = None) -> None:
    """Attention of the step's tokens over the cache; picks the kernel for the
    dtype and the shape of the step.  ``step`` carries positions, slots and
    sequence boundaries (engine.step.StepState).  Value heads of another width than the
    key heads (``value_dim``) run on the any-shape kernel; the tensor-core kernels take
    one width for both."""
    if value_dim is not None and value_dim != head_dim:
        attention_simt(q, k_pool, v_pool, page_table, step.slot_of_token, step.positions, out,
                       num_heads, num_kv_heads, head_dim, scale, window, value_dim=value_dim)
        return
    if step.is_decode and attention_decode_supported(q.dtype, num_heads, num_kv_heads, head_dim):
        splits = decode_splits(q.shape[0], num_kv_heads)
        cluster = decode_cluster_size(q.shape[0], num_kv_heads, head_dim, getattr(step, "long_context", False),
                                      getattr(step, "length_spread", 3))
        if cluster:
            # nothing to deal: equal chunks a sequence as one cluster, combined through shared memory,
            # or every sequence whole
            order = None
            derived = getattr(step, "derived", None)
            if cluster == 1 and derived is not None and decode_order_wanted(q.shape[0], num_kv_heads, head_dim):
                order = derived.get(("decode_order", int(window)))
                if order is None:
                    order = derived[("decode_order", int(window))] = decode_order(step.seq_slots, step.kv_lens, window)
            attention_decode(q, k_pool, v_pool, page_table, step.seq_slots, step.kv_lens, out,
                             num_heads, num_kv_heads, head_dim, scale, window, num_splits=cluster, plan=order,
                             cluster=cluster > 1)
            return
        plan = None
        derived = getattr(step, "derived", None)     # what layers of one step share
        if splits > 1 and q.shape[0] > 1 and derived is not None:
            key = ("decode_plan", int(window), splits)
            plan = derived.get(key)
            if plan is None:
                plan = derived[key] = decode_plan(step.seq_slots, step.kv_lens, window, splits)
        attention_decode(q, k_pool, v_pool, page_table, step.seq_slots, step.kv_lens, out,
                         num_heads, num_kv_heads, head_dim, scale, window, num_splits=splits, plan=plan)
        return
    if not step.is_decode and attention_prefill_tc_supported(q.dtype, num_heads, num_kv_heads, head_dim) \
            and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0:
        order = None
        derived = getattr(step, "derived", None)
        if derived is not None and len(step.q_lens) > 1:     # one sequence: the kernel's own reverse order is the heaviest first
            order = derived.get("prefill_tile_order")
            if order is None:
                order = derived["prefill_tile_order"] = prefill_tile_order(step.q_lens, step.kv_lens_host, q.device)
        attention_prefill_tc(q, k_pool, v_pool, page_table, step.cu_seqlens, step.seq_slots, step.kv_lens,
                             step.q_lens, out, num_heads, num_kv_heads, head_dim, scale, window, tile_order=order)
        return
    if not step.is_decode and attention_prefill_supported(q.dtype, num_heads, num_kv_heads, head_dim):
        attention_prefill(q, k_pool, v_pool, page_table, step.cu_seqlens, step.seq_slots, step.kv_lens,
                          step.q_lens, out, num_heads, num_kv_heads, head_dim, scale, window)
        return
    attention_simt(q, k_pool, v_pool, page_table, step.slot_of_token, step.positions, out,
                   num_heads, num_kv_heads, head_dim, scale, window)


from .sampling.config import MAX_TOP_K  # noqa: E402  (one definition, host side)


def sample_candidates(logits: torch.Tensor, temperature: torch.Tensor, uniform: torch.Tensor,
                      min_p: torch.Tensor, out: torch.Tensor,
                      topk_rows: Optional[torch.Tensor], topk_k: Optional[torch.Tensor], topk_p: Optional[torch.Tensor],
                      topp_rows: Optional[torch.Tensor], topp_p: Optional[torch.Tensor]) -> None:
    """Rows that sample from a candidate set.  ``topk_rows`` (int32 row indices, on the
    device) with their ``topk_k`` (int32, each at most ``MAX_TOP_K``) and ``topk_p`` (float32)
    take the top-k path; ``topp_rows`` with ``topp_p`` the top-p path over the whole
    vocabulary; ``None`` = no such rows.  temperature / uniform / min_p / out are indexed by
    logits row."""
    _need(logits, "logits", torch.float32); _need(out, "out", torch.int32)
    _need(temperature, "temperature", torch.float32); _need(uniform, "uniform", torch.float32)
    _need(min_p, "min_p", torch.float32)
    n_k = n_p = 0
    if topk_rows is not None:
        _need(topk_rows, "topk_rows", torch.int32); _need(topk_k, "topk_k", torch.int32); _need(topk_p, "topk_p", torch.float32)
        n_k = topk_rows.numel()
        assert topk_k.numel() == n_k and topk_p.numel() == n_k
    if topp_rows is not None:
        _need(topp_rows, "topp_rows", torch.int32); _need(topp_p, "topp_p", torch.float32)
        n_p = topp_rows.numel()
        assert topp_p.numel() == n_p
    if n_k == 0 and n_p == 0:
        return
    _check(library().rl_sample_candidates(logits.data_ptr(), logits.shape[1], _ptr(topk_rows), _ptr(topk_k), _ptr(topk_p),
                                          n_k, _ptr(topp_rows), _ptr(topp_p), n_p,
                                          temperature.data_ptr(), uniform.data_ptr(), min_p.data_ptr(), out.data_ptr(),
                                          _stream()), "rl_sample_candidates")
    _count((1 if n_k else 0) + (1 if n_p else 0))
