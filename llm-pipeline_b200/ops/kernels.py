"""Python bindings of the CUDA entry points (``csrc/*.cu``), one function per kernel.

Arguments are CUDA tensors; the functions check types, contiguity and sizes, pass raw pointers
and the current stream to the library, and raise ``KernelError`` with the library's message when
an entry point refuses its arguments. There is no CPU implementation behind these functions: a
tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import ctypes
import os
from typing import Optional, Sequence

import torch

from .build import library

F32, BF16 = 0, 1
_P = ctypes.c_void_p
_I = ctypes.c_int
_L = ctypes.c_long
_F = ctypes.c_float


class KernelError(RuntimeError):
    pass


def dtype_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {dtype}; the kernels take float32 and bfloat16")


_SIGNATURES = {
    "llmp_embedding": [_P, _P, _I, _P, _I, _I, _I, _P],
    "llmp_rope_tables": [_P, _P, _F, _P, _P, _I, _I, _P],
    "llmp_add_rmsnorm": [_P, _P, _P, _I, _P, _I, _F, _P, _I, _P, _I, _I, _P],
    "llmp_qkv_post": [_P, _I, _P, _I, _P, _P, _I, _F, _P, _P, _I, _P, _P, _I, _I, _I, _I, _I, _P],
    "llmp_swiglu": [_P, _P, _I, _I, _I, _P],
    "llmp_gemm_simt": [_P, _P, _P, _I, _P, _I, _I, _I, _I, _I, _L, _L, _L, _P],
    "llmp_gemm_skinny": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P],
    "llmp_gemm_tc": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream_swiglu": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_gemm_stream_tc": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _P, _P],
    "llmp_paged_attention": [_P, _L, _P, _L, _P, _I, _I, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _F, _I,
                             _P, _P],
    "llmp_gemm_stream_fused": [_P, _P, _P, _I, _I, _I, _I, _L, _L, _L, _I, _P, _I, _F, _F, _P, _L, _P, _I, _P, _L, _P, _P, _P],
    "llmp_decode_attention": [_P, _L, _P, _L, _P, _I, _I, _P, _I, _P, _I, _I, _I, _I, _I, _I, _I, _F, _P, _L, _P, _I, _P, _P],
    "llmp_argmax": [_P, _L, _I, _I, _P, _P, _P],
    "llmp_repetition_penalty": [_P, _L, _I, _I, _P, _P, _P, _P],
    "llmp_sample": [_P, _L, _I, _I, _P, _P, _P, _P],
    "llmp_entropy": [_P, _L, _I, _I, _F, _P, _P],
    "llmp_bounded_wait_check": [_P, _I, _P, _P],
    "llmp_gemm_stream_chain": [_P, _I, _I, _P, _P, _P],
}
_bound = {}
launch_count = 0   # kernels of this library launched so far (captured launches count once per capture)


def _fn(name: str):
    fn = _bound.get(name)
    if fn is None:
        lib = library()
        fn = getattr(lib, name)
        fn.argtypes = _SIGNATURES[name]
        fn.restype = ctypes.c_int
        _bound[name] = fn
    return fn


def _call(name: str, *args) -> None:
    global launch_count
    launch_count += 1
    rc = _fn(name)(*args)
    if rc != 0:
        lib = library()
        lib.llmp_last_error.restype = ctypes.c_char_p
        raise KernelError(lib.llmp_last_error().decode(errors="replace"))


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    if t is None:
        return None
    if not t.is_cuda:
        raise KernelError("a kernel was given a tensor that is not on a CUDA device; this engine has no CPU path")
    return t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current CUDA stream of the current device as a raw handle (the fast accessor where torch has it:
    ``torch.cuda.current_stream()`` costs about 15 microseconds a call, several milliseconds per eager step)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


def _need(cond: bool, message: str) -> None:
    if not cond:
        raise KernelError(message)


def _i32(t: torch.Tensor, name: str) -> None:
    _need(t.dtype == torch.int32 and t.is_contiguous(), f"{name} must be a contiguous int32 tensor")


def tokens_per_attention_tile(num_heads: int, num_kv_heads: int, dtype: torch.dtype = torch.float32,
                              head_dim: int = 0, page_size: int = 0) -> int:
    """Query tokens per tile of the general attention kernel that serves this type, head size and page
    size (0: not known, which rules out the kernels that depend on the page size)."""
    fn = library().llmp_attention_tokens_per_tile
    fn.argtypes = [_I, _I, _I, _I, _I]
    fn.restype = _I
    n = fn(num_heads, num_kv_heads, dtype_code(dtype), head_dim, page_size)
    _need(n > 0, f"{num_heads} query heads cannot share {num_kv_heads} key/value heads")
    return n


def attention_max_segments(num_heads: int, num_kv_heads: int, dtype: torch.dtype, head_dim: int, page_size: int) -> int:
    """How many items of the tile list may share the keys of one tile in the general attention kernel that serves
    these sizes (1: it takes whole tiles only)."""
    fn = library().llmp_attention_max_segments
    fn.argtypes = [_I, _I, _I, _I, _I]
    fn.restype = _I
    return int(fn(num_heads, num_kv_heads, dtype_code(dtype), head_dim, page_size))


ATTENTION_MAX_PLACES = 8192          # places for the sums of items that share a tile, per launch
_attention_counters: dict = {}
_place_floats: Optional[int] = None


def attention_place_floats() -> int:
    global _place_floats
    if _place_floats is None:
        fn = library().llmp_attention_place_floats
        fn.argtypes = []
        fn.restype = _L
        _place_floats = int(fn())
    return _place_floats


def attention_counters(device: torch.device, count: int) -> torch.Tensor:
    """Counters with which the items that share a tile find out who finishes last; every launch leaves them zero.
    One set per device, as for ``decode_counters``."""
    key = torch.device(device).index or 0
    counters = _attention_counters.get(key)
    if counters is None or counters.numel() < count:
        _need(not torch.cuda.is_current_stream_capturing(), "attention counters must exist before a graph is captured")
        counters = _attention_counters[key] = torch.zeros(max(count, 65536), dtype=torch.int32, device=device)
    return counters


def embedding(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, :] = float32(table[ids[n], :])"""
    _i32(ids, "ids")
    _need(table.dim() == 2 and table.is_contiguous(), "embedding table must be a contiguous matrix")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (ids.numel(), table.shape[1]),
          "embedding output must be float32 [tokens, hidden]")
    _call("llmp_embedding", _ptr(ids), _ptr(table), dtype_code(table.dtype), _ptr(out), ids.numel(),
          table.shape[1], table.shape[0], _stream())
    return out


def rope_tables(positions: torch.Tensor, inv_freq: torch.Tensor, scaling: float, cos: torch.Tensor,
                sin: torch.Tensor) -> None:
    """cos/sin[n, j] = cos/sin(float(positions[n]) * inv_freq[j]) * scaling, all float32."""
    _i32(positions, "positions")
    half = inv_freq.numel()
    _need(inv_freq.dtype == torch.float32 and inv_freq.is_contiguous(), "inv_freq must be contiguous float32")
    for t in (cos, sin):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (positions.numel(), half),
              "rotary tables must be float32 [tokens, rotary_dim / 2]")
    _call("llmp_rope_tables", _ptr(positions), _ptr(inv_freq), float(scaling), _ptr(cos), _ptr(sin),
          positions.numel(), half, _stream())


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], weight: torch.Tensor, eps: float,
                out: torch.Tensor, delta_bias: Optional[torch.Tensor] = None,
                rows: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x = residual + delta (+ delta_bias); residual = x (unless ``rows`` selects rows);
    out = weight * (x * rsqrt(mean(x^2) + eps)).  residual is float32, delta/out have the compute type."""
    H = residual.shape[-1]
    _need(residual.dtype == torch.float32 and residual.is_contiguous() and residual.dim() == 2,
          "residual must be a contiguous float32 matrix")
    M = rows.numel() if rows is not None else residual.shape[0]
    _need(out.is_contiguous() and out.shape == (M, H), "norm output has the wrong shape")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.is_contiguous() and delta.shape == residual.shape,
              "delta must match the residual's shape and the output's type")
    _need(weight.numel() == H and weight.is_contiguous(), "norm weight has the wrong size")
    if delta_bias is not None:
        _need(delta_bias.numel() == H and delta_bias.is_contiguous(), "delta bias has the wrong size")
    if rows is not None:
        _i32(rows, "rows")
    _call("llmp_add_rmsnorm", _ptr(residual), _ptr(delta), _ptr(delta_bias),
          dtype_code(delta_bias.dtype) if delta_bias is not None else F32, _ptr(weight), dtype_code(weight.dtype),
          float(eps), _ptr(out), dtype_code(out.dtype), _ptr(rows), M, H, _stream())
    return out


# ---- the library product into a float32 residual ---------------------------------------------------------------------
_cublas = None
_CUDA_R_16BF, _CUDA_R_32F, _CUBLAS_COMPUTE_32F, _CUBLAS_OP_N, _CUBLAS_OP_T, _CUBLAS_GEMM_DEFAULT = 14, 0, 68, 0, 1, -1


def _cublas_gemm_ex():
    """cuBLAS's cublasGemmEx from the library that torch has loaded (None when it cannot be had)."""
    global _cublas
    if _cublas is None:
        _cublas = False
        for name in ("libcublas.so.12", "libcublas.so"):
            try:
                fn = ctypes.CDLL(name).cublasGemmEx
            except (OSError, AttributeError):
                continue
            fn.restype = ctypes.c_int
            fn.argtypes = [_P, _I, _I, _I, _I, _I, _P, _P, _I, _I, _P, _I, _I, _P, _P, _I, _I, _I, _I]
            _cublas = fn
            break
    return _cublas or None


_ONE = ctypes.c_float(1.0)
_ONE_REF = ctypes.byref(_ONE)


def library_add_product(residual: torch.Tensor, x: torch.Tensor, w: torch.Tensor) -> bool:
    """residual[M, N] (float32) += x[M, K] @ w[N, K]^T (bfloat16 operands, float32 sums) by the library's matrix
    product with the residual as its float32 C operand: the product is never rounded to bfloat16 and the norm kernel
    after it has nothing to add. On torch's cuBLAS handle and current stream, like ``torch.mm``; where the engine uses
    a library product for the rows of a prompt portion (the reference's ``nn.Linear`` is the same library,
    src/llm_pipeline/models/qwen3/custom_builder.py:124-131). False, and nothing done, when the operands are not of
    these types, not row-major, not 16-byte aligned, or the library cannot be had."""
    gemm = _cublas or _cublas_gemm_ex()
    M, K = x.shape
    N = w.shape[0]
    if (not gemm or residual.dtype != torch.float32 or x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or M == 0 or
            not residual.is_cuda or x.stride(1) != 1 or w.stride(1) != 1 or residual.stride(1) != 1 or w.shape[1] != K or
            residual.shape != (M, N)):
        return False
    xp, wp, rp = x.data_ptr(), w.data_ptr(), residual.data_ptr()
    if (xp | wp | rp) % 16:
        return False
    # row-major residual[M, N] is column-major [N, M]: (w as [K, N] column-major, transposed) times (x as [K, M])
    rc = gemm(torch.cuda.current_blas_handle(), _CUBLAS_OP_T, _CUBLAS_OP_N, N, M, K, _ONE_REF, wp, _CUDA_R_16BF, w.stride(0),
              xp, _CUDA_R_16BF, x.stride(0), _ONE_REF, rp, _CUDA_R_32F, residual.stride(0), _CUBLAS_COMPUTE_32F,
              _CUBLAS_GEMM_DEFAULT)
    if rc != 0:
        raise KernelError(f"cublasGemmEx failed with status {rc}")
    return True


def qkv_post(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, head_dim: int, *,
             bias: Optional[torch.Tensor], q_weight: Optional[torch.Tensor], k_weight: Optional[torch.Tensor],
             eps: float, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], rotary_dim: int,
             slots: Optional[torch.Tensor], pages: Optional[torch.Tensor], page_size: int) -> None:
    """In place on qkv [N, (nq + 2 nkv) d]: bias, per-head RMSNorm of q and k, rotary; k and v are
    stored to their page slots (pages [P, 2, nkv, page_size, d])."""
    N = qkv.shape[0]
    _need(qkv.is_contiguous() and qkv.shape[1] == (num_heads + 2 * num_kv_heads) * head_dim,
          "qkv must be contiguous [tokens, (heads + 2 kv heads) * head_dim]")
    if pages is not None:
        _need(pages.dtype == qkv.dtype and pages.is_contiguous() and
              tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim), "pages have the wrong layout")
        _need(slots is not None, "a page write needs slots")
    if slots is not None:
        _i32(slots, "slots")
        _need(slots.numel() == N, "one slot per token")
    w_dtype = F32
    if q_weight is not None:
        _need(k_weight is not None and q_weight.dtype == k_weight.dtype and q_weight.numel() == head_dim and
              k_weight.numel() == head_dim, "q/k norm weights must have head_dim entries of one type")
        w_dtype = dtype_code(q_weight.dtype)
    if rotary_dim:
        _need(cos is not None and sin is not None and cos.shape == (N, rotary_dim // 2) and cos.dtype == torch.float32
              and cos.is_contiguous() and sin.is_contiguous(), "rotary tables must be float32 [tokens, rotary_dim / 2]")
    if bias is not None:
        _need(bias.numel() == qkv.shape[1] and bias.is_contiguous(), "qkv bias has the wrong size")
    _call("llmp_qkv_post", _ptr(qkv), dtype_code(qkv.dtype), _ptr(bias),
          dtype_code(bias.dtype) if bias is not None else F32, _ptr(q_weight), _ptr(k_weight), w_dtype, float(eps),
          _ptr(cos), _ptr(sin), int(rotary_dim), _ptr(slots), _ptr(pages), N, num_heads, num_kv_heads, head_dim,
          int(page_size), _stream())


def swiglu(gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[n, i] = silu(gate_up[n, i]) * gate_up[n, I + i]"""
    N, two_i = gate_up.shape
    _need(gate_up.is_contiguous() and out.is_contiguous() and out.shape == (N, two_i // 2) and
          out.dtype == gate_up.dtype and two_i % 2 == 0, "swiglu shapes do not match")
    _call("llmp_swiglu", _ptr(gate_up), _ptr(out), dtype_code(out.dtype), N, two_i // 2, _stream())
    return out


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T (+ bias) on the CUDA cores with float32 accumulation."""
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(a.dtype == w.dtype, "gemm operands must have one type")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    if bias is not None:
        _need(bias.numel() == N and bias.is_contiguous(), "gemm bias has the wrong size")
    _call("llmp_gemm_simt", _ptr(a), _ptr(w), _ptr(bias), dtype_code(bias.dtype) if bias is not None else F32,
          _ptr(out), dtype_code(a.dtype), dtype_code(out.dtype), M, N, K, a.stride(0), w.stride(0), out.stride(0),
          _stream())
    return out


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for M <= 16, bfloat16 operands, bfloat16 or float32 output: the
    weight-streaming tensor-core kernel of the decode step."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_skinny takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _call("llmp_gemm_skinny", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), _stream())
    return out


_error_flag: Optional[torch.Tensor] = None


def error_flag() -> torch.Tensor:
    """One int32 in pinned host memory that kernels with bounded waits set to 1 when a wait ran out.
    The device writes it through its mapped address; the host may read it after any synchronisation."""
    global _error_flag
    if _error_flag is None:
        _error_flag = torch.zeros(1, dtype=torch.int32).pin_memory()
    return _error_flag


def check_error_flag() -> None:
    if _error_flag is not None and int(_error_flag[0]) != 0:
        _error_flag[0] = 0
        raise KernelError("a kernel gave up waiting on one of its barriers (bounded wait ran out); its output is not valid")


def bounded_wait_check(limit: int = 1024) -> bool:
    """Self-check of the bounded waits: launches one thread that waits, with the kernels' own wait and a limit of
    ``limit`` tries, on a barrier that nothing completes. True when the wait gave up; ``check_error_flag()`` then raises
    after the next synchronisation, as it does when a wait of a real kernel runs out."""
    gave_up = torch.zeros(1, dtype=torch.int32, device="cuda")
    _call("llmp_bounded_wait_check", error_flag().data_ptr(), int(limit), _ptr(gave_up), _stream())
    return bool(int(gave_up.item()))


def gemm_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T on the tcgen05 tensor cores (TMA loads, accumulator in tensor
    memory); bfloat16 operands, bfloat16 or float32 output."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_tc takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_tc takes CUDA tensors")
    _call("llmp_gemm_tc", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_supports(M: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, N, K, ldx, ldw))


def gemm_stream(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for at most 64 rows (see ``gemm_stream_supports``): one persistent block per SM streams its share of
    ``w`` through a ring of TMA boxes; bfloat16 operands, bfloat16 or float32 output, K a multiple of 64."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_stream takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_stream takes CUDA tensors")
    _call("llmp_gemm_stream", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_tc_supports(M: int, N: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_tc_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, N, K, ldx, ldw))


def gemm_stream_tc(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[M, N] = x[M, K] @ w[N, K]^T for at most 64 rows: the weight stream of ``gemm_stream`` with the
    products by tcgen05.mma and the accumulator in tensor memory; bfloat16 operands, K a multiple of 64."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16, "gemm_stream_tc takes bfloat16 operands")
    _need(w.shape[1] == K and out.shape == (M, N), "gemm shapes do not match")
    _need(x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w.is_cuda and out.is_cuda, "gemm_stream_tc takes CUDA tensors")
    _call("llmp_gemm_stream_tc", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype), M, N, K, x.stride(0), w.stride(0),
          out.stride(0), error_flag().data_ptr(), _stream())
    return out


def gemm_stream_blocks(M: int, N: int, K: int, ldx: int, ldw: int) -> int:
    """Blocks that ``gemm_stream`` deals a product of these sizes out to (0: sizes it does not take)."""
    fn = library().llmp_gemm_stream_blocks
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return int(fn(M, N, K, ldx, ldw))


def gemm_stream_fused(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], *, glu: bool = False,
                      in_sumsq: Optional[torch.Tensor] = None, in_parts: int = 0, in_width: int = 0, in_eps: float = 0.0,
                      residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                      xw: Optional[torch.Tensor] = None, out_sumsq: Optional[torch.Tensor] = None) -> None:
    """The streaming product (at most 8 rows of x) with the work of the RMSNorm around it folded in.

    ``in_sumsq`` [parts, 8] float32: the rows of ``x`` still lack the factor rsqrt(sum(in_sumsq[:in_parts, m]) / in_width +
    in_eps); the product is multiplied by it (with ``glu`` before the SwiGLU of ``w`` = [gate rows; up rows]).
    ``residual`` [M, N] float32: the product is added into it; ``xw`` [M, N] bfloat16 receives residual * norm_weight and
    ``out_sumsq`` [gemm_stream_blocks(...), 8] each block's sums of residual^2, which are what the next product takes as
    ``x`` and ``in_sumsq``; ``out`` is then not written and may be None."""
    M, K = x.shape
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and M <= 8, "gemm_stream_fused takes up to 8 bfloat16 rows")
    _need(w.shape[1] == K and x.stride(1) == 1 and w.stride(1) == 1, "gemm operands must be row-major and match")
    if out is not None:
        _need(out.shape == (M, N // 2 if glu else N) and out.stride(1) == 1, "gemm output has the wrong shape")
    if in_sumsq is not None:
        _need(in_sumsq.dtype == torch.float32 and in_sumsq.is_contiguous() and in_sumsq.shape[1] == 8 and
              0 < in_parts <= in_sumsq.shape[0] and in_width > 0, "sums of squares must be [parts, 8] float32")
    if residual is not None:
        _need(not glu and out_sumsq is not None and xw is not None and norm_weight is not None,
              "the residual form needs a norm weight, xw and out_sumsq, and no SwiGLU")
        _need(residual.dtype == torch.float32 and residual.shape == (M, N) and residual.stride(1) == 1, "residual must be [M, N] float32")
        _need(xw.dtype == torch.bfloat16 and xw.shape == (M, N) and xw.stride(1) == 1, "xw must be [M, N] bfloat16")
        _need(norm_weight.numel() == N and norm_weight.is_contiguous() and norm_weight.dtype in (torch.float32, torch.bfloat16),
              "the norm weight must have N entries")
        _need(out_sumsq.dtype == torch.float32 and out_sumsq.is_contiguous() and out_sumsq.shape[1] == 8 and
              out_sumsq.shape[0] >= gemm_stream_blocks(M, N, K, x.stride(0), w.stride(0)) > 0, "out_sumsq must be [blocks, 8] float32")
    else:
        _need(out is not None, "a product that is no residual addend needs an output")
    _call("llmp_gemm_stream_fused", _ptr(x), _ptr(w), _ptr(out), dtype_code(out.dtype) if out is not None else BF16, M, N, K,
          x.stride(0), w.stride(0), out.stride(0) if out is not None else 0, N // 2 if glu else 0,
          _ptr(in_sumsq), int(in_parts), 1.0 / in_width if in_width else 0.0, float(in_eps),
          _ptr(residual), residual.stride(0) if residual is not None else 0, _ptr(norm_weight),
          dtype_code(norm_weight.dtype) if norm_weight is not None else F32, _ptr(xw), xw.stride(0) if xw is not None else 0,
          _ptr(out_sumsq), error_flag().data_ptr(), _stream())


class ChainPhase(ctypes.Structure):
    """One product of ``gemm_stream_chain`` as the library reads it (``LlmpChainPhase`` in csrc/gemm_stream_chain.cu)."""

    _fields_ = [("X", _P), ("W", _P), ("Y", _P), ("ldx", _L), ("ldw", _L), ("ldy", _L),
                ("N", _I), ("K", _I), ("out_dtype", _I), ("glu_rows", _I),
                ("in_sumsq", _P), ("in_parts", _I), ("in_inv_width", _F), ("in_eps", _F),
                ("residual", _P), ("ldr", _L), ("norm_w", _P), ("norm_w_dtype", _I),
                ("xw", _P), ("ldxw", _L), ("out_sumsq", _P)]


def chain_phase(x: torch.Tensor, w: torch.Tensor, out: Optional[torch.Tensor], *, glu: bool = False,
                in_sumsq: Optional[torch.Tensor] = None, in_parts: int = 0, in_width: int = 0, in_eps: float = 0.0,
                residual: Optional[torch.Tensor] = None, norm_weight: Optional[torch.Tensor] = None,
                xw: Optional[torch.Tensor] = None, out_sumsq: Optional[torch.Tensor] = None) -> ChainPhase:
    """A phase of a chain, with the arguments of ``gemm_stream_fused``."""
    K = x.shape[1]
    N = w.shape[0]
    _need(x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == K,
          "a chain takes row-major bfloat16 operands that match")
    phase = ChainPhase()
    phase.X, phase.W, phase.Y = _ptr(x), _ptr(w), _ptr(out)
    phase.ldx, phase.ldw, phase.ldy = x.stride(0), w.stride(0), out.stride(0) if out is not None else 0
    phase.N, phase.K, phase.out_dtype = N, K, dtype_code(out.dtype) if out is not None else BF16
    phase.glu_rows = N // 2 if glu else 0
    phase.in_sumsq, phase.in_parts = _ptr(in_sumsq), int(in_parts)
    phase.in_inv_width, phase.in_eps = (1.0 / in_width if in_width else 0.0), float(in_eps)
    phase.residual, phase.ldr = _ptr(residual), residual.stride(0) if residual is not None else 0
    phase.norm_w = _ptr(norm_weight)
    phase.norm_w_dtype = dtype_code(norm_weight.dtype) if norm_weight is not None else F32
    phase.xw, phase.ldxw = _ptr(xw), xw.stride(0) if xw is not None else 0
    phase.out_sumsq = _ptr(out_sumsq)
    return phase


_chain_counters: dict = {}
_chain_max_phases: Optional[int] = None


def gemm_stream_chain_max_phases() -> int:
    global _chain_max_phases
    if _chain_max_phases is None:
        fn = library().llmp_gemm_stream_chain_max_phases
        fn.argtypes = []
        fn.restype = _I
        _chain_max_phases = int(fn())
    return _chain_max_phases


def gemm_stream_chain_supports(phases: Sequence[ChainPhase], M: int) -> bool:
    fn = library().llmp_gemm_stream_chain_supports
    fn.argtypes = [_P, _I, _I]
    fn.restype = _I
    array = (ChainPhase * len(phases))(*phases)
    return bool(fn(ctypes.cast(array, _P), len(phases), M))


def gemm_stream_chain(phases: Sequence[ChainPhase], M: int, device: torch.device) -> None:
    """The products of ``phases`` (at most 8 rows of X each, every phase reading what the phase before wrote) in one
    persistent cooperative launch whose ring of weight boxes never drains between them; the results are those of
    ``gemm_stream_fused`` called phase by phase, bit for bit. The blocks tell each other through counters in global
    memory that a phase is complete; one set per device, so chains on a device must follow one another in one stream."""
    key = torch.device(device).index or 0
    counters = _chain_counters.get(key)
    if counters is None:
        _need(not torch.cuda.is_current_stream_capturing(), "the chain's counters must exist before a graph is captured")
        fn = library().llmp_gemm_stream_chain_counters
        fn.argtypes = []
        fn.restype = _I
        counters = _chain_counters[key] = torch.zeros(int(fn()), dtype=torch.int32, device=device)
    array = (ChainPhase * len(phases))(*phases)
    _call("llmp_gemm_stream_chain", ctypes.cast(array, _P), len(phases), int(M), _ptr(counters), error_flag().data_ptr(),
          _stream())


def gemm_stream_swiglu_supports(M: int, I: int, K: int, ldx: int, ldw: int) -> bool:
    fn = library().llmp_gemm_stream_swiglu_supports
    fn.argtypes = [_I, _I, _I, _L, _L]
    fn.restype = _I
    return bool(fn(M, I, K, ldx, ldw))


def gemm_stream_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[m, i] = silu(x[m] . w[i]) * (x[m] . w[I + i]) for ``w_gate_up`` = [gate rows; up rows] ([2 I, K]): the
    gate/up product of a SwiGLU feed-forward and its activation in one streaming kernel (at most 16 rows of x)."""
    M, K = x.shape
    I = w_gate_up.shape[0] // 2
    _need(x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16, "gemm_stream_swiglu takes bfloat16 operands")
    _need(w_gate_up.shape == (2 * I, K) and out.shape == (M, I), "gemm_stream_swiglu shapes do not match")
    _need(x.stride(1) == 1 and w_gate_up.stride(1) == 1 and out.stride(1) == 1, "gemm operands must be row-major")
    _need(x.is_cuda and w_gate_up.is_cuda and out.is_cuda, "gemm_stream_swiglu takes CUDA tensors")
    _call("llmp_gemm_stream_swiglu", _ptr(x), _ptr(w_gate_up), _ptr(out), dtype_code(out.dtype), M, I, K, x.stride(0),
          w_gate_up.stride(0), out.stride(0), error_flag().data_ptr(), _stream())
    return out


def paged_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, pages: torch.Tensor,
                    block_tables: torch.Tensor, q_start: torch.Tensor, ctx_len: torch.Tensor,
                    tile_req: torch.Tensor, tile_tok0: torch.Tensor, num_heads: int, num_kv_heads: int,
                    head_dim: int, page_size: int, window: int, scale: float, tokens_per_tile: int,
                    tile_seg: Optional[torch.Tensor] = None, tile_slot: Optional[torch.Tensor] = None,
                    places: int = 0) -> torch.Tensor:
    """Causal attention of the step's query rows over the paged keys and values (any portion sizes).
    ``tokens_per_tile`` is the step the tile list was built with (``tokens_per_attention_tile``).
    With ``tile_seg`` the list holds items that share the keys of a tile (see ``attention_max_segments``): item i is
    number ``tile_seg[i] & 255`` of ``tile_seg[i] >> 8`` consecutive items of its tile, and ``tile_slot[i]`` is the
    first of the tile's ``places`` (one per item) for their sums."""
    for name, t in (("block_tables", block_tables), ("q_start", q_start), ("ctx_len", ctx_len),
                    ("tile_req", tile_req), ("tile_tok0", tile_tok0)):
        _i32(t, name)
    _need(q.dtype == pages.dtype == out.dtype, "q, pages and out must have one type")
    _need(out.is_contiguous() and out.shape[1] == num_heads * head_dim, "attention output must be [tokens, heads * head_dim]")
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim),
          "pages have the wrong layout")
    seg = slot = partials = counters = None
    if tile_seg is not None:
        _i32(tile_seg, "tile_seg")
        _i32(tile_slot, "tile_slot")
        _need(tile_seg.numel() == tile_req.numel() == tile_slot.numel() and 0 < places <= ATTENTION_MAX_PLACES,
              "tile_seg and tile_slot must have an entry per item, and the places a count within bounds")
        partials = torch.empty(places * num_kv_heads * attention_place_floats(), dtype=torch.float32, device=q.device)
        counters = attention_counters(q.device, places * num_kv_heads)
        seg, slot = tile_seg, tile_slot
    _call("llmp_paged_attention", _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(pages), pages.shape[0],
          dtype_code(q.dtype), _ptr(block_tables), block_tables.stride(0), _ptr(q_start), _ptr(ctx_len),
          _ptr(tile_req), _ptr(tile_tok0), _ptr(seg), _ptr(slot), _ptr(partials), _ptr(counters), tile_req.numel(),
          num_heads, num_kv_heads, head_dim, page_size, int(window), float(scale), int(tokens_per_tile),
          error_flag().data_ptr(), _stream())
    return out


def decode_scratch_floats(rows: int, num_heads: int, head_dim: int, max_ctx: int) -> int:
    fn = library().llmp_decode_scratch_floats
    fn.argtypes = [_I, _I, _I, _I]
    fn.restype = _L
    return int(fn(rows, num_heads, head_dim, max_ctx))


_decode_counters: dict = {}
DECODE_RANGE = 128                   # keys per fixed range of the decode attention kernels
DECODE_MAX_KEYS = 1024 * DECODE_RANGE   # the longest context the decode attention kernels take
_DECODE_LIST = os.environ.get("LLMP_B200_DECODE_LIST", "")


_sm_count: Optional[int] = None


def sm_count() -> int:
    global _sm_count
    if _sm_count is None:
        _sm_count = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count
    return _sm_count


def decode_prefers_list(longest: int, total: int, rows: int, num_kv_heads: int, sms: Optional[int] = None) -> bool:
    """Whether a decode step over ``rows`` requests that see ``total`` keys together, the longest ``longest``, is
    better served by the kernel that deals the key ranges of all requests out evenly over the SMs than by the one
    that gives every (request, key/value head) pair blocks of its own. The latter walks as many keys per block as
    the longest request needs with the up to 8 blocks a pair can get; the former the average, plus the adding up of
    shared sums through global memory (worth about a thousand keys of reading). Also with many more pairs than SMs:
    whole pairs per block then leave SMs idle in the last round (Qwen3-8B heads, 2,048 keys each: from 64 requests on)."""
    sms = sms or sm_count()
    pairs = rows * num_kv_heads
    if pairs > 2 * sms:
        return True
    blocks = 1
    while blocks < 8 and pairs * blocks * 2 <= sms:
        blocks *= 2
    own = longest * -(-pairs // sms) / blocks
    even = total * num_kv_heads / sms
    return own > 1.25 * even + 1024


def decode_counters(device: torch.device) -> torch.Tensor:
    """The counters with which the blocks of the streaming decode kernel that share a long request find out who
    finishes last. Every launch leaves them zero. One set per device: decode launches on a device must follow one
    another (one stream, or streams ordered by events), as they do in the engine. They are made outside a graph
    capture (the engine runs every shape once before it captures it)."""
    key = torch.device(device).index or 0
    counters = _decode_counters.get(key)
    if counters is None:
        _need(not torch.cuda.is_current_stream_capturing(), "decode counters must exist before a graph is captured")
        fn = library().llmp_decode_counters
        fn.argtypes = []
        fn.restype = _I
        counters = _decode_counters[key] = torch.zeros(int(fn()), dtype=torch.int32, device=device)
    return counters


def decode_attention(q: torch.Tensor, q_stride: int, out: torch.Tensor, pages: torch.Tensor,
                     block_tables: torch.Tensor, ctx_len: torch.Tensor, max_ctx: int, num_heads: int,
                     num_kv_heads: int, head_dim: int, page_size: int, window: int, scale: float,
                     scratch: Optional[torch.Tensor] = None, uneven: bool = False) -> torch.Tensor:
    """Attention of one query row per request (row r belongs to request r, at position ctx_len[r] - 1)
    over the request's pages; keys are split into fixed ranges whose partial results go through
    ``scratch`` (float32, at least ``decode_scratch_floats(...)`` entries; allocated when None).
    ``uneven`` (see ``decode_prefers_list``) picks, where there is a choice, the kernel that deals the key ranges of
    all requests out evenly over the SMs instead of giving every request blocks of its own; the result is the same
    beyond rounding. ``LLMP_B200_DECODE_LIST=0`` or ``1`` overrides it."""
    if _DECODE_LIST in ("0", "1"):
        uneven = _DECODE_LIST == "1"
    _i32(block_tables, "block_tables")
    _i32(ctx_len, "ctx_len")
    R = ctx_len.numel()
    _need(q.dtype == pages.dtype == out.dtype, "q, pages and out must have one type")
    _need(out.is_contiguous() and out.shape == (R, num_heads * head_dim), "decode output must be [requests, heads * head_dim]")
    _need(pages.is_contiguous() and tuple(pages.shape[1:]) == (2, num_kv_heads, page_size, head_dim),
          "pages have the wrong layout")
    need = decode_scratch_floats(R, num_heads, head_dim, max_ctx)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    _need(scratch.dtype == torch.float32 and scratch.is_contiguous() and scratch.numel() >= need,
          f"decode scratch must hold {need} float32 values")
    _call("llmp_decode_attention", _ptr(q), int(q_stride), _ptr(out), out.stride(0), _ptr(pages), pages.shape[0],
          dtype_code(q.dtype), _ptr(block_tables), block_tables.stride(0), _ptr(ctx_len), R, int(max_ctx), num_heads,
          num_kv_heads, head_dim, page_size, int(window), float(scale), _ptr(scratch), scratch.numel(),
          _ptr(decode_counters(q.device)), int(bool(uneven)), error_flag().data_ptr(), _stream())
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _i32(out, "out")
    scratch = torch.empty(logits.shape[0] * 64, dtype=torch.int32, device=logits.device)   # slices' best values and indices
    _call("llmp_argmax", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(out), _ptr(scratch),
          _stream())
    return out


def repetition_penalty(logits: torch.Tensor, tokens: torch.Tensor, offsets: torch.Tensor, penalty: torch.Tensor) -> None:
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _i32(tokens, "tokens")
    _i32(offsets, "offsets")
    _need(penalty.dtype == torch.float32 and penalty.numel() == logits.shape[0], "one penalty per row")
    _call("llmp_repetition_penalty", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(tokens),
          _ptr(offsets), _ptr(penalty), _stream())


def entropy(logits: torch.Tensor, temperature: float) -> torch.Tensor:
    """Entropy in nats of softmax(logits / temperature) for every row of float32 ``logits [rows, vocab]`` (the logits
    as they are when ``temperature`` is not positive); float32 ``[rows]``."""
    _need(logits.dtype == torch.float32 and logits.dim() == 2 and logits.stride(1) == 1, "logits must be float32 rows")
    out = torch.empty(logits.shape[0], dtype=torch.float32, device=logits.device)
    _call("llmp_entropy", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], float(temperature), _ptr(out),
          _stream())
    return out


def sample(logits: torch.Tensor, params: torch.Tensor, out: torch.Tensor, out_u: Optional[torch.Tensor] = None) -> torch.Tensor:
    """params: int32 [M, 8] rows {temperature, top_k, top_p, min_p, typical_p, seed low, seed high, step}
    with the float fields stored by bit pattern."""
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "logits must be float32 rows")
    _need(params.dtype == torch.int32 and params.is_contiguous() and params.shape == (logits.shape[0], 8),
          "sampling parameters must be int32 [rows, 8]")
    _i32(out, "out")
    _call("llmp_sample", _ptr(logits), logits.stride(0), logits.shape[0], logits.shape[1], _ptr(params), _ptr(out),
          _ptr(out_u), _stream())
    return out
