"""y = x W^T (+ bias): which matrix product runs for which types and sizes.

* float32 operands: always the CUDA-core kernel of ``csrc/gemm_simt.cu`` — a true 32-bit product
  whose result for a row does not depend on the other rows.
* bfloat16 operands: this package's tensor-core kernels where they cover the shape (registered in
  ``_BF16_KERNELS`` by the modules that bind them), else the library product (cuBLAS through
  ``torch``), which is what the reference's ``nn.Linear`` layers call
  (src/llm_pipeline/models/qwen3/custom_builder.py:75-78,201-203,387).
"""

from __future__ import annotations

import os
from typing import Callable, List, Optional

import torch

from . import kernels

# Each entry: fn(x, weight, out_dtype) -> tensor or None (None: "not my shape").
_BF16_KERNELS: List[Callable] = []


def register_bf16_kernel(fn: Callable) -> None:
    _BF16_KERNELS.append(fn)


# ---- a norm between two streaming products, folded into them ------------------------------------------------
# A decode step of a few rows spends as long between kernels as in them, and the residual add with its RMSNorm is a
# kernel of its own between the product before it and the product after it. RMSNorm is a factor per row: x_norm[m] =
# (r[m] * w) * rsqrt(mean(r[m]^2) + eps). So the product before it can add its result into the residual r, leave r * w
# (rounded once to bfloat16, as the norm's output is) and its share of the rows' sums of squares, and the product
# after it multiplies its result by the rows' factors: no kernel in between. FUSE_NORM=0 (LLMP_B200_FUSE_NORM) keeps
# the norm kernel.
FUSE_NORM = os.environ.get("LLMP_B200_FUSE_NORM", "1") == "1"


class PendingProduct:
    """``x @ weight^T`` that has not been taken yet. A norm that can fold the product into its own work asks for
    ``x`` (a tensor, or ``LazyRows``) and ``weight``; everybody else calls ``value()``."""

    def __init__(self, x, weight: torch.Tensor, accumulate: bool = False):
        self.x, self.weight = x, weight
        # True: many rows; whoever adds the product to a float32 residual may let the library's product do the adding
        # (``kernels.library_add_product``) instead of taking the value and adding it
        self.accumulate = accumulate

    def value(self) -> torch.Tensor:
        return linear(self.x, self.weight)


# ---- several products of a decode step in one launch ------------------------------------------------------------
# The products of a decode step of at most 8 rows follow one another, each needing the whole result of the one before:
# o -> (residual, norm) -> gate/up with SwiGLU -> down -> (residual, norm) -> the next layer's qkv. Launched one by one,
# each drains its ring of weight boxes and the next fills its own again. ``kernels.gemm_stream_chain`` runs up to four
# of them as phases of one persistent launch whose ring never drains. The parts do not know of it: the functions below
# (``residual_product``, ``gate_up_swiglu``, ``pending_product``, ``linear``) do not launch a product whose only
# reader will be the next of them, but note it in the open chain and hand out a handle (``ScaledRows`` or ``LazyRows``
# with ``chain`` set); a product whose result leaves as a tensor ends the chain and launches it. Whoever needs a tensor
# from a handle calls ``value()``, which launches what is noted first. A chain gives the same bits as its products
# launched one by one. It is off unless LLMP_B200_CHAIN=1: measured on a B200 (Qwen3-8B shape, batch 8) a step through
# chains takes 4.55 ms against 3.63 ms, because as dependent launches the separate products already fill their rings
# while the kernel before them ends, each with a ring of its own stage size (see csrc/gemm_stream_chain.cu).
CHAIN = os.environ.get("LLMP_B200_CHAIN", "0") == "1"
# Rows from which a product that is an addend of the residual (output and down projection) is left to the library's
# product with the float32 residual as its C operand (0: never): the norm after it then only reads the residual.
# Measured on a B200 (Qwen3-8B shape): a 2,048-token prefill 27.2 -> 26.6 ms. The call costs the host a few
# microseconds more than torch.mm, which a step that waits for the host pays for in full (the continuous-batching mix
# at the Qwen3-0.6B shape: 85 -> 75 thousand tokens/s with it), so it is taken only for many rows of a large matrix.
ACCUMULATE_MIN_ROWS = int(os.environ.get("LLMP_B200_ACCUMULATE_MIN_M", "1024"))
ACCUMULATE_MIN_WEIGHTS = 1 << 24


class _Chain:
    def __init__(self, rows: int, device: torch.device):
        self.rows, self.device = rows, device
        self.noted = []                 # (x tensor, weight, out tensor or None, keyword arguments of gemm_stream_fused)
        self.launched = False

    def has_room(self) -> bool:
        return not self.launched and len(self.noted) < kernels.gemm_stream_chain_max_phases()

    def note(self, x: torch.Tensor, weight: torch.Tensor, out: Optional[torch.Tensor], **extras) -> None:
        self.noted.append((x, weight, out, extras))

    def launch(self) -> None:
        global _open_chain
        if self.launched:
            return
        self.launched = True
        if _open_chain is self:
            _open_chain = None
        if len(self.noted) == 1:
            x, weight, out, extras = self.noted[0]
            kernels.gemm_stream_fused(x, weight, out, **extras)
        elif self.noted:
            kernels.gemm_stream_chain([kernels.chain_phase(x, weight, out, **extras) for x, weight, out, extras in self.noted],
                                      self.rows, self.device)
        self.noted = []


_open_chain: Optional[_Chain] = None
_chain_shapes: dict = {}                # (rows, shapes of the phases) -> whether they run as one chain


def begin_step() -> None:
    """A step begins: a chain that an abandoned step left open is dropped (nobody waits for its results)."""
    global _open_chain
    _open_chain = None


def _chain_takes(chain: _Chain, x: torch.Tensor, weight: torch.Tensor, glu: bool) -> bool:
    """Whether the open chain can take one more product of these sizes (the plans of all its phases fit one ring)."""
    if not chain.has_room():
        return False
    shapes = tuple((w.shape[0], w.shape[1], a.stride(0), w.stride(0), bool(e.get("glu", False))) for a, w, _o, e in chain.noted)
    shapes += ((weight.shape[0], weight.shape[1], x.stride(0), weight.stride(0), glu),)
    key = (chain.rows, shapes)
    ok = _chain_shapes.get(key)
    if ok is None:
        phases = []
        for N, K, ldx, ldw, g in shapes:
            phase = kernels.ChainPhase()
            phase.N, phase.K, phase.ldx, phase.ldw, phase.glu_rows = N, K, ldx, ldw, (N // 2 if g else 0)
            phases.append(phase)
        ok = _chain_shapes[key] = kernels.gemm_stream_chain_supports(phases, chain.rows)
    return ok


class LazyRows:
    """Rows [M, width] that a product noted in an open chain will write: ``values`` is their tensor, valid once the
    chain is launched. ``linear()`` and ``pending_product()`` take the handle; everybody else calls ``value()``."""

    def __init__(self, values: torch.Tensor, chain: _Chain):
        self.values, self.chain = values, chain

    shape = property(lambda self: self.values.shape)
    dtype = property(lambda self: self.values.dtype)
    device = property(lambda self: self.values.device)

    def value(self) -> torch.Tensor:
        self.chain.launch()
        return self.values


class ScaledRows:
    """Rows that still lack a factor each: ``values`` [M, width] bfloat16 and, per row m, the factor
    rsqrt(sum(sumsq[:parts, m]) / width + eps). A product that can apply the factors to its result takes the fields;
    everybody else calls ``value()``, which has ``materialise`` (given by whoever made the rows) build the finished rows."""

    def __init__(self, values: torch.Tensor, sumsq: torch.Tensor, parts: int, eps: float, materialise: Callable[[], torch.Tensor],
                 chain: Optional[_Chain] = None):
        self.values, self.sumsq, self.parts, self.eps = values, sumsq, int(parts), float(eps)
        self._materialise = materialise
        self._value: Optional[torch.Tensor] = None
        self.chain = chain              # set while the product that writes ``values`` and ``sumsq`` is only noted in a chain

    shape = property(lambda self: self.values.shape)
    dtype = property(lambda self: self.values.dtype)
    device = property(lambda self: self.values.device)

    def value(self) -> torch.Tensor:
        if self._value is None:
            if self.chain is not None:
                self.chain.launch()
            self._value = self._materialise()
        return self._value


def pending_product(x: torch.Tensor, weight: torch.Tensor):
    """``x @ weight^T`` as a PendingProduct where a following norm could fold it in (the sizes of the streaming
    product for at most 8 bfloat16 rows), else the product itself."""
    M, K = x.shape
    rows = x.values if isinstance(x, LazyRows) else x
    if (FUSE_NORM and STREAM_GEMM and isinstance(rows, torch.Tensor) and rows.dtype == torch.bfloat16 and 0 < M <= 8 and
            rows.stride(1) == 1 and weight.stride(1) == 1 and not rows.data_ptr() % 16 and not weight.data_ptr() % 16 and
            kernels.gemm_stream_blocks(M, weight.shape[0], K, rows.stride(0), weight.stride(0)) > 0):
        return PendingProduct(x, weight)
    if (ACCUMULATE_MIN_ROWS and isinstance(x, torch.Tensor) and x.dtype == torch.bfloat16 and M >= ACCUMULATE_MIN_ROWS and
            weight.numel() >= ACCUMULATE_MIN_WEIGHTS and x.is_cuda and x.stride(1) == 1 and weight.stride(1) == 1 and not x.data_ptr() % 16 and not weight.data_ptr() % 16):
        return PendingProduct(x, weight, accumulate=True)
    return linear(x, weight)


def residual_product(product: PendingProduct, residual: torch.Tensor, norm_weight: torch.Tensor, eps: float,
                     materialise: Callable[[], torch.Tensor]) -> ScaledRows:
    """residual += product; returns residual * norm_weight with the rows' factors still to be applied."""
    global _open_chain
    x, weight = product.x, product.weight
    M, N = x.shape[0], weight.shape[0]
    chain = None
    if isinstance(x, LazyRows):
        # the rows come out of the open chain: one more phase of it, if it takes one
        if CHAIN and x.chain is _open_chain and _chain_takes(x.chain, x.values, weight, False):
            chain, x = x.chain, x.values
        else:
            x = x.value()
    elif CHAIN:
        if _open_chain is not None:
            _open_chain.launch()
        chain = _open_chain = _Chain(M, x.device)
    blocks = kernels.gemm_stream_blocks(M, N, x.shape[1], x.stride(0), weight.stride(0))
    xw = torch.empty((M, N), dtype=torch.bfloat16, device=x.device)
    sumsq = torch.empty((blocks, 8), dtype=torch.float32, device=x.device)
    if chain is not None:
        chain.note(x, weight, None, residual=residual, norm_weight=norm_weight, xw=xw, out_sumsq=sumsq)
        return ScaledRows(xw, sumsq, blocks, eps, materialise, chain)
    kernels.gemm_stream_fused(x, weight, None, residual=residual, norm_weight=norm_weight, xw=xw, out_sumsq=sumsq)
    return ScaledRows(xw, sumsq, blocks, eps, materialise)


def _scaled_stream(x: ScaledRows, weight: torch.Tensor, glu: bool) -> Optional[torch.Tensor]:
    values = x.values
    M, K = values.shape
    N = weight.shape[0]
    if not STREAM_GEMM or weight.stride(1) != 1 or weight.data_ptr() % 16 or (glu and N % 2):
        return None
    if glu:
        if not kernels.gemm_stream_swiglu_supports(M, N // 2, K, values.stride(0), weight.stride(0)):
            return None
    elif not kernels.gemm_stream_supports(M, N, K, values.stride(0), weight.stride(0)):
        return None
    out = torch.empty((M, N // 2 if glu else N), dtype=values.dtype, device=values.device)
    chain = x.chain
    if chain is not None and chain is _open_chain and _chain_takes(chain, values, weight, glu):
        chain.note(values, weight, out, glu=glu, in_sumsq=x.sumsq, in_parts=x.parts, in_width=K, in_eps=x.eps)
        if glu:
            return LazyRows(out, chain)         # its reader is the next product
        chain.launch()                          # plain rows leave as a tensor: the chain ends here
        return out
    if chain is not None:
        chain.launch()
    kernels.gemm_stream_fused(values, weight, out, glu=glu, in_sumsq=x.sumsq, in_parts=x.parts, in_width=K, in_eps=x.eps)
    return out


def _stream(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The weight-streaming kernel for the few rows of a decode step: one persistent block per SM, the rows
    of the weight matrix dealt out evenly, a ring of TMA boxes fed by a load warp."""
    M, K = x.shape
    if not STREAM_GEMM or not 0 < M <= STREAM_MAX_M or x.stride(1) != 1 or weight.stride(1) != 1:
        return None
    if x.data_ptr() % 16 or weight.data_ptr() % 16 or out_dtype not in (torch.bfloat16, torch.float32):
        return None
    if not kernels.gemm_stream_supports(M, weight.shape[0], K, x.stride(0), weight.stride(0)):
        return None
    if M > 8 and weight.shape[0] > STREAM_MAX_N:
        return None
    out = torch.empty((M, weight.shape[0]), dtype=out_dtype, device=x.device)
    return kernels.gemm_stream(x, weight, out)


def _stream_tc(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The weight stream with tcgen05 products, for 9 to 32 rows against a very tall weight matrix (the output
    head), where a block's share of rows fills most of the 128-row side of the MMA. Measured on a B200 against
    the head of Qwen3-8B (151,936 x 4,096): 197 us at 16 rows and 211 at 32 (library 213 and 215); at 64 rows, and
    for the layer's products at any row count (28 to 167 weight rows per block, so most of the 128 rows that the
    MMA reads from shared memory are padding), it is slower than the library and is not used."""
    M, K = x.shape
    if not STREAM_GEMM or not 8 < M <= 32 or weight.shape[0] < STREAM_TC_MIN_N or x.stride(1) != 1 or weight.stride(1) != 1:
        return None
    if x.data_ptr() % 16 or weight.data_ptr() % 16 or out_dtype not in (torch.bfloat16, torch.float32):
        return None
    if not kernels.gemm_stream_tc_supports(M, weight.shape[0], K, x.stride(0), weight.stride(0)):
        return None
    out = torch.empty((M, weight.shape[0]), dtype=out_dtype, device=x.device)
    return kernels.gemm_stream_tc(x, weight, out)


def gate_up_swiglu(x: torch.Tensor, w_gate_up: torch.Tensor) -> Optional[torch.Tensor]:
    """silu(x gate^T) * (x up^T) for ``w_gate_up`` = [gate rows; up rows] in one streaming kernel, where that kernel
    serves the gate/up product anyway (bfloat16, at most 8 rows); None otherwise: the caller then takes the product
    and the activation kernel. ``x`` may be ScaledRows."""
    if isinstance(x, ScaledRows):
        # None leaves the rows as they are: the caller's linear() takes them
        return _scaled_stream(x, w_gate_up, glu=True) if x.shape[1] >= FUSED_SWIGLU_MIN_K else None
    M, K = x.shape
    if not STREAM_GEMM or x.dtype != torch.bfloat16 or not 0 < M <= 8 or x.stride(1) != 1 or w_gate_up.stride(1) != 1:
        return None
    if K < FUSED_SWIGLU_MIN_K:
        return None
    if x.data_ptr() % 16 or w_gate_up.data_ptr() % 16 or w_gate_up.shape[0] % 2:
        return None
    I = w_gate_up.shape[0] // 2
    if not kernels.gemm_stream_swiglu_supports(M, I, K, x.stride(0), w_gate_up.stride(0)):
        return None
    out = torch.empty((M, I), dtype=x.dtype, device=x.device)
    return kernels.gemm_stream_swiglu(x, w_gate_up, out)


def _tensor_memory(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The tcgen05 kernel (TMA, accumulator in tensor memory, cluster split-K) for at most 16 rows of a decode
    step against a long K, where it reads the weights faster than the library product does."""
    M, K = x.shape
    if not 0 < M <= 16 or K < 8192 or K % 8 or x.stride(1) != 1 or weight.stride(1) != 1:
        return None
    if x.stride(0) % 8 or weight.stride(0) % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return None
    if out_dtype not in (torch.bfloat16, torch.float32):
        return None
    out = torch.empty((M, weight.shape[0]), dtype=out_dtype, device=x.device)
    return kernels.gemm_tc(x, weight, out)


def _skinny(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The weight-streaming mma.sync kernel for at most 16 rows against a narrow output (few tiles),
    where it matches or beats the library product."""
    M, K = x.shape
    if not 0 < M <= 16 or weight.shape[0] > 4096 or K % 8 or x.stride(1) != 1 or weight.stride(1) != 1:
        return None
    if x.stride(0) % 8 or weight.stride(0) % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return None
    if out_dtype not in (torch.bfloat16, torch.float32):
        return None
    out = torch.empty((M, weight.shape[0]), dtype=out_dtype, device=x.device)
    return kernels.gemm_skinny(x, weight, out)


def _tensor_memory_prefill(x: torch.Tensor, weight: torch.Tensor, out_dtype: torch.dtype) -> Optional[torch.Tensor]:
    """The persistent tcgen05 kernel (128 x 256 tiles, two accumulators in tensor memory so that the epilogue
    of one tile overlaps the products of the next) for the many rows of a prompt portion."""
    M, K = x.shape
    if OWN_PREFILL_GEMM == "1":
        wanted = M >= PREFILL_TC_MIN_ROWS
    else:
        wanted = OWN_PREFILL_GEMM == "auto" and M >= PREFILL_TC_SMALL_MIN_ROWS and weight.numel() <= PREFILL_TC_SMALL_WEIGHTS
    if not wanted or K % 8 or x.stride(1) != 1 or weight.stride(1) != 1:
        return None
    if x.stride(0) % 8 or weight.stride(0) % 8 or x.data_ptr() % 16 or weight.data_ptr() % 16:
        return None
    if out_dtype not in (torch.bfloat16, torch.float32):
        return None
    out = torch.empty((M, weight.shape[0]), dtype=out_dtype, device=x.device)
    return kernels.gemm_tc(x, weight, out)


# Measured on a B200 at 2,048 rows (Qwen3-8B shapes): this kernel reaches 1.14-1.44 PFLOP/s, the library product
# 1.32-1.59, so the library product stays the default for prompt portions; LLMP_B200_OWN_PREFILL_GEMM=1 (or setting
# this flag) routes portions of at least PREFILL_TC_MIN_ROWS rows through the own kernel. Fewer rows leave too few
# 128-row tiles to fill the SMs.
# Small matrices are another matter: a prompt portion's product then takes the device a few microseconds and the
# host, through the library, some 35 (every step of a continuous batch has another number of rows, and the library
# chooses its kernel anew for each); the own kernel costs the host a plain call. The continuous-batching mix at the
# Qwen3-0.6B shape: 70 to 73 thousand tokens/s with the library product, 81 to 85 with the own kernel for portions of
# 1,024 rows or more; at the Qwen3-8B shape 38.2 against 36.0. "auto" (the default) takes the own kernel for matrices
# of at most PREFILL_TC_SMALL_WEIGHTS entries and portions of at least PREFILL_TC_SMALL_MIN_ROWS rows (from 65 rows: 80
# thousand tokens/s; from 256 or from 1,024: 85).
OWN_PREFILL_GEMM = os.environ.get("LLMP_B200_OWN_PREFILL_GEMM", "auto")
PREFILL_TC_MIN_ROWS = 1024
PREFILL_TC_SMALL_MIN_ROWS = int(os.environ.get("LLMP_B200_OWN_PREFILL_SMALL_MIN_M", "256"))
PREFILL_TC_SMALL_WEIGHTS = 8 << 20

# Measured on a B200 (Qwen3-8B shapes, replayed decode graph, ms per step): every product of the step through the
# streaming kernel 3.34 at 1 row, 3.64 at 4, 3.95 at 8; the streaming kernel only for the output and down projections
# (5,120 weight rows at most) and the library product for qkv, gate/up and the head 3.53, 3.82, 4.10; without the
# streaming kernel (skinny kernel, tcgen05 split-K, library) 3.66, 3.96, 4.23. At 16 rows the wide products are
# faster through the library (4.67 against 4.84 all streaming). Qwen3-32B shapes at 8 rows: 13.9 all streaming, 14.3
# narrow products only, 16.9 without; Qwen3-0.6B: 1.32, 1.40, 1.35. Hence: up to 8 rows every product streams, from 9
# to 16 rows those with at most STREAM_MAX_N weight rows. LLMP_B200_STREAM_GEMM=0 turns the kernel off.
STREAM_GEMM = os.environ.get("LLMP_B200_STREAM_GEMM", "1") == "1"
STREAM_MAX_N = int(os.environ.get("LLMP_B200_STREAM_MAX_N", "5120"))
# More than 16 rows make the kernel compute-bound on its four mma.sync warps (batch 64: 9.57 ms per step against 7.72
# with the library product), so the limit on the rows of x stays at 16 although the kernel takes up to 64.
STREAM_MAX_M = int(os.environ.get("LLMP_B200_STREAM_MAX_M", "16"))

STREAM_TC_MIN_N = 32768
# The fused gate/up kernel walks a block's rows as two chunks (gate rows, up rows); with a short K the chunks' ends
# weigh more than the activation kernel saved (Qwen3-0.6B shape, K = 1,024: 1.35 ms per step fused, 1.27 not fused;
# Qwen3-8B shape, K = 4,096: 3.79 fused, 3.81 not).
FUSED_SWIGLU_MIN_K = int(os.environ.get("LLMP_B200_FUSED_SWIGLU_MIN_K", "4096"))

register_bf16_kernel(_stream)
register_bf16_kernel(_stream_tc)
register_bf16_kernel(_tensor_memory)
register_bf16_kernel(_skinny)
register_bf16_kernel(_tensor_memory_prefill)


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None,
           out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    """x [M, K], weight [N, K] -> [M, N] in ``out_dtype`` (default: x's type). ``x`` may be ScaledRows or LazyRows."""
    if isinstance(x, LazyRows):
        chain, values = x.chain, x.values
        if (bias is None and out_dtype in (None, values.dtype) and chain is _open_chain and weight.stride(1) == 1 and
                not weight.data_ptr() % 16 and _chain_takes(chain, values, weight, False)):
            out = torch.empty((values.shape[0], weight.shape[0]), dtype=values.dtype, device=values.device)
            chain.note(values, weight, out)
            chain.launch()
            return out
        x = x.value()
    if isinstance(x, ScaledRows):
        if bias is None and out_dtype in (None, x.dtype):
            out = _scaled_stream(x, weight, glu=False)
            if out is not None:
                return out
        x = x.value()
    if not x.is_cuda:
        raise kernels.KernelError("linear() was given a CPU tensor; this engine has no CPU path")
    out_dtype = out_dtype or x.dtype
    M, N = x.shape[0], weight.shape[0]
    if x.dtype == torch.float32:
        out = torch.empty((M, N), dtype=torch.float32, device=x.device)
        if M:
            kernels.gemm_simt(x, weight, out, bias)
        return out
    for fn in _BF16_KERNELS:
        out = fn(x, weight, out_dtype)
        if out is not None:
            return out if bias is None else out.add_(bias.to(out.dtype))
    if M == 0:
        return torch.empty((0, N), dtype=out_dtype, device=x.device)
    if out_dtype == x.dtype:
        out = torch.mm(x, weight.t())
    else:
        out = torch.mm(x, weight.t(), out_dtype=out_dtype)
    return out if bias is None else out.add_(bias.to(out.dtype))
