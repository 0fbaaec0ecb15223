"""Where a step's time goes, without a profiler: CUDA events around every kernel launch, and NVTX ranges.

Every kernel of this library is launched through ``kernels._call`` and the library matrix product through
``torch.mm``; ``KernelTimes`` puts a pair of CUDA events around each such call while it is active and adds the
intervals up per label. It times eager steps (a replayed CUDA graph makes no calls), so a caller that wants a
breakdown of a decode step runs it with graphs off; the intervals are the kernels' own times, without the overlap
that dependent launches give them inside a graph.

``LLMP_B200_KERNEL_TIMES=1`` makes every ``ModelRunner`` time all its steps this way (eagerly) and report the sums in
``runner.kernel_times.table()`` and ``GenerationEngine.stats()["kernel_times"]``. ``LLMP_B200_NVTX=1`` makes the model
and the runner push NVTX ranges (step, embedding, each scheduled layer with its mixer and feed-forward, head) for a
timeline tool to show; inside a captured graph they mark the capture, not the replays.

The reference's nearest thing are the counters of its batcher and cache
(src/llm_pipeline/inference/continuous_batching.py:448-463, inference/paged_attention.py:288-299)."""

from __future__ import annotations

import contextlib
import os
from typing import Callable, Dict, List, Optional, Tuple

import torch

TIME_KERNELS = os.environ.get("LLMP_B200_KERNEL_TIMES", "0") == "1"
NVTX = os.environ.get("LLMP_B200_NVTX", "0") == "1"

# entry points whose arguments 4..6 are M, N, K of a matrix product
_PRODUCTS = ("llmp_gemm_stream", "llmp_gemm_stream_fused", "llmp_gemm_stream_swiglu", "llmp_gemm_stream_tc", "llmp_gemm_tc",
             "llmp_gemm_skinny")


@contextlib.contextmanager
def nvtx_range(name: str):
    """An NVTX range around the block when ``LLMP_B200_NVTX=1``; nothing otherwise."""
    if not NVTX:
        yield
        return
    torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        torch.cuda.nvtx.range_pop()


class KernelTimes:
    """``with KernelTimes() as times: runner.step(...)`` then ``times.table()``.

    ``label(name, work)`` may rename a launch: ``name`` is the entry point without its ``llmp_`` prefix (or ``"mm"`` for
    the library product, ``"mm+residual"`` for the library product that adds into the float32 residual), ``work`` is
    (M, N, K) for a matrix product and None otherwise. Events are kept until
    ``fold()`` (called by ``table()``), which waits for the device and adds the intervals up; a long-running user calls
    ``fold()`` now and then."""

    def __init__(self, label: Optional[Callable[[str, Optional[Tuple[int, int, int]]], str]] = None):
        self._label = label
        self.items: List[tuple] = []             # (label, work, start event, stop event) not yet added up
        self.sums: Dict[str, Dict[str, float]] = {}
        self._saved = None
        self._depth = 0

    # -- switching on and off ----------------------------------------------------------------
    def __enter__(self):
        from . import kernels
        self._depth += 1
        if self._depth > 1:
            return self
        self._saved = (kernels._call, torch.mm, kernels.library_add_product)
        call_before, mm_before, add_before = self._saved
        outer = self

        def timed(label, work, fn, *args, **kwargs):
            start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            out = fn(*args, **kwargs)
            stop.record()
            outer.items.append((label, work, start, stop))
            return out

        def call(name, *args):
            short, work = name[5:] if name.startswith("llmp_") else name, None
            if name in _PRODUCTS:
                M, N, K = args[4], args[5], args[6]
                if name == "llmp_gemm_stream_swiglu":
                    N *= 2                                   # I gate rows and I up rows
                work = (M, N, K)
                if name == "llmp_gemm_stream_swiglu" or (name == "llmp_gemm_stream_fused" and args[10]):
                    short += "+swiglu"
            return timed(outer._label(short, work) if outer._label else short, work, call_before, name, *args)

        def mm(a, b, **kwargs):
            work = (a.shape[0], b.shape[1], a.shape[1])
            return timed(outer._label("mm", work) if outer._label else "mm (library)", work, mm_before, a, b, **kwargs)

        def add_product(residual, x, w):
            work = (x.shape[0], w.shape[0], x.shape[1])
            label = outer._label("mm+residual", work) if outer._label else "mm into the residual (library)"
            return timed(label, work, add_before, residual, x, w)

        kernels._call, torch.mm, kernels.library_add_product = call, mm, add_product
        return self

    def __exit__(self, *exc):
        from . import kernels
        self._depth -= 1
        if self._depth == 0:
            kernels._call, torch.mm, kernels.library_add_product = self._saved
            self._saved = None

    # -- results -----------------------------------------------------------------------------
    def fold(self) -> None:
        if not self.items:
            return
        torch.cuda.synchronize()
        for label, work, start, stop in self.items:
            entry = self.sums.setdefault(label, {"launches": 0, "us": 0.0, "bytes": 0.0, "flops": 0.0, "rows": 0})
            entry["launches"] += 1
            entry["us"] += start.elapsed_time(stop) * 1e3
            if work is not None:
                M, N, K = work
                entry["bytes"] += 2.0 * N * K + 2.0 * M * K + 2.0 * M * N        # bfloat16 operands and result
                entry["flops"] += 2.0 * M * N * K
                entry["rows"] = M
        self.items = []

    def table(self) -> Dict[str, Dict[str, float]]:
        """label -> launches, microseconds, and for matrix products their bytes, flops and rows; longest first."""
        self.fold()
        return dict(sorted(((k, dict(v)) for k, v in self.sums.items()), key=lambda kv: -kv[1]["us"]))
