"""The allocation-free argmax entry point, called through its exported C symbol.

Some hosts of the library cannot allocate device memory when they call it (they gave the whole GPU
to their own pool, or cannot afford an allocation's device-wide synchronisation), so
``llmp_argmax_no_alloc`` keeps its scratch inside the library image. This file is named to be
collected last: should it fail, every other test has already run."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _entry():
    from llm_pipeline_b200.ops.build import build_library
    lib = ctypes.CDLL(build_library())
    fn = lib.llmp_argmax_no_alloc
    fn.argtypes = [ctypes.c_void_p, ctypes.c_long, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    lib.llmp_last_error.restype = ctypes.c_char_p
    return lib, fn


def test_no_alloc_argmax_matches_the_regular_entry_point_twice_in_a_row():
    from llm_pipeline_b200.ops import kernels
    lib, fn = _entry()
    gen = torch.Generator().manual_seed(5)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, vocab) in enumerate(((8, 151936), (64, 33001))):      # two calls in a row share the scratch
        logits = torch.randn(rows, vocab, generator=gen).cuda()
        logits[1, 77] = logits[1, vocab - 5] = logits[1].max() + 1          # a tie: the lower index wins
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        before = torch.cuda.memory_allocated()
        rc = fn(logits.data_ptr(), logits.stride(0), rows, vocab, got.data_ptr(), stream)
        assert rc == 0, lib.llmp_last_error().decode()
        assert torch.cuda.memory_allocated() == before                     # nothing went through torch's allocator
        want = kernels.argmax(logits, torch.empty(rows, dtype=torch.int32, device="cuda"))
        torch.cuda.synchronize()
        assert got.tolist() == want.tolist() == logits.cpu().argmax(dim=-1).tolist(), call
        assert got[1] == 77


def test_no_alloc_argmax_refuses_more_rows_than_its_scratch_holds():
    lib, fn = _entry()
    logits = torch.zeros(4, 16, device="cuda")
    out = torch.zeros(2000, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(logits.data_ptr(), 16, 1025, 16, out.data_ptr(), stream) != 0
    assert b"1..1024" in lib.llmp_last_error()
    assert fn(logits.data_ptr(), 16, 0, 16, out.data_ptr(), stream) != 0
    assert fn(logits.data_ptr(), 16, 4, 16, out.data_ptr(), stream) == 0   # still usable after a refusal
    torch.cuda.synchronize()
    assert out[:4].tolist() == [0, 0, 0, 0]


def test_no_alloc_source_names_no_allocating_call():
    """The check on torch's allocator above cannot see a raw runtime allocation inside the library, so the source
    is read: the file names none of the runtime's allocating or freeing calls."""
    import os
    import re
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    with open(os.path.join(root, "llm-pipeline_b200", "csrc", "argmax_no_alloc.cu")) as f:
        code = re.sub(r"//[^\n]*", "", f.read())
    for name in ("cudaMalloc", "cudaFree", "cudaMallocAsync", "cudaHostAlloc", "cuMemAlloc", "new ", "malloc("):
        assert name not in code, name
