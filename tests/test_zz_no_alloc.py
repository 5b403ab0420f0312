"""The allocation-free reduction entry point, called through its exported C symbol.

Some callers of the native library cannot allocate device memory when they need a fixed-order
sum: code that runs while the rollout engine or the trainer owns every free byte of the GPU, a
C / ctypes host without PyTorch's caching allocator, or a probe that must not disturb the memory
it observes. For them ``ix_reduce_sum_noalloc`` keeps its stage-1 partial sums in an array that
is part of the library image. This test checks it against the regular entry point
(``ix_reduce_sum``, which takes caller-provided scratch): same bits, on two calls in a row, the
second shorter than the first so that stale partials of the first call sit in the shared array.
The file name sorts last so a run that stops at the first failure has already run every other test.
"""
import ctypes as C

import pytest
import torch

from skyrl_isoexec_b200.ops import _native

pytestmark = pytest.mark.gpu


def _bind():
    lib = _native.lib()
    fn = lib.ix_reduce_sum_noalloc
    fn.argtypes = [C.c_void_p, C.c_longlong, C.c_int, C.c_int, C.c_void_p, C.c_int, C.c_void_p]
    fn.restype = C.c_int
    lib.ix_reduce_sum_noalloc_max_elems.restype = C.c_longlong
    return lib, fn


def _reference(lib, x, square):
    n = x.numel()
    scratch = torch.empty(max(1, lib.ix_reduce_scratch_elems(n)), device=x.device, dtype=torch.float32)
    out = torch.zeros(1, device=x.device, dtype=torch.float32)
    _native.check(lib.ix_reduce_sum(x.data_ptr(), n, int(x.dtype == torch.float32), int(square), scratch.data_ptr(),
                                    out.data_ptr(), 0, _native.stream()), "ix_reduce_sum")
    return out


def test_noalloc_reduce_matches_regular_entry_point_twice_in_a_row():
    lib, fn = _bind()
    torch.manual_seed(0)
    dev = "cuda"
    cases = [(torch.randn(3_000_017, device=dev), True),                 # first call: many partials
             (torch.randn(70_001, device=dev).bfloat16(), False)]        # second call: fewer, stale ones remain
    for x, square in cases:
        out = torch.full((1,), float("nan"), device=dev, dtype=torch.float32)   # caller-owned output, made before the call
        stream = _native.stream()
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        rc = fn(x.data_ptr(), x.numel(), int(x.dtype == torch.float32), int(square), out.data_ptr(), 0, stream)
        assert rc == 0, lib.ix_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before                    # nothing came from the torch allocator
        want = _reference(lib, x, square)
        assert torch.equal(out.view(torch.int32), want.view(torch.int32))  # same bits as the regular entry point
        ref64 = (x.double() ** 2).sum() if square else x.double().sum()
        assert abs(out.item() - ref64.item()) <= 1e-4 * max(1.0, abs(ref64.item()))
    # accumulate flag adds to the existing value
    x = torch.ones(5000, device=dev)
    out = torch.tensor([2.0], device=dev)
    assert fn(x.data_ptr(), x.numel(), 1, 0, out.data_ptr(), 1, _native.stream()) == 0
    torch.cuda.synchronize()
    assert out.item() == 5002.0


def test_noalloc_reduce_of_bf16_squares_and_of_an_empty_input():
    lib, fn = _bind()
    dev = "cuda"
    torch.manual_seed(1)
    x = torch.randn(123_457, device=dev).bfloat16()
    out = torch.full((1,), float("nan"), device=dev)
    assert fn(x.data_ptr(), x.numel(), 0, 1, out.data_ptr(), 0, _native.stream()) == 0
    torch.cuda.synchronize()
    assert torch.equal(out.view(torch.int32), _reference(lib, x, True).view(torch.int32))
    ref64 = (x.double() ** 2).sum().item()
    assert abs(out.item() - ref64) <= 1e-4 * ref64
    # no elements: the output is set to zero, or left alone when accumulating; the input pointer is not read
    out = torch.tensor([7.5], device=dev)
    assert fn(None, 0, 1, 0, out.data_ptr(), 1, _native.stream()) == 0
    torch.cuda.synchronize()
    assert out.item() == 7.5
    assert fn(None, 0, 1, 0, out.data_ptr(), 0, _native.stream()) == 0
    torch.cuda.synchronize()
    assert out.item() == 0.0
    assert fn(x.data_ptr(), -1, 0, 0, out.data_ptr(), 0, _native.stream()) != 0


def test_noalloc_reduce_rejects_oversized_input():
    lib, fn = _bind()
    limit = lib.ix_reduce_sum_noalloc_max_elems()
    assert limit == 65536 * 4096
    out = torch.zeros(1, device="cuda")
    x = torch.zeros(16, device="cuda")
    rc = fn(x.data_ptr(), limit + 1, 1, 0, out.data_ptr(), 0, _native.stream())   # size is checked before any access
    assert rc != 0 and b"exceed" in lib.ix_last_error()
