"""The allocation-free greedy selection, called through its exported C symbol.

Some hosts cannot allocate device memory when they pick tokens (their pool owns the whole device, or
they are called from inside another framework's step).  ``gesso_argmax_rows_static`` keeps its
scratch inside the library; this test calls it as such a host would, with plain pointers through
ctypes, twice in a row on one stream, and compares with the regular entry point.  The file sorts last
on purpose: a run that stops at its first failure has then run every other test already.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 256
TOO_MANY_ROWS, BAD_ARGUMENT = -10, -11


def entry_point():
    from gesso_b200.csrc import lib
    fn = lib.library().gesso_argmax_rows_static
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return fn


def call(fn, logits, ids, bad):
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    return fn(ctypes.c_void_p(logits.data_ptr()), logits.shape[0], logits.shape[1], ctypes.c_void_p(ids.data_ptr()),
              ctypes.c_void_p(bad.data_ptr()), stream)


def test_static_argmax_matches_the_regular_entry_point_twice_in_a_row():
    from gesso_b200 import ops
    fn = entry_point()
    g = torch.Generator().manual_seed(11)
    first = torch.randn(8, 65536, generator=g)
    first[0, 70] = first[0, 60000] = 9.0           # a tie: the lowest index wins
    first[3, 12345] = float("nan")
    second = torch.randn(64, 503, generator=g)     # other sizes, the same scratch
    second[5, 502] = 50.0
    second[9, 0] = float("inf")
    # everything the host needs exists before the calls: they must not allocate
    bufs = []
    for x in (first, second):
        x = x.cuda()
        bufs.append((x, torch.full((x.shape[0],), -7, dtype=torch.int32, device="cuda"),
                     torch.full((x.shape[0],), -7, dtype=torch.int32, device="cuda")))
    # the set-up call: the first call on a device looks the scratch array's address up, and the driver loads
    # the kernels' code at their first launch; neither is what the calls below may do
    warm = torch.zeros(2, 65536, device="cuda")
    warm_small = torch.zeros(2, 503, device="cuda")
    for w in (warm, warm_small):
        assert call(fn, w, torch.zeros(2, dtype=torch.int32, device="cuda"),
                    torch.zeros(2, dtype=torch.int32, device="cuda")) == 0
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()         # torch's own allocator ...
    free_before, _ = torch.cuda.mem_get_info()     # ... and the driver's view: a cudaMalloc inside would show here
    for x, ids, bad in bufs:                       # two calls in a row, the second reuses the scratch
        assert call(fn, x, ids, bad) == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    assert torch.cuda.mem_get_info()[0] == free_before, "the device's free memory changed: something allocated"
    for x, ids, bad in bufs:
        want_ids, want_bad = ops.argmax_rows(x)
        assert torch.equal(ids, want_ids) and torch.equal(bad, want_bad)
    assert bufs[0][1][0].item() == 70 and bufs[0][2].tolist()[3] == 1 and bufs[1][1][5].item() == 502
    # and again on the first input: stale partial results of the second call must not leak in
    x, ids, bad = bufs[0]
    ids.fill_(-7)
    assert call(fn, x, ids, bad) == 0
    assert torch.equal(ids, ops.argmax_rows(x)[0])


def test_static_argmax_refuses_what_it_cannot_hold():
    fn = entry_point()
    x = torch.zeros(MAX_ROWS + 1, 16, device="cuda")
    ids = torch.full((MAX_ROWS + 1,), -7, dtype=torch.int32, device="cuda")
    bad = torch.zeros(MAX_ROWS + 1, dtype=torch.int32, device="cuda")
    assert call(fn, x, ids, bad) == TOO_MANY_ROWS
    torch.cuda.synchronize()
    assert bool((ids == -7).all())                 # nothing ran
    assert call(fn, x[:MAX_ROWS], ids, bad) == 0   # the largest size it takes
    torch.cuda.synchronize()
    assert bool((ids[:MAX_ROWS] == 0).all())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    assert fn(None, 1, 16, ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(bad.data_ptr()), stream) == BAD_ARGUMENT
    assert fn(ctypes.c_void_p(x.data_ptr()), 1, 0, ctypes.c_void_p(ids.data_ptr()), ctypes.c_void_p(bad.data_ptr()),
              stream) == BAD_ARGUMENT
