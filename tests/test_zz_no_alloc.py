"""The allocation-free cross-entropy entry point, called through its exported C symbol.

Some callers of this library cannot call cudaMalloc at the point where they need the loss (a
framework callback that forbids allocation, a latency-critical loop, a process whose memory is
owned by another pool), so they cannot hand ``tmpi_xent_fwd_bwd`` the scratch buffer it wants.
``tmpi_xent_fwd_bwd_noalloc`` keeps that scratch in an array inside the library.  This test calls
it twice in a row (the shared array keeps the previous call's contents) and compares both results
with the ordinary entry point, and checks that an oversized request is refused with a message.
The file sorts last so that a run that stops at the first failure has already run everything else.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _symbols():
    from torchmpi_b200 import _lib
    fn = _lib.lib.tmpi_xent_fwd_bwd_noalloc          # the exported C symbol itself
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_float, C.c_void_p]
    return _lib, fn


def test_noalloc_xent_matches_regular_entry_point_twice():
    _lib, noalloc = _symbols()
    lib = _lib.lib
    torch.cuda.set_device(0)
    torch.manual_seed(7)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, cols) in enumerate(((256, 1000), (1000, 4099))):     # two calls in a row, different shapes
        logits = (torch.randn(rows, cols, device="cuda") * 2).to(torch.bfloat16)
        labels = torch.randint(0, cols, (rows,), device="cuda")
        loss_a, loss_b = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
        d_a, d_b = torch.empty_like(logits), torch.empty_like(logits)
        scratch = torch.zeros(lib.tmpi_xent_scratch_bytes(rows), dtype=torch.uint8, device="cuda")
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        st = noalloc(logits.data_ptr(), 6, labels.data_ptr(), rows, cols, loss_a.data_ptr(), d_a.data_ptr(),
                     1.0 / rows, stream)
        assert st == 0, _lib.last_error()
        assert torch.cuda.memory_allocated() == before       # nothing was taken from torch's allocator either
        _lib.check(lib.tmpi_xent_fwd_bwd(logits.data_ptr(), 6, labels.data_ptr(), rows, cols, loss_b.data_ptr(),
                                         d_b.data_ptr(), 1.0 / rows, scratch.data_ptr(), stream))
        torch.cuda.synchronize()
        assert torch.allclose(loss_a, loss_b, atol=1e-4, rtol=1e-5), (call, loss_a.item(), loss_b.item())
        assert torch.allclose(d_a.float(), d_b.float(), atol=1e-6, rtol=2e-2)
        ref = torch.nn.functional.cross_entropy(logits.float(), labels, reduction="sum")
        assert torch.allclose(loss_a[0], ref, atol=1e-2, rtol=1e-4)


def _both(lib_mod, noalloc, logits, labels, want_grad, stream_ptr):
    """(loss, dlogits) from the allocation-free entry point and from the ordinary one, on one stream."""
    lib = lib_mod.lib
    rows, cols = logits.shape
    loss_a, loss_b = torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda")
    d_a = torch.empty_like(logits) if want_grad else None
    d_b = torch.empty_like(logits) if want_grad else None
    scratch = torch.zeros(lib.tmpi_xent_scratch_bytes(rows), dtype=torch.uint8, device="cuda")
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info()[0]
    st = noalloc(logits.data_ptr(), 6, labels.data_ptr(), rows, cols, loss_a.data_ptr(),
                 d_a.data_ptr() if want_grad else None, 1.0 / rows, stream_ptr)
    assert st == 0, lib_mod.last_error()
    torch.cuda.synchronize()
    # the driver's own count of free device memory: a cudaMalloc inside the library would show here
    assert torch.cuda.mem_get_info()[0] == free_before
    lib_mod.check(lib.tmpi_xent_fwd_bwd(logits.data_ptr(), 6, labels.data_ptr(), rows, cols, loss_b.data_ptr(),
                                        d_b.data_ptr() if want_grad else None, 1.0 / rows, scratch.data_ptr(), stream_ptr))
    torch.cuda.synchronize()
    return loss_a, loss_b, d_a, d_b


def test_noalloc_xent_largest_row_count_and_no_gradient():
    """rows == TMPI_XENT_NOALLOC_MAX_ROWS is accepted; dlogits == NULL computes the loss only."""
    _lib, noalloc = _symbols()
    torch.cuda.set_device(0)
    torch.manual_seed(11)
    stream = torch.cuda.current_stream().cuda_stream
    warm = (torch.randn(8, 64, device="cuda")).to(torch.bfloat16)          # first call on the device does the set-up
    _both(_lib, noalloc, warm, torch.randint(0, 64, (8,), device="cuda"), True, stream)
    logits = torch.randn(16384, 136, device="cuda").to(torch.bfloat16)
    labels = torch.randint(0, 136, (16384,), device="cuda")
    for want_grad in (True, False):
        la, lb, da, db = _both(_lib, noalloc, logits, labels, want_grad, stream)
        assert torch.allclose(la, lb, atol=1e-3, rtol=1e-5)
        if want_grad:
            assert torch.allclose(da.float(), db.float(), atol=1e-6, rtol=2e-2)


def test_noalloc_xent_on_a_side_stream_after_the_default_stream():
    """Two calls in sequence on one non-default stream, right after a call on the default stream: the
    shared array is cleared per call on the caller's stream, so each result must match."""
    _lib, noalloc = _symbols()
    torch.cuda.set_device(0)
    torch.manual_seed(13)
    logits = (torch.randn(512, 777, device="cuda") * 3).to(torch.bfloat16)
    labels = torch.randint(0, 777, (512,), device="cuda")
    la, lb, _, _ = _both(_lib, noalloc, logits, labels, True, torch.cuda.current_stream().cuda_stream)
    assert torch.allclose(la, lb, atol=1e-4, rtol=1e-5)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):
            la, lb, da, db = _both(_lib, noalloc, logits, labels, True, side.cuda_stream)
            assert torch.allclose(la, lb, atol=1e-4, rtol=1e-5)
            assert torch.allclose(da.float(), db.float(), atol=1e-6, rtol=2e-2)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()


def test_noalloc_xent_rejects_too_many_rows():
    _lib, noalloc = _symbols()
    rows = 16384 + 1
    x = torch.zeros(1, device="cuda")
    st = noalloc(x.data_ptr(), 7, x.data_ptr(), rows, 8, x.data_ptr(), None, 1.0,
                 torch.cuda.current_stream().cuda_stream)
    assert st == _lib.ERR_INVALID
    assert "16384" in _lib.last_error()
