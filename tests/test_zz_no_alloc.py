"""ql_amax_scale_noalloc: the allocation-free variant of ql_amax_scale, for callers that may not
allocate device memory while they run (a runtime with a fixed, pre-planned memory budget; a
serving loop that cannot afford an allocator stall).  Its accumulators sit in a fixed array inside
the library, so this file checks four things through the C ABI: the results are bit-identical
to ql_amax_scale's, a second call right after the first is not disturbed by what the first left
in the shared array, a request larger than the array is refused with a clear message, and
repeated calls change neither the driver's free memory nor torch's reservation.
The file name keeps it last in collection order, so a failure here cannot hide other results."""
import pytest
import torch

import qlinear as ql
from qlinear import _lib
from qlinear.tensor import current_stream, ql_view

pytestmark = pytest.mark.gpu


def _both(x, scale_shape, axis, maxbound, scale_dtype):
    """(ql_amax_scale, ql_amax_scale_noalloc) outputs for the same request."""
    L = _lib.lib()
    outs = []
    for fn in (L.ql_amax_scale, L.ql_amax_scale_noalloc):
        s = torch.full(scale_shape, -1.0, dtype=scale_dtype, device=x.device)
        tx, ts = ql_view(x), ql_view(s)
        _lib.check(fn(tx, ts, _lib.make_attrs(axis), maxbound, current_stream(x.device)))
        outs.append(s)
    torch.cuda.synchronize()
    return outs


def test_two_calls_in_a_row_match_the_allocating_entry_point():
    g = torch.Generator(device="cpu").manual_seed(77)
    # first call: many groups with large maxima (per-row scales of a wide bf16 matrix)
    a = (torch.randn((512, 1024), generator=g) * 50).to(torch.bfloat16).cuda()
    want, got = _both(a, (512,), 0, 127.0, torch.bfloat16)
    assert torch.equal(want.view(torch.int16), got.view(torch.int16))
    # second call straight after: fewer groups and much smaller values, so stale maxima left in
    # the shared array by the first call would show up as wrong (too large) scales
    b = (torch.randn((64, 256), generator=g) * 0.01).to(torch.float16).cuda()
    want, got = _both(b, (64,), 0, 448.0, torch.float16)
    assert torch.equal(want.view(torch.int16), got.view(torch.int16))
    # per-tensor and block groupings, f32 scales
    want, got = _both(b, (), None, 7.0, torch.float16)
    assert torch.equal(want.view(torch.int16), got.view(torch.int16))
    c = torch.randn((128, 512), generator=g).cuda()
    want, got = _both(c, (128, 4), None, 7.0, torch.float32)
    assert torch.equal(want, got)


def test_no_device_memory_is_allocated():
    """What the entry point is for: after its first call on the device, further calls leave both the driver's free
    memory and the stream-ordered pool's reservation where they were (16-bit scales are the case in which
    ql_amax_scale takes scratch from that pool)."""
    x = (torch.randn((2048, 512)) * 3).to(torch.bfloat16).cuda()
    s = torch.empty((2048,), dtype=torch.bfloat16, device="cuda")
    L = _lib.lib()
    call = lambda: _lib.check(L.ql_amax_scale_noalloc(ql_view(x), ql_view(s), _lib.make_attrs(0), 448.0, current_stream(x.device)))
    call()   # the first call on a device looks the array's address up
    torch.cuda.synchronize()
    free0, _ = torch.cuda.mem_get_info()
    reserved0 = torch.cuda.memory_reserved()
    for _ in range(8):
        call()
    torch.cuda.synchronize()
    free1, _ = torch.cuda.mem_get_info()
    assert free1 == free0 and torch.cuda.memory_reserved() == reserved0


def test_request_beyond_the_fixed_array_is_refused():
    n = 65536 + 16
    x = torch.ones((n, 2), dtype=torch.float16, device="cuda")
    s = torch.zeros((n,), dtype=torch.float16, device="cuda")
    rc = _lib.lib().ql_amax_scale_noalloc(ql_view(x), ql_view(s), _lib.make_attrs(0), 127.0, current_stream(x.device))
    assert rc == _lib.ERR_UNSUPPORTED
    msg = _lib.lib().ql_last_error().decode()
    assert "65536" in msg and "ql_amax_scale" in msg
    # the allocating entry point takes the same request
    _lib.check(_lib.lib().ql_amax_scale(ql_view(x), ql_view(s), _lib.make_attrs(0), 127.0, current_stream(x.device)))
    torch.cuda.synchronize()
    assert float(s[0]) == pytest.approx(1.0 / 127.0, rel=1e-3)
