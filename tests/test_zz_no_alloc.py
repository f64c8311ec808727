"""The allocation-free norm backward (``hg_norm_bwd_noalloc``) against the regular entry point.

Called through the exported C symbol, twice in a row with different inputs, so that the second call runs on
scratch that still holds the first call's partial sums.  Collected last on purpose: it must pass both on its own
and after every other GPU test has used the device."""
import ctypes

import pytest
import torch

from hetu_galvatron_b200.ops import _lib

pytestmark = pytest.mark.gpu
MAX_H, PARTS, TOO_WIDE, NULL_ARG = 8192, 148, -2, -3


def _symbol():
    lib = _lib.load()
    fn = lib.hg_norm_bwd_noalloc
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_int] * 4 + [ctypes.c_void_p]
    fn.restype = ctypes.c_int
    return lib, fn


def _inputs(rows, H, rms, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    r = lambda *s: torch.randn(*s, device="cuda", generator=g)  # noqa: E731
    h = r(rows, H).bfloat16()
    dy = r(rows, H).bfloat16()
    dres = r(rows, H).bfloat16()
    w = (1.0 + 0.1 * r(H)).bfloat16()
    hf = h.float()
    mean = None if rms else hf.mean(-1).contiguous()
    var = hf.pow(2).mean(-1) if rms else hf.var(-1, unbiased=False)
    rstd = torch.rsqrt(var + 1e-5).contiguous()
    return dy, h, w, rstd, mean, dres


def _run_regular(lib, t, rows, H, rms):
    dy, h, w, rstd, mean, dres = t
    dx = torch.empty_like(h)
    dw = torch.empty(H, dtype=torch.float32, device="cuda")
    db = None if rms else torch.zeros(H, dtype=torch.float32, device="cuda")
    partial = torch.empty(2 * PARTS * H, dtype=torch.float32, device="cuda")
    rc = lib.hg_norm_bwd(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(mean), dres.data_ptr(),
                         dx.data_ptr(), dw.data_ptr(), _lib.ptr(db), partial.data_ptr(), PARTS, rows, H, int(rms), 0,
                         _lib.stream())
    assert rc == 0
    return dx, dw, db


def _run_noalloc(fn, t, rows, H, rms, check_driver_memory=False):
    dy, h, w, rstd, mean, dres = t
    dx = torch.empty_like(h)
    dw = torch.empty(H, dtype=torch.float32, device="cuda")
    db = None if rms else torch.zeros(H, dtype=torch.float32, device="cuda")
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    rc = fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), _lib.ptr(mean), dres.data_ptr(),
            dx.data_ptr(), dw.data_ptr(), _lib.ptr(db), rows, H, int(rms), 0, _lib.stream())
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    if check_driver_memory:
        # the driver's own count of free device memory also sees a raw cudaMalloc, which torch's counter does not
        # (the first call on a device may still load the kernels' module, so only later calls are held to this)
        assert torch.cuda.mem_get_info()[0] >= free_before
    return dx, dw, db


def _close(a, b, tol=1e-5):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item() < tol


@pytest.mark.parametrize("rms", [True, False])
def test_noalloc_matches_regular_on_two_calls_in_a_row(rms):
    lib, fn = _symbol()
    # second call: fewer rows than scratch rows and a different width, on top of the first call's leftovers
    # then the widest supported row and a width between the two kernel instantiations
    for call, (rows, H, seed) in enumerate(((1000, 4096, 1), (90, 2048, 2), (300, 8192, 3), (257, 5120, 4))):
        t = _inputs(rows, H, rms, seed)
        want = _run_regular(lib, t, rows, H, rms)
        got = _run_noalloc(fn, t, rows, H, rms, check_driver_memory=call > 0)
        torch.cuda.synchronize()
        for g, w_ in zip(got, want):
            if w_ is not None:
                assert _close(g, w_)
    _lib.assert_healthy()


def test_noalloc_rejects_widths_beyond_the_static_array():
    _, fn = _symbol()
    x = torch.zeros(8, device="cuda")
    p = x.data_ptr()
    assert fn(p, p, p, p, 0, 0, p, p, 0, 4, 2 * MAX_H, 1, 0, _lib.stream()) == TOO_WIDE
    assert fn(p, p, p, p, 0, 0, p, p, 0, 4, 100, 1, 0, _lib.stream()) == -1


def test_noalloc_rejects_null_pointers_before_launching():
    _, fn = _symbol()
    x = torch.zeros(8, device="cuda")
    p = x.data_ptr()
    st = _lib.stream()
    assert fn(0, p, p, p, 0, 0, p, p, 0, 1, 8, 1, 0, st) == NULL_ARG        # dy
    assert fn(p, p, p, p, 0, 0, 0, p, 0, 1, 8, 1, 0, st) == NULL_ARG        # dx
    assert fn(p, p, p, p, 0, 0, p, 0, 0, 1, 8, 1, 0, st) == NULL_ARG        # dw
    assert fn(p, p, p, p, 0, 0, p, p, 0, 1, 8, 0, 0, st) == NULL_ARG        # LayerNorm without mean
    torch.cuda.synchronize()
    _lib.assert_healthy()
