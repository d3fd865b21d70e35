"""Failure reporting without a fault: a bounded wait that runs out sets the device status word, the kernel
returns normally and the device stays usable.  Every wait inside the library's kernels goes through the same
routine (csrc/mx8_ptx.cuh, mbar_wait); mx8_selftest_bounded_wait makes one of them expire on purpose by
waiting, for a few milliseconds at most, on a barrier that nothing signals."""
import ctypes
import time

import pytest
import torch

import mx8
from mx8 import _lib
from oracle import mx8_oracle as O

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_expired_wait_is_reported_and_the_device_stays_usable():
    lib = mx8.load()
    st = torch.cuda.current_stream().cuda_stream
    assert mx8.device_status() == 0
    t0 = time.perf_counter()
    assert lib.mx8_selftest_bounded_wait(3000, st) == _lib.OK          # 3 ms
    word = ctypes.c_int(0)
    rc = lib.mx8_device_status(ctypes.byref(word), st)
    elapsed = time.perf_counter() - t0
    assert rc == _lib.ERR_DEVICE_TIMEOUT and word.value == 8
    assert 0.003 <= elapsed < 1.0                                       # gave up after its limit, not the library's 2 s
    assert b"bounded wait" in lib.mx8_strerror(rc)
    # the Python host raises on a set word, and the read cleared it
    assert lib.mx8_selftest_bounded_wait(1000, st) == _lib.OK
    with pytest.raises(mx8.Mx8Error):
        mx8.device_status()
    assert mx8.device_status() == 0
    # the next launches work and are correct
    x = O.make_input(256, 384, seed=1, outliers=True)
    got = mx8.mxfp8_quantize(x.to(DEV), True, True)
    want = O.quantize_both(x)
    assert mx8.device_status() == 0
    for g, w in zip(got, want):
        assert torch.equal(g.view(torch.uint8).cpu(), w)


def test_selftest_limit_is_bounded():
    lib = mx8.load()
    assert lib.mx8_selftest_bounded_wait(0, None) == _lib.ERR_ARG
    assert lib.mx8_selftest_bounded_wait(2000000, None) == _lib.ERR_ARG   # never more than a second
