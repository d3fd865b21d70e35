"""mx8_moe_schedule_static: the routing schedule for hosts that cannot supply scratch memory.

Such hosts (a serving process with a memory plan frozen at start-up, a plugin living under another
component's allocator) call this entry point instead of mx8_moe_schedule; its scratch is an array
inside the library.  The test calls it through the C ABI several times in a row on different inputs and
requires exactly the outputs of the caller-scratch entry point, which shows that nothing left in
the shared array by one call leaks into the next; it also reads the device's free memory around the
calls, which an allocation on the way would lower."""
import ctypes

import pytest
import torch

import mx8
from mx8 import _lib

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _routing(W, T, E_total, k, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.topk(torch.randn(W * T, E_total, generator=g), k, dim=1).indices.to(torch.int32).view(W, T, k)


def _run(lib, fn_static, topk_all, E_local, cap, rank):
    W, T, k = topk_all.shape
    dev_topk = topk_all.to(DEV)
    outs = []
    for static in (False, True):
        pr = torch.full((cap,), -7, dtype=torch.int32, device=DEV)
        pt = torch.full((cap,), -7, dtype=torch.int32, device=DEV)
        nt = torch.full((1,), -7, dtype=torch.int32, device=DEV)
        tpe = torch.full((E_local,), -7, dtype=torch.int32, device=DEV)
        stream = torch.cuda.current_stream().cuda_stream
        if static:
            rc = fn_static(dev_topk.data_ptr(), W, T, k, E_local, cap, rank, pr.data_ptr(), pt.data_ptr(), nt.data_ptr(),
                           tpe.data_ptr(), stream)
        else:
            scratch = torch.empty(E_local * (W + 1), dtype=torch.int32, device=DEV)
            rc = lib.mx8_moe_schedule(dev_topk.data_ptr(), W, T, k, E_local, cap, rank, pr.data_ptr(), pt.data_ptr(),
                                      nt.data_ptr(), tpe.data_ptr(), scratch.data_ptr(), scratch.numel() * 4, stream)
        assert rc == _lib.OK
        assert mx8.device_status() == 0
        outs.append((pr.cpu(), pt.cpu(), nt.cpu(), tpe.cpu()))
    return outs


def test_static_scratch_schedule_matches_and_repeats():
    lib = mx8.load()
    fn = lib.mx8_moe_schedule_static
    # calls in a row: a large problem first, then a smaller one with other routing, so stale counts from
    # the first call would corrupt the second if they were not cleared.  The first two fit the
    # counting-sort form into the built-in array; the third needs 16672 ints for it (64 chunks per rank
    # x 8 ranks x 32 experts + 288), so the entry point takes the scan-per-expert form there, which must
    # clear the counters the earlier calls left dirty
    for (W, T, E_local, k, rank, seed) in ((8, 512, 32, 8, 3, 1), (2, 256, 4, 4, 1, 2), (8, 8192, 32, 8, 5, 3)):
        topk_all = _routing(W, T, W * E_local, k, seed)
        cap = ((W * T * k) // 256 + E_local) * 256
        ref, got = _run(lib, fn, topk_all, E_local, cap, rank)
        valid = ref[0] >= 0
        assert torch.equal(got[0], ref[0]) and torch.equal(got[2], ref[2]) and torch.equal(got[3], ref[3])
        assert torch.equal(got[1][valid], ref[1][valid])


def test_static_scratch_schedule_leaves_free_memory_alone():
    lib = mx8.load()
    W, T, E_local, k, rank = 4, 1024, 8, 4, 2
    topk_all = _routing(W, T, W * E_local, k, 7).to(DEV)
    cap = ((W * T * k) // 256 + E_local) * 256
    pr = torch.empty(cap, dtype=torch.int32, device=DEV)
    pt = torch.empty(cap, dtype=torch.int32, device=DEV)
    nt = torch.empty(1, dtype=torch.int32, device=DEV)
    tpe = torch.empty(E_local, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda: lib.mx8_moe_schedule_static(topk_all.data_ptr(), W, T, k, E_local, cap, rank, pr.data_ptr(), pt.data_ptr(),
                                               nt.data_ptr(), tpe.data_ptr(), stream)
    assert call() == _lib.OK            # the first call on a device resolves the array's address
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(0)[0]
    for _ in range(3):
        assert call() == _lib.OK
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(0)[0] == free_before
    assert mx8.device_status() == 0


def test_static_scratch_limit_is_an_error():
    lib = mx8.load()
    p = ctypes.c_void_p(4096)
    rc = lib.mx8_moe_schedule_static(p, 64, 16, 2, 300, 256, 0, p, p, p, p, None)     # 300 * 65 > 16384
    assert rc == _lib.ERR_LIMIT
    assert b"16384" in lib.mx8_last_cuda_error()
