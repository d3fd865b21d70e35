"""Reentrancy of the C ABI: host threads calling the library at the same time on streams of their own.
The entry points keep per-device caches (SM count, kernel attributes, launch limits) that the first calls fill;
here those first calls race on purpose, in a fresh process, and every result is compared with the oracle."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r'''
import sys, threading
sys.path.insert(0, ROOT); sys.path.insert(0, ROOT + "/gpu-experiments_b200")
import torch
import mx8
from oracle import mx8_oracle as O
DEV = "cuda:0"
torch.zeros(1, device=DEV)                       # context only: no library call before the threads start
inputs = [O.make_input(256 + 128 * (i % 3), 384, seed=70 + i, outliers=(i % 2 == 0)) for i in range(4)]
ops = [tuple(t.to(DEV) for t in O.quantize_tiled(O.make_input(256, 512, seed=90 + i, std=512 ** -0.25)) +
             O.quantize_tiled(O.make_input(384, 512, seed=95 + i, std=512 ** -0.25))) for i in range(4)]
want_q = [O.quantize_both(x) for x in inputs]
want_c = [O.gemm_ref(*[t.cpu() for t in o]) for o in ops]
errors, barrier = [], threading.Barrier(4)

def worker(i):
    try:
        s = torch.cuda.Stream(device=DEV)
        x = inputs[i].to(DEV)
        barrier.wait()
        with torch.cuda.stream(s):
            for rep in range(25):
                got = mx8.mxfp8_quantize(x, True, True)
                c = torch.empty(256, 384, dtype=torch.bfloat16, device=DEV)
                mx8.kernel(*ops[i], c)
                s.synchronize()
                for g, w in zip(got, want_q[i]):
                    if not torch.equal(g.view(torch.uint8).cpu().reshape(w.shape), w):
                        errors.append(("quantize", i, rep))
                if O.rel_frobenius(c.cpu(), want_c[i]) > 2e-3:
                    errors.append(("gemm", i, rep))
    except Exception as e:                        # noqa: BLE001
        errors.append(("exception", i, repr(e)))

threads = [threading.Thread(target=worker, args=(i,)) for i in range(4)]
for t in threads: t.start()
for t in threads: t.join()
assert not errors, errors[:5]
assert mx8.device_status() == 0
print("THREADS_OK")
'''


def test_four_host_threads_share_the_library():
    r = subprocess.run([sys.executable, "-c", "ROOT = %r\n" % ROOT + CHILD], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "THREADS_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
