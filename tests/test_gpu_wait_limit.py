"""The bounded device-side waits, exercised without faulting or hanging anything.

A test-only switch (NUMR_B200_TEST_HOLD_ARRIVAL=1) makes the MMA issuer withhold one mbarrier
arrival: the "accumulator complete" signal of a one-tile problem. No copy or MMA is outstanding when
the epilogue warps then wait for it, so after NUMR_B200_WAIT_LIMIT_MS their wait runs out, the kernel
records the code, frees its TMEM and returns; the context stays usable. Runs in a child process so
the switches (read once per process unless re-read) and the status word start clean.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import os, sys, time
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/tests")
import numpy as np, torch
from numr_b200 import CudaClient, _lib
from oracle import oracle as O
from helpers import to_torch, to_numpy, random_operand, assert_ulp_close

dev = torch.device("cuda:0")
client = CudaClient(0)
rng = np.random.default_rng(3)
m, n, k = {m}, 64, 64
a = random_operand(rng, (m, k), O.BF16); b = random_operand(rng, (k, n), O.BF16)
ta, tb = to_torch(a, O.BF16, dev), to_torch(b, O.BF16, dev)
for attempt in range(2):   # the first launch of a process also loads the kernels: time the second
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    out = client.matmul(ta, tb)   # the arrival is withheld
    torch.cuda.synchronize()
    waited = time.perf_counter() - t0
    st = client.device_status()
    assert st == 4, f"expected status 4 (epilogue wait ran out), got {{st}}"
    assert client.device_status() == 0, "reading the status word must clear it"
assert waited < 0.5, f"the kernel took {{waited:.3f}} s to give up (limit 5 ms per wait)"
# the context is intact: with the switch off an ordinary GEMM in the same process is right
del os.environ["NUMR_B200_TEST_HOLD_ARRIVAL"]
_lib.load().numr_b200_reload_tuning()
a = random_operand(rng, (200, 264), O.BF16); b = random_operand(rng, (264, 304), O.BF16, 0.1)
out = client.matmul(to_torch(a, O.BF16, dev), to_torch(b, O.BF16, dev))
want = O.gemm(O.BF16, a, b)
assert_ulp_close(to_numpy(out, O.BF16), want, O.BF16, floor=1e-5, what="GEMM after a timed-out one")
assert client.device_status() == 0
print("ok")
"""


@pytest.mark.parametrize("m,pair", [(128, "0"), (256, "1")], ids=["single-cta", "cta-pair"])
def test_epilogue_wait_runs_out_and_the_context_survives(m, pair):
    env = dict(os.environ)
    env.update({"NUMR_B200_WAIT_LIMIT_MS": "5", "NUMR_B200_TEST_HOLD_ARRIVAL": "1", "NUMR_B200_FORCE_PAIR": pair})
    r = subprocess.run([sys.executable, "-c", CHILD.format(root=str(ROOT), m=m)], env=env, capture_output=True,
                       text=True, timeout=300)
    assert r.returncode == 0 and r.stdout.strip().endswith("ok"), f"child failed:\n{r.stdout}\n{r.stderr}"
