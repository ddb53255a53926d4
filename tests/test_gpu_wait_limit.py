"""A bounded wait that runs out: the kernel reports it and returns, and the GPU stays usable.

Uses a test build of the library (`-DB200_WAIT_TEST=1 -DB200_WAIT_LIMIT_CYCLES=3000000`, about
2 ms, made by `__graft_entry__.build()` as `mlops_b200/libb200moe_waittest.so`) whose GEMM
producers can be told to load nothing: the issuers' and the epilogues' waits then run out,
status[0] becomes 1 (ERR_WAIT_TIMEOUT), every role unwinds and the kernel ends. Nothing traps,
faults or spins without a limit. The case runs in a process of its own because a process loads
one build of the library."""

import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
VARIANT = ROOT / "mlops_b200" / "libb200moe_waittest.so"

SCRIPT = r"""
import ctypes, os, sys, time
import torch
sys.path.insert(0, os.environ["B200MOE_ROOT"])
from mlops_b200 import ops
from mlops_b200._lib import NativeError
lib = ctypes.CDLL(os.environ["B200MOE_LIBRARY"])
dev = "cuda:0"
g = torch.Generator(device=dev).manual_seed(0)
a = torch.randn(600, 512, device=dev, generator=g).bfloat16()
a_q, a_s = ops.quantize_rows(a)
b_q, b_s = ops.quantize_blocks(torch.randn(3, 384, 512, device=dev, generator=g).bfloat16())
offsets = torch.tensor([0, 130, 130, 600], dtype=torch.int32, device=dev)
good = ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets)
torch.cuda.synchronize()
ops.check_status(dev)
lib.b200moe_debug_withhold_loads(1)
start = time.perf_counter()
ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets)
torch.cuda.synchronize()                      # the kernel RETURNED although nothing ever arrived
elapsed = time.perf_counter() - start
status = ops.status_block(dev).tolist()
assert status[0] == 1, status                 # ERR_WAIT_TIMEOUT, with the role that gave up first
try:
    ops.check_status(dev)
    raise SystemExit("check_status did not raise")
except NativeError as error:
    assert "bounded wait ran out" in str(error)
lib.b200moe_debug_withhold_loads(0)
again = ops.grouped_gemm_fp8(a_q, a_s, b_q, b_s, offsets)   # the next launch is healthy
torch.cuda.synchronize()
ops.check_status(dev)
assert torch.equal(again, good)
print(f"wait limit ok: status={status} returned after {elapsed * 1e3:.1f} ms")
"""


def test_a_wait_that_runs_out_is_reported_and_the_next_launch_is_healthy():
    if not VARIANT.exists():
        pytest.skip("the wait-test build of the library is missing (run __graft_entry__.build())")
    env = dict(os.environ, B200MOE_LIBRARY=str(VARIANT), B200MOE_ROOT=str(ROOT))
    done = subprocess.run([sys.executable, "-c", SCRIPT], capture_output=True, text=True, timeout=300, env=env)
    assert done.returncode == 0, done.stdout[-2000:] + done.stderr[-3000:]
    assert "wait limit ok" in done.stdout
