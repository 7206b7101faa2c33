"""The debug build of the kernels (-DHIPRESS_DEBUG, loaded with HIPRESS_DEBUG=1):
every payload-slot index is checked against its inbox; a violation is recorded in the
status word and the access is skipped.  It stands in for compute-sanitizer where that
tool cannot be used.  The test runs in a child process because the choice of library
is made once per process."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]

CHILD = r"""
import torch
from hipress_b200._native import lib
from hipress_b200.ops import Compressor
from hipress_b200.parallel.fused import FusedDenseBucket, HipressTimeoutError, decode_status
L = lib.cuda()
assert L.hp_cuda_debug_build() == 1
c = Compressor("tbq")
N, n = 2, 60000
# 1. a correct launch passes every check
b = FusedDenseBucket(c.spec, "ring", [n], N, 0, ctas=8, emulate=True, timeout_s=2.0).bind_local("cuda")
G = torch.randn(N, n, device="cuda") * 0.02
R = torch.zeros(N, n, device="cuda")
O = torch.zeros(N, n, device="cuda")
b.launch([G], [R], [O])
torch.cuda.synchronize()
b.check_status()
assert torch.equal(O[0], O[1]) and float(O.abs().sum()) > 0
# 2. pretend the inboxes are half as long: the checks fire, nothing outside the
#    pretended limit is touched, the launch ends (the skipped tiles never arrive, so
#    their waits expire) and the first recorded status is the bounds violation
assert L.hp_cuda_debug_set_inbox_limit(b.inbox_bytes // 2) == 0
b2 = FusedDenseBucket(c.spec, "ring", [n], N, 0, ctas=8, emulate=True, timeout_s=0.3).bind_local("cuda")
b2.launch([G], [R], [O])
torch.cuda.synchronize()
words = [w & 0xFFFFFFFF for w in b2.status.cpu().tolist()]
assert any(w & 0x20000000 and not w & 0x80000000 for w in words), [hex(w) for w in words]
assert "left its inbox" in decode_status(next(w for w in words if w & 0x20000000))
tail = b2._arena[b2.inbox_bytes // 2:b2.inbox_bytes]      # rank 0's inbox beyond the limit
assert int(tail.count_nonzero()) == 0, "a skipped access still wrote"
# 3. back to the real limit: the context is intact and the kernel works
assert L.hp_cuda_debug_set_inbox_limit(0) == 0
b3 = FusedDenseBucket(c.spec, "ring", [n], N, 0, ctas=8, emulate=True).bind_local("cuda")
b3.launch([G], [R], [O])
torch.cuda.synchronize()
b3.check_status()
print("DEBUG_BUILD_OK")
"""


def test_debug_build_checks_record_and_skip():
    env = dict(os.environ, HIPRESS_DEBUG="1", PYTHONPATH=str(ROOT))
    r = subprocess.run([sys.executable, "-c", CHILD], env=env, capture_output=True, text=True, timeout=900,
                       cwd=ROOT)
    assert r.returncode == 0 and "DEBUG_BUILD_OK" in r.stdout, r.stdout[-2000:] + r.stderr[-4000:]
