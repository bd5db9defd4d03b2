"""The checked build of the kernel library (-DRB_DEBUG_BOUNDS, loaded with RANNC_KERNEL_DEBUG=1): an index that
comes from data and lies outside its table is reported through the device error word -- nothing traps, nothing
reads or writes out of bounds, and the context stays usable."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CODE = r"""
import torch
from rannc_b200.ops import _lib
from rannc_b200.ops import kernels as K
table = torch.randn(100, 64, device="cuda", dtype=torch.bfloat16)
good = torch.randint(0, 100, (4, 8), device="cuda")
out = K.embed_fwd(good, table)
torch.cuda.synchronize()
assert _lib.read_error() == 0
assert torch.equal(out, table[good])
bad = good.clone()
bad[1, 3] = 100          # one past the end of the table
bad[2, 0] = -5
out = K.embed_fwd(bad, table)
torch.cuda.synchronize()
err = _lib.read_error()
assert err == 3, err      # ERR_BOUNDS
assert (out[1, 3] == 0).all() and (out[2, 0] == 0).all() and torch.equal(out[0], table[good[0]])
# labels of a loss: class index beyond the vocabulary (the ignore marker itself is fine)
logits = torch.randn(6, 64, device="cuda", dtype=torch.bfloat16)
labels = torch.tensor([1, 2, -100, 3, 64, 5], device="cuda")
K.xent_fwd(logits, labels, 64)
torch.cuda.synchronize()
assert _lib.read_error() == 3
labels[4] = 63
loss, _, _ = K.xent_fwd(logits, labels, 64)
torch.cuda.synchronize()
assert _lib.read_error() == 0 and torch.isfinite(loss)
print("CHECKED_BUILD_OK", _lib.lib()._dll._name)
"""


def test_checked_build_reports_out_of_range_indices():
    env = dict(os.environ, RANNC_KERNEL_DEBUG="1")
    r = subprocess.run([sys.executable, "-c", CODE], env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "CHECKED_BUILD_OK" in r.stdout, (r.stdout[-2000:], r.stderr[-3000:])
    assert "_kernels_debug.so" in r.stdout
