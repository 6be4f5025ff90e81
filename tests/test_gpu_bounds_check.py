"""GPU: the debug flavour of the library (libaxconv_check.so, -DAXC_BOUNDS_CHECK), in which every shared-memory address
the kernels compute and every global index they form is checked before use and a violation is recorded instead of
trapping.  A child process loads that flavour, runs dense and depthwise shapes that exercise every kernel variant
(scheduled kernel with main and tail launches, kernel without a plan, reference-order kernel, expanded-table depthwise
kernels with TMA and with plain loads, the small depthwise kernels) against the CPU checker, and must end with an empty
violation record.  The normal build answers the same call with Unimplemented."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import ctypes as C, sys
import numpy as np, torch
sys.path.insert(0, %r)
import tf_approximate_b200 as ax
from tf_approximate_b200 import _lib
from oracle import oracle as O
L = _lib.load()
rec = (C.c_uint32 * 4)()
assert L.axc_debug_bounds_record(0, rec) == 0, "not the debug flavour"
lut = ax.noisy_table(3555)
t = ax.Table(array=lut)
rng = np.random.Generator(np.random.PCG64(55))
dense = [(2, 9, 11, 5, 3, 3, 7, 1, "SAME"), (1, 17, 13, 8, 3, 3, 40, 1, "SAME"), (1, 21, 19, 3, 7, 7, 64, 2, "SAME"),
         (1, 4, 4, 512, 3, 3, 33, 1, "SAME"), (2, 112, 112, 8, 3, 3, 32, 1, "SAME"), (1, 64, 64, 32, 1, 1, 160, 1, "SAME"),
         (1, 64, 64, 16, 3, 3, 144, 1, "SAME"), (1, 30, 30, 2, 5, 5, 3, 3, "VALID")]
for n, h, w, c, kh, kw, co, s, pad in dense:
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    ref = O.conv2d(O.desc(n, h, w, c, kh, kw, co, (s, s), (1, 1), pad), lut, x, f, *mm, want=("out_exact", "out_ref"))
    xd, fd = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    for kw_, key in (({}, "out_exact"), ({"plan": "none"}, "out_exact"), ({"accumulate": "reference"}, "out_ref")):
        y = ax.approx_conv2d_with_min_max_vars(xd, fd, *mm, [1, s, s, 1], 8, t, pad, **kw_)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref[key].view(np.uint32)), (n, h, w, c, kh, kw, co, kw_)
dw = [(2, 14, 14, 32, 3, 1, 1), (2, 28, 28, 144, 3, 1, 1), (2, 57, 55, 96, 3, 2, 1), (1, 45, 47, 33, 3, 1, 1), (1, 80, 40, 7, 3, 2, 3),
      (1, 12, 12, 16, 5, 1, 1)]
for n, h, w, c, k, s, mult in dw:
    x = rng.uniform(0, 2, (n, h, w, c)).astype(np.float32)
    f = rng.normal(0, 0.3, (k, k, c, mult)).astype(np.float32)
    mm = (0.0, 2.0, float(f.min()), float(f.max()))
    pad = "VALID" if mult == 3 or c == 33 else "SAME"
    ref = O.depthwise_conv2d(O.desc(n, h, w, c, k, k, mult, (s, s), (1, 1), pad), lut, x, f, *mm)
    y = ax.approx_depthwise_conv2d_with_min_max_vars(torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda(), *mm, [1, s, s, 1], 8, t, pad)
    assert np.array_equal(y.cpu().numpy().view(np.uint32), ref["out_ref"].view(np.uint32)), (n, h, w, c, k, s, mult)
torch.cuda.synchronize()
assert L.axc_debug_bounds_record(0, rec) == 0
print("violations", rec[0], "site", rec[1], "value", rec[2] | (rec[3] << 32))
assert rec[0] == 0
"""


def test_checked_flavour_finds_no_violation(built):
    env = dict(os.environ, AXC_LIBRARY_FLAVOUR="check")
    r = subprocess.run([sys.executable, "-c", CHILD % ROOT], env=env, capture_output=True, text=True, timeout=900)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "violations 0" in r.stdout


def test_normal_build_has_no_bounds_record(built):
    import ctypes as C
    from tf_approximate_b200 import _lib
    rec = (C.c_uint32 * 4)()
    assert _lib.load().axc_debug_bounds_record(0, rec) == 12      # Unimplemented
