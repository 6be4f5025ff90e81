"""CPU: the C restatement against the reference's own CPU kernels compiled from the reference
checkout (oracle/_ref/libaxc_ref.so, built by oracle/Makefile), on random shapes, bit for bit."""
import numpy as np
import pytest

import cases
from oracle import oracle as O


@pytest.fixture(scope="module")
def ref(built):
    if not O.ref_available():
        pytest.skip("oracle/_ref/libaxc_ref.so not built (no reference checkout)")
    return True


def test_quant_props_bitwise(ref):
    rng = np.random.Generator(np.random.PCG64(1))
    op = O.RefOp("")
    ranges = [(-1.0, 1.0, -0.4, 0.37), (0.0, 6.0, -0.1, 0.1), (0.0, 0.0, -1.0, 1.0), (0.5, 2.0, -3.0, -1.0)]
    ranges += [tuple(float(v) for v in np.sort(rng.normal(0, 2, 2))) + tuple(float(v) for v in np.sort(rng.normal(0, .3, 2)))
               for _ in range(50)]
    for mm in ranges:
        q = O.quant_props(*mm)
        mine = np.array([q.input.scale, q.input.inv_scale, q.input.offset, q.filter.scale, q.filter.inv_scale,
                         q.filter.offset, q.s1s2, q.m1, q.m2, q.m1m2], np.float32)
        assert np.array_equal(mine.view(np.uint32), op.quant(*mm).view(np.uint32)), mm


def test_random_shapes_bitwise(ref, tmp_path):
    import tf_approximate_b200 as ax
    rng = np.random.Generator(np.random.PCG64(2))
    lut = cases.make_table(("noisy", 77))
    path = str(tmp_path / "t.bin")
    ax.write_table(path, lut)
    op = O.RefOp(path)
    for it in range(40):
        n, c, co = int(rng.integers(1, 3)), int(rng.integers(1, 20)), int(rng.integers(1, 20))
        kh, kw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        dh, dw = int(rng.integers(1, 3)), int(rng.integers(1, 3))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        pad = "SAME" if rng.integers(0, 2) else "VALID"
        h = int(rng.integers((kh - 1) * dh + 1, (kh - 1) * dh + 12))
        w = int(rng.integers((kw - 1) * dw + 1, (kw - 1) * dw + 12))
        x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
        mm = (-1.0, 1.0, float(f.min()) - 1e-3, float(f.max()) + 1e-3)
        d = O.desc(n, h, w, c, kh, kw, co, (sh, sw), (dh, dw), pad)
        a = O.conv2d(d, lut, x, f, *mm, want=("out_ref",))["out_ref"]
        b = op.conv2d(d, x, f, *mm)
        assert np.array_equal(a.view(np.uint32), b.view(np.uint32)), (it, n, h, w, c, kh, kw, co, sh, sw, dh, dw, pad)
