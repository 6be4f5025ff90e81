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


# ---------------------------------------------------------------------------------------------------
# First-generation op (tf1/axqconv): the op's own Compute(), compiled from the reference checkout.
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def axq(built):
    if not O.axq_ref_available():
        pytest.skip("oracle/_ref/libaxq_ref.so not built (no reference checkout)")
    return True


AXQ_MULTIPLIERS = ["mul8u_1JFF", "mul8u_L40", "mul8u_2AC", "mul8u_125K", "mul8u_YX7", "mul8u_QKX"]


def test_weight_tuning_bitwise(axq):
    import os
    names = sorted(n[:-2] for n in os.listdir(os.path.join(O.reference_root(), "tf1", "axqconv", "axmult")) if n.endswith(".c")) \
        if os.path.isdir(os.path.join(O.reference_root(), "tf1", "axqconv", "axmult")) else AXQ_MULTIPLIERS
    changed = 0
    for name in names:
        plain = O.axq_ref_table(name, False)
        assert plain.min() >= 0 and plain.max() <= 65535, name
        tuned = O.axq_ref_table(name, True)
        mine = O.tune_table(plain.astype(np.uint16))
        assert np.array_equal(mine.astype(np.int32), tuned), name
        changed += int(not np.array_equal(plain, tuned))
    assert changed > 0                       # the tuning does something for the approximate multipliers
    exact = O.axq_ref_table("mul8u_1JFF", False).reshape(256, 256)
    assert np.array_equal(exact, np.outer(np.arange(256), np.arange(256)))


def test_quantised_op_bitwise(axq):
    """Random shapes, strides, paddings and ranges - among them ranges that do not contain 0, whose zero points
    lie outside 0..255 and wrap when the functor stores them as a padded tap."""
    rng = np.random.Generator(np.random.PCG64(4))
    tables = {}
    done = outside = 0
    for it in range(150):
        n, h, w = int(rng.integers(1, 3)), int(rng.integers(3, 12)), int(rng.integers(3, 12))
        c, co = int(rng.integers(1, 9)), int(rng.integers(1, 9))
        kh, kw = int(rng.integers(1, 5)), int(rng.integers(1, 5))
        stride = int(rng.integers(1, 4))
        pad = "SAME" if rng.integers(0, 2) else "VALID"
        if pad == "VALID" and (h < kh or w < kw):
            continue
        name = AXQ_MULTIPLIERS[it % len(AXQ_MULTIPLIERS)]
        tune = bool((it // len(AXQ_MULTIPLIERS)) % 2)
        if (name, tune) not in tables:
            plain = O.axq_ref_table(name, False).astype(np.uint16)
            tables[(name, tune)] = O.tune_table(plain) if tune else plain
        qin = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
        qf = rng.integers(0, 256, (kh, kw, c, co), dtype=np.uint8)
        if it % 3 == 0:                      # ranges around 0: zero points inside 0..255
            mm = (-float(np.float32(rng.uniform(0.1, 3))), float(np.float32(rng.uniform(0.1, 3))),
                  -float(np.float32(rng.uniform(0.05, 1))), float(np.float32(rng.uniform(0.05, 1))))
        else:
            a = np.sort(rng.normal(0, 2, 2)).astype(np.float32)
            b = np.sort(rng.normal(0, 0.5, 2)).astype(np.float32)
            mm = (float(a[0]), float(a[1]), float(b[0]), float(b[1]))
        want, lo, hi = O.axq_ref_conv2d(name, tune, qin, qf, *mm, stride, pad)
        zi, zf = O.quantized_zero_point(mm[0], mm[1]), O.quantized_zero_point(mm[2], mm[3])
        if max(abs(zi), abs(zf)) > 20000:    # int32 overflow in the functor's zero-point terms: undefined there
            continue
        d = O.desc(n, h, w, c, kh, kw, co, (stride, stride), (1, 1), pad)
        got = O.qconv2d(d, tables[(name, tune)], qin, qf, zi, zf)
        assert np.array_equal(got, want), (it, name, tune, mm, zi, zf, (n, h, w, c, kh, kw, co, stride, pad))
        assert (lo, hi) == O.quantized_output_range(*mm), (it, mm)
        done += 1
        outside += int(not (0 <= zi <= 255 and 0 <= zf <= 255))
    assert done > 100 and outside > 20
