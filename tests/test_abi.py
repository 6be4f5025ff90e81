"""CPU: the C-ABI library loads, exports every symbol include/axconv.h declares, and its host-side
logic (geometry, status codes, table files, quantisation parameters) behaves like the reference op.
No compute call is made here."""
import ctypes as C
import os
import re

import numpy as np
import pytest

from oracle import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def L(built):
    from tf_approximate_b200 import _lib
    return _lib.load()


def test_exports_every_declared_symbol(L):
    header = open(os.path.join(ROOT, "include", "axconv.h")).read()
    declared = set(re.findall(r"\b(axc_[a-z0-9_]+)\s*\(", header))
    assert len(declared) >= 16
    from tf_approximate_b200 import _lib
    assert declared == set(_lib.SYMBOLS)
    for name in declared:
        assert hasattr(L, name), name


def test_status_strings(L):
    assert L.axc_status_string(0) == b"OK"
    assert L.axc_status_string(3) == b"InvalidArgument"
    assert L.axc_status_string(12) == b"Unimplemented"
    assert L.axc_status_string(13) == b"Internal"
    assert L.axc_status_string(100) == b"CudaError"


def _desc(n, h, w, c, kh, kw, fc, co, s=(1, 1), d=(1, 1), pad=0, fmt=0):
    from tf_approximate_b200 import _lib
    return _lib.ConvDesc(n, h, w, c, kh, kw, fc, co, s[0], s[1], d[0], d[1], pad, fmt)


def test_output_dims_match_tensorflow_window_arithmetic(L):
    rng = np.random.Generator(np.random.PCG64(3))
    out = (C.c_int64 * 4)()
    for _ in range(300):
        kh, kw = int(rng.integers(1, 8)), int(rng.integers(1, 8))
        dh, dw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        pad = int(rng.integers(0, 2))
        h = int(rng.integers((kh - 1) * dh + 1, 70))
        w = int(rng.integers((kw - 1) * dw + 1, 70))
        d = _desc(2, h, w, 3, kh, kw, 3, 5, (sh, sw), (dh, dw), pad)
        assert L.axc_conv2d_output_dims(C.byref(d), out) == 0
        oh, ow, _, _ = O.out_dims(O.desc(2, h, w, 3, kh, kw, 5, (sh, sw), (dh, dw), "SAME" if pad == 0 else "VALID"))
        assert tuple(out) == (2, oh, ow, 5)
        if pad == 0:
            assert (oh, ow) == (-(-h // sh), -(-w // sw))
    d = _desc(4, 10, 10, 6, 3, 3, 6, 2)
    assert L.axc_depthwise_conv2d_output_dims(C.byref(d), out) == 0 and tuple(out) == (4, 10, 10, 12)


def test_error_codes_follow_the_reference_op(L):
    out = (C.c_int64 * 4)()
    # NCHW and EXPLICIT padding: Unimplemented (tf2/src/approx_nn_conv_ops.cpp:160-163, 224-225)
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 4, 4, fmt=1)), out) == 12
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 4, 4, pad=2)), out) == 12
    # grouped convolution: Unimplemented (:229-232); indivisible depth: InvalidArgument (:338-341)
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 2, 4)), out) == 12
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 3, 4)), out) == 3
    # strides / dilations must be positive (:274-303)
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 4, 4, s=(0, 1))), out) == 3
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 8, 8, 4, 3, 3, 4, 4, d=(1, 0))), out) == 3
    # VALID window larger than the image: negative output size
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 2, 2, 4, 5, 5, 4, 4, pad=1)), out) == 3
    # patch larger than the reference's 4 Mi-element chunk (:120-121)
    assert L.axc_conv2d_output_dims(C.byref(_desc(1, 3000, 3000, 1, 2100, 2100, 1, 1)), out) == 3
    assert L.axc_conv2d_output_dims(None, out) == 3
    # forward with an empty output returns OK before touching any device (:449-450)
    t = C.c_void_p()
    assert L.axc_table_create_exact(C.byref(t)) == 0
    assert L.axc_conv2d_forward(t, C.byref(_desc(0, 8, 8, 4, 3, 3, 4, 4)), None, None, 0.0, 1.0, 0.0, 1.0, None,
                                None, 0, None, 0, None) == 0
    # missing workspace: Internal
    assert L.axc_conv2d_forward(t, C.byref(_desc(1, 8, 8, 4, 3, 3, 4, 4)), 256, 256, 0.0, 1.0, 0.0, 1.0, 256,
                                None, 0, None, 0, None) == 13
    L.axc_table_destroy(t)


def test_workspace_size(L):
    sz = C.c_size_t()
    assert L.axc_conv2d_workspace_bytes(C.byref(_desc(1, 8, 8, 16, 3, 3, 16, 32)), C.byref(sz)) == 0
    assert sz.value >= (144 // 4) * 32 * 16 + 32 * 4 and sz.value % 256 == 0
    assert L.axc_depthwise_conv2d_workspace_bytes(C.byref(_desc(1, 8, 8, 16, 3, 3, 16, 1)), C.byref(sz)) == 0
    assert sz.value >= 9 * 16 * 4 + 16 * 4


def test_table_files(L, tmp_path):
    import tf_approximate_b200 as ax
    lut = ax.noisy_table(5)
    p = str(tmp_path / "t.bin")
    ax.write_table(p, lut)
    t = ax.Table(p, 8)
    assert np.array_equal(t.numpy(), lut)
    assert np.array_equal(ax.read_table(p), lut)
    assert np.array_equal(ax.Table("", 8).numpy(), ax.exact_table())
    (tmp_path / "short.bin").write_bytes(b"\1" * 4096)
    with pytest.raises(ax.InvalidArgumentError):
        ax.Table(str(tmp_path / "short.bin"), 8)
    with pytest.raises(ax.InvalidArgumentError):
        ax.Table(str(tmp_path / "nope.bin"), 8)
    with pytest.raises(ax.InvalidArgumentError):
        ax.Table("", 4)  # only 8-bit tables exist (tf2/src/approx_ops_types.h:110-117)


def test_quant_props_equal_checker_bits(L):
    rng = np.random.Generator(np.random.PCG64(4))
    out = (C.c_float * 3)()
    ranges = [(-1.0, 1.0), (0.0, 0.0), (0.0, 6.0), (1.0, 2.0), (-2.0, -1.0), (-0.4, 0.37)]
    ranges += [tuple(float(v) for v in np.sort(rng.normal(0, 3, 2))) for _ in range(200)]
    for mn, mx in ranges:
        assert L.axc_quant_props(mn, mx, out) == 0
        q = O.quant_props(mn, mx, 0.0, 1.0).input
        mine = np.array(list(out), np.float32)
        want = np.array([q.scale, q.inv_scale, q.offset], np.float32)
        assert np.array_equal(mine.view(np.uint32), want.view(np.uint32)), (mn, mx)


def test_python_mirror_argument_checks(built):
    import torch
    import tf_approximate_b200 as ax
    assert ax.conv2d_output_shape((8, 32, 32, 16), (3, 3, 16, 32), (1, 1, 1, 1), "SAME") == (8, 32, 32, 32)
    assert ax.conv2d_output_shape((256, 224, 224, 3), (7, 7, 3, 64), (1, 2, 2, 1), "SAME") == (256, 112, 112, 64)
    with pytest.raises(ax.InvalidArgumentError):
        ax.conv2d_output_shape((8, 32, 32, 16), (3, 3, 16, 32), (1, 1, 1), "SAME")
    with pytest.raises(ax.InvalidArgumentError):
        ax.conv2d_output_shape((8, 32, 32, 16), (3, 3, 16, 32), (2, 1, 1, 1), "SAME")
    with pytest.raises(ax.UnimplementedError):
        ax.conv2d_output_shape((8, 16, 32, 32), (3, 3, 16, 32), (1, 1, 1, 1), "SAME", data_format="NCHW")
    with pytest.raises(ax.InvalidArgumentError):  # CPU tensors: this build has no CPU kernel
        ax.approx_conv2d_with_min_max_vars(torch.zeros(1, 4, 4, 4), torch.zeros(1, 1, 4, 4), 0., 1., 0., 1.,
                                           [1, 1, 1, 1], 8, "", "SAME")


def test_fake_quant_matches_op_quantiser(built):
    """Snapping to the grid and then quantising in the op must return the same level."""
    import torch
    import tf_approximate_b200 as ax
    rng = np.random.Generator(np.random.PCG64(6))
    x = rng.uniform(-1.3, 1.2, 5000).astype(np.float32)
    mn, mx = -1.0, 0.9
    xq = ax.fake_quant_with_min_max_vars(torch.from_numpy(x), mn, mx).numpy()
    q = O.quant_props(mn, mx, 0.0, 1.0).input
    lv = np.array([O.lib().axo_quantize(float(v), q.offset, q.inv_scale) for v in xq])
    raw = np.array([O.lib().axo_quantize(float(np.clip(v, q.offset, q.offset + 255 * q.scale)), q.offset, q.inv_scale)
                    for v in x])
    assert np.array_equal(lv, raw)
    assert np.abs(xq - (lv * np.float32(q.scale) + np.float32(q.offset))).max() < 1e-6
