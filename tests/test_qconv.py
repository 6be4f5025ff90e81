"""The quantised entry point (uint8 operands in, int32 sums out) - the contract of the reference's first-generation
op AxConv2D (tf1/axqconv/axqconv.cc:66-94, 132-263) - and the table-less op ApproxConv2D
(tf2/src/approx_nn_ops.cpp:24-36).

CPU part: the checker's restatement of the integer functor against the plain integer convolution it must equal
with the exact-product table, and the library's host arithmetic for offsets and output range against the checker's
restatement of tf1/axqconv/quantization_utils.h.  GPU part: the CUDA path through the C ABI against the checker,
bit for bit."""
import ctypes as C

import numpy as np
import pytest

import cases
from oracle import oracle as O


def _int_conv(qin, qf, off_in, off_f, stride, pad):
    """sum (a - off_in) * (b - off_f) with zero contribution outside the image, TensorFlow window placement."""
    import torch
    n, h, w, c = qin.shape
    kh, kw, _, co = qf.shape
    d = O.desc(n, h, w, c, kh, kw, co, (stride, stride), (1, 1), pad)
    oh, ow, ph, pw = O.out_dims(d)
    a = torch.from_numpy(qin.astype(np.float64) - off_in).permute(0, 3, 1, 2)
    b = torch.from_numpy(qf.astype(np.float64) - off_f).permute(3, 2, 0, 1)
    need_h = max((oh - 1) * stride + kh - h, 0)
    need_w = max((ow - 1) * stride + kw - w, 0)
    a = torch.nn.functional.pad(a, (pw, need_w - pw, ph, need_h - ph))
    return torch.nn.functional.conv2d(a, b, stride=stride).permute(0, 2, 3, 1).numpy().astype(np.int64)


QSHAPES = [
    # n, h, w, c, kh, kw, cout, stride, padding, (min_in, max_in), (min_f, max_f)
    (2, 9, 11, 5, 3, 3, 7, 1, "SAME", (-1.0, 1.0), (-0.4, 0.6)),
    (1, 12, 12, 16, 3, 3, 40, 2, "SAME", (0.0, 6.0), (-0.5, 0.5)),      # input offset 0
    (2, 8, 8, 64, 1, 1, 96, 1, "VALID", (-2.0, 2.0), (-1.0, 1.0)),
    (1, 14, 14, 8, 5, 5, 33, 1, "VALID", (-1.0, 3.0), (-0.3, 0.1)),
    (1, 21, 19, 3, 7, 7, 64, 2, "SAME", (-1.0, 1.0), (-0.2, 0.2)),
    # ranges that do not contain 0: zero points outside 0..255; a padded tap then reads offset mod 256
    (1, 10, 12, 6, 3, 3, 24, 1, "SAME", (0.5, 2.0), (-0.3, 0.1)),
    (2, 9, 9, 10, 3, 3, 17, 2, "SAME", (-3.0, -1.0), (0.2, 0.9)),
]


def _operands(shape, seed):
    n, h, w, c, kh, kw, co = shape[:7]
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.integers(0, 256, (n, h, w, c), dtype=np.uint8), rng.integers(0, 256, (kh, kw, c, co), dtype=np.uint8)


@pytest.mark.parametrize("shape", QSHAPES, ids=["-".join(str(v) for v in s[:9]) for s in QSHAPES])
def test_checker_functor_equals_integer_convolution_with_exact_table(built, shape):
    n, h, w, c, kh, kw, co, stride, pad, rin, rf = shape
    qin, qf = _operands(shape, 5)
    off_in, off_f = O.quantized_zero_point(*rin), O.quantized_zero_point(*rf)
    if not 0 <= off_in <= 255:
        pytest.skip("a padded tap wraps modulo 256 there: not the plain integer convolution")
    got = O.qconv2d(O.desc(n, h, w, c, kh, kw, co, (stride, stride), (1, 1), pad), O.exact_table(), qin, qf, off_in, off_f)
    assert np.array_equal(got.astype(np.int64), _int_conv(qin, qf, off_in, off_f, stride, pad))


def test_offsets_and_output_range_match_checker(built):
    from tf_approximate_b200 import _lib
    L = _lib.load()
    rng = np.random.Generator(np.random.PCG64(6))
    ranges = [(-1.0, 1.0), (0.0, 6.0), (0.0, 0.0), (-3.5, 0.25), (1e-3, 2e-3)] + \
             [tuple(sorted(rng.normal(0, 3, 2).astype(np.float32).tolist())) for _ in range(200)]
    for lo, hi in ranges:
        o = C.c_int32(-1)
        assert L.axc_quantized_zero_point(lo, hi, C.byref(o)) == 0
        assert o.value == O.quantized_zero_point(lo, hi), (lo, hi)
        r = (C.c_float * 2)()
        assert L.axc_quantized_output_range(lo, hi, -0.5, 0.75, r) == 0
        want = O.quantized_output_range(lo, hi, -0.5, 0.75)
        assert np.float32(r[0]).view(np.uint32) == np.float32(want[0]).view(np.uint32)
        assert np.float32(r[1]).view(np.uint32) == np.float32(want[1]).view(np.uint32)


@pytest.mark.gpu
@pytest.mark.parametrize("shape", QSHAPES, ids=["-".join(str(v) for v in s[:9]) for s in QSHAPES])
def test_ax_conv2d_matches_checker(built, shape):
    import torch
    import tf_approximate_b200 as ax
    n, h, w, c, kh, kw, co, stride, pad, rin, rf = shape
    qin, qf = _operands(shape, 7)
    lut = cases.make_table(("noisy", 61))
    off_in, off_f = O.quantized_zero_point(*rin), O.quantized_zero_point(*rf)
    d = O.desc(n, h, w, c, kh, kw, co, (stride, stride), (1, 1), pad)
    for tune in (False, True):
        y, lo, hi = ax.ax_conv2d(torch.from_numpy(qin).cuda(), torch.from_numpy(qf).cuda(), rin[0], rin[1], rf[0], rf[1],
                                 [1, stride, stride, 1], pad, table=ax.Table(array=lut), ax_tune=tune)
        torch.cuda.synchronize()
        want = O.qconv2d(d, O.tune_table(lut) if tune else lut, qin, qf, off_in, off_f)
        assert np.array_equal(y.cpu().numpy(), want), tune
        assert (lo, hi) == O.quantized_output_range(rin[0], rin[1], rf[0], rf[1])


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.AXQ_CASES, ids=[c[0] for c in cases.AXQ_CASES])
def test_ax_conv2d_matches_the_reference_op(built, case):
    """Against outputs of the reference's own AxConv2D (tests/golden/ref_axq.npz, made by tests/golden/make_golden.py
    from the op compiled out of the reference checkout), with the reference's multiplier tables."""
    import os
    import torch
    import tf_approximate_b200 as ax
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(cases.__file__)), "ref_axq.npz"))
    name, ishape, fshape3, stride, pad, mult, tune, rin, rf, seed = case
    qin, qf = cases.make_axq_operands(ishape, fshape3, seed)
    y, lo, hi = ax.ax_conv2d(torch.from_numpy(qin).cuda(), torch.from_numpy(qf).cuda(), rin[0], rin[1], rf[0], rf[1],
                             [1, stride, stride, 1], pad, table=ax.Table(array=gold["table_" + mult]), ax_tune=tune)
    torch.cuda.synchronize()
    assert np.array_equal(y.cpu().numpy(), gold[name + "_out"])
    assert np.array_equal(np.array([lo, hi], np.float32).view(np.uint32), gold[name + "_range"].view(np.uint32))


@pytest.mark.gpu
def test_ax_conv2d_refuses_what_the_reference_refuses(built):
    import torch
    import tf_approximate_b200 as ax
    x = torch.zeros((1, 20, 20, 4), dtype=torch.uint8, device="cuda")
    f = torch.zeros((3, 3, 4, 8), dtype=torch.uint8, device="cuda")
    with pytest.raises(ax.InvalidArgumentError):          # unequal strides (tf1/axqconv/axqconv.cc:309-313)
        ax.ax_conv2d(x, f, -1, 1, -1, 1, [1, 1, 2, 1], "SAME")
    with pytest.raises(ax.InvalidArgumentError):          # dilation (:320-323)
        ax.ax_conv2d(x, f, -1, 1, -1, 1, [1, 1, 1, 1], "SAME", dilations=[1, 2, 2, 1])
    x21 = torch.zeros((1, 21, 21, 4), dtype=torch.uint8, device="cuda")
    with pytest.raises(ax.InvalidArgumentError):          # a range far from 0: the functor's int32 total would overflow
        ax.ax_conv2d(x, f, 1000.0, 1000.5, -1, 1, [1, 1, 1, 1], "SAME")
    with pytest.raises(ax.UnimplementedError):            # stride 8 over a 3x3 window on 21 pixels: the functor would start
        ax.ax_conv2d(x21, f, -1, 1, -1, 1, [1, 8, 8, 1], "SAME")   # the window at +1 (:153-163), TensorFlow's padding rule at 0


@pytest.mark.gpu
def test_table_less_op_is_the_exact_product_table_with_data_ranges(built):
    import torch
    import tf_approximate_b200 as ax
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.rand((2, 16, 16, 24), device="cuda", generator=g) * 3 - 1
    f = torch.randn((3, 3, 24, 40), device="cuda", generator=g) * 0.2
    y = ax.approx_conv2d(x, f, [1, 1, 1, 1], "SAME")
    want = ax.approx_conv2d_with_min_max_vars(x, f, float(x.min()), float(x.max()), float(f.min()), float(f.max()),
                                              [1, 1, 1, 1], 8, "", "SAME")
    assert torch.equal(y.view(torch.int32), want.view(torch.int32))
    # and it is an 8-bit convolution: close to the float convolution, not equal to it
    ref = torch.nn.functional.conv2d(x.permute(0, 3, 1, 2).double(), f.permute(3, 2, 0, 1).double(), padding=1).permute(0, 2, 3, 1)
    err = float((y.double() - ref).abs().max() / ref.abs().max())
    assert 0 < err < 0.05


@pytest.mark.gpu
def test_ax_conv2d_as_cuda_graph(built):
    """After a first call the quantised entry point only enqueues work on the caller's stream: captured once, replayed
    on new codes, same integers."""
    import torch
    import tf_approximate_b200 as ax
    shape = QSHAPES[0]
    n, h, w, c, kh, kw, co, stride, pad, rin, rf = shape
    qin, qf = _operands(shape, 8)
    qin2, _ = _operands(shape, 9)
    table = ax.Table(array=cases.make_table(("noisy", 62)))
    xd, xd2, fd = torch.from_numpy(qin).cuda(), torch.from_numpy(qin2).cuda(), torch.from_numpy(qf).cuda()

    def call(x, out=None):
        return ax.ax_conv2d(x, fd, rin[0], rin[1], rf[0], rf[1], [1, stride, stride, 1], pad, table=table, out=out)[0]
    want, want2 = call(xd), call(xd2)
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    static_x = xd.clone()
    with torch.cuda.stream(side):
        static_y = call(static_x)
    side.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        call(static_x, out=static_y)
    for src, ref in ((xd2, want2), (xd, want)):
        static_x.copy_(src)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static_y, ref)
