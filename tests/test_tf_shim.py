"""The TensorFlow op-kernel shim (tf-approximate_b200/tf_op/approx_conv2d_axconv.cc) is real source, not prose.
TensorFlow itself is not installed here, so the shim is compiled against include/axconv.h and a small stand-in for
the TensorFlow op-kernel API (tests/tf_api_stub/, written for this repository) and driven by a harness that does
what TensorFlow's executor would: look the kernel up by op name, construct it from attributes, call Compute() with
the tensors in device memory and the four ranges in host memory.

CPU part: the shim compiles without warnings, keeps the reference's registration, and its constructor reports the
reference's errors.  GPU part: Compute() reproduces the reference's CPU outputs (tests/golden/ref_dense.npz) and the
Python path bit for bit.  What stays unproved: behaviour inside a real TensorFlow runtime."""
import ctypes as C
import os
import shutil
import subprocess

import numpy as np
import pytest

import cases

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "tf-approximate_b200", "tf_op", "approx_conv2d_axconv.cc")
DW_SHIM = os.path.join(ROOT, "tf-approximate_b200", "tf_op", "approx_depthwise_conv2d_axconv.cc")
DW_OP = b"ApproxDepthwiseConv2DWithMinMaxVars"
CUDA = "/usr/local/cuda"
OP = b"ApproxConv2DWithMinMaxVars"


def _toolchain():
    gxx = shutil.which("g++")
    if gxx is None or not os.path.exists(os.path.join(CUDA, "include", "cuda_runtime_api.h")):
        pytest.skip("needs g++ and the CUDA runtime headers")
    return gxx


@pytest.mark.parametrize("src", [SHIM, DW_SHIM], ids=["dense", "depthwise"])
def test_shim_compiles_against_the_header(src):
    gxx = _toolchain()
    cmd = [gxx, "-std=c++14", "-Wall", "-Wextra", "-Werror", "-c", "-o", os.devnull,
           "-I" + os.path.join(ROOT, "tests", "tf_api_stub"), "-I" + os.path.join(ROOT, "include"), "-I" + CUDA + "/include", src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


@pytest.fixture(scope="module")
def harness(built, tmp_path_factory):
    """The shim + the harness + libaxconv.so as one test-only shared library."""
    gxx = _toolchain()
    libdir = os.path.join(ROOT, "tf-approximate_b200")
    cudart = os.path.join(CUDA, "lib64")
    if not os.path.exists(os.path.join(cudart, "libcudart.so")):
        pytest.skip("needs the CUDA runtime library")
    so = str(tmp_path_factory.mktemp("shim") / "libshimtest.so")
    cmd = [gxx, "-std=c++14", "-Wall", "-Wextra", "-Werror", "-fPIC", "-shared", "-o", so,
           "-I" + os.path.join(ROOT, "tests", "tf_api_stub"), "-I" + os.path.join(ROOT, "include"), "-I" + CUDA + "/include",
           SHIM, DW_SHIM, os.path.join(ROOT, "tests", "tf_api_stub", "shim_harness.cc"),
           "-L" + libdir, "-laxconv", "-L" + cudart, "-lcudart", "-Wl,-rpath," + libdir, "-Wl,-rpath," + cudart]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    L = C.CDLL(so)
    L.shimtest_create.restype = C.c_void_p
    L.shimtest_create.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_char_p,
                                  C.c_char_p, C.POINTER(C.c_int), C.c_char_p, C.c_int]
    L.shimtest_destroy.argtypes = [C.c_void_p]
    L.shimtest_compute.argtypes = [C.c_void_p, C.c_void_p, C.POINTER(C.c_longlong), C.c_void_p, C.POINTER(C.c_longlong),
                                   C.POINTER(C.c_float), C.c_void_p, C.POINTER(C.c_longlong), C.c_void_p, C.c_char_p, C.c_int]
    return L


def _create(L, table_file, strides=(1, 1, 1, 1), dilations=(1, 1, 1, 1), padding=b"SAME", data_format=b"NHWC", num_bits=8,
            op_name=OP):
    code, msg = C.c_int(-1), C.create_string_buffer(256)
    op = L.shimtest_create(op_name, table_file, num_bits, (C.c_int * 4)(*strides), (C.c_int * 4)(*dilations), padding,
                           data_format, C.byref(code), msg, 256)
    return op, code.value, msg.value.decode()


def test_shim_keeps_the_reference_registration(harness):
    """Same op name, device and host-memory pins as the reference's kernel builder
    (tf2/src/approx_nn_conv_ops.cpp:686-699); the type constraint is checked in the source."""
    dev, hm = C.create_string_buffer(32), C.create_string_buffer(256)
    assert harness.shimtest_registration(OP, dev, 32, hm, 256) == 1
    assert dev.value == b"GPU"
    assert hm.value == b"input_min,input_max,filter_min,filter_max"
    assert '.TypeConstraint<float>("T")' in open(SHIM).read()
    # the depthwise op (no counterpart in the reference) is registered the same way under its own name
    assert harness.shimtest_registration(DW_OP, dev, 32, hm, 256) == 1
    assert dev.value == b"GPU" and hm.value == b"input_min,input_max,filter_min,filter_max"


def test_shim_constructor_reports_the_reference_errors(harness, tmp_path):
    op, code, msg = _create(harness, str(tmp_path / "missing.bin").encode())
    assert op is None and code == 3 and msg == "ApproxTF: Couldn't read the lookup table!"    # approx_ops_types.h:213
    op, code, msg = _create(harness, b"", strides=(2, 1, 1, 1))
    assert op is None and code == 3 and "strides in the batch and depth dimensions" in msg     # approx_nn_conv_ops.cpp:286-291
    op, code, msg = _create(harness, b"", data_format=b"NCHW_VECT_C")
    assert op is None and code == 3 and msg == "Invalid data format"                            # :262-263
    op, code, msg = _create(harness, b"", num_bits=4)
    assert op is None and code == 3
    op, code, msg = _create(harness, b"")
    assert op is not None and code == 0
    harness.shimtest_destroy(op)


def _compute(L, op, x, f, mm, oshape):
    import torch
    out = torch.full(oshape, float("nan"), dtype=torch.float32, device=x.device)
    dims, msg = (C.c_longlong * 4)(), C.create_string_buffer(256)
    code = L.shimtest_compute(op, x.data_ptr(), (C.c_longlong * 4)(*x.shape), f.data_ptr(), (C.c_longlong * 4)(*f.shape),
                              (C.c_float * 4)(*mm), out.data_ptr(), dims, C.c_void_p(torch.cuda.current_stream().cuda_stream),
                              msg, 256)
    torch.cuda.synchronize()
    return code, msg.value.decode(), tuple(dims), out


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.DENSE_CASES[:8], ids=[c[0] for c in cases.DENSE_CASES[:8]])
def test_shim_compute_reproduces_the_reference(harness, tmp_path, case):
    import torch
    import tf_approximate_b200 as ax
    name, ishape, (kh, kw, cout), stride, dil, pad, tspec, in_range, seed = case
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(cases.__file__)), "ref_dense.npz"))[name]
    lut = cases.make_table(tspec)
    path = str(tmp_path / "table.bin")
    ax.write_table(path, lut)
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], cout), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    xd, fd = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    op, code, msg = _create(harness, path.encode(), strides=(1, stride[0], stride[1], 1), dilations=(1, dil[0], dil[1], 1),
                            padding=pad.encode())
    assert op is not None, (code, msg)
    try:
        for _ in range(2):                                  # the second call finds the lookup plan in the op's workspace
            code, msg, dims, out = _compute(harness, op, xd, fd, mm, gold.shape)
            assert code == 0, msg
            assert dims == gold.shape
            want = ax.approx_conv2d_with_min_max_vars(xd, fd, *mm, [1, stride[0], stride[1], 1], 8, path, pad,
                                                      dilations=[1, dil[0], dil[1], 1])
            assert torch.equal(out.view(torch.int32), want.view(torch.int32))
            err = float(np.abs(out.cpu().numpy() - gold).max() / np.abs(gold).max())
            assert err < 1e-5, err                          # the reference's own metric (test_table_approx_conv_2d.py:62)
    finally:
        harness.shimtest_destroy(op)


@pytest.mark.gpu
@pytest.mark.parametrize("case", cases.DEPTHWISE_CASES, ids=[c[0] for c in cases.DEPTHWISE_CASES])
def test_depthwise_shim_compute_matches_the_checker(harness, tmp_path, case):
    import torch
    import tf_approximate_b200 as ax
    name, ishape, (kh, kw, mult), stride, dil, pad, tspec, in_range, seed = case
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(cases.__file__)), "oracle_aux.npz"))[name + "_out_exact"]
    path = str(tmp_path / "table.bin")
    ax.write_table(path, cases.make_table(tspec))
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], mult), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    xd, fd = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    op, code, msg = _create(harness, path.encode(), strides=(1, stride[0], stride[1], 1), dilations=(1, dil[0], dil[1], 1),
                            padding=pad.encode(), op_name=DW_OP)
    assert op is not None, (code, msg)
    try:
        code, msg, dims, out = _compute(harness, op, xd, fd, mm, gold.shape)
        assert code == 0, msg
        assert dims == gold.shape
        assert np.array_equal(out.cpu().numpy().view(np.uint32), gold.view(np.uint32))
    finally:
        harness.shimtest_destroy(op)


@pytest.mark.gpu
def test_shim_compute_error_paths(harness):
    import torch
    x = torch.zeros((1, 8, 8, 4), device="cuda")
    f = torch.zeros((3, 3, 4, 8), device="cuda")
    op, code, msg = _create(harness, b"", data_format=b"NCHW")
    assert op is not None
    code, msg, _, _ = _compute(harness, op, x, f, (-1.0, 1.0, -1.0, 1.0), (1, 8, 8, 8))
    assert code == 12                                       # Unimplemented, as the reference's CPU kernel (:224-225)
    harness.shimtest_destroy(op)
    op, code, msg = _create(harness, b"")
    f_bad = torch.zeros((3, 3, 5, 8), device="cuda")        # depth mismatch: InvalidArgument (:338-341)
    code, msg, _, _ = _compute(harness, op, x, f_bad, (-1.0, 1.0, -1.0, 1.0), (1, 8, 8, 8))
    assert code == 3
    empty = torch.zeros((0, 8, 8, 4), device="cuda")        # empty output: returns without a launch (:449-450)
    code, msg, dims, _ = _compute(harness, op, empty, f, (-1.0, 1.0, -1.0, 1.0), (0, 8, 8, 8))
    assert code == 0 and dims == (0, 8, 8, 8)
    harness.shimtest_destroy(op)


# ---------------------------------------------------------------------------------------------------
# The first-generation op's shim (tf-approximate_b200/tf_op/axconv2d_axconv.cc), through the stand-in for the
# TensorFlow 1.x API that also carries the reference's own op in the checker (oracle/tf1_stub/).
# ---------------------------------------------------------------------------------------------------
AXQ_SHIM = os.path.join(ROOT, "tf-approximate_b200", "tf_op", "axconv2d_axconv.cc")
REF_DIR = os.path.join(ROOT, "oracle", "_ref")


def _axq_build(tmp, link):
    gxx = _toolchain()
    if not (os.path.exists(os.path.join(REF_DIR, "axmult.h")) and os.path.exists(os.path.join(REF_DIR, "libaxq_ref.so"))):
        pytest.skip("oracle/_ref not built (no reference checkout): the multiplier sources are the reference's")
    so = os.path.join(tmp, "libaxqshim.so")
    cmd = [gxx, "-std=c++14", "-Wall", "-Wextra", "-Werror", "-fPIC"] + (["-shared", "-o", so] if link else ["-c", "-o", os.devnull]) + \
          ["-I" + os.path.join(ROOT, "tf-approximate_b200", "tf_op"), "-I" + os.path.join(ROOT, "oracle", "tf1_stub"), "-I" + REF_DIR,
           "-I" + os.path.join(ROOT, "include"), "-I" + CUDA + "/include", os.path.join(ROOT, "tests", "tf_api_stub", "axq_shim_harness.cc")]
    if link:
        libdir, cudart = os.path.join(ROOT, "tf-approximate_b200"), os.path.join(CUDA, "lib64")
        cmd += ["-L" + libdir, "-laxconv", "-L" + REF_DIR, "-laxq_ref", "-L" + cudart, "-lcudart",
                "-Wl,-rpath," + libdir, "-Wl,-rpath," + REF_DIR, "-Wl,-rpath," + cudart]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr
    return so


def test_first_generation_shim_compiles(built, tmp_path):
    _axq_build(str(tmp_path), link=False)
    text = open(AXQ_SHIM).read()
    for needle in ('Name("AxConv2D")', ".Device(DEVICE_CPU)", '.TypeConstraint<quint8>("Tinput")',
                   '.TypeConstraint<quint8>("Tfilter")', '.TypeConstraint<qint32>("out_type")'):
        assert needle in text, needle                      # the reference's registration, tf1/axqconv/axqconv.cc:453-459


@pytest.mark.gpu
def test_first_generation_shim_reproduces_the_reference_op(built, tmp_path):
    """Same entry point as the one around the reference's own AxConv2D (oracle/ref_axq_driver.cpp), the op replaced by
    the shim: identical int32 outputs and ranges on the golden cases (tests/golden/ref_axq.npz)."""
    so = _axq_build(str(tmp_path), link=True)
    L = C.CDLL(so)
    L.shimq_conv2d.argtypes = [C.c_char_p, C.c_int, C.c_void_p] + [C.c_int] * 4 + [C.c_void_p] + [C.c_int] * 3 + [C.c_float] * 4 + \
                              [C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
    gold = np.load(os.path.join(os.path.dirname(os.path.abspath(cases.__file__)), "ref_axq.npz"))
    for name, ishape, fshape3, stride, pad, mult, tune, rin, rf, seed in cases.AXQ_CASES:
        qin, qf = cases.make_axq_operands(ishape, fshape3, seed)
        want = gold[name + "_out"]
        out = np.full(want.shape, -1, np.int32)
        lo, hi = C.c_float(), C.c_float()
        rc = L.shimq_conv2d(mult.encode(), int(tune), qin.ctypes.data, *ishape, qf.ctypes.data, *fshape3, rin[0], rin[1], rf[0], rf[1],
                            stride, 1 if pad == "SAME" else 0, out.ctypes.data, C.byref(lo), C.byref(hi))
        assert rc == 0, name
        assert np.array_equal(out, want), name
        assert np.array_equal(np.array([lo.value, hi.value], np.float32).view(np.uint32), gold[name + "_range"].view(np.uint32)), name
    # an unknown multiplier is the constructor's InvalidArgument (tf1/axqconv/approximate_selector.h:33-37)
    qin, qf = cases.make_axq_operands((1, 4, 4, 2), (1, 1, 3), 1)
    out = np.zeros((1, 4, 4, 3), np.int32)
    lo, hi = C.c_float(), C.c_float()
    assert L.shimq_conv2d(b"mul8u_none", 0, qin.ctypes.data, 1, 4, 4, 2, qf.ctypes.data, 1, 1, 3, -1.0, 1.0, -1.0, 1.0, 1, 1,
                          out.ctypes.data, C.byref(lo), C.byref(hi)) == 1
