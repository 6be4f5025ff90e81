"""CPU: the TensorFlow op-kernel shim (tf-approximate_b200/tf_op/approx_conv2d_axconv.cc) is real source, not prose:
it compiles against include/axconv.h and a declaration-only stand-in for the TensorFlow op-kernel API
(tests/tf_api_stub/, written for this repository; TensorFlow itself is not installed here).  What this proves: every
call the shim makes into the C ABI type-checks against the header, and the TensorFlow-side calls have the shapes
TensorFlow 2.x declares.  What it does not prove: behaviour inside a TensorFlow runtime."""
import os
import shutil
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shim_compiles_against_the_header():
    gxx = shutil.which("g++")
    cuda_inc = "/usr/local/cuda/include"
    if gxx is None or not os.path.exists(os.path.join(cuda_inc, "cuda_runtime_api.h")):
        pytest.skip("needs g++ and the CUDA runtime headers")
    src = os.path.join(ROOT, "tf-approximate_b200", "tf_op", "approx_conv2d_axconv.cc")
    cmd = [gxx, "-std=c++14", "-Wall", "-Wextra", "-Werror", "-c", "-o", os.devnull,
           "-I" + os.path.join(ROOT, "tests", "tf_api_stub"), "-I" + os.path.join(ROOT, "include"), "-I" + cuda_inc, src]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr


def test_shim_keeps_the_reference_registration():
    """Same op name, device, type constraint and host-memory pins as the reference's kernel builder
    (tf2/src/approx_nn_conv_ops.cpp:686-699)."""
    text = open(os.path.join(ROOT, "tf-approximate_b200", "tf_op", "approx_conv2d_axconv.cc")).read()
    for needle in ('Name("ApproxConv2DWithMinMaxVars")', ".Device(DEVICE_GPU)", '.TypeConstraint<float>("T")',
                   '.HostMemory("input_min")', '.HostMemory("input_max")', '.HostMemory("filter_min")',
                   '.HostMemory("filter_max")'):
        assert needle in text, needle
