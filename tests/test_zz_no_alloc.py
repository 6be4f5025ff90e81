"""GPU: the depthwise entry point that allocates nothing (scratch in a fixed array inside the library)
against the ordinary depthwise entry point and against the CPU checker, called through the C ABI.

It is for callers that cannot allocate device memory themselves - an op kernel inside a framework whose
allocator owns the whole GPU, or a latency-critical loop that must not hit cudaMalloc's device-wide
synchronisation.  The file name sorts last on purpose, so a run that stops at the first failure has
already executed every other test."""
import ctypes as C

import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def test_noalloc_depthwise_matches_workspace_entry_point(built):
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import _lib
    assert torch.cuda.is_available()
    L = _lib.load()
    dev = torch.device("cuda", 0)
    table = ax.Table(array=ax.noisy_table(3999))      # the same table as `lut` below
    table.ensure_device(0)                       # the only allocation: done by a caller who may allocate

    lut = ax.noisy_table(3999)
    rng = np.random.Generator(np.random.PCG64(4242))
    shapes = [(2, 20, 20, 96, 3, 1), (1, 17, 19, 40, 3, 2)]
    data = []
    for n, h, w, c, k, stride in shapes:
        data.append((rng.uniform(0, 2, (n, h, w, c)).astype(np.float32), rng.normal(0, 0.3, (k, k, c, 1)).astype(np.float32)))
    # the third call repeats the first shape: each call rewrites the part of the shared scratch that it reads,
    # whatever the previous call (another shape) left there
    for call, si in enumerate([0, 1, 0]):
        n, h, w, c, k, stride = shapes[si]
        x = torch.from_numpy(data[si][0]).to(dev)
        f = torch.from_numpy(data[si][1]).to(dev)
        mm = (0.0, 2.0, float(f.min()), float(f.max()))
        d = _lib.ConvDesc(n, h, w, c, k, k, c, 1, stride, stride, 1, 1, 0, 0)
        dims = (C.c_int64 * 4)()
        assert L.axc_depthwise_conv2d_output_dims(C.byref(d), dims) == 0
        want = torch.empty(tuple(dims), dtype=torch.float32, device=dev)
        got = torch.full(tuple(dims), float("nan"), dtype=torch.float32, device=dev)
        wsz = C.c_size_t()
        assert L.axc_depthwise_conv2d_workspace_bytes(C.byref(d), C.byref(wsz)) == 0
        ws = torch.empty(wsz.value, dtype=torch.uint8, device=dev)
        stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
        st = L.axc_depthwise_conv2d_forward(table.handle, C.byref(d), x.data_ptr(), f.data_ptr(), *mm,
                                            want.data_ptr(), ws.data_ptr(), ws.numel(), None, 0, stream)
        assert st == 0
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info(dev)[0]
        st = L.axc_depthwise_conv2d_forward_noalloc(table.handle, C.byref(d), x.data_ptr(), f.data_ptr(), *mm,
                                                    got.data_ptr(), 0, stream)
        assert st == 0, L.axc_status_string(st)
        torch.cuda.synchronize()
        word = C.c_int32(-1)
        assert L.axc_depthwise_conv2d_status(C.byref(d), None, C.byref(word), 0, stream) == 0 and word.value == 0
        if call > 0:   # the first call on a device may load the module that holds the array; later ones must not move the needle
            assert torch.cuda.mem_get_info(dev)[0] == free_before, "the entry point allocated device memory"
        # integer table sums and tap-order fp32 sums: the two entry points agree bit for bit
        assert torch.equal(got.view(torch.int32), want.view(torch.int32)), "call %d differs" % call
        # and both carry the bits of the CPU checker
        ref = O.depthwise_conv2d(O.desc(n, h, w, c, k, k, 1, (stride, stride), (1, 1), "SAME"), lut, data[si][0],
                                 data[si][1], *mm)
        assert np.array_equal(got.cpu().numpy().view(np.uint32), ref["out_ref"].view(np.uint32)), "call %d vs checker" % call

    # a filter beyond the fixed scratch is refused before anything is launched
    big = _lib.ConvDesc(1, 8, 8, 40000, 3, 3, 40000, 1, 1, 1, 1, 1, 0, 0)   # 1.6 MB of scratch
    assert L.axc_depthwise_conv2d_forward_noalloc(table.handle, C.byref(big), 256, 256, 0.0, 1.0, 0.0, 1.0, 256,
                                                  0, None) == 3
    # a table that was never uploaded to the device is refused too (uploading would allocate)
    cold = ax.Table(array=ax.exact_table())
    small = _lib.ConvDesc(1, 8, 8, 8, 3, 3, 8, 1, 1, 1, 1, 1, 0, 0)
    assert L.axc_depthwise_conv2d_forward_noalloc(cold.handle, C.byref(small), 256, 256, 0.0, 1.0, 0.0, 1.0, 256,
                                                  0, None) == 13
