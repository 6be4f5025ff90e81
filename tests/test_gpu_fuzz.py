"""GPU: seeded random shapes, strides, dilations, paddings, ranges and call options against the CPU checker, bit for
bit.  The fixed parity tests walk the kernel variants on purpose; this one walks the space between them.
AXC_FUZZ_SCALE=n multiplies the number of cases, AXC_FUZZ_SEED=s offsets the seeds (for a longer hunt by hand)."""
import os

import numpy as np
import pytest

import cases
from oracle import oracle as O

pytestmark = pytest.mark.gpu

SCALE, SEED = int(os.environ.get("AXC_FUZZ_SCALE", "1")), int(os.environ.get("AXC_FUZZ_SEED", "0"))
N_DENSE, N_DEPTHWISE = 70 * SCALE, 40 * SCALE


def _ranges(rng, x, f, loose):
    """Ranges around the data; `loose`: narrower than the data now and then, so that values saturate."""
    lo, hi = float(x.min()), float(x.max())
    if loose and rng.integers(0, 3) == 0:
        lo, hi = lo * 0.7, hi * 0.8
    if rng.integers(0, 4) == 0:
        lo = 0.0 if lo > 0 else lo
    return (np.float32(lo).item(), np.float32(hi).item(), float(f.min()), float(f.max()))


def test_dense_random_cases(built):
    import torch
    import tf_approximate_b200 as ax
    rng = np.random.Generator(np.random.PCG64(7001 + SEED))
    tables = [cases.make_table(("noisy", 71)), cases.make_table(("truncated",)), cases.make_table(("exact",))]
    handles = [ax.Table(array=t) for t in tables]
    for it in range(N_DENSE):
        n = int(rng.integers(1, 4))
        c = int(rng.choice([1, 2, 3, 4, 5, 8, 12, 16, 20, 32, 48, 64, 96]))
        co = int(rng.choice([1, 3, 8, 16, 17, 32, 33, 40, 64, 96, 100, 128, 160, 256, 272]))
        kh, kw = int(rng.integers(1, 6)), int(rng.integers(1, 6))
        dh, dw = (int(rng.integers(1, 3)), int(rng.integers(1, 3))) if rng.integers(0, 4) == 0 else (1, 1)
        sh, sw = int(rng.integers(1, 4)), int(rng.integers(1, 4))
        pad = "SAME" if rng.integers(0, 3) else "VALID"
        h = int(rng.integers((kh - 1) * dh + 1, (kh - 1) * dh + 1 + int(rng.choice([3, 9, 30]))))
        w = int(rng.integers((kw - 1) * dw + 1, (kw - 1) * dw + 1 + int(rng.choice([3, 9, 30]))))
        ti = int(rng.integers(0, 3))
        kind = rng.integers(0, 3)          # input distribution: symmetric, post-ReLU, with negative values to be floored
        x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        if kind == 1:
            x = np.maximum(x, 0)
        f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
        input_relu = bool(kind == 2 and rng.integers(0, 2))
        seen = np.maximum(x, 0) if input_relu else x
        mm = _ranges(rng, seen, f, loose=True)
        d = O.desc(n, h, w, c, kh, kw, co, (sh, sw), (dh, dw), pad)
        ref = O.conv2d(d, tables[ti], seen, f, *mm, want=("out_exact", "out_ref", "acc"))
        opts = {}
        mode = int(rng.integers(0, 4))
        if mode == 1:
            opts["plan"] = "none"
        key = "out_exact"
        if mode == 2:
            opts["accumulate"] = "reference"
            key = "out_ref"
        xd, fd = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
        y, dbg = ax.approx_conv2d_with_min_max_vars(xd, fd, *mm, [1, sh, sw, 1], 8, handles[ti], pad,
                                                    dilations=[1, dh, dw, 1], debug=True, input_relu=input_relu, **opts)
        what = (it, n, h, w, c, kh, kw, co, sh, sw, dh, dw, pad, ti, mode, input_relu)
        if mode != 2:
            assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"]), what
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref[key].view(np.uint32)), what
        if mode == 3:                      # the steps that ride along: bias, shortcut, ReLU
            bias = torch.from_numpy(rng.normal(0, 0.5, co).astype(np.float32)).cuda()
            res = torch.from_numpy(rng.normal(0, 0.5, ref["out_exact"].shape).astype(np.float32)).cuda()
            z = ax.approx_conv2d_with_min_max_vars(xd, fd, *mm, [1, sh, sw, 1], 8, handles[ti], pad, dilations=[1, dh, dw, 1],
                                                   input_relu=input_relu, bias=bias, residual=res, relu=True)
            want = torch.relu((torch.from_numpy(ref["out_exact"]).cuda() + bias) + res)
            assert torch.equal(z.view(torch.int32), want.view(torch.int32)), what


def test_depthwise_random_cases(built):
    import torch
    import tf_approximate_b200 as ax
    rng = np.random.Generator(np.random.PCG64(7002 + SEED))
    lut = cases.make_table(("noisy", 72))
    table = ax.Table(array=lut)
    for it in range(N_DEPTHWISE):
        n = int(rng.integers(1, 4))
        c = int(rng.choice([1, 3, 7, 16, 32, 33, 40, 64, 96, 144, 200]))
        mult = int(rng.choice([1, 1, 1, 2, 3]))
        k = int(rng.choice([3, 3, 3, 1, 2, 5]))
        s = int(rng.integers(1, 3))
        dil = 2 if (k > 1 and rng.integers(0, 6) == 0) else 1
        pad = "SAME" if rng.integers(0, 3) else "VALID"
        big = rng.integers(0, 3) == 0       # large enough for the expanded-table kernels
        span = (k - 1) * dil + 1
        h = int(rng.integers(span, span + (90 if big else 12)))
        w = int(rng.integers(span, span + (90 if big else 12)))
        if big:
            n, h, w = max(n, 2), max(h, 40), max(w, 40)
        x = rng.uniform(0, 2, (n, h, w, c)).astype(np.float32)
        f = rng.normal(0, 0.3, (k, k, c, mult)).astype(np.float32)
        mm = _ranges(rng, x, f, loose=False)
        d = O.desc(n, h, w, c, k, k, mult, (s, s), (dil, dil), pad)
        ref = O.depthwise_conv2d(d, lut, x, f, *mm)
        y, dbg = ax.approx_depthwise_conv2d_with_min_max_vars(torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda(), *mm,
                                                              [1, s, s, 1], 8, table, pad, dilations=[1, dil, dil, 1], debug=True)
        what = (it, n, h, w, c, k, mult, s, dil, pad)
        assert dbg["status"] == 0, what
        assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"]), what
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref["out_exact"].view(np.uint32)), what


def test_quantised_random_cases(built):
    """The uint8-in / int32-out entry point: random shapes, ranges with zero points inside and outside 0..255, weight
    tuning on and off."""
    import torch
    import tf_approximate_b200 as ax
    rng = np.random.Generator(np.random.PCG64(7003 + SEED))
    lut = cases.make_table(("noisy", 73))
    tuned = O.tune_table(lut)
    table = ax.Table(array=lut)
    done = 0
    for it in range(40 * SCALE):
        n, h, w = int(rng.integers(1, 3)), int(rng.integers(3, 20)), int(rng.integers(3, 20))
        c = int(rng.choice([1, 3, 4, 8, 16, 32, 64]))
        co = int(rng.choice([1, 5, 16, 32, 40, 96, 130]))
        k = int(rng.integers(1, 5))
        stride = int(rng.integers(1, 3))
        pad = "SAME" if rng.integers(0, 2) else "VALID"
        if pad == "VALID" and (h < k or w < k):
            continue
        if it % 2:
            a = np.sort(rng.normal(0, 2, 2)).astype(np.float32)
            b = np.sort(rng.normal(0, 0.5, 2)).astype(np.float32)
            rin, rf = (float(a[0]), float(a[1])), (float(b[0]), float(b[1]))
        else:
            rin, rf = (-float(np.float32(rng.uniform(0.1, 3))), float(np.float32(rng.uniform(0.1, 3)))), (-0.5, 0.25)
        zi, zf = O.quantized_zero_point(*rin), O.quantized_zero_point(*rf)
        if max(abs(zi), abs(zf), 255) ** 2 * k * k * c > 2 ** 31 - 1:
            continue                        # the functor's int32 total could overflow: refused by the library
        tune = bool(rng.integers(0, 2))
        qin = rng.integers(0, 256, (n, h, w, c), dtype=np.uint8)
        qf = rng.integers(0, 256, (k, k, c, co), dtype=np.uint8)
        d = O.desc(n, h, w, c, k, k, co, (stride, stride), (1, 1), pad)
        want = O.qconv2d(d, tuned if tune else lut, qin, qf, zi, zf)
        try:
            y, lo, hi = ax.ax_conv2d(torch.from_numpy(qin).cuda(), torch.from_numpy(qf).cuda(), rin[0], rin[1], rf[0], rf[1],
                                     [1, stride, stride, 1], pad, table=table, ax_tune=tune)
        except ax.UnimplementedError:
            continue                        # window placement differs from the functor's (stride much larger than the window)
        assert np.array_equal(y.cpu().numpy(), want), (it, n, h, w, c, k, co, stride, pad, rin, rf, zi, zf, tune)
        assert (lo, hi) == O.quantized_output_range(rin[0], rin[1], rf[0], rf[1])
        done += 1
    assert done >= 25 * SCALE
