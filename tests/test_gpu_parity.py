"""GPU: the CUDA path, called through the C ABI (ctypes -> libaxconv.so), against the CPU checker.

Bars: quantised uint8 operands and int32 accumulators bit for bit.  The fp32 output is compared
 - default mode (exact integer sum): bit for bit with the checker's epilogue applied to the exact sum (the
   kernels add the patch and filter sums in the reference's order and round every operation separately),
   hence bit for bit with the reference whenever its fp32 running total is exact (always for K <= 256);
 - accumulate="reference" (fp32 running total in K order): bit for bit with the reference-order result for
   every K, including the shapes on which the reference itself rounds (partial sums beyond 2^24);
 - on the benchmark configurations' shapes the default mode is additionally held to the stated tolerance
   1e-5 against the reference-order result, in the reference's metric max|out - ref| / max|ref|
   (tf2/test/test_table_approx_conv_2d.py:62)."""
import numpy as np
import pytest

import cases
from oracle import oracle as O

pytestmark = pytest.mark.gpu

TOL_REF = 1e-5     # vs. the reference-order fp32 arithmetic (north-star tolerance)


@pytest.fixture(scope="module")
def ax(built):
    import torch
    assert torch.cuda.is_available()
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import _lib
    _lib.load()  # raises when the CUDA library is missing: there is no fallback
    return ax


def linf(a, ref):
    m = np.abs(ref).max()
    return float(np.abs(a - ref).max() / (m if m > 0 else 1.0))


def run_dense(ax, lut, x, f, mm, stride, dil, pad, accumulate="exact"):
    import torch
    t = ax.Table(array=lut)
    y, dbg = ax.approx_conv2d_with_min_max_vars(torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda(), *mm,
                                                strides=[1, stride[0], stride[1], 1], num_bits=8, mul_map_file=t,
                                                padding=pad, dilations=[1, dil[0], dil[1], 1], debug=True,
                                                accumulate=accumulate)
    torch.cuda.synchronize()
    assert dbg["plan"]["status"] == 0
    return y.cpu().numpy(), {k: (v if k == "plan" else v.cpu().numpy()) for k, v in dbg.items()}


def rounding_share(ref):
    """Share of outputs on which the reference's fp32 running total differs from the exact sum, and the
    distance between the two results in the reference's metric."""
    return float((ref["out_ref"] != ref["out_exact"]).mean()), linf(ref["out_exact"], ref["out_ref"])


def check_dense(ax, lut, x, f, mm, stride=(1, 1), dil=(1, 1), pad="SAME"):
    n, h, w, c = x.shape
    kh, kw, _, co = f.shape
    d = O.desc(n, h, w, c, kh, kw, co, stride, dil, pad)
    ref = O.conv2d(d, lut, x, f, *mm, want=("out_ref", "out_exact", "acc", "qinput", "qfilter"))
    y, dbg = run_dense(ax, lut, x, f, mm, stride, dil, pad)
    assert y.shape == ref["out_exact"].shape
    assert np.array_equal(dbg["qinput"], ref["qinput"])
    assert np.array_equal(dbg["qfilter"], ref["qfilter"])
    assert np.array_equal(dbg["acc"], ref["acc"])
    assert np.array_equal(y.view(np.uint32), ref["out_exact"].view(np.uint32))
    if kh * kw * c <= 256:
        assert np.array_equal(y.view(np.uint32), ref["out_ref"].view(np.uint32))
        assert linf(y, ref["out_ref"]) < TOL_REF
    # the reference's own arithmetic (fp32 running total in K order): its bits, whatever K
    y_ro, dbg_ro = run_dense(ax, lut, x, f, mm, stride, dil, pad, accumulate="reference")
    assert np.array_equal(y_ro.view(np.uint32), ref["out_ref"].view(np.uint32))
    assert np.array_equal(dbg_ro["qinput"], ref["qinput"]) and np.array_equal(dbg_ro["qfilter"], ref["qfilter"])
    return y, ref


@pytest.mark.parametrize("case", cases.DENSE_CASES, ids=[c[0] for c in cases.DENSE_CASES])
def test_golden_dense(ax, golden, case):
    name, ishape, (kh, kw, cout), stride, dil, pad, tspec, in_range, seed = case
    lut = cases.make_table(tspec)
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], cout), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    y, dbg = run_dense(ax, lut, x, f, mm, stride, dil, pad)
    assert np.array_equal(dbg["acc"], golden["aux"][name + "_acc"])
    assert np.array_equal(dbg["qinput"], golden["aux"][name + "_qinput"])
    assert np.array_equal(dbg["qfilter"], golden["aux"][name + "_qfilter"])
    exact = golden["aux"][name + "_out_exact"]
    assert np.array_equal(y.view(np.uint32), exact.view(np.uint32))
    want = golden["ref"][name]   # output of the reference's own CPU kernels
    y_ro, _ = run_dense(ax, lut, x, f, mm, stride, dil, pad, accumulate="reference")
    assert np.array_equal(y_ro.view(np.uint32), want.view(np.uint32))        # reference order: its bits, every K
    if name in cases.ROUNDING_CASES:
        # the reference's fp32 running total rounds here (partial sums pass 2^24): the default mode keeps the
        # exact sum and therefore differs from the reference by the reference's own rounding
        assert (want != exact).mean() > 0.5 and 1e-5 < linf(y, want) < 1e-3
    else:
        assert np.array_equal(y.view(np.uint32), want.view(np.uint32))
        assert linf(y, want) < TOL_REF


def test_reference_recipe(ax, golden):
    """tf2/test/test_table_approx_conv_2d.py: exact table, fake-quantised [0,1] operands, SAME, 8x8 window."""
    xq, fq = cases.recipe_inputs()
    y, _ = run_dense(ax, ax.exact_table(), xq, fq, (0.0, 1.0, 0.0, 1.0), (1, 1), (1, 1), "SAME")
    assert np.array_equal(y.view(np.uint32), golden["ref"]["recipe"].view(np.uint32))
    assert linf(y, golden["ref"]["recipe"]) < TOL_REF


def test_config1_full(ax):
    """N=8, 32x32x16 -> 32, 3x3 SAME, exact table, input [-1,1], filter range from the data."""
    rng = np.random.Generator(np.random.PCG64(1001))
    x = rng.uniform(-1, 1, (8, 32, 32, 16)).astype(np.float32)
    f = np.random.Generator(np.random.PCG64(2100)).normal(0, 0.1, (3, 3, 16, 32)).astype(np.float32)
    check_dense(ax, ax.exact_table(), x, f, (-1.0, 1.0, float(f.min()), float(f.max())))


SHAPES = [
    # n, h, w, c, kh, kw, cout, stride, dil, pad
    (2, 9, 11, 5, 3, 3, 7, (1, 1), (1, 1), "SAME"),       # C % 4 != 0, Cout < 32
    (1, 17, 13, 8, 3, 3, 40, (1, 1), (1, 1), "SAME"),     # Cout tail in the second warp column
    (1, 10, 10, 12, 3, 3, 70, (2, 2), (1, 1), "SAME"),    # two channel tiles, tail in the second
    (2, 12, 10, 4, 3, 2, 6, (2, 1), (2, 1), "VALID"),     # dilation + anisotropic stride
    (3, 8, 8, 16, 1, 1, 32, (1, 1), (1, 1), "SAME"),      # 1x1 fused form
    (2, 8, 8, 64, 1, 1, 256, (1, 1), (1, 1), "VALID"),    # bottleneck expand
    (2, 9, 9, 256, 1, 1, 64, (2, 2), (1, 1), "SAME"),     # strided projection
    (3, 6, 5, 4, 6, 5, 9, (1, 1), (1, 1), "VALID"),       # filter == image
    (1, 21, 19, 3, 7, 7, 64, (2, 2), (1, 1), "SAME"),     # stem: K = 147, scalar loader
    (1, 5, 5, 1, 3, 3, 1, (1, 1), (1, 1), "SAME"),        # smallest
    (1, 4, 4, 512, 3, 3, 33, (1, 1), (1, 1), "SAME"),     # K = 4608, many chunks
    (5, 7, 7, 20, 3, 3, 64, (1, 1), (1, 1), "SAME"),      # K = 180: chunk tail, pixel tail
    (1, 30, 30, 2, 5, 5, 3, (3, 3), (1, 1), "VALID"),
    (1, 9, 9, 6, 2, 2, 5, (1, 1), (3, 3), "SAME"),
    # more tile groups than SMs: several rounds per CTA, main launch + tail launch with smaller tile groups
    (2, 112, 112, 8, 3, 3, 32, (1, 1), (1, 1), "SAME"),
    (4, 100, 100, 4, 3, 3, 12, (1, 1), (1, 1), "SAME"),   # at most 16 channels: two pixel tiles per warp
    (1, 120, 120, 16, 1, 1, 96, (1, 1), (1, 1), "SAME"),  # three channel groups in a launch of four
    (1, 150, 150, 8, 3, 3, 33, (1, 1), (1, 1), "VALID"),  # runs of 1 + 1 groups, odd channel tail
    # extremes
    (1, 6, 6, 3, 1, 1, 2100, (1, 1), (1, 1), "SAME"),     # 66 channel groups, K = 3
    (2, 5, 5, 1, 1, 1, 1, (1, 1), (1, 1), "SAME"),        # K = 1
    (1, 9, 9, 512, 7, 7, 20, (1, 1), (1, 1), "SAME"),     # K = 25088: 25 chunks
    (1, 20, 20, 4, 3, 3, 17, (4, 4), (1, 1), "SAME"),     # stride larger than the window
    (1, 1, 300, 4, 1, 3, 16, (1, 1), (1, 1), "SAME"),     # one row
    (1, 64, 64, 32, 3, 3, 224, (1, 1), (1, 1), "SAME"),   # 7 channel groups in a launch of 8
    (1, 64, 64, 32, 1, 1, 160, (1, 1), (1, 1), "SAME"),   # 5 groups: 4 + 1
    (1, 64, 64, 32, 1, 1, 192, (2, 2), (1, 1), "SAME"),   # 6 groups: 4 + 2
    (1, 64, 64, 16, 3, 3, 144, (1, 1), (1, 1), "SAME"),   # 4 + 1 groups, the last with 16 channels on two pixel tiles
    (1, 40, 40, 8, 1, 1, 267, (1, 1), (1, 1), "SAME"),    # 8 + 1 groups, the last with 11 channels
    # few pixels, many channels: fewer CTA tiles than SMs, or a last round that is mostly empty
    (2, 7, 7, 512, 3, 3, 512, (1, 1), (1, 1), "SAME"),    # K = 4608 in chunks, 16 groups
    (32, 7, 7, 512, 1, 1, 512, (1, 1), (1, 1), "SAME"),   # K = 512 in one chunk, several tile groups per CTA
    (8, 7, 7, 128, 1, 1, 128, (1, 1), (1, 1), "SAME"),    # a run of 4 groups
    (32, 7, 7, 64, 3, 3, 128, (1, 1), (1, 1), "SAME"),    # a run of 4 groups, several tile groups per CTA
    (4, 7, 7, 256, 1, 1, 224, (1, 1), (1, 1), "SAME"),    # 7 groups in a run of 8
]


@pytest.mark.parametrize("shape", SHAPES, ids=["-".join(str(v) for v in s[:7]) for s in SHAPES])
def test_dense_shapes(ax, shape):
    n, h, w, c, kh, kw, co, stride, dil, pad = shape
    rng = np.random.Generator(np.random.PCG64(hash(shape[:7]) % (1 << 30)))
    x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
    f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
    check_dense(ax, cases.make_table(("noisy", 31)), x, f, (-1.0, 1.0, float(f.min()), float(f.max())), stride, dil, pad)


def test_reference_order_where_the_reference_rounds(ax):
    """K = 4608 and K = 25 088 with a noisy table: almost every output of the reference carries the rounding of
    its fp32 running total (the exact-sum result is 1e-4 .. 1e-2 away in the reference's metric).
    accumulate="reference" reproduces those bits; the default mode reproduces the exact sum."""
    for shape in [(1, 4, 4, 512, 3, 3, 33), (1, 9, 9, 512, 7, 7, 20)]:
        n, h, w, c, kh, kw, co = shape
        rng = np.random.Generator(np.random.PCG64(77 + c * kh))
        x = rng.uniform(0, 2, (n, h, w, c)).astype(np.float32)
        f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
        _, ref = check_dense(ax, cases.make_table(("noisy", 31)), x, f, (0.0, 2.0, float(f.min()), float(f.max())))
        share, dist = rounding_share(ref)
        print("K=%d: %.1f %% of the reference's outputs rounded, exact-sum result %.2e away" % (kh * kw * c, 100 * share, dist))
        assert share > 0.5 and dist > TOL_REF


CONFIG_SHAPES = [
    # the benchmark configurations' layer shapes at their real K, spatial size / batch reduced: (table, shape)
    (("truncated",), (2, 56, 56, 64, 3, 3, 64, 1)),      # config 2a
    (("noisy", 202), (2, 56, 56, 64, 3, 3, 64, 1)),      # config 2b
    (("truncated",), (1, 14, 14, 1024, 1, 1, 256, 1)),   # config 4: K = 1024
    (("truncated",), (1, 7, 7, 2048, 1, 1, 512, 1)),     # K = 2048
    (("truncated",), (1, 14, 14, 256, 3, 3, 256, 1)),    # K = 2304
    (("truncated",), (1, 14, 14, 512, 3, 3, 512, 2)),    # K = 4608, stride 2
    (("noisy", 305), (2, 8, 8, 64, 3, 3, 64, 1)),        # config 3: K = 576
    (("noisy", 500), (2, 14, 14, 384, 1, 1, 384, 1)),    # config 5: K = 384
]


@pytest.mark.parametrize("tspec,shape", CONFIG_SHAPES, ids=["%s-%s" % (t[0], "-".join(str(v) for v in s)) for t, s in CONFIG_SHAPES])
def test_config_shapes_within_tolerance_of_reference_order(ax, tspec, shape):
    """Default (exact-sum) mode against the reference-order result on the configurations' shapes: within 1e-5,
    and the share of outputs on which the reference rounded is reported.  With the truncated table every entry
    is a multiple of 64, so the fp32 running total cannot round below K = 16 512 and accumulate="reference" is
    served by the scheduled kernel too (its plan is present in the workspace afterwards)."""
    import torch
    n, h, w, c, kh, kw, co, s = shape
    rng = np.random.Generator(np.random.PCG64(900 + c + co))
    x = np.maximum(rng.uniform(-1, 1, (n, h, w, c)), 0 if c > 64 else -1).astype(np.float32)   # deeper layers see ReLU outputs
    f = rng.normal(0, np.sqrt(2.0 / (kh * kw * c)), (kh, kw, c, co)).astype(np.float32)
    lut = cases.make_table(tspec)
    mm = (float(x.min()), float(x.max()), float(f.min()), float(f.max()))
    y, ref = check_dense(ax, lut, x, f, mm, (s, s), (1, 1), "SAME")
    share, dist = rounding_share(ref)
    print("K=%d %s: reference rounded on %.2f %% of the outputs, exact-sum result %.2e away" % (kh * kw * c, tspec[0], 100 * share, dist))
    assert linf(y, ref["out_ref"]) < TOL_REF
    if tspec[0] == "truncated":
        assert share == 0.0
        f2 = torch.from_numpy(f).cuda().clone()        # a filter storage of its own: a fresh workspace
        y2, dbg2 = ax.approx_conv2d_with_min_max_vars(torch.from_numpy(x).cuda(), f2, *mm, [1, s, s, 1], 8,
                                                      ax.Table(array=lut), "SAME", debug=True, accumulate="reference")
        assert dbg2["plan"]["steps_per_mille"] >= 1000 and dbg2["plan"]["fallback"] == 0
        assert np.array_equal(y2.cpu().numpy().view(np.uint32), ref["out_ref"].view(np.uint32))


def test_out_of_range_inputs_saturate(ax):
    """Values outside [min,max] clamp to levels 0/255 (the reference's cast is undefined there)."""
    rng = np.random.Generator(np.random.PCG64(12))
    x = rng.uniform(-3, 3, (1, 8, 8, 8)).astype(np.float32)
    f = rng.normal(0, 0.3, (3, 3, 8, 16)).astype(np.float32)
    check_dense(ax, cases.make_table(("noisy", 32)), x, f, (-1.0, 1.0, -0.2, 0.2))


def test_zero_ranges(ax):
    """min == max == 0 gives scale = 1/scale = offset = 0 (tf2/src/approx_ops_types.h:135-152)."""
    rng = np.random.Generator(np.random.PCG64(13))
    x = rng.uniform(-1, 1, (1, 6, 6, 4)).astype(np.float32)
    f = rng.normal(0, 0.1, (3, 3, 4, 8)).astype(np.float32)
    check_dense(ax, cases.make_table(("noisy", 33)), x, f, (0.0, 0.0, float(f.min()), float(f.max())))
    check_dense(ax, cases.make_table(("noisy", 33)), x, f, (-1.0, 1.0, 0.0, 0.0))


def test_plan_reuse_and_fallback(ax):
    """The lookup plan lives in the per-filter workspace: built on the first call, reused while the filter is
    unchanged, rebuilt when a filter value changes; a filter whose weights all fall into one table column cannot
    be scheduled and is served by the common-K kernel - every case with the same bits as the checker."""
    import torch
    rng = np.random.Generator(np.random.PCG64(21))
    lut = cases.make_table(("noisy", 35))
    t = ax.Table(array=lut)
    x = rng.uniform(-1, 1, (2, 10, 10, 16)).astype(np.float32)
    f = rng.normal(0, 0.1, (3, 3, 16, 40)).astype(np.float32)
    xd, fd = torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda()
    mm = (-1.0, 1.0, -0.45, 0.45)
    d = O.desc(2, 10, 10, 16, 3, 3, 40)

    def run():
        y, dbg = ax.approx_conv2d_with_min_max_vars(xd, fd, *mm, [1, 1, 1, 1], 8, t, "SAME", debug=True)
        ref = O.conv2d(d, lut, x, fd.cpu().numpy(), *mm, want=("out_exact", "acc"))
        assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"])
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref["out_exact"].view(np.uint32))
        return dbg["plan"]

    p1 = run()
    assert p1["rebuilt"] == 1 and p1["fallback"] == 0 and 1000 <= p1["steps_per_mille"] < 1500
    p2 = run()
    assert p2["rebuilt"] == 0 and p2["fallback"] == 0
    fd[1, 1, 3, 7] += 0.2                      # same storage, one weight changed
    p3 = run()
    assert p3["rebuilt"] == 1
    fd.fill_(0.1)                              # every weight in one column: no conflict-free schedule
    p4 = run()
    assert p4["rebuilt"] == 1 and p4["fallback"] == 1
    p5 = run()
    assert p5["rebuilt"] == 0 and p5["fallback"] == 1


def test_device_resident_ranges_match_host_ranges(ax):
    """Ranges handed over in device memory: the quantisation parameters are derived on the GPU; the result has
    the bits of the call with the same four values passed from the host, and of the CPU checker."""
    import torch
    rng = np.random.Generator(np.random.PCG64(31))
    lut = cases.make_table(("noisy", 36))
    t = ax.Table(array=lut)
    for mm in [(-1.0, 1.0, -0.37, 0.41), (0.0, 2.5, -0.2, 0.3), (0.0, 0.0, -0.3, 0.3), (0.3, 1.7, -0.9, -0.1)]:
        x = torch.from_numpy(rng.uniform(mm[0], mm[1] if mm[1] > mm[0] else 1.0, (2, 11, 9, 12)).astype(np.float32)).cuda()
        f = torch.from_numpy(rng.uniform(mm[2], mm[3], (3, 3, 12, 20)).astype(np.float32)).cuda()
        y_host, d_host = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", debug=True)
        dev_mm = [torch.tensor(v, dtype=torch.float32, device="cuda") for v in mm]
        y_dev, d_dev = ax.approx_conv2d_with_min_max_vars(x, f, *dev_mm, [1, 1, 1, 1], 8, t, "SAME", debug=True)
        assert torch.equal(d_host["acc"], d_dev["acc"]) and torch.equal(d_host["qinput"], d_dev["qinput"])
        assert torch.equal(y_host.view(torch.int32), y_dev.view(torch.int32)), mm
        ref = O.conv2d(O.desc(2, 11, 9, 12, 3, 3, 20), lut, x.cpu().numpy(), f.cpu().numpy(), *mm, want=("out_ref", "acc"))
        assert np.array_equal(d_dev["acc"].cpu().numpy(), ref["acc"])
        assert np.array_equal(y_dev.cpu().numpy().view(np.uint32), ref["out_ref"].view(np.uint32)), mm


def test_two_streams_two_layers(ax):
    """Calls on different streams, each with its own workspace, may be in flight together: two layers
    launched back to back on two streams, several times over, give the bits each gives alone."""
    import torch
    rng = np.random.Generator(np.random.PCG64(41))
    lut = cases.make_table(("noisy", 36))
    t = ax.Table(array=lut)
    xa = torch.from_numpy(rng.uniform(-1, 1, (4, 40, 40, 16)).astype(np.float32)).cuda()
    fa = torch.from_numpy(rng.normal(0, 0.1, (3, 3, 16, 64)).astype(np.float32)).cuda()
    xb = torch.from_numpy(rng.uniform(-1, 1, (2, 28, 28, 64)).astype(np.float32)).cuda()
    fb = torch.from_numpy(rng.normal(0, 0.1, (1, 1, 64, 160)).astype(np.float32)).cuda()

    def conv(x, f):
        return ax.approx_conv2d_with_min_max_vars(x, f, -1.0, 1.0, -0.4, 0.4, strides=[1, 1, 1, 1], num_bits=8,
                                                  mul_map_file=t, padding="SAME")
    ya, yb = conv(xa, fa), conv(xb, fb)
    torch.cuda.synchronize()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    outs = []
    for _ in range(5):
        with torch.cuda.stream(sa):
            oa = conv(xa, fa)
        with torch.cuda.stream(sb):
            ob = conv(xb, fb)
        outs.append((oa, ob))
    torch.cuda.synchronize()
    for oa, ob in outs:
        assert torch.equal(oa, ya) and torch.equal(ob, yb)


def test_first_use_of_a_table_on_a_non_blocking_stream(ax):
    """A table's 128 KiB replica is uploaded at its first use.  The upload must be complete before the call's kernels
    read it, also when the caller's stream is a non-blocking one, which does not wait for the legacy stream that a
    copy from pageable host memory is ordered on.  Fresh table handles, first use on a side stream, many times."""
    import torch
    rng = np.random.Generator(np.random.PCG64(43))
    x = torch.from_numpy(rng.uniform(-1, 1, (1, 6, 6, 8)).astype(np.float32)).cuda()
    f = torch.from_numpy(rng.normal(0, 0.1, (1, 1, 8, 32)).astype(np.float32)).cuda()
    side = torch.cuda.Stream()
    for i in range(40):
        lut = cases.make_table(("noisy", 500 + i))
        t_first = ax.Table(array=lut)
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            y = ax.approx_conv2d_with_min_max_vars(x, f, -1.0, 1.0, -0.4, 0.4, [1, 1, 1, 1], 8, t_first, "SAME")
        side.synchronize()
        want = ax.approx_conv2d_with_min_max_vars(x, f, -1.0, 1.0, -0.4, 0.4, [1, 1, 1, 1], 8, ax.Table(array=lut), "SAME")
        torch.cuda.synchronize()
        assert torch.equal(y, want), i


def test_host_threads_call_concurrently(ax):
    """Four host threads, each with its own table handle, stream and workspace, call the op at the same time (ctypes
    releases the interpreter lock during a call): every result equals the one computed alone."""
    import threading
    import torch
    rng = np.random.Generator(np.random.PCG64(44))
    jobs = []
    for i in range(4):
        x = torch.from_numpy(rng.uniform(-1, 1, (2, 14 + i, 14, 16)).astype(np.float32)).cuda()
        f = torch.from_numpy(rng.normal(0, 0.1, (3, 3, 16, 32 * (i + 1))).astype(np.float32)).cuda()
        lut = cases.make_table(("noisy", 600 + i))
        want = ax.approx_conv2d_with_min_max_vars(x, f, -1.0, 1.0, -0.4, 0.4, [1, 1, 1, 1], 8, ax.Table(array=lut), "SAME")
        jobs.append((x, f, lut, want))
    torch.cuda.synchronize()
    errors = []

    def work(x, f, lut, want):
        try:
            stream = torch.cuda.Stream()
            table = ax.Table(array=lut)                    # first use of this handle happens inside the thread
            with torch.cuda.stream(stream):
                for _ in range(10):
                    y = ax.approx_conv2d_with_min_max_vars(x, f, -1.0, 1.0, -0.4, 0.4, [1, 1, 1, 1], 8, table, "SAME")
                    stream.synchronize()
                    if not torch.equal(y, want):
                        errors.append("mismatch")
        except Exception as e:                             # noqa: BLE001 - reported by the assertion below
            errors.append(repr(e))

    threads = [threading.Thread(target=work, args=j) for j in jobs]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors


def test_empty_batch(ax):
    import torch
    y = ax.approx_conv2d_with_min_max_vars(torch.zeros(0, 8, 8, 4).cuda(), torch.zeros(3, 3, 4, 8).cuda(),
                                           -1., 1., -1., 1., [1, 1, 1, 1], 8, "", "SAME")
    assert tuple(y.shape) == (0, 8, 8, 8)


def test_non_symmetric_table_pins_operand_order(ax):
    """LUT[activation][weight], not the transpose."""
    lut = np.zeros((256, 256), np.uint16)
    lut[:, :] = np.arange(256, dtype=np.uint16)[:, None]          # value = activation level
    x = np.full((1, 3, 3, 4), 0.5, np.float32)
    f = np.full((1, 1, 4, 2), 0.25, np.float32)
    y, dbg = run_dense(ax, lut.reshape(-1), x, f, (0.0, 1.0, 0.0, 1.0), (1, 1), (1, 1), "SAME")
    qa, qb = int(dbg["qinput"][0, 0, 0, 0]), int(dbg["qfilter"][0, 0])
    assert qa in (127, 128) and qb in (63, 64) and qa != qb
    assert (dbg["acc"] == 4 * qa).all()


# ---- depthwise -----------------------------------------------------------------------------
def run_depthwise(ax, lut, x, f, mm, stride, dil, pad):
    import torch
    y, dbg = ax.approx_depthwise_conv2d_with_min_max_vars(
        torch.from_numpy(x).cuda(), torch.from_numpy(f).cuda(), *mm, strides=[1, stride[0], stride[1], 1],
        num_bits=8, mul_map_file=ax.Table(array=lut), padding=pad, dilations=[1, dil[0], dil[1], 1], debug=True)
    torch.cuda.synchronize()
    assert dbg["status"] == 0
    return y.cpu().numpy(), {k: v.cpu().numpy() for k, v in dbg.items() if k != "status"}


@pytest.mark.parametrize("case", cases.DEPTHWISE_CASES, ids=[c[0] for c in cases.DEPTHWISE_CASES])
def test_golden_depthwise(ax, golden, case):
    name, ishape, (kh, kw, mult), stride, dil, pad, tspec, in_range, seed = case
    lut = cases.make_table(tspec)
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], mult), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    y, dbg = run_depthwise(ax, lut, x, f, mm, stride, dil, pad)
    assert np.array_equal(dbg["acc"], golden["aux"][name + "_acc"])
    # K = KH*KW <= 256 and tap-order sums: the checker's fp32 result is reproduced bit for bit
    assert np.array_equal(y.view(np.uint32), golden["aux"][name + "_out_ref"].view(np.uint32))


DW_SHAPES = [
    (2, 14, 14, 32, 3, 3, 1, (1, 1), (1, 1), "SAME"),
    (1, 15, 17, 96, 3, 3, 1, (2, 2), (1, 1), "SAME"),
    (1, 29, 31, 33, 3, 3, 1, (1, 1), (1, 1), "VALID"),   # run tail, channel tail
    (1, 9, 9, 7, 3, 3, 3, (2, 2), (1, 1), "VALID"),      # multiplier 3
    (2, 8, 8, 5, 1, 1, 1, (1, 1), (1, 1), "SAME"),
    (1, 12, 12, 16, 5, 5, 1, (1, 1), (1, 1), "SAME"),
    (1, 12, 12, 16, 3, 3, 1, (1, 2), (1, 1), "SAME"),    # anisotropic stride -> generic kernel
    # 1024 output pixels and more: the kernel with the per-channel-group expanded table
    (2, 28, 28, 144, 3, 3, 1, (1, 1), (1, 1), "SAME"),   # 4.5 channel groups, 4 bands of 7 rows
    (1, 56, 56, 40, 3, 3, 1, (1, 1), (1, 1), "SAME"),    # channel tail of 8
    (2, 57, 55, 96, 3, 3, 1, (2, 2), (1, 1), "SAME"),    # stride 2, odd sizes: padding before and after
    (1, 112, 112, 32, 3, 3, 1, (2, 2), (1, 1), "SAME"),  # stride 2, even sizes: padding after only
    (1, 45, 47, 33, 3, 3, 1, (1, 1), (1, 1), "VALID"),   # 43 output rows: a band of one row at the bottom
    (1, 80, 40, 7, 3, 3, 3, (2, 2), (1, 1), "VALID"),    # multiplier 3, stride 2
    (3, 33, 35, 64, 3, 3, 1, (1, 1), (1, 1), "SAME"),
    (1, 36, 36, 16, 3, 3, 2, (1, 1), (1, 1), "SAME"),    # multiplier 2
    (8, 56, 56, 144, 3, 3, 1, (1, 1), (1, 1), "SAME"),   # 320 units on 148 CTAs: CTAs whose range crosses a channel group
    (6, 56, 56, 96, 3, 3, 1, (2, 2), (1, 1), "SAME"),    # the same for stride 2
]


@pytest.mark.parametrize("shape", DW_SHAPES, ids=["-".join(str(v) for v in s[:7]) for s in DW_SHAPES])
def test_depthwise_shapes(ax, shape):
    n, h, w, c, kh, kw, mult, stride, dil, pad = shape
    rng = np.random.Generator(np.random.PCG64(hash(shape[:7]) % (1 << 30)))
    x = rng.uniform(0, 2, (n, h, w, c)).astype(np.float32)
    f = rng.normal(0, 0.3, (kh, kw, c, mult)).astype(np.float32)
    mm = (0.0, 2.0, float(f.min()), float(f.max()))
    lut = cases.make_table(("noisy", 34))
    ref = O.depthwise_conv2d(O.desc(n, h, w, c, kh, kw, mult, stride, dil, pad), lut, x, f, *mm)
    y, dbg = run_depthwise(ax, lut, x, f, mm, stride, dil, pad)
    assert np.array_equal(dbg["acc"], ref["acc"])
    assert np.array_equal(y.view(np.uint32), ref["out_ref"].view(np.uint32))
    q = O.quant_props(*mm).input
    want_q = np.clip(np.floor((x - np.float32(q.offset)) * np.float32(q.inv_scale) + np.float32(0.5)), 0, 255)
    assert np.array_equal(dbg["qinput"], want_q.astype(np.uint8))


# ---- full-size properties --------------------------------------------------------------------
def _acc_checksum(torch, qin, qf, lut, kh, kw, stride, pad_before, pad_after, pad_q, oh, ow):
    """Sum over all outputs of the integer accumulators, from per-tap histograms of the quantised input:
    sum_{p,j} acc = sum_{tap,c} sum_a hist_{tap,c}(a) * sum_j LUT[a][qf[tap,c,j]]."""
    n, h, w, c = qin.shape
    lut_t = torch.from_numpy(lut.astype(np.int64)).cuda().view(256, 256)
    padded = torch.nn.functional.pad(qin.permute(0, 3, 1, 2).long(),
                                     (pad_before[1], pad_after[1], pad_before[0], pad_after[0]), value=int(pad_q))
    total = 0
    qf = qf.view(kh, kw, c, -1).long()
    for ky in range(kh):
        for kx in range(kw):
            sl = padded[:, :, ky:ky + (oh - 1) * stride + 1:stride, kx:kx + (ow - 1) * stride + 1:stride]  # n,c,oh,ow
            onehot_hist = torch.zeros(c, 256, dtype=torch.long, device="cuda")
            idx = sl.permute(1, 0, 2, 3).reshape(c, -1)
            onehot_hist.scatter_add_(1, idx, torch.ones_like(idx))
            colsum = lut_t[:, qf[ky, kx]].sum(dim=2)          # [256, c]: sum_j LUT[a][b_cj]
            total += int((onehot_hist * colsum.t()).sum().item())
    return total


@pytest.mark.parametrize("tspec", [("truncated",), ("noisy", 2)], ids=["truncated", "noisy"])
def test_config2_full_size_checksum(ax, tspec):
    """N=256, 56x56x64 -> 64, 3x3 SAME (2.96e10 table MACs): the sum of all int32 accumulators equals the
    histogram identity above, the quantised operands equal a torch restatement of the quantiser, and a
    16-image slice equals the same images convolved alone (what batch sharding relies on)."""
    import torch
    lut = ax.truncated_table() if tspec[0] == "truncated" else ax.noisy_table(3000 + 200 + tspec[1])
    g = torch.Generator(device="cuda").manual_seed(1002)
    x = torch.rand((256, 56, 56, 64), device="cuda", generator=g) * 2 - 1
    f = torch.randn((3, 3, 64, 64), device="cuda", generator=g) * 0.1
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    t = ax.Table(array=lut)
    y, dbg = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", debug=True)
    torch.cuda.synchronize()
    q = O.quant_props(*mm)
    want_q = torch.clamp(torch.floor((x - q.input.offset) * q.input.inv_scale + 0.5), 0, 255).to(torch.uint8)
    assert torch.equal(dbg["qinput"], want_q)
    pad_q = O.lib().axo_quantize(0.0, q.input.offset, q.input.inv_scale)
    chk = _acc_checksum(torch, dbg["qinput"], dbg["qfilter"], lut, 3, 3, 1, (1, 1), (1, 1), pad_q, 56, 56)
    assert int(dbg["acc"].sum(dtype=torch.int64).item()) == chk
    y16, dbg16 = ax.approx_conv2d_with_min_max_vars(x[100:116].contiguous(), f, *mm, [1, 1, 1, 1], 8, t, "SAME", debug=True)
    assert torch.equal(dbg16["acc"], dbg["acc"][100:116]) and torch.equal(y16, y[100:116])
    # CPU checker on two images of the full-size problem
    xs = x[37:39].cpu().numpy()
    ref = O.conv2d(O.desc(2, 56, 56, 64, 3, 3, 64), lut, xs, f.cpu().numpy(), *mm, want=("acc", "out_exact"))
    assert np.array_equal(dbg["acc"][37:39].cpu().numpy(), ref["acc"])
    assert np.array_equal(y[37:39].cpu().numpy().view(np.uint32), ref["out_exact"].view(np.uint32))


def test_exact_table_equals_integer_convolution_full_size(ax):
    """With the exact table the accumulators are the integer convolution of the quantised operands."""
    import torch
    g = torch.Generator(device="cuda").manual_seed(5)
    x = torch.rand((64, 56, 56, 64), device="cuda", generator=g) * 2 - 1
    f = torch.randn((3, 3, 64, 64), device="cuda", generator=g) * 0.1
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    y, dbg = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, "", "SAME", debug=True)
    q = O.quant_props(*mm)
    pad_q = float(O.lib().axo_quantize(0.0, q.input.offset, q.input.inv_scale))
    qa = torch.nn.functional.pad(dbg["qinput"].permute(0, 3, 1, 2).double(), (1, 1, 1, 1), value=pad_q)
    qb = dbg["qfilter"].view(3, 3, 64, 64).permute(3, 2, 0, 1).double()
    want = torch.nn.functional.conv2d(qa, qb).permute(0, 2, 3, 1)
    assert torch.equal(dbg["acc"].double(), want)
