"""CPU: the C restatement against the golden material of the reference.

 - outputs of the reference's own CPU kernels on the seeded dense cases (tests/golden/ref_dense.npz,
   produced by tests/golden/make_golden.py from the reference's compiled kernels): bit for bit;
 - the reference's op-test recipe and its expected error level (tf2/README.md:30-31);
 - the reference's truth-table files (digests in tests/golden/tables.json; compared where a
   reference checkout is present);
 - known answers of the range nudging (tf2/src/approx_ops_types.h:29-49).
"""
import hashlib
import json
import os

import numpy as np
import pytest

import cases
from oracle import oracle as O

GDIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
REF_ROOT = O.reference_root()


@pytest.mark.parametrize("case", cases.DENSE_CASES, ids=[c[0] for c in cases.DENSE_CASES])
def test_dense_cases_match_reference_bits(built, golden, case):
    name, ishape, (kh, kw, cout), stride, dil, pad, tspec, in_range, seed = case
    lut = cases.make_table(tspec)
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], cout), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    r = O.conv2d(O.desc(*ishape, kh, kw, cout, stride, dil, pad), lut, x, f, *mm,
                 want=("out_ref", "out_exact", "acc", "qinput", "qfilter"))
    want = golden["ref"][name]
    assert r["out_ref"].shape == want.shape
    assert np.array_equal(r["out_ref"].view(np.uint32), want.view(np.uint32))
    # self-consistency of the additions the reference has no output for
    assert np.array_equal(r["acc"], golden["aux"][name + "_acc"])
    assert np.array_equal(r["qinput"], golden["aux"][name + "_qinput"])
    assert np.array_equal(r["qfilter"], golden["aux"][name + "_qfilter"])
    k = kh * kw * ishape[3]
    if k <= 256:  # every partial sum < 2^24: the fp32 running total is the exact integer
        assert np.array_equal(r["out_ref"].view(np.uint32), r["out_exact"].view(np.uint32))


def test_integer_accumulator_is_a_plain_table_sum(built):
    """acc[p][j] recomputed in numpy from qinput/qfilter for a 1x1 case."""
    rng = np.random.Generator(np.random.PCG64(9))
    lut = cases.make_table(("noisy", 40))
    x = rng.uniform(-1, 1, (2, 5, 5, 12)).astype(np.float32)
    f = rng.normal(0, 0.1, (1, 1, 12, 10)).astype(np.float32)
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    r = O.conv2d(O.desc(2, 5, 5, 12, 1, 1, 10), lut, x, f, *mm, want=("acc", "qinput", "qfilter"))
    qa = r["qinput"].reshape(-1, 12).astype(np.int64)
    qb = r["qfilter"].astype(np.int64)
    acc = lut.astype(np.int64)[(qa[:, :, None] << 8) | qb[None, :, :]].sum(axis=1)
    assert np.array_equal(acc, r["acc"].reshape(-1, 10))


def test_reference_recipe_error_level(built, golden):
    """The reference's op test: exact table, fake-quantised [0,1] operands, compared with the float
    convolution; README states 3.07e-07 'or a different negligible number'."""
    xq, fq = cases.recipe_inputs()
    d = O.desc(1, xq.shape[1], xq.shape[2], 1, 8, 8, 1, (1, 1), (1, 1), "SAME")
    r = O.conv2d(d, O.exact_table(), xq, fq, 0.0, 1.0, 0.0, 1.0, want=("out_ref",))
    assert np.array_equal(r["out_ref"].view(np.uint32), golden["ref"]["recipe"].view(np.uint32))
    import torch
    ref = torch.nn.functional.conv2d(torch.from_numpy(xq).permute(0, 3, 1, 2).double(),
                                     torch.from_numpy(fq).permute(3, 2, 0, 1).double(),
                                     padding=0)
    # SAME padding for an 8x8 window: 3 before, 4 after
    xp = torch.nn.functional.pad(torch.from_numpy(xq).permute(0, 3, 1, 2).double(), (3, 4, 3, 4))
    ref = torch.nn.functional.conv2d(xp, torch.from_numpy(fq).permute(3, 2, 0, 1).double())
    ref = ref.permute(0, 2, 3, 1).numpy()
    linf = np.abs(r["out_ref"] - ref).max() / np.abs(ref).max()
    assert linf < 1e-6, linf


def test_direct_loop_restatement_agrees(built):
    """Second, independent restatement (tf2/src/approx_nn_conv_ops_ref.cpp:231-317) on shapes where its
    centre-based offsets coincide with TensorFlow's."""
    rng = np.random.Generator(np.random.PCG64(17))
    lut = cases.make_table(("noisy", 41))
    for (n, h, w, c, kh, kw, co, s, p) in [(1, 9, 9, 4, 3, 3, 5, (1, 1), "SAME"), (2, 8, 10, 3, 3, 3, 4, (2, 2), "SAME"),
                                          (1, 7, 7, 6, 1, 1, 8, (1, 1), "VALID"), (1, 9, 9, 2, 3, 3, 3, (1, 1), "VALID")]:
        x = rng.uniform(-1, 1, (n, h, w, c)).astype(np.float32)
        f = rng.normal(0, 0.1, (kh, kw, c, co)).astype(np.float32)
        mm = (-1.0, 1.0, float(f.min()), float(f.max()))
        d = O.desc(n, h, w, c, kh, kw, co, s, (1, 1), p)
        a = O.conv2d(d, lut, x, f, *mm, want=("out_ref",))["out_ref"]
        b = O.conv2d_direct(d, lut, x, f, *mm)
        assert np.abs(a - b).max() <= 2e-6 * np.abs(a).max()


@pytest.mark.parametrize("case", cases.DEPTHWISE_CASES, ids=[c[0] for c in cases.DEPTHWISE_CASES])
def test_depthwise_regression(built, golden, case):
    """Depthwise has no reference counterpart (parity unpinned): regression against stored outputs and
    a check against the dense restatement applied channel by channel."""
    name, ishape, (kh, kw, mult), stride, dil, pad, tspec, in_range, seed = case
    lut = cases.make_table(tspec)
    x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], mult), in_range, seed)
    mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
    r = O.depthwise_conv2d(O.desc(*ishape, kh, kw, mult, stride, dil, pad), lut, x, f, *mm)
    assert np.array_equal(r["acc"], golden["aux"][name + "_acc"])
    assert np.array_equal(r["out_ref"].view(np.uint32), golden["aux"][name + "_out_ref"].view(np.uint32))
    c = ishape[3] // 2
    dd = O.desc(ishape[0], ishape[1], ishape[2], 1, kh, kw, mult, stride, dil, pad)
    one = O.conv2d(dd, lut, x[..., c:c + 1], f[:, :, c:c + 1, :], *mm, want=("acc",))
    if not (kh == ishape[1] and kw == ishape[2]):
        assert np.array_equal(one["acc"], r["acc"][..., c * mult:(c + 1) * mult])


def test_nudge_known_answers(built):
    q = O.quant_props(-1.0, 1.0, 0.0, 1.0)
    assert q.input.scale == np.float32(2.0) / np.float32(255.0)
    # zero point of [-1,1]: fp32 1/(2/255) lands just below 127.5, so it rounds to 127 (the compiled
    # reference kernels give the same bits, see test_oracle_vs_ref.py)
    assert q.input.offset == np.float32(-127.0) * np.float32(q.input.scale)
    # [-1, 0.9921875]: zero point exactly 128.0
    q2 = O.quant_props(-1.0, 0.9921875, 0.0, 1.0)
    assert q2.input.scale == np.float32(0.0078125) and q2.input.offset == np.float32(-1.0)
    assert q.filter.scale == np.float32(1.0) / np.float32(255.0) and q.filter.offset == 0.0
    assert q.s1s2 == np.float32(q.input.scale) * np.float32(q.filter.scale) and q.m1m2 == 0.0
    z = O.quant_props(0.0, 0.0, 0.0, 0.0)
    assert (z.input.scale, z.input.inv_scale, z.input.offset) == (0.0, 0.0, 0.0)
    # a range entirely above zero clamps the zero point to 0; entirely below, to 255
    assert O.quant_props(1.0, 2.0, 0.0, 1.0).input.offset == 0.0
    qn = O.quant_props(-2.0, -1.0, 0.0, 1.0)
    assert qn.input.offset == np.float32(-255.0) * np.float32(qn.input.scale)


def test_quantiser_rounds_half_up_and_saturates(built):
    q = O.quant_props(0.0, 255.0, 0.0, 1.0)  # scale exactly 1
    L = O.lib()
    assert L.axo_quantize(0.49, q.input.offset, q.input.inv_scale) == 0
    assert L.axo_quantize(0.5, q.input.offset, q.input.inv_scale) == 1
    assert L.axo_quantize(254.5, q.input.offset, q.input.inv_scale) == 255
    assert L.axo_quantize(300.0, q.input.offset, q.input.inv_scale) == 255
    assert L.axo_quantize(-3.0, q.input.offset, q.input.inv_scale) == 0


def test_exact_table_matches_reference_test_table():
    """tf2/test/test_mul_table.bin is the exact product and equals mul8u_1JFF.bin (tf2/README.md:117)."""
    digests = json.load(open(os.path.join(GDIR, "tables.json")))
    import tf_approximate_b200 as ax
    mine = hashlib.sha256(ax.exact_table().astype("<u2").tobytes()).hexdigest()
    assert digests["tf2/test/test_mul_table.bin"]["sha256"] == mine
    assert digests["tf2/examples/axmul_8x8/mul8u_1JFF.bin"]["sha256"] == mine
    assert len(digests) == 37 and all(v["bytes"] == 131072 for v in digests.values())
    assert np.array_equal(O.exact_table(), ax.exact_table())


@pytest.mark.skipif(not os.path.isdir(REF_ROOT), reason="no reference checkout on this machine")
def test_table_loader_reads_reference_files(built):
    digests = json.load(open(os.path.join(GDIR, "tables.json")))
    for rel, info in digests.items():
        t = O.load_table(os.path.join(REF_ROOT, rel))
        assert hashlib.sha256(t.astype("<u2").tobytes()).hexdigest() == info["sha256"]
        assert [int(t[i]) for i in info["sample_index"]] == info["sample_value"]
    # operand order: non-symmetric tables exist, so (a << 8) | b is observable
    assert not digests["tf2/examples/axmul_8x8/mul8u_L40.bin"]["symmetric"]


def test_table_loader_rejects_short_file(built, tmp_path):
    p = tmp_path / "short.bin"
    p.write_bytes(b"\0" * 1000)
    with pytest.raises(ValueError):
        O.load_table(str(p))
    with pytest.raises(ValueError):
        O.load_table(str(tmp_path / "missing.bin"))


def test_quantised_op_golden(built):
    """The checker's integer functor, weight tuning, zero points and output range against outputs of the
    reference's own AxConv2D (ref_axq.npz)."""
    gold = np.load(os.path.join(GDIR, "ref_axq.npz"))
    for name in cases.AXQ_MULTIPLIERS:
        plain = gold["table_" + name]
        tuned = plain.reshape(256, 256)[:, gold["tuned_columns_" + name]].reshape(-1)
        assert np.array_equal(O.tune_table(plain), tuned), name
    for name, ishape, fshape3, stride, pad, mult, tune, rin, rf, seed in cases.AXQ_CASES:
        qin, qf = cases.make_axq_operands(ishape, fshape3, seed)
        lut = gold["table_" + mult]
        if tune:
            lut = O.tune_table(lut)
        d = O.desc(*ishape, fshape3[0], fshape3[1], fshape3[2], (stride, stride), (1, 1), pad)
        got = O.qconv2d(d, lut, qin, qf, O.quantized_zero_point(*rin), O.quantized_zero_point(*rf))
        assert np.array_equal(got, gold[name + "_out"]), name
        lo, hi = O.quantized_output_range(rin[0], rin[1], rf[0], rf[1])
        assert np.array_equal(np.array([lo, hi], np.float32).view(np.uint32), gold[name + "_range"].view(np.uint32)), name
