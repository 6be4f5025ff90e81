"""Generates tests/golden/*.npz and tables.json.  Run in the build container, where the reference
checkout is mounted: `python tests/golden/make_golden.py [/path/to/tf-approximate]`.

  ref_dense.npz   outputs of the REFERENCE's own CPU kernels (oracle/_ref/libaxc_ref.so: the reference's
                  tf2/src/approx_nn_conv_kernels.cpp compiled where it lies) on the seeded dense cases
                  and on the reference's op-test recipe
  oracle_aux.npz  integer accumulators / quantised operands of the dense cases and all outputs of the
                  depthwise cases, from the C restatement (the reference keeps no integer outputs and
                  has no depthwise path)
  ref_axq.npz     outputs of the REFERENCE's first-generation op AxConv2D (oracle/_ref/libaxq_ref.so: the
                  reference's tf1/axqconv/axqconv.cc compiled where it lies) on the seeded quantised cases, the
                  plain tables of the multipliers those cases name and their tuned forms, both from the
                  reference's own multiplier selector
  tables.json     sha256 + 32 sampled entries of each truth-table file shipped by the reference
"""
import hashlib
import json
import os
import sys
import tempfile

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)

import cases  # noqa: E402
import tf_approximate_b200 as ax  # noqa: E402
from oracle import oracle as O  # noqa: E402


def main(ref_root):
    O.build(ref_root)
    assert O.ref_available(), "the reference kernels did not build"
    ref_out, aux = {}, {}
    with tempfile.TemporaryDirectory() as tmp:
        for name, ishape, (kh, kw, cout), stride, dil, pad, tspec, in_range, seed in cases.DENSE_CASES:
            lut = cases.make_table(tspec)
            path = "" if tspec[0] == "exact" else os.path.join(tmp, name + ".bin")
            if path:
                ax.write_table(path, lut)
            x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], cout), in_range, seed)
            mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
            d = O.desc(*ishape, kh, kw, cout, stride, dil, pad)
            op = O.RefOp(path)
            assert np.array_equal(op.table(), lut)
            ref_out[name] = op.conv2d(d, x, f, *mm)
            r = O.conv2d(d, lut, x, f, *mm, want=("out_ref", "out_exact", "acc", "qinput", "qfilter"))
            assert np.array_equal(r["out_ref"].view(np.uint32), ref_out[name].view(np.uint32)), name
            aux[name + "_acc"] = r["acc"]
            aux[name + "_out_exact"] = r["out_exact"]
            aux[name + "_qinput"] = r["qinput"]
            aux[name + "_qfilter"] = r["qfilter"]
            op.close()
        # the reference's own test recipe
        xq, fq = cases.recipe_inputs()
        op = O.RefOp("")
        d = O.desc(1, xq.shape[1], xq.shape[2], 1, 8, 8, 1, (1, 1), (1, 1), "SAME")
        ref_out["recipe"] = op.conv2d(d, xq, fq, 0.0, 1.0, 0.0, 1.0)
        op.close()
    for name, ishape, (kh, kw, mult), stride, dil, pad, tspec, in_range, seed in cases.DEPTHWISE_CASES:
        lut = cases.make_table(tspec)
        x, f = cases.make_inputs(ishape, (kh, kw, ishape[3], mult), in_range, seed)
        mm = (in_range[0], in_range[1], float(f.min()), float(f.max()))
        r = O.depthwise_conv2d(O.desc(*ishape, kh, kw, mult, stride, dil, pad), lut, x, f, *mm)
        aux[name + "_acc"] = r["acc"]
        aux[name + "_out_ref"] = r["out_ref"]
        aux[name + "_out_exact"] = r["out_exact"]
    assert O.axq_ref_available(), "the reference's first-generation op did not build"
    axq = {}
    for name in cases.AXQ_MULTIPLIERS:
        plain, tuned = O.axq_ref_table(name, False), O.axq_ref_table(name, True)
        assert plain.min() >= 0 and plain.max() <= 65535
        axq["table_" + name] = plain.astype(np.uint16)
        # the tuned table is a column selection of the plain one: keep the selection
        cols = np.array([next(w2 for w2 in ([w] + list(range(256)))
                              if np.array_equal(tuned.reshape(256, 256)[:, w], plain.reshape(256, 256)[:, w2]))
                         for w in range(256)], np.uint8)
        assert np.array_equal(plain.reshape(256, 256)[:, cols].reshape(-1), tuned)
        axq["tuned_columns_" + name] = cols
    for name, ishape, fshape3, stride, pad, mult, tune, rin, rf, seed in cases.AXQ_CASES:
        qin, qf = cases.make_axq_operands(ishape, fshape3, seed)
        out, lo, hi = O.axq_ref_conv2d(mult, tune, qin, qf, rin[0], rin[1], rf[0], rf[1], stride, pad)
        axq[name + "_out"] = out
        axq[name + "_range"] = np.array([lo, hi], np.float32)
    np.savez_compressed(os.path.join(HERE, "ref_axq.npz"), **axq)
    np.savez_compressed(os.path.join(HERE, "ref_dense.npz"), **ref_out)
    np.savez_compressed(os.path.join(HERE, "oracle_aux.npz"), **aux)

    tables = {}
    tdir = os.path.join(ref_root, "tf2", "examples", "axmul_8x8")
    files = [os.path.join(tdir, n) for n in sorted(os.listdir(tdir)) if n.endswith(".bin")]
    files.append(os.path.join(ref_root, "tf2", "test", "test_mul_table.bin"))
    idx = np.random.Generator(np.random.PCG64(5)).integers(0, 65536, 32)
    for p in files:
        raw = open(p, "rb").read()
        t = np.frombuffer(raw, dtype="<u2")
        rel = os.path.relpath(p, ref_root)
        tables[rel] = {"bytes": len(raw), "sha256": hashlib.sha256(raw).hexdigest(),
                       "sample_index": [int(i) for i in idx], "sample_value": [int(t[i]) for i in idx],
                       "symmetric": bool(np.array_equal(t.reshape(256, 256), t.reshape(256, 256).T))}
    with open(os.path.join(HERE, "tables.json"), "w") as fjson:
        json.dump(tables, fjson, indent=1, sort_keys=True)
    print("wrote", len(ref_out), "reference outputs,", len(aux), "aux arrays,", len(tables), "table digests")


if __name__ == "__main__":
    main(sys.argv[1] if len(sys.argv) > 1 else O.reference_root())
