"""CPU: truth-table tooling - generation from a function or a C source (the reference's recipe,
tf2/README.md:104-117), the file format check (tf2/src/approx_ops_types.h:205-216) and the table report."""
import numpy as np
import pytest

from tf_approximate_b200 import tables as T


def test_function_tabulation_matches_the_builtin_tables():
    assert np.array_equal(T.table_from_function(lambda a, b: a * b), T.exact_table())
    assert np.array_equal(T.table_from_function(lambda a, b: (a * b) & 0xFFC0), T.truncated_table())
    # scalar-only callables work too; index order is (activation << 8) | weight
    t = T.table_from_function(lambda a, b: int(a) * 2 + (1 if int(b) > 100 else 0))
    assert t[(7 << 8) | 3] == 14 and t[(7 << 8) | 200] == 15
    with pytest.raises(ValueError):
        T.table_from_function(lambda a, b: a * b * 2 + 70000)


def test_c_source_tabulation(tmp_path):
    """A multiplier in the form of the reference's tf1/axqconv/axmult/*.c files: uint16_t f(uint8_t, uint8_t)."""
    src = tmp_path / "mul8u_demo.c"
    src.write_text("#include <stdint.h>\n"
                   "uint16_t mul8u_demo(uint8_t a, uint8_t b) { return (uint16_t)(((unsigned)a * b) & 0xFFC0u); }\n")
    t = T.table_from_c_source(str(src), "mul8u_demo")
    assert np.array_equal(t, T.truncated_table())


def test_c_source_tabulation_64_bit_form(tmp_path):
    """The other form the reference ships: uint64_t f(const uint64_t B, const uint64_t A); the first parameter is
    the activation (tf1/axqconv/approximate_selector.h:38-41)."""
    src = tmp_path / "mul8u_demo64.c"
    src.write_text("#include <stdint.h>\n"
                   "uint64_t mul8u_demo64(const uint64_t B,const uint64_t A) { return B * 2 + (A > 100 ? 1 : 0); }\n")
    t = T.table_from_c_source(str(src), "mul8u_demo64")
    assert t[(7 << 8) | 3] == 14 and t[(7 << 8) | 200] == 15
    with pytest.raises(ValueError):
        T.table_from_c_source(str(src), "no_such_function")


def test_weight_tuning_matches_checker():
    """axc_table_tune_weights against the checker's restatement of tf1/axqconv/approximate_selector.h:46-78."""
    from oracle import oracle as O
    O.build()
    a = np.arange(256)
    skewed = T.table_from_function(lambda x, y: np.minimum((x * y * 1.1 + 3 * (y % 7)).astype(np.int64), 65535))
    shifted = np.roll(T.exact_table().reshape(256, 256), 5, axis=1).reshape(-1)       # column w holds i * (w - 5)
    for lut in (T.exact_table(), T.truncated_table(), T.noisy_table(9), skewed, shifted):
        got = T.tune_table(lut)
        assert np.array_equal(got, O.tune_table(lut))
    assert np.array_equal(T.tune_table(T.exact_table()), T.exact_table())             # nothing beats the exact column
    assert np.array_equal(T.tune_table(shifted), T.exact_table())                     # every column finds its exact one
    assert not np.array_equal(T.tune_table(skewed), skewed)
    # in place
    from tf_approximate_b200 import _lib
    buf = np.ascontiguousarray(skewed.copy())
    assert _lib.load().axc_table_tune_weights(buf.ctypes.data, buf.ctypes.data) == 0
    assert np.array_equal(buf, O.tune_table(skewed)) and a.size == 256


def test_reference_multipliers_tabulate_like_the_reference_selector():
    """With a reference checkout: table_from_c_source on its multiplier sources (both signatures) against the table
    its own selector builds, and tune_table against the selector's tuning."""
    import os
    from oracle import oracle as O
    src_dir = os.path.join(O.reference_root(), "tf1", "axqconv", "axmult")
    if not (os.path.isdir(src_dir) and O.axq_ref_available()):
        pytest.skip("no reference checkout")
    for name in ("mul8u_1JFF", "mul8u_L40", "mul8u_2AC"):
        t = T.table_from_c_source(os.path.join(src_dir, name + ".c"), name)
        assert np.array_equal(t.astype(np.int32), O.axq_ref_table(name, False)), name
        assert np.array_equal(T.tune_table(t).astype(np.int32), O.axq_ref_table(name, True)), name


def test_file_validation_and_report(tmp_path):
    p = tmp_path / "t.bin"
    T.write_table(str(p), T.noisy_table(5))
    rep = T.validate_table_file(str(p))
    assert rep["bytes"] == 131072 and rep["trailing_bytes"] == 0 and not rep["exact"] and not rep["symmetric"]
    assert 0 < rep["mean_rel_error"] < 0.05 and len(rep["sha256"]) == 64
    assert np.array_equal(T.read_table(str(p)), T.noisy_table(5))
    T.write_table(str(p), T.exact_table())
    rep = T.validate_table_file(str(p))
    assert rep["exact"] and rep["symmetric"] and rep["max_abs_error"] == 0 and rep["zero_row_is_zero"]
    short = tmp_path / "short.bin"
    short.write_bytes(b"\0" * 1000)
    with pytest.raises(ValueError):
        T.validate_table_file(str(short))
    with pytest.raises(ValueError):
        T.read_table(str(short))
