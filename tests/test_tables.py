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
