"""Truth tables of 8x8-bit approximate multipliers: 65536 uint16 entries, index (a << 8) | b with
a the activation and b the weight; on disk raw little-endian without header
(tf2/src/approx_ops_types.h:110-117, 205-216; generation recipe tf2/README.md:104-117)."""
import numpy as np


def exact_table():
    a = np.arange(256, dtype=np.uint32)
    return (a[:, None] * a[None, :]).astype(np.uint16).reshape(-1)


def truncated_table(zero_low_bits=6):
    """a*b with the low bits of the product cleared."""
    mask = np.uint16((0xFFFF >> zero_low_bits) << zero_low_bits)
    return exact_table() & mask


def noisy_table(seed, rel_sigma=0.02):
    """clip(round(a*b*(1+e)), 0, 65535), e ~ N(0, rel_sigma) drawn per entry in float64."""
    rng = np.random.Generator(np.random.PCG64(seed))
    e = rng.normal(0.0, rel_sigma, 65536)
    v = np.floor(exact_table().astype(np.float64) * (1.0 + e) + 0.5)
    return np.clip(v, 0, 65535).astype(np.uint16)


def write_table(path, table):
    t = np.ascontiguousarray(table, dtype="<u2").reshape(-1)
    if t.size != 65536:
        raise ValueError("a truth table has 65536 entries")
    t.tofile(path)


def read_table(path):
    t = np.fromfile(path, dtype="<u2")
    if t.size < 65536:
        raise ValueError("ApproxTF: Couldn't read the lookup table!")
    return t[:65536].astype(np.uint16)


def table_from_function(fn):
    """Tabulates fn(a, b) -> product for all 8-bit a (activation) and b (weight), the loop of the reference's
    generation recipe (tf2/README.md:104-117).  `fn` may take numpy arrays (tried first) or scalars."""
    a = np.repeat(np.arange(256, dtype=np.uint32), 256)
    b = np.tile(np.arange(256, dtype=np.uint32), 256)
    try:
        v = np.asarray(fn(a, b))
        if v.shape != (65536,):
            raise TypeError
    except Exception:
        v = np.array([fn(int(x), int(y)) for x, y in zip(a, b)])
    if v.min() < 0 or v.max() > 65535:
        raise ValueError("a table entry does not fit 16 bits")
    return v.astype(np.uint16)


def table_from_c_source(c_path, symbol, cc="gcc"):
    """Compiles a C file that defines the multiplier `symbol(a, b)` and tabulates it.  Handles the two forms of
    the EvoApprox multipliers the reference ships (tf1/axqconv/axmult/*.c): `uint16_t f(uint8_t a, uint8_t b)` and
    `uint64_t f(const uint64_t B, const uint64_t A)`; the first parameter is the activation either way (the
    reference calls f(data, weight), tf1/axqconv/approximate_selector.h:38-41)."""
    import ctypes
    import os
    import re
    import subprocess
    import tempfile
    with open(c_path) as fh:
        m = re.search(r"(uint\d+_t)\s+" + re.escape(symbol) + r"\s*\(\s*(?:const\s+)?(uint\d+_t)", fh.read())
    if m is None:
        raise ValueError("no function %s with unsigned integer parameters in %s" % (symbol, c_path))
    ctype = {"uint8_t": ctypes.c_uint8, "uint16_t": ctypes.c_uint16, "uint32_t": ctypes.c_uint32, "uint64_t": ctypes.c_uint64}
    with tempfile.TemporaryDirectory() as tmp:
        so = os.path.join(tmp, "mul.so")
        subprocess.run([cc, "-O2", "-shared", "-fPIC", "-o", so, c_path], check=True, capture_output=True)
        lib = ctypes.CDLL(so)
        f = getattr(lib, symbol)
        f.restype = ctype[m.group(1)]
        f.argtypes = [ctype[m.group(2)]] * 2
        return table_from_function(lambda a, b: f(a, b))


def tune_table(table):
    """Weight tuning of the reference's first-generation op (attribute AxTune of AxConv2D, on by default there;
    tf1/axqconv/approximate_selector.h:46-78): every weight column is replaced by the column that is closest to the
    exact products."""
    import ctypes
    from . import _lib
    from .errors import raise_for_status
    t = np.ascontiguousarray(table, dtype=np.uint16).reshape(-1)
    if t.size != 65536:
        raise ValueError("a truth table has 65536 entries")
    out = np.empty(65536, np.uint16)
    raise_for_status(_lib.load().axc_table_tune_weights(ctypes.c_void_p(t.ctypes.data), ctypes.c_void_p(out.ctypes.data)), "table tuning")
    return out


def table_report(table):
    """Figures that characterise an approximate multiplier table against the exact product."""
    t = np.asarray(table, dtype=np.int64).reshape(256, 256)
    e = exact_table().astype(np.int64).reshape(256, 256)
    err = t - e
    return {"exact": bool((err == 0).all()),
            "symmetric": bool((t == t.T).all()),          # operand order matters for the others
            "max_abs_error": int(np.abs(err).max()),
            "mean_abs_error": float(np.abs(err).mean()),
            "mean_rel_error": float((np.abs(err)[1:, 1:] / e[1:, 1:]).mean()),
            "zero_row_is_zero": bool((t[0] == 0).all() and (t[:, 0] == 0).all())}


def validate_table_file(path):
    """Checks the on-disk format (raw little-endian uint16, at least 65536 entries, no header:
    tf2/src/approx_ops_types.h:205-216) and returns table_report() of its content plus size and sha256."""
    import hashlib
    import os
    size = os.path.getsize(path)
    if size < 131072:
        raise ValueError("ApproxTF: Couldn't read the lookup table! (%d bytes, 131072 needed)" % size)
    with open(path, "rb") as fh:
        raw = fh.read(131072)
    rep = table_report(np.frombuffer(raw, dtype="<u2"))
    rep.update({"bytes": size, "trailing_bytes": size - 131072, "sha256": hashlib.sha256(raw).hexdigest()})
    return rep
