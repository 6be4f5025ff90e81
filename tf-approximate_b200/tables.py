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
