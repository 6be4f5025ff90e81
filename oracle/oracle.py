"""TEST INFRASTRUCTURE - ctypes bindings of the checker libraries.

`libaxc_oracle.so` is the C restatement (oracle/axc_oracle.c); `_ref/libaxc_ref.so`
is the reference's own CPU kernel translation unit and `_ref/libaxq_ref.so` its
first-generation quantised op, both built by oracle/Makefile from the reference checkout.
Only tests, the smoke check and the CPU-baseline leg of the benchmark may import
this module; the shipped package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "libaxc_oracle.so")
REF_SO = os.path.join(_HERE, "_ref", "libaxc_ref.so")
AXQ_REF_SO = os.path.join(_HERE, "_ref", "libaxq_ref.so")

SAME, VALID = 0, 1


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int) for n in
                ("n", "h", "w", "c", "kh", "kw", "cout", "stride_h", "stride_w", "dil_h", "dil_w", "padding")]


class VarQuant(C.Structure):
    _fields_ = [("scale", C.c_float), ("inv_scale", C.c_float), ("offset", C.c_float)]


class Quant(C.Structure):
    _fields_ = [("input", VarQuant), ("filter", VarQuant),
                ("s1s2", C.c_float), ("m1", C.c_float), ("m2", C.c_float), ("m1m2", C.c_float)]


def reference_root():
    """Where the reference checkout lies: $AXC_REFERENCE_ROOT, else a directory `reference` beside the repository."""
    return os.environ.get("AXC_REFERENCE_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")


def build(ref_root=None):
    """Compile the checker libraries (gcc only; seconds)."""
    subprocess.run(["make", "-C", _HERE, "REF=" + (ref_root or reference_root())], check=True, stdout=subprocess.DEVNULL)


_lib = None
_ref = None


def _ptr(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build()
        L = C.CDLL(ORACLE_SO)
        L.axo_quant_props.argtypes = [C.c_float] * 4 + [C.POINTER(Quant)]
        L.axo_quant_props.restype = None
        L.axo_quantize.argtypes = [C.c_float] * 3
        L.axo_quantize.restype = C.c_uint8
        L.axo_exact_table.argtypes = [C.POINTER(C.c_uint16)]
        L.axo_load_table.argtypes = [C.c_char_p, C.POINTER(C.c_uint16)]
        L.axo_out_dims.argtypes = [C.POINTER(ConvDesc)] + [C.POINTER(C.c_int)] * 4
        L.axo_conv2d.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_uint16), C.POINTER(C.c_float),
                                 C.POINTER(C.c_float)] + [C.c_float] * 4 + \
                                [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_int32),
                                 C.POINTER(C.c_uint8), C.POINTER(C.c_uint8), C.POINTER(C.c_uint8), C.c_int]
        L.axo_conv2d_direct.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_uint16), C.POINTER(C.c_float),
                                        C.POINTER(C.c_float)] + [C.c_float] * 4 + [C.POINTER(C.c_float)]
        L.axo_depthwise_conv2d.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_uint16), C.POINTER(C.c_float),
                                           C.POINTER(C.c_float)] + [C.c_float] * 4 + \
                                          [C.POINTER(C.c_float), C.POINTER(C.c_float), C.POINTER(C.c_int32), C.c_int]
        L.axo_qconv2d.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_uint16), C.POINTER(C.c_uint8), C.POINTER(C.c_uint8),
                                  C.c_int, C.c_int, C.POINTER(C.c_int32)]
        L.axo_tune_table.argtypes = [C.POINTER(C.c_uint16), C.POINTER(C.c_uint16)]
        L.axo_tune_table.restype = None
        L.axo_quantized_zero_point.argtypes = [C.c_float, C.c_float]
        L.axo_quantized_zero_point.restype = C.c_int32
        L.axo_quantized_output_range.argtypes = [C.c_float] * 4 + [C.POINTER(C.c_float)] * 2
        L.axo_quantized_output_range.restype = None
        L.axo_max_threads.restype = C.c_int
        _lib = L
    return _lib


def desc(n, h, w, c, kh, kw, cout, stride=(1, 1), dilation=(1, 1), padding="SAME"):
    pad = {"SAME": SAME, "VALID": VALID}[padding]
    return ConvDesc(n, h, w, c, kh, kw, cout, stride[0], stride[1], dilation[0], dilation[1], pad)


def out_dims(d):
    oh, ow, ph, pw = C.c_int(), C.c_int(), C.c_int(), C.c_int()
    rc = lib().axo_out_dims(C.byref(d), C.byref(oh), C.byref(ow), C.byref(ph), C.byref(pw))
    if rc:
        raise ValueError("axo_out_dims status %d" % rc)
    return oh.value, ow.value, ph.value, pw.value


def quant_props(in_min, in_max, f_min, f_max):
    q = Quant()
    lib().axo_quant_props(in_min, in_max, f_min, f_max, C.byref(q))
    return q


def exact_table():
    t = np.empty(65536, np.uint16)
    lib().axo_exact_table(_ptr(t, C.c_uint16))
    return t


def load_table(path):
    t = np.empty(65536, np.uint16)
    rc = lib().axo_load_table(path.encode(), _ptr(t, C.c_uint16))
    if rc:
        raise ValueError("ApproxTF: Couldn't read the lookup table!")
    return t


def max_threads():
    return lib().axo_max_threads()


def conv2d(d, lut, x, f, in_min, in_max, f_min, f_max, want=("out_ref", "out_exact", "acc"), nthreads=0):
    """Run the restated forward pass.  Returns a dict of the requested outputs."""
    oh, ow, _, _ = out_dims(d)
    x = np.ascontiguousarray(x, np.float32)
    f = np.ascontiguousarray(f, np.float32)
    lut = np.ascontiguousarray(lut, np.uint16)
    oshape = (d.n, oh, ow, d.cout)
    r = {}
    if "out_ref" in want:
        r["out_ref"] = np.zeros(oshape, np.float32)
    if "out_exact" in want:
        r["out_exact"] = np.zeros(oshape, np.float32)
    if "acc" in want:
        r["acc"] = np.zeros(oshape, np.int32)
    if "qinput" in want:
        r["qinput"] = np.zeros((d.n, d.h, d.w, d.c), np.uint8)
    if "qfilter" in want:
        r["qfilter"] = np.zeros((d.kh * d.kw * d.c, d.cout), np.uint8)
    padq = np.zeros(1, np.uint8)
    rc = lib().axo_conv2d(C.byref(d), _ptr(lut, C.c_uint16), _ptr(x, C.c_float), _ptr(f, C.c_float),
                          in_min, in_max, f_min, f_max,
                          _ptr(r.get("out_ref"), C.c_float), _ptr(r.get("out_exact"), C.c_float),
                          _ptr(r.get("acc"), C.c_int32), _ptr(r.get("qinput"), C.c_uint8),
                          _ptr(r.get("qfilter"), C.c_uint8), _ptr(padq, C.c_uint8), nthreads)
    if rc:
        raise ValueError("axo_conv2d status %d" % rc)
    r["pad_q"] = int(padq[0])
    return r


def conv2d_direct(d, lut, x, f, in_min, in_max, f_min, f_max):
    oh, ow, _, _ = out_dims(d)
    x = np.ascontiguousarray(x, np.float32)
    f = np.ascontiguousarray(f, np.float32)
    lut = np.ascontiguousarray(lut, np.uint16)
    out = np.zeros((d.n, oh, ow, d.cout), np.float32)
    rc = lib().axo_conv2d_direct(C.byref(d), _ptr(lut, C.c_uint16), _ptr(x, C.c_float), _ptr(f, C.c_float),
                                 in_min, in_max, f_min, f_max, _ptr(out, C.c_float))
    if rc:
        raise ValueError("axo_conv2d_direct status %d" % rc)
    return out


def qconv2d(d, lut, qin, qf, input_offset, filter_offset):
    """The first-generation op's integer functor (tf1/axqconv/axqconv.cc:132-263): uint8 in, int32 out."""
    oh, ow, _, _ = out_dims(d)
    qin = np.ascontiguousarray(qin, np.uint8)
    qf = np.ascontiguousarray(qf, np.uint8)
    lut = np.ascontiguousarray(lut, np.uint16)
    out = np.zeros((d.n, oh, ow, d.cout), np.int32)
    rc = lib().axo_qconv2d(C.byref(d), _ptr(lut, C.c_uint16), _ptr(qin, C.c_uint8), _ptr(qf, C.c_uint8),
                           int(input_offset), int(filter_offset), _ptr(out, C.c_int32))
    if rc:
        raise ValueError("axo_qconv2d status %d" % rc)
    return out


def tune_table(lut):
    """Weight tuning of the first-generation op (tf1/axqconv/approximate_selector.h:46-78)."""
    lut = np.ascontiguousarray(lut, np.uint16).reshape(65536)
    out = np.zeros(65536, np.uint16)
    lib().axo_tune_table(_ptr(lut, C.c_uint16), _ptr(out, C.c_uint16))
    return out


def quantized_zero_point(range_min, range_max):
    return int(lib().axo_quantized_zero_point(range_min, range_max))


def quantized_output_range(min_a, max_a, min_b, max_b):
    lo, hi = C.c_float(), C.c_float()
    lib().axo_quantized_output_range(min_a, max_a, min_b, max_b, C.byref(lo), C.byref(hi))
    return lo.value, hi.value


def depthwise_conv2d(d, lut, x, f, in_min, in_max, f_min, f_max, nthreads=0):
    """d.cout is the channel multiplier; filter [KH,KW,C,mult]."""
    oh, ow, _, _ = out_dims(d)
    x = np.ascontiguousarray(x, np.float32)
    f = np.ascontiguousarray(f, np.float32)
    lut = np.ascontiguousarray(lut, np.uint16)
    oshape = (d.n, oh, ow, d.c * d.cout)
    r = {"out_ref": np.zeros(oshape, np.float32), "out_exact": np.zeros(oshape, np.float32),
         "acc": np.zeros(oshape, np.int32)}
    rc = lib().axo_depthwise_conv2d(C.byref(d), _ptr(lut, C.c_uint16), _ptr(x, C.c_float), _ptr(f, C.c_float),
                                    in_min, in_max, f_min, f_max, _ptr(r["out_ref"], C.c_float),
                                    _ptr(r["out_exact"], C.c_float), _ptr(r["acc"], C.c_int32), nthreads)
    if rc:
        raise ValueError("axo_depthwise_conv2d status %d" % rc)
    return r


# --------------------------------------------------------------------------------------
# The reference's own kernels (compiled from the reference checkout).
# --------------------------------------------------------------------------------------
def ref_available():
    return os.path.exists(REF_SO)


def ref_lib():
    global _ref
    if _ref is None:
        R = C.CDLL(REF_SO)
        R.axr_create.argtypes = [C.c_char_p, C.c_int]
        R.axr_create.restype = C.c_void_p
        R.axr_destroy.argtypes = [C.c_void_p]
        R.axr_update.argtypes = [C.c_void_p] + [C.c_float] * 4
        R.axr_get_quant.argtypes = [C.c_void_p, C.POINTER(C.c_float)]
        R.axr_get_table.argtypes = [C.c_void_p, C.POINTER(C.c_uint16)]
        R.axr_conv2d.argtypes = [C.c_void_p] + [C.c_int] * 12 + [C.POINTER(C.c_float)] * 2 + \
                                [C.c_float] * 4 + [C.POINTER(C.c_float)]
        _ref = R
    return _ref


_axq = None


def axq_ref_available():
    return os.path.exists(AXQ_REF_SO)


def axq_ref_lib():
    global _axq
    if _axq is None:
        R = C.CDLL(AXQ_REF_SO)
        R.refq_table.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_int32)]
        R.refq_conv2d.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_uint8)] + [C.c_int] * 4 + [C.POINTER(C.c_uint8)] + \
                                 [C.c_int] * 3 + [C.c_float] * 4 + [C.c_int, C.c_int, C.POINTER(C.c_int32),
                                                                    C.POINTER(C.c_float), C.POINTER(C.c_float)]
        _axq = R
    return _axq


def axq_ref_table(name, tune):
    """The table the reference's multiplier selector builds for `name` (e.g. 'mul8u_L40'), int32[65536]."""
    t = np.zeros(65536, np.int32)
    if axq_ref_lib().refq_table(name.encode(), 1 if tune else 0, _ptr(t, C.c_int32)):
        raise ValueError("unknown multiplier " + name)
    return t


def axq_ref_conv2d(name, tune, qin, qf, min_input, max_input, min_filter, max_filter, stride, padding):
    """One Compute() of the reference's AxConv2D: (int32 output, min_output, max_output)."""
    qin = np.ascontiguousarray(qin, np.uint8)
    qf = np.ascontiguousarray(qf, np.uint8)
    n, h, w, c = qin.shape
    kh, kw, _, co = qf.shape
    oh, ow, _, _ = out_dims(desc(n, h, w, c, kh, kw, co, (stride, stride), (1, 1), padding))
    out = np.zeros((n, oh, ow, co), np.int32)
    lo, hi = C.c_float(), C.c_float()
    rc = axq_ref_lib().refq_conv2d(name.encode(), 1 if tune else 0, _ptr(qin, C.c_uint8), n, h, w, c, _ptr(qf, C.c_uint8),
                                   kh, kw, co, min_input, max_input, min_filter, max_filter, stride,
                                   1 if padding == "SAME" else 0, _ptr(out, C.c_int32), C.byref(lo), C.byref(hi))
    if rc:
        raise ValueError("the reference op reported an error")
    return out, lo.value, hi.value


class RefOp:
    """The reference's TableApproxOpType_t<CPU> plus its CPU kernels."""

    def __init__(self, mul_map_file="", num_bits=8):
        self._h = ref_lib().axr_create(mul_map_file.encode(), num_bits)
        if not self._h:
            raise ValueError("ApproxTF: Couldn't read the lookup table!")

    def close(self):
        if self._h:
            ref_lib().axr_destroy(self._h)
            self._h = None

    def __del__(self):
        self.close()

    def table(self):
        t = np.empty(65536, np.uint16)
        ref_lib().axr_get_table(self._h, _ptr(t, C.c_uint16))
        return t

    def quant(self, in_min, in_max, f_min, f_max):
        ref_lib().axr_update(self._h, in_min, in_max, f_min, f_max)
        q = np.empty(10, np.float32)
        ref_lib().axr_get_quant(self._h, _ptr(q, C.c_float))
        return q

    def conv2d(self, d, x, f, in_min, in_max, f_min, f_max):
        oh, ow, _, _ = out_dims(d)
        x = np.ascontiguousarray(x, np.float32)
        f = np.ascontiguousarray(f, np.float32)
        out = np.zeros((d.n, oh, ow, d.cout), np.float32)
        rc = ref_lib().axr_conv2d(self._h, d.n, d.h, d.w, d.c, d.kh, d.kw, d.cout, d.stride_h, d.stride_w,
                                  d.dil_h, d.dil_w, d.padding, _ptr(x, C.c_float), _ptr(f, C.c_float),
                                  in_min, in_max, f_min, f_max, _ptr(out, C.c_float))
        if rc:
            raise ValueError("axr_conv2d status %d" % rc)
        return out
