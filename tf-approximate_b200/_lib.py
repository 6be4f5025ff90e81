"""ctypes view of libaxconv.so (C ABI: include/axconv.h).  There is no fallback: when the
library is missing or does not load, every operator of this package raises."""
import ctypes as C
import os

from . import _build

# every symbol include/axconv.h declares
SYMBOLS = [
    "axc_table_create_from_file", "axc_table_create_from_memory", "axc_table_create_exact",
    "axc_table_destroy", "axc_table_tune_weights", "axc_table_host_data", "axc_table_ensure_device",
    "axc_conv2d_output_dims", "axc_depthwise_conv2d_output_dims",
    "axc_conv2d_workspace_bytes", "axc_depthwise_conv2d_workspace_bytes", "axc_conv2d_plan_info",
    "axc_conv2d_forward", "axc_conv2d_forward_device_ranges", "axc_depthwise_conv2d_forward",
    "axc_depthwise_conv2d_forward_noalloc", "axc_depthwise_conv2d_status",
    "axc_quant_props", "axc_status_string", "axc_last_cuda_error", "axc_launch_count", "axc_measure_lookup_peak", "axc_debug_bounds_record",
    "axc_add_residual", "axc_max_pool_same", "axc_conv2d_forward_fused", "axc_depthwise_conv2d_forward_fused", "axc_tensor_range", "axc_fake_quant", "axc_conv2d_forward_sharded", "axc_gather_outputs",
    "axc_qconv2d_workspace_bytes", "axc_qconv2d_forward", "axc_quantized_zero_point", "axc_quantized_output_range",
]


class ConvDesc(C.Structure):
    _fields_ = [(n, C.c_int32) for n in
                ("n", "h", "w", "c", "kh", "kw", "filter_c", "cout", "stride_h", "stride_w",
                 "dil_h", "dil_w", "padding", "data_format", "accumulate", "plan")]


class Shard(C.Structure):
    _fields_ = [("device", C.c_int32), ("n", C.c_int32), ("input", C.c_void_p), ("filter", C.c_void_p),
                ("output", C.c_void_p), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("stream", C.c_void_p)]


class Epilogue(C.Structure):
    _fields_ = [("bias", C.c_void_p), ("residual", C.c_void_p), ("relu", C.c_int32), ("input_relu", C.c_int32)]


class DebugOut(C.Structure):
    _fields_ = [("qinput", C.c_void_p), ("qfilter", C.c_void_p), ("acc", C.c_void_p)]


_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    # AXC_LIBRARY_FLAVOUR=check loads the debug flavour with bounds checks (libaxconv_check.so)
    check = os.environ.get("AXC_LIBRARY_FLAVOUR", "") == "check"
    path = _build.LIB_CHECK if check else _build.LIB
    if not os.path.exists(path):
        raise RuntimeError("libaxconv.so is not built (%s): run `python -c \"import __graft_entry__ as g; "
                           "g.build()\"` at the repository root; there is no CPU fallback" % path)
    L = C.CDLL(path)
    fwd = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float,
           C.c_float, C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(DebugOut), C.c_int, C.c_void_p]
    L.axc_table_create_from_file.argtypes = [C.c_char_p, C.c_int, C.POINTER(C.c_void_p)]
    L.axc_table_create_from_memory.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    L.axc_table_create_exact.argtypes = [C.POINTER(C.c_void_p)]
    L.axc_table_tune_weights.argtypes = [C.c_void_p, C.c_void_p]
    L.axc_table_destroy.argtypes = [C.c_void_p]
    L.axc_table_destroy.restype = None
    L.axc_table_host_data.argtypes = [C.c_void_p, C.POINTER(C.POINTER(C.c_uint16))]
    L.axc_table_ensure_device.argtypes = [C.c_void_p, C.c_int]
    L.axc_conv2d_output_dims.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_int64)]
    L.axc_depthwise_conv2d_output_dims.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_int64)]
    L.axc_conv2d_workspace_bytes.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_size_t)]
    L.axc_depthwise_conv2d_workspace_bytes.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_size_t)]
    L.axc_conv2d_plan_info.argtypes = [C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_void_p]
    L.axc_conv2d_forward.argtypes = fwd
    L.axc_depthwise_conv2d_forward.argtypes = fwd
    L.axc_conv2d_forward_device_ranges.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_void_p,
                                                   C.c_void_p, C.c_void_p, C.c_size_t, C.POINTER(DebugOut), C.c_int,
                                                   C.c_void_p]
    L.axc_depthwise_conv2d_forward_noalloc.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_float,
                                                       C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_int, C.c_void_p]
    L.axc_depthwise_conv2d_status.argtypes = [C.POINTER(ConvDesc), C.c_void_p, C.POINTER(C.c_int32), C.c_int, C.c_void_p]
    L.axc_qconv2d_workspace_bytes.argtypes = [C.POINTER(ConvDesc), C.POINTER(C.c_size_t)]
    L.axc_qconv2d_forward.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_int32, C.c_int32, C.c_void_p,
                                      C.c_void_p, C.c_size_t, C.c_int, C.c_void_p]
    L.axc_quantized_zero_point.argtypes = [C.c_float, C.c_float, C.POINTER(C.c_int32)]
    L.axc_quantized_output_range.argtypes = [C.c_float, C.c_float, C.c_float, C.c_float, C.POINTER(C.c_float)]
    L.axc_conv2d_forward_fused.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_float, C.c_float,
                                           C.c_float, C.c_void_p, C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_size_t,
                                           C.POINTER(DebugOut), C.c_int, C.c_void_p]
    L.axc_depthwise_conv2d_forward_fused.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.c_void_p, C.c_void_p, C.c_float, C.c_float,
                                                     C.c_float, C.c_float, C.POINTER(Epilogue), C.c_void_p, C.c_void_p, C.c_size_t,
                                                     C.POINTER(DebugOut), C.c_int, C.c_void_p]
    L.axc_add_residual.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_int, C.c_void_p]
    L.axc_max_pool_same.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 6 + [C.c_int, C.c_void_p]
    L.axc_conv2d_forward_sharded.argtypes = [C.c_void_p, C.POINTER(ConvDesc), C.POINTER(Shard), C.c_int32, C.c_float, C.c_float,
                                             C.c_float, C.c_float, C.POINTER(C.c_int32)]
    L.axc_gather_outputs.argtypes = [C.POINTER(Shard), C.c_int32, C.c_size_t, C.c_void_p, C.c_int32]
    L.axc_tensor_range.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_int, C.c_void_p]
    L.axc_fake_quant.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_int, C.c_void_p]
    L.axc_quant_props.argtypes = [C.c_float, C.c_float, C.POINTER(C.c_float)]
    L.axc_status_string.argtypes = [C.c_int]
    L.axc_status_string.restype = C.c_char_p
    L.axc_last_cuda_error.restype = C.c_int
    L.axc_launch_count.restype = C.c_uint64
    L.axc_debug_bounds_record.argtypes = [C.c_int, C.POINTER(C.c_uint32)]
    L.axc_measure_lookup_peak.argtypes = [C.c_int, C.c_void_p, C.c_size_t, C.c_void_p, C.POINTER(C.c_double)]
    _lib = L
    return L
