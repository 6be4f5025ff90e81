"""Host-side mirror of the reference op on torch CUDA tensors.

`approx_conv2d_with_min_max_vars` keeps the name, the argument order and the error behaviour of
the generated TensorFlow wrapper of `ApproxConv2DWithMinMaxVars`
(tf2/src/approx_nn_ops.cpp:38-54; call site tf2/test/test_table_approx_conv_2d.py:46-49).
torch is used for device memory and streams only."""
import collections
import ctypes as C
import hashlib
import threading

import numpy as np
import torch

from . import _lib
from .errors import InvalidArgumentError, raise_for_status

_PADDING = {"SAME": 0, "VALID": 1, "EXPLICIT": 2}
_FORMAT = {"NHWC": 0, "NCHW": 1}
_ACCUMULATE = {"exact": 0, "reference": 1}
_PLAN = {"keep": 0, "none": 1}


class Table:
    """A truth table handle: host copy plus lazily created per-GPU replicas
    (reference: BaseTableApproxOpType_t, tf2/src/approx_ops_types.h:99-122)."""

    def __init__(self, mul_map_file="", num_bits=8, array=None):
        L = _lib.load()
        h = C.c_void_p()
        if array is not None:
            a = np.ascontiguousarray(array, dtype=np.uint16).reshape(-1)
            if a.size != 65536:
                raise InvalidArgumentError("a truth table has 65536 entries")
            st = L.axc_table_create_from_memory(a.ctypes.data, C.byref(h))
        else:
            if isinstance(mul_map_file, bytes):
                mul_map_file = mul_map_file.decode()
            st = L.axc_table_create_from_file(mul_map_file.encode(), int(num_bits), C.byref(h))
        raise_for_status(st, "table", "ApproxTF: Couldn't read the lookup table!" if num_bits == 8 else
                         "only num_bits == 8 is supported")
        self._h = h

    @property
    def handle(self):
        return self._h

    def numpy(self):
        p = C.POINTER(C.c_uint16)()
        raise_for_status(_lib.load().axc_table_host_data(self._h, C.byref(p)), "table data")
        return np.ctypeslib.as_array(p, shape=(65536,)).copy()

    def tuned(self):
        """The table after the first-generation op's weight tuning (tables.tune_table), made once per table."""
        t = getattr(self, "_tuned", None)
        if t is None:
            from .tables import tune_table
            t = self._tuned = Table(array=tune_table(self.numpy()))
        return t

    def ensure_device(self, device):
        raise_for_status(_lib.load().axc_table_ensure_device(self._h, int(device)), "table upload", _cuda_detail())

    def __del__(self):
        try:
            if getattr(self, "_h", None):
                _lib.load().axc_table_destroy(self._h)
                self._h = None
        except Exception:
            pass


_tables = {}
_tables_lock = threading.Lock()


def _table_for(mul_map_file, num_bits):
    if isinstance(mul_map_file, Table):
        return mul_map_file
    key = (mul_map_file or "", int(num_bits))
    if mul_map_file:
        # key by content, so that a file rewritten under the same name is not served from the cache and two
        # names of the same table share one device replica; an unreadable file goes on to raise in Table()
        try:
            with open(mul_map_file, "rb") as fh:
                key = ("sha256", hashlib.sha256(fh.read(131072)).hexdigest(), int(num_bits))
        except OSError:
            pass
    with _tables_lock:
        t = _tables.get(key)
        if t is None:
            t = Table(mul_map_file or "", num_bits)
            _tables[key] = t
        return t


def _cuda_detail():
    return "cudaError %d" % _lib.load().axc_last_cuda_error()


def _scalar(v):
    if isinstance(v, torch.Tensor):
        return float(v.item())  # host-memory scalar input of the op (tf2/src/approx_nn_conv_ops.cpp:691-694)
    return float(v)


def _desc(input_shape, filter_shape, strides, padding, data_format, dilations, explicit_paddings, accumulate="exact",
          plan="keep"):
    if accumulate not in _ACCUMULATE:
        raise InvalidArgumentError("accumulate must be 'exact' or 'reference'")
    if plan not in _PLAN:
        raise InvalidArgumentError("plan must be 'keep' or 'none'")
    if len(input_shape) != 4:
        raise InvalidArgumentError("input must be 4-dimensional %s" % (tuple(input_shape),))
    if len(filter_shape) != 4:
        raise InvalidArgumentError("filter must be 4-dimensional %s" % (tuple(filter_shape),))
    if data_format not in _FORMAT:
        raise InvalidArgumentError("Invalid data format")
    if len(strides) != 4:
        raise InvalidArgumentError("Sliding window strides must specify 4 dimensions")
    if len(dilations) != 4:
        raise InvalidArgumentError("Sliding window dilations field must specify 4 dimensions")
    pad = padding.upper() if isinstance(padding, str) else padding
    if pad not in _PADDING:
        raise InvalidArgumentError("unknown padding %r" % (padding,))
    if pad != "EXPLICIT" and len(explicit_paddings) != 0:
        raise InvalidArgumentError("explicit_paddings attribute must be empty if the padding attribute is not EXPLICIT")
    # NHWC positions; an NCHW request is rejected by the library as Unimplemented
    n_i, h_i, w_i, c_i = (0, 1, 2, 3) if data_format == "NHWC" else (0, 2, 3, 1)
    if strides[n_i] != 1 or strides[c_i] != 1:
        raise InvalidArgumentError("Current implementation does not yet support strides in the batch and depth dimensions.")
    if dilations[n_i] != 1 or dilations[c_i] != 1:
        raise InvalidArgumentError("Current implementation does not yet support dilations in the batch and depth dimensions.")
    return _lib.ConvDesc(int(input_shape[n_i]), int(input_shape[h_i]), int(input_shape[w_i]), int(input_shape[c_i]),
                         int(filter_shape[0]), int(filter_shape[1]), int(filter_shape[2]), int(filter_shape[3]),
                         int(strides[h_i]), int(strides[w_i]), int(dilations[h_i]), int(dilations[w_i]),
                         _PADDING[pad], _FORMAT[data_format], _ACCUMULATE[accumulate], _PLAN[plan])


def conv2d_output_shape(input_shape, filter_shape, strides, padding, data_format="NHWC", dilations=(1, 1, 1, 1),
                        depthwise=False):
    """Output shape as the op's shape function gives it (tf2/src/approx_nn_conv_ops.cpp:311-404)."""
    d = _desc(input_shape, filter_shape, strides, padding, data_format, dilations, [])
    out = (C.c_int64 * 4)()
    L = _lib.load()
    fn = L.axc_depthwise_conv2d_output_dims if depthwise else L.axc_conv2d_output_dims
    raise_for_status(fn(C.byref(d), out), "output dims")
    return tuple(int(v) for v in out)


_ws_cache = collections.OrderedDict()
_ws_lock = threading.Lock()
_WS_CACHE_ENTRIES = 256
_WS_CACHE_BYTES = 1 << 30


def _workspace(device, nbytes, key):
    """Per-filter workspace for callers that do not bring their own (`workspace=`).  The library keeps the
    prepared filter (quantised copy, lookup schedule, filter sums) in it and re-uses that preparation while the
    filter values it was built from are unchanged, so every (device, stream, filter storage, shape, table) gets
    its own buffer, the way the reference's op instance owns its table (tf2/src/approx_ops_types.h:222).  A buffer
    serves one stream at a time, hence the stream in the key.  The cache is bounded in entries and in bytes; a
    caller whose filter tensor is a temporary (a new address every call) should own the buffer instead, as
    `layers.FakeApproxConv2D` does."""
    key = (device.index, torch.cuda.current_stream(device).cuda_stream) + key
    with _ws_lock:
        buf = _ws_cache.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.zeros(nbytes, dtype=torch.uint8, device=device)
            _ws_cache[key] = buf
            total = sum(b.numel() for b in _ws_cache.values())
            while len(_ws_cache) > 1 and (len(_ws_cache) > _WS_CACHE_ENTRIES or total > _WS_CACHE_BYTES):
                _, old = _ws_cache.popitem(last=False)
                total -= old.numel()
        else:
            _ws_cache.move_to_end(key)
        return buf


def workspace_bytes(input_shape, filter_shape, strides, padding, dilations=(1, 1, 1, 1), depthwise=False):
    """Bytes of device scratch a forward call of this shape needs (axc_conv2d_workspace_bytes)."""
    L = _lib.load()
    d = _desc(input_shape, filter_shape, strides, padding, "NHWC", list(dilations), [])
    wsz = C.c_size_t()
    fn = L.axc_depthwise_conv2d_workspace_bytes if depthwise else L.axc_conv2d_workspace_bytes
    raise_for_status(fn(C.byref(d), C.byref(wsz)), "workspace size")
    return int(wsz.value)


def _device_index(dev):
    """CUDA ordinal of a torch device; a device without an index means the current one."""
    return dev.index if dev.index is not None else torch.cuda.current_device()


def _forward(depthwise, input, filter, input_min, input_max, filter_min, filter_max, strides, num_bits,
             mul_map_file, padding, explicit_paddings, data_format, dilations, out, debug, accumulate="exact",
             plan="keep", workspace=None, ranges=None, bias=None, residual=None, relu=False, input_relu=False):
    L = _lib.load()
    if not isinstance(input, torch.Tensor) or not isinstance(filter, torch.Tensor):
        raise InvalidArgumentError("input and filter must be torch tensors")
    if not input.is_cuda or not filter.is_cuda:
        raise InvalidArgumentError("input and filter must live on a CUDA device (this build has no CPU kernel)")
    if input.dtype != torch.float32 or filter.dtype != torch.float32:
        raise InvalidArgumentError("only T = float is registered for the table op")
    if filter.device != input.device:
        raise InvalidArgumentError("input and filter are on different devices")
    table = _table_for(mul_map_file, num_bits)
    d = _desc(input.shape, filter.shape, strides, padding, data_format, dilations, explicit_paddings, accumulate, plan)
    dims = (C.c_int64 * 4)()
    dims_fn = L.axc_depthwise_conv2d_output_dims if depthwise else L.axc_conv2d_output_dims
    raise_for_status(dims_fn(C.byref(d), dims), "ApproxConv2D")
    oshape = tuple(int(v) for v in dims)
    dev = input.device
    x = input.contiguous()
    f = filter.contiguous()
    if out is None:
        out = torch.empty(oshape, dtype=torch.float32, device=dev)
    elif tuple(out.shape) != oshape or out.dtype != torch.float32 or not out.is_contiguous() or out.device != dev:
        raise InvalidArgumentError("out has the wrong shape, dtype, layout or device")
    wsz = C.c_size_t()
    ws_fn = L.axc_depthwise_conv2d_workspace_bytes if depthwise else L.axc_conv2d_workspace_bytes
    raise_for_status(ws_fn(C.byref(d), C.byref(wsz)), "workspace size")
    if workspace is not None:
        if (workspace.dtype != torch.uint8 or workspace.device != dev or not workspace.is_contiguous()
                or workspace.numel() < wsz.value or workspace.data_ptr() % 256):
            raise InvalidArgumentError("workspace must be a contiguous uint8 tensor on the input's device, 256-byte "
                                       "aligned, of at least %d bytes" % wsz.value)
        ws = workspace
    else:
        ws = _workspace(dev, wsz.value, (f.data_ptr(), tuple(f.shape), id(table), depthwise))
    dbg_ptr = None
    dbg_t = None
    if debug:
        kdim = int(f.shape[0] * f.shape[1] * (1 if depthwise else f.shape[2]))
        ncol = int(f.shape[2] * f.shape[3]) if depthwise else int(f.shape[3])
        dbg_t = {"qinput": torch.empty(tuple(x.shape), dtype=torch.uint8, device=dev),
                 "qfilter": torch.empty((kdim, ncol), dtype=torch.uint8, device=dev),
                 "acc": torch.empty(oshape, dtype=torch.int32, device=dev)}
        dbg = _lib.DebugOut(dbg_t["qinput"].data_ptr(), dbg_t["qfilter"].data_ptr(), dbg_t["acc"].data_ptr())
        dbg_ptr = C.byref(dbg)
    stream = torch.cuda.current_stream(dev).cuda_stream
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    four = (input_min, input_max, filter_min, filter_max)
    if ranges is not None and depthwise:
        raise InvalidArgumentError("device-resident ranges are an option of the dense op")
    if ranges is not None and (ranges.dtype != torch.float32 or ranges.device != dev or ranges.numel() != 4
                               or not ranges.is_contiguous()):
        raise InvalidArgumentError("ranges must be four contiguous fp32 values on the input's device")
    # fused additions to the output (bias of the layer, shortcut of a residual block, ReLU)
    ep_ptr, keep = None, []
    if bias is not None or residual is not None or relu or input_relu:
        for name, t, shape in (("bias", bias, (oshape[3],)), ("residual", residual, oshape)):
            if t is not None and (t.dtype != torch.float32 or t.device != dev or tuple(t.shape) != shape):
                raise InvalidArgumentError("%s must be a fp32 tensor of shape %s on the input's device" % (name, shape))
        keep = [t.contiguous() if t is not None else None for t in (bias, residual)]
        ep = _lib.Epilogue(keep[0].data_ptr() if keep[0] is not None else None,
                           keep[1].data_ptr() if keep[1] is not None else None, 1 if relu else 0, 1 if input_relu else 0)
        ep_ptr = C.byref(ep)
    if not depthwise and (ranges is not None or all(isinstance(v, torch.Tensor) and v.is_cuda for v in four)):
        # the four scalars already live on the GPU (e.g. fresh reductions): hand them over as they are, no
        # device-to-host synchronisation
        r = ranges if ranges is not None else torch.stack([v.reshape(()).to(torch.float32) for v in four]).contiguous()
        st = L.axc_conv2d_forward_fused(table.handle, C.byref(d), x.data_ptr(), f.data_ptr(), 0.0, 0.0, 0.0, 0.0, r.data_ptr(),
                                        ep_ptr, out.data_ptr(), ws.data_ptr(), ws.numel(), dbg_ptr, dev_index,
                                        C.c_void_p(stream))
    elif depthwise:
        st = L.axc_depthwise_conv2d_forward_fused(table.handle, C.byref(d), x.data_ptr(), f.data_ptr(), _scalar(input_min),
                                                  _scalar(input_max), _scalar(filter_min), _scalar(filter_max), ep_ptr,
                                                  out.data_ptr(), ws.data_ptr(), ws.numel(), dbg_ptr, dev_index,
                                                  C.c_void_p(stream))
    else:
        st = L.axc_conv2d_forward_fused(table.handle, C.byref(d), x.data_ptr(), f.data_ptr(), _scalar(input_min),
                                        _scalar(input_max), _scalar(filter_min), _scalar(filter_max), None, ep_ptr,
                                        out.data_ptr(), ws.data_ptr(), ws.numel(), dbg_ptr, dev_index, C.c_void_p(stream))
    raise_for_status(st, "ApproxConv2D", _cuda_detail() if st == 100 else "")
    if debug:
        if not depthwise:
            info = (C.c_int32 * 4)()
            raise_for_status(L.axc_conv2d_plan_info(ws.data_ptr(), info, dev_index, C.c_void_p(stream)), "plan info")
            dbg_t["plan"] = {"rebuilt": int(info[0]), "fallback": int(info[1]), "status": int(info[2]),
                             "steps_per_mille": int(info[3])}
        else:
            word = C.c_int32(-1)
            raise_for_status(L.axc_depthwise_conv2d_status(C.byref(d), ws.data_ptr(), C.byref(word), dev_index,
                                                           C.c_void_p(stream)), "depthwise status")
            dbg_t["status"] = int(word.value)
        return out, dbg_t
    return out


def approx_conv2d_with_min_max_vars(input, filter, input_min, input_max, filter_min, filter_max, strides, num_bits,
                                    mul_map_file, padding, explicit_paddings=(), data_format="NHWC",
                                    dilations=(1, 1, 1, 1), name=None, out=None, debug=False, accumulate="exact",
                                    plan="keep", workspace=None, ranges=None, bias=None, residual=None, relu=False, input_relu=False):
    """Forward pass of `ApproxConv2DWithMinMaxVars`.

    input [N,H,W,C] and filter [KH,KW,C,Cout] are fp32 CUDA tensors; the four min/max values are
    host scalars (Python floats or 0-d CPU tensors) or - all four - 0-d CUDA tensors, which are then consumed on
    the device without a host round trip; `mul_map_file` is the raw uint16[65536] table file
    ('' = exact products) or a `Table`.  Returns the fp32 output [N,OH,OW,Cout]; with `debug=True`
    also the quantised operands and the int32 accumulators.

    accumulate: "exact" (default) dequantises the exact integer sum of the looked-up products; "reference"
    reproduces the reference's fp32 running total added in K order (tf2/src/approx_nn_conv_kernels.cpp:245-246),
    whose roundings show once a partial sum passes 2^24 - the output then has the reference's bits for every K.

    plan: "keep" (default) prepares a lookup plan for the filter in the workspace and reuses it while the filter is
    unchanged; "none" is for filters that change every call (training).  workspace: a uint8 CUDA tensor of at least
    `workspace_bytes(...)` bytes that the caller keeps for this layer (default: a cache keyed by the filter's
    address).  ranges: the four range scalars as one fp32 CUDA tensor {input_min, input_max, filter_min,
    filter_max} (then the four positional range arguments are ignored and may be None).

    bias [Cout], residual (a tensor of the output's shape) and relu are fused into the kernel's dequantisation:
    y = conv; y += bias; y += residual; y = max(y, 0) - with the bits of the same steps done by separate kernels.
    input_relu: every input element counts as max(x, 0) (the ReLU of the layer that produced the input, applied by
    this call's loaders for free)."""
    return _forward(False, input, filter, input_min, input_max, filter_min, filter_max, strides, num_bits,
                    mul_map_file, padding, list(explicit_paddings), data_format, list(dilations), out, debug, accumulate,
                    plan, workspace, ranges, bias, residual, relu, input_relu)


def approx_depthwise_conv2d_with_min_max_vars(input, filter, input_min, input_max, filter_min, filter_max, strides,
                                              num_bits, mul_map_file, padding, explicit_paddings=(),
                                              data_format="NHWC", dilations=(1, 1, 1, 1), name=None, out=None,
                                              debug=False, bias=None, residual=None, relu=False, input_relu=False):
    """Depthwise variant: filter [KH,KW,C,mult] (DepthwiseConv2dNative layout), output [N,OH,OW,C*mult]."""
    return _forward(True, input, filter, input_min, input_max, filter_min, filter_max, strides, num_bits,
                    mul_map_file, padding, list(explicit_paddings), data_format, list(dilations), out, debug,
                    bias=bias, residual=residual, relu=relu, input_relu=input_relu)


def ax_conv2d(input, filter, min_input, max_input, min_filter, max_filter, strides, padding, table="",
              dilations=(1, 1, 1, 1), out=None, ax_tune=True):
    """Mirror of the reference's first-generation op `AxConv2D` (tf1/axqconv/axqconv.cc:66-94): quantised uint8
    input [N,H,W,C] and filter [KH,KW,C,Cout] with their float ranges in; returns (output int32 [N,OH,OW,Cout],
    min_output, max_output).  `table` stands for the op's AxMult attribute: a `Table` or a table file ('' = exact
    products); `ax_tune` for its AxTune attribute (default true, as there): the table's weight columns are re-mapped
    to the closest ones first (tf1/axqconv/approximate_selector.h:46-78).  The offsets are the codes of 0.0 in the
    two ranges (:365-368); the int32 output is the table sum with the functor's zero-point terms (:241-246)."""
    L = _lib.load()
    if input.dtype != torch.uint8 or filter.dtype != torch.uint8 or not input.is_cuda or not filter.is_cuda:
        raise InvalidArgumentError("input and filter must be uint8 CUDA tensors")
    tab = _table_for(table, 8)
    if ax_tune:
        tab = tab.tuned()
    d = _desc(input.shape, filter.shape, strides, padding, "NHWC", list(dilations), [])
    dims = (C.c_int64 * 4)()
    raise_for_status(L.axc_conv2d_output_dims(C.byref(d), dims), "AxConv2D")
    oshape = tuple(int(v) for v in dims)
    dev = input.device
    x, f = input.contiguous(), filter.contiguous()
    if out is None:
        out = torch.empty(oshape, dtype=torch.int32, device=dev)
    off_in, off_f = C.c_int32(), C.c_int32()
    raise_for_status(L.axc_quantized_zero_point(float(min_input), float(max_input), C.byref(off_in)), "input offset")
    raise_for_status(L.axc_quantized_zero_point(float(min_filter), float(max_filter), C.byref(off_f)), "filter offset")
    wsz = C.c_size_t()
    raise_for_status(L.axc_qconv2d_workspace_bytes(C.byref(d), C.byref(wsz)), "workspace size")
    ws = _workspace(dev, wsz.value, (f.data_ptr(), tuple(f.shape), id(tab), "q"))
    dev_index = dev.index if dev.index is not None else torch.cuda.current_device()
    st = L.axc_qconv2d_forward(tab.handle, C.byref(d), x.data_ptr(), f.data_ptr(), off_in.value, off_f.value,
                               out.data_ptr(), ws.data_ptr(), ws.numel(), dev_index,
                               C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
    raise_for_status(st, "AxConv2D", _cuda_detail() if st == 100 else "")
    rng = (C.c_float * 2)()
    raise_for_status(L.axc_quantized_output_range(float(min_input), float(max_input), float(min_filter), float(max_filter), rng),
                     "output range")
    return out, float(rng[0]), float(rng[1])


def approx_conv2d(input, filter, strides, padding, explicit_paddings=(), data_format="NHWC", dilations=(1, 1, 1, 1),
                  name=None, out=None):
    """The op the reference registers without a table and without range inputs, `ApproxConv2D`
    (tf2/src/approx_nn_ops.cpp:24-36).  There it is an fp32 convolution; here it is served by the same table path
    with the exact-product table and the ranges of the data - an 8-bit quantised convolution whose products are
    exact.  The four ranges are reduced on the device and consumed there (no host round trip)."""
    in_min, in_max = torch.aminmax(input)
    f_min, f_max = torch.aminmax(filter)
    return _forward(False, input, filter, in_min, in_max, f_min, f_max, strides, 8, "", padding, list(explicit_paddings),
                    data_format, list(dilations), out, False)


def add_residual_(out, residual, relu=True):
    """In place: out = out + residual, then ReLU - the shortcut step of a residual block in one pass."""
    if (out.dtype != torch.float32 or residual.dtype != torch.float32 or not out.is_cuda or residual.device != out.device
            or out.shape != residual.shape or not out.is_contiguous()):
        raise InvalidArgumentError("add_residual_ expects two fp32 CUDA tensors of one shape, the first contiguous")
    r = residual.contiguous()
    dev_index = out.device.index if out.device.index is not None else torch.cuda.current_device()
    st = _lib.load().axc_add_residual(out.data_ptr(), r.data_ptr(), out.numel(), 1 if relu else 0, dev_index,
                                      C.c_void_p(torch.cuda.current_stream(out.device).cuda_stream))
    raise_for_status(st, "add residual", _cuda_detail() if st == 100 else "")
    return out


def max_pool_same(x, k=3, stride=2, out=None):
    """Max pooling of an NHWC fp32 CUDA tensor, k x k window, TensorFlow's SAME padding - the pooling step of the
    ResNet workloads without a layout copy."""
    if not x.is_cuda or x.dtype != torch.float32 or x.dim() != 4:
        raise InvalidArgumentError("max_pool_same expects a 4-D fp32 CUDA tensor (NHWC)")
    x = x.contiguous()
    n, h, w, c = (int(v) for v in x.shape)
    oshape = (n, -(-h // stride), -(-w // stride), c)
    if out is None:
        out = torch.empty(oshape, dtype=torch.float32, device=x.device)
    elif tuple(out.shape) != oshape or out.dtype != torch.float32 or out.device != x.device or not out.is_contiguous():
        raise InvalidArgumentError("out must be a contiguous fp32 tensor of shape %s on the input's device" % (oshape,))
    st = _lib.load().axc_max_pool_same(x.data_ptr(), out.data_ptr(), n, h, w, c, int(k), int(stride), _device_index(x.device),
                                       C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    raise_for_status(st, "max pool", _cuda_detail() if st == 100 else "")
    return out


def tensor_range(x, out=None):
    """{min, max} of a fp32 CUDA tensor as two floats in device memory (one reduction kernel, no host round trip):
    the wrapper's reduce_min / reduce_max (tf2/python/keras/layers/fake_approx_convolutional.py:233-240)."""
    if not x.is_cuda or x.dtype != torch.float32:
        raise InvalidArgumentError("tensor_range expects a fp32 CUDA tensor")
    x = x.contiguous()
    if out is None:
        out = torch.empty(2, dtype=torch.float32, device=x.device)
    dev_index = x.device.index if x.device.index is not None else torch.cuda.current_device()
    st = _lib.load().axc_tensor_range(x.data_ptr(), x.numel(), out.data_ptr(), dev_index,
                                      C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    raise_for_status(st, "tensor range", _cuda_detail() if st == 100 else "")
    return out


def fake_quant_device_range(x, range2, out=None):
    """Forward of FakeQuantWithMinMaxVars (8 bits) with the range {min, max} read from device memory."""
    if not x.is_cuda or x.dtype != torch.float32:
        raise InvalidArgumentError("fake_quant_device_range expects a fp32 CUDA tensor")
    x = x.contiguous()
    if out is None:
        out = torch.empty_like(x)
    dev_index = x.device.index if x.device.index is not None else torch.cuda.current_device()
    st = _lib.load().axc_fake_quant(x.data_ptr(), x.numel(), range2.data_ptr(), out.data_ptr(), dev_index,
                                    C.c_void_p(torch.cuda.current_stream(x.device).cuda_stream))
    raise_for_status(st, "fake quant", _cuda_detail() if st == 100 else "")
    return out


def launch_count():
    """Kernels launched by libaxconv in this process so far."""
    return int(_lib.load().axc_launch_count())


def measure_lookup_peak(device=None):
    """Conflict-free 16-bit shared-memory loads one SM sustains, in lookups per clock (32 by construction)."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    scratch = torch.zeros(8192, dtype=torch.uint8, device=dev)
    out = C.c_double()
    st = _lib.load().axc_measure_lookup_peak(_device_index(dev), scratch.data_ptr(), scratch.numel(),
                                             C.c_void_p(torch.cuda.current_stream(dev).cuda_stream), C.byref(out))
    raise_for_status(st, "lookup peak", _cuda_detail() if st == 100 else "")
    return float(out.value)
