"""The layer-level caller of the op, mirroring the reference's Keras wrapper
(tf2/python/keras/layers/fake_approx_convolutional.py): per-batch min/max, fake quantisation of
input and kernel, the table convolution, then bias and activation; the backward pass is the exact
convolution's (the reference registers `conv2d_backprop_input/filter` as the gradient, :264-302)."""
import torch

from . import ops
from .ops import approx_conv2d_with_min_max_vars


def _nudge(min_v, max_v, num_bits=8):
    """TensorFlow fake-quant range nudging (restated in the reference at tf2/src/approx_ops_types.h:29-49), in fp32
    like the op.  Works on 0-d tensors of any device, so nothing is synchronised with the host.  Returns tensors
    (nudged_min, nudged_max, scale); a zero range gives zeros (tf2/src/approx_ops_types.h:135-152)."""
    f32 = torch.float32
    mn = torch.as_tensor(min_v, dtype=f32)
    mx = torch.as_tensor(max_v, dtype=f32).to(mn.device)
    qmin = torch.zeros((), dtype=f32, device=mn.device)
    qmax = torch.full((), float((1 << num_bits) - 1), dtype=f32, device=mn.device)
    zero_range = (mn == 0) & (mx == 0)
    scale = (mx - mn) / (qmax - qmin)
    safe = torch.where(zero_range, torch.ones_like(scale), scale)
    zp_from_min = qmin - mn / safe
    rounded = torch.sign(zp_from_min) * torch.floor(torch.abs(zp_from_min) + 0.5)   # half away from zero
    zp = torch.where(zp_from_min < qmin, qmin, torch.where(zp_from_min > qmax, qmax, rounded))
    nudged_min = (qmin - zp) * safe
    nudged_max = (qmax - zp) * safe
    z = torch.zeros_like(scale)
    return (torch.where(zero_range, z, nudged_min), torch.where(zero_range, z, nudged_max),
            torch.where(zero_range, z, scale))


def fake_quant_with_min_max_vars(x, min_v, max_v, num_bits=8):
    """Forward of TensorFlow's FakeQuantWithMinMaxVars: clamp to the nudged range and snap to its grid.
    The reference applies it to input and kernel before the op
    (tf2/python/keras/layers/fake_approx_convolutional.py:233-242).  min_v / max_v may be Python floats or 0-d
    tensors on x's device (then no host synchronisation happens)."""
    mn = torch.as_tensor(min_v, dtype=torch.float32).to(x.device)
    mx = torch.as_tensor(max_v, dtype=torch.float32).to(x.device)
    nmin, nmax, scale = _nudge(mn, mx, num_bits)
    zero_range = scale == 0
    inv = torch.ones((), dtype=torch.float32, device=x.device) / torch.where(zero_range, torch.ones_like(scale), scale)
    clamped = torch.minimum(torch.maximum(x, nmin), nmax)
    q = torch.floor((clamped - nmin) * inv + 0.5)
    return torch.where(zero_range, torch.zeros_like(x), q * scale + nmin)


class _FakeQuantFn(torch.autograd.Function):
    """Fake quantisation with a device-resident range (one kernel); straight-through gradient - every element lies
    inside its own tensor's range, where TensorFlow's fake-quant gradient is the identity."""

    @staticmethod
    def forward(ctx, x, range2):
        return ops.fake_quant_device_range(x, range2)

    @staticmethod
    def backward(ctx, grad):
        return grad, None


class _ApproxConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, ranges, strides, padding, mul_map_file, num_bits, dilations, plan, workspace):
        ctx.save_for_backward(x, w)
        ctx.cfg = (strides, padding, dilations)
        return approx_conv2d_with_min_max_vars(x, w, None, None, None, None, strides=strides, num_bits=num_bits,
                                               mul_map_file=mul_map_file, padding=padding, dilations=dilations,
                                               plan=plan, workspace=workspace, ranges=ranges)

    @staticmethod
    def backward(ctx, grad):
        x, w = ctx.saved_tensors
        strides, padding, dilations = ctx.cfg
        with torch.enable_grad():
            xc = x.detach().permute(0, 3, 1, 2).requires_grad_(True)
            wc = w.detach().permute(3, 2, 0, 1).requires_grad_(True)
            kh, kw = w.shape[0], w.shape[1]
            sh, sw, dh, dw = strides[1], strides[2], dilations[1], dilations[2]
            if padding == "SAME":
                oh, ow = -(-x.shape[1] // sh), -(-x.shape[2] // sw)
                ph = max((oh - 1) * sh + (kh - 1) * dh + 1 - x.shape[1], 0)
                pw = max((ow - 1) * sw + (kw - 1) * dw + 1 - x.shape[2], 0)
                xp = torch.nn.functional.pad(xc, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2))
            else:
                xp = xc
            y = torch.nn.functional.conv2d(xp, wc, stride=(sh, sw), dilation=(dh, dw))
            gx, gw = torch.autograd.grad(y, (xc, wc), grad.permute(0, 3, 1, 2))
        return gx.permute(0, 2, 3, 1), gw.permute(2, 3, 1, 0), None, None, None, None, None, None, None, None


class FakeApproxConv2D(torch.nn.Module):
    """Conv2D whose multiplications go through a truth table
    (reference: FakeApproxConv2D, tf2/python/keras/layers/fake_approx_convolutional.py:176-261).
    Tensors are NHWC, the kernel is [KH, KW, Cin, filters]."""

    def __init__(self, in_channels, filters, kernel_size, strides=(1, 1), padding="valid", dilation_rate=(1, 1),
                 activation=None, use_bias=True, num_bits=8, mul_map_file=""):
        super().__init__()
        ks = (kernel_size, kernel_size) if isinstance(kernel_size, int) else tuple(kernel_size)
        self.strides = (strides, strides) if isinstance(strides, int) else tuple(strides)
        self.dilation_rate = (dilation_rate, dilation_rate) if isinstance(dilation_rate, int) else tuple(dilation_rate)
        self.padding = "VALID" if padding.lower() in ("valid", "causal") else padding.upper()
        self.activation = activation
        self.num_bits = num_bits
        self.mul_map_file = mul_map_file
        fan_in, fan_out = ks[0] * ks[1] * in_channels, ks[0] * ks[1] * filters
        limit = (6.0 / (fan_in + fan_out)) ** 0.5  # glorot_uniform, the Keras default
        self.kernel = torch.nn.Parameter(torch.empty(ks[0], ks[1], in_channels, filters).uniform_(-limit, limit))
        self.bias = torch.nn.Parameter(torch.zeros(filters)) if use_bias else None
        # owned by the layer, like the op instance's state in the reference: the four range scalars and the op's
        # workspace (the lookup plan of the kernel lives there between calls)
        self._ranges = None
        self._workspace = None

    def _own_buffers(self, inputs, strides4, dilations4):
        dev = inputs.device
        if self._ranges is None or self._ranges.device != dev:
            self._ranges = torch.empty(4, dtype=torch.float32, device=dev)
            self._workspace = None
        need = ops.workspace_bytes(inputs.shape, self.kernel.shape, strides4, self.padding, dilations4)
        if self._workspace is None or self._workspace.numel() < need:
            self._workspace = torch.zeros(need, dtype=torch.uint8, device=dev)
        return self._ranges, self._workspace

    def plan_info(self):
        """{rebuilt in the last call, fallback, status, steps per mille} of the lookup plan in the layer's workspace
        (blocks until the current stream is idle)."""
        import ctypes as C
        from . import _lib
        if self._workspace is None:
            return None
        info = (C.c_int32 * 4)()
        dev = self._workspace.device
        st = _lib.load().axc_conv2d_plan_info(self._workspace.data_ptr(), info, ops._device_index(dev),
                                              C.c_void_p(torch.cuda.current_stream(dev).cuda_stream))
        ops.raise_for_status(st, "plan info")
        return {"rebuilt": int(info[0]), "fallback": int(info[1]), "status": int(info[2]), "steps_per_mille": int(info[3])}

    def forward(self, inputs):
        if self.num_bits != 8:
            raise ops.InvalidArgumentError("only num_bits == 8 is supported")
        strides4 = (1, self.strides[0], self.strides[1], 1)
        dilations4 = (1, self.dilation_rate[0], self.dilation_rate[1], 1)
        ranges, workspace = self._own_buffers(inputs, strides4, dilations4)
        # per-batch ranges: one reduction kernel each, written where the op reads them - no host round trip
        ops.tensor_range(inputs.detach(), ranges[0:2])
        ops.tensor_range(self.kernel.detach(), ranges[2:4])
        q_in = _FakeQuantFn.apply(inputs, ranges[0:2])
        q_k = _FakeQuantFn.apply(self.kernel, ranges[2:4])
        # while the weights are being trained they change every step: no lookup plan then (nothing to rebuild)
        plan = "none" if (self.training and self.kernel.requires_grad) else "keep"
        y = _ApproxConvFn.apply(q_in, q_k, ranges, strides4, self.padding, self.mul_map_file, self.num_bits, dilations4,
                                plan, workspace)
        if self.bias is not None:
            y = y + self.bias
        if self.activation is not None:
            y = self.activation(y)
        return y
