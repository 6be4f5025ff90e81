"""The layer-level caller of the op, mirroring the reference's Keras wrapper
(tf2/python/keras/layers/fake_approx_convolutional.py): per-batch min/max, fake quantisation of
input and kernel, the table convolution, then bias and activation; the backward pass is the exact
convolution's (the reference registers `conv2d_backprop_input/filter` as the gradient, :264-302)."""
import torch

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


class _ApproxConvFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, mins_maxs, strides, padding, mul_map_file, num_bits, dilations):
        ctx.save_for_backward(x, w)
        ctx.cfg = (strides, padding, dilations)
        return approx_conv2d_with_min_max_vars(x, w, *mins_maxs, strides=strides, num_bits=num_bits,
                                               mul_map_file=mul_map_file, padding=padding, dilations=dilations)

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
        return gx.permute(0, 2, 3, 1), gw.permute(2, 3, 1, 0), None, None, None, None, None, None


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

    def forward(self, inputs):
        # per-batch ranges stay on the device: 0-d tensors, consumed by the op without a host round trip
        input_min, input_max = torch.aminmax(inputs.detach())
        q_in = fake_quant_with_min_max_vars(inputs, input_min, input_max, self.num_bits)
        k_min, k_max = torch.aminmax(self.kernel.detach())
        q_k = fake_quant_with_min_max_vars(self.kernel, k_min, k_max, self.num_bits)
        # straight-through estimator for the fake-quant steps, as TF's fake-quant gradient inside the range
        q_in = inputs + (q_in - inputs).detach()
        q_k = self.kernel + (q_k - self.kernel).detach()
        y = _ApproxConvFn.apply(q_in, q_k, (input_min, input_max, k_min, k_max),
                                (1, self.strides[0], self.strides[1], 1), self.padding, self.mul_map_file,
                                self.num_bits, (1, self.dilation_rate[0], self.dilation_rate[1], 1))
        if self.bias is not None:
            y = y + self.bias
        if self.activation is not None:
            y = self.activation(y)
        return y
