"""The layer-level caller of the op, mirroring the reference's Keras wrapper
(tf2/python/keras/layers/fake_approx_convolutional.py): per-batch min/max, fake quantisation of
input and kernel, the table convolution, then bias and activation; the backward pass is the exact
convolution's (the reference registers `conv2d_backprop_input/filter` as the gradient, :264-302)."""
import torch

from .ops import approx_conv2d_with_min_max_vars


def _nudge(min_v, max_v, num_bits=8):
    """TensorFlow fake-quant range nudging (restated in the reference at tf2/src/approx_ops_types.h:29-49),
    in fp32 like the op."""
    f32 = torch.float32
    qmin, qmax = 0.0, float((1 << num_bits) - 1)
    mn = torch.as_tensor(min_v, dtype=f32)
    mx = torch.as_tensor(max_v, dtype=f32)
    scale = (mx - mn) / torch.tensor(qmax - qmin, dtype=f32)
    zp_from_min = torch.tensor(qmin, dtype=f32) - mn / scale
    zp = torch.where(zp_from_min < qmin, torch.tensor(qmin), torch.where(
        zp_from_min > qmax, torch.tensor(qmax), torch.sign(zp_from_min) * torch.floor(torch.abs(zp_from_min) + 0.5)))
    nudged_min = (torch.tensor(qmin, dtype=f32) - zp) * scale
    nudged_max = (torch.tensor(qmax, dtype=f32) - zp) * scale
    return float(nudged_min), float(nudged_max), float(scale)


def fake_quant_with_min_max_vars(x, min_v, max_v, num_bits=8):
    """Forward of TensorFlow's FakeQuantWithMinMaxVars: clamp to the nudged range and snap to its grid.
    The reference applies it to input and kernel before the op
    (tf2/python/keras/layers/fake_approx_convolutional.py:233-242)."""
    min_v = float(min_v)
    max_v = float(max_v)
    if min_v == 0.0 and max_v == 0.0:
        return torch.zeros_like(x)
    nmin, nmax, scale = _nudge(min_v, max_v, num_bits)
    inv = torch.tensor(1.0, dtype=torch.float32) / torch.tensor(scale, dtype=torch.float32)
    clamped = torch.clamp(x, nmin, nmax)
    q = torch.floor((clamped - nmin) * float(inv) + 0.5)
    return q * scale + nmin


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
        input_min, input_max = float(inputs.detach().min()), float(inputs.detach().max())
        q_in = fake_quant_with_min_max_vars(inputs, input_min, input_max, self.num_bits)
        k_min, k_max = float(self.kernel.detach().min()), float(self.kernel.detach().max())
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
