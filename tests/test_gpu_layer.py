"""GPU: the layer-level caller (mirror of the reference's Keras `FakeApproxConv2D`,
tf2/python/keras/layers/fake_approx_convolutional.py:176-302): per-batch ranges, fake quantisation of input and
kernel, table convolution, bias; backward pass = the exact convolution's gradients."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_layer_forward_matches_op_and_float_conv(built):
    import torch
    import tf_approximate_b200 as ax
    torch.manual_seed(3)
    layer = ax.FakeApproxConv2D(in_channels=8, filters=12, kernel_size=3, padding="same", mul_map_file="").cuda()
    with torch.no_grad():
        layer.bias.uniform_(-0.1, 0.1)
    x = torch.rand(2, 9, 9, 8, device="cuda") * 2 - 1
    y = layer(x)
    # the same thing spelled out with the op
    xq = ax.fake_quant_with_min_max_vars(x, float(x.min()), float(x.max()))
    wq = ax.fake_quant_with_min_max_vars(layer.kernel.detach(), float(layer.kernel.detach().min()), float(layer.kernel.detach().max()))
    y_op = ax.approx_conv2d_with_min_max_vars(xq, wq, float(x.min()), float(x.max()), float(layer.kernel.detach().min()),
                                              float(layer.kernel.detach().max()), [1, 1, 1, 1], 8, "", "SAME") + layer.bias.detach()
    assert torch.equal(y.detach(), y_op)
    # exact table + fake-quantised operands = the float convolution of those operands (the reference's own test)
    ref = torch.nn.functional.conv2d(xq.permute(0, 3, 1, 2).double(), wq.permute(3, 2, 0, 1).double(), padding=1)
    ref = ref.permute(0, 2, 3, 1) + layer.bias.detach().double()
    err = float((y.detach().double() - ref).abs().max() / ref.abs().max())
    assert err < 1e-5, err


def test_layer_gradients_are_the_exact_convolutions(built):
    import torch
    import tf_approximate_b200 as ax
    torch.manual_seed(4)
    layer = ax.FakeApproxConv2D(in_channels=4, filters=6, kernel_size=3, strides=2, padding="same",
                                mul_map_file="").cuda()
    x = (torch.rand(2, 8, 8, 4, device="cuda") * 2 - 1).requires_grad_(True)
    y = layer(x)
    g = torch.randn_like(y)
    y.backward(g)
    # reference gradients: exact conv on the fake-quantised operands, straight-through to x and the kernel
    x2 = x.detach().clone().requires_grad_(True)
    w2 = layer.kernel.detach().clone().requires_grad_(True)
    xq = x2 + (ax.fake_quant_with_min_max_vars(x2, float(x2.min()), float(x2.max())) - x2).detach()
    wq = w2 + (ax.fake_quant_with_min_max_vars(w2, float(w2.min()), float(w2.max())) - w2).detach()
    xp = torch.nn.functional.pad(xq.permute(0, 3, 1, 2), (0, 1, 0, 1))   # SAME, 3x3 stride 2 on 8x8: pad 0 before, 1 after
    y2 = torch.nn.functional.conv2d(xp, wq.permute(3, 2, 0, 1), stride=2).permute(0, 2, 3, 1)
    y2.backward(g)
    assert torch.allclose(x.grad, x2.grad, atol=1e-5, rtol=1e-5)
    assert torch.allclose(layer.kernel.grad, w2.grad, atol=1e-5, rtol=1e-5)
    assert torch.allclose(layer.bias.grad, g.sum(dim=(0, 1, 2)), atol=1e-5)


def test_tensor_range_and_fake_quant_kernels(built):
    """The device-side prologue: one reduction kernel for {min, max}, one kernel for the fake quantisation with the
    range read from device memory - against torch.aminmax and the element-wise torch restatement, bit for bit."""
    import torch
    from tf_approximate_b200 import ops
    import tf_approximate_b200 as ax
    g = torch.Generator(device="cuda").manual_seed(11)
    for n, lo, hi in [(2, -1.0, 1.0), (7, 0.5, 2.0), (1000, -3.0, -1.0), (4097, -1.0, 1.0), (3 * 1024 * 1024 + 5, -2.0, 5.0)]:
        x = torch.rand(n + 1, device="cuda", generator=g)[1:] * (hi - lo) + lo     # an unaligned view as well
        for t in (x, x.clone()):
            r = ops.tensor_range(t)
            mn, mx = torch.aminmax(t)
            assert float(r[0]) == float(mn) and float(r[1]) == float(mx), n
            fq = ops.fake_quant_device_range(t, r)
            want = ax.fake_quant_with_min_max_vars(t, float(mn), float(mx))
            assert torch.equal(fq.view(torch.int32), want.view(torch.int32)), n
    z = torch.zeros(100, device="cuda")
    r = ops.tensor_range(z)
    assert float(r[0]) == 0.0 and float(r[1]) == 0.0
    assert torch.equal(ops.fake_quant_device_range(z, r), z)             # zero range: all zeros


def test_layer_keeps_its_plan_between_calls(built):
    """The layer owns its workspace: in evaluation mode the lookup plan is built by the first forward pass and found
    intact by the following ones, although the fake-quantised kernel is a new temporary every time; in training mode
    no plan is built at all (the weights change every step) and the output has the same bits."""
    import torch
    import tf_approximate_b200 as ax
    torch.manual_seed(5)
    layer = ax.FakeApproxConv2D(in_channels=16, filters=40, kernel_size=3, padding="same", mul_map_file="").cuda().eval()
    xs = [torch.rand(2, 12, 12, 16, device="cuda") * 2 - 1 for _ in range(4)]
    outs = []
    with torch.no_grad():
        for i, x in enumerate(xs):
            junk = torch.empty(1 << (10 + i), device="cuda")          # perturbs the allocator between calls
            outs.append(layer(x))
            info = layer.plan_info()
            assert info["status"] == 0 and info["fallback"] == 0 and info["steps_per_mille"] >= 1000
            assert info["rebuilt"] == (1 if i == 0 else 0), (i, info)
            del junk
    layer.train()
    y_train = layer(xs[0])
    assert torch.equal(y_train.detach().view(torch.int32), outs[0].view(torch.int32))
