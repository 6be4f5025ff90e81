"""GPU: the five benchmark configurations as layer stacks.  Every convolution of the network is run on the
GPU and re-run by the CPU checker ON THE SAME INPUT TENSOR (the GPU's own activation of the previous layer),
so each layer is compared bit for bit - int32 accumulators and fp32 output - without errors compounding.
The first three tests reduce spatial size and batch so that the checker finishes in seconds; channel counts,
kernel sizes, strides and table kinds are those of the configurations.  The full-size tests run configurations 4
and 5 at their real spatial size (224x224 and 112x112) on one or two images against the checker, and at their
real batch (256 and 512) compare a slice of the batch with the same images run alone - the property batch
sharding relies on."""
import numpy as np
import pytest

from oracle import oracle as O

pytestmark = pytest.mark.gpu


def _run_network(kind, hw, batch, table_for_layer, seed_cfg):
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import workloads as W
    net = W.Network(kind, hw)
    filters = W.make_filters(net.convs, 2000 + 100 * seed_cfg)
    tables = [table_for_layer(i) for i in range(len(net.convs))]
    handles = [ax.Table(array=t) for t in tables]
    x0 = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1000 + seed_cfg)).cuda()
    checked = []

    def conv(i, x):
        spec, _ = net.convs[i]
        f = filters[i]
        lo, hi = float(x.min()), float(x.max())
        mm = (lo, hi, float(f.min()), float(f.max()))
        fn = ax.approx_depthwise_conv2d_with_min_max_vars if spec.depthwise else ax.approx_conv2d_with_min_max_vars
        y, dbg = fn(x, torch.from_numpy(f).cuda(), *mm, [1, spec.stride, spec.stride, 1], 8, handles[i], "SAME",
                    debug=True)
        xn = x.cpu().numpy()
        d = O.desc(xn.shape[0], xn.shape[1], xn.shape[2], xn.shape[3], spec.k, spec.k, f.shape[3],
                   (spec.stride, spec.stride), (1, 1), "SAME")
        if spec.depthwise:
            ref = O.depthwise_conv2d(d, tables[i], xn, f, *mm)
        else:
            ref = O.conv2d(d, tables[i], xn, f, *mm, want=("out_exact", "acc"))
        assert np.array_equal(dbg["acc"].cpu().numpy(), ref["acc"]), "layer %d (%s): accumulators" % (i, spec.name)
        assert np.array_equal(y.cpu().numpy().view(np.uint32), ref["out_exact"].view(np.uint32)), \
            "layer %d (%s): fp32 output" % (i, spec.name)
        checked.append(spec.name)
        return y

    out = net.forward(x0, conv, torch.relu, W.torch_maxpool3s2)
    assert len(checked) == len(net.convs)
    assert torch.isfinite(out).all()
    return out


def test_config3_resnet20_layers(built):
    """CIFAR ResNet-20: 3x3 convs, 16/32/64 channels, stride 2 at the stage transitions, a noisy table per layer."""
    import tf_approximate_b200 as ax
    _run_network("resnet20", 32, 4, lambda i: ax.noisy_table(3000 + 300 + i), 3)


def test_config4_resnet50_layers(built):
    """ImageNet ResNet-50 layer shapes (7x7/2 stem, 1x1/3x3/1x1 bottlenecks, widths 64..2048), truncated table;
    64x64 input instead of 224x224."""
    import tf_approximate_b200 as ax
    t = ax.truncated_table()
    _run_network("resnet50", 64, 1, lambda i: t, 4)


def test_config5_depthwise_separable_stack(built):
    """3x3 depthwise (stride 1 and 2, 32..384 channels) interleaved with 1x1 pointwise convs, noisy table;
    28x28 input instead of 112x112."""
    import tf_approximate_b200 as ax
    t = ax.noisy_table(3000 + 500)
    _run_network("mobilenet_stack", 28, 2, lambda i: t, 5)


def test_config4_resnet50_full_size_layers(built):
    """224x224 input, two images: every one of the 53 convolutions against the checker, bit for bit (the tile
    scheduling of the large layers: several rounds per CTA, main + tail launches)."""
    import tf_approximate_b200 as ax
    t = ax.truncated_table()
    _run_network("resnet50", 224, 2, lambda i: t, 4)


def test_config5_stack_full_size_layers(built):
    """112x112x32 input, one image, the per-configuration noisy table: all 14 layers against the checker."""
    import tf_approximate_b200 as ax
    t = ax.noisy_table(3000 + 500)
    _run_network("mobilenet_stack", 112, 1, lambda i: t, 5)


def _slice_equals_alone(kind, batch, table, seed_cfg, lo, hi):
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import workloads as W
    net = W.Network(kind)
    filters = W.make_filters(net.convs, 2000 + 100 * seed_cfg)
    dev = torch.device("cuda", 0)
    runner = W.GpuRunner(net, [table], filters, dev)
    x = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1000 + seed_cfg)).to(dev)
    runner.calibrate(x)                     # frozen per-layer ranges, as in the benchmark
    y_all = runner.forward(x)
    y_few = runner.forward(x[lo:hi].contiguous())
    torch.cuda.synchronize()
    assert torch.isfinite(y_all).all()
    assert torch.equal(y_all[lo:hi].view(torch.int32), y_few.view(torch.int32))


def test_config4_batch256_slice_equals_alone(built):
    """The ResNet-50 workload at its real size: images 100..103 of the batch of 256 give the bits they give alone."""
    import tf_approximate_b200 as ax
    _slice_equals_alone("resnet50", 256, ax.truncated_table(), 4, 100, 104)


def test_config5_batch512_slice_equals_alone(built):
    import tf_approximate_b200 as ax
    _slice_equals_alone("mobilenet_stack", 512, ax.noisy_table(3000 + 500), 5, 300, 303)


@pytest.mark.parametrize("kind,hw,batch", [("resnet50", 64, 2), ("resnet20", 32, 4), ("mobilenet_stack", 56, 2)])
def test_fused_epilogue_equals_separate_steps(built, kind, hw, batch):
    """Shortcut addition and ReLU fused into the convolution kernels' dequantisation give the bits of the same steps
    done by separate element-wise kernels, through the whole network."""
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import workloads as W
    net = W.Network(kind, hw)
    filters = W.make_filters(net.convs, 2000 + 100 * 4)
    dev = torch.device("cuda", 0)
    runner = W.GpuRunner(net, [ax.noisy_table(3090)], filters, dev)
    x = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1004)).to(dev)
    runner.calibrate(x)
    y_fused = runner.forward(x, fused=True)
    y_plain = runner.forward(x, fused=False)
    assert torch.isfinite(y_plain).all() and float(y_plain.abs().max()) > 0
    assert torch.equal(y_fused, y_plain)


def test_op_epilogue_bias_residual_relu(built):
    """The op-level epilogue on every kernel that has one: scheduled kernel, kernel without a plan, reference-order
    kernel, expanded-table depthwise kernel, small depthwise kernels."""
    import torch
    import tf_approximate_b200 as ax
    g = torch.Generator(device="cuda").manual_seed(9)
    t = ax.Table(array=ax.noisy_table(3091))
    x = torch.rand((2, 40, 40, 48), device="cuda", generator=g) * 2 - 1
    f = torch.randn((3, 3, 48, 72), device="cuda", generator=g) * 0.1
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    bias = torch.randn(72, device="cuda", generator=g)
    res = torch.randn((2, 40, 40, 72), device="cuda", generator=g)
    for kw in ({}, {"plan": "none"}, {"accumulate": "reference"}):
        y0 = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", **kw)
        y1 = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", bias=bias, residual=res, relu=True, **kw)
        assert torch.equal(y1, torch.relu((y0 + bias) + res)), kw
        y2 = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", relu=True, **kw)
        assert torch.equal(y2, torch.relu(y0)), kw
        # the producer's ReLU applied by this call's loaders: the bits of the call on the activated tensor
        y3 = ax.approx_conv2d_with_min_max_vars(x, f, *mm, [1, 1, 1, 1], 8, t, "SAME", input_relu=True, **kw)
        y4 = ax.approx_conv2d_with_min_max_vars(torch.relu(x), f, *mm, [1, 1, 1, 1], 8, t, "SAME", **kw)
        assert torch.equal(y3, y4) and not torch.equal(y3, y0), kw
    for shape, stride in (((2, 40, 40, 48), 1), ((2, 41, 39, 40), 2), ((1, 9, 9, 16), 1)):
        xd = torch.rand(shape, device="cuda", generator=g) * 2
        fd = torch.randn((3, 3, shape[3], 1), device="cuda", generator=g) * 0.3
        mmd = (0.0, 2.0, float(fd.min()), float(fd.max()))
        y0 = ax.approx_depthwise_conv2d_with_min_max_vars(xd, fd, *mmd, [1, stride, stride, 1], 8, t, "SAME")
        b = torch.randn(shape[3], device="cuda", generator=g)
        r = torch.randn(tuple(y0.shape), device="cuda", generator=g)
        y1 = ax.approx_depthwise_conv2d_with_min_max_vars(xd, fd, *mmd, [1, stride, stride, 1], 8, t, "SAME", bias=b, residual=r,
                                                          relu=True)
        assert torch.equal(y1, torch.relu((y0 + b) + r)), shape
        xs = xd - 1.0                                   # negative values as well
        y3 = ax.approx_depthwise_conv2d_with_min_max_vars(xs, fd, *mmd, [1, stride, stride, 1], 8, t, "SAME", input_relu=True)
        y4 = ax.approx_depthwise_conv2d_with_min_max_vars(torch.relu(xs), fd, *mmd, [1, stride, stride, 1], 8, t, "SAME")
        assert torch.equal(y3, y4), shape


def test_forward_as_cuda_graph(built):
    """After a warm-up the calls only enqueue kernels on the caller's stream, so a whole forward pass (dense layers with
    ReLUs and shortcuts riding along, depthwise layers fed by TMA) can be captured once and replayed on new inputs:
    same bits as the calls made one by one."""
    import torch
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import workloads as W
    dev = torch.device("cuda", 0)
    for kind, hw, batch in (("resnet50", 64, 2), ("mobilenet_stack", 56, 4)):
        net = W.Network(kind, hw=hw)
        filters = W.make_filters(net.convs, 2600)
        runner = W.GpuRunner(net, [ax.noisy_table(3095)], filters, dev)
        x = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1006)).to(dev)
        x2 = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1007)).to(dev)
        runner.calibrate(torch.cat([x, x2]))
        want, want2 = runner.forward(x), runner.forward(x2)
        torch.cuda.synchronize()
        replay, static_x, static_y = runner.capture(x)
        for src, ref in ((x2, want2), (x, want), (x2, want2)):
            static_x.copy_(src)
            replay()
            torch.cuda.synchronize()
            assert torch.equal(static_y.view(torch.int32), ref.view(torch.int32)), kind


def test_max_pool_same_matches_torch(built):
    """The NHWC pooling kernel against torch's max_pool2d with -inf padding placed as TensorFlow's SAME rule does."""
    import torch
    import tf_approximate_b200 as ax
    g = torch.Generator(device="cuda").manual_seed(9)
    for n, h, w, c, k, s in [(2, 112, 112, 64, 3, 2), (1, 7, 9, 5, 3, 2), (3, 8, 8, 16, 2, 2), (1, 13, 11, 12, 3, 1), (2, 1, 1, 4, 3, 2),
                             (1, 6, 5, 3, 5, 3)]:
        x = torch.randn((n, h, w, c), device="cuda", generator=g)
        oh, ow = -(-h // s), -(-w // s)
        ph, pw = max((oh - 1) * s + k - h, 0), max((ow - 1) * s + k - w, 0)
        xc = torch.nn.functional.pad(x.permute(0, 3, 1, 2), (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2), value=float("-inf"))
        want = torch.nn.functional.max_pool2d(xc, k, s).permute(0, 2, 3, 1).contiguous()
        got = ax.ops.max_pool_same(x, k, s)
        assert got.shape == want.shape and torch.equal(got, want), (n, h, w, c, k, s)
        sliced = x[:, :, :, : max(c - 1, 1)]                       # a non-contiguous view, odd channel count
        got2 = ax.ops.max_pool_same(sliced, k, s)
        assert torch.equal(got2, want[..., : max(c - 1, 1)])
    assert ax.ops.max_pool_same(torch.zeros((0, 8, 8, 4), device="cuda")).shape == (0, 4, 4, 4)
