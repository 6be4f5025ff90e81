"""Synthetic workloads in the shapes the benchmark configurations name: random-init networks whose
every convolution is the table-driven op.  No dataset is involved; inputs are seeded uniform[-1,1]
tensors, filters are seeded He-scaled normals, and each layer's input range is calibrated once and
then frozen (the wrapper's per-batch reduce_min/max, tf2/python/keras/layers/fake_approx_convolutional.py:
233-242, would be a cross-GPU reduction under batch sharding).

The forward harness is backend-agnostic: `gpu` runs the CUDA op on torch tensors, `cpu` takes any
callable conv(x, f, mins_maxs, stride, padding, table_index) on numpy arrays (the tests and the CPU
baseline pass the checker there)."""
import numpy as np


class ConvSpec:
    __slots__ = ("name", "cin", "cout", "k", "stride", "depthwise", "relu")

    def __init__(self, name, cin, cout, k, stride=1, depthwise=False, relu=True):
        self.name, self.cin, self.cout, self.k, self.stride = name, cin, cout, k, stride
        self.depthwise, self.relu = depthwise, relu


def out_hw(h, stride):
    return -(-h // stride)  # SAME padding


# ---------------------------------------------------------------------------------------------------
# ResNet-50 (v1.5: the stride of a bottleneck sits on its 3x3), ImageNet shape
# ---------------------------------------------------------------------------------------------------
def resnet50_blocks():
    """[(stage, block, width, out_channels, stride, has_projection)]"""
    blocks = []
    for stage, (n, width) in enumerate([(3, 64), (4, 128), (6, 256), (3, 512)]):
        for b in range(n):
            stride = 2 if (b == 0 and stage > 0) else 1
            blocks.append((stage, b, width, width * 4, stride, b == 0))
    return blocks


def resnet50_convs(hw=224):
    """All 53 convolutions with their input size: [(ConvSpec, in_hw)]."""
    convs = [(ConvSpec("stem", 3, 64, 7, 2), hw)]
    h = out_hw(out_hw(hw, 2), 2)  # stem stride 2, then 3x3/2 max pool
    cin = 64
    for stage, b, width, cout, stride, proj in resnet50_blocks():
        tag = "s%db%d" % (stage + 1, b)
        convs.append((ConvSpec(tag + "_1x1a", cin, width, 1, 1), h))
        convs.append((ConvSpec(tag + "_3x3", width, width, 3, stride), h))
        h2 = out_hw(h, stride)
        convs.append((ConvSpec(tag + "_1x1b", width, cout, 1, 1, relu=False), h2))
        if proj:
            convs.append((ConvSpec(tag + "_proj", cin, cout, 1, stride, relu=False), h))
        cin, h = cout, h2
    return convs


def conv_macs(spec, in_hw, batch=1):
    o = out_hw(in_hw, spec.stride)
    if spec.depthwise:
        return batch * o * o * spec.cin * spec.k * spec.k
    return batch * o * o * spec.cout * spec.k * spec.k * spec.cin


def conv_io_bytes(spec, in_hw, batch=1):
    """Algorithmic HBM bytes of one layer: fp32 input + fp32 output + fp32 filter."""
    o = out_hw(in_hw, spec.stride)
    cout = spec.cin if spec.depthwise else spec.cout
    fil = spec.k * spec.k * spec.cin * (1 if spec.depthwise else spec.cout)
    return 4 * (batch * in_hw * in_hw * spec.cin + batch * o * o * cout + fil)


# ---------------------------------------------------------------------------------------------------
# CIFAR ResNet-20 and the depthwise-separable stack
# ---------------------------------------------------------------------------------------------------
def resnet20_convs(hw=32):
    convs = [(ConvSpec("stem", 3, 16, 3, 1), hw)]
    cin, h = 16, hw
    for stage, width in enumerate([16, 32, 64]):
        for b in range(3):
            stride = 2 if (b == 0 and stage > 0) else 1
            convs.append((ConvSpec("s%db%d_a" % (stage + 1, b), cin, width, 3, stride), h))
            h = out_hw(h, stride)
            convs.append((ConvSpec("s%db%d_b" % (stage + 1, b), width, width, 3, 1, relu=False), h))
            cin = width
    return convs


def mobilenet_stack_convs(hw=112):
    """dw32@112 s1, pw32->96; dw96@112 s2, pw96->144@56; dw144@56 s1, pw144->144; dw144@56 s2,
    pw144->192@28; dw192@28 s1, pw192->192; dw192@28 s2, pw192->384@14; dw384@14 s1, pw384->384."""
    plan = [(32, 1, 96), (96, 2, 144), (144, 1, 144), (144, 2, 192), (192, 1, 192), (192, 2, 384), (384, 1, 384)]
    convs, h = [], hw
    for i, (c, s, co) in enumerate(plan):
        convs.append((ConvSpec("dw%d" % i, c, c, 3, s, depthwise=True), h))
        h = out_hw(h, s)
        convs.append((ConvSpec("pw%d" % i, c, co, 1, 1), h))
    return convs


# ---------------------------------------------------------------------------------------------------
# parameters
# ---------------------------------------------------------------------------------------------------
def make_filters(convs, seed_base):
    """He-scaled normal filters, HWIO (depthwise: [k,k,C,1]), seeded per layer."""
    out = []
    for i, (spec, _) in enumerate(convs):
        rng = np.random.Generator(np.random.PCG64(seed_base + i))
        if spec.depthwise:
            shape, fan = (spec.k, spec.k, spec.cin, 1), spec.k * spec.k
        else:
            shape, fan = (spec.k, spec.k, spec.cin, spec.cout), spec.k * spec.k * spec.cin
        out.append(rng.normal(0.0, np.sqrt(2.0 / fan), shape).astype(np.float32))
    return out


def make_input(batch, hw, channels, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    return rng.uniform(-1.0, 1.0, (batch, hw, hw, channels)).astype(np.float32)


# ---------------------------------------------------------------------------------------------------
# forward harnesses
# ---------------------------------------------------------------------------------------------------
class Network:
    """A stack of table convolutions with frozen per-layer ranges.

    kind: "resnet50" | "resnet20" | "mobilenet_stack".  `conv(i, x)` runs layer i on x and is supplied by
    the backend; the glue (ReLU, residual add, max pool) is written once against an array namespace
    that is either torch or numpy."""

    def __init__(self, kind, hw=None):
        self.kind = kind
        if kind == "resnet50":
            self.hw = hw or 224
            self.convs = resnet50_convs(self.hw)
            self.in_channels = 3
        elif kind == "resnet20":
            self.hw = hw or 32
            self.convs = resnet20_convs(self.hw)
            self.in_channels = 3
        elif kind == "mobilenet_stack":
            self.hw = hw or 112
            self.convs = mobilenet_stack_convs(self.hw)
            self.in_channels = 32
        else:
            raise ValueError(kind)
        self.index = {spec.name: i for i, (spec, _) in enumerate(self.convs)}

    def macs_per_image(self):
        return sum(conv_macs(s, h) for s, h in self.convs)

    def io_bytes(self, batch):
        return sum(conv_io_bytes(s, h, batch) for s, h in self.convs)

    def forward(self, x, conv, relu, maxpool3s2, fused=False):
        """conv(i, x) -> y;  relu(x) -> x;  maxpool3s2(x) -> x (3x3, stride 2, SAME).
        fused=True: the backend's conv takes (i, x, input_relu=bool, relu=bool, residual=tensor or None).  A ReLU that
        follows a convolution is then not executed where it stands: the tensor is passed on as "ReLU pending" and the
        convolution that consumes it applies max(x, 0) while loading (free for the lookup kernels); a shortcut addition
        with its ReLU is one pass of the backend.  Where a pending tensor is needed as it is (as a shortcut, as the
        network's output) the ReLU is executed.  Max pooling commutes with the ReLU.  Same arithmetic either way."""
        ix = self.index

        def mat(xp):
            t, pending = xp
            return relu(t) if pending else t

        def c(i, xp, act=False, res=None):
            t, pending = xp
            if not fused:
                y = conv(i, mat(xp))
                if res is not None:
                    y = y + mat(res)
                return (relu(y) if act else y, False)
            if res is not None:
                return (conv(i, t, input_relu=pending, relu=act, residual=mat(res)), False)
            return (conv(i, t, input_relu=pending, relu=False, residual=None), act)

        xp = (x, False)
        if self.kind == "resnet50":
            t, pending = c(ix["stem"], xp, act=True)
            xp = (maxpool3s2(t), pending)
            for stage, b, width, cout, stride, proj in resnet50_blocks():
                tag = "s%db%d" % (stage + 1, b)
                y = c(ix[tag + "_1x1a"], xp, act=True)
                y = c(ix[tag + "_3x3"], y, act=True)
                sc = c(ix[tag + "_proj"], xp) if proj else xp
                xp = c(ix[tag + "_1x1b"], y, act=True, res=sc)
            return mat(xp)
        if self.kind == "resnet20":
            xp = c(ix["stem"], xp, act=True)
            for stage in range(3):
                for b in range(3):
                    tag = "s%db%d" % (stage + 1, b)
                    first = self.convs[ix[tag + "_a"]][0]
                    y = c(ix[tag + "_a"], xp, act=True)
                    sc = xp
                    if first.stride != 1 or first.cin != first.cout:
                        # option-A shortcut: subsample, zero-pad the new channels (both commute with a pending ReLU)
                        sc = (_pad_channels(xp[0][:, ::first.stride, ::first.stride, :], first.cout), xp[1])
                    xp = c(ix[tag + "_b"], y, act=True, res=sc)
            return mat(xp)
        for i in range(len(self.convs)):
            xp = c(i, xp, act=True)
        return mat(xp)


def _pad_channels(x, c):
    if isinstance(x, np.ndarray):
        out = np.zeros(x.shape[:3] + (c,), x.dtype)
        out[..., :x.shape[3]] = x
        return out
    import torch
    return torch.nn.functional.pad(x, (0, c - x.shape[3]))


def np_relu(x):
    return np.maximum(x, 0.0)


def np_maxpool3s2(x):
    n, h, w, c = x.shape
    oh, ow = out_hw(h, 2), out_hw(w, 2)
    ph = max((oh - 1) * 2 + 3 - h, 0)
    pw = max((ow - 1) * 2 + 3 - w, 0)
    xp = np.full((n, h + ph, w + pw, c), -np.inf, x.dtype)
    xp[:, ph // 2:ph // 2 + h, pw // 2:pw // 2 + w, :] = x
    out = np.full((n, oh, ow, c), -np.inf, x.dtype)
    for ky in range(3):
        for kx in range(3):
            out = np.maximum(out, xp[:, ky:ky + (oh - 1) * 2 + 1:2, kx:kx + (ow - 1) * 2 + 1:2, :])
    return out


def gpu_maxpool3s2(x):
    """3x3, stride 2, SAME on an NHWC CUDA tensor: the library's pooling kernel (no layout copy)."""
    from . import ops
    return ops.max_pool_same(x, 3, 2)


def torch_maxpool3s2(x):
    import torch
    n, h, w, c = x.shape
    oh, ow = out_hw(h, 2), out_hw(w, 2)
    ph = max((oh - 1) * 2 + 3 - h, 0)
    pw = max((ow - 1) * 2 + 3 - w, 0)
    xc = x.permute(0, 3, 1, 2)  # a channels-last view: no copy
    xc = torch.nn.functional.pad(xc, (pw // 2, pw - pw // 2, ph // 2, ph - ph // 2), value=float("-inf"))
    y = torch.nn.functional.max_pool2d(xc, 3, 2)
    return y.permute(0, 2, 3, 1).contiguous()


class GpuRunner:
    """Runs a Network with the CUDA op.  Filters, tables and ranges live on one device."""

    def __init__(self, net, tables, filters, device):
        import torch
        import tf_approximate_b200 as ax
        self.ax, self.torch, self.net, self.device = ax, torch, net, device
        self.tables = [ax.Table(array=t) for t in tables]       # one per layer, or a single shared one
        for t in self.tables:
            t.ensure_device(device.index or 0)
        self.filters = [torch.from_numpy(f).to(device) for f in filters]
        self.f_ranges = [(float(f.min()), float(f.max())) for f in filters]
        self.in_ranges = [None] * len(filters)
        self.calibrating = False
        self.conv_events = None   # when a list: (start, end) CUDA events around every conv call

    def _conv(self, i, x, input_relu=False, relu=False, residual=None):
        spec, _ = self.net.convs[i]
        if self.calibrating:
            seen = self.torch.relu(x) if input_relu else x
            self.in_ranges[i] = (float(seen.min()), float(seen.max()))
        lo, hi = self.in_ranges[i]
        table = self.tables[i if len(self.tables) > 1 else 0]
        fn = (self.ax.approx_depthwise_conv2d_with_min_max_vars if spec.depthwise
              else self.ax.approx_conv2d_with_min_max_vars)
        if self.conv_events is not None:
            e0 = self.torch.cuda.Event(enable_timing=True)
            e1 = self.torch.cuda.Event(enable_timing=True)
            e0.record()
        # a shortcut (with its ReLU) is added by the library's one-pass kernel right after the convolution - outside the
        # convolution's event pair, so that the per-layer times stay those of the table convolution
        y = fn(x, self.filters[i], lo, hi, self.f_ranges[i][0], self.f_ranges[i][1],
               [1, spec.stride, spec.stride, 1], 8, table, "SAME", input_relu=input_relu, relu=relu and residual is None)
        if self.conv_events is not None:
            e1.record()
            self.conv_events.append((i, e0, e1))
        if residual is not None:
            self.ax.ops.add_residual_(y, residual, relu=relu)
        return y

    def calibrate(self, x):
        self.calibrating = True
        try:
            self.forward(x)
        finally:
            self.calibrating = False

    def forward(self, x, fused=True):
        """fused: shortcut additions and ReLUs inside the convolution kernels (default) or as separate torch kernels."""
        return self.net.forward(x, self._conv, self.torch.relu, gpu_maxpool3s2 if fused else torch_maxpool3s2, fused=fused)

    def capture(self, x, stream=None, warmup=2):
        """The forward pass of a batch shaped like `x` as a CUDA graph: returns (replay, static_input, static_output).
        Copy a batch into `static_input`, call `replay()`, read `static_output`.  The ranges must be calibrated.  The
        warm-up calls leave everything a call needs outside the stream in place (table replicas, lookup plans in the
        cached workspaces), so that the captured calls only enqueue kernels."""
        torch = self.torch
        stream = stream or torch.cuda.Stream(device=self.device)
        static_x = x.clone()
        stream.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(stream):
            for _ in range(warmup):
                self.forward(static_x)
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            static_y = self.forward(static_x)
        return graph.replay, static_x, static_y


class CpuRunner:
    """Runs a Network on numpy arrays with a caller-supplied convolution
    conv(spec, table_index, x, f, in_min, in_max, f_min, f_max) -> y."""

    def __init__(self, net, filters, in_ranges, conv, shared_table=True):
        self.net, self.filters, self.in_ranges, self.conv = net, filters, in_ranges, conv
        self.f_ranges = [(float(f.min()), float(f.max())) for f in filters]
        self.shared_table = shared_table

    def _conv(self, i, x):
        spec, _ = self.net.convs[i]
        lo, hi = self.in_ranges[i]
        return self.conv(spec, 0 if self.shared_table else i, x, self.filters[i], lo, hi, *self.f_ranges[i])

    def forward(self, x):
        return self.net.forward(x, self._conv, np_relu, np_maxpool3s2)
