"""Benchmark of the table-driven convolution path on the ResNet-50-shaped workload.

  python bench.py [--gpus N] [--steps K] [--warmup W]            this build (CUDA, one process per GPU)
  python bench.py --impl reference [--steps K] [--warmup W]      the reference's CPU kernels on host cores

A step is one forward pass over one batch: the 53 convolutions of an ImageNet-shaped ResNet-50
(every one a table convolution with the truncated truth table, batch 256 per GPU) plus the ReLU /
residual / max-pool glue.  `value` is table MACs per second of the whole job with the batch already in
HBM; `e2e` repeats the measurement with the batch in pinned host memory, copied in every step, and the
result copied back.  Prints one JSON line on rank 0.
"""
import argparse
import json
import multiprocessing as mp
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

SM_COUNT = 148
LOOKUPS_PER_CLK_PER_SM = 32   # one 32-bit shared-memory bank transaction per lane per clock
NCU_DRAM_OVER_ALGORITHMIC = (205.0 + 162.1) / 411.2


# name -> (description for `config.workload`, default batch per GPU, input description, configuration number)
# Seeds follow the configuration number: 1000+cfg (input), 2000+100*cfg+layer (filters), 3000+100*cfg+layer (tables).
WORKLOADS = {
    "resnet50": ("resnet50_approx_conv (BASELINE config 4): ImageNet-shaped ResNet-50 v1.5, 53 table "
                 "convolutions, truncated truth table, random He-init filters, frozen per-layer ranges",
                 256, "224x224x3 fp32 NHWC", 4),
    "resnet20": ("resnet20_approx_conv (BASELINE config 3): CIFAR-shaped ResNet-20, 3x3 table convolutions with "
                 "16/32/64 channels, a seeded noisy truth table per layer, random He-init filters, frozen per-layer "
                 "ranges", 1024, "32x32x3 fp32 NHWC", 3),
    "mobilenet_stack": ("mobilenet_stack_approx_conv (BASELINE config 5): 3x3 depthwise + 1x1 pointwise table "
                        "convolutions, 32-384 channels at 112/56/28/14, seeded noisy truth table, random He-init "
                        "filters, frozen per-layer ranges", 512, "112x112x32 fp32 NHWC", 5),
}


def build_params(kind):
    """(network, filters, truth tables: one for all layers or one per layer, configuration number)."""
    from tf_approximate_b200 import workloads as W
    import tf_approximate_b200 as ax
    cfg = WORKLOADS[kind][3]
    net = W.Network(kind)
    filters = W.make_filters(net.convs, 2000 + 100 * cfg)
    if kind == "resnet50":
        tables = [ax.truncated_table()]
    elif kind == "resnet20":
        tables = [ax.noisy_table(3000 + 100 * cfg + i) for i in range(len(net.convs))]
    else:
        tables = [ax.noisy_table(3000 + 100 * cfg)]
    return net, filters, tables, cfg


# ------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the reference's CPU kernels (oracle/_ref) or the C restatement
# ------------------------------------------------------------------------------------------------
def _cpu_worker(args):
    """One image through all convolutions on one host core.  Returns (seconds, macs, kind)."""
    kind, seed = args
    os.environ["OMP_NUM_THREADS"] = "1"
    from tf_approximate_b200 import workloads as W
    from oracle import oracle as O
    import tf_approximate_b200 as ax
    net, filters, tables, _ = build_params(kind)
    x = W.make_input(1, net.hw, net.in_channels, seed)
    # the reference's kernels have no depthwise path: such a workload is timed with the restatement
    use_ref = O.ref_available() and not any(spec.depthwise for spec, _ in net.convs)
    tmps, ops = [], []
    if use_ref:
        for lut in tables:
            tmp = tempfile.NamedTemporaryFile(suffix=".bin", delete=False)
            tmp.close()
            ax.write_table(tmp.name, lut)
            tmps.append(tmp.name)
            ops.append(O.RefOp(tmp.name))

    def conv(spec, table_index, xx, f, lo, hi, flo, fhi):
        lo, hi = float(xx.min()), float(xx.max())   # per-call range: a single image calibrates itself
        d = O.desc(xx.shape[0], xx.shape[1], xx.shape[2], xx.shape[3], f.shape[0], f.shape[1], f.shape[3],
                   (spec.stride, spec.stride), (1, 1), "SAME")
        if spec.depthwise:
            return O.depthwise_conv2d(d, tables[table_index], xx, f, lo, hi, flo, fhi, nthreads=1)["out_ref"]
        if use_ref:
            return ops[table_index].conv2d(d, xx, f, lo, hi, flo, fhi)
        return O.conv2d(d, tables[table_index], xx, f, lo, hi, flo, fhi, want=("out_ref",), nthreads=1)["out_ref"]

    runner = W.CpuRunner(net, filters, [(0.0, 0.0)] * len(filters), conv, shared_table=len(tables) == 1)
    t0 = time.perf_counter()
    runner.forward(x)
    dt = time.perf_counter() - t0
    for op, name in zip(ops, tmps):
        op.close()
        os.unlink(name)
    return dt, net.macs_per_image(), "reference" if use_ref else "port"


def run_cpu(kind, steps, warmup, workers=None):
    """Each step: `workers` images, one per process, through the reference's single-threaded kernels."""
    workers = workers or max(1, min(os.cpu_count() or 1, 32))
    ctx = mp.get_context("spawn")
    times, macs, impl_kind = [], 0, "port"
    with ctx.Pool(workers) as pool:
        for s in range(warmup + steps):
            res = pool.map(_cpu_worker, [(kind, 1000 + WORKLOADS[kind][3] + 17 * i) for i in range(workers)])
            if s >= warmup:
                times.append(max(r[0] for r in res))   # the workers run side by side: slowest forward pass
            macs = sum(r[1] for r in res)
            impl_kind = res[0][2]
    sec = sum(times) / len(times)
    return {"value": macs / sec, "unit": "LUT-MAC/s", "cores": workers, "kind": impl_kind,
            "sample": "%d images of the same %s forward per step, one per process (the reference's "
                      "kernels are single-threaded)" % (workers, kind),
            "seconds_per_step": sec, "images_per_s": workers / sec, "macs_per_step": macs}


# ------------------------------------------------------------------------------------------------
# clocks
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile(suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu_index), "--query-gpu=" + self.FIELDS,
                                          "--format=csv,noheader,nounits", "-lms", "100"], stdout=f,
                                         stderr=subprocess.DEVNULL)
            f.close()
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, reasons, smax = [], set(), None
        try:
            for line in open(self.path):
                p = [v.strip() for v in line.split(",")]
                if len(p) < 9:
                    continue
                try:
                    sm.append(float(p[1]))
                    smax = float(p[2])
                except ValueError:
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), p[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            busy = [v for v in sm if v >= 0.5 * max(sm)]
            out.update(sm_mhz=statistics.median(busy), sm_max_mhz=smax, reasons=sorted(reasons), samples=len(sm))
        return out


# ------------------------------------------------------------------------------------------------
# this build
# ------------------------------------------------------------------------------------------------
def run_gpu(args):
    import torch
    import torch.distributed as dist
    import tf_approximate_b200 as ax
    from tf_approximate_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    net, filters, tables, cfg = build_params(args.workload)
    batch = args.batch if args.batch else WORKLOADS[args.workload][1]
    runner = W.GpuRunner(net, tables, filters, dev)
    if args.unfused:       # shortcut additions and ReLUs as separate element-wise kernels instead of inside the convolutions
        fused_forward = runner.forward
        runner.forward = lambda xx: fused_forward(xx, fused=False)
    x_host = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1000 + cfg + rank)).pin_memory()
    x = x_host.to(dev)

    # Frozen per-layer input ranges: calibrated on rank 0's batch, identical on every rank, so that
    # no collective sits on the compute path.
    from tf_approximate_b200 import parallel
    if rank == 0:
        runner.calibrate(x)
    runner.in_ranges = parallel.broadcast_ranges(runner.in_ranges, src=0)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        y = runner.forward(x)
    barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # ---- timed region 1: batch resident in HBM --------------------------------------------------
    runner.conv_events = []
    launches0 = ax.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(args.steps):
        y = runner.forward(x)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = ax.launch_count() - launches0
    conv_events, runner.conv_events = runner.conv_events, None

    # ---- timed region 2: end to end from pinned host memory ----------------------------------------
    # Every step copies its batch from pinned host memory and its result back.  The copies run on streams of
    # their own (two device input buffers), so the copy of the next batch and the read-back of the last result
    # overlap with the convolutions, as a serving loop would arrange it; all of it lies between f0 and f1.
    y_host = torch.empty(tuple(y.shape), dtype=y.dtype).pin_memory()
    main = torch.cuda.current_stream()
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    x_bufs = [torch.empty_like(x), torch.empty_like(x)]

    def e2e_steps(steps, start_event):
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        s_in.wait_event(start_event)
        with torch.cuda.stream(s_in):
            x_bufs[0].copy_(x_host, non_blocking=True)
            ready[0].record(s_in)
        for i in range(steps):
            b = i & 1
            if i + 1 < steps:
                if i >= 1:
                    s_in.wait_event(consumed[b ^ 1])     # the forward pass that read this buffer has finished
                with torch.cuda.stream(s_in):
                    x_bufs[b ^ 1].copy_(x_host, non_blocking=True)
                    ready[b ^ 1].record(s_in)
            main.wait_event(ready[b])
            out = runner.forward(x_bufs[b])
            consumed[b].record(main)
            s_out.wait_event(consumed[b])
            with torch.cuda.stream(s_out):
                y_host.copy_(out, non_blocking=True)
            out.record_stream(s_out)
        main.wait_stream(s_out)
        main.wait_stream(s_in)

    warm = torch.cuda.Event()
    warm.record(main)
    e2e_steps(2, warm)
    barrier()
    f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    f0.record(main)
    e2e_steps(args.steps, f0)
    f1.record(main)
    barrier()
    ms_e2e = f0.elapsed_time(f1)

    # ---- timed region 3 (N > 1): ONE batch of the workload's size cut into contiguous slabs, one per GPU ------
    # ("batch 256 sharded across 1/2/4/8 GPUs"): the same seeded global batch on every rank, rank r keeps
    # parallel.shard_batch(x).  Then, separately timed and never inside the convolution timing, the optional
    # all-gather of the final output over NCCL.
    ms_strong, ms_gather, gather_bytes, shard = ms_total, 0.0, 0, batch
    if world > 1:
        x_glob = torch.from_numpy(W.make_input(batch, net.hw, net.in_channels, 1000 + cfg))
        x_s = parallel.shard_batch(x_glob, world, rank).to(dev)
        shard = int(x_s.shape[0])
        del x_glob
        for _ in range(max(args.warmup, 3)):
            y_s = runner.forward(x_s)
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        g0.record()
        for _ in range(args.steps):
            y_s = runner.forward(x_s)
        g1.record()
        barrier()
        ms_strong = g0.elapsed_time(g1)
        y_all = parallel.gather_outputs(y_s)          # warm-up of the collective (communicator set-up)
        h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        h0.record()
        for _ in range(args.steps):
            y_all = parallel.gather_outputs(y_s)
        h1.record()
        barrier()
        ms_gather = h0.elapsed_time(h1)
        gather_bytes = y_all.numel() * 4
    # ---- timed region 4: the step of region 1 captured once as a CUDA graph and replayed ----------------------
    # (after their first call the library's calls only enqueue kernels on the caller's stream, so a serving loop can
    # replay the whole forward pass with one launch; reported beside the headline, which stays the call-by-call figure)
    ms_graph = 0.0
    if not args.no_graph:
        gstream = torch.cuda.Stream()
        replay, static_x, static_y = runner.capture(x, stream=gstream)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(gstream):
            for _ in range(max(args.warmup, 3)):
                replay()
        gstream.synchronize()
        barrier()
        with torch.cuda.stream(gstream):
            k0.record()
            for _ in range(args.steps):
                replay()
            k1.record()
        gstream.synchronize()
        barrier()
        ms_graph = k0.elapsed_time(k1)
        graph_equal = bool(torch.equal(static_y, runner.forward(x)))
        del replay, static_x, static_y
    clocks = sampler.stop() if rank == 0 else None

    t = torch.tensor([ms_total, ms_e2e, ms_strong, ms_gather, ms_graph], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total, ms_e2e, ms_strong, ms_gather, ms_graph = (float(v) for v in t)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    macs_step = net.macs_per_image() * batch * world
    ms_step = ms_total / args.steps
    value = macs_step / (ms_step * 1e-3)

    # per-layer conv time on rank 0 (filter preparation + main kernel), from the same timed region
    per_layer = {}
    for i, a, b in conv_events:
        per_layer[i] = per_layer.get(i, 0.0) + a.elapsed_time(b)
    dense_ms = sum(v for i, v in per_layer.items() if not net.convs[i][0].depthwise) / args.steps
    dense_macs = sum(W.conv_macs(s, h, batch) for s, h in net.convs if not s.depthwise)
    dense_launches = sum(1 for s, _ in net.convs if not s.depthwise)
    io_bytes = sum(W.conv_io_bytes(s, h, batch) for s, h in net.convs if not s.depthwise)
    sm_mhz = clocks["sm_mhz"] or 1965.0
    achieved = dense_macs / (dense_ms * 1e-3)
    peak = SM_COUNT * LOOKUPS_PER_CLK_PER_SM * sm_mhz * 1e6
    # the same peak measured on this GPU: conflict-free 16-bit shared-memory loads per clock and SM (one short kernel)
    measured_per_clk = ax.measure_lookup_peak(dev)
    peak_measured = SM_COUNT * measured_per_clk * sm_mhz * 1e6
    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except Exception:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    # DRAM bytes per launch: ncu on the single 3x3 layer N=256, 56x56x64->64 read 205.0 MB and wrote 162.1 MB
    # against 411.2 MB algorithmic; the whole step is too large to capture, so the measured ratio is applied to
    # the average algorithmic bytes of a launch here.
    traffic = NCU_DRAM_OVER_ALGORITHMIC * io_bytes / dense_launches
    slowest = sorted(per_layer.items(), key=lambda kv: -kv[1])[:3]
    roofline = {
        "kernel": "dense_sched_kernel (table convolution, %d convolution calls per step)" % dense_launches,
        "bound": "smem_lookup",
        "achieved": achieved / 1e9, "peak": peak / 1e9, "unit": "GLUT-MAC/s", "frac": achieved / peak,
        "peak_basis": "148 SMs x 32 shared-memory lookups/clk x %.0f MHz (median SM clock sampled during this run); "
                      "%.0f GLUT-MAC/s at the 1965 MHz maximum" % (sm_mhz, SM_COUNT * 32 * 1965e6 / 1e9),
        "peak_measured": peak_measured / 1e9, "frac_of_measured": achieved / peak_measured,
        "peak_measured_basis": "%.2f conflict-free 16-bit shared-memory loads per clock and SM, measured in this run "
                               "by axc_measure_lookup_peak (512 threads per SM, 16 independent loads per thread and "
                               "iteration), x 148 SMs x the sampled clock" % measured_per_clk,
        "units_per_launch": dense_macs / dense_launches, "ms_per_launch": dense_ms / dense_launches,
        "traffic": traffic, "traffic_unit": "bytes per launch (scaled from an ncu capture of one layer)",
        "hbm": {"algorithmic_bytes_per_step": io_bytes, "achieved_gbs": io_bytes / (dense_ms * 1e-3) / 1e9,
                "peak_gbs": hbm_peak, "frac": io_bytes / (dense_ms * 1e-3) / 1e9 / hbm_peak,
                "peak_source": "measured" if "hbm_gbs" in peaks else "fallback"},
        "slowest_layers_ms": [[net.convs[i][0].name, v / args.steps] for i, v in slowest],
    }
    if args.per_layer:
        roofline["layers"] = [[net.convs[i][0].name, net.convs[i][1], net.convs[i][0].cin, net.convs[i][0].cout,
                               net.convs[i][0].k, net.convs[i][0].stride, per_layer[i] / args.steps,
                               W.conv_macs(net.convs[i][0], net.convs[i][1], batch) / (per_layer[i] / args.steps * 1e-3)
                               / (SM_COUNT * sm_mhz * 1e6)] for i in sorted(per_layer)]

    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        cpu = run_cpu(args.workload, 1, 0)

    in_bytes = x_host.numel() * 4
    out_bytes = y_host.numel() * 4
    ms_e2e_step = ms_e2e / args.steps
    line = {
        "metric": "lut_macs_per_s", "value": value, "unit": "LUT-MAC/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u8 operands, u16 table entries, i32 accumulate", "data": "synthetic",
        "config": {"workload": WORKLOADS[args.workload][0],
                   "batch_per_gpu": batch, "global_batch": batch * world, "input": WORKLOADS[args.workload][2],
                   "parallelism": "dp%d (batch shards, per-GPU table replica, no collective in the step)" % world,
                   "l2": "not flushed: every layer's input and output are larger than the 126 MB L2"},
        "images_per_s": batch * world / (ms_step * 1e-3),
        "conv_only_lut_macs_per_s_rank0": achieved,
        "strong_bs%d" % batch: {
            "what": "one batch of %d images cut into contiguous slabs of %d per GPU (parallel.shard_batch), same "
                    "frozen ranges, no collective in the step" % (batch, shard),
            "scaling": "strong", "global_batch": batch, "batch_per_gpu": shard,
            "ms_per_step": ms_strong / args.steps,
            "value": net.macs_per_image() * batch / (ms_strong / args.steps * 1e-3), "unit": "LUT-MAC/s",
            "images_per_s": batch / (ms_strong / args.steps * 1e-3),
            "output_gather": None if world == 1 else {
                "what": "all-gather of the final layer's output over NCCL (parallel.gather_outputs), timed on its own",
                "ms": ms_gather / args.steps, "bytes_gathered_per_rank": gather_bytes,
                "algbw_gbs": gather_bytes / (ms_gather / args.steps * 1e-3) / 1e9}},
        "cuda_graph": None if args.no_graph else {
            "what": "the same step captured once as a CUDA graph and replayed (one launch per forward pass)",
            "ms_per_step": ms_graph / args.steps, "value": macs_step / (ms_graph / args.steps * 1e-3), "unit": "LUT-MAC/s",
            "images_per_s": batch * world / (ms_graph / args.steps * 1e-3), "same_bits_as_the_calls": graph_equal},
        "e2e": {"value": macs_step / (ms_e2e_step * 1e-3), "unit": "LUT-MAC/s", "ms_per_step": ms_e2e_step,
                "images_per_s": batch * world / (ms_e2e_step * 1e-3),
                "h2d_bytes_per_step": in_bytes * world, "d2h_bytes_per_step": out_bytes * world},
        "gpu_launches": int(launches),
        "clocks": clocks,
        "roofline": roofline,
    }
    if cpu is not None:
        line["cpu_baseline"] = cpu
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_layer(args):
    """One convolution, repeated: `--layer N,H,W,C,K,Cout,stride[,dw]` (SAME padding, seeded inputs as in the
    single-layer configurations: input uniform[-1,1], filter normal(0,0.1), input range [-1,1])."""
    import torch
    import tf_approximate_b200 as ax
    v = args.layer.split(",")
    n, h, w, c, k, cout, stride = (int(t) for t in v[:7])
    dw = len(v) > 7 and v[7] == "dw"
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(1002)
    x = torch.rand((n, h, w, c), device=dev, generator=g) * 2 - 1
    f = torch.randn((k, k, c, 1 if dw else cout), device=dev, generator=g) * 0.1
    lut = {"truncated": ax.truncated_table(), "noisy": ax.noisy_table(3202), "exact": ax.exact_table()}[args.table]
    table = ax.Table(array=lut)
    mm = (-1.0, 1.0, float(f.min()), float(f.max()))
    fn = ax.approx_depthwise_conv2d_with_min_max_vars if dw else ax.approx_conv2d_with_min_max_vars
    kw = {} if dw else {"accumulate": args.accumulate}
    if args.via_layer and not dw:
        # the layer-level caller: per-batch range reductions and fake quantisation on the device, then the op with
        # device-resident ranges; "train": the weights count as changing every step (no lookup plan is kept)
        layer = ax.FakeApproxConv2D(c, cout, k, strides=stride, padding="same", use_bias=False, mul_map_file=table).to(dev)
        with torch.no_grad():
            layer.kernel.copy_(f)
        layer.train(args.via_layer == "train")

        def fn(x_, f_, *a, **k_):      # noqa: F811 - same call shape as the op
            with torch.no_grad():
                return layer(x_)
    if args.quantised and not dw:
        # the first-generation op's contract: uint8 codes in, int32 sums with zero-point terms out (weight tuning is a
        # transformation of the table, done once, outside the timed calls)
        xq = torch.randint(0, 256, (n, h, w, c), device=dev, generator=g, dtype=torch.uint8)
        fq = torch.randint(0, 256, (k, k, c, cout), device=dev, generator=g, dtype=torch.uint8)
        x, f = xq, fq
        mm = (-1.0, 1.0, -0.5, 0.5)
        tuned = table.tuned()

        def fn(x_, f_, a, b, c_, d, strides, bits, tab, pad, out=None, **k_):      # noqa: F811 - same call shape as the op
            return ax.ax_conv2d(x_, f_, a, b, c_, d, strides, pad, table=tuned, out=out, ax_tune=False)[0]
    out = None
    for _ in range(args.warmup):
        out = fn(x, f, *mm, [1, stride, stride, 1], 8, table, "SAME", out=out, **kw)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        out = fn(x, f, *mm, [1, stride, stride, 1], 8, table, "SAME", out=out, **kw)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    oh, ow = -(-h // stride), -(-w // stride)
    macs = n * oh * ow * k * k * c * (1 if dw else cout)
    io = x.numel() * x.element_size() + out.numel() * out.element_size() + f.numel() * f.element_size()
    print(json.dumps({"layer": args.layer, "table": args.table, "accumulate": args.accumulate, "via_layer": args.via_layer,
                      "quantised": bool(args.quantised),
                      "ms": ms, "lut_macs": macs,
                      "glut_macs_per_s": macs / ms / 1e6, "lookups_per_clk_per_sm_at_1965MHz": macs / (ms * 1e-3) / (SM_COUNT * 1965e6),
                      "io_gbs": io / ms / 1e6}))


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = run_cpu(args.workload, args.steps, max(args.warmup, 0))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    line = {
        "impl": "reference", "metric": "lut_macs_per_s", "value": r["value"], "unit": "LUT-MAC/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["seconds_per_step"] * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "u8 operands, u16 table entries, fp32 accumulate", "data": "synthetic",
        "config": {"workload": "%s, bounded sample: %s" % (WORKLOADS[args.workload][0].split(":")[0], r["sample"])},
        "images_per_s": r["images_per_s"],
        "cpu_baseline": {k: r[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": r["value"], "unit": "LUT-MAC/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="images per GPU (default: the workload's own batch)")
    ap.add_argument("--workload", default="resnet50", choices=["resnet50", "resnet20", "mobilenet_stack"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true", help="skip the CUDA-graph replay of the step")
    ap.add_argument("--per-layer", action="store_true", help="add per-layer times and lookups/clk/SM to the JSON line")
    ap.add_argument("--layer", default=None, help="time one layer instead: N,H,W,C,K,Cout,stride[,dw]")
    ap.add_argument("--table", default="truncated", choices=["truncated", "noisy", "exact"])
    ap.add_argument("--unfused", action="store_true",
                    help="run shortcut additions and ReLUs as separate element-wise kernels (default: fused into the convolutions)")
    ap.add_argument("--via-layer", default=None, choices=["eval", "train"],
                    help="--layer only: time the layer-level caller (range reductions + fake quantisation + op)")
    ap.add_argument("--quantised", action="store_true",
                    help="--layer only: time the uint8-in / int32-out entry point (first-generation op) on random codes")
    ap.add_argument("--accumulate", default="exact", choices=["exact", "reference"],
                    help="--layer only: exact integer sum (default) or the reference's fp32 running total in K order")
    args = ap.parse_args()
    if args.layer:
        run_layer(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_gpu(args)


if __name__ == "__main__":
    main()
