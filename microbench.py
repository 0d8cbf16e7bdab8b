"""Per-operator measurements on one B200 for the workloads next to the headline benchmark: the quantized MLP, the fused
LSTM-cell elementwise group, the MatMulInteger / QLinearMatMul sweep, MobileNetV2, QuantizeLinear / DequantizeLinear and
single depthwise layers.  One JSON line per measurement on stdout.

    python microbench.py [mlp] [eltwise] [gemm] [mobilenet] [quant] [depthwise] [nchw] [prepare] [onnx] [stem[=BATCH]]

`bench.py` imports `secondary()` from here for the `secondary` block of its JSON line.

Timing: CUDA events on the launching stream, 3 warm-up calls, median of 10 (3 for the largest GEMMs), a 256 MB buffer
rewritten between calls so that nothing is served from L2.  `gbs` is algorithmic bytes (every input read once, every
output written once) per second; `frac_hbm` divides it by the measured copy bandwidth of MEASURED_PEAKS.json when that file
is next to bench.py (else by the 6.65 TB/s fallback)."""
import json
import os
import sys

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def hbm_peak_gbs():
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


NOMINAL_HBM_GBS = 8000.0    # the figure the benchmark specification quotes for B200
NOMINAL_INT8_TOPS = 4500.0  # NVIDIA's dense int8 figure for B200


def run(which, dev, emit_line=None, gemm_sizes=(1024, 4096, 8192, 16384), mobilenet_cuda_cores=True):
    """Runs the measurements named in `which` on `dev`; returns the list of result dicts (and passes each to emit_line)."""
    pkg = entry.load_package()
    from chainer_compiler_b200 import fusion, models, ops
    from chainer_compiler_b200._lib import check
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    peak, peak_src = hbm_peak_gbs()
    results = []

    def timeit(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return float(np.median(ts))

    def emit(name, ms, **kw):
        line = {"bench": name, "ms": ms}
        line.update(kw)
        if "gbs" in kw:
            line["frac_hbm"] = kw["gbs"] / peak
            line["hbm_peak"] = "%s %.0f GB/s" % (peak_src, peak)
            line["frac_hbm_nominal_8tbs"] = kw["gbs"] / NOMINAL_HBM_GBS
        if "tops" in kw:
            line["frac_nominal_int8_4500"] = kw["tops"] / NOMINAL_INT8_TOPS
        results.append(line)
        if emit_line is not None:
            emit_line(line)

    if "quant" in which:
        # the ResNet-50 input batch (a 40 us kernel: launch ramp and tail are ~10 % of it) and a 1.3 GB stream
        for n, label in ((256 * 3 * 224 * 224, "38.5 M"), (1 << 28, "268 M")):
            x = torch.rand(n, device=dev)
            ms = timeit(lambda: ops.QuantizeLinear(x, 1 / 255.0, np.uint8(0)))
            emit("QuantizeLinear f32->u8, %s elements, round half up (reference)" % label, ms, gbs=n * 5 / ms / 1e6)
            ms = timeit(lambda: ops.QuantizeLinear(x, 1 / 255.0, np.uint8(0), round_mode=1))
            emit("QuantizeLinear f32->u8, %s elements, round half to even" % label, ms, gbs=n * 5 / ms / 1e6)
            q = ops.QuantizeLinear(x, 1 / 255.0, np.uint8(0))
            ms = timeit(lambda: ops.DequantizeLinear(q, 1 / 255.0, np.uint8(0)))
            emit("DequantizeLinear u8->f32, %s elements" % label, ms, gbs=n * 5 / ms / 1e6)
            del x, q

    if "eltwise" in which:
        nodes = fusion.lstm_cell_group()
        g = fusion.fuse_elementwise(nodes, {}, ["c_next", "h"])[0]
        code = fusion.build_program(nodes, 1, g.inputs, g.outputs)
        ins = [torch.randn((4096, 4096), device=dev) for _ in g.inputs]
        ms = timeit(lambda: ops.ElementWiseNvrtc(ins, 2, code, 1))
        emit("ElementWiseNvrtc LSTM cell, 5 inputs + 2 outputs of fp32 [4096,4096]", ms, gbs=7 * 4096 * 4096 * 4 / ms / 1e6)

    if "gemm" in which:
        for S in gemm_sizes:
            a = torch.randint(0, 256, (S, S), dtype=torch.uint8, device=dev)
            b = torch.randint(-127, 128, (S, S), dtype=torch.int8, device=dev)
            za = torch.tensor([128], dtype=torch.uint8, device=dev)
            it = 3 if S >= 8192 else 10
            ms = timeit(lambda: ops.MatMulInteger(a, b, za, None, path=2), iters=it)
            emit("MatMulInteger u8[%d,%d] (zp 128) x s8[%d,%d] -> s32" % (S, S, S, S), ms, tops=2 * S ** 3 / ms / 1e9)
            ms = timeit(lambda: ops.QLinearMatMul(a, 0.01, np.uint8(128), b, 0.001, np.int8(0), 1e-3 * S, np.uint8(0), path=2), iters=it)
            emit("QLinearMatMul u8[%d,%d] (zp 128) x s8[%d,%d] -> u8" % (S, S, S, S), ms, tops=2 * S ** 3 / ms / 1e9)

    if "mlp" in which:
        net = models.QuantizedMLP(dev, seed=0)
        x = torch.rand((64, 784), generator=torch.Generator().manual_seed(0)).to(dev)
        ms = timeit(lambda: net.forward(x))
        emit("quantized MLP 784-1000-1000-10, batch 64, five ops per call", ms, samples_per_s=64 / ms * 1e3)
        ms = timeit(lambda: net.forward_packed(x))
        emit("quantized MLP, batch 64, weights packed once (MatMuls as packed 1x1 convolutions)", ms, samples_per_s=64 / ms * 1e3)
        net.forward_packed(x)
        torch.cuda.synchronize()
        gp = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gp):
            yp = net.forward_packed(x)
        ms = timeit(gp.replay)
        emit("quantized MLP, batch 64, weights packed once, replayed from a CUDA graph", ms, samples_per_s=64 / ms * 1e3)
        # the same five kernels replayed from a CUDA graph: what is left when the host's per-op work is taken away
        net.forward(x)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            y = net.forward(x)
        ms = timeit(g.replay)
        emit("quantized MLP 784-1000-1000-10, batch 64, five kernels replayed from a CUDA graph", ms, samples_per_s=64 / ms * 1e3)

    if "mobilenet" in which:
        B = 512
        x = torch.rand((B, 3, 224, 224), generator=torch.Generator().manual_seed(1)).to(dev)
        # default: 3x3 depthwise layers on the CUDA-core row kernel (rows staged by TMA); second run (on request): all of them as
        # diagonal blocks on the tensor cores (chxq_tc_variant 3)
        for variant in ((0, 3) if mobilenet_cuda_cores else (0,)):
            check(pkg.lib().chxq_tc_variant(variant))
            net = models.MobileNetV2Int8(B, dev, seed=0)
            net.calibrate(x)
            graph, logits = net.capture(x, fold=True)
            ms = timeit(graph.replay)
            dense, dw = net.macs_per_image()
            emit("MobileNetV2-1.0 int8, batch 512, depthwise on %s, folded requantization" % ("tensor cores (diagonal blocks)" if variant else "CUDA cores (row-dp4a kernel, TMA-staged rows)"), ms,
                 img_per_s=B / ms * 1e3, gmac_per_image=(dense + dw) / 1e9)
            del net, graph, logits
            torch.cuda.empty_cache()
        check(pkg.lib().chxq_tc_variant(0))

    if "depthwise" in which:
        N = 512
        for C, H, s in ((96, 112, 2), (144, 56, 1), (384, 14, 1), (960, 7, 1)):
            x = torch.randint(0, 256, (N, C, H, H), dtype=torch.uint8, device=dev).contiguous(memory_format=torch.channels_last)
            w = torch.randint(-127, 128, (C, 1, 3, 3), dtype=torch.int8, device=dev)
            ws = torch.full((C,), 1e-3, device=dev)
            wz = torch.zeros(C, dtype=torch.int8, device=dev)
            y = ops.QLinearConv(x, 0.02, np.uint8(0), w, ws, wz, 0.05, np.uint8(0), None, (s, s), (1, 1), C)
            nbytes = x.numel() + y.numel()
            ms = timeit(lambda: ops.QLinearConv(x, 0.02, np.uint8(0), w, ws, wz, 0.05, np.uint8(0), None, (s, s), (1, 1), C))
            emit("depthwise 3x3 QLinearConv C%d %dx%d stride %d batch %d, op signature, reference-order requantization (row-dp4a kernel, rows staged by TMA)" % (C, H, H, s, N), ms, gbs=nbytes / ms / 1e6)
            pk = ops.PackedConv(w, wz, x.shape, (s, s), (1, 1), group=C)
            ms = timeit(lambda: ops.QLinearConvPacked(x, pk, 0.02, np.uint8(0), ws, wz, 0.05, np.uint8(0), fold_scales=True))
            emit("depthwise 3x3 QLinearConv C%d %dx%d stride %d batch %d, packed entry, the library's choice" % (C, H, H, s, N), ms, gbs=nbytes / ms / 1e6)
            check(pkg.lib().chxq_tc_variant(3))
            ms = timeit(lambda: ops.QLinearConvPacked(x, pk, 0.02, np.uint8(0), ws, wz, 0.05, np.uint8(0), fold_scales=True))
            check(pkg.lib().chxq_tc_variant(0))
            emit("depthwise 3x3 QLinearConv C%d %dx%d stride %d batch %d, packed entry, tensor cores (diagonal blocks) on request" % (C, H, H, s, N), ms,
                 gbs=nbytes / ms / 1e6)
    if "nchw" in which:
        # the literal drop-in call of the reference's op (NCHW in, NCHW out, unpacked weights) on a res3 3x3 layer, beside the
        # packed NHWC entry the benchmark network uses
        N, C, H = 256, 128, 28
        x = torch.randint(0, 256, (N, C, H, H), dtype=torch.uint8, device=dev)
        w = torch.randint(-127, 128, (C, C, 3, 3), dtype=torch.int8, device=dev)
        ws = torch.full((C,), 1e-3, device=dev)
        wz = torch.zeros(C, dtype=torch.int8, device=dev)
        ms = timeit(lambda: ops.QLinearConv(x, 0.02, np.uint8(0), w, ws, wz, 0.05, np.uint8(0), None, (1, 1), (1, 1)))
        emit("QLinearConv 3x3 C128 28x28 batch 256, NCHW in / NCHW out through the op signature (transposes + tensor cores)", ms,
             tops=2 * N * H * H * C * C * 9 / ms / 1e9)
        ms = timeit(lambda: ops.QLinearConv(x, 0.02, np.uint8(0), w, ws, wz, 0.05, np.uint8(0), None, (1, 1), (1, 1), path=1))
        emit("the same call on the general CUDA-core kernel", ms, tops=2 * N * H * H * C * C * 9 / ms / 1e9)
        xl = x.contiguous(memory_format=torch.channels_last)
        pk = ops.PackedConv(w, wz, x.shape, (1, 1), (1, 1))
        ms = timeit(lambda: ops.QLinearConvPacked(xl, pk, 0.02, np.uint8(0), ws, wz, 0.05, np.uint8(0)))
        emit("the same layer through the packed NHWC entry", ms, tops=2 * N * H * H * C * C * 9 / ms / 1e9)
    if "prepare" in which:
        # model preparation: batch-norm folding + per-channel int8 weight quantization of every ResNet-50 convolution
        import time
        net_shapes = [(64, 3, 7, 7)]
        cin = 64
        for width, blocks in ((64, 3), (128, 4), (256, 6), (512, 3)):
            for b in range(blocks):
                net_shapes += [(width, cin, 1, 1), (width, width, 3, 3), (width * 4, width, 1, 1)]
                if b == 0:
                    net_shapes.append((width * 4, cin, 1, 1))
                cin = width * 4
        rng = np.random.default_rng(0)
        host = [(rng.standard_normal(s, dtype=np.float32) * 0.05) for s in net_shapes]
        bns = [tuple(rng.uniform(0.5, 1.5, s[0]).astype(np.float32) for _ in range(4)) for s in net_shapes]
        devw = [torch.from_numpy(w).to(dev) for w in host]
        devbn = [tuple(torch.from_numpy(v).to(dev) for v in bn) for bn in bns]
        nw = sum(w.size for w in host)

        def on_device():
            for w, bn in zip(devw, devbn):
                ops.PrepareWeights(w, bn, None, 2e-5, True, True)
        ms = timeit(on_device)
        emit("batch-norm folding + int8 per-channel weight quantization, %d convolutions of ResNet-50 (%.1f M weights), device" % (len(host), nw / 1e6),
             ms, weights_per_s=nw / ms * 1e3, launches=2 * len(host))
        t0 = time.perf_counter()
        for w, bn in zip(host, bns):
            g, be, mu, var = bn
            s = (g / np.sqrt(var + np.float32(2e-5))).astype(np.float32)
            models.quantize_weights((w * s.reshape(-1, 1, 1, 1)).astype(np.float32), per_channel=True, to_int8=True)
        emit("the same on one host core (NumPy merge + the library's host quantizer)", (time.perf_counter() - t0) * 1e3)
    for token in sorted(which):
        if token != "stem" and not token.startswith("stem="):
            continue
        # the head of ResNet-50 on a uint8 image batch: 7x7 / 2 stem convolution (64 channels) and 3x3 / 2 max pooling, as two
        # calls and as one
        from chainer_compiler_b200 import _lib as L
        B = int(token.split("=")[1]) if "=" in token else 256
        rng = np.random.default_rng(0)
        xq = torch.randint(0, 256, (B, 3, 224, 224), dtype=torch.uint8, device=dev)
        w = torch.from_numpy(rng.integers(-127, 128, (64, 3, 7, 7)).astype(np.int8)).to(dev)
        wz = torch.zeros(64, dtype=torch.int8, device=dev)
        ws = torch.full((64,), 1e-3, device=dev)
        bias = torch.zeros(64, dtype=torch.int32, device=dev)
        pk = ops.PackedConv(w, wz, xq.shape, (2, 2), (3, 3), x_layout=L.NCHW)
        args = (pk, 1 / 255.0, np.uint8(0), ws, wz, 0.05, np.uint8(0))
        ms = timeit(lambda: ops.QLinearConvPacked(xq, *args, b=bias, fold_scales=True))
        emit("stem 7x7/2 QLinearConv, batch %d: space-to-depth repack + tensor-core kernel (halo tiles)" % B, ms)
        y = ops.QLinearConvPacked(xq, *args, b=bias, fold_scales=True)
        ms = timeit(lambda: ops.MaxPoolU8(y, 3, 2, 0, cover_all=True))
        emit("3x3/2 MaxPool of the stem output, batch %d" % B, ms, gbs=(y.numel() * 1.25) / ms / 1e6)
        ms = timeit(lambda: ops.QLinearConvMaxPoolPacked(xq, *args, b=bias, cover_all=True, fold_scales=True))
        emit("stem QLinearConv + MaxPool as one call, batch %d" % B, ms)
        del xq, y

    if "onnx" in which:
        # the run_onnx entry point on a statically quantized ResNet-50 file (written from the calibrated hand-built network):
        # Elapsed as the reference's tool reports it, inputs staged on the device before the clock starts
        import tempfile
        from chainer_compiler_b200 import onnx_io, run_onnx
        B = 256
        net = models.ResNet50Int8(B, dev, seed=0)
        x = torch.rand((B, 3, 224, 224), generator=torch.Generator().manual_seed(1))
        net.calibrate(x.to(dev))
        want = net.forward(x.to(dev), fused=True, fold=True).cpu().numpy()
        with tempfile.TemporaryDirectory() as d:
            onnx_io.write_test_dir(d, net.to_onnx(), [({"x": x.numpy()}, [("logits", want)])])
            del net
            torch.cuda.empty_cache()
            for extra in ([], ["--fold_scales"], ["--fold_scales", "--cuda_graph"]):
                rep = os.path.join(d, "report.json")
                rc = run_onnx.run_onnx(["--test", d, "-I", "20", "--rtol", "1e-2", "--atol", "%g" % (1e-2 * float(np.abs(want).max())), "--report_json", rep, "-q"]
                                       + extra)
                r = json.load(open(rep))
                emit("run_onnx --test <int8 ResNet-50 directory, batch 256> -I 20 %s" % " ".join(extra), r["best_ms"], avg_ms=r["elapsed_ms"],
                     img_per_s=B / r["best_ms"] * 1e3, outputs_within_tolerance=(rc == 0))
    ops.device_status()
    del pkg, flush
    torch.cuda.empty_cache()
    return results


def secondary(dev):
    """The workloads beside the headline benchmark, for the `secondary` block of bench.py's JSON line: QuantizeLinear /
    DequantizeLinear and the fused LSTM-cell group in GB/s (against the measured copy bandwidth and against the nominal
    8 TB/s), the MatMulInteger / QLinearMatMul sweep in TOPS, MobileNetV2 batch 512 in img/s and depthwise layers in GB/s."""
    return run({"quant", "eltwise", "gemm", "mobilenet", "depthwise", "mlp", "nchw"}, dev, mobilenet_cuda_cores=False)


def gemm_sharded():
    """The MatMulInteger sweep with the rows of A sharded over the ranks of a torchrun job (B replicated, no gather inside the
    timed region: the product stays sharded, as a following row-wise operator would consume it); rank 0 prints one line per
    size with the aggregate TOPS (max over ranks of the CUDA-event time).  Run as
        python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 microbench.py gemm_sharded"""
    import torch.distributed as dist
    entry.load_package()
    from chainer_compiler_b200 import dataparallel as dp, ops
    rank, local_rank, world = dp.init()
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)
    for S in (4096, 8192, 16384):
        b0, e0 = dp.shard_bounds(S, world, rank)
        gen = torch.Generator(device=dev).manual_seed(S)  # the same B on every rank
        b = torch.randint(-127, 128, (S, S), dtype=torch.int8, device=dev, generator=gen)
        a = torch.randint(0, 256, (e0 - b0, S), dtype=torch.uint8, device=dev)
        za = torch.tensor([128], dtype=torch.uint8, device=dev)
        fn = lambda: dp.sharded_matmul_integer(a, b, za, None, total_rows=S, world=world, rank=rank, gather=False)  # noqa: E731
        for _ in range(3):
            fn()
        ts = []
        for _ in range(5):
            flush.zero_()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize(dev)
            e_a, e_b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e_a.record()
            fn()
            e_b.record()
            torch.cuda.synchronize(dev)
            ts.append(dp.max_over_ranks(e_a.elapsed_time(e_b), dev, world))
        ms = float(np.median(ts))
        if rank == 0:
            print(json.dumps({"bench": "MatMulInteger %d^3, rows of A sharded over %d GPU(s), B replicated" % (S, world), "ms": ms,
                              "tops": 2 * S ** 3 / ms / 1e9, "n_gpus": world}), flush=True)
        del a, b
    ops.device_status()
    if world > 1:
        dist.destroy_process_group()


def main():
    if "gemm_sharded" in sys.argv[1:]:
        return gemm_sharded()
    if not torch.cuda.is_available():
        raise SystemExit("microbench.py needs a CUDA device: this package has no CPU path")
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    which = set(sys.argv[1:]) or {"mlp", "eltwise", "gemm", "mobilenet", "quant", "depthwise", "prepare", "onnx", "stem", "nchw"}
    run(which, dev, emit_line=lambda line: print(json.dumps(line), flush=True))


if __name__ == "__main__":
    main()
