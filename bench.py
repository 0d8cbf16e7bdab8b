"""Benchmark of the quantized-inference hot path: int8 ResNet-50 v1 inference, batch 256 per GPU, 3x224x224.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One JSON line on stdout (rank 0).  `value` is whole-job img/s with the fp32 input batch resident in HBM; `e2e` is the same
metric through the public host-buffer call (pinned host input copied in, logits copied out, inside the timed region).
Data are synthetic: uniform [0,1) images and randomly initialised weights of the ResNet-50 v1 architecture.
`--impl reference` times the reference's own algorithm for the path (dequantize -> fp32 convolution -> quantize per
QLinearConv) as restated by the CPU oracle, on the host cores, on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

IMAGE = 224
BATCH_PER_GPU = 256
METRIC = "int8 ResNet-50 img/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="chxq", choices=["chxq", "reference"])
    ap.add_argument("--batch", type=int, default=BATCH_PER_GPU, help="images per GPU")
    ap.add_argument("--cpu-sample", type=int, default=8, help="images of the CPU-baseline sample")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU baseline and the parity check that shares its sample")
    ap.add_argument("--no-secondary", action="store_true", help="skip the measurements of the workloads beside the headline")
    ap.add_argument("--no-u8-extra", action="store_true", help="skip the extra end-to-end measurement with uint8 host batches")
    ap.add_argument("--sustain-s", type=float, default=2.0, help="seconds of the sustained loop that follows the timed region")
    ap.add_argument("--tc-variant", type=int, default=0, choices=[0, 1, 2, 3, 4, 5, 6, 7],
                    help="tensor-core kernel choice (chxq_tc_variant): 0 by shape, 1 one tile per step, 2 grouped tiles")
    ap.add_argument("--no-chain", action="store_true", help="run conv2 and conv3 of every bottleneck as two kernels (default: one kernel where faster)")
    ap.add_argument("--exact-requant", action="store_true",
                    help="requantize in the reference's operation order (multiply by x_scale*w_scale, divide by y_scale) instead of one "
                         "folded multiplier per channel")
    return ap.parse_args()


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], bf16_sustained=p["bf16_tflops_sustained"], bf16_burst=p["bf16_tflops"], source="measured")
    return dict(hbm_gbs=6650.0, bf16_sustained=1400.0, bf16_burst=1590.0, source="fallback")


class ClockSampler:
    """nvidia-smi clock and throttle-reason samples while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.QUERY, "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out = self.proc.communicate(timeout=5)[0]
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out = self.proc.communicate()[0]
        sm, mx, reasons = [], [], set()
        for line in out.strip().splitlines():
            f = [v.strip() for v in line.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference_params(orc, networks, seed, sample):
    """Network parameters for the CPU arm without touching a GPU: same architecture and initialisation; activation scales
    calibrated on the sample with the oracle's own ops."""
    import __graft_entry__ as entry
    entry.load_package()
    from chainer_compiler_b200 import models
    import torch
    net = models.ResNet50Int8(batch=sample.shape[0], device="cpu", seed=seed, image=IMAGE)
    xq = orc.quantize_linear(sample, net.in_scale, 0)

    def calib(c, x, x_scale, relu):
        c.x_scale = np.float32(x_scale)
        mult = (np.float32(x_scale) * c.w_scale).astype(np.float32)
        c.bias_q = np.rint(c.b_f.astype(np.float64) / mult.astype(np.float64)).clip(-2**31, 2**31 - 1).astype(np.int32)
        acc = orc.conv_integer(x, c.w_q, 0, None, strides=(c.stride, c.stride), pads=(c.pad, c.pad))
        yf = (acc + c.bias_q.reshape(1, -1, 1, 1)).astype(np.float32) * mult.reshape(1, -1, 1, 1)
        lo, hi = float(yf.min()), float(yf.max())
        if relu:
            c.y_scale, c.y_zp = np.float32(max(hi, 1e-6) / 255.0), 0
        else:
            lo, hi = min(lo, 0.0), max(hi, 0.0)
            c.y_scale = np.float32(max(hi - lo, 1e-6) / 255.0)
            c.y_zp = int(np.clip(np.rint(-lo / float(c.y_scale)), 0, 255))
        return orc.requantize(acc, x_scale, c.w_scale, c.y_scale, c.y_zp, bias=c.bias_q, channel_axis=1)

    h = calib(net.stem, xq, net.in_scale, True)
    h = orc.maxpool_u8(h, 3, 2, 0, cover_all=True)
    h_scale = net.stem.y_scale
    for b in net.blocks:
        h1 = calib(b["conv1"], h, h_scale, True)
        h2 = calib(b["conv2"], h1, b["conv1"].y_scale, True)
        h3 = calib(b["conv3"], h2, b["conv2"].y_scale, False)
        if b["proj"] is not None:
            sc = calib(b["proj"], h, h_scale, False)
            sc_scale, sc_zp = b["proj"].y_scale, b["proj"].y_zp
        else:
            sc, sc_scale, sc_zp = h, h_scale, 0
        sf = (h3.astype(np.float32) - b["conv3"].y_zp) * b["conv3"].y_scale + (sc.astype(np.float32) - sc_zp) * np.float32(sc_scale)
        b["out_scale"] = np.float32(max(float(np.maximum(sf, 0).max()), 1e-6) / 255.0)
        b["res"] = (sc_scale, sc_zp)
        h = orc.qadd_relu(h3, b["conv3"].y_scale, b["conv3"].y_zp, sc, sc_scale, sc_zp, b["out_scale"], 0, relu=True)
        h_scale = b["out_scale"]
    net.final_scale = h_scale
    del torch
    return net.export_numpy()


def run_reference(args):
    """CPU arm: rank 0 alone works; other ranks exit 0 without work."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import __graft_entry__ as entry
    orc = entry.load_oracle()
    from oracle import networks
    # every host core this process may run on (torchrun exports OMP_NUM_THREADS=1, which is not what the reference arm is for)
    orc.set_num_threads(len(os.sched_getaffinity(0)))
    cores = orc.num_threads()
    n_img = 8 if cores >= 8 else 2
    rng = np.random.default_rng(0)
    sample = rng.uniform(0, 1, (n_img, 3, IMAGE, IMAGE)).astype(np.float32)
    params = cpu_reference_params(orc, networks, 0, sample)
    for _ in range(max(1, min(args.warmup, 2))):
        networks.resnet50_forward(params, sample, mode="emulate")
    times = []
    budget_t0 = time.perf_counter()
    for _ in range(args.steps):
        t0 = time.perf_counter()
        networks.resnet50_forward(params, sample, mode="emulate")
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - budget_t0 > 150:  # keep the whole run within a few minutes
            break
    ms = 1000.0 * float(np.mean(times))
    value = n_img / (ms / 1000.0)
    sample_txt = "%d images of 3x%dx%d per step through the oracle's QLinearConv chain (dequantize, fp32 conv, quantize), %d steps timed" % (
        n_img, IMAGE, IMAGE, len(times))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "img/s", "n_gpus": args.gpus, "steps": len(times), "warmup": args.warmup,
        "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "ResNet-50 v1 int8 inference, 3x224x224 (configs[4]); CPU sample of %d images per step" % n_img,
                   "batch_per_gpu": args.batch, "note": "the reference binary cannot be built here (ChainerX/ONNX/protobuf submodules empty); "
                   "this is the oracle restatement of its algorithm on the host cores.  The oracle's fp32 convolution is a direct loop "
                   "(OpenMP over output channels), not the im2col + GEMM a tuned native backend would run, so this is a pessimistic CPU figure.  "
                   "The arm imports this repository's models module to generate the seeded weights only (that loads libchxq.so for the host-side "
                   "weight quantizer); the timed region runs nothing but the oracle"},
        "cpu_baseline": {"value": value, "unit": "img/s", "cores": cores, "kind": "port", "sample": sample_txt},
        "e2e": {"value": value, "unit": "img/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def csrc_digest():
    """SHA-256 over the kernel sources: ties a recorded DRAM-traffic figure to the code it was captured on."""
    import glob
    import hashlib
    h = hashlib.sha256()
    for path in sorted(glob.glob(os.path.join(ROOT, "chainer-compiler_b200", "csrc", "*.cu*")) + glob.glob(os.path.join(ROOT, "chainer-compiler_b200", "csrc", "*.h"))):
        h.update(os.path.basename(path).encode())
        h.update(open(path, "rb").read())
    return h.hexdigest()


def recorded_traffic(batch, fold):
    """DRAM bytes per tensor-core launch from profiles/tc_dram_traffic.json (one ncu pass of dram__bytes_read.sum +
    dram__bytes_write.sum over the convolutions of one step), or (None, why) when the record is for other kernel sources."""
    path = os.path.join(ROOT, "profiles", "tc_dram_traffic.json")
    if not os.path.exists(path):
        return None, "no record in profiles/"
    rec = json.load(open(path))
    if rec.get("csrc_sha256") != csrc_digest():
        return None, "the record in profiles/tc_dram_traffic.json was captured on other kernel sources"
    if not fold or not rec.get("fold", True):
        return None, "the record is for the folded requantization only"
    per_launch = rec["bytes_per_step"] / rec["launches_per_step"] * (batch / float(rec["batch"]))
    note = "ncu capture at batch %d" % rec["batch"]
    if rec["batch"] != batch:
        note += ", scaled to batch %d by the images per step (activation traffic grows with the batch; the 23.5 MB of weights do not)" % batch
    return per_launch, note


def int8_probe(dev):
    """Dense int8 GEMM throughput of this GPU through the vendor library (torch._int_mm, 8192^3), best of 10: a MEASUREMENT of
    the tensor pipe's int8 peak beside the bf16 figures of MEASURED_PEAKS.json, never a product path."""
    import torch
    try:
        n = 8192
        a = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
        b = torch.randint(-127, 128, (n, n), dtype=torch.int8, device=dev)
        for _ in range(3):
            torch._int_mm(a, b)
        torch.cuda.synchronize(dev)
        best = None
        for _ in range(10):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._int_mm(a, b)
            e1.record()
            torch.cuda.synchronize(dev)
            t = e0.elapsed_time(e1)
            best = t if best is None else min(best, t)
        return 2.0 * n ** 3 / (best / 1000.0) / 1e12, None
    except Exception as exc:  # the probe is optional: say why there is no number
        return None, "%s: %s" % (type(exc).__name__, str(exc)[:120])


def h2d_ceiling(host_x, dev, world, dp, repeats=8):
    """Aggregate GB/s of plain pinned-memory host-to-device copies of one step's input, every rank copying at once and nothing
    else running: the platform's ceiling for the end-to-end number."""
    import torch
    import torch.distributed as dist
    dst = torch.empty_like(host_x, device=dev)
    dst.copy_(host_x, non_blocking=True)
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(repeats):
        dst.copy_(host_x, non_blocking=True)
    e1.record()
    torch.cuda.synchronize(dev)
    ms = dp.max_over_ranks(e0.elapsed_time(e1), dev, world) / repeats
    del dst
    return host_x.numel() * 4 * world / (ms / 1000.0) / 1e9


def run_chxq(args):
    import torch
    import torch.distributed as dist
    import __graft_entry__ as entry
    pkg = entry.load_package()
    from chainer_compiler_b200 import dataparallel as dp, models, ops
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: this package has no CPU path")
    rank, local_rank, world = dp.init()
    if world != args.gpus:
        raise SystemExit("--gpus %d does not match WORLD_SIZE %d" % (args.gpus, world))
    dev = torch.device("cuda", local_rank)
    torch.cuda.set_device(dev)
    L = pkg.lib()
    pkg._lib.check(L.chxq_tc_variant(args.tc_variant))

    # Same seeded weights on every rank; every rank works on its own seeded images (weak scaling: 256 images per GPU).
    net = models.ResNet50Int8(batch=args.batch, device=dev, seed=0, image=IMAGE)
    net.use_chain = not args.no_chain
    fold = not args.exact_requant
    gop_per_image = 2.0 * net.macs_per_image() / 1e9
    eng = dp.InferenceEngine(net, world, fold=fold, rank=rank)
    gen = torch.Generator(device="cpu").manual_seed(1234)
    calib = torch.rand((args.batch, 3, IMAGE, IMAGE), generator=gen, dtype=torch.float32)
    eng.prepare(calib.to(dev))
    gen_r = torch.Generator(device="cpu").manual_seed(99 + rank)
    host_x = dp.pinned_like((args.batch, 3, IMAGE, IMAGE), torch.float32, local_rank)
    host_x.copy_(torch.rand((args.batch, 3, IMAGE, IMAGE), generator=gen_r, dtype=torch.float32))
    eng.set_resident_input(host_x)
    ops.device_status()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # kernels per step (counted on one eager pass; a graph replay launches the same kernels)
    c0 = L.chxq_launch_count()
    net.forward(eng.x_dev, fold=fold)
    torch.cuda.synchronize(dev)
    launches_per_step = int(L.chxq_launch_count() - c0)

    def timed(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            eng.step_device()
        eng.drain()  # the last steps' logits all-gathers belong to the region
        e1.record()
        barrier()
        return dp.max_over_ranks(e0.elapsed_time(e1), dev, world)

    # ---- device-resident timed region -----------------------------------------------------------------
    for _ in range(max(3, args.warmup)):
        eng.step_device()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    ms_total = timed(args.steps)
    clocks_burst = sampler.stop() if rank == 0 else None
    ms_per_step = ms_total / args.steps
    value = args.batch * world / (ms_per_step / 1000.0)

    # ---- the same loop for >= 2 s: what the GPU sustains once it sits at its power limit ----------------------
    sustained_steps = max(args.steps, int(args.sustain_s * 1000.0 / ms_per_step) + 1)
    sampler2 = ClockSampler(local_rank)
    if rank == 0:
        sampler2.start()
    ms_sus = timed(sustained_steps)
    clocks = sampler2.stop() if rank == 0 else None
    ops.device_status()
    sus_ms_per_step = ms_sus / sustained_steps
    sustained = None
    if rank == 0:
        mhz = clocks.get("sm_mhz") if clocks else None
        sustained = {"img_s": args.batch * world / (sus_ms_per_step / 1000.0), "ms_per_step": sus_ms_per_step, "steps": sustained_steps,
                     "seconds": ms_sus / 1000.0, "sm_mhz_median": mhz, "time_x_mhz": sus_ms_per_step * mhz if mhz else None,
                     "reasons": clocks.get("reasons") if clocks else None}
        if clocks is not None:
            clocks["note"] = "sampled over the %.1f s sustained loop that follows the timed region; burst-region samples: %s" % (
                ms_sus / 1000.0, json.dumps(clocks_burst))

    # ---- end to end through the public host-buffer call ---------------------------------------------------
    # run_stream double-buffers: batch i+1 crosses PCIe while batch i computes; every step still copies its own input from
    # pinned host memory and its logits back, and the region ends when the last logits are on the host.
    for _ in eng.run_stream([host_x] * 3):
        pass
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    e0.record()
    for _ in eng.run_stream([host_x] * args.steps):
        pass
    e1.record()
    barrier()
    e2e_ms = dp.max_over_ranks(e0.elapsed_time(e1), dev, world) / args.steps
    e2e_wall_ms = 1000.0 * (time.perf_counter() - t0) / args.steps
    e2e_value = args.batch * world / (e2e_ms / 1000.0)
    h2d = host_x.numel() * 4
    d2h = eng.slots[0]["host"].numel() * 4  # rank 0: the gathered logits of the whole job; other ranks copy their own rows only
    ceiling_gbs = h2d_ceiling(host_x, dev, world, dp)
    e2e_h2d_gbs = h2d * world / (e2e_ms / 1000.0) / 1e9

    # ---- extra (never the headline): the same public call fed batches the host has already quantized ------------------
    # The configuration's input is fp32, and its 154 MB per step is what bounds e2e.  With uint8 batches (QuantizeLinear with the
    # network's input scale done by whoever produces the images) a quarter of the bytes cross PCIe and the logits are the same.
    e2e_u8 = None
    if not args.no_u8_extra:
        eng8 = dp.InferenceEngine(net, world, fold=fold, rank=rank, input_dtype=torch.uint8)
        eng8.prepare(calib)
        host_q = dp.pinned_like((args.batch, 3, IMAGE, IMAGE), torch.uint8, local_rank)
        host_q.copy_(ops.QuantizeLinear(host_x.to(dev), net.in_scale, np.uint8(0)).cpu())
        same = bool(torch.equal(eng8.run_host(host_q).clone(), eng.run_host(host_x).clone()))
        for _ in eng8.run_stream([host_q] * 3):
            pass
        barrier()
        q0, q1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        q0.record()
        for _ in eng8.run_stream([host_q] * args.steps):
            pass
        q1.record()
        barrier()
        u8_ms = dp.max_over_ranks(q0.elapsed_time(q1), dev, world) / args.steps
        e2e_u8 = {"value": args.batch * world / (u8_ms / 1000.0), "unit": "img/s", "ms_per_step": u8_ms, "h2d_bytes_per_step": host_q.numel(),
                  "d2h_bytes_per_step": d2h, "logits_equal_fp32_input_run": same,
                  "note": "extra, not the headline: host batches already quantized to uint8 with the network's input scale, same public call "
                          "(InferenceEngine.run_stream, input_dtype=uint8); the configuration itself feeds fp32 (e2e)"}
        del eng8
        ops.device_status()

    # ---- roofline of the dominant kernel (tcgen05 implicit GEMM), timed with CUDA events per launch ---------
    roof = cpu = parity = None
    emulate_logits = None
    if rank == 0:
        L.chxq_tc_profile(1)
        prof_steps = 3
        for _ in range(prof_steps):
            net.forward(eng.x_dev, fold=fold)
        import ctypes
        tms, n, macs = ctypes.c_double(), ctypes.c_int64(), ctypes.c_double()
        L.chxq_tc_profile_read(ctypes.byref(tms), ctypes.byref(n), ctypes.byref(macs))
        L.chxq_tc_profile(0)
        # an event pair around nothing still measures a few microseconds: take that off every launch
        gaps = []
        for _ in range(50):
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            b.record()
            gaps.append((a, b))
        torch.cuda.synchronize(dev)
        pair_ms = float(np.median([a.elapsed_time(b) for a, b in gaps]))
        raw_ms = tms.value
        tms.value = max(raw_ms - pair_ms * n.value, 0.5 * raw_ms)
        pk = peaks()
        achieved = 2.0 * macs.value / (tms.value / 1000.0) / 1e12
        peak = 2.0 * pk["bf16_burst"]  # the per-launch events above time a short burst at full clocks
        traffic, traffic_note = recorded_traffic(args.batch, fold)
        probe_tops, probe_err = int8_probe(dev)
        share = (tms.value / prof_steps) / ms_per_step
        sus_tops = achieved * (ms_per_step / sus_ms_per_step)  # same kernels, same share of the step, at the sustained clocks
        roof = {"bound": "tensor", "kernel": "tc_igemm2_kernel + tc_igemm3_kernel + tc_chain_kernel (tcgen05 kind::i8 implicit GEMM: grouped tiles, CTA pairs, two convolutions per kernel; all 53 convolutions)",
                "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak, "traffic": traffic, "traffic_note": traffic_note,
                "peak_source": "2 x bf16_tflops (burst) of MEASURED_PEAKS.json (%s; the file has no int8 entry; int8 ops counted as 2 per MAC); of %s"
                               % (pk["source"], "measured" if pk["source"] == "measured" else "fallback"),
                "int8_probe_tops": probe_tops, "int8_probe_note": probe_err or "torch._int_mm 8192^3 on this GPU, best of 10 (vendor library; measurement only)",
                "frac_of_int8_probe": achieved / probe_tops if probe_tops else None,
                "frac_of_nominal_4500_tops": achieved / 4500.0,
                "sustained": {"achieved": sus_tops, "peak": 2.0 * pk["bf16_sustained"], "frac": sus_tops / (2.0 * pk["bf16_sustained"]),
                              "peak_source": "2 x bf16_tflops_sustained"},
                "launches_per_step": int(n.value // prof_steps), "kernel_ms_per_step": tms.value / prof_steps,
                "event_pair_overhead_us": pair_ms * 1000.0, "kernel_ms_per_step_uncorrected": raw_ms / prof_steps,
                "share_of_step": share, "algorithmic_gop_per_step": 2.0 * macs.value / prof_steps / 1e9}
        if not args.no_cpu_baseline:
            orc = entry.load_oracle()
            from oracle import networks
            orc.set_num_threads(len(os.sched_getaffinity(0)))
            sample = host_x[: args.cpu_sample].numpy()
            params = net.export_numpy()
            networks.resnet50_forward(params, sample[:1], mode="emulate")  # first run discarded (tools/run_onnx.cc:468-469 of the reference)
            t0 = time.perf_counter()
            emulate_logits = networks.resnet50_forward(params, sample, mode="emulate")
            sec = time.perf_counter() - t0
            cpu = {"value": args.cpu_sample / sec, "unit": "img/s", "cores": orc.num_threads(), "kind": "port",
                   "sample": "%d of the %d images of one step through the oracle's reference-algorithm chain (dequantize, fp32 conv, quantize per "
                             "QLinearConv; the convolution is a direct loop, not im2col + GEMM), one timed pass after a discarded first run"
                             % (args.cpu_sample, args.batch)}
            # ---- parity on this very configuration: the images of the CPU sample through the GPU network, tapped per operator ----
            taps = {}
            gl = net.forward(eng.x_dev, fold=fold, taps=taps, detail=True)
            k = args.cpu_sample
            to_np = lambda t: t[:k].contiguous().cpu().numpy()  # noqa: E731  (logically NCHW; .contiguous() undoes channels_last)
            np_taps = {name: to_np(t) for name, t in taps.items()}
            graph_logits = eng.slots[0]["logits"]
            eng.slots[0]["graph"].replay()
            torch.cuda.synchronize(dev)
            parity = networks.resnet50_parity(params, sample, np_taps, gl[:k].cpu().numpy(), fold=fold, emulate_logits=emulate_logits)
            parity["config"] = "ResNet-50 v1 224x224 full width, the first %d images of rank 0's batch of %d" % (k, args.batch)
            parity["captured_graph_logits_equal_tapped_run"] = bool(torch.equal(graph_logits, gl))
            parity["ok"] = bool(parity["ok"] and parity["captured_graph_logits_equal_tapped_run"])
            del taps, np_taps
    if world > 1:
        dist.barrier()
    # ---- the same step with the reference's operation order in every requantization (multiply, divide), for comparison ------
    ref_order = None
    if rank == 0 and world == 1 and fold:
        logits_fold = net.forward(eng.x_dev, fold=True).clone()
        g_exact, logits_exact = net.capture(eng.slots[0]["x"], fold=False)
        for _ in range(3):
            g_exact.replay()
        torch.cuda.synchronize(dev)
        n_exact = max(3, args.steps // 4)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(n_exact):
            g_exact.replay()
        b.record()
        torch.cuda.synchronize(dev)
        ms_exact = a.elapsed_time(b) / n_exact
        ref_order = {"ms_per_step": ms_exact, "value": args.batch / (ms_exact / 1000.0), "unit": "img/s", "steps": n_exact,
                     "top1_agreement_with_folded": float((logits_fold.argmax(1) == logits_exact.argmax(1)).float().mean().item()),
                     "max_abs_logit_difference": float((logits_fold - logits_exact).abs().max().item()),
                     "max_abs_logit": float(logits_exact.abs().max().item()),
                     "note": "fold_scales off: every QLinearConv requantizes with the reference's multiply and divide (runtime/ops/quantize.cc:16-35); "
                             "the headline runs the single-multiplier form, at most one output step apart per operator (see parity)"}
        del g_exact
        ops.device_status()
    # ---- the workloads beside the headline (rank 0, after every timed region) --------------------------------------------
    secondary = None
    if rank == 0 and not args.no_secondary:
        del eng, net
        torch.cuda.empty_cache()
        import microbench
        t0 = time.perf_counter()
        try:
            secondary = {"results": microbench.secondary(dev), "seconds": None,
                         "note": "per-operator measurements of microbench.py: CUDA events, 3 warm-ups, median of 10 (3 for the largest GEMMs), a 256 MB "
                                 "buffer rewritten between calls; GB/s are algorithmic bytes, fractions against the measured copy bandwidth and "
                                 "against the nominal 8 TB/s; TOPS against the nominal 4.5 POPS"}
        except Exception as exc:
            secondary = {"error": "%s: %s" % (type(exc).__name__, str(exc)[:200])}
        secondary["seconds"] = time.perf_counter() - t0
    if world > 1:
        dist.barrier()
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": "img/s", "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "ResNet-50 v1 int8 inference (configs[4]): batch %d per GPU, 3x224x224 fp32 NCHW input -> QuantizeLinear -> 53 "
                                   "QLinearConv (per-channel int8 weights, uint8 activations, bias, ReLU, residual tails fused) -> fp32 FC logits"
                                   % args.batch,
                       "batch_per_gpu": args.batch, "global_batch": args.batch * world, "parallelism": "dp%d" % world,
                       "l2": "inputs (154 MB fp32 per step) and activations are larger than the 126 MB L2; no explicit flush",
                       "gop_per_image": gop_per_image, "cuda_graph": True,
                       "requantization": "one folded multiplier per channel (fold_scales)" if fold else "reference operation order",
                       "parity_class": ("folded requantization: bit-exact against the oracle's restatement of that arithmetic, at most one output step "
                                        "from the reference's operation order per operator (see parity); --exact-requant runs the reference's order")
                       if fold else "reference operation order: bit-exact against the integer-domain oracle",
                       "vs_baseline_note": "null: the reference publishes no number for this metric; cpu_baseline is measured in this run"},
            "clocks": clocks,
            "sustained": sustained,
            "e2e": {"value": e2e_value, "unit": "img/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms,
                    "wall_ms_per_step": e2e_wall_ms, "h2d_gbs": e2e_h2d_gbs, "h2d_ceiling_gbs": ceiling_gbs,
                    "frac_of_h2d_ceiling": e2e_h2d_gbs / ceiling_gbs if ceiling_gbs else None,
                    "note": "h2d_ceiling_gbs: every rank copying the same pinned input at once with nothing else running (aggregate over ranks); "
                            "d2h bytes are rank 0's (the whole job's logits), other ranks copy their own rows"},
            "e2e_uint8_host_input": e2e_u8,
            "gpu_launches": launches_per_step * args.steps,
            "roofline": roof,
            "cpu_baseline": cpu,
            "parity": parity,
            "reference_order_requantization": ref_order,
            "secondary": secondary,
            "tops": gop_per_image * args.batch * world / (ms_per_step / 1000.0) / 1e3,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if parity is not None and not parity["ok"]:
        sys.stderr.write("bench.py: parity check failed: %s\n" % json.dumps(parity))
        sys.exit(1)


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_chxq(args)


if __name__ == "__main__":
    main()
