"""Synthetic int8 networks built from the quantized VM ops (the benchmark configurations).

Weights are random with the stated initialisation (no checkpoint or dataset is involved); batch
norms are folded into the preceding convolution before quantization; weights are quantized per
output channel with the reference's weight quantizer (``compiler/quantize.cc:70-129``); activation
scales are calibrated once, offline, on one seeded batch.  Convolution outputs that feed a residual
addition (no ReLU in front of them) get an asymmetric uint8 zero point so that their negative half is
representable; every other activation has zero point 0, where ReLU is the saturation at 0.

The op sequence per bottleneck block is the one a QLinear-mode graph holds:
``QLinearConv`` x3 (+ projection), then ``DequantizeLinear, DequantizeLinear, Add, Relu, QuantizeLinear``;
``forward`` runs that tail inside the last convolution's epilogue, ``forward_unfused`` runs it as the
separate one-pass kernel -- both give bit-identical maps.
"""
import ctypes

import numpy as np
import torch

from . import _lib, ops
from ._lib import check, lib

# (blocks, mid channels, out channels, stride of the first block): scripts/resnet50.py:86-90 of the reference.
RESNET50_STAGES = [(3, 64, 256, 1), (4, 128, 512, 2), (6, 256, 1024, 2), (3, 512, 2048, 2)]


def quantize_weights(w, per_channel=True, to_int8=True):
    """fp32 OIHW / [M, inner] weights -> (q, scales[M or 1], zero_points[M or 1]) with the reference's weight quantizer."""
    w = np.ascontiguousarray(w, np.float32)
    M = w.shape[0]
    inner = w.size // M
    q = np.empty(w.shape, np.int8 if to_int8 else np.uint8)
    n = M if per_channel else 1
    s = np.empty(n, np.float32)
    z = np.empty(n, np.int32)
    check(lib().chxq_quantize_weights_host(w.ctypes.data, M, inner, int(to_int8), int(per_channel), q.ctypes.data, s.ctypes.data, z.ctypes.data))
    return q, s, z


class _Conv:
    """One convolution of the network: float parameters, their quantized form and the packed device copy."""

    def __init__(self, name, cin, cout, k, stride, pad, rng, he_fan_in=None):
        self.name, self.cin, self.cout, self.k, self.stride, self.pad = name, cin, cout, k, stride, pad
        fan_in = he_fan_in or cin * k * k
        w = rng.standard_normal((cout, cin, k, k), dtype=np.float32) * np.float32(np.sqrt(2.0 / fan_in))
        # batch norm of a trained network, folded: w' = w * g / sqrt(v + eps), b' = beta - mean * g / sqrt(v + eps)
        gamma = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        beta = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        mean = (rng.standard_normal(cout) * 0.1).astype(np.float32)
        var = rng.uniform(0.5, 1.5, cout).astype(np.float32)
        inv = gamma / np.sqrt(var + np.float32(2e-5))
        self.w_f = (w * inv[:, None, None, None]).astype(np.float32)
        self.b_f = (beta - mean * inv).astype(np.float32)
        self.w_q, self.w_scale, wz = quantize_weights(self.w_f, per_channel=True, to_int8=True)
        self.w_zp = wz.astype(np.int8)
        # filled by calibration
        self.x_scale = None
        self.y_scale = None
        self.y_zp = 0
        self.bias_q = None
        self.packed = None
        self.dev = {}


class ResNet50Int8:
    """ResNet-50 v1 (stride on the first 1x1 of a stage and on its projection, scripts/resnet50.py:12-31,75-104 of the
    reference), int8 weights per channel, uint8 activations per tensor, fp32 classifier."""

    def __init__(self, batch, device, seed=0, image=224, num_classes=1000, width_mult=1.0):
        self.batch, self.device, self.image = int(batch), torch.device(device), int(image)
        rng = np.random.default_rng(seed)
        wm = lambda c: max(16, int(c * width_mult) // 16 * 16)  # noqa: E731
        self.stem = _Conv("conv1", 3, wm(64), 7, 2, 3, rng)
        self.blocks = []
        cin = wm(64)
        for si, (n_blocks, mid, cout, stride) in enumerate(RESNET50_STAGES):
            mid, cout = wm(mid), wm(cout)
            for bi in range(n_blocks):
                s = stride if bi == 0 else 1
                nm = "res%d_%d" % (si + 2, bi)
                blk = {
                    "conv1": _Conv(nm + "_conv1", cin, mid, 1, s, 0, rng),
                    "conv2": _Conv(nm + "_conv2", mid, mid, 3, 1, 1, rng),
                    "conv3": _Conv(nm + "_conv3", mid, cout, 1, 1, 0, rng),
                    "proj": _Conv(nm + "_proj", cin, cout, 1, s, 0, rng) if bi == 0 else None,
                    "out_scale": None,
                }
                self.blocks.append(blk)
                cin = cout
        self.feat = cin
        self.fc_w = (rng.standard_normal((num_classes, cin), dtype=np.float32) * np.float32(0.01))
        self.fc_b = np.zeros(num_classes, np.float32)
        self.in_scale = np.float32(1.0 / 255.0)
        self.calibrated = False
        self.use_chain = True  # conv2 -> conv3 of a bottleneck as one kernel (ops.QLinearConvChainPacked) where that is faster
        self._graph = None

    # ---- enumeration helpers -------------------------------------------------------------------
    def convs(self):
        yield self.stem
        for b in self.blocks:
            for k in ("conv1", "conv2", "conv3", "proj"):
                if b[k] is not None:
                    yield b[k]

    def macs_per_image(self):
        """Multiply-accumulates of one image (convolutions + classifier)."""
        total = 0
        hw = self.image // 2  # stem output 112
        total += self.stem.cout * 3 * 49 * hw * hw
        hw = (hw - 3 + 1) // 2 + 1  # max pool 3x3/2, cover_all
        for b in self.blocks:
            s = b["conv1"].stride
            ho = (hw - 1) // s + 1
            total += b["conv1"].cin * b["conv1"].cout * ho * ho
            total += b["conv2"].cin * b["conv2"].cout * 9 * ho * ho
            total += b["conv3"].cin * b["conv3"].cout * ho * ho
            if b["proj"] is not None:
                total += b["proj"].cin * b["proj"].cout * ho * ho
            hw = ho
        total += self.fc_w.size
        return total

    # ---- device upload / packing -----------------------------------------------------------------
    def _upload(self, c, x_shape, x_nchw=False):
        dev = self.device
        c.dev["w"] = torch.from_numpy(c.w_q).to(dev)
        c.dev["w_scale"] = torch.from_numpy(c.w_scale).to(dev)
        c.dev["w_zp"] = torch.from_numpy(c.w_zp).to(dev)
        c.packed = ops.PackedConv(c.dev["w"], c.dev["w_zp"], x_shape, strides=(c.stride, c.stride), pads=(c.pad, c.pad),
                                  x_layout=_lib.NCHW if x_nchw else _lib.NHWC)
        if not c.packed.eligible:
            raise _lib.ChxqError(_lib.ERR_UNSUPPORTED, "%s is not eligible for the tensor-core path" % c.name)
        return (c.packed.g.N, c.packed.g.M, c.packed.g.Ho, c.packed.g.Wo)

    def _conv_acc(self, c, x):
        """Exact int32 accumulator of convolution c over the uint8 map x (ConvInteger on the packed weights)."""
        g = c.packed.g
        y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.int32, device=self.device, memory_format=torch.channels_last)
        ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), 0, c.packed.flags)
        ws = ops.workspace(ws_bytes, self.device)
        check(lib().chxq_conv_integer_packed(ops._ptr(x), ops._ptr(c.packed.blob), ctypes.byref(g), 1, 0, c.packed.flags, ops._ptr(y),
                                             ops._ptr(ws), ws_bytes, ops._stream()))
        return y

    def _calibrate_conv(self, c, x, x_scale, relu):
        """Sets the bias, the output scale and zero point of c from the batch x; returns the quantized output."""
        c.x_scale = np.float32(x_scale)
        mult = (np.float32(x_scale) * c.w_scale).astype(np.float32)
        c.bias_q = np.rint(c.b_f.astype(np.float64) / mult.astype(np.float64)).astype(np.int64).clip(-2**31, 2**31 - 1).astype(np.int32)
        c.dev["bias"] = torch.from_numpy(c.bias_q).to(self.device)
        acc = self._conv_acc(c, x)
        yf = (acc + c.dev["bias"].view(1, -1, 1, 1)).float() * torch.from_numpy(mult).to(self.device).view(1, -1, 1, 1)
        hi = float(yf.amax().item())
        lo = float(yf.amin().item())
        del yf, acc
        if relu:
            c.y_scale = np.float32(max(hi, 1e-6) / 255.0)
            c.y_zp = 0
        else:
            lo, hi = min(lo, 0.0), max(hi, 0.0)
            c.y_scale = np.float32(max(hi - lo, 1e-6) / 255.0)
            c.y_zp = int(np.clip(np.rint(-lo / float(c.y_scale)), 0, 255))
        return self._run_conv(c, x)

    def _run_conv(self, c, x, residual=None, res_scale=1.0, res_zp=0, out_scale=1.0, out=None, fold=False):
        return ops.QLinearConvPacked(x, c.packed, c.x_scale, np.uint8(0), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                                     b=c.dev["bias"], residual=residual, res_scale=res_scale, res_zero_point=res_zp, res_relu=True,
                                     out_scale=out_scale, out_zero_point=0, out=out, fold_scales=fold)

    def _conv_args(self, c, fold, **tail):
        d = dict(x_scale=c.x_scale, x_zero_point=np.uint8(0), w_scale=c.dev["w_scale"], w_zero_point=c.dev["w_zp"], y_scale=c.y_scale,
                 y_zero_point=np.uint8(c.y_zp), b=c.dev["bias"], fold_scales=fold)
        d.update(tail)
        return d

    def _run_tail(self, b, h1, sc, sc_scale, sc_zp, fold):
        """conv2 -> conv3 + residual join of one bottleneck.  With folded requantizations the two convolutions run as one kernel
        (ops.QLinearConvChainPacked) where one exists for the block's width; bit-identical to the two calls."""
        # (measured at batch 256: one kernel wins for 64 and 128 channels between the layers, 140 against 153 us and 79 against 90 us per
        # block; at 256 channels the pair of kernels on CTA pairs is as fast, 63 us)
        if fold and self.use_chain and b.get("chain", b["conv2"].cout <= 128):
            try:
                return ops.QLinearConvChainPacked(
                    h1, b["conv2"].packed, self._conv_args(b["conv2"], fold), b["conv3"].packed,
                    self._conv_args(b["conv3"], fold, residual=sc, res_scale=sc_scale, res_zero_point=sc_zp, res_relu=True, out_scale=b["out_scale"],
                                    out_zero_point=0))
            except _lib.ChxqError as e:
                if e.code != _lib.ERR_UNSUPPORTED:
                    raise
                b["chain"] = False  # no fused kernel for this width: two calls from now on
        h2 = self._run_conv(b["conv2"], h1, fold=fold)
        return self._run_conv(b["conv3"], h2, residual=sc, res_scale=sc_scale, res_zp=sc_zp, out_scale=b["out_scale"], fold=fold)

    def calibrate(self, x):
        """Uploads and packs the weights, then walks the network once over the fp32 NCHW batch x to fix every scale."""
        assert tuple(x.shape) == (self.batch, 3, self.image, self.image) and x.dtype == torch.float32
        xq = ops.QuantizeLinear(x.contiguous(), self.in_scale, np.uint8(0))
        shape = self._upload(self.stem, tuple(xq.shape), x_nchw=True)
        h = self._calibrate_conv(self.stem, xq, self.in_scale, relu=True)
        h = ops.MaxPoolU8(h, 3, 2, 0, cover_all=True)
        h_scale = self.stem.y_scale
        shape = tuple(h.shape)
        for b in self.blocks:
            s1 = self._upload(b["conv1"], shape)
            h1 = self._calibrate_conv(b["conv1"], h, h_scale, relu=True)
            self._upload(b["conv2"], s1)
            h2 = self._calibrate_conv(b["conv2"], h1, b["conv1"].y_scale, relu=True)
            s3 = self._upload(b["conv3"], tuple(h2.shape))
            h3 = self._calibrate_conv(b["conv3"], h2, b["conv2"].y_scale, relu=False)
            if b["proj"] is not None:
                self._upload(b["proj"], shape)
                sc = self._calibrate_conv(b["proj"], h, h_scale, relu=False)
                sc_scale, sc_zp = b["proj"].y_scale, b["proj"].y_zp
            else:
                sc, sc_scale, sc_zp = h, h_scale, 0
            # scale of the block output: max of relu(DQ(h3) + DQ(sc)) over the batch
            sf = (h3.float() - b["conv3"].y_zp) * float(b["conv3"].y_scale) + (sc.float() - sc_zp) * float(sc_scale)
            b["out_scale"] = np.float32(max(float(sf.clamp_min(0).amax().item()), 1e-6) / 255.0)
            del sf
            b["res"] = (sc_scale, sc_zp)
            h = ops.QAddU8(h3, b["conv3"].y_scale, b["conv3"].y_zp, sc, sc_scale, sc_zp, b["out_scale"], 0, relu=True)
            h_scale = b["out_scale"]
            shape = s3
        self.dev_fc_w = torch.from_numpy(self.fc_w).to(self.device)
        self.dev_fc_b = torch.from_numpy(self.fc_b).to(self.device)
        self.final_scale = h_scale
        self.calibrated = True
        torch.cuda.synchronize(self.device)

    # ---- inference ----------------------------------------------------------------------------------
    def forward(self, x, fused=True, taps=None, fold=False, detail=False):
        """fp32 NCHW batch -> fp32 logits [N, classes].  taps (a dict) receives intermediate uint8 maps when given: 'stem',
        'block<i>' and 'pooled'; with detail=True also the input and output of every operator ('pool', 'b<i>_h1', 'b<i>_h2',
        'b<i>_h3' = the last convolution's own output before the residual join, 'b<i>_sc' = the shortcut), so that each operator
        can be checked on its own against the reference's arithmetic fed the same bytes.
        fold=True requantizes every convolution with one multiplier per channel (QLinearConv's fold_scales)."""
        assert self.calibrated
        assert fused or not fold, "the folded residual tail exists only inside the convolution epilogue"
        c = self.stem
        if fused and taps is None:
            # the input's QuantizeLinear runs inside the stem convolution's repack pass and the max pooling on its output tiles:
            # neither the uint8 image nor the full-resolution stem output reaches memory
            h = ops.QLinearConvMaxPoolPacked(x, c.packed, c.x_scale, np.uint8(0), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                                             b=c.dev["bias"], cover_all=True, fold_scales=fold)
        else:
            if fused:
                h = ops.QuantizeLinearConvPacked(x, c.packed, c.x_scale, np.uint8(0), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                                                 b=c.dev["bias"], fold_scales=fold)
            else:
                xq = ops.QuantizeLinear(x, self.in_scale, np.uint8(0))
                h = self._run_conv(c, xq, fold=fold)
            if taps is not None:
                taps["stem"] = h
            h = ops.MaxPoolU8(h, 3, 2, 0, cover_all=True)
            if taps is not None and detail:
                taps["pool"] = h
        h_scale = self.stem.y_scale
        for i, b in enumerate(self.blocks):
            h1 = self._run_conv(b["conv1"], h, fold=fold)
            if b["proj"] is not None:
                sc = self._run_conv(b["proj"], h, fold=fold)
            else:
                sc = h
            sc_scale, sc_zp = b["res"]
            chained = fused and fold and not (taps is not None and detail)
            h2 = None if chained else self._run_conv(b["conv2"], h1, fold=fold)
            if taps is not None and detail:
                taps["b%d_h1" % i], taps["b%d_h2" % i], taps["b%d_sc" % i] = h1, h2, sc
                taps["b%d_h3" % i] = self._run_conv(b["conv3"], h2, fold=fold)
            if chained:
                h = self._run_tail(b, h1, sc, sc_scale, sc_zp, fold)
            elif fused:
                h = self._run_conv(b["conv3"], h2, residual=sc, res_scale=sc_scale, res_zp=sc_zp, out_scale=b["out_scale"], fold=fold)
            else:
                h3 = self._run_conv(b["conv3"], h2)
                h = ops.QAddU8(h3, b["conv3"].y_scale, b["conv3"].y_zp, sc, sc_scale, sc_zp, b["out_scale"], 0, relu=True)
            h_scale = b["out_scale"]
            if taps is not None:
                taps["block%d" % i] = h
        pooled = ops.GlobalAveragePoolDequant(h, h_scale, 0)
        logits = ops.Linear(pooled, self.dev_fc_w, self.dev_fc_b)
        if taps is not None:
            taps["pooled"] = pooled
        return logits

    def capture(self, x_static, fold=False):
        """Captures forward(x_static) into a CUDA graph; returns (graph, logits).  Replaying needs no host work per layer."""
        self.forward(x_static, fold=fold)  # warm-up: sizes the workspace and sets kernel attributes outside the capture
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            logits = self.forward(x_static, fold=fold)
        return g, logits

    def to_onnx(self):
        """The calibrated network as a statically quantized ONNX graph (an onnx_io.Model) of standard nodes: QuantizeLinear,
        QLinearConv with int32 bias (a zero output zero point makes the uint8 saturation the ReLU), MaxPool on uint8 with
        ceil_mode (Chainer's cover_all), per residual join DequantizeLinear x2, Add, Relu, QuantizeLinear, then
        DequantizeLinear, GlobalAveragePool, Flatten and an fp32 Gemm.  `run_onnx` executes this file on the same kernels the
        hand-built forward() uses."""
        from . import onnx_io
        assert self.calibrated
        N, f32, u8 = onnx_io.Node, np.float32, np.uint8
        inits, nodes = {"zero_u8": u8(0).reshape(())}, []

        def scalar(name, v, dt=f32):
            inits[name] = np.asarray(v, dt).reshape(())
            return name

        def conv(c, x, x_scale_name, out):
            n = c.name
            inits[n + "_w"], inits[n + "_ws"], inits[n + "_wz"], inits[n + "_b"] = c.w_q, c.w_scale, c.w_zp, c.bias_q
            ys, zy = scalar(n + "_ys", c.y_scale), scalar(n + "_zy", c.y_zp, u8)
            attrs = {"kernel_shape": [c.k, c.k], "strides": [c.stride, c.stride], "pads": [c.pad] * 4}
            nodes.append(N("QLinearConv", [x, x_scale_name, "zero_u8", n + "_w", n + "_ws", n + "_wz", ys, zy, n + "_b"], [out], attrs, n))
            return ys, zy

        in_s = scalar("in_scale", self.in_scale)
        nodes.append(N("QuantizeLinear", ["x", in_s, "zero_u8"], ["xq"], {}))
        h_s, _ = conv(self.stem, "xq", in_s, "stem")
        nodes.append(N("MaxPool", ["stem"], ["pool"], {"kernel_shape": [3, 3], "strides": [2, 2], "ceil_mode": 1}))
        h = "pool"
        for i, b in enumerate(self.blocks):
            p = "b%d_" % i
            s1, _ = conv(b["conv1"], h, h_s, p + "h1")
            s2, _ = conv(b["conv2"], p + "h1", s1, p + "h2")
            s3, z3 = conv(b["conv3"], p + "h2", s2, p + "h3")
            if b["proj"] is not None:
                ss, zs = conv(b["proj"], h, h_s, p + "sc")
                sc = p + "sc"
            else:
                sc, ss, zs = h, h_s, "zero_u8"
            out_s = scalar(p + "out_scale", b["out_scale"])
            nodes.append(N("DequantizeLinear", [p + "h3", s3, z3], [p + "f3"], {}))
            nodes.append(N("DequantizeLinear", [sc, ss, zs], [p + "fs"], {}))
            nodes.append(N("Add", [p + "f3", p + "fs"], [p + "sum"], {}))
            nodes.append(N("Relu", [p + "sum"], [p + "relu"], {}))
            nodes.append(N("QuantizeLinear", [p + "relu", out_s, "zero_u8"], [p + "out"], {}))
            h, h_s = p + "out", out_s
        inits["fc_w"], inits["fc_b"] = self.fc_w, self.fc_b
        nodes.append(N("DequantizeLinear", [h, h_s, "zero_u8"], ["feat"], {}))
        nodes.append(N("GlobalAveragePool", ["feat"], ["gap"], {}))
        nodes.append(N("Flatten", ["gap"], ["flat"], {"axis": 1}))
        nodes.append(N("Gemm", ["flat", "fc_w", "fc_b"], ["logits"], {"transB": 1}))
        return onnx_io.Model(nodes, inits, ["x"], ["logits"], ir_version=5, opset=12, name="resnet50_int8")

    def export_numpy(self):
        """Everything the CPU oracle needs to run the same network."""
        def conv(c):
            return dict(name=c.name, w=c.w_q, w_scale=c.w_scale, w_zp=c.w_zp.astype(np.int32), bias=c.bias_q, x_scale=c.x_scale,
                        y_scale=c.y_scale, y_zp=c.y_zp, stride=c.stride, pad=c.pad)
        return dict(in_scale=self.in_scale, stem=conv(self.stem),
                    blocks=[dict(conv1=conv(b["conv1"]), conv2=conv(b["conv2"]), conv3=conv(b["conv3"]),
                                 proj=conv(b["proj"]) if b["proj"] is not None else None, res=b["res"], out_scale=b["out_scale"])
                            for b in self.blocks],
                    fc_w=self.fc_w, fc_b=self.fc_b, final_scale=self.final_scale)


class QuantizedMLP:
    """784-1000-1000-10 MLP: QuantizeLinear -> (QLinearMatMul -> ReLU)x2 -> QLinearMatMul -> DequantizeLinear.
    Weights N(0, 0.05), per-tensor symmetric int8 (scale = max|w| / 127, zero point 0); activations uint8 with
    scale 1/255 and zero point 0, where the uint8 saturation at 0 is the ReLU."""

    def __init__(self, device, seed=0, sizes=(784, 1000, 1000, 10)):
        rng = np.random.default_rng(seed)
        self.device = torch.device(device)
        self.layers = []
        for fin, fout in zip(sizes[:-1], sizes[1:]):
            w = (rng.standard_normal((fin, fout)) * 0.05).astype(np.float32)  # [K, N] as MatMul consumes it
            q, s, z = quantize_weights(w.reshape(1, -1), per_channel=False, to_int8=True)
            self.layers.append(dict(w_q=q.reshape(fin, fout), w_scale=np.float32(s[0]), dev=torch.from_numpy(q.reshape(fin, fout)).to(self.device)))
        self.act_scale = np.float32(1.0 / 255.0)

    def forward(self, x, path=_lib.PATH_AUTO):
        h = ops.QuantizeLinear(x, self.act_scale, np.uint8(0))
        for l in self.layers:
            h = ops.QLinearMatMul(h, self.act_scale, np.uint8(0), l["dev"], l["w_scale"], np.int8(0), self.act_scale, np.uint8(0), path=path)
        return ops.DequantizeLinear(h, self.act_scale, np.uint8(0))

    def forward_packed(self, x):
        """The same five ops with the constant weights packed once: each QLinearMatMul runs as a packed 1x1 QLinearConv over the
        batch seen as an [N, K, 1, 1] map (no per-call repacking of B).  Same results as forward().  Layers whose inner
        dimension is not a multiple of 16 keep the QLinearMatMul entry."""
        h = ops.QuantizeLinear(x, self.act_scale, np.uint8(0))
        n = h.shape[0]
        for l in self.layers:
            k, m = l["w_q"].shape
            if k % 16 or m % 16:
                h = ops.QLinearMatMul(h, self.act_scale, np.uint8(0), l["dev"], l["w_scale"], np.int8(0), self.act_scale, np.uint8(0))
                continue
            key = ("packed", n)
            if key not in l:
                w = l["dev"].t().contiguous().reshape(m, k, 1, 1)
                zw = torch.zeros((), dtype=torch.int8, device=self.device)
                l[key] = (ops.PackedConv(w, zw, (n, k, 1, 1)), torch.tensor(float(l["w_scale"]), device=self.device), zw)
            pk, ws, zw = l[key]
            hm = h.reshape(n, k, 1, 1).contiguous(memory_format=torch.channels_last)
            if pk.eligible:
                h = ops.QLinearConvPacked(hm, pk, self.act_scale, np.uint8(0), ws, zw, self.act_scale, np.uint8(0)).reshape(n, m)
            else:
                h = ops.QLinearMatMul(h, self.act_scale, np.uint8(0), l["dev"], l["w_scale"], np.int8(0), self.act_scale, np.uint8(0))
        return ops.DequantizeLinear(h, self.act_scale, np.uint8(0))


# (expansion t, output channels c, repeats n, stride s) of MobileNetV2-1.0.
MOBILENETV2_BLOCKS = [(1, 16, 1, 1), (6, 24, 2, 2), (6, 32, 3, 2), (6, 64, 4, 2), (6, 96, 3, 1), (6, 160, 3, 2), (6, 320, 1, 1)]


def _pad16(c):
    return (c + 15) // 16 * 16


class _QLayer:
    """One quantized convolution of MobileNetV2 (dense 1x1 / stem, or depthwise 3x3) with its calibration results."""

    def __init__(self, name, cin, cout, k, stride, pad, group, rng, relu6, cin_real=None, cout_real=None):
        self.name, self.cin, self.cout, self.k, self.stride, self.pad, self.group, self.relu6 = name, cin, cout, k, stride, pad, group, relu6
        cin_real, cout_real = cin_real or cin, cout_real or cout
        cg = cin // group
        w = np.zeros((cout, cg, k, k), np.float32)
        if group == 1:
            w[:cout_real, :cin_real] = rng.standard_normal((cout_real, cin_real, k, k)).astype(np.float32) * np.float32(0.02) * np.float32(
                np.sqrt(2.0 / (cin_real * k * k)) / 0.02)
        else:
            w[:cout_real] = rng.standard_normal((cout_real, 1, k, k)).astype(np.float32) * np.float32(np.sqrt(2.0 / (k * k)))
        self.w_f = w
        self.b_f = np.zeros(cout, np.float32)
        self.b_f[:cout_real] = (rng.standard_normal(cout_real) * 0.1).astype(np.float32)
        self.w_q, self.w_scale, wz = quantize_weights(w, per_channel=True, to_int8=True)
        self.w_scale = np.where(self.w_scale > 0, self.w_scale, np.float32(1.0)).astype(np.float32)  # all-zero padded channels
        self.w_zp = wz.astype(np.int8)
        self.x_scale = self.y_scale = None
        self.y_zp = 0
        self.clamp = None
        self.bias_q = None
        self.packed = None
        self.dev = {}


class MobileNetV2Int8:
    """MobileNetV2-1.0 (inverted residuals, expansion 6, depthwise 3x3, ReLU6), per-channel symmetric int8 weights, uint8
    activations.  Channel counts that are not multiples of 16 (24) are zero-padded to the next multiple of 16 in storage, so
    every NHWC row starts on a 16-byte boundary; the padded channels carry zero weights in and out.  Dense 1x1 layers run on
    the tensor cores (packed weights), depthwise layers on the depthwise kernel, ReLU6 is the upper clamp of the
    requantization, linear bottleneck outputs get an asymmetric zero point, residual joins run in the projecting
    convolution's epilogue (DequantizeLinear x2, Add, QuantizeLinear; no Relu)."""

    def __init__(self, batch, device, seed=0, image=224, num_classes=1000, depthwise_on_tensor_cores=True):
        self.batch, self.device, self.image = int(batch), torch.device(device), int(image)
        self.depthwise_on_tensor_cores = bool(depthwise_on_tensor_cores)
        rng = np.random.default_rng(seed)
        self.stem = _QLayer("stem", 3, 32, 3, 2, 1, 1, rng, True)
        self.blocks = []
        cin, cin_real = 32, 32
        for bi, (t, c, n, s) in enumerate(MOBILENETV2_BLOCKS):
            for i in range(n):
                stride = s if i == 0 else 1
                mid = cin_real * t
                cout, cout_real = _pad16(c), c
                nm = "b%d_%d" % (bi, i)
                blk = {
                    "expand": _QLayer(nm + "_expand", cin, mid, 1, 1, 0, 1, rng, True, cin_real=cin_real) if t != 1 else None,
                    "dw": _QLayer(nm + "_dw", mid, mid, 3, stride, 1, mid, rng, True),
                    "project": _QLayer(nm + "_project", mid, cout, 1, 1, 0, 1, rng, False, cout_real=cout_real),
                    "residual": stride == 1 and cin_real == cout_real,
                }
                self.blocks.append(blk)
                cin, cin_real = cout, cout_real
        self.head = _QLayer("head", cin, 1280, 1, 1, 0, 1, rng, True, cin_real=cin_real)
        self.fc_w = (rng.standard_normal((num_classes, 1280), dtype=np.float32) * np.float32(0.01))
        self.fc_b = np.zeros(num_classes, np.float32)
        self.in_scale = np.float32(1.0 / 255.0)
        self.calibrated = False

    def layers(self):
        yield self.stem
        for b in self.blocks:
            for k in ("expand", "dw", "project"):
                if b[k] is not None:
                    yield b[k]
        yield self.head

    def macs_per_image(self):
        """(dense multiply-accumulates, depthwise multiply-accumulates) of one image, counted on the real channel counts."""
        dense = dw = 0
        hw = self.image // 2
        dense += 32 * 3 * 9 * hw * hw
        cin = 32
        for (t, c, n, s) in MOBILENETV2_BLOCKS:
            for i in range(n):
                stride = s if i == 0 else 1
                mid = cin * t
                if t != 1:
                    dense += cin * mid * hw * hw
                hw = (hw + 2 - 3) // stride + 1
                dw += mid * 9 * hw * hw
                dense += mid * c * hw * hw
                cin = c
        dense += cin * 1280 * hw * hw + 1280 * self.fc_w.shape[0]
        return dense, dw

    # ---- execution of one layer -----------------------------------------------------------------------------------------
    def _upload(self, c, x_shape, x_nchw=False):
        dev = self.device
        c.dev["w"] = torch.from_numpy(c.w_q).to(dev)
        c.dev["w_scale"] = torch.from_numpy(c.w_scale).to(dev)
        c.dev["w_zp"] = torch.from_numpy(c.w_zp).to(dev)
        if c.group == 1 or self.depthwise_on_tensor_cores:
            c.packed = ops.PackedConv(c.dev["w"], c.dev["w_zp"], x_shape, strides=(c.stride, c.stride), pads=(c.pad, c.pad), group=c.group,
                                      x_layout=_lib.NCHW if x_nchw else _lib.NHWC)
            if not c.packed.eligible:
                if c.group == 1:
                    raise _lib.ChxqError(_lib.ERR_UNSUPPORTED, "%s is not eligible for the tensor-core path" % c.name)
                c.packed = None

    def _acc(self, c, x):
        if c.packed is not None:
            g = c.packed.g
            y = torch.empty((g.N, g.M, g.Ho, g.Wo), dtype=torch.int32, device=self.device, memory_format=torch.channels_last)
            ws_bytes = lib().chxq_conv_packed_workspace(ctypes.byref(g), 0, c.packed.flags)
            ws = ops.workspace(ws_bytes, self.device)
            check(lib().chxq_conv_integer_packed(ops._ptr(x), ops._ptr(c.packed.blob), ctypes.byref(g), 1, 0, c.packed.flags, ops._ptr(y),
                                                 ops._ptr(ws), ws_bytes, ops._stream()))
            return y
        return ops.ConvInteger(x, c.dev["w"], np.uint8(0), None, (c.stride, c.stride), (c.pad, c.pad), c.group, path=_lib.PATH_SIMT)

    def _run(self, c, x, fold=False, residual=None, res_scale=1.0, res_zp=0, out_scale=1.0, out_zp=0):
        kw = dict(b=c.dev["bias"], clamp_hi_q=c.clamp, residual=residual, res_scale=res_scale, res_zero_point=res_zp, res_relu=False,
                  out_scale=out_scale, out_zero_point=out_zp, fold_scales=fold)
        if c.packed is not None:
            return ops.QLinearConvPacked(x, c.packed, c.x_scale, np.uint8(0), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp), **kw)
        return ops.QLinearConv(x, c.x_scale, np.uint8(0), c.dev["w"], c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                               strides=(c.stride, c.stride), pads=(c.pad, c.pad), group=c.group, **kw)

    def _calibrate(self, c, x, x_scale, x_nchw=False):
        self._upload(c, tuple(x.shape), x_nchw)
        c.x_scale = np.float32(x_scale)
        mult = (np.float32(x_scale) * c.w_scale).astype(np.float32)
        c.bias_q = np.rint(c.b_f.astype(np.float64) / mult.astype(np.float64)).clip(-2**31, 2**31 - 1).astype(np.int32)
        c.dev["bias"] = torch.from_numpy(c.bias_q).to(self.device)
        acc = self._acc(c, x)
        yf = (acc + c.dev["bias"].view(1, -1, 1, 1)).float() * torch.from_numpy(mult).to(self.device).view(1, -1, 1, 1)
        lo, hi = float(yf.amin().item()), float(yf.amax().item())
        del yf, acc
        if c.relu6:
            c.y_scale, c.y_zp = np.float32(max(min(hi, 6.0), 1e-6) / 255.0), 0
            c.clamp = int(min(255, np.rint(6.0 / float(c.y_scale))))
        else:
            lo, hi = min(lo, 0.0), max(hi, 0.0)
            c.y_scale = np.float32(max(hi - lo, 1e-6) / 255.0)
            c.y_zp = int(np.clip(np.rint(-lo / float(c.y_scale)), 0, 255))
        return self._run(c, x)

    def calibrate(self, x):
        xq = ops.QuantizeLinear(x.contiguous(), self.in_scale, np.uint8(0))
        h = self._calibrate(self.stem, xq, self.in_scale, x_nchw=True)
        h_scale, h_zp = self.stem.y_scale, 0
        for b in self.blocks:
            inp, inp_scale, inp_zp = h, h_scale, h_zp
            # every convolution here takes a zero activation zero point: block inputs with an asymmetric zero point (linear
            # bottleneck outputs) are handled through x_zero_point of the consuming layer
            if b["expand"] is not None:
                b["expand"].x_zp = inp_zp
                h = self._calibrate_zp(b["expand"], h, inp_scale, inp_zp)
                e_scale = b["expand"].y_scale
            else:
                e_scale = inp_scale
            b["dw"].x_zp = 0 if b["expand"] is not None else inp_zp
            h = self._calibrate_zp(b["dw"], h, e_scale, b["dw"].x_zp)
            b["project"].x_zp = 0
            p = self._calibrate_zp(b["project"], h, b["dw"].y_scale, 0)
            if b["residual"]:
                sf = (p.float() - b["project"].y_zp) * float(b["project"].y_scale) + (inp.float() - inp_zp) * float(inp_scale)
                lo, hi = min(float(sf.amin().item()), 0.0), max(float(sf.amax().item()), 0.0)
                del sf
                b["out_scale"] = np.float32(max(hi - lo, 1e-6) / 255.0)
                b["out_zp"] = int(np.clip(np.rint(-lo / float(b["out_scale"])), 0, 255))
                b["res"] = (inp_scale, inp_zp)
                h = ops.QAddU8(p, b["project"].y_scale, b["project"].y_zp, inp, inp_scale, inp_zp, b["out_scale"], b["out_zp"], relu=False)
                h_scale, h_zp = b["out_scale"], b["out_zp"]
            else:
                h, h_scale, h_zp = p, b["project"].y_scale, b["project"].y_zp
        self.head.x_zp = h_zp
        h = self._calibrate_zp(self.head, h, h_scale, h_zp)
        self.dev_fc_w = torch.from_numpy(self.fc_w).to(self.device)
        self.dev_fc_b = torch.from_numpy(self.fc_b).to(self.device)
        self.calibrated = True
        torch.cuda.synchronize(self.device)

    def _calibrate_zp(self, c, x, x_scale, x_zp):
        """_calibrate for a layer whose input has zero point x_zp (recorded in c.x_zp and used by _run_zp)."""
        c.x_zp = int(x_zp)
        if x_zp == 0:
            return self._calibrate(c, x, x_scale)
        self._upload(c, tuple(x.shape))
        c.x_scale = np.float32(x_scale)
        mult = (np.float32(x_scale) * c.w_scale).astype(np.float32)
        c.bias_q = np.rint(c.b_f.astype(np.float64) / mult.astype(np.float64)).clip(-2**31, 2**31 - 1).astype(np.int32)
        c.dev["bias"] = torch.from_numpy(c.bias_q).to(self.device)
        acc = ops.ConvInteger(x, c.dev["w"], np.uint8(x_zp), None, (c.stride, c.stride), (c.pad, c.pad), c.group,
                              path=_lib.PATH_TENSOR if c.group == 1 else _lib.PATH_SIMT)
        yf = (acc + c.dev["bias"].view(1, -1, 1, 1)).float() * torch.from_numpy(mult).to(self.device).view(1, -1, 1, 1)
        lo, hi = float(yf.amin().item()), float(yf.amax().item())
        del yf, acc
        if c.relu6:
            c.y_scale, c.y_zp = np.float32(max(min(hi, 6.0), 1e-6) / 255.0), 0
            c.clamp = int(min(255, np.rint(6.0 / float(c.y_scale))))
        else:
            lo, hi = min(lo, 0.0), max(hi, 0.0)
            c.y_scale = np.float32(max(hi - lo, 1e-6) / 255.0)
            c.y_zp = int(np.clip(np.rint(-lo / float(c.y_scale)), 0, 255))
        return self._run_zp(c, x)

    def _run_zp(self, c, x, fold=False, **kw):
        if getattr(c, "x_zp", 0) == 0:
            return self._run(c, x, fold=fold, **kw)
        args = dict(b=c.dev["bias"], clamp_hi_q=c.clamp, fold_scales=fold, res_relu=False)
        args.update({"residual": kw.get("residual"), "res_scale": kw.get("res_scale", 1.0), "res_zero_point": kw.get("res_zp", 0),
                     "out_scale": kw.get("out_scale", 1.0), "out_zero_point": kw.get("out_zp", 0)})
        if c.packed is not None and (c.group == 1 or c.pad == 0):  # grouped layers with padding need a zero activation zero point there
            return ops.QLinearConvPacked(x, c.packed, c.x_scale, np.uint8(c.x_zp), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                                         **args)
        return ops.QLinearConv(x, c.x_scale, np.uint8(c.x_zp), c.dev["w"], c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                               strides=(c.stride, c.stride), pads=(c.pad, c.pad), group=c.group, **args)

    def forward(self, x, fused=True, fold=False, taps=None):
        assert self.calibrated
        c = self.stem
        if fused:  # the input's QuantizeLinear runs inside the stem convolution's repack pass
            h = ops.QuantizeLinearConvPacked(x, c.packed, c.x_scale, np.uint8(0), c.dev["w_scale"], c.dev["w_zp"], c.y_scale, np.uint8(c.y_zp),
                                             b=c.dev["bias"], clamp_hi_q=c.clamp, fold_scales=fold)
        else:
            xq = ops.QuantizeLinear(x, self.in_scale, np.uint8(0))
            h = self._run(c, xq, fold=fold)
        if taps is not None:
            taps["stem"] = h
        for i, b in enumerate(self.blocks):
            inp = h
            if b["expand"] is not None:
                h = self._run_zp(b["expand"], h, fold=fold)
            h = self._run_zp(b["dw"], h, fold=fold)
            if b["residual"] and fused:
                h = self._run_zp(b["project"], h, fold=fold, residual=inp, res_scale=b["res"][0], res_zp=b["res"][1], out_scale=b["out_scale"],
                                 out_zp=b["out_zp"])
            else:
                h = self._run_zp(b["project"], h, fold=fold)
                if b["residual"]:
                    h = ops.QAddU8(h, b["project"].y_scale, b["project"].y_zp, inp, b["res"][0], b["res"][1], b["out_scale"], b["out_zp"], relu=False)
            if taps is not None:
                taps["block%d" % i] = h
        h = self._run_zp(self.head, h, fold=fold)
        pooled = ops.GlobalAveragePoolDequant(h, self.head.y_scale, 0)
        if taps is not None:
            taps["pooled"] = pooled
        return ops.Linear(pooled, self.dev_fc_w, self.dev_fc_b)

    def capture(self, x_static, fold=False):
        """Captures forward(x_static) into a CUDA graph; returns (graph, logits)."""
        self.forward(x_static, fold=fold)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            logits = self.forward(x_static, fold=fold)
        return g, logits

    def export_numpy(self):
        def lay(c):
            return None if c is None else dict(name=c.name, w=c.w_q, w_scale=c.w_scale, w_zp=c.w_zp.astype(np.int32), bias=c.bias_q,
                                               x_scale=c.x_scale, x_zp=getattr(c, "x_zp", 0), y_scale=c.y_scale, y_zp=c.y_zp, clamp=c.clamp,
                                               stride=c.stride, pad=c.pad, group=c.group)
        return dict(in_scale=self.in_scale, stem=lay(self.stem), head=lay(self.head),
                    blocks=[dict(expand=lay(b["expand"]), dw=lay(b["dw"]), project=lay(b["project"]), residual=b["residual"],
                                 res=b.get("res"), out_scale=b.get("out_scale"), out_zp=b.get("out_zp")) for b in self.blocks],
                    fc_w=self.fc_w, fc_b=self.fc_b)
