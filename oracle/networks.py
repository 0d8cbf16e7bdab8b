"""CPU restatement of the benchmark networks as chains of the oracle's ops (TEST INFRASTRUCTURE ONLY; PARITY UNPINNED,
see chxq_oracle.c).  `params` is what ``models.ResNet50Int8.export_numpy()`` returns.

mode="emulate": every QLinearConv runs as the reference does (runtime/ops/quantize.cc:62-94: dequantize, fp32 convolution,
quantize) -- this is the reference's CPU path and what the bench times as the CPU baseline.
mode="exact": every QLinearConv requantizes the exact int32 accumulator -- the arithmetic of the CUDA kernels, which the
GPU results must match bit for bit.
mode="fold": as "exact" with the library's optional single-multiplier requantization and folded residual tail.
"""
import numpy as np

from . import oracle as orc


def _qconv(c, x, mode):
    wz = np.asarray(c["w_zp"], np.int32)
    if mode == "emulate":
        return orc.qlinear_conv(x, c["x_scale"], 0, c["w"], c["w_scale"], wz, c["y_scale"], c["y_zp"], b=c["bias"],
                                strides=(c["stride"], c["stride"]), pads=(c["pad"], c["pad"]))
    acc = orc.conv_integer(x, c["w"], 0, wz, strides=(c["stride"], c["stride"]), pads=(c["pad"], c["pad"]))
    return orc.requantize(acc, c["x_scale"], c["w_scale"], c["y_scale"], c["y_zp"], bias=c["bias"], channel_axis=1, fold=(mode == "fold"))


def resnet50_forward(params, x, mode="exact", taps=None):
    """x: fp32 NCHW.  Returns fp32 logits.  taps (dict) receives the uint8 NCHW maps 'stem', 'block<i>' and 'pooled'."""
    xq = orc.quantize_linear(x, params["in_scale"], 0)
    h = _qconv(params["stem"], xq, mode)
    if taps is not None:
        taps["stem"] = h
    h = orc.maxpool_u8(h, 3, 2, 0, cover_all=True)
    h_scale = params["stem"]["y_scale"]
    for i, b in enumerate(params["blocks"]):
        h1 = _qconv(b["conv1"], h, mode)
        h2 = _qconv(b["conv2"], h1, mode)
        h3 = _qconv(b["conv3"], h2, mode)
        sc = _qconv(b["proj"], h, mode) if b["proj"] is not None else h
        sc_scale, sc_zp = b["res"]
        h = orc.qadd_relu(h3, b["conv3"]["y_scale"], b["conv3"]["y_zp"], sc, sc_scale, sc_zp, b["out_scale"], 0, relu=True, fold=(mode == "fold"))
        h_scale = b["out_scale"]
        if taps is not None:
            taps["block%d" % i] = h
    pooled = orc.global_avgpool_dq(h, h_scale, 0)
    if taps is not None:
        taps["pooled"] = pooled
    return orc.linear_f32(pooled, params["fc_w"], params["fc_b"])


def _lsb(a, b):
    d = np.abs(np.asarray(a).astype(np.int32) - np.asarray(b).astype(np.int32))
    return int(d.max()) if d.size else 0, int(np.count_nonzero(d)), int(d.size)


def resnet50_parity(params, x, gpu_taps, gpu_logits, fold=True, emulate_logits=None):
    """Checks a run of the library's ResNet-50 against the oracle on the same images.

    x: fp32 NCHW images; gpu_taps: the detailed taps of the library's forward pass over the same images as numpy NCHW arrays
    (``models.ResNet50Int8.forward(..., taps=, detail=True)``); gpu_logits: its logits.

    (1) whole network, bit for bit: the chain restated in the library's arithmetic (mode "fold" or "exact"), fed its own
        outputs from the input image on, must reproduce every tapped map.
    (2) every operator on its own against the REFERENCE's arithmetic (runtime/ops/quantize.cc:62-94: dequantize, fp32
        convolution, quantize; joins: DequantizeLinear x2, Add, Relu, QuantizeLinear), fed the very bytes the library's
        operator was fed: at most one output step apart.
    Returns a dict of counts; 'ok' says whether both bounds hold."""
    mode = "fold" if fold else "exact"
    ot = {}
    o_logits = resnet50_forward(params, x, mode=mode, taps=ot)
    mism = total = 0
    first_bad = None
    for k, v in ot.items():
        if k not in gpu_taps:
            continue
        g = np.asarray(gpu_taps[k])
        bad = int(np.count_nonzero(g != v))
        mism += bad
        total += int(v.size)
        if bad and first_bad is None:
            first_bad = k
    exact = {"mismatches": mism, "total": total, "first_differing_tap": first_bad,
             "logits_max_abs_difference": float(np.abs(o_logits - gpu_logits).max())}

    worst = {"max_lsb": 0, "mismatches": 0, "total": 0, "worst_layer": None, "layers": 0}

    def check(name, ref, got):
        mx, cnt, tot = _lsb(ref, got)
        worst["mismatches"] += cnt
        worst["total"] += tot
        worst["layers"] += 1
        if mx > worst["max_lsb"]:
            worst["max_lsb"], worst["worst_layer"] = mx, name
    xq = orc.quantize_linear(x, params["in_scale"], 0)
    check("stem", _qconv(params["stem"], xq, "emulate"), gpu_taps["stem"])
    h = gpu_taps["pool"]
    for i, b in enumerate(params["blocks"]):
        t = lambda k: gpu_taps["b%d_%s" % (i, k)]  # noqa: E731
        check(b["conv1"]["name"], _qconv(b["conv1"], h, "emulate"), t("h1"))
        check(b["conv2"]["name"], _qconv(b["conv2"], t("h1"), "emulate"), t("h2"))
        check(b["conv3"]["name"], _qconv(b["conv3"], t("h2"), "emulate"), t("h3"))
        if b["proj"] is not None:
            check(b["proj"]["name"], _qconv(b["proj"], h, "emulate"), t("sc"))
        sc_scale, sc_zp = b["res"]
        join = orc.qadd_relu(t("h3"), b["conv3"]["y_scale"], b["conv3"]["y_zp"], t("sc"), sc_scale, sc_zp, b["out_scale"], 0, relu=True)
        check("block%d_join" % i, join, gpu_taps["block%d" % i])
        h = gpu_taps["block%d" % i]
    out = {"images": int(x.shape[0]), "arithmetic": mode, "whole_network_vs_arithmetic_mirror": exact,
           "each_operator_vs_reference_chain_same_input": worst}
    if emulate_logits is not None:
        out["logits_top1_agreement_with_reference_chain"] = float(np.mean(np.argmax(emulate_logits, 1) == np.argmax(gpu_logits, 1)))
    out["ok"] = bool(mism == 0 and worst["max_lsb"] <= 1)
    return out


def mlp_forward(layers, act_scale, x, mode="emulate"):
    """QuantizeLinear -> QLinearMatMul x n -> DequantizeLinear; layers: list of dict(w_q [K,N] int8, w_scale)."""
    h = orc.quantize_linear(x, act_scale, 0)
    for l in layers:
        if mode == "emulate":
            h = orc.qlinear_matmul(h, act_scale, 0, l["w_q"], l["w_scale"], 0, act_scale, 0)
        else:
            acc = orc.matmul_integer(h, l["w_q"])
            h = orc.requantize(acc, act_scale, np.array([l["w_scale"]], np.float32), act_scale, 0)
    return orc.dequantize_linear(h, act_scale, 0)


def _mb_layer(c, x, mode):
    wz = np.asarray(c["w_zp"], np.int32)
    clamp = -1 if c["clamp"] is None else c["clamp"]
    s, p, g = (c["stride"], c["stride"]), (c["pad"], c["pad"]), c["group"]
    if mode == "emulate":
        return orc.qlinear_conv(x, c["x_scale"], c["x_zp"], c["w"], c["w_scale"], wz, c["y_scale"], c["y_zp"], b=c["bias"], strides=s, pads=p,
                                group=g, clamp_hi_q=clamp)
    acc = orc.conv_integer(x, c["w"], c["x_zp"], wz, strides=s, pads=p, group=g)
    return orc.requantize(acc, c["x_scale"], c["w_scale"], c["y_scale"], c["y_zp"], bias=c["bias"], channel_axis=1, clamp_hi_q=clamp,
                          fold=(mode == "fold"))


def mobilenetv2_forward(params, x, mode="exact", taps=None):
    """params: ``models.MobileNetV2Int8.export_numpy()``; x: fp32 NCHW.  Modes as in resnet50_forward."""
    xq = orc.quantize_linear(x, params["in_scale"], 0)
    h = _mb_layer(params["stem"], xq, mode)
    if taps is not None:
        taps["stem"] = h
    for i, b in enumerate(params["blocks"]):
        inp = h
        if b["expand"] is not None:
            h = _mb_layer(b["expand"], h, mode)
        h = _mb_layer(b["dw"], h, mode)
        h = _mb_layer(b["project"], h, mode)
        if b["residual"]:
            h = orc.qadd_relu(h, b["project"]["y_scale"], b["project"]["y_zp"], inp, b["res"][0], b["res"][1], b["out_scale"], b["out_zp"],
                              relu=False, fold=(mode == "fold"))
        if taps is not None:
            taps["block%d" % i] = h
    h = _mb_layer(params["head"], h, mode)
    pooled = orc.global_avgpool_dq(h, params["head"]["y_scale"], 0)
    if taps is not None:
        taps["pooled"] = pooled
    return orc.linear_f32(pooled, params["fc_w"], params["fc_b"])


def _f32(v):
    return np.float32(np.asarray(v).reshape(()))


def _sigmoid(v):
    # 1 / (1 + exp(-x)); the reference's generated kernel writes tanh(x / 2) / 2 + 1 / 2 (compiler/nvrtc_builder.cc:133-136), the
    # same function within 1e-5 relative
    one = np.float32(1.0)
    return one / (one + np.exp(-v))


_ONNX_DTYPE = {1: np.float32, 2: np.uint8, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.bool_, 10: np.float16, 11: np.float64}
_EW = {"Add": np.add, "Sub": np.subtract, "Mul": np.multiply, "Tanh": np.tanh, "Sigmoid": _sigmoid, "Exp": np.exp, "Identity": lambda v: v}


def run_program(program, inputs, trace=None, conv_mode="emulate"):
    """CPU evaluation of a `run_onnx` program (the instruction list `chainer-compiler_b200/run_onnx.py::compile_model`
    produces) with the oracle's ops: the checker for the quantized graph the reference's `--quantize` pass builds
    (compiler/quantize.cc:142-281).  program: an object with .insts (op, inputs, outputs, attrs), .constants (numpy),
    .outputs.  Glue ops are numpy expressions.  conv_mode: how a QLinearConv node is evaluated -- "emulate" as the reference
    does (dequantize, fp32 convolution, quantize), "exact" by requantizing the exact int32 accumulator (the arithmetic of the
    CUDA kernels; the two agree within one step of the output scale)."""
    env = dict(program.constants)
    env.update({k: np.asarray(v) for k, v in inputs.items()})
    for inst in program.insts:
        a, x, op = inst.attrs, [env[i] if i != "" else None for i in inst.inputs], inst.op
        if op == "ReduceMinMax":
            out = [np.float32(x[0].min()), np.float32(x[0].max())]
        elif op == "DynamicQuantParamsU8":
            rmin, rmax = np.float32(x[0]), np.float32(x[1])
            scale = np.float32((rmax - rmin) / np.float32(255.0)) if rmax != rmin else np.float32(1.0)
            out = [scale, np.uint8(int(np.clip(np.floor(np.float32((np.float32(0.0) - rmin) / scale)), 0, 255)))]
        elif op == "QuantizeLinear":
            zp = np.asarray(x[2]).reshape(()) if len(x) > 2 else np.uint8(0)
            out = [orc.quantize_linear(x[0], _f32(x[1]), int(zp), out_dtype=zp.dtype)]
        elif op == "DequantizeLinear":
            out = [orc.dequantize_linear(x[0], _f32(x[1]), int(np.asarray(x[2]).reshape(())) if len(x) > 2 else 0)]
        elif op in ("ConvInteger", "QLinearConv"):
            auto_pad = a.get("auto_pad", "NOTSET")
            auto_pad = "" if auto_pad == "NOTSET" else auto_pad
            pads = list(a.get("pads", []))
            strides, pads, group = tuple(a.get("strides", [])), tuple(pads[:len(pads) // 2]), a.get("group", 1)
            if op == "ConvInteger":
                zx = int(np.asarray(x[2]).reshape(())) if len(x) > 2 else None
                zw = np.asarray(x[3]).astype(np.int32) if len(x) > 3 else None
                out = [orc.conv_integer(x[0], x[1], zx, zw, strides, pads, group, auto_pad)]
            else:
                zy = np.asarray(x[7]).reshape(())
                bias = x[8] if len(x) > 8 and inst.inputs[8] != "" else None
                if a.get("quantize_input"):  # run_onnx's stem peephole: the QuantizeLinear in front of the convolution
                    x[0] = orc.quantize_linear(x[0], _f32(x[1]), int(np.asarray(x[2]).reshape(())))
                if conv_mode == "exact":
                    acc = orc.conv_integer(x[0], x[3], int(np.asarray(x[2]).reshape(())), np.asarray(x[5]).astype(np.int32).reshape(-1), strides, pads, group, auto_pad)
                    out = [orc.requantize(acc, _f32(x[1]), np.asarray(x[4], np.float32), _f32(x[6]), int(zy), bias=bias, channel_axis=1, y_dtype=zy.dtype.type)]
                else:
                    out = [orc.qlinear_conv(x[0], _f32(x[1]), int(np.asarray(x[2]).reshape(())), x[3], np.asarray(x[4], np.float32), np.asarray(x[5]),
                                            _f32(x[6]), zy[()], bias, strides, pads, group, auto_pad)]
                if a.get("residual"):
                    # the join run_onnx's second peephole moved into the convolution: DequantizeLinear x2, Add, [Relu], QuantizeLinear
                    out = [orc.qadd_relu(out[0], _f32(x[6]), int(zy), x[9], _f32(x[10]), int(np.asarray(x[11]).reshape(())), _f32(x[12]),
                                         int(np.asarray(x[13]).reshape(())), relu=bool(a.get("res_relu", 0)))]
                if a.get("pool"):  # ... and the MaxPool(3, 2, 0) behind it (2 = ceil_mode)
                    out = [orc.maxpool_u8(out[0], 3, 2, 0, cover_all=(a["pool"] == 2))]
        elif op == "MatMulInteger":
            out = [orc.matmul_integer(x[0], x[1], np.asarray(x[2]).reshape(-1) if len(x) > 2 else None,
                                      np.asarray(x[3]).reshape(-1) if len(x) > 3 else None)]
        elif op == "QLinearMatMul":
            zy = np.asarray(x[7]).reshape(())
            out = [orc.qlinear_matmul(x[0], _f32(x[1]), int(np.asarray(x[2]).reshape(())), x[3], _f32(x[4]), int(np.asarray(x[5]).reshape(())),
                                      _f32(x[6]), int(zy), y_dtype=zy.dtype.type)]
        elif op == "ElementWiseNvrtc":
            # the group's member nodes one by one, as the reference's CPU path runs a fusion group (compiler/chxvm/emitter.cc:702-726)
            local = {}
            get = lambda k: local[k] if k in local else env[k]  # noqa: E731
            for mop, mins, mouts in a["members"]:
                v = [np.asarray(get(k), np.float32) for k in mins]
                local[mouts[0]] = _EW[mop](*v).astype(np.float32)
            out = [np.broadcast_to(local[o], np.broadcast_shapes(*[np.shape(env[k]) for k in inst.inputs])).copy() for o in inst.outputs]
        elif op == "BatchNormalization":
            shape = [1, -1] + [1] * (x[0].ndim - 2)
            f = np.float32
            out = [((x[0] - x[3].reshape(shape)) / np.sqrt(x[4].reshape(shape) + f(a.get("epsilon", 1e-5))) * x[1].reshape(shape) + x[2].reshape(shape)).astype(f)]
        elif op == "ScaleProduct":
            m = (np.asarray(x[0], np.float32) * np.asarray(x[1], np.float32)).astype(np.float32)
            out = [m.reshape(a["shape"]) if a.get("shape") else m]
        elif op == "Cast":
            to = a.get("to", "float32")
            out = [np.asarray(x[0]).astype(to if isinstance(to, str) else _ONNX_DTYPE[int(to)])]
        elif op in ("ReduceMin", "ReduceMax"):
            v = np.float32(x[0].min() if op == "ReduceMin" else x[0].max())
            out = [v.reshape([1] * x[0].ndim) if a.get("keepdims", 1) else v.reshape(())]
        elif op == "Floor":
            out = [np.floor(x[0])]
        elif op in ("Add", "Sub", "Mul", "Div"):
            f = {"Add": np.add, "Sub": np.subtract, "Mul": np.multiply, "Div": np.divide}[op]
            out = [f(x[0], x[1]).astype(np.float32)]
        elif op == "Relu":
            out = [np.maximum(x[0], np.float32(0))]
        elif op == "Reshape":
            shape = [x[0].shape[i] if d == 0 else int(d) for i, d in enumerate(x[1])]
            out = [x[0].reshape(shape)]
        elif op == "QAddU8":
            # DequantizeLinear, DequantizeLinear, Add, [Relu], QuantizeLinear as run_onnx's peephole groups them
            out = [orc.qadd_relu(x[0], _f32(x[1]), int(np.asarray(x[2]).reshape(())), x[3], _f32(x[4]), int(np.asarray(x[5]).reshape(())), _f32(x[6]),
                                 int(np.asarray(x[7]).reshape(())), relu=bool(a.get("relu", 0)))]
        elif op == "GlobalAveragePool":
            out = [x[0].astype(np.float32).mean(axis=tuple(range(2, x[0].ndim)), keepdims=True, dtype=np.float32)]
        elif op == "Flatten":
            ax = a.get("axis", 1)
            out = [x[0].reshape(int(np.prod(x[0].shape[:ax])), -1)]
        elif op == "Gemm":
            if a.get("transA", 0) or not a.get("transB", 0) or a.get("alpha", 1.0) != 1.0 or a.get("beta", 1.0) != 1.0:
                raise NotImplementedError("Gemm other than x . w^T + b")
            out = [orc.linear_f32(x[0], x[1], x[2] if len(x) > 2 else None)]
        elif op == "MaxPool" and x[0].dtype == np.uint8:
            k, s = a["kernel_shape"], a.get("strides", [1, 1])
            p = list(a.get("pads", [0, 0, 0, 0]))
            if k[0] != k[1] or s[0] != s[1] or len(set(p)) != 1:
                raise NotImplementedError("uint8 MaxPool with a non-square window")
            out = [orc.maxpool_u8(x[0], k[0], s[0], p[0], cover_all=bool(a.get("ceil_mode", 0)))]
        elif op == "MaxPool":
            k, s = a["kernel_shape"], a.get("strides", [1, 1])
            N, C, H, W = x[0].shape
            Ho, Wo = (H - k[0]) // s[0] + 1, (W - k[1]) // s[1] + 1
            y = np.full((N, C, Ho, Wo), -np.inf, np.float32)
            for i in range(k[0]):
                for j in range(k[1]):
                    y = np.maximum(y, x[0][:, :, i:i + s[0] * Ho:s[0], j:j + s[1] * Wo:s[1]])
            out = [y]
        else:
            raise NotImplementedError(op)
        for name, v in zip(inst.outputs, out):
            env[name] = v
            if trace is not None:
                trace[name] = v
    return [(o, env[o]) for o in program.outputs]
