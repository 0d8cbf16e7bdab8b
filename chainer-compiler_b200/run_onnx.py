"""`run_onnx`: loads an ONNX model or test directory, optionally rewrites it with the reference's quantization pass, and runs
it on the VM ops of this package (reference entry point: tools/run_onnx.cc:289-315, Python wrapper tools/run_onnx.py;
`run_onnx(argv)` mirrors tools/run_onnx_core.cc:18-21).

    python chainer-compiler_b200/run_onnx.py --test DIR [--quantize] [-d cuda:0] [-I 3] [--rtol 1e-4] [--atol 1e-6]

What runs where: with `--quantize` every Conv (without bias input) and MatMul becomes the dynamic IntegerOps sequence of
compiler/quantize.cc:142-281 -- ReduceMin / ReduceMax -> scale, zero point -> QuantizeLinear -> ConvInteger / MatMulInteger
-> Cast -> Mul -- and those ops run on this package's kernels (ops.MinMax, ops.QuantizeLinear, ops.ConvInteger,
ops.MatMulInteger).  The float glue between them (Add, Relu, MaxPool, Reshape, Cast, Mul, ...) is outside the quantized hot
path and runs as torch tensor expressions on the same device.  Without `--quantize` a float Conv / MatMul has no kernel here
and is refused, unless `--float_ops_via_torch` asks for the torch expression (useful to check a test directory's expected
outputs; not a code path of the product).

Flags kept from the reference: positional or --test DIR / --onnx FILE, -d/--device, -I/--iterations, --rtol, --atol,
--equal_nan, --no_check_values, --always_show_diff, --check_nans, --check_infs, --dump_outputs_dir, --report_json,
--verbose/-v, --quiet/-q, --quantize, --disable_per_channel_quantize, --compile_only, --dump_chxvm (prints the program)."""
import argparse
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


# ---- program ---------------------------------------------------------------------------------------------------------
class Inst:
    def __init__(self, op, inputs, outputs, **attrs):
        self.op, self.inputs, self.outputs, self.attrs = op, list(inputs), list(outputs), attrs

    def __repr__(self):
        a = ", ".join("%s=%r" % kv for kv in self.attrs.items() if not isinstance(kv[1], np.ndarray))
        return "%s(%s%s) -> (%s)" % (self.op, ", ".join("$" + i for i in self.inputs), (", " + a) if a else "", ", ".join("$" + o for o in self.outputs))


class Program:
    def __init__(self, insts, constants, inputs, outputs):
        self.insts, self.constants, self.inputs, self.outputs = insts, constants, inputs, outputs

    def dump(self):
        return "\n".join(repr(i) for i in self.insts)


def _fold_constants(model):
    """Reshape / Cast of initializers become initializers (the reference's constant propagation does the same before the
    weights reach the quantizer)."""
    consts = dict(model.initializers)
    nodes = []
    for n in model.nodes:
        if n.op_type == "Reshape" and all(i in consts for i in n.inputs):
            consts[n.outputs[0]] = consts[n.inputs[0]].reshape([int(d) for d in consts[n.inputs[1]]])
        else:
            nodes.append(n)
    return nodes, consts


def quantize_weight(w, per_channel, to_int8):
    """compiler/quantize.cc:70-129 through the library's host quantizer (chxq_quantize_weights_host)."""
    from chainer_compiler_b200.models import quantize_weights
    q, scale, zp = quantize_weights(np.ascontiguousarray(w, np.float32), per_channel=per_channel, to_int8=to_int8)
    return q, scale.astype(np.float32), zp.astype(q.dtype)


def compile_model(model, quantize=False, per_channel=True, asymmetric_input_types=False):
    """ONNX graph -> Program.  quantize: the reference's `--quantize` (dynamic, IntegerOps; weights uint8 unless
    asymmetric_input_types, which makes them int8: compiler/quantize.cc:392-400)."""
    nodes, consts = _fold_constants(model)
    insts, tmp = [], [0]

    def fresh(base):
        tmp[0] += 1
        return "%s@q%d" % (base, tmp[0])

    def quantized_activation(x):
        # compiler/quantize.cc:172-207, uint8 inputs (Linear_NonScaled)
        rmin, rmax, scale, zp, xq = fresh("rmin"), fresh("rmax"), fresh("scale"), fresh("zp"), fresh(x)
        insts.append(Inst("ReduceMinMax", [x], [rmin, rmax]))
        insts.append(Inst("DynamicQuantParamsU8", [rmin, rmax], [scale, zp]))
        insts.append(Inst("QuantizeLinear", [x, scale, zp], [xq]))
        return xq, scale, zp

    for n in nodes:
        if quantize and n.op_type == "Conv" and len(n.inputs) == 2 and n.inputs[1] in consts:
            w = consts[n.inputs[1]]
            wq, ws, wz = quantize_weight(w, per_channel, asymmetric_input_types)
            wname, wsn, wzn = fresh("wq"), fresh("wscale"), fresh("wzp")
            consts[wname], consts[wsn], consts[wzn] = wq, ws, wz
            xq, xs, xz = quantized_activation(n.inputs[0])
            acc, accf, mul = fresh("convint"), fresh("cast"), fresh("scales")
            insts.append(Inst("ConvInteger", [xq, wname, xz, wzn], [acc], strides=n.attrs.get("strides", []), pads=n.attrs.get("pads", []),
                              group=n.attrs.get("group", 1), auto_pad=n.attrs.get("auto_pad", "NOTSET"), dilations=n.attrs.get("dilations", [])))
            insts.append(Inst("Cast", [acc], [accf], to="float32"))
            insts.append(Inst("ScaleProduct", [xs, wsn], [mul], shape=[-1] + [1] * (w.ndim - 2) if ws.size > 1 else []))
            insts.append(Inst("Mul", [accf, mul], [n.outputs[0]]))
        elif quantize and n.op_type == "MatMul":
            a, b = n.inputs
            if b in consts:
                bq, bs, bz = quantize_weight(consts[b], False, asymmetric_input_types)
                bname, bsn, bzn = fresh("wq"), fresh("wscale"), fresh("wzp")
                consts[bname], consts[bsn], consts[bzn] = bq, bs.reshape(()), bz.reshape(-1)[:1]
            else:
                bname, bsn, bzn = quantized_activation(b)
            if a in consts:
                aq, as_, az = quantize_weight(consts[a], False, False)
                aname, asn, azn = fresh("wq"), fresh("wscale"), fresh("wzp")
                consts[aname], consts[asn], consts[azn] = aq, as_.reshape(()), az.reshape(-1)[:1]
            else:
                aname, asn, azn = quantized_activation(a)
            acc, accf, mul = fresh("matmulint"), fresh("cast"), fresh("scales")
            insts.append(Inst("MatMulInteger", [aname, bname, azn, bzn], [acc]))
            insts.append(Inst("Cast", [acc], [accf], to="float32"))
            insts.append(Inst("ScaleProduct", [asn, bsn], [mul], shape=[]))
            insts.append(Inst("Mul", [accf, mul], [n.outputs[0]]))
        else:
            insts.append(Inst(n.op_type, n.inputs, n.outputs, **n.attrs))
    return Program(insts, consts, list(model.inputs), list(model.outputs))


# ---- execution -------------------------------------------------------------------------------------------------------
def dynamic_params_u8(rmin, rmax):
    """scale = (rmax - rmin) / 255; zero point = uint8(floor((0 - rmin) / scale)), in fp32 as the emitted Sub / Div / Floor /
    Cast nodes compute them (compiler/quantize.cc:196-207).  The range is NOT forced to include zero (unlike weights).  A
    constant input (rmax == rmin) would divide by zero in the reference; scale 1 is used here."""
    rmin, rmax = np.float32(rmin), np.float32(rmax)
    scale = np.float32((rmax - rmin) / np.float32(255.0)) if rmax != rmin else np.float32(1.0)
    zp = np.floor(np.float32((np.float32(0.0) - rmin) / scale))
    return scale, np.uint8(int(np.clip(zp, 0, 255)))


def _pool_pads(attrs, ndim):
    pads = list(attrs.get("pads", [])) or [0] * (2 * ndim)
    return pads


class Executor:
    """Runs a Program on one CUDA device.  Quantized ops go through chainer_compiler_b200.ops; glue ops are torch expressions."""

    def __init__(self, program, device="cuda:0", float_ops_via_torch=False):
        import torch
        sys.path.insert(0, ROOT)
        import __graft_entry__ as entry
        entry.load_package()
        from chainer_compiler_b200 import ops
        self.torch, self.ops = torch, ops
        self.program, self.float_ok = program, float_ops_via_torch
        if not str(device).startswith("cuda"):
            raise SystemExit("run_onnx: device %r is not supported, this package runs on CUDA devices only" % (device,))
        self.device = torch.device(device if ":" in str(device) else "cuda:0")
        self.consts = {}
        for k, v in program.constants.items():
            self.consts[k] = torch.from_numpy(np.ascontiguousarray(v)).to(self.device)
        self.host_consts = program.constants

    def run(self, inputs, trace=None):
        t, ops = self.torch, self.ops
        env = dict(self.consts)
        host = {}  # host-side scalars (dynamic quantization parameters)
        for k, v in inputs.items():
            env[k] = t.from_numpy(np.ascontiguousarray(v)).to(self.device)
        for inst in self.program.insts:
            a = inst.attrs
            x = [env.get(i) if i in env else host.get(i) for i in inst.inputs]
            op = inst.op
            if op == "ReduceMinMax":
                mm = ops.MinMax(x[0].contiguous()).cpu().numpy()  # the device-to-host read the reference does per scalar argument
                host[inst.outputs[0]], host[inst.outputs[1]] = np.float32(mm[0]), np.float32(mm[1])
            elif op == "DynamicQuantParamsU8":
                host[inst.outputs[0]], host[inst.outputs[1]] = dynamic_params_u8(host[inst.inputs[0]], host[inst.inputs[1]])
            elif op == "QuantizeLinear":
                env[inst.outputs[0]] = ops.QuantizeLinear(x[0].contiguous(), host[inst.inputs[1]], host[inst.inputs[2]])
            elif op == "ConvInteger":
                if any(d != 1 for d in a.get("dilations", [])):
                    raise NotImplementedError("ConvInteger: dilation must be 1 (compiler/chxvm/simple_node_emitter.cc:655)")
                zx = host[inst.inputs[2]]
                auto_pad = a.get("auto_pad", "NOTSET")
                env[inst.outputs[0]] = ops.ConvInteger(x[0], x[1], zx, x[3], tuple(a.get("strides", [])), self._sym_pads(a.get("pads", [])), a.get("group", 1),
                                                       "" if auto_pad == "NOTSET" else auto_pad)
            elif op == "MatMulInteger":
                za = x[2] if inst.inputs[2] in env else t.tensor([int(host[inst.inputs[2]])], dtype=t.uint8, device=self.device)
                zb = x[3] if inst.inputs[3] in env else t.tensor([int(host[inst.inputs[3]])], dtype=t.uint8, device=self.device)
                env[inst.outputs[0]] = ops.MatMulInteger(x[0].contiguous(), x[1].contiguous(), za, zb)
            elif op == "ScaleProduct":
                s0 = x[0] if inst.inputs[0] in env else t.tensor(float(host[inst.inputs[0]]), dtype=t.float32, device=self.device)
                s1 = x[1] if inst.inputs[1] in env else t.tensor(float(host[inst.inputs[1]]), dtype=t.float32, device=self.device)
                m = s0 * s1
                env[inst.outputs[0]] = m.reshape(a["shape"]) if a.get("shape") else m
            elif op == "Cast":
                env[inst.outputs[0]] = x[0].to(getattr(t, a["to"]) if isinstance(a["to"], str) else t.float32)
            elif op in ("Add", "Sub", "Mul", "Div"):
                f = {"Add": t.add, "Sub": t.sub, "Mul": t.mul, "Div": t.div}[op]
                env[inst.outputs[0]] = f(x[0], x[1])
            elif op == "Relu":
                env[inst.outputs[0]] = t.relu(x[0])
            elif op == "Reshape":
                shape = [int(d) for d in self.host_consts[inst.inputs[1]]] if inst.inputs[1] in self.host_consts else [int(d) for d in x[1].cpu()]
                shape = [x[0].shape[i] if d == 0 else d for i, d in enumerate(shape)]
                env[inst.outputs[0]] = x[0].reshape(shape)
            elif op == "MaxPool":
                k, s = a["kernel_shape"], a.get("strides", [1] * len(a["kernel_shape"]))
                p = _pool_pads(a, len(k))
                if any(p[i] != p[i + len(k)] for i in range(len(k))):
                    raise NotImplementedError("MaxPool: asymmetric pads")
                env[inst.outputs[0]] = t.nn.functional.max_pool2d(x[0], k, s, p[:len(k)])
            elif op == "Flatten":
                ax = a.get("axis", 1)
                env[inst.outputs[0]] = x[0].reshape(int(np.prod(x[0].shape[:ax])), -1)
            elif op in ("Conv", "MatMul", "Gemm"):
                if not self.float_ok:
                    raise SystemExit("run_onnx: float %s has no kernel in this package; run with --quantize (or --float_ops_via_torch to "
                                     "evaluate it as a torch expression outside the product path)" % op)
                if op == "Conv":
                    auto_pad = a.get("auto_pad", "NOTSET")
                    pads = self._sym_pads(a.get("pads", []))
                    xin = x[0]
                    if auto_pad == "SAME_UPPER":
                        from chainer_compiler_b200.ops import conv_geometry_from_shapes  # the library's geometry rule
                        g = conv_geometry_from_shapes(tuple(xin.shape), 6, tuple(x[1].shape), 2, tuple(a.get("strides", [])), (), a.get("group", 1), "SAME_UPPER")
                        xin = t.nn.functional.pad(xin, (g.pad_left, g.pad_right, g.pad_top, g.pad_bottom))
                        pads = (0, 0)
                    env[inst.outputs[0]] = t.nn.functional.conv2d(xin, x[1], x[2] if len(x) > 2 else None, tuple(a.get("strides", [1, 1])), pads or 0, 1,
                                                                  a.get("group", 1))
                elif op == "MatMul":
                    env[inst.outputs[0]] = x[0] @ x[1]
                else:
                    A = x[0].t() if a.get("transA", 0) else x[0]
                    B = x[1].t() if a.get("transB", 0) else x[1]
                    y = a.get("alpha", 1.0) * (A @ B)
                    env[inst.outputs[0]] = y + a.get("beta", 1.0) * x[2] if len(x) > 2 else y
            else:
                raise NotImplementedError("run_onnx: op %s" % op)
            if trace is not None:
                for o in inst.outputs:
                    trace[o] = env[o] if o in env else host[o]
        ops.device_status()
        return [(o, env[o]) for o in self.program.outputs]

    @staticmethod
    def _sym_pads(pads):
        pads = list(pads)
        if not pads:
            return ()
        n = len(pads) // 2
        if pads[:n] != pads[n:]:
            raise NotImplementedError("asymmetric pads (compiler/chxvm/simple_node_emitter.cc:76-86)")
        return tuple(pads[:n])


# ---- entry point -----------------------------------------------------------------------------------------------------
def parse_args(argv):
    ap = argparse.ArgumentParser(prog="run_onnx", description=__doc__.split("\n\n")[0])
    ap.add_argument("positional", nargs="?", help="test directory or .onnx file")
    ap.add_argument("--test")
    ap.add_argument("--onnx")
    ap.add_argument("-d", "--device", default="cuda")
    ap.add_argument("-I", "--iterations", type=int, default=1)
    ap.add_argument("--rtol", type=float, default=1e-4)
    ap.add_argument("--atol", type=float, default=1e-6)
    ap.add_argument("--equal_nan", action="store_true")
    ap.add_argument("--no_check_values", action="store_true")
    ap.add_argument("--always_show_diff", action="store_true")
    ap.add_argument("--check_nans", action="store_true")
    ap.add_argument("--check_infs", action="store_true")
    ap.add_argument("--dump_outputs_dir")
    ap.add_argument("--report_json")
    ap.add_argument("--compile_only", action="store_true")
    ap.add_argument("--dump_chxvm", action="store_true")
    ap.add_argument("--quantize", action="store_true")
    ap.add_argument("--disable_per_channel_quantize", action="store_true")
    ap.add_argument("--float_ops_via_torch", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-q", "--quiet", action="store_true")
    return ap.parse_args(argv)


def run_onnx(argv):
    """Returns 0 when every checked output is within tolerance, 1 otherwise (the reference CHECK-fails instead)."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from chainer_compiler_b200 import onnx_io
    args = parse_args(argv)
    target = args.test or args.onnx or args.positional
    if not target:
        raise SystemExit("run_onnx: give a test directory or an .onnx file")
    if os.path.isdir(target):
        model, cases = onnx_io.load_test_dir(target)
    else:
        model, cases = onnx_io.load_model(target), []
    program = compile_model(model, quantize=args.quantize, per_channel=not args.disable_per_channel_quantize)
    if args.dump_chxvm:
        print(program.dump())
    if args.compile_only:
        return 0
    import torch
    ex = Executor(program, args.device, args.float_ops_via_torch)
    failures, elapsed, report = 0, [], []
    for ci, (ins, expected) in enumerate(cases):
        outs = None
        for it in range(max(1, args.iterations)):
            torch.cuda.synchronize(ex.device)
            t0 = time.perf_counter()
            outs = ex.run(ins)
            torch.cuda.synchronize(ex.device)
            if it > 0 or args.iterations == 1:  # the first iteration is discarded when there are several (tools/run_onnx.cc:468-469)
                elapsed.append(time.perf_counter() - t0)
        got = {k: v.detach().cpu().numpy() for k, v in outs}
        if args.dump_outputs_dir:
            os.makedirs(args.dump_outputs_dir, exist_ok=True)
            for k, v in got.items():
                np.save(os.path.join(args.dump_outputs_dir, "%d_%s.npy" % (ci, k.replace("/", "_"))), v)
        for name, want in expected:
            y = got.get(name)
            ok = y is not None and y.shape == want.shape
            if ok and args.check_nans and np.isnan(y).any():
                ok = False
            if ok and args.check_infs and np.isinf(y).any():
                ok = False
            if ok and not args.no_check_values:
                ok = bool(np.allclose(y, want, rtol=args.rtol, atol=args.atol, equal_nan=args.equal_nan))
            if (not ok or args.always_show_diff) and not args.quiet and y is not None and y.shape == want.shape:
                d = np.abs(y.astype(np.float64) - want.astype(np.float64))
                print("case %d output %s: max abs diff %.6g, max rel diff %.6g" % (ci, name, d.max(), (d / np.maximum(np.abs(want), 1e-30)).max()))
            if not ok:
                failures += 1
            report.append({"case": ci, "output": name, "ok": bool(ok)})
        if args.verbose and not args.quiet:
            print("case %d: %s" % (ci, {k: v.shape for k, v in got.items()}))
    if not cases and not args.quiet:
        print("run_onnx: model compiled (%d instructions); no test data to run" % len(program.insts))
    avg_ms = 1000.0 * float(np.mean(elapsed)) if elapsed else 0.0
    if not args.quiet:
        print("Elapsed: %.3f msec" % avg_ms)
        print("OK!" if failures == 0 else "FAILED: %d output(s) out of tolerance" % failures)
    if args.report_json:
        with open(args.report_json, "w") as f:
            json.dump({"elapsed_ms": avg_ms, "failures": failures, "outputs": report, "quantize": bool(args.quantize)}, f)
    return 0 if failures == 0 else 1


if __name__ == "__main__":
    sys.exit(run_onnx(sys.argv[1:]))
