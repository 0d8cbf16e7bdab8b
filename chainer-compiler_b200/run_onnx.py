"""`run_onnx`: loads an ONNX model or test directory, optionally rewrites it with the reference's quantization pass, and runs
it on the VM ops of this package (reference entry point: tools/run_onnx.cc:289-315, Python wrapper tools/run_onnx.py;
`run_onnx(argv)` mirrors tools/run_onnx_core.cc:18-21).

    python chainer-compiler_b200/run_onnx.py --test DIR [--quantize] [-d cuda:0] [-I 3] [--rtol 1e-4] [--atol 1e-6]

What runs where.  QuantizeLinear, DequantizeLinear, QLinearConv, QLinearMatMul, ConvInteger and MatMulInteger nodes of the
file run on this package's kernels; their scale / zero-point operands may be initializers or graph inputs (one element each,
read on the host once per call as the reference's GetScalar does, runtime/chxvm_var.cc:70-76).  With `--quantize` every Conv
without a bias input and every MatMul first becomes the dynamic IntegerOps sequence of compiler/quantize.cc:142-281 --
ReduceMin / ReduceMax -> scale, zero point -> QuantizeLinear -> ConvInteger / MatMulInteger -> Cast -> Mul.  With
`--fuse_operations --use_nvrtc` the float Add / Sub / Mul / Tanh / Sigmoid / Exp glue is grouped as the reference groups it
(compiler/fusion_elementwise.cc:10-40) and every group runs as one generated kernel (ElementWiseNvrtc).  The remaining float
glue (Relu, MaxPool, Reshape, Cast, BatchNormalization, ...) is outside the quantized hot path and runs as torch tensor
expressions on the same device.  A float Conv / MatMul / Gemm has no kernel here and is refused, unless
`--float_ops_via_torch` asks for the torch expression (useful to check a test directory's expected outputs; not a code path of
the product).

Compile passes, in the reference's order (compiler/passes.cc:121-128): constant folding of Reshape over initializers,
Quantize, then MergeConvBN (compiler/merge.cc:142-215) over the Conv nodes that are still float.  `--fold_bn_first` swaps the
last two, so that a Conv + BatchNormalization pair is quantized as one convolution; the bias the merge creates is then added
in fp32 after the scale-back Mul (the reference leaves a Conv with bias unquantized, compiler/quantize.cc:366-369).

On a statically quantized graph two peepholes run unless `--no_peephole` is given: DequantizeLinear x2 + Add + [Relu] +
QuantizeLinear (a residual join) becomes one uint8 kernel, and a QLinearConv whose only reader is such a join takes it into its
epilogue; both keep every output bit.  Convolutions with constant weights are packed once and run on the tensor-core kernels
over channels_last activations.  Options of this build beyond the reference's: `--fold_scales` (one fp32 multiplier per output
channel in the requantization instead of a multiply and a divide; up to one output step of difference) and `--cuda_graph`
(with -I > 1 a program without device-to-host reads is captured after the first iteration and replayed).

Flags kept from the reference: positional or --test DIR / --onnx FILE, -d/--device, -I/--iterations, --rtol, --atol,
--equal_nan, --no_check_values, --always_show_diff, --check_nans, --check_infs, --dump_outputs_dir (one
`<instruction id, 5 digits>_<value name>.npy` per instruction output, runtime/chxvm.cc:70-92), --chrome_tracing FILE (one
complete event per instruction, runtime/chrome_tracing.cc:39-67), --report_json, --trace/-t, --verbose/-v, --quiet/-q,
--quantize, --disable_per_channel_quantize, --fuse_operations, --use_nvrtc, --compile_only, --skip_inference, --dump_chxvm,
--dump_onnx, --out_onnx FILE, --backend (only `chxvm`), --skip_runtime_type_check and --use_cuda (accepted, no effect: there is
one backend and one device kind)."""
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
        a = ", ".join("%s=%r" % kv for kv in self.attrs.items() if not isinstance(kv[1], (np.ndarray, list)) or kv[0] in ("strides", "pads", "kernel_shape"))
        return "%s(%s%s) -> (%s)" % (self.op, ", ".join("$" + i for i in self.inputs), (", " + a) if a else "", ", ".join("$" + o for o in self.outputs))


class Program:
    def __init__(self, insts, constants, inputs, outputs):
        self.insts, self.constants, self.inputs, self.outputs = insts, constants, inputs, outputs

    def dump(self):
        return "\n".join("%5d: %r" % (pc, i) for pc, i in enumerate(self.insts))


def _fold_constants(model):
    """Reshape of initializers becomes an initializer, Constant nodes become initializers (the reference's constant
    propagation does the same before the weights reach the quantizer)."""
    consts = dict(model.initializers)
    nodes = []
    for n in model.nodes:
        if n.op_type == "Reshape" and all(i in consts for i in n.inputs):
            consts[n.outputs[0]] = consts[n.inputs[0]].reshape([int(d) for d in consts[n.inputs[1]]])
        elif n.op_type == "Constant" and isinstance(n.attrs.get("value"), np.ndarray):
            consts[n.outputs[0]] = n.attrs["value"]
        else:
            nodes.append(n)
    return nodes, consts


def quantize_weight(w, per_channel, to_int8):
    """compiler/quantize.cc:70-129 through the library's host quantizer (chxq_quantize_weights_host)."""
    from chainer_compiler_b200.models import quantize_weights
    q, scale, zp = quantize_weights(np.ascontiguousarray(w, np.float32), per_channel=per_channel, to_int8=to_int8)
    return q, scale.astype(np.float32), zp.astype(q.dtype)


def merge_conv_bn(nodes, consts, graph_outputs=(), only=None):
    """MergeConvBN (compiler/merge.cc:142-215): a Conv whose only user is a one-output BatchNormalization with constant
    scale, bias, mean and variance, and whose own weight (and bias, if any) is constant, becomes one Conv:
        s = scale / sqrt(var + eps);  W'[m] = W[m] * s[m];  b' = (b - mean) * s + bn_bias      (all fp32)
    Returns the new node list; the new parameters are added to `consts`.  only: a predicate that selects the Conv nodes the
    pass may touch."""
    from chainer_compiler_b200.onnx_io import Node
    users = {}
    for n in nodes:
        for i in n.inputs:
            users.setdefault(i, []).append(n)
    out, dropped = [], set()
    for n in nodes:
        if id(n) in dropped:
            continue
        if n.op_type != "Conv" or n.outputs[0] in graph_outputs or len(users.get(n.outputs[0], [])) != 1 or (only and not only(n)):
            out.append(n)
            continue
        bn = users[n.outputs[0]][0]
        ok = bn.op_type == "BatchNormalization" and bn.inputs[0] == n.outputs[0] and len(bn.outputs) == 1 and len(bn.inputs) == 5
        ok = ok and all(v in consts for v in bn.inputs[1:5]) and n.inputs[1] in consts and (len(n.inputs) < 3 or n.inputs[2] in consts)
        if not ok:
            out.append(n)
            continue
        f32 = np.float32
        scale, bn_bias, mean, var = (np.asarray(consts[v], f32) for v in bn.inputs[1:5])
        w = np.asarray(consts[n.inputs[1]], f32)
        bc = np.asarray(consts[n.inputs[2]], f32) if len(n.inputs) == 3 else np.zeros(scale.shape[0], f32)
        eps = f32(bn.attrs.get("epsilon", 1e-5))
        s = (scale / np.sqrt(var + eps)).astype(f32)
        if w.shape[0] != s.shape[0]:
            raise ValueError("MergeConvBN: %d output channels but %d batch-norm scales" % (w.shape[0], s.shape[0]))
        new_w = (w * s.reshape((-1,) + (1,) * (w.ndim - 1))).astype(f32)
        new_b = ((bc - mean) * s + bn_bias).astype(f32)
        wn, bname = n.inputs[1] + "@bn", (n.inputs[2] if len(n.inputs) == 3 else bn.inputs[2]) + "@bn"
        consts[wn], consts[bname] = new_w, new_b
        out.append(Node("Conv", [n.inputs[0], wn, bname], list(bn.outputs), dict(n.attrs), n.name))
        dropped.add(id(bn))
    return [n for n in out if id(n) not in dropped]


def compile_model(model, quantize=False, per_channel=True, asymmetric_input_types=False, fold_bn_first=False, fuse=False, peephole=True):
    """ONNX graph -> Program.  quantize: the reference's `--quantize` (dynamic, IntegerOps; weights uint8 unless
    asymmetric_input_types, which makes them int8: compiler/quantize.cc:392-400).  fuse: group elementwise float nodes into
    ElementWiseNvrtc instructions (`--fuse_operations --use_nvrtc`).  peephole: True = fuse_quantized_add, then fuse_conv_residual;
    "join" = the first only; False = neither."""
    nodes, consts = _fold_constants(model)

    def quantizable(n):
        if n.op_type != "Conv" or n.inputs[1] not in consts:
            return False
        # compiler/quantize.cc:366-369 skips a Conv with bias; after --fold_bn_first the merged bias is handled below
        return len(n.inputs) == 2 or (fold_bn_first and n.inputs[2] in consts)

    if fold_bn_first:
        nodes = merge_conv_bn(nodes, consts, model.outputs)
    else:
        # Quantize runs before MergeConvBN (compiler/passes.cc:121-128): a Conv the quantizer rewrites is no longer a Conv when
        # the merge pass looks, so only the convolutions that stay float are merged with their BatchNormalization.
        nodes = merge_conv_bn(nodes, consts, model.outputs, only=lambda n: not (quantize and quantizable(n)))
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
        if quantize and quantizable(n):
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
            if len(n.inputs) == 3:
                scaled, bname = fresh("scaled"), fresh("bias")
                consts[bname] = np.asarray(consts[n.inputs[2]], np.float32).reshape([1, -1] + [1] * (w.ndim - 2))
                insts.append(Inst("Mul", [accf, mul], [scaled]))
                insts.append(Inst("Add", [scaled, bname], [n.outputs[0]]))
            else:
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
    program = Program(insts, consts, list(model.inputs), list(model.outputs))
    if peephole:
        program = fuse_quantized_add(program)
        if peephole != "join":
            program = fuse_stem(fuse_conv_residual(program))
    if fuse:
        program = fuse_elementwise(program)
    return program


def fuse_quantized_add(program):
    """Peephole over a statically quantized graph: DequantizeLinear(a), DequantizeLinear(b), Add, [Relu], QuantizeLinear with
    single-use intermediates and constant scalar parameters -- the join of a residual block -- becomes one QAddU8
    instruction (five full-tensor passes, three of them over fp32 data, become one uint8 pass).  The kernel evaluates the
    same fp32 chain per element, so the result is bit-identical to the five nodes."""
    insts = program.insts
    users, producer = {}, {}
    for k, i in enumerate(insts):
        for v in i.inputs:
            users.setdefault(v, []).append(k)
        for v in i.outputs:
            producer[v] = k
    consts = program.constants

    def scalar_const(name):
        return name in consts and np.asarray(consts[name]).size == 1

    def single_use(v):
        return len(users.get(v, [])) == 1 and v not in program.outputs

    replaced, drop = {}, set()
    for k, q in enumerate(insts):
        if q.op != "QuantizeLinear" or len(q.inputs) != 3 or not (scalar_const(q.inputs[1]) and scalar_const(q.inputs[2])):
            continue
        if np.asarray(consts[q.inputs[2]]).dtype != np.uint8:
            continue
        chain, v, relu = [], q.inputs[0], False
        pk = producer.get(v)
        if pk is not None and insts[pk].op == "Relu" and single_use(v):
            relu, v = True, insts[pk].inputs[0]
            chain.append(pk)
            pk = producer.get(v)
        if pk is None or insts[pk].op != "Add" or not single_use(v):
            continue
        add = insts[pk]
        chain.append(pk)
        dqs = [producer.get(t) for t in add.inputs]
        if any(d is None or insts[d].op != "DequantizeLinear" or len(insts[d].inputs) != 3 or not single_use(t) for d, t in zip(dqs, add.inputs)):
            continue
        if dqs[0] == dqs[1]:
            continue
        if not all(scalar_const(insts[d].inputs[1]) and scalar_const(insts[d].inputs[2]) and np.asarray(consts[insts[d].inputs[2]]).dtype == np.uint8
                   for d in dqs):
            continue
        a, b = insts[dqs[0]], insts[dqs[1]]
        replaced[k] = Inst("QAddU8", [a.inputs[0], a.inputs[1], a.inputs[2], b.inputs[0], b.inputs[1], b.inputs[2], q.inputs[1], q.inputs[2]],
                           q.outputs, relu=int(relu))
        drop.update(chain + dqs)
    if not replaced:
        return program
    new = [replaced.get(k, i) for k, i in enumerate(insts) if k not in drop]
    return Program(new, program.constants, program.inputs, program.outputs)


def fuse_conv_residual(program):
    """Second peephole: a QLinearConv with constant weights whose only reader is a QAddU8 takes the join into its epilogue
    (the residual map is read once, the convolution output never reaches memory).  The fused instruction sits where the
    QAddU8 was, so the other operand is always computed before it.  Inputs 0-8 are QLinearConv's, 9-13 are the residual map,
    its scale and zero point, and the join's output scale and zero point."""
    insts = program.insts
    users, producer = {}, {}
    for k, i in enumerate(insts):
        for v in i.inputs:
            users.setdefault(v, []).append(k)
        for v in i.outputs:
            producer[v] = k
    consts = program.constants
    replaced, drop = {}, set()
    for k, q in enumerate(insts):
        if q.op != "QAddU8":
            continue
        for side in (0, 3):
            v = q.inputs[side]
            pk = producer.get(v)
            if pk is None or pk in drop or insts[pk].op != "QLinearConv" or len(users.get(v, [])) != 1 or v in program.outputs:
                continue
            conv = insts[pk]
            if conv.inputs[3] not in consts or conv.attrs.get("residual"):
                continue
            if [conv.inputs[6], conv.inputs[7]] != q.inputs[side + 1:side + 3]:  # the join must dequantize with the convolution's output parameters
                continue
            other = 3 - side
            ins = list(conv.inputs) + [""] * (9 - len(conv.inputs)) + [q.inputs[other], q.inputs[other + 1], q.inputs[other + 2], q.inputs[6], q.inputs[7]]
            replaced[k] = Inst("QLinearConv", ins, q.outputs, **dict(conv.attrs, residual=1, res_relu=int(q.attrs.get("relu", 0)), conv_output=v))
            drop.add(pk)
            break
    if not replaced:
        return program
    new = [replaced.get(k, i) for k, i in enumerate(insts) if k not in drop]
    return Program(new, program.constants, program.inputs, program.outputs)


def fuse_stem(program):
    """Third peephole, for network stems: a QLinearConv with constant weights takes (a) the QuantizeLinear in front of it when
    that node quantizes a float value with the convolution's own input scale and zero point and has no other reader
    (attribute quantize_input: input 0 is then the float value), and (b) the uint8 MaxPool(kernel 3, stride 2, no padding)
    behind it when that is its only reader (attribute pool = ceil_mode of the MaxPool; the instruction's output is the pooled
    map).  Whether the fused kernels apply depends on the geometry, which is known at run time: the executor falls back to
    the separate kernels when the library refuses, with the same results."""
    insts = program.insts
    users, producer = {}, {}
    for k, i in enumerate(insts):
        for v in i.inputs:
            users.setdefault(v, []).append(k)
        for v in i.outputs:
            producer[v] = k
    consts = program.constants
    replaced, drop = {}, set()
    for k, conv in enumerate(insts):
        if conv.op != "QLinearConv" or conv.inputs[3] not in consts or conv.attrs.get("residual"):
            continue
        ins, attrs, outs = list(conv.inputs), dict(conv.attrs), list(conv.outputs)
        qk = producer.get(ins[0])
        if qk is not None and insts[qk].op == "QuantizeLinear" and len(users.get(ins[0], [])) == 1 and ins[0] not in program.outputs \
                and len(insts[qk].inputs) == 3 and insts[qk].inputs[1:3] == ins[1:3] and all(v in consts for v in ins[1:3]) \
                and np.asarray(consts[ins[2]]).dtype == np.uint8:
            attrs["quantize_input"] = 1
            attrs["quantized_name"] = ins[0]
            ins[0] = insts[qk].inputs[0]
            drop.add(qk)
        u = users.get(outs[0], [])
        if len(u) == 1 and outs[0] not in program.outputs and insts[u[0]].op == "MaxPool":
            mp = insts[u[0]]
            a = mp.attrs
            pads = list(a.get("pads", [])) or [0, 0, 0, 0]
            if list(a.get("kernel_shape", [])) == [3, 3] and list(a.get("strides", [1, 1])) == [2, 2] and not any(pads) \
                    and not any(d != 1 for d in a.get("dilations", [])) and len(mp.outputs) == 1 \
                    and np.asarray(consts.get(ins[7], np.int8(0))).dtype == np.uint8:
                attrs["pool"] = 1 + int(bool(a.get("ceil_mode", 0)))  # 1 = floor, 2 = ceil_mode
                attrs["conv_output"] = outs[0]
                outs = list(mp.outputs)
                drop.add(u[0])
        if attrs != conv.attrs:
            replaced[k] = Inst("QLinearConv", ins, outs, **attrs)
    if not replaced:
        return program
    new = [replaced.get(k, i) for k, i in enumerate(insts) if k not in drop]
    return Program(_topological(new, set(program.constants) | set(program.inputs)), program.constants, program.inputs, program.outputs)


# ---- elementwise fusion over a program -----------------------------------------------------------------------------------
_NP_NAME = {np.dtype(np.float32): "float32", np.dtype(np.float64): "float64", np.dtype(np.float16): "float16", np.dtype(np.int8): "int8",
            np.dtype(np.uint8): "uint8", np.dtype(np.int32): "int32", np.dtype(np.int64): "int64", np.dtype(np.bool_): "bool", np.dtype(np.int16): "int16"}
_ONNX_TO_NAME = {1: "float32", 2: "uint8", 3: "int8", 5: "int16", 6: "int32", 7: "int64", 9: "bool", 10: "float16", 11: "float64"}


def infer_dtypes(program):
    """Value name -> dtype name, by the ops' typing rules (inputs of unknown dtype are taken as float32)."""
    dt = {k: _NP_NAME.get(np.asarray(v).dtype) for k, v in program.constants.items()}
    for k in program.inputs:
        dt.setdefault(k, "float32")
    for inst in program.insts:
        first = dt.get(inst.inputs[0], "float32") if inst.inputs else "float32"
        if inst.op == "QuantizeLinear":
            o = [dt.get(inst.inputs[2], "uint8") if len(inst.inputs) > 2 else "uint8"]
        elif inst.op in ("ConvInteger", "MatMulInteger"):
            o = ["int32"]
        elif inst.op in ("QLinearConv", "QLinearMatMul"):
            o = [dt.get(inst.inputs[7], "uint8")]
        elif inst.op == "DequantizeLinear":
            o = ["float32"]
        elif inst.op == "Cast":
            to = inst.attrs.get("to", 1)
            o = [to if isinstance(to, str) else _ONNX_TO_NAME.get(int(to), "float32")]
        elif inst.op == "DynamicQuantParamsU8":
            o = ["float32", "uint8"]
        elif inst.op == "Shape":
            o = ["int64"]
        else:
            o = [first] * len(inst.outputs)
        for name, d in zip(inst.outputs, o):
            dt[name] = d
    return dt


def fuse_elementwise(program):
    """`--fuse_operations --use_nvrtc`: the reference's grouping (compiler/fusion_elementwise.cc:10-40 over
    compiler/fusion.cc:165-214, here chxq_fuse_elementwise) decides the groups; each becomes one ElementWiseNvrtc instruction
    whose `code` attribute is the generated kernel source (compiler/nvrtc_builder.cc:91-206, here chxq_eltwise_codegen).  The
    member nodes stay in the `members` attribute (a CPU evaluation runs them one by one, as the reference's CPU path does:
    compiler/chxvm/emitter.cc:702-726)."""
    from chainer_compiler_b200 import fusion
    dt = infer_dtypes(program)
    nodes = [fusion.Node(i.op, list(i.inputs), list(i.outputs)) for i in program.insts]
    groups = fusion.fuse_elementwise(nodes, dt, program.outputs)
    if not groups:
        return program
    member_of = {}
    for g in groups:
        for idx in g.node_indices:
            member_of[idx] = g
    insts, emitted = [], set()
    for idx, inst in enumerate(program.insts):
        g = member_of.get(idx)
        if g is None:
            insts.append(inst)
        elif g.fusion_id not in emitted and idx == max(g.node_indices):
            emitted.add(g.fusion_id)
            members = [nodes[k] for k in g.node_indices]
            code = fusion.build_program(members, g.fusion_id, g.inputs, g.outputs, dt.get(g.outputs[0]) or "float32")
            insts.append(Inst("ElementWiseNvrtc", g.inputs, g.outputs, num_outputs=len(g.outputs), code=code, fusion_id=g.fusion_id,
                              members=[(m.op_type, list(m.inputs), list(m.outputs)) for m in members]))
    return Program(_topological(insts, set(program.constants) | set(program.inputs)), program.constants, program.inputs, program.outputs)


def _topological(insts, available):
    """Stable topological order: a fused group sits where its last member was, which can be after a reader of one of its
    earlier outputs."""
    done, out, rest = set(available), [], list(insts)
    while rest:
        progressed = False
        for k, inst in enumerate(rest):
            if all(i in done or i == "" for i in inst.inputs):
                out.append(inst)
                done.update(inst.outputs)
                del rest[k]
                progressed = True
                break
        if not progressed:
            raise ValueError("program has a cycle or reads an undefined value: %r" % rest[0])
    return out


# ---- ONNX export of a program ----------------------------------------------------------------------------------------------
def program_to_onnx(program, name="graph"):
    """The program as an ONNX graph of standard nodes (`--out_onnx`): the dynamic-quantization helper instructions are written
    out as the node sequences compiler/quantize.cc:172-207,232-244 emits (ReduceMin, ReduceMax, Sub, Div, Floor, Cast, Mul,
    Reshape); fused groups are written as their member nodes."""
    from chainer_compiler_b200 import onnx_io
    consts = dict(program.constants)
    nodes = []
    N = onnx_io.Node
    code_of = {"float32": onnx_io.FLOAT, "uint8": onnx_io.UINT8, "int8": onnx_io.INT8, "int32": onnx_io.INT32, "int64": onnx_io.INT64,
               "float16": onnx_io.FLOAT16, "float64": onnx_io.DOUBLE, "bool": onnx_io.BOOL, "int16": onnx_io.INT16}
    for pc, i in enumerate(program.insts):
        t = lambda s: "%s@x%d" % (s, pc)  # noqa: E731
        if i.op == "ReduceMinMax":
            nodes.append(N("ReduceMin", i.inputs, [i.outputs[0]], {"keepdims": 0}))
            nodes.append(N("ReduceMax", i.inputs, [i.outputs[1]], {"keepdims": 0}))
        elif i.op == "DynamicQuantParamsU8":
            consts[t("qrange")], consts[t("zero")] = np.float32(255.0).reshape(()), np.float32(0.0).reshape(())
            nodes.append(N("Sub", [i.inputs[1], i.inputs[0]], [t("span")], {}))
            nodes.append(N("Div", [t("span"), t("qrange")], [i.outputs[0]], {}))
            nodes.append(N("Sub", [t("zero"), i.inputs[0]], [t("zsub")], {}))
            nodes.append(N("Div", [t("zsub"), i.outputs[0]], [t("zdiv")], {}))
            nodes.append(N("Floor", [t("zdiv")], [t("zfloor")], {}))
            nodes.append(N("Cast", [t("zfloor")], [i.outputs[1]], {"to": onnx_io.UINT8}))
        elif i.op == "ScaleProduct":
            if i.attrs.get("shape"):
                consts[t("shape")] = np.asarray(i.attrs["shape"], np.int64)
                nodes.append(N("Mul", i.inputs, [t("prod")], {}))
                nodes.append(N("Reshape", [t("prod"), t("shape")], i.outputs, {}))
            else:
                nodes.append(N("Mul", i.inputs, i.outputs, {}))
        elif i.op == "ElementWiseNvrtc":
            for op, ins, outs in i.attrs["members"]:
                nodes.append(N(op, ins, outs, {}))
        elif i.op == "QLinearConv" and (i.attrs.get("quantize_input") or i.attrs.get("pool")):
            skip = ("quantize_input", "quantized_name", "pool", "conv_output")
            attrs = {k: v for k, v in i.attrs.items() if k not in skip and v is not None and not (isinstance(v, (list, tuple)) and len(v) == 0)}
            cin = list(i.inputs)
            if i.attrs.get("quantize_input"):
                nodes.append(N("QuantizeLinear", [cin[0], cin[1], cin[2]], [i.attrs["quantized_name"]], {}))
                cin[0] = i.attrs["quantized_name"]
            while cin and cin[-1] == "":
                cin.pop()
            if i.attrs.get("pool"):
                nodes.append(N("QLinearConv", cin, [i.attrs["conv_output"]], attrs))
                pattrs = {"kernel_shape": [3, 3], "strides": [2, 2]}
                if i.attrs["pool"] == 2:
                    pattrs["ceil_mode"] = 1
                nodes.append(N("MaxPool", [i.attrs["conv_output"]], i.outputs, pattrs))
            else:
                nodes.append(N("QLinearConv", cin, i.outputs, attrs))
        elif i.op == "QLinearConv" and i.attrs.get("residual"):
            attrs = {k: v for k, v in i.attrs.items() if k not in ("residual", "res_relu", "conv_output") and v is not None
                     and not (isinstance(v, (list, tuple)) and len(v) == 0)}
            cin = [v for v in i.inputs[:9]]
            while cin and cin[-1] == "":
                cin.pop()
            h = i.attrs["conv_output"]
            nodes.append(N("QLinearConv", cin, [h], attrs))
            nodes.append(N("DequantizeLinear", [h, i.inputs[6], i.inputs[7]], [t("fa")], {}))
            nodes.append(N("DequantizeLinear", i.inputs[9:12], [t("fb")], {}))
            nodes.append(N("Add", [t("fa"), t("fb")], [t("sum")], {}))
            if i.attrs.get("res_relu"):
                nodes.append(N("Relu", [t("sum")], [t("relu")], {}))
            nodes.append(N("QuantizeLinear", [t("relu") if i.attrs.get("res_relu") else t("sum"), i.inputs[12], i.inputs[13]], i.outputs, {}))
        elif i.op == "QAddU8":
            nodes.append(N("DequantizeLinear", i.inputs[0:3], [t("fa")], {}))
            nodes.append(N("DequantizeLinear", i.inputs[3:6], [t("fb")], {}))
            nodes.append(N("Add", [t("fa"), t("fb")], [t("sum")], {}))
            if i.attrs.get("relu"):
                nodes.append(N("Relu", [t("sum")], [t("relu")], {}))
            nodes.append(N("QuantizeLinear", [t("relu") if i.attrs.get("relu") else t("sum"), i.inputs[6], i.inputs[7]], i.outputs, {}))
        elif i.op == "Cast":
            to = i.attrs.get("to", 1)
            nodes.append(N("Cast", i.inputs, i.outputs, {"to": code_of[to] if isinstance(to, str) else int(to)}))
        else:
            attrs = {k: v for k, v in i.attrs.items() if v is not None and not (isinstance(v, (list, tuple)) and len(v) == 0)}
            if attrs.get("auto_pad") == "NOTSET":
                del attrs["auto_pad"]
            nodes.append(N(i.op, i.inputs, i.outputs, attrs))
    used = {v for n in nodes for v in n.inputs}
    inits = {k: np.asarray(v) for k, v in consts.items() if k in used}
    return onnx_io.Model(nodes, inits, list(program.inputs), list(program.outputs), name=name)


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


def _contiguous(v):
    v = np.asarray(v)
    return np.ascontiguousarray(v).reshape(v.shape)  # ascontiguousarray alone turns a 0-d array into a 1-d one


class ChromeTracing:
    """One complete ("ph":"X") event per executed instruction with category, name, start and duration in microseconds and the
    program counter, in the layout runtime/chrome_tracing.cc:39-67 writes.  The executor synchronizes the device after each
    traced instruction, so a duration covers the kernels the instruction launched."""

    def __init__(self):
        self.base = time.perf_counter()
        self.events = []

    def add(self, category, name, pc, start, end):
        self.events.append({"cat": category, "name": name, "ts": int((start - self.base) * 1e6), "dur": int((end - start) * 1e6), "tid": 1, "pid": 1,
                            "args": {"pc": pc}, "ph": "X"})

    def emit(self, path):
        with open(path, "w") as f:
            f.write("[\n" + ",\n".join(json.dumps(e, separators=(",", ":")) for e in self.events) + "]\n")


class Executor:
    """Runs a Program on one CUDA device.  Quantized ops go through chainer_compiler_b200.ops; glue ops are torch expressions."""

    def __init__(self, program, device="cuda:0", float_ops_via_torch=False, fold_scales=False, device_scalars=True):
        """fold_scales: requantize every QLinearConv with one fp32 multiplier per output channel (x_scale * w_scale / y_scale
        folded on the host) instead of the reference's multiply and divide; outputs can differ from the default by one step
        on exact ties of the intermediate rounding.
        device_scalars: the scale and zero point of a dynamically quantized activation (the ReduceMin / ReduceMax -> Sub, Div,
        Floor, Cast sub-graph of `--quantize`) stay on the device and are read by the kernels that consume them; False reads
        them back to the host per operator, as the reference's VM does (runtime/chxvm_var.cc:70-76).  Same results."""
        import torch
        sys.path.insert(0, ROOT)
        import __graft_entry__ as entry
        entry.load_package()
        from chainer_compiler_b200 import _lib, ops
        self.torch, self.ops, self.NCHW = torch, ops, _lib.NCHW
        self.program, self.float_ok = program, float_ops_via_torch
        if not str(device).startswith("cuda"):
            raise SystemExit("run_onnx: device %r is not supported, this package runs on CUDA devices only" % (device,))
        self.device = torch.device(device if ":" in str(device) else "cuda:0")
        self.consts = {}
        for k, v in program.constants.items():
            self.consts[k] = torch.from_numpy(_contiguous(v)).to(self.device)
        self.host_consts = program.constants
        self.packed = {}
        self.fold_scales = bool(fold_scales)
        self.device_scalars = bool(device_scalars)
        self._graph = None

    def _scalar(self, name, env, host):
        """A Scalar operand on the host, keeping its dtype (the zero point's dtype selects the output dtype)."""
        if name in host:
            return host[name]
        if name in self.host_consts:
            v = np.asarray(self.host_consts[name])
        else:
            v = env[name].cpu().numpy()  # the device-to-host read of runtime/chxvm_var.cc:70-76
        if v.size != 1:
            raise ValueError("run_onnx: %s must have one element, has shape %s" % (name, v.shape))
        return v.reshape(())[()]

    _SCALAR_OPERANDS = {"QuantizeLinear": (1, 2), "DequantizeLinear": (1, 2), "QLinearConv": (1, 2, 6, 7, 10, 11, 12, 13), "QLinearMatMul": (1, 2, 4, 5, 6, 7),
                        "ConvInteger": (2,), "QAddU8": (1, 2, 4, 5, 6, 7), "Clip": (1, 2), "Reshape": (1,)}

    def stage(self, v):
        """An input array on the device (the reference stages the inputs before it starts the clock, tools/run_onnx.cc:421-427)."""
        t = self.torch
        return v.to(self.device) if isinstance(v, t.Tensor) else t.from_numpy(_contiguous(v)).to(self.device)

    def is_static(self):
        """True when running the program needs no device-to-host read: every scalar operand is an initializer and there is no
        dynamic-quantization instruction.  Such a program can be captured in a CUDA graph."""
        dev_scalars = set()  # values the device-scalar path keeps on the device
        for inst in self.program.insts:
            if inst.op in ("ReduceMinMax", "DynamicQuantParamsU8"):
                if not self.device_scalars:
                    return False
                dev_scalars.update(inst.outputs)
                continue
            if inst.op in ("ReduceMin", "ReduceMax"):
                return False
            for k in self._SCALAR_OPERANDS.get(inst.op, ()):
                if k < len(inst.inputs) and inst.inputs[k] != "" and inst.inputs[k] not in self.host_consts:
                    if inst.inputs[k] in dev_scalars and inst.op in ("QuantizeLinear", "ConvInteger"):
                        continue  # these two read a device scalar themselves
                    return False
        return True

    def capture(self, inputs):
        """Captures one run over device copies of `inputs` in a CUDA graph (static programs only).  Afterwards replay(inputs)
        copies new input values into the captured buffers, replays, and returns the (captured) output tensors.  The library's
        scratch buffer must not grow after the capture: run every other workload of the process first."""
        t = self.torch
        if not self.is_static():
            raise ValueError("run_onnx: the program reads scalars back from the device and cannot be captured")
        self._static_in = {k: self.stage(v).clone() for k, v in inputs.items()}
        host = {}
        for _ in range(2):  # warm-up: packs the weights, sizes the scratch buffer, compiles generated kernels
            env = dict(self.consts, **self._static_in)
            for inst in self.program.insts:
                self._step(inst, env, host)
        t.cuda.synchronize(self.device)
        self._graph = t.cuda.CUDAGraph()
        with t.cuda.graph(self._graph):
            env = dict(self.consts, **self._static_in)
            for inst in self.program.insts:
                self._step(inst, env, host)
            self._static_out = [(o, env[o]) for o in self.program.outputs]
        return self

    def replay(self, inputs):
        t = self.torch
        for k, v in inputs.items():
            self._static_in[k].copy_(v if isinstance(v, t.Tensor) else t.from_numpy(_contiguous(v)), non_blocking=True)
        self._graph.replay()
        self.ops.device_status()
        return self._static_out

    def run(self, inputs, trace=None, tracer=None, log=None):
        """trace: a dict that receives every instruction output; tracer: a ChromeTracing; log: a file the instructions are
        printed to as they run (`--trace`)."""
        t, ops = self.torch, self.ops
        env = dict(self.consts)
        host = {}  # host-side scalars (dynamic quantization parameters)
        for k, v in inputs.items():
            env[k] = self.stage(v)
        for pc, inst in enumerate(self.program.insts):
            if log is not None:
                log.write("%5d: %r\n" % (pc, inst))
            if tracer is not None:
                t.cuda.synchronize(self.device)
                t0 = time.perf_counter()
            self._step(inst, env, host)
            if tracer is not None:
                t.cuda.synchronize(self.device)
                tracer.add("ChxVM", inst.op, pc, t0, time.perf_counter())
            if trace is not None:
                for o in inst.outputs:
                    trace[o] = env[o] if o in env else host[o]
        ops.device_status()
        return [(o, env[o]) for o in self.program.outputs]

    def _step(self, inst, env, host):
        t, ops = self.torch, self.ops
        a, op = inst.attrs, inst.op
        x = [env.get(i) if i in env else host.get(i) for i in inst.inputs]
        sc = lambda k: self._scalar(inst.inputs[k], env, host)  # noqa: E731
        has = lambda k: len(inst.inputs) > k and inst.inputs[k] != ""  # noqa: E731
        out = inst.outputs[0]
        auto_pad = a.get("auto_pad", "NOTSET")
        auto_pad = "" if auto_pad == "NOTSET" else auto_pad
        dev_scalar = lambda k: has(k) and inst.inputs[k] in env and inst.inputs[k] not in self.host_consts and self.device_scalars \
            and env[inst.inputs[k]].numel() == 1  # noqa: E731
        if op == "ReduceMinMax":
            mm = ops.MinMax(x[0].contiguous())
            if self.device_scalars:
                env[inst.outputs[0]], env[inst.outputs[1]] = mm[0:1], mm[1:2]  # stay on the device
            else:
                mm = mm.cpu().numpy()  # the device-to-host read the reference does per scalar argument
                host[inst.outputs[0]], host[inst.outputs[1]] = np.float32(mm[0]), np.float32(mm[1])
        elif op == "DynamicQuantParamsU8":
            if inst.inputs[0] in env:
                env[inst.outputs[0]], env[inst.outputs[1]] = ops.DynamicQuantParamsU8(x[0], x[1])
            else:
                host[inst.outputs[0]], host[inst.outputs[1]] = dynamic_params_u8(host[inst.inputs[0]], host[inst.inputs[1]])
        elif op == "QuantizeLinear" and dev_scalar(1):
            env[out] = ops.QuantizeLinear(x[0].contiguous(), x[1], x[2] if has(2) else None)
        elif op == "QuantizeLinear":
            env[out] = ops.QuantizeLinear(x[0].contiguous(), sc(1), sc(2) if has(2) else None)
        elif op == "DequantizeLinear":
            env[out] = ops.DequantizeLinear(x[0].contiguous(), sc(1), sc(2) if has(2) else None)
        elif op in ("ConvInteger", "QLinearConv"):
            if any(d != 1 for d in a.get("dilations", [])):
                raise NotImplementedError("%s: dilation must be 1 (compiler/chxvm/simple_node_emitter.cc:655)" % op)
            strides, pads, group = tuple(a.get("strides", [])), self._sym_pads(a.get("pads", [])), a.get("group", 1)
            wk, zk = (1, 3) if op == "ConvInteger" else (3, 5)
            xin, packed = x[0], None
            fq, fpool = bool(a.get("quantize_input")), int(a.get("pool", 0))
            if fq or fpool:
                y = self._stem(inst, x, sc, has, strides, pads, group, auto_pad, fq, fpool)
                if y is not None:
                    env[out] = y
                    return
                if fq:  # the library refused the fused form: the separate kernels, same results
                    xin = ops.QuantizeLinear(xin.contiguous(), sc(1), sc(2))
            if xin.dim() == 4 and xin.dtype == t.uint8 and inst.inputs[wk] in self.host_consts and (not has(zk) or inst.inputs[zk] in self.host_consts):
                # constant weights: pack them once per input shape and keep the activations channels_last, which is the layout
                # the tensor-core kernels read (the first convolution of a graph pays one layout pass)
                # (a network stem with at most four input channels is read as NCHW by the packed entry itself)
                wz = x[zk] if has(zk) else None
                key = (id(inst), tuple(xin.shape))
                packed = self.packed.get(key)
                if packed is None:
                    if xin.shape[1] <= 4 and xin.is_contiguous():
                        packed = ops.PackedConv(x[wk], wz, tuple(xin.shape), strides, pads, group, auto_pad, x_layout=self.NCHW)
                    if packed is None or not packed.eligible:
                        packed = ops.PackedConv(x[wk], wz, tuple(xin.shape), strides, pads, group, auto_pad)
                    self.packed[key] = packed
                if packed.g.x_layout != self.NCHW:
                    xin = ops.to_channels_last(xin)
                if not packed.eligible:
                    packed = None
            if op == "ConvInteger" and dev_scalar(2):
                # the zero point was computed on the device: the general kernel reads it there (no host round trip)
                env[out] = ops.ConvInteger(x[0], x[1], x[2], x[3] if has(3) else None, strides, pads, group, auto_pad)
            elif op == "ConvInteger":
                if packed is not None:
                    env[out] = ops.ConvIntegerPacked(xin, packed, sc(2) if has(2) else None)
                else:
                    env[out] = ops.ConvInteger(xin, x[1], sc(2) if has(2) else None, x[3] if has(3) else None, strides, pads, group, auto_pad)
            else:
                res = {}
                if a.get("residual"):
                    r = ops.to_channels_last(x[9]) if x[9].dim() == 4 else x[9]
                    if int(sc(13)) != 0:
                        raise NotImplementedError("QLinearConv with a fused join: the join's output zero point must be 0")
                    res = dict(residual=r, res_scale=sc(10), res_zero_point=int(sc(11)), res_relu=bool(a.get("res_relu", 0)), out_scale=sc(12),
                               out_zero_point=0)
                    if xin.dim() == 4 and packed is None:
                        xin = ops.to_channels_last(xin)  # the residual map and the output share the NHWC layout
                if packed is not None:
                    y = ops.QLinearConvPacked(xin, packed, sc(1), sc(2), x[4], x[5], sc(6), sc(7), b=x[8] if has(8) else None,
                                              fold_scales=self.fold_scales, **res)
                else:
                    y = ops.QLinearConv(xin, sc(1), sc(2), x[3], x[4], x[5], sc(6), sc(7), x[8] if has(8) else None, strides, pads, group,
                                        auto_pad, fold_scales=self.fold_scales, **res)
                if fpool:
                    y = ops.MaxPoolU8(ops.to_channels_last(y), 3, 2, 0, cover_all=(fpool == 2))
                env[out] = y
        elif op == "QAddU8":
            qa, qb = x[0], x[3]
            if qa.stride() != qb.stride():  # one operand came from a kernel of the other layout
                qa, qb = (ops.to_channels_last(qa), ops.to_channels_last(qb)) if qa.dim() == 4 else (qa.contiguous(), qb.contiguous())
            env[out] = ops.QAddU8(qa, sc(1), sc(2), qb, sc(4), sc(5), sc(6), sc(7), relu=bool(a.get("relu", 0)))
        elif op == "MatMulInteger":
            def zp_arr(k, like):
                if not has(k):
                    return None
                if inst.inputs[k] in env:
                    return env[inst.inputs[k]]
                return t.tensor([int(host[inst.inputs[k]])], dtype=like.dtype, device=self.device)
            env[out] = ops.MatMulInteger(x[0].contiguous(), x[1].contiguous(), zp_arr(2, x[0]), zp_arr(3, x[1]))
        elif op == "QLinearMatMul":
            env[out] = ops.QLinearMatMul(x[0].contiguous(), sc(1), sc(2), x[3].contiguous(), sc(4), sc(5), sc(6), sc(7))
        elif op == "ElementWiseNvrtc":
            outs = ops.ElementWiseNvrtc(x, a["num_outputs"], a["code"], a["fusion_id"])
            for name, y in zip(inst.outputs, outs):
                env[name] = y
        elif op == "ScaleProduct":
            s0 = x[0] if inst.inputs[0] in env else t.tensor(float(host[inst.inputs[0]]), dtype=t.float32, device=self.device)
            s1 = x[1] if inst.inputs[1] in env else t.tensor(float(host[inst.inputs[1]]), dtype=t.float32, device=self.device)
            m = s0 * s1
            env[out] = m.reshape(a["shape"]) if a.get("shape") else m
        elif op == "Cast":
            to = a.get("to", 1)
            env[out] = x[0].to(getattr(t, to if isinstance(to, str) else _ONNX_TO_NAME[int(to)]))
        elif op in ("Add", "Sub", "Mul", "Div", "Max", "Min"):
            f = {"Add": t.add, "Sub": t.sub, "Mul": t.mul, "Div": t.div, "Max": t.maximum, "Min": t.minimum}[op]
            env[out] = f(x[0], x[1])
        elif op in ("Relu", "Tanh", "Sigmoid", "Exp", "Floor", "Abs", "Identity"):
            f = {"Relu": t.relu, "Tanh": t.tanh, "Sigmoid": t.sigmoid, "Exp": t.exp, "Floor": t.floor, "Abs": t.abs, "Identity": lambda v: v}[op]
            env[out] = f(x[0])
        elif op in ("ReduceMin", "ReduceMax"):
            if a.get("axes"):
                raise NotImplementedError("%s over chosen axes" % op)
            mm = ops.MinMax(x[0].contiguous())
            y = mm[0] if op == "ReduceMin" else mm[1]
            env[out] = y.reshape(()) if not a.get("keepdims", 1) else y.reshape([1] * x[0].dim())
        elif op == "Clip":
            lo = a.get("min", float(sc(1)) if has(1) else None)
            hi = a.get("max", float(sc(2)) if has(2) else None)
            env[out] = t.clamp(x[0], lo, hi)
        elif op == "BatchNormalization":
            shape = [1, -1] + [1] * (x[0].dim() - 2)
            eps = np.float32(a.get("epsilon", 1e-5))
            env[out] = (x[0] - x[3].reshape(shape)) / t.sqrt(x[4].reshape(shape) + float(eps)) * x[1].reshape(shape) + x[2].reshape(shape)
        elif op == "Reshape":
            shape = [int(d) for d in self.host_consts[inst.inputs[1]]] if inst.inputs[1] in self.host_consts else [int(d) for d in x[1].cpu()]
            shape = [x[0].shape[i] if d == 0 else d for i, d in enumerate(shape)]
            env[out] = x[0].reshape(shape)
        elif op == "MaxPool":
            k, s = a["kernel_shape"], a.get("strides", [1] * len(a["kernel_shape"]))
            p = _pool_pads(a, len(k))
            if any(p[i] != p[i + len(k)] for i in range(len(k))):
                raise NotImplementedError("MaxPool: asymmetric pads")
            ceil = bool(a.get("ceil_mode", 0))
            if x[0].dtype == t.uint8:
                if len(k) != 2 or k[0] != k[1] or s[0] != s[1] or len(set(p)) != 1:
                    raise NotImplementedError("uint8 MaxPool with a non-square window")
                env[out] = ops.MaxPoolU8(ops.to_channels_last(x[0]), k[0], s[0], p[0], cover_all=ceil)
            else:
                env[out] = t.nn.functional.max_pool2d(x[0], k, s, p[:len(k)], ceil_mode=ceil)
        elif op == "GlobalAveragePool":
            env[out] = x[0].mean(dim=tuple(range(2, x[0].dim())), keepdim=True)
        elif op == "Flatten":
            ax = a.get("axis", 1)
            env[out] = x[0].reshape(int(np.prod(x[0].shape[:ax])), -1)
        elif op == "Gemm" and a.get("transB", 0) and not a.get("transA", 0) and a.get("alpha", 1.0) == 1.0 and a.get("beta", 1.0) == 1.0 \
                and x[0].dtype == t.float32 and x[0].dim() == 2:
            env[out] = ops.Linear(x[0].contiguous(), x[1].contiguous(), x[2] if has(2) else None)  # the classifier of a quantized CNN
        elif op in ("Conv", "MatMul", "Gemm"):
            if not self.float_ok:
                raise SystemExit("run_onnx: float %s has no kernel in this package; run with --quantize (or --float_ops_via_torch to "
                                 "evaluate it as a torch expression outside the product path)" % op)
            if op == "Conv":
                pads = self._sym_pads(a.get("pads", []))
                xin = x[0]
                if auto_pad == "SAME_UPPER":
                    from chainer_compiler_b200.ops import conv_geometry_from_shapes  # the library's geometry rule
                    g = conv_geometry_from_shapes(tuple(xin.shape), 6, tuple(x[1].shape), 2, tuple(a.get("strides", [])), (), a.get("group", 1), "SAME_UPPER")
                    xin = t.nn.functional.pad(xin, (g.pad_left, g.pad_right, g.pad_top, g.pad_bottom))
                    pads = (0, 0)
                env[out] = t.nn.functional.conv2d(xin, x[1], x[2] if len(x) > 2 else None, tuple(a.get("strides", [1, 1])), pads or 0, 1, a.get("group", 1))
            elif op == "MatMul":
                env[out] = x[0] @ x[1]
            else:
                A = x[0].t() if a.get("transA", 0) else x[0]
                B = x[1].t() if a.get("transB", 0) else x[1]
                y = a.get("alpha", 1.0) * (A @ B)
                env[out] = y + a.get("beta", 1.0) * x[2] if len(x) > 2 else y
        else:
            raise NotImplementedError("run_onnx: op %s" % op)

    def _stem(self, inst, x, sc, has, strides, pads, group, auto_pad, fq, fpool):
        """The fused forms of a stem convolution (QuantizeLinear in front and / or MaxPool behind); None when the library has no
        fused kernel for the geometry."""
        t, ops = self.torch, self.ops
        from chainer_compiler_b200 import _lib
        xin = x[0]
        if xin.dim() != 4 or not (xin.dtype == t.float32 if fq else xin.dtype == t.uint8):
            return None
        wz = x[5] if has(5) else None
        key = (id(inst), tuple(xin.shape), "stem")
        entry = self.packed.get(key)
        if entry is None:
            entry = False
            layouts = (self.NCHW,) if (xin.shape[1] <= 4 and xin.is_contiguous()) else ()
            for layout in layouts + (None,):
                pk = ops.PackedConv(x[3], wz, tuple(xin.shape), strides, pads, group, auto_pad) if layout is None else \
                    ops.PackedConv(x[3], wz, tuple(xin.shape), strides, pads, group, auto_pad, x_layout=layout)
                if pk.eligible:
                    entry = pk
                    break
            self.packed[key] = entry
        if entry is False:
            return None
        if entry.g.x_layout != self.NCHW:
            xin = ops.to_channels_last(xin)
        args = (xin, entry, sc(1), sc(2), x[4], x[5], sc(6), sc(7))
        kw = dict(b=x[8] if has(8) else None, fold_scales=self.fold_scales)
        try:
            if fpool:
                return ops.QLinearConvMaxPoolPacked(*args, cover_all=(fpool == 2), **kw)
            return ops.QuantizeLinearConvPacked(*args, **kw)
        except _lib.ChxqError as e:
            if e.code != _lib.ERR_UNSUPPORTED:
                raise
        if fq and fpool:  # the pooling may be what was refused: the fused quantization alone
            try:
                y = ops.QuantizeLinearConvPacked(*args, **kw)
                return ops.MaxPoolU8(y, 3, 2, 0, cover_all=(fpool == 2))
            except _lib.ChxqError as e:
                if e.code != _lib.ERR_UNSUPPORTED:
                    raise
        self.packed[key] = False  # do not try again
        return None

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
    ap.add_argument("--chrome_tracing")
    ap.add_argument("--report_json")
    ap.add_argument("--compile_only", action="store_true")
    ap.add_argument("--skip_inference", action="store_true")
    ap.add_argument("--dump_chxvm", action="store_true")
    ap.add_argument("--dump_onnx", action="store_true")
    ap.add_argument("--out_onnx")
    ap.add_argument("--quantize", action="store_true")
    ap.add_argument("--disable_per_channel_quantize", action="store_true")
    ap.add_argument("--fold_bn_first", action="store_true")
    ap.add_argument("--fold_scales", action="store_true")
    ap.add_argument("--cuda_graph", action="store_true")
    ap.add_argument("--host_scalars", action="store_true",
                    help="read dynamic-quantization scales and zero points back to the host per operator, as the reference's VM does; "
                         "default: they stay on the device (same results, no synchronization, the program can be captured in a CUDA graph)")
    ap.add_argument("--no_peephole", action="store_true")
    ap.add_argument("--fuse_operations", action="store_true")
    ap.add_argument("--use_nvrtc", action="store_true")
    ap.add_argument("--use_cuda", action="store_true")
    ap.add_argument("--skip_runtime_type_check", action="store_true")
    ap.add_argument("--backend", default="chxvm")
    ap.add_argument("--float_ops_via_torch", action="store_true")
    ap.add_argument("-t", "--trace", action="store_true")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-q", "--quiet", action="store_true")
    return ap.parse_args(argv)


def _file_name(value_name):
    return value_name.replace("/", "_").replace(os.sep, "_")


def run_onnx(argv):
    """Returns 0 when every checked output is within tolerance, 1 otherwise (the reference CHECK-fails instead)."""
    sys.path.insert(0, ROOT)
    import __graft_entry__ as entry
    entry.load_package()
    from chainer_compiler_b200 import onnx_io
    args = parse_args(argv)
    if args.backend != "chxvm":
        raise SystemExit("run_onnx: unknown backend %r (this package has the chxvm backend only)" % args.backend)
    target = args.test or args.onnx or args.positional
    if not target:
        raise SystemExit("run_onnx: give a test directory or an .onnx file")
    if os.path.isdir(target):
        model, cases = onnx_io.load_test_dir(target)
    else:
        model, cases = onnx_io.load_model(target), []
    unfused = compile_model(model, quantize=args.quantize, per_channel=not args.disable_per_channel_quantize, fold_bn_first=args.fold_bn_first,
                            peephole=not args.no_peephole)
    # the reference fuses for NVRTC only when both flags are given (compiler/passes.cc: fusion needs a code generator)
    program = fuse_elementwise(unfused) if (args.fuse_operations and args.use_nvrtc) else unfused
    if args.dump_onnx or args.out_onnx:
        exported = program_to_onnx(unfused, model.name)
        if args.dump_onnx:
            sys.stderr.write("=== vvv after simplification vvv ===\n%s\n=== ^^^ after simplification ^^^ ===\n" % "\n".join(repr(n) for n in exported.nodes))
        if args.out_onnx:
            with open(args.out_onnx, "wb") as f:
                f.write(onnx_io.serialize_model(exported))
    if args.dump_chxvm:
        print(program.dump())
    if args.compile_only or args.skip_inference:
        return 0
    import torch
    ex = Executor(program, args.device, args.float_ops_via_torch, fold_scales=args.fold_scales, device_scalars=not args.host_scalars)
    tracer = ChromeTracing() if args.chrome_tracing else None
    # --cuda_graph: after the first (discarded) iteration of a case the remaining ones replay a captured graph
    use_graph = args.cuda_graph and args.iterations > 1 and ex.is_static() and not (args.chrome_tracing or args.dump_outputs_dir or args.trace)
    failures, elapsed, report = 0, [], []
    for ci, (ins, expected) in enumerate(cases):
        outs, values = None, ({} if args.dump_outputs_dir else None)
        ins = {k: ex.stage(v) for k, v in ins.items()}
        for it in range(max(1, args.iterations)):
            torch.cuda.synchronize(ex.device)
            t0 = time.perf_counter()
            if use_graph and it == 1:
                ex.capture(ins)
                torch.cuda.synchronize(ex.device)
                t0 = time.perf_counter()
            if use_graph and it >= 1:
                outs = ex.replay(ins)
            else:
                outs = ex.run(ins, trace=values, tracer=tracer, log=sys.stderr if args.trace else None)
            torch.cuda.synchronize(ex.device)
            if it > 0 or args.iterations == 1:  # the first iteration is discarded when there are several (tools/run_onnx.cc:468-469)
                elapsed.append(time.perf_counter() - t0)
        got = {k: v.detach().cpu().numpy() for k, v in outs}
        if args.dump_outputs_dir:
            os.makedirs(args.dump_outputs_dir, exist_ok=True)
            for pc, inst in enumerate(program.insts):
                for o in inst.outputs:
                    v = values.get(o)
                    if v is not None and o:
                        np.save(os.path.join(args.dump_outputs_dir, "%05d_%s.npy" % (pc, _file_name(o))), v.detach().cpu().numpy() if hasattr(v, "detach") else np.asarray(v))
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
                print("case %d output %s: max abs diff %.6g, max rel diff %.6g" % (ci, name, d.max(), (d / np.maximum(np.abs(want.astype(np.float64)), 1e-30)).max()))
            if not ok:
                failures += 1
            report.append({"case": ci, "output": name, "ok": bool(ok)})
        if args.verbose and not args.quiet:
            print("case %d: %s" % (ci, {k: v.shape for k, v in got.items()}))
    if tracer is not None:
        tracer.emit(args.chrome_tracing)
    if not cases and not args.quiet:
        print("run_onnx: model compiled (%d instructions); no test data to run" % len(program.insts))
    avg_ms = 1000.0 * float(np.mean(elapsed)) if elapsed else 0.0
    if not args.quiet:
        print("Elapsed: %.3f msec" % avg_ms)
        if len(elapsed) > 1:
            sys.stderr.write("Average elapsed: %.3f msec\nBest elapsed: %.3f msec\n" % (avg_ms, 1000.0 * min(elapsed)))
        print("OK!" if failures == 0 else "FAILED: %d output(s) out of tolerance" % failures)
    if args.report_json:
        with open(args.report_json, "w") as f:
            json.dump({"elapsed_ms": avg_ms, "best_ms": 1000.0 * min(elapsed) if elapsed else 0.0, "cuda_graph": bool(use_graph), "failures": failures, "outputs": report, "quantize": bool(args.quantize)}, f)
    return 0 if failures == 0 else 1


if __name__ == "__main__":
    sys.exit(run_onnx(sys.argv[1:]))
