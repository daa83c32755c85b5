"""Runs a parsed `.espdl` graph node by node on the CPU with the plain-C oracle (test infrastructure).

Batch N is executed the way a caller of the reference has to: every conv / pool / resize node is applied to
each image independently (the oracle's batch loop), Gemm folds the leading dims into rows."""
import ctypes as C

import numpy as np

import cases
import checkers
from espdl_b200 import abi, espdl_file

ACT = {"Linear": abi.ACT_LINEAR, "Relu": abi.ACT_RELU}
QDT = {"S8": abi.DTYPE_INT8, "S16": abi.DTYPE_INT16}


def _exponents(m):
    e = {v["name"]: (v["exponents"][0] if v["exponents"] else 0) for v in list(m["value_info"].values()) + m["inputs"] + m["outputs"]}
    return e


def _dtypes(m):
    return {v["name"]: v["elem_type"] for v in list(m["value_info"].values()) + m["inputs"] + m["outputs"]}


class _RefBackend:
    """The reference's own operators (oracle/_ref) behind the oracle's call names."""

    def __init__(self):
        self.r = checkers.ref()

    def oracle_conv2d(self, d):
        c = d._obj if hasattr(d, "_obj") else d
        gemm = int(c.n == 1 and c.in_h == 1 and c.kh == 1 and c.kw == 1 and c.group == 1)
        return self.r.ref_conv2d(d, gemm)

    def oracle_eltwise(self, d):
        return self.r.ref_eltwise(d)

    def oracle_pool(self, d):
        return self.r.ref_pool(d)

    def oracle_resize(self, d):
        return self.r.ref_resize(d)


def matmul(o, a, b, e_a, e_b, e_out, dtype, act, round_mode):
    """MatMul as the reference's generic C path computes it (dl_module_matmul.hpp:125-526 over dl_base_conv2d.cpp:23-32):
    one Gemm per broadcast batch slice with input1's memory read as the filter, i.e. as [N][K]."""
    K = a.shape[-1]
    M = 1 if a.ndim == 1 else a.shape[-2]
    N = 1 if b.ndim == 1 else b.shape[-1]
    ba, bb = a.shape[:-2] if a.ndim >= 2 else (), b.shape[:-2] if b.ndim >= 2 else ()
    nb = max(len(ba), len(bb))
    ba, bb = (1,) * (nb - len(ba)) + tuple(ba), (1,) * (nb - len(bb)) + tuple(bb)
    ob = tuple(max(x, y) for x, y in zip(ba, bb))
    a3, b3 = a.reshape(ba + (M, K)), b.reshape(bb + (K * N,))
    out = np.zeros(ob + (M, N), dtype=a.dtype)
    for idx in np.ndindex(*ob):
        ia = tuple(0 if ba[i] == 1 else idx[i] for i in range(nb))
        ib = tuple(0 if bb[i] == 1 else idx[i] for i in range(nb))
        case = cases.gemm_case(seed=0, dtype=dtype, m=M, k=K, n_out=N, e_in=e_a, e_w=(e_b, e_b), e_out=e_out, act=act, bias=False,
                               round_mode=round_mode)
        case["x"] = np.ascontiguousarray(a3[ia]).reshape(case["x"].shape)
        case["w"] = np.ascontiguousarray(b3[ib]).reshape(case["w"].shape)
        assert o.oracle_conv2d(cases.conv_desc(case)) == 0
        out[idx] = case["out"].reshape(M, N)
    if a.ndim == 1 and b.ndim == 1:
        return out.reshape(1)
    if a.ndim == 1:
        return out.reshape(ob + (N,))
    if b.ndim == 1:
        return out.reshape(ob + (M,))
    return out


def run_graph(m, inputs, round_mode=abi.ROUND_HALF_UP, target=None, backend="port"):
    """m: espdl_file.read() result; inputs: {name: NHWC array with any batch}.  Returns {tensor name: array}.
    backend "port" = the plain-C oracle, "reference" = the reference's compiled operators (per-tensor exponents only)."""
    o = checkers.oracle() if backend == "port" else _RefBackend()
    target = target or m["metadata"].get("target") or "c"
    exps, dts = _exponents(m), _dtypes(m)
    init = m["initializers"]
    t = dict(inputs)
    for node in m["nodes"]:
        op, ins, outs, at = node["op_type"], node["inputs"], node["outputs"], node["attrs"]
        x = t[ins[0]] if ins[0] in t else None
        if op in ("Conv", "Gemm"):
            dt = QDT[at["quant_type"]]
            wt = init[ins[1]]
            bias = init[ins[2]]["data"] if len(ins) > 2 else None
            per_channel = len(wt["exponents"]) > 1
            if op == "Gemm":
                k, n_out = wt["dims"][2], wt["dims"][3]
                w = espdl_file.filter_to_ohwi(wt["data"], wt["dims"], target)
                rows = x.size // k
                case = cases.gemm_case(m=rows, k=k, n_out=n_out, dtype=dt)
                case["x"] = np.ascontiguousarray(x.reshape(1, 1, rows, k))
                out_shape = x.shape[:-1] + (n_out,)
            else:
                group = at.get("group", 1)
                conv1d = len(wt["dims"]) == 3  # [N, W, C] with filter [K, Cin, Cout]: one row (esp-dl/dl/base/dl_base.hpp:150-182)
                wdims = [1] + list(wt["dims"]) if conv1d else wt["dims"]
                if conv1d:
                    x = x.reshape(x.shape[0], 1, x.shape[1], x.shape[2])
                kh, kw, cin, cout = wdims
                depthwise = group != 1
                if depthwise:
                    w = espdl_file.depthwise_filter_to_hwc(wt["data"], wdims, target)
                    cout = cin
                else:
                    w = espdl_file.filter_to_ohwi(wt["data"], wdims, target)
                pads = at.get("pads", [0, 0, 0, 0])  # ONNX [t, l, b, r]
                strides = at.get("strides", [1, 1])
                dil = at.get("dilations", [1, 1])
                if conv1d:
                    pads = [0, pads[0], 0, pads[1]] if len(pads) == 2 else pads
                    strides, dil = [1, strides[0]], [1, dil[0]]
                n, h, wd, c = x.shape
                case = cases.conv_case(dtype=dt, n=n, h=h, w=wd, cin=c, cout=cout, kh=kh, kw=kw, stride=tuple(strides), dil=tuple(dil),
                                       pad=(pads[0], pads[2], pads[1], pads[3]), depthwise=depthwise)
                case["x"] = np.ascontiguousarray(x)
                out_shape = (n, case["out_w"], cout) if conv1d else (n, case["out_h"], case["out_w"], cout)
            case.update(w=np.ascontiguousarray(w), b=bias, lut=None, per_channel=int(per_channel),
                        ew=np.asarray(wt["exponents"], dtype=np.int32) if per_channel else None,
                        filter_exponent=0 if per_channel else wt["exponents"][0], in_exponent=exps[ins[0]], out_exponent=exps[outs[0]],
                        activation=ACT[at.get("activation", "Linear")], round_mode=round_mode)
            case["out"] = np.zeros(case["out"].shape, dtype=cases.NP[dt])
            st = o.oracle_conv2d(cases.conv_desc(case))
            assert st == 0, (node["name"], st)
            t[outs[0]] = case["out"].reshape(out_shape)
        elif op in ("Add", "Sub", "Mul", "Div", "Max", "Min", "Mod", "Pow"):
            a, b = t[ins[0]], t.get(ins[1], None)
            if b is None:
                b = init[ins[1]]["data"]
            eop = {"Add": abi.ELT_ADD, "Sub": abi.ELT_SUB, "Mul": abi.ELT_MUL, "Div": abi.ELT_DIV, "Max": abi.ELT_MAX, "Min": abi.ELT_MIN,
                   "Mod": abi.ELT_MOD, "Pow": abi.ELT_POW}[op]
            out_shape = np.broadcast_shapes(a.shape, b.shape)
            nd = len(out_shape)
            case = cases.eltwise_case(eop, dtype=QDT[at["quant_type"]], out_shape=out_shape, in0_shape=(1,) * (nd - a.ndim) + a.shape,
                                      in1_shape=(1,) * (nd - b.ndim) + b.shape, e0=exps[ins[0]],
                                      e1=exps.get(ins[1], init.get(ins[1], {}).get("exponents", [0])[0] if ins[1] in init else 0), eo=exps[outs[0]],
                                      round_mode=round_mode)
            case["a"], case["b"] = np.ascontiguousarray(a), np.ascontiguousarray(b)
            assert nd <= 4
            assert o.oracle_eltwise(cases.eltwise_desc(case)) == 0
            t[outs[0]] = case["out"]
        elif op in ("RequantizeLinear", "QuantizeLinear", "DequantizeLinear"):
            idt = dts.get(ins[0], abi.DTYPE_INT8)
            odt = dts.get(outs[0], abi.DTYPE_INT8)
            case = cases.eltwise_case(abi.ELT_REQUANTIZE, in_dtype=idt, out_dtype=odt, out_shape=(x.size,), e0=exps[ins[0]], eo=exps[outs[0]],
                                      round_mode=round_mode)
            case["a"] = np.ascontiguousarray(x.reshape(-1))
            assert o.oracle_eltwise(cases.eltwise_desc(case)) == 0
            t[outs[0]] = case["out"].reshape(x.shape)
        elif "lut" in at:
            table = init[at["lut"]]["data"]
            if x.dtype == np.int16:  # 65536 / step + 1 entries (dl_module_lut.hpp:33-36)
                step = (65536 // (table.size - 1)) if table.size > 1 else 1
                case = cases.eltwise_case(abi.ELT_LUT, dtype=abi.DTYPE_INT16, out_shape=(x.size,), lut_shift=int(step).bit_length() - 1,
                                          round_mode=round_mode)
            else:
                case = cases.eltwise_case(abi.ELT_LUT, out_shape=(x.size,))
            case["a"], case["b"] = np.ascontiguousarray(x.reshape(-1)), np.ascontiguousarray(table)
            assert o.oracle_eltwise(cases.eltwise_desc(case)) == 0
            t[outs[0]] = case["out"].reshape(x.shape)
        elif op in ("GlobalAveragePool", "MaxPool", "AveragePool"):
            pop = {"GlobalAveragePool": abi.POOL_GLOBAL_AVG, "MaxPool": abi.POOL_MAX, "AveragePool": abi.POOL_AVG}[op]
            pool1d = x.ndim == 3  # [N, W, C]: one row (dl_module_average_pool.hpp / dl_module_max_pool.hpp, 1-D form)
            x4 = x.reshape(x.shape[0], 1, x.shape[1], x.shape[2]) if pool1d else x
            n, h, wd, c = x4.shape
            ks = at.get("kernel_shape", [h, wd])
            pads = at.get("pads", [0, 0, 0, 0])
            st = at.get("strides", [1, 1])
            if pool1d and op != "GlobalAveragePool":
                ks, st, pads = [1, ks[0]], [1, st[0]], [0, pads[0], 0, pads[1]]
            case = cases.pool_case(pop, dtype=QDT[at["quant_type"]], n=n, h=h, w=wd, c=c, kh=ks[0], kw=ks[1], stride=(st[0], st[1]),
                                   pad=(pads[0], pads[2], pads[1], pads[3]), e_in=exps[ins[0]], e_out=exps[outs[0]])
            case["x"] = np.ascontiguousarray(x4)
            assert o.oracle_pool(cases.pool_desc(case)) == 0
            if pool1d:
                case["out"] = case["out"].reshape(n, case["out"].shape[2], c)
            t[outs[0]] = case["out"]
        elif op == "Transpose":
            t[outs[0]] = np.ascontiguousarray(x.transpose(at["perm"]))
        elif op == "Flatten":
            ax = at.get("axis", 1)
            t[outs[0]] = x.reshape(int(np.prod(x.shape[:ax])), -1)
        elif op == "Reshape":
            shp = [int(v) for v in init[ins[1]]["data"]]
            shp = [x.shape[i] if v == 0 else v for i, v in enumerate(shp)]
            if -1 not in shp and int(np.prod(shp)) != x.size:
                shp[0] = x.shape[0]
            t[outs[0]] = x.reshape(shp)
        elif op == "Concat":
            t[outs[0]] = np.concatenate([t[i] for i in ins], axis=at["axis"])
        elif op == "Resize":
            scales = init[ins[2]]["data"]
            n, h, wd, c = x.shape
            case = cases.resize_case(n=n, h=h, w=wd, c=c, scale=(float(scales[2]), float(scales[3])), e_in=exps[ins[0]], e_out=exps[outs[0]])
            case["x"] = np.ascontiguousarray(x)
            assert o.oracle_resize(cases.resize_desc(case)) == 0
            t[outs[0]] = case["out"]
        elif op == "Split":
            ax = at.get("axis", 0) % x.ndim
            if len(ins) > 1 and ins[1] in init:
                sizes = [int(v) for v in init[ins[1]]["data"]]
            else:
                sizes = [x.shape[ax] // len(outs)] * len(outs)
            pos = 0
            for name, sz in zip(outs, sizes):
                t[name] = np.ascontiguousarray(np.take(x, range(pos, pos + sz), axis=ax))
                pos += sz
        elif op in ("GRU", "LSTM"):
            def operand(i):
                if i >= len(ins) or not ins[i]:
                    return None, 0
                if ins[i] in t:
                    return np.ascontiguousarray(t[ins[i]]), exps[ins[i]]
                return np.ascontiguousarray(init[ins[i]]["data"].reshape(init[ins[i]]["dims"])), (init[ins[i]]["exponents"] or [0])[0]
            d = abi.RnnDesc()
            hid, dirs = at["hidden_size"], 2 if at.get("direction", "forward") == "bidirectional" else 1
            d.op, d.dtype = (abi.RNN_GRU if op == "GRU" else abi.RNN_LSTM), QDT[at["quant_type"]]
            d.seq_length, d.input_size, d.hidden_size, d.directions = x.shape[0], x.shape[2], hid, dirs
            (w, ew), (r, er), (b, _), (h0, _), (c0, _) = operand(1), operand(2), operand(3), operand(5), operand(6)
            d.x_exponent, d.w_exponent, d.r_exponent = exps[ins[0]], ew, er
            d.y_exponent, d.h_exponent = exps[outs[0]], exps[outs[1]]
            d.c_exponent = d.gate_exponent = at.get("gate_exponent", -8)
            d.round_mode = round_mode
            tabs = []
            for which in (0, 1):
                n = o.oracle_rnn_table(d.gate_exponent, which, None)
                tb = np.zeros(n + 1, dtype=np.float32)
                o.oracle_rnn_table(d.gate_exponent, which, tb.ctypes.data)
                tabs.append((tb, n))
            xc = np.ascontiguousarray(x)
            y = np.zeros((x.shape[0], dirs, 1, hid), dtype=x.dtype)
            yh, yc = np.zeros((dirs, 1, hid), dtype=x.dtype), np.zeros((dirs, 1, hid), dtype=np.int16)
            d.x, d.w, d.r = xc.ctypes.data, w.ctypes.data, r.ctypes.data
            d.b = b.ctypes.data if b is not None else None
            d.initial_h = h0.ctypes.data if h0 is not None else None
            d.initial_c = c0.ctypes.data if c0 is not None else None
            d.y, d.y_h, d.y_c = y.ctypes.data, yh.ctypes.data, yc.ctypes.data
            d.sigmoid_table, d.tanh_table, d.sigmoid_max, d.tanh_max = tabs[0][0].ctypes.data, tabs[1][0].ctypes.data, tabs[0][1], tabs[1][1]
            assert o.oracle_rnn(C.byref(d)) == 0
            t[outs[0]], t[outs[1]] = y, yh
            if op == "LSTM" and len(outs) > 2:
                t[outs[2]] = yc
        elif op == "LpNormalization":
            ax = at.get("axis", -1) % x.ndim
            d = abi.NormDesc()
            d.op, d.dtype, d.len, d.p = abi.NORM_LP, QDT[at["quant_type"]], x.shape[ax], at.get("p", 2)
            d.inner = int(np.prod(x.shape[ax + 1:], dtype=np.int64))
            d.rows = x.size // x.shape[ax]
            d.in_exponent, d.out_exponent, d.round_mode = exps[ins[0]], exps[outs[0]], round_mode
            xc, y = np.ascontiguousarray(x), np.zeros_like(x)
            d.input, d.output = xc.ctypes.data, y.ctypes.data
            assert o.oracle_norm(C.byref(d)) == 0
            t[outs[0]] = y
        elif op == "ReverseSequence":
            lens = np.ascontiguousarray(t[ins[1]] if ins[1] in t else init[ins[1]]["data"]).astype(np.int64)
            d = abi.ReverseSequenceDesc()
            d.elem_size, d.batch_axis, d.dim0, d.dim1 = x.dtype.itemsize, at.get("batch_axis", 1), x.shape[0], x.shape[1]
            d.feature = int(np.prod(x.shape[2:], dtype=np.int64))
            xc, y = np.ascontiguousarray(x), np.zeros_like(x)
            d.input, d.output = xc.ctypes.data, y.ctypes.data
            assert o.oracle_reverse_sequence(C.byref(d), lens.ctypes.data) == 0
            t[outs[0]] = y
        elif op == "ScatterND":
            idx = np.ascontiguousarray(t[ins[1]] if ins[1] in t else init[ins[1]]["data"].reshape(init[ins[1]]["dims"])).astype(np.int64)
            upd = np.ascontiguousarray(t[ins[2]] if ins[2] in t else init[ins[2]]["data"].reshape(init[ins[2]]["dims"]))
            d = abi.ScatterNDDesc()
            depth = idx.shape[-1]
            d.dtype, d.index_depth, d.n_slices = QDT[at["quant_type"]], depth, idx.size // depth
            d.reduction = {"none": 0, "add": 1, "mul": 2, "max": 3, "min": 4}.get(at.get("reduction", "none"), 0)
            d.slice_size, d.data_size = int(np.prod(x.shape[depth:], dtype=np.int64)), x.size
            for k in range(depth):
                d.axis_offset[k] = int(np.prod(x.shape[k + 1:], dtype=np.int64))
            xc, y = np.ascontiguousarray(x), np.zeros_like(x)
            d.data, d.indices, d.updates, d.output = xc.ctypes.data, idx.ctypes.data, upd.ctypes.data, y.ctypes.data
            assert o.oracle_scatter_nd(C.byref(d)) == 0
            t[outs[0]] = y
        elif op == "LogSoftmax":
            ax = at.get("axis", -1) % x.ndim
            table = np.zeros(256, dtype=np.float32)
            o.oracle_softmax_table(table.ctypes.data, exps[ins[0]])
            d = abi.SoftmaxDesc()
            d.len, d.inner, d.log, d.in_exponent = x.shape[ax], int(np.prod(x.shape[ax + 1:], dtype=np.int64)), 1, exps[ins[0]]
            d.rows, d.out_dtype = x.size // x.shape[ax], abi.DTYPE_FLOAT
            xc, y = np.ascontiguousarray(x), np.zeros(x.shape, dtype=np.float32)
            d.input, d.output, d.exp_table = xc.ctypes.data, y.ctypes.data, table.ctypes.data
            assert o.oracle_softmax(C.byref(d)) == 0
            t[outs[0]] = y
        elif op == "Softmax":
            ax = at.get("axis", -1) % x.ndim
            assert ax == x.ndim - 1
            table = np.zeros(256, dtype=np.float32)
            o.oracle_softmax_table(table.ctypes.data, exps[ins[0]])
            xs = np.ascontiguousarray(x.reshape(-1, x.shape[-1]))
            y = np.zeros(xs.shape, dtype=np.float32)
            assert o.oracle_softmax(cases.softmax_desc(xs.ctypes.data, y.ctypes.data, table.ctypes.data, xs.shape[0], xs.shape[1], abi.DTYPE_FLOAT, 0)) == 0
            t[outs[0]] = y.reshape(x.shape)
        elif op == "MatMul":
            b_op = t[ins[1]] if ins[1] in t else init[ins[1]]["data"].reshape(init[ins[1]]["dims"])
            e_b = exps[ins[1]] if ins[1] in exps else init[ins[1]]["exponents"][0]
            t[outs[0]] = matmul(o, x, b_op, exps[ins[0]], e_b, exps[outs[0]], QDT[at["quant_type"]],
                                ACT[at.get("activation", "Linear")], round_mode)
        elif op in ("ReduceMean", "ReduceSum", "ReduceMax", "ReduceMin", "ReduceProd", "ReduceLogSum", "ReduceLogSumExp"):
            axes = [int(a) % x.ndim for a in init[ins[1]]["data"]] if len(ins) > 1 and ins[1] in init else list(range(x.ndim))
            d = abi.ReduceDesc()
            d.op = {"ReduceMean": abi.REDUCE_MEAN, "ReduceSum": abi.REDUCE_SUM, "ReduceMax": abi.REDUCE_MAX, "ReduceMin": abi.REDUCE_MIN,
                    "ReduceProd": abi.REDUCE_PROD, "ReduceLogSum": abi.REDUCE_LOG_SUM, "ReduceLogSumExp": abi.REDUCE_LOG_SUM_EXP}[op]
            d.dtype, d.ndim = QDT[at["quant_type"]], x.ndim
            for i, sz in enumerate(x.shape):
                d.shape[i], d.reduce[i] = sz, int(i in axes)
            d.in_exponent, d.out_exponent, d.round_mode = exps[ins[0]], exps[outs[0]], round_mode
            keep = at.get("keepdims", 1)
            shape = [1 if i in axes else sz for i, sz in enumerate(x.shape)] if keep else ([sz for i, sz in enumerate(x.shape) if i not in axes] or [1])
            y = np.zeros(shape, dtype=x.dtype)
            xc = np.ascontiguousarray(x)
            d.input, d.output = xc.ctypes.data, y.ctypes.data
            assert o.oracle_reduce(C.byref(d)) == 0
            t[outs[0]] = y
        elif op == "Slice":
            starts, ends = [int(v) for v in init[ins[1]]["data"]], [int(v) for v in init[ins[2]]["data"]]
            axes = [int(v) for v in init[ins[3]]["data"]] if len(ins) > 3 else list(range(len(starts)))
            steps = [int(v) for v in init[ins[4]]["data"]] if len(ins) > 4 else [1] * len(starts)
            idx = [slice(None)] * x.ndim
            for s0, e0, a, st in zip(starts, ends, axes, steps):
                idx[a % x.ndim] = slice(s0, min(e0, x.shape[a % x.ndim]) if e0 >= 0 else e0, st)   # ONNX Slice = numpy slicing for st > 0
            t[outs[0]] = np.ascontiguousarray(x[tuple(idx)])
        elif op == "InsertZeros":  # esp-dl/dl/module/include/dl_module_insert_zeros.hpp:33-58,76-128
            sp = x.ndim - 2
            stride = list(at.get("stride", [1]))
            opad = list(at.get("output_padding", [0]))
            stride = stride * sp if len(stride) == 1 else stride
            opad = opad * sp if len(opad) == 1 else opad
            shape = list(x.shape)
            for i in range(sp):
                shape[1 + i] = x.shape[1 + i] + (stride[i] - 1) * (x.shape[1 + i] - 1) + opad[i]
            y = np.zeros(shape, dtype=x.dtype)
            idx = (slice(None),) + tuple(slice(0, (x.shape[1 + i] - 1) * stride[i] + 1, stride[i]) for i in range(sp)) + (slice(None),)
            y[idx] = x
            t[outs[0]] = y
        elif op in ("Squeeze", "Unsqueeze", "Identity"):
            shape = m["value_info"][outs[0]]["shape"] if op != "Identity" else list(x.shape)
            t[outs[0]] = np.ascontiguousarray(x).reshape([x.shape[0]] + list(shape[1:]) if len(shape) and shape[0] == 1 and x.size != int(np.prod(shape)) else shape)
        elif op == "PRelu":  # without a `lut` attribute: slopes per channel (esp-dl/dl/base/dl_base_prelu.cpp:5-19)
            alpha = init[ins[1]]
            case = cases.eltwise_case(abi.ELT_PRELU, dtype=QDT[at["quant_type"]], out_shape=(x.size // x.shape[-1], x.shape[-1]),
                                      e0=exps[ins[0]], e1=alpha["exponents"][0], eo=exps[outs[0]], round_mode=round_mode)
            case["a"], case["b"] = np.ascontiguousarray(x.reshape(-1, x.shape[-1])), np.ascontiguousarray(alpha["data"].reshape(-1))
            assert case["b"].size == x.shape[-1], "per-channel slopes expected"
            assert o.oracle_eltwise(cases.eltwise_desc(case)) == 0
            t[outs[0]] = case["out"].reshape(x.shape)
        else:
            raise NotImplementedError(op)
    return t
