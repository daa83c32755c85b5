"""Pow, LogSoftmax, LpNormalization, ReverseSequence, ScatterND: the oracle against the reference's own modules compiled
for the host (pin), the CUDA kernels against the oracle through the C ABI.  Bit-exact except where a transcendental
function runs on the device (Pow on int16, LogSoftmax's logf): there the results agree within one code / one unit in the
last place of the logarithm."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

NPT = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16, abi.DTYPE_FLOAT: np.float32}


# ------------------------------------------------------------------------------------------ Pow
POW_SHAPES = [((2, 5, 7, 16), (2, 5, 7, 16)), ((2, 5, 7, 16), (1,)), ((1,), (3, 4, 8)), ((4, 1, 8), (4, 6, 8)), ((33,), (33,))]


def pow_case(dt, s0, s1, seed):
    rng = np.random.default_rng(seed)
    t = NPT[dt]
    info = np.iinfo(t)
    # bases of both signs (a negative base with a fractional power is NaN -> the minimum), small powers
    a = rng.integers(info.min // 2, info.max // 2, size=s0, dtype=t)
    b = rng.integers(-3 * (info.max // 8), 3 * (info.max // 8), size=s1, dtype=t)
    if a.size == 1:
        a = (np.abs(a.astype(np.int32)) + info.max // 3).astype(t)  # one base for all powers: a positive one
    out_shape = np.broadcast_shapes(s0, s1)
    nd = len(out_shape)
    e0, e1, eo = (-5, -6, -3) if dt == abi.DTYPE_INT8 else (-13, -14, -9)
    d = abi.EltwiseDesc()
    d.op, d.in_dtype, d.out_dtype, d.ndim = abi.ELT_POW, dt, dt, nd
    for i in range(nd):
        d.out_shape[i] = out_shape[i]
        d.in0_shape[i] = ([1] * (nd - len(s0)) + list(s0))[i]
        d.in1_shape[i] = ([1] * (nd - len(s1)) + list(s1))[i]
    d.in0_exponent, d.in1_exponent, d.out_exponent, d.round_mode = e0, e1, eo, abi.ROUND_HALF_UP
    return d, a, b, np.zeros(out_shape, dtype=t)


def run_host(fn, d, a, b, out):
    d.input0, d.input1, d.output = a.ctypes.data, b.ctypes.data, out.ctypes.data
    assert fn(C.byref(d)) == 0
    return out


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("s0,s1", POW_SHAPES)
def test_pow_oracle_matches_reference(dt, s0, s1):
    d, a, b, out = pow_case(dt, s0, s1, seed=len(s0) * 7 + len(s1))
    want = run_host(checkers.ref().ref_eltwise, d, a, b, out.copy())
    got = run_host(checkers.oracle().oracle_eltwise, d, a, b, out.copy())
    np.testing.assert_array_equal(got, want)
    assert len(np.unique(want)) > 3


def pow_table(e0, e1, eo):
    """The 256 x 256 answers of int8 Pow, computed by the oracle on the host (the host module does the same with powf)."""
    a = (np.arange(256).astype(np.uint8) ^ 0x80).astype(np.uint8).view(np.int8).reshape(256, 1).copy()
    b = (np.arange(256).astype(np.uint8) ^ 0x80).astype(np.uint8).view(np.int8).reshape(1, 256).copy()
    d = abi.EltwiseDesc()
    d.op, d.in_dtype, d.out_dtype, d.ndim = abi.ELT_POW, abi.DTYPE_INT8, abi.DTYPE_INT8, 2
    d.out_shape[0], d.out_shape[1], d.in0_shape[0], d.in0_shape[1], d.in1_shape[0], d.in1_shape[1] = 256, 256, 256, 1, 1, 256
    d.in0_exponent, d.in1_exponent, d.out_exponent, d.round_mode = e0, e1, eo, abi.ROUND_HALF_UP
    return run_host(checkers.oracle().oracle_eltwise, d, a, b, np.zeros((256, 256), dtype=np.int8))


@pytest.mark.gpu
@pytest.mark.parametrize("dt,table", [(abi.DTYPE_INT8, True), (abi.DTYPE_INT8, False), (abi.DTYPE_INT16, False)])
@pytest.mark.parametrize("s0,s1", POW_SHAPES)
def test_pow_gpu_matches_oracle(dt, table, s0, s1):
    import gpu_util
    d, a, b, out = pow_case(dt, s0, s1, seed=3)
    want = run_host(checkers.oracle().oracle_eltwise, d, a, b, out.copy())
    with gpu_util.DeviceBuffers() as dev:
        d.input0, d.input1, d.output = dev.upload(a), dev.upload(b), dev.upload(np.full_like(out, 0x55))
        if table:
            d.table = dev.upload(pow_table(d.in0_exponent, d.in1_exponent, d.out_exponent))
        abi.check(dev.lib.espdl_b200_eltwise(C.byref(d), None), "pow")
        got = dev.download(d.output, out)
    if table:
        np.testing.assert_array_equal(got, want)
    else:  # powf on the device
        diff = np.abs(got.astype(np.int64) - want.astype(np.int64))
        assert diff.max() <= 1 and (diff != 0).mean() < 0.01


# ------------------------------------------------------------------------------------------ LogSoftmax
def softmax_desc(rows, length, inner, e_in, log, out_dtype=abi.DTYPE_FLOAT, e_out=0):
    d = abi.SoftmaxDesc()
    d.rows, d.len, d.inner, d.log, d.in_exponent, d.out_dtype, d.out_exponent = rows, length, inner, log, e_in, out_dtype, e_out
    return d


LSM = [(6, 33, 1), (4, 10, 7), (1, 1000, 1), (3, 5, 16), (100, 33, 1), (5, 40, 20), (300, 400, 1), (70, 1000, 1)]  # outer, len, inner


@pytest.mark.parametrize("outer,length,inner", LSM)
def test_log_softmax_oracle_matches_reference(outer, length, inner):
    rng = np.random.default_rng(outer + length)
    x = rng.integers(-128, 128, size=(outer, length, inner), dtype=np.int8)
    table = np.zeros(256, dtype=np.float32)
    checkers.oracle().oracle_softmax_table(table.ctypes.data, -4)
    outs = []
    for fn, extra in ((checkers.ref().ref_softmax, (-4,)), (checkers.oracle().oracle_softmax, ())):
        d = softmax_desc(outer * inner, length, inner, -4, 1)
        y = np.zeros(x.shape, dtype=np.float32)
        d.input, d.output, d.exp_table = x.ctypes.data, y.ctypes.data, table.ctypes.data
        assert fn(C.byref(d), *extra) == 0
        outs.append(y)
    np.testing.assert_array_equal(outs[1], outs[0])


@pytest.mark.gpu
@pytest.mark.parametrize("outer,length,inner", LSM)
@pytest.mark.parametrize("log,out_dtype", [(1, abi.DTYPE_FLOAT), (1, abi.DTYPE_INT16), (0, abi.DTYPE_FLOAT), (0, abi.DTYPE_INT8)])
def test_softmax_any_axis_gpu_matches_oracle(outer, length, inner, log, out_dtype):
    import gpu_util
    rng = np.random.default_rng(5)
    x = rng.integers(-128, 128, size=(outer, length, inner), dtype=np.int8)
    table = np.zeros(256, dtype=np.float32)
    checkers.oracle().oracle_softmax_table(table.ctypes.data, -4)
    e_out = {abi.DTYPE_FLOAT: 0, abi.DTYPE_INT16: -10, abi.DTYPE_INT8: -7}[out_dtype]
    want = np.zeros(x.shape, dtype=NPT[out_dtype])
    d = softmax_desc(outer * inner, length, inner, -4, log, out_dtype, e_out)
    d.input, d.output, d.exp_table = x.ctypes.data, want.ctypes.data, table.ctypes.data
    assert checkers.oracle().oracle_softmax(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        d.input, d.output, d.exp_table = dev.upload(x), dev.upload(np.zeros_like(want)), dev.upload(table)
        abi.check(dev.lib.espdl_b200_softmax(C.byref(d), None), "softmax")
        got = dev.download(d.output, want)
    if not log:
        np.testing.assert_array_equal(got, want)  # the sum and the divisions are correctly rounded on both sides
    elif out_dtype == abi.DTYPE_FLOAT:
        # logf on the device (its last bit may differ from the host's), then a subtraction: an absolute error of one
        # unit in the last place of log(sum), which is below 16 here
        assert np.abs(got - want).max() <= 2 * np.spacing(np.float32(16.0))
    else:
        assert np.abs(got.astype(np.int32) - want.astype(np.int32)).max() <= 1


# ------------------------------------------------------------------------------------------ LpNormalization
LPN = [(6, 33, 1), (4, 10, 7), (2, 512, 1), (3, 5, 16), (1, 1, 9)]


def lp_desc(dt, outer, length, inner, p, e_out):
    d = abi.NormDesc()
    d.op, d.dtype, d.rows, d.len, d.inner, d.p = abi.NORM_LP, dt, outer * inner, length, inner, p
    d.in_exponent, d.out_exponent, d.round_mode = -5, e_out, abi.ROUND_HALF_UP
    return d


def lp_input(dt, outer, length, inner, seed):
    rng = np.random.default_rng(seed)
    info = np.iinfo(NPT[dt])
    x = rng.integers(info.min, info.max + 1, size=(outer, length, inner), dtype=NPT[dt])
    x[0, :, 0] = 0  # a row whose norm is zero
    return x


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("outer,length,inner", LPN)
def test_lp_norm_oracle_matches_reference(dt, p, outer, length, inner):
    x = lp_input(dt, outer, length, inner, seed=p * 10 + length)
    outs = []
    for fn in (checkers.ref().ref_lp_norm, checkers.oracle().oracle_norm):
        d = lp_desc(dt, outer, length, inner, p, -7 if dt == abi.DTYPE_INT8 else -15)
        y = np.zeros_like(x)
        d.input, d.output = x.ctypes.data, y.ctypes.data
        assert fn(C.byref(d)) == 0
        outs.append(y)
    np.testing.assert_array_equal(outs[1], outs[0])
    assert np.abs(outs[0]).max() > 0 or length == 1


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("p", [1, 2])
@pytest.mark.parametrize("outer,length,inner", LPN + [(64, 96, 49)])
def test_lp_norm_gpu_matches_oracle(dt, p, outer, length, inner):
    import gpu_util
    x = lp_input(dt, outer, length, inner, seed=4)
    d = lp_desc(dt, outer, length, inner, p, -7 if dt == abi.DTYPE_INT8 else -15)
    want = np.zeros_like(x)
    d.input, d.output = x.ctypes.data, want.ctypes.data
    assert checkers.oracle().oracle_norm(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        d.input, d.output = dev.upload(x), dev.upload(np.full_like(x, 0x55))
        abi.check(dev.lib.espdl_b200_norm(C.byref(d), None), "lp norm")
        got = dev.download(d.output, want)
    np.testing.assert_array_equal(got, want)


# ------------------------------------------------------------------------------------------ ReverseSequence
RSQ = [(0, 4, 9, 5), (1, 9, 4, 5), (0, 1, 6, 1), (1, 17, 3, 32)]  # batch_axis, dim0, dim1, feature


def rs_desc(dt, batch_axis, d0, d1, feature):
    d = abi.ReverseSequenceDesc()
    d.elem_size, d.batch_axis, d.dim0, d.dim1, d.feature = np.dtype(NPT[dt]).itemsize, batch_axis, d0, d1, feature
    return d


def rs_data(dt, batch_axis, d0, d1, feature, seed):
    rng = np.random.default_rng(seed)
    x = rng.integers(-100, 100, size=(d0, d1, feature)).astype(NPT[dt])
    batch, time = (d0, d1) if batch_axis == 0 else (d1, d0)
    lens = rng.integers(0, time + 1, size=batch).astype(np.int64)
    lens[0] = time
    return x, lens


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16, abi.DTYPE_FLOAT])
@pytest.mark.parametrize("batch_axis,d0,d1,feature", RSQ)
def test_reverse_sequence_oracle_matches_reference(dt, batch_axis, d0, d1, feature):
    x, lens = rs_data(dt, batch_axis, d0, d1, feature, seed=d0 + d1)
    outs = []
    for fn in (checkers.ref().ref_reverse_sequence, checkers.oracle().oracle_reverse_sequence):
        d = rs_desc(dt, batch_axis, d0, d1, feature)
        y = np.zeros_like(x)
        d.input, d.output = x.ctypes.data, y.ctypes.data
        assert fn(C.byref(d), lens.ctypes.data) == 0
        outs.append(y)
    np.testing.assert_array_equal(outs[1], outs[0])
    b = 0
    row = x[b] if batch_axis == 0 else x[:, b]
    np.testing.assert_array_equal(outs[0][b] if batch_axis == 0 else outs[0][:, b], row[::-1])


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16, abi.DTYPE_FLOAT])
@pytest.mark.parametrize("batch_axis,d0,d1,feature", RSQ + [(0, 64, 50, 256)])
def test_reverse_sequence_gpu_matches_oracle(dt, batch_axis, d0, d1, feature):
    import gpu_util
    x, lens = rs_data(dt, batch_axis, d0, d1, feature, seed=2)
    d = rs_desc(dt, batch_axis, d0, d1, feature)
    want = np.zeros_like(x)
    d.input, d.output = x.ctypes.data, want.ctypes.data
    assert checkers.oracle().oracle_reverse_sequence(C.byref(d), lens.ctypes.data) == 0
    with gpu_util.DeviceBuffers() as dev:
        d.input, d.output, d.seq_lens = dev.upload(x), dev.upload(np.zeros_like(x)), dev.upload(lens)
        abi.check(dev.lib.espdl_b200_reverse_sequence(C.byref(d), None), "reverse_sequence")
        got = dev.download(d.output, want)
    np.testing.assert_array_equal(got, want)


# ------------------------------------------------------------------------------------------ ScatterND
SND = [((6, 5, 8), 1, 9), ((6, 5, 8), 2, 14), ((6, 5, 8), 3, 40), ((50,), 1, 30), ((4, 300), 1, 7)]  # data shape, index depth, slices


def snd_case(dt, shape, depth, n_slices, reduction, seed):
    rng = np.random.default_rng(seed)
    if dt == abi.DTYPE_FLOAT:
        data = rng.standard_normal(shape).astype(np.float32)
        upd_vals = lambda s: rng.standard_normal(s).astype(np.float32)
    else:
        info = np.iinfo(NPT[dt])
        lim = 12 if reduction == abi.SCATTER_MUL else info.max  # products that sometimes saturate, sometimes not
        data = rng.integers(-lim, lim + 1, size=shape).astype(NPT[dt])
        upd_vals = lambda s: rng.integers(-lim, lim + 1, size=s).astype(NPT[dt])
    # index tuples with repeats: the order of the updates matters
    idx = np.stack([rng.integers(0, shape[k], size=n_slices) for k in range(depth)], axis=1).astype(np.int64)
    idx[-1] = idx[0]
    upd = upd_vals((n_slices,) + tuple(shape[depth:]))
    d = abi.ScatterNDDesc()
    d.dtype, d.reduction, d.index_depth, d.n_slices = dt, reduction, depth, n_slices
    d.slice_size = int(np.prod(shape[depth:], dtype=np.int64))
    d.data_size = int(np.prod(shape, dtype=np.int64))
    for k in range(depth):
        d.axis_offset[k] = int(np.prod(shape[k + 1:], dtype=np.int64))
    return d, data, idx, upd


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16, abi.DTYPE_FLOAT])
@pytest.mark.parametrize("reduction", range(5))
@pytest.mark.parametrize("shape,depth,n_slices", SND)
def test_scatter_nd_oracle_matches_reference(dt, reduction, shape, depth, n_slices):
    d, data, idx, upd = snd_case(dt, shape, depth, n_slices, reduction, seed=reduction + depth)
    outs = []
    for which in range(2):
        y = np.zeros_like(data)
        d.data, d.indices, d.updates, d.output = data.ctypes.data, idx.ctypes.data, upd.ctypes.data, y.ctypes.data
        if which == 0:
            sh = (C.c_int * len(shape))(*shape)
            assert checkers.ref().ref_scatter_nd(C.byref(d), sh, len(shape)) == 0
        else:
            assert checkers.oracle().oracle_scatter_nd(C.byref(d)) == 0
        outs.append(y)
    np.testing.assert_array_equal(outs[1], outs[0])
    assert not np.array_equal(outs[0], data)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16, abi.DTYPE_FLOAT])
@pytest.mark.parametrize("reduction", range(5))
@pytest.mark.parametrize("shape,depth,n_slices", SND)
def test_scatter_nd_gpu_matches_oracle(dt, reduction, shape, depth, n_slices):
    import gpu_util
    d, data, idx, upd = snd_case(dt, shape, depth, n_slices, reduction, seed=1)
    want = np.zeros_like(data)
    d.data, d.indices, d.updates, d.output = data.ctypes.data, idx.ctypes.data, upd.ctypes.data, want.ctypes.data
    assert checkers.oracle().oracle_scatter_nd(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        d.data, d.indices, d.updates, d.output = dev.upload(data), dev.upload(idx), dev.upload(upd), dev.upload(np.zeros_like(data))
        abi.check(dev.lib.espdl_b200_scatter_nd(C.byref(d), None), "scatter_nd")
        got = dev.download(d.output, want)
    np.testing.assert_array_equal(got, want)


# ------------------------------------------------------------------------------------------ the modules inside dl::Model
@pytest.mark.gpu
def test_new_operator_nodes_in_a_model(tmp_path):
    """A graph with Pow, ReduceProd, ReduceLogSumExp, LpNormalization (both axis kinds), ReverseSequence, ScatterND and
    LogSoftmax nodes, loaded and run by dl::Model: the bit-exact nodes equal the graph oracle, the two with a device
    logarithm stay within one code / one unit in the last place of the logarithm."""
    import graph_oracle
    from espdl_b200 import espdl_file, model, zoo
    g = zoo._Net("more_ops", 1).g
    g.add_input("x", np.int8, [1, 6, 5, 16], -5)
    g.add_initializer("two", np.array([64], dtype=np.int8), exponents=[-5])          # the power 2.0
    g.add_node("Pow", "pow", ["x", "two"], ["xp"], quant_type="S8")
    g.add_value_info("xp", np.int8, [1, 6, 5, 16], -3)
    g.add_initializer("axes_c", np.array([-1], dtype=np.int64))
    g.add_initializer("axes_w", np.array([2], dtype=np.int64))
    g.add_node("ReduceProd", "prod", ["x", "axes_w"], ["pr"], keepdims=0, quant_type="S8")
    g.add_value_info("pr", np.int8, [1, 6, 16], -3)
    g.add_node("ReduceLogSumExp", "lse", ["x", "axes_c"], ["ls"], keepdims=1, quant_type="S8")
    g.add_value_info("ls", np.int8, [1, 6, 5, 1], -4)
    g.add_node("LpNormalization", "l2c", ["x"], ["n2"], axis=-1, p=2, quant_type="S8")
    g.add_value_info("n2", np.int8, [1, 6, 5, 16], -7)
    g.add_node("LpNormalization", "l1h", ["x"], ["n1"], axis=1, p=1, quant_type="S8")
    g.add_value_info("n1", np.int8, [1, 6, 5, 16], -7)
    g.add_initializer("idx", np.array([[0, 2], [0, 4], [0, 2]], dtype=np.int64))
    g.add_initializer("upd", np.random.default_rng(1).integers(-128, 128, size=(3, 5, 16), dtype=np.int8), exponents=[-5])
    g.add_node("ScatterND", "scat", ["x", "idx", "upd"], ["sc"], reduction="add", quant_type="S8")
    g.add_value_info("sc", np.int8, [1, 6, 5, 16], -5)
    g.add_node("LogSoftmax", "lsm", ["x"], ["lf"], axis=-1, quant_type="S8")
    g.add_value_info("lf", np.float32, [1, 6, 5, 16], 0)
    exp = {"xp": -3, "pr": -3, "ls": -4, "n2": -7, "n1": -7, "sc": -5}
    for name, shape in (("xp", [1, 6, 5, 16]), ("pr", [1, 6, 16]), ("ls", [1, 6, 5, 1]), ("n2", [1, 6, 5, 16]), ("n1", [1, 6, 5, 16]), ("sc", [1, 6, 5, 16])):
        g.outputs.append((name, np.int8, shape, [exp[name]]))
    g.outputs.append(("lf", np.float32, [1, 6, 5, 16], [0]))
    g.value_info = [v for v in g.value_info if v[0] not in ("xp", "pr", "ls", "n2", "n1", "sc", "lf")]
    path = str(tmp_path / "more.espdl")
    g.save(path)
    m = model.Model(path, batch=1)
    x = np.random.default_rng(3).integers(-128, 128, size=m.inputs[0].array.shape, dtype=np.int8)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(espdl_file.read(path), {"x": x})
    assert len(m.outputs) == 7
    for out in m.outputs:
        if out.name == "lf":
            assert np.abs(out.array - want[out.name]).max() <= 2 * np.spacing(np.float32(16.0))
        elif out.name == "ls":
            assert np.abs(out.array.astype(np.int32) - want[out.name].astype(np.int32)).max() <= 1
        else:
            np.testing.assert_array_equal(out.array, want[out.name], err_msg=out.name)
    m.close()


@pytest.mark.gpu
def test_reverse_sequence_node_in_a_model(tmp_path):
    import graph_oracle
    from espdl_b200 import espdl_file, model, zoo
    g = zoo._Net("revseq", 1).g
    g.add_input("x", np.int16, [7, 3, 12], -9)       # [time, batch, feature]
    g.add_initializer("lens", np.array([7, 0, 4], dtype=np.int64))
    g.add_node("ReverseSequence", "rev", ["x", "lens"], ["y"], batch_axis=1, time_axis=0, quant_type="S16")
    g.outputs.append(("y", np.int16, [7, 3, 12], [-9]))
    path = str(tmp_path / "rev.espdl")
    g.save(path)
    m = model.Model(path)
    x = np.random.default_rng(4).integers(-32768, 32768, size=(7, 3, 12)).astype(np.int16)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(espdl_file.read(path), {"x": x})
    np.testing.assert_array_equal(m.outputs[0].array, want["y"])
    np.testing.assert_array_equal(m.outputs[0].array[:, 0], x[::-1, 0])
    m.close()
