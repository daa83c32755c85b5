"""ReduceMean / ReduceSum / ReduceMax / ReduceMin / ReduceL1 / ReduceSumSquare / ReduceL2 / ReduceProd / ReduceLogSum /
ReduceLogSumExp: the oracle against the reference's own modules compiled for the host (pin), the CUDA kernel against the
oracle.  The two logarithm reductions call logf / expf on the device: their results may differ from the host's by one
code where the last bit of logf decides a rounding; everything else is bit-exact."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

# (shape, reduced axes)
SHAPES = [((2, 7, 7, 40), (1, 2)), ((3, 5, 6, 8), (3,)), ((4, 9, 16), (0, 2)), ((6, 33), (1,)), ((6, 33), (0,)), ((5, 4, 3, 2), (0, 1, 2, 3)),
          ((2, 3, 4, 5), (0, 3)), ((17,), (0,))]


def make(op, dtype, shape, axes, e_in, e_out, seed, inp=None, out=None, keep=None):
    rng = np.random.default_rng(seed)
    t = np.int8 if dtype == abi.DTYPE_INT8 else np.int16
    info = np.iinfo(t)
    x = rng.integers(info.min, info.max + 1, size=shape, dtype=t)
    if op == abi.REDUCE_LOG_SUM:      # a sum that has a logarithm
        x = np.abs(x.astype(np.int32)).clip(0, info.max).astype(t)
    if op == abi.REDUCE_PROD:         # factors around one, so that products of a few dozen of them stay in range
        x = (x.astype(np.int32) // 3 + (info.max + 1) // 2).clip(info.min, info.max).astype(t)
    kept = [s for i, s in enumerate(shape) if i not in axes] or [1]
    y = np.zeros(kept, dtype=t)
    d = abi.ReduceDesc()
    d.op, d.dtype, d.ndim = op, dtype, len(shape)
    for i, s in enumerate(shape):
        d.shape[i], d.reduce[i] = s, int(i in axes)
    d.in_exponent, d.out_exponent, d.round_mode = e_in, e_out, abi.ROUND_HALF_UP
    d.input = x.ctypes.data if inp is None else inp
    d.output = y.ctypes.data if out is None else out
    if op == abi.REDUCE_LOG_SUM_EXP and dtype == abi.DTYPE_INT8:
        # tool::gen_lut_8bit(expf) as the host module builds it
        table = np.zeros(256, dtype=np.float32)
        checkers.oracle().oracle_softmax_table(table.ctypes.data, e_in)
        if keep is not None:
            keep.append(table)
        d.exp_table = table.ctypes.data
        d._table = table
    return d, x, y


CASES = [(op, dt, sh, ax) for op in range(10) for dt in (abi.DTYPE_INT8, abi.DTYPE_INT16) for sh, ax in SHAPES]
LOG_OPS = (abi.REDUCE_LOG_SUM, abi.REDUCE_LOG_SUM_EXP)


def exps(op, dt):
    if op == abi.REDUCE_SUM:
        return (-7, -3) if dt == abi.DTYPE_INT8 else (-14, -9)
    if op == abi.REDUCE_MEAN:
        return (-6, -7) if dt == abi.DTYPE_INT8 else (-12, -13)
    if op == abi.REDUCE_L1:
        return (-6, -1) if dt == abi.DTYPE_INT8 else (-14, -8)
    if op == abi.REDUCE_SUM_SQUARE:
        return (-6, 0) if dt == abi.DTYPE_INT8 else (-14, -7)
    if op == abi.REDUCE_L2:
        return (-6, -3) if dt == abi.DTYPE_INT8 else (-14, -11)
    if op == abi.REDUCE_PROD:
        return (-6, -5) if dt == abi.DTYPE_INT8 else (-14, -12)
    if op == abi.REDUCE_LOG_SUM:
        return (-5, -4) if dt == abi.DTYPE_INT8 else (-12, -11)
    if op == abi.REDUCE_LOG_SUM_EXP:
        return (-5, -4) if dt == abi.DTYPE_INT8 else (-13, -11)
    return (-5, -5)


@pytest.mark.parametrize("op,dt,shape,axes", CASES)
def test_oracle_matches_reference(op, dt, shape, axes):
    e_in, e_out = exps(op, dt)
    d, x, want = make(op, dt, shape, axes, e_in, e_out, seed=op * 100 + len(shape))
    assert checkers.ref().ref_reduce(C.byref(d)) == 0
    d2, x2, got = make(op, dt, shape, axes, e_in, e_out, seed=op * 100 + len(shape))
    assert checkers.oracle().oracle_reduce(C.byref(d2)) == 0
    np.testing.assert_array_equal(got, want)
    if op == abi.REDUCE_MAX:
        np.testing.assert_array_equal(got.reshape(-1), x.max(axis=axes).reshape(-1))


@pytest.mark.gpu
@pytest.mark.parametrize("op,dt,shape,axes", CASES + [(abi.REDUCE_MEAN, abi.DTYPE_INT8, (64, 14, 14, 576), (1, 2))])
def test_gpu_matches_oracle(op, dt, shape, axes):
    import gpu_util
    e_in, e_out = exps(op, dt)
    d, x, want = make(op, dt, shape, axes, e_in, e_out, seed=7)
    assert checkers.oracle().oracle_reduce(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        out = dev.upload(np.full_like(want, 0x55))
        dg, _, _ = make(op, dt, shape, axes, e_in, e_out, seed=7, inp=dev.upload(x), out=out)
        if dg.exp_table:
            dg.exp_table = dev.upload(dg._table)
        abi.check(dev.lib.espdl_b200_reduce(C.byref(dg), None), "reduce")
        got = dev.download(out, want)
    if op in LOG_OPS:  # logf / expf on the device: one code where their last bit decides the rounding
        assert np.abs(got.astype(np.int32) - want.astype(np.int32)).max() <= 1
    else:
        np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
def test_reduce_and_slice_nodes_in_a_model(tmp_path):
    """A graph with ReduceMean (spatial mean, keepdims), ReduceMax over channels and two Slice nodes, loaded and run by
    dl::Model: every node output equals the graph oracle's."""
    import graph_oracle
    from espdl_b200 import espdl_file, model
    g = espdl_file.GraphBuilder("reduce_slice") if hasattr(espdl_file, "GraphBuilder") else None
    if g is None:
        from espdl_b200 import zoo
        g = zoo._Net("reduce_slice", 1).g
    g.add_input("x", np.int8, [1, 12, 10, 32], -5)
    g.add_initializer("axes_hw", np.array([1, 2], dtype=np.int64))
    g.add_initializer("axes_c", np.array([-1], dtype=np.int64))
    g.add_node("ReduceMean", "mean", ["x", "axes_hw"], ["m"], keepdims=1, quant_type="S8")
    g.add_value_info("m", np.int8, [1, 1, 1, 32], -6)
    g.add_node("ReduceMax", "cmax", ["x", "axes_c"], ["c"], keepdims=0, quant_type="S8")
    g.add_value_info("c", np.int8, [1, 12, 10], -5)
    for name, arr in (("s0", [2, 1]), ("e0", [11, 9]), ("a0", [1, 2]), ("t0", [3, 2]), ("s1", [8]), ("e1", [1000]), ("a1", [-1])):
        g.add_initializer(name, np.array(arr, dtype=np.int64))
    g.add_node("Slice", "strided", ["x", "s0", "e0", "a0", "t0"], ["p"], quant_type="S8")
    g.add_value_info("p", np.int8, [1, 3, 4, 32], -5)
    g.add_node("Slice", "tail", ["x", "s1", "e1", "a1"], ["q"], quant_type="S8")
    g.add_value_info("q", np.int8, [1, 12, 10, 24], -5)
    for name, shape, e in (("m", [1, 1, 1, 32], -6), ("c", [1, 12, 10], -5), ("p", [1, 3, 4, 32], -5), ("q", [1, 12, 10, 24], -5)):
        g.outputs.append((name, np.int8, shape, [e]))
    g.value_info = [v for v in g.value_info if v[0] not in ("m", "c", "p", "q")]
    path = str(tmp_path / "rs.espdl")
    g.save(path)
    m = model.Model(path, batch=3)
    x = np.random.default_rng(3).integers(-128, 128, size=m.inputs[0].array.shape, dtype=np.int8)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(espdl_file.read(path), {"x": x})
    assert len(m.outputs) == 4
    for out in m.outputs:
        np.testing.assert_array_equal(out.array, want[out.name])
    m.close()
