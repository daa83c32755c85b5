"""RMSNormalization and LayerNormalization (int8 / int16): the oracle against the reference's own modules compiled for
the host, the CUDA kernel against the oracle through the C ABI.  Bit-exact: the kernel adds the variance terms in
element order and rounds every fp32 operation separately, as the reference's loops do."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

NP = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16}
SHAPES = [(6, 64), (3, 100), (17, 33), (1, 768), (40, 7), (5, 1)]


def make(op, dt, rows, n, seed, scale=True, bias=True, stats=True, round_mode=abi.ROUND_HALF_UP):
    rng = np.random.default_rng(seed)
    t = NP[dt]
    info = np.iinfo(t)
    is8 = dt == abi.DTYPE_INT8
    a = dict(op=op, dt=dt, rows=rows, n=n, round_mode=round_mode)
    a["x"] = rng.integers(info.min, info.max + 1, size=(rows, n), dtype=t)
    if rows > 2:
        a["x"][1, :] = 5       # a constant row: zero variance
        a["x"][2, :] = 0       # an all-zero row
    a["y"] = np.zeros((rows, n), dtype=t)
    a["e_in"], a["e_out"] = (-5, -6) if is8 else (-12, -13)
    a["scale"] = a["bias"] = a["mean"] = a["inv"] = None
    if op == abi.NORM_RMS:
        a["scale"] = (rng.standard_normal(n) * 0.5 + 1.0).astype(np.float32)
    else:
        if scale:
            a["scale"] = rng.integers(info.max // 4, info.max + 1, size=n, dtype=t)
        if scale and bias:
            a["bias"] = rng.integers(info.min, info.max + 1, size=n, dtype=t)
        if stats:
            a["mean"], a["inv"] = np.zeros(rows, dtype=t), np.zeros(rows, dtype=t)
    a["e_scale"], a["e_bias"] = (-6, -7) if is8 else (-14, -15)
    a["e_mean"], a["e_inv"] = (-4, -3) if is8 else (-11, -9)
    return a


def desc(a, ptrs=None):
    d = abi.NormDesc()
    names = dict(input="x", output="y", scale="scale", bias="bias", mean="mean", inv_std_dev="inv")
    for field, key in names.items():
        arr = a[key]
        setattr(d, field, None if arr is None else (ptrs[key] if ptrs else arr.ctypes.data))
    d.op, d.dtype, d.rows, d.len = a["op"], a["dt"], a["rows"], a["n"]
    d.in_exponent, d.out_exponent, d.scale_exponent, d.bias_exponent = a["e_in"], a["e_out"], a["e_scale"], a["e_bias"]
    d.mean_exponent, d.inv_std_dev_exponent = a["e_mean"], a["e_inv"]
    d.epsilon, d.round_mode = 1e-5, a["round_mode"]
    return d


def fresh(a):
    return dict(a, y=np.zeros_like(a["y"]), mean=None if a["mean"] is None else np.zeros_like(a["mean"]),
                inv=None if a["inv"] is None else np.zeros_like(a["inv"]))


VARIANTS = [(abi.NORM_RMS, {}), (abi.NORM_LAYER, {}), (abi.NORM_LAYER, dict(bias=False)), (abi.NORM_LAYER, dict(scale=False, bias=False, stats=False))]


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op,kw", VARIANTS)
@pytest.mark.parametrize("rows,n", SHAPES)
def test_oracle_matches_reference(op, kw, rows, n, dt):
    a = make(op, dt, rows, n, seed=rows * 10 + n, **kw)
    o, r = fresh(a), fresh(a)
    assert checkers.oracle().oracle_norm(C.byref(desc(o))) == 0
    assert checkers.ref().ref_norm(C.byref(desc(r))) == 0
    np.testing.assert_array_equal(o["y"], r["y"])
    if a["mean"] is not None:
        np.testing.assert_array_equal(o["mean"], r["mean"])
        np.testing.assert_array_equal(o["inv"], r["inv"])
    if n > 8:
        assert o["y"].std() > 0


@pytest.mark.gpu
@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op,kw", VARIANTS)
@pytest.mark.parametrize("rows,n", SHAPES + [(1024, 384), (3, 5000), (70, 96), (33, 36), (64, 260), (32, 4)])
def test_gpu_matches_oracle(op, kw, rows, n, dt, round_mode):
    import gpu_util
    a = make(op, dt, rows, n, seed=rows + n, round_mode=round_mode, **kw)
    want = fresh(a)
    assert checkers.oracle().oracle_norm(C.byref(desc(want))) == 0
    with gpu_util.DeviceBuffers() as dev:
        ptrs = {k: (None if a[k] is None else dev.upload(a[k] if k in ("x", "scale", "bias") else np.full_like(a[k], 0x55)))
                for k in ("x", "y", "scale", "bias", "mean", "inv")}
        abi.check(dev.lib.espdl_b200_norm(C.byref(desc(a, ptrs)), None), "norm")
        np.testing.assert_array_equal(dev.download(ptrs["y"], a["y"]), want["y"])
        if a["mean"] is not None:
            np.testing.assert_array_equal(dev.download(ptrs["mean"], a["mean"]), want["mean"])
            np.testing.assert_array_equal(dev.download(ptrs["inv"], a["inv"]), want["inv"])


@pytest.mark.gpu
@pytest.mark.parametrize("op", [abi.NORM_RMS, abi.NORM_LAYER])
def test_gpu_in_place(op):
    """The planner runs these modules in place: output aliasing input gives the same result."""
    import gpu_util
    a = make(op, abi.DTYPE_INT8, 50, 96, seed=4)
    want = fresh(a)
    assert checkers.oracle().oracle_norm(C.byref(desc(want))) == 0
    with gpu_util.DeviceBuffers() as dev:
        ptrs = {k: (None if a[k] is None else dev.upload(a[k])) for k in ("x", "scale", "bias", "mean", "inv")}
        ptrs["y"] = ptrs["x"]
        abi.check(dev.lib.espdl_b200_norm(C.byref(desc(a, ptrs)), None), "norm")
        np.testing.assert_array_equal(dev.download(ptrs["y"], a["y"]), want["y"])


@pytest.mark.gpu
@pytest.mark.parametrize("op", [abi.NORM_RMS, abi.NORM_LAYER])
@pytest.mark.parametrize("shape,axis", [((2, 9, 64), -1), ((3, 4, 5, 16), 2)])
def test_modules_in_a_model(tmp_path, op, shape, axis):
    """RMSNormalization (float scale parameter) and LayerNormalization (int8 scale and bias parameters, mean and
    inv_std_dev outputs) loaded from a one-node .espdl graph and run by dl::Model."""
    from espdl_b200 import espdl_file, model
    ax = axis % len(shape)
    rows, n = int(np.prod(shape[:ax])), int(np.prod(shape[ax:]))
    a = make(op, abi.DTYPE_INT8, rows, n, seed=21)
    want = fresh(a)
    assert checkers.oracle().oracle_norm(C.byref(desc(want))) == 0
    g = espdl_file.GraphBuilder("norm", metadata={"target": "c"})
    g.add_input("x", np.int8, list(shape), a["e_in"])
    pshape = list(shape[ax:])
    stat_shape = list(shape[:ax]) + [1] * (len(shape) - ax)
    if op == abi.NORM_RMS:
        g.add_initializer("scale", a["scale"].reshape(pshape))
        g.add_node("RMSNormalization", "n", ["x", "scale"], ["y"], quant_type="S8", axis=axis, epsilon=1e-5)
    else:
        g.add_initializer("scale", a["scale"].reshape(pshape), [a["e_scale"]])
        g.add_initializer("bias", a["bias"].reshape(pshape), [a["e_bias"]])
        g.add_node("LayerNormalization", "n", ["x", "scale", "bias"], ["y", "mean", "inv"], quant_type="S8", axis=axis, epsilon=1e-5)
        g.add_output("mean", np.int8, stat_shape, a["e_mean"])
        g.add_output("inv", np.int8, stat_shape, a["e_inv"])
    g.add_output("y", np.int8, list(shape), a["e_out"])
    path = str(tmp_path / "norm.espdl")
    g.save(path)
    m = model.Model(path)
    m.inputs[0].array[...] = a["x"].reshape(shape)
    m.run()
    outs = {t.name: np.asarray(t.array) for t in m.outputs}
    np.testing.assert_array_equal(outs["y"].reshape(rows, n), want["y"])
    if op == abi.NORM_LAYER:
        np.testing.assert_array_equal(outs["mean"].reshape(-1), want["mean"])
        np.testing.assert_array_equal(outs["inv"].reshape(-1), want["inv"])
    m.close()
