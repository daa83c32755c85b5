"""Gather, SpaceToDepth, DepthToSpace ("DCR" / "CRD") and InsertZeros: the oracle against the reference's own modules compiled
for the host, the gather kernel against the oracle through the C ABI, and the modules through one-node .espdl graphs."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

NP = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16}

# (input shape, axis, indices)
GATHER = [((6, 5, 16), 0, [5, 0, 0, 3]), ((2, 9, 32), 1, [8, 1, 4, 4, 0, 7, 2]), ((3, 4, 7), 2, [6, 0, 3]), ((11,), 0, [10, 0, 5, 5]),
          ((4, 6, 3, 5), 2, [2]), ((2, 64, 48), 1, list(range(63, -1, -3)))]
# (mode, n, h, w, c, blocksize): mode 0 SpaceToDepth, 1 DepthToSpace DCR, 2 DepthToSpace CRD
DEPTH_SPACE = [(0, 2, 4, 6, 3, 2), (0, 1, 9, 6, 16, 3), (0, 2, 8, 8, 5, 4), (2, 2, 3, 5, 12, 2), (2, 1, 4, 4, 18, 3), (2, 2, 2, 3, 64, 4),
               (1, 2, 3, 5, 8, 2), (1, 1, 4, 2, 27, 3)]


def gather_desc(x, idx, axis, out, ptrs=None):
    d = abi.GatherDesc()
    d.input, d.output, d.indices = ptrs if ptrs else (x.ctypes.data, out.ctypes.data, idx.ctypes.data)
    d.elem_size, d.num_indices = x.dtype.itemsize, idx.size
    d.outer = int(np.prod(x.shape[:axis], dtype=np.int64))
    d.axis_size = x.shape[axis]
    d.inner = int(np.prod(x.shape[axis + 1:], dtype=np.int64))
    return d


def gather_data(shape, axis, indices, dt, seed):
    info = np.iinfo(NP[dt])
    x = np.random.default_rng(seed).integers(info.min, info.max + 1, size=shape, dtype=NP[dt])
    idx = np.asarray(indices, dtype=np.int32)
    return x, idx, np.take(x, idx, axis=axis)


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("shape,axis,indices", GATHER)
def test_gather_oracle_matches_reference_and_numpy(shape, axis, indices, dt):
    x, idx, want = gather_data(shape, axis, indices, dt, 3)
    got = np.zeros_like(want)
    assert checkers.oracle().oracle_gather(C.byref(gather_desc(x, idx, axis, got))) == 0
    np.testing.assert_array_equal(got, want)
    ref = np.zeros_like(want)
    sh = (C.c_int * len(shape))(*shape)
    assert checkers.ref().ref_gather(x.ctypes.data, ref.ctypes.data, idx.ctypes.data, idx.size, sh, len(shape), axis, dt) == 0
    np.testing.assert_array_equal(ref, want)


def depth_space_data(mode, n, h, w, c, bs, dt, seed):
    info = np.iinfo(NP[dt])
    x = np.random.default_rng(seed).integers(info.min, info.max + 1, size=(n, h, w, c), dtype=NP[dt])
    oshape = (n, h // bs, w // bs, c * bs * bs) if mode == 0 else (n, h * bs, w * bs, c // (bs * bs))
    return x, oshape


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("mode,n,h,w,c,bs", DEPTH_SPACE)
def test_depth_space_oracle_matches_reference(mode, n, h, w, c, bs, dt):
    x, oshape = depth_space_data(mode, n, h, w, c, bs, dt, 5)
    got, ref = np.zeros(oshape, dtype=x.dtype), np.zeros(oshape, dtype=x.dtype)
    assert checkers.oracle().oracle_depth_space(x.ctypes.data, got.ctypes.data, x.dtype.itemsize, n, h, w, c, bs, mode) == 0
    assert checkers.ref().ref_depth_space(x.ctypes.data, ref.ctypes.data, dt, n, h, w, c, bs, mode) == 0
    np.testing.assert_array_equal(got, ref)
    assert sorted(got.reshape(-1).tolist()) == sorted(x.reshape(-1).tolist())  # a permutation of the input
    if mode == 0:  # SpaceToDepth followed by DepthToSpace CRD gives the input back
        back = np.zeros_like(x)
        assert checkers.oracle().oracle_depth_space(got.ctypes.data, back.ctypes.data, x.dtype.itemsize, *oshape, bs, 2) == 0
        np.testing.assert_array_equal(back, x)


def test_depth_to_space_dcr_needs_blocksize_output_channels():
    x, oshape = depth_space_data(1, 1, 2, 2, 12, 2, abi.DTYPE_INT8, 1)
    out = np.zeros(oshape, dtype=np.int8)
    assert checkers.oracle().oracle_depth_space(x.ctypes.data, out.ctypes.data, 1, 1, 2, 2, 12, 2, 1) == abi.ERR_UNSUPPORTED


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("shape,axis,indices", GATHER)
def test_gather_gpu_matches_oracle(shape, axis, indices, dt):
    import gpu_util
    x, idx, _ = gather_data(shape, axis, indices, dt, 7)
    want = np.zeros(np.take(x, idx, axis=axis).shape, dtype=x.dtype)
    assert checkers.oracle().oracle_gather(C.byref(gather_desc(x, idx, axis, want))) == 0
    with gpu_util.DeviceBuffers() as dev:
        out = dev.upload(np.full_like(want, 0x55))
        d = gather_desc(x, idx, axis, want, ptrs=(dev.upload(x), out, dev.upload(idx)))
        abi.check(dev.lib.espdl_b200_gather(C.byref(d), None), "gather")
        got = dev.download(out, want)
    np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("index_dtype", [np.int64, np.int32])
@pytest.mark.parametrize("shape,axis,indices", GATHER[:3] + GATHER[4:])
def test_gather_module(tmp_path, shape, axis, indices, index_dtype):
    from espdl_b200 import espdl_file, model
    x, idx, want = gather_data(shape, axis, indices, abi.DTYPE_INT8, 9)
    g = espdl_file.GraphBuilder("gather", metadata={"target": "c"})
    g.add_input("x", np.int8, list(shape), -5)
    g.add_initializer("idx", idx.astype(index_dtype))
    g.add_node("Gather", "g", ["x", "idx"], ["y"], quant_type="S8", axis=axis - len(shape))  # negative axis as exporters write it
    g.add_output("y", np.int8, list(want.shape), -5)
    path = str(tmp_path / "gather.espdl")
    g.save(path)
    m = model.Model(path)
    m.inputs[0].array[...] = x
    m.run()
    np.testing.assert_array_equal(np.asarray(m.outputs[0].array).reshape(want.shape), want)
    m.close()


@pytest.mark.gpu
@pytest.mark.parametrize("dt,qt", [(abi.DTYPE_INT8, "S8"), (abi.DTYPE_INT16, "S16")])
@pytest.mark.parametrize("mode,n,h,w,c,bs", DEPTH_SPACE + [(0, 4, 64, 64, 16, 2), (2, 4, 32, 32, 64, 2)])
def test_depth_space_modules(tmp_path, mode, n, h, w, c, bs, dt, qt):
    from espdl_b200 import espdl_file, model
    x, oshape = depth_space_data(mode, n, h, w, c, bs, dt, 11)
    want = np.zeros(oshape, dtype=x.dtype)
    assert checkers.oracle().oracle_depth_space(x.ctypes.data, want.ctypes.data, x.dtype.itemsize, n, h, w, c, bs, mode) == 0
    g = espdl_file.GraphBuilder("ds", metadata={"target": "c"})
    g.add_input("x", x.dtype.type, [n, h, w, c], -5)
    if mode == 0:
        g.add_node("SpaceToDepth", "s", ["x"], ["y"], quant_type=qt, blocksize=bs)
    else:
        g.add_node("DepthToSpace", "d", ["x"], ["y"], quant_type=qt, blocksize=bs, mode="DCR" if mode == 1 else "CRD")
    g.add_output("y", x.dtype.type, list(oshape), -5)
    path = str(tmp_path / "ds.espdl")
    g.save(path)
    m = model.Model(path)
    m.inputs[0].array[...] = x
    m.run()
    np.testing.assert_array_equal(np.asarray(m.outputs[0].array).reshape(oshape), want)
    m.close()


# (input shape, stride per spatial axis, output padding per spatial axis)
INSERT_ZEROS = [((2, 5, 6, 8), (2, 2), (1, 1)), ((1, 7, 3, 16), (3, 2), (0, 1)), ((2, 9, 12), (2,), (1,)), ((1, 4, 4, 5), (1, 1), (0, 0))]


def insert_zeros_graph(shape, stride, opad, dt):
    """One-node graph as the exporter writes it, for the graph oracle and for dl::Model."""
    from espdl_b200 import espdl_file
    g = espdl_file.GraphBuilder("iz", metadata={"target": "c"})
    g.add_input("x", NP[dt], list(shape), -5)
    oshape = list(shape)
    for i, (s, p) in enumerate(zip(stride, opad)):
        oshape[1 + i] = shape[1 + i] + (s - 1) * (shape[1 + i] - 1) + p
    g.add_node("InsertZeros", "iz", ["x"], ["y"], quant_type="S8" if dt == abi.DTYPE_INT8 else "S16", stride=list(stride), output_padding=list(opad))
    g.add_output("y", NP[dt], oshape, -5)
    return g, oshape


@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("shape,stride,opad", INSERT_ZEROS)
def test_insert_zeros_graph_oracle_matches_reference(tmp_path, shape, stride, opad, dt):
    import graph_oracle
    from espdl_b200 import espdl_file
    g, oshape = insert_zeros_graph(shape, stride, opad, dt)
    path = str(tmp_path / "iz.espdl")
    g.save(path)
    info = np.iinfo(NP[dt])
    x = np.random.default_rng(13).integers(info.min, info.max + 1, size=shape, dtype=NP[dt])
    got = graph_oracle.run_graph(espdl_file.read(path), {"x": x})["y"]
    ref = np.full(oshape, 0x55, dtype=NP[dt])
    ci = lambda v: (C.c_int * len(v))(*v)
    assert checkers.ref().ref_insert_zeros(x.ctypes.data, ref.ctypes.data, dt, ci(shape), len(shape), ci(stride), ci(opad)) == 0
    np.testing.assert_array_equal(got, ref)


@pytest.mark.gpu
@pytest.mark.parametrize("dt", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("shape,stride,opad", INSERT_ZEROS + [((4, 40, 40, 64), (2, 2), (1, 1))])
def test_insert_zeros_module(tmp_path, shape, stride, opad, dt):
    import graph_oracle
    from espdl_b200 import espdl_file, model
    g, oshape = insert_zeros_graph(shape, stride, opad, dt)
    path = str(tmp_path / "iz.espdl")
    g.save(path)
    info = np.iinfo(NP[dt])
    x = np.random.default_rng(17).integers(info.min, info.max + 1, size=shape, dtype=NP[dt])
    want = graph_oracle.run_graph(espdl_file.read(path), {"x": x})["y"]
    m = model.Model(path)
    m.inputs[0].array[...] = x
    m.run()
    np.testing.assert_array_equal(np.asarray(m.outputs[0].array).reshape(oshape), want)
    m.close()
