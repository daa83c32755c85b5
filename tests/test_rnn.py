"""GRU and LSTM (quantized, batch 1): the oracle against the reference's own modules compiled for the host (pin), the
CUDA kernel against the oracle through the C ABI - bit-exact, every step of every direction."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

NPT = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16}


def tables(gate_exponent):
    o = checkers.oracle()
    out = []
    for which in (0, 1):
        n = o.oracle_rnn_table(gate_exponent, which, None)
        t = np.zeros(n + 1, dtype=np.float32)
        assert o.oracle_rnn_table(gate_exponent, which, t.ctypes.data) == n
        out.append((t, n))
    return out


def rnn_case(op, dt, seq, isz, hid, dirs, bias, init, seed, gate_exponent=-8):
    rng = np.random.default_rng(seed)
    t = NPT[dt]
    info = np.iinfo(t)
    G = 3 if op == abi.RNN_GRU else 4
    a = {}
    a["x"] = rng.integers(info.min, info.max + 1, size=(seq, 1, isz), dtype=t)
    a["w"] = rng.integers(info.min // 2, info.max // 2, size=(dirs, G * hid, isz), dtype=t)
    a["r"] = rng.integers(info.min // 2, info.max // 2, size=(dirs, G * hid, hid), dtype=t)
    a["b"] = rng.integers(-300, 300, size=(dirs, 2 * G * hid)).astype(np.int16) if bias else None
    a["h0"] = rng.integers(info.min, info.max + 1, size=(dirs, 1, hid), dtype=t) if init else None
    a["c0"] = rng.integers(-400, 400, size=(dirs, 1, hid)).astype(np.int16) if init and op == abi.RNN_LSTM else None
    a["y"] = np.zeros((seq, dirs, 1, hid), dtype=t)
    a["yh"] = np.zeros((dirs, 1, hid), dtype=t)
    a["yc"] = np.zeros((dirs, 1, hid), dtype=np.int16)
    d = abi.RnnDesc()
    d.op, d.dtype, d.seq_length, d.input_size, d.hidden_size, d.directions = op, dt, seq, isz, hid, dirs
    # exponents chosen so that the pre-activations spread over the tables' range
    if dt == abi.DTYPE_INT8:
        d.x_exponent, d.w_exponent, d.r_exponent, d.h_exponent, d.y_exponent = -6, -8, -8, -7, -7
    else:
        d.x_exponent, d.w_exponent, d.r_exponent, d.h_exponent, d.y_exponent = -14, -16, -16, -15, -15
    d.c_exponent = d.gate_exponent = gate_exponent
    d.round_mode = abi.ROUND_HALF_UP
    return d, a


def bind(d, a, put=lambda v: v.ctypes.data, tabs=None):
    (sig, smax), (tnh, tmax) = tabs
    d.x, d.w, d.r = put(a["x"]), put(a["w"]), put(a["r"])
    d.b = put(a["b"]) if a["b"] is not None else None
    d.initial_h = put(a["h0"]) if a["h0"] is not None else None
    d.initial_c = put(a["c0"]) if a["c0"] is not None else None
    d.y, d.y_h, d.y_c = put(a["y"]), put(a["yh"]), put(a["yc"])
    d.sigmoid_table, d.tanh_table, d.sigmoid_max, d.tanh_max = put(sig), put(tnh), smax, tmax


CASES = [(op, dt, seq, isz, hid, dirs, bias, init)
         for op in (abi.RNN_GRU, abi.RNN_LSTM) for dt in (abi.DTYPE_INT8, abi.DTYPE_INT16)
         for (seq, isz, hid, dirs, bias, init) in [(5, 16, 8, 1, True, True), (7, 10, 12, 2, True, True), (3, 24, 16, 2, True, False),
                                                   (4, 8, 5, 1, False, False), (1, 3, 2, 2, True, True)]]


@pytest.mark.parametrize("op,dt,seq,isz,hid,dirs,bias,init", CASES)
def test_oracle_matches_reference(op, dt, seq, isz, hid, dirs, bias, init):
    tabs = tables(-8)
    outs = []
    for fn in (checkers.ref().ref_rnn, checkers.oracle().oracle_rnn):
        d, a = rnn_case(op, dt, seq, isz, hid, dirs, bias, init, seed=seq * 31 + hid)
        bind(d, a, tabs=tabs)
        assert fn(C.byref(d)) == 0
        outs.append(a)
    for k in ("y", "yh") + (("yc",) if op == abi.RNN_LSTM else ()):
        np.testing.assert_array_equal(outs[1][k], outs[0][k], err_msg=k)
    assert len(np.unique(outs[0]["y"])) > 3


@pytest.mark.gpu
@pytest.mark.parametrize("op,dt,seq,isz,hid,dirs,bias,init", CASES + [(abi.RNN_GRU, abi.DTYPE_INT8, 50, 64, 128, 2, True, True),
                                                               (abi.RNN_LSTM, abi.DTYPE_INT16, 40, 40, 96, 2, True, True)])
def test_gpu_matches_oracle(op, dt, seq, isz, hid, dirs, bias, init):
    import gpu_util
    tabs = tables(-8)
    d, want = rnn_case(op, dt, seq, isz, hid, dirs, bias, init, seed=9)
    bind(d, want, tabs=tabs)
    assert checkers.oracle().oracle_rnn(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        dg, a = rnn_case(op, dt, seq, isz, hid, dirs, bias, init, seed=9)
        bind(dg, a, put=dev.upload, tabs=tabs)
        abi.check(dev.lib.espdl_b200_rnn(C.byref(dg), None), "rnn")
        for k, p in (("y", dg.y), ("yh", dg.y_h)) + ((("yc", dg.y_c),) if op == abi.RNN_LSTM else ()):
            np.testing.assert_array_equal(dev.download(p, want[k]), want[k], err_msg=k)


@pytest.mark.gpu
@pytest.mark.parametrize("op", ["GRU", "LSTM"])
def test_rnn_node_in_a_model(tmp_path, op):
    """A bidirectional GRU / LSTM node with bias and initial states, loaded and run by dl::Model: Y, Y_h (and Y_c) equal
    the graph oracle."""
    import graph_oracle
    from espdl_b200 import espdl_file, model, zoo
    rng = np.random.default_rng(11)
    seq, isz, hid, G = 9, 20, 24, 3 if op == "GRU" else 4
    g = zoo._Net("rnn", 1).g
    g.add_input("x", np.int8, [seq, 1, isz], -6)
    g.add_initializer("w", rng.integers(-64, 64, size=(2, G * hid, isz), dtype=np.int8), exponents=[-8])
    g.add_initializer("r", rng.integers(-64, 64, size=(2, G * hid, hid), dtype=np.int8), exponents=[-8])
    g.add_initializer("b", rng.integers(-300, 300, size=(2, 2 * G * hid)).astype(np.int16), exponents=[-8])
    g.add_initializer("lens", np.array([seq], dtype=np.int64))
    g.add_initializer("h0", rng.integers(-128, 128, size=(2, 1, hid), dtype=np.int8), exponents=[-7])
    ins = ["x", "w", "r", "b", "lens", "h0"]
    outs = [("y", np.int8, [seq, 2, 1, hid], -7), ("yh", np.int8, [2, 1, hid], -7)]
    attrs = dict(hidden_size=hid, direction="bidirectional", layout=0, gate_exponent=-8, quant_type="S8")
    if op == "GRU":
        attrs["linear_before_reset"] = 1
    else:
        g.add_initializer("c0", rng.integers(-400, 400, size=(2, 1, hid)).astype(np.int16), exponents=[-8])
        ins.append("c0")
        outs.append(("yc", np.int16, [2, 1, hid], -8))
    g.add_node(op, "rnn", ins, [o[0] for o in outs], **attrs)
    for name, dt, shape, e in outs:
        g.outputs.append((name, dt, shape, [e]))
    path = str(tmp_path / "rnn.espdl")
    g.save(path)
    m = model.Model(path)
    x = rng.integers(-128, 128, size=(seq, 1, isz), dtype=np.int8)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(espdl_file.read(path), {"x": x})
    assert len(m.outputs) == len(outs)
    for out in m.outputs:
        np.testing.assert_array_equal(out.array, want[out.name], err_msg=out.name)
    m.close()
