"""The plain-C oracle replays every Gemm golden model the reference ships (tests/golden/espdl, copied from
the reference's test_apps by tests/golden/make_golden.py) and must reproduce the embedded expected output
exactly - the check the reference's own Model::test() performs on device."""
import glob
import os

import numpy as np
import pytest

import cases
import checkers
import graph_oracle
from espdl_b200 import abi, espdl_file

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "espdl")
GEMM_FILES = sorted(glob.glob(os.path.join(GOLDEN, "*__linear_*.espdl"))) + sorted(glob.glob(os.path.join(GOLDEN, "*__sin_mlp.espdl")))
TCN_FILES = sorted(glob.glob(os.path.join(GOLDEN, "*__streaming_tcn.espdl")))
ACT = {"Linear": abi.ACT_LINEAR, "Relu": abi.ACT_RELU}


def replay_gemm_chain(path, run_conv, round_mode):
    """Run the model's Gemm nodes in order with `run_conv(case) -> out` and return {tensor name: array}."""
    m = espdl_file.read(path)
    target = m["metadata"].get("target") or os.path.basename(path).split("__")[0]
    exps = {v["name"]: v["exponents"][0] for v in list(m["value_info"].values()) + m["inputs"] + m["outputs"]}
    tensors = {k: t["data"] for k, t in m["test_inputs"].items()}
    for node in m["nodes"]:
        assert node["op_type"] == "Gemm"
        x = tensors[node["inputs"][0]]
        wt = m["initializers"][node["inputs"][1]]
        w = espdl_file.filter_to_ohwi(wt["data"], wt["dims"], target)
        b = m["initializers"][node["inputs"][2]]["data"] if len(node["inputs"]) > 2 else None
        k, n_out = wt["dims"][2], wt["dims"][3]
        rows = x.size // k
        case = cases.gemm_case(m=rows, k=k, n_out=n_out)
        case.update(x=np.ascontiguousarray(x.reshape(1, 1, rows, k)), w=w, b=b, ew=None, per_channel=0,
                    filter_exponent=wt["exponents"][0], in_exponent=exps[node["inputs"][0]],
                    out_exponent=exps[node["outputs"][0]], activation=ACT[node["attrs"]["activation"]], round_mode=round_mode)
        case["out"] = np.zeros((1, 1, rows, n_out), dtype=np.int8)
        out = run_conv(case)
        tensors[node["outputs"][0]] = out.reshape(x.shape[:-1] + (n_out,))
    return m, tensors


def oracle_conv(case):
    assert checkers.oracle().oracle_conv2d(cases.conv_desc(case)) == 0
    return case["out"]


def test_golden_files_present():
    assert len(GEMM_FILES) == 11


@pytest.mark.parametrize("path", GEMM_FILES, ids=os.path.basename)
def test_oracle_reproduces_golden_gemm(path):
    # ESP32-P4 exports are checked with its round-half-even, the other targets with round-half-up
    mode = abi.ROUND_HALF_EVEN if "esp32p4" in os.path.basename(path) else abi.ROUND_HALF_UP
    m, tensors = replay_gemm_chain(path, oracle_conv, mode)
    assert m["test_outputs"]
    for name, t in m["test_outputs"].items():
        np.testing.assert_array_equal(tensors[name].reshape(-1), t["data"].reshape(-1))


@pytest.mark.skipif(not checkers.have_ref(), reason="oracle/_ref/libespdl_ref.so not built")
@pytest.mark.parametrize("path", [p for p in GEMM_FILES if os.path.basename(p).startswith("c__")], ids=os.path.basename)
def test_reference_build_reproduces_golden_gemm(path):
    """The x86 build of the reference itself (oracle/_ref) passes its own "c"-target vectors."""
    def ref_conv(case):
        assert checkers.ref().ref_conv2d(cases.conv_desc(case), 1) == 0
        return case["out"]
    m, tensors = replay_gemm_chain(path, ref_conv, abi.ROUND_HALF_UP)
    for name, t in m["test_outputs"].items():
        np.testing.assert_array_equal(tensors[name].reshape(-1), t["data"].reshape(-1))


def test_streaming_tcn_files_present():
    assert [os.path.basename(p).split("__")[0] for p in TCN_FILES] == ["esp32p4", "esp32s3"]


@pytest.mark.parametrize("path", TCN_FILES, ids=os.path.basename)
def test_oracle_reproduces_the_streaming_tcn_vector(path):
    """The streaming tutorial model (examples/tutorial/how_to_deploy_streaming_model) embeds a test input and the
    output the exporter computed for it: the only shipped vector that runs through Conv1d, dilated depthwise conv,
    LUT-Sigmoid, Mul, Add, AveragePool, Slice and Gemm, with ESP32-P4 half-to-even / ESP32-S3 half-up rounding and the
    16-wide filter layout.  The graph oracle has to reproduce it exactly (the check of the reference's Model::test(),
    esp-dl/dl/model/src/dl_model_base.cpp:442-519)."""
    target = os.path.basename(path).split("__")[0]
    mode = abi.ROUND_HALF_EVEN if target == "esp32p4" else abi.ROUND_HALF_UP
    m = espdl_file.read(path)
    assert m["test_inputs"] and m["test_outputs"]
    ops = {n["op_type"] for n in m["nodes"]}
    assert {"Conv", "Gemm", "Mul", "Add"} <= ops
    shapes = {v["name"]: v["shape"] for v in m["inputs"]}
    inputs = {k: t["data"].reshape(shapes[k]) for k, t in m["test_inputs"].items()}
    got = graph_oracle.run_graph(m, inputs, round_mode=mode, target=target)
    for name, t in m["test_outputs"].items():
        np.testing.assert_array_equal(np.asarray(got[name]).reshape(-1), t["data"].reshape(-1))
        assert t["data"].astype(np.float32).std() > 0
