"""Graph-level pin of the oracle: a whole generated network (per-tensor filter exponents, which the reference's C
path supports) run node by node through the plain-C oracle and through the reference's own operators gives the
same bytes at every node."""
import numpy as np
import pytest

import checkers
import graph_oracle
from espdl_b200 import abi, espdl_file, zoo


def per_tensor(g):
    g.initializers = [(n, a, ([e[0]] if e is not None and len(e) > 1 else e)) for n, a, e in g.initializers]
    return g


@pytest.mark.skipif(not checkers.have_ref(), reason="oracle/_ref/libespdl_ref.so not built")
@pytest.mark.parametrize("net", ["block", "mobilenet"])
def test_oracle_graph_equals_reference_graph(net):
    g = zoo.inverted_residual_block(seed=4, hw=28) if net == "block" else zoo.mobilenet_v2(seed=5, input_hw=64)
    m = espdl_file.read(per_tensor(g).serialize())
    rng = np.random.default_rng(3)
    shape = [2] + m["inputs"][0]["shape"][1:]
    x = rng.integers(-128, 128, size=shape, dtype=np.int8)
    a = graph_oracle.run_graph(m, {m["inputs"][0]["name"]: x}, backend="port")
    b = graph_oracle.run_graph(m, {m["inputs"][0]["name"]: x}, backend="reference")
    for node in m["nodes"]:
        for name in node["outputs"]:
            assert np.array_equal(a[name], b[name]), (node["op_type"], node["name"])
    out = a[m["outputs"][0]["name"]]
    assert out.std() > 3


def test_generated_mobilenet_activations_are_not_degenerate():
    """The synthetic weights keep every layer's activations inside the int8 range without saturating everywhere."""
    m = espdl_file.read(zoo.mobilenet_v2(seed=5, input_hw=96).serialize())
    x = np.random.default_rng(0).integers(-128, 128, size=(1, 96, 96, 3), dtype=np.int8)
    t = graph_oracle.run_graph(m, {"input": x})
    for node in m["nodes"]:
        if node["op_type"] == "Conv":
            v = t[node["outputs"][0]].astype(np.int32)
            assert (np.abs(v) >= 127).mean() < 0.35, node["name"]
            assert v.std() > 2, node["name"]


def test_yolo11n_style_generator_runs_through_the_oracle(tmp_path):
    """The detector-shaped graph: node mix of the configuration, and a full oracle pass at 64x64 whose attention block
    and heads produce non-degenerate values."""
    import collections
    g = zoo.yolo11n_style(seed=6, input_hw=64)
    path = str(tmp_path / "det.espdl")
    g.save(path)
    m = espdl_file.read(path)
    ops = collections.Counter(n["op_type"] for n in m["nodes"])
    assert ops["Conv"] >= 60 and ops["Swish"] >= 50 and ops["MatMul"] == 2 and ops["Softmax"] == 1 and ops["MaxPool"] == 3
    assert ops["Resize"] == 2 and ops["Concat"] >= 10 and ops["Split"] >= 8 and len(m["outputs"]) == 6
    x = np.random.default_rng(3).integers(-128, 128, size=(1, 64, 64, 3), dtype=np.int8)
    t = graph_oracle.run_graph(m, {"input": x})
    for node in m["nodes"]:
        if node["op_type"] in ("MatMul", "QuantizeLinear"):
            assert t[node["outputs"][0]].std() > 0.5, node["name"]
    for o in m["outputs"]:
        v = t[o["name"]].astype(int)
        assert v.std() > 5 and (np.abs(v) >= 127).mean() < 0.3


@pytest.mark.parametrize("name", ["esp32p4__zoo_mobilenetv2.espdl", "esp32p4__zoo_yolo11n_320.espdl", "esp32p4__zoo_face_mnp.espdl",
                                  "esp32p4__zoo_ocr_det.espdl", "esp32p4__zoo_person_reid.espdl"])
def test_shipped_zoo_models_run_through_the_oracle(name):
    """The model-zoo files as shipped parse with the own FlatBuffers reader (ESP32-P4 filter layout, per-channel exponents) and
    run through the graph oracle with half-to-even rounding: outputs of the declared shapes, not saturated, and - the
    network has no cross-image step - independent of what else is in the batch."""
    import os
    parsed = espdl_file.read(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "espdl", name))
    inp = parsed["inputs"][0]
    x = np.random.default_rng(3).integers(-128, 128, size=inp["shape"], dtype=np.int8)
    want = graph_oracle.run_graph(parsed, {inp["name"]: x}, round_mode=abi.ROUND_HALF_EVEN, target="esp32p4")
    for out in parsed["outputs"]:
        y = want[out["name"]]
        assert list(y.shape) == list(out["shape"])
        assert y.astype(np.float32).std() > 0 and (np.abs(y.astype(np.int32)) == 127).mean() < 0.5


def test_yolo11n_640_topology_graph_is_well_formed():
    """The 640x640 detector built from the shipped graph's topology: 249 nodes with the shipped operator mix, and the graph
    oracle's activations use the int8 range in every node (not all zero, not all saturated)."""
    import collections
    import os
    from espdl_b200 import espdl_file, zoo
    import graph_oracle
    topo = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "yolo11n_640_topology.json")
    blob = zoo.yolo11n_640(topo, seed=6).serialize()
    m = espdl_file.read(blob)
    kinds = collections.Counter(n["op_type"] for n in m["nodes"])
    assert len(m["nodes"]) == 249 and kinds["Conv"] == 87 and kinds["Swish"] == 77 and kinds["Concat"] == 17 and kinds["MatMul"] == 2
    assert m["inputs"][0]["shape"] == [1, 640, 640, 3] and len(m["outputs"]) == 6
    x = np.random.default_rng(1).integers(-128, 128, size=(1, 640, 640, 3), dtype=np.int8)
    out = graph_oracle.run_graph(m, {"images": x})
    for n in m["nodes"]:
        for o in n["outputs"]:
            a = out[o]
            if a.dtype == np.int8:
                assert a.astype(np.float32).std() >= 2 and (np.abs(a.astype(int)) >= 127).mean() <= 0.5, (n["name"], o)
