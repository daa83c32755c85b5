"""GPU parity at the model level: .espdl file -> C++ dl::Model (loader, planner, modules, CUDA graph) -> CUDA kernels,
compared with the plain-C oracle run node by node over the same graph, and the reference's own Model::test()
golden check on every golden model it ships for this path."""
import glob
import os

import numpy as np
import pytest

import graph_oracle
from espdl_b200 import abi, espdl_file, model, zoo

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "espdl")
GEMM_MODELS = (sorted(glob.glob(os.path.join(GOLDEN, "*__linear_*.espdl"))) + sorted(glob.glob(os.path.join(GOLDEN, "*__sin_mlp.espdl"))) +
               sorted(glob.glob(os.path.join(GOLDEN, "*__streaming_tcn.espdl"))))


@pytest.mark.parametrize("path", GEMM_MODELS, ids=os.path.basename)
def test_model_test_passes_on_shipped_golden_models(path, monkeypatch):
    """dl::Model::test(): embedded test inputs in, every embedded expected output compared - on the GPU.  The Gemm and
    sin-MLP files pin the Gemm path in all three filter layouts; the streaming-TCN files pin Conv1d, dilated depthwise
    conv, LUT-Sigmoid, Mul, Add, AveragePool and Slice under ESP32-P4 (half-to-even) and ESP32-S3 (half-up) rules."""
    monkeypatch.setenv("ESPDL_B200_TARGET", os.path.basename(path).split("__")[0])  # the tutorial models carry no target tag
    m = model.Model(path)
    assert m.test() == 0
    m.close()


@pytest.mark.parametrize("op_type,op,bool_out", [("Max", abi.ELT_MAX, False), ("Min", abi.ELT_MIN, False), ("Div", abi.ELT_DIV, False),
                                                 ("Mod", abi.ELT_MOD, False), ("Greater", abi.ELT_GREATER, True),
                                                 ("GreaterOrEqual", abi.ELT_GREATER_EQUAL, True), ("Equal", abi.ELT_EQUAL, True),
                                                 ("Less", abi.ELT_LESS, True), ("LessOrEqual", abi.ELT_LESS_EQUAL, True)])
@pytest.mark.parametrize("sa,sb", [((2, 6, 5, 16), (2, 6, 5, 16)), ((2, 6, 5, 16), (1, 1, 1, 16)), ((2, 6, 5, 16), (2, 6, 5, 1)), ((3, 1, 8), (4, 1))])
def test_two_operand_modules(tmp_path, op_type, op, bool_out, sa, sb):
    """Max / Min / Div / Mod and the comparisons loaded from a one-node .espdl graph and run through the C++ module
    (the module merges the broadcast shapes before it fills the descriptor) against the oracle on the unmerged shapes."""
    import cases
    e_a, e_b, e_out = -5, -4, -6
    so = list(np.broadcast_shapes(sa, sb))
    g = espdl_file.GraphBuilder("two", metadata={"target": "c"})
    g.add_input("a", np.int8, list(sa), e_a)
    g.add_input("b", np.int8, list(sb), e_b)
    g.add_node(op_type, "n", ["a", "b"], ["y"], quant_type="S8")
    g.add_output("y", np.bool_ if bool_out else np.int8, so, 0 if bool_out else e_out)
    path = str(tmp_path / "two.espdl")
    g.save(path)
    m = model.Model(path)
    nd = len(so)
    case = cases.eltwise_case(op, seed=31, in_dtype=abi.DTYPE_INT8, out_dtype=abi.DTYPE_BOOL if bool_out else abi.DTYPE_INT8, out_shape=tuple(so),
                              in0_shape=(1,) * (nd - len(sa)) + tuple(sa), in1_shape=(1,) * (nd - len(sb)) + tuple(sb), e0=e_a, e1=e_b,
                              eo=0 if bool_out else e_out)
    ins = {t.name: t for t in m.inputs}
    ins["a"].array[...] = case["a"].reshape(sa)
    ins["b"].array[...] = case["b"].reshape(sb)
    m.run()
    assert __import__("checkers").oracle().oracle_eltwise(cases.eltwise_desc(case)) == 0
    np.testing.assert_array_equal(np.asarray(m.outputs[0].array).view(np.uint8 if bool_out else np.int8).reshape(so), case["out"])
    m.close()


ZOO_MODELS = sorted(glob.glob(os.path.join(GOLDEN, "esp32*__zoo_*.espdl")))


@pytest.mark.parametrize("path", ZOO_MODELS, ids=os.path.basename)
def test_shipped_zoo_models_match_the_oracle(path, monkeypatch):
    """Model-zoo files as shipped (ImageNet MobileNetV2, YOLO11n at 320x320, face / pedestrian detectors, person
    re-identification, text detection: ESP32-P4 and ESP32-S3 filter layouts, per-channel exponents, half-to-even or half-up
    rounding, negative Transpose perms, Slice / Reshape / MatMul / Softmax, PRelu, InsertZeros) loaded by dl::Model and run
    on a seeded random image: every graph output equals the graph oracle's."""
    target = os.path.basename(path).split("__")[0]
    monkeypatch.setenv("ESPDL_B200_TARGET", target)  # the zoo files carry no target tag
    round_mode = abi.ROUND_HALF_EVEN if target == "esp32p4" else abi.ROUND_HALF_UP
    parsed = espdl_file.read(path)
    m = model.Model(path)
    x = np.random.default_rng(3).integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(parsed, {m.inputs[0].name: x}, round_mode=round_mode, target=target)
    assert len(m.outputs) >= 1
    for out in m.outputs:
        w = want[out.name]
        np.testing.assert_array_equal(np.asarray(out.array).reshape(w.shape), w)
        assert w.astype(np.float32).std() > 0
    m.close()


def run_and_compare(tmp_path, g, batch, seed, check_intermediates):
    path = str(tmp_path / "net.espdl")
    g.save(path)
    parsed = espdl_file.read(path)
    m = model.Model(path, batch=batch, graph=not check_intermediates, reuse=not check_intermediates)
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    m.inputs[0].array[...] = x
    m.run()
    want = graph_oracle.run_graph(parsed, {m.inputs[0].name: x})
    if check_intermediates:
        for node in parsed["nodes"]:
            for name in node["outputs"]:
                got = m.read_tensor(name, want[name].dtype, want[name].shape)
                assert np.array_equal(got, want[name]), f"{node['op_type']} {node['name']} -> {name} differs"
    for out in m.outputs:
        np.testing.assert_array_equal(out.array, want[out.name])
    return m, want


def test_mobilenet_v2_every_tensor_matches_oracle(tmp_path):
    """Full MobileNetV2-1.0 at 224x224, two images, no buffer reuse: every node output is compared."""
    m, want = run_and_compare(tmp_path, zoo.mobilenet_v2(seed=5), batch=2, seed=50, check_intermediates=True)
    logits = want[m.outputs[0].name]
    assert logits.shape == (2, 1000) and logits.std() > 4 and (np.abs(logits.astype(int)) == 127).mean() < 0.5
    assert not np.array_equal(logits[0], logits[1])
    m.close()


def test_mobilenet_v2_planned_arena_and_cuda_graph(tmp_path):
    """Same network with lifetime-based buffer reuse, in-place Adds and CUDA-graph replay: logits still identical,
    repeated runs identical, and a larger batch gives the same rows (images are independent units)."""
    m, want = run_and_compare(tmp_path, zoo.mobilenet_v2(seed=5), batch=2, seed=50, check_intermediates=False)
    first = m.outputs[0].array.copy()
    for _ in range(3):
        m.run()
        np.testing.assert_array_equal(m.outputs[0].array, first)
    assert m.arena_bytes < 2 * 14.4e6 * 0.6   # far below the sum of all node outputs (about 14.3 MB per image)
    m5 = model.Model(str(tmp_path / "net.espdl"), batch=5)
    x = np.concatenate([m.inputs[0].array, m.inputs[0].array[::-1], m.inputs[0].array[:1]], axis=0)
    m5.inputs[0].array[...] = x
    m5.run()
    np.testing.assert_array_equal(m5.outputs[0].array[:2], first)
    np.testing.assert_array_equal(m5.outputs[0].array[2:4], first[::-1])
    m.close()
    m5.close()


def test_inverted_residual_block(tmp_path):
    """The inverted-residual block configuration (112x112x32 -> 192 -> depthwise -> 32 + residual), three images."""
    m, want = run_and_compare(tmp_path, zoo.inverted_residual_block(seed=4), batch=3, seed=40, check_intermediates=True)
    out = want[m.outputs[0].name]
    assert out.std() > 10
    m.close()


def test_inverted_residual_block_full_batch(tmp_path):
    """The block configuration at its full size, 256 images of 112x112x32: the images are independent units, so the
    oracle (run on eight images picked from all over the batch) pins those rows, and every row must equal the row a
    batch of eight gives for the same image."""
    path = str(tmp_path / "block.espdl")
    zoo.inverted_residual_block(seed=4).save(path)
    parsed = espdl_file.read(path)
    m = model.Model(path, batch=256)
    rng = np.random.default_rng(41)
    x = rng.integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    x[17] = x[200]                      # two equal images far apart must give equal rows
    m.inputs[0].array[...] = x
    m.run()
    got = m.outputs[0].array.copy()
    m.close()
    picks = [0, 1, 17, 63, 128, 200, 254, 255]
    want = graph_oracle.run_graph(parsed, {"input": np.ascontiguousarray(x[picks])})[parsed["outputs"][0]["name"]]
    np.testing.assert_array_equal(got[picks], want)
    np.testing.assert_array_equal(got[17], got[200])
    m8 = model.Model(path, batch=8)
    for start in (8, 120, 248):
        m8.inputs[0].array[...] = x[start:start + 8]
        m8.run()
        np.testing.assert_array_equal(m8.outputs[0].array, got[start:start + 8])
    m8.close()


def test_submit_wait_pipeline_equals_run(tmp_path):
    """submit()/wait(): a stream of different batches through the pipelined entry points gives run()'s results, in
    order, with the input array refilled right after every submit."""
    path = str(tmp_path / "net.espdl")
    zoo.inverted_residual_block(seed=4, hw=28).save(path)
    m = model.Model(path, batch=4)
    rng = np.random.default_rng(2)
    batches = [rng.integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8) for _ in range(5)]
    want = []
    for b in batches:
        m.inputs[0].array[...] = b
        m.run()
        want.append(m.outputs[0].array.copy())
    got = []
    for i, b in enumerate(batches):
        m.inputs[0].array[...] = b
        m.submit()
        m.inputs[0].array[...] = 0x11        # the host buffer is free again
        if i >= 1:
            m.wait()
            got.append(m.outputs[0].array.copy())
    m.wait()
    got.append(m.outputs[0].array.copy())
    for g, w in zip(got, want):
        np.testing.assert_array_equal(g, w)
    with pytest.raises(RuntimeError):
        m.wait()                             # nothing outstanding
    m.close()


@pytest.mark.parametrize("sa,sb", [((3, 5, 32), (3, 32, 16)), ((2, 2, 7, 16), (1, 2, 16, 24)), ((6, 48), (48, 40)), ((4, 9, 24), (24, 8))])
def test_matmul_module(tmp_path, sa, sb):
    """MatMul of two graph inputs through the C++ module (one tile-kernel Gemm per broadcast slice; K = 24 takes the
    CUDA-core kernel) against the restatement that is pinned to the reference's own MatMul."""
    g = espdl_file.GraphBuilder("matmul", metadata={"target": "c"})
    e_a, e_b, e_out = -5, -6, -3
    g.add_input("a", np.int8, list(sa), e_a)
    g.add_input("b", np.int8, list(sb), e_b)
    so = list(np.matmul(np.zeros(sa), np.zeros(sb)).shape)
    g.add_node("MatMul", "mm", ["a", "b"], ["y"], quant_type="S8", activation="Relu")
    g.add_output("y", np.int8, so, e_out)
    path = str(tmp_path / "mm.espdl")
    g.save(path)
    m = model.Model(path)
    rng = np.random.default_rng(9)
    ins = {t.name: t for t in m.inputs}
    a = rng.integers(-128, 128, size=sa, dtype=np.int8)
    b = rng.integers(-128, 128, size=sb, dtype=np.int8)
    ins["a"].array[...] = a
    ins["b"].array[...] = b
    m.run()
    want = graph_oracle.matmul(__import__("checkers").oracle(), a, b, e_a, e_b, e_out, abi.DTYPE_INT8, abi.ACT_RELU, abi.ROUND_HALF_UP)
    np.testing.assert_array_equal(m.outputs[0].array, want.reshape(m.outputs[0].array.shape))
    assert want.std() > 0
    m.close()


def test_yolo11n_style_every_tensor_matches_oracle(tmp_path):
    """The detector-shaped graph (Conv + Swish LUT, C3k2 with Split / Add / Concat, SPPF max-pools, the attention
    block with two int8 MatMuls, Mul, Softmax and QuantizeLinear, Resize + Concat neck, three heads) at 96x96, two
    images, no buffer reuse: every one of its node outputs is compared."""
    m, want = run_and_compare(tmp_path, zoo.yolo11n_style(seed=6, input_hw=96), batch=2, seed=60, check_intermediates=True)
    assert len(m.outputs) == 6
    for out in m.outputs:
        assert want[out.name].std() > 5
    m.close()


def test_yolo11n_style_planned_arena_and_cuda_graph(tmp_path):
    """Same graph at 160x160 (25 tokens in the attention block), three images, with buffer reuse and CUDA-graph replay."""
    m, want = run_and_compare(tmp_path, zoo.yolo11n_style(seed=6, input_hw=160), batch=3, seed=61, check_intermediates=False)
    first = [o.array.copy() for o in m.outputs]
    m.run()
    for o, f in zip(m.outputs, first):
        np.testing.assert_array_equal(o.array, f)
    m.close()


def test_staged_run_equals_single_run(tmp_path):
    """run(stage_num, stage_index) over all stages gives run()'s result (reference: test_dl_api.cpp:70-98)."""
    path = str(tmp_path / "net.espdl")
    zoo.inverted_residual_block(seed=4, hw=28).save(path)
    m = model.Model(path, batch=2, graph=False)
    rng = np.random.default_rng(1)
    m.inputs[0].array[...] = rng.integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    m.run()
    a = m.outputs[0].array.copy()
    m.outputs[0].array[...] = 0
    m.run()   # determinism (reference: test_dl_api.cpp:115-179)
    np.testing.assert_array_equal(m.outputs[0].array, a)
    m.close()


def test_profile_lists_every_module(tmp_path):
    path = str(tmp_path / "net.espdl")
    zoo.inverted_residual_block(seed=4, hw=28).save(path)
    m = model.Model(path, batch=2)
    rows = m.profile()
    # with buffers planned for reuse the residual Add is folded into the project conv's epilogue
    assert [r[1] for r in rows] == ["Conv", "Conv", "Conv"] and all(r[2] > 0 for r in rows)
    m.close()
    m = model.Model(path, batch=2, reuse=False)
    assert [r[1] for r in m.profile()] == ["Conv", "Conv", "Conv", "Add"]
    m.close()


def test_minimize_keeps_inference_working(tmp_path):
    """dl::Model::minimize() (dl_model_base.cpp:431-440 of the reference): the host copies of the device-resident
    parameters go, results stay the same, and a model created afterwards finds the operator registry again."""
    path = str(tmp_path / "net.espdl")
    zoo.mobilenet_v2(seed=9, input_hw=64, num_classes=16).save(path)
    m = model.Model(path, batch=3)
    rng = np.random.default_rng(5)
    m.inputs[0].array[...] = rng.integers(-128, 128, m.inputs[0].array.shape, dtype=np.int8)
    m.run()
    before = m.outputs[0].array.copy()
    m.minimize()
    m.outputs[0].array[...] = 0
    m.run()
    np.testing.assert_array_equal(m.outputs[0].array, before)
    m2 = model.Model(path, batch=3)
    m2.inputs[0].array[...] = m.inputs[0].array
    m2.run()
    np.testing.assert_array_equal(m2.outputs[0].array, before)
    m.close()
    m2.close()


def test_unsupported_operator_fails_to_load(tmp_path):
    g = espdl_file.GraphBuilder("bad", {"target": "c"})
    g.add_input("x", np.int8, [1, 4], -4)
    g.add_output("y", np.int8, [1, 4], -4)
    g.add_node("NoSuchOp", "n0", ["x"], ["y"], quant_type="S8")
    path = str(tmp_path / "bad.espdl")
    g.save(path)
    with pytest.raises(RuntimeError):
        model.Model(path)


def test_block_fusion_pass(tmp_path, monkeypatch):
    """ESPDL_B200_FUSE_BLOCKS=1: expand -> depthwise -> project (-> Add) chains become one FusedBlock module each, the
    tensors between the stages never exist, and the network's output is still the oracle's bit for bit."""
    monkeypatch.setenv("ESPDL_B200_FUSE_BLOCKS", "1")
    path = str(tmp_path / "block.espdl")
    zoo.inverted_residual_block(seed=4, hw=28).save(path)
    m = model.Model(path, batch=2)
    assert [r[1] for r in m.profile()] == ["FusedBlock"]
    m.close()
    m, want = run_and_compare(tmp_path, zoo.inverted_residual_block(seed=4, hw=56), batch=3, seed=42, check_intermediates=False)
    m.close()
    # MobileNetV2: the blocks whose input channels are a multiple of 16 are fused (14 of 17), the others stay as they were
    m, want = run_and_compare(tmp_path, zoo.mobilenet_v2(seed=5), batch=2, seed=50, check_intermediates=False)
    kinds = [r[1] for r in m.profile()]
    assert kinds.count("FusedBlock") >= 12, kinds
    first = m.outputs[0].array.copy()
    m.run()
    np.testing.assert_array_equal(m.outputs[0].array, first)
    m.close()


@pytest.mark.parametrize("target", ["esp32p4", "esp32s3"])
def test_streaming_model_equals_the_whole_sequence_model(target, monkeypatch):
    """The reference's own check of its streaming tutorial (examples/tutorial/how_to_deploy_streaming_model/
    test_streaming_model/main/app_main.cpp:8-72): the model with StreamingCache nodes, fed the sequence three frames at a
    time, ends on the output the whole-sequence model gives; after reset() it does so again."""
    monkeypatch.setenv("ESPDL_B200_TARGET", target)
    whole = model.Model(os.path.join(GOLDEN, f"{target}__streaming_tcn.espdl"))
    chunked = model.Model(os.path.join(GOLDEN, f"{target}__streaming_tcn_chunked.espdl"))
    frames, step = whole.inputs[0].shape[1], chunked.inputs[0].shape[1]
    assert frames % step == 0 and chunked.inputs[0].shape[2:] == whole.inputs[0].shape[2:]
    for seed in (1, 2):
        x = np.random.default_rng(seed).integers(-128, 128, size=whole.inputs[0].shape, dtype=np.int8)
        whole.inputs[0].array[...] = x
        whole.run()
        for k in range(frames // step):
            chunked.inputs[0].array[...] = x[:, k * step:(k + 1) * step]
            chunked.run()
        np.testing.assert_array_equal(np.asarray(chunked.outputs[0].array), np.asarray(whole.outputs[0].array))
        assert np.asarray(whole.outputs[0].array).astype(np.float32).std() > 0
        chunked.reset()
    whole.close()
    chunked.close()


@pytest.mark.parametrize("dt,qt,sa,sb", [(np.int16, "S16", (1, 40, 80), (80, 520)), (np.int16, "S16", (3, 24, 64), (64, 48)),
                                         (np.int8, "S8", (1, 40, 160), (160, 80))])
def test_matmul_with_a_constant_operand(tmp_path, dt, qt, sa, sb):
    """MatMul whose second operand is a parameter of the file (the recognition head of a text model): the module uploads
    it and, for int16, sizes the tile kernel's byte-plane scratch from its own shapes."""
    e_a, e_b, e_out = (-12, -14, -9) if dt == np.int16 else (-5, -6, -3)
    rng = np.random.default_rng(12)
    info = np.iinfo(dt)
    w = rng.integers(info.min // 8, info.max // 8, size=sb, dtype=dt)
    g = espdl_file.GraphBuilder("matmul_const", metadata={"target": "c"})
    g.add_input("a", dt, list(sa), e_a)
    g.add_initializer("w", w, [e_b])
    g.add_node("MatMul", "mm", ["a", "w"], ["y"], quant_type=qt, activation="Linear")
    so = list(sa[:-1]) + [sb[-1]]
    g.add_output("y", dt, so, e_out)
    path = str(tmp_path / "mmc.espdl")
    g.save(path)
    m = model.Model(path)
    a = rng.integers(info.min // 8, info.max // 8, size=sa, dtype=dt)
    m.inputs[0].array[...] = a
    m.run()
    dtype = abi.DTYPE_INT16 if dt == np.int16 else abi.DTYPE_INT8
    want = graph_oracle.matmul(__import__("checkers").oracle(), a, w, e_a, e_b, e_out, dtype, abi.ACT_LINEAR, abi.ROUND_HALF_UP)
    np.testing.assert_array_equal(np.asarray(m.outputs[0].array).reshape(so), want.reshape(so))
    assert want.std() > 0
    m.close()


def _conv_node(g, rng, name, x, out, cin, cout, k, e_in, e_out, bias):
    """A Conv node with stride 1 and no padding, random per-channel weights; returns the output's (h, w) shrink."""
    ew = rng.integers(-8, -5, size=cout)
    w = rng.integers(-20, 21, size=(cout, k, k, cin)).astype(np.int8)      # payload order of target "c"
    g.add_initializer(name + ".weight", w.reshape(k, k, cin, cout), list(ew))
    inputs = [x, name + ".weight"]
    if bias:
        g.add_initializer(name + ".bias", rng.integers(-2000, 2000, size=cout).astype(np.int32), list(ew + e_in))
        inputs.append(name + ".bias")
    g.add_node("Conv", name, inputs, [out], activation="Linear", dilations=[1, 1], group=1, kernel_shape=[k, k], pads=[0, 0, 0, 0],
               quant_type="S8", strides=[1, 1])


@pytest.mark.parametrize("fold", ["1", "0"])
@pytest.mark.parametrize("kind", ["pointwise_without_bias", "valid_3x3"])
def test_add_behind_a_conv_that_cannot_or_need_not_take_it(tmp_path, monkeypatch, kind, fold):
    """The Add-folding pass may only touch pointwise convs, and a conv without a bias (which the reference allows,
    dl_module_conv.hpp:137-140) must not mistake the appended residual for its bias.  With the pass on and off the
    output equals the oracle's."""
    monkeypatch.setenv("ESPDL_B200_FOLD_ADD", fold)
    rng = np.random.default_rng(17)
    g = espdl_file.GraphBuilder("fold", metadata={"target": "c"})
    e = -5
    if kind == "pointwise_without_bias":
        g.add_input("x", np.int8, [1, 12, 12, 32], e)
        _conv_node(g, rng, "pw", "x", "y", 32, 32, 1, e, e, bias=False)
        g.add_value_info("y", np.int8, [1, 12, 12, 32], e)
        g.add_node("Add", "add", ["y", "x"], ["out"], quant_type="S8")
        g.add_output("out", np.int8, [1, 12, 12, 32], e)
    else:
        g.add_input("x", np.int8, [1, 12, 12, 16], e)
        _conv_node(g, rng, "c0", "x", "z", 16, 16, 3, e, e, bias=True)
        g.add_value_info("z", np.int8, [1, 10, 10, 16], e)
        _conv_node(g, rng, "c1", "x", "y", 16, 16, 3, e, e, bias=True)
        g.add_value_info("y", np.int8, [1, 10, 10, 16], e)
        g.add_node("Add", "add", ["y", "z"], ["out"], quant_type="S8")
        g.add_output("out", np.int8, [1, 10, 10, 16], e)
    m, want = run_and_compare(tmp_path, g, batch=3, seed=18, check_intermediates=False)
    kinds = [r[1] for r in m.profile()]
    if kind == "pointwise_without_bias" and fold == "1":
        assert kinds == ["Conv"], kinds                  # folded, and still right
    else:
        assert kinds.count("Add") == 1, kinds            # a 3x3 conv keeps its Add
    assert want[m.outputs[0].name].std() > 3
    m.close()


def _full_size_parity(path, batch, picks, small_batch, windows, seed):
    """A model at its benchmarked batch: the oracle runs on the picked images, and every row of the windows must equal
    the row a small-batch model gives for the same image (images are independent units)."""
    parsed = espdl_file.read(path)
    m = model.Model(path, batch=batch)
    rng = np.random.default_rng(seed)
    x = rng.integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
    x[picks[1]] = x[picks[-2]]                     # two equal images far apart must give equal rows
    m.inputs[0].array[...] = x
    m.run()
    got = {o.name: np.array(o.array, copy=True) for o in m.outputs}
    m.run()                                        # a second pass over the planned arena gives the same bytes
    for o in m.outputs:
        np.testing.assert_array_equal(o.array, got[o.name])
    m.close()
    want = graph_oracle.run_graph(parsed, {parsed["inputs"][0]["name"]: np.ascontiguousarray(x[picks])})
    for name, g in got.items():
        np.testing.assert_array_equal(g[picks].reshape(want[name].shape), want[name])
        np.testing.assert_array_equal(g[picks[1]], g[picks[-2]])
        assert want[name].astype(np.float32).std() > 3
    ms = model.Model(path, batch=small_batch)
    for start in windows:
        ms.inputs[0].array[...] = x[start:start + small_batch]
        ms.run()
        for o in ms.outputs:
            np.testing.assert_array_equal(o.array, got[o.name][start:start + small_batch])
    ms.close()


def test_mobilenet_v2_at_the_benchmarked_batch(tmp_path):
    """MobileNetV2-1.0 at batch 1024, the size bench.py times: different tile counts, persistent-loop trip counts and
    arena offsets than the batch-2 comparison.  Eight images from all over the batch (first, last, both sides of the
    128-row tile boundaries of the late 7x7 layers) are checked against the graph oracle, windows of eight against a
    batch-8 model."""
    path = str(tmp_path / "mbv2.espdl")
    zoo.mobilenet_v2(seed=5).save(path)
    _full_size_parity(path, batch=1024, picks=[0, 1, 2, 3, 511, 512, 1022, 1023], small_batch=8, windows=(8, 504, 1016), seed=51)


TOPOLOGY_640 = os.path.join(os.path.dirname(GOLDEN), "yolo11n_640_topology.json")


def test_yolo11n_640_at_the_benchmarked_batch(tmp_path):
    """The 249-node YOLO11n graph the reference ships for 640x640 (topology from its model file, seeded random weights) at
    batch 512: four images through the graph oracle, windows of two against a batch-2 model, all six heads."""
    path = str(tmp_path / "yolo640.espdl")
    zoo.yolo11n_640(TOPOLOGY_640, seed=6).save(path)
    _full_size_parity(path, batch=512, picks=[0, 255, 510, 511], small_batch=2, windows=(2, 300), seed=62)


def test_lut_folding_pass(tmp_path, monkeypatch):
    """Swish tables behind dense convs whose input channels are a multiple of 16 are applied in the conv's epilogue (table
    in shared memory): the nodes leave the plan, the outputs stay the oracle's, with the pass on and off."""
    g = zoo.yolo11n_style(seed=6, input_hw=96)
    m, want = run_and_compare(tmp_path, g, batch=2, seed=63, check_intermediates=False)
    folded = [r[1] for r in m.profile()]
    first = {o.name: np.array(o.array, copy=True) for o in m.outputs}
    m.close()
    monkeypatch.setenv("ESPDL_B200_FOLD_LUT", "0")
    m, _ = run_and_compare(tmp_path, g, batch=2, seed=63, check_intermediates=False)
    plain = [r[1] for r in m.profile()]
    for o in m.outputs:
        np.testing.assert_array_equal(o.array, first[o.name])
    m.close()
    assert plain.count("Swish") >= 50 and folded.count("Swish") <= plain.count("Swish") - 45, (plain.count("Swish"), folded.count("Swish"))
    assert len(folded) == len(plain) - (plain.count("Swish") - folded.count("Swish"))


def test_concat_and_split_as_channel_slices(tmp_path, monkeypatch):
    """The planner places Concat inputs inside the Concat's output and makes Split outputs windows into the Split's input
    wherever the producers / readers take a row stride: fewer bytes move, every tensor still equals the oracle's, and the
    outputs equal those of the plan with the pass switched off."""
    g = zoo.yolo11n_style(seed=6, input_hw=96)
    m, want = run_and_compare(tmp_path, g, batch=2, seed=64, check_intermediates=True)
    assert m.num_slice_views() >= 8, m.num_slice_views()
    m.close()
    m, _ = run_and_compare(tmp_path, g, batch=2, seed=64, check_intermediates=False)   # planned arena + CUDA graph
    views = m.num_slice_views()
    first = {o.name: np.array(o.array, copy=True) for o in m.outputs}
    m.run()
    for o in m.outputs:
        np.testing.assert_array_equal(o.array, first[o.name])
    m.close()
    monkeypatch.setenv("ESPDL_B200_SLICE_VIEWS", "0")
    m, _ = run_and_compare(tmp_path, g, batch=2, seed=64, check_intermediates=False)
    assert m.num_slice_views() == 0 and views >= 8
    for o in m.outputs:
        np.testing.assert_array_equal(o.array, first[o.name])
    m.close()


def test_prelu_folding_pass(monkeypatch):
    """The MNP face detector: eight Conv -> PRelu pairs (first layer, pointwise and depthwise convs).  Every PRelu becomes
    per-channel tables of its conv (espdl_conv_desc.lut_channel_stride): 15 launches instead of 23, same bytes as the graph
    oracle and as the plan with the pass switched off."""
    path = os.path.join(GOLDEN, "esp32p4__zoo_face_mnp.espdl")
    if not os.path.exists(path):
        pytest.skip("fixture not present")
    monkeypatch.setenv("ESPDL_B200_TARGET", "esp32p4")
    parsed = espdl_file.read(path)
    x = None
    outs = {}
    for fold in ("1", "0"):
        monkeypatch.setenv("ESPDL_B200_FOLD_PRELU", fold)
        m = model.Model(path)
        if x is None:
            x = np.random.default_rng(4).integers(-128, 128, size=m.inputs[0].shape, dtype=np.int8)
        m.inputs[0].array[...] = x
        m.run()
        kinds = [r[1] for r in m.profile()]
        outs[fold] = ({o.name: np.array(o.array, copy=True) for o in m.outputs}, kinds)
        m.close()
    assert outs["0"][1].count("PRelu") == 8 and outs["1"][1].count("PRelu") == 0
    assert len(outs["1"][1]) == len(outs["0"][1]) - 8
    want = graph_oracle.run_graph(parsed, {parsed["inputs"][0]["name"]: x}, round_mode=abi.ROUND_HALF_EVEN, target="esp32p4")
    for name, got in outs["1"][0].items():
        np.testing.assert_array_equal(got.reshape(want[name].shape), want[name])
        np.testing.assert_array_equal(got, outs["0"][0][name])
        assert want[name].astype(np.float32).std() > 0
