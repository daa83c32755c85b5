"""CPU tests of the host layer: the C++ `.espdl` reader against the Python reader/writer on the reference's shipped
golden files and on generated networks, and the lifetime-based arena planner."""
import ctypes as C
import glob
import os

import numpy as np
import pytest

from espdl_b200 import espdl_file, model, zoo

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "espdl")


@pytest.fixture(scope="module")
def host():
    if not os.path.exists(model.HOST_LIB_PATH):
        from espdl_b200 import build
        build.build()
    L = model.host_lib()
    L.espdl_fbs_describe.restype = C.c_char_p
    L.espdl_fbs_describe.argtypes = [C.c_char_p]
    L.espdl_plan_arena.restype = C.c_size_t
    L.espdl_plan_arena.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.POINTER(C.c_int),
                                   C.POINTER(C.c_size_t), C.c_int]
    return L


def describe(host, path):
    text = host.espdl_fbs_describe(os.fsencode(path))
    assert text is not None, path
    nodes, params = [], {}
    for line in text.decode().splitlines():
        f = line.split("\t")
        if f[0] == "node":
            nodes.append(f)
        elif f[0] == "param":
            params[f[1]] = f
    return nodes, params


@pytest.mark.parametrize("path", sorted(glob.glob(os.path.join(GOLDEN, "*.espdl"))), ids=os.path.basename)
def test_cpp_reader_matches_python_reader_on_shipped_models(host, path):
    m = espdl_file.read(path)
    nodes, params = describe(host, path)
    assert [n[2] for n in nodes] == [n["name"] for n in m["nodes"]]        # exported order is already topological
    assert [n[1] for n in nodes] == [n["op_type"] for n in m["nodes"]]
    for n, ref in zip(nodes, m["nodes"]):
        assert n[3].rstrip(",").split(",") == ref["inputs"]
    for name, f in params.items():
        t = m["initializers"][name]
        assert int(f[2]) == t["data_type"]
        assert f[3] == "[" + ", ".join(str(d) for d in (t["dims"] or [1])) + "]"
        assert int(f[4]) == max(1, len(t["exponents"]))
        assert int(f[5]) == int(np.ascontiguousarray(t["data"]).reshape(-1).view(np.uint8).astype(np.int64).sum())


def test_cpp_reader_reads_generated_network(host, tmp_path):
    g = zoo.mobilenet_v2(seed=5)
    path = tmp_path / "mbv2.espdl"
    g.save(path)
    m = espdl_file.read(str(path))
    nodes, params = describe(host, str(path))
    assert len(nodes) == len(m["nodes"]) and len(nodes) >= 66
    ops = [n[1] for n in nodes]
    assert ops.count("Conv") == 52 and ops.count("Add") == 10 and ops.count("Gemm") == 1 and ops.count("GlobalAveragePool") == 1
    first = nodes[0]
    assert "pads=[1, 1, 1, 1]" in first and "activation=Relu" in first
    assert first[4].startswith("features.0_out,[1, 112, 112, 32],")
    for name, f in params.items():
        t = m["initializers"][name]
        assert int(f[5]) == int(np.ascontiguousarray(t["data"]).reshape(-1).view(np.uint8).astype(np.int64).sum())
    assert int(params["features.0.weight"][4]) == 32   # per-channel exponents


def test_corrupt_and_missing_files_are_rejected(host, tmp_path):
    assert host.espdl_fbs_describe(os.fsencode(tmp_path / "missing.espdl")) is None
    bad = tmp_path / "bad.espdl"
    bad.write_bytes(b"XXXX" + bytes(64))
    assert host.espdl_fbs_describe(os.fsencode(bad)) is None
    enc = tmp_path / "enc.espdl"
    enc.write_bytes(b"EDL2" + np.array([1, 64, 0], dtype=np.uint32).tobytes() + bytes(64))  # mode 1 = encrypted
    assert host.espdl_fbs_describe(os.fsencode(enc)) is None                                  # no key given


def _golden_model():
    here = os.path.dirname(os.path.abspath(__file__))
    return os.path.join(here, "golden", "espdl", "c__linear_ishap_1_64_kshap_32_64_relu_s8.espdl")


def test_encrypted_model_loads_with_its_key(host, tmp_path):
    """EDL2 with mode 1: the FlatBuffer is AES-128-CTR encrypted, counter block 10..1F (fbs_loader.cpp:86-124).  The
    file is produced here with an independent AES implementation."""
    from cryptography.hazmat.primitives.ciphers import Cipher, algorithms, modes
    host.espdl_fbs_describe_key.restype = C.c_char_p
    host.espdl_fbs_describe_key.argtypes = [C.c_char_p, C.c_char_p]
    plain = open(_golden_model(), "rb").read()
    assert plain[:4] == b"EDL2"
    mode, size = np.frombuffer(plain[4:12], dtype=np.uint32)
    assert mode == 0
    key = bytes(range(0x40, 0x50))
    enc = Cipher(algorithms.AES(key), modes.CTR(bytes(range(0x10, 0x20)))).encryptor()
    body = enc.update(plain[16:16 + int(size)]) + enc.finalize()
    path = tmp_path / "secret.espdl"
    path.write_bytes(b"EDL2" + np.array([1, size, 0], dtype=np.uint32).tobytes() + body)
    want = host.espdl_fbs_describe(os.fsencode(_golden_model()))
    assert want is not None
    want = bytes(want)
    assert host.espdl_fbs_describe(os.fsencode(path)) is None
    got = host.espdl_fbs_describe_key(os.fsencode(path), key)
    assert got is not None and bytes(got) == want
    wrong = host.espdl_fbs_describe_key(os.fsencode(path), bytes(16))
    assert wrong is None or bytes(wrong) != want


def test_pdl3_package_digest(host, tmp_path):
    """PDL3: magic, version[16], package_size, sha256[32], model count, (data offset, name offset, name length) per
    model (fbs_loader.hpp:13-97); the digest covers [0, package_size) with its own field zeroed."""
    import hashlib
    host.espdl_fbs_verify_package.restype = C.c_int
    host.espdl_fbs_verify_package.argtypes = [C.c_char_p, C.c_char_p, C.POINTER(C.c_uint)]
    model = open(_golden_model(), "rb").read()
    name = b"linear"
    header = 60 + 12
    name_off = header
    data_off = (name_off + len(name) + 15) // 16 * 16
    total = data_off + len(model)
    pkg = bytearray(total + 32)                                  # trailing bytes outside package_size are not hashed
    pkg[0:4] = b"PDL3"
    pkg[4:4 + 6] = b"1.2.3\0"
    pkg[20:24] = np.uint32(total).tobytes()
    pkg[56:60] = np.uint32(1).tobytes()
    pkg[60:72] = np.array([data_off, name_off, len(name)], dtype=np.uint32).tobytes()
    pkg[name_off:name_off + len(name)] = name
    pkg[data_off:data_off + len(model)] = model
    digest = hashlib.sha256(bytes(pkg[:24]) + bytes(32) + bytes(pkg[56:total])).digest()
    pkg[24:56] = digest
    path = tmp_path / "pack.espdl"
    path.write_bytes(bytes(pkg))
    version = C.create_string_buffer(16)
    size = C.c_uint(0)
    assert host.espdl_fbs_verify_package(os.fsencode(path), version, C.byref(size)) == 1
    assert version.value == b"1.2.3" and size.value == total
    assert bytes(host.espdl_fbs_describe(os.fsencode(path))) == bytes(host.espdl_fbs_describe(os.fsencode(_golden_model())))
    pkg[data_off + 40] ^= 1                                      # one flipped bit inside the package
    path.write_bytes(bytes(pkg))
    assert host.espdl_fbs_verify_package(os.fsencode(path), None, None) == 0
    assert host.espdl_fbs_verify_package(os.fsencode(_golden_model()), None, None) == -1   # not a PDL3 package


def plan(host, first, last, nbytes, alias=None, reuse=1):
    n = len(first)
    alias = alias or [-1] * n
    off = (C.c_size_t * n)()
    arena = host.espdl_plan_arena(n, (C.c_int * n)(*first), (C.c_int * n)(*last), (C.c_size_t * n)(*nbytes), (C.c_int * n)(*alias), off, reuse)
    return arena, list(off)


def test_arena_planner_reuses_dead_buffers_and_never_overlaps_live_ones(host):
    rng = np.random.default_rng(0)
    n = 60
    first = sorted(int(v) for v in rng.integers(-1, 40, size=n))
    last = [f + int(rng.integers(1, 6)) for f in first]
    nbytes = [int(v) for v in rng.integers(1, 5000, size=n)]
    arena, off = plan(host, first, last, nbytes)
    for i in range(n):
        assert off[i] % 256 == 0 and off[i] + nbytes[i] <= arena
        for j in range(i):
            overlap_time = first[i] <= last[j] and first[j] <= last[i]
            overlap_mem = off[i] < off[j] + nbytes[j] and off[j] < off[i] + nbytes[i]
            assert not (overlap_time and overlap_mem), (i, j)
    no_reuse, _ = plan(host, first, last, nbytes, reuse=0)
    assert arena < no_reuse


def test_arena_planner_aliases_share_the_root_buffer(host):
    # t1 is an in-place result of t0, t2 a view of t1: one buffer, alive until t2's last reader
    arena, off = plan(host, [0, 1, 2, 3], [1, 2, 5, 4], [1000, 1000, 1000, 512], alias=[-1, 0, 1, -1])
    assert off[0] == off[1] == off[2]
    assert not (off[3] < off[0] + 1000 and off[0] < off[3] + 512)
    assert arena == 1024 + 512


def test_arena_planner_places_channel_slices_inside_their_wide_tensor(host):
    """Three slices of a Concat output (tensor 0, produced at step 6) are written at steps 1, 3 and 5: the wide buffer is
    alive from step 1 on, the slices sit at their channel offsets inside it and add nothing to its size, and a tensor that
    lives meanwhile does not share its bytes; a tensor that is dead before step 1 may."""
    host.espdl_plan_arena_slices.restype = C.c_size_t
    host.espdl_plan_arena_slices.argtypes = [C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.POINTER(C.c_int),
                                             C.POINTER(C.c_size_t), C.POINTER(C.c_int), C.POINTER(C.c_size_t), C.c_int]
    first = [6, 1, 3, 5, 2, -1, 0]
    last = [8, 6, 6, 6, 4, 0, 0]
    nbytes = [4800, 1600, 1600, 1600, 7000, 3000, 512]
    alias = [-1, 0, 0, 0, -1, -1, -1]
    view = [0, 0, 16, 32, 0, 0, 0]
    stride = [0, 48, 48, 48, 0, 0, 0]
    n = len(first)
    off = (C.c_size_t * n)()
    arena = host.espdl_plan_arena_slices(n, (C.c_int * n)(*first), (C.c_int * n)(*last), (C.c_size_t * n)(*nbytes), (C.c_int * n)(*alias),
                                         (C.c_size_t * n)(*view), (C.c_int * n)(*stride), off, 1)
    off = list(off)
    assert [off[1] - off[0], off[2] - off[0], off[3] - off[0]] == [0, 16, 32]
    wide = (off[0], off[0] + 4800)
    assert off[4] >= wide[1] or off[4] + 7000 <= wide[0]           # alive during steps 2..4, while the slices are written
    assert off[5] + 3000 <= arena and arena <= 4864 + 7168 + 3072 + 512


def test_python_writer_round_trip():
    g = zoo.inverted_residual_block(seed=4, hw=16)
    m = espdl_file.read(g.serialize())
    assert [n["op_type"] for n in m["nodes"]] == ["Conv", "Conv", "Conv", "Add"]
    assert m["nodes"][1]["attrs"]["group"] == 192 and m["initializers"]["dw.weight"]["dims"] == [3, 3, 192, 1]
    assert m["metadata"]["target"] == "c"


def registered_ops(host):
    host.espdl_registered_ops.restype = C.c_char_p
    return set(host.espdl_registered_ops().decode().split())


def test_every_operator_of_the_shipped_fixtures_has_a_creator(host):
    """The creator registry (dl::module::ModuleCreator) knows every operator type that occurs in the committed model files."""
    ops = registered_ops(host)
    for path in sorted(glob.glob(os.path.join(GOLDEN, "*.espdl"))):
        used = {n["op_type"] for n in espdl_file.read(path)["nodes"]}
        assert used <= ops, (os.path.basename(path), sorted(used - ops))


def test_registry_covers_the_reference_creator_list(host):
    """Operator types of the reference's own registry (esp-dl/dl/module/include/dl_module_creator.hpp:134-204).  Those
    without a creator here would be listed explicitly (none at present), so that a regression or a new operator shows up in this test."""
    reference = """Conv Add Sub Mul Div Pow Mod Resize GlobalAveragePool AveragePool Concat Sigmoid Tanh Relu LeakyRelu HardSigmoid
        HardSwish Gelu LUT Gemm QuantizeLinear DequantizeLinear RequantizeLinear PRelu Clip Flatten Reshape Transpose Exp Log Sqrt Squeeze
        Unsqueeze Softmax LogSoftmax MaxPool Slice Pad MatMul Neg SpaceToDepth Split Gather Elu Greater GreaterOrEqual Equal Less
        LessOrEqual ReverseSequence ScatterND Identity Swish ReduceL1 ReduceL2 ReduceMin ReduceMax ReduceSum ReduceProd ReduceMean
        ReduceSumSquare ReduceLogSum ReduceLogSumExp GRU LSTM DepthToSpace StreamingCache InsertZeros LayerNormalization LpNormalization
        RMSNormalization""".split()
    missing = set()
    assert set(reference) - registered_ops(host) == missing


def test_truncated_and_damaged_files_are_refused_not_read_out_of_bounds(host, tmp_path):
    """Every offset and length of the FlatBuffer is checked when a model is loaded: a file cut short at any point either
    fails to load or (when the cut lies past everything the reader uses) loads like the whole file; a file with flipped
    bytes either fails to load or describes without touching memory outside its buffer.  The child process would die on
    an out-of-bounds read of the freed tail (the loader's copy is exactly as long as the payload)."""
    import subprocess
    import sys
    good = open(_golden_model(), "rb").read()
    want = host.espdl_fbs_describe(os.fsencode(_golden_model()))
    assert want
    want = bytes(want)
    cuts = sorted(set([0, 3, 4, 15, 16, 17, 40, 100, 500] + [len(good) * k // 23 for k in range(1, 23)] + [len(good) - 1]))
    refused = 0
    for n in cuts:
        path = tmp_path / f"cut_{n}.espdl"
        path.write_bytes(good[:n])
        got = host.espdl_fbs_describe(os.fsencode(path))
        if got is None:
            refused += 1
        else:
            assert bytes(got) == want
    assert refused == len(cuts)  # the header's size field no longer fits the file: every cut is refused
    # the same cuts with the header's size field patched to the shortened payload: now the FlatBuffer itself is short
    refused = 0
    for n in [c for c in cuts if c > 64]:
        blob = bytearray(good[:n])
        blob[8:12] = (n - 16).to_bytes(4, "little")
        path = tmp_path / f"short_{n}.espdl"
        path.write_bytes(bytes(blob))
        got = host.espdl_fbs_describe(os.fsencode(path))
        refused += got is None
        if got is not None:
            assert bytes(got) == want
    assert refused >= 10
    # flipped bytes, in a child process per batch so that a crash would be seen as a failure of this test
    rng = np.random.default_rng(7)
    files = []
    for k in range(60):
        blob = bytearray(good)
        for _ in range(1 + k % 4):
            pos = int(rng.integers(16, len(blob)))
            blob[pos] ^= int(rng.integers(1, 256))
        path = tmp_path / f"flip_{k}.espdl"
        path.write_bytes(bytes(blob))
        files.append(str(path))
    code = ("import ctypes as C, os, sys\n"
            f"L = C.CDLL({model.HOST_LIB_PATH!r})\n"
            "L.espdl_fbs_describe.restype = C.c_char_p\nL.espdl_fbs_describe.argtypes = [C.c_char_p]\n"
            "n = sum(L.espdl_fbs_describe(os.fsencode(p)) is not None for p in sys.argv[1:])\nprint(n)\n")
    r = subprocess.run([sys.executable, "-c", code] + files, capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    assert 0 <= int(r.stdout.strip().splitlines()[-1]) <= len(files)


def test_pdl_package_table_is_checked_against_the_file(host, tmp_path):
    """A PDL package whose model table points outside the file is refused (names and data offsets are checked)."""
    good = open(_golden_model(), "rb").read()
    name = b"m0"
    header = b"PDL2" + (1).to_bytes(4, "little")
    table_at = len(header)
    data_off = table_at + 12 + len(name)
    data_off += (-data_off) % 16
    entry = data_off.to_bytes(4, "little") + (table_at + 12).to_bytes(4, "little") + len(name).to_bytes(4, "little")
    blob = header + entry + name
    blob += b"\0" * (data_off - len(blob)) + good
    ok = tmp_path / "ok.espdl"
    ok.write_bytes(blob)
    assert host.espdl_fbs_describe(os.fsencode(ok)) is not None
    for field, value in ((0, len(blob) + 100), (4, len(blob) - 1), (8, 1 << 20)):
        bad = bytearray(blob)
        bad[table_at + field:table_at + field + 4] = value.to_bytes(4, "little")
        path = tmp_path / f"bad_{field}.espdl"
        path.write_bytes(bytes(bad))
        assert host.espdl_fbs_describe(os.fsencode(path)) is None
    count = bytearray(blob)
    count[4:8] = (1 << 28).to_bytes(4, "little")
    path = tmp_path / "bad_count.espdl"
    path.write_bytes(bytes(count))
    assert host.espdl_fbs_describe(os.fsencode(path)) is None


def _plan(host, path, batch=0, reuse=1):
    host.espdl_model_plan.restype = C.c_int
    host.espdl_model_plan.argtypes = [C.c_char_p, C.c_int, C.c_int, C.POINTER(C.c_size_t), C.POINTER(C.c_int), C.c_char_p, C.c_size_t]
    arena, slices = C.c_size_t(), C.c_int()
    text = C.create_string_buffer(1 << 16)
    n = host.espdl_model_plan(os.fsencode(path), batch, reuse, C.byref(arena), C.byref(slices), text, len(text))
    assert n > 0, n
    rows = [line.split("\t") for line in text.value.decode().splitlines()]
    return n, arena.value, slices.value, {r[0]: (r[1], int(r[2]), int(r[3])) for r in rows}


def test_planner_places_concat_inputs_and_split_outputs_as_channel_slices(host, tmp_path, monkeypatch):
    """The arena plan of the detector-shaped graph, made without a device: tensors that feed a Concat along the channel axis
    from a producer that can write strided rows live inside the Concat's output, Split outputs whose readers can read such
    rows are windows into the Split's input; slices start and stride on 32-byte boundaries; the plan with the pass switched
    off has none and needs more memory."""
    g = zoo.yolo11n_style(seed=6, input_hw=96)
    path = str(tmp_path / "det.espdl")
    g.save(path)
    parsed = espdl_file.read(path)
    n, arena, slices, views = _plan(host, path, batch=2)
    assert slices == len(views) >= 8
    producer = {o: nd for nd in parsed["nodes"] for o in nd["outputs"]}
    consumers = {}
    for nd in parsed["nodes"]:
        for i in nd["inputs"]:
            consumers.setdefault(i, []).append(nd)
    for name, (wide, offset, stride) in views.items():
        assert offset % 32 == 0 and stride % 32 == 0
        into_concat = producer.get(wide, {}).get("op_type") == "Concat" and name in producer[wide]["inputs"]
        from_split = producer.get(name, {}).get("op_type") == "Split" and producer[name]["inputs"][0] == wide
        assert into_concat or from_split, (name, wide)
        # the table lookups that were folded into their convs are gone from the plan: what reads or writes a slice takes a row stride
        for c in consumers.get(name, []):
            assert c["op_type"] in ("Conv", "Concat", "Add", "RequantizeLinear", "Swish", "Mul"), (name, c["op_type"])
    monkeypatch.setenv("ESPDL_B200_SLICE_VIEWS", "0")
    n0, arena0, slices0, _ = _plan(host, path, batch=2)
    assert n0 == n and slices0 == 0 and arena0 > arena


def test_planner_leaves_ragged_concats_alone(host):
    """The face detector concatenates 48 + 24 + 24 channels: 24-byte parts are no whole 32-byte units, nothing becomes a slice."""
    path = os.path.join(GOLDEN, "esp32p4__zoo_face_msr.espdl")
    if not os.path.exists(path):
        pytest.skip("fixture not present")
    n, arena, slices, views = _plan(host, path)
    assert n > 40 and slices == 0 and arena > 0
