"""Detection post-processing: the device candidate scan plus the host decode / sort / NMS of dl::detect::yolo11PostProcessor
against the oracle's sequential restatement of the reference, on the three heads of the generated detector and on
synthetic head tensors.  The reference ships no vectors for this step; the restatement is pinned against the
reference's own post-processor classes compiled for the host (oracle/_ref: dl_detect_postprocessor.cpp and
dl_detect_yolo11_postprocessor.cpp, unmodified, behind stand-ins for dl::Model and dl::image::ImagePreprocessor)."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi


class Stage(C.Structure):
    _fields_ = [("score", C.c_void_p), ("box", C.c_void_p), ("h", C.c_int), ("w", C.c_int), ("classes", C.c_int),
                ("score_exponent", C.c_int), ("box_exponent", C.c_int), ("stride_y", C.c_int), ("stride_x", C.c_int),
                ("offset_y", C.c_int), ("offset_x", C.c_int)]


def oracle_detect(heads, score_thr, nms_thr, top_k, width, height, max_results=300):
    """heads: [(score [h][w][classes] int8, box [h][w][64] int8, e_score, e_box, stride)] of ONE image."""
    L = checkers.oracle()
    L.oracle_yolo11_postprocess.restype = C.c_int
    L.oracle_yolo11_postprocess.argtypes = [C.POINTER(Stage), C.c_int, C.c_float, C.c_float, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int,
                                            C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float)]
    st = (Stage * len(heads))()
    keep = []
    for i, (s, b, es, eb, stride) in enumerate(heads):
        s, b = np.ascontiguousarray(s), np.ascontiguousarray(b)
        keep += [s, b]
        st[i] = Stage(s.ctypes.data, b.ctypes.data, s.shape[0], s.shape[1], s.shape[2], es, eb, stride, stride, stride // 2, stride // 2)
    boxes, scores = (C.c_int * (5 * max_results))(), (C.c_float * max_results)()
    n = L.oracle_yolo11_postprocess(st, len(heads), score_thr, nms_thr, top_k, 1.0, 1.0, 0, 0, width, height, 0, max_results, boxes, scores)
    return [(boxes[5 * i], scores[i], tuple(boxes[5 * i + 1:5 * i + 5])) for i in range(n)]


def reference_detect(heads, score_thr, nms_thr, top_k, width, height, inv_scale=(1.0, 1.0), border=(0, 0), max_results=300):
    """The same call on the reference's own yolo11PostProcessor (oracle/_ref)."""
    R = checkers.ref()
    R.ref_yolo11_postprocess.restype = C.c_int
    R.ref_yolo11_postprocess.argtypes = [C.POINTER(Stage), C.c_int, C.c_float, C.c_float, C.c_int, C.c_float, C.c_float, C.c_int, C.c_int,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float)]
    st = (Stage * len(heads))()
    keep = []
    for i, (s, b, es, eb, stride) in enumerate(heads):
        s, b = np.ascontiguousarray(s), np.ascontiguousarray(b)
        keep += [s, b]
        st[i] = Stage(s.ctypes.data, b.ctypes.data, s.shape[0], s.shape[1], s.shape[2], es, eb, stride, stride, stride // 2, stride // 2)
    boxes, scores = (C.c_int * (5 * max_results))(), (C.c_float * max_results)()
    n = R.ref_yolo11_postprocess(st, len(heads), score_thr, nms_thr, top_k, inv_scale[0], inv_scale[1], border[0], border[1], width, height,
                                 0, max_results, boxes, scores)
    assert n >= 0
    return [(boxes[5 * i], scores[i], tuple(boxes[5 * i + 1:5 * i + 5])) for i in range(n)]


@pytest.mark.skipif(not checkers.have_ref(), reason="oracle/_ref/libespdl_ref.so not built")
@pytest.mark.parametrize("seed,score_thr,nms_thr,top_k,hot", [(1, 0.5, 0.5, 100, 60), (2, 0.25, 0.7, 20, 200), (3, 0.6, 0.3, 5, 40), (4, 0.9, 0.45, 300, 400)])
def test_oracle_post_processor_equals_the_reference(seed, score_thr, nms_thr, top_k, hot):
    """Random heads of three strides with a few hundred scores above the threshold, overlapping boxes, equal scores
    (the stable order of the sorted list matters) and boxes that leave the image: the restatement returns the
    reference's list - categories, float scores bit for bit, boxes - for several thresholds and top-k limits."""
    rng = np.random.default_rng(seed)
    heads = []
    for stride, hw in ((8, 20), (16, 10), (32, 5)):
        score = rng.integers(-128, -40, size=(hw, hw, 7), dtype=np.int8)
        idx = rng.integers(0, score.size, size=hot // 3)
        score.reshape(-1)[idx] = rng.integers(-10, 90, size=idx.size).astype(np.int8) // 8 * 8      # many ties
        box = rng.integers(-30, 100, size=(hw, hw, 64), dtype=np.int8)
        heads.append((score, box, -4, -3, stride))
    got = oracle_detect(heads, score_thr, nms_thr, top_k, 150, 140)
    want = reference_detect(heads, score_thr, nms_thr, top_k, 150, 140)
    assert len(want) > 3
    assert [g[0] for g in got] == [w[0] for w in want]
    assert [np.float32(g[1]).tobytes() for g in got] == [np.float32(w[1]).tobytes() for w in want]
    assert [g[2] for g in got] == [w[2] for w in want]


def test_oracle_keeps_the_best_box_of_a_cluster():
    """Two strongly overlapping candidates of one head and a distant one: NMS drops the weaker of the pair."""
    score = np.full((20, 20, 2), -100, dtype=np.int8)
    box = np.zeros((20, 20, 64), dtype=np.int8)
    box[..., 3::16] = 60                      # every side's distribution peaks at bin 3: boxes of 6 x 6 cells
    score[4, 4, 0], score[4, 5, 0], score[15, 15, 1] = 90, 80, 70
    got = oracle_detect([(score, box, -4, -3, 8)], 0.5, 0.3, 10, 160, 160)
    assert [g[0] for g in got] == [0, 1] and got[0][1] > got[1][1]
    assert 40 <= got[0][2][2] - got[0][2][0] <= 50     # about six cells of stride 8
    assert got[0][2][0] < 36 + 4 < got[0][2][2]         # around the centre of cell (4, 4)


@pytest.mark.gpu
def test_candidate_scan_finds_every_score_above_the_threshold():
    import gpu_util
    rng = np.random.default_rng(5)
    n, h, w, classes = 3, 20, 24, 80
    score = rng.integers(-128, 100, size=(n, h, w, classes), dtype=np.int8)
    box = rng.integers(-128, 128, size=(n, h, w, 64), dtype=np.int8)
    thr = 96
    with gpu_util.DeviceBuffers() as dev:
        cap = 4096
        rec = dev.alloc(cap * C.sizeof(abi.DetectRecord))
        cnt = dev.upload(np.zeros(4, dtype=np.uint32))
        d = abi.DetectDesc(dev.upload(score), dev.upload(box), rec, cnt, n, h, w, classes, 64, thr, cap, 2)
        abi.check(dev.lib.espdl_b200_detect_candidates(C.byref(d), None), "detect_candidates")
        count = int(dev.download(cnt, np.zeros(4, dtype=np.uint32))[0])
        raw = dev.download(rec, np.zeros(cap * C.sizeof(abi.DetectRecord), dtype=np.uint8))
    want = np.argwhere(score > thr)
    assert count == len(want) and 0 < count <= cap
    recs = (abi.DetectRecord * count).from_buffer_copy(raw[:count * C.sizeof(abi.DetectRecord)].tobytes())
    got = sorted((r.image, r.y, r.x, r.category, r.score, bytes(r.box)) for r in recs)
    exp = sorted((int(i), int(y), int(x), int(c), int(score[i, y, x, c]), box[i, y, x].tobytes()) for i, y, x, c in want)
    assert [g[:5] for g in got] == [e[:5] for e in exp]
    assert all(g[5] == e[5] for g, e in zip(got, exp))
    assert all(r.stage == 2 for r in recs)


@pytest.mark.gpu
def test_detector_heads_through_the_post_processor(tmp_path):
    """The generated detector at 160x160, three images: dl::detect::yolo11PostProcessor on the device-resident heads
    equals the oracle run over the downloaded heads, image by image."""
    from espdl_b200 import model, zoo
    path = str(tmp_path / "det.espdl")
    zoo.yolo11n_style(seed=6, input_hw=160).save(path)
    m = model.Model(path, batch=3)
    m.inputs[0].array[...] = np.random.default_rng(12).integers(-128, 128, size=m.inputs[0].array.shape, dtype=np.int8)
    m.run()
    outs = {o.name: o for o in m.outputs}
    heads = [(f"head{i}.box_out", f"head{i}.cls_out") for i in range(3)]
    strides = [8, 16, 32]
    # a threshold that a few hundred class scores exceed
    allscores = np.concatenate([outs[c].array.reshape(-1).astype(np.float32) * 2.0 ** outs[c].exponent for _, c in heads])
    logit = np.sort(allscores)[-400]
    thr = float(1.0 / (1.0 + np.exp(-logit)))
    for image in range(3):
        per = [(outs[c].array[image], outs[b].array[image], outs[c].exponent, outs[b].exponent, s) for (b, c), s in zip(heads, strides)]
        # random weights give large, overlapping boxes: with the usual IoU threshold few survive, with a threshold no IoU
        # exceeds all of the best fifty are kept, and a huge frame keeps the decoded coordinates unclamped
        for nms_thr, size in ((0.5, 160), (1.5, 1 << 20)):
            got = m.detect(heads, strides, thr, nms_thr, 50, size, size, image=image)
            want = oracle_detect(per, thr, nms_thr, 50, size, size)
            assert len(want) >= (3 if nms_thr < 1 else 49)
            assert got == want
    m.close()
