"""Image pre-processing (espdl_b200_image_preprocess) against the oracle's restatement of the reference's
ImagePreprocessor: crop, nearest-neighbour resize, letterbox, R/B swap, normalise + quantise table.  The reference
ships no vectors for this step (parity pinned by the restatement only); the table formula is checked against a
direct evaluation."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

MEAN, STD = (123.675, 116.28, 103.53), (58.395, 57.12, 57.375)


def table(channels, exponent, bits=8, mean=MEAN, std=STD):
    L = checkers.oracle()
    L.oracle_norm_quant_table.restype = None
    L.oracle_norm_quant_table.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int, C.c_int, C.c_int]
    t = np.zeros((channels, 256), dtype=np.int8 if bits == 8 else np.int16)
    L.oracle_norm_quant_table(t.ctypes.data, channels, (C.c_float * 3)(*mean), (C.c_float * 3)(*std), exponent, bits, 0)
    return t


@pytest.mark.skipif(not checkers.have_ref(), reason="oracle/_ref/libespdl_ref.so not built")
@pytest.mark.parametrize("bits", [8, 16])
@pytest.mark.parametrize("exponent", [-7, -5, -4, 0, 2])
@pytest.mark.parametrize("mean,std", [(MEAN, STD), ((0.0, 0.0, 0.0), (1.0, 1.0, 1.0)), ((127.5, 127.5, 127.5), (128.0, 64.0, 255.0))])
def test_oracle_norm_quant_table_equals_the_reference(bits, exponent, mean, std):
    """The normalise + quantise table against the reference's own NormQuant (vision/image/dl_image_norm_quant.hpp,
    compiled into oracle/_ref): all 3 x 256 entries, int8 and int16, exponents on both sides of zero."""
    R = checkers.ref()
    R.ref_norm_quant_table.restype = C.c_int
    R.ref_norm_quant_table.argtypes = [C.c_void_p, C.POINTER(C.c_float), C.POINTER(C.c_float), C.c_int, C.c_int]
    want = np.zeros((3, 256), dtype=np.int8 if bits == 8 else np.int16)
    assert R.ref_norm_quant_table(want.ctypes.data, (C.c_float * 3)(*mean), (C.c_float * 3)(*std), exponent, bits) == 0
    np.testing.assert_array_equal(table(3, exponent, bits, mean, std), want)
    assert exponent > 0 or want.std() > 0


def letterbox(src_w, src_h, dst_w, dst_h):
    """dl_image_preprocessor.cpp:108-131"""
    sx, sy = np.float32(dst_w) / np.float32(src_w), np.float32(dst_h) / np.float32(src_h)
    s = min(sx, sy)
    if sx < sy:
        pad = dst_h - int(s * np.float32(src_h))
        return pad // 2, pad - pad // 2, 0, 0
    pad = dst_w - int(s * np.float32(src_w))
    return 0, 0, pad // 2, pad - pad // 2


def make_desc(case, inp, out, lut):
    d = abi.ImageDesc()
    d.input, d.output, d.lut = inp, out, lut
    n, sh, sw, ch = case["x"].shape
    d.n, d.src_h, d.src_w, d.channels = n, sh, sw, ch
    d.dst_h, d.dst_w = case["dst"]
    d.out_dtype = abi.DTYPE_INT8 if case["bits"] == 8 else abi.DTYPE_INT16
    crop = case.get("crop") or (0, 0, 0, 0)
    d.crop_x0, d.crop_y0, d.crop_x1, d.crop_y1 = crop
    cw, chh = (crop[2] - crop[0], crop[3] - crop[1]) if case.get("crop") else (sw, sh)
    border = letterbox(cw, chh, d.dst_w, d.dst_h) if case.get("letterbox") else (0, 0, 0, 0)
    d.border_top, d.border_bottom, d.border_left, d.border_right = border
    d.swap_rb = int(case.get("swap", False))
    for i, b in enumerate(case.get("bg", (114, 114, 114))):
        d.bg[i] = b
    d.inv_scale_x = float(np.float32(cw) / np.float32(d.dst_w - border[2] - border[3]))
    d.inv_scale_y = float(np.float32(chh) / np.float32(d.dst_h - border[0] - border[1]))
    return d


def image_case(seed, n, sh, sw, ch, dst, bits=8, **kw):
    x = np.random.default_rng(seed).integers(0, 256, size=(n, sh, sw, ch), dtype=np.uint8)
    return dict(x=x, dst=dst, bits=bits, lut=table(ch, -5 if bits == 8 else -12, bits), **kw)


def run_oracle(case):
    L = checkers.oracle()
    L.oracle_image_preprocess.restype = C.c_int
    L.oracle_image_preprocess.argtypes = [C.POINTER(abi.ImageDesc)]
    out = np.zeros((case["x"].shape[0],) + tuple(case["dst"]) + (case["x"].shape[3],), dtype=case["lut"].dtype)
    d = make_desc(case, case["x"].ctypes.data, out.ctypes.data, case["lut"].ctypes.data)
    assert L.oracle_image_preprocess(C.byref(d)) == 0
    return out


CASES = [
    dict(seed=1, n=2, sh=480, sw=640, ch=3, dst=(224, 224)),                                   # plain resize down
    dict(seed=2, n=1, sh=100, sw=60, ch=3, dst=(224, 224), swap=True),                         # resize up, BGR order
    dict(seed=3, n=3, sh=360, sw=640, ch=3, dst=(640, 640), letterbox=True),                   # letterbox top/bottom
    dict(seed=4, n=1, sh=500, sw=300, ch=3, dst=(320, 320), letterbox=True, bg=(0, 10, 255)),  # letterbox left/right
    dict(seed=5, n=2, sh=240, sw=320, ch=3, dst=(96, 96), crop=(17, 33, 211, 200)),            # crop, then resize
    dict(seed=6, n=2, sh=224, sw=224, ch=3, dst=(224, 224), swap=True),                        # same size: identity map
    dict(seed=7, n=2, sh=120, sw=160, ch=1, dst=(64, 64)),                                     # gray
    dict(seed=8, n=1, sh=480, sw=640, ch=3, dst=(224, 224), bits=16),                          # int16 model input
]


def test_table_follows_the_reference_formula():
    t = table(3, -5)
    for c in range(3):
        inv_std = np.float32(1.0) / np.float32(STD[c])
        x = (np.arange(256, dtype=np.float32) - np.float32(MEAN[c])) * inv_std
        want = np.clip(np.floor(x * np.float32(32.0) + np.float32(0.5)), -128, 127).astype(np.int8)
        np.testing.assert_array_equal(t[c], want)


@pytest.mark.parametrize("kw", CASES, ids=lambda k: f"seed{k['seed']}")
def test_oracle_against_direct_indexing(kw):
    """The restatement itself, against an independent numpy evaluation of the same index maps."""
    case = image_case(**kw)
    got = run_oracle(case)
    d = make_desc(case, 0, 0, 0)
    n, sh, sw, ch = case["x"].shape
    x0, y0, x1, y1 = (d.crop_x0, d.crop_y0, d.crop_x1, d.crop_y1) if case.get("crop") else (0, 0, sw, sh)
    iw, ih = d.dst_w - d.border_left - d.border_right, d.dst_h - d.border_top - d.border_bottom
    if (x1 - x0, y1 - y0) == (iw, ih):
        xs, ys = np.arange(iw) + x0, np.arange(ih) + y0
    else:
        xs = np.minimum((np.arange(iw, dtype=np.float32) * np.float32(d.inv_scale_x)).astype(np.int32) + x0, x1 - 1)
        ys = np.minimum((np.arange(ih, dtype=np.float32) * np.float32(d.inv_scale_y)).astype(np.int32) + y0, y1 - 1)
    src = np.empty((n, d.dst_h, d.dst_w, ch), dtype=np.uint8)
    src[...] = np.array(list(d.bg)[:ch], dtype=np.uint8)
    src[:, d.border_top:d.border_top + ih, d.border_left:d.border_left + iw] = case["x"][:, ys][:, :, xs]
    if case.get("swap"):
        src = src[..., ::-1]
    want = np.stack([case["lut"][c][src[..., c]] for c in range(ch)], axis=-1)
    np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("kw", CASES, ids=lambda k: f"seed{k['seed']}")
def test_gpu_matches_oracle(kw):
    import gpu_util
    case = image_case(**kw)
    want = run_oracle(case)
    with gpu_util.DeviceBuffers() as dev:
        out = dev.upload(np.full_like(want, 0x55))
        d = make_desc(case, dev.upload(case["x"]), out, dev.upload(case["lut"]))
        abi.check(dev.lib.espdl_b200_image_preprocess(C.byref(d), None), "image_preprocess")
        got = dev.download(out, want)
    np.testing.assert_array_equal(got, want)


@pytest.mark.gpu
@pytest.mark.parametrize("letterbox,swap,crop", [(None, False, None), (114, True, None), (None, False, (40, 20, 600, 440))])
def test_model_preprocessor_fills_the_input_tensor(tmp_path, letterbox, swap, crop):
    """dl::image::ImagePreprocessor on a model: host images -> device conversion -> the model's input tensor; the network
    then runs on what is resident and gives the logits of the oracle-converted input."""
    from espdl_b200 import model, zoo, espdl_file
    import graph_oracle
    path = str(tmp_path / "net.espdl")
    zoo.mobilenet_v2(seed=5, input_hw=96).save(path)
    m = model.Model(path, batch=3)
    name = m.inputs[0].name
    e_in = m.inputs[0].exponent
    imgs = np.random.default_rng(11).integers(0, 256, size=(3, 480, 640, 3), dtype=np.uint8)
    m.preprocess(imgs, MEAN, STD, rgb_swap=swap, letterbox=letterbox, crop=crop)
    case = dict(x=imgs, dst=(96, 96), bits=8, lut=table(3, e_in), swap=swap, crop=crop, letterbox=letterbox is not None,
                bg=(letterbox or 0,) * 3)
    want_in = run_oracle(case)
    got_in = m.read_tensor(name, np.int8, want_in.shape)
    np.testing.assert_array_equal(got_in, want_in)
    m.run_device()
    want = graph_oracle.run_graph(espdl_file.read(path), {name: want_in})
    out = m.outputs[0]
    got = m.read_tensor(out.name, np.int8, out.array.shape)
    np.testing.assert_array_equal(got, want[out.name])
    # dl::cls::ClsPostprocessor: softmax of the logits with the reference's exp table, threshold, sort, top-k
    import cases
    logits = want[out.name]
    table_f = np.zeros(256, dtype=np.float32)
    checkers.oracle().oracle_softmax_table(table_f.ctypes.data, out.exponent)
    probs = np.zeros(logits.shape, dtype=np.float32)
    assert checkers.oracle().oracle_softmax(cases.softmax_desc(logits.ctypes.data, probs.ctypes.data, table_f.ctypes.data, logits.shape[0],
                                                               logits.shape[1], abi.DTYPE_FLOAT, 0)) == 0
    for image in range(3):
        top = m.classify(image=image, top_k=5, score_thr=0.0)
        order = np.argsort(-probs[image], kind="stable")[:5]
        assert len(top) == 5
        np.testing.assert_array_equal(np.array([s for _, s in top], dtype=np.float32), probs[image][order])
        for cat, score in top:
            assert probs[image][cat] == np.float32(score)
    m.close()
