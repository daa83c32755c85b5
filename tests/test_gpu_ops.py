"""GPU parity: every CUDA-core kernel behind the C ABI against the plain-C oracle, bit for bit, on seeded
inputs (sizes the oracle finishes in well under a second)."""
import ctypes as C

import numpy as np
import pytest

import cases
import checkers
import gpu_util
from espdl_b200 import abi
from test_oracle_vs_reference import CONV_CASES

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("idx", range(len(CONV_CASES)))
def test_conv_simt(idx, dtype, per_channel, round_mode):
    kw = dict(CONV_CASES[idx])
    if dtype == abi.DTYPE_INT16:
        kw.setdefault("e_in", -14)
        kw.setdefault("e_w", (-15, -13))
        kw.setdefault("e_out", -12)
    case = cases.conv_case(seed=200 + idx, dtype=dtype, per_channel=per_channel, round_mode=round_mode, **kw)
    got = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT)
    np.testing.assert_array_equal(got, gpu_util.run_conv_oracle(case))


def test_conv_simt_config1_exact_shape():
    """The single-image 3x3 conv configuration: 1x56x56x64 -> 64, per-channel exponents in {-9..-6}, ReLU."""
    case = cases.conv_case(seed=1, n=1, h=56, w=56, cin=64, cout=64, kh=3, kw=3, per_channel=True, e_in=-7, e_out=-6, e_w=(-9, -6))
    got = gpu_util.run_conv_gpu(case)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(got, want)
    assert 0.05 < (want == 0).mean() < 0.95 and (want == 127).mean() < 0.5


def test_conv_lut_and_pixel_strides():
    case = cases.conv_case(seed=31, n=2, h=7, w=6, cin=8, cout=12, kh=3, kw=3, lut=True, in_stride=24, out_stride=40, per_channel=True)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), gpu_util.run_conv_oracle(case))


def test_conv_first_layer_shape():
    """3-channel 3x3 stride-2 stem (224x224x3 -> 112x112x32), two images."""
    case = cases.conv_case(seed=33, n=2, h=224, w=224, cin=3, cout=32, kh=3, kw=3, stride=2, pad=(0, 1, 0, 1), per_channel=True,
                           e_in=-7, e_out=-5, e_w=(-8, -6))
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("kw", [
    dict(h=8, w=8, cin=16, kh=3, kw=3),
    dict(n=3, h=14, w=14, cin=96, kh=3, kw=3, stride=2, pad=(0, 1, 0, 1)),       # vector path, stride 2
    dict(n=2, h=9, w=11, cin=24, kh=3, kw=3, stride=2),                          # 24 channels: scalar path
    dict(h=10, w=10, cin=25, kh=7, kw=7, stride=(1, 2), pad=(2, 2, 2, 2)),
    dict(h=8, w=8, cin=32, kh=3, kw=3, dil=2, pad=(2, 2, 2, 2)),
    dict(n=2, h=6, w=7, cin=32, kh=3, kw=3, act=abi.ACT_LINEAR, bias=False),
    dict(n=2, h=6, w=7, cin=32, kh=3, kw=3, in_stride=48, out_stride=64, lut=True),
])
def test_depthwise(kw, dtype, round_mode):
    kw = dict(kw)
    if dtype == abi.DTYPE_INT16:
        kw.update(e_in=-13, e_w=(-14, -12), e_out=-11)
        kw.pop("lut", None)
    case = cases.conv_case(seed=41, dtype=dtype, depthwise=True, per_channel=True, round_mode=round_mode, **kw)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))


DW_SHAPES = [
    dict(n=2, h=28, w=28, cin=32),                         # one 32-channel block, pitch 32
    dict(n=2, h=14, w=14, cin=384),                        # three channel groups, pitch 16
    dict(n=3, h=7, w=7, cin=960),                          # whole image inside one tile, mostly overhang
    dict(n=2, h=56, w=56, cin=144),                        # odd number of 16-channel chunks (144 = 128 + 16)
    dict(n=1, h=33, w=45, cin=48),                         # ragged tiles in both directions
    dict(n=2, h=112, w=112, cin=96, stride=2),             # stride 2, pads [1,1,1,1] on an even image
    dict(n=2, h=56, w=56, cin=144, stride=2),
    dict(n=2, h=14, w=14, cin=576, stride=2),
    dict(n=1, h=15, w=17, cin=16, stride=2, pad=(0, 1, 0, 1)),
    dict(n=2, h=20, w=20, cin=64, pad=(0, 0, 0, 0)),       # no padding
    dict(n=2, h=20, w=20, cin=64, pad=(2, 2, 2, 2)),       # more padding than the filter needs
]


@pytest.mark.parametrize("narrow", [False, True], ids=["auto", "tma-narrow"])
@pytest.mark.parametrize("kw", DW_SHAPES, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items() if a != "pad"))
def test_depthwise_3x3_shapes(kw, narrow, monkeypatch):
    """The 3x3 depthwise kernels on the network's layer shapes, ragged extents and unusual paddings, against the oracle:
    the TMA-fed kernel (the default from 64 channels on; with ESPDL_B200_DW_TMA_NARROW=1 also below) and the kernel that
    reads global memory directly (ESPDL_KERNEL_SIMT).  A depthwise conv has no tensor-core form, so asking for one is
    refused."""
    if narrow:
        if kw["cin"] >= 64:
            pytest.skip("already on the TMA-fed kernel")
        monkeypatch.setenv("ESPDL_B200_DW_TMA_NARROW", "1")
    case = cases.conv_case(seed=61, depthwise=True, kh=3, kw=3, per_channel=True, e_in=-5, e_out=-5, e_w=(-9, -5), **kw)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), want)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), want)
    gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05, expect=abi.ERR_UNSUPPORTED)
    assert want.std() > 0


@pytest.mark.parametrize("round_mode,act,bias,lut", [(abi.ROUND_HALF_EVEN, abi.ACT_RELU, True, False), (abi.ROUND_HALF_UP, abi.ACT_LINEAR, False, False),
                                                     (abi.ROUND_HALF_UP, abi.ACT_RELU, True, True)])
def test_depthwise_3x3_epilogue_variants(round_mode, act, bias, lut):
    case = cases.conv_case(seed=63, n=2, h=19, w=23, cin=80, depthwise=True, kh=3, kw=3, per_channel=True, round_mode=round_mode, act=act,
                           bias=bias, lut=lut, in_stride=96, out_stride=112)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))


def test_depthwise_block_shape():
    """The inverted-residual block's depthwise layer shape: 112x112x192, 3x3 stride 1 (two images)."""
    case = cases.conv_case(seed=43, n=2, h=112, w=112, cin=192, kh=3, kw=3, depthwise=True, per_channel=True, e_in=-5, e_out=-5, e_w=(-9, -5))
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))


def run_eltwise(case, inplace=None):
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input0=dev.upload(case["a"]), input1=dev.upload(case["b"]), output=dev.upload(case["out"]))
        if inplace:
            ptrs["output"] = ptrs[inplace]
        d = cases.eltwise_desc(case, ptrs)
        abi.check(dev.lib.espdl_b200_eltwise(C.byref(d), None), "eltwise")
        got = dev.download(ptrs["output"], case["out"])
    want = case["out"].copy()
    assert checkers.oracle().oracle_eltwise(cases.eltwise_desc(dict(case, out=want))) == 0
    return got, want


BROADCASTS = [
    ((2, 5, 7, 16), None, None), ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 16)), ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 1)),
    ((2, 5, 7, 16), (1, 1, 1, 1), (2, 5, 7, 16)), ((2, 5, 7, 16), (2, 5, 7, 1), (2, 5, 7, 16)), ((2, 5, 7, 16), (2, 5, 7, 16), (2, 5, 7, 1)),
    ((2, 5, 7, 16), (2, 1, 7, 1), (1, 5, 1, 16)), ((2, 5, 7, 1), (2, 5, 7, 1), (1, 5, 1, 1)), ((3, 20), (3, 1), (1, 20)), ((37,), None, None),
    ((1,), None, None),
]


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_MAX, abi.ELT_MIN, abi.ELT_DIV, abi.ELT_MOD])
@pytest.mark.parametrize("shapes", BROADCASTS)
def test_max_min_div_mod(op, dtype, shapes, round_mode):
    e = dict(e0=-5, e1=-5, eo=-5)
    if op == abi.ELT_DIV:
        e = dict(e0=-5, e1=-4, eo=-6) if dtype == abi.DTYPE_INT8 else dict(e0=-12, e1=-9, eo=-10)
    if op == abi.ELT_MOD:
        e = dict(e0=-5, e1=-6, eo=-6) if dtype == abi.DTYPE_INT8 else dict(e0=-12, e1=-13, eo=-11)
    case = cases.eltwise_case(op, seed=23, dtype=dtype, out_shape=shapes[0], in0_shape=shapes[1], in1_shape=shapes[2], round_mode=round_mode, **e)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_GREATER, abi.ELT_GREATER_EQUAL, abi.ELT_EQUAL, abi.ELT_LESS, abi.ELT_LESS_EQUAL])
@pytest.mark.parametrize("shapes", BROADCASTS[:3] + BROADCASTS[6:10])
def test_comparisons(op, dtype, shapes):
    case = cases.eltwise_case(op, seed=29, in_dtype=dtype, out_dtype=abi.DTYPE_BOOL, out_shape=shapes[0], in0_shape=shapes[1],
                              in1_shape=shapes[2], e0=-5, e1=-5, eo=0)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)
    assert op == abi.ELT_EQUAL or (want.any() and not want.all())


def test_comparison_needs_a_bool_output():
    case = cases.eltwise_case(abi.ELT_LESS, seed=1)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input0=dev.upload(case["a"]), input1=dev.upload(case["b"]), output=dev.upload(case["out"]))
        assert dev.lib.espdl_b200_eltwise(C.byref(cases.eltwise_desc(case, ptrs)), None) == abi.ERR_UNSUPPORTED


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_ADD, abi.ELT_SUB, abi.ELT_MUL])
@pytest.mark.parametrize("shapes", [
    ((2, 5, 7, 16), None, None), ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 16)), ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 1)),
    ((2, 5, 7, 16), (1, 1, 1, 1), (2, 5, 7, 16)), ((2, 5, 7, 16), (2, 1, 7, 1), (1, 5, 1, 16)), ((3, 20), (3, 1), (1, 20)), ((37,), None, None),
])
def test_binary(op, dtype, shapes, round_mode):
    e = dict(e0=-5, e1=-6, eo=-8) if op == abi.ELT_MUL else dict(e0=-5, e1=-5, eo=-5)
    if dtype == abi.DTYPE_INT16 and op == abi.ELT_MUL:
        e = dict(e0=-12, e1=-13, eo=-11)
    case = cases.eltwise_case(op, seed=3, dtype=dtype, out_shape=shapes[0], in0_shape=shapes[1], in1_shape=shapes[2],
                              round_mode=round_mode, **e)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("inplace", ["input0", "input1"])
def test_add_in_place(inplace):
    """The planner runs Add in place: the output may alias either input."""
    case = cases.eltwise_case(abi.ELT_ADD, seed=5, out_shape=(4, 14, 14, 32), e0=-5, e1=-5, eo=-5)
    got, want = run_eltwise(case, inplace=inplace)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("idt,odt,e0,eo", [
    (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -2), (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -6), (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -4),
    (abi.DTYPE_INT16, abi.DTYPE_INT16, -10, -7), (abi.DTYPE_INT16, abi.DTYPE_INT8, -10, -5), (abi.DTYPE_INT8, abi.DTYPE_INT16, -5, -10),
    (abi.DTYPE_INT16, abi.DTYPE_INT8, -7, -7), (abi.DTYPE_INT8, abi.DTYPE_INT16, -7, -7),
    (abi.DTYPE_FLOAT, abi.DTYPE_INT8, 0, -4), (abi.DTYPE_FLOAT, abi.DTYPE_INT16, 0, -11),
    (abi.DTYPE_INT8, abi.DTYPE_FLOAT, -4, 0), (abi.DTYPE_INT16, abi.DTYPE_FLOAT, -9, 0),
])
def test_requantize(idt, odt, e0, eo):
    case = cases.eltwise_case(abi.ELT_REQUANTIZE, seed=5, in_dtype=idt, out_dtype=odt, out_shape=(3, 4, 5, 16), e0=e0, eo=eo)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("shape", [(1, 4, 6, 24), (2, 8, 8, 32)])  # scalar and 128-bit paths
@pytest.mark.parametrize("op,dtype,kw", [
    (abi.ELT_LUT, abi.DTYPE_INT8, {}),
    (abi.ELT_LUT, abi.DTYPE_INT16, dict(lut_shift=5)),
    (abi.ELT_LUT, abi.DTYPE_INT16, dict(lut_shift=5, round_mode=abi.ROUND_HALF_EVEN)),
    (abi.ELT_LUT, abi.DTYPE_INT16, dict(lut_shift=0)),
    (abi.ELT_CLIP, abi.DTYPE_INT8, dict(e0=-4, eo=-4, clip=(0, 96))),
    (abi.ELT_CLIP, abi.DTYPE_INT8, dict(e0=-4, eo=-5, clip=(0, 96))),
    (abi.ELT_CLIP, abi.DTYPE_INT16, dict(e0=-10, eo=-9, clip=(-3000, 6000))),
    (abi.ELT_RELU, abi.DTYPE_INT8, dict(e0=-4, eo=-4)),
    (abi.ELT_RELU, abi.DTYPE_INT8, dict(e0=-4, eo=-6)),
    (abi.ELT_RELU, abi.DTYPE_INT16, dict(e0=-9, eo=-7)),
    (abi.ELT_PRELU, abi.DTYPE_INT8, dict(e0=-4, e1=-7, eo=-4)),
    (abi.ELT_PRELU, abi.DTYPE_INT16, dict(e0=-10, e1=-15, eo=-10)),
])
def test_unary(op, dtype, kw, shape):
    case = cases.eltwise_case(op, seed=9, dtype=dtype, out_shape=shape, **kw)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)


def test_lut_all_codes():
    """All 256 input codes through a LUT (the reference's own primitive test pattern, test_apps/dl_pie_func test_lut.cpp)."""
    case = cases.eltwise_case(abi.ELT_LUT, seed=11, out_shape=(256,))
    case["a"] = np.arange(-128, 128, dtype=np.int8)
    got, want = run_eltwise(case)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(got, case["b"][(case["a"].astype(np.int32) + 128)])


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op,kw", [
    (abi.POOL_MAX, dict(kh=3, kw=3, stride=2, pad=(1, 1, 1, 1))),
    (abi.POOL_MAX, dict(h=20, w=20, c=128, kh=5, kw=5, stride=1, pad=(2, 2, 2, 2))),
    (abi.POOL_MAX, dict(kh=2, kw=2, stride=2, pad=(0, 0, 0, 0))),
    (abi.POOL_MAX, dict(n=3, h=24, w=9, c=32, kh=5, kw=5, stride=1, pad=(0, 0, 0, 0))),     # the column walk, no padding
    (abi.POOL_MAX, dict(n=2, h=43, w=11, c=16, kh=5, kw=5, stride=1, pad=(2, 1, 0, 3))),    # uneven pads, columns cut into runs of rows
    (abi.POOL_MAX, dict(n=2, h=13, w=21, c=48, kh=3, kw=3, stride=1, pad=(1, 1, 1, 1))),
    (abi.POOL_MAX, dict(n=1, h=80, w=5, c=16, kh=3, kw=3, stride=1, pad=(0, 2, 2, 0))),
    (abi.POOL_AVG, dict(kh=2, kw=2, stride=2, pad=(0, 0, 0, 0))),
    (abi.POOL_AVG, dict(kh=3, kw=3, stride=2, pad=(1, 1, 1, 1), e_out=-4)),
    (abi.POOL_GLOBAL_AVG, dict(h=7, w=7, c=40, e_in=-4, e_out=-5)),
    (abi.POOL_GLOBAL_AVG, dict(n=4, h=7, w=7, c=1280, e_in=-5, e_out=-5)),
])
def test_pool(op, kw, dtype):
    case = cases.pool_case(op, seed=13, dtype=dtype, **kw)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), output=dev.upload(case["out"]))
        d = cases.pool_desc(case, ptrs)
        abi.check(dev.lib.espdl_b200_pool(C.byref(d), None), "pool")
        got = dev.download(ptrs["output"], case["out"])
    want = case["out"].copy()
    assert checkers.oracle().oracle_pool(cases.pool_desc(dict(case, out=want))) == 0
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("kw", [dict(scale=(2.0, 2.0)), dict(scale=(2.0, 2.0), e_in=-5, e_out=-4), dict(scale=(2.0, 2.0), e_in=-5, e_out=-6),
                                dict(scale=(3.0, 2.0)), dict(scale=(1.5, 2.5), h=8, w=8), dict(scale=(0.5, 0.5), h=8, w=10),
                                dict(scale=(2.0, 2.0), n=2, h=20, w=20, c=64, out_stride=192)])
def test_resize(kw):
    case = cases.resize_case(seed=17, **kw)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), output=dev.upload(case["out"]))
        d = cases.resize_desc(case, ptrs)
        abi.check(dev.lib.espdl_b200_resize(C.byref(d), None), "resize")
        got = dev.download(ptrs["output"], case["out"])
    want = case["out"].copy()
    assert checkers.oracle().oracle_resize(cases.resize_desc(dict(case, out=want))) == 0
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("kw", [dict(scale=(2.0, 2.0), mode=1), dict(scale=(2.0, 2.0), mode=2), dict(scale=(2.0, 2.0), e_in=-5, e_out=-4, mode=1),
          dict(scale=(1.5, 2.5), h=8, w=8, e_in=-5, e_out=-6, mode=1), dict(scale=(0.5, 0.5), h=8, w=10, mode=1),
          dict(scale=(3.0, 1.7), h=7, w=9, c=5, mode=2), dict(scale=(1.0, 2.0), h=1, w=12, c=24, mode=1),
          dict(scale=(1.0, 3.5), h=1, w=9, c=7, e_in=-6, e_out=-5, mode=2), dict(scale=(4.0, 4.0), n=3, h=13, w=11, c=32, mode=1)] + [dict(scale=(2.0, 2.0), n=2, h=20, w=20, c=64, out_stride=192, mode=1)])
def test_linear_resize(kw):
    case = cases.resize_case(seed=19, **kw)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), output=dev.upload(case["out"]))
        d = cases.resize_desc(case, ptrs)
        abi.check(dev.lib.espdl_b200_resize(C.byref(d), None), "resize")
        got = dev.download(ptrs["output"], case["out"])
    want = case["out"].copy()
    assert checkers.oracle().oracle_resize(cases.resize_desc(dict(case, out=want))) == 0
    np.testing.assert_array_equal(got, want)


def test_resize_int16_is_rejected():
    case = cases.resize_case(seed=17, dtype=abi.DTYPE_INT16)
    with gpu_util.DeviceBuffers() as dev:
        d = cases.resize_desc(case, dict(input=dev.upload(case["x"]), output=dev.upload(case["out"])))
        assert dev.lib.espdl_b200_resize(C.byref(d), None) == abi.ERR_UNSUPPORTED


@pytest.mark.parametrize("es,dtype", [(1, np.int8), (2, np.int16), (4, np.float32)])
def test_copy_concat_and_transpose(es, dtype):
    rng = np.random.default_rng(23)
    a = rng.integers(-100, 100, size=(2, 3, 4, 8)).astype(dtype)
    b = rng.integers(-100, 100, size=(2, 3, 4, 24)).astype(dtype)
    with gpu_util.DeviceBuffers() as dev:
        pa, pb = dev.upload(a), dev.upload(b)
        out = np.zeros((2, 3, 4, 32), dtype=dtype)
        po = dev.upload(out)
        for src, off, c in ((pa, 0, 8), (pb, 8, 24)):       # channel Concat = one strided copy per input
            d = cases.copy_desc(src, po + off * es, es, (24, c), (c, 1), (32, 1))
            abi.check(dev.lib.espdl_b200_copy(C.byref(d), None), "copy")
        np.testing.assert_array_equal(dev.download(po, out), np.concatenate([a, b], axis=3))
        # Transpose NHWC -> NCHW: permuted source strides
        t = np.zeros((2, 8, 3, 4), dtype=dtype)
        pt = dev.upload(t)
        d = cases.copy_desc(pa, pt, es, (2, 8, 3, 4), (96, 1, 32, 8), (96, 12, 4, 1))
        abi.check(dev.lib.espdl_b200_copy(C.byref(d), None), "copy")
        np.testing.assert_array_equal(dev.download(pt, t), a.transpose(0, 3, 1, 2))


@pytest.mark.parametrize("dtype", [np.int8, np.int16])
@pytest.mark.parametrize("shape,perm", [((2, 70, 75, 96), (0, 3, 1, 2)), ((3, 130, 17), (0, 2, 1)), ((2, 2, 100, 33), (0, 1, 3, 2)), ((200, 300), (1, 0)),
                                        ((2, 64, 64, 128), (0, 3, 1, 2)), ((4, 19, 64, 16), (2, 0, 3, 1))])
def test_copy_tiled_transposes(shape, perm, dtype):
    """Transposes whose destination runs along an axis that is strided in the source take the shared-memory tile kernel:
    ragged extents, several outer axes, 1- and 2-byte elements."""
    a = np.random.default_rng(29).integers(-30000, 30000, size=shape).astype(dtype)
    want = np.ascontiguousarray(a.transpose(perm))
    es = a.dtype.itemsize
    src_strides = [a.strides[p] // es for p in perm]
    dst_strides = [st // es for st in want.strides]
    with gpu_util.DeviceBuffers() as dev:
        pt = dev.upload(np.full_like(want, 0x55))
        d = cases.copy_desc(dev.upload(a), pt, es, want.shape, src_strides, dst_strides)
        abi.check(dev.lib.espdl_b200_copy(C.byref(d), None), "copy")
        np.testing.assert_array_equal(dev.download(pt, want), want)


@pytest.mark.parametrize("odt,eo", [(abi.DTYPE_FLOAT, 0), (abi.DTYPE_INT8, -7), (abi.DTYPE_INT16, -15)])
@pytest.mark.parametrize("e_in,rows,length", [(-4, 64, 400), (-3, 3, 37), (-6, 5, 64)])
def test_softmax(e_in, rows, length, odt, eo):
    rng = np.random.default_rng(19)
    x = rng.integers(-128, 128, size=(rows, length), dtype=np.int8)
    table = np.zeros(256, dtype=np.float32)
    checkers.oracle().oracle_softmax_table(table.ctypes.data, e_in)
    want = np.zeros((rows, length), dtype=cases.NP[odt])
    assert checkers.oracle().oracle_softmax(cases.softmax_desc(x.ctypes.data, want.ctypes.data, table.ctypes.data, rows, length, odt, eo)) == 0
    with gpu_util.DeviceBuffers() as dev:
        px, pt, po = dev.upload(x), dev.upload(table), dev.upload(np.zeros_like(want))
        d = cases.softmax_desc(px, po, pt, rows, length, odt, eo)
        abi.check(dev.lib.espdl_b200_softmax(C.byref(d), None), "softmax")
        got = dev.download(po, want)
    np.testing.assert_array_equal(got.view(np.uint8), want.view(np.uint8))


def test_invalid_arguments_are_rejected():
    L = gpu_util.lib()
    assert L.espdl_b200_conv2d(None, None) == abi.ERR_INVALID_ARG
    case = cases.conv_case(seed=1)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), filter=dev.upload(case["w"]), bias=dev.upload(case["b"]), filter_exponents=None,
                    lut=None, output=dev.upload(case["out"]))
        bad = cases.conv_desc(dict(case, out_h=case["out_h"] + 1), ptrs)
        assert L.espdl_b200_conv2d(C.byref(bad), None) == abi.ERR_INVALID_ARG
        bad = cases.conv_desc(dict(case, activation=3), ptrs)
        assert L.espdl_b200_conv2d(C.byref(bad), None) == abi.ERR_UNSUPPORTED
        bad = cases.conv_desc(dict(case, per_channel=1), ptrs)
        assert L.espdl_b200_conv2d(C.byref(bad), None) == abi.ERR_INVALID_ARG
        empty = cases.conv_desc(dict(case, n=0), ptrs)
        assert L.espdl_b200_conv2d(C.byref(empty), None) == abi.OK  # empty batch: nothing to do
    assert b"invalid" in L.espdl_b200_strerror(abi.ERR_INVALID_ARG)


def test_a_bounded_wait_that_runs_out_is_reported_and_the_next_launch_works(monkeypatch):
    """Every mbarrier wait of the persistent kernels has a limit.  With ESPDL_B200_DEBUG_WAIT_EXPIRY the TMA-fed depthwise
    kernel withholds one arrival and shortens the limit to a few milliseconds: the wait runs out, the CTA raises its flag,
    every role leaves (nothing traps, nothing spins on), espdl_b200_stream_sync reports ESPDL_ERR_TIMEOUT - and the same
    launch without the switch gives the oracle's result on the same context."""
    import ctypes as C
    case = cases.conv_case(seed=71, n=96, h=56, w=56, cin=64, kh=3, kw=3, depthwise=True, per_channel=True, e_in=-5, e_out=-5, e_w=(-9, -5))
    want = gpu_util.run_conv_oracle(case)
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), filter=dev.upload(case["w"]), bias=dev.upload(case["b"]),
                    filter_exponents=dev.upload(case["ew"]), lut=None, residual=None, output=dev.upload(np.full_like(case["out"], 0x55)))
        d = cases.conv_desc(case, ptrs)
        monkeypatch.setenv("ESPDL_B200_DEBUG_WAIT_EXPIRY", "5")
        assert dev.lib.espdl_b200_conv2d(C.byref(d), None) == abi.OK          # the launch itself succeeds
        assert dev.lib.espdl_b200_stream_sync(None) == abi.ERR_TIMEOUT        # ... and reports that a wait expired
        assert b"wait expired" in dev.lib.espdl_b200_last_error()
        assert dev.lib.espdl_b200_stream_sync(None) == abi.OK                 # the status word was cleared by the read
        monkeypatch.delenv("ESPDL_B200_DEBUG_WAIT_EXPIRY")
        assert dev.lib.espdl_b200_conv2d(C.byref(d), None) == abi.OK
        got = dev.download(ptrs["output"], case["out"])
    np.testing.assert_array_equal(got, want)


# Channel slices: rows of the innermost axis that sit `stride` elements apart inside wider tensors (what the model's
# planner makes of Concat inputs and Split outputs).  The oracle computes the dense case; the device sees slices.
SLICED = [
    (abi.ELT_ADD, abi.DTYPE_INT8, 32, (96, 64, 48), {}),                    # 16-byte kernels, all three strided
    (abi.ELT_REQUANTIZE, abi.DTYPE_INT8, 16, (48, 0, 48), dict(e0=-5, eo=-4)),
    (abi.ELT_REQUANTIZE, abi.DTYPE_INT8, 64, (0, 0, 192), dict(e0=-4, eo=-6)),
    (abi.ELT_LUT, abi.DTYPE_INT8, 48, (64, 0, 0), {}),
    (abi.ELT_MUL, abi.DTYPE_INT8, 16, (32, 48, 0), {}),
    (abi.ELT_ADD, abi.DTYPE_INT8, 24, (40, 24, 56), {}),                    # rows that are no 16-byte units: the scalar kernel
    (abi.ELT_ADD, abi.DTYPE_INT16, 16, (48, 32, 16), {}),
    (abi.ELT_MAX, abi.DTYPE_INT8, 32, (0, 64, 64), {}),
]


@pytest.mark.parametrize("op,dtype,c,strides,kw", SLICED)
def test_eltwise_on_channel_slices(op, dtype, c, strides, kw):
    shape = (3, 5, 7, c)
    rows = 3 * 5 * 7
    case = cases.eltwise_case(op, seed=41, dtype=dtype, out_shape=shape, **kw)
    want = case["out"].copy()
    assert checkers.oracle().oracle_eltwise(cases.eltwise_desc(dict(case, out=want))) == 0
    rng = np.random.default_rng(8)
    es = case["out"].dtype.itemsize

    def widen(arr, stride, lead):
        """The dense rows of `arr` placed `lead` elements into rows of `stride` elements; the rest is random filler."""
        if not stride:
            return np.ascontiguousarray(arr), 0
        wide = rng.integers(-100, 100, size=(rows, stride)).astype(arr.dtype)
        wide[:, lead:lead + c] = arr.reshape(rows, c)
        return wide, lead

    two = case["b"] is not None and case["b"].shape == case["a"].shape
    wa, la = widen(case["a"], strides[0], 16 if strides[0] >= c + 16 else 0)
    wb, lb = widen(case["b"], strides[1], 0) if two else (case["b"], 0)
    wo, lo = widen(case["out"], strides[2], 16 if strides[2] >= c + 16 else 0)
    before = wo.copy()
    with gpu_util.DeviceBuffers() as dev:
        pa, pb, po = dev.upload(wa), dev.upload(wb), dev.upload(wo)
        d = cases.eltwise_desc(case, dict(input0=pa + la * es, input1=(pb + lb * es) if pb else None, output=po + lo * es))
        d.in0_row_stride, d.in1_row_stride, d.out_row_stride = strides[0], strides[1] if two else 0, strides[2]
        d.ndim = 2
        for name in ("out_shape", "in0_shape", "in1_shape"):
            getattr(d, name)[0], getattr(d, name)[1] = rows, c
        if not two:
            d.in1_shape[0] = d.in1_shape[1] = 1
        abi.check(dev.lib.espdl_b200_eltwise(C.byref(d), None), "eltwise")
        got = dev.download(po, wo)
    if strides[2]:
        np.testing.assert_array_equal(got[:, lo:lo + c], want.reshape(rows, c))
        before[:, lo:lo + c] = want.reshape(rows, c)
        np.testing.assert_array_equal(got, before)          # nothing outside the slice was written
    else:
        np.testing.assert_array_equal(got, want)
    assert want.astype(np.float32).std() > 0


def test_eltwise_rejects_bad_row_strides():
    case = cases.eltwise_case(abi.ELT_ADD, seed=1, out_shape=(4, 16))
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input0=dev.upload(case["a"]), input1=dev.upload(case["b"]), output=dev.upload(case["out"]))
        d = cases.eltwise_desc(case, ptrs)
        d.out_row_stride = 8                                 # shorter than a row
        assert dev.lib.espdl_b200_eltwise(C.byref(d), None) == abi.ERR_INVALID_ARG
        d = cases.eltwise_desc(dict(case, op=abi.ELT_DIV), ptrs)
        d.in0_row_stride = 32
        assert dev.lib.espdl_b200_eltwise(C.byref(d), None) == abi.ERR_UNSUPPORTED


@pytest.mark.parametrize("split", [0, 1])
def test_concat_split_with_slices_and_parts_in_place(split):
    """Parts whose rows sit a stride apart, and a part that already lives inside the wide tensor (left alone)."""
    rng = np.random.default_rng(12)
    rows, widths = 37, [32, 16, 48]
    wide = rng.integers(-128, 128, size=(rows, sum(widths)), dtype=np.int8)
    holder = rng.integers(-128, 128, size=(rows, 80), dtype=np.int8)      # part 1 lives at columns 32..48 of 80-byte rows
    dense2 = rng.integers(-128, 128, size=(rows, widths[2]), dtype=np.int8)
    with gpu_util.DeviceBuffers() as dev:
        pw, ph, p2 = dev.upload(wide), dev.upload(holder), dev.upload(dense2)
        d = abi.PartsDesc()
        d.wide, d.n_parts, d.split, d.rows = pw, 3, split, rows
        for i, w in enumerate(widths):
            d.part_bytes[i] = w
        d.parts[0], d.skip[0] = None, 1
        d.parts[1], d.part_stride[1] = ph + 32, 80
        d.parts[2] = p2
        abi.check(dev.lib.espdl_b200_concat_split(C.byref(d), None), "concat_split")
        got_w, got_h, got_2 = dev.download(pw, wide), dev.download(ph, holder), dev.download(p2, dense2)
    if split:
        np.testing.assert_array_equal(got_w, wide)
        want_h = holder.copy()
        want_h[:, 32:48] = wide[:, 32:48]
        np.testing.assert_array_equal(got_h, want_h)
        np.testing.assert_array_equal(got_2, wide[:, 48:])
    else:
        want_w = wide.copy()
        want_w[:, 32:48] = holder[:, 32:48]
        want_w[:, 48:] = dense2
        np.testing.assert_array_equal(got_w, want_w)
        np.testing.assert_array_equal(got_h, holder)
