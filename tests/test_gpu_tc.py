"""GPU parity of the tcgen05 tile kernel (pointwise conv / Gemm, int8 and int16) against the plain-C oracle,
and replay of the reference's golden Gemm models through the C ABI."""
import os

import numpy as np
import pytest

import cases
import gpu_util
from espdl_b200 import abi
from test_golden_vectors import GEMM_FILES, replay_gemm_chain

pytestmark = pytest.mark.gpu

# (M, K, N): ragged M, every K swizzle width (32 / 64 / 128 byte rows, partial last K block),
# N below / not a multiple of 16, N split over several tiles.
TC_SHAPES = [
    (128, 128, 128), (256, 64, 64), (100, 32, 32), (1, 16, 16), (300, 16, 96), (777, 96, 24), (130, 144, 32),
    (257, 192, 32), (384, 32, 192), (50, 384, 64), (64, 576, 96), (33, 960, 160), (200, 320, 1280), (129, 1280, 1000),
    (512, 160, 960), (90, 48, 17), (128, 256, 256), (1000, 64, 40),
]


@pytest.mark.parametrize("shape", TC_SHAPES, ids=lambda s: "x".join(map(str, s)))
def test_gemm_s8_tc(shape):
    m, k, n = shape
    case = cases.gemm_case(seed=sum(shape), m=m, k=k, n_out=n, per_channel=True, e_in=-7, e_out=-5 + (k > 256), e_w=(-9, -6))
    want = gpu_util.run_conv_oracle(case)
    got = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05)
    np.testing.assert_array_equal(got, want)
    assert want.std() > 0


@pytest.mark.parametrize("round_mode", [abi.ROUND_HALF_UP, abi.ROUND_HALF_EVEN])
@pytest.mark.parametrize("act", [abi.ACT_LINEAR, abi.ACT_RELU])
def test_gemm_s8_tc_epilogue_variants(act, round_mode):
    for per_channel, bias, lut in [(False, True, False), (True, False, False), (True, True, True)]:
        case = cases.gemm_case(seed=5, m=300, k=64, n_out=48, per_channel=per_channel, bias=bias, lut=lut, act=act, round_mode=round_mode)
        np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), gpu_util.run_conv_oracle(case))


def test_pointwise_conv_tc_nhwc_and_strides():
    """A 1x1 conv over an NHWC batch, reading a channel slice of a wider tensor and writing into a Concat slice."""
    case = cases.conv_case(seed=7, n=3, h=14, w=14, cin=32, cout=64, kh=1, kw=1, pad=(0, 0, 0, 0), per_channel=True,
                           in_stride=48, out_stride=96)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), gpu_util.run_conv_oracle(case))


def test_tc_and_simt_agree_and_auto_picks_tc():
    case = cases.gemm_case(seed=9, m=500, k=96, n_out=144, per_channel=True)
    a = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05)
    b = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT)
    c = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_AUTO)
    np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(a, c)


def test_tc_rejects_shapes_it_cannot_run():
    case = cases.gemm_case(seed=9, m=64, k=24, n_out=16)  # K not a multiple of 16
    gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05, expect=abi.ERR_UNSUPPORTED)
    case = cases.conv_case(seed=9, cin=24, cout=16, kh=3, kw=3)  # 3x3 with Cin not a multiple of 16
    gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05, expect=abi.ERR_UNSUPPORTED)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(cases.gemm_case(seed=9, m=64, k=24, n_out=16)),
                                  gpu_util.run_conv_oracle(cases.gemm_case(seed=9, m=64, k=24, n_out=16)))


@pytest.mark.parametrize("shape", [(128, 128, 128), (100, 64, 48), (300, 1024, 200), (64, 16, 16), (257, 144, 130)],
                         ids=lambda s: "x".join(map(str, s)))
def test_gemm_s16_tc(shape):
    """int16 through 8-bit limbs: full-range operands, int64 bias, shift 17 (the int16 Gemm configuration's exponents)."""
    m, k, n = shape
    case = cases.gemm_case(seed=sum(shape), dtype=abi.DTYPE_INT16, m=m, k=k, n_out=n, e_in=-14, e_w=(-15, -15), e_out=-12, wide=True,
                           bias_mag=1 << 20)
    want = gpu_util.run_conv_oracle(case)
    got = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05)
    np.testing.assert_array_equal(got, want)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), want)
    assert want.std() > 0


def test_gemm_s16_tc_extreme_values():
    """All operands at -32768 / 32767: the limb partial sums reach their largest magnitude."""
    case = cases.gemm_case(seed=1, dtype=abi.DTYPE_INT16, m=130, k=2048, n_out=32, e_in=-14, e_w=(-15, -15), e_out=-2, wide=True)
    case["x"][:] = -32768
    case["w"][:] = -32768
    case["x"][0, 0, 1::2] = 32767
    case["w"][1::2] = 32767
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), gpu_util.run_conv_oracle(case))


def test_config2_int8_gemm_full_size():
    """int8 Gemm 4096x1024x1024, per-channel exponents in {-9..-6}, int32 bias, output exponent -5, no activation."""
    case = cases.gemm_case(seed=2, m=4096, k=1024, n_out=1024, per_channel=True, e_in=-7, e_out=-5, e_w=(-9, -6))
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), want)
    assert (np.abs(want.astype(np.int32)) < 127).mean() > 0.3


def test_config2_int16_gemm_full_size():
    """int16 variant: A/B over the full int16 range, exponents -14/-15, output exponent -12 (shift 17)."""
    case = cases.gemm_case(seed=3, dtype=abi.DTYPE_INT16, m=4096, k=1024, n_out=1024, e_in=-14, e_w=(-15, -15), e_out=-12, wide=True,
                           bias_mag=1 << 20)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), want)


@pytest.mark.parametrize("path", GEMM_FILES, ids=os.path.basename)
def test_gpu_reproduces_golden_gemm(path):
    mode = abi.ROUND_HALF_EVEN if "esp32p4" in os.path.basename(path) else abi.ROUND_HALF_UP
    m, tensors = replay_gemm_chain(path, lambda case: gpu_util.run_conv_gpu(case), mode)
    for name, t in m["test_outputs"].items():
        np.testing.assert_array_equal(tensors[name].reshape(-1), t["data"].reshape(-1))


STEM_SHAPES = [
    dict(n=2, h=224, w=224, cout=32, pad=(0, 1, 0, 1)),     # the classifier's first layer
    dict(n=1, h=96, w=96, cout=16, pad=(1, 1, 1, 1)),       # left/top padding: window shifted by 16 bytes, first row index -1
    dict(n=3, h=64, w=80, cout=32, pad=(0, 1, 0, 1), act=abi.ACT_LINEAR, bias=False),
    dict(n=9, h=32, w=48, cout=32, pad=(1, 0, 1, 0)),       # two image groups, the second almost empty
    dict(n=5, h=33, w=48, cout=16, pad=(0, 0, 0, 0)),       # 23 output columns (ragged last group of eight), odd height
    dict(n=2, h=48, w=64, cout=32, pad=(1, 1, 1, 1), round_mode=abi.ROUND_HALF_EVEN),   # general epilogue
    dict(n=2, h=48, w=64, cout=16, pad=(0, 1, 0, 1), lut=True),
]


@pytest.mark.parametrize("kw", STEM_SHAPES, ids=lambda k: f"n{k['n']}-{k['h']}x{k['w']}-c{k['cout']}-p{''.join(map(str, k['pad']))}")
def test_stem_conv_tensor_core(kw):
    """3x3 stride-2 RGB first layer through the banded-filter tensor-core kernel, against the oracle and the CUDA-core kernel."""
    case = cases.conv_case(seed=91, cin=3, kh=3, kw=3, stride=2, per_channel=True, e_in=-7, e_out=-5, e_w=(-8, -6), **kw)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), want)
    assert want.std() > 0


@pytest.mark.parametrize("m,k,n,rm", [(1, 64, 32, abi.ROUND_HALF_EVEN), (130, 64, 32, abi.ROUND_HALF_UP), (200, 128, 256, abi.ROUND_HALF_UP),
                                      (300, 96, 1000, abi.ROUND_HALF_UP), (77, 160, 240, abi.ROUND_HALF_EVEN)])
def test_tile_kernel_direct_row_stores(m, k, n, rm, monkeypatch):
    """The same tiles with the staged (TMA-store) epilogue switched off: rows go out of registers directly."""
    case = cases.gemm_case(seed=17, m=m, k=k, n_out=n, round_mode=rm, per_channel=True)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    monkeypatch.setenv("ESPDL_B200_DIRECT_STORES", "1")
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)


CONV_TC_SHAPES = [
    dict(n=1, h=56, w=56, cin=64, cout=64),                                   # the single-image 3x3 configuration
    dict(n=3, h=20, w=17, cin=16, cout=48),                                   # ragged tiles, 16-channel rows
    dict(n=2, h=14, w=14, cin=96, cout=200),                                  # Cin fills three quarters of a 128-byte row, ragged Cout
    dict(n=2, h=28, w=28, cin=160, cout=64),                                  # two channel blocks per tap
    dict(n=2, h=33, w=29, cin=32, cout=32, stride=2, pad=(0, 1, 0, 1)),       # stride 2 through TMA element strides
    dict(n=2, h=31, w=30, cin=48, cout=80, stride=2),
    dict(n=1, h=24, w=24, cin=32, cout=64, kh=5, kw=5, pad=(2, 2, 2, 2)),     # 25 taps
    dict(n=2, h=19, w=23, cin=32, cout=16, kh=3, kw=3, dil=2, pad=(2, 2, 2, 2)),
    dict(n=2, h=12, w=40, cin=64, cout=320, kh=1, kw=3, pad=(0, 0, 1, 1)),    # two tiles along Cout
    dict(n=2, h=16, w=16, cin=64, cout=64, kh=1, kw=1, stride=2, pad=(0, 0, 0, 0)),  # strided pointwise (downsample shortcut)
    dict(n=2, h=9, w=9, cin=32, cout=32, pad=(0, 0, 0, 0)),                   # no padding
]


@pytest.mark.parametrize("kw", CONV_TC_SHAPES, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items() if a != "pad"))
def test_conv_implicit_gemm_tensor_core(kw):
    """Dense conv with a real filter window through the implicit-GEMM tile kernel, against the oracle and the CUDA-core kernel."""
    kw = dict(kw)
    kw.setdefault("kh", 3)
    kw.setdefault("kw", 3)
    case = cases.conv_case(seed=77, per_channel=True, e_in=-7, e_out=-6, e_w=(-9, -6), **kw)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), want)
    assert want.std() > 0


@pytest.mark.parametrize("round_mode,act,bias,lut,direct", [(abi.ROUND_HALF_EVEN, abi.ACT_RELU, True, False, False), (abi.ROUND_HALF_UP, abi.ACT_LINEAR, False, False, False),
                                                            (abi.ROUND_HALF_UP, abi.ACT_RELU, True, True, False), (abi.ROUND_HALF_UP, abi.ACT_RELU, True, False, True)])
def test_conv_implicit_gemm_epilogue_variants(round_mode, act, bias, lut, direct, monkeypatch):
    if direct:
        monkeypatch.setenv("ESPDL_B200_DIRECT_STORES", "1")
    case = cases.conv_case(seed=78, n=2, h=18, w=22, cin=32, cout=48, kh=3, kw=3, per_channel=True, round_mode=round_mode, act=act, bias=bias, lut=lut,
                           e_in=-7, e_out=-6, e_w=(-9, -6))
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), gpu_util.run_conv_oracle(case))


@pytest.mark.parametrize("n,m,k,nout,kernel", [(6, 100, 32, 100, abi.KERNEL_TCGEN05), (3, 400, 400, 64, abi.KERNEL_TCGEN05), (5, 130, 64, 40, abi.KERNEL_AUTO),
                                               (4, 9, 24, 7, abi.KERNEL_AUTO)])
def test_batched_matrix_products(n, m, k, nout, kernel):
    """filter_image_stride: image i multiplies by its own filter - all slices of a MatMul in one launch of the tile
    kernel (the last case, K = 24, takes the one-call-per-image fallback)."""
    rng = np.random.default_rng(5)
    case = cases.conv_case(seed=21, n=n, h=1, w=m, cin=k, cout=nout, kh=1, kw=1, pad=(0, 0, 0, 0), per_channel=False, bias=False,
                           act=abi.ACT_LINEAR, e_in=-6, e_w=(-7, -7), e_out=-4)
    case["w"] = rng.integers(-127, 128, size=(n, nout, 1, 1, k), dtype=np.int8)   # one [N][K] filter per image
    case["filter_image_stride"] = nout * k
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 5
    for i in range(n):   # the oracle's batched form equals n separate Gemms
        one = cases.gemm_case(seed=0, m=m, k=k, n_out=nout, per_channel=False, bias=False, e_in=-6, e_w=(-7, -7), e_out=-4)
        one["x"], one["w"] = np.ascontiguousarray(case["x"][i:i + 1]), np.ascontiguousarray(case["w"][i])
        np.testing.assert_array_equal(gpu_util.run_conv_oracle(one)[0], want[i])
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=kernel), want)


@pytest.mark.parametrize("m,k,n,act,kernel,direct", [(300, 96, 32, abi.ACT_LINEAR, abi.KERNEL_TCGEN05, False), (1000, 384, 64, abi.ACT_RELU, abi.KERNEL_TCGEN05, False),
                                                    (200, 64, 250, abi.ACT_LINEAR, abi.KERNEL_TCGEN05, False), (257, 144, 24, abi.ACT_LINEAR, abi.KERNEL_TCGEN05, True),
                                                    (90, 24, 40, abi.ACT_LINEAR, abi.KERNEL_SIMT, False)])
def test_pointwise_conv_with_folded_add(m, k, n, act, kernel, direct, monkeypatch):
    """espdl_conv_desc::residual: out = sat(sat(conv) + residual), the Add of equal exponents that follows a project conv."""
    if direct:
        monkeypatch.setenv("ESPDL_B200_DIRECT_STORES", "1")
    case = cases.gemm_case(seed=33, m=m, k=k, n_out=n, per_channel=True, act=act, e_in=-7, e_out=-6, e_w=(-9, -7))
    case["res"] = np.random.default_rng(34).integers(-128, 128, size=case["out"].shape, dtype=np.int8)
    want = gpu_util.run_conv_oracle(case)
    plain = gpu_util.run_conv_oracle(dict(case, res=None))
    np.testing.assert_array_equal(want, np.clip(plain.astype(np.int32) + case["res"], -128, 127).astype(np.int8))
    assert (want != plain).mean() > 0.5 and (np.abs(want.astype(int)) == 127).mean() < 0.6
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=kernel), want)


@pytest.mark.parametrize("m,k,n,rm,act", [
    (4096, 1024, 1024, abi.ROUND_HALF_UP, abi.ACT_LINEAR),    # benchmark configuration 2
    (2304, 512, 256, abi.ROUND_HALF_UP, abi.ACT_RELU),        # one tile column, nine row pairs
    (2200, 528, 320, abi.ROUND_HALF_UP, abi.ACT_LINEAR),      # ragged M and K, two tiles of 160 columns
    (2176, 640, 1000, abi.ROUND_HALF_UP, abi.ACT_RELU),       # odd number of row tiles: the last pair's second CTA has no rows; ragged N
    (2048, 512, 512, abi.ROUND_HALF_EVEN, abi.ACT_LINEAR),    # general epilogue
])
def test_gemm_s8_cta_pairs(m, k, n, rm, act, monkeypatch):
    """Large int8 products on pairs of CTAs (tcgen05.mma.cta_group::2, 256-row tiles; ESPDL_B200_CTA_PAIRS=1): same
    bits as the oracle."""
    monkeypatch.setenv("ESPDL_B200_CTA_PAIRS", "1")
    case = cases.gemm_case(seed=m + n, m=m, k=k, n_out=n, per_channel=True, e_in=-7, e_out=-5 + (k > 512), e_w=(-9, -6), act=act, round_mode=rm)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)


def test_gemm_s8_same_shape_without_cta_pairs(monkeypatch):
    monkeypatch.delenv("ESPDL_B200_CTA_PAIRS", raising=False)
    case = cases.gemm_case(seed=77, m=2304, k=512, n_out=256, per_channel=True, e_in=-7, e_out=-5, e_w=(-9, -6))
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), gpu_util.run_conv_oracle(case))


# 3x3 convs with 8 or 16 input channels: the banded-filter kernel over 128-byte row windows (conv_band_tc.cu).
# (cin, cout, stride, pad (t, b, l, r), n, h, w)
BAND = [(16, 8, 1, (1, 1, 1, 1), 3, 20, 24), (8, 16, 1, (1, 1, 1, 1), 2, 17, 26), (16, 32, 2, (0, 1, 0, 1), 5, 32, 32),
        (16, 32, 2, (1, 1, 1, 1), 2, 21, 40), (16, 32, 1, (1, 1, 1, 1), 9, 16, 16), (16, 16, 1, (0, 0, 0, 0), 1, 9, 11),
        (8, 32, 2, (1, 0, 1, 0), 4, 30, 36), (8, 8, 1, (1, 1, 1, 1), 1, 12, 100), (16, 64, 1, (1, 1, 1, 1), 2, 10, 7),
        (16, 8, 1, (1, 1, 1, 1), 16, 160, 160)]


@pytest.mark.parametrize("cin,cout,stride,pad,n,h,w", BAND)
@pytest.mark.parametrize("act,per_channel,lut", [(abi.ACT_RELU, True, False), (abi.ACT_LINEAR, False, False), (abi.ACT_LINEAR, True, True)])
def test_small_channel_conv_banded_kernel(cin, cout, stride, pad, n, h, w, act, per_channel, lut):
    case = cases.conv_case(seed=cin + cout + h, n=n, h=h, w=w, cin=cin, cout=cout, kh=3, kw=3, stride=stride, pad=pad, act=act,
                           per_channel=per_channel, e_in=-6, e_out=-5, e_w=(-9, -7), lut=lut)
    want = gpu_util.run_conv_oracle(case)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), want)
    # the CUDA-core kernels give the same bytes
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_SIMT), want)


@pytest.mark.parametrize("round_mode,lut", [(abi.ROUND_HALF_EVEN, False), (abi.ROUND_HALF_UP, True), (abi.ROUND_HALF_EVEN, True)])
def test_small_channel_conv_general_epilogue(round_mode, lut):
    """Half-even rounding takes the banded kernel's general epilogue; a fused table is applied in the staged epilogue."""
    case = cases.conv_case(seed=3, n=2, h=18, w=22, cin=16, cout=16, kh=3, kw=3, per_channel=True, round_mode=round_mode, lut=lut)
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), gpu_util.run_conv_oracle(case))


# Stride-1 windows over 32, 64 or 128 input channels: one input patch per tile, taps as shifted descriptor starts, the
# filter resident in shared memory (conv_patch_kernel in conv_tc.cu).
PATCH = [
    dict(n=2, h=80, w=80, cin=64, cout=64),                                   # the detector's 3x3 at its largest map
    dict(n=3, h=20, w=17, cin=128, cout=48),                                  # ragged in both directions, one 32-position row per image row
    dict(n=2, h=40, w=40, cin=128, cout=64),
    dict(n=1, h=33, w=70, cin=64, cout=128),
    dict(n=1, h=9, w=124, cin=64, cout=32),                                   # 128 positions per row
    dict(n=2, h=24, w=24, cin=64, cout=32, kh=5, kw=5, pad=(2, 2, 2, 2)),     # 25 resident taps
    dict(n=2, h=12, w=40, cin=64, cout=256, kh=1, kw=3, pad=(0, 0, 1, 1)),    # 256 columns: two epilogue parts per tile
    dict(n=2, h=15, w=15, cin=64, cout=192, pad=(0, 0, 0, 0)),                # no padding, 96-column parts (unswizzled staging)
    dict(n=5, h=7, w=7, cin=128, cout=16, pad=(1, 0, 0, 1)),                  # uneven pads, the smallest tile
    dict(n=2, h=80, w=80, cin=32, cout=16),                                   # 32-byte rows, three taps side by side in 48 columns
    dict(n=3, h=21, w=35, cin=32, cout=32, kh=2, kw=2, pad=(0, 1, 0, 1)),     # two taps side by side
    dict(n=2, h=13, w=31, cin=32, cout=96),                                   # 32-byte rows, taps one by one
    dict(n=2, h=11, w=45, cin=64, cout=48, kh=3, kw=4, pad=(1, 1, 1, 2)),     # four taps side by side
    dict(n=2, h=40, w=40, cin=128, cout=128),                                 # two taps in an N = 256 MMA, the third alone; 144 KB filter, rows out of registers
    dict(n=2, h=17, w=33, cin=64, cout=96),                                   # two taps side by side (192 columns), 48-column epilogue parts
    dict(n=1, h=20, w=31, cin=64, cout=64, kh=5, kw=5, pad=(2, 2, 2, 2)),     # four of five taps side by side
    dict(n=2, h=9, w=61, cin=32, cout=128),                                   # 32-byte rows, two taps side by side
]


@pytest.mark.parametrize("kw", PATCH, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items() if a != "pad"))
@pytest.mark.parametrize("act,per_channel,lut,round_mode", [(abi.ACT_RELU, True, False, abi.ROUND_HALF_UP), (abi.ACT_LINEAR, False, True, abi.ROUND_HALF_UP),
                                                            (abi.ACT_LINEAR, True, False, abi.ROUND_HALF_EVEN)])
def test_conv_one_patch_per_tile(kw, act, per_channel, lut, round_mode, monkeypatch):
    kw = dict(kw)
    kw.setdefault("kh", 3)
    kw.setdefault("kw", 3)
    case = cases.conv_case(seed=91, per_channel=per_channel, e_in=-7, e_out=-6, e_w=(-9, -7), act=act, lut=lut, round_mode=round_mode, **kw)
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 0
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    monkeypatch.setenv("ESPDL_B200_NO_TAP_STACK", "1")    # one MMA per tap instead of one per filter row
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    monkeypatch.setenv("ESPDL_B200_NO_CONV_PATCH", "1")   # the tap-per-box kernel gives the same bytes
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)


@pytest.mark.parametrize("m,k,n,act,direct", [(1000, 512, 256, abi.ACT_LINEAR, False), (700, 384, 256, abi.ACT_RELU, False), (300, 64, 48, abi.ACT_LINEAR, True),
                                              (260, 96, 200, abi.ACT_RELU, True)])
def test_fused_table_on_rows_that_leave_unstaged(m, k, n, act, direct, monkeypatch):
    """Long reductions with 256 columns keep their shared memory for load stages, so their rows leave out of registers;
    a fused table is then applied to the packed words of the one-add-one-shift form (ragged N in the last case)."""
    if direct:
        monkeypatch.setenv("ESPDL_B200_DIRECT_STORES", "1")
    case = cases.gemm_case(seed=m + k, m=m, k=k, n_out=n, per_channel=True, act=act, lut=True, e_in=-7, e_out=-5 + (k > 256), e_w=(-9, -7))
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 5
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)


@pytest.mark.parametrize("direct", [False, True])
def test_strided_conv_with_fused_table_and_256_columns(direct, monkeypatch):
    """3x3 stride 2 over 128 -> 256 channels with a fused table (the detector's downsampling conv): conv_tc_kernel without staging tiles."""
    if direct:
        monkeypatch.setenv("ESPDL_B200_DIRECT_STORES", "1")
    case = cases.conv_case(seed=15, n=2, h=20, w=22, cin=128, cout=256, kh=3, kw=3, stride=2, per_channel=True, lut=True, act=abi.ACT_LINEAR,
                           e_in=-7, e_out=-5, e_w=(-9, -7))
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 5
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)


# One table per output channel (espdl_conv_desc.lut_channel_stride): what a folded PRelu becomes.  Every conv kernel takes it
# in its general epilogue.
CHANNEL_TABLES = [
    dict(n=1, h=1, w=300, cin=64, cout=48, kh=1, kw=1, pad=(0, 0, 0, 0)),            # tile kernel
    dict(n=2, h=18, w=22, cin=32, cout=48),                                          # implicit GEMM, one MMA per tap
    dict(n=2, h=20, w=20, cin=64, cout=64),                                          # one patch per tile, stacked taps
    dict(n=2, h=18, w=22, cin=16, cout=16),                                          # banded filter
    dict(n=2, h=48, w=64, cin=3, cout=16, stride=2, pad=(0, 1, 0, 1)),               # first layer
    dict(n=2, h=19, w=23, cin=80, cout=80, depthwise=True),                          # depthwise, TMA patches
    dict(n=2, h=15, w=15, cin=24, cout=24, depthwise=True, stride=2, pad=(0, 1, 0, 1)),  # depthwise, narrow
    dict(n=2, h=9, w=9, cin=20, cout=12),                                            # CUDA-core conv
]


@pytest.mark.parametrize("kw", CHANNEL_TABLES, ids=lambda k: "-".join(f"{a}{b}" for a, b in k.items() if a != "pad"))
@pytest.mark.parametrize("act", [abi.ACT_LINEAR, abi.ACT_RELU])
def test_conv_with_per_channel_tables(kw, act):
    kw = dict(kw)
    kw.setdefault("kh", 3)
    kw.setdefault("kw", 3)
    case = cases.conv_case(seed=17, per_channel=True, e_in=-7, e_out=-6, e_w=(-9, -7), act=act, lut="channels", **kw)
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 5
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case), want)
    one = dict(case, lut=np.ascontiguousarray(case["lut"][:256]))        # the same conv with the first channel's table for all
    assert not np.array_equal(gpu_util.run_conv_oracle(one), want)


@pytest.mark.parametrize("m,k,n", [(3000, 192, 256), (1000, 256, 256), (700, 160, 960), (900, 144, 250)])
def test_wide_tiles_with_two_k_blocks_take_64_byte_stages(m, k, n, monkeypatch):
    """Reductions of two 128-byte blocks under 256-column tiles leave room for two or three stages only; the plan then
    halves the blocks (64-byte swizzle, more stages in flight).  Same bytes either way."""
    case = cases.gemm_case(seed=k + n, m=m, k=k, n_out=n, per_channel=True, e_in=-7, e_out=-5, e_w=(-9, -7), act=abi.ACT_RELU)
    want = gpu_util.run_conv_oracle(case)
    assert want.std() > 5
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
    monkeypatch.setenv("ESPDL_B200_NO_NARROW_K", "1")
    np.testing.assert_array_equal(gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05), want)
