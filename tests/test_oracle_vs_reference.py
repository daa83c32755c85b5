"""Pins the plain-C oracle to the reference's own operators (oracle/_ref, built from the reference
sources by oracle/Makefile) on seeded inputs.  Skipped where the reference build is absent."""
import numpy as np
import pytest

import cases
import checkers
from espdl_b200 import abi

pytestmark = pytest.mark.skipif(not checkers.have_ref(), reason="oracle/_ref/libespdl_ref.so not built")


def run_conv_both(case, gemm=0):
    o = checkers.oracle()
    r = checkers.ref()
    out_o = case["out"].copy()
    case_o = dict(case, out=out_o)
    assert o.oracle_conv2d(cases.conv_desc(case_o)) == 0
    out_r = case["out"].copy()
    case_r = dict(case, out=out_r)
    assert r.ref_conv2d(cases.conv_desc(case_r), gemm) == 0
    return out_o, out_r


CONV_CASES = [
    dict(h=8, w=8, cin=16, cout=16, kh=3, kw=3),
    dict(h=9, w=7, cin=5, cout=7, kh=3, kw=3, stride=2),                        # odd sizes, stride 2
    dict(h=12, w=11, cin=8, cout=4, kh=5, kw=5, stride=2, pad=(2, 2, 2, 2)),    # 5x5 s2 (published operator shape family)
    dict(h=10, w=10, cin=6, cout=9, kh=3, kw=3, dil=2, pad=(2, 2, 2, 2)),       # dilation
    dict(h=7, w=9, cin=22, cout=33, kh=3, kw=3),                                # "unaligned" channels 22 -> 33
    dict(h=6, w=6, cin=16, cout=32, kh=1, kw=1, pad=(0, 0, 0, 0)),              # pointwise
    dict(h=8, w=8, cin=3, cout=8, kh=3, kw=3, stride=2, pad=(0, 1, 0, 1)),      # asymmetric pads
    dict(h=6, w=8, cin=4, cout=4, kh=3, kw=1, pad=(1, 1, 0, 0)),                # non-square filter
    dict(h=8, w=8, cin=16, cout=16, kh=3, kw=3, bias=False, act=abi.ACT_LINEAR),
    dict(h=5, w=5, cin=8, cout=8, kh=3, kw=3, e_in=-2, e_out=-12, e_w=(-3, -3)),  # negative shift (left shift + saturate)
    dict(n=3, h=6, w=6, cin=8, cout=8, kh=3, kw=3),                             # batch = repeated single-image calls
]


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("idx", range(len(CONV_CASES)))
def test_conv_matches_reference(idx, dtype):
    kw = dict(CONV_CASES[idx])
    if dtype == abi.DTYPE_INT16:
        kw.setdefault("e_in", -14)
        kw.setdefault("e_w", (-15, -13))
        kw.setdefault("e_out", -12)
    case = cases.conv_case(seed=100 + idx, dtype=dtype, **kw)
    out_o, out_r = run_conv_both(case)
    np.testing.assert_array_equal(out_o, out_r)
    assert out_o.std() > 0  # not degenerate (all saturated / all zero)


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("kw", [
    dict(h=8, w=8, cin=16, kh=3, kw=3),
    dict(h=9, w=11, cin=24, kh=3, kw=3, stride=2),
    dict(h=10, w=10, cin=25, kh=7, kw=7, stride=(1, 2), pad=(2, 2, 2, 2)),   # 7x7 s(1,2) p2 (published operator shape)
    dict(h=8, w=8, cin=7, kh=3, kw=3, dil=2, pad=(2, 2, 2, 2)),
    dict(n=2, h=6, w=7, cin=32, kh=3, kw=3, act=abi.ACT_LINEAR, bias=False),
])
def test_depthwise_matches_reference(kw, dtype):
    if dtype == abi.DTYPE_INT16:
        kw = dict(kw, e_in=-13, e_w=(-14, -12), e_out=-11)
    case = cases.conv_case(seed=7, dtype=dtype, depthwise=True, **kw)
    out_o, out_r = run_conv_both(case)
    np.testing.assert_array_equal(out_o, out_r)
    assert out_o.std() > 0


@pytest.mark.parametrize("dtype,m,k,n", [(abi.DTYPE_INT8, 33, 64, 17), (abi.DTYPE_INT8, 128, 96, 48),
                                         (abi.DTYPE_INT16, 40, 128, 24)])
def test_gemm_module_matches(dtype, m, k, n):
    kw = {}
    if dtype == abi.DTYPE_INT16:
        kw = dict(e_in=-14, e_w=(-15, -15), e_out=-12, wide=True)
    case = cases.gemm_case(seed=11, dtype=dtype, m=m, k=k, n_out=n, **kw)
    out_o, out_r = run_conv_both(case, gemm=1)
    np.testing.assert_array_equal(out_o, out_r)
    assert out_o.std() > 0


def run_elt_both(case):
    o, r = checkers.oracle(), checkers.ref()
    co, cr = dict(case, out=case["out"].copy()), dict(case, out=case["out"].copy())
    assert o.oracle_eltwise(cases.eltwise_desc(co)) == 0
    assert r.ref_eltwise(cases.eltwise_desc(cr)) == 0
    return co["out"], cr["out"]


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_ADD, abi.ELT_SUB, abi.ELT_MUL])
@pytest.mark.parametrize("shapes", [
    ((2, 5, 7, 16), None, None),
    ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 16)),     # per-channel broadcast
    ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 1)),      # scalar operand (mul_n_1 path)
    ((2, 5, 7, 16), (1, 1, 1, 1), (2, 5, 7, 16)),      # scalar first operand
    ((2, 5, 7, 16), (2, 1, 7, 1), (1, 5, 1, 16)),      # two-sided broadcast
    ((3, 20), (3, 1), (1, 20)),
    ((37,), None, None),
])
def test_binary_matches_reference(op, dtype, shapes):
    e = dict(e0=-5, e1=-6, eo=-8) if op == abi.ELT_MUL else dict(e0=-5, e1=-5, eo=-5)
    if dtype == abi.DTYPE_INT16 and op == abi.ELT_MUL:
        e = dict(e0=-12, e1=-13, eo=-11)
    case = cases.eltwise_case(op, seed=3, dtype=dtype, out_shape=shapes[0], in0_shape=shapes[1], in1_shape=shapes[2], **e)
    a, b = run_elt_both(case)
    np.testing.assert_array_equal(a, b)
    assert a.std() > 0


BROADCASTS = [
    ((2, 5, 7, 16), None, None),
    ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 16)),
    ((2, 5, 7, 16), (2, 5, 7, 16), (1, 1, 1, 1)),      # scalar divisor: a * (R / b), tabulated for int8
    ((2, 5, 7, 16), (1, 1, 1, 1), (2, 5, 7, 16)),      # scalar dividend: tabulated by divisor for int8
    ((2, 5, 7, 16), (2, 5, 7, 1), (2, 5, 7, 16)),      # dividend broadcast along the innermost axis
    ((2, 5, 7, 16), (2, 5, 7, 16), (2, 5, 7, 1)),      # divisor broadcast along the innermost axis
    ((2, 5, 7, 16), (2, 1, 7, 1), (1, 5, 1, 16)),
    ((2, 5, 7, 1), (2, 5, 7, 1), (1, 5, 1, 1)),
    ((3, 20), (3, 1), (1, 20)),
    ((37,), None, None),
    ((1,), None, None),
]


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_MAX, abi.ELT_MIN, abi.ELT_DIV, abi.ELT_MOD])
@pytest.mark.parametrize("shapes", BROADCASTS)
def test_max_min_div_mod_match_reference(op, dtype, shapes):
    e = dict(e0=-5, e1=-5, eo=-5)
    if op == abi.ELT_DIV:
        e = dict(e0=-5, e1=-4, eo=-6) if dtype == abi.DTYPE_INT8 else dict(e0=-12, e1=-9, eo=-10)
    if op == abi.ELT_MOD:
        e = dict(e0=-5, e1=-6, eo=-6) if dtype == abi.DTYPE_INT8 else dict(e0=-12, e1=-13, eo=-11)
    case = cases.eltwise_case(op, seed=23, dtype=dtype, out_shape=shapes[0], in0_shape=shapes[1], in1_shape=shapes[2], **e)
    a, b = run_elt_both(case)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op", [abi.ELT_GREATER, abi.ELT_GREATER_EQUAL, abi.ELT_EQUAL, abi.ELT_LESS, abi.ELT_LESS_EQUAL])
@pytest.mark.parametrize("shapes", BROADCASTS[:3] + BROADCASTS[6:10])
def test_comparisons_match_reference(op, dtype, shapes):
    case = cases.eltwise_case(op, seed=29, in_dtype=dtype, out_dtype=abi.DTYPE_BOOL, out_shape=shapes[0], in0_shape=shapes[1],
                              in1_shape=shapes[2], e0=-5, e1=-5, eo=0)
    a, b = run_elt_both(case)
    np.testing.assert_array_equal(a, b)
    assert set(np.unique(a)) <= {0, 1}


@pytest.mark.parametrize("idt,odt,e0,eo", [
    (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -2), (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -6), (abi.DTYPE_INT8, abi.DTYPE_INT8, -4, -4),
    (abi.DTYPE_INT16, abi.DTYPE_INT16, -10, -7), (abi.DTYPE_INT16, abi.DTYPE_INT8, -10, -5), (abi.DTYPE_INT8, abi.DTYPE_INT16, -5, -10),
    (abi.DTYPE_INT16, abi.DTYPE_INT8, -7, -7), (abi.DTYPE_INT8, abi.DTYPE_INT16, -7, -7),
    (abi.DTYPE_FLOAT, abi.DTYPE_INT8, 0, -4), (abi.DTYPE_FLOAT, abi.DTYPE_INT16, 0, -11),
    (abi.DTYPE_INT8, abi.DTYPE_FLOAT, -4, 0), (abi.DTYPE_INT16, abi.DTYPE_FLOAT, -9, 0),
])
def test_requantize_matches_reference(idt, odt, e0, eo):
    case = cases.eltwise_case(abi.ELT_REQUANTIZE, seed=5, in_dtype=idt, out_dtype=odt, out_shape=(3, 4, 5, 8), e0=e0, eo=eo)
    a, b = run_elt_both(case)
    np.testing.assert_array_equal(a, b)


@pytest.mark.parametrize("op,dtype,kw", [
    (abi.ELT_LUT, abi.DTYPE_INT8, {}),
    (abi.ELT_LUT, abi.DTYPE_INT16, dict(eo=-4, lut_shift=5)),   # the 2049-entry table with nearest-index rounding
    (abi.ELT_LUT, abi.DTYPE_INT16, dict(eo=-4, lut_shift=3)),
    (abi.ELT_CLIP, abi.DTYPE_INT8, dict(e0=-4, eo=-4, clip=(0, 96))),
    (abi.ELT_CLIP, abi.DTYPE_INT8, dict(e0=-4, eo=-5, clip=(0, 96))),
    (abi.ELT_CLIP, abi.DTYPE_INT16, dict(e0=-10, eo=-9, clip=(-3000, 6000))),
    (abi.ELT_RELU, abi.DTYPE_INT8, dict(e0=-4, eo=-4)),
    (abi.ELT_RELU, abi.DTYPE_INT8, dict(e0=-4, eo=-6)),
    (abi.ELT_RELU, abi.DTYPE_INT16, dict(e0=-9, eo=-7)),
    (abi.ELT_PRELU, abi.DTYPE_INT8, dict(e0=-4, e1=-7, eo=-4)),
    (abi.ELT_PRELU, abi.DTYPE_INT16, dict(e0=-10, e1=-15, eo=-10)),
])
def test_unary_matches_reference(op, dtype, kw):
    case = cases.eltwise_case(op, seed=9, dtype=dtype, out_shape=(1, 4, 6, 24), **kw)
    a, b = run_elt_both(case)
    np.testing.assert_array_equal(a, b)
    assert a.std() > 0


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8, abi.DTYPE_INT16])
@pytest.mark.parametrize("op,kw", [
    (abi.POOL_MAX, dict(kh=3, kw=3, stride=2, pad=(1, 1, 1, 1))),
    (abi.POOL_MAX, dict(h=20, w=20, c=16, kh=5, kw=5, stride=1, pad=(2, 2, 2, 2))),   # SPPF-style 5x5 s1 p2
    (abi.POOL_MAX, dict(kh=2, kw=2, stride=2, pad=(0, 0, 0, 0))),
    (abi.POOL_AVG, dict(kh=2, kw=2, stride=2, pad=(0, 0, 0, 0))),
    (abi.POOL_AVG, dict(kh=3, kw=3, stride=1, pad=(0, 0, 0, 0), e_out=-4)),
    (abi.POOL_GLOBAL_AVG, dict(h=7, w=7, c=40, e_in=-4, e_out=-5)),
    (abi.POOL_GLOBAL_AVG, dict(h=7, w=7, c=1280, e_in=-5, e_out=-5)),
])
def test_pool_matches_reference(op, kw, dtype):
    case = cases.pool_case(op, seed=13, dtype=dtype, **kw)
    co, cr = dict(case, out=case["out"].copy()), dict(case, out=case["out"].copy())
    assert checkers.oracle().oracle_pool(cases.pool_desc(co)) == 0
    assert checkers.ref().ref_pool(cases.pool_desc(cr)) == 0
    np.testing.assert_array_equal(co["out"], cr["out"])


@pytest.mark.parametrize("dtype", [abi.DTYPE_INT8])  # the reference's int16 resize is an empty function
@pytest.mark.parametrize("kw", [dict(scale=(2.0, 2.0)), dict(scale=(2.0, 2.0), e_in=-5, e_out=-4), dict(scale=(2.0, 2.0), e_in=-5, e_out=-6),
                                dict(scale=(3.0, 2.0)), dict(scale=(1.5, 2.5), h=8, w=8), dict(scale=(0.5, 0.5), h=8, w=10)])
def test_resize_matches_reference(kw, dtype):
    case = cases.resize_case(seed=17, dtype=dtype, **kw)
    co, cr = dict(case, out=case["out"].copy()), dict(case, out=case["out"].copy())
    assert checkers.oracle().oracle_resize(cases.resize_desc(co)) == 0
    assert checkers.ref().ref_resize(cases.resize_desc(cr)) == 0
    np.testing.assert_array_equal(co["out"], cr["out"])


LINEAR_RESIZE = [dict(scale=(2.0, 2.0), mode=1), dict(scale=(2.0, 2.0), mode=2), dict(scale=(2.0, 2.0), e_in=-5, e_out=-4, mode=1),
          dict(scale=(1.5, 2.5), h=8, w=8, e_in=-5, e_out=-6, mode=1), dict(scale=(0.5, 0.5), h=8, w=10, mode=1),
          dict(scale=(3.0, 1.7), h=7, w=9, c=5, mode=2), dict(scale=(1.0, 2.0), h=1, w=12, c=24, mode=1),
          dict(scale=(1.0, 3.5), h=1, w=9, c=7, e_in=-6, e_out=-5, mode=2), dict(scale=(4.0, 4.0), n=3, h=13, w=11, c=32, mode=1)]


@pytest.mark.parametrize("kw", LINEAR_RESIZE)
def test_linear_resize_matches_reference(kw):
    """Linear resize (half-pixel and align_corners coordinates, 2-D and along w only) against the reference's Resize module."""
    case = cases.resize_case(seed=19, **kw)
    co, cr = dict(case, out=case["out"].copy()), dict(case, out=case["out"].copy())
    assert checkers.oracle().oracle_resize(cases.resize_desc(co)) == 0
    assert checkers.ref().ref_resize(cases.resize_desc(cr)) == 0
    assert co["out"].any()
    np.testing.assert_array_equal(co["out"], cr["out"])


@pytest.mark.parametrize("e_in,rows,length", [(-4, 6, 400), (-3, 3, 37), (-6, 5, 64)])
def test_softmax_matches_reference(e_in, rows, length):
    rng = np.random.default_rng(19)
    x = rng.integers(-128, 128, size=(rows, length), dtype=np.int8)
    table = np.zeros(256, dtype=np.float32)
    checkers.oracle().oracle_softmax_table(table.ctypes.data, e_in)
    yo = np.zeros((rows, length), dtype=np.float32)
    yr = np.zeros((rows, length), dtype=np.float32)
    assert checkers.oracle().oracle_softmax(cases.softmax_desc(x.ctypes.data, yo.ctypes.data, table.ctypes.data, rows, length, abi.DTYPE_FLOAT, 0)) == 0
    assert checkers.ref().ref_softmax(cases.softmax_desc(x.ctypes.data, yr.ctypes.data, None, rows, length, abi.DTYPE_FLOAT, 0), e_in) == 0
    np.testing.assert_array_equal(yo.view(np.uint32), yr.view(np.uint32))  # bit-identical floats


def test_concat_copy_matches_reference():
    import ctypes as C
    rng = np.random.default_rng(23)
    a = rng.integers(-128, 128, size=(2, 3, 4, 8), dtype=np.int8)
    b = rng.integers(-128, 128, size=(2, 3, 4, 24), dtype=np.int8)
    out_r = np.zeros((2, 3, 4, 32), dtype=np.int8)
    sa = (C.c_int * 4)(*a.shape)
    sb = (C.c_int * 4)(*b.shape)
    assert checkers.ref().ref_concat2(a.ctypes.data, b.ctypes.data, out_r.ctypes.data, sa, sb, 4, 3) == 0
    out_o = np.zeros_like(out_r)
    # channel concat = two strided copies into slices of the output pixel
    o = checkers.oracle()
    assert o.oracle_copy(cases.copy_desc(a.ctypes.data, out_o.ctypes.data, 1, (24, 8), (8, 1), (32, 1))) == 0
    assert o.oracle_copy(cases.copy_desc(b.ctypes.data, out_o.ctypes.data + 8, 1, (24, 24), (24, 1), (32, 1))) == 0
    np.testing.assert_array_equal(out_o, out_r)


@pytest.mark.parametrize("sa,sb", [((3, 16), (16, 5)), ((16,), (16, 7)), ((4, 32), (32,)), ((2, 3, 16), (2, 16, 5)), ((2, 3, 16), (16, 5)),
                                   ((2, 2, 3, 8), (2, 2, 8, 4)), ((1, 2, 3, 8), (2, 1, 8, 4)), ((5, 24), (24, 9))])
@pytest.mark.parametrize("relu", [0, 1])
def test_matmul_matches_reference(sa, sb, relu):
    """MatMul of two activations: the restatement (input1's memory read as [N][K], one Gemm per broadcast slice) against
    the reference's own MatMul module compiled for the host."""
    import ctypes as C
    import graph_oracle
    rng = np.random.default_rng(31)
    a = rng.integers(-128, 128, size=sa, dtype=np.int8)
    b = rng.integers(-128, 128, size=sb, dtype=np.int8)
    e_a, e_b, e_out = -5, -6, -3
    want_shape = np.matmul(np.zeros(sa), np.zeros(sb)).shape or (1,)
    out_r = np.zeros(want_shape, dtype=np.int8)
    assert checkers.ref().ref_matmul(a.ctypes.data, (C.c_int * len(sa))(*sa), len(sa), e_a, b.ctypes.data, (C.c_int * len(sb))(*sb), len(sb), e_b,
                                     out_r.ctypes.data, e_out, abi.DTYPE_INT8, relu) == 0
    got = graph_oracle.matmul(checkers.oracle(), a, b, e_a, e_b, e_out, abi.DTYPE_INT8, abi.ACT_RELU if relu else abi.ACT_LINEAR, abi.ROUND_HALF_UP)
    np.testing.assert_array_equal(got.reshape(out_r.shape), out_r)
    assert out_r.std() > 0
