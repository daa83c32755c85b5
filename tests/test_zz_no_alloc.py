"""The allocation-free int16 Gemm entry point (espdl_b200_gemm_s16_static) against the regular entry point.

Some callers of this library may not allocate device memory while they run (allocation-fenced real-time loops,
processes whose device memory is owned by a pool).  For them the int16 tensor-core Gemm keeps its scratch in a
fixed array inside the library.  Two calls in a row must give the regular entry point's bytes - the second call
finds the first call's leftovers in the shared array - and a problem beyond the fixed size must be refused."""
import ctypes as C

import numpy as np
import pytest

import cases
import gpu_util
from espdl_b200 import abi

pytestmark = pytest.mark.gpu


def run_static(case, expect=abi.OK):
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), filter=dev.upload(case["w"]), bias=dev.upload(case["b"]),
                    filter_exponents=dev.upload(case["ew"]), lut=None, output=dev.upload(np.full_like(case["out"], 0x55)))
        d = cases.conv_desc(case, ptrs)
        st = dev.lib.espdl_b200_gemm_s16_static(C.byref(d), None)
        assert st == expect, (st, dev.lib.espdl_b200_last_error())
        if expect != abi.OK:
            return None
        return dev.download(ptrs["output"], case["out"])


def test_static_scratch_matches_regular_entry_point_twice():
    first = cases.gemm_case(seed=71, dtype=abi.DTYPE_INT16, m=700, k=512, n_out=200, e_in=-14, e_w=(-15, -15), e_out=-12, wide=True,
                            bias_mag=1 << 20)
    second = cases.gemm_case(seed=72, dtype=abi.DTYPE_INT16, m=130, k=64, n_out=48, e_in=-13, e_w=(-15, -13), e_out=-11, wide=True,
                             per_channel=True, act=abi.ACT_RELU)
    for case in (first, second, first):
        want = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05)   # regular entry point, tolerance: exact
        got = run_static(case)
        np.testing.assert_array_equal(got, want)
        np.testing.assert_array_equal(got, gpu_util.run_conv_oracle(case))


def test_static_scratch_rejects_what_does_not_fit_or_does_not_apply():
    too_big = cases.gemm_case(seed=73, dtype=abi.DTYPE_INT16, m=8192, k=1024, n_out=64, e_in=-14, e_w=(-15, -15), e_out=-12)
    run_static(too_big, expect=abi.ERR_TOO_LARGE)       # 2*(8192*1024 + 64*1024) bytes > 16 MiB
    int8_case = cases.gemm_case(seed=74, m=64, k=64, n_out=32)
    run_static(int8_case, expect=abi.ERR_UNSUPPORTED)
    odd_k = cases.gemm_case(seed=75, dtype=abi.DTYPE_INT16, m=64, k=24, n_out=32, e_in=-14, e_w=(-15, -15), e_out=-12)
    run_static(odd_k, expect=abi.ERR_UNSUPPORTED)
