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


def free_bytes(lib):
    free = C.c_size_t()
    abi.check(lib.espdl_b200_mem_info(C.byref(free), None), "mem_info")
    return free.value


def run_static(case, expect=abi.OK, calls=1, edit=None):
    """Runs the entry point `calls` times on the same buffers; returns (output, free device memory seen after each
    call, with the stream drained)."""
    with gpu_util.DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), filter=dev.upload(case["w"]), bias=dev.upload(case["b"]),
                    filter_exponents=dev.upload(case["ew"]), lut=None, output=dev.upload(np.full_like(case["out"], 0x55)))
        d = cases.conv_desc(case, ptrs)
        if edit:
            edit(d)
        free = []
        for _ in range(calls):
            st = dev.lib.espdl_b200_gemm_s16_static(C.byref(d), None)
            assert st == expect, (st, dev.lib.espdl_b200_last_error())
            if expect == abi.OK:
                abi.check(dev.lib.espdl_b200_stream_sync(None), "sync")
            free.append(free_bytes(dev.lib))
        if expect != abi.OK:
            return None, free
        return dev.download(ptrs["output"], case["out"]), free


def test_static_scratch_matches_regular_entry_point_twice():
    first = cases.gemm_case(seed=71, dtype=abi.DTYPE_INT16, m=700, k=512, n_out=200, e_in=-14, e_w=(-15, -15), e_out=-12, wide=True,
                            bias_mag=1 << 20)
    second = cases.gemm_case(seed=72, dtype=abi.DTYPE_INT16, m=130, k=64, n_out=48, e_in=-13, e_w=(-15, -13), e_out=-11, wide=True,
                             per_channel=True, act=abi.ACT_RELU)
    for case in (first, second, first):
        want = gpu_util.run_conv_gpu(case, kernel=abi.KERNEL_TCGEN05)   # regular entry point, tolerance: exact
        got, _ = run_static(case)
        np.testing.assert_array_equal(got, want)
        np.testing.assert_array_equal(got, gpu_util.run_conv_oracle(case))


def test_static_scratch_calls_leave_free_device_memory_unchanged():
    """After the warm-up call (which loads the kernels and looks up the array's address) further calls must not change
    the device's free memory: nothing is allocated, nothing is freed."""
    case = cases.gemm_case(seed=76, dtype=abi.DTYPE_INT16, m=512, k=256, n_out=96, e_in=-14, e_w=(-15, -15), e_out=-12, wide=True)
    run_static(case)                                   # warm-up, outside the measured region
    got, free = run_static(case, calls=4)
    assert len(set(free)) == 1, free
    np.testing.assert_array_equal(got, gpu_util.run_conv_oracle(case))


def test_static_scratch_rejects_what_does_not_fit_or_does_not_apply():
    too_big = cases.gemm_case(seed=73, dtype=abi.DTYPE_INT16, m=8192, k=1024, n_out=64, e_in=-14, e_w=(-15, -15), e_out=-12)
    run_static(too_big, expect=abi.ERR_TOO_LARGE)       # 2*(8192*1024 + 64*1024) bytes > 16 MiB
    int8_case = cases.gemm_case(seed=74, m=64, k=64, n_out=32)
    run_static(int8_case, expect=abi.ERR_UNSUPPORTED)
    odd_k = cases.gemm_case(seed=75, dtype=abi.DTYPE_INT16, m=64, k=24, n_out=32, e_in=-14, e_w=(-15, -15), e_out=-12)
    run_static(odd_k, expect=abi.ERR_UNSUPPORTED)


def test_static_scratch_checks_the_descriptor_before_launching():
    """Descriptors the regular entry point refuses are refused here too, on the host, before any kernel could read a
    null exponent array or run past the input."""
    def ok_case():
        return cases.gemm_case(seed=77, dtype=abi.DTYPE_INT16, m=64, k=64, n_out=32, e_in=-14, e_w=(-15, -15), e_out=-12)

    def per_channel_without_exponents(d):
        d.per_channel, d.filter_exponents = 1, None

    def mismatched_width(d):
        d.out_w = d.out_w + 8

    def negative_batch(d):
        d.n = -1

    def with_residual(d):
        d.residual = d.output

    launches = gpu_util.lib().espdl_b200_launch_count()
    run_static(ok_case(), expect=abi.ERR_INVALID_ARG, edit=per_channel_without_exponents)
    run_static(ok_case(), expect=abi.ERR_INVALID_ARG, edit=mismatched_width)
    run_static(ok_case(), expect=abi.ERR_INVALID_ARG, edit=negative_batch)
    run_static(ok_case(), expect=abi.ERR_UNSUPPORTED, edit=with_residual)
    assert gpu_util.lib().espdl_b200_launch_count() == launches
