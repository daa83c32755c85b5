"""Pad (constant / edge / reflect): the oracle against the reference's own module compiled for the host, the CUDA
kernel against the oracle."""
import ctypes as C

import numpy as np
import pytest

import checkers
from espdl_b200 import abi

CASES = [((1, 5, 6, 8), (0, 1, 2, 0), (0, 2, 1, 0)), ((2, 9, 4), (1, 0, 3), (0, 2, 1)), ((7, 11), (2, 3), (4, 1)), ((13,), (5,), (2,)),
         ((2, 6, 6, 16), (0, 1, 1, 0), (0, 1, 1, 0))]


def make(shape, begin, end, mode, es, seed, inp=None, out=None):
    t = np.int8 if es == 1 else np.int16
    info = np.iinfo(t)
    x = np.random.default_rng(seed).integers(info.min, info.max + 1, size=shape, dtype=t)
    oshape = [s + b + e for s, b, e in zip(shape, begin, end)]
    y = np.zeros(oshape, dtype=t)
    d = abi.PadDesc()
    d.elem_size, d.ndim, d.mode, d.constant = es, len(shape), mode, -3
    for i in range(len(shape)):
        d.shape[i], d.pad_begin[i], d.pad_end[i] = shape[i], begin[i], end[i]
    d.input = x.ctypes.data if inp is None else inp
    d.output = y.ctypes.data if out is None else out
    return d, x, y


ALL = [(c, m, es) for c in CASES for m in range(3) for es in (1, 2)]


@pytest.mark.parametrize("case,mode,es", ALL)
def test_oracle_matches_reference_and_numpy(case, mode, es):
    shape, begin, end = case
    d, x, got = make(shape, begin, end, mode, es, 5)
    assert checkers.oracle().oracle_pad(C.byref(d)) == 0
    widths = list(zip(begin, end))
    want = np.pad(x, widths, mode=["constant", "edge", "reflect"][mode], **({"constant_values": -3} if mode == 0 else {}))
    np.testing.assert_array_equal(got, want)
    d2, _, ref = make(shape, begin, end, mode, es, 5)
    assert checkers.ref().ref_pad(C.byref(d2)) == 0
    np.testing.assert_array_equal(ref, want)


@pytest.mark.gpu
@pytest.mark.parametrize("case,mode,es", ALL)
def test_gpu_matches_oracle(case, mode, es):
    import gpu_util
    shape, begin, end = case
    d, x, want = make(shape, begin, end, mode, es, 6)
    assert checkers.oracle().oracle_pad(C.byref(d)) == 0
    with gpu_util.DeviceBuffers() as dev:
        out = dev.upload(np.full_like(want, 0x55))
        dg, _, _ = make(shape, begin, end, mode, es, 6, inp=dev.upload(x), out=out)
        abi.check(dev.lib.espdl_b200_pad(C.byref(dg), None), "pad")
        got = dev.download(out, want)
    np.testing.assert_array_equal(got, want)
