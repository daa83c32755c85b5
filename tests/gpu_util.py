"""Helpers for the GPU parity tests: device buffers through the C ABI itself (no torch on this path)."""
import ctypes as C

import numpy as np

from espdl_b200 import abi

_initialised = False


def lib():
    global _initialised
    L = abi.load()
    if not _initialised:
        abi.check(L.espdl_b200_init(0), "espdl_b200_init")
        _initialised = True
    return L


class DeviceBuffers:
    """Uploads numpy arrays, hands out device addresses, frees everything on exit."""

    def __init__(self):
        self.lib = lib()
        self.ptrs = []

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        for p in self.ptrs:
            self.lib.espdl_b200_arena_free(p)
        self.ptrs = []

    def alloc(self, nbytes):
        p = C.c_void_p()
        abi.check(self.lib.espdl_b200_arena_alloc(max(int(nbytes), 16), C.byref(p)), "arena_alloc")
        self.ptrs.append(p)
        return p.value

    def upload(self, arr):
        if arr is None:
            return None
        arr = np.ascontiguousarray(arr)
        p = self.alloc(arr.nbytes)
        abi.check(self.lib.espdl_b200_upload(p, arr.ctypes.data, arr.nbytes, None), "upload")
        abi.check(self.lib.espdl_b200_stream_sync(None), "sync")
        return p

    def download(self, ptr, like):
        out = np.empty_like(like)
        abi.check(self.lib.espdl_b200_stream_sync(None), "sync")
        abi.check(self.lib.espdl_b200_download(out.ctypes.data, ptr, out.nbytes, None), "download")
        abi.check(self.lib.espdl_b200_stream_sync(None), "sync")
        return out


def run_conv_gpu(case, kernel=abi.KERNEL_AUTO, expect=abi.OK):
    import cases
    with DeviceBuffers() as dev:
        ptrs = dict(input=dev.upload(case["x"]), filter=dev.upload(case["w"]), bias=dev.upload(case["b"]),
                    filter_exponents=dev.upload(case["ew"]), lut=dev.upload(case["lut"]), residual=dev.upload(case.get("res")),
                    output=dev.upload(np.full_like(case["out"], 0x55)))
        d = cases.conv_desc(dict(case, kernel=kernel), ptrs)
        st = dev.lib.espdl_b200_conv2d(C.byref(d), None)
        if expect != abi.OK:
            assert st == expect
            return None
        abi.check(st, "espdl_b200_conv2d")
        return dev.download(ptrs["output"], case["out"])


def run_conv_oracle(case):
    import cases
    import checkers
    out = np.full_like(case["out"], 0x55)
    assert checkers.oracle().oracle_conv2d(cases.conv_desc(dict(case, out=out))) == 0
    return out


def run_block_oracle(case):
    """The block as the reference runs it: one conv per node, every intermediate tensor in memory."""
    import cases
    import checkers
    h = case["x"]
    if case["expand"] is not None:
        c1 = dict(case["expand"], x=h, out=np.zeros_like(case["expand"]["out"]))
        assert checkers.oracle().oracle_conv2d(cases.conv_desc(c1)) == 0
        h = np.minimum(c1["out"], case["clip1"]).astype(np.int8)
    c2 = dict(case["dw"], x=h, out=np.zeros_like(case["dw"]["out"]))
    assert checkers.oracle().oracle_conv2d(cases.conv_desc(c2)) == 0
    h = np.minimum(c2["out"], case["clipdw"]).astype(np.int8)
    c3 = dict(case["project"], x=h, out=np.zeros_like(case["project"]["out"]))
    if case["residual"]:
        c3["res"] = np.ascontiguousarray(case["x"])
    assert checkers.oracle().oracle_conv2d(cases.conv_desc(c3)) == 0
    return c3["out"]


def run_block_gpu(case, expect=abi.OK):
    import cases
    with DeviceBuffers() as dev:
        x = dev.upload(case["x"])
        ptrs = dict(input=x, output=dev.upload(np.full_like(case["out"], 0x55)), residual=x if case["residual"] else None)
        for name, key in (("expand", "expand"), ("dw", "dw"), ("project", "project")):
            c = case[key]
            if c is None:
                continue
            ptrs[name + "_filter"] = dev.upload(c["w"])
            ptrs[name + "_bias"] = dev.upload(c["b"])
            ptrs[name + "_filter_exponents"] = dev.upload(c["ew"])
        d = cases.block_desc(case, ptrs)
        st = dev.lib.espdl_b200_fused_block(C.byref(d), None)
        if expect != abi.OK:
            assert st == expect
            return None
        abi.check(st, "espdl_b200_fused_block")
        abi.check(dev.lib.espdl_b200_stream_sync(None), "stream_sync")
        return dev.download(ptrs["output"], case["out"])
