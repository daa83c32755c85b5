#!/usr/bin/env python
"""Times ONE quantized conv / Gemm layer through the C ABI (espdl_b200_conv2d) on the current GPU.

    python esp-dl_b200/opbench.py --case pw32_192 [--iters 10] [--kernel auto|simt|tc]
    python esp-dl_b200/opbench.py --conv n,h,w,cin,cout,k,stride,depthwise(0/1),bits(8/16)
    python esp-dl_b200/opbench.py --list

Device memory, streams and events come from the library itself; between timed launches a buffer larger than the
L2 cache is overwritten so that every launch starts cold.  Prints one line per case: median milliseconds, integer
TOPS (2 ops per MAC) and GB/s over the algorithmic bytes (input + filter + output, each once).  The named cases are
layer shapes of MobileNetV2 at a batch that keeps the tensors well above the L2 size and a few GB at most, which is
also what a profiler capture of a single launch wants.
"""
import argparse
import ctypes as C
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import abi  # noqa: E402

CASES = {
    # name: n, h, w, cin, cout, k, stride, depthwise, bits
    "pw32_192": (64, 112, 112, 32, 192, 1, 1, 0, 8),
    "pw16_96": (64, 112, 112, 16, 96, 1, 1, 0, 8),
    "pw192_32": (64, 112, 112, 192, 32, 1, 1, 0, 8),
    "pw144_32": (256, 56, 56, 144, 32, 1, 1, 0, 8),
    "pw576_96": (256, 14, 14, 576, 96, 1, 1, 0, 8),
    "pw320_1280": (256, 7, 7, 320, 1280, 1, 1, 0, 8),
    "dw192": (32, 112, 112, 192, 192, 3, 1, 1, 8),
    "dw96_s2": (64, 112, 112, 96, 96, 3, 2, 1, 8),
    "dw384": (256, 14, 14, 384, 384, 3, 1, 1, 8),
    "stem": (64, 224, 224, 3, 32, 3, 2, 0, 8),
    "conv3x3_64": (64, 56, 56, 64, 64, 3, 1, 0, 8),
    "gemm_4096": (1, 1, 4096, 1024, 1024, 1, 1, 0, 8),
    "gemm_65536": (1, 1, 65536, 1024, 1024, 1, 1, 0, 8),
    "gemm_4096_s16": (1, 1, 4096, 1024, 1024, 1, 1, 0, 16),
}
KERNELS = {"auto": abi.KERNEL_AUTO, "simt": abi.KERNEL_SIMT, "tc": abi.KERNEL_TCGEN05}
FLUSH_BYTES = 256 << 20


class Dev:
    def __init__(self, device):
        self.L = abi.load()
        abi.check(self.L.espdl_b200_init(device), "init")
        self.bufs = []

    def put(self, arr):
        p = C.c_void_p()
        abi.check(self.L.espdl_b200_arena_alloc(max(arr.nbytes, 16), C.byref(p)), "arena_alloc")
        self.bufs.append(p)
        arr = np.ascontiguousarray(arr)
        abi.check(self.L.espdl_b200_upload(p, arr.ctypes.data_as(C.c_void_p), arr.nbytes, None), "upload")
        abi.check(self.L.espdl_b200_stream_sync(None), "sync")
        return p

    def empty(self, nbytes):
        p = C.c_void_p()
        abi.check(self.L.espdl_b200_arena_alloc(nbytes, C.byref(p)), "arena_alloc")
        self.bufs.append(p)
        return p

    def close(self):
        for p in self.bufs:
            self.L.espdl_b200_arena_free(p)
        self.bufs = []


def run_case(dev, spec, iters, warm, kernel):
    n, h, w, cin, cout, k, stride, dw, bits = spec
    L = dev.L
    pad = k // 2
    oh, ow = (h + 2 * pad - k) // stride + 1, (w + 2 * pad - k) // stride + 1
    es = bits // 8
    dt = np.int8 if bits == 8 else np.int16
    rng = np.random.default_rng(3)
    x = rng.integers(-128, 128, size=(n, h, w, cin), dtype=np.int8).astype(dt)
    wt = rng.integers(-127, 128, size=((k, k, cin) if dw else (cout, k, k, cin)), dtype=np.int8).astype(dt)
    bias = rng.integers(-4096, 4096, size=cout).astype(np.int32 if bits == 8 else np.int64)
    ew = rng.integers(-9, -5, size=cout).astype(np.int32)
    d = abi.ConvDesc()
    d.input, d.filter, d.bias, d.filter_exponents = dev.put(x), dev.put(wt), dev.put(bias), dev.put(ew)
    out_bytes = n * oh * ow * cout * es
    d.output = dev.empty(out_bytes)
    d.dtype = abi.DTYPE_INT8 if bits == 8 else abi.DTYPE_INT16
    d.n, d.in_h, d.in_w, d.in_c, d.out_h, d.out_w, d.out_c = n, h, w, cin, oh, ow, cout
    d.kh = d.kw = k
    d.stride_h = d.stride_w = stride
    d.dilation_h = d.dilation_w = 1
    d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = pad
    d.group = cin if dw else 1
    d.in_exponent, d.out_exponent, d.per_channel = -7, -5, 1
    d.activation, d.kernel = abi.ACT_RELU, kernel
    flush = dev.empty(FLUSH_BYTES)
    e0, e1 = C.c_void_p(), C.c_void_p()
    L.espdl_b200_event_create(C.byref(e0))
    L.espdl_b200_event_create(C.byref(e1))
    times = []
    for i in range(warm + iters):
        abi.check(L.espdl_b200_memset(flush, i & 0x7F, FLUSH_BYTES, None), "flush")
        L.espdl_b200_event_record(e0, None)
        abi.check(L.espdl_b200_conv2d(C.byref(d), None), "conv2d")
        L.espdl_b200_event_record(e1, None)
        ms = C.c_float()
        abi.check(L.espdl_b200_event_elapsed_ms(e0, e1, C.byref(ms)), "elapsed")
        if i >= warm:
            times.append(ms.value)
    abi.check(L.espdl_b200_stream_sync(None), "final sync")
    L.espdl_b200_event_destroy(e0)
    L.espdl_b200_event_destroy(e1)
    dev.close()
    ms = float(np.median(times))
    macs = n * oh * ow * cout * k * k * (1 if dw else cin)
    algo = x.nbytes + wt.nbytes + out_bytes
    return ms, 2 * macs / ms / 1e9, algo / ms / 1e6, algo


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", action="append", default=[])
    ap.add_argument("--conv", action="append", default=[])
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernel", default="auto", choices=sorted(KERNELS))
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    if a.list:
        for name, spec in CASES.items():
            print(name, spec)
        return
    todo = [(name, CASES[name]) for name in (a.case or ([] if a.conv else list(CASES)))]
    todo += [(c, tuple(int(v) for v in c.split(","))) for c in a.conv]
    dev = Dev(a.device)
    for name, spec in todo:
        ms, tops, gbs, algo = run_case(dev, spec, a.iters, a.warmup, KERNELS[a.kernel])
        print(f"{name:16s} {ms:9.4f} ms {tops:9.2f} TOPS {gbs:9.1f} GB/s  algorithmic_bytes={algo}", flush=True)


if __name__ == "__main__":
    main()
