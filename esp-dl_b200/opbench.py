#!/usr/bin/env python
"""Times ONE quantized conv / Gemm layer through the C ABI (espdl_b200_conv2d) on the current GPU.

    python esp-dl_b200/opbench.py --case pw32_192 [--iters 10] [--kernel auto|simt|tc]
    python esp-dl_b200/opbench.py --conv n,h,w,cin,cout,k,stride,depthwise(0/1),bits(8/16)
    python esp-dl_b200/opbench.py --block n,h,w,cin,hidden,cout,stride      (or a name from BLOCKS)
    python esp-dl_b200/opbench.py --mem add|lut|requant|clip|mul|maxpool|resize2|rmsnorm|layernorm|gather|transpose   (or all)
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
BLOCKS = {
    # inverted-residual blocks: n, h, w, cin, hidden, cout, stride  (hidden == cin and no expand conv when hidden = 0)
    "block_c3": (256, 112, 112, 32, 192, 32, 1),      # the benchmark's block configuration
    "block_16_96_24": (256, 112, 112, 16, 96, 24, 2),
    "block_32_192_64": (512, 28, 28, 32, 192, 64, 2),
    "block_64_384_64": (1024, 14, 14, 64, 384, 64, 1),
    "block_96_576_96": (1024, 14, 14, 96, 576, 96, 1),
    "block_160_960_160": (1024, 7, 7, 160, 960, 160, 1),
    "block_dw32_16": (256, 112, 112, 32, 0, 16, 1),
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


def _time(L, flush, fn, iters, warm):
    e0, e1 = C.c_void_p(), C.c_void_p()
    L.espdl_b200_event_create(C.byref(e0))
    L.espdl_b200_event_create(C.byref(e1))
    times = []
    for i in range(warm + iters):
        abi.check(L.espdl_b200_memset(flush, i & 0x7F, FLUSH_BYTES, None), "flush")
        L.espdl_b200_event_record(e0, None)
        fn()
        L.espdl_b200_event_record(e1, None)
        ms = C.c_float()
        abi.check(L.espdl_b200_event_elapsed_ms(e0, e1, C.byref(ms)), "elapsed")
        if i >= warm:
            times.append(ms.value)
    abi.check(L.espdl_b200_stream_sync(None), "final sync")
    L.espdl_b200_event_destroy(e0)
    L.espdl_b200_event_destroy(e1)
    return float(np.median(times))


def run_block(dev, spec, iters, warm):
    """One inverted-residual block: the fused launch (espdl_b200_fused_block) and the same block as separate
    convolutions with the Add folded into the project conv, which is how the model runs it without the fusion."""
    n, h, w, cin, chid, cout, stride = spec
    L = dev.L
    expand = chid > 0
    chid = chid or cin
    oh, ow = (h + 2 - 3) // stride + 1, (w + 2 - 3) // stride + 1
    residual = stride == 1 and cin == cout
    rng = np.random.default_rng(4)
    x = dev.put(rng.integers(-128, 128, size=(n, h, w, cin), dtype=np.int8))
    hid = dev.empty(n * h * w * chid)
    hid2 = dev.empty(n * oh * ow * chid)
    out = dev.empty(n * oh * ow * cout)

    def params(co, shape):
        return (dev.put(rng.integers(-127, 128, size=shape, dtype=np.int8)), dev.put(rng.integers(-1024, 1024, size=co).astype(np.int32)),
                dev.put(rng.integers(-11, -8, size=co).astype(np.int32)))
    w1 = params(chid, (chid, cin)) if expand else (None, None, None)
    w2 = params(chid, (3, 3, chid))
    w3 = params(cout, (cout, chid))
    b = abi.BlockDesc()
    b.input, b.output, b.residual = x, out, (x if residual else None)
    b.expand_filter, b.expand_bias, b.expand_filter_exponents = w1
    b.dw_filter, b.dw_bias, b.dw_filter_exponents = w2
    b.project_filter, b.project_bias, b.project_filter_exponents = w3
    b.dtype, b.n, b.in_h, b.in_w, b.in_c, b.hidden_c, b.out_h, b.out_w, b.out_c = abi.DTYPE_INT8, n, h, w, cin, chid, oh, ow, cout
    b.stride, b.pad_top, b.pad_left = stride, 1, 1
    b.in_exponent, b.expand_exponent, b.dw_exponent, b.out_exponent = -5, -6, -6, -5
    b.per_channel, b.expand_activation, b.dw_activation, b.project_activation = 7, abi.ACT_RELU, abi.ACT_RELU, abi.ACT_LINEAR
    b.expand_clip_max = b.dw_clip_max = 127

    def conv(inp, outp, prm, ih, iw, ci, co, k, s, dw, e_in, e_out, act, res=None):
        d = abi.ConvDesc()
        d.input, d.output, d.filter, d.bias, d.filter_exponents, d.residual = inp, outp, prm[0], prm[1], prm[2], res
        d.dtype, d.n, d.in_h, d.in_w, d.in_c = abi.DTYPE_INT8, n, ih, iw, ci
        d.out_h, d.out_w, d.out_c = (ih + 2 * (k // 2) - k) // s + 1, (iw + 2 * (k // 2) - k) // s + 1, co
        d.kh = d.kw = k
        d.stride_h = d.stride_w = s
        d.dilation_h = d.dilation_w = 1
        d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = k // 2
        d.group = ci if dw else 1
        d.in_exponent, d.out_exponent, d.per_channel, d.activation = e_in, e_out, 1, act
        return d
    chain = []
    if expand:
        chain.append(conv(x, hid, w1, h, w, cin, chid, 1, 1, 0, -5, -6, abi.ACT_RELU))
    chain.append(conv(hid if expand else x, hid2, w2, h, w, chid, chid, 3, stride, 1, -6 if expand else -5, -6, abi.ACT_RELU))
    chain.append(conv(hid2, out, w3, oh, ow, chid, cout, 1, 1, 0, -6, -5, abi.ACT_LINEAR, x if residual else None))
    flush = dev.empty(FLUSH_BYTES)

    def fused():
        abi.check(L.espdl_b200_fused_block(C.byref(b), None), "fused_block")

    def separate():
        for d in chain:
            abi.check(L.espdl_b200_conv2d(C.byref(d), None), "conv2d")
    ms_f = _time(L, flush, fused, iters, warm)
    ms_s = _time(L, flush, separate, iters, warm)
    dev.close()
    macs = n * (h * w * cin * chid * (1 if expand else 0) + oh * ow * chid * 9 + oh * ow * chid * cout)
    algo = n * (h * w * cin + oh * ow * cout * (2 if residual else 1))  # input once, output once (+ the residual read)
    return ms_f, ms_s, 2 * macs / ms_f / 1e9, algo / ms_f / 1e6, algo


MEM_CASES = ("add", "lut", "requant", "clip", "mul", "maxpool", "resize2", "rmsnorm", "layernorm", "gather", "transpose")


def run_mem(dev, name, iters, warm):
    """One bandwidth-bound kernel on an int8 tensor of 256x56x56x96 (77 MB, below L2 only after the flush): median ms and
    GB/s over the algorithmic bytes (every input and output once)."""
    L = dev.L
    rng = np.random.default_rng(5)
    n, h, w, c = 256, 56, 56, 96
    x = rng.integers(-128, 128, size=(n, h, w, c), dtype=np.int8)
    px = dev.put(x)
    algo = 2 * x.nbytes
    if name in ("add", "mul", "lut", "requant", "clip"):
        d = abi.EltwiseDesc()
        d.op = {"add": abi.ELT_ADD, "mul": abi.ELT_MUL, "lut": abi.ELT_LUT, "requant": abi.ELT_REQUANTIZE, "clip": abi.ELT_CLIP}[name]
        d.input0, d.output = px, dev.empty(x.nbytes)
        if name in ("add", "mul"):
            d.input1 = dev.put(rng.integers(-128, 128, size=x.shape, dtype=np.int8))
            algo = 3 * x.nbytes
        elif name == "lut":
            d.input1 = dev.put(rng.integers(-128, 128, size=256, dtype=np.int8))
        d.in_dtype = d.out_dtype = abi.DTYPE_INT8
        d.ndim = 1
        d.out_shape[0] = d.in0_shape[0] = x.size
        d.in1_shape[0] = x.size if name in ("add", "mul") else 1
        d.in0_exponent, d.in1_exponent, d.out_exponent = (-5, -5, -5) if name == "add" else (-5, -6, -7)
        d.clip_lo, d.clip_hi = 0, 96
        fn = lambda: abi.check(L.espdl_b200_eltwise(C.byref(d), None), name)
    elif name in ("maxpool", "resize2"):
        if name == "maxpool":
            d = abi.PoolDesc()
            d.op, d.dtype = abi.POOL_MAX, abi.DTYPE_INT8
            d.n, d.in_h, d.in_w, d.c, d.out_h, d.out_w = n, h, w, c, h, w
            d.kh = d.kw = 5
            d.stride_h = d.stride_w = 1
            d.pad_top = d.pad_bottom = d.pad_left = d.pad_right = 2
            d.in_exponent = d.out_exponent = -5
            d.input, d.output = px, dev.empty(x.nbytes)
            fn = lambda: abi.check(L.espdl_b200_pool(C.byref(d), None), name)
        else:
            d = abi.ResizeDesc()
            d.dtype = abi.DTYPE_INT8
            d.n, d.in_h, d.in_w, d.c, d.out_h, d.out_w = n, h, w, c, 2 * h, 2 * w
            d.scale_h = d.scale_w = 2.0
            d.in_exponent = d.out_exponent = -5
            d.input, d.output = px, dev.empty(4 * x.nbytes)
            algo = 5 * x.nbytes
            fn = lambda: abi.check(L.espdl_b200_resize(C.byref(d), None), name)
    elif name in ("rmsnorm", "layernorm"):
        d = abi.NormDesc()
        d.op, d.dtype = (abi.NORM_RMS if name == "rmsnorm" else abi.NORM_LAYER), abi.DTYPE_INT8
        d.rows, d.len = x.size // 768, 768
        d.input, d.output = px, dev.empty(x.nbytes)
        d.scale = dev.put(np.ones(768, dtype=np.float32)) if name == "rmsnorm" else dev.put(np.full(768, 64, dtype=np.int8))
        d.in_exponent, d.out_exponent, d.scale_exponent, d.epsilon = -5, -5, -6, 1e-5
        fn = lambda: abi.check(L.espdl_b200_norm(C.byref(d), None), name)
    elif name == "gather":
        d = abi.GatherDesc()
        idx = rng.permutation(h * w).astype(np.int32)
        d.input, d.output, d.indices = px, dev.empty(x.nbytes), dev.put(idx)
        d.elem_size, d.num_indices, d.outer, d.axis_size, d.inner = 1, idx.size, n, h * w, c
        fn = lambda: abi.check(L.espdl_b200_gather(C.byref(d), None), name)
    else:  # NHWC -> NCHW transpose of every image
        d = abi.CopyDesc()
        d.src, d.dst, d.elem_size, d.ndim = px, dev.empty(x.nbytes), 1, 3
        for i, (sz, ss, ds) in enumerate([(n, h * w * c, h * w * c), (c, 1, h * w), (h * w, c, 1)]):
            d.shape[i], d.src_stride[i], d.dst_stride[i] = sz, ss, ds
        fn = lambda: abi.check(L.espdl_b200_copy(C.byref(d), None), name)
    flush = dev.empty(FLUSH_BYTES)
    ms = _time(L, flush, fn, iters, warm)
    dev.close()
    return ms, algo / ms / 1e6, algo


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", action="append", default=[])
    ap.add_argument("--conv", action="append", default=[])
    ap.add_argument("--block", action="append", default=[])
    ap.add_argument("--mem", action="append", default=[])
    ap.add_argument("--list", action="store_true")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--kernel", default="auto", choices=sorted(KERNELS))
    ap.add_argument("--device", type=int, default=0)
    a = ap.parse_args()
    if a.list:
        for name, spec in CASES.items():
            print(name, spec)
        for name, spec in BLOCKS.items():
            print(name, spec)
        return
    todo = [(name, CASES[name]) for name in (a.case or ([] if (a.conv or a.block or a.mem) else list(CASES)))]
    todo += [(c, tuple(int(v) for v in c.split(","))) for c in a.conv]
    dev = Dev(a.device)
    for name, spec in todo:
        ms, tops, gbs, algo = run_case(dev, spec, a.iters, a.warmup, KERNELS[a.kernel])
        print(f"{name:16s} {ms:9.4f} ms {tops:9.2f} TOPS {gbs:9.1f} GB/s  algorithmic_bytes={algo}", flush=True)


    for name in (MEM_CASES if a.mem == ["all"] else a.mem):
        ms, gbs, algo = run_mem(dev, name, a.iters, a.warmup)
        print(f"{name:16s} {ms:9.4f} ms {gbs:9.1f} GB/s  algorithmic_bytes={algo}", flush=True)
    for name in a.block:
        spec = BLOCKS[name] if name in BLOCKS else tuple(int(v) for v in name.split(","))
        ms_f, ms_s, tops, gbs, algo = run_block(dev, spec, a.iters, a.warmup)
        print(f"{name:20s} fused {ms_f:9.4f} ms  separate convs {ms_s:9.4f} ms  {tops:8.2f} TOPS {gbs:8.1f} GB/s  "
              f"algorithmic_bytes={algo}", flush=True)


if __name__ == "__main__":
    main()
