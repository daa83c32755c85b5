"""Seeded operator cases shared by the CPU (oracle vs reference) and GPU (CUDA vs oracle) parity tests.

A case is a dict of numpy arrays plus the scalar fields of the matching C-ABI descriptor; `*_desc`
turns it into a descriptor whose pointers address either the host arrays or device copies."""
import ctypes as C

import numpy as np

from espdl_b200 import abi

NP = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16, abi.DTYPE_FLOAT: np.float32, abi.DTYPE_BOOL: np.uint8}
TWO_OPERAND_OPS = (abi.ELT_ADD, abi.ELT_MUL, abi.ELT_SUB) + tuple(range(abi.ELT_MAX, abi.ELT_LESS_EQUAL + 1))


def conv_out(size, k, s, d, p0, p1):
    return (size + p0 + p1 - d * (k - 1) - 1) // s + 1


def conv_case(seed=0, dtype=abi.DTYPE_INT8, n=1, h=8, w=8, cin=16, cout=16, kh=3, kw=3, stride=1, dil=1, pad=None,
              depthwise=False, bias=True, per_channel=False, act=abi.ACT_RELU, round_mode=abi.ROUND_HALF_UP,
              e_in=-7, e_out=-6, e_w=(-9, -6), lut=False, in_stride=0, out_stride=0, bias_mag=1 << 12, wide=False):
    """Random conv / depthwise / Gemm case.  Value ranges follow the benchmark configs: inputs uniform over the
    full integer range, weights uniform in [-127, 127] (int8), bias uniform in [-2^12, 2^12]."""
    rng = np.random.default_rng(seed)
    t = NP[dtype]
    if pad is None:
        pad = (kh // 2, kh // 2, kw // 2, kw // 2)
    pt, pb, pl, pr = pad
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    dh, dw = (dil, dil) if isinstance(dil, int) else dil
    oh, ow = conv_out(h, kh, sh, dh, pt, pb), conv_out(w, kw, sw, dw, pl, pr)
    if depthwise:
        cout = cin
    ips = in_stride or cin
    ops = out_stride or cout
    info = np.iinfo(t)
    x = rng.integers(info.min, info.max + 1, size=(n, h, w, ips), dtype=t)
    wlim = 127 if dtype == abi.DTYPE_INT8 else 32767
    wshape = (kh, kw, cin) if depthwise else (cout, kh, kw, cin)
    wt = rng.integers(-wlim, wlim + 1, size=wshape, dtype=t)
    if wide and dtype == abi.DTYPE_INT16:
        wt = rng.integers(-32768, 32768, size=wshape, dtype=t)
    btype = np.int32 if dtype == abi.DTYPE_INT8 else np.int64
    b = rng.integers(-bias_mag, bias_mag + 1, size=(cout,)).astype(btype) if bias else None
    if per_channel:
        ew = rng.integers(e_w[0], e_w[1] + 1, size=(cout,)).astype(np.int32)
        ew_scalar = 0
    else:
        ew = None
        ew_scalar = int(rng.integers(e_w[0], e_w[1] + 1))
    # lut=True: one 256-entry table; lut="channels": one table per output channel (lut_channel_stride = 256)
    table = rng.integers(-128, 128, size=((cout if not depthwise else cin) * 256 if lut == "channels" else 256,), dtype=np.int8) if lut else None
    out = np.zeros((n, oh, ow, ops), dtype=t)
    return dict(x=x, w=wt, b=b, ew=ew, lut=table, out=out, dtype=dtype, n=n, in_h=h, in_w=w, in_c=cin, out_h=oh, out_w=ow,
                out_c=cout, kh=kh, kw=kw, stride_h=sh, stride_w=sw, dilation_h=dh, dilation_w=dw, pad_top=pt,
                pad_bottom=pb, pad_left=pl, pad_right=pr, group=cin if depthwise else 1,
                in_pixel_stride=in_stride, out_pixel_stride=out_stride, in_exponent=e_in, out_exponent=e_out,
                filter_exponent=ew_scalar, per_channel=int(per_channel), activation=act, round_mode=round_mode, kernel=0,
                filter_image_stride=0)


def gemm_case(seed=0, dtype=abi.DTYPE_INT8, m=64, k=64, n_out=32, **kw):
    """A[M,K] x W[N][K]: the conv call with n=1, in_h=1, in_w=M, 1x1 filter (dl_module_gemm.hpp:85-123)."""
    kw.setdefault("act", abi.ACT_LINEAR)
    return conv_case(seed=seed, dtype=dtype, n=1, h=1, w=m, cin=k, cout=n_out, kh=1, kw=1, pad=(0, 0, 0, 0), **kw)


_SCALARS = [f for f, t in abi.ConvDesc._fields_ if t is abi.i32 and f != "lut_channel_stride"]


def conv_desc(case, ptrs=None):
    """ptrs: optional dict name -> integer address overriding the host arrays (device copies)."""
    d = abi.ConvDesc()
    host = dict(input=case["x"], filter=case["w"], bias=case["b"], output=case["out"], filter_exponents=case["ew"], lut=case["lut"],
                residual=case.get("res"))
    for k, a in host.items():
        if ptrs is not None:
            setattr(d, k, ptrs.get(k))
        else:
            setattr(d, k, None if a is None else a.ctypes.data)
    for f in _SCALARS:
        setattr(d, f, int(case.get(f, 0)))
    d.lut_channel_stride = 256 if case["lut"] is not None and case["lut"].size > 256 else 0
    return d


def eltwise_case(op, seed=0, dtype=abi.DTYPE_INT8, out_shape=(2, 5, 7, 16), in0_shape=None, in1_shape=None,
                 e0=-5, e1=-6, eo=-4, out_dtype=None, in_dtype=None, clip=(0, 96), round_mode=abi.ROUND_HALF_UP, lut_shift=5):
    rng = np.random.default_rng(seed)
    in_dtype = in_dtype or dtype
    out_dtype = out_dtype or dtype
    in0_shape = tuple(in0_shape or out_shape)
    in1_shape = tuple(in1_shape or out_shape)

    def rnd(shape, dt):
        if dt == abi.DTYPE_FLOAT:
            return (rng.standard_normal(shape) * 4).astype(np.float32)
        info = np.iinfo(NP[dt])
        return rng.integers(info.min, info.max + 1, size=shape, dtype=NP[dt])

    a = rnd(in0_shape, in_dtype)
    b = None
    if op in TWO_OPERAND_OPS:
        b = rnd(in1_shape, in_dtype)
        if op in (abi.ELT_DIV, abi.ELT_MOD) or op >= abi.ELT_GREATER:
            # zeros in both operands (division by zero, 0 / x, 0 / 0) and equal pairs for the comparisons
            if a.size > 1:
                a.reshape(-1)[rng.integers(0, a.size, size=max(a.size // 8, 1))] = 0
            if b.size > 1:
                b.reshape(-1)[rng.integers(0, b.size, size=max(b.size // 8, 1))] = 0
            elif b.reshape(-1)[0] == 0:
                b.reshape(-1)[0] = 3  # the reference's table for a zero scalar divisor converts an infinity to int
            if op >= abi.ELT_GREATER and a.shape == b.shape:
                idx = rng.integers(0, a.size, size=max(a.size // 6, 1))
                b.reshape(-1)[idx] = a.reshape(-1)[idx]
    elif op == abi.ELT_LUT and in_dtype == abi.DTYPE_INT16:
        b = rng.integers(-32768, 32768, size=((65536 >> lut_shift) + 1,), dtype=np.int16)
        in1_shape = (1,) * len(out_shape)
    elif op == abi.ELT_LUT:
        b = rng.integers(-128, 128, size=(256,), dtype=np.int8)
        in1_shape = (1,) * len(out_shape)
    elif op == abi.ELT_PRELU:
        b = rnd((out_shape[-1],), in_dtype)
        in1_shape = (1,) * (len(out_shape) - 1) + (out_shape[-1],)
    else:
        in1_shape = (1,) * len(out_shape)
    out = np.zeros(out_shape, dtype=NP[out_dtype])
    return dict(a=a, b=b, out=out, op=op, in_dtype=in_dtype, out_dtype=out_dtype, ndim=len(out_shape), out_shape=out_shape,
                in0_shape=in0_shape, in1_shape=in1_shape, in0_exponent=e0, in1_exponent=e1, out_exponent=eo,
                clip_lo=clip[0], clip_hi=clip[1], round_mode=round_mode, lut_shift=lut_shift if in_dtype == abi.DTYPE_INT16 else 0)


def eltwise_desc(case, ptrs=None):
    d = abi.EltwiseDesc()
    host = dict(input0=case["a"], input1=case["b"], output=case["out"])
    for k, a in host.items():
        setattr(d, k, (ptrs.get(k) if ptrs is not None else (None if a is None else a.ctypes.data)))
    for f in ("op", "in_dtype", "out_dtype", "ndim", "in0_exponent", "in1_exponent", "out_exponent", "clip_lo", "clip_hi", "round_mode"):
        setattr(d, f, int(case[f]))
    d.lut_shift = int(case.get("lut_shift", 0))
    for f in ("out_shape", "in0_shape", "in1_shape"):
        arr = getattr(d, f)
        for i, v in enumerate(case[f]):
            arr[i] = int(v)
    return d


def pool_case(op, seed=0, dtype=abi.DTYPE_INT8, n=2, h=9, w=10, c=24, kh=3, kw=3, stride=2, pad=(1, 1, 1, 1), e_in=-5, e_out=-5):
    rng = np.random.default_rng(seed)
    info = np.iinfo(NP[dtype])
    x = rng.integers(info.min, info.max + 1, size=(n, h, w, c), dtype=NP[dtype])
    sh, sw = (stride, stride) if isinstance(stride, int) else stride
    if op == abi.POOL_GLOBAL_AVG:
        oh = ow = 1
        kh, kw, sh, sw, pad = h, w, 1, 1, (0, 0, 0, 0)
    else:
        oh = (h + pad[0] + pad[1] - kh) // sh + 1
        ow = (w + pad[2] + pad[3] - kw) // sw + 1
    out = np.zeros((n, oh, ow, c), dtype=NP[dtype])
    return dict(x=x, out=out, op=op, dtype=dtype, n=n, in_h=h, in_w=w, c=c, out_h=oh, out_w=ow, kh=kh, kw=kw,
                stride_h=sh, stride_w=sw, pad_top=pad[0], pad_bottom=pad[1], pad_left=pad[2], pad_right=pad[3],
                in_exponent=e_in, out_exponent=e_out)


def pool_desc(case, ptrs=None):
    d = abi.PoolDesc()
    d.input = ptrs["input"] if ptrs is not None else case["x"].ctypes.data
    d.output = ptrs["output"] if ptrs is not None else case["out"].ctypes.data
    for f, _ in abi.PoolDesc._fields_[2:]:
        setattr(d, f, int(case[f]))
    return d


def resize_case(seed=0, dtype=abi.DTYPE_INT8, n=2, h=5, w=6, c=16, scale=(2.0, 2.0), e_in=-5, e_out=-5, out_stride=0, mode=0):
    rng = np.random.default_rng(seed)
    info = np.iinfo(NP[dtype])
    x = rng.integers(info.min, info.max + 1, size=(n, h, w, c), dtype=NP[dtype])
    oh, ow = int(h * np.float32(scale[0])), int(w * np.float32(scale[1]))
    out = np.zeros((n, oh, ow, out_stride or c), dtype=NP[dtype])
    return dict(x=x, out=out, dtype=dtype, n=n, in_h=h, in_w=w, c=c, out_h=oh, out_w=ow, scale_h=scale[0], scale_w=scale[1],
                in_exponent=e_in, out_exponent=e_out, out_pixel_stride=out_stride, mode=mode)


def resize_desc(case, ptrs=None):
    d = abi.ResizeDesc()
    d.input = ptrs["input"] if ptrs is not None else case["x"].ctypes.data
    d.output = ptrs["output"] if ptrs is not None else case["out"].ctypes.data
    for f in ("dtype", "n", "in_h", "in_w", "c", "out_h", "out_w", "in_exponent", "out_exponent", "out_pixel_stride", "mode"):
        setattr(d, f, int(case[f]))
    d.scale_h, d.scale_w = case["scale_h"], case["scale_w"]
    return d


def copy_desc(src, dst, elem_size, shape, src_stride, dst_stride):
    d = abi.CopyDesc()
    d.src, d.dst, d.elem_size, d.ndim = src, dst, elem_size, len(shape)
    for i, (s, a, b) in enumerate(zip(shape, src_stride, dst_stride)):
        d.shape[i], d.src_stride[i], d.dst_stride[i] = int(s), int(a), int(b)
    return d


def softmax_desc(inp, out, table, rows, length, out_dtype, out_exponent):
    d = abi.SoftmaxDesc()
    d.input, d.output, d.exp_table = inp, out, table
    d.rows, d.len, d.out_dtype, d.out_exponent = rows, length, out_dtype, out_exponent
    return d


# ------------------------------------------------------------------------------------------ fused inverted-residual block
def block_case(seed=0, n=1, h=14, w=14, cin=32, chid=192, cout=32, stride=1, expand=True, residual=None, per_channel=True,
               clip1=127, clipdw=127, round_mode=abi.ROUND_HALF_UP, e=(-5, -6, -5, -5), bias_mag=1 << 10, relu=(True, True, False)):
    """expand 1x1 (ReLU) -> depthwise 3x3 (ReLU) -> project 1x1 (linear) [-> Add] as three conv cases that share
    their tensors, the way the separate nodes of the reference's graph do.  e = exponents of input, expanded,
    depthwise output and block output."""
    rng = np.random.default_rng(seed)
    if residual is None:
        residual = stride == 1 and cin == cout
    acts = [abi.ACT_RELU if r else abi.ACT_LINEAR for r in relu]
    x = rng.integers(-128, 128, size=(n, h, w, cin), dtype=np.int8)
    stages = []
    if expand:
        c1 = conv_case(seed=seed * 7 + 1, n=n, h=h, w=w, cin=cin, cout=chid, kh=1, kw=1, pad=(0, 0, 0, 0), per_channel=per_channel,
                       act=acts[0], round_mode=round_mode, e_in=e[0], e_out=e[1], e_w=(-12, -9), bias_mag=bias_mag)
        c1["x"] = x
        stages.append(c1)
    else:
        chid = cin
    c2 = conv_case(seed=seed * 7 + 2, n=n, h=h, w=w, cin=chid, kh=3, kw=3, stride=stride, depthwise=True, per_channel=per_channel,
                   act=acts[1], round_mode=round_mode, e_in=e[1] if expand else e[0], e_out=e[2], e_w=(-9, -7), bias_mag=bias_mag)
    oh, ow = c2["out_h"], c2["out_w"]
    c3 = conv_case(seed=seed * 7 + 3, n=n, h=oh, w=ow, cin=chid, cout=cout, kh=1, kw=1, pad=(0, 0, 0, 0), per_channel=per_channel,
                   act=acts[2], round_mode=round_mode, e_in=e[2], e_out=e[3], e_w=(-12, -9), bias_mag=bias_mag)
    if residual:
        c3["res"] = x
    return dict(x=x, expand=stages[0] if expand else None, dw=c2, project=c3, clip1=clip1, clipdw=clipdw, residual=residual,
                out=np.zeros((n, oh, ow, cout), dtype=np.int8))


def block_desc(case, ptrs):
    """ptrs: name -> address (host arrays' or device copies') for input, output, residual and w/b/ew of each stage."""
    d = abi.BlockDesc()
    for k, v in ptrs.items():
        setattr(d, k, v)
    c1, c2, c3 = case["expand"], case["dw"], case["project"]
    d.dtype, d.n, d.in_h, d.in_w, d.in_c = abi.DTYPE_INT8, c2["n"], c2["in_h"], c2["in_w"], case["x"].shape[3]
    d.hidden_c, d.out_h, d.out_w, d.out_c = c2["in_c"], c2["out_h"], c2["out_w"], c3["out_c"]
    d.stride, d.pad_top, d.pad_left = c2["stride_h"], c2["pad_top"], c2["pad_left"]
    d.in_exponent = c1["in_exponent"] if c1 else c2["in_exponent"]
    d.expand_exponent, d.dw_exponent, d.out_exponent = c2["in_exponent"], c2["out_exponent"], c3["out_exponent"]
    d.expand_filter_exponent = c1["filter_exponent"] if c1 else 0
    d.dw_filter_exponent, d.project_filter_exponent = c2["filter_exponent"], c3["filter_exponent"]
    d.per_channel = ((c1["per_channel"] if c1 else 0) | (c2["per_channel"] << 1) | (c3["per_channel"] << 2))
    d.expand_activation = c1["activation"] if c1 else 0
    d.dw_activation, d.project_activation = c2["activation"], c3["activation"]
    d.expand_clip_max, d.dw_clip_max, d.round_mode = case["clip1"], case["clipdw"], c2["round_mode"]
    return d
