"""ctypes mirror of include/espdl_b200.h and loader of the CUDA backend library.

This is plumbing for tests and the benchmark: the descriptors are the C structs
of the C ABI, field for field.  The library is built in-tree by build.py; loading
fails loudly (RuntimeError) when it is missing - there is no CPU fallback.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libespdl_b200.so")

OK, ERR_INVALID_ARG, ERR_UNSUPPORTED, ERR_CUDA, ERR_NO_DEVICE, ERR_NO_MEM, ERR_TIMEOUT, ERR_TOO_LARGE = 0, -1, -2, -3, -4, -5, -6, -7
DTYPE_FLOAT, DTYPE_INT8, DTYPE_INT16, DTYPE_INT32, DTYPE_INT64, DTYPE_BOOL = 1, 3, 5, 6, 7, 9
ACT_LINEAR, ACT_RELU = 0, 1
ROUND_HALF_UP, ROUND_HALF_EVEN = 0, 1
KERNEL_AUTO, KERNEL_SIMT, KERNEL_TCGEN05 = 0, 1, 2
ELT_ADD, ELT_MUL, ELT_REQUANTIZE, ELT_LUT, ELT_CLIP, ELT_RELU, ELT_PRELU, ELT_SUB = range(8)
ELT_MAX, ELT_MIN, ELT_DIV, ELT_MOD, ELT_GREATER, ELT_GREATER_EQUAL, ELT_EQUAL, ELT_LESS, ELT_LESS_EQUAL, ELT_POW = range(8, 18)
POOL_MAX, POOL_AVG, POOL_GLOBAL_AVG = 0, 1, 2

i32 = C.c_int32


class ConvDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("filter", C.c_void_p), ("bias", C.c_void_p), ("output", C.c_void_p),
        ("filter_exponents", C.c_void_p), ("lut", C.c_void_p),
        ("dtype", i32), ("n", i32), ("in_h", i32), ("in_w", i32), ("in_c", i32),
        ("out_h", i32), ("out_w", i32), ("out_c", i32), ("kh", i32), ("kw", i32),
        ("stride_h", i32), ("stride_w", i32), ("dilation_h", i32), ("dilation_w", i32),
        ("pad_top", i32), ("pad_bottom", i32), ("pad_left", i32), ("pad_right", i32),
        ("group", i32), ("in_pixel_stride", i32), ("out_pixel_stride", i32),
        ("in_exponent", i32), ("out_exponent", i32), ("filter_exponent", i32), ("per_channel", i32),
        ("activation", i32), ("round_mode", i32), ("kernel", i32), ("filter_image_stride", i32),
        ("residual", C.c_void_p), ("residual_pixel_stride", i32), ("lut_channel_stride", i32),
    ]


class EltwiseDesc(C.Structure):
    _fields_ = [
        ("input0", C.c_void_p), ("input1", C.c_void_p), ("output", C.c_void_p),
        ("op", i32), ("in_dtype", i32), ("out_dtype", i32), ("ndim", i32),
        ("out_shape", i32 * 4), ("in0_shape", i32 * 4), ("in1_shape", i32 * 4),
        ("in0_exponent", i32), ("in1_exponent", i32), ("out_exponent", i32),
        ("clip_lo", i32), ("clip_hi", i32), ("round_mode", i32), ("lut_shift", i32), ("table", C.c_void_p),
        ("in0_row_stride", C.c_int64), ("in1_row_stride", C.c_int64), ("out_row_stride", C.c_int64),
    ]


class PoolDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("output", C.c_void_p), ("op", i32), ("dtype", i32),
        ("n", i32), ("in_h", i32), ("in_w", i32), ("c", i32), ("out_h", i32), ("out_w", i32),
        ("kh", i32), ("kw", i32), ("stride_h", i32), ("stride_w", i32),
        ("pad_top", i32), ("pad_bottom", i32), ("pad_left", i32), ("pad_right", i32),
        ("in_exponent", i32), ("out_exponent", i32),
    ]


class ResizeDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("output", C.c_void_p), ("dtype", i32),
        ("n", i32), ("in_h", i32), ("in_w", i32), ("c", i32), ("out_h", i32), ("out_w", i32),
        ("scale_h", C.c_float), ("scale_w", C.c_float),
        ("in_exponent", i32), ("out_exponent", i32), ("out_pixel_stride", i32), ("mode", i32),
    ]


class CopyDesc(C.Structure):
    _fields_ = [
        ("src", C.c_void_p), ("dst", C.c_void_p), ("elem_size", i32), ("ndim", i32),
        ("shape", i32 * 6), ("src_stride", C.c_int64 * 6), ("dst_stride", C.c_int64 * 6),
    ]


class PartsDesc(C.Structure):
    _fields_ = [("wide", C.c_void_p), ("parts", C.c_void_p * 8), ("part_bytes", C.c_int64 * 8), ("n_parts", i32), ("split", i32),
                ("rows", C.c_int64), ("part_stride", C.c_int64 * 8), ("skip", i32 * 8)]


class SoftmaxDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("output", C.c_void_p), ("exp_table", C.c_void_p),
        ("rows", i32), ("len", i32), ("out_dtype", i32), ("out_exponent", i32), ("inner", i32), ("log", i32), ("in_exponent", i32), ("round_mode", i32),
    ]


class BlockDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("output", C.c_void_p),
        ("expand_filter", C.c_void_p), ("expand_bias", C.c_void_p), ("expand_filter_exponents", C.c_void_p),
        ("dw_filter", C.c_void_p), ("dw_bias", C.c_void_p), ("dw_filter_exponents", C.c_void_p),
        ("project_filter", C.c_void_p), ("project_bias", C.c_void_p), ("project_filter_exponents", C.c_void_p),
        ("residual", C.c_void_p),
        ("dtype", i32), ("n", i32), ("in_h", i32), ("in_w", i32), ("in_c", i32), ("hidden_c", i32),
        ("out_h", i32), ("out_w", i32), ("out_c", i32), ("stride", i32), ("pad_top", i32), ("pad_left", i32),
        ("in_exponent", i32), ("expand_exponent", i32), ("dw_exponent", i32), ("out_exponent", i32),
        ("expand_filter_exponent", i32), ("dw_filter_exponent", i32), ("project_filter_exponent", i32),
        ("per_channel", i32), ("expand_activation", i32), ("dw_activation", i32), ("project_activation", i32),
        ("expand_clip_max", i32), ("dw_clip_max", i32), ("round_mode", i32), ("reserved", i32 * 2),
    ]


class ImageDesc(C.Structure):
    _fields_ = [
        ("input", C.c_void_p), ("output", C.c_void_p), ("lut", C.c_void_p),
        ("n", i32), ("src_h", i32), ("src_w", i32), ("channels", i32), ("dst_h", i32), ("dst_w", i32), ("out_dtype", i32),
        ("crop_x0", i32), ("crop_y0", i32), ("crop_x1", i32), ("crop_y1", i32),
        ("border_top", i32), ("border_bottom", i32), ("border_left", i32), ("border_right", i32),
        ("swap_rb", i32), ("bg", C.c_uint8 * 4), ("inv_scale_x", C.c_float), ("inv_scale_y", C.c_float),
    ]


class DetectRecord(C.Structure):
    _fields_ = [("image", C.c_uint16), ("stage", C.c_uint16), ("y", C.c_uint16), ("x", C.c_uint16), ("category", C.c_uint16),
                ("score", C.c_int8), ("pad", C.c_uint8), ("reserved", C.c_uint32), ("box", C.c_int8 * 64)]


class DetectDesc(C.Structure):
    _fields_ = [("score", C.c_void_p), ("box", C.c_void_p), ("records", C.c_void_p), ("count", C.c_void_p),
                ("n", i32), ("h", i32), ("w", i32), ("classes", i32), ("box_channels", i32),
                ("score_threshold", i32), ("capacity", i32), ("stage", i32)]


class ReduceDesc(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("op", i32), ("dtype", i32), ("ndim", i32), ("shape", i32 * 6),
                ("reduce", i32 * 6), ("in_exponent", i32), ("out_exponent", i32), ("round_mode", i32), ("exp_table", C.c_void_p)]


(REDUCE_MEAN, REDUCE_SUM, REDUCE_MAX, REDUCE_MIN, REDUCE_L1, REDUCE_SUM_SQUARE, REDUCE_L2, REDUCE_PROD, REDUCE_LOG_SUM,
 REDUCE_LOG_SUM_EXP) = range(10)


class PadDesc(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("elem_size", i32), ("ndim", i32), ("mode", i32), ("shape", i32 * 6),
                ("pad_begin", i32 * 6), ("pad_end", i32 * 6), ("constant", C.c_int64)]


PAD_CONSTANT, PAD_EDGE, PAD_REFLECT = range(3)


class NormDesc(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("scale", C.c_void_p), ("bias", C.c_void_p), ("mean", C.c_void_p),
                ("inv_std_dev", C.c_void_p), ("op", i32), ("dtype", i32), ("rows", C.c_int64), ("len", i32), ("in_exponent", i32),
                ("out_exponent", i32), ("scale_exponent", i32), ("bias_exponent", i32), ("mean_exponent", i32),
                ("inv_std_dev_exponent", i32), ("epsilon", C.c_float), ("round_mode", i32), ("p", i32), ("inner", C.c_int64)]


NORM_RMS, NORM_LAYER, NORM_LP = range(3)


class ReverseSequenceDesc(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("seq_lens", C.c_void_p), ("elem_size", i32), ("batch_axis", i32),
                ("dim0", i32), ("dim1", i32), ("feature", C.c_int64)]


class ScatterNDDesc(C.Structure):
    _fields_ = [("data", C.c_void_p), ("indices", C.c_void_p), ("updates", C.c_void_p), ("output", C.c_void_p), ("dtype", i32),
                ("reduction", i32), ("index_depth", i32), ("n_slices", i32), ("slice_size", C.c_int64), ("data_size", C.c_int64),
                ("axis_offset", C.c_int64 * 6)]


SCATTER_NONE, SCATTER_ADD, SCATTER_MUL, SCATTER_MAX, SCATTER_MIN = range(5)


class RnnDesc(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("r", C.c_void_p), ("b", C.c_void_p), ("initial_h", C.c_void_p),
                ("initial_c", C.c_void_p), ("y", C.c_void_p), ("y_h", C.c_void_p), ("y_c", C.c_void_p), ("sigmoid_table", C.c_void_p),
                ("tanh_table", C.c_void_p), ("sigmoid_max", i32), ("tanh_max", i32), ("op", i32), ("dtype", i32), ("seq_length", i32),
                ("input_size", i32), ("hidden_size", i32), ("directions", i32), ("x_exponent", i32), ("w_exponent", i32),
                ("r_exponent", i32), ("h_exponent", i32), ("y_exponent", i32), ("c_exponent", i32), ("gate_exponent", i32),
                ("round_mode", i32)]


RNN_GRU, RNN_LSTM = range(2)


class GatherDesc(C.Structure):
    _fields_ = [("input", C.c_void_p), ("output", C.c_void_p), ("indices", C.c_void_p), ("elem_size", i32), ("num_indices", i32),
                ("outer", C.c_int64), ("axis_size", C.c_int64), ("inner", C.c_int64)]


# every symbol include/espdl_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "espdl_b200_init": (C.c_int, [C.c_int]),
    "espdl_b200_shutdown": (None, []),
    "espdl_b200_strerror": (C.c_char_p, [C.c_int]),
    "espdl_b200_last_error": (C.c_char_p, []),
    "espdl_b200_arena_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "espdl_b200_arena_free": (C.c_int, [C.c_void_p]),
    "espdl_b200_upload": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "espdl_b200_download": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "espdl_b200_download_rows": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]),
    "espdl_b200_memset": (C.c_int, [C.c_void_p, C.c_int, C.c_size_t, C.c_void_p]),
    "espdl_b200_stream_sync": (C.c_int, [C.c_void_p]),
    "espdl_b200_host_alloc": (C.c_int, [C.c_size_t, C.POINTER(C.c_void_p)]),
    "espdl_b200_host_free": (C.c_int, [C.c_void_p]),
    "espdl_b200_launch_count": (C.c_uint64, []),
    "espdl_b200_mem_info": (C.c_int, [C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "espdl_b200_stream_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "espdl_b200_stream_destroy": (C.c_int, [C.c_void_p]),
    "espdl_b200_event_create": (C.c_int, [C.POINTER(C.c_void_p)]),
    "espdl_b200_event_destroy": (C.c_int, [C.c_void_p]),
    "espdl_b200_event_record": (C.c_int, [C.c_void_p, C.c_void_p]),
    "espdl_b200_event_elapsed_ms": (C.c_int, [C.c_void_p, C.c_void_p, C.POINTER(C.c_float)]),
    "espdl_b200_event_sync": (C.c_int, [C.c_void_p]),
    "espdl_b200_stream_wait_event": (C.c_int, [C.c_void_p, C.c_void_p]),
    "espdl_b200_device_copy": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "espdl_b200_graph_begin": (C.c_int, [C.c_void_p]),
    "espdl_b200_graph_end": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "espdl_b200_graph_launch": (C.c_int, [C.c_void_p, C.c_void_p]),
    "espdl_b200_graph_destroy": (C.c_int, [C.c_void_p]),
    "espdl_b200_conv2d": (C.c_int, [C.POINTER(ConvDesc), C.c_void_p]),
    "espdl_b200_conv2d_workspace_bytes": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(C.c_size_t)]),
    "espdl_b200_conv2d_ws": (C.c_int, [C.POINTER(ConvDesc), C.c_void_p, C.c_size_t, C.c_void_p]),
    "espdl_b200_gemm_s16_static": (C.c_int, [C.POINTER(ConvDesc), C.c_void_p]),
    "espdl_b200_eltwise": (C.c_int, [C.POINTER(EltwiseDesc), C.c_void_p]),
    "espdl_b200_pool": (C.c_int, [C.POINTER(PoolDesc), C.c_void_p]),
    "espdl_b200_resize": (C.c_int, [C.POINTER(ResizeDesc), C.c_void_p]),
    "espdl_b200_copy": (C.c_int, [C.POINTER(CopyDesc), C.c_void_p]),
    "espdl_b200_concat_split": (C.c_int, [C.POINTER(PartsDesc), C.c_void_p]),
    "espdl_b200_softmax": (C.c_int, [C.POINTER(SoftmaxDesc), C.c_void_p]),
    "espdl_b200_gemm_scatter": (C.c_int, [C.POINTER(ConvDesc), C.POINTER(C.c_void_p), C.c_int, C.c_void_p]),
    "espdl_b200_ipc_export": (C.c_int, [C.c_void_p, C.c_void_p]),
    "espdl_b200_ipc_open": (C.c_int, [C.c_void_p, C.POINTER(C.c_void_p)]),
    "espdl_b200_ipc_close": (C.c_int, [C.c_void_p]),
    "espdl_b200_fused_block": (C.c_int, [C.POINTER(BlockDesc), C.c_void_p]),
    "espdl_b200_fused_block_supported": (C.c_int, [C.POINTER(BlockDesc)]),
    "espdl_b200_image_preprocess": (C.c_int, [C.POINTER(ImageDesc), C.c_void_p]),
    "espdl_b200_detect_candidates": (C.c_int, [C.POINTER(DetectDesc), C.c_void_p]),
    "espdl_b200_reduce": (C.c_int, [C.POINTER(ReduceDesc), C.c_void_p]),
    "espdl_b200_pad": (C.c_int, [C.POINTER(PadDesc), C.c_void_p]),
    "espdl_b200_gather": (C.c_int, [C.POINTER(GatherDesc), C.c_void_p]),
    "espdl_b200_norm": (C.c_int, [C.POINTER(NormDesc), C.c_void_p]),
    "espdl_b200_reverse_sequence": (C.c_int, [C.POINTER(ReverseSequenceDesc), C.c_void_p]),
    "espdl_b200_scatter_nd": (C.c_int, [C.POINTER(ScatterNDDesc), C.c_void_p]),
    "espdl_b200_rnn": (C.c_int, [C.POINTER(RnnDesc), C.c_void_p]),
}

_lib = None


def bind(lib, symbols=SYMBOLS):
    for name, (res, args) in symbols.items():
        fn = getattr(lib, name)  # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    return lib


def load():
    """Load libespdl_b200.so (built by build.py).  Raises if it is absent: no fallback exists."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -c 'import __graft_entry__ as g; g.build()'`; "
                "the backend has no CPU or PyTorch fallback")
        _lib = bind(C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL))
    return _lib


def check(status, what=""):
    if status != OK:
        lib = load()
        raise RuntimeError(
            f"{what}: {lib.espdl_b200_strerror(status).decode()} ({status}) {lib.espdl_b200_last_error().decode()}")
