"""Loaders for the two CPU checkers (test infrastructure): the plain-C oracle and, when it was
built, the reference's own operators (oracle/_ref).  Both take the C-ABI descriptors with host pointers."""
import ctypes as C
import os
import subprocess

import numpy as np

from espdl_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
ORACLE_SO = os.path.join(ROOT, "oracle", "libespdl_oracle.so")
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libespdl_ref.so")

_oracle = None
_ref = None


def oracle():
    global _oracle
    if _oracle is None:
        if not os.path.exists(ORACLE_SO):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "oracle"], stdout=subprocess.DEVNULL)
        lib = C.CDLL(ORACLE_SO)
        for name, desc in [("oracle_conv2d", abi.ConvDesc), ("oracle_eltwise", abi.EltwiseDesc), ("oracle_pool", abi.PoolDesc),
                           ("oracle_resize", abi.ResizeDesc), ("oracle_copy", abi.CopyDesc), ("oracle_softmax", abi.SoftmaxDesc),
                           ("oracle_reduce", abi.ReduceDesc), ("oracle_pad", abi.PadDesc), ("oracle_gather", abi.GatherDesc), ("oracle_norm", abi.NormDesc)]:
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(desc)]
        lib.oracle_softmax_table.restype = None
        lib.oracle_softmax_table.argtypes = [C.c_void_p, C.c_int]
        lib.oracle_num_threads.restype = C.c_int
        lib.oracle_depth_space.restype = C.c_int
        lib.oracle_depth_space.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 7
        lib.oracle_reverse_sequence.restype = C.c_int
        lib.oracle_reverse_sequence.argtypes = [C.POINTER(abi.ReverseSequenceDesc), C.c_void_p]
        lib.oracle_scatter_nd.restype = C.c_int
        lib.oracle_scatter_nd.argtypes = [C.POINTER(abi.ScatterNDDesc)]
        lib.oracle_rnn.restype = C.c_int
        lib.oracle_rnn.argtypes = [C.POINTER(abi.RnnDesc)]
        lib.oracle_rnn_table.restype = C.c_int
        lib.oracle_rnn_table.argtypes = [C.c_int, C.c_int, C.c_void_p]
        _oracle = lib
    return _oracle


def have_ref():
    return os.path.exists(REF_SO)


def ref():
    global _ref
    if _ref is None:
        lib = C.CDLL(REF_SO)
        lib.ref_conv2d.restype = C.c_int
        lib.ref_conv2d.argtypes = [C.POINTER(abi.ConvDesc), C.c_int]
        for name, desc in [("ref_eltwise", abi.EltwiseDesc), ("ref_pool", abi.PoolDesc), ("ref_resize", abi.ResizeDesc)]:
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.POINTER(desc)]
        lib.ref_softmax.restype = C.c_int
        lib.ref_softmax.argtypes = [C.POINTER(abi.SoftmaxDesc), C.c_int]
        lib.ref_concat2.restype = C.c_int
        lib.ref_concat2.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.POINTER(C.c_int), C.POINTER(C.c_int), C.c_int, C.c_int]
        lib.ref_matmul.restype = C.c_int
        lib.ref_matmul.argtypes = [C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_void_p,
                                   C.c_int, C.c_int, C.c_int]
        lib.ref_pad.restype = C.c_int
        lib.ref_pad.argtypes = [C.POINTER(abi.PadDesc)]
        lib.ref_reduce.restype = C.c_int
        lib.ref_reduce.argtypes = [C.POINTER(abi.ReduceDesc)]
        lib.ref_num_threads.restype = C.c_int
        lib.ref_gather.restype = C.c_int
        lib.ref_gather.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_int, C.c_int, C.c_int]
        lib.ref_norm.restype = C.c_int
        lib.ref_norm.argtypes = [C.POINTER(abi.NormDesc)]
        lib.ref_insert_zeros.restype = C.c_int
        lib.ref_insert_zeros.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.POINTER(C.c_int), C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_int)]
        lib.ref_depth_space.restype = C.c_int
        lib.ref_depth_space.argtypes = [C.c_void_p, C.c_void_p] + [C.c_int] * 7
        lib.ref_lp_norm.restype = C.c_int
        lib.ref_lp_norm.argtypes = [C.POINTER(abi.NormDesc)]
        lib.ref_reverse_sequence.restype = C.c_int
        lib.ref_reverse_sequence.argtypes = [C.POINTER(abi.ReverseSequenceDesc), C.c_void_p]
        lib.ref_scatter_nd.restype = C.c_int
        lib.ref_scatter_nd.argtypes = [C.POINTER(abi.ScatterNDDesc), C.POINTER(C.c_int), C.c_int]
        lib.ref_rnn.restype = C.c_int
        lib.ref_rnn.argtypes = [C.POINTER(abi.RnnDesc)]
        _ref = lib
    return _ref


def ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


NP = {abi.DTYPE_INT8: np.int8, abi.DTYPE_INT16: np.int16, abi.DTYPE_FLOAT: np.float32,
      abi.DTYPE_INT32: np.int32, abi.DTYPE_INT64: np.int64}
