"""CPU-side checks of the C ABI: the built library loads and exports every symbol include/espdl_b200.h
declares, the ctypes mirrors have the C structs' sizes, and calls fail cleanly (no compute) without a GPU."""
import ctypes as C
import os
import re
import subprocess

import pytest

from espdl_b200 import abi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "espdl_b200.h")


@pytest.fixture(scope="module")
def library():
    if not os.path.exists(abi.LIB_PATH):
        from espdl_b200 import build
        build.build()
    return abi.bind(C.CDLL(abi.LIB_PATH))


def test_every_declared_symbol_is_exported(library):
    text = open(HEADER).read()
    declared = set(re.findall(r"\b(espdl_b200_\w+)\s*\(", text))
    assert declared == set(abi.SYMBOLS), declared ^ set(abi.SYMBOLS)
    for name in declared:
        assert hasattr(library, name)


def test_struct_sizes_match_the_header(tmp_path):
    src = tmp_path / "sizes.c"
    src.write_text('#include <stdio.h>\n#include "espdl_b200.h"\nint main(void){printf("%zu %zu %zu %zu %zu %zu %zu %zu\\n",'
                   "sizeof(espdl_conv_desc),sizeof(espdl_eltwise_desc),sizeof(espdl_pool_desc),sizeof(espdl_resize_desc),"
                   "sizeof(espdl_copy_desc),sizeof(espdl_softmax_desc),sizeof(espdl_gather_desc),sizeof(espdl_norm_desc));return 0;}\n")
    exe = tmp_path / "sizes"
    subprocess.check_call(["/usr/bin/gcc", "-std=c99", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe)])
    sizes = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    mirrors = [abi.ConvDesc, abi.EltwiseDesc, abi.PoolDesc, abi.ResizeDesc, abi.CopyDesc, abi.SoftmaxDesc, abi.GatherDesc, abi.NormDesc]
    assert sizes == [C.sizeof(m) for m in mirrors]


def test_argument_validation_needs_no_gpu(library):
    assert library.espdl_b200_conv2d(None, None) == abi.ERR_INVALID_ARG
    assert library.espdl_b200_eltwise(None, None) == abi.ERR_INVALID_ARG
    assert library.espdl_b200_pool(None, None) == abi.ERR_INVALID_ARG
    assert library.espdl_b200_strerror(abi.ERR_TIMEOUT) == b"device-side wait timed out"
    assert library.espdl_b200_launch_count() == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    monkeypatch.setattr(abi, "LIB_PATH", str(tmp_path / "nope.so"))
    monkeypatch.setattr(abi, "_lib", None)
    with pytest.raises(RuntimeError, match="no CPU or PyTorch fallback"):
        abi.load()
