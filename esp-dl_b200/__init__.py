"""B200 (sm_100a) backend for ESP-DL's quantized operator forward path - Python plumbing.

The product is the C-ABI shared library built from csrc/ (declared in include/espdl_b200.h) and
the C++ host layer in host/; this package only binds them for tests and the benchmark."""
from . import abi  # noqa: F401
