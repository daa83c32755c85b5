"""ctypes binding of the C++ host layer (dl::Model) for tests and the benchmark."""
import ctypes as C
import os

import numpy as np

from . import abi

HOST_LIB_PATH = os.path.join(abi.HERE, "libespdl_b200_host.so")
NP = {1: np.float32, 3: np.int8, 5: np.int16, 6: np.int32, 7: np.int64, 9: np.uint8}
_host = None


def host_lib():
    global _host
    if _host is None:
        abi.load()  # the CUDA library first (RTLD_GLOBAL), the host layer links against it
        if not os.path.exists(HOST_LIB_PATH):
            raise RuntimeError(f"{HOST_LIB_PATH} is missing: run the build; there is no fallback")
        L = C.CDLL(HOST_LIB_PATH)
        L.espdl_model_create.restype = C.c_void_p
        L.espdl_model_create.argtypes = [C.c_char_p, C.c_int, C.c_int]
        L.espdl_model_destroy.argtypes = [C.c_void_p]
        L.espdl_model_num_io.argtypes = [C.c_void_p, C.c_int]
        L.espdl_model_io_info.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.POINTER(C.c_int),
                                          C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p)]
        L.espdl_model_run.argtypes = [C.c_void_p]
        L.espdl_model_run_device.argtypes = [C.c_void_p, C.c_int]
        L.espdl_model_submit.argtypes = [C.c_void_p]
        L.espdl_model_wait.argtypes = [C.c_void_p]
        L.espdl_model_test.argtypes = [C.c_void_p]
        L.espdl_model_stream.restype = C.c_void_p
        L.espdl_model_stream.argtypes = [C.c_void_p]
        L.espdl_model_arena_bytes.restype = C.c_size_t
        L.espdl_model_arena_bytes.argtypes = [C.c_void_p]
        L.espdl_model_num_modules.argtypes = [C.c_void_p]
        L.espdl_model_num_slice_views.argtypes = [C.c_void_p]
        L.espdl_model_read_tensor.restype = C.c_longlong
        L.espdl_model_read_tensor.argtypes = [C.c_void_p, C.c_char_p, C.c_void_p, C.c_size_t]
        L.espdl_model_preprocess.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_float),
                                             C.POINTER(C.c_float), C.c_int, C.c_int, C.POINTER(C.c_int)]
        L.espdl_model_classify.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float)]
        L.espdl_model_detect.argtypes = [C.c_void_p, C.c_int, C.c_int, C.POINTER(C.c_char_p), C.POINTER(C.c_int), C.c_float, C.c_float, C.c_int,
                                         C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int), C.POINTER(C.c_float)]
        L.espdl_model_profile.restype = C.c_char_p
        L.espdl_model_profile.argtypes = [C.c_void_p]
        _host = L
    return _host


class IO:
    def __init__(self, name, shape, dtype, exponent, host, device):
        self.name, self.shape, self.dtype, self.exponent, self.host_ptr, self.device_ptr = name, shape, dtype, exponent, host, device
        n = int(np.prod(shape))
        self.nbytes = n * np.dtype(NP[dtype]).itemsize
        # numpy view of the pinned host buffer the C++ side owns
        buf = (C.c_char * self.nbytes).from_address(host)
        self.array = np.frombuffer(buf, dtype=NP[dtype], count=n).reshape(shape)


class Model:
    """dl::Model on cuda:0.  `batch` overrides dim 0 of the graph inputs."""

    def __init__(self, path, batch=0, graph=True, reuse=True, device=0):
        L = abi.load()
        abi.check(L.espdl_b200_init(device), "espdl_b200_init")
        self.lib = host_lib()
        flags = (0 if graph else 1) | (0 if reuse else 2)
        self.h = self.lib.espdl_model_create(os.fsencode(path), int(batch), flags)
        if not self.h:
            raise RuntimeError(f"failed to load / build {path}: {L.espdl_b200_last_error().decode()}")
        self.inputs = [self._io(0, i) for i in range(self.lib.espdl_model_num_io(self.h, 0))]
        self.outputs = [self._io(1, i) for i in range(self.lib.espdl_model_num_io(self.h, 1))]

    def _io(self, is_output, index):
        name, ndim, shape = C.c_char_p(), C.c_int(), (C.c_int * 8)()
        dtype, exponent, host, device = C.c_int(), C.c_int(), C.c_void_p(), C.c_void_p()
        abi.check(self.lib.espdl_model_io_info(self.h, is_output, index, C.byref(name), C.byref(ndim), shape, C.byref(dtype),
                                               C.byref(exponent), C.byref(host), C.byref(device)), "io_info")
        return IO(name.value.decode(), tuple(shape[:ndim.value]), dtype.value, exponent.value, host.value, device.value)

    def run(self):
        """Host buffers -> device, execute, device -> host buffers (the call a user of dl::Model makes)."""
        abi.check(self.lib.espdl_model_run(self.h), "Model::run")

    def reset(self):
        """dl::Model::reset(): clears what modules keep between runs (streaming caches)."""
        self.lib.espdl_model_reset.restype = None
        self.lib.espdl_model_reset.argtypes = [C.c_void_p]
        self.lib.espdl_model_reset(self.h)

    def minimize(self):
        """dl::Model::minimize(): releases what inference does not need (host copies of the parameters that are resident
        on the device, name maps, module registry).  test() is no longer possible afterwards."""
        self.lib.espdl_model_minimize.restype = None
        self.lib.espdl_model_minimize.argtypes = [C.c_void_p]
        self.lib.espdl_model_minimize(self.h)

    def submit(self):
        """Pipelined run(): uploads the input arrays (they may be refilled when this returns) and enqueues the pass."""
        abi.check(self.lib.espdl_model_submit(self.h), "Model::submit")

    def wait(self):
        """Blocks until the oldest submitted pass is done; its results are then in the output arrays."""
        abi.check(self.lib.espdl_model_wait(self.h), "Model::wait")

    def preprocess(self, images, mean, std, rgb_swap=False, letterbox=None, crop=None):
        """dl::image::ImagePreprocessor: uint8 images [n][h][w][c] (host) -> the model's first input tensor on the device
        (crop, nearest resize, optional letterbox with that background value, normalise + quantise).  Follow with
        run_device(), which executes on what is resident."""
        images = np.ascontiguousarray(images, dtype=np.uint8)
        n, h, w, c = images.shape
        mean = (C.c_float * 3)(*(list(np.atleast_1d(mean)) + [0, 0])[:3])
        std = (C.c_float * 3)(*(list(np.atleast_1d(std)) + [1, 1])[:3])
        crop_arr = (C.c_int * 4)(*crop) if crop is not None else None
        st = self.lib.espdl_model_preprocess(self.h, images.ctypes.data, n, h, w, c, mean, std, int(rgb_swap),
                                             -1 if letterbox is None else int(letterbox), crop_arr)
        if st != 0:
            raise RuntimeError("ImagePreprocessor::preprocess failed")

    def classify(self, image=0, top_k=5, score_thr=0.0, need_softmax=True):
        """dl::cls::ClsPostprocessor: [(category, score)] of one image of the batch, best first."""
        cats, scores = (C.c_int * top_k)(), (C.c_float * top_k)()
        n = self.lib.espdl_model_classify(self.h, image, top_k, score_thr, int(need_softmax), cats, scores)
        if n < 0:
            raise RuntimeError("ClsPostprocessor::postprocess failed")
        return [(cats[i], scores[i]) for i in range(n)]

    def detect(self, heads, strides, score_thr, nms_thr, top_k, width, height, image=0, max_results=300):
        """dl::detect::yolo11PostProcessor: heads = [(box output name, score output name)] per stage.  Returns
        [(category, score, (x0, y0, x1, y1))] of one image, best first."""
        names = (C.c_char_p * (2 * len(heads)))(*[n.encode() for pair in heads for n in pair])
        boxes, scores = (C.c_int * (5 * max_results))(), (C.c_float * max_results)()
        n = self.lib.espdl_model_detect(self.h, image, len(heads), names, (C.c_int * len(heads))(*strides), score_thr, nms_thr, top_k,
                                        width, height, max_results, boxes, scores)
        if n < 0:
            raise RuntimeError("yolo11PostProcessor::postprocess failed")
        return [(boxes[5 * i], scores[i], tuple(boxes[5 * i + 1:5 * i + 5])) for i in range(n)]

    def run_device(self, sync=True):
        abi.check(self.lib.espdl_model_run_device(self.h, 1 if sync else 0), "Model::run_device")

    def test(self):
        return self.lib.espdl_model_test(self.h)

    @property
    def stream(self):
        return self.lib.espdl_model_stream(self.h)

    @property
    def arena_bytes(self):
        return self.lib.espdl_model_arena_bytes(self.h)

    @property
    def num_modules(self):
        return self.lib.espdl_model_num_modules(self.h)

    def num_slice_views(self):
        """Tensors that live as channel slices inside a Concat output / Split input (ESPDL_B200_SLICE_VIEWS=0: none)."""
        return self.lib.espdl_model_num_slice_views(self.h)

    def read_tensor(self, name, dtype, shape):
        out = np.empty(shape, dtype=dtype)
        n = self.lib.espdl_model_read_tensor(self.h, name.encode(), out.ctypes.data, out.nbytes)
        if n < 0 or n != out.nbytes:
            raise RuntimeError(f"read_tensor({name}) -> {n}, expected {out.nbytes}")
        return out

    def profile(self):
        rows = []
        for line in self.lib.espdl_model_profile(self.h).decode().splitlines():
            idx, typ, us, name = line.split("\t")
            rows.append((int(idx), typ, float(us), name))
        return rows

    def close(self):
        if self.h:
            self.lib.espdl_model_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
