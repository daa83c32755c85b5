"""Reader and writer for the `.espdl` model container (EDL2 header + FlatBuffers `espdl.Model`).

Format facts (reference: esp-dl/fbs_loader/espdl.fbs:1-215 for the schema,
esp-dl/fbs_loader/src/fbs_loader.cpp:278-301 for the 16-byte EDL2 header
"EDL2" | u32 mode | u32 size | u32 pad):
  * tensors are NHWC, conv filters are declared [KH,KW,Cin,Cout], payload lives in
    `raw_data` (a vector of 16-byte structs), `exponents` has length 1 (per tensor) or Cout;
  * node attributes are typed (`i`, `f`, `s`, `ints`, `floats`, ...).

The writer exists because the tool that normally exports `.espdl` files (esp-ppq) is a separate
project: tests and the benchmark build their synthetic networks with it.  It emits a forward-laid-out
FlatBuffer (every uoffset points forward, vtables precede their tables), which any FlatBuffers reader
accepts.  Only the plain (mode 0, unencrypted) EDL2 container is written.
"""
import struct

import numpy as np

# ----------------------------------------------------------------------------- schema (field ids)
MODEL = dict(ir_version=0, opset_import=1, producer_name=2, producer_version=3, domain=4, model_version=5,
             doc_string=6, graph=7, metadata_props=8, functions=9)
GRAPH = dict(node=0, name=1, initializer=2, doc_string=3, input=4, output=5, value_info=6,
             quantization_annotation=7, test_inputs_value=8, test_outputs_value=9)
NODE = dict(input=0, output=1, name=2, op_type=3, domain=4, attribute=5, doc_string=6)
ATTR = dict(name=0, ref_attr_name=1, doc_string=2, attr_type=3, f=4, i=5, s=6, t=7, g=8, tp=9, floats=10, ints=11,
            strings=12, tensors=13, graphs=14, type_protos=15)
TENSOR = dict(dims=0, data_type=1, float_data=2, int32_data=3, string_data=4, int64_data=5, name=6, doc_string=7,
              raw_data=8, external_data=9, data_location=10, double_data=11, uint64_data=12, exponents=13)
VALUE_INFO = dict(name=0, value_info_type=1, doc_string=2, exponents=3)
TYPE_INFO = dict(value_type=0, value=1, denotation=2)  # a union occupies two slots: type tag, then value
TENSOR_TYPE = dict(elem_type=0, shape=1)
SHAPE = dict(dim=0)
DIMENSION = dict(value=0, denotation=1)
DIM_VALUE = dict(dim_type=0, dim_value=1, dim_param=2)
KV = dict(key=0, value=1)

ATTR_FLOAT, ATTR_INT, ATTR_STRING, ATTR_TENSOR, ATTR_FLOATS, ATTR_INTS = 1, 2, 3, 4, 6, 7
DT_FLOAT, DT_UINT8, DT_INT8, DT_UINT16, DT_INT16, DT_INT32, DT_INT64 = 1, 2, 3, 4, 5, 6, 7
NP_OF = {DT_FLOAT: np.float32, DT_UINT8: np.uint8, DT_INT8: np.int8, DT_UINT16: np.uint16, DT_INT16: np.int16,
         DT_INT32: np.int32, DT_INT64: np.int64, 9: np.bool_, 11: np.float64}
DT_OF = {np.dtype(v): k for k, v in NP_OF.items()}


# ----------------------------------------------------------------------------- reader
class _Table:
    def __init__(self, buf, pos):
        self.buf, self.pos = buf, pos
        self.vt = pos - struct.unpack_from("<i", buf, pos)[0]
        self.vt_size = struct.unpack_from("<H", buf, self.vt)[0]

    def _off(self, fid):
        o = 4 + 2 * fid
        if o >= self.vt_size:
            return 0
        return struct.unpack_from("<H", self.buf, self.vt + o)[0]

    def scalar(self, fid, fmt, default=0):
        o = self._off(fid)
        return struct.unpack_from("<" + fmt, self.buf, self.pos + o)[0] if o else default

    def _indirect(self, fid):
        o = self._off(fid)
        if not o:
            return None
        p = self.pos + o
        return p + struct.unpack_from("<I", self.buf, p)[0]

    def table(self, fid):
        p = self._indirect(fid)
        return _Table(self.buf, p) if p is not None else None

    def string(self, fid):
        p = self._indirect(fid)
        if p is None:
            return None
        n = struct.unpack_from("<I", self.buf, p)[0]
        return bytes(self.buf[p + 4:p + 4 + n]).decode("utf-8", "replace")

    def vector(self, fid, fmt=None, elem_size=None):
        """Scalar vector -> numpy array (fmt = numpy dtype); raw struct vector -> bytes (elem_size)."""
        p = self._indirect(fid)
        if p is None:
            return None
        n = struct.unpack_from("<I", self.buf, p)[0]
        if fmt is not None:
            return np.frombuffer(self.buf, dtype=fmt, count=n, offset=p + 4).copy()
        return bytes(self.buf[p + 4:p + 4 + n * elem_size])

    def tables(self, fid):
        p = self._indirect(fid)
        if p is None:
            return []
        n = struct.unpack_from("<I", self.buf, p)[0]
        out = []
        for i in range(n):
            q = p + 4 + 4 * i
            out.append(_Table(self.buf, q + struct.unpack_from("<I", self.buf, q)[0]))
        return out

    def strings(self, fid):
        p = self._indirect(fid)
        if p is None:
            return []
        n = struct.unpack_from("<I", self.buf, p)[0]
        out = []
        for i in range(n):
            q = p + 4 + 4 * i
            s = q + struct.unpack_from("<I", self.buf, q)[0]
            ln = struct.unpack_from("<I", self.buf, s)[0]
            out.append(bytes(self.buf[s + 4:s + 4 + ln]).decode())
        return out


def _read_tensor(t):
    dims = t.vector(TENSOR["dims"], np.int64)
    dims = [] if dims is None else [int(x) for x in dims]
    dt = t.scalar(TENSOR["data_type"], "i")
    raw = t.vector(TENSOR["raw_data"], elem_size=16)
    npdt = NP_OF.get(dt)
    numel = int(np.prod(dims)) if dims else 1
    data = None
    if raw is not None and npdt is not None:
        data = np.frombuffer(raw, dtype=npdt, count=numel).reshape(dims if dims else ()).copy()
    else:
        for fid, fmt in ((TENSOR["float_data"], np.float32), (TENSOR["int32_data"], np.int32), (TENSOR["int64_data"], np.int64)):
            v = t.vector(fid, fmt)
            if v is not None and len(v):
                data = v.reshape(dims) if dims else v
                break
    exps = t.vector(TENSOR["exponents"], np.int64)
    return dict(name=t.string(TENSOR["name"]), dims=dims, data_type=dt, data=data,
                exponents=[] if exps is None else [int(e) for e in exps])


def _read_value_info(v):
    ti = v.table(VALUE_INFO["value_info_type"])
    shape, elem = None, 0
    if ti is not None and ti.scalar(TYPE_INFO["value_type"], "B") == 1:
        tt = ti.table(TYPE_INFO["value"])
        elem = tt.scalar(TENSOR_TYPE["elem_type"], "i")
        sh = tt.table(TENSOR_TYPE["shape"])
        if sh is not None:
            shape = []
            for dim in sh.tables(SHAPE["dim"]):
                dv = dim.table(DIMENSION["value"])
                shape.append(int(dv.scalar(DIM_VALUE["dim_value"], "q")) if dv is not None else -1)
    exps = v.vector(VALUE_INFO["exponents"], np.int64)
    return dict(name=v.string(VALUE_INFO["name"]), elem_type=elem, shape=shape,
                exponents=[] if exps is None else [int(e) for e in exps])


def _read_attr(a):
    ty = a.scalar(ATTR["attr_type"], "i")
    name = a.string(ATTR["name"])
    if ty == ATTR_INT:
        o = a._off(ATTR["i"])
        val = struct.unpack_from("<q", a.buf, a.pos + o)[0] if o else 0
    elif ty == ATTR_FLOAT:
        o = a._off(ATTR["f"])
        val = struct.unpack_from("<f", a.buf, a.pos + o)[0] if o else 0.0
    elif ty == ATTR_STRING:
        v = a.vector(ATTR["s"], np.uint8)
        val = bytes(v).decode() if v is not None else ""
    elif ty == ATTR_INTS:
        v = a.vector(ATTR["ints"], np.int64)
        val = [] if v is None else [int(x) for x in v]
    elif ty == ATTR_FLOATS:
        v = a.vector(ATTR["floats"], np.float32)
        val = [] if v is None else [float(x) for x in v]
    elif ty == ATTR_TENSOR:
        t = a.table(ATTR["t"])
        val = _read_tensor(t) if t is not None else None
    else:
        val = None
    return name, ty, val


def payload(blob):
    """Strip the container header and return the FlatBuffer bytes."""
    magic = bytes(blob[:4])
    if magic == b"EDL2":
        mode, size = struct.unpack_from("<II", blob, 4)
        if mode != 0:
            raise ValueError("encrypted .espdl is not supported by this reader")
        return memoryview(blob)[16:16 + size]
    if magic == b"EDL1":
        mode, size = struct.unpack_from("<II", blob, 4)
        if mode != 0:
            raise ValueError("encrypted .espdl is not supported by this reader")
        return memoryview(blob)[12:12 + size]
    raise ValueError(f"unknown container magic {magic!r}")


def read(path_or_bytes):
    """Parse an .espdl file into plain Python structures (dict of nodes / tensors / value infos)."""
    blob = path_or_bytes if isinstance(path_or_bytes, (bytes, bytearray)) else open(path_or_bytes, "rb").read()
    buf = payload(blob)
    root = _Table(buf, struct.unpack_from("<I", buf, 0)[0])
    g = root.table(MODEL["graph"])
    meta = {kv.string(KV["key"]): kv.string(KV["value"]) for kv in root.tables(MODEL["metadata_props"])}
    nodes = []
    for n in g.tables(GRAPH["node"]):
        attrs = {}
        for a in n.tables(NODE["attribute"]):
            name, ty, val = _read_attr(a)
            attrs[name] = val
        nodes.append(dict(name=n.string(NODE["name"]), op_type=n.string(NODE["op_type"]), inputs=n.strings(NODE["input"]),
                          outputs=n.strings(NODE["output"]), attrs=attrs))
    return dict(
        name=g.string(GRAPH["name"]), metadata=meta, nodes=nodes,
        doc_string=root.string(MODEL["doc_string"]), version=root.scalar(MODEL["model_version"], "q"),
        initializers={t["name"]: t for t in map(_read_tensor, g.tables(GRAPH["initializer"]))},
        inputs=[_read_value_info(v) for v in g.tables(GRAPH["input"])],
        outputs=[_read_value_info(v) for v in g.tables(GRAPH["output"])],
        value_info={v["name"]: v for v in map(_read_value_info, g.tables(GRAPH["value_info"]))},
        test_inputs={t["name"]: t for t in map(_read_tensor, g.tables(GRAPH["test_inputs_value"]))},
        test_outputs={t["name"]: t for t in map(_read_tensor, g.tables(GRAPH["test_outputs_value"]))},
    )


# ----------------------------------------------------------------------------- writer
class _Obj:
    """A node of the object tree to serialise.  kind: 'table', 'string', 'vec_scalar', 'vec_off', 'vec_raw16'."""
    __slots__ = ("kind", "data", "pos", "fmt")

    def __init__(self, kind, data, fmt=None):
        self.kind, self.data, self.fmt, self.pos = kind, data, fmt, None


def fb_string(s):
    return _Obj("string", s.encode() if isinstance(s, str) else bytes(s))


def fb_vec(values, fmt):
    return _Obj("vec_scalar", np.asarray(values, dtype=fmt), fmt)


def fb_vec_off(objs):
    return _Obj("vec_off", list(objs))


def fb_raw16(b):
    b = bytes(b)
    b += bytes((-len(b)) % 16)
    return _Obj("vec_raw16", b)


def fb_table(fields):
    """fields: dict field_id -> ('q', value) scalar | ('struct', bytes, align) | _Obj child."""
    return _Obj("table", fields)


class _Writer:
    def __init__(self):
        self.buf = bytearray()
        self.patches = []  # (location of a uoffset, target object)

    def align(self, a):
        self.buf += bytes((-len(self.buf)) % a)

    def emit(self, root):
        self.buf += bytes(4)  # root uoffset
        self.buf += bytes(12)  # keep the first object 16-byte aligned
        order = [root]
        i = 0
        while i < len(order):  # breadth-first: every child is laid out after its parent => forward uoffsets
            o = order[i]
            i += 1
            self._emit_one(o, order)
        struct.pack_into("<I", self.buf, 0, root.pos)
        for loc, target in self.patches:
            assert target.pos > loc
            struct.pack_into("<I", self.buf, loc, target.pos - loc)
        return bytes(self.buf)

    def _emit_one(self, o, order):
        if o.pos is not None:
            return
        b = self.buf
        if o.kind == "string":
            self.align(4)
            o.pos = len(b)
            b += struct.pack("<I", len(o.data)) + o.data + b"\0"
        elif o.kind == "vec_scalar":
            item = o.data.dtype.itemsize
            self.align(4)
            while (len(b) + 4) % max(item, 4):
                b += b"\0"
            o.pos = len(b)
            b += struct.pack("<I", len(o.data)) + o.data.tobytes()
        elif o.kind == "vec_raw16":
            self.align(4)
            while (len(b) + 4) % 16:
                b += b"\0"
            o.pos = len(b)
            b += struct.pack("<I", len(o.data) // 16) + o.data
        elif o.kind == "vec_off":
            self.align(4)
            o.pos = len(b)
            b += struct.pack("<I", len(o.data))
            for child in o.data:
                self.patches.append((len(b), child))
                b += bytes(4)
                order.append(child)
        elif o.kind == "table":
            fields = o.data
            nf = (max(fields) + 1) if fields else 0
            # layout of the table body: soffset(4) then fields, each aligned to its size
            body = bytearray(4)
            offs = [0] * nf
            child_locs = []
            for fid in sorted(fields, key=lambda f: -self._fsize(fields[f])):  # big scalars first: less padding
                v = fields[fid]
                size = self._fsize(v)
                while len(body) % size:
                    body += b"\0"
                offs[fid] = len(body)
                if isinstance(v, _Obj):
                    child_locs.append((len(body), v))
                    body += bytes(4)
                elif v[0] == "struct":
                    body += v[1]
                else:
                    body += struct.pack("<" + v[0], v[1])
            vt = struct.pack("<HH", 4 + 2 * nf, len(body)) + b"".join(struct.pack("<H", x) for x in offs)
            self.align(2)
            # place the vtable so that the table body that follows is 8-byte aligned
            while (len(b) + len(vt)) % 8:
                b += b"\0"
            vt_pos = len(b)
            b += vt
            o.pos = len(b)
            struct.pack_into("<i", body, 0, o.pos - vt_pos)
            b += body
            for loc, child in child_locs:
                self.patches.append((o.pos + loc, child))
                order.append(child)

    @staticmethod
    def _fsize(v):
        if isinstance(v, _Obj):
            return 4
        if v[0] == "struct":
            return v[2]
        return struct.calcsize("<" + v[0])


def _tensor_obj(name, arr, exponents=None):
    arr = np.ascontiguousarray(arr)
    f = {TENSOR["dims"]: fb_vec(list(arr.shape), np.int64), TENSOR["data_type"]: ("i", DT_OF[arr.dtype]),
         TENSOR["name"]: fb_string(name), TENSOR["raw_data"]: fb_raw16(arr.tobytes())}
    if exponents is not None:
        f[TENSOR["exponents"]] = fb_vec(list(exponents), np.int64)
    return fb_table(f)


def _value_info_obj(name, np_dtype, shape, exponents=None):
    dims = [fb_table({DIMENSION["value"]: fb_table({DIM_VALUE["dim_type"]: ("b", 1), DIM_VALUE["dim_value"]: ("q", int(s))})})
            for s in shape]
    tt = fb_table({TENSOR_TYPE["elem_type"]: ("i", DT_OF[np.dtype(np_dtype)]),
                   TENSOR_TYPE["shape"]: fb_table({SHAPE["dim"]: fb_vec_off(dims)})})
    ti = fb_table({TYPE_INFO["value_type"]: ("B", 1), TYPE_INFO["value"]: tt})
    f = {VALUE_INFO["name"]: fb_string(name), VALUE_INFO["value_info_type"]: ti}
    if exponents is not None:
        f[VALUE_INFO["exponents"]] = fb_vec(list(exponents), np.int64)
    return fb_table(f)


def _attr_obj(name, value):
    f = {ATTR["name"]: fb_string(name)}
    if isinstance(value, bool) or isinstance(value, (int, np.integer)):
        f[ATTR["attr_type"]] = ("i", ATTR_INT)
        f[ATTR["i"]] = ("struct", struct.pack("<q", int(value)), 8)
    elif isinstance(value, float):
        f[ATTR["attr_type"]] = ("i", ATTR_FLOAT)
        f[ATTR["f"]] = ("struct", struct.pack("<f", value), 4)
    elif isinstance(value, str):
        f[ATTR["attr_type"]] = ("i", ATTR_STRING)
        f[ATTR["s"]] = fb_vec(np.frombuffer(value.encode(), dtype=np.uint8), np.uint8)
    elif isinstance(value, (list, tuple)) and all(isinstance(v, (int, np.integer)) for v in value):
        f[ATTR["attr_type"]] = ("i", ATTR_INTS)
        f[ATTR["ints"]] = fb_vec(list(value), np.int64)
    elif isinstance(value, (list, tuple)):
        f[ATTR["attr_type"]] = ("i", ATTR_FLOATS)
        f[ATTR["floats"]] = fb_vec(list(value), np.float32)
    else:
        raise TypeError(f"attribute {name}: unsupported value {value!r}")
    return fb_table(f)


class GraphBuilder:
    """Collects nodes / tensors and serialises them as an EDL2 `.espdl` blob."""

    def __init__(self, name="model", metadata=None):
        self.name = name
        self.metadata = dict(metadata or {})
        self.nodes, self.initializers, self.inputs, self.outputs = [], [], [], []
        self.value_info, self.test_inputs, self.test_outputs = [], [], []

    def add_initializer(self, name, arr, exponents=None):
        self.initializers.append((name, np.asarray(arr), exponents))
        return name

    def add_value_info(self, name, np_dtype, shape, exponent=None):
        self.value_info.append((name, np_dtype, list(shape), None if exponent is None else [exponent]))
        return name

    def add_input(self, name, np_dtype, shape, exponent):
        self.inputs.append((name, np_dtype, list(shape), [exponent]))
        return name

    def add_output(self, name, np_dtype, shape, exponent):
        self.outputs.append((name, np_dtype, list(shape), [exponent]))
        return name

    def add_node(self, op_type, name, inputs, outputs, **attrs):
        self.nodes.append((op_type, name, list(inputs), list(outputs), attrs))
        return outputs[0]

    def add_test_value(self, name, arr, exponent, is_input):
        (self.test_inputs if is_input else self.test_outputs).append((name, np.asarray(arr), [exponent]))

    def serialize(self):
        nodes = []
        for op, name, ins, outs, attrs in self.nodes:
            f = {NODE["input"]: fb_vec_off([fb_string(s) for s in ins]), NODE["output"]: fb_vec_off([fb_string(s) for s in outs]),
                 NODE["name"]: fb_string(name), NODE["op_type"]: fb_string(op)}
            if attrs:
                f[NODE["attribute"]] = fb_vec_off([_attr_obj(k, v) for k, v in attrs.items()])
            nodes.append(fb_table(f))
        g = {GRAPH["node"]: fb_vec_off(nodes), GRAPH["name"]: fb_string(self.name),
             GRAPH["initializer"]: fb_vec_off([_tensor_obj(*t) for t in self.initializers]),
             GRAPH["input"]: fb_vec_off([_value_info_obj(*v) for v in self.inputs]),
             GRAPH["output"]: fb_vec_off([_value_info_obj(*v) for v in self.outputs]),
             GRAPH["value_info"]: fb_vec_off([_value_info_obj(*v) for v in self.value_info])}
        if self.test_inputs:
            g[GRAPH["test_inputs_value"]] = fb_vec_off([_tensor_obj(*t) for t in self.test_inputs])
        if self.test_outputs:
            g[GRAPH["test_outputs_value"]] = fb_vec_off([_tensor_obj(*t) for t in self.test_outputs])
        m = {MODEL["ir_version"]: ("i", 1), MODEL["producer_name"]: fb_string("espdl_b200"), MODEL["graph"]: fb_table(g)}
        if self.metadata:
            m[MODEL["metadata_props"]] = fb_vec_off(
                [fb_table({KV["key"]: fb_string(k), KV["value"]: fb_string(v)}) for k, v in self.metadata.items()])
        fb = _Writer().emit(fb_table(m))
        fb += bytes((-len(fb)) % 16)
        return b"EDL2" + struct.pack("<III", 0, len(fb), 0) + fb

    def save(self, path):
        with open(path, "wb") as f:
            f.write(self.serialize())


# ----------------------------------------------------------------------------- filter memory layouts
def filter_to_ohwi(flat, dims, target):
    """Re-order a conv / Gemm filter payload into [Cout][KH][KW][Cin].

    The declared shape is always [KH,KW,Cin,Cout] but the byte order depends on the export target
    (esp-dl/dl/base/dl_base_conv2d.cpp:23-32,140-162; esp-dl/dl/base/dl_base.hpp:305-310):
      "c"                 [Cout][KH][KW][Cin]
      "esp32p4"/"esp32s3" [Cout/u][KH][KW][Cin][u] followed by the Cout%u tail as [n][KH][KW][Cin], u = 16 bytes / itemsize
    """
    flat = np.asarray(flat).reshape(-1)
    kh, kw, cin, cout = [int(d) for d in dims]
    if target in (None, "", "c"):
        return flat.reshape(cout, kh, kw, cin).copy()
    u = 16 // flat.dtype.itemsize
    nb = cout // u
    out = np.empty((cout, kh, kw, cin), dtype=flat.dtype)
    body = flat[:nb * u * kh * kw * cin].reshape(nb, kh, kw, cin, u)
    out[:nb * u] = body.transpose(0, 4, 1, 2, 3).reshape(nb * u, kh, kw, cin)
    tail = flat[nb * u * kh * kw * cin:cout * kh * kw * cin]
    if cout % u:
        out[nb * u:] = tail.reshape(cout % u, kh, kw, cin)
    return out


def depthwise_filter_to_hwc(flat, dims, target):
    """Depthwise filter payload -> [KH][KW][C].  Declared [KH,KW,C,1]; "c" stores [KH][KW][C]
    (esp-dl/dl/base/dl_base_depthwise_conv2d.cpp:47-66); the SIMD targets store
    [C/u][KH][KW][u] followed by the C%u tail as [KH][KW][C%u] (esp-dl/dl/base/dl_base.hpp:1255-1262)."""
    flat = np.asarray(flat).reshape(-1)
    kh, kw, c = int(dims[0]), int(dims[1]), int(dims[2])
    if target in (None, "", "c"):
        return flat.reshape(kh, kw, c).copy()
    u = 16 // flat.dtype.itemsize
    nb = c // u
    out = np.empty((kh, kw, c), dtype=flat.dtype)
    body = flat[:nb * u * kh * kw].reshape(nb, kh, kw, u)
    out[:, :, :nb * u] = body.transpose(1, 2, 0, 3).reshape(kh, kw, nb * u)
    if c % u:
        out[:, :, nb * u:] = flat[nb * u * kh * kw:c * kh * kw].reshape(kh, kw, c % u)
    return out
