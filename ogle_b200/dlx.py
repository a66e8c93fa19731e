"""dlx model files in Python: message classes, proto3 wire encoder and decoder.

A dlx file is the binary protobuf encoding of dlxnet.ModelProto
(ogl_runtime/opengl/core/dlxnet.proto in kl456123/OGLE). No protoc is needed:
the few wire rules in use (varint, fixed32, length-delimited, packed repeated
scalars) are implemented here. The C++ runtime has its own reader
(csrc/runtime/dlx.cc); tests round-trip files between the two.
"""
import struct

import numpy as np

# dlxnet.TensorProto.DataFormat / DataType
NCHW, NHWC, NHWC4, HWN4C4, ANY, ANY4 = 0, 1, 3, 4, 5, 6
FLOAT32, FLOAT16, INT32, INT8 = 0, 1, 2, 3

# Attribute sub-message field numbers (dlxnet.proto:158-182)
ATTR_FIELDS = {
    "conv2d_attr": 1, "const_attr": 2, "batchnorm_attr": 3, "relu_attr": 4, "maxpool_attr": 5, "avepool_attr": 6,
    "flatten_attr": 7, "binary_attr": 8, "gemm_attr": 9, "input_attr": 10, "clip_attr": 11, "transpose_attr": 12,
    "shape_attr": 13, "gather_attr": 14, "unsqueeze_attr": 15, "concat_attr": 16, "reshape_attr": 17,
}
# per sub-message: field name -> (number, kind); kinds: ints (packed varints), int, float, str, tensor
ATTR_SCHEMAS = {
    "conv2d_attr": {"kernel_shape": (1, "ints"), "strides": (2, "ints"), "pads": (3, "ints"), "dilations": (4, "ints"),
                    "group": (5, "int"), "activation_type": (6, "str"), "min": (7, "float"), "max": (8, "float")},
    "const_attr": {"value": (1, "tensor")},
    "batchnorm_attr": {"momentum": (1, "float"), "epsilon": (2, "float")},
    "relu_attr": {"slope": (1, "float")},
    "maxpool_attr": {"kernel_shape": (1, "ints"), "strides": (2, "ints"), "pads": (3, "ints")},
    "avepool_attr": {"kernel_shape": (1, "ints"), "strides": (2, "ints"), "pads": (3, "ints")},
    "flatten_attr": {"axis": (1, "int")},
    "binary_attr": {"binary_op_type": (1, "str")},
    "gemm_attr": {"alpha": (1, "float"), "beta": (2, "float"), "transB": (3, "int")},
    "input_attr": {"dims": (3, "ints")},
    "clip_attr": {"min": (1, "float"), "max": (2, "float")},
    "transpose_attr": {"perm": (1, "ints")},
    "shape_attr": {},
    "gather_attr": {"axis": (1, "int")},
    "unsqueeze_attr": {"axes": (1, "ints")},
    "concat_attr": {"axis": (1, "int")},
    "reshape_attr": {"axis": (1, "int")},
}


# ------------------------------------------------------------------ encoding
def _varint(v):
    v &= (1 << 64) - 1          # negative values use the 64-bit two's complement
    out = bytearray()
    while v >= 0x80:
        out.append((v & 0x7F) | 0x80)
        v >>= 7
    out.append(v)
    return bytes(out)


def _tag(field, wire):
    return _varint(field << 3 | wire)


def _bytes(field, b):
    return _tag(field, 2) + _varint(len(b)) + b


def _int(field, v):
    return _tag(field, 0) + _varint(int(v)) if v else b""


def _float(field, v):
    b = struct.pack("<f", v)
    return _tag(field, 5) + b if b != b"\0\0\0\0" else b""


def _str(field, s):
    return _bytes(field, s.encode()) if s else b""


def _ints(field, vs):
    vs = list(vs)
    return _bytes(field, b"".join(_varint(int(v)) for v in vs)) if vs else b""


class Tensor:
    """dlxnet.TensorProto"""

    def __init__(self, dims, float_data, data_format=ANY, target_data_format=ANY4, data_type=FLOAT32):
        self.dims = [int(d) for d in dims]
        self.float_data = np.ascontiguousarray(float_data, dtype="<f4").reshape(-1)
        self.int32_data = []
        self.data_format = data_format
        self.target_data_format = target_data_format
        self.data_type = data_type

    def encode(self):
        out = _int(1, self.data_format) + _int(2, self.data_type) + _ints(3, self.dims)
        if self.float_data.size:
            out += _bytes(4, self.float_data.tobytes())
        out += _ints(5, self.int32_data)
        out += _int(8, self.target_data_format)
        return out


def _encode_attr_message(kind, values):
    out = b""
    for name, (num, k) in sorted(ATTR_SCHEMAS[kind].items(), key=lambda kv: kv[1][0]):
        if name not in values:
            continue
        v = values[name]
        if k == "ints":
            out += _ints(num, v)
        elif k == "int":
            out += _int(num, v)
        elif k == "float":
            out += _float(num, v)
        elif k == "str":
            out += _str(num, v)
        elif k == "tensor":
            out += _bytes(num, v.encode())
    return out


class Node:
    """dlxnet.NodeProto. attr: {"conv2d_attr": {...}, ...}"""

    def __init__(self, name, type_, inputs=(), outputs=(), attr=None, doc_string=""):
        self.name, self.type = name, type_
        self.input_index, self.output_index = list(inputs), list(outputs)
        self.attr = attr or {}
        self.doc_string = doc_string

    def encode(self):
        a = b""
        for kind in sorted(self.attr, key=lambda k: ATTR_FIELDS[k]):
            a += _bytes(ATTR_FIELDS[kind], _encode_attr_message(kind, self.attr[kind]))
        out = _ints(1, self.input_index) + _ints(2, self.output_index)
        if a:
            out += _bytes(3, a)
        return out + _str(4, self.doc_string) + _str(5, self.name) + _str(6, self.type)


class Model:
    """dlxnet.ModelProto with its GraphProto flattened in."""

    def __init__(self, producer_name="ONNX", version="0.1", doc_string=""):
        self.producer_name, self.version, self.doc_string = producer_name, version, doc_string
        self.graph_name = ""
        self.nodes, self.tensor_names, self.input_names, self.output_names = [], [], [], []

    def encode(self):
        g = b"".join(_bytes(1, n.encode()) for n in self.nodes)
        g += _str(2, self.graph_name)
        g += b"".join(_bytes(3, s.encode()) for s in self.tensor_names)
        g += b"".join(_bytes(4, s.encode()) for s in self.output_names)
        g += b"".join(_bytes(5, s.encode()) for s in self.input_names)
        return _bytes(1, g) + _str(2, self.version) + _str(3, self.producer_name) + _str(4, self.doc_string)

    def save(self, path):
        with open(path, "wb") as f:
            f.write(self.encode())


# ------------------------------------------------------------------ decoding
class _Reader:
    def __init__(self, buf, pos=0, end=None):
        self.buf, self.pos, self.end = buf, pos, len(buf) if end is None else end

    def done(self):
        return self.pos >= self.end

    def varint(self):
        v, shift = 0, 0
        while True:
            if self.pos >= self.end:
                raise ValueError("truncated varint")
            b = self.buf[self.pos]
            self.pos += 1
            v |= (b & 0x7F) << shift
            if not b & 0x80:
                return v
            shift += 7
            if shift > 63:
                raise ValueError("varint too long")

    def sub(self):
        n = self.varint()
        if self.pos + n > self.end:
            raise ValueError("length-delimited field overruns its parent")
        r = _Reader(self.buf, self.pos, self.pos + n)
        self.pos += n
        return r

    def raw(self):
        r = self.sub()
        return bytes(self.buf[r.pos:r.end])

    def fixed32(self):
        if self.pos + 4 > self.end:
            raise ValueError("truncated fixed32")
        b = self.buf[self.pos:self.pos + 4]
        self.pos += 4
        return b

    def skip(self, wire):
        if wire == 0:
            self.varint()
        elif wire == 1:
            self.pos += 8
        elif wire == 2:
            self.sub()
        elif wire == 5:
            self.pos += 4
        else:
            raise ValueError("unsupported wire type %d" % wire)

    def fields(self):
        while not self.done():
            t = self.varint()
            yield t >> 3, t & 7


def _signed(v):
    return v - (1 << 64) if v >= 1 << 63 else v


def _read_ints(r, wire, out):
    if wire == 2:
        s = r.sub()
        while not s.done():
            out.append(_signed(s.varint()))
    else:
        out.append(_signed(r.varint()))


def _decode_tensor(r):
    t = Tensor([], np.zeros(0, np.float32), NCHW, NCHW)
    floats = []
    for f, w in r.fields():
        if f == 1:
            t.data_format = r.varint()
        elif f == 2:
            t.data_type = r.varint()
        elif f == 3:
            _read_ints(r, w, t.dims)
        elif f == 4:
            floats.append(np.frombuffer(r.raw(), dtype="<f4") if w == 2 else np.frombuffer(r.fixed32(), dtype="<f4"))
        elif f == 5:
            _read_ints(r, w, t.int32_data)
        elif f == 8:
            t.target_data_format = r.varint()
        else:
            r.skip(w)
    if floats:
        t.float_data = np.concatenate(floats)
    return t


def _decode_attr_message(kind, r):
    schema = {num: (name, k) for name, (num, k) in ATTR_SCHEMAS[kind].items()}
    vals = {}
    for f, w in r.fields():
        if f not in schema:
            r.skip(w)
            continue
        name, k = schema[f]
        if k == "ints":
            _read_ints(r, w, vals.setdefault(name, []))
        elif k == "int":
            vals[name] = _signed(r.varint())
        elif k == "float":
            vals[name] = struct.unpack("<f", r.fixed32())[0]
        elif k == "str":
            vals[name] = r.raw().decode()
        elif k == "tensor":
            vals[name] = _decode_tensor(r.sub())
    return vals


def decode(buf):
    """bytes -> Model"""
    m = Model("", "", "")
    kinds = {v: k for k, v in ATTR_FIELDS.items()}
    for f, w in (r := _Reader(memoryview(buf))).fields():
        if f == 1 and w == 2:
            g = r.sub()
            for gf, gw in g.fields():
                if gf == 1 and gw == 2:
                    nr = g.sub()
                    n = Node("", "")
                    for nf, nw in nr.fields():
                        if nf == 1:
                            _read_ints(nr, nw, n.input_index)
                        elif nf == 2:
                            _read_ints(nr, nw, n.output_index)
                        elif nf == 3 and nw == 2:
                            ar = nr.sub()
                            for af, aw in ar.fields():
                                if af in kinds and aw == 2:
                                    n.attr[kinds[af]] = _decode_attr_message(kinds[af], ar.sub())
                                else:
                                    ar.skip(aw)
                        elif nf == 4:
                            n.doc_string = nr.raw().decode()
                        elif nf == 5:
                            n.name = nr.raw().decode()
                        elif nf == 6:
                            n.type = nr.raw().decode()
                        else:
                            nr.skip(nw)
                    m.nodes.append(n)
                elif gf == 2:
                    m.graph_name = g.raw().decode()
                elif gf == 3:
                    m.tensor_names.append(g.raw().decode())
                elif gf == 4:
                    m.output_names.append(g.raw().decode())
                elif gf == 5:
                    m.input_names.append(g.raw().decode())
                else:
                    g.skip(gw)
        elif f == 2:
            m.version = r.raw().decode()
        elif f == 3:
            m.producer_name = r.raw().decode()
        elif f == 4:
            m.doc_string = r.raw().decode()
        else:
            r.skip(w)
    return m


def load(path):
    with open(path, "rb") as f:
        return decode(f.read())


# ---------------------------------------------------------- graph building
class Scope:
    """In-memory graph builder with the call shapes of the reference's Scope and
    nn_ops helpers (ogl_runtime/opengl/core/scope.cc:5-33, nn/apis/nn_ops.cc:6-197):
    each Add* returns the id of the tensor it produces, and tensor name == node name."""

    def __init__(self):
        self.model = Model("ONNX", "0.1", "ignored")

    def add_tensor(self, name):
        self.model.tensor_names.append(name)
        return len(self.model.tensor_names) - 1

    def _node(self, name, type_, inputs, attr=None):
        tid = self.add_tensor(name)
        self.model.nodes.append(Node(name, type_, inputs, [tid], attr))
        return tid

    def add_input(self, name, dims):
        """ONNX graph input: dims are NCHW (onnx_converter.cc:43-62)."""
        self.model.input_names.append(name)
        return self._node(name, "Input", [], {"input_attr": {"dims": list(dims)}})

    def add_const(self, name, array, data_format=ANY, target_data_format=ANY4):
        a = np.asarray(array, dtype=np.float32)
        t = Tensor(a.shape, a, data_format, target_data_format)
        return self._node(name, "Const", [], {"const_attr": {"value": t}})

    def add_conv(self, name, x, w, b=None, kernel=1, stride=1, pad=0, dilation=1, group=1, activation="", min_=0.0,
                 max_=0.0):
        attr = {"kernel_shape": [kernel] * 2, "strides": [stride] * 2, "pads": [pad] * 4, "dilations": [dilation] * 2,
                "group": group}
        if activation:
            attr.update(activation_type=activation, min=min_, max=max_)
        ins = [x, w] + ([b] if b is not None else [])
        return self._node(name, "Conv", ins, {"conv2d_attr": attr})

    def add_node(self, name, type_, inputs, attr=None):
        return self._node(name, type_, list(inputs), attr)

    def add_output_name(self, name):
        self.model.output_names.append(name)
