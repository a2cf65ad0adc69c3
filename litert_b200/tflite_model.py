"""Dependency-free reader (and a small writer) for `.tflite` flatbuffers, limited to what the hot path
needs: tensors with their quantization (per-tensor, per-channel, blockwise), constant buffers, and the
operators with the options of FULLY_CONNECTED, BATCH_MATMUL and STABLEHLO_COMPOSITE.

Field numbers follow tflite/converter/schema/schema.fbs (tables Model :1697, SubGraph :1609, Tensor :249,
QuantizationParameters :114, BlockwiseQuantization :84, Buffer :1634, OperatorCode :1522, Operator :1559,
FullyConnectedOptions :962, BatchMatMulOptions :1412, StableHLOCompositeOptions :1544); the runtime's own
reader is InterpreterBuilder (tflite/core/interpreter_builder.cc:334 ParseNodes, :407 ParseQuantization,
:711 ParseTensors). The binary layout is the flatbuffers wire format: a root offset, tables that point
back to a vtable of 16-bit field offsets, vectors and strings with a 32-bit length prefix.
"""
import struct
from dataclasses import dataclass, field
from typing import List, Optional

import numpy as np

# TensorType (schema.fbs:41) -> numpy dtype and bytes per element (None: packed sub-byte)
TENSOR_TYPES = {0: ("FLOAT32", np.float32), 1: ("FLOAT16", np.float16), 2: ("INT32", np.int32), 3: ("UINT8", np.uint8),
                4: ("INT64", np.int64), 6: ("BOOL", np.bool_), 7: ("INT16", np.int16), 9: ("INT8", np.int8),
                10: ("FLOAT64", np.float64), 17: ("INT4", None), 18: ("BFLOAT16", None), 19: ("INT2", None)}
BUILTIN_FULLY_CONNECTED, BUILTIN_CUSTOM, BUILTIN_BATCH_MATMUL, BUILTIN_STABLEHLO_COMPOSITE = 9, 32, 126, 206
OPTIONS_FULLY_CONNECTED, OPTIONS_BATCH_MATMUL, OPTIONS2_STABLEHLO_COMPOSITE = 8, 101, 21
PLACEHOLDER_FOR_GREATER_OP_CODES = 127


class ModelError(ValueError):
    pass


@dataclass
class Quantization:
    scale: np.ndarray                 # float32 [0], [1] or [channels]
    zero_point: np.ndarray            # int64, same length (may be empty)
    quantized_dimension: int = 0
    blockwise_scales: int = -1        # tensor index of the per-block scales, -1 if not blockwise
    blockwise_zero_points: int = -1
    block_size: int = 0


@dataclass
class Tensor:
    name: str
    shape: List[int]
    type: int
    buffer: int
    quantization: Optional[Quantization]
    is_variable: bool = False
    data: Optional[bytes] = None      # constant contents (None for activations)

    @property
    def type_name(self):
        return TENSOR_TYPES.get(self.type, (f"TYPE_{self.type}", None))[0]

    def array(self):
        """Constant contents as a numpy array of the tensor's shape (packed sub-byte types: raw bytes)."""
        if self.data is None:
            return None
        dt = TENSOR_TYPES.get(self.type, (None, None))[1]
        if dt is None:
            return np.frombuffer(self.data, np.uint8)
        return np.frombuffer(self.data, dt).reshape(self.shape)


@dataclass
class Operator:
    builtin_code: int
    custom_code: str
    version: int
    inputs: List[int]
    outputs: List[int]
    options: dict = field(default_factory=dict)
    custom_options: bytes = b""


@dataclass
class SubGraph:
    name: str
    tensors: List[Tensor]
    inputs: List[int]
    outputs: List[int]
    operators: List[Operator]


@dataclass
class Model:
    version: int
    description: str
    subgraphs: List[SubGraph]


class _Table:
    """One flatbuffers table: position + vtable."""

    def __init__(self, buf, pos):
        if pos < 0 or pos + 4 > len(buf):
            raise ModelError("table offset outside the file")
        self.buf, self.pos = buf, pos
        self.vt = pos - struct.unpack_from("<i", buf, pos)[0]
        if self.vt < 0 or self.vt + 4 > len(buf):
            raise ModelError("vtable offset outside the file")
        self.vt_size = struct.unpack_from("<H", buf, self.vt)[0]

    def _off(self, field_id):
        slot = 4 + 2 * field_id
        if slot + 2 > self.vt_size:
            return 0
        return struct.unpack_from("<H", self.buf, self.vt + slot)[0]

    def scalar(self, field_id, fmt, default=0):
        off = self._off(field_id)
        return struct.unpack_from("<" + fmt, self.buf, self.pos + off)[0] if off else default

    def _indirect(self, field_id):
        off = self._off(field_id)
        if not off:
            return None
        at = self.pos + off
        target = at + struct.unpack_from("<I", self.buf, at)[0]
        if target + 4 > len(self.buf):
            raise ModelError("offset outside the file")
        return target

    def table(self, field_id):
        t = self._indirect(field_id)
        return None if t is None else _Table(self.buf, t)

    def string(self, field_id, default=""):
        t = self._indirect(field_id)
        if t is None:
            return default
        n = struct.unpack_from("<I", self.buf, t)[0]
        return bytes(self.buf[t + 4:t + 4 + n]).decode("utf-8", "replace")

    def vector(self, field_id, dtype):
        """Vector of scalars as a numpy array (a view of the file)."""
        t = self._indirect(field_id)
        if t is None:
            return np.zeros(0, dtype)
        n = struct.unpack_from("<I", self.buf, t)[0]
        if t + 4 + n * np.dtype(dtype).itemsize > len(self.buf):
            raise ModelError("vector runs past the end of the file")
        return np.frombuffer(self.buf, dtype, n, t + 4)

    def tables(self, field_id):
        t = self._indirect(field_id)
        if t is None:
            return []
        n = struct.unpack_from("<I", self.buf, t)[0]
        out = []
        for i in range(n):
            at = t + 4 + 4 * i
            out.append(_Table(self.buf, at + struct.unpack_from("<I", self.buf, at)[0]))
        return out


def _quantization(q):
    if q is None:
        return None
    out = Quantization(scale=np.array(q.vector(2, np.float32)), zero_point=np.array(q.vector(3, np.int64)),
                       quantized_dimension=q.scalar(6, "i"))
    if q.scalar(4, "B") == 2:  # QuantizationDetails.BlockwiseQuantization
        bw = q.table(5)
        if bw is not None:
            out.blockwise_scales = bw.scalar(0, "i")
            out.blockwise_zero_points = bw.scalar(1, "i")
            out.block_size = bw.scalar(2, "i")
    if out.scale.size == 0 and out.blockwise_scales < 0:
        return None
    return out


def _options(op):
    opts = {}
    kind = op.scalar(3, "B")
    t = op.table(4)
    if kind == OPTIONS_FULLY_CONNECTED and t is not None:
        opts = dict(fused_activation_function=t.scalar(0, "b"), weights_format=t.scalar(1, "b"),
                    keep_num_dims=bool(t.scalar(2, "B")), asymmetric_quantize_inputs=bool(t.scalar(3, "B")),
                    quantized_bias_type=t.scalar(4, "b"))
    elif kind == OPTIONS_BATCH_MATMUL and t is not None:
        opts = dict(adj_x=bool(t.scalar(0, "B")), adj_y=bool(t.scalar(1, "B")),
                    asymmetric_quantize_inputs=bool(t.scalar(2, "B")))
    if op.scalar(11, "B") == OPTIONS2_STABLEHLO_COMPOSITE:
        t2 = op.table(12)
        if t2 is not None:
            opts = dict(name=t2.string(0), decomposition_subgraph_index=t2.scalar(1, "i"),
                        composite_attributes=bytes(t2.vector(2, np.uint8)), version=t2.scalar(4, "i"))
    return opts


def read_model(data) -> Model:
    """Parses a `.tflite` file (bytes or a path)."""
    if isinstance(data, str):
        with open(data, "rb") as f:
            data = f.read()
    buf = memoryview(bytes(data))
    if len(buf) < 8:
        raise ModelError("file too short")
    if bytes(buf[4:8]) not in (b"TFL3",):
        raise ModelError("not a TFLite flatbuffer (file identifier is not TFL3)")
    root = _Table(buf, struct.unpack_from("<I", buf, 0)[0])
    codes = []
    for c in root.tables(1):
        builtin = c.scalar(3, "i")
        legacy = c.scalar(0, "b")
        # the wide field wins unless it is unset (old files carry only the byte)
        code = builtin if builtin >= PLACEHOLDER_FOR_GREATER_OP_CODES or legacy == 0 else legacy
        if builtin == 0 and legacy != 0:
            code = legacy
        codes.append((code, c.string(1), c.scalar(2, "i", 1)))
    buffers = []
    for b in root.tables(4):
        data_vec = b.vector(0, np.uint8)
        offset, size = b.scalar(1, "Q"), b.scalar(2, "Q")
        if data_vec.size == 0 and offset > 1 and size > 0:   # stored outside the flatbuffer proper
            if offset + size > len(buf):
                raise ModelError("external buffer range outside the file")
            buffers.append(bytes(buf[offset:offset + size]))
        else:
            buffers.append(bytes(data_vec))
    subgraphs = []
    for sg in root.tables(2):
        tensors = []
        for t in sg.tables(0):
            bidx = t.scalar(2, "I")
            if bidx >= len(buffers) and len(buffers):
                raise ModelError("tensor refers to a buffer that does not exist")
            content = buffers[bidx] if 0 < bidx < len(buffers) and len(buffers[bidx]) else None
            tensors.append(Tensor(name=t.string(3), shape=[int(v) for v in t.vector(0, np.int32)], type=t.scalar(1, "b"),
                                  buffer=bidx, quantization=_quantization(t.table(4)),
                                  is_variable=bool(t.scalar(5, "B")), data=content))
        ops = []
        for op in sg.tables(3):
            idx = op.scalar(0, "I")
            if idx >= len(codes):
                raise ModelError("operator refers to an operator code that does not exist")
            code, custom, version = codes[idx]
            ops.append(Operator(builtin_code=code, custom_code=custom, version=version,
                                inputs=[int(v) for v in op.vector(1, np.int32)],
                                outputs=[int(v) for v in op.vector(2, np.int32)], options=_options(op),
                                custom_options=bytes(op.vector(5, np.uint8))))
        subgraphs.append(SubGraph(name=sg.string(4), tensors=tensors, inputs=[int(v) for v in sg.vector(1, np.int32)],
                                  outputs=[int(v) for v in sg.vector(2, np.int32)], operators=ops))
    return Model(version=root.scalar(0, "I"), description=root.string(3), subgraphs=subgraphs)


# ---- writer ---------------------------------------------------------------------------------------
class _Builder:
    """Back-to-front flatbuffer builder, just enough for write_model."""

    def __init__(self):
        self.buf = bytearray()   # grows at the front: buf holds the END of the file

    def _pad(self, align, extra=0):
        while (len(self.buf) + extra) % align:
            self.buf[0:0] = b"\0"

    def _push(self, raw):
        self.buf[0:0] = raw
        return len(self.buf)   # "offset" = distance from the end of the file

    def vector(self, raw, count, elem_align=4):
        self._pad(max(4, elem_align), len(raw))
        self._push(raw)
        return self._push(struct.pack("<I", count))

    def scalars(self, values, fmt, align=None):
        size = struct.calcsize(fmt)
        return self.vector(b"".join(struct.pack("<" + fmt, v) for v in values), len(values), align or size)

    def string(self, text):
        raw = text.encode("utf-8") + b"\0"
        self._pad(4, len(raw))
        self._push(raw)
        return self._push(struct.pack("<I", len(raw) - 1))

    def offsets(self, offs):
        """Vector of tables/strings: elements are offsets relative to their own position."""
        self._pad(4)
        for i, o in enumerate(reversed(offs)):
            here = len(self.buf) + 4
            self._push(struct.pack("<I", here - o))
        return self._push(struct.pack("<I", len(offs)))

    def table(self, fields):
        """fields: list of (field_id, kind, value) with kind in 'b','B','i','I','Q' (scalars) or 'o' (offset)."""
        if not fields:
            fields = []
        nfields = max([f[0] for f in fields], default=-1) + 1
        # lay the table out: soffset, then fields by decreasing size
        order = sorted(fields, key=lambda f: -(4 if f[1] == "o" else struct.calcsize(f[1])))
        body, slots, pos = bytearray(4), {}, 4
        for fid, kind, value in order:
            size = 4 if kind == "o" else struct.calcsize(kind)
            while pos % size:
                body += b"\0"
                pos += 1
            slots[fid] = (pos, kind, value)
            body += b"\0" * size
            pos += size
        while len(body) % 4:
            body += b"\0"
        self._pad(8 if any(k == "Q" for _, k, _ in fields) else 4, len(body))
        start_from_end = len(self.buf) + len(body)   # position of the table start, from the end
        for fid, (p, kind, value) in slots.items():
            if kind == "o":
                field_from_end = start_from_end - p
                struct.pack_into("<I", body, p, field_from_end - value)
            else:
                struct.pack_into("<" + kind, body, p, value)
        self._push(bytes(body))
        table = len(self.buf)
        vt = struct.pack("<HH", 4 + 2 * nfields, len(body))
        vt += b"".join(struct.pack("<H", slots[i][0] if i in slots else 0) for i in range(nfields))
        if len(vt) % 4:
            vt += b"\0\0"
        self._push(vt)
        vtable = len(self.buf)
        # soffset = table position - vtable position (vtable sits in front of the table)
        struct.pack_into("<i", self.buf, len(self.buf) - table, vtable - table)
        return table

    def finish(self, root, identifier=b"TFL3"):
        self._pad(16, 8)
        self._push(identifier)
        self._push(struct.pack("<I", len(self.buf) + 4 - root))
        return bytes(self.buf)


def write_model(model: Model) -> bytes:
    """Serialises a Model (one or more subgraphs) to `.tflite` bytes: the inverse of read_model for the
    fields it knows. Constant tensors get a buffer each; buffer 0 is the empty sentinel."""
    b = _Builder()
    codes, code_index = [], {}
    buffers = [b""]
    sub_offs = []
    for sg in model.subgraphs:
        op_offs = []
        for op in sg.operators:
            key = (op.builtin_code, op.custom_code, op.version)
            if key not in code_index:
                code_index[key] = len(codes)
                codes.append(key)
            f = [(0, "I", code_index[key]), (1, "o", b.scalars(op.inputs, "i")), (2, "o", b.scalars(op.outputs, "i"))]
            o = op.options
            if op.builtin_code == BUILTIN_FULLY_CONNECTED:
                t = b.table([(0, "b", o.get("fused_activation_function", 0)), (1, "b", o.get("weights_format", 0)),
                             (2, "B", int(o.get("keep_num_dims", False))),
                             (3, "B", int(o.get("asymmetric_quantize_inputs", False)))])
                f += [(3, "B", OPTIONS_FULLY_CONNECTED), (4, "o", t)]
            elif op.builtin_code == BUILTIN_BATCH_MATMUL:
                t = b.table([(0, "B", int(o.get("adj_x", False))), (1, "B", int(o.get("adj_y", False))),
                             (2, "B", int(o.get("asymmetric_quantize_inputs", False)))])
                f += [(3, "B", OPTIONS_BATCH_MATMUL), (4, "o", t)]
            elif op.builtin_code == BUILTIN_STABLEHLO_COMPOSITE:
                attrs = o.get("composite_attributes", b"")
                t = b.table([(0, "o", b.string(o.get("name", ""))), (1, "i", o.get("decomposition_subgraph_index", 0)),
                             (2, "o", b.vector(bytes(attrs), len(attrs), 1)), (4, "i", o.get("version", 0))])
                f += [(11, "B", OPTIONS2_STABLEHLO_COMPOSITE), (12, "o", t)]
            if op.custom_options:
                f.append((5, "o", b.vector(bytes(op.custom_options), len(op.custom_options), 1)))
            op_offs.append(b.table(f))
        t_offs = []
        for t in sg.tensors:
            f = [(0, "o", b.scalars(t.shape, "i")), (1, "b", t.type), (3, "o", b.string(t.name))]
            if t.data is not None:
                buffers.append(bytes(t.data))
                f.append((2, "I", len(buffers) - 1))
            q = t.quantization
            if q is not None:
                qf = [(2, "o", b.scalars([float(v) for v in q.scale], "f")),
                      (3, "o", b.scalars([int(v) for v in q.zero_point], "q")), (6, "i", q.quantized_dimension)]
                if q.blockwise_scales >= 0:
                    bw = b.table([(0, "i", q.blockwise_scales), (1, "i", q.blockwise_zero_points), (2, "i", q.block_size)])
                    qf += [(4, "B", 2), (5, "o", bw)]
                f.append((4, "o", b.table(qf)))
            if t.is_variable:
                f.append((5, "B", 1))
            t_offs.append(b.table(f))
        sub_offs.append(b.table([(0, "o", b.offsets(t_offs)), (1, "o", b.scalars(sg.inputs, "i")),
                                 (2, "o", b.scalars(sg.outputs, "i")), (3, "o", b.offsets(op_offs)),
                                 (4, "o", b.string(sg.name))]))
    buf_offs = []
    for raw in buffers:
        buf_offs.append(b.table([(0, "o", b.vector(raw, len(raw), 16))] if raw else []))
    code_offs = []
    for code, custom, version in codes:
        f = [(0, "b", min(code, PLACEHOLDER_FOR_GREATER_OP_CODES)), (2, "i", version), (3, "i", code)]
        if custom:
            f.append((1, "o", b.string(custom)))
        code_offs.append(b.table(f))
    root = b.table([(0, "I", model.version), (1, "o", b.offsets(code_offs)), (2, "o", b.offsets(sub_offs)),
                    (3, "o", b.string(model.description)), (4, "o", b.offsets(buf_offs))])
    return b.finish(root)
