"""Python handle on the mini runtime (tests/minirt/minirt.cc) and on the delegate plugin.

TEST INFRASTRUCTURE ONLY. The mini runtime is compiled against the LiteRT C headers where they
lie (environment variable LITERT_ROOT); a prebuilt libminirt.so is used when they are absent.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
LITERT_ROOT = os.environ.get("LITERT_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
LIB = os.path.join(HERE, "libminirt.so")

# TfLiteType values (tflite/core/c/c_api_types.h)
F32, I32, U8, I64, I16, I8, F16, I4 = 1, 2, 3, 4, 7, 9, 10, 18
_NP = {F32: np.float32, I32: np.int32, U8: np.uint8, I8: np.int8, F16: np.float16, I4: np.uint8, I64: np.int64,
       I16: np.int16, 6: np.bool_, 11: np.float64}
# builtin operator codes (tflite/builtin_ops.h)
OP_ADD, OP_FULLY_CONNECTED, OP_SOFTMAX = 0, 9, 25


def build():
    from litert_b200 import build_delegate

    src = os.path.join(HERE, "minirt.cc")
    have = os.path.exists(os.path.join(LITERT_ROOT, "tflite", "core", "c", "common.h"))
    if not have:
        if os.path.exists(LIB):
            return LIB
        raise RuntimeError("libminirt.so is missing and the LiteRT headers are not available to build it")
    if os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(src):
        return LIB
    subprocess.check_call(["g++", "-O1", "-std=c++17", "-fPIC", "-fvisibility=hidden", "-shared", "-o", LIB, src,
                           os.path.join(LITERT_ROOT, "tflite", "core", "c", "common.cc"),
                           os.path.join(LITERT_ROOT, "tflite", "array.cc"), "-I" + LITERT_ROOT,
                           "-I" + build_delegate.generated_include_dir(), "-ldl"])
    return LIB


_CB = ctypes.CFUNCTYPE(ctypes.c_int, ctypes.c_int)
_ERR = ctypes.CFUNCTYPE(None, ctypes.c_char_p)


class Delegate:
    """Loads the plugin the way tflite/delegates/external/external_delegate.cc:39-64 does."""

    def __init__(self, options=None, path=None):
        from litert_b200 import build_delegate

        path = path or build_delegate.build()
        self.lib = ctypes.CDLL(path)
        self.lib.tflite_plugin_create_delegate.restype = ctypes.c_void_p
        self.lib.tflite_plugin_create_delegate.argtypes = [ctypes.POINTER(ctypes.c_char_p),
                                                           ctypes.POINTER(ctypes.c_char_p), ctypes.c_size_t, _ERR]
        self.lib.tflite_plugin_destroy_delegate.argtypes = [ctypes.c_void_p]
        self.lib.b200_delegate_num_claimed_nodes.argtypes = [ctypes.c_void_p]
        self.errors = []
        self._err = _ERR(lambda m: self.errors.append(m.decode()))
        options = options or {}
        n = len(options)
        keys = (ctypes.c_char_p * max(n, 1))(*[k.encode() for k in options])
        vals = (ctypes.c_char_p * max(n, 1))(*[str(v).encode() for v in options.values()])
        self.ptr = self.lib.tflite_plugin_create_delegate(keys, vals, n, self._err)

    @property
    def claimed(self):
        return self.lib.b200_delegate_num_claimed_nodes(self.ptr)

    def close(self):
        if self.ptr:
            self.lib.tflite_plugin_destroy_delegate(self.ptr)
            self.ptr = None


class Accelerator:
    """The LiteRT accelerator library loaded the way the LiteRT environment loads it; `.ptr` is the
    TfLiteDelegate it created (usable with MiniRuntime.apply)."""

    def __init__(self, path=None):
        from litert_b200 import build_delegate

        path = path or build_delegate.build_accelerator()
        self.lib = ctypes.CDLL(build())
        name = ctypes.create_string_buffer(64)
        version = (ctypes.c_int * 3)()
        hw, size = ctypes.c_int(), ctypes.c_int()
        wrapped, delegate = ctypes.c_void_p(), ctypes.c_void_p()
        self.lib.mrt_accelerator_probe.argtypes = [ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int,
                                                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int),
                                                   ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_void_p),
                                                   ctypes.POINTER(ctypes.c_void_p)]
        self.lib.mrt_accelerator_release.argtypes = [ctypes.c_void_p]
        self.rc = self.lib.mrt_accelerator_probe(path.encode(), name, 64, version, ctypes.byref(hw), ctypes.byref(size),
                                                 ctypes.byref(wrapped), ctypes.byref(delegate))
        self.name, self.version, self.hardware, self.struct_size = name.value.decode(), tuple(version), hw.value, size.value
        self._wrapped = wrapped
        self.ptr = delegate.value

    def close(self):
        if self._wrapped:
            self.lib.mrt_accelerator_release(self._wrapped)
            self._wrapped = None


class MiniRuntime:
    def __init__(self):
        # global symbols: the delegate looks the runtime's MarkSubgraphAsDelegationSkippable up with dlsym
        self.lib = ctypes.CDLL(build(), mode=ctypes.RTLD_GLOBAL)
        L = self.lib
        L.mrt_create.restype = ctypes.c_void_p
        L.mrt_last_error.restype = ctypes.c_char_p
        L.mrt_tensor_data.restype = ctypes.c_void_p
        L.mrt_tensor_bytes.restype = ctypes.c_size_t
        for name in ("mrt_destroy", "mrt_last_error", "mrt_clear_error", "mrt_num_partitions", "mrt_plan_size",
                     "mrt_num_skippable_subgraphs",
                     "mrt_num_cpu_nodes_in_plan", "mrt_invoke"):
            getattr(L, name).argtypes = [ctypes.c_void_p]
        L.mrt_apply_delegate.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        L.mrt_tensor_data.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.mrt_tensor_bytes.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.mrt_tensor_is_stale.argtypes = [ctypes.c_void_p, ctypes.c_int]
        L.mrt_set_cpu_callback.argtypes = [ctypes.c_void_p, _CB]
        L.mrt_add_tensor.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                     ctypes.c_int, ctypes.c_void_p, ctypes.c_float, ctypes.c_int, ctypes.c_int,
                                     ctypes.c_void_p, ctypes.c_int]
        L.mrt_set_blockwise.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int]
        L.mrt_add_fully_connected.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 8
        L.mrt_add_batch_matmul.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 6
        L.mrt_add_composite.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_char_p, ctypes.c_int, ctypes.c_int,
                                        ctypes.POINTER(ctypes.c_int), ctypes.c_int]
        L.mrt_add_custom.argtypes = L.mrt_add_composite.argtypes
        L.mrt_add_other.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                    ctypes.c_int]
        L.mrt_add_node.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int),
                                   ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_void_p, ctypes.c_int, ctypes.c_char_p,
                                   ctypes.c_int]
        L.mrt_set_io.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_int), ctypes.c_int,
                                 ctypes.POINTER(ctypes.c_int)]
        self.h = L.mrt_create()
        self.meta = []  # (type, shape)
        self._cb = None

    # ---- graph construction
    def tensor(self, ttype, shape, data=None, scale=0.0, zero_point=0, channel_scales=None, quantized_dimension=0):
        dims = (ctypes.c_int * max(len(shape), 1))(*shape)
        buf = None
        if data is not None:
            buf = np.ascontiguousarray(data)
            ptr = buf.ctypes.data_as(ctypes.c_void_p)
        else:
            ptr = None
        cs = None if channel_scales is None else np.ascontiguousarray(channel_scales, np.float32)
        idx = self.lib.mrt_add_tensor(self.h, ttype, len(shape), dims, 1 if data is not None else 0, ptr,
                                      float(scale), int(zero_point), 0 if cs is None else cs.size,
                                      None if cs is None else cs.ctypes.data_as(ctypes.c_void_p), quantized_dimension)
        self.meta.append((ttype, tuple(shape)))
        return idx

    def set_blockwise(self, tensor, scale_tensor, blocksize):
        self.lib.mrt_set_blockwise(self.h, tensor, scale_tensor, blocksize)

    def fully_connected(self, x, w, bias, y, activation=0, keep_num_dims=False, asymmetric=True, weights_format=0):
        return self.lib.mrt_add_fully_connected(self.h, x, w, -1 if bias is None else bias, y, activation,
                                                int(keep_num_dims), int(asymmetric), weights_format)

    def batch_matmul(self, x, y, out, adj_x=False, adj_y=False, asymmetric=True):
        return self.lib.mrt_add_batch_matmul(self.h, x, y, out, int(adj_x), int(adj_y), int(asymmetric))

    def _ints(self, v):
        return (ctypes.c_int * max(len(v), 1))(*v)

    def composite(self, name, attributes, ins, out):
        return self.lib.mrt_add_composite(self.h, name.encode(), attributes, len(attributes), len(ins),
                                          self._ints(ins), out)

    def custom(self, name, init_data, ins, out):
        return self.lib.mrt_add_custom(self.h, name.encode(), init_data, len(init_data), len(ins), self._ints(ins), out)

    def node(self, builtin_code, ins, outs, params=b"", custom_name="", init_data=b""):
        """Any builtin or custom node; `params` is the op's builtin-data struct as bytes (see the helpers below)."""
        buf = ctypes.create_string_buffer(params, len(params)) if params else None
        return self.lib.mrt_add_node(self.h, builtin_code, custom_name.encode(), len(ins), self._ints(ins), len(outs),
                                     self._ints(outs), ctypes.cast(buf, ctypes.c_void_p) if buf else None, len(params),
                                     init_data if init_data else None, len(init_data))

    # ---- the builtins a decoder-only graph is made of (builtin codes: tflite/builtin_ops.h; parameter structs:
    # tflite/core/c/builtin_op_data.h, all plain ints / bools / floats)
    def add(self, a, b, out):
        import struct
        return self.node(0, [a, b], [out], struct.pack("<i?xxx", 0, False))          # TfLiteAddParams

    def mul(self, a, b, out):
        import struct
        return self.node(18, [a, b], [out], struct.pack("<i", 0))                    # TfLiteMulParams

    def gelu(self, x, out, approximate=True):
        import struct
        return self.node(150, [x], [out], struct.pack("<?", approximate))            # TfLiteGeluParams

    def reshape(self, x, out):
        import struct
        shape = self.meta[out][1]
        return self.node(22, [x], [out], struct.pack("<8ii", *(list(shape) + [0] * (8 - len(shape))), len(shape)))  # TfLiteReshapeParams

    def slice(self, x, begin, size, out):
        """begin / size: constant int32 tensors are created here."""
        b = self.tensor(I32, (len(begin),), np.asarray(begin, np.int32))
        s = self.tensor(I32, (len(size),), np.asarray(size, np.int32))
        return self.node(65, [x, b, s], [out])

    def concatenation(self, ins, out, axis):
        import struct
        return self.node(2, list(ins), [out], struct.pack("<ii", axis, 0))           # TfLiteConcatenationParams

    def embedding_lookup(self, ids, table, out):
        return self.node(7, [ids, table], [out])

    def arg_max(self, x, out, axis=-1):
        import struct
        a = self.tensor(I32, (1,), np.asarray([axis], np.int32))
        out_type = self.meta[out][0]
        return self.node(56, [x, a], [out], struct.pack("<i", out_type))             # TfLiteArgMaxParams

    def other(self, builtin_code, ins, out):
        return self.lib.mrt_add_other(self.h, builtin_code, len(ins), self._ints(ins), out)

    def set_io(self, ins, outs):
        self.lib.mrt_set_io(self.h, len(ins), self._ints(ins), len(outs), self._ints(outs))

    # ---- execution
    def apply(self, delegate):
        return self.lib.mrt_apply_delegate(self.h, delegate.ptr)

    def set_cpu(self, fn):
        self._cb = _CB(fn)
        self.lib.mrt_set_cpu_callback(self.h, self._cb)

    def invoke(self):
        return self.lib.mrt_invoke(self.h)

    def view(self, tensor):
        ttype, shape = self.meta[tensor]
        nbytes = self.lib.mrt_tensor_bytes(self.h, tensor)
        raw = (ctypes.c_uint8 * nbytes).from_address(self.lib.mrt_tensor_data(self.h, tensor))
        arr = np.frombuffer(raw, dtype=_NP[ttype])
        return arr if ttype == I4 else arr.reshape(shape)

    def write(self, tensor, data):
        self.view(tensor)[...] = np.asarray(data).reshape(self.meta[tensor][1])

    @property
    def error(self):
        return self.lib.mrt_last_error(self.h).decode()

    @property
    def partitions(self):
        return self.lib.mrt_num_partitions(self.h)

    @property
    def cpu_nodes(self):
        return self.lib.mrt_num_cpu_nodes_in_plan(self.h)

    @property
    def skippable_subgraphs(self):
        return self.lib.mrt_num_skippable_subgraphs(self.h)

    @property
    def plan_size(self):
        return self.lib.mrt_plan_size(self.h)

    def close(self):
        if self.h:
            self.lib.mrt_destroy(self.h)
            self.h = None


def flex_map(values):
    """Encodes {key: float or int} as a FlexBuffers map with 4-byte inline scalars -- the form the SDPA
    composite's attribute blob ({"scale": float}) and the kv-cache op's initial data ({"kv_cache_max": int,
    ...}) take. Layout, back to front: root (offset to the map, type, width);
    map = [keys vector offset][keys width][size][values...][value types]; keys vector of offsets to
    NUL-terminated strings, sorted by key."""
    import struct

    keys = sorted(values)
    buf = bytearray()
    key_pos = []
    for k in keys:
        key_pos.append(len(buf))
        buf += k.encode() + b"\0"
    while len(buf) % 4:
        buf += b"\0"
    # keys vector (width 4): size, then offsets
    buf += struct.pack("<I", len(keys))
    keys_vec = len(buf)
    for i, kp in enumerate(key_pos):
        here = keys_vec + 4 * i
        buf += struct.pack("<I", here - kp)
    # map prefix: offset to keys vector, keys byte width, size
    here = len(buf)
    buf += struct.pack("<I", here - keys_vec)
    buf += struct.pack("<I", 4)
    buf += struct.pack("<I", len(keys))
    map_pos = len(buf)
    for k in keys:
        buf += struct.pack("<i", values[k]) if isinstance(values[k], (int, np.integer)) else struct.pack("<f", values[k])
    for k in keys:
        buf += bytes([((1 if isinstance(values[k], (int, np.integer)) else 3) << 2) | 2])  # INT or FLOAT, 4 bytes
    while len(buf) % 4:
        buf += b"\0"
    root = len(buf)
    buf += struct.pack("<I", root - map_pos)
    buf += bytes([(9 << 2) | 2, 4])  # MAP with 4-byte elements; root width 4
    return bytes(buf)


# schema TensorType -> TfLiteType (ConvertTensorType, tflite/core/api/flatbuffer_conversions.cc)
_SCHEMA_TO_TFLITE = {0: 1, 1: 10, 2: 2, 3: 3, 4: 4, 5: 5, 6: 6, 7: 7, 8: 8, 9: 9, 10: 11, 11: 12, 12: 13, 13: 14, 14: 15,
                     15: 16, 16: 17, 17: 18, 18: 19, 19: 20}


def load_model(model, subgraph=0):
    """Builds a MiniRuntime graph from a parsed `.tflite` model (litert_b200.tflite_model.Model): what
    InterpreterBuilder does for the tensors, quantization and nodes of one subgraph
    (tflite/core/interpreter_builder.cc:334-518, 711-900), for the node kinds the delegate can claim;
    every other builtin becomes a node for the test's CPU callback."""
    from litert_b200 import tflite_model as tm

    sg = model.subgraphs[subgraph]
    rt = MiniRuntime()
    for t in sg.tensors:
        ttype = _SCHEMA_TO_TFLITE[t.type]
        if ttype not in _NP:
            raise ValueError(f"tensor type {t.type_name} is not handled by the mini runtime")
        data = None
        if t.data is not None:
            data = np.frombuffer(t.data, np.uint8) if ttype == I4 else np.frombuffer(t.data, _NP[ttype])
        q = t.quantization
        scale, zp, cs, qdim = 0.0, 0, None, 0
        if q is not None and q.scale.size == 1:
            scale, zp = float(q.scale[0]), int(q.zero_point[0]) if q.zero_point.size else 0
        elif q is not None and q.scale.size > 1:
            cs, qdim = q.scale, q.quantized_dimension
        shape = list(t.shape) if t.shape else [1]
        rt.tensor(ttype, shape, data, scale, zp, cs, qdim)
    for i, t in enumerate(sg.tensors):
        q = t.quantization
        if q is not None and q.blockwise_scales >= 0:
            rt.set_blockwise(i, q.blockwise_scales, q.block_size)
    for op in sg.operators:
        o = op.options
        if op.builtin_code == tm.BUILTIN_FULLY_CONNECTED:
            bias = op.inputs[2] if len(op.inputs) > 2 and op.inputs[2] >= 0 else None
            rt.fully_connected(op.inputs[0], op.inputs[1], bias, op.outputs[0], o.get("fused_activation_function", 0),
                               o.get("keep_num_dims", False), o.get("asymmetric_quantize_inputs", False),
                               o.get("weights_format", 0))
        elif op.builtin_code == tm.BUILTIN_BATCH_MATMUL:
            rt.batch_matmul(op.inputs[0], op.inputs[1], op.outputs[0], o.get("adj_x", False), o.get("adj_y", False),
                            o.get("asymmetric_quantize_inputs", False))
        elif op.builtin_code == tm.BUILTIN_STABLEHLO_COMPOSITE:
            rt.composite(o.get("name", ""), o.get("composite_attributes", b""), op.inputs, op.outputs[0])
        elif op.builtin_code == tm.BUILTIN_CUSTOM:
            rt.custom(op.custom_code, op.custom_options, op.inputs, op.outputs[0])
        else:
            rt.other(op.builtin_code, [i for i in op.inputs if i >= 0], op.outputs[0])
    rt.set_io(sg.inputs, sg.outputs)
    return rt

