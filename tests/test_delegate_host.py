"""Host-side logic of the delegate, exercised without a GPU through the mini runtime: plugin
exports and options, the support predicate (what is claimed, what is left to the CPU kernels),
loud failure plus roll-back when no CUDA device can be initialised, the device-arena planner
against the reference's own arena code, and the FlexBuffers attribute reader."""
import ctypes
import os
import re

import numpy as np
import pytest

from tests import minirt
from tests.minirt import F16, F32, I4, I8, I32

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_plugin_exports_the_external_delegate_symbols(plugin_path):
    lib = ctypes.CDLL(plugin_path)
    text = open(os.path.join(ROOT, "include", "litert_b200_delegate.h")).read()
    names = set(re.findall(r"\b(tflite_plugin_[a-z_]+|b200_[a-z0-9_]+)\s*\(", text))
    assert {"tflite_plugin_create_delegate", "tflite_plugin_destroy_delegate"} <= names
    for n in names:
        assert hasattr(lib, n), n
    lib.tflite_plugin_destroy_delegate(None)  # NULL is allowed


def test_options(plugin_path):
    d = minirt.Delegate({"device": 0, "buffer_handles": 1, "claim_bmm": 0})
    assert d.ptr and not d.errors
    d.close()
    bad = minirt.Delegate({"no_such_option": "x"})
    assert bad.ptr is None and "unknown option" in bad.errors[0]
    inj = minirt.Delegate({"fail_on": "create"})
    assert inj.ptr is None and "injected" in inj.errors[0]


def _fc_graph(m, x_type, w_type, y_type, *, w_const=True, bias_type=None, per_channel=False, activation=0,
              weights_format=0, w_shape=(3, 10), blockwise=False, sparse=False):
    n, k = w_shape
    x = m.tensor(x_type, (2, k), scale=0.5 if x_type == I8 else 0.0, zero_point=-1)
    wdata = np.ones(w_shape, np.int8) if w_type == I8 else np.zeros((n, (k + 1) // 2), np.uint8)
    kw = {}
    if per_channel:
        kw = dict(channel_scales=np.full(n, 0.25, np.float32))
    elif w_type == I8:
        kw = dict(scale=0.25)
    w = m.tensor(w_type, w_shape, wdata if w_const else None, **kw)
    if blockwise:
        s = m.tensor(F16, (n, k // 32), np.ones((n, k // 32), np.float16))
        m.set_blockwise(w, s, 32)
    b = None
    if bias_type is not None:
        b = m.tensor(bias_type, (n,), np.zeros(n, np.int32 if bias_type == I32 else np.float32), scale=0.125)
    y = m.tensor(y_type, (2, n), scale=1.0 if y_type == I8 else 0.0, zero_point=-1)
    m.fully_connected(x, w, b, y, activation=activation, weights_format=weights_format)
    m.set_io([x], [y])


CLAIM_CASES = [
    ("int8 per tensor", dict(x_type=I8, w_type=I8, y_type=I8, bias_type=I32), 1),
    ("int8 per channel", dict(x_type=I8, w_type=I8, y_type=I8, per_channel=True), 1),
    ("hybrid", dict(x_type=F32, w_type=I8, y_type=F32, bias_type=F32, activation=4), 1),
    ("blockwise int4", dict(x_type=F32, w_type=I4, y_type=F32, w_shape=(4, 64), blockwise=True), 1),
    ("int4 without block scales", dict(x_type=F32, w_type=I4, y_type=F32, w_shape=(4, 64)), 0),
    ("non-constant weights", dict(x_type=F32, w_type=I8, y_type=F32, w_const=False), 0),
    ("shuffled weights format", dict(x_type=I8, w_type=I8, y_type=I8, weights_format=1), 0),
    ("int8 with tanh", dict(x_type=I8, w_type=I8, y_type=I8, activation=4), 0),
    ("float weights", dict(x_type=F32, w_type=F32, y_type=F32), 0),
    ("int8 in, float out", dict(x_type=I8, w_type=I8, y_type=F32), 0),
]


@pytest.mark.parametrize("name,kwargs,claimed", CLAIM_CASES, ids=[c[0] for c in CLAIM_CASES])
def test_support_predicate_fully_connected(plugin_path, name, kwargs, claimed):
    m, d = minirt.MiniRuntime(), minirt.Delegate()
    if kwargs.get("w_type") == F32:
        x = m.tensor(F32, (2, 10))
        w = m.tensor(F32, (3, 10), np.ones((3, 10), np.float32))
        y = m.tensor(F32, (2, 3))
        m.fully_connected(x, w, None, y)
        m.set_io([x], [y])
    else:
        _fc_graph(m, **kwargs)
    rc = m.apply(d)
    assert d.claimed == claimed
    if claimed == 0:
        assert rc == 0 and m.partitions == 0 and m.cpu_nodes == 1  # nothing claimed is not an error
    m.close()
    d.close()


def test_support_predicate_bmm_and_sdpa(plugin_path):
    m, d = minirt.MiniRuntime(), minirt.Delegate()
    x = m.tensor(F32, (2, 10))
    w = m.tensor(I8, (10, 3), np.ones((10, 3), np.int8), scale=0.1)
    y0 = m.tensor(F32, (2, 3))
    m.batch_matmul(x, w, y0)                       # claimed: hybrid, constant rhs
    w2 = m.tensor(I8, (3, 10), scale=0.1)          # not constant: repacked at every invocation
    y1 = m.tensor(F32, (2, 10))
    m.batch_matmul(y0, w2, y1)                     # claimed
    q = m.tensor(F32, (1, 1, 8, 64))
    k = m.tensor(F32, (1, 32, 2, 64))
    v = m.tensor(F32, (1, 32, 2, 64))
    mask = m.tensor(F32, (1, 1, 1, 32))
    o = m.tensor(F32, (1, 1, 8, 64))
    m.composite("odml.scaled_dot_product_attention", minirt.flex_map({"scale": 0.125}), [q, k, v, mask], o)  # claimed
    o2 = m.tensor(F32, (1, 1, 8, 64))
    m.composite("odml.rms_norm", b"", [q], o2)     # the norm composite of a decoder graph: claimed
    o2b = m.tensor(F32, (1, 1, 8, 64))
    m.composite("odml.group_norm", b"", [q], o2b)  # some other composite: not claimed
    o3 = m.tensor(F32, (1, 1, 8, 64))
    m.custom("odml.scaled_dot_product_attention", b"", [q, k, v, mask], o3)  # custom-op form: claimed
    q4 = m.tensor(F32, (1, 4, 8, 64))
    mask4 = m.tensor(F32, (1, 1, 4, 32))
    o4 = m.tensor(F32, (1, 4, 8, 64))
    m.custom("odml.scaled_dot_product_attention", b"", [q4, k, v, mask4], o4)  # 4 query tokens: claimed
    q5 = m.tensor(F16, (1, 1, 8, 64))
    o5 = m.tensor(F16, (1, 1, 8, 64))
    m.custom("odml.scaled_dot_product_attention", b"", [q5, k, v, mask], o5)   # mixed float16 / float32: not claimed
    x6 = m.tensor(F32, (2, 5, 10))
    w6 = m.tensor(I8, (3, 10, 3), np.ones((3, 10, 3), np.int8), scale=0.1)
    y6 = m.tensor(F32, (3, 5, 3))
    m.batch_matmul(x6, w6, y6)                     # batch dimensions 2 and 3 do not broadcast: not claimed
    w7 = m.tensor(I8, (10, 3), np.ones((10, 3), np.int8), channel_scales=np.full(10, 0.1, np.float32), quantized_dimension=0)
    y7 = m.tensor(F32, (2, 3))
    m.batch_matmul(x, w7, y7)                      # per-channel scales along k: not claimed
    x8 = m.tensor(F32, (3, 5, 2, 10))
    y8 = m.tensor(F32, (3, 5, 2, 3))
    m.batch_matmul(x8, w, y8)                      # hybrid over two batch dimensions (the reference kernel mixes up
                                                   # the rows' parameters there): not claimed
    m.set_io([x, w2, q, k, v, mask, q4, mask4, q5, x6, x8], [y1, o, o2, o2b, o3, o4, o5, y6, y7, y8])
    m.apply(d)
    assert d.claimed == 6
    assert m.skippable_subgraphs == 2              # the two claimed STABLEHLO_COMPOSITE nodes carry a decomposition each
    m.close()
    d.close()


def test_support_predicate_leaves_constant_activations_and_bad_shapes_alone(plugin_path):
    """A node whose run-time operand is a constant would never see its data on the device (only run-time
    tensors get arena slots), and a bias or output whose size disagrees with the weights would be read
    or written out of bounds: none of these is claimed."""
    def claimed(build):
        m, d = minirt.MiniRuntime(), minirt.Delegate()
        build(m)
        m.apply(d)
        n = d.claimed
        m.close()
        d.close()
        return n

    def fc(m, x_data=None, bias_len=3, y_cols=3):
        x = m.tensor(F32, (2, 10), x_data)
        w = m.tensor(I8, (3, 10), np.ones((3, 10), np.int8), scale=0.25)
        b = m.tensor(F32, (bias_len,), np.zeros(bias_len, np.float32))
        y = m.tensor(F32, (2, y_cols))
        m.fully_connected(x, w, b, y)
        m.set_io([x] if x_data is None else [], [y])

    assert claimed(lambda m: fc(m)) == 1
    assert claimed(lambda m: fc(m, x_data=np.ones((2, 10), np.float32))) == 0   # constant input
    assert claimed(lambda m: fc(m, bias_len=2)) == 0                            # bias shorter than the units
    assert claimed(lambda m: fc(m, y_cols=4)) == 0                              # output of the wrong size

    def bmm_const_lhs(m):
        x = m.tensor(F32, (2, 10), np.ones((2, 10), np.float32))
        w = m.tensor(I8, (10, 3), np.ones((10, 3), np.int8), scale=0.1)
        y = m.tensor(F32, (2, 3))
        m.batch_matmul(x, w, y)
        m.set_io([], [y])

    assert claimed(bmm_const_lhs) == 0

    def sdpa(m, const_k):
        q = m.tensor(F32, (1, 1, 8, 64))
        k = m.tensor(F32, (1, 32, 2, 64), np.zeros((1, 32, 2, 64), np.float32) if const_k else None)
        v = m.tensor(F32, (1, 32, 2, 64))
        o = m.tensor(F32, (1, 1, 8, 64))
        m.custom("odml.scaled_dot_product_attention", b"", [q, k, v], o)
        m.set_io([q, v] if const_k else [q, k, v], [o])

    assert claimed(lambda m: sdpa(m, False)) == 1
    assert claimed(lambda m: sdpa(m, True)) == 0


def test_support_predicate_decoder_glue_ops(plugin_path):
    """The float32 ops between a decoder's projections: claimed in the forms a converter emits, left alone
    otherwise (fused activations, run-time shapes, other axes, constant-only operands)."""
    import struct

    def claimed(build, options=None):
        m, d = minirt.MiniRuntime(), minirt.Delegate(options)
        build(m)
        m.apply(d)
        n = d.claimed
        m.close()
        d.close()
        return n

    def binary(m, act=0, b_shape=(1, 4, 1, 8), const_both=False):
        a = m.tensor(F32, (1, 4, 3, 8), np.ones((1, 4, 3, 8), np.float32) if const_both else None)
        b = m.tensor(F32, b_shape, np.ones(b_shape, np.float32) if const_both else None)
        y = m.tensor(F32, (1, 4, 3, 8))
        m.node(18, [a, b], [y], struct.pack("<i", act))
        m.set_io([] if const_both else [a, b], [y])

    assert claimed(binary) == 1
    assert claimed(binary, {"claim_glue": 0}) == 0
    assert claimed(lambda m: binary(m, act=1)) == 0                       # fused RELU
    assert claimed(lambda m: binary(m, b_shape=(1, 4, 2, 8))) == 0        # does not broadcast
    assert claimed(lambda m: binary(m, const_both=True)) == 0

    def argmax(m, axis):
        x = m.tensor(F32, (3, 50))
        y = m.tensor(I32, (3,) if axis in (-1, 1) else (50,))
        m.arg_max(x, y, axis=axis)
        m.set_io([x], [y])

    assert claimed(lambda m: argmax(m, -1)) == 1
    assert claimed(lambda m: argmax(m, 0)) == 0

    def kv(m, batch=1, dtype_pos=4):
        pos = m.tensor(dtype_pos, (1,))
        k = m.tensor(F32, (batch, 2, 1, 16))
        v = m.tensor(F32, (batch, 2, 1, 16))
        kf, vf = m.tensor(F32, (batch, 24, 1, 16)), m.tensor(F32, (batch, 24, 1, 16))
        m.node(32, [pos, k, v], [kf, vf], custom_name="odml.update_kv_cache", init_data=minirt.flex_map({"kv_cache_max": 24}))
        m.set_io([pos, k, v], [kf, vf])

    assert claimed(kv) == 1
    assert claimed(lambda m: kv(m, batch=2)) == 0                         # the reference op is batch 1 only
    assert claimed(lambda m: kv(m, dtype_pos=I32)) == 0                   # positions are int64

    def embedding(m, table_const=True):
        ids = m.tensor(I32, (5,))
        table = m.tensor(I8, (40, 16), np.ones((40, 16), np.int8) if table_const else None,
                         channel_scales=np.full(40, 0.1, np.float32))
        y = m.tensor(F32, (5, 16))
        m.embedding_lookup(ids, table, y)
        m.set_io([ids] if table_const else [ids, table], [y])

    assert claimed(embedding) == 1
    assert claimed(lambda m: embedding(m, table_const=False)) == 0


def test_no_cuda_device_fails_loudly_and_rolls_back(plugin_path):
    """On a host without a usable CUDA device the kernel's init must fail (no CPU fallback inside
    the delegate), and the runtime must be left with its original plan."""
    import torch

    if torch.cuda.is_available():
        pytest.skip("a CUDA device is present")
    m, d = minirt.MiniRuntime(), minirt.Delegate()
    _fc_graph(m, x_type=F32, w_type=I8, y_type=F32)
    assert m.apply(d) == 2  # kTfLiteDelegateError
    assert "cudaSetDevice" in m.error
    assert m.partitions == 0 and m.cpu_nodes == 1 and m.plan_size == 1
    m.close()
    d.close()


# ----------------------------------------------------------------------------- arena planner
def _plan(lib, sizes, first, last, num_ops):
    n = len(sizes)
    offs = (ctypes.c_size_t * n)()
    lib.b200_arena_plan.restype = ctypes.c_size_t
    total = lib.b200_arena_plan(n, (ctypes.c_size_t * n)(*sizes), (ctypes.c_int * n)(*first), (ctypes.c_int * n)(*last),
                                num_ops, offs)
    return total, list(offs)


def test_arena_planner_no_live_overlap_and_reuse(plugin_path):
    lib = ctypes.CDLL(plugin_path)
    rng = np.random.default_rng(4)
    for trial in range(50):
        n, ops = int(rng.integers(1, 40)), int(rng.integers(1, 12))
        sizes = [int(s) for s in rng.integers(0, 5000, n)]
        first = [int(f) for f in rng.integers(0, ops, n)]
        last = [int(min(ops - 1, f + rng.integers(0, 4))) for f in first]
        total, offs = _plan(lib, sizes, first, last, ops)
        for i in range(n):
            assert offs[i] % 256 == 0 and offs[i] + sizes[i] <= total
            for j in range(i):
                if sizes[i] == 0 or sizes[j] == 0:
                    continue
                alive_together = not (last[i] < first[j] or last[j] < first[i])
                overlap = offs[i] < offs[j] + sizes[j] and offs[j] < offs[i] + sizes[i]
                assert not (alive_together and overlap)
    # a chain of equal-sized temporaries ping-pongs between two slots
    total, offs = _plan(lib, [1000] * 6, [0, 1, 2, 3, 4, 5], [1, 2, 3, 4, 5, 5], 6)
    assert total == 2 * 1024 and len(set(offs)) == 2


def test_arena_planner_matches_reference_arena(plugin_path, oracle):
    """Same ordering policy fed to the reference's SimpleMemoryArena (compiled from its own source)
    must give the same offsets."""
    ref = oracle.ref_lib()
    if ref is None or not hasattr(ref, "ref_arena_offsets"):
        pytest.skip("oracle/_ref not built")
    ref.ref_arena_offsets.restype = ctypes.c_size_t
    lib = ctypes.CDLL(plugin_path)
    rng = np.random.default_rng(5)
    for trial in range(30):
        n, ops = int(rng.integers(2, 30)), int(rng.integers(2, 10))
        sizes = [int(s) * 256 for s in rng.integers(1, 40, n)]
        first = [int(f) for f in rng.integers(0, ops, n)]
        last = [int(min(ops - 1, f + rng.integers(0, 3))) for f in first]
        total, offs = _plan(lib, sizes, first, last, ops)
        whole = [first[i] <= 0 and last[i] >= ops - 1 for i in range(n)]
        order = sorted(range(n), key=lambda i: (not whole[i], -sizes[i], first[i], i))
        roffs = (ctypes.c_size_t * n)()
        rtotal = ref.ref_arena_offsets(n, (ctypes.c_size_t * n)(*sizes), (ctypes.c_int * n)(*first),
                                       (ctypes.c_int * n)(*last), (ctypes.c_int * n)(*order), 256, roffs)
        assert (total, offs) == (rtotal, list(roffs))


# ----------------------------------------------------------------------------- attribute blob
def test_flex_map_reader_through_the_predicate(plugin_path):
    """The encoder used by the tests writes the documented FlexBuffers map layout; check a few
    structural facts so the GPU tests' `scale` really reaches the kernel."""
    blob = minirt.flex_map({"scale": 0.125, "logit_cap": 30.0})
    assert blob[-1] == 4 and blob[-2] >> 2 == 9
    assert b"logit_cap\0" in blob and b"scale\0" in blob
    assert blob.index(b"logit_cap") < blob.index(b"scale")  # keys sorted


def test_litert_accelerator_definition(plugin_path):
    """libLiteRtGpuAccelerator.so as the LiteRT environment sees it: the LiteRtAcceleratorImpl table
    (litert/c/internal/litert_accelerator_def.h:40-66), its ABI header, and a delegate out of
    create_delegate through the runtime context's wrap_delegate."""
    import subprocess

    from litert_b200 import build_delegate

    path = build_delegate.build_accelerator()
    if path is None:
        pytest.skip("accelerator library not built and LiteRT headers absent")
    exported = subprocess.run(["nm", "-D", "--defined-only", path], capture_output=True, text=True).stdout
    names = {line.split()[-1] for line in exported.splitlines() if line.strip()}
    assert "LiteRtAcceleratorImpl" in names
    acc = minirt.Accelerator(path)
    assert acc.rc == 0
    assert acc.name == "B200" and acc.version == (1, 0, 0)
    assert acc.hardware == 2          # kLiteRtHwAcceleratorGpu
    assert acc.struct_size == 200     # sizeof(LiteRtAcceleratorDefV1), asserted by the reference header too
    assert acc.ptr
    # the delegate it hands out is the plugin's: it partitions like the external delegate does
    m = minirt.MiniRuntime()
    w = m.tensor(minirt.I8, (4, 32), np.ones((4, 32), np.int8), channel_scales=np.full(4, 0.01, np.float32))
    x = m.tensor(minirt.F32, (2, 32))
    y = m.tensor(minirt.F32, (2, 4))
    m.fully_connected(x, w, None, y)
    m.set_io([x], [y])
    m.apply(acc)   # without a CUDA device: claimed in Prepare, kernel init fails, the plan is restored
    assert m.cpu_nodes + m.partitions >= 1
    m.close()
    acc.close()

