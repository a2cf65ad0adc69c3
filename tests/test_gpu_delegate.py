"""The delegate end to end on a GPU, driven through the mini runtime the way the reference
interpreter drives an external delegate: reference goldens through FULLY_CONNECTED /
BATCH_MATMUL nodes, the SDPA composite and custom op against the oracle, mixed graphs with
CPU nodes in between, buffer handles, and host-side fault injection with roll-back."""
import numpy as np
import pytest

from tests import minirt
from tests.golden import reference_vectors as gv
from tests.minirt import F16, F32, I4, I8, I32, OP_SOFTMAX

pytestmark = pytest.mark.gpu


@pytest.fixture()
def rt():
    m = minirt.MiniRuntime()
    yield m
    m.close()


@pytest.fixture()
def delegate():
    d = minirt.Delegate()
    yield d
    d.close()


def _int8_fc_graph(m, case, keep_num_dims=False):
    in_scale, in_zp = gv.quantization_params_int8(*case["input_range"])
    out_scale, out_zp = gv.quantization_params_int8(*case["output_range"])
    xin = np.asarray(case["input"], np.float32)
    xq = gv.quantize(xin, in_scale, in_zp).astype(np.int8)
    n = len(case["weights"])
    if case["kind"] == "per_tensor":
        w_scale, w_zp = gv.quantization_params_int8(*case["weight_range"])
        wq = gv.quantize(case["weights"], w_scale, w_zp).astype(np.int8)
        w = m.tensor(I8, wq.shape, wq, scale=w_scale, zero_point=w_zp)
        bs = np.float32(in_scale * w_scale)
        bq = gv.quantize(case["bias"], bs, 0, -2**31, 2**31 - 1).astype(np.int32)
        b = m.tensor(I32, (n,), bq, scale=bs)
    else:
        scales = np.asarray(case["scales"], np.float32)
        wq = gv.per_channel_symmetric_quantize(case["weights"], scales)
        w = m.tensor(I8, wq.shape, wq, channel_scales=scales)
        bq = np.asarray([round(bv / float(np.float32(s * in_scale))) for bv, s in zip(case["bias"], scales)], np.int32)
        b = m.tensor(I32, (n,), bq, channel_scales=scales * in_scale)
    x = m.tensor(I8, xq.shape, scale=in_scale, zero_point=in_zp)
    y = m.tensor(I8, (xq.shape[0], n), scale=out_scale, zero_point=out_zp)
    m.fully_connected(x, w, b, y, activation=1, keep_num_dims=keep_num_dims)
    m.set_io([x], [y])
    m.write(x, xq)
    return x, y


@pytest.mark.parametrize("name", sorted(gv.FC_INT8))
def test_int8_fc_goldens_through_the_delegate(rt, delegate, name):
    x, y = _int8_fc_graph(rt, gv.FC_INT8[name])
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    assert rt.invoke() == 0, rt.error
    assert rt.view(y).reshape(-1).tolist() == gv.FC_INT8[name]["expected"]
    assert rt.invoke() == 0  # a second invocation reuses the packed weights
    assert rt.view(y).reshape(-1).tolist() == gv.FC_INT8[name]["expected"]


@pytest.mark.parametrize("name", sorted(gv.HYBRID_FC))
def test_hybrid_fc_goldens_through_the_delegate(rt, delegate, oracle, name):
    case = gv.HYBRID_FC[name]
    if case["per_channel_scales"] is None:
        wq, scale = gv.symmetric_quantize(case["weights"])
        w = rt.tensor(I8, wq.shape, wq, scale=scale)
        scales = np.asarray([scale], np.float32)
    else:
        scales = np.asarray(case["per_channel_scales"], np.float32)
        wq = gv.per_channel_symmetric_quantize(case["weights"], scales)
        w = rt.tensor(I8, wq.shape, wq, channel_scales=scales)
    xin = np.asarray(case["input"], np.float32)
    b = rt.tensor(F32, (3,), np.asarray([1, 2, 3], np.float32))
    x = rt.tensor(F32, xin.shape)
    y = rt.tensor(F32, (2, 3))
    rt.fully_connected(x, w, b, y, activation=1, asymmetric=case["asymmetric"])
    rt.set_io([x], [y])
    rt.write(x, xin)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    np.testing.assert_allclose(rt.view(y).reshape(-1), case["expected"], atol=case["max_abs_err"], rtol=0)
    want = oracle.fc_hybrid(xin, wq, scales, np.asarray([1, 2, 3], np.float32), case["asymmetric"], oracle.ACT_RELU)
    assert np.array_equal(rt.view(y), want)


def test_blockwise_int4_fc_through_the_delegate(rt, delegate, oracle):
    from litert_b200 import workloads

    c = workloads.config3(3, 200, 320, seed=11)
    w = rt.tensor(I4, (200, 320), c["w4"])
    s = rt.tensor(F16, (200, 10), c["scales"])
    rt.set_blockwise(w, s, 32)
    bias = np.linspace(-1, 1, 200).astype(np.float32)
    b = rt.tensor(F32, (200,), bias)
    x = rt.tensor(F32, (3, 320))
    y = rt.tensor(F32, (3, 200))
    rt.fully_connected(x, w, b, y)
    rt.set_io([x], [y])
    rt.write(x, c["x"])
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    want = oracle.fc_blockwise4(c["x"], c["w4"], c["scales"], 32, bias)
    np.testing.assert_allclose(rt.view(y), want, rtol=1e-3, atol=1e-3 * np.abs(want).max())


@pytest.mark.parametrize("name", ["SimpleTestQuantizedInt8", "MultipleNumBatchQuantizedInt8",
                                  "BatchesAndUnitsGreaterThanAccumDimSize",
                                  "BatchesAndUnitsGreaterThanAccumDimSizeAdjY"])
def test_hybrid_bmm_goldens_through_the_delegate(rt, delegate, name):
    c = gv.BMM_HYBRID[name]
    yq, y_scale = gv.symmetric_quantize(c["y"])
    w = rt.tensor(I8, c["y_shape"], yq.reshape(c["y_shape"]), scale=y_scale)
    x = rt.tensor(F32, c["x_shape"])
    out = rt.tensor(F32, c["out_shape"])
    rt.batch_matmul(x, w, out, adj_y=c["adj_y"])
    rt.set_io([x], [out])
    rt.write(x, np.asarray(c["x"], np.float32))
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    np.testing.assert_allclose(rt.view(out).reshape(-1), c["expected"], atol=c["max_abs_err"], rtol=0)


@pytest.mark.parametrize("name", sorted(gv.BMM_INT8))
def test_int8_bmm_goldens_through_the_delegate(rt, delegate, name):
    c = gv.BMM_INT8[name]
    (xs, xzp), (ys, yzp), (os_, ozp) = [gv.quantization_params_int8(*r) for r in c["ranges"]]
    xq = gv.quantize(c["x"], xs, xzp).astype(np.int8).reshape(c["x_shape"])
    yq = gv.quantize(c["y"], ys, yzp).astype(np.int8).reshape(c["y_shape"])
    w = rt.tensor(I8, c["y_shape"], yq, scale=ys, zero_point=yzp)
    x = rt.tensor(I8, c["x_shape"], scale=xs, zero_point=xzp)
    out = rt.tensor(I8, (2, 3), scale=os_, zero_point=ozp)
    rt.batch_matmul(x, w, out, adj_y=c["adj_y"])
    rt.set_io([x], [out])
    rt.write(x, xq)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    assert rt.view(out).reshape(-1).tolist() == c["expected"]


@pytest.mark.parametrize("form", ["composite", "custom"])
@pytest.mark.parametrize("name", sorted(gv.SDPA_SHAPES))
def test_sdpa_reference_shapes_through_the_delegate(rt, delegate, oracle, name, form):
    p = gv.SDPA_SHAPES[name]
    rng = np.random.default_rng(21)
    shapes = [(p["b"], p["t"], p["n"], p["h"]), (p["b"], p["s"], p["nkv"], p["h"]), (p["b"], p["s"], p["nkv"], p["h"]),
              (p["b"], 1, p["t"], p["s"])]
    data = [rng.uniform(0, 1, s).astype(np.float32) for s in shapes]
    ins = [rt.tensor(F32, s) for s in shapes]
    out = rt.tensor(F32, shapes[0])
    scale = 0.37
    blob = minirt.flex_map({"scale": scale})
    if form == "composite":
        rt.composite("odml.scaled_dot_product_attention", blob, ins, out)
    else:
        rt.custom("odml.scaled_dot_product_attention", blob, ins, out)
    rt.set_io(ins, [out])
    for t, d in zip(ins, data):
        rt.write(t, d)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1
    assert rt.invoke() == 0, rt.error
    want = oracle.sdpa_f32(*data, scale=scale)
    np.testing.assert_allclose(rt.view(out), want, rtol=1e-4, atol=1e-5)
    assert np.array_equal(rt.view(ins[0]), data[0])  # the query tensor is not scaled in place


def test_sdpa_decode_shape_default_scale(rt, delegate, oracle):
    rng = np.random.default_rng(22)
    b, n, nkv, h, s = 2, 8, 1, 256, 384
    shapes = [(b, 1, n, h), (b, s, nkv, h), (b, s, nkv, h), (b, 1, 1, s)]
    q, k, v = [rng.standard_normal(sh).astype(np.float32) for sh in shapes[:3]]
    mask = np.where(np.arange(s)[None, None, None, :] < np.asarray([300, 77])[:, None, None, None], 0, -1e30)
    mask = mask.astype(np.float32)
    ins = [rt.tensor(F32, sh) for sh in shapes]
    out = rt.tensor(F32, shapes[0])
    rt.composite("odml.scaled_dot_product_attention", b"", ins, out)  # no attributes: 1/sqrt(h)
    rt.set_io(ins, [out])
    for t, d in zip(ins, (q, k, v, mask)):
        rt.write(t, d)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    want = oracle.sdpa_f32(q, k, v, mask)
    assert np.max(np.abs(rt.view(out) - want)) / np.max(np.abs(want)) <= 2e-2


def _two_fc_with_cpu_node_between(m, rng):
    w1 = np.clip(np.rint(rng.standard_normal((24, 40)) * 40), -127, 127).astype(np.int8)
    w2 = np.clip(np.rint(rng.standard_normal((8, 24)) * 40), -127, 127).astype(np.int8)
    x = m.tensor(F32, (5, 40))
    t1 = m.tensor(F32, (5, 24))
    t2 = m.tensor(F32, (5, 24))
    y = m.tensor(F32, (5, 8))
    a = m.tensor(I8, w1.shape, w1, scale=0.01)
    b = m.tensor(I8, w2.shape, w2, scale=0.02)
    m.fully_connected(x, a, None, t1)
    m.other(OP_SOFTMAX, [t1], t2)  # stays on the CPU
    m.fully_connected(t2, b, None, y)
    m.set_io([x], [y])
    return x, t1, t2, y, w1, w2


@pytest.mark.parametrize("buffer_handles", [0, 1])
def test_mixed_graph_two_partitions_with_a_cpu_node_between(rt, oracle, buffer_handles):
    rng = np.random.default_rng(30)
    d = minirt.Delegate({"buffer_handles": buffer_handles})
    x, t1, t2, y, w1, w2 = _two_fc_with_cpu_node_between(rt, rng)
    xin = rng.standard_normal((5, 40)).astype(np.float32)
    rt.write(x, xin)
    stale_seen = []

    def cpu(node):
        stale_seen.append(rt.lib.mrt_tensor_is_stale(rt.h, t1))
        e = np.exp(rt.view(t1) - rt.view(t1).max(-1, keepdims=True))
        rt.write(t2, e / e.sum(-1, keepdims=True))
        return 0

    rt.set_cpu(cpu)
    assert rt.apply(d) == 0, rt.error
    assert d.claimed == 2 and rt.partitions == 2 and rt.cpu_nodes == 1
    assert rt.invoke() == 0, rt.error
    h1 = oracle.fc_hybrid(xin, w1, np.asarray([0.01], np.float32))
    e = np.exp(h1 - h1.max(-1, keepdims=True))
    want = oracle.fc_hybrid((e / e.sum(-1, keepdims=True)).astype(np.float32), w2, np.asarray([0.02], np.float32))
    assert np.array_equal(rt.view(t1), h1)
    assert np.array_equal(rt.view(y), want)
    assert stale_seen == [0]  # the runtime made the tensor readable before the CPU node ran
    rt.close()
    rt.h = None
    d.close()


def test_chain_in_one_partition_keeps_the_intermediate_on_the_device(rt, delegate, oracle):
    rng = np.random.default_rng(31)
    w1 = np.clip(np.rint(rng.standard_normal((300, 70)) * 40), -127, 127).astype(np.int8)
    w2 = np.clip(np.rint(rng.standard_normal((33, 300)) * 40), -127, 127).astype(np.int8)
    s1 = rng.uniform(1e-3, 1e-2, 300).astype(np.float32)
    s2 = rng.uniform(1e-3, 1e-2, 33).astype(np.float32)
    x = rt.tensor(F32, (9, 70))
    t = rt.tensor(F32, (9, 300))
    y = rt.tensor(F32, (9, 33))
    rt.fully_connected(x, rt.tensor(I8, w1.shape, w1, channel_scales=s1), None, t, activation=1)
    rt.fully_connected(t, rt.tensor(I8, w2.shape, w2, channel_scales=s2), None, y)
    rt.set_io([x], [y])
    xin = rng.standard_normal((9, 70)).astype(np.float32)
    rt.write(x, xin)
    rt.write(t, np.full((9, 300), 7.0, np.float32))
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1
    assert rt.invoke() == 0, rt.error
    h = oracle.fc_hybrid(xin, w1, s1, activation=oracle.ACT_RELU)
    assert np.array_equal(rt.view(y), oracle.fc_hybrid(h, w2, s2))
    assert np.all(rt.view(t) == 7.0)  # the intermediate never came back to the host


@pytest.mark.parametrize("where", ["init", "prepare", "alloc"])
def test_injected_failures_roll_back_to_the_cpu_plan(rt, where):
    rng = np.random.default_rng(32)
    d = minirt.Delegate({"fail_on": where})
    x, t1, t2, y, w1, w2 = _two_fc_with_cpu_node_between(rt, rng)
    assert rt.apply(d) == 2  # kTfLiteDelegateError
    assert rt.partitions == 0 and rt.cpu_nodes == 3 and rt.plan_size == 3
    ran = []
    rt.set_cpu(lambda node: ran.append(node) or 0)
    assert rt.invoke() == 0  # the untouched plan still runs, on the CPU kernels
    assert ran == [0, 1, 2]
    d.close()


def test_injected_invoke_failure_is_reported(rt):
    d = minirt.Delegate({"fail_on": "invoke"})
    _int8_fc_graph(rt, gv.FC_INT8["SimpleTestPerChannelQuantizedInt8"])
    assert rt.apply(d) == 0
    assert rt.invoke() == 2
    assert "injected failure in invoke" in rt.error
    d.close()


# ---- graphs ingested from `.tflite` files -------------------------------------------------------
def _model_from_file(kind, seed, m=5, n=200, k=320):
    """A `.tflite` file written and parsed again (litert_b200.tflite_model), so that every tensor, scale
    and option below reaches the delegate through the flatbuffer, as a user's model would."""
    import test_tflite_model as tt
    from litert_b200 import tflite_model as tm

    return tm.read_model(tm.write_model(tt._fc_model(np.random.default_rng(seed), m=m, n=n, k=k, kind=kind)))


def test_hybrid_fc_from_tflite_file(delegate, oracle):
    model = _model_from_file("hybrid", 21)
    sg = model.subgraphs[0]
    rt = minirt.load_model(model)
    x = np.random.default_rng(5).standard_normal((5, 320)).astype(np.float32)
    rt.write(sg.inputs[0], x)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    assert rt.invoke() == 0, rt.error
    w = sg.tensors[1]
    want = oracle.fc_hybrid(x, w.array(), w.quantization.scale, None, True, oracle.ACT_NONE)
    assert np.array_equal(rt.view(sg.outputs[0]).reshape(5, 200), want)
    rt.close()


def test_int8_fc_from_tflite_file(delegate, oracle):
    model = _model_from_file("int8", 22)
    sg = model.subgraphs[0]
    rt = minirt.load_model(model)
    xq = np.random.default_rng(6).integers(-128, 128, (5, 320)).astype(np.int8)
    rt.write(sg.inputs[0], xq)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    xt, wt, bt, yt = sg.tensors
    want = oracle.fc_int8_per_channel(xq, wt.array(), bt.array(), int(xt.quantization.zero_point[0]),
                                      float(xt.quantization.scale[0]), wt.quantization.scale,
                                      float(yt.quantization.scale[0]), int(yt.quantization.zero_point[0]),
                                      oracle.ACT_RELU)
    assert np.array_equal(rt.view(sg.outputs[0]).reshape(5, 200), want)
    rt.close()


def test_blockwise_int4_fc_from_tflite_file(delegate, oracle):
    model = _model_from_file("w4", 23)
    sg = model.subgraphs[0]
    rt = minirt.load_model(model)
    x = np.random.default_rng(7).standard_normal((5, 320)).astype(np.float32)
    rt.write(sg.inputs[0], x)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    w4 = np.frombuffer(sg.tensors[1].data, np.uint8).reshape(200, 160)
    scales = sg.tensors[3].array()
    want = oracle.fc_blockwise4(x, w4, scales, 32, None)
    np.testing.assert_allclose(rt.view(sg.outputs[0]).reshape(5, 200), want, rtol=1e-3, atol=1e-3 * np.abs(want).max())
    rt.close()


def test_hybrid_fc_through_the_litert_accelerator(rt, oracle):
    """The same delegate reached the LiteRT way: LiteRtAcceleratorImpl.create_delegate."""
    acc = minirt.Accelerator()
    assert acc.rc == 0 and acc.ptr
    rng = np.random.default_rng(31)
    wq = rng.integers(-127, 128, (48, 96)).astype(np.int8)
    scales = rng.uniform(1e-3, 1e-2, 48).astype(np.float32)
    xin = rng.standard_normal((3, 96)).astype(np.float32)
    w = rt.tensor(I8, wq.shape, wq, channel_scales=scales)
    x = rt.tensor(F32, xin.shape)
    y = rt.tensor(F32, (3, 48))
    rt.fully_connected(x, w, None, y, asymmetric=True)
    rt.set_io([x], [y])
    rt.write(x, xin)
    assert rt.apply(acc) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    assert rt.invoke() == 0, rt.error
    assert np.array_equal(rt.view(y), oracle.fc_hybrid(xin, wq, scales, None, True, oracle.ACT_NONE))
    rt.close()
    acc.close()



# ---- BATCH_MATMUL beyond a constant 2-D right-hand side ------------------------------------------------------
def _w8(rng, shape):
    return np.clip(np.rint(rng.standard_normal(shape) * 40), -127, 127).astype(np.int8)


BMM_CASES = [
    # (lhs shape, rhs shape, adj_x, adj_y, constant rhs, per-channel)
    ((15, 17, 40), (40, 24), False, False, True, False),        # the leading dimension folds into the rows (255 rows)
    ((1, 5, 17, 40), (24, 40), False, True, True, True),        # adj_y, per-channel scales along n
    ((2, 40, 17), (40, 24), True, False, True, False),          # adj_x: the LHS is transposed on the device
    ((3, 17, 40), (3, 40, 24), False, False, True, False),      # batched constant RHS
    ((1, 17, 40), (3, 40, 24), False, False, True, True),       # the LHS broadcasts over the RHS's batch
    ((4, 9, 130), (4, 130, 33), False, False, False, False),    # run-time RHS: repacked every invocation
    ((4, 130, 9), (4, 33, 130), True, True, False, False),      # both adjoint, run-time RHS
    ((1, 1, 300), (300, 1), False, False, True, False),         # a single output
]
# int8 x int8 has no per-row parameters: several broadcast batch dimensions as well
BMM_INT8_CASES = [c[:5] for c in BMM_CASES] + [
    ((3, 5, 17, 40), (40, 24), False, False, True),
    ((2, 3, 17, 40), (2, 1, 40, 24), False, False, True),
    ((1, 3, 17, 40), (2, 3, 40, 24), False, False, False),
]


@pytest.mark.parametrize("asymmetric", [True, False])
@pytest.mark.parametrize("xs,ws,adj_x,adj_y,const,per_channel", BMM_CASES)
def test_hybrid_bmm_random_shapes_against_the_oracle(rt, delegate, oracle, xs, ws, adj_x, adj_y, const, per_channel, asymmetric):
    """Bit-equal to the reference arithmetic, including the zero-point correction through float
    (tflite/kernels/internal/reference/batch_matmul.h:189,197)."""
    rng = np.random.default_rng(abs(hash((xs, ws, adj_x, adj_y))) % 2**31)
    x_data = (rng.standard_normal(xs) * 2.0 + 0.7).astype(np.float32)
    w_data = _w8(rng, ws)
    n = ws[-2] if adj_y else ws[-1]
    kw = dict(scale=0.013)
    pc = None
    if per_channel:
        pc = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
        kw = dict(channel_scales=pc, quantized_dimension=len(ws) - 2 if adj_y else len(ws) - 1)
    w = rt.tensor(I8, ws, w_data if const else None, **kw)
    x = rt.tensor(F32, xs)
    want = oracle.batch_matmul_hybrid(x_data, w_data, 0.013, adj_x, adj_y, asymmetric, per_channel_scales=pc)
    out = rt.tensor(F32, want.shape)
    rt.batch_matmul(x, w, out, adj_x=adj_x, adj_y=adj_y, asymmetric=asymmetric)
    rt.set_io([x] if const else [x, w], [out])
    rt.write(x, x_data)
    if not const:
        rt.write(w, w_data)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    for _ in range(2):   # twice: a run-time RHS is repacked per invocation, temporaries are reused
        assert rt.invoke() == 0, rt.error
        assert np.array_equal(rt.view(out), want), np.max(np.abs(rt.view(out) - want))


def test_hybrid_bmm_zero_point_correction_goes_through_float(rt, delegate, oracle):
    """abs(row_sum x zero_point) above 2^24: the reference's `total -= row_sum * batch_offset` (float
    batch_offset) rounds where int32 arithmetic would not. The delegate reproduces it; FULLY_CONNECTED on the
    same data (int32 correction) must differ from it somewhere, or the case would prove nothing."""
    rng = np.random.default_rng(5)
    k, n, m = 4096, 64, 6
    w_data = rng.integers(100, 128, (k, n)).astype(np.int8)      # row sums near 4.7e5, with many significant bits
    x_data = rng.uniform(0.05, 0.15, (m, k)).astype(np.float32)  # all positive: zero point -128 ...
    x_data[:, 0] = 5.0                                           # ... and nearly every value quantizes close to it
    q, s, zp = oracle.batch_quantize_floats(x_data)
    assert np.all(np.abs(zp.astype(np.int64) * 127 * k) > 2**24)
    w = rt.tensor(I8, (k, n), w_data, scale=0.01)
    x = rt.tensor(F32, (m, k))
    out = rt.tensor(F32, (m, n))
    rt.batch_matmul(x, w, out)
    rt.set_io([x], [out])
    rt.write(x, x_data)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.invoke() == 0, rt.error
    want = oracle.batch_matmul_hybrid(x_data, w_data, 0.01)
    assert np.array_equal(rt.view(out), want)
    as_fc = oracle.fc_hybrid(x_data, np.ascontiguousarray(w_data.T), np.float32(0.01))
    assert not np.array_equal(as_fc, want), "the float detour is not exercised by this data"


@pytest.mark.parametrize("xs,ws,adj_x,adj_y,const", BMM_INT8_CASES)
def test_int8_bmm_random_shapes_bit_exact(rt, delegate, oracle, xs, ws, adj_x, adj_y, const):
    rng = np.random.default_rng(abs(hash((xs, ws, adj_x, adj_y, 8))) % 2**31)
    x_data = rng.integers(-128, 128, xs).astype(np.int8)
    w_data = _w8(rng, ws)
    x_scale, x_zp, w_scale, w_zp, o_scale, o_zp = 0.05, -7, 0.02, 3, 4.0, -11
    want = oracle.batch_matmul_int8(x_data, x_zp, x_scale, w_data, w_zp, w_scale, o_scale, o_zp, adj_x, adj_y)
    w = rt.tensor(I8, ws, w_data if const else None, scale=w_scale, zero_point=w_zp)
    x = rt.tensor(I8, xs, scale=x_scale, zero_point=x_zp)
    out = rt.tensor(I8, want.shape, scale=o_scale, zero_point=o_zp)
    rt.batch_matmul(x, w, out, adj_x=adj_x, adj_y=adj_y)
    rt.set_io([x] if const else [x, w], [out])
    rt.write(x, x_data)
    if not const:
        rt.write(w, w_data)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    assert rt.invoke() == 0, rt.error
    assert np.array_equal(rt.view(out), want)
    assert want.size < 100 or len(np.unique(want)) > 20


# ---- the composite with several query tokens, float16 tensors, and the reference's own models ---------------
@pytest.mark.parametrize("dtype", ["f32", "f16"])
@pytest.mark.parametrize("b,t,n,nkv,h,s", [(2, 5, 8, 1, 256, 300), (1, 33, 8, 2, 64, 70), (2, 3, 6, 6, 24, 40)])
def test_sdpa_with_several_query_tokens_through_the_delegate(rt, delegate, oracle, dtype, b, t, n, nkv, h, s):
    """A prompt-shaped composite: [b, t, n, h] queries, an arbitrary additive mask [b, 1, t, s] (here causal
    behind a cached prefix, with noise where it is open), float32 or float16 tensors."""
    rng = np.random.default_rng(b * 100 + t)
    np_t = np.float32 if dtype == "f32" else np.float16
    tt = F32 if dtype == "f32" else F16
    q = rng.standard_normal((b, t, n, h)).astype(np_t)
    k = rng.standard_normal((b, s, nkv, h)).astype(np_t)
    v = rng.standard_normal((b, s, nkv, h)).astype(np_t)
    prefix = s - t
    open_ = np.arange(s)[None, None, None, :] <= (prefix + np.arange(t))[None, None, :, None]
    mask = np.where(open_, rng.uniform(-1, 0, (b, 1, t, s)), -1e30).astype(np.float32)
    ins = [rt.tensor(tt, q.shape), rt.tensor(tt, k.shape), rt.tensor(tt, v.shape), rt.tensor(F32, mask.shape)]
    out = rt.tensor(tt, q.shape)
    rt.composite("odml.scaled_dot_product_attention", minirt.flex_map({"scale": 0.11}), ins, out)
    rt.set_io(ins, [out])
    for tensor, d in zip(ins, (q, k, v, mask)):
        rt.write(tensor, d)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0
    assert rt.skippable_subgraphs == 1   # the composite's decomposition subgraph was marked for the runtime
    assert rt.invoke() == 0, rt.error
    want = oracle.sdpa_f32(q.astype(np.float32), k.astype(np.float32), v.astype(np.float32), mask, 0.11)
    got = rt.view(out).astype(np.float32)
    assert np.max(np.abs(got - want)) / np.max(np.abs(want)) <= (2e-2 if h in (64, 128, 256) or dtype == "f16" else 1e-4)


@pytest.mark.parametrize("name", ["mha", "mqa", "gqa"])
def test_reference_sdpa_composite_models_run_on_the_device(delegate, oracle, name):
    """The models the reference keeps for its differential test of the composite
    (tflite/delegates/xnnpack/odml_sdpa_composite_{mha,mqa,gqa}.tflite.bin, regenerated into tests/golden by
    make_sdpa_models.py), loaded from their .tflite bytes, claimed whole and executed, inputs drawn as
    tflite/delegates/xnnpack/odml_sdpa_tester.cc:81-99 draws them (uniform in [0, 1))."""
    import os

    from litert_b200 import tflite_model as tm

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", f"odml_sdpa_composite_{name}.tflite")
    model = tm.read_model(open(path, "rb").read())
    rt = minirt.load_model(model)
    sg = model.subgraphs[0]
    op = sg.operators[0]
    rng = np.random.default_rng(31)
    data = [rng.uniform(0, 1, sg.tensors[i].shape).astype(np.float32) for i in op.inputs]
    for i, d in zip(op.inputs, data):
        rt.write(i, d)
    assert rt.apply(delegate) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0 and delegate.claimed == 1
    assert rt.invoke() == 0, rt.error
    import struct
    # The node's attribute blob is a FlexBuffers map {"scale": float}: the delegate decodes it; here every
    # aligned float in the blob is a candidate, and exactly the right one reproduces the device's output.
    attrs = op.options["composite_attributes"]
    candidates = {float(struct.unpack_from("<f", attrs, o)[0]) for o in range(0, max(len(attrs) - 3, 0))}
    best = min((float(np.max(np.abs(rt.view(op.outputs[0]) - oracle.sdpa_f32(*data, scale=c))))
                for c in candidates if 1e-3 < c < 10), default=1.0)
    assert best <= 1e-4, best
    rt.close()


# ---- a whole decoder behind the delegate ------------------------------------------------------------------------
def _host_weights(cfg, seed):
    from litert_b200 import decoder as dec

    w = dec.make_weights(cfg, seed=seed, device="cpu")
    out = dict(layers=[{k: v.numpy() for k, v in lw.items()} for lw in w["layers"]])
    for k in ("embed", "embed_scales", "final_norm"):
        out[k] = w[k].numpy()
    return out


@pytest.mark.parametrize("tokens_per_call", [1, 6])
def test_gemma_shaped_graph_is_one_partition_and_matches_the_cpu_graph(oracle, tokens_per_call):
    """The graph a converter would emit for a Gemma-shaped decoder (EMBEDDING_LOOKUP, odml.rms_norm, hybrid
    FULLY_CONNECTED, RESHAPE, the rotary embedding out of SLICE / MUL / CONCATENATION / ADD, odml.update_kv_cache,
    the attention composite, GELU, residual ADDs, the LM head, ARG_MAX): every node is claimed, the plan is ONE
    delegate kernel with no CPU node, the kv caches stay on the device between invocations, and the logits follow
    the CPU restatement of the same graph (float32 cache, as the reference's kv-cache op keeps it) step by step."""
    from tests.minirt.decoder_graph import DecoderGraph

    cfg = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=1, head_dim=64, d_ff=512, vocab=1000)
    host = _host_weights(cfg, 77)
    S, T = 32, tokens_per_call
    rt, d = minirt.MiniRuntime(), minirt.Delegate()
    g = DecoderGraph(rt, cfg, host, T, S)
    n_nodes = rt.plan_size
    assert rt.apply(d) == 0, rt.error
    assert rt.partitions == 1 and rt.cpu_nodes == 0 and d.claimed == n_nodes
    assert rt.skippable_subgraphs >= cfg["n_layers"]          # the composites' decomposition subgraphs
    ref = oracle.DecoderRef(cfg, host, 1, S, fast=False, kv_mode=0)
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, cfg["vocab"], 18).astype(np.int32)
    pos, worst = 0, 0.0
    while pos + T <= tokens.size:
        g.feed(tokens[pos:pos + T], pos)
        assert rt.invoke() == 0, rt.error
        logits = rt.view(g.logits).copy()
        picked = rt.view(g.tokens).copy()
        for i in range(T):
            nxt_r, lr = ref.step(tokens[pos + i:pos + i + 1], want_logits=True)
            err = np.linalg.norm(logits[i] - lr[0]) / np.linalg.norm(lr[0])
            worst = max(worst, err)
            assert err <= 6e-2, (pos, i, err)
            assert picked[i] == int(np.argmax(logits[i])), "ARG_MAX is the first index of the row's maximum"
            top2 = np.sort(lr[0])[-2:]
            if top2[1] - top2[0] > 4 * np.max(np.abs(logits[i] - lr[0])):
                assert picked[i] == nxt_r[0]
        pos += T
    print(f"decoder graph through the delegate, {T} token(s) per call: worst relative L2 {worst:.3e}")
    # the same graph with the fusion pass off (every node its own kernels) and without the logits as an output
    # (the LM head then picks the token in its epilogue): same tokens where the margin is clear
    for options, logits_out in (({"fuse": 0}, True), ({}, False)):
        rt2, d2 = minirt.MiniRuntime(), minirt.Delegate(options)
        g2 = DecoderGraph(rt2, cfg, host, T, S, want_logits=logits_out)
        assert rt2.apply(d2) == 0 and rt2.partitions == 1 and rt2.cpu_nodes == 0
        ref2 = oracle.DecoderRef(cfg, host, 1, S, fast=False, kv_mode=0)
        for p0 in range(0, (tokens.size // T) * T, T):
            g2.feed(tokens[p0:p0 + T], p0)
            assert rt2.invoke() == 0, rt2.error
            picked = rt2.view(g2.tokens).copy()
            for i in range(T):
                nxt_r, lr = ref2.step(tokens[p0 + i:p0 + i + 1], want_logits=True)
                top2 = np.sort(lr[0])[-2:]
                if top2[1] - top2[0] > 0.1 * (lr[0].max() - lr[0].min()):
                    assert picked[i] == nxt_r[0], (options, p0, i)
        rt2.close()
        d2.close()
        ref2.close()
    # a write past the cache's last slot is refused with an error, not executed
    g.feed(tokens[:T], S - T + 1)
    assert rt.invoke() != 0 and "cache" in rt.error
    rt.close()
    d.close()
    ref.close()
