"""The `.tflite` reader / writer (litert_b200/tflite_model.py) and real-graph ingestion into the mini
runtime: round trips, the reference's own checked-in models (read where they lie, when the reference
tree is present), malformed files, and what the delegate claims in graphs loaded from files."""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import minirt  # noqa: E402
from litert_b200 import tflite_model as tm  # noqa: E402

REF = os.environ.get("LITERT_ROOT") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))),
                                                     "reference")
needs_reference = pytest.mark.skipif(not os.path.isdir(REF + "/tflite"), reason="reference tree not present")


def _fc_model(rng, m=3, n=16, k=64, kind="hybrid"):
    """One FULLY_CONNECTED in the three weight encodings the delegate claims."""
    T = tm.Tensor
    tensors, ops = [], []
    if kind == "int8":
        w = rng.integers(-127, 128, (n, k)).astype(np.int8)
        tensors = [T("x", [m, k], 9, 0, tm.Quantization(np.float32([0.02]), np.int64([-3]))),
                   T("w", [n, k], 9, 0, tm.Quantization(rng.uniform(1e-3, 1e-2, n).astype(np.float32), np.zeros(n, np.int64), 0),
                     data=w.tobytes()),
                   T("b", [n], 2, 0, None, data=rng.integers(-500, 500, n).astype(np.int32).tobytes()),
                   T("y", [m, n], 9, 0, tm.Quantization(np.float32([0.05]), np.int64([0])))]
        ops = [tm.Operator(tm.BUILTIN_FULLY_CONNECTED, "", 5, [0, 1, 2], [3], dict(fused_activation_function=1))]
    elif kind == "hybrid":
        w = rng.integers(-127, 128, (n, k)).astype(np.int8)
        tensors = [T("x", [m, k], 0, 0, None),
                   T("w", [n, k], 9, 0, tm.Quantization(rng.uniform(1e-3, 1e-2, n).astype(np.float32), np.zeros(n, np.int64), 0),
                     data=w.tobytes()),
                   T("y", [m, n], 0, 0, None)]
        ops = [tm.Operator(tm.BUILTIN_FULLY_CONNECTED, "", 9, [0, 1, -1], [2],
                           dict(asymmetric_quantize_inputs=True, keep_num_dims=True))]
    else:  # blockwise int4, fp16 scales, block 32
        packed = rng.integers(0, 256, (n, k // 2)).astype(np.uint8)
        scales = rng.uniform(1e-3, 2e-2, (n, k // 32)).astype(np.float16)
        tensors = [T("x", [m, k], 0, 0, None),
                   T("w4", [n, k], 17, 0, tm.Quantization(np.zeros(0, np.float32), np.zeros(0, np.int64), 0, 3, -1, 32),
                     data=packed.tobytes()),
                   T("y", [m, n], 0, 0, None),
                   T("w4_scales", [n, k // 32], 1, 0, None, data=scales.tobytes())]
        ops = [tm.Operator(tm.BUILTIN_FULLY_CONNECTED, "", 13, [0, 1], [2], dict(asymmetric_quantize_inputs=True))]
    sg = tm.SubGraph("main", tensors, [0], [ops[0].outputs[0]], ops)
    return tm.Model(3, f"fully connected, {kind}", [sg])


@pytest.mark.parametrize("kind", ["int8", "hybrid", "w4"])
def test_write_then_read_round_trip(kind):
    model = _fc_model(np.random.default_rng(1), kind=kind)
    blob = tm.write_model(model)
    assert blob[4:8] == b"TFL3"
    back = tm.read_model(blob)
    assert back.version == 3 and back.description == model.description
    a, b = model.subgraphs[0], back.subgraphs[0]
    assert (a.name, a.inputs, a.outputs) == (b.name, b.inputs, b.outputs)
    for ta, tb in zip(a.tensors, b.tensors):
        assert (ta.name, ta.shape, ta.type, ta.data) == (tb.name, tb.shape, tb.type, tb.data)
        if ta.quantization is None:
            assert tb.quantization is None
        else:
            qa, qb = ta.quantization, tb.quantization
            assert np.array_equal(qa.scale, qb.scale) and np.array_equal(qa.zero_point, qb.zero_point)
            assert (qa.quantized_dimension, qa.blockwise_scales, qa.block_size) == (
                qb.quantized_dimension, qb.blockwise_scales, qb.block_size)
    for oa, ob in zip(a.operators, b.operators):
        assert (oa.builtin_code, oa.inputs, oa.outputs, oa.version) == (ob.builtin_code, ob.inputs, ob.outputs, ob.version)
        for key, value in oa.options.items():
            assert ob.options[key] == value


def test_composite_and_custom_round_trip():
    attrs = minirt.flex_map({"scale": 0.125})
    T = tm.Tensor
    tensors = [T("q", [1, 1, 8, 64], 0, 0, None), T("k", [1, 32, 1, 64], 0, 0, None), T("v", [1, 32, 1, 64], 0, 0, None),
               T("mask", [1, 1, 1, 32], 0, 0, None), T("o", [1, 1, 8, 64], 0, 0, None), T("o2", [1, 1, 8, 64], 0, 0, None)]
    ops = [tm.Operator(tm.BUILTIN_STABLEHLO_COMPOSITE, "", 1, [0, 1, 2, 3], [4],
                       dict(name="odml.scaled_dot_product_attention", composite_attributes=attrs,
                            decomposition_subgraph_index=1)),
           tm.Operator(tm.BUILTIN_CUSTOM, "odml.scaled_dot_product_attention", 1, [0, 1, 2, 3], [5], {}, b"\x01\x02")]
    back = tm.read_model(tm.write_model(tm.Model(3, "", [tm.SubGraph("main", tensors, [0, 1, 2, 3], [4, 5], ops)])))
    o0, o1 = back.subgraphs[0].operators
    assert o0.builtin_code == tm.BUILTIN_STABLEHLO_COMPOSITE and o0.options["name"] == "odml.scaled_dot_product_attention"
    assert o0.options["composite_attributes"] == attrs and o0.options["decomposition_subgraph_index"] == 1
    assert o1.builtin_code == tm.BUILTIN_CUSTOM and o1.custom_code == "odml.scaled_dot_product_attention"
    assert o1.custom_options == b"\x01\x02"


def test_malformed_files_are_refused():
    good = tm.write_model(_fc_model(np.random.default_rng(2)))
    with pytest.raises(tm.ModelError):
        tm.read_model(b"")
    with pytest.raises(tm.ModelError):
        tm.read_model(good[:4] + b"XXXX" + good[8:])   # wrong file identifier
    with pytest.raises((tm.ModelError, Exception)):
        tm.read_model(good[:len(good) // 3])             # truncated: some offset points past the end
    with pytest.raises(tm.ModelError):
        tm.read_model(b"\xff\xff\xff\x7fTFL3" + good[8:])  # root offset outside the file


@needs_reference
def test_reference_sdpa_composite_models():
    """tflite/delegates/xnnpack/odml_sdpa_composite_{mha,mqa,gqa}.tflite.bin: the composite node, its
    name, its attribute map and the decomposition subgraph."""
    expect = {"mha": (32, 32), "mqa": (32, 1), "gqa": (32, None)}
    for name, (q_heads, kv_heads) in expect.items():
        m = tm.read_model(f"{REF}/tflite/delegates/xnnpack/odml_sdpa_composite_{name}.tflite.bin")
        main = m.subgraphs[0]
        assert len(m.subgraphs) == 2 and len(main.operators) == 1
        op = main.operators[0]
        assert op.builtin_code == tm.BUILTIN_STABLEHLO_COMPOSITE
        assert op.options["name"] == "odml.scaled_dot_product_attention"
        assert op.options["decomposition_subgraph_index"] == 1 and len(op.options["composite_attributes"]) > 0
        q, k = main.tensors[op.inputs[0]], main.tensors[op.inputs[1]]
        assert q.shape[2] == q_heads and (kv_heads is None or k.shape[2] == kv_heads)
        # the decomposition holds the two BATCH_MATMULs and a SOFTMAX of the float path
        codes = [o.builtin_code for o in m.subgraphs[1].operators]
        assert codes.count(tm.BUILTIN_BATCH_MATMUL) == 2 and 25 in codes


@needs_reference
def test_reference_blockwise_fc_model_is_claimed(plugin_path):
    """litert/test/testdata/qwen_fc_blockwise_quantized.tflite: int4 weights [1024, 1024], fp16 block scales,
    block 32, asymmetric inputs: the blockwise FULLY_CONNECTED the delegate claims."""
    m = tm.read_model(f"{REF}/litert/test/testdata/qwen_fc_blockwise_quantized.tflite")
    sg = m.subgraphs[0]
    op = sg.operators[0]
    w = sg.tensors[op.inputs[1]]
    assert op.builtin_code == tm.BUILTIN_FULLY_CONNECTED and w.type_name == "INT4" and w.shape == [1024, 1024]
    q = w.quantization
    assert q.block_size == 32 and sg.tensors[q.blockwise_scales].type_name == "FLOAT16"
    assert sg.tensors[q.blockwise_scales].shape == [1024, 32] and len(w.data) == 1024 * 1024 // 2
    rt, d = minirt.load_model(m), minirt.Delegate()
    rt.apply(d)   # no CUDA device here: the claim is counted in Prepare, kernel init then fails and rolls back
    assert d.claimed == 1
    rt.close()
    d.close()


@pytest.mark.parametrize("kind", ["int8", "hybrid", "w4"])
def test_generated_models_load_and_are_claimed(plugin_path, kind):
    model = tm.read_model(tm.write_model(_fc_model(np.random.default_rng(3), kind=kind)))
    rt, d = minirt.load_model(model), minirt.Delegate()
    rt.apply(d)
    assert d.claimed == 1, d.errors
    rt.close()
    d.close()
