"""Regenerates tests/golden/odml_sdpa_composite_{mha,mqa,gqa}.tflite from the models the reference keeps
for its own differential test of the composite (tflite/delegates/xnnpack/odml_sdpa_composite_*.tflite.bin,
used by tflite/delegates/xnnpack/odml_sdpa_test.cc:81-110).

    LITERT_ROOT=<LiteRT checkout> python tests/golden/make_sdpa_models.py

Each model is read with litert_b200.tflite_model where it lies and written back with the same module's
writer: the main subgraph (the STABLEHLO_COMPOSITE node, its name, its attribute blob, the tensor shapes)
is kept as it is; of the decomposition subgraph the tensors and the operators' codes and wiring are kept
(the writer serialises builtin options only for the ops the delegate claims, and the delegate never runs a
decomposition). The GPU tests execute these files through the delegate; no test reads the checkout at run
time.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from litert_b200 import tflite_model as tm  # noqa: E402


def main():
    ref = os.environ.get("LITERT_ROOT") or os.path.join(os.path.dirname(ROOT), "reference")
    for name in ("mha", "mqa", "gqa"):
        src = os.path.join(ref, "tflite", "delegates", "xnnpack", f"odml_sdpa_composite_{name}.tflite.bin")
        model = tm.read_model(open(src, "rb").read())
        subgraphs = []
        for i, sg in enumerate(model.subgraphs):
            ops = []
            for op in sg.operators:
                keep = op.options if i == 0 else {}
                ops.append(tm.Operator(op.builtin_code, op.custom_code, op.version, list(op.inputs), list(op.outputs), keep,
                                       op.custom_options if i == 0 else b""))
            tensors = [tm.Tensor(t.name, list(t.shape), t.type, 0, t.quantization, t.is_variable, t.data if i == 0 else None)
                       for t in sg.tensors]
            subgraphs.append(tm.SubGraph(sg.name, tensors, list(sg.inputs), list(sg.outputs), ops))
        out = os.path.join(HERE, f"odml_sdpa_composite_{name}.tflite")
        data = tm.write_model(tm.Model(model.version, model.description, subgraphs))
        back = tm.read_model(data)
        op = back.subgraphs[0].operators[0]
        assert op.options["name"] == "odml.scaled_dot_product_attention"
        with open(out, "wb") as f:
            f.write(data)
        print(out, len(data), "bytes;", [back.subgraphs[0].tensors[t].shape for t in op.inputs])


if __name__ == "__main__":
    main()
