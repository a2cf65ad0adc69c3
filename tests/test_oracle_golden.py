"""Pins the CPU oracle to the reference: every golden vector and known-answer test the
reference's own unit tests hold for the path, plus the reference's own source files where they
compile on their own (oracle/_ref)."""
import ctypes

import numpy as np
import pytest

from tests.golden import reference_vectors as gv


def test_mbqm_int32_known_answers(oracle):
    for x, mult, expected in gv.MBQM_INT32_KATS:
        q, s = oracle.quantize_multiplier(mult)
        assert oracle.multiply_by_quantized_multiplier(x, q, s) == expected, (x, mult)
    # tflite/kernels/internal/quantization_util_test.cc:474-484
    x = m = 2**31 - 1
    expected = int(round(x * m / float(1 << 34)))
    assert oracle.multiply_by_quantized_multiplier(x, m, -3) == expected
    assert oracle.multiply_by_quantized_multiplier(-x, m, -3) == -expected


def test_mbqm_int64_known_answers(oracle):
    for x, mult, expected in gv.MBQM_INT64_KATS:
        q, s = oracle.quantize_multiplier(mult)
        assert oracle.multiply_by_quantized_multiplier_i64(x, q, s) == expected, (x, mult)
    x, m, shift, expected = gv.MBQM_INT64_MAX
    assert oracle.multiply_by_quantized_multiplier_i64(x, m, shift) == expected
    assert oracle.multiply_by_quantized_multiplier_i64(-x, m, shift) == -expected


def test_mbqm_matches_exact_rational_rounding(oracle):
    """The two primitives against their arithmetic definition in exact integers."""
    rng = np.random.default_rng(7)
    lib = oracle.lib()
    for _ in range(20000):
        a = int(rng.integers(-2**31, 2**31))
        b = int(rng.integers(-2**31, 2**31))
        if a == b == -2**31:
            continue
        # nearest to a*b/2^31, ties toward +inf
        want = (a * b + (1 << 30)) >> 31
        assert lib.orc_saturating_rounding_doubling_high_mul(a, b) == want
        e = int(rng.integers(0, 31))
        x = int(rng.integers(-2**31, 2**31))
        q, r = divmod(x, 1 << e)
        if e and (2 * r > (1 << e) or (2 * r == (1 << e) and x >= 0)):
            q += 1
        assert lib.orc_rounding_divide_by_pot(x, e) == q
    assert lib.orc_saturating_rounding_doubling_high_mul(-2**31, -2**31) == 2**31 - 1


def test_quantize_multiplier_matches_reference_source(oracle):
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(11)
    vals = np.concatenate([
        rng.uniform(0, 1, 20000) * 10.0 ** rng.uniform(-12, 4, 20000),
        -rng.uniform(0, 1, 2000) * 10.0 ** rng.uniform(-6, 2, 2000),
        [0.0, 1.0, 0.5, 0.99999999999, 2.0 ** -31, 2.0 ** -32, 2.0 ** -33, 1e-30]])
    for m in vals:
        q1, s1 = ctypes.c_int32(), ctypes.c_int()
        ref.ref_quantize_multiplier(ctypes.c_double(m), ctypes.byref(q1), ctypes.byref(s1))
        assert oracle.quantize_multiplier(float(m)) == (q1.value, s1.value), m


def test_activation_range_and_conv_multiplier_match_reference_source(oracle):
    ref = oracle.ref_lib()
    if ref is None:
        pytest.skip("oracle/_ref not built (reference tree absent)")
    rng = np.random.default_rng(12)
    for _ in range(2000):
        act = int(rng.integers(0, 4))
        scale = float(np.float32(10.0 ** rng.uniform(-3, 0.5)))
        zp = int(rng.integers(-128, 128))
        lo, hi = ctypes.c_int32(), ctypes.c_int32()
        rc = ref.ref_activation_range_int8(act, ctypes.c_float(scale), zp, ctypes.byref(lo), ctypes.byref(hi))
        assert rc == 0
        assert oracle.activation_range_int8(act, scale, zp) == (lo.value, hi.value)
        s_in = float(np.float32(10.0 ** rng.uniform(-3, 0)))
        s_w = float(np.float32(10.0 ** rng.uniform(-3, 0)))
        s_out = float(np.float32(10.0 ** rng.uniform(-2, 0)))
        mult = ctypes.c_double()
        rc = ref.ref_conv_multiplier(ctypes.c_float(s_in), ctypes.c_float(s_w), 0, ctypes.c_float(0),
                                     ctypes.c_float(s_out), ctypes.byref(mult))
        assert rc == 0
        assert oracle.fc_per_tensor_multiplier(s_in, s_w, None, s_out) == oracle.quantize_multiplier(mult.value)


def _int8_case(case):
    in_scale, in_zp = gv.quantization_params_int8(*case["input_range"])
    out_scale, out_zp = gv.quantization_params_int8(*case["output_range"])
    x = gv.quantize(case["input"], in_scale, in_zp).astype(np.int8)
    return in_scale, in_zp, out_scale, out_zp, x


@pytest.mark.parametrize("requant", [0, 1], ids=["mbqm", "float_ref"])
@pytest.mark.parametrize("name", sorted(gv.FC_INT8))
def test_fc_int8_goldens(oracle, name, requant):
    case = gv.FC_INT8[name]
    in_scale, in_zp, out_scale, out_zp, x = _int8_case(case)
    assert (float(in_scale), in_zp, float(out_scale), out_zp) == (0.5, -1, 1.0, -1)
    if case["kind"] == "per_tensor":
        if requant == 1:
            pytest.skip("float requant exists only for the per-channel kernel")
        w_scale, w_zp = gv.quantization_params_int8(*case["weight_range"])
        w = gv.quantize(case["weights"], w_scale, w_zp).astype(np.int8)
        bias = gv.quantize(case["bias"], np.float32(in_scale * w_scale), 0, -2**31, 2**31 - 1).astype(np.int32)
        y = oracle.fc_int8_per_tensor(x, w, bias, in_zp, in_scale, w_zp, w_scale, out_scale, out_zp,
                                      activation=oracle.ACT_RELU)
    else:
        scales = np.asarray(case["scales"], np.float32)
        w = gv.per_channel_symmetric_quantize(case["weights"], scales)
        bias = np.asarray([round(b / float(np.float32(s * in_scale))) for b, s in zip(case["bias"], scales)],
                          np.int32)
        y = oracle.fc_int8_per_channel(x, w, bias, in_zp, in_scale, scales, out_scale, out_zp,
                                       activation=oracle.ACT_RELU, requant=requant)
    assert y.reshape(-1).tolist() == case["expected"]


@pytest.mark.parametrize("name", sorted(gv.HYBRID_FC))
def test_fc_hybrid_goldens(oracle, name):
    case = gv.HYBRID_FC[name]
    if case["per_channel_scales"] is None:
        w, scale = gv.symmetric_quantize(case["weights"])
        scales = np.asarray([scale], np.float32)
    else:
        scales = np.asarray(case["per_channel_scales"], np.float32)
        w = gv.per_channel_symmetric_quantize(case["weights"], scales)
    y = oracle.fc_hybrid(np.asarray(case["input"], np.float32), w, scales, bias=np.asarray([1, 2, 3], np.float32),
                         asymmetric_inputs=case["asymmetric"], activation=oracle.ACT_RELU)
    np.testing.assert_allclose(y.reshape(-1), case["expected"], atol=case["max_abs_err"], rtol=0)


@pytest.mark.parametrize("zero_row", [False, True])
def test_int4_goldens_pin_nibble_order_and_blockwise_math(oracle, zero_row):
    """The reference's 4-bit hybrid goldens, fed to the blockwise restatement as one block per
    row with unit scale: same quantized inputs, same nibble order, same sum."""
    w = np.asarray(gv.HYBRID_INT4_WEIGHTS, np.int8)
    w4 = oracle.pack_int4(w)
    scales = np.ones((5, 1), np.float16)
    x = np.asarray(gv.HYBRID_INT4_INPUT_ZERO_ROW if zero_row else gv.HYBRID_INT4_INPUT, np.float32)
    y = oracle.fc_blockwise4(x, w4, scales, blocksize=40, bias=np.asarray(gv.HYBRID_INT4_BIAS, np.float32))
    want = gv.HYBRID_INT4_EXPECTED_ZERO_ROW if zero_row else gv.HYBRID_INT4_EXPECTED
    np.testing.assert_allclose(np.maximum(y, 0).reshape(-1), want, atol=gv.HYBRID_INT4_MAX_ABS_ERR, rtol=0)
    assert oracle.unpack_int4(w4, w.size).tolist() == w.reshape(-1).tolist()


def test_blockwise4_matches_independent_dequantized_matmul(oracle):
    rng = np.random.default_rng(3)
    m, n, k, bs = 3, 24, 128, 32
    w = rng.integers(-8, 8, (n, k)).astype(np.int8)
    sc = rng.uniform(1e-3, 2e-2, (n, k // bs)).astype(np.float16)
    x = rng.standard_normal((m, k)).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32)
    y = oracle.fc_blockwise4(x, oracle.pack_int4(w), sc, bs, bias)
    wf = w.astype(np.float64) * np.repeat(sc.astype(np.float64), bs, axis=1)
    want = x.astype(np.float64) @ wf.T + bias
    # 8-bit activation quantization noise: loose bound, catches layout mistakes only
    assert np.max(np.abs(y - want)) < 0.05 * np.max(np.abs(want))


@pytest.mark.parametrize("name", sorted(gv.BMM_FLOAT))
def test_bmm_float_goldens(oracle, name):
    c = gv.BMM_FLOAT[name]
    out = oracle.batch_matmul_float(np.asarray(c["x"], np.float32).reshape(c["x_shape"]),
                                    np.asarray(c["y"], np.float32).reshape(c["y_shape"]), c["adj_x"], c["adj_y"])
    assert out.shape == c["out_shape"]
    assert out.reshape(-1).tolist() == c["expected"]


@pytest.mark.parametrize("name", sorted(gv.BMM_HYBRID))
def test_bmm_hybrid_goldens(oracle, name):
    c = gv.BMM_HYBRID[name]
    yq, y_scale = gv.symmetric_quantize(c["y"])
    out = oracle.batch_matmul_hybrid(np.asarray(c["x"], np.float32).reshape(c["x_shape"]),
                                     yq.reshape(c["y_shape"]), y_scale, c["adj_x"], c["adj_y"], True)
    assert out.shape == c["out_shape"]
    np.testing.assert_allclose(out.reshape(-1), c["expected"], atol=c["max_abs_err"], rtol=0)


@pytest.mark.parametrize("name", sorted(gv.BMM_INT8))
def test_bmm_int8_goldens(oracle, name):
    c = gv.BMM_INT8[name]
    (xs, xzp), (ys, yzp), (os_, ozp) = [gv.quantization_params_int8(*r) for r in c["ranges"]]
    x = gv.quantize(c["x"], xs, xzp).astype(np.int8).reshape(c["x_shape"])
    y = gv.quantize(c["y"], ys, yzp).astype(np.int8).reshape(c["y_shape"])
    out = oracle.batch_matmul_int8(x, xzp, xs, y, yzp, ys, os_, ozp, adj_x=False, adj_y=c["adj_y"])
    assert out.reshape(-1).tolist() == c["expected"]


@pytest.mark.parametrize("name", sorted(gv.SDPA_SHAPES))
def test_sdpa_matches_float64_attention(oracle, name):
    """No numeric goldens exist for SDPA; the restatement is checked against a float64 numpy
    attention on the reference's own test shapes, at the tolerance its differential test uses
    (tflite/delegates/xnnpack/odml_sdpa_tester.cc:108-116), widened for float32 summation."""
    p = gv.SDPA_SHAPES[name]
    rng = np.random.default_rng(5)
    q = rng.uniform(0, 1, (p["b"], p["t"], p["n"], p["h"])).astype(np.float32)
    k = rng.uniform(0, 1, (p["b"], p["s"], p["nkv"], p["h"])).astype(np.float32)
    v = rng.uniform(0, 1, (p["b"], p["s"], p["nkv"], p["h"])).astype(np.float32)
    mask = rng.uniform(0, 1, (p["b"], 1, p["t"], p["s"])).astype(np.float32)
    out = oracle.sdpa_f32(q, k, v, mask)
    g = p["n"] // p["nkv"]
    kk = np.repeat(k.astype(np.float64), g, axis=2)
    vv = np.repeat(v.astype(np.float64), g, axis=2)
    logits = np.einsum("btnh,bsnh->bnts", q.astype(np.float64) / np.sqrt(p["h"]), kk) + mask.astype(np.float64)
    pr = np.exp(logits - logits.max(-1, keepdims=True))
    pr /= pr.sum(-1, keepdims=True)
    want = np.einsum("bnts,bsnh->btnh", pr, vv)
    np.testing.assert_allclose(out, want, atol=1e-5, rtol=1e-5)


def test_config1_spread_between_requant_flavours(oracle):
    """Full-int8 config (scaled down in M): the fixed-point and the float requantizations of the
    reference disagree by at most one LSB and rarely; recorded so the parity target is explicit."""
    rng = np.random.default_rng(1001)
    m, n, k = 8, 256, 2048
    x = rng.integers(-128, 128, (m, k)).astype(np.int8)
    w = np.clip(np.round(rng.normal(0, 40, (n, k))), -127, 127).astype(np.int8)
    fs = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    bias = rng.integers(-5000, 5001, n).astype(np.int32)
    a = oracle.fc_int8_per_channel(x, w, bias, -3, 0.02, fs, 0.05, 0, requant=oracle.REQUANT_MBQM)
    b = oracle.fc_int8_per_channel(x, w, bias, -3, 0.02, fs, 0.05, 0, requant=oracle.REQUANT_FLOAT_REF)
    diff = np.abs(a.astype(np.int32) - b.astype(np.int32))
    assert diff.max() <= 1
    assert (diff != 0).mean() < 0.02
