"""Golden vectors and known answers copied (numbers only) from the reference's own unit tests.

Each entry names the reference test file and lines it comes from (paths relative to the
reference project root). The helpers at the top restate, in numpy float32 arithmetic, how the
reference's test harness turns the float literals of a test into quantized tensors
(tflite/kernels/test_util.h): they are needed to reach the same int8 inputs the tests feed.
"""
import numpy as np

f32 = np.float32


# ---- tflite/kernels/test_util.h:1123-1203 (QuantizationParams<int8_t>) --------------------
def quantization_params_int8(f_min, f_max):
    qmin, qmax = f32(-128), f32(127)
    f_min, f_max = f32(f_min), f32(f_max)
    if f_min == f_max:
        return f32(0), 0
    scale = f32(f32(f_max - f_min) / f32(qmax - qmin))
    zp_from_min = f32(qmin - f32(f_min / scale))
    zp_from_max = f32(qmax - f32(f_max / scale))
    err_min = f32(abs(qmin) + abs(f32(f_min / scale)))
    err_max = f32(abs(qmax) + abs(f32(f_max / scale)))
    zp = zp_from_min if err_min < err_max else zp_from_max
    if zp < qmin:
        nudged = -128
    elif zp > qmax:
        nudged = 127
    else:
        nudged = int(np.floor(abs(float(zp)) + 0.5) * np.sign(float(zp)))  # std::round
    return scale, nudged


def _round_away(x):
    x = np.asarray(x, np.float32)
    return np.sign(x) * np.floor(np.abs(x) + f32(0.5))


# ---- tflite/kernels/test_util.h:197-220 (Quantize<T>) ------------------------------------
def quantize(data, scale, zero_point, lo=-128, hi=127):
    d = np.asarray(data, np.float32)
    q = _round_away(f32(zero_point) + d / f32(scale))
    return np.clip(q, lo, hi).astype(np.int32)


# ---- tflite/kernels/test_util.h:1407-1420 (QuantizeTensor -> SymmetricQuantizeFloats) ----
def symmetric_quantize(data):
    d = np.asarray(data, np.float32)
    rng = f32(max(abs(d.min()), abs(d.max())))
    scale = f32(rng / f32(127))
    inv = f32(f32(127) / rng)
    q = np.clip(_round_away(d * inv), -127, 127).astype(np.int8)
    return q, scale


# ---- tflite/kernels/test_util.h:753-815 (PerChannelSymmetricQuantizeAndPopulate, dim 0) ---
def per_channel_symmetric_quantize(data, scales):
    d = np.asarray(data, np.float32)
    inv = (f32(1.0) / np.asarray(scales, np.float32))[:, None]
    return np.clip(_round_away(d * inv), -127, 127).astype(np.int8)


# =========================================================================================
# tflite/kernels/internal/quantization_util_test.cc:447-485 -- (x, real multiplier, expected)
MBQM_INT32_KATS = [
    (0, 0.1, 0),
    (1, 0.0, 0),
    (10000, 0.00097656, 10),
    (-10000, 0.00097656, -10),
    (-(2**31), 0.00001, -21475),
    (2**31 - 1, 0.00001, 21475),
    (10000, -0.00097656, -10),
    (-10000, -0.00097656, 10),
    (-(2**31), -0.00001, 21475),
    (2**31 - 1, -0.00001, -21475),
]
# same file :487-515 -- int64 overload
MBQM_INT64_KATS = [
    (0, 0.1, 0),
    (1, 0.0, 0),
    (10000, 0.00097656, 10),
    (-10000, 0.00097656, -10),
    (-(2**47), 0.00001, -1407385600),
    (2**47 - 1, 0.00001, 1407385600),
]
# :503-514 -- (x, quantized_multiplier, shift, expected)
MBQM_INT64_MAX = ((2**47) - 1, 2**31 - 1, -31, 65534)

# =========================================================================================
# Full-integer FULLY_CONNECTED. Default fused activation of these test models is RELU
# (tflite/kernels/fully_connected_test.cc:151).
_FC_W = [[1, 2, 3, 4, 5, 6, 7, 8, 9, 10]] * 3
_FC_X = [[1, 2, 3, 4, 5, 6, 7, 8, -9, -10], [1, 2, 3, 4, 5, 6, 7, -8, 9, -10]]

FC_INT8 = {
    # tflite/kernels/fully_connected_test.cc:816-840
    "SimpleTestQuantizedInt8": dict(
        kind="per_tensor", input_range=(-63.5, 64), weight_range=(-63.5, 64), output_range=(-127, 128),
        weights=_FC_W, bias=[1, 2, 3], input=_FC_X, expected=[23, 24, 25, 57, 58, 59]),
    # tflite/kernels/fully_connected_test.cc:863-888
    "SimpleTestPerChannelQuantizedInt8": dict(
        kind="per_channel", input_range=(-63.5, 64), scales=[0.2, 0.25, 0.5], output_range=(-127, 128),
        weights=_FC_W, bias=[1, 2, 3], input=_FC_X, expected=[23, 24, 25, 57, 58, 59]),
    # tflite/kernels/fully_connected_test.cc:890-948 (input [2,2,5], keep_num_dims)
    "SimpleTestPerChannelQuantizedOutputShape3DInt8": dict(
        kind="per_channel", input_range=(-63.5, 64), scales=[0.2, 0.25, 0.5], output_range=(-127, 128),
        weights=[[1, 2, 3, 4, 5]] * 3, bias=[1, 2, 3],
        input=[[1, 2, 3, 4, -5], [1, 2, 3, -4, 5], [1, 2, -3, 4, 5], [1, -2, 3, 4, 5]],
        expected=[5, 6, 7, 23, 24, 25, 37, 38, 39, 47, 48, 49]),
}

# =========================================================================================
# Hybrid FULLY_CONNECTED (float in/out, int8 weights), activation RELU, bias {1,2,3}.
HYBRID_FC = {
    # tflite/kernels/fully_connected_test.cc:1728-1758 (symmetric inputs)
    "SimpleTestQuantizedInt8": dict(
        weights=_FC_W, per_channel_scales=None, asymmetric=False, input=_FC_X,
        expected=[24, 25, 26, 58, 59, 60], max_abs_err=1.3),
    # :1872-1904 (asymmetric inputs)
    "AsymmetricSimpleTestQuantizedInt8": dict(
        weights=_FC_W, per_channel_scales=None, asymmetric=True, input=_FC_X,
        expected=[24, 25, 26, 58, 59, 60], max_abs_err=1.3),
    # :1906-1948 (asymmetric inputs, per-channel weight scales {10,20,30}/127)
    "AsymmetricSimpleTestQuantizedPerChannelInt8": dict(
        weights=[list(range(1, 11)), list(range(11, 21)), list(range(21, 31))],
        per_channel_scales=[10.0 / 127.0, 20.0 / 127.0, 30.0 / 127.0], asymmetric=True, input=_FC_X,
        expected=[24, 195, 366, 58, 251, 441], max_abs_err=1.3),
}

# =========================================================================================
# tflite/kernels/fully_connected_4bit_test.cc:103-146 and :148-185. int4 weights with unit
# scale, 5 units x 40 columns, bias {1,2,3,1,2}, RELU, asymmetric inputs, batch 4.
_W4_A = [-1, 2, 3, 4, 5, 6, 7, 1, 2, 3]
_W4_B = [1, 2, 3, 4, 5, 6, 7, 1, 2, -3]
HYBRID_INT4_WEIGHTS = [
    _W4_A * 4,
    _W4_B + _W4_A * 3,
    _W4_B + _W4_A * 3,
    _W4_B + _W4_A * 3,
    _W4_A * 4,
]
_X4_A = [1, 2, 3, 4, 5, 6, 7, 8, -9, -10]
_X4_B = [1, 2, 3, 4, 5, 6, 7, -8, 9, -10]
HYBRID_INT4_BIAS = [1, 2, 3, 1, 2]
HYBRID_INT4_INPUT = [_X4_A * 4, _X4_B + _X4_A * 3, _X4_A * 4, _X4_A * 4]
HYBRID_INT4_EXPECTED = [393., 456., 457., 455., 394., 413., 476., 477., 475., 414.,
                        393., 456., 457., 455., 394., 393., 456., 457., 455., 394.]
HYBRID_INT4_INPUT_ZERO_ROW = [_X4_A * 4, _X4_B + _X4_A * 3, _X4_A * 4, [0] * 40]
HYBRID_INT4_EXPECTED_ZERO_ROW = HYBRID_INT4_EXPECTED[:15] + [1, 2, 3, 1, 2]
HYBRID_INT4_MAX_ABS_ERR = 1.3

# =========================================================================================
# BATCH_MATMUL
_BMM_RHS_3x2x4 = list(range(7, 31))
_BMM_BROADCAST2_OUT = [
    29., 32., 35., 38., 65., 72., 79., 86., 101., 112., 123., 134., 53., 56., 59., 62., 121., 128.,
    135., 142., 189., 200., 211., 222., 77., 80., 83., 86., 177., 184., 191., 198., 277., 288.,
    299., 310., 137., 152., 167., 182., 173., 192., 211., 230., 209., 232., 255., 278., 257., 272.,
    287., 302., 325., 344., 363., 382., 393., 416., 439., 462., 377., 392., 407., 422., 477., 496.,
    515., 534., 577., 600., 623., 646.]
BMM_FLOAT = {
    # tflite/kernels/batch_matmul_test.cc:118-130
    "Float32Test_Simple": dict(x_shape=(1, 2, 3), x=[1, 2, 3, 4, 5, 6], y_shape=(1, 3, 4),
                               y=list(range(7, 19)), adj_x=False, adj_y=False,
                               expected=[74., 80., 86., 92., 173., 188., 203., 218.], out_shape=(1, 2, 4)),
    # :159-170
    "Float32Test_SimpleRHSAdjoint": dict(x_shape=(1, 2, 3), x=[1, 2, 3, 4, 5, 6], y_shape=(1, 4, 3),
                                         y=[7, 11, 15, 8, 12, 16, 9, 13, 17, 10, 14, 18], adj_x=False,
                                         adj_y=True, expected=[74., 80., 86., 92., 173., 188., 203., 218.],
                                         out_shape=(1, 2, 4)),
    # :214-228
    "Float32Test_BroadcastLHSAdjoint": dict(
        x_shape=(2, 3, 2), x=[1, 4, 2, 5, 3, 6, 7, 10, 8, 11, 9, 12], y_shape=(3, 4), y=list(range(7, 19)),
        adj_x=True, adj_y=False,
        expected=[74., 80., 86., 92., 173., 188., 203., 218., 272., 296., 320., 344., 371., 404., 437., 470.],
        out_shape=(2, 2, 4)),
    # :230-253
    "Float32Test_Broadcast2": dict(x_shape=(2, 1, 3, 2), x=list(range(1, 13)), y_shape=(3, 2, 4),
                                   y=_BMM_RHS_3x2x4, adj_x=False, adj_y=False, expected=_BMM_BROADCAST2_OUT,
                                   out_shape=(2, 3, 3, 4)),
    # :255-278
    "Float32Test_Broadcast2LHSAdjoint": dict(
        x_shape=(2, 1, 2, 3), x=[1, 3, 5, 2, 4, 6, 7, 9, 11, 8, 10, 12], y_shape=(3, 2, 4), y=_BMM_RHS_3x2x4,
        adj_x=True, adj_y=False, expected=_BMM_BROADCAST2_OUT, out_shape=(2, 3, 3, 4)),
    # :280-303
    "Float32Test_Broadcast2RHSAdjoint": dict(
        x_shape=(2, 1, 3, 2), x=list(range(1, 13)), y_shape=(3, 4, 2),
        y=[7, 11, 8, 12, 9, 13, 10, 14, 15, 19, 16, 20, 17, 21, 18, 22, 23, 27, 24, 28, 25, 29, 26, 30],
        adj_x=False, adj_y=True, expected=_BMM_BROADCAST2_OUT, out_shape=(2, 3, 3, 4)),
}

BMM_HYBRID = {
    # tflite/kernels/batch_matmul_test.cc:504-533
    "SimpleTestQuantizedInt8": dict(
        x_shape=(2, 10), x=[11, 12, 13, 14, 15, 16, 17, 18, -19, -20, 11, 12, 13, 14, 15, 16, 17, -18, 19, -20],
        y_shape=(10, 3), y=[v for v in range(1, 11) for _ in range(3)], adj_x=False, adj_y=False,
        expected=[193, 193, 193, 247, 247, 247], max_abs_err=3.0, out_shape=(2, 3)),
    # :535-566
    "MultipleNumBatchQuantizedInt8": dict(
        x_shape=(1, 2, 2, 3), x=[11, 12, 13] * 4, y_shape=(3, 10),
        y=[1] * 5 + [2] * 5 + [3] * 5 + [1] * 5 + [2] * 5 + [3] * 5, adj_x=False, adj_y=False,
        expected=[73] * 40, max_abs_err=0.64, out_shape=(1, 2, 2, 10)),
    # :599-630
    "BatchesAndUnitsGreaterThanAccumDimSize": dict(
        x_shape=(6, 3), x=[11, 12, 13] * 6, y_shape=(3, 8), y=[1] * 8 + [2] * 8 + [3] * 8, adj_x=False,
        adj_y=False, expected=[74] * 48, max_abs_err=0.15, out_shape=(6, 8)),
    # :632-660
    "BatchesAndUnitsGreaterThanAccumDimSizeAdjX": dict(
        x_shape=(3, 6), x=[11] * 6 + [12] * 6 + [13] * 6, y_shape=(3, 8), y=[1] * 8 + [2] * 8 + [3] * 8,
        adj_x=True, adj_y=False, expected=[74] * 48, max_abs_err=0.15, out_shape=(6, 8)),
    # :662-696
    "BatchesAndUnitsGreaterThanAccumDimSizeAdjY": dict(
        x_shape=(6, 3), x=[11, 12, 13] * 6, y_shape=(8, 3), y=[1, 2, 3] * 8, adj_x=False, adj_y=True,
        expected=[74] * 48, max_abs_err=0.15, out_shape=(6, 8)),
}

_BMM_I8_W = [v for v in range(1, 11) for _ in range(3)]
BMM_INT8 = {
    # tflite/kernels/batch_matmul_test.cc:1045-1066
    "SimpleTestQuantizedInt8": dict(
        x_shape=(2, 10), x=sum(_FC_X, []), y_shape=(10, 3), y=_BMM_I8_W, adj_y=False,
        ranges=((-63.5, 64), (-63.5, 64), (-127, 128)), expected=[22, 22, 22, 56, 56, 56]),
    # :1068-1089
    "SimpleTestQuantizedInt8AdjRHS": dict(
        x_shape=(2, 10), x=sum(_FC_X, []), y_shape=(3, 10), y=_BMM_I8_W, adj_y=True,
        ranges=((-63.5, 64), (-63.5, 64), (-127, 128)), expected=[13, 64, 127, 19, 94, 127]),
}

# =========================================================================================
# tflite/delegates/xnnpack/odml_sdpa_test.cc:81-110 -- shapes of the custom-op differential tests
# (B, T, N, H) query; (B, S, Nkv, H) key/value. No numeric goldens exist for SDPA.
SDPA_SHAPES = {
    "MQA": dict(b=1, t=1, n=32, h=4, s=64, nkv=1),
    "MHA": dict(b=1, t=1, n=32, h=4, s=64, nkv=32),
    "GQA": dict(b=1, t=1, n=32, h=4, s=64, nkv=4),
}
