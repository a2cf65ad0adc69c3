"""Parity of the CUDA path with the CPU oracle, through the C ABI (litert_b200.ops is a thin ctypes
mirror). Integer paths must be bit-exact; the hybrid and blockwise paths are compared at rel 1e-3
(and are in fact expected to be bit-equal, which is asserted where the summation order is fixed);
SDPA at 2e-2 against the fp32 oracle on up-converted inputs."""
import numpy as np
import pytest
import torch

from litert_b200 import workloads
from tests.golden import reference_vectors as gv

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ops():
    from litert_b200 import ops as _ops

    return _ops


@pytest.fixture(scope="module")
def ws(ops):
    w = ops.Workspace("cuda", scratch_bytes=64 << 20)
    yield w
    w.check_status()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return np.max(np.abs(a - b)) / max(np.max(np.abs(b)), 1e-30)


# --------------------------------------------------------------------------- quantization
def _quant_rows(rng, m, k):
    x = rng.standard_normal((m, k)).astype(np.float32)
    if m > 1:
        x[1] = 0.0                       # all-zero row: scale 1, zero point 0
    if m > 2:
        x[2] = np.abs(x[2]) + 0.5        # strictly positive row: rmin clamps to 0
    if m > 3:
        x[3] = -np.abs(x[3]) - 0.5       # strictly negative row
    if m > 4:
        x[4] = 3.0                       # constant row
    if m > 5:
        x[5] *= 1e-20                    # tiny magnitudes
    if m > 6:
        x[6] *= 1e6
    return x


@pytest.mark.parametrize("asymmetric", [True, False])
@pytest.mark.parametrize("m,k", [(1, 10), (9, 40), (7, 1000), (16, 4096), (3, 2049)])
def test_quantize_rows_bit_exact(ops, oracle, m, k, asymmetric):
    rng = np.random.default_rng(100 + m + k)
    x = _quant_rows(rng, m, k)
    q, s, z = ops.quantize_rows(dev(x), asymmetric)
    qo, so, zo = oracle.batch_quantize_floats(x, asymmetric)
    assert np.array_equal(z.cpu().numpy(), zo)
    assert np.array_equal(s.cpu().numpy().view(np.uint32), so.view(np.uint32))
    assert np.array_equal(q.cpu().numpy(), qo)


# --------------------------------------------------------------------------- full-integer FC
def _run_fc_int8(ops, oracle, ws, c, activation=0):
    mult, shift = oracle.fc_per_channel_multipliers(c["input_scale"], c["output_scale"], c["filter_scales"])
    lo, hi = oracle.activation_range_int8(activation, float(c["output_scale"]), c["output_zp"])
    wp = ops.PackedInt8Weights(dev(c["w"]))
    bias = None if c.get("bias") is None else dev(c["bias"])
    y = ops.fully_connected_int8(dev(c["x"]), wp, bias, c["input_zp"], c["output_zp"], dev(mult), dev(shift), lo, hi,
                                 ws=ws)
    want = oracle.fc_int8_per_channel(c["x"], c["w"], c.get("bias"), c["input_zp"], c["input_scale"],
                                      c["filter_scales"], c["output_scale"], c["output_zp"], activation)
    return y.cpu().numpy(), want


def test_fc_int8_config1_bit_exact(ops, oracle, ws):
    got, want = _run_fc_int8(ops, oracle, ws, workloads.config1())
    assert got.shape == (32, 2048)
    assert np.array_equal(got, want)
    assert len(np.unique(got)) > 100  # not saturated: the comparison means something


# The last two rows aim at the kernels chosen by shape: few n tiles with a long reduction (cluster
# split-K, splits of 8 / 6 / 3 / 2 and a k range that leaves some CTAs of a cluster without work), and
# more than 128 activation rows (the persistent prefill kernel: partial last pass, partial last n tile,
# an output row length that rules out 16-byte stores).
@pytest.mark.parametrize("m,n,k", [(1, 1, 1), (1, 130, 100), (5, 64, 16), (17, 257, 333), (33, 128, 128),
                                   (64, 300, 2048), (65, 129, 257), (130, 40, 70),
                                   (1, 384, 4096), (5, 2560, 2048), (17, 2000, 300), (33, 1000, 1100), (64, 128, 8200),
                                   (100, 2048, 2048), (128, 300, 700),
                                   (257, 20000, 256), (300, 19001, 130), (512, 18944, 384), (600, 37890, 100)])
def test_fc_int8_ragged_shapes_bit_exact(ops, oracle, ws, m, n, k):
    c = workloads.config1(m, n, k, seed=7 + m + n + k)
    if (m + n) % 2:
        c["bias"] = None
    got, want = _run_fc_int8(ops, oracle, ws, c, activation=(m + k) % 4)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("name", sorted(gv.FC_INT8))
def test_fc_int8_reference_goldens(ops, oracle, ws, name):
    case = gv.FC_INT8[name]
    in_scale, in_zp = gv.quantization_params_int8(*case["input_range"])
    out_scale, out_zp = gv.quantization_params_int8(*case["output_range"])
    x = gv.quantize(case["input"], in_scale, in_zp).astype(np.int8)
    lo, hi = oracle.activation_range_int8(oracle.ACT_RELU, float(out_scale), out_zp)
    if case["kind"] == "per_tensor":
        w_scale, w_zp = gv.quantization_params_int8(*case["weight_range"])
        w = gv.quantize(case["weights"], w_scale, w_zp).astype(np.int8)
        bias = gv.quantize(case["bias"], np.float32(in_scale * w_scale), 0, -2**31, 2**31 - 1).astype(np.int32)
        m_, s_ = oracle.fc_per_tensor_multiplier(in_scale, w_scale, np.float32(in_scale * w_scale), out_scale)
        mult, shift = np.asarray([m_], np.int32), np.asarray([s_], np.int32)
        fzp = w_zp
    else:
        scales = np.asarray(case["scales"], np.float32)
        w = gv.per_channel_symmetric_quantize(case["weights"], scales)
        bias = np.asarray([round(b / float(np.float32(s * in_scale))) for b, s in zip(case["bias"], scales)], np.int32)
        mult, shift = oracle.fc_per_channel_multipliers(in_scale, out_scale, scales)
        fzp = 0
    wp = ops.PackedInt8Weights(dev(w))
    y = ops.fully_connected_int8(dev(x), wp, dev(bias), in_zp, out_zp, dev(mult), dev(shift), lo, hi,
                                 filter_zero_point=fzp, ws=ws)
    assert y.cpu().numpy().reshape(-1).tolist() == case["expected"]


def _requant_on_device(ops, ws, acc, mult, shift, output_offset):
    """Pushes int32 accumulators through the kernel's fixed-point requantization: one output channel per
    value, weight 1 x input 0, the accumulator as the channel's bias, so y[n] = clamp(MBQM(acc[n]) + offset)."""
    n = len(acc)
    w = ops.PackedInt8Weights(dev(np.ones((n, 1), np.int8)))
    y = ops.fully_connected_int8(dev(np.zeros((1, 1), np.int8)), w, dev(np.asarray(acc, np.int32)), 0, output_offset,
                                 dev(np.asarray(mult, np.int32)), dev(np.asarray(shift, np.int32)), -128, 127, ws=ws)
    return y.cpu().numpy().reshape(-1).astype(np.int64)


def test_requantization_known_answers_on_the_device(ops, oracle, ws):
    """tflite/kernels/internal/quantization_util_test.cc:447-485 through the device's requantize_mbqm: zero
    multiplier, INT32_MIN / INT32_MAX inputs, negative multipliers, and max x max at shift -3. The int8
    output clamps, so each case runs with the output offset that brings its expected value to 5."""
    cases = []
    for x, real, expected in gv.MBQM_INT32_KATS:
        q, s = oracle.quantize_multiplier(real)
        cases.append((x, q, s, expected))
    m = 2**31 - 1
    e = int(round(m * m / float(1 << 34)))
    cases += [(m, m, -3, e), (-m, m, -3, -e)]
    # left shifts (real multipliers above 1) and the saturating INT32_MIN x INT32_MIN product
    for x, real in [(25, 3.7), (-25, 3.7), (1000, 1.0), (-7, 100.5), (12345, 2.0**-40)]:
        q, s = oracle.quantize_multiplier(real)
        cases.append((x, q, s, oracle.multiply_by_quantized_multiplier(x, q, s)))
    cases.append((-(2**31), -(2**31), 0, oracle.multiply_by_quantized_multiplier(-(2**31), -(2**31), 0)))
    for x, q, s, expected in cases:
        assert oracle.multiply_by_quantized_multiplier(x, q, s) == expected
        off = 5 - expected
        if not -(2**31) <= off < 2**31:
            off = -(2**31) + 1 if off < 0 else 2**31 - 1
        want = max(-128, min(127, ((expected + off + 2**31) % 2**32) - 2**31))
        got = _requant_on_device(ops, ws, [x], [q], [s], off)
        assert got[0] == want, (x, q, s, expected, got[0])


def test_requantization_random_sweep_on_the_device(ops, oracle, ws):
    """4096 channels with random accumulators, multipliers and shifts from -20 to +3, against the oracle."""
    rng = np.random.default_rng(77)
    n = 4096
    shift = rng.integers(-20, 4, n).astype(np.int32)
    mult = rng.integers(2**30, 2**31, n).astype(np.int64)
    mult[::7] *= -1
    mult[5] = 0
    # accumulators sized so that most results land inside int8
    mag = np.clip(60.0 * 2.0 ** (-shift.astype(np.float64)), 1, 2**31 - 1)
    acc = (rng.uniform(-1, 1, n) * mag).astype(np.int64)
    want = np.asarray([max(-128, min(127, oracle.multiply_by_quantized_multiplier(int(a), int(q), int(s))))
                       for a, q, s in zip(acc, mult, shift)])
    got = _requant_on_device(ops, ws, acc, mult, shift, 0)
    assert np.array_equal(got, want)
    assert len(np.unique(want)) > 100


# --------------------------------------------------------------------------- hybrid FC
@pytest.mark.parametrize("name", sorted(gv.HYBRID_FC))
def test_fc_hybrid_reference_goldens(ops, oracle, ws, name):
    case = gv.HYBRID_FC[name]
    if case["per_channel_scales"] is None:
        w, scale = gv.symmetric_quantize(case["weights"])
        scales = np.asarray([scale], np.float32)
    else:
        scales = np.asarray(case["per_channel_scales"], np.float32)
        w = gv.per_channel_symmetric_quantize(case["weights"], scales)
    x = np.asarray(case["input"], np.float32)
    bias = np.asarray([1, 2, 3], np.float32)
    y = ops.fully_connected_hybrid(dev(x), ops.PackedInt8Weights(dev(w)), dev(scales), dev(bias), case["asymmetric"],
                                   ops.ACT_RELU, ws=ws).cpu().numpy()
    np.testing.assert_allclose(y.reshape(-1), case["expected"], atol=case["max_abs_err"], rtol=0)
    want = oracle.fc_hybrid(x, w, scales, bias, case["asymmetric"], oracle.ACT_RELU)
    assert np.array_equal(y, want)


@pytest.mark.parametrize("m", [1, 8, 64])
def test_fc_hybrid_config2(ops, oracle, ws, m):
    c = workloads.config2(m)
    wp = ops.PackedInt8Weights(dev(c["w"]))
    y = ops.fully_connected_hybrid(dev(c["x"]), wp, dev(c["filter_scales"]), ws=ws).cpu().numpy()
    orc_fast = oracle.fast()
    want = np.empty((m, 14336), np.float32)
    import ctypes

    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    orc_fast.orcf_fc_hybrid(m, 14336, 4096, p(c["x"]), p(c["w"]), p(c["filter_scales"]), 1, None, 1, 0, None, p(want))
    assert rel_err(y, want) <= 1e-3
    assert np.array_equal(y, want)  # same integer sums, same float operation order
    if m == 1:  # the scalar restatement itself, on a slice of the output channels
        ref = oracle.fc_hybrid(c["x"], c["w"][:512], c["filter_scales"][:512])
        assert np.array_equal(y[:, :512], ref)


def test_fc_hybrid_config2_m512(ops, oracle, ws):
    m = 512
    c = workloads.config2(m)
    wp = ops.PackedInt8Weights(dev(c["w"]))
    y = ops.fully_connected_hybrid(dev(c["x"]), wp, dev(c["filter_scales"]), ws=ws).cpu().numpy()
    # size-independent property at the full size: rows are independent, so any row equals the
    # single-row result; checked against the oracle on a sample of rows
    import ctypes

    rows = [0, 63, 64, 200, 511]
    xs = np.ascontiguousarray(c["x"][rows])
    want = np.empty((len(rows), 14336), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    oracle.fast().orcf_fc_hybrid(len(rows), 14336, 4096, p(xs), p(c["w"]), p(c["filter_scales"]), 1, None, 1, 0, None,
                                 p(want))
    assert np.array_equal(y[rows], want)


@pytest.mark.parametrize("m,n,k", [(1, 3, 10), (2, 130, 100), (9, 257, 333), (16, 128, 4096), (40, 77, 129),
                                   (70, 200, 64),
                                   (1, 2048, 16384), (3, 1536, 2048), (32, 2049, 1000), (64, 640, 260), (128, 1030, 520),
                                   (200, 19000, 200), (513, 18945, 96)])
@pytest.mark.parametrize("asymmetric,per_channel", [(True, True), (False, True), (True, False)])
def test_fc_hybrid_ragged_shapes(ops, oracle, ws, m, n, k, asymmetric, per_channel):
    rng = np.random.default_rng(m * 1000 + n + k)
    x = rng.standard_normal((m, k)).astype(np.float32)
    if m > 1:
        x[m // 2] = 0.0
    w = workloads.int8_weights(rng, n, k)
    scales = rng.uniform(1e-3, 1e-2, n if per_channel else 1).astype(np.float32)
    bias = rng.standard_normal(n).astype(np.float32) if (n % 2) else None
    act = (m + n) % 7
    y = ops.fully_connected_hybrid(dev(x), ops.PackedInt8Weights(dev(w)), dev(scales),
                                   None if bias is None else dev(bias), asymmetric, act, ws=ws).cpu().numpy()
    want = oracle.fc_hybrid(x, w, scales, bias, asymmetric, act)
    if act in (oracle.ACT_TANH, oracle.ACT_SIGMOID):
        np.testing.assert_allclose(y, want, rtol=1e-5, atol=1e-6)  # libm vs device transcendental
    else:
        assert np.array_equal(y, want)


def test_fc_hybrid_all_zero_input_returns_activated_bias(ops, oracle, ws):
    # tflite/kernels/fully_connected.cc:789-795
    w = workloads.int8_weights(np.random.default_rng(3), 40, 64)
    bias = np.linspace(-1, 1, 40).astype(np.float32)
    x = np.zeros((3, 64), np.float32)
    y = ops.fully_connected_hybrid(dev(x), ops.PackedInt8Weights(dev(w)), dev(np.asarray([0.01], np.float32)),
                                   dev(bias), True, ops.ACT_RELU, ws=ws).cpu().numpy()
    assert np.array_equal(y, np.maximum(np.tile(bias, (3, 1)), 0))


# --------------------------------------------------------------------------- blockwise int4
@pytest.mark.parametrize("m", [1, 8])
def test_fc_w4_config3(ops, oracle, ws, m):
    c = workloads.config3(m)
    wp = ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), c["blocksize"])
    y = ops.fully_connected_blockwise4(dev(c["x"]), wp, ws=ws).cpu().numpy()
    n_check = 16384 if m == 1 else 2048
    want = oracle.fc_blockwise4(c["x"], c["w4"][:n_check], c["scales"][:n_check], c["blocksize"])
    assert rel_err(y[:, :n_check], want) <= 1e-3
    # up to 8 rows the block sums are exact integers, as in the reference; only the order of the float additions differs
    assert rel_err(y[:, :n_check], want) <= 2e-6


@pytest.mark.parametrize("m,n,k", [(1, 130, 96), (2, 257, 320), (2, 1024, 4096), (5, 300, 2048), (8, 512, 1024), (3, 16384, 256)])
def test_fc_w4_decode_sized_batches_have_exact_block_sums(ops, oracle, ws, m, n, k):
    c = workloads.config3(m, n, k, seed=7 * m + n + k)
    x = (c["x"] + 1.5).astype(np.float32)
    bias = np.random.default_rng(3).standard_normal(n).astype(np.float32)
    wp = ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), 32)
    y = ops.fully_connected_blockwise4(dev(x), wp, dev(bias), ws=ws).cpu().numpy()
    assert rel_err(y, oracle.fc_blockwise4(x, c["w4"], c["scales"], 32, bias)) <= 2e-6


def test_fc_w4_config3_m512(ops, oracle, ws):
    import ctypes

    c = workloads.config3(512)
    wp = ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), c["blocksize"])
    y = ops.fully_connected_blockwise4(dev(c["x"]), wp, ws=ws).cpu().numpy()
    want = np.empty((512, 16384), np.float32)
    p = lambda a: a.ctypes.data_as(ctypes.c_void_p)
    oracle.fast().orcf_fc_blockwise4(512, 16384, 2048, 32, p(c["x"]), p(c["w4"]), p(c["scales"].view(np.uint16)), None,
                                     p(want))
    assert rel_err(y, want) <= 1e-3


@pytest.mark.parametrize("m,n,k", [(1, 4, 32), (3, 130, 96), (9, 257, 320), (20, 64, 2048)])
def test_fc_w4_ragged_shapes(ops, oracle, ws, m, n, k):
    c = workloads.config3(m, n, k, seed=m + n + k)
    bias = np.random.default_rng(1).standard_normal(n).astype(np.float32)
    wp = ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), 32)
    assert np.array_equal(wp.kfsum.cpu().numpy(),
                          _kfsum(c["w"], c["scales"]))  # zero-point term: same order as the reference, bit-equal
    y = ops.fully_connected_blockwise4(dev(c["x"]), wp, dev(bias), ws=ws).cpu().numpy()
    want = oracle.fc_blockwise4(c["x"], c["w4"], c["scales"], 32, bias)
    np.testing.assert_allclose(y, want, rtol=1e-3, atol=1e-3 * np.abs(want).max())


@pytest.mark.parametrize("m,n,k,blocksize", [(4, 256, 4096, 32), (40, 384, 1024, 64), (100, 200, 512, 128),
                                             (300, 256, 768, 256), (16, 1024, 2048, 2048), (513, 130, 320, 32)])
def test_fc_w4_row_passes_block_sizes_and_split_reductions(ops, oracle, ws, m, n, k, blocksize):
    """Every rows-per-pass variant (16 .. 256 and several passes), block sizes beyond 32 (one scale per
    block, whatever its length), and shapes with so few output tiles that the reduction is cut across
    SMs and merged through the scratch slots; inputs far from zero, so that the zero-point term counts."""
    c = workloads.config3(m, n, k, blocksize=blocksize, seed=m + n + k)
    x = (c["x"] * 0.25 + 3.0).astype(np.float32)
    bias = np.random.default_rng(2).standard_normal(n).astype(np.float32)
    wp = ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), blocksize)
    y = ops.fully_connected_blockwise4(dev(x), wp, dev(bias), ws=ws).cpu().numpy()
    y2 = ops.fully_connected_blockwise4(dev(x), wp, dev(bias), ws=ws).cpu().numpy()
    assert np.array_equal(y, y2)  # the merge order is fixed: no run-to-run differences
    want = oracle.fc_blockwise4(x, c["w4"], c["scales"], blocksize, bias)
    assert rel_err(y, want) <= 1e-3


def _kfsum(w, scales_f16):
    n, k = w.shape
    nb = scales_f16.shape[1]
    ksum = w.reshape(n, nb, k // nb).astype(np.int32).sum(-1)
    acc = np.zeros(n, np.float32)
    sc = scales_f16.astype(np.float32)
    for b in range(nb):
        acc = acc + sc[:, b] * ksum[:, b].astype(np.float32)
    return acc


def test_fc_w4_reference_int4_goldens(ops, ws):
    """The reference's 4-bit goldens need one 40-wide block per row; blocks are 32-wide here, so
    the same numbers are reached by zero-padding k to 64 with two unit-scale blocks."""
    w = np.zeros((5, 64), np.int8)
    w[:, :40] = np.asarray(gv.HYBRID_INT4_WEIGHTS, np.int8)
    x = np.zeros((4, 64), np.float32)
    x[:, :40] = np.asarray(gv.HYBRID_INT4_INPUT_ZERO_ROW, np.float32)
    u = w.astype(np.uint8) & 0xF
    w4 = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    wp = ops.PackedInt4Weights(dev(w4), dev(np.ones((5, 2), np.float16)), 32)
    y = ops.fully_connected_blockwise4(dev(x), wp, dev(np.asarray(gv.HYBRID_INT4_BIAS, np.float32)), ws=ws)
    np.testing.assert_allclose(np.maximum(y.cpu().numpy(), 0).reshape(-1), gv.HYBRID_INT4_EXPECTED_ZERO_ROW,
                               atol=gv.HYBRID_INT4_MAX_ABS_ERR, rtol=0)


# --------------------------------------------------------------------------- SDPA decode
def _sdpa_oracle(oracle, q, k, v, lengths, scale, k_scale=None, v_scale=None, mask=None, logit_cap=0.0):
    qf, kf, vf = q.astype(np.float32), k.astype(np.float32), v.astype(np.float32)
    if k_scale is not None:
        kf = kf * k_scale[..., None]
        vf = vf * v_scale[..., None]
    b, _, n, h = q.shape
    out = np.empty((b, 1, n, h), np.float32)
    for i in range(b):
        L = int(lengths[i]) if lengths is not None else k.shape[1]
        mk = None if mask is None else mask[i:i + 1, :, :, :L]
        out[i] = oracle.sdpa_f32(qf[i:i + 1], kf[i:i + 1, :L], vf[i:i + 1, :L], mk, scale, logit_cap)[0]
    return out


@pytest.mark.parametrize("kv", ["f16", "i8"])
def test_sdpa_config4(ops, oracle, ws, kv):
    c = workloads.config4(b=16, s_max=2048, min_len=1)  # oracle-sized: same heads and head dim, shorter cache
    c["lengths"][0] = 1
    c["lengths"][1] = 2048
    c["lengths"][2] = 513
    ksc = vsc = None
    k, v = c["k"], c["v"]
    if kv == "i8":
        k, ksc = workloads.quantize_kv_per_token(c["k"])
        v, vsc = workloads.quantize_kv_per_token(c["v"])
    out = ops.sdpa_decode(dev(c["q"]), dev(k), dev(v), dev(c["lengths"]), scale=c["scale"],
                          k_scale=None if ksc is None else dev(ksc), v_scale=None if vsc is None else dev(vsc), ws=ws)
    want = _sdpa_oracle(oracle, c["q"], k, v, c["lengths"], c["scale"], ksc, vsc)
    assert rel_err(out.float().cpu().numpy(), want) <= 2e-2


@pytest.mark.parametrize("kv", ["f16", "i8"])
def test_sdpa_config4_at_its_stated_size_against_the_oracle(ops, oracle, ws, kv):
    """16 sequences, ragged lengths uniform in [128, 8192], 8 query heads on one KV head of 256: every
    sequence against the float32 restatement on the up-converted cache."""
    c = workloads.config4()
    assert c["k"].shape == (16, 8192, 1, 256) and c["lengths"].min() >= 128
    ksc = vsc = None
    k, v = c["k"], c["v"]
    if kv == "i8":
        k, ksc = workloads.quantize_kv_per_token(c["k"])
        v, vsc = workloads.quantize_kv_per_token(c["v"])
    out = ops.sdpa_decode(dev(c["q"]), dev(k), dev(v), dev(c["lengths"]), scale=c["scale"],
                          k_scale=None if ksc is None else dev(ksc), v_scale=None if vsc is None else dev(vsc), ws=ws)
    want = _sdpa_oracle(oracle, c["q"], k, v, c["lengths"], c["scale"], ksc, vsc)
    got = out.float().cpu().numpy()
    worst = max(rel_err(got[i], want[i]) for i in range(16))
    print(f"config 4 ({kv} cache), {int(c['lengths'].sum())} cached tokens: worst sequence {worst:.3e}")
    assert worst <= 2e-2


def test_sdpa_empty_and_out_of_range_lengths(ops, oracle, ws):
    """A batch slot with no cached tokens is a normal serving state: its output is zeros, not NaN, and a
    length beyond the cache is read as the whole cache."""
    c = workloads.config4(b=4, s_max=512, min_len=5)
    L = c["lengths"].copy()
    L[1] = 0
    L[2] = -3
    L[3] = 9999
    out = ops.sdpa_decode(dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(L), scale=c["scale"], ws=ws).float().cpu().numpy()
    assert np.all(out[1] == 0) and np.all(out[2] == 0)
    Lc = np.clip(L, 0, 512)
    want = _sdpa_oracle(oracle, c["q"][[0, 3]], c["k"][[0, 3]], c["v"][[0, 3]], Lc[[0, 3]], c["scale"])
    assert rel_err(out[[0, 3]], want) <= 2e-2


def test_sdpa_config4_full_size_properties(ops, ws):
    """Full-size ragged batch: each sequence must equal the same sequence run alone, and a
    sequence with its cache doubled by repetition must give the same output."""
    c = workloads.config4()
    q, k, v, L = dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(c["lengths"])
    out = ops.sdpa_decode(q, k, v, L, scale=c["scale"], ws=ws)
    assert torch.isfinite(out.float()).all()
    for i in (0, 7, 15):
        alone = ops.sdpa_decode(q[i:i + 1], k[i:i + 1], v[i:i + 1], L[i:i + 1], scale=c["scale"], ws=ws)
        # the split of a sequence into chunks depends on the batch, so the sums associate differently
        torch.testing.assert_close(alone.float(), out[i:i + 1].float(), rtol=4e-3, atol=2e-4)
    i = int(np.argmin(c["lengths"]))
    n0 = int(c["lengths"][i])
    if 2 * n0 <= 8192:
        k2, v2 = k[i:i + 1].clone(), v[i:i + 1].clone()
        k2[:, n0:2 * n0] = k2[:, :n0]
        v2[:, n0:2 * n0] = v2[:, :n0]
        twice = ops.sdpa_decode(q[i:i + 1], k2, v2, dev(np.asarray([2 * n0], np.int32)), scale=c["scale"], ws=ws)
        assert rel_err(twice.float().cpu().numpy(), out[i:i + 1].float().cpu().numpy()) <= 2e-2


@pytest.mark.parametrize("n,nkv,h", [(8, 8, 64), (8, 2, 128), (4, 1, 256), (32, 4, 256), (6, 3, 64)])
def test_sdpa_group_shapes(ops, oracle, ws, n, nkv, h):
    c = workloads.config4(b=3, n=n, nkv=nkv, h=h, s_max=300, min_len=1, seed=n * 100 + h)
    out = ops.sdpa_decode(dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(c["lengths"]), ws=ws)  # default scale
    want = _sdpa_oracle(oracle, c["q"], c["k"], c["v"], c["lengths"], None)
    assert rel_err(out.float().cpu().numpy(), want) <= 2e-2


@pytest.mark.parametrize("name", sorted(gv.SDPA_SHAPES))
def test_sdpa_reference_test_shapes_f32_with_mask(ops, oracle, ws, name):
    """The reference's own differential-test shapes (fp32 tensors, additive mask, head size 4)."""
    p = gv.SDPA_SHAPES[name]
    rng = np.random.default_rng(9)
    q = rng.uniform(0, 1, (p["b"], p["t"], p["n"], p["h"])).astype(np.float32)
    k = rng.uniform(0, 1, (p["b"], p["s"], p["nkv"], p["h"])).astype(np.float32)
    v = rng.uniform(0, 1, (p["b"], p["s"], p["nkv"], p["h"])).astype(np.float32)
    mask = rng.uniform(0, 1, (p["b"], 1, p["t"], p["s"])).astype(np.float32)
    out = ops.sdpa_decode(dev(q), dev(k), dev(v), None, dev(mask), ws=ws).cpu().numpy()
    want = oracle.sdpa_f32(q, k, v, mask)
    np.testing.assert_allclose(out, want, rtol=1e-4, atol=1e-5)


def test_sdpa_f32_cache_mask_and_logit_cap_fast_path(ops, oracle, ws):
    rng = np.random.default_rng(10)
    b, n, nkv, h, s = 2, 8, 1, 256, 700
    q = rng.standard_normal((b, 1, n, h)).astype(np.float32)
    k = rng.standard_normal((b, s, nkv, h)).astype(np.float32)
    v = rng.standard_normal((b, s, nkv, h)).astype(np.float32)
    mask = np.where(np.arange(s)[None, None, None, :] < np.asarray([650, 33])[:, None, None, None], 0.0,
                    -1e30).astype(np.float32)
    out = ops.sdpa_decode(dev(q), dev(k), dev(v), None, dev(mask), logit_cap=30.0, ws=ws).cpu().numpy()
    want = oracle.sdpa_f32(q, k, v, mask, None, 30.0)
    assert rel_err(out, want) <= 2e-2


@pytest.mark.parametrize("n,nkv,h", [(8, 1, 256), (8, 1, 128), (4, 2, 64), (3, 1, 256), (16, 2, 128)])
@pytest.mark.parametrize("kv", ["f16", "i8", "f32"])
def test_sdpa_rows_causal_prompt(ops, oracle, n, nkv, h, kv):
    """Several query tokens of one sequence (the prompt pass): row r attends over the cached tokens up to
    its own position, start + r. 301 rows behind 37 cached tokens: a last CTA with one row, chunks that
    end inside a 64-token stage, rows whose limit falls inside the CTA's first stage."""
    rng = np.random.default_rng(n * 1000 + h + nkv)
    rows, start, s_max = 301, 37, 400
    q = rng.standard_normal((rows, n, h)).astype(np.float16)
    k = rng.standard_normal((s_max, nkv, h)).astype(np.float16)
    v = rng.standard_normal((s_max, nkv, h)).astype(np.float16)
    lengths = (start + 1 + np.arange(rows)).astype(np.int32)
    scale = 1.0 / np.sqrt(h)
    ksc = vsc = None
    kd, vd = k, v
    if kv == "i8":
        kd, ksc = workloads.quantize_kv_per_token(k[None])
        vd, vsc = workloads.quantize_kv_per_token(v[None])
        kd, vd, ksc, vsc = kd[0], vd[0], ksc[0], vsc[0]
    elif kv == "f32":
        kd, vd = k.astype(np.float32), v.astype(np.float32)
    out = ops.sdpa_rows(dev(q), dev(kd), dev(vd), dev(lengths), scale=scale,
                        k_scale=None if ksc is None else dev(ksc), v_scale=None if vsc is None else dev(vsc))
    kf = kd.astype(np.float32) if ksc is None else kd.astype(np.float32) * ksc[..., None]
    vf = vd.astype(np.float32) if vsc is None else vd.astype(np.float32) * vsc[..., None]
    got = out.float().cpu().numpy()
    for r in list(range(0, rows, 7)) + [rows - 1]:
        L = int(lengths[r])
        want = oracle.sdpa_f32(q[r][None, None].astype(np.float32), kf[None, :L], vf[None, :L], None, scale)[0, 0]
        assert rel_err(got[r], want) <= 2e-2, r
