"""numpy front end of the CPU oracle (liboracle.so, built by oracle/Makefile).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the
CPU-baseline leg of the benchmark. The shipped package never imports it.
Each function forwards to the C restatement in oracle.c, which cites the
reference file and lines it follows.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

ACT_NONE, ACT_RELU, ACT_RELU_N1_TO_1, ACT_RELU6, ACT_TANH, ACT_SIGN_BIT, ACT_SIGMOID = range(7)
REQUANT_MBQM, REQUANT_FLOAT_REF = 0, 1


def build(force=False):
    """Compile liboracle.so / liboracle_fast.so (and oracle/_ref when the reference tree exists)."""
    targets = ["liboracle.so", "liboracle_fast.so"]
    sources = [f for f in os.listdir(_HERE) if f.endswith((".c", ".h"))]
    newest = max(os.path.getmtime(os.path.join(_HERE, f)) for f in sources)
    stale = not all(os.path.exists(os.path.join(_HERE, t)) and os.path.getmtime(os.path.join(_HERE, t)) >= newest
                    for t in targets)
    if force or stale:
        subprocess.check_call(["make", "-C", _HERE, "-s", "liboracle.so", "liboracle_fast.so"])
    # the LiteRT checkout: $LITERT_ROOT, else a directory `reference` beside this repository
    ref_root = os.environ.get("LITERT_ROOT") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if os.path.isdir(os.path.join(ref_root, "tflite")) and (
        force or not os.path.exists(os.path.join(_HERE, "_ref", "libref_quant.so"))
    ):
        subprocess.check_call(["make", "-C", _HERE, "-s", "ref", "REF=" + ref_root])


_lib = None
_fast = None


def lib():
    global _lib
    if _lib is None:
        path = os.path.join(_HERE, "liboracle.so")
        if not os.path.exists(path):
            build()
        _lib = ctypes.CDLL(path)
        _lib.orc_multiply_by_quantized_multiplier.restype = ctypes.c_int32
        _lib.orc_multiply_by_quantized_multiplier_i64.restype = ctypes.c_int32
        _lib.orc_saturating_rounding_doubling_high_mul.restype = ctypes.c_int32
        _lib.orc_rounding_divide_by_pot.restype = ctypes.c_int32
        _lib.orc_half_to_float.restype = ctypes.c_float
        _lib.orc_float_to_half.restype = ctypes.c_uint16
    return _lib


def fast():
    """The vectorised / multi-threaded twin used only for CPU-baseline timing."""
    global _fast
    if _fast is None:
        path = os.path.join(_HERE, "liboracle_fast.so")
        if not os.path.exists(path):
            build()
        _fast = ctypes.CDLL(path)
        _fast.orcf_num_threads.restype = ctypes.c_int
    return _fast


def ref_lib():
    """Reference sources compiled as they are (oracle/_ref); None when not built."""
    path = os.path.join(_HERE, "_ref", "libref_quant.so")
    return ctypes.CDLL(path) if os.path.exists(path) else None


def _p(a):
    return None if a is None else a.ctypes.data_as(ctypes.c_void_p)


def _c(a, dtype):
    return None if a is None else np.ascontiguousarray(a, dtype=dtype)


_f = ctypes.c_float
_d = ctypes.c_double
_i = ctypes.c_int
_i32 = ctypes.c_int32


# ---- requantization -------------------------------------------------------
def quantize_multiplier(m):
    q, s = _i32(), _i()
    lib().orc_quantize_multiplier(_d(m), ctypes.byref(q), ctypes.byref(s))
    return q.value, s.value


def multiply_by_quantized_multiplier(x, mult, shift):
    return lib().orc_multiply_by_quantized_multiplier(_i32(x), _i32(mult), _i(shift))


def multiply_by_quantized_multiplier_i64(x, mult, shift):
    return lib().orc_multiply_by_quantized_multiplier_i64(ctypes.c_int64(x), _i32(mult), _i(shift))


def activation_range_int8(activation, out_scale, out_zp):
    lo, hi = _i32(), _i32()
    rc = lib().orc_activation_range_int8(_i(activation), _f(out_scale), _i32(out_zp), ctypes.byref(lo), ctypes.byref(hi))
    if rc:
        raise ValueError("activation range overflow")
    return lo.value, hi.value


def fc_per_channel_multipliers(input_scale, output_scale, filter_scales):
    fs = _c(filter_scales, np.float32)
    n = fs.size
    mult = np.empty(n, np.int32)
    shift = np.empty(n, np.int32)
    lib().orc_fc_per_channel_multipliers(_f(input_scale), _f(output_scale), _p(fs), _i(n), _p(mult), _p(shift))
    return mult, shift


def fc_per_tensor_multiplier(input_scale, filter_scale, bias_scale, output_scale):
    q, s = _i32(), _i()
    rc = lib().orc_fc_per_tensor_multiplier(
        _f(input_scale), _f(filter_scale), _i(0 if bias_scale is None else 1),
        _f(0.0 if bias_scale is None else bias_scale), _f(output_scale), ctypes.byref(q), ctypes.byref(s))
    if rc:
        raise ValueError("bias scale check failed")
    return q.value, s.value


# ---- full-integer FC ------------------------------------------------------
def fc_int8_per_channel(x, w, bias, input_zp, input_scale, filter_scales, output_scale, output_zp,
                        activation=ACT_NONE, requant=REQUANT_MBQM):
    x = _c(x, np.int8)
    w = _c(w, np.int8)
    n, k = w.shape
    m = x.size // k
    bias = _c(bias, np.int32)
    fs = _c(filter_scales, np.float32)
    mult, shift = fc_per_channel_multipliers(input_scale, output_scale, fs)
    lo, hi = activation_range_int8(activation, output_scale, output_zp)
    y = np.empty((m, n), np.int8)
    lib().orc_fc_int8_per_channel(_i(requant), _i(m), _i(n), _i(k), _p(x), _p(w), _p(bias), _i32(-input_zp),
                                  _i32(output_zp), _p(mult), _p(shift), _f(input_scale), _f(output_scale),
                                  _p(fs), _i32(lo), _i32(hi), _p(y))
    return y


def fc_int8_per_tensor(x, w, bias, input_zp, input_scale, filter_zp, filter_scale, output_scale, output_zp,
                       activation=ACT_NONE, bias_scale=None):
    x = _c(x, np.int8)
    w = _c(w, np.int8)
    n, k = w.shape
    m = x.size // k
    bias = _c(bias, np.int32)
    if bias is not None and bias_scale is None:
        bias_scale = np.float32(input_scale) * np.float32(filter_scale)
    mult, shift = fc_per_tensor_multiplier(input_scale, filter_scale, bias_scale if bias is not None else None,
                                           output_scale)
    lo, hi = activation_range_int8(activation, output_scale, output_zp)
    y = np.empty((m, n), np.int8)
    lib().orc_fc_int8_per_tensor(_i(m), _i(n), _i(k), _p(x), _p(w), _p(bias), _i32(-input_zp), _i32(-filter_zp),
                                 _i32(output_zp), _i32(mult), _i(shift), _i32(lo), _i32(hi), _p(y))
    return y


# ---- hybrid ---------------------------------------------------------------
def batch_quantize_floats(x, asymmetric=True):
    x = _c(x, np.float32)
    m, k = x.shape
    q = np.empty((m, k), np.int8)
    scales = np.empty(m, np.float32)
    zps = np.zeros(m, np.int32)
    lib().orc_batch_quantize_floats(_p(x), _i(m), _i(k), _p(q), _p(scales), _p(zps), _i(1 if asymmetric else 0))
    return q, scales, zps


def fc_hybrid(x, w, filter_scales, bias=None, asymmetric_inputs=True, activation=ACT_NONE):
    w = _c(w, np.int8)
    n, k = w.shape
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    fs = np.atleast_1d(_c(filter_scales, np.float32))
    per_channel = 1 if fs.size > 1 else 0
    bias = _c(bias, np.float32)
    y = np.empty((m, n), np.float32)
    lib().orc_fc_hybrid(_i(m), _i(n), _i(k), _p(x), _p(w), _p(fs), _i(per_channel), _p(bias),
                        _i(1 if asymmetric_inputs else 0), _i(activation), _p(y))
    return y


def fc_blockwise4(x, w4, scales_f16, blocksize, bias=None):
    """w4: uint8 [n, ceil(k/2)] packed low nibble first; scales_f16: float16 [n, k/blocksize]."""
    w4 = _c(w4, np.uint8)
    sc = np.ascontiguousarray(scales_f16, dtype=np.float16)
    n = w4.shape[0]
    k = sc.shape[1] * blocksize
    x = _c(x, np.float32).reshape(-1, k)
    m = x.shape[0]
    bias = _c(bias, np.float32)
    y = np.empty((m, n), np.float32)
    lib().orc_fc_blockwise4(_i(m), _i(n), _i(k), _i(blocksize), _p(x), _p(w4), _p(sc.view(np.uint16)), _p(bias),
                            _p(y))
    return y


def unpack_int4(w4, num_elements):
    w4 = _c(w4, np.uint8)
    out = np.empty(num_elements, np.int8)
    lib().orc_unpack_int4(_p(w4), _i(num_elements), _p(out))
    return out


def pack_int4(values):
    """int8 values in [-8,7], last dim even -> uint8 packed, element 2i in the low nibble."""
    v = np.asarray(values, np.int8)
    assert v.shape[-1] % 2 == 0
    u = (v.astype(np.uint8) & 0xF)
    return (u[..., 0::2] | (u[..., 1::2] << 4)).astype(np.uint8)


# ---- BATCH_MATMUL ---------------------------------------------------------
def _dims(a):
    return (ctypes.c_int * a.ndim)(*a.shape)


def _bmm_out_shape(x, y, adj_x, adj_y):
    xs, ys = list(x.shape), list(y.shape)
    a = xs[-1] if adj_x else xs[-2]
    c = ys[-2] if adj_y else ys[-1]
    rank = max(len(xs), len(ys))
    xb = [1] * (rank - len(xs)) + xs[:-2]
    yb = [1] * (rank - len(ys)) + ys[:-2]
    batch = [max(p, q) for p, q in zip(xb, yb)]
    return tuple(batch + [a, c])


def batch_matmul_float(x, y, adj_x=False, adj_y=False):
    x = _c(x, np.float32)
    y = _c(y, np.float32)
    out = np.empty(_bmm_out_shape(x, y, adj_x, adj_y), np.float32)
    lib().orc_batch_matmul_float(_i(x.ndim), _dims(x), _p(x), _i(y.ndim), _dims(y), _p(y), _i(adj_x), _i(adj_y),
                                 _p(out))
    return out


def batch_matmul_hybrid(x, y, y_scale, adj_x=False, adj_y=False, asymmetric_inputs=True, per_channel_scales=None):
    """per_channel_scales: one scale per output column (replaces y_scale)."""
    x = _c(x, np.float32)
    y = _c(y, np.int8)
    pc = _c(per_channel_scales, np.float32)
    out = np.empty(_bmm_out_shape(x, y, adj_x, adj_y), np.float32)
    lib().orc_batch_matmul_hybrid_pc(_i(x.ndim), _dims(x), _p(x), _i(y.ndim), _dims(y), _p(y), _f(y_scale or 0.0),
                                     _p(pc), _i(adj_x), _i(adj_y), _i(1 if asymmetric_inputs else 0), _p(out))
    return out


def batch_matmul_int8(x, x_zp, x_scale, y, y_zp, y_scale, out_scale, out_zp, adj_x=False, adj_y=False):
    x = _c(x, np.int8)
    y = _c(y, np.int8)
    # tflite/kernels/batch_matmul.cc:315-321: multiplier from the float product of the two scales.
    mult, shift = fc_per_tensor_multiplier(x_scale, y_scale, None, out_scale)
    out = np.empty(_bmm_out_shape(x, y, adj_x, adj_y), np.int8)
    lib().orc_batch_matmul_int8(_i(x.ndim), _dims(x), _p(x), _i32(x_zp), _i(y.ndim), _dims(y), _p(y), _i32(y_zp),
                                _i(adj_x), _i(adj_y), _i32(mult), _i(shift), _i32(out_zp), _p(out))
    return out


# ---- SDPA -----------------------------------------------------------------
def sdpa_f32(q, k, v, mask=None, scale=None, logit_cap=0.0):
    q = _c(q, np.float32)
    k = _c(k, np.float32)
    v = _c(v, np.float32)
    b, t, n, h = q.shape
    s, nkv = k.shape[1], k.shape[2]
    if scale is None or scale <= 0:
        scale = 1.0 / np.sqrt(np.float32(h))  # tflite/experimental/genai/sdpa.cc:99-105
    mask = _c(mask, np.float32)
    out = np.empty_like(q)
    lib().orc_sdpa_f32(_i(b), _i(t), _i(n), _i(nkv), _i(h), _i(s), _p(q), _p(k), _p(v), _p(mask),
                       _f(scale), _f(logit_cap), _p(out))
    return out


# ---- stages of the decoder graph, one function each (oracle/decoder_ref.c) -----------------
def stage_embed(tokens, table, row_scales, embed_scale):
    tok = _c(tokens, np.int32)
    table = _c(table, np.int8)
    rs = _c(row_scales, np.float32)
    d = table.shape[1]
    h = np.empty((tok.size, d), np.float32)
    fast().orc_stage_embed(_p(tok), _i(tok.size), _p(table), _p(rs), _i(d), _f(embed_scale), _p(h))
    return h


def stage_add_rmsnorm(h, delta, gain, eps):
    """Returns (h + delta, rms_norm(h + delta) * gain); delta may be None."""
    h = np.array(h, np.float32, copy=True, order="C")
    delta = _c(delta, np.float32)
    gain = _c(gain, np.float32)
    rows, d = h.shape
    x = np.empty_like(h)
    fast().orc_stage_add_rmsnorm(_p(h), _p(delta), _p(gain), _i(rows), _i(d), _f(eps), _p(x))
    return h, x


def rope_table(max_seq, head_dim, base=10000.0):
    """float32 [max_seq, head_dim / 2, 2] = (cos, sin) of the rotation angles."""
    cs = np.empty((max_seq, head_dim // 2, 2), np.float32)
    fast().orc_rope_table(_i(max_seq), _i(head_dim), _f(base), _p(cs))
    return cs


def stage_rope(x, positions, base=10000.0):
    """x [rows, heads, head_dim] rotated (copy), row r at positions[r]."""
    x = np.array(x, np.float32, copy=True, order="C")
    pos = _c(positions, np.int32)
    rows, heads, hd = x.shape
    fast().orc_stage_rope(_p(x), _i(rows), _i(heads), _i(hd), _p(pos), _f(base))
    return x


def stage_kv_round(rows, mode):
    """Cache rows [..., head_dim] as the device keeps them (1: binary16, 2: int8 per row), as float32."""
    x = np.array(rows, np.float32, copy=True, order="C")
    hd = x.shape[-1]
    flat = x.reshape(-1, hd)
    for r in range(flat.shape[0]):
        fast().orc_stage_kv_round(flat[r].ctypes.data_as(ctypes.c_void_p), _i(hd), _i(mode))
    return x


def stage_geglu(gate, up):
    gate = _c(gate, np.float32)
    up = _c(up, np.float32)
    out = np.empty_like(gate)
    fast().orc_stage_geglu(_p(gate), _p(up), ctypes.c_size_t(gate.size), _p(out))
    return out


def stage_softcap(logits, cap):
    x = np.array(logits, np.float32, copy=True, order="C")
    fast().orc_stage_softcap(_p(x), ctypes.c_size_t(x.size), _f(cap))
    return x


def stage_argmax(logits):
    lg = _c(logits, np.float32)
    rows, n = lg.shape
    out = np.empty(rows, np.int32)
    fast().orc_stage_argmax(_p(lg), _i(rows), _i(n), _p(out))
    return out


# ---- Gemma-shaped decoder (oracle/decoder_ref.c) ------------------------------------------
class _DecCfg(ctypes.Structure):
    _fields_ = [(n, ctypes.c_int) for n in ("n_layers", "d_model", "n_heads", "n_kv_heads", "head_dim", "d_ff",
                                            "vocab", "max_seq")] + \
               [(n, ctypes.c_float) for n in ("rms_eps", "rope_base", "embed_scale")]


class _DecLayer(ctypes.Structure):
    _fields_ = [(n, ctypes.c_void_p) for n in ("wq", "wk", "wv", "wo", "wgate", "wup", "wdown", "sq", "sk", "sv", "so",
                                               "sgate", "sup", "sdown", "norm1", "norm2")]


_REDUCE_FN = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.POINTER(ctypes.c_float), ctypes.c_size_t)


def shard_decoder(cfg, weights, tp_size, rank):
    """Tensor-parallel shard `rank` of `tp_size`: (shard cfg, shard weights, (first LM row, LM rows)).
    Query heads, feed-forward units and LM-head rows are split evenly; q/gate/up are cut by output
    rows, o/down by input columns; a KV head shared by several ranks is replicated on each."""
    H, KVH, HD, F, V = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"], cfg["vocab"]
    assert H % tp_size == 0 and F % tp_size == 0 and V % tp_size == 0
    hl, fl = H // tp_size, F // tp_size
    if KVH % tp_size == 0:
        kvl = KVH // tp_size
        kv0 = rank * kvl
    else:
        assert tp_size % KVH == 0
        kvl = 1
        kv0 = rank // (tp_size // KVH)
    q0, q1 = rank * hl * HD, (rank + 1) * hl * HD
    k0, k1 = kv0 * HD, (kv0 + kvl) * HD
    f0, f1 = rank * fl, (rank + 1) * fl
    layers = []
    for lw in weights["layers"]:
        layers.append(dict(
            wq=lw["wq"][q0:q1], sq=lw["sq"][q0:q1], wk=lw["wk"][k0:k1], sk=lw["sk"][k0:k1],
            wv=lw["wv"][k0:k1], sv=lw["sv"][k0:k1], wo=lw["wo"][:, q0:q1], so=lw["so"],
            wgate=lw["wgate"][f0:f1], sgate=lw["sgate"][f0:f1], wup=lw["wup"][f0:f1], sup=lw["sup"][f0:f1],
            wdown=lw["wdown"][:, f0:f1], sdown=lw["sdown"], norm1=lw["norm1"], norm2=lw["norm2"]))
    scfg = dict(cfg, n_heads=hl, n_kv_heads=kvl, d_ff=fl)
    sw = dict(layers=layers, embed=weights["embed"], embed_scales=weights["embed_scales"],
              final_norm=weights["final_norm"])
    return scfg, sw, (rank * (V // tp_size), V // tp_size)


class DecoderRef:
    """CPU decode steps over numpy weights (dict of layers / embed / embed_scales / final_norm with
    the key names of _DecLayer). fast=True uses the vectorised multi-threaded kernels."""

    def __init__(self, cfg, weights, batch, max_seq, rms_eps=1e-6, rope_base=10000.0, fast=False, reduce=None,
                 lm_rows=None, kv_mode=0):
        """reduce(arr): sums a float32 array over tensor-parallel ranks in place (shard decoders only);
        lm_rows=(first, rows) limits the LM head to those rows of the table."""
        use_fast = bool(fast)
        self.lib = fast_lib = globals()["fast"]()
        self.cfg = cfg
        self.batch = batch
        c = _DecCfg(cfg["n_layers"], cfg["d_model"], cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"],
                    cfg["vocab"], max_seq, rms_eps, rope_base, float(np.sqrt(np.float32(cfg["d_model"]))))
        fast_lib.orc_decoder_create.restype = ctypes.c_void_p
        self.h = ctypes.c_void_p(fast_lib.orc_decoder_create(ctypes.byref(c), batch, 1 if use_fast else 0))
        self._keep = []
        for i, lw in enumerate(weights["layers"]):
            st = _DecLayer()
            for k in lw:
                arr = np.ascontiguousarray(lw[k], np.int8 if k.startswith("w") else np.float32)
                self._keep.append(arr)
                setattr(st, k, arr.ctypes.data)
            fast_lib.orc_decoder_set_layer(self.h, i, ctypes.byref(st))
        e = np.ascontiguousarray(weights["embed"], np.int8)
        es = np.ascontiguousarray(weights["embed_scales"], np.float32)
        fn = np.ascontiguousarray(weights["final_norm"], np.float32)
        self._keep += [e, es, fn]
        fast_lib.orc_decoder_set_embedding(self.h, _p(e), _p(es), _p(fn))
        if kv_mode:  # keep cache rows as the device does: 1 binary16, 2 int8 per token
            fast_lib.orc_decoder_set_kv_mode(self.h, int(kv_mode))
        self.lm_rows = cfg["vocab"]
        if lm_rows is not None:
            self.lm_rows = int(lm_rows[1])
            fast_lib.orc_decoder_set_lm_rows(self.h, int(lm_rows[0]), int(lm_rows[1]))
        self._reduce_cb = None
        if reduce is not None:
            def _cb(_user, buf, count):
                arr = np.ctypeslib.as_array(buf, shape=(count,))
                reduce(arr)
            self._reduce_cb = _REDUCE_FN(_cb)
            fast_lib.orc_decoder_set_reduce(self.h, self._reduce_cb, None)

    def reset(self):
        self.lib.orc_decoder_reset(self.h)

    def set_lengths(self, lengths):
        """Declares that many tokens already cached per sequence (the cache rows keep what they hold)."""
        L = np.ascontiguousarray(lengths, np.int32)
        assert L.size == self.batch
        self.lib.orc_decoder_set_lengths(self.h, _p(L))

    def step(self, tokens, want_logits=True):
        tok = np.ascontiguousarray(tokens, np.int32)
        logits = np.empty((self.batch, self.lm_rows), np.float32) if want_logits else None
        nxt = np.empty(self.batch, np.int32)
        self.lib.orc_decoder_step(self.h, _p(tok), _p(logits), _p(nxt))
        return nxt, logits

    def close(self):
        if self.h:
            self.lib.orc_decoder_destroy(self.h)
            self.h = None


class DecoderRefTP:
    """tp_size shard decoders stepped side by side on CPU threads (scalar kernels); the partial
    outputs of the input-sharded projections are summed in rank order. step() returns the next
    tokens and the logits over the whole vocabulary."""

    def __init__(self, cfg, weights, tp_size, batch, max_seq, **kw):
        import threading
        self.tp = tp_size
        self.batch = batch
        self._barrier = threading.Barrier(tp_size)
        self._bufs = [None] * tp_size
        self.shards = []
        for r in range(tp_size):
            scfg, sw, lm = shard_decoder(cfg, weights, tp_size, r)
            self.shards.append(DecoderRef(scfg, sw, batch, max_seq, reduce=self._make_reduce(r), lm_rows=lm, **kw))

    def _make_reduce(self, r):
        def red(arr):
            self._bufs[r] = arr
            self._barrier.wait()
            total = self._bufs[0].copy()
            for j in range(1, self.tp):
                total += self._bufs[j]
            self._barrier.wait()  # every rank holds its sum before any buffer changes
            arr[:] = total
        return red

    def step(self, tokens):
        import threading
        out = [None] * self.tp

        def run(r):
            out[r] = self.shards[r].step(tokens, want_logits=True)
        threads = [threading.Thread(target=run, args=(r,)) for r in range(self.tp)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        logits = np.concatenate([o[1] for o in out], axis=1)
        return np.argmax(logits, axis=1).astype(np.int32), logits

    def close(self):
        for s in self.shards:
            s.close()

