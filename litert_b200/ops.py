"""Host-side mirror of the reference operators on the hot path, over the C ABI.

Each function takes torch CUDA tensors in the reference's own layouts, and mirrors the argument
meaning of the reference kernel it replaces (cited per function; paths are inside the LiteRT
source tree). torch only provides device memory and the current stream. There is no CPU
fallback: every call goes to liblitert_b200.so.
"""
import ctypes
import math

import torch

from . import _lib
from ._lib import B200Error, check

ACT_NONE, ACT_RELU, ACT_RELU_N1_TO_1, ACT_RELU6, ACT_TANH, ACT_SIGN_BIT, ACT_SIGMOID = range(7)
DTYPE_F16, DTYPE_I8, DTYPE_F32 = 0, 1, 2


def _ptr(t):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _need(t, dtype, name):
    if t is None:
        return None
    if not t.is_cuda:
        raise B200Error(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise B200Error(f"{name} must be {dtype}, got {t.dtype}")
    return t.contiguous()


class Workspace:
    """The two device buffers every op on one stream shares (see include/litert_b200.h)."""

    def __init__(self, device="cuda", scratch_bytes=1 << 20):
        lib = _lib.load()
        self.device = torch.device(device)
        self.zero = torch.empty(lib.b200_zero_workspace_bytes(), dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            check(lib.b200_zero_workspace_init(_ptr(self.zero), _stream()))
        self.scratch = torch.empty(scratch_bytes, dtype=torch.uint8, device=self.device)
        self.sdpa = None

    def scratch_for(self, m, k):
        need = _lib.load().b200_fc_scratch_bytes(m, k)
        if self.scratch.numel() < need:
            self.scratch = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self.scratch

    def sdpa_for(self, b, n, nkv, h, s_max):
        need = _lib.load().b200_sdpa_workspace_bytes(b, n, nkv, h, s_max)
        if self.sdpa is None or self.sdpa.numel() < need:
            self.sdpa = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self.sdpa

    def check_status(self):
        """Synchronises and raises if a device-side bounded wait ran out."""
        st = ctypes.c_int(0)
        check(_lib.load().b200_read_status(_ptr(self.zero), _stream(), ctypes.byref(st)))


class PackedInt8Weights:
    """int8 filter [n,k] repacked once into the streamed tile layout, with its row sums
    (the reference's persistent row_sums temporary, tflite/kernels/fully_connected.cc:697-708)."""

    def __init__(self, w):
        lib = _lib.load()
        w = _need(w, torch.int8, "weights")
        self.n, self.k = w.shape
        self.packed = torch.empty(lib.b200_packed_w8_bytes(self.n, self.k), dtype=torch.uint8, device=w.device)
        self.row_sums = torch.empty(self.n, dtype=torch.int32, device=w.device)
        check(lib.b200_pack_w8(_ptr(w), self.n, self.k, _ptr(self.packed), _ptr(self.row_sums), _stream()))


class PackedInt4Weights:
    """Blockwise int4 filter (packed nibbles [n, ceil(k/2)], fp16 scales [n, k/blocksize])."""

    def __init__(self, w4, scales_f16, blocksize):
        lib = _lib.load()
        w4 = _need(w4, torch.uint8, "w4")
        sc = _need(scales_f16, torch.float16, "scales")
        self.n = w4.shape[0]
        self.k = sc.shape[1] * blocksize
        self.blocksize = blocksize
        if w4.shape[1] != (self.k + 1) // 2:
            raise B200Error("w4 row length does not match the scales")
        self.packed = torch.empty(lib.b200_packed_w4_bytes(self.n, self.k), dtype=torch.uint8, device=w4.device)
        self.kfsum = torch.empty(self.n, dtype=torch.float32, device=w4.device)
        check(lib.b200_pack_w4(_ptr(w4), _ptr(sc), self.n, self.k, blocksize, _ptr(self.packed), _ptr(self.kfsum),
                               _stream()))


def quantize_rows(x, asymmetric=True):
    """tensor_utils::BatchQuantizeFloats (tflite/kernels/internal/portable_tensor_utils.h:158-176)."""
    x = _need(x, torch.float32, "x")
    m, k = x.shape
    q = torch.empty((m, k), dtype=torch.int8, device=x.device)
    scales = torch.empty(m, dtype=torch.float32, device=x.device)
    zps = torch.zeros(m, dtype=torch.int32, device=x.device)
    check(_lib.load().b200_quantize_rows(_ptr(x), m, k, 1 if asymmetric else 0, _ptr(q), _ptr(scales), _ptr(zps),
                                         _stream()))
    return q, scales, zps


def fully_connected_int8(x, weights, bias, input_zero_point, output_zero_point, multipliers, shifts, act_min=-128,
                         act_max=127, filter_zero_point=0, ws=None, out=None):
    """Full-integer FULLY_CONNECTED (tflite/kernels/fully_connected.cc:1383-1421 per channel, 1255-1285 per
    tensor). x int8 [..., k]; multipliers/shifts int32 tensors with n entries (per channel) or one."""
    lib = _lib.load()
    x = _need(x, torch.int8, "x")
    k = weights.k
    m = x.numel() // k
    bias = _need(bias, torch.int32, "bias")
    mult = _need(multipliers, torch.int32, "multipliers")
    shift = _need(shifts, torch.int32, "shifts")
    per_channel = 1 if mult.numel() > 1 else 0
    ws = ws or Workspace(x.device)
    y = out if out is not None else torch.empty((m, weights.n), dtype=torch.int8, device=x.device)
    scratch = ws.scratch_for(m, k)
    check(lib.b200_fc_int8(_ptr(x), m, k, _ptr(weights.packed), weights.n, _ptr(weights.row_sums), _ptr(bias),
                           -int(input_zero_point), -int(filter_zero_point), int(output_zero_point), _ptr(mult),
                           _ptr(shift), per_channel, int(act_min), int(act_max), _ptr(y), _ptr(ws.zero),
                           _ptr(scratch), scratch.numel(), _stream()))
    return y


def fully_connected_hybrid(x, weights, filter_scales, bias=None, asymmetric_quantize_inputs=True,
                           activation=ACT_NONE, ws=None, out=None):
    """Dynamic-range FULLY_CONNECTED, EvalHybridDense (tflite/kernels/fully_connected.cc:763-858)."""
    lib = _lib.load()
    x = _need(x, torch.float32, "x")
    k = weights.k
    m = x.numel() // k
    fs = _need(filter_scales, torch.float32, "filter_scales").reshape(-1)
    if fs.numel() not in (1, weights.n):
        raise B200Error("filter_scales must have 1 or n entries")
    bias = _need(bias, torch.float32, "bias")
    ws = ws or Workspace(x.device)
    y = out if out is not None else torch.empty((m, weights.n), dtype=torch.float32, device=x.device)
    scratch = ws.scratch_for(m, k)
    check(lib.b200_fc_hybrid(_ptr(x), m, k, _ptr(weights.packed), weights.n, _ptr(weights.row_sums), _ptr(fs),
                             1 if fs.numel() > 1 else 0, _ptr(bias), 1 if asymmetric_quantize_inputs else 0,
                             int(activation), _ptr(y), _ptr(ws.zero), _ptr(scratch), scratch.numel(), _stream()))
    return y


def fully_connected_blockwise4(x, weights, bias=None, ws=None, out=None):
    """Blockwise int4 FULLY_CONNECTED, EvalBlockwise4Bit (tflite/kernels/fully_connected.cc:1014-1086)."""
    lib = _lib.load()
    x = _need(x, torch.float32, "x")
    k = weights.k
    m = x.numel() // k
    bias = _need(bias, torch.float32, "bias")
    ws = ws or Workspace(x.device)
    y = out if out is not None else torch.empty((m, weights.n), dtype=torch.float32, device=x.device)
    scratch = ws.scratch_for(m, k)
    check(lib.b200_fc_w4(_ptr(x), m, k, _ptr(weights.packed), weights.n, weights.blocksize, _ptr(weights.kfsum),
                         _ptr(bias), _ptr(y), _ptr(ws.zero), _ptr(scratch), scratch.numel(), _stream()))
    return y


_DT = {torch.float16: DTYPE_F16, torch.int8: DTYPE_I8, torch.float32: DTYPE_F32}


def sdpa_decode(q, k, v, lengths=None, mask=None, scale=None, logit_cap=0.0, k_scale=None, v_scale=None, ws=None):
    """odml.scaled_dot_product_attention for one query token per sequence
    (tflite/experimental/genai/sdpa.cc:361-662). q [b,1,n,h]; k, v [b,s_max,nkv,h]."""
    lib = _lib.load()
    if q.dtype not in (torch.float16, torch.float32) or k.dtype not in _DT or v.dtype != k.dtype:
        raise B200Error("unsupported dtypes for sdpa_decode")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    b, t, n, h = q.shape
    if t != 1:
        raise B200Error("sdpa_decode handles one query token per sequence")
    s_max, nkv = k.shape[1], k.shape[2]
    lengths = _need(lengths, torch.int32, "lengths")
    mask = _need(mask, torch.float32, "mask")
    k_scale = _need(k_scale, torch.float32, "k_scale")
    v_scale = _need(v_scale, torch.float32, "v_scale")
    ws = ws or Workspace(q.device)
    out = torch.empty_like(q)
    wsb = ws.sdpa_for(b, n, nkv, h, s_max)
    check(lib.b200_sdpa_decode(_ptr(q), _ptr(k), _ptr(v), _ptr(k_scale), _ptr(v_scale), _ptr(lengths), _ptr(mask),
                               _ptr(out), b, n, nkv, h, s_max, _DT[q.dtype], _DT[k.dtype],
                               float(scale) if scale else 0.0, float(logit_cap), _ptr(wsb), wsb.numel(), _stream()))
    return out


def sdpa_rows(q, k, v, lengths, scale=None, logit_cap=0.0, k_scale=None, v_scale=None):
    """The composite with several query tokens of ONE sequence: q [rows, n, h]; k, v [s_max, nkv, h] (that
    sequence's cache); row r attends over the first lengths[r] cached tokens (lengths[r] = start + r + 1 is
    the causal mask). Returns [rows, n, h] in q's dtype."""
    lib = _lib.load()
    if q.dtype not in (torch.float16, torch.float32) or k.dtype not in _DT or v.dtype != k.dtype:
        raise B200Error("unsupported dtypes for sdpa_rows")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    rows, n, h = q.shape
    s_max, nkv = k.shape[0], k.shape[1]
    lengths = _need(lengths, torch.int32, "lengths")
    k_scale = _need(k_scale, torch.float32, "k_scale")
    v_scale = _need(v_scale, torch.float32, "v_scale")
    out = torch.empty_like(q)
    need = lib.b200_sdpa_rows_workspace_bytes(rows, n, nkv, h, s_max)
    wsb = torch.empty(max(int(need), 16), dtype=torch.uint8, device=q.device)
    check(lib.b200_sdpa_rows(_ptr(q), _ptr(k), _ptr(v), _ptr(k_scale), _ptr(v_scale), _ptr(lengths), _ptr(out), rows, n,
                             nkv, h, s_max, _DT[q.dtype], _DT[k.dtype], float(scale) if scale else 0.0,
                             float(logit_cap), _ptr(wsb), wsb.numel(), _stream()))
    return out


# ---- decoder glue ops (include/litert_b200.h, "decoder glue ops") ---------------------------------------
def _gcheck(rc):
    if rc != 0:
        raise B200Error(f"litert_b200 error {rc}: {_lib.load().b200_glue_last_error().decode()}")


class QuantizedRows:
    """m activation rows of k int8 values in the tiled layout the GEMM kernels stream, with one scale and
    zero point per row: the output of the fused glue ops and the input of fully_connected_hybrid_quantized."""

    def __init__(self, m, k, device):
        self.m, self.k = m, k
        self.tiled = torch.empty(max(int(_lib.load().b200_tiled_rows_bytes(m, k)), 128), dtype=torch.uint8, device=device)
        self.scales = torch.zeros(max(m, 256), dtype=torch.float32, device=device)
        self.zero_points = torch.zeros(max(m, 256), dtype=torch.int32, device=device)

    def rows(self):
        """Row-major int8 [m, k] view of the quantized values."""
        out = torch.empty((self.m, self.k), dtype=torch.int8, device=self.tiled.device)
        _gcheck(_lib.load().b200_untile_rows(_ptr(self.tiled), self.m, self.k, _ptr(out), _stream()))
        return out


def embedding_lookup(ids, table, row_scales, out_scale=1.0):
    """Hybrid EMBEDDING_LOOKUP (tflite/kernels/embedding_lookup.cc, EvalHybrid) times a constant."""
    ids = _need(ids, torch.int32, "ids").reshape(-1)
    table = _need(table, torch.int8, "table")
    row_scales = _need(row_scales, torch.float32, "row_scales")
    vocab, d = table.shape
    out = torch.empty((ids.numel(), d), dtype=torch.float32, device=table.device)
    _gcheck(_lib.load().b200_embedding_lookup(_ptr(ids), ids.numel(), _ptr(table), _ptr(row_scales), vocab, d,
                                              float(out_scale), _ptr(out), _stream()))
    return out


def add_rmsnorm_quantize(h, delta, gain, eps=1e-6):
    """h += delta (in place; delta may be None); returns the quantized rows of rms_norm(h) * gain."""
    h = _need(h, torch.float32, "h")
    if not h.is_contiguous():
        raise B200Error("h must be contiguous (it is updated in place)")
    delta = _need(delta, torch.float32, "delta")
    gain = _need(gain, torch.float32, "gain")
    rows, d = h.shape
    q = QuantizedRows(rows, d, h.device)
    _gcheck(_lib.load().b200_add_rmsnorm_quantize(_ptr(h), _ptr(delta), _ptr(gain), rows, d, float(eps), _ptr(q.tiled),
                                                  _ptr(q.scales), _ptr(q.zero_points), _stream()))
    return q


def geglu_quantize(gate_up):
    """gate_up [rows, 2 f] (gate then up) -> quantized rows of gelu_tanh(gate) * up."""
    gate_up = _need(gate_up, torch.float32, "gate_up")
    rows, f2 = gate_up.shape
    q = QuantizedRows(rows, f2 // 2, gate_up.device)
    _gcheck(_lib.load().b200_geglu_quantize(_ptr(gate_up), rows, f2 // 2, _ptr(q.tiled), _ptr(q.scales),
                                            _ptr(q.zero_points), _stream()))
    return q


def rope_table(positions, head_dim, base=10000.0, device="cuda"):
    """float32 [positions, head_dim / 2, 2] = (cos, sin), computed on the host as the reference's host side does."""
    import numpy as np
    cs = np.empty((positions, head_dim // 2, 2), np.float32)
    _gcheck(_lib.load().b200_rope_table(cs.ctypes.data_as(ctypes.c_void_p), positions, head_dim, float(base)))
    return torch.from_numpy(cs).to(device)


def rope_kv_append(qkv, heads, kv_heads, head_dim, table, positions, k_cache, v_cache, k_scale=None, v_scale=None,
                   one_sequence=False):
    """Rotates q and k of qkv [rows, (heads + 2 kv_heads) * head_dim], appends k and v to the caches
    [batch, max_seq, kv_heads, head_dim] (fp16 or int8) at `positions`; returns q [rows, heads, head_dim]."""
    qkv = _need(qkv, torch.float32, "qkv")
    positions = _need(positions, torch.int32, "positions")
    table = _need(table, torch.float32, "table")
    rows = qkv.shape[0]
    max_seq = k_cache.shape[-3]
    if table.shape[0] < max_seq + 1:
        raise B200Error("the rope table must cover positions 0..max_seq")
    q = torch.empty((rows, heads, head_dim), dtype=torch.float32, device=qkv.device)
    _gcheck(_lib.load().b200_rope_kv_append(_ptr(qkv), rows, heads, kv_heads, head_dim, _ptr(table), _ptr(positions),
                                            max_seq, _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(k_scale), _ptr(v_scale),
                                            _DT[k_cache.dtype], 1 if one_sequence else 0, _stream()))
    return q


def argmax_rows(logits, soft_cap=0.0):
    logits = _need(logits, torch.float32, "logits")
    rows, n = logits.shape
    out = torch.empty(rows, dtype=torch.int32, device=logits.device)
    need = int(_lib.load().b200_argmax_workspace_bytes(rows))
    wsb = torch.empty(need, dtype=torch.uint8, device=logits.device)
    _gcheck(_lib.load().b200_argmax_rows(_ptr(logits), rows, n, float(soft_cap), _ptr(out), _ptr(wsb), need, _stream()))
    return out


def attention_step(qkv, positions, table, k_cache, v_cache, heads, head_dim, k_scale=None, v_scale=None, scale=0.0):
    """One decode step of a multi-query layer's attention in one launch: rotation, cache append, attention
    over the cached prefix and the new token, row quantization. Returns QuantizedRows [batch, heads * head_dim]."""
    qkv = _need(qkv, torch.float32, "qkv")
    positions = _need(positions, torch.int32, "positions")
    batch = qkv.shape[0]
    max_seq = k_cache.shape[1]
    q = QuantizedRows(batch, heads * head_dim, qkv.device)
    _gcheck(_lib.load().b200_attention_step(_ptr(qkv), _ptr(positions), _ptr(table), _ptr(k_cache), _ptr(v_cache),
                                            _ptr(k_scale), _ptr(v_scale), batch, heads, head_dim, max_seq,
                                            _DT[k_cache.dtype], float(scale), _ptr(q.tiled), _ptr(q.scales),
                                            _ptr(q.zero_points), _stream()))
    return q


def sdpa_decode_quantized(q, k, v, lengths, scale=0.0, k_scale=None, v_scale=None):
    """sdpa_decode whose result leaves as quantized rows [b, n * h]."""
    lib = _lib.load()
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    b, t, n, h = q.shape
    s_max, nkv = k.shape[1], k.shape[2]
    lengths = _need(lengths, torch.int32, "lengths")
    out = QuantizedRows(b, n * h, q.device)
    need = int(lib.b200_sdpa_workspace_bytes(b, n, nkv, h, s_max))
    wsb = torch.empty(max(need, 16), dtype=torch.uint8, device=q.device)
    _gcheck(lib.b200_sdpa_decode_quantized(_ptr(q), _ptr(k), _ptr(v), _ptr(k_scale), _ptr(v_scale), _ptr(lengths), b, n,
                                           nkv, h, s_max, _DT[q.dtype], _DT[k.dtype], float(scale), _ptr(out.tiled),
                                           _ptr(out.scales), _ptr(out.zero_points), _ptr(wsb), wsb.numel(), _stream()))
    return out


def fully_connected_hybrid_quantized(rows, weights, filter_scales, bias=None, activation=ACT_NONE, ws=None):
    """The int8 dot products and dequantization of EvalHybridDense on rows that are already quantized."""
    fs = _need(filter_scales, torch.float32, "filter_scales").reshape(-1)
    bias = _need(bias, torch.float32, "bias")
    ws = ws or Workspace(rows.tiled.device)
    if rows.k != weights.k:
        raise B200Error("row width does not match the weights")
    y = torch.empty((rows.m, weights.n), dtype=torch.float32, device=rows.tiled.device)
    _gcheck(_lib.load().b200_fc_hybrid_quantized(_ptr(rows.tiled), _ptr(rows.scales), _ptr(rows.zero_points), rows.m,
                                                 rows.k, _ptr(weights.packed), weights.n, _ptr(weights.row_sums),
                                                 _ptr(fs), 1 if fs.numel() > 1 else 0, _ptr(bias), int(activation),
                                                 _ptr(y), _ptr(ws.zero), _stream()))
    return y


def lm_head_greedy(rows, weights, filter_scales, soft_cap=0.0, want_logits=False, ws=None):
    """The vocabulary projection with the greedy pick in its epilogue (at most 16 rows): returns
    (tokens int32 [m], logits [m, n] or None)."""
    lib = _lib.load()
    fs = _need(filter_scales, torch.float32, "filter_scales").reshape(-1)
    ws = ws or Workspace(rows.tiled.device)
    dev = rows.tiled.device
    tokens = torch.empty(rows.m, dtype=torch.int32, device=dev)
    logits = torch.empty((rows.m, weights.n), dtype=torch.float32, device=dev) if want_logits else None
    need = int(lib.b200_lm_head_workspace_bytes(rows.m))
    wsb = torch.empty(need, dtype=torch.uint8, device=dev)
    _gcheck(lib.b200_lm_head_greedy(_ptr(rows.tiled), _ptr(rows.scales), _ptr(rows.zero_points), rows.m, rows.k,
                                    _ptr(weights.packed), weights.n, _ptr(weights.row_sums), _ptr(fs), float(soft_cap),
                                    _ptr(logits), _ptr(tokens), _ptr(wsb), need, _ptr(ws.zero), _stream()))
    return tokens, logits
