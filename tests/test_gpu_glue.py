"""The ops between a decoder layer's projections, one kernel at a time, against the matching stage of the
CPU restatement of the graph (oracle/decoder_ref.c), on the ORACLE's inputs and at the widths of the
decode benchmark: d_model 2048, feed-forward 16384, 8 query heads of 256 on one KV head, vocabulary
256000. Every call goes through the C ABI ("decoder glue ops" in include/litert_b200.h).

What "equal" means per stage:
 * embedding, rotary embedding and cache append, arg-max: bit-exact;
 * stages ending in a row quantization (norm, GeGLU): the device reduces a row's sum of squares in a
   tree and evaluates tanhf with CUDA's libm, the oracle sums 2048 squares serially in float32 (error
   up to a few 1e-6 relative, which is the reference's own) and uses glibc, so the float row may differ
   in its last bits; after quantization that is the row's scale within 1e-5 relative and int8 values
   within 1 step, with the number of differing values bounded and printed;
 * attention: 2e-2 of the output's magnitude against the float32 restatement on the up-converted cache.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

D_MODEL, D_FF, HEADS, HEAD_DIM, VOCAB = 2048, 16384, 8, 256, 256000


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def _compare_quantized(oracle, got, want_rows, label, max_flip_frac=5e-3):
    """got: ops.QuantizedRows; want_rows: the oracle's float rows before quantization."""
    q_ref, s_ref, z_ref = oracle.batch_quantize_floats(want_rows, asymmetric=True)
    m = want_rows.shape[0]
    q = got.rows().cpu().numpy().astype(np.int32)
    s = got.scales[:m].cpu().numpy()
    z = got.zero_points[:m].cpu().numpy()
    assert np.allclose(s, s_ref, rtol=1e-5, atol=0), (label, s, s_ref)
    assert np.max(np.abs(z - z_ref)) <= 1, (label, z, z_ref)
    diff = np.abs(q - q_ref.astype(np.int32))
    assert diff.max() <= 1, (label, diff.max())
    frac = float((diff != 0).mean())
    print(f"{label}: {int((diff != 0).sum())} of {diff.size} int8 values differ by one step ({frac:.2e}); "
          f"zero points equal: {bool(np.array_equal(z, z_ref))}")
    assert frac <= max_flip_frac, (label, frac)


def test_embedding_lookup_bit_exact(oracle):
    from litert_b200 import ops

    rng = np.random.default_rng(51)
    table = rng.integers(-127, 128, (VOCAB, D_MODEL), dtype=np.int8)
    scales = rng.uniform(1e-3, 1e-2, VOCAB).astype(np.float32)
    ids = np.concatenate([[0, VOCAB - 1], rng.integers(0, VOCAB, 30)]).astype(np.int32)
    embed_scale = float(np.sqrt(np.float32(D_MODEL)))
    got = ops.embedding_lookup(_dev(ids), _dev(table), _dev(scales), embed_scale).cpu().numpy()
    want = oracle.stage_embed(ids, table, scales, embed_scale)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("rows", [1, 32, 40])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm_quantize(oracle, rows, with_delta):
    from litert_b200 import ops

    rng = np.random.default_rng(60 + rows)
    h = (rng.standard_normal((rows, D_MODEL)) * 3.0).astype(np.float32)
    delta = (rng.standard_normal((rows, D_MODEL)) * 2.0).astype(np.float32) if with_delta else None
    gain = (rng.standard_normal(D_MODEL) * 0.02 + 1.0).astype(np.float32)
    h_dev = _dev(h)
    got = ops.add_rmsnorm_quantize(h_dev, None if delta is None else _dev(delta), _dev(gain), eps=1e-6)
    h_ref, x_ref = oracle.stage_add_rmsnorm(h, delta, gain, 1e-6)
    assert np.array_equal(h_dev.cpu().numpy(), h_ref), "residual stream after the add"
    _compare_quantized(oracle, got, x_ref, f"add_rmsnorm_quantize rows={rows} delta={with_delta}")


def test_add_rmsnorm_quantize_keeps_eps_and_zero_rows(oracle):
    """A norm that dropped eps would turn an all-zero row into NaNs, and a tiny row into a large one."""
    from litert_b200 import ops

    h = np.zeros((3, D_MODEL), np.float32)
    h[1] = 1e-4
    h[2, 5] = 1.0
    gain = np.ones(D_MODEL, np.float32)
    got = ops.add_rmsnorm_quantize(_dev(h), None, _dev(gain), eps=1e-6)
    _, x_ref = oracle.stage_add_rmsnorm(h, None, gain, 1e-6)
    _compare_quantized(oracle, got, x_ref, "add_rmsnorm_quantize eps / zero row", max_flip_frac=1e-2)


@pytest.mark.parametrize("rows", [1, 32, 40])
def test_geglu_quantize(oracle, rows):
    from litert_b200 import ops

    rng = np.random.default_rng(70 + rows)
    gate_up = (rng.standard_normal((rows, 2 * D_FF)) * 4.0).astype(np.float32)
    got = ops.geglu_quantize(_dev(gate_up))
    f_ref = oracle.stage_geglu(gate_up[:, :D_FF], gate_up[:, D_FF:])
    _compare_quantized(oracle, got, f_ref, f"geglu_quantize rows={rows}")


@pytest.mark.parametrize("kv", ["f16", "i8"])
@pytest.mark.parametrize("rows,one_sequence", [(1, False), (32, False), (40, True)])
def test_rope_kv_append_bit_exact(oracle, kv, rows, one_sequence):
    from litert_b200 import ops

    max_seq = 8192
    rng = np.random.default_rng(80 + rows)
    qkv = (rng.standard_normal((rows, (HEADS + 2) * HEAD_DIM)) * 5.0).astype(np.float32)
    if one_sequence:
        pos = (7000 + np.arange(rows)).astype(np.int32)
    else:
        pos = rng.integers(0, max_seq, rows).astype(np.int32)
        pos[0] = max_seq - 1
    batch = 1 if one_sequence else rows
    table = ops.rope_table(max_seq + 1, HEAD_DIM)
    assert np.array_equal(table.cpu().numpy(), oracle.rope_table(max_seq + 1, HEAD_DIM)), "host-side cos / sin table"
    dt = torch.float16 if kv == "f16" else torch.int8
    kc = torch.zeros((batch, max_seq, 1, HEAD_DIM), dtype=dt, device="cuda")
    vc = torch.zeros_like(kc)
    ks = torch.zeros((batch, max_seq, 1), dtype=torch.float32, device="cuda") if kv == "i8" else None
    vs = torch.zeros_like(ks) if kv == "i8" else None
    q = ops.rope_kv_append(_dev(qkv), HEADS, 1, HEAD_DIM, table, _dev(pos), kc, vc, ks, vs, one_sequence=one_sequence)
    x = qkv.reshape(rows, HEADS + 2, HEAD_DIM)
    q_ref = oracle.stage_rope(x[:, :HEADS], pos)
    k_ref = oracle.stage_rope(x[:, HEADS:HEADS + 1], pos)[:, 0]
    v_ref = x[:, HEADS + 1]
    assert np.array_equal(q.cpu().numpy(), q_ref), "rotated queries"
    seq = np.zeros(rows, np.int64) if one_sequence else np.arange(rows)
    k_got = kc.cpu().numpy()[seq, pos, 0]
    v_got = vc.cpu().numpy()[seq, pos, 0]
    if kv == "f16":
        assert np.array_equal(k_got, k_ref.astype(np.float16)) and np.array_equal(v_got, v_ref.astype(np.float16))
    else:
        for name, got, ref, sc in (("k", k_got, k_ref, ks), ("v", v_got, v_ref, vs)):
            s_got = sc.cpu().numpy()[seq, pos, 0]
            want = oracle.stage_kv_round(ref, 2)
            assert np.array_equal(got.astype(np.float32) * s_got[:, None], want), name
    # nothing else was written
    assert int((kc != 0).any(dim=-1).sum().item()) <= rows


@pytest.mark.parametrize("t,heads_q,heads_kv,h,position", [(1, 8, 1, 256, 1030), (6, 4, 2, 64, 0), (3, 4, 1, 64, 29)])
def test_rope_and_kv_cache_update_in_one_launch_bit_exact(t, heads_q, heads_kv, h, position):
    """b200_rope_kv_cache_update_f32 against the graph's own arithmetic (x * cos + concat(-x2, x1) * sin, every
    product and the sum rounded on their own) and odml.update_kv_cache's slot rule; a write past the last slot sets
    status 201 and leaves the caches alone."""
    import ctypes

    from litert_b200 import _lib

    lib = _lib.load()
    max_entries = 1040 if position > 100 else 32
    rng = np.random.default_rng(t * 100 + h)
    q = (rng.standard_normal((t, heads_q, h)) * 3).astype(np.float32)
    k = (rng.standard_normal((t, heads_kv, h)) * 3).astype(np.float32)
    v = rng.standard_normal((t, heads_kv, h)).astype(np.float32)
    ang = rng.uniform(-3.0, 3.0, (t, h)).astype(np.float32)
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)

    def rope(x):
        rot = np.concatenate([x[..., h // 2:] * np.float32(-1.0), x[..., :h // 2]], axis=-1)
        return (x * cos[:, None, :]) + (rot * sin[:, None, :])

    def run(pos):
        d = {n: _dev(a) for n, a in (("q", q), ("k", k), ("v", v), ("cos", cos), ("sin", sin))}
        d_pos = _dev(np.asarray([pos], np.int64))
        q_out = torch.empty_like(d["q"])
        kc = torch.zeros((max_entries, heads_kv * h), dtype=torch.float32, device="cuda")
        vc = torch.zeros_like(kc)
        ws = torch.zeros(64, dtype=torch.int32, device="cuda")
        p = lambda x: ctypes.c_void_p(x.data_ptr())
        rc = lib.b200_rope_kv_cache_update_f32(p(d_pos), p(d["q"]), p(d["k"]), p(d["v"]), p(d["cos"]), p(d["sin"]), p(q_out), t,
                                               heads_q, heads_kv, h, max_entries, p(kc), p(vc), p(ws),
                                               ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0
        torch.cuda.synchronize()
        return q_out.cpu().numpy(), kc.cpu().numpy(), vc.cpu().numpy(), int(ws[0].item())

    q_out, kc, vc, status = run(position)
    assert status == 0
    assert np.array_equal(q_out, rope(q)), "rotated queries"
    want_k = np.zeros_like(kc)
    want_v = np.zeros_like(vc)
    want_k[position:position + t] = rope(k).reshape(t, -1)
    want_v[position:position + t] = v.reshape(t, -1)
    assert np.array_equal(kc, want_k) and np.array_equal(vc, want_v)
    q_out, kc, vc, status = run(max_entries - t + 1)
    assert status == 201 and not kc.any() and not vc.any()
    assert np.array_equal(q_out, rope(q))


def test_argmax_rows_first_index_and_nan_rule(oracle):
    from litert_b200 import ops

    rng = np.random.default_rng(90)
    lg = rng.standard_normal((8, VOCAB)).astype(np.float32)
    lg[1, [77, 200000]] = 9.0           # a tie: the lower index wins
    lg[2, 0] = np.nan                   # a NaN at index 0 wins outright
    lg[3, 12345] = np.nan               # a NaN elsewhere never wins
    lg[3, 255999] = 8.0
    lg[4, :] = -np.inf                  # nothing beats the first element
    lg[5, :] = np.nan
    lg[6, VOCAB - 1] = 50.0
    lg[7, 1] = np.inf
    got = ops.argmax_rows(_dev(lg)).cpu().numpy()
    want = oracle.stage_argmax(lg)
    assert np.array_equal(got, want), (got, want)
    assert list(want[:5]) == [int(np.argmax(lg[0])), 77, 0, 255999, 0]
    one = ops.argmax_rows(_dev(lg[:1])).cpu().numpy()
    assert one[0] == want[0]


def test_argmax_rows_soft_cap(oracle):
    from litert_b200 import ops

    rng = np.random.default_rng(91)
    lg = (rng.standard_normal((4, 5000)) * 20.0).astype(np.float32)
    lg[0, [10, 4000]] = [400.0, 900.0]  # both saturate at the cap: the lower index wins
    got = ops.argmax_rows(_dev(lg), soft_cap=30.0).cpu().numpy()
    want = oracle.stage_argmax(oracle.stage_softcap(lg, 30.0))
    # CUDA's tanhf and glibc's may differ in the last bit: accept either index when the capped values tie there
    capped = oracle.stage_softcap(lg, 30.0)
    for r in range(4):
        assert got[r] == want[r] or abs(capped[r, got[r]] - capped[r, want[r]]) <= 4e-6 * 30.0, (r, got[r], want[r])
    assert want[0] == 10


def _attention_reference(oracle, q_rot, k_rows, v_rows, scale):
    """q_rot [heads, hd]; k_rows / v_rows [len, hd] as float32 -> [heads, hd]."""
    out = oracle.sdpa_f32(q_rot[None, None], k_rows[None, :, None, :], v_rows[None, :, None, :], None, scale)
    return out[0, 0]


@pytest.mark.parametrize("kv", ["f16", "i8"])
@pytest.mark.parametrize("positions", [[0], [69], [1039], [1250], [1299], [2440], [7999], [3, 70, 1040, 5000]])
def test_attention_step_against_the_float_restatement(oracle, kv, positions):
    """attn_step_cluster_kernel: rotation + append + attention + quantization in one launch, at 1, 70,
    1040 and 8000 cached tokens (the new one included); 1251, 1300 and 2441 tokens give a CTA a share a
    little longer than its staging area (fp16 and int8 rows), whose tail is read from the cache."""
    from litert_b200 import ops

    max_seq = 8192
    batch = len(positions)
    pos = np.asarray(positions, np.int32)
    rng = np.random.default_rng(100 + int(pos.sum()))
    qkv = rng.standard_normal((batch, (HEADS + 2) * HEAD_DIM)).astype(np.float32)
    k_hist = rng.standard_normal((batch, max_seq, HEAD_DIM)).astype(np.float32)
    v_hist = rng.standard_normal((batch, max_seq, HEAD_DIM)).astype(np.float32)
    mode = 1 if kv == "f16" else 2
    if kv == "f16":
        kc, vc = _dev(k_hist.astype(np.float16)[:, :, None]), _dev(v_hist.astype(np.float16)[:, :, None])
        ks = vs = None
        k_f32, v_f32 = k_hist.astype(np.float16).astype(np.float32), v_hist.astype(np.float16).astype(np.float32)
    else:
        from litert_b200 import workloads
        kq, ksc = workloads.quantize_kv_per_token(k_hist)
        vq, vsc = workloads.quantize_kv_per_token(v_hist)
        kc, vc, ks, vs = _dev(kq[:, :, None]), _dev(vq[:, :, None]), _dev(ksc[:, :, None]), _dev(vsc[:, :, None])
        k_f32, v_f32 = kq.astype(np.float32) * ksc[..., None], vq.astype(np.float32) * vsc[..., None]
    table = ops.rope_table(max_seq + 1, HEAD_DIM)
    got = ops.attention_step(_dev(qkv), _dev(pos), table, kc, vc, HEADS, HEAD_DIM, ks, vs)
    x = qkv.reshape(batch, HEADS + 2, HEAD_DIM)
    q_rot = oracle.stage_rope(x[:, :HEADS], pos)
    k_new = oracle.stage_kv_round(oracle.stage_rope(x[:, HEADS:HEADS + 1], pos)[:, 0], mode)
    v_new = oracle.stage_kv_round(x[:, HEADS + 1], mode)
    want = np.empty((batch, HEADS * HEAD_DIM), np.float32)
    for b in range(batch):
        n = int(pos[b])
        kr = np.concatenate([k_f32[b, :n], k_new[b:b + 1]])
        vr = np.concatenate([v_f32[b, :n], v_new[b:b + 1]])
        want[b] = _attention_reference(oracle, q_rot[b], kr, vr, 1.0 / np.sqrt(HEAD_DIM)).reshape(-1)
        # the appended cache rows are the rounded rotated key and the rounded value, bit for bit
        if kv == "f16":
            assert np.array_equal(kc[b, n, 0].float().cpu().numpy(), k_new[b])
            assert np.array_equal(vc[b, n, 0].float().cpu().numpy(), v_new[b])
        else:
            assert np.array_equal(kc[b, n, 0].float().cpu().numpy() * ks[b, n, 0].item(), k_new[b])
    q = got.rows().cpu().numpy().astype(np.float32)
    s = got.scales[:batch].cpu().numpy()
    z = got.zero_points[:batch].cpu().numpy()
    deq = (q - z[:, None]) * s[:, None]
    err = np.max(np.abs(deq - want), axis=1) / np.max(np.abs(want), axis=1)
    print(f"attention step kv={kv} positions={positions}: max error {err.max():.3e} of the output's magnitude")
    assert err.max() <= 2e-2, err
    # and the row parameters are those of the reference quantizer on a row this close
    _, s_ref, _ = oracle.batch_quantize_floats(want)
    assert np.allclose(s, s_ref, rtol=2e-2)


@pytest.mark.parametrize("kv", ["f16", "i8"])
def test_sdpa_decode_quantized_merge(oracle, kv):
    """sdpa_decode + sdpa_merge_quant_kernel (the path wide batches take): 12 sequences at ragged depths."""
    from litert_b200 import ops, workloads

    s_max = 8192
    lengths = np.asarray([1, 70, 1040, 8000, 17, 129, 4096, 8192, 2, 300, 64, 5555], np.int32)
    b = lengths.size
    rng = np.random.default_rng(110)
    q = rng.standard_normal((b, 1, HEADS, HEAD_DIM)).astype(np.float32)
    k = rng.standard_normal((b, s_max, 1, HEAD_DIM)).astype(np.float32)
    v = rng.standard_normal((b, s_max, 1, HEAD_DIM)).astype(np.float32)
    if kv == "f16":
        kd, vd, ks, vs = _dev(k.astype(np.float16)), _dev(v.astype(np.float16)), None, None
        k32, v32 = k.astype(np.float16).astype(np.float32), v.astype(np.float16).astype(np.float32)
    else:
        kq, ksc = workloads.quantize_kv_per_token(k)
        vq, vsc = workloads.quantize_kv_per_token(v)
        kd, vd, ks, vs = _dev(kq), _dev(vq), _dev(ksc), _dev(vsc)
        k32, v32 = kq.astype(np.float32) * ksc[..., None], vq.astype(np.float32) * vsc[..., None]
    got = ops.sdpa_decode_quantized(_dev(q), kd, vd, _dev(lengths), 0.0, ks, vs)
    rows = got.rows().cpu().numpy().astype(np.float32)
    s = got.scales[:b].cpu().numpy()
    z = got.zero_points[:b].cpu().numpy()
    deq = (rows - z[:, None]) * s[:, None]
    for i in range(b):
        n = int(lengths[i])
        want = oracle.sdpa_f32(q[i:i + 1], k32[i:i + 1, :n], v32[i:i + 1, :n], None, 1.0 / np.sqrt(HEAD_DIM)).reshape(-1)
        err = np.max(np.abs(deq[i] - want)) / np.max(np.abs(want))
        assert err <= 2e-2, (i, n, err)


def _hybrid_from_quantized(q, scales, zps, w, w_scales):
    """EvalHybridDense after the quantization (tflite/kernels/fully_connected.cc:797-858), exactly: int32 dot
    products (float64 BLAS sums of int8 products are exact), minus zero point x row sum, times
    float32(in_scale * w_scale)."""
    n = w.shape[0]
    out = np.empty((q.shape[0], n), np.float32)
    qd = q.astype(np.float64)
    for r0 in range(0, n, 32768):
        wc = w[r0:r0 + 32768]
        dot = (qd @ wc.astype(np.float64).T).astype(np.int64)
        rs = wc.astype(np.int64).sum(axis=1)
        acc = (dot - rs[None, :] * zps[:, None].astype(np.int64)).astype(np.int32)
        sc = (scales[:, None].astype(np.float32) * w_scales[None, r0:r0 + 32768].astype(np.float32)).astype(np.float32)
        out[:, r0:r0 + 32768] = acc.astype(np.float32) * sc
    return out


@pytest.mark.parametrize("m", [1, 32])
@pytest.mark.parametrize("n,k,name", [(2560, 2048, "qkv"), (2048, 2048, "attention output"), (32768, 2048, "gate/up"),
                                      (2048, 16384, "down"), (VOCAB, 2048, "LM head")])
def test_projection_at_decoder_widths_bit_exact(oracle, m, n, k, name):
    """Every GEMV shape of the decode benchmark (cluster split-K, whole-tile and the 296-CTA LM-head launch)
    on rows quantized by the norm kernel: bit-equal to the reference arithmetic."""
    from litert_b200 import ops

    rng = np.random.default_rng(120 + n % 97 + m)
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    ws = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    h = (rng.standard_normal((m, k)) * 2.0).astype(np.float32)
    gain = np.ones(k, np.float32)
    if k <= 12288:
        rows = ops.add_rmsnorm_quantize(_dev(h), None, _dev(gain))
    else:
        rows = ops.geglu_quantize(_dev(np.concatenate([h, np.ones_like(h)], axis=1)))
    packed = ops.PackedInt8Weights(_dev(w))
    y = ops.fully_connected_hybrid_quantized(rows, packed, _dev(ws)).cpu().numpy()
    want = _hybrid_from_quantized(rows.rows().cpu().numpy(), rows.scales[:m].cpu().numpy(),
                                  rows.zero_points[:m].cpu().numpy(), w, ws)
    assert np.array_equal(y, want), (name, np.max(np.abs(y - want)))


@pytest.mark.parametrize("m", [1, 5, 16])
def test_lm_head_greedy_fused_pick(oracle, m):
    """The vocabulary GEMV with the pick in its epilogue (256000 rows: the 296-CTA launch): the tokens are those
    of the serial scan over the bit-exact logits, with ties, a NaN logit at index 0 (wins) and elsewhere (never
    wins), and under a soft-cap."""
    from litert_b200 import ops

    rng = np.random.default_rng(130 + m)
    n, k = VOCAB, D_MODEL
    w = rng.integers(-127, 128, (n, k), dtype=np.int8)
    w[70000] = w[3]                       # two equal columns: the lower index wins a tie
    ws = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    ws[70000] = ws[3]
    h = (rng.standard_normal((m, k)) * 2.0).astype(np.float32)
    rows = ops.add_rmsnorm_quantize(_dev(h), None, _dev(np.ones(k, np.float32)))
    packed = ops.PackedInt8Weights(_dev(w))
    want_logits = _hybrid_from_quantized(rows.rows().cpu().numpy(), rows.scales[:m].cpu().numpy(),
                                         rows.zero_points[:m].cpu().numpy(), w, ws)
    tok, logits = ops.lm_head_greedy(rows, packed, _dev(ws), want_logits=True)
    assert np.array_equal(logits.cpu().numpy(), want_logits)
    assert np.array_equal(tok.cpu().numpy(), oracle.stage_argmax(want_logits))
    tok2, none = ops.lm_head_greedy(rows, packed, _dev(ws))        # without the logits: nothing else changes
    assert none is None and np.array_equal(tok2.cpu().numpy(), tok.cpu().numpy())
    # soft-cap: compare on the capped logits (the cap saturates the largest ones into ties)
    tok3, capped = ops.lm_head_greedy(rows, packed, _dev(ws), soft_cap=30.0, want_logits=True)
    cap_ref = oracle.stage_softcap(want_logits, 30.0)
    got_capped = capped.cpu().numpy()
    assert np.max(np.abs(got_capped - cap_ref)) <= 1e-4
    assert np.array_equal(tok3.cpu().numpy(), oracle.stage_argmax(got_capped))
    # NaN rule: a NaN scale makes that vocabulary row's logit NaN
    for bad, expect_zero in ((0, True), (12345, False)):
        ws_nan = ws.copy()
        ws_nan[bad] = np.nan
        tok4, lg4 = ops.lm_head_greedy(rows, packed, _dev(ws_nan), want_logits=True)
        ref = oracle.stage_argmax(lg4.cpu().numpy())
        assert np.array_equal(tok4.cpu().numpy(), ref)
        assert np.all(ref == 0) if expect_zero else np.all(ref != bad)
