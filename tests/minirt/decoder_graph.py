"""A Gemma-shaped decoder-only graph authored node by node through the mini runtime, the way
tensor/examples/gemma3/gemma3_graph.cc authors it out of TFLite ops and composites (Gemma-1 layout: one KV
head, no q/k norms, no post-norms): hybrid EMBEDDING_LOOKUP, odml.rms_norm, dynamic-range FULLY_CONNECTED
projections, RESHAPE, the rotary embedding as SLICE / MUL / CONCATENATION / MUL / ADD over host-prepared cos
and sin inputs, the odml.update_kv_cache custom op, the odml.scaled_dot_product_attention composite, GELU x up,
residual ADDs, the tied LM head and ARG_MAX. TEST / BENCHMARK INFRASTRUCTURE: the graph a user's converter
would hand the interpreter, used to drive the delegate with a whole decoder in one partition."""
import numpy as np

from . import F32, I8, I32, I64, flex_map


class DecoderGraph:
    def __init__(self, rt, cfg, weights, tokens_per_call, max_seq, rms_eps=1e-6, rope_base=10000.0, want_logits=True):
        """weights: numpy dict as litert_b200.decoder.make_weights lays it out (layers / embed / embed_scales /
        final_norm). tokens_per_call: 1 for decode steps, more for a prompt chunk."""
        self.rt, self.cfg, self.T, self.S = rt, cfg, tokens_per_call, max_seq
        D, N, H, F, V = cfg["d_model"], cfg["n_heads"], cfg["head_dim"], cfg["d_ff"], cfg["vocab"]
        assert cfg["n_kv_heads"] == 1
        T, S = self.T, self.S
        self.rope_base = rope_base
        t = rt.tensor
        self.ids = t(I32, (T,))
        self.pos = t(I64, (1,))
        self.cos = t(F32, (1, T, 1, H))
        self.sin = t(F32, (1, T, 1, H))
        self.mask = t(F32, (1, 1, T, S))
        table = t(I8, (V, D), weights["embed"], channel_scales=weights["embed_scales"], quantized_dimension=0)
        h0 = t(F32, (T, D))
        rt.embedding_lookup(self.ids, table, h0)
        h = t(F32, (T, D))
        rt.mul(h0, t(F32, (1,), np.asarray([np.sqrt(np.float32(D))], np.float32)), h)
        minus_one = t(F32, (1,), np.asarray([-1.0], np.float32))
        eps_blob = flex_map({"epsilon": float(rms_eps)})

        def norm(x, gain):
            y = t(F32, (T, D))
            rt.composite("odml.rms_norm", eps_blob, [x, t(F32, (D,), gain)], y)
            return y

        def fc(x, w, s):
            n = w.shape[0]
            y = t(F32, (T, n))
            rt.fully_connected(x, t(I8, w.shape, w, channel_scales=s), None, y, asymmetric=True)
            return y

        def rope(x4, heads):
            half = H // 2
            x1, x2 = t(F32, (1, T, heads, half)), t(F32, (1, T, heads, half))
            rt.slice(x4, [0, 0, 0, 0], [1, T, heads, half], x1)
            rt.slice(x4, [0, 0, 0, half], [1, T, heads, half], x2)
            nx2 = t(F32, (1, T, heads, half))
            rt.mul(x2, minus_one, nx2)
            rot = t(F32, (1, T, heads, H))
            rt.concatenation([nx2, x1], rot, axis=3)
            xc, rs, out = t(F32, (1, T, heads, H)), t(F32, (1, T, heads, H)), t(F32, (1, T, heads, H))
            rt.mul(x4, self.cos, xc)
            rt.mul(rot, self.sin, rs)
            rt.add(xc, rs, out)
            return out

        sdpa_blob = flex_map({"scale": float(1.0 / np.sqrt(np.float32(H)))})
        for l, lw in enumerate(weights["layers"]):
            x = norm(h, lw["norm1"])
            q, k, v = fc(x, lw["wq"], lw["sq"]), fc(x, lw["wk"], lw["sk"]), fc(x, lw["wv"], lw["sv"])
            q4, k4, v4 = t(F32, (1, T, N, H)), t(F32, (1, T, 1, H)), t(F32, (1, T, 1, H))
            rt.reshape(q, q4)
            rt.reshape(k, k4)
            rt.reshape(v, v4)
            qr, kr = rope(q4, N), rope(k4, 1)
            kfull, vfull = t(F32, (1, S, 1, H)), t(F32, (1, S, 1, H))
            rt.node(32, [self.pos, kr, v4], [kfull, vfull], custom_name="odml.update_kv_cache",
                    init_data=flex_map({"kv_cache_max": int(S), "num_layers": int(cfg["n_layers"]), "layer_index": int(l)}))
            att = t(F32, (1, T, N, H))
            rt.composite("odml.scaled_dot_product_attention", sdpa_blob, [qr, kfull, vfull, self.mask], att)
            a2 = t(F32, (T, N * H))
            rt.reshape(att, a2)
            o = fc(a2, lw["wo"], lw["so"])
            h1 = t(F32, (T, D))
            rt.add(h, o, h1)
            x2 = norm(h1, lw["norm2"])
            g, u = fc(x2, lw["wgate"], lw["sgate"]), fc(x2, lw["wup"], lw["sup"])
            gg, f = t(F32, (T, F)), t(F32, (T, F))
            rt.gelu(g, gg, approximate=True)
            rt.mul(gg, u, f)
            dn = fc(f, lw["wdown"], lw["sdown"])
            h = t(F32, (T, D))
            rt.add(h1, dn, h)
        xf = norm(h, weights["final_norm"])
        self.logits = fc(xf, weights["embed"], weights["embed_scales"])
        self.tokens = t(I32, (T,))
        rt.arg_max(self.logits, self.tokens)
        rt.set_io([self.ids, self.pos, self.cos, self.sin, self.mask], [self.logits, self.tokens] if want_logits else [self.tokens])
        self._table = None

    def feed(self, ids, position):
        """Host side of one call: token ids, the first position, cos / sin of the rotation angles (as the
        reference's host side prepares them) and the causal mask behind `position` cached tokens."""
        T, S, H = self.T, self.S, self.cfg["head_dim"]
        if self._table is None:
            import ctypes

            from litert_b200 import _lib

            self._table = np.empty((S + T, H // 2, 2), np.float32)
            rc = _lib.load().b200_rope_table(self._table.ctypes.data_as(ctypes.c_void_p), S + T, H, float(self.rope_base))
            assert rc == 0
        rt = self.rt
        rt.write(self.ids, np.asarray(ids, np.int32))
        rt.write(self.pos, np.asarray([position], np.int64))
        cs = self._table[position:position + T]                       # [T, H/2, 2]
        rt.write(self.cos, np.concatenate([cs[:, :, 0], cs[:, :, 0]], axis=1).reshape(1, T, 1, H))
        rt.write(self.sin, np.concatenate([cs[:, :, 1], cs[:, :, 1]], axis=1).reshape(1, T, 1, H))
        open_ = np.arange(S)[None, :] <= (position + np.arange(T))[:, None]
        rt.write(self.mask, np.where(open_, 0.0, -1e30).astype(np.float32).reshape(1, 1, T, S))
