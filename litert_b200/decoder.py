"""Python handle on the resident decoder (b200_decoder_* in include/litert_b200.h) and the seeded
synthetic Gemma-shaped weights the decode benchmark uses (random init, as the configuration says;
no checkpoint is involved)."""
import ctypes
import math

import numpy as np
import torch

from . import _lib
from ._lib import B200Error

GEMMA_2B = dict(n_layers=18, d_model=2048, n_heads=8, n_kv_heads=1, head_dim=256, d_ff=16384, vocab=256000)
TINY = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=1, head_dim=64, d_ff=512, vocab=1000)


def _check(rc):
    if rc != 0:
        raise B200Error(f"decoder error {rc}: {_lib.load().b200_decoder_last_error().decode()}")


def make_weights(cfg, seed=1005, device="cuda"):
    """int8 per-channel weights ~ clip(round(N(0,40)), +-127) with scales ~ U[1e-3,1e-2]; RMS-norm
    gains ~ N(1, 0.02). Generated on `device` with a seeded torch generator, layer by layer."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)

    def w(n, k):
        out = torch.empty((n, k), dtype=torch.int8, device=device)
        step = max(1, (1 << 26) // k)
        for r in range(0, n, step):
            rows = min(step, n - r)
            out[r:r + rows] = torch.randn((rows, k), generator=g, device=device).mul_(40).round_().clamp_(-127, 127)
        return out

    def s(n):
        return torch.rand(n, generator=g, device=device) * (1e-2 - 1e-3) + 1e-3

    def gain(n):
        return torch.randn(n, generator=g, device=device) * 0.02 + 1.0

    d, qd, kd, f = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["d_ff"]
    layers = []
    for _ in range(cfg["n_layers"]):
        layers.append(dict(wq=w(qd, d), wk=w(kd, d), wv=w(kd, d), wo=w(d, qd), wgate=w(f, d), wup=w(f, d),
                           wdown=w(d, f), sq=s(qd), sk=s(kd), sv=s(kd), so=s(d), sgate=s(f), sup=s(f), sdown=s(d),
                           norm1=gain(d), norm2=gain(d)))
    return dict(layers=layers, embed=w(cfg["vocab"], d), embed_scales=s(cfg["vocab"]), final_norm=gain(d))


def shard_weights(cfg, weights, tp_size, rank):
    """This rank's slices of the whole model's weights (tensors of make_weights' layout): q, gate and up by
    output rows, o and down by input columns, k/v by KV head (replicated when ranks share a head). The
    embedding table stays whole: the decoder takes its LM-head rows itself."""
    H, KVH, HD, F = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["d_ff"]
    if H % tp_size or F % tp_size or cfg["vocab"] % tp_size or (KVH % tp_size and tp_size % KVH):
        raise ValueError("heads, d_ff and vocab must divide by tp_size")
    hl, fl = H // tp_size, F // tp_size
    if KVH % tp_size == 0:
        kvl, kv0 = KVH // tp_size, rank * (KVH // tp_size)
    else:
        kvl, kv0 = 1, rank // (tp_size // KVH)
    q0, q1, k0, k1, f0, f1 = rank * hl * HD, (rank + 1) * hl * HD, kv0 * HD, (kv0 + kvl) * HD, rank * fl, (rank + 1) * fl
    layers = []
    for lw in weights["layers"]:
        layers.append({
            "wq": lw["wq"][q0:q1].contiguous(), "sq": lw["sq"][q0:q1].contiguous(),
            "wk": lw["wk"][k0:k1].contiguous(), "sk": lw["sk"][k0:k1].contiguous(),
            "wv": lw["wv"][k0:k1].contiguous(), "sv": lw["sv"][k0:k1].contiguous(),
            "wo": lw["wo"][:, q0:q1].contiguous(), "so": lw["so"],
            "wgate": lw["wgate"][f0:f1].contiguous(), "sgate": lw["sgate"][f0:f1].contiguous(),
            "wup": lw["wup"][f0:f1].contiguous(), "sup": lw["sup"][f0:f1].contiguous(),
            "wdown": lw["wdown"][:, f0:f1].contiguous(), "sdown": lw["sdown"],
            "norm1": lw["norm1"], "norm2": lw["norm2"]})
    return {"layers": layers, "embed": weights["embed"], "embed_scales": weights["embed_scales"],
            "final_norm": weights["final_norm"]}


class Decoder:
    def __init__(self, cfg, max_seq, max_batch, weights=None, kv_dtype="f16", rms_eps=1e-6, rope_base=10000.0,
                 seed=1005, device="cuda", keep_weights=False, tp_size=1, tp_rank=0):
        """cfg holds the whole model's sizes. With tp_size > 1 this is rank tp_rank's shard: `weights` (whole
        model, default: seeded random) is cut with shard_weights, and connect() must run before the first
        step."""
        self.lib = _lib.load()
        self.tp_size, self.tp_rank = tp_size, tp_rank
        self.cfg = dict(cfg)
        self.device = torch.device(device)
        c = _lib.DecoderConfig(
            n_layers=cfg["n_layers"], d_model=cfg["d_model"], n_heads=cfg["n_heads"], n_kv_heads=cfg["n_kv_heads"],
            head_dim=cfg["head_dim"], d_ff=cfg["d_ff"], vocab=cfg["vocab"], max_seq=max_seq, max_batch=max_batch,
            rms_eps=rms_eps, rope_base=rope_base, embed_scale=math.sqrt(cfg["d_model"]),
            kv_dtype=1 if kv_dtype == "i8" else 0, tp_size=tp_size, tp_rank=tp_rank)
        self.config_struct = c
        self.rms_eps, self.rope_base, self.max_seq, self.max_batch = rms_eps, rope_base, max_seq, max_batch
        self._batch = None
        self.handle = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            self.stream = torch.cuda.Stream()
            _check(self.lib.b200_decoder_create(ctypes.byref(c), ctypes.c_void_p(self.stream.cuda_stream),
                                                ctypes.byref(self.handle)))
            weights = weights or make_weights(cfg, seed, device)
            whole = weights
            if tp_size > 1:
                weights = shard_weights(cfg, whole, tp_size, tp_rank)
            for i, lw in enumerate(weights["layers"]):
                st = _lib.DecoderLayerWeights(**{k: lw[k].data_ptr() for k in lw})
                _check(self.lib.b200_decoder_set_layer(self.handle, i, ctypes.byref(st)))
            _check(self.lib.b200_decoder_set_embedding(self.handle, weights["embed"].data_ptr(),
                                                       weights["embed_scales"].data_ptr(),
                                                       weights["final_norm"].data_ptr()))
            torch.cuda.synchronize()
        self.weights = whole if keep_weights else None

    def connect(self, mode="peer", group=None):
        """Joins the tensor-parallel ranks of `group` (torch.distributed, any backend; group rank = tp_rank).
        'peer': the ranks swap the CUDA IPC handles of their exchange buffers and the consuming kernels
        read the peers' partial sums themselves; 'nccl': an NCCL communicator of the ranks' own."""
        import torch.distributed as dist
        if self.tp_size == 1:
            return
        with torch.cuda.device(self.device):
            if mode == "peer":
                buf = ctypes.create_string_buffer(64)
                _check(self.lib.b200_decoder_exchange_handle(self.handle, buf, 64))
                handles = [None] * self.tp_size
                dist.all_gather_object(handles, bytes(buf.raw), group=group)
                blob = b"".join(handles)
                _check(self.lib.b200_decoder_connect_peers(self.handle, blob, 64))
            elif mode == "nccl":
                ids = [None]
                if self.tp_rank == 0:
                    buf = ctypes.create_string_buffer(128)
                    _check(self.lib.b200_nccl_unique_id(buf, 128))
                    ids[0] = bytes(buf.raw)
                src = dist.get_global_rank(group, 0) if group is not None else 0
                dist.broadcast_object_list(ids, src=src, group=group)
                _check(self.lib.b200_decoder_init_nccl(self.handle, ids[0]))
            else:
                raise ValueError("mode must be 'peer' or 'nccl'")
            dist.barrier(group=group)

    def reset(self):
        _check(self.lib.b200_decoder_reset(self.handle))

    def set_positions(self, positions):
        pos = np.ascontiguousarray(positions, np.int32)
        _check(self.lib.b200_decoder_set_positions(self.handle, pos.ctypes.data_as(ctypes.c_void_p), pos.size))

    def step(self, tokens, want_logits=False):
        """tokens: host int32 array [batch] -> (next tokens [batch], logits or None)."""
        tok = np.ascontiguousarray(tokens, np.int32)
        nxt = np.empty_like(tok)
        logits = None
        with torch.cuda.device(self.device):
            if want_logits:
                # with tensor parallelism: this rank's columns [tp_rank * vocab / tp_size, ...)
                logits = torch.empty((tok.size, self.cfg["vocab"] // self.tp_size), dtype=torch.float32,
                                     device=self.device)
            _check(self.lib.b200_decoder_step(self.handle, tok.ctypes.data_as(ctypes.c_void_p), tok.size,
                                              nxt.ctypes.data_as(ctypes.c_void_p),
                                              None if logits is None else ctypes.c_void_p(logits.data_ptr())))
        return nxt, logits

    def prefill(self, tokens, seq=0):
        """Prompt pass of sequence `seq` over the host int32 array `tokens`: fills the sequence's cache
        behind what is already there and returns the first generated token (also kept on the device,
        where run(None, ...) picks it up)."""
        tok = np.ascontiguousarray(tokens, np.int32).reshape(-1)
        nxt = ctypes.c_int32()
        with torch.cuda.device(self.device):
            _check(self.lib.b200_decoder_prefill(self.handle, int(seq), tok.ctypes.data_as(ctypes.c_void_p), tok.size,
                                                 ctypes.byref(nxt)))
        return int(nxt.value)

    def run(self, first_tokens, steps, fetch=True, batch=None):
        """`steps` greedy steps on the device. first_tokens None: continue from the tokens the last step
        or prompt pass left there (give `batch` when no step has run yet)."""
        tok = None if first_tokens is None else np.ascontiguousarray(first_tokens, np.int32)
        batch = (batch or self._batch) if tok is None else tok.size
        self._batch = batch
        nxt = np.empty(batch, np.int32) if fetch else None
        with torch.cuda.device(self.device):
            _check(self.lib.b200_decoder_run(self.handle, None if tok is None else tok.ctypes.data_as(ctypes.c_void_p),
                                             batch, steps, None if nxt is None else nxt.ctypes.data_as(ctypes.c_void_p)))
        return nxt

    def profile_step(self, tokens):
        """One eager step with per-launch CUDA events: {'gemv','attention','glue'} -> (ms, launches)."""
        tok = np.ascontiguousarray(tokens, np.int32)
        ms = (ctypes.c_float * 3)()
        n = (ctypes.c_int * 3)()
        with torch.cuda.device(self.device):
            _check(self.lib.b200_decoder_profile_step(self.handle, tok.ctypes.data_as(ctypes.c_void_p), tok.size, ms, n))
        return {k: (ms[i], n[i]) for i, k in enumerate(("gemv", "attention", "glue"))}

    def time_gemv(self, batch, reps=20):
        """(ms, launches) of one step's projections alone, replayed as a CUDA graph (see the header)."""
        ms, n = ctypes.c_float(), ctypes.c_int()
        with torch.cuda.device(self.device):
            _check(self.lib.b200_decoder_time_gemv(self.handle, batch, reps, ctypes.byref(ms), ctypes.byref(n)))
        return ms.value, n.value

    @property
    def launches_per_step(self):
        return self.lib.b200_decoder_launches_per_step(self.handle)

    def weight_bytes_per_step(self):
        c = self.cfg
        qd, kd = c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"]
        per_layer = c["d_model"] * (qd + 2 * kd) + qd * c["d_model"] + 3 * c["d_model"] * c["d_ff"]
        return c["n_layers"] * per_layer + c["vocab"] * c["d_model"]

    def close(self):
        if self.handle:
            self.lib.b200_decoder_destroy(self.handle)
            self.handle = None
