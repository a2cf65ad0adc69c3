"""Seeded synthetic inputs for the five benchmark configurations (numpy, host side).

There is no public dataset behind these: every tensor is drawn from a fixed seed with the shapes,
dtypes and value distributions the configurations name; random-init weights stand in for real ones.
"""
import numpy as np

SEEDS = {1: 1001, 2: 1002, 3: 1003, 4: 1004, 5: 1005}


def int8_weights(rng, n, k):
    """N(0,40) rounded and clipped to +-127."""
    out = np.empty((n, k), np.int8)
    step = max(1, (1 << 24) // max(k, 1))
    for r0 in range(0, n, step):
        r1 = min(n, r0 + step)
        out[r0:r1] = np.clip(np.rint(rng.standard_normal((r1 - r0, k), dtype=np.float32) * 40.0), -127, 127)
    return out


def config1(m=32, n=2048, k=2048, seed=SEEDS[1]):
    """Full-integer int8 FULLY_CONNECTED."""
    rng = np.random.default_rng(seed)
    return dict(
        x=rng.integers(-128, 128, (m, k), dtype=np.int64).astype(np.int8),
        w=int8_weights(rng, n, k),
        filter_scales=rng.uniform(1e-3, 1e-2, n).astype(np.float32),
        bias=rng.integers(-5000, 5001, n, dtype=np.int64).astype(np.int32),
        input_scale=np.float32(0.02), input_zp=-3, output_scale=np.float32(0.05), output_zp=0)


def config2(m, n=14336, k=4096, seed=SEEDS[2]):
    """Dynamic-range hybrid FULLY_CONNECTED, hidden -> FFN shape."""
    rng = np.random.default_rng(seed)
    w = int8_weights(rng, n, k)
    scales = rng.uniform(1e-3, 1e-2, n).astype(np.float32)
    x = rng.standard_normal((m, k), dtype=np.float32)
    return dict(x=x, w=w, filter_scales=scales)


def config3(m, n=16384, k=2048, blocksize=32, seed=SEEDS[3]):
    """Blockwise int4 weights, fp16 block scales."""
    rng = np.random.default_rng(seed)
    w = rng.integers(-8, 8, (n, k), dtype=np.int64).astype(np.int8)
    u = w.astype(np.uint8) & 0xF
    w4 = (u[:, 0::2] | (u[:, 1::2] << 4)).astype(np.uint8)
    scales = rng.uniform(1e-3, 2e-2, (n, k // blocksize)).astype(np.float16)
    x = rng.standard_normal((m, k), dtype=np.float32)
    return dict(x=x, w=w, w4=w4, scales=scales, blocksize=blocksize)


def config4(b=16, n=8, nkv=1, h=256, s_max=8192, min_len=128, seed=SEEDS[4]):
    """SDPA decode step: ragged lengths, fp16 q/k/v; int8 per-token-scaled variants included."""
    rng = np.random.default_rng(seed)
    lengths = rng.integers(min_len, s_max + 1, b, dtype=np.int64).astype(np.int32)
    q = rng.standard_normal((b, 1, n, h), dtype=np.float32).astype(np.float16)
    k = rng.standard_normal((b, s_max, nkv, h), dtype=np.float32).astype(np.float16)
    v = rng.standard_normal((b, s_max, nkv, h), dtype=np.float32).astype(np.float16)
    return dict(q=q, k=k, v=v, lengths=lengths, scale=1.0 / np.sqrt(h))


def quantize_kv_per_token(x):
    """Symmetric int8 per cached token and kv head: scale = max|row| / 127."""
    xf = x.astype(np.float32)
    amax = np.abs(xf).max(axis=-1)
    scale = np.where(amax > 0, amax / 127.0, 1.0).astype(np.float32)
    q = np.clip(np.rint(xf / scale[..., None]), -127, 127).astype(np.int8)
    return q, scale
