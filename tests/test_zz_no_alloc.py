"""The allocation-free attention entry point (b200_sdpa_decode_static) against the regular one.

Some users of this library cannot call cudaMalloc where they call us: a serving loop that froze
its allocator after start-up, a plugin inside a host with a fixed memory budget, code that is being
recorded for replay. They cannot hand b200_sdpa_decode the workspace it wants, so the library also
offers a variant whose workspace is a built-in device array. This test calls that variant through
the C ABI twice in a row on different inputs (the array keeps the previous call's contents, so the
second call shows that nothing stale leaks into a result) and requires exactly the output of the
regular entry point, which runs the same kernels. It also checks that an over-sized shape is
refused with a clear error instead of overrunning the array.

Collected last on purpose (file name): a failure here must not hide any other test's result.
"""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(lib, q, k, v, lengths, scale, k_scale=None, v_scale=None, mask=None, out=None):
    out = torch.empty_like(q) if out is None else out
    b, _, n, h = q.shape
    s_max, nkv = k.shape[1], k.shape[2]
    dt = {torch.float16: 0, torch.int8: 1, torch.float32: 2}
    ptr = lambda t: None if t is None else t.data_ptr()
    rc = lib.b200_sdpa_decode_static(q.data_ptr(), k.data_ptr(), v.data_ptr(), ptr(k_scale), ptr(v_scale), ptr(lengths),
                                     ptr(mask), out.data_ptr(), b, n, nkv, h, s_max, dt[q.dtype], dt[k.dtype],
                                     float(scale), 0.0, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


def test_static_workspace_variant_matches_regular_entry_point_twice():
    from litert_b200 import _lib, ops, workloads

    lib = _lib.load()
    ws = ops.Workspace("cuda")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    for call, (seed, b, s_max) in enumerate([(41, 4, 2048), (42, 3, 1500)]):
        c = workloads.config4(b=b, s_max=s_max, min_len=1, seed=seed)
        q, k, v, lengths = dev(c["q"]), dev(c["k"]), dev(c["v"]), dev(c["lengths"])
        want = ops.sdpa_decode(q, k, v, lengths, scale=c["scale"], ws=ws)
        rc, got = _call_static(lib, q, k, v, lengths, c["scale"])
        assert rc == 0, lib.b200_sdpa_static_last_error().decode()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}: outputs differ"
        assert torch.isfinite(got.float()).all()


def test_static_workspace_variant_allocates_nothing_and_covers_int8_caches_and_masks():
    """No device memory may be allocated by the call itself: neither through torch's allocator nor behind
    its back (free device memory as the driver reports it stays where it was). Also the int8 cache with
    per-token scales, and float32 tensors with the reference's additive mask."""
    from litert_b200 import _lib, ops, workloads

    lib = _lib.load()
    ws = ops.Workspace("cuda")
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    c = workloads.config4(b=3, s_max=1024, min_len=1, seed=43)
    k8, ks = workloads.quantize_kv_per_token(c["k"])
    v8, vs = workloads.quantize_kv_per_token(c["v"])
    q, k, v, ksc, vsc, lengths = dev(c["q"]), dev(k8), dev(v8), dev(ks), dev(vs), dev(c["lengths"])
    want = ops.sdpa_decode(q, k, v, lengths, scale=c["scale"], k_scale=ksc, v_scale=vsc, ws=ws)
    out = torch.empty_like(q)
    rc, _ = _call_static(lib, q, k, v, lengths, c["scale"], ksc, vsc, out=out)  # first call on this device: set-up
    assert rc == 0, lib.b200_sdpa_static_last_error().decode()
    torch.cuda.synchronize()
    before_torch, before_free = torch.cuda.memory_allocated(), torch.cuda.mem_get_info()[0]
    for _ in range(2):
        rc, _ = _call_static(lib, q, k, v, lengths, c["scale"], ksc, vsc, out=out)
        assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before_torch
    assert torch.cuda.mem_get_info()[0] == before_free, "free device memory changed across the calls"
    assert torch.equal(out, want)
    # float32 tensors with the additive mask of the reference op
    rng = np.random.default_rng(44)
    b, n, nkv, h, s = 2, 8, 1, 256, 600
    qf = rng.standard_normal((b, 1, n, h)).astype(np.float32)
    kf = rng.standard_normal((b, s, nkv, h)).astype(np.float32)
    vf = rng.standard_normal((b, s, nkv, h)).astype(np.float32)
    mask = np.where(np.arange(s)[None, None, None, :] < np.asarray([590, 17])[:, None, None, None], 0.0, -1e30).astype(np.float32)
    want = ops.sdpa_decode(dev(qf), dev(kf), dev(vf), None, dev(mask), ws=ws)
    rc, got = _call_static(lib, dev(qf), dev(kf), dev(vf), None, 0.0, mask=dev(mask))
    assert rc == 0, lib.b200_sdpa_static_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(got, want)


def test_static_workspace_variant_rejects_shapes_beyond_its_limit():
    from litert_b200 import _lib

    lib = _lib.load()
    limit = lib.b200_sdpa_static_workspace_limit()
    assert limit == 8 << 20
    b, n, h, s_max = 64, 8, 256, 8192
    assert lib.b200_sdpa_workspace_bytes(b, n, 8, h, s_max) > limit
    x = torch.zeros(16, device="cuda")  # never dereferenced: the size check comes first
    rc = lib.b200_sdpa_decode_static(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, None, None, x.data_ptr(), b,
                                     n, 8, h, s_max, 0, 0, 0.0, 0.0, None)
    assert rc == 4  # B200_ERR_UNSUPPORTED
    assert b"built-in one holds" in lib.b200_sdpa_static_last_error()
