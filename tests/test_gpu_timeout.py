"""A bounded device-side wait that runs out: the step reports B200_ERR_KERNEL_TIMEOUT instead of hanging,
and the decoder is usable again afterwards. The failure is made on purpose in the one allowed form: a
flag that nothing ever sets, waited for with a budget of two milliseconds. No fault, trap or unbounded
wait is involved and the context stays usable (which is what the test then checks)."""
import ctypes
import time

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _memcpy_h2d(dst_ptr, data):
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaMemcpy.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_size_t, ctypes.c_int]
    buf = np.ascontiguousarray(data)
    assert rt.cudaMemcpy(ctypes.c_void_p(dst_ptr), buf.ctypes.data_as(ctypes.c_void_p), buf.nbytes, 1) == 0


def test_a_peer_that_never_arrives_times_out_and_the_decoder_recovers():
    """Rank 0 of a two-rank tensor-parallel decoder whose peer never steps: rank 1's exchange buffer is a
    zeroed allocation on the same GPU, so the flag rank 0 waits for is never advanced."""
    from litert_b200 import _lib
    from litert_b200 import decoder as dec
    from litert_b200._lib import B200Error

    lib = _lib.load()
    cfg = dict(dec.TINY)
    d = dec.Decoder(cfg, max_seq=16, max_batch=2, weights=dec.make_weights(cfg, seed=4), tp_size=2, tp_rank=0)
    nbytes = lib.b200_decoder_exchange_bytes(d.handle)
    assert nbytes > 0
    absent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(None, absent_peer.data_ptr())
    assert lib.b200_decoder_connect_peer_pointers(d.handle, ptrs) == 0
    assert lib.b200_decoder_set_wait_budget(d.handle, 2_000_000) == 0  # 2 ms
    tok = np.asarray([3, 5], np.int32)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with pytest.raises(B200Error, match="wait ran out"):
        d.step(tok)
    assert time.perf_counter() - t0 < 5.0, "one budget, not one per exchange: later waits give up at once"
    # the context is alive and other work on the device is unaffected
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0
    # recovery: the step cleared the fault state itself; now the peer "arrives" for every later exchange
    # (its flag in rank 0's own exchange buffer jumps far ahead, its partial sums stay zero)
    own = lib.b200_decoder_exchange_buffer(d.handle)
    _memcpy_h2d(own + 8 * 1, np.asarray([1 << 62], np.uint64))
    d.reset()
    nxt, logits = d.step(tok, want_logits=True)
    assert torch.isfinite(logits).all()
    nxt2, _ = d.step(nxt)   # the graph path as well
    assert nxt2.shape == (2,)
    # an explicit clear is harmless on a healthy decoder
    assert lib.b200_decoder_clear_fault(d.handle) == 0
    d.step(nxt2)
    d.close()


def test_pushed_partials_that_never_arrive_time_out_too():
    """The same absent peer at widths where the decode-sized exchange is the pushed one (the attention-output and
    down projections run on the cluster kernel and send {value, epoch} messages; the norm stage polls its own
    memory): the messages of rank 1 never come, the poll gives up after its budget, the step reports the time-out
    and the context stays usable."""
    from litert_b200 import _lib
    from litert_b200 import decoder as dec
    from litert_b200._lib import B200Error

    lib = _lib.load()
    cfg = dict(n_layers=2, d_model=512, n_heads=4, n_kv_heads=1, head_dim=128, d_ff=1024, vocab=1000)
    d = dec.Decoder(cfg, max_seq=16, max_batch=2, weights=dec.make_weights(cfg, seed=5), tp_size=2, tp_rank=0)
    nbytes = lib.b200_decoder_exchange_bytes(d.handle)
    absent_peer = torch.zeros(nbytes, dtype=torch.uint8, device="cuda")
    ptrs = (ctypes.c_void_p * 2)(None, absent_peer.data_ptr())
    assert lib.b200_decoder_connect_peer_pointers(d.handle, ptrs) == 0
    assert lib.b200_decoder_set_wait_budget(d.handle, 2_000_000) == 0  # 2 ms
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    with pytest.raises(B200Error, match="wait ran out"):
        d.step(np.asarray([3, 5], np.int32))
    assert time.perf_counter() - t0 < 5.0
    assert float(torch.ones(8, device="cuda").sum().item()) == 8.0
    # rank 0 pushed its own partials into the absent peer's message area: proof that this path ran
    # (a flag handshake would have left one 8-byte flag there, the push two rows of 512 messages)
    area = absent_peer.cpu().numpy()
    assert np.count_nonzero(area) > 1000, "the cluster kernel's messages landed in the peer's buffer"
    d.close()


def test_status_word_of_the_op_level_workspace_can_be_cleared():
    """b200_clear_status after a recorded time-out: ops on the same workspace work again (the status word
    is written by hand here: the op-level kernels have no wait that a test could starve)."""
    from litert_b200 import _lib, ops, workloads
    from litert_b200._lib import B200Error

    lib = _lib.load()
    ws = ops.Workspace("cuda")
    _memcpy_h2d(ws.zero.data_ptr(), np.asarray([101], np.int32))
    with pytest.raises(B200Error):
        ws.check_status()
    assert lib.b200_clear_status(ctypes.c_void_p(ws.zero.data_ptr()), None) == 0
    ws.check_status()
    c = workloads.config2(3, 300, 700)
    dev = lambda a: torch.from_numpy(a).cuda()
    y = ops.fully_connected_hybrid(dev(c["x"]), ops.PackedInt8Weights(dev(c["w"])), dev(c["filter_scales"]), ws=ws)
    assert torch.isfinite(y).all()
    ws.check_status()
    # a shorter budget set through the workspace leaves results unchanged
    assert lib.b200_set_wait_budget(ctypes.c_void_p(ws.zero.data_ptr()), 50_000_000, None) == 0
    y2 = ops.fully_connected_hybrid(dev(c["x"]), ops.PackedInt8Weights(dev(c["w"])), dev(c["filter_scales"]), ws=ws)
    assert torch.equal(y, y2)
    ws.check_status()
