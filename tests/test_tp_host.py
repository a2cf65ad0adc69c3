"""Tensor-parallel host logic on CPU: the shard plan, and two gloo ranks stepping oracle shards."""
import os
import socket
import subprocess
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
import tp_worker  # noqa: E402


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def run_ranks(args_per_rank, timeout=600):
    procs = [subprocess.Popen([sys.executable, os.path.join(HERE, "tp_worker.py")] + [str(a) for a in args],
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True) for args in args_per_rank]
    outs = []
    try:
        for p in procs:
            out, _ = p.communicate(timeout=timeout)
            outs.append(out)
    finally:
        for p in procs:
            if p.poll() is None:
                p.kill()
    for p, out in zip(procs, outs):
        assert p.returncode == 0, out[-4000:]


def test_shard_plan_matches_oracle_plan():
    """litert_b200.decoder.shard_weights (torch) cuts the same slices as the oracle's numpy plan."""
    from litert_b200 import decoder as dec
    import oracle
    hw = tp_worker.host_weights()
    tw = dict(layers=[{k: torch.from_numpy(v) for k, v in lw.items()} for lw in hw["layers"]])
    for k in ("embed", "embed_scales", "final_norm"):
        tw[k] = torch.from_numpy(hw[k])
    for tp in (2, 4):
        for r in range(tp):
            mine = dec.shard_weights(tp_worker.CFG, tw, tp, r)
            _, theirs, lm = oracle.shard_decoder(tp_worker.CFG, hw, tp, r)
            assert lm == (r * 1000 // tp, 1000 // tp)
            for a, b in zip(mine["layers"], theirs["layers"]):
                assert a.keys() == b.keys()
                for k in a:
                    assert np.array_equal(a[k].numpy(), b[k]), (tp, r, k)


def test_sharded_sum_equals_whole_projection():
    """Integer part of the input-sharded projection: the shards' dot products add up to the whole one."""
    rng = np.random.default_rng(0)
    w = rng.integers(-127, 128, (64, 256), dtype=np.int64)
    x = rng.integers(-128, 128, 256, dtype=np.int64)
    whole = w @ x
    for tp in (2, 4, 8):
        parts = [w[:, r * 256 // tp:(r + 1) * 256 // tp] @ x[r * 256 // tp:(r + 1) * 256 // tp] for r in range(tp)]
        assert np.array_equal(sum(parts), whole)


def test_two_gloo_ranks_equal_threaded_shards(tmp_path, oracle):
    """world_size 2 over gloo: each process steps one oracle shard, partial sums go through all_reduce,
    the token pick through all_gather. Must equal the same two shards stepped in one process."""
    port = free_port()
    run_ranks([("cpu", r, 2, port, tmp_path) for r in range(2)])
    got = [np.load(tmp_path / f"rank{r}.npz") for r in range(2)]
    ref = oracle.DecoderRefTP(tp_worker.CFG, tp_worker.host_weights(), 2, tp_worker.BATCH, tp_worker.MAX_SEQ)
    tok = tp_worker.first_tokens()
    for s in range(tp_worker.STEPS):
        tok, logits = ref.step(tok)
        both = np.concatenate([got[0]["logits"][s], got[1]["logits"][s]], axis=1)
        assert np.array_equal(both, logits), s
        assert np.array_equal(got[0]["tokens"][s], tok) and np.array_equal(got[1]["tokens"][s], tok)
    ref.close()
