"""One tensor-parallel rank, run as a child process by the tensor-parallel tests.

  python tests/tp_worker.py gpu  <rank> <world> <port> <out_dir> <mode> <kv>   one GPU per rank (cuda:<rank>)
  python tests/tp_worker.py cpu  <rank> <world> <port> <out_dir>               CPU oracle shard over gloo

Each rank writes <out_dir>/rank<r>.npz with its next tokens and logits shard per step.
"""
import os
import sys

import numpy as np

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

CFG = dict(n_layers=2, d_model=256, n_heads=4, n_kv_heads=1, head_dim=64, d_ff=512, vocab=1000)
BATCH, STEPS, MAX_SEQ, SEED = 3, 5, 16, 11
PROMPT = 9


def host_weights(seed=SEED):
    """Whole-model weights as numpy, the same values on every rank and in the parent."""
    rng = np.random.default_rng(seed)
    c = CFG
    D, QD, KD, F, V = c["d_model"], c["n_heads"] * c["head_dim"], c["n_kv_heads"] * c["head_dim"], c["d_ff"], c["vocab"]

    def w(n, k):
        return np.clip(np.rint(rng.normal(0, 40, (n, k))), -127, 127).astype(np.int8)

    def s(n, k):
        return (rng.uniform(0.5, 1.5, n) / (40.0 * np.sqrt(k))).astype(np.float32)

    layers = []
    for _ in range(c["n_layers"]):
        layers.append(dict(wq=w(QD, D), sq=s(QD, D), wk=w(KD, D), sk=s(KD, D), wv=w(KD, D), sv=s(KD, D),
                           wo=w(D, QD), so=s(D, QD), wgate=w(F, D), sgate=s(F, D), wup=w(F, D), sup=s(F, D),
                           wdown=w(D, F), sdown=s(D, F),
                           norm1=rng.uniform(0.8, 1.2, D).astype(np.float32),
                           norm2=rng.uniform(0.8, 1.2, D).astype(np.float32)))
    return dict(layers=layers, embed=w(V, D), embed_scales=(rng.uniform(0.5, 1.5, V) / 40.0).astype(np.float32),
                final_norm=rng.uniform(0.8, 1.2, D).astype(np.float32))


def first_tokens():
    return np.random.default_rng(5).integers(0, CFG["vocab"], BATCH).astype(np.int32)


def init_group(rank, world, port):
    import torch.distributed as dist
    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    return dist


def run_gpu(rank, world, port, out_dir, mode, kv):
    import torch
    from litert_b200 import decoder as dec
    dist = init_group(rank, world, port)
    torch.cuda.set_device(rank)
    dev = f"cuda:{rank}"
    hw = host_weights()
    weights = dict(layers=[{k: torch.from_numpy(v).to(dev) for k, v in lw.items()} for lw in hw["layers"]])
    for k in ("embed", "embed_scales", "final_norm"):
        weights[k] = torch.from_numpy(hw[k]).to(dev)
    d = dec.Decoder(CFG, max_seq=MAX_SEQ, max_batch=4, weights=weights, kv_dtype=kv, device=dev, tp_size=world,
                    tp_rank=rank)
    d.connect(mode)
    tok = first_tokens()
    toks, logits = [], []
    for _ in range(STEPS):
        tok, lg = d.step(tok, want_logits=True)   # eager path (caller-owned logits)
        toks.append(tok.copy())
        logits.append(lg.cpu().numpy())
    # the captured-graph path must give the same continuation from the same start
    d.reset()
    dist.barrier()
    replay = d.run(first_tokens(), STEPS)
    # prompt pass against stepping the same prompts: sequences 0 and 1, PROMPT tokens each
    extra = {}
    prompts = np.random.default_rng(9).integers(0, CFG["vocab"], (2, PROMPT)).astype(np.int32)
    d.reset()
    dist.barrier()
    for t in range(PROMPT):
        stepped_tok, stepped_logits = d.step(prompts[:, t], want_logits=True)
    _, stepped_next = d.step(stepped_tok, want_logits=True)
    d.reset()
    dist.barrier()
    if mode == "nccl":
        first = np.array([d.prefill(prompts[b], seq=b) for b in range(2)], np.int32)
        _, filled_next = d.step(stepped_tok, want_logits=True)
        extra = dict(stepped_tok=stepped_tok, stepped_logits=stepped_logits.cpu().numpy(), prefill_tok=first,
                     stepped_next=stepped_next.cpu().numpy(), filled_next=filled_next.cpu().numpy())
    else:
        # the peer exchange is a decode-step mechanism: a prompt pass needs the all-reduce
        from litert_b200._lib import B200Error
        try:
            d.prefill(prompts[0], seq=0)
            extra = dict(prefill_refused=np.array(0))
        except B200Error:
            extra = dict(prefill_refused=np.array(1))
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), tokens=np.stack(toks), logits=np.stack(logits), replay=replay, **extra)
    dist.barrier()
    d.close()
    dist.destroy_process_group()


def run_cpu(rank, world, port, out_dir):
    import torch
    import oracle
    dist = init_group(rank, world, port)
    hw = host_weights()
    scfg, sw, lm = oracle.shard_decoder(CFG, hw, world, rank)

    def reduce(arr):
        t = torch.from_numpy(arr)
        dist.all_reduce(t)   # in place: t shares arr's memory

    ref = oracle.DecoderRef(scfg, sw, BATCH, MAX_SEQ, reduce=reduce, lm_rows=lm)
    tok = first_tokens()
    toks, logits = [], []
    for _ in range(STEPS):
        nxt, lg = ref.step(tok)
        # winner over the ranks' vocabulary shards: larger value, then lower index
        best_val = torch.from_numpy(lg.max(axis=1).copy())
        cand = [None] * world
        dist.all_gather_object(cand, (best_val.numpy(), nxt))
        vals = np.stack([c[0] for c in cand])
        idxs = np.stack([c[1] for c in cand])
        pick = np.argmax(vals, axis=0)   # first maximum = lowest rank = lowest index
        tok = idxs[pick, np.arange(BATCH)].astype(np.int32)
        toks.append(tok.copy())
        logits.append(lg)
    np.savez(os.path.join(out_dir, f"rank{rank}.npz"), tokens=np.stack(toks), logits=np.stack(logits))
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    kind, rank, world, port, out_dir = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4]), sys.argv[5]
    if kind == "gpu":
        run_gpu(rank, world, port, out_dir, sys.argv[6], sys.argv[7])
    else:
        run_cpu(rank, world, port, out_dir)
