"""Run one named workload of the hot path a few times on cuda:0 and exit.

This is the command line that profiler captures are taken on (one kernel family, few launches, a few GB at
most on the device), and a quick way to exercise a single op from a shell:

    python -m litert_b200.run_case fc_hybrid --m 1 --n 14336 --k 4096 --reps 6
    python -m litert_b200.run_case fc_int8   --m 512 --n 2048 --k 2048
    python -m litert_b200.run_case fc_w4     --m 1
    python -m litert_b200.run_case sdpa      --kv f16
    python -m litert_b200.run_case decode    --batch 1 --context 1024 --steps 3
    python -m litert_b200.run_case prefill   --context 1024 --layers 2

Every case prints one line with the shapes it ran and "ok".
"""
import argparse
import sys

import numpy as np
import torch

from . import decoder as dec
from . import ops, workloads


def _dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def case_fc_hybrid(a):
    c = workloads.config2(a.m, n=a.n, k=a.k)
    ws = ops.Workspace("cuda", 64 << 20)
    # three copies of the weights, used in turn, so that no launch finds its weights in L2
    wps = [ops.PackedInt8Weights(_dev(c["w"])) for _ in range(3)]
    x, fs = _dev(c["x"]), _dev(c["filter_scales"])
    out = torch.empty((a.m, a.n), device="cuda")
    for i in range(a.reps):
        ops.fully_connected_hybrid(x, wps[i % 3], fs, ws=ws, out=out)
    return f"fc_hybrid m={a.m} n={a.n} k={a.k} reps={a.reps}"


def _quantize_multipliers(real):
    """Q31 significand and power-of-two shift of each real multiplier (the decomposition
    tflite/kernels/internal/quantization_util.cc:53-112 performs at Prepare time)."""
    frac, shift = np.frexp(np.asarray(real, np.float64))
    q = np.rint(frac * (1 << 31)).astype(np.int64)
    shift = shift.astype(np.int64)
    bump = q == (1 << 31)
    q[bump] //= 2
    shift[bump] += 1
    q[shift < -31] = 0
    shift[shift < -31] = 0
    return q.astype(np.int32), shift.astype(np.int32)


def case_fc_int8(a):
    c = workloads.config1(m=a.m, n=a.n, k=a.k)
    ws = ops.Workspace("cuda", 64 << 20)
    wps = [ops.PackedInt8Weights(_dev(c["w"])) for _ in range(3)]
    x, bias = _dev(c["x"]), _dev(c["bias"])
    real = np.float64(c["input_scale"]) * c["filter_scales"].astype(np.float64) / np.float64(c["output_scale"])
    mult, shift = (_dev(t) for t in _quantize_multipliers(real))
    for i in range(a.reps):
        ops.fully_connected_int8(x, wps[i % 3], bias, c["input_zp"], c["output_zp"], mult, shift, ws=ws)
    return f"fc_int8 m={a.m} n={a.n} k={a.k} reps={a.reps}"


def case_fc_w4(a):
    c = workloads.config3(a.m)
    ws = ops.Workspace("cuda", 64 << 20)
    wps = [ops.PackedInt4Weights(_dev(c["w4"]), _dev(c["scales"]), c["blocksize"]) for _ in range(3)]
    x = _dev(c["x"])
    for i in range(a.reps):
        ops.fully_connected_blockwise4(x, wps[i % 3], ws=ws)
    return f"fc_w4 m={a.m} n={wps[0].n} k={wps[0].k} reps={a.reps}"


def case_sdpa(a):
    c = workloads.config4()
    ws = ops.Workspace("cuda", 64 << 20)
    q, L = _dev(c["q"]), _dev(c["lengths"])
    if a.kv == "i8":
        k8, ks = workloads.quantize_kv_per_token(c["k"])
        v8, vs = workloads.quantize_kv_per_token(c["v"])
        k, v, ksc, vsc = _dev(k8), _dev(v8), _dev(ks), _dev(vs)
    else:
        k, v, ksc, vsc = _dev(c["k"]), _dev(c["v"]), None, None
    for _ in range(a.reps):
        ops.sdpa_decode(q, k, v, L, scale=c["scale"], k_scale=ksc, v_scale=vsc, ws=ws)
    return f"sdpa kv={a.kv} b=16 n=8 nkv=1 h=256 s_max=8192 reps={a.reps}"


def case_decode(a):
    cfg = dict(dec.GEMMA_2B if a.model == "gemma2b" else dec.TINY)
    d = dec.Decoder(cfg, max_seq=a.context + a.steps + 8, max_batch=a.batch, kv_dtype=a.kv)
    d.set_positions(np.full(a.batch, a.context, np.int32))
    tok = np.arange(a.batch, dtype=np.int32) + 5
    for _ in range(a.steps):
        tok, _ = d.step(tok)
    return f"decode model={a.model} batch={a.batch} context={a.context} steps={a.steps} launches/step={d.launches_per_step}"


def case_prefill(a):
    cfg = dict(dec.GEMMA_2B if a.model == "gemma2b" else dec.TINY)
    if a.layers:
        cfg["n_layers"] = a.layers
    d = dec.Decoder(cfg, max_seq=a.context + 8, max_batch=1, kv_dtype=a.kv)
    prompt = np.random.default_rng(3).integers(0, cfg["vocab"], a.context).astype(np.int32)
    for _ in range(a.reps):
        d.reset()
        d.prefill(prompt)
    return f"prefill model={a.model} layers={cfg['n_layers']} prompt={a.context} reps={a.reps}"


CASES = {"fc_hybrid": case_fc_hybrid, "fc_int8": case_fc_int8, "fc_w4": case_fc_w4, "sdpa": case_sdpa,
         "decode": case_decode, "prefill": case_prefill}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("case", choices=sorted(CASES))
    ap.add_argument("--m", type=int, default=1)
    ap.add_argument("--n", type=int, default=None)
    ap.add_argument("--k", type=int, default=None)
    ap.add_argument("--reps", type=int, default=6)
    ap.add_argument("--kv", default="f16", choices=["f16", "i8"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=1024)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--model", default="gemma2b", choices=["gemma2b", "tiny"])
    ap.add_argument("--layers", type=int, default=0, help="prefill: layer count override (0 = the model's)")
    a = ap.parse_args(argv)
    default_nk = {"fc_int8": (2048, 2048)}.get(a.case, (14336, 4096))
    a.n = a.n or default_nk[0]
    a.k = a.k or default_nk[1]
    if not torch.cuda.is_available():
        print("run_case needs a CUDA device", file=sys.stderr)
        return 2
    msg = CASES[a.case](a)
    torch.cuda.synchronize()
    print(msg, "ok")
    return 0


if __name__ == "__main__":
    sys.exit(main())
