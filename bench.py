#!/usr/bin/env python
"""Decode benchmark: tokens/s of a Gemma-2B-shaped int8 (dynamic-range) decoder, with the HBM
roofline of its dominant kernel (the streamed int8 GEMV), a parity record against the CPU graph on the
same weights, the CPU baseline beside it, and one timed record per single-op configuration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--context C] [--impl ours|reference]

One "step" is one decode step (one new token per sequence) over a KV cache that already holds
`context` tokens. All inputs are synthetic: seeded random-init weights of the named architecture and
random token ids. With --gpus N > 1 (launched under torchrun, one rank per GPU) every rank decodes
its own batch on its own replica (independent invocations partitioned across GPUs, no data-path
collective): weak scaling, aggregate tokens/s; the same batch is also run tensor-parallel over all
ranks and reported with its strong-scaling efficiency.

--impl reference times the CPU implementation of the same graph (the oracle's vectorised,
multi-threaded restatement of the reference kernels; the reference's own ruy/XNNPACK kernels cannot
be built offline) on the host cores of the box, at the same context depth.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "decode tokens/s (Gemma-2B-shaped int8) + GEMV HBM GB/s vs peak"
DTYPE = "int8 weights x int8 dynamically quantized activations, int32 accumulate, fp32 outputs"


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--context", type=int, default=1024, help="tokens already in the KV cache when timing starts")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--model", default="gemma2b", choices=["gemma2b", "tiny"])
    ap.add_argument("--kv", default="f16", choices=["f16", "i8"])
    ap.add_argument("--cpu-steps", type=int, default=6, help="decode steps of the CPU baseline sample")
    ap.add_argument("--side-batch", type=int, default=32,
                    help="also time this batch size (reported beside the headline; 0 = skip)")
    ap.add_argument("--tp", default="both", choices=["both", "peer", "nccl", "off"],
                    help="with --gpus > 1 also time ONE batch run tensor-parallel over all ranks")
    ap.add_argument("--configs", default="on", choices=["on", "off"],
                    help="one timed record per single-op configuration (1-4), at --gpus 1")
    return ap.parse_args()


def model_config(name):
    from litert_b200 import decoder as dec

    return dict(dec.GEMMA_2B if name == "gemma2b" else dec.TINY)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
            return p.get("hbm_gbs"), p.get("bf16_tflops"), "measured"
    return 6650.0, 1590.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons, sampled while the timed region runs."""

    def __init__(self, gpu_index):
        self.samples = []
        self.proc = None
        self.gpu_index = gpu_index

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "25"], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            # nvidia-smi needs a moment to come up: wait for its first line so that short timed regions are covered
            t_end = time.time() + 5.0
            while not self.samples and time.time() < t_end:
                time.sleep(0.01)
            self.samples.clear()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for s in self.samples:
            parts = [p.strip() for p in s.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------- CPU arm
def host_weights(cfg, seed=1005):
    """The same distributions as litert_b200.decoder.make_weights, drawn on the host (used when no GPU
    arm runs in this process: --impl reference)."""
    import torch

    g = torch.Generator()
    g.manual_seed(seed)

    def w(n, k):
        out = torch.empty((n, k), dtype=torch.int8)
        step = max(1, (1 << 24) // k)
        for r in range(0, n, step):
            rows = min(step, n - r)
            out[r:r + rows] = torch.randn((rows, k), generator=g).mul_(40).round_().clamp_(-127, 127)
        return out.numpy()

    def s(n):
        return (torch.rand(n, generator=g) * (1e-2 - 1e-3) + 1e-3).numpy()

    def gain(n):
        return (torch.randn(n, generator=g) * 0.02 + 1.0).numpy()

    d, qd, kd, f = cfg["d_model"], cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"], cfg["d_ff"]
    layers = [dict(wq=w(qd, d), wk=w(kd, d), wv=w(kd, d), wo=w(d, qd), wgate=w(f, d), wup=w(f, d), wdown=w(d, f),
                   sq=s(qd), sk=s(kd), sv=s(kd), so=s(d), sgate=s(f), sup=s(f), sdown=s(d), norm1=gain(d),
                   norm2=gain(d)) for _ in range(cfg["n_layers"])]
    return dict(layers=layers, embed=w(cfg["vocab"], d), embed_scales=s(cfg["vocab"]), final_norm=gain(d))


def to_host(weights):
    out = dict(layers=[{k: v.cpu().numpy() for k, v in lw.items()} for lw in weights["layers"]])
    for k in ("embed", "embed_scales", "final_norm"):
        out[k] = weights[k].cpu().numpy()
    return out


def cpu_decode_rate(cfg, weights, batch, context, steps, threads=None, seed=1005):
    """tokens/s of the CPU graph at `context` cached tokens per sequence (the cache rows hold zeros: the
    work does not depend on their values). threads None = all host threads."""
    import oracle

    oracle.build()
    fast = oracle.fast()
    all_threads = fast.orcf_num_threads()
    if threads:
        fast.orcf_set_num_threads(int(threads))
    try:
        ref = oracle.DecoderRef(cfg, weights, batch, context + steps + 4, fast=True)
        ref.set_lengths(np.full(batch, context, np.int32))
        tok = np.random.default_rng(seed).integers(0, cfg["vocab"], batch).astype(np.int32)
        tok, _ = ref.step(tok, want_logits=False)  # warm-up: page the weights in
        t0 = time.perf_counter()
        for _ in range(steps):
            tok, _ = ref.step(tok, want_logits=False)
        dt = time.perf_counter() - t0
        ref.close()
    finally:
        fast.orcf_set_num_threads(all_threads)
    return batch * steps / dt, dt / steps * 1e3, (int(threads) if threads else all_threads)


def cpu_baseline_record(cfg, weights, args):
    steps = max(1, args.cpu_steps)
    tps, ms, cores = cpu_decode_rate(cfg, weights, args.batch, args.context, steps)
    one_steps = max(1, min(2, steps))
    tps1, ms1, _ = cpu_decode_rate(cfg, weights, args.batch, args.context, one_steps, threads=1)
    return {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "ms_per_step": ms,
            "sample": f"{steps} decode steps after 1 warm-up, batch {args.batch}, {args.context} cached tokens per sequence, "
                      f"all {cores} host threads (vectorised restatement of the reference kernels; ruy / XNNPACK "
                      "cannot be built offline)",
            "one_thread": {"value": tps1, "unit": "tokens/s", "cores": 1, "ms_per_step": ms1, "steps": one_steps,
                           "note": "the reference's default thread count (kDefaultNumThreadpoolThreads = 1) and "
                                   "the only mode of its hybrid kernel"}}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = model_config(args.model)
    steps = max(1, min(args.steps, args.cpu_steps))
    weights = host_weights(cfg)
    tps, ms, cores = cpu_decode_rate(cfg, weights, args.batch, args.context, steps)
    sample = (f"{steps} decode steps after 1 warm-up, batch {args.batch}, {args.context} cached tokens per sequence "
              f"(the {weight_bytes(cfg) / 1e9:.2f} GB of weights per step dominate), all {cores} host threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": 1, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": DTYPE, "data": "synthetic", "config": workload_config(args, cfg),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the CPU arm times a bounded sample (its step costs the same at every step of the run: the weights "
                "dominate), the device arm the requested number of steps; both at the same context depth",
    }
    emit(line)


# DRAM bytes moved per algorithmic byte by the GEMV kernels, from ncu captures of single launches
# (dram__bytes_read.sum + dram__bytes_write.sum over the launch's algorithmic bytes): 1.002 for
# fc_umma_kernel on [14336, 4096] and 1.008 for fc_cluster_kernel on [2048, 16384]; the summaries
# are profiles/fc_umma_kernel_hybrid_14336x4096_m1.md and profiles/fc_cluster_kernel_hybrid_2048x16384_m1.md.
# A whole step's 2.5 GB cannot be captured under the profiler's size rule, so the per-launch traffic
# reported here is this ratio times the launch's algorithmic bytes (traffic grows with the weights).
NCU_TRAFFIC_PER_ALGORITHMIC_BYTE = 1.004


def weight_bytes(cfg):
    qd, kd = cfg["n_heads"] * cfg["head_dim"], cfg["n_kv_heads"] * cfg["head_dim"]
    per_layer = cfg["d_model"] * (qd + 2 * kd) + qd * cfg["d_model"] + 3 * cfg["d_model"] * cfg["d_ff"]
    return cfg["n_layers"] * per_layer + cfg["vocab"] * cfg["d_model"]


def workload_config(args, cfg):
    return {"workload": f"config 5: Gemma-2B-shaped decoder, decode step, batch {args.batch} per GPU, "
                        f"{args.context}-token prompt pass then decode" if args.model == "gemma2b" else f"tiny decoder, batch {args.batch}",
            "layers": cfg["n_layers"], "d_model": cfg["d_model"], "heads": cfg["n_heads"], "kv_heads": cfg["n_kv_heads"],
            "head_dim": cfg["head_dim"], "d_ff": cfg["d_ff"], "vocab": cfg["vocab"], "batch_per_gpu": args.batch,
            "context": args.context, "kv_cache": args.kv, "parallelism": f"replica x{args.gpus} (independent batches)",
            "l2": "inputs larger than L2: every step streams the full weight set (2.5 GB >> 126 MB)"}


# ------------------------------------------------------------------------------------------- parity
def parity_record(cfg, d, host, kv):
    """The device decoder against the CPU graph on the SAME weights, outside every timed region: a
    16-token prompt through the prompt pass, then two decode steps compared on their logits. The CPU
    graph keeps its cache rounded as the device does; `cpu_self_rel_l2` is the same CPU graph against
    itself with a float32 cache, i.e. how far two correct evaluations of this random-init graph drift
    apart from one rounding per cached value (the attention softmax is nearly a hard maximum)."""
    import oracle

    mode = 1 if kv == "f16" else 2
    ref = oracle.DecoderRef(cfg, host, 1, 32, fast=True, kv_mode=mode)
    ref32 = oracle.DecoderRef(cfg, host, 1, 32, fast=True, kv_mode=0)
    rng = np.random.default_rng(77)
    prompt = rng.integers(0, cfg["vocab"], 16).astype(np.int32)
    for t in range(prompt.size):
        nxt_r, _ = ref.step(prompt[t:t + 1], want_logits=False)
        ref32.step(prompt[t:t + 1], want_logits=False)
    d.reset()
    first = d.prefill(prompt, seq=0)
    tok = nxt_r
    errs, selfs, equal, steps = [], [], int(first == int(nxt_r[0])), 2
    for _ in range(steps):
        nxt_g, lg = d.step(tok, want_logits=True)
        nxt_r, lr = ref.step(tok, want_logits=True)
        _, ls = ref32.step(tok, want_logits=True)
        g = lg.cpu().numpy()
        errs.append(float(np.linalg.norm(g - lr) / np.linalg.norm(lr)))
        selfs.append(float(np.linalg.norm(ls - lr) / np.linalg.norm(lr)))
        equal += int(nxt_g[0] == nxt_r[0])
        tok = nxt_r
    ref.close()
    ref32.close()
    return {"checked": True, "rel_l2": max(errs), "cpu_self_rel_l2": max(selfs), "tokens_equal": equal,
            "tokens_compared": steps + 1, "against": "CPU restatement of the graph (oracle) on the same weights, "
            "16-token prompt pass + 2 decode steps, logits over the whole vocabulary",
            "per_kernel": "bit-exact / 1-LSB parity of every kernel at these widths: tests/test_gpu_glue.py"}


# ------------------------------------------------------------------------------------------- the plugin, end to end
def plugin_decode_e2e(cfg, host, args, invokes):
    """The same decode step through the reference-facing boundary: the Gemma-shaped graph a converter would
    emit (tests/minirt/decoder_graph.py: EMBEDDING_LOOKUP, odml.rms_norm, hybrid FULLY_CONNECTED, rotary
    embedding out of SLICE / MUL / CONCATENATION / ADD, odml.update_kv_cache, the attention composite, GELU,
    residual ADDs, LM head, ARG_MAX) handed to tflite_plugin_create_delegate, one partition, and invoked with
    HOST tensors: every step copies the token id, the position, the cos / sin rows and the mask to the device and
    the picked token back, inside the timed region. The cache holds `context` slots of zeros plus the steps'
    own rows (the graph attends over all its slots through the mask, so the work does not depend on what the
    earlier slots hold)."""
    from tests import minirt
    from tests.minirt.decoder_graph import DecoderGraph

    S = args.context + invokes + 8
    rt, d = minirt.MiniRuntime(), minirt.Delegate()
    g = DecoderGraph(rt, cfg, host, 1, S, want_logits=False)
    nodes = rt.plan_size
    if rt.apply(d) != 0 or rt.partitions != 1 or rt.cpu_nodes != 0:
        return {"error": f"graph not delegated as one partition: {rt.error[:200]}"}
    tok = np.asarray([17], np.int32)
    pos = args.context
    for _ in range(4):  # warm-up: the first invocation sets kernels up, the second records the CUDA graph
        g.feed(tok, pos)
        if rt.invoke() != 0:
            return {"error": rt.error[:200]}
        tok = rt.view(g.tokens).copy()
        pos += 1
    t0 = time.perf_counter()
    for _ in range(invokes - 4):
        g.feed(tok, pos)
        rt.invoke()
        tok = rt.view(g.tokens).copy()
        pos += 1
    dt = time.perf_counter() - t0
    n = invokes - 4
    rt.close()
    d.close()
    H = cfg["head_dim"]
    return {"value": n / dt, "unit": "tokens/s", "ms_per_step": dt / n * 1e3, "steps": n, "graph_nodes": nodes,
            "partitions": 1, "cpu_nodes": 0, "h2d_bytes_per_step": 4 + 8 + 2 * 4 * H + 4 * S, "d2h_bytes_per_step": 4,
            "through": "tflite_plugin_create_delegate -> Prepare -> invoke on the Gemma-shaped graph (mini runtime), "
                       "host tensors in and out every step, float32 kv cache as the reference's odml.update_kv_cache keeps it"}


# ------------------------------------------------------------------------------------------- single-op configurations
def _median_launch_us(fn, launches=50, repeats=5, warm=3):
    """Median over `repeats` of the device time per launch of `launches` back-to-back calls of fn(i),
    replayed as one CUDA graph (the Python call overhead would otherwise hide kernels of a few us)."""
    import torch

    s = torch.cuda.Stream()
    times = []
    with torch.cuda.stream(s):
        for i in range(warm):
            fn(i)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for i in range(launches):
                fn(i)
        g.replay()
        s.synchronize()
        for _ in range(repeats):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(s)
            g.replay()
            e1.record(s)
            s.synchronize()
            times.append(e0.elapsed_time(e1) * 1e3 / launches)
    return float(np.median(times))


def _delegate_invoke_us(build_graph, invokes=10):
    """The same op end to end through the plugin: tflite_plugin_create_delegate -> Prepare -> invoke with
    HOST tensors (host-to-device copy of the inputs, launches, device-to-host copy of the outputs and a
    stream synchronisation inside every invoke), driven by the mini runtime."""
    try:
        from tests import minirt
    except Exception as exc:  # headers and prebuilt runtime both absent
        return None, f"mini runtime unavailable: {exc}"
    try:
        m, d = minirt.MiniRuntime(), minirt.Delegate()
        build_graph(m, minirt)
        if m.apply(d) != 0 or m.partitions != 1 or m.cpu_nodes != 0:
            return None, f"not delegated: {m.error}"
        for _ in range(2):
            if m.invoke() != 0:
                return None, m.error
        t0 = time.perf_counter()
        for _ in range(invokes):
            m.invoke()
        us = (time.perf_counter() - t0) / invokes * 1e6
        m.close()
        d.close()
        return us, None
    except Exception as exc:
        return None, str(exc)[:200]


def config_records(hbm_peak, i8_peak_ops):
    """One record per single-op configuration and row count: device time of the op through the C ABI
    (median of 5 x 50 graph-replayed launches, distinct weight copies used in turn so that no launch
    finds its weights in L2), its roofline fraction, and the same op through the delegate with host
    tensors."""
    import torch

    from litert_b200 import ops, run_case, workloads

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    out = []

    def record(cfg_no, label, m, us, alg_bytes, op_count, bound, copies, e2e, extra=None):
        gbs = alg_bytes / (us * 1e-6) / 1e9
        pops = op_count / (us * 1e-6) / 1e15
        r = {"config": cfg_no, "op": label, "m": m, "us": us, "algorithmic_bytes": alg_bytes, "ops": op_count,
             "gb_per_s": gbs, "pop_per_s": pops, "bound": bound, "frac_of_hbm_peak": gbs / hbm_peak,
             "frac_of_int8_tensor_peak": (op_count / (us * 1e-6)) / i8_peak_ops if i8_peak_ops else None,
             "frac": gbs / hbm_peak if bound == "hbm" else ((op_count / (us * 1e-6)) / i8_peak_ops if i8_peak_ops else None),
             "weight_copies": copies, "timing": "median of 5 x 50 graph-replayed launches after 3 warm-ups",
             "delegate_invoke_us": e2e[0], "delegate_invoke_note": e2e[1] or
             "host tensors in and out through tflite_plugin_create_delegate -> Prepare -> invoke (mini runtime)"}
        if extra:
            r.update(extra)
        out.append(r)

    ws = ops.Workspace("cuda", 64 << 20)
    # ---- config 1: full-integer int8 [32, 2048] x [2048, 2048]: 64 weight copies (256 MB > L2)
    c = workloads.config1()
    real = np.float64(c["input_scale"]) * c["filter_scales"].astype(np.float64) / np.float64(c["output_scale"])
    mult, shift = (dev(t) for t in run_case._quantize_multipliers(real))
    wps = [ops.PackedInt8Weights(dev(c["w"])) for _ in range(64)]
    x, bias = dev(c["x"]), dev(c["bias"])
    y = torch.empty((32, 2048), dtype=torch.int8, device="cuda")
    us = _median_launch_us(lambda i: ops.fully_connected_int8(x, wps[i % 64], bias, c["input_zp"], c["output_zp"], mult,
                                                              shift, ws=ws, out=y), launches=64)

    def g1(m, rt):
        w = m.tensor(rt.I8, (2048, 2048), c["w"], channel_scales=c["filter_scales"])
        b = m.tensor(rt.I32, (2048,), c["bias"], channel_scales=c["filter_scales"] * c["input_scale"])
        xi = m.tensor(rt.I8, (32, 2048), scale=float(c["input_scale"]), zero_point=c["input_zp"])
        yo = m.tensor(rt.I8, (32, 2048), scale=float(c["output_scale"]), zero_point=c["output_zp"])
        m.fully_connected(xi, w, b, yo)
        m.set_io([xi], [yo])
        m.write(xi, c["x"])

    record(1, "FULLY_CONNECTED full-integer int8 [32,2048]x[2048,2048]", 32, us, 4349952, 2 * 32 * 2048 * 2048, "hbm", 64,
           _delegate_invoke_us(g1))
    del wps
    torch.cuda.empty_cache()
    # ---- config 2: hybrid [M, 4096] x [14336, 4096]
    n, k = 14336, 4096
    c = workloads.config2(512)
    wps = [ops.PackedInt8Weights(dev(c["w"])) for _ in range(3)]
    fs = dev(c["filter_scales"])
    for m_rows in (1, 8, 64, 512):
        x = dev(c["x"][:m_rows])
        y = torch.empty((m_rows, n), device="cuda")
        us = _median_launch_us(lambda i: ops.fully_connected_hybrid(x, wps[i % 3], fs, ws=ws, out=y))
        alg = 58720256 + 57344 + m_rows * 16384 + m_rows * 57344

        def g2(m, rt, m_rows=m_rows):
            w = m.tensor(rt.I8, (n, k), c["w"], channel_scales=c["filter_scales"])
            xi = m.tensor(rt.F32, (m_rows, k))
            yo = m.tensor(rt.F32, (m_rows, n))
            m.fully_connected(xi, w, None, yo, asymmetric=True)
            m.set_io([xi], [yo])
            m.write(xi, c["x"][:m_rows])

        record(2, "FULLY_CONNECTED hybrid [M,4096]x[14336,4096]", m_rows, us, alg, 2 * m_rows * n * k,
               "tensor" if m_rows >= 256 else "hbm", 3, _delegate_invoke_us(g2))
    del wps
    torch.cuda.empty_cache()
    # ---- config 3: blockwise int4 [M, 2048] x [16384, 2048]
    c = workloads.config3(512)
    wps = [ops.PackedInt4Weights(dev(c["w4"]), dev(c["scales"]), c["blocksize"]) for _ in range(8)]
    for m_rows in (1, 512):
        x = dev(c["x"][:m_rows])
        y = torch.empty((m_rows, 16384), device="cuda")
        us = _median_launch_us(lambda i: ops.fully_connected_blockwise4(x, wps[i % 8], ws=ws, out=y))
        alg = 16777216 + 2097152 + m_rows * 8192 + m_rows * 65536

        def g3(m, rt, m_rows=m_rows):
            w = m.tensor(rt.I4, (16384, 2048), c["w4"])
            s = m.tensor(rt.F16, (16384, 64), c["scales"])
            m.set_blockwise(w, s, 32)
            xi = m.tensor(rt.F32, (m_rows, 2048))
            yo = m.tensor(rt.F32, (m_rows, 16384))
            m.fully_connected(xi, w, None, yo, asymmetric=True)
            m.set_io([xi], [yo])
            m.write(xi, c["x"][:m_rows])

        extra = None
        if m_rows >= 256:
            # this kernel runs on the f16 pipe (block scales folded into fp16 weights): half the int8 rate
            bf16 = measured_peaks()[1]
            flops = 2.0 * m_rows * 16384 * 2048 / (us * 1e-6)
            extra = {"pipe": "tcgen05 kind::f16", "frac_of_measured_bf16_peak": flops / (bf16 * 1e12) if bf16 else None}
        record(3, "FULLY_CONNECTED blockwise int4 [M,2048]x[16384,2048]", m_rows, us, alg, 2 * m_rows * 16384 * 2048,
               "tensor" if m_rows >= 256 else "hbm", 8, _delegate_invoke_us(g3), extra)
    del wps
    torch.cuda.empty_cache()
    # ---- config 4: flash-decode, 16 ragged sequences, 8 heads on one KV head of 256; two copies of the cache
    c = workloads.config4()
    total = int(c["lengths"].sum())
    q, L = dev(c["q"]), dev(c["lengths"])
    for kv in ("f16", "i8"):
        if kv == "i8":
            k8, ks = workloads.quantize_kv_per_token(c["k"])
            v8, vs = workloads.quantize_kv_per_token(c["v"])
            caches = [(dev(k8), dev(v8), dev(ks), dev(vs)) for _ in range(2)]
        else:
            caches = [(dev(c["k"]), dev(c["v"]), None, None) for _ in range(2)]
        us = _median_launch_us(lambda i: ops.sdpa_decode(q, caches[i % 2][0], caches[i % 2][1], L, scale=c["scale"],
                                                         k_scale=caches[i % 2][2], v_scale=caches[i % 2][3], ws=ws))
        alg = (1024 if kv == "f16" else 520) * total + 131136
        e2e = (None, "the composite's tensors are float32 in a graph: see the f32 record of the delegate tests")
        if kv == "f16":
            def g4(m, rt):
                qi = m.tensor(rt.F32, (16, 1, 8, 256))
                ki = m.tensor(rt.F32, (16, 8192, 1, 256))
                vi = m.tensor(rt.F32, (16, 8192, 1, 256))
                mk = m.tensor(rt.F32, (16, 1, 1, 8192))
                yo = m.tensor(rt.F32, (16, 1, 8, 256))
                m.composite("odml.scaled_dot_product_attention", rt.flex_map({"scale": float(c["scale"])}), [qi, ki, vi, mk], yo)
                m.set_io([qi, ki, vi, mk], [yo])
                m.write(qi, c["q"].astype(np.float32))
                m.write(ki, c["k"].astype(np.float32))
                m.write(vi, c["v"].astype(np.float32))
                m.write(mk, np.where(np.arange(8192)[None, None, None, :] < c["lengths"][:, None, None, None], 0.0,
                                     -1e30).astype(np.float32))
            e2e = _delegate_invoke_us(g4, invokes=3)
            if e2e[0] is not None:
                e2e = (e2e[0], "float32 q / k / v and the additive mask as host tensors (268 MB of cache per invoke), as "
                               "the composite appears in a graph")
        record(4, f"odml.scaled_dot_product_attention decode, {kv} cache, 16 sequences, {total} cached tokens", 16, us, alg,
               8192 * total, "hbm", 2, e2e)
        del caches
        torch.cuda.empty_cache()
    return out


# ------------------------------------------------------------------------------------------- device arm
def tensor_parallel_run(args, cfg, mode, world, rank, local, barrier, one_gpu):
    """One batch decoded by all ranks together: every rank holds 1/world of each projection. The logits
    of the first step after the prompt are compared with the one-GPU decoder's (same weights, same
    prompt): per-shard row quantization makes the sharded graph a different float computation."""
    import torch
    import torch.distributed as dist

    from litert_b200 import decoder as dec

    max_seq = args.context + args.warmup + args.steps + 16
    d = dec.Decoder(cfg, max_seq=max_seq, max_batch=args.batch, kv_dtype=args.kv, seed=1005, device=f"cuda:{local}",
                    tp_size=world, tp_rank=rank)
    d.connect(mode)
    rng = np.random.default_rng(4242)
    probe = rng.integers(0, cfg["vocab"], (12, args.batch)).astype(np.int32)
    # ---- parity against the one-GPU decoder: 12 fixed tokens per sequence, logits of the last step
    for t in range(probe.shape[0]):
        _, lg = d.step(probe[t], want_logits=(t == probe.shape[0] - 1))
    gathered = [torch.empty_like(lg) for _ in range(world)]
    dist.all_gather(gathered, lg)
    rel = None
    if rank == 0 and one_gpu is not None:
        full = torch.cat(gathered, dim=1).cpu().numpy()
        rel = float(np.linalg.norm(full - one_gpu) / np.linalg.norm(one_gpu))
    d.reset()
    first = np.random.default_rng(1005).integers(0, cfg["vocab"], args.batch).astype(np.int32)
    d.run(first, args.context, fetch=True)
    d.run(None, args.warmup, fetch=True)
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(d.stream):
        e0.record(d.stream)
        d.run(None, args.steps, fetch=False)
        e1.record(d.stream)
    barrier()
    t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    tok = d.run(None, 1, fetch=True)   # also checks the device status word
    agree = torch.tensor(tok.astype(np.int64), device="cuda")
    lo, hi = agree.clone(), agree.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)
    launches = d.launches_per_step
    d.close()
    del d
    torch.cuda.empty_cache()
    ms = t.item() / args.steps
    return {"tokens_per_s": args.batch / (ms * 1e-3), "ms_per_step": ms, "ranks": world, "scaling": "strong",
            "launches_per_step_per_rank": launches, "ranks_agree_on_tokens": bool(torch.equal(lo, hi)),
            "max_rel_l2_vs_one_gpu": rel,
            "exchange": ("partial sums read from peer memory inside the consuming kernels (flag handshake, no "
                         "collective launch)") if mode == "peer" else "NCCL all-reduce between the kernels"}


def run_ours(args):
    import torch
    import torch.distributed as dist

    from litert_b200 import _lib
    from litert_b200 import decoder as dec

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (there is no CPU fallback in this package)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = model_config(args.model)
    max_seq = args.context + args.warmup + 2 * args.steps + 16
    side_batch = 0 if args.side_batch == args.batch else args.side_batch
    # the checks that need the CPU graph (parity, CPU baseline) run on rank 0 of a one-GPU run, on the
    # SAME weights: drawn once on the device, copied to the host for the CPU side
    with_cpu = world == 1
    weights = dec.make_weights(cfg, seed=1005 + rank, device=f"cuda:{local}")
    host = to_host(weights) if with_cpu else None
    d = dec.Decoder(cfg, max_seq=max_seq, max_batch=max(args.batch, side_batch), kv_dtype=args.kv, weights=weights,
                    device=f"cuda:{local}")
    del weights
    torch.cuda.empty_cache()
    rng = np.random.default_rng(1005 + rank)
    stream = d.stream

    def prompt_pass(batch):
        """Prompt pass of `context` random token ids for each of `batch` sequences (one call per sequence,
        host tokens in, first generated token out); returns prompt tokens per second."""
        prompts = rng.integers(0, cfg["vocab"], (batch, args.context)).astype(np.int32)
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for b in range(batch):
            d.prefill(prompts[b], seq=b)
        torch.cuda.synchronize()
        return batch * args.context / (time.perf_counter() - t0)

    prefill = None
    if args.context > 0:
        prompt_pass(1)  # untimed: scratch allocation and one-time kernel setup at the timed shapes
        d.reset()
        prefill = {"tokens_per_s_per_gpu": prompt_pass(args.batch), "prompt_tokens": args.context, "sequences": args.batch,
                   "timing": "host clock around b200_decoder_prefill per sequence (host token ids in, first token out)"}
    else:
        d.run(rng.integers(0, cfg["vocab"], args.batch).astype(np.int32), 1, fetch=True)

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    # ---- device-resident timing: K steps of the captured graph, tokens fed back on the device
    d.run(None, args.warmup, fetch=True, batch=args.batch)
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        e0.record(stream)
        d.run(None, args.steps, fetch=False)
        e1.record(stream)
    barrier()
    dev_ms = e0.elapsed_time(e1)
    # ---- end to end through the public call: host tokens in, host tokens out, every step
    tok = d.run(None, 1, fetch=True)
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        tok, _ = d.step(tok)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    # ---- per-kernel-class device time of one step (CUDA events around every launch)
    prof = d.profile_step(tok)
    launches = d.launches_per_step
    # ---- the dominant kernel alone: the step's GEMV launches replayed back to back as one graph
    gemv_ms, gemv_launches = d.time_gemv(args.batch, reps=max(8, min(64, args.steps)))

    # ---- the other batch size of the workload, same decoder, its own prompt pass
    side = None
    side_prefill = None
    if side_batch > 0:
        d.reset()
        if args.context > 0:
            side_prefill = prompt_pass(side_batch)
            d.run(None, max(3, args.warmup), fetch=True, batch=side_batch)
        else:
            d.run(rng.integers(0, cfg["vocab"], side_batch).astype(np.int32), max(3, args.warmup), fetch=True)
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            s0.record(stream)
            d.run(None, args.steps, fetch=False)
            s1.record(stream)
        barrier()
        side_ms = s0.elapsed_time(s1) / args.steps
        side_gemv_ms, _ = d.time_gemv(side_batch, reps=8)
        side = {"batch_per_gpu": side_batch, "tokens_per_s_per_gpu": side_batch / (side_ms * 1e-3),
                "ms_per_step": side_ms, "gemv_ms_per_step": side_gemv_ms,
                "gemv_gbs": weight_bytes(cfg) / (side_gemv_ms * 1e-3) / 1e9,
                "prefill_tokens_per_s_per_gpu": side_prefill}

    # ---- parity of this very decoder against the CPU graph on the same weights (untimed)
    parity = None
    if with_cpu and rank == 0:
        try:
            parity = parity_record(cfg, d, host, args.kv)
        except Exception as exc:
            parity = {"checked": False, "error": str(exc)[:300]}

    # ---- one-GPU logits for the tensor-parallel comparison (rank 0's replica has seed 1005: the TP weights)
    one_gpu_logits = None
    if world > 1 and args.tp != "off" and rank == 0:
        probe = np.random.default_rng(4242).integers(0, cfg["vocab"], (12, args.batch)).astype(np.int32)
        d.reset()
        for t in range(probe.shape[0]):
            _, lg = d.step(probe[t], want_logits=(t == probe.shape[0] - 1))
        one_gpu_logits = lg.cpu().numpy()

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    line = None
    if rank == 0:
        tokens = args.batch * args.steps * world
        peak, bf16_peak, peak_kind = measured_peaks()
        wbytes = weight_bytes(cfg)
        # algorithmic bytes of the GEMV launches of one step: every int8 weight once, plus per launch the
        # per-channel scales and row sums (8 B per output channel), the quantized activation rows and the
        # float outputs
        n_out = cfg["n_layers"] * ((cfg["n_heads"] + 2 * cfg["n_kv_heads"]) * cfg["head_dim"] + 2 * cfg["d_model"]
                                   + 2 * cfg["d_ff"]) + cfg["vocab"]
        k_in = cfg["n_layers"] * (2 * cfg["d_model"] + cfg["n_heads"] * cfg["head_dim"] + cfg["d_ff"]) + cfg["d_model"]
        gemv_bytes = wbytes + 8 * n_out + args.batch * (k_in + 4 * n_out)
        achieved = gemv_bytes / (gemv_ms * 1e-3) / 1e9 if gemv_ms > 0 else None
        line = {
            "metric": METRIC, "value": tokens / (dev_ms * 1e-3), "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": dev_ms / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": DTYPE,
            "data": "synthetic", "config": workload_config(args, cfg),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                    "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": e2e_ms / args.steps,
                    "through": "b200_decoder_step: host token ids in, host token ids out, one synchronisation per step"},
            "gpu_launches": launches * args.steps,
            "launches_per_step": launches,
            "clocks": clocks,
            "roofline": {"bound": "hbm", "kernel": "fc_umma_kernel + fc_cluster_kernel (streamed int8 GEMV, all projections of one step)",
                         "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak if achieved else None,
                         "peak_kind": peak_kind,
                         "traffic": NCU_TRAFFIC_PER_ALGORITHMIC_BYTE * gemv_bytes / gemv_launches,
                         "traffic_unit": "bytes per launch (average over the step's GEMV launches), ncu ratio x "
                                         "algorithmic bytes",
                         "algorithmic_bytes_per_launch": gemv_bytes / gemv_launches, "launches": gemv_launches,
                         "algorithmic_bytes_per_step": gemv_bytes, "gemv_ms_per_step": gemv_ms,
                         "avg_launch_us": gemv_ms * 1e3 / gemv_launches,
                         "timing": "CUDA events around a graph of the step's GEMV launches alone, on the launching stream",
                         "whole_step_frac": (wbytes / (dev_ms / args.steps * 1e-3) / 1e9) / peak},
            "step_breakdown_ms": {k: v[0] for k, v in prof.items()},
        }
        if parity is not None:
            line["parity"] = parity
        if side:
            line["side_batch"] = side
        if prefill:
            # 2 int8 operations per weight and prompt token (the LM head runs for the last token only)
            ops_per_token = 2.0 * (wbytes - cfg["vocab"] * cfg["d_model"])
            prefill["int8_pops"] = prefill["tokens_per_s_per_gpu"] * ops_per_token / 1e15
            line["prefill"] = prefill
    d.close()
    del d
    torch.cuda.empty_cache()
    if rank == 0 and with_cpu:
        try:
            line["cpu_baseline"] = cpu_baseline_record(cfg, host, args)
        except Exception as exc:  # the baseline is a report, not part of the product path
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port",
                                    "sample": f"not run: {exc}"}
        if args.batch == 1:
            # the headline end-to-end number is the one through the reference-facing plugin; the resident
            # decoder's own C-ABI call (host token ids in and out) is kept beside it
            try:
                plug = plugin_decode_e2e(cfg, host, args, invokes=max(12, min(132, args.steps + 4)))
            except Exception as exc:
                plug = {"error": str(exc)[:300]}
            if "value" in plug:
                line["e2e_c_abi"] = line["e2e"]
                line["e2e"] = plug
            else:
                line["e2e_plugin"] = plug
        host = None
        # ---- the int8 tensor peak of this device, and the single-op configurations against it
        i8_peak = None
        try:
            ops_s, ms = ctypes_double(), ctypes_double()
            if _lib.load().b200_measure_int8_tensor_peak(20000, ops_s, ms) == 0:
                i8_peak = ops_s.value
                line["int8_tensor_peak"] = {"pop_per_s": i8_peak / 1e15, "kernel_ms": ms.value,
                                            "how": "one CTA per SM, resident-operand tcgen05.mma kind::i8 M128 N256 K32 back "
                                                   "to back (b200_measure_int8_tensor_peak), best of 3",
                                            "twice_measured_bf16_pop_per_s": 2 * bf16_peak / 1e3}
                if prefill:
                    prefill["frac_of_int8_tensor_peak"] = prefill["int8_pops"] * 1e15 / i8_peak
        except Exception as exc:
            line["int8_tensor_peak"] = {"error": str(exc)[:200]}
        if args.configs == "on" and args.model == "gemma2b":
            try:
                line["configs"] = config_records(peak, i8_peak)
            except Exception as exc:
                line["configs"] = [{"error": str(exc)[:300]}]
    elif rank == 0:
        line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port",
                                "sample": "timed at --gpus 1 only"}
    # ---- the same batch run tensor-parallel over all ranks (strong scaling of one sequence batch)
    tp = {}
    if world > 1 and args.tp != "off":
        for mode in (["peer", "nccl"] if args.tp == "both" else [args.tp]):
            try:
                tp[mode] = tensor_parallel_run(args, cfg, mode, world, rank, local, barrier, one_gpu_logits)
                if rank == 0:
                    one_ms = dev_ms / args.steps
                    tp[mode]["speedup_vs_one_gpu"] = one_ms / tp[mode]["ms_per_step"]
                    tp[mode]["strong_efficiency"] = one_ms / tp[mode]["ms_per_step"] / world
            except Exception as exc:  # reported, the replica line above stands on its own
                tp[mode] = {"error": str(exc)[:300]}
    if rank == 0:
        if tp:
            line["tensor_parallel"] = tp
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def ctypes_double():
    import ctypes

    return ctypes.c_double(0.0)


_RESULT_FD = None


def emit(line):
    """Writes the result line to the process's original standard output."""
    data = (json.dumps(line) + "\n").encode()
    if _RESULT_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_RESULT_FD, data)


def main():
    global _RESULT_FD
    args = parse_args()
    # Standard output carries the one result line and nothing else: libraries that print there
    # (NCCL's version banner, for one) are sent to standard error for the length of the run.
    sys.stdout.flush()
    _RESULT_FD = os.dup(1)
    os.dup2(2, 1)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
