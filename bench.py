#!/usr/bin/env python
"""Decode benchmark: tokens/s of a Gemma-2B-shaped int8 (dynamic-range) decoder, with the HBM
roofline of its dominant kernel (the streamed int8 GEMV) and a CPU baseline beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--batch B] [--context C] [--impl ours|reference]

One "step" is one decode step (one new token per sequence) over a KV cache that already holds
`context` tokens. All inputs are synthetic: seeded random-init weights of the named architecture and
random token ids. With --gpus N > 1 (launched under torchrun, one rank per GPU) every rank decodes
its own batch on its own replica (independent invocations partitioned across GPUs, no data-path
collective): weak scaling, aggregate tokens/s.

--impl reference times the CPU implementation of the same graph (the oracle's vectorised,
multi-threaded restatement of the reference kernels; the reference's own ruy/XNNPACK kernels cannot
be built offline) on the host cores of the box, on a bounded sample of the workload.
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


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
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
    return ap.parse_args()


def model_config(name):
    from litert_b200 import decoder as dec

    return dict(dec.GEMMA_2B if name == "gemma2b" else dec.TINY)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f).get("hbm_gbs"), "measured"
    return 6650.0, "fallback"


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


def cpu_reference_run(cfg, batch, steps, warmup, seed=1005):
    """The CPU arm: all host threads, weights generated on the host with the same distributions."""
    import oracle
    import torch

    oracle.build()
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
    weights = dict(layers=layers, embed=w(cfg["vocab"], d), embed_scales=s(cfg["vocab"]), final_norm=gain(d))
    ref = oracle.DecoderRef(cfg, weights, batch, warmup + steps + 2, fast=True)
    cores = oracle.fast().orcf_num_threads()
    rng = np.random.default_rng(seed)
    tok = rng.integers(0, cfg["vocab"], batch).astype(np.int32)
    for _ in range(warmup):
        tok, _ = ref.step(tok, want_logits=False)
    t0 = time.perf_counter()
    for _ in range(steps):
        tok, _ = ref.step(tok, want_logits=False)
    dt = time.perf_counter() - t0
    ref.close()
    return batch * steps / dt, dt / steps * 1e3, cores


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = model_config(args.model)
    steps = max(1, min(args.steps, args.cpu_steps))
    warm = 1
    tps, ms, cores = cpu_reference_run(cfg, args.batch, steps, warm)
    sample = (f"{steps} decode steps after {warm} warm-up, batch {args.batch}, context {warm}..{warm + steps} tokens "
              f"(attention over a short cache; the {weight_bytes(cfg) / 1e9:.2f} GB of weights per step dominate)")
    line = {
        "impl": "reference", "metric": METRIC, "value": tps, "unit": "tokens/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "int8 weights x int8 dynamically quantized activations, int32 accumulate, fp32 outputs",
        "data": "synthetic",
        "config": workload_config(args, cfg),
        "cpu_baseline": {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": tps, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
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


def tensor_parallel_run(args, cfg, mode, world, rank, local, barrier):
    """One batch decoded by all ranks together: every rank holds 1/world of each projection."""
    import torch
    import torch.distributed as dist

    from litert_b200 import decoder as dec

    max_seq = args.context + args.warmup + args.steps + 16
    d = dec.Decoder(cfg, max_seq=max_seq, max_batch=args.batch, kv_dtype=args.kv, seed=1005, device=f"cuda:{local}",
                    tp_size=world, tp_rank=rank)
    d.connect(mode)
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
            "exchange": ("partial sums read from peer memory inside the consuming kernels (flag handshake, no "
                         "collective launch)") if mode == "peer" else "NCCL all-reduce between the kernels"}


def run_ours(args):
    import torch
    import torch.distributed as dist

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
    d = dec.Decoder(cfg, max_seq=max_seq, max_batch=max(args.batch, side_batch), kv_dtype=args.kv, seed=1005 + rank,
                    device=f"cuda:{local}")
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

    times = torch.tensor([dev_ms, e2e_s * 1e3], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(times, op=dist.ReduceOp.MAX)
    dev_ms, e2e_ms = times.tolist()
    if rank == 0:
        tokens = args.batch * args.steps * world
        peak, peak_kind = measured_peaks()
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
            "scaling": "weak", "vs_baseline": None,
            "dtype": "int8 weights x int8 dynamically quantized activations, int32 accumulate, fp32 outputs",
            "data": "synthetic", "config": workload_config(args, cfg),
            "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tokens/s", "h2d_bytes_per_step": 4 * args.batch,
                    "d2h_bytes_per_step": 4 * args.batch, "ms_per_step": e2e_ms / args.steps},
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
        if side:
            line["side_batch"] = side
        if prefill:
            # 2 int8 operations per weight and prompt token (the LM head runs for the last token only)
            ops = 2.0 * (wbytes - cfg["vocab"] * cfg["d_model"])
            prefill["int8_pops"] = prefill["tokens_per_s_per_gpu"] * ops / 1e15
            line["prefill"] = prefill
        try:
            if world > 1:
                raise RuntimeError("timed at --gpus 1 only")
            steps = max(1, min(args.cpu_steps, args.steps))
            tps, ms, cores = cpu_reference_run(cfg, args.batch, steps, 1)
            line["cpu_baseline"] = {"value": tps, "unit": "tokens/s", "cores": cores, "kind": "port",
                                    "sample": f"{steps} decode steps, batch {args.batch}, short context, all host threads"}
        except Exception as exc:  # the baseline is a report, not part of the product path
            line["cpu_baseline"] = {"value": None, "unit": "tokens/s", "cores": 0, "kind": "port",
                                    "sample": f"not run: {exc}"}
    d.close()
    del d
    torch.cuda.empty_cache()
    # ---- the same batch run tensor-parallel over all ranks (strong scaling of one sequence batch)
    tp = {}
    if world > 1 and args.tp != "off":
        for mode in (["peer", "nccl"] if args.tp == "both" else [args.tp]):
            try:
                tp[mode] = tensor_parallel_run(args, cfg, mode, world, rank, local, barrier)
            except Exception as exc:  # reported, the replica line above stands on its own
                tp[mode] = {"error": str(exc)[:300]}
    if rank == 0:
        if tp:
            line["tensor_parallel"] = tp
        emit(line)
    if world > 1:
        dist.destroy_process_group()


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
