"""The resident decoder against the CPU restatement of the same graph (oracle/decoder_ref.c): a
small Gemma-shaped configuration, several decode steps, ragged positions across the batch."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _host(weights):
    out = dict(layers=[{k: v.cpu().numpy() for k, v in lw.items()} for lw in weights["layers"]])
    for k in ("embed", "embed_scales", "final_norm"):
        out[k] = weights[k].cpu().numpy()
    return out


# Tolerance: the graph re-quantizes activations to int8 before every projection, so a relative
# perturbation of 1e-4 anywhere (fp16 cache rounding, a different summation order in a norm) flips a
# few int8 values and moves this small model's logits by 1-3 % of their range -- the CPU restatement
# shows the same sensitivity to such a perturbation of its own inputs. Element-wise parity of every
# kernel is asserted exactly in test_gpu_parity.py; here the bound is on the whole graph.
@pytest.mark.parametrize("kv_dtype,tol", [("f16", 6e-2), ("i8", 2e-1)])
def test_decoder_matches_cpu_graph(oracle, kv_dtype, tol):
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    batch, steps, max_seq = 3, 6, 16
    weights = dec.make_weights(cfg, seed=7)
    gpu = dec.Decoder(cfg, max_seq=max_seq, max_batch=4, weights=weights, kv_dtype=kv_dtype)
    ref = oracle.DecoderRef(cfg, _host(weights), batch, max_seq, fast=False, kv_mode=1 if kv_dtype == "f16" else 2)
    rng = np.random.default_rng(3)
    tokens = rng.integers(0, cfg["vocab"], batch).astype(np.int32)
    worst = 0.0
    for s in range(steps):
        nxt_g, logits_g = gpu.step(tokens, want_logits=True)
        nxt_r, logits_r = ref.step(tokens)
        lg = logits_g.cpu().numpy()
        err = np.linalg.norm(lg - logits_r) / np.linalg.norm(logits_r)  # relative L2 over the logits
        worst = max(worst, err)
        assert err <= tol, (s, err)
        # greedy tokens agree wherever the reference's top-2 margin is larger than the error
        top2 = np.sort(logits_r, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4 * np.max(np.abs(lg - logits_r))
        assert np.array_equal(nxt_g[clear], nxt_r[clear])
        tokens = nxt_r  # feed both the same continuation
    gpu.close()
    ref.close()


@pytest.mark.parametrize("kv_dtype,tol", [("f16", 8e-2), ("i8", 2.5e-1)])
def test_decoder_long_context_attention_step(oracle, kv_dtype, tol):
    """Seventy tokens deep: the one-launch attention step then gives every CTA of its cluster several
    16-token groups (first CTAs) or none (last ones), and the warps of a CTA unequal shares. The
    bound is looser than above because the divergence of two int8-requantizing graphs grows with depth."""
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    batch, steps, max_seq = 2, 70, 96
    weights = dec.make_weights(cfg, seed=12)
    gpu = dec.Decoder(cfg, max_seq=max_seq, max_batch=batch, weights=weights, kv_dtype=kv_dtype)
    ref = oracle.DecoderRef(cfg, _host(weights), batch, max_seq, fast=True, kv_mode=1 if kv_dtype == "f16" else 2)
    tokens = np.random.default_rng(6).integers(0, cfg["vocab"], batch).astype(np.int32)
    for s in range(steps):
        check = s in (0, 17, 33, 50, 69)
        _, logits_g = gpu.step(tokens, want_logits=check)
        nxt_r, logits_r = ref.step(tokens, want_logits=True)
        if check:
            err = np.linalg.norm(logits_g.cpu().numpy() - logits_r) / np.linalg.norm(logits_r)
            assert err <= tol, (s, err)
        tokens = nxt_r
    gpu.close()
    ref.close()


def test_decoder_wide_batch_uses_chunked_attention(oracle):
    """Twelve sequences: past the size where one cluster per sequence pays, the step goes through the
    rotary / flash-decode / merge kernels instead. Same bound as above."""
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    batch, steps, max_seq = 12, 4, 12
    weights = dec.make_weights(cfg, seed=9)
    gpu = dec.Decoder(cfg, max_seq=max_seq, max_batch=batch, weights=weights)
    ref = oracle.DecoderRef(cfg, _host(weights), batch, max_seq, fast=False)
    tokens = np.random.default_rng(4).integers(0, cfg["vocab"], batch).astype(np.int32)
    for s in range(steps):
        _, logits_g = gpu.step(tokens, want_logits=True)
        nxt_r, logits_r = ref.step(tokens)
        err = np.linalg.norm(logits_g.cpu().numpy() - logits_r) / np.linalg.norm(logits_r)
        assert err <= 6e-2, (s, err)
        tokens = nxt_r
    gpu.close()
    ref.close()


def test_decoder_greedy_pick_is_the_first_index_argmax_of_its_logits(oracle):
    """The token the step returns (picked inside the LM-head GEMV's epilogue) is the serial first-index
    arg-max of the logits the same call hands out, with and without the logits soft-cap, and the graph path
    (no logits written at all) returns the same tokens."""
    from litert_b200 import _lib
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    d = dec.Decoder(cfg, max_seq=16, max_batch=3, weights=dec.make_weights(cfg, seed=31))
    tok = np.asarray([1, 500, 999], np.int32)
    for cap in (0.0, 2.0):
        assert _lib.load().b200_decoder_set_logit_soft_cap(d.handle, cap) == 0
        d.reset()
        nxt, logits = d.step(tok, want_logits=True)
        lg = logits.cpu().numpy()
        assert np.array_equal(nxt, oracle.stage_argmax(lg))
        if cap:
            assert np.max(np.abs(lg)) <= cap + 1e-6
        d.reset()
        nxt_graph, _ = d.step(tok)
        assert np.array_equal(nxt_graph, nxt)
    d.close()


def test_decoder_graph_path_equals_eager_path_and_is_repeatable():
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    weights = dec.make_weights(cfg, seed=8)
    d = dec.Decoder(cfg, max_seq=32, max_batch=2, weights=weights)
    first = np.asarray([5, 17], np.int32)

    def greedy(use_run):
        d.reset()
        if use_run:
            return d.run(first, 8)
        tok = first
        for _ in range(8):
            tok, _ = d.step(tok)
        return tok

    a = greedy(False)
    b = greedy(True)   # device-resident feedback loop over the captured graph
    c = greedy(False)
    assert np.array_equal(a, b) and np.array_equal(a, c)
    assert d.launches_per_step > 0
    d.close()


@pytest.mark.parametrize("kv_dtype,tol", [("f16", 8e-2), ("i8", 2.5e-1)])
def test_prefill_matches_token_by_token_cpu_graph(oracle, kv_dtype, tol):
    """A prompt pass (all prompt rows through each projection as one GEMM, causal attention over the
    rows just appended) must leave the caches and predict the token that the CPU graph reaches by
    stepping the same prompt one token at a time; the decode steps after it are compared as above."""
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    batch, prompt_len, max_seq = 2, 45, 64
    weights = dec.make_weights(cfg, seed=21)
    gpu = dec.Decoder(cfg, max_seq=max_seq, max_batch=batch, weights=weights, kv_dtype=kv_dtype)
    ref = oracle.DecoderRef(cfg, _host(weights), batch, max_seq, fast=True, kv_mode=1 if kv_dtype == "f16" else 2)
    prompts = np.random.default_rng(8).integers(0, cfg["vocab"], (batch, prompt_len)).astype(np.int32)
    for t in range(prompt_len):
        nxt_r, logits_r = ref.step(prompts[:, t], want_logits=True)
    first = np.array([gpu.prefill(prompts[b], seq=b) for b in range(batch)], np.int32)
    top2 = np.sort(logits_r, axis=-1)[:, -2:]
    spread = logits_r.max(axis=-1) - logits_r.min(axis=-1)
    clear = (top2[:, 1] - top2[:, 0]) > 0.1 * spread
    assert np.array_equal(first[clear], nxt_r[clear])
    tokens = nxt_r
    for s in range(4):
        _, logits_g = gpu.step(tokens, want_logits=True)
        nxt_r, logits_r = ref.step(tokens, want_logits=True)
        err = np.linalg.norm(logits_g.cpu().numpy() - logits_r) / np.linalg.norm(logits_r)
        assert err <= tol, (s, err)
        tokens = nxt_r
    gpu.close()
    ref.close()


@pytest.mark.parametrize("kv_dtype", ["f16", "i8"])
@pytest.mark.parametrize("split", [(1100,), (600, 500), (1, 1029, 70)])
def test_prefill_equals_stepping_on_the_device(kv_dtype, split):
    """Prompts longer than one 1024-row chunk, and prompts fed in several calls (each behind the
    tokens already cached), against the same decoder fed one token per step. The integer GEMMs are
    exact in either form; attention sums in a different order, hence a bound and not equality."""
    from litert_b200 import decoder as dec

    cfg = dict(dec.TINY)
    total, max_seq = sum(split), 1120
    weights = dec.make_weights(cfg, seed=5)
    prompt = np.random.default_rng(11).integers(0, cfg["vocab"], total).astype(np.int32)
    stepped = dec.Decoder(cfg, max_seq=max_seq, max_batch=2, weights=weights, kv_dtype=kv_dtype)
    for t in range(total):
        nxt_s, logits_s = stepped.step(prompt[t:t + 1], want_logits=(t == total - 1))
    filled = dec.Decoder(cfg, max_seq=max_seq, max_batch=2, weights=weights, kv_dtype=kv_dtype)
    filled.set_positions(np.array([7, 0], np.int32))  # another sequence's state must not matter
    done = 0
    for part in split:
        first = filled.prefill(prompt[done:done + part], seq=1)
        done += part
    # the stepped decoder holds the prompt in sequence 0, the filled one in sequence 1
    ls = logits_s.cpu().numpy()[0]
    top2 = np.sort(ls)[-2:]
    if top2[1] - top2[0] > 0.05 * (ls.max() - ls.min()):
        assert first == int(nxt_s[0])
    tok = nxt_s[:1]
    for s in range(3):
        nxt_s, logits_s = stepped.step(tok, want_logits=True)
        _, logits_f = filled.step(np.array([3, tok[0]], np.int32), want_logits=True)
        a, b = logits_f.cpu().numpy()[1], logits_s.cpu().numpy()[0]
        err = np.linalg.norm(a - b) / np.linalg.norm(b)
        assert err <= 3e-2, (s, err)
        tok = nxt_s[:1]
    stepped.close()
    filled.close()


def test_prefill_rejects_what_does_not_fit():
    from litert_b200 import decoder as dec
    from litert_b200._lib import B200Error

    cfg = dict(dec.TINY)
    d = dec.Decoder(cfg, max_seq=32, max_batch=1, weights=dec.make_weights(cfg, seed=1))
    with pytest.raises(B200Error):
        d.prefill(np.zeros(33, np.int32))
    with pytest.raises(B200Error):
        d.prefill(np.array([cfg["vocab"]], np.int32))
    with pytest.raises(B200Error):
        d.prefill(np.zeros(4, np.int32), seq=1)
    d.prefill(np.zeros(30, np.int32))
    with pytest.raises(B200Error):
        d.prefill(np.zeros(3, np.int32))  # 30 cached + 3 > 32
    d.close()


@pytest.mark.parametrize("head_dim,heads", [(128, 4), (256, 8), (256, 3)])
@pytest.mark.parametrize("kv_dtype", ["f16", "i8"])
def test_prefill_at_wide_heads_equals_stepping(kv_dtype, head_dim, heads):
    """The benchmark's head size (256, eight query heads on one KV head) and 128, which the small test
    model above does not reach: prompt pass against the same decoder fed one token per step. The two
    differ only in the order attention sums over tokens, but this shape (a 2048-wide attention output
    quantized to int8 in front of a 256-wide model) turns those last-bit differences into int8 flips
    more often than the small model: 0.02-0.04 relative L2 measured for every attention kernel variant
    against every other, hence the whole-graph bound used against the CPU graph."""
    from litert_b200 import decoder as dec

    cfg = dict(n_layers=2, d_model=256, n_heads=heads, n_kv_heads=1, head_dim=head_dim, d_ff=512, vocab=800)
    total, max_seq = 333, 352
    weights = dec.make_weights(cfg, seed=17)
    prompt = np.random.default_rng(23).integers(0, cfg["vocab"], total).astype(np.int32)
    stepped = dec.Decoder(cfg, max_seq=max_seq, max_batch=1, weights=weights, kv_dtype=kv_dtype)
    for t in range(total):
        nxt_s, logits_s = stepped.step(prompt[t:t + 1], want_logits=(t == total - 1))
    filled = dec.Decoder(cfg, max_seq=max_seq, max_batch=1, weights=weights, kv_dtype=kv_dtype)
    first = filled.prefill(prompt)
    ls = logits_s.cpu().numpy()[0]
    top2 = np.sort(ls)[-2:]
    if top2[1] - top2[0] > 0.05 * (ls.max() - ls.min()):
        assert first == int(nxt_s[0])
    tok = nxt_s[:1]
    for s in range(3):
        nxt_s, logits_s = stepped.step(tok, want_logits=True)
        _, logits_f = filled.step(tok, want_logits=True)
        a, b = logits_f.cpu().numpy()[0], logits_s.cpu().numpy()[0]
        err = np.linalg.norm(a - b) / np.linalg.norm(b)
        assert err <= 6e-2, (s, err)
        tok = nxt_s[:1]
    stepped.close()
    filled.close()


def test_gemma2b_shaped_decoder_against_cpu_graph(oracle):
    """The benchmark's own configuration (18 layers, d_model 2048, 8 heads of 256 on one KV head,
    feed-forward 16384, vocabulary 256000), weights generated ONCE and handed to both sides: a 64-token
    prompt through the prompt pass and three decode steps at batch 1, then 32 sequences with short
    prompts (the CPU graph needs about a second per 32-row step) and three decode steps at batch 32.

    How close can two correct implementations of this graph be? With random-init weights the attention
    logits have a standard deviation near 100, so the softmax is almost a hard maximum and a relative
    change of 2e-4 in a cached key moves a head's output by percents; every activation row is then
    re-quantized to int8. The test measures that sensitivity on the CPU graph itself: the same graph
    with its cache rows kept in float32 instead of rounded to binary16 (one rounding per cached value,
    nothing else changed). The device must agree with the CPU graph (cache rounded as on the device)
    at least as well as 1.5 x that self-difference, and pick the same token wherever the margin is clear.
    Both numbers are printed. Exact per-kernel parity at these widths is in test_gpu_glue.py."""
    from litert_b200 import decoder as dec

    cfg = dict(dec.GEMMA_2B)
    max_seq = 96
    weights = dec.make_weights(cfg, seed=1005)
    host = _host(weights)
    gpu = dec.Decoder(cfg, max_seq=max_seq, max_batch=32, weights=weights, kv_dtype="f16")
    del weights
    torch.cuda.empty_cache()
    rng = np.random.default_rng(2024)

    def rl2(a, b):
        return float(np.linalg.norm(a - b) / np.linalg.norm(b))

    def compare(tag, logits_g, logits_r, logits_self, nxt_g, nxt_r):
        lg = logits_g.cpu().numpy()
        err, self_err = rl2(lg, logits_r), rl2(logits_self, logits_r)
        top2 = np.sort(logits_r, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 4 * np.max(np.abs(lg - logits_r), axis=-1)
        agree = int(np.sum(nxt_g[clear] == nxt_r[clear]))
        print(f"gemma-2b-shaped {tag}: device vs CPU graph relative L2 {err:.3e}; CPU graph vs itself with a float32 "
              f"cache {self_err:.3e}; greedy tokens equal on {agree} of {int(clear.sum())} rows with a clear margin "
              f"({int(np.sum(nxt_g == nxt_r))} of {nxt_r.size} overall)")
        assert err <= max(1.5 * self_err, 2e-2), (tag, err, self_err)
        assert agree == int(clear.sum()), tag

    def run(batch, prompt_len):
        ref = oracle.DecoderRef(cfg, host, batch, max_seq, fast=True, kv_mode=1)    # the arbiter
        ref32 = oracle.DecoderRef(cfg, host, batch, max_seq, fast=True, kv_mode=0)  # its float32-cache twin
        prompts = rng.integers(0, cfg["vocab"], (batch, prompt_len)).astype(np.int32)
        for t in range(prompt_len):
            nxt_r, logits_r = ref.step(prompts[:, t], want_logits=(t == prompt_len - 1))
            ref32.step(prompts[:, t], want_logits=False)
        first = np.array([gpu.prefill(prompts[b], seq=b) for b in range(batch)], np.int32)
        top2 = np.sort(logits_r, axis=-1)[:, -2:]
        clear = (top2[:, 1] - top2[:, 0]) > 0.1 * (logits_r.max(axis=-1) - logits_r.min(axis=-1))
        assert np.array_equal(first[clear], nxt_r[clear]), "first generated tokens after the prompt pass"
        tok = nxt_r
        for s in range(3):
            nxt_g, logits_g = gpu.step(tok, want_logits=True)
            nxt_r, logits_r = ref.step(tok, want_logits=True)
            _, logits_self = ref32.step(tok, want_logits=True)
            compare(f"batch {batch} step {s}", logits_g, logits_r, logits_self, nxt_g, nxt_r)
            tok = nxt_r
        ref.close()
        ref32.close()

    run(1, 64)
    gpu.reset()
    run(32, 4)
    gpu.close()
