"""Benchmark: decode tokens a second of the engine on Llama-3.2-1B shapes
(random weights, synthetic tokens), one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference]

A step is one decode step of a batch of 8 requests at context 4096.  `value`
times K steps on the device (CUDA events) through the step function and the
sampler; `e2e` times the same through the Python entry point
(LLMEngine.step(): host tokens in, host tokens out).  The line also carries a
2,048-token prefill, decode at batch 1 and 64, and the decode step's HBM
roofline.  Every step reads all weights (2.5 GB) and the live cache, far more
than the 126 MB L2, so nothing is served from cache between timed steps.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LLAMA_1B = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 128256, "hidden_size": 2048,
    "intermediate_size": 8192, "num_hidden_layers": 16, "num_attention_heads": 32, "num_key_value_heads": 8,
    "head_dim": 64, "max_position_embeddings": 131072, "rms_norm_eps": 1e-5, "rope_theta": 500000.0,
    "rope_scaling": {"rope_type": "llama3", "factor": 32.0, "low_freq_factor": 1.0, "high_freq_factor": 4.0,
                     "original_max_position_embeddings": 8192},
    "tie_word_embeddings": True, "hidden_act": "silu", "attention_bias": False, "mlp_bias": False,
    "bos_token_id": 128000, "eos_token_id": 128001, "torch_dtype": "bfloat16",
}
# The same architecture at the sizes of Llama-3.2-3B and Llama-3.1-8B, for --only runs at further sizes.
LLAMA_3B = dict(LLAMA_1B, hidden_size=3072, num_hidden_layers=28, num_attention_heads=24, head_dim=128)
LLAMA_8B = dict(LLAMA_1B, hidden_size=4096, intermediate_size=14336, num_hidden_layers=32, head_dim=128,
                tie_word_embeddings=False,
                rope_scaling=dict(LLAMA_1B["rope_scaling"], factor=8.0))
SHAPES = {"1b": LLAMA_1B, "3b": LLAMA_3B, "8b": LLAMA_8B}
CONTEXT = 4096
PREFILL_TOKENS = 2048
BLOCK_SIZE = 16
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    out = dict(FALLBACK_PEAKS, source="fallback")
    try:
        with open(path) as f:
            raw = json.load(f)
        for key in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
            if key in raw and isinstance(raw[key], (int, float)):
                out[key] = float(raw[key])
        out["source"] = "measured"
    except (OSError, ValueError):
        pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self):
        self.rows = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(",")])

    def mark(self):
        return len(self.rows)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self, begin=0, end=None):
        rows = [r for r in self.rows[begin:end] if len(r) >= 7]
        if not rows:
            rows = [r for r in self.rows if len(r) >= 7]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = sorted(int(float(r[0])) for r in rows)
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(r[3 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": int(float(rows[0][1])), "reasons": reasons,
                "samples": len(rows), "power_w": max(float(r[2]) for r in rows)}


def decode_bytes(cfg, batch, context):
    """Bytes one decode step must read: every weight it uses once, and the
    keys and values of the live requests (bfloat16)."""
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    weights = 2 * (L * per_layer + V * H) + 4 * (2 * L + 1) * H   # the head's table; the embedding reads `batch` rows
    kv = 2 * batch * context * 2 * nkv * hd * L
    return weights + kv


def prefill_flops(cfg, tokens):
    H, I, V, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"], cfg["num_hidden_layers"]
    nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 2 * I * H + H * I
    linear = 2 * tokens * L * per_layer + 2 * V * H
    attention = 4 * nh * hd * tokens * (tokens + 1) // 2 * L
    return linear + attention


def make_rig(cfg, context, max_batch, page):
    """A model of the given shapes with random weights, an engine around it with
    room for `max_batch` requests of `context` tokens, and the three timed
    loops (decode steps, prompts, decode steps beside a prompt portion)."""
    import gc
    import types

    import torch

    from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, build, load_model, ops

    host = build.load_host()
    num_blocks = (max_batch * (context + 64) + 2 * PREFILL_TOKENS + context) // page
    loaded = load_model(config=cfg, random_seed=0, dtype="bfloat16", device="cuda:0", max_model_len=context + 64)
    engine = LLMEngine(loaded, EngineConfig(num_blocks=num_blocks, block_size=page, max_num_seqs=max_batch,
                                            max_num_batched_tokens=8192, dtype="bfloat16", device="cuda:0",
                                            max_model_len=context + 64))
    runner, manager, sampler = engine.runner, engine.block_manager, engine.sampler
    gen = torch.Generator().manual_seed(0)
    vocab = cfg["vocab_size"] if "vocab_size" in cfg else cfg["vocab"]
    # Synthetic cache content: timing does not depend on what the pages hold,
    # but a softmax over zeros would be a degenerate case.
    for pools in engine.cache.streams:
        for s in pools:
            s.k.normal_(0, 1)
            s.v.normal_(0, 1)
    greedy = SamplingParams(temperature=0.0, max_tokens=1 << 30, ignore_eos=True)
    def timed_decode(batch, steps, warmup, context_end):
        """K decode steps of `batch` requests whose last step runs at
        `context_end` tokens: step function + sampler, timed on the device."""
        start_len = context_end - (steps + warmup)
        seqs = []
        for i in range(batch):
            ids = torch.randint(0, vocab, (start_len + 1,), generator=gen).tolist()
            s = host.Sequence(10_000 + i, ids, host.SamplingParams())
            assert manager.grow(s, start_len)
            s.set_num_computed_tokens(start_len)
            seqs.append(s)
        params = [greedy] * batch
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def one_step():
            entries = []
            for s in seqs:
                n = s.get_num_computed_tokens()
                assert manager.grow(s, n + 1)
                entries.append(host.StepEntry(s, n, 1, [0]))
            logits = runner.step(entries)
            ids = sampler.sample(logits, params, [0] * batch)
            for s in seqs:
                s.set_num_computed_tokens(s.get_num_computed_tokens() + 1)
                s.extend_prompt([1])
            return ids

        for _ in range(warmup):
            one_step()
        torch.cuda.synchronize()
        before = dict(ops.counters)
        graph_before = runner.num_graph_steps
        begin.record()
        for _ in range(steps):
            one_step()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        for s in seqs:
            manager.free(s)
        return ms, runner.num_graph_steps - graph_before, before

    def timed_prefill(tokens, repeats, warmup):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        best = []
        for r in range(warmup + repeats):
            ids = torch.randint(0, vocab, (tokens,), generator=gen).tolist()
            s = host.Sequence(20_000 + r, ids, host.SamplingParams())
            assert manager.grow(s, tokens)
            torch.cuda.synchronize()
            begin.record()
            logits = runner.step([host.StepEntry(s, 0, tokens, [tokens - 1])])
            sampler.sample(logits, [greedy], [0])
            end.record()
            torch.cuda.synchronize()
            if r >= warmup:
                best.append(begin.elapsed_time(end))
            manager.free(s)
        best.sort()
        return best[len(best) // 2]

    def timed_mixed(batch, steps, warmup, context_end, chunk):
        """K steps of `batch` decoding requests beside one `chunk`-token
        portion of a prompt (a new prompt starts when one is through)."""
        start_len = context_end - (steps + warmup)
        seqs = []
        for i in range(batch):
            ids = torch.randint(0, vocab, (start_len + 1,), generator=gen).tolist()
            s = host.Sequence(30_000 + i, ids, host.SamplingParams())
            assert manager.grow(s, start_len)
            s.set_num_computed_tokens(start_len)
            seqs.append(s)
        prompt_len = context_end // chunk * chunk
        state = {"prompt": None, "made": 0, "keys": 0}
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

        def one_step(count):
            if state["prompt"] is None:
                ids = torch.randint(0, vocab, (prompt_len,), generator=gen).tolist()
                state["prompt"] = host.Sequence(40_000 + state["made"], ids, host.SamplingParams())
                state["made"] += 1
            pr = state["prompt"]
            done = pr.get_num_computed_tokens()
            assert manager.grow(pr, done + chunk)
            entries = [host.StepEntry(pr, done, chunk, [chunk - 1])]
            for s in seqs:
                n = s.get_num_computed_tokens()
                assert manager.grow(s, n + 1)
                entries.append(host.StepEntry(s, n, 1, [0]))
            logits = runner.step(entries)
            sampler.sample(logits, [greedy] * (batch + 1), [0] * (batch + 1))
            if count:   # keys that the step's queries read: the portion's causal triangle and every decode context
                state["keys"] += chunk * done + chunk * (chunk + 1) // 2 + sum(s.get_num_computed_tokens() + 1 for s in seqs)
            for s in seqs:
                s.set_num_computed_tokens(s.get_num_computed_tokens() + 1)
                s.extend_prompt([1])
            pr.set_num_computed_tokens(done + chunk)
            if done + chunk >= prompt_len:
                manager.free(pr)
                state["prompt"] = None

        for _ in range(warmup):
            one_step(False)
        torch.cuda.synchronize()
        begin.record()
        for _ in range(steps):
            one_step(True)
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / steps
        for s in seqs:
            manager.free(s)
        if state["prompt"] is not None:
            manager.free(state["prompt"])
        return ms, state["keys"] / steps

    def close():
        """Gives the device memory back (the next rig may need all of it)."""
        nonlocal engine, loaded, runner, manager, sampler
        engine = loaded = runner = manager = sampler = None
        rig.engine = rig.runner = rig.manager = rig.sampler = None
        gc.collect()
        torch.cuda.empty_cache()

    rig = types.SimpleNamespace(engine=engine, runner=runner, manager=manager, sampler=sampler, host=host, gen=gen, vocab=vocab,
                                timed_decode=timed_decode, timed_prefill=timed_prefill, timed_mixed=timed_mixed, close=close)
    return rig


def leave_out(what, cfg):
    """Replaces one kind of kernel of a decode step by nothing, so that the step
    can be timed without it: the difference to the whole step is what the
    kernel costs inside the chain (the rest computes on stale buffers, which
    changes no launch and no byte moved)."""
    from lyapunov_engine_b200 import ops

    H, I, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    product = ops.gemm_skinny

    def products_but(skip):
        def run(out, a, w, splits=1, gated=False):
            if not skip(w, gated):
                product(out, a, w, splits=splits, gated=gated)
        return run
    if what == "norms":
        ops.rmsnorm = lambda *a, **k: None
    elif what == "qkv":
        ops.gemm_skinny_rotary = lambda *a, **k: None
    elif what == "attention":
        ops.attention_decode_bf16 = lambda *a, **k: None
    elif what == "o":
        ops.gemm_skinny = products_but(lambda w, gated: not gated and tuple(w.shape) == (H, cfg["num_attention_heads"] * cfg["head_dim"]) and w.shape[0] < V)
    elif what == "gate_up":
        ops.gemm_skinny = products_but(lambda w, gated: gated)
    elif what == "down":
        ops.gemm_skinny = products_but(lambda w, gated: not gated and tuple(w.shape) == (H, I))
    elif what == "head":
        ops.gemm_skinny = products_but(lambda w, gated: w.shape[0] == V)


def further_points(pk, page, context=8192, steps=24, warmup=6):
    """Decode at batch 1, 8 and 64 and prefill of 2,048 and 8,192 tokens at the
    3B and 8B shapes (context 8192), and the 8B mixed step (64 decoding requests
    beside a 2,048-token portion): tokens a second, with the fraction of the
    HBM or bfloat16 peak each reaches."""
    import torch

    out = {}
    for name in ("3b", "8b"):
        cfg = dict(SHAPES[name])
        # weights, the cache of 65 requests of `context` tokens, activations: leave the size out if it does not fit
        H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
        nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
        weights = 2 * (L * ((nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H) + (1 if cfg["tie_word_embeddings"] else 2) * cfg["vocab_size"] * H)
        cache = 2 * 2 * nkv * hd * L * (65 * (context + 64) + 2 * PREFILL_TOKENS + context)
        free, _ = torch.cuda.mem_get_info()
        if weights + cache + (6 << 30) > free:
            out[f"{name}_skipped"] = f"needs {(weights + cache) >> 30} GiB of device memory, {free >> 30} GiB are free"
            continue
        rig = make_rig(cfg, context, 65, page)
        for b in (1, 8, 64):
            rig.timed_decode(b, 3, 2, context - 200)          # (captures the graph)
            ms, _, _ = rig.timed_decode(b, steps, warmup, context)
            out[f"{name}_decode_b{b}"] = round(b * 1000.0 / ms, 1)
            out[f"{name}_decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, context - (steps - 1) // 2) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
        for tokens in (2048, 8192):
            ms = rig.timed_prefill(tokens, 3, 2)
            out[f"{name}_prefill_{tokens}"] = round(tokens * 1000.0 / ms, 1)
            out[f"{name}_prefill_{tokens}_frac"] = round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
        if name == "8b":
            ms, _ = rig.timed_mixed(64, 8, 3, context, 2048)
            out["8b_mixed_64_2048"] = round((64 + 2048) * 1000.0 / ms, 1)
            out["8b_mixed_64_2048_ms"] = round(ms, 3)
        rig.close()
        del rig
    return out


def run_ours(args):
    global BLOCK_SIZE, CONTEXT
    import torch
    BLOCK_SIZE = args.page
    if args.only and args.context:
        CONTEXT = args.context

    from lyapunov_engine_b200 import SamplingParams, ops

    cfg = dict(SHAPES[args.shapes if args.only else "1b"])
    layers_full = cfg["num_hidden_layers"]
    if args.layers:
        cfg["num_hidden_layers"] = args.layers
    pk = peaks()
    torch.cuda.set_device(0)
    # room for the batches the run times (the prompt beside the decoding requests of a mixed step holds a slot too)
    max_batch = (max(args.batch, args.max_num_seqs, 1) + (args.only == "mixed")) if args.only else 64
    rig = make_rig(cfg, CONTEXT, max_batch, BLOCK_SIZE)
    engine, runner, manager, sampler, host, gen, vocab = rig.engine, rig.runner, rig.manager, rig.sampler, rig.host, rig.gen, rig.vocab
    timed_decode, timed_prefill, timed_mixed = rig.timed_decode, rig.timed_prefill, rig.timed_mixed

    if args.only and args.without:
        leave_out(args.without, cfg)
    if args.only:
        # A short run of one kind of step, for profilers: no CUDA graph, so
        # that every kernel shows as its own launch.
        runner.use_cuda_graphs = not args.no_cuda_graphs
        if args.only == "decode":
            ms, _, _ = timed_decode(args.batch, args.steps, args.warmup, args.context or CONTEXT)
            nbytes = decode_bytes(cfg, args.batch, (args.context or CONTEXT) - (args.steps - 1) // 2)
            print(json.dumps({"only": "decode", "shapes": args.shapes, "batch": args.batch, "context": args.context or CONTEXT,
                              "ms_per_step": round(ms, 4), "tokens_per_s": round(args.batch * 1000.0 / ms, 1),
                              "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4),
                              "layers": cfg["num_hidden_layers"], "cuda_graph": runner.use_cuda_graphs}))
        elif args.only == "mixed":
            chunk = args.tokens or PREFILL_TOKENS
            ms, keys = timed_mixed(args.batch, args.steps, args.warmup, CONTEXT, chunk)
            H, I, L = cfg["hidden_size"], cfg["intermediate_size"], cfg["num_hidden_layers"]
            nh, nkv, hd = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
            per_layer = (nh + 2 * nkv) * hd * H + H * nh * hd + 3 * I * H
            flops = 2 * (chunk + args.batch) * L * per_layer + 2 * (args.batch + 1) * cfg["vocab_size"] * H + 4 * nh * hd * keys * L
            nbytes = decode_bytes(cfg, args.batch, CONTEXT - (args.steps - 1) // 2)
            print(json.dumps({"only": "mixed", "shapes": args.shapes, "decoding": args.batch, "portion": chunk, "context": CONTEXT,
                              "ms_per_step": round(ms, 4), "tokens_per_s": round((args.batch + chunk) * 1000.0 / ms, 1),
                              "layers": cfg["num_hidden_layers"],
                              "tflops": round(flops / (ms * 1e-3) / 1e12, 1),
                              "flops_frac": round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4),
                              "hbm_frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)}))
        else:
            tokens = args.tokens or PREFILL_TOKENS
            ms = timed_prefill(tokens, args.steps, args.warmup)
            print(json.dumps({"only": "prefill", "shapes": args.shapes, "tokens": tokens, "ms": round(ms, 4),
                              "layers": cfg["num_hidden_layers"],
                              "tflops": round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12, 1),
                              "flops_frac": round(prefill_flops(cfg, tokens) / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}))
        return 0

    clocks = ClockSampler()
    clocks.start()
    time.sleep(0.3)

    # ---- headline: batch 8 at context 4096
    batch = 8
    kernels_per_step = None
    # captures the graph for this batch outside the timed call, and runs long enough (some 60 ms) for the clocks
    # to come up from idle: the sampler's start above left the GPU waiting, and a short timed run (20 steps are
    # 16 ms) would otherwise sit on the ramp
    timed_decode(batch, 64, 8, CONTEXT - 200)
    ops.counters["own_kernels"] = ops.counters["library_products"] = 0
    m0 = clocks.mark()
    ms8, graph_steps, _ = timed_decode(batch, args.steps, args.warmup, CONTEXT)
    m1 = clocks.mark()
    value = batch * 1000.0 / ms8

    # kernels per decode step: count launches of one eager step of the same shape
    runner.use_cuda_graphs = False
    ops.counters["own_kernels"] = ops.counters["library_products"] = 0
    timed_decode(batch, 1, 0, CONTEXT - 300)
    kernels_per_step = dict(ops.counters)
    runner.use_cuda_graphs = True

    points = {}
    for b in (1, 64):
        timed_decode(b, 4, 2, CONTEXT - 200)
        ms, _, _ = timed_decode(b, args.steps, args.warmup, CONTEXT)
        points[f"decode_b{b}"] = round(b * 1000.0 / ms, 1)
        points[f"decode_b{b}_ms"] = round(ms, 4)
        points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(cfg, b, CONTEXT - (args.steps - 1) // 2) / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    # ---- prefill of 2,048 tokens
    pre_ms = timed_prefill(PREFILL_TOKENS, 5, 3)
    flops = prefill_flops(cfg, PREFILL_TOKENS)
    prefill = {"value": round(PREFILL_TOKENS * 1000.0 / pre_ms, 1), "tokens": PREFILL_TOKENS, "ms": round(pre_ms, 3),
               "frac": round(flops / (pre_ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)}

    # ---- end to end through the entry point: host tokens in, host tokens out
    # The requests live past the timed window (it holds K steps of all `batch` requests and nothing else); they
    # end afterwards four steps apart, and that drain (8 requests down to none, smaller batch buckets) is timed
    # by itself.
    e2e_steps, e2e_warm = args.steps, args.warmup
    ahead_of_window = 8                      # steps in which requests get their first tokens one after the other
    # The prefill of 8 x 4,000 tokens draws the full 1 kW; for some 0.1 s afterwards the power cap holds the SM
    # clock down (1,725 of 1,965 MHz sampled), which a decode step, bound by latencies, feels.  The window
    # measures steady decoding, so untimed decode steps run first until that has passed.
    settle = 200
    prompt_len = CONTEXT - (e2e_steps + e2e_warm + settle) - ahead_of_window - 1   # the window ends at CONTEXT at the latest
    for i in range(batch):
        sp = SamplingParams(temperature=0.0, max_tokens=e2e_steps + e2e_warm + settle + ahead_of_window + 4 * (i + 1),
                            ignore_eos=True)
        engine.add_request(f"bench-{i}", torch.randint(0, vocab, (prompt_len,), generator=gen).tolist(), sp)
    engine.warm_up(contexts=[CONTEXT, CONTEXT + 64], batches=[1, 2, 4, batch])   # as a server does before its first request
    while any(seq.get_output_len() == 0 for seq, _, _ in engine.active_sequences.values()):
        engine.step()                               # prefill (portions under the token budget)
    for _ in range(settle + e2e_warm):
        engine.step()
    torch.cuda.synchronize()
    m2 = clocks.mark()
    d2h0 = engine.d2h_bytes
    t0 = time.perf_counter()
    produced = 0
    slowest = 0.0
    for _ in range(e2e_steps):
        t1 = time.perf_counter()
        produced += len(engine.step())
        slowest = max(slowest, time.perf_counter() - t1)
    torch.cuda.synchronize()
    e2e_s = time.perf_counter() - t0
    m3 = clocks.mark()
    assert produced == batch * e2e_steps, (produced, batch, e2e_steps)
    d2h = (engine.d2h_bytes - d2h0) / e2e_steps
    live = [host.StepEntry(seq, seq.get_num_computed_tokens(), 1, [0]) for seq, _, _ in engine.active_sequences.values()]
    width = runner._table_width(max(e.start for e in live) + 1)    # as the runner packs a captured decode step
    layout = host.pack_step(live, manager, runner.tile_sizes, batch, [min(width, w) for w in runner.fixed_max_blocks], 0, 0)
    h2d = 4 * layout.total
    t0 = time.perf_counter()
    drain_steps = drain_tokens = 0
    while engine.has_unfinished_requests():
        drain_tokens += len(engine.step())
        drain_steps += 1
    torch.cuda.synchronize()
    drain_s = time.perf_counter() - t0
    e2e = {"value": round(produced / e2e_s, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d,
           "d2h_bytes_per_step": int(d2h), "ms_per_step": round(e2e_s * 1000 / e2e_steps, 4),
           "slowest_step_ms": round(slowest * 1000, 3), "settle_steps": settle,
           "sm_mhz": clocks.summary(m2, max(m3, m2 + 1)).get("sm_mhz"),
           "drain": {"steps": drain_steps, "tokens": drain_tokens, "ms_per_step": round(drain_s * 1000 / max(drain_steps, 1), 4)}}
    clocks.stop()

    # ---- further sizes: the same steps at the layer sizes of Llama-3.2-3B and Llama-3.1-8B, context 8192
    if args.points == "all":
        rig.close()
        del rig, engine, runner, manager, sampler
        try:
            points.update(further_points(pk, BLOCK_SIZE))
        except Exception as e:       # the headline does not depend on the further sizes (they need 90 GB of device memory)
            points["further_sizes_failed"] = f"{type(e).__name__}: {str(e)[:160]}"

    # the timed steps run at contexts CONTEXT - steps + 1 .. CONTEXT: count the bytes of their mean
    mean_context = CONTEXT - (args.steps - 1) // 2
    nbytes = decode_bytes(cfg, batch, mean_context)
    achieved = nbytes / (ms8 * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s, Llama-3.2-1B shapes, batch 8, context 4096",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(ms8, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "config": {"model": "Llama-3.2-1B shapes", "layers": cfg["num_hidden_layers"], "layers_of_model": layers_full,
                   "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
                   "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
                   "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"], "global_batch": batch,
                   "seq_len": CONTEXT, "page": BLOCK_SIZE, "parallelism": "single GPU",
                   "timing": "CUDA events; working set per step > L2", "cuda_graph": graph_steps > 0,
                   "peaks": pk["source"]},
        "clocks": clocks.summary(m0, m1),
        "e2e": e2e,
        "gpu_launches": kernels_per_step["own_kernels"] * args.steps,
        "library_products": kernels_per_step["library_products"] * args.steps,
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4), "bytes_per_step": nbytes, "mean_context": mean_context},
        "points": points,
    }
    print(json.dumps(line))
    return 0


def run_reference(args):
    """The unmodified reference (installed under baseline/_ref with its own
    setup.py, CUDA extension built for sm_100 through its TORCH_CUDA_ARCH_LIST
    switch) through its own public API: LlamaForCausalLM with random weights,
    LLMEngine.add_request / step.  Same shapes, batch, context and greedy
    sampling as the other arm; float16, the only type its kernels take."""
    why = reference_unavailable()
    if why:
        print(json.dumps({"impl": "reference", "unavailable": why}))
        return 0
    try:
        line = _reference_line(args)
    except Exception as e:  # the reference's own failure is a result, not a crash of the benchmark
        line = {"impl": "reference", "unavailable": f"the reference failed while running: {type(e).__name__}: {str(e)[:200]}"}
    print(json.dumps(line))
    return 0


def reference_unavailable() -> str:
    ref = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref, "lyapunov_engine")):
        return "IanConery/lyapunov-engine is not installed under baseline/_ref (pip install --no-index --target baseline/_ref of the reference)"
    if not any(f.startswith("_C") and f.endswith(".so") for f in os.listdir(os.path.join(ref, "lyapunov_engine"))):
        return "the reference was installed without its CUDA extension; its engine then returns nothing from step()"
    return ""


def _reference_line(args):
    import torch

    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    from lyapunov_engine.engine.llm_engine import EngineConfig, LLMEngine
    from lyapunov_engine.engine.sampling import SamplingParams
    from lyapunov_engine.models.llama import LlamaConfig, LlamaForCausalLM

    c = LLAMA_1B
    torch.manual_seed(0)
    torch.cuda.set_device(0)
    config = LlamaConfig(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], intermediate_size=c["intermediate_size"],
                         num_hidden_layers=c["num_hidden_layers"], num_attention_heads=c["num_attention_heads"],
                         num_key_value_heads=c["num_key_value_heads"], head_dim=c["head_dim"],
                         max_position_embeddings=c["max_position_embeddings"], rms_norm_eps=c["rms_norm_eps"],
                         rope_theta=c["rope_theta"])
    model = LlamaForCausalLM(config)
    with torch.no_grad():
        for name, p in model.named_parameters():
            if p.dim() == 2:
                p.normal_(0.0, 0.02)
    model = model.to(dtype=torch.float16, device="cuda:0").eval()
    batch = 8
    steps, warmup = args.steps, max(args.warmup, 3)
    prompt_len = CONTEXT - (steps + warmup) - 1
    engine = LLMEngine(model, EngineConfig(model_config=config, num_blocks=batch * (CONTEXT // BLOCK_SIZE + 2),
                                           block_size=BLOCK_SIZE, max_num_seqs=64,
                                           max_num_batched_tokens=batch * CONTEXT + 64, dtype=torch.float16,
                                           device="cuda:0"))
    gen = torch.Generator().manual_seed(0)
    sp = SamplingParams(temperature=0.0, max_tokens=steps + warmup + 1, ignore_eos=True)
    for i in range(batch):
        engine.add_request(f"bench-{i}", torch.randint(0, c["vocab_size"], (prompt_len,), generator=gen).tolist(), sp)
    clocks = ClockSampler()
    clocks.start()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    engine.step()                                   # the reference runs every waiting prompt whole in one step
    torch.cuda.synchronize()
    prefill_s = time.perf_counter() - t0
    for _ in range(warmup):
        engine.step()
    torch.cuda.synchronize()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    m0 = clocks.mark()
    t0 = time.perf_counter()
    begin.record()
    produced = 0
    for _ in range(steps):
        produced += len(engine.step())
    end.record()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    m1 = clocks.mark()
    clocks.stop()
    ms = begin.elapsed_time(end) / steps
    nbytes = decode_bytes(c, batch, CONTEXT)
    pk = peaks()
    return {
        "impl": "reference",
        "metric": "decode tokens/s, Llama-3.2-1B shapes, batch 8, context 4096",
        "value": round(batch * 1000.0 / ms, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "fp16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "config": {"model": "Llama-3.2-1B shapes", "layers": c["num_hidden_layers"], "layers_of_model": c["num_hidden_layers"],
                   "global_batch": batch, "seq_len": CONTEXT, "page": BLOCK_SIZE, "parallelism": "single GPU",
                   "timing": "CUDA events around LLMEngine.step(); working set per step > L2",
                   "note": "the reference's model never writes its KV cache, so its decode reads pages it never filled"},
        "clocks": clocks.summary(m0, m1),
        "e2e": {"value": round(produced / wall, 1), "unit": "tokens/s", "h2d_bytes_per_step": None, "d2h_bytes_per_step": None,
                "ms_per_step": round(wall * 1000 / steps, 4)},
        "gpu_launches": None,
        "prefill": {"value": round(batch * prompt_len / prefill_s, 1), "tokens": batch * prompt_len, "ms": round(prefill_s * 1000, 2)},
        "roofline": {"bound": "hbm", "achieved": round(nbytes / (ms * 1e-3) / 1e9, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)},
    }


# The reference's serving benchmark (benchmarks/bench_serving.py:10-43: the model; 46-77: what is timed): a small
# Llama with random weights, every request a prompt of 128 tokens (ids 100, 101, ...), 32 tokens generated
# greedily, batches of 1, 4, 8, 16.  TTFT is the first step (all prompts in it), ITL the mean of the steps after
# it, each with a device synchronisation on both sides; tok/s counts prompt and generated tokens over the sum of
# those times.  Here in bfloat16, and each batch runs twice untimed first (kernels compiled, step graphs captured).
SERVING_MODEL = {
    "architectures": ["LlamaForCausalLM"], "model_type": "llama", "vocab_size": 32000, "hidden_size": 1024,
    "intermediate_size": 4096, "num_hidden_layers": 8, "num_attention_heads": 16, "num_key_value_heads": 4,
    "head_dim": 64, "max_position_embeddings": 8192, "rms_norm_eps": 1e-5, "rope_theta": 10000.0,
    "rope_scaling": None, "tie_word_embeddings": False, "hidden_act": "silu", "attention_bias": False,
    "mlp_bias": False, "bos_token_id": 1, "eos_token_id": 2, "torch_dtype": "bfloat16",
}


def run_serving(args):
    import torch

    from lyapunov_engine_b200 import EngineConfig, LLMEngine, SamplingParams, load_model

    prompt_len, generated = 128, 32
    loaded = load_model(config=dict(SERVING_MODEL), random_seed=0, dtype="bfloat16", device="cuda:0", max_model_len=1024)
    rows = []
    for batch in args.batch_sizes:
        engine = LLMEngine(loaded, EngineConfig(num_blocks=2048, block_size=BLOCK_SIZE, max_num_seqs=batch,
                                                max_num_batched_tokens=4096, dtype="bfloat16", device="cuda:0",
                                                max_model_len=1024))
        for run in range(3):        # two untimed runs (a prompt step is captured as a graph at its second use), one timed
            for _ in range(batch):
                engine.add_request([100 + i for i in range(prompt_len)],
                                   SamplingParams(temperature=0.0, max_tokens=generated, ignore_eos=True))
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            engine.step()
            torch.cuda.synchronize()
            ttft = (time.perf_counter() - t0) * 1e3
            steps = []
            while engine.has_unfinished_requests():
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                engine.step()
                torch.cuda.synchronize()
                steps.append((time.perf_counter() - t0) * 1e3)
        total_s = (ttft + sum(steps)) / 1e3
        rows.append({"batch": batch, "ttft_ms": round(ttft, 3), "itl_ms": round(sum(steps) / max(len(steps), 1), 4),
                     "decode_steps": len(steps),
                     "tokens_per_s": round(batch * (prompt_len + generated) / total_s, 1)})
        print(f"batch {batch:3d}: TTFT {ttft:7.3f} ms   ITL {rows[-1]['itl_ms']:7.4f} ms   {rows[-1]['tokens_per_s']:10.1f} tok/s",
              file=sys.stderr)
        del engine
    print(json.dumps({"only": "serving", "model": "V32000 H1024 I4096 L8 nh16 nkv4 hd64, random weights", "dtype": "bf16",
                      "prompt": prompt_len, "generated": generated, "rows": rows}))
    return 0


# The reference's kernel benchmark (benchmarks/bench_kernels.py:7-27: CUDA events, the median of 100 launches after
# 25 warm-ups; 40-41 and 74-79: the grids): RMSNorm with the residual add over widths 2048, 4096, 8192 and 32 to
# 4,096 tokens; causal attention of one prompt of 512 to 4,096 tokens, 32 heads of 128 in 8 groups (here over the
# paged cache, pages of 16).  Each row carries the bytes or flops the kernel must move and the share of the measured
# peak that makes.  Every launch works on a fresh set of tensors until 256 MB have gone round (more than L2 holds).
def run_kernels(args):
    import torch

    from lyapunov_engine_b200 import ops

    pk = peaks()
    dev = "cuda:0"

    def median_us(launch, sets):
        for i in range(25):
            launch(i % sets)
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(100)]
        torch.cuda.synchronize()
        for i, (a, b) in enumerate(events):
            a.record()
            launch(i % sets)
            b.record()
        torch.cuda.synchronize()
        times = sorted(a.elapsed_time(b) * 1e3 for a, b in events)
        return times[len(times) // 2]

    rows = []
    for hidden in (2048, 4096, 8192):
        for tokens in (32, 256, 1024, 4096):
            nbytes = tokens * hidden * (4 + 2 + 4 + 2) + 4 * hidden       # residual in and out (float32), delta in, normed out
            sets = max(2, min(64, (256 << 20) // nbytes + 1))
            resid = [torch.randn(tokens, hidden, device=dev) for _ in range(sets)]
            delta = [torch.randn(tokens, hidden, device=dev).bfloat16() for _ in range(sets)]
            out = [torch.empty(tokens, hidden, device=dev, dtype=torch.bfloat16) for _ in range(sets)]
            weight = torch.ones(hidden, device=dev)
            us = median_us(lambda i: ops.rmsnorm(out[i], resid[i], delta[i], weight, 1e-5), sets)
            rows.append({"kernel": "rmsnorm + residual", "hidden": hidden, "tokens": tokens, "us": round(us, 2),
                         "gbs": round(nbytes / us / 1e3, 1), "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)})
            del resid, delta, out
    nh, nkv, hd, page = 32, 8, 128, BLOCK_SIZE
    status = ops.new_status(dev)
    for seq in (512, 1024, 2048, 4096):
        pages = seq // page
        k = torch.randn(pages + 1, nkv, page, hd, device=dev).bfloat16()
        v = torch.randn(pages + 1, nkv, page, hd, device=dev).bfloat16()
        q = torch.randn(seq, (nh + 2 * nkv) * hd, device=dev).bfloat16()
        out = torch.empty(seq, nh * hd, device=dev, dtype=torch.bfloat16)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        cu = torch.tensor([0, seq], dtype=torch.int32, device=dev)
        ctx = torch.zeros(1, dtype=torch.int32, device=dev)
        tiles = (seq + 127) // 128
        tile_request = torch.zeros(tiles, dtype=torch.int32, device=dev)
        tile_q0 = torch.arange(0, seq, 128, dtype=torch.int32, device=dev)
        us = median_us(lambda i: ops.attention_prefill_tc_bf16(out, q, q.stride(0), k, v, table, cu, ctx, tile_request, tile_q0,
                                                               tiles, nh, nkv, hd, page, 0, hd ** -0.5, status), 1)
        flops = 4 * nh * hd * seq * (seq + 1) // 2
        rows.append({"kernel": "prefill attention (tcgen05), 32 heads of 128 in 8 groups", "tokens": seq, "us": round(us, 2),
                     "tflops": round(flops / us / 1e6, 1), "bf16_frac": round(flops / us / 1e6 / pk["bf16_tflops"], 3)})
    ops.check_status(status)
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items()), file=sys.stderr)
    print(json.dumps({"only": "kernels", "peaks": pk["source"], "rows": rows}))
    return 0


# ---------------------------------------------------------------- the Sulepel design beside Llama at equal sizes
SULEPEL_CHUNK = 2048       # keys a chunked layer's query sees at most
SULEPEL_LATENT = 128       # latent size (the tensor-core attention kernels end at a head size of 128)


def sulepel_config(llama: dict) -> dict:
    """A Sulepel model with the width, feed-forward size, heads, head size, layer count and vocabulary of the given
    Llama shapes: three latent-attention layers, then one chunked-attention layer, and so on."""
    nh, nkv, hd = llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"]
    mlp = {"kind": "dense", "ff": llama["intermediate_size"], "limit": 7.0}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": nh, "dim": hd, "vdim": hd, "kv_rank": SULEPEL_LATENT, "scale": hd ** -0.5}}
    chunked = {"type": "attention", "mlp": mlp,
               "mixer": {"heads": nh, "kv_heads": nkv, "dim": hd, "vdim": hd, "mask": {"size": SULEPEL_CHUNK}, "scale": hd ** -0.5}}
    return {"architecture": "Sulepel", "vocab": llama["vocab_size"], "width": llama["hidden_size"],
            "norm": {"eps": 1e-5, "groups": 4}, "canon": {"taps": 4},
            "layers": [chunked if i % 4 == 3 else latent for i in range(llama["num_hidden_layers"])]}


def sulepel_decode_bytes(cfg, batch, context):
    """Bytes one decode step of a Sulepel model must read (bfloat16 weights once, the cached latents and the keys and
    values of the current chunk of every live request)."""
    W, V = cfg["width"], cfg["vocab"]
    total = 2 * V * W + 4 * W
    for layer in cfg["layers"]:
        m, F = layer["mixer"], layer["mlp"]["ff"]
        nh, d, e = m["heads"], m["dim"], m["vdim"]
        total += 2 * 3 * F * W + 4 * (2 + cfg["canon"]["taps"]) * W
        if layer["type"] == "latent_attention":
            r = m["kv_rank"]
            total += 2 * ((nh * d + r + nh) * W + nh * d * r + nh * e * r + W * nh * e) + 2 * batch * context * r
        else:
            seen = (context - 1) % m["mask"]["size"] + 1
            total += 2 * ((nh * d + m["kv_heads"] * (d + e) + nh) * W + W * nh * e) + 2 * batch * seen * m["kv_heads"] * (d + e)
    return total


def sulepel_prefill_flops(cfg, tokens):
    W, V = cfg["width"], cfg["vocab"]
    flops = 2 * V * W
    pairs = tokens * (tokens + 1) // 2
    for layer in cfg["layers"]:
        m, F = layer["mixer"], layer["mlp"]["ff"]
        nh, d, e = m["heads"], m["dim"], m["vdim"]
        flops += 2 * tokens * 3 * F * W
        if layer["type"] == "latent_attention":
            r = m["kv_rank"]
            # as computed here: queries carried into the latent space, attention over latents, results carried out
            flops += 2 * tokens * ((nh * d + r + nh) * W + nh * d * r + nh * e * r + W * nh * e) + 4 * nh * r * pairs
        else:
            c = m["mask"]["size"]
            full, rest = divmod(tokens, c)
            seen = full * (c * (c + 1) // 2) + rest * (rest + 1) // 2
            flops += 2 * tokens * ((nh * d + m["kv_heads"] * (d + e) + nh) * W + W * nh * e) + 2 * nh * (d + e) * seen
    return flops


def sulepel_kernel_rows(pk, llama):
    """Each kernel the design adds, alone, beside the like kernel of the Llama path at the same sizes: microseconds
    per launch inside a captured graph, over rotating tensors, and the share of the measured copy bandwidth that the
    bytes it must move make."""
    import torch

    from lyapunov_engine_b200 import ops

    dev = "cuda:0"
    W, nh, nkv, hd, F = llama["hidden_size"], llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["intermediate_size"]
    r, page = SULEPEL_LATENT, BLOCK_SIZE
    rows = []

    def median_us(launch, sets):
        """Microseconds per launch inside a captured graph of at least 16 launches over rotating tensors (a launch
        by itself from the host costs more than these kernels run; inside a step they are nodes of such a graph)."""
        n = max(sets, 16)
        for i in range(n):
            launch(i % sets)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                launch(i % sets)
        for _ in range(3):
            graph.replay()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(15)]
        torch.cuda.synchronize()
        for a, b in events:
            a.record()
            graph.replay()
            b.record()
        torch.cuda.synchronize()
        times = sorted(a.elapsed_time(b) * 1e3 / n for a, b in events)
        return times[len(times) // 2]

    def row(kernel, like, tokens, nbytes, launch, sets):
        us = median_us(launch, sets)
        rows.append({"kernel": kernel, "like": like, "tokens": tokens, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                     "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)})

    def sets_for(nbytes):
        return max(2, min(64, (256 << 20) // max(nbytes, 1) + 1))

    bf = torch.bfloat16
    status = ops.new_status(dev)
    for T in (8, 2048):
        # norms
        nbytes = T * W * (4 + 2 + 4 + 2) + 4 * W
        n = sets_for(nbytes)
        resid = [torch.randn(T, W, device=dev) for _ in range(n)]
        delta = [torch.randn(T, W, device=dev).to(bf) for _ in range(n)]
        out = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(n)]
        weight = torch.ones(W, device=dev)
        row("rmsnorm in 4 groups + residual", "", T, nbytes, lambda i: ops.rmsnorm(out[i], resid[i], delta[i], weight, 1e-5, groups=4), n)
        row("rmsnorm + residual", "rmsnorm in 4 groups + residual", T, nbytes, lambda i: ops.rmsnorm(out[i], resid[i], delta[i], weight, 1e-5), n)
        # the short convolution (4 taps): reads and writes the rows once, the state of every request once
        reqs = T if T <= 64 else 1
        q_lens = [T // reqs] * reqs
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        treq = torch.tensor([b for b, m in enumerate(q_lens) for _ in range(0, m, 16)], dtype=torch.int32, device=dev)
        tq0 = torch.tensor([s0 for m in q_lens for s0 in range(0, m, 16)], dtype=torch.int32, device=dev)
        slots = torch.arange(reqs, dtype=torch.int32, device=dev)
        state = torch.zeros(reqs + 1, 3, W, device=dev)
        taps = torch.randn(4, W, device=dev)
        nbytes = T * W * 4 + reqs * 3 * W * 8 + 16 * W
        row("short convolution, 4 taps", "", T, nbytes, lambda i: ops.short_conv(delta[i], out[i], taps, state, slots, cu, treq, tq0, treq.numel()), n)
        # embeddings
        table = torch.randn(32000, W, device=dev).to(bf)
        ids = torch.randint(0, 32000, (T,), dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        rates = torch.rand((W + 1) // 2, device=dev)
        nbytes = T * W * 6
        row("embedding + sinusoid", "", T, nbytes, lambda i: ops.embed_sinusoid(resid[i], table, ids, pos, rates, status), n)
        row("embedding", "embedding + sinusoid", T, nbytes, lambda i: ops.embed(resid[i], table, ids, status), n)
        del resid, delta, out
        # cache writes: the latent with its norm, unrotated keys and values, and the rotary write of the Llama path
        pages = (T + page - 1) // page + 1
        btab = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        req0 = torch.zeros(T, dtype=torch.int32, device=dev)
        width_l = nh * hd + r + 8
        proj = torch.randn(T, width_l, device=dev).to(bf)
        lat = torch.zeros(pages + 1, 1, page, r, device=dev, dtype=bf)
        wn = torch.ones(r, device=dev)
        row("latent norm + cache write", "", T, T * r * 4, lambda i: ops.latent_norm_store(proj, nh * hd, r, wn, 1e-5, lat, pos, req0, btab, page, status), 1)
        qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev).to(bf)
        kc = torch.zeros(pages + 1, nkv, page, hd, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        row("key/value cache write", "", T, T * 2 * nkv * hd * 4, lambda i: ops.kv_store(qkv, nh * hd, (nh + nkv) * hd, kc, vc, pos, req0, btab, nkv, hd, page, status), 1)
        cos_sin = torch.randn(max(T, 16), hd, device=dev)
        row("rotary + key/value cache write", "latent norm + cache write; key/value cache write", T, T * ((nh + nkv) * hd * 4 + nkv * hd * 4),
            lambda i: ops.rope_kv_write(qkv, kc, vc, cos_sin, pos, req0, btab, nh, nkv, hd, page, True, status), 1)
        # per-head products and the gate
        w_into = torch.randn(nh, r, hd, device=dev).to(bf)
        w_out = torch.randn(nh, hd, r, device=dev).to(bf)
        ql = torch.empty(T, nh * r, device=dev, dtype=bf)
        ho = torch.empty(T, nh * hd, device=dev, dtype=bf)
        gate = torch.randn(T, nh, device=dev).to(bf)
        nbytes = 2 * (nh * r * hd + T * nh * (hd + r))
        if T <= 64:
            row("per-head product into the latent space (FP32 pipes)", "", T, nbytes, lambda i: ops.gemm_heads(ql, proj[:, :nh * hd], w_into), 1)
            row("per-head product out of it, with gate (FP32 pipes)", "", T, nbytes, lambda i: ops.gemm_heads(ho, ql, w_out, gate), 1)
        else:
            row("per-head gate", "", T, T * nh * hd * 4, lambda i: ops.head_gate(ho, gate, nh, hd), 1)
        # gated products
        x = torch.randn(T, W, device=dev).to(bf)
        wgu = [torch.randn(2 * F, W, device=dev).to(bf) for _ in range(4)]
        act = torch.empty(T, F, device=dev, dtype=bf)
        nbytes = 2 * (2 * F * W + T * W + T * F)
        ws = None
        from lyapunov_engine_b200.engine.runtime import Workspace
        ws = Workspace(torch.device(dev))
        row("gate/up product, clamped activation", "", T, nbytes, lambda i: ops.gated_linear(act, x, wgu[i], ws, status, (ops.GLU_CLAMPED, 1.702, 7.0)), 4)
        row("gate/up product, SiLU", "gate/up product, clamped activation", T, nbytes, lambda i: ops.gated_linear(act, x, wgu[i], ws, status), 4)
        del wgu
    # decode attention, 8 requests at 4,096 keys: all heads over one pool of latents, beside grouped-query attention
    B, ctx = 8, 4096
    pages = B * ctx // page
    btab = torch.arange(pages, dtype=torch.int32, device=dev).view(B, -1).contiguous()
    cu = torch.arange(B + 1, dtype=torch.int32, device=dev)
    before = torch.full((B,), ctx - 1, dtype=torch.int32, device=dev)
    lat = torch.randn(pages + 1, 1, page, r, device=dev).to(bf)
    q = torch.randn(B, nh * r, device=dev).to(bf)
    o = torch.empty(B, nh * r, device=dev, dtype=bf)
    from lyapunov_engine_b200.parts import attention_kernels as ak
    splits = ak.decode_splits(B, nh, 1, ctx, r)
    floats = ops.attention_decode_scratch_floats(r, B, nh, splits)
    scratch = torch.zeros(max(floats, 1), device=dev)
    row(f"decode attention over latents ({nh} heads on one pool of {r}, {splits} splits)", "", B, 2 * B * ctx * r,
        lambda i: ops.attention_decode_bf16(o, scratch, q, q.stride(0), lat, lat, btab, cu, before, None, B, nh, 1, r, page, 0, hd ** -0.5, splits, status), 1)
    kc = torch.randn(pages + 1, nkv, page, hd, device=dev).to(bf)
    vc = torch.randn(pages + 1, nkv, page, hd, device=dev).to(bf)
    q2 = torch.randn(B, nh * hd, device=dev).to(bf)
    o2 = torch.empty(B, nh * hd, device=dev, dtype=bf)
    splits2 = ak.decode_splits(B, nh, nkv, ctx, hd)
    scratch2 = torch.zeros(max(ops.attention_decode_scratch_floats(hd, B, nh, splits2), 1), device=dev)
    hs = torch.rand(nh, device=dev) + 0.5
    row(f"decode attention, {nh} heads of {hd} in {nkv} groups ({splits2} splits)", "decode attention over latents", B, 2 * B * ctx * 2 * nkv * hd,
        lambda i: ops.attention_decode_bf16(o2, scratch2, q2, q2.stride(0), kc, vc, btab, cu, before, None, B, nh, nkv, hd, page, 0, hd ** -0.5, splits2, status), 1)
    row("the same with a factor per head and chunks", "", B, 2 * B * ((ctx - 1) % SULEPEL_CHUNK + 1) * 2 * nkv * hd,
        lambda i: ops.attention_decode_bf16(o2, scratch2, q2, q2.stride(0), kc, vc, btab, cu, before, None, B, nh, nkv, hd, page, -SULEPEL_CHUNK, hd ** -0.5,
                                            ak.decode_splits(B, nh, nkv, SULEPEL_CHUNK, hd), status, head_scale=hs), 1)
    ops.check_status(status)
    return rows


def run_sulepel(args):
    """--only sulepel: decode (1 and 8 requests at --context) and prefill (2,048 tokens) of a Sulepel model beside the
    Llama model of the same width, feed-forward size, heads, layers and vocabulary (random weights, bfloat16), and
    the design's own kernels alone beside their likes."""
    global BLOCK_SIZE
    import torch

    BLOCK_SIZE = args.page
    pk = peaks()
    context = args.context or CONTEXT
    if args.profile_step:
        # a few steps launch by launch (no captured graph) of a model of --layers layers (4 by default), for a profiler
        llama = dict(SHAPES[args.shapes])
        llama["num_hidden_layers"] = args.layers or 4
        rig = make_rig(sulepel_config(llama), context, 8, args.page)
        rig.runner.use_cuda_graphs = False
        if args.profile_step == "decode":
            ms, _, _ = rig.timed_decode(args.batch, 2, 2, context)
        else:
            ms = rig.timed_prefill(args.tokens or PREFILL_TOKENS, 1, 2)
        print(json.dumps({"only": "sulepel", "profile_step": args.profile_step, "layers": llama["num_hidden_layers"], "ms": round(ms, 3)}))
        return 0
    out = {"only": "sulepel", "peaks": pk["source"], "context": context, "sizes": {}}
    for name in ([args.shapes] if args.shapes != "1b" or args.layers else ["1b", "3b"]):
        llama = dict(SHAPES[name])
        if args.layers:
            llama["num_hidden_layers"] = args.layers
        su = sulepel_config(llama)
        res = {}
        for label, cfg in (("sulepel", su), ("llama", llama)):
            rig = make_rig(cfg, context, 8, args.page)
            for b in (1, 8):
                rig.timed_decode(b, 3, 2, context - 200)
                ms, graph_steps, _ = rig.timed_decode(b, 24, 6, context)
                nbytes = sulepel_decode_bytes(cfg, b, context - 12) if label == "sulepel" else decode_bytes(cfg, b, context - 12)
                res[f"{label}_decode_b{b}_ms"] = round(ms, 4)
                res[f"{label}_decode_b{b}_tokens_per_s"] = round(b * 1000.0 / ms, 1)
                res[f"{label}_decode_b{b}_hbm_frac"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                res[f"{label}_decode_b{b}_graph_steps"] = graph_steps
            ms = rig.timed_prefill(PREFILL_TOKENS, 3, 2)
            flops = sulepel_prefill_flops(cfg, PREFILL_TOKENS) if label == "sulepel" else prefill_flops(cfg, PREFILL_TOKENS)
            res[f"{label}_prefill_{PREFILL_TOKENS}_ms"] = round(ms, 3)
            res[f"{label}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS * 1000.0 / ms, 1)
            res[f"{label}_prefill_{PREFILL_TOKENS}_bf16_frac"] = round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
            rig.close()
            del rig
            torch.cuda.empty_cache()
        out["sizes"][name] = res
        for k, v in res.items():
            print(f"{name}  {k} = {v}", file=sys.stderr)
    rows = sulepel_kernel_rows(pk, dict(SHAPES["1b"]))
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items() if v != ""), file=sys.stderr)
    out["kernels"] = rows
    print(json.dumps(out))
    return 0


def kaditar_config(llama: dict, window: int = 2048) -> dict:
    """A Kaditar model with the width, layer count, vocabulary and projection sizes of the given Llama shapes: as
    many heads, each with two maps of half the head size (the same rows of q, k, v and o; a key head in the cache is
    as wide as Llama's), four copies of the stream, dense layers in turn with routed ones whose two
    chosen experts and shared expert together have the dense layer's size."""
    nh, nkv, hd, I = llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["intermediate_size"]
    mixer = {"heads": nh, "kv_heads": nkv, "dim": hd // 2, "vdim": hd, "scale": (hd // 2) ** -0.5, "diff": 0.3,
             "rot": {"dims": hd // 4, "base": float(llama["rope_theta"])}, "mask": {"size": window}}
    dense = {"kind": "dense", "ff": I}
    routed = {"kind": "moe", "expert": {"ff": I // 4}, "router": {"experts": 16, "top": 2}, "shared": {"ff": I // 2}}
    return {"architecture": "Kaditar", "vocab": llama["vocab_size"], "width": llama["hidden_size"], "norm": {"eps": 1e-5},
            "streams": 4, "logit_softcap": 30.0,
            "layers": [{"type": "attention", "mixer": mixer, "mlp": routed if i % 2 else dense}
                       for i in range(llama["num_hidden_layers"])]}


def kaditar_decode_bytes(cfg, batch, context):
    """Bytes one decode step of a Kaditar model must read: every weight it uses once (of the routed layers the shared
    expert and at most batch * top experts), the keys and values inside every live request's window."""
    W, V = cfg["width"], cfg["vocab"]
    total = 2 * V * W + 8 * W
    for layer in cfg["layers"]:
        m, f = layer["mixer"], layer["mlp"]
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        total += 2 * ((H * 2 * d + G * 2 * d + G * e) * W + W * H * e) + 16 * W
        total += 2 * batch * min(context, m["mask"]["size"]) * G * 2 * max(2 * d, e)
        if f["kind"] == "dense":
            total += 2 * 3 * f["ff"] * W
        else:
            used = min(f["router"]["experts"], batch * f["router"]["top"])
            total += 2 * 3 * W * (used * f["expert"]["ff"] + f["shared"]["ff"]) + 4 * (f["router"]["experts"] + 1) * W
    return total


def kaditar_prefill_flops(cfg, tokens):
    """As computed here: scores over keys that hold both maps side by side (twice the needed width)."""
    W, V = cfg["width"], cfg["vocab"]
    flops = 2 * V * W
    for layer in cfg["layers"]:
        m, f = layer["mixer"], layer["mlp"]
        H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        w = m["mask"]["size"]
        seen = sum(min(t + 1, w) for t in range(tokens))
        flops += 2 * tokens * ((H * 2 * d + G * 2 * d + G * e) * W + W * H * e) + 4 * (2 * H) * max(2 * d, e) * seen
        if f["kind"] == "dense":
            flops += 2 * tokens * 3 * f["ff"] * W
        else:
            flops += 2 * tokens * (3 * W * (f["router"]["top"] * f["expert"]["ff"] + f["shared"]["ff"]) + (f["router"]["experts"] + 1) * W)
    return flops


def kaditar_kernel_rows(pk, llama):
    """Each kernel the design adds, alone, beside the like kernel of the Llama path at the same sizes: microseconds
    per launch inside a captured graph over rotating tensors, the share of the measured copy bandwidth that the bytes
    it must move make, and for the products the share of the measured bfloat16 rate."""
    import torch

    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Workspace

    dev, bf = "cuda:0", torch.bfloat16
    cfg = kaditar_config(llama)
    W, nh, nkv, hd, I = llama["hidden_size"], llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["intermediate_size"]
    m = cfg["layers"][0]["mixer"]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    khd = max(2 * d, e)
    moe = cfg["layers"][1]["mlp"]
    E, top, F = moe["router"]["experts"], moe["router"]["top"], moe["expert"]["ff"]
    page = BLOCK_SIZE
    rows = []

    def median_us(launch, sets):
        n = max(sets, 16)
        for i in range(n):
            launch(i % sets)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(n):
                launch(i % sets)
        for _ in range(3):
            graph.replay()
        events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(15)]
        torch.cuda.synchronize()
        for a, b in events:
            a.record()
            graph.replay()
            b.record()
        torch.cuda.synchronize()
        times = sorted(a.elapsed_time(b) * 1e3 / n for a, b in events)
        return times[len(times) // 2]

    def row(kernel, like, tokens, nbytes, launch, sets, flops=0):
        us = median_us(launch, sets)
        r = {"kernel": kernel, "like": like, "tokens": tokens, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
             "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if flops:
            r["tflops"] = round(flops / us / 1e6, 1)
            r["bf16_frac"] = round(flops / us / 1e6 / pk["bf16_tflops"], 3)
        rows.append(r)

    def sets_for(nbytes):
        return max(2, min(64, (256 << 20) // max(nbytes, 1) + 1))

    status = ops.new_status(dev)
    ws = Workspace(dev)
    for T in (1, 8, 2048):
        S = cfg["streams"]
        nbytes = T * W * (8 * S + 2 + 2) + 8 * W
        n = sets_for(nbytes)
        copies = [torch.randn(T, S, W, device=dev) for _ in range(n)]
        delta = [torch.randn(T, W, device=dev).to(bf) for _ in range(n)]
        out = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(n)]
        weight, bias = torch.ones(W, device=dev), torch.zeros(W, device=dev)
        mix, post, pre = torch.eye(S, device=dev).contiguous(), torch.ones(S, device=dev), torch.full((S,), 1.0 / S, device=dev)
        row(f"stream of {S} copies: update + read + layer norm", "rmsnorm + residual", T, nbytes,
            lambda i: ops.stream_norm(out[i], copies[i], weight, bias, 1e-5, delta=delta[i], mix=mix, post=post, pre=pre), n)
        resid = [c[:, 0].contiguous() for c in copies]
        row("rmsnorm + residual", "", T, T * W * 12 + 4 * W, lambda i: ops.rmsnorm(out[i], resid[i], delta[i], weight, 1e-5), n)
        # rotary pairs + bias + spread queries + cache write, beside the rotary write of the Llama path
        cols = (H + G) * 2 * d + G * e
        nbytes = T * 2 * (cols + 2 * H * khd + 2 * G * khd) + 4 * cols
        n = sets_for(nbytes)
        pages = (T + page - 1) // page
        src = [torch.randn(T, cols, device=dev).to(bf) for _ in range(n)]
        qw = [torch.empty(T, 2 * H * khd, device=dev, dtype=bf) for _ in range(n)]
        kc = torch.zeros(pages + 1, G, page, khd, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        b_ = torch.zeros(cols, device=dev)
        rates = torch.rand(m["rot"]["dims"] // 2, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        req = torch.zeros(T, dtype=torch.int32, device=dev)
        table = torch.arange(pages, dtype=torch.int32, device=dev)[None, :].contiguous()
        row("rotary pairs + bias + spread queries + cache write", "rotary + cache write", T, nbytes,
            lambda i: ops.rope_pairs_store(qw[i], src[i], b_, kc, vc, rates, pos, req, table, H, G, 2, d, e, m["rot"]["dims"],
                                           khd, page, True, status), n)
        qkv = [torch.randn(T, (nh + 2 * nkv) * hd, device=dev).to(bf) for _ in range(n)]
        kc2 = torch.zeros(pages + 1, nkv, page, hd, device=dev, dtype=bf)
        vc2 = torch.zeros_like(kc2)
        cos_sin = torch.rand(T + 1, hd, device=dev)
        row("rotary + cache write", "", T, T * 2 * ((nh + 2 * nkv) * hd + (nh + 2 * nkv) * hd), 
            lambda i: ops.rope_kv_write(qkv[i], kc2, vc2, cos_sin, pos, req, table, nh, nkv, hd, page, True, status), n)
        # the maps of a head combined
        nbytes = T * 2 * (2 * H * khd + H * e)
        n = sets_for(nbytes)
        attn = [torch.randn(T, 2 * H * khd, device=dev).to(bf) for _ in range(n)]
        comb = [torch.empty(T, H * e, device=dev, dtype=bf) for _ in range(n)]
        coef = torch.tensor([1.0, -0.5], device=dev)
        row("two maps combined + unit norm per head", "", T, nbytes,
            lambda i: ops.maps_combine(comb[i], attn[i], coef, H, 2, khd, e, 1e-5, 0.7), n)
        # routed experts, step by step
        x = [torch.randn(T, W, device=dev).to(bf) for _ in range(4)]
        wr, br, sg = torch.randn(E, W, device=dev) * 0.05, torch.zeros(E, device=dev), torch.randn(W, device=dev) * 0.02
        ids = torch.zeros(T, top, dtype=torch.int32, device=dev)
        share = torch.zeros(T, top, device=dev)
        gate = torch.zeros(T, device=dev)
        zbuf = torch.zeros(T * (E + 1), device=dev)
        row("router: logits, top, softmax, shared gate", "", T, T * W * 2 + 4 * (E + 1) * W,
            lambda i: ops.moe_route(ids, share, gate, x[i % 4], wr, br, sg, top, scratch=zbuf), 4)
        pairs = T * top
        wide = ops.moe_wide_tiles(pairs, E, bf, W, F)
        max_tiles = ops.moe_max_tiles(pairs, E, wide)
        tiles = torch.zeros(3, max_tiles, dtype=torch.int32, device=dev)
        meta = torch.zeros(4, dtype=torch.int32, device=dev)
        wgu = torch.randn(E, 2 * F, W, device=dev).to(bf) * 0.02
        wd = torch.randn(E, W, F, device=dev).to(bf) * 0.02
        used = min(E, pairs)
        shared_out = torch.randn(T, W, device=dev).to(bf)
        o2 = torch.empty(T, W, device=dev, dtype=bf)
        if wide:
            # many rows per expert: slots padded to whole tiles, rows gathered, the tcgen05 product in its grouped form
            cap = max_tiles * ops.moe_tile_rows(True)
            slots = torch.zeros(cap, dtype=torch.int32, device=dev)
            pair_slot = torch.zeros(pairs, dtype=torch.int32, device=dev)
            row("pairs grouped by expert, slots padded to tiles", "", T, pairs * 12,
                lambda i: ops.moe_group(ids, E, slots, tiles, meta, True, padded=True, pair_slot=pair_slot), 2)
            xs = torch.zeros(cap, W, device=dev, dtype=bf)
            row("rows gathered into slot order", "", T, 2 * 2 * pairs * W, lambda i: ops.moe_gather(xs, x[i % 4], slots, meta, top), 4)
            act = torch.empty(cap, F, device=dev, dtype=bf)
            y = torch.empty(cap, W, device=dev, dtype=bf)
            row("experts' gate/up product, silu (tcgen05, grouped)", "gate/up product, silu", T,
                2 * (used * 2 * F * W + pairs * W + pairs * F),
                lambda i: ops.gemm_tc_grouped(act, xs, wgu, tiles[0], meta, gated=True, status=status), 2, flops=2 * pairs * 2 * F * W)
            row("experts' down product (tcgen05, grouped)", "down product", T, 2 * (used * F * W + pairs * F + pairs * W),
                lambda i: ops.gemm_tc_grouped(y, act, wd, tiles[0], meta, status=status), 2, flops=2 * pairs * F * W)
            row("experts' outputs weighted and summed + gated shared expert", "", T, pairs * W * 2 + T * W * 4,
                lambda i: ops.moe_combine_sorted(o2, y, pair_slot, share, top, shared_out, gate), 2)
        else:
            slots = torch.zeros(pairs, dtype=torch.int32, device=dev)
            row("pairs grouped by expert", "", T, pairs * 8, lambda i: ops.moe_group(ids, E, slots, tiles, meta, wide), 2)
            act = torch.empty(pairs, F, device=dev, dtype=bf)
            y = torch.empty(pairs, W, device=dev)
            row("experts' gate/up product, silu (mma.sync)", "gate/up product, silu", T, 2 * (used * 2 * F * W + T * W + pairs * F),
                lambda i: ops.moe_grouped(act, x[i % 4], wgu, slots, tiles, meta, max_tiles, src_div=top, scatter=False, gated=True, wide=wide), 4,
                flops=2 * pairs * 2 * F * W)
            row("experts' down product, weighted (mma.sync)", "down product", T, 2 * (used * F * W + pairs * F) + 4 * pairs * W,
                lambda i: ops.moe_grouped(y, act, wd, slots, tiles, meta, max_tiles, src_div=0, scatter=True, pair_weight=share.view(-1), wide=wide), 2,
                flops=2 * pairs * F * W)
            row("experts' outputs summed + gated shared expert", "", T, pairs * W * 4 + T * W * 4,
                lambda i: ops.moe_combine(o2, y, top, shared_out, gate), 2)
        # the like products of the dense path, with the rows and sizes the chosen experts have together
        wl = torch.randn(2 * top * F, W, device=dev).to(bf) * 0.02
        al = torch.empty(T, top * F, device=dev, dtype=bf)
        row("gate/up product, silu", "", T, 2 * (2 * top * F * W + T * W + T * top * F),
            lambda i: ops.gated_linear(al, x[i % 4], wl, ws, status), 4, flops=2 * T * 2 * top * F * W)
        wl2 = torch.randn(W, top * F, device=dev).to(bf) * 0.02
        ol = torch.empty(T, W, device=dev, dtype=bf)
        row("down product", "", T, 2 * (top * F * W + T * top * F + T * W), lambda i: ops.linear(ol, al, wl2, status), 2,
            flops=2 * T * top * F * W)
    V = llama["vocab_size"]
    logits = torch.randn(8, V, device=dev)
    row("capped logits", "", 8, 8 * V * 8, lambda i: ops.softcap(logits, 30.0), 2)
    return rows


def run_kaditar(args):
    """--only kaditar: decode (1 and 8 requests at --context) and prefill (2,048 tokens) of a Kaditar model beside the
    Llama model of the same width, projection sizes, layers and vocabulary (random weights, bfloat16), and the
    design's own kernels alone beside their likes."""
    global BLOCK_SIZE
    import torch

    BLOCK_SIZE = args.page
    pk = peaks()
    context = args.context or CONTEXT
    if args.profile_step:
        llama = dict(SHAPES[args.shapes])
        llama["num_hidden_layers"] = args.layers or 4
        rig = make_rig(kaditar_config(llama), context, 8, args.page)
        rig.runner.use_cuda_graphs = False
        if args.profile_step == "decode":
            ms, _, _ = rig.timed_decode(args.batch, 2, 2, context)
        else:
            ms = rig.timed_prefill(args.tokens or PREFILL_TOKENS, 1, 2)
        print(json.dumps({"only": "kaditar", "profile_step": args.profile_step, "layers": llama["num_hidden_layers"], "ms": round(ms, 3)}))
        return 0
    out = {"only": "kaditar", "peaks": pk["source"], "context": context, "sizes": {}}
    for name in ([args.shapes] if args.shapes != "1b" or args.layers else ["1b", "3b"]):
        llama = dict(SHAPES[name])
        if args.layers:
            llama["num_hidden_layers"] = args.layers
        ka = kaditar_config(llama)
        res = {}
        for label, cfg in (("kaditar", ka), ("llama", llama)):
            rig = make_rig(cfg, context, 8, args.page)
            for b in (1, 8):
                rig.timed_decode(b, 3, 2, context - 200)
                ms, graph_steps, _ = rig.timed_decode(b, 24, 6, context)
                nbytes = kaditar_decode_bytes(cfg, b, context - 12) if label == "kaditar" else decode_bytes(cfg, b, context - 12)
                res[f"{label}_decode_b{b}_ms"] = round(ms, 4)
                res[f"{label}_decode_b{b}_tokens_per_s"] = round(b * 1000.0 / ms, 1)
                res[f"{label}_decode_b{b}_hbm_frac"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                res[f"{label}_decode_b{b}_graph_steps"] = graph_steps
            ms = rig.timed_prefill(PREFILL_TOKENS, 3, 2)
            flops = kaditar_prefill_flops(cfg, PREFILL_TOKENS) if label == "kaditar" else prefill_flops(cfg, PREFILL_TOKENS)
            res[f"{label}_prefill_{PREFILL_TOKENS}_ms"] = round(ms, 3)
            res[f"{label}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS * 1000.0 / ms, 1)
            res[f"{label}_prefill_{PREFILL_TOKENS}_bf16_frac"] = round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
            rig.close()
            del rig
            torch.cuda.empty_cache()
        out["sizes"][name] = res
        for k, v in res.items():
            print(f"{name}  {k} = {v}", file=sys.stderr)
    rows = kaditar_kernel_rows(pk, dict(SHAPES["1b"]))
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items() if v != ""), file=sys.stderr)
    out["kernels"] = rows
    print(json.dumps(out))
    return 0


ZEPILIX_WINDOW = 2048       # keys a latent layer's query sees at most
ZEPILIX_LATENT = 96         # latent size; with the turned part the cached row has 128 entries (the tensor-core kernels' largest head)
ZEPILIX_TURNED = 32
ZEPILIX_DELTA_HEAD = 128    # query/key and value size of a delta-rule head
ZEPILIX_SIDE = 256          # entries of the input per token and layer


def zepilix_config(llama: dict) -> dict:
    """A Zepilix model with the width, feed-forward size, heads, head size, vocabulary and number of layer runs of the
    given Llama shapes: delta rule, attention, delta rule, latent attention with a window, and so on; layers 4 to 7 run
    twice (so four layers fewer carry weights), every layer has the input per token."""
    nh, nkv, hd, W = llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["hidden_size"]
    mlp = {"kind": "dense", "ff": llama["intermediate_size"]}
    dh = W // ZEPILIX_DELTA_HEAD
    delta = {"type": "delta", "mlp": mlp,
             "mixer": {"heads": dh, "kv_heads": dh // 2, "dim": ZEPILIX_DELTA_HEAD, "vdim": ZEPILIX_DELTA_HEAD, "conv": 4}}
    attention = {"type": "attention", "mlp": mlp,
                 "mixer": {"heads": nh, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5,
                           "rot": {"dims": hd, "base": 500000.0}}}
    latent = {"type": "latent_attention", "mlp": mlp,
              "mixer": {"heads": nh, "dim": hd, "rot_dim": ZEPILIX_TURNED, "vdim": hd, "kv_rank": ZEPILIX_LATENT,
                        "q_rank": W * 3 // 8, "scale": (hd + ZEPILIX_TURNED) ** -0.5, "mask": {"size": ZEPILIX_WINDOW},
                        "rot": {"dims": ZEPILIX_TURNED, "base": 1000000.0}}}
    runs = llama["num_hidden_layers"]
    looped = 4 if runs >= 12 else 0
    kinds = (delta, attention, delta, latent)
    cfg = {"architecture": "Zepilix", "vocab": llama["vocab_size"], "width": W, "norm": {"eps": 1e-6},
           "token_side": {"dim": ZEPILIX_SIDE}, "layers": [kinds[i % 4] for i in range(runs - looped)]}
    if looped:
        cfg["loop"] = {"start": 4, "stop": 8, "times": 2}
    return cfg


def zepilix_runs(cfg):
    """The layers in the order they run (a looped layer once per pass)."""
    n = len(cfg["layers"])
    lp = cfg.get("loop")
    order = list(range(n)) if not lp else (list(range(lp["start"])) + list(range(lp["start"], lp["stop"])) * lp["times"]
                                           + list(range(lp["stop"], n)))
    return [cfg["layers"][i] for i in order]


def zepilix_decode_bytes(cfg, batch, context):
    """Bytes one decode step of a Zepilix model must move: the bfloat16 weights of every layer run once (a looped
    stretch is larger than the L2, so each pass reads it again), each live request's state matrices read and written
    (32-bit), its keys and its values' pool, or its window of cached latents."""
    W, V, s = cfg["width"], cfg["vocab"], cfg["token_side"]["dim"]
    total = 2 * V * W + 4 * W
    for layer in zepilix_runs(cfg):
        m, F = layer["mixer"], layer["mlp"]["ff"]
        nh, d, e = m["heads"], m["dim"], m["vdim"]
        total += 2 * 3 * F * W + 4 * (2 * F + W) + 4 * 2 * W + 2 * (2 * s * W + batch * s) + 4 * W
        if layer["type"] == "delta":
            G = m["kv_heads"]
            total += 2 * ((2 * G * d + 2 * nh * e + 2 * nh) * W + W * nh * e)
            total += batch * (2 * 4 * nh * d * e + 2 * 4 * (m["conv"] - 1) * (2 * G * d + nh * e))
        elif layer["type"] == "attention":
            G = m["kv_heads"]
            total += 2 * ((nh + G) * d * W + W * nh * e) + 2 * batch * context * 2 * G * d
        else:
            r, t, qr = m["kv_rank"], m["rot_dim"], m["q_rank"]
            seen = min(context, m["mask"]["size"])
            total += 2 * ((qr + r + t) * W + nh * (d + t) * qr + nh * d * r + nh * e * r + W * nh * e) + 2 * batch * seen * (r + t)
    return total


def zepilix_prefill_flops(cfg, tokens):
    """(flops of the matrix products and the attentions as computed here, flops of the delta rule's recurrence, which
    runs on the FP32 pipes: six per entry of the state and token)."""
    W, V, s = cfg["width"], cfg["vocab"], cfg["token_side"]["dim"]
    flops, scan = 2 * V * W, 0
    pairs = tokens * (tokens + 1) // 2
    for layer in zepilix_runs(cfg):
        m, F = layer["mixer"], layer["mlp"]["ff"]
        nh, d, e = m["heads"], m["dim"], m["vdim"]
        flops += 2 * tokens * (3 * F * W + 2 * s * W)
        if layer["type"] == "delta":
            G = m["kv_heads"]
            flops += 2 * tokens * ((2 * G * d + 2 * nh * e + 2 * nh) * W + W * nh * e)
            scan += 6 * tokens * nh * d * e
        elif layer["type"] == "attention":
            flops += 2 * tokens * ((nh + m["kv_heads"]) * d * W + W * nh * e) + 2 * nh * (d + e) * pairs
        else:
            r, t, qr = m["kv_rank"], m["rot_dim"], m["q_rank"]
            w = m["mask"]["size"]
            seen = pairs if tokens <= w else w * (w + 1) // 2 + (tokens - w) * w
            flops += 2 * tokens * ((qr + r + t) * W + nh * (d + t) * qr + nh * d * r + nh * e * r + W * nh * e)
            flops += 2 * nh * (2 * r + t) * seen
    return flops, scan


def graph_median_us(launch, sets):
    """Microseconds per launch inside a captured graph of at least 16 launches over rotating tensors (a launch by
    itself from the host costs more than small kernels run; inside a step they are nodes of such a graph)."""
    import torch
    n = max(sets, 16)
    for i in range(n):
        launch(i % sets)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for i in range(n):
            launch(i % sets)
    for _ in range(3):
        graph.replay()
    events = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(15)]
    torch.cuda.synchronize()
    for a, b in events:
        a.record()
        graph.replay()
        b.record()
    torch.cuda.synchronize()
    times = sorted(a.elapsed_time(b) * 1e3 / n for a, b in events)
    return times[len(times) // 2]


def zepilix_kernel_rows(pk, llama):
    """Each kernel the design adds, alone, beside the like kernel of the closest existing path at the same sizes:
    microseconds per launch inside a captured graph over rotating tensors, the share of the measured copy bandwidth
    that the bytes it must move make, and for the recurrence its share of the FP32 pipes."""
    import torch

    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.engine.runtime import Workspace
    from lyapunov_engine_b200.parts.rope import pair_rates

    dev = "cuda:0"
    cfg = zepilix_config(llama)
    W, nh, nkv, hd, F = llama["hidden_size"], llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["intermediate_size"]
    dm = cfg["layers"][0]["mixer"]
    H, G, d, e = dm["heads"], dm["kv_heads"], dm["dim"], dm["vdim"]
    r, t, page, s = ZEPILIX_LATENT, ZEPILIX_TURNED, BLOCK_SIZE, ZEPILIX_SIDE
    rows = []

    def row(kernel, like, tokens, nbytes, launch, sets, fp32_flops=0):
        us = graph_median_us(launch, sets)
        entry = {"kernel": kernel, "like": like, "tokens": tokens, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                 "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if fp32_flops:
            # 148 multiprocessors x 128 lanes x 2 flops at the highest clock (1,965 MHz): 74.4 TFLOP/s
            entry["fp32_frac"] = round(fp32_flops / us / 1e6 / 74.4, 3)
        rows.append(entry)

    def sets_for(nbytes):
        return max(2, min(64, (256 << 20) // max(nbytes, 1) + 1))

    bf = torch.bfloat16
    status = ops.new_status(dev)
    ws = Workspace(torch.device(dev))
    for T in (8, 2048):
        # the two norms of one row, with the normed addend of the token's input; the Llama path's norm + residual
        nbytes = T * W * (4 + 2 + 4 + 2 + 2) + 12 * W
        n = sets_for(nbytes)
        resid = [torch.randn(T, W, device=dev) for _ in range(n)]
        addend = [torch.randn(T, W, device=dev).to(bf) for _ in range(n)]
        o1 = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(n)]
        o2 = [torch.empty(T, W, device=dev, dtype=bf) for _ in range(n)]
        w1, w2, wa = (torch.ones(W, device=dev) for _ in range(3))
        row("two norms of one row + normed addend", "", T, nbytes,
            lambda i: ops.rmsnorm_pair(o1[i], o2[i], resid[i], w1, w2, 1e-6, addend=addend[i], addend_weight=wa, addend_eps=1e-6), n)
        row("rmsnorm + residual", "two norms of one row + normed addend", T, T * W * 12 + 4 * W,
            lambda i: ops.rmsnorm(o1[i], resid[i], addend[i], w1, 1e-5), n)
        # both sub-layers' outputs and the bias into the stream, with the copy the token's input reads
        bias = torch.randn(W, device=dev)
        row("sum of both sub-layers into the stream + copy", "", T, T * W * (8 + 2 + 2 + 2) + 4 * W,
            lambda i: ops.residual_add(resid[i], addend[i], o2[i], bias, o1[i]), n)
        # the gate of the token's input, and what a pass adds
        z = torch.randn(T, s, device=dev).to(bf)
        table = torch.randn(32000, 4 * s, device=dev).to(bf)
        ids = torch.randint(0, 32000, (T,), dtype=torch.int32, device=dev)
        gz = torch.empty(T, s, device=dev, dtype=bf)
        row("gelu gate times the token's table row", "", T, T * s * 6, lambda i: ops.gate_rows(gz, z, table, s, ids, status), 1)
        emb = torch.randn(32000, W, device=dev).to(bf)
        vec = torch.randn(W, device=dev)
        row("pass entry (embedding + vector into the stream)", "", T, T * W * 10, lambda i: ops.stream_entry(resid[i], emb, ids, vec, status), n)
        row("embedding", "pass entry", T, T * W * 6, lambda i: ops.embed(resid[i], emb, ids, status), n)
        del resid, addend, o1, o2
        # the delta rule's chain: convolution with silu over q | k | v, the recurrence, the gated norm per head
        C = 2 * G * d + H * e
        width = C + H * e + 2 * H
        width = (width + 7) // 8 * 8
        reqs = T if T <= 64 else 1
        q_lens = [T // reqs] * reqs
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        treq = torch.tensor([b for b, m in enumerate(q_lens) for _ in range(0, m, ops.SHORT_CONV_TILE)], dtype=torch.int32, device=dev)
        tq0 = torch.tensor([s0 for m in q_lens for s0 in range(0, m, ops.SHORT_CONV_TILE)], dtype=torch.int32, device=dev)
        slots = torch.arange(reqs, dtype=torch.int32, device=dev)
        proj = torch.randn(T, width, device=dev).to(bf)
        conv = torch.empty(T, C, device=dev, dtype=bf)
        taps_state = torch.zeros(reqs + 1, 3, C, device=dev)
        taps = torch.randn(4, C, device=dev)
        if T <= 64:
            launch = lambda i: ops.short_conv_general(conv, proj[:, :C], taps, taps_state, slots, cu, None, None, reqs, add_input=False, silu=True)
        else:
            launch = lambda i: ops.short_conv_general(conv, proj[:, :C], taps, taps_state, slots, cu, treq, tq0, treq.numel(), add_input=False, silu=True)
        row(f"convolution (4 taps) + silu over {C} channels", "short convolution, 4 taps (Sulepel, 2,048 channels)", T,
            T * C * 4 + reqs * 3 * C * 8 + 16 * C, launch, 1)
        state_sets = 4 if T <= 64 else 2
        states = [torch.zeros(reqs + 1, H, e, d, device=dev) for _ in range(state_sets)]
        o = torch.empty(T, H * e, device=dev)
        a_log, dt_bias = torch.zeros(H, device=dev), torch.zeros(H, device=dev)
        conv.normal_()
        row(f"delta rule, {H} heads of {d} x {e}, {reqs} request(s)", "", T, reqs * 2 * 4 * H * d * e + T * (C * 2 + H * e * 4),
            lambda i: ops.gated_delta_scan(o, conv, 0, G * d, 2 * G * d, proj, C + H * e, C + H * e + H, a_log, dt_bias, states[i],
                                           slots, cu, reqs, H, G, d, e, 1e-6, d ** -0.5), state_sets, fp32_flops=6 * T * H * d * e)
        gated = torch.empty(T, H * e, device=dev, dtype=bf)
        wn = torch.ones(e, device=dev)
        row("norm per head times silu gate", "", T, T * H * e * 8, lambda i: ops.head_norm_gate(gated, o, proj[:, C:C + H * e], wn, 1e-6, H, e), 1)
        # cache writes
        pages = (T + page - 1) // page + 1
        btab = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        req0 = torch.zeros(T, dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        qk = torch.randn(T, (nh + nkv) * hd, device=dev).to(bf)
        kc = torch.zeros(pages + 1, nkv, page, hd, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        rates = pair_rates(hd, 5e5).to(dev)
        row("turn of pairs + norm + cache write (values are the keys)", "", T, T * ((nh + nkv) * hd * 4 + nkv * hd * 2),
            lambda i: ops.rope_norm_store(qk, kc, vc, rates, pos, req0, btab, nh, nkv, hd, 0, hd, 1e-6, hd, page, True, True, status), 1)
        qkv = torch.randn(T, (nh + 2 * nkv) * hd, device=dev).to(bf)
        cos_sin = torch.randn(max(T, 16), hd, device=dev)
        row("rotary + key/value cache write", "turn of pairs + norm + cache write", T, T * ((nh + nkv) * hd * 4 + nkv * hd * 4),
            lambda i: ops.rope_kv_write(qkv, kc, vc, cos_sin, pos, req0, btab, nh, nkv, hd, page, True, status), 1)
        qr = W * 3 // 8
        down = torch.randn(T, qr + r + t, device=dev).to(bf)
        lat = torch.zeros(pages + 1, 1, page, r + t, device=dev, dtype=bf)
        wl, wq = torch.ones(r, device=dev), torch.ones(qr, device=dev)
        cq = torch.empty(T, qr, device=dev, dtype=bf)
        rates_l = pair_rates(t, 1e6).to(dev)
        row("both latents' norms + turned key part + cache write", "", T, T * (qr + r + t) * 4,
            lambda i: ops.latent_rope_store(down, qr, r, t, r + t, wl, 1e-6, rates_l, lat, pos, req0, btab, page, status, second=(0, qr, wq, cq)), 1)
        lat2 = torch.zeros(pages + 1, 1, page, 128, device=dev, dtype=bf)
        proj2 = torch.randn(T, 128 + 8, device=dev).to(bf)
        wl2 = torch.ones(128, device=dev)
        row("latent norm + cache write", "both latents' norms + turned key part + cache write", T, T * 128 * 4,
            lambda i: ops.latent_norm_store(proj2, 0, 128, wl2, 1e-5, lat2, pos, req0, btab, page, status), 1)
        # gated products with and without biases
        x = torch.randn(T, W, device=dev).to(bf)
        wgu = [torch.randn(2 * F, W, device=dev).to(bf) for _ in range(4)]
        act = torch.empty(T, F, device=dev, dtype=bf)
        b2 = torch.randn(2 * F, device=dev)
        nbytes = 2 * (2 * F * W + T * W + T * F)
        row("gate/up product, biases + SiLU", "", T, nbytes + 8 * F, lambda i: ops.gated_linear_bias(act, x, wgu[i], b2, ws, status), 4)
        row("gate/up product, SiLU", "gate/up product, biases + SiLU", T, nbytes, lambda i: ops.gated_linear(act, x, wgu[i], ws, status), 4)
        del wgu
    ops.check_status(status)
    return rows


def run_zepilix(args):
    """--only zepilix: decode (1 and 8 requests at --context) and prefill (2,048 tokens) of a Zepilix model beside the
    Sulepel model (the closest existing design: latent attention, short convolutions, state rows per request) and the
    Llama model of the same width, feed-forward size, heads, layer runs and vocabulary (random weights, bfloat16),
    and the design's own kernels alone beside their likes."""
    global BLOCK_SIZE
    import torch

    BLOCK_SIZE = args.page
    pk = peaks()
    context = args.context or CONTEXT
    if args.profile_step:
        # a few steps launch by launch (no captured graph) of a model of --layers layer runs (4 by default), for a profiler
        llama = dict(SHAPES[args.shapes])
        llama["num_hidden_layers"] = args.layers or 4
        rig = make_rig(zepilix_config(llama), context, 8, args.page)
        rig.runner.use_cuda_graphs = False
        if args.profile_step == "decode":
            ms, _, _ = rig.timed_decode(args.batch, 2, 2, context)
        else:
            ms = rig.timed_prefill(args.tokens or PREFILL_TOKENS, 1, 2)
        print(json.dumps({"only": "zepilix", "profile_step": args.profile_step, "layers": llama["num_hidden_layers"], "ms": round(ms, 3)}))
        return 0
    out = {"only": "zepilix", "peaks": pk["source"], "context": context, "sizes": {}}
    for name in ([args.shapes] if args.shapes != "1b" or args.layers else ["1b", "3b"]):
        llama = dict(SHAPES[name])
        if args.layers:
            llama["num_hidden_layers"] = args.layers
        res = {}
        for label, cfg in (("zepilix", zepilix_config(llama)), ("sulepel", sulepel_config(llama)), ("llama", llama)):
            rig = make_rig(cfg, context, 8, args.page)
            for b in (1, 8):
                rig.timed_decode(b, 3, 2, context - 200)
                ms, graph_steps, _ = rig.timed_decode(b, 24, 6, context)
                nbytes = {"zepilix": zepilix_decode_bytes, "sulepel": sulepel_decode_bytes, "llama": decode_bytes}[label](cfg, b, context - 12)
                res[f"{label}_decode_b{b}_ms"] = round(ms, 4)
                res[f"{label}_decode_b{b}_tokens_per_s"] = round(b * 1000.0 / ms, 1)
                res[f"{label}_decode_b{b}_hbm_frac"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                res[f"{label}_decode_b{b}_graph_steps"] = graph_steps
            ms = rig.timed_prefill(PREFILL_TOKENS, 3, 2)
            if label == "zepilix":
                flops, scan = zepilix_prefill_flops(cfg, PREFILL_TOKENS)
                res["zepilix_prefill_fp32_recurrence_gflop"] = round(scan / 1e9, 2)
            else:
                flops = sulepel_prefill_flops(cfg, PREFILL_TOKENS) if label == "sulepel" else prefill_flops(cfg, PREFILL_TOKENS)
            res[f"{label}_prefill_{PREFILL_TOKENS}_ms"] = round(ms, 3)
            res[f"{label}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS * 1000.0 / ms, 1)
            res[f"{label}_prefill_{PREFILL_TOKENS}_bf16_frac"] = round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
            rig.close()
            del rig
            torch.cuda.empty_cache()
        out["sizes"][name] = res
        for k, v in res.items():
            print(f"{name}  {k} = {v}", file=sys.stderr)
    rows = zepilix_kernel_rows(pk, dict(SHAPES["1b"]))
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items() if v != ""), file=sys.stderr)
    out["kernels"] = rows
    print(json.dumps(out))
    return 0


# ---------------------------------------------------------------------------------------------- Ribozen
RIBOZEN_WINDOW = 1024       # keys an attention layer's query sees at most, beside the first RIBOZEN_KEPT
RIBOZEN_KEPT = 8
RIBOZEN_STATE = 128         # numbers of state per channel of a state-space-duality layer
RIBOZEN_SCAN_STATE = 16     # of a selective-scan channel
RIBOZEN_EXPERTS, RIBOZEN_TOP = 8, 2


def ribozen_config(llama: dict) -> dict:
    """A Ribozen model with the width, heads, head size, vocabulary and number of layers of the given Llama shapes:
    state-space duality, state-space duality, matrix memory, attention beside a selective scan, and so on; every
    layer has eight routed experts (two per token) and a shared one, each a quarter of the Llama feed-forward's
    size, so that a token's feed-forward products are three quarters of the Llama layer's."""
    nh, nkv, hd, W = llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"], llama["hidden_size"]
    ff = llama["intermediate_size"] // 4
    mlp = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": RIBOZEN_EXPERTS, "top": RIBOZEN_TOP}, "shared": {"ff": ff}}
    duality = {"type": "mamba2", "mlp": mlp,
               "mixer": {"heads": 2 * W // 64, "vdim": 64, "state": RIBOZEN_STATE, "groups": 8, "conv": 4, "norm_groups": 8}}
    memory = {"type": "mlstm", "mlp": mlp, "mixer": {"heads": W // 256, "dim": 128, "vdim": 256, "gate_cap": 15.0}}
    pair = {"type": "parallel", "mlp": mlp,
            "mixer": {"left_scale": 0.7, "right_scale": 1.0,
                      "left": {"heads": nh, "kv_heads": nkv, "dim": hd, "vdim": hd, "scale": hd ** -0.5, "softcap": 30.0,
                               "rot": {"dims": hd, "base": 500000.0,
                                       "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}},
                               "mask": {"size": RIBOZEN_WINDOW, "keep_first": RIBOZEN_KEPT}},
                      "right": {"inner": W, "state": RIBOZEN_SCAN_STATE, "dt_rank": W // 16, "conv": 4}}}
    kinds = (duality, duality, memory, pair)
    return {"architecture": "Ribozen", "vocab": llama["vocab_size"], "width": W, "norm": {"eps": 1e-5},
            "embedding": {"scale": W ** 0.5}, "layers": [kinds[i % 4] for i in range(llama["num_hidden_layers"])]}


def ribozen_decode_bytes(cfg, batch, context):
    """Bytes one decode step of a Ribozen model must move: the bfloat16 weights it touches (of the routed experts
    those that batch * top tokens can reach), each live request's states read and written (32-bit), and its window
    of keys and values."""
    W, V = cfg["width"], cfg["vocab"]
    total = 2 * 2 * V * W + 4 * W
    for layer in cfg["layers"]:
        m, f = layer["mixer"], layer["mlp"]
        F, E, top, S = f["expert"]["ff"], f["router"]["experts"], f["router"]["top"], f["shared"]["ff"]
        total += 2 * 3 * W * (F * min(E, batch * top) + S) + 4 * E * W + 4 * 4 * W
        if layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * P, H * P + 2 * G * N
            total += 2 * ((2 * inner + 2 * G * N + H) * W + W * inner) + batch * (2 * 4 * inner * N + 2 * 4 * (m["conv"] - 1) * C)
        elif layer["type"] == "mlstm":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            total += 2 * ((2 * H * d + 2 * H * e + 2 * H) * W + W * H * e) + batch * 2 * 4 * H * (e + 1) * d
        else:
            a, r = m["left"], m["right"]
            nh, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            seen = min(context, a["mask"]["size"] + a["mask"]["keep_first"])
            total += 2 * ((nh * d + G * d + G * e + nh * e) * W + W * nh * e) + 2 * batch * seen * G * (d + e)
            C, N, R = r["inner"], r["state"], r["dt_rank"]
            total += 2 * (2 * C * W + (R + 2 * N) * C + C * R + W * C) + 4 * C * N + batch * (2 * 4 * C * N + 2 * 4 * (r["conv"] - 1) * C)
    return total


def ribozen_prefill_flops(cfg, tokens):
    """(flops of the matrix products and the attentions as computed here, flops of the recurrences, which run on the
    FP32 pipes: six per entry of a state-space state and token, four per entry of a matrix memory)."""
    W, V = cfg["width"], cfg["vocab"]
    flops, scan = 2 * V * W, 0
    for layer in cfg["layers"]:
        m, f = layer["mixer"], layer["mlp"]
        F, E, top, S = f["expert"]["ff"], f["router"]["experts"], f["router"]["top"], f["shared"]["ff"]
        flops += 2 * tokens * (3 * W * (top * F + S) + E * W)
        if layer["type"] == "mamba2":
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            flops += 2 * tokens * ((2 * H * P + 2 * G * N + H) * W + W * H * P)
            scan += 6 * tokens * H * P * N
        elif layer["type"] == "mlstm":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            flops += 2 * tokens * ((2 * H * d + 2 * H * e + 2 * H) * W + W * H * e)
            scan += 4 * tokens * H * d * (e + 1)
        else:
            a, r = m["left"], m["right"]
            nh, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            w = a["mask"]["size"]
            seen = tokens * (tokens + 1) // 2 if tokens <= w else w * (w + 1) // 2 + (tokens - w) * (w + a["mask"]["keep_first"])
            flops += 2 * tokens * ((nh * d + G * d + G * e + nh * e) * W + W * nh * e) + 2 * nh * (d + e) * seen
            C, N, R = r["inner"], r["state"], r["dt_rank"]
            flops += 2 * tokens * (2 * C * W + (R + 2 * N) * C + C * R + W * C)
            scan += 6 * tokens * C * N
    return flops, scan


def ribozen_kernel_rows(pk, llama):
    """Each kernel the design adds, alone, beside the like kernel of the closest existing path at like sizes:
    microseconds per launch inside a captured graph over rotating tensors, the share of the measured copy bandwidth
    that the bytes it must move make, and for the recurrences their share of the FP32 pipes."""
    import torch

    from lyapunov_engine_b200 import ops
    from lyapunov_engine_b200.parts.rope import pair_rates, ramped_rates

    dev = "cuda:0"
    cfg = ribozen_config(llama)
    W, nh, nkv, hd = llama["hidden_size"], llama["num_attention_heads"], llama["num_key_value_heads"], llama["head_dim"]
    page = BLOCK_SIZE
    rows = []

    def row(kernel, like, tokens, nbytes, launch, sets, fp32_flops=0):
        us = graph_median_us(launch, sets)
        entry = {"kernel": kernel, "like": like, "tokens": tokens, "us": round(us, 2), "gbs": round(nbytes / us / 1e3, 1),
                 "hbm_frac": round(nbytes / us / 1e3 / pk["hbm_gbs"], 3)}
        if fp32_flops:
            # 148 multiprocessors x 128 lanes x 2 flops at the highest clock (1,965 MHz): 74.4 TFLOP/s
            entry["fp32_frac"] = round(fp32_flops / us / 1e6 / 74.4, 3)
        rows.append(entry)

    bf = torch.bfloat16
    status = ops.new_status(dev)
    dm, mm, pm = cfg["layers"][0]["mixer"], cfg["layers"][2]["mixer"], cfg["layers"][3]["mixer"]
    for T in (8, 2048):
        reqs = T if T <= 64 else 1
        q_lens = [T // reqs] * reqs
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        slots = torch.arange(reqs, dtype=torch.int32, device=dev)
        state_sets = 4 if T <= 64 else 2
        # state-space duality: one decay per head
        H, P, N, G = dm["heads"], dm["vdim"], dm["state"], dm["groups"]
        inner, C = H * P, H * P + 2 * G * N
        conv = torch.randn(T, C, device=dev).to(bf)
        proj = torch.randn(T, inner + H + 8, device=dev).to(bf)
        y = torch.empty(T, inner, device=dev)
        states = [torch.zeros(reqs + 1, inner, N, device=dev) for _ in range(state_sets)]
        zeros_h = torch.zeros(H, device=dev)
        row(f"state-space recurrence, {H} heads of {P} x {N} (one decay per head), {reqs} request(s)",
            "delta rule, 16 heads of 128 x 128", T, reqs * 2 * 4 * inner * N + T * (C * 2 + inner * 6 + H * 2),
            lambda i: ops.ssm_scan(y, conv[:, :inner], conv, inner, inner + G * N, proj[:, inner:inner + H], proj[:, :inner], zeros_h,
                                   zeros_h, zeros_h, states[i], slots, cu, reqs, N, P, (H // G) * P, per_row=False), state_sets,
            fp32_flops=6 * T * inner * N)
        normed = torch.empty(T, inner, device=dev, dtype=bf)
        wn = torch.ones(inner, device=dev)
        row("norm in 8 parts of the gated channels", "norm per head times silu gate", T, T * inner * 6,
            lambda i: ops.rmsnorm(normed, y, None, wn, 1e-5, groups=8), 1)
        del states
        # selective scan: a decay per channel and state
        r = pm["right"]
        Cs, Ns, R = r["inner"], r["state"], r["dt_rank"]
        convs = torch.randn(T, Cs, device=dev).to(bf)
        low = torch.randn(T, (R + 2 * Ns + 7) // 8 * 8, device=dev).to(bf)
        dt = torch.randn(T, Cs, device=dev).to(bf)
        z = torch.randn(T, Cs, device=dev).to(bf)
        outs = torch.empty(T, Cs, device=dev, dtype=bf)
        states = [torch.zeros(reqs + 1, Cs, Ns, device=dev) for _ in range(state_sets)]
        a_log, zeros_c = torch.zeros(Cs, Ns, device=dev), torch.zeros(Cs, device=dev)
        row(f"state-space recurrence, {Cs} channels x {Ns} (a decay per channel and state), {reqs} request(s)",
            "delta rule, 16 heads of 128 x 128", T, reqs * 2 * 4 * Cs * Ns + 4 * Cs * Ns + T * (Cs * 8 + Ns * 4),
            lambda i: ops.ssm_scan(outs, convs, low, R, R + Ns, dt, z, zeros_c, a_log, zeros_c, states[i], slots, cu, reqs, Ns, 1, Cs,
                                   per_row=True, out_scale=1.0), state_sets, fp32_flops=6 * T * Cs * Ns)
        del states
        # matrix memory
        Hm, d, e = mm["heads"], mm["dim"], mm["vdim"]
        width = (2 * Hm * d + 2 * Hm * e + 2 * Hm + 7) // 8 * 8
        rows_m = torch.randn(T, width, device=dev).to(bf)
        o = torch.empty(T, Hm * e, device=dev)
        states = [torch.zeros(reqs + 1, *ops.mlstm_state_shape(Hm, d, e), device=dev) for _ in range(state_sets)]
        zeros_m = torch.zeros(Hm, device=dev)
        row(f"matrix memory, {Hm} heads of {d} x {e}, {reqs} request(s)", "delta rule, 16 heads of 128 x 128", T,
            reqs * 2 * states[0][0].numel() * 4 + T * (width * 2 + Hm * e * 4),
            lambda i: ops.mlstm_scan(o, rows_m, 0, Hm * d, 2 * Hm * d, 2 * Hm * d + 2 * Hm * e, 2 * Hm * d + 2 * Hm * e + Hm, zeros_m,
                                     zeros_m, states[i], slots, cu, reqs, Hm, d, e, 15.0, d ** -0.5), state_sets,
            fp32_flops=4 * T * Hm * d * (e + 1))
        gated = torch.empty(T, Hm * e, device=dev, dtype=bf)
        wm = torch.ones(Hm * e, device=dev)
        row("norm per head (a weight per head) times sigmoid gate", "norm per head times silu gate", T, T * Hm * e * 8,
            lambda i: ops.head_norm_gate(gated, o, rows_m[:, 2 * Hm * d + Hm * e:2 * Hm * d + 2 * Hm * e], wm, 1e-5, Hm, e, sigmoid=True), 1)
        del states
        # the delta rule at its own sizes, as the yardstick of the recurrences
        Hd, Gd, dd = W // 128, W // 256, 128
        Cd = 2 * Gd * dd + Hd * dd
        wd = (Cd + Hd * dd + 2 * Hd + 7) // 8 * 8
        projd = torch.randn(T, wd, device=dev).to(bf)
        convd = torch.randn(T, Cd, device=dev).to(bf)
        od = torch.empty(T, Hd * dd, device=dev)
        states = [torch.zeros(reqs + 1, Hd, dd, dd, device=dev) for _ in range(state_sets)]
        zeros_d = torch.zeros(Hd, device=dev)
        row(f"delta rule, {Hd} heads of {dd} x {dd}, {reqs} request(s)", "", T, reqs * 2 * 4 * Hd * dd * dd + T * (Cd * 2 + Hd * dd * 4),
            lambda i: ops.gated_delta_scan(od, convd, 0, Gd * dd, 2 * Gd * dd, projd, Cd + Hd * dd, Cd + Hd * dd + Hd, zeros_d, zeros_d,
                                           states[i], slots, cu, reqs, Hd, Gd, dd, dd, 1e-6, dd ** -0.5), state_sets,
            fp32_flops=6 * T * Hd * dd * dd)
        del states
        # bias, norm over whole projections, turn, cache write; beside the turn of pairs with its norm per head
        pages = (T + page - 1) // page + 1
        btab = torch.arange(pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
        req0 = torch.zeros(T, dtype=torch.int32, device=dev)
        pos = torch.arange(T, dtype=torch.int32, device=dev)
        qkv = torch.randn(T, (2 * nh + 2 * nkv) * hd, device=dev).to(bf)
        kc = torch.zeros(pages + 1, nkv, page, hd, device=dev, dtype=bf)
        vc = torch.zeros_like(kc)
        rates, magnitude = ramped_rates(hd, 5e5, {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0})
        rates = rates.to(dev)
        bias = torch.zeros((nh + 2 * nkv) * hd, device=dev)
        wq, wk = torch.ones(nh * hd, device=dev), torch.ones(nkv * hd, device=dev)
        row("bias + norm over all of q and of k + turn of halves + cache write", "turn of pairs + norm + cache write", T,
            T * ((nh + nkv) * hd * 4 + nkv * hd * 4) + 4 * (2 * nh + 3 * nkv) * hd,
            lambda i: ops.rope_qknorm_store(qkv, bias, wq, wk, 1e-5, nh * hd, nkv * hd, rates, hd, magnitude, kc, vc, pos, req0, btab,
                                            nh, nkv, hd, page, True, status), 1)
        qk = torch.randn(T, (nh + nkv) * hd, device=dev).to(bf)
        rates_p = pair_rates(hd, 5e5).to(dev)
        row("turn of pairs + norm + cache write (values are the keys)", "", T, T * ((nh + nkv) * hd * 4 + nkv * hd * 2),
            lambda i: ops.rope_norm_store(qk, kc, vc, rates_p, pos, req0, btab, nh, nkv, hd, 0, hd, 1e-6, hd, page, True, True, status), 1)
        attn = torch.randn(T, nh * hd, device=dev).to(bf)
        side = torch.empty(T, nh * hd + W, device=dev, dtype=bf)
        row("gate per entry (sigmoid) into the shared buffer", "norm per head times silu gate", T, T * nh * hd * 6,
            lambda i: ops.sigmoid_gate(side[:, :nh * hd], attn, qkv[:, (nh + 2 * nkv) * hd:], 0.7), 1)
        # the layer scale in the norm's kernel
        resid = [torch.randn(T, W, device=dev) for _ in range(8)]
        delta = torch.randn(T, W, device=dev).to(bf)
        normed_w = torch.empty(T, W, device=dev, dtype=bf)
        w1, ls = torch.ones(W, device=dev), torch.ones(W, device=dev)
        row("rmsnorm + residual with a factor per column", "rmsnorm + residual", T, T * W * 12 + 8 * W,
            lambda i: ops.rmsnorm(normed_w, resid[i], delta, w1, 1e-5, delta_scale=ls), 8)
        row("rmsnorm + residual", "", T, T * W * 12 + 4 * W, lambda i: ops.rmsnorm(normed_w, resid[i], delta, w1, 1e-5), 8)
        del resid
    # attention over a window with kept first keys and capped scores, beside the same window plain
    for label, q_lens, ctx in (("decode, 8 requests at 4,096", [1] * 8, [4095] * 8), ("prompt of 2,048", [2048], [0])):
        T = sum(q_lens)
        B = len(q_lens)
        total = [c + n for c, n in zip(ctx, q_lens)]
        per = (max(total) + page - 1) // page
        btab = torch.arange(B * per, dtype=torch.int32, device=dev).view(B, per).contiguous()
        kc = torch.randn(B * per + 1, nkv, page, hd, device=dev).to(bf)
        vc = torch.randn(B * per + 1, nkv, page, hd, device=dev).to(bf)
        q = torch.randn(T, nh * hd, device=dev).to(bf)
        out = torch.empty(T, nh * hd, device=dev, dtype=bf)
        cu = torch.tensor([0] + list(torch.tensor(q_lens).cumsum(0)), dtype=torch.int32, device=dev)
        before = torch.tensor(ctx, dtype=torch.int32, device=dev)
        seen = sum(min(t, RIBOZEN_WINDOW + RIBOZEN_KEPT) for t in total) if T == B else \
            sum(min(p + 1, RIBOZEN_WINDOW + RIBOZEN_KEPT) for p in range(2048)) // 128       # keys a 128-row tile reads, roughly
        nbytes = (seen if T == B else 2048 * 16 // 128 * 0 + 16 * (RIBOZEN_WINDOW + 128)) * nkv * hd * 4 + T * nh * hd * 4
        for name, keep, cap in (("kept first keys + capped scores", RIBOZEN_KEPT, 30.0), ("window alone", 0, 0.0)):
            if T == B:
                splits = 4
                scratch = torch.zeros(max(ops.attention_decode_scratch_floats(hd, B, nh, splits), 1), device=dev)
                launch = lambda i, keep=keep, cap=cap: ops.attention_decode_bf16(
                    out, scratch, q, q.stride(0), kc, vc, btab, cu, before, None, B, nh, nkv, hd, page, RIBOZEN_WINDOW, hd ** -0.5, splits,
                    status, keep_first=keep, softcap=cap)
            else:
                req = torch.zeros(T // 128, dtype=torch.int32, device=dev)
                q0 = torch.arange(0, T, 128, dtype=torch.int32, device=dev)
                launch = lambda i, keep=keep, cap=cap: ops.attention_prefill_bf16(
                    out, q, q.stride(0), kc, vc, btab, cu, before, req, q0, T // 128, nh, nkv, hd, page, RIBOZEN_WINDOW, hd ** -0.5, status,
                    keep_first=keep, softcap=cap)
            row(f"attention (mma.sync), window of {RIBOZEN_WINDOW}: {name}; {label}", "" if keep == 0 else "window alone", T, nbytes, launch, 1)
        if T != B and ops.attention_tc_available(hd, page):
            launch = lambda i: ops.attention_prefill_tc_bf16(out, q, q.stride(0), kc, vc, btab, cu, before, req, q0, T // 128, nh, nkv, hd,
                                                              page, RIBOZEN_WINDOW, hd ** -0.5, status)
            row(f"attention (tcgen05), window of {RIBOZEN_WINDOW}: window alone; {label}", "", T, nbytes, launch, 1)
    ops.check_status(status)
    return rows


def run_ribozen(args):
    """--only ribozen: decode (1 and 8 requests at --context) and prefill (2,048 tokens) of a Ribozen model beside the
    Zepilix model (the closest existing design: a recurrence with a matrix of state per head, short convolutions, a
    windowed attention, state rows per request) and the Llama model of the same width, heads, layers and vocabulary
    (random weights, bfloat16), and the design's own kernels alone beside their likes."""
    global BLOCK_SIZE
    import torch

    BLOCK_SIZE = args.page
    pk = peaks()
    context = args.context or CONTEXT
    if args.profile_step:
        llama = dict(SHAPES[args.shapes])
        llama["num_hidden_layers"] = args.layers or 4
        rig = make_rig(ribozen_config(llama), context, 8, args.page)
        rig.runner.use_cuda_graphs = False
        if args.profile_step == "decode":
            ms, _, _ = rig.timed_decode(args.batch, 2, 2, context)
        else:
            ms = rig.timed_prefill(args.tokens or PREFILL_TOKENS, 1, 2)
        print(json.dumps({"only": "ribozen", "profile_step": args.profile_step, "layers": llama["num_hidden_layers"], "ms": round(ms, 3)}))
        return 0
    out = {"only": "ribozen", "peaks": pk["source"], "context": context, "sizes": {}}
    for name in ([args.shapes] if args.shapes != "1b" or args.layers else ["1b", "3b"]):
        llama = dict(SHAPES[name])
        if args.layers:
            llama["num_hidden_layers"] = args.layers
        res = {}
        for label, cfg in (("ribozen", ribozen_config(llama)), ("zepilix", zepilix_config(llama)), ("llama", llama)):
            rig = make_rig(cfg, context, 8, args.page)
            for b in (1, 8):
                rig.timed_decode(b, 3, 2, context - 200)
                ms, graph_steps, _ = rig.timed_decode(b, 24, 6, context)
                nbytes = {"ribozen": ribozen_decode_bytes, "zepilix": zepilix_decode_bytes, "llama": decode_bytes}[label](cfg, b, context - 12)
                res[f"{label}_decode_b{b}_ms"] = round(ms, 4)
                res[f"{label}_decode_b{b}_tokens_per_s"] = round(b * 1000.0 / ms, 1)
                res[f"{label}_decode_b{b}_hbm_frac"] = round(nbytes / (ms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)
                res[f"{label}_decode_b{b}_graph_steps"] = graph_steps
            ms = rig.timed_prefill(PREFILL_TOKENS, 3, 2)
            if label == "ribozen":
                flops, scan = ribozen_prefill_flops(cfg, PREFILL_TOKENS)
                res["ribozen_prefill_fp32_recurrence_gflop"] = round(scan / 1e9, 2)
            elif label == "zepilix":
                flops, scan = zepilix_prefill_flops(cfg, PREFILL_TOKENS)
                res["zepilix_prefill_fp32_recurrence_gflop"] = round(scan / 1e9, 2)
            else:
                flops = prefill_flops(cfg, PREFILL_TOKENS)
            res[f"{label}_prefill_{PREFILL_TOKENS}_ms"] = round(ms, 3)
            res[f"{label}_prefill_{PREFILL_TOKENS}_tokens_per_s"] = round(PREFILL_TOKENS * 1000.0 / ms, 1)
            res[f"{label}_prefill_{PREFILL_TOKENS}_bf16_frac"] = round(flops / (ms * 1e-3) / 1e12 / pk["bf16_tflops"], 4)
            rig.close()
            del rig
            torch.cuda.empty_cache()
        out["sizes"][name] = res
        for k, v in res.items():
            print(f"{name}  {k} = {v}", file=sys.stderr)
    rows = ribozen_kernel_rows(pk, dict(SHAPES["1b"]))
    for r in rows:
        print("  ".join(f"{k}={v}" for k, v in r.items() if v != ""), file=sys.stderr)
    out["kernels"] = rows
    print(json.dumps(out))
    return 0


def main():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=256)
    p.add_argument("--warmup", type=int, default=16)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--layers", type=int, default=0, help="fewer layers than the model has (named in config)")
    p.add_argument("--only", choices=["decode", "prefill", "mixed", "serving", "kernels", "sulepel", "kaditar", "zepilix", "ribozen"], default=None,
                   help="run one kind of step and exit (for profilers and for further sizes); mixed = --batch decoding "
                        "requests beside one --tokens portion of a prompt in every step; serving = the reference's "
                        "serving benchmark (small model, prompts of 128 tokens, 32 generated: TTFT, ITL, tokens/s); "
                        "kernels = its kernel benchmark (RMSNorm and prefill attention over a grid of sizes); "
                        "sulepel = the Sulepel design beside Llama at equal sizes (decode, prefill, its kernels alone); "
                        "kaditar = the same for the Kaditar design; zepilix = the Zepilix design beside Sulepel and Llama; "
                        "ribozen = the Ribozen design beside Zepilix and Llama")
    p.add_argument("--batch-sizes", nargs="+", type=int, default=[1, 4, 8, 16], help="with --only serving")
    p.add_argument("--shapes", choices=sorted(SHAPES), default="1b", help="with --only: layer sizes of Llama-3.2-1B, 3.2-3B or 3.1-8B")
    p.add_argument("--batch", type=int, default=8, help="batch of --only decode")
    p.add_argument("--max-num-seqs", type=int, default=0,
                   help="with --only decode: the most requests the engine is set up for (0: --batch); a smaller batch "
                        "then runs as a partly filled step of the next power of two")
    p.add_argument("--page", type=int, default=BLOCK_SIZE, help="tokens per page of the cache")
    p.add_argument("--tokens", type=int, default=0, help="with --only prefill or mixed: tokens of the prompt or of its portion (at most the context and 8192)")
    p.add_argument("--context", type=int, default=0, help="with --only decode: the context the last step ends at")
    p.add_argument("--no-cuda-graphs", action="store_true", help="with --only decode: launch every kernel by itself")
    p.add_argument("--without", choices=["norms", "qkv", "attention", "o", "gate_up", "down", "head"], default=None,
                   help="with --only decode (batches up to 16): time the step with this kind of kernel left out")
    p.add_argument("--profile-step", choices=["decode", "prefill"], default=None,
                   help="with --only sulepel, kaditar, zepilix or ribozen: run a few steps of that kind launch by launch (no captured graph) on a model of "
                        "--layers layers (4 by default) and exit; for profilers")
    p.add_argument("--points", choices=["all", "1b"], default="all",
                   help="all: also decode, prefill and the mixed step at the 3B and 8B shapes (context 8192) in `points`")
    args = p.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if not args.only:
        args.warmup = max(args.warmup, 3)
    if args.only == "serving" and args.impl == "ours":
        return run_serving(args)
    if args.only == "kernels" and args.impl == "ours":
        return run_kernels(args)
    if args.only == "sulepel" and args.impl == "ours":
        return run_sulepel(args)
    if args.only == "kaditar" and args.impl == "ours":
        return run_kaditar(args)
    if args.only == "zepilix" and args.impl == "ours":
        return run_zepilix(args)
    if args.only == "ribozen" and args.impl == "ours":
        return run_ribozen(args)
    if args.impl == "reference":
        return run_reference(args)
    return run_ours(args)


if __name__ == "__main__":
    sys.exit(main())
