"""Zepilix models through the framework (its loader, cache and state manager,
step function and kernels, driven by the trace replay program and by the
generation entry point) against the plain implementation of
tests/plain_zepilix.py: whole prompts, token-by-token decoding, portions down to
two tokens, mixed batches on a pool whose pages and state slots are used again,
long decoding over window and page borders from the first token on, greedy
generation.  The configurations differ from one another in every size and in
the order of their layers; one takes the values that make mechanisms vanish
(a loop that runs once, one head, one tap, a window of one key and one longer
than any sequence, no rotary width), one leaves out every key that may be
absent and has sizes the tensor-core kernels take whole, one has sizes no
kernel takes in 16-byte pieces.  Scores are sharp, so that a window that is off
by one key or a far key that is lost moves the logits far beyond the
tolerance (asserted)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_zepilix as pz
import replay_util as ru

pytestmark = pytest.mark.gpu


def delta(heads, kv_heads, dim, vdim, conv, ff):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def attn(heads, kv_heads, dim, rot, base, scale, ff):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale,
                                           "rot": {"dims": rot, "base": base}},
            "mlp": {"kind": "dense", "ff": ff} if ff else None}


def latent(heads, dim, rot_dim, vdim, kv_rank, q_rank, window, base, scale, ff):
    mixer = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "q_rank": q_rank,
             "scale": scale, "rot": {"dims": rot_dim, "base": base}}
    if window:
        mixer["mask"] = {"size": window}
    return {"type": "latent_attention", "mixer": mixer, "mlp": {"kind": "dense", "ff": ff} if ff else None}


CONFIGS = {
    # every size its own; the loop opens with a delta layer without feed-forward and runs three times
    "a": ({"architecture": "Zepilix", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "token_side": {"dim": 24},
           "loop": {"start": 1, "stop": 3, "times": 3},
           "layers": [latent(3, 16, 8, 24, 40, 56, 21, 1e4, 0.3, 160),
                      delta(4, 2, 16, 24, 3, 0),
                      attn(4, 2, 32, 16, 5e5, 0.4, 72),
                      delta(2, 2, 48, 16, 5, 40)]}, 8),
    # the values that make a mechanism vanish or equal to 1
    "b": ({"architecture": "Zepilix", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "token_side": {"dim": 8},
           "loop": {"start": 0, "stop": 2, "times": 1},
           "layers": [delta(1, 1, 16, 16, 1, 32),
                      latent(1, 16, 0, 16, 16, 8, 1, 1e4, 0.5, 48),
                      attn(1, 1, 16, 0, 1e4, 0.7, 0),
                      latent(2, 8, 4, 8, 12, 16, 100000, 7.0, 0.6, 40)]}, 4),
    # every key that may be absent is absent (no loop, no input per token, all keys visible); sizes the tensor-core
    # kernels take whole (cached heads of 64 and 128, 128 rows and more per step), pages of 16
    "c": ({"architecture": "Zepilix", "vocab": 300, "width": 128, "norm": {"eps": 1e-5},
           "layers": [attn(4, 2, 64, 64, 1e4, 0.25, 256),
                      delta(2, 1, 128, 64, 4, 128),
                      latent(4, 32, 16, 32, 112, 64, 0, 1e6, 0.2, 128),
                      attn(2, 2, 128, 32, 5e5, 0.15, 0)]}, 16),
    # sizes no kernel takes in 16-byte pieces; heads that are padded in the cache; a loop that ends with the last layer
    "d": ({"architecture": "Zepilix", "vocab": 130, "width": 100, "norm": {"eps": 1e-5}, "token_side": {"dim": 5},
           "loop": {"start": 1, "stop": 3, "times": 2},
           "layers": [attn(3, 1, 24, 10, 1e3, 0.5, 44),
                      delta(3, 1, 20, 12, 2, 36),
                      latent(2, 12, 6, 12, 50, 20, 9, 1e4, 0.4, 0)]}, 8),
}
LENGTHS = {"a": (23, 47, 75, 141), "b": (9, 70, 35, 101), "c": (40, 130, 301, 215), "d": (12, 66, 31, 90)}
PROMPTS = {"a": (3, 30, 41, 100), "b": (1, 64, 2, 67), "c": (8, 128, 260, 101), "d": (2, 40, 30, 51)}


def write_folder(folder, cfg, weights, dtype):
    from safetensors.torch import save_file
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as f:
        json.dump(cfg, f)
    save_file({k: v.to(dtype).contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))


def make_model(tmp_path_factory, name, cfg, page, weights, lengths, prompts, seed=7):
    folders = {}
    for dtype in (torch.float32, torch.bfloat16):
        tag = "float32" if dtype == torch.float32 else "bfloat16"
        d = str(tmp_path_factory.mktemp(f"zepilix_{name}_{tag}"))
        write_folder(d, cfg, weights, dtype)
        folders[tag] = d
    g = torch.Generator().manual_seed(seed)
    requests = {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    exact = {r: pz.forward(cfg, weights, ids) for r, ids in requests.items()}
    rounded = {r: pz.forward(cfg, weights, ids, round_to=torch.bfloat16) for r, ids in requests.items()}
    noise = float(np.sqrt(np.mean([float((rounded[r] - exact[r]).pow(2).mean()) for r in requests])))
    return dict(cfg=cfg, page=page, w=weights, folders=folders, requests=requests, exact=exact, rounded=rounded, noise=noise,
                prompt_lens={f"r{i}": n for i, n in enumerate(prompts)})


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: make_model(tmp_path_factory, name, cfg, page, pz.random_weights(cfg, seed=len(name) + cfg["width"]),
                             LENGTHS[name], PROMPTS[name]) for name, (cfg, page) in CONFIGS.items()}


def check(m, trace, dtype, out_dir, pool=None, what="", extra=()):
    """Runs the trace and compares every wanted place.  float32: tight.
    bfloat16: in units of what rounding activations to bfloat16 moves the plain
    implementation's own logits by (root mean square over all places): the
    median place within 1.5 units, no place beyond 30 (a key wrongly seen or
    missed moves a place by 50 and more), and no more loud places than twice
    what the plain implementation's own rounded run has."""
    pool = pool or sum((len(v) + 63) // 64 * 64 for v in m["requests"].values())
    got = ru.run_trace(trace, m["folders"][dtype], dtype, str(out_dir), pool, m["page"], extra=extra)
    assert len(got) == sum(len(w) for w in trace.wanted)
    if dtype == "float32":
        return ru.compare(got, {r: v.float() for r, v in m["exact"].items()}, atol=3e-4, rtol=3e-4, what=what)
    units, own = [], []
    for (rid, p), row in sorted(got.items()):
        assert np.all(np.isfinite(row))
        d = row.astype(np.float64) - m["exact"][rid][p].numpy()
        units.append(float(np.sqrt(np.mean(d * d))) / m["noise"])
        own.append(float((m["rounded"][rid][p] - m["exact"][rid][p]).pow(2).mean().sqrt()) / m["noise"])
    worst = int(np.argmax(units))
    assert units[worst] <= 30.0, f"{what}: place {sorted(got)[worst]}: {units[worst]:.1f} units of rounding noise"
    assert float(np.median(units)) <= 1.5, f"{what}: the median place lies {np.median(units):.2f} units of rounding noise off"
    loud, loud_own = sum(u > 4.0 for u in units), sum(u > 4.0 for u in own)
    assert loud <= 2 * loud_own + max(2, len(units) // 50), \
        f"{what}: {loud} of {len(units)} places above 4 units of rounding noise (the plain rounded run: {loud_own})"
    return float(np.median(units))


def test_a_window_that_is_one_key_off_would_show(models):
    """The plain implementation with every window one key longer or shorter
    moves the logits by far more than the comparisons allow."""
    m = models["a"]
    ids = m["requests"]["r2"]
    for change in (1, -1):
        cfg = copy.deepcopy(m["cfg"])
        for layer in cfg["layers"]:
            if "mask" in layer["mixer"]:
                layer["mixer"]["mask"]["size"] += change
        moved = (pz.forward(cfg, m["w"], ids) - m["exact"]["r2"]).abs().amax(dim=-1)
        assert float(moved[:20].max()) == 0.0              # (places that see fewer keys than the window holds)
        assert float(moved[30:].median()) > 100 * 3e-4 and float(moved[30:].pow(2).mean().sqrt()) > 10 * m["noise"]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompts(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.whole_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prefill_then_token_by_token(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.tail_trace(m["requests"], tail=44), dtype, tmp_path, what=f"{name} {dtype} decode")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_portions_down_to_two_tokens(models, name, dtype, tmp_path):
    m = models[name]
    check(m, ru.portions_trace(m["requests"]), dtype, tmp_path, what=f"{name} {dtype} portions")
    check(m, ru.portions_trace(m["requests"], sizes=(2, 2, 3, 2, 129, 2)), dtype, tmp_path, what=f"{name} {dtype} small portions")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_mixed_batches_on_a_pool_that_is_used_again(models, name, dtype, tmp_path):
    """Twice the requests, up to four live on four state slots, on a pool that
    just holds the peak: late requests get pages and state rows that others
    gave back with their keys and state still in them."""
    m = models[name]
    requests, prompts, exact, rounded = dict(m["requests"]), dict(m["prompt_lens"]), dict(m["exact"]), dict(m["rounded"])
    g = torch.Generator().manual_seed(11)
    for rid, ids in list(m["requests"].items()):
        requests[rid + "x"] = torch.randint(0, m["cfg"]["vocab"], (len(ids),), generator=g).tolist()
        prompts[rid + "x"] = m["prompt_lens"][rid]
        exact[rid + "x"] = pz.forward(m["cfg"], m["w"], requests[rid + "x"])
        rounded[rid + "x"] = pz.forward(m["cfg"], m["w"], requests[rid + "x"], round_to=torch.bfloat16)
    trace = ru.mixed_trace(requests, prompts, chunk=16, max_live=4, seed=5)
    assert any(len(s["entries"]) >= 3 for s in trace.steps)
    m2 = dict(m, requests=requests, exact=exact, rounded=rounded)
    check(m2, trace, dtype, tmp_path, pool=ru.peak_pool_tokens(trace, m["page"]), what=f"{name} {dtype} mixed",
          extra=("--max-num-seqs", "4"))
    pages = ru.read_pages(str(tmp_path))
    assert pages["allocations"] > pages["pool_pages"] and pages["reuses"] > 0, pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["a", "d"])
def test_first_tokens_and_long_decoding(models, name, dtype, tmp_path):
    """One request token by token from its first token on, far past every
    window and many pages (the captured decode step serves it; the delta rule's
    state and the convolutions' last inputs pass from step to step 170 times),
    beside a second request that joins late."""
    m = models[name]
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, m["cfg"]["vocab"], (170,), generator=g).tolist()
    other = m["requests"]["r1"]
    exact = {"long": pz.forward(m["cfg"], m["w"], ids), "r1": m["exact"]["r1"]}
    rounded = {"long": pz.forward(m["cfg"], m["w"], ids, round_to=torch.bfloat16), "r1": m["rounded"]["r1"]}
    t = ru.Trace()
    for i, tok in enumerate(ids):
        entries = [("long", [tok], [0])]
        j = i - 100
        if 0 <= j < len(other):
            entries.append(("r1", [other[j]], [0]))
        t.step(entries, end=(["long"] if i == len(ids) - 1 else []) + (["r1"] if j == len(other) - 1 else []))
    check(dict(m, exact=exact, rounded=rounded), t, dtype, tmp_path, pool=256, what=f"{name} {dtype} long decoding")
    assert ru.read_pages(str(tmp_path))["graph_steps"] > 100


def test_a_far_key_decides(tmp_path_factory, tmp_path):
    """One attention layer whose weights make one token look for another: its
    query is the other token's key (the query projection is a turn of the
    space, and this token's embedding is the other's turned back), and the
    values are the keys, so what it reads is the other token's vector.  The
    other token stands once, hundreds of positions and many pages back, and
    decides the output.  Losing that key (shown on the plain implementation by
    changing the far token) moves the logits by orders of magnitude more than
    the comparison allows; the engine must agree with the plain implementation
    in a whole prompt, in portions and token by token."""
    W = 32
    cfg = {"architecture": "Zepilix", "vocab": 40, "width": W, "norm": {"eps": 1e-6},
           "layers": [attn(2, 1, 32, 8, 1e4, 0.6, 0)]}
    w = pz.random_weights(cfg, seed=5)
    g = torch.Generator().manual_seed(1)
    turn = torch.linalg.qr(torch.randn(W, W, generator=g, dtype=torch.float64))[0]
    eye = torch.eye(W, dtype=torch.float64)
    w["l0.mix.k"] = eye.clone()
    w["l0.mix.q"] = torch.cat([turn, turn], dim=0)
    w["l0.mix.o"] = torch.cat([eye, eye], dim=1) * 0.5
    w["l0.norm1"] = torch.zeros(W, dtype=torch.float64)
    w["embed"][36] = turn.T @ w["embed"][35]
    ids = torch.randint(1, 30, (400,), generator=g).tolist()
    ids[5] = 35
    ids += [36, 3]
    m = make_model(tmp_path_factory, "far", cfg, 8, w, (1,), (1,))
    m["requests"] = {"far": ids}
    m["exact"] = {"far": pz.forward(cfg, w, ids)}
    m["rounded"] = {"far": pz.forward(cfg, w, ids, round_to=torch.bfloat16)}
    lost = list(ids)
    lost[5] = 7
    moved = (pz.forward(cfg, w, lost)[400] - m["exact"]["far"][400]).abs().max()
    assert float(moved) > 1000 * 3e-4
    for dtype in ("float32", "bfloat16"):
        for k, trace in enumerate((ru.whole_trace(m["requests"]), ru.tail_trace(m["requests"], tail=12),
                                   ru.portions_trace(m["requests"], sizes=(3, 130, 2, 64, 200, 2)))):
            check(m, trace, dtype, tmp_path / f"{dtype}{k}", what=f"far key {dtype} {k}")


def test_state_rows_and_pages_are_given_back_and_zeroed(models, tmp_path):
    """Two state slots for five requests: every late request starts in a row
    that still holds an earlier request's state, and must start from zero."""
    from lyapunov_engine_b200 import LLMEngine, SamplingParams
    m = models["a"]
    engine = LLMEngine.from_pretrained(m["folders"]["float32"], dtype="float32", num_blocks=40, block_size=m["page"],
                                       max_num_seqs=2, max_num_batched_tokens=24, max_model_len=160)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, m["cfg"]["vocab"], (n,), generator=g).tolist() for n in (3, 37, 1, 26, 12)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=9, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == pz.greedy(m["cfg"], m["w"], p, 9), (p, o.output_tokens)
        assert o.finish_reason == "length"
    assert engine.block_manager.audit() == ""


@pytest.mark.parametrize("name", ["b", "c"])
def test_greedy_generation_through_the_entry_point(models, name):
    from lyapunov_engine_b200 import LLMEngine, SamplingParams
    m = models[name]
    engine = LLMEngine.from_pretrained(m["folders"]["float32"], dtype="float32", num_blocks=64, block_size=m["page"],
                                       max_num_seqs=3, max_num_batched_tokens=32, max_model_len=192)
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, m["cfg"]["vocab"], (n,), generator=g).tolist() for n in (5, 41, 2, 19)]
    outs = engine.generate(prompts, SamplingParams(temperature=0.0, max_tokens=7, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert o.output_tokens == pz.greedy(m["cfg"], m["w"], p, 7), (p, o.output_tokens)


def test_window_pages_are_given_back_while_a_request_lives(models):
    """Every pass of a windowed layer holds one request's window, not its whole context."""
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner
    m = models["d"]
    host = build.load_host()
    loaded = load_model(m["folders"]["float32"], "float32", "cuda:0", max_model_len=256)
    cache = DeviceCache(loaded.model, loaded.runtime, num_blocks=32, block_size=8, max_num_seqs=2)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 256, 2, 256, use_cuda_graphs=False, check_status=True)
    ids = m["requests"]["r3"]
    seq = host.Sequence(0, ids, host.SamplingParams())
    got, pos = [], 0
    for n in (50, 3, 1, 1, 20, 2, 13):
        assert cache.manager.grow(seq, pos + n)
        got.append(runner.step([host.StepEntry(seq, pos, n, list(range(n)))]).cpu())
        pos += n
        seq.set_num_computed_tokens(pos)
        cache.manager.release_passed(seq)
        for gi, group in enumerate(loaded.model.groups):
            if group.window:
                assert cache.manager.get_num_used_blocks(gi) <= (group.window + 7) // 8 + 1
        assert cache.manager.audit() == ""
    torch.testing.assert_close(torch.cat(got), m["exact"]["r3"].float(), atol=3e-4, rtol=3e-4)


def test_the_stream_after_every_layer_run(models):
    """The residual stream after every run of a layer (looped layers count each
    time; what is still pending entered) against the plain implementation."""
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner
    from lyapunov_engine_b200.parts.base import NormedAddend
    m = models["a"]
    host = build.load_host()
    loaded = load_model(m["folders"]["float32"], "float32", "cuda:0", max_model_len=128)
    cache = DeviceCache(loaded.model, loaded.runtime, 32, m["page"], 1)
    runner = ModelRunner(loaded.model, cache, loaded.runtime, 128, 1, 128, use_cuda_graphs=False, check_status=True)
    ids = m["requests"]["r1"]
    seen = []

    def observe(index, stream):
        x = stream.resid.clone()
        y = stream.pending
        if y is not None:
            y = (y.sum(0) if y.dim() == 3 else y).float()
            if isinstance(stream.update, NormedAddend):
                y = y / torch.sqrt(y.pow(2).mean(-1, keepdim=True) + stream.update.eps) * stream.update.weight
            x = x + y
        seen.append(x.cpu())

    forward = loaded.model.forward
    loaded.model.forward = lambda ctx, c: forward(ctx, c, observe=observe)
    seq = host.Sequence(0, ids, host.SamplingParams())
    assert cache.manager.grow(seq, len(ids))
    runner.step([host.StepEntry(seq, 0, len(ids), [0])])
    want = []
    pz.forward(m["cfg"], m["w"], ids, layers_out=want)
    assert len(seen) == len(want) == 1 + 2 * 3 + 1
    for got, ref in zip(seen, want):
        torch.testing.assert_close(got, ref.float(), atol=2e-4, rtol=2e-4)


def draw_config(rng):
    """A configuration with every size, the order of the layers and the loop drawn at random."""
    def mlp():
        return 0 if rng.random() < 0.15 else rng.choice([192, 256, 328, 448, 520, 1000])

    def a_delta():
        heads = rng.choice([1, 2, 4, 8])
        return delta(heads, rng.choice([g for g in (1, 2, 4, 8) if heads % g == 0]), rng.choice([16, 32, 48, 64, 96, 128]),
                     rng.choice([16, 32, 64, 80, 128]), rng.choice([2, 3, 4]), mlp())

    def an_attention():
        heads, dim = rng.choice([2, 4, 6, 8]), rng.choice([32, 64, 96, 128])
        return attn(heads, rng.choice([g for g in (1, 2, 3, 4, 8) if heads % g == 0]), dim, rng.choice([dim, dim // 2, 16, 8]),
                    rng.choice([1e4, 5e4, 5e5, 1e6]), rng.uniform(0.1, 0.3), mlp())

    def a_latent():
        return latent(rng.choice([2, 4, 5, 8]), rng.choice([32, 64, 128]), rng.choice([8, 16, 32, 64]), rng.choice([32, 64, 80, 128]),
                      rng.choice([32, 48, 64, 96, 128, 160]), rng.choice([48, 80, 96, 128]),
                      rng.choice([0, 17, 40, 64, 100, 150]), rng.choice([1e4, 1e6]), rng.uniform(0.08, 0.2), mlp())

    n = rng.choice([3, 4, 5])
    kinds = [a_delta, an_attention, a_latent] + [rng.choice([a_delta, an_attention, a_latent]) for _ in range(n - 3)]
    rng.shuffle(kinds)
    cfg = {"architecture": "Zepilix", "vocab": rng.choice([300, 512, 777, 1000]), "width": rng.choice([128, 192, 256, 320, 384]),
           "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": [kind() for kind in kinds]}
    if rng.random() < 0.85:
        cfg["token_side"] = {"dim": rng.choice([8, 16, 24, 32])}
    if rng.random() < 0.8:
        start = rng.randrange(0, n)
        cfg["loop"] = {"start": start, "stop": rng.randrange(start + 1, n + 1), "times": rng.choice([2, 2, 3])}
    return cfg


@pytest.mark.parametrize("seed", [21, 22, 23])
def test_configurations_drawn_at_random(seed, tmp_path_factory, tmp_path):
    """Sizes, layer order, loop and page size drawn at random: whole prompts,
    portions and a mixed batch on a pool that just holds the peak, both types."""
    import random
    rng = random.Random(seed)
    cfg, page = draw_config(rng), rng.choice([16, 32, 64])
    m = make_model(tmp_path_factory, f"drawn{seed}", cfg, page, pz.random_weights(cfg, seed=seed), (150, 70, 260, 33),
                   (120, 64, 200, 2))
    for dtype in ("float32", "bfloat16"):
        check(m, ru.whole_trace(m["requests"]), dtype, tmp_path / f"w{dtype}", what=f"drawn {seed} {dtype} whole")
        check(m, ru.portions_trace(m["requests"]), dtype, tmp_path / f"p{dtype}", what=f"drawn {seed} {dtype} portions")
        trace = ru.mixed_trace(m["requests"], m["prompt_lens"], chunk=16, max_live=4, seed=5)
        check(m, trace, dtype, tmp_path / f"m{dtype}", pool=ru.peak_pool_tokens(trace, page), what=f"drawn {seed} {dtype} mixed",
              extra=("--max-num-seqs", "4"))


def test_command_line_generates_from_random_weights(tmp_path):
    """`generate --random-weights` builds a Zepilix model from a config.json alone."""
    import subprocess
    import sys
    cfg = CONFIGS["b"][0]
    folder = tmp_path / "cfg"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "lyapunov"), "generate", "--model", str(folder),
                           "--random-weights", "--prompt-ids", "1,2,3", "--max-tokens", "4", "--temperature", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
