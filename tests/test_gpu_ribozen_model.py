"""Ribozen models through the framework (its loader, cache and state manager,
step function and kernels, driven by the trace replay program and by the
generation entry point) against the plain implementation of
tests/plain_ribozen.py: whole prompts, token-by-token decoding, portions down to
two tokens, mixed batches on a pool whose pages and state slots are used again,
long decoding over window and page borders from the first token on, greedy
generation.  The configurations differ from one another in every size and in
the order of their layers; one takes the values that make mechanisms vanish or
equal 1 (one head, one group, one tap, one expert, a window of one key, no
rotary width, a side whose constant is 0), one leaves out every key that may
be absent and has sizes the tensor-core kernels take whole, one has sizes no
kernel takes in 16-byte pieces.  Scores are sharp and some channels remember
hundreds of tokens, so that a window that is off by one key, a kept first key
that is lost or a state that is dropped moves the logits far beyond the
tolerance (asserted)."""
import copy
import json
import os

import numpy as np
import pytest
import torch

import plain_ribozen as pr
import replay_util as ru

pytestmark = pytest.mark.gpu


def moe(ff, experts, top, shared):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared:
        m["shared"] = {"ff": shared}
    return m


def mlstm(heads, dim, vdim, cap, mlp):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}, "mlp": mlp}


def mamba2(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def parallel(left, right, left_scale, right_scale, mlp):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale},
            "mlp": mlp}


def left(heads, kv_heads, dim, vdim, scale, rot, base, window=0, keep_first=None, softcap=None, scaling=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "rot": {"dims": rot, "base": base}}
    if scaling:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    if window:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if softcap:
        m["softcap"] = softcap
    return m


def right(inner, state, dt_rank, conv):
    return {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}


CONFIGS = {
    # every size its own; a layer without feed-forward, one without a shared expert
    "a": ({"architecture": "Ribozen", "vocab": 211, "width": 96, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.5},
           "layers": [mamba2(4, 24, 20, 2, 3, 4, moe(40, 5, 2, 56)),
                      parallel(left(4, 2, 16, 24, 0.9, 8, 1e4, window=21, keep_first=3, softcap=9.0, scaling=(8.0, 64, 16.0, 2.0)),
                               right(72, 10, 5, 2), 0.7, 1.2, None),
                      mlstm(3, 20, 12, 6.0, moe(24, 3, 1, 0)),
                      mamba2(2, 40, 12, 1, 4, 1, moe(32, 4, 3, 16))]}, 8),
    # the values that make a mechanism vanish or equal to 1
    "b": ({"architecture": "Ribozen", "vocab": 97, "width": 64, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
           "layers": [mlstm(1, 16, 16, 15.0, moe(32, 1, 1, 32)),
                      parallel(left(1, 1, 16, 16, 1.2, 0, 1e4, window=1, keep_first=0), right(16, 1, 1, 1), 1.0, 0.0,
                               moe(16, 2, 2, 0)),
                      mamba2(1, 16, 1, 1, 1, 1, None),
                      parallel(left(2, 2, 8, 8, 0.8, 8, 7.0, window=100000, keep_first=2, softcap=1000.0), right(24, 4, 2, 2),
                               0.0, 1.0, moe(24, 2, 1, 8))]}, 4),
    # every key that may be absent is absent (no mask, no cap on the scores, plain rates, no shared expert, no
    # feed-forward); sizes the tensor-core kernels take whole (cached heads of 64 and 128, steps of 128 rows and more),
    # a window whose kept first keys lie in tiles of their own
    "c": ({"architecture": "Ribozen", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 11.3},
           "layers": [parallel(left(4, 2, 64, 64, 0.25, 64, 1e4), right(128, 16, 8, 4), 0.5, 0.5, moe(128, 8, 2, 0)),
                      mamba2(4, 32, 64, 2, 4, 2, None),
                      parallel(left(6, 2, 64, 32, 0.3, 32, 5e5, window=70, keep_first=5, softcap=30.0, scaling=(6.0, 128, 16.0, 2.0)),
                               right(256, 16, 16, 4), 0.6, 1.1, moe(64, 4, 1, 64)),
                      mlstm(2, 64, 64, 12.0, None),
                      parallel(left(2, 2, 128, 128, 0.15, 64, 1e6, window=33, keep_first=1), right(64, 8, 4, 3), 1.3, 0.4, None)]}, 16),
    # sizes no kernel takes in 16-byte pieces; heads that are padded in the cache
    "d": ({"architecture": "Ribozen", "vocab": 130, "width": 100, "norm": {"eps": 1e-5}, "embedding": {"scale": 10.0},
           "layers": [parallel(left(3, 1, 24, 10, 0.5, 10, 1e3, window=9, keep_first=2, softcap=5.0, scaling=(2.0, 16, 4.0, 0.5)),
                               right(52, 7, 3, 3), 0.9, 0.8, moe(36, 3, 2, 20)),
                      mlstm(3, 12, 20, 4.0, moe(44, 2, 1, 0)),
                      mamba2(3, 12, 7, 3, 2, 3, None)]}, 8),
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
        d = str(tmp_path_factory.mktemp(f"ribozen_{name}_{tag}"))
        write_folder(d, cfg, weights, dtype)
        folders[tag] = d
    g = torch.Generator().manual_seed(seed)
    requests = {f"r{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate(lengths)}
    exact = {r: pr.forward(cfg, weights, ids) for r, ids in requests.items()}
    rounded = {r: pr.forward(cfg, weights, ids, round_to=torch.bfloat16) for r, ids in requests.items()}
    noise = float(np.sqrt(np.mean([float((rounded[r] - exact[r]).pow(2).mean()) for r in requests])))
    return dict(cfg=cfg, page=page, w=weights, folders=folders, requests=requests, exact=exact, rounded=rounded, noise=noise,
                prompt_lens={f"r{i}": n for i, n in enumerate(prompts)})


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return {name: make_model(tmp_path_factory, name, cfg, page, pr.random_weights(cfg, seed=len(name) + cfg["width"]),
                             LENGTHS[name], PROMPTS[name]) for name, (cfg, page) in CONFIGS.items()}


CLOSE_CALL = 0.05      # router logits nearer than this: rounding to bfloat16 may choose either expert


def close_calls(cfg, weights, ids):
    """Per position: whether some router's last chosen logit lies within
    CLOSE_CALL of the first one not chosen, here or at an earlier position
    (a choice that falls the other way also moves what the states carry on)."""
    margins = []
    pr.forward(cfg, weights, ids, margins_out=margins)
    if not margins:
        return np.zeros(len(ids), dtype=bool)
    close = (torch.stack(margins).amin(dim=0) < CLOSE_CALL).numpy()
    return np.maximum.accumulate(close)


def check(m, trace, dtype, out_dir, pool=None, what="", extra=()):
    """Runs the trace and compares every wanted place.  float32: tight.
    bfloat16: in units of what rounding activations to bfloat16 moves the plain
    implementation's own logits by (root mean square over all places): the
    median place within 1.5 units, no place beyond 30 (a key wrongly seen or
    missed, or a lost state, moves a place by 50 and more; where rounding
    alone flips a router's choice the plain implementation's own rounded run
    is as far off, and the place is measured from that run instead; places
    at or behind a router's close call are left out of this bound: no
    comparison rests on which way such a call falls), and no more loud places
    than twice what the plain implementation's own rounded run has."""
    pool = pool or sum((len(v) + 63) // 64 * 64 for v in m["requests"].values())
    got = ru.run_trace(trace, m["folders"][dtype], dtype, str(out_dir), pool, m["page"], extra=extra)
    assert len(got) == sum(len(w) for w in trace.wanted)
    if dtype == "float32":
        return ru.compare(got, {r: v.float() for r, v in m["exact"].items()}, atol=3e-4, rtol=3e-4, what=what)
    units, own, near = [], [], []
    close = m.setdefault("close", {})
    for (rid, p), row in sorted(got.items()):
        assert np.all(np.isfinite(row))
        if rid not in close:
            close[rid] = close_calls(m["cfg"], m["w"], m["requests"][rid])
        d = row.astype(np.float64) - m["exact"][rid][p].numpy()
        units.append(float(np.sqrt(np.mean(d * d))) / m["noise"])
        own.append(float((m["rounded"][rid][p] - m["exact"][rid][p]).pow(2).mean().sqrt()) / m["noise"])
        d = row.astype(np.float64) - m["rounded"][rid][p].numpy()
        near.append(0.0 if close[rid][p] else min(units[-1], float(np.sqrt(np.mean(d * d))) / m["noise"]))
    worst = int(np.argmax(near))
    assert near[worst] <= 30.0, f"{what}: place {sorted(got)[worst]}: {near[worst]:.1f} units of rounding noise"
    assert float(np.median(units)) <= 1.5, f"{what}: the median place lies {np.median(units):.2f} units of rounding noise off"
    loud, loud_own = sum(u > 4.0 for u in units), sum(u > 4.0 for u in own)
    assert loud <= 2 * loud_own + max(2, len(units) // 50), \
        f"{what}: {loud} of {len(units)} places above 4 units of rounding noise (the plain rounded run: {loud_own})"
    return float(np.median(units))


def test_a_window_or_a_kept_key_that_is_one_off_would_show(models):
    """The plain implementation with every window one key longer or shorter,
    or one more or one fewer first key kept, moves the logits by far more than
    the comparisons allow."""
    m = models["a"]
    ids = m["requests"]["r2"]
    for key, change in (("size", 1), ("size", -1), ("keep_first", 1), ("keep_first", -1)):
        cfg = copy.deepcopy(m["cfg"])
        cfg["layers"][1]["mixer"]["left"]["mask"][key] += change
        moved = (pr.forward(cfg, m["w"], ids) - m["exact"]["r2"]).abs().amax(dim=-1)
        assert float(moved[:20].max()) == 0.0              # (places that see fewer keys than the window holds)
        # (the float32 comparison allows 3e-4; the bfloat16 one counts places beyond 4 units of rounding noise)
        assert float(moved[30:].median()) > 10 * 3e-4 and float(moved[30:].pow(2).mean().sqrt()) > 4 * m["noise"], (key, change)


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
        exact[rid + "x"] = pr.forward(m["cfg"], m["w"], requests[rid + "x"])
        rounded[rid + "x"] = pr.forward(m["cfg"], m["w"], requests[rid + "x"], round_to=torch.bfloat16)
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
    window and many pages (the captured decode step serves it; the matrix
    memory, the scans' states and the convolutions' last inputs pass from step
    to step 170 times), beside a second request that joins late."""
    m = models[name]
    g = torch.Generator().manual_seed(3)
    ids = torch.randint(0, m["cfg"]["vocab"], (170,), generator=g).tolist()
    other = m["requests"]["r1"]
    exact = {"long": pr.forward(m["cfg"], m["w"], ids), "r1": m["exact"]["r1"]}
    rounded = {"long": pr.forward(m["cfg"], m["w"], ids, round_to=torch.bfloat16), "r1": m["rounded"]["r1"]}
    t = ru.Trace()
    for i, tok in enumerate(ids):
        entries = [("long", [tok], [0])]
        j = i - 100
        if 0 <= j < len(other):
            entries.append(("r1", [other[j]], [0]))
        t.step(entries, end=(["long"] if i == len(ids) - 1 else []) + (["r1"] if j == len(other) - 1 else []))
    check(dict(m, requests={"long": ids, "r1": other}, exact=exact, rounded=rounded), t, dtype, tmp_path, pool=256,
          what=f"{name} {dtype} long decoding")
    assert ru.read_pages(str(tmp_path))["graph_steps"] > 100


def test_a_kept_first_key_decides(tmp_path_factory, tmp_path):
    """One layer of attention beside a scan whose constant is 0, a window of 16
    keys that keeps the first two: hundreds of positions on, what the first
    two tokens were still moves the logits (through nothing but their kept
    keys, by many times what the comparison allows), and what the third was moves nothing.  The engine must agree with the
    plain implementation in a whole prompt, in portions and token by token."""
    cfg = {"architecture": "Ribozen", "vocab": 50, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 2.0},
           "layers": [parallel(left(2, 1, 16, 16, 1.0, 8, 1e4, window=16, keep_first=2, softcap=20.0), right(16, 4, 2, 2),
                               1.0, 0.0, None)]}
    w = pr.random_weights(cfg, seed=5, sharp=6.0)
    g = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 50, (330,), generator=g).tolist()
    m = make_model(tmp_path_factory, "kept", cfg, 8, w, (1,), (1,))
    m["requests"] = {"kept": ids}
    m["exact"] = {"kept": pr.forward(cfg, w, ids)}
    m["rounded"] = {"kept": pr.forward(cfg, w, ids, round_to=torch.bfloat16)}
    for at, moves in ((0, True), (1, True), (2, False)):
        other = list(ids)
        other[at] = (ids[at] + 7) % 50
        moved = (pr.forward(cfg, w, other)[300:] - m["exact"]["kept"][300:]).abs().amax(dim=-1)
        if moves:
            assert float(moved.median()) > 10 * 3e-4, at
        else:
            assert float(moved.max()) == 0.0, at
    for dtype in ("float32", "bfloat16"):
        for k, trace in enumerate((ru.whole_trace(m["requests"]), ru.tail_trace(m["requests"], tail=40),
                                   ru.portions_trace(m["requests"], sizes=(3, 130, 2, 64, 100, 2)))):
            check(m, trace, dtype, tmp_path / f"{dtype}{k}", what=f"kept key {dtype} {k}")


def test_a_far_token_decides_through_the_states(tmp_path_factory, tmp_path):
    """A state-space layer and a matrix memory that hardly forget: what a
    token hundreds of positions back was moves the last logits by many times
    what the comparison allows, through nothing but the states.
    The engine must agree with the plain implementation in a whole prompt, in
    portions and token by token (a state that is lost or zeroed on the way
    would show)."""
    cfg = {"architecture": "Ribozen", "vocab": 40, "width": 32, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.5},
           "layers": [mamba2(2, 16, 8, 1, 2, 2, None), mlstm(2, 16, 16, 12.0, None)]}
    w = pr.random_weights(cfg, seed=9)
    w["l0.mix.A_log"] = torch.full((2,), -7.0, dtype=torch.float64)
    w["l1.mix.f.b"] = torch.full((2,), 9.0, dtype=torch.float64)
    g = torch.Generator().manual_seed(2)
    ids = torch.randint(0, 40, (402,), generator=g).tolist()
    m = make_model(tmp_path_factory, "far", cfg, 8, w, (1,), (1,))
    m["requests"] = {"far": ids}
    m["exact"] = {"far": pr.forward(cfg, w, ids)}
    m["rounded"] = {"far": pr.forward(cfg, w, ids, round_to=torch.bfloat16)}
    lost = list(ids)
    lost[5] = (ids[5] + 3) % 40
    moved = (pr.forward(cfg, w, lost)[401] - m["exact"]["far"][401]).abs().max()
    assert float(moved) > 10 * 3e-4
    for dtype in ("float32", "bfloat16"):
        for k, trace in enumerate((ru.whole_trace(m["requests"]), ru.tail_trace(m["requests"], tail=12),
                                   ru.portions_trace(m["requests"], sizes=(3, 130, 2, 64, 200, 2)))):
            check(m, trace, dtype, tmp_path / f"{dtype}{k}", what=f"far token {dtype} {k}")


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
        assert o.output_tokens == pr.greedy(m["cfg"], m["w"], p, 9), (p, o.output_tokens)
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
        assert o.output_tokens == pr.greedy(m["cfg"], m["w"], p, 7), (p, o.output_tokens)


def test_window_pages_are_given_back_but_the_kept_keys_pages_stay(models):
    """A windowed layer holds one request's window and the pages of its kept
    first keys, not its whole context."""
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
                kept = (group.keep_first + 7) // 8
                assert kept <= cache.manager.get_num_used_blocks(gi) <= (group.window + 7) // 8 + 1 + kept
                assert seq.get_block_tables()[gi][0] >= 0             # the page of the kept keys is still held
        assert cache.manager.audit() == ""
    torch.testing.assert_close(torch.cat(got), m["exact"]["r3"].float(), atol=3e-4, rtol=3e-4)


def test_the_stream_after_every_layer(models):
    """The residual stream after every layer (what is still pending entered)
    against the plain implementation."""
    from lyapunov_engine_b200 import build
    from lyapunov_engine_b200.cache import DeviceCache
    from lyapunov_engine_b200.engine.llm_engine import load_model
    from lyapunov_engine_b200.engine.step import ModelRunner
    from lyapunov_engine_b200.parts.base import ScaledAddend
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
            if isinstance(stream.update, ScaledAddend):
                y = y * stream.update.weight
            x = x + y
        seen.append(x.cpu())

    forward = loaded.model.forward
    loaded.model.forward = lambda ctx, c: forward(ctx, c, observe=observe)
    seq = host.Sequence(0, ids, host.SamplingParams())
    assert cache.manager.grow(seq, len(ids))
    runner.step([host.StepEntry(seq, 0, len(ids), [0])])
    want = []
    pr.forward(m["cfg"], m["w"], ids, layers_out=want)
    assert len(seen) == len(want) == len(m["cfg"]["layers"])
    for got, ref in zip(seen, want):
        torch.testing.assert_close(got, ref.float(), atol=2e-4, rtol=2e-4)


def draw_config(rng):
    """A configuration with every size and the order of the layers drawn at random."""
    def mlp():
        if rng.random() < 0.2:
            return None
        experts = rng.choice([2, 4, 8, 16])
        return moe(rng.choice([64, 96, 128, 200]), experts, rng.choice([t for t in (1, 2, 4) if t <= experts]),
                   rng.choice([0, 64, 96, 160]))

    def a_matrix_memory():
        return mlstm(rng.choice([1, 2, 4]), rng.choice([16, 32, 48, 64, 96]), rng.choice([16, 32, 64, 80, 128]),
                     rng.choice([5.0, 12.0, 20.0]), mlp())

    def a_duality():
        heads = rng.choice([2, 4, 6, 8])
        vdim = rng.choice([16, 32, 48, 64])
        return mamba2(heads, vdim, rng.choice([16, 24, 48, 64, 128]), rng.choice([g for g in (1, 2, 3, 4) if heads % g == 0]),
                      rng.choice([2, 3, 4]), rng.choice([g for g in (1, 2, 4) if (heads * vdim) % g == 0]), mlp())

    def a_pair():
        heads, dim = rng.choice([2, 4, 6, 8]), rng.choice([32, 64, 96, 128])
        scaling = None if rng.random() < 0.3 else (rng.choice([2.0, 4.0, 8.0]), rng.choice([64, 256, 2048]),
                                                   rng.choice([16.0, 32.0]), rng.choice([1.0, 2.0]))
        window = rng.choice([0, 17, 40, 64, 100, 150])
        return parallel(left(heads, rng.choice([g for g in (1, 2, 3, 4, 8) if heads % g == 0]), dim,
                             rng.choice([dim, dim // 2, 32, 16]), rng.uniform(0.1, 0.3), rng.choice([dim, dim // 2, 16, 8]),
                             rng.choice([1e4, 5e4, 5e5, 1e6]), window=window,
                             keep_first=rng.choice([None, 0, 1, 4, 20]) if window else None,
                             softcap=rng.choice([None, 10.0, 50.0]), scaling=scaling),
                        right(rng.choice([64, 128, 192, 320]), rng.choice([8, 16, 24, 64]), rng.choice([4, 8, 12, 16]),
                              rng.choice([2, 3, 4])), rng.uniform(0.4, 1.3), rng.uniform(0.4, 1.3), mlp())

    n = rng.choice([3, 4, 5])
    kinds = [a_matrix_memory, a_duality, a_pair] + [rng.choice([a_matrix_memory, a_duality, a_pair]) for _ in range(n - 3)]
    rng.shuffle(kinds)
    return {"architecture": "Ribozen", "vocab": rng.choice([300, 512, 777, 1000]), "width": rng.choice([128, 192, 256, 320, 384]),
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "embedding": {"scale": rng.uniform(1.0, 20.0)},
            "layers": [kind() for kind in kinds]}


@pytest.mark.parametrize("seed", [31, 32, 33])
def test_configurations_drawn_at_random(seed, tmp_path_factory, tmp_path):
    """Sizes, layer order and page size drawn at random: whole prompts,
    portions and a mixed batch on a pool that just holds the peak, both types."""
    import random
    rng = random.Random(seed)
    cfg, page = draw_config(rng), rng.choice([16, 32, 64])
    m = make_model(tmp_path_factory, f"drawn{seed}", cfg, page, pr.random_weights(cfg, seed=seed), (150, 70, 260, 33),
                   (120, 64, 200, 2))
    for dtype in ("float32", "bfloat16"):
        check(m, ru.whole_trace(m["requests"]), dtype, tmp_path / f"w{dtype}", what=f"drawn {seed} {dtype} whole")
        check(m, ru.portions_trace(m["requests"]), dtype, tmp_path / f"p{dtype}", what=f"drawn {seed} {dtype} portions")
        trace = ru.mixed_trace(m["requests"], m["prompt_lens"], chunk=16, max_live=4, seed=5)
        check(m, trace, dtype, tmp_path / f"m{dtype}", pool=ru.peak_pool_tokens(trace, page), what=f"drawn {seed} {dtype} mixed",
              extra=("--max-num-seqs", "4"))


def test_command_line_generates_from_random_weights(tmp_path):
    """`generate --random-weights` builds a Ribozen model from a config.json alone."""
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
