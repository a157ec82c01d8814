"""What of the Ribozen design needs no GPU: config.json key by key, what the
cache and the state slots must hold, pages of kept first keys that a window
never gives back, the ramped rotary rates, and the plain implementation's own
pieces against each other."""
import copy
import math

import pytest
import torch

import plain_ribozen as pr
from lyapunov_engine_b200 import build
from lyapunov_engine_b200.config.base import ConfigError
from lyapunov_engine_b200.config.ribozen import RibozenConfig
from lyapunov_engine_b200.models.model import Model
from lyapunov_engine_b200.parts.rope import ramped_rates
from lyapunov_engine_b200.registry import spec_for

MOE = {"kind": "moe", "expert": {"ff": 24}, "router": {"experts": 4, "top": 2}, "shared": {"ff": 16}}
CFG = {"architecture": "Ribozen", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
       "layers": [{"type": "mamba2", "mixer": {"heads": 4, "vdim": 8, "state": 6, "groups": 2, "conv": 3, "norm_groups": 2},
                   "mlp": MOE},
                  {"type": "parallel",
                   "mixer": {"left_scale": 0.8, "right_scale": 1.3,
                             "left": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "scale": 0.3, "softcap": 20.0,
                                      "rot": {"dims": 4, "base": 100.0,
                                              "scaling": {"factor": 3.0, "original": 32, "fast": 8.0, "slow": 1.0}},
                                      "mask": {"size": 6, "keep_first": 2}},
                             "right": {"inner": 24, "state": 5, "dt_rank": 3, "conv": 2}},
                   "mlp": None},
                  {"type": "mlstm", "mixer": {"heads": 2, "dim": 8, "vdim": 12, "gate_cap": 9.0},
                   "mlp": {"kind": "moe", "expert": {"ff": 16}, "router": {"experts": 3, "top": 1}}}]}


def edit(cfg, path, value=None, delete=False):
    broken = copy.deepcopy(cfg)
    at = broken
    for key in path[:-1]:
        at = at[key]
    if delete:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return broken


def test_config_is_read_key_by_key():
    c = RibozenConfig.from_dict(CFG)
    assert (c.vocab, c.width, c.norm_eps, c.embedding_scale) == (50, 32, 1e-5, 3.0)
    assert [layer.kind for layer in c.layers] == ["mamba2", "parallel", "mlstm"]
    left = c.layers[1].mixer.left
    assert (left.window, left.keep_first, left.softcap, left.rot_scaling.factor) == (6, 2, 20.0, 3.0)
    assert c.layers[1].feed_forward is None and c.layers[2].feed_forward.shared_ff == 0 and c.layers[0].feed_forward.shared_ff == 16
    required = [("vocab",), ("width",), ("norm",), ("embedding", "scale"), ("layers", 0, "mixer", "heads"),
                ("layers", 0, "mixer", "state"), ("layers", 0, "mixer", "groups"), ("layers", 0, "mixer", "conv"),
                ("layers", 0, "mixer", "norm_groups"), ("layers", 0, "mlp", "expert"), ("layers", 0, "mlp", "router", "top"),
                ("layers", 1, "mixer", "left_scale"), ("layers", 1, "mixer", "right"), ("layers", 1, "mixer", "left", "scale"),
                ("layers", 1, "mixer", "left", "kv_heads"), ("layers", 1, "mixer", "left", "rot", "base"),
                ("layers", 1, "mixer", "left", "rot", "scaling", "slow"), ("layers", 1, "mixer", "left", "mask", "size"),
                ("layers", 1, "mixer", "right", "dt_rank"), ("layers", 1, "mixer", "right", "inner"),
                ("layers", 2, "mixer", "gate_cap"), ("layers", 2, "mixer", "vdim")]
    for path in required:
        with pytest.raises(ConfigError, match=str(path[-1])):
            RibozenConfig.from_dict(edit(CFG, path, delete=True))
    for path, value in ((("layers", 0, "mixer", "groups"), 3), (("layers", 0, "mixer", "norm_groups"), 5),
                        (("layers", 1, "mixer", "left", "kv_heads"), 3), (("layers", 1, "mixer", "left", "rot", "dims"), 3),
                        (("layers", 1, "mixer", "left", "rot", "dims"), 10), (("layers", 0, "mlp", "router", "top"), 5),
                        (("layers", 0, "type"), "other"), (("layers", 0, "mlp", "kind"), "dense")):
        with pytest.raises(ConfigError):
            RibozenConfig.from_dict(edit(CFG, path, value))


def test_keys_that_may_be_absent():
    for path in (("layers", 1, "mixer", "left", "mask"), ("layers", 1, "mixer", "left", "mask", "keep_first"),
                 ("layers", 1, "mixer", "left", "softcap"), ("layers", 1, "mixer", "left", "rot", "scaling"),
                 ("layers", 0, "mlp", "shared"), ("embedding",)):
        c = RibozenConfig.from_dict(edit(CFG, path, delete=True))
        if path[-1] == "embedding":
            assert c.embedding_scale == 1.0
        left = c.layers[1].mixer.left
        if path[-1] == "mask":
            assert (left.window, left.keep_first) == (0, 0)
        if path[-1] == "keep_first":
            assert (left.window, left.keep_first) == (6, 0)
        if path[-1] == "softcap":
            assert left.softcap == 0.0
        if path[-1] == "scaling":
            assert left.rot_scaling is None
        if path[-1] == "shared":
            assert c.layers[0].feed_forward.shared_ff == 0


def test_what_the_cache_and_the_state_slots_hold():
    model = Model(spec_for(CFG))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == pr.tensor_shapes(CFG)
    assert len(model.groups) == 1
    g = model.groups[0]
    assert (g.num_kv_heads, g.head_dim, g.window, g.keep_first) == (2, 16, 6, 2)     # heads of 8 and 12 share pages of 16
    shapes = [tuple(s.shape) for s in model.states]
    # the duality layer's state and taps, the scan's state and taps (listed by the pair), the matrix memory
    assert shapes[:4] == [(32, 6), (2, 32 + 2 * 2 * 6), (24, 5), (1, 24)]
    heads, parts, rows, dim = shapes[4]
    assert (heads, dim) == (2, 8) and parts * (rows - 2) == 12
    assert [r.group for r in model.runs] == [None, 0, None]
    no_mask = Model(spec_for(edit(CFG, ("layers", 1, "mixer", "left", "mask"), delete=True)))
    assert (no_mask.groups[0].window, no_mask.groups[0].keep_first) == (None, 0)


def test_pages_of_kept_first_keys_are_never_given_back():
    host = build.load_host()
    manager = host.BlockSpaceManager([host.CacheGroupSpec(block_size=4, window=6, num_blocks=12, keep_first=5),
                                      host.CacheGroupSpec(block_size=4, window=6, num_blocks=12)], 2)
    seq = host.Sequence(0, list(range(40)), host.SamplingParams())
    assert manager.grow(seq, 40)
    seq.set_num_computed_tokens(40)
    manager.release_passed(seq)
    kept, plain = seq.get_block_tables()
    # the next query stands at 40 and reads keys 35 ..: pages 0 .. 7 are passed; the first two hold keys 0 .. 4
    assert [p >= 0 for p in kept] == [True, True] + [False] * 6 + [True, True]
    assert [p >= 0 for p in plain] == [False] * 8 + [True, True]
    assert manager.audit() == ""
    manager.free(seq)
    assert manager.get_num_free_blocks(0) == 12 and manager.get_num_free_blocks(1) == 12 and manager.audit() == ""


def test_ramped_rates():
    for dims, base, scaling in ((8, 1e4, None), (64, 5e4, {"factor": 6.0, "original": 1024, "fast": 16.0, "slow": 2.0}),
                                (6, 50.0, {"factor": 8.0, "original": 16, "fast": 4.0, "slow": 0.25})):
        rates, magnitude = ramped_rates(dims, base, scaling)
        want, want_magnitude = pr.scaled_rates(dims, base, scaling)
        torch.testing.assert_close(rates, want, rtol=1e-13, atol=0)
        assert abs(magnitude - want_magnitude) < 1e-13
        plain = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * torch.arange(dims // 2, dtype=torch.float64) / dims)
        if scaling is None:
            assert magnitude == 1.0 and torch.equal(rates, plain)
        else:
            assert magnitude == 0.1 * math.log(scaling["factor"]) + 1.0
            assert torch.all(rates <= plain) and torch.all(rates >= plain / scaling["factor"] * (1 - 1e-12))
            assert rates[0] == plain[0] or rates[-1] < plain[-1]


def test_the_plain_implementation_is_causal_and_its_pieces_agree():
    w = pr.random_weights(CFG, seed=3)
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, 50, (30,), generator=g).tolist()
    whole = pr.forward(CFG, w, ids)
    torch.testing.assert_close(pr.forward(CFG, w, ids[:17]), whole[:17], atol=1e-12, rtol=1e-12)
    other = list(ids)
    other[20] = (ids[20] + 1) % 50
    moved = (pr.forward(CFG, w, other) - whole).abs().amax(dim=-1)
    assert float(moved[:20].max()) == 0.0 and float(moved[20:].min()) > 0.0
    # a weight on an expert's input is a factor on both of its first products
    h = torch.randn(5, 32, generator=g, dtype=torch.float64)
    p, weight = "l0.mlp.e1.", 0.37
    direct = pr.expert(weight * h, w, p, None)
    a = pr.silu(weight * (h @ w[p + "gate"].T)) * (weight * (h @ w[p + "up"].T))
    torch.testing.assert_close(direct, a @ w[p + "down"].T, atol=1e-12, rtol=1e-12)
    assert pr.greedy(CFG, w, ids[:5], 3) == [int(pr.forward(CFG, w, ids[:5])[-1].argmax())] + pr.greedy(
        CFG, w, ids[:5] + [int(pr.forward(CFG, w, ids[:5])[-1].argmax())], 2)
