"""What of the Zepilix design needs no GPU: config.json key by key, the layers'
run order and what opens a pass, what the cache and the state slots must hold,
and the plain implementation's own pieces against each other."""
import copy

import pytest
import torch

import plain_zepilix as pz
from lyapunov_engine_b200.config.base import ConfigError
from lyapunov_engine_b200.config.zepilix import ZepilixConfig
from lyapunov_engine_b200.models.model import Model
from lyapunov_engine_b200.registry import spec_for

CFG = {"architecture": "Zepilix", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "token_side": {"dim": 4},
       "loop": {"start": 1, "stop": 3, "times": 3},
       "layers": [{"type": "attention",
                   "mixer": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 16, "scale": 0.3, "rot": {"dims": 8, "base": 100.0}},
                   "mlp": {"kind": "dense", "ff": 48}},
                  {"type": "delta", "mixer": {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 12, "conv": 3}, "mlp": None},
                  {"type": "latent_attention",
                   "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 12, "kv_rank": 20, "q_rank": 10, "scale": 0.3,
                             "rot": {"dims": 4, "base": 100.0}, "mask": {"size": 6}},
                   "mlp": {"kind": "dense", "ff": 24}},
                  {"type": "delta", "mixer": {"heads": 1, "kv_heads": 1, "dim": 16, "vdim": 16, "conv": 1},
                   "mlp": {"kind": "dense", "ff": 16}}]}


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
    c = ZepilixConfig.from_dict(CFG)
    assert (c.vocab, c.width, c.side_dim, c.loop) == (50, 32, 4, (1, 3, 3))
    assert c.passes() == pz.passes(CFG) == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert c.layers[1].ff == 0 and c.layers[2].mixer.window == 6 and c.layers[3].mixer.taps == 1
    for path in (("vocab",), ("width",), ("norm",), ("layers", 0, "mixer", "heads"), ("layers", 0, "mixer", "scale"),
                 ("layers", 0, "mixer", "rot"), ("layers", 0, "mixer", "rot", "base"), ("layers", 1, "mixer", "conv"),
                 ("layers", 1, "mixer", "vdim"), ("layers", 1, "mixer", "kv_heads"), ("layers", 2, "mixer", "kv_rank"),
                 ("layers", 2, "mixer", "q_rank"), ("layers", 2, "mixer", "rot_dim"), ("layers", 0, "mlp", "ff"),
                 ("loop", "times"), ("token_side", "dim")):
        with pytest.raises(ConfigError, match=str(path[-1])):
            ZepilixConfig.from_dict(edit(CFG, path, delete=True))
    for path, value in ((("layers", 0, "mixer", "kv_heads"), 3), (("layers", 0, "mixer", "rot", "dims"), 5),
                        (("layers", 0, "mixer", "rot", "dims"), 18), (("layers", 0, "mixer", "vdim"), 8),
                        (("layers", 2, "mixer", "rot", "dims"), 6), (("loop", "stop"), 5), (("loop", "stop"), 1),
                        (("layers", 0, "type"), "other"), (("layers", 0, "mlp", "kind"), "moe")):
        with pytest.raises(ConfigError):
            ZepilixConfig.from_dict(edit(CFG, path, value))


def test_keys_that_may_be_absent():
    cfg = copy.deepcopy(CFG)
    del cfg["loop"], cfg["token_side"], cfg["layers"][2]["mixer"]["mask"]
    c = ZepilixConfig.from_dict(cfg)
    assert c.loop is None and c.side_dim == 0 and c.layers[2].mixer.window == 0
    assert [i for i, _ in c.passes()] == [0, 1, 2, 3]
    model = Model(spec_for(cfg))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == pz.tensor_shapes(cfg)
    assert not any("side" in d.name or "loop" in d.name for d in model.tensors())
    assert all(e is None for e in model.entries)
    assert [g.window for g in model.groups] == [None, None]


def test_the_plan_has_pages_and_state_per_pass():
    model = Model(spec_for(CFG))
    assert {d.name: tuple(d.shape) for d in model.tensors()} == pz.tensor_shapes(CFG)
    assert [r.layer for r in model.runs] == pz.run_order(CFG) == [0, 1, 2, 1, 2, 1, 2, 3]
    # what opens a pass runs before the loop's first layer, once per pass; only later passes add the embedding again
    opened = [(i, e.row, e.embedding_name) for i, e in enumerate(model.entries) if e is not None]
    assert opened == [(1, 0, None), (3, 1, "embed"), (5, 2, "embed")]
    # grouped-query attention keeps keys and values (the values are the keys as projected: a pool of their own);
    # the latent layer keeps one pool of latent + rotated part, padded to 16, in a window; a pool (pair) per pass
    assert [(g.num_kv_heads, g.head_dim, g.window, g.values) for g in model.groups] == [(2, 16, None, True), (1, 32, 6, False)]
    assert model.streams_per_group == [1, 3]
    # the delta layers: a matrix of state per head (kept transposed) and the convolutions' last inputs, per pass;
    # one tap keeps no inputs
    shapes = [tuple(s.shape) for s in model.states]
    assert shapes == [(4, 12, 8), (2, 2 * 2 * 8 + 4 * 12)] * 3 + [(1, 16, 16)]
    assert [r.state is not None for r in model.runs] == [False, True, False, True, False, True, False, True]
    assert len({r.state for r in model.runs if r.state is not None}) == 4


def test_random_weights_follow_the_declarations(tmp_path):
    from lyapunov_engine_b200.weights.loader import write_random_model
    from lyapunov_engine_b200.weights import safetensors_io
    folder = write_random_model(str(tmp_path / "m"), CFG, seed=3)
    table = safetensors_io.open_folder(folder)
    assert {n: tuple(table[n].shape) for n in table} == pz.tensor_shapes(CFG)


def test_plain_pieces_agree_with_each_other():
    g = torch.Generator().manual_seed(0)
    f64 = torch.float64
    # a turn by an angle keeps each pair's length, position 0 turns nothing, entries from `rot` on pass
    v = torch.randn(7, 2, 10, generator=g, dtype=f64)
    r = pz.turn_pairs(v, torch.arange(7), 6, 100.0)
    assert torch.equal(r[0], v[0]) and torch.equal(r[..., 6:], v[..., 6:])
    torch.testing.assert_close(r[..., 0:6].reshape(7, 2, 3, 2).norm(dim=-1), v[..., 0:6].reshape(7, 2, 3, 2).norm(dim=-1))
    # scores of turned queries and keys depend on the distance only
    q, k = torch.randn(1, 1, 6, generator=g, dtype=f64), torch.randn(1, 1, 6, generator=g, dtype=f64)
    a = (pz.turn_pairs(q, torch.tensor([9]), 6, 50.0) * pz.turn_pairs(k, torch.tensor([4]), 6, 50.0)).sum()
    c = (pz.turn_pairs(q, torch.tensor([105]), 6, 50.0) * pz.turn_pairs(k, torch.tensor([100]), 6, 50.0)).sum()
    torch.testing.assert_close(a, c)
    # the delta rule with step size 1, no decay and orthonormal keys stores each value under its key and gives it
    # back; writing a key again replaces what it held
    keys = torch.eye(4, dtype=f64)[[0, 1, 2, 1]]
    vals = torch.randn(4, 3, generator=g, dtype=f64)
    out = pz.delta_rule_head(keys, keys, vals, torch.ones(4, dtype=f64), torch.ones(4, dtype=f64))
    torch.testing.assert_close(out, vals)
    probe = pz.delta_rule_head(torch.eye(4, dtype=f64)[[3, 3, 3, 1]], keys, vals, torch.ones(4, dtype=f64), torch.ones(4, dtype=f64))
    torch.testing.assert_close(probe[3], vals[3])
    assert float(probe[:3].abs().max()) == 0.0
    # with decay g the stored value fades by g per token
    faded = pz.delta_rule_head(torch.eye(4, dtype=f64)[[0, 0, 0, 0]], keys, vals, torch.full((4,), 0.5, dtype=f64),
                               torch.ones(4, dtype=f64))
    torch.testing.assert_close(faded[3], vals[0] * 0.125)
    # the convolution's last tap is the current token's; zeros before the start
    x = torch.randn(5, 2, generator=g, dtype=f64)
    taps = torch.tensor([[0.0, 0.0, 1.0], [1.0, 0.0, 0.0]], dtype=f64)
    y = pz.conv_silu(x, taps)
    torch.testing.assert_close(y[:, 0], pz.silu(x[:, 0]))
    torch.testing.assert_close(y[2:, 1], pz.silu(x[:3, 1]))
    assert float(y[:2, 1].abs().max()) == 0.0
    # whole sequences against prefixes: position t depends on tokens up to t only
    w = pz.random_weights(CFG, seed=1)
    ids = list(range(3, 20))
    full = pz.forward(CFG, w, ids)
    torch.testing.assert_close(pz.forward(CFG, w, ids[:9]), full[:9])
    assert len(pz.greedy(CFG, w, [1, 2, 3], 3)) == 3
