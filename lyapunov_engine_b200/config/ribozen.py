"""RibozenConfig: the keys of a Ribozen checkpoint's config.json, typed.

    {"architecture": "Ribozen", "vocab": V, "width": W, "norm": {"eps": ..}, "embedding": {"scale": ..},
     "layers": [{"type": "mlstm",
                 "mixer": {"heads", "dim", "vdim", "gate_cap"}, "mlp": ..},
                {"type": "mamba2",
                 "mixer": {"heads", "vdim", "state", "groups", "conv", "norm_groups"}, "mlp": ..},
                {"type": "parallel",
                 "mixer": {"left_scale", "right_scale",
                           "left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                    "rot": {"dims", "base", "scaling": {"factor", "original", "fast", "slow"}},
                                    "mask": {"size", "keep_first"}},
                           "right": {"inner", "state", "dt_rank", "conv"}}, "mlp": ..}, ...]}
    "mlp": {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top"}, "shared": {"ff"}} | null

Every size and constant a layer uses is read from its own entry; nothing has a
default.  Keys that may be absent, and what their absence means: ``embedding``
(the embedding is not scaled), ``mlp`` null (a layer without feed-forward),
``shared`` (no shared expert), an attention's ``mask`` (every earlier key is
visible; ``keep_first`` absent: the window keeps no first keys), ``softcap``
(scores are not capped), ``rot.scaling`` (plain rotary rates).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class MatrixMemory:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class StateSpaceDuality:
    heads: int
    vdim: int
    state: int
    groups: int
    taps: int
    norm_groups: int


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class WindowedAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float           # 0: none
    rot_dims: int
    rot_base: float
    rot_scaling: RotaryScaling | None
    window: int              # 0: every earlier key
    keep_first: int


@dataclass(frozen=True)
class SelectiveScan:
    inner: int
    state: int
    dt_rank: int
    taps: int


@dataclass(frozen=True)
class SideBySide:
    left: WindowedAttention
    right: SelectiveScan
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class RoutedFeedForward:
    ff: int
    experts: int
    top: int
    shared_ff: int           # 0: no shared expert


@dataclass(frozen=True)
class RibozenLayer:
    kind: str                # "mlstm", "mamba2" or "parallel"
    mixer: object
    feed_forward: RoutedFeedForward | None


@dataclass(frozen=True)
class RibozenConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float
    layers: tuple[RibozenLayer, ...]
    raw: dict

    @staticmethod
    def from_dict(raw: dict, source: str = "config.json") -> "RibozenConfig":
        r = KeyReader(raw, source)
        width = r.integer("width")
        norm = KeyReader(r.mapping("norm"), source + ": norm")
        raw_embedding = r.mapping("embedding", None)
        embedding = KeyReader(raw_embedding, source + ": embedding") if raw_embedding is not None else None
        entries = raw.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{source}: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"{source}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            e = KeyReader(entry, where)
            kind = e.string("type")
            m = KeyReader(e.mapping("mixer"), where + ".mixer")
            if kind == "mlstm":
                mixer = MatrixMemory(heads=m.integer("heads"), dim=m.integer("dim"), vdim=m.integer("vdim"),
                                     gate_cap=m.number("gate_cap"))
            elif kind == "mamba2":
                mixer = StateSpaceDuality(heads=m.integer("heads"), vdim=m.integer("vdim"), state=m.integer("state"),
                                          groups=m.integer("groups"), taps=m.integer("conv"),
                                          norm_groups=m.integer("norm_groups"))
                if mixer.heads % mixer.groups:
                    raise ConfigError(f"{where}.mixer: {mixer.heads} heads do not divide into {mixer.groups} groups")
                if (mixer.heads * mixer.vdim) % mixer.norm_groups:
                    raise ConfigError(f"{where}.mixer: {mixer.heads * mixer.vdim} channels do not divide into "
                                      f"{mixer.norm_groups} norm_groups")
            elif kind == "parallel":
                mixer = SideBySide(left=_attention(KeyReader(m.mapping("left"), where + ".mixer.left")),
                                   right=_selective_scan(KeyReader(m.mapping("right"), where + ".mixer.right")),
                                   left_scale=m.number("left_scale", positive=False),
                                   right_scale=m.number("right_scale", positive=False))
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'mlstm', 'mamba2', 'parallel')")
            feed_forward = None
            if entry.get("mlp") is not None:
                f = KeyReader(e.mapping("mlp"), where + ".mlp")
                ff_kind = f.string("kind")
                if ff_kind != "moe":
                    raise ConfigError(f"{where}.mlp: unknown kind {ff_kind!r} (known: 'moe')")
                expert = KeyReader(f.mapping("expert"), where + ".mlp.expert")
                router = KeyReader(f.mapping("router"), where + ".mlp.router")
                shared = f.mapping("shared", None)
                feed_forward = RoutedFeedForward(
                    ff=expert.integer("ff"), experts=router.integer("experts"), top=router.integer("top"),
                    shared_ff=KeyReader(shared, where + ".mlp.shared").integer("ff") if shared is not None else 0)
                if feed_forward.top > feed_forward.experts:
                    raise ConfigError(f"{where}.mlp.router: a token cannot use {feed_forward.top} of "
                                      f"{feed_forward.experts} experts")
            layers.append(RibozenLayer(kind, mixer, feed_forward))
        return RibozenConfig(architecture=r.string("architecture"), vocab=r.integer("vocab"), width=width,
                             norm_eps=norm.number("eps"),
                             embedding_scale=embedding.number("scale", positive=False) if embedding is not None else 1.0,
                             layers=tuple(layers), raw=dict(raw))


def _attention(m: KeyReader) -> WindowedAttention:
    heads, kv_heads = m.integer("heads"), m.integer("kv_heads")
    if heads % kv_heads:
        raise ConfigError(f"{m.source}: {heads} heads do not divide into {kv_heads} kv_heads")
    rot = KeyReader(m.mapping("rot"), m.source + ".rot")
    dims = rot.integer("dims", minimum=0)
    dim = m.integer("dim")
    if dims % 2 or dims > dim:
        raise ConfigError(f"{m.source}.rot: dims {dims} must be even and at most dim {dim}")
    scaling = None
    raw_scaling = rot.mapping("scaling", None)
    if raw_scaling is not None:
        s = KeyReader(raw_scaling, m.source + ".rot.scaling")
        scaling = RotaryScaling(factor=s.number("factor"), original=s.number("original"), fast=s.number("fast"),
                                slow=s.number("slow"))
    window = keep_first = 0
    mask = m.mapping("mask", None)
    if mask is not None:
        k = KeyReader(mask, m.source + ".mask")
        window = k.integer("size")
        keep_first = k.integer("keep_first", 0, minimum=0)
    return WindowedAttention(heads=heads, kv_heads=kv_heads, dim=dim, vdim=m.integer("vdim"), scale=m.number("scale"),
                             softcap=m.number("softcap", 0.0, positive=False), rot_dims=dims,
                             rot_base=rot.number("base") if dims else 1.0, rot_scaling=scaling, window=window,
                             keep_first=keep_first)


def _selective_scan(m: KeyReader) -> SelectiveScan:
    return SelectiveScan(inner=m.integer("inner"), state=m.integer("state"), dt_rank=m.integer("dt_rank"),
                         taps=m.integer("conv"))
