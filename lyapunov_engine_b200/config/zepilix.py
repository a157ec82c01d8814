"""ZepilixConfig: the keys of a Zepilix checkpoint's config.json, typed.

    {"architecture": "Zepilix", "vocab": V, "width": W, "norm": {"eps": ..},
     "token_side": {"dim": s}, "loop": {"start": a, "stop": b, "times": n},
     "layers": [{"type": "delta",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "conv"}, "mlp": ..},
                {"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "rot": {"dims", "base"}}, "mlp": ..},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
                           "rot": {"dims", "base"}, "mask": {"size"}}, "mlp": ..}, ...]}
    "mlp": {"kind": "dense", "ff": ..} | null

Every size and constant a layer uses is read from its own entry; nothing has a
default.  Keys that may be absent, and what their absence means: ``loop``
(every layer runs once), ``token_side`` (no input per token and layer), a
latent mixer's ``mask`` (every earlier key is visible), ``mlp`` null (a layer
without feed-forward).
"""
from __future__ import annotations

from dataclasses import dataclass

from .base import ConfigError, KeyReader


@dataclass(frozen=True)
class ZepilixMixer:
    kind: str              # "delta", "attention" or "latent_attention"
    heads: int
    kv_heads: int          # (latent attention: every head has keys of its own)
    dim: int
    vdim: int
    taps: int = 0          # delta
    scale: float = 0.0     # the attentions
    rot_dims: int = 0
    rot_base: float = 1.0
    rot_dim: int = 0       # latent attention: the rotated part of queries and keys
    kv_rank: int = 0
    q_rank: int = 0
    window: int = 0        # 0: every earlier key


@dataclass(frozen=True)
class ZepilixLayer:
    mixer: ZepilixMixer
    ff: int                # 0: no feed-forward


@dataclass(frozen=True)
class ZepilixConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    side_dim: int                      # 0: no input per token and layer
    loop: tuple[int, int, int] | None  # (start, stop, times)
    layers: tuple[ZepilixLayer, ...]
    raw: dict

    def passes(self) -> list[tuple[int, int | None]]:
        """The run order as (layer, number of the pass that this run opens or None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        order = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    @staticmethod
    def from_dict(raw: dict, source: str = "config.json") -> "ZepilixConfig":
        r = KeyReader(raw, source)
        width = r.integer("width")
        norm = KeyReader(r.mapping("norm"), source + ": norm")
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

            def rotary():
                rr = KeyReader(m.mapping("rot"), where + ".mixer.rot")
                return rr.integer("dims", minimum=0), rr.number("base")

            if kind == "delta":
                mixer = ZepilixMixer(kind, heads=m.integer("heads"), kv_heads=m.integer("kv_heads"), dim=m.integer("dim"),
                                     vdim=m.integer("vdim"), taps=m.integer("conv"))
            elif kind == "attention":
                dims, base = rotary()
                mixer = ZepilixMixer(kind, heads=m.integer("heads"), kv_heads=m.integer("kv_heads"), dim=m.integer("dim"),
                                     vdim=m.integer("vdim"), scale=m.number("scale"), rot_dims=dims, rot_base=base)
                if mixer.vdim != mixer.dim:
                    raise ConfigError(f"{where}.mixer: the values are the keys, so 'vdim' must equal 'dim'")
                if dims % 2 or dims > mixer.dim:
                    raise ConfigError(f"{where}.mixer.rot: dims {dims} must be even and at most dim {mixer.dim}")
            elif kind == "latent_attention":
                dims, base = rotary()
                mask = m.mapping("mask", None)
                window = KeyReader(mask, where + ".mixer.mask").integer("size") if mask is not None else 0
                heads = m.integer("heads")
                mixer = ZepilixMixer(kind, heads=heads, kv_heads=heads, dim=m.integer("dim"), vdim=m.integer("vdim"),
                                     scale=m.number("scale"), rot_dims=dims, rot_base=base,
                                     rot_dim=m.integer("rot_dim", minimum=0), kv_rank=m.integer("kv_rank"),
                                     q_rank=m.integer("q_rank"), window=window)
                if dims != mixer.rot_dim:
                    raise ConfigError(f"{where}.mixer: rot.dims {dims} must equal rot_dim {mixer.rot_dim}")
                if mixer.rot_dim % 2 or mixer.kv_rank % 2:
                    raise ConfigError(f"{where}.mixer: rot_dim and kv_rank must be even")
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (known: 'delta', 'attention', 'latent_attention')")
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"{where}.mixer: {mixer.heads} heads do not divide into {mixer.kv_heads} kv_heads")
            ff = 0
            if entry.get("mlp") is not None:
                f = KeyReader(e.mapping("mlp"), where + ".mlp")
                ff_kind = f.string("kind")
                if ff_kind != "dense":
                    raise ConfigError(f"{where}.mlp: unknown kind {ff_kind!r} (known: 'dense')")
                ff = f.integer("ff")
            layers.append(ZepilixLayer(mixer, ff))
        loop = None
        raw_loop = r.mapping("loop", None)
        if raw_loop is not None:
            lp = KeyReader(raw_loop, source + ": loop")
            loop = (lp.integer("start", minimum=0), lp.integer("stop", minimum=0), lp.integer("times", minimum=1))
            if not loop[0] < loop[1] <= len(layers):
                raise ConfigError(f"{source}: loop {loop[0]}..{loop[1]} does not lie within the {len(layers)} layers")
        side = r.mapping("token_side", None)
        side_dim = KeyReader(side, source + ": token_side").integer("dim") if side is not None else 0
        return ZepilixConfig(architecture=r.string("architecture"), vocab=r.integer("vocab"), width=width,
                             norm_eps=norm.number("eps"), side_dim=side_dim, loop=loop, layers=tuple(layers), raw=dict(raw))
