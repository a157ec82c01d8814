"""Mixers side by side: several mixers read the same input and their outputs
are added, each times a constant:

    y = sum_j scale_j * mixer_j(x)

Every mixer ends in an output projection, so the sum is one product: the
mixers leave what their projections would read side by side in one buffer,
each times its constant (taken in 32 bits, in the kernel that writes those
numbers), and the projections' matrices stand side by side too, y = [a_0 | a_1
| ...] [W_0 | W_1 | ...]^T.  Pages belong to at most one of the mixers; every
mixer's state buffers are the block's, under names of their own.
"""
from __future__ import annotations

import torch

from .. import ops
from ..cache.storage import CacheBinding
from .base import MIXERS, Mixer, PartSpec, register_mixer


@register_mixer("side_by_side")
class SideBySideMixer(Mixer):
    def __init__(self, hidden_size: int, mixers: tuple, scales: tuple):
        if len(mixers) != len(scales) or not mixers:
            raise ValueError("mixers side by side: as many constants as mixers, at least one")
        self.hidden_size = int(hidden_size)
        self.mixers = [MIXERS.build(m) if isinstance(m, PartSpec) else m for m in mixers]
        self.scales = [float(s) for s in scales]
        for m in self.mixers:
            if not all(hasattr(m, a) for a in ("forward_inner", "inner_width", "output_weight")):
                raise ValueError(f"{type(m).__name__} cannot stand side by side: it does not hand on what its output projection reads")
        if sum(m.cache_need() is not None for m in self.mixers) > 1:
            raise ValueError("of mixers side by side at most one keeps pages")
        # columns of the shared buffer, each mixer's start a 16-byte multiple
        self.cols, at = [], 0
        for m in self.mixers:
            self.cols.append(at)
            at += (m.inner_width() + 7) // 8 * 8
        self.width = at
        self.w_o = None
        self.runtime = None

    def cache_need(self):
        for m in self.mixers:
            if m.cache_need() is not None:
                return m.cache_need()
        return None

    def state_need(self):
        return None         # (every mixer's buffers are listed by name below)

    def extra_state_needs(self):
        needs = {}
        for j, m in enumerate(self.mixers):
            if m.state_need() is not None:
                needs[f"side{j}.state"] = m.state_need()
            for name, need in m.extra_state_needs().items():
                needs[f"side{j}.{name}"] = need
        return needs

    def tile_sizes(self):
        return [t for m in self.mixers for t in m.tile_sizes()]

    def decode_variant(self, fill, num_decode, context_bound):
        found = tuple(m.decode_variant(fill, num_decode, context_bound) for m in self.mixers)
        return found if any(v is not None for v in found) else None

    def tensors(self):
        return [d for m in self.mixers for d in m.tensors()]

    def bind(self, get, runtime):
        for m in self.mixers:
            m.bind(get, runtime)
        first = self.mixers[0].output_weight()
        self.w_o = torch.zeros((self.hidden_size, self.width), dtype=first.dtype, device=first.device)
        for m, col in zip(self.mixers, self.cols):
            w = m.output_weight()
            self.w_o[:, col:col + w.shape[1]] = w
        self.runtime = runtime

    def forward(self, x, ctx, cache):
        ws = ctx.workspace
        T = x.shape[0]
        side = ws.get("side_by_side", (T, self.width), self.runtime.dtype)
        extra = cache.extra or {}
        for j, (m, col, scale) in enumerate(zip(self.mixers, self.cols, self.scales)):
            prefix = f"side{j}."
            own = {name[len(prefix):]: buf for name, buf in extra.items() if name.startswith(prefix)}
            binding = CacheBinding(cache.kv if m.cache_need() is not None else None, cache.write, own.pop("state", None), own)
            width = m.inner_width()
            end = self.cols[j + 1] if j + 1 < len(self.mixers) else self.width
            if end > col + width:           # (columns that only pad a mixer's share meet zero columns of W: keep them finite)
                side[:, col + width:end].zero_()
            m.forward_inner(x, ctx, binding, out=side[:, col:col + width], scale=scale)
        return ops.linear_for_residual(side, self.w_o, ws, "mixer_out", ctx.status)
