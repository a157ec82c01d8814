"""Block arrangements: how norms, mixer and feed-forward sit around the
residual stream.

"prenorm" is the reference's decoder layer
(python/lyapunov_engine/models/llama.py:136-165):
    h = h + mixer(norm1(h));  h = h + feed_forward(norm2(h))
The additions happen inside the following norm's kernel, in 32 bits: a block
leaves its feed-forward output ``pending`` and the next norm (of the next
block, or the final one) adds it.  Two options: ``mixer_input``, an input
filter between the first norm and the mixer (h = filter(norm1(h)) is what the
mixer reads), and a block without a feed-forward (``feed_forward`` None: only
the first line above).  With layer scales (``mixer_scale_name``,
``feed_forward_scale_name``: a learned factor per column, 32-bit) a
sub-layer's output enters the stream times its factor, h = h + s1 *
mixer(norm1(h)); h = h + s2 * feed_forward(norm2(h)); the norm's kernel that
adds the output multiplies it.

"parallel": both sub-layers read the same stream (see ``ParallelBlock``).
"""
from __future__ import annotations

from .. import ops
from .base import (BLOCKS, FEED_FORWARDS, INPUT_FILTERS, MIXERS, NORMS, STREAM_INPUTS, Block, PartSpec, ScaledAddend,
                   TensorDecl, register_block)


@register_block("prenorm")
class PreNormBlock(Block):
    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec | None, mixer_input: PartSpec | None = None,
                 mixer_scale_name: str | None = None, feed_forward_scale_name: str | None = None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward_norm = NORMS.build(feed_forward_norm) if feed_forward_norm is not None else None
        self.mixer_input = INPUT_FILTERS.build(mixer_input) if mixer_input is not None else None
        self.mixer_scale_name = mixer_scale_name
        self.feed_forward_scale_name = feed_forward_scale_name if feed_forward is not None else None
        self.mixer_scale = self.feed_forward_scale = None
        if (mixer_scale_name or self.feed_forward_scale_name) and mixer_input is not None:
            raise ValueError("layer scales beside an input filter are not supported")

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer_input, self.mixer, self.feed_forward_norm, self.feed_forward)
                if p is not None]

    def extra_state_needs(self):
        needs = dict(self.mixer.extra_state_needs())
        need = self.mixer_input.state_need() if self.mixer_input is not None else None
        if need is not None:
            needs["mixer_input"] = need
        return needs

    def tile_sizes(self):
        return list(self.mixer.tile_sizes()) + (self.mixer_input.tile_sizes() if self.mixer_input is not None else [])

    def tensors(self):
        width = getattr(self.mixer_norm, "hidden_size", None)
        scales = [TensorDecl(name, (width,), role="vector", init="ones_jitter")
                  for name in (self.mixer_scale_name, self.feed_forward_scale_name) if name]
        return [d for p in self.parts() for d in p.tensors()] + scales

    def bind(self, get, runtime):
        for p in self.parts():
            p.bind(get, runtime)
        self.mixer_scale = get(self.mixer_scale_name).contiguous() if self.mixer_scale_name else None
        self.feed_forward_scale = get(self.feed_forward_scale_name).contiguous() if self.feed_forward_scale_name else None

    def _leave(self, stream, output, scale) -> None:
        stream.pending = output
        stream.update = ScaledAddend(scale) if scale is not None else None

    def forward(self, stream, ctx, cache) -> None:
        if self.mixer_scale is not None or self.feed_forward_scale is not None or isinstance(stream.update, ScaledAddend):
            # (a pending output with a factor per column: the norms' kernels multiply as they add)
            n = self.mixer_norm.apply_stream(stream, workspace=ctx.workspace)
            a = self.mixer.forward(n, ctx, cache)
            if self.feed_forward is None:
                self._leave(stream, a, self.mixer_scale)
                return
            n = self.feed_forward_norm.apply(stream.resid, a, workspace=ctx.workspace, delta_scale=self.mixer_scale)
            self._leave(stream, self.feed_forward.forward(n, ctx), self.feed_forward_scale)
            return
        n = None
        if self.mixer_input is not None:
            # an input filter may know how to run the norm before it in its own kernel
            state = (cache.extra or {}).get("mixer_input")
            fused = getattr(self.mixer_input, "after_norm", None)
            if fused is not None:
                n = fused(self.mixer_norm, stream.resid, stream.pending, ctx, state)
            if n is None:
                n = self.mixer_input.forward(self.mixer_norm.apply(stream.resid, stream.pending, workspace=ctx.workspace),
                                             ctx, state)
        else:
            n = self.mixer_norm.apply(stream.resid, stream.pending, workspace=ctx.workspace)
        a = self.mixer.forward(n, ctx, cache)
        if self.feed_forward is None:
            stream.pending = a
            return
        n = self.feed_forward_norm.apply(stream.resid, a, workspace=ctx.workspace)
        stream.pending = self.feed_forward.forward(n, ctx)


@register_block("parallel")
class ParallelBlock(Block):
    """The mixer and the feed-forward read the same stream, each through a
    norm of its own, and their outputs enter together:
        h = h + (mixer(norm1(h)) + feed_forward(norm2(h)))
    (one kernel makes both norms; one adds both outputs, and the feed-forward's
    output bias, in 32 bits).  ``after``: a stream input that runs on the new
    h, after the sub-layers (an embedding per token behind a gate, say); what
    it leaves pending enters in the next norm's kernel."""

    def __init__(self, mixer: PartSpec, feed_forward: PartSpec | None, mixer_norm: PartSpec,
                 feed_forward_norm: PartSpec | None, after: PartSpec | None = None):
        if (feed_forward is None) != (feed_forward_norm is None):
            raise ValueError("a block has a feed-forward and its norm, or neither")
        self.mixer = MIXERS.build(mixer)
        self.feed_forward = FEED_FORWARDS.build(feed_forward) if feed_forward is not None else None
        self.mixer_norm = NORMS.build(mixer_norm)
        self.feed_forward_norm = NORMS.build(feed_forward_norm) if feed_forward_norm is not None else None
        self.after = STREAM_INPUTS.build(after) if after is not None else None
        if not hasattr(self.mixer_norm, "apply_pair"):
            raise ValueError("the parallel arrangement needs norms that run as a pair (rmsnorm)")

    def parts(self):
        return [p for p in (self.mixer_norm, self.mixer, self.feed_forward_norm, self.feed_forward, self.after)
                if p is not None]

    def tensors(self):
        return [d for p in self.parts() for d in p.tensors()]

    def bind(self, get, runtime):
        self.runtime = runtime
        for p in self.parts():
            p.bind(get, runtime)

    def forward(self, stream, ctx, cache) -> None:
        n1, n2 = self.mixer_norm.apply_pair(stream, self.feed_forward_norm, workspace=ctx.workspace)
        a = self.mixer.forward(n1, ctx, cache)
        f = bias = None
        if self.feed_forward is not None:
            f = self.feed_forward.forward(n2, ctx)
            bias = getattr(self.feed_forward, "output_bias", None)     # (a bias the feed-forward leaves to the addition)
        copy = None
        if self.after is not None and getattr(self.after, "reads_stream", False):
            copy = ctx.workspace.get("stream_copy", tuple(stream.resid.shape), self.runtime.dtype)
        ops.residual_add(stream.resid, a, f, bias, copy)
        if self.after is not None:
            self.after.forward(stream, ctx, copy)
