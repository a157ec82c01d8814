"""Gated feed-forward: down(act(gate(x), up(x))).

"gated_silu" (SwiGLU): act(g, u) = silu(g) * u.  "gated_relu": act(g, u) =
max(g, 0) * u.  "gated_clamped": with a limit
L and a slope a, g' = min(g, L), u' = clamp(u, -L, L), act = g' * sigmoid(a g')
* (u' + 1).

Gate and up are one projection [2 I, H], gate rows first, as the reference
fuses them at load (python/lyapunov_engine/models/weight_loader.py:155-163;
python/lyapunov_engine/models/llama.py:109-122).  The activation is computed in
32 bits and rounded once (csrc/kernels/fused_rmsnorm_swiglu.cu:170-176).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FeedForward, TensorDecl, register_feed_forward


@register_feed_forward("gated_silu")
class GatedFeedForward(FeedForward):
    activation = (ops.GLU_SILU, 1.0, 0.0)      # (kind, slope, limit) as the kernels take them

    def __init__(self, hidden_size: int, intermediate_size: int, gate_name: str, up_name: str, down_name: str,
                 bias_suffix: str | None = None):
        """``bias_suffix`` s: each of the three projections has a bias, stored
        as <its name>s.  Gate's and up's are added before the activation (in
        32 bits); the output's is left to whoever adds the result to the
        residual stream (``output_bias``), or added here where nobody does
        (``forward_plain``)."""
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.names = (gate_name, up_name, down_name)
        self.bias_suffix = bias_suffix
        self.w_gate_up = self.w_down = self.gate_up_bias = self.output_bias = None
        self.runtime = None

    def tensors(self):
        g, u, d = self.names
        H, I = self.hidden_size, self.intermediate_size
        decls = [TensorDecl(g, (I, H)), TensorDecl(u, (I, H)), TensorDecl(d, (H, I))]
        if self.bias_suffix:
            s = self.bias_suffix
            decls += [TensorDecl(g + s, (I,), role="vector", init="taps"), TensorDecl(u + s, (I,), role="vector", init="taps"),
                      TensorDecl(d + s, (H,), role="vector", init="taps")]
        return decls

    def bind(self, get, runtime):
        g, u, d = self.names
        self.w_gate_up = torch.cat([get(g), get(u)], dim=0).contiguous()
        self.w_down = get(d)
        if self.bias_suffix:
            s = self.bias_suffix
            self.gate_up_bias = torch.cat([get(g + s), get(u + s)]).contiguous()
            self.output_bias = get(d + s).contiguous()
        self.runtime = runtime

    def _activated(self, x, ctx, key):
        ws = ctx.workspace
        act = ws.get(key, (x.shape[0], self.intermediate_size), self.runtime.dtype)
        if self.gate_up_bias is None:
            ops.gated_linear(act, x, self.w_gate_up, ws, ctx.status, self.activation)
        else:
            ops.gated_linear_bias(act, x, self.w_gate_up, self.gate_up_bias, ws, ctx.status, self.activation)
        return act

    def forward(self, x, ctx):
        """The output without its bias (see ``output_bias``)."""
        act = self._activated(x, ctx, "ffn_act")
        return ops.linear_for_residual(act, self.w_down, ctx.workspace, "ffn_out", ctx.status)

    def forward_plain(self, x, ctx, key: str = "ffn_plain"):
        """The same as one tensor [T, H] in the activations' type (``forward``
        may return partial sums for the norm to add), for a caller that goes
        on computing with it; buffers of its own, so that it can run inside
        another feed-forward."""
        rt = self.runtime
        ws = ctx.workspace
        act = self._activated(x, ctx, key + "_act")
        out = ws.get(key, (x.shape[0], self.hidden_size), rt.dtype)
        ops.linear(out, act, self.w_down, ctx.status)
        if self.output_bias is not None:
            raise NotImplementedError("a feed-forward with an output bias is added to the residual stream by its block")
        return out


@register_feed_forward("gated_relu")
class ReluGatedFeedForward(GatedFeedForward):
    activation = (ops.GLU_RELU, 1.0, 0.0)


@register_feed_forward("gated_clamped")
class ClampedGatedFeedForward(GatedFeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, gate_name: str, up_name: str, down_name: str,
                 limit: float, slope: float = 1.702, bias_suffix: str | None = None):
        super().__init__(hidden_size, intermediate_size, gate_name, up_name, down_name, bias_suffix)
        if not limit > 0:
            raise ValueError(f"the clamped activation needs a positive limit, got {limit}")
        self.activation = (ops.GLU_CLAMPED, float(slope), float(limit))
