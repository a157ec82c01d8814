"""The mLSTM's matrix memory: a mixer whose memory is a matrix per head with
exponential gates kept in range by a running maximum.

With x the mixer's input, H heads, d the query/key size and e the value size:

    q = Wq x * d^-1/2,  k = Wk x   [H, d]        v = Wv x   [H, e]
    i = cap tanh((Wi x + b_i) / cap)             f = logsigmoid(cap tanh((Wf x + b_f) / cap))     per head
    m' = max(f + m, i)                           (m starts at 0)
    S <- e^(f + m - m') S + e^(i - m') k v^T     n <- e^(f + m - m') n + e^(i - m') k
    o = S^T q / (max(|n . q|, e^(-m')) + 1e-6)
    y = Wo concat_h( o_h / sqrt(mean(o_h^2) + eps) * w_h * sigmoid(Wg x)_h )

S, n and m are carried from token to token in 32 bits, per request and head
(``state_need``).  One product makes all six projections; the recurrence and
the gated norm are a kernel each (ops.mlstm_scan, ops.head_norm_gate).  The
gates, the recurrence and the norm are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_mixer


@register_mixer("matrix_memory")
class MatrixMemoryMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, gate_cap: float, norm_eps: float,
                 q_name: str, k_name: str, v_name: str, gate_name: str, input_gate_name: str, forget_gate_name: str,
                 norm_name: str, o_name: str, bias_suffix: str = ".b"):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.value_dim = int(head_dim), int(value_dim)
        self.gate_cap, self.norm_eps = float(gate_cap), float(norm_eps)
        if not self.gate_cap > 0:
            raise ValueError(f"the gates' cap must be positive, got {gate_cap}")
        if not 1 <= self.head_dim <= 512:
            raise ValueError(f"the matrix memory takes heads of up to 512 entries, got {head_dim}")
        self.names = (q_name, k_name, v_name, gate_name, input_gate_name, forget_gate_name)
        self.norm_name, self.o_name, self.bias_suffix = norm_name, o_name, bias_suffix
        H, d, e = self.num_heads, self.head_dim, self.value_dim
        self.q_col, self.k_col, self.v_col = 0, H * d, 2 * H * d
        self.gate_col = 2 * H * d + H * e
        self.i_col = self.gate_col + H * e
        self.f_col = self.i_col + H
        self.width = (self.f_col + H + 7) // 8 * 8
        self.runtime = None

    def state_need(self):
        return StateNeed(ops.mlstm_state_shape(self.num_heads, self.head_dim, self.value_dim), torch.float32)

    def tensors(self):
        q, k, v, g, i, f = self.names
        W, H, d, e = self.hidden_size, self.num_heads, self.head_dim, self.value_dim
        return [TensorDecl(q, (H * d, W)), TensorDecl(k, (H * d, W)), TensorDecl(v, (H * e, W)), TensorDecl(g, (H * e, W)),
                TensorDecl(i, (H, W)), TensorDecl(f, (H, W)),
                TensorDecl(i + self.bias_suffix, (H,), role="vector", init="zeros"),
                TensorDecl(f + self.bias_suffix, (H,), role="vector", init="ones_jitter"),
                TensorDecl(self.norm_name, (H * e,), role="vector", init="ones_jitter"),
                TensorDecl(self.o_name, (W, H * e))]

    def bind(self, get, runtime):
        rows = [get(n) for n in self.names]
        pad = self.width - sum(r.shape[0] for r in rows)
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.i_bias = get(self.names[4] + self.bias_suffix).contiguous()
        self.f_bias = get(self.names[5] + self.bias_suffix).contiguous()
        self.norm_weight = get(self.norm_name).contiguous()
        self.w_o = get(self.o_name)
        self.runtime = runtime

    def inner_width(self) -> int:
        return self.num_heads * self.value_dim

    def output_weight(self):
        return self.w_o

    def forward(self, x, ctx, cache):
        return ops.linear_for_residual(self.forward_inner(x, ctx, cache), self.w_o, ctx.workspace, "mixer_out", ctx.status)

    def forward_inner(self, x, ctx, cache, out=None, scale: float = 1.0):
        """The normed, gated heads before the output projection [T, H * e],
        into ``out`` where given, times ``scale``."""
        rt, ws = self.runtime, ctx.workspace
        H, d, e = self.num_heads, self.head_dim, self.value_dim
        T = x.shape[0]
        proj = ws.get("mlstm_proj", (T, self.width), rt.dtype)
        ops.linear(proj, x, self.w_in, ctx.status)
        o = ws.get("mlstm_out", (T, H * e), torch.float32)
        ops.mlstm_scan(o, proj, self.q_col, self.k_col, self.v_col, self.i_col, self.f_col, self.i_bias, self.f_bias,
                       cache.state, ctx.state_slots, ctx.cu_q, ctx.num_requests, H, d, e, self.gate_cap, d ** -0.5)
        if out is None:
            out = ws.get("mlstm_gated", (T, H * e), rt.dtype)
        ops.head_norm_gate(out, o, proj[:, self.gate_col:self.gate_col + H * e], self.norm_weight, self.norm_eps, H, e,
                           sigmoid=True, out_scale=scale)
        return out
