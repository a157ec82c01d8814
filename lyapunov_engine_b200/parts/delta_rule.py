"""The gated delta rule: a mixer whose memory is a matrix of state per head
instead of a cache of keys.

With x the mixer's input, H heads, G key groups (head h uses group h // (H /
G)), d the query/key size and e the value size:

    q, k = conv(Wq x), conv(Wk x)   [G, d]      v = conv(Wv x)   [H, e]
    conv: a causal convolution over time per channel (``taps`` taps, the last
          one the current token's, zeros before the request's start), then silu
    q, k <- q / sqrt(sum q^2 + 1e-6) * d^-1/2,   k / sqrt(sum k^2 + 1e-6)     per group
    beta = sigmoid(Wb x)   [H]        g = exp(-exp(A_log) * softplus(Wa x + dt_bias))   [H]
    per head:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    y = Wo concat_h( o_h / sqrt(mean(o_h^2) + eps) * w * silu(Wg x)_h )

S [d, e] starts at zero and is carried from token to token in 32 bits, one
matrix per request and head (``state_need``); the convolutions' last taps - 1
inputs are state of the request too (``extra_state_needs``).  One product makes
all six projections; the convolution, the recurrence and the gated norm are a
kernel each (ops.short_conv_general, ops.gated_delta_scan, ops.head_norm_gate).
Unit vectors, decays, step sizes, the recurrence and the norm are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_mixer

UNIT_EPS = 1e-6


@register_mixer("gated_delta")
class GatedDeltaMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, value_dim: int, taps: int,
                 norm_eps: float, q_name: str, k_name: str, v_name: str, beta_name: str, decay_name: str, gate_name: str,
                 o_name: str, a_log_name: str, dt_bias_name: str, norm_name: str, conv_suffix: str = ".conv"):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} groups")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.head_dim, self.value_dim, self.taps = int(head_dim), int(value_dim), int(taps)
        if not 1 <= self.head_dim <= ops.GATED_DELTA_MAX_DIM:
            raise ValueError(f"the delta rule takes heads of up to {ops.GATED_DELTA_MAX_DIM} entries, got {head_dim}")
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"a short convolution takes 1..{ops.SHORT_CONV_MAX_TAPS} taps, got {taps}")
        self.norm_eps = float(norm_eps)
        self.names = (q_name, k_name, v_name, gate_name, beta_name, decay_name)
        self.o_name, self.a_log_name, self.dt_bias_name, self.norm_name = o_name, a_log_name, dt_bias_name, norm_name
        self.conv_suffix = conv_suffix
        G, H, d, e = self.num_kv_heads, self.num_heads, self.head_dim, self.value_dim
        self.channels = 2 * G * d + H * e                 # what the convolution runs over: q | k | v
        self.q_col, self.k_col, self.v_col = 0, G * d, 2 * G * d
        self.gate_col = self.channels
        self.beta_col = self.gate_col + H * e
        self.decay_col = self.beta_col + H
        self.width = (self.decay_col + H + 7) // 8 * 8    # rows of the projection stay 16-byte multiples
        self.runtime = None

    def state_need(self):
        # (kept transposed: a column of S is consecutive)
        return StateNeed((self.num_heads, self.value_dim, self.head_dim), torch.float32)

    def extra_state_needs(self):
        if self.taps == 1:
            return {}
        return {"mixer_taps": StateNeed((self.taps - 1, self.channels), torch.float32)}

    def tile_sizes(self):
        return [ops.SHORT_CONV_TILE]

    def tensors(self):
        q, k, v, gate, beta, decay = self.names
        W, G, H, d, e = self.hidden_size, self.num_kv_heads, self.num_heads, self.head_dim, self.value_dim
        decls = [TensorDecl(q, (G * d, W)), TensorDecl(k, (G * d, W)), TensorDecl(v, (H * e, W)),
                 TensorDecl(gate, (H * e, W)), TensorDecl(beta, (H, W)), TensorDecl(decay, (H, W)),
                 TensorDecl(self.o_name, (W, H * e)),
                 TensorDecl(self.a_log_name, (H,), role="vector", init="zeros"),
                 TensorDecl(self.dt_bias_name, (H,), role="vector", init="zeros"),
                 TensorDecl(self.norm_name, (e,), role="vector", init="ones_jitter")]
        for name, rows in ((q, G * d), (k, G * d), (v, H * e)):
            decls.append(TensorDecl(name + self.conv_suffix, (rows, self.taps), role="vector", init="taps"))
        return decls

    def bind(self, get, runtime):
        q, k, v, gate, beta, decay = self.names
        rows = [get(n) for n in self.names]
        pad = self.width - sum(r.shape[0] for r in rows)
        if pad:
            rows.append(torch.zeros((pad, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_taps = torch.cat([get(n + self.conv_suffix) for n in (q, k, v)], dim=0).t().contiguous()   # [taps, channels]
        self.w_o = get(self.o_name)
        self.a_log, self.dt_bias, self.norm_weight = get(self.a_log_name), get(self.dt_bias_name), get(self.norm_name)
        self.runtime = runtime

    def forward(self, x, ctx, cache):
        rt = self.runtime
        H, G, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        T = x.shape[0]
        ws = ctx.workspace
        proj = ws.get("delta_proj", (T, self.width), rt.dtype)
        ops.linear(proj, x, self.w_in, ctx.status)
        conv = ws.get("delta_conv", (T, self.channels), rt.dtype)
        taps_state = (cache.extra or {}).get("mixer_taps")
        if ctx.pure_decode:
            ops.short_conv_general(conv, proj[:, :self.channels], self.w_taps, taps_state, ctx.state_slots, ctx.cu_q, None,
                                   None, ctx.num_requests, add_input=False, silu=True)
        else:
            tile_request, tile_q0, num_tiles, _ = ctx.tiles[ops.SHORT_CONV_TILE]
            ops.short_conv_general(conv, proj[:, :self.channels], self.w_taps, taps_state, ctx.state_slots, ctx.cu_q,
                                   tile_request, tile_q0, num_tiles, add_input=False, silu=True)
        o = ws.get("delta_out", (T, H * e), torch.float32)
        scratch = ws.get("delta_numbers", (T, ops.gated_delta_scratch_width(H, G)), torch.float32)
        ops.gated_delta_scan(o, conv, self.q_col, self.k_col, self.v_col, proj, self.beta_col, self.decay_col, self.a_log,
                             self.dt_bias, cache.state, ctx.state_slots, ctx.cu_q, ctx.num_requests, H, G, d, e, UNIT_EPS,
                             d ** -0.5, scratch=scratch)
        gated = ws.get("delta_gated", (T, H * e), rt.dtype)
        ops.head_norm_gate(gated, o, proj[:, self.gate_col:self.gate_col + H * e], self.norm_weight, self.norm_eps, H, e)
        return ops.linear_for_residual(gated, self.w_o, ws, "mixer_out", ctx.status)
