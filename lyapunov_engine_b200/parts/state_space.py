"""State-space mixers: a state of fixed size per request instead of a cache of
keys, carried from token to token in 32 bits.

"state_space_duality" (Mamba-2).  With x the mixer's input, H heads of P
channels, N numbers of state per channel, G groups (head h uses group h // (H /
G)), inner = H * P:

    [z | x' | B | C | dt] = W_in x          (inner, inner, G N, G N, H)
    [x' | B | C] <- silu(conv([x' | B | C]) + b)   a causal convolution over time per channel (``taps`` taps,
                                                   the last one the current token's, zeros before the start)
    dt <- softplus(dt + dt_bias)            per head
    per head, channel p:  S[p] <- exp(-exp(A_log_h) dt) S[p] + dt x'_p B;   y_p = S[p] . C + D_h x'_p
    y <- y * silu(z);  each of ``norm_groups`` equal parts of y / its root mean square;  * w;  W_o

"selective_scan" (Mamba).  inner channels, N numbers of state each:

    [x' | z] = W_in x;   x' <- silu(conv(x') + b)
    [dt' | B | C] = W_x x'   (dt_rank, N, N);   dt = softplus(W_dt dt' + b_dt)   per channel
    per channel c:  S[c] <- exp(dt_c A[c]) S[c] + dt_c x'_c B;   y_c = S[c] . C + D_c x'_c,   A = -exp(A_log) [inner, N]
    y <- y * silu(z);  W_o

Both recurrences run in one kernel (ops.ssm_scan), with the gate in its
epilogue; the convolution is the package's short convolution with a bias and
silu; the last taps - 1 inputs of the convolution are state of the request too
(``extra_state_needs``).  Step sizes, decays, the recurrence and the norm are
32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import Mixer, StateNeed, TensorDecl, register_mixer


def _conv(out, rows, channels, mixer, ctx, cache):
    """The mixer's short convolution over the first ``channels`` columns of ``rows``."""
    taps_state = (cache.extra or {}).get("mixer_taps")
    if ctx.pure_decode:
        ops.short_conv_general(out, rows[:, :channels], mixer.w_taps, taps_state, ctx.state_slots, ctx.cu_q, None, None,
                               ctx.num_requests, add_input=False, silu=True, bias=mixer.conv_bias)
    else:
        tile_request, tile_q0, num_tiles, _ = ctx.tiles[ops.SHORT_CONV_TILE]
        ops.short_conv_general(out, rows[:, :channels], mixer.w_taps, taps_state, ctx.state_slots, ctx.cu_q, tile_request,
                               tile_q0, num_tiles, add_input=False, silu=True, bias=mixer.conv_bias)


def _pad_rows(rows: list, width: int):
    have = sum(r.shape[0] for r in rows)
    if width > have:
        rows.append(torch.zeros((width - have, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
    return torch.cat(rows, dim=0).contiguous()


@register_mixer("state_space_duality")
class StateSpaceDualityMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, value_dim: int, state_dim: int, groups: int, taps: int,
                 norm_groups: int, norm_eps: float, in_name: str, conv_name: str, conv_bias_name: str, dt_bias_name: str,
                 a_log_name: str, d_name: str, norm_name: str, o_name: str):
        self.hidden_size, self.num_heads, self.value_dim = int(hidden_size), int(num_heads), int(value_dim)
        self.state_dim, self.groups, self.taps, self.norm_groups = int(state_dim), int(groups), int(taps), int(norm_groups)
        if self.num_heads % self.groups:
            raise ValueError(f"{num_heads} heads do not divide into {groups} groups")
        self.inner = self.num_heads * self.value_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} channels do not divide into {norm_groups} parts for the norm")
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"a short convolution takes 1..{ops.SHORT_CONV_MAX_TAPS} taps, got {taps}")
        if not 1 <= self.state_dim <= ops.SSM_MAX_STATE:
            raise ValueError(f"a channel keeps 1..{ops.SSM_MAX_STATE} numbers of state, got {state_dim}")
        self.norm_eps = float(norm_eps)
        self.in_name, self.conv_name, self.conv_bias_name = in_name, conv_name, conv_bias_name
        self.dt_bias_name, self.a_log_name, self.d_name, self.norm_name, self.o_name = dt_bias_name, a_log_name, d_name, norm_name, o_name
        GN = self.groups * self.state_dim
        self.channels = self.inner + 2 * GN                    # what the convolution runs over: x' | B | C
        # the fused projection's rows, reordered so that the convolution's channels come first: x' | B | C | z | dt
        self.z_col = (self.channels + 7) // 8 * 8
        self.dt_col = self.z_col + (self.inner + 7) // 8 * 8
        self.width = self.dt_col + (self.num_heads + 7) // 8 * 8
        self.runtime = None

    def state_need(self):
        return StateNeed((self.inner, self.state_dim), torch.float32)

    def extra_state_needs(self):
        if self.taps == 1:
            return {}
        return {"mixer_taps": StateNeed((self.taps - 1, self.channels), torch.float32)}

    def tile_sizes(self):
        return [ops.SHORT_CONV_TILE]

    def tensors(self):
        W, H, GN = self.hidden_size, self.num_heads, self.groups * self.state_dim
        return [TensorDecl(self.in_name, (2 * self.inner + 2 * GN + H, W)),
                TensorDecl(self.conv_name, (self.channels, self.taps), role="vector", init="taps"),
                TensorDecl(self.conv_bias_name, (self.channels,), role="vector", init="taps"),
                TensorDecl(self.dt_bias_name, (H,), role="vector", init="zeros"),
                TensorDecl(self.a_log_name, (H,), role="vector", init="zeros"),
                TensorDecl(self.d_name, (H,), role="vector", init="ones_jitter"),
                TensorDecl(self.norm_name, (self.inner,), role="vector", init="ones_jitter"),
                TensorDecl(self.o_name, (W, self.inner))]

    def bind(self, get, runtime):
        w = get(self.in_name)
        inner, GN, H = self.inner, self.groups * self.state_dim, self.num_heads
        z, xbc, dt = w[:inner], w[inner:2 * inner + 2 * GN], w[2 * inner + 2 * GN:]
        self.w_in = _pad_rows([_pad_rows([xbc], self.z_col), _pad_rows([z], self.dt_col - self.z_col), dt], self.width)
        self.w_taps = get(self.conv_name).t().contiguous()          # [taps, channels]
        self.conv_bias = get(self.conv_bias_name).contiguous()
        self.dt_bias, self.a_log, self.d_skip = get(self.dt_bias_name), get(self.a_log_name), get(self.d_name)
        self.norm_weight = get(self.norm_name)
        self.w_o = get(self.o_name)
        self.runtime = runtime

    def inner_width(self) -> int:
        return self.inner

    def output_weight(self):
        return self.w_o

    def forward(self, x, ctx, cache):
        return ops.linear_for_residual(self.forward_inner(x, ctx, cache), self.w_o, ctx.workspace, "mixer_out", ctx.status)

    def forward_inner(self, x, ctx, cache, out=None, scale: float = 1.0):
        """The gated, normed channels before the output projection [T, inner]."""
        rt, ws = self.runtime, ctx.workspace
        T, inner, N, H = x.shape[0], self.inner, self.state_dim, self.num_heads
        if out is not None or scale != 1.0:
            raise ValueError("the state-space duality mixer's norm writes its own buffer, unscaled")
        proj = ws.get("ssd_proj", (T, self.width), rt.dtype)
        ops.linear(proj, x, self.w_in, ctx.status)
        conv = ws.get("ssd_conv", (T, self.channels), rt.dtype)
        _conv(conv, proj, self.channels, self, ctx, cache)
        y = ws.get("ssd_y", (T, inner), torch.float32)
        ops.ssm_scan(y, conv[:, :inner], conv, inner, inner + self.groups * N, proj[:, self.dt_col:self.dt_col + H],
                     proj[:, self.z_col:self.z_col + inner], self.dt_bias, self.a_log, self.d_skip, cache.state, ctx.state_slots,
                     ctx.cu_q, ctx.num_requests, N, self.value_dim, (H // self.groups) * self.value_dim, per_row=False)
        normed = ws.get("ssd_normed", (T, inner), rt.dtype)
        ops.rmsnorm(normed, y, None, self.norm_weight, self.norm_eps, groups=self.norm_groups)
        return normed


@register_mixer("selective_scan")
class SelectiveScanMixer(Mixer):
    def __init__(self, hidden_size: int, inner: int, state_dim: int, dt_rank: int, taps: int, in_name: str, conv_name: str,
                 conv_bias_name: str, x_name: str, dt_name: str, dt_bias_name: str, a_log_name: str, d_name: str, o_name: str):
        self.hidden_size, self.inner, self.state_dim = int(hidden_size), int(inner), int(state_dim)
        self.dt_rank, self.taps = int(dt_rank), int(taps)
        if not 1 <= self.taps <= ops.SHORT_CONV_MAX_TAPS:
            raise ValueError(f"a short convolution takes 1..{ops.SHORT_CONV_MAX_TAPS} taps, got {taps}")
        if not 1 <= self.state_dim <= ops.SSM_MAX_STATE:
            raise ValueError(f"a channel keeps 1..{ops.SSM_MAX_STATE} numbers of state, got {state_dim}")
        self.in_name, self.conv_name, self.conv_bias_name, self.x_name = in_name, conv_name, conv_bias_name, x_name
        self.dt_name, self.dt_bias_name, self.a_log_name, self.d_name, self.o_name = dt_name, dt_bias_name, a_log_name, d_name, o_name
        self.channels = self.inner
        # the low projection's rows: dt' (padded to a 16-byte multiple) | B | C
        self.b_col = (self.dt_rank + 7) // 8 * 8
        self.c_col = self.b_col + self.state_dim
        self.low_width = (self.c_col + self.state_dim + 7) // 8 * 8
        self.z_col = (self.inner + 7) // 8 * 8
        self.runtime = None

    def state_need(self):
        return StateNeed((self.inner, self.state_dim), torch.float32)

    def extra_state_needs(self):
        if self.taps == 1:
            return {}
        return {"mixer_taps": StateNeed((self.taps - 1, self.channels), torch.float32)}

    def tile_sizes(self):
        return [ops.SHORT_CONV_TILE]

    def tensors(self):
        W, C, N, R = self.hidden_size, self.inner, self.state_dim, self.dt_rank
        return [TensorDecl(self.in_name, (2 * C, W)),
                TensorDecl(self.conv_name, (C, self.taps), role="vector", init="taps"),
                TensorDecl(self.conv_bias_name, (C,), role="vector", init="taps"),
                TensorDecl(self.x_name, (R + 2 * N, C)),
                TensorDecl(self.dt_name, (C, R)),
                TensorDecl(self.dt_bias_name, (C,), role="vector", init="zeros"),
                TensorDecl(self.a_log_name, (C, N), role="vector", init="zeros"),
                TensorDecl(self.d_name, (C,), role="vector", init="ones_jitter"),
                TensorDecl(self.o_name, (W, C))]

    def bind(self, get, runtime):
        C, N, R = self.inner, self.state_dim, self.dt_rank
        w = get(self.in_name)
        self.w_in = _pad_rows([_pad_rows([w[:C]], self.z_col), w[C:]], self.z_col + (C + 7) // 8 * 8)
        self.w_taps = get(self.conv_name).t().contiguous()
        self.conv_bias = get(self.conv_bias_name).contiguous()
        wx = get(self.x_name)
        self.w_x = _pad_rows([_pad_rows([wx[:R]], self.b_col), wx[R:]], self.low_width)
        # the step sizes' projection reads the low projection's whole rows: its columns under B and C are zero
        wdt = get(self.dt_name)
        self.w_dt = torch.zeros((C, self.low_width), dtype=wdt.dtype, device=wdt.device)
        self.w_dt[:, :R] = wdt
        self.dt_bias, self.a_log, self.d_skip = get(self.dt_bias_name), get(self.a_log_name).contiguous(), get(self.d_name)
        self.w_o = get(self.o_name)
        self.runtime = runtime

    def inner_width(self) -> int:
        return self.inner

    def output_weight(self):
        return self.w_o

    def forward(self, x, ctx, cache):
        return ops.linear_for_residual(self.forward_inner(x, ctx, cache), self.w_o, ctx.workspace, "mixer_out", ctx.status)

    def forward_inner(self, x, ctx, cache, out=None, scale: float = 1.0):
        """The gated channels before the output projection [T, inner], into
        ``out`` where given (a column range of wider rows is fine), times ``scale``."""
        rt, ws = self.runtime, ctx.workspace
        T, C, N = x.shape[0], self.inner, self.state_dim
        proj = ws.get("scan_proj", (T, self.w_in.shape[0]), rt.dtype)
        ops.linear(proj, x, self.w_in, ctx.status)
        conv = ws.get("scan_conv", (T, C), rt.dtype)
        _conv(conv, proj, C, self, ctx, cache)
        low = ws.get("scan_low", (T, self.low_width), rt.dtype)
        ops.linear(low, conv, self.w_x, ctx.status)
        dt = ws.get("scan_dt", (T, C), rt.dtype)
        ops.linear(dt, low, self.w_dt, ctx.status)
        if out is None:
            out = ws.get("scan_gated", (T, C), rt.dtype)
        ops.ssm_scan(out, conv, low, self.b_col, self.c_col, dt, proj[:, self.z_col:self.z_col + C], self.dt_bias, self.a_log,
                     self.d_skip, cache.state, ctx.state_slots, ctx.cu_q, ctx.num_requests, N, 1, C, per_row=True,
                     out_scale=scale)
        return out
