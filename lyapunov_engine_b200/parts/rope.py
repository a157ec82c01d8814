"""Rotary position encoding: the frequency table and its use on queries and
keys, fused with the cache write.

Frequencies f_j = theta^(-2j/rot) in float32 as the reference builds them
(python/lyapunov_engine/models/llama.py:180-184); angles p * f_j, their cosines
and sines in float32 (llama.py:186-194); rotate-half pairing (llama.py:23-31).
The reference then casts cos/sin to the activations' type and rotates in it;
here the table stays 32-bit and so does the rotation, as in the reference's own
fused kernel (csrc/kernels/fused_rope_paged.cu:26-46).

"llama3" scaling is not in the reference.  By the meaning of its config.json
keys: a frequency whose wavelength 2*pi/f is shorter than original_max /
high_freq_factor is kept; one longer than original_max / low_freq_factor is
divided by ``factor``; in between the two are blended linearly in
original_max / wavelength.
"""
from __future__ import annotations

import math

import torch

from .. import ops
from .base import PositionEncoding, register_position_encoding


def inverse_frequencies(rot: int, theta: float, scaling: dict | None) -> torch.Tensor:
    exponents = torch.arange(0, rot, 2, dtype=torch.float32) / rot
    inv_freq = 1.0 / (theta ** exponents)
    if not scaling:
        return inv_freq
    if scaling.get("rope_type") != "llama3":
        raise ValueError(f"rotary scaling {scaling.get('rope_type')!r} is not supported")
    factor, low, high = float(scaling["factor"]), float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    original = float(scaling["original_max_position_embeddings"])
    scaled = []
    for f in inv_freq.tolist():
        wavelength = 2.0 * math.pi / f
        if wavelength < original / high:
            scaled.append(f)
        elif wavelength > original / low:
            scaled.append(f / factor)
        else:
            blend = (original / wavelength - low) / (high - low)
            scaled.append((1.0 - blend) * f / factor + blend * f)
    return torch.tensor(scaled, dtype=torch.float32)


@register_position_encoding("rotary")
class RotaryEncoding(PositionEncoding):
    """``rot`` leading dimensions of each head are rotated (rot = head_dim for
    Llama); the table covers positions 0 .. max_positions - 1."""

    def __init__(self, head_dim: int, theta: float, max_positions: int, scaling: dict | None = None,
                 rot: int | None = None):
        self.head_dim = int(head_dim)
        self.rot = int(rot if rot is not None else head_dim)
        if self.rot % 2 or not 0 < self.rot <= self.head_dim:
            raise ValueError(f"rotary width {self.rot} must be even and at most head_dim {self.head_dim}")
        self.theta = float(theta)
        self.scaling = dict(scaling) if scaling else None
        self.max_positions = int(max_positions)
        self.table = None

    def build_table(self, max_positions: int | None = None) -> torch.Tensor:
        """[positions, rot] float32 on the CPU: cos(rot/2) || sin(rot/2)."""
        n = int(max_positions or self.max_positions)
        inv_freq = inverse_frequencies(self.rot, self.theta, self.scaling)
        angles = torch.outer(torch.arange(n, dtype=torch.float32), inv_freq)
        return torch.cat((angles.cos(), angles.sin()), dim=-1).contiguous()

    def bind(self, get, runtime):
        n = min(self.max_positions, runtime.max_model_len) if runtime.max_model_len else self.max_positions
        key = ("rotary", self.rot, self.theta, repr(self.scaling), n)
        table = runtime.shared.get(key)
        if table is None:
            table = self.build_table(n).to(runtime.device)
            runtime.shared[key] = table
        self.table = table

    def product_encode_store(self, qkv, x, w_qkv, geometry, ctx, kv, write: bool) -> bool:
        """qkv = x @ w_qkv^T, rotated and stored, as one kernel where that exists
        (few rows, bfloat16, the whole head rotates).  False: nothing was done,
        the caller runs the product and encode_and_store."""
        nh, nkv, hd = geometry
        if not ops.FUSE_ROTARY or x.dtype != torch.bfloat16 or not ops.rotary_product_applies(x, w_qkv, hd, self.table.shape[1]):
            return False
        ops.gemm_skinny_rotary(qkv, x, w_qkv, kv.k if kv is not None else None, kv.v if kv is not None else None, self.table,
                               ctx.positions, ctx.request_of_token,
                               ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0], nh, nkv, hd,
                               kv.page_size if kv is not None else 1, write and kv is not None, ctx.status)
        return True

    def encode_and_store(self, qkv, geometry, ctx, kv, write: bool) -> None:
        nh, nkv, hd = geometry
        ops.rope_kv_write(qkv, kv.k if kv is not None else None, kv.v if kv is not None else None, self.table,
                          ctx.positions, ctx.request_of_token, ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0],
                          nh, nkv, hd, kv.page_size if kv is not None else 1, write and kv is not None, ctx.status)


def pair_rates(rot: int, base: float) -> torch.Tensor:
    """f_i = base^(-2i / rot), i < rot / 2: made in 64 bits, kept as float32."""
    i = torch.arange(0, rot, 2, dtype=torch.float64)
    return torch.pow(torch.tensor(float(base), dtype=torch.float64), -i / max(rot, 1)).to(torch.float32)


@register_position_encoding("rotary_pairs")
class RotaryPairsEncoding(PositionEncoding):
    """Rotary positions on neighbouring entries: in every head of queries and
    keys the pair (2i, 2i + 1), 2i + 1 < ``rot``, turns by the angle p * f_i,
    f_i = base^(-2i / rot): (a, b) -> (a cos - b sin, b cos + a sin); the
    entries from ``rot`` on pass unchanged.  ``unit_eps`` not None: after the
    turn every head of queries and keys is divided by sqrt(mean(head^2) +
    unit_eps) (a norm without a weight).  ``values_are_keys``: the projection
    has no values of its own; the value pool receives the keys as projected,
    before turn and norm.  No table: the angle (position times rate), sine and
    cosine are computed in 32 bits from the step's own positions, so there is no
    longest position.  ``head_dim`` is the real size of queries and keys; the
    heads the kernels see may be padded with zeros behind it."""
    padded_heads_ok = True

    def __init__(self, head_dim: int, rot: int, base: float, unit_eps: float | None = None, values_are_keys: bool = False):
        self.head_dim, self.rot, self.base = int(head_dim), int(rot), float(base)
        if self.rot % 2 or not 0 <= self.rot <= self.head_dim:
            raise ValueError(f"rotary width {rot} must be even and at most the head size {head_dim}")
        self.unit_eps = float(unit_eps) if unit_eps is not None else None
        self.values_are_keys = bool(values_are_keys)
        self.rates = None

    def bind(self, get, runtime):
        key = ("rotary_pairs", self.rot, self.base)
        rates = runtime.shared.get(key)
        if rates is None:
            rates = runtime.shared[key] = pair_rates(max(self.rot, 2), self.base).to(runtime.device).contiguous()
        self.rates = rates

    def encode_and_store(self, qkv, geometry, ctx, kv, write: bool) -> None:
        nh, nkv, hd = geometry
        write = write and kv is not None
        ops.rope_norm_store(qkv, kv.k if write else None, kv.v if write else None, self.rates, ctx.positions,
                            ctx.request_of_token, ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0],
                            nh, nkv, hd, 0, self.rot, self.unit_eps, self.head_dim, kv.page_size if kv is not None else 1,
                            write, self.values_are_keys, ctx.status)
        if write and not self.values_are_keys:
            # (values of their own: stored as projected; the store kernel writes two pools, both are the values' here)
            ops.kv_store(qkv, (nh + nkv) * hd, (nh + nkv) * hd, kv.v, kv.v, ctx.positions, ctx.request_of_token,
                         ctx.block_tables[kv.group], nkv, hd, kv.page_size, ctx.status)


def ramped_rates(rot: int, base: float, scaling: dict | None) -> tuple[torch.Tensor, float]:
    """(rates f_i for i < rot / 2, the factor on cosines and sines).  Plain:
    f_i = base^(-2i / rot) and 1.  With ``scaling`` = {factor, original, fast,
    slow} (the blend known as YaRN): the pair index at which a rate makes t
    turns over ``original`` positions is d(t) = rot ln(original / (2 pi t)) /
    (2 ln base); between lo = max(floor(d(fast)), 0) and hi = min(ceil(d(slow)),
    rot - 1) a ramp r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1) blends
    f_i (fast pairs, r = 0) into f_i / factor (slow pairs, r = 1), and cosines
    and sines are multiplied by 0.1 ln(factor) + 1.  64-bit numbers."""
    i = torch.arange(max(rot, 2) // 2, dtype=torch.float64)
    rates = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / max(rot, 2))
    if not scaling:
        return rates, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:
        return rot * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), rot - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    rates = rates / factor * ramp + rates * (1.0 - ramp)
    return rates, 0.1 * math.log(factor) + 1.0


@register_position_encoding("rotary_normed")
class NormedRotaryEncoding(PositionEncoding):
    """Rotary positions in the rotate-half layout (entry i < rot / 2 of a head
    turns with entry i + rot / 2), with what a projection may want before the
    turn, all in one kernel with the cache write: biases on q, k and v
    (``bias_names``), and a norm over the whole of q and over the whole of k
    (not per head): x / sqrt(mean(x^2) + eps) * w with ``q_norm_name`` [heads
    * head_dim] and ``k_norm_name`` [kv_heads * head_dim].  ``scaling``: see
    ramped_rates.  No table: the angle (position times a 64-bit rate, taken
    in 64 bits) and its cosine and sine (kept in 32 bits) are made from the
    step's own positions.  ``head_dim`` is the real size of queries and
    keys (``value_dim`` of values); the heads the kernels see may be padded
    with zeros behind it (``set_geometry``)."""
    padded_heads_ok = True
    takes_gate_columns = True       # the kernel walks rows by their stride: columns behind q | k | v are left alone

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, rot: int, base: float, scaling: dict | None = None,
                 norm_eps: float | None = None, q_norm_name: str | None = None, k_norm_name: str | None = None,
                 bias_names: tuple | None = None, value_dim: int | None = None):
        self.num_heads, self.num_kv_heads, self.head_dim = int(num_heads), int(num_kv_heads), int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.head_dim
        self.rot, self.base = int(rot), float(base)
        if self.rot % 2 or not 0 <= self.rot <= self.head_dim:
            raise ValueError(f"rotary width {rot} must be even and at most the head size {head_dim}")
        if (q_norm_name is None) != (k_norm_name is None):
            raise ValueError("queries and keys are normed both or neither")
        if q_norm_name is not None and norm_eps is None:
            raise ValueError("a norm over the projections needs its eps")
        self.scaling = dict(scaling) if scaling else None
        self.norm_eps = float(norm_eps) if norm_eps is not None else 0.0
        self.q_norm_name, self.k_norm_name = q_norm_name, k_norm_name
        self.bias_names = tuple(bias_names) if bias_names else None
        self.padded = self.head_dim
        self.rates = self.bias = self.w_q = self.w_k = None
        self.magnitude = 1.0

    def set_geometry(self, padded_head_dim: int) -> None:
        """The head size of kernels and pages (at least the real sizes)."""
        self.padded = int(padded_head_dim)

    def tensors(self):
        from .base import TensorDecl
        nh, nkv, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        decls = []
        if self.q_norm_name:
            decls += [TensorDecl(self.q_norm_name, (nh * d,), role="vector", init="ones_jitter"),
                      TensorDecl(self.k_norm_name, (nkv * d,), role="vector", init="ones_jitter")]
        if self.bias_names:
            qb, kb, vb = self.bias_names
            decls += [TensorDecl(qb, (nh * d,), role="vector", init="taps"), TensorDecl(kb, (nkv * d,), role="vector", init="taps"),
                      TensorDecl(vb, (nkv * e,), role="vector", init="taps")]
        return decls

    def _padded(self, t: torch.Tensor, heads: int, size: int) -> torch.Tensor:
        if size == self.padded:
            return t.reshape(-1).contiguous()
        out = torch.zeros((heads, self.padded), dtype=t.dtype, device=t.device)
        out[:, :size] = t.view(heads, size)
        return out.view(-1)

    def bind(self, get, runtime):
        key = ("rotary_normed", self.rot, self.base, repr(self.scaling))
        found = runtime.shared.get(key)
        if found is None:
            rates, magnitude = ramped_rates(self.rot, self.base, self.scaling)
            found = runtime.shared[key] = (rates.to(runtime.device).contiguous(), magnitude)
        self.rates, self.magnitude = found
        nh, nkv, d, e = self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim
        if self.q_norm_name:
            self.w_q = self._padded(get(self.q_norm_name).to(torch.float32), nh, d)
            self.w_k = self._padded(get(self.k_norm_name).to(torch.float32), nkv, d)
        if self.bias_names:
            qb, kb, vb = (get(n).to(torch.float32) for n in self.bias_names)
            self.bias = torch.cat([self._padded(qb, nh, d), self._padded(kb, nkv, d), self._padded(vb, nkv, e)]).contiguous()

    def encode_and_store(self, qkv, geometry, ctx, kv, write: bool) -> None:
        nh, nkv, hd = geometry
        if (nh, nkv, hd) != (self.num_heads, self.num_kv_heads, self.padded):
            raise ValueError(f"the encoding was built for {self.num_heads} + {self.num_kv_heads} heads of {self.padded}, "
                             f"the mixer brings {nh} + {nkv} of {hd}")
        write = write and kv is not None
        ops.rope_qknorm_store(qkv, self.bias, self.w_q, self.w_k, self.norm_eps, nh * self.head_dim, nkv * self.head_dim,
                              self.rates, self.rot, self.magnitude, kv.k if write else None, kv.v if write else None,
                              ctx.positions, ctx.request_of_token,
                              ctx.block_tables[kv.group] if kv is not None else ctx.block_tables[0], nh, nkv, hd,
                              kv.page_size if kv is not None else 1, write, ctx.status)
