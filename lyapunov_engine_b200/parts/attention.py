"""Grouped-query attention over the paged cache.

One projection = rows q || k || v (the reference keeps three matrices,
python/lyapunov_engine/models/llama.py:45-47), position encoding of q and k
fused with the cache write (or a plain cache write, for keys that carry no
positions), attention of every query token over the keys of its request up to
its own position, output projection.  Head h of the queries uses key/value
head h // (nh / nkv) (csrc/kernels/flash_attn_v2.cu:30-31).

What a description may choose beyond the reference's Llama layer:

* ``window`` w: only the last w keys; ``chunk`` c: only the keys of the
  query's own chunk of c positions, chunks counted from position 0 of the
  request (the cache manager gives back the pages before the window or chunk);
* ``scale``: the factor on q . k (default 1 / sqrt(head_dim), as
  csrc/bindings.cpp:131-133); ``head_scale_name``: a tensor [nh] with one more
  factor per query head, applied to the 32-bit scores;
* ``value_dim``: values of another size than queries and keys.  Kernels and
  pages take one head size, the larger of the two rounded up to a multiple of
  16: the projections' rows are padded with zero rows (and the output
  projection with zero columns), which changes no result;
* ``position`` None: queries and keys are used as projected;
* ``gate_name``: a tensor [nh, H]; head h's output is multiplied by
  sigmoid(gate_h . x) before the output projection (the gate's rows ride at
  the end of the fused projection); with ``gate_per_entry`` the tensor is
  [nh * value_dim, H] and every entry of the heads' outputs has a gate of
  its own;
* ``keep_first`` n (with a window): the keys at positions below n stay
  visible to every later query, with their true positions; their pages are
  never given back;
* ``softcap`` c: a score s (after the scale) becomes c * tanh(s / c);
* ``v_name`` None: there is no value projection, the values are the keys as
  projected (before any position encoding or norm of the keys); the position
  encoding then fills the value pool itself (it is built with
  ``values_are_keys=True``).

The reference runs attention two ways, FlashAttention on the step's own keys
for a whole prompt and PagedAttention for one decoded token
(llama.py:82-104), and its prompt path never writes the cache.  Here there is
one way: write the step's keys and values to the pages, then attend through the
block table; which kernel does it is chosen by the step's shape and the type.
"""
from __future__ import annotations

import torch

from .. import ops
from . import attention_kernels
from .base import KVNeed, Mixer, POSITION_ENCODINGS, PartSpec, TensorDecl, register_mixer


def pad_head_rows(w: torch.Tensor, heads: int, size: int, padded: int) -> torch.Tensor:
    """[heads * size, K] -> [heads * padded, K], each head's rows followed by zero rows."""
    if padded == size:
        return w
    out = torch.zeros((heads, padded, w.shape[1]), dtype=w.dtype, device=w.device)
    out[:, :size] = w.view(heads, size, w.shape[1])
    return out.view(heads * padded, w.shape[1])


def pad_head_columns(w: torch.Tensor, heads: int, size: int, padded: int) -> torch.Tensor:
    """[N, heads * size] -> [N, heads * padded], each head's columns followed by zero columns."""
    if padded == size:
        return w
    out = torch.zeros((w.shape[0], heads, padded), dtype=w.dtype, device=w.device)
    out[:, :, :size] = w.view(w.shape[0], heads, size)
    return out.view(w.shape[0], heads * padded).contiguous()


def signed_scale(scale: float, head_scale: torch.Tensor | None, num_heads: int, device):
    """(scale >= 0, per-head factors or None, whether all factors are positive):
    the kernels keep running maxima in units of ``scale``, so a negative sign
    moves into the per-head factors, which are applied before the maximum."""
    if scale < 0:
        head_scale = -(head_scale if head_scale is not None else torch.ones(num_heads, dtype=torch.float32, device=device))
        scale = -scale
    positive = head_scale is None or bool((head_scale > 0).all().item())
    return float(scale), (head_scale.contiguous() if head_scale is not None else None), positive


@register_mixer("attention")
class AttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, position: PartSpec | None,
                 q_name: str, k_name: str, v_name: str | None, o_name: str, window: int | None = None,
                 chunk: int | None = None, scale: float | None = None, value_dim: int | None = None,
                 head_scale_name: str | None = None, gate_name: str | None = None, gate_per_entry: bool = False,
                 keep_first: int = 0, softcap: float | None = None):
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads do not divide into {num_kv_heads} groups")
        self.qk_dim = int(head_dim)
        self.value_dim = int(value_dim) if value_dim else self.qk_dim
        self.values_are_keys = v_name is None
        if self.values_are_keys and (position is None or self.value_dim != self.qk_dim):
            raise ValueError("values that are the keys need a position encoding that stores them, and the keys' size")
        # the one head size of kernels and pages
        self.head_dim = (max(self.qk_dim, self.value_dim) + 15) // 16 * 16
        self.position = None
        if position is not None:
            self.position = (POSITION_ENCODINGS.build(position, values_are_keys=True) if self.values_are_keys
                             else POSITION_ENCODINGS.build(position))
        if position is not None and self.head_dim != self.qk_dim and not getattr(self.position, "padded_heads_ok", False):
            raise ValueError(f"a position encoding needs a query/key size that is a multiple of 16 and not below the "
                             f"value size, got {head_dim} and {self.value_dim}")
        if hasattr(self.position, "set_geometry"):
            self.position.set_geometry(self.head_dim)
        if position is not None and gate_name and not getattr(self.position, "takes_gate_columns", False):
            raise ValueError("an output gate beside a position encoding is not supported (the encoding's kernels take "
                             "the projection's rows without gate columns)")
        if not 16 <= self.head_dim <= attention_kernels.MAX_HEAD_DIM:
            raise ValueError(f"attention takes head sizes up to {attention_kernels.MAX_HEAD_DIM}, got {head_dim} / {self.value_dim}")
        self.hidden_size, self.num_heads, self.num_kv_heads = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.window = int(window) if window else None
        self.chunk = int(chunk) if chunk else None
        self.reach = ops.reach_code(self.window, self.chunk)
        self.keep_first = int(keep_first or 0) if self.window else 0      # (without a window every key is visible anyway)
        if self.keep_first < 0:
            raise ValueError(f"keep_first must not be negative, got {keep_first}")
        self.softcap = float(softcap) if softcap else 0.0
        if self.softcap < 0:
            raise ValueError(f"a cap on the scores must be positive, got {softcap}")
        self.scale = float(scale) if scale is not None else 1.0 / (self.qk_dim ** 0.5)
        self.names = (q_name, k_name, v_name, o_name)
        self.head_scale_name, self.gate_name = head_scale_name, gate_name
        self.gate_per_entry = bool(gate_per_entry) and bool(gate_name)
        # rows of the projection stay 16-byte multiples
        self.gate_rows = 0
        if gate_name:
            self.gate_rows = self.num_heads * self.head_dim if self.gate_per_entry else (self.num_heads + 7) // 8 * 8
        self.w_qkv = self.w_o = self.head_scale = None
        self.head_scale_positive = True
        self.runtime = None

    def cache_need(self):
        return KVNeed(self.num_kv_heads, self.head_dim, self.window, self.chunk, keep_first=self.keep_first)

    def tile_sizes(self):
        return attention_kernels.tile_sizes()

    def decode_variant(self, fill, num_decode, context_bound):
        if self.runtime is None or self.runtime.dtype != torch.bfloat16:
            return None                       # the float32 kernel takes every shape the same way
        return attention_kernels.decode_variant(fill, self.num_heads, self.num_kv_heads, self.head_dim, context_bound,
                                                self.reach, keep_first=self.keep_first)

    def tensors(self):
        q, k, v, o = self.names
        H, nh, nkv = self.hidden_size, self.num_heads, self.num_kv_heads
        decls = [TensorDecl(q, (nh * self.qk_dim, H)), TensorDecl(k, (nkv * self.qk_dim, H)),
                 TensorDecl(o, (H, nh * self.value_dim))]
        if not self.values_are_keys:
            decls.insert(2, TensorDecl(v, (nkv * self.value_dim, H)))
        if self.head_scale_name:
            decls.append(TensorDecl(self.head_scale_name, (nh,), role="vector", init="ones_jitter"))
        if self.gate_name:
            decls.append(TensorDecl(self.gate_name, (nh * self.value_dim if self.gate_per_entry else nh, H)))
        return decls + (self.position.tensors() if self.position is not None else [])

    def bind(self, get, runtime):
        q, k, v, o = self.names
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        rows = [pad_head_rows(get(q), nh, self.qk_dim, hd), pad_head_rows(get(k), nkv, self.qk_dim, hd)]
        if not self.values_are_keys:
            rows.append(pad_head_rows(get(v), nkv, self.value_dim, hd))
        if self.gate_name and self.gate_per_entry:
            rows.append(pad_head_rows(get(self.gate_name), nh, self.value_dim, hd))
        elif self.gate_name:
            gate = get(self.gate_name)
            pad = torch.zeros((self.gate_rows - nh, gate.shape[1]), dtype=gate.dtype, device=gate.device)
            rows += [gate, pad]
        self.w_qkv = torch.cat(rows, dim=0).contiguous()
        self.w_o = pad_head_columns(get(o), nh, self.value_dim, hd)
        self.runtime = runtime
        head_scale = get(self.head_scale_name).to(torch.float32) if self.head_scale_name else None
        self.kernel_scale, self.head_scale, self.head_scale_positive = signed_scale(self.scale, head_scale, nh, runtime.device)
        if self.position is not None:
            self.position.bind(get, runtime)
        attention_kernels.prepare(self.head_dim)

    def inner_width(self) -> int:
        """Columns of what the output projection reads (the heads as the kernels hold them)."""
        return self.num_heads * self.head_dim

    def output_weight(self):
        return self.w_o

    def forward(self, x, ctx, cache):
        return ops.linear_for_residual(self.forward_inner(x, ctx, cache), self.w_o, ctx.workspace, "mixer_out", ctx.status)

    def forward_inner(self, x, ctx, cache, out=None, scale: float = 1.0):
        """The heads' outputs, gated, before the output projection: [T, nh *
        head_dim], into ``out`` where given (a column range of wider rows is
        fine) and times ``scale``: for a caller that has its own use for
        them.  Only a mixer with a gate per entry writes elsewhere than its
        own buffer or scales."""
        rt = self.runtime
        nh, nkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        T = x.shape[0]
        ws = ctx.workspace
        width = (nh + (1 if self.values_are_keys else 2) * nkv) * hd
        qkv = ws.get("qkv", (T, width + self.gate_rows), rt.dtype)
        # a position encoding may know how to run the product itself, with its own work in the epilogue
        fused = getattr(self.position, "product_encode_store", None) if not self.gate_rows else None
        if fused is None or not fused(qkv, x, self.w_qkv, (nh, nkv, hd), ctx, cache.kv, cache.write):
            ops.linear(qkv, x, self.w_qkv, ctx.status)
            if self.position is not None:
                self.position.encode_and_store(qkv, (nh, nkv, hd), ctx, cache.kv, cache.write)
            elif cache.write:
                ops.kv_store(qkv, nh * hd, (nh + nkv) * hd, cache.kv.k, cache.kv.v, ctx.positions, ctx.request_of_token,
                             ctx.block_tables[cache.kv.group], nkv, hd, cache.kv.page_size, ctx.status)
        attn = ws.get("attn", (T, nh * hd), rt.dtype)
        attention_kernels.run(attn, qkv, ctx, cache.kv, nh, nkv, hd, self.reach, self.kernel_scale, self.head_scale,
                              self.head_scale_positive, keep_first=self.keep_first, softcap=self.softcap)
        if self.gate_per_entry:
            target = out if out is not None else attn
            ops.sigmoid_gate(target, attn, qkv[:, width:width + nh * hd], scale)
            return target
        if out is not None or scale != 1.0:
            raise ValueError("only a mixer with a gate per entry hands its heads' outputs on elsewhere or scaled")
        if self.gate_rows:
            ops.head_gate(attn, qkv[:, width:width + nh], nh, hd)
        return attn
