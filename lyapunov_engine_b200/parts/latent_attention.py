"""Latent attention: every head's keys and values are linear maps of one
normed latent vector per token, and only that vector is cached.

With x the mixer's input (width H), nh heads, d query/key size, e value size
and r the latent size:

    q_h = Wq_h x                     c = rmsnorm(Wdkv x) * w_c           (r values, 32-bit norm)
    k_h(j) = Wuk_h c_j               v_h(j) = Wuv_h c_j
    score_h(i, j) = (q_h(i) . k_h(j)) * scale,   j <= i (optionally a window or chunks)
    out = Wo concat_h( sigmoid(g_h . x) * sum_j softmax_j(score_h) v_h(j) )

No positions enter.  Because k and v are linear in c, the step never builds
them: q_h . (Wuk_h c) = (Wuk_h^T q_h) . c, so each head's query is carried into
the latent space (one small product per head), attention runs over the cached
latents as both keys and values -- all heads share the one "key/value head" of
size r, the existing paged kernels serve it -- and each head's attended latent
is carried out through Wuv_h (again one small product per head, with the
head's output gate in its epilogue).  The cache holds r values per token and
layer, in one pool that the kernels read as keys and as values (the pool's rows
are padded with zeros to a multiple of 16).

Two options beyond that:

* ``rot_dim`` > 0: beside the latent every token has one rotated key part of
  rot_dim entries, shared by all heads (the last rot_dim rows of the down
  projection, not normed), and every head's query has rot_dim more entries
  behind its head_dim unrotated ones; both turn in neighbouring pairs by
  position * rot_base^(-2i / rot_dim), and the score is (q_unrotated .
  k_unrotated + q_rotated . k_rotated) * scale.  The cached row is [latent |
  rotated part]; a head's query in the latent space gets its own turned part
  behind it, so the one dot product over the row gives the score; the way out
  of the latent space reads the latent's columns only.
* ``q_rank`` > 0: the queries go through a latent of their own, q = Wuq
  rmsnorm(Wdq x) * w_q (``q_down_name``, ``q_norm_name``; ``q_name`` is then
  Wuq, [heads * (head_dim + rot_dim), q_rank]).

Per-head products: the package's FP32-pipe kernel (float32, and bfloat16 steps
of few rows); bfloat16 steps of many rows go to the library's batched product,
as the other many-row products do.
"""
from __future__ import annotations

import os

import torch

from .. import ops
from . import attention_kernels
from .attention import signed_scale
from .base import KVNeed, Mixer, TensorDecl, register_mixer
from .rope import pair_rates

LIBRARY_ROWS = 64       # bfloat16 steps with more rows than this run the per-head products in the library
# The most ways a decoded token's latents are cut.  (Capping it at 8, the most that merge inside a thread-block
# cluster without a second kernel, was measured and is slower: all heads of a request share one pool, so a request is
# two blocks before splitting, and 512 keys a block cost more than the merge kernel: 1.03 against 0.93 ms a step.)
MAX_DECODE_SPLITS = int(os.environ.get("LYAPUNOV_LATENT_SPLITS", str(attention_kernels.DECODE_MAX_SPLITS)))


@register_mixer("latent_attention")
class LatentAttentionMixer(Mixer):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, value_dim: int, latent_dim: int, scale: float,
                 norm_eps: float, q_name: str, down_name: str, latent_norm_name: str, up_k_name: str, up_v_name: str,
                 o_name: str, gate_name: str | None = None, window: int | None = None, chunk: int | None = None,
                 rot_dim: int = 0, rot_base: float | None = None, q_rank: int = 0, q_down_name: str | None = None,
                 q_norm_name: str | None = None):
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.qk_dim, self.value_dim, self.latent_dim = int(head_dim), int(value_dim), int(latent_dim)
        self.rot_dim, self.rot_base, self.q_rank = int(rot_dim), rot_base, int(q_rank)
        if self.rot_dim and (self.rot_dim % 2 or self.latent_dim % 2 or rot_base is None):
            raise ValueError(f"a rotated part needs an even size, an even latent and a base, got {rot_dim}, {latent_dim}, {rot_base}")
        if self.q_rank and not (q_down_name and q_norm_name):
            raise ValueError("queries through a latent need the names of its projection and of its norm's weight")
        if gate_name and (self.rot_dim or self.q_rank):
            raise ValueError("an output gate beside a rotated part or a query latent is not supported")
        self.q_names = (q_down_name, q_norm_name)
        self.q_head = self.qk_dim + self.rot_dim                         # a head's query: unrotated, then rotated
        self.padded_latent = (self.latent_dim + self.rot_dim + 15) // 16 * 16   # the head size of kernels and pages
        if not 16 <= self.padded_latent <= attention_kernels.MAX_HEAD_DIM:
            raise ValueError(f"latent attention takes latent sizes up to {attention_kernels.MAX_HEAD_DIM}, got {latent_dim}")
        self.scale, self.norm_eps = float(scale), float(norm_eps)
        self.reach = ops.reach_code(window, chunk)
        self.window, self.chunk = (int(window) if window else None), (int(chunk) if chunk else None)
        self.names = (q_name, down_name, latent_norm_name, up_k_name, up_v_name, o_name)
        self.gate_name = gate_name
        self.gate_rows = (self.num_heads + 7) // 8 * 8 if gate_name else 0
        self.runtime = None

    def cache_need(self):
        return KVNeed(1, self.padded_latent, self.window, self.chunk, values=False)

    def tile_sizes(self):
        return attention_kernels.tile_sizes()

    def decode_variant(self, fill, num_decode, context_bound):
        if self.runtime is None or self.runtime.dtype != torch.bfloat16:
            return None
        return attention_kernels.decode_variant(fill, self.num_heads, 1, self.padded_latent, context_bound, self.reach,
                                                MAX_DECODE_SPLITS)

    def tensors(self):
        q, down, norm, uk, uv, o = self.names
        H, nh, d, e, r = self.hidden_size, self.num_heads, self.qk_dim, self.value_dim, self.latent_dim
        decls = [TensorDecl(q, (nh * self.q_head, self.q_rank or H)), TensorDecl(down, (r + self.rot_dim, H)),
                 TensorDecl(norm, (r,), role="vector", init="ones_jitter"),
                 TensorDecl(uk, (nh * d, r)), TensorDecl(uv, (nh * e, r)), TensorDecl(o, (H, nh * e))]
        if self.gate_name:
            decls.append(TensorDecl(self.gate_name, (nh, H)))
        if self.q_rank:
            decls += [TensorDecl(self.q_names[0], (self.q_rank, H)),
                      TensorDecl(self.q_names[1], (self.q_rank,), role="vector", init="ones_jitter")]
        return decls

    def bind(self, get, runtime):
        q, down, norm, uk, uv, o = self.names
        nh, d, e, r, rp = self.num_heads, self.qk_dim, self.value_dim, self.latent_dim, self.padded_latent
        rd, qh = self.rot_dim, self.q_head
        # the projection's first rows: the queries themselves, or their latent
        rows = [get(self.q_names[0]) if self.q_rank else get(q), get(down)]
        self.q_width = self.q_rank or nh * qh
        self.w_up_q = get(q) if self.q_rank else None
        self.q_norm_weight = get(self.q_names[1]) if self.q_rank else None
        self.rates = pair_rates(max(rd, 2), self.rot_base).to(runtime.device).contiguous() if rd else None
        # the latent's columns start on a 16-byte boundary of the projection's rows, and so do the gate's
        self.latent_col = (self.q_width + 7) // 8 * 8
        if self.latent_col != self.q_width:
            rows.insert(1, torch.zeros((self.latent_col - self.q_width, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        self.gate_col = (self.latent_col + r + rd + 7) // 8 * 8
        if self.gate_col != self.latent_col + r + rd:
            rows.append(torch.zeros((self.gate_col - self.latent_col - r - rd, self.hidden_size), dtype=rows[0].dtype, device=rows[0].device))
        if self.gate_name:
            gate = get(self.gate_name)
            rows += [gate, torch.zeros((self.gate_rows - nh, self.hidden_size), dtype=gate.dtype, device=gate.device)]
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.norm_weight = get(norm)
        # into the latent space: [nh, r (padded), d (+ rd)], head h's key map transposed; the rotated entries of a
        # head's query pass through to the columns behind the latent (a product with ones and zeros is exact)
        into = torch.zeros((nh, rp, qh), dtype=runtime.dtype, device=runtime.device)
        into[:, :r, :d] = get(uk).view(nh, d, r).transpose(1, 2)
        for j in range(rd):
            into[:, r + j, d + j] = 1.0
        self.w_into = into.contiguous()
        # out of it: [nh, e, r (padded)]
        out_of = torch.zeros((nh, e, rp), dtype=runtime.dtype, device=runtime.device)
        out_of[:, :, :r] = get(uv).view(nh, e, r)
        self.w_out_of = out_of.contiguous()
        self.w_o = get(o)
        self.runtime = runtime
        self.kernel_scale, self.head_scale, self.head_scale_positive = signed_scale(self.scale, None, nh, runtime.device)
        attention_kernels.prepare(rp)

    def _per_head(self, out, a, w, gate, heads):
        """out[t, h, :] = w[h] @ a[t, h, :] (times the head's gate)."""
        T = a.shape[0]
        if a.dtype == torch.bfloat16 and T > LIBRARY_ROWS:
            ops.counters["library_products"] += 1
            K, N = w.shape[2], w.shape[1]
            torch.bmm(a.view(T, heads, K).transpose(0, 1), w.transpose(1, 2), out=out.view(T, heads, N).transpose(0, 1))
            if gate is not None:
                ops.head_gate(out, gate, heads, N)
            return
        ops.gemm_heads(out, a, w, gate)

    def forward(self, x, ctx, cache):
        rt = self.runtime
        nh, r, rp, e = self.num_heads, self.latent_dim, self.padded_latent, self.value_dim
        T = x.shape[0]
        ws = ctx.workspace
        proj = ws.get("latent_proj", (T, self.w_in.shape[0]), rt.dtype)
        ops.linear(proj, x, self.w_in, ctx.status)
        kv = cache.kv
        q_latent = ws.get("latent_q", (T, nh * rp), rt.dtype)
        if self.rot_dim or self.q_rank:
            table = ctx.block_tables[kv.group]
            queries = proj[:, :self.q_width]
            second = None
            if self.q_rank:
                q_normed = ws.get("latent_q_normed", (T, self.q_rank), rt.dtype)
                second = (0, self.q_rank, self.q_norm_weight, q_normed)
            # the latent's norm, the rotated part's turn and the cache write (and the queries' latent's norm)
            ops.latent_rope_store(proj, self.latent_col, r, self.rot_dim, rp, self.norm_weight, self.norm_eps, self.rates,
                                  kv.k if cache.write else None, ctx.positions, ctx.request_of_token, table, kv.page_size,
                                  ctx.status, second=second)
            if self.q_rank:
                queries = ws.get("latent_queries", (T, nh * self.q_head), rt.dtype)
                ops.linear(queries, q_normed, self.w_up_q, ctx.status)
            self._per_head(q_latent, queries, self.w_into, None, nh)
            if self.rot_dim:
                ops.rope_norm_store(q_latent, None, None, self.rates, ctx.positions, ctx.request_of_token, table, nh, 0, rp,
                                    r, self.rot_dim, None, rp, kv.page_size, False, False, ctx.status)
        elif ops.latent_prepare_applies(proj, self.qk_dim):
            # few rows: the latent's norm and store and the queries' way into the latent space as one launch
            ops.latent_prepare(q_latent, proj, self.w_into, self.latent_col, r, self.norm_weight, self.norm_eps,
                               kv.k if cache.write else None, ctx.positions, ctx.request_of_token,
                               ctx.block_tables[kv.group], kv.page_size, ctx.status)
        else:
            if cache.write:
                ops.latent_norm_store(proj, self.latent_col, r, self.norm_weight, self.norm_eps, kv.k, ctx.positions,
                                      ctx.request_of_token, ctx.block_tables[kv.group], kv.page_size, ctx.status)
            self._per_head(q_latent, proj[:, :self.q_width], self.w_into, None, nh)
        attended = ws.get("latent_attn", (T, nh * rp), rt.dtype)
        attention_kernels.run(attended, q_latent, ctx, kv, nh, 1, rp, self.reach, self.kernel_scale, self.head_scale,
                              self.head_scale_positive, max_splits=MAX_DECODE_SPLITS)
        heads_out = ws.get("attn", (T, nh * e), rt.dtype)
        gate = proj[:, self.gate_col:self.gate_col + nh] if self.gate_name else None
        self._per_head(heads_out, attended, self.w_out_of, gate, nh)
        return ops.linear_for_residual(heads_out, self.w_o, ws, "mixer_out", ctx.status)
