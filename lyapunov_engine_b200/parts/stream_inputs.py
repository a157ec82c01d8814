"""Inputs that enter the residual stream beside the layers' sub-layers.

"gated_token_embedding": every token brings a small embedding of its own for
the layer, e = table[id, col : col + dim].  With x the stream as the layer's
sub-layers left it,
    g = gelu_tanh(Wg x) * e,    y = Wp g,    x <- x + y / sqrt(mean(y^2) + eps) * w
(the tanh form of gelu; the norm has a plain weight).  The last step is not a
launch of its own: y stays pending as a ``NormedAddend`` and the next norm's
kernel lets it in.

"pass_entry": x[t] <- x[t] + E[id_t] + v, what a pass over a stretch of layers
adds before its first layer: the embedding's output again (``embedding_name``
None: not) and row ``row`` of a table of vectors [rows, W] (one per pass).
"""
from __future__ import annotations

import torch

from .. import ops
from .base import NormedAddend, StreamInput, TensorDecl, register_stream_input


@register_stream_input("gated_token_embedding")
class GatedTokenEmbedding(StreamInput):
    reads_stream = True

    def __init__(self, hidden_size: int, vocab_size: int, dim: int, table_name: str, table_width: int, col: int,
                 gate_name: str, proj_name: str, norm_name: str, eps: float):
        self.hidden_size, self.vocab_size, self.dim = int(hidden_size), int(vocab_size), int(dim)
        self.table_width, self.col = int(table_width), int(col)
        if not 0 <= self.col <= self.table_width - self.dim:
            raise ValueError(f"columns {col}..{col + dim} lie outside a table of {table_width} columns")
        self.names = (table_name, gate_name, proj_name, norm_name)
        self.eps = float(eps)
        self.table = self.w_gate = self.w_proj = self.addend = None
        self.runtime = None

    def tensors(self):
        table, gate, proj, norm = self.names
        return [TensorDecl(table, (self.vocab_size, self.table_width)), TensorDecl(gate, (self.dim, self.hidden_size)),
                TensorDecl(proj, (self.hidden_size, self.dim)),
                TensorDecl(norm, (self.hidden_size,), role="vector", init="ones_jitter")]

    def bind(self, get, runtime):
        table, gate, proj, norm = self.names
        self.table, self.w_gate, self.w_proj = get(table), get(gate), get(proj)
        self.addend = NormedAddend(get(norm), self.eps)
        self.runtime = runtime

    def forward(self, stream, ctx, copy=None) -> None:
        if stream.pending is not None or copy is None:
            raise ValueError("the gated token embedding reads a stream with nothing pending, as rows in the activations' type")
        ws = ctx.workspace
        T = copy.shape[0]
        z = ws.get("token_gate", (T, self.dim), self.runtime.dtype)
        ops.linear(z, copy, self.w_gate, ctx.status)
        g = ws.get("token_gated", (T, self.dim), self.runtime.dtype)
        ops.gate_rows(g, z, self.table, self.col, ctx.token_ids, ctx.status)
        stream.pending = ops.linear_for_residual(g, self.w_proj, ws, "token_input", ctx.status)
        stream.update = self.addend


@register_stream_input("pass_entry")
class PassEntry(StreamInput):
    def __init__(self, hidden_size: int, vocab_size: int, embedding_name: str | None, vector_name: str | None,
                 vector_rows: int = 0, row: int = 0):
        self.hidden_size, self.vocab_size = int(hidden_size), int(vocab_size)
        self.embedding_name, self.vector_name = embedding_name, vector_name
        self.vector_rows, self.row = int(vector_rows), int(row)
        if vector_name is not None and not 0 <= self.row < self.vector_rows:
            raise ValueError(f"row {row} of a table of {vector_rows} vectors")
        self.table = self.vector = None

    def tensors(self):
        decls = []
        if self.embedding_name is not None:
            decls.append(TensorDecl(self.embedding_name, (self.vocab_size, self.hidden_size)))
        if self.vector_name is not None:
            decls.append(TensorDecl(self.vector_name, (self.vector_rows, self.hidden_size), role="vector", init="taps"))
        return decls

    def bind(self, get, runtime):
        self.table = get(self.embedding_name) if self.embedding_name is not None else None
        self.vector = get(self.vector_name)[self.row].contiguous() if self.vector_name is not None else None

    def forward(self, stream, ctx, copy=None) -> None:
        # (an addition: it commutes with whatever is still pending)
        if stream.copies != 1:
            raise ValueError("a pass entry adds to a stream in one copy")
        if self.table is not None or self.vector is not None:
            ops.stream_entry(stream.resid, self.table, ctx.token_ids, self.vector, ctx.status)
