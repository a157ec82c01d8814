"""Routed experts: every token goes through ``top`` of ``experts`` small gated
feed-forward layers, chosen by a router, plus (optionally) a shared expert
that every token uses.

    z = Wr h + br                      router logits, 32-bit
    chosen = the top largest z         (ties: the lower index)
    p = softmax over the chosen z only          (``scoring`` "softmax_chosen")
        or sigmoid(z) of each chosen one alone  (``scoring`` "sigmoid")
    y = sum_j p_j * expert_{chosen_j}(h)  [+ sigmoid(sg . h) * shared(h)]     (``weight_on`` "output")
        or sum_j expert_{chosen_j}(p_j * h)  [+ ...]                          (``weight_on`` "input")
    expert(h) = Wd (act(Wg h) * (Wu h)),  no biases

A weight on the input reaches the activation through both of the expert's
first products, which are linear: act(p * (Wg h)) * (p * (Wu h)), taken in 32
bits in those products' epilogues (the tensor-core path over sorted rows
multiplies the gathered rows instead).

The (token, choice) pairs are sorted by expert on the device (no number of
the step ever reaches the host, so a step's shape is fixed by its rows and it
can be captured), the experts' products run over the sorted groups, and a last
kernel adds each token's outputs in the order of its choices.
"""
from __future__ import annotations

import torch

from .. import ops
from .base import FEED_FORWARDS, FeedForward, PartSpec, TensorDecl, register_feed_forward

ACTIVATIONS = {"silu": (ops.GLU_SILU, 1.0, 0.0), "relu": (ops.GLU_RELU, 1.0, 0.0)}
SCORINGS = {"softmax_chosen": ops.MOE_SOFTMAX_CHOSEN, "sigmoid": ops.MOE_SIGMOID}


@register_feed_forward("routed_experts")
class RoutedExperts(FeedForward):
    def __init__(self, hidden_size: int, intermediate_size: int, num_experts: int, top: int, router_name: str,
                 router_bias_name: str | None, expert_names: str, activation: str = "silu", shared: PartSpec | None = None,
                 shared_gate_name: str | None = None, scoring: str = "softmax_chosen", weight_on: str = "output"):
        """``expert_names``: a pattern with ``{expert}`` and ``{part}`` (gate, up, down)."""
        self.hidden_size, self.intermediate_size = int(hidden_size), int(intermediate_size)
        self.num_experts, self.top = int(num_experts), int(top)
        if not 1 <= self.top <= self.num_experts:
            raise ValueError(f"a token uses 1 to {num_experts} experts, got {top}")
        if activation not in ACTIVATIONS:
            raise ValueError(f"unknown expert activation {activation!r} (known: {', '.join(sorted(ACTIVATIONS))})")
        self.activation = ACTIVATIONS[activation]
        if scoring not in SCORINGS:
            raise ValueError(f"unknown router scoring {scoring!r} (known: {', '.join(sorted(SCORINGS))})")
        if weight_on not in ("output", "input"):
            raise ValueError(f"an expert's weight sits on its 'output' or its 'input', not on {weight_on!r}")
        self.scoring, self.weight_on_input = SCORINGS[scoring], weight_on == "input"
        self.router_name, self.router_bias_name, self.expert_names = router_name, router_bias_name, expert_names
        self.shared = FEED_FORWARDS.build(shared) if shared is not None else None
        self.shared_gate_name = shared_gate_name if shared is not None else None
        self.w_router = self.b_router = self.w_gate_up = self.w_down = self.w_shared_gate = None
        self.runtime = None

    def _name(self, expert: int, part: str) -> str:
        return self.expert_names.format(expert=expert, part=part)

    def tensors(self):
        W, F, E = self.hidden_size, self.intermediate_size, self.num_experts
        decls = [TensorDecl(self.router_name, (E, W), role="vector", init="normal")]
        if self.router_bias_name:
            decls.append(TensorDecl(self.router_bias_name, (E,), role="vector", init="zeros"))
        for e in range(E):
            decls += [TensorDecl(self._name(e, "gate"), (F, W)), TensorDecl(self._name(e, "up"), (F, W)),
                      TensorDecl(self._name(e, "down"), (W, F))]
        if self.shared is not None:
            decls += self.shared.tensors()
            if self.shared_gate_name:
                decls.append(TensorDecl(self.shared_gate_name, (1, W), role="vector", init="normal"))
        return decls

    def bind(self, get, runtime):
        E = self.num_experts
        self.w_router = get(self.router_name).contiguous()
        self.b_router = get(self.router_bias_name).contiguous() if self.router_bias_name else None
        self.w_gate_up = torch.stack([torch.cat([get(self._name(e, "gate")), get(self._name(e, "up"))], dim=0)
                                      for e in range(E)]).contiguous()
        self.w_down = torch.stack([get(self._name(e, "down")) for e in range(E)]).contiguous()
        if self.shared is not None:
            self.shared.bind(get, runtime)
            if self.shared_gate_name:
                self.w_shared_gate = get(self.shared_gate_name).reshape(-1).contiguous()
        self.runtime = runtime

    def forward(self, x, ctx):
        rt = self.runtime
        ws = ctx.workspace
        T, W, F, E, top = x.shape[0], self.hidden_size, self.intermediate_size, self.num_experts, self.top
        pairs = T * top
        ids = ws.get("moe_ids", (T, top), torch.int32)
        share = ws.get("moe_share", (T, top), torch.float32)
        gate = ws.get("moe_shared_gate", (T,), torch.float32) if self.w_shared_gate is not None else None
        logits = ws.get("moe_logits", (T * (E + 1),), torch.float32)
        ops.moe_route(ids, share, gate, x, self.w_router, self.b_router, self.w_shared_gate, top, scratch=logits,
                      scoring=self.scoring)
        on_input = self.weight_on_input
        wide = ops.moe_wide_tiles(pairs, E, rt.dtype, W, F)
        max_tiles = ops.moe_max_tiles(pairs, E, wide)
        tiles = ws.get("moe_tiles", (3, max_tiles), torch.int32)
        meta = ws.get("moe_meta", (4,), torch.int32)
        shared_out = self.shared.forward_plain(x, ctx) if self.shared is not None else None
        out = ws.get("ffn_out", (T, W), rt.dtype)
        if wide and ops.TC_EXPERTS and ops.tc_applies(x, self.w_gate_up[0]):
            # many rows per expert: whole tiles of 128 sorted rows through the tcgen05 product
            rows = max_tiles * ops.moe_tile_rows(True)
            slot_pair = ws.get("moe_slots", (rows,), torch.int32)
            pair_slot = ws.get("moe_pair_slots", (pairs,), torch.int32)
            ops.moe_group(ids, E, slot_pair, tiles, meta, True, padded=True, pair_slot=pair_slot)
            x_sorted = ws.get("moe_x_sorted", (rows, W), rt.dtype)
            ops.moe_gather(x_sorted, x, slot_pair, meta, top, pair_weight=share.view(-1) if on_input else None)
            act = ws.get("moe_act", (rows, F), rt.dtype)
            ops.gemm_tc_grouped(act, x_sorted, self.w_gate_up, tiles[0], meta, gated=True, status=ctx.status,
                                activation=self.activation)
            y = ws.get("moe_y_sorted", (rows, W), rt.dtype)
            ops.gemm_tc_grouped(y, act, self.w_down, tiles[0], meta, status=ctx.status)
            ops.moe_combine_sorted(out, y, pair_slot, None if on_input else share, top, shared_out, gate)
            return out
        slot_pair = ws.get("moe_slots", (pairs,), torch.int32)
        ops.moe_group(ids, E, slot_pair, tiles, meta, wide)
        act = ws.get("moe_act", (pairs, F), rt.dtype)
        ops.moe_grouped(act, x, self.w_gate_up, slot_pair, tiles, meta, max_tiles, src_div=top, scatter=False, gated=True,
                        pair_weight=share.view(-1) if on_input else None, activation=self.activation, wide=wide)
        y = ws.get("moe_y", (pairs, W), torch.float32)
        ops.moe_grouped(y, act, self.w_down, slot_pair, tiles, meta, max_tiles, src_div=0, scatter=True,
                        pair_weight=None if on_input else share.view(-1), wide=wide)
        ops.moe_combine(out, y, top, shared_out, gate)
        return out
