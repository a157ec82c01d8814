"""The Ribozen decoder as a description: which parts, with which numbers and
tensor names, in which order.

Token embedding times a constant; pre-norm layers, x <- x + s1 * mixer(norm1(x));
x <- x + s2 * ff(norm2(x)), with RMS norms and a learned factor per column on
each sub-layer's output (``ls1``, ``ls2``).  The mixer is the mLSTM's matrix
memory, a state-space-duality layer (Mamba-2), or two mixers side by side on
the same input: grouped-query attention with biases, a norm over the whole of q
and of k, rotate-half positions with ramped rates, capped scores, a sliding
window that keeps the first keys and a gate per output entry, beside a
selective scan (Mamba), their outputs added with a constant each.  The
feed-forward is routed experts whose weights are the chosen scores' sigmoids,
unnormalized, applied to the expert's input, plus a shared expert.  The last
norm is the model's; the head is a matrix of its own.  Tensor names: ``embed``,
``l<i>.norm1|norm2|ls1|ls2``, ``l<i>.mix.*``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.ribozen import RibozenConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

# Positions are computed, not looked up: the limit is where a float32 stops counting exactly.
MAX_POSITIONS = 1 << 24


def ribozen_spec(raw_config: dict) -> ModelSpec:
    c = RibozenConfig.from_dict(raw_config)
    W = c.width

    def norm(name):
        return PartSpec("rmsnorm", {"hidden_size": W, "eps": c.norm_eps, "weight_name": name})

    def gated(prefix, ff):
        return PartSpec("gated_silu", {"hidden_size": W, "intermediate_size": ff, "gate_name": prefix + "gate",
                                       "up_name": prefix + "up", "down_name": prefix + "down"})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}.mix."
        m = layer.mixer
        if layer.kind == "mlstm":
            mixer = PartSpec("matrix_memory", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "gate_cap": m.gate_cap,
                "norm_eps": c.norm_eps, "q_name": p + "q", "k_name": p + "k", "v_name": p + "v", "gate_name": p + "g",
                "input_gate_name": p + "i", "forget_gate_name": p + "f", "norm_name": p + "norm", "o_name": p + "o"})
        elif layer.kind == "mamba2":
            mixer = PartSpec("state_space_duality", {
                "hidden_size": W, "num_heads": m.heads, "value_dim": m.vdim, "state_dim": m.state, "groups": m.groups,
                "taps": m.taps, "norm_groups": m.norm_groups, "norm_eps": c.norm_eps, "in_name": p + "in",
                "conv_name": p + "conv", "conv_bias_name": p + "conv.b", "dt_bias_name": p + "dt_bias",
                "a_log_name": p + "A_log", "d_name": p + "D", "norm_name": p + "norm", "o_name": p + "o"})
        else:
            a, s = m.left, m.right
            l, r = p + "left.", p + "right."
            scaling = None
            if a.rot_scaling is not None:
                scaling = {"factor": a.rot_scaling.factor, "original": a.rot_scaling.original, "fast": a.rot_scaling.fast,
                           "slow": a.rot_scaling.slow}
            position = PartSpec("rotary_normed", {
                "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim, "rot": a.rot_dims,
                "base": a.rot_base, "scaling": scaling, "norm_eps": c.norm_eps, "q_norm_name": l + "q.norm",
                "k_norm_name": l + "k.norm", "bias_names": (l + "q.b", l + "k.b", l + "v.b")})
            attention = PartSpec("attention", {
                "hidden_size": W, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
                "position": position, "q_name": l + "q", "k_name": l + "k", "v_name": l + "v", "o_name": l + "o",
                "window": a.window or None, "keep_first": a.keep_first, "scale": a.scale, "softcap": a.softcap or None,
                "gate_name": l + "g", "gate_per_entry": True})
            scan = PartSpec("selective_scan", {
                "hidden_size": W, "inner": s.inner, "state_dim": s.state, "dt_rank": s.dt_rank, "taps": s.taps,
                "in_name": r + "in", "conv_name": r + "conv", "conv_bias_name": r + "conv.b", "x_name": r + "x",
                "dt_name": r + "dt", "dt_bias_name": r + "dt.b", "a_log_name": r + "A_log", "d_name": r + "D", "o_name": r + "o"})
            mixer = PartSpec("side_by_side", {"hidden_size": W, "mixers": (attention, scan),
                                              "scales": (m.left_scale, m.right_scale)})
        feed_forward = None
        f = layer.feed_forward
        q = f"l{i}.mlp."
        if f is not None:
            feed_forward = PartSpec("routed_experts", {
                "hidden_size": W, "intermediate_size": f.ff, "num_experts": f.experts, "top": f.top,
                "router_name": q + "router", "router_bias_name": None, "expert_names": q + "e{expert}.{part}",
                "activation": "silu", "shared": gated(q + "shared.", f.shared_ff) if f.shared_ff else None,
                "shared_gate_name": None, "scoring": "sigmoid", "weight_on": "input"})
        layers.append(LayerSpec(PartSpec("prenorm", {
            "mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(f"l{i}.norm1"),
            "feed_forward_norm": norm(f"l{i}.norm2") if feed_forward is not None else None,
            "mixer_scale_name": f"l{i}.ls1", "feed_forward_scale_name": f"l{i}.ls2" if feed_forward is not None else None})))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=W,
        vocab_size=c.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed",
                                               "scale": c.embedding_scale}),
        layers=tuple(layers),
        run_order=tuple(RunSpec(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "head", "tied_to": None}),
        config_json=dict(c.raw),
    )
