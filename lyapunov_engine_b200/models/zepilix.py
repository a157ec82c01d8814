"""The Zepilix decoder as a description: which parts, with which numbers and
tensor names, in which order.

Token embedding; layers in the parallel arrangement, x <- x + (mixer(norm1(x))
+ ff(norm2(x))), with RMS norms whose weights are stored around zero (factor 1
+ w); after the sub-layers of every layer a small embedding per token and layer
enters behind a gelu gate and a norm (``token_side``); the mixer is the gated
delta rule (a matrix of state per head, short convolutions on q, k, v),
grouped-query attention whose values are the keys (rotary positions on
neighbouring pairs, a weightless norm on queries and keys after the turn), or
latent attention with a query latent, a rotated key part shared by the heads
and a sliding window; the feed-forward is silu-gated with biases.  A stretch of
consecutive layers may run several times in a row, each pass with a cache and
state of its own (the run order names those layers again); before every pass
but the first the embedding's output is added to the stream again, and before
every pass a learned vector of that pass.  The last norm is the model's, the
head is the embedding matrix.  Tensor names: ``embed``, ``loop.step``,
``side.embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*[.b]``,
``l<i>.side.gate|proj|norm``, ``final.norm``.
"""
from __future__ import annotations

from ..config.zepilix import ZepilixConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, RunSpec

# Positions are computed, not looked up: the limit is where a float32 stops counting exactly.
MAX_POSITIONS = 1 << 24


def zepilix_spec(raw_config: dict) -> ModelSpec:
    c = ZepilixConfig.from_dict(raw_config)
    W = c.width

    def norm(name):
        return PartSpec("rmsnorm", {"hidden_size": W, "eps": c.norm_eps, "weight_name": name, "offset": 1.0})

    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        m = layer.mixer
        if m.kind == "delta":
            mixer = PartSpec("gated_delta", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "taps": m.taps, "norm_eps": c.norm_eps, "q_name": p + "mix.q", "k_name": p + "mix.k", "v_name": p + "mix.v",
                "beta_name": p + "mix.b", "decay_name": p + "mix.a", "gate_name": p + "mix.g", "o_name": p + "mix.o",
                "a_log_name": p + "mix.A_log", "dt_bias_name": p + "mix.dt_bias", "norm_name": p + "mix.norm"})
        elif m.kind == "attention":
            position = PartSpec("rotary_pairs", {"head_dim": m.dim, "rot": m.rot_dims, "base": m.rot_base,
                                                 "unit_eps": c.norm_eps})
            mixer = PartSpec("attention", {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "position": position,
                "q_name": p + "mix.q", "k_name": p + "mix.k", "v_name": None, "o_name": p + "mix.o", "scale": m.scale})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "value_dim": m.vdim, "latent_dim": m.kv_rank,
                "scale": m.scale, "norm_eps": c.norm_eps, "q_name": p + "mix.uq", "down_name": p + "mix.dkv",
                "latent_norm_name": p + "mix.dkv.norm", "up_k_name": p + "mix.uk", "up_v_name": p + "mix.uv",
                "o_name": p + "mix.o", "window": m.window or None, "rot_dim": m.rot_dim, "rot_base": m.rot_base,
                "q_rank": m.q_rank, "q_down_name": p + "mix.dq", "q_norm_name": p + "mix.dq.norm"})
        feed_forward = None
        if layer.ff:
            feed_forward = PartSpec("gated_silu", {"hidden_size": W, "intermediate_size": layer.ff, "gate_name": p + "mlp.gate",
                                                   "up_name": p + "mlp.up", "down_name": p + "mlp.down", "bias_suffix": ".b"})
        after = None
        if c.side_dim:
            after = PartSpec("gated_token_embedding", {
                "hidden_size": W, "vocab_size": c.vocab, "dim": c.side_dim, "table_name": "side.embed",
                "table_width": c.side_dim * len(c.layers), "col": i * c.side_dim, "gate_name": p + "side.gate",
                "proj_name": p + "side.proj", "norm_name": p + "side.norm", "eps": c.norm_eps})
        layers.append(LayerSpec(PartSpec("parallel", {
            "mixer": mixer, "feed_forward": feed_forward, "mixer_norm": norm(p + "norm1"),
            "feed_forward_norm": norm(p + "norm2") if feed_forward is not None else None, "after": after})))
    times = c.loop[2] if c.loop is not None else 0
    run_order = []
    for layer, opens in c.passes():
        entry = None
        if opens is not None:
            entry = PartSpec("pass_entry", {"hidden_size": W, "vocab_size": c.vocab,
                                            "embedding_name": "embed" if opens > 0 else None, "vector_name": "loop.step",
                                            "vector_rows": times, "row": opens})
        run_order.append(RunSpec(layer, entry=entry))
    return ModelSpec(
        architecture=c.architecture,
        hidden_size=W,
        vocab_size=c.vocab,
        max_positions=MAX_POSITIONS,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed"}),
        layers=tuple(layers),
        run_order=tuple(run_order),
        final_norm=norm("final.norm"),
        head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": W, "weight_name": "embed", "tied_to": None}),
        config_json=dict(c.raw),
    )
