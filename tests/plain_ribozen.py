"""A plain, slow implementation of the Ribozen decoder for the tests: whole
sequences, no cache, no state carried between calls, one function per
mechanism, on the CPU in the type asked for (float64 as the yardstick).  It
shares no code with the package.

``round_to``: activations are rounded to that type (and widened again) after
every matrix product and after every norm or gate whose output feeds one,
which is where a pipeline that computes in that type rounds; everything the
design keeps 32-bit (the stream, norms, scores, softmax, routers, the
recurrences and what enters them) stays wide.

The model is given as a config dictionary (the keys of config.json) and a
dictionary of tensors by checkpoint name.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces
def _r(x, round_to):
    return x if round_to is None else x.to(round_to).to(x.dtype)


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z):
    return -softplus(-z)


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, n] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([x.new_zeros(n - 1, C), x], dim=0)
    y = sum(padded[j:j + T] * taps[:, j][None, :] for j in range(n))
    return y + bias[None, :]


# ------------------------------------------------------------------ rotary positions
def scaled_rates(dims, base, scaling):
    """The rates of the rotated pairs, i < dims / 2, and the factor on cosines and sines."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.as_tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(scaling["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, dims, base, scaling):
    """x [T, heads, n]: entry i < dims / 2 pairs with entry i + dims / 2."""
    if dims == 0:
        return x
    rates, magnitude = scaled_rates(dims, base, scaling)
    angle = positions.to(torch.float64)[:, None, None] * rates[None, None, :]
    c, s = (torch.cos(angle) * magnitude).to(x.dtype), (torch.sin(angle) * magnitude).to(x.dtype)
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ------------------------------------------------------------------ mixers
def windowed_attention(h, w, p, m, eps, round_to):
    """The left half of the 'parallel' mixer: grouped-query attention with
    biases, a norm over the whole of q and of k, rotate-half positions, capped
    scores, a window that keeps the first tokens, and an output gate."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = _r(h @ w[p + "q"].T + w[p + "q.b"], round_to)
    k = _r(h @ w[p + "k"].T + w[p + "k.b"], round_to)
    v = _r(h @ w[p + "v"].T + w[p + "v.b"], round_to)
    q = unit_rms(q, eps) * w[p + "q.norm"]
    k = unit_rms(k, eps) * w[p + "k.norm"]
    positions = torch.arange(T)
    rot = m["rot"]
    q = _r(rotate_half(q.view(T, H, d), positions, rot["dims"], rot["base"], rot.get("scaling")), round_to)
    k = _r(rotate_half(k.view(T, G, d), positions, rot["dims"], rot["base"], rot.get("scaling")), round_to)
    v = v.view(T, G, e)
    gap = positions[:, None] - positions[None, :]
    seen = gap >= 0
    mask = m.get("mask")
    if mask:
        seen = seen & ((gap < mask["size"]) | (positions[None, :] < mask.get("keep_first", 0)))
    cap = m.get("softcap")
    heads = []
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        if cap:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(~seen, -math.inf)
        heads.append(torch.softmax(s, dim=-1) @ v[:, g])
    o = torch.cat(heads, dim=-1)
    gate = _r(h @ w[p + "g"].T, round_to)
    o = _r(o * torch.sigmoid(gate), round_to)
    return _r(o @ w[p + "o"].T, round_to)


def selective_scan(h, w, p, m, round_to):
    """The right half of the 'parallel' mixer: Mamba's selective scan."""
    T = h.shape[0]
    inner, N, rank = m["inner"], m["state"], m["dt_rank"]
    xz = _r(h @ w[p + "in"].T, round_to)
    x, z = xz[:, :inner], xz[:, inner:]
    x = _r(silu(causal_conv(x, w[p + "conv"], w[p + "conv.b"])), round_to)
    low = _r(x @ w[p + "x"].T, round_to)
    dt_low, B, C = low[:, :rank], low[:, rank:rank + N], low[:, rank + N:]
    dt = softplus(_r(dt_low @ w[p + "dt"].T, round_to) + w[p + "dt.b"])
    A = -torch.exp(w[p + "A_log"])
    S = h.new_zeros(inner, N)
    ys = []
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        ys.append(S @ C[t] + w[p + "D"] * x[t])
    y = torch.stack(ys)
    y = _r(y * silu(z), round_to)
    return _r(y @ w[p + "o"].T, round_to)


def parallel_mixer(h, w, p, m, eps, round_to):
    left = windowed_attention(h, w, p + "left.", m["left"], eps, round_to)
    right = selective_scan(h, w, p + "right.", m["right"], round_to)
    return m["left_scale"] * left + m["right_scale"] * right


def state_space_duality(h, w, p, m, eps, round_to):
    """The 'mamba2' mixer."""
    T = h.shape[0]
    H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * e
    proj = _r(h @ w[p + "in"].T, round_to)
    z = proj[:, :inner]
    xbc = proj[:, inner:2 * inner + 2 * G * N]
    dt = proj[:, 2 * inner + 2 * G * N:]
    xbc = _r(silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"])), round_to)
    x = xbc[:, :inner].view(T, H, e)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"])[None, :] * dt)
    S = h.new_zeros(H, N, e)
    ys = []
    for t in range(T):
        y = []
        for head in range(H):
            g = head // (H // G)
            S[head] = decay[t, head] * S[head] + dt[t, head] * B[t, g][:, None] * x[t, head][None, :]
            y.append(S[head].T @ C[t, g] + w[p + "D"][head] * x[t, head])
        ys.append(torch.cat(y))
    y = torch.stack(ys) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.view(T, parts, inner // parts), eps).reshape(T, inner) * w[p + "norm"]
    return _r(_r(y, round_to) @ w[p + "o"].T, round_to)


def matrix_memory(h, w, p, m, eps, round_to):
    """The 'mlstm' mixer."""
    T = h.shape[0]
    H, d, e, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = _r(h @ w[p + "q"].T, round_to).view(T, H, d) * d ** -0.5
    k = _r(h @ w[p + "k"].T, round_to).view(T, H, d)
    v = _r(h @ w[p + "v"].T, round_to).view(T, H, e)
    i_gate = cap * torch.tanh((_r(h @ w[p + "i"].T, round_to) + w[p + "i.b"]) / cap)
    f_gate = log_sigmoid(cap * torch.tanh((_r(h @ w[p + "f"].T, round_to) + w[p + "f.b"]) / cap))
    outs = []
    for head in range(H):
        S = h.new_zeros(d, e)
        n = h.new_zeros(d)
        m_run = h.new_zeros(())
        rows = []
        for t in range(T):
            m_new = torch.maximum(f_gate[t, head] + m_run, i_gate[t, head])
            keep, take = torch.exp(f_gate[t, head] + m_run - m_new), torch.exp(i_gate[t, head] - m_new)
            S = keep * S + take * k[t, head][:, None] * v[t, head][None, :]
            n = keep * n + take * k[t, head]
            m_run = m_new
            below = torch.maximum(torch.abs(n @ q[t, head]), torch.exp(-m_run)) + 1e-6
            rows.append(S.T @ q[t, head] / below)
        outs.append(unit_rms(torch.stack(rows), eps))
    o = torch.cat(outs, dim=-1) * w[p + "norm"]
    gate = _r(h @ w[p + "g"].T, round_to)
    o = _r(o * torch.sigmoid(gate), round_to)
    return _r(o @ w[p + "o"].T, round_to)


# ------------------------------------------------------------------ feed-forward
def expert(h, w, p, round_to):
    a = _r(silu(_r(h @ w[p + "gate"].T, round_to)) * _r(h @ w[p + "up"].T, round_to), round_to)
    return _r(a @ w[p + "down"].T, round_to)


def routed_experts(h, w, p, mlp, round_to, margins=None):
    """``margins``: a list that receives, per token, how far the last chosen
    router logit lies above the first one not chosen (inf where all are chosen)."""
    experts, top = mlp["router"]["experts"], mlp["router"]["top"]
    logits = h @ w[p + "router"].T
    if margins is not None:
        ordered = torch.sort(logits, dim=-1, descending=True).values
        margins.append(ordered[:, top - 1] - ordered[:, top] if experts > top else torch.full_like(ordered[:, 0], math.inf))
    scores = torch.sigmoid(logits)
    out = torch.zeros_like(h)
    chosen = torch.topk(scores, top, dim=-1).indices
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += expert(_r(scores[t, e] * h[t], round_to)[None, :], w, f"{p}e{e}.", round_to)[0]
    if mlp.get("shared") is not None:
        out = out + expert(h, w, p + "shared.", round_to)
    return out


# ------------------------------------------------------------------ the model
def forward(config, weights, tokens, dtype=torch.float64, round_to=None, layers_out=None, margins_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out``: a list that
    receives the stream after every layer.  ``margins_out``: a list that
    receives every routed layer's margins (see routed_experts)."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = config["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * config["embedding"]["scale"]

    def norm(x, name):
        return _r(unit_rms(x, eps) * w[name], round_to)

    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        h = norm(x, p + "norm1")
        kind, m = layer["type"], layer["mixer"]
        if kind == "mlstm":
            y = matrix_memory(h, w, p + "mix.", m, eps, round_to)
        elif kind == "mamba2":
            y = state_space_duality(h, w, p + "mix.", m, eps, round_to)
        elif kind == "parallel":
            y = parallel_mixer(h, w, p + "mix.", m, eps, round_to)
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        x = x + y * w[p + "ls1"]
        if layer.get("mlp") is not None:
            h = norm(x, p + "norm2")
            x = x + routed_experts(h, w, p + "mlp.", layer["mlp"], round_to, margins_out) * w[p + "ls2"]
        if layers_out is not None:
            layers_out.append(x.clone())
    return norm(x, "final.norm") @ w["head"].T


def greedy(config, weights, prompt, n):
    ids = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(config, weights, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out


# ------------------------------------------------------------------ tensors
def tensor_shapes(config):
    W, V = config["width"], config["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,), "head": (V, W)}
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "ls1"] = (W,)
        q = p + "mix."
        if layer["type"] == "mlstm":
            H, d, e = m["heads"], m["dim"], m["vdim"]
            shapes.update({q + "q": (H * d, W), q + "k": (H * d, W), q + "v": (H * e, W), q + "g": (H * e, W),
                           q + "o": (W, H * e), q + "norm": (H * e,), q + "i": (H, W), q + "i.b": (H,), q + "f": (H, W),
                           q + "f.b": (H,)})
        elif layer["type"] == "mamba2":
            H, e, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, C = H * e, H * e + 2 * G * N
            shapes.update({q + "in": (2 * inner + 2 * G * N + H, W), q + "conv": (C, m["conv"]), q + "conv.b": (C,),
                           q + "dt_bias": (H,), q + "A_log": (H,), q + "D": (H,), q + "norm": (inner,), q + "o": (W, inner)})
        else:
            a, s = m["left"], m["right"]
            H, G, d, e = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
            l, r = q + "left.", q + "right."
            shapes.update({l + "q": (H * d, W), l + "q.b": (H * d,), l + "k": (G * d, W), l + "k.b": (G * d,),
                           l + "v": (G * e, W), l + "v.b": (G * e,), l + "q.norm": (H * d,), l + "k.norm": (G * d,),
                           l + "g": (H * e, W), l + "o": (W, H * e)})
            C, N, R = s["inner"], s["state"], s["dt_rank"]
            shapes.update({r + "in": (2 * C, W), r + "conv": (C, s["conv"]), r + "conv.b": (C,), r + "x": (R + 2 * N, C),
                           r + "dt": (C, R), r + "dt.b": (C,), r + "A_log": (C, N), r + "D": (C,), r + "o": (W, C)})
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = shapes[p + "ls2"] = (W,)
            F = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{p}mlp.e{e}.gate": (F, W), f"{p}mlp.e{e}.up": (F, W), f"{p}mlp.e{e}.down": (W, F)})
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
            if mlp.get("shared") is not None:
                S = mlp["shared"]["ff"]
                shapes.update({p + "mlp.shared.gate": (S, W), p + "mlp.shared.up": (S, W), p + "mlp.shared.down": (W, S)})
    return shapes


def random_weights(config, seed, sharp=3.0):
    """Values of bfloat16 precision (so that a folder stored in either type
    holds the same model).  Matrices N(0, 1 / fan-in) times a factor; norm
    weights of queries and keys are large enough that single keys decide a
    softmax (``sharp``: roughly the spread of the scores before the config's
    scale); step sizes and decays are spread so that some channels remember
    hundreds of tokens and others a few; routers are wide apart."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(config).items():
        tail = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        n = lambda *s: torch.randn(s or shape, generator=g)
        u = lambda lo, hi: lo + (hi - lo) * torch.rand(shape, generator=g)
        if tail in ("norm1", "norm2", "mix.norm") or name == "final.norm":
            t = 1.0 + 0.2 * n()
        elif tail in ("ls1", "ls2"):
            t = u(0.4, 1.3)
        elif tail in ("mix.left.q.norm", "mix.left.k.norm"):
            t = math.sqrt(sharp) * (1.0 + 0.3 * n())
        elif tail.endswith("conv"):
            t = 0.6 * n()
        elif tail == "mix.A_log":
            t = u(-4.0, 0.5)
        elif tail == "mix.right.A_log":
            t = u(-3.0, 1.0)
        elif tail in ("mix.dt_bias", "mix.right.dt.b"):
            t = u(-4.0, 0.0)
        elif tail in ("mix.D", "mix.right.D"):
            t = 1.0 + 0.3 * n()
        elif tail == "mix.f.b":
            t = u(1.0, 5.0)
        elif len(shape) == 1:
            t = 0.3 * n()
        elif name == "embed":
            t = n()
        else:
            t = n() / math.sqrt(shape[1])
            if tail == "mlp.router":
                t = t * 4.0
            if tail.endswith(".o") or tail.endswith(".down"):
                t = t * 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float64)
    return out
