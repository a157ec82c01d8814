"""A plain, slow implementation of the Zepilix decoder for the tests: whole
sequences, no cache, no state carried between calls, one function per
mechanism, on the CPU in the type asked for (float64 as the yardstick).  It
shares no code with the package.

``round_to``: activations are rounded to that type (and widened again) after
every matrix product and after every norm whose output feeds one, which is
where a pipeline that computes in that type rounds; everything the design
keeps 32-bit (the stream, norms, scores, softmax, the recurrence) stays wide.
"""
from __future__ import annotations

import math

import torch


# ------------------------------------------------------------------ small pieces
def _r(x, round_to):
    return x if round_to is None else x.to(round_to).to(x.dtype)


def unit_rms(x, eps):
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x, w, eps):
    """x / rms(x) * (1 + w): the model's norm, its weight stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z.pow(3))))


def turn_pairs(x, positions, rot, base):
    """x [T, heads, n]: entries (2i, 2i + 1) below ``rot`` turn by positions * base^(-2i / rot)."""
    if rot == 0:
        return x
    i = torch.arange(rot // 2, dtype=x.dtype)
    rates = torch.as_tensor(base, dtype=x.dtype) ** (-2.0 * i / rot)
    angle = positions.to(x.dtype)[:, None, None] * rates[None, None, :]
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = x[..., 0:rot:2], x[..., 1:rot:2]
    out = x.clone()
    out[..., 0:rot:2] = a * c - b * s
    out[..., 1:rot:2] = b * c + a * s
    return out


def conv_silu(x, taps):
    """x [T, C], taps [C, n] with the last column the current token's; zeros before the start."""
    T, C = x.shape
    n = taps.shape[1]
    padded = torch.cat([x.new_zeros(n - 1, C), x], dim=0)
    y = sum(padded[j:j + T] * taps[:, j][None, :] for j in range(n))
    return silu(y)


def softmax_attention(q, k, v, scale, window=None):
    """q [T, d], k [T, d], v [T, e]; position i sees j <= i (and i - j < window)."""
    T = q.shape[0]
    i = torch.arange(T)
    gap = i[:, None] - i[None, :]
    seen = gap >= 0
    if window:
        seen = seen & (gap < window)
    s = (q @ k.T) * scale
    s = s.masked_fill(~seen, -math.inf)
    return torch.softmax(s, dim=-1) @ v


# ------------------------------------------------------------------ mixers
def delta_rule_head(q, k, v, g, beta):
    """One head of the gated delta rule, token by token.  q, k [T, d] (already
    unit vectors), v [T, e], g and beta [T]."""
    T, d = q.shape
    S = q.new_zeros(d, v.shape[1])
    out = []
    for t in range(T):
        S = g[t] * S
        u = beta[t] * (v[t] - S.T @ k[t])
        S = S + torch.outer(k[t], u)
        out.append(S.T @ q[t])
    return torch.stack(out)


def delta_mixer(h, w, p, m, eps, round_to=None):
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    lin = lambda name: _r(h @ w[p + name].T, round_to)
    q = _r(conv_silu(lin("q"), w[p + "q.conv"]), round_to).view(T, G, d)
    k = _r(conv_silu(lin("k"), w[p + "k.conv"]), round_to).view(T, G, d)
    v = _r(conv_silu(lin("v"), w[p + "v.conv"]), round_to).view(T, H, e)
    q = q / torch.sqrt(q.pow(2).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt(k.pow(2).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(lin("b"))
    g = torch.exp(-torch.exp(w[p + "A_log"])[None] * torch.nn.functional.softplus(lin("a") + w[p + "dt_bias"][None]))
    gate = silu(lin("g")).view(T, H, e)
    heads = [delta_rule_head(q[:, j // (H // G)], k[:, j // (H // G)], v[:, j], g[:, j], beta[:, j]) for j in range(H)]
    o = torch.stack(heads, dim=1)
    o = _r(unit_rms(o, eps) * w[p + "norm"][None, None, :] * gate, round_to)
    return _r(o.reshape(T, H * e) @ w[p + "o"].T, round_to)


def attention_mixer(h, w, p, m, eps, positions, round_to=None):
    """Grouped queries; the values are the keys as projected; queries and keys
    are turned, then divided by their root mean square."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = _r(h @ w[p + "q"].T, round_to).view(T, H, d)
    k = _r(h @ w[p + "k"].T, round_to).view(T, G, d)
    v = k
    q = _r(unit_rms(turn_pairs(q, positions, m["rot"]["dims"], m["rot"]["base"]), eps), round_to)
    k = _r(unit_rms(turn_pairs(k, positions, m["rot"]["dims"], m["rot"]["base"]), eps), round_to)
    heads = [softmax_attention(q[:, j], k[:, j // (H // G)], v[:, j // (H // G)], m["scale"]) for j in range(H)]
    o = _r(torch.stack(heads, dim=1), round_to)
    return _r(o.reshape(T, H * d) @ w[p + "o"].T, round_to)


def latent_mixer(h, w, p, m, eps, positions, round_to=None):
    T = h.shape[0]
    H, d, rd, e, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = _r(unit_rms(_r(h @ w[p + "dq"].T, round_to), eps) * w[p + "dq.norm"][None], round_to)
    q = _r(cq @ w[p + "uq"].T, round_to).view(T, H, d + rd)
    down = _r(h @ w[p + "dkv"].T, round_to)
    c = _r(unit_rms(down[:, :r], eps) * w[p + "dkv.norm"][None], round_to)
    q_turned = turn_pairs(q[..., d:].contiguous(), positions, rd, m["rot"]["base"])
    k_turned = turn_pairs(down[:, r:].reshape(T, 1, rd), positions, rd, m["rot"]["base"])[:, 0]
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, e)
    window = m["mask"]["size"] if m.get("mask") else None
    heads = []
    for j in range(H):
        qj = torch.cat([q[:, j, :d], q_turned[:, j]], dim=-1)
        kj = torch.cat([k_plain[:, j], k_turned], dim=-1)
        heads.append(softmax_attention(qj, kj, v[:, j], m["scale"], window))
    o = _r(torch.stack(heads, dim=1), round_to)
    return _r(o.reshape(T, H * e) @ w[p + "o"].T, round_to)


def dense_feed_forward(h, w, p, round_to=None):
    g = h @ w[p + "gate"].T + w[p + "gate.b"]
    u = h @ w[p + "up"].T + w[p + "up.b"]
    return (_r(silu(g) * u, round_to) @ w[p + "down"].T) + w[p + "down.b"]


def token_side(x, w, p, ids, col, dim, eps, round_to=None):
    e = w["side.embed"][ids][:, col:col + dim]
    z = _r(_r(x, round_to) @ w[p + "side.gate"].T, round_to)
    y = _r(gelu_tanh(z) * e, round_to) @ w[p + "side.proj"].T
    return x + unit_rms(y, eps) * w[p + "side.norm"][None]


# ------------------------------------------------------------------ the model
def passes(cfg):
    """(layer, number of the pass this run opens or None) in run order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def run_order(cfg):
    return [i for i, _ in passes(cfg)]


def forward(cfg, weights, ids, dtype=torch.float64, round_to=None, layers_out=None):
    """Logits [T, vocab] for the whole sequence ``ids``."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(len(ids))
    x0 = w["embed"][ids]
    x = x0.clone()
    side = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    for i, opens in passes(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + w["loop.step"][opens][None]
        h1 = _r(offset_norm(x, w[p + "norm1"], eps), round_to)
        kind, m = layer["type"], layer["mixer"]
        if kind == "delta":
            a = delta_mixer(h1, w, p + "mix.", m, eps, round_to)
        elif kind == "attention":
            a = attention_mixer(h1, w, p + "mix.", m, eps, positions, round_to)
        else:
            a = latent_mixer(h1, w, p + "mix.", m, eps, positions, round_to)
        f = 0.0
        if layer.get("mlp"):
            f = dense_feed_forward(_r(offset_norm(x, w[p + "norm2"], eps), round_to), w, p + "mlp.", round_to)
        x = x + (a + f)
        if side:
            x = token_side(x, w, p, ids, i * side, side, eps, round_to)
        if layers_out is not None:
            layers_out.append(x.clone())
    return _r(offset_norm(x, w["final.norm"], eps), round_to) @ w["embed"].T


def greedy(cfg, weights, prompt, n):
    ids = list(prompt)
    out = []
    for _ in range(n):
        nxt = int(forward(cfg, weights, ids)[-1].argmax())
        out.append(nxt)
        ids.append(nxt)
    return out


# ------------------------------------------------------------------ tensors
def tensor_shapes(cfg):
    W, V = cfg["width"], cfg["vocab"]
    shapes = {"embed": (V, W), "final.norm": (W,)}
    if cfg.get("loop"):
        shapes["loop.step"] = (cfg["loop"]["times"], W)
    side = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    if side:
        shapes["side.embed"] = (V, side * len(cfg["layers"]))
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "delta":
            H, G, d, e, n = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["conv"]
            shapes.update({p + "mix.q": (G * d, W), p + "mix.k": (G * d, W), p + "mix.v": (H * e, W),
                           p + "mix.q.conv": (G * d, n), p + "mix.k.conv": (G * d, n), p + "mix.v.conv": (H * e, n),
                           p + "mix.b": (H, W), p + "mix.a": (H, W), p + "mix.g": (H * e, W), p + "mix.o": (W, H * e),
                           p + "mix.A_log": (H,), p + "mix.dt_bias": (H,), p + "mix.norm": (e,)})
        elif layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            shapes.update({p + "mix.q": (H * d, W), p + "mix.k": (G * d, W), p + "mix.o": (W, H * d)})
        else:
            H, d, rd, e, r, qr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"], m["q_rank"]
            shapes.update({p + "mix.dq": (qr, W), p + "mix.dq.norm": (qr,), p + "mix.uq": (H * (d + rd), qr),
                           p + "mix.dkv": (r + rd, W), p + "mix.dkv.norm": (r,), p + "mix.uk": (H * d, r),
                           p + "mix.uv": (H * e, r), p + "mix.o": (W, H * e)})
        if layer.get("mlp"):
            F = layer["mlp"]["ff"]
            shapes[p + "norm2"] = (W,)
            shapes.update({p + "mlp.gate": (F, W), p + "mlp.gate.b": (F,), p + "mlp.up": (F, W), p + "mlp.up.b": (F,),
                           p + "mlp.down": (W, F), p + "mlp.down.b": (W,)})
        if side:
            shapes.update({p + "side.gate": (side, W), p + "side.proj": (W, side), p + "side.norm": (W,)})
    return shapes


def random_weights(cfg, seed, sharp=3.0):
    """Values of bfloat16 precision (so that a folder stored in either type
    holds the same model).  Matrices N(0, 1 / fan-in) times a factor; the
    matrices that make scores are scaled so that single keys decide a softmax
    (``sharp``: roughly the spread of the scores)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        tail = name.split(".", 1)[1] if name.startswith("l") and "." in name else name
        if len(shape) == 1 or tail.endswith(".conv"):
            if tail in ("norm1", "norm2", "mix.dq.norm", "mix.dkv.norm", "mix.norm", "side.norm") or name == "final.norm":
                base = 0.0 if tail in ("norm1", "norm2") or name == "final.norm" else 1.0
                t = base + 0.2 * torch.randn(shape, generator=g)
            elif tail == "mix.A_log":
                t = -1.0 + 0.7 * torch.randn(shape, generator=g)
            elif tail.endswith(".conv"):
                t = 0.6 * torch.randn(shape, generator=g)
            else:
                t = 0.3 * torch.randn(shape, generator=g)
        elif name in ("embed", "side.embed", "loop.step"):
            t = torch.randn(shape, generator=g) * (0.5 if name == "loop.step" else 1.0)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if tail in ("mix.uq", "mix.uk"):
                t = t * math.sqrt(sharp)
            if tail in ("mix.o", "mlp.down"):
                t = t * 0.5
        out[name] = t.to(torch.bfloat16).to(torch.float64)
    return out
