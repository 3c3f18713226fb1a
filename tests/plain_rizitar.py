"""Rizitar from its equations: a plain, slow restatement in float64, whole sequences at a time,
no cache, no batching, one function per mechanism.  It shares no code with the package: it
reads the raw config.json object and a ``{name: tensor}`` dictionary of the weight file.

Notation: ``T`` tokens, ``D`` width, positions ``0 .. T-1``; a linear weight ``W`` is stored
``[out, in]`` and applied as ``x @ W.T``.
"""
from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_unit(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms_unit(x, eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(x):
    return torch.log1p(torch.exp(-x.abs())) + torch.clamp(x, min=0)


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    neg = torch.clamp(z, max=0.0)
    return torch.where(z > 0, ap * z * z + 0.5 * z, an * (torch.expm1(neg) - neg) + 0.5 * z)


def relu_squared(z):
    return torch.clamp(z, min=0.0) ** 2


# ------------------------------------------------------------------------------ rotation
def rotary_frequencies(rot):
    """Per pair ``i`` of the rotated dimensions its angular frequency, and the factor on cos/sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    f = f / factor * ramp + f * (1.0 - ramp)
    return f, 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x [T, heads, dim]: the first ``dims`` numbers of each head are turned, dimension ``i``
    paired with ``i + dims/2``."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f, m = rotary_frequencies(rot)
    ang = positions.to(F64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * m)[:, None, :], (torch.sin(ang) * m)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ------------------------------------------------------------------------------ mixers
def seen_attention(q, k, v, scale, size, P, sink):
    """q [T, H, d], k and v [T, G, d] as the cache holds them: position ``i`` sees the tokens
    ``j`` with ``0 <= i - j < size`` (all earlier ones if ``size`` is 0) and, for every block of
    ``P`` tokens that lies wholly before that window (``bP + P - 1 <= i - size``), the mean of
    its keys and the mean of its values; one softmax over both, whose denominator also holds
    ``exp(sink_h)``.  Returns [T, H, d]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for i in range(T):
        lo = max(0, i - size + 1) if size > 0 else 0
        keys, vals = [k[lo:i + 1]], [v[lo:i + 1]]
        if size > 0 and P > 0:
            b = 0
            while b * P + P - 1 <= i - size:
                keys.append(k[b * P:b * P + P].mean(0, keepdim=True))
                vals.append(v[b * P:b * P + P].mean(0, keepdim=True))
                b += 1
        kk, vv = torch.cat(keys), torch.cat(vals)              # [n, G, d]
        for hh in range(H):
            g = hh // (H // G)
            s = (kk[:, g] @ q[i, hh]) * scale
            sk = None if sink is None else sink[hh]
            m = s.max() if sk is None else torch.maximum(s.max(), sk)
            e = torch.exp(s - m)
            den = e.sum() + (torch.exp(sk - m) if sk is not None else 0.0)
            out[i, hh] = (e / den) @ vv[:, g]
    return out


def pooled_window_attention(h, w, mx, eps):
    """The attention mixer on normed rows ``h`` [T, D]; ``w``: the layer's ``mix.*`` tensors by
    their short names; ``mx``: the layer's mixer object of config.json."""
    T = h.shape[0]
    H, G, d = int(mx["heads"]), int(mx.get("kv_heads", mx["heads"])), int(mx["dim"])
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = k.clone()                                    # the values are the keys as projected
    q = rms_norm(q, w["q.norm"], eps)
    k = rms_norm(k, w["k.norm"], eps)
    pos = torch.arange(T)
    q, k = rotate(q, pos, mx.get("rot")), rotate(k, pos, mx.get("rot"))
    mask = mx.get("mask") or {}
    out = seen_attention(q, k, v, float(mx["scale"]), int(mask.get("size", 0)),
                         int(mask.get("pool") or 0), w.get("sink"))
    return out.reshape(T, -1) @ w["o"].T


def delta_recurrence(r, k, v, decay, a, S=None):
    """r, k, v, decay, a: [T, H, d].  From the state ``S`` [H, d, d] (key channel, value channel;
    zeros if ``None``): ``S <- diag(decay) S - (a * u)(u^T S) + k v^T`` with the unit key ``u``,
    both subtracted terms reading the old state, then ``o = S^T r``.  Returns (o [T, H, d], S)."""
    T, H, d = r.shape
    u = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    S = torch.zeros(H, d, d, dtype=F64) if S is None else S.clone()
    o = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        old = S
        removed = torch.einsum("hk,hkv->hv", u[t], old)            # u^T S
        S = decay[t][:, :, None] * old - (a[t] * u[t])[:, :, None] * removed[:, None, :] \
            + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, r[t])
    return o, S


def decay_of(logits):
    return torch.exp(-math.exp(-0.5) * torch.sigmoid(logits))


def general_delta(h, w, mx, eps):
    """The generalized delta rule on normed rows ``h`` [T, D]."""
    T = h.shape[0]
    H, d = int(mx["heads"]), int(mx["dim"])
    r = (h @ w["r"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, d)
    decay = decay_of(torch.tanh(h @ w["w1"].T) @ w["w2"].T + w["w0"]).view(T, H, d)
    a = torch.sigmoid(h @ w["a"].T + w["a.b"]).view(T, H, d)
    o, _ = delta_recurrence(r, k, v, decay, a)
    o = rms_unit(o, eps).reshape(T, H * d) * w["norm"]
    o = o * torch.sigmoid(h @ w["g"].T)
    return o @ w["o"].T


# ------------------------------------------------------------------------------ feed-forwards
def dense_ff(h, w):
    z = h @ w["up"].T + w["up.b"]
    return xielu(z, w["act"][0], w["act"][1]) @ w["down"].T + w["down.b"]


def route(h, router, top):
    """Chosen experts [T, top] (largest scores first, of equal scores the lower index) and their
    softmax scores."""
    s = torch.softmax(h @ router.T, dim=-1)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
    return order, torch.gather(s, 1, order)


def moe_ff(h, w, ff, follow=None, margin=0.0):
    """``follow``: [T, top] experts that someone else chose.  Where that choice differs from the
    one made here and the router's logits of the last expert in and the first one out are
    closer than ``margin`` (a close call that rounding may settle either way), it is followed."""
    E, top = int(ff["router"]["experts"]), int(ff["router"]["top"])
    z = h @ w["router"].T
    s = torch.softmax(z, dim=-1)
    order, score = route(h, w["router"], top)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        mine = order[t]
        if follow is not None and top < E and set(follow[t].tolist()) != set(mine.tolist()):
            ranked = torch.sort(z[t], descending=True, stable=True).values
            if float(ranked[top - 1] - ranked[top]) < margin:
                mine = follow[t]
        for e in mine.tolist():
            out[t] += s[t, e] * (relu_squared(h[t] @ w[f"e{e}.up"].T) @ w[f"e{e}.down"].T)
    return out


def token_side(x, tokens, w, table, layer, dim, eps):
    e = table[tokens][:, layer * dim:(layer + 1) * dim]
    g = gelu_tanh(x @ w["gate"].T) * e
    y = g @ w["proj"].T
    return rms_unit(y, eps) * w["norm"]


# ------------------------------------------------------------------------------ the model
def _sub(tensors, prefix):
    n = len(prefix)
    return {k[n:]: v.to(F64) for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, return_layers: bool = False, routed=None,
            margin: float = 0.0):
    """Logits [T, vocab] of one sequence (float64); with ``return_layers`` also the stream after
    every layer [layers, T, D].  ``routed``: per layer with routed experts, in order, the
    [T, top] experts someone else chose (see :func:`moe_ff`)."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    eps = float(cfg["norm"]["eps"])
    embed = tensors["embed"].to(F64)
    x = embed[tokens] * float((cfg.get("embedding") or {}).get("scale", 1.0))
    side_dim = int(cfg["token_side"]["dim"]) if cfg.get("token_side") else 0
    after, n_routed = [], 0
    for i, layer in enumerate(cfg["layers"]):
        w = _sub(tensors, f"l{i}.")
        mix = _sub(tensors, f"l{i}.mix.")
        h = rms_norm(x, w["norm1"], eps)
        if layer["type"] == "general_delta":
            y = general_delta(h, mix, layer["mixer"], eps)
        elif layer["type"] == "attention":
            y = pooled_window_attention(h, mix, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, w["norm1b"], eps)
        ff = layer.get("mlp")
        if ff is not None:
            h = rms_norm(x, w["norm2"], eps)
            mlp = _sub(tensors, f"l{i}.mlp.")
            if ff["kind"] == "dense":
                y = dense_ff(h, mlp)
            else:
                y = moe_ff(h, mlp, ff, None if routed is None else routed[n_routed], margin)
                n_routed += 1
            x = x + rms_norm(y, w["norm2b"], eps)
        if side_dim:
            x = x + token_side(x, tokens, _sub(tensors, f"l{i}.side."),
                               tensors["side.embed"].to(F64), i, side_dim, eps)
        after.append(x)
    logits = rms_norm(x, tensors["final.norm"].to(F64), eps) @ embed.T
    return (logits, torch.stack(after)) if return_layers else logits
