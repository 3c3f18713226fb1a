"""A plain, slow restatement of the Runesun design, one function per mechanism, in torch on
the CPU.  Whole sequences, no cache, no batching; nothing here is shared with the package.

Notation: ``x`` is the residual stream ``[T, width]`` of one sequence, ``P`` a dict of tensors
by their names in a weight file (``l<i>.norm1``, ``l<i>.mix.q`` ...), ``cfg`` the parsed
config.json.  Every function computes in the element type of its inputs (float64 in tests).

Design, in this file's own words:

* ``x_0 = embed[token]``; for every layer ``h = rms(x) * norm1`` and
  ``x <- x + (mixer(h) + ff(h))`` (both sublayers read the same ``h``; ``ff`` may be absent);
  logits ``= head @ (rms(x) * final.norm)``.
* ``rms(x) = x / sqrt(mean(x^2) + eps)``.
* mixer "latent_attention": ``q = Wq h``; a latent ``c = rms(Wdkv h) * dkv.norm``; per head
  ``k = Wuk c``, ``v = Wuv c``; ``score_ij = scale * q_i . k_j`` for ``j <= i``; weights
  ``exp(score_ij) / (sum_j exp(score_ij) + exp(sink))`` with one learned ``sink`` per head;
  the head's weighted sum of values is multiplied by ``sigmoid(Wg h)`` of that head; ``Wo``
  maps the concatenated heads back.
* ff "moe": ``s = softmax(Wrouter h)`` over all experts; the ``top`` largest are used, each
  weighted by its own ``s`` (no renormalisation); an expert is
  ``Wdown (silu(Wgate h) * (Wup h))``.
* a layer with ``weights_of: j`` uses layer ``j``'s tensors.
"""
from __future__ import annotations

import math

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """``scores`` [..., n] (masked places are -inf), ``sink`` broadcastable to ``scores[..., 0]``:
    weights whose denominator has one more term, exp(sink), that belongs to no key."""
    m = torch.maximum(scores.max(-1).values, sink)
    e = torch.exp(scores - m[..., None])
    return e / (e.sum(-1) + torch.exp(sink - m))[..., None]


def latent_attention(h: torch.Tensor, P: dict, pre: str, mx: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, dim, vdim, scale = mx["heads"], mx["dim"], mx["vdim"], mx["scale"]
    q = (h @ P[pre + "q"].T).view(T, H, dim)
    c = rms_norm(h @ P[pre + "dkv"].T, P[pre + "dkv.norm"], eps)
    k = (c @ P[pre + "uk"].T).view(T, H, dim)
    v = (c @ P[pre + "uv"].T).view(T, H, vdim)
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    future = torch.ones(T, T, dtype=torch.bool).triu(1)
    s = s.masked_fill(future, -math.inf)
    w = sink_softmax(s, P[pre + "sink"][:, None].expand(H, T))
    o = torch.einsum("hij,jhv->ihv", w, v)
    gate = torch.sigmoid(h @ P[pre + "g"].T)            # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * vdim) @ P[pre + "o"].T


def silu(z):
    return z * torch.sigmoid(z)


def expert(h, P, pre):
    return (silu(h @ P[pre + "gate"].T) * (h @ P[pre + "up"].T)) @ P[pre + "down"].T


def route(h, P, pre, n_top):
    """Scores over all experts, and the ``n_top`` chosen per token (largest score first; of
    equal scores the lower index)."""
    s = torch.softmax(h @ P[pre + "router"].T, dim=-1)
    order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :n_top]
    return s, order


def moe(h, P, pre, ff: dict, told=None, margin=0.0):
    """``told`` (optional, [T, top]): what another implementation chose.  Where this one's own
    choice is a close call (the last chosen and the first left-out expert's logits are less than
    ``margin`` apart) it follows ``told``; everywhere else ``told`` must be its own choice."""
    n_top = ff["router"]["top"]
    s, chosen = route(h, P, pre, n_top)
    if told is not None:
        z = torch.sort(h @ P[pre + "router"].T, dim=-1, descending=True).values
        gap = z[:, n_top - 1] - z[:, n_top] if n_top < z.shape[1] else torch.full((h.shape[0],), math.inf)
        for t in range(h.shape[0]):
            mine, theirs = sorted(chosen[t].tolist()), sorted(told[t].tolist())
            if float(gap[t]) >= margin:
                assert mine == theirs, f"{pre} token {t}: chose {theirs}, plain says {mine} (gap {float(gap[t]):.3f})"
            else:
                assert len(set(theirs)) == n_top and all(0 <= e < s.shape[1] for e in theirs)
                chosen[t] = torch.tensor(theirs)
    out = torch.zeros(h.shape[0], P[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            out[t] += s[t, e] * expert(h[t:t + 1], P, f"{pre}e{e}.")[0]
    return out


def layer(x, P, cfg, i, told=None, margin=0.0):
    entry = cfg["layers"][i]
    src = entry.get("weights_of", i)
    eps = cfg["norm"]["eps"]
    pre = f"l{src}."
    h = rms_norm(x, P[pre + "norm1"], eps)
    if entry["type"] != "latent_attention":
        raise ValueError(entry["type"])
    y = latent_attention(h, P, pre + "mix.", entry["mixer"], eps)
    if entry.get("mlp") is not None:
        if entry["mlp"]["kind"] != "moe":
            raise ValueError(entry["mlp"]["kind"])
        y = y + moe(h, P, pre + "mlp.", entry["mlp"], told, margin)
    return x + y


def forward(tokens, P, cfg, dtype=torch.float64, keep_layers=False, routed=None, margin=0.0):
    """Logits at every position of one sequence, ``[T, vocab]`` (and the residual stream after
    every layer run when ``keep_layers``).  ``routed``: per layer run with routed experts, in
    order, the experts another implementation chose ``[T, top]`` (see :func:`moe`)."""
    P = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in P.items()}
    x = P["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    streams = []
    routed = list(routed) if routed is not None else None
    for i in range(len(cfg["layers"])):
        told = routed.pop(0) if routed is not None and cfg["layers"][i].get("mlp") is not None else None
        x = layer(x, P, cfg, i, told, margin)
        streams.append(x)
    logits = rms_norm(x, P["final.norm"], cfg["norm"]["eps"]) @ P["head"].T
    return (logits, torch.stack(streams)) if keep_layers else logits
