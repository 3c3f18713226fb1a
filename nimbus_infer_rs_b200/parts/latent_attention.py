"""Causal attention whose keys and values are low-rank: only a latent per token is cached."""
from __future__ import annotations

import torch

from .base import MATRIX, VECTOR, KVRequest, Mixer, ParamSpec, register_part
from .linear import Linear


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    """Multi-head attention over a shared latent, without positions.

    ``q = Wq h`` (``n_heads`` heads of ``head_dim``); ``c = rms(Wdown h) * latent_norm`` is the
    token's latent (``latent_dim`` numbers, the only thing cached); head ``i`` has keys
    ``k_i = Wk_i c`` and values ``v_i = Wv_i c`` (``value_dim`` numbers); scores
    ``scale * q_i . k_i`` over positions ``j <= p``; with ``sink`` the softmax's denominator
    has one more term ``exp(sink_i)`` per head that belongs to no key; with ``gate`` head
    ``i``'s result is multiplied by ``sigmoid(Wgate h)_i``; ``Wout`` maps the concatenated
    heads back into the stream.

    How it runs: one product gives ``[q | Wdown h | gate logits]`` in fp32 (plus whatever
    else reads the same rows: ``extra_outputs`` columns that a feed-forward beside it picks up,
    e.g. its router's logits).  Keys and values are never formed: ``Wk_i`` moves to the query
    (``a_i = Wk_i^T q_i``, then ``a_i . c_j = q_i . k_i(j)``) and ``Wv_i`` behind the weighted
    sum (``Wv_i sum_j p_j c_j``), so every head attends over the same cached rows, which are
    key and value at once.  The latent's norm, the scores, the softmax and the sink are fp32.
    """
    graph_safe = True

    def __init__(self, width: int, n_heads: int, head_dim: int, value_dim: int, latent_dim: int,
                 scale: float, eps: float, sink: bool = True, gate: bool = True, window: int = 0,
                 extra_outputs: int = 0):
        self.width, self.n_heads = int(width), int(n_heads)
        self.head_dim, self.value_dim, self.latent_dim = int(head_dim), int(value_dim), int(latent_dim)
        self.scale, self.eps, self.window = float(scale), float(eps), int(window)
        self.has_sink, self.has_gate = bool(sink), bool(gate)
        self.extra_outputs = int(extra_outputs)
        self.q_width = self.n_heads * self.head_dim
        # columns of the fused projection's result
        self.col_latent = self.q_width
        self.col_gate = self.col_latent + self.latent_dim
        self.col_extra = self.col_gate + (self.n_heads if self.has_gate else 0)
        # rows of zeros fill the projection up to a multiple of 8 outputs, so that its fp32 rows
        # start on 32-byte boundaries whatever the numbers of heads and extra outputs are
        self.proj_outputs = -(-(self.col_extra + self.extra_outputs) // 8) * 8
        self.proj = Linear(self.width, self.proj_outputs, bias=False)
        self.out = Linear(self.n_heads * self.value_dim, self.width, bias=False)
        self.latent_norm = self.key_up = self.value_up = self.sink = None

    def children(self):
        return {"proj": self.proj, "out": self.out}

    def param_specs(self):
        specs = {
            "latent_norm": ParamSpec((self.latent_dim,), VECTOR),
            # per head, held for the products that run: [latent_dim, head_dim] = Wk_i transposed
            "key_up": ParamSpec((self.n_heads, self.latent_dim, self.head_dim), MATRIX),
            "value_up": ParamSpec((self.n_heads, self.value_dim, self.latent_dim), MATRIX),
        }
        if self.has_sink:
            specs["sink"] = ParamSpec((self.n_heads,), VECTOR)
        return specs

    def cache_request(self):
        return KVRequest(1, self.latent_dim, self.window, planes=1)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor) -> None:
        lay, kv, ops = ctx.layout, ctx.kv, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        ctx.shared_projection = (fused, self.col_extra)       # for a reader of the extra columns
        if ctx.writes_cache:
            ops.latent_append(fused, self.col_latent, self.latent_norm, self.eps, lay, kv)
        a = torch.empty((n, self.n_heads * self.latent_dim), device=dev, dtype=act)
        ops.head_linear(fused, 0, self.key_up, a, lay)
        mix = torch.empty((n, self.n_heads * self.latent_dim), device=dev, dtype=act)
        ops.attention_latent(a, lay, kv, self.n_heads, self.sink, mix, self.scale, self.window)
        heads = torch.empty((n, self.n_heads * self.value_dim), device=dev, dtype=act)
        ops.head_linear(mix, 0, self.value_up, heads, lay,
                        gate=fused if self.has_gate else None, gate_col=self.col_gate)
        self.out(ctx, heads, residual=residual)
