"""Sliding-window attention that also sees pooled blocks of what left the window."""
from __future__ import annotations

import torch

from .base import VECTOR, KVRequest, Mixer, ParamSpec, register_part
from .linear import Linear
from .rotary import rotary_frequencies


@register_part("mixer", "pooled_window_attention")
class PooledWindowAttention(Mixer):
    """Multi-head attention with ``n_kv_heads`` shared key heads whose values are its keys.

    ``q = Wq h``, ``k = Wk h`` (one fused product, fp32 result); the value of a token is ``k``
    as projected.  Queries and keys then get a per-head RMS norm (weights ``q_norm``,
    ``k_norm`` of ``head_dim`` numbers, shared by the heads; fp32) and, with ``rot_dims`` > 0,
    a rotation by position of their first ``rot_dims`` numbers (``parts/rotary.py``); the
    values get neither.  Scores are ``scale * q . k``.

    What position ``i`` sees: the tokens ``j`` with ``0 <= i - j < window`` (all earlier
    tokens if ``window`` is 0) and, with ``pool`` = P > 0, one key and one value for every
    block of P consecutive tokens that lies wholly before the window (block ``b`` = positions
    ``bP .. bP+P-1``, seen once ``bP + P - 1 <= i - window``): the mean of the block's keys as
    the cache holds them, and the mean of its values.  A token that has left the window while
    its block is not yet seen is not seen.  Tokens and blocks share one softmax, whose
    denominator has, with ``sink``, one more term ``exp(sink_h)`` per head without key or value.

    Storage: the paged key/value store (pages are given back once no later token needs them:
    neither its window nor the mean of its block), and a second paged store with one entry per
    block, written when a block's last token arrives.
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, n_heads: int, n_kv_heads: int, head_dim: int, scale: float,
                 eps: float, window: int = 0, pool: int = 0, sink: bool = True,
                 rot_dims: int = 0, rot_base: float = 10000.0, rot_scaling: dict | None = None):
        self.width, self.n_heads, self.n_kv_heads = int(width), int(n_heads), int(n_kv_heads)
        self.head_dim, self.scale, self.eps = int(head_dim), float(scale), float(eps)
        self.window, self.pool = int(window), int(pool)
        if self.n_heads % self.n_kv_heads:
            raise ValueError("n_heads must be divisible by n_kv_heads")
        if self.window <= 0:
            self.pool = 0                   # nothing ever leaves a window that is not there
        self.has_sink = bool(sink)
        self.rot_dims = int(rot_dims)
        if self.rot_dims > self.head_dim:
            raise ValueError("more rotated dimensions than the head has")
        self.rot_freq_host, self.rot_amplitude = (None, 1.0) if not self.rot_dims else \
            rotary_frequencies(self.rot_dims, rot_base, rot_scaling)
        self.rot_freq = None
        self.q_width = self.n_heads * self.head_dim
        self.kv_width = self.n_kv_heads * self.head_dim
        self.proj = Linear(self.width, self.q_width + self.kv_width, bias=False)
        self.out = Linear(self.q_width, self.width, bias=False)
        self.q_norm = self.k_norm = self.sink = None

    def children(self):
        return {"proj": self.proj, "out": self.out}

    def param_specs(self):
        specs = {"q_norm": ParamSpec((self.head_dim,), VECTOR),
                 "k_norm": ParamSpec((self.head_dim,), VECTOR)}
        if self.has_sink:
            specs["sink"] = ParamSpec((self.n_heads,), VECTOR)
        return specs

    def bind(self, params, runtime) -> None:
        super().bind(params, runtime)
        if self.rot_freq_host is not None:
            self.rot_freq = self.rot_freq_host.to(runtime.device)

    def cache_request(self):
        # a token's page is kept while the token is in some later window, or its block is not
        # complete yet (the block's mean reads all of its keys)
        keep = max(self.window, self.pool) if self.window > 0 else 0
        return KVRequest(self.n_kv_heads, self.head_dim, keep)

    def extra_cache_requests(self):
        if self.pool <= 0:
            return ()
        return (KVRequest(self.n_kv_heads, self.head_dim, 0, 2, every=self.pool),)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, kv, ops = ctx.layout, ctx.kv, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        q = torch.empty((n, self.q_width), device=dev, dtype=act)
        ops.qk_norm_rope_append(fused, 0, self.q_width, self.q_norm, self.k_norm, self.eps,
                                self.rot_freq, self.rot_dims, self.rot_amplitude, lay, kv,
                                self.n_heads, q, ctx.writes_cache)
        blocks = ctx.kv_extra[0] if self.pool > 0 else None
        if blocks is not None and ctx.writes_cache:
            ops.pool_blocks(lay, kv, blocks, self.pool)
        attn = torch.empty((n, self.q_width), device=dev, dtype=act)
        ops.attention_pooled(q, lay, kv, blocks, self.n_heads, self.sink, attn, self.scale,
                             self.window, self.pool)
        if accumulate:
            self.out(ctx, attn, residual=residual)
        else:
            self.out(ctx, attn, out=residual)
