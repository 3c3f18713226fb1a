"""A per-layer input that depends on the token itself."""
from __future__ import annotations

import torch

from ..csrc.ops import ACT_GELU_TANH
from .base import TABLE, VECTOR, ParamSpec, Side, register_part
from .linear import Linear


@register_part("side", "gated_token_input")
class GatedTokenInput(Side):
    """``x += rms(Wproj (gelu_tanh(Wgate x) * e)) * norm``, where ``e`` is the token's row of this
    layer's table (``dim`` numbers) and ``rms`` divides by the root mean square (``eps`` inside
    the root; plain weight).  ``Wgate`` reads the stream itself, not a normed copy of it."""
    graph_safe = True

    def __init__(self, width: int, dim: int, vocab_size: int, eps: float):
        self.width, self.dim, self.vocab_size = int(width), int(dim), int(vocab_size)
        self.eps = float(eps)
        self.gate = Linear(self.width, self.dim, bias=False)
        self.proj = Linear(self.dim, self.width, bias=False)
        self.table = self.norm = None

    def children(self):
        return {"gate": self.gate, "proj": self.proj}

    def param_specs(self):
        return {"table": ParamSpec((self.vocab_size, self.dim), TABLE),
                "norm": ParamSpec((self.width,), VECTOR)}

    def forward(self, ctx, x: torch.Tensor, x_act: torch.Tensor) -> None:
        lay, ops = ctx.layout, ctx.ops
        g = self.gate(ctx, x_act, out_dtype=torch.float32, act=ACT_GELU_TANH)
        ge = torch.empty((lay.n_rows, self.dim), device=x.device, dtype=ctx.rt.act_dtype)
        ops.gather_mul(g, self.table, lay.tokens, ge)
        y = self.proj(ctx, ge, out_dtype=torch.float32)
        ops.rms_add(y, self.norm, self.eps, x, None, 0.0, None, None)
