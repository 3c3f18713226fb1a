"""A linear-recurrent mixer: the generalized delta rule with a per-channel decay."""
from __future__ import annotations

import torch

from ..csrc.ops import ACT_TANH
from .base import VECTOR, Mixer, ParamSpec, StateRequest, register_part
from .linear import Linear


@register_part("mixer", "delta_rule")
class DeltaRule(Mixer):
    """Per head a state matrix ``S`` (key channels x value channels, fp32, zero at the start of
    a sequence) that every token updates and then reads:

        S_t = diag(w_t) S_(t-1) - (a_t * u_t) (u_t^T S_(t-1)) + k_t v_t^T,    o_t = S_t^T r_t

    with ``r, k, v = Wr h, Wk h, Wv h`` (``n_heads`` heads of ``head_dim``), the unit key
    ``u = k / sqrt(sum k^2 + key_eps)`` per head, the decay ``w = exp(-decay_rate * sigmoid(W2
    tanh(W1 h) + w0))`` and the removal rate ``a = sigmoid(Wa h + a_bias)``, both per head and
    key channel.  Both the decayed and the removed term read the old state.  Each head's
    ``o`` is divided by its root mean square (``eps`` inside the root), the heads side by side
    are multiplied by the weight ``norm`` and by ``sigmoid(Wg h)``, and ``Wout`` maps them back.

    How it runs: one product gives ``[r | k | v | g logits | a logits | W1 h]`` in fp32; a row
    pass takes the tanh; a small product gives the decay's logits; one kernel per step walks
    each sequence's tokens in order with the state in registers, computes decays, rates, unit
    keys, the head norm and the gate in fp32, and leaves the state in the sequence's fixed-size
    state row.  Nothing grows with the sequence.
    """
    graph_safe = True
    can_overwrite = True

    def __init__(self, width: int, n_heads: int, head_dim: int, decay_rank: int, eps: float,
                 decay_rate: float = 0.6065306597126334, key_eps: float = 1e-6):
        self.width, self.n_heads, self.head_dim = int(width), int(n_heads), int(head_dim)
        self.decay_rank, self.eps = int(decay_rank), float(eps)
        self.decay_rate, self.key_eps = float(decay_rate), float(key_eps)
        self.inner = self.n_heads * self.head_dim
        # columns of the fused projection's result
        self.col_r, self.col_k, self.col_v = 0, self.inner, 2 * self.inner
        self.col_g, self.col_a, self.col_w1 = 3 * self.inner, 4 * self.inner, 5 * self.inner
        # rows of zeros fill it up to a multiple of 8 outputs (fp32 rows on 32-byte boundaries)
        self.proj_outputs = -(-(self.col_w1 + self.decay_rank) // 8) * 8
        self.proj = Linear(self.width, self.proj_outputs, bias=False)
        self.decay_up = Linear(self.decay_rank, self.inner, bias="required")      # W2 and w0
        self.out = Linear(self.inner, self.width, bias=False)
        self.a_bias = self.norm = None

    def children(self):
        return {"proj": self.proj, "decay_up": self.decay_up, "out": self.out}

    def param_specs(self):
        return {"a_bias": ParamSpec((self.inner,), VECTOR), "norm": ParamSpec((self.inner,), VECTOR)}

    def state_request(self):
        return StateRequest(self.n_heads * self.head_dim * self.head_dim)

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        lay, ops = ctx.layout, ctx.ops
        n, dev, act = lay.n_rows, h.device, ctx.rt.act_dtype
        fused = self.proj(ctx, h, out_dtype=torch.float32)
        t = torch.empty((n, self.decay_rank), device=dev, dtype=act)
        ops.act_rows(fused, self.col_w1, ACT_TANH, None, t)
        decay_logits = self.decay_up(ctx, t, out_dtype=torch.float32)
        o = torch.empty((n, self.inner), device=dev, dtype=act)
        ops.delta_rule(fused, self.col_r, self.col_k, self.col_v, self.col_g, self.col_a,
                       decay_logits, self.a_bias, self.norm, self.eps, self.decay_rate,
                       self.key_eps, lay, ctx.state, self.n_heads, self.head_dim, o)
        if accumulate:
            self.out(ctx, o, residual=residual)
        else:
            self.out(ctx, o, out=residual)
