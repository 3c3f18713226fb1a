"""A feed-forward of routed experts."""
from __future__ import annotations

import torch

from ..csrc.ops import GATE_ACTIVATIONS
from .base import MATRIX, FeedForward, ParamSpec, register_part
from .linear import Linear


@register_part("ffn", "routed_experts")
class RoutedExperts(FeedForward):
    """``residual += sum_{e in chosen} s_e * down_e(act(gate_e h) * (up_e h))``, or, with
    ``gated=False``, ``s_e * down_e(act(up_e h))`` (experts of two matrices).

    ``s = softmax(router h)`` over all ``n_experts`` in fp32; the ``top`` experts with the
    largest scores are chosen per token (of equal scores the lower index); their weights are
    their own scores, divided by the chosen scores' sum only if ``renormalize``.  Experts have
    no biases; ``activation`` is the gate's (``silu``, ``gelu_tanh``, ``gelu_erf``, ``none``).

    The router's logits are a product of the same rows as the mixer's projections in a block
    whose sublayers share one norm; ``router_from_mixer`` then reads them from the columns the
    mixer's fused projection appended for it (``ctx.shared_projection``) and this part has no
    router product of its own, only the router's weight rows inside that projection.

    The step's (token, choice) pairs are grouped by expert on the device; a tiled product per
    group runs the gated first half, another the second half, and the weighted results are added
    into the stream in the order of the choices.  Nothing comes back to the host.
    """
    graph_safe = True

    def __init__(self, width: int, n_experts: int, top: int, hidden: int, activation: str = "silu",
                 renormalize: bool = False, router_from_mixer: bool = False, gated: bool = True):
        if activation not in GATE_ACTIVATIONS:
            raise ValueError(f"unknown activation {activation!r} (have {sorted(GATE_ACTIVATIONS)})")
        self.width, self.n_experts, self.top, self.hidden = int(width), int(n_experts), int(top), int(hidden)
        if not 1 <= self.top <= self.n_experts:
            raise ValueError(f"top={top} of {n_experts} experts")
        self.activation = activation
        self.act_code = GATE_ACTIVATIONS[activation]
        self.renormalize = bool(renormalize)
        self.router_from_mixer = bool(router_from_mixer)
        self.gated = bool(gated)
        self.router = None if self.router_from_mixer else Linear(self.width, self.n_experts, bias=False)
        self.gate = self.up = self.down = None

    def children(self):
        return {} if self.router is None else {"router": self.router}

    def param_specs(self):
        e, f, d = self.n_experts, self.hidden, self.width
        specs = {"up": ParamSpec((e, f, d), MATRIX), "down": ParamSpec((e, d, f), MATRIX)}
        if self.gated:
            specs["gate"] = ParamSpec((e, f, d), MATRIX)
        return specs

    can_overwrite = True

    def forward(self, ctx, h: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        if not accumulate:
            residual.zero_()
        lay, ops, dev = ctx.layout, ctx.ops, h.device
        n, top = lay.n_rows, self.top
        if self.router_from_mixer:
            logits, col = ctx.shared_projection
        else:
            logits, col = self.router(ctx, h, out_dtype=torch.float32), 0
        idx = torch.empty((n, top), device=dev, dtype=torch.int32)
        weight = torch.empty((n, top), device=dev, dtype=torch.float32)
        ops.moe_route(logits, col, self.n_experts, top, self.renormalize, lay, idx, weight)
        offsets = torch.empty(self.n_experts + 1, device=dev, dtype=torch.int32)
        order = torch.empty(n * top, device=dev, dtype=torch.int32)
        place = torch.empty(n * top, device=dev, dtype=torch.int32)
        ops.moe_group(idx, self.n_experts, offsets, order, place)
        mid = torch.empty((n * top, self.hidden), device=dev, dtype=ctx.rt.act_dtype)
        if self.gated:
            ops.moe_linear(h, order, top, offsets, self.gate, self.up, mid, self.act_code)
        else:
            ops.moe_linear(h, order, top, offsets, self.up, None, mid, self.act_code)
        y = torch.empty((n * top, self.width), device=dev, dtype=torch.float32)
        ops.moe_linear(mid, None, 1, offsets, self.down, None, y)
        ops.moe_combine(y, place, weight, residual)
