"""Runesun as data: how its configuration maps onto parts, and where its parameters are found
in a weight file.  This is the only file that knows the architecture.

Structure: token embedding (no positions); layers in which one RMS norm feeds a latent
attention mixer and, beside it, a feed-forward of routed experts (or none), both added to the
stream at once; a final RMS norm; an output head of its own.  A layer may run with another
layer's tensors: the model then has one set of parts for both and the run order names it twice,
each run with its own cache.

Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.mix.{q, dkv, dkv.norm, uk, uv, sink, g, o}``,
``l<i>.mlp.router``, ``l<i>.mlp.e<k>.{gate, up, down}``, ``final.norm``, ``head``; every linear
weight stored ``(out, in)``.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import Architecture, register_architecture
from ..config.runesun import RunesunConfig
from ..engine.spec import LayerSpec, ModelSpec
from ..parts.base import PartSpec
from ..weights.loader import Recipe, Source, WeightPlan, take


def _owners(cfg: RunesunConfig) -> list[int]:
    """The layers that have tensors of their own, in order."""
    return [i for i in range(len(cfg.layers)) if cfg.layers[i].weights_of is None]


def build_spec(cfg: RunesunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"width": cfg.width, "eps": cfg.norm_eps})
    owners = _owners(cfg)
    layers = []
    for i in owners:
        l = cfg.layers[i]
        mx, ff = l.mixer, l.mlp
        layers.append(LayerSpec(
            mixer=PartSpec("latent_attention", {
                "width": cfg.width, "n_heads": mx.heads, "head_dim": mx.dim, "value_dim": mx.vdim,
                "latent_dim": mx.kv_rank, "scale": mx.scale, "eps": cfg.norm_eps, "sink": True,
                "gate": True, "extra_outputs": ff.experts if ff is not None else 0}),
            ffn=None if ff is None else PartSpec("routed_experts", {
                "width": cfg.width, "n_experts": ff.experts, "top": ff.top, "hidden": ff.ff,
                "activation": "silu", "renormalize": False, "router_from_mixer": True}),
            norm_mixer=norm, norm_ffn=None, block=PartSpec("parallel")))
    place = {i: n for n, i in enumerate(owners)}
    schedule = tuple(place[cfg.owner(i)] for i in range(len(cfg.layers)))
    return ModelSpec(
        architecture="runesun", vocab_size=cfg.vocab_size, width=cfg.width, max_seq_len=None,
        position=PartSpec("none"), layers=tuple(layers), final_norm=norm, tie_head=False,
        schedule=schedule)


def _rows(names_shapes, multiple: int = 1) -> Recipe:
    """Several ``(out_i, in)`` matrices, one under the other, then rows of zeros up to a
    multiple of ``multiple`` rows."""
    srcs = [Source(n, (tuple(s),)) for n, s in names_shapes]

    def combine(ts):
        kinds = {t.dtype for t in ts}
        if len(kinds) > 1:
            ts = [t.to(torch.float32) for t in ts]
        rows = sum(t.shape[0] for t in ts)
        pad = -rows % multiple
        if pad:
            ts = list(ts) + [torch.zeros((pad, ts[0].shape[1]), dtype=ts[0].dtype)]
        return torch.cat(list(ts), dim=0).contiguous()
    return Recipe(srcs, combine)


def _stack(names, shape) -> Recipe:
    srcs = [Source(n, (tuple(shape),)) for n in names]
    return Recipe(srcs, lambda ts: torch.stack(list(ts), dim=0).contiguous())


def weight_plan(cfg: RunesunConfig, spec: ModelSpec, names: set[str]) -> WeightPlan:
    D, V = cfg.width, cfg.vocab_size
    r: dict[str, Recipe] = {"embedding.table": take("embed", (V, D)),
                            "final_norm.weight": take("final.norm", (D,)),
                            "head.weight": take("head", (V, D))}
    for n, i in enumerate(_owners(cfg)):
        l = cfg.layers[i]
        mx, ff = l.mixer, l.mlp
        H, d, dv, R = mx.heads, mx.dim, mx.vdim, mx.kv_rank
        p, L = f"l{i}.", f"layers.{n}."
        r[L + "norm_mixer.weight"] = take(p + "norm1", (D,))
        fused = [(p + "mix.q", (H * d, D)), (p + "mix.dkv", (R, D)), (p + "mix.g", (H, D))]
        if ff is not None:
            fused.append((p + "mlp.router", (ff.experts, D)))
        r[L + "mixer.proj.weight"] = _rows(fused, multiple=8)
        r[L + "mixer.latent_norm"] = take(p + "mix.dkv.norm", (R,))
        # stored [H*d, R]: head i's rows map the latent to its keys; held transposed per head
        r[L + "mixer.key_up"] = Recipe(
            [Source(p + "mix.uk", ((H * d, R),))],
            lambda ts, H=H, d=d, R=R: ts[0].view(H, d, R).transpose(1, 2).contiguous())
        r[L + "mixer.value_up"] = Recipe(
            [Source(p + "mix.uv", ((H * dv, R),))],
            lambda ts, H=H, dv=dv, R=R: ts[0].view(H, dv, R).contiguous())
        r[L + "mixer.sink"] = take(p + "mix.sink", (H,))
        r[L + "mixer.out.weight"] = take(p + "mix.o", (D, H * dv))
        if ff is not None:
            E, F = ff.experts, ff.ff
            r[L + "ffn.gate"] = _stack([f"{p}mlp.e{k}.gate" for k in range(E)], (F, D))
            r[L + "ffn.up"] = _stack([f"{p}mlp.e{k}.up" for k in range(E)], (F, D))
            r[L + "ffn.down"] = _stack([f"{p}mlp.e{k}.down" for k in range(E)], (D, F))
    return WeightPlan(r, set())


def random_tensors(cfg: RunesunConfig, seed: int, *, gain: float = 1.0, std: float | None = None,
                   sink_std: float = 1.0, gamma_jitter: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16) -> dict:
    """Random Runesun tensors under the names of a weight file.  Matrices ~N(0, gain^2 / in) (or
    ~N(0, std^2) if ``std`` is given), embeddings ~N(0, 1), norm weights 1 + N(0,
    gamma_jitter^2), sinks ~N(0, sink_std^2); drawn in fp32 from a seeded CPU generator in a
    fixed order and stored in ``dtype``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))

    def mat(n_out, n_in, s=None):
        s = (gain / math.sqrt(n_in) if std is None else std) if s is None else s
        return (torch.randn(n_out, n_in, generator=g, dtype=torch.float32) * s).to(dtype)

    def vec(n, s, mean=0.0):
        return (torch.randn(n, generator=g, dtype=torch.float32) * s + mean).to(dtype)

    D, V = cfg.width, cfg.vocab_size
    out: dict[str, torch.Tensor] = {"embed": mat(V, D, 1.0)}
    for i in _owners(cfg):
        l = cfg.layers[i]
        mx, ff = l.mixer, l.mlp
        H, d, dv, R = mx.heads, mx.dim, mx.vdim, mx.kv_rank
        p = f"l{i}."
        out[p + "norm1"] = vec(D, gamma_jitter, 1.0)
        out[p + "mix.q"] = mat(H * d, D)
        out[p + "mix.dkv"] = mat(R, D)
        out[p + "mix.dkv.norm"] = vec(R, gamma_jitter, 1.0)
        out[p + "mix.uk"] = mat(H * d, R)
        out[p + "mix.uv"] = mat(H * dv, R)
        out[p + "mix.sink"] = vec(H, sink_std)
        out[p + "mix.g"] = mat(H, D)
        out[p + "mix.o"] = mat(D, H * dv)
        if ff is not None:
            for k in range(ff.experts):
                out[f"{p}mlp.e{k}.gate"] = mat(ff.ff, D)
                out[f"{p}mlp.e{k}.up"] = mat(ff.ff, D)
                out[f"{p}mlp.e{k}.down"] = mat(D, ff.ff)
            out[p + "mlp.router"] = mat(ff.experts, D)
    out["final.norm"] = vec(D, gamma_jitter, 1.0)
    out["head"] = mat(V, D)
    return out


ARCHITECTURE = register_architecture(Architecture(
    name="runesun", config_cls=RunesunConfig, build_spec=build_spec, weight_plan=weight_plan,
    aliases=("Runesun",), random_tensors=random_tensors), replace=True)
