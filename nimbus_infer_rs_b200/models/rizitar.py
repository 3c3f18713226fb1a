"""Rizitar as data: how its configuration maps onto parts, and where its parameters are found
in a weight file.  This is the only file that knows the architecture.

Structure: token embedding times a constant (no position table); layers in any order of two
kinds, a linear-recurrent one (``general_delta``: the generalized delta rule) and an attention
one (``attention``: a sliding window that also sees pooled blocks of what left it, values that
are the keys, a sink); every sublayer between two RMS norms, its normed result added to the
stream; a feed-forward per layer that is dense (an activation with learned numbers), routed
experts (two matrices each, squared relu) or absent; after it a per-token input gated by the
stream; a final RMS norm and the embedding table as the output head.

Tensor names: ``embed``, ``side.embed`` (all layers' per-token rows side by side),
``final.norm``, and per layer ``l<i>.``: ``norm1``, ``norm1b``, ``norm2``, ``norm2b``,
``mix.{r, k, v, g, a, a.b, w1, w2, w0, norm, o}`` or ``mix.{q, k, q.norm, k.norm, sink, o}``,
``mlp.{up, up.b, down, down.b, act}`` or ``mlp.{router, e<k>.up, e<k>.down}``,
``side.{gate, proj, norm}``; every linear weight stored ``(out, in)``.
"""
from __future__ import annotations

import math

import torch

from ..config.registry import Architecture, register_architecture
from ..config.rizitar import DenseFFConfig, MoEFFConfig, RizitarConfig
from ..engine.spec import LayerSpec, ModelSpec
from ..parts.base import PartSpec
from ..weights.loader import Recipe, Source, WeightPlan, take
from .runesun import _rows, _stack

DEFAULT_DECAY_RANK = 32      # of a model made here without a weight file to give it


def _decay_rank(mx) -> int:
    return mx.decay_rank if mx.decay_rank is not None else DEFAULT_DECAY_RANK


def build_spec(cfg: RizitarConfig) -> ModelSpec:
    D = cfg.width
    norm = PartSpec("rmsnorm", {"width": D, "eps": cfg.norm_eps})
    layers = []
    for l in cfg.layers:
        mx, ff = l.mixer, l.mlp
        if l.type == "general_delta":
            mixer = PartSpec("delta_rule", {
                "width": D, "n_heads": mx.heads, "head_dim": mx.dim,
                "decay_rank": _decay_rank(mx), "eps": cfg.norm_eps,
                "decay_rate": math.exp(-0.5), "key_eps": 1e-6})
        else:
            rot = mx.rot
            scaling = None if rot is None or rot.scaling is None else {
                "factor": rot.scaling.factor, "original": rot.scaling.original,
                "fast": rot.scaling.fast, "slow": rot.scaling.slow}
            mixer = PartSpec("pooled_window_attention", {
                "width": D, "n_heads": mx.heads, "n_kv_heads": mx.kv_heads, "head_dim": mx.dim,
                "scale": mx.scale, "eps": cfg.norm_eps, "window": mx.window, "pool": mx.pool,
                "sink": True, "rot_dims": 0 if rot is None else rot.dims,
                "rot_base": 10000.0 if rot is None else rot.base, "rot_scaling": scaling})
        if ff is None:
            ffn = None
        elif isinstance(ff, DenseFFConfig):
            ffn = PartSpec("dense_mlp", {"width": D, "hidden": ff.ff, "activation": "xielu",
                                         "bias": "required"})
        else:
            ffn = PartSpec("routed_experts", {
                "width": D, "n_experts": ff.experts, "top": ff.top, "hidden": ff.ff,
                "activation": "relu2", "renormalize": False, "gated": False})
        side = None if not cfg.side_dim else PartSpec("gated_token_input", {
            "width": D, "dim": cfg.side_dim, "vocab_size": cfg.vocab_size, "eps": cfg.norm_eps})
        layers.append(LayerSpec(
            mixer=mixer, ffn=ffn, norm_mixer=norm, norm_ffn=None if ffn is None else norm,
            block=PartSpec("sandwich"), post_norm_mixer=norm,
            post_norm_ffn=None if ffn is None else norm, side=side))
    return ModelSpec(
        architecture="rizitar", vocab_size=cfg.vocab_size, width=D, max_seq_len=None,
        position=PartSpec("none"), layers=tuple(layers), final_norm=norm, tie_head=True,
        embedding_scale=cfg.embedding_scale)


def _columns(name: str, shape, lo: int, hi: int) -> Recipe:
    """Columns ``lo .. hi`` of a stored table, held as a table of their own."""
    return Recipe([Source(name, (tuple(shape),))], lambda ts: ts[0][:, lo:hi].contiguous())


def weight_plan(cfg: RizitarConfig, spec: ModelSpec, names: set[str]) -> WeightPlan:
    D, V, n_layers = cfg.width, cfg.vocab_size, len(cfg.layers)
    r: dict[str, Recipe] = {"embedding.table": take("embed", (V, D)),
                            "final_norm.weight": take("final.norm", (D,))}
    for i, l in enumerate(cfg.layers):
        mx, ff = l.mixer, l.mlp
        p, L = f"l{i}.", f"layers.{i}."
        r[L + "norm_mixer.weight"] = take(p + "norm1", (D,))
        r[L + "post_norm_mixer.weight"] = take(p + "norm1b", (D,))
        if l.type == "general_delta":
            hd, rank = mx.heads * mx.dim, _decay_rank(mx)
            r[L + "mixer.proj.weight"] = _rows(
                [(p + "mix.r", (hd, D)), (p + "mix.k", (hd, D)), (p + "mix.v", (hd, D)),
                 (p + "mix.g", (hd, D)), (p + "mix.a", (hd, D)), (p + "mix.w1", (rank, D))],
                multiple=8)
            r[L + "mixer.decay_up.weight"] = take(p + "mix.w2", (hd, rank))
            r[L + "mixer.decay_up.bias"] = take(p + "mix.w0", (hd,))
            r[L + "mixer.a_bias"] = take(p + "mix.a.b", (hd,))
            r[L + "mixer.norm"] = take(p + "mix.norm", (hd,))
            r[L + "mixer.out.weight"] = take(p + "mix.o", (D, hd))
        else:
            H, G, d = mx.heads, mx.kv_heads, mx.dim
            r[L + "mixer.proj.weight"] = _rows([(p + "mix.q", (H * d, D)), (p + "mix.k", (G * d, D))])
            r[L + "mixer.q_norm"] = take(p + "mix.q.norm", (d,))
            r[L + "mixer.k_norm"] = take(p + "mix.k.norm", (d,))
            r[L + "mixer.sink"] = take(p + "mix.sink", (H,))
            r[L + "mixer.out.weight"] = take(p + "mix.o", (D, H * d))
        if ff is not None:
            r[L + "norm_ffn.weight"] = take(p + "norm2", (D,))
            r[L + "post_norm_ffn.weight"] = take(p + "norm2b", (D,))
        if isinstance(ff, DenseFFConfig):
            r[L + "ffn.fc.weight"] = take(p + "mlp.up", (ff.ff, D))
            r[L + "ffn.fc.bias"] = take(p + "mlp.up.b", (ff.ff,))
            r[L + "ffn.proj.weight"] = take(p + "mlp.down", (D, ff.ff))
            r[L + "ffn.proj.bias"] = take(p + "mlp.down.b", (D,))
            r[L + "ffn.act"] = take(p + "mlp.act", (2,))
        elif isinstance(ff, MoEFFConfig):
            r[L + "ffn.router.weight"] = take(p + "mlp.router", (ff.experts, D))
            r[L + "ffn.up"] = _stack([f"{p}mlp.e{k}.up" for k in range(ff.experts)], (ff.ff, D))
            r[L + "ffn.down"] = _stack([f"{p}mlp.e{k}.down" for k in range(ff.experts)], (D, ff.ff))
        if cfg.side_dim:
            n = cfg.side_dim
            r[L + "side.table"] = _columns("side.embed", (V, n_layers * n), i * n, (i + 1) * n)
            r[L + "side.gate.weight"] = take(p + "side.gate", (n, D))
            r[L + "side.proj.weight"] = take(p + "side.proj", (D, n))
            r[L + "side.norm"] = take(p + "side.norm", (D,))
    # a layer without a feed-forward may still carry the norms around it in the file
    ignored = {f"l{i}.{n}" for i, l in enumerate(cfg.layers) if l.mlp is None
               for n in ("norm2", "norm2b")}
    return WeightPlan(r, ignored)


def complete_config(cfg: RizitarConfig, shapes: dict) -> RizitarConfig:
    return cfg.with_shapes(shapes)


def random_tensors(cfg: RizitarConfig, seed: int, *, gain: float = 1.0, std: float | None = None,
                   sink_std: float = 1.0, gamma_jitter: float = 0.1,
                   dtype: torch.dtype = torch.bfloat16) -> dict:
    """Random Rizitar tensors under the names of a weight file.  Matrices ~N(0, gain^2 / in) (or
    ~N(0, std^2) if ``std`` is given), embeddings ~N(0, 1) (divided by the embedding's scale, so
    that the stream starts near unit size), norm weights 1 + N(0, gamma_jitter^2), biases and
    learned activation numbers small, sinks ~N(0, sink_std^2); drawn in fp32 from a seeded CPU
    generator in a fixed order and stored in ``dtype``."""
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))

    def mat(n_out, n_in, s=None):
        s = (gain / math.sqrt(n_in) if std is None else std) if s is None else s
        return (torch.randn(n_out, n_in, generator=g, dtype=torch.float32) * s).to(dtype)

    def vec(n, s, mean=0.0):
        return (torch.randn(n, generator=g, dtype=torch.float32) * s + mean).to(dtype)

    D, V = cfg.width, cfg.vocab_size
    out: dict[str, torch.Tensor] = {"embed": mat(V, D, 1.0 / max(abs(cfg.embedding_scale), 1e-6))}
    if cfg.side_dim:
        out["side.embed"] = mat(V, cfg.side_dim * len(cfg.layers), 1.0)
    for i, l in enumerate(cfg.layers):
        mx, ff = l.mixer, l.mlp
        p = f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if ff is not None else ()):
            out[p + n] = vec(D, gamma_jitter, 1.0)
        if l.type == "general_delta":
            hd, rank = mx.heads * mx.dim, _decay_rank(mx)
            for n in ("r", "k", "v", "g", "a"):
                out[p + "mix." + n] = mat(hd, D)
            out[p + "mix.a.b"] = vec(hd, 0.5)
            out[p + "mix.w1"] = mat(rank, D)
            out[p + "mix.w2"] = mat(hd, rank)
            out[p + "mix.w0"] = vec(hd, 1.0)
            out[p + "mix.norm"] = vec(hd, gamma_jitter, 1.0)
            out[p + "mix.o"] = mat(D, hd)
        else:
            H, G, d = mx.heads, mx.kv_heads, mx.dim
            out[p + "mix.q"] = mat(H * d, D)
            out[p + "mix.k"] = mat(G * d, D)
            out[p + "mix.q.norm"] = vec(d, gamma_jitter, 1.0)
            out[p + "mix.k.norm"] = vec(d, gamma_jitter, 1.0)
            out[p + "mix.sink"] = vec(H, sink_std)
            out[p + "mix.o"] = mat(D, H * d)
        if isinstance(ff, DenseFFConfig):
            out[p + "mlp.up"] = mat(ff.ff, D)
            out[p + "mlp.up.b"] = vec(ff.ff, 0.1)
            out[p + "mlp.down"] = mat(D, ff.ff)
            out[p + "mlp.down.b"] = vec(D, 0.1)
            out[p + "mlp.act"] = vec(2, 0.5)
        elif isinstance(ff, MoEFFConfig):
            for k in range(ff.experts):
                out[f"{p}mlp.e{k}.up"] = mat(ff.ff, D)
                out[f"{p}mlp.e{k}.down"] = mat(D, ff.ff)
            out[p + "mlp.router"] = mat(ff.experts, D)
        if cfg.side_dim:
            out[p + "side.gate"] = mat(cfg.side_dim, D)
            out[p + "side.proj"] = mat(D, cfg.side_dim)
            out[p + "side.norm"] = vec(D, gamma_jitter, 1.0)
    out["final.norm"] = vec(D, gamma_jitter, 1.0)
    return out


ARCHITECTURE = register_architecture(Architecture(
    name="rizitar", config_cls=RizitarConfig, build_spec=build_spec, weight_plan=weight_plan,
    aliases=("Rizitar",), random_tensors=random_tensors, complete_config=complete_config),
    replace=True)
