"""Typed configuration of the Rizitar decoder.

config.json of this design::

    {"architecture": "Rizitar", "vocab": V, "width": D, "norm": {"eps": e},
     "embedding": {"scale": s}, "token_side": {"dim": n} (optional),
     "layers": [
       {"type": "general_delta", "mixer": {"heads": H, "dim": d},
        "mlp": {"kind": "dense", "ff": F} | {"kind": "moe", "expert": {"ff": F},
               "router": {"experts": E, "top": k}} | null},
       {"type": "attention",
        "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": d, "scale": c,
                  "mask": {"size": W, "pool": P},
                  "rot": {"dims": r, "base": b,
                          "scaling": {"factor": f, "original": n, "fast": x, "slow": y}}},
        "mlp": ...}, ...]}

Every size and constant is read from there; layers come in any order and may differ from one
another.  ``mask``, ``mask.pool``, ``rot`` and ``rot.scaling`` may be left out (then there is no
window, no pooled block, no rotation, no frequency scaling).  One size is not in config.json:
the rank of the decay's two-step projection in a ``general_delta`` mixer, which the weight
file's tensor shapes give (``decay_rank``; a config written by this library carries it).
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Any

from .base import ConfigError
from .runesun import _float, _int

MIXER_TYPES = ("general_delta", "attention")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RotaryConfig:
    dims: int
    base: float
    scaling: RotaryScaling | None = None


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    window: int = 0          # 0: every earlier token is seen
    pool: int = 0            # 0: no pooled blocks before the window
    rot: RotaryConfig | None = None


@dataclass(frozen=True)
class DeltaMixerConfig:
    heads: int
    dim: int
    decay_rank: int | None = None     # from the weight file's shapes when config.json has none


@dataclass(frozen=True)
class DenseFFConfig:
    ff: int


@dataclass(frozen=True)
class MoEFFConfig:
    experts: int
    top: int
    ff: int


@dataclass(frozen=True)
class RizitarLayerConfig:
    type: str
    mixer: Any
    mlp: Any            # DenseFFConfig, MoEFFConfig or None


def _read_rot(problems, where, m) -> RotaryConfig | None:
    rot = m.get("rot") if isinstance(m, dict) else None
    if rot is None:
        return None
    if not isinstance(rot, dict):
        problems.append(f"{where}.rot: expected an object")
        return None
    dims = _int(problems, where + ".rot", rot, "dims", minimum=2)
    if dims % 2:
        problems.append(f"{where}.rot.dims: must be even (got {dims})")
    base = _float(problems, where + ".rot", rot, "base")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        scaling = RotaryScaling(
            factor=_float(problems, where + ".rot.scaling", sc, "factor"),
            original=_float(problems, where + ".rot.scaling", sc, "original"),
            fast=_float(problems, where + ".rot.scaling", sc, "fast"),
            slow=_float(problems, where + ".rot.scaling", sc, "slow"))
    return RotaryConfig(dims, base, scaling)


def _read_mixer(problems, where, kind, m):
    if kind == "general_delta":
        rank = None
        if isinstance(m, dict) and m.get("decay_rank") is not None:
            rank = _int(problems, where, m, "decay_rank")
        return DeltaMixerConfig(heads=_int(problems, where, m, "heads"),
                                dim=_int(problems, where, m, "dim"), decay_rank=rank)
    heads = _int(problems, where, m, "heads")
    kv_heads = _int(problems, where, m, "kv_heads") if isinstance(m, dict) and "kv_heads" in m else heads
    dim = _int(problems, where, m, "dim")
    if heads % kv_heads:
        problems.append(f"{where}: heads={heads} is no multiple of kv_heads={kv_heads}")
    if isinstance(m, dict) and m.get("vdim") is not None and m.get("vdim") != dim:
        # the values are the keys as projected, so they have the keys' size
        problems.append(f"{where}.vdim: must equal dim={dim} (got {m.get('vdim')!r})")
    window = pool = 0
    mask = m.get("mask") if isinstance(m, dict) else None
    if mask is not None:
        window = _int(problems, where + ".mask", mask, "size")
        if isinstance(mask, dict) and mask.get("pool") is not None:
            pool = _int(problems, where + ".mask", mask, "pool")
    rot = _read_rot(problems, where, m)
    if rot is not None and rot.dims > dim:
        problems.append(f"{where}.rot.dims: {rot.dims} is more than the head's {dim}")
    return AttentionMixerConfig(heads=heads, kv_heads=kv_heads, dim=dim,
                                scale=_float(problems, where, m, "scale", positive=False),
                                window=window, pool=pool, rot=rot)


def _read_mlp(problems, where, f):
    if f is None:
        return None
    if not isinstance(f, dict) or f.get("kind") not in MLP_KINDS:
        problems.append(f"{where}.kind: unknown feed-forward "
                        f"{f.get('kind') if isinstance(f, dict) else f!r} "
                        f"(known: {list(MLP_KINDS)}, or null)")
        return None
    if f["kind"] == "dense":
        return DenseFFConfig(ff=_int(problems, where, f, "ff"))
    mlp = MoEFFConfig(experts=_int(problems, where + ".router", f.get("router"), "experts"),
                      top=_int(problems, where + ".router", f.get("router"), "top"),
                      ff=_int(problems, where + ".expert", f.get("expert"), "ff"))
    if mlp.top > mlp.experts:
        problems.append(f"{where}.router: top={mlp.top} of {mlp.experts} experts")
    return mlp


@dataclass(frozen=True)
class RizitarConfig:
    architecture = "rizitar"

    vocab_size: int
    width: int
    norm_eps: float
    embedding_scale: float
    side_dim: int                 # 0: no per-layer token input
    layers: tuple[RizitarLayerConfig, ...]
    name: str = "model"

    @classmethod
    def from_json(cls, obj: dict) -> "RizitarConfig":
        if not isinstance(obj, dict):
            raise ConfigError("config.json must hold a JSON object")
        problems: list[str] = []
        vocab = _int(problems, "config", obj, "vocab")
        width = _int(problems, "config", obj, "width")
        eps = _float(problems, "norm", obj.get("norm"), "eps")
        scale = 1.0
        if obj.get("embedding") is not None:
            scale = _float(problems, "embedding", obj.get("embedding"), "scale", positive=False)
        side = 0
        if obj.get("token_side") is not None:
            side = _int(problems, "token_side", obj.get("token_side"), "dim")
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("bad config.json: layers: expected a non-empty list"
                              + ("; " + "; ".join(problems) if problems else ""))
        layers = []
        for i, entry in enumerate(raw_layers):
            where = f"layers[{i}]"
            if not isinstance(entry, dict):
                problems.append(f"{where}: expected an object")
                continue
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                problems.append(f"{where}.type: unknown mixer {kind!r} (known: {list(MIXER_TYPES)})")
                continue
            mixer = _read_mixer(problems, where + ".mixer", kind, entry.get("mixer"))
            mlp = _read_mlp(problems, where + ".mlp", entry.get("mlp"))
            layers.append(RizitarLayerConfig(kind, mixer, mlp))
        if problems:
            raise ConfigError("bad config.json: " + "; ".join(problems))
        return cls(vocab_size=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   side_dim=side, layers=tuple(layers), name=str(obj.get("name", "model")))

    def with_shapes(self, shapes: dict) -> "RizitarConfig":
        """The sizes that only the weight file knows, read off its tensor shapes
        (``{name: shape}``): the rank of every ``general_delta`` mixer's decay projection."""
        layers = []
        for i, l in enumerate(self.layers):
            if l.type == "general_delta" and l.mixer.decay_rank is None:
                shape = shapes.get(f"l{i}.mix.w1")
                if shape is not None and len(shape) == 2:
                    l = replace(l, mixer=replace(l.mixer, decay_rank=int(shape[0])))
            layers.append(l)
        return replace(self, layers=tuple(layers))

    def n_params(self, *_unused) -> int:
        D, total = self.width, self.vocab_size * self.width + self.width
        total += self.vocab_size * self.side_dim * len(self.layers)
        for l in self.layers:
            m = l.mixer
            total += (4 if l.mlp is not None else 2) * D + (2 * self.side_dim * D + D if self.side_dim else 0)
            if l.type == "general_delta":
                hd, r = m.heads * m.dim, m.decay_rank or 0
                total += 6 * hd * D + r * D + hd * r + 3 * hd
            else:
                total += 2 * m.heads * m.dim * D + m.kv_heads * m.dim * D + 2 * m.dim + m.heads
            if isinstance(l.mlp, DenseFFConfig):
                total += 2 * l.mlp.ff * D + l.mlp.ff + D + 2
            elif isinstance(l.mlp, MoEFFConfig):
                total += l.mlp.experts * (2 * l.mlp.ff * D + D)
        return total

    def to_json(self) -> dict[str, Any]:
        out = []
        for l in self.layers:
            m = l.mixer
            if l.type == "general_delta":
                mx: dict[str, Any] = {"heads": m.heads, "dim": m.dim}
                if m.decay_rank is not None:
                    mx["decay_rank"] = m.decay_rank
            else:
                mx = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.dim,
                      "scale": m.scale}
                if m.window:
                    mx["mask"] = {"size": m.window, **({"pool": m.pool} if m.pool else {})}
                if m.rot is not None:
                    mx["rot"] = {"dims": m.rot.dims, "base": m.rot.base}
                    if m.rot.scaling is not None:
                        s = m.rot.scaling
                        mx["rot"]["scaling"] = {"factor": s.factor, "original": s.original,
                                                "fast": s.fast, "slow": s.slow}
            if l.mlp is None:
                ff = None
            elif isinstance(l.mlp, DenseFFConfig):
                ff = {"kind": "dense", "ff": l.mlp.ff}
            else:
                ff = {"kind": "moe", "expert": {"ff": l.mlp.ff},
                      "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            out.append({"type": l.type, "mixer": mx, "mlp": ff})
        obj: dict[str, Any] = {"architecture": "Rizitar", "name": self.name, "vocab": self.vocab_size,
                               "width": self.width, "norm": {"eps": self.norm_eps},
                               "embedding": {"scale": self.embedding_scale}, "layers": out}
        if self.side_dim:
            obj["token_side"] = {"dim": self.side_dim}
        return obj
