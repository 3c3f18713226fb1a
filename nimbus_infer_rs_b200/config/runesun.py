"""Typed configuration of the Runesun decoder.

config.json of this design::

    {"architecture": "Runesun", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "vdim": dv, "kv_rank": r, "scale": s},
                 "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k}}
                        | null,
                 "weights_of": j (optional)}, ...]}

Every size and constant is read from there; layers may differ from one another.  A layer with
``weights_of: j`` has no tensors of its own and runs with layer ``j``'s (its own cache).
Nothing bounds the length of a sequence (there is no position encoding).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any

from .base import ConfigError

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("moe",)


@dataclass(frozen=True)
class LatentMixerConfig:
    heads: int
    dim: int          # query/key size per head
    vdim: int         # value size per head
    kv_rank: int      # size of the cached latent
    scale: float      # multiplies the scores


@dataclass(frozen=True)
class MoEConfig:
    experts: int
    top: int
    ff: int           # an expert's hidden size


@dataclass(frozen=True)
class RunesunLayerConfig:
    type: str
    mixer: LatentMixerConfig
    mlp: MoEConfig | None
    weights_of: int | None = None


def _int(problems, where, obj, key, minimum=1):
    v = obj.get(key) if isinstance(obj, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)) or float(v) != int(v):
        problems.append(f"{where}.{key}: expected an integer, got {v!r}")
        return minimum
    if int(v) < minimum:
        problems.append(f"{where}.{key}: must be at least {minimum} (got {v!r})")
        return minimum
    return int(v)


def _float(problems, where, obj, key, positive=True):
    v = obj.get(key) if isinstance(obj, dict) else None
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        problems.append(f"{where}.{key}: expected a number, got {v!r}")
        return 1.0
    if positive and not float(v) > 0:
        problems.append(f"{where}.{key}: must be positive (got {v!r})")
        return 1.0
    return float(v)


@dataclass(frozen=True)
class RunesunConfig:
    architecture = "runesun"

    vocab_size: int
    width: int
    norm_eps: float
    layers: tuple[RunesunLayerConfig, ...]
    name: str = "model"

    @classmethod
    def from_json(cls, obj: dict) -> "RunesunConfig":
        if not isinstance(obj, dict):
            raise ConfigError("config.json must hold a JSON object")
        problems: list[str] = []
        vocab = _int(problems, "config", obj, "vocab")
        width = _int(problems, "config", obj, "width")
        eps = _float(problems, "norm", obj.get("norm"), "eps")
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
            m = entry.get("mixer")
            mixer = LatentMixerConfig(
                heads=_int(problems, where + ".mixer", m, "heads"),
                dim=_int(problems, where + ".mixer", m, "dim"),
                vdim=_int(problems, where + ".mixer", m, "vdim"),
                kv_rank=_int(problems, where + ".mixer", m, "kv_rank"),
                scale=_float(problems, where + ".mixer", m, "scale", positive=False))
            mlp = None
            f = entry.get("mlp")
            if f is not None:
                if not isinstance(f, dict) or f.get("kind") not in MLP_KINDS:
                    problems.append(f"{where}.mlp.kind: unknown feed-forward "
                                    f"{f.get('kind') if isinstance(f, dict) else f!r} "
                                    f"(known: {list(MLP_KINDS)}, or null)")
                else:
                    mlp = MoEConfig(
                        experts=_int(problems, where + ".mlp.router", f.get("router"), "experts"),
                        top=_int(problems, where + ".mlp.router", f.get("router"), "top"),
                        ff=_int(problems, where + ".mlp.expert", f.get("expert"), "ff"))
                    if mlp.top > mlp.experts:
                        problems.append(f"{where}.mlp.router: top={mlp.top} of {mlp.experts} experts")
            wo = entry.get("weights_of")
            if wo is not None:
                if isinstance(wo, bool) or not isinstance(wo, int) or not 0 <= wo < len(raw_layers) \
                        or wo == i:
                    problems.append(f"{where}.weights_of: {wo!r} is not another layer")
                    wo = None
            layers.append(RunesunLayerConfig(kind, mixer, mlp, wo))
        if problems:
            raise ConfigError("bad config.json: " + "; ".join(problems))
        cfg = cls(vocab_size=vocab, width=width, norm_eps=eps, layers=tuple(layers),
                  name=str(obj.get("name", "model")))
        for i in range(len(layers)):
            cfg.owner(i)                  # a chain that never reaches tensors fails here
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer ``i`` runs with (``i`` itself if it has its own)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"bad config.json: layers[{i}].weights_of goes round in a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def n_params(self, *_unused) -> int:
        """Parameters of the layers that have tensors of their own, the embedding and the head."""
        total = 2 * self.vocab_size * self.width + self.width
        for i, l in enumerate(self.layers):
            if l.weights_of is not None:
                continue
            m, D = l.mixer, self.width
            total += D + m.heads * m.dim * D + m.kv_rank * D + m.kv_rank + m.heads * m.dim * m.kv_rank \
                + m.heads * m.vdim * m.kv_rank + m.heads + m.heads * D + D * m.heads * m.vdim
            if l.mlp is not None:
                total += l.mlp.experts * (3 * l.mlp.ff * D + D)
        return total

    def to_json(self) -> dict[str, Any]:
        out = []
        for l in self.layers:
            e: dict[str, Any] = {"type": l.type, "mixer": {
                "heads": l.mixer.heads, "dim": l.mixer.dim, "vdim": l.mixer.vdim,
                "kv_rank": l.mixer.kv_rank, "scale": l.mixer.scale}}
            e["mlp"] = None if l.mlp is None else {
                "kind": "moe", "expert": {"ff": l.mlp.ff},
                "router": {"experts": l.mlp.experts, "top": l.mlp.top}}
            if l.weights_of is not None:
                e["weights_of"] = l.weights_of
            out.append(e)
        return {"architecture": "Runesun", "name": self.name, "vocab": self.vocab_size,
                "width": self.width, "norm": {"eps": self.norm_eps}, "layers": out}
