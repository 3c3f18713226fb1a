"""Small Rizitar configurations with random weights for the tests, made here (own drawing of
the values; the weight file is written by the Runesun tests' own writer) so that the engine
reads them as it reads any model folder and the plain implementation gets the very same numbers
as a dict."""
from __future__ import annotations

import math
from pathlib import Path

import torch

from runesun_models import write_model


def delta(heads, dim, mlp=None):
    return {"type": "general_delta", "mixer": {"heads": heads, "dim": dim}, "mlp": mlp}


def attn(heads, kv_heads, dim, scale, size=None, pool=None, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size, **({"pool": pool} if pool else {})}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


# A: odd sizes; both mixers twice; a window shorter than a page with pooled blocks, one longer
#    than a page; part of a head rotated with scaled frequencies, and a whole head without; a
#    layer without feed-forward; one expert of several; grouped and ungrouped key heads
# B: multiples of 16 (the tensor-core products), heads of 64, a window of two pages, top = all
#    experts, no per-token input, an embedding scale of one
# C: the smallest of everything: one head of two numbers, a window of one token with blocks of
#    one, one expert, a per-token input of one number; an attention layer that sees everything
# D: a window shorter than its blocks (a block's tokens leave the window before the block is
#    complete), blocks that straddle pages, heads of 33 and 96 channels in the delta rule
CONFIGS = {
    "A": {"architecture": "Rizitar", "vocab": 257, "width": 72, "norm": {"eps": 3e-5},
          "embedding": {"scale": 3.0}, "token_side": {"dim": 10}, "layers": [
        attn(4, 2, 16, 0.3, size=24, pool=4, rot=rot(8, 5000.0, (8.0, 64, 4.0, 0.5)), mlp=moe(5, 2, 24)),
        delta(3, 20, mlp=dense(100)),
        attn(3, 3, 24, 0.2, size=70, pool=5, rot=rot(24, 300.0), mlp=None),
        delta(2, 12, mlp=moe(3, 1, 40)),
    ]},
    "B": {"architecture": "Rizitar", "vocab": 320, "width": 128, "norm": {"eps": 1e-6},
          "embedding": {"scale": 1.0}, "layers": [
        delta(2, 64, mlp=moe(4, 4, 64)),
        attn(8, 2, 32, 0.18, size=128, pool=16, rot=rot(32, 10000.0, (2.0, 256, 16.0, 2.0)), mlp=dense(256)),
        attn(4, 1, 64, 0.12, size=130, pool=32, rot=rot(16, 10000.0), mlp=moe(8, 3, 32)),
    ]},
    "C": {"architecture": "Rizitar", "vocab": 31, "width": 8, "norm": {"eps": 1e-5},
          "embedding": {"scale": 0.5}, "token_side": {"dim": 1}, "layers": [
        attn(1, 1, 2, 1.0, size=1, pool=1, rot=rot(2, 10.0), mlp=moe(1, 1, 1)),
        delta(1, 1, mlp=dense(1)),
        attn(2, 1, 3, 0.7, mlp=dense(5)),
    ]},
    "D": {"architecture": "Rizitar", "vocab": 99, "width": 40, "norm": {"eps": 1e-6},
          "embedding": {"scale": 7.0}, "token_side": {"dim": 3}, "layers": [
        attn(2, 1, 8, 0.4, size=3, pool=7, rot=rot(6, 50.0), mlp=dense(24)),
        delta(1, 33, mlp=None),
        attn(4, 4, 8, 0.35, size=9, pool=9, mlp=moe(6, 2, 16)),
        delta(2, 96, mlp=dense(16)),
    ]},
}
# E: nothing is a multiple of 8 (the products' and the attention's paths for ragged sizes)
CONFIGS["E"] = {"architecture": "Rizitar", "vocab": 333, "width": 100, "norm": {"eps": 2e-6},
                "embedding": {"scale": 10.0}, "token_side": {"dim": 7}, "layers": [
    delta(3, 10, mlp=moe(5, 2, 30)),
    attn(5, 5, 20, 0.22, size=50, pool=3, rot=rot(10, 777.0, (3.0, 100, 5.0, 1.0)), mlp=dense(50)),
    attn(6, 2, 12, 0.3, size=13, pool=11, rot=rot(12, 2000.0), mlp=None),
]}
SEEDS = {"A": 11, "B": 12, "C": 13, "D": 14, "E": 15}
DECAY_RANK = {"A": 6, "B": 8, "C": 1, "D": 5, "E": 3}


def make_tensors(cfg: dict, seed: int, decay_rank: int, sink_std: float = 1.5) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).float()

    D, V = cfg["width"], cfg["vocab"]
    scale = cfg["embedding"]["scale"]
    out = {"embed": rnd(V, D, s=1.0 / scale)}
    n_side = cfg["token_side"]["dim"] if cfg.get("token_side") else 0
    if n_side:
        out["side.embed"] = rnd(V, n_side * len(cfg["layers"]))
    for i, l in enumerate(cfg["layers"]):
        m, ff, p = l["mixer"], l["mlp"], f"l{i}."
        for n in ("norm1", "norm1b") + (("norm2", "norm2b") if ff else ()):
            out[p + n] = rnd(D, s=0.2, mean=1.0)
        if l["type"] == "general_delta":
            hd = m["heads"] * m["dim"]
            for n in ("r", "k", "v", "g", "a"):
                out[p + "mix." + n] = rnd(hd, D, s=1.5 / math.sqrt(D))
            out[p + "mix.a.b"] = rnd(hd, s=0.7)
            out[p + "mix.w1"] = rnd(decay_rank, D, s=1.5 / math.sqrt(D))
            out[p + "mix.w2"] = rnd(hd, decay_rank, s=2.0 / math.sqrt(decay_rank))
            out[p + "mix.w0"] = rnd(hd, s=1.5)
            out[p + "mix.norm"] = rnd(hd, s=0.2, mean=1.0)
            out[p + "mix.o"] = rnd(D, hd, s=1 / math.sqrt(hd))
        else:
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            out[p + "mix.q"] = rnd(H * d, D, s=1.5 / math.sqrt(D))
            out[p + "mix.k"] = rnd(G * d, D, s=1.5 / math.sqrt(D))
            out[p + "mix.q.norm"] = rnd(d, s=0.3, mean=1.2)
            out[p + "mix.k.norm"] = rnd(d, s=0.3, mean=1.2)
            out[p + "mix.sink"] = rnd(H, s=sink_std)
            out[p + "mix.o"] = rnd(D, H * d, s=1 / math.sqrt(H * d))
        if ff and ff["kind"] == "dense":
            out[p + "mlp.up"] = rnd(ff["ff"], D, s=1.5 / math.sqrt(D))
            out[p + "mlp.up.b"] = rnd(ff["ff"], s=0.3)
            out[p + "mlp.down"] = rnd(D, ff["ff"], s=1 / math.sqrt(ff["ff"]))
            out[p + "mlp.down.b"] = rnd(D, s=0.3)
            out[p + "mlp.act"] = rnd(2, s=1.0)
        elif ff:
            E, F = ff["router"]["experts"], ff["expert"]["ff"]
            for k in range(E):
                out[f"{p}mlp.e{k}.up"] = rnd(F, D, s=1.5 / math.sqrt(D))
                out[f"{p}mlp.e{k}.down"] = rnd(D, F, s=1 / math.sqrt(F))
            out[p + "mlp.router"] = rnd(E, D, s=3 / math.sqrt(D))
        if n_side:
            out[p + "side.gate"] = rnd(n_side, D, s=1 / math.sqrt(D))
            out[p + "side.proj"] = rnd(D, n_side, s=1 / math.sqrt(n_side))
            out[p + "side.norm"] = rnd(D, s=0.2, mean=0.5)
    out["final.norm"] = rnd(D, s=0.2, mean=1.0)
    return out


def make(root: Path, name: str):
    """``(folder, config, tensors)`` of configuration ``name``."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, SEEDS[name], DECAY_RANK[name])
    return write_model(Path(root) / f"rizitar_{name}", cfg, tensors), cfg, tensors
