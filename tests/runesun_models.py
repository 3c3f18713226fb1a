"""Small Runesun configurations with random weights for the tests, made here (own drawing of
the values, own writer of the weight file) so that the engine reads them as it reads any model
folder and the plain implementation gets the very same numbers as a dict."""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch


def _layer(heads, dim, vdim, rank, scale, moe=None, weights_of=None):
    e = {"type": "latent_attention",
         "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale},
         "mlp": None if moe is None else {"kind": "moe", "expert": {"ff": moe[2]},
                                          "router": {"experts": moe[0], "top": moe[1]}}}
    if weights_of is not None:
        e["weights_of"] = weights_of
    return e


# P: sizes that are all different and mostly odd; a layer without feed-forward; one expert of
#    one; a single head; a layer run twice
# Q: multiples of 8/16 (the tensor-core kernels' shapes), top = all experts in one layer
# R: the smallest of everything
# S: sizes that take the tensor-core kernels with ragged tiles (latents of 72, 8 and 200 in tiles
#    of 96, 32 and 256; 7 heads; experts narrower than a tile), the first layer running with a
#    later layer's tensors
CONFIGS = {
    "P": {"architecture": "Runesun", "vocab": 257, "width": 72, "norm": {"eps": 3e-5}, "layers": [
        _layer(3, 20, 12, 40, 0.3, moe=(5, 2, 24)),
        _layer(1, 16, 24, 24, 0.25),
        _layer(3, 20, 12, 40, 0.3, moe=(5, 2, 24), weights_of=0),
        _layer(4, 8, 8, 16, 0.5, moe=(3, 1, 40)),
    ]},
    "Q": {"architecture": "Runesun", "vocab": 320, "width": 128, "norm": {"eps": 1e-6}, "layers": [
        _layer(8, 32, 16, 64, 0.2, moe=(8, 3, 32)),
        _layer(16, 16, 32, 128, 0.25, moe=(4, 4, 64)),
        _layer(16, 16, 32, 128, 0.25, moe=(4, 4, 64), weights_of=1),
    ]},
    "R": {"architecture": "Runesun", "vocab": 31, "width": 8, "norm": {"eps": 1e-5}, "layers": [
        _layer(1, 1, 1, 1, 1.0, moe=(1, 1, 1)),
        _layer(2, 3, 1, 2, 0.7, moe=(2, 1, 5)),
    ]},
}
CONFIGS["S"] = {"architecture": "Runesun", "vocab": 333, "width": 200, "norm": {"eps": 1e-5}, "layers": [
    _layer(7, 24, 40, 72, 0.2, moe=(3, 3, 8), weights_of=2),
    _layer(2, 8, 8, 8, 0.35, moe=(9, 4, 200)),
    _layer(7, 24, 40, 72, 0.2, moe=(3, 3, 8)),
    _layer(5, 16, 24, 200, 0.25),
]}
SEEDS = {"P": 5, "Q": 6, "R": 7, "S": 8}


def make_tensors(cfg: dict, seed: int, sink_std: float = 1.5) -> dict[str, torch.Tensor]:
    """fp32 tensors whose values are exact in bfloat16."""
    g = torch.Generator().manual_seed(seed)

    def rnd(*shape, s=1.0, mean=0.0):
        return (torch.randn(*shape, generator=g) * s + mean).to(torch.bfloat16).float()

    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": rnd(V, D)}
    for i, l in enumerate(cfg["layers"]):
        if "weights_of" in l:
            continue
        m, p = l["mixer"], f"l{i}."
        H, d, dv, R = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
        out[p + "norm1"] = rnd(D, s=0.2, mean=1.0)
        out[p + "mix.q"] = rnd(H * d, D, s=1.5 / math.sqrt(D))
        out[p + "mix.dkv"] = rnd(R, D, s=1 / math.sqrt(D))
        out[p + "mix.dkv.norm"] = rnd(R, s=0.2, mean=1.0)
        out[p + "mix.uk"] = rnd(H * d, R, s=1.5 / math.sqrt(R))
        out[p + "mix.uv"] = rnd(H * dv, R, s=1 / math.sqrt(R))
        out[p + "mix.sink"] = rnd(H, s=sink_std)
        out[p + "mix.g"] = rnd(H, D, s=2 / math.sqrt(D))
        out[p + "mix.o"] = rnd(D, H * dv, s=1 / math.sqrt(H * dv))
        if l["mlp"] is not None:
            E, F = l["mlp"]["router"]["experts"], l["mlp"]["expert"]["ff"]
            for k in range(E):
                out[f"{p}mlp.e{k}.gate"] = rnd(F, D, s=1.5 / math.sqrt(D))
                out[f"{p}mlp.e{k}.up"] = rnd(F, D, s=1 / math.sqrt(D))
                out[f"{p}mlp.e{k}.down"] = rnd(D, F, s=1 / math.sqrt(F))
            out[p + "mlp.router"] = rnd(E, D, s=3 / math.sqrt(D))
    out["final.norm"] = rnd(D, s=0.2, mean=1.0)
    out["head"] = rnd(V, D, s=1 / math.sqrt(D))
    return out


def write_model(folder: Path, cfg: dict, tensors: dict[str, torch.Tensor]) -> Path:
    """config.json and model.safetensors (bfloat16): 8 bytes of header length, the JSON header,
    the data."""
    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    header, blobs, at = {}, [], 0
    for name, t in tensors.items():
        bits = (t.contiguous().view(torch.int32).numpy().astype(np.uint32) >> 16).astype("<u2")
        raw = bits.tobytes()
        header[name] = {"dtype": "BF16", "shape": list(t.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    head = json.dumps(header).encode()
    head += b" " * (-len(head) % 8)
    with open(folder / "model.safetensors", "wb") as f:
        f.write(struct.pack("<Q", len(head)))
        f.write(head)
        for b in blobs:
            f.write(b)
    return folder


def make(root: Path, name: str):
    """``(folder, config, tensors)`` of configuration ``name``."""
    cfg = CONFIGS[name]
    tensors = make_tensors(cfg, SEEDS[name])
    return write_model(Path(root) / f"runesun_{name}", cfg, tensors), cfg, tensors
