"""Runesun without a GPU: its configuration and weight plan, and the engine's host side (run
order of layers that share tensors, caches per run, slots, pages, batches, the generation loop)
on the torch-CPU stand-in of the kernel library, against the plain implementation."""
import copy
import json

import pytest
import torch

import plain_runesun as PR
import runesun_models as RM
from nimbus_infer_rs_b200 import Engine, SamplingParams
from nimbus_infer_rs_b200.config import ConfigError, RunesunConfig
from nimbus_infer_rs_b200.config.registry import load_config, resolve_architecture
from nimbus_infer_rs_b200.weights.loader import WeightError


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("runesun")
    return {n: RM.make(root, n) for n in RM.CONFIGS}


def _tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _close(got, ref, tol=2e-5):
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= tol * float(ref.abs().max())


def test_config_is_read_and_recognised(models):
    folder, cfg, _ = models["P"]
    arch, typed = load_config(folder)
    assert arch.name == "runesun" and isinstance(typed, RunesunConfig)
    assert resolve_architecture({"architecture": "runesun"}).name == "runesun"
    assert typed.vocab_size == 257 and typed.width == 72 and typed.norm_eps == 3e-5
    assert [l.weights_of for l in typed.layers] == [None, None, 0, None]
    assert typed.layers[1].mlp is None and typed.layers[3].mlp.top == 1
    assert typed.layers[0].mixer.kv_rank == 40 and typed.layers[0].mixer.scale == 0.3
    again = RunesunConfig.from_json(typed.to_json())
    assert again == typed


def test_config_errors_name_every_bad_key():
    bad = copy.deepcopy(RM.CONFIGS["P"])
    bad["layers"][0]["mixer"]["heads"] = 0
    bad["layers"][1]["type"] = "something_else"
    bad["layers"][3]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["weights_of"] = 2
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        RunesunConfig.from_json(bad)
    text = str(e.value)
    for piece in ("layers[0].mixer.heads", "layers[1].type", "top=9", "layers[2].weights_of", "norm.eps"):
        assert piece in text, piece
    loop = copy.deepcopy(RM.CONFIGS["P"])
    loop["layers"][0]["weights_of"] = 2
    with pytest.raises(ConfigError, match="circle"):
        RunesunConfig.from_json(loop)


def test_layers_that_share_tensors_are_one_set_of_parts_run_twice(models, cpu_backend):
    folder, cfg, _ = models["P"]
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=256)
    assert len(e.model.layers) == 3 and e.model.run_order == (0, 1, 0, 2)
    kv, _ = e.model.storage_requests()
    assert sorted(kv) == [0, 1, 2, 3]                       # a cache per run, not per layer
    assert all(r.planes == 1 and r.n_kv_heads == 1 for r in kv.values())
    assert kv[0].head_dim == 40 and kv[1].head_dim == 24 and kv[3].head_dim == 16
    assert e.model.layers[1].ffn is None and e.model.layers[1].norm_ffn is None
    assert e.spec.max_seq_len == 256                         # bounded by the cache only
    assert e.graph_safe


def test_missing_and_misshapen_tensors_are_listed(models, tmp_path):
    _, cfg, tensors = models["P"]
    t = dict(tensors)
    del t["l0.mix.sink"]
    t["l3.mlp.e1.up"] = t["l3.mlp.e1.up"][:, :-1].contiguous()
    t["l2.norm1"] = t["l0.norm1"]                            # layer 2 has no tensors of its own
    folder = RM.write_model(tmp_path / "bad", cfg, t)
    with pytest.raises(WeightError) as e:
        Engine.load(folder, dtype="float32", device="cpu")
    assert "l0.mix.sink" in e.value.missing
    assert "l2.norm1" in e.value.unexpected
    assert any("l3.mlp.e1.up" in w for w in e.value.wrong_shape)


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompts_and_token_by_token(models, cpu_backend, name):
    folder, cfg, P = models[name]
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=512)
    for n in (1, 2, 70):
        toks = _tokens(cfg["vocab"], n, 100 + n)
        ref = PR.forward(toks, P, cfg)
        s = e.alloc_slot()
        _close(e.step([(s, toks, list(range(n)))]), ref)
        e.free_slot(s)
        s = e.alloc_slot()
        outs = [e.step([(s, [t], [0])]) for t in toks[:min(n, 6)]]
        e.free_slot(s)
        _close(torch.cat(outs), ref[:min(n, 6)])


def test_unequal_batch_then_decoded_together_on_reused_slots_and_pages(models, cpu_backend):
    folder, cfg, P = models["P"]
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=4 * 64, n_slots=3)
    for round_ in range(2):                                  # the second round reuses everything
        seqs = [_tokens(257, n, 7 * round_ + n) for n in (66, 3, 61)]
        heads = [60, 1, 59]
        refs = [PR.forward(t, P, cfg) for t in seqs]
        slots = [e.alloc_slot() for _ in seqs]
        out = e.step([(s, t[:h], [h - 1]) for s, t, h in zip(slots, seqs, heads)])
        _close(out, torch.stack([r[h - 1] for r, h in zip(refs, heads)]))
        live = [0, 1, 2]
        for k in range(6):
            live = [i for i in live if heads[i] + k < len(seqs[i])]
            out = e.step([(slots[i], [seqs[i][heads[i] + k]], [0]) for i in live])
            _close(out, torch.stack([refs[i][heads[i] + k] for i in live]))
        for s in slots:
            e.free_slot(s)
        assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_portions_down_to_two_tokens(models, cpu_backend):
    folder, cfg, P = models["Q"]
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=256)
    toks = _tokens(320, 75, 1)
    ref = PR.forward(toks, P, cfg)
    s = e.alloc_slot()
    at, outs = 0, []
    for size in (2, 61, 2, 3, 7):
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    e.free_slot(s)
    _close(torch.cat(outs), ref)


def test_greedy_generation_through_the_engines_loop(models, cpu_backend):
    folder, cfg, P = models["P"]
    e = Engine.load(folder, dtype="float32", device="cpu", cache_tokens=6 * 64, n_slots=2)
    prompts = [_tokens(257, n, 40 + n) for n in (5, 62, 1)]
    out = e.generate(prompts, SamplingParams(max_new_tokens=5, temperature=0.0), max_batch=2)
    for p, got in zip(prompts, out):
        ctx = list(p)
        for tok in got:
            logits = PR.forward(ctx, P, cfg)[-1]
            assert tok == int(torch.argmax(logits))
            ctx.append(tok)
        assert len(got) == 5
    assert e.cache.slots.n_free == 2


def test_random_weights_mode_and_inspect(cpu_backend):
    cfg = RunesunConfig.from_json(RM.CONFIGS["R"])
    a = Engine.random(cfg, seed=1, dtype="float32", device="cpu", cache_tokens=64)
    b = Engine.random(RM.CONFIGS["R"], seed=1, dtype="float32", device="cpu", cache_tokens=64)
    s, t = a.alloc_slot(), b.alloc_slot()
    assert torch.equal(a.step([(s, [1, 2, 3], [2])]), b.step([(t, [1, 2, 3], [2])]))
    info = a.inspect()
    assert info["architecture"] == "runesun" and info["mixer"] == "latent_attention"
    assert info["ffn"] == "routed_experts" and info["norm"] == "rmsnorm" and info["pos"] == "none"
    json.dumps(info)


def test_command_line_and_trace_replay_take_the_design(cpu_backend, tmp_path, monkeypatch, capsys):
    """`random` writes a model folder of the preset; `logits` and trace replay read it back
    through the registry like any other model."""
    import importlib.machinery
    import importlib.util
    import io
    import sys
    from pathlib import Path

    import numpy as np

    from nimbus_infer_rs_b200.__main__ import main
    folder = tmp_path / "m"
    assert main(["random", "--out", str(folder), "--preset", "runesun-tiny", "--seed", "3"]) == 0
    wrote = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    cfg = json.loads((folder / "config.json").read_text())
    assert cfg["architecture"] == "Runesun" and cfg["layers"][2]["weights_of"] == 0
    from nimbus_infer_rs_b200.weights.safetensors_io import SafeTensorsFile
    with SafeTensorsFile(folder / "model.safetensors") as f:
        assert wrote["n_params"] == sum(f.tensor(n).numel() for n in f.names())
    Engine.load(folder, dtype="float32", device="cpu", cache_tokens=128)

    root = Path(__file__).resolve().parent.parent
    loader = importlib.machinery.SourceFileLoader("trace_run_program", str(root / "bin" / "trace_run"))
    mod = importlib.util.module_from_spec(importlib.util.spec_from_loader(loader.name, loader))
    loader.exec_module(mod)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": [1, 2, 3, 4], "want": [1, 3]},
                                     {"id": "b", "tokens": [9], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [5], "want": [0]},
                                     {"id": "b", "tokens": [8], "want": [0]}], "end": ["a", "b"]}]
    out = tmp_path / "out"
    monkeypatch.setattr(sys, "argv", ["trace_run", "--model", str(folder), "--dtype", "float32", "--out",
                                      str(out), "--max-tokens", "128", "--device", "cpu"])
    monkeypatch.setattr(sys, "stdin", io.StringIO("".join(json.dumps(s) + "\n" for s in steps)))
    assert mod.main() == 0
    assert [l for l in capsys.readouterr().out.split("\n") if l] == ["done 0", "done 1"]
    from nimbus_infer_rs_b200.weights.safetensors_io import SafeTensorsFile
    with SafeTensorsFile(folder / "model.safetensors") as f:
        P = {n: f.tensor(n).float() for n in f.names()}
    a, b = PR.forward([1, 2, 3, 4, 5], P, cfg), PR.forward([9, 8], P, cfg)
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1))
    _close(got0, a[[1, 3]])
    _close(got1, torch.stack([a[4], b[1]]))
