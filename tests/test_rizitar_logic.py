"""Rizitar without a GPU: its configuration and weight plan, and the engine's host side (state
rows, the two paged stores of an attention layer, slots, pages, batches, the generation loop)
on the torch-CPU stand-in of the kernel library, against the plain implementation."""
import copy

import pytest
import torch

import plain_rizitar as PZ
import rizitar_models as ZM
from nimbus_infer_rs_b200 import Engine, SamplingParams
from nimbus_infer_rs_b200.config import ConfigError, RizitarConfig
from nimbus_infer_rs_b200.config.registry import load_config, resolve_architecture
from nimbus_infer_rs_b200.parts.rotary import rotary_frequencies
from nimbus_infer_rs_b200.weights.loader import WeightError


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    root = tmp_path_factory.mktemp("rizitar")
    return {n: ZM.make(root, n) for n in ZM.CONFIGS}


def _tokens(vocab, n, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


def _close(got, ref, tol=3e-5):
    got, ref = got.double(), ref.double()
    assert got.shape == ref.shape
    assert float((got - ref).abs().max()) <= tol * float(ref.abs().max())


def _engine(models, name, **kw):
    kw.setdefault("cache_tokens", 1024)
    return Engine.load(models[name][0], dtype="float32", device="cpu", **kw)


def test_config_is_read_and_recognised(models):
    folder, cfg, _ = models["A"]
    arch, typed = load_config(folder)
    assert arch.name == "rizitar" and isinstance(typed, RizitarConfig)
    assert resolve_architecture({"architecture": "rizitar"}).name == "rizitar"
    assert typed.vocab_size == 257 and typed.width == 72 and typed.norm_eps == 3e-5
    assert typed.embedding_scale == 3.0 and typed.side_dim == 10
    a0, d1, a2 = typed.layers[0].mixer, typed.layers[1].mixer, typed.layers[2].mixer
    assert (a0.heads, a0.kv_heads, a0.dim, a0.window, a0.pool) == (4, 2, 16, 24, 4)
    assert a0.rot.dims == 8 and a0.rot.scaling.factor == 8.0 and a2.rot.scaling is None
    assert (d1.heads, d1.dim, d1.decay_rank) == (3, 20, None)
    assert typed.layers[2].mlp is None and typed.layers[3].mlp.top == 1
    assert RizitarConfig.from_json(typed.to_json()) == typed
    # the decay's rank comes from the weight file's shapes
    full = typed.with_shapes({"l1.mix.w1": (6, 72), "l3.mix.w1": (6, 72)})
    assert full.layers[1].mixer.decay_rank == 6
    assert RizitarConfig.from_json(full.to_json()) == full
    c = RizitarConfig.from_json(ZM.CONFIGS["C"])
    assert c.layers[2].mixer.window == 0 and c.layers[2].mixer.rot is None


def test_config_errors_name_every_bad_key():
    bad = copy.deepcopy(ZM.CONFIGS["A"])
    bad["layers"][0]["mixer"]["heads"] = 3           # no multiple of kv_heads
    bad["layers"][0]["mixer"]["rot"]["dims"] = 7
    bad["layers"][1]["type"] = "something_else"
    bad["layers"][2]["mixer"]["vdim"] = 8
    bad["layers"][3]["mlp"]["router"]["top"] = 9
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        RizitarConfig.from_json(bad)
    text = str(e.value)
    for piece in ("kv_heads=2", "rot.dims", "layers[1].type", "vdim", "top=9", "norm.eps"):
        assert piece in text, piece


def test_weight_errors_are_listed_together(models, tmp_path):
    folder, cfg, tensors = models["D"]
    t = dict(tensors)
    del t["l1.mix.w0"]
    t["l0.mix.sink"] = torch.zeros(3)
    t["stray"] = torch.zeros(2)
    ZM.write_model(tmp_path / "bad", cfg, t)
    with pytest.raises(WeightError) as e:
        Engine.load(tmp_path / "bad", dtype="float32", device="cpu")
    assert "l1.mix.w0" in e.value.missing and "stray" in e.value.unexpected
    assert any("l0.mix.sink" in w for w in e.value.wrong_shape)


def test_rotary_frequencies_against_the_plain_ones():
    for dims, base, sc in ((8, 5000.0, (8.0, 64, 4.0, 0.5)), (24, 300.0, None), (2, 10.0, None),
                           (64, 1e6, (32.0, 4096, 32.0, 1.0)), (6, 50.0, (1.5, 16, 2.0, 1.0))):
        r = {"dims": dims, "base": base}
        scaling = None
        if sc:
            scaling = dict(zip(("factor", "original", "fast", "slow"), sc))
            r["scaling"] = scaling
        f, amp = rotary_frequencies(dims, base, scaling)
        pf, pamp = PZ.rotary_frequencies(r)
        assert f.dtype == torch.float32 and f.shape == (dims // 2,)
        assert torch.allclose(f.double(), pf, rtol=1e-7, atol=0) and abs(amp - pamp) < 1e-12


@pytest.mark.parametrize("name", ["A", "C", "D", "E"])
def test_whole_prompts_and_token_by_token(models, cpu_backend, name):
    _, cfg, P = models[name]
    e = _engine(models, name)
    for n in (1, 2, 37, 80):
        toks = _tokens(cfg["vocab"], n, n)
        ref = PZ.forward(cfg, P, toks)
        s = e.alloc_slot()
        _close(e.step([(s, toks, list(range(n)))]), ref)
        e.free_slot(s)
        s = e.alloc_slot()
        one = torch.cat([e.step([(s, [t], [0])]) for t in toks])
        _close(one, ref)
        e.free_slot(s)


def test_layer_by_layer(models, cpu_backend):
    _, cfg, P = models["A"]
    e = _engine(models, "A")
    snaps = []
    for layer in e.model.layers:
        f = layer.block.forward
        layer.block.forward = lambda ctx, x, l, f=f: (f(ctx, x, l), snaps.append(x.clone()))[0]
    toks = _tokens(257, 50, 5)
    s = e.alloc_slot()
    e.step([(s, toks, [0])])
    _, ref = PZ.forward(cfg, P, toks, return_layers=True)
    for got, want in zip(snaps, ref):
        _close(got[:50], want)


def test_portions_down_to_two_tokens(models, cpu_backend):
    _, cfg, P = models["D"]
    e = _engine(models, "D")
    toks = _tokens(99, 150, 3)
    s, at, outs = e.alloc_slot(), 0, []
    for size in (2, 61, 1, 2, 64, 3, 17):        # ends on and beside page, window and block ends
        outs.append(e.step([(s, toks[at:at + size], list(range(size)))]))
        at += size
    _close(torch.cat(outs), PZ.forward(cfg, P, toks))


def test_unequal_batch_on_slots_and_pages_used_again(models, cpu_backend):
    """Two batches of unequal prompts decoded together on a cache that holds one batch: the
    second gets the slots, pages and state rows of the first."""
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=5 * 64, n_slots=3)
    for round_, lens in enumerate(((100, 5, 66), (1, 90, 30))):
        seqs = [_tokens(257, n, 17 * round_ + i) for i, n in enumerate(lens)]
        heads = [max(1, n - 3 - i) for i, n in enumerate(lens)]
        slots = [e.alloc_slot() for _ in lens]
        got = {i: [] for i in range(3)}
        out = e.step([(slots[i], seqs[i][:heads[i]], [heads[i] - 1]) for i in range(3)])
        for i in range(3):
            got[i].append(out[i])
        k = 0
        while True:
            live = [i for i in range(3) if heads[i] + k < lens[i]]
            if not live:
                break
            out = e.step([(slots[i], [seqs[i][heads[i] + k]], [0]) for i in live])
            for j, i in enumerate(live):
                got[i].append(out[j])
            k += 1
        for i in range(3):
            ref = PZ.forward(cfg, P, seqs[i])
            _close(torch.stack(got[i]), ref[heads[i] - 1:])
            e.free_slot(slots[i])
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_pages_go_back_once_window_and_block_have_passed(models, cpu_backend):
    """A windowed layer keeps a page while one of its tokens is in a later window or its block
    is incomplete; the store of blocks grows by an entry per complete block."""
    e = _engine(models, "D")
    s = e.alloc_slot()
    toks = _tokens(99, 300, 1)
    for t in toks:
        e.step([(s, [t], [])])
    by_every = {}
    for g in e.cache.groups:
        by_every.setdefault((g.request.every, g.request.window), []).append(len(g.pages_of(s)))
    assert by_every[(1, 7)] == [1] or by_every[(1, 7)] == [2]        # window 3 under blocks of 7
    assert by_every[(7, 0)] == [1]                                    # 42 blocks: one page
    assert by_every[(9, 0)] == [1]
    e.free_slot(s)
    assert all(g.pool.n_free == g.pool.n_pages for g in e.cache.groups)


def test_state_rows_start_at_zero_for_every_new_sequence(models, cpu_backend):
    _, cfg, P = models["D"]
    e = _engine(models, "D", n_slots=1)
    ref = PZ.forward(cfg, P, _tokens(99, 20, 4))
    for _ in range(2):
        s = e.alloc_slot()
        _close(e.step([(s, _tokens(99, 20, 4), list(range(20)))]), ref)
        e.free_slot(s)


def test_greedy_generation_through_the_engines_loop(models, cpu_backend):
    _, cfg, P = models["A"]
    e = _engine(models, "A", cache_tokens=6 * 64, n_slots=3)
    prompts = [_tokens(257, n, 50 + n) for n in (5, 30, 1, 64)]
    out = e.generate(prompts, SamplingParams(max_new_tokens=8, temperature=0.0), max_batch=3)
    for p, got in zip(prompts, out):
        assert len(got) == 8
        ctx = list(p)
        for tok in got:
            logits = PZ.forward(cfg, P, ctx)[-1]
            want = int(torch.argmax(logits))
            if tok != want:
                assert float(logits[want] - logits[tok]) <= 1e-4 * float(logits.abs().max())
                break
            ctx.append(tok)
    assert e.cache.slots.n_free == 3


def test_random_weights_mode_and_inspect(cpu_backend):
    cfg = RizitarConfig.from_json(ZM.CONFIGS["A"])
    e = Engine.random(cfg, seed=3, dtype="float32", device="cpu", cache_tokens=256)
    s = e.alloc_slot()
    out = e.step([(s, [1, 2, 3], [2])])
    assert out.shape == (1, 257) and torch.isfinite(out).all()
    info = e.inspect()
    assert info["architecture"] == "rizitar" and info["layers"] == 4 and info["tie_head"] is True


def test_command_line_and_trace_replay_take_the_design(cpu_backend, tmp_path, monkeypatch, capsys):
    """`random` writes a Rizitar folder from a preset (its config.json carries the decay's rank,
    so the folder reads back without the hook on the shapes too); `trace_run` replays steps on it."""
    import importlib.machinery
    import importlib.util
    import io
    import json
    import sys
    from pathlib import Path

    import numpy as np

    from nimbus_infer_rs_b200.__main__ import main
    from nimbus_infer_rs_b200.weights.safetensors_io import SafeTensorsFile
    folder = tmp_path / "m"
    assert main(["random", "--out", str(folder), "--preset", "rizitar-tiny", "--seed", "3"]) == 0
    wrote = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    cfg = json.loads((folder / "config.json").read_text())
    assert cfg["architecture"] == "Rizitar" and cfg["layers"][0]["mixer"]["decay_rank"] == 8
    with SafeTensorsFile(folder / "model.safetensors") as f:
        assert wrote["n_params"] == sum(f.tensor(n).numel() for n in f.names())
        P = {n: f.tensor(n).float() for n in f.names()}
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
    a, b = PZ.forward(cfg, P, [1, 2, 3, 4, 5]), PZ.forward(cfg, P, [9, 8])
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, -1))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(2, -1))
    _close(got0, a[[1, 3]])
    _close(got1, torch.stack([a[4], b[1]]))
