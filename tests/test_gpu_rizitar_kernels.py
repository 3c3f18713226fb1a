"""Rizitar's mechanisms alone on the GPU, each against its plain restatement in float64, with
inputs made so that a fault shows: a query that points at one far block among hundreds of keys,
keys just inside and just outside a window, blocks just seen and not yet seen, a sink that takes
all the weight, a state that has to remember its first token, portions and page ends."""
import math

import pytest
import torch

import plain_rizitar as PZ
from nimbus_infer_rs_b200.cache import SequenceCache
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.csrc.ops import ACT_RELU2, ACT_TANH, ACT_XIELU
from nimbus_infer_rs_b200.engine.batch import build_layout
from nimbus_infer_rs_b200.parts.base import KVRequest
from nimbus_infer_rs_b200.parts.rotary import rotary_frequencies

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
ACT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def ops():
    return ops_mod.backend()


def _rnd(*shape, seed=0, s=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * s


def _close(got, ref, tol, what=""):
    got, ref = got.double().cpu(), ref.double().cpu()
    assert got.shape == ref.shape, what
    assert torch.isfinite(got).all(), what
    err = float((got - ref).abs().max())
    assert err <= tol * max(float(ref.abs().max()), 1e-30), f"{what}: {err:.3e}"


# ----------------------------------------------------------------------------- row passes
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [1, 7, 72, 256, 1000, 4100])
def test_norm_of_a_result_added_to_the_stream(ops, dtype, d):
    n = 9
    y, x = _rnd(n, d, seed=1, s=3.0), _rnd(n, d, seed=2)
    g, g2 = _rnd(d, seed=3) + 1.0, _rnd(d, seed=4) + 1.0
    x1 = x.double() + PZ.rms_norm(y.double(), g.double(), 1e-5)
    want_next = PZ.rms_norm(x1, g2.double(), 3e-4)
    for with_next, with_cast in ((True, False), (False, True), (False, False), (True, True)):
        xd = x.to(DEV)
        nxt = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_next else None
        cast = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_cast else None
        ops.rms_add(y.to(DEV), g.to(DEV), 1e-5, xd, g2.to(DEV) if with_next else None, 3e-4, nxt, cast)
        _close(xd, x1, 2e-6, "stream")
        if with_next:
            _close(nxt, want_next, TOL[dtype] / 2, "next norm")
        if with_cast:
            _close(cast, x1, TOL[dtype] / 2, "rounded stream")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("d", [128, 384, 2048])
def test_norm_of_a_result_added_to_the_stream_a_warp_per_row(ops, dtype, d):
    """Many rows of a width that is a multiple of 128: the variant with a warp per row."""
    n = 70
    y, x = _rnd(n, d, seed=1, s=3.0), _rnd(n, d, seed=2)
    g, g2 = _rnd(d, seed=3) + 1.0, _rnd(d, seed=4) + 1.0
    x1 = x.double() + PZ.rms_norm(y.double(), g.double(), 1e-5)
    for with_next, with_cast in ((True, False), (False, True), (False, False), (True, True)):
        xd = x.to(DEV)
        nxt = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_next else None
        cast = torch.empty(n, d, device=DEV, dtype=ACT[dtype]) if with_cast else None
        ops.rms_add(y.to(DEV), g.to(DEV), 1e-5, xd, g2.to(DEV) if with_next else None, 3e-4, nxt, cast)
        _close(xd, x1, 2e-6, "stream")
        if with_next:
            _close(nxt, PZ.rms_norm(x1, g2.double(), 3e-4), TOL[dtype] / 2, "next norm")
        if with_cast:
            _close(cast, x1, TOL[dtype] / 2, "rounded stream")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_row_activations_and_the_gathered_gate(ops, dtype):
    n, d, col = 13, 37, 5
    x = _rnd(n, col + d + 3, seed=5, s=3.0)
    x[0, col] = 0.0
    x[1, col] = -40.0
    x[2, col] = 40.0
    pq = torch.tensor([0.7, -1.3])
    out = torch.empty(n, d, device=DEV, dtype=ACT[dtype])
    ops.act_rows(x.to(DEV), col, ACT_XIELU, pq.to(DEV), out)
    z = x[:, col:col + d].double()
    _close(out, PZ.xielu(z, pq[0].double(), pq[1].double()), TOL[dtype] / 2, "xielu")
    ops.act_rows(x.to(DEV), col, ACT_TANH, None, out)
    _close(out, torch.tanh(z), TOL[dtype] / 2, "tanh")
    table = _rnd(50, d, seed=6).to(ACT[dtype])
    tokens = torch.tensor([3, 49, 0, -1, 7, 7, 1, 2, 3, 4, 5, 6, 8], dtype=torch.int32)
    g = _rnd(n, d, seed=7)
    ops.gather_mul(g.to(DEV), table.to(DEV), tokens.to(DEV), out)
    want = g.double() * table.double()[tokens.long().clamp(min=0)]
    want[3] = 0.0
    _close(out, want, TOL[dtype] / 2, "gate times the token's row")


def test_embedding_scale(ops):
    table = _rnd(20, 12, seed=8).to(torch.bfloat16)
    tokens = torch.tensor([4, 19, -1, 0], dtype=torch.int32, device=DEV)
    out = torch.empty(4, 12, device=DEV)
    ops.embed_pos(tokens, torch.zeros(4, dtype=torch.int32, device=DEV), table.to(DEV), None, out, 2.5)
    want = table.float()[[4, 19, 0, 0]] * 2.5
    want[2] = 0
    assert torch.equal(out.cpu(), want)


# ----------------------------------------------------------------------------- attention
def _attention(ops, dtype, q, k, gq, gk, eps, rot, scale, window, pool, sink, pieces, page_fill=None):
    """Runs norm + rotation + append, block pooling and attention over one sequence cut into
    ``pieces``; returns [T, H, d].  q [T, H, d], k [T, G, d]: projected rows (fp32)."""
    T, H, d = q.shape
    G = k.shape[1]
    keep = max(window, pool) if window else 0
    extra = {(0, 0): KVRequest(G, d, 0, 2, every=pool)} if pool and window else {}
    cache = SequenceCache({0: KVRequest(G, d, keep)}, {}, cache_tokens=T + 64, max_seq_len=T + 64,
                          dtype=ACT[dtype], device=torch.device(DEV), extra_kv_requests=extra)
    if page_fill is not None:           # what an earlier owner of the pages left behind
        for g in cache.groups:
            g.storage.fill_(page_fill)
    freq, amp, dims = None, 1.0, 0
    if rot:
        dims = rot["dims"]
        freq, amp = rotary_frequencies(dims, rot["base"], rot.get("scaling"))
        freq = freq.to(DEV)
    fused = torch.cat([q.reshape(T, H * d), k.reshape(T, G * d)], dim=1).to(DEV)
    slot, at, outs = cache.alloc_slot(), 0, []
    for n in pieces:
        cache.reserve([(slot, n)])
        lay = build_layout([(slot, [0] * n, [])], [at], DEV)
        kv, blocks = cache.layer_kv(0), (cache.layer_kv_extra(0) or (None,))[0]
        rows = fused[at:at + n].contiguous()
        qo = torch.empty(n, H * d, device=DEV, dtype=ACT[dtype])
        ops.qk_norm_rope_append(rows, 0, H * d, gq.to(DEV), gk.to(DEV), eps, freq, dims, amp, lay,
                                kv, H, qo, True)
        if blocks is not None:
            ops.pool_blocks(lay, kv, blocks, pool)
        out = torch.empty(n, H * d, device=DEV, dtype=ACT[dtype])
        ops.attention_pooled(qo, lay, kv, blocks, H, None if sink is None else sink.to(DEV), out,
                             scale, window, pool)
        outs.append(out.float().cpu())
        cache.advance(slot, n)
        at += n
    assert at == T
    return torch.cat(outs).view(T, H, d)


def _plain_attention(q, k, gq, gk, eps, rot, scale, window, pool, sink):
    T = q.shape[0]
    qn = PZ.rotate(PZ.rms_norm(q.double(), gq.double(), eps), torch.arange(T), rot)
    kn = PZ.rotate(PZ.rms_norm(k.double(), gk.double(), eps), torch.arange(T), rot)
    return PZ.seen_attention(qn, kn, k.double(), scale, window, pool,
                             None if sink is None else sink.double())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", [
    dict(H=4, G=2, d=16, window=24, pool=4, rot=dict(dims=8, base=5000.0, scaling=dict(factor=8.0, original=64, fast=4.0, slow=0.5))),
    dict(H=3, G=3, d=24, window=70, pool=5, rot=dict(dims=24, base=300.0)),
    dict(H=2, G=1, d=8, window=3, pool=7, rot=dict(dims=6, base=50.0)),
    dict(H=1, G=1, d=2, window=1, pool=1, rot=dict(dims=2, base=10.0)),
    dict(H=2, G=1, d=3, window=0, pool=0, rot=None),
    dict(H=2, G=2, d=40, window=64, pool=64, rot=None),
    dict(H=4, G=1, d=64, window=128, pool=0, rot=dict(dims=32, base=1e4)),
])
def test_attention_whole_in_portions_and_token_by_token(ops, dtype, case):
    T, H, G, d = 200, case["H"], case["G"], case["d"]
    q, k = _rnd(T, H, d, seed=1, s=2.0), _rnd(T, G, d, seed=2, s=2.0)
    gq, gk = _rnd(d, seed=3, s=0.3) + 1.2, _rnd(d, seed=4, s=0.3) + 1.2
    sink = _rnd(H, seed=5, s=1.5)
    args = (gq, gk, 1e-5, case["rot"], 0.3, case["window"], case["pool"], sink)
    ref = _plain_attention(q, k, *args)
    for pieces in ([T], [2, 61, 1, 2, 64, 3, 67], [60] + [1] * 140):
        got = _attention(ops, dtype, q, k, *args, pieces, page_fill=float("nan"))
        _close(got, ref, TOL[dtype], f"{case} in {len(pieces)} pieces")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_query_that_points_at_one_far_block(ops, dtype):
    """700 tokens; every query points along one direction that only the keys of one block of
    eight, far back, share.  Before the block is pooled its last token is seen alone; from then on
    the block's mean carries nearly all the weight, at every later position."""
    T, d, W, P, b = 700, 16, 24, 8, 5
    a = torch.zeros(d)
    a[3] = 1.0
    k = _rnd(T, 1, d, seed=9)
    k[:, 0, 3] = 0.0                                   # everyone else is orthogonal to `a`
    k[b * P:(b + 1) * P, 0] = a * torch.arange(1, P + 1)[:, None] * 0.5     # raw sizes 0.5 .. 4
    q = (a * 5.0).repeat(T, 2, 1)
    one = torch.ones(d)
    ref = _plain_attention(q, k, one, one, 1e-6, None, 2.0, W, P, None)
    for pieces in ([T], [71, 1, 1, 627], [300] + [1] * 400):
        got = _attention(ops, dtype, q, k, one, one, 1e-6, None, 2.0, W, P, None, pieces)
        _close(got, ref, TOL[dtype], "far block")
    first_seen = b * P + P - 1 + W                     # the first position that sees the block
    mean_value = k[b * P:(b + 1) * P, 0].mean(0)
    for i in (first_seen, first_seen + 1, 400, T - 1):
        assert float((got[i, 0] - mean_value).abs().max()) < 0.05 * float(mean_value.abs().max())
    # one position earlier only the block's last token is left in the window
    assert float((got[first_seen - 1, 0] - k[(b + 1) * P - 1, 0]).abs().max()) < 0.05 * 4.0
    # and once that has left, before the block counts, nothing points along `a`
    W2 = 4                                             # a window shorter than the block
    got2 = _attention(ops, dtype, q, k, one, one, 1e-6, None, 2.0, W2, P, None, [T])
    ref2 = _plain_attention(q, k, one, one, 1e-6, None, 2.0, W2, P, None)
    _close(got2, ref2, TOL[dtype], "window shorter than the block")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_window_edges_and_a_sink_that_takes_everything(ops, dtype):
    """One loud key: positions that still have it in their window follow it, the next one does
    not; with a huge sink every output goes to zero."""
    T, d, W = 130, 8, 64
    k = _rnd(T, 1, d, seed=11, s=0.1)
    k[:, 0, 0] = 0.0
    k[40, 0] = 0.0
    k[40, 0, 0] = 6.0
    q = torch.zeros(T, 1, d)
    q[:, 0, 0] = 1.0
    one = torch.ones(d)
    got = _attention(ops, dtype, q, k, one, one, 1e-6, None, 4.0, W, 0, None, [100] + [1] * 30)
    _close(got, _plain_attention(q, k, one, one, 1e-6, None, 4.0, W, 0, None), TOL[dtype], "edge")
    assert float(got[40 + W - 1, 0, 0]) > 5.5            # the last position that sees key 40
    assert abs(float(got[40 + W, 0, 0])) < 0.5           # the first that does not
    sink = torch.tensor([80.0])
    got = _attention(ops, dtype, q, k, one, one, 1e-6, None, 4.0, W, 0, sink, [T])
    assert float(got.abs().max()) < 1e-6


# ----------------------------------------------------------------------------- the delta rule
def _delta(ops, dtype, r, k, v, g, a_logits, decay_logits, a_bias, norm_w, eps, pieces, state=None,
           slot=0, n_slots=2):
    T, H, d = r.shape
    hd = H * d
    fused = torch.cat([x.reshape(T, hd) for x in (r, k, v, g, a_logits)], dim=1).to(DEV)
    if state is None:
        state = torch.zeros(n_slots, hd * d, device=DEV)
    outs, at = [], 0
    for n in pieces:
        lay = build_layout([(slot, [0] * n, [])], [at], DEV)
        out = torch.empty(n, hd, device=DEV, dtype=ACT[dtype])
        ops.delta_rule(fused[at:at + n].contiguous(), 0, hd, 2 * hd, 3 * hd, 4 * hd,
                       decay_logits.reshape(T, hd)[at:at + n].contiguous().to(DEV), a_bias.to(DEV),
                       norm_w.to(DEV), eps, math.exp(-0.5), 1e-6, lay, state, H, d, out)
        outs.append(out.float().cpu())
        at += n
    return torch.cat(outs).view(T, H, d), state


def _plain_delta(r, k, v, g, a_logits, decay_logits, a_bias, norm_w, eps):
    T, H, d = r.shape
    a = torch.sigmoid(a_logits.double() + a_bias.double().view(H, d))
    o, S = PZ.delta_recurrence(r.double(), k.double(), v.double(), PZ.decay_of(decay_logits.double()), a)
    o = PZ.rms_unit(o, eps) * norm_w.double().view(H, d) * torch.sigmoid(g.double())
    return o, S


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,d", [(3, 20), (2, 64), (1, 1), (1, 33), (2, 96), (1, 130)])
def test_delta_rule_whole_in_portions_and_token_by_token(ops, dtype, H, d):
    T = 90
    r, k, v, g, al, dl = (_rnd(T, H, d, seed=s, s=1.5) for s in range(20, 26))
    ab, nw = _rnd(H * d, seed=30, s=0.7), _rnd(H * d, seed=31, s=0.2) + 1.0
    ref, S = _plain_delta(r, k, v, g, al, dl, ab, nw, 1e-5)
    for pieces in ([T], [2, 15, 1, 16, 17, 39], [1] * T):
        got, state = _delta(ops, dtype, r, k, v, g, al, dl, ab, nw, 1e-5, pieces)
        _close(got, ref, TOL[dtype], f"{H}x{d} in {len(pieces)} pieces")
        _close(state[0].view(H, d, d), S, 1e-4, "state")
        assert float(state[1].abs().max()) == 0.0            # nobody else's state row is touched


def test_delta_rule_remembers_its_first_token_and_forgets_by_its_decay(ops):
    """Without decay and removal the state is the sum of k v^T: asking along the first key, which
    no other key shares, gives back the first value after 400 tokens.  With a decay it fades by
    exactly the product of the decays; with full removal a later key along the same direction
    replaces it."""
    T, d = 400, 16
    k = _rnd(T, 1, d, seed=40)
    k[:, 0, 0] = 0.0
    k[0, 0] = 0.0
    k[0, 0, 0] = 2.0
    v = _rnd(T, 1, d, seed=41)
    r = torch.zeros(T, 1, d)
    r[:, 0, 0] = 1.0
    g = torch.full((T, 1, d), 30.0)                      # gate open
    off = torch.full((T, 1, d), -40.0)
    one, zero = torch.ones(d), torch.zeros(d)
    args = dict(a_bias=zero, norm_w=one, eps=1e-6)
    got, state = _delta(ops, "float32", r, k, v, g, off, off, pieces=[200, 1, 199], **args)
    ref, _ = _plain_delta(r, k, v, g, off, off, zero, one, 1e-6)
    _close(got, ref, 2e-5, "no decay")
    want = PZ.rms_unit(2.0 * v[0, 0].double(), 1e-6)      # o = S^T r = 2 v_0, then the head's norm
    _close(got[T - 1, 0], want, 1e-4, "the first value, 400 tokens later")
    dl = torch.full((T, 1, d), 40.0)                      # decay exp(-exp(-1/2)) per token
    got, state = _delta(ops, "float32", r, k, v, g, off, dl, pieces=[T], **args)
    ref, S = _plain_delta(r, k, v, g, off, dl, zero, one, 1e-6)
    _close(got, ref, 2e-5, "decay")
    _close(state[0].view(1, d, d), S, 1e-4, "decayed state")
    k2 = k.clone()
    k2[300, 0] = 0.0
    k2[300, 0, 0] = 1.0                                   # the same direction again
    on = torch.full((T, 1, d), 40.0)                      # removal rate 1
    got, _ = _delta(ops, "float32", r, k2, v, g, on, off, pieces=[T], **args)
    ref, _ = _plain_delta(r, k2, v, g, on, off, zero, one, 1e-6)
    _close(got, ref, 2e-5, "removal")
    _close(got[T - 1, 0], PZ.rms_unit(v[300, 0].double(), 1e-6), 1e-3, "replaced, not added")


def test_a_batch_of_unequal_sequences_is_each_alone(ops):
    H, d = 2, 24
    lens = [5, 1, 40, 17]
    state = torch.zeros(6, H * d * d, device=DEV)
    data = [[_rnd(n, H, d, seed=100 * i + s) for s in range(6)] for i, n in enumerate(lens)]
    ab, nw = _rnd(H * d, seed=1), _rnd(H * d, seed=2) + 1.0
    hd = H * d
    fused = torch.cat([torch.cat([x.reshape(n, hd) for x in dat[:5]], dim=1)
                       for dat, n in zip(data, lens)]).to(DEV)
    dl = torch.cat([dat[5].reshape(n, hd) for dat, n in zip(data, lens)]).to(DEV)
    slots = [4, 0, 5, 2]
    lay = build_layout([(s, [0] * n, []) for s, n in zip(slots, lens)], [0] * 4, DEV, pad_rows_to=64)
    rows = torch.zeros(lay.n_rows, fused.shape[1], device=DEV)
    rows[:sum(lens)] = fused
    dls = torch.zeros(lay.n_rows, hd, device=DEV)
    dls[:sum(lens)] = dl
    out = torch.full((lay.n_rows, hd), float("nan"), device=DEV)
    ops.delta_rule(rows, 0, hd, 2 * hd, 3 * hd, 4 * hd, dls, ab.to(DEV), nw.to(DEV), 1e-5,
                   math.exp(-0.5), 1e-6, lay, state, H, d, out)
    at = 0
    for dat, n, s in zip(data, lens, slots):
        ref, S = _plain_delta(*dat[:5], dat[5], ab, nw, 1e-5)
        _close(out[at:at + n].view(n, H, d), ref, 2e-5, "in a batch")
        _close(state[s].view(H, d, d), S, 1e-4, "state of the slot")
        at += n
    assert float(out[at:].abs().max()) == 0.0               # padding rows
    assert float(state[[1, 3]].abs().max()) == 0.0


# ----------------------------------------------------------------------------- experts
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("n,top", [(9, 2), (700, 2)])
def test_experts_of_two_matrices_with_squared_relu(ops, dtype, n, top):
    E, D, F = 4, 64, 32
    h = _rnd(n, D, seed=50).to(ACT[dtype])
    up = (_rnd(E, F, D, seed=51) / 8).to(ACT[dtype])
    idx = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(i))[:top]
                       for i in range(n)]).to(torch.int32).to(DEV)
    offsets = torch.empty(E + 1, device=DEV, dtype=torch.int32)
    order = torch.empty(n * top, device=DEV, dtype=torch.int32)
    place = torch.empty(n * top, device=DEV, dtype=torch.int32)
    ops.moe_group(idx, E, offsets, order, place)
    mid = torch.empty(n * top, F, device=DEV, dtype=ACT[dtype])
    ops.moe_linear(h.to(DEV), order, top, offsets, up.to(DEV), None, mid, ACT_RELU2)
    pl = place.cpu().view(n, top)
    for t in range(0, n, max(1, n // 40)):
        for j in range(top):
            e = int(idx[t, j])
            want = PZ.relu_squared(h[t].double() @ up[e].double().T)
            _close(mid[int(pl[t, j])], want, TOL[dtype], "expert's first half")
