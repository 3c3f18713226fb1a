"""Each new mechanism alone, kernel against a plain float64 computation: the RMS norm; the
latent store and the attention over it (CUDA-core and tensor-core kernels, prompts and
one-token steps, with and without splits) with inputs in which one far key, a page's edge, a
window's edge, the sink or a stale row decides the result; the per-head linear map with its
gate; and the routed experts' kernels (choice, grouping, products, weighted sum)."""
import math

import pytest
import torch

import plain_runesun as PR
from nimbus_infer_rs_b200.cache import PAGE, LayerKV
from nimbus_infer_rs_b200.csrc import ops as ops_mod
from nimbus_infer_rs_b200.engine.batch import build_layout

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    return ops_mod.backend()


def _rnd(*shape, seed=0, s=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * s


def _rel(got, ref):
    ref = ref.double()
    return float((got.double().cpu() - ref).abs().max()) / max(1e-30, float(ref.abs().max()))


@pytest.mark.parametrize("d", [1, 7, 96, 1000, 4099])
def test_rms_norm_of_a_slice_with_gathered_rows(ops, d):
    x = _rnd(9, d + 5, seed=d).to(DEV)
    w = (_rnd(d, seed=1) * 0.3 + 1).to(DEV)
    rows = torch.tensor([3, -1, 0, 8], dtype=torch.int32, device=DEV)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 5e-3)):
        out = torch.empty((4, d), dtype=dt, device=DEV)
        ops.rmsnorm(x, w, 1e-5, out, rows, x_col=3)
        src = x[[3, 0, 0, 8], 3:3 + d].double().cpu()
        ref = PR.rms_norm(src, w.double().cpu(), 1e-5)
        ref[1] = 0
        assert _rel(out, ref) < tol
        out2 = torch.empty((9, d), dtype=dt, device=DEV)
        ops.rmsnorm(x, None, 1e-5, out2, None, x_col=0)
        assert _rel(out2, PR.rms(x[:, :d].double().cpu(), 1e-5)) < tol


def _store(lens, rank, dtype, seed, extra_pages=2, stale=None):
    """A one-plane paged store with the pages of the sequences dealt out in a scrambled order;
    returns (LayerKV, [latents per sequence in float64]).  Slots are 1, 2, ...; slot 0 is unused.
    Rows no sequence has written hold `stale` (NaN, inf) if given."""
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // PAGE) for n in lens) + extra_pages
    perm = torch.randperm(n_pages, generator=g).tolist()
    max_pages = max(-(-n // PAGE) for n in lens) + 1
    k = torch.zeros(n_pages, 1, PAGE, rank)
    if stale is not None:
        k.fill_(stale)
    table = torch.zeros(len(lens) + 1, max_pages, dtype=torch.int32)
    cs = []
    for i, n in enumerate(lens):
        c = torch.randn(n, rank, generator=g).to(dtype).float()
        cs.append(c.double())
        for j in range(-(-n // PAGE)):
            pg = perm.pop()
            table[i + 1, j] = pg
            rows = c[j * PAGE:(j + 1) * PAGE]
            k[pg, 0, :rows.shape[0]] = rows
    kv = LayerKV(k.to(dtype).to(DEV), None, table.to(DEV), PAGE, 1, rank)
    return kv, cs


def _attend_ref(a, c, pos, sink, scale, window=0):
    """a [H, rank] (float64), c [n, rank]: the row's result [H, rank]."""
    lo = max(0, pos + 1 - window) if window > 0 else 0
    keys = c[lo:pos + 1]
    s = (a @ keys.T) * scale
    w = PR.sink_softmax(s, sink if sink is not None else torch.full((a.shape[0],), -math.inf, dtype=a.dtype))
    return w @ keys


def _check_attention(ops, lens, new, H, rank, dtype, *, sink=True, window=0, scale=0.3, seed=3,
                     mma=True, boost=None, stale=None, tol=None):
    """Sequences of `lens` cached tokens of which the last `new` are this step's rows."""
    kv, cs = _store(lens, rank, dtype, seed, stale=stale)
    entries = [(i + 1, [0] * m, []) for i, m in enumerate(new)]
    lay = build_layout(entries, [n - m for n, m in zip(lens, new)], DEV, pad_rows_to=8)
    g = torch.Generator().manual_seed(seed + 1)
    a = torch.randn(lay.n_rows, H, rank, generator=g).to(dtype).float()
    if boost is not None:       # make one key decide: row, head, key index, strength
        seq, r_in_seq, h, key, strength = boost
        r = sum(new[:seq]) + r_in_seq
        a[r, h] = (cs[seq][key] * strength / (scale * float(cs[seq][key] @ cs[seq][key]))).to(dtype).float()
    sk = (torch.randn(H, generator=g) * 2).to(DEV) if sink else None
    out = torch.full((lay.n_rows, H * rank), float("nan"), dtype=dtype, device=DEV)
    was = ops.use_mma
    ops.use_mma = mma
    try:
        ops.attention_latent(a.reshape(lay.n_rows, -1).to(dtype).to(DEV), lay, kv, H, sk, out, scale, window)
    finally:
        ops.use_mma = was
    torch.cuda.synchronize()
    ops.raise_device_errors()
    tol = tol or (2e-5 if dtype == torch.float32 else 1.5e-2)
    r = 0
    for i, (n, m) in enumerate(zip(lens, new)):
        for t in range(m):
            ref = _attend_ref(a[r].double(), cs[i], n - m + t, None if sk is None else sk.double().cpu(),
                              scale, window)
            got = out[r].float().cpu().view(H, rank)
            assert torch.isfinite(got).all(), (i, t)
            assert _rel(got, ref) < tol, (i, t, _rel(got, ref))
            r += 1
    assert (out[r:] == 0).all() or r == lay.n_rows     # padding rows
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mma", [False, True])
@pytest.mark.parametrize("H,rank", [(1, 8), (6, 40), (16, 64), (5, 96), (3, 200), (20, 256)])
def test_latent_attention_prompts_and_single_tokens(ops, dtype, mma, H, rank):
    if mma and dtype != torch.bfloat16:
        pytest.skip("the tensor-core kernel is the bfloat16 path")
    # prompts from the first token, portions that start inside a page, one-token steps
    _check_attention(ops, [1, 2, 63, 64, 65, 200], [1, 2, 63, 64, 65, 200], H, rank, dtype, mma=mma)
    _check_attention(ops, [70, 129, 300], [7, 65, 2], H, rank, dtype, mma=mma, seed=4)
    _check_attention(ops, [1, 64, 65, 128, 129, 700], [1] * 6, H, rank, dtype, mma=mma, seed=5)
    _check_attention(ops, [1500], [1], H, rank, dtype, mma=mma, seed=6, sink=False)


@pytest.mark.parametrize("dtype,mma", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_one_key_decides_far_away_at_page_edges_and_first(ops, dtype, mma):
    """A query made to point at one cached latent: the result is (nearly) that latent, so a
    kernel that drops or misplaces the key gives something else entirely."""
    H, rank, L = 4, 64, 1400
    for key in (0, 1, 63, 64, 127, 128, 1023, 1024, 1025, L - 65, L - 2, L - 1):
        out = _check_attention(ops, [L, 200], [1, 1], H, rank, dtype, mma=mma, boost=(0, 0, 2, key, 40.0),
                               seed=8)
        kv, cs = _store([L, 200], rank, dtype, 8)
        got = out[0].float().cpu().view(H, rank)[2].double()
        assert _rel(got, cs[0][key]) < 0.05, key
    # the same inside a prompt's portion: row 5 of the 70 new rows looks at a key 1100 back
    _check_attention(ops, [L], [70], H, rank, dtype, mma=mma, boost=(0, 5, 1, L - 70 + 5 - 1100, 40.0), seed=9)


@pytest.mark.parametrize("dtype,mma", [(torch.float32, False), (torch.bfloat16, True)])
def test_window_edges(ops, dtype, mma):
    """With a window of w the key w-1 back is the last one seen: a boosted key just inside decides
    the result, the same key just outside leaves no trace (both against the plain computation)."""
    H, rank = 2, 32
    for window in (1, 5, 64, 65, 130):
        for L, m in ((300, 1), (300, 70)):
            r_in = m - 1
            pos = L - 1
            inside, outside = pos - window + 1, pos - window
            _check_attention(ops, [L], [m], H, rank, dtype, mma=mma, window=window,
                             boost=(0, r_in, 1, inside, 30.0), seed=10)
            if outside >= 0:
                _check_attention(ops, [L], [m], H, rank, dtype, mma=mma, window=window,
                                 boost=(0, r_in, 1, outside, 30.0), seed=10)


@pytest.mark.parametrize("dtype,mma", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
def test_rows_nobody_wrote_do_not_reach_the_result(ops, dtype, mma):
    for stale in (float("nan"), float("inf")):
        _check_attention(ops, [3, 65, 130], [3, 2, 1], 6, 48, dtype, mma=mma, stale=stale, seed=12)


def test_a_large_sink_takes_the_weight(ops):
    kv, cs = _store([50], 32, torch.float32, 1)
    lay = build_layout([(1, [0], [])], [49], DEV)
    a = _rnd(1, 2 * 32, seed=2).to(DEV)
    out = torch.empty((1, 64), device=DEV)
    for s, factor in ((-1e4, 1.0), (30.0, None)):
        ops.attention_latent(a, lay, kv, 2, torch.tensor([s, -1e4], device=DEV), out, 0.2)
        ref0 = _attend_ref(a.cpu().double().view(2, 32), cs[0], 49, torch.tensor([s, -1e4]).double(), 0.2)
        assert _rel(out.view(2, 32), ref0) < 2e-5
    assert float(out.view(2, 32)[0].abs().max()) < 1e-6        # head 0: all weight on the sink
    assert float(out.view(2, 32)[1].abs().max()) > 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_append_norms_and_places_rows(ops, dtype):
    rank = 40
    kv, _ = _store([130, 70], rank, dtype, 2)
    before = kv.k.clone()
    lay = build_layout([(1, [0, 0, 0], []), (2, [0], [])], [127, 69], DEV, pad_rows_to=8)
    src = _rnd(lay.n_rows, rank + 9, seed=5).to(DEV)
    w = (_rnd(rank, seed=6) * 0.2 + 1).to(DEV)
    ops.latent_append(src, 4, w, 1e-5, lay, kv)
    ref = PR.rms_norm(src[:4, 4:4 + rank].double().cpu(), w.double().cpu(), 1e-5)
    tol = 2e-6 if dtype == torch.float32 else 5e-3
    table = kv.block_table.cpu()
    changed = torch.zeros_like(before, dtype=torch.bool)
    for r, (slot, pos) in enumerate(((1, 127), (1, 128), (1, 129), (2, 69))):
        pg = int(table[slot, pos // PAGE])
        assert _rel(kv.k[pg, 0, pos % PAGE], ref[r]) < tol
        changed[pg, 0, pos % PAGE] = True
    assert torch.equal(kv.k[~changed], before[~changed])       # nothing else was touched


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_per_head_linear_with_gate(ops, dt):
    for H, n_in, n_out, rows in ((1, 1, 1, 1), (3, 20, 40, 11), (16, 128, 64, 70)):
        lay = build_layout([(1, [0] * rows, [])], [0], DEV, pad_rows_to=8)
        x = _rnd(lay.n_rows, 5 + H * n_in, seed=1).to(dt)
        w = _rnd(H, n_out, n_in, seed=2, s=1 / math.sqrt(n_in)).to(dt)
        gate = _rnd(lay.n_rows, H + 3, seed=3)
        out = torch.empty((lay.n_rows, H * n_out), dtype=dt, device=DEV)
        ops.head_linear(x.to(DEV), 5, w.to(DEV), out, lay, gate=gate.to(DEV), gate_col=2)
        xs = x[:rows, 5:].double().view(rows, H, n_in)
        ref = torch.einsum("rhi,hoi->rho", xs, w.double()) * torch.sigmoid(gate[:rows, 2:2 + H].double())[:, :, None]
        assert _rel(out[:rows].view(rows, H, n_out), ref) < (2e-5 if dt == torch.float32 else 1e-2)
        assert (out[rows:] == 0).all()
        ops.head_linear(x.to(DEV), 5, w.to(DEV), out, lay)
        assert _rel(out[:rows].view(rows, H, n_out), torch.einsum("rhi,hoi->rho", xs, w.double())) < \
            (2e-5 if dt == torch.float32 else 1e-2)


@pytest.mark.parametrize("x_dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("mma", [False, True])
def test_per_head_linear_on_the_tensor_cores(ops, x_dt, mma):
    """bf16 weights and results, rows in 32-bit (a slice of a wider 32-bit matrix) or bf16; sizes
    with ragged tiles; padding rows give zeros whatever their inputs hold."""
    for H, n_in, n_out, rows in ((2, 8, 8, 1), (5, 24, 72, 67), (16, 128, 256, 130), (3, 256, 40, 9)):
        lay = build_layout([(1, [0] * rows, [])], [0], DEV, pad_rows_to=8)
        x = _rnd(lay.n_rows, 16 + H * n_in, seed=1).to(x_dt)
        x[rows:] = float("nan")
        w = _rnd(H, n_out, n_in, seed=2, s=1 / math.sqrt(n_in)).to(torch.bfloat16)
        gate = _rnd(lay.n_rows, H + 3, seed=3)
        out = torch.full((lay.n_rows, H * n_out), float("nan"), dtype=torch.bfloat16, device=DEV)
        was = ops.use_mma
        ops.use_mma = mma
        try:
            ops.head_linear(x.to(DEV), 16, w.to(DEV), out, lay, gate=gate.to(DEV), gate_col=2)
        finally:
            ops.use_mma = was
        xs = x[:rows, 16:].to(torch.bfloat16).double().view(rows, H, n_in)
        ref = torch.einsum("rhi,hoi->rho", xs, w.double()) * torch.sigmoid(gate[:rows, 2:2 + H].double())[:, :, None]
        assert _rel(out[:rows].view(rows, H, n_out), ref) < 1e-2
        assert (out[rows:] == 0).all()


def test_router_choice_order_ties_and_weights(ops):
    lay = build_layout([(1, [0] * 5, [])], [0], DEV, pad_rows_to=8)
    E, top = 7, 3
    z = _rnd(lay.n_rows, E + 4, seed=4, s=2.0)
    z[0, 2:2 + E] = torch.tensor([1.0, 3.0, 3.0, -2.0, 3.0, 0.5, 1.0])      # ties: lower index first
    z[1, 2:2 + E] = 0.0                                                      # all equal
    idx = torch.empty((lay.n_rows, top), dtype=torch.int32, device=DEV)
    wt = torch.empty((lay.n_rows, top), dtype=torch.float32, device=DEV)
    for renorm in (False, True):
        ops.moe_route(z.to(DEV), 2, E, top, renorm, lay, idx, wt)
        s = torch.softmax(z[:5, 2:2 + E].double(), -1)
        order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
        assert torch.equal(idx[:5].cpu().long(), order)
        assert idx[0].tolist() == [1, 2, 4] and idx[1].tolist() == [0, 1, 2]
        ref = torch.gather(s, 1, order)
        if renorm:
            ref = ref / ref.sum(-1, keepdim=True)
        assert _rel(wt[:5], ref) < 2e-6
        assert (idx[5:] == -1).all() and (wt[5:] == 0).all()
    # many experts, top = all of them and top = 1
    E = 200
    z = _rnd(lay.n_rows, E, seed=5, s=3.0)
    for top in (1, 8, E):
        idx = torch.empty((lay.n_rows, top), dtype=torch.int32, device=DEV)
        wt = torch.empty((lay.n_rows, top), dtype=torch.float32, device=DEV)
        ops.moe_route(z.to(DEV), 0, E, top, False, lay, idx, wt)
        s = torch.softmax(z[:5].double(), -1)
        order = torch.sort(s, dim=-1, descending=True, stable=True).indices[:, :top]
        assert torch.equal(idx[:5].cpu().long(), order)


@pytest.mark.parametrize("dt,mma", [(torch.float32, False), (torch.bfloat16, False), (torch.bfloat16, True)])
@pytest.mark.parametrize("rows,E,top,D,F", [(1, 1, 1, 8, 8), (3, 5, 2, 72, 24), (70, 4, 4, 64, 40),
                                            (300, 8, 3, 128, 96), (9, 64, 6, 256, 72),
                                            # many pairs: tcgen05 tiles (with tiles that reach
                                            # into the next expert's rows and weight rows)
                                            (700, 8, 3, 128, 96), (600, 3, 2, 320, 256), (1100, 40, 1, 64, 136)])
def test_routed_experts_from_choice_to_sum(ops, dt, mma, rows, E, top, D, F):
    lay = build_layout([(1, [0] * rows, [])], [0], DEV, pad_rows_to=8)
    n = lay.n_rows
    g = torch.Generator().manual_seed(rows + E)
    h = torch.randn(n, D, generator=g).to(dt)
    Wg, Wu = (torch.randn(E, F, D, generator=g) / math.sqrt(D)).to(dt), (torch.randn(E, F, D, generator=g) / math.sqrt(D)).to(dt)
    Wd = (torch.randn(E, D, F, generator=g) / math.sqrt(F)).to(dt)
    idx = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    idx[rows:] = -1
    wt = torch.rand(n, top, generator=g)
    res0 = torch.randn(n, D, generator=g)
    offsets = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    order = torch.empty(n * top, dtype=torch.int32, device=DEV)
    place = torch.empty(n * top, dtype=torch.int32, device=DEV)
    ops.moe_group(idx.to(DEV), E, offsets, order, place)
    off, od, pl = offsets.cpu(), order.cpu(), place.cpu()
    assert int(off[E]) == rows * top and int(off[0]) == 0
    flat = idx.reshape(-1)
    for e in range(E):
        mine = sorted(od[int(off[e]):int(off[e + 1])].tolist())
        assert mine == torch.nonzero(flat == e).reshape(-1).tolist()
    assert all(int(pl[p]) == -1 for p in range(rows * top, n * top))
    assert all(int(od[int(pl[p])]) == p for p in range(rows * top))
    was = ops.use_mma
    ops.use_mma = mma
    try:
        mid = torch.zeros((n * top, F), dtype=dt, device=DEV)
        ops.moe_linear(h.to(DEV), order, top, offsets, Wg.to(DEV), Wu.to(DEV), mid, ops_mod.ACT_SILU)
        y = torch.zeros((n * top, D), dtype=torch.float32, device=DEV)
        ops.moe_linear(mid, None, 1, offsets, Wd.to(DEV), None, y)
    finally:
        ops.use_mma = was
    res = res0.clone().to(DEV)
    ops.moe_combine(y, place, wt.to(DEV), res)
    ref = res0.double().clone()
    hd = h.double()
    for r in range(rows):
        for k in range(top):
            e = int(idx[r, k])
            m = PR.silu(Wg[e].double() @ hd[r]) * (Wu[e].double() @ hd[r])
            ref[r] += float(wt[r, k]) * (Wd[e].double() @ m)
    tol = 2e-5 if dt == torch.float32 else 2e-2
    assert _rel(res[:rows], ref[:rows]) < tol
    assert torch.equal(res[rows:].cpu(), res0[rows:])
