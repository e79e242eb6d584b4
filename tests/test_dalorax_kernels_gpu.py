"""The kernels Dalorax brought, each alone against plain torch in float64: the sinusoid at the embedding, the Dynamic
Tanh norm and the stream update through it, attention with a soft cap, kept first positions and a gate per column
(on the CUDA cores and on tensor cores, as portions and as single rows), the router, the plan that sorts a step's
(token, choice) slots by expert, and the experts' products."""
import math

import pytest
import torch

import plain_dalorax as plain
from test_nufetar_kernels_gpu import DEV, i32, paged

pytestmark = pytest.mark.gpu

ACT = [torch.float32, torch.bfloat16]


def stream():
    from mlx_lm_b200 import ops
    return ops.current_stream()


@pytest.mark.parametrize("D", [64, 50, 7])
def test_sinusoid_at_the_embedding(D):
    from mlx_lm_b200 import ops
    torch.manual_seed(D)
    V, T = 40, 33
    table = torch.randn(V, D).to(torch.bfloat16).to(DEV)
    tok = torch.randint(0, V, (T,))
    pos = torch.tensor([0, 1, 2, 3, 63, 64, 65, 1000, 4095] + list(range(100, 100 + T - 9)))
    freq = (10000.0 ** (-2.0 * torch.arange((D + 1) // 2, dtype=torch.float64) / D)).float().to(DEV)
    out = torch.zeros(T, D, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops.embed_pos(i32(tok.tolist()), i32(pos.tolist()), table, None, out, status, stream(), freq=freq)
    assert int(status.item()) == 0
    want = table.double().cpu()[tok] + plain.sinusoid(4096, D, torch.float64)[pos]
    # the angle is a float32 product: at position 4095 it is exact to about 4095 * 6e-8
    assert float((out.double().cpu() - want).abs().max()) < 6e-4
    assert float((out.double().cpu()[:7] - want[:7]).abs().max()) < 1e-5


@pytest.mark.parametrize("out_dtype", ACT)
@pytest.mark.parametrize("D", [64, 50])
def test_dynamic_tanh(out_dtype, D):
    from mlx_lm_b200 import ops
    torch.manual_seed(D)
    T = 37
    x = (3 * torch.randn(T, D)).to(DEV)
    alpha, w, b = torch.tensor([0.7], device=DEV), torch.randn(D, device=DEV), torch.randn(D, device=DEV)
    tol = 1e-6 if out_dtype == torch.float32 else 2e-2
    want = torch.tanh(0.7 * x.double().cpu()) * w.double().cpu() + b.double().cpu()
    out = torch.zeros(T, D, dtype=out_dtype, device=DEV)
    ops.dyt_norm(x, alpha, w, b, out, stream())
    assert float((out.double().cpu() - want).abs().max()) < tol
    rows = [5, 0, 36]
    out = torch.zeros(3, D, dtype=out_dtype, device=DEV)
    ops.dyt_norm(x, alpha, w, None, out, stream(), rows=i32(rows), out_scale=2.5)
    assert float((out.double().cpu() - 2.5 * (want[rows] - b.double().cpu())).abs().max()) < 2.5 * tol


@pytest.mark.parametrize("next_dtype", ACT)
@pytest.mark.parametrize("D,terms", [(64, 1), (64, 3), (50, 2), (7, 1)])
def test_stream_update_through_a_norm(next_dtype, D, terms):
    from mlx_lm_b200 import ops
    torch.manual_seed(D + terms)
    T = 29
    x0 = torch.randn(T, D)
    br = 2 * torch.randn(T * terms, D)
    a1, w1, b1 = torch.tensor([0.4]), torch.randn(D), torch.randn(D)
    a2, w2, b2 = torch.tensor([1.3]), torch.randn(D), torch.randn(D)
    req = [0] * T
    req[4] = -1
    y = br.double().view(T, terms, D).sum(1)
    new = x0.double() + torch.tanh(0.4 * y) * w1.double() + b1.double()
    nxt = torch.tanh(1.3 * new) * w2.double() + b2.double()
    dev = lambda *ts: tuple(t.to(DEV) for t in ts)
    x = x0.to(DEV)
    out = torch.full((T, D), 7.0, dtype=next_dtype, device=DEV)
    ops.dyt_residual(x, br.to(DEV), stream(), post=dev(a1, w1, b1), nxt=dev(a2, w2, b2), next_out=out, terms=terms,
                     token_req=i32(req))
    live = [t for t in range(T) if t != 4]
    assert float((x.double().cpu()[live] - new[live]).abs().max()) < 2e-6
    assert float((out.double().cpu()[live] - nxt[live]).abs().max()) < (2e-6 if next_dtype == torch.float32 else 3e-2)
    assert bool((x[4].cpu() == x0[4]).all()) and bool((out[4] == 7.0).all())
    # without norms it is the sum alone
    x = x0.to(DEV)
    ops.dyt_residual(x, br.to(DEV), stream(), terms=terms)
    assert float((x.double().cpu() - (x0.double() + y)).abs().max()) < 2e-6
    # a norm on the branch, none after
    x = x0.to(DEV)
    ops.dyt_residual(x, br.to(DEV), stream(), post=dev(a1, w1, b1), terms=terms)
    assert float((x.double().cpu() - new).abs().max()) < 2e-6


def check_tiles(ops, qd, qhs, table, kp, vp, H, dk, dv, scale, window, gate, softcap, keep_first, want, T):
    """The tensor-core kernel over the same request: portions in tiles of up to 128 queries (one cut short, one
    empty), single-token rows, and single rows whose keys are split over several CTAs and merged."""
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kw = dict(window=window, gate=gate, softcap=softcap, keep_first=keep_first)
    tiles = i32([[128, T - 128, 0, 128], [0, 0, 0, 0], [0, 128, 0, 0]])
    for out_dtype in (torch.float32, torch.bfloat16):
        out = torch.full((T, H * dv), 7.0, dtype=out_dtype, device=DEV)
        ops.attention_wide_tiles(qd, qhs, tiles, 3, 128, table, kp, vp, out, dv, H, dk, dv, scale, status, stream(), **kw)
        assert int(status.item()) == 0
        err = float((out.double().cpu().view(T, H, dv) - want).abs().max())
        assert err < (6e-3 if out_dtype == torch.float32 else 2e-2), ("tiles", out_dtype, err)
    rows = sorted({0, 1, keep_first, keep_first + 1, window - 1, window, window + 1, window + keep_first, 63, 64, 65, 127,
                   128, 129, T - 1} & set(range(T)))
    singles = i32([[r, 1, 0, r] for r in rows] + [[5, 0, 0, 0]])
    for max_len in (0, 4096):
        need = ops.attention_wide_scratch(len(rows) + 1, H, dv, window, 0, max_len, keep_first) if max_len else 0
        scratch = torch.full((need,), float("nan"), device=DEV) if need else None
        out = torch.full((T, H * dv), 7.0, device=DEV)
        ops.attention_wide_tiles(qd, qhs, singles, len(rows) + 1, 1, table, kp, vp, out, dv, H, dk, dv, scale, status,
                                 stream(), scratch=scratch, max_len=max_len, **kw)
        assert int(status.item()) == 0
        got = out.double().cpu().view(T, H, dv)
        assert float((got[rows] - want[rows]).abs().max()) < 6e-3, max_len
        untouched = [r for r in range(T) if r not in rows]
        assert bool((out[untouched] == 7.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,dk,dv,window,keep_first,softcap,column_gate", [
    (4, 2, 32, 16, 24, 3, 8.0, True),
    (4, 1, 64, 64, 44, 6, 25.0, True),
    (3, 3, 48, 40, 2, 70, 2.0, True),         # kept positions beyond a block of 64 keys, a window of two
    (6, 2, 24, 8, 100, 7, 0.0, True),         # no cap
    (8, 2, 64, 64, 140, 64, 30.0, False),     # a window over several blocks; no gate
    (8, 8, 64, 64, 1000, 0, 5.0, True),       # every key visible: single rows split over several CTAs
    (3, 1, 12, 10, 9, 2, 1.5, True),          # rows that are no multiple of 16 bytes
    (1, 1, 8, 8, 1, 1, 4.0, True),
    (2, 1, 128, 64, 33, 150, 50.0, True),     # every position is a kept one
])
def test_attention_with_a_cap_kept_positions_and_a_gate_per_column(act, H, G, dk, dv, window, keep_first, softcap,
                                                                   column_gate):
    from mlx_lm_b200 import ops
    torch.manual_seed(H * dk + dv + window + keep_first)
    T, page = 150, 16
    q = torch.randn(T, H, dk) * 2.0
    k = torch.randn(T, G, dk).to(act).float()
    v = torch.randn(T, G, dv).to(act).float()
    gt = torch.randn(T, H * dv).to(act).float() if column_gate else None
    scale = 3.0 / math.sqrt(dk)
    rep = H // G
    see = plain.visible(T, window, keep_first)
    heads = []
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // rep].double().T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~see, -math.inf)
        heads.append(torch.softmax(s, dim=-1) @ v[:, h // rep].double())
    want = torch.stack(heads, dim=1)
    if column_gate:
        want = want * torch.sigmoid(gt.double()).view(T, H, dv)
    n_pages = (T + page - 1) // page
    order = list(reversed(range(n_pages)))
    krow, vrow = (dk + 7) // 8 * 8, (dv + 7) // 8 * 8
    kp, vp = paged(k, G, krow, page, act, n_pages + 1, order), paged(v, G, vrow, page, act, n_pages + 1, order)
    table = i32([order + [-1] * 3])
    qd = torch.zeros(T, H * krow, device=DEV)
    qd.view(T, H, krow)[:, :, :dk] = q.to(DEV)
    gate = gt.to(act).to(DEV) if column_gate else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for out_dtype in {act, torch.float32}:
        out = torch.zeros(T, H * dv, dtype=out_dtype, device=DEV)
        ops.attention_wide(qd, krow, i32(list(range(T))), i32([0] * T), table, kp, vp, out, dv, H, dk, dv, scale, status,
                           stream(), window=window, gate=gate, softcap=softcap, keep_first=keep_first)
        assert int(status.item()) == 0
        err = float((out.double().cpu().view(T, H, dv) - want).abs().max())
        assert err < (3e-5 if out_dtype == torch.float32 else 2e-2), (out_dtype, err)
    if act == torch.bfloat16:
        assert ops.attention_wide_tc_supported(kp, vp, H, dk, dv, False) == (dk % 8 == 0 and dv % 8 == 0)
        if ops.attention_wide_tc_supported(kp, vp, H, dk, dv, False):
            check_tiles(ops, qd, krow, table, kp, vp, H, dk, dv, scale, window, gate, softcap, keep_first, want, T)


def test_a_kept_position_far_back_and_the_one_after_it():
    """One key among hundreds carries the answer: with a score that stands out, position p reads the value of the
    last kept position and not that of the first one that is not kept (nor, in a window, the one just outside)."""
    from mlx_lm_b200 import ops
    T, page, dk, dv, keep, window = 700, 16, 16, 16, 5, 30
    for act in ACT:
        k = torch.zeros(T, 1, dk)
        v = torch.zeros(T, 1, dv)
        k[keep - 1, 0, 0] = 1.0          # the last kept position
        k[keep, 0, 1] = 1.0              # the first that is not
        k[T - 1 - window, 0, 2] = 1.0    # just outside the window of the last position
        k[T - window, 0, 3] = 1.0        # just inside
        v[keep - 1, 0, 0] = v[keep, 0, 1] = v[T - 1 - window, 0, 2] = v[T - window, 0, 3] = 1.0
        q = torch.zeros(T, 1, dk)
        q[T - 1, 0, :4] = 30.0           # the last position asks for all four alike
        n_pages = (T + page - 1) // page
        order = list(range(n_pages))
        kp, vp = paged(k, 1, dk, page, act, n_pages, order), paged(v, 1, dv, page, act, n_pages, order)
        table = i32([order])
        qd = q.view(T, dk).to(DEV).contiguous()
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.zeros(T, dv, device=DEV)
        ops.attention_wide(qd, dk, i32(list(range(T))), i32([0] * T), table, kp, vp, out, dv, 1, dk, dv, 1.0, status,
                           stream(), window=window, softcap=40.0, keep_first=keep, rows=i32([T - 1]))
        got = out[T - 1, :4].cpu()
        assert torch.allclose(got, torch.tensor([0.5, 0.0, 0.0, 0.5]), atol=1e-3), got
        if act == torch.bfloat16:
            for max_len in (0, 4096):
                need = ops.attention_wide_scratch(1, 1, dv, window, 0, max_len, keep) if max_len else 0
                out = torch.zeros(T, dv, device=DEV)
                ops.attention_wide_tiles(qd, dk, i32([[T - 1, 1, 0, T - 1]]), 1, 1, table, kp, vp, out, dv, 1, dk, dv, 1.0,
                                         status, stream(), window=window, softcap=40.0, keep_first=keep,
                                         scratch=torch.zeros(need, device=DEV) if need else None, max_len=max_len)
                assert torch.allclose(out[T - 1, :4].cpu(), torch.tensor([0.5, 0.0, 0.0, 0.5]), atol=1e-3)
            out = torch.zeros(T, dv, device=DEV)
            first = T - 100
            ops.attention_wide_tiles(qd, dk, i32([[first, 100, 0, first]]), 1, 128, table, kp, vp, out, dv, 1, dk, dv, 1.0,
                                     status, stream(), window=window, softcap=40.0, keep_first=keep)
            assert torch.allclose(out[T - 1, :4].cpu(), torch.tensor([0.5, 0.0, 0.0, 0.5]), atol=1e-3)
        assert int(status.item()) == 0


@pytest.mark.parametrize("E,top,score,renorm", [(11, 1, "sigmoid", False), (6, 2, "sigmoid", False), (5, 5, "sigmoid", False),
                                                (40, 3, "sigmoid", True), (9, 4, "softmax", False), (70, 8, "softmax", True)])
def test_router(E, top, score, renorm):
    from mlx_lm_b200 import ops
    torch.manual_seed(E + top)
    T = 45
    z = torch.randn(T, E) * 2
    z[3, :] = 0.25                      # all equal: the lowest experts win, in order
    z[7, 2] = z[7, 4] = 5.0             # a tie at the top
    req = [0] * T
    req[9] = -1
    ld = (E + 7) // 8 * 8
    zd = torch.zeros(T, ld, device=DEV)
    zd[:, :E] = z.to(DEV)
    sel_e = torch.full((T * top,), -7, dtype=torch.int32, device=DEV)
    sel_w = torch.full((T * top,), -7.0, device=DEV)
    ops.moe_route(zd[:, :E], i32(req), top, sel_e, sel_w, stream(), score=score, renormalize=renorm)
    s = torch.sigmoid(z.double()) if score == "sigmoid" else torch.softmax(z.double(), dim=-1)
    got_e, got_w = sel_e.cpu().view(T, top), sel_w.cpu().view(T, top).double()
    for t in range(T):
        if t == 9:
            assert got_e[t].tolist() == [-1] * top
            continue
        order = sorted(range(E), key=lambda e: (-float(s[t, e].float()), e))[:top]
        if t not in (3, 7):
            assert got_e[t].tolist() == order, t
        want = s[t, got_e[t].long()]
        if renorm:
            want = want / want.sum()
        assert float((got_w[t] - want).abs().max()) < 1e-6
    assert got_e[3].tolist() == list(range(top))
    assert got_e[7, 0].item() == 2 and (top == 1 or got_e[7, 1].item() == 4)


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("T,D,F,E,top", [(70, 64, 32, 6, 2), (300, 96, 128, 5, 3), (1, 64, 64, 10, 1), (37, 50, 14, 5, 2),
                                          (200, 128, 64, 16, 2), (9, 48, 16, 9, 9)])
def test_experts_products(act, T, D, F, E, top):
    """The plan covers every slot once, in tiles of one expert; the two products over it give what each slot's expert
    makes of its token's row scaled by the routing weight."""
    from mlx_lm_b200 import ops
    torch.manual_seed(T + D + F + E)
    S = T * top
    x = torch.randn(T, D).to(act)
    w_in = (torch.randn(E, 2 * F, D) * D ** -0.5).to(act)
    w_out = (torch.randn(E, D, F) * F ** -0.5).to(act)
    sel_e = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    if T > 20:
        sel_e[11] = -1                   # a row that pads the step
    sel_w = torch.rand(S) + 0.2
    tc = act == torch.bfloat16 and D % 8 == 0 and F % 8 == 0
    # tiles of 64 on tensor cores (or 16 on the CUDA cores), and the tiles of 4 of steps with few tokens
    for rows in [ops.moe_tile_rows(tc)] + ([ops.moe_few_rows()] if tc else []):
        max_tiles = ops.moe_max_tiles(S, E, rows)
        order = torch.full((S,), -1, dtype=torch.int32, device=DEV)
        tiles = torch.full((3 * max_tiles + 1,), -1, dtype=torch.int32, device=DEV)
        ops.moe_plan(sel_e.flatten().to(DEV), S, E, rows, order, tiles, tiles[3 * max_tiles:], stream())
        n = int(tiles[3 * max_tiles].item())
        info = tiles[:3 * n].cpu().view(n, 3)
        flat = sel_e.flatten()
        live = int((flat >= 0).sum())
        seen = []
        for e, first, cnt in info.tolist():
            assert 0 < cnt <= rows
            slots = order[first:first + cnt].cpu().tolist()
            assert all(int(flat[s]) == e for s in slots)
            seen += slots
        assert sorted(seen) == [s for s in range(S) if flat[s] >= 0] and len(seen) == live
        assert n <= max_tiles and n <= (live + rows - 1) // rows + E
        xd, wi, wo = x.to(DEV), w_in.to(DEV), w_out.to(DEV)
        h = torch.full((S, F), 7.0, dtype=act, device=DEV)
        ops.moe_gemm(xd, top, wi, F, order, tiles, tiles[3 * max_tiles:], max_tiles, rows, h, stream(), sel_weight=sel_w.to(DEV),
                     gated=True)
        y = torch.full((S, D), 7.0, device=DEV)
        ops.moe_gemm(h, 1, wo, D, order, tiles, tiles[3 * max_tiles:], max_tiles, rows, y, stream())
        tol = 2e-5 if act == torch.float32 else 3e-2
        for s in range(S):
            e = int(flat[s])
            if e < 0:
                assert bool((y[s] == 7.0).all())
                continue
            xs = sel_w[s].double() * x[s // top].double()
            g, u = w_in[e, :F].double() @ xs, w_in[e, F:].double() @ xs
            hs = g / (1 + torch.exp(-g)) * u
            assert float((h[s].double().cpu() - hs).abs().max()) < tol * max(1.0, float(hs.abs().max())), ("hidden", s)
            want = w_out[e].double() @ h[s].double().cpu()
            assert float((y[s].double().cpu() - want).abs().max()) < tol * max(1.0, float(want.abs().max())), ("out", s)


@pytest.mark.parametrize("T,D,F,E,top", [(300, 96, 128, 5, 3), (700, 128, 72, 16, 2), (5, 64, 64, 3, 2), (260, 200, 136, 7, 1),
                                          (1024, 256, 192, 4, 2), (40, 64, 8, 30, 4)])
@pytest.mark.parametrize("tile_width", [128, 256])
def test_experts_products_on_tcgen05(T, D, F, E, top, tile_width, monkeypatch):
    """Tiles of 128 slots of one expert: the rows gathered in the plan's order, the gated product's result in that
    order too, the second product's rows back at the slots' own places.  Inner sizes that are no multiple of the
    64-column stages or of the 64 / 128 output columns a CTA makes, experts without a slot, one expert with many
    tiles, a row that pads the step; tiles that take 128 and 256 rows of the weights."""
    from mlx_lm_b200 import ops
    monkeypatch.setenv("MLXB_MOE_BN", str(tile_width))
    torch.manual_seed(T + D + F + E)
    S = T * top
    act = torch.bfloat16
    x = torch.randn(T, D).to(act)
    w_in = (torch.randn(E, 2 * F, D) * D ** -0.5).to(act)
    w_out = (torch.randn(E, D, F) * F ** -0.5).to(act)
    sel_e = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    if T > 600:
        sel_e[: T // 2] = torch.tensor([E - 1, 1][:top], dtype=torch.int32)     # one expert with several full tiles
    if T > 20:
        sel_e[11] = -1
    sel_w = torch.rand(S) + 0.2
    rows = ops.moe_tc05_tile_rows()
    max_tiles = ops.moe_max_tiles(S, E, rows)
    order = torch.full((S,), -1, dtype=torch.int32, device=DEV)
    tiles = torch.full((3 * max_tiles + 1,), -1, dtype=torch.int32, device=DEV)
    n_tiles = tiles[3 * max_tiles:]
    ops.moe_plan(sel_e.flatten().to(DEV), S, E, rows, order, tiles, n_tiles, stream())
    xd, wi, wo = x.to(DEV), w_in.to(DEV), w_out.to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    xs = torch.full((S, D), float("nan"), dtype=act, device=DEV)
    ops.moe_gather(xd, top, order, tiles, n_tiles, max_tiles, xs, stream())
    h = torch.full((S, F), 7.0, dtype=act, device=DEV)
    ops.moe_gemm_tc05(xs, wi, F, order, tiles, n_tiles, max_tiles, h, status, stream(), sel_weight=sel_w.to(DEV), gated=True)
    y = torch.full((S, D), 7.0, device=DEV)
    ops.moe_gemm_tc05(h, wo, D, order, tiles, n_tiles, max_tiles, y, status, stream())
    assert int(status.item()) == 0
    flat = sel_e.flatten()
    live = int((flat >= 0).sum())
    place = order.cpu().tolist()
    assert sorted(place[:live]) == [s for s in range(S) if flat[s] >= 0]
    assert bool((h[live:] == 7.0).all())
    xsc, hc, yc = xs.cpu(), h.double().cpu(), y.double().cpu()
    tol = 3e-2
    for i, s in enumerate(place[:live]):
        e = int(flat[s])
        assert torch.equal(xsc[i], x[s // top])
        xv = sel_w[s].double() * x[s // top].double()
        g, u = w_in[e, :F].double() @ xv, w_in[e, F:].double() @ xv
        hs = g / (1 + torch.exp(-g)) * u
        assert float((hc[i] - hs).abs().max()) < tol * max(1.0, float(hs.abs().max())), ("hidden", s)
        want = w_out[e].double() @ hc[i]
        assert float((yc[s] - want).abs().max()) < tol * max(1.0, float(want.abs().max())), ("out", s)
    for s in range(S):
        if flat[s] < 0:
            assert bool((y[s] == 7.0).all())


@pytest.mark.parametrize("H,G,window,keep_first,softcap,gated", [
    (4, 2, 100, 5, 25.0, True),        # kept positions in the first block, the window several blocks on
    (4, 1, 100, 130, 10.0, True),      # kept positions over two blocks
    (2, 2, 300, 300, 0.0, False),      # no cap, no gate; the kept blocks meet the window's
    (8, 2, 40, 1, 3.0, True),
    (4, 4, 0, 0, 7.0, True),           # every key visible
    (4, 2, 64, 0, 50.0, False),        # a window without kept positions
])
def test_portions_of_plain_heads_on_tcgen05(H, G, window, keep_first, softcap, gated):
    """The tcgen05 kernel for prompt portions with a cap, kept first positions and a gate per column: tiles of 128
    queries of one request that begin at many positions (block borders, the window's and the kept positions' edges
    inside a tile), one cut short, one empty; rounded queries, float32 scores and softmax."""
    from mlx_lm_b200 import ops
    torch.manual_seed(H + window + keep_first)
    T, page, d = 700, 16, 64
    act = torch.bfloat16
    q = (torch.randn(T, H, d) * 2.0).to(act).float()
    k = torch.randn(T, G, d).to(act).float()
    v = torch.randn(T, G, d).to(act).float()
    gt = torch.randn(T, H * d).to(act).float()
    scale = 3.0 / math.sqrt(d)
    see = plain.visible(T, window or T + 1, keep_first)
    heads = []
    for h in range(H):
        s = (q[:, h].double() @ k[:, h // (H // G)].double().T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        heads.append(torch.softmax(s.masked_fill(~see, -math.inf), dim=-1) @ v[:, h // (H // G)].double())
    want = torch.stack(heads, dim=1)
    if gated:
        want = want * torch.sigmoid(gt.double()).view(T, H, d)
    n_pages = (T + page - 1) // page
    order = list(reversed(range(n_pages)))
    # rows nobody wrote hold a finite number, as in the engine's pools: the kernel multiplies them by zero
    kp = torch.nan_to_num(paged(k, G, d, page, act, n_pages + 1, order), nan=3.0)
    vp = torch.nan_to_num(paged(v, G, d, page, act, n_pages + 1, order), nan=3.0)
    row = list(order)
    if window and window < 500:
        # pages wholly behind the window of the step's first position and beyond the kept ones are not the request's
        gone = [lp for lp in range(n_pages) if (lp + 1) * page <= 512 - window + 1 and lp * page >= keep_first]
        for lp in gone:
            row[lp] = -1
    table = i32([order + [-1] * 3, row + [-1] * 3])
    qd = q.view(T, H * d).to(act).to(DEV)
    gate = gt.to(act).to(DEV) if gated else None
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    starts = [0, 128, 256, 384, 512, 640]
    tiles = i32([[s0, min(128, T - s0), 0, s0] for s0 in starts] + [[0, 0, 0, 0]])
    out = torch.full((T, H * d), 7.0, dtype=act, device=DEV)
    assert ops.attention_portions_tc_supported(qd, out, kp, vp)
    ops.attention_portions(qd, tiles, len(starts) + 1, table, kp, vp, out, H, scale, window, status, stream(),
                           keep_first=keep_first, softcap=softcap, gate=gate)
    assert int(status.item()) == 0
    err = (out.double().cpu().view(T, H, d) - want).abs().amax(dim=(1, 2))
    assert float(err.max()) < 2e-2, (float(err.max()), int(err.argmax()))
    # the same request after the cache gave back the pages behind the window of position 512
    out1 = torch.full((T, H * d), 7.0, dtype=act, device=DEV)
    ops.attention_portions(qd, i32([[512, 128, 1, 512], [640, T - 640, 1, 640]]), 2, table, kp, vp, out1, H, scale, window,
                           status, stream(), keep_first=keep_first, softcap=softcap, gate=gate)
    assert int(status.item()) == 0
    assert torch.equal(out1[512:], out[512:])
    # tiles that begin anywhere: a portion that starts in the middle of a block, of the window, of the kept positions
    for s0, n in ((keep_first + 1, 100), (window + 3, 128), (200, 1), (333, 77), (T - 2, 2)):
        if s0 + n > T:
            continue
        out2 = torch.full((T, H * d), 7.0, dtype=act, device=DEV)
        ops.attention_portions(qd, i32([[s0, n, 0, s0]]), 1, table, kp, vp, out2, H, scale, window, status, stream(),
                               keep_first=keep_first, softcap=softcap, gate=gate)
        got = out2.double().cpu().view(T, H, d)
        assert float((got[s0:s0 + n] - want[s0:s0 + n]).abs().max()) < 2e-2, (s0, n)
        assert bool((out2[:s0] == 7.0).all()) and bool((out2[s0 + n:] == 7.0).all())
    assert int(status.item()) == 0
