"""The kernels Zuluvik brought or widened, each alone against the plain implementation's functions in float64: the
router with a correction, groups, identity experts and scaled weights; the sum over a token's choices with identity
experts; the bounded gated unit (alone, and in the experts' products on the CUDA cores, on mma.sync and on tcgen05);
the short convolution without an activation, with its state across steps; queries and keys turned with a stretched
rotation and normed per head, values with fewer heads than the keys; attention with several score maps over the same
values; the difference of the two maps; the latent row with a stretched rotation."""
import math

import pytest
import torch

import plain_zuluvik as plain
from test_nufetar_kernels_gpu import DEV, i32, paged
from zuluvik_cases import rot, stretch

pytestmark = pytest.mark.gpu

ACT = [torch.float32, torch.bfloat16]


def stream():
    from mlx_lm_b200 import ops
    return ops.current_stream()


@pytest.mark.parametrize("outputs,identity,top,groups,scale", [(6, 2, 2, (3, 1), 1.5), (16, 6, 4, (4, 3), 1.25), (16, 0, 4, (4, 2), 1.0),
                                                                (70, 5, 6, (7, 3), 0.25), (5, 1, 3, None, 2.0), (9, 9, 2, (3, 2), 1.0),
                                                                (12, 0, 12, (2, 2), 3.0), (64, 8, 8, (8, 1), 1.0)])
def test_router_with_correction_groups_and_identity_experts(outputs, identity, top, groups, scale):
    from mlx_lm_b200 import ops
    torch.manual_seed(outputs + top)
    T = 53
    z = (torch.randn(T, outputs) * 1.5).float()
    corr = (torch.randn(outputs) * 0.05).float()
    req = [0] * T
    req[9] = -1
    ld = (outputs + 7) // 8 * 8
    zd = torch.zeros(T, ld, device=DEV)
    zd[:, :outputs] = z.to(DEV)
    sel_e = torch.full((T * top,), -7, dtype=torch.int32, device=DEV)
    sel_w = torch.full((T * top,), -7.0, device=DEV)
    ops.moe_route(zd[:, :outputs], i32(req), top, sel_e, sel_w, stream(), score="softmax", renormalize=True,
                  correction=corr.to(DEV), groups=groups[0] if groups else 1, keep_groups=groups[1] if groups else 1,
                  identity=identity, renormalize_eps=1e-20, weight_scale=scale)
    router = {"top": top, "scale": scale, "experts": outputs - identity, "identity": identity}
    if groups:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    w = {"m.router": torch.eye(outputs, dtype=torch.float64), "m.correction": corr.double()}
    want_w, want_e = plain.route(z.double(), w, "m", router)
    got_e, got_w = sel_e.cpu().view(T, top), sel_w.cpu().view(T, top).double()
    n_real = outputs - identity
    for t in range(T):
        if t == 9:
            assert got_e[t].tolist() == [-1] * top
            continue
        marked = [e if e < n_real else -2 for e in want_e[t].tolist()]
        # the plain choice's order is by choice score; the kernel's too
        assert got_e[t].tolist() == marked, (t, got_e[t].tolist(), marked)
        assert float((got_w[t] - want_w[t]).abs().max()) < 2e-6 * scale
    # without a correction, groups and identity experts it is the router it was
    ops.moe_route(zd[:, :outputs], i32(req), top, sel_e, sel_w, stream(), score="softmax", renormalize=False)
    s = torch.softmax(z.double(), dim=-1)
    for t in (0, 5, 20):
        order = sorted(range(outputs), key=lambda e: (-float(s[t, e].float()), e))[:top]
        assert sel_e.cpu().view(T, top)[t].tolist() == order


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("D,top", [(64, 3), (50, 2), (7, 1)])
def test_sum_over_choices_with_identity_experts(act, D, top):
    from mlx_lm_b200 import ops
    torch.manual_seed(D)
    T = 31
    x0, y, h = torch.randn(T, D), torch.randn(T * top, D), torch.randn(T, D).to(act)
    e = torch.randint(-2, 4, (T * top,), dtype=torch.int32)
    e[e == -1] = 0
    wgt = torch.rand(T * top)
    req = [0] * T
    req[4] = -1
    x = x0.clone().to(DEV)
    ops.moe_combine(x, y.to(DEV), e.to(DEV), wgt.to(DEV), h.to(DEV), top, stream(), token_req=i32(req))
    want = x0.double().clone()
    for t in range(T):
        if t == 4:
            continue
        for c in range(top):
            s = t * top + c
            want[t] += y[s].double() if e[s] >= 0 else wgt[s].double() * h[t].double()
    assert float((x.double().cpu() - want).abs().max()) < 1e-5
    assert torch.equal(x[4].cpu(), x0[4])


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("T,F,limit", [(37, 64, 1.5), (5, 50, 0.7), (130, 24, 7.0)])
def test_bounded_gated_unit(act, T, F, limit):
    from mlx_lm_b200 import ops
    torch.manual_seed(T + F)
    both = (3 * torch.randn(T, 2 * F)).to(act)
    out = torch.zeros(T, F, dtype=act, device=DEV)
    ops.gated_unit(both.to(DEV), out, stream(), unit="bounded", limit=limit)
    g, u = both[:, :F].double().clamp(max=limit), both[:, F:].double().clamp(-limit, limit)
    want = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    close = lambda got, ref: float(((got.double().cpu() - ref).abs() / ref.abs().clamp_min(1.0)).max())
    assert close(out, want) < (1e-5 if act == torch.float32 else 5e-3)
    silu = torch.zeros(T, F, dtype=act, device=DEV)
    ops.gated_unit(both.to(DEV), silu, stream())
    plain_silu = both[:, :F].double() * torch.sigmoid(both[:, :F].double()) * both[:, F:].double()
    assert close(silu, plain_silu) < (1e-5 if act == torch.float32 else 5e-3)


def expert_rows(x, w_in, w_out, sel_e, sel_w, limit):
    """Every slot's expert output times its weight, float64; None for slots without an expert."""
    T, top = sel_e.shape
    out = []
    for t in range(T):
        for c in range(top):
            e = int(sel_e[t, c])
            if e < 0:
                out.append(None)
                continue
            F = w_in.shape[1] // 2
            w = {"e.gate": w_in[e, :F].double(), "e.up": w_in[e, F:].double(), "e.down": w_out[e].double()}
            out.append(sel_w[t * top + c].double() * plain.bounded_unit(x[t:t + 1].double(), w, "e", limit)[0])
    return out


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("T,D,F,E,top,limit", [(70, 64, 32, 6, 2, 1.5), (300, 96, 128, 5, 3, 0.8), (1, 64, 64, 10, 1, 2.0),
                                                (37, 50, 14, 5, 2, 1.0), (9, 48, 16, 9, 9, 3.0)])
def test_experts_products_with_the_bounded_unit(act, T, D, F, E, top, limit):
    """The weight multiplies the unit's output; slots of identity experts (-2) and of rows that pad the step (-1) are
    passed over by the plan."""
    from mlx_lm_b200 import ops
    torch.manual_seed(T + D + F + E)
    S = T * top
    x = torch.randn(T, D).to(act)
    w_in = (2 * torch.randn(E, 2 * F, D) * D ** -0.5).to(act)
    w_out = (torch.randn(E, D, F) * F ** -0.5).to(act)
    sel_e = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    if T > 20:
        sel_e[11] = -1
        sel_e[12, 0] = -2
        sel_e[30:33, -1] = -2
    sel_w = torch.rand(S) + 0.2
    want = expert_rows(x, w_in, w_out, sel_e, sel_w, limit)
    tc = act == torch.bfloat16 and D % 8 == 0 and F % 8 == 0
    for rows in [ops.moe_tile_rows(tc)] + ([ops.moe_few_rows()] if tc else []):
        max_tiles = ops.moe_max_tiles(S, E, rows)
        order = torch.full((S,), -1, dtype=torch.int32, device=DEV)
        tiles = torch.full((3 * max_tiles + 1,), -1, dtype=torch.int32, device=DEV)
        ops.moe_plan(sel_e.flatten().to(DEV), S, E, rows, order, tiles, tiles[3 * max_tiles:], stream())
        xd, wi, wo = x.to(DEV), w_in.to(DEV), w_out.to(DEV)
        h = torch.full((S, F), 7.0, dtype=act, device=DEV)
        ops.moe_gemm(xd, top, wi, F, order, tiles, tiles[3 * max_tiles:], max_tiles, rows, h, stream(), sel_weight=sel_w.to(DEV),
                     gated=True, unit="bounded", limit=limit)
        y = torch.full((S, D), 7.0, device=DEV)
        ops.moe_gemm(h, 1, wo, D, order, tiles, tiles[3 * max_tiles:], max_tiles, rows, y, stream())
        tol = 3e-5 if act == torch.float32 else 5e-2
        for s in range(S):
            if want[s] is None:
                assert bool((y[s] == 7.0).all())
            else:
                assert float((y[s].double().cpu() - want[s]).abs().max()) < tol * max(1.0, float(want[s].abs().max())), (rows, s)


@pytest.mark.parametrize("T,D,F,E,top,limit", [(700, 64, 64, 4, 2, 1.5), (1100, 128, 192, 12, 4, 0.9)])
def test_experts_products_with_the_bounded_unit_on_tcgen05(T, D, F, E, top, limit):
    from mlx_lm_b200 import ops
    torch.manual_seed(T + D + F + E)
    S = T * top
    act = torch.bfloat16
    x = torch.randn(T, D).to(act)
    w_in = (2 * torch.randn(E, 2 * F, D) * D ** -0.5).to(act)
    w_out = (torch.randn(E, D, F) * F ** -0.5).to(act)
    sel_e = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32)
    sel_e[11] = -1
    sel_e[12:40, 0] = -2
    sel_w = torch.rand(S) + 0.2
    want = expert_rows(x, w_in, w_out, sel_e, sel_w, limit)
    rows = ops.moe_tc05_tile_rows()
    max_tiles = ops.moe_max_tiles(S, E, rows)
    order = torch.full((S,), -1, dtype=torch.int32, device=DEV)
    tiles = torch.full((3 * max_tiles + 1,), -1, dtype=torch.int32, device=DEV)
    n_tiles = tiles[3 * max_tiles:]
    ops.moe_plan(sel_e.flatten().to(DEV), S, E, rows, order, tiles, n_tiles, stream())
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    xs = torch.zeros((S, D), dtype=act, device=DEV)
    ops.moe_gather(x.to(DEV), top, order, tiles, n_tiles, max_tiles, xs, stream())
    h = torch.full((S, F), 7.0, dtype=act, device=DEV)
    ops.moe_gemm_tc05(xs, w_in.to(DEV), F, order, tiles, n_tiles, max_tiles, h, status, stream(), sel_weight=sel_w.to(DEV),
                      gated=True, unit="bounded", limit=limit)
    y = torch.full((S, D), 7.0, device=DEV)
    ops.moe_gemm_tc05(h, w_out.to(DEV), D, order, tiles, n_tiles, max_tiles, y, status, stream())
    assert int(status.item()) == 0
    yc = y.double().cpu()
    for s in range(0, S, 3):
        if want[s] is None:
            assert bool((y[s] == 7.0).all())
        else:
            assert float((yc[s] - want[s]).abs().max()) < 5e-2 * max(1.0, float(want[s].abs().max())), s


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("C,taps", [(64, 4), (50, 3), (24, 2), (16, 1), (40, 7)])
def test_convolution_without_activation_keeps_its_state_across_steps(act, C, taps):
    """Two requests, cut into steps of 1, 2, 3 and more rows (shorter and longer than the taps), side by side in a
    batch, in slots that held something else before."""
    from mlx_lm_b200 import ops
    torch.manual_seed(C + taps)
    n = {0: 45, 1: 19}
    u = {r: torch.randn(n[r], C).to(act) for r in n}
    wt = torch.randn(C, taps).to(torch.bfloat16).float()
    want = {r: plain.short_convolution(u[r].double(), wt.double()) for r in n}
    slots_of = {0: 2, 1: 0}
    state = torch.full((3, max(taps - 1, 0), C), 5.0, device=DEV)
    for s in slots_of.values():
        state[s].zero_()                      # what taking a slot does
    done = {0: 0, 1: 0}
    cuts = [(1, 2), (2, 1), (3, 1), (1, 3), (20, 1), (2, 11), (16, 0)]
    wd, wtd = wt.to(DEV).contiguous(), wt.t().contiguous().to(DEV)
    worst = 0.0
    for cut in cuts:
        entries = [(r, done[r], min(m, n[r] - done[r])) for r, m in enumerate(cut) if min(m, n[r] - done[r]) > 0]
        x = torch.cat([u[r][p0:p0 + m] for r, p0, m in entries]).to(DEV)
        T = x.shape[0]
        req = [k for k, (_, _, m) in enumerate(entries) for _ in range(m)]
        pos = [p for _, p0, m in entries for p in range(p0, p0 + m)]
        first_tok = [sum(m for _, _, m in entries[:k]) for k in range(len(entries))] + [T]
        out = torch.zeros(T, C, dtype=act, device=DEV)
        ops.conv_silu(x, wd, None, state, i32([slots_of[r] for r, _, _ in entries]), i32(pos), i32(req), i32(first_tok),
                      i32([p0 for _, p0, _ in entries]), out, stream(), weight_by_tap=wtd, activation=False)
        o = out.double().cpu()
        for k, (r, p0, m) in enumerate(entries):
            worst = max(worst, float((o[first_tok[k]:first_tok[k] + m] - want[r][p0:p0 + m]).abs().max()))
            done[r] += m
    assert done == n
    assert worst < (1e-5 if act == torch.float32 else 0.06), worst
    if taps > 1:
        assert bool((state[1] == 5.0).all())          # nobody's slot: untouched


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,Hv,dk,dv,dims,base,scaling,head_norm", [
    (4, 2, 2, 32, 16, 24, 5000.0, stretch(8.0, 32, 4.0, 1.0), True),
    (8, 2, 2, 64, 64, 64, 50000.0, stretch(16.0, 128), True),
    (3, 1, 1, 12, 10, 6, 77.0, stretch(3.0, 20, 5.0, 0.7), True),
    (2, 2, 2, 16, 32, 16, 100.0, None, True),
    (4, 2, 2, 16, 8, 0, 100.0, None, True),
    (12, 4, 2, 16, 24, 0, 100.0, None, False),          # two score maps a key/value head: half as many value heads
    (6, 6, 3, 6, 10, 0, 100.0, None, False),
])
def test_queries_keys_and_values_on_their_way_to_the_pages(act, H, G, Hv, dk, dv, dims, base, scaling, head_norm):
    from mlx_lm_b200 import ops
    from mlx_lm_b200.parts import rotation_frequencies
    torch.manual_seed(H * dk + dv)
    T, page, n_pages, eps = 37, 16, 5, 1e-5
    Dh, Dvr = (dk + 7) // 8 * 8, (dv + 7) // 8 * 8
    n = (H + G) * dk + Hv * dv
    proj = torch.randn(T, n).to(act)
    positions = list(range(3, 3 + T))
    order = [3, 0, 4]
    table = torch.full((1, 8), -1, dtype=torch.int32)
    table[0, :3] = torch.tensor(order)
    kp = torch.full((n_pages, G, page, Dh), float("nan"), dtype=act, device=DEV)
    vp = torch.full((n_pages, Hv, page, Dvr), float("nan"), dtype=act, device=DEV)
    q_out = torch.full((T, H * Dh), float("nan"), device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    freq, mag = (None, 1.0)
    if dims:
        f, mag = rotation_frequencies(dims, base, scaling)
        freq = torch.tensor(f, dtype=torch.float64).float().to(DEV)
    ops.qkv_prepare(proj.to(DEV), 0, H * dk, (H + G) * dk, H, G, dk, dv, None, None, eps, freq, i32(positions), i32([0] * T),
                    table.to(DEV), kp, vp, q_out, True, status, stream(), interleaved=True, mscale=mag,
                    head_norm_eps=eps if head_norm else None)
    assert int(status.item()) == 0
    p64 = proj.double()
    q, k = p64[:, :H * dk].view(T, H, dk), p64[:, H * dk:(H + G) * dk].view(T, G, dk)
    v = p64[:, (H + G) * dk:].view(T, Hv, dv)
    if dims:
        cos, sin = plain.yarn_table(3 + T, rot(dims, base, scaling))
        q, k = plain.turn(q, cos[3:], sin[3:], dims), plain.turn(k, cos[3:], sin[3:], dims)
    if head_norm:
        q, k = plain.rms(q, eps), plain.rms(k, eps)
    tol = 2e-5 if act == torch.float32 else 0.03
    got_q = q_out.double().cpu().view(T, H, Dh)
    assert float((got_q[:, :, :dk] - q).abs().max()) < (2e-5 if act == torch.float32 else 4e-4 * max(1.0, mag))   # float32 out of rounded inputs
    assert bool((got_q[:, :, dk:] == 0).all())
    for t in range(T):
        p = positions[t]
        pg, r = order[p // page], p % page
        assert float((kp[pg, :, r, :dk].double().cpu() - k[t]).abs().max()) < tol
        assert float((vp[pg, :, r, :dv].double().cpu() - v[t]).abs().max()) < (1e-6 if act == torch.float32 else 1e-6)
        assert bool((kp[pg, :, r, dk:] == 0).all()) and bool((vp[pg, :, r, dv:] == 0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,G,dk,dv", [(4, 2, 32, 64), (6, 2, 16, 24), (3, 3, 6, 10), (8, 4, 64, 64), (3, 1, 48, 40), (4, 2, 64, 128),
                                       (6, 1, 64, 192)])
def test_two_score_maps_over_the_same_values(act, H, G, dk, dv):
    """``2 H`` query heads in the kernels' order, ``2 G`` key heads, ``G`` value heads: every map is an attention of its
    own over its key/value head's values; then the difference of the maps, normed per head.  On the CUDA cores and,
    in bfloat16, on tensor cores as portions and as single rows (whole, and split over CTAs); maps of 64 over values of
    a multiple of 64 also on the tcgen05 kernel for portions (bfloat16 queries, float32 and bfloat16 results)."""
    from mlx_lm_b200 import ops
    torch.manual_seed(H + dk + dv)
    T, page, scale, lam, eps, post = 150, 16, 0.4, 0.37, 1e-5, 0.7
    rep = H // G
    q = torch.randn(T, H, 2, dk)
    k = torch.randn(T, G, 2, dk).to(act)
    v = torch.randn(T, G, dv).to(act)
    q[:, :, :, 0] *= 3.0                   # a few sharp scores
    n_pages = (T + page - 1) // page + 2
    order = list(reversed(range(n_pages)))
    Dh, Dvr = (dk + 7) // 8 * 8, (dv + 7) // 8 * 8
    kp = paged(k.reshape(T, 2 * G, dk), 2 * G, Dh, page, act, n_pages, order)
    vp = paged(v, G, Dvr, page, act, n_pages, order)
    table = torch.full((1, n_pages), -1, dtype=torch.int32)
    table[0] = torch.tensor(order)
    # the kernels' order of the query heads: key head, map, head of the group
    qk = torch.stack([q[:, g * rep + r, m] for g in range(G) for m in range(2) for r in range(rep)], dim=1)      # [T, 2H, dk]
    qd = torch.zeros(T, 2 * H * Dh, device=DEV)
    qd.view(T, 2 * H, Dh)[:, :, :dk] = qk.to(DEV)
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    maps = torch.zeros(T, 2 * H, dv, dtype=torch.float64)
    for a in range(H):
        c, r = a // rep, a % rep
        first = plain.causal_softmax_values(q[:, a, 0].double(), k[:, c, 0].double(), v[:, c].double(), scale)
        second = plain.causal_softmax_values(q[:, a, 1].double(), k[:, c, 1].double(), v[:, c].double(), scale)
        maps[:, (2 * c) * rep + r], maps[:, (2 * c + 1) * rep + r] = first, second
        want[:, a] = plain.rms(first - lam * second, eps) * post
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 2e-5 if act == torch.float32 else 2e-2
    out = torch.full((T, 2 * H * dv), 7.0, device=DEV)
    ops.attention_wide(qd, Dh, i32(list(range(T))), i32([0] * T), table.to(DEV), kp, vp, out, dv, 2 * H, dk, dv, scale, status,
                       stream())
    assert int(status.item()) == 0
    assert float((out.double().cpu().view(T, 2 * H, dv) - maps).abs().max()) < tol
    o = torch.zeros(T, H * dv, dtype=act, device=DEV)
    ops.head_difference(out, rep, dv, lam, eps, post, o, stream(), token_req=i32([0] * 5 + [-1] + [0] * (T - 6)))
    got = o.double().cpu().view(T, H, dv)
    keep = [t for t in range(T) if t != 5]
    assert float((got[keep] - want[keep]).abs().max()) < (1e-4 if act == torch.float32 else 4e-2)
    assert bool((o[5] == 0).all())
    if act == torch.bfloat16 and ops.attention_wide_tc_supported(kp, vp, 2 * H, dk, dv, False):
        tiles = i32([[128, T - 128, 0, 128], [0, 0, 0, 0], [0, 128, 0, 0]])
        out2 = torch.full((T, 2 * H * dv), 7.0, device=DEV)
        ops.attention_wide_tiles(qd, Dh, tiles, 3, 128, table.to(DEV), kp, vp, out2, dv, 2 * H, dk, dv, scale, status, stream())
        assert int(status.item()) == 0
        assert float((out2.double().cpu().view(T, 2 * H, dv) - maps).abs().max()) < tol
        q16 = qd.to(torch.bfloat16)
        if dk == 64 and dv % 64 == 0 and ops.attention_portions_tc_supported(q16, out2, kp, vp):
            # the same queries rounded to bfloat16, as the tcgen05 kernel takes them
            maps16 = torch.zeros(T, 2 * H, dv, dtype=torch.float64)
            qr = q.to(torch.bfloat16).double()
            for a in range(H):
                c, r = a // rep, a % rep
                for m in range(2):
                    maps16[:, (2 * c + m) * rep + r] = plain.causal_softmax_values(qr[:, a, m], k[:, c, m].double(), v[:, c].double(), scale)
            # (this kernel fetches whole blocks of 128 keys and multiplies the values of masked keys by zero: its pools
            # are finite everywhere, as the engine's, which are zero-filled when they are made)
            kz, vz = torch.nan_to_num(kp), torch.nan_to_num(vp)
            for odt in (torch.float32, torch.bfloat16):
                out4 = torch.full((T, 2 * H * dv), 7.0, dtype=odt, device=DEV)
                ops.attention_portions(q16, tiles, 3, table.to(DEV), kz, vz, out4, 2 * H, scale, 0, status, stream())
                assert int(status.item()) == 0
                assert float((out4.double().cpu().view(T, 2 * H, dv) - maps16).abs().max()) < tol
        rows = [0, 1, 63, 64, 65, 127, 128, T - 1]
        singles = i32([[r, 1, 0, r] for r in rows] + [[5, 0, 0, 0]])
        for split in (False, True):
            out3 = torch.full((T, 2 * H * dv), 7.0, device=DEV)
            scratch = None
            if split:
                need = ops.attention_wide_scratch(len(rows) + 1, 2 * H, dv, 0, 0, 4096)
                scratch = torch.full((need,), float("nan"), device=DEV)
            ops.attention_wide_tiles(qd, Dh, singles, len(rows) + 1, 1, table.to(DEV), kp, vp, out3, dv, 2 * H, dk, dv, scale,
                                     status, stream(), scratch=scratch, max_len=4096 if split else 0)
            assert int(status.item()) == 0
            assert float((out3.double().cpu().view(T, 2 * H, dv)[rows] - maps[rows]).abs().max()) < tol
            assert bool((out3[5] == 7.0).all())


@pytest.mark.parametrize("act", ACT)
@pytest.mark.parametrize("H,d,dr,R,base,scaling", [(4, 16, 8, 40, 10000.0, stretch(4.0, 64, 8.0, 0.5)), (5, 10, 6, 21, 50.0, None),
                                                    (8, 64, 32, 128, 10000.0, stretch(2.0, 256, 16.0, 2.0))])
def test_latent_row_with_a_stretched_rotation(act, H, d, dr, R, base, scaling):
    from mlx_lm_b200 import ops
    from mlx_lm_b200.parts import rotation_frequencies
    torch.manual_seed(H + d + R)
    T, page, n_pages, eps = 29, 16, 4, 1e-5
    lat = R + dr
    row = (lat + 7) // 8 * 8
    proj = torch.randn(T, H * (d + dr) + lat).to(act)
    nw = (1 + 0.1 * torch.randn(R)).float()
    positions = list(range(7, 7 + T))
    order = [2, 0, 3]
    table = torch.full((1, 6), -1, dtype=torch.int32)
    table[0, :3] = torch.tensor(order)
    pool = torch.full((n_pages, 1, page, row), float("nan"), dtype=act, device=DEV)
    q_lat = torch.full((T, H * lat), 7.0, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    f, mag = rotation_frequencies(dr, base, scaling)
    freq = torch.tensor(f, dtype=torch.float64).float().to(DEV)
    ops.latent_prepare(proj.to(DEV), 0, H * (d + dr), H, d, dr, R, nw.to(DEV), eps, freq, True, i32(positions), i32([0] * T),
                       table.to(DEV), pool, True, q_lat, lat, status, stream(), mscale=mag)
    assert int(status.item()) == 0
    p64 = proj.double()
    cos, sin = plain.yarn_table(7 + T, rot(dr, base, scaling))
    qr = plain.turn(p64[:, :H * (d + dr)].view(T, H, d + dr)[:, :, d:], cos[7:], sin[7:], dr)
    down = p64[:, H * (d + dr):]
    c = plain.rms(down[:, :R], eps) * nw.double()
    kr = plain.turn(down[:, None, R:], cos[7:], sin[7:], dr)[:, 0]
    tol = 2e-5 if act == torch.float32 else 0.03
    assert float((q_lat.double().cpu().view(T, H, lat)[:, :, R:] - qr).abs().max()) < 2e-5 * max(1.0, mag) * 4
    for t in range(T):
        p = positions[t]
        got = pool[order[p // page], 0, p % page].double().cpu()
        assert float((got[:R] - c[t]).abs().max()) < tol and float((got[R:lat] - kr[t]).abs().max()) < tol
        assert bool((got[lat:] == 0).all())
