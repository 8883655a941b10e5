"""The kernels added for Kapitar, one by one, against float64 restatements (tests/plain_kapitar.py and
this file): norms on both sides of a sublayer, bias + activation, the gated unit norm, the linear-attention
recurrence (serial and cut into chunks, from a given state), the router (groups, kept groups, top
experts), the experts' grouped products with the routing given, their weighted sum."""

import math

import numpy as np
import pytest
import torch

import plain_kapitar as K

pytestmark = pytest.mark.gpu

DEV = "cuda"


def rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("hidden", [96, 320, 2500, 4100])     # (4,100: beyond the rows the register kernel takes)
def test_norms_around_a_sublayer(dtype, tol, hidden):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(hidden)
    T = 19
    res = (torch.randn(T, hidden, generator=g) * 3 + 1.5).to(DEV)          # a mean well away from zero
    delta = (torch.randn(T, hidden, generator=g) * 2 - 0.7).to(dtype).to(DEV)
    wb = (1 + 0.2 * torch.randn(hidden, generator=g)).to(dtype).to(DEV)
    wn = (1 + 0.2 * torch.randn(hidden, generator=g)).to(dtype).to(DEV)
    eps = 1e-5
    for kind, norm in ((kernels.NORM_LAYER, K.layer_norm),
                       (kernels.NORM_RMS, lambda x, w, e: K.unit_rms(x, e) * w)):
        r = res.clone()
        out = torch.empty(T, hidden, dtype=dtype, device=DEV)
        kernels.sandwich_norm(r, delta, wb, wn, out, eps, kind)
        want_r = res.double() + norm(delta.double(), wb.double(), eps)
        assert rel(r, want_r) < 2e-6
        assert rel(out, norm(want_r, wn.double(), eps)) < tol
        # a plain add, then the norm; and rows picked by index without an add
        r = res.clone()
        kernels.sandwich_norm(r, delta, None, wn, out, eps, kind)
        assert rel(r, res.double() + delta.double()) < 1e-6
        idx = torch.tensor([5, 0, 5, 18], dtype=torch.int32, device=DEV)
        picked = torch.empty(4, hidden, dtype=dtype, device=DEV)
        r = res.clone()
        kernels.sandwich_norm(r, None, None, wn, picked, eps, kind, rows_idx=idx)
        assert torch.equal(r, res)
        assert rel(picked, norm(res.double()[idx.long()], wn.double(), eps)) < tol
        # only the normed add
        r = res.clone()
        kernels.sandwich_norm(r, delta, wb, None, None, eps, kind)
        assert rel(r, want_r) < 2e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-6), (torch.bfloat16, 1e-2)])
def test_bias_activation_and_gated_norm(dtype, tol):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(1)
    x = (torch.randn(7, 200, generator=g) * 2).to(dtype).to(DEV)
    b = torch.randn(120, generator=g).to(DEV)
    for name, f in (("relu_squared", lambda z: torch.relu(z) ** 2), ("gelu", K.gelu_erf), ("silu", K.silu),
                    ("gelu_tanh", lambda z: 0.5 * z * (1 + torch.tanh(math.sqrt(2 / math.pi) * (z + 0.044715 * z ** 3))))):
        y = x.clone()
        kernels.bias_act(y, b, kernels.ACTIVATIONS[name], cols=120)
        z = (x[:, :120].double() + b.double())
        if dtype == torch.bfloat16:
            z = z.to(dtype).double()
        assert rel(y[:, :120], f(z)) < tol
        assert torch.equal(y[:, 120:], x[:, 120:])
    o = (torch.randn(9, 72, generator=g) * 5).to(DEV)
    buf = torch.randn(9, 200, generator=g).to(dtype).to(DEV)
    w = (1 + 0.1 * torch.randn(72, generator=g)).to(dtype).to(DEV)
    out = torch.empty(9, 72, dtype=dtype, device=DEV)
    kernels.gated_rmsnorm(o, buf[:, 100:172], w, out, 1e-6)
    want = K.unit_rms(o.double(), 1e-6) * w.double() * torch.sigmoid(buf[:, 100:172].double())
    assert rel(out, want) < tol


def recurrence(q, k, v, decay, S):
    """q, k [T, H, D], v [T, H, DV], S [H, D, DV] float64 -> (o [T, H, DV], final S)."""
    S = S.clone()
    o = torch.zeros(q.shape[0], q.shape[1], v.shape[2], dtype=torch.float64)
    for t in range(q.shape[0]):
        for h in range(q.shape[1]):
            S[h] = decay[h] * S[h] + torch.outer(k[t, h], v[t, h])
            o[t, h] = S[h].T @ q[t, h]
    return o, S


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,D,DV", [(3, 16, 24), (1, 40, 130), (2, 64, 64)])
def test_linear_attention_from_a_state_serial_and_in_chunks(dtype, H, D, DV):
    """Three sequences of unequal length in one launch (one of a single token), each from its own
    non-zero state in its own slot; long ones cut into chunks, with a last chunk of another length."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(D)
    lens = [333, 1, 70]
    slots = [4, 0, 2]
    decay = [0.999, 0.6, 0.9][:H]
    T = sum(lens)
    width = 2 * H * D + H * DV + 5
    proj = (torch.randn(T, width, generator=g) * 0.5).to(dtype)
    state0 = torch.randn(6, H, D, DV, generator=g)
    seq_of = torch.tensor(sum(([i] * n for i, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    want_o, want_S = [], {}
    at = 0
    for n, s in zip(lens, slots):
        p = proj[at:at + n].double()
        o, S = recurrence(p[:, :H * D].view(n, H, D), p[:, H * D:2 * H * D].view(n, H, D),
                          p[:, 2 * H * D:2 * H * D + H * DV].view(n, H, DV), decay, state0[s].double())
        want_o.append(o.reshape(n, H * DV))
        want_S[s] = S
        at += n
    want_o = torch.cat(want_o)
    for chunked in (False, True):
        state = state0.clone().to(DEV)
        out = torch.zeros(T, H * DV, device=DEV)
        chunk, max_chunks = (64, (max(lens) + 63) // 64) if chunked else (0, 1)
        scratch = torch.full((3 * max_chunks * H * D * DV,), float("nan"), device=DEV) if chunked else None
        kernels.linear_attention(proj.to(DEV), 0, H * D, 2 * H * D, seq_of, slot_t, dec, state, out, T, 3, H, D, DV,
                                 scratch, chunk, max_chunks)
        assert rel(out, want_o) < (2e-5 if dtype == torch.float32 else 2e-5), chunked
        for s in range(6):
            if s in want_S:
                assert rel(state[s], want_S[s]) < 2e-5
            else:
                assert torch.equal(state[s].cpu(), state0[s])          # other requests' slots are not touched
    assert kernels.linear_attention_chunks(100) == (0, 1)
    c, m = kernels.linear_attention_chunks(5000)
    assert c * m >= 5000 and m <= kernels.LINEAR_ATTN_MAX_CHUNKS


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,groups,keep,top", [(8, 4, 2, 3), (16, 2, 1, 4), (6, 1, 1, 1), (12, 3, 3, 5), (64, 8, 3, 6)])
def test_router(dtype, E, groups, keep, top):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(E + top)
    T, W = 200, 72
    x = torch.randn(T, W, generator=g).to(dtype)
    wr = (torch.randn(E, W, generator=g) * 0.3).to(dtype)
    r = {"groups": {"count": groups, "keep": keep}, "top": top}
    choice, weight = K.route(x.double(), wr.double(), r)
    got_c = torch.zeros(T, top, dtype=torch.int32, device=DEV)
    got_w = torch.zeros(T, top, dtype=torch.float32, device=DEV)
    kernels.moe_route(x.to(DEV), wr.to(DEV), got_c, got_w, T, groups, keep, 2, top)
    # tokens whose choice hangs on a difference below the float32 noise of the scores are left out
    s = torch.sigmoid(x.double() @ wr.double().T)
    per = E // groups
    gscore = s.view(T, groups, per).topk(min(2, per), dim=-1).values.sum(-1).sort(dim=-1, descending=True).values
    clear = torch.ones(T, dtype=torch.bool)
    if keep < groups:
        clear &= (gscore[:, keep - 1] - gscore[:, keep]) > 1e-5
    allowed = torch.zeros(T, E, dtype=torch.bool)
    allowed.scatter_(1, choice, True)
    ranked = torch.where(allowed, torch.full_like(s, 2.0), s)
    kept_groups = torch.zeros(T, groups, dtype=torch.bool)
    kept_groups.scatter_(1, choice // per, True)
    runner_up = torch.where(kept_groups.repeat_interleave(per, dim=1) & ~allowed, s, torch.full_like(s, -1.0)).max(-1).values
    clear &= (weight.min(-1).values - runner_up) > 1e-5
    sorted_w = weight.sort(dim=-1, descending=True).values
    if top > 1:
        clear &= (sorted_w[:, :-1] - sorted_w[:, 1:]).min(-1).values > 1e-5
    assert clear.float().mean() > 0.9
    assert torch.equal(got_c.cpu().long()[clear], choice[clear])
    assert rel(got_w.cpu()[clear], weight[clear]) < 1e-5
    del ranked


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 1e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("T,E,top,W,ff", [(70, 8, 3, 96, 40), (5, 16, 4, 64, 24), (300, 4, 2, 72, 100), (1, 6, 1, 40, 8),
                                          (70, 8, 3, 100, 28)])     # (the last: no 16-byte pieces, no tensor-core tiles)
def test_experts_with_the_routing_given(dtype, tol, T, E, top, W, ff):
    """Pairs listed expert by expert in tiles, both grouped products and the weighted sum, against the
    plain expert applied pair by pair.  Some experts get no token, one gets more than a tile."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(T)
    x = torch.randn(T, W, generator=g).to(dtype)
    up = (torch.randn(E, ff, W, generator=g) / math.sqrt(W)).to(dtype)
    down = (torch.randn(E, W, ff, generator=g) / math.sqrt(ff)).to(dtype)
    shared = torch.randn(T, W, generator=g).to(dtype)
    choice = torch.stack([torch.randperm(E - 1, generator=g)[:top] for _ in range(T)]).to(torch.int32)   # expert E-1: none
    if T >= 70:
        choice[:70, 0] = 0                                                                               # expert 0: more than a tile of pairs
        for t in range(70):
            if (choice[t, 1:] == 0).any():
                choice[t, 1:][choice[t, 1:] == 0] = E - 1
    weight = torch.rand(T, top, generator=g)
    w = {}
    for e in range(E):
        w[f"e{e}.up"], w[f"e{e}.down"] = up[e].float(), down[e].float()
    K.STORE_DTYPE = None if dtype == torch.float32 else dtype
    try:
        want = torch.zeros(T, W, dtype=torch.float64)
        for t in range(T):
            for k in range(top):
                y = K.expert(x[t:t + 1].double(), w, f"e{int(choice[t, k])}.")[0]
                want[t] += float(weight[t, k]) * K.stored(y)
        want += shared.double()
    finally:
        K.STORE_DTYPE = None
    pairs = T * top
    tiles = kernels.moe_max_tiles(pairs, E)
    i32 = lambda n: torch.zeros(n, dtype=torch.int32, device=DEV)      # noqa: E731
    order, te, tb, trw, meta = i32(pairs), i32(tiles), i32(tiles), i32(tiles), i32(4)
    kernels.moe_group(choice.to(DEV).reshape(-1), pairs, E, order, te, tb, trw, meta)
    n_tiles = int(meta[0])
    counts = torch.bincount(choice.reshape(-1).long(), minlength=E)
    assert n_tiles == int(((counts + 63) // 64).sum())
    assert sorted(order.cpu().tolist()) == list(range(pairs))
    listed = choice.reshape(-1)[order.cpu().long()]
    assert torch.equal(listed, listed.sort().values)                    # expert by expert
    act = torch.full((pairs, ff), float("nan"), dtype=dtype, device=DEV)
    y = torch.full((pairs, W), float("nan"), dtype=dtype, device=DEV)
    xd = x.to(DEV)
    for few in (False, True):          # the tiled products, and the ones that stream the weights pair by pair
        act.fill_(float("nan"))
        y.fill_(float("nan"))
        kernels.moe_gemm(xd, top, up.to(DEV).reshape(E * ff, W), act, order, te, tb, trw, meta, tiles,
                         act=kernels.ACT_GELU_ERF, few_pairs=few)
        kernels.moe_gemm(act, 1, down.to(DEV).reshape(E * W, ff), y, order, te, tb, trw, meta, tiles, few_pairs=few)
        out = torch.empty(T, W, dtype=dtype, device=DEV)
        kernels.moe_combine(y, weight.to(DEV), shared.to(DEV), out, T, top)
        assert rel(out, want) < tol, few


def attend(q, k, v, pos0, size, keep, scale, cap, lam, post, eps, unit):
    """q [n, H, M, D] at positions pos0 .. pos0 + n - 1, k [L, G, M, D], v [L, G, DV], float64."""
    n, H, M, D = q.shape
    G = k.shape[1]
    out = torch.zeros(n, H, v.shape[2], dtype=torch.float64)
    for t in range(n):
        i = pos0 + t
        vis = torch.tensor([K.visible(i, j, size, keep) if size > 0 else j <= i for j in range(k.shape[0])])
        for h in range(H):
            g = h // (H // G)
            maps = []
            for m in range(M):
                s = (k[:, g, m] @ q[t, h, m]) * scale
                if cap > 0:
                    s = cap * torch.tanh(s / cap)
                s = s.masked_fill(~vis, -math.inf)
                maps.append(torch.softmax(s, 0) @ v[:, g])
            o = maps[0] if M == 1 else maps[0] - lam * maps[1]
            out[t, h] = K.unit_rms(o, eps) * post if unit else o
    return out.reshape(n, -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,M,D,DV,size,keep,cap", [
    (4, 2, 2, 16, 32, 24, 3, 12.0), (2, 1, 2, 48, 96, 40, 4, 20.0), (3, 3, 1, 32, 16, 0, 0, 0.0),
    (8, 2, 2, 64, 128, 100, 0, 30.0), (2, 2, 2, 24, 20, 9, 9, 5.0)])
def test_attention_with_maps_over_shuffled_pages(dtype, H, G, M, D, DV, size, keep, cap):
    """A portion of 150 tokens after 70 cached ones (tiles of 128 and 22 rows) and, in the same cache, single
    tokens at several contexts, over pages handed out in a shuffled order; cache rows that no query may
    read hold NaN.  The tensor-core kernel where it applies (bfloat16, sizes that are multiples of 16), the
    CUDA-core kernel, and the partitioned single-token kernel with its merge, against float64."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * D + DV)
    ps, L, p0 = 16, 220, 70
    n = L - p0
    scale, lam, post, eps = 0.2, 0.37, 0.6, 1e-5
    q = torch.randn(L, H, M, D, generator=g).to(dtype)
    k = torch.randn(L, G, M, D, generator=g).to(dtype)
    v = torch.randn(L, G, DV, generator=g).to(dtype)
    pages = (L + ps - 1) // ps
    perm = (torch.randperm(pages + 3, generator=g) + 1)[:pages].to(torch.int32)         # page 0 is never handed out
    kc = torch.full((pages + 4, G * M, ps, D), float("nan"), dtype=dtype)
    vc = torch.full((pages + 4, G, ps, DV), float("nan"), dtype=dtype)
    for j in range(L):
        kc[perm[j // ps], :, j % ps] = k[j].reshape(G * M, D)
        vc[perm[j // ps], :, j % ps] = v[j]
    if size > 0:       # what every query's window has passed (and is not kept) may hold anything: poison it
        for j in range(keep, max(0, p0 - size + 1)):
            kc[perm[j // ps], :, j % ps] = float("nan")
            vc[perm[j // ps], :, j % ps] = float("nan")
    kc, vc = kc.to(DEV), vc.to(DEV)
    table = torch.zeros(1, pages + 2, dtype=torch.int32)
    table[0, :pages] = perm
    table = table.to(DEV)
    want = attend(q[p0:].double(), k.double(), v.double(), p0, size, keep, scale, cap, lam, post, eps, True)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    qd = q[p0:].reshape(n, -1).contiguous().to(DEV)
    positions = torch.arange(p0, L, dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    tile_seq, tile_tok, tile_rows = i32([0, 0]), i32([0, 128]), i32([128, n - 128])
    impls = [1] + ([2] if dtype == torch.bfloat16 and D % 16 == 0 and DV % 16 == 0 else [])
    for impl in impls:
        out = torch.full((n, H * DV), float("nan"), dtype=dtype, device=DEV)
        kernels.maps_attn_prefill(qd, qd.stride(0), kc, vc, table, tile_seq, tile_tok, tile_rows, positions, out, 2,
                                  128, H, G, D, DV, M, ps, size, keep, scale, cap, lam, post, eps, True, impl=impl)
        assert rel(out, want) < tol, impl
    # single tokens: the last token of contexts that end at several places (also across a 128-key partition)
    ends = [p0 + 1, 128, 129, 130, L]
    rows = [e - 1 - p0 for e in ends]
    items = i32([[r, 0, e, 0] for r, e in zip(rows, ends)])
    parts = (L + 127) // 128
    part_o = torch.full((len(ends) * H * M * parts * DV,), float("nan"), device=DEV)
    part_ml = torch.full((len(ends) * H * M * parts * 2,), float("nan"), device=DEV)
    out = torch.zeros((n, H * DV), dtype=dtype, device=DEV)
    kernels.maps_attn_decode(qd, qd.stride(0), kc, vc, table, items, part_o, part_ml, parts, out, len(ends), H, G, D, DV,
                             M, ps, size, keep, scale, cap, lam, post, eps, True)
    assert rel(out[rows], want[rows]) < tol
