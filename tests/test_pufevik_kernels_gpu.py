"""The kernels added for Pufevik, one by one, against the float64 functions of tests/plain_pufevik.py: the add of
a normed sublayer output with the stream handed on as it is, the gated activation, the scaled embedding, the
norm / rotation / value blend of attention heads between projection and cache, attention with a sink and an
output gate over shuffled pages (tensor-core, CUDA-core and single-token kernels), and the matrix memory
(gates with stabiliser, recurrence from a given state, division + unit norm + gate)."""

import math

import pytest
import torch

import plain_pufevik as P

pytestmark = pytest.mark.gpu

DEV = "cuda"


def rel(a, b):
    return float((a.double().cpu() - b.double().cpu()).abs().max() / (b.double().abs().max() + 1e-30))


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("hidden", [100, 256, 4100])     # (4,100: beyond the rows the register kernel takes)
def test_normed_add_hands_the_stream_on_as_it_is(dtype, tol, hidden):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(hidden)
    T = 13
    res = (torch.randn(T, hidden, generator=g) * 3 + 0.5).to(DEV)
    delta = (torch.randn(T, hidden, generator=g) * 0.01).to(dtype).to(DEV)      # a small output: the norm must blow it up
    w = (1 + 0.2 * torch.randn(hidden, generator=g)).to(dtype).to(DEV)
    r = res.clone()
    out = torch.full((T, hidden), float("nan"), dtype=dtype, device=DEV)
    kernels.sandwich_norm(r, delta, w, None, out, 1e-5, kernels.NORM_RMS)
    want = res.double() + P.rms_norm(delta.double(), w.double(), 1e-5)
    assert rel(r, want) < 2e-6 and rel(out, want) < tol
    assert torch.equal(out, r.to(dtype))            # the copy is the stream, rounded once
    # without an addend: the copy alone, the stream untouched
    out.fill_(float("nan"))
    kernels.sandwich_norm(r, None, None, None, out, 0.0, kernels.NORM_RMS)
    assert torch.equal(out, r.to(dtype)) and rel(r, want) < 2e-6


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-6), (torch.bfloat16, 1e-2)])
def test_gated_activation_and_scaled_embedding(dtype, tol):
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(0)
    gu = (3 * torch.randn(9, 2 * 52, generator=g)).to(dtype).to(DEV)
    out = torch.empty(9, 52, dtype=dtype, device=DEV)
    kernels.gated_act(gu, out, kernels.ACTIVATIONS["gelu_tanh"])
    assert rel(out, P.gelu_tanh(gu[:, :52].double()) * gu[:, 52:].double()) < tol
    table = torch.randn(11, 40, generator=g).to(dtype).to(DEV)
    ids = torch.tensor([3, 0, 10, 3], dtype=torch.int32, device=DEV)
    res = torch.empty(4, 40, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    kernels.embedding(ids, table, res, status, 0.7)
    assert rel(res, table[ids.long()].double() * 0.7) < 1e-7 and int(status.item()) == 0


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 3e-6), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,G,D,DV,rot,mode", [(4, 2, 16, 8, 8, "each"), (3, 1, 20, 12, 20, "whole"), (2, 2, 32, 16, 2, "whole"),
                                               (8, 8, 64, 64, 0, "each"), (2, 1, 12, 4, 6, "none")])
def test_heads_between_projection_and_cache(dtype, tol, H, G, D, DV, rot, mode):
    """Norm per head or over the whole projection, rotation of the first entries in neighbouring pairs at
    scattered positions, and the values kept or blended; the gate columns behind them stay as they are."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * D + rot)
    T, eps, base, lam = 23, 1e-5, 300.0, 0.3
    positions = torch.randperm(500, generator=g)[:T]          # scattered, each once
    qs, ks, vs, extra = H * D, G * D, G * DV, 5
    x = (2 * torch.randn(T, qs + ks + vs + extra, generator=g)).to(dtype)
    whole = mode == "whole"
    wq = (1 + 0.3 * torch.randn(qs if whole else D, generator=g)).to(dtype)
    wk = (1 + 0.3 * torch.randn(ks if whole else D, generator=g)).to(dtype)
    first = torch.randn(T, vs, generator=g).to(dtype)

    def expect(sec, heads, w):
        s = sec.double()
        if mode == "each":
            s = P.rms_norm(s.view(T, heads, D), w.double(), eps)
        elif whole:
            s = P.rms_norm(s, w.double(), eps).view(T, heads, D)
        else:
            s = s.view(T, heads, D)
        if rot:
            big = torch.zeros(500, heads, D, dtype=P.F64)
            big[positions] = s
            s = P.rotate_pairs(big, base, rot)[positions]
        return s.reshape(T, -1)

    cos = sin = None
    if rot:
        a = torch.arange(500, dtype=P.F64)[:, None] * torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=P.F64)
        cos, sin = torch.cos(a).float().to(DEV), torch.sin(a).float().to(DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    norm_mode = {"none": kernels.HEAD_NORM_NONE, "each": kernels.HEAD_NORM_EACH, "whole": kernels.HEAD_NORM_WHOLE}[mode]
    for mix_mode in (kernels.VALUE_MIX_KEEP, kernels.VALUE_MIX_BLEND, kernels.VALUE_MIX_NONE):
        xd, fd = x.clone().to(DEV), first.clone().to(DEV)
        kernels.head_prep(xd, positions.to(torch.int32).to(DEV), T, 0, H, qs, G, D, status,
                          wq.to(DEV) if mode != "none" else None, wk.to(DEV) if mode != "none" else None, norm_mode, eps,
                          cos, sin, qs + ks, vs, fd if mix_mode else None, mix_mode, lam)
        assert rel(xd[:, :qs], expect(x[:, :qs], H, wq)) < tol
        assert rel(xd[:, qs:qs + ks], expect(x[:, qs:qs + ks], G, wk)) < tol
        v = x[:, qs + ks:qs + ks + vs].double()
        if mix_mode == kernels.VALUE_MIX_BLEND:
            assert rel(xd[:, qs + ks:qs + ks + vs], (1 - lam) * v + lam * first.double()) < tol
        else:
            assert torch.equal(xd[:, qs + ks:qs + ks + vs].cpu(), x[:, qs + ks:qs + ks + vs])
        assert torch.equal(fd.cpu(), x[:, qs + ks:qs + ks + vs] if mix_mode == kernels.VALUE_MIX_KEEP else first)
        assert torch.equal(xd[:, qs + ks + vs:].cpu(), x[:, qs + ks + vs:])
    assert int(status.item()) == 0
    # the same with the finished keys and values written to their paged caches: shuffled slots, one token without
    ps, pages = 8, 9
    slots = torch.randperm(ps * pages, generator=g)[:T].to(torch.int32)
    slots[3] = -1
    kc = torch.full((pages, G, ps, D), float("nan"), dtype=dtype, device=DEV)
    vc = torch.full((pages, G, ps, DV), float("nan"), dtype=dtype, device=DEV)
    xd, fd = x.clone().to(DEV), first.clone().to(DEV)
    kernels.head_prep(xd, positions.to(torch.int32).to(DEV), T, 0, H, qs, G, D, status,
                      wq.to(DEV) if mode != "none" else None, wk.to(DEV) if mode != "none" else None, norm_mode, eps,
                      cos, sin, qs + ks, vs, fd, kernels.VALUE_MIX_BLEND, lam, slots.to(DEV), kc, vc, ps)
    assert rel(xd[:, :qs], expect(x[:, :qs], H, wq)) < tol and int(status.item()) == 0
    written = torch.zeros(pages * ps, dtype=torch.bool)
    for t in range(T):
        sl = int(slots[t])
        if sl < 0:
            continue
        written[sl] = True
        assert torch.equal(kc[sl // ps, :, sl % ps].reshape(-1), xd[t, qs:qs + ks])
        assert torch.equal(vc[sl // ps, :, sl % ps].reshape(-1), xd[t, qs + ks:qs + ks + vs])
    assert torch.isnan(kc.permute(0, 2, 1, 3).reshape(pages * ps, -1)[~written]).all()
    assert torch.isnan(vc.permute(0, 2, 1, 3).reshape(pages * ps, -1)[~written]).all()
    slots[5] = pages * ps            # beyond the pool: flagged, not written
    kernels.head_prep(x.clone().to(DEV), positions.to(torch.int32).to(DEV), T, 0, H, qs, G, D, status, None, None,
                      kernels.HEAD_NORM_NONE, eps, None, None, qs + ks, vs, None, kernels.VALUE_MIX_NONE, 0.0,
                      slots.to(DEV), kc, vc, ps)
    assert int(status.item()) == 4
    status.zero_()
    if rot:      # a position beyond the tables is flagged, not read
        kernels.head_prep(x.clone().to(DEV), torch.full((T,), 500, dtype=torch.int32, device=DEV), T, 0, H, qs, G, D, status,
                          None, None, kernels.HEAD_NORM_NONE, eps, cos, sin)
        assert int(status.item()) == 2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,D,DV,size,sink,gate", [
    (4, 1, 80, 32, 56, True, 1), (4, 2, 16, 48, 24, True, 1), (2, 2, 32, 16, 0, False, 2), (8, 2, 64, 64, 130, True, 2),
    (3, 3, 20, 12, 9, True, 1), (2, 1, 112, 80, 0, False, 2), (2, 2, 16, 16, 1, True, 0), (2, 1, 7, 5, 30, True, 2),
    (4, 2, 33, 18, 0, True, 1)])
def test_attention_with_a_sink_and_a_gate_over_shuffled_pages(dtype, H, G, D, DV, size, sink, gate):
    """A portion of 150 tokens after 70 cached ones and, in the same cache, single tokens at several contexts,
    over pages handed out in a shuffled order; cache rows that no query may read hold NaN.  One sink is made
    so large that it takes most of its head's weight, one so small that it takes none."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * D + DV + size)
    ps, L, p0 = 16, 220, 70
    n = L - p0
    scale, post = 0.2, 0.8
    q = torch.randn(L, H, D, generator=g).to(dtype)
    k = torch.randn(L, G, D, generator=g).to(dtype)
    v = torch.randn(L, G, DV, generator=g).to(dtype)
    sk = torch.randn(H, generator=g)
    sk[0], sk[-1] = 6.0, -30.0
    gates = torch.randn(L, H if gate == 1 else H * DV, generator=g).to(dtype)
    pages = (L + ps - 1) // ps
    perm = (torch.randperm(pages + 3, generator=g) + 1)[:pages].to(torch.int32)
    kc = torch.full((pages + 4, G, ps, D), float("nan"), dtype=dtype)
    vc = torch.full((pages + 4, G, ps, DV), float("nan"), dtype=dtype)
    for j in range(L):
        kc[perm[j // ps], :, j % ps] = k[j]
        vc[perm[j // ps], :, j % ps] = v[j]
    if size > 0:
        for j in range(0, max(0, p0 - size + 1)):
            kc[perm[j // ps], :, j % ps] = float("nan")
            vc[perm[j // ps], :, j % ps] = float("nan")
    kc, vc = kc.to(DEV), vc.to(DEV)
    table = torch.zeros(1, pages + 2, dtype=torch.int32)
    table[0, :pages] = perm
    table = table.to(DEV)
    o = P.softmax_attention(q.double(), k.double(), v.double(), scale, window=size, sink=sk.double() if sink else None)[p0:]
    if gate == 1:
        o = o * P.sigmoid(gates[p0:].double())[:, :, None]
    elif gate == 2:
        o = o * P.sigmoid(gates[p0:].double()).view(n, H, DV)
    want = (o * post).reshape(n, -1)
    tol = 2e-5 if dtype == torch.float32 else 1.5e-2
    # queries and gates side by side in one buffer, as a fused projection leaves them
    buf = torch.cat([q[p0:].reshape(n, -1), gates[p0:]], dim=1).contiguous().to(DEV)
    gd = buf[:, H * D:] if gate else None
    skd = sk.to(DEV) if sink else None
    positions = torch.arange(p0, L, dtype=torch.int32, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)      # noqa: E731
    tile_seq, tile_tok, tile_rows = i32([0, 0]), i32([0, 128]), i32([128, n - 128])
    impls = [1] + ([2] if dtype == torch.bfloat16 and D % 16 == 0 and DV % 16 == 0 else [])
    for impl in impls:
        # the output as columns of a wider buffer, as a mixer beside another one writes it
        wide = torch.full((n, H * DV + 6), float("nan"), dtype=dtype, device=DEV)
        out = wide[:, 4:4 + H * DV]
        kernels.maps_attn_prefill(buf, buf.stride(0), kc, vc, table, tile_seq, tile_tok, tile_rows, positions, out, 2,
                                  128, H, G, D, DV, 1, ps, size, 0, scale, 0.0, 0.0, post, 1e-5, False, skd, gd, gate,
                                  impl=impl)
        assert rel(out, want) < tol, impl
        assert torch.isnan(wide[:, :4]).all() and torch.isnan(wide[:, 4 + H * DV:]).all()
    ends = [p0 + 1, 128, 129, 130, L]
    rows = [e - 1 - p0 for e in ends]
    items = i32([[r, 0, e, 0] for r, e in zip(rows, ends)])
    parts = (L + 127) // 128
    part_o = torch.full((len(ends) * H * parts * DV,), float("nan"), device=DEV)
    part_ml = torch.full((len(ends) * H * parts * 2,), float("nan"), device=DEV)
    out = torch.zeros((n, H * DV), dtype=dtype, device=DEV)
    kernels.maps_attn_decode(buf, buf.stride(0), kc, vc, table, items, part_o, part_ml, parts, out, len(ends), H, G, D, DV,
                             1, ps, size, 0, scale, 0.0, 0.0, post, 1e-5, False, skd, gd, gate)
    assert rel(out[rows], want[rows]) < tol


@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-5), (torch.bfloat16, 1e-2)])
@pytest.mark.parametrize("H,D,DV,cap,lens", [
    (3, 16, 24, 14.0, (37, 1, 150)), (1, 32, 64, 4.0, (37, 1, 150)), (4, 8, 16, 30.0, (37, 1, 150)),
    (2, 10, 20, 8.0, (37, 1, 150)), (2, 64, 200, 11.0, (37, 1, 150)), (2, 16, 24, 13.0, (300, 1, 700)),
    (1, 32, 130, 6.0, (257, 64, 65))])
def test_matrix_memory_from_given_states(dtype, tol, H, D, DV, cap, lens):
    """Three unequal sequences of one step (one of a single token) from states that earlier steps left, in
    slots out of order; the slot of no sequence stays as it is.  Gates large enough for the stabiliser to
    matter (input gates up to the cap).  Long sequences are cut into chunks that run side by side (the last
    chunk of one is a single token, another has exactly one chunk, another one chunk and a token)."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(H * D + DV)
    lens, slots = list(lens), [2, 0, 3]
    T, W = sum(lens), 2 * H * D + 2 * H * DV
    floats = kernels.matrix_memory_state_floats(H, D, DV)
    proj = torch.randn(T, W, generator=g).to(dtype)
    zi, zf = 6 * torch.randn(T, H, generator=g), 3 * torch.randn(T, H, generator=g) + 2
    bi, bf = torch.randn(H, generator=g), torch.randn(H, generator=g)
    wn = (1 + 0.2 * torch.randn(H * DV, generator=g)).to(dtype)
    # states as a run over some earlier tokens would have left them
    state = torch.zeros(5, floats)
    plain_states = {}
    for s in slots + [1]:
        st = [dict() for _ in range(H)]
        t0 = 9
        q0, k0, v0 = torch.randn(t0, H, D, generator=g).double(), torch.randn(t0, H, D, generator=g).double(), torch.randn(t0, H, DV, generator=g).double()
        i0, f0 = 3 * torch.randn(t0, H, generator=g).double(), P.log_sigmoid(torch.randn(t0, H, generator=g).double())
        for h in range(H):
            P.matrix_memory(q0[:, h], k0[:, h], v0[:, h], i0[:, h], f0[:, h], st[h])
            plane = torch.cat([st[h]["S"], st[h]["n"][:, None]], dim=1)            # [D, DV + 1]
            state[s, h * D * (DV + 1):(h + 1) * D * (DV + 1)] = plane.reshape(-1).float()
            state[s, H * D * (DV + 1) + h] = st[h]["m"]
        plain_states[s] = st
    # (the float32 copy is what the kernel starts from)
    for s, st in plain_states.items():
        for h in range(H):
            plane = state[s, h * D * (DV + 1):(h + 1) * D * (DV + 1)].double().view(D, DV + 1)
            st[h].update(S=plane[:, :DV].clone(), n=plane[:, DV].clone(), m=float(state[s, H * D * (DV + 1) + h]))
    ig = cap * torch.tanh((zi.double() + bi.double()) / cap)
    fg = P.log_sigmoid(cap * torch.tanh((zf.double() + bf.double()) / cap))
    pd = proj.double()
    want = torch.zeros(T, H, DV, dtype=P.F64)
    t = 0
    for n, s in zip(lens, slots):
        for h in range(H):
            want[t:t + n, h] = P.matrix_memory(pd[t:t + n, h * D:(h + 1) * D] * D ** -0.5,
                                               pd[t:t + n, H * D + h * D:H * D + (h + 1) * D],
                                               pd[t:t + n, 2 * H * D + h * DV:2 * H * D + (h + 1) * DV],
                                               ig[t:t + n, h], fg[t:t + n, h], plain_states[s][h])
        t += n
    gate = pd[:, 2 * H * D + H * DV:]
    want_y = (P.rms_norm(want, None, 1e-5).reshape(T, -1) * wn.double() * P.sigmoid(gate)) * 0.5

    sd = state.clone().to(DEV)
    gates = torch.cat([zi, zf], dim=1).contiguous().to(DEV)
    seq_of_token = torch.tensor(sum(([i] * n for i, n in enumerate(lens)), []), dtype=torch.int32, device=DEV)
    slot_t = torch.tensor(slots, dtype=torch.int32, device=DEV)
    stab, qn = torch.empty(T, H, device=DEV), torch.empty(T, H, device=DEV)
    num = torch.empty(T, H * DV, device=DEV)
    xd = proj.to(DEV)
    chunk, max_chunks = kernels.linear_attention_chunks(max(lens))
    assert (max_chunks > 1) == (max(lens) >= 256)
    chunks = torch.full((3 * max_chunks * H * D * (DV + 1),), float("nan"), device=DEV) if max_chunks > 1 else None
    kernels.matrix_memory(xd, 0, H * D, 2 * H * D, D ** -0.5, gates, bi.to(DEV), bf.to(DEV), cap, seq_of_token, slot_t, sd,
                          stab, num, qn, T, 3, H, D, DV, chunks, chunk, max_chunks)
    wide = torch.full((T, H * DV + 3), float("nan"), dtype=dtype, device=DEV)
    y = wide[:, 3:]
    kernels.matrix_memory_output(num, qn, stab, xd[:, 2 * H * D + H * DV:], wn.to(DEV), y, T, H, D, DV, 1e-5,
                                 P.DENOMINATOR_FLOOR, 0.5)
    assert rel(y, want_y) < tol
    assert torch.isnan(wide[:, :3]).all()
    assert torch.equal(sd[1].cpu(), state[1]) and torch.equal(sd[4].cpu(), state[4])
    for s in slots:                      # the states left behind
        for h in range(H):
            st = plain_states[s][h]
            plane = sd[s, h * D * (DV + 1):(h + 1) * D * (DV + 1)].view(D, DV + 1)
            assert rel(plane[:, :DV], st["S"]) < 2e-5 and rel(plane[:, DV], st["n"]) < 2e-5
            assert abs(float(sd[s, H * D * (DV + 1) + h]) - st["m"]) < 1e-5 * max(1.0, abs(st["m"]))


@pytest.mark.parametrize("M,N,K", [(128, 64, 64), (300, 384, 256), (1000, 704, 512)])
def test_gated_product_with_the_tanh_gelu_on_the_tensor_cores(M, N, K):
    """The tcgen05 product whose epilogue forms gelu_tanh(gate) * up, against the plain product of the same
    bfloat16 operands (gate and up rounded to bfloat16 before the activation, as the unfused path stores them)."""
    from redline_b200.ops import kernels
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * N, K, generator=g) / math.sqrt(K) * 2).to(torch.bfloat16)
    gu = (x.double() @ w.double().T).to(torch.bfloat16).double()
    want = P.gelu_tanh(gu[:, :N]) * gu[:, N:]
    y = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    xd, wd = x.to(DEV), w.to(DEV)
    assert kernels.gemm_tc_ok(xd, wd)
    kernels.gemm_tc(xd, wd, y, kernels.EPI_GEGLU_TANH)
    assert int(kernels.tc_status(xd.device).item()) == 0
    assert rel(y, want) < 1.5e-2
    # the unfused path: product, then the activation kernel
    buf = torch.empty(M, 2 * N, dtype=torch.bfloat16, device=DEV)
    torch.mm(xd, wd.t(), out=buf)
    y2 = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
    kernels.gated_act(buf, y2, kernels.ACTIVATIONS["gelu_tanh"])
    assert rel(y2, want) < 1.5e-2
