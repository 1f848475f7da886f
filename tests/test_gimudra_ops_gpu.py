"""The mechanisms of the Gimudra design one at a time, kernels against the plain float64 oracle (oracle/gimudra_ref.py):
sinusoidal positions, the closing kernel of pre-norm layers (scaled residual add, bias, pass-through share, depth
average, next norm, token shift), the token shift over portions, attention in blocks with biases and the distance
penalty (keys planted just inside / outside a block, at page borders, far back), the shared cache, the router with
groups and the squared-ReLU experts.  Slots and caches hold garbage before use."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import gimudra_ref as R  # noqa: E402

DEV = "cuda:0"
F64 = torch.float64


def meta(entries):
    """entries [(slot, rows, first position)] -> row_ent, ent on the device."""
    row_ent, ent, at = [], [], 0
    for i, (slot, n, pos) in enumerate(entries):
        row_ent += [i] * n
        ent += [slot, at, n, pos]
        at += n
    return (torch.tensor(row_ent, dtype=torch.int32, device=DEV), torch.tensor(ent, dtype=torch.int32, device=DEV))


# ---------------------------------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("width", [48, 30, 7])
@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_embedding_with_sinusoidal_positions(width, dt):
    from dli_b200 import ops

    torch.manual_seed(0)
    table = torch.randn(50, width).to(dt)
    ids = torch.randint(0, 50, (9,))
    entries = [(2, 4, 0), (0, 1, 700), (1, 4, 1021)]      # a prompt's start, a decoded token, a portion far into a sequence
    row_ent, ent = meta(entries)
    freq = torch.tensor([10000.0 ** (-2.0 * i / width) for i in range((width + 1) // 2)], dtype=F64).float().to(DEV)
    x = torch.empty(9, width, dtype=torch.float32, device=DEV)
    x2 = torch.empty_like(x)
    ops.embedding_f32(ids.to(torch.int32).to(DEV), table.to(DEV), x, 3.5, out2=x2, row_ent=row_ent, ent=ent, inv_freq=freq)
    at = 0
    for _, n, pos in entries:
        ref = R.embed(ids[at:at + n].tolist(), table, 3.5, first_pos=pos)
        # angles are 32-bit: at position p an angle carries an error of up to p * 2^-24
        assert (x[at:at + n].double().cpu() - ref).abs().max() < 2e-6 + (pos + n) * 1.5e-7
        at += n
    assert torch.equal(x, x2)


# ---------------------------------------------------------------------------------------------------- closing kernel
def close_ref(x, y, bias, idw, h_in, ls, xs, dwa, w_next, eps):
    v = x.clone()
    if y is not None:
        t = y.clone()
        if bias is not None:
            t = t + bias
        if idw is not None:
            t = t + idw[:, None] * h_in
        v = v + (t * ls if ls is not None else t)
    stored = v.clone()
    if dwa is not None:
        v = sum(dwa[j] * xs[j] for j in range(len(xs))) + dwa[len(xs)] * stored
    h = R.rms_norm(v, w_next, eps) if w_next is not None else None
    return v, stored, h


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width", [(5, 48), (70, 40), (3, 2048)])
@pytest.mark.parametrize("opts", ["plain", "bias", "pass", "avg", "all", "norm_only"])
def test_layer_close_against_reference(dt, rows, width, opts):
    from dli_b200 import ops

    torch.manual_seed(1)
    n_prev = 3
    x = torch.randn(rows, width)
    y = None if opts == "norm_only" else torch.randn(rows, width).to(dt)
    bias = torch.randn(width) if opts in ("bias", "all") else None
    idw = torch.rand(rows) if opts in ("pass", "all") else None
    h_in = torch.randn(rows, width) if idw is not None else None
    ls = None if opts in ("plain", "norm_only") else torch.rand(width) + 0.2
    dwa = torch.randn(n_prev + 1) if opts in ("avg", "all") else None
    w_next = torch.rand(width) + 0.5
    xs_host = torch.randn(n_prev, rows + 6, width)           # row capacity above the step's rows
    xs = torch.cat((xs_host, torch.full((2, rows + 6, width), 1e4))).to(DEV)
    g = lambda t: None if t is None else t.to(DEV)  # noqa: E731
    xd = x.clone().to(DEV)
    out_f = torch.empty(rows, width, dtype=torch.float32, device=DEV)
    out_e = torch.empty(rows, width, dtype=dt, device=DEV)
    ops.layer_close(xd, g(y), bias=g(bias), idw=g(idw), h_in=g(h_in), ls=g(ls), xs=xs if dwa is not None else None,
                    n_prev=n_prev, dwa=g(dwa), w_next=g(w_next), out_f=out_f, out_e=out_e, eps=1e-5)
    d = lambda t: None if t is None else t.double()  # noqa: E731
    v, stored, h = close_ref(x.double(), d(y), d(bias), d(idw), d(h_in), d(ls), [xs_host[j, :rows].double() for j in range(n_prev)],
                             d(dwa), w_next.double(), 1e-5)
    assert (xd.double().cpu() - v).abs().max() < 1e-5 * max(1.0, float(v.abs().max()))
    assert (out_f.double().cpu() - h).abs().max() < 2e-5 * max(1.0, float(h.abs().max()))
    assert (out_e.double().cpu() - h).abs().max() < (2e-5 if dt == torch.float32 else 0.02) * max(1.0, float(h.abs().max()))
    if dwa is not None:
        assert (xs[n_prev, :rows].double().cpu() - stored).abs().max() < 1e-5 * max(1.0, float(stored.abs().max()))
        assert torch.equal(xs[:n_prev, :rows].cpu(), xs_host[:, :rows])      # the earlier results are only read


def test_layer_close_with_the_shift_of_single_rows_and_the_ragged_shift_agree_with_the_oracle():
    """A sequence of 23 positions in slot 2 (garbage in every slot before): normed rows shifted (a) token by token by
    the closing kernel, (b) in portions of 7, 2, 1, 13 by the ragged kernel; a second sequence shares the steps."""
    from dli_b200 import ops

    torch.manual_seed(2)
    width, T, eps = 40, 23, 1e-5
    xa, xb = torch.randn(T, width), torch.randn(T, width)
    w, s = torch.rand(width) + 0.5, torch.rand(width)
    refs = [R.token_shift(R.rms_norm(t.double(), w.double(), eps), s.double()) for t in (xa, xb)]
    wd, sd = w.to(DEV), s.to(DEV)
    # (a) one row per entry and step
    tail = torch.full((4, width), 1e4, device=DEV)
    got = [torch.empty(T, width), torch.empty(T, width)]
    for t in range(T):
        _, ent = meta([(2, 1, t), (0, 1, t)])
        x = torch.stack((xa[t], xb[t])).to(DEV)
        out = torch.empty(2, width, device=DEV)
        ops.layer_close(x, w_next=wd, shift=sd, tail=tail, ent=ent, out_e=out, eps=eps)
        got[0][t], got[1][t] = out[0].cpu(), out[1].cpu()
    for k in range(2):
        assert (got[k].double() - refs[k]).abs().max() < 1e-5
    # (b) portions; the second sequence is cut differently and joins later
    tail = torch.full((4, width), 1e4, device=DEV)
    got = [[], []]
    plan = [[(2, 7)], [(2, 2), (0, 5)], [(2, 1), (0, 1)], [(0, 17)], [(2, 13)]]
    at = {2: 0, 0: 0}
    src = {2: xa, 0: xb}
    for step in plan:
        row_ent, ent = meta([(slot, n, at[slot]) for slot, n in step])
        x = torch.cat([src[slot][at[slot]:at[slot] + n] for slot, n in step]).to(DEV)
        hs = torch.empty_like(x)
        ops.layer_close(x, w_next=wd, out_f=hs, eps=eps)
        out = torch.empty_like(x)
        ops.token_shift_ragged(hs, sd, tail, row_ent, ent, out)
        o = 0
        for slot, n in step:
            got[0 if slot == 2 else 1].append(out[o:o + n].cpu())
            o += n
            at[slot] += n
    for k in range(2):
        assert (torch.cat(got[k]).double() - refs[k]).abs().max() < 1e-5


def test_silu_mul_with_biases():
    """Sizes that take the 2-byte and the 16-byte accesses, a row stride above 2F."""
    from dli_b200 import ops

    torch.manual_seed(3)
    for F, ld in ((20, 44), (24, 56), (512, 1024)):
        for dt, tol in ((torch.float32, 1e-5), (torch.bfloat16, 0.03)):
            gu = torch.randn(6, ld).to(dt)
            b = torch.randn(2 * F)
            out = torch.empty(6, F, dtype=dt, device=DEV)
            ops.silu_mul(gu.to(DEV), out, bias=b.to(DEV))
            g, u = gu[:, :F].double() + b[:F].double(), gu[:, F:2 * F].double() + b[F:].double()
            assert (out.double().cpu() - R.silu(g) * u).abs().max() < tol * max(1.0, float((R.silu(g) * u).abs().max()))
            ops.silu_mul(gu.to(DEV), out)
            ref = R.silu(gu[:, :F].double()) * gu[:, F:2 * F].double()
            assert (out.double().cpu() - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


# ---------------------------------------------------------------------------------------------------- attention
def run_attn(q, k, v, m, r1, r2, bias, cuts, page_size, dt=torch.float32, tc=False, q_only_from=None):
    """The kernels on one sequence cut into portions `cuts`, pages handed out in a scrambled order, caches holding
    garbage.  q / k / v are the projection's outputs WITHOUT the biases.  q_only_from = (kc, vc, pt): a second layer that
    only makes queries and reads those caches.  Returns (out, (kc, vc, pt))."""
    from dli_b200 import ops

    T = q.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = (q if q_only_from else torch.cat((q, k, v), dim=1)).to(dt).to(DEV).contiguous()
    n_pages = (T + page_size - 1) // page_size
    if q_only_from:
        kc, vc, pt = q_only_from
    else:
        perm = torch.randperm(n_pages + 3, generator=torch.Generator().manual_seed(3))[:n_pages].to(torch.int32)
        pt = torch.zeros(2, n_pages, dtype=torch.int32)
        pt[1] = perm
        pt = pt.to(DEV)
        kc = torch.full((n_pages + 3, G, page_size, D), 7.0, dtype=dt, device=DEV)
        vc = torch.full((n_pages + 3, G, page_size, V), -5.0, dtype=dt, device=DEV)
    out = torch.empty(T, H * V, dtype=dt, device=DEV)
    bd = None if bias is None else bias.float().to(DEV)
    at = 0
    for n in cuts:
        n = min(n, T - at)
        if n <= 0:
            break
        row_ent, ent = meta([(1, n, at)])
        qbuf = torch.empty(n, H * D, dtype=torch.float32, device=DEV)
        pr = proj[at:at + n].contiguous()
        ops.attn_prep_append(pr, qbuf, kc, vc, row_ent, ent, pt, H, G, D, V, 0, 0, H * D, H * D + G * D, None, None, 0.0,
                             None, None, None, None, bias=bd, q_only=q_only_from is not None)
        o = torch.empty(n, H * V, dtype=dt, device=DEV)
        kw = dict(chunk=m["mask"]["size"], r1=r1.float().to(DEV), r2=r2.float().to(DEV))
        if tc and n >= 16:
            tiles = torch.tensor([[0, q0] for q0 in range(0, n, 64)], dtype=torch.int32, device=DEV)
            ops.attn_ragged_tc(qbuf, kc, vc, None, o, ent, tiles, pt, H, G, D, V, m["scale"], **kw)
        elif n <= 2:
            part = torch.empty(n * H * 3 * (V + 2), dtype=torch.float32, device=DEV)
            ops.attn_ragged(qbuf, kc, vc, None, o, row_ent, ent, pt, H, G, D, V, m["scale"], splits=3, part=part, **kw)
        else:
            ops.attn_ragged(qbuf, kc, vc, None, o, row_ent, ent, pt, H, G, D, V, m["scale"], **kw)
        out[at:at + n] = o
        at += n
    assert at == T
    return out, (kc, vc, pt)


def attn_oracle(q, k, v, m, r1, r2, bias):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = q.shape[0]
    b = torch.zeros(H * D + G * D + G * V, dtype=F64) if bias is None else bias.double()
    qq = (q.double() + b[:H * D]).reshape(T, H, D)
    kk = (k.double() + b[H * D:H * D + G * D]).reshape(T, G, D)
    vv = (v.double() + b[H * D + G * D:]).reshape(T, G, V)
    return R.attention_scores_softmax(qq, kk, vv, m["scale"], m["mask"]["size"], r1, r2).reshape(T, H * V)


@pytest.mark.parametrize("cuts", [[200], [1] * 200, [37, 2, 2, 50, 1, 1, 1, 3, 64, 64], [150] + [1] * 50])
@pytest.mark.parametrize("size", [48, 0, 1])
def test_attention_random_inputs(cuts, size):
    torch.manual_seed(2)
    m = {"heads": 6, "kv_heads": 2, "dim": 12, "vdim": 20, "scale": 0.4, "mask": {"size": size}}
    T = 140
    q, k, v = torch.randn(T, 6 * 12), torch.randn(T, 2 * 12), torch.randn(T, 2 * 20)
    r1, r2 = torch.rand(6) * 2, torch.rand(6) * 0.5 + 0.05
    r1[0] = 0.0
    bias = torch.randn(6 * 12 + 2 * 12 + 2 * 20) * 0.5
    ref = attn_oracle(q, k, v, m, r1, r2, bias)
    got, _ = run_attn(q, k, v, m, r1, r2, bias, cuts, page_size=8)
    assert (got.double().cpu() - ref).abs().max() < 2e-4
    nobias, _ = run_attn(q, k, v, m, r1, r2, None, cuts, page_size=8)
    assert (nobias.double().cpu() - attn_oracle(q, k, v, m, r1, r2, None)).abs().max() < 2e-4


@pytest.mark.parametrize("cuts", [[300], [130, 2] + [1] * 170, [249, 2, 9]])
@pytest.mark.parametrize("target", ["first_in_block", "last_of_previous_block", "page_border", "second_in_block", "itself"])
def test_attention_one_key_stands_out(cuts, target):
    """The query at position i scores high with ONE key j and 0 with every other: inside the block the head's output
    is v_j; one position outside it, v_j must not appear at all (the weight spreads evenly over the block)."""
    torch.manual_seed(4)
    block, page = 100, 16                      # block edges that are neither page nor tile borders
    m = {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 4.0, "mask": {"size": block}}
    T, i = 260, 250                            # block of i: positions 200..299
    j = {"first_in_block": 200, "last_of_previous_block": 199, "page_border": 208, "second_in_block": 201, "itself": 250}[target]
    q, k, v = torch.randn(T, 16), torch.randn(T, 8), torch.randn(T, 8)
    k[:, 3] = 0
    q[i, :8] = 0
    q[i, 3] = 6.0
    k[j] = 0
    k[j, 3] = 6.0                              # score 36 * 4 with key j, exactly 0 with the others
    zero = torch.zeros(2)
    ref = attn_oracle(q, k, v, m, zero, zero, None)
    got, _ = run_attn(q, k, v, m, zero, zero, None, cuts, page_size=page)
    assert (got.double().cpu() - ref).abs().max() < 2e-4
    inside = j >= 200
    assert bool((ref[i, :8] - v[j].double()).abs().max() < 1e-6) == inside
    if not inside:
        assert (ref[i, :8] - v[200:251].double().mean(0)).abs().max() < 1e-9


def test_attention_distance_penalty_decides():
    """Equal scores everywhere; head 0 has no penalty (even weights over the block), head 1 a penalty so steep that the
    query's own position takes the weight, head 2 a mild one whose weights are (1 + r2 d)^-r1 — a penalty left out, applied
    to the wrong head, or measured from the portion's start instead of the sequence's shows in each."""
    m = {"heads": 3, "kv_heads": 1, "dim": 4, "vdim": 6, "scale": 1.0, "mask": {"size": 0}}
    T = 90
    torch.manual_seed(5)
    q, k, v = torch.zeros(T, 12), torch.zeros(T, 4), torch.randn(T, 6)
    r1, r2 = torch.tensor([0.0, 40.0, 1.5]), torch.tensor([0.3, 2.0, 0.25])
    ref = attn_oracle(q, k, v, m, r1, r2, None)
    for cuts in ([90], [50, 3, 30, 2] + [1] * 5):
        got, _ = run_attn(q, k, v, m, r1, r2, None, cuts, page_size=4)
        assert (got.double().cpu() - ref).abs().max() < 2e-5
    i = 80
    assert (ref[i, :6] - v[:i + 1].double().mean(0)).abs().max() < 1e-9
    assert (ref[i, 6:12] - v[i].double()).abs().max() < 1e-9
    wts = (1.0 + 0.25 * torch.arange(i, -1, -1, dtype=F64)) ** -1.5
    assert (ref[i, 12:] - (wts[:, None] * v[:i + 1].double()).sum(0) / wts.sum()).abs().max() < 1e-9


def test_attention_far_key_among_hundreds():
    """No blocks: position 600 finds key 3 among 600 others, through a penalty that grows with the distance."""
    torch.manual_seed(6)
    m = {"heads": 2, "kv_heads": 2, "dim": 8, "vdim": 4, "scale": 1.0, "mask": {"size": 0}}
    T, i, j = 610, 600, 3
    q, k, v = torch.randn(T, 16) * 0.1, torch.randn(T, 16) * 0.1, torch.randn(T, 8)
    q[i, 8:] = 0
    q[i, 9] = 8.0
    k[:, 9] = 0
    k[j, 9] = 8.0
    r1, r2 = torch.tensor([0.5, 1.0]), torch.tensor([0.2, 0.1])
    ref = attn_oracle(q, k, v, m, r1, r2, None)
    assert (ref[i, 4:] - v[j, 4:].double()).abs().max() < 1e-6
    for cuts in ([610], [590, 7] + [1] * 13):
        got, _ = run_attn(q, k, v, m, r1, r2, None, cuts, page_size=16)
        assert (got.double().cpu() - ref).abs().max() < 2e-4


def test_a_second_layer_reads_the_first_layers_cache():
    """The reading layer has its own queries (and query biases), distance penalty and block size; it appends nothing."""
    torch.manual_seed(7)
    m1 = {"heads": 4, "kv_heads": 2, "dim": 8, "vdim": 6, "scale": 0.5, "mask": {"size": 32}}
    m2 = dict(m1, scale=0.3, mask={"size": 20})
    T = 75
    q1, k, v, q2 = torch.randn(T, 32), torch.randn(T, 16), torch.randn(T, 12), torch.randn(T, 32)
    b1 = torch.randn(32 + 16 + 12)
    b2 = torch.randn(32)
    r1a, r2a, r1b, r2b = torch.rand(4), torch.rand(4), torch.rand(4) * 2, torch.rand(4)
    for cuts in ([75], [20, 2, 1, 1, 30, 21]):
        _, caches = run_attn(q1, k, v, m1, r1a, r2a, b1, cuts, page_size=8)
        before = [t.clone() for t in caches[:2]]
        got, _ = run_attn(q2, None, None, m2, r1b, r2b, b2, cuts, page_size=8, q_only_from=caches)
        assert torch.equal(before[0], caches[0]) and torch.equal(before[1], caches[1])
        full_b = torch.cat((b2, b1[32:]))
        ref = attn_oracle(q2, k, v, m2, r1b, r2b, full_b)
        assert (got.double().cpu() - ref).abs().max() < 2e-4


@pytest.mark.parametrize("dims", [(64, 64), (128, 128), (64, 128)])
@pytest.mark.parametrize("cuts", [[230], [100, 3, 64, 63], [17, 1, 130, 2, 80]])
def test_attention_tensor_core_tiles_with_the_penalty(dims, cuts):
    """The tensor-core kernel on portions that start anywhere (single rows beside them): block edges that are no multiple
    of the tile, pages smaller than the tile, grouped heads, biases, the penalty in the base-2 exponent; bf16 operands."""
    D, V = dims
    torch.manual_seed(8)
    m = {"heads": 4, "kv_heads": 2, "dim": D, "vdim": V, "scale": D ** -0.5, "mask": {"size": 75}}
    T = 230
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    q, k, v = bf(torch.randn(T, 4 * D)), bf(torch.randn(T, 2 * D)), bf(torch.randn(T, 2 * V))
    r1, r2 = torch.tensor([0.0, 1.8, 0.7, 30.0]), torch.tensor([0.1, 0.45, 0.08, 1.0])
    ref = attn_oracle(q, k, v, m, r1, r2, None)
    got, _ = run_attn(q, k, v, m, r1, r2, None, cuts, page_size=16, dt=torch.bfloat16, tc=True)
    plain, _ = run_attn(q, k, v, m, r1, r2, None, cuts, page_size=16, dt=torch.bfloat16, tc=False)
    assert (got.double().cpu() - ref).abs().max() < 0.03
    assert (plain.double().cpu() - ref).abs().max() < 0.03


# ---------------------------------------------------------------------------------------------------- mixture of experts
def route_kernel(h, w, c, n_real, top, groups, keep, scale):
    from dli_b200 import ops

    rows = h.shape[0]
    wts = torch.full((rows, max(n_real, 1)), 9.0, device=DEV)
    idw = torch.full((rows,), 9.0, device=DEV)
    si = torch.zeros(rows, top, dtype=torch.int32, device=DEV)
    sw = torch.zeros(rows, top, device=DEV)
    ops.moe_route(h.float().to(DEV), w.float().to(DEV), c.float().to(DEV), wts, idw, si, sw, n_real, top, groups=groups,
                  keep=keep, wscale=scale, renorm=False)
    return wts.cpu(), idw.cpu(), si.cpu(), sw.cpu()


@pytest.mark.parametrize("shape", [(10, 2, 3, 4, 2, 2.5), (6, 2, 2, 4, 3, 0.5), (5, 0, 5, 1, 1, 1.0), (4, 4, 2, 2, 1, 1.0),
                                   (9, 0, 3, 3, 3, 3.0)])
def test_router_with_groups_against_oracle(shape):
    """(experts, pass-through outputs, top, groups, kept groups, scale): negative choice scores throughout (a group set
    to 0 instead of minus infinity would win), a correction that changes the choice but not the weights."""
    E, I, top, count, keep, scale = shape
    torch.manual_seed(9)
    rows, d = 40, 24
    h, w = torch.randn(rows, d), torch.randn(E + I, d) * 0.6
    c = -1.0 - torch.rand(E + I) * 2
    r = {"experts": E, "identity": I, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}
    idx, wt = R.route(h.double(), w.double(), c.double(), r)
    wts, idw, si, sw = route_kernel(h, w, c, E, top, count, keep, scale)
    for t in range(rows):
        assert sorted(si[t].tolist()) == sorted(idx[t].tolist()), f"row {t}"
        ref_dense = torch.zeros(E + I, dtype=F64)
        ref_dense[idx[t]] = wt[t]
        if E:
            assert (wts[t, :E].double() - ref_dense[:E]).abs().max() < 1e-6
        assert abs(float(idw[t]) - float(ref_dense[E:].sum())) < 1e-6
    # the choice differs from the one without correction or groups for some rows (the test would not see them otherwise)
    plain, _ = R.route(h.double(), w.double(), torch.zeros(E + I, dtype=F64), dict(r, groups={"count": 1, "keep": 1}))
    if count > 1 and keep < count:
        assert any(sorted(plain[t].tolist()) != sorted(idx[t].tolist()) for t in range(rows))


@pytest.mark.parametrize("rows,d", [(3, 24), (70, 40), (5, 2048)])
def test_router_inside_the_closing_kernel_equals_the_router_alone(rows, d):
    """The closing kernel norms a row and routes it at once; choice and weights are those of the router kernel on the
    normed rows it wrote, bit for bit, and the rows themselves are those of the kernel without the router."""
    from dli_b200 import ops

    torch.manual_seed(10)
    E, I, top, count, keep, scale = 6, 2, 3, 4, 2, 1.7
    x, y = torch.randn(rows, d, device=DEV), torch.randn(rows, d, device=DEV).to(torch.bfloat16)
    ls, wn = torch.rand(d, device=DEV) + 0.2, torch.rand(d, device=DEV) + 0.5
    w, c = (torch.randn(E + I, d) * 0.6).to(DEV), (-1.0 - torch.rand(E + I)).to(DEV)

    def buffers():
        return (torch.full((rows, E), 9.0, device=DEV), torch.full((rows,), 9.0, device=DEV),
                torch.zeros(rows, top, dtype=torch.int32, device=DEV), torch.zeros(rows, top, device=DEV))

    kw = dict(n_real=E, top=top, groups=count, keep=keep, wscale=scale, renorm=False)
    wts, idw, si, sw = buffers()
    hn, he = torch.empty(rows, d, device=DEV), torch.empty(rows, d, dtype=torch.bfloat16, device=DEV)
    xc = x.clone()
    ops.layer_close(xc, y, ls=ls, w_next=wn, out_f=hn, out_e=he, eps=1e-5,
                    route=dict(w_router=w, correction=c, wts=wts, idw=idw, sel_idx=si, sel_w=sw, **kw))
    wts2, idw2, si2, sw2 = buffers()
    ops.moe_route(hn, w, c, wts2, idw2, si2, sw2, E, top, groups=count, keep=keep, wscale=scale, renorm=False)
    for a_, b_ in ((wts, wts2), (idw, idw2), (si, si2), (sw, sw2)):
        assert torch.equal(a_, b_)
    hn2, he2, xc2 = torch.empty_like(hn), torch.empty_like(he), x.clone()
    ops.layer_close(xc2, y, ls=ls, w_next=wn, out_f=hn2, out_e=he2, eps=1e-5)
    assert torch.equal(xc, xc2) and (hn - hn2).abs().max() < 1e-5 and (he.float() - he2.float()).abs().max() < 0.05
    idx, wt = R.route(hn.double().cpu(), w.double().cpu(), c.double().cpu(),
                      {"experts": E, "identity": I, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}})
    assert all(sorted(si[t].tolist()) == sorted(idx[t].tolist()) for t in range(rows))


def moe_tensors(E, I, ff, d, seed):
    g = torch.Generator().manual_seed(seed)
    bf = lambda t: t.to(torch.bfloat16).float()  # noqa: E731
    sd = {"router": bf(torch.randn(E + I, d, generator=g) * 0.6), "correction": bf(-1.0 - torch.rand(E + I, generator=g))}
    for e in range(E):
        sd[f"e{e}.up"] = bf(torch.randn(ff, d, generator=g) * 0.3)
        sd[f"e{e}.down"] = bf(torch.randn(d, ff, generator=g) * 0.3)
    return sd


@pytest.mark.parametrize("dt,tol", [(torch.float32, 2e-5), (torch.bfloat16, 0.03)])
@pytest.mark.parametrize("shape", [(6, 2, 2, 4, 2, 12, 1.5), (3, 0, 3, 1, 1, 8, 1.0), (4, 1, 1, 5, 5, 16, 2.0)])
def test_experts_all_at_once_against_oracle(dt, tol, shape):
    """Router + ONE up projection over all experts + squared ReLU times the routing weight + ONE down projection, and the
    pass-through share, against the oracle's per-token loop."""
    from dli_b200 import ops

    E, I, top, count, keep, ff, scale = shape
    d, rows = 32, 21
    sd = moe_tensors(E, I, ff, d, 11)
    torch.manual_seed(12)
    h = torch.randn(rows, d).to(torch.bfloat16).float()
    mlp = {"router": {"experts": E, "identity": I, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    ref = R.moe_ff(h.double(), {k: v for k, v in sd.items()}, "", mlp)
    wts, idw, si, sw = route_kernel(h, sd["router"], sd["correction"], E, top, count, keep, scale)
    w_up = torch.cat([sd[f"e{e}.up"] for e in range(E)]).to(dt).to(DEV)
    w_down = torch.cat([sd[f"e{e}.down"] for e in range(E)], dim=1).to(dt).to(DEV).contiguous()
    gu = torch.empty(rows, E * ff, dtype=dt, device=DEV)
    ops.linear_any(h.to(dt).to(DEV), w_up, gu)
    act = torch.empty(rows, E * ff, dtype=dt, device=DEV)
    ops.moe_act(gu, wts.to(DEV), act, E, ff, 0.0, gated=False)
    y = torch.empty(rows, d, dtype=dt, device=DEV)
    ops.linear_any(act, w_down, y)
    got = y.double().cpu() + idw.double()[:, None] * h.double()
    assert (got - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))


def test_chosen_experts_only_equal_all_experts():
    """Few rows in bf16: the kernels that stream only the chosen experts' weights against the oracle."""
    from dli_b200 import ops

    E, I, top, count, keep, ff, scale = 8, 2, 2, 5, 2, 24, 1.5
    d, rows = 64, 5
    sd = moe_tensors(E, I, ff, d, 13)
    torch.manual_seed(14)
    h = torch.randn(rows, d).to(torch.bfloat16).float()
    mlp = {"router": {"experts": E, "identity": I, "top": top, "scale": scale, "groups": {"count": count, "keep": keep}}}
    ref = R.moe_ff(h.double(), sd, "", mlp)
    wts, idw, si, sw = route_kernel(h, sd["router"], sd["correction"], E, top, count, keep, scale)
    assert ops.moe_sel_supported(d, ff, 0, top)
    w_up = torch.cat([sd[f"e{e}.up"] for e in range(E)]).to(torch.bfloat16).to(DEV)
    w_down = torch.cat([sd[f"e{e}.down"] for e in range(E)], dim=1).to(torch.bfloat16).to(DEV).contiguous()
    act = torch.empty(rows, top * ff, dtype=torch.bfloat16, device=DEV)
    y = torch.empty(rows, d, dtype=torch.bfloat16, device=DEV)
    ops.moe_sel(h.to(torch.bfloat16).to(DEV), w_up, w_down, si.to(DEV), sw.to(DEV), act, y, E, top, ff, 0.0, gated=False)
    got = y.double().cpu() + idw.double()[:, None] * h.double()
    assert (got - ref).abs().max() < 0.03 * max(1.0, float(ref.abs().max()))
