"""Each mechanism of the Fubepel design alone, kernels against the oracle's function for it (oracle/fubepel_ref.py), on
inputs made so that a fault shows: queries that equal ONE key just inside or just outside the window, among the kept
first positions or right after them, far back or at a page border, under a softmax sharp enough that this key takes
nearly all the weight; a sink that swallows one head's softmax; a second layer reading the first layer's cache; a delta
rule that forgets slowly, so that a lost state shows hundreds of tokens later; slots holding garbage."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import fubepel_ref as R  # noqa: E402
from test_fubepel_engine_gpu import attention, config, delta, dense, latent  # noqa: E402

DEV = "cuda:0"
F64 = torch.float64


def engine_of(layers, width=32, page_size=4, max_seq_len=512, seed=0, std=0.3, side=0, dtype=torch.float32):
    from dli_b200 import fubepel
    from dli_b200.ragged_engine import RaggedEngine

    cfg = config(layers, width=width, side=side)
    spec = fubepel.spec_from_config(cfg)
    sd = {k: v.float() for k, v in fubepel.random_state_dict(spec, seed=seed, std=std).items()}
    eng = RaggedEngine(spec, max_batch=4, max_seq_len=max_seq_len, page_size=page_size, dtype=dtype)
    eng.load_tensors(fubepel.model_tensors(spec, sd))
    for t in eng.slots.tensors.values():
        t.fill_(1e4)                          # whatever the slots held before
    return eng, cfg, sd


def views_of(entries):
    """entries [(slot, n, start)] -> the device views a step hands to the mixers, with its 64-row tiles."""
    row_ent, ent, tiles, r = [], [], [], 0
    for i, (slot, n, start) in enumerate(entries):
        ent += [slot, r, n, start]
        row_ent += [i] * n
        tiles += [[i, q0] for q0 in range(0, n, 64)]
        r += n
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    return (z, torch.tensor(row_ent, dtype=torch.int32, device=DEV), torch.tensor(ent, dtype=torch.int32, device=DEV), z,
            torch.tensor(tiles, dtype=torch.int32, device=DEV))


def run_mixers(eng, us, cuts, tiles=False, delta_blocked=False):
    """us: per layer the mixer's input projection [T, columns] (made on the host), fed through the engine's mixer kernels
    in portions of the given sizes (then token by token) -> per layer the mixer's output before its out-projection."""
    T = us[0].shape[0]
    eng.open_sequence()                       # take a slot that is not the first one
    slot = eng.open_sequence()
    outs, at, sizes = [[] for _ in us], 0, list(cuts)
    while at < T:
        n = min(sizes.pop(0) if sizes else 1, T - at)
        eng._workspace(n)
        if eng.attn_layers:
            eng.kv.reserve(slot, at + n)
            eng.kv.commit()
            eng._step_pages = (min(eng.kv.owned[slot]), max(eng.kv.owned[slot]))
        views = views_of([(slot, n, at)])
        for li, u in enumerate(us):
            m, P = eng.spec.layers[li].mixer, eng.layers[li]
            proj = torch.zeros(n, P["w_proj"].shape[0], device=DEV, dtype=eng.dtype)
            proj[:, :u.shape[1]] = u[at:at + n].to(DEV).to(eng.dtype)
            mix = torch.empty(n, m.heads * m.vdim, device=DEV, dtype=eng.dtype)
            if m.kind == "attention":
                eng._attention(li, m, P, proj, mix, n, views, tiles and n >= 16)
            elif m.kind == "latent_attention":
                eng._latent_attention(li, m, P, proj, mix, n, views, tiles and n >= 16)
            else:
                eng._delta(li, m, P, proj, mix, n, views, long_step=delta_blocked and n >= 2)   # 16 rows at a time
            outs[li].append(mix.double().cpu())
        at += n
    return [torch.cat(o) for o in outs]


def planted(T, dim, targets, seed):
    """Unit directions k_j and queries q_t = k_(targets(t)) (a random direction where the target is None)."""
    g = torch.Generator().manual_seed(seed)
    k = torch.randn(T, dim, generator=g, dtype=F64)
    k = k / k.norm(dim=-1, keepdim=True)
    q = torch.randn(T, dim, generator=g, dtype=F64)
    for t in range(T):
        j = targets(t)
        if j is not None and 0 <= j <= t:
            q[t] = k[j]
    return q, k


@pytest.mark.parametrize("cuts", [[170], [3, 2, 61, 70], [40], []])
def test_window_edges_and_kept_first_positions_with_sharp_scores(cuts):
    """Window of 23, 5 kept first positions, pages of 4.  Query t equals the key just inside the window, just outside
    it, the last kept position, the one after it, itself, or one far back, in turn; scale 8 on normed vectors of 8
    entries makes that key's weight ~1 when it is visible."""
    size, keep, H, D, V = 23, 5, 2, 8, 6
    eng, cfg, sd = engine_of([(attention(heads=H, kv_heads=1, dim=D, vdim=V, scale=8.0, size=size, keep_first=keep), None)])
    T = 170
    cases = [lambda t: t - size + 1, lambda t: t - size, lambda t: keep - 1, lambda t: keep, lambda t: t,
             lambda t: max(keep + 1, t - 100), lambda t: (t // 4) * 4 - 1]
    qs, ks = zip(*[planted(T, D, lambda t, h=h: cases[(t + 3 * h) % len(cases)](t), 5 + h) for h in range(H)])
    g = torch.Generator().manual_seed(9)
    v = torch.randn(T, V, generator=g, dtype=F64)
    k = ks[0]
    for h in range(H):                        # both heads share the one key head: plant against ITS keys
        for t in range(T):
            j = cases[(t + 3 * h) % len(cases)](t)
            if j is not None and 0 <= j <= t:
                qs[h][t] = k[j]
    u = torch.cat([q * 3.0 for q in qs] + [k * 0.2, v], dim=1)   # the head norms remove the lengths
    got = run_mixers(eng, [u], cuts)[0].reshape(T, H, V)
    vis = R.visible(T, size, keep)
    kn = R.rms_norm(k * 0.2, None, 1e-5)
    for h in range(H):
        want = R.softmax_attend((R.rms_norm(qs[h] * 3.0, None, 1e-5) @ kn.T) * 8.0, v, vis)
        assert (got[:, h] - want).abs().max() < 2e-4, f"head {h}"
    # the planted keys matter: with the window one position longer the answer is another one
    other = R.softmax_attend((R.rms_norm(qs[0] * 3.0, None, 1e-5) @ kn.T) * 8.0, v, R.visible(T, size + 1, keep))
    assert (other - got[:, 0]).abs().max() > 0.1


@pytest.mark.parametrize("cuts,tiles", [([130], False), ([3, 2, 61], False), ([], False)])
def test_latent_attention_sharp_scores_sink_and_another_layers_cache(cuts, tiles):
    """Scale 6: nearly every query picks one key among up to 130 (pages of 4); head 0's sink (1000) is so large that it takes
    the whole softmax, head 1's so small that it does nothing; layer 1 has no cache of its own and reads layer 0's."""
    L0 = latent(heads=2, dim=6, rot_dim=8, vdim=10, kv_rank=16, scale=6.0, base=50.0)
    L1 = latent(heads=3, dim=4, rot_dim=8, vdim=6, kv_rank=16, scale=3.0, base=50.0, kv_from=0)
    eng, cfg, sd = engine_of([(L0, None), (L1, None)])
    eng.layers[0]["sink"].copy_(torch.tensor([1e3, -1e3]))
    sd["l0.mix.sink"] = torch.tensor([1e3, -1e3])
    T = 130
    torch.manual_seed(1)
    h = torch.randn(T, 32, dtype=F64)
    P0, P1 = R._sub(sd, "l0.mix."), R._sub(sd, "l1.mix.")
    u0 = torch.cat((h @ P0["q"].T, h @ P0["dkv"].T), 1)
    u1 = h @ P1["q"].T
    eye = lambda n: torch.eye(n, dtype=F64)
    P0["o"], P1["o"] = eye(20), eye(18)
    m0, m1 = cfg["layers"][0]["mixer"], cfg["layers"][1]["mixer"]
    want0 = R.latent_attention(h, P0, m0, 1e-5)
    want1 = R.latent_attention(h, P1, m1, 1e-5, cached=R.latent_kv(h, P0, m0, 1e-5))
    got0, got1 = run_mixers(eng, [u0, u1], cuts, tiles)
    assert (got0 - want0).abs().max() < 2e-4 and (got1 - want1).abs().max() < 2e-4
    assert want0[:, :10].abs().max() < 1e-6 < want0[:, 10:].abs().max()     # the sink swallowed head 0


@pytest.mark.parametrize("blocked", [False, True])
@pytest.mark.parametrize("cuts", [[260], [1, 1, 2, 3], [64, 17, 2, 100], []])
@pytest.mark.parametrize("shape", [(4, 2, 8, 6, 3), (2, 2, 40, 3, 1), (3, 1, 5, 33, 4), (1, 1, 168, 5, 2)])
def test_delta_rule_that_forgets_slowly(cuts, shape, blocked):
    """Decay ~0.999 per token: what the first tokens wrote is still in the read-out 260 tokens later, so a state that
    is lost or started from a slot's old content shows; value heads sharing query/key heads; a key size that leaves
    lanes empty; more value columns than one CTA takes; a key size beyond what a pass prefetches; row by row and 16 rows at a time (portions that end inside a block
    of 16, blocks of one and two rows)."""
    H, G, D, V, conv = shape
    eng, cfg, sd = engine_of([(delta(heads=H, kv_heads=G, dim=D, vdim=V, conv=conv), None)], std=0.4)
    eng.layers[0]["a_log"].fill_(-6.0)
    sd["l0.mix.A_log"] = torch.full((H,), -6.0)
    T = 260 if cuts != [] else 90
    torch.manual_seed(2)
    h = torch.randn(T, 32, dtype=F64)
    P = R._sub(sd, "l0.mix.")
    u = torch.cat([h @ P[k].T for k in ("q", "k", "v", "g", "b", "a")], 1)
    P["o"] = torch.eye(H * V, dtype=F64)
    want = R.gated_delta(h, P, cfg["layers"][0]["mixer"], 1e-5)
    got = run_mixers(eng, [u], cuts, delta_blocked=blocked)[0]
    assert (got - want).abs().max() < 3e-4 * max(1.0, want.abs().max())
    # forgetting really is slow here: cutting the history changes the last outputs
    short = R.gated_delta(h[T // 2:], P, cfg["layers"][0]["mixer"], 1e-5)
    assert (short[-1] - want[-1]).abs().max() > 1e-3


def test_delta_rule_one_token_against_the_equations():
    """One step of the rule by hand: S = k u^T with u = beta v on an empty state, read out by q."""
    q = torch.tensor([[1.0, 0.0, 0.0]], dtype=F64)
    k = torch.tensor([[0.6, 0.8, 0.0]], dtype=F64)
    v = torch.tensor([[2.0, -1.0]], dtype=F64)
    o = R.delta_rule(q, k, v, torch.tensor([0.5], dtype=F64), torch.tensor([0.9], dtype=F64))
    assert torch.allclose(o, torch.tensor([[0.6, -0.3]], dtype=F64))
    # a second token with the same key and beta 1 replaces what the first one wrote (the delta rule)
    o2 = R.delta_rule(q.repeat(2, 1), k.repeat(2, 1), torch.stack((v[0], -v[0])), torch.ones(2, dtype=F64),
                      torch.ones(2, dtype=F64))
    assert torch.allclose(o2[1], -0.6 * v[0])


def test_output_norm_with_weight_vector_and_token_input():
    from dli_b200 import ops

    torch.manual_seed(0)
    rows, W, n, vocab = 9, 40, 6, 11
    x = torch.randn(rows, W, device=DEV) * 3
    y = torch.randn(rows, W, device=DEV) * torch.linspace(0.01, 20, W, device=DEV)
    w = torch.randn(W, device=DEV)
    he = torch.empty(rows, W, dtype=torch.bfloat16, device=DEV)
    want = x.double().cpu() + R.rms_norm(y.double().cpu(), w.double().cpu(), 1e-5)
    got = ops.postnorm_vec_add(y, x.clone(), w, 1e-5)
    assert torch.allclose(got.double().cpu(), want, atol=1e-5, rtol=1e-5)
    xb = x.clone()
    ops.postnorm_vec_add(y.bfloat16(), xb, w, 1e-5, he=he)
    assert torch.allclose(he.double().cpu(), xb.double().cpu(), atol=0.1, rtol=1e-2)
    # per-layer token input: fused kernel and separate steps against the oracle
    table = torch.randn(vocab, 3 * n, device=DEV)
    ids = torch.randint(0, vocab, (rows,), device=DEV, dtype=torch.int32)
    wg, wp = torch.randn(n, W, device=DEV) * 0.3, torch.randn(W, n, device=DEV)
    P = {"gate": wg.double().cpu(), "proj": wp.double().cpu(), "norm": w.double().cpu()}
    want = R.token_side(x.double().cpu(), table.double().cpu()[ids.long().cpu()][:, n:2 * n], P, 1e-5)
    fused = ops.token_side(x.clone(), ids, table, n, wg, wp, w, 1e-5)
    assert torch.allclose(fused.double().cpu(), want, atol=2e-5, rtol=1e-5)
    s = x @ wg.T
    g = ops.token_side_act(s.contiguous(), ids, table, n, torch.empty(rows, n, device=DEV))
    assert torch.allclose(g.double().cpu(), R.gelu_tanh(s.double().cpu()) * table.double().cpu()[ids.long().cpu()][:, n:2 * n],
                          atol=1e-5)


def test_clamped_feed_forward_activation():
    """The gate is cut from above only, the up projection on both sides; the engine's kernel for it is the experts'."""
    from dli_b200 import ops

    h = torch.tensor([[10.0, -10.0, 0.3, -0.2]], dtype=F64)
    eye = torch.eye(4, dtype=F64)
    want = R.clamped_ff(h, {"gate": eye, "up": eye.flip(0), "down": eye}, 1.5)
    g0 = 1.5 * torch.sigmoid(torch.tensor(1.702 * 1.5, dtype=F64)) * (-0.2 + 1)
    g1 = -10.0 * torch.sigmoid(torch.tensor(-17.02, dtype=F64)) * (0.3 + 1)
    assert torch.allclose(want[0, :2], torch.stack((g0, g1)), atol=1e-12)
    gu = torch.cat((h, h.flip(1)), 1).float().to(DEV)
    act = ops.moe_act(gu, None, torch.empty(1, 4, device=DEV), 0, 0, 0.0, ff_s=4, limit_s=1.5, alpha=1.702)
    assert torch.allclose(act.double().cpu(), want, atol=1e-6)


def test_head_norm_and_gate():
    from dli_b200 import ops

    torch.manual_seed(3)
    rows, H, V = 5, 3, 10
    o = torch.randn(rows, H * V, device=DEV) * 7
    proj = torch.randn(rows, 4 + H * V, device=DEV)
    w = torch.randn(V, device=DEV)
    out = ops.head_rmsnorm_gate(o, proj, w, torch.empty(rows, H * V, device=DEV), H, V, 1e-5, gate=1, g_off=4)
    want = R.rms_norm(o.double().cpu().view(rows, H, V), w.double().cpu(), 1e-5) * R.silu(proj.double().cpu()[:, 4:]).view(rows, H, V)
    assert torch.allclose(out.double().cpu().view(rows, H, V), want, atol=1e-5, rtol=1e-5)


@pytest.mark.parametrize("cuts", [[200], [70, 3, 64, 20]])
def test_tensor_core_tiles_with_kept_first_positions(cuts):
    """bfloat16, head sizes with a tensor-core tile: the kept first positions lie in tiles far below the window's, in
    the window's own first tile, or the window reaches back over them."""
    for size, keep in ((20, 70), (70, 5), (100, 130), (64, 64), (3, 1)):
        eng, cfg, sd = engine_of([(attention(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.4, size=size, keep_first=keep), None)],
                                 width=64, page_size=16, dtype=torch.bfloat16)
        T = 200
        torch.manual_seed(size)
        u = torch.randn(T, 4 * 64, dtype=F64).bfloat16().double()
        got = run_mixers(eng, [u], cuts, tiles=True)[0].reshape(T, 2, 64)
        vis = R.visible(T, size, keep)
        kn = R.rms_norm(u[:, 128:192], None, 1e-5)
        for h in range(2):
            want = R.softmax_attend((R.rms_norm(u[:, 64 * h:64 * h + 64], None, 1e-5) @ kn.T) * 0.4, u[:, 192:], vis)
            assert (got[:, h] - want).abs().max() < 0.06, (size, keep, h)


@pytest.mark.parametrize("rows", [1, 2, 5, 40, 200])
def test_clamped_activation_as_the_projection_epilogue(rows):
    """bfloat16 weights with ff a multiple of 128: the gate/up projection carries the clamped activation in its
    epilogue on every path (weight stream, split-K stream, tensor-core GEMM); against the oracle on the same weights."""
    from dli_b200 import ops

    torch.manual_seed(rows)
    W, ff, limit = 128, 256, 1.1
    x = (torch.randn(rows, W) * 1.5).bfloat16()
    wg, wu = (torch.randn(ff, W) * 0.2).bfloat16(), (torch.randn(ff, W) * 0.2).bfloat16()
    w_gu = ops.pack_gate_up(wg, wu).to(DEV)
    act = torch.tensor([limit, 1.702], device=DEV)
    scratch = torch.zeros(ops.gemm_splitk_scratch_bytes(128, 2 * ff), dtype=torch.uint8, device=DEV)
    got = ops.linear_gated_act(x.to(DEV), w_gu, act, scratch if 2 < rows <= 128 else None)
    want = R.clamped_ff(x.double(), {"gate": wg.double(), "up": wu.double(), "down": torch.eye(ff, dtype=F64)}, limit)
    assert (want.abs() > 1.5).any() and (got.double().cpu() - want).abs().max() < 0.03
