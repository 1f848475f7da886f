"""The Togalorn design on the ragged engine against the plain float64 oracle (oracle/togalorn_ref.py).

Small made-up configurations with random weights.  The float32 engine must agree with the oracle to ~1e-4 of the
logits' spread at EVERY position — a key that is one position off, a lost recurrent state or convolution history,
a wrong expert or a stale slot changes logits by orders of magnitude more — whatever the schedule: whole prompts,
token-by-token decoding, portions down to two tokens, mixed batches, small page pools and reused slots.  The
bfloat16 engine is held to a bf16-sized bound and to agreement between schedules.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import togalorn_ref as R  # noqa: E402


def latent(heads=3, dim=8, rot_dim=4, vdim=12, kv_rank=20, q_rank=14, scale=0.4, base=1000.0):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim,
                                                  "kv_rank": kv_rank, "q_rank": q_rank, "scale": scale,
                                                  "rot": {"base": base, "dims": rot_dim}}}


def mamba(heads=4, vdim=6, state=10, groups=2, norm_groups=3, conv=3):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups,
                                        "norm_groups": norm_groups, "conv": conv}}


def moe(experts=4, identity=2, top=2, ff=24, limit=1.2, shared=(16, 0.8)):
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity,
                                                                              "top": top}}
    if shared:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def config(layers, width=48, vocab=97, taps=3, eps=1e-5, groups=4, loop=None, scale=3.0):
    out = []
    for L, mlp in layers:
        L = dict(L)
        L["mlp"] = mlp
        out.append(L)
    cfg = {"architecture": "Togalorn", "vocab": vocab, "width": width, "embedding": {"scale": scale},
           "norm": {"eps": eps, "groups": groups}, "canon": {"taps": taps}, "layers": out}
    if loop:
        cfg["loop"] = {"start": loop[0], "stop": loop[1], "times": loop[2]}
    return cfg


def cfg_a():
    """state-space, latent attention, state-space, latent attention without feed-forward; layers 1..2 run twice."""
    return config([(mamba(), moe()), (latent(), moe()), (mamba(heads=2, vdim=16, state=8, groups=1, norm_groups=1, conv=4),
                                                          moe(top=3)), (latent(heads=2, dim=6, rot_dim=6, vdim=8), None)],
                  loop=(1, 3, 2))


def cfg_b():
    """other sizes: one norm group, two taps, no loop, no pass-through experts, no shared expert, one expert per token,
    one head, rotated part larger than the unrotated one, odd vocabulary, a width that is no multiple of 16."""
    return config([(latent(heads=1, dim=4, rot_dim=10, vdim=6, kv_rank=12, q_rank=6, scale=0.7), moe(experts=3, identity=0,
                                                                                                         top=1, ff=20, shared=None)),
                   (mamba(heads=1, vdim=8, state=4, groups=1, norm_groups=2, conv=2), None),
                   (mamba(heads=6, vdim=4, state=18, groups=3, norm_groups=1, conv=5), moe(experts=2, identity=3, top=4, ff=8))],
                  width=40, vocab=53, taps=2, groups=1, scale=1.0)


def cfg_c():
    """one tap everywhere (no convolution history), the whole stack looped three times, every expert used by every
    token, five norm groups."""
    return config([(mamba(heads=2, vdim=5, state=3, groups=2, norm_groups=2, conv=1), moe(experts=2, identity=1, top=3, ff=12)),
                   (latent(heads=2, dim=2, rot_dim=2, vdim=2, kv_rank=4, q_rank=2, scale=1.0), None)],
                  width=20, vocab=19, taps=1, groups=5, loop=(0, 2, 3))


def cfg_d():
    """state-space layers only (no paged cache at all), the last two looped; one without feed-forward."""
    return config([(mamba(), moe(top=1)), (mamba(heads=3, vdim=8, state=6, groups=3, norm_groups=4, conv=2), None),
                   (mamba(heads=2, vdim=12, state=5, groups=1, norm_groups=1, conv=3), moe(identity=0))], width=32, groups=2,
                  loop=(1, 3, 2))


def cfg_e():
    """latent-attention layers only, the first one looped three times by itself."""
    return config([(latent(), moe()), (latent(heads=1, dim=16, rot_dim=2, vdim=4, kv_rank=6, q_rank=10, scale=0.3), None)],
                  width=32, groups=8, loop=(0, 1, 3), taps=4)


def build(cfg, dtype, seed=0, max_batch=4, max_seq_len=256, pool=None, page_size=4):
    from dli_b200 import togalorn
    from dli_b200.ragged_engine import RaggedEngine

    spec = togalorn.spec_from_config(cfg)
    sd = togalorn.random_state_dict(spec, seed=seed, std=0.15)
    eng = RaggedEngine(spec, max_batch=max_batch, max_seq_len=max_seq_len, page_size=page_size, kv_pool_tokens=pool,
                       dtype=dtype)
    eng.load_tensors(togalorn.model_tensors(spec, sd))
    return eng, sd


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def rel_err(got, ref):
    """Per position: RMS of the logit difference (mean removed) over the RMS spread of the reference logits."""
    d = got.double().cpu() - ref
    d = d - d.mean(-1, keepdim=True)
    spread = (ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def run_schedule(eng, toks, cuts):
    """One sequence alone, cut into portions of the given sizes (the rest token by token); logits at every position."""
    slot = eng.open_sequence()
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(eng.step([(slot, toks[at:at + n])], [list(range(n))]).float().cpu())
        at += n
    eng.close_sequence(slot)
    return torch.cat(out)


TOL32, TOL16 = 2e-4, 0.08


def close16(err):
    """bfloat16: every position within the bf16-sized bound, except for the few where rounding upstream turns a near-tie
    of the router the other way (another expert: a larger but still small difference)."""
    return bool((err < TOL16).double().mean() >= 0.97 and err.max() < 0.5)


@pytest.mark.parametrize("make", [cfg_a, cfg_b, cfg_c, cfg_d, cfg_e])
def test_whole_prompt_float32_matches_oracle_at_every_position(make):
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(45, cfg["vocab"], 1)
    ref, _ = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, [45]), ref).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_c])
def test_residual_stream_after_every_layer_run(make):
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(19, cfg["vocab"], 2)
    _, layers = R.forward(cfg, sd, toks)
    eng.layer_trace = []
    run_schedule(eng, toks, [19])
    assert len(eng.layer_trace) == layers.shape[0] == len(R.layer_runs(cfg))
    for got, ref in zip(eng.layer_trace, layers):
        assert (got.double().cpu() - ref).abs().max() < 1e-4 * ref.abs().max()


@pytest.mark.parametrize("make", [cfg_a, cfg_b, cfg_c, cfg_d, cfg_e])
@pytest.mark.parametrize("cuts", [[], [1, 1, 2], [2, 2, 3, 5, 7, 11], [17, 2, 16, 3], [30]])
def test_portions_and_decoding_float32(make, cuts):
    """Token by token from the first token; portions of 2..; a prompt then decoding over page borders."""
    cfg = make()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(52, cfg["vocab"], 3)
    ref, _ = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, cuts), ref).max() < TOL32


@pytest.mark.parametrize("make", [cfg_a, cfg_b])
def test_bfloat16_engine_is_close_and_schedules_agree(make):
    cfg = make()
    eng, sd = build(cfg, torch.bfloat16)
    toks = prompt(40, cfg["vocab"], 4)
    ref, _ = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [40])
    parts = run_schedule(eng, toks, [7, 2, 9, 3])
    assert close16(rel_err(whole, ref))
    assert close16(rel_err(parts, ref))
    assert close16(rel_err(parts, whole.double()))


def test_bfloat16_sizes_of_the_tensor_core_projections():
    """Widths and sizes in multiples of 64 / 128, where projections run on the tensor-core GEMMs and the split-K weight
    stream; long portions beside short ones."""
    cfg = config([(mamba(heads=4, vdim=32, state=16, groups=2, norm_groups=2, conv=4), moe(experts=4, identity=1, top=2, ff=64,
                                                                                         shared=(128, 1.0))),
                  (latent(heads=4, dim=32, rot_dim=16, vdim=32, kv_rank=64, q_rank=48, scale=0.15), moe(ff=32))],
                 width=128, vocab=200, loop=(0, 2, 2))
    eng, sd = build(cfg, torch.bfloat16, max_seq_len=256, page_size=16)
    toks = prompt(150, cfg["vocab"], 6)
    ref, _ = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [150])
    parts = run_schedule(eng, toks, [70, 3, 64])
    assert close16(rel_err(whole, ref))
    assert close16(rel_err(parts, ref))


def test_mixed_batches_of_unequal_requests_match_each_alone():
    """Four requests of different lengths move through shared steps in portions of different sizes, some decoding
    while others are in their prompt, some skipping steps; each position equals the oracle's for that request alone."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, pool=160, max_seq_len=160)
    lens = [37, 9, 58, 1]
    reqs = [prompt(n, cfg["vocab"], 10 + i) for i, n in enumerate(lens)]
    refs = [R.forward(cfg, sd, t)[0] for t in reqs]
    slots = [eng.open_sequence() for _ in reqs]
    at = [0] * len(reqs)
    got = [[] for _ in reqs]
    pattern = [[5, 2, 9, 1], [1, 0, 16, 0], [3, 1, 1, 0], [0, 3, 2, 0], [8, 1, 7, 0], [1, 1, 1, 0], [19, 1, 22, 0]]
    k = 0
    while any(a < n for a, n in zip(at, lens)):
        sizes = pattern[k % len(pattern)]
        k += 1
        batch, want, who = [], [], []
        for i, n in enumerate(sizes):
            n = min(n, lens[i] - at[i])
            if n > 0:
                batch.append((slots[i], reqs[i][at[i]:at[i] + n]))
                want.append(list(range(n)))
                who.append((i, n))
        if not batch:
            continue
        lg = eng.step(batch, want).float().cpu()
        o = 0
        for i, n in who:
            got[i].append(lg[o:o + n])
            o += n
            at[i] += n
    for i in range(len(reqs)):
        assert rel_err(torch.cat(got[i]), refs[i]).max() < TOL32, f"request {i}"


def test_pages_and_slots_are_used_again():
    """A pool that holds two sequences at most and two slots: six sequences pass through in turn, each against the
    oracle; a slot's previous state (recurrent state, convolution histories, pages) must not leak into the next one."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=2, pool=64, max_seq_len=64, page_size=4)
    for r in range(3):
        ta, tb = prompt(29 + r, cfg["vocab"], 20 + r), prompt(11 + 2 * r, cfg["vocab"], 30 + r)
        ra, rb = R.forward(cfg, sd, ta)[0], R.forward(cfg, sd, tb)[0]
        sa, sb = eng.open_sequence(), eng.open_sequence()
        la = [eng.step([(sa, ta[:13])], [list(range(13))])]
        both = eng.step([(sa, ta[13:]), (sb, tb)], [list(range(len(ta) - 13)), list(range(len(tb)))])
        la.append(both[:len(ta) - 13])
        assert rel_err(torch.cat(la), ra).max() < TOL32
        assert rel_err(both[len(ta) - 13:], rb).max() < TOL32
        eng.close_sequence(sb if r % 2 else sa)   # give the slots back in changing order
        eng.close_sequence(sa if r % 2 else sb)
    assert len(eng.kv.free) == eng.kv.num_pages and len(eng.slots.free) == 2


def test_long_decoding_float32():
    """150 tokens one by one: the recurrent state is carried 150 times, pages fill and follow."""
    cfg = cfg_b()
    eng, sd = build(cfg, torch.float32)
    toks = prompt(150, cfg["vocab"], 5)
    ref, _ = R.forward(cfg, sd, toks)
    assert rel_err(run_schedule(eng, toks, [3]), ref).max() < TOL32


def test_greedy_generation_through_the_scheduler():
    """generate() -> RaggedBatcher -> step(): three prompts of one length share steps; tokens equal the oracle's greedy
    continuation (float32 engine: no near-ties at these sizes)."""
    cfg = cfg_a()
    eng, sd = build(cfg, torch.float32, max_batch=3)
    eng.prefill_chunk = 8   # prompts go in portions of at most 8 tokens per step, shared between the requests
    ids = torch.tensor([prompt(13, cfg["vocab"], 40 + i) for i in range(3)])
    out = eng.generate(ids, max_length=13 + 5)
    for b in range(3):
        assert out[b].tolist() == R.greedy(cfg, sd, ids[b].tolist(), 5)
    assert len(eng.slots.free) == 3 and len(eng.kv.free) == eng.kv.num_pages


def test_decode_steps_replayed_as_a_graph_equal_eager_steps():
    """Steps of single tokens are captured once per batch size and replayed; the logits equal the eager launches' bit
    for bit, also when the batch size changes and a sequence leaves in between."""
    cfg = cfg_a()
    outs = []
    for graph in (True, False):
        eng, sd = build(cfg, torch.float32, max_batch=3)
        eng.use_cuda_graph = graph
        seqs = [prompt(30, cfg["vocab"], 60 + i) for i in range(3)]
        slots = [eng.open_sequence() for _ in seqs]
        got = [eng.step([(slots[i], seqs[i][:9]) for i in range(3)])]
        for t in range(9, 20):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in range(3)]))
        eng.close_sequence(slots[1])
        for t in range(20, 30):
            got.append(eng.step([(slots[i], [seqs[i][t]]) for i in (0, 2)]))
        outs.append(torch.cat([g.float().cpu() for g in got]))
        if graph:
            assert any(isinstance(v, tuple) for v in eng._graphs.values())
    assert torch.equal(outs[0], outs[1])


def test_bfloat16_portions_of_latent_attention_on_the_tensor_cores():
    """Head sizes that have a tensor-core tile: steps with portions of 16 rows and more expand the cached latents to
    per-head keys and values and take that kernel (also for the short entries beside them, and with the pages in use
    starting anywhere in the pool), other steps attend over the latents themselves; both against the oracle and
    against each other."""
    cfg = config([(latent(heads=4, dim=32, rot_dim=32, vdim=64, kv_rank=64, q_rank=48, scale=0.125), None),
                  (mamba(), moe()),
                  (latent(heads=2, dim=64, rot_dim=64, vdim=128, kv_rank=96, q_rank=32, scale=0.09), moe())], width=128)
    eng, sd = build(cfg, torch.bfloat16, max_seq_len=256, page_size=16, pool=512)
    assert "w_ukv" in eng.layers[0] and "w_ukv" in eng.layers[2]
    toks = prompt(170, cfg["vocab"], 6)
    ref, _ = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [170])
    hold = eng.open_sequence()                 # another sequence holds the first pages of the pool meanwhile
    eng.step([(hold, prompt(40, cfg["vocab"], 7))])
    parts = run_schedule(eng, toks, [70, 3, 64, 20])
    eng.close_sequence(hold)
    eng.tc_min_rows = 10 ** 9
    rowwise = run_schedule(eng, toks, [170])
    for got in (whole, parts, rowwise):
        assert close16(rel_err(got, ref))
    assert close16(rel_err(whole, rowwise.double()))
    # a long portion beside a decoding sequence in one step
    eng.tc_min_rows = 16
    a, b = eng.open_sequence(), eng.open_sequence()
    eng.step([(a, toks[:50])])
    both = eng.step([(a, [toks[50]]), (b, toks[:90])], [[0], list(range(90))]).float().cpu()
    assert close16(rel_err(both[:1], ref[50:51])) and close16(rel_err(both[1:], ref[:90]))


def test_bfloat16_decode_rows_of_a_sparse_mixture_read_only_the_chosen_experts():
    """8 experts, 2 per token, no shared expert: decode steps take the kernel that streams the chosen experts' weights
    only, portions of prompts the GEMMs over all experts; both against the oracle and against each other."""
    cfg = config([(mamba(), moe(experts=8, identity=1, top=2, ff=24, shared=None)),
                  (latent(), moe(experts=8, identity=0, top=1, ff=16, shared=(8, 1.0)))], width=64)
    eng, sd = build(cfg, torch.bfloat16)
    e = eng.spec.layers[0].moe
    eng.moe_sel_min_bytes = 0                     # the engine keeps these kernels for large mixtures; here they run at a small one
    assert eng._moe_sel_ok(e, 1)
    toks = prompt(40, cfg["vocab"], 8)
    ref, _ = R.forward(cfg, sd, toks)
    whole = run_schedule(eng, toks, [40])
    single = run_schedule(eng, toks, [20])        # 20 decode steps
    eng.moe_sel_max_rows = 0
    dense = run_schedule(eng, toks, [20])
    for got in (whole, single, dense):
        assert close16(rel_err(got, ref))
    assert close16(rel_err(single, dense.double()))
