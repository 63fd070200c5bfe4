"""Bevovik through the engine (scheduler bookkeeping, page / state-slot managers, batch builder, runner) against the
plain oracle in bevovik_oracle.py: mechanisms alone, chunking, batching, re-use of pages and slots, far keys and page
borders, convolution edges, router corner cases, degenerate sizes, greedy generation. Runs on the CPU path in fp32;
test_bevovik_gpu.py repeats the scenarios on the kernels."""
import math

import numpy as np
import pytest
import torch

import bevovik_oracle as oracle
import bevovik_util as U

TOL = 2e-4
EPS = 1e-5


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


CONFIGS = {
    "rglru_only": U.make_config([U.rglru(mlp=U.moe()), U.rglru(width=16, blocks=1, conv=4)]),
    "gla_only": U.make_config([U.gla(mlp=U.moe()), U.gla(heads=3, dim=4, vdim=4, tau=2.0)]),
    "latent_only": U.make_config([U.latent(mlp=U.moe()),
                                  U.latent(heads=2, dim=6, rot_dim=6, vdim=10, q_rank=7, kv_rank=9, scaling=None)]),
    "mixed": U.make_config([U.gla(mlp=U.moe()), U.latent(mlp=U.moe(experts=5, identity=1, top=3, groups=(3, 2))),
                            U.rglru(mlp=None), U.rglru(conv=2, mlp=U.moe(identity=0, top=1, shared=None)),
                            U.latent(heads=1, rot_dim=2, mlp=U.moe(groups=None))]),
    "ones": U.make_config([U.rglru(width=4, blocks=4, conv=1, mlp=U.moe(experts=1, identity=0, top=1, ff=4,
                                                                         groups=(1, 1), scale=1.0, shared=(4, 9.0))),
                           U.gla(heads=1, dim=2, vdim=2, tau=1.0, mlp=U.moe(experts=2, identity=2, top=4, ff=4,
                                                                            groups=(4, 4))),
                           U.latent(heads=1, dim=2, rot_dim=2, vdim=2, q_rank=1, kv_rank=1, scale=1.0,
                                    scaling={"factor": 1.0, "original": 8, "fast": 2.0, "slow": 1.0},
                                    mlp=U.moe(experts=1, identity=3, top=2, ff=2, groups=(2, 1), limit=0.25))],
                          width=8, vocab=17),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=60 + i, low_rank=3 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


# -- each mechanism alone, against its own oracle function -----------------------------------------------------
def build_mixer(layer_cfg, w, width, device="cpu", dtype=torch.float32):
    from gllm_b200.models.hybrid import HybridSpec, make_mixer
    spec = HybridSpec("bevovik", width, 61, EPS, 1.0, [layer_cfg], dtype=dtype, block="branchnorm",
                      ff_act="glu_clamp")
    mc = dict(layer_cfg["mixer"])
    if layer_cfg["type"] == "gla":
        mc["low_rank"] = w["l0.mix.a1"].shape[0]
    m = make_mixer(layer_cfg["type"], mc, spec, device)

    def put(p, t):
        assert tuple(p.shape) == tuple(t.shape)
        p.data.copy_(t)

    m.load(U.DictReader(w), "l0.mix.", put)
    return m


ORACLE_MIXER = {"rglru": oracle.rglru_mixer, "gla": oracle.gla_mixer, "latent_attention": oracle.latent_attention_mixer}


def _mixer_alone(layer_cfg, seed, n=19, cuts=((19,), (7, 1, 1, 2, 8), (2,) * 9 + (1,), (1,) * 19), page_size=4,
                 width=20, low_rank=5, device="cpu", dtype=torch.float32, tol=2e-4):
    cfg = U.make_config([layer_cfg], width=width)
    w = U.random_weights(cfg, seed, low_rank)
    m = build_mixer(layer_cfg, w, width, device, dtype)
    h = torch.randn(n, width, generator=torch.Generator().manual_seed(seed))
    if dtype == torch.bfloat16:
        h = h.bfloat16().float()
    wd = {k: v.double() for k, v in w.items()}
    want = ORACLE_MIXER[layer_cfg["type"]](h.double(), wd, "l0.mix.", layer_cfg["mixer"], EPS).float()
    for cut in cuts:
        got = U.drive_mixer(m, h, cut, page_size, device, dtype)
        assert torch.allclose(got, want, atol=tol * (1 + want.abs().max().item()), rtol=tol), cut


def test_rglru_mixer_alone():
    _mixer_alone(U.rglru(), 1)
    _mixer_alone(U.rglru(width=10, blocks=5, conv=4), 2)
    _mixer_alone(U.rglru(width=8, blocks=1, conv=1), 3)
    _mixer_alone(U.rglru(width=12, blocks=12, conv=2), 4)


def test_gla_mixer_alone():
    _mixer_alone(U.gla(), 5)
    _mixer_alone(U.gla(heads=1, dim=3, vdim=7, tau=1.0), 6, low_rank=1)
    _mixer_alone(U.gla(heads=4, dim=8, vdim=2, tau=32.0), 7, low_rank=9)


def test_latent_attention_mixer_alone():
    _mixer_alone(U.latent(), 8)
    _mixer_alone(U.latent(heads=1, dim=4, rot_dim=8, vdim=3, q_rank=3, kv_rank=5, scaling=None), 9, page_size=8)
    _mixer_alone(U.latent(heads=5, dim=2, rot_dim=2, vdim=9, q_rank=16, kv_rank=4,
                          scaling={"factor": 16.0, "original": 6, "fast": 3.0, "slow": 0.5}), 10, page_size=16)


def test_rotary_frequencies_and_rotation():
    """YaRN's ramp over the pair index, its clamps at both ends, no scaling, and the pair layout at far positions."""
    from gllm_b200.ops import ref
    cases = [(16, 30000.0, None), (8, 100.0, U.YARN), (32, 10000.0, {"factor": 6.0, "original": 64, "fast": 24.0,
                                                                     "slow": 1.0}),
             (4, 10.0, {"factor": 2.0, "original": 4, "fast": 1000.0, "slow": 0.001}),      # ramp clamps to [0, 3]
             (6, 500.0, {"factor": 1.0, "original": 100, "fast": 4.0, "slow": 2.0}),
             (12, 1000.0, {"factor": 40.0, "original": 4096, "fast": 1.0, "slow": 1.0})]    # lo == hi: the 0.001 floor
    for dims, base, sc in cases:
        f, mag = ref.pair_rotary_frequencies(dims, base, sc)
        f2, mag2 = oracle.yarn_frequencies(dims, base, sc)
        assert torch.allclose(f.double(), f2, rtol=1e-6, atol=0), (dims, base, sc)
        assert abs(mag - mag2) < 1e-7
    # by hand, for one case: dims 8, base 100, factor 4, original 16, fast 8, slow 1
    where = lambda t: 8 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(100.0))      # noqa: E731
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 7)
    f, mag = ref.pair_rotary_frequencies(8, 100.0, U.YARN)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        fi = 100.0 ** (-2 * i / 8)
        assert abs(f[i].item() - (fi / 4 * ramp + fi * (1 - ramp))) < 1e-7
    assert abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-7


def _route_case(n_exp, identity, top, groups, scale, corr, seed, t=40, width=12, device="cpu"):
    from gllm_b200.layers import functional as Fn
    g = torch.Generator().manual_seed(seed)
    n = n_exp + identity
    h = torch.randn(t, width, generator=g)
    wr = torch.randn(n, width, generator=g)
    r = {"experts": n_exp, "identity": identity, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    ids2, wt2 = oracle.route(h.double(), {"router": wr.double(), "correction": corr.double()}, "", r)
    gc, keep = groups or (1, 1)
    wt1, ids1 = Fn.grouped_router(h.to(device), wr.to(device), corr.float().to(device), top, gc, keep, scale)
    o1, o2 = ids1.cpu().long().sort(-1), ids2.sort(-1)
    assert torch.equal(o1.values, o2.values), (n_exp, identity, top, groups)
    assert torch.allclose(wt1.cpu().double().gather(1, o1.indices), wt2.gather(1, o2.indices), atol=1e-5)
    return ids2


def test_router_corner_cases():
    # a correction that makes every choice score negative: the group limit must mask with -inf, not 0
    ids = _route_case(6, 2, 2, (2, 1), 1.5, torch.full((8,), -3.0) + torch.randn(8) * 0.01, 1)
    assert all(len({int(e) // 4 for e in row}) == 1 for row in ids)          # both choices from one group
    # the correction steers the choice but not the weights; one group is pushed up so that it always wins
    ids = _route_case(6, 2, 3, (4, 2), 2.5, torch.tensor([0, 0, 0, 0, 0, 0, 5.0, 5.0]), 2)
    assert all(6 in row.tolist() and 7 in row.tolist() for row in ids)       # the identity pair is always chosen
    _route_case(8, 0, 2, (2, 1), 1.0, torch.randn(8) * 0.2, 3)
    _route_case(5, 1, 6, (3, 3), 0.5, torch.randn(6) * 0.2, 4)               # everything is chosen
    _route_case(7, 0, 1, None, 1.0, torch.randn(7), 5)
    _route_case(3, 9, 4, (4, 2), 3.0, torch.randn(12) * 0.3, 6)
    _route_case(64, 8, 6, (8, 3), 2.5, torch.randn(72) * 0.05, 7, t=70)


def test_feed_forward_alone():
    """Routed experts with identity experts and the shared expert, against the oracle's per-token loop."""
    from gllm_b200.models.hybrid import HybridSpec, make_ff
    for seed, mlp in enumerate([U.moe(), U.moe(experts=3, identity=3, top=4, groups=(3, 2), limit=0.3),
                                U.moe(experts=4, identity=0, top=2, groups=None, shared=None),
                                U.moe(experts=1, identity=1, top=2, groups=(1, 1), shared=(4, 0.1))]):
        cfg = U.make_config([U.rglru(mlp=mlp)])
        w = U.random_weights(cfg, 30 + seed)
        spec = HybridSpec("bevovik", 20, 61, EPS, 1.0, cfg["layers"], dtype=torch.float32, block="branchnorm",
                          ff_act="glu_clamp")
        f = make_ff(mlp, spec, "cpu")
        f.router_w.data.copy_(w["l0.mlp.router"])
        f.correction.data.copy_(w["l0.mlp.correction"])
        for e in range(mlp["router"]["experts"]):
            f.load_expert(e, *[w["l0.mlp.e%d.%s" % (e, n)] for n in ("gate", "up", "down")])
        if f.shared is not None:
            f.shared.load(*[w["l0.mlp.shared." + n] for n in ("gate", "up", "down")])
        h = torch.randn(33, 20, generator=torch.Generator().manual_seed(seed)) * 2.0
        want = oracle.moe_ff(h.double(), {k: v.double() for k, v in w.items()}, "l0.mlp.", mlp).float()
        assert torch.allclose(f(h), want, atol=2e-4, rtol=2e-4), seed


def test_clamped_activation_limits():
    """The gate is clamped from above only, the up projection on both sides, and 1 is added after the clamp."""
    from gllm_b200.layers import functional as Fn
    gu = torch.tensor([[-7.0, 0.5, 3.0, 9.0, -7.0, 0.5, 3.0, -9.0]])
    got = Fn.glu_clamp(gu, 2.0)
    g = torch.tensor([-7.0, 0.5, 2.0, 2.0])
    u = torch.tensor([-2.0, 0.5, 2.0, -2.0])
    assert torch.allclose(got, (g * torch.sigmoid(1.702 * g) * (u + 1))[None], atol=1e-6)


# -- whole models ----------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_matches_oracle(models, name):
    cfg, w, path = models[name]
    t = toks(37, cfg["vocab"], 1)
    s = U.session(path)
    got = s.step([{"id": "a", "tokens": t, "want": list(range(len(t)))}], ["a"])
    assert U.rel_err(got, U.expected_logits(cfg, w, t)) < TOL


def test_residual_stream_after_every_layer(models):
    cfg, w, path = models["mixed"]
    t = toks(11, cfg["vocab"], 8)
    trace = []
    oracle.forward(cfg, w, t, torch.float64, trace)
    s = U.session(path)
    s.runner.model.trace = []
    s.step([{"id": "a", "tokens": t, "want": []}], ["a"])
    got = s.runner.model.trace
    assert len(got) == len(trace) == len(cfg["layers"])
    for a, b in zip(got, trace):
        assert torch.allclose(a.double(), b, atol=1e-4)


@pytest.mark.parametrize("name", ["mixed", "ones", "rglru_only", "latent_only"])
def test_token_by_token_equals_prefill(models, name):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 2)        # long decoding: crosses 11 pages
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, []), want) < TOL
    assert U.rel_err(U.run_chunks(s, "b", t, [len(t)]), want) < TOL


@pytest.mark.parametrize("cuts", [[2, 2, 2, 3, 5], [7, 1, 1, 2, 9, 4], [16, 2], [1, 30], [33, 2, 2], [6, 1, 7, 7]])
def test_portions(models, cuts):
    cfg, w, path = models["mixed"]
    t = toks(41, cfg["vocab"], 3)
    s = U.session(path)
    assert U.rel_err(U.run_chunks(s, "a", t, cuts), U.expected_logits(cfg, w, t)) < TOL


def test_mixed_batch_equals_alone_and_reuses_pages_and_slots(models):
    cfg, w, path = models["mixed"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26),
                                                              ("f", 12)])}
    want = {k: U.expected_logits(cfg, w, t) for k, t in reqs.items()}
    # pool of 64 tokens and 3 slots: the six requests cannot all be resident, pages and slots are handed on
    s = U.session(path, max_tokens=64, page_size=4, state_slots=3)
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    got = U.run_plan(s, reqs, plan)
    for k in reqs:
        assert U.rel_err(got[k], want[k]) < TOL, k
    mm = s.scheduler.mm
    assert mm.get_num_free_state_slots() == 3 and mm.get_num_free_pages() == mm.usable_pages


def test_stale_slot_and_page_contents_do_not_leak(models):
    cfg, w, path = models["mixed"]
    s = U.session(path, max_tokens=32, page_size=4, state_slots=1)
    a, b = toks(19, cfg["vocab"], 5), toks(7, cfg["vocab"], 6)
    U.run_chunks(s, "a", a, [10, 9])
    assert U.rel_err(U.run_chunks(s, "b", b, [3, 2, 2]), U.expected_logits(cfg, w, b)) < TOL


def test_first_tokens_of_a_sequence(models):
    cfg, w, path = models["mixed"]
    t = toks(6, cfg["vocab"], 9)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path)
    for cuts in ([1], [1, 1, 1], [2, 1], [3, 3]):
        assert U.rel_err(U.run_chunks(s, "x%d" % len(cuts), t, cuts), want) < TOL


# -- edges that random weights would hide ----------------------------------------------------------------------
def far_key_probe(n, back, page_size, device="cpu", dtype=torch.float32, heads=2, dim=16, rank=16, vdim=4):
    """Latent attention whose query and key paths share their weights up to a permutation of the input (q_rank =
    kv_rank, W_dq = the latent rows of W_dkv with permuted columns, every head's unrotated query map = its key map,
    no rotated part in the scores), every head's key map orthogonal and the latent's norm weight 1, so that all keys
    have the same length and a query scores highest with the key equal to it, and a large softmax scale: a query
    then picks out the key that was made from the permuted input. The last token's input is the permuted input of the token `back` places before it (back = 0: of
    itself before the permutation, so nothing is marked), all other inputs are random. -> (oracle, outputs for several ways of cutting, the
    oracle with the marked token's input replaced)."""
    g = torch.Generator().manual_seed(back * 7 + page_size)
    width, rot = 12, 2
    layer = U.latent(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, q_rank=rank, kv_rank=rank, scale=12.0,
                     scaling=None)
    cfg = U.make_config([layer], width=width)
    w = U.random_weights(cfg, 99)
    assert dim == rank
    w["l0.mix.dkv"][rank:] = 0                                  # no rotated key part
    w["l0.mix.dkv.norm"] = torch.ones(rank)
    w["l0.mix.uk"] = torch.cat([torch.linalg.qr(torch.randn(rank, rank, generator=g))[0] for _ in range(heads)], 0)
    perm = torch.roll(torch.arange(width), 5)                  # query path(h) = key path(h') with h'[perm] = h
    w["l0.mix.dq"] = w["l0.mix.dkv"][:rank][:, perm].clone()
    w["l0.mix.dq.norm"] = w["l0.mix.dkv.norm"].clone()
    uq = torch.zeros(heads, dim + rot, rank)
    uq[:, :dim] = w["l0.mix.uk"].reshape(heads, dim, rank)
    w["l0.mix.uq"] = uq.reshape(heads * (dim + rot), rank)
    m = build_mixer(layer, w, width, device, dtype)
    h = torch.randn(n, width, generator=g)
    tgt = n - 1 - back
    h[n - 1] = h[tgt][perm]                                    # the last query equals the marked token's key
    wd = {k: v.double() for k, v in w.items()}
    want = oracle.latent_attention_mixer(h.double(), wd, "l0.mix.", layer["mixer"], EPS).float()
    h2 = h.clone()
    if back > 0:
        h2[tgt] = torch.randn(width, generator=g)
    other = oracle.latent_attention_mixer(h2.double(), wd, "l0.mix.", layer["mixer"], EPS).float()
    cuts = [[n], [n - 1, 1], [n - back - 1, 1] + [back] * (back > 0), [max(n - 40, 1)] + [2] * 19]
    outs = []
    for c in cuts:
        c = [x for x in c if x > 0]
        rest = n - sum(c)
        assert rest >= 0
        outs.append(U.drive_mixer(m, h, c + [1] * rest, page_size, device, dtype, pool=1024))
    return want, outs, other


@pytest.mark.parametrize("page_size", [4, 16])
def test_far_keys_and_page_borders(page_size):
    n = 331
    for back in (0, 1, 2, page_size - 1, page_size, page_size + 1, 63, 64, 65, 200, 329, 330):
        want, outs, other = far_key_probe(n, back, page_size)
        if back > 0:          # the oracle's last row rests on the marked key
            assert (want[-1] - other[-1]).abs().max() > 0.05 * want[-1].abs().max(), back
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4 * want.abs().max().item(), rtol=2e-4), (page_size, back)


def conv_edge_probe(taps, back, device="cpu", dtype=torch.float32):
    """The recurrent block's convolution: the input `back` tokens before the last one is made huge. It reaches the
    last output only through the convolution's taps (the recurrence is switched off by a decay of ~0: lam large), so
    it shows for back < taps and not for back >= taps."""
    width, c = 8, 6
    layer = U.rglru(width=c, blocks=2, conv=taps)
    cfg = U.make_config([layer], width=width)
    w = U.random_weights(cfg, 3)
    w["l0.mix.lam"] = torch.full((c,), 30.0)                     # a = exp(-8 r * 30) ~ 0: no memory besides the taps
    w["l0.mix.ra.b"] = torch.full((2, c // 2), 4.0)
    m = build_mixer(layer, w, width, device, dtype)
    n = 23
    h = torch.randn(n, width, generator=torch.Generator().manual_seed(taps * 10 + back)) * 0.1
    base = oracle.rglru_mixer(h.double(), {k: v.double() for k, v in w.items()}, "l0.mix.", layer["mixer"], EPS)
    h[n - 1 - back] += 5.0
    want = oracle.rglru_mixer(h.double(), {k: v.double() for k, v in w.items()}, "l0.mix.", layer["mixer"], EPS)
    outs = [U.drive_mixer(m, h, cuts, 4, device, dtype)
            for cuts in ([n], [n - 1, 1], [n - back - 1] + [1] * (back + 1), [2] * (n // 2) + [1], [1] * n,
                         [n - 2, 2] if back != 1 else [n - 3, 2, 1])]
    return base.float(), want.float(), outs


@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_convolution_edges(taps):
    for back in range(0, taps + 2):
        base, want, outs = conv_edge_probe(taps, back)
        seen = (want[-1] - base[-1]).abs().max().item() > 1e-3
        assert seen == (back < taps), (taps, back)
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4, rtol=1e-4), (taps, back)


def far_state_model(kind):
    """One recurrent mixer whose decay stays close to 1, so that the first token still shows 300 tokens later."""
    if kind == "gla":
        cfg = U.make_config([U.gla(heads=2, dim=4, vdim=5, tau=64.0, mlp=None)], width=16, vocab=11)
        w = U.random_weights(cfg, 77)
        w["l0.mix.a2.b"] = torch.full_like(w["l0.mix.a2.b"], 4.0)      # sigmoid(~4)^(1/64): decay ~ 0.9997
    else:
        cfg = U.make_config([U.rglru(width=12, blocks=2, conv=2, mlp=None)], width=16, vocab=11)
        w = U.random_weights(cfg, 78)
        w["l0.mix.lam"] = torch.full_like(w["l0.mix.lam"], -7.0)       # softplus ~ 9e-4: decay ~ 0.996 per token
    return cfg, w


@pytest.mark.parametrize("kind", ["gla", "rglru"])
def test_far_state_survives_long_decoding(kind):
    cfg, w = far_state_model(kind)
    path = U.save_model(cfg, w)
    t = [3] + [5] * 300
    t2 = [7] + [5] * 300                      # differs in the first token only
    a, b = U.expected_logits(cfg, w, t), U.expected_logits(cfg, w, t2)
    assert np.abs(a[-1] - b[-1]).max() > 1e-3            # the oracle itself still sees the first token
    s = U.session(path, max_tokens=512, page_size=16)
    assert U.rel_err(U.run_chunks(s, "a", t, [200, 50, 2, 2]), a) < TOL
    assert U.rel_err(U.run_chunks(s, "b", t2, [1, 250]), b) < TOL


def test_low_rank_of_the_decay_comes_from_the_checkpoint(models):
    """config.json does not carry the rank of a gla mixer's decay projection: the loader reads it off the tensor."""
    for rank in (1, 4, 11):
        cfg = U.make_config([U.gla(mlp=None)])
        w = U.random_weights(cfg, rank, low_rank=rank)
        path = U.save_model(cfg, w)
        t = toks(9, cfg["vocab"], rank)
        s = U.session(path)
        got = s.step([{"id": "a", "tokens": t, "want": list(range(9))}], ["a"])
        assert U.rel_err(got, U.expected_logits(cfg, w, t)) < TOL


def test_greedy_generation_through_the_engine(models):
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed"]
    llm = LLM(path, dtype="float32", page_size=4, maxp=16, maxd=8, num_cpu_pages=64, model_max_length=96,
              log_stats=False, device="cpu", num_state_slots=2)
    prompts = [toks(21, cfg["vocab"], 31), toks(3, cfg["vocab"], 32), toks(9, cfg["vocab"], 33)]
    lens = [7, 12, 5]
    seqs = llm.generate(tokens=prompts, output_lens=lens, temperature=0.0, top_k=1)
    for p, n, s in zip(prompts, lens, seqs):
        cur = list(p)
        for _ in range(n):
            cur.append(int(oracle.forward(cfg, w, cur, torch.float64)[-1].argmax()))
        assert s.token_ids == cur


def test_side_benchmark_configuration_is_served():
    """The layer-like configuration of `bench.py --design bevovik` (scaled down) is a valid model of this design:
    it builds with random weights and generates through the engine."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from benchmarks.design_bench import _bevovik_cfg
    from gllm_b200.engine.llm_engine import LLM
    cfg = _bevovik_cfg(256, 1, 97)
    assert [L["type"] for L in cfg["layers"]] == ["rglru", "gla", "latent_attention", "rglru"]
    r = cfg["layers"][0]["mlp"]["router"]
    assert (r["experts"] + r["identity"]) % r["groups"]["count"] == 0
    cfg["torch_dtype"] = "float32"
    llm = LLM(cfg, load_format="dummy", page_size=4, maxp=16, maxd=4, num_cpu_pages=32, model_max_length=64,
              log_stats=False, device="cpu", num_state_slots=2)
    seqs = llm.generate(tokens=[toks(9, 97, 1), toks(4, 97, 2)], output_lens=[3, 2], temperature=0.0, top_k=1)
    assert [len(s.token_ids) for s in seqs] == [12, 6]
