"""Notadra through the engine (scheduler bookkeeping, page / state-slot managers, batch builder, runner) against the
plain oracle in notadra_oracle.py: mechanisms alone, chunking, batching, re-use of pages and slots, far keys and page
borders, the carried previous token, router corner cases, shared keys and values, degenerate sizes, greedy
generation. Runs on the CPU path in fp32; test_notadra_gpu.py repeats the scenarios on the kernels."""
import math

import numpy as np
import pytest
import torch

import notadra_oracle as oracle
import notadra_util as U

TOL = 2e-4
EPS = 1e-5


def toks(n, vocab, seed):
    return torch.randint(0, vocab, (n,), generator=torch.Generator().manual_seed(seed)).tolist()


CONFIGS = {
    # own keys in 0 and 1; 2 and 4 read layer 0, 3 reads layer 1; a layer without feed-forward; unequal head counts
    "mixed": U.make_config([U.attn(mlp=U.moe()), U.attn(heads=2, kv_heads=1, dim=6, vdim=10, rot_dims=6, mlp=None),
                            U.attn(kv_from=0, mlp=U.moe(experts=8, top=3, groups=(4, 2))),
                            U.attn(heads=2, kv_heads=1, dim=6, vdim=10, rot_dims=6, kv_from=1,
                                   mlp=U.moe(experts=5, top=2, groups=None)),
                            U.attn(kv_from=0, softcap=50.0, scale=0.2, mlp=None)]),
    "own_only": U.make_config([U.attn(heads=3, kv_heads=3, dim=4, vdim=4, rot_dims=2, scaling=None, mlp=U.moe()),
                               U.attn(heads=6, kv_heads=2, dim=10, vdim=3, rot_dims=10,
                                      mlp=U.moe(top=4, groups=(2, 2)))],
                              bigram=(7, 1000003, 999983), logit_scale=1.0),
    # sizes of one, values that other models make equal or 1
    "ones": U.make_config([U.attn(heads=1, kv_heads=1, dim=2, vdim=1, rot_dims=2, scale=1.0, softcap=1.0,
                                  scaling={"factor": 1.0, "original": 8, "fast": 2.0, "slow": 1.0},
                                  mlp=U.moe(experts=1, top=1, ff=1, groups=(1, 1))),
                           U.attn(heads=2, kv_heads=2, dim=2, vdim=2, rot_dims=2, kv_from=None,
                                  mlp=U.moe(experts=2, top=2, ff=3, groups=(2, 2))),
                           U.attn(heads=1, kv_heads=1, dim=2, vdim=1, rot_dims=2, scale=1.0, softcap=1.0,
                                  scaling={"factor": 1.0, "original": 8, "fast": 2.0, "slow": 1.0}, kv_from=0,
                                  mlp=U.moe(experts=4, top=1, ff=2, groups=(4, 1)))],
                          width=8, vocab=17, bigram=(1, 3, 2), logit_scale=2.5),
}


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=80 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


# -- each mechanism alone, against its own oracle function -----------------------------------------------------
def test_norm_gain_is_one_plus_the_stored_weight():
    from gllm_b200.layers import functional as Fn
    g = torch.Generator().manual_seed(1)
    x = torch.randn(5, 12, generator=g) * 3
    y = torch.randn(5, 12, generator=g)
    w_post, w_pre = torch.randn(12, generator=g) * 0.3, torch.randn(12, generator=g) * 0.3
    x2 = x.clone()
    h = Fn.resid_norm(x2, y, w_post, None, w_pre, EPS, torch.float32, False, None, 1.0)
    want_x = x.double() + oracle.norm(y.double(), w_post, EPS)
    assert torch.allclose(x2.double(), want_x, atol=1e-5)
    assert torch.allclose(h.double(), oracle.norm(want_x, w_pre, EPS), atol=1e-5)
    # a weight of zero is the plain RMS norm, not a zero output
    h0 = Fn.resid_norm(x.clone(), None, None, None, torch.zeros(12), EPS, torch.float32, False, None, 1.0)
    assert torch.allclose(h0.double(), oracle.rms(x.double(), EPS), atol=1e-5)


class _Inp:
    def __init__(self, tokens, positions, qsl, slots):
        self.tokens = torch.tensor(tokens, dtype=torch.int32)
        self.positions = torch.tensor(positions, dtype=torch.int32)
        self.query_start_loc = torch.tensor(qsl, dtype=torch.int32)
        self.rec_slots = torch.tensor(slots, dtype=torch.int32)


def test_pair_embedding_rows_and_carried_token():
    from gllm_b200.layers import functional as Fn
    g = torch.Generator().manual_seed(2)
    vocab, width = 50, 6
    for buckets, a, b in ((11, 7, 3), (1, 5, 9), (13, 2 ** 31 - 1, 2 ** 31 - 19), (4, 0, 1)):
        cfg = {"embedding": {"bigram": {"buckets": buckets, "mul_prev": a, "mul_cur": b}}}
        wt = {"embed": torch.randn(vocab, width, generator=g), "bigram": torch.randn(buckets + 1, width, generator=g)}
        s0, s1 = toks(9, vocab, 3), toks(5, vocab, 4)
        want0, want1 = oracle.embed(s0, wt, cfg).float(), oracle.embed(s1, wt, cfg).float()
        state = torch.full((3,), 7, dtype=torch.int32)         # stale contents of earlier sequences
        # step 1: s0[:4] in slot 2 beside s1[:1] in slot 0; step 2: one token of each; step 3: the rest
        plan = [((0, 4), (0, 1)), ((4, 5), (1, 2)), ((5, 9), (2, 5))]
        got0, got1 = [], []
        for (a0, b0), (a1, b1) in plan:
            inp = _Inp(s0[a0:b0] + s1[a1:b1], list(range(a0, b0)) + list(range(a1, b1)),
                       [0, b0 - a0, b0 - a0 + b1 - a1], [2, 0])
            x = Fn.embedding_pair_hash(inp, wt["embed"], wt["bigram"], a, b, buckets, state)
            got0.append(x[:b0 - a0])
            got1.append(x[b0 - a0:])
        assert torch.allclose(torch.cat(got0), want0, atol=1e-6), (buckets, a, b)
        assert torch.allclose(torch.cat(got1), want1, atol=1e-6), (buckets, a, b)
        assert state.tolist() == [s1[-1], 7, s0[-1]]


def test_rotary_frequencies_and_rotation():
    """The scaled frequency per pair, the clamps of the ramp at both ends, no scaling, and the half-split pair layout
    with entries beyond the rotated ones passing through, also far out."""
    from gllm_b200.ops import ref
    cases = [(16, 30000.0, None), (8, 100.0, U.YARN), (32, 10000.0, {"factor": 6.0, "original": 64, "fast": 24.0,
                                                                     "slow": 1.0}),
             (4, 10.0, {"factor": 2.0, "original": 4, "fast": 1000.0, "slow": 0.001}),
             (6, 500.0, {"factor": 1.0, "original": 100, "fast": 4.0, "slow": 2.0}),
             (12, 1000.0, {"factor": 40.0, "original": 4096, "fast": 1.0, "slow": 1.0})]
    pos = torch.tensor([0, 1, 2, 17, 1000, 70001], dtype=torch.int32)
    for dims, base, sc in cases:
        rot = {"dims": dims, "base": base}
        if sc:
            rot["scaling"] = sc
        cos, sin = oracle.rotary_table(rot, 70002)
        f, mag = ref.pair_rotary_frequencies(dims, base, sc, dtype=torch.float64)
        x = torch.randn(6, 3, dims + 5, generator=torch.Generator().manual_seed(dims))
        got = ref.rotate_half_pairs(x, pos, dims, base, f, mag)
        want = oracle.rotate(x.double(), cos[pos.long()], sin[pos.long()])
        assert torch.allclose(got.double(), want, atol=2e-5), (dims, base, sc)
        assert torch.equal(got[..., dims:], x[..., dims:])
    # by hand: dims 8, base 100, factor 4, original 16, fast 8, slow 1
    where = lambda t: 8 * math.log(16 / (2 * math.pi * t)) / (2 * math.log(100.0))      # noqa: E731
    lo, hi = max(math.floor(where(8.0)), 0), min(math.ceil(where(1.0)), 7)
    f, mag = ref.pair_rotary_frequencies(8, 100.0, U.YARN, dtype=torch.float64)
    for i in range(4):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        fi = 100.0 ** (-2 * i / 8)
        assert abs(float(f[i]) - (fi / 4 * ramp + fi * (1 - ramp))) < 1e-12
    assert abs(mag - (0.1 * math.log(4.0) + 1)) < 1e-12


def _attention_alone(layer_cfg, seed, n=19, cuts=((19,), (7, 1, 1, 2, 8), (2,) * 9 + (1,), (1,) * 19), page_size=4,
                     width=20, device="cpu", dtype=torch.float32, tol=2e-4):
    cfg = U.make_config([layer_cfg], width=width)
    w = U.random_weights(cfg, seed)
    m = U.build_mixer(layer_cfg, w, width, device, dtype)
    h = torch.randn(n, width, generator=torch.Generator().manual_seed(seed))
    if dtype == torch.bfloat16:
        h = h.bfloat16().float()
    want = U.oracle_mixer(h.double(), layer_cfg, w).float()
    for cut in cuts:
        got = U.drive_mixers([m], [m.cache_entry()], [h], cut, page_size, device, dtype)[0]
        assert torch.allclose(got, want, atol=tol * (1 + want.abs().max().item()), rtol=tol), cut


def test_attention_mixer_alone():
    _attention_alone(U.attn(), 1)
    _attention_alone(U.attn(heads=1, kv_heads=1, dim=4, vdim=9, rot_dims=2, scaling=None), 2, page_size=8)
    _attention_alone(U.attn(heads=6, kv_heads=3, dim=6, vdim=2, rot_dims=6, softcap=0.7, scale=1.3,
                            scaling={"factor": 16.0, "original": 6, "fast": 3.0, "slow": 0.5}), 3, page_size=16)
    _attention_alone(U.attn(heads=8, kv_heads=1, dim=12, vdim=12, rot_dims=8, softcap=30.0), 4)


def test_score_cap_and_unit_sink_show():
    """Queries scaled up so that raw scores pass the cap by far: leaving the cap out would give a one-hot softmax.
    Queries scaled to nothing: all scores are 0 and position i weighs each of its i + 1 values by 1 / (i + 2)."""
    layer = U.attn(heads=2, kv_heads=1, dim=8, vdim=5, rot_dims=4, softcap=2.0, scale=1.0)
    cfg = U.make_config([layer])
    w = U.random_weights(cfg, 5)
    w["l0.mix.q"] *= 16
    n = 13
    h = torch.randn(n, 20, generator=torch.Generator().manual_seed(5))
    want = U.oracle_mixer(h.double(), layer, w).float()
    uncapped = dict(layer, mixer=dict(layer["mixer"], softcap=0.0))
    assert (U.oracle_mixer(h.double(), uncapped, w).float() - want).abs().max() > 0.1 * want.abs().max()
    m = U.build_mixer(layer, w, 20)
    for cut in ([n], [5, 1, 7], [1] * n):
        got = U.drive_mixers([m], [m.cache_entry()], [h], cut)[0]
        assert torch.allclose(got, want, atol=2e-4 * (1 + want.abs().max().item())), cut
    w["l0.mix.q"] *= 0
    w["l0.mix.q.b"] *= 0
    m = U.build_mixer(layer, w, 20)
    wd = {k: v.double() for k, v in w.items()}
    _, v = oracle.keys_values(h.double(), layer["mixer"], wd, "l0.mix.")
    mean = torch.cumsum(v[:, 0], 0) / (torch.arange(n, dtype=torch.float64)[:, None] + 2.0)      # the sink's share
    want = (mean.repeat(1, 2) @ wd["l0.mix.o"].T).float()
    for cut in ([n], [1] * n):
        got = U.drive_mixers([m], [m.cache_entry()], [h], cut)[0]
        assert torch.allclose(got, want, atol=2e-4 * (1 + want.abs().max().item())), cut


def test_layer_reads_another_layers_keys_and_values():
    """Two mixers over one cache entry: the second has no key / value tensors and no pages of its own."""
    own = U.attn(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4)
    reader = U.attn(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, kv_from=0, softcap=9.0, scale=0.9)
    cfg = U.make_config([own, reader])
    w = U.random_weights(cfg, 6)
    assert "l1.mix.k" not in w and "l1.mix.v.b" not in w
    m0, m1 = U.build_mixer(own, w, 20), U.build_mixer(reader, w, 20, pre="l1.mix.")
    assert m1.in_w.shape[0] == 4 * 8 and m1.cache_entry() == {"kind": "shared", "layer": 0}
    g = torch.Generator().manual_seed(6)
    n = 21
    h0, h1 = torch.randn(n, 20, generator=g), torch.randn(n, 20, generator=g)
    wd = {k: v.double() for k, v in w.items()}
    kv = oracle.keys_values(h0.double(), own["mixer"], wd, "l0.mix.")
    want0 = oracle.attention(h0.double(), own["mixer"], wd, "l0.mix.", kv).float()
    want1 = oracle.attention(h1.double(), reader["mixer"], wd, "l1.mix.", kv).float()
    layout = [m0.cache_entry(), {"kind": "shared", "source": 0}]
    for cut in ([n], [6, 1, 1, 2, 11], [2] * 10 + [1], [1] * n):
        got0, got1 = U.drive_mixers([m0, m1], layout, [h0, h1], cut)
        assert torch.allclose(got0, want0, atol=2e-4 * (1 + want0.abs().max().item())), cut
        assert torch.allclose(got1, want1, atol=2e-4 * (1 + want1.abs().max().item())), cut


def test_shared_pages_are_the_source_layers_storage(models):
    cfg, w, path = models["mixed"]
    s = U.session(path)
    c = s.runner.kv_cache
    assert c.k_cache[2] is c.k_cache[0] and c.v_cache[4] is c.v_cache[0] and c.k_cache[3] is c.k_cache[1]
    assert c.k_cache[1] is not c.k_cache[0] and c.token_state is not None
    from gllm_b200.memory_manager import HybridCache
    own = HybridCache.bytes_per_page(s.runner.model.cache_layout(), 4, 4)
    assert own == 4 * 4 * (2 * (8 + 6) + 1 * (6 + 10))          # layers 0 and 1 only


def test_router_corner_cases():
    from gllm_b200.ops import ref
    h = torch.eye(8)

    def both(logits, corr, top, cnt, keep):
        wr = torch.log(torch.tensor(logits) / (1 - torch.tensor(logits))).t().contiguous()      # sigmoid^-1
        wt = {"r.router": wr.double(), "r.correction": torch.tensor(corr).double()}
        n = wr.shape[0]
        r = {"experts": n, "top": top, "groups": {"count": cnt, "keep": keep}}
        ids, ws = oracle.route(torch.eye(wr.shape[1], dtype=torch.float64)[:1], r, wt, "r.")
        gw, gi = ref.grouped_router(torch.eye(wr.shape[1])[:1], wr, torch.tensor(corr), top, cnt, keep, 1.0,
                                    "sigmoid", 2, False)
        assert gi[0].tolist() == ids[0], (gi, ids)
        assert np.allclose(gw[0].numpy(), ws[0], atol=1e-6)
        return ids[0], ws[0]

    # the group with the single best expert loses to the group with the better pair
    ids, ws = both([[0.9, 0.1, 0.6, 0.55]], [0.0] * 4, 2, 2, 1)
    assert ids == [2, 3] and abs(ws[0] - 0.6) < 1e-6
    # corrections decide the choice and stay out of the weights; choice scores may be negative: a barred group
    # counts as minus infinity, so negative eligible experts still beat it
    ids, ws = both([[0.2, 0.3, 0.9, 0.8]], [-1.0, -1.0, -3.0, -3.0], 2, 2, 1)
    assert ids == [1, 0] and abs(ws[0] - 0.3) < 1e-6 and abs(ws[1] - 0.2) < 1e-6
    # all groups kept, one group, one expert per group, weights are not renormalised
    ids, ws = both([[0.5, 0.7, 0.6, 0.1]], [0.0] * 4, 3, 2, 2)
    assert ids == [1, 2, 0] and abs(sum(ws) - 1.8) < 1e-6
    both([[0.5, 0.7, 0.6, 0.1]], [0.1, 0.0, 0.3, 0.0], 2, 1, 1)
    ids, _ = both([[0.5, 0.7, 0.6, 0.1]], [0.0] * 4, 2, 4, 2)
    assert ids == [1, 2]
    # the whole of the kept groups is taken
    ids, _ = both([[0.5, 0.1, 0.2, 0.3, 0.45, 0.44]], [0.0] * 6, 4, 3, 2)
    assert sorted(ids) == [0, 1, 4, 5]
    del h


def test_feed_forward_alone():
    g = torch.Generator().manual_seed(7)
    for mlp, width in ((U.moe(), 20), (U.moe(experts=10, top=3, ff=5, groups=(2, 1)), 12),
                       (U.moe(experts=3, top=3, ff=7, groups=None), 9),
                       (U.moe(experts=4, top=1, ff=2, groups=(4, 3)), 8)):
        cfg = U.make_config([U.attn(mlp=mlp)], width=width)
        w = U.random_weights(cfg, 7)
        f = U.build_ff(mlp, w, width)
        h = torch.randn(33, width, generator=g)
        want = oracle.moe(h.double(), mlp, {k: v.double() for k, v in w.items()}, "l0.mlp.").float()
        assert torch.allclose(f(h), want, atol=2e-4 * (1 + want.abs().max().item()))


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
    oracle.forward(cfg, w, t, trace)
    s = U.session(path)
    s.runner.model.trace = []
    s.step([{"id": "a", "tokens": t, "want": []}], ["a"])
    got = s.runner.model.trace
    assert len(got) == len(trace) == len(cfg["layers"])
    for a, b in zip(got, trace):
        assert torch.allclose(a.double(), b, atol=1e-4)


@pytest.mark.parametrize("name", list(CONFIGS))
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
    """One slot, a pool of two requests' size: the second request finds the first one's last token in its slot and
    the first one's keys in its pages."""
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
    # the first token's row of the pair table is the last one, whatever the token
    x = oracle.embed([5], {"embed": torch.zeros(61, 20), "bigram": w["bigram"]}, cfg)
    assert torch.equal(x[0].float(), w["bigram"][-1])


def test_previous_token_is_carried_between_steps(models):
    """Two requests that differ in one token only: the logits of the token AFTER it differ too when that token
    starts a new portion (the hashed pair reaches back over the cut), and match the oracle."""
    cfg, w, path = models["own_only"]
    a = toks(12, cfg["vocab"], 10)
    b = list(a)
    b[6] = (a[6] + 1) % cfg["vocab"]
    s = U.session(path)
    for t in (a, b):
        got = U.run_chunks(s, "r", t, [7, 1, 4])
        assert U.rel_err(got, U.expected_logits(cfg, w, t)) < TOL


# -- edges that random weights would hide ----------------------------------------------------------------------
def far_key_probe(n, back, page_size, device="cpu", dtype=torch.float32, heads=2, dim=32, vdim=4):
    """Attention whose query map is its key map after a permutation of the input (no biases, nothing rotated in the
    scores' part: the rotated entries' rows are zero), orthogonal key maps, unit-length inputs and a large scale
    under a cap far above it: a query then picks out the key made from the permuted input. The last token's input is
    the permuted input of the token `back` places before it (back = 0: nothing is marked), all other inputs are
    random. -> (oracle, outputs for several ways of cutting, the oracle with the marked token's input replaced)."""
    g = torch.Generator().manual_seed(back * 7 + page_size)
    width, rot = dim, 2
    layer = U.attn(heads=heads, kv_heads=heads, dim=dim, vdim=vdim, rot_dims=rot, scale=60.0, softcap=600.0,
                   scaling=None)
    cfg = U.make_config([layer], width=width)
    w = U.random_weights(cfg, 99)
    wk = torch.cat([torch.linalg.qr(torch.randn(dim, dim, generator=g))[0] for _ in range(heads)], 0)
    wk = wk.reshape(heads, dim, width)
    wk[:, :rot] = 0                                             # the rotated entries stay out of the scores
    wk = wk.reshape(heads * dim, width)
    perm = torch.roll(torch.arange(width), 5)                  # query(h) = key(h') with h'[perm] = h
    w["l0.mix.k"] = wk
    w["l0.mix.q"] = wk[:, perm].clone()
    w["l0.mix.q.b"] = torch.zeros(heads * dim)
    w["l0.mix.k.b"] = torch.zeros(heads * dim)
    m = U.build_mixer(layer, w, width, device, dtype)
    h = torch.randn(n, width, generator=g)
    h = h / h.norm(dim=-1, keepdim=True)
    tgt = n - 1 - back
    h[n - 1] = h[tgt][perm]                                    # the last query equals the marked token's key
    want = U.oracle_mixer(h.double(), layer, w).float()
    h2 = h.clone()
    if back > 0:
        x = torch.randn(width, generator=g)
        h2[tgt] = x / x.norm()
    other = U.oracle_mixer(h2.double(), layer, w).float()
    cuts = [[n], [n - 1, 1], [n - back - 1, 1] + [back] * (back > 0), [max(n - 40, 1)] + [2] * 19]
    outs = []
    for c in cuts:
        c = [x for x in c if x > 0]
        rest = n - sum(c)
        assert rest >= 0
        outs.append(U.drive_mixers([m], [m.cache_entry()], [h], c + [1] * rest, page_size, device, dtype,
                                   pool=1024)[0])
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


def test_far_positions_keep_their_angles(models):
    """Long decoding after a long prompt: positions in the hundreds through the scaled frequencies."""
    cfg, w, path = models["own_only"]
    t = toks(260, cfg["vocab"], 11)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path, max_tokens=512, page_size=16)
    got = U.run_chunks(s, "a", t, [200, 3, 2])
    assert U.rel_err(got[190:], want[190:]) < TOL


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
            cur.append(int(oracle.forward(cfg, w, cur)[-1].argmax()))
        assert s.token_ids == cur


def test_side_benchmark_configuration_is_served():
    """The layer-like configuration of `bench.py --design notadra` (scaled down) is a valid model of this design:
    it builds with random weights and generates through the engine."""
    import os
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    from benchmarks.design_bench import _notadra_cfg
    from gllm_b200.engine.llm_engine import LLM
    cfg = _notadra_cfg(256, 4, 97)
    assert [L["mixer"].get("kv_from") for L in cfg["layers"]] == [None, 0, None, 2]
    r = cfg["layers"][0]["mlp"]["router"]
    assert r["experts"] % r["groups"]["count"] == 0
    cfg["torch_dtype"] = "float32"
    llm = LLM(cfg, load_format="dummy", page_size=4, maxp=16, maxd=4, num_cpu_pages=32, model_max_length=64,
              log_stats=False, device="cpu", num_state_slots=2)
    seqs = llm.generate(tokens=[toks(9, 97, 1), toks(4, 97, 2)], output_lens=[3, 2], temperature=0.0, top_k=1)
    assert [len(s.token_ids) for s in seqs] == [12, 6]
