"""Notadra on the sm_100a kernels: the kernels this design added or extended (pair-hash embedding, norm gain offset,
biased products, rotary write with a frequency table, capped scores with a unit sink in the plain and tensor-core
paged attention, the sigmoid / top-2-group router, squared-ReLU experts, scaled logits) against their unfused PyTorch
forms, the mixers alone against the plain oracle, and the engine scenarios of test_notadra_cpu.py (portions, mixed
batches, page / slot re-use, far keys, generation with CUDA graphs) in fp32 (tight) and bf16 (rounding-sized
tolerance)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import notadra_oracle as oracle
import notadra_util as U
from test_notadra_cpu import CONFIGS, _attention_alone, far_key_probe, toks

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL32 = 2e-4


class Expect:
    """What a run is held to. fp32: the oracle, tightly. bf16: the error that rounding alone causes is measured by
    running the unfused PyTorch forms on the CPU with the same rounding points (bf16 weights, activations and cache,
    fp32 accumulation); the kernels may be at most twice as far from the oracle on the median row. A router's close
    call can flip under one bf16 rounding in these tiny sizes and move every later row on either device, so the
    worst row is held only in models without a choice."""

    def __init__(self, cfg, w, path, tokens, dtype):
        self.want = U.expected_logits(cfg, w, tokens)
        self.dtype = dtype
        self.routed = any(L["mlp"] and L["mlp"]["router"]["top"] < L["mlp"]["router"]["experts"]
                          for L in cfg["layers"])
        if dtype == "bfloat16":
            s = U.session(path, "bfloat16", "cpu", max_tokens=max(256, len(tokens) + 64), page_size=16)
            got = s.step([{"id": "r", "tokens": tokens, "want": list(range(len(tokens)))}], ["r"])
            self.noise = U.row_errs(got, self.want)

    def check(self, got):
        e = U.row_errs(got, self.want)
        if self.dtype == "float32":
            assert e.max() < TOL32, e.max()
        elif self.routed:
            assert np.median(e) < max(2 * np.median(self.noise), 0.25), (np.median(e), np.median(self.noise))
        else:
            assert np.median(e) <= 2 * np.median(self.noise) + 1e-2
            assert e.max() <= 2 * self.noise.max() + 2e-2


def close(a, b, tol):
    return (a.float() - b.float()).abs().max().item() <= tol * (b.float().abs().max().item() + 1e-9)


def _batch(qlens, ctx, ps, pages):
    """Batch metadata of unequal requests (context `ctx` + `qlens` new tokens each) on random pages; single-token
    requests come first, as the scheduler orders them."""
    qsl = torch.tensor([0] + np.cumsum(qlens).tolist(), dtype=torch.int32, device=DEV)
    sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
    per = max((c + q + ps - 1) // ps for c, q in zip(ctx, qlens))
    bt = torch.randperm(pages - 1)[: len(qlens) * per].reshape(len(qlens), per).to(torch.int32).to(DEV)
    pos = torch.cat([torch.arange(c, c + q) for c, q in zip(ctx, qlens)]).to(torch.int32).to(DEV)
    seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(DEV)
    slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
    ndec = 0
    for q in qlens:
        if q != 1:
            break
        ndec += 1
    return SimpleNamespace(query_start_loc=qsl, seq_lens=sl, block_table=bt, positions=pos, slot_mapping=slots,
                           max_q_len=max(qlens), num_decode_seqs=ndec, num_seqs=len(qlens), padded_tokens=0,
                           rec_slots=torch.randperm(len(qlens) + 3)[: len(qlens)].to(torch.int32).to(DEV))


# -- kernels against their unfused forms ---------------------------------------------------------------------------
@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
def test_stream_norm_offset_scale_and_bias(dt, tol):
    from gllm_b200.ops import ref, sm100_seq as K
    torch.manual_seed(1)
    for T, width in ((1, 8), (37, 100), (300, 1024)):
        x = torch.randn(T, width, device=DEV) * 3
        y = torch.randn(T, width + 8, device=DEV).to(dt)[:, :width]
        wp, wq = (torch.randn(width, device=DEV) * 0.3).to(dt), (torch.randn(width, device=DEV) * 0.3).to(dt)
        x1, x2 = x.clone(), x.clone()
        o1 = K.resid_norm(x1, y, wp, None, wq, 1e-5, dt, False, None, 1.0)
        o2 = ref.resid_norm(x2, y, wp, None, wq, 1e-5, dt, False, None, 1.0)
        assert close(x1, x2, 1e-5) and close(o1, o2, tol), (T, width)
    for m, k, n in ((5, 20, 36), (130, 64, 72), (64, 256, 1792), (3, 100, 7)):
        a = torch.randn(m, k, device=DEV).to(dt)
        w = (torch.randn(n, k, device=DEV) * k ** -0.5).to(dt)
        b = torch.randn(n, device=DEV).to(dt)
        want = (a.float() @ w.float().t() + b.float())
        assert close(K.linear_any(a, w, b), want, tol), (m, k, n)
        assert close(K.gemm_simt(a, w, b), want, tol), (m, k, n)
    x = torch.randn(9, 50, device=DEV)
    wq = (torch.randn(50, device=DEV) * 0.3).to(dt)
    o1 = K.resid_norm(x.clone(), None, None, None, wq, 1e-5, dt, False, None, 1.0, 0.37)          # scaled final norm
    assert close(o1, ref.resid_norm(x.clone(), None, None, None, wq, 1e-5, dt, False, None, 1.0, 0.37), tol)


@pytest.mark.parametrize("dt", [torch.float32, torch.bfloat16])
def test_pair_embedding_on_the_device(dt):
    from gllm_b200.ops import ref, sm100_pair as P
    torch.manual_seed(2)
    vocab, width = 300, 40
    for buckets, a, b in ((11, 7, 3), (1, 5, 9), (499, 2 ** 31 - 1, 2 ** 31 - 19), (4, 0, 1)):
        table = torch.randn(vocab, width, device=DEV).to(dt)
        pair = torch.randn(buckets + 1, width, device=DEV).to(dt)
        for qlens, ctx in (([1, 1, 5, 9], [4, 0, 0, 17]), ([7], [0]), ([1, 1, 1], [3, 9, 0]),
                           ([2, 2, 64], [5, 0, 100])):
            bt = _batch(qlens, ctx, 4, 2 + len(qlens) * max((c + q + 3) // 4 for c, q in zip(ctx, qlens)))
            T = int(bt.query_start_loc[-1])
            ids = torch.randint(0, vocab, (T,), dtype=torch.int32, device=DEV)
            st1 = torch.randint(0, vocab, (len(qlens) + 3,), dtype=torch.int32, device=DEV)
            st2 = st1.clone().cpu()
            got = P.embedding_pair_hash(ids, table, pair, a, b, buckets, bt.positions, st1, bt.rec_slots,
                                        bt.query_start_loc)
            want = ref.embedding_pair_hash(ids.cpu(), table.cpu(), pair.cpu(), a, b, buckets, bt.positions.cpu(), st2,
                                           bt.rec_slots.cpu(), bt.query_start_loc.cpu())
            assert torch.equal(got.cpu(), want), (buckets, qlens)
            assert torch.equal(st1.cpu(), st2)


def _attn_case(dt, heads, kvh, dim, vdim, rot, qlens, ctx, ps, softcap, scaling, own=True):
    """bias-free projection rows -> rotary write (frequency table) -> attention with cap and unit sink, on a mixed
    batch whose earlier tokens are already cached; -> (kernel results, unfused results)."""
    from gllm_b200.memory_manager import kv_cache_shape
    from gllm_b200.ops import ref, sm100_seq as K
    pages = 2 + len(qlens) * max((c + q + ps - 1) // ps for c, q in zip(ctx, qlens))
    b = _batch(qlens, ctx, ps, pages)
    T = int(b.query_start_loc[-1])
    f, mag = (None, 1.0) if scaling is None else ref.pair_rotary_frequencies(rot, 5000.0, scaling, dtype=torch.float64)
    f = f.to(DEV) if f is not None else None
    kc1 = torch.zeros(kv_cache_shape(pages, kvh, dim, ps), dtype=dt, device=DEV)
    vc1 = torch.zeros(kv_cache_shape(pages, kvh, vdim, ps), dtype=dt, device=DEV)
    n_in = heads * dim + kvh * (dim + vdim)
    for s, c in enumerate(ctx):               # the context rows, written through the unfused form
        if c:
            pos = torch.arange(c, device=DEV, dtype=torch.int32)
            sl = (b.block_table[s, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
            ref.qk_norm_rope_kv_write(torch.randn(c, n_in, device=DEV).to(dt), heads, kvh, dim, vdim, None, None, 1e-5,
                                      pos, rot, 5000.0, kc1, vc1, sl, f, mag)
    kc2, vc2 = kc1.clone(), vc1.clone()
    qkv = torch.randn(T, n_in + 8, device=DEV).to(dt)[:, :n_in]
    g = kvh if own else 0
    rows = qkv if own else qkv[:, :heads * dim]
    q1 = K.qk_norm_rope_kv_write(rows, heads, g, dim, vdim, None, None, 1e-5, b.positions, rot, 5000.0, kc1, vc1,
                                 b.slot_mapping, f, mag)
    q2 = ref.qk_norm_rope_kv_write(rows, heads, g, dim, vdim, None, None, 1e-5, b.positions, rot, 5000.0, kc2, vc2,
                                   b.slot_mapping, f, mag)
    sink = torch.zeros(heads, dtype=torch.float32, device=DEV)
    scale = dim ** -0.5 * 2.0
    o1 = K.window_attention(q1, kc1, vc1, b.block_table, b.seq_lens, b.query_start_loc, b.positions, scale, heads, dim,
                            None, sink, num_decode_seqs=b.num_decode_seqs, max_q_len=b.max_q_len, v_dim=vdim,
                            softcap=softcap)
    o2 = ref.window_attention(q2, kc2, vc2, b.block_table, b.seq_lens, b.query_start_loc, scale, heads, dim, None, sink,
                              v_dim=vdim, softcap=softcap)
    o3 = K.window_attention(q1, kc1, vc1, b.block_table, b.seq_lens, b.query_start_loc, b.positions, scale, heads, dim,
                            None, sink, num_decode_seqs=b.num_decode_seqs, max_q_len=b.max_q_len, v_dim=vdim,
                            softcap=softcap, simt=True)
    return (q1, kc1, vc1, o1, o3), (q2, kc2, vc2, o2, o2)


YARN2 = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 1.0}


@pytest.mark.parametrize("dt,tol", [(torch.float32, 5e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,kvh,dim,vdim,rot", [(4, 2, 8, 6, 4), (1, 1, 2, 1, 2), (8, 4, 128, 80, 32),
                                                    (8, 2, 128, 128, 64), (4, 4, 64, 64, 64), (6, 3, 256, 256, 32),
                                                    (6, 2, 64, 64, 16), (3, 1, 128, 128, 128),
                                                    (5, 5, 24, 40, 24)])
def test_rotary_write_and_capped_sink_attention(dt, tol, heads, kvh, dim, vdim, rot):
    """Sizes that take the plain kernel (values narrower than keys, fp32) and sizes that take the tensor-core
    kernels (bf16, equal widths of 64 / 128 / 256); decode rows beside prompt portions; the capped scores reach
    well into the flat part of the cap."""
    torch.manual_seed(5)
    for qlens, ctx, ps, cap, sc in (([1, 1, 9, 3], [35, 16, 0, 2], 16, 3.0, YARN2),
                                    ([1, 70, 33], [200, 0, 31], 16, 30.0, None),
                                    ([1, 1, 1], [0, 77, 15], 8, 1.5, YARN2),
                                    ([1, 40, 150], [5, 0, 130], 16, 0.0, None)):          # sink without a cap
        got, want = _attn_case(dt, heads, kvh, dim, vdim, rot, qlens, ctx, ps, cap, sc)
        for g, w, name in zip(got, want, ("queries", "keys", "values", "attention", "attention (plain)")):
            assert close(g, w, tol), (name, qlens)
    got, want = _attn_case(dt, heads, kvh, dim, vdim, rot, [1, 12], [9, 3], 16, 4.0, YARN2, own=False)
    assert close(got[0], want[0], tol) and torch.equal(got[1], want[1]) and close(got[3], want[3], tol)


def test_router_on_the_device():
    from gllm_b200.ops import ref, sm100_latent as K
    torch.manual_seed(7)
    for n, top, cnt, keep, corr_std, width, T in ((6, 2, 3, 2, 0.3, 20, 33), (14, 3, 2, 1, 0.5, 192, 700),
                                                  (8, 8, 1, 1, 0.0, 16, 9), (4, 1, 4, 1, 2.0, 8, 5),
                                                  (64, 6, 8, 3, 0.05, 64, 300), (256, 8, 8, 4, 0.01, 128, 64),
                                                  (1, 1, 1, 1, 0.0, 8, 3), (10, 4, 5, 2, 3.0, 32, 40)):
        for dt in (torch.float32, torch.bfloat16):
            h = torch.randn(T, width, device=DEV).to(dt)
            w = (torch.randn(n, width, device=DEV) * 3 * width ** -0.5).to(dt)
            corr = torch.randn(n, device=DEV) * corr_std - (1.0 if corr_std > 1 else 0.0)     # also negative choices
            w1, i1 = K.grouped_router(h, w, corr, top, cnt, keep, 1.0, "sigmoid", 2, False)
            w2, i2 = ref.grouped_router(h, w, corr, top, cnt, keep, 1.0, "sigmoid", 2, False)
            same = (i1 == i2).all(-1)
            assert same.float().mean() > 0.98, (n, top, cnt, keep)        # a close call may flip on summation order
            assert torch.allclose(w1[same], w2[same], atol=2e-5)
            assert (w1 <= 1).all() and not torch.allclose(w1.sum(-1), torch.ones(T, device=DEV))


def test_squared_relu_experts_grouped_against_plain():
    from gllm_b200.ops import ref, sm100_pair as P
    torch.manual_seed(6)
    for T, width, ff, n, top in ((1, 128, 64, 4, 2), (77, 256, 192, 6, 3), (400, 128, 128, 3, 2), (33, 256, 64, 12, 3),
                                 (50, 72, 40, 5, 2)):
        dt = torch.bfloat16
        h = torch.randn(T, width, device=DEV).to(dt)
        w1 = (torch.randn(n, ff, width, device=DEV) * width ** -0.5 * 2).to(dt)
        w2 = (torch.randn(n, width, ff, device=DEV) * ff ** -0.5).to(dt)
        ids = torch.stack([torch.randperm(n)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
        wts = torch.rand(T, top, device=DEV)
        want = ref.routed_relu2_experts(h, w1, w2, wts, ids)
        assert close(P.routed_relu2_experts(h, w1, w2, wts, ids, False), want, 2e-2), (T, width, ff)
        assert close(P.routed_relu2_experts(h, w1, w2, wts, ids, True), want, 2e-2), (T, width, ff)
        h32, a, b = h.float(), w1.float(), w2.float()
        assert close(P.routed_relu2_experts(h32, a, b, wts, ids, False), ref.routed_relu2_experts(h32, a, b, wts, ids),
                     5e-5)


# -- mixers alone and the engine -----------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 4e-2)])
def test_attention_mixer_alone_on_the_device(dtype, tol):
    _attention_alone(U.attn(), 1, device=DEV, dtype=dtype, tol=tol)
    _attention_alone(U.attn(heads=6, kv_heads=3, dim=6, vdim=2, rot_dims=6, softcap=0.7, scale=1.3,
                            scaling={"factor": 16.0, "original": 6, "fast": 3.0, "slow": 0.5}), 3, page_size=16,
                     device=DEV, dtype=dtype, tol=tol)
    _attention_alone(U.attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, softcap=30.0, scale=0.125), 4,
                     page_size=16, width=64, device=DEV, dtype=dtype, tol=tol)


@pytest.mark.parametrize("page_size", [4, 16])
def test_far_keys_and_page_borders_on_the_device(page_size):
    n = 331
    for back in (0, 1, page_size - 1, page_size, page_size + 1, 64, 65, 200, 330):
        want, outs, other = far_key_probe(n, back, page_size, device=DEV)
        if back > 0:
            assert (want[-1] - other[-1]).abs().max() > 0.05 * want[-1].abs().max(), back
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4 * want.abs().max().item(), rtol=2e-4), (page_size, back)


@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=80 + i)
        out[name] = (cfg, w, U.save_model(cfg, w))
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_whole_prompt_decoding_and_portions(models, name, dtype):
    cfg, w, path = models[name]
    t = toks(45, cfg["vocab"], 2)
    ex = Expect(cfg, w, path, t, dtype)
    s = U.session(path, dtype, DEV)
    ex.check(U.run_chunks(s, "a", t, [len(t)]))
    ex.check(U.run_chunks(s, "b", t, [13]))                    # the rest token by token
    ex.check(U.run_chunks(s, "c", t, []))
    for cuts in ([2, 2, 2, 3, 5], [7, 1, 1, 2, 9, 4, 21], [16, 2], [1, 30], [33, 2, 2]):
        ex.check(U.run_chunks(s, "d", t, cuts))


def test_residual_stream_after_every_layer_on_the_device(models):
    cfg, w, path = models["mixed"]
    t = toks(11, cfg["vocab"], 8)
    trace = []
    oracle.forward(cfg, w, t, trace)
    s = U.session(path, "float32", DEV)
    s.runner.model.trace = []
    s.step([{"id": "a", "tokens": t, "want": []}], ["a"])
    got = s.runner.model.trace
    assert len(got) == len(trace)
    for a, b in zip(got, trace):
        assert torch.allclose(a.double().cpu(), b, atol=1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_mixed_batches_reuse_pages_and_slots(models, dtype):
    cfg, w, path = models["mixed"]
    v = cfg["vocab"]
    reqs = {k: toks(n, v, 20 + i) for i, (k, n) in enumerate([("a", 30), ("b", 9), ("c", 17), ("d", 2), ("e", 26),
                                                              ("f", 12)])}
    s = U.session(path, dtype, DEV, max_tokens=64, page_size=4, state_slots=3)
    plan = [[("a", 11), ("b", 9)], [("a", 1), ("c", 5)], [("a", 2), ("c", 1)], [("c", 11), ("a", 16), ("d", 2)],
            [("e", 3)], [("e", 1), ("f", 12)], [("e", 22)]]
    got = U.run_plan(s, reqs, plan)
    for k, t in reqs.items():
        Expect(cfg, w, path, t, dtype).check(got[k])
    mm = s.scheduler.mm
    assert mm.get_num_free_state_slots() == 3 and mm.get_num_free_pages() == mm.usable_pages
    # a slot and pages with another request's leftovers
    s = U.session(path, dtype, DEV, max_tokens=32, page_size=4, state_slots=1)
    a, b = toks(19, v, 5), toks(7, v, 6)
    U.run_chunks(s, "a", a, [10, 9])
    Expect(cfg, w, path, b, dtype).check(U.run_chunks(s, "b", b, [3, 2, 2]))


def test_long_decoding_on_the_device(models):
    cfg, w, path = models["own_only"]
    t = toks(260, cfg["vocab"], 11)
    want = U.expected_logits(cfg, w, t)
    s = U.session(path, "float32", DEV, max_tokens=512, page_size=16)
    assert U.rel_err(U.run_chunks(s, "a", t, [150, 3, 2]), want) < TOL32


def test_tensor_core_sized_model_in_bf16():
    """Sizes at which every tensor-core path is taken (tcgen05 GEMMs with the bias epilogue, grouped expert GEMMs
    with the squared-ReLU epilogue, the tensor-core paged attention with cap and sink, also over another layer's
    pages), against the oracle with the bf16 CPU run as the measure of rounding."""
    layers = [U.attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=10000.0, scale=0.125, softcap=20.0,
                     mlp=U.moe(experts=8, top=2, ff=128, groups=(4, 2))),
              U.attn(heads=2, kv_heads=2, dim=128, vdim=128, rot_dims=128, base=10000.0, scale=0.09, softcap=30.0,
                     scaling={"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0}, mlp=None),
              U.attn(heads=4, kv_heads=2, dim=64, vdim=64, rot_dims=32, base=10000.0, scale=0.125, softcap=20.0,
                     kv_from=0, mlp=U.moe(experts=6, top=3, ff=64, groups=(2, 1))),
              U.attn(heads=2, kv_heads=2, dim=128, vdim=128, rot_dims=128, base=10000.0, scale=0.09, softcap=30.0,
                     scaling={"factor": 4.0, "original": 128, "fast": 32.0, "slow": 1.0}, kv_from=1, mlp=None)]
    cfg = U.make_config(layers, vocab=512, width=256, bigram=(251, 89, 13))
    w = U.random_weights(cfg, 5)
    path = U.save_model(cfg, w)
    t = toks(300, 512, 4)
    for dtype in ("bfloat16", "float32"):
        ex = Expect(cfg, w, path, t, dtype)
        s = U.session(path, dtype, DEV, max_tokens=1024, page_size=16)
        ex.check(U.run_chunks(s, "a", t, [300]))
        ex.check(U.run_chunks(s, "b", t, [260, 2, 30]))
        ex.check(U.run_chunks(s, "c", t, [31, 257]))


def test_greedy_generation_with_cuda_graphs(models):
    """The engine's own entry point with captured decode steps, against the oracle's greedy continuation in fp32."""
    from gllm_b200.engine.llm_engine import LLM
    cfg, w, path = models["mixed"]
    llm = LLM(path, dtype="float32", page_size=4, maxp=16, maxd=8, num_gpu_pages=64, model_max_length=96,
              log_stats=False, num_state_slots=4, max_cuda_graph_bs=4)
    prompts = [toks(21, cfg["vocab"], 31), toks(3, cfg["vocab"], 32), toks(9, cfg["vocab"], 33)]
    lens = [7, 12, 5]
    seqs = llm.generate(tokens=prompts, output_lens=lens, temperature=0.0, top_k=1)
    assert llm.worker.runner.stats["graph_steps"] > 0
    for p, n, s in zip(prompts, lens, seqs):
        cur = list(p)
        for _ in range(n):
            cur.append(int(oracle.forward(cfg, w, cur)[-1].argmax()))
        assert s.token_ids == cur
