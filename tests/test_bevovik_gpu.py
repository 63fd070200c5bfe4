"""Bevovik on the sm_100a kernels: every kernel of csrc/seq/latent_ops.cu (and the extended stream, convolution,
state and expert kernels) against its unfused PyTorch form, the mixers alone against the plain oracle, and the engine
scenarios of test_bevovik_cpu.py (portions, mixed batches, page / slot re-use, far keys, edges, generation with
CUDA graphs) in fp32 (tight) and bf16 (rounding-sized tolerance)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import bevovik_oracle as oracle
import bevovik_util as U
from test_bevovik_cpu import (CONFIGS, _mixer_alone, _route_case, conv_edge_probe, far_key_probe, far_state_model,
                              toks)

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
        self.routed = any(L["mlp"] and L["mlp"]["router"]["top"] <
                          L["mlp"]["router"]["experts"] + L["mlp"]["router"].get("identity", 0)
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
    """Batch metadata of unequal requests (context `ctx` + `qlens` new tokens each) on random pages."""
    qsl = torch.tensor([0] + np.cumsum(qlens).tolist(), dtype=torch.int32, device=DEV)
    sl = torch.tensor([c + q for c, q in zip(ctx, qlens)], dtype=torch.int32, device=DEV)
    per = max((c + q + ps - 1) // ps for c, q in zip(ctx, qlens))
    bt = torch.randperm(pages - 1)[: len(qlens) * per].reshape(len(qlens), per).to(torch.int32).to(DEV)
    pos = torch.cat([torch.arange(c, c + q) for c, q in zip(ctx, qlens)]).to(torch.int32).to(DEV)
    seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(DEV)
    slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
    return SimpleNamespace(query_start_loc=qsl, seq_lens=sl, block_table=bt, positions=pos, slot_mapping=slots,
                           tok_seq=seqi.to(torch.int32), max_q_len=max(qlens),
                           rec_slots=torch.randperm(len(qlens) + 3)[: len(qlens)].to(torch.int32).to(DEV))


# -- kernels against their unfused forms ---------------------------------------------------------------------------
@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
def test_stream_norm_and_small_kernels(dt, tol):
    from gllm_b200.ops import ref, sm100_latent as K, sm100_seq as S
    torch.manual_seed(0)
    T, W = 37, 200
    # stream update with a layer scale, emitting the stream itself / the final norm
    x = torch.randn(T, W, device=DEV)
    y, w = torch.randn(T, W, device=DEV).to(dt), (torch.rand(W, device=DEV) + 0.5).to(dt)
    ls = torch.randn(W, device=DEV)
    for w_pre, plain in ((None, True), (w, False), (None, False)):
        x1, x2 = x.clone(), x.clone()
        h1 = S.resid_norm(x1, y, w, None, w_pre, 1e-5, dt, plain, ls)
        h2 = ref.resid_norm(x2, y, w, None, w_pre, 1e-5, dt, plain, ls)
        assert close(x1, x2, 1e-5)
        assert (h1 is None) == (h2 is None) and (h1 is None or close(h1, h2, tol))
    # strided-row RMS norm
    big = torch.randn(T, 3 * 70, device=DEV).to(dt)
    wn = (torch.rand(70, device=DEV) + 0.5).to(dt)
    assert close(K.rms_rows(big[:, 70:140], wn, 1e-5), ref.rms_rows(big[:, 70:140], wn, 1e-5), tol)
    assert close(K.rms_rows(big[:, :1], wn[:1], 1e-5), ref.rms_rows(big[:, :1], wn[:1], 1e-5), tol)
    # clamped gated activation
    gu = (torch.randn(T, 2 * 50, device=DEV) * 3).to(dt)
    assert close(K.glu_clamp(gu, 1.25), ref.glu_clamp(gu, 1.25), tol)
    assert close(K.glu_clamp(gu[:, :6], 0.5, 1.0), ref.glu_clamp(gu[:, :6], 0.5, 1.0), tol)
    # block-diagonal and batched products (plain kernels: odd sizes, fp32 result)
    xb, wb = torch.randn(T, 5 * 7, device=DEV).to(dt), torch.randn(5, 11, 7, device=DEV).to(dt)
    assert close(K.block_linear(xb, wb), ref.block_linear(xb, wb), tol)
    assert close(K.block_linear(xb, wb, torch.float32), ref.block_linear(xb, wb, torch.float32), 1e-5)
    a = torch.randn(T, 3, 13, device=DEV).to(dt)[:, :, :9]
    w3 = torch.randn(3, 6, 9, device=DEV).to(dt)
    o1 = torch.zeros(T, 3, 10, device=DEV, dtype=dt)
    o2 = o1.clone()
    K.linear_batched(a, w3, o1[:, :, 2:8])
    ref.linear_batched(a, w3, o2[:, :, 2:8])
    assert close(o1, o2, tol) and float(o1[:, :, :2].abs().max()) == 0


def test_batched_products_on_the_tensor_cores():
    from gllm_b200.ops import ref, sm100_latent as K
    torch.manual_seed(1)
    dt = torch.bfloat16
    for T in (1, 5, 300):
        xb, wb = torch.randn(T, 4 * 64, device=DEV).to(dt), (torch.randn(4, 128, 64, device=DEV) / 8).to(dt)
        assert close(K.block_linear(xb, wb), ref.block_linear(xb, wb), 2e-2)
        q = torch.randn(T, 3, 64 + 16, device=DEV).to(dt)
        w3 = (torch.randn(3, 96, 64, device=DEV) / 8).to(dt)
        o1 = torch.zeros(T, 3, 96 + 16, device=DEV, dtype=dt)
        o2 = o1.clone()
        K.linear_batched(q[:, :, :64], w3, o1[:, :, :96])
        ref.linear_batched(q[:, :, :64], w3, o2[:, :, :96])
        assert close(o1, o2, 2e-2)


def test_products_with_fp32_result_on_the_tensor_cores():
    """bf16 operands, fp32 accumulation AND result: the block-diagonal gate product and the router logits on the
    16-byte-load mma kernel (odd row counts, column counts off the tile, strided batch views), against fp32 matmul of
    the same bf16 values; a row's result does not depend on the rows beside it."""
    from gllm_b200.ops import sm100_latent as K, sm100_seq as S
    torch.manual_seed(11)
    dt = torch.bfloat16
    for T in (1, 17, 300):
        for nb, n, k in ((4, 128, 64), (3, 40, 32), (1, 264, 96)):
            x = torch.randn(T, nb * k, device=DEV).to(dt)
            w = (torch.randn(nb, n, k, device=DEV) / k ** 0.5).to(dt)
            assert S.mma_f32out_ok(x.view(T, nb, k), w)
            got = K.block_linear(x, w, torch.float32)
            want = torch.einsum("tbk,bnk->tbn", x.float().view(T, nb, k), w.float()).reshape(T, nb * n)
            assert got.dtype == torch.float32 and close(got, want, 1e-5), (T, nb, n, k)
            if T > 1:
                assert torch.equal(K.block_linear(x[T // 2:T // 2 + 1], w, torch.float32), got[T // 2:T // 2 + 1])
        h = torch.randn(T, 5 * 64 + 8, device=DEV).to(dt)[:, 8:]          # rows 16-byte aligned, base offset 16 bytes
        for e in (3, 10, 24, 70):
            wr = (torch.randn(e, 5 * 64, device=DEV) / 16).to(dt)
            got = S.router_logits(h, wr, force="mma")
            assert close(got, h.float() @ wr.float().T, 1e-5), (T, e)
        h2 = torch.randn(T, 640, device=DEV).to(dt)                       # wide and narrow: K split over the warps
        for e in (5, 16, 30):
            wr = (torch.randn(e, 640, device=DEV) / 25).to(dt)
            got = S.router_logits(h2, wr, force="mma")
            assert close(got, h2.float() @ wr.float().T, 1e-5), (T, e)
            if T > 1:
                assert torch.equal(S.router_logits(h2[T - 1:], wr, force="mma"), got[T - 1:])


@pytest.mark.parametrize("dt,tol", [(torch.float32, 3e-5), (torch.bfloat16, 2e-2)])
def test_convolution_without_activation_and_input_bias(dt, tol):
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(2)
    for taps in (1, 2, 4):
        C = 24
        b = _batch([9, 1, 3, 1], [0, 5, 2, 0], 4, 64)
        T = int(b.query_start_loc[-1])
        xz = torch.randn(T, 2 * C, device=DEV).to(dt)
        w, cb, ib = torch.randn(C, taps, device=DEV), torch.randn(C, device=DEV), torch.randn(C, device=DEV)
        st1 = torch.randn(8, max(taps - 1, 0), C, device=DEV).to(dt) if taps > 1 else None
        st2 = st1.clone() if st1 is not None else None
        o1 = S.causal_conv_silu(xz[:, C:], C, w, cb, st1, b.rec_slots, b.seq_lens, b.query_start_loc, "none", ib)
        o2 = ref.causal_conv_silu(xz[:, C:], C, w, cb, st2, b.rec_slots, b.seq_lens, b.query_start_loc, "none", ib)
        assert close(o1, o2, tol), taps
        if st1 is not None:
            assert close(st1, st2, tol)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 5e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("qlens,ctx", [([9, 1, 3, 1], [0, 5, 2, 0]), ([300, 1, 257, 64], [0, 40, 7, 0]),
                                       ([1000], [3])])
def test_gated_recurrent_unit_scan(dt, tol, qlens, ctx):
    """Short portions take the token-serial kernel, long ones the two-pass chunked form; both carry the state."""
    from gllm_b200.ops import ref, sm100_latent as K
    torch.manual_seed(3)
    C, block = 40, 8
    b = _batch(qlens, ctx, 16, 256)
    T = int(b.query_start_loc[-1])
    u = torch.randn(T, C, device=DEV).to(dt)
    gates = torch.randn(T, 2 * C, device=DEV)
    gb, yb = torch.randn(2 * C, device=DEV), torch.randn(C, device=DEV)
    cdec = -8.0 * torch.nn.functional.softplus(torch.randn(C, device=DEV) - 3.0)     # some channels remember long
    ypre = torch.randn(T, 2 * C + 3, device=DEV).to(dt)[:, :2 * C]
    s1 = torch.randn(8, 1, C, device=DEV)
    s2 = s1.clone()
    o1 = K.rglru_scan(u, gates, gb, cdec, ypre, yb, s1, b.rec_slots, b.seq_lens, b.query_start_loc, block, dt,
                      max_q_len=b.max_q_len)
    o2 = ref.rglru_scan(u, gates, gb, cdec, ypre, yb, s2, b.rec_slots, b.seq_lens, b.query_start_loc, block, dt)
    assert close(o1, o2, tol)
    assert close(s1, s2, 1e-4)
    if b.max_q_len >= 256:        # the serial kernel on the same long input
        s3 = torch.randn(8, 1, C, device=DEV)
        s4 = s3.clone()
        o3 = K.rglru_scan(u, gates, gb, cdec, ypre, yb, s3, b.rec_slots, b.seq_lens, b.query_start_loc, block, dt)
        o4 = ref.rglru_scan(u, gates, gb, cdec, ypre, yb, s4, b.rec_slots, b.seq_lens, b.query_start_loc, block, dt)
        assert close(o3, o4, tol) and close(s3, s4, 1e-4)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 5e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,dim,vdim", [(2, 6, 10), (1, 3, 7), (3, 64, 64), (2, 40, 24), (2, 128, 128)])
def test_key_channel_decay_state_scan(dt, tol, heads, dim, vdim):
    from gllm_b200.ops import ref, sm100_seq as S
    torch.manual_seed(4)
    for qlens, ctx in (([9, 1, 3, 1], [0, 5, 2, 0]), ([150, 1], [0, 9])):
        b = _batch(qlens, ctx, 16, 64)
        T = int(b.query_start_loc[-1])
        q, k = (torch.randn(T, heads * dim, device=DEV).to(dt) for _ in range(2))
        v = torch.randn(T, heads * vdim, device=DEV).to(dt)
        zk = (torch.randn(T, heads * dim, device=DEV) * 2).to(dt)
        zb = torch.randn(heads * dim, device=DEV) + 2.0
        s1 = torch.randn(8, heads, dim, vdim, device=DEV)
        s2 = s1.clone()
        args = (heads, heads, dim, vdim, False, False, dim ** -0.5, False)
        o1 = S.linear_state_scan(q, k, v, None, None, None, None, None, s1, b.rec_slots, b.seq_lens,
                                 b.query_start_loc, *args, zk=zk, zk_bias=zb, inv_tau=1 / 16.0)
        o2 = ref.linear_state_scan(q, k, v, None, None, None, None, None, s2, b.rec_slots, b.seq_lens,
                                   b.query_start_loc, *args, zk=zk, zk_bias=zb, inv_tau=1 / 16.0)
        assert close(o1, o2, tol) and close(s1, s2, 1e-4), (qlens, heads, dim, vdim)


def _latent_case(dt, heads, dim, rot, rank, qlens, ctx, ps, scale=0.3):
    """norm + rotation + cache write and the attention over the paged latent cache on a mixed batch whose earlier
    tokens are already cached; -> (kernel result, unfused result)."""
    from gllm_b200.memory_manager import kv_cache_shape
    from gllm_b200.ops import ref, sm100_latent as K
    pages = 2 + len(qlens) * max((c + q + ps - 1) // ps for c, q in zip(ctx, qlens))
    b = _batch(qlens, ctx, ps, pages)
    T = int(b.query_start_loc[-1])
    f, mag = ref.pair_rotary_frequencies(rot, 30000.0, {"factor": 6.0, "original": 64, "fast": 24.0, "slow": 1.0})
    f = f.to(DEV)
    nw = (torch.rand(rank, device=DEV) + 0.5).to(dt)
    c1 = torch.zeros(kv_cache_shape(pages, 1, rank + rot, ps), dtype=dt, device=DEV)
    # the context rows, written through the unfused form at their own positions
    for s, c in enumerate(ctx):
        if c:
            pos = torch.arange(c, device=DEV, dtype=torch.int32)
            sl = (b.block_table[s, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
            ref.latent_norm_rope_write(torch.zeros(c, heads, dim + rot, device=DEV, dtype=dt),
                                       torch.randn(c, rank + rot, device=DEV).to(dt), rank, rot, nw, 1e-5, pos, f,
                                       mag, torch.zeros(c, heads, rank + rot, device=DEV, dtype=dt), c1, sl)
    c2 = c1.clone()
    q = torch.randn(T, heads, dim + rot + 2, device=DEV).to(dt)[:, :, :dim + rot]
    dkv = torch.randn(T, rank + rot + 8, device=DEV).to(dt)[:, :rank + rot]
    qf1 = torch.randn(T, heads, rank + rot, device=DEV).to(dt)
    qf2 = qf1.clone()
    K.latent_norm_rope_write(q, dkv, rank, rot, nw, 1e-5, b.positions, f, mag, qf1, c1, b.slot_mapping)
    ref.latent_norm_rope_write(q, dkv, rank, rot, nw, 1e-5, b.positions, f, mag, qf2, c2, b.slot_mapping)
    o1 = K.latent_attention(qf1, c1, b, scale, rank)
    o2 = ref.latent_attention(qf2, c2, b.block_table, b.seq_lens, b.query_start_loc, scale, rank)
    return (qf1, c1, o1), (qf2, c2, o2)


@pytest.mark.parametrize("dt,tol", [(torch.float32, 5e-5), (torch.bfloat16, 2e-2)])
@pytest.mark.parametrize("heads,dim,rot,rank", [(3, 8, 4, 12), (1, 2, 2, 1), (6, 64, 16, 160), (5, 24, 6, 40),
                                                (2, 32, 64, 96), (16, 128, 64, 512)])
def test_latent_rotation_cache_write_and_attention(dt, tol, heads, dim, rot, rank):
    torch.manual_seed(5)
    for qlens, ctx, ps in (([9, 1, 3, 1], [0, 35, 2, 16], 4), ([70, 1, 1, 33], [0, 200, 15, 31], 16)):
        got, want = _latent_case(dt, heads, dim, rot, rank, qlens, ctx, ps)
        for g, w, name in zip(got, want, ("queries", "cache", "attention")):
            assert close(g, w, tol), (name, heads, dim, rot, rank, qlens)


def test_router_on_the_device():
    for args in [(6, 2, 2, (2, 1), 1.5, torch.full((8,), -3.0) + torch.randn(8) * 0.01, 1),
                 (6, 2, 3, (4, 2), 2.5, torch.tensor([0, 0, 0, 0, 0, 0, 5.0, 5.0]), 2),
                 (8, 0, 2, (2, 1), 1.0, torch.randn(8) * 0.2, 3), (5, 1, 6, (3, 3), 0.5, torch.randn(6) * 0.2, 4),
                 (7, 0, 1, None, 1.0, torch.randn(7), 5), (3, 9, 4, (4, 2), 3.0, torch.randn(12) * 0.3, 6),
                 (64, 8, 6, (8, 3), 2.5, torch.randn(72) * 0.05, 7), (250, 6, 8, (8, 4), 2.5, torch.randn(256) * 0.01, 8),
                 (1, 0, 1, (1, 1), 1.0, torch.zeros(1), 9)]:
        _route_case(*args, device=DEV)
        _route_case(*args, t=700, width=64, device=DEV)            # the large-batch logits path


def test_clamped_experts_grouped_against_plain():
    """The grouped tcgen05 GEMM pair with the clamped gated epilogue, identity experts skipped and added by their own
    kernel, against the plain per-slot kernels and the unfused form; and the dense gated epilogue."""
    from gllm_b200.ops import ref, sm100_latent as K
    torch.manual_seed(6)
    dt = torch.bfloat16
    for T, width, ff, n_real, n_id, top in ((1, 128, 64, 4, 2, 2), (77, 256, 192, 6, 2, 3), (400, 128, 128, 3, 0, 2),
                                            (33, 128, 64, 2, 4, 4)):
        h = torch.randn(T, width, device=DEV).to(dt)
        w13 = (torch.randn(n_real, 2 * ff, width, device=DEV) * width ** -0.5 * 2).to(dt)
        w2 = (torch.randn(n_real, width, ff, device=DEV) * ff ** -0.5).to(dt)
        ids = torch.stack([torch.randperm(n_real + n_id)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
        wts = torch.rand(T, top, device=DEV)
        want = ref.routed_glu_experts(h, w13, w2, wts, ids, 1.5)
        plain = K.routed_glu_experts(h, w13, w2, wts, ids, 1.5, False, 1.702, n_real + n_id)
        w13i = torch.stack([ref.interleave_gate_up(w13[e], 64) for e in range(n_real)])
        fused = K.routed_glu_experts(h, w13i, w2, wts, ids, 1.5, True, 1.702, n_real + n_id)
        assert close(plain, want, 2e-2) and close(fused, want, 2e-2), (T, width, ff)
    for T in (1, 9, 300):
        x = torch.randn(T, 192, device=DEV).to(dt)
        w = (torch.randn(2 * 256, 192, device=DEV) * 0.15).to(dt)
        wi = ref.interleave_gate_up(w, 128)
        assert close(K.linear_glu_clamp(x, wi, 0.75), ref.glu_clamp(torch.nn.functional.linear(x, w), 0.75), 2e-2)


@pytest.mark.parametrize("dt", [torch.float32])
def test_plain_experts_in_fp32(dt):
    from gllm_b200.ops import ref, sm100_latent as K
    torch.manual_seed(7)
    T, width, ff, n_real, n_id, top = 41, 20, 8, 3, 3, 4
    h = torch.randn(T, width, device=DEV)
    w13, w2 = torch.randn(n_real, 2 * ff, width, device=DEV) * 0.4, torch.randn(n_real, width, ff, device=DEV) * 0.4
    ids = torch.stack([torch.randperm(n_real + n_id)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
    wts = torch.rand(T, top, device=DEV)
    got = K.routed_glu_experts(h, w13, w2, wts, ids, 0.7, False, 1.702, n_real + n_id)
    assert close(got, ref.routed_glu_experts(h, w13, w2, wts, ids, 0.7), 3e-5)


# -- the mixers alone on the device, against the plain oracle --------------------------------------------------------
@pytest.mark.parametrize("dtype,tol", [(torch.float32, 2e-4), (torch.bfloat16, 4e-2)])
def test_mixers_alone_on_the_device(dtype, tol):
    kw = dict(device=DEV, dtype=dtype, tol=tol)
    _mixer_alone(U.rglru(), 1, **kw)
    _mixer_alone(U.rglru(width=10, blocks=5, conv=4), 2, **kw)
    _mixer_alone(U.rglru(width=8, blocks=1, conv=1), 3, **kw)
    _mixer_alone(U.rglru(width=128, blocks=2, conv=2), 4, width=64, **kw)          # batched GEMM on the tensor cores
    _mixer_alone(U.gla(), 5, **kw)
    _mixer_alone(U.gla(heads=1, dim=3, vdim=7, tau=1.0), 6, low_rank=1, **kw)
    _mixer_alone(U.gla(heads=4, dim=8, vdim=2, tau=32.0), 7, low_rank=9, **kw)
    _mixer_alone(U.gla(heads=2, dim=64, vdim=32, tau=16.0), 7, low_rank=16, width=64, **kw)
    _mixer_alone(U.latent(), 8, **kw)
    _mixer_alone(U.latent(heads=1, dim=4, rot_dim=8, vdim=3, q_rank=3, kv_rank=5, scaling=None), 9, page_size=8, **kw)
    _mixer_alone(U.latent(heads=5, dim=2, rot_dim=2, vdim=9, q_rank=16, kv_rank=4,
                          scaling={"factor": 16.0, "original": 6, "fast": 3.0, "slow": 0.5}), 10, page_size=16, **kw)
    _mixer_alone(U.latent(heads=4, dim=32, rot_dim=16, vdim=32, q_rank=40, kv_rank=64, scale=0.15), 11, page_size=16,
                 width=64, **kw)


@pytest.mark.parametrize("page_size", [4, 16])
def test_far_keys_and_page_borders_on_the_device(page_size):
    n = 331
    for back in (0, 1, page_size - 1, page_size, page_size + 1, 64, 200, 330):
        want, outs, other = far_key_probe(n, back, page_size, DEV)
        if back > 0:
            assert (want[-1] - other[-1]).abs().max() > 0.05 * want[-1].abs().max(), back
        for o in outs:
            assert torch.allclose(o, want, atol=2e-4 * want.abs().max().item(), rtol=2e-4), (page_size, back)


@pytest.mark.parametrize("taps", [1, 2, 3, 4])
def test_convolution_edges_on_the_device(taps):
    for back in range(0, taps + 2):
        base, want, outs = conv_edge_probe(taps, back, DEV)
        assert ((want[-1] - base[-1]).abs().max().item() > 1e-3) == (back < taps), (taps, back)
        for o in outs:
            assert torch.allclose(o, want, atol=1e-4, rtol=1e-4), (taps, back)


# -- whole models through the engine -----------------------------------------------------------------------------
@pytest.fixture(scope="module")
def models():
    out = {}
    for i, (name, cfg) in enumerate(CONFIGS.items()):
        w = U.random_weights(cfg, seed=60 + i, low_rank=3 + i)
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
    oracle.forward(cfg, w, t, torch.float64, trace)
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


@pytest.mark.parametrize("kind", ["gla", "rglru"])
def test_far_state_survives_long_decoding_on_the_device(kind):
    cfg, w = far_state_model(kind)
    path = U.save_model(cfg, w)
    t = [3] + [5] * 300
    t2 = [7] + [5] * 300
    a, b = U.expected_logits(cfg, w, t), U.expected_logits(cfg, w, t2)
    assert np.abs(a[-1] - b[-1]).max() > 1e-3
    s = U.session(path, "float32", DEV, max_tokens=512, page_size=16)
    assert U.rel_err(U.run_chunks(s, "a", t, [200, 50, 2, 2]), a) < TOL32
    assert U.rel_err(U.run_chunks(s, "b", t2, [1, 250]), b) < TOL32
    assert U.rel_err(U.run_chunks(s, "c", t2, [299]), b) < TOL32            # the two-pass recurrence over a long portion


def test_tensor_core_sized_model_in_bf16():
    """Sizes at which every tensor-core path is taken (tcgen05 GEMMs with the gated epilogue, grouped expert GEMMs,
    batched per-head products, the 512 + 64 latent attention kernel), against the oracle with the bf16 CPU run as
    the measure of rounding; prompt portions long enough for the chunked recurrence."""
    layers = [U.rglru(width=256, blocks=4, conv=4, mlp=U.moe(experts=6, identity=2, top=2, ff=64, groups=(4, 2),
                                                             scale=2.5, shared=(128, 1.0))),
              U.latent(heads=4, dim=64, rot_dim=64, vdim=64, q_rank=96, kv_rank=512, base=10000.0, scale=0.09,
                       mlp=U.moe(experts=8, identity=0, top=2, ff=128, groups=(2, 1), shared=(256, 2.0))),
              U.gla(heads=2, dim=64, vdim=128, tau=16.0, mlp=None),
              U.latent(heads=4, dim=32, rot_dim=32, vdim=64, q_rank=64, kv_rank=128, scale=0.12, mlp=None)]
    cfg = U.make_config(layers, vocab=512, width=256)
    w = U.random_weights(cfg, 5, low_rank=16)
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
            cur.append(int(oracle.forward(cfg, w, cur, torch.float64)[-1].argmax()))
        assert s.token_ids == cur
