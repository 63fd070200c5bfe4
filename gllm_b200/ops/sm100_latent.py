"""Python front-ends of csrc/seq/latent_ops.cu (ctypes -> libgllm_b200.so): kernels of the branch-norm layer-list
decoder — strided-row RMS norm, batched / block-diagonal products, the real-gated linear recurrent unit, latent
attention (norm + pair rotary + latent-cache write, attention over the latent cache), the grouped router and the
clamped gated experts.

bf16 and fp32 operands; norms, angles, softmax, gates, decays and recurrent state are fp32 in both. No fallback: a
missing library on a GPU box raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from gllm_b200.ops import lib as _lib
from gllm_b200.ops import sm100, sm100_seq
from gllm_b200.ops.lib import check, stream_ptr

_declared = False
_BF16 = torch.bfloat16
_RGLRU_CHUNK = 64          # tokens per chunk of the two-pass recurrence
_RGLRU_CHUNKED_MIN = 256   # prompts portions at least this long take the two-pass form


def _L():
    global _declared
    L = _lib.load()
    if not _declared:
        P, I, G, F = c_void_p, c_int, c_long, c_float
        sigs = {
            "gllm_lat_rms_rows": [P, G, P, P, I, I, F, I, P],
            "gllm_lat_gemm_batched": [P, G, G, P, G, G, P, G, G, I, I, I, I, I, I, P],
            "gllm_lat_rglru_scan": [P, P, P, P, P, G, P, P, P, P, P, I, I, I, P, I, I, P, I, P],
            "gllm_lat_norm_rope_write": [P, G, G, I, I, P, G, I, I, P, F, P, P, F, P, P, P, I, I, I, I, P],
            "gllm_lat_attention": [P, P, P, I, P, P, I, I, F, I, I, I, P, I, I, I, P],
            "gllm_lat_grouped_router_select": [P, P, I, I, I, I, I, F, P, P, I, I, I, P],
            "gllm_lat_glu_clamp": [P, G, I, I, P, F, F, I, P],
            "gllm_lat_identity_experts_add": [P, G, P, P, I, I, I, I, P, I, P],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.argtypes, fn.restype = args, c_int
        _declared = True
    return L


def _p(t: Optional[torch.Tensor]):
    return None if t is None else ctypes.c_void_p(t.data_ptr())


def _f32(t: torch.Tensor) -> int:
    assert t.dtype in (torch.bfloat16, torch.float32), t.dtype
    return 1 if t.dtype == torch.float32 else 0


def rms_rows(x, w, eps):
    t, n = x.shape
    assert x.stride(1) == 1 and w.dtype == x.dtype and w.shape[0] == n
    out = torch.empty(t, n, dtype=x.dtype, device=x.device)
    check(_L().gllm_lat_rms_rows(_p(x), x.stride(0), _p(w), _p(out), t, n, float(eps), _f32(x), stream_ptr()),
          "lat_rms_rows")
    sm100._count()
    return out


def _gemm_batched_plain(a, lda, sa, w, ldw, sw, out, ldc, sc, m, n, k, b):
    check(_L().gllm_lat_gemm_batched(_p(a), lda, sa, _p(w), ldw, sw, _p(out), ldc, sc, m, n, k, b, _f32(a),
                                     1 if out.dtype == torch.float32 else 0, stream_ptr()), "lat_gemm_batched")
    sm100._count()
    return out


def _tc_batched_ok(a, w, out) -> bool:
    k, n = a.shape[2], w.shape[1]
    return a.dtype == _BF16 and out.dtype == _BF16 and k % 8 == 0 and n % 8 == 0 and k >= 32 and n >= 32 and \
        all(s % 8 == 0 for s in (a.stride(0), a.stride(1), out.stride(0), out.stride(1))) and \
        a.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0


def linear_batched(a, w, out):
    """out[:, b, :] = a[:, b, :] @ w[b].T; a [T, B, K] / out [T, B, N] strided views, w [B, N, K] contiguous."""
    t, b, k = a.shape
    n = w.shape[1]
    assert w.shape == (b, n, k) and w.is_contiguous() and out.shape == (t, b, n) and a.dtype == w.dtype
    assert a.stride(2) == 1 and out.stride(2) == 1
    if t == 0:
        return out
    if _tc_batched_ok(a, w, out):
        return sm100.gemm_batched(a, w, out)
    return _gemm_batched_plain(a, a.stride(0), a.stride(1), w, k, n * k, out, out.stride(0), out.stride(1), t, n, k, b)


def block_linear(x, w, out_dtype=None):
    """x [T, B * K] x w [B, N, K] -> [T, B * N] (block-diagonal map); fp32 result on request (plain kernel)."""
    t = x.shape[0]
    nb, n, k = w.shape
    assert x.shape[1] == nb * k and x.stride(1) == 1 and w.is_contiguous() and x.dtype == w.dtype
    odt = out_dtype or x.dtype
    out = torch.empty(t, nb * n, dtype=odt, device=x.device)
    if t == 0:
        return out
    if odt == _BF16:
        a3, o3 = x.view(t, nb, k) if x.is_contiguous() else x.unflatten(1, (nb, k)), out.view(t, nb, n)
        if _tc_batched_ok(a3, w, o3):
            sm100.gemm_batched(a3, w, o3)
            return out
    assert odt in (x.dtype, torch.float32)
    if odt == torch.float32 and x.dtype == _BF16:
        a3 = x.view(t, nb, k) if x.is_contiguous() else x.unflatten(1, (nb, k))
        if sm100_seq.mma_f32out_ok(a3, w):       # whatever the batch size: one rounding behaviour per shape
            sm100_seq.gemm_mma_f32out(a3, w, out.view(t, nb, n))
            return out
    return _gemm_batched_plain(x, x.stride(0), k, w, k, n * k, out, nb * n, n, t, n, k, nb)


_rglru_ws = {}


def rglru_scan(u, gates, gate_bias, c_decay, y_pre, y_bias, state, rec_slots, seq_lens, query_start_loc, block,
               out_dtype, max_q_len: Optional[int] = None):
    t, c = u.shape
    assert u.is_contiguous() and gates.is_contiguous() and gates.dtype == torch.float32 and gates.shape[1] == 2 * c
    assert y_pre.stride(1) == 1 and y_pre.dtype == u.dtype and out_dtype == u.dtype
    for x in (gate_bias, c_decay, y_bias):
        assert x.dtype == torch.float32 and x.is_contiguous()
    assert state is None or (state.dtype == torch.float32 and state.is_contiguous())
    out = torch.empty(t, c, dtype=out_dtype, device=u.device)
    nseq = seq_lens.shape[0]
    chunk, nchunks, ws = 0, 0, None
    if max_q_len is not None and max_q_len >= _RGLRU_CHUNKED_MIN and \
            not torch.cuda.is_current_stream_capturing():
        chunk = _RGLRU_CHUNK
        nchunks = (max_q_len + chunk - 1) // chunk
        need = nseq * nchunks * c * 2
        key = torch.device(u.device)
        ws = _rglru_ws.get(key)
        if ws is None or ws.numel() < need:
            ws = torch.empty(need, dtype=torch.float32, device=u.device)
            _rglru_ws[key] = ws
    check(_L().gllm_lat_rglru_scan(_p(u), _p(gates), _p(gate_bias), _p(c_decay), _p(y_pre), y_pre.stride(0),
                                   _p(y_bias), _p(state), _p(rec_slots), _p(seq_lens), _p(query_start_loc), nseq, c,
                                   int(block), _p(out), chunk, nchunks, _p(ws), _f32(u), stream_ptr()),
          "lat_rglru_scan")
    sm100._count(2 if chunk else 1)
    return out


def latent_norm_rope_write(q, dkv, rank, rot, norm_w, eps, positions, freqs, mag, q_full, cache, slots):
    t, h = q.shape[0], q.shape[1]
    dim = q.shape[2] - rot
    assert q.stride(2) == 1 and dkv.stride(1) == 1 and q_full.is_contiguous() and q_full.shape == (t, h, rank + rot)
    assert freqs.dtype == torch.float32 and freqs.shape[0] == rot // 2 and positions.dim() == 1
    assert cache is None or (cache.dtype == q.dtype and cache.shape[1] == 1)
    ps, slab = (cache.shape[3], cache.shape[4]) if cache is not None else (1, rank + rot)
    check(_L().gllm_lat_norm_rope_write(_p(q), q.stride(0), q.stride(1), h, dim, _p(dkv), dkv.stride(0), rank, rot,
                                        _p(norm_w), float(eps), _p(positions), _p(freqs), float(mag), _p(q_full),
                                        _p(cache), _p(slots if cache is not None else None), ps, slab, t, _f32(q),
                                        stream_ptr()), "lat_norm_rope_write")
    sm100._count()


def latent_attention(q_full, cache, inp, scale, rank, plain: bool = False):
    """Causal multi-query attention over the latent cache. bf16 with a 512-wide latent and a 64-wide rotated part
    (pages of 8 to 64 tokens) runs on the tensor-core latent kernel (csrc/attn/mla_attention.cu, split over the keys
    for small batches);
    every other shape and fp32 on the plain kernel."""
    t, h, dl = q_full.shape
    assert q_full.is_contiguous() and cache.dtype == q_full.dtype
    ps, slab = cache.shape[3], cache.shape[4]
    if not plain and q_full.dtype == _BF16 and rank == 512 and dl == 576 and slab == 64 and ps >= 8 and 64 % ps == 0:
        return sm100.mla_attention(q_full, cache, inp.block_table, inp.tok_seq, inp.positions, scale)
    out = torch.empty(t, h, rank, dtype=q_full.dtype, device=q_full.device)
    bt = inp.block_table
    check(_L().gllm_lat_attention(_p(q_full), _p(cache), _p(bt), bt.stride(0), _p(inp.query_start_loc),
                                  _p(inp.positions), t, inp.seq_lens.shape[0], float(scale), h, dl, rank, _p(out), ps,
                                  slab, _f32(q_full), stream_ptr()), "lat_attention")
    sm100._count()
    return out


def grouped_router(h, w, correction, top_k, n_groups, keep_groups, scale, score="softmax", group_top=1, renorm=True):
    t, e = h.shape[0], w.shape[0]
    assert correction is None or (correction.dtype == torch.float32 and correction.is_contiguous())
    logits = sm100_seq.router_logits(h, w)
    wout = torch.empty(t, top_k, dtype=torch.float32, device=h.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=h.device)
    check(_L().gllm_lat_grouped_router_select(_p(logits), _p(correction), t, e, int(top_k), int(n_groups),
                                              int(keep_groups), float(scale), _p(wout), _p(ids),
                                              int(score == "sigmoid"), int(group_top), int(renorm), stream_ptr()),
          "lat_grouped_router_select")
    sm100._count()
    return wout, ids


def glu_clamp(gu, limit, alpha=1.702):
    t, f = gu.shape[0], gu.shape[1] // 2
    assert gu.stride(1) == 1
    out = torch.empty(t, f, dtype=gu.dtype, device=gu.device)
    check(_L().gllm_lat_glu_clamp(_p(gu), gu.stride(0), t, f, _p(out), float(limit), float(alpha), _f32(gu),
                                  stream_ptr()), "lat_glu_clamp")
    sm100._count()
    return out


def linear_glu_clamp(x, w_interleaved, limit, alpha=1.702):
    """Gate / up projection with the clamped gated epilogue on the tcgen05 GEMM (rows interleaved per 128)."""
    assert x.dtype == _BF16 and w_interleaved.dtype == _BF16 and x.stride(1) == 1
    m, k = x.shape
    n = w_interleaved.shape[0]
    out = torch.empty(m, n // 2, dtype=_BF16, device=x.device)
    if m == 0:
        return out
    ws, _, tcnt = sm100._smallm_workspace(x.device)
    check(_L().gllm_gemm_bf16_glu(_p(x), x.stride(0), _p(w_interleaved), w_interleaved.stride(0), _p(out),
                                  out.stride(0), m, n, k, float(limit), float(alpha), _p(ws), ws.numel() * 4,
                                  _p(tcnt), sm100._SPLITK_MAX_TILES, stream_ptr()), "gemm_bf16_glu")
    sm100._count()
    return out


_maps = {}


def _identity_map(n_real: int, n_all: int, device) -> torch.Tensor:
    """expert id -> slab index for the grouped GEMMs, -1 for identity experts (their slots are skipped)."""
    key = (n_real, n_all, torch.device(device))
    m = _maps.get(key)
    if m is None:
        m = torch.full((n_all,), -1, dtype=torch.int32)
        m[:n_real] = torch.arange(n_real, dtype=torch.int32)
        m = m.to(device)
        _maps[key] = m
    return m


def routed_glu_experts(h, w13, w2, weights, ids, limit, interleaved, alpha=1.702, n_all: Optional[int] = None):
    """Clamped gated experts over (weights, ids); ids >= w13.shape[0] are identity experts. `interleaved`: the
    grouped tcgen05 GEMM pair (align + gather, gate / up GEMM with the clamped epilogue, down GEMM, combine) and one
    kernel that adds the identity experts' share; otherwise the plain per-slot kernels."""
    n_real = w13.shape[0]
    if not interleaved:
        return sm100_seq.routed_experts(h, w13, w2, weights, ids, limit, alpha, n_real)
    from gllm_b200.ops import sm100_moe
    t, width = h.shape
    n_all = n_all if n_all is not None else n_real
    if n_all <= n_real:
        return sm100_moe.fused_experts(h, w13, w2, weights, ids, None, glu=(float(limit), float(alpha)))
    emap = _identity_map(n_real, n_all, h.device)
    out = sm100_moe.fused_experts(h, w13, w2, weights, ids, emap, glu=(float(limit), float(alpha)))
    check(_L().gllm_lat_identity_experts_add(_p(h), h.stride(0), _p(ids), _p(weights), t, ids.shape[1], n_real,
                                             width, _p(out), _f32(h), stream_ptr()), "lat_identity_experts_add")
    sm100._count()
    return out
