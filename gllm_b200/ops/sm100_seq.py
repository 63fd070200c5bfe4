"""Python front-ends of csrc/seq/seq_ops.cu (ctypes -> libgllm_b200.so): the kernels of the layer-list decoder.

bf16 and fp32 operands; the residual stream, norms, softmax and recurrent state are fp32 in both. No fallback: a
missing library on a GPU box raises.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_long, c_void_p
from typing import Optional

import torch

from gllm_b200.ops import lib as _lib
from gllm_b200.ops import sm100
from gllm_b200.ops.lib import check, stream_ptr

_declared = False
_TC_MIN = 64     # the tcgen05 GEMM takes over from this K and N on (smaller ones are latency-bound anyway)


def _L():
    global _declared
    L = _lib.load()
    if not _declared:
        P, I, G, F = c_void_p, c_int, c_long, c_float
        sigs = {
            "gllm_seq_embed_scale": [P, P, P, I, I, I, F, I, P],
            "gllm_seq_resid_norm": [P, P, G, P, P, P, P, P, I, I, F, I, I, F, F, P],
            "gllm_seq_qk_norm_kv_write": [P, G, I, I, I, I, P, P, F, P, P, P, P, I, I, I, P],
            "gllm_seq_window_attention": [P, P, P, P, I, P, P, I, I, F, I, I, I, I, I, I, P, P, G, F, I, I, I, I, F, P],
            "gllm_seq_postnorm": [P, P, G, P, P, I, I, F, F, I, P],
            "gllm_seq_qk_norm_rope_kv_write": [P, G, I, I, I, I, I, P, P, F, P, I, ctypes.c_double, P, P, P, P, I, I, I,
                                               I, P, F, P],
            "gllm_seq_linear_state": [P, G, P, G, P, G, P, G, P, G, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P,
                                      I, I, P, G, P],
            "gllm_seq_key_decay": [P, G, P, F, P, I, I, I, P],
            "gllm_seq_gemm_mma_f32out": [P, G, G, P, G, G, P, G, G, I, I, I, I, P],
            "gllm_seq_gated_group_norm": [P, I, P, G, P, I, I, F, I, F, P, G, I, I, P],
            "gllm_seq_silu_mul": [P, G, I, I, P, I, P],
            "gllm_seq_router_select": [P, I, I, I, P, P, P],
            "gllm_seq_router_logits": [P, G, P, I, I, I, P, I, P],
            "gllm_seq_router_logits_mma": [P, G, P, I, I, I, P, P],
            "gllm_seq_gemm_simt_f32out": [P, G, P, G, P, G, I, I, I, I, P],
            "gllm_seq_routed_experts": [P, G, P, P, P, P, I, I, I, I, P, P, I, I, F, F, I, P],
            "gllm_seq_softcap": [P, G, I, I, F, I, P],
            "gllm_seq_conv_silu": [P, G, I, I, I, P, P, I, P, P, P, P, P, I, I, P, P],
            "gllm_seq_selective_scan": [P, P, P, G, P, G, P, P, P, P, P, P, P, I, I, I, I, P, I, I, P],
            "gllm_seq_relu2": [P, P, G, I, P],
            "gllm_seq_gemm_simt": [P, G, P, G, P, G, I, I, I, I, P, P],
            "gllm_attn_decode_win": [P, G, P, P, P, G, P, P, I, I, I, I, I, I, I, F, I, P, P],
            "gllm_attn_prefill_win": [P, G, P, P, P, G, P, P, P, I, I, I, I, I, I, I, I, F, I, P, P],
            "gllm_attn_prefill_tc_cap": [P, G, P, P, P, G, P, P, P, I, I, I, I, I, I, I, I, F, I, P, F, P],
            "gllm_attn_decode_mask": [P, G, P, G, P, P, G, P, P, I, I, I, I, I, I, I, F, I, I, P, F, F, P],
            "gllm_attn_prefill_mask": [P, G, P, G, P, P, G, P, P, P, I, I, I, I, I, I, I, I, F, I, I, P, F, F, P],
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


def gemm_simt(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    assert x.dtype == w.dtype and x.stride(1) == 1 and w.stride(1) == 1 and x.shape[1] == w.shape[1]
    assert bias is None or (bias.dtype == x.dtype and bias.is_contiguous() and bias.shape[0] >= w.shape[0])
    m, k = x.shape
    n = w.shape[0]
    out = torch.empty(m, n, dtype=x.dtype, device=x.device)
    check(_L().gllm_seq_gemm_simt(_p(x), x.stride(0), _p(w), w.stride(0), _p(out), out.stride(0), m, n, k, _f32(x),
                                  _p(bias), stream_ptr()), "seq_gemm_simt")
    sm100._count()
    return out


def linear_any(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    m, k = x.shape
    n = w.shape[0]
    if x.dtype == torch.bfloat16 and k >= _TC_MIN and n >= _TC_MIN and k % 8 == 0 and n % 8 == 0 and \
            x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and \
            (bias is None or bias.data_ptr() % 16 == 0):
        return sm100.linear(x, w, bias)
    return gemm_simt(x, w, bias)


def embedding_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    t, width = ids.shape[0], table.shape[1]
    out = torch.empty(t, width, dtype=torch.float32, device=table.device)
    check(_L().gllm_seq_embed_scale(_p(ids), _p(table), _p(out), t, width, table.shape[0], float(scale), _f32(table),
                                    stream_ptr()), "seq_embed_scale")
    sm100._count()
    return out


def resid_norm(x, y, w_post, add, w_pre, eps, out_dtype, emit_plain=False, post_scale=None, w_offset=0.0,
               out_mul=1.0):
    assert x.dtype == torch.float32 and x.is_contiguous()
    t, width = x.shape
    plain = bool(emit_plain) and w_pre is None
    if plain and out_dtype == torch.float32:
        plain, ret_x = False, True          # the fp32 stream is its own copy
    else:
        ret_x = False
    out = torch.empty(t, width, dtype=out_dtype, device=x.device) if (w_pre is not None or plain) else None
    assert post_scale is None or (post_scale.dtype == torch.float32 and post_scale.is_contiguous())
    ref_t = w_pre if w_pre is not None else (w_post if w_post is not None else None)
    is32 = 1 if (ref_t is not None and ref_t.dtype == torch.float32) or (ref_t is None and out_dtype == torch.float32) \
        else 0
    if y is not None:
        assert y.stride(1) == 1 and y.dtype == w_post.dtype
    if add is not None:
        assert add.dtype == torch.float32 and add.is_contiguous()
    if y is None and add is None and w_pre is None and not plain:
        return x if ret_x else None
    check(_L().gllm_seq_resid_norm(_p(x), _p(y), y.stride(0) if y is not None else 0, _p(w_post), _p(post_scale),
                                   _p(add), _p(w_pre), _p(out), t, width, float(eps), int(plain), is32, float(w_offset),
                                   float(out_mul), stream_ptr()),
          "seq_resid_norm")
    sm100._count()
    return x if ret_x else out


def qk_norm_kv_write(qk, num_heads, num_kv_heads, dim, q_norm_w, k_norm_w, eps, k_cache, v_cache, slots):
    t = qk.shape[0]
    assert qk.stride(1) == 1 and k_cache.dtype == qk.dtype
    q = torch.empty(t, num_heads * dim, dtype=qk.dtype, device=qk.device)
    ps, slab = k_cache.shape[3], k_cache.shape[4]
    check(_L().gllm_seq_qk_norm_kv_write(_p(qk), qk.stride(0), t, num_heads, num_kv_heads, dim, _p(q_norm_w),
                                         _p(k_norm_w), float(eps), _p(q), _p(k_cache), _p(v_cache), _p(slots), ps,
                                         slab, _f32(qk), stream_ptr()), "seq_qk_norm_kv_write")
    sm100._count()
    return q


def window_attention(q, k_cache, v_cache, block_table, seq_lens, query_start_loc, positions, scale, num_q_heads,
                     head_dim, window, sink, num_decode_seqs: int = 0, max_q_len: Optional[int] = None,
                     simt: bool = False, chunk: Optional[int] = None, v_dim: Optional[int] = None,
                     out_scale: float = 1.0, out: Optional[torch.Tensor] = None, softcap: float = 0.0):
    """Masked paged attention: sliding window (None / 0 = full causal) and / or chunk mask, optional per-head softmax
    sink, values `v_dim` wide, result times `out_scale` into `out` (any row stride). bf16 with v_dim == head_dim
    in 64 / 128 / 256 and pages of 8..64 tokens runs on the tensor-core paged-attention kernels
    (csrc/attn/paged_attention.cu: the first `num_decode_seqs` sequences, one token each, on the decode kernel, the
    rest on the prefill kernel); everything else (fp32, other head sizes or page sizes) on the plain kernel."""
    t = q.shape[0]
    v_dim = head_dim if v_dim is None else v_dim
    if out is None:
        out = torch.empty(t, num_q_heads * v_dim, dtype=q.dtype, device=q.device)
    ps, slab = k_cache.shape[3], k_cache.shape[4]
    assert q.is_contiguous() and block_table.stride(1) == 1 and positions.dim() == 1
    assert out.stride(1) == 1 and out.dtype == q.dtype and v_cache.shape[3] == ps
    nseq = seq_lens.shape[0]
    # the tensor-core kernels store 8-byte vectors: rows and head offsets of `out` must keep that alignment
    tc_ok = v_dim == head_dim and out.stride(0) % 4 == 0 and out.data_ptr() % 8 == 0
    if not simt and tc_ok and q.dtype == torch.bfloat16 and head_dim in (64, 128, 256) and slab == 64 and ps >= 8 and \
            64 % ps == 0 and max_q_len is not None:
        L, st = _L(), stream_ptr()
        pages, hkv = k_cache.shape[0], k_cache.shape[1]
        if num_decode_seqs > 0:
            check(L.gllm_attn_decode_mask(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), pages,
                                          _p(block_table), _p(seq_lens), num_decode_seqs, 0, block_table.stride(0),
                                          num_q_heads, hkv, head_dim, ps, float(scale), int(window or 0),
                                          int(chunk or 0), _p(sink), float(out_scale), float(softcap), st),
                  "attn_decode_mask")
            sm100._count()
        rest = nseq > num_decode_seqs
        if rest and not window and not chunk and sm100.ATTN_TC and out_scale == 1.0 and \
                out.stride(0) == num_q_heads * head_dim and head_dim in (64, 128) and sm100.ATTN_TC_KV % ps == 0:
            # full causal (cap and sink only): the tcgen05 prefill kernel
            rc = L.gllm_attn_prefill_tc_cap(_p(q), q.stride(0), _p(out), _p(k_cache), _p(v_cache), pages,
                                            _p(block_table), _p(seq_lens), _p(query_start_loc), nseq - num_decode_seqs,
                                            num_decode_seqs, max_q_len, block_table.stride(0), num_q_heads, hkv,
                                            head_dim, ps, float(scale), sm100.ATTN_TC_KV, _p(sink), float(softcap), st)
            if rc != 2:                     # 2 = shape outside that kernel's envelope -> the mma.sync kernel
                check(rc, "attn_prefill_tc_cap")
                sm100._count()
                rest = False
        if rest:
            check(L.gllm_attn_prefill_mask(_p(q), q.stride(0), _p(out), out.stride(0), _p(k_cache), _p(v_cache), pages,
                                           _p(block_table), _p(seq_lens), _p(query_start_loc), nseq - num_decode_seqs,
                                           num_decode_seqs, max_q_len, block_table.stride(0), num_q_heads, hkv,
                                           head_dim, ps, float(scale), int(window or 0), int(chunk or 0), _p(sink),
                                           float(out_scale), float(softcap), st), "attn_prefill_mask")
            sm100._count()
        return out
    check(_L().gllm_seq_window_attention(_p(q), _p(k_cache), _p(v_cache), _p(block_table), block_table.stride(0),
                                         _p(query_start_loc), _p(positions), t, seq_lens.shape[0], float(scale),
                                         num_q_heads, k_cache.shape[1], head_dim, v_dim, int(window or 0),
                                         int(chunk or 0), _p(sink), _p(out), out.stride(0), float(out_scale), ps, slab,
                                         v_cache.shape[4], _f32(q), float(softcap), stream_ptr()),
          "seq_window_attention")
    sm100._count()
    return out


def causal_conv_silu(xz, channels, w, b, conv_state, rec_slots, seq_lens, query_start_loc, act="silu", in_bias=None):
    t = xz.shape[0]
    assert xz.stride(1) == 1 and w.dtype == torch.float32 and b.dtype == torch.float32
    assert in_bias is None or (in_bias.dtype == torch.float32 and in_bias.is_contiguous())
    out = torch.empty(t, channels, dtype=xz.dtype, device=xz.device)
    check(_L().gllm_seq_conv_silu(_p(xz), xz.stride(0), t, seq_lens.shape[0], channels, _p(w), _p(b), w.shape[1],
                                  _p(conv_state), _p(rec_slots), _p(seq_lens), _p(query_start_loc), _p(out), _f32(xz),
                                  0 if act == "silu" else 1, _p(in_bias), stream_ptr()), "seq_conv_silu")
    sm100._count(2 if conv_state is not None else 1)
    return out


def selective_scan(xc, dt_raw, proj, xz, a, d_skip, dt_bias, ssm_state, rec_slots, seq_lens, query_start_loc,
                   channels, nstate, dt_rank):
    assert xc.is_contiguous() and dt_raw.is_contiguous() and proj.stride(1) == 1 and xz.stride(1) == 1
    assert a.dtype == torch.float32 and a.is_contiguous()
    out = torch.empty_like(xc)
    # long chunks of few sequences: 4 threads per channel (more warps in flight); decode-like batches: 1
    nseq = seq_lens.shape[0]
    parts = 4 if (nstate % 4 == 0 and nstate >= 8 and xc.shape[0] >= 16 * nseq and nseq * channels < (1 << 20)) else 1
    check(_L().gllm_seq_selective_scan(_p(xc), _p(dt_raw), _p(proj), proj.stride(0), _p(xz), xz.stride(0), _p(a),
                                       _p(d_skip), _p(dt_bias), _p(ssm_state), _p(rec_slots), _p(seq_lens),
                                       _p(query_start_loc), seq_lens.shape[0], channels, nstate, dt_rank, _p(out),
                                       _f32(xc), parts, stream_ptr()), "seq_selective_scan")
    sm100._count()
    return out


def relu2(x):
    x = x.contiguous()
    out = torch.empty_like(x)
    check(_L().gllm_seq_relu2(_p(x), _p(out), x.numel(), _f32(x), stream_ptr()), "seq_relu2")
    sm100._count()
    return out


def postnorm(x, y, alpha, w, eps, out_dtype):
    assert x.dtype == torch.float32 and x.is_contiguous() and y.stride(1) == 1 and y.dtype == w.dtype
    t, width = x.shape
    out = None if out_dtype == torch.float32 else torch.empty(t, width, dtype=out_dtype, device=x.device)
    check(_L().gllm_seq_postnorm(_p(x), _p(y), y.stride(0), _p(w), _p(out), t, width, float(alpha), float(eps),
                                 _f32(y), stream_ptr()), "seq_postnorm")
    sm100._count()
    return x if out is None else out


def qk_norm_rope_kv_write(qkv, num_heads, num_kv_heads, dim, v_dim, q_norm_w, k_norm_w, eps, positions, rot_dims,
                          rot_base, k_cache, v_cache, slots, freqs=None, mag=1.0):
    import math
    t = qkv.shape[0]
    assert qkv.stride(1) == 1 and k_cache.dtype == qkv.dtype and positions.dim() == 1
    assert freqs is None or (freqs.dtype == torch.float64 and freqs.is_contiguous() and
                             freqs.shape[0] == rot_dims // 2)
    q = torch.empty(t, num_heads * dim, dtype=qkv.dtype, device=qkv.device)
    ps = k_cache.shape[3]
    check(_L().gllm_seq_qk_norm_rope_kv_write(_p(qkv), qkv.stride(0), t, num_heads, num_kv_heads, dim, v_dim,
                                              _p(q_norm_w), _p(k_norm_w), float(eps), _p(positions), int(rot_dims),
                                              math.log2(rot_base) if rot_dims > 0 else 0.0, _p(q), _p(k_cache),
                                              _p(v_cache), _p(slots), ps, k_cache.shape[4], v_cache.shape[4],
                                              _f32(qkv), _p(freqs), float(mag), stream_ptr()),
          "seq_qk_norm_rope_kv_write")
    sm100._count()
    return q


def linear_state_scan(q, k, v, beta, a, neg_a, dt_bias, decay, state, rec_slots, seq_lens, query_start_loc, heads,
                      qk_heads, dim, v_dim, silu_in, unit_qk, q_scale, delta, zk=None, zk_bias=None, inv_tau=1.0):
    t = q.shape[0]
    for x in (q, k, v, beta, a, zk):
        assert x is None or (x.stride(1) == 1 and x.dtype == q.dtype)
    assert state is None or (state.dtype == torch.float32 and state.is_contiguous())
    assert (decay is not None) + (a is not None) + (zk is not None) == 1 and (not delta or beta is not None)
    assert zk_bias is None or (zk_bias.dtype == torch.float32 and zk_bias.is_contiguous())
    out = torch.empty(t, heads * v_dim, dtype=torch.float32, device=q.device)
    ld = lambda x: x.stride(0) if x is not None else 0   # noqa: E731
    gk = None
    if zk is not None:
        # the decays sigmoid(zk + bias)^inv_tau in fp32, once per (token, key channel) and off the serial chain
        gk = torch.empty(t, heads * dim, dtype=torch.float32, device=q.device)
        check(_L().gllm_seq_key_decay(_p(zk), zk.stride(0), _p(zk_bias), float(inv_tau), _p(gk), t, heads * dim,
                                      _f32(zk), stream_ptr()), "seq_key_decay")
        sm100._count()
    # long chunks on a grid that leaves SMs idle: 8 lanes per state column (twice the warps on the serial chain;
    # 4 x 2048 tokens, head size 128: 8 heads 1.9x faster, 32 heads 1.4x slower than 4 lanes). Otherwise 4: decode-like
    # batches want the wider contiguous runs of the state rows, whose read + write is all that a single token costs
    nseq = seq_lens.shape[0]
    blocks = nseq * heads * ((v_dim + 31) // 32)
    parts = 8 if (dim > 64 and t >= 16 * nseq and blocks <= 2 * _NUM_SMS) else 4
    check(_L().gllm_seq_linear_state(_p(q), q.stride(0), _p(k), k.stride(0), _p(v), v.stride(0), _p(beta), ld(beta),
                                     _p(a), ld(a), _p(neg_a), _p(dt_bias), _p(decay), _p(state), _p(rec_slots),
                                     _p(seq_lens), _p(query_start_loc), seq_lens.shape[0], heads, qk_heads, dim, v_dim,
                                     int(silu_in), int(unit_qk), float(q_scale), int(delta), _p(out), _f32(q),
                                     parts, _p(gk), ld(gk), stream_ptr()), "seq_linear_state")
    sm100._count()
    return out


def gated_group_norm(o, gate, w, group, eps, act, out_scale=1.0, out=None, out_dtype=None):
    t, n = o.shape
    assert o.dtype == torch.float32 and o.is_contiguous() and gate.stride(1) == 1 and gate.dtype == w.dtype
    if out is None:
        out = torch.empty(t, n, dtype=out_dtype or gate.dtype, device=o.device)
    assert out.stride(1) == 1 and out.dtype == gate.dtype
    check(_L().gllm_seq_gated_group_norm(_p(o), n, _p(gate), gate.stride(0), _p(w), w.shape[0], int(group), float(eps),
                                         1 if act == "sigmoid" else 0, float(out_scale), _p(out), out.stride(0), t,
                                         _f32(gate), stream_ptr()), "seq_gated_group_norm")
    sm100._count()
    return out


def silu_mul(gu):
    t, f = gu.shape[0], gu.shape[1] // 2
    assert gu.stride(1) == 1
    out = torch.empty(t, f, dtype=gu.dtype, device=gu.device)
    check(_L().gllm_seq_silu_mul(_p(gu), gu.stride(0), t, f, _p(out), _f32(gu), stream_ptr()), "seq_silu_mul")
    sm100._count()
    return out


_ROUTER_MMA_MIN_TOKENS = 256
_NUM_SMS = 148


def router_logits(h, w, force: Optional[str] = None):
    """fp32 router logits h . w^T [T, E]. Small batches: one warp per (token, expert); large bf16 batches on the
    tensor cores (mma.sync, fp32 accumulation and fp32 result); large fp32 batches: the plain GEMM with fp32 result."""
    t, width = h.shape
    e = w.shape[0]
    assert h.stride(1) == 1 and w.is_contiguous() and h.dtype == w.dtype
    logits = torch.empty(t, e, dtype=torch.float32, device=h.device)
    L, st = _L(), stream_ptr()
    mma_ok = h.dtype == torch.bfloat16 and width % 16 == 0 and h.stride(0) % 2 == 0 and h.data_ptr() % 4 == 0
    if force in (None, "mma") and h.dtype == torch.bfloat16 and (t >= _ROUTER_MMA_MIN_TOKENS or force == "mma") \
            and mma_f32out_ok(h.unsqueeze(1), w.unsqueeze(0)):
        return gemm_mma_f32out(h.unsqueeze(1), w.unsqueeze(0), logits.unsqueeze(1)).squeeze(1)
    path = force or ("token" if t < _ROUTER_MMA_MIN_TOKENS else ("mma" if mma_ok else "gemm"))
    if path == "token":
        check(L.gllm_seq_router_logits(_p(h), h.stride(0), _p(w), t, width, e, _p(logits), _f32(h), st),
              "seq_router_logits")
    elif path == "mma":
        check(L.gllm_seq_router_logits_mma(_p(h), h.stride(0), _p(w), t, width, e, _p(logits), st),
              "seq_router_logits_mma")
    else:
        check(L.gllm_seq_gemm_simt_f32out(_p(h), h.stride(0), _p(w), w.stride(0), _p(logits), e, t, e, width, _f32(h),
                                          st), "seq_gemm_simt_f32out")
    sm100._count()
    return logits


def mma_f32out_ok(a, w) -> bool:
    """a [T, B, K] (strided), w [B, N, K] contiguous, both bf16: shapes the fp32-result tensor-core product takes."""
    k = a.shape[2]
    return a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and k % 32 == 0 and a.stride(2) == 1 and \
        a.stride(0) % 8 == 0 and (a.shape[1] == 1 or a.stride(1) % 8 == 0) and a.data_ptr() % 16 == 0 and \
        w.is_contiguous() and w.data_ptr() % 16 == 0


def gemm_mma_f32out(a, w, out):
    """out[:, b, :] (fp32) = a[:, b, :] @ w[b].T with bf16 operands on mma.sync, fp32 accumulation and result."""
    t, b, k = a.shape
    n = w.shape[1]
    assert out.dtype == torch.float32 and out.shape == (t, b, n) and out.stride(2) == 1 and mma_f32out_ok(a, w)
    check(_L().gllm_seq_gemm_mma_f32out(_p(a), a.stride(0), a.stride(1) if b > 1 else 0, _p(w), k, n * k, _p(out),
                                        out.stride(0), out.stride(1) if b > 1 else 0, t, n, k, b, stream_ptr()),
          "seq_gemm_mma_f32out")
    sm100._count()
    return out


def router_topk(h, w, top_k, force: Optional[str] = None):
    """fp32 router logits (`router_logits`), then the top_k largest per token and the softmax over the chosen (one
    warp per token)."""
    t, e = h.shape[0], w.shape[0]
    assert e <= 1024
    wout = torch.empty(t, top_k, dtype=torch.float32, device=h.device)
    ids = torch.empty(t, top_k, dtype=torch.int32, device=h.device)
    logits = router_logits(h, w, force)
    L, st = _L(), stream_ptr()
    check(L.gllm_seq_router_select(_p(logits), t, e, top_k, _p(wout), _p(ids), st), "seq_router_select")
    sm100._count()
    return wout, ids


def routed_experts(h, w13, w2, weights, ids, limit: float = 0.0, alpha: float = 1.702, n_real: Optional[int] = None,
                   ungated: bool = False):
    """Plain per-slot experts. limit > 0: the clamped gated activation; ids >= n_real: identity experts; `ungated`:
    w13 is [E, F, W] (up rows only) and the activation relu(up h)^2."""
    t, width = h.shape
    n_real = w13.shape[0] if n_real is None else n_real
    f, k = (w13.shape[1] if ungated else w13.shape[1] // 2), ids.shape[1]
    assert h.stride(1) == 1 and w13.is_contiguous() and w2.is_contiguous() and weights.is_contiguous()
    act = torch.empty(t * k, f, dtype=h.dtype, device=h.device)
    out = torch.empty(t, width, dtype=h.dtype, device=h.device)
    check(_L().gllm_seq_routed_experts(_p(h), h.stride(0), _p(w13), _p(w2), _p(ids), _p(weights), t, k, width, f,
                                       _p(act), _p(out), _f32(h), int(n_real), float(limit), float(alpha),
                                       int(ungated), stream_ptr()), "seq_routed_experts")
    sm100._count(2)
    return out


def softcap(z, cap):
    assert z.stride(1) == 1
    check(_L().gllm_seq_softcap(_p(z), z.stride(0), z.shape[0], z.shape[1], float(cap), _f32(z), stream_ptr()),
          "seq_softcap")
    sm100._count()
    return z
