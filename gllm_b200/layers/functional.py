"""Device-directed op entry points used by the model code.

CUDA tensors always run the hand-written sm_100a kernels (`ops.sm100`); CPU tensors run the
PyTorch oracle (`ops.ref`) — that is the CPU plumbing/test path only, never a GPU fallback.
"""
from __future__ import annotations

from typing import Optional

import torch

from gllm_b200.ops import ref


def _sm():
    from gllm_b200.ops import sm100
    return sm100


def linear(x, w, bias=None, out=None):
    if isinstance(w, tuple):  # (e4m3 weight, fp32 block scale_inv): block-scaled fp8 GEMM
        if x.is_cuda:
            return _sm().linear_fp8_block(x, w[0], w[1], bias, out=out)
        return ref.linear_fp8_block(x, w[0], w[1], bias)
    if x.is_cuda:
        return _sm().linear(x, w, bias, out=out)
    return ref.linear(x, w, bias)


def linear_silu_mul(x, w_interleaved):
    if x.is_cuda:
        return _sm().linear_silu_mul(x, w_interleaved)
    return ref.linear_silu_mul(x, w_interleaved)


def rmsnorm(x, w, eps, residual=None, out=None):
    """-> (normed, residual_out). With `residual`, computes residual += x first (in place on GPU)."""
    if x.is_cuda:
        return _sm().rmsnorm(x, w, eps, residual, out=out)
    o, r = ref.rmsnorm(x, w, eps, residual)
    if out is not None:
        out.copy_(o)
        o = out
    if residual is not None:
        residual.copy_(r)  # same in-place contract as the GPU kernel
        r = residual
    return o, r


def silu_and_mul(x):
    if x.is_cuda:
        return _sm().silu_and_mul(x)
    return ref.silu_and_mul(x)


def embedding(ids, table, vocab_start=0, vocab_end=None):
    if table.is_cuda:
        return _sm().embedding(ids, table, vocab_start, vocab_end)
    return ref.embedding(ids, table, vocab_start, vocab_end)


def gather_rows(src, idx):
    if src.is_cuda:
        return _sm().gather_rows(src.contiguous(), idx)
    return src[idx.long()]


def rope_kv_write(q, k, v, positions, cos_sin, rot_dim, neox, q_norm_w, k_norm_w, eps, k_cache, v_cache, slots,
                  mrope_section=None):
    if q.is_cuda:
        return _sm().rope_kv_write(q, k, v, positions, cos_sin, rot_dim, neox, q_norm_w, k_norm_w, eps, k_cache,
                                   v_cache, slots, mrope_section)
    return ref.rope_kv_write(q, k, v, positions, cos_sin, rot_dim, neox, q_norm_w, k_norm_w, eps, k_cache,
                             v_cache, slots, mrope_section)


def paged_attention(q, k_cache, v_cache, inp, scale, num_q_heads, head_dim):
    """`inp` is the worker's InputData (device batch state)."""
    if q.is_cuda:
        return _sm().paged_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc, scale,
                                     num_q_heads, head_dim, inp.padded_tokens or inp.num_decode_seqs,
                                     inp.padded_tokens or inp.num_seqs, inp.max_q_len, inp.max_seq_len,
                                     splits=inp.decode_splits)
    return ref.paged_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc, scale,
                               num_q_heads, head_dim)


def sample(logits, inp, seen_bits=None, seed=0, step=None):
    b = logits.shape[0]
    if logits.is_cuda:
        sm = _sm()
        if inp.batch is not None and inp.batch.all_greedy and not inp.batch.need_penalty:
            return sm.sample(logits)
        return sm.sample(logits, inp.temperature[:b], inp.top_k[:b], inp.top_p[:b],
                         inp.rep_penalty[:b] if seen_bits is not None else None, seen_bits,
                         inp.state_slot[:b] if seen_bits is not None else None, seed=seed, step=step)
    seen_mask = None
    if seen_bits is not None:
        v = logits.shape[1]
        rows = seen_bits[inp.state_slot[:b].long()]
        bits = (rows.unsqueeze(-1) >> torch.arange(32, dtype=torch.int32)) & 1
        seen_mask = bits.reshape(b, -1)[:, :v].bool()
    g = torch.Generator().manual_seed(seed + (int(step) if step is not None else 0))
    return ref.sample(logits, inp.temperature[:b], inp.top_k[:b], inp.top_p[:b],
                      inp.rep_penalty[:b] if seen_bits is not None else None, seen_mask, generator=g)


# -- fp32-residual blocks, windowed sink attention, recurrent mixers (csrc/seq) ----------------------------
def _seq():
    from gllm_b200.ops import sm100_seq
    return sm100_seq


def linear_any(x, w, bias=None):
    """y = x @ w.T (+ bias, added to the fp32 accumulator) for bf16 or fp32 operands of any shape: the tcgen05 GEMM
    when it applies (bf16, 16-byte aligned rows), else the plain fp32-accumulating kernel (true fp32 for fp32
    operands, no TF32)."""
    if x.is_cuda:
        return _seq().linear_any(x, w, bias)
    return ref.linear(x, w, bias)


def embedding_scaled(ids, table, scale):
    if table.is_cuda:
        return _seq().embedding_scaled(ids, table, scale)
    return ref.embedding_scaled(ids, table, scale)


def resid_norm(x, y, w_post, add, w_pre, eps, out_dtype, emit_plain=False, post_scale=None, w_offset=0.0,
               out_mul=1.0):
    fn = _seq().resid_norm if x.is_cuda else ref.resid_norm
    return fn(x, y, w_post, add, w_pre, eps, out_dtype, emit_plain, post_scale, w_offset, out_mul)


def qk_norm_kv_write(qk, num_heads, num_kv_heads, dim, q_norm_w, k_norm_w, eps, k_cache, v_cache, slots):
    if qk.is_cuda:
        return _seq().qk_norm_kv_write(qk, num_heads, num_kv_heads, dim, q_norm_w, k_norm_w, eps, k_cache, v_cache,
                                       slots)
    return ref.qk_norm_kv_write(qk, num_heads, num_kv_heads, dim, q_norm_w, k_norm_w, eps, k_cache, v_cache, slots)


def window_attention(q, k_cache, v_cache, inp, scale, num_q_heads, head_dim, window, sink):
    if q.is_cuda:
        return _seq().window_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc,
                                       inp.positions, scale, num_q_heads, head_dim, window, sink,
                                       num_decode_seqs=inp.padded_tokens or inp.num_decode_seqs,
                                       max_q_len=inp.max_q_len)
    return ref.window_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc, scale,
                                num_q_heads, head_dim, window, sink)


def causal_conv_silu(xz, channels, w, b, conv_state, inp, act="silu", in_bias=None):
    """Depthwise causal convolution with carried taps; `act` "silu" | "none"; `in_bias` is added to every input
    that exists (not to the zeros before a sequence's start)."""
    slots = inp.rec_slots if conv_state is not None else None
    fn = _seq().causal_conv_silu if xz.is_cuda else ref.causal_conv_silu
    return fn(xz, channels, w, b, conv_state, slots, inp.seq_lens, inp.query_start_loc, act, in_bias)


def selective_scan(xc, dt_raw, proj, xz, a, d_skip, dt_bias, ssm_state, inp, channels, nstate, dt_rank):
    slots = inp.rec_slots if ssm_state is not None else None
    fn = _seq().selective_scan if xc.is_cuda else ref.selective_scan
    return fn(xc, dt_raw, proj, xz, a, d_skip, dt_bias, ssm_state, slots, inp.seq_lens, inp.query_start_loc,
              channels, nstate, dt_rank)


def relu2(x):
    if x.is_cuda:
        return _seq().relu2(x)
    return ref.relu2(x)


# -- norm-after-sum blocks, rotary chunk attention, matrix-state recurrences, routed feed-forward (csrc/seq) ---
def postnorm(x, y, alpha, w, eps, out_dtype):
    """x <- rms(alpha * x + y) * w in place on the fp32 stream; returns x in the compute dtype."""
    if x.is_cuda:
        return _seq().postnorm(x, y, alpha, w, eps, out_dtype)
    return ref.postnorm(x, y, alpha, w, eps, out_dtype)


def qk_norm_rope_kv_write(qkv, num_heads, num_kv_heads, dim, v_dim, q_norm_w, k_norm_w, eps, positions, rot_dims,
                          rot_base, k_cache, v_cache, slots, freqs=None, mag=1.0):
    """num_kv_heads == 0: the rows hold queries only (keys and values are another layer's); `freqs` (fp64 per
    pair) and `mag`: scaled rotary frequencies and the factor on cos / sin."""
    fn = _seq().qk_norm_rope_kv_write if qkv.is_cuda else ref.qk_norm_rope_kv_write
    return fn(qkv, num_heads, num_kv_heads, dim, v_dim, q_norm_w, k_norm_w, eps, positions, rot_dims, rot_base,
              k_cache, v_cache, slots, freqs, mag)


def masked_attention(q, k_cache, v_cache, inp, scale, num_q_heads, head_dim, v_dim, window=None, chunk=None, sink=None,
                     out_scale=1.0, out=None, softcap=0.0):
    """Paged causal attention with a sliding window and / or a chunk mask, values of their own width, an optional
    per-head sink logit in the denominator and an optional tanh cap on the scaled scores."""
    if q.is_cuda:
        return _seq().window_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc,
                                       inp.positions, scale, num_q_heads, head_dim, window, sink,
                                       num_decode_seqs=inp.padded_tokens or inp.num_decode_seqs,
                                       max_q_len=inp.max_q_len, chunk=chunk, v_dim=v_dim, out_scale=out_scale, out=out,
                                       softcap=softcap)
    return ref.window_attention(q, k_cache, v_cache, inp.block_table, inp.seq_lens, inp.query_start_loc, scale,
                                num_q_heads, head_dim, window, sink, chunk=chunk, v_dim=v_dim, out_scale=out_scale,
                                out=out, softcap=softcap)


def linear_state_scan(q, k, v, beta, a, neg_a, dt_bias, decay, state, inp, heads, qk_heads, dim, v_dim, silu_in,
                      unit_qk, q_scale, delta, zk=None, zk_bias=None, inv_tau=1.0):
    slots = inp.rec_slots if state is not None else None
    fn = _seq().linear_state_scan if q.is_cuda else ref.linear_state_scan
    return fn(q, k, v, beta, a, neg_a, dt_bias, decay, state, slots, inp.seq_lens, inp.query_start_loc, heads,
              qk_heads, dim, v_dim, silu_in, unit_qk, q_scale, delta, zk, zk_bias, inv_tau)


def gated_group_norm(o, gate, w, group, eps, act, out_scale=1.0, out=None, out_dtype=None):
    fn = _seq().gated_group_norm if o.is_cuda else ref.gated_group_norm
    return fn(o, gate, w, group, eps, act, out_scale, out, out_dtype)


def silu_mul(gu):
    if gu.is_cuda:
        if gu.dtype == torch.bfloat16 and gu.is_contiguous():
            return _sm().silu_and_mul(gu)
        return _seq().silu_mul(gu)
    return ref.silu_mul(gu)


def router_topk(h, w, top_k):
    if h.is_cuda:
        return _seq().router_topk(h, w, top_k)
    return ref.router_topk(h, w, top_k)


def routed_experts(h, w13, w2, weights, ids, interleaved):
    """sum_k weights[t, k] * expert_{ids[t, k]}(h[t]); w13 [E, 2F, W] = [gate rows ; up rows] (per-64 interleaved
    when `interleaved`: the grouped tcgen05 GEMM's layout), w2 [E, W, F]."""
    if h.is_cuda:
        if interleaved:
            from gllm_b200.ops import sm100_moe
            return sm100_moe.fused_experts(h, w13, w2, weights, ids, None)
        return _seq().routed_experts(h, w13, w2, weights, ids)
    return ref.fused_experts(h, w13, w2, weights, ids, None)


def softcap(z, cap):
    if z.is_cuda:
        return _seq().softcap(z, cap)
    return ref.softcap(z, cap)


# -- branch-norm blocks, key-decay linear attention, latent attention, gated linear recurrent unit, grouped routing
# with identity experts and clamped gated experts (csrc/seq/latent_ops.cu) ------------------------------------
def _lat():
    from gllm_b200.ops import sm100_latent
    return sm100_latent


def rms_rows(x, w, eps):
    return _lat().rms_rows(x, w, eps) if x.is_cuda else ref.rms_rows(x, w, eps)


def block_linear(x, w, out_dtype=None):
    """Block-diagonal linear map x [T, B * K] x w [B, N, K] -> [T, B * N]."""
    return _lat().block_linear(x, w, out_dtype) if x.is_cuda else ref.block_linear(x, w, out_dtype)


def linear_batched(a, w, out):
    """out[:, b, :] = a[:, b, :] @ w[b].T (strided views allowed): the tcgen05 GEMM's batched mode for aligned
    bf16 operands, the plain batched kernel otherwise (true fp32 for fp32 operands)."""
    return _lat().linear_batched(a, w, out) if a.is_cuda else ref.linear_batched(a, w, out)


def rglru_scan(u, gates, gate_bias, c_decay, y_pre, y_bias, state, inp, block, out_dtype):
    slots = inp.rec_slots if state is not None else None
    if u.is_cuda:
        return _lat().rglru_scan(u, gates, gate_bias, c_decay, y_pre, y_bias, state, slots, inp.seq_lens,
                                 inp.query_start_loc, block, out_dtype, max_q_len=getattr(inp, "max_q_len", None))
    return ref.rglru_scan(u, gates, gate_bias, c_decay, y_pre, y_bias, state, slots, inp.seq_lens,
                          inp.query_start_loc, block, out_dtype)


def latent_norm_rope_write(q, dkv, rank, rot, norm_w, eps, positions, freqs, mag, q_full, cache, slots):
    fn = _lat().latent_norm_rope_write if q.is_cuda else ref.latent_norm_rope_write
    return fn(q, dkv, rank, rot, norm_w, eps, positions, freqs, mag, q_full, cache, slots)


def latent_attention(q_full, cache, inp, scale, rank):
    """Causal multi-query attention over the paged latent cache (values = the first `rank` columns of the keys)."""
    if q_full.is_cuda:
        return _lat().latent_attention(q_full, cache, inp, scale, rank)
    return ref.latent_attention(q_full, cache, inp.block_table, inp.seq_lens, inp.query_start_loc, scale, rank)


def grouped_router(h, w, correction, top_k, n_groups, keep_groups, scale, score="softmax", group_top=1, renorm=True):
    fn = _lat().grouped_router if h.is_cuda else ref.grouped_router
    return fn(h, w, correction, top_k, n_groups, keep_groups, scale, score, group_top, renorm)


def glu_clamp(gu, limit, alpha=1.702):
    return _lat().glu_clamp(gu, limit, alpha) if gu.is_cuda else ref.glu_clamp(gu, limit, alpha)


def linear_glu_clamp(x, w_interleaved, limit, alpha=1.702):
    """glu_clamp(x @ w^T) as the tcgen05 GEMM's gated epilogue (gate / up rows interleaved per 128)."""
    if x.is_cuda:
        return _lat().linear_glu_clamp(x, w_interleaved, limit, alpha)
    return ref.linear_glu_clamp(x, w_interleaved, limit, alpha)


def routed_glu_experts(h, w13, w2, weights, ids, limit, interleaved, alpha=1.702, n_all=None):
    """Clamped gated experts; ids >= the number of experts are identity experts (n_all: experts + identity)."""
    if h.is_cuda:
        return _lat().routed_glu_experts(h, w13, w2, weights, ids, limit, interleaved, alpha, n_all)
    return ref.routed_glu_experts(h, w13, w2, weights, ids, limit, alpha)


# -- hashed pair embedding with a carried previous token (csrc/seq/pair_ops.cu), ungated squared-ReLU experts ----
def _pair():
    from gllm_b200.ops import sm100_pair
    return sm100_pair


def embedding_pair_hash(inp, table, pair_table, mul_prev, mul_cur, buckets, prev_state):
    """fp32 stream: table[token] + pair_table[hash(previous token, token)]; the token before a portion's first row
    is carried in prev_state [state slots] (None: no history, e.g. a memory probe)."""
    slots = inp.rec_slots if prev_state is not None else None
    fn = _pair().embedding_pair_hash if table.is_cuda else ref.embedding_pair_hash
    return fn(inp.tokens, table, pair_table, mul_prev, mul_cur, buckets, inp.positions, prev_state, slots,
              inp.query_start_loc)


def routed_relu2_experts(h, w1, w2, weights, ids, grouped):
    """sum_k weights[t, k] * down_e(relu(up_e h)^2); `grouped`: the grouped tcgen05 GEMM pair with the squared-ReLU
    epilogue on the first product, otherwise the plain per-slot kernels."""
    if h.is_cuda:
        return _pair().routed_relu2_experts(h, w1, w2, weights, ids, grouped)
    return ref.routed_relu2_experts(h, w1, w2, weights, ids)
