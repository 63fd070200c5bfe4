"""Pure-PyTorch reference implementations of every op (CPU-capable).

These are the correctness oracle for the sm_100a kernels (tests compare against them in
fp32) and the execution path for the CPU plumbing tests (BASELINE config #1: scheduler +
paged-KV on CPU). They are NOT a product path: on a GPU box the engine always runs the
hand-written kernels in `gllm_b200.ops.sm100`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


def kv_slab(head_dim: int) -> int:
    """Width of the innermost KV-cache slab (64 on the product path)."""
    return 64 if head_dim % 64 == 0 else head_dim


def kv_cache_shape(num_pages: int, num_kv_heads: int, head_dim: int, page_size: int):
    w = kv_slab(head_dim)
    return (num_pages, num_kv_heads, head_dim // w, page_size, w)


# ----------------------------------------------------------------------------------------------
# dense ops
# ----------------------------------------------------------------------------------------------
def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, residual: Optional[torch.Tensor] = None):
    """Returns (normed, new_residual). new_residual is None when residual is None."""
    if residual is not None:
        r = (x.float() + residual.float()).to(x.dtype)
        xf = r.float()
    else:
        r = None
        xf = x.float()
    var = xf.pow(2).mean(-1, keepdim=True)
    out = (xf * torch.rsqrt(var + eps) * w.float()).to(x.dtype)
    return out, r


def linear(x: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    return F.linear(x, w, bias)


def silu_and_mul(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return (F.silu(x[..., :d].float()) * x[..., d:].float()).to(x.dtype)


def interleave_gate_up(w: torch.Tensor, block: int = 128) -> torch.Tensor:
    """[2I, K] (gate rows then up rows) -> per-`block` interleaved layout used by the fused
    SiLU-gate GEMM epilogue: tile j = [gate[j*b:(j+1)*b]; up[j*b:(j+1)*b]]."""
    two_i, k = w.shape
    i = two_i // 2
    assert i % block == 0, (i, block)
    g = w[:i].reshape(i // block, block, k)
    u = w[i:].reshape(i // block, block, k)
    return torch.cat([g, u], dim=1).reshape(two_i, k).contiguous()


def linear_silu_mul(x: torch.Tensor, w_interleaved: torch.Tensor, block: int = 128) -> torch.Tensor:
    y = F.linear(x, w_interleaved)
    t, two_i = y.shape
    y = y.reshape(t, two_i // (2 * block), 2, block)
    return (F.silu(y[:, :, 0].float()) * y[:, :, 1].float()).to(x.dtype).reshape(t, two_i // 2)


def embedding(ids: torch.Tensor, table: torch.Tensor, vocab_start: int = 0, vocab_end: Optional[int] = None):
    vocab_end = table.shape[0] + vocab_start if vocab_end is None else vocab_end
    mask = (ids >= vocab_start) & (ids < vocab_end)
    local = torch.where(mask, ids - vocab_start, torch.zeros_like(ids)).long()
    out = F.embedding(local, table)
    out = out * mask.unsqueeze(-1).to(out.dtype)
    return out


# ----------------------------------------------------------------------------------------------
# rope + kv cache write
# ----------------------------------------------------------------------------------------------
def build_cos_sin_cache(rot_dim: int, max_pos: int, base: float, inv_freq: Optional[torch.Tensor] = None,
                        mscale: float = 1.0) -> torch.Tensor:
    """fp32 [max_pos, rot_dim]: cos | sin."""
    if inv_freq is None:
        inv_freq = 1.0 / (base ** (torch.arange(0, rot_dim, 2, dtype=torch.float32) / rot_dim))
    t = torch.arange(max_pos, dtype=torch.float32)
    freqs = torch.outer(t, inv_freq.float())
    return torch.cat([freqs.cos() * mscale, freqs.sin() * mscale], dim=-1).contiguous()


def _rope_one(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, rot: int, neox: bool) -> torch.Tensor:
    # x [T, H, D] fp32; cos/sin [T, rot/2]
    xr, xp = x[..., :rot], x[..., rot:]
    c, s = cos.unsqueeze(1), sin.unsqueeze(1)
    if neox:
        x1, x2 = xr[..., : rot // 2], xr[..., rot // 2:]
        o = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1)
    else:
        x1, x2 = xr[..., 0::2], xr[..., 1::2]
        o = torch.stack([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).flatten(-2)
    return torch.cat([o, xp], dim=-1)


def write_kv_cache(k: torch.Tensor, v: Optional[torch.Tensor], k_cache: torch.Tensor,
                   v_cache: Optional[torch.Tensor], slots: torch.Tensor):
    """k/v [T, Hkv, D]; caches [pages, Hkv, D/W, page, W]; slots [T] (negative = skip)."""
    pages, hkv, nslab, page_size, w = k_cache.shape
    valid = slots >= 0
    if not bool(valid.all()):
        k, slots_v = k[valid], slots[valid]
        v = v[valid] if v is not None else None
    else:
        slots_v = slots
    page = (slots_v // page_size).long()
    off = (slots_v % page_size).long()
    t = k.shape[0]
    k_cache[page, :, :, off, :] = k.reshape(t, hkv, nslab, w).to(k_cache.dtype)
    if v is not None and v_cache is not None:
        v_cache[page, :, :, off, :] = v.reshape(t, hkv, nslab, w).to(v_cache.dtype)


def rope_kv_write(q: torch.Tensor, k: torch.Tensor, v: Optional[torch.Tensor], positions: torch.Tensor,
                  cos_sin: Optional[torch.Tensor], rot_dim: int, neox: bool,
                  q_norm_w: Optional[torch.Tensor], k_norm_w: Optional[torch.Tensor], eps: float,
                  k_cache: Optional[torch.Tensor], v_cache: Optional[torch.Tensor],
                  slots: Optional[torch.Tensor], mrope_section=None):
    """In place on q [T,Hq,D] and k [T,Hkv,D] (views allowed): optional per-head RMSNorm, RoPE,
    then K/V scatter into the paged cache."""
    dt = q.dtype
    qf, kf = q.float(), k.float()
    if q_norm_w is not None:
        qf = (qf * torch.rsqrt(qf.pow(2).mean(-1, keepdim=True) + eps) * q_norm_w.float()).to(dt).float()
    if k_norm_w is not None:
        kf = (kf * torch.rsqrt(kf.pow(2).mean(-1, keepdim=True) + eps) * k_norm_w.float()).to(dt).float()
    if rot_dim > 0 and cos_sin is not None:
        half = rot_dim // 2
        if mrope_section is not None and positions.dim() == 2:
            # positions [3, T]; pair index i picks the section's position row
            sec = torch.zeros(half, dtype=torch.long, device=positions.device)
            if len(mrope_section) > 3 and mrope_section[3]:   # interleaved THWTHW.. (Qwen3-VL)
                sec[1:mrope_section[1] * 3:3] = 1
                sec[2:mrope_section[2] * 3:3] = 2
            else:
                s0, s1 = mrope_section[0], mrope_section[1]
                sec[s0:s0 + s1] = 1
                sec[s0 + s1:] = 2
            cs = cos_sin.to(positions.device)[positions.long()]  # [3, T, rot]
            idx = sec.view(1, 1, half).expand(1, positions.shape[1], half)
            cos = torch.gather(cs[..., :half], 0, idx)[0]
            sin = torch.gather(cs[..., half:], 0, idx)[0]
        else:
            pos = positions if positions.dim() == 1 else positions[0]
            cs = cos_sin.to(pos.device)[pos.long()]
            cos, sin = cs[..., :half], cs[..., half:]
        qf = _rope_one(qf, cos, sin, rot_dim, neox)
        kf = _rope_one(kf, cos, sin, rot_dim, neox)
    q.copy_(qf.to(dt))
    k.copy_(kf.to(dt))
    if k_cache is not None and slots is not None:
        write_kv_cache(k, v, k_cache, v_cache, slots)


# ----------------------------------------------------------------------------------------------
# paged attention
# ----------------------------------------------------------------------------------------------
def gather_kv(cache: torch.Tensor, block_row: torch.Tensor, seq_len: int) -> torch.Tensor:
    """-> [seq_len, Hkv, D]"""
    pages, hkv, nslab, page_size, w = cache.shape
    n_pages = (seq_len + page_size - 1) // page_size
    blk = cache[block_row[:n_pages].long()]  # [n, Hkv, nslab, page, W]
    blk = blk.permute(0, 3, 1, 2, 4).reshape(n_pages * page_size, hkv, nslab * w)
    return blk[:seq_len]


def paged_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                    seq_lens: torch.Tensor, query_start_loc: torch.Tensor, scale: float,
                    num_q_heads: int, head_dim: int) -> torch.Tensor:
    """q [T, Hq*D] -> out [T, Hq*D]. Causal with context offset (chunked prefill / prefix cache):
    query i of a sequence sits at absolute position (seq_len - q_len + i)."""
    t = q.shape[0]
    hq, d = num_q_heads, head_dim
    hkv = k_cache.shape[1]
    g = hq // hkv
    out = torch.zeros(t, hq * d, dtype=q.dtype, device=q.device)
    qsl = query_start_loc.tolist()
    sl = seq_lens.tolist()
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        ql = q1 - q0
        if ql <= 0:
            continue
        kk = gather_kv(k_cache, block_table[s], sl[s]).float()  # [L, Hkv, D]
        vv = gather_kv(v_cache, block_table[s], sl[s]).float()
        qq = q[q0:q1].reshape(ql, hq, d).float()
        kk = kk.repeat_interleave(g, dim=1)
        vv = vv.repeat_interleave(g, dim=1)
        att = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        ctx = sl[s] - ql
        qi = torch.arange(ql, device=q.device).view(ql, 1) + ctx
        kj = torch.arange(sl[s], device=q.device).view(1, sl[s])
        att = att.masked_fill((kj > qi).unsqueeze(0), float("-inf"))
        p = torch.softmax(att, dim=-1)
        o = torch.einsum("hqk,khd->qhd", p, vv)
        out[q0:q1] = o.reshape(ql, hq * d).to(q.dtype)
    return out


def varlen_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: torch.Tensor,
                     scale: float, causal: bool) -> torch.Tensor:
    """Non-paged varlen attention (ViT towers, MLA prefill). q [T,H,Dq] k [T,Hk,Dq] v [T,Hk,Dv]."""
    out = torch.empty(q.shape[0], q.shape[1], v.shape[-1], dtype=q.dtype, device=q.device)
    cs = cu_seqlens.tolist()
    g = q.shape[1] // k.shape[1]
    for i in range(len(cs) - 1):
        a, b = cs[i], cs[i + 1]
        if b <= a:
            continue
        qq, kk, vv = q[a:b].float(), k[a:b].float(), v[a:b].float()
        if g > 1:
            kk, vv = kk.repeat_interleave(g, 1), vv.repeat_interleave(g, 1)
        att = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        if causal:
            n = b - a
            m = torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1)
            att = att.masked_fill(m.unsqueeze(0), float("-inf"))
        out[a:b] = torch.einsum("hqk,khd->qhd", torch.softmax(att, -1), vv).to(q.dtype)
    return out


# ----------------------------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------------------------
def apply_penalty_temperature(logits: torch.Tensor, temperature, rep_penalty, seen_mask) -> torch.Tensor:
    x = logits.float().clone()
    if rep_penalty is not None and seen_mask is not None:
        pen = rep_penalty.view(-1, 1).float()
        x = torch.where(seen_mask, torch.where(x > 0, x / pen, x * pen), x)
    if temperature is not None:
        t = temperature.float().clone()
        t[t <= 1e-5] = 1.0
        x = x / t.view(-1, 1)
    return x


def sample_filter(logits: torch.Tensor, temperature=None, top_k=None, top_p=None, rep_penalty=None,
                  seen_mask=None) -> torch.Tensor:
    """Returns the filtered probability distribution [B, V] the sampler draws from
    (reference semantics: gllm/layers/sampler.py:22-54)."""
    x = apply_penalty_temperature(logits, temperature, rep_penalty, seen_mask)
    b, v = x.shape
    if top_k is not None:
        k = top_k.clone().long()
        k[(k <= 0) | (k > v)] = v
        srt, _ = torch.sort(x, dim=-1, descending=True)
        thr = srt.gather(1, (k - 1).view(-1, 1))
        x = x.masked_fill(x < thr, float("-inf"))
    if top_p is not None:
        probs = torch.softmax(x, dim=-1)
        sp, si = torch.sort(probs, dim=-1, descending=True)
        cum = sp.cumsum(-1)
        # keep the smallest prefix whose mass reaches top_p
        drop = (cum - sp) >= top_p.view(-1, 1).float()
        drop_orig = torch.zeros_like(drop).scatter(1, si, drop)
        x = x.masked_fill(drop_orig, float("-inf"))
    return torch.softmax(x, dim=-1)


def sample(logits: torch.Tensor, temperature=None, top_k=None, top_p=None, rep_penalty=None,
           seen_mask=None, generator: Optional[torch.Generator] = None) -> torch.Tensor:
    b, v = logits.shape
    greedy = top_k is None or bool((top_k == 1).all())
    if greedy:
        x = apply_penalty_temperature(logits, temperature, rep_penalty, seen_mask)
        return x.argmax(-1).to(torch.int32)
    probs = sample_filter(logits, temperature, top_k, top_p, rep_penalty, seen_mask)
    g = torch.empty_like(probs).exponential_(1.0, generator=generator)
    tok = (probs / g).argmax(-1)
    # rows with top_k == 1 are exactly greedy
    return tok.to(torch.int32)


def vp_candidates(shard: torch.Tensor, valid: int, v_full: int, c: int, temperature=None, top_k=None, top_p=None,
                  rep_penalty=None, seen_mask=None, race_exp: Optional[torch.Tensor] = None,
                  vocab_offset: int = 0) -> torch.Tensor:
    """PyTorch model of csrc/sample/sampler.cu:vp_candidates_kernel — per-row record [B, 2c+4]: the shard's c best
    candidates after penalty / temperature (values, then token ids bit-cast to float), shard max, shard sum-exp, and
    for unfiltered rows the shard's exponential-race winner (score relative to the shard max, token id).
    `seen_mask` / `race_exp` are [B, valid] slices for this shard."""
    b = shard.shape[0]
    out = torch.full((b, 2 * c + 4), float("-inf"), dtype=torch.float32)
    out[:, c:2 * c] = 0.0
    out[:, 2 * c + 1] = 0.0
    out[:, 2 * c + 3] = 0.0
    if valid <= 0:
        return out
    x = apply_penalty_temperature(shard[:, :valid], temperature, rep_penalty, seen_mask)
    m = x.max(dim=-1).values
    out[:, 2 * c] = m
    out[:, 2 * c + 1] = torch.exp(x - m.view(-1, 1)).sum(-1)
    ck = min(c, valid)
    vals, idx = torch.topk(x, ck, dim=-1)
    out[:, :ck] = vals
    out[:, c:c + ck] = (idx + vocab_offset).to(torch.int32).view(torch.float32)
    k = top_k.long() if top_k is not None else torch.ones(b, dtype=torch.long)
    k = torch.where((k <= 0) | (k > v_full), torch.full_like(k, v_full), k)
    p = top_p.float() if top_p is not None else torch.ones(b)
    free = (k >= v_full) & (p >= 1.0)
    if bool(free.any()) and race_exp is not None:
        score = (x - m.view(-1, 1)) - torch.log(race_exp[:, :valid])
        best, bi = score.max(dim=-1)
        out[free, 2 * c + 2] = best[free]
        out[free, 2 * c + 3] = (bi[free] + vocab_offset).to(torch.int32).view(torch.float32)
    return out


def vp_final(gathered: torch.Tensor, c: int, v_full: int, top_k=None, top_p=None,
             generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """PyTorch model of vp_final_kernel: finish top-k / top-p / draw on the gathered candidates [tp, B, 2c+4] with
    the exact global normalisation (the mass of non-candidate tokens is known from the per-shard sum-exp)."""
    tp, b, _ = gathered.shape
    vals = gathered[:, :, :c].permute(1, 0, 2).reshape(b, tp * c)
    toks = gathered[:, :, c:2 * c].contiguous().view(torch.int32).permute(1, 0, 2).reshape(b, tp * c).long()
    ms, zs = gathered[:, :, 2 * c], gathered[:, :, 2 * c + 1]
    gm = ms.max(dim=0).values
    gz = (zs * torch.exp(torch.where(zs > 0, ms - gm.view(1, -1), torch.zeros_like(ms)))).sum(0)
    n = tp * c
    k = top_k.long() if top_k is not None else torch.ones(b, dtype=torch.long)
    k = torch.where((k <= 0) | (k > v_full), torch.full_like(k, v_full), k)
    p = top_p.float() if top_p is not None else torch.ones(b)
    out = torch.zeros(b, dtype=torch.int32)
    e_all = torch.empty(b, n).exponential_(1.0, generator=generator)
    for r in range(b):
        if k[r] >= v_full and p[r] >= 1.0:
            sc = gathered[:, r, 2 * c + 2] + (ms[:, r] - gm[r])
            out[r] = gathered[int(sc.argmax()), r, 2 * c + 3].view(torch.int32)
            continue
        x, t = vals[r], toks[r]
        order = torch.argsort(x, descending=True, stable=True)
        x, t = x[order], t[order]
        kk = int(min(k[r], n))
        if kk == 1:
            out[r] = t[0]
            continue
        prob = torch.exp(x - gm[r])
        keep = torch.zeros(n, dtype=torch.bool)
        keep[:kk] = True
        keep &= x >= x[kk - 1]
        keep |= (x == x[kk - 1]) & (x > float("-inf"))      # ties at the threshold survive (as in the kernel)
        mass = prob[keep].sum() if kk < v_full else gz[r]
        if p[r] < 1.0:
            cum = torch.cumsum(torch.where(keep, prob, torch.zeros_like(prob)), 0)
            keep &= (cum - prob) < p[r] * mass
        keep &= x > float("-inf")
        score = torch.where(keep, torch.log(prob) - torch.log(e_all[r]), torch.full_like(prob, float("-inf")))
        out[r] = t[int(score.argmax())]
    return out


# ----------------------------------------------------------------------------------------------
# MoE
# ----------------------------------------------------------------------------------------------
def topk_softmax(gate_logits: torch.Tensor, top_k: int, renormalize: bool):
    probs = torch.softmax(gate_logits.float(), dim=-1)
    w, ids = torch.topk(probs, top_k, dim=-1)
    if renormalize:
        w = w / w.sum(-1, keepdim=True)
    return w, ids.to(torch.int32)


def grouped_topk(gate_logits: torch.Tensor, top_k: int, renormalize: bool, num_groups: int,
                 topk_group: int, scoring: str = "softmax", bias: Optional[torch.Tensor] = None,
                 routed_scaling: float = 1.0):
    """DeepSeek group-limited routing (reference: gllm/layers/moe/topk.py:87-138)."""
    x = gate_logits.float()
    scores = torch.softmax(x, -1) if scoring == "softmax" else torch.sigmoid(x)
    t, e = scores.shape
    sel = scores + bias.float().view(1, -1) if bias is not None else scores
    grp = sel.view(t, num_groups, e // num_groups)
    if bias is not None:
        gscore = grp.topk(2, dim=-1)[0].sum(-1)
    else:
        gscore = grp.max(-1)[0]
    gidx = gscore.topk(topk_group, dim=-1)[1]
    gmask = torch.zeros_like(gscore).scatter(1, gidx, 1.0)
    mask = gmask.unsqueeze(-1).expand(t, num_groups, e // num_groups).reshape(t, e)
    masked = sel.masked_fill(mask == 0, float("-inf"))
    ids = masked.topk(top_k, dim=-1)[1]
    w = scores.gather(1, ids)
    if renormalize:
        w = w / (w.sum(-1, keepdim=True) + 1e-20)
    return w * routed_scaling, ids.to(torch.int32)


def fused_experts(x: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, topk_w: torch.Tensor,
                  topk_ids: torch.Tensor, expert_map: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [T,H]; w13 [E_local, 2I, H]; w2 [E_local, H, I]; ids are GLOBAL expert ids, expert_map maps
    global -> local (or -1). Non-local experts contribute zero (reference EP semantics)."""
    t, h = x.shape
    out = torch.zeros(t, h, dtype=torch.float32, device=x.device)
    e_local = w13.shape[0]
    ids = topk_ids.long()
    if expert_map is not None:
        ids = expert_map.to(ids.device)[ids].long()
    for e in range(e_local):
        tok, slot = torch.where(ids == e)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        hdn = silu_and_mul(F.linear(xe, w13[e]))
        ye = F.linear(hdn, w2[e]).float()
        out.index_add_(0, tok, ye * topk_w[tok, slot].float().unsqueeze(-1))
    return out.to(x.dtype)


# ----------------------------------------------------------------------------------------------
# fp8 block quantisation (reference semantics: gllm/layers/quantization/fp8.py)
# ----------------------------------------------------------------------------------------------
FP8_MAX = 448.0


def fp8_quant_group(x: torch.Tensor, group: int = 128):
    """Dynamic per-token-group quantisation -> (e4m3 tensor, fp32 scales [T, K/group])."""
    t, k = x.shape
    xg = x.float().reshape(t, k // group, group)
    amax = xg.abs().amax(-1).clamp_min(1e-10)
    scale = amax / FP8_MAX
    q = (xg / scale.unsqueeze(-1)).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q.reshape(t, k), scale


def fp8_block_dequant(w: torch.Tensor, scale_inv: torch.Tensor, block: int = 128) -> torch.Tensor:
    n, k = w.shape
    s = scale_inv.float().repeat_interleave(block, 0)[:n].repeat_interleave(block, 1)[:, :k]
    return w.float() * s


def linear_fp8_block(x: torch.Tensor, w: torch.Tensor, w_scale_inv: torch.Tensor,
                     bias: Optional[torch.Tensor] = None, block: int = 128) -> torch.Tensor:
    xq, xs = fp8_quant_group(x, block)
    xd = (xq.float().reshape(x.shape[0], -1, block) * xs.unsqueeze(-1)).reshape(x.shape[0], -1)
    wd = fp8_block_dequant(w, w_scale_inv, block)
    y = xd @ wd.t()
    if bias is not None:
        y = y + bias.float()
    return y.to(x.dtype)


def merge_attn_states(o1: torch.Tensor, lse1: torch.Tensor, o2: torch.Tensor, lse2: torch.Tensor):
    """LSE-weighted merge of two partial attention results. o [T,H,D], lse [T,H] (natural log)."""
    m = torch.maximum(lse1, lse2)
    w1, w2 = torch.exp(lse1 - m), torch.exp(lse2 - m)
    den = w1 + w2
    o = (o1.float() * (w1 / den).unsqueeze(-1) + o2.float() * (w2 / den).unsqueeze(-1)).to(o1.dtype)
    return o, m + torch.log(den)


# ----------------------------------------------------------------------------------------------
# fp32-residual blocks, windowed attention with a sink, short convolution + selective scan
# (unfused PyTorch forms of csrc/seq/*.cu; the CPU engine path and the kernels' numerics oracle)
# ----------------------------------------------------------------------------------------------
def embedding_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float) -> torch.Tensor:
    """fp32 residual stream from token ids: table[id] * scale."""
    return table[ids.long()].float() * scale


def resid_norm(x: torch.Tensor, y: Optional[torch.Tensor], w_post: Optional[torch.Tensor],
               add: Optional[torch.Tensor], w_pre: Optional[torch.Tensor], eps: float, out_dtype,
               emit_plain: bool = False, post_scale: Optional[torch.Tensor] = None, w_offset: float = 0.0,
               out_mul: float = 1.0):
    """In place on the fp32 stream x [T, W]:  x += rms(y) * w_post ;  x += add ;  returns rms(x) * w_pre cast to
    `out_dtype` (None when w_pre is None). Every step is optional. All arithmetic in fp32. `post_scale` [W] fp32
    (a layer scale) multiplies the normed branch element by element: x += rms(y) * w_post * post_scale. `emit_plain` (with w_pre None): returns the stream itself rounded to
    `out_dtype` — x for fp32 — for sublayers that read the stream without a norm in front. `w_offset` is added to
    both norm weights in fp32 (1.0 for weights stored around zero); `out_mul` multiplies the normed result before it
    is rounded (a logit scale folded into the final norm)."""
    if y is not None:
        yf = y.float()
        br = yf * torch.rsqrt((yf * yf).mean(-1, keepdim=True) + eps) * (w_post.float() + w_offset)
        x += br * post_scale.float() if post_scale is not None else br
    if add is not None:
        x += add
    if w_pre is None:
        if emit_plain:
            return x if out_dtype == torch.float32 else x.to(out_dtype)
        return None
    return (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps) * (w_pre.float() + w_offset) * out_mul).to(out_dtype)


def _cache_rows_write(cache: torch.Tensor, slots: torch.Tensor, rows: torch.Tensor):
    """rows [T, Hkv, D] -> paged cache [pages, Hkv, D/w, page_size, w] at flat slots (negative slots skipped)."""
    ps, w = cache.shape[3], cache.shape[4]
    keep = slots >= 0
    s = slots[keep].long()
    r = rows[keep]
    cache[s // ps, :, :, s % ps, :] = r.reshape(r.shape[0], r.shape[1], -1, w).to(cache.dtype)


def qk_norm_kv_write(qk: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, q_norm_w, k_norm_w, eps: float,
                     k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor) -> torch.Tensor:
    """qk [T, (H + G) * D] = [queries | keys]. Per-head RMS norm of q and k (weights optional); the normed key goes
    to the K cache, the key as projected to the V cache (the values of this attention are its raw keys).
    Returns the normed queries [T, H * D]."""
    t = qk.shape[0]
    q = qk[:, : num_heads * dim].reshape(t, num_heads, dim).float()
    k = qk[:, num_heads * dim:].reshape(t, num_kv_heads, dim).float()
    kn = k
    if q_norm_w is not None:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w.float()
    if k_norm_w is not None:
        kn = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm_w.float()
    _cache_rows_write(k_cache, slots, kn.to(qk.dtype))
    _cache_rows_write(v_cache, slots, k.to(qk.dtype))
    return q.to(qk.dtype).reshape(t, num_heads * dim)


def window_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, block_table: torch.Tensor,
                     seq_lens: torch.Tensor, query_start_loc: torch.Tensor, scale: float, num_q_heads: int,
                     head_dim: int, window: Optional[int], sink: Optional[torch.Tensor],
                     chunk: Optional[int] = None, v_dim: Optional[int] = None, out_scale: float = 1.0,
                     out: Optional[torch.Tensor] = None, softcap: float = 0.0) -> torch.Tensor:
    """Causal paged attention where position i sees j with 0 <= i - j < window (None: all of the past), and, with
    `chunk`, only j of its own chunk (floor(i / chunk) == floor(j / chunk), counted from position 0); the softmax
    denominator has one more term exp(sink[h]) that carries no value (None: plain softmax). Values may be wider or
    narrower than keys (`v_dim`); the result is multiplied by `out_scale` and written to `out` [T, H * v_dim] (any
    row stride) when given. `softcap` > 0 bounds every scaled score: s <- softcap * tanh(s / softcap), before the
    mask and the softmax."""
    t = q.shape[0]
    hq, d = num_q_heads, head_dim
    dv = d if v_dim is None else v_dim
    g = hq // k_cache.shape[1]
    if out is None:
        out = torch.zeros(t, hq * dv, dtype=q.dtype, device=q.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        ql = q1 - q0
        if ql <= 0:
            continue
        kk = gather_kv(k_cache, block_table[s], sl[s]).float().repeat_interleave(g, dim=1)
        vv = gather_kv(v_cache, block_table[s], sl[s]).float().repeat_interleave(g, dim=1)
        qq = q[q0:q1].reshape(ql, hq, d).float()
        att = torch.einsum("qhd,khd->hqk", qq, kk) * scale
        if softcap > 0:
            att = softcap * torch.tanh(att / softcap)
        qi = torch.arange(ql, device=q.device).view(ql, 1) + (sl[s] - ql)
        kj = torch.arange(sl[s], device=q.device).view(1, sl[s])
        dead = kj > qi
        if window is not None:
            dead = dead | (qi - kj >= window)
        if chunk is not None:
            dead = dead | (qi // chunk != kj // chunk)
        att = att.masked_fill(dead.unsqueeze(0), float("-inf"))
        if sink is not None:
            att = torch.cat([att, sink.float().view(hq, 1, 1).expand(hq, ql, 1)], dim=-1)
        p = torch.softmax(att, dim=-1)[..., : sl[s]]
        out[q0:q1] = (torch.einsum("hqk,khd->qhd", p, vv).reshape(ql, hq * dv) * out_scale).to(q.dtype)
    return out


def causal_conv_silu(xz: torch.Tensor, channels: int, w: torch.Tensor, b: torch.Tensor,
                     conv_state: Optional[torch.Tensor], rec_slots: Optional[torch.Tensor], seq_lens: torch.Tensor,
                     query_start_loc: torch.Tensor, act: str = "silu", in_bias: Optional[torch.Tensor] = None,
                     out_dtype=None) -> torch.Tensor:
    """Depthwise causal convolution + SiLU over the first `channels` columns of xz [T, >= channels], per sequence.
    w [channels, taps] (last tap = current token), b [channels]. conv_state [slots, taps - 1, channels] holds the
    last taps - 1 inputs of every sequence; a sequence whose chunk starts at position 0 starts from zeros.
    `act`: "silu" | "none". `in_bias` [channels] fp32 is added to every input that exists (the zeros before the
    start of a sequence stay zeros); the carried state holds the inputs without it. `out_dtype`: the result's type
    (default: that of xz)."""
    taps = w.shape[1]
    odt = out_dtype or xz.dtype
    out = torch.empty(xz.shape[0], channels, dtype=odt, device=xz.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        n = q1 - q0
        if n <= 0:
            continue
        x = xz[q0:q1, :channels].float()
        hist = torch.zeros(taps - 1, channels, dtype=torch.float32, device=xz.device)
        have = min(sl[s] - n, taps - 1)              # carried inputs that exist (the rest precede position 0)
        if conv_state is not None and sl[s] - n > 0:
            hist = conv_state[int(rec_slots[s])][: taps - 1].float()
        xp = torch.cat([hist, x], 0)
        xin = xp + in_bias.float() if in_bias is not None else xp.clone()
        xin[: taps - 1 - max(have, 0)] = 0.0         # nothing precedes position 0, whatever the slot held
        acc = b.float().expand(n, channels).clone()
        for j in range(taps):
            acc = acc + xin[j:j + n] * w[:, j].float()
        out[q0:q1] = (F.silu(acc) if act == "silu" else acc).to(odt)
        if conv_state is not None and taps > 1:
            conv_state[int(rec_slots[s])] = xp[n:].to(conv_state.dtype)
    return out


def selective_scan(xc: torch.Tensor, dt_raw: torch.Tensor, proj: torch.Tensor, xz: torch.Tensor, a: torch.Tensor,
                   d_skip: torch.Tensor, dt_bias: torch.Tensor, ssm_state: Optional[torch.Tensor],
                   rec_slots: Optional[torch.Tensor], seq_lens: torch.Tensor, query_start_loc: torch.Tensor,
                   channels: int, nstate: int, dt_rank: int) -> torch.Tensor:
    """Selective state-space recurrence, fp32, token by token:
        dt = softplus(dt_raw + dt_bias);  S <- exp(dt * A) * S + dt * x * B;  y = S . C + D * x;  out = y * silu(z)
    xc [T, C] conv output, dt_raw [T, C], proj [T, R + 2N] = [.. | B | C], xz [T, 2C] = [.. | z], a [C, N] (negative),
    ssm_state [slots, N, C] fp32 carried between chunks (zeros for a chunk that starts at position 0)."""
    out = torch.empty(xc.shape[0], channels, dtype=xc.dtype, device=xc.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    af = a.float()
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        n = q1 - q0
        if n <= 0:
            continue
        st = torch.zeros(channels, nstate, dtype=torch.float32, device=xc.device)
        if ssm_state is not None and sl[s] - n > 0:
            st = ssm_state[int(rec_slots[s])].t().clone()
        dt = F.softplus(dt_raw[q0:q1].float() + dt_bias.float())
        x = xc[q0:q1].float()
        bm = proj[q0:q1, dt_rank:dt_rank + nstate].float()
        cm = proj[q0:q1, dt_rank + nstate:dt_rank + 2 * nstate].float()
        z = xz[q0:q1, channels:2 * channels].float()
        ys = torch.empty(n, channels, dtype=torch.float32, device=xc.device)
        for i in range(n):
            st = torch.exp(dt[i].unsqueeze(1) * af) * st + (dt[i] * x[i]).unsqueeze(1) * bm[i].unsqueeze(0)
            ys[i] = st @ cm[i] + d_skip.float() * x[i]
        out[q0:q1] = (ys * F.silu(z)).to(xc.dtype)
        if ssm_state is not None:
            ssm_state[int(rec_slots[s])] = st.t()
    return out


def relu2(x: torch.Tensor) -> torch.Tensor:
    r = torch.relu(x.float())
    return (r * r).to(x.dtype)


# ----------------------------------------------------------------------------------------------
# norm-after-sum blocks, rotary q/k norm + cache write, matrix-state linear recurrences (delta rule, constant
# decay), group norm with a gate, top-k router, plain experts, logit cap (PyTorch forms of csrc/seq/state_ops.cu)
# ----------------------------------------------------------------------------------------------
def postnorm(x: torch.Tensor, y: torch.Tensor, alpha: float, w: torch.Tensor, eps: float, out_dtype):
    """In place on the fp32 stream: x <- rms(alpha * x + y) * w. Returns x in `out_dtype` (x itself for fp32)."""
    v = alpha * x + y.float()
    x.copy_(v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps) * w.float())
    return x if out_dtype == torch.float32 else x.to(out_dtype)


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, rot_dims: int, base: float,
                      freqs: Optional[torch.Tensor] = None, mag: float = 1.0) -> torch.Tensor:
    """x [T, heads, D] fp32: entries i and i + rot_dims / 2 (i < rot_dims / 2) turn by positions * base^(-2i/rot_dims);
    entries from rot_dims on pass through. Angles are formed in fp64. `freqs` [rot_dims / 2] fp64 replaces the
    powers of the base (scaled frequencies); cos and sin are multiplied by `mag`."""
    if rot_dims <= 0:
        return x
    half = rot_dims // 2
    if freqs is not None:
        freq = freqs.to(torch.float64)
    else:
        freq = torch.exp2(-(2.0 * torch.arange(half, dtype=torch.float64, device=x.device) / rot_dims) *
                          math.log2(base))
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mag).float()[:, None, :], (torch.sin(ang) * mag).float()[:, None, :]
    a, b = x[..., :half], x[..., half:rot_dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., rot_dims:]], -1)


def qk_norm_rope_kv_write(qkv: torch.Tensor, num_heads: int, num_kv_heads: int, dim: int, v_dim: int, q_norm_w,
                          k_norm_w, eps: float, positions: torch.Tensor, rot_dims: int, rot_base: float,
                          k_cache: torch.Tensor, v_cache: torch.Tensor, slots: torch.Tensor,
                          freqs: Optional[torch.Tensor] = None, mag: float = 1.0) -> torch.Tensor:
    """qkv [T, >= H*D + G*D + G*Dv] = [queries | keys | values]. Per-head RMS norm of q and k (weights optional),
    then the rotate-half rotation of both; rotated keys go to the K cache, values as projected to the V cache.
    Returns the queries [T, H * D]. With num_kv_heads == 0 the row holds queries only (a layer that reads another
    layer's keys and values) and no cache is touched. `freqs`, `mag`: see `rotate_half_pairs`."""
    t = qkv.shape[0]
    hd, gd = num_heads * dim, num_kv_heads * dim
    q = qkv[:, :hd].reshape(t, num_heads, dim).float()
    if num_kv_heads == 0:
        if q_norm_w is not None:
            q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w.float()
        return rotate_half_pairs(q, positions, rot_dims, rot_base, freqs, mag).to(qkv.dtype).reshape(t, hd)
    k = qkv[:, hd:hd + gd].reshape(t, num_kv_heads, dim).float()
    v = qkv[:, hd + gd:hd + gd + num_kv_heads * v_dim].reshape(t, num_kv_heads, v_dim)
    if q_norm_w is not None:
        q = q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps) * q_norm_w.float()
    if k_norm_w is not None:
        k = k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps) * k_norm_w.float()
    q = rotate_half_pairs(q, positions, rot_dims, rot_base, freqs, mag)
    k = rotate_half_pairs(k, positions, rot_dims, rot_base, freqs, mag)
    _cache_rows_write(k_cache, slots, k.to(qkv.dtype))
    _cache_rows_write(v_cache, slots, v)
    return q.to(qkv.dtype).reshape(t, hd)


def linear_state_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: Optional[torch.Tensor],
                      a: Optional[torch.Tensor], neg_a: Optional[torch.Tensor], dt_bias: Optional[torch.Tensor],
                      decay: Optional[torch.Tensor], state: Optional[torch.Tensor], rec_slots, seq_lens, query_start_loc,
                      heads: int, qk_heads: int, dim: int, v_dim: int, silu_in: bool, unit_qk: bool, q_scale: float,
                      delta: bool, zk: Optional[torch.Tensor] = None, zk_bias: Optional[torch.Tensor] = None,
                      inv_tau: float = 1.0) -> torch.Tensor:
    """Matrix-state recurrence per head, fp32, token by token, S [dim, v_dim]:
        g = exp(neg_a[h] * softplus(a + dt_bias[h]))   (or the constant decay[h]; or, with `zk` [T, heads * dim]
            and `zk_bias` [heads * dim], one decay per key channel, g[d] = sigmoid(zk + zk_bias)^inv_tau, acting
            on row d of S)
        S <- g S;   u = beta * (v - S^T k) with `delta`, else u = v;   S <- S + k u^T;   o = S^T q
    q, k [T, qk_heads * dim] (head h reads group h // (heads / qk_heads)), v [T, heads * v_dim], beta / a [T, heads].
    `silu_in`: q, k, v pass SiLU first; `unit_qk`: q and k are scaled to unit length (1e-6 inside the root);
    q is multiplied by q_scale. state [slots, heads, dim, v_dim] fp32 carries S between chunks (zeros for a chunk
    that starts at position 0). Returns o [T, heads * v_dim] fp32."""
    t = q.shape[0]
    out = torch.zeros(t, heads * v_dim, dtype=torch.float32, device=q.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    rep = heads // qk_heads
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        n = q1 - q0
        if n <= 0:
            continue
        qq = q[q0:q1].float().reshape(n, qk_heads, dim)
        kk = k[q0:q1].float().reshape(n, qk_heads, dim)
        vv = v[q0:q1].float().reshape(n, heads, v_dim)
        if silu_in:
            qq, kk, vv = F.silu(qq), F.silu(kk), F.silu(vv)
        if unit_qk:
            qq = qq / torch.sqrt((qq * qq).sum(-1, keepdim=True) + 1e-6)
            kk = kk / torch.sqrt((kk * kk).sum(-1, keepdim=True) + 1e-6)
        qq = (qq * q_scale).repeat_interleave(rep, 1)
        kk = kk.repeat_interleave(rep, 1)
        if zk is not None:
            zz = zk[q0:q1].float() + (zk_bias.float() if zk_bias is not None else 0.0)
            g = torch.exp(F.logsigmoid(zz) * inv_tau).reshape(n, heads, dim, 1)
        elif decay is not None:
            g = decay.float().view(1, heads).expand(n, heads)
        else:
            g = torch.exp(neg_a.float() * F.softplus(a[q0:q1].float() + dt_bias.float()))
        b = torch.sigmoid(beta[q0:q1].float()) if delta else None
        st = torch.zeros(heads, dim, v_dim, dtype=torch.float32, device=q.device)
        if state is not None and sl[s] - n > 0:
            st = state[int(rec_slots[s])].clone()
        o = torch.empty(n, heads, v_dim, dtype=torch.float32, device=q.device)
        for i in range(n):
            st = st * (g[i] if zk is not None else g[i].view(heads, 1, 1))
            u = vv[i]
            if delta:
                u = b[i].view(heads, 1) * (u - torch.einsum("hdv,hd->hv", st, kk[i]))
            st = st + kk[i].unsqueeze(-1) * u.unsqueeze(1)
            o[i] = torch.einsum("hdv,hd->hv", st, qq[i])
        out[q0:q1] = o.reshape(n, heads * v_dim)
        if state is not None:
            state[int(rec_slots[s])] = st
    return out


def gated_group_norm(o: torch.Tensor, gate: torch.Tensor, w: torch.Tensor, group: int, eps: float, act: str,
                     out_scale: float = 1.0, out: Optional[torch.Tensor] = None, out_dtype=None) -> torch.Tensor:
    """o [T, n] fp32 is RMS-normed over consecutive groups of `group` columns, multiplied by w (w[i % len(w)]) and
    by act(gate) (act: "silu" | "sigmoid"), times out_scale."""
    t, n = o.shape
    x = o.float().reshape(t, n // group, group)
    x = (x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)).reshape(t, n)
    x = x * w.float().repeat(n // w.shape[0])
    gf = gate.float()
    x = x * (F.silu(gf) if act == "silu" else torch.sigmoid(gf)) * out_scale
    dt = out.dtype if out is not None else (out_dtype or gate.dtype)
    if out is None:
        return x.to(dt)
    out.copy_(x.to(dt))
    return out


def silu_mul(gu: torch.Tensor) -> torch.Tensor:
    """gu [T, 2F] = [gate | up] -> silu(gate) * up."""
    f = gu.shape[1] // 2
    return (F.silu(gu[:, :f].float()) * gu[:, f:].float()).to(gu.dtype)


def router_topk(h: torch.Tensor, w: torch.Tensor, top_k: int):
    """fp32 router logits h . w^T; the top_k largest per token, weights = softmax over the chosen logits only.
    -> (weights fp32 [T, k], ids int32 [T, k])"""
    z = h.float() @ w.float().t()
    val, ids = torch.topk(z, top_k, dim=-1)
    return torch.softmax(val, -1), ids.to(torch.int32)


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return (cap * torch.tanh(z.float() / cap)).to(z.dtype)


# ----------------------------------------------------------------------------------------------
# branch-norm blocks with layer scale, key-channel-decay linear attention, latent attention with pair-wise (YaRN)
# rotary, the real-gated linear recurrent unit, grouped routing with identity experts, clamped gated experts
# (PyTorch forms of csrc/seq/latent_ops.cu)
# ----------------------------------------------------------------------------------------------
def block_linear(x: torch.Tensor, w: torch.Tensor, out_dtype=None) -> torch.Tensor:
    """Block-diagonal linear map: x [T, B * K] is cut into B parts, part b times w[b] [N, K] ([out, in]);
    -> [T, B * N] in `out_dtype` (default: that of x), fp32 accumulation."""
    t = x.shape[0]
    nb, n, k = w.shape
    y = torch.einsum("tbk,bnk->tbn", x.float().reshape(t, nb, k), w.float()).reshape(t, nb * n)
    return y.to(out_dtype or x.dtype)


def rglru_scan(u: torch.Tensor, gates: torch.Tensor, gate_bias: torch.Tensor, c_decay: torch.Tensor,
               y_pre: torch.Tensor, y_bias: torch.Tensor, state: Optional[torch.Tensor], rec_slots, seq_lens,
               query_start_loc, block: int, out_dtype) -> torch.Tensor:
    """Real-gated linear recurrent unit, one fp32 state per channel, token by token:
        r = sigmoid(gate_r + bias_r);  i = sigmoid(gate_i + bias_i)
        a = exp(c_decay * r);  S <- a S + sqrt(1 - a^2) * i * u;  out = S * gelu_tanh(y_pre + y_bias)
    u [T, C]; gates [T, 2C] (any float type) and gate_bias [2C] are laid out per block of `block` channels as
    [r of the block | i of the block] (the result of one block-diagonal product with stacked weights);
    c_decay [C] fp32 (negative), y_pre [T, C] (any row stride). state
    [slots, 1, C] fp32 carries S between chunks (zeros for a chunk that starts at position 0, also for its first
    token)."""
    t, c = u.shape
    out = torch.empty(t, c, dtype=out_dtype, device=u.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    gz = (gates.float() + gate_bias.float()).reshape(t, c // block, 2, block)
    r = torch.sigmoid(gz[:, :, 0]).reshape(t, c)
    ig = torch.sigmoid(gz[:, :, 1]).reshape(t, c)
    log_a = c_decay.float() * r
    a = torch.exp(log_a)
    b = torch.sqrt(-torch.expm1(2.0 * log_a)) * ig * u.float()
    z = y_pre[:, :c].float() + y_bias.float()
    y = 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z * z * z)))
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        n = q1 - q0
        if n <= 0:
            continue
        st = torch.zeros(c, dtype=torch.float32, device=u.device)
        if state is not None and sl[s] - n > 0:
            st = state[int(rec_slots[s])].reshape(-1)[:c].clone()
        for i in range(q0, q1):
            st = a[i] * st + b[i]
            out[i] = (st * y[i]).to(out_dtype)
        if state is not None:
            state[int(rec_slots[s])].reshape(-1)[:c] = st
    return out


def pair_rotary_frequencies(dims: int, base: float, scaling: Optional[dict] = None, dtype=torch.float32):
    """-> (frequency per pair [dims / 2] in `dtype`, factor on cos and sin). Pair i turns by position * base^(-2i/dims);
    with YaRN `scaling` {factor, original, fast, slow}: where(t) = dims ln(original / (2 pi t)) / (2 ln base),
    lo = max(floor(where(fast)), 0), hi = min(ceil(where(slow)), dims - 1), ramp_i = clamp((i - lo) / max(hi - lo,
    0.001), 0, 1), frequency f_i / factor * ramp_i + f_i (1 - ramp_i), magnitude 0.1 ln(factor) + 1."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.exp(-(2.0 * i / dims) * math.log(base))
    mag = 1.0
    if scaling:
        factor, orig = float(scaling["factor"]), float(scaling["original"])

        def where(turns):
            return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

        lo = max(math.floor(where(float(scaling["fast"]))), 0)
        hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        f = f / factor * ramp + f * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    return f.to(dtype), float(mag)


def rotate_adjacent_pairs(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, mag: float) -> torch.Tensor:
    """x [T, ..., D] fp32: entries 2i and 2i + 1 (i < len(freqs)) turn by the fp32 angle positions * freqs[i], cos
    and sin times `mag`; later entries pass through."""
    n = freqs.shape[0]
    if n == 0:
        return x
    ang = positions.to(torch.float32)[:, None] * freqs.to(torch.float32)[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [n]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    a, b = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
    out = x.clone()
    out[..., 0:2 * n:2] = a * c - b * s
    out[..., 1:2 * n:2] = b * c + a * s
    return out


def rms_rows(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm of every row of x [T, n] (any row stride) times w [n]; fp32 arithmetic, result in x's dtype."""
    xf = x.float()
    return (xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()).to(x.dtype)


def linear_batched(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out[:, b, :] = a[:, b, :] @ w[b].T for every b: a [T, B, K] and out [T, B, N] may be strided views."""
    out.copy_(torch.einsum("tbk,bnk->tbn", a.float(), w.float()).to(out.dtype))
    return out


def latent_norm_rope_write(q: torch.Tensor, dkv: torch.Tensor, rank: int, rot: int, norm_w: torch.Tensor, eps: float,
                           positions: torch.Tensor, freqs: torch.Tensor, mag: float, q_full: torch.Tensor,
                           cache: Optional[torch.Tensor], slots: Optional[torch.Tensor]):
    """Latent attention, between the projections and the attention: q [T, H, dim + rot] (view) — its last `rot`
    entries per head are rotated into q_full[:, :, rank:] (q_full [T, H, rank + rot]; the first `rank` columns are
    the caller's: the absorbed queries). dkv [T, rank + rot]: the first `rank` columns are RMS-normed with norm_w
    (the latent), the last `rot` rotated (the key part all heads share); the row [latent | rotated key] goes to
    the paged latent cache [pages, 1, (rank + rot) / slab, page, slab] at `slots`. Norm, angles and rotation in
    fp32."""
    t, h = q.shape[0], q.shape[1]
    dim = q.shape[2] - rot
    q_full[:, :, rank:] = rotate_adjacent_pairs(q[:, :, dim:].float(), positions, freqs, mag).to(q_full.dtype)
    c = dkv[:, :rank].float()
    c = c * torch.rsqrt((c * c).mean(-1, keepdim=True) + eps) * norm_w.float()
    kr = rotate_adjacent_pairs(dkv[:, rank:rank + rot].float(), positions, freqs, mag)
    if cache is not None:
        _cache_rows_write(cache, slots, torch.cat([c, kr], -1).to(cache.dtype).reshape(t, 1, rank + rot))


def latent_attention(q_full: torch.Tensor, cache: torch.Tensor, block_table: torch.Tensor, seq_lens: torch.Tensor,
                     query_start_loc: torch.Tensor, scale: float, rank: int) -> torch.Tensor:
    """Causal multi-query attention over the paged latent cache: every head's query q_full [T, H, rank + rot]
    meets the one shared key row [latent | rotated key]; the values are the row's first `rank` columns.
    -> out [T, H, rank] in q_full's dtype. Scores and softmax in fp32."""
    t, h, d = q_full.shape
    out = torch.zeros(t, h, rank, dtype=q_full.dtype, device=q_full.device)
    qsl, sl = query_start_loc.tolist(), seq_lens.tolist()
    for s in range(len(sl)):
        q0, q1 = qsl[s], qsl[s + 1]
        ql = q1 - q0
        if ql <= 0:
            continue
        lat = gather_kv(cache, block_table[s], sl[s])[:, 0].float()            # [L, rank + rot]
        att = torch.einsum("qhd,kd->hqk", q_full[q0:q1].float(), lat) * scale
        qi = torch.arange(ql, device=q_full.device).view(ql, 1) + (sl[s] - ql)
        kj = torch.arange(sl[s], device=q_full.device).view(1, sl[s])
        att = att.masked_fill((kj > qi).unsqueeze(0), float("-inf"))
        out[q0:q1] = torch.einsum("hqk,kd->qhd", torch.softmax(att, -1), lat[:, :rank]).to(q_full.dtype)
    return out


def grouped_router(h: torch.Tensor, w: torch.Tensor, correction: Optional[torch.Tensor], top_k: int, n_groups: int,
                   keep_groups: int, scale: float, score: str = "softmax", group_top: int = 1,
                   renorm: bool = True):
    """fp32 router: scores = softmax(h . w^T) over all outputs (`score` "sigmoid": the logistic function of every
    logit by itself); choice = scores + correction; outputs form `n_groups` equal groups of neighbours, a group's
    score is the sum of its `group_top` largest choice scores (1: its largest) and only the best `keep_groups`
    groups stay eligible (the others count as -inf); the top_k largest eligible choice scores are chosen (ties: the
    lower index); weights = chosen scores / (their sum + 1e-20) * scale, or with `renorm` False the chosen scores
    themselves * scale.
    -> (weights fp32 [T, k], ids int32 [T, k])"""
    z = h.float() @ w.float().t()
    sc = torch.sigmoid(z) if score == "sigmoid" else torch.softmax(z, -1)
    choice = sc + correction.float() if correction is not None else sc
    t, n = sc.shape
    if n_groups > 1:
        per = n // n_groups
        best = torch.topk(choice.reshape(t, n_groups, per), min(group_top, per), dim=-1).values.sum(-1)
        kept = torch.topk(best, keep_groups, dim=-1).indices
        ok = torch.zeros(t, n_groups, dtype=torch.bool, device=h.device).scatter_(1, kept, True)
        choice = choice.masked_fill(~ok.repeat_interleave(per, 1), float("-inf"))
    ids = torch.topk(choice, top_k, dim=-1).indices
    sel = sc.gather(1, ids)
    if not renorm:
        return sel * scale, ids.to(torch.int32)
    return sel / (sel.sum(-1, keepdim=True) + 1e-20) * scale, ids.to(torch.int32)


def glu_clamp(gu: torch.Tensor, limit: float, alpha: float = 1.702) -> torch.Tensor:
    """gu [T, 2F] = [gate | up] -> g sigmoid(alpha g) (u + 1) with g = min(gate, limit), u = clamp(up, +-limit)."""
    f = gu.shape[1] // 2
    g = gu[:, :f].float().clamp(max=limit)
    u = gu[:, f:].float().clamp(-limit, limit)
    return (g * torch.sigmoid(alpha * g) * (u + 1.0)).to(gu.dtype)


def linear_glu_clamp(x: torch.Tensor, w_interleaved: torch.Tensor, limit: float, alpha: float = 1.702,
                     block: int = 128) -> torch.Tensor:
    """`glu_clamp` of x @ w^T for a weight whose gate / up rows are interleaved per `block`."""
    y = F.linear(x, w_interleaved)
    t, two_i = y.shape
    y = y.reshape(t, two_i // (2 * block), 2, block)
    gu = torch.cat([y[:, :, 0].reshape(t, -1), y[:, :, 1].reshape(t, -1)], 1)
    return glu_clamp(gu, limit, alpha)


def routed_glu_experts(h: torch.Tensor, w13: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor, ids: torch.Tensor,
                       limit: float, alpha: float = 1.702) -> torch.Tensor:
    """sum_k weights[t, k] * expert_{ids[t, k]}(h[t]) with clamped gated experts (`glu_clamp` between the two
    products); an id >= the number of experts names an identity expert, whose result is h[t] itself.
    w13 [E, 2F, W] = [gate rows ; up rows], w2 [E, W, F]."""
    e_real = w13.shape[0]
    out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
    for kk in range(ids.shape[1]):
        for e in ids[:, kk].unique().tolist():
            rows = (ids[:, kk] == e).nonzero().flatten()
            x = h[rows]
            if e >= e_real:
                y = x.float()
            else:
                a = glu_clamp(linear(x, w13[e]), limit, alpha)
                y = linear(a, w2[e]).float()
            out[rows] += weights[rows, kk].float().unsqueeze(1) * y
    return out.to(h.dtype)


# ----------------------------------------------------------------------------------------------
# hashed pair embedding with a carried previous token, ungated squared-ReLU experts
# (PyTorch forms of the kernels in csrc/seq/pair_ops.cu)
# ----------------------------------------------------------------------------------------------
def embedding_pair_hash(ids: torch.Tensor, table: torch.Tensor, pair_table: torch.Tensor, mul_prev: int, mul_cur: int,
                        buckets: int, positions: torch.Tensor, prev_state: Optional[torch.Tensor], rec_slots,
                        query_start_loc: torch.Tensor) -> torch.Tensor:
    """fp32 residual stream from token ids: table[id] + pair_table[(prev * mul_prev + id * mul_cur) mod buckets],
    where prev is the token before in the same sequence; a token at position 0 takes row `buckets` (the last row).
    The token before the first row of a portion that starts later comes from prev_state [slots] int32 at the
    sequence's state slot, and the portion's last token is left there for the next step."""
    x = table[ids.long()].float()
    qsl = query_start_loc.tolist()
    idl, pos = ids.tolist(), positions.tolist()
    rows = []
    for s in range(len(qsl) - 1):
        q0, q1 = qsl[s], qsl[s + 1]
        for r in range(q0, q1):
            if pos[r] == 0:
                rows.append(buckets)
                continue
            if r > q0:
                prev = idl[r - 1]
            else:
                prev = int(prev_state[int(rec_slots[s])]) if prev_state is not None else 0
            rows.append((prev * mul_prev + idl[r] * mul_cur) % buckets)
        if prev_state is not None and q1 > q0:
            prev_state[int(rec_slots[s])] = idl[q1 - 1]
    return x + pair_table[torch.tensor(rows, dtype=torch.long, device=ids.device)].float()


def routed_relu2_experts(h: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, weights: torch.Tensor,
                         ids: torch.Tensor) -> torch.Tensor:
    """sum_k weights[t, k] * down_e(relu(up_e h[t])^2) with e = ids[t, k]; w1 [E, F, W] (up), w2 [E, W, F] (down);
    the activation is rounded to h's dtype between the two products."""
    out = torch.zeros(h.shape, dtype=torch.float32, device=h.device)
    for kk in range(ids.shape[1]):
        for e in ids[:, kk].unique().tolist():
            rows = (ids[:, kk] == e).nonzero().flatten()
            a = relu2(linear(h[rows], w1[e]))
            out[rows] += weights[rows, kk].float().unsqueeze(1) * linear(a, w2[e]).float()
    return out.to(h.dtype)
