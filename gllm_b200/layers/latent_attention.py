"""Latent attention for the layer-list decoder: queries, keys and values pass low-rank latents, and only the
key / value latent and one rotated key part shared by all heads are cached.

    c_q = rms(W_dq h) * n_q;  q = W_uq c_q                    per head [dim unrotated | rot_dim rotated]
    [c' | k_r] = W_dkv h;  c = rms(c') * n_kv                 c: kv_rank, k_r: rot_dim (not normed)
    k_h = W_uk[h] c,  v_h = W_uv[h] c;   score = (q_h . k_h + rot(q_r) . rot(k_r)) * scale;   causal softmax

The cache row of a token is [c | rot(k_r)] (one "head" of width kv_rank + rot_dim in the paged layout). The
attention runs in the absorbed form: q_h . (W_uk[h] c) = (W_uk[h]^T q_h) . c, so every head's query becomes a
kv_rank + rot_dim vector that meets the cached row directly (multi-query attention whose values are the row's
first kv_rank columns), and W_uv[h] is applied to the attention result. Both per-head products are one batched
GEMM each. With kv_rank 512 and rot_dim 64 in bf16 the attention is the tensor-core latent kernel shared with
DeepSeek MLA (csrc/attn/mla_attention.cu); other sizes and fp32 run the plain latent kernel.

Rotation: adjacent pairs (2i, 2i + 1) of the rotated part, fp32 angles position * f_i with optional YaRN-scaled
frequencies and magnitude (`ops.ref.pair_rotary_frequencies`); the softmax scale is the caller's and is not
touched by the scaling.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from gllm_b200.layers import functional as Fn
from gllm_b200.ops import ref


class LatentAttention(nn.Module):
    uses_pages, uses_state = True, False
    needs_tok_seq = True

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, v_dim: int, q_rank: int, kv_rank: int,
                 scale: float, rot_base: float, rot_scaling: Optional[dict], eps: float, dtype, device):
        super().__init__()
        assert rot_dim % 2 == 0, rot_dim
        self.hidden, self.heads, self.dim, self.rot_dim, self.v_dim = hidden, heads, dim, rot_dim, v_dim
        self.q_rank, self.kv_rank, self.scale, self.eps = q_rank, kv_rank, float(scale), eps

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        self.n_in = q_rank + kv_rank + rot_dim
        self.in_w = par((self.n_in + 7) // 8 * 8, hidden)             # [W_dq ; W_dkv], pad rows stay zero
        self.q_norm_w = par(q_rank)
        self.kv_norm_w = par(kv_rank)
        self.uq_w = par(heads * (dim + rot_dim), q_rank)
        self.uk_t = par(heads, kv_rank, dim)                          # [h] = W_uk[h]^T: the batched GEMM's [N, K]
        self.uv = par(heads, v_dim, kv_rank)                          # [h] = W_uv[h]
        self.o_w = par(hidden, heads * v_dim)
        f, mag = ref.pair_rotary_frequencies(rot_dim, rot_base, rot_scaling)
        self.register_buffer("freqs", f.to(device), persistent=False)
        self.mag = mag

    def cache_entry(self):
        return {"kind": "latent", "dim": self.kv_rank + self.rot_dim}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        t, nh, qr, r, rot = h.shape[0], self.heads, self.q_rank, self.kv_rank, self.rot_dim
        proj = Fn.linear_any(h, self.in_w)
        cq = Fn.rms_rows(proj[:, :qr], self.q_norm_w, self.eps)
        q = Fn.linear_any(cq, self.uq_w).view(t, nh, self.dim + rot)
        if cache is None:          # memory probe without a cache
            return Fn.linear_any(h.new_zeros(t, nh * self.v_dim), self.o_w)
        lat = cache.k_cache[run_id]
        q_full = torch.empty(t, nh, r + rot, dtype=h.dtype, device=h.device)
        Fn.linear_batched(q[:, :, :self.dim], self.uk_t, q_full[:, :, :r])
        Fn.latent_norm_rope_write(q, proj[:, qr:qr + r + rot], r, rot, self.kv_norm_w, self.eps, inp.positions,
                                  self.freqs, self.mag, q_full, lat, inp.slot_mapping)
        o_lat = Fn.latent_attention(q_full, lat, inp, self.scale, r)
        o = torch.empty(t, nh, self.v_dim, dtype=h.dtype, device=h.device)
        Fn.linear_batched(o_lat, self.uv, o)
        return Fn.linear_any(o.view(t, nh * self.v_dim), self.o_w)

    def load(self, reader, pre: str, put):
        w = torch.cat([reader.get(pre + "dq"), reader.get(pre + "dkv")], 0)
        self.in_w.data[: w.shape[0]].copy_(w)
        put(self.q_norm_w, reader.get(pre + "dq.norm"))
        put(self.kv_norm_w, reader.get(pre + "dkv.norm"))
        put(self.uq_w, reader.get(pre + "uq"))
        put(self.uk_t, reader.get(pre + "uk").reshape(self.heads, self.dim, self.kv_rank).transpose(1, 2))
        put(self.uv, reader.get(pre + "uv").reshape(self.heads, self.v_dim, self.kv_rank))
        put(self.o_w, reader.get(pre + "o"))
