"""Sliding-window grouped-query attention over the paged cache with an optional softmax sink.

Mechanism (parameters, so other designs can use it):
  * per-head RMS norm of queries and keys with one weight vector shared by all heads (`qk_norm`);
  * no positional rotation — scores depend on content only;
  * `window`: position i attends to j with 0 <= i - j < window (None = the whole past);
  * `use_sink`: one learned logit per query head joins the softmax denominator and carries no value;
  * `values="key"`: there is no value projection, the values are the keys as projected (before their norm). The
    K cache holds the normed keys and the V cache the raw keys, so the attention kernel itself is an ordinary
    paged K/V attention.
"""
from __future__ import annotations

from typing import Optional

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


class SinkWindowAttention(nn.Module):
    uses_pages = True
    state_shapes = None

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, scale: float, window: Optional[int],
                 eps: float, dtype, device, use_sink: bool = True, qk_norm: bool = True, values: str = "key"):
        super().__init__()
        assert values == "key", "only key-valued attention is implemented"
        assert heads % kv_heads == 0, (heads, kv_heads)
        self.hidden, self.heads, self.kv_heads, self.dim = hidden, heads, kv_heads, dim
        self.scale, self.window, self.eps = float(scale), window, eps

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        self.qk_w = par((heads + kv_heads) * dim, hidden)        # [q rows ; k rows]
        self.q_norm_w = par(dim) if qk_norm else None
        self.k_norm_w = par(dim) if qk_norm else None
        self.sink = par(heads, dt=torch.float32) if use_sink else None
        self.o_w = par(hidden, heads * dim)

    def cache_entry(self):
        return {"kind": "kv", "heads": self.kv_heads, "dim": self.dim}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        qk = Fn.linear_any(h, self.qk_w)
        hd = self.heads * self.dim
        if cache is None:      # memory probe without a cache
            return Fn.linear_any(qk[:, :hd].contiguous(), self.o_w)
        kc, vc = cache.k_cache[run_id], cache.v_cache[run_id]
        q = Fn.qk_norm_kv_write(qk, self.heads, self.kv_heads, self.dim, self.q_norm_w, self.k_norm_w, self.eps,
                                kc, vc, inp.slot_mapping)
        a = Fn.window_attention(q, kc, vc, inp, self.scale, self.heads, self.dim, self.window, self.sink)
        return Fn.linear_any(a, self.o_w)


class RotaryChunkCore(nn.Module):
    """Grouped-query softmax attention over the paged cache with
      * per-head RMS norm of q and k (weights shared by the heads), applied before the rotation (`qk_norm`);
      * rotary positions on the first `rot_dims` entries of each head, entry i paired with i + rot_dims / 2; with
        `rot_scaling` {factor, original, fast, slow} the pair frequencies are the YaRN blend of
        `ops.ref.pair_rotary_frequencies` and cos / sin carry its magnitude;
      * a mask made of the causal rule and, optionally, a sliding `window` and / or a `chunk`: position i sees j only
        if floor(i / chunk) == floor(j / chunk), chunks counted from the start of the sequence;
      * `softcap` > 0: every scaled score s becomes softcap * tanh(s / softcap);
      * `unit_sink`: the softmax denominator has one more term exp(0) = 1 that carries no value;
      * values of their own width `v_dim`;
      * `bias`: the q / k / v projections have biases (the mixer adds them in the joint projection);
      * `kv_from` (a layer index): the core has no key / value projections and no cache of its own; it reads the
        pages that layer wrote (rotated keys, values) with its own queries and mask.
    A core in the sense of layers/parallel_mixer.py: it reads [q | k | v] rows of a joint projection."""
    uses_pages, uses_state = True, False

    def __init__(self, heads: int, kv_heads: int, dim: int, v_dim: int, scale: float, rot_dims: int, rot_base: float,
                 chunk: Optional[int], window: Optional[int], eps: float, dtype, device, qk_norm: bool = True,
                 rot_scaling: Optional[dict] = None, softcap: float = 0.0, unit_sink: bool = False,
                 bias: bool = False, kv_from: Optional[int] = None):
        super().__init__()
        assert heads % kv_heads == 0, (heads, kv_heads)
        assert rot_dims % 2 == 0 and rot_dims <= dim, (rot_dims, dim)
        self.heads, self.kv_heads, self.dim, self.v_dim = heads, kv_heads, dim, v_dim
        self.scale, self.rot_dims, self.rot_base, self.chunk, self.window, self.eps = \
            float(scale), int(rot_dims), float(rot_base), chunk, window, eps
        self.softcap, self.has_bias, self.kv_from = float(softcap or 0.0), bool(bias), kv_from
        if kv_from is None:
            self.in_names = ("q", "k", "v")
            self.in_rows = (heads * dim, kv_heads * dim, kv_heads * v_dim)
        else:
            self.in_names = ("q",)
            self.in_rows = (heads * dim,)
        self.n_in, self.n_out = sum(self.in_rows), heads * v_dim
        self.q_norm_w = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False) if qk_norm \
            else None
        self.k_norm_w = nn.Parameter(torch.zeros(dim, dtype=dtype, device=device), requires_grad=False) if qk_norm \
            else None
        self.mag = 1.0
        if rot_scaling and rot_dims > 0:
            from gllm_b200.ops import ref
            f, self.mag = ref.pair_rotary_frequencies(rot_dims, rot_base, rot_scaling, dtype=torch.float64)
            self.register_buffer("freqs", f.to(device), persistent=False)
        else:
            self.freqs = None
        if unit_sink:
            self.register_buffer("sink", torch.zeros(heads, dtype=torch.float32, device=device), persistent=False)
        else:
            self.sink = None

    def cache_entry(self):
        if self.kv_from is not None:
            return {"kind": "shared", "layer": int(self.kv_from)}
        return {"kind": "kv", "heads": self.kv_heads, "dim": self.dim, "vdim": self.v_dim}

    def core(self, inp, proj, cache, run_id, out, out_scale=1.0):
        if cache is None:      # memory probe without a cache
            out.zero_()
            return out
        kc, vc = cache.k_cache[run_id], cache.v_cache[run_id]
        own = self.kv_from is None
        q = Fn.qk_norm_rope_kv_write(proj, self.heads, self.kv_heads if own else 0, self.dim, self.v_dim,
                                     self.q_norm_w, self.k_norm_w, self.eps, inp.positions, self.rot_dims,
                                     self.rot_base, kc, vc, inp.slot_mapping, self.freqs, self.mag)
        return Fn.masked_attention(q, kc, vc, inp, self.scale, self.heads, self.dim, self.v_dim, self.window,
                                   self.chunk, self.sink, out_scale, out, self.softcap)

    def load_extra(self, reader, pre, put):
        if self.q_norm_w is not None:
            put(self.q_norm_w, reader.get(pre + "q.norm"))
            put(self.k_norm_w, reader.get(pre + "k.norm"))
