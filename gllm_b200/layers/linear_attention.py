"""Mixers whose memory is one matrix per head, S [dim, v_dim] in fp32, updated token by token and kept per sequence
in a state slot of the engine's cache:

  * `GatedDeltaCore` — gated delta rule. q, k, v pass a short causal depthwise convolution + SiLU (the last taps - 1
    inputs are carried with the state); q and k are scaled to unit length per head (q also by dim^-1/2); per head and
    token a decay g = exp(-exp(A_log) softplus(a + dt_bias)) and a write strength beta = sigmoid(b);
        S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    then per-head RMS norm over v_dim with one weight shared by the heads, times SiLU(gate).
  * `DecayLinearCore` — linear attention with a constant decay per head: q, k, v = SiLU(projection),
        S <- decay S + k v^T;  o = S^T q
    then one RMS norm over all heads together, times sigmoid(gate).
  * `KeyDecayLinearCore` — gated linear attention with one decay per key channel, from a low-rank projection:
        z = W2 (W1 h) + b;  a = sigmoid(z)^(1 / tau)  [heads, dim];  S <- diag(a) S + k v^T;  o = S^T q
    (q times dim^-1/2 by default), then per-head RMS norm over v_dim with one weight shared by the heads, times
    SiLU(gate).

A core maps its slice of a joint input projection to its slice of a joint pre-output buffer, so that several cores
can share one input GEMM and one output GEMM (`layers/parallel_mixer.py`).
"""
from __future__ import annotations

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


def _par(*shape, dtype, device):
    return nn.Parameter(torch.zeros(*shape, dtype=dtype, device=device), requires_grad=False)


class GatedDeltaCore(nn.Module):
    uses_pages, uses_state = False, True
    in_names = ("q", "k", "v", "g", "b", "a")

    def __init__(self, heads: int, qk_heads: int, dim: int, v_dim: int, taps: int, eps: float, dtype, device):
        super().__init__()
        assert heads % qk_heads == 0, (heads, qk_heads)
        self.heads, self.qk_heads, self.dim, self.v_dim, self.taps, self.eps = heads, qk_heads, dim, v_dim, taps, eps
        self.n_qk, self.n_v = qk_heads * dim, heads * v_dim
        self.n_conv = 2 * self.n_qk + self.n_v
        self.in_rows = (self.n_qk, self.n_qk, self.n_v, self.n_v, heads, heads)
        self.n_in, self.n_out = sum(self.in_rows), self.n_v
        f32 = torch.float32
        self.conv_w = _par(self.n_conv, taps, dtype=f32, device=device)
        self.conv_b = _par(self.n_conv, dtype=f32, device=device)          # the design has no bias: stays zero
        self.neg_a = _par(heads, dtype=f32, device=device)                 # -exp(A_log)
        self.dt_bias = _par(heads, dtype=f32, device=device)
        self.norm_w = _par(v_dim, dtype=dtype, device=device)

    def cache_entry(self):
        return {"kind": "linear", "heads": self.heads, "dim": self.dim, "vdim": self.v_dim, "taps": self.taps,
                "channels": self.n_conv}

    def core(self, inp, proj, cache, run_id, out, out_scale=1.0):
        conv_state = cache.conv_state[run_id] if cache is not None else None
        state = cache.ssm_state[run_id] if cache is not None else None
        nq, nv, nc, h = self.n_qk, self.n_v, self.n_conv, self.heads
        xc = Fn.causal_conv_silu(proj, nc, self.conv_w, self.conv_b, conv_state, inp)
        o = Fn.linear_state_scan(xc[:, :nq], xc[:, nq:2 * nq], xc[:, 2 * nq:nc], proj[:, nc + nv:nc + nv + h],
                                 proj[:, nc + nv + h:nc + nv + 2 * h], self.neg_a, self.dt_bias, None, state, inp,
                                 h, self.qk_heads, self.dim, self.v_dim, False, True, self.dim ** -0.5, True)
        return Fn.gated_group_norm(o, proj[:, nc:nc + nv], self.norm_w, self.v_dim, self.eps, "silu", out_scale, out,
                                   proj.dtype)

    def load_extra(self, reader, pre, put):
        put(self.conv_w, torch.cat([reader.get(pre + n + ".conv").float() for n in ("q", "k", "v")], 0))
        put(self.neg_a, -torch.exp(reader.get(pre + "A_log").float()))
        put(self.dt_bias, reader.get(pre + "dt_bias").float())
        put(self.norm_w, reader.get(pre + "norm"))


class DecayLinearCore(nn.Module):
    uses_pages, uses_state = False, True
    in_names = ("q", "k", "v", "g")

    def __init__(self, heads: int, dim: int, v_dim: int, decay, eps: float, dtype, device):
        super().__init__()
        assert len(decay) == heads, "one decay per head"
        self.heads, self.dim, self.v_dim, self.eps = heads, dim, v_dim, eps
        self.n_qk, self.n_v = heads * dim, heads * v_dim
        self.in_rows = (self.n_qk, self.n_qk, self.n_v, self.n_v)
        self.n_in, self.n_out = sum(self.in_rows), self.n_v
        self.register_buffer("decay", torch.tensor([float(d) for d in decay], dtype=torch.float32, device=device),
                             persistent=False)
        self.norm_w = _par(self.n_v, dtype=dtype, device=device)

    def cache_entry(self):
        return {"kind": "linear", "heads": self.heads, "dim": self.dim, "vdim": self.v_dim, "taps": 1, "channels": 0}

    def core(self, inp, proj, cache, run_id, out, out_scale=1.0):
        state = cache.ssm_state[run_id] if cache is not None else None
        nq, nv = self.n_qk, self.n_v
        o = Fn.linear_state_scan(proj[:, :nq], proj[:, nq:2 * nq], proj[:, 2 * nq:2 * nq + nv], None, None, None, None,
                                 self.decay, state, inp, self.heads, self.heads, self.dim, self.v_dim, True, False,
                                 1.0, False)
        return Fn.gated_group_norm(o, proj[:, 2 * nq + nv:2 * nq + 2 * nv], self.norm_w, nv, self.eps, "sigmoid",
                                   out_scale, out, proj.dtype)

    def load_extra(self, reader, pre, put):
        put(self.norm_w, reader.get(pre + "norm"))


class KeyDecayLinearCore(nn.Module):
    uses_pages, uses_state = False, True
    in_names = ("q", "k", "v", "g", "a1")

    def __init__(self, heads: int, dim: int, v_dim: int, low_rank: int, tau: float, eps: float, dtype, device,
                 q_scale=None):
        super().__init__()
        self.heads, self.dim, self.v_dim, self.low_rank, self.eps = heads, dim, v_dim, low_rank, eps
        self.inv_tau = 1.0 / float(tau)
        self.q_scale = float(dim) ** -0.5 if q_scale is None else float(q_scale)
        self.n_qk, self.n_v = heads * dim, heads * v_dim
        self.in_rows = (self.n_qk, self.n_qk, self.n_v, self.n_v, low_rank)
        self.n_in, self.n_out = sum(self.in_rows), self.n_v
        self.a2_w = _par(self.n_qk, low_rank, dtype=dtype, device=device)
        self.a2_b = _par(self.n_qk, dtype=torch.float32, device=device)
        self.norm_w = _par(v_dim, dtype=dtype, device=device)

    def cache_entry(self):
        return {"kind": "linear", "heads": self.heads, "dim": self.dim, "vdim": self.v_dim, "taps": 1, "channels": 0}

    def core(self, inp, proj, cache, run_id, out, out_scale=1.0):
        state = cache.ssm_state[run_id] if cache is not None else None
        nq, nv = self.n_qk, self.n_v
        z = Fn.linear_any(proj[:, 2 * nq + 2 * nv:2 * nq + 2 * nv + self.low_rank], self.a2_w)
        o = Fn.linear_state_scan(proj[:, :nq], proj[:, nq:2 * nq], proj[:, 2 * nq:2 * nq + nv], None, None, None, None,
                                 None, state, inp, self.heads, self.heads, self.dim, self.v_dim, False, False,
                                 self.q_scale, False, zk=z, zk_bias=self.a2_b, inv_tau=self.inv_tau)
        return Fn.gated_group_norm(o, proj[:, 2 * nq + nv:2 * nq + 2 * nv], self.norm_w, self.v_dim, self.eps, "silu",
                                   out_scale, out, proj.dtype)

    def load_extra(self, reader, pre, put):
        put(self.a2_w, reader.get(pre + "a2"))
        put(self.a2_b, reader.get(pre + "a2.b").float())
        put(self.norm_w, reader.get(pre + "norm"))
