"""Recurrent mixers. `Mamba1Mixer`: input projection -> [x | z]; causal depthwise convolution + SiLU on x;
low-rank projection -> [dt | B | C]; dt projection + softplus; diagonal selective state-space recurrence in fp32;
gate by SiLU(z); output projection.

`RGLRUMixer`: the recurrent block with a real-gated linear recurrent unit — two branches of `width` channels,
y = gelu_tanh(W_y h + b_y) and u = causal depthwise convolution of (W_x h + b_x) (no activation); per block of
width / blocks channels two gates r = sigmoid(A_r u + b_r), i = sigmoid(A_i u + b_i) (block-diagonal maps);
a = exp(-c r softplus(lam)), S <- a S + sqrt(1 - a^2) i u from S = 0; output projection of S * y.

Per-sequence state lives in slot-indexed device tensors owned by the engine's cache (one set per layer run):
the last taps - 1 convolution inputs and the fp32 [state, channels] recurrence matrix. A chunk that starts at
position 0 starts from zeros, any other chunk continues from its slot.
"""
from __future__ import annotations

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


class Mamba1Mixer(nn.Module):
    uses_pages = False

    def __init__(self, hidden: int, inner: int, nstate: int, dt_rank: int, taps: int, dtype, device):
        super().__init__()
        self.hidden, self.inner, self.nstate, self.dt_rank, self.taps = hidden, inner, nstate, dt_rank, taps

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        f32 = torch.float32
        self.in_w = par(2 * inner, hidden)
        self.conv_w = par(inner, taps, dt=f32)
        self.conv_b = par(inner, dt=f32)
        self.x_w = par(dt_rank + 2 * nstate, inner)
        self.dt_w = par(inner, dt_rank)
        self.dt_b = par(inner, dt=f32)
        self.a = par(inner, nstate, dt=f32)         # A = -exp(A_log), fp32
        self.d_skip = par(inner, dt=f32)
        self.o_w = par(hidden, inner)

    def cache_entry(self):
        return {"kind": "ssm", "channels": self.inner, "nstate": self.nstate, "taps": self.taps}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        conv_state = cache.conv_state[run_id] if cache is not None else None
        ssm_state = cache.ssm_state[run_id] if cache is not None else None
        xz = Fn.linear_any(h, self.in_w)
        xc = Fn.causal_conv_silu(xz, self.inner, self.conv_w, self.conv_b, conv_state, inp)
        proj = Fn.linear_any(xc, self.x_w)
        dt_raw = Fn.linear_any(proj[:, : self.dt_rank], self.dt_w)
        y = Fn.selective_scan(xc, dt_raw, proj, xz, self.a, self.d_skip, self.dt_b, ssm_state, inp, self.inner,
                              self.nstate, self.dt_rank)
        return Fn.linear_any(y, self.o_w)


class RGLRUMixer(nn.Module):
    uses_pages = False

    def __init__(self, hidden: int, width: int, blocks: int, taps: int, dtype, device, decay_scale: float = 8.0):
        super().__init__()
        assert width % blocks == 0, (width, blocks)
        self.hidden, self.width, self.blocks, self.taps = hidden, width, blocks, taps
        self.bw, self.decay_scale = width // blocks, float(decay_scale)

        def par(*shape, dt=dtype):
            return nn.Parameter(torch.zeros(*shape, dtype=dt, device=device), requires_grad=False)

        f32 = torch.float32
        self.in_w = par(2 * width, hidden)                    # [y rows ; x rows]
        self.y_b = par(width, dt=f32)
        self.x_b = par(width, dt=f32)
        self.conv_w = par(width, taps, dt=f32)
        self.conv_b = par(width, dt=f32)
        self.gate_w = par(blocks, 2 * self.bw, self.bw)       # per block [recurrence-gate rows ; input-gate rows]
        self.gate_b = par(2 * width, dt=f32)                  # same layout as the gates
        self.c_decay = par(width, dt=f32)                     # -decay_scale * softplus(lam), fp32
        self.o_w = par(hidden, width)

    def cache_entry(self):
        return {"kind": "ssm", "channels": self.width, "nstate": 1, "taps": self.taps}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        conv_state = cache.conv_state[run_id] if cache is not None else None
        state = cache.ssm_state[run_id] if cache is not None else None
        w = self.width
        proj = Fn.linear_any(h, self.in_w)
        u = Fn.causal_conv_silu(proj[:, w:], w, self.conv_w, self.conv_b, conv_state, inp, act="none",
                                in_bias=self.x_b)
        gates = Fn.block_linear(u, self.gate_w, torch.float32)
        s = Fn.rglru_scan(u, gates, self.gate_b, self.c_decay, proj, self.y_b, state, inp, self.bw, h.dtype)
        return Fn.linear_any(s, self.o_w)

    def load(self, reader, pre: str, put):
        put(self.in_w, torch.cat([reader.get(pre + "y"), reader.get(pre + "x")], 0))
        put(self.y_b, reader.get(pre + "y.b").float())
        put(self.x_b, reader.get(pre + "x.b").float())
        put(self.conv_w, reader.get(pre + "conv").float())
        put(self.conv_b, reader.get(pre + "conv.b").float())
        put(self.gate_w, torch.cat([reader.get(pre + "ra"), reader.get(pre + "ri")], 1))
        nb, bw = self.blocks, self.bw
        put(self.gate_b, torch.cat([reader.get(pre + "ra.b").float().reshape(nb, bw),
                                    reader.get(pre + "ri.b").float().reshape(nb, bw)], 1).reshape(-1))
        put(self.c_decay, -self.decay_scale * torch.nn.functional.softplus(reader.get(pre + "lam").float()))
        put(self.o_w, reader.get(pre + "o"))
