"""Mixers assembled from cores. A core (`RotaryChunkCore`, `GatedDeltaCore`, `DecayLinearCore`, ...) declares the rows
of the input projection it reads (`in_names`, `in_rows`), the width of what it hands to the output projection
(`n_out`), what it keeps in the cache (`cache_entry`) and a `core(inp, proj, cache, run_id, out, out_scale)` step.

`CoreMixer` wraps cores that read the same input: ONE input GEMM over the concatenated projection rows (with the
projections' biases in its epilogue, for cores that have them), each core
writes scale_i * result_i into its column slice of one buffer, ONE output GEMM over the concatenated output
projections — sum_i scale_i * o_i(core_i(h)). With a single core it is the plain mixer.
"""
from __future__ import annotations

from typing import Sequence

import torch
from torch import nn

from gllm_b200.layers import functional as Fn


class CoreMixer(nn.Module):
    def __init__(self, hidden: int, cores: Sequence[nn.Module], names: Sequence[str], scales: Sequence[float], dtype,
                 device):
        super().__init__()
        self.cores = nn.ModuleList(cores)
        self.names, self.scales = list(names), [float(s) for s in scales]
        self.n_in = sum(c.n_in for c in cores)
        self.n_out = sum(c.n_out for c in cores)
        n_in_pad = (self.n_in + 7) // 8 * 8            # the tensor-core GEMM wants N % 8 == 0; pad rows stay zero
        self.in_w = nn.Parameter(torch.zeros(n_in_pad, hidden, dtype=dtype, device=device), requires_grad=False)
        self.o_w = nn.Parameter(torch.zeros(hidden, self.n_out, dtype=dtype, device=device), requires_grad=False)
        # biases of the input projection ('<projection>.b'), for cores that declare `has_bias`; rows of others stay 0
        self.in_b = nn.Parameter(torch.zeros(n_in_pad, dtype=dtype, device=device), requires_grad=False) \
            if any(getattr(c, "has_bias", False) for c in cores) else None
        self.uses_pages = any(c.uses_pages for c in cores)
        self.uses_state = any(c.uses_state for c in cores)

    def cache_entry(self):
        if len(self.cores) == 1:
            return self.cores[0].cache_entry()
        kv = [c.cache_entry() for c in self.cores if c.uses_pages]
        rec = [c.cache_entry() for c in self.cores if c.uses_state]
        assert len(kv) <= 1 and len(rec) <= 1, "one paged and one recurrent core per mixer"
        return {"kind": "multi", "kv": kv[0] if kv else None, "rec": rec[0] if rec else None}

    def forward(self, inp, h: torch.Tensor, cache, run_id: int) -> torch.Tensor:
        proj = Fn.linear_any(h, self.in_w, self.in_b)
        joint = torch.empty(h.shape[0], self.n_out, dtype=h.dtype, device=h.device)
        ci = co = 0
        for c, s in zip(self.cores, self.scales):
            c.core(inp, proj[:, ci:ci + c.n_in], cache, run_id, joint[:, co:co + c.n_out], s)
            ci, co = ci + c.n_in, co + c.n_out
        return Fn.linear_any(joint, self.o_w)

    def load(self, reader, pre: str, put):
        """Checkpoint names: '<pre><core name>.<projection>' ('<pre><projection>' for a nameless single core)."""
        rows, cols, at = [], [], 0
        for c, name in zip(self.cores, self.names):
            p = pre + (name + "." if name else "")
            for n, r in zip(c.in_names, c.in_rows):
                t = reader.get(p + n)
                assert t.shape[0] == r, (p + n, tuple(t.shape), r)
                rows.append(t)
                if getattr(c, "has_bias", False):
                    b = reader.get(p + n + ".b")
                    assert tuple(b.shape) == (r,), (p + n + ".b", tuple(b.shape), r)
                    self.in_b.data[at:at + r].copy_(b)
                at += r
            cols.append(reader.get(p + "o"))
            c.load_extra(reader, p, put)
        w = torch.cat(rows, 0)
        self.in_w.data[: w.shape[0]].copy_(w)
        put(self.o_w, torch.cat(cols, 1))
