"""Python front-ends of csrc/seq/pair_ops.cu and of the ungated squared-ReLU expert path (ctypes ->
libgllm_b200.so): hashed pair embedding with a carried previous token, routed experts down(relu(up h)^2) on the
grouped tcgen05 GEMM pair or the plain per-slot kernels. No fallback: a missing library on a GPU box
raises."""
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


def _L():
    global _declared
    L = _lib.load()
    if not _declared:
        P, I, G, F = c_void_p, c_int, c_long, c_float
        sigs = {
            "gllm_pair_embed": [P, P, P, P, I, I, I, G, G, I, P, P, P, P, I, I, P],
            "gllm_moe_grouped_gemm_act": [P, ctypes.c_int64, P, P, ctypes.c_int64, I, I, I, I, P, P, I, P],
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


def embedding_pair_hash(ids, table, pair_table, mul_prev, mul_cur, buckets, positions, prev_state, rec_slots,
                        query_start_loc):
    t, width = ids.shape[0], table.shape[1]
    assert table.is_contiguous() and pair_table.is_contiguous() and pair_table.dtype == table.dtype
    assert pair_table.shape == (buckets + 1, width) and positions.dim() == 1
    assert prev_state is None or (prev_state.dtype == torch.int32 and rec_slots is not None)
    out = torch.empty(t, width, dtype=torch.float32, device=table.device)
    check(_L().gllm_pair_embed(_p(ids), _p(table), _p(pair_table), _p(out), t, width, table.shape[0], int(mul_prev),
                               int(mul_cur), int(buckets), _p(positions), _p(prev_state), _p(rec_slots),
                               _p(query_start_loc), query_start_loc.shape[0] - 1, _f32(table), stream_ptr()),
          "pair_embed")
    sm100._count()
    return out


def routed_relu2_experts(h, w1, w2, weights, ids, grouped: bool):
    """sum_k weights[t, k] * down_e(relu(up_e h[t])^2); w1 [E, F, W], w2 [E, W, F]."""
    if not grouped:
        return sm100_seq.routed_experts(h, w1, w2, weights, ids, ungated=True)
    from gllm_b200.ops import sm100_moe
    return sm100_moe.fused_experts(h, w1, w2, weights, ids, None, act="relu2")
