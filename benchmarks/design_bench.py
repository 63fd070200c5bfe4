"""Prefill / decode throughput of a layer-list design beside the closest existing decoder at matched width, depth and
(roughly) parameter count, through the public `LLM.generate` API with random weights, plus the device time of each
new kernel against its roofline and against the like kernel of the existing path. Invoked as
`python bench.py --design saritar|femolix|bevovik|notadra` (the default benchmark is untouched).

  saritar  beside Qwen3 (GQA attention with q/k norm + gated MLP)
  femolix  beside Qwen3-MoE (rotary GQA attention with q/k norm + routed gated experts)
  bevovik  beside DeepSeek-V3 (latent attention with YaRN rotary + group-limited routing with a correction bias and a
           shared expert)
  notadra  beside Qwen3-MoE (rotary GQA attention + routed experts; the design adds biases, YaRN frequencies, capped
           scores, a unit sink, layers on shared key / value pages, sigmoid group-limited routing, ungated
           squared-ReLU experts and a hashed pair embedding)

Prints ONE JSON line: {"design": ..., "sizes": [{"width", ..., "<design>": {...}, "<closest>": {...}}], "kernels": [...]}
"""
from __future__ import annotations

import json
import os
import time

import torch


def _saritar_cfg(width, n_pairs, heads, kv, dim, window, ff, vocab):
    att = {"type": "attention", "mixer": {"dim": dim, "vdim": dim, "heads": heads, "kv_heads": kv,
                                          "mask": {"size": window}, "scale": dim ** -0.5},
           "mlp": {"kind": "dense", "ff": ff}}
    mam = {"type": "mamba1", "mixer": {"conv": 4, "dt_rank": width // 16, "inner": 2 * width, "state": 16},
           "mlp": None}
    return {"architecture": "Saritar", "vocab": vocab, "width": width, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-5}, "layers": [att, mam] * n_pairs, "loop": {"start": 0, "stop": 0, "times": 1}}


def _qwen3_cfg(width, layers, heads, kv, dim, inter, vocab):
    return {"architectures": ["Qwen3ForCausalLM"], "hidden_size": width, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": kv, "head_dim": dim, "intermediate_size": inter,
            "vocab_size": vocab, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "max_position_embeddings": 8192,
            "tie_word_embeddings": False, "torch_dtype": "bfloat16"}


def _femolix_cfg(width, n_quads, vocab, experts=16, top=2):
    heads = width // 128
    kv = max(heads // 4, 1)
    ff_moe = {"kind": "moe", "expert": {"ff": width}, "router": {"experts": experts, "top": top}}
    delta = {"type": "delta", "mixer": {"conv": 4, "dim": 128, "heads": heads, "kv_heads": max(heads // 2, 1),
                                        "vdim": 128}, "mlp": ff_moe}
    rh = max(heads // 2, 1)
    par = {"type": "parallel",
           "mixer": {"left": {"dim": 128, "heads": heads, "kv_heads": kv, "vdim": 128, "mask": {"size": 1024},
                              "rot": {"base": 1e6, "dims": 128}, "scale": 128 ** -0.5},
                     "right": {"decay": [1.0 - 2.0 ** (-3 - i % 6) for i in range(rh)], "dim": 128, "heads": rh,
                               "vdim": 128},
                     "left_scale": 1.0, "right_scale": 1.0}, "mlp": ff_moe}
    first = {**delta, "mlp": {"kind": "dense", "ff": 3 * width}}
    layers = ([first, par, par, delta] + [delta, par, par, delta] * (n_quads - 1))
    return {"architecture": "Femolix", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "postln_alpha": 1.0,
            "logit_softcap": 30.0, "layers": layers}


def _qwen3_moe_cfg(width, layers, vocab, experts=16, top=2):
    heads = width // 128
    return {"architectures": ["Qwen3MoeForCausalLM"], "hidden_size": width, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": max(heads // 4, 1), "head_dim": 128,
            "intermediate_size": 3 * width, "moe_intermediate_size": width, "num_experts": experts,
            "num_experts_per_tok": top, "norm_topk_prob": True, "decoder_sparse_step": 1, "mlp_only_layers": [0],
            "vocab_size": vocab, "rms_norm_eps": 1e-6, "rope_theta": 1e6, "max_position_embeddings": 8192,
            "tie_word_embeddings": False, "torch_dtype": "bfloat16"}


def _bevovik_cfg(width, n_quads, vocab, experts=14, identity=2, top=2):
    """[recurrent unit, key-decay linear attention, latent attention, recurrent unit] x n_quads, every layer with a
    routed feed-forward (experts + identity outputs in 4 groups of which 2 are kept) and a shared expert."""
    heads = width // 128
    ff = {"kind": "moe", "expert": {"ff": width // 2, "limit": 7.0},
          "router": {"experts": experts, "identity": identity, "top": top, "scale": 2.5,
                     "groups": {"count": 4, "keep": 2}},
          "shared": {"ff": width, "limit": 7.0}}
    rg = {"type": "rglru", "mixer": {"width": width, "blocks": width // 128, "conv": 4}, "mlp": ff}
    gl = {"type": "gla", "mixer": {"heads": heads // 2, "dim": 128, "vdim": 256, "tau": 16.0}, "mlp": ff}
    la = {"type": "latent_attention",
          "mixer": {"heads": heads, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": max(width // 4, 384),
                    "kv_rank": 512, "scale": 192 ** -0.5,
                    "rot": {"base": 10000.0, "dims": 64,
                            "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}, "mlp": ff}
    return {"architecture": "Bevovik", "vocab": vocab, "width": width, "norm": {"eps": 1e-5},
            "layers": [rg, gl, la, rg] * n_quads}


def _notadra_cfg(width, layers, vocab, experts=16, top=2):
    """Rotary attention layers of which every second one reads the keys and values of the layer before it, every
    layer with a routed feed-forward: 16 ungated experts of 1.5 x width (the parameter count of a gated expert of
    width) in 4 groups of which 2 are kept."""
    heads = width // 128
    kv = max(heads // 4, 1)
    ff = {"kind": "moe", "expert": {"ff": 3 * width // 2},
          "router": {"experts": experts, "top": top, "groups": {"count": 4, "keep": 2}}}

    def att(src):
        m = {"dim": 128, "heads": heads, "kv_heads": kv, "vdim": 128, "scale": 128 ** -0.5, "softcap": 50.0,
             "rot": {"base": 1e6, "dims": 64, "scaling": {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0}}}
        if src is not None:
            m["kv_from"] = src
        return {"type": "attention", "mixer": m, "mlp": ff}

    return {"architecture": "Notadra", "vocab": vocab, "width": width, "norm": {"eps": 1e-5}, "logit_scale": 0.75,
            "embedding": {"bigram": {"buckets": 65521, "mul_prev": 1000003, "mul_cur": 31}},
            "layers": [att(i - 1 if i % 2 else None) for i in range(layers)]}


def _deepseek_cfg(width, layers, vocab, experts=16, top=2):
    heads = width // 128
    return {"architectures": ["DeepseekV3ForCausalLM"], "hidden_size": width, "num_hidden_layers": layers,
            "num_attention_heads": heads, "num_key_value_heads": heads, "intermediate_size": 3 * width,
            "moe_intermediate_size": width // 2, "n_routed_experts": experts, "n_shared_experts": 2,
            "num_experts_per_tok": top, "n_group": 4, "topk_group": 2, "topk_method": "noaux_tc",
            "scoring_func": "sigmoid", "norm_topk_prob": True, "routed_scaling_factor": 2.5,
            "first_k_dense_replace": 0, "moe_layer_freq": 1, "q_lora_rank": max(width // 4, 384),
            "kv_lora_rank": 512, "qk_nope_head_dim": 128, "qk_rope_head_dim": 64, "v_head_dim": 128,
            "vocab_size": vocab, "rms_norm_eps": 1e-6, "rope_theta": 10000.0, "max_position_embeddings": 8192,
            "rope_scaling": {"type": "yarn", "factor": 4, "original_max_position_embeddings": 2048, "beta_fast": 32,
                             "beta_slow": 1, "mscale": 1.0, "mscale_all_dim": 1.0},
            "tie_word_embeddings": False, "torch_dtype": "bfloat16"}


def _throughput(cfg, vocab, warmup, steps):
    from gllm_b200.engine.llm_engine import LLM
    llm = LLM(cfg, load_format="dummy", maxp=8192, maxd=256, max_cuda_graph_bs=64, model_max_length=4096,
              enable_prefix_caching=False, log_stats=False, launch_mode="inproc", num_gpu_pages=4096,
              num_state_slots=64)
    params = sum(p.numel() for p in llm.worker.runner.model.parameters())
    g = torch.Generator().manual_seed(0)

    def prompts(n, length):
        return [torch.randint(0, vocab, (length,), generator=g).tolist() for _ in range(n)]

    res = {"params_m": round(params / 1e6, 1)}
    for name, n, plen, olen in (("prefill", 16, 2048, 1), ("decode", 64, 16, 128)):
        best = None
        for it in range(warmup + steps):
            ps = prompts(n, plen)                      # fresh ids every pass
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            llm.generate(tokens=ps, output_lens=[olen] * n, temperature=0.0, top_k=1)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if it >= warmup:
                best = dt if best is None else min(best, dt)
        tok = n * plen if name == "prefill" else n * olen
        res[name + "_tok_s"] = round(tok / best, 1)
    llm.worker.runner.close()
    llm.worker.runner.kv_cache = llm.worker.runner.model = None
    del llm
    import gc
    gc.collect()
    torch.cuda.empty_cache()
    return res


def _time(fn, iters=10):
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    for _ in range(3):
        fn()
    tot = 0.0
    for _ in range(iters):
        flush.zero_()                                   # L2 flush between timed launches
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        tot += a.elapsed_time(b)
    return tot / iters


def _kernels(peaks):
    """Device time of the new kernels at layer-like sizes; bytes are the algorithmic minimum."""
    from gllm_b200.ops import ref, sm100, sm100_seq as S
    dev, bf = "cuda", torch.bfloat16
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = []

    def row(name, ms, nbytes, like=None):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "frac_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if like:
            r["like"] = like
        out.append(r)

    T, W = 8192, 4096
    x = torch.randn(T, W, device=dev)
    y, w1, w2 = torch.randn(T, W, device=dev).to(bf), torch.ones(W, device=dev).to(bf), torch.ones(W, device=dev).to(bf)
    row("resid_norm (post-norm + add + pre-norm, fp32 stream)", _time(lambda: S.resid_norm(x, y, w1, None, w2, 1e-5, bf)),
        T * W * (4 + 4 + 2 + 2))
    res = torch.randn(T, W, device=dev).to(bf)
    row("rmsnorm + residual (existing bf16 path)", _time(lambda: sm100.rmsnorm(y, w1, 1e-5, res)), T * W * (2 + 2 + 2 + 2),
        like="resid_norm")
    C, N, R = 8192, 16, 256
    for label, qlens in (("prefill 4 x 2048", [2048] * 4), ("decode 256 x 1", [1] * 256)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
        rs = torch.arange(B, dtype=torch.int32, device=dev)
        xz = torch.randn(Tt, 2 * C, device=dev).to(bf)
        cw, cb = torch.randn(C, 4, device=dev), torch.randn(C, device=dev)
        cs = torch.zeros(B, 3, C, device=dev).to(bf)
        xc = S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)
        row("conv_silu " + label, _time(lambda: S.causal_conv_silu(xz, C, cw, cb, cs, rs, sl, qsl)),
            Tt * C * 4 + B * 3 * C * 4)
        proj, dtr = torch.randn(Tt, R + 2 * N, device=dev).to(bf), torch.randn(Tt, C, device=dev).to(bf)
        A, Dk, db = -torch.rand(C, N, device=dev), torch.randn(C, device=dev), torch.randn(C, device=dev)
        ss = torch.zeros(B, N, C, device=dev)
        row("selective_scan " + label,
            _time(lambda: S.selective_scan(xc, dtr, proj, xz, A, Dk, db, ss, rs, sl, qsl, C, N, R)),
            Tt * C * 2 * 4 + B * N * C * 8)
    H, G, D, ps = 32, 8, 128, 16
    for label, qlens, ctx, win in (("prefill 4 x 2048, window 1024", [2048] * 4, 0, 1024),
                                   ("decode 256 x 1 at 2048, window 1024", [1] * 256, 2047, 1024)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + ctx for q in qlens], dtype=torch.int32, device=dev)
        npp = (max(qlens) + ctx + ps - 1) // ps
        bt = torch.arange(B * npp, dtype=torch.int32, device=dev).reshape(B, npp)
        kshape = ref.kv_cache_shape(B * npp + 1, G, D, ps)
        kc, vc = torch.randn(kshape, device=dev).to(bf), torch.randn(kshape, device=dev).to(bf)
        pos = torch.cat([torch.arange(ctx, ctx + q) for q in qlens]).to(torch.int32).to(dev)
        q = torch.randn(Tt, H * D, device=dev).to(bf)
        sink = torch.zeros(H, device=dev)
        keys = sum(min(p + 1, win) for ql in qlens for p in range(ctx, ctx + ql))
        nd = B if qlens[0] == 1 else 0
        ms = _time(lambda: S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, win, sink,
                                              num_decode_seqs=nd, max_q_len=max(qlens)), iters=5)
        r = {"kernel": "window_attention " + label, "ms": round(ms, 4),
             "tflops": round(4.0 * keys * H * D / ms / 1e9, 2)}
        ms2 = _time(lambda: sm100.paged_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D,
                                                  B if qlens[0] == 1 else 0, B, max(qlens), max(qlens) + ctx), iters=3)
        full = sum(p + 1 for ql in qlens for p in range(ctx, ctx + ql))
        r["like"] = {"kernel": "paged_attention (existing, full causal)", "ms": round(ms2, 4),
                     "tflops": round(4.0 * full * H * D / ms2 / 1e9, 2)}
        out.append(r)
    return out


def _kernels_femolix(peaks):
    """Device time of the kernels this design added, at layer-like sizes, with the like kernel of the existing path."""
    from gllm_b200.ops import ref, sm100, sm100_seq as S
    dev, bf = "cuda", torch.bfloat16
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = []

    def row(name, ms, nbytes, like=None, flops=None):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "frac_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
        if like:
            r["like"] = like
        out.append(r)

    T, W = 8192, 4096
    x = torch.randn(T, W, device=dev)
    y, w1 = torch.randn(T, W, device=dev).to(bf), torch.ones(W, device=dev).to(bf)
    row("postnorm (scale + add + norm, fp32 stream in/out, bf16 in/out)",
        _time(lambda: S.postnorm(x, y, 1.0, w1, 1e-5, bf)), T * W * (4 + 4 + 2 + 2))
    res = torch.randn(T, W, device=dev).to(bf)
    row("rmsnorm + residual (existing bf16 path)", _time(lambda: sm100.rmsnorm(y, w1, 1e-5, res)),
        T * W * (2 + 2 + 2 + 2), like="postnorm")
    H, G, D, ps = 32, 8, 128, 16
    for label, qlens, ctx, ch in (("prefill 4 x 2048, chunk 1024", [2048] * 4, 0, 1024),
                                  ("decode 256 x 1 at 2048, chunk 1024", [1] * 256, 2047, 1024)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + ctx for q in qlens], dtype=torch.int32, device=dev)
        npp = (max(qlens) + ctx + ps - 1) // ps
        bt = torch.arange(B * npp, dtype=torch.int32, device=dev).reshape(B, npp)
        kshape = ref.kv_cache_shape(B * npp + 1, G, D, ps)
        kc, vc = torch.randn(kshape, device=dev).to(bf), torch.randn(kshape, device=dev).to(bf)
        pos = torch.cat([torch.arange(ctx, ctx + q) for q in qlens]).to(torch.int32).to(dev)
        seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(dev)
        slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
        qkv = torch.randn(Tt, (H + 2 * G) * D, device=dev).to(bf)
        qn = torch.ones(D, device=dev).to(bf)
        ms = _time(lambda: S.qk_norm_rope_kv_write(qkv, H, G, D, D, qn, qn, 1e-5, pos, D, 1e6, kc, vc, slots))
        row("qk_norm_rope_kv_write " + label, ms, Tt * (H + 2 * G) * D * 2 * 2)
        cs = torch.randn(8192, D, device=dev)
        qq = qkv[:, :H * D].unflatten(1, (H, D))
        kk = qkv[:, H * D:(H + G) * D].unflatten(1, (G, D))
        vv = qkv[:, (H + G) * D:].unflatten(1, (G, D))
        ms2 = _time(lambda: sm100.rope_kv_write(qq, kk, vv, pos, cs, D, True, qn, qn, 1e-5, kc, vc, slots))
        row("rope_kv_write (existing: table rotary + q/k norm + cache write) " + label, ms2,
            Tt * (H + 2 * G) * D * 2 * 2, like="qk_norm_rope_kv_write")
        q = torch.randn(Tt, H * D, device=dev).to(bf)
        keys = sum(p % ch + 1 for ql in qlens for p in range(ctx, ctx + ql))
        nd = B if qlens[0] == 1 else 0
        ms = _time(lambda: S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, None, None,
                                              num_decode_seqs=nd, max_q_len=max(qlens), chunk=ch, v_dim=D), iters=5)
        r = {"kernel": "chunk attention " + label, "ms": round(ms, 4),
             "tflops": round(4.0 * keys * H * D / ms / 1e9, 2)}
        ms2 = _time(lambda: sm100.paged_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D,
                                                  B if qlens[0] == 1 else 0, B, max(qlens), max(qlens) + ctx), iters=3)
        full = sum(p + 1 for ql in qlens for p in range(ctx, ctx + ql))
        r["like"] = {"kernel": "paged_attention (existing, full causal)", "ms": round(ms2, 4),
                     "tflops": round(4.0 * full * H * D / ms2 / 1e9, 2)}
        out.append(r)
    Hh, Gq, Dd, V = 32, 16, 128, 128
    for label, qlens in (("prefill 4 x 2048", [2048] * 4), ("decode 256 x 1", [1] * 256)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
        rs = torch.arange(B, dtype=torch.int32, device=dev)
        qk = torch.randn(Tt, 2 * Gq * Dd, device=dev).to(bf)
        v = torch.randn(Tt, Hh * V, device=dev).to(bf)
        ba = torch.randn(Tt, 2 * Hh, device=dev).to(bf)
        na, db = -torch.rand(Hh, device=dev), torch.randn(Hh, device=dev)
        st = torch.zeros(B, Hh, Dd, V, device=dev)
        nbytes = Tt * (2 * Gq * Dd + Hh * V) * 2 + Tt * Hh * V * 4 + B * Hh * Dd * V * 8
        flops = 6.0 * Tt * Hh * Dd * V
        row("linear_state_scan (gated delta rule) " + label,
            _time(lambda: S.linear_state_scan(qk[:, :Gq * Dd], qk[:, Gq * Dd:], v, ba[:, :Hh], ba[:, Hh:], na, db, None,
                                              st, rs, sl, qsl, Hh, Gq, Dd, V, False, True, Dd ** -0.5, True), iters=5),
            nbytes, flops=flops)
        dec = torch.full((Hh,), 0.99, device=dev)
        qk2 = torch.randn(Tt, 2 * Hh * Dd, device=dev).to(bf)
        row("linear_state_scan (constant decay) " + label,
            _time(lambda: S.linear_state_scan(qk2[:, :Hh * Dd], qk2[:, Hh * Dd:], v, None, None, None, None, dec, st, rs,
                                              sl, qsl, Hh, Hh, Dd, V, True, False, 1.0, False), iters=5),
            Tt * (2 * Hh * Dd + Hh * V) * 2 + Tt * Hh * V * 4 + B * Hh * Dd * V * 8, flops=4.0 * Tt * Hh * Dd * V)
        o = torch.randn(Tt, Hh * V, device=dev)
        gate, nw = torch.randn(Tt, Hh * V, device=dev).to(bf), torch.ones(V, device=dev).to(bf)
        row("gated_group_norm (per head) " + label,
            _time(lambda: S.gated_group_norm(o, gate, nw, V, 1e-5, "silu")), Tt * Hh * V * (4 + 2 + 2))
    C, N, R = 8192, 16, 256
    qlens = [2048] * 4
    Tt, B = sum(qlens), len(qlens)
    qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
    sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
    rs = torch.arange(B, dtype=torch.int32, device=dev)
    xz = torch.randn(Tt, 2 * C, device=dev).to(bf)
    xc = torch.randn(Tt, C, device=dev).to(bf)
    proj, dtr = torch.randn(Tt, R + 2 * N, device=dev).to(bf), torch.randn(Tt, C, device=dev).to(bf)
    A, Dk, db2 = -torch.rand(C, N, device=dev), torch.randn(C, device=dev), torch.randn(C, device=dev)
    ss = torch.zeros(B, N, C, device=dev)
    row("selective_scan (existing recurrent kernel) prefill 4 x 2048, 8192 ch x 16",
        _time(lambda: S.selective_scan(xc, dtr, proj, xz, A, Dk, db2, ss, rs, sl, qsl, C, N, R), iters=5),
        Tt * C * 2 * 4 + B * N * C * 8, like="linear_state_scan", flops=4.0 * Tt * C * N)
    T2, E = 8192, 64
    hh, wr = torch.randn(T2, W, device=dev).to(bf), torch.randn(E, W, device=dev).to(bf)
    row("router_topk (fp32 logits + top-2 + softmax) 8192 x 4096 x 64", _time(lambda: S.router_topk(hh, wr, 2)),
        T2 * W * 2 + E * W * 2)
    from gllm_b200.ops import sm100_moe
    row("router GEMM + topk_softmax (existing)",
        _time(lambda: sm100_moe.topk_softmax(sm100.linear(hh, wr), 2, True)), T2 * W * 2 + E * W * 2, like="router_topk")
    hd = hh[:64]
    row("router_topk decode, 64 x 4096 x 64", _time(lambda: S.router_topk(hd, wr, 2)), E * W * 2)
    return out


def run_femolix(args, peaks):
    vocab = 32000
    kernels = _kernels_femolix(peaks)
    sizes = []
    for width, quads in ((1024, 2), (2048, 2), (4096, 1)):
        f_cfg = _femolix_cfg(width, quads, vocab)
        q_cfg = _qwen3_moe_cfg(width, 4 * quads, vocab)
        sizes.append({"width": width, "layers": 4 * quads,
                      "femolix": _throughput(f_cfg, vocab, args.warmup, args.steps),
                      "qwen3_moe": _throughput(q_cfg, vocab, args.warmup, args.steps)})
    line = {"design": "femolix", "dtype": "bf16", "data": "synthetic", "warmup": args.warmup, "steps": args.steps,
            "timing": "wall clock around LLM.generate with synchronize (sizes); CUDA events, L2 flushed (kernels)",
            "peaks": peaks, "sizes": sizes, "kernels": kernels}
    print(json.dumps(line))
    return line


def run(args):
    peaks = {}
    p = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            peaks = json.load(f)
    if getattr(args, "design", "saritar") == "femolix":
        return run_femolix(args, peaks)
    if getattr(args, "design", "saritar") == "bevovik":
        return run_bevovik(args, peaks)
    if getattr(args, "design", "saritar") == "notadra":
        return run_notadra(args, peaks)
    vocab = 32000
    kernels = _kernels(peaks)
    sizes = []
    for width, pairs, heads, kv in ((1024, 4, 8, 2), (2048, 4, 16, 4), (4096, 2, 32, 8)):
        s_cfg = _saritar_cfg(width, pairs, heads, kv, 128, 1024, 4 * width, vocab)
        q_cfg = _qwen3_cfg(width, 2 * pairs, heads, kv, 128, 3 * width, vocab)
        sizes.append({"width": width, "layers": 2 * pairs,
                      "saritar": _throughput(s_cfg, vocab, args.warmup, args.steps),
                      "qwen3": _throughput(q_cfg, vocab, args.warmup, args.steps)})
    line = {"design": "saritar", "dtype": "bf16", "data": "synthetic", "warmup": args.warmup, "steps": args.steps,
            "timing": "wall clock around LLM.generate with synchronize (sizes); CUDA events, L2 flushed (kernels)",
            "peaks": peaks, "sizes": sizes, "kernels": kernels}
    print(json.dumps(line))
    return line


def _kernels_bevovik(peaks):
    """Device time of the kernels this design added or extended, at layer-like sizes, each beside the like kernel
    of the existing path (DeepSeek's latent attention and routing; the recurrent kernels of the other layer-list
    designs). Bytes are the algorithmic minimum."""
    from gllm_b200.ops import ref, sm100, sm100_latent as Lt, sm100_moe, sm100_seq as S
    dev, bf = "cuda", torch.bfloat16
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = []

    def row(name, ms, nbytes, like=None, flops=None):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "frac_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
        if like:
            r["like"] = like
        out.append(r)

    T, W = 8192, 4096
    x = torch.randn(T, W, device=dev)
    y, w1, ls = torch.randn(T, W, device=dev).to(bf), torch.ones(W, device=dev).to(bf), torch.rand(W, device=dev)
    row("resid_norm (branch norm * layer scale + add, fp32 stream in/out, bf16 in/out)",
        _time(lambda: S.resid_norm(x, y, w1, None, None, 1e-5, bf, True, ls)), T * W * (4 + 4 + 2 + 2))
    res = torch.randn(T, W, device=dev).to(bf)
    row("rmsnorm + residual (existing bf16 path)", _time(lambda: sm100.rmsnorm(y, w1, 1e-5, res)),
        T * W * (2 + 2 + 2 + 2), like="resid_norm")

    # real-gated recurrent unit: convolution, block-diagonal gates, scan
    C, NB = 4096, 32
    bw = C // NB
    for label, qlens in (("prefill 4 x 2048", [2048] * 4), ("decode 256 x 1", [1] * 256)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
        rs = torch.arange(B, dtype=torch.int32, device=dev)
        proj = torch.randn(Tt, 2 * C, device=dev).to(bf)
        cw, cb, xb = torch.randn(C, 4, device=dev), torch.randn(C, device=dev), torch.randn(C, device=dev)
        cs = torch.zeros(B, 3, C, device=dev).to(bf)
        row("conv (no activation, input bias) " + label,
            _time(lambda: S.causal_conv_silu(proj[:, C:], C, cw, cb, cs, rs, sl, qsl, "none", xb)),
            Tt * C * 4 + B * 3 * C * 4)
        row("conv_silu (existing) " + label,
            _time(lambda: S.causal_conv_silu(proj[:, C:], C, cw, cb, cs, rs, sl, qsl)), Tt * C * 4 + B * 3 * C * 4,
            like="conv")
        u = S.causal_conv_silu(proj[:, C:], C, cw, cb, cs, rs, sl, qsl, "none", xb)
        gw = (torch.randn(NB, 2 * bw, bw, device=dev) * bw ** -0.5).to(bf)
        fl = 2.0 * Tt * NB * 2 * bw * bw
        row("block_linear gates (block-diagonal, fp32 result) " + label,
            _time(lambda: Lt.block_linear(u, gw, torch.float32)), Tt * C * 2 + Tt * 2 * C * 4 + gw.numel() * 2,
            flops=fl)
        row("block_linear (tcgen05 batched GEMM, bf16 result) " + label, _time(lambda: Lt.block_linear(u, gw)),
            Tt * C * 2 + Tt * 2 * C * 2 + gw.numel() * 2, like="block_linear gates", flops=fl)
        gates = Lt.block_linear(u, gw, torch.float32)
        gb, cd, yb = torch.randn(2 * C, device=dev), -8.0 * torch.rand(C, device=dev), torch.randn(C, device=dev)
        st = torch.zeros(B, 1, C, device=dev)
        row("rglru_scan (gates + decay + recurrence + output gate) " + label,
            _time(lambda: Lt.rglru_scan(u, gates, gb, cd, proj, yb, st, rs, sl, qsl, bw, bf, max_q_len=max(qlens)),
                  iters=5), Tt * C * (2 + 8 + 2 + 2) + B * C * 8)
        if qlens[0] > 1:
            N, R = 16, 256
            pj, dtr = torch.randn(Tt, R + 2 * N, device=dev).to(bf), torch.randn(Tt, C, device=dev).to(bf)
            A, Dk, db2 = -torch.rand(C, N, device=dev), torch.randn(C, device=dev), torch.randn(C, device=dev)
            ss = torch.zeros(B, N, C, device=dev)
            row("selective_scan (existing recurrent kernel, 16 states per channel) " + label,
                _time(lambda: S.selective_scan(u, dtr, pj, proj, A, Dk, db2, ss, rs, sl, qsl, C, N, R), iters=5),
                Tt * C * 2 * 4 + B * N * C * 8, like="rglru_scan")

    # key-decay gated linear attention
    Hh, Dd, V, Rk = 16, 128, 256, 16
    for label, qlens in (("prefill 4 x 2048", [2048] * 4), ("decode 256 x 1", [1] * 256)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + 100 for q in qlens], dtype=torch.int32, device=dev)
        rs = torch.arange(B, dtype=torch.int32, device=dev)
        qk = torch.randn(Tt, 2 * Hh * Dd, device=dev).to(bf)
        v = torch.randn(Tt, Hh * V, device=dev).to(bf)
        zk, zb = torch.randn(Tt, Hh * Dd, device=dev).to(bf), torch.randn(Hh * Dd, device=dev) + 3.0
        st = torch.zeros(B, Hh, Dd, V, device=dev)
        nbytes = Tt * (3 * Hh * Dd + Hh * V) * 2 + Tt * Hh * V * 4 + B * Hh * Dd * V * 8
        row("linear_state_scan (decay per key channel) " + label,
            _time(lambda: S.linear_state_scan(qk[:, :Hh * Dd], qk[:, Hh * Dd:], v, None, None, None, None, None, st, rs,
                                              sl, qsl, Hh, Hh, Dd, V, False, False, Dd ** -0.5, False, zk=zk,
                                              zk_bias=zb, inv_tau=1.0 / 16), iters=5),
            nbytes, flops=5.0 * Tt * Hh * Dd * V)
        dec = torch.full((Hh,), 0.99, device=dev)
        row("linear_state_scan (existing: one constant decay per head) " + label,
            _time(lambda: S.linear_state_scan(qk[:, :Hh * Dd], qk[:, Hh * Dd:], v, None, None, None, None, dec, st, rs,
                                              sl, qsl, Hh, Hh, Dd, V, True, False, 1.0, False), iters=5),
            nbytes - Tt * Hh * Dd * 2, like="linear_state_scan (decay per key channel)",
            flops=4.0 * Tt * Hh * Dd * V)

    # latent attention: norm + pair rotary + cache write, then the attention over the latent cache
    H, Dn, rot, rank, ps = 32, 128, 64, 512, 16
    for label, qlens, ctx in (("prefill 4 x 2048", [2048] * 4, 0), ("decode 256 x 1 at 2048", [1] * 256, 2047)):
        Tt, B = sum(qlens), len(qlens)
        npp = (max(qlens) + ctx + ps - 1) // ps
        bt = torch.arange(B * npp, dtype=torch.int32, device=dev).reshape(B, npp)
        cache = torch.randn(B * npp + 1, 1, (rank + rot) // 64, ps, 64, device=dev).to(bf)
        pos = torch.cat([torch.arange(ctx, ctx + q) for q in qlens]).to(torch.int32).to(dev)
        seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(dev)
        slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
        q = torch.randn(Tt, H, Dn + rot, device=dev).to(bf)
        dkv = torch.randn(Tt, rank + rot, device=dev).to(bf)
        q_full = torch.randn(Tt, H, rank + rot, device=dev).to(bf)
        nw = torch.ones(rank, device=dev).to(bf)
        fr, mag = ref.pair_rotary_frequencies(rot, 10000.0, {"factor": 4.0, "original": 2048, "fast": 32.0,
                                                             "slow": 1.0})
        fr = fr.to(dev)
        nb = Tt * (H * rot * 2 * 2 + (rank + rot) * 2 * 2)
        row("latent_norm_rope_write (latent norm + pair rotary from fp32 angles + cache write) " + label,
            _time(lambda: Lt.latent_norm_rope_write(q, dkv, rank, rot, nw, 1e-5, pos, fr, mag, q_full, cache, slots)),
            nb)
        cs = torch.randn(8192, rot, device=dev)
        kvn = torch.randn(Tt, rank, device=dev).to(bf)
        row("rmsnorm(latent) + mla_rope_cache (existing: table rotary + cache write) " + label,
            _time(lambda: (sm100.rmsnorm(dkv[:, :rank], nw, 1e-5),
                           sm100.mla_rope_cache(q[:, :, Dn:], q_full, dkv[:, rank:], kvn, cs, pos, slots, cache))),
            nb + Tt * rank * 2 * 2, like="latent_norm_rope_write")
        tok_seq = seqi.to(torch.int32)
        keys = sum(p + 1 for ql in qlens for p in range(ctx, ctx + ql))
        ms = _time(lambda: sm100.mla_attention(q_full, cache, bt, tok_seq, pos, 192 ** -0.5), iters=3)
        out.append({"kernel": "latent attention 512 + 64 (the DeepSeek tensor-core kernel itself) " + label,
                    "ms": round(ms, 4), "tflops": round(2.0 * keys * H * (2 * rank + rot) / ms / 1e9, 2)})

    # router and experts
    T2, E, top = 8192, 16, 2
    hh = torch.randn(T2, W, device=dev).to(bf)
    wr, corr = (torch.randn(E, W, device=dev) * W ** -0.5).to(bf), torch.randn(E, device=dev) * 0.1
    row("grouped_router (fp32 logits + softmax + correction + group limit + top-2) 8192 x 4096 x 16",
        _time(lambda: Lt.grouped_router(hh, wr, corr, top, 4, 2, 2.5)), T2 * W * 2 + E * W * 2)
    row("router GEMM + grouped_topk (existing)",
        _time(lambda: sm100_moe.grouped_topk(sm100.linear(hh, wr), top, True, 4, 2, "sigmoid", corr, 2.5)),
        T2 * W * 2 + E * W * 2, like="grouped_router")
    hd = hh[:64]
    row("grouped_router decode, 64 x 4096 x 16", _time(lambda: Lt.grouped_router(hd, wr, corr, top, 4, 2, 2.5)),
        E * W * 2 + 64 * W * 2)
    row("router GEMM + grouped_topk decode (existing)",
        _time(lambda: sm100_moe.grouped_topk(sm100.linear(hd, wr), top, True, 4, 2, "sigmoid", corr, 2.5)),
        E * W * 2 + 64 * W * 2, like="grouped_router decode")
    F = 2048
    n_real = E - 2
    w13 = (torch.randn(n_real, 2 * F, W, device=dev) * W ** -0.5).to(bf)
    w2 = (torch.randn(n_real, W, F, device=dev) * F ** -0.5).to(bf)
    wts, ids = Lt.grouped_router(hh, wr, corr, top, 4, 2, 2.5)
    fl = 6.0 * T2 * top * W * F * n_real / E
    row("routed_glu_experts (grouped tcgen05 GEMMs, clamped gated epilogue, 2 identity experts of 16)",
        _time(lambda: Lt.routed_glu_experts(hh, w13, w2, wts, ids, 7.0, True, 1.702, E), iters=5),
        w13.numel() * 2 + w2.numel() * 2 + T2 * W * 2 * 2, flops=fl)
    ids2 = ids % n_real
    row("fused_experts (existing: SiLU-gate epilogue, 14 experts)",
        _time(lambda: sm100_moe.fused_experts(hh, w13, w2, wts, ids2), iters=5),
        w13.numel() * 2 + w2.numel() * 2 + T2 * W * 2 * 2, like="routed_glu_experts", flops=6.0 * T2 * top * W * F)
    Fs = 4096
    wgu = (torch.randn(2 * Fs, W, device=dev) * W ** -0.5).to(bf)
    row("linear_glu_clamp (tcgen05 GEMM, clamped gated epilogue) 8192 x 4096 -> 4096",
        _time(lambda: Lt.linear_glu_clamp(hh, wgu, 7.0), iters=5), wgu.numel() * 2 + T2 * (W + Fs) * 2,
        flops=4.0 * T2 * W * Fs)
    row("linear_silu_mul (existing epilogue)", _time(lambda: sm100.linear_silu_mul(hh, wgu), iters=5),
        wgu.numel() * 2 + T2 * (W + Fs) * 2, like="linear_glu_clamp", flops=4.0 * T2 * W * Fs)
    return out


def run_bevovik(args, peaks):
    vocab = 32000
    kernels = _kernels_bevovik(peaks)
    sizes = []
    for width, quads in ((1024, 2), (2048, 2), (4096, 1)):
        b_cfg = _bevovik_cfg(width, quads, vocab)
        d_cfg = _deepseek_cfg(width, 4 * quads, vocab)
        sizes.append({"width": width, "layers": 4 * quads,
                      "bevovik": _throughput(b_cfg, vocab, args.warmup, args.steps),
                      "deepseek_v3": _throughput(d_cfg, vocab, args.warmup, args.steps)})
    line = {"design": "bevovik", "dtype": "bf16", "data": "synthetic", "warmup": args.warmup, "steps": args.steps,
            "timing": "wall clock around LLM.generate with synchronize (sizes); CUDA events, L2 flushed (kernels)",
            "peaks": peaks, "sizes": sizes, "kernels": kernels}
    print(json.dumps(line))
    return line


def _kernels_notadra(peaks):
    """Device time of the kernels this design added or extended, at layer-like sizes, each beside the like kernel of
    the existing path (Qwen3-MoE's rotary write, paged attention, router and gated experts). Bytes are the
    algorithmic minimum."""
    from gllm_b200.ops import ref, sm100, sm100_latent as Lt, sm100_moe, sm100_pair as Pr, sm100_seq as S
    dev, bf = "cuda", torch.bfloat16
    hbm = float(peaks.get("hbm_gbs", 6650.0))
    out = []

    def row(name, ms, nbytes, like=None, flops=None):
        r = {"kernel": name, "ms": round(ms, 4), "gbs": round(nbytes / ms / 1e6, 1),
             "frac_hbm": round(nbytes / ms / 1e6 / hbm, 3)}
        if flops:
            r["tflops"] = round(flops / ms / 1e9, 2)
        if like:
            r["like"] = like
        out.append(r)

    T, W, V = 8192, 4096, 32000
    ids = torch.randint(0, V, (T,), dtype=torch.int32, device=dev)
    table, pair = torch.randn(V, W, device=dev).to(bf), torch.randn(65522, W, device=dev).to(bf)
    qsl4 = torch.tensor([0, 2048, 4096, 6144, 8192], dtype=torch.int32, device=dev)
    pos4 = torch.arange(2048, dtype=torch.int32, device=dev).repeat(4)
    st = torch.zeros(8, dtype=torch.int32, device=dev)
    rs = torch.arange(4, dtype=torch.int32, device=dev)
    row("pair_embed (token row + hashed pair row -> fp32 stream) 8192 x 4096",
        _time(lambda: Pr.embedding_pair_hash(ids, table, pair, 1000003, 31, 65521, pos4, st, rs, qsl4)),
        T * W * (2 + 2 + 4))
    row("embedding (existing: one row, bf16 out)", _time(lambda: sm100.embedding(ids, table)), T * W * (2 + 2),
        like="pair_embed")
    x = torch.randn(T, W, device=dev)
    y, w1 = torch.randn(T, W, device=dev).to(bf), torch.zeros(W, device=dev).to(bf)
    row("resid_norm with gain 1 + w (post-norm + add + pre-norm, fp32 stream in/out, bf16 in/out)",
        _time(lambda: S.resid_norm(x, y, w1, None, w1, 1e-5, bf, False, None, 1.0)), T * W * (4 + 4 + 2 + 2))
    res = torch.randn(T, W, device=dev).to(bf)
    row("rmsnorm + residual (existing bf16 path)", _time(lambda: sm100.rmsnorm(y, w1, 1e-5, res)),
        T * W * (2 + 2 + 2 + 2), like="resid_norm")
    H, G, D, ps = 32, 8, 128, 16
    fr, mag = ref.pair_rotary_frequencies(64, 1e6, {"factor": 4.0, "original": 2048, "fast": 32.0, "slow": 1.0},
                                          dtype=torch.float64)
    fr = fr.to(dev)
    sink = torch.zeros(H, device=dev)
    for label, qlens, ctx in (("prefill 4 x 2048", [2048] * 4, 0), ("decode 256 x 1 at 2048", [1] * 256, 2047)):
        Tt, B = sum(qlens), len(qlens)
        qsl = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), dtype=torch.int32, device=dev)
        sl = torch.tensor([q + ctx for q in qlens], dtype=torch.int32, device=dev)
        npp = (max(qlens) + ctx + ps - 1) // ps
        bt = torch.arange(B * npp, dtype=torch.int32, device=dev).reshape(B, npp)
        kshape = ref.kv_cache_shape(B * npp + 1, G, D, ps)
        kc, vc = torch.randn(kshape, device=dev).to(bf), torch.randn(kshape, device=dev).to(bf)
        pos = torch.cat([torch.arange(ctx, ctx + q) for q in qlens]).to(torch.int32).to(dev)
        seqi = torch.cat([torch.full((q,), i) for i, q in enumerate(qlens)]).to(dev)
        slots = (bt[seqi, (pos // ps).long()] * ps + pos % ps).to(torch.int32)
        qkv = torch.randn(Tt, (H + 2 * G) * D, device=dev).to(bf)
        ms = _time(lambda: S.qk_norm_rope_kv_write(qkv, H, G, D, D, None, None, 1e-5, pos, 64, 1e6, kc, vc, slots, fr,
                                                   mag))
        row("rotary write (frequency table, first 64 of 128 entries, cache write) " + label, ms,
            Tt * (H + 2 * G) * D * 2 * 2)
        ms = _time(lambda: S.qk_norm_rope_kv_write(qkv[:, :H * D], H, 0, D, D, None, None, 1e-5, pos, 64, 1e6, kc, vc,
                                                   slots, fr, mag))
        row("rotary write, queries only (layer on shared pages) " + label, ms, Tt * H * D * 2 * 2)
        cs = torch.randn(8192, D, device=dev)
        qq = qkv[:, :H * D].unflatten(1, (H, D))
        kk = qkv[:, H * D:(H + G) * D].unflatten(1, (G, D))
        vv = qkv[:, (H + G) * D:].unflatten(1, (G, D))
        ms2 = _time(lambda: sm100.rope_kv_write(qq, kk, vv, pos, cs, D, True, None, None, 1e-5, kc, vc, slots))
        row("rope_kv_write (existing: table rotary + cache write) " + label, ms2, Tt * (H + 2 * G) * D * 2 * 2,
            like="rotary write")
        q = torch.randn(Tt, H * D, device=dev).to(bf)
        keys = sum(p + 1 for ql in qlens for p in range(ctx, ctx + ql))
        nd = B if qlens[0] == 1 else 0
        ms = _time(lambda: S.window_attention(q, kc, vc, bt, sl, qsl, pos, D ** -0.5, H, D, None, sink,
                                              num_decode_seqs=nd, max_q_len=max(qlens), v_dim=D, softcap=50.0),
                   iters=5)
        r = {"kernel": "capped sink attention (tcgen05 prefill kernel for portions, tensor-core paged kernel for "
                       "decode rows) " + label, "ms": round(ms, 4),
             "tflops": round(4.0 * keys * H * D / ms / 1e9, 2)}
        ms2 = _time(lambda: sm100.paged_attention(q, kc, vc, bt, sl, qsl, D ** -0.5, H, D, nd, B, max(qlens),
                                                  max(qlens) + ctx), iters=3)
        r["like"] = {"kernel": "paged_attention (existing, no cap, no sink)", "ms": round(ms2, 4),
                     "tflops": round(4.0 * keys * H * D / ms2 / 1e9, 2)}
        out.append(r)
    T2, E, top = 8192, 16, 2
    hh = torch.randn(T2, W, device=dev).to(bf)
    wr, corr = (torch.randn(E, W, device=dev) * W ** -0.5).to(bf), torch.randn(E, device=dev) * 0.1
    row("grouped_router (fp32 logits + sigmoid + correction + top-2-sum group limit + top-2) 8192 x 4096 x 16",
        _time(lambda: Lt.grouped_router(hh, wr, corr, top, 4, 2, 1.0, "sigmoid", 2, False)), T2 * W * 2 + E * W * 2)
    row("router GEMM + topk_softmax (existing)",
        _time(lambda: sm100_moe.topk_softmax(sm100.linear(hh, wr), top, True)), T2 * W * 2 + E * W * 2,
        like="grouped_router")
    hd = hh[:64]
    row("grouped_router decode, 64 x 4096 x 16",
        _time(lambda: Lt.grouped_router(hd, wr, corr, top, 4, 2, 1.0, "sigmoid", 2, False)), E * W * 2 + 64 * W * 2)
    row("router GEMM + topk_softmax decode (existing)",
        _time(lambda: sm100_moe.topk_softmax(sm100.linear(hd, wr), top, True)), E * W * 2 + 64 * W * 2,
        like="grouped_router decode")
    F = 3072
    wu = (torch.randn(E, F, W, device=dev) * W ** -0.5).to(bf)
    wd = (torch.randn(E, W, F, device=dev) * F ** -0.5).to(bf)
    wts, idx = Lt.grouped_router(hh, wr, corr, top, 4, 2, 1.0, "sigmoid", 2, False)
    row("routed_relu2_experts (grouped tcgen05 GEMMs, squared-ReLU epilogue, ff 3072)",
        _time(lambda: Pr.routed_relu2_experts(hh, wu, wd, wts, idx, True), iters=5),
        wu.numel() * 2 + wd.numel() * 2 + T2 * W * 2 * 2, flops=4.0 * T2 * top * W * F)
    Fg = 2048
    w13 = (torch.randn(E, 2 * Fg, W, device=dev) * W ** -0.5).to(bf)
    w2 = (torch.randn(E, W, Fg, device=dev) * Fg ** -0.5).to(bf)
    row("fused_experts (existing: SiLU-gate epilogue, ff 2048: the same weights' size)",
        _time(lambda: sm100_moe.fused_experts(hh, w13, w2, wts, idx), iters=5),
        w13.numel() * 2 + w2.numel() * 2 + T2 * W * 2 * 2, like="routed_relu2_experts",
        flops=6.0 * T2 * top * W * Fg)
    hd64 = hh[:64]
    wt64, id64 = wts[:64].contiguous(), idx[:64].contiguous()
    row("routed_relu2_experts decode, 64 tokens", _time(lambda: Pr.routed_relu2_experts(hd64, wu, wd, wt64, id64, True)),
        wu.numel() * 2 + wd.numel() * 2, flops=4.0 * 64 * top * W * F)
    row("fused_experts decode, 64 tokens (existing)", _time(lambda: sm100_moe.fused_experts(hd64, w13, w2, wt64, id64)),
        w13.numel() * 2 + w2.numel() * 2, like="routed_relu2_experts decode", flops=6.0 * 64 * top * W * Fg)
    return out


def run_notadra(args, peaks):
    vocab = 32000
    kernels = _kernels_notadra(peaks)
    sizes = []
    for width, layers in ((1024, 8), (2048, 8), (4096, 4)):
        n_cfg = _notadra_cfg(width, layers, vocab)
        q_cfg = _qwen3_moe_cfg(width, layers, vocab)
        sizes.append({"width": width, "layers": layers,
                      "notadra": _throughput(n_cfg, vocab, args.warmup, args.steps),
                      "qwen3_moe": _throughput(q_cfg, vocab, args.warmup, args.steps)})
    line = {"design": "notadra", "dtype": "bf16", "data": "synthetic", "warmup": args.warmup, "steps": args.steps,
            "timing": "wall clock around LLM.generate with synchronize (sizes); CUDA events, L2 flushed (kernels)",
            "peaks": peaks, "sizes": sizes, "kernels": kernels}
    print(json.dumps(line))
    return line
