"""Helpers of the Bevovik tests: small random checkpoints on disk, the replay session, comparisons."""
import json
import os

import numpy as np
import torch

import bevovik_oracle as oracle
from conftest import scratch_dir

YARN = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}


def rglru(width=24, blocks=3, conv=3, mlp=None):
    return {"type": "rglru", "mixer": {"blocks": blocks, "conv": conv, "width": width}, "mlp": mlp}


def gla(heads=2, dim=6, vdim=10, tau=8.0, mlp=None):
    return {"type": "gla", "mixer": {"dim": dim, "heads": heads, "tau": tau, "vdim": vdim}, "mlp": mlp}


def latent(heads=3, dim=8, rot_dim=4, vdim=6, q_rank=10, kv_rank=12, base=100.0, scale=0.4, scaling=YARN, mlp=None):
    rot = {"base": base, "dims": rot_dim}
    if scaling is not None:
        rot["scaling"] = dict(scaling)
    return {"type": "latent_attention",
            "mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "q_rank": q_rank, "rot": rot, "rot_dim": rot_dim,
                      "scale": scale, "vdim": vdim},
            "mlp": mlp}


def moe(experts=6, identity=2, top=2, ff=8, limit=1.5, groups=(2, 1), scale=1.5, shared=(12, 0.8)):
    r = {"experts": experts, "identity": identity, "scale": scale, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": r}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def make_config(layers, vocab=61, width=20, eps=1e-5):
    return {"architecture": "Bevovik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


def random_weights(cfg, seed=0, low_rank=5):
    """name -> bf16-representable fp32 tensor, in checkpoint naming. `low_rank`: rows of a gla mixer's a1 (a size
    that only the tensor's shape gives)."""
    g = torch.Generator().manual_seed(seed)
    w = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).bfloat16().float()

    wd, v = cfg["width"], cfg["vocab"]
    w["embed"] = rnd(v, wd, std=1.0)
    w["head"] = rnd(v, wd, std=3.0 * wd ** -0.5)
    w["final.norm"] = 1 + rnd(wd, std=0.2)

    def lin(name, out, inp, gain=1.0):
        w[name] = rnd(out, inp, std=gain * inp ** -0.5)

    def expert(p, ff):
        lin(p + "gate", ff, wd, 2.0)
        lin(p + "up", ff, wd, 2.0)
        lin(p + "down", wd, ff, 2.0)

    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        w[p + "norm1"] = 1 + rnd(wd, std=0.2)
        w[p + "ls1"] = 0.6 + rnd(wd, std=0.3)
        q = p + "mix."
        if L["type"] == "rglru":
            c, nb, taps = m["width"], m["blocks"], m["conv"]
            lin(q + "y", c, wd, 2.0)
            w[q + "y.b"] = rnd(c, std=0.3)
            lin(q + "x", c, wd, 2.0)
            w[q + "x.b"] = rnd(c, std=0.3)
            w[q + "conv"] = rnd(c, taps, std=0.6)
            w[q + "conv.b"] = rnd(c, std=0.3)
            bw = c // nb
            for n in ("ra", "ri"):
                w[q + n] = rnd(nb, bw, bw, std=2.0 * bw ** -0.5)
                w[q + n + ".b"] = rnd(nb, bw, std=0.5)
            w[q + "lam"] = rnd(c, std=1.5) - 2.0
            lin(q + "o", wd, c, 2.0)
        elif L["type"] == "gla":
            h, d, dv = m["heads"], m["dim"], m["vdim"]
            lin(q + "q", h * d, wd, 2.0)
            lin(q + "k", h * d, wd, 2.0)
            lin(q + "v", h * dv, wd, 2.0)
            lin(q + "g", h * dv, wd, 2.0)
            lin(q + "o", wd, h * dv, 2.0)
            w[q + "norm"] = 1 + rnd(dv, std=0.3)
            lin(q + "a1", low_rank, wd, 2.0)
            lin(q + "a2", h * d, low_rank, 2.0)
            w[q + "a2.b"] = rnd(h * d, std=1.0) + 2.0
        else:
            h, d, dr, dv, qr, kr = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["q_rank"], m["kv_rank"]
            lin(q + "dq", qr, wd, 2.0)
            w[q + "dq.norm"] = 1 + rnd(qr, std=0.3)
            lin(q + "uq", h * (d + dr), qr, 2.0)
            lin(q + "dkv", kr + dr, wd, 2.0)
            w[q + "dkv.norm"] = 1 + rnd(kr, std=0.3)
            lin(q + "uk", h * d, kr, 2.0)
            lin(q + "uv", h * dv, kr, 2.0)
            lin(q + "o", wd, h * dv, 2.0)
        mlp = L["mlp"]
        if mlp:
            r = mlp["router"]
            w[p + "norm2"] = 1 + rnd(wd, std=0.2)
            w[p + "ls2"] = 0.6 + rnd(wd, std=0.3)
            n_out = r["experts"] + r.get("identity", 0)
            lin(p + "mlp.router", n_out, wd, 4.0)
            w[p + "mlp.correction"] = rnd(n_out, std=0.1)
            for e in range(r["experts"]):
                expert("%smlp.e%d." % (p, e), mlp["expert"]["ff"])
            if mlp.get("shared"):
                expert(p + "mlp.shared.", mlp["shared"]["ff"])
    return {k: t.bfloat16().float() for k, t in w.items()}     # exactly what the bf16 checkpoint holds


def save_model(cfg, weights):
    from safetensors.torch import save_file
    d = scratch_dir("bevovik_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def session(path, dtype="float32", device="cpu", max_tokens=256, page_size=4, state_slots=4):
    from gllm_b200.entrypoints.trace_run import TraceSession
    return TraceSession(path, dtype, max_tokens, device, page_size, state_slots)


def expected_logits(cfg, weights, tokens):
    return oracle.forward(cfg, weights, tokens, torch.float64).float().numpy()


def row_errs(got, want):
    """per row: root mean square of the difference over the vocabulary (means removed) / rms of the expected row"""
    d = got - want
    d = d - d.mean(-1, keepdims=True)
    w = want - want.mean(-1, keepdims=True)
    return np.sqrt((d ** 2).mean(-1)) / (np.sqrt((w ** 2).mean(-1)) + 1e-9)


def rel_err(got, want):
    return float(row_errs(got, want).max())


def run_chunks(sess, rid, tokens, cuts):
    """Feed `tokens` of request `rid` alone in portions of the sizes `cuts` (the rest one by one); all logits."""
    outs, at = [], 0
    sizes = list(cuts)
    while at < len(tokens):
        n = min(sizes.pop(0) if sizes else 1, len(tokens) - at)
        end = [rid] if at + n == len(tokens) else []
        outs.append(sess.step([{"id": rid, "tokens": tokens[at:at + n], "want": list(range(n))}], end))
        at += n
    return np.concatenate(outs, 0)


def run_plan(sess, reqs, plan):
    """plan: steps of [(request, n tokens)]; -> {request: logits of all its tokens}"""
    at = {k: 0 for k in reqs}
    got = {k: [] for k in reqs}
    for step in plan:
        entries, end = [], []
        for k, n in step:
            entries.append({"id": k, "tokens": reqs[k][at[k]:at[k] + n], "want": list(range(n))})
            at[k] += n
            if at[k] == len(reqs[k]):
                end.append(k)
        out = sess.step(entries, end)
        o = 0
        for k, n in step:
            got[k].append(out[o:o + n])
            o += n
    assert all(at[k] == len(reqs[k]) for k in reqs)
    return {k: np.concatenate(v, 0) for k, v in got.items()}


class DictReader:
    """The two reader calls that a mixer's `load` makes, over a dict of tensors."""

    def __init__(self, w):
        self.w = w

    def get(self, name):
        return self.w[name]

    def shape(self, name):
        return tuple(self.w[name].shape)


def drive_mixer(m, h, cuts, page_size=4, device="cpu", dtype=torch.float32, pool=512):
    """One mixer alone through the page / slot managers and the batch builder: `h` [T, width] fed in portions of the
    sizes `cuts`; -> the mixer's outputs [T, width] (fp32, CPU)."""
    from gllm_b200.input_data import InputData, build_batch
    from gllm_b200.memory_manager import HybridCache, MemoryManager
    from gllm_b200.scheduler import ScheduledSeq
    from gllm_b200.sequence import Sequence
    n = h.shape[0]
    mm = MemoryManager(pool // page_size, page_size, num_state_slots=2)
    cache = HybridCache([m.cache_entry()], pool // page_size, page_size, 2, dtype, device)
    inp = InputData(max(pool, 64), 4, pool // page_size, device)
    inp.need_tok_seq = bool(getattr(m, "needs_tok_seq", False))
    seq = Sequence(0, list(range(n)), [])
    assert mm.acquire_state(seq)
    got, at = [], 0
    for c in cuts:
        seq.scheduled_token_num = at + c
        mm.pre_allocate_page([seq])
        inp.load(build_batch([ScheduledSeq(seq, at, c)], page_size, 100))
        got.append(m(inp, h[at:at + c].to(device=device, dtype=dtype), cache, 0).float().cpu())
        at += c
    assert at == n
    return torch.cat(got)
