"""Helpers of the Notadra tests: small configurations, random checkpoints on disk, comparisons. The replay session and
the portion / plan drivers are the ones the other layer-list designs' tests use."""
import json
import os

import torch

import notadra_oracle as oracle
from bevovik_util import DictReader, rel_err, row_errs, run_chunks, run_plan, session  # noqa: F401
from conftest import scratch_dir

YARN = {"factor": 4.0, "original": 16, "fast": 8.0, "slow": 1.0}


def attn(heads=4, kv_heads=2, dim=8, vdim=6, rot_dims=4, base=100.0, scaling=YARN, scale=0.4, softcap=5.0,
         kv_from=None, mlp=None):
    rot = {"base": base, "dims": rot_dims}
    if scaling is not None:
        rot["scaling"] = dict(scaling)
    m = {"dim": dim, "heads": heads, "kv_heads": kv_heads, "rot": rot, "scale": scale, "softcap": softcap,
         "vdim": vdim}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def moe(experts=6, top=2, ff=8, groups=(3, 2)):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def make_config(layers, vocab=61, width=20, eps=1e-5, bigram=(23, 31, 5), logit_scale=0.7):
    cfg = {"architecture": "Notadra", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers,
           "logit_scale": logit_scale}
    if bigram is not None:
        cfg["embedding"] = {"bigram": {"buckets": bigram[0], "mul_prev": bigram[1], "mul_cur": bigram[2]}}
    return cfg


def random_weights(cfg, seed=0):
    """name -> bf16-representable fp32 tensor, in checkpoint naming."""
    g = torch.Generator().manual_seed(seed)
    w = {}

    def rnd(*shape, std=1.0):
        return (torch.randn(*shape, generator=g) * std).bfloat16().float()

    wd, v = cfg["width"], cfg["vocab"]
    w["embed"] = rnd(v, wd)
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        w["bigram"] = rnd(bg["buckets"] + 1, wd)
    w["head"] = rnd(v, wd, std=3.0 * wd ** -0.5)
    w["final.norm"] = rnd(wd, std=0.2)

    def lin(name, out, inp, gain=1.0):
        w[name] = rnd(out, inp, std=gain * inp ** -0.5)

    for i, L in enumerate(cfg["layers"]):
        p, m = "l%d." % i, L["mixer"]
        for n in ("norm1", "norm1b"):
            w[p + n] = rnd(wd, std=0.3)
        h, g_, d, dv = m["heads"], m["kv_heads"], m["dim"], m.get("vdim", m["dim"])
        q = p + "mix."
        lin(q + "q", h * d, wd, 2.0)
        w[q + "q.b"] = rnd(h * d, std=0.5)
        if m.get("kv_from") is None:
            lin(q + "k", g_ * d, wd, 2.0)
            w[q + "k.b"] = rnd(g_ * d, std=0.5)
            lin(q + "v", g_ * dv, wd, 2.0)
            w[q + "v.b"] = rnd(g_ * dv, std=0.5)
        lin(q + "o", wd, h * dv, 2.0)
        mlp = L["mlp"]
        if mlp:
            r = mlp["router"]
            for n in ("norm2", "norm2b"):
                w[p + n] = rnd(wd, std=0.3)
            lin(p + "mlp.router", r["experts"], wd, 4.0)
            w[p + "mlp.correction"] = rnd(r["experts"], std=0.3)
            for e in range(r["experts"]):
                lin("%smlp.e%d.up" % (p, e), mlp["expert"]["ff"], wd, 2.0)
                lin("%smlp.e%d.down" % (p, e), wd, mlp["expert"]["ff"], 2.0)
    return {k: t.bfloat16().float() for k, t in w.items()}     # exactly what the bf16 checkpoint holds


def save_model(cfg, weights):
    from safetensors.torch import save_file
    d = scratch_dir("notadra_")
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.bfloat16().contiguous() for k, v in weights.items()}, os.path.join(d, "model.safetensors"))
    return d


def expected_logits(cfg, weights, tokens):
    return oracle.forward(cfg, weights, tokens).float().numpy()


def build_mixer(layer_cfg, w, width, device="cpu", dtype=torch.float32, eps=1e-5, pre="l0.mix."):
    from gllm_b200.models.hybrid import HybridSpec, make_mixer
    spec = HybridSpec("notadra", width, 61, eps, 1.0, [layer_cfg], dtype=dtype, block="sandwich", ff_act="relu2",
                      norm_offset=1.0)
    m = make_mixer(layer_cfg["type"], dict(layer_cfg["mixer"]), spec, device)

    def put(p, t):
        assert tuple(p.shape) == tuple(t.shape)
        p.data.copy_(t)

    m.load(DictReader(w), pre, put)
    return m


def build_ff(mlp_cfg, w, width, device="cpu", dtype=torch.float32, pre="l0.mlp."):
    from gllm_b200.models.hybrid import HybridSpec, make_ff
    spec = HybridSpec("notadra", width, 61, 1e-5, 1.0, [], dtype=dtype, block="sandwich", ff_act="relu2",
                      norm_offset=1.0)
    f = make_ff(mlp_cfg, spec, device)
    f.router_w.data.copy_(w[pre + "router"])
    f.correction.data.copy_(w[pre + "correction"].float())
    for e in range(f.num_experts):
        f.load_expert(e, w["%se%d.up" % (pre, e)].to(device), w["%se%d.down" % (pre, e)].to(device))
    return f


def drive_mixers(mixers, layout, hs, cuts, page_size=4, device="cpu", dtype=torch.float32, pool=512):
    """Mixers that share one cache (layout: one entry per mixer, "shared" entries name their source) through the
    page / slot managers and the batch builder: mixer i reads hs[i] [T, width], fed in portions of the sizes `cuts`;
    -> their outputs [T, width] (fp32, CPU)."""
    from gllm_b200.input_data import InputData, build_batch
    from gllm_b200.memory_manager import HybridCache, MemoryManager
    from gllm_b200.scheduler import ScheduledSeq
    from gllm_b200.sequence import Sequence
    n = hs[0].shape[0]
    mm = MemoryManager(pool // page_size, page_size, num_state_slots=2)
    cache = HybridCache(layout, pool // page_size, page_size, 2, dtype, device)
    inp = InputData(max(pool, 64), 4, pool // page_size, device)
    seq = Sequence(0, list(range(n)), [])
    assert mm.acquire_state(seq)
    got, at = [[] for _ in mixers], 0
    for c in cuts:
        seq.scheduled_token_num = at + c
        mm.pre_allocate_page([seq])
        inp.load(build_batch([ScheduledSeq(seq, at, c)], page_size, 100))
        for i, m in enumerate(mixers):
            got[i].append(m(inp, hs[i][at:at + c].to(device=device, dtype=dtype), cache, i).float().cpu())
        at += c
    assert at == n
    return [torch.cat(g) for g in got]


def oracle_mixer(h, layer_cfg, w, pre="l0.mix.", kv=None):
    """One attention mixer of the oracle on h [T, width] (float64); `kv`: keys and values of another layer."""
    wd = {k: v.double() for k, v in w.items()}
    m = layer_cfg["mixer"]
    if kv is None:
        kv = oracle.keys_values(h, m, wd, pre)
    return oracle.attention(h, m, wd, pre, kv)
