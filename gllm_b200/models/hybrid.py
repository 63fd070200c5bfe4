"""Layer-list decoder: a stack whose every layer names its own mixer and an optional feed-forward, over an fp32
residual stream. Two block forms: sandwich norms around each sublayer with an optional loop that re-runs a span of
layers with shared weights (architecture `Saritar`: windowed sink attention and Mamba-1 mixers, squared-ReLU
feed-forward), and norm-after-sum blocks (architecture `Femolix`: gated delta rule mixers and parallel mixers of
chunk-masked rotary attention beside constant-decay linear attention, gated SiLU feed-forward, dense or routed, capped
logits), and branch-norm blocks with a layer scale (architecture `Bevovik`: real-gated linear recurrent units,
key-decay gated linear attention and latent attention with YaRN rotary, a grouped mixture of clamped gated experts
with identity experts and a shared expert); and sandwich blocks whose norm weights are stored around zero (architecture
`Notadra`: rotary attention with biased projections, YaRN-scaled partial rotation, capped scores, a unit sink in the
softmax denominator, values of their own width and layers that read an earlier layer's keys and values; a
sigmoid-scored, group-limited mixture of ungated squared-ReLU experts; a hashed embedding of the (previous, current)
token pair added to the token embedding; logits scaled through the final norm):

    x = embed[token]
    per layer:  x += ls1 * rms(mixer(x)) * n1 ;  x += ls2 * rms(ff(x)) * n2            (sublayers read x itself)
    logits = head @ (rms(x) * final_norm)

The norm-after-sum form:

    x = embed[token]
    per layer:  x <- rms(alpha x + mixer(x)) * n1 ;  x <- rms(alpha x + ff(x)) * n2     (second line only with a ff)
    logits = cap * tanh(head @ (rms(x) * final_norm) / cap)

The sandwich form:

    x = embed[token] * embed_scale                                   (fp32 from here on)
    per layer:  x += rms(mixer(rms(x) * n1)) * n1b ;  x += rms(ff(rms(x) * n2)) * n2b   (second line only with a ff)
    loop (start, stop, times): layers start..stop-1 run `times` times back to back; every pass has its own cache
        entries ("layer runs"), and before each pass but the first the embedding output is added to x
    logits = head @ (rms(x) * final_norm)

Dataflow on the device: every residual update is ONE kernel that applies the post-norm, adds into the fp32 stream,
optionally adds the embedding (loop re-entry) and emits the next sublayer's pre-normed input in the compute dtype
(`Fn.resid_norm`), so the stream is read and written once per sublayer.

In the norm-after-sum form one kernel per sublayer (`Fn.postnorm`) scales the stream, adds the sublayer's output,
norms, writes the stream back and emits it in the compute dtype for the next sublayer.

In the branch-norm form one kernel per sublayer (`Fn.resid_norm` with a layer scale) norms the branch, adds it into
the stream and emits the stream in the compute dtype for the next sublayer (the stream itself in fp32).

Notadra (the sandwich form with gains 1 + w):

    x = embed[token] + pair[(previous token * mul_prev + token * mul_cur) mod buckets]   (row `buckets` at position 0)
    per layer:  x += rms(mixer(rms(x) (1 + n1))) (1 + n1b) ;  x += rms(ff(rms(x) (1 + n2))) (1 + n2b)
    logits = head @ (logit_scale * rms(x) (1 + final_norm))

config.json keys read here: architecture, vocab, width, embedding.scale, embedding.bigram.{buckets, mul_prev,
mul_cur}, logit_scale, layers[i].mixer.{kv_from, softcap, rot.scaling.{factor, original, fast, slow}},
norm.eps, loop.{start,stop,times},
postln_alpha, logit_softcap, layers[i].{type, mixer{...}, mlp{kind, ff | expert.{ff, limit}, router.{experts, top,
identity, scale, groups.{count, keep}}, shared.{ff, limit}} | null}, optional torch_dtype. Tensor names: embed, bigram,
head, l<i>.mix.{q,k,v}.b, l<i>.mlp.e<j>.{up,down}, final.norm, l<i>.norm1|norm1b|norm2|norm2b|ls1|ls2, l<i>.mix.*, l<i>.mlp.up|down|gate|router|correction|
e<j>.{gate,up,down}|shared.{gate,up,down}.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Callable, List, Optional

import torch
from torch import nn

from gllm_b200.layers import functional as Fn
from gllm_b200.layers.latent_attention import LatentAttention
from gllm_b200.layers.linear_attention import DecayLinearCore, GatedDeltaCore, KeyDecayLinearCore
from gllm_b200.layers.moe import GroupedGLUMoE, GroupedRelu2MoE, SelectedSoftmaxMoE
from gllm_b200.layers.parallel_mixer import CoreMixer
from gllm_b200.layers.ssm import Mamba1Mixer, RGLRUMixer
from gllm_b200.layers.window_attention import RotaryChunkCore, SinkWindowAttention
from gllm_b200.parallel import state as ps

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32, torch.bfloat16: torch.bfloat16,
           torch.float32: torch.float32}


@dataclass
class HybridSpec:
    arch: str
    hidden_size: int
    vocab_size: int
    rms_eps: float
    embed_scale: float
    layers: List[dict]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1
    dtype: torch.dtype = torch.bfloat16
    # "sandwich": x += post(f(pre(x))) | "postnorm": x <- norm(alpha x + f(x)) | "branchnorm": x += ls * post(f(x))
    block: str = "sandwich"
    resid_alpha: float = 1.0
    logit_softcap: float = 0.0         # 0: none
    # "relu2": down(relu(up h)^2) | "silu_gate": down(silu(gate h) * up h) | "glu_clamp": clamped gate and up,
    # down(g sigmoid(1.702 g) (u + 1))
    ff_act: str = "relu2"
    norm_offset: float = 0.0           # added to every norm weight in fp32 (1.0: weights stored around zero)
    logit_scale: float = 1.0
    # {"buckets", "mul_prev", "mul_cur"}: a second embedding table indexed by a hash of the (previous, current) pair
    pair_hash: Optional[dict] = None
    eos_token_id: Optional[object] = None
    use_mla: bool = False
    quant: Optional[str] = None
    extra: dict = field(default_factory=dict)

    @property
    def num_layers(self) -> int:
        return len(self.layers)


def spec_saritar(cfg) -> HybridSpec:
    loop = cfg.get("loop") or {}
    dt = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    if dt not in _DTYPES:
        raise ValueError(f"unsupported dtype {dt} for this architecture (bfloat16 | float32)")
    return HybridSpec(arch="saritar", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
                      rms_eps=float(cfg["norm"]["eps"]), embed_scale=float((cfg.get("embedding") or {}).get("scale", 1.0)),
                      layers=[dict(x) for x in cfg["layers"]], loop_start=int(loop.get("start", 0)),
                      loop_stop=int(loop.get("stop", 0)), loop_times=int(loop.get("times", 1)), dtype=_DTYPES[dt],
                      eos_token_id=cfg.get("eos_token_id"))


def spec_femolix(cfg) -> HybridSpec:
    dt = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    if dt not in _DTYPES:
        raise ValueError(f"unsupported dtype {dt} for this architecture (bfloat16 | float32)")
    return HybridSpec(arch="femolix", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
                      rms_eps=float(cfg["norm"]["eps"]), embed_scale=1.0, layers=[dict(x) for x in cfg["layers"]],
                      dtype=_DTYPES[dt], block="postnorm", resid_alpha=float(cfg.get("postln_alpha", 1.0)),
                      logit_softcap=float(cfg.get("logit_softcap") or 0.0), ff_act="silu_gate",
                      eos_token_id=cfg.get("eos_token_id"))


def spec_bevovik(cfg) -> HybridSpec:
    dt = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    if dt not in _DTYPES:
        raise ValueError(f"unsupported dtype {dt} for this architecture (bfloat16 | float32)")
    return HybridSpec(arch="bevovik", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
                      rms_eps=float(cfg["norm"]["eps"]), embed_scale=1.0, layers=[dict(x) for x in cfg["layers"]],
                      dtype=_DTYPES[dt], block="branchnorm", ff_act="glu_clamp", eos_token_id=cfg.get("eos_token_id"))


def spec_notadra(cfg) -> HybridSpec:
    dt = cfg.get("torch_dtype", cfg.get("dtype", "bfloat16"))
    if dt not in _DTYPES:
        raise ValueError(f"unsupported dtype {dt} for this architecture (bfloat16 | float32)")
    bg = (cfg.get("embedding") or {}).get("bigram")
    pair = {k: int(bg[k]) for k in ("buckets", "mul_prev", "mul_cur")} if bg else None
    return HybridSpec(arch="notadra", hidden_size=int(cfg["width"]), vocab_size=int(cfg["vocab"]),
                      rms_eps=float(cfg["norm"]["eps"]), embed_scale=1.0, layers=[dict(x) for x in cfg["layers"]],
                      dtype=_DTYPES[dt], block="sandwich", ff_act="relu2", norm_offset=1.0,
                      logit_scale=float(cfg.get("logit_scale", 1.0)), pair_hash=pair,
                      eos_token_id=cfg.get("eos_token_id"))


def layer_runs(n_layers: int, start: int, stop: int, times: int):
    """[(layer index, add_embed)] in execution order; add_embed marks the first layer of every pass but the first."""
    if times <= 1 or stop <= start:
        return [(i, False) for i in range(n_layers)]
    runs = [(i, False) for i in range(start)]
    for r in range(times):
        runs += [(i, r > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n_layers)]


class Relu2MLP(nn.Module):
    """down(relu(up(h))^2)"""

    def __init__(self, hidden: int, ff: int, dtype, device):
        super().__init__()
        self.up_w = nn.Parameter(torch.zeros(ff, hidden, dtype=dtype, device=device), requires_grad=False)
        self.down_w = nn.Parameter(torch.zeros(hidden, ff, dtype=dtype, device=device), requires_grad=False)

    def forward(self, h):
        return Fn.linear_any(Fn.relu2(Fn.linear_any(h, self.up_w)), self.down_w)


def make_mixer(kind: str, m: dict, spec: HybridSpec, device):
    h, dt = spec.hidden_size, spec.dtype
    if kind == "attention" and spec.arch == "notadra":
        rot = m.get("rot") or {}
        src = m.get("kv_from")
        core = RotaryChunkCore(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]),
                               int(m.get("vdim", m["dim"])), float(m["scale"]), int(rot.get("dims", 0)),
                               float(rot.get("base", 10000.0)), None, None, spec.rms_eps, dt, device, qk_norm=False,
                               rot_scaling=rot.get("scaling"), softcap=float(m.get("softcap") or 0.0), unit_sink=True,
                               bias=True, kv_from=int(src) if src is not None else None)
        return CoreMixer(h, [core], [""], [1.0], dt, device)
    if kind == "attention":
        assert int(m.get("vdim", m["dim"])) == int(m["dim"]), "values are the keys: vdim must equal dim"
        window = (m.get("mask") or {}).get("size")
        return SinkWindowAttention(h, int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), float(m["scale"]),
                                   int(window) if window is not None else None, spec.rms_eps, dt, device)
    if kind == "mamba1":
        return Mamba1Mixer(h, int(m["inner"]), int(m["state"]), int(m["dt_rank"]), int(m["conv"]), dt, device)
    if kind == "delta":
        core = GatedDeltaCore(int(m["heads"]), int(m.get("kv_heads", m["heads"])), int(m["dim"]),
                              int(m.get("vdim", m["dim"])), int(m.get("conv", 1)), spec.rms_eps, dt, device)
        return CoreMixer(h, [core], [""], [1.0], dt, device)
    if kind == "parallel":
        l, r = m["left"], m["right"]
        rot, mask = l.get("rot") or {}, l.get("mask") or {}
        left = RotaryChunkCore(int(l["heads"]), int(l.get("kv_heads", l["heads"])), int(l["dim"]),
                               int(l.get("vdim", l["dim"])), float(l["scale"]), int(rot.get("dims", 0)),
                               float(rot.get("base", 10000.0)), int(mask["size"]) if mask.get("size") else None, None,
                               spec.rms_eps, dt, device)
        right = DecayLinearCore(int(r["heads"]), int(r["dim"]), int(r.get("vdim", r["dim"])), list(r["decay"]),
                                spec.rms_eps, dt, device)
        return CoreMixer(h, [left, right], ["left", "right"], [float(m.get("left_scale", 1.0)),
                                                               float(m.get("right_scale", 1.0))], dt, device)
    if kind == "gla":
        a1 = m.get("low_rank")
        core = KeyDecayLinearCore(int(m["heads"]), int(m["dim"]), int(m.get("vdim", m["dim"])),
                                  int(a1) if a1 is not None else 16, float(m["tau"]), spec.rms_eps, dt, device)
        return CoreMixer(h, [core], [""], [1.0], dt, device)
    if kind == "rglru":
        return RGLRUMixer(h, int(m["width"]), int(m["blocks"]), int(m["conv"]), dt, device)
    if kind == "latent_attention":
        rot = m.get("rot") or {}
        rd = int(m.get("rot_dim", rot.get("dims", 0)))
        assert int(rot.get("dims", rd)) == rd, "the rotated part is rotated whole"
        return LatentAttention(h, int(m["heads"]), int(m["dim"]), rd, int(m.get("vdim", m["dim"])), int(m["q_rank"]),
                               int(m["kv_rank"]), float(m["scale"]), float(rot.get("base", 10000.0)),
                               rot.get("scaling"), spec.rms_eps, dt, device)
    raise ValueError(f"unknown mixer type {kind!r}")


class GatedMLP(nn.Module):
    """down(silu(gate h) * (up h)); gate and up rows share one GEMM. On CUDA in bf16 with ff % 128 == 0 the rows are
    stored interleaved per 128 and the product is the tcgen05 GEMM's SiLU-gate epilogue (one kernel)."""

    def __init__(self, hidden: int, ff: int, dtype, device):
        super().__init__()
        self.ff = ff
        self.fused = torch.device(device).type == "cuda" and dtype == torch.bfloat16 and ff % 128 == 0 and \
            hidden % 8 == 0
        self.gate_up_w = nn.Parameter(torch.zeros(2 * ff, hidden, dtype=dtype, device=device), requires_grad=False)
        self.down_w = nn.Parameter(torch.zeros(hidden, ff, dtype=dtype, device=device), requires_grad=False)

    def load(self, gate, up, down):
        from gllm_b200.ops import ref
        gu = torch.cat([gate, up], 0)
        self.gate_up_w.data.copy_(ref.interleave_gate_up(gu, 128) if self.fused else gu)
        self.down_w.data.copy_(down)

    def forward(self, h):
        if self.fused:
            return Fn.linear_any(Fn.linear_silu_mul(h, self.gate_up_w), self.down_w)
        return Fn.linear_any(Fn.silu_mul(Fn.linear_any(h, self.gate_up_w)), self.down_w)


def make_ff(mlp: dict, spec: HybridSpec, device):
    h, dt = spec.hidden_size, spec.dtype
    kind = mlp.get("kind", "dense")
    if kind == "dense":
        return (GatedMLP if spec.ff_act == "silu_gate" else Relu2MLP)(h, int(mlp["ff"]), dt, device)
    if kind == "moe" and spec.ff_act == "relu2":
        r = mlp["router"]
        groups = r.get("groups") or {}
        count = int(groups.get("count", 1))
        return GroupedRelu2MoE(int(r["experts"]), int(r["top"]), h, int(mlp["expert"]["ff"]), count,
                               int(groups.get("keep", count)), dt, device, group_top=2, renorm=False)
    if kind == "moe" and spec.ff_act == "silu_gate":
        return SelectedSoftmaxMoE(int(mlp["router"]["experts"]), int(mlp["router"]["top"]), h,
                                  int(mlp["expert"]["ff"]), dt, device)
    if kind == "moe" and spec.ff_act == "glu_clamp":
        r, e, sh = mlp["router"], mlp["expert"], mlp.get("shared") or {}
        groups = r.get("groups") or {}
        return GroupedGLUMoE(int(r["experts"]), int(r.get("identity", 0)), int(r["top"]), h, int(e["ff"]),
                             float(e["limit"]), int(groups.get("count", 1)), int(groups.get("keep", 1)),
                             float(r.get("scale", 1.0)), dt, device, shared_ff=int(sh.get("ff", 0)),
                             shared_limit=float(sh.get("limit", 0.0)))
    raise ValueError(f"unknown feed-forward kind {kind!r}")


class HybridLayer(nn.Module):
    def __init__(self, spec: HybridSpec, layer_id: int, device):
        super().__init__()
        L = spec.layers[layer_id]
        h, dt = spec.hidden_size, spec.dtype

        def norm():
            return nn.Parameter(torch.ones(h, dtype=dt, device=device), requires_grad=False)

        self.layer_id = layer_id
        self.kind = L["type"]
        sandwich = spec.block == "sandwich"
        scaled = spec.block == "branchnorm"          # a layer scale per sublayer, fp32

        def scale():
            return nn.Parameter(torch.ones(h, dtype=torch.float32, device=device), requires_grad=False)

        self.norm1_w, self.norm1b_w = norm(), (norm() if sandwich else None)
        self.ls1 = scale() if scaled else None
        self.mixer = make_mixer(L["type"], L["mixer"], spec, device)
        mlp = L.get("mlp")
        if mlp is not None:
            self.norm2_w, self.norm2b_w = norm(), (norm() if sandwich else None)
            self.ls2 = scale() if scaled else None
            self.mlp = make_ff(mlp, spec, device)
        else:
            self.mlp = None


class HybridLM(nn.Module):
    ret_residual = False
    is_hybrid = True

    def __init__(self, spec: HybridSpec, device="cpu"):
        super().__init__()
        assert ps.get_world_size() == 1, "layer-list decoders run on one GPU (no TP / PP sharding yet)"
        assert spec.logit_scale == 1.0 or spec.block == "sandwich", \
            "the logit scale rides on the sandwich form's final norm"
        self.spec = spec
        self.device = torch.device(device)
        h, dt = spec.hidden_size, spec.dtype
        self.embed_w = nn.Parameter(torch.zeros(spec.vocab_size, h, dtype=dt, device=device), requires_grad=False)
        self.pair_w = nn.Parameter(torch.zeros(spec.pair_hash["buckets"] + 1, h, dtype=dt, device=device),
                                   requires_grad=False) if spec.pair_hash else None
        self.layers = nn.ModuleList([HybridLayer(spec, i, device) for i in range(spec.num_layers)])
        self.final_norm_w = nn.Parameter(torch.ones(h, dtype=dt, device=device), requires_grad=False)
        self.lm_head_w = nn.Parameter(torch.zeros(spec.vocab_size, h, dtype=dt, device=device), requires_grad=False)
        self.runs = layer_runs(spec.num_layers, spec.loop_start, spec.loop_stop, spec.loop_times)
        # the pair embedding keeps every sequence's last token in its state slot
        self.has_state = any(getattr(l.mixer, "uses_state", not l.mixer.uses_pages) for l in self.layers) or \
            spec.pair_hash is not None
        self.has_pages = any(l.mixer.uses_pages for l in self.layers)
        self.needs_tok_seq = any(getattr(l.mixer, "needs_tok_seq", False) for l in self.layers)
        self.trace: Optional[list] = None     # debugging: when a list, the stream after every layer run is appended

    # -- what the runner asks ---------------------------------------------------------------------
    @property
    def num_layers(self): return len(self.runs)

    @property
    def hidden_size(self): return self.spec.hidden_size

    def cache_layout(self):
        """One entry per layer RUN (a looped layer has one per pass). A mixer that reads another layer's pages
        ({"kind": "shared", "layer": j}) is resolved to that layer's latest run before it ("source": run index);
        with a pair embedding one more entry {"kind": "tokens"} follows the runs (the carried previous token)."""
        out, last_run = [], {}
        for r, (i, _) in enumerate(self.runs):
            e = self.layers[i].mixer.cache_entry()
            if e["kind"] == "shared":
                j = e["layer"]
                assert j in last_run, f"layer {i} reads the keys and values of layer {j}, which has not run before it"
                src = out[last_run[j]]
                assert src["kind"] == "kv", f"layer {j} keeps no keys and values of its own"
                m, ms = self.layers[i].mixer.cores[0], self.layers[j].mixer.cores[0]
                assert (m.kv_heads, m.dim, m.v_dim) == (ms.kv_heads, ms.dim, ms.v_dim), "shared pages: sizes differ"
                e = {"kind": "shared", "source": last_run[j]}
            out.append(e)
            last_run[i] = r
        if self.spec.pair_hash is not None:
            out.append({"kind": "tokens"})
        return out

    # -- forward ----------------------------------------------------------------------------------
    def forward(self, inp, cache, tpc=None, hidden=None, residual=None, **_):
        spec, eps, dt = self.spec, self.spec.rms_eps, self.spec.dtype
        if spec.block == "postnorm":
            return self._forward_postnorm(inp, cache), None
        if spec.block == "branchnorm":
            return self._forward_branchnorm(inp, cache), None
        off = spec.norm_offset
        if spec.pair_hash is not None:
            ph = spec.pair_hash
            x0 = Fn.embedding_pair_hash(inp, self.embed_w, self.pair_w, ph["mul_prev"], ph["mul_cur"], ph["buckets"],
                                        cache.token_state if cache is not None else None)
        else:
            x0 = Fn.embedding_scaled(inp.tokens, self.embed_w, spec.embed_scale)
        x = x0.clone() if any(a for _, a in self.runs) else x0
        n = len(self.runs)
        # the logit scale rides on the final norm (applied in fp32 before the head's input is rounded)
        h = Fn.resid_norm(x, None, None, None, self.layers[self.runs[0][0]].norm1_w if n else self.final_norm_w,
                          eps, dt, False, None, off, 1.0 if n else spec.logit_scale)
        for r, (li, _) in enumerate(self.runs):
            L = self.layers[li]
            y = L.mixer(inp, h, cache, r)
            post = L.norm1b_w
            if L.mlp is not None:
                h = Fn.resid_norm(x, y, post, None, L.norm2_w, eps, dt, False, None, off)
                y = L.mlp(h)
                post = L.norm2b_w
            last = r + 1 == n
            w_pre = self.final_norm_w if last else self.layers[self.runs[r + 1][0]].norm1_w
            add = x0 if (not last and self.runs[r + 1][1]) else None
            mul = spec.logit_scale if last else 1.0
            if self.trace is not None:
                Fn.resid_norm(x, y, post, None, None, eps, dt, False, None, off)
                self.trace.append(x.clone())
                h = Fn.resid_norm(x, None, None, add, w_pre, eps, dt, False, None, off, mul)
            else:
                h = Fn.resid_norm(x, y, post, add, w_pre, eps, dt, False, None, off, mul)
        return h, None

    def _forward_postnorm(self, inp, cache):
        spec, eps, dt, alpha = self.spec, self.spec.rms_eps, self.spec.dtype, self.spec.resid_alpha
        x = Fn.embedding_scaled(inp.tokens, self.embed_w, spec.embed_scale)
        h = x if dt == torch.float32 else x.to(dt)       # exact: the table holds compute-dtype values
        for r, (li, _) in enumerate(self.runs):
            L = self.layers[li]
            h = Fn.postnorm(x, L.mixer(inp, h, cache, r), alpha, L.norm1_w, eps, dt)
            if L.mlp is not None:
                h = Fn.postnorm(x, L.mlp(h), alpha, L.norm2_w, eps, dt)
            if self.trace is not None:
                self.trace.append(x.clone())
        return Fn.resid_norm(x, None, None, None, self.final_norm_w, eps, dt)

    def _forward_branchnorm(self, inp, cache):
        """x += ls * rms(f(x)) * n per sublayer; f reads the stream itself (rounded to the compute dtype). The last
        sublayer's update also applies the final norm."""
        spec, eps, dt = self.spec, self.spec.rms_eps, self.spec.dtype
        x = Fn.embedding_scaled(inp.tokens, self.embed_w, spec.embed_scale)
        n = len(self.runs)
        if n == 0:
            return Fn.resid_norm(x, None, None, None, self.final_norm_w, eps, dt)
        h = x if dt == torch.float32 else x.to(dt)       # exact: the table holds compute-dtype values
        for r, (li, _) in enumerate(self.runs):
            L = self.layers[li]
            last = r + 1 == n and self.trace is None
            y = L.mixer(inp, h, cache, r)
            if L.mlp is not None:
                h = Fn.resid_norm(x, y, L.norm1_w, None, None, eps, dt, True, L.ls1)
                y = L.mlp(h)
                w_post, ls = L.norm2_w, L.ls2
            else:
                w_post, ls = L.norm1_w, L.ls1
            h = Fn.resid_norm(x, y, w_post, None, self.final_norm_w if last else None, eps, dt, not last, ls)
            if self.trace is not None:
                self.trace.append(x.clone())
        if self.trace is not None:
            h = Fn.resid_norm(x, None, None, None, self.final_norm_w, eps, dt)
        return h

    def compute_logits(self, inp, hidden, tpc=None, all_rows: bool = False, local: bool = False):
        rows = hidden if all_rows else hidden.index_select(0, inp.logits_idx.long())
        z = Fn.linear_any(rows, self.lm_head_w)
        return Fn.softcap(z, self.spec.logit_softcap) if self.spec.logit_softcap > 0 else z

    # -- weights ----------------------------------------------------------------------------------
    def process_weights(self):
        """After the weights are final and before any CUDA-graph capture: workspaces whose addresses captured graphs
        keep (the split-KV partials of the tensor-core latent attention)."""
        if self.device.type == "cuda" and self.spec.dtype == torch.bfloat16:
            for L in self.layers:
                m = L.mixer
                if isinstance(m, LatentAttention) and m.kv_rank == 512 and m.rot_dim == 64:
                    from gllm_b200.ops import sm100
                    sm100._mla_workspace(self.device, m.heads)

    def init_dummy(self, seed: int = 0):
        g = torch.Generator(device="cpu").manual_seed(seed)

        def rnd(p, std):
            p.data.copy_((torch.randn(p.shape, generator=g) * std).to(p.dtype))

        for name, p in self.named_parameters():
            if name.endswith("norm_w") or "norm1" in name or "norm2" in name:
                p.data.fill_(1.0 - self.spec.norm_offset)
            elif name.endswith("in_b") or name.endswith("correction"):
                rnd(p, 0.1)
            elif name.endswith(".a"):
                p.data.copy_(-torch.exp(torch.rand(p.shape, generator=g) * 2.0 - 1.0))
            elif name.endswith("dt_b"):
                p.data.copy_(torch.rand(p.shape, generator=g) * 2.0 - 3.0)
            elif name.endswith("d_skip"):
                p.data.fill_(1.0)
            elif name.endswith("neg_a"):
                p.data.copy_(-torch.exp(torch.rand(p.shape, generator=g) * 2.0 - 1.0))
            elif name.endswith("dt_bias"):
                p.data.copy_(torch.rand(p.shape, generator=g) * 2.0 - 3.0)
            elif name.endswith("conv_b") and "cores" in name:
                p.data.zero_()
            elif name.endswith("sink") or name.endswith("conv_b"):
                rnd(p, 0.5)
            elif name.endswith("conv_w"):
                rnd(p, 0.4)
            elif p.dim() >= 2:
                rnd(p, 1.0 / max(p.shape[-1], 1) ** 0.5)
            else:
                rnd(p, 0.02)

    def load_weights(self, reader, progress: Optional[Callable[[int, int], None]] = None):
        total = len(self.layers) + 2

        def put(param, t):
            assert tuple(param.shape) == tuple(t.shape), (tuple(param.shape), tuple(t.shape))
            param.data.copy_(t)

        put(self.embed_w, reader.get("embed"))
        if self.pair_w is not None:
            put(self.pair_w, reader.get("bigram"))
        for n, L in enumerate(self.layers):
            pre = f"l{L.layer_id}."
            put(L.norm1_w, reader.get(pre + "norm1"))
            if L.norm1b_w is not None:
                put(L.norm1b_w, reader.get(pre + "norm1b"))
            m = L.mixer
            mp = pre + "mix."
            if isinstance(m, SinkWindowAttention):
                put(m.qk_w, torch.cat([reader.get(mp + "q"), reader.get(mp + "k")], 0))
                if m.q_norm_w is not None:
                    put(m.q_norm_w, reader.get(mp + "q.norm"))
                    put(m.k_norm_w, reader.get(mp + "k.norm"))
                if m.sink is not None:
                    put(m.sink, reader.get(mp + "sink").float())
                put(m.o_w, reader.get(mp + "o"))
            elif isinstance(m, Mamba1Mixer):
                put(m.in_w, reader.get(mp + "in"))
                put(m.conv_w, reader.get(mp + "conv").float())
                put(m.conv_b, reader.get(mp + "conv.b").float())
                put(m.x_w, reader.get(mp + "x"))
                put(m.dt_w, reader.get(mp + "dt"))
                put(m.dt_b, reader.get(mp + "dt.b").float())
                put(m.a, -torch.exp(reader.get(mp + "A_log").float()))
                put(m.d_skip, reader.get(mp + "D").float())
                put(m.o_w, reader.get(mp + "o"))
            elif isinstance(m, CoreMixer):
                m.load(reader, mp, put)
            elif isinstance(m, (RGLRUMixer, LatentAttention)):
                m.load(reader, mp, put)
            if L.ls1 is not None:
                put(L.ls1, reader.get(pre + "ls1").float())
            if L.mlp is not None:
                put(L.norm2_w, reader.get(pre + "norm2"))
                if L.norm2b_w is not None:
                    put(L.norm2b_w, reader.get(pre + "norm2b"))
                f = L.mlp
                if L.ls2 is not None:
                    put(L.ls2, reader.get(pre + "ls2").float())
                if isinstance(f, GroupedRelu2MoE):
                    put(f.router_w, reader.get(pre + "mlp.router"))
                    if f.correction is not None:
                        put(f.correction, reader.get(pre + "mlp.correction").float())
                    for e in range(f.num_experts):
                        f.load_expert(e, reader.get(f"{pre}mlp.e{e}.up"), reader.get(f"{pre}mlp.e{e}.down"))
                elif isinstance(f, GroupedGLUMoE):
                    put(f.router_w, reader.get(pre + "mlp.router"))
                    put(f.correction, reader.get(pre + "mlp.correction").float())
                    for e in range(f.num_experts):
                        ep = f"{pre}mlp.e{e}."
                        f.load_expert(e, reader.get(ep + "gate"), reader.get(ep + "up"), reader.get(ep + "down"))
                    if f.shared is not None:
                        sp = pre + "mlp.shared."
                        f.shared.load(reader.get(sp + "gate"), reader.get(sp + "up"), reader.get(sp + "down"))
                elif isinstance(f, SelectedSoftmaxMoE):
                    put(f.router_w, reader.get(pre + "mlp.router"))
                    for e in range(f.num_experts):
                        ep = f"{pre}mlp.e{e}."
                        f.load_expert(e, reader.get(ep + "gate"), reader.get(ep + "up"), reader.get(ep + "down"))
                elif isinstance(f, GatedMLP):
                    f.load(reader.get(pre + "mlp.gate"), reader.get(pre + "mlp.up"), reader.get(pre + "mlp.down"))
                else:
                    put(f.up_w, reader.get(pre + "mlp.up"))
                    put(f.down_w, reader.get(pre + "mlp.down"))
            if progress is not None:
                progress(n + 2, total)
        put(self.final_norm_w, reader.get("final.norm"))
        put(self.lm_head_w, reader.get("head"))
        if progress is not None:
            progress(total, total)


def build_saritar(cfg, device):
    return HybridLM(spec_saritar(cfg), device)


def build_femolix(cfg, device):
    return HybridLM(spec_femolix(cfg), device)


def build_bevovik(cfg, device):
    return HybridLM(spec_bevovik(cfg), device)


def build_notadra(cfg, device):
    return HybridLM(spec_notadra(cfg), device)
