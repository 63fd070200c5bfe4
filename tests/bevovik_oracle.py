"""Plain, slow restatement of the Bevovik design: one function per mechanism, whole sequences, no cache, no batching.
Shares no code with gllm_b200. `w` maps checkpoint names to tensors; `cfg` is the parsed config.json.

    block:    x <- x + ls1 * (rms(mixer(x)) * n1);  x <- x + ls2 * (rms(ff(x)) * n2)     (norm on the branch only)
    gla:      gated linear attention, one decay per key channel, S <- diag(a) S + k v^T, o = S^T q
    latent_attention:  queries and keys / values through low-rank latents, a shared rotated key part, YaRN rotary
    rglru:    gelu branch times a real-gated linear recurrent unit behind a short causal convolution
    ff:       grouped top-k mixture with a correction on the choice, identity experts, clamped gated experts, shared
    logits:   head . (rms(x) * final_norm)
"""
import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


# -- gated linear attention -----------------------------------------------------------------------------------
def gla_mixer(h, w, p, m, eps):
    t = h.shape[0]
    nh, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w[p + "q"].T).reshape(t, nh, d) * d ** -0.5
    k = (h @ w[p + "k"].T).reshape(t, nh, d)
    v = (h @ w[p + "v"].T).reshape(t, nh, dv)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).reshape(t, nh, d)
    gate = silu(h @ w[p + "g"].T).reshape(t, nh, dv)
    out = h.new_zeros(t, nh, dv)
    for hd in range(nh):
        s = h.new_zeros(d, dv)
        for i in range(t):
            s = alpha[i, hd][:, None] * s + torch.outer(k[i, hd], v[i, hd])
            out[i, hd] = s.T @ q[i, hd]
    out = rms(out, eps) * w[p + "norm"] * gate
    return out.reshape(t, nh * dv) @ w[p + "o"].T


# -- rotary with YaRN scaling ---------------------------------------------------------------------------------
def yarn_frequencies(dims, base, scaling, dtype=torch.float64):
    """-> (frequency per pair [dims / 2], factor applied to cos and sin)"""
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def where(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(where(float(scaling["fast"]))), 0)
    hi = min(math.ceil(where(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, pos, dims, base, scaling):
    """x [T, ..., D]: the first `dims` entries rotate, entry 2i pairs with entry 2i + 1."""
    f, mag = yarn_frequencies(dims, base, scaling, x.dtype)
    ang = pos.to(x.dtype)[:, None] * f[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(ang) * mag).reshape(shape), (torch.sin(ang) * mag).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# -- latent attention -------------------------------------------------------------------------------------------
def latent_attention_mixer(h, w, p, m, eps):
    t = h.shape[0]
    nh, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    rot = m["rot"]
    pos = torch.arange(t)
    cq = rms(h @ w[p + "dq"].T, eps) * w[p + "dq.norm"]
    q = (cq @ w[p + "uq"].T).reshape(t, nh, d + dr)
    ckr = h @ w[p + "dkv"].T
    c = rms(ckr[:, :rank], eps) * w[p + "dkv.norm"]
    kr = rotate_pairs(ckr[:, rank:], pos, rot["dims"], rot["base"], rot.get("scaling"))          # [T, dr]
    qr = rotate_pairs(q[..., d:], pos, rot["dims"], rot["base"], rot.get("scaling"))             # [T, H, dr]
    kn = (c @ w[p + "uk"].T).reshape(t, nh, d)
    v = (c @ w[p + "uv"].T).reshape(t, nh, dv)
    s = (torch.einsum("ihd,jhd->hij", q[..., :d], kn) + torch.einsum("ihd,jd->hij", qr, kr)) * float(m["scale"])
    mask = pos[:, None] >= pos[None, :]
    s = s.masked_fill(~mask[None], float("-inf"))
    a = torch.softmax(s, -1)
    o = torch.einsum("hij,jhd->ihd", a, v).reshape(t, nh * dv)
    return o @ w[p + "o"].T


# -- recurrent block with a real-gated linear recurrent unit ---------------------------------------------------
def short_conv(x, w, b):
    """x [T, C], w [C, taps], b [C]; output t = b + sum_j w[:, j] * x[t - (taps - 1) + j], zeros before the start."""
    t, c = x.shape
    taps = w.shape[1]
    xp = torch.cat([x.new_zeros(taps - 1, c), x], 0)
    acc = b.expand(t, c).clone()
    for j in range(taps):
        acc = acc + xp[j:j + t] * w[:, j]
    return acc


def rglru_mixer(h, w, p, m, eps):
    t = h.shape[0]
    width, nb = m["width"], m["blocks"]
    bw = width // nb
    y = gelu_tanh(h @ w[p + "y"].T + w[p + "y.b"])
    u = short_conv(h @ w[p + "x"].T + w[p + "x.b"], w[p + "conv"], w[p + "conv.b"])
    ub = u.reshape(t, nb, bw)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ra"]) + w[p + "ra.b"]).reshape(t, width)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "ri"]) + w[p + "ri.b"]).reshape(t, width)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "lam"])
    a = torch.exp(log_a)
    mult = torch.sqrt(1.0 - a * a)
    s = h.new_zeros(width)
    out = h.new_zeros(t, width)
    for n in range(t):
        s = a[n] * s + mult[n] * i[n] * u[n]
        out[n] = s
    return (out * y) @ w[p + "o"].T


# -- feed-forward --------------------------------------------------------------------------------------------------
def clamped_expert(h, gate, up, down, limit):
    g = (h @ gate.T).clamp(max=limit)
    u = (h @ up.T).clamp(-limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, w, p, r):
    """-> (ids [T, top], weights [T, top]); ids >= experts name identity experts."""
    n, top = r["experts"] + r.get("identity", 0), r["top"]
    s = torch.softmax(h @ w[p + "router"].T, -1)
    choice = s + w[p + "correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    gc, keep = groups["count"], groups["keep"]
    per = n // gc
    best = choice.reshape(-1, gc, per).max(-1).values
    kept = best.topk(keep, -1).indices
    allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True).repeat_interleave(per, 1)
    ids = choice.masked_fill(~allowed, float("-inf")).topk(top, -1).indices
    sel = s.gather(1, ids)
    return ids, sel / (sel.sum(-1, keepdim=True) + 1e-20) * float(r["scale"])


def moe_ff(h, w, p, mlp):
    r, e = mlp["router"], mlp["expert"]
    ids, wt = route(h, w, p, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for j in range(ids.shape[1]):
            x = int(ids[t, j])
            if x >= r["experts"]:
                out[t] += wt[t, j] * h[t]
            else:
                q = "%se%d." % (p, x)
                out[t] += wt[t, j] * clamped_expert(h[t:t + 1], w[q + "gate"], w[q + "up"], w[q + "down"],
                                                    float(e["limit"]))[0]
    sh = mlp.get("shared")
    if sh:
        out = out + clamped_expert(h, w[p + "shared.gate"], w[p + "shared.up"], w[p + "shared.down"],
                                   float(sh["limit"]))
    return out


# -- the model -------------------------------------------------------------------------------------------------------
MIXERS = {"gla": gla_mixer, "latent_attention": latent_attention_mixer, "rglru": rglru_mixer}


def forward(cfg, w, tokens, dtype=torch.float64, stream=None):
    """tokens: list of ids -> logits [T, vocab]; `stream`, when a list, receives the residual after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        p = "l%d." % i
        y = MIXERS[L["type"]](x, w, p + "mix.", L["mixer"], eps)
        x = x + rms(y, eps) * w[p + "norm1"] * w[p + "ls1"]
        if L.get("mlp"):
            y = moe_ff(x, w, p + "mlp.", L["mlp"])
            x = x + rms(y, eps) * w[p + "norm2"] * w[p + "ls2"]
        if stream is not None:
            stream.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T
