"""Plain, slow Notadra: one function per mechanism, whole sequences only, float64 throughout, no cache. The tests
compare the framework with it; it shares no code with the product path.

`cfg` is the parsed config.json, `wt` a dict name -> tensor (any float type; int tables excepted)."""
import math

import torch

F64 = torch.float64


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm(x, w, eps):
    """The stored weight lies around zero: the gain is 1 + w."""
    return rms(x, eps) * (1.0 + w.to(F64))


def embed(tokens, wt, cfg):
    """Token row plus a hashed row of the (previous, current) pair; a sequence's first token takes the table's
    last row."""
    x = wt["embed"].to(F64)[tokens]
    bg = (cfg.get("embedding") or {}).get("bigram")
    if bg:
        n, a, b = int(bg["buckets"]), int(bg["mul_prev"]), int(bg["mul_cur"])
        rows = [n if i == 0 else (tokens[i - 1] * a + tokens[i] * b) % n for i in range(len(tokens))]
        x = x + wt["bigram"].to(F64)[rows]
    return x


def rotary_table(rot, n_pos):
    """-> cos, sin [n_pos, dims / 2] with the YaRN frequency blend and magnitude."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    mag = 1.0
    sc = rot.get("scaling")
    if sc:
        factor, orig = float(sc["factor"]), float(sc["original"])

        def at(turns):
            return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

        lo = max(math.floor(at(float(sc["fast"]))), 0)
        hi = min(math.ceil(at(float(sc["slow"]))), dims - 1)
        for i in range(half):
            ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
            f[i] = f[i] / factor * ramp + f[i] * (1.0 - ramp)
        mag = 0.1 * math.log(factor) + 1.0
    ang = torch.arange(n_pos, dtype=F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]
    return torch.cos(ang) * mag, torch.sin(ang) * mag


def rotate(x, cos, sin):
    """x [T, heads, dim]; entry i pairs with i + dims / 2 for i < dims / 2; the rest of the head passes."""
    half = cos.shape[1]
    if half == 0:
        return x
    u, v, rest = x[..., :half], x[..., half:2 * half], x[..., 2 * half:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s, rest], -1)


def keys_values(h, m, wt, pre):
    """Rotated keys [T, G, dim] and values [T, G, vdim] of a layer that projects its own."""
    t = h.shape[0]
    g, d, dv = int(m["kv_heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    k = (h @ wt[pre + "k"].to(F64).T + wt[pre + "k.b"].to(F64)).reshape(t, g, d)
    v = (h @ wt[pre + "v"].to(F64).T + wt[pre + "v.b"].to(F64)).reshape(t, g, dv)
    rot = m.get("rot")
    if rot and int(rot.get("dims", 0)) > 0:
        k = rotate(k, *rotary_table(rot, t))
    return k, v


def attention(h, m, wt, pre, kv):
    """Causal grouped-query attention with capped scores and one extra unit term in the softmax denominator."""
    t = h.shape[0]
    nh, g, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m.get("vdim", m["dim"]))
    q = (h @ wt[pre + "q"].to(F64).T + wt[pre + "q.b"].to(F64)).reshape(t, nh, d)
    rot = m.get("rot")
    if rot and int(rot.get("dims", 0)) > 0:
        q = rotate(q, *rotary_table(rot, t))
    k, v = kv
    out = torch.zeros(t, nh, dv, dtype=F64)
    cap = float(m.get("softcap") or 0.0)
    for a in range(nh):
        b = a // (nh // g)
        s = (q[:, a] @ k[:, b].T) * float(m["scale"])
        if cap > 0:
            s = cap * torch.tanh(s / cap)
        s = s.masked_fill(torch.triu(torch.ones(t, t, dtype=torch.bool), 1), float("-inf"))
        e = torch.exp(s)
        p = e / (1.0 + e.sum(-1, keepdim=True))
        out[:, a] = p @ v[:, b]
    return out.reshape(t, nh * dv) @ wt[pre + "o"].to(F64).T


def route(h, r, wt, pre):
    """-> (ids [T, top], weights [T, top]); sigmoid scores, correction for the choice only, best groups by the sum
    of their two largest choice scores, weights the plain scores."""
    n, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ wt[pre + "router"].to(F64).T)
    choice = s + wt[pre + "correction"].to(F64) if (pre + "correction") in wt else s.clone()
    groups = r.get("groups") or {}
    cnt, keep = int(groups.get("count", 1)), int(groups.get("keep", groups.get("count", 1)))
    ids, ws = [], []
    for t in range(h.shape[0]):
        c = choice[t].clone()
        if cnt > 1:
            per = n // cnt
            gs = []
            for gi in range(cnt):
                part = sorted(c[gi * per:(gi + 1) * per].tolist(), reverse=True)
                gs.append(sum(part[:2]))
            best = sorted(range(cnt), key=lambda gi: (-gs[gi], gi))[:keep]
            for gi in range(cnt):
                if gi not in best:
                    c[gi * per:(gi + 1) * per] = float("-inf")
        pick = sorted(range(n), key=lambda e: (-float(c[e]), e))[:top]
        ids.append(pick)
        ws.append([float(s[t, e]) for e in pick])
    return ids, ws


def moe(h, mlp, wt, pre):
    ids, ws = route(h, mlp["router"], wt, pre)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], ws[t]):
            a = torch.relu(wt[f"{pre}e{e}.up"].to(F64) @ h[t])
            out[t] += w * (wt[f"{pre}e{e}.down"].to(F64) @ (a * a))
    return out


def forward(cfg, wt, tokens, trace=None):
    """-> logits [T, vocab] float64; `trace` (a list) receives the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = embed(list(tokens), wt, cfg)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        assert layer["type"] == "attention", layer["type"]
        m, pre = layer["mixer"], f"l{i}."
        h = norm(x, wt[pre + "norm1"], eps)
        src = m.get("kv_from")
        if src is None:
            kept[i] = keys_values(h, m, wt, pre + "mix.")
            src = i
        x = x + norm(attention(h, m, wt, pre + "mix.", kept[int(src)]), wt[pre + "norm1b"], eps)
        if layer.get("mlp") is not None:
            assert layer["mlp"].get("kind", "moe") == "moe"
            h = norm(x, wt[pre + "norm2"], eps)
            x = x + norm(moe(h, layer["mlp"], wt, pre + "mlp."), wt[pre + "norm2b"], eps)
        if trace is not None:
            trace.append(x.clone())
    return (norm(x, wt["final.norm"], eps) @ wt["head"].to(F64).T) * float(cfg.get("logit_scale", 1.0))
