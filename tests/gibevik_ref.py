"""Plain, slow restatement of the Gibevik decoder, one function per mechanism, written from its equations and sharing
no code with the product path.  Whole sequences at once, any float dtype (the tests use float64).  Test oracle only.

Notation: n tokens at positions 0 .. n-1, stream x [n, width]; a linear weight W is stored [out, in] and applied as
x @ W.T.  unit(z) = z / sqrt(mean(z^2) + eps) over the last axis."""
from __future__ import annotations

import math

import torch


def unit(z, eps):
    return z / torch.sqrt((z * z).mean(-1, keepdim=True) + eps)


def norm(z, w, eps):
    return unit(z, eps) * w


def position_vector(n, width, dtype, base=10000.0):
    """[n, width]: entry 2i = sin(p base^(-2i / width)), entry 2i + 1 = cos of the same angle."""
    out = torch.zeros(n, width, dtype=dtype)
    for p in range(n):
        for i in range(width // 2):
            a = p * base ** (-2.0 * i / width)
            out[p, 2 * i], out[p, 2 * i + 1] = math.sin(a), math.cos(a)
    return out


def head_slope(h, heads):
    return 2.0 ** (-8.0 * (h + 1) / heads)


def query_temperature(p, coef, every):
    return 1.0 + coef * math.log((p + 1) // every + 1)


def causal_softmax_rows(scores):
    """scores [n, n] (row = query position i, column = key position j): softmax over j <= i, zero elsewhere."""
    n = scores.shape[0]
    out = torch.zeros_like(scores)
    for i in range(n):
        s = scores[i, :i + 1]
        e = torch.exp(s - s.max())
        out[i, :i + 1] = e / e.sum()
    return out


def biased_attention(h, w, p, m, eps):
    """Grouped-head softmax attention whose values are the projected keys: per-head q / k norm with a shared weight,
    query temperature, distance bias, gate per output element."""
    n = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).reshape(n, H, D)
    k = (h @ w[p + "k"].T).reshape(n, G, D)
    v = k                                               # the raw rows: the key norm below does not touch them
    qn = norm(q, w[p + "q.norm"], eps)
    kn = norm(k, w[p + "k.norm"], eps)
    qt = m.get("q_temp")
    if qt:
        for i in range(n):
            qn[i] = qn[i] * query_temperature(i, qt["coef"], qt["every"])
    dist = torch.tensor([[float(i - j) for j in range(n)] for i in range(n)], dtype=h.dtype)
    heads = []
    for hh in range(H):
        g = hh // (H // G)
        s = (qn[:, hh] @ kn[:, g].T) * m["scale"] - head_slope(hh, H) * dist
        heads.append(causal_softmax_rows(s) @ v[:, g])
    out = torch.cat(heads, -1) * torch.sigmoid(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


def latent_of(h, w, p, eps):
    """The normed latent a latent-attention layer caches."""
    return norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)


def latent_attention(h, c, w, p, m):
    """Attention whose keys and values are expanded from the latent c [n, kv_rank]; gate per head."""
    n = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(n, H, D)
    k = (c @ w[p + "uk"].T).reshape(n, H, D)
    v = (c @ w[p + "uv"].T).reshape(n, H, Dv)
    gate = torch.sigmoid(h @ w[p + "g"].T)              # [n, H]
    heads = []
    for hh in range(H):
        s = (q[:, hh] @ k[:, hh].T) * m["scale"]
        heads.append(causal_softmax_rows(s) @ v[:, hh] * gate[:, hh:hh + 1])
    return torch.cat(heads, -1) @ w[p + "o"].T


def dense_ff(h, w, p):
    g = h @ w[p + "gate"].T
    return (g * torch.sigmoid(g) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def relu2_ff(h, w, p):
    return (torch.relu(h @ w[p + "up"].T) ** 2) @ w[p + "down"].T


def route(z, correction, top, groups, keep):
    """z [E] router logits of one token -> (chosen indices, their weights).  Choice by softmax + correction among the
    members of the `keep` groups with the largest best member; weights are the plain softmax values."""
    s = torch.softmax(z, -1)
    choice = s + correction if correction is not None else s.clone()
    E = z.shape[0]
    allowed = [True] * E
    if groups:
        per = E // groups
        best = [max(choice[g * per:(g + 1) * per].tolist()) for g in range(groups)]
        order = sorted(range(groups), key=lambda g: (-best[g], g))[:keep]
        allowed = [(e // per) in order for e in range(E)]
    cand = sorted([e for e in range(E) if allowed[e]], key=lambda e: (-choice[e].item(), e))[:top]
    return cand, [s[e] for e in cand]


def moe_ff(h, w, p, mlp):
    r = mlp["router"]
    E, ident = r["experts"], r.get("identity", 0)
    groups = r.get("groups") or {}
    z = h @ w[p + "router"].T
    corr = w.get(p + "correction")
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        idx, wt = route(z[t], corr, r["top"], groups.get("count", 0), groups.get("keep", 0))
        for e, a in zip(idx, wt):
            out[t] += a * (h[t] if e >= E else relu2_ff(h[t:t + 1], w, f"{p}e{e}.")[0])
    if mlp.get("shared"):
        y = relu2_ff(h, w, p + "shared.")
        if p + "shared.sg" in w:
            y = y * torch.sigmoid(h @ w[p + "shared.sg"].T)
        out = out + y
    return out


def forward(cfg, tensors, tokens, dtype=torch.float64, trace=None):
    """Logits [n, vocab] of one sequence; trace (a list) receives the stream after every layer."""
    w = {k: v.to(dtype) for k, v in tensors.items()}
    eps, n = cfg["norm"]["eps"], len(tokens)
    x = w["embed"][torch.tensor(tokens)] + position_vector(n, cfg["width"], dtype)
    latents = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "attention":
            y = biased_attention(x, w, p, m, eps)
        else:
            src = m.get("kv_from")
            if src is None:
                latents[i] = latent_of(x, w, p, eps)
                src = i
            y = latent_attention(x, latents[src], w, p, m)
        x = x + norm(y, w[f"l{i}.norm1"], eps)
        mlp = layer.get("mlp")
        if mlp:
            y = dense_ff(x, w, f"l{i}.mlp.") if mlp["kind"] == "dense" else moe_ff(x, w, f"l{i}.mlp.", mlp)
            x = x + norm(y, w[f"l{i}.norm2"], eps)
        if trace is not None:
            trace.append(x.clone())
    return norm(x, w["final.norm"], eps) @ w["head"].T
