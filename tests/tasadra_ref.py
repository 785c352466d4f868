"""A plain, slow restatement of the Tasadra decoder in double precision, one function per mechanism.  It shares no code
with the product path (vllm_rs_b200/models/tasadra.py arranges weights for CUDA kernels; this file multiplies them out
on the CPU) and is what the GPU tests compare the framework with.

Notation: T tokens at positions 0 .. T-1, stream x [T, D].  Layer i:
    h  = shift(N1(x));            x <- x + m * mixer(h)
    x <- x + m * ff(N2(x))                                   (where the layer has a feed-forward)
    X_(i+1) = x;                  x <- sum_{j <= i+1} c_i[j] X_j          (X_0 = the embedding rows)
N(x) = tanh(alpha x) w + b, shift(h)[t] = h[t] + (h[t-1] - h[t]) * s with h[-1] = 0."""
from __future__ import annotations

import math

import torch

D64 = torch.float64


def dyn_tanh(x, w, b, alpha):
    return torch.tanh(alpha * x) * w + (0 if b is None else b)


def token_shift(h, s, before=None):
    """h [T, D]; `before`: the un-shifted row of the token before the first one (None: zeros)."""
    first = torch.zeros(1, h.shape[1], dtype=h.dtype) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], 0)
    return h + (prev - h) * s


def depth_average(results, c):
    """results: X_0 .. X_n; c: n + 1 weights."""
    assert len(results) == len(c)
    return sum(c[j] * results[j] for j in range(len(results)))


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def pair_frequencies(n, base, scaling=None):
    """(f [n / 2], factor on cos and sin).  f_i = base^(-2i / n); with scaling {factor s, original L, fast, slow}: the pair
    index at which a frequency makes t turns over L positions is d(t) = n ln(L / (2 pi t)) / (2 ln base); between
    lo = floor(d(fast)) and hi = ceil(d(slow)) (kept inside 0 .. n - 1) a ramp r goes from 0 to 1 and
    f_i <- (1 - r_i) f_i + r_i f_i / s; cos and sin are multiplied by 0.1 ln s + 1."""
    i = torch.arange(n // 2, dtype=D64)
    f = torch.tensor(float(base), dtype=D64) ** (-2.0 * i / n)
    if not scaling:
        return f, 1.0
    s, L = float(scaling["factor"]), float(scaling["original"])
    d = lambda t: n * math.log(L / (2 * math.pi * t)) / (2 * math.log(base))      # noqa: E731
    lo, hi = max(math.floor(d(scaling["fast"])), 0), min(math.ceil(d(scaling["slow"])), n - 1)
    r = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return (1 - r) * f + r * f / s, 0.1 * math.log(s) + 1.0


def turn_halves(x, angle, factor=1.0):
    """x [T, heads, n], angle [T, n / 2]: entry i is paired with entry i + n / 2 and the pair turns by angle[:, i]."""
    n = x.shape[-1]
    a, b = x[..., :n // 2], x[..., n // 2:]
    c, s = (torch.cos(angle) * factor)[:, None, :], (torch.sin(angle) * factor)[:, None, :]
    return torch.cat([a * c - b * s, b * c + a * s], -1)


def softmax_rows(scores, visible):
    scores = scores.masked_fill(~visible, float("-inf"))
    e = torch.exp(scores - scores.max(-1, keepdim=True).values)
    return e / e.sum(-1, keepdim=True)


def attention(h, W, p, m, eps, pos):
    """Grouped softmax attention; q / k RMS-normed per head, turned by position (first rot.dims entries of each head),
    capped scores, values turned by their own position and the weighted sum turned back by the query's."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = unit_rms((h @ W[p + "q"].T).view(T, H, dk), eps) * W[p + "q.norm"]
    k = unit_rms((h @ W[p + "k"].T).view(T, G, dk), eps) * W[p + "k.norm"]
    v = (h @ W[p + "v"].T).view(T, G, dv)
    rot = m.get("rot")
    va = None
    if rot:
        n = rot["dims"]
        if n:
            f, fac = pair_frequencies(n, rot["base"], rot.get("scaling"))
            ang = pos[:, None].to(D64) * f[None]
            q = torch.cat([turn_halves(q[..., :n], ang, fac), q[..., n:]], -1)
            k = torch.cat([turn_halves(k[..., :n], ang, fac), k[..., n:]], -1)
        va = pos[:, None].to(D64) * pair_frequencies(dv, rot["base"])[0][None]
        v = turn_halves(v, va)
    k, v = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    s = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    w = softmax_rows(s, pos[:, None] >= pos[None, :])
    o = torch.einsum("hij,jhd->ihd", w, v)
    if va is not None:
        o = turn_halves(o, -va)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def short_conv_silu(x, w):
    """x [T, C], w [C, taps] (last column: the current token); zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    xp = torch.cat([torch.zeros(taps - 1, x.shape[1], dtype=x.dtype), x], 0)
    y = sum(xp[j:j + T] * w[:, j] for j in range(taps))
    return y * torch.sigmoid(y)


def channel_delta(h, W, p, m, eps):
    """Gated delta rule with a decay per head and key channel.  Per head, S [dk, dv] from zero:
    S <- diag(g_t) S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = short_conv_silu(h @ W[p + "q"].T, W[p + "q.conv"]).view(T, G, dk)
    k = short_conv_silu(h @ W[p + "k"].T, W[p + "k.conv"]).view(T, G, dk)
    v = short_conv_silu(h @ W[p + "v"].T, W[p + "v.conv"]).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) / math.sqrt(dk)
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    q, k = q.repeat_interleave(H // G, 1), k.repeat_interleave(H // G, 1)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    z = (h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]
    g = torch.exp(-torch.exp(W[p + "A_log"])[None, :, None] * torch.nn.functional.softplus(z).view(T, H, dk))
    S = torch.zeros(H, dk, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = g[t][:, :, None] * S
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + k[t][:, :, None] * u[:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = unit_rms(o, eps) * W[p + "norm"]
    o = o * torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T).view(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + "o"].T


def differential_lambda(W, p, diff):
    return torch.exp((W[p + "lq1"] * W[p + "lk1"]).sum()) - torch.exp((W[p + "lq2"] * W[p + "lk2"]).sum()) + diff


def differential_attention(h, W, p, m, eps, pos, kv=None):
    """Two softmax maps per head over the same values, o = a_1 - lambda a_2, RMS norm per head (no weight) times
    (1 - diff), a gate per element; keys of position j are visible from i if j <= i and both lie in the same run of
    mask.size positions.  kv: (k [T, G, 2, dk], v [T, G, dv]) of another layer, or None.  Returns (output, (k, v))."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + "q"].T).view(T, H, 2, dk)
    k, v = kv if kv is not None else ((h @ W[p + "k"].T).view(T, G, 2, dk), (h @ W[p + "v"].T).view(T, G, dv))
    kk, vv = k.repeat_interleave(H // G, 1), v.repeat_interleave(H // G, 1)
    size = (m.get("mask") or {}).get("size", 0)
    see = pos[:, None] >= pos[None, :]
    if size:
        see = see & (torch.div(pos, size, rounding_mode="floor")[:, None] == torch.div(pos, size, rounding_mode="floor")[None, :])
    w = softmax_rows(torch.einsum("ihmd,jhmd->hmij", q, kk) * m["scale"], see)
    a = torch.einsum("hmij,jhd->ihmd", w, vv)
    diff = m.get("diff", 0.0)
    o = a[:, :, 0] - differential_lambda(W, p, diff) * a[:, :, 1]
    o = unit_rms(o, eps) * (1.0 - diff)
    o = o.reshape(T, H * dv) * torch.sigmoid(h @ W[p + "g"].T)
    return o @ W[p + "o"].T, (k, v)


def feed_forward(h, W, p):
    u = torch.relu(h @ W[p + "up"].T + W[p + "up.b"]) ** 2
    return u @ W[p + "down"].T + W[p + "down.b"]


def forward(cfg, tensors, tokens, dtype=D64, layers_out=None):
    """Logits [T, vocab] of one sequence; layers_out (a list) receives the stream after every layer."""
    W = {k: v.to(dtype) for k, v in tensors.items()}
    eps, m = cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    x = W["embed"][torch.tensor(tokens)]
    pos = torch.arange(x.shape[0])
    results, kvs = [x], {}
    for i, L in enumerate(cfg["layers"]):
        n, p, mx = f"l{i}.", f"l{i}.mix.", L["mixer"]
        h = dyn_tanh(x, W[n + "norm1"], W.get(n + "norm1.b"), W[n + "norm1.alpha"])
        h = token_shift(h, W[n + "shift"])
        if L["type"] == "attention":
            y = attention(h, W, p, mx, eps, pos)
        elif L["type"] == "channel_delta":
            y = channel_delta(h, W, p, mx, eps)
        elif L["type"] == "attention_2":
            src = mx.get("kv_from")
            y, kvs[i] = differential_attention(h, W, p, mx, eps, pos, None if src is None else kvs[src])
        else:
            raise ValueError(L["type"])
        x = x + m * y
        if L.get("mlp"):
            x = x + m * feed_forward(dyn_tanh(x, W[n + "norm2"], W.get(n + "norm2.b"), W[n + "norm2.alpha"]), W, n + "mlp.")
        results.append(x)
        x = depth_average(results, W[n + "dwa"])
        if layers_out is not None:
            layers_out.append(x)
    x = dyn_tanh(x, W["final.norm"], W.get("final.norm.b"), W["final.norm.alpha"])
    return x @ W["head"].T
