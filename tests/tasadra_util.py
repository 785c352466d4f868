"""Small Tasadra configurations with random weights.  Test infrastructure; the driver that feeds portions through the
scheduler and the runner is fidasun_util.Driver, the random schedules are zalalix_util.random_schedule."""
from __future__ import annotations

import torch


def attn_cfg(**kw):
    m = dict(heads=6, kv_heads=2, dim=24, vdim=20, scale=0.2, softcap=30.0,
             rot={"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}})
    m.update(kw)
    return m


def delta_cfg(**kw):
    m = dict(heads=4, kv_heads=2, dim=24, vdim=40, conv=3, a_rank=6, g_rank=10)
    m.update(kw)
    return m


def diff_cfg(**kw):
    m = dict(heads=4, kv_heads=2, dim=20, vdim=24, scale=0.25, diff=0.3, mask={"size": 37})
    m.update(kw)
    return m


def layer(kind, ff=40, **kw):
    m = {"attention": attn_cfg, "channel_delta": delta_cfg, "attention_2": diff_cfg}[kind](**kw)
    return {"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def make_cfg(layers, width=48, vocab=96, eps=1e-5, mult=0.7):
    return {"architecture": "Tasadra", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult,
            "layers": layers}


def full_cfg(**kw):
    """All three mixers, one layer that reads another's pages, one without a feed-forward; sizes pairwise different."""
    return make_cfg([layer("attention_2"), layer("channel_delta"), layer("attention", ff=0),
                     layer("attention_2", kv_from=0, ff=56), layer("attention", heads=4, kv_heads=4, dim=16, vdim=32,
                                                                   rot={"base": 500.0, "dims": 8}),
                     layer("channel_delta", heads=2, kv_heads=2, dim=16, vdim=24, conv=4, a_rank=3, g_rank=5)], **kw)


def random_tensors(cfg, seed=0):
    """name -> CPU tensor, all bf16 (exact in both operand dtypes).  The low-rank sizes of a channel_delta mixer are
    read from its `a_rank` / `g_rank` entries, which the model file ignores (it reads the tensors' shapes)."""
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(n, k, gain=1.0):
        return (torch.randn(n, k, generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.2):
        return (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def norm(name):
        out[name], out[name + ".b"] = vec(D, 1.0, 0.3), vec(D, 0.0, 0.2)
        out[name + ".alpha"] = (0.4 + 0.5 * torch.rand((), generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    out["head"] = lin(cfg["vocab"], D)
    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        norm(p + "norm1")
        out[p + "shift"] = torch.rand(D, generator=g).to(torch.bfloat16)
        c = torch.rand(i + 2, generator=g) + 0.2
        out[p + "dwa"] = (c / c.sum() * (0.8 + 0.4 * torch.rand((), generator=g))).to(torch.bfloat16)
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            out[p + "mix.q"], out[p + "mix.k"], out[p + "mix.v"] = lin(H * dk, D, 2.0), lin(G * dk, D, 2.0), lin(G * dv, D, 2.0)
            out[p + "mix.q.norm"], out[p + "mix.k.norm"] = vec(dk, 1.0, 0.3), vec(dk, 1.0, 0.3)
            out[p + "mix.g"] = lin(H, D, 2.0)
        elif L["type"] == "channel_delta":
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[p + f"mix.{n}"] = lin(rows, D, 2.0)
                out[p + f"mix.{n}.conv"] = vec(rows * m["conv"], 0.0, 0.6).reshape(rows, m["conv"])
            out[p + "mix.b"] = lin(H, D, 2.0)
            out[p + "mix.A_log"] = vec(H, -0.5, 0.7)
            out[p + "mix.dt_bias"] = vec(H * dk, -1.0, 0.7)
            out[p + "mix.a1"], out[p + "mix.a2"] = lin(m["a_rank"], D, 2.0), lin(H * dk, m["a_rank"], 2.0)
            out[p + "mix.g1"], out[p + "mix.g2"] = lin(m["g_rank"], D, 2.0), lin(H * dv, m["g_rank"], 2.0)
            out[p + "mix.norm"] = vec(dv, 1.0, 0.3)
        else:
            out[p + "mix.q"] = lin(H * 2 * dk, D, 2.0)
            if m.get("kv_from") is None:
                out[p + "mix.k"], out[p + "mix.v"] = lin(G * 2 * dk, D, 2.0), lin(G * dv, D, 2.0)
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[p + "mix." + n] = vec(dk, 0.0, 0.25)
            out[p + "mix.g"] = lin(H * dv, D, 2.0)
        out[p + "mix.o"] = lin(D, H * dv)
        if L.get("mlp"):
            F = L["mlp"]["ff"]
            norm(p + "norm2")
            out[p + "mlp.up"], out[p + "mlp.up.b"] = lin(F, D, 2.0), vec(F, 0.0, 0.3)
            out[p + "mlp.down"], out[p + "mlp.down.b"] = lin(D, F), vec(D, 0.0, 0.3)
    return out


def random_layers(rng, count):
    """`count` layers drawn at random; a differential-attention layer may read the pages of an earlier one with the same
    head counts and sizes."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]              # noqa: E731
    layers, sources = [], []
    for i in range(count):
        r = rng.random()
        if r < 0.35:
            G = pick(1, 2, 3)
            dk = pick(8, 16, 32, 40, 80)
            rot = {"base": pick(100.0, 10000.0, 1000000.0), "dims": pick(2, dk // 2, dk) // 2 * 2}
            if rng.random() < 0.6:
                rot["scaling"] = {"factor": pick(2.0, 8.0), "original": pick(32, 128), "fast": pick(8.0, 16.0),
                                  "slow": pick(1.0, 2.0)}
            m = dict(heads=G * pick(1, 2, 4, 9), kv_heads=G, dim=dk, vdim=pick(8, 16, 32, 50, 96), scale=pick(0.125, 0.3),
                     softcap=pick(0.0, 5.0, 20.0), rot=rot)
            kind = "attention"
        elif r < 0.65:
            G = pick(1, 2)
            m = dict(heads=G * pick(1, 2, 3), kv_heads=G, dim=pick(8, 16, 40, 64), vdim=pick(8, 24, 64), conv=pick(1, 2, 4),
                     a_rank=pick(1, 4, 12), g_rank=pick(1, 8, 20))
            kind = "channel_delta"
        else:
            G = pick(1, 2)
            m = dict(heads=G * pick(1, 2, 4), kv_heads=G, dim=pick(8, 16, 32, 40), vdim=pick(8, 16, 32, 64, 80),
                     scale=pick(0.2, 0.35), diff=pick(0.1, 0.4, 0.8), mask={"size": pick(1, 5, 64, 100, 129)})
            if sources and rng.random() < 0.5:               # its own queries, mask and constants on another layer's pages
                m["kv_from"] = pick(*sources)
                m.update({n: layers[m["kv_from"]]["mixer"][n] for n in ("heads", "kv_heads", "dim", "vdim")})
            else:
                sources.append(i)
            kind = "attention_2"
        ff = pick(0, 24, 64, 100)
        layers.append({"type": kind, "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None})
    return layers
