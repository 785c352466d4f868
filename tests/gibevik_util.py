"""Small Gibevik configurations with random weights.  Test infrastructure; the driver that feeds portions through the
scheduler and the runner is fidasun_util.Driver, the random schedules come from zalalix_util.random_schedule (both are
model-agnostic)."""
from __future__ import annotations

import torch


def attn_cfg(**kw):
    m = dict(heads=6, kv_heads=3, dim=16, vdim=16, scale=0.25, q_temp={"coef": 0.3, "every": 7})
    m.update(kw)
    if "vdim" not in kw:
        m["vdim"] = m["dim"]
    return m


def latent_cfg(**kw):
    m = dict(heads=3, dim=12, vdim=20, kv_rank=24, scale=0.3)
    m.update(kw)
    return m


def moe_cfg(**kw):
    m = dict(kind="moe", expert={"ff": 24}, shared={"ff": 40},
             router=dict(experts=9, identity=3, top=4, groups={"count": 4, "keep": 2}))
    m.update(kw)
    return m


def dense_cfg(ff=56):
    return {"kind": "dense", "ff": ff}


def layer(kind, mlp=None, **kw):
    """kind: "attention" or "latent_attention"; mlp: None, dense_cfg() or moe_cfg()."""
    return {"type": kind, "mixer": attn_cfg(**kw) if kind == "attention" else latent_cfg(**kw), "mlp": mlp}


def make_cfg(layers, width=48, vocab=96, eps=1e-5):
    return {"architecture": "Gibevik", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}


def full_cfg(**kw):
    """Both mixers with every feed-forward kind, a latent cache shared by two later layers, sizes pairwise different."""
    return make_cfg([layer("attention", dense_cfg()),
                     layer("latent_attention", moe_cfg()),
                     layer("latent_attention", dense_cfg(40), kv_from=1, heads=2, dim=20, vdim=8),
                     layer("attention", moe_cfg(shared=None, router=dict(experts=5, identity=0, top=2)),
                           heads=4, kv_heads=1, dim=32, q_temp={"coef": 1.5, "every": 64}),
                     layer("latent_attention", None, kv_from=1, heads=5, dim=8, vdim=16)], **kw)


def random_tensors(cfg, seed=0):
    """name -> CPU tensor; everything is bf16 (exact in both operand dtypes)."""
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}

    def lin(n, k, gain=1.0):
        return (torch.randn(n, k, generator=g) * gain / k ** 0.5).to(torch.bfloat16)

    def vec(n, mean=0.0, std=0.2):
        return (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    out["head"] = lin(cfg["vocab"], D)
    out["final.norm"] = vec(D, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"] = vec(D, 1.0)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, dk = m["heads"], m["kv_heads"], m["dim"]
            out[q + "q"], out[q + "k"] = lin(H * dk, D, 2.0), lin(G * dk, D, 2.0)
            out[q + "q.norm"], out[q + "k.norm"] = vec(dk, 1.0, 0.4), vec(dk, 1.0, 0.4)
            out[q + "g"], out[q + "o"] = lin(H * dk, D, 2.0), lin(D, H * dk)
        else:
            H, R = m["heads"], m["kv_rank"]
            out[q + "q"] = lin(H * m["dim"], D, 2.0)
            if m.get("kv_from") is None:
                out[q + "dkv"], out[q + "dkv.norm"] = lin(R, D, 2.0), vec(R, 1.0, 0.4)
            out[q + "uk"], out[q + "uv"] = lin(H * m["dim"], R, 2.0), lin(H * m["vdim"], R)
            out[q + "g"], out[q + "o"] = lin(H, D, 3.0), lin(D, H * m["vdim"])
        mlp = L.get("mlp")
        if not mlp:
            continue
        out[p + "norm2"] = vec(D, 1.0)
        q = p + "mlp."
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            out[q + "gate"], out[q + "up"], out[q + "down"] = lin(F, D, 2.0), lin(F, D, 2.0), lin(D, F)
        else:
            r = mlp["router"]
            E, n_all, F = r["experts"], r["experts"] + r.get("identity", 0), mlp["expert"]["ff"]
            out[q + "router"] = lin(n_all, D, 3.0)
            out[q + "correction"] = vec(n_all, 0.0, 0.15)
            for e in range(E):
                out[f"{q}e{e}.up"], out[f"{q}e{e}.down"] = lin(F, D, 2.0), lin(D, F, 2.0)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                out[q + "shared.up"], out[q + "shared.down"] = lin(Fs, D, 2.0), lin(D, Fs)
                out[q + "shared.sg"] = lin(1, D, 3.0)
    return out


def random_layers(rng, count):
    """`count` layers drawn at random; a latent-attention layer may read an earlier one's latent cache."""
    pick = lambda *xs: xs[int(rng.integers(len(xs)))]              # noqa: E731
    layers, sources = [], []
    for i in range(count):
        if rng.random() < 0.45:
            G = pick(1, 2, 3)
            m = dict(heads=G * pick(1, 2, 4, 9), kv_heads=G, dim=pick(8, 16, 32, 48, 72), scale=pick(0.125, 0.3),
                     q_temp=pick(None, {"coef": pick(0.1, 1.0), "every": pick(1, 5, 64, 100)}))
            m["vdim"] = m["dim"]
            kind = "attention"
        else:
            m = dict(heads=pick(1, 2, 5, 17), dim=pick(4, 16, 40), vdim=pick(8, 24, 64), kv_rank=pick(16, 64, 72),
                     scale=pick(0.2, 0.35))
            same = [j for j in sources if layers[j]["mixer"]["kv_rank"] == m["kv_rank"]]
            if same and rng.random() < 0.6:
                m["kv_from"] = pick(*same)
            else:
                sources.append(i)
            kind = "latent_attention"
        r = rng.random()
        if r < 0.25:
            mlp = None
        elif r < 0.55:
            mlp = dense_cfg(pick(24, 64, 100))
        else:
            groups = pick(None, {"count": 1, "keep": 1}, {"count": 2, "keep": 1}, {"count": 4, "keep": 3})
            per = pick(1, 2, 3) * (groups["count"] if groups else 1)
            ident = pick(0, 0, 1, 2)
            if groups:                       # experts and identity experts together split into the groups
                n_all = per
                ident = min(ident, n_all - 1)
                E = n_all - ident
            else:
                E, n_all = per, per + ident
            avail = n_all // groups["count"] * groups["keep"] if groups else n_all
            router = dict(experts=E, identity=ident, top=min(pick(1, 2, 3), avail))
            if groups:
                router["groups"] = groups
            mlp = dict(kind="moe", expert={"ff": pick(8, 40, 72)}, router=router,
                       shared=pick(None, {"ff": pick(16, 50)}))
        layers.append({"type": kind, "mixer": m, "mlp": mlp})
    return layers
