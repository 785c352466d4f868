"""Throughput of the Gibevik decoder at layer sizes that resemble a real model (random weights), next to the closest
existing model of the framework, the Fidasun hybrid decoder (latent attention and routed experts with a shared expert
on the same runner), at equal width and depth: `python bench.py --config gibevik`.

Per size: prefill tokens/s (one prompt of `prefill` tokens in one step) and decode tokens/s (`batch` sequences at
context `ctx`, one token each) of both models, CUDA events after warm-up, and a table of the new design's kernels timed
alone at the same shapes with their algorithmic bytes / flops against the measured copy bandwidth and cuBLAS bf16 peak.
Every row of a kernel that gained an option is followed by a row of the SAME kernel at the SAME shape with the option
off (`like`: the form the other models use), so the cost of the option reads off directly."""
from __future__ import annotations

import numpy as np
import torch

from . import bench_hybrid, ops
from .bench_hybrid import _meta, _say, _time
from .models.gibevik import head_slopes

SIZES = {
    "w2048": dict(width=2048, vocab=32000, ff=5632,
                  attn=dict(heads=16, kv_heads=4, dim=128, every=512, coef=0.1),
                  latent=dict(heads=16, dim=64, vdim=64, kv_rank=256),
                  moe=dict(experts=14, identity=2, top=4, ff=512, shared=1024, groups=4, keep=2)),
    "w4096": dict(width=4096, vocab=32000, ff=11008,
                  attn=dict(heads=32, kv_heads=8, dim=128, every=512, coef=0.1),
                  latent=dict(heads=32, dim=64, vdim=64, kv_rank=512),
                  moe=dict(experts=28, identity=4, top=4, ff=1024, shared=2048, groups=4, keep=2)),
}
# (mixer, feed-forward); the third layer reads the second layer's latents
ORDER = [("attention", "dense"), ("latent_attention", "moe"), ("latent_shared", "dense"), ("attention", "moe")]


def config(size, layers):
    s = SIZES[size]
    a, la, mo = s["attn"], s["latent"], s["moe"]
    attn = dict(heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["dim"], scale=a["dim"] ** -0.5,
                q_temp={"coef": a["coef"], "every": a["every"]})
    latent = dict(heads=la["heads"], dim=la["dim"], vdim=la["vdim"], kv_rank=la["kv_rank"], scale=la["dim"] ** -0.5)
    mlps = {"dense": {"kind": "dense", "ff": s["ff"]},
            "moe": {"kind": "moe", "expert": {"ff": mo["ff"]}, "shared": {"ff": mo["shared"]},
                    "router": {"experts": mo["experts"], "identity": mo["identity"], "top": mo["top"],
                               "groups": {"count": mo["groups"], "keep": mo["keep"]}}}}
    out, source = [], None
    for i in range(layers):
        kind, ff = ORDER[i % 4]
        if kind == "attention":
            out.append({"type": "attention", "mixer": attn, "mlp": mlps[ff]})
        elif kind == "latent_shared" and source is not None:
            out.append({"type": "latent_attention", "mixer": dict(latent, kv_from=source), "mlp": mlps[ff]})
        else:
            source = i
            out.append({"type": "latent_attention", "mixer": latent, "mlp": mlps[ff]})
    return {"architecture": "Gibevik", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6}, "layers": out}


def random_tensors(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}
    lin = lambda n, k: (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)         # noqa: E731
    vec = lambda n, m=0.0, s=0.1: (m + s * torch.randn(n, generator=g)).to(torch.bfloat16)   # noqa: E731
    out["embed"] = (torch.randn(cfg["vocab"], D, generator=g) / D ** 0.5).to(torch.bfloat16)
    out["head"], out["final.norm"] = lin(cfg["vocab"], D), vec(D, 1.0)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        out[p + "norm1"], out[p + "norm2"] = vec(D, 1.0), vec(D, 1.0)
        q = p + "mix."
        if L["type"] == "attention":
            H, G, dk = m["heads"], m["kv_heads"], m["dim"]
            out.update({q + "q": lin(H * dk, D), q + "k": lin(G * dk, D), q + "q.norm": vec(dk, 1.0),
                        q + "k.norm": vec(dk, 1.0), q + "g": lin(H * dk, D), q + "o": lin(D, H * dk)})
        else:
            H, R = m["heads"], m["kv_rank"]
            out.update({q + "q": lin(H * m["dim"], D), q + "uk": lin(H * m["dim"], R), q + "uv": lin(H * m["vdim"], R),
                        q + "g": lin(H, D), q + "o": lin(D, H * m["vdim"])})
            if m.get("kv_from") is None:
                out.update({q + "dkv": lin(R, D), q + "dkv.norm": vec(R, 1.0)})
        mlp, q = L["mlp"], p + "mlp."
        if mlp["kind"] == "dense":
            F = mlp["ff"]
            out.update({q + "gate": lin(F, D), q + "up": lin(F, D), q + "down": lin(D, F)})
        else:
            r, F, Fs = mlp["router"], mlp["expert"]["ff"], mlp["shared"]["ff"]
            out.update({q + "router": lin(r["experts"] + r["identity"], D),
                        q + "correction": vec(r["experts"] + r["identity"], 0.0, 0.02),
                        q + "shared.up": lin(Fs, D), q + "shared.down": lin(D, Fs), q + "shared.sg": lin(1, D)})
            for e in range(r["experts"]):
                out.update({f"{q}e{e}.up": lin(F, D), f"{q}e{e}.down": lin(D, F)})
    return out


def kernel_table(size, prefill, batch, ctx, peaks):
    """Each kernel of the design alone at the prefill shape (one sequence of `prefill` tokens) and the decode shape
    (`batch` sequences at context `ctx`): ms, achieved and the fraction of the bound it should sit on; `like` rows are
    the same kernel at the same shape with the new options off."""
    s, dev = SIZES[size], "cuda"
    hbm, tc = float(peaks["hbm_gbs"]) * 1e9, float(peaks["bf16_tflops"]) * 1e12
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *sh: torch.randn(*sh, generator=g, device=dev)          # noqa: E731
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)       # noqa: E731
    rows = []

    def add(name, phase, ms, flops=0.0, nbytes=0.0, bound="hbm", note=""):
        _say(f"{name} {phase}: {ms:.3f} ms")
        ach_f, ach_b = flops / (ms * 1e-3), nbytes / (ms * 1e-3)
        frac = {"hbm": ach_b / hbm, "tensor": ach_f / tc}[bound]
        rows.append(dict(kernel=name, phase=phase, ms=round(ms, 4), tflops=round(ach_f / 1e12, 3),
                         gbs=round(ach_b / 1e9, 1), bound=bound, frac=round(frac, 4), note=note))

    for phase, B, q_len, cx_len in (("prefill", 1, prefill, prefill), ("decode", batch, 1, ctx)):
        T, nblk = B * q_len, (cx_len + 63) // 64
        cu, cl = i32((np.arange(B + 1) * q_len).tolist()), i32([cx_len] * B)
        bt = i32(np.arange(B * nblk).reshape(B, nblk).tolist())
        keys = sum(p + 1 for p in range(cx_len - q_len, cx_len)) * B            # full causal context
        # grouped-head attention: distance bias + gate per element, against the plain form with a gate per head
        a = s["attn"]
        H, G, dk = a["heads"], a["kv_heads"], a["dim"]
        kc = (rnd(B * nblk, 64, G, dk) * 0.3).to(torch.bfloat16)
        vc = (rnd(B * nblk, 64, G, dk) * 0.3).to(torch.bfloat16)
        q, gate_e, gate_h, slopes = rnd(T, H, dk) * 0.3, rnd(T, H * dk), rnd(T, H), head_slopes(H).to(dev)
        for name, gate, sl in (("attention (distance bias, element gate)", gate_e, slopes), ("like: attention (head gate)", gate_h, None)):
            ms = _time(lambda: ops.window_attn(q, kc, vc, None, gate, cu, cl, bt, window=0, keep_first=0, scale=dk ** -0.5,
                                               dist_slopes=sl), 3)
            if phase == "decode":
                add(name, phase, ms, 4.0 * H * keys * dk, keys * G * dk * 4.0, "hbm",
                    "bytes = visible K and V rows, read once per key / value head")
            else:
                add(name, phase, ms, 4.0 * H * keys * dk, 0.0, "tensor", "mma.sync form")
        n_in = H * dk + G * dk + H * dk
        proj, qn, kn = rnd(T, n_in), rnd(dk), rnd(dk)
        pos = torch.arange(cx_len - q_len, cx_len, device=dev).repeat(B)
        slot = ((torch.arange(B, device=dev) * nblk).repeat_interleave(q_len) + pos // 64) * 64 + pos % 64
        ms = _time(lambda: ops.window_attn_prep(proj, None, qn, kn, None, pos, slot, kc, vc, heads=H, rot_dims=0, eps=1e-6,
                                                head_norm=True, v_from_k=True, q_temp=(a["coef"], a["every"])), 3)
        add("attention prep (head norms, values = keys, temperature)", phase, ms, 0.0,
            T * ((H + G) * dk * 4.0 + H * dk * 4.0 + 2 * G * dk * 2.0), "hbm")
        proj2, qn2, kn2 = rnd(T, H * dk + 2 * G * dk + H), rnd(H * dk), rnd(G * dk)
        ms = _time(lambda: ops.window_attn_prep(proj2, None, qn2, kn2, None, pos, slot, kc, vc, heads=H, rot_dims=0,
                                                eps=1e-6), 3)
        add("like: attention prep (whole-projection norms, own values)", phase, ms, 0.0,
            T * ((H + 2 * G) * dk * 4.0 + H * dk * 4.0 + 2 * G * dk * 2.0), "hbm")
        del kc, vc, q, proj, proj2
        # latent attention over the whole context with a gate per head, against the ungated call
        la = s["latent"]
        Hl, r = la["heads"], la["kv_rank"]
        cache = (rnd(B * nblk, 64, r) * 0.3).to(torch.bfloat16)
        ql, gl = rnd(T, Hl, r) * 0.1, rnd(T, Hl)
        for name, gate in (("latent attention (head gate)", gl), ("like: latent attention", None)):
            ms = _time(lambda: ops.latent_attn(ql, cache, None, cu, cl, bt, kv_rank=r, rot_dim=0, window=0, scale=0.1,
                                               gate=gate), 3)
            if phase == "decode":
                add(name, phase, ms, 4.0 * Hl * keys * r, keys * r * 2.0, "hbm",
                    "bytes = visible cache rows, read once for all heads")
            else:
                add(name, phase, ms, 4.0 * Hl * keys * r, 0.0, "tensor", "mma.sync form")
        del cache, ql
        # router and experts
        mo, D = s["moe"], s["width"]
        E, ident, top, F = mo["experts"], mo["identity"], mo["top"], mo["ff"]
        z, bias = rnd(T, E + ident), rnd(E + ident) * 0.02
        ms = _time(lambda: ops.moe_route_ex(z, bias, top, 1.0, mo["groups"], mo["keep"]), 3)
        add("router (bias, groups)", phase, ms, 0.0, T * ((E + ident) * 4.0 + top * 8.0), "hbm")
        ms = _time(lambda: ops.moe_route(z, top, 1.0), 3)
        add("like: router", phase, ms, 0.0, T * ((E + ident) * 4.0 + top * 8.0), "hbm")
        h = (rnd(T, D) * 0.5).to(torch.bfloat16)
        up = (rnd(E, F, D) / D ** 0.5).to(torch.bfloat16)
        gu = (rnd(E, 2 * F, D) / D ** 0.5).to(torch.bfloat16)
        dn = (rnd(E, D, F) / F ** 0.5).to(torch.bfloat16)
        idx, w = ops.moe_route_ex(z, bias, top, 1.0, mo["groups"], mo["keep"])
        real = int((idx < E).sum().item())                       # (token, choice) pairs that reach a real expert
        hit = int(torch.unique(idx[idx < E]).numel())
        xo = torch.zeros(T, D, device=dev)
        ms = _time(lambda: ops.moe_experts_ex(xo, h, idx, w, up, dn, act="relu2", identity=ident, accumulate=False), 3)
        if phase == "decode":
            add("experts (squared ReLU, identity experts)", phase, ms, 4.0 * real * F * D, hit * 2.0 * F * D * 2, "hbm",
                "bytes = weights of the experts hit")
        else:
            add("experts (squared ReLU, identity experts)", phase, ms, 4.0 * real * F * D, 0.0, "tensor",
                "mma.sync grouped GEMM")
        idx2 = torch.where(idx < E, idx, idx - E).contiguous()
        hit2 = int(torch.unique(idx2).numel())
        ms = _time(lambda: ops.moe_experts(xo, h, idx2, w, gu, dn), 3)
        if phase == "decode":
            add("like: experts (SiLU gate)", phase, ms, 6.0 * T * top * F * D, hit2 * 3.0 * F * D * 2, "hbm",
                "bytes = weights of the experts hit")
        else:
            add("like: experts (SiLU gate)", phase, ms, 6.0 * T * top * F * D, 0.0, "tensor", "mma.sync grouped GEMM")
        del h, up, gu, dn
        torch.cuda.empty_cache()
    return rows


def run(size="w2048", layers=4, prefill=4096, batch=32, ctx=2048, reps=5):
    import json
    from pathlib import Path

    from . import models
    pk = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peaks = json.loads(pk.read_text()) if pk.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    s = SIZES[size]
    res = {"size": size, "layers": layers, "order": [f"{m} + {f}" for m, f in ORDER[:layers]], "prefill_tokens": prefill,
           "decode_batch": batch, "decode_context": ctx}
    nblk = (max(prefill, ctx) + 63) // 64
    mp, md = _meta(1, prefill, prefill, nblk, s["vocab"]), _meta(batch, 1, ctx, nblk, s["vocab"])
    arms = (("gibevik", config(size, layers), random_tensors),
            ("fidasun", bench_hybrid.config(size, layers), bench_hybrid.random_tensors))
    for name, cfg, make in arms:
        r = models.build_runner(cfg, make(cfg), dtype=torch.bfloat16, device="cuda", num_blocks=batch * nblk,
                                max_blocks_per_seq=nblk, max_seqs=batch, max_tokens=max(prefill, batch),
                                num_state_slots=batch)
        for c in list(r.kv_cache.values()) + list(r.v_cache.values()):
            c.normal_(std=0.3)
        ms = _time(lambda: r.step(mp, [prefill - 1]), 1, warm=1)
        ms = _time(lambda: r.step(mp, [prefill - 1]), reps, warm=1)
        res[name] = {"prefill_ms": ms, "prefill_tok_s": prefill * 1e3 / ms, "launches": int(r.launches_per_step)}
        ms = _time(lambda: r.step(md, list(range(batch))), reps * 4, warm=3)
        res[name].update(decode_ms=ms, decode_tok_s=batch * 1e3 / ms)
        _say(f"{name}: {res[name]}")
        del r
        torch.cuda.empty_cache()
    res["kernels"] = kernel_table(size, prefill, batch, ctx, peaks)
    return res
