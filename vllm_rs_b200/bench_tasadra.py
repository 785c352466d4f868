"""Throughput of the Tasadra decoder at layer sizes that resemble a real model (random weights), next to the closest
existing model of the framework, the Zalalix decoder (grouped-head softmax attention with rotary positions, capped
scores and a head gate, a recurrent mixer with a low-rank decay per key channel, dense feed-forwards, on the same
runner), at equal width and depth: `python bench.py --config tasadra`.

Per size: prefill tokens/s (one prompt of `prefill` tokens in one step) and decode tokens/s (`batch` sequences at
context `ctx`, one token each) of both models, CUDA events after warm-up, and a table of the new design's kernels timed
alone at the same shapes with their algorithmic bytes / flops against the measured copy bandwidth and cuBLAS bf16 peak
(the token-serial scans against the nominal fp32 FMA rate).  Every row of a kernel that gained an option, and every new
kernel, is followed by a `like` row: the same kernel at the same shape with the option off, or the closest kernel the
other models use."""
from __future__ import annotations

import numpy as np
import torch

from . import bench_zalalix, ops
from .bench_hybrid import _meta, _say, _time
from .rotary import rotary_frequencies

SIZES = {
    # attention; the delta rule with a decay per key channel; differential attention (two maps of `dim` over values of
    # `vdim`) under a chunked mask; ungated feed-forward with as many weights as a gated one of 5 632 / 11 008
    "w2048": dict(width=2048, vocab=32000, ff=8448,
                  attn=dict(heads=16, kv_heads=4, dim=128, vdim=128, rot_dims=64),
                  delta=dict(heads=16, kv_heads=16, dim=128, vdim=128, conv=4, a_rank=64, g_rank=128),
                  diff=dict(heads=8, kv_heads=2, dim=64, vdim=128, chunk=1024)),
    "w4096": dict(width=4096, vocab=32000, ff=16512,
                  attn=dict(heads=32, kv_heads=8, dim=128, vdim=128, rot_dims=64),
                  delta=dict(heads=32, kv_heads=32, dim=128, vdim=128, conv=4, a_rank=128, g_rank=256),
                  diff=dict(heads=16, kv_heads=4, dim=64, vdim=128, chunk=2048)),
}
ORDER = ["attention", "channel_delta", "attention_2", "attention_2 (shared pages)"]


def config(size, layers):
    s = SIZES[size]
    a, de, di = s["attn"], s["delta"], s["diff"]
    mix = {"attention": dict(heads=a["heads"], kv_heads=a["kv_heads"], dim=a["dim"], vdim=a["vdim"], scale=a["dim"] ** -0.5,
                             softcap=30.0, rot={"base": 10000.0, "dims": a["rot_dims"],
                                                "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}}),
           "channel_delta": dict(heads=de["heads"], kv_heads=de["kv_heads"], dim=de["dim"], vdim=de["vdim"], conv=de["conv"],
                                 a_rank=de["a_rank"], g_rank=de["g_rank"]),
           "attention_2": dict(heads=di["heads"], kv_heads=di["kv_heads"], dim=di["dim"], vdim=di["vdim"],
                               scale=di["dim"] ** -0.5, diff=0.4, mask={"size": di["chunk"]})}
    out, source = [], None
    for i in range(layers):
        kind = ORDER[i % 4]
        if kind.startswith("attention_2"):
            m = dict(mix["attention_2"])
            if kind.endswith("(shared pages)") and source is not None:
                m["kv_from"] = source
            else:
                source = i
            out.append({"type": "attention_2", "mixer": m, "mlp": {"kind": "dense", "ff": s["ff"]}})
        else:
            out.append({"type": kind, "mixer": mix[kind], "mlp": {"kind": "dense", "ff": s["ff"]}})
    return {"architecture": "Tasadra", "width": s["width"], "vocab": s["vocab"], "norm": {"eps": 1e-6},
            "residual_mult": 0.6, "layers": out}


def random_tensors(cfg, seed=0):
    g = torch.Generator().manual_seed(seed)
    D, out = cfg["width"], {}
    lin = lambda n, k: (torch.randn(n, k, generator=g) / k ** 0.5).to(torch.bfloat16)         # noqa: E731
    vec = lambda n, m=0.0, s=0.1: (m + s * torch.randn(n, generator=g)).to(torch.bfloat16)   # noqa: E731

    def norm(name):
        out[name], out[name + ".b"], out[name + ".alpha"] = vec(D, 1.0), vec(D), torch.tensor(0.7).to(torch.bfloat16)

    out["embed"] = torch.randn(cfg["vocab"], D, generator=g).to(torch.bfloat16)
    out["head"] = lin(cfg["vocab"], D)
    norm("final.norm")
    for i, L in enumerate(cfg["layers"]):
        p, q, m = f"l{i}.", f"l{i}.mix.", L["mixer"]
        norm(p + "norm1"), norm(p + "norm2")
        out[p + "shift"] = torch.rand(D, generator=g).to(torch.bfloat16)
        out[p + "dwa"] = torch.full((i + 2,), 1.0 / (i + 2)).to(torch.bfloat16)
        H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        if L["type"] == "attention":
            out.update({q + "q": lin(H * dk, D), q + "k": lin(G * dk, D), q + "v": lin(G * dv, D), q + "g": lin(H, D),
                        q + "q.norm": vec(dk, 1.0), q + "k.norm": vec(dk, 1.0)})
        elif L["type"] == "channel_delta":
            for n, rows in (("q", G * dk), ("k", G * dk), ("v", H * dv)):
                out[q + n], out[q + n + ".conv"] = lin(rows, D), vec(rows * m["conv"], 0.0, 0.5).reshape(rows, m["conv"])
            out.update({q + "b": lin(H, D), q + "A_log": vec(H, -0.5, 0.5), q + "dt_bias": vec(H * dk, -1.0, 0.5),
                        q + "a1": lin(m["a_rank"], D), q + "a2": lin(H * dk, m["a_rank"]), q + "g1": lin(m["g_rank"], D),
                        q + "g2": lin(H * dv, m["g_rank"]), q + "norm": vec(dv, 1.0)})
        else:
            out.update({q + "q": lin(H * 2 * dk, D), q + "g": lin(H * dv, D)})
            if m.get("kv_from") is None:
                out.update({q + "k": lin(G * 2 * dk, D), q + "v": lin(G * dv, D)})
            for n in ("lq1", "lk1", "lq2", "lk2"):
                out[q + n] = vec(dk, 0.0, 0.1)
        out[q + "o"] = lin(D, H * dv)
        F = L["mlp"]["ff"]
        out.update({p + "mlp.up": lin(F, D), p + "mlp.up.b": vec(F), p + "mlp.down": lin(D, F), p + "mlp.down.b": vec(D)})
    return out


def kernel_table(size, prefill, batch, ctx, peaks):
    """Each kernel of the design alone at the prefill shape (one sequence of `prefill` tokens) and the decode shape
    (`batch` sequences at context `ctx`): ms, achieved and the fraction of the bound it should sit on; `like` rows are
    the same kernel with the new options off, or the closest kernel of the other models, at the same shape."""
    s, dev = SIZES[size], "cuda"
    hbm, tc = float(peaks["hbm_gbs"]) * 1e9, float(peaks["bf16_tflops"]) * 1e12
    fma = 148 * 128 * 2 * 1.9e9                      # fp32 FMA peak of the CUDA cores (nominal clocks)
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *sh: torch.randn(*sh, generator=g, device=dev)          # noqa: E731
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=dev)       # noqa: E731
    rows, D = [], s["width"]

    def add(name, phase, ms, flops=0.0, nbytes=0.0, bound="hbm", note=""):
        _say(f"{name} {phase}: {ms:.3f} ms")
        ach_f, ach_b = flops / (ms * 1e-3), nbytes / (ms * 1e-3)
        frac = {"hbm": ach_b / hbm, "tensor": ach_f / tc, "fp32": ach_f / fma}[bound]
        rows.append(dict(kernel=name, phase=phase, ms=round(ms, 4), tflops=round(ach_f / 1e12, 3),
                         gbs=round(ach_b / 1e9, 1), bound=bound, frac=round(frac, 4), note=note))

    for phase, B, q_len, cx_len in (("prefill", 1, prefill, prefill), ("decode", batch, 1, ctx)):
        T, nblk = B * q_len, (cx_len + 63) // 64
        cu, cl = i32((np.arange(B + 1) * q_len).tolist()), i32([cx_len] * B)
        bt = i32(np.arange(B * nblk).reshape(B, nblk).tolist())
        slots = i32(list(range(B)))
        pos = torch.arange(cx_len - q_len, cx_len, device=dev).repeat(B)
        slot = ((torch.arange(B, device=dev) * nblk).repeat_interleave(q_len) + pos // 64) * 64 + pos % 64
        causal = sum(p + 1 for p in range(cx_len - q_len, cx_len)) * B
        # ---- attention: full causal, capped; its sums go to the finish kernel in fp32 (the values are rotated)
        a = s["attn"]
        H, G, dk, dv = a["heads"], a["kv_heads"], a["dim"], a["vdim"]
        kc = (rnd(B * nblk, 64, G, dk) * 0.3).to(torch.bfloat16)
        vc = (rnd(B * nblk, 64, G, dv) * 0.3).to(torch.bfloat16)
        q, gate_h = rnd(T, H, dk) * 0.3, rnd(T, H)
        for name, f32, gate in (("attention (fp32 sums for the finish kernel)", True, None), ("like: attention (head gate inside)", False, gate_h)):
            ms = _time(lambda: ops.window_attn(q, kc, vc, None, gate, cu, cl, bt, window=0, keep_first=0, scale=dk ** -0.5,
                                               softcap=30.0, out_f32=f32), 3)
            if phase == "decode":
                add(name, phase, ms, 4.0 * H * causal * dk, causal * G * (dk + dv) * 2.0, "hbm",
                    "bytes = visible K and V rows, read once per key / value head")
            else:
                add(name, phase, ms, 2.0 * H * causal * (dk + dv), 0.0, "tensor", "mma.sync form")
        sums, fv = rnd(T, H, dv), torch.from_numpy(rotary_frequencies(dv, 10000.0)[0]).to(dev)
        ms = _time(lambda: ops.attn_finish(sums, gate_h, pos, heads=H, v_rot_freq=fv, dtype=torch.bfloat16), 3)
        add("attention finish (turn back, head gate)", phase, ms, 0.0, T * H * dv * 6.0, "hbm")
        freq, mag = rotary_frequencies(a["rot_dims"], 10000.0, {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0})
        freq = torch.from_numpy(freq).to(dev)
        proj, qn, kn = rnd(T, H * dk + G * (dk + dv) + H), rnd(dk), rnd(dk)
        io = T * ((H * dk + G * (dk + dv)) * 4.0 + H * dk * 4.0 + G * (dk + dv) * 2.0)
        ms = _time(lambda: ops.window_attn_prep(proj, None, qn, kn, freq, pos, slot, kc, vc, heads=H, rot_dims=a["rot_dims"],
                                                eps=1e-6, head_norm=True, rot_half=True, rot_mag=mag, v_rot_freq=fv), 3)
        add("attention prep (head norms, two-halves rotary, rotated values)", phase, ms, 0.0, io, "hbm")
        ms = _time(lambda: ops.window_attn_prep(proj, None, qn, kn, freq, pos, slot, kc, vc, heads=H, rot_dims=a["rot_dims"],
                                                eps=1e-6, head_norm=True), 3)
        add("like: attention prep (head norms, interleaved rotary)", phase, ms, 0.0, io, "hbm")
        del kc, vc, q, proj, sums
        # ---- differential attention: two maps over one set of values, chunked mask, then the finish kernel
        di = s["diff"]
        H, G, dk, dv, ch = di["heads"], di["kv_heads"], di["dim"], di["vdim"], di["chunk"]
        kc = (rnd(B * nblk, 64, 2 * G, dk) * 0.3).to(torch.bfloat16)
        vc = (rnd(B * nblk, 64, G, dv) * 0.3).to(torch.bfloat16)
        q2 = rnd(T, 2 * H, dk) * 0.3
        seen = sum(p % ch + 1 for p in range(cx_len - q_len, cx_len)) * B
        ms = _time(lambda: ops.window_attn(q2, kc, vc, None, None, cu, cl, bt, window=0, keep_first=0, scale=dk ** -0.5,
                                           chunk=ch, out_f32=True), 3)
        if phase == "decode":
            add("differential attention (two maps, chunked mask)", phase, ms, 4.0 * H * seen * (dk + dv),
                seen * G * (2 * dk + dv) * 2.0, "hbm", "bytes = visible K rows of both maps and V rows")
        else:
            add("differential attention (two maps, chunked mask)", phase, ms, 4.0 * H * seen * (dk + dv), 0.0, "tensor",
                "mma.sync form")
        kc1 = (rnd(B * nblk, 64, G, 2 * dk) * 0.3).to(torch.bfloat16)
        q1, gate_e = rnd(T, H, 2 * dk) * 0.3, rnd(T, H * dv)
        ms = _time(lambda: ops.window_attn(q1, kc1, vc, None, gate_e, cu, cl, bt, window=ch, keep_first=0,
                                           scale=dk ** -0.5), 3)
        wseen = sum(min(p + 1, ch) for p in range(cx_len - q_len, cx_len)) * B
        if phase == "decode":
            add("like: one map of twice the key size, sliding window of the chunk's size", phase, ms,
                2.0 * H * wseen * (2 * dk + dv), wseen * G * (2 * dk + dv) * 2.0, "hbm")
        else:
            add("like: one map of twice the key size, sliding window of the chunk's size", phase, ms,
                2.0 * H * wseen * (2 * dk + dv), 0.0, "tensor", "mma.sync form")
        sums2 = rnd(T, 2 * H, dv)
        ms = _time(lambda: ops.attn_finish(sums2, gate_e, None, heads=H, maps=2, lam=0.6, head_norm=True, out_scale=0.5,
                                           dtype=torch.bfloat16), 3)
        add("attention finish (two maps, head norm, element gate)", phase, ms, 0.0, T * H * dv * (8.0 + 4.0 + 2.0), "hbm")
        yv, wv = rnd(T, H * dv), rnd(dv)
        ms = _time(lambda: ops.gated_group_norm(yv, gate_e, wv, dv, 1e-6, False, dtype=torch.bfloat16, gate_act="sigmoid"), 3)
        add("like: gated group norm", phase, ms, 0.0, T * H * dv * (4.0 + 4.0 + 2.0), "hbm")
        del kc, kc1, vc, q1, q2, sums2
        # ---- the delta rule with a decay per key channel
        de = s["delta"]
        H, G, dk, dv, ra = de["heads"], de["kv_heads"], de["dim"], de["vdim"], de["a_rank"]
        low, w2, bias, a_log = rnd(T, ra), rnd(H * dk, ra) * 0.1, rnd(H * dk) - 1.0, rnd(H) * 0.5 - 0.5
        ms = _time(lambda: ops.channel_decay(low, w2, bias, a_log, dk), 3)
        add("channel decay (low rank -> exp(-exp(A) softplus))", phase, ms, 2.0 * T * H * dk * ra, T * (ra + H * dk) * 4.0, "hbm")
        ms = _time(lambda: ops.lowrank_decay(low, w2, bias, 16.0), 3)
        add("like: low-rank decay (sigmoid^(1/tau))", phase, ms, 2.0 * T * H * dk * ra, T * (ra + H * dk) * 4.0, "hbm")
        decay = ops.channel_decay(low, w2, bias, a_log, dk).view(T, H, dk)
        qd, kd, vd, bd, ad = rnd(T, G, dk), rnd(T, G, dk), rnd(T, H, dv), rnd(T, H), rnd(T, H)
        state = torch.zeros(B, H, dk, dv, device=dev)
        dtb = rnd(H) - 1.0
        sbytes = B * H * dk * dv * 8.0
        for name, fn in (("delta rule (decay per key channel)", lambda: ops.delta_rule_chan(qd, kd, vd, bd, decay, state, slots, cu, cl)),
                         ("like: delta rule (decay per head)", lambda: ops.delta_rule(qd, kd, vd, bd, ad, a_log, dtb, state, slots, cu, cl))):
            ms = _time(fn, 3)
            if phase == "decode":
                add(name, phase, ms, 6.0 * T * H * dk * dv, sbytes, "hbm", "bytes = state read + write")
            else:
                add(name, phase, ms, 6.0 * T * H * dk * dv, 0.0, "fp32", "token-serial scan")
        del state, decay, qd, kd, vd
        # ---- the row kernels of the layer
        x, w, b, sh = rnd(T, D), rnd(D), rnd(D), torch.rand(D, generator=g, device=dev)
        st = torch.zeros(B, D, device=dev)
        ms = _time(lambda: ops.stream_norm(x, w, b, kind="dyntanh", alpha=0.7, shift_w=sh, shift_state=st, state_slots=slots,
                                           cu_seqlens_q=cu, context_lens=cl, dtype=torch.bfloat16), 3)
        add("dynamic-tanh norm + token shift", phase, ms, 0.0, T * D * 6.0, "hbm")
        ms = _time(lambda: ops.resid_rmsnorm(x, w, 1e-6), 3)
        add("like: RMS norm of the stream", phase, ms, 0.0, T * D * 6.0, "hbm")
        hist, cw = rnd(5, T, D), rnd(5)
        ms = _time(lambda: ops.depth_mix(hist, cw), 3)
        add("depth-weighted sum of 5 streams", phase, ms, 0.0, 6.0 * T * D * 4.0, "hbm")
        y = rnd(T, D)
        ms = _time(lambda: ops.resid_add_rmsnorm(x, y, w, 1e-6), 3)
        add("like: norm + residual sum", phase, ms, 0.0, 3.0 * T * D * 4.0, "hbm")
        del x, hist, y
        torch.cuda.empty_cache()
    return rows


def run(size="w2048", layers=4, prefill=4096, batch=32, ctx=2048, reps=5):
    import json
    from pathlib import Path

    from . import models
    pk = Path(__file__).resolve().parent.parent / "MEASURED_PEAKS.json"
    peaks = json.loads(pk.read_text()) if pk.exists() else {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}
    s = SIZES[size]
    res = {"size": size, "layers": layers, "order": ORDER[:layers], "prefill_tokens": prefill, "decode_batch": batch,
           "decode_context": ctx}
    nblk = (max(prefill, ctx) + 63) // 64
    mp, md = _meta(1, prefill, prefill, nblk, s["vocab"]), _meta(batch, 1, ctx, nblk, s["vocab"])
    zcfg = bench_zalalix.config(size, layers)
    arms = (("tasadra", config(size, layers), random_tensors),
            ("zalalix", zcfg, lambda c: bench_zalalix.random_tensors(c, size)))
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
