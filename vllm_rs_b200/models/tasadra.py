"""Tasadra checkpoints -> hybrid.HybridRunner.

config.json: {"architecture": "Tasadra", "width", "vocab", "residual_mult", "norm": {"eps"}, "layers": [{"type",
"mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}, ...]}; tensors are named "embed", "l<i>.norm1" (+ ".b",
".alpha"), "l<i>.norm2", "l<i>.shift", "l<i>.dwa", "l<i>.mix.*", "l<i>.mlp.*", "final.norm", "head"; linear weights
[out, in].  Every layer is pre-norm with dynamic-tanh norms (tanh(alpha x) w + b), both sublayers are added to the
stream times residual_mult, the mixer reads its normed input through a token shift (h[t] + (h[t-1] - h[t]) * shift),
and after each layer the stream is replaced by a weighted sum (l<i>.dwa) of the embedding and all layer results so far.
Mixer types:
  attention     : softmax attention with grouped key / value heads, RMS norm per q / k head with one weight shared by the
                  heads, rotary positions in the two-halves layout with YaRN frequency scaling, capped scores, values
                  that are rotated by their position before they are cached and turned back by the query's position
                  after the weighted sum, a sigmoid gate per head
  channel_delta : the gated delta rule behind short convolutions, with one decay per head and key channel from a
                  low-rank projection and a low-rank sigmoid output gate
  attention_2   : differential attention (two score maps over one set of values, a_1 - lambda a_2, RMS norm per head,
                  a gate per element) under a chunked causal mask, without positions; with `kv_from` the layer has no
                  key / value projections and reads that earlier layer's pages
Feed-forward: W_down relu(W_up h + b_up)^2 + b_down.
This file only arranges weights for the launch plan (fused input projections, the maps of differential attention laid
out one after the other, fp32 small parameters, frequency tables, lambda); the arithmetic is in the CUDA kernels."""
from __future__ import annotations

import math

import numpy as np
import torch

from ..hybrid import (LAYOUT_PRENORM, MIXER_DELTA_RULE, MIXER_WINDOW_ATTN, NORM_DYNTANH, HybridRunner, LayerSpec)
from ..rotary import rotary_frequencies
from . import register

_ZERO = dict(heads=0, kv_heads=0, dim=0, rot_dim=0, rot_dims=0, vdim=0, kv_rank=0, window=0, state=0, conv_taps=0,
             norm_groups=0, scale=0.0, rot_mag=1.0, experts=0, top=0, expert_ff=0, shared_ff=0, route_scale=1.0,
             layout=LAYOUT_PRENORM, out_scale=1.0, gated=0, norm_kind=NORM_DYNTANH)


def map_major(w: torch.Tensor, heads: int, maps: int, dim: int) -> torch.Tensor:
    """Rows stored head by head as [map 0 | map 1 | ...] -> all heads of map 0, then all heads of map 1, ..."""
    return w.reshape(heads, maps, dim, -1).transpose(0, 1).reshape(heads * maps * dim, -1)


def differential_lambda(lq1, lk1, lq2, lk2, diff: float) -> float:
    """exp(lq1 . lk1) - exp(lq2 . lk2) + diff, in double."""
    d = lambda a, b: float((a.to(torch.float64) * b.to(torch.float64)).sum())      # noqa: E731
    return math.exp(d(lq1, lk1)) - math.exp(d(lq2, lk2)) + float(diff)


@register("Tasadra")
def build(cfg, tensors, *, dtype=torch.bfloat16, device="cuda", num_blocks, max_blocks_per_seq, max_seqs, max_tokens,
          num_state_slots=None, layer_trace=False, **_):
    dtype = dtype or torch.bfloat16
    dev = torch.device(device)
    width, mult = int(cfg["width"]), float(cfg.get("residual_mult", 1.0))

    def mat(*ts):                         # matrix-product operand(s), fused along the output rows
        ts = [tensors[t] if isinstance(t, str) else t for t in ts]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(dtype).contiguous().to(dev)

    def vec(*names):                      # small parameters stay fp32
        ts = [tensors[n].to(torch.float32).reshape(-1) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).contiguous().to(dev)

    def f64(a):
        return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float64)).to(dev)

    def norm(name, prefix):               # a dynamic-tanh norm: weight, bias, the scalar inside the tanh
        return {prefix + "_w": vec(name), prefix + "_b": vec(name + ".b") if name + ".b" in tensors else None}, \
            float(tensors[name + ".alpha"].to(torch.float32))

    specs = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        d = dict(_ZERO, out_scale=mult, ff_scale=mult)
        t, d["norm_alpha"] = norm(f"l{i}.norm1", "norm")
        if f"l{i}.shift" in tensors:
            t["shift_w"] = vec(f"l{i}.shift")
        if f"l{i}.dwa" in tensors:
            if tensors[f"l{i}.dwa"].numel() != i + 2:
                raise ValueError(f"layer {i}: the depth weights cover the embedding and the results of layers 0 .. {i}")
            t["depth_w"] = vec(f"l{i}.dwa")
        cache_from = None
        if kind == "attention":
            mixer = MIXER_WINDOW_ATTN
            H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            rot = m.get("rot") or {}
            rd = int(rot.get("dims", 0))
            d.update(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=float(m["scale"]), softcap=float(m.get("softcap") or 0.0),
                     gated=1, head_norm=1, rot_dims=rd, rot_half=1)
            t.update(w_in=mat(p + "q", p + "k", p + "v", p + "g"), w_o=mat(p + "o"), q_norm_w=vec(p + "q.norm"),
                     k_norm_w=vec(p + "k.norm"))
            if rd:
                freq, mag = rotary_frequencies(rd, float(rot["base"]), rot.get("scaling"))
                d["rot_mag"] = float(mag)
                t["rot_freq"] = f64(freq)
            if rot:                       # values turn with the plain frequencies over all of vdim, whatever the keys use
                if dv % 2:
                    raise ValueError(f"layer {i}: rotated values need an even vdim")
                t["v_rot_freq"] = f64(rotary_frequencies(dv, float(rot["base"]))[0])
        elif kind == "channel_delta":
            mixer = MIXER_DELTA_RULE
            H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            d.update(heads=H, kv_heads=G, dim=dk, vdim=dv, conv_taps=int(m["conv"]), gate_act=1,
                     chan_rank=int(tensors[p + "a1"].shape[0]), gate_rank=int(tensors[p + "g1"].shape[0]))
            t.update(w_in=mat(p + "q", p + "k", p + "v", p + "b", p + "a1", p + "g1"), w_o=mat(p + "o"),
                     conv_w=vec(p + "q.conv", p + "k.conv", p + "v.conv"), a_log=vec(p + "A_log"),
                     dt_bias=vec(p + "dt_bias"), out_norm_w=vec(p + "norm"),
                     w_decay2=tensors[p + "a2"].to(torch.float32).contiguous().to(dev),
                     w_gate2=tensors[p + "g2"].to(torch.float32).contiguous().to(dev))
        elif kind == "attention_2":
            mixer = MIXER_WINDOW_ATTN
            H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            diff = float(m.get("diff", 0.0))
            d.update(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=float(m["scale"]), gated=2, score_maps=2,
                     chunk=int((m.get("mask") or {}).get("size", 0)), diff_norm=1, diff_out_scale=1.0 - diff,
                     diff_lambda=differential_lambda(tensors[p + "lq1"], tensors[p + "lk1"], tensors[p + "lq2"],
                                                     tensors[p + "lk2"], diff))
            q = map_major(tensors[p + "q"], H, 2, dk)
            if m.get("kv_from") is not None:
                cache_from = int(m["kv_from"])
                src = cfg["layers"][cache_from] if 0 <= cache_from < i else None
                if src is None or src["type"] != kind or src["mixer"].get("kv_from") is not None:
                    raise ValueError(f"layer {i}: kv_from must name an earlier layer of the same type with key / value "
                                     "projections of its own")
                t.update(w_in=mat(q, p + "g"))
            else:
                t.update(w_in=mat(q, map_major(tensors[p + "k"], G, 2, dk), p + "v", p + "g"))
            t.update(w_o=mat(p + "o"))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] != "dense":
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
            q = f"l{i}.mlp."
            n2, d["ff_norm_alpha"] = norm(f"l{i}.norm2", "ff_norm")
            t.update(n2)
            d.update(shared_ff=int(mlp["ff"]), shared_act=1)
            t.update(w_shared_gate_up=mat(q + "up"), w_shared_down=mat(q + "down"),
                     ff_up_bias=vec(q + "up.b") if q + "up.b" in tensors else None,
                     ff_down_bias=vec(q + "down.b") if q + "down.b" in tensors else None)
        specs.append(LayerSpec(mixer, d, t, cache_from=cache_from))
    fin, alpha = norm("final.norm", "f")
    return HybridRunner(width=width, vocab=int(cfg["vocab"]), layers=specs, embed=mat("embed"), final_norm=fin["f_w"],
                        lm_head=mat("head"), norm_eps=float(cfg["norm"]["eps"]), norm_weight_offset=0.0, dtype=dtype,
                        num_blocks=num_blocks, max_blocks_per_seq=max_blocks_per_seq, max_seqs=max_seqs,
                        max_tokens=max_tokens, num_state_slots=num_state_slots or max_seqs, device=device,
                        layer_trace=layer_trace, final_norm_kind=NORM_DYNTANH, final_norm_bias=fin["f_b"],
                        final_norm_alpha=alpha)
