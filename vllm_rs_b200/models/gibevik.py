"""Gibevik checkpoints -> hybrid.HybridRunner.

config.json: {"architecture": "Gibevik", "width", "vocab", "norm": {"eps"}, "layers": [{"type", "mixer": {...},
"mlp": {...} | null}, ...]}; tensors are named "embed", "l<i>.norm1", "l<i>.norm2", "l<i>.mix.*", "l<i>.mlp.*",
"final.norm", "head", linear weights [out, in].  A sinusoidal position vector joins the embedding row, and every layer
is post-norm: x += norm1(mixer(x)), then x += norm2(ff(x)), with x going into the sublayers un-normed.  Mixer types:
  attention        : softmax attention with grouped key heads whose raw, un-normed rows double as the values (no value
                     projection), RMS norm per q / k head with one weight shared by the heads, no rotation, a query
                     temperature that grows with the logarithm of the position, a linear distance bias with one fixed
                     slope per head, and an output gate per element
  latent_attention : latent (compressed key / value) attention without positions and with a gate per head; with
                     `kv_from` the layer has no latent projection and reads that earlier layer's cached latents
Feed-forward kinds: `dense` (SiLU-gated) and `moe`: ungated squared-ReLU experts behind a softmax router whose choice
uses a correction bias and groups of neighbouring experts, with identity experts and a sigmoid-gated shared expert.
This file only arranges weights for the launch plan (fused input projections, stacked experts, fp32 small parameters,
the heads' slopes); the arithmetic is in the CUDA kernels."""
from __future__ import annotations

import torch

from ..hybrid import LAYOUT_POSTNORM, MIXER_LATENT_ATTN, MIXER_WINDOW_ATTN, HybridRunner, LayerSpec
from . import register

POSITION_BASE = 10000.0           # wavelengths of the sinusoidal position vector grow geometrically up to 2 pi base
SLOPE_EXPONENT = 8.0              # head h of H takes the slope 2^(-SLOPE_EXPONENT (h + 1) / H)

_ZERO = dict(heads=0, kv_heads=0, dim=0, rot_dim=0, rot_dims=0, vdim=0, kv_rank=0, window=0, state=0, conv_taps=0,
             norm_groups=0, scale=0.0, rot_mag=1.0, experts=0, top=0, expert_ff=0, shared_ff=0, route_scale=1.0,
             layout=LAYOUT_POSTNORM, out_scale=1.0, gated=0)


def head_slopes(heads: int) -> torch.Tensor:
    """slope_h = 2^(-8 (h + 1) / H), h = 0 .. H - 1 (fp32)."""
    h = torch.arange(1, heads + 1, dtype=torch.float64)
    return torch.pow(torch.tensor(2.0, dtype=torch.float64), -SLOPE_EXPONENT * h / heads).to(torch.float32)


@register("Gibevik")
def build(cfg, tensors, *, dtype=torch.bfloat16, device="cuda", num_blocks, max_blocks_per_seq, max_seqs, max_tokens,
          num_state_slots=None, layer_trace=False, **_):
    dtype = dtype or torch.bfloat16
    dev = torch.device(device)

    def mat(*names):                      # matrix-product operand(s), fused along the output rows
        ts = [tensors[n] for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).to(dtype).contiguous().to(dev)

    def vec(*names):                      # small parameters stay fp32
        ts = [tensors[n].to(torch.float32).reshape(-1) for n in names]
        return (torch.cat(ts, 0) if len(ts) > 1 else ts[0]).contiguous().to(dev)

    specs = []
    for i, layer in enumerate(cfg["layers"]):
        p, m, kind = f"l{i}.mix.", layer["mixer"], layer["type"]
        d, t = dict(_ZERO), {"post_norm_w": vec(f"l{i}.norm1")}
        cache_from = None
        if kind == "attention":
            mixer = MIXER_WINDOW_ATTN
            H, G, dk, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
            if dv != dk:
                raise ValueError(f"layer {i}: the raw key rows serve as values, so vdim must equal dim")
            qt = m.get("q_temp") or {}
            d.update(heads=H, kv_heads=G, dim=dk, vdim=dv, scale=float(m["scale"]), gated=2, head_norm=1, v_from_k=1,
                     q_temp_every=int(qt.get("every", 0)), q_temp_coef=float(qt.get("coef", 0.0)))
            t.update(w_in=mat(p + "q", p + "k", p + "g"), w_o=mat(p + "o"), q_norm_w=vec(p + "q.norm"),
                     k_norm_w=vec(p + "k.norm"), dist_slopes=head_slopes(H).to(dev))
        elif kind == "latent_attention":
            mixer = MIXER_LATENT_ATTN
            H = int(m["heads"])
            d.update(heads=H, dim=int(m["dim"]), vdim=int(m["vdim"]), kv_rank=int(m["kv_rank"]), scale=float(m["scale"]),
                     gated=1)
            if m.get("kv_from") is not None:
                cache_from = int(m["kv_from"])
                src = cfg["layers"][cache_from] if 0 <= cache_from < i else None
                if (src is None or src["type"] != "latent_attention" or src["mixer"].get("kv_from") is not None or
                        int(src["mixer"]["kv_rank"]) != d["kv_rank"]):
                    raise ValueError(f"layer {i}: kv_from must name an earlier latent-attention layer with a latent "
                                     "projection of its own and the same kv_rank")
                t.update(w_in=mat(p + "q", p + "g"))
            else:
                t.update(w_in=mat(p + "q", p + "dkv", p + "g"), latent_norm_w=vec(p + "dkv.norm"))
            t.update(w_uk=mat(p + "uk"), w_uv=mat(p + "uv"), w_o=mat(p + "o"))
        else:
            raise ValueError(f"layer {i}: unknown mixer type {kind!r}")
        mlp = layer.get("mlp")
        if mlp:
            q = f"l{i}.mlp."
            t["ff_post_norm_w"] = vec(f"l{i}.norm2")
            if mlp["kind"] == "dense":
                d["shared_ff"] = int(mlp["ff"])
                t.update(w_shared_gate_up=mat(q + "gate", q + "up"), w_shared_down=mat(q + "down"))
            elif mlp["kind"] == "moe":
                r = mlp["router"]
                E, ident = int(r["experts"]), int(r.get("identity", 0))
                groups = r.get("groups") or {}
                d.update(experts=E, identity_experts=ident, top=int(r["top"]), expert_ff=int(mlp["expert"]["ff"]),
                         expert_act=1, route_groups=int(groups.get("count", 0)), route_keep=int(groups.get("keep", 0)))
                if tuple(tensors[q + "router"].shape) != (E + ident, cfg["width"]):
                    raise ValueError(f"layer {i}: the router has one output per expert and identity expert")
                t.update(w_router=mat(q + "router"),
                         w_gate_up=torch.stack([mat(f"{q}e{e}.up") for e in range(E)]).contiguous(),
                         w_down=torch.stack([mat(f"{q}e{e}.down") for e in range(E)]).contiguous(),
                         route_bias=vec(q + "correction") if q + "correction" in tensors else None)
                if mlp.get("shared"):
                    gated = q + "shared.sg" in tensors
                    d.update(shared_ff=int(mlp["shared"]["ff"]), shared_act=1, shared_gated=int(gated))
                    t.update(w_shared_gate_up=mat(*([q + "shared.up"] + ([q + "shared.sg"] if gated else []))),
                             w_shared_down=mat(q + "shared.down"))
            else:
                raise ValueError(f"layer {i}: unknown feed-forward kind {mlp['kind']!r}")
        specs.append(LayerSpec(mixer, d, t, cache_from=cache_from))
    return HybridRunner(width=cfg["width"], vocab=cfg["vocab"], layers=specs, embed=mat("embed"),
                        final_norm=vec("final.norm"), lm_head=mat("head"), norm_eps=float(cfg["norm"]["eps"]),
                        norm_weight_offset=0.0, embed_pos_base=POSITION_BASE, dtype=dtype, num_blocks=num_blocks,
                        max_blocks_per_seq=max_blocks_per_seq, max_seqs=max_seqs, max_tokens=max_tokens,
                        num_state_slots=num_state_slots or max_seqs, device=device, layer_trace=layer_trace)
