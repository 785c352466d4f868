"""Runner of hybrid decoders with an fp32 residual stream over the C++ launch plan (b200_hybrid_*,
csrc/host/hybrid_runner.cpp): the sibling of engine.ModelRunner for models whose layers choose between latent
attention, windowed softmax attention, the gated delta rule, the SSD scan and decayed linear attention (one mixer, or
two side by side), with a routed mixture of experts or a dense feed-forward, in a parallel, a sandwich
(norm before and after each sublayer), a post-norm (sublayer results normed on their way into the stream) or a
pre-norm layout (RMS or dynamic-tanh norms, optional token shift and depth-weighted average of the layers' results).

This module holds no model arithmetic.  It allocates what the C side borrows -- the paged latent caches, the
paged K / V caches, the slot-indexed recurrent state pools, the workspace, pinned staging -- describes the layers to it, and moves a step's
metadata and results.  A model file (vllm_rs_b200/models/*.py) turns a checkpoint into `LayerSpec`s.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np
import torch

from . import _lib
from ._lib import HybridConfig, HybridLayer

MIXER_LATENT_ATTN, MIXER_DELTA_RULE, MIXER_SSD, MIXER_WINDOW_ATTN, MIXER_DECAY_ATTN = 0, 1, 2, 3, 4
LAYOUT_PARALLEL, LAYOUT_SANDWICH, LAYOUT_POSTNORM, LAYOUT_PRENORM = 0, 1, 2, 3
NORM_RMS, NORM_DYNTANH = 0, 1
PAGE = 64


@dataclass
class LayerSpec:
    """One layer: integer / float fields of b200_hybrid_layer by name, and its tensors by field name.  Matrix-product
    weights must be in the runner's operand dtype, small parameters fp32, rot_freq float64; all on the device."""
    mixer: int
    dims: dict
    tensors: dict = field(default_factory=dict)
    side: "LayerSpec | None" = None      # a second mixer beside the first (reads the same norm; outputs are summed)
    cache_from: "int | None" = None      # latent / window attention: read layer cache_from's cache (no cache of its own)


class HybridRunner:
    def __init__(self, *, width, vocab, layers: list[LayerSpec], embed, final_norm, lm_head, norm_eps,
                 norm_weight_offset=0.0, embed_scale=1.0, embed_pos_base=0.0, dtype=torch.bfloat16, num_blocks, max_blocks_per_seq, max_seqs, max_tokens,
                 num_state_slots, device="cuda", layer_trace=False, final_norm_kind=NORM_RMS, final_norm_bias=None,
                 final_norm_alpha=1.0):
        if dtype not in (torch.bfloat16, torch.float32):
            raise ValueError("hybrid decoders run with bfloat16 or float32 operands")
        self._l = _lib.lib()
        self.device = torch.device(device)
        self.dtype = dtype
        self.cfg = HybridConfig(width=width, vocab=vocab, num_layers=len(layers), dt=int(dtype == torch.float32),
                                block_size=PAGE, num_blocks=num_blocks, max_blocks_per_seq=max_blocks_per_seq,
                                max_seqs=max_seqs, max_tokens=max_tokens, num_state_slots=num_state_slots,
                                norm_eps=norm_eps, norm_weight_offset=norm_weight_offset, embed_scale=embed_scale,
                                embed_pos_base=embed_pos_base, final_norm_kind=final_norm_kind)
        self._h = self._l.b200_hybrid_new(C.byref(self.cfg))
        _lib.check()
        self._keep = [embed, final_norm, lm_head, final_norm_bias]
        self.kv_cache, self.v_cache, self.conv_state, self.rec_state, self.shift_state = {}, {}, {}, {}, {}
        f32 = dict(dtype=torch.float32, device=self.device)

        def describe(key, spec):
            """The C description of one mixer; allocates the caches / state pools it needs under `key`."""
            d, t = spec.dims, dict(spec.tensors)
            if spec.mixer == MIXER_LATENT_ATTN and spec.cache_from is not None:
                src = spec.cache_from
                if not (isinstance(key, int) and 0 <= src < key and layers[src].mixer == MIXER_LATENT_ATTN and
                        layers[src].cache_from is None and
                        layers[src].dims["kv_rank"] + layers[src].dims["rot_dim"] == d["kv_rank"] + d["rot_dim"]):
                    raise ValueError(f"layer {key}: a shared latent cache comes from an earlier latent-attention layer "
                                     "of the same row size that writes its own")
                t["kv_cache"] = self.kv_cache[src]
                d = {**d, "shared_cache": 1}
            elif spec.mixer == MIXER_LATENT_ATTN:
                self.kv_cache[key] = torch.zeros(num_blocks, PAGE, d["kv_rank"] + d["rot_dim"], dtype=dtype,
                                                 device=self.device)
                t["kv_cache"] = self.kv_cache[key]
            elif spec.mixer == MIXER_WINDOW_ATTN and spec.cache_from is not None:
                src = spec.cache_from
                same = ("kv_heads", "dim", "vdim", "score_maps")
                if not (isinstance(key, int) and 0 <= src < key and layers[src].mixer == MIXER_WINDOW_ATTN and
                        layers[src].cache_from is None and
                        all(layers[src].dims.get(n, 0) == d.get(n, 0) for n in same)):
                    raise ValueError(f"layer {key}: shared K / V pages come from an earlier attention layer of the same "
                                     "head counts and sizes that writes its own")
                t["kv_cache"], t["v_cache"] = self.kv_cache[src], self.v_cache[src]
                d = {**d, "shared_cache": 1}
            elif spec.mixer == MIXER_WINDOW_ATTN:
                maps = max(int(d.get("score_maps", 0)), 1)      # the maps' key heads lie one map after the other
                self.kv_cache[key] = torch.zeros(num_blocks, PAGE, maps * d["kv_heads"], d["dim"], dtype=dtype,
                                                 device=self.device)
                self.v_cache[key] = torch.zeros(num_blocks, PAGE, d["kv_heads"], d["vdim"], dtype=dtype, device=self.device)
                t["kv_cache"], t["v_cache"] = self.kv_cache[key], self.v_cache[key]
            elif spec.mixer == MIXER_DECAY_ATTN:
                self.rec_state[key] = torch.zeros(num_state_slots, d["heads"], d["dim"], d["vdim"], **f32)
                t["rec_state"] = self.rec_state[key]
            else:
                taps = d["conv_taps"]
                if spec.mixer == MIXER_DELTA_RULE:
                    nconv = 2 * d["kv_heads"] * d["dim"] + d["heads"] * d["vdim"]
                    rows = d["dim"]
                else:
                    nconv = d["heads"] * d["vdim"] + 2 * d["kv_heads"] * d["state"]
                    rows = d["state"]
                self.conv_state[key] = torch.zeros(num_state_slots, max(taps - 1, 1), nconv, **f32)
                self.rec_state[key] = torch.zeros(num_state_slots, d["heads"], rows, d["vdim"], **f32)
                t["conv_state"], t["rec_state"] = self.conv_state[key], self.rec_state[key]
            if t.get("shift_w") is not None:     # the previous token's normed row, per sequence
                self.shift_state[key] = torch.zeros(num_state_slots, width, **f32)
                t["shift_state"] = self.shift_state[key]
            lw = HybridLayer(mixer=spec.mixer, **{"out_scale": 1.0, "q_scale": 1.0, "k_scale": 1.0, "ff_scale": 1.0, **d})
            for name, ten in t.items():
                if ten is None:
                    continue
                if not ten.is_cuda or not ten.is_contiguous():
                    raise ValueError(f"layer {key}: tensor {name} must be a contiguous device tensor")
                setattr(lw, name, ten.data_ptr())
            self._keep.append(t)
            return lw

        for i, spec in enumerate(layers):
            self._l.b200_hybrid_set_layer(self._h, i, C.byref(describe(i, spec)))
            _lib.check()
            if spec.side is not None:
                self._l.b200_hybrid_set_layer_side(self._h, i, C.byref(describe((i, "side"), spec.side)))
                _lib.check()
        self._l.b200_hybrid_set_globals(self._h, embed.data_ptr(), final_norm.data_ptr(), lm_head.data_ptr())
        if final_norm_kind != NORM_RMS:
            self._l.b200_hybrid_set_final_norm(self._h, 0 if final_norm_bias is None else final_norm_bias.data_ptr(),
                                               float(final_norm_alpha))
        nbytes = self._l.b200_hybrid_workspace_bytes(self._h)
        self.workspace = torch.zeros(nbytes, dtype=torch.uint8, device=self.device)
        self._l.b200_hybrid_set_workspace(self._h, self.workspace.data_ptr(), nbytes)
        _lib.check()
        self.trace = None
        if layer_trace:
            self.trace = torch.zeros(len(layers), max_tokens, width, **f32)
            self._l.b200_hybrid_set_layer_trace(self._h, self.trace.data_ptr())
        T, B, mb = max_tokens, max_seqs, max_blocks_per_seq

        def pin(n, dt):
            return torch.zeros(n, dtype=dt).pin_memory().numpy()

        self.pinned = dict(input_ids=pin(T, torch.int32).view(np.uint32), positions=pin(T, torch.int64),
                           slot_mapping=pin(T, torch.int64), cu_seqlens_q=pin(B + 1, torch.int32).view(np.uint32),
                           context_lens=pin(B, torch.int32).view(np.uint32),
                           block_tables=pin(B * mb, torch.int32).view(np.uint32), state_slots=pin(B, torch.int32))
        self.out_rows = pin(T, torch.int32).view(np.uint32)
        self.out_ids = pin(T, torch.int32).view(np.uint32)
        self.out_logits = None          # pinned [rows, vocab], grown on demand
        # steps run on a stream of their own (small steps are replayed as CUDA graphs, which the legacy default
        # stream cannot capture); everything above was issued on the current stream
        self.stream = torch.cuda.Stream(device=self.device)
        torch.cuda.synchronize(self.device)

    def __del__(self):
        if getattr(self, "_h", None):
            self._l.b200_hybrid_free(self._h)
            self._h = None

    def set_sampling(self, strategy=0, k=0, p=1.0, t=1.0):
        """strategy as b200_sampling_strategy returns it: 0 greedy, 1 whole vocabulary, 2-4 top-k / top-p."""
        rc = self._l.b200_hybrid_set_sampling(self._h, int(strategy), int(k), float(p), float(t))
        _lib.check()
        assert rc == 0

    def set_step_seed(self, seed, stream=None):
        st = stream if stream is not None else self.stream.cuda_stream
        self._l.b200_hybrid_set_step_seed(self._h, int(seed) & ((1 << 64) - 1), st)
        _lib.check()

    def step(self, meta, out_rows, want_logits=False, want_ids=True):
        """One ragged step from Scheduler.prepare_ragged metadata (host, ideally this runner's pinned buffers).
        out_rows: token rows whose logits / sampled ids are wanted.  Returns (logits f32 numpy [rows, vocab] | None,
        ids uint32 numpy [rows] | None)."""
        B, T, R = meta["num_seqs"], meta["num_tokens"], len(out_rows)
        self.out_rows[:R] = np.asarray(out_rows, dtype=np.uint32)
        lg = None
        if want_logits and R:
            need = R * self.cfg.vocab
            if self.out_logits is None or self.out_logits.size < need:
                self.out_logits = torch.zeros(need, dtype=torch.float32).pin_memory().numpy()
            lg = self.out_logits[:need].reshape(R, self.cfg.vocab)
        self.stream.wait_stream(torch.cuda.current_stream(self.device))     # e.g. caches filled by the caller
        rc = self._l.b200_hybrid_step_host(
            self._h, meta["input_ids"].ctypes.data, meta["positions"].ctypes.data, meta["slot_mapping"].ctypes.data,
            meta["cu_seqlens_q"].ctypes.data, meta["context_lens"].ctypes.data, meta["block_tables"].ctypes.data,
            meta["state_slots"].ctypes.data, self.out_rows.ctypes.data, B, T, meta["max_blocks"], R,
            0 if lg is None else lg.ctypes.data, self.out_ids.ctypes.data if (want_ids and R) else 0,
            self.stream.cuda_stream)
        _lib.check()
        if rc != 0:
            raise _lib.B200Error("hybrid step failed")
        return lg, (self.out_ids[:R].copy() if want_ids else None)

    @property
    def launches_per_step(self):
        return self._l.b200_hybrid_launches_per_step(self._h)
