"""Host-side operator layer over the C ABI (torch tensors are only memory + streams).

Names follow the reference's layer vocabulary (src/models/layers/*.rs): WNA16 repack +
gptq_matmul, FusedRope, PagedAttention, rms_norm ...  Every function launches hand-written
sm_100a kernels from libb200_vllm.so; there is no CPU or eager-torch fallback.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib

QFMT_AWQ, QFMT_GPTQ = 0, 1
EPI_NONE, EPI_SILU_MUL = 0, 1
VARIANT_AUTO, VARIANT_GEMV, VARIANT_TC = 0, 1, 2


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _p(t):
    return 0 if t is None else t.data_ptr()


def _sym(stem: str, t: torch.Tensor):
    """The `_f16` or `_bf16` flavour of an entry point, by the dtype of the activations (bf16 is the reference's
    default dtype, utils/mod.rs:1919-1925)."""
    if t.dtype == torch.bfloat16:
        return getattr(_lib.lib(), stem + "_bf16")
    if t.dtype != torch.float16:
        raise TypeError(f"{stem}: activations must be fp16 or bf16, got {t.dtype}")
    return getattr(_lib.lib(), stem + "_f16")


def _cuda(*ts):
    for t in ts:
        if t is not None and not (t.is_cuda and t.is_contiguous()):
            raise ValueError("b200 ops need contiguous CUDA tensors")


# ------------------------------------------------------------------ quantised linear
def awq_prepack(qweight: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """MarlinRepack for AWQ (gptq.rs:314-324): qweight i32 [K, N/8] -> tile-major u32."""
    _cuda(qweight)
    out = torch.empty_like(qweight)
    _lib.lib().b200_awq_prepack(_p(qweight), _p(out), qweight.shape[0], qweight.shape[1], bits,
                                _stream())
    _lib.check()
    return out


def gptq_prepack(qweight: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """MarlinRepack for GPTQ (gptq.rs:325-333): qweight i32 [K/pack, N] -> tile-major u32."""
    _cuda(qweight)
    out = torch.empty_like(qweight)
    _lib.lib().b200_gptq_prepack(_p(qweight), _p(out), qweight.shape[0], qweight.shape[1], bits,
                                 _stream())
    _lib.check()
    return out


def wna16_workspace(max_m: int, max_n: int, device="cuda") -> torch.Tensor:
    n = _lib.lib().b200_wna16_workspace_bytes(max_m, max_n)
    return torch.zeros(n, dtype=torch.uint8, device=device)


def wna16_gemm(x, w_packed, scales, qzeros, workspace, *, k: int, n: int, bits=4, group_size=128,
               qfmt=QFMT_AWQ, bias=None, epilogue=EPI_NONE, variant=VARIANT_AUTO, out=None):
    """gptq_matmul (gptq.rs:243-263): y[M, N] = x[M, K] @ dequant(W)."""
    _cuda(x, w_packed, scales, qzeros, bias, workspace)
    m = x.shape[0]
    n_out = n // 2 if epilogue == EPI_SILU_MUL else n
    if out is None:
        out = torch.empty(m, n_out, dtype=torch.float16, device=x.device)
    _lib.lib().b200_wna16_gemm_ex(_p(x), _p(w_packed), _p(scales), _p(qzeros), _p(bias), _p(out),
                                  m, k, n, bits, group_size, qfmt, epilogue, variant,
                                  _p(workspace), _stream())
    _lib.check()
    return out


DENSE_AUTO, DENSE_CUBLAS, DENSE_TC1, DENSE_TC2 = -1, 0, 1, 2


def dense_gemm(x, w_nk, out_f32=False, out=None, bias=None, mode=DENSE_AUTO):
    """Linear::forward (linear.rs:75-123): y = x @ W^T (+ bias), W [N, K] fp16."""
    _cuda(x, w_nk, bias)
    m, k = x.shape
    n = w_nk.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32 if out_f32 else torch.float16, device=x.device)
    _lib.lib().b200_dense_gemm_ex(_p(x), _p(w_nk), _p(bias), _p(out), m, n, k, int(out_f32), mode, _stream())
    _lib.check()
    return out


def wna16_dequant(w_packed, scales, qzeros, *, k: int, n: int, bits=4, group_size=128, qfmt=QFMT_AWQ, out=None):
    """Prepacked W4 / W8 weight -> fp16 [N, K] (the weight operand of dense_gemm)."""
    _cuda(w_packed, scales, qzeros)
    if out is None:
        out = torch.empty(n, k, dtype=torch.float16, device=w_packed.device)
    _lib.lib().b200_wna16_dequant_f16(_p(w_packed), _p(scales), _p(qzeros), _p(out), k, n, bits, group_size,
                                      qfmt, _stream())
    _lib.check()
    return out


# ------------------------------------------------------------------ attention side
def _is_l1(k_cache, v_cache) -> bool:
    """The reference's default-build layout (kvcache_allocator.rs:150-173): K [nb, Hkv, D/8, 64, 8] is 5-D."""
    return k_cache is not None and k_cache.dim() == 5


def rope_kv_write(q, k, v, cos, sin, positions, slot_mapping=None, k_cache=None, v_cache=None,
                  rot_dim=None, interleaved=False):
    """FusedRope::apply_inplace + cache write (rotary_emb.rs:88-104, attention.rs:808-820)."""
    _cuda(q, k, v, cos, sin, positions, slot_mapping, k_cache, v_cache)
    T, H, D = q.shape
    Hkv = k.shape[1]
    if _is_l1(k_cache, v_cache):
        _lib.lib().b200_rope_kv_write_l1(
            _p(q), _p(k), _p(v), _p(cos), _p(sin), _p(positions), _p(slot_mapping), _p(k_cache), _p(v_cache), T, H,
            Hkv, D, rot_dim or D, k_cache.shape[3], int(interleaved), int(cos.dtype == torch.float32),
            int(q.dtype == torch.bfloat16), _stream())
        _lib.check()
        return
    bs = k_cache.shape[1] if k_cache is not None else 64
    fp8 = k_cache is not None and k_cache.dtype == torch.uint8        # --fp8-kvcache: e4m3 bytes
    fn = _lib.lib().b200_rope_kv_write_fp8kv_f16 if fp8 else _sym("b200_rope_kv_write", q)
    fn(
        _p(q), _p(k), _p(v), _p(cos), _p(sin), _p(positions), _p(slot_mapping), _p(k_cache),
        _p(v_cache), T, H, Hkv, D, rot_dim or D, bs, int(interleaved),
        int(cos.dtype == torch.float32), _stream())
    _lib.check()


def kv_write(k, v, k_cache, v_cache, slot_mapping):
    _cuda(k, v, k_cache, v_cache, slot_mapping)
    T, Hkv, D = k.shape
    if _is_l1(k_cache, v_cache):
        _lib.lib().b200_kv_write_l1(_p(k), _p(v), _p(k_cache), _p(v_cache), _p(slot_mapping), T, Hkv, D,
                                    k_cache.shape[3], _stream())
        _lib.check()
        return
    _lib.lib().b200_kv_write_f16(_p(k), _p(v), _p(k_cache), _p(v_cache), _p(slot_mapping), T, Hkv,
                                 D, k_cache.shape[1], _stream())
    _lib.check()


def swap_blocks(src_cache, dst_cache, mapping):
    """attention_rs::cache::swap_blocks (runner.rs:1626-1645): dst[d] = src[s] for every (s, d) of `mapping`
    (dict or list of pairs).  Caches are [num_blocks, ...] tensors on the GPU or in PINNED host memory."""
    pairs = list(mapping.items()) if isinstance(mapping, dict) else list(mapping)
    if not pairs:
        return
    for t in (src_cache, dst_cache):
        assert t.is_contiguous() and (t.is_cuda or t.is_pinned()), "caches must be CUDA or pinned host tensors"
    block_bytes = src_cache[0].numel() * src_cache.element_size()
    assert block_bytes == dst_cache[0].numel() * dst_cache.element_size()
    dev = src_cache.device if src_cache.is_cuda else dst_cache.device
    pd = torch.tensor(pairs, dtype=torch.int64).to(dev)
    _lib.lib().b200_swap_blocks(_p(src_cache), _p(dst_cache), _p(pd), len(pairs), block_bytes, _stream())
    _lib.check()
    return pd            # keep alive until the stream has run the copy


def paged_attn_workspace(batch, num_heads, head_dim, max_blocks, device="cuda"):
    n = _lib.lib().b200_paged_attn_workspace_bytes(batch, num_heads, head_dim, max_blocks)
    return torch.zeros(n, dtype=torch.uint8, device=device)     # arrival counters start at rest


def paged_attention_decode(q, k_cache, v_cache, block_tables, context_lens, scale, workspace=None,
                           softcap=0.0, window=0, out=None):
    """PagedAttention::forward, decode branch.  q [B,H,D]; caches [nb, 64, Hkv, D];
    block_tables u32/i32 [B, max_blocks]; context_lens u32/i32 [B]."""
    _cuda(q, k_cache, v_cache, block_tables, context_lens)
    B, H, D = q.shape
    l1 = _is_l1(k_cache, v_cache)
    nb, bs, Hkv = (k_cache.shape[0], k_cache.shape[3], k_cache.shape[1]) if l1 else k_cache.shape[:3]
    mb = block_tables.shape[1]
    if workspace is None:
        workspace = paged_attn_workspace(B, H, D, mb, q.device)
    if out is None:
        out = torch.empty_like(q)
    if l1:
        _lib.lib().b200_paged_attn_decode_l1(
            _p(out), _p(q), _p(k_cache), _p(v_cache), _p(block_tables), _p(context_lens), B, H, Hkv, D, bs, mb, nb,
            float(scale), float(softcap), int(window), _p(workspace), int(q.dtype == torch.bfloat16), _stream())
        _lib.check()
        return out
    fp8 = k_cache.dtype == torch.uint8                                # --fp8-kvcache: e4m3 bytes
    fn = _lib.lib().b200_paged_attn_decode_fp8kv_f16 if fp8 else _sym("b200_paged_attn_decode", q)
    fn(_p(out), _p(q), _p(k_cache), _p(v_cache), _p(block_tables), _p(context_lens), B, H, Hkv, D, bs,
       mb, nb, float(scale), float(softcap), int(window), _p(workspace), _stream())
    _lib.check()
    return out


ATTN_AUTO, ATTN_MMA, ATTN_TC, ATTN_TC_SWAPDESC = -1, 0, 1, 2


def attention_prefill(q, k_cache, v_cache, cu_seqlens_q, context_lens, block_tables, max_seqlen_q,
                      scale, out=None, mode=ATTN_AUTO):
    """PagedAttention::forward, prefill branch over the paged cache (see b200_attn_prefill_ex_f16)."""
    _cuda(q, k_cache, v_cache, cu_seqlens_q, context_lens, block_tables)
    T, H, D = q.shape
    l1 = _is_l1(k_cache, v_cache)
    nb, bs, Hkv = (k_cache.shape[0], k_cache.shape[3], k_cache.shape[1]) if l1 else k_cache.shape[:3]
    B = cu_seqlens_q.shape[0] - 1
    if out is None:
        out = torch.empty_like(q)
    if l1:
        _lib.lib().b200_attn_prefill_l1(
            _p(out), _p(q), _p(k_cache), _p(v_cache), _p(cu_seqlens_q), _p(context_lens), _p(block_tables), B, H,
            Hkv, D, bs, block_tables.shape[1], nb, int(max_seqlen_q), T, mode, float(scale),
            int(q.dtype == torch.bfloat16), _stream())
        _lib.check()
        return out
    _sym("b200_attn_prefill_ex", q)(_p(out), _p(q), _p(k_cache), _p(v_cache), _p(cu_seqlens_q),
                                    _p(context_lens), _p(block_tables), B, H, Hkv, D, bs,
                                    block_tables.shape[1], nb, int(max_seqlen_q), T, mode, float(scale),
                                    _stream())
    _lib.check()
    return out


# ------------------------------------------------------------------ glue
def rmsnorm(x, w, eps, out=None):
    _cuda(x, w)
    out = torch.empty_like(x) if out is None else out
    _sym("b200_rmsnorm", x)(_p(out), _p(x), _p(w), x.shape[0], x.shape[1], eps, _stream())
    _lib.check()
    return out


def add_rmsnorm(residual, x, w, eps, out=None):
    """residual += x (in place); returns rmsnorm(residual) * w."""
    _cuda(residual, x, w)
    out = torch.empty_like(x) if out is None else out
    _sym("b200_add_rmsnorm", x)(_p(out), _p(residual), _p(x), _p(w), x.shape[0], x.shape[1], eps, _stream())
    _lib.check()
    return out


def silu_mul(gate_up, out=None):
    _cuda(gate_up)
    T, n2 = gate_up.shape
    out = torch.empty(T, n2 // 2, dtype=gate_up.dtype, device=gate_up.device) if out is None else out
    _sym("b200_silu_mul", gate_up)(_p(out), _p(gate_up), T, n2 // 2, _stream())
    _lib.check()
    return out


def embedding(table, ids, out=None):
    _cuda(table, ids)
    T = ids.shape[0]
    out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device) if out is None else out
    _lib.lib().b200_embedding_f16(_p(out), _p(table), _p(ids), T, table.shape[1], table.shape[0],
                                  _stream())
    _lib.check()
    return out


def argmax(logits):
    _cuda(logits)
    out = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    _lib.lib().b200_argmax_f32(_p(out), _p(logits), logits.shape[0], logits.shape[1], _stream())
    _lib.check()
    return out


# ------------------------------------------------------------------ sampling
def sample_topk_topp(logits, top_k, top_p, temperature, seed, out=None):
    """Device sampler (logits_processor.rs:199-231): logits f32 [B, V] -> ids i32 [B].  `seed` is a
    python int (copied to a device u64) or a 1-element int64 CUDA tensor."""
    _cuda(logits)
    B, V = logits.shape
    if not torch.is_tensor(seed):
        seed = torch.tensor([seed - (1 << 64) if seed >= (1 << 63) else seed], dtype=torch.int64).to(logits.device)
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    _lib.lib().b200_sample_topk_topp_f32(_p(out), _p(logits), B, V, top_k, float(top_p), float(temperature),
                                         _p(seed), _stream())
    _lib.check()
    return out


def apply_penalties(logits, context, context_lens, frequency_penalty, presence_penalty):
    """apply_batch_repeat_penalty (logits_processor.rs:308-343), in place.  context i32 [B, cap]."""
    _cuda(logits, context, context_lens)
    B, V = logits.shape
    _lib.lib().b200_apply_penalties_f32(_p(logits), B, V, _p(context), _p(context_lens), context.shape[1],
                                        float(frequency_penalty), float(presence_penalty), _stream())
    _lib.check()
    return logits


def sampling_strategy(temperature=None, top_k=None, top_p=None):
    """LogitsProcessor::get_strategy (logits_processor.rs:48-70): (strategy, k, p, t) for the runners' set_sampling."""
    import ctypes as C
    k, p, t = C.c_int32(0), C.c_float(1.0), C.c_float(1.0)
    s = _lib.lib().b200_sampling_strategy(int(temperature is not None), float(temperature or 0.0),
                                          int(top_k is not None), int(top_k or 0), int(top_p is not None),
                                          float(top_p or 0.0), C.byref(k), C.byref(p), C.byref(t))
    return s, k.value, p.value, t.value


# ------------------------------------------------------------------ mixers of the fp32-residual hybrid decoders
# Ragged steps: cu_seqlens_q i32 [B + 1], context_lens i32 [B] (length after the step), block_tables i32 [B, max_blocks],
# state_slots i32 [B].  `dtype` of an output that feeds a matrix product: torch.bfloat16 or torch.float32.
def _dt(dtype) -> int:
    if dtype == torch.bfloat16:
        return 0
    if dtype == torch.float32:
        return 1
    raise TypeError("operand dtype must be bfloat16 or float32")


def resid_rmsnorm(x, w, eps, w_offset=0.0, dtype=torch.bfloat16):
    """RMS norm of an fp32 stream x [T, D] with fp32 weight (w_offset + w)."""
    _cuda(x, w)
    out = torch.empty(x.shape, dtype=dtype, device=x.device)
    _lib.lib().b200_resid_rmsnorm(_p(out), _p(x), _p(w), x.shape[0], x.shape[1], float(eps), float(w_offset),
                                  _dt(dtype), _stream())
    _lib.check()
    return out


def gated_group_norm(y, gate, w, group, eps, gate_first, dtype=torch.bfloat16, gate_act="silu"):
    """y, gate fp32 [T, C]; groups of `group` channels; w fp32 [C] or [group] (shared by the groups) or None;
    gate_act: "silu" or "sigmoid"."""
    _cuda(y, gate, w)
    T, Cn = y.shape
    out = torch.empty(T, Cn, dtype=dtype, device=y.device)
    _lib.lib().b200_gated_group_norm(_p(out), _p(y), Cn, _p(gate), Cn, _p(w), w.numel() if w is not None else 1, T, Cn,
                                     int(group), float(eps), int(bool(gate_first)), {"silu": 0, "sigmoid": 1}[gate_act],
                                     _dt(dtype), _stream())
    _lib.check()
    return out


def latent_prep(qc, cache, latent_norm_w, rot_freq, rot_mag, positions, slot_mapping, *, heads, dim, rot_dim, rot_dims,
                kv_rank, eps):
    """Returns (q_plain [T, heads, dim] in the cache dtype, q_full fp32 [T, heads, kv_rank + rot_dim] with the
    rotated parts filled and the first kv_rank entries of every head left for the absorbed query)."""
    _cuda(qc, cache, latent_norm_w, rot_freq, positions, slot_mapping)
    T = qc.shape[0]
    q_plain = torch.empty(T, heads, dim, dtype=cache.dtype, device=qc.device)
    q_full = torch.zeros(T, heads, kv_rank + rot_dim, dtype=torch.float32, device=qc.device)
    _lib.lib().b200_latent_prep(_p(qc), qc.shape[1], _p(q_plain), _p(q_full), _p(cache), _p(latent_norm_w),
                                _p(rot_freq), float(rot_mag), _p(positions), _p(slot_mapping), T, heads, dim, rot_dim,
                                rot_dims, kv_rank, float(eps), _dt(cache.dtype), _stream())
    _lib.check()
    return q_plain, q_full


def latent_prep_queries(q, rot_freq, rot_mag, positions, *, heads, dim, rot_dim, rot_dims, kv_rank, dtype):
    """latent_prep for a layer that reads another layer's cache: q fp32 [T, heads (dim + rot_dim)] holds queries only."""
    _cuda(q, rot_freq, positions)
    T = q.shape[0]
    q_plain = torch.empty(T, heads, dim, dtype=dtype, device=q.device)
    q_full = torch.zeros(T, heads, kv_rank + rot_dim, dtype=torch.float32, device=q.device)
    _lib.lib().b200_latent_prep_queries(_p(q), q.shape[1], _p(q_plain), _p(q_full), _p(rot_freq), float(rot_mag),
                                        _p(positions), T, heads, dim, rot_dim, rot_dims, kv_rank, _dt(dtype), _stream())
    _lib.check()
    return q_plain, q_full


def latent_attn(q_full, cache, sink, cu_seqlens_q, context_lens, block_tables, *, kv_rank, rot_dim, window, scale,
                split=True, gate=None):
    """Attention-weighted latents [T, heads, kv_rank] in the cache dtype.  split: give the kernel the workspace that
    lets steps of few rows spread a row's keys over several blocks.  gate fp32 [T, heads] logits or None: head h's
    result is multiplied by sigmoid(gate[t, h])."""
    _cuda(q_full, cache, sink, cu_seqlens_q, context_lens, block_tables, gate)
    T, H, _ = q_full.shape
    out = torch.empty(T, H, kv_rank, dtype=cache.dtype, device=q_full.device)
    nbytes = _lib.lib().b200_latent_attn_workspace_bytes(T, H, kv_rank, int(window)) if split else 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q_full.device) if nbytes else None
    _lib.lib().b200_latent_attn_gated(_p(out), _p(q_full), _p(cache), _p(sink), _p(gate),
                                      gate.shape[1] if gate is not None else 0, _p(cu_seqlens_q), _p(context_lens),
                                      _p(block_tables), block_tables.shape[1], context_lens.shape[0], T, H, kv_rank,
                                      rot_dim, int(window), float(scale), _dt(cache.dtype), _p(ws), _stream())
    _lib.check()
    return out


def short_conv_silu(x, taps_w, bias, state, state_slots, cu_seqlens_q, context_lens):
    """x fp32 [T, C] -> silu(causal conv) fp32 [T, C]; state fp32 [slots, taps - 1, C] is read and updated."""
    _cuda(x, taps_w, bias, state, state_slots, cu_seqlens_q, context_lens)
    out = torch.empty_like(x)
    _lib.lib().b200_short_conv_silu(_p(out), x.shape[1], _p(x), x.shape[1], _p(taps_w), _p(bias), _p(state),
                                    _p(state_slots), _p(cu_seqlens_q), _p(context_lens), context_lens.shape[0],
                                    x.shape[0], x.shape[1], taps_w.shape[1], _stream())
    _lib.check()
    return out


def delta_rule(q, k, v, b_raw, a_raw, a_log, dt_bias, state, state_slots, cu_seqlens_q, context_lens):
    """q, k fp32 [T, kv_heads, dim], v [T, heads, vdim], b_raw / a_raw [T, heads] -> o fp32 [T, heads, vdim]."""
    T, Hk, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    row = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), b_raw, a_raw], 1).contiguous()
    _cuda(row, a_log, dt_bias, state, state_slots, cu_seqlens_q, context_lens)
    out = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    ld, e = row.shape[1], 4
    base = row.data_ptr()
    _lib.lib().b200_delta_rule(_p(out), base, base + Hk * dk * e, base + 2 * Hk * dk * e, ld,
                               base + (2 * Hk * dk + H * dv) * e, base + (2 * Hk * dk + H * dv + H) * e, ld, _p(a_log),
                               _p(dt_bias), _p(state), _p(state_slots), _p(cu_seqlens_q), _p(context_lens),
                               context_lens.shape[0], H, Hk, dk, dv, _stream())
    _lib.check()
    return out


def ssd_scan(x, Bm, Cm, dt_raw, a_log, dt_bias, d_skip, state, state_slots, cu_seqlens_q, context_lens):
    """x fp32 [T, heads, vdim], Bm / Cm [T, groups, nstate], dt_raw [T, heads] -> y fp32 [T, heads, vdim]."""
    T, H, P = x.shape
    G, N = Bm.shape[1], Bm.shape[2]
    row = torch.cat([x.reshape(T, -1), Bm.reshape(T, -1), Cm.reshape(T, -1), dt_raw], 1).contiguous()
    _cuda(row, a_log, dt_bias, d_skip, state, state_slots, cu_seqlens_q, context_lens)
    out = torch.empty(T, H, P, dtype=torch.float32, device=x.device)
    ld, e, base = row.shape[1], 4, row.data_ptr()
    _lib.lib().b200_ssd_scan(_p(out), base, base + H * P * e, base + (H * P + G * N) * e, ld,
                             base + (H * P + 2 * G * N) * e, ld, _p(a_log), _p(dt_bias), _p(d_skip), _p(state),
                             _p(state_slots), _p(cu_seqlens_q), _p(context_lens), context_lens.shape[0], H, G, N, P,
                             _stream())
    _lib.check()
    return out


def moe_route(logits, top, scale):
    _cuda(logits)
    T, E = logits.shape
    idx = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    _lib.lib().b200_moe_route(_p(logits), T, E, int(top), float(scale), _p(idx), _p(w), _stream())
    _lib.check()
    return idx, w


def moe_experts(x, h, top_idx, top_w, w_gate_up, w_down):
    """x fp32 [T, D] += routed experts of h [T, D]; w_gate_up [E, 2 F, D], w_down [E, D, F] in h's dtype."""
    _cuda(x, h, top_idx, top_w, w_gate_up, w_down)
    T, D = x.shape
    E, F2, _ = w_gate_up.shape
    top = top_idx.shape[1]
    nbytes = _lib.lib().b200_moe_workspace_bytes(T, E, top, D, F2 // 2)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    _lib.lib().b200_moe_experts(_p(x), _p(h), _p(top_idx), _p(top_w), _p(w_gate_up), _p(w_down), T, E, top, D, F2 // 2,
                                _dt(h.dtype), _p(ws), _stream())
    _lib.check()
    return x


def moe_route_ex(logits, bias, top, scale=1.0, groups=0, keep=0):
    """Router with a selection bias (fp32 [E] or None) and groups: see b200_moe_route_ex."""
    _cuda(logits, bias)
    T, E = logits.shape
    idx = torch.empty(T, top, dtype=torch.int32, device=logits.device)
    w = torch.empty(T, top, dtype=torch.float32, device=logits.device)
    _lib.lib().b200_moe_route_ex(_p(logits), _p(bias), T, E, int(top), int(groups), int(keep), float(scale), _p(idx),
                                 _p(w), _stream())
    _lib.check()
    return idx, w


def moe_experts_ex(out, h, top_idx, top_w, w_up, w_down, *, act="silu_gate", identity=0, accumulate=True, ident=None):
    """out fp32 [T, D] (+)= the chosen experts of h [T, D]; act "silu_gate": w_up [E, 2 F, D]; "relu2": w_up [E, F, D];
    indices >= E are identity experts and return the rows of `ident` (fp32 or h's dtype; default h)."""
    ident = h if ident is None else ident
    _cuda(out, h, top_idx, top_w, w_up, w_down, ident)
    T, D = out.shape
    E, rows, _ = w_up.shape
    F = rows // 2 if act == "silu_gate" else rows
    top = top_idx.shape[1]
    nbytes = _lib.lib().b200_moe_workspace_bytes(T, E + identity, top, D, F)
    ws = torch.empty(nbytes, dtype=torch.uint8, device=out.device)
    _lib.lib().b200_moe_experts_ex(_p(out), _p(h), _p(top_idx), _p(top_w), _p(w_up), _p(w_down), T, E, int(identity), top,
                                   D, F, {"silu_gate": 0, "relu2": 1}[act], int(bool(accumulate)), _p(ident),
                                   int(ident.dtype == torch.float32), _dt(h.dtype), _p(ws), _stream())
    _lib.check()
    return out


def resid_add_rmsnorm(x, y, w, eps, w_offset=0.0):
    """x fp32 [T, D] += y / rms(y) * (w_offset + w), in place."""
    _cuda(x, y, w)
    _lib.lib().b200_resid_add_rmsnorm(_p(x), _p(y), _p(w), x.shape[0], x.shape[1], float(eps), float(w_offset), _stream())
    _lib.check()
    return x


def _attn_options(head_norm=False, v_from_k=False, q_temp=None, dist_slopes=None, gate_elems=False, rot_half=False,
                  rot_mag=1.0, v_rot_freq=None, v_heads=0, chunk=0, out_f32=False, no_cache=False):
    """b200_attn_options; q_temp = (coef, every) or None.  Keep the returned object alive during the call."""
    o = _lib.AttnOptions(head_norm=int(bool(head_norm)), v_from_k=int(bool(v_from_k)),
                         q_temp_every=int(q_temp[1]) if q_temp else 0, gate_elems=int(bool(gate_elems)),
                         q_temp_coef=float(q_temp[0]) if q_temp else 0.0,
                         dist_slopes=dist_slopes.data_ptr() if dist_slopes is not None else None,
                         rot_half=int(bool(rot_half)), rot_mag=float(rot_mag),
                         v_rot_freq=v_rot_freq.data_ptr() if v_rot_freq is not None else None, v_heads=int(v_heads),
                         chunk=int(chunk), out_f32=int(bool(out_f32)), no_cache=int(bool(no_cache)))
    return o


def window_attn_prep(proj, bias, q_norm_w, k_norm_w, rot_freq, positions, slot_mapping, k_cache, v_cache, *, heads,
                     rot_dims, eps, head_norm=False, v_from_k=False, q_temp=None, rot_half=False, rot_mag=1.0,
                     v_rot_freq=None):
    """proj fp32 [T, >= heads dim + kv_heads (dim + vdim)] -> q fp32 [T, heads, dim]; writes the K / V cache rows
    (k_cache [blocks, 64, kv_heads, dim], v_cache [blocks, 64, kv_heads, vdim]).  head_norm: q_norm_w / k_norm_w are
    [dim] and every head is normed on its own; v_from_k: no v block, the raw key rows are the values; q_temp =
    (coef, every): the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1).  rot_half: rotary
    pairs are (i, i + rot_dims / 2); rot_mag multiplies cos and sin; v_rot_freq f64 [vdim / 2]: the value rows are
    rotated by their position over all of vdim.  The value cache may have fewer heads than the key cache (several score
    maps over one set of values)."""
    _cuda(proj, bias, q_norm_w, k_norm_w, rot_freq, positions, slot_mapping, k_cache, v_cache, v_rot_freq)
    T = proj.shape[0]
    G, dk, dv = k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
    q = torch.empty(T, heads, dk, dtype=torch.float32, device=proj.device)
    opt = _attn_options(head_norm, v_from_k, q_temp, rot_half=rot_half, rot_mag=rot_mag, v_rot_freq=v_rot_freq,
                        v_heads=v_cache.shape[2])
    _lib.lib().b200_window_attn_prep_ex(_p(proj), proj.shape[1], _p(bias), _p(q_norm_w), _p(k_norm_w), _p(rot_freq),
                                        _p(positions), _p(slot_mapping), _p(q), _p(k_cache), _p(v_cache), T, heads, G, dk,
                                        dv, int(rot_dims), float(eps), _dt(k_cache.dtype), C.byref(opt), _stream())
    _lib.check()
    return q


def window_attn(q, k_cache, v_cache, sink, gate, cu_seqlens_q, context_lens, block_tables, *, window, keep_first, scale,
                softcap=0.0, split=True, dist_slopes=None, chunk=0, out_f32=False):
    """q fp32 [T, heads, dim] -> [T, heads, vdim] in the cache dtype (fp32 with out_f32); gate fp32 logits [T, heads]
    (one per head) or [T, heads vdim] (one per output element) or None; dist_slopes fp32 [heads]: scores are lowered by
    slope (i - j); chunk > 0: position i sees j <= i of its own chunk only.  A value cache with fewer heads than the key
    cache: key head g reads value head g % v_heads."""
    _cuda(q, k_cache, v_cache, sink, gate, cu_seqlens_q, context_lens, block_tables, dist_slopes)
    T, H, dk = q.shape
    G, dv = k_cache.shape[2], v_cache.shape[3]
    out = torch.empty(T, H, dv, dtype=torch.float32 if out_f32 else k_cache.dtype, device=q.device)
    nbytes = _lib.lib().b200_window_attn_workspace_bytes_ex(T, H, G, v_cache.shape[2], dv, int(window),
                                                            int(keep_first)) if split else 0
    ws = torch.empty(nbytes, dtype=torch.uint8, device=q.device) if nbytes else None
    opt = _attn_options(dist_slopes=dist_slopes, gate_elems=gate is not None and gate.shape[1] == H * dv and dv > 1,
                        v_heads=v_cache.shape[2], chunk=chunk, out_f32=out_f32)
    _lib.lib().b200_window_attn_ex(_p(out), _p(q), _p(k_cache), _p(v_cache), _p(sink), _p(gate),
                                   gate.shape[1] if gate is not None else 0, _p(cu_seqlens_q), _p(context_lens),
                                   _p(block_tables), block_tables.shape[1], context_lens.shape[0], T, H, G, dk, dv,
                                   int(window), int(keep_first), float(scale), float(softcap), _dt(k_cache.dtype), _p(ws),
                                   C.byref(opt), _stream())
    _lib.check()
    return out


def lowrank_decay(low, w2, bias, tau):
    """low fp32 [T, rank], w2 fp32 [C, rank], bias fp32 [C] or None -> sigmoid(bias + low w2^T)^(1 / tau) fp32 [T, C]."""
    _cuda(low, w2, bias)
    T, C = low.shape[0], w2.shape[0]
    out = torch.empty(T, C, dtype=torch.float32, device=low.device)
    _lib.lib().b200_lowrank_decay(_p(out), _p(low), low.shape[1], _p(w2), _p(bias), float(tau), T, C, w2.shape[1], _stream())
    _lib.check()
    return out


def decay_attn(q, k, v, state, state_slots, cu_seqlens_q, context_lens, *, head_decay=None, chan_decay=None, q_scale=1.0,
               k_scale=1.0, act=False):
    """q, k fp32 [T, heads, dim], v [T, heads, vdim]; head_decay fp32 [heads] or chan_decay fp32 [T, heads, dim];
    state fp32 [slots, heads, dim, vdim] is read and updated -> o fp32 [T, heads, vdim]."""
    T, H, dk = q.shape
    dv = v.shape[2]
    row = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).contiguous()
    if chan_decay is not None:
        chan_decay = chan_decay.reshape(T, -1).contiguous()
    _cuda(row, head_decay, chan_decay, state, state_slots, cu_seqlens_q, context_lens)
    out = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    ld, e, base = row.shape[1], 4, row.data_ptr()
    _lib.lib().b200_decay_attn(_p(out), base, base + H * dk * e, base + 2 * H * dk * e, ld, _p(head_decay),
                               _p(chan_decay), H * dk, float(q_scale), float(k_scale), int(bool(act)), _p(state),
                               _p(state_slots), _p(cu_seqlens_q), _p(context_lens), context_lens.shape[0], H, dk, dv,
                               _stream())
    _lib.check()
    return out


def attn_finish(a, gate, positions, *, heads, maps=1, lam=0.0, v_rot_freq=None, rot_half=True, head_norm=False, eps=1e-6,
                out_scale=1.0, dtype=torch.float32):
    """a fp32 [T, maps * heads, vdim] (map after map) -> [T, heads, vdim] in `dtype`: a[map 0] - lam a[map 1] (maps == 2),
    turned back by -position * v_rot_freq (f64 [vdim / 2] or None), RMS-normed per head without a weight (head_norm),
    times out_scale, times the sigmoid of gate ([T, heads] or [T, heads vdim] or None)."""
    _cuda(a, gate, positions, v_rot_freq)
    T, dv = a.shape[0], a.shape[2]
    out = torch.empty(T, heads, dv, dtype=dtype, device=a.device)
    _lib.lib().b200_attn_finish(_p(out), _p(a), _p(gate), gate.shape[1] if gate is not None else 0,
                                int(gate is not None and gate.shape[1] == heads * dv and dv > 1), _p(positions),
                                _p(v_rot_freq), int(bool(rot_half)), int(maps), float(lam), int(bool(head_norm)), float(eps),
                                float(out_scale), T, heads, dv, _dt(dtype), _stream())
    _lib.check()
    return out


def stream_norm(x, w, bias, *, kind="dyntanh", alpha=1.0, eps=1e-6, w_offset=0.0, shift_w=None, shift_state=None,
                state_slots=None, cu_seqlens_q=None, context_lens=None, dtype=torch.float32):
    """x fp32 [T, D] -> norm(x) in `dtype`: kind "rms" (x / rms(x) * (w_offset + w)) or "dyntanh" (tanh(alpha x) w + b).
    With shift_w the token shift follows: out[t] = n[t] + (n[t-1] - n[t]) * shift_w, n[t-1] from the row above or, for a
    portion's first row, from shift_state [slots, D] (zeros at position 0); shift_state is updated."""
    _cuda(x, w, bias, shift_w, shift_state, state_slots, cu_seqlens_q, context_lens)
    T, D = x.shape
    out = torch.empty(T, D, dtype=dtype, device=x.device)
    _lib.lib().b200_stream_norm(_p(out), _p(x), _p(w), _p(bias), float(alpha), {"rms": 0, "dyntanh": 1}[kind], float(eps),
                                float(w_offset), None, _p(shift_w), _p(shift_state), _p(state_slots), _p(cu_seqlens_q),
                                _p(context_lens), context_lens.shape[0] if context_lens is not None else 0, T, D,
                                _dt(dtype), _stream())
    _lib.check()
    return out


def depth_mix(hist, w):
    """hist fp32 [n, ...] (contiguous), w fp32 [n] -> sum_j w[j] hist[j]."""
    _cuda(hist, w)
    out = torch.empty_like(hist[0])
    _lib.lib().b200_depth_mix(_p(out), _p(hist), hist[0].numel(), _p(w), hist.shape[0], hist[0].numel(), _stream())
    _lib.check()
    return out


def channel_decay(low, w2, bias, a_log, period):
    """low fp32 [T, rank], w2 fp32 [C, rank], bias fp32 [C], a_log fp32 [C / period] ->
    exp(-exp(a_log[c / period]) softplus(bias + low w2^T)) fp32 [T, C]."""
    _cuda(low, w2, bias, a_log)
    T, C_ = low.shape[0], w2.shape[0]
    out = torch.empty(T, C_, dtype=torch.float32, device=low.device)
    _lib.lib().b200_lowrank_decay_ex(_p(out), _p(low), low.shape[1], _p(w2), _p(bias), 1.0, 1, _p(a_log), int(period), T, C_,
                                     w2.shape[1], _stream())
    _lib.check()
    return out


def delta_rule_chan(q, k, v, b_raw, decay, state, state_slots, cu_seqlens_q, context_lens):
    """The gated delta rule with ready-made decays per head and key channel: q, k fp32 [T, kv_heads, dim], v
    [T, heads, vdim], b_raw [T, heads], decay [T, heads, dim] -> o fp32 [T, heads, vdim]; state is read and updated."""
    T, Hk, dk = q.shape
    H, dv = v.shape[1], v.shape[2]
    row = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1), b_raw], 1).contiguous()
    decay = decay.reshape(T, -1).contiguous()
    _cuda(row, decay, state, state_slots, cu_seqlens_q, context_lens)
    out = torch.empty(T, H, dv, dtype=torch.float32, device=q.device)
    ld, e, base = row.shape[1], 4, row.data_ptr()
    _lib.lib().b200_delta_rule_chan(_p(out), base, base + Hk * dk * e, base + 2 * Hk * dk * e, ld,
                                    base + (2 * Hk * dk + H * dv) * e, ld, _p(decay), H * dk, _p(state), _p(state_slots),
                                    _p(cu_seqlens_q), _p(context_lens), context_lens.shape[0], H, Hk, dk, dv, _stream())
    _lib.check()
    return out
