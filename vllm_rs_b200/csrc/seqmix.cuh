// Shared pieces of the sequence-mixer kernels (latent and windowed attention, gated delta rule, SSD scan, decayed
// linear attention, routed experts)
// of hybrid decoders whose residual stream, norms, softmax, routers and recurrent state are kept in fp32.
//
// Activation dtype: every buffer that FEEDS a matrix product (and the latent KV cache) is either bf16 or fp32,
// chosen per model (`dt`: 0 = bf16, 1 = fp32); matrix products accumulate and store fp32.  A step is a ragged
// batch: `num_seqs` sequences, sequence b brings the token rows [cu[b], cu[b+1]) at positions
// ctx[b] - (cu[b+1] - cu[b]) .. ctx[b] - 1 (ctx = length after the step), so a prompt portion and a single
// decoded token are the same case.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/b200_vllm.h"
#include "common.cuh"

namespace b200 {
namespace seqmix {

constexpr int kPage = 64;          // tokens per cache page (the block manager's block size)

template <typename T> __device__ __forceinline__ float ld(const T* p);
template <> __device__ __forceinline__ float ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T> __device__ __forceinline__ void st(T* p, float v);
template <> __device__ __forceinline__ void st<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

__device__ __forceinline__ float lanes_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float lanes_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
// sum over the block; `red` holds at least 33 floats; every thread gets the result
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = lanes_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  if (w == 0) {
    float s = lane < nw ? red[lane] : 0.f;
    s = lanes_sum(s);
    if (lane == 0) red[32] = s;
  }
  __syncthreads();
  return red[32];
}
__device__ __forceinline__ float silu_f(float z) { return z / (1.f + __expf(-z)); }
__device__ __forceinline__ float silu_exact(float z) { return z / (1.f + expf(-z)); }
__device__ __forceinline__ float softplus_f(float z) { return z > 20.f ? z : log1pf(expf(z)); }
__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }

// sequence that owns token row t (cu is ascending, cu[0] = 0, cu[n] = total rows)
__device__ __forceinline__ int seq_of_row(const uint32_t* __restrict__ cu, int n, int t) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (static_cast<int>(cu[mid]) <= t) lo = mid; else hi = mid - 1;
  }
  return lo;
}

}  // namespace seqmix

// ---- launchers (seq_norms.cu, latent_attn.cu, window_attn.cu, linear_recurrence.cu, moe.cu, gemm_lib.cu); dt: 0 bf16, 1 fp32
// positions / pos_base: pos_base > 0 adds the sinusoidal position vector (sin at even, cos at odd entries); cast_out
// (bf16 runs, may be NULL): the rows rounded to bf16 as well
void launch_embed_f32(float* x, const void* table, const uint32_t* ids, const int64_t* positions, float pos_base, int T,
                      int width, int vocab, float scale, int dt, void* cast_out, cudaStream_t st);
void launch_resid_rmsnorm(void* out, const float* x, const float* w, int T, int width, float eps, float w_offset,
                          const uint32_t* rows, int dt, cudaStream_t st);
void launch_gated_group_norm(void* out, const float* y, int ldy, const float* gate, int ldg, const float* w, int w_period,
                             int T, int C, int group, float eps, int gate_first, int gate_act, int dt, cudaStream_t st);
// cast_out (may be NULL): the updated rows rounded to bf16 as well
void launch_resid_add_rmsnorm(float* x, const float* y, const float* w, int T, int width, float eps, float w_offset,
                              void* cast_out, cudaStream_t st);
void launch_bias_rows(float* y, const float* bias, float scale, int T, int n, cudaStream_t st);
void launch_cast_rows(void* out, const float* in, int ld_in, int T, int n, int dt, cudaStream_t st);
void launch_silu_mul_f32(void* out, const float* gate_up, int T, int ff, int dt, cudaStream_t st);
// out [T, ff] = relu(up[t, d])^2 (* sigmoid(up[t, gate_col]) when gate_col >= 0); up fp32 with row stride ld
// bias (may be NULL): fp32 [ff], added before the activation
void launch_relu2_f32(void* out, const float* up, int ld, int T, int ff, int gate_col, const float* bias, int dt,
                      cudaStream_t st);
// norm of the stream (kind B200_NORM_*), optionally followed by the token shift (see b200_stream_norm)
void launch_stream_norm(void* out, const float* x, const float* w, const float* bias, float alpha, int kind, float eps,
                        float w_offset, const uint32_t* rows, const float* shift_w, float* shift_state,
                        const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int T, int width,
                        int dt, cudaStream_t st);
void launch_depth_mix(float* out, const float* hist, size_t stride, const float* w, int count, size_t n, cudaStream_t st);

void launch_latent_prep(const float* qc, int ldq, void* q_plain, float* q_full, void* cache, const float* latent_norm_w,
                        const double* rot_freq, float rot_mag, const int64_t* positions, const int64_t* slots, int T,
                        int heads, int dim, int rot_dim, int rot_dims, int kv_rank, float eps, int dt, cudaStream_t st);
// cache == nullptr: the row holds queries only (a layer that reads another layer's cache); gate: per-head output gate
void launch_latent_attn(void* out, const float* q_full, const void* cache, const float* sink, const float* gate,
                        int ld_gate, const uint32_t* cu, const uint32_t* ctx, const uint32_t* block_tables,
                        int max_blocks, int num_seqs, int T, int heads, int kv_rank, int rot_dim, int window, float scale,
                        int dt, void* workspace, cudaStream_t st);
size_t latent_attn_workspace_bytes(int T, int heads, int kv_rank, int window);

void launch_window_attn_prep(const float* proj, int ld, const float* bias, const float* q_norm_w, const float* k_norm_w,
                             const double* rot_freq, const int64_t* positions, const int64_t* slots, float* q_out,
                             void* k_cache, void* v_cache, int T, int heads, int kv_heads, int dim, int vdim,
                             int rot_dims, float eps, int dt, const b200_attn_options* opt, cudaStream_t st);
void launch_window_attn(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                        const float* gate, int ld_gate, const uint32_t* cu, const uint32_t* ctx,
                        const uint32_t* block_tables, int max_blocks, int num_seqs, int T, int heads, int kv_heads,
                        int dim, int vdim, int window, int keep_first, float scale, float softcap, int dt,
                        void* workspace, const b200_attn_options* opt, cudaStream_t st);
// v_heads (0: kv_heads): heads of the value cache where several score maps share the values
size_t window_attn_workspace_bytes(int T, int heads, int kv_heads, int vdim, int window, int keep_first, int v_heads = 0);
// the combination of score maps, the turn back of rotated values, the per-head norm, scale and gate (see b200_attn_finish)
void launch_attn_finish(void* out, const float* a, const float* gate, int ld_gate, int gate_elems,
                        const int64_t* positions, const double* v_rot_freq, int rot_half, int maps, float lambda,
                        int head_norm, float eps, float out_scale, int T, int heads, int vdim, int dt, cudaStream_t st);

void launch_short_conv_silu(float* out, int ldo, const float* x, int ldx, const float* taps_w, const float* bias,
                            float* state, const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs,
                            int num_rows, int C, int taps, cudaStream_t st);
// chan_decay (may be NULL): ready-made decays per head and key channel [T, heads, dim] (row stride ld_decay); with it
// a_raw, a_log and dt_bias are not used
void launch_delta_rule(float* out, const float* q, const float* k, const float* v, int ld, const float* b_raw,
                       const float* a_raw, int ld_ba, const float* a_log, const float* dt_bias, const float* chan_decay,
                       int ld_decay, float* state, const int32_t* slots, const uint32_t* cu, const uint32_t* ctx,
                       int num_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t st);
void launch_ssd_scan(float* out, const float* x, const float* Bm, const float* Cm, int ld, const float* dt_raw,
                     int ld_dt, const float* a_log, const float* dt_bias, const float* d_skip, float* state,
                     const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int heads, int groups,
                     int nstate, int vdim, cudaStream_t st);

// a_log (may be NULL): the delta rule's decay exp(-exp(a_log[c / a_period]) softplus(z)) instead of sigmoid(z)^(1/tau)
void launch_lowrank_decay(float* out, const float* low, int ld_low, const float* w2, const float* bias, float tau,
                          const float* a_log, int a_period, int T, int C, int rank, cudaStream_t st);
void launch_decay_attn(float* out, const float* q, const float* k, const float* v, int ld, const float* head_decay,
                       const float* chan_decay, int ld_decay, float q_scale, float k_scale, int act, float* state,
                       const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int heads, int dim,
                       int vdim, cudaStream_t st);

void launch_moe_route(const float* logits, const float* bias, int T, int E, int top, int groups, int keep, float scale,
                      int32_t* top_idx, float* top_w, cudaStream_t st);
void launch_moe_sort(const int32_t* top_idx, int pairs, int E, int32_t* expert_off, int32_t* pair_of_slot,
                     int32_t* slot_of_pair, cudaStream_t st);
// act 0: SiLU(gate) * up over [gate | up] rows; act 1: relu(up)^2 over up rows
void launch_moe_gate_up(void* act_out, const void* h, const void* w_up, const int32_t* expert_off,
                        const int32_t* pair_of_slot, int pairs, int top, int E, int width, int ff, int act, int dt,
                        cudaStream_t st);
void launch_moe_down(float* out, const void* act, const void* w_down, const int32_t* expert_off, int pairs, int E,
                     int width, int ff, int dt, cudaStream_t st);
// x = (accumulate ? x : 0) + sum of the choices; choices >= E are identity experts and read `ident`
void launch_moe_combine(float* x, const float* down, const int32_t* slot_of_pair, const int32_t* top_idx,
                        const float* top_w, int T, int top, int width, int E, const void* ident, int ident_f32, int dt,
                        int accumulate, cudaStream_t st);

// C[M, N] (fp32, ldc) = beta * C + A[M, K] (lda) x W[N, K]^T (ldw); operands bf16 or fp32, fp32 accumulation, no
// reduced-precision mode for fp32 operands.  `batch` > 1: strided batches.  w_kn != 0: W is stored [K, N] (ldw >= N).
bool gemm_f32out(const void* a, int lda, long long stride_a, const void* w, int ldw, long long stride_w, float* c, int ldc,
                 long long stride_c, int M, int N, int K, int batch, float beta, int w_kn, int dt, cudaStream_t st);
// the same with C = alpha * A x W^T + beta * C
bool gemm_f32out_scaled(const void* a, int lda, long long stride_a, const void* w, int ldw, long long stride_w, float* c,
                        int ldc, long long stride_c, int M, int N, int K, int batch, float alpha, float beta, int w_kn,
                        int dt, cudaStream_t st);

}  // namespace b200
