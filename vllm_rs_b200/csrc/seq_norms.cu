// Row kernels of decoders that keep the residual stream in fp32: embedding lookup into the stream, RMS norm of the
// stream (weight stored either plainly or as an offset from one), the grouped RMS norm with a SiLU gate that follows
// a recurrent mixer (gate applied before or after the normalisation), SiLU * mul over an fp32 gate|up block, and
// the rounding of fp32 rows to the dtype that feeds the next matrix product, the norm of the stream with a choice of
// kind (RMS / dynamic tanh) and a token shift, and the weighted sum of the stored results of earlier layers.  All arithmetic is fp32; the output
// dtype is bf16 or fp32.  Beside the fp16 / bf16 row kernels of glue.cu (rmsnorm_kernel, silu_mul_kernel), which
// keep a 16-bit residual.
#include "../../include/b200_vllm.h"
#include "seqmix.cuh"

namespace b200 {
using namespace seqmix;

// pos_base > 0: the sinusoidal position vector of the token's position p joins the row: entry 2i is
// sin(p * base^(-2i / width)), entry 2i + 1 the cosine of the same angle (frequency, angle, sine and cosine in fp32)
template <typename T>
__global__ void embed_f32_kernel(float* __restrict__ x, const T* __restrict__ table, const uint32_t* __restrict__ ids,
                                 const int64_t* __restrict__ positions, float pos_base, int width, int vocab,
                                 float scale, T* __restrict__ cast_out) {
  const int t = blockIdx.x;
  uint32_t id = ids[t];
  if (id >= static_cast<uint32_t>(vocab)) id = 0;
  const T* row = table + static_cast<size_t>(id) * width;
  const bool with_pos = pos_base > 0.f && positions != nullptr;
  const float p = with_pos ? static_cast<float>(positions[t]) : 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float v = ld(row + d) * scale;
    if (with_pos) {
      const float freq = powf(pos_base, -static_cast<float>(d & ~1) / static_cast<float>(width));
      const float ang = p * freq;
      v += (d & 1) ? cosf(ang) : sinf(ang);
    }
    x[static_cast<size_t>(t) * width + d] = v;
    if (cast_out) st(cast_out + static_cast<size_t>(t) * width + d, v);     // the row as the first sublayer reads it
  }
}

// out[r] = x[row(r)] / sqrt(mean(x^2) + eps) * (w_offset + w); rows == nullptr: row(r) = r
template <typename T>
__global__ void resid_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                     int width, float eps, float w_offset, const uint32_t* __restrict__ rows) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const float* xr = x + static_cast<size_t>(rows ? rows[r] : r) * width;
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) ss += xr[d] * xr[d];
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x)
    st(out + static_cast<size_t>(r) * width + d, xr[d] * inv * (w_offset + w[d]));
}

// One block per (token, group of `group` channels).  gate_first: u = y * act(g), out = u / rms(u) * w;
// otherwise out = y / rms(y) * w * act(g).  w is indexed by (channel % w_period); w == nullptr: no weight.
// act = SiLU (gate_act 0) or the logistic sigmoid (gate_act 1).
template <typename T>
__global__ void gated_group_norm_kernel(T* __restrict__ out, const float* __restrict__ y, int ldy,
                                        const float* __restrict__ gate, int ldg, const float* __restrict__ w,
                                        int w_period, int C, int group, float eps, int gate_first, int gate_act) {
  __shared__ float red[33];
  const int t = blockIdx.x, g0 = blockIdx.y * group;
  const float* yr = y + static_cast<size_t>(t) * ldy + g0;
  const float* gr = gate + static_cast<size_t>(t) * ldg + g0;
  float ss = 0.f;
  for (int d = threadIdx.x; d < group; d += blockDim.x) {
    const float u = gate_first ? yr[d] * (gate_act ? sigmoid_f(gr[d]) : silu_exact(gr[d])) : yr[d];
    ss += u * u;
  }
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(group) + eps);
  for (int d = threadIdx.x; d < group; d += blockDim.x) {
    const float s = gate_act ? sigmoid_f(gr[d]) : silu_exact(gr[d]);
    const float wv = w ? w[(g0 + d) % w_period] : 1.f;
    const float v = gate_first ? yr[d] * s * inv * wv : yr[d] * inv * wv * s;
    st(out + static_cast<size_t>(t) * C + g0 + d, v);
  }
}


// x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * (w_offset + w): the norm AFTER a sublayer, folded into the residual sum.
// cast_out (may be NULL): the new row rounded to bf16, for a next sublayer whose input is the un-normed stream.
__global__ void resid_add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w,
                                         int width, float eps, float w_offset, __nv_bfloat16* __restrict__ cast_out) {
  __shared__ float red[33];
  const int t = blockIdx.x;
  const float* yr = y + static_cast<size_t>(t) * width;
  float ss = 0.f;
  for (int d = threadIdx.x; d < width; d += blockDim.x) ss += yr[d] * yr[d];
  ss = block_sum(ss, red);
  const float inv = 1.f / sqrtf(ss / static_cast<float>(width) + eps);
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const size_t i = static_cast<size_t>(t) * width + d;
    const float v = x[i] + yr[d] * inv * (w_offset + w[d]);
    x[i] = v;
    if (cast_out) cast_out[i] = __float2bfloat16_rn(v);
  }
}

// y[t, d] += scale * bias[d]
__global__ void bias_rows_kernel(float* __restrict__ y, const float* __restrict__ bias, float scale, int n, size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x)
    y[i] += scale * bias[i % n];
}

template <typename T>
__global__ void cast_rows_kernel(T* __restrict__ out, const float* __restrict__ in, int ld_in, int n, size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / n, d = i % n;
    st(out + i, in[t * ld_in + d]);
  }
}

template <typename T>
__global__ void silu_mul_f32_kernel(T* __restrict__ out, const float* __restrict__ gu, int ff, size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / ff, d = i % ff;
    st(out + i, silu_exact(gu[t * 2 * ff + d]) * gu[t * 2 * ff + ff + d]);
  }
}

template <typename T>
__global__ void relu2_f32_kernel(T* __restrict__ out, const float* __restrict__ up, int ld, int ff, int gate_col,
                                 const float* __restrict__ bias, size_t total) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    const size_t t = i / ff, d = i % ff;
    const float u = fmaxf(up[t * ld + d] + (bias ? bias[d] : 0.f), 0.f);
    const float g = gate_col >= 0 ? sigmoid_f(up[t * ld + gate_col]) : 1.f;
    st(out + i, u * u * g);
  }
}

// One block per output row: a norm of the stream (RMS, or the dynamic tanh  tanh(alpha x) w + b  that needs no
// statistics) and, with shift_w, the token shift behind it:  out[t] = n[t] + (n[t-1] - n[t]) * shift_w, where n[t-1] is
// the un-shifted norm of the sequence's previous token -- recomputed from the row above, or, for the first row of a
// portion, read from the sequence's shift state (zeros at position 0).  The block of a sequence's FIRST row also writes
// the state: the un-shifted norm of the sequence's last row of the step.  Every thread reads the state entries it later
// overwrites, so the portion's first row sees the old state whatever the order of the blocks.
template <typename T>
__global__ void stream_norm_kernel(T* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                   const float* __restrict__ bias, float alpha, int kind, int width, float eps,
                                   float w_offset, const uint32_t* __restrict__ rows, const float* __restrict__ shift_w,
                                   float* __restrict__ shift_state, const int32_t* __restrict__ slots,
                                   const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx, int num_seqs) {
  __shared__ float red[33];
  const int r = blockIdx.x;
  const int t = rows ? static_cast<int>(rows[r]) : r;
  const float* xr = x + static_cast<size_t>(t) * width;
  // inverse root mean square of a row (RMS kind only)
  auto inv_rms = [&](const float* row) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < width; d += blockDim.x) ss += row[d] * row[d];
    ss = block_sum(ss, red);
    return 1.f / sqrtf(ss / static_cast<float>(width) + eps);
  };
  auto normed = [&](const float* row, float inv, int d) {
    return kind == B200_NORM_DYNTANH ? tanhf(alpha * row[d]) * w[d] + (bias ? bias[d] : 0.f)
                                     : row[d] * inv * (w_offset + w[d]);
  };
  const float inv = kind == B200_NORM_DYNTANH ? 1.f : inv_rms(xr);
  if (!shift_w) {
    for (int d = threadIdx.x; d < width; d += blockDim.x) st(out + static_cast<size_t>(r) * width + d, normed(xr, inv, d));
    return;
  }
  const int b = seq_of_row(cu, num_seqs, t);
  const int t0 = static_cast<int>(cu[b]), t1 = static_cast<int>(cu[b + 1]);
  const bool first = t == t0;
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;          // the sequence starts in this step
  float* sp = shift_state + static_cast<size_t>(slots[b]) * width;
  const float* xp = xr - width;                                      // the row above (same sequence unless `first`)
  const float* xl = x + static_cast<size_t>(t1 - 1) * width;         // the sequence's last row of the step
  const float inv_p = (kind == B200_NORM_DYNTANH || first) ? 1.f : inv_rms(xp);
  const float inv_l = (kind == B200_NORM_DYNTANH || !first) ? 1.f : (t1 - 1 == t ? inv : inv_rms(xl));
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    const float n = normed(xr, inv, d);
    const float prev = first ? (fresh ? 0.f : sp[d]) : normed(xp, inv_p, d);
    st(out + static_cast<size_t>(r) * width + d, n + (prev - n) * shift_w[d]);
    if (first) sp[d] = t1 - 1 == t ? n : normed(xl, inv_l, d);
  }
}

// out[i] = sum_j w[j] * hist[j * stride + i], V floats per thread and step
template <int V>
__global__ void depth_mix_kernel(float* __restrict__ out, const float* __restrict__ hist, size_t stride,
                                 const float* __restrict__ w, int count, size_t n) {
  for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n;
       i += static_cast<size_t>(gridDim.x) * blockDim.x) {
    if constexpr (V == 4) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int j = 0; j < count; ++j) {
        const float wj = w[j];
        const float4 v = *reinterpret_cast<const float4*>(hist + j * stride + i * 4);
        acc.x += wj * v.x; acc.y += wj * v.y; acc.z += wj * v.z; acc.w += wj * v.w;
      }
      *reinterpret_cast<float4*>(out + i * 4) = acc;
    } else {
      float acc = 0.f;
      for (int j = 0; j < count; ++j) acc += w[j] * hist[j * stride + i];
      out[i] = acc;
    }
  }
}

static int flat_grid(size_t total) {
  const size_t b = (total + 255) / 256;
  return static_cast<int>(b < 1 ? 1 : (b > 148 * 16 ? 148 * 16 : b));
}

void launch_embed_f32(float* x, const void* table, const uint32_t* ids, const int64_t* positions, float pos_base, int T,
                      int width, int vocab, float scale, int dt, void* cast_out, cudaStream_t st_) {
  if (T <= 0) return;
  if (dt)
    embed_f32_kernel<float><<<T, 256, 0, st_>>>(x, (const float*)table, ids, positions, pos_base, width, vocab, scale,
                                                nullptr);
  else
    embed_f32_kernel<__nv_bfloat16><<<T, 256, 0, st_>>>(x, (const __nv_bfloat16*)table, ids, positions, pos_base, width,
                                                        vocab, scale, (__nv_bfloat16*)cast_out);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_resid_rmsnorm(void* out, const float* x, const float* w, int T, int width, float eps, float w_offset,
                          const uint32_t* rows, int dt, cudaStream_t st_) {
  if (T <= 0) return;
  if (dt)
    resid_rmsnorm_kernel<float><<<T, 256, 0, st_>>>((float*)out, x, w, width, eps, w_offset, rows);
  else
    resid_rmsnorm_kernel<__nv_bfloat16><<<T, 256, 0, st_>>>((__nv_bfloat16*)out, x, w, width, eps, w_offset, rows);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_gated_group_norm(void* out, const float* y, int ldy, const float* gate, int ldg, const float* w,
                             int w_period, int T, int C, int group, float eps, int gate_first, int gate_act, int dt,
                             cudaStream_t st_) {
  if (T <= 0) return;
  const dim3 grid(T, C / group);
  const int threads = group >= 256 ? 256 : (group >= 128 ? 128 : 64);
  if (dt)
    gated_group_norm_kernel<float><<<grid, threads, 0, st_>>>((float*)out, y, ldy, gate, ldg, w, w_period, C, group,
                                                              eps, gate_first, gate_act);
  else
    gated_group_norm_kernel<__nv_bfloat16><<<grid, threads, 0, st_>>>((__nv_bfloat16*)out, y, ldy, gate, ldg, w,
                                                                      w_period, C, group, eps, gate_first, gate_act);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_resid_add_rmsnorm(float* x, const float* y, const float* w, int T, int width, float eps, float w_offset,
                              void* cast_out, cudaStream_t st_) {
  if (T <= 0) return;
  resid_add_rmsnorm_kernel<<<T, 256, 0, st_>>>(x, y, w, width, eps, w_offset, (__nv_bfloat16*)cast_out);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_bias_rows(float* y, const float* bias, float scale, int T, int n, cudaStream_t st_) {
  const size_t total = static_cast<size_t>(T) * n;
  if (total == 0) return;
  bias_rows_kernel<<<flat_grid(total), 256, 0, st_>>>(y, bias, scale, n, total);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_cast_rows(void* out, const float* in, int ld_in, int T, int n, int dt, cudaStream_t st_) {
  const size_t total = static_cast<size_t>(T) * n;
  if (total == 0) return;
  if (dt)
    cast_rows_kernel<float><<<flat_grid(total), 256, 0, st_>>>((float*)out, in, ld_in, n, total);
  else
    cast_rows_kernel<__nv_bfloat16><<<flat_grid(total), 256, 0, st_>>>((__nv_bfloat16*)out, in, ld_in, n, total);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_silu_mul_f32(void* out, const float* gate_up, int T, int ff, int dt, cudaStream_t st_) {
  const size_t total = static_cast<size_t>(T) * ff;
  if (total == 0) return;
  if (dt)
    silu_mul_f32_kernel<float><<<flat_grid(total), 256, 0, st_>>>((float*)out, gate_up, ff, total);
  else
    silu_mul_f32_kernel<__nv_bfloat16><<<flat_grid(total), 256, 0, st_>>>((__nv_bfloat16*)out, gate_up, ff, total);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_relu2_f32(void* out, const float* up, int ld, int T, int ff, int gate_col, const float* bias, int dt,
                      cudaStream_t st_) {
  const size_t total = static_cast<size_t>(T) * ff;
  if (total == 0) return;
  if (dt)
    relu2_f32_kernel<float><<<flat_grid(total), 256, 0, st_>>>((float*)out, up, ld, ff, gate_col, bias, total);
  else
    relu2_f32_kernel<__nv_bfloat16><<<flat_grid(total), 256, 0, st_>>>((__nv_bfloat16*)out, up, ld, ff, gate_col, bias,
                                                                       total);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_stream_norm(void* out, const float* x, const float* w, const float* bias, float alpha, int kind, float eps,
                        float w_offset, const uint32_t* rows, const float* shift_w, float* shift_state,
                        const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int T, int width,
                        int dt, cudaStream_t st_) {
  if (T <= 0) return;
  if (dt)
    stream_norm_kernel<float><<<T, 256, 0, st_>>>((float*)out, x, w, bias, alpha, kind, width, eps, w_offset, rows, shift_w,
                                                  shift_state, slots, cu, ctx, num_seqs);
  else
    stream_norm_kernel<__nv_bfloat16><<<T, 256, 0, st_>>>((__nv_bfloat16*)out, x, w, bias, alpha, kind, width, eps, w_offset,
                                                          rows, shift_w, shift_state, slots, cu, ctx, num_seqs);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_depth_mix(float* out, const float* hist, size_t stride, const float* w, int count, size_t n, cudaStream_t st_) {
  if (n == 0 || count <= 0) return;
  if (n % 4 == 0 && stride % 4 == 0 && (reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(hist)) % 16 == 0)
    depth_mix_kernel<4><<<flat_grid(n / 4), 256, 0, st_>>>(out, hist, stride, w, count, n / 4);
  else
    depth_mix_kernel<1><<<flat_grid(n), 256, 0, st_>>>(out, hist, stride, w, count, n);
  B200_CUDA_LAUNCH_CHECK();
}

}  // namespace b200

extern "C" {
// RMS norm of an fp32 residual stream: out[r] (bf16 when dt == 0, fp32 when dt == 1) = x[r] / sqrt(mean(x[r]^2) + eps)
// * (w_offset + w); w fp32 [width]; w_offset = 1 for weights stored around zero, 0 for plain weights.
void b200_resid_rmsnorm(void* out, const float* x, const float* w, int32_t num_tokens, int32_t width, float eps,
                        float w_offset, int32_t dt, int64_t stream) {
  B200_CHECK_ARG(out && x && w && width > 0 && (dt == 0 || dt == 1), "resid_rmsnorm: bad arguments");
  b200::launch_resid_rmsnorm(out, x, w, num_tokens, width, eps, w_offset, nullptr, dt,
                             reinterpret_cast<cudaStream_t>(stream));
}
// Grouped RMS norm with a SiLU gate over fp32 rows y [T, C] (row stride ldy), gate [T, C] (row stride ldg); groups of
// `group` consecutive channels are normalised separately; w fp32 is indexed by channel % w_period (a per-head weight
// shared by all heads has w_period = group; w NULL: no weight).  gate_first != 0: norm(y * act(gate)) * w; else
// norm(y) * w * act(gate); act = SiLU (gate_act 0) or sigmoid (gate_act 1).
void b200_gated_group_norm(void* out, const float* y, int32_t ldy, const float* gate, int32_t ldg, const float* w,
                           int32_t w_period, int32_t num_tokens, int32_t channels, int32_t group, float eps,
                           int32_t gate_first, int32_t gate_act, int32_t dt, int64_t stream) {
  B200_CHECK_ARG(out && y && gate && group > 0 && channels % group == 0 && w_period > 0 && (dt == 0 || dt == 1),
                 "gated_group_norm: bad arguments");
  b200::launch_gated_group_norm(out, y, ldy, gate, ldg, w, w_period, num_tokens, channels, group, eps, gate_first,
                                gate_act, dt, reinterpret_cast<cudaStream_t>(stream));
}
// x fp32 [T, width] += y / sqrt(mean(y^2) + eps) * (w_offset + w): the norm that follows a sublayer, with its residual sum.
void b200_resid_add_rmsnorm(float* x, const float* y, const float* w, int32_t num_tokens, int32_t width, float eps,
                            float w_offset, int64_t stream) {
  B200_CHECK_ARG(x && y && w && width > 0, "resid_add_rmsnorm: bad arguments");
  b200::launch_resid_add_rmsnorm(x, y, w, num_tokens, width, eps, w_offset, nullptr,
                                 reinterpret_cast<cudaStream_t>(stream));
}
void b200_stream_norm(void* out, const float* x, const float* w, const float* bias, float alpha, int32_t kind,
                      float eps, float w_offset, const uint32_t* rows, const float* shift_w, float* shift_state,
                      const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                      int32_t num_seqs, int32_t num_tokens, int32_t width, int32_t dt, int64_t stream) {
  B200_CHECK_ARG(out && x && w && width > 0 && (dt == 0 || dt == 1) && (kind == B200_NORM_RMS || kind == B200_NORM_DYNTANH) &&
                     (!shift_w || (!rows && shift_state && state_slots && cu_seqlens_q && context_lens && num_seqs > 0)),
                 "stream_norm: bad arguments (a token shift needs the step's sequences and a state, and no row list)");
  b200::launch_stream_norm(out, x, w, bias, alpha, kind, eps, w_offset, rows, shift_w, shift_state, state_slots,
                           cu_seqlens_q, context_lens, num_seqs, num_tokens, width, dt,
                           reinterpret_cast<cudaStream_t>(stream));
}
void b200_depth_mix(float* out, const float* hist, int64_t stride, const float* w, int32_t count, int64_t n,
                    int64_t stream) {
  B200_CHECK_ARG(out && hist && w && count > 0 && stride >= 0 && n >= 0, "depth_mix: bad arguments");
  b200::launch_depth_mix(out, hist, static_cast<size_t>(stride), w, count, static_cast<size_t>(n),
                         reinterpret_cast<cudaStream_t>(stream));
}
}
