// Recurrent sequence mixers with a per-sequence state slot, for ragged steps (a prompt portion of any length or one
// decoded token per sequence): the short causal convolution in front of them, the gated delta rule, and the
// scalar-decay state-space scan (SSD form of Mamba-2).  State lives in fp32 in slot-indexed pools owned by the caller;
// a sequence that starts at position 0 in this step (context == rows of the step) starts from zeros whatever its
// slot held before, so slots can be handed on without clearing.  Everything here is fp32.
//
//   short_conv_silu : y[t, c] = silu(bias[c] + sum_j w[c, j] * x[t - (taps-1) + j, c]); the last taps-1 inputs of a
//                     sequence are its conv state  [slots, taps-1, C].  Token chunks run in parallel; a second small
//                     launch rolls the state forward.
//   delta_rule      : per head, S [dim, vdim]:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
//                     with q, k unit-normalised per head (q also times dim^-1/2), beta = sigmoid(b),
//                     g = exp(-exp(a_log) * softplus(a + dt_bias)).  state [slots, heads, dim, vdim].  In the
//                     channel form g is one decay per head AND key channel (row i of S is multiplied by g[i]), handed
//                     in ready-made (lowrank_decay kind 1 makes it from a low-rank projection).
//   ssd_scan        : per head, S [nstate, vdim]:  dt = softplus(dt_raw + dt_bias);  S <- exp(-exp(a_log) dt) S + dt B x^T;
//                     y = S^T C + D x.  state [slots, heads, nstate, vdim].
//   decay_attn      : per head, S [dim, vdim]:  S <- diag(a_t) S + k_t v_t^T;  o_t = S^T q_t  (linear attention with a decayed
//                     state, no softmax or denominator).  a_t is one constant per head (retention-style fixed decays) or
//                     one value per key channel and token (gated linear attention; lowrank_decay makes it from a
//                     low-rank projection: sigmoid(z)^(1/tau)).  Optional SiLU on q, k, v and scales on q and k.
//                     state [slots, heads, dim, vdim].
// In the scans eight lanes share one column of S (one value channel), each holding every eighth row in registers,
// and walk the sequence's tokens in order: the exact recurrence, no chunked reformulation, so a portion boundary
// cannot change the arithmetic.  The tokens' inputs are staged in shared memory a pass at a time through two buffers
// filled by cp.async, so the walk never waits for global memory.
#include "../../include/b200_vllm.h"
#include "seqmix.cuh"

namespace b200 {
using namespace seqmix;

constexpr int kMaxTaps = 8;

constexpr int kConvChunk = 64;      // tokens per thread

// grid = (channel blocks, sequences, token chunks): every thread convolves one channel over one chunk of a sequence's
// rows; the taps-1 inputs before the chunk come from the rows before it or, at the start of the step, from the
// sequence's state (zeros when the sequence starts here).  out must not alias x.
template <int TAPS>
__global__ void short_conv_silu_kernel(float* __restrict__ out, int ldo, const float* __restrict__ x, int ldx,
                                       const float* __restrict__ taps_w, const float* __restrict__ bias,
                                       const float* __restrict__ state, const int32_t* __restrict__ slots,
                                       const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx, int C) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu[b], t1 = cu[b + 1];
  const int start = t0 + static_cast<int>(blockIdx.z) * kConvChunk;
  if (start >= t1) return;
  const int end = min(t1, start + kConvChunk);
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;
  constexpr int P = TAPS - 1;                  // inputs remembered between tokens
  float w[TAPS], win[P > 0 ? P : 1];
#pragma unroll
  for (int j = 0; j < TAPS; ++j) w[j] = taps_w[static_cast<size_t>(c) * TAPS + j];
  const float* sp = state + static_cast<size_t>(slots[b]) * P * C + c;
#pragma unroll
  for (int j = 0; j < P; ++j) {                // oldest first
    const int idx = start - P + j;
    win[j] = idx >= t0 ? x[static_cast<size_t>(idx) * ldx + c] : (fresh ? 0.f : sp[static_cast<size_t>(P + idx - t0) * C]);
  }
  const float bv = bias ? bias[c] : 0.f;
  for (int t = start; t < end; ++t) {
    const float xv = x[static_cast<size_t>(t) * ldx + c];
    float acc = bv;
#pragma unroll
    for (int j = 0; j < P; ++j) acc += w[j] * win[j];
    acc += w[P] * xv;
    out[static_cast<size_t>(t) * ldo + c] = silu_exact(acc);
#pragma unroll
    for (int j = 0; j + 1 < P; ++j) win[j] = win[j + 1];
    if (P > 0) win[P > 0 ? P - 1 : 0] = xv;
  }
}

// the sequence's last taps-1 inputs become its state (older ones slide over from the previous state)
template <int TAPS>
__global__ void short_conv_state_kernel(const float* __restrict__ x, int ldx, float* __restrict__ state,
                                        const int32_t* __restrict__ slots, const uint32_t* __restrict__ cu,
                                        const uint32_t* __restrict__ ctx, int C) {
  constexpr int P = TAPS - 1;
  const int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
  if (c >= C || P == 0) return;
  const int t0 = cu[b], t1 = cu[b + 1];
  if (t1 <= t0) return;
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;
  float* sp = state + static_cast<size_t>(slots[b]) * P * C + c;
  float keep[P > 0 ? P : 1];
#pragma unroll
  for (int j = 0; j < P; ++j) {
    const int idx = t1 - P + j;
    keep[j] = idx >= t0 ? x[static_cast<size_t>(idx) * ldx + c] : (fresh ? 0.f : sp[static_cast<size_t>(P + idx - t0) * C]);
  }
#pragma unroll
  for (int j = 0; j < P; ++j) sp[static_cast<size_t>(j) * C] = keep[j];
}

// tokens staged in shared memory per pass; there are two such buffers (static shared memory stays under 48 KB for
// the widest state): the next pass's rows arrive by cp.async while the current pass's tokens are walked
constexpr int chunk_for(int rows) { return rows > 128 ? 8 : rows > 64 ? 16 : 32; }
__device__ __forceinline__ void cp_async4(float* smem, const float* gmem) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
               "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async16(float* smem, const float* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
               "l"(gmem)
               : "memory");
}
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
constexpr int kRowSplit = 8;       // lanes that share one column of S (each holds every 8th row)
constexpr int kScanThreads = 128, kScanCols = kScanThreads / kRowSplit;      // columns of S per block

// grid = (column blocks, heads, sequences); block = 128 threads = 16 columns x kRowSplit lanes.  DK = compile-time
// bound of `dim`; a lane holds the rows i = j * kRowSplit + part of its column.
// CHAN: the decay is one value per head, key channel and token, read ready-made from chan_decay [T, heads, dim] (row
// stride ld_decay; a_raw, a_log and dt_bias are not used); otherwise one value per head and token computed here.
template <int DK, bool CHAN>
__global__ void __launch_bounds__(128)
delta_rule_kernel(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k,
                  const float* __restrict__ v, int ld, const float* __restrict__ b_raw,
                  const float* __restrict__ a_raw, int ld_ba, const float* __restrict__ a_log,
                  const float* __restrict__ dt_bias, const float* __restrict__ chan_decay, int ld_decay,
                  float* __restrict__ state, const int32_t* __restrict__ slots,
                  const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx, int heads, int kv_heads, int dim,
                  int vdim) {
  // a third staged row set halves the tokens per pass where the rows are long (static shared memory stays under 48 KB)
  constexpr int RS = kRowSplit, NR = DK / RS, kChunk = (CHAN && DK >= 64) ? chunk_for(DK) / 2 : chunk_for(DK);
  __shared__ float ks[2][kChunk][DK], qs[2][kChunk][DK], vs[2][kChunk][kScanCols], gs[2][kChunk], bs[2][kChunk];
  __shared__ float as[CHAN ? 2 : 1][CHAN ? kChunk : 1][CHAN ? DK : 1];
  const int h = blockIdx.y, b = blockIdx.z;
  const int part = threadIdx.x % RS;
  const int col = blockIdx.x * (blockDim.x / RS) + threadIdx.x / RS;
  const bool live = col < vdim;
  const int t0 = cu[b], t1 = cu[b + 1];
  if (t1 <= t0) return;
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;
  const int hk = h / (heads / kv_heads);
  float* sp = state + ((static_cast<size_t>(slots[b]) * heads + h) * dim) * vdim + col;
  float s[NR];
#pragma unroll
  for (int j = 0; j < NR; ++j) {
    const int i = j * RS + part;
    s[j] = (!fresh && live && i < dim) ? sp[static_cast<size_t>(i) * vdim] : 0.f;
  }
  const float neg_a = CHAN ? 0.f : -expf(a_log[h]), dtb = CHAN ? 0.f : dt_bias[h];
  const float qscale = rsqrtf(static_cast<float>(dim));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  if (dim < DK)                                                           // the padding past `dim` stays zero
    for (int e = threadIdx.x; e < 2 * kChunk * DK; e += kScanThreads) {
      (&ks[0][0][0])[e] = (&qs[0][0][0])[e] = 0.f;
      if (CHAN) (&as[0][0][0])[e] = 0.f;
    }
  for (int e = threadIdx.x; e < 2 * kChunk * kScanCols; e += kScanThreads) (&vs[0][0][0])[e] = 0.f;
  __syncthreads();
  // raw rows of one pass -> buffer `buf` (asynchronous; committed as one group)
  auto fetch = [&](int c0, int buf) {
    const int n = min(kChunk, t1 - c0);
    for (int e = threadIdx.x; e < n * dim; e += kScanThreads) {
      const int r = e / dim, i = e - r * dim;
      cp_async4(&ks[buf][r][i], k + static_cast<size_t>(c0 + r) * ld + hk * dim + i);
      cp_async4(&qs[buf][r][i], q + static_cast<size_t>(c0 + r) * ld + hk * dim + i);
      if (CHAN) cp_async4(&as[buf][r][i], chan_decay + static_cast<size_t>(c0 + r) * ld_decay + h * dim + i);
    }
    for (int e = threadIdx.x; e < n * kScanCols; e += kScanThreads) {
      const int r = e / kScanCols, c = blockIdx.x * kScanCols + e % kScanCols;
      if (c < vdim) cp_async4(&vs[buf][r][e % kScanCols], v + static_cast<size_t>(c0 + r) * ld + h * vdim + c);
    }
    if (threadIdx.x < n) {
      cp_async4(&bs[buf][threadIdx.x], b_raw + static_cast<size_t>(c0 + threadIdx.x) * ld_ba + h);
      if (!CHAN) cp_async4(&gs[buf][threadIdx.x], a_raw + static_cast<size_t>(c0 + threadIdx.x) * ld_ba + h);
    }
    cp_async_commit();
  };
  fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += kChunk, buf ^= 1) {
    const int n = min(kChunk, t1 - c0);
    if (c0 + kChunk < t1) {
      fetch(c0 + kChunk, buf ^ 1);         // the other buffer's tokens were walked before the last barrier
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // unit-normalise q, k of the pass in place: one warp per token row
    for (int r = warp; r < n; r += nw) {
      float sk = 0.f, sq = 0.f;
      for (int i = lane; i < dim; i += 32) {
        sk += ks[buf][r][i] * ks[buf][r][i];
        sq += qs[buf][r][i] * qs[buf][r][i];
      }
      sk = lanes_sum(sk);
      sq = lanes_sum(sq);
      const float ik = 1.f / sqrtf(sk + 1e-6f), iq = qscale / sqrtf(sq + 1e-6f);
      for (int i = lane; i < dim; i += 32) {
        ks[buf][r][i] *= ik;
        qs[buf][r][i] *= iq;
      }
      if (lane == 0) {
        bs[buf][r] = sigmoid_f(bs[buf][r]);
        if (!CHAN) gs[buf][r] = expf(neg_a * softplus_f(gs[buf][r] + dtb));
      }
    }
    __syncthreads();
    for (int r = 0; r < n; ++r) {          // every lane runs the shuffles; dead columns carry zeros
      const float vv = vs[buf][r][threadIdx.x / RS];
      const float g = CHAN ? 0.f : gs[buf][r];
      float d0 = 0.f, d1 = 0.f;
#pragma unroll
      for (int j = 0; j < NR; j += 2) {
        s[j] *= CHAN ? as[CHAN ? buf : 0][CHAN ? r : 0][CHAN ? j * RS + part : 0] : g;
        d0 += ks[buf][r][j * RS + part] * s[j];
        if (j + 1 < NR) {
          s[j + 1] *= CHAN ? as[CHAN ? buf : 0][CHAN ? r : 0][CHAN ? (j + 1) * RS + part : 0] : g;
          d1 += ks[buf][r][(j + 1) * RS + part] * s[j + 1];
        }
      }
      float dot = d0 + d1;
#pragma unroll
      for (int o = 1; o < RS; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = bs[buf][r] * (vv - dot);
      float o0 = 0.f, o1 = 0.f;
#pragma unroll
      for (int j = 0; j < NR; j += 2) {
        s[j] += ks[buf][r][j * RS + part] * u;
        o0 += qs[buf][r][j * RS + part] * s[j];
        if (j + 1 < NR) {
          s[j + 1] += ks[buf][r][(j + 1) * RS + part] * u;
          o1 += qs[buf][r][(j + 1) * RS + part] * s[j + 1];
        }
      }
      float o = o0 + o1;
#pragma unroll
      for (int x = 1; x < RS; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (live && part == 0) out[(static_cast<size_t>(c0 + r) * heads + h) * vdim + col] = o;
    }
    __syncthreads();                       // this buffer is refilled by the next pass's fetch
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      const int i = j * RS + part;
      if (i < dim) sp[static_cast<size_t>(i) * vdim] = s[j];
    }
  }
}

template <int NS>
__global__ void __launch_bounds__(128)
ssd_scan_kernel(float* __restrict__ out, const float* __restrict__ x, const float* __restrict__ Bm,
                const float* __restrict__ Cm, int ld, const float* __restrict__ dt_raw, int ld_dt,
                const float* __restrict__ a_log, const float* __restrict__ dt_bias, const float* __restrict__ d_skip,
                float* __restrict__ state, const int32_t* __restrict__ slots, const uint32_t* __restrict__ cu,
                const uint32_t* __restrict__ ctx, int heads, int groups, int nstate, int vdim) {
  constexpr int RS = kRowSplit, NR = NS / RS, kChunk = chunk_for(NS);
  __shared__ float Bs[2][kChunk][NS], Cs[2][kChunk][NS], xs[2][kChunk][kScanCols], dts[2][kChunk], das[2][kChunk];
  const int h = blockIdx.y, b = blockIdx.z;
  const int part = threadIdx.x % RS;
  const int col = blockIdx.x * (blockDim.x / RS) + threadIdx.x / RS;
  const bool live = col < vdim;
  const int t0 = cu[b], t1 = cu[b + 1];
  if (t1 <= t0) return;
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;
  const int g = h / (heads / groups);
  float* sp = state + ((static_cast<size_t>(slots[b]) * heads + h) * nstate) * vdim + col;
  float s[NR];
#pragma unroll
  for (int j = 0; j < NR; ++j) {
    const int i = j * RS + part;
    s[j] = (!fresh && live && i < nstate) ? sp[static_cast<size_t>(i) * vdim] : 0.f;
  }
  const float neg_a = -expf(a_log[h]), dtb = dt_bias[h], dsk = d_skip ? d_skip[h] : 0.f;
  if (nstate < NS)                                                        // the padding past `nstate` stays zero
    for (int e = threadIdx.x; e < 2 * kChunk * NS; e += kScanThreads) (&Bs[0][0][0])[e] = (&Cs[0][0][0])[e] = 0.f;
  for (int e = threadIdx.x; e < 2 * kChunk * kScanCols; e += kScanThreads) (&xs[0][0][0])[e] = 0.f;
  __syncthreads();
  // raw rows of one pass -> buffer `buf` (asynchronous; committed as one group)
  auto fetch = [&](int c0, int buf) {
    const int n = min(kChunk, t1 - c0);
    for (int e = threadIdx.x; e < n * nstate; e += kScanThreads) {
      const int r = e / nstate, i = e - r * nstate;
      cp_async4(&Bs[buf][r][i], Bm + static_cast<size_t>(c0 + r) * ld + g * nstate + i);
      cp_async4(&Cs[buf][r][i], Cm + static_cast<size_t>(c0 + r) * ld + g * nstate + i);
    }
    for (int e = threadIdx.x; e < n * kScanCols; e += kScanThreads) {
      const int r = e / kScanCols, c = blockIdx.x * kScanCols + e % kScanCols;
      if (c < vdim) cp_async4(&xs[buf][r][e % kScanCols], x + static_cast<size_t>(c0 + r) * ld + h * vdim + c);
    }
    if (threadIdx.x < n) cp_async4(&dts[buf][threadIdx.x], dt_raw + static_cast<size_t>(c0 + threadIdx.x) * ld_dt + h);
    cp_async_commit();
  };
  fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += kChunk, buf ^= 1) {
    const int n = min(kChunk, t1 - c0);
    if (c0 + kChunk < t1) {
      fetch(c0 + kChunk, buf ^ 1);         // the other buffer's tokens were walked before the last barrier
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    if (threadIdx.x < n) {
      const float dt = softplus_f(dts[buf][threadIdx.x] + dtb);
      dts[buf][threadIdx.x] = dt;
      das[buf][threadIdx.x] = expf(neg_a * dt);
    }
    __syncthreads();
    for (int r = 0; r < n; ++r) {
      const float xv = xs[buf][r][threadIdx.x / RS];
      const float a = das[buf][r], dx = dts[buf][r] * xv;
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int j = 0; j < NR; j += 2) {
        s[j] = a * s[j] + dx * Bs[buf][r][j * RS + part];
        y0 += Cs[buf][r][j * RS + part] * s[j];
        if (j + 1 < NR) {
          s[j + 1] = a * s[j + 1] + dx * Bs[buf][r][(j + 1) * RS + part];
          y1 += Cs[buf][r][(j + 1) * RS + part] * s[j + 1];
        }
      }
      float y = y0 + y1;
#pragma unroll
      for (int o = 1; o < RS; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (live && part == 0) out[(static_cast<size_t>(c0 + r) * heads + h) * vdim + col] = y + dsk * xv;
    }
    __syncthreads();                       // this buffer is refilled by the next pass's fetch
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      const int i = j * RS + part;
      if (i < nstate) sp[static_cast<size_t>(i) * vdim] = s[j];
    }
  }
}


// out[t, c] = sigmoid(z)^(1 / tau) with z = bias[c] + sum_r w2[c, r] * low[t, r]: the per-channel decay of gated linear
// attention from the low-rank half of its projection.  Computed as exp(log sigmoid(z) / tau), all fp32.
// a_log != NULL (kind 1): out[t, c] = exp(-exp(a_log[c / a_period]) * softplus(z)), the decay of a gated delta rule per
// head and key channel.
// grid = (channel blocks, token tiles): a thread owns one channel and kDecayTile tokens; the tokens' low-rank rows sit in
// shared memory, the channel's row of w2 is read once per tile (each thread whole sectors), the stores are coalesced.
constexpr int kDecayTile = 16;
__global__ void __launch_bounds__(256)
lowrank_decay_kernel(float* __restrict__ out, const float* __restrict__ low, int ld_low, const float* __restrict__ w2,
                     const float* __restrict__ bias, float inv_tau, const float* __restrict__ a_log, int a_period, int T,
                     int C, int rank) {
  extern __shared__ float lr[];          // [kDecayTile][rank]
  const int t0 = blockIdx.y * kDecayTile, nt = min(kDecayTile, T - t0);
  for (int e = threadIdx.x; e < nt * rank; e += blockDim.x)
    lr[e] = low[static_cast<size_t>(t0 + e / rank) * ld_low + e % rank];
  __syncthreads();
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  float z[kDecayTile];
  const float b = bias ? bias[c] : 0.f;
#pragma unroll
  for (int i = 0; i < kDecayTile; ++i) z[i] = b;
  const float* w = w2 + static_cast<size_t>(c) * rank;
  for (int r = 0; r < rank; ++r) {
    const float wv = w[r];
#pragma unroll
    for (int i = 0; i < kDecayTile; ++i) z[i] += wv * lr[(i < nt ? i : 0) * rank + r];
  }
#pragma unroll
  for (int i = 0; i < kDecayTile; ++i) {
    if (i >= nt) break;
    if (a_log) {
      out[static_cast<size_t>(t0 + i) * C + c] = expf(-expf(a_log[c / a_period]) * softplus_f(z[i]));
      continue;
    }
    const float ls = z[i] >= 0.f ? -log1pf(expf(-z[i])) : z[i] - log1pf(expf(z[i]));
    out[static_cast<size_t>(t0 + i) * C + c] = expf(ls * inv_tau);
  }
}

// tokens per pass of the decayed-state scan (two buffers of this many; a per-channel decay stages a third row set)
constexpr int decay_chunk_for(int rows, bool chan) { return (chan ? 8 : 16) / (rows > 128 ? 2 : 1); }
constexpr int kDecayPad = 4;       // floats between the row segments of two lanes: 16-byte loads without bank conflicts

// grid = (column blocks, heads, sequences); block = 128 threads = 16 columns x kRowSplit lanes.  Unlike the scans above
// a lane holds NR = DK / 8 CONSECUTIVE rows of its column (rows part * NR ..), and a token's k / q / decay rows lie in
// shared memory as eight padded segments, so a lane reads its segment with 16-byte loads; four tokens are walked per
// round so that their read-out reductions (shuffles) overlap the next tokens' state updates.
// CHAN: the decay is per key channel and token (chan_decay [T, heads, dim], row stride ld_decay); otherwise one
// constant per head (head_decay [heads]).
template <int DK, bool CHAN>
__global__ void __launch_bounds__(128)
decay_attn_kernel(float* __restrict__ out, const float* __restrict__ q, const float* __restrict__ k,
                  const float* __restrict__ v, int ld, const float* __restrict__ head_decay,
                  const float* __restrict__ chan_decay, int ld_decay, float q_scale, float k_scale, int act,
                  float* __restrict__ state, const int32_t* __restrict__ slots, const uint32_t* __restrict__ cu,
                  const uint32_t* __restrict__ ctx, int heads, int dim, int vdim) {
  constexpr int RS = kRowSplit, NR = DK / RS, SEG = NR + kDecayPad, DKP = RS * SEG, kChunk = decay_chunk_for(DK, CHAN);
  constexpr int UN = 4;              // tokens per round of the walk
  __shared__ __align__(16) float ks[2][kChunk][DKP], qs[2][kChunk][DKP],
      as[CHAN ? 2 : 1][CHAN ? kChunk : 1][CHAN ? DKP : 4], vs[2][kChunk][kScanCols];
  const int h = blockIdx.y, b = blockIdx.z;
  const int part = threadIdx.x % RS;
  const int col = blockIdx.x * (blockDim.x / RS) + threadIdx.x / RS;
  const bool live = col < vdim;
  const int t0 = cu[b], t1 = cu[b + 1];
  if (t1 <= t0) return;
  const bool fresh = static_cast<int>(ctx[b]) == t1 - t0;
  float* sp = state + ((static_cast<size_t>(slots[b]) * heads + h) * dim) * vdim + col;
  float s[NR];
#pragma unroll
  for (int j = 0; j < NR; ++j) {
    const int i = part * NR + j;
    s[j] = (!fresh && live && i < dim) ? sp[static_cast<size_t>(i) * vdim] : 0.f;
  }
  const float hd = CHAN ? 0.f : head_decay[h];
  if (dim < DK)                          // rows past `dim` stay zero (the padding between segments is never read)
    for (int e = threadIdx.x; e < 2 * kChunk * DKP; e += kScanThreads) {
      (&ks[0][0][0])[e] = (&qs[0][0][0])[e] = 0.f;
      if (CHAN) (&as[0][0][0])[e] = 0.f;
    }
  for (int e = threadIdx.x; e < 2 * kChunk * kScanCols; e += kScanThreads) (&vs[0][0][0])[e] = 0.f;
  __syncthreads();
  auto at = [](int i) { return i + (i / NR) * kDecayPad; };       // place of row i in a padded token row
  // 16-byte copies where four consecutive rows share a segment and every source address is 16-byte aligned
  const bool wide = NR % 4 == 0 && dim % 4 == 0 && ld % 4 == 0 && (!CHAN || ld_decay % 4 == 0) &&
                    ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                      (CHAN ? reinterpret_cast<uintptr_t>(chan_decay) : 0)) & 15) == 0;
  auto fetch = [&](int c0, int buf) {
    const int n = min(kChunk, t1 - c0);
    if (wide) {
      const int d4 = dim / 4;
      for (int e = threadIdx.x; e < n * d4; e += kScanThreads) {
        const int r = e / d4, i = (e - r * d4) * 4;
        cp_async16(&ks[buf][r][at(i)], k + static_cast<size_t>(c0 + r) * ld + h * dim + i);
        cp_async16(&qs[buf][r][at(i)], q + static_cast<size_t>(c0 + r) * ld + h * dim + i);
        if (CHAN) cp_async16(&as[buf][r][at(i)], chan_decay + static_cast<size_t>(c0 + r) * ld_decay + h * dim + i);
      }
    } else {
      for (int e = threadIdx.x; e < n * dim; e += kScanThreads) {
        const int r = e / dim, i = e - r * dim;
        cp_async4(&ks[buf][r][at(i)], k + static_cast<size_t>(c0 + r) * ld + h * dim + i);
        cp_async4(&qs[buf][r][at(i)], q + static_cast<size_t>(c0 + r) * ld + h * dim + i);
        if (CHAN) cp_async4(&as[buf][r][at(i)], chan_decay + static_cast<size_t>(c0 + r) * ld_decay + h * dim + i);
      }
    }
    for (int e = threadIdx.x; e < n * kScanCols; e += kScanThreads) {
      const int r = e / kScanCols, c = blockIdx.x * kScanCols + e % kScanCols;
      if (c < vdim) cp_async4(&vs[buf][r][e % kScanCols], v + static_cast<size_t>(c0 + r) * ld + h * vdim + c);
    }
    cp_async_commit();
  };
  // NR floats of a lane's segment: 16-byte loads where the segment is a whole number of them
  auto load_seg = [&](float* dst, const float* src) {
    if constexpr (NR % 4 == 0) {
#pragma unroll
      for (int j = 0; j < NR; j += 4) {
        const float4 x = *reinterpret_cast<const float4*>(src + j);
        dst[j] = x.x; dst[j + 1] = x.y; dst[j + 2] = x.z; dst[j + 3] = x.w;
      }
    } else {
#pragma unroll
      for (int j = 0; j < NR; ++j) dst[j] = src[j];
    }
  };
  fetch(t0, 0);
  int buf = 0;
  for (int c0 = t0; c0 < t1; c0 += kChunk, buf ^= 1) {
    const int n = min(kChunk, t1 - c0);
    if (c0 + kChunk < t1) {
      fetch(c0 + kChunk, buf ^ 1);         // the other buffer's tokens were walked before the last barrier
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    // activation and scales of the pass, in place
    if (act || q_scale != 1.f || k_scale != 1.f) {
      for (int e = threadIdx.x; e < n * dim; e += kScanThreads) {
        const int r = e / dim, i = at(e - r * dim);
        const float kv = ks[buf][r][i], qv = qs[buf][r][i];
        ks[buf][r][i] = (act ? silu_exact(kv) : kv) * k_scale;
        qs[buf][r][i] = (act ? silu_exact(qv) : qv) * q_scale;
      }
      if (act)
        for (int e = threadIdx.x; e < n * kScanCols; e += kScanThreads)
          vs[buf][e / kScanCols][e % kScanCols] = silu_exact(vs[buf][e / kScanCols][e % kScanCols]);
      __syncthreads();
    }
    for (int r = 0; r < n; r += UN) {      // n is the same in every thread: the guards below do not diverge
      float y[UN];
#pragma unroll
      for (int u = 0; u < UN; ++u) {
        y[u] = 0.f;
        if (r + u < n) {
          float kr[NR], qr[NR], ar[CHAN ? NR : 1];
          load_seg(kr, &ks[buf][r + u][part * SEG]);
          load_seg(qr, &qs[buf][r + u][part * SEG]);
          if (CHAN) load_seg(ar, &as[buf][r + u][part * SEG]);
          const float vv = vs[buf][r + u][threadIdx.x / RS];
          float y0 = 0.f, y1 = 0.f;
#pragma unroll
          for (int j = 0; j < NR; j += 2) {
            s[j] = (CHAN ? ar[j] : hd) * s[j] + kr[j] * vv;
            y0 += qr[j] * s[j];
            if (j + 1 < NR) {
              s[j + 1] = (CHAN ? ar[CHAN ? j + 1 : 0] : hd) * s[j + 1] + kr[j + 1] * vv;
              y1 += qr[j + 1] * s[j + 1];
            }
          }
          y[u] = y0 + y1;
        }
      }
#pragma unroll
      for (int o = 1; o < RS; o <<= 1)
#pragma unroll
        for (int u = 0; u < UN; ++u) y[u] += __shfl_xor_sync(0xffffffffu, y[u], o);
#pragma unroll
      for (int u = 0; u < UN; ++u)           // lane `u` of the column stores token r + u
        if (live && part == u && r + u < n) out[(static_cast<size_t>(c0 + r + u) * heads + h) * vdim + col] = y[u];
    }
    __syncthreads();                       // this buffer is refilled by the next pass's fetch
  }
  if (live) {
#pragma unroll
    for (int j = 0; j < NR; ++j) {
      const int i = part * NR + j;
      if (i < dim) sp[static_cast<size_t>(i) * vdim] = s[j];
    }
  }
}

void launch_short_conv_silu(float* out, int ldo, const float* x, int ldx, const float* taps_w, const float* bias,
                            float* state, const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs,
                            int num_rows, int C, int taps, cudaStream_t st_) {
  if (num_seqs <= 0 || C <= 0 || num_rows <= 0) return;
  if (taps < 1 || taps > kMaxTaps) {
    set_error(1, "short_conv: between 1 and 8 taps are supported");
    return;
  }
  if (out == x) {
    set_error(1, "short_conv: the output must not alias the input (chunks of a sequence run in parallel)");
    return;
  }
  const dim3 grid((C + 127) / 128, num_seqs, (num_rows + kConvChunk - 1) / kConvChunk);
  const dim3 sgrid((C + 127) / 128, num_seqs);
#define B200_CONV(K)                                                                                              \
  case K:                                                                                                         \
    short_conv_silu_kernel<K><<<grid, 128, 0, st_>>>(out, ldo, x, ldx, taps_w, bias, state, slots, cu, ctx, C); \
    if (K > 1) short_conv_state_kernel<K><<<sgrid, 128, 0, st_>>>(x, ldx, state, slots, cu, ctx, C);           \
    break
  switch (taps) {
    B200_CONV(1); B200_CONV(2); B200_CONV(3); B200_CONV(4); B200_CONV(5); B200_CONV(6); B200_CONV(7); B200_CONV(8);
  }
#undef B200_CONV
  B200_CUDA_LAUNCH_CHECK();
}

void launch_delta_rule(float* out, const float* q, const float* k, const float* v, int ld, const float* b_raw,
                       const float* a_raw, int ld_ba, const float* a_log, const float* dt_bias, const float* chan_decay,
                       int ld_decay, float* state, const int32_t* slots, const uint32_t* cu, const uint32_t* ctx,
                       int num_seqs, int heads, int kv_heads, int dim, int vdim, cudaStream_t st_) {
  if (num_seqs <= 0) return;
  const int th = kScanThreads;
  const dim3 grid((vdim + kScanCols - 1) / kScanCols, heads, num_seqs);
#define B200_DELTA2(DK, CH)                                                                                        \
  delta_rule_kernel<DK, CH><<<grid, th, 0, st_>>>(out, q, k, v, ld, b_raw, a_raw, ld_ba, a_log, dt_bias, chan_decay, \
                                                  ld_decay, state, slots, cu, ctx, heads, kv_heads, dim, vdim)
#define B200_DELTA(DK)                     \
  {                                        \
    if (chan_decay) B200_DELTA2(DK, true); \
    else B200_DELTA2(DK, false);           \
  }
  if (dim <= 16) B200_DELTA(16)
  else if (dim <= 32) B200_DELTA(32)
  else if (dim <= 64) B200_DELTA(64)
  else if (dim <= 128) B200_DELTA(128)
  else if (dim <= 256) B200_DELTA(256)
  else {
    set_error(1, "delta_rule: key dimension above 256 is not supported");
    return;
  }
#undef B200_DELTA
#undef B200_DELTA2
  B200_CUDA_LAUNCH_CHECK();
}

void launch_ssd_scan(float* out, const float* x, const float* Bm, const float* Cm, int ld, const float* dt_raw,
                     int ld_dt, const float* a_log, const float* dt_bias, const float* d_skip, float* state,
                     const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int heads, int groups,
                     int nstate, int vdim, cudaStream_t st_) {
  if (num_seqs <= 0) return;
  const int th = kScanThreads;
  const dim3 grid((vdim + kScanCols - 1) / kScanCols, heads, num_seqs);
#define B200_SSD(NS)                                                                                               \
  ssd_scan_kernel<NS><<<grid, th, 0, st_>>>(out, x, Bm, Cm, ld, dt_raw, ld_dt, a_log, dt_bias, d_skip, state, slots, \
                                            cu, ctx, heads, groups, nstate, vdim)
  if (nstate <= 16) B200_SSD(16);
  else if (nstate <= 32) B200_SSD(32);
  else if (nstate <= 64) B200_SSD(64);
  else if (nstate <= 128) B200_SSD(128);
  else if (nstate <= 256) B200_SSD(256);
  else {
    set_error(1, "ssd_scan: state size above 256 is not supported");
    return;
  }
#undef B200_SSD
  B200_CUDA_LAUNCH_CHECK();
}


void launch_lowrank_decay(float* out, const float* low, int ld_low, const float* w2, const float* bias, float tau,
                          const float* a_log, int a_period, int T, int C, int rank, cudaStream_t st_) {
  if (T <= 0 || C <= 0) return;
  if (rank <= 0 || rank > 512) {
    set_error(1, "lowrank_decay: the rank must be between 1 and 512");
    return;
  }
  const dim3 grid((C + 255) / 256, (T + kDecayTile - 1) / kDecayTile);
  lowrank_decay_kernel<<<grid, 256, static_cast<size_t>(kDecayTile) * rank * 4, st_>>>(
      out, low, ld_low, w2, bias, a_log ? 0.f : 1.f / tau, a_log, a_period > 0 ? a_period : 1, T, C, rank);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_decay_attn(float* out, const float* q, const float* k, const float* v, int ld, const float* head_decay,
                       const float* chan_decay, int ld_decay, float q_scale, float k_scale, int act, float* state,
                       const int32_t* slots, const uint32_t* cu, const uint32_t* ctx, int num_seqs, int heads, int dim,
                       int vdim, cudaStream_t st_) {
  if (num_seqs <= 0) return;
  const int th = kScanThreads;
  const dim3 grid((vdim + kScanCols - 1) / kScanCols, heads, num_seqs);
#define B200_DECAY2(DK, CH)                                                                                          \
  decay_attn_kernel<DK, CH><<<grid, th, 0, st_>>>(out, q, k, v, ld, head_decay, chan_decay, ld_decay, q_scale, k_scale, \
                                                  act, state, slots, cu, ctx, heads, dim, vdim)
#define B200_DECAY(DK)          \
  {                             \
    if (chan_decay) B200_DECAY2(DK, true); \
    else B200_DECAY2(DK, false);           \
  }
  if (dim <= 16) B200_DECAY(16)
  else if (dim <= 32) B200_DECAY(32)
  else if (dim <= 64) B200_DECAY(64)
  else if (dim <= 128) B200_DECAY(128)
  else if (dim <= 256) B200_DECAY(256)
  else {
    set_error(1, "decay_attn: key dimension above 256 is not supported");
    return;
  }
#undef B200_DECAY
#undef B200_DECAY2
  B200_CUDA_LAUNCH_CHECK();
}

}  // namespace b200

extern "C" {
void b200_short_conv_silu(float* out, int32_t ldo, const float* x, int32_t ldx, const float* taps_w, const float* bias,
                          float* state, const int32_t* state_slots, const uint32_t* cu_seqlens_q,
                          const uint32_t* context_lens, int32_t num_seqs, int32_t num_tokens, int32_t channels,
                          int32_t taps, int64_t stream) {
  B200_CHECK_ARG(out && x && taps_w && state && state_slots && cu_seqlens_q && context_lens, "short_conv: bad arguments");
  b200::launch_short_conv_silu(out, ldo, x, ldx, taps_w, bias, state, state_slots, cu_seqlens_q, context_lens, num_seqs,
                               num_tokens, channels, taps, reinterpret_cast<cudaStream_t>(stream));
}
void b200_delta_rule(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* b_raw,
                     const float* a_raw, int32_t ld_ba, const float* a_log, const float* dt_bias, float* state,
                     const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                     int32_t num_seqs, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int64_t stream) {
  B200_CHECK_ARG(out && q && k && v && b_raw && a_raw && a_log && dt_bias && state && state_slots && cu_seqlens_q &&
                     context_lens && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0,
                 "delta_rule: bad arguments");
  b200::launch_delta_rule(out, q, k, v, ld, b_raw, a_raw, ld_ba, a_log, dt_bias, nullptr, 0, state, state_slots,
                          cu_seqlens_q, context_lens, num_seqs, heads, kv_heads, dim, vdim,
                          reinterpret_cast<cudaStream_t>(stream));
}
void b200_delta_rule_chan(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* b_raw,
                          int32_t ld_b, const float* chan_decay, int32_t ld_decay, float* state,
                          const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                          int32_t num_seqs, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int64_t stream) {
  B200_CHECK_ARG(out && q && k && v && b_raw && chan_decay && state && state_slots && cu_seqlens_q && context_lens &&
                     heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0,
                 "delta_rule_chan: bad arguments");
  b200::launch_delta_rule(out, q, k, v, ld, b_raw, nullptr, ld_b, nullptr, nullptr, chan_decay, ld_decay, state,
                          state_slots, cu_seqlens_q, context_lens, num_seqs, heads, kv_heads, dim, vdim,
                          reinterpret_cast<cudaStream_t>(stream));
}
void b200_ssd_scan(float* out, const float* x, const float* Bm, const float* Cm, int32_t ld, const float* dt_raw,
                   int32_t ld_dt, const float* a_log, const float* dt_bias, const float* d_skip, float* state,
                   const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                   int32_t num_seqs, int32_t heads, int32_t groups, int32_t nstate, int32_t vdim, int64_t stream) {
  B200_CHECK_ARG(out && x && Bm && Cm && dt_raw && a_log && dt_bias && state && state_slots && cu_seqlens_q &&
                     context_lens && heads > 0 && groups > 0 && heads % groups == 0 && nstate > 0 && vdim > 0,
                 "ssd_scan: bad arguments");
  b200::launch_ssd_scan(out, x, Bm, Cm, ld, dt_raw, ld_dt, a_log, dt_bias, d_skip, state, state_slots, cu_seqlens_q,
                        context_lens, num_seqs, heads, groups, nstate, vdim, reinterpret_cast<cudaStream_t>(stream));
}
void b200_lowrank_decay(float* out, const float* low, int32_t ld_low, const float* w2, const float* bias, float tau,
                         int32_t num_tokens, int32_t channels, int32_t rank, int64_t stream) {
  B200_CHECK_ARG(out && low && w2 && tau > 0.f && channels > 0 && rank > 0 && rank <= 512, "lowrank_decay: bad arguments (rank up to 512)");
  b200::launch_lowrank_decay(out, low, ld_low, w2, bias, tau, nullptr, 1, num_tokens, channels, rank,
                             reinterpret_cast<cudaStream_t>(stream));
}
void b200_lowrank_decay_ex(float* out, const float* low, int32_t ld_low, const float* w2, const float* bias, float tau,
                           int32_t kind, const float* a_log, int32_t a_period, int32_t num_tokens, int32_t channels,
                           int32_t rank, int64_t stream) {
  B200_CHECK_ARG(out && low && w2 && channels > 0 && rank > 0 && rank <= 512 &&
                     (kind == 0 ? tau > 0.f : (kind == 1 && a_log && a_period > 0 && channels % a_period == 0)),
                 "lowrank_decay: bad arguments (rank up to 512; kind 0 needs tau, kind 1 a_log)");
  b200::launch_lowrank_decay(out, low, ld_low, w2, bias, tau, kind == 1 ? a_log : nullptr, a_period, num_tokens, channels,
                             rank, reinterpret_cast<cudaStream_t>(stream));
}
void b200_decay_attn(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* head_decay,
                     const float* chan_decay, int32_t ld_decay, float q_scale, float k_scale, int32_t act, float* state,
                     const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                     int32_t num_seqs, int32_t heads, int32_t dim, int32_t vdim, int64_t stream) {
  B200_CHECK_ARG(out && q && k && v && ((head_decay != nullptr) != (chan_decay != nullptr)) && state && state_slots &&
                     cu_seqlens_q && context_lens && heads > 0 && dim > 0 && vdim > 0,
                 "decay_attn: bad arguments (exactly one of head_decay / chan_decay)");
  b200::launch_decay_attn(out, q, k, v, ld, head_decay, chan_decay, ld_decay, q_scale, k_scale, act, state, state_slots,
                          cu_seqlens_q, context_lens, num_seqs, heads, dim, vdim, reinterpret_cast<cudaStream_t>(stream));
}
}
