// Routed mixture of experts for ragged steps: softmax router with top-k selection, grouping of (token, choice) pairs
// by expert, the experts' gated feed-forward as two grouped matrix products, and the weighted sum back into the
// fp32 residual stream.
//
//   route    : s = softmax(logits) over all experts (fp32); the `top` largest choice scores (ties: lowest index) keep
//              their own probability times `scale`; nothing is renormalised.  The choice score is s plus an optional
//              per-expert bias; with groups, the experts form equal runs of neighbours, a run's score is its largest
//              choice score, and members of all but the `keep` best runs cannot be chosen.
//   sort     : pair p = token * top + choice; pairs are bucketed by expert into slots [off[e], off[e+1]).  The order
//              inside a bucket is arbitrary and does not influence any result: every pair is one independent row.
//   gate_up  : act[slot, f] = silu(h[token] . Wg[e, f]) * (h[token] . Wu[e, f]);  W_gate_up [E, 2F, width] (gate rows
//              first), h in the activation dtype, fp32 accumulation, act stored in the activation dtype.  Ungated
//              experts: act[slot, f] = relu(h[token] . Wu[e, f])^2, W_up [E, F, width].
//   down     : y[slot, d] = act[slot] . Wd[e, d];  W_down [E, width, F]; fp32 out.
//   combine  : x[token] (+)= sum_choice w[token, choice] * y[slot(token, choice)], choices added in order (no atomics).
//              Router outputs past the last real expert are identity experts: y = the token's own input row.
// The grouped products run on the tensor cores (mma.sync m16n8k16, bf16 x bf16 -> fp32) for bf16 activations and as
// plain fp32 FMAs for fp32 activations; both walk K in the same order for a row wherever the row sits in a tile.
#include "../../include/b200_vllm.h"
#include "seqmix.cuh"

namespace b200 {
using namespace seqmix;

// one warp per token.  sm per warp: s[E] (probabilities) | c[E] (choice scores; -inf: not available) | gs[groups]
__global__ void moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ bias, int T, int E, int top,
                                 int groups, int keep, float scale, int32_t* __restrict__ top_idx,
                                 float* __restrict__ top_w) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const int t = blockIdx.x * nw + warp;
  if (t >= T) return;
  float* s = sm + static_cast<size_t>(warp) * (2 * E + groups);
  float* c = s + E;
  float* gs = c + E;
  const float* z = logits + static_cast<size_t>(t) * E;
  float mx = -INFINITY;
  for (int e = lane; e < E; e += 32) mx = fmaxf(mx, z[e]);
  mx = lanes_max(mx);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(z[e] - mx);
    s[e] = p;
    sum += p;
  }
  sum = lanes_sum(sum);
  __syncwarp();
  for (int e = lane; e < E; e += 32) {
    const float p = s[e] / sum;
    s[e] = p;
    c[e] = p + (bias ? bias[e] : 0.f);
  }
  __syncwarp();
  if (groups > 0) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -INFINITY;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, c[e]);
      gs[g] = best;
    }
    __syncwarp();
    // a run stays available while fewer than `keep` runs beat it (a tie goes to the lower index)
    for (int g = lane; g < groups; g += 32) {
      int ahead = 0;
      for (int o = 0; o < groups; ++o) ahead += (gs[o] > gs[g] || (gs[o] == gs[g] && o < g)) ? 1 : 0;
      if (ahead >= keep)
        for (int e = g * per; e < (g + 1) * per; ++e) c[e] = -INFINITY;
    }
    __syncwarp();
  }
  for (int j = 0; j < top; ++j) {
    float best = -INFINITY;
    int bi = E;
    for (int e = lane; e < E; e += 32) {
      const float p = c[e];
      if (p > best) {          // ascending e per lane: the lowest index wins a tie inside a lane
        best = p;
        bi = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) {
        best = ob;
        bi = oi;
      }
    }
    if (lane == 0) {
      if (bi >= E) bi = 0;     // fewer available experts than `top` (rejected by the launcher; keeps the index valid)
      top_idx[static_cast<size_t>(t) * top + j] = bi;
      top_w[static_cast<size_t>(t) * top + j] = s[bi] * scale;
      c[bi] = -INFINITY;
    }
    __syncwarp();
  }
}

// single block: histogram, exclusive scan, scatter
__global__ void moe_sort_kernel(const int32_t* __restrict__ top_idx, int pairs, int E, int32_t* __restrict__ expert_off,
                                int32_t* __restrict__ pair_of_slot, int32_t* __restrict__ slot_of_pair) {
  extern __shared__ int cnt[];       // [E] counts, then cursors
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&cnt[top_idx[p]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      expert_off[e] = run;
      cnt[e] = run;
      run += c;
    }
    expert_off[E] = run;
  }
  __syncthreads();
  for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
    const int slot = atomicAdd(&cnt[top_idx[p]], 1);
    pair_of_slot[slot] = p;
    slot_of_pair[p] = slot;
  }
}

constexpr int TM = 32, TN = 32, TK = 32;

// block tile -> (expert, first slot, rows); false when the tile index is past the last bucket
__device__ __forceinline__ bool find_tile(const int32_t* __restrict__ off, int E, int tile, int* e_out, int* s0,
                                          int* rows) {
  int acc = 0;
  for (int e = 0; e < E; ++e) {
    const int n = off[e + 1] - off[e];
    const int tiles = (n + TM - 1) / TM;
    if (tile < acc + tiles) {
      const int k = tile - acc;
      *e_out = e;
      *s0 = off[e] + k * TM;
      *rows = min(TM, n - k * TM);
      return true;
    }
    acc += tiles;
  }
  return false;
}

// ACT: 0 = plain product over slot rows, fp32 out (the down projection); 1 = gathered token rows, two weight matrices,
// SiLU(gate) * up; 2 = gathered token rows, one matrix, relu(.)^2.  ACT != 0 stores the activation dtype.
// fp32 path (and the generic one): 256 threads, each 2 rows x 2 columns (x 2 matrices when gated)
template <typename T, int ACT>
__global__ void __launch_bounds__(256)
grouped_linear_fma_kernel(void* __restrict__ out_, const T* __restrict__ a, const T* __restrict__ w,
                          const int32_t* __restrict__ off, const int32_t* __restrict__ pair_of_slot, int top, int E,
                          int K, int N) {
  constexpr bool GATED = ACT == 1, GATHER = ACT != 0;
  __shared__ float As[TM][TK + 1], W0[TN][TK + 1], W1[GATED ? TN : 1][TK + 1];
  int e, s0, rows;
  if (!find_tile(off, E, blockIdx.x, &e, &s0, &rows)) return;
  const int n0 = blockIdx.y * TN;
  const T* we = w + static_cast<size_t>(e) * (GATED ? 2 : 1) * N * K;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  float acc0[2][2] = {}, acc1[2][2] = {};
  for (int k0 = 0; k0 < K; k0 += TK) {
    __syncthreads();
    for (int i = threadIdx.x; i < TM * TK; i += 256) {
      const int r = i / TK, k = i % TK;
      float v = 0.f;
      if (r < rows && k0 + k < K) {
        const int slot = s0 + r;
        const size_t row = GATHER ? static_cast<size_t>(pair_of_slot[slot] / top) : static_cast<size_t>(slot);
        v = ld(a + row * K + k0 + k);
      }
      As[r][k] = v;
    }
    for (int i = threadIdx.x; i < TN * TK; i += 256) {
      const int n = i / TK, k = i % TK;
      const bool ok = n0 + n < N && k0 + k < K;
      W0[n][k] = ok ? ld(we + static_cast<size_t>(n0 + n) * K + k0 + k) : 0.f;
      if (GATED) W1[n][k] = ok ? ld(we + static_cast<size_t>(N + n0 + n) * K + k0 + k) : 0.f;
    }
    __syncthreads();
#pragma unroll 8
    for (int k = 0; k < TK; ++k) {
      const float a0 = As[ty * 2][k], a1 = As[ty * 2 + 1][k];
      const float b0 = W0[tx * 2][k], b1 = W0[tx * 2 + 1][k];
      acc0[0][0] += a0 * b0; acc0[0][1] += a0 * b1; acc0[1][0] += a1 * b0; acc0[1][1] += a1 * b1;
      if (GATED) {
        const float c0 = W1[tx * 2][k], c1 = W1[tx * 2 + 1][k];
        acc1[0][0] += a0 * c0; acc1[0][1] += a0 * c1; acc1[1][0] += a1 * c0; acc1[1][1] += a1 * c1;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int r = ty * 2 + i, n = n0 + tx * 2 + j;
      if (r < rows && n < N) {
        const size_t o = static_cast<size_t>(s0 + r) * N + n;
        if (GATED) {
          st(reinterpret_cast<T*>(out_) + o, silu_exact(acc0[i][j]) * acc1[i][j]);
        } else if (ACT == 2) {
          const float u = fmaxf(acc0[i][j], 0.f);
          st(reinterpret_cast<T*>(out_) + o, u * u);
        } else {
          reinterpret_cast<float*>(out_)[o] = acc0[i][j];
        }
      }
    }
}

// bf16 path on the tensor cores: block = 4 warps, tile 32 slots x 64 columns, K chunks of 32 through shared memory.
// warp w owns columns [16 w, 16 w + 16) for both 16-row halves; GATED keeps a second accumulator set for the up rows.
constexpr int MN = 64, MK = 32, MP = MK + 8;      // MP: row pitch in bf16 elements (conflict-free 32-bit fragment loads)
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, const uint32_t* b) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem))),
               "l"(gmem)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int ACT>
__global__ void __launch_bounds__(128)
grouped_linear_mma_kernel(void* __restrict__ out_, const __nv_bfloat16* __restrict__ a,
                          const __nv_bfloat16* __restrict__ w, const int32_t* __restrict__ off,
                          const int32_t* __restrict__ pair_of_slot, int top, int E, int K, int N) {
  constexpr bool GATED = ACT == 1, GATHER = ACT != 0;
  // two stages: the 16-byte asynchronous copies of K chunk i + 1 run under the MMAs of chunk i
  __shared__ __align__(16) __nv_bfloat16 As[2][TM][MP], W0[2][MN][MP], W1[2][GATED ? MN : 1][MP];
  __shared__ size_t arow[TM];
  int e, s0, rows;
  if (!find_tile(off, E, blockIdx.x, &e, &s0, &rows)) return;
  const int n0 = blockIdx.y * MN;
  const __nv_bfloat16* we = w + static_cast<size_t>(e) * (GATED ? 2 : 1) * N * K;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  if (threadIdx.x < TM) {
    const int slot = s0 + min(static_cast<int>(threadIdx.x), rows - 1);
    arow[threadIdx.x] = GATHER ? static_cast<size_t>(pair_of_slot[slot] / top) : static_cast<size_t>(slot);
  }
  __syncthreads();
  float acc0[2][2][4] = {}, acc1[2][2][4] = {};      // [row half][8-column block][fragment]
  const bool vec = (K % 8) == 0;                     // every row start is 16-byte aligned
  const uint4 zero4 = make_uint4(0, 0, 0, 0);
  auto load_async = [&](int st, int k0) {
    for (int i = threadIdx.x; i < TM * (MK / 8); i += 128) {
      const int r = i / (MK / 8), k = (i % (MK / 8)) * 8;
      if (r < rows && k0 + k < K) cp_async16(&As[st][r][k], a + arow[r] * K + k0 + k);
      else *reinterpret_cast<uint4*>(&As[st][r][k]) = zero4;
    }
    for (int i = threadIdx.x; i < MN * (MK / 8); i += 128) {
      const int n = i / (MK / 8), k = (i % (MK / 8)) * 8;
      const bool ok = n0 + n < N && k0 + k < K;
      if (ok) cp_async16(&W0[st][n][k], we + static_cast<size_t>(n0 + n) * K + k0 + k);
      else *reinterpret_cast<uint4*>(&W0[st][n][k]) = zero4;
      if (GATED) {
        if (ok) cp_async16(&W1[st][n][k], we + static_cast<size_t>(N + n0 + n) * K + k0 + k);
        else *reinterpret_cast<uint4*>(&W1[st][n][k]) = zero4;
      }
    }
    cp_async_commit();
  };
  auto load_plain = [&](int st, int k0) {
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (int i = threadIdx.x; i < TM * MK; i += 128) {
      const int r = i / MK, k = i % MK;
      As[st][r][k] = (r < rows && k0 + k < K) ? a[arow[r] * K + k0 + k] : zero;
    }
    for (int i = threadIdx.x; i < MN * MK; i += 128) {
      const int n = i / MK, k = i % MK;
      const bool ok = n0 + n < N && k0 + k < K;
      W0[st][n][k] = ok ? we[static_cast<size_t>(n0 + n) * K + k0 + k] : zero;
      if (GATED) W1[st][n][k] = ok ? we[static_cast<size_t>(N + n0 + n) * K + k0 + k] : zero;
    }
  };
  int st = 0;
  if (vec) load_async(0, 0);
  for (int k0 = 0; k0 < K; k0 += MK, st ^= 1) {
    if (vec) {
      const bool more = k0 + MK < K;
      if (more) load_async(st ^ 1, k0 + MK);
      if (more) cp_async_wait<1>(); else cp_async_wait<0>();
    } else {
      load_plain(st, k0);
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MK; kk += 16) {
      uint32_t af[2][4];
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        af[hf][0] = *reinterpret_cast<const uint32_t*>(&As[st][hf * 16 + g][kk + 2 * tq]);
        af[hf][1] = *reinterpret_cast<const uint32_t*>(&As[st][hf * 16 + g + 8][kk + 2 * tq]);
        af[hf][2] = *reinterpret_cast<const uint32_t*>(&As[st][hf * 16 + g][kk + 2 * tq + 8]);
        af[hf][3] = *reinterpret_cast<const uint32_t*>(&As[st][hf * 16 + g + 8][kk + 2 * tq + 8]);
      }
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const int n = warp * 16 + nb * 8 + g;
        uint32_t bf[2];
        bf[0] = *reinterpret_cast<const uint32_t*>(&W0[st][n][kk + 2 * tq]);
        bf[1] = *reinterpret_cast<const uint32_t*>(&W0[st][n][kk + 2 * tq + 8]);
        mma_bf16(acc0[0][nb], af[0], bf);
        mma_bf16(acc0[1][nb], af[1], bf);
        if (GATED) {
          bf[0] = *reinterpret_cast<const uint32_t*>(&W1[st][n][kk + 2 * tq]);
          bf[1] = *reinterpret_cast<const uint32_t*>(&W1[st][n][kk + 2 * tq + 8]);
          mma_bf16(acc1[0][nb], af[0], bf);
          mma_bf16(acc1[1][nb], af[1], bf);
        }
      }
    }
    __syncthreads();          // the stage is free before the next round's copies land in it
  }
#pragma unroll
  for (int hf = 0; hf < 2; ++hf)
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int r = hf * 16 + g + (f >> 1) * 8;
        const int n = n0 + warp * 16 + nb * 8 + 2 * tq + (f & 1);
        if (r < rows && n < N) {
          const size_t o = static_cast<size_t>(s0 + r) * N + n;
          if (GATED) {
            reinterpret_cast<__nv_bfloat16*>(out_)[o] =
                __float2bfloat16_rn(silu_exact(acc0[hf][nb][f]) * acc1[hf][nb][f]);
          } else if (ACT == 2) {
            const float u = fmaxf(acc0[hf][nb][f], 0.f);
            reinterpret_cast<__nv_bfloat16*>(out_)[o] = __float2bfloat16_rn(u * u);
          } else {
            reinterpret_cast<float*>(out_)[o] = acc0[hf][nb][f];
          }
        }
      }
}

// choices >= E are identity experts: their row is the token's own input (ident, fp32 or the activation dtype)
template <typename TI>
__global__ void moe_combine_kernel(float* __restrict__ x, const float* __restrict__ down,
                                   const int32_t* __restrict__ slot_of_pair, const int32_t* __restrict__ top_idx,
                                   const float* __restrict__ top_w, int top, int width, int E,
                                   const TI* __restrict__ ident, int accumulate) {
  const int t = blockIdx.x;
  for (int d = threadIdx.x; d < width; d += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < top; ++j) {
      const size_t p = static_cast<size_t>(t) * top + j;
      const float row = (ident && top_idx[p] >= E) ? ld(ident + static_cast<size_t>(t) * width + d)
                                                   : down[static_cast<size_t>(slot_of_pair[p]) * width + d];
      acc += top_w[p] * row;
    }
    float* o = x + static_cast<size_t>(t) * width + d;
    *o = accumulate ? *o + acc : acc;
  }
}

void launch_moe_route(const float* logits, const float* bias, int T, int E, int top, int groups, int keep, float scale,
                      int32_t* top_idx, float* top_w, cudaStream_t st_) {
  if (T <= 0) return;
  if (groups < 0 || (groups > 0 && (E % groups != 0 || keep < 1 || keep > groups))) {
    set_error(1, "moe_route: the experts do not split into that many equal groups, or keep is out of range");
    return;
  }
  const int available = groups > 0 ? E / groups * keep : E;
  const size_t per_warp = (2 * static_cast<size_t>(E) + groups) * 4;
  int nw = 4;
  while (nw > 1 && nw * per_warp > 48 * 1024) nw >>= 1;
  if (nw * per_warp > 48 * 1024 || top > available) {
    set_error(1, "moe_route: too many experts, or top above the number that can be chosen");
    return;
  }
  moe_route_kernel<<<(T + nw - 1) / nw, nw * 32, nw * per_warp, st_>>>(logits, bias, T, E, top, groups, keep, scale,
                                                                      top_idx, top_w);
  B200_CUDA_LAUNCH_CHECK();
}

void launch_moe_sort(const int32_t* top_idx, int pairs, int E, int32_t* expert_off, int32_t* pair_of_slot,
                     int32_t* slot_of_pair, cudaStream_t st_) {
  if (pairs <= 0) return;
  if (E > 8192) {
    set_error(1, "moe_sort: more than 8192 experts");
    return;
  }
  moe_sort_kernel<<<1, 1024, static_cast<size_t>(E) * 4, st_>>>(top_idx, pairs, E, expert_off, pair_of_slot,
                                                                slot_of_pair);
  B200_CUDA_LAUNCH_CHECK();
}

static bool use_mma() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_MOE_MMA");       // 0: the FMA kernel also for bf16 (A/B arm)
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

template <int ACT>
static void grouped_linear(void* out, const void* a, const void* w, const int32_t* off, const int32_t* pair_of_slot,
                           int pairs, int top, int E, int K, int N, int dt, cudaStream_t st_) {
  if (pairs <= 0) return;
  const int tiles = (pairs + TM - 1) / TM + E;
  if (dt) {
    grouped_linear_fma_kernel<float, ACT><<<dim3(tiles, (N + TN - 1) / TN), 256, 0, st_>>>(
        out, (const float*)a, (const float*)w, off, pair_of_slot, top, E, K, N);
  } else if (use_mma()) {
    grouped_linear_mma_kernel<ACT><<<dim3(tiles, (N + MN - 1) / MN), 128, 0, st_>>>(
        out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, off, pair_of_slot, top, E, K, N);
  } else {
    grouped_linear_fma_kernel<__nv_bfloat16, ACT><<<dim3(tiles, (N + TN - 1) / TN), 256, 0, st_>>>(
        out, (const __nv_bfloat16*)a, (const __nv_bfloat16*)w, off, pair_of_slot, top, E, K, N);
  }
  B200_CUDA_LAUNCH_CHECK();
}

void launch_moe_gate_up(void* act_out, const void* h, const void* w_up, const int32_t* expert_off,
                        const int32_t* pair_of_slot, int pairs, int top, int E, int width, int ff, int act, int dt,
                        cudaStream_t st_) {
  if (act == 0)
    grouped_linear<1>(act_out, h, w_up, expert_off, pair_of_slot, pairs, top, E, width, ff, dt, st_);
  else
    grouped_linear<2>(act_out, h, w_up, expert_off, pair_of_slot, pairs, top, E, width, ff, dt, st_);
}
void launch_moe_down(float* out, const void* act, const void* w_down, const int32_t* expert_off, int pairs, int E,
                     int width, int ff, int dt, cudaStream_t st_) {
  grouped_linear<0>(out, act, w_down, expert_off, nullptr, pairs, 1, E, ff, width, dt, st_);
}
void launch_moe_combine(float* x, const float* down, const int32_t* slot_of_pair, const int32_t* top_idx,
                        const float* top_w, int T, int top, int width, int E, const void* ident, int ident_f32, int dt,
                        int accumulate, cudaStream_t st_) {
  if (T <= 0) return;
  if (!ident || ident_f32 || dt)
    moe_combine_kernel<float><<<T, 256, 0, st_>>>(x, down, slot_of_pair, top_idx, top_w, top, width, E,
                                                  (const float*)ident, accumulate);
  else
    moe_combine_kernel<__nv_bfloat16><<<T, 256, 0, st_>>>(x, down, slot_of_pair, top_idx, top_w, top, width, E,
                                                          (const __nv_bfloat16*)ident, accumulate);
  B200_CUDA_LAUNCH_CHECK();
}

}  // namespace b200

extern "C" {
// Router: logits fp32 [T, E] -> top_idx i32 [T, top], top_w fp32 [T, top] = softmax(logits)[idx] * scale.
void b200_moe_route(const float* logits, int32_t num_tokens, int32_t experts, int32_t top, float scale,
                    int32_t* top_idx, float* top_w, int64_t stream) {
  B200_CHECK_ARG(logits && top_idx && top_w && experts > 0 && top > 0, "moe_route: bad arguments");
  b200::launch_moe_route(logits, nullptr, num_tokens, experts, top, 0, 0, scale, top_idx, top_w,
                         reinterpret_cast<cudaStream_t>(stream));
}
void b200_moe_route_ex(const float* logits, const float* bias, int32_t num_tokens, int32_t experts, int32_t top,
                       int32_t groups, int32_t keep, float scale, int32_t* top_idx, float* top_w, int64_t stream) {
  B200_CHECK_ARG(logits && top_idx && top_w && experts > 0 && top > 0, "moe_route_ex: bad arguments");
  b200::launch_moe_route(logits, bias, num_tokens, experts, top, groups, keep, scale, top_idx, top_w,
                         reinterpret_cast<cudaStream_t>(stream));
}
// The experts' feed-forward of routed tokens, added into the fp32 stream x [T, width]: h [T, width] and the weights
// in the activation dtype (dt 0 bf16, 1 fp32).  workspace: b200_moe_workspace_bytes() bytes.
int64_t b200_moe_workspace_bytes(int32_t num_tokens, int32_t experts, int32_t top, int32_t width, int32_t ff) {
  const int64_t P = static_cast<int64_t>(num_tokens) * top;
  return 256 * 6 + (experts + 1) * 4 + P * 8 + P * ff * 4 + P * width * 4;
}
void b200_moe_experts_ex(float* out, const void* h, const int32_t* top_idx, const float* top_w, const void* w_up,
                         const void* w_down, int32_t num_tokens, int32_t experts, int32_t identity, int32_t top,
                         int32_t width, int32_t ff, int32_t act, int32_t accumulate, const void* ident,
                         int32_t ident_f32, int32_t dt, void* workspace, int64_t stream) {
  B200_CHECK_ARG(out && h && top_idx && top_w && w_up && w_down && workspace && (dt == 0 || dt == 1) &&
                     (act == 0 || act == 1) && identity >= 0 && (identity == 0 || ident),
                 "moe_experts: bad arguments");
  cudaStream_t st_ = reinterpret_cast<cudaStream_t>(stream);
  const int P = num_tokens * top, all = experts + identity;
  auto up = [](size_t v) { return (v + 255) / 256 * 256; };
  uint8_t* p = reinterpret_cast<uint8_t*>(up(reinterpret_cast<size_t>(workspace)));
  int32_t* off = reinterpret_cast<int32_t*>(p); p += up((all + 1) * 4);
  int32_t* pos = reinterpret_cast<int32_t*>(p); p += up(static_cast<size_t>(P) * 4);
  int32_t* sop = reinterpret_cast<int32_t*>(p); p += up(static_cast<size_t>(P) * 4);
  void* actb = p; p += up(static_cast<size_t>(P) * ff * 4);
  float* down = reinterpret_cast<float*>(p);
  // identity experts take buckets past the real ones; the grouped products walk the first `experts` buckets only
  b200::launch_moe_sort(top_idx, P, all, off, pos, sop, st_);
  b200::launch_moe_gate_up(actb, h, w_up, off, pos, P, top, experts, width, ff, act, dt, st_);
  b200::launch_moe_down(down, actb, w_down, off, P, experts, width, ff, dt, st_);
  b200::launch_moe_combine(out, down, sop, top_idx, top_w, num_tokens, top, width, experts, identity ? ident : nullptr,
                           ident_f32, dt, accumulate, st_);
}
void b200_moe_experts(float* x, const void* h, const int32_t* top_idx, const float* top_w, const void* w_gate_up,
                      const void* w_down, int32_t num_tokens, int32_t experts, int32_t top, int32_t width, int32_t ff,
                      int32_t dt, void* workspace, int64_t stream) {
  b200_moe_experts_ex(x, h, top_idx, top_w, w_gate_up, w_down, num_tokens, experts, 0, top, width, ff, 0, 1, nullptr, 0,
                      dt, workspace, stream);
}
}
