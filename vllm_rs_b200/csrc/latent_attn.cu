// Latent (compressed-KV) attention over the paged cache, for ragged steps (prompt portions and decoded tokens alike).
//
// The cache holds ONE row per token and layer: [c (kv_rank) | k_rot (rot_dim)], c = the RMS-normed latent, k_rot the
// rotated key part shared by all heads.  Pages are the block manager's 64-token blocks:
//   cache [num_blocks, 64, kv_rank + rot_dim]   (bf16 or fp32).
// Queries come in "absorbed" form: q_full [T, H, kv_rank + rot_dim] fp32 where the first kv_rank entries are
// W_uk[h]^T q_plain[h] (a batched matrix product made by the runner) and the rest the rotated query part, so that
//   score(i, j, h) = (q_full[i, h] . cache[j]) * scale
// and the kernel returns the attention-weighted LATENT sum_j p_j c_j [T, H, kv_rank]; the runner expands it with
// W_uv[h].  All heads of a token read the same cache rows (multi-query form), which is what makes the latent cache
// cheap to stream.  Options: sliding window (position i sees j with 0 <= i - j < window; window <= 0 = all), and a
// learned per-head sink logit that joins the softmax denominator without a key or value, and a per-head output gate
// (head h's result times sigmoid(gate[t, h]); the gate commutes with the value expansion that follows).  A layer may
// read ANOTHER layer's cache (latent_prep with no cache: queries only), with its own W_uk / W_uv folded in around it.
// Two kernels: an fp32 FMA form (any sizes, both dtypes; rows of small steps split their keys over several blocks and
// merge) and a bf16 tensor-core form for steps of many rows (kv_rank a multiple of 64 up to 512, kv_rank + rot_dim a
// multiple of 16).  Beside paged_attn_decode.cu / attn_prefill*.cu (per-head K / V caches, fp16 / bf16, no window
// over prompts).
//
// latent_prep_kernel: from the fused projection row [q (H x (dim + rot_dim)) | c_raw (kv_rank) | k_rot_raw (rot_dim)]
// (fp32) it RMS-norms the latent (plain weight), rotates the first rot_dims entries of every head's rotated query
// part and of the shared key part as interleaved pairs (2i, 2i+1) by the angle position * freq[i] (angles in double,
// cos / sin scaled by rot_mag), writes the cache row at the token's slot, and splits the queries.
#include "../../include/b200_vllm.h"
#include <algorithm>
#include <cstdlib>

#include "seqmix.cuh"

namespace b200 {
using namespace seqmix;

template <typename T>
__global__ void latent_prep_kernel(const float* __restrict__ qc, int ldq, T* __restrict__ q_plain,
                                   float* __restrict__ q_full, T* __restrict__ cache,
                                   const float* __restrict__ latent_norm_w, const double* __restrict__ rot_freq,
                                   float rot_mag, const int64_t* __restrict__ positions,
                                   const int64_t* __restrict__ slots, int heads, int dim, int rot_dim, int rot_dims,
                                   int kv_rank, float eps) {
  extern __shared__ float sm[];          // cos[rot_dims/2] | sin[rot_dims/2] | red[33]
  const int half = rot_dims / 2;
  float* cs = sm;
  float* sn = sm + half;
  float* red = sm + 2 * half;
  const int t = blockIdx.x;
  const float* row = qc + static_cast<size_t>(t) * ldq;
  const bool own_latent = cache != nullptr;            // otherwise the row holds the queries only
  const float* craw = row + static_cast<size_t>(heads) * (dim + rot_dim);
  const float* kraw = craw + kv_rank;
  const double pos = static_cast<double>(positions[t]);
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos(pos * rot_freq[i], &s, &c);
    cs[i] = static_cast<float>(c) * rot_mag;
    sn[i] = static_cast<float>(s) * rot_mag;
  }
  float ss = 0.f;
  if (own_latent)
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) ss += craw[d] * craw[d];
  ss = block_sum(ss, red);           // also orders the cos / sin writes before their use
  const float inv = 1.f / sqrtf(ss / static_cast<float>(kv_rank) + eps);
  const int64_t slot = own_latent ? slots[t] : -1;
  const int R = kv_rank + rot_dim;
  if (slot >= 0) {
    T* crow = cache + static_cast<size_t>(slot) * R;
    for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) st(crow + d, craw[d] * inv * latent_norm_w[d]);
    for (int d = threadIdx.x; d < rot_dim; d += blockDim.x) {
      float v = kraw[d];
      if (d < rot_dims) {
        const int i = d >> 1;
        const float a = kraw[2 * i], b = kraw[2 * i + 1];
        v = (d & 1) ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
      }
      st(crow + kv_rank + d, v);
    }
  }
  const int hd = dim + rot_dim;
  for (int e = threadIdx.x; e < heads * hd; e += blockDim.x) {
    const int h = e / hd, d = e % hd;
    const float* qh = row + static_cast<size_t>(h) * hd;
    if (d < dim) {
      st(q_plain + (static_cast<size_t>(t) * heads + h) * dim + d, qh[d]);
    } else {
      const int r = d - dim;
      float v = qh[d];
      if (r < rot_dims) {
        const int i = r >> 1;
        const float a = qh[dim + 2 * i], b = qh[dim + 2 * i + 1];
        v = (r & 1) ? b * cs[i] + a * sn[i] : a * cs[i] - b * sn[i];
      }
      q_full[(static_cast<size_t>(t) * heads + h) * R + kv_rank + r] = v;
    }
  }
}

// grid = (token rows, head groups); a block's warps each own one head at a time.  Key rows of a tile are staged once
// in shared memory (fp32) and used by every head of the group.
template <typename T>
__global__ void latent_attn_kernel(T* __restrict__ out, const float* __restrict__ q_full, const T* __restrict__ cache,
                                   const float* __restrict__ sink, const float* __restrict__ gate, int ld_gate,
                                   const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx,
                                   const uint32_t* __restrict__ block_tables, int max_blocks, int num_seqs, int heads,
                                   int kv_rank, int rot_dim, int window, float scale, int key_tile, int nsplit,
                                   float* __restrict__ part_o, float* __restrict__ part_ml) {
  extern __shared__ float sm[];
  const int R = kv_rank + rot_dim, Rp = R | 1;        // odd row pitch: a lane per key reads conflict-free
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ks = sm;                                      // [key_tile][Rp]
  float* qs = ks + static_cast<size_t>(key_tile) * Rp;  // [nw][R]
  float* os = qs + static_cast<size_t>(nw) * R;        // [nw][kv_rank]
  const int t = blockIdx.x;
  const int b = seq_of_row(cu, num_seqs, t);
  const int qlen = static_cast<int>(cu[b + 1] - cu[b]);
  const int pos = static_cast<int>(ctx[b]) - qlen + (t - static_cast<int>(cu[b]));
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const int h = blockIdx.y * nw + warp;
  const bool live = h < heads;
  if (live) {
    const float* q = q_full + (static_cast<size_t>(t) * heads + h) * R;
    for (int d = lane; d < R; d += 32) qs[warp * R + d] = q[d];
    for (int d = lane; d < kv_rank; d += 32) os[warp * kv_rank + d] = 0.f;
  }
  float m = -1e30f, l = 0.f;
  if (live && sink && nsplit == 1) {       // split runs add the sink when the parts are merged
    m = sink[h];
    l = 1.f;
  }
  const uint32_t* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  // blockIdx.z owns a contiguous run of key tiles (nsplit == 1: all of them)
  const int ntiles = (pos - lo + key_tile) / key_tile;
  const int per = (ntiles + nsplit - 1) / nsplit;
  const int first = lo + static_cast<int>(blockIdx.z) * per * key_tile;
  const int last = min(pos, first + per * key_tile - 1);
  for (int j0 = first; j0 <= last; j0 += key_tile) {
    const int nk = min(key_tile, last - j0 + 1);
    __syncthreads();
    for (int e = threadIdx.x; e < nk * R; e += blockDim.x) {
      const int k = e / R, d = e % R, j = j0 + k;
      const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
      ks[k * Rp + d] = ld(cache + slot * R + d);
    }
    __syncthreads();
    if (!live) continue;
    for (int k0 = 0; k0 < nk; k0 += 32) {
      const int k = k0 + lane;
      float s = -1e30f;
      if (k < nk) {
        float acc = 0.f;
        const float* kr = ks + k * Rp;
        const float* qw = qs + warp * R;
        for (int d = 0; d < R; ++d) acc += qw[d] * kr[d];
        s = acc * scale;
      }
      const float mt = lanes_max(s);
      const float mn = fmaxf(m, mt);
      const float alpha = expf(m - mn);
      const float p = k < nk ? expf(s - mn) : 0.f;
      l = l * alpha + lanes_sum(p);
      m = mn;
      const int cnt = min(32, nk - k0);
      for (int d0 = 0; d0 < kv_rank; d0 += 32) {       // every lane takes part in the shuffles
        const int d = d0 + lane;
        const bool ok = d < kv_rank;
        float acc = ok ? os[warp * kv_rank + d] * alpha : 0.f;
        for (int kk = 0; kk < cnt; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, p, kk);
          if (ok) acc += pk * ks[(k0 + kk) * Rp + d];
        }
        if (ok) os[warp * kv_rank + d] = acc;
      }
    }
  }
  if (live && nsplit == 1) {
    float inv = l > 0.f ? 1.f / l : 0.f;
    if (gate) inv *= sigmoid_f(gate[static_cast<size_t>(t) * ld_gate + h]);
    T* o = out + (static_cast<size_t>(t) * heads + h) * kv_rank;
    for (int d = lane; d < kv_rank; d += 32) st(o + d, os[warp * kv_rank + d] * inv);
  } else if (live) {
    const size_t pi = (static_cast<size_t>(t) * heads + h) * nsplit + blockIdx.z;
    for (int d = lane; d < kv_rank; d += 32) part_o[pi * kv_rank + d] = os[warp * kv_rank + d];
    if (lane == 0) {
      part_ml[pi * 2] = m;
      part_ml[pi * 2 + 1] = l;
    }
  }
}

// one block per (token, head): the parts of a split run and the sink meet in one softmax
template <typename T>
__global__ void latent_attn_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, const float* __restrict__ sink,
                                         const float* __restrict__ gate, int ld_gate, int heads, int kv_rank,
                                         int nsplit) {
  const size_t th = blockIdx.x;
  const int h = static_cast<int>(th % heads);
  const float* ml = part_ml + th * nsplit * 2;
  float m = sink ? sink[h] : -1e30f;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, ml[2 * z]);
  float l = sink ? expf(sink[h] - m) : 0.f;
  for (int z = 0; z < nsplit; ++z) l += ml[2 * z + 1] * expf(ml[2 * z] - m);
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate) inv *= sigmoid_f(gate[(th / heads) * ld_gate + h]);
  for (int d = threadIdx.x; d < kv_rank; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < nsplit; ++z) acc += part_o[(th * nsplit + z) * kv_rank + d] * expf(ml[2 * z] - m);
    st(out + th * kv_rank + d, acc * inv);
  }
}

void launch_latent_prep(const float* qc, int ldq, void* q_plain, float* q_full, void* cache, const float* latent_norm_w,
                        const double* rot_freq, float rot_mag, const int64_t* positions, const int64_t* slots, int T,
                        int heads, int dim, int rot_dim, int rot_dims, int kv_rank, float eps, int dt, cudaStream_t st_) {
  if (T <= 0) return;
  const size_t smem = (static_cast<size_t>(rot_dims) + 40) * 4;
  if (dt)
    latent_prep_kernel<float><<<T, 256, smem, st_>>>(qc, ldq, (float*)q_plain, q_full, (float*)cache, latent_norm_w,
                                                     rot_freq, rot_mag, positions, slots, heads, dim, rot_dim,
                                                     rot_dims, kv_rank, eps);
  else
    latent_prep_kernel<__nv_bfloat16><<<T, 256, smem, st_>>>(qc, ldq, (__nv_bfloat16*)q_plain, q_full,
                                                             (__nv_bfloat16*)cache, latent_norm_w, rot_freq, rot_mag,
                                                             positions, slots, heads, dim, rot_dim, rot_dims, kv_rank,
                                                             eps);
  B200_CUDA_LAUNCH_CHECK();
}

// ---- bf16 tensor-core form for steps of many rows (prompt portions).  Block = 4 warps = one head x 16 consecutive
// token rows of ONE sequence.  Per tile of 64 keys: every warp computes the scores of 16 keys (S = Q K^T, mma.sync
// m16n8k16 bf16 -> fp32, Q and K from shared memory), the fp32 scores meet in shared memory, every warp runs the same
// fp32 online softmax over all 64 (sink as the initial denominator, window and causal mask per element) and
// multiplies P (bf16) with ITS quarter of the latent columns (V fragments by ldmatrix.trans from the same key tile).
constexpr int MQ = 16, MKT = 64;
__device__ __forceinline__ void mma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// NT = n-tiles (8 latent columns each) per warp = kv_rank / 32.  HROWS = false: the 16 MMA rows are 16 consecutive token
// rows of one head (prompt portions).  HROWS = true (steps of few rows, decoding): the 16 rows are 16 HEADS of one
// token -- all heads share the key rows, so one pass over the cache serves them all -- and blockIdx.z owns a
// contiguous run of key tiles; with nsplit > 1 the unnormalised parts go to part_o / part_ml and
// latent_attn_merge_kernel finishes the softmax (it adds the sink).
template <int NT, bool HROWS>
__global__ void __launch_bounds__(128)
latent_attn_mma_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ q_full,
                       const __nv_bfloat16* __restrict__ cache, const float* __restrict__ sink,
                       const float* __restrict__ gate, int ld_gate,
                       const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx,
                       const uint32_t* __restrict__ block_tables, int max_blocks, int num_seqs, int heads, int kv_rank,
                       int rot_dim, int window, float scale, int nsplit, float* __restrict__ part_o,
                       float* __restrict__ part_ml) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int R = kv_rank + rot_dim, P = R + 8;             // P: row pitch in bf16 elements (16-byte multiple)
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);              // [MKT][P]
  __nv_bfloat16* Qs = Ks + static_cast<size_t>(MKT) * P;                    // [MQ][P]
  float* Ss = reinterpret_cast<float*>(Qs + static_cast<size_t>(MQ) * P);   // [MQ][MKT + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  // which rows does this block own?
  int b = -1, row0 = 0, nrows = 0, h = blockIdx.y, pos0 = 0;
  if (HROWS) {                                   // one token, heads [16 blockIdx.y, +16)
    row0 = blockIdx.x;
    b = seq_of_row(cu, num_seqs, row0);
    h = blockIdx.y * MQ;
    nrows = min(MQ, heads - h);
    pos0 = static_cast<int>(ctx[b]) - static_cast<int>(cu[b + 1] - cu[b]) + (row0 - static_cast<int>(cu[b]));
  } else {                                       // 16 token rows of one sequence (tiles never straddle sequences)
    int acc = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = static_cast<int>(cu[s + 1] - cu[s]), tiles = (n + MQ - 1) / MQ;
      if (static_cast<int>(blockIdx.x) < acc + tiles) {
        const int k = blockIdx.x - acc;
        b = s;
        row0 = cu[s] + k * MQ;
        nrows = min(MQ, n - k * MQ);
        break;
      }
      acc += tiles;
    }
    if (b < 0) return;
    pos0 = static_cast<int>(ctx[b]) - static_cast<int>(cu[b + 1] - cu[b]) + (row0 - static_cast<int>(cu[b]));
  }
  const int pos_last = HROWS ? pos0 : pos0 + nrows - 1;
  const int key_lo = window > 0 ? max(0, pos0 - window + 1) : 0;
  // stage Q (bf16) once
  for (int e = threadIdx.x; e < MQ * R; e += blockDim.x) {
    const int r = e / R, d = e % R;
    const size_t qrow = HROWS ? static_cast<size_t>(row0) * heads + h + r : static_cast<size_t>(row0 + r) * heads + h;
    const float v = r < nrows ? q_full[qrow * R + d] : 0.f;
    Qs[r * P + d] = __float2bfloat16_rn(v);
  }
  float m[2], l[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int hh = HROWS ? min(h + g + rr * 8, heads - 1) : h;
    const bool with_sink = sink && nsplit == 1;          // split runs add the sink when the parts are merged
    m[rr] = with_sink ? sink[hh] : -1e30f;
    l[rr] = with_sink ? 1.f : 0.f;
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const uint32_t* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int rowp[2] = {HROWS ? pos0 : pos0 + g, HROWS ? pos0 : pos0 + g + 8};   // positions of this lane's two rows
  // the run of key tiles of this block (nsplit == 1: all of them)
  const int ntiles = (pos_last - key_lo + MKT) / MKT, per = (ntiles + nsplit - 1) / nsplit;
  const int first = key_lo + static_cast<int>(blockIdx.z) * per * MKT;
  const int last_key = min(pos_last, first + per * MKT - 1);
  for (int j0 = first; j0 <= last_key; j0 += MKT) {
    __syncthreads();
    // key tile: 16-byte copies (R % 8 == 0), zero rows past the last visible key
    const int vec = R / 8;
    for (int e = threadIdx.x; e < MKT * vec; e += blockDim.x) {
      const int k = e / vec, d = (e % vec) * 8, j = j0 + k;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j <= last_key) {
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        v = *reinterpret_cast<const uint4*>(cache + slot * R + d);
      }
      *reinterpret_cast<uint4*>(Ks + static_cast<size_t>(k) * P + d) = v;
    }
    __syncthreads();
    // scores of keys [16 warp, 16 warp + 16)
    float sc[2][4] = {};
    for (int kk = 0; kk < R; kk += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(Qs + g * P + kk + 2 * tq);
      a[1] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * P + kk + 2 * tq);
      a[2] = *reinterpret_cast<const uint32_t*>(Qs + g * P + kk + 2 * tq + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * P + kk + 2 * tq + 8);
#pragma unroll
      for (int nb = 0; nb < 2; ++nb) {
        const __nv_bfloat16* kr = Ks + static_cast<size_t>(warp * 16 + nb * 8 + g) * P + kk + 2 * tq;
        mma_bf16_16816(sc[nb], a, *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
      }
    }
#pragma unroll
    for (int nb = 0; nb < 2; ++nb)
#pragma unroll
      for (int f = 0; f < 4; ++f) {
        const int r = g + (f >> 1) * 8, kcol = warp * 16 + nb * 8 + 2 * tq + (f & 1);
        Ss[r * (MKT + 1) + kcol] = sc[nb][f] * scale;
      }
    __syncthreads();
    // the same online softmax in every warp; this lane's P entries are exactly its A fragments
    float p[2][16];
    float mx[2] = {-1e30f, -1e30f};
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int r = g + rr * 8;
      const int lo = window > 0 ? max(0, rowp[rr] - window + 1) : 0;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int kcol = ks * 16 + 2 * tq + (c & 1) + (c >> 1) * 8, j = j0 + kcol;
          const bool ok = r < nrows && j >= lo && j <= rowp[rr] && j <= last_key;
          const float v = ok ? Ss[r * (MKT + 1) + kcol] : -1e30f;
          p[rr][ks * 4 + c] = v;
          mx[rr] = fmaxf(mx[rr], v);
        }
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 1));
      mx[rr] = fmaxf(mx[rr], __shfl_xor_sync(0xffffffffu, mx[rr], 2));
    }
    float alpha[2];
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const float mn = fmaxf(m[rr], mx[rr]);
      alpha[rr] = expf(m[rr] - mn);
      float sum = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float e = p[rr][i] > -1e29f ? expf(p[rr][i] - mn) : 0.f;
        p[rr][i] = e;
        sum += e;
      }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[rr] = l[rr] * alpha[rr] + sum;
      m[rr] = mn;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    // O += P V over this warp's latent columns [warp * NT * 8, +NT * 8)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a[4];
      a[0] = pack_bf16(p[0][ks * 4 + 0], p[0][ks * 4 + 1]);
      a[1] = pack_bf16(p[1][ks * 4 + 0], p[1][ks * 4 + 1]);
      a[2] = pack_bf16(p[0][ks * 4 + 2], p[0][ks * 4 + 3]);
      a[3] = pack_bf16(p[1][ks * 4 + 2], p[1][ks * 4 + 3]);
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        // four 8 x 8 blocks: (keys 0-7 | 8-15 of the step) x (columns d0 .. d0+7 | d0+8 .. d0+15), transposed on load
        const int d0 = (warp * NT + n) * 8;
        const __nv_bfloat16* src = Ks + static_cast<size_t>(ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * P + d0 + (lane >> 4) * 8;
        uint32_t r0, r1, r2, r3;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(src));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
        mma_bf16_16816(o[n], a, r0, r1);
        if (n + 1 < NT) mma_bf16_16816(o[n + 1], a, r2, r3);
      }
    }
  }
  float inv[2] = {l[0] > 0.f ? 1.f / l[0] : 0.f, l[1] > 0.f ? 1.f / l[1] : 0.f};
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = g + rr * 8;
    if (r >= nrows) continue;
    const size_t orow = HROWS ? static_cast<size_t>(row0) * heads + h + r : static_cast<size_t>(row0 + r) * heads + h;
    if (gate && nsplit == 1)            // orow = token row * heads + head
      inv[rr] *= sigmoid_f(gate[(orow / heads) * ld_gate + (orow % heads)]);
    if (nsplit == 1) {
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int d = (warp * NT + n) * 8 + 2 * tq;
        __nv_bfloat162 v = __floats2bfloat162_rn(o[n][rr * 2] * inv[rr], o[n][rr * 2 + 1] * inv[rr]);
        *reinterpret_cast<__nv_bfloat162*>(out + orow * kv_rank + d) = v;
      }
    } else {
      const size_t pi = orow * nsplit + blockIdx.z;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int d = (warp * NT + n) * 8 + 2 * tq;
        part_o[pi * kv_rank + d] = o[n][rr * 2];
        part_o[pi * kv_rank + d + 1] = o[n][rr * 2 + 1];
      }
      if (warp == 0 && tq == 0) {
        part_ml[pi * 2] = m[rr];
        part_ml[pi * 2 + 1] = l[rr];
      }
    }
  }
}

static bool latent_mma_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_LATENT_MMA");       // 0: the FMA kernel for every step (A/B arm)
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
static bool latent_mma_shape_ok(int kv_rank, int rot_dim) {
  const int R = kv_rank + rot_dim;
  if (R % 16 != 0 || kv_rank % 64 != 0 || kv_rank > 512) return false;
  return static_cast<size_t>(MKT + MQ) * (R + 8) * 2 + static_cast<size_t>(MQ) * (MKT + 1) * 4 <= 200 * 1024;
}
// key splits of the heads-as-rows form: two blocks per SM, at most one split per key tile of the window, at most 16
static int latent_attn_mma_splits(int T, int heads, int window) {
  const int blocks = T * ((heads + MQ - 1) / MQ);
  int n = (2 * sm_count() + blocks - 1) / blocks;
  if (window > 0) n = std::min(n, (window + MKT - 1) / MKT);
  return std::max(1, std::min(n, 16));
}
// true when the tensor-core kernel took the step.  hrows: steps of few rows (heads as MMA rows, keys split).
static bool launch_latent_attn_mma(void* out, const float* q_full, const void* cache, const float* sink,
                                   const float* gate, int ld_gate, const uint32_t* cu, const uint32_t* ctx, const uint32_t* block_tables, int max_blocks,
                                   int num_seqs, int T, int heads, int kv_rank, int rot_dim, int window, float scale,
                                   bool hrows, void* workspace, cudaStream_t st_) {
  const int R = kv_rank + rot_dim;
  if (!latent_mma_enabled() || !latent_mma_shape_ok(kv_rank, rot_dim)) return false;
  const size_t smem = static_cast<size_t>(MKT + MQ) * (R + 8) * 2 + static_cast<size_t>(MQ) * (MKT + 1) * 4;
  const int nsplit = hrows && workspace ? latent_attn_mma_splits(T, heads, window) : 1;
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o ? part_o + static_cast<size_t>(T) * heads * nsplit * kv_rank : nullptr;
  const dim3 grid = hrows ? dim3(T, (heads + MQ - 1) / MQ, nsplit) : dim3((T + MQ - 1) / MQ + num_seqs, heads, 1);
#define B200_LMMA2(NT, HR)                                                                                        \
  {                                                                                                                \
    auto kern = latent_attn_mma_kernel<NT, HR>;                                                                    \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));               \
    kern<<<grid, 128, smem, st_>>>((__nv_bfloat16*)out, q_full, (const __nv_bfloat16*)cache, sink, gate, ld_gate,  \
                                   cu, ctx, block_tables, max_blocks, num_seqs, heads, kv_rank, rot_dim, window,   \
                                   scale, nsplit, part_o, part_ml);                                                \
  }
#define B200_LMMA(NT)                 \
  if (hrows) B200_LMMA2(NT, true)     \
  else B200_LMMA2(NT, false)
  switch (kv_rank / 32) {
    case 2: B200_LMMA(2) break;
    case 4: B200_LMMA(4) break;
    case 6: B200_LMMA(6) break;
    case 8: B200_LMMA(8) break;
    case 10: B200_LMMA(10) break;
    case 12: B200_LMMA(12) break;
    case 14: B200_LMMA(14) break;
    case 16: B200_LMMA(16) break;
    default: return false;
  }
#undef B200_LMMA
#undef B200_LMMA2
  B200_CUDA_LAUNCH_CHECK();
  if (nsplit > 1) {
    latent_attn_merge_kernel<__nv_bfloat16><<<T * heads, kv_rank >= 256 ? 256 : 128, 0, st_>>>(
        (__nv_bfloat16*)out, part_o, part_ml, sink, gate, ld_gate, heads, kv_rank, nsplit);
    B200_CUDA_LAUNCH_CHECK();
  }
  return true;
}

int latent_attn_splits(int T, int heads, int window) {
  const int nw = heads >= 8 ? 8 : (heads >= 4 ? 4 : (heads >= 2 ? 2 : 1));
  const int blocks = T * ((heads + nw - 1) / nw);
  int n = (2 * sm_count() + blocks - 1) / blocks;           // aim at two blocks per SM
  if (window > 0) n = std::min(n, (window + 31) / 32);
  return std::max(1, std::min(n, 16));
}
size_t latent_attn_workspace_bytes(int T, int heads, int kv_rank, int window) {
  const int n = std::max(latent_attn_splits(T, heads, window), latent_attn_mma_splits(T, heads, window));
  return n == 1 ? 0 : static_cast<size_t>(T) * heads * n * (kv_rank + 2) * 4;
}

void launch_latent_attn(void* out, const float* q_full, const void* cache, const float* sink, const float* gate,
                        int ld_gate, const uint32_t* cu, const uint32_t* ctx, const uint32_t* block_tables,
                        int max_blocks, int num_seqs, int T, int heads, int kv_rank, int rot_dim, int window, float scale,
                        int dt, void* workspace, cudaStream_t st_) {
  if (T <= 0) return;
  // steps of many rows in bf16: the tensor-core kernel (small steps keep the split form below)
  if (!dt && launch_latent_attn_mma(out, q_full, cache, sink, gate, ld_gate, cu, ctx, block_tables, max_blocks, num_seqs, T, heads,
                                    kv_rank, rot_dim, window, scale, /*hrows=*/T <= 2 * sm_count() / 4, workspace, st_))
    return;
  const int R = kv_rank + rot_dim, Rp = R | 1;
  const int nw = heads >= 8 ? 8 : (heads >= 4 ? 4 : (heads >= 2 ? 2 : 1));
  int key_tile = 32;
  auto bytes = [&](int kt) { return (static_cast<size_t>(kt) * Rp + static_cast<size_t>(nw) * (R + kv_rank)) * 4; };
  while (key_tile > 1 && bytes(key_tile) > 200 * 1024) key_tile >>= 1;
  const size_t smem = bytes(key_tile);
  if (smem > 220 * 1024) {
    set_error(1, "latent_attn: kv_rank + rot_dim too large for the shared-memory tile");
    return;
  }
  // few token rows (decoding): the keys of a row are split over several blocks and merged afterwards
  const int nsplit = workspace ? latent_attn_splits(T, heads, window) : 1;
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o ? part_o + static_cast<size_t>(T) * heads * nsplit * kv_rank : nullptr;
  const dim3 grid(T, (heads + nw - 1) / nw, nsplit);
  if (dt) {
    auto kern = latent_attn_kernel<float>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, nw * 32, smem, st_>>>((float*)out, q_full, (const float*)cache, sink, gate, ld_gate, cu, ctx,
                                       block_tables, max_blocks, num_seqs, heads, kv_rank, rot_dim, window, scale,
                                       key_tile, nsplit, part_o, part_ml);
  } else {
    auto kern = latent_attn_kernel<__nv_bfloat16>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, nw * 32, smem, st_>>>((__nv_bfloat16*)out, q_full, (const __nv_bfloat16*)cache, sink, gate, ld_gate,
                                       cu, ctx, block_tables, max_blocks, num_seqs, heads, kv_rank, rot_dim, window,
                                       scale, key_tile, nsplit, part_o, part_ml);
  }
  B200_CUDA_LAUNCH_CHECK();
  if (nsplit > 1) {
    const int th = kv_rank >= 256 ? 256 : 128;
    if (dt)
      latent_attn_merge_kernel<float><<<T * heads, th, 0, st_>>>((float*)out, part_o, part_ml, sink, gate, ld_gate,
                                                                 heads, kv_rank, nsplit);
    else
      latent_attn_merge_kernel<__nv_bfloat16><<<T * heads, th, 0, st_>>>((__nv_bfloat16*)out, part_o, part_ml, sink,
                                                                         gate, ld_gate, heads, kv_rank, nsplit);
    B200_CUDA_LAUNCH_CHECK();
  }
}

}  // namespace b200

extern "C" {
void b200_latent_prep(const float* qc, int32_t ldq, void* q_plain, float* q_full, void* cache,
                      const float* latent_norm_w, const double* rot_freq, float rot_mag, const int64_t* positions,
                      const int64_t* slot_mapping, int32_t num_tokens, int32_t heads, int32_t dim, int32_t rot_dim,
                      int32_t rot_dims, int32_t kv_rank, float eps, int32_t dt, int64_t stream) {
  B200_CHECK_ARG(qc && q_plain && q_full && cache && latent_norm_w && (rot_dims == 0 || rot_freq) && positions && slot_mapping &&
                     heads > 0 && dim >= 0 && rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim &&
                     rot_dims % 2 == 0 && kv_rank > 0 && (dt == 0 || dt == 1),
                 "latent_prep: bad arguments");
  b200::launch_latent_prep(qc, ldq, q_plain, q_full, cache, latent_norm_w, rot_freq, rot_mag, positions, slot_mapping,
                           num_tokens, heads, dim, rot_dim, rot_dims, kv_rank, eps, dt,
                           reinterpret_cast<cudaStream_t>(stream));
}
void b200_latent_prep_queries(const float* qc, int32_t ldq, void* q_plain, float* q_full, const double* rot_freq,
                              float rot_mag, const int64_t* positions, int32_t num_tokens, int32_t heads, int32_t dim,
                              int32_t rot_dim, int32_t rot_dims, int32_t kv_rank, int32_t dt, int64_t stream) {
  B200_CHECK_ARG(qc && q_plain && q_full && (rot_dims == 0 || rot_freq) && positions && heads > 0 && dim >= 0 &&
                     rot_dim >= 0 && rot_dims >= 0 && rot_dims <= rot_dim && rot_dims % 2 == 0 && kv_rank > 0 &&
                     (dt == 0 || dt == 1),
                 "latent_prep_queries: bad arguments");
  b200::launch_latent_prep(qc, ldq, q_plain, q_full, nullptr, nullptr, rot_freq, rot_mag, positions, nullptr, num_tokens,
                           heads, dim, rot_dim, rot_dims, kv_rank, 0.f, dt, reinterpret_cast<cudaStream_t>(stream));
}
void b200_latent_attn_gated(void* out, const float* q_full, const void* cache, const float* sink, const float* gate,
                            int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                            const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs,
                            int32_t num_tokens, int32_t heads, int32_t kv_rank, int32_t rot_dim, int32_t window,
                            float scale, int32_t dt, void* workspace, int64_t stream) {
  B200_CHECK_ARG(out && q_full && cache && cu_seqlens_q && context_lens && block_tables && num_seqs > 0 && heads > 0 &&
                     kv_rank > 0 && rot_dim >= 0 && (dt == 0 || dt == 1),
                 "latent_attn: bad arguments");
  b200::launch_latent_attn(out, q_full, cache, sink, gate, ld_gate, cu_seqlens_q, context_lens, block_tables,
                           max_blocks_per_seq, num_seqs, num_tokens, heads, kv_rank, rot_dim, window, scale, dt,
                           workspace, reinterpret_cast<cudaStream_t>(stream));
}
void b200_latent_attn(void* out, const float* q_full, const void* cache, const float* sink,
                      const uint32_t* cu_seqlens_q, const uint32_t* context_lens, const uint32_t* block_tables,
                      int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens, int32_t heads, int32_t kv_rank,
                      int32_t rot_dim, int32_t window, float scale, int32_t dt, void* workspace, int64_t stream) {
  b200_latent_attn_gated(out, q_full, cache, sink, nullptr, 0, cu_seqlens_q, context_lens, block_tables,
                         max_blocks_per_seq, num_seqs, num_tokens, heads, kv_rank, rot_dim, window, scale, dt, workspace,
                         stream);
}
int64_t b200_latent_attn_workspace_bytes(int32_t num_tokens, int32_t heads, int32_t kv_rank, int32_t window) {
  return static_cast<int64_t>(b200::latent_attn_workspace_bytes(num_tokens, heads, kv_rank, window));
}
}
