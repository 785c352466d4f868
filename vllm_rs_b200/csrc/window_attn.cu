// Softmax attention with grouped key / value heads over paged K and V caches, for ragged steps (prompt portions and
// decoded tokens alike), for decoders that keep queries, scores and the softmax in fp32.  Beside latent_attn.cu (one
// shared latent row per token) and paged_attn_decode.cu / attn_prefill*.cu (fp16 / bf16 residual models).
//
// Caches, one row per token and layer, pages of 64 tokens (the block manager's blocks):
//   k_cache [num_blocks, 64, kv_heads, dim]    v_cache [num_blocks, 64, kv_heads, vdim]    (bf16 or fp32)
// Query head h reads key / value head h / (heads / kv_heads).  Options, each a parameter:
//   * sliding window that keeps the first tokens: position i sees j <= i with i - j < window or j < keep_first
//     (window <= 0: every j <= i); nothing is re-numbered: rotary angles and distances use the true positions
//   * capped scores: s <- cap * tanh(s / cap)  (cap <= 0: off), applied after the scale
//   * a per-head sink logit that joins the softmax denominator without a key or value (NULL: none); a logit of 0
//     contributes exp(0) = 1, i.e. p_j = e^(s_j) / (1 + sum_k e^(s_k))
//   * a per-head output gate: the head's output is multiplied by sigmoid(gate[t, h]) (NULL: none), or a gate per
//     output element (gate[t, h * vdim + d])
//   * a distance bias: the score of query position i against key position j is lowered by slope_h * (i - j), after
//     scale and cap (slopes fp32 per head, NULL: none)
//   * in the prep kernel: q / k norms per head with one weight of size dim shared by the heads (instead of over the
//     whole projection), values that are the un-normed key rows (no v projection), and a query temperature
//     1 + coef * ln(floor((p + 1) / every) + 1) at position p
//   * rotary pairs either interleaved (2i, 2i+1) or as the two halves of the rotated part (i, i + rot_dims / 2), with a
//     factor on cos and sin
//   * rotated values: the value row of position j is turned by j (all of vdim) before it is cached, and
//     attn_finish_kernel turns a head's output back by its own position, so that a value enters the output turned by
//     the distance between key and query
//   * a chunked mask: position i sees j <= i only inside its own chunk of `chunk` positions (chunk c holds the true
//     positions c * chunk .. c * chunk + chunk - 1, however a prompt is cut)
//   * several score maps over one set of values (differential attention): the maps' query and key heads are laid out
//     map after map, the value cache has v_heads heads and key head g reads value head g % v_heads; the maps' outputs
//     are written in fp32 and attn_finish_kernel combines them (a_0 - lambda a_1), norms per head, scales and gates
//
// window_attn_prep_kernel: from the fused projection row [q (heads x dim) | k (kv_heads x dim) | v (kv_heads x vdim) | ...]
// (fp32) it adds the projection biases, RMS-norms q and k over their WHOLE projection (all heads at once, weights of
// that size; NULL: no norm), rotates the first rot_dims entries of every q and k head as interleaved pairs (2i, 2i+1)
// by the angle position * freq[i] (angles in double), writes the K and V rows at the token's slot and the query in fp32.
//
// Two attention kernels: an fp32 FMA form (any sizes, both dtypes; the rows of small steps split their keys over several
// blocks and merge) and bf16 tensor-core forms: for steps of many rows 64 token rows per block with the softmax in the
// accumulator registers (dim and vdim multiples of 16, vdim up to 128; otherwise 16 rows per block, vdim a multiple of
// 32), for steps of few rows the query heads of one key / value head as the MMA rows with the keys split over blocks.
#include "../../include/b200_vllm.h"
#include <algorithm>
#include <cstdlib>

#include "seqmix.cuh"

namespace b200 {
using namespace seqmix;

template <typename T>
__global__ void window_attn_prep_kernel(const float* __restrict__ proj, int ld, const float* __restrict__ bias,
                                        const float* __restrict__ q_norm_w, const float* __restrict__ k_norm_w,
                                        const double* __restrict__ rot_freq, const int64_t* __restrict__ positions,
                                        const int64_t* __restrict__ slots, float* __restrict__ q_out,
                                        T* __restrict__ k_cache, T* __restrict__ v_cache, int heads, int kv_heads,
                                        int dim, int vdim, int rot_dims, float eps, int head_norm, int v_from_k,
                                        int q_temp_every, float q_temp_coef, int rot_half, float rot_mag,
                                        const double* __restrict__ v_rot_freq, int v_heads) {
  extern __shared__ float sm[];          // cos[rot_dims/2] | sin[rot_dims/2] | red[36] | hinv[heads + kv_heads] | vcos, vsin[vdim/2]
  const int half = rot_dims / 2, vhalf = vdim / 2;
  float* cs = sm;
  float* sn = sm + half;
  float* red = sm + 2 * half;
  float* hinv = red + 36;
  float* vcs = hinv + heads + kv_heads;
  float* vsn = vcs + vhalf;
  const int t = blockIdx.x;
  const int nq = heads * dim, nk = kv_heads * dim, nv = v_heads * vdim;
  const float* qr = proj + static_cast<size_t>(t) * ld;
  const float* kr = qr + nq;
  const float* vr = v_from_k ? kr : kr + nk;            // the value row is a copy of the raw key row (vdim == dim)
  const float* bq = bias;
  const float* bk = bias ? bias + nq : nullptr;
  const float* bv = bias ? (v_from_k ? bk : bias + nq + nk) : nullptr;
  const double pos = static_cast<double>(positions[t]);
  const float q_temp = q_temp_every > 0
                           ? 1.f + q_temp_coef * logf(static_cast<float>((positions[t] + 1) / q_temp_every) + 1.f)
                           : 1.f;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    double s, c;
    sincos(pos * rot_freq[i], &s, &c);
    cs[i] = static_cast<float>(c) * rot_mag;
    sn[i] = static_cast<float>(s) * rot_mag;
  }
  if (v_rot_freq)
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
      double s, c;
      sincos(pos * v_rot_freq[i], &s, &c);
      vcs[i] = static_cast<float>(c);
      vsn[i] = static_cast<float>(s);
    }
  float inv_q = 1.f, inv_k = 1.f;
  const bool with_k = k_cache != nullptr;          // a row of queries only has no key block to norm
  if (head_norm) {                       // every q and k head on its own: a warp per head
    const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int hh = warp; hh < heads + (with_k ? kv_heads : 0); hh += nw) {
      const bool isq = hh < heads;
      const float* src = isq ? qr + hh * dim : kr + (hh - heads) * dim;
      const float* b = isq ? (bq ? bq + hh * dim : nullptr) : (bk ? bk + (hh - heads) * dim : nullptr);
      float ss = 0.f;
      for (int d = lane; d < dim; d += 32) {
        const float v = src[d] + (b ? b[d] : 0.f);
        ss += v * v;
      }
      ss = lanes_sum(ss);
      if (lane == 0) hinv[hh] = (isq ? q_norm_w : k_norm_w) ? 1.f / sqrtf(ss / static_cast<float>(dim) + eps) : 1.f;
    }
  } else if (q_norm_w) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < nq; d += blockDim.x) {
      const float v = qr[d] + (bq ? bq[d] : 0.f);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    inv_q = 1.f / sqrtf(ss / static_cast<float>(nq) + eps);
  }
  if (!head_norm && k_norm_w && with_k) {
    float ss = 0.f;
    for (int d = threadIdx.x; d < nk; d += blockDim.x) {
      const float v = kr[d] + (bk ? bk[d] : 0.f);
      ss += v * v;
    }
    ss = block_sum(ss, red);
    inv_k = 1.f / sqrtf(ss / static_cast<float>(nk) + eps);
  }
  __syncthreads();                       // the cos / sin table is complete
  // one (possibly rotated) entry of a projection whose heads are `dim` wide
  auto entry = [&](const float* raw, const float* b, const float* w, float inv, int hbase, int e) {
    auto plain = [&](int i) {
      const float v = raw[i] + (b ? b[i] : 0.f);
      return head_norm ? v * hinv[hbase + i / dim] * (w ? w[i % dim] : 1.f) : v * inv * (w ? w[i] : 1.f);
    };
    const int d = e % dim;
    if (d >= rot_dims) return plain(e);
    // the pair (u, v) this entry belongs to, and whether it is the pair's second member
    const bool second = rot_half ? d >= half : (d & 1) != 0;
    const int i = rot_half ? (second ? d - half : d) : d >> 1;
    const int eu = rot_half ? e - d + i : e - (d & 1), ev = rot_half ? eu + half : eu + 1;
    const float u = plain(eu), v = plain(ev);
    return second ? v * cs[i] + u * sn[i] : u * cs[i] - v * sn[i];
  };
  for (int e = threadIdx.x; e < nq; e += blockDim.x)
    q_out[static_cast<size_t>(t) * nq + e] = entry(qr, bq, q_norm_w, inv_q, 0, e) * q_temp;
  const int64_t slot = slots[t];
  if (slot >= 0 && k_cache) {            // no cache: the row brought queries only
    for (int e = threadIdx.x; e < nk; e += blockDim.x)
      st(k_cache + static_cast<size_t>(slot) * nk + e, entry(kr, bk, k_norm_w, inv_k, heads, e));
    for (int e = threadIdx.x; e < nv; e += blockDim.x) {
      float val = vr[e] + (bv ? bv[e] : 0.f);
      if (v_rot_freq) {                  // the value row turned by its own position, all of vdim
        const int d = e % vdim;
        const bool second = rot_half ? d >= vhalf : (d & 1) != 0;
        const int i = rot_half ? (second ? d - vhalf : d) : d >> 1;
        const int eo = second ? (rot_half ? e - vhalf : e - 1) : (rot_half ? e + vhalf : e + 1);   // the other member
        const float other = vr[eo] + (bv ? bv[eo] : 0.f);
        val = second ? val * vcs[i] + other * vsn[i] : val * vcs[i] - other * vsn[i];
      }
      st(v_cache + static_cast<size_t>(slot) * nv + e, val);
    }
  }
}

// The keys that position `pos` sees, as one run of indices 0 .. count-1: first the kept tokens that have left the
// window, then the window itself.
// first position of the window (and, with a chunked mask, of the chunk) that position `pos` sees
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  return chunk > 0 ? max(lo, pos / chunk * chunk) : lo;
}
template <typename T> __device__ __forceinline__ void st_out(T* out, size_t i, float v, int f32) {
  if (f32) reinterpret_cast<float*>(out)[i] = v;
  else st(out + i, v);
}
struct Visible {
  int n_first, lo, count;
  __device__ __forceinline__ Visible(int pos, int window, int keep_first, int chunk = 0) {
    lo = first_visible(pos, window, chunk);
    n_first = min(max(keep_first, 0), lo);
    count = n_first + (pos - lo + 1);
  }
  __device__ __forceinline__ int key(int idx) const { return idx < n_first ? idx : lo + (idx - n_first); }
};

__device__ __forceinline__ float cap_score(float s, float cap) { return cap > 0.f ? cap * tanhf(s / cap) : s; }

// grid = (token rows, kv heads, key splits); a block's warps each own one query head of the group at a time.  The K and
// V rows of a tile of visible keys are staged once in shared memory (fp32) and used by every head of the group.
template <typename T>
__global__ void window_attn_kernel(T* __restrict__ out, const float* __restrict__ q, const T* __restrict__ k_cache,
                                   const T* __restrict__ v_cache, const float* __restrict__ sink,
                                   const float* __restrict__ gate, int ld_gate, const uint32_t* __restrict__ cu,
                                   const uint32_t* __restrict__ ctx, const uint32_t* __restrict__ block_tables,
                                   int max_blocks, int num_seqs, int heads, int kv_heads, int dim, int vdim, int window,
                                   int keep_first, float scale, float softcap, int key_tile, int nsplit,
                                   float* __restrict__ part_o, float* __restrict__ part_ml,
                                   const float* __restrict__ slopes, int gate_elems, int chunk, int v_heads,
                                   int out_f32) {
  extern __shared__ float sm[];
  const int Dp = dim | 1;                               // odd row pitch: a lane per key reads conflict-free
  const int nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* ks = sm;                                       // [key_tile][Dp]
  float* vs = ks + static_cast<size_t>(key_tile) * Dp;  // [key_tile][vdim]
  float* qs = vs + static_cast<size_t>(key_tile) * vdim;   // [nw][dim]
  float* os = qs + static_cast<size_t>(nw) * dim;       // [nw][vdim]
  const int t = blockIdx.x, g = blockIdx.y;
  const int b = seq_of_row(cu, num_seqs, t);
  const int qlen = static_cast<int>(cu[b + 1] - cu[b]);
  const int pos = static_cast<int>(ctx[b]) - qlen + (t - static_cast<int>(cu[b]));
  const Visible vis(pos, window, keep_first, chunk);
  const int per_group = heads / kv_heads;
  const int gv = g % v_heads;                           // the value head this key head reads
  const uint32_t* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int ntiles = (vis.count + key_tile - 1) / key_tile;
  const int per = (ntiles + nsplit - 1) / nsplit;
  const int first = static_cast<int>(blockIdx.z) * per * key_tile;
  const int last = min(vis.count, first + per * key_tile);            // exclusive
  for (int h0 = 0; h0 < per_group; h0 += nw) {                         // groups wider than the block take several rounds
    const int hg = h0 + warp;
    const bool live = hg < per_group;
    const int h = g * per_group + hg;
    __syncthreads();
    if (live) {
      const float* qh = q + (static_cast<size_t>(t) * heads + h) * dim;
      for (int d = lane; d < dim; d += 32) qs[warp * dim + d] = qh[d];
      for (int d = lane; d < vdim; d += 32) os[warp * vdim + d] = 0.f;
    }
    float m = -1e30f, l = 0.f;
    if (live && sink && nsplit == 1) {        // split runs add the sink when the parts are merged
      m = sink[h];
      l = 1.f;
    }
    const float slope = (live && slopes) ? slopes[h] : 0.f;
    for (int i0 = first; i0 < last; i0 += key_tile) {
      const int nk = min(key_tile, last - i0);
      __syncthreads();
      for (int e = threadIdx.x; e < nk * dim; e += blockDim.x) {
        const int k = e / dim, d = e % dim, j = vis.key(i0 + k);
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        ks[k * Dp + d] = ld(k_cache + (slot * kv_heads + g) * dim + d);
      }
      for (int e = threadIdx.x; e < nk * vdim; e += blockDim.x) {
        const int k = e / vdim, d = e % vdim, j = vis.key(i0 + k);
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        vs[k * vdim + d] = ld(v_cache + (slot * v_heads + gv) * vdim + d);
      }
      __syncthreads();
      if (!live) continue;
      for (int k0 = 0; k0 < nk; k0 += 32) {
        const int k = k0 + lane;
        float s = -1e30f;
        if (k < nk) {
          float acc = 0.f;
          const float* kr = ks + k * Dp;
          const float* qw = qs + warp * dim;
          for (int d = 0; d < dim; ++d) acc += qw[d] * kr[d];
          s = cap_score(acc * scale, softcap) - slope * static_cast<float>(pos - vis.key(i0 + k));
        }
        const float mt = lanes_max(s);
        const float mn = fmaxf(m, mt);
        const float alpha = expf(m - mn);
        const float p = k < nk ? expf(s - mn) : 0.f;
        l = l * alpha + lanes_sum(p);
        m = mn;
        const int cnt = min(32, nk - k0);
        for (int d0 = 0; d0 < vdim; d0 += 32) {          // every lane takes part in the shuffles
          const int d = d0 + lane;
          const bool ok = d < vdim;
          float acc = ok ? os[warp * vdim + d] * alpha : 0.f;
          for (int kk = 0; kk < cnt; ++kk) {
            const float pk = __shfl_sync(0xffffffffu, p, kk);
            if (ok) acc += pk * vs[(k0 + kk) * vdim + d];
          }
          if (ok) os[warp * vdim + d] = acc;
        }
      }
    }
    if (live && nsplit == 1) {
      float inv = l > 0.f ? 1.f / l : 0.f;
      if (gate && !gate_elems) inv *= sigmoid_f(gate[static_cast<size_t>(t) * ld_gate + h]);
      const float* ge = (gate && gate_elems) ? gate + static_cast<size_t>(t) * ld_gate + static_cast<size_t>(h) * vdim : nullptr;
      const size_t o = (static_cast<size_t>(t) * heads + h) * vdim;
      for (int d = lane; d < vdim; d += 32) st_out(out, o + d, os[warp * vdim + d] * inv * (ge ? sigmoid_f(ge[d]) : 1.f), out_f32);
    } else if (live) {
      const size_t pi = (static_cast<size_t>(t) * heads + h) * nsplit + blockIdx.z;
      for (int d = lane; d < vdim; d += 32) part_o[pi * vdim + d] = os[warp * vdim + d];
      if (lane == 0) {
        part_ml[pi * 2] = m;
        part_ml[pi * 2 + 1] = l;
      }
    }
  }
}

// one block per (token, head): the parts of a split run and the sink meet in one softmax; the gate is applied here
template <typename T>
__global__ void window_attn_merge_kernel(T* __restrict__ out, const float* __restrict__ part_o,
                                         const float* __restrict__ part_ml, const float* __restrict__ sink,
                                         const float* __restrict__ gate, int ld_gate, int heads, int vdim, int nsplit,
                                         int gate_elems, int out_f32) {
  const size_t th = blockIdx.x;
  const int h = static_cast<int>(th % heads);
  const size_t t = th / heads;
  const float* ml = part_ml + th * nsplit * 2;
  float m = sink ? sink[h] : -1e30f;
  for (int z = 0; z < nsplit; ++z) m = fmaxf(m, ml[2 * z]);
  float l = sink ? expf(sink[h] - m) : 0.f;
  for (int z = 0; z < nsplit; ++z) l += ml[2 * z + 1] * expf(ml[2 * z] - m);
  float inv = l > 0.f ? 1.f / l : 0.f;
  if (gate && !gate_elems) inv *= sigmoid_f(gate[t * ld_gate + h]);
  const float* ge = (gate && gate_elems) ? gate + t * ld_gate + static_cast<size_t>(h) * vdim : nullptr;
  for (int d = threadIdx.x; d < vdim; d += blockDim.x) {
    float acc = 0.f;
    for (int z = 0; z < nsplit; ++z) acc += part_o[(th * nsplit + z) * vdim + d] * expf(ml[2 * z] - m);
    st_out(out, th * vdim + d, acc * inv * (ge ? sigmoid_f(ge[d]) : 1.f), out_f32);
  }
}

void launch_window_attn_prep(const float* proj, int ld, const float* bias, const float* q_norm_w, const float* k_norm_w,
                             const double* rot_freq, const int64_t* positions, const int64_t* slots, float* q_out,
                             void* k_cache, void* v_cache, int T, int heads, int kv_heads, int dim, int vdim,
                             int rot_dims, float eps, int dt, const b200_attn_options* opt, cudaStream_t st_) {
  if (T <= 0) return;
  const int head_norm = opt ? opt->head_norm : 0, v_from_k = opt ? opt->v_from_k : 0;
  const int q_every = opt ? opt->q_temp_every : 0;
  const float q_coef = opt ? opt->q_temp_coef : 0.f;
  const int rot_half = opt ? opt->rot_half : 0;
  const float rot_mag = (opt && opt->rot_mag != 0.f) ? opt->rot_mag : 1.f;
  const double* v_rot = opt ? opt->v_rot_freq : nullptr;
  const int v_heads = (opt && opt->v_heads > 0) ? opt->v_heads : kv_heads;
  if (opt && opt->no_cache) k_cache = v_cache = nullptr;
  if (v_from_k && (vdim != dim || v_heads != kv_heads)) {
    set_error(1, "window_attn_prep: values taken from the key rows need vdim == dim and as many value heads as key heads");
    return;
  }
  if ((v_rot && (vdim % 2 != 0 || v_from_k)) || kv_heads % v_heads != 0) {
    set_error(1, "window_attn_prep: rotated values need an even vdim and a projection of their own; kv_heads is a multiple of v_heads");
    return;
  }
  const size_t smem = (static_cast<size_t>(rot_dims) + 40 + heads + kv_heads + vdim + 2) * 4;
  if (dt)
    window_attn_prep_kernel<float><<<T, 256, smem, st_>>>(proj, ld, bias, q_norm_w, k_norm_w, rot_freq, positions, slots,
                                                          q_out, (float*)k_cache, (float*)v_cache, heads, kv_heads, dim,
                                                          vdim, rot_dims, eps, head_norm, v_from_k, q_every, q_coef,
                                                          rot_half, rot_mag, v_rot, v_heads);
  else
    window_attn_prep_kernel<__nv_bfloat16><<<T, 256, smem, st_>>>(proj, ld, bias, q_norm_w, k_norm_w, rot_freq, positions,
                                                                  slots, q_out, (__nv_bfloat16*)k_cache,
                                                                  (__nv_bfloat16*)v_cache, heads, kv_heads, dim, vdim,
                                                                  rot_dims, eps, head_norm, v_from_k, q_every, q_coef,
                                                                  rot_half, rot_mag, v_rot, v_heads);
  B200_CUDA_LAUNCH_CHECK();
}

// ---- bf16 tensor-core form for steps of many rows (prompt portions).  Block = 4 warps = one query head x 16
// consecutive token rows of ONE sequence.  Per tile of 64 visible-key candidates: every warp computes the scores of 16
// keys (S = Q K^T, mma.sync m16n8k16 bf16 -> fp32, Q and K from shared memory), the fp32 scores meet in shared memory,
// every warp runs the same fp32 online softmax over all 64 (cap, window / kept-first / causal mask per element, sink as
// the initial denominator) and multiplies P (bf16) with ITS quarter of the value columns (V fragments by
// ldmatrix.trans).  Tiles are 64-aligned runs of positions: first those that hold kept tokens, then those from the
// window's start of the block's first row to its last row; a tile is visited once.
constexpr int WQ = 16, WKT = 64;
__device__ __forceinline__ void wmma_bf16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t wpack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// NT = n-tiles (8 value columns each) per warp = vdim / 32.  HROWS = false: the 16 MMA rows are 16 consecutive token
// rows of one query head (prompt portions).  HROWS = true (steps of few rows, decoding): the 16 rows are the query
// heads of ONE key / value head's group at one token -- they share the K and V rows, so one pass over the cache serves
// them all -- and blockIdx.z owns a contiguous run of tiles of the token's visible keys (kept tokens first, then the
// window); with nsplit > 1 the unnormalised parts go to part_o / part_ml and window_attn_merge_kernel finishes the
// softmax (it adds the sink and the gate).  Where several score maps share one set of values (kv_heads = maps x
// v_heads), the rows of a block are the group's heads under EVERY map (map after map): the K tiles of all maps are
// staged, each map's scores are computed against its own keys, and the V tile is read once for all of them.
template <int NT, bool HROWS>
__global__ void __launch_bounds__(128)
window_attn_mma_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ q,
                       const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                       const float* __restrict__ sink, const float* __restrict__ gate, int ld_gate,
                       const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx,
                       const uint32_t* __restrict__ block_tables, int max_blocks, int num_seqs, int heads, int kv_heads,
                       int dim, int vdim, int window, int keep_first, float scale, float softcap, int nsplit,
                       float* __restrict__ part_o, float* __restrict__ part_ml, const float* __restrict__ slopes,
                       int gate_elems, int chunk, int v_heads, int out_f32) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int P = dim + 8, PV = vdim + 8;                   // row pitches in bf16 elements (16-byte multiples)
  // maps whose K tiles a block stages: all of them in the heads-as-rows form, the one of the block's head otherwise
  const int maps = HROWS ? kv_heads / v_heads : 1;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);              // [maps][WKT][P]
  __nv_bfloat16* Vs = Ks + static_cast<size_t>(maps) * WKT * P;             // [WKT][PV]
  __nv_bfloat16* Qs = Vs + static_cast<size_t>(WKT) * PV;                   // [WQ][P]
  float* Ss = reinterpret_cast<float*>(Qs + static_cast<size_t>(WQ) * P);   // [WQ][WKT + 1]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const int per_group = heads / kv_heads;
  int b = -1, row0 = 0, nrows = 0, h = blockIdx.y, kvh = 0, nh = 1;
  if (HROWS) {          // one token; nh heads of value head kvh's group under every map: row r = map (r / nh), head h + r % nh
    const int hpg = min(per_group, WQ / maps), rounds = (per_group + hpg - 1) / hpg;
    row0 = blockIdx.x;
    b = seq_of_row(cu, num_seqs, row0);
    kvh = blockIdx.y / rounds;                   // (the value head; map m reads key head m * v_heads + kvh)
    const int first_in_group = (blockIdx.y % rounds) * hpg;
    h = kvh * per_group + first_in_group;
    nh = min(hpg, per_group - first_in_group);
    nrows = nh * maps;
  } else {                                       // 16 token rows of one sequence (tiles never straddle sequences)
    int acc = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = static_cast<int>(cu[s + 1] - cu[s]), tiles = (n + WQ - 1) / WQ;
      if (static_cast<int>(blockIdx.x) < acc + tiles) {
        const int k = blockIdx.x - acc;
        b = s;
        row0 = cu[s] + k * WQ;
        nrows = min(WQ, n - k * WQ);
        break;
      }
      acc += tiles;
    }
    if (b < 0) return;
    kvh = h / per_group;
  }
  const int pos0 = static_cast<int>(ctx[b]) - static_cast<int>(cu[b + 1] - cu[b]) + (row0 - static_cast<int>(cu[b]));
  const int pos_last = HROWS ? pos0 : pos0 + nrows - 1;
  const int key_lo = first_visible(pos0, window, chunk);               // first key of the window of the first row
  const int vh = kvh % v_heads;                                         // the value head this key head reads
  // heads-as-rows: the query head of row r (the heads of map m are m * heads / maps ..)
  auto head_of = [&](int r) { return (r / nh) * (heads / maps) + h + r % nh; };
  for (int e = threadIdx.x; e < WQ * dim; e += blockDim.x) {
    const int r = e / dim, d = e % dim;
    const size_t qrow = HROWS ? static_cast<size_t>(row0) * heads + head_of(min(r, nrows - 1))
                              : static_cast<size_t>(row0 + r) * heads + h;
    const float v = r < nrows ? q[qrow * dim + d] : 0.f;
    Qs[r * P + d] = __float2bfloat16_rn(v);
  }
  float m[2], l[2], slope[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int hh = HROWS ? head_of(min(g + rr * 8, nrows - 1)) : h;
    const bool with_sink = sink && nsplit == 1;            // split runs add the sink when the parts are merged
    m[rr] = with_sink ? sink[hh] : -1e30f;
    l[rr] = with_sink ? 1.f : 0.f;
    slope[rr] = slopes ? slopes[hh] : 0.f;
  }
  float o[NT][4];
#pragma unroll
  for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const uint32_t* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int rowp[2] = {HROWS ? pos0 : pos0 + g, HROWS ? pos0 : pos0 + g + 8};   // positions of this lane's two rows
  // Token rows: 64-aligned tiles of positions, [0, kept_end) holds the kept tokens outside the window and
  // [win_begin, pos_last] the window.  Head rows: tiles of the one token's visible keys, this block's run of them.
  const int win_begin = (key_lo / WKT) * WKT;
  const int kept_end = min(win_begin, ((min(max(keep_first, 0), key_lo) + WKT - 1) / WKT) * WKT);
  const Visible vis(pos0, window, keep_first, chunk);
  const int ntiles = (vis.count + WKT - 1) / WKT, per = (ntiles + nsplit - 1) / nsplit;
  const int t_first = HROWS ? static_cast<int>(blockIdx.z) * per * WKT : 0;
  const int t_end = HROWS ? min(vis.count, t_first + per * WKT) : pos_last + 1;       // exclusive
  for (int j0 = t_first; j0 < t_end; j0 += WKT) {
    if (!HROWS && j0 >= kept_end && j0 < win_begin) j0 = win_begin;
    __syncthreads();
    const int kvec = dim / 8, vvec = vdim / 8;
    // key j of tile row k (head rows: the k-th visible key of the run); rows past the run are zero
    auto tile_key = [&](int k) { return HROWS ? vis.key(min(j0 + k, t_end - 1)) : j0 + k; };
    for (int e = threadIdx.x; e < maps * WKT * kvec; e += blockDim.x) {
      const int mp = e / (WKT * kvec), k = (e / kvec) % WKT, d = (e % kvec) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j0 + k < t_end) {
        const int j = tile_key(k);
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        v = *reinterpret_cast<const uint4*>(k_cache + (slot * kv_heads + (HROWS ? mp * v_heads + kvh : kvh)) * dim + d);
      }
      *reinterpret_cast<uint4*>(Ks + (static_cast<size_t>(mp) * WKT + k) * P + d) = v;
    }
    for (int e = threadIdx.x; e < WKT * vvec; e += blockDim.x) {
      const int k = e / vvec, d = (e % vvec) * 8;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j0 + k < t_end) {
        const int j = tile_key(k);
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        v = *reinterpret_cast<const uint4*>(v_cache + (slot * v_heads + vh) * vdim + d);
      }
      *reinterpret_cast<uint4*>(Vs + static_cast<size_t>(k) * PV + d) = v;
    }
    __syncthreads();
    // scores of keys [16 warp, 16 warp + 16): every map's keys against all rows, each row keeps its own map's
    for (int mp = 0; mp < maps; ++mp) {
      const __nv_bfloat16* Km = Ks + static_cast<size_t>(mp) * WKT * P;
      float sc[2][4] = {};
      for (int kk = 0; kk < dim; kk += 16) {
        uint32_t a[4];
        a[0] = *reinterpret_cast<const uint32_t*>(Qs + g * P + kk + 2 * tq);
        a[1] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * P + kk + 2 * tq);
        a[2] = *reinterpret_cast<const uint32_t*>(Qs + g * P + kk + 2 * tq + 8);
        a[3] = *reinterpret_cast<const uint32_t*>(Qs + (g + 8) * P + kk + 2 * tq + 8);
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          const __nv_bfloat16* kr = Km + static_cast<size_t>(warp * 16 + nb * 8 + g) * P + kk + 2 * tq;
          wmma_bf16_16816(sc[nb], a, *reinterpret_cast<const uint32_t*>(kr), *reinterpret_cast<const uint32_t*>(kr + 8));
        }
      }
#pragma unroll
      for (int nb = 0; nb < 2; ++nb)
#pragma unroll
        for (int f = 0; f < 4; ++f) {
          const int r = g + (f >> 1) * 8, kcol = warp * 16 + nb * 8 + 2 * tq + (f & 1);
          if (maps == 1 || r / nh == mp) Ss[r * (WKT + 1) + kcol] = cap_score(sc[nb][f] * scale, softcap);
        }
    }
    __syncthreads();
    // the same online softmax in every warp; this lane's P entries are exactly its A fragments
    float p[2][16];
    float mx[2] = {-1e30f, -1e30f};
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int r = g + rr * 8;
      const int lo = first_visible(rowp[rr], window, chunk);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int kcol = ks * 16 + 2 * tq + (c & 1) + (c >> 1) * 8, j = j0 + kcol;
          const bool ok = HROWS ? (r < nrows && j < t_end) : (r < nrows && j <= rowp[rr] && (j >= lo || j < keep_first));
          const int jpos = HROWS ? vis.key(min(j, t_end - 1)) : j;         // the key's position
          const float v = ok ? Ss[r * (WKT + 1) + kcol] - slope[rr] * static_cast<float>(rowp[rr] - jpos) : -1e30f;
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
    // O += P V over this warp's value columns [warp * NT * 8, +NT * 8)
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a[4];
      a[0] = wpack_bf16(p[0][ks * 4 + 0], p[0][ks * 4 + 1]);
      a[1] = wpack_bf16(p[1][ks * 4 + 0], p[1][ks * 4 + 1]);
      a[2] = wpack_bf16(p[0][ks * 4 + 2], p[0][ks * 4 + 3]);
      a[3] = wpack_bf16(p[1][ks * 4 + 2], p[1][ks * 4 + 3]);
#pragma unroll
      for (int n = 0; n < NT; n += 2) {
        // four 8 x 8 blocks: (keys 0-7 | 8-15 of the step) x (columns d0 .. d0+7 | d0+8 .. d0+15), transposed on load
        const int d0 = (warp * NT + n) * 8;
        const __nv_bfloat16* src = Vs + static_cast<size_t>(ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PV + d0 + (lane >> 4) * 8;
        uint32_t r0, r1, r2, r3;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(src));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
        wmma_bf16_16816(o[n], a, r0, r1);
        if (n + 1 < NT) wmma_bf16_16816(o[n + 1], a, r2, r3);
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    const int r = g + rr * 8;
    if (r >= nrows) continue;
    const int hh = HROWS ? head_of(r) : h;
    const size_t trow = HROWS ? row0 : row0 + r;
    const size_t orow = trow * heads + hh;
    if (nsplit == 1) {
      float inv = l[rr] > 0.f ? 1.f / l[rr] : 0.f;
      if (gate && !gate_elems) inv *= sigmoid_f(gate[trow * ld_gate + hh]);
      const float* ge = (gate && gate_elems) ? gate + trow * ld_gate + static_cast<size_t>(hh) * vdim : nullptr;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int d = (warp * NT + n) * 8 + 2 * tq;
        const float g0 = ge ? sigmoid_f(ge[d]) : 1.f, g1 = ge ? sigmoid_f(ge[d + 1]) : 1.f;
        if (out_f32) {
          *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + orow * vdim + d) =
              make_float2(o[n][rr * 2] * inv * g0, o[n][rr * 2 + 1] * inv * g1);
        } else {
          __nv_bfloat162 v = __floats2bfloat162_rn(o[n][rr * 2] * inv * g0, o[n][rr * 2 + 1] * inv * g1);
          *reinterpret_cast<__nv_bfloat162*>(out + orow * vdim + d) = v;
        }
      }
    } else {
      const size_t pi = orow * nsplit + blockIdx.z;
#pragma unroll
      for (int n = 0; n < NT; ++n) {
        const int d = (warp * NT + n) * 8 + 2 * tq;
        part_o[pi * vdim + d] = o[n][rr * 2];
        part_o[pi * vdim + d + 1] = o[n][rr * 2 + 1];
      }
      if (warp == 0 && tq == 0) {
        part_ml[pi * 2] = m[rr];
        part_ml[pi * 2 + 1] = l[rr];
      }
    }
  }
}


// ---- token rows, second form (value sizes up to 128): block = 4 warps = one query head x 64 consecutive token rows of
// ONE sequence, every warp owning 16 rows outright.  A warp computes the scores of its rows against all 64 keys of a
// tile (8 n-tiles of fp32 accumulators, K fragments by ldmatrix), runs the fp32 online softmax on them in registers --
// the score accumulators ARE the A fragments of P, so nothing passes through shared memory and no warp repeats
// another's exponentials -- and multiplies P (bf16) with all value columns (V fragments by ldmatrix.trans).  The K / V
// tile in shared memory serves four times as many rows as in the form above.  Tiles as there: 64-aligned runs of
// positions, first those that hold kept tokens outside the window, then the window of the block's rows.
constexpr int RQ = 64;
template <int NTV>                   // n-tiles of 8 value columns = vdim / 8
__global__ void __launch_bounds__(128)
window_attn_rows_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ q,
                        const __nv_bfloat16* __restrict__ k_cache, const __nv_bfloat16* __restrict__ v_cache,
                        const float* __restrict__ sink, const float* __restrict__ gate, int ld_gate,
                        const uint32_t* __restrict__ cu, const uint32_t* __restrict__ ctx,
                        const uint32_t* __restrict__ block_tables, int max_blocks, int num_seqs, int heads, int kv_heads,
                        int dim, int vdim, int window, int keep_first, float scale, float softcap,
                        const float* __restrict__ slopes, int gate_elems, int chunk, int v_heads, int out_f32) {
  extern __shared__ __align__(16) unsigned char smraw[];
  const int P = dim + 8, PV = vdim + 8;
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);              // [WKT][P]
  __nv_bfloat16* Vs = Ks + static_cast<size_t>(WKT) * P;                    // [WKT][PV]
  __nv_bfloat16* Qs = Vs + static_cast<size_t>(WKT) * PV;                   // [RQ][P]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  int b = -1, row0 = 0, nrows = 0;
  {
    int acc = 0;
    for (int s = 0; s < num_seqs; ++s) {
      const int n = static_cast<int>(cu[s + 1] - cu[s]), tiles = (n + RQ - 1) / RQ;
      if (static_cast<int>(blockIdx.x) < acc + tiles) {
        const int k = blockIdx.x - acc;
        b = s;
        row0 = cu[s] + k * RQ;
        nrows = min(RQ, n - k * RQ);
        break;
      }
      acc += tiles;
    }
    if (b < 0) return;
  }
  const int h = blockIdx.y, kvh = h / (heads / kv_heads), vh = kvh % v_heads;
  const float slope = slopes ? slopes[h] : 0.f;
  const int pos0 = static_cast<int>(ctx[b]) - static_cast<int>(cu[b + 1] - cu[b]) + (row0 - static_cast<int>(cu[b]));
  const int pos_last = pos0 + nrows - 1;
  const int key_lo = first_visible(pos0, window, chunk);
  for (int e = threadIdx.x; e < RQ * dim; e += blockDim.x) {
    const int r = e / dim, d = e % dim;
    const float v = r < nrows ? q[(static_cast<size_t>(row0 + r) * heads + h) * dim + d] : 0.f;
    Qs[r * P + d] = __float2bfloat16_rn(v);
  }
  const int wr = warp * 16;                                // this warp's first row within the block
  const int rowi[2] = {wr + g, wr + g + 8};
  const int rowp[2] = {pos0 + rowi[0], pos0 + rowi[1]};
  float m[2], l[2];
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    m[rr] = sink ? sink[h] : -1e30f;
    l[rr] = sink ? 1.f : 0.f;
  }
  float o[NTV][4];
#pragma unroll
  for (int n = 0; n < NTV; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  const uint32_t* bt = block_tables + static_cast<size_t>(b) * max_blocks;
  const int win_begin = (key_lo / WKT) * WKT;
  const int kept_end = min(win_begin, ((min(max(keep_first, 0), key_lo) + WKT - 1) / WKT) * WKT);
  const int kvec = dim / 8, vvec = vdim / 8;
  for (int j0 = 0; j0 <= pos_last; j0 += WKT) {
    if (j0 >= kept_end && j0 < win_begin) j0 = win_begin;
    __syncthreads();
    for (int e = threadIdx.x; e < WKT * kvec; e += blockDim.x) {
      const int k = e / kvec, d = (e % kvec) * 8, j = j0 + k;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j <= pos_last) {
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        v = *reinterpret_cast<const uint4*>(k_cache + (slot * kv_heads + kvh) * dim + d);
      }
      *reinterpret_cast<uint4*>(Ks + static_cast<size_t>(k) * P + d) = v;
    }
    for (int e = threadIdx.x; e < WKT * vvec; e += blockDim.x) {
      const int k = e / vvec, d = (e % vvec) * 8, j = j0 + k;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (j <= pos_last) {
        const size_t slot = static_cast<size_t>(bt[j / kPage]) * kPage + (j % kPage);
        v = *reinterpret_cast<const uint4*>(v_cache + (slot * v_heads + vh) * vdim + d);
      }
      *reinterpret_cast<uint4*>(Vs + static_cast<size_t>(k) * PV + d) = v;
    }
    __syncthreads();
    // this warp's rows see nothing of the tile: every key is later than its last row, or the tile lies wholly between
    // the kept tokens and the window of its first row
    const int w_first = pos0 + wr, w_last = min(pos0 + wr + 15, pos_last);
    const int w_lo = first_visible(w_first, window, chunk);
    if (wr >= nrows || j0 > w_last || (j0 + WKT <= w_lo && j0 >= keep_first)) continue;
    float sc[8][4];
#pragma unroll
    for (int n = 0; n < 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
    for (int kk = 0; kk < dim; kk += 16) {
      uint32_t a[4];
      a[0] = *reinterpret_cast<const uint32_t*>(Qs + rowi[0] * P + kk + 2 * tq);
      a[1] = *reinterpret_cast<const uint32_t*>(Qs + rowi[1] * P + kk + 2 * tq);
      a[2] = *reinterpret_cast<const uint32_t*>(Qs + rowi[0] * P + kk + 2 * tq + 8);
      a[3] = *reinterpret_cast<const uint32_t*>(Qs + rowi[1] * P + kk + 2 * tq + 8);
#pragma unroll
      for (int np = 0; np < 4; ++np) {        // n-tiles 2 np, 2 np + 1: matrices (tile, k half) = lane >> 3
        const int mi = lane >> 3;
        const __nv_bfloat16* src = Ks + static_cast<size_t>((2 * np + (mi >> 1)) * 8 + (lane & 7)) * P + kk + (mi & 1) * 8;
        uint32_t r0, r1, r2, r3;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(src));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
        wmma_bf16_16816(sc[2 * np], a, r0, r1);
        wmma_bf16_16816(sc[2 * np + 1], a, r2, r3);
      }
    }
    // scale, cap, mask; row maxima over the lane's entries and the quad
    float mx[2] = {-1e30f, -1e30f};
#pragma unroll
    for (int rr = 0; rr < 2; ++rr) {
      const int lo = first_visible(rowp[rr], window, chunk);
#pragma unroll
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int j = j0 + n * 8 + 2 * tq + c;
          const bool ok = rowi[rr] < nrows && j <= rowp[rr] && (j >= lo || j < keep_first);
          const float v = ok ? cap_score(sc[n][rr * 2 + c] * scale, softcap) - slope * static_cast<float>(rowp[rr] - j)
                             : -1e30f;
          sc[n][rr * 2 + c] = v;
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
      for (int n = 0; n < 8; ++n)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const float v = sc[n][rr * 2 + c];
          const float e = v > -1e29f ? expf(v - mn) : 0.f;
          sc[n][rr * 2 + c] = e;
          sum += e;
        }
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      l[rr] = l[rr] * alpha[rr] + sum;
      m[rr] = mn;
    }
#pragma unroll
    for (int n = 0; n < NTV; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }
    // O += P V: per 16 keys the A fragments are two neighbouring score tiles
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      uint32_t a[4];
      a[0] = wpack_bf16(sc[2 * ks][0], sc[2 * ks][1]);
      a[1] = wpack_bf16(sc[2 * ks][2], sc[2 * ks][3]);
      a[2] = wpack_bf16(sc[2 * ks + 1][0], sc[2 * ks + 1][1]);
      a[3] = wpack_bf16(sc[2 * ks + 1][2], sc[2 * ks + 1][3]);
#pragma unroll
      for (int n = 0; n < NTV; n += 2) {
        const __nv_bfloat16* src = Vs + static_cast<size_t>(ks * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * PV + n * 8 + (lane >> 4) * 8;
        uint32_t r0, r1, r2, r3;
        const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(src));
        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                     : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
        wmma_bf16_16816(o[n], a, r0, r1);
        wmma_bf16_16816(o[n + 1], a, r2, r3);
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < 2; ++rr) {
    if (rowi[rr] >= nrows) continue;
    const size_t trow = static_cast<size_t>(row0 + rowi[rr]);
    float inv = l[rr] > 0.f ? 1.f / l[rr] : 0.f;
    if (gate && !gate_elems) inv *= sigmoid_f(gate[trow * ld_gate + h]);
    const float* ge = (gate && gate_elems) ? gate + trow * ld_gate + static_cast<size_t>(h) * vdim : nullptr;
#pragma unroll
    for (int n = 0; n < NTV; ++n) {
      const int d = n * 8 + 2 * tq;
      const float g0 = ge ? sigmoid_f(ge[d]) : 1.f, g1 = ge ? sigmoid_f(ge[d + 1]) : 1.f;
      if (out_f32) {
        *reinterpret_cast<float2*>(reinterpret_cast<float*>(out) + (trow * heads + h) * vdim + d) =
            make_float2(o[n][rr * 2] * inv * g0, o[n][rr * 2 + 1] * inv * g1);
      } else {
        __nv_bfloat162 v = __floats2bfloat162_rn(o[n][rr * 2] * inv * g0, o[n][rr * 2 + 1] * inv * g1);
        *reinterpret_cast<__nv_bfloat162*>(out + (trow * heads + h) * vdim + d) = v;
      }
    }
  }
}

static bool window_mma_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_WINDOW_MMA");       // 0: the FMA kernel for every step (A/B arm)
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
static bool window_rows_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_WINDOW_ROWS");      // 0: token rows take the 16-row form (A/B arm)
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}
// maps: score maps whose K tiles a block stages (heads-as-rows form with several maps over one set of values)
static size_t window_mma_smem(int dim, int vdim, int maps = 1) {
  return static_cast<size_t>(maps * WKT + WQ) * (dim + 8) * 2 + static_cast<size_t>(WKT) * (vdim + 8) * 2 +
         static_cast<size_t>(WQ) * (WKT + 1) * 4;
}
static bool window_mma_shape_ok(int dim, int vdim, int maps = 1) {
  return dim % 16 == 0 && vdim % 32 == 0 && vdim <= 256 && maps <= WQ && window_mma_smem(dim, vdim, maps) <= 200 * 1024;
}
// blocks per token of the heads-as-rows form: a value head's group takes ceil(per_group / hpg) blocks
static int window_mma_row_blocks(int heads, int kv_heads, int v_heads) {
  const int maps = std::max(1, kv_heads / v_heads), per_group = heads / kv_heads;
  const int hpg = std::max(1, std::min(per_group, WQ / std::min(maps, WQ)));
  return v_heads * ((per_group + hpg - 1) / hpg);
}

static int window_attn_warps(int heads, int kv_heads) {
  const int pg = heads / kv_heads;
  return pg >= 8 ? 8 : (pg >= 4 ? 4 : (pg >= 2 ? 2 : 1));
}
int window_attn_splits(int T, int heads, int kv_heads, int window, int keep_first) {
  (void)heads;
  const int blocks = T * kv_heads;
  int n = (2 * sm_count() + blocks - 1) / blocks;           // aim at two blocks per SM
  if (window > 0) n = std::min(n, (window + std::max(keep_first, 0) + 31) / 32);
  return std::max(1, std::min(n, 16));
}
// key splits of the heads-as-rows tensor-core form: four blocks per SM, at most one split per key tile, at most 16
static int window_attn_mma_splits(int T, int heads, int kv_heads, int window, int keep_first, int v_heads) {
  const int blocks = T * window_mma_row_blocks(heads, kv_heads, v_heads);
  int n = (4 * sm_count() + blocks - 1) / blocks;
  if (window > 0) n = std::min(n, (window + std::max(keep_first, 0) + WKT - 1) / WKT);
  return std::max(1, std::min(n, 16));
}
size_t window_attn_workspace_bytes(int T, int heads, int kv_heads, int vdim, int window, int keep_first, int v_heads) {
  if (v_heads <= 0 || kv_heads % v_heads != 0) v_heads = kv_heads;
  const int n = std::max(window_attn_splits(T, heads, kv_heads, window, keep_first),
                         window_attn_mma_splits(T, heads, kv_heads, window, keep_first, v_heads));
  return n == 1 ? 0 : static_cast<size_t>(T) * heads * n * (vdim + 2) * 4;
}

void launch_window_attn(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                        const float* gate, int ld_gate, const uint32_t* cu, const uint32_t* ctx,
                        const uint32_t* block_tables, int max_blocks, int num_seqs, int T, int heads, int kv_heads,
                        int dim, int vdim, int window, int keep_first, float scale, float softcap, int dt,
                        void* workspace, const b200_attn_options* opt, cudaStream_t st_) {
  if (T <= 0) return;
  const float* slopes = opt ? opt->dist_slopes : nullptr;
  const int gate_elems = opt ? opt->gate_elems : 0;
  const int chunk = opt ? opt->chunk : 0, out_f32 = opt ? opt->out_f32 : 0;
  const int v_heads = (opt && opt->v_heads > 0) ? opt->v_heads : kv_heads;
  if (kv_heads % v_heads != 0) {
    set_error(1, "window_attn: kv_heads is a multiple of v_heads");
    return;
  }
  // bf16, steps of many rows, value sizes up to 128: the tensor-core form with 64 token rows per block
  if (!dt && window_mma_enabled() && T > 2 * sm_count() / 4 && window_rows_enabled() && dim % 16 == 0 && vdim % 16 == 0 &&
      vdim <= 128) {
    const size_t smem = (static_cast<size_t>(WKT + RQ) * (dim + 8) + static_cast<size_t>(WKT) * (vdim + 8)) * 2;
    const dim3 grid((T + RQ - 1) / RQ + num_seqs, heads, 1);
#define B200_WROWS(NTV)                                                                                           \
  {                                                                                                                \
    auto kern = window_attn_rows_kernel<NTV>;                                                                      \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));               \
    kern<<<grid, 128, smem, st_>>>((__nv_bfloat16*)out, q, (const __nv_bfloat16*)k_cache,                          \
                                   (const __nv_bfloat16*)v_cache, sink, gate, ld_gate, cu, ctx, block_tables,      \
                                   max_blocks, num_seqs, heads, kv_heads, dim, vdim, window, keep_first, scale,    \
                                   softcap, slopes, gate_elems, chunk, v_heads, out_f32);                          \
  }
    bool done = smem <= 200 * 1024;
    if (done) switch (vdim / 8) {
      case 2: B200_WROWS(2) break;
      case 4: B200_WROWS(4) break;
      case 6: B200_WROWS(6) break;
      case 8: B200_WROWS(8) break;
      case 10: B200_WROWS(10) break;
      case 12: B200_WROWS(12) break;
      case 14: B200_WROWS(14) break;
      case 16: B200_WROWS(16) break;
      default: done = false;
    }
#undef B200_WROWS
    if (done) {
      B200_CUDA_LAUNCH_CHECK();
      return;
    }
  }
  // bf16: the tensor-core kernel; steps of few rows take its heads-as-rows form with the keys split over blocks
  const bool hrows = T <= 2 * sm_count() / 4;
  if (!dt && window_mma_enabled() && window_mma_shape_ok(dim, vdim, hrows ? kv_heads / v_heads : 1)) {
    const size_t smem = window_mma_smem(dim, vdim, hrows ? kv_heads / v_heads : 1);
    const int nsplit = hrows && workspace ? window_attn_mma_splits(T, heads, kv_heads, window, keep_first, v_heads) : 1;
    float* part_o = reinterpret_cast<float*>(workspace);
    float* part_ml = part_o ? part_o + static_cast<size_t>(T) * heads * nsplit * vdim : nullptr;
    const dim3 grid = hrows ? dim3(T, window_mma_row_blocks(heads, kv_heads, v_heads), nsplit)
                            : dim3((T + WQ - 1) / WQ + num_seqs, heads, 1);
#define B200_WMMA2(NT, HR)                                                                                        \
  {                                                                                                                \
    auto kern = window_attn_mma_kernel<NT, HR>;                                                                    \
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));               \
    kern<<<grid, 128, smem, st_>>>((__nv_bfloat16*)out, q, (const __nv_bfloat16*)k_cache,                          \
                                   (const __nv_bfloat16*)v_cache, sink, gate, ld_gate, cu, ctx, block_tables,      \
                                   max_blocks, num_seqs, heads, kv_heads, dim, vdim, window, keep_first, scale,    \
                                   softcap, nsplit, part_o, part_ml, slopes, gate_elems, chunk, v_heads, out_f32); \
  }
#define B200_WMMA(NT)                 \
  if (hrows) B200_WMMA2(NT, true)     \
  else B200_WMMA2(NT, false)
    bool done = true;
    switch (vdim / 32) {
      case 1: B200_WMMA(1) break;
      case 2: B200_WMMA(2) break;
      case 3: B200_WMMA(3) break;
      case 4: B200_WMMA(4) break;
      case 6: B200_WMMA(6) break;
      case 8: B200_WMMA(8) break;
      default: done = false;
    }
#undef B200_WMMA
#undef B200_WMMA2
    if (done) {
      B200_CUDA_LAUNCH_CHECK();
      if (nsplit > 1) {
        const int th = vdim >= 256 ? 256 : (vdim >= 128 ? 128 : 64);
        window_attn_merge_kernel<__nv_bfloat16><<<T * heads, th, 0, st_>>>((__nv_bfloat16*)out, part_o, part_ml, sink,
                                                                           gate, ld_gate, heads, vdim, nsplit, gate_elems,
                                                                           out_f32);
        B200_CUDA_LAUNCH_CHECK();
      }
      return;
    }
  }
  const int Dp = dim | 1;
  const int nw = window_attn_warps(heads, kv_heads);
  int key_tile = 32;
  auto bytes = [&](int kt) {
    return (static_cast<size_t>(kt) * (Dp + vdim) + static_cast<size_t>(nw) * (dim + vdim)) * 4;
  };
  while (key_tile > 1 && bytes(key_tile) > 200 * 1024) key_tile >>= 1;
  const size_t smem = bytes(key_tile);
  if (smem > 220 * 1024) {
    set_error(1, "window_attn: dim + vdim too large for the shared-memory tile");
    return;
  }
  // few token rows (decoding): the keys of a row are split over several blocks and merged afterwards
  const int nsplit = workspace ? window_attn_splits(T, heads, kv_heads, window, keep_first) : 1;
  float* part_o = reinterpret_cast<float*>(workspace);
  float* part_ml = part_o ? part_o + static_cast<size_t>(T) * heads * nsplit * vdim : nullptr;
  const dim3 grid(T, kv_heads, nsplit);
  if (dt) {
    auto kern = window_attn_kernel<float>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, nw * 32, smem, st_>>>((float*)out, q, (const float*)k_cache, (const float*)v_cache, sink, gate, ld_gate,
                                       cu, ctx, block_tables, max_blocks, num_seqs, heads, kv_heads, dim, vdim, window,
                                       keep_first, scale, softcap, key_tile, nsplit, part_o, part_ml, slopes, gate_elems,
                                       chunk, v_heads, out_f32);
  } else {
    auto kern = window_attn_kernel<__nv_bfloat16>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<grid, nw * 32, smem, st_>>>((__nv_bfloat16*)out, q, (const __nv_bfloat16*)k_cache,
                                       (const __nv_bfloat16*)v_cache, sink, gate, ld_gate, cu, ctx, block_tables,
                                       max_blocks, num_seqs, heads, kv_heads, dim, vdim, window, keep_first, scale,
                                       softcap, key_tile, nsplit, part_o, part_ml, slopes, gate_elems, chunk, v_heads,
                                       out_f32);
  }
  B200_CUDA_LAUNCH_CHECK();
  if (nsplit > 1) {
    const int th = vdim >= 256 ? 256 : (vdim >= 128 ? 128 : 64);
    if (dt)
      window_attn_merge_kernel<float><<<T * heads, th, 0, st_>>>((float*)out, part_o, part_ml, sink, gate, ld_gate,
                                                                 heads, vdim, nsplit, gate_elems, out_f32);
    else
      window_attn_merge_kernel<__nv_bfloat16><<<T * heads, th, 0, st_>>>((__nv_bfloat16*)out, part_o, part_ml, sink,
                                                                         gate, ld_gate, heads, vdim, nsplit, gate_elems,
                                                                         out_f32);
    B200_CUDA_LAUNCH_CHECK();
  }
}

// One block per token, a warp per head at a time: what follows the softmax-weighted sums where more than a gate does.
//   o = a[map 0] - lambda * a[map 1]                (maps == 2; the maps lie one after the other: a [T, maps, heads, vdim])
//   o turned back by -position * v_rot_freq[m]      (rotated values; cos / sin of the token's angles in shared memory,
//                                                    angles in double as where the values were turned)
//   o / sqrt(mean(o^2) + eps) per head, no weight   (head_norm)
//   o * out_scale * sigmoid(gate)                   (gate per head or per element)
template <typename T>
__global__ void attn_finish_kernel(T* __restrict__ out, const float* __restrict__ a, const float* __restrict__ gate,
                                   int ld_gate, int gate_elems, const int64_t* __restrict__ positions,
                                   const double* __restrict__ v_rot_freq, int rot_half, int maps, float lambda,
                                   int head_norm, float eps, float out_scale, int heads, int vdim) {
  extern __shared__ float sm[];          // cos[vdim/2] | sin[vdim/2]
  const int vhalf = vdim / 2;
  float* cs = sm;
  float* sn = sm + vhalf;
  const int t = blockIdx.x, nw = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (v_rot_freq) {
    const double pos = static_cast<double>(positions[t]);
    for (int i = threadIdx.x; i < vhalf; i += blockDim.x) {
      double s, c;
      sincos(pos * v_rot_freq[i], &s, &c);
      cs[i] = static_cast<float>(c);
      sn[i] = static_cast<float>(s);
    }
    __syncthreads();
  }
  const size_t map_stride = static_cast<size_t>(heads) * vdim;
  for (int h = warp; h < heads; h += nw) {
    const float* a0 = a + (static_cast<size_t>(t) * maps * heads + h) * vdim;
    auto val = [&](int d) { return maps == 2 ? a0[d] - lambda * a0[map_stride + d] : a0[d]; };
    float inv = out_scale;
    if (head_norm) {
      float ss = 0.f;
      for (int d = lane; d < vdim; d += 32) ss += val(d) * val(d);
      ss = lanes_sum(ss);
      inv *= 1.f / sqrtf(ss / static_cast<float>(vdim) + eps);
    }
    if (gate && !gate_elems) inv *= sigmoid_f(gate[static_cast<size_t>(t) * ld_gate + h]);
    const float* ge = (gate && gate_elems) ? gate + static_cast<size_t>(t) * ld_gate + static_cast<size_t>(h) * vdim : nullptr;
    T* o = out + (static_cast<size_t>(t) * heads + h) * vdim;
    for (int d = lane; d < vdim; d += 32) {
      float v = val(d);
      if (v_rot_freq) {                  // the inverse turn: (u, w) -> (u cos + w sin, w cos - u sin)
        const bool second = rot_half ? d >= vhalf : (d & 1) != 0;
        const int i = rot_half ? (second ? d - vhalf : d) : d >> 1;
        const float other = val(second ? (rot_half ? d - vhalf : d - 1) : (rot_half ? d + vhalf : d + 1));
        v = second ? v * cs[i] - other * sn[i] : v * cs[i] + other * sn[i];
      }
      st(o + d, v * inv * (ge ? sigmoid_f(ge[d]) : 1.f));
    }
  }
}

void launch_attn_finish(void* out, const float* a, const float* gate, int ld_gate, int gate_elems,
                        const int64_t* positions, const double* v_rot_freq, int rot_half, int maps, float lambda,
                        int head_norm, float eps, float out_scale, int T, int heads, int vdim, int dt, cudaStream_t st_) {
  if (T <= 0) return;
  if (maps < 1 || maps > 2 || (v_rot_freq && (vdim % 2 != 0 || !positions))) {
    set_error(1, "attn_finish: one or two score maps; turning values back needs an even vdim and the positions");
    return;
  }
  const int threads = heads >= 8 ? 256 : (heads >= 4 ? 128 : 64);
  const size_t smem = static_cast<size_t>(vdim + 2) * 4;
  if (dt)
    attn_finish_kernel<float><<<T, threads, smem, st_>>>((float*)out, a, gate, ld_gate, gate_elems, positions, v_rot_freq,
                                                         rot_half, maps, lambda, head_norm, eps, out_scale, heads, vdim);
  else
    attn_finish_kernel<__nv_bfloat16><<<T, threads, smem, st_>>>((__nv_bfloat16*)out, a, gate, ld_gate, gate_elems, positions,
                                                                 v_rot_freq, rot_half, maps, lambda, head_norm, eps,
                                                                 out_scale, heads, vdim);
  B200_CUDA_LAUNCH_CHECK();
}

}  // namespace b200

extern "C" {
void b200_attn_finish(void* out, const float* a, const float* gate, int32_t ld_gate, int32_t gate_elems,
                      const int64_t* positions, const double* v_rot_freq, int32_t rot_half, int32_t maps, float lambda,
                      int32_t head_norm, float eps, float out_scale, int32_t num_tokens, int32_t heads, int32_t vdim,
                      int32_t dt, int64_t stream) {
  B200_CHECK_ARG(out && a && heads > 0 && vdim > 0 && (dt == 0 || dt == 1), "attn_finish: bad arguments");
  b200::launch_attn_finish(out, a, gate, ld_gate, gate_elems, positions, v_rot_freq, rot_half, maps, lambda, head_norm,
                           eps, out_scale, num_tokens, heads, vdim, dt, reinterpret_cast<cudaStream_t>(stream));
}
void b200_window_attn_prep_ex(const float* proj, int32_t ld, const float* bias, const float* q_norm_w,
                              const float* k_norm_w, const double* rot_freq, const int64_t* positions,
                              const int64_t* slot_mapping, float* q_out, void* k_cache, void* v_cache,
                              int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                              int32_t rot_dims, float eps, int32_t dt, const b200_attn_options* opt, int64_t stream) {
  B200_CHECK_ARG(proj && positions && slot_mapping && q_out && ((k_cache && v_cache) || (opt && opt->no_cache)) && heads > 0 && kv_heads > 0 &&
                     heads % kv_heads == 0 && dim > 0 && vdim > 0 && rot_dims >= 0 && rot_dims <= dim &&
                     rot_dims % 2 == 0 && (rot_dims == 0 || rot_freq) && (dt == 0 || dt == 1),
                 "window_attn_prep: bad arguments");
  b200::launch_window_attn_prep(proj, ld, bias, q_norm_w, k_norm_w, rot_freq, positions, slot_mapping, q_out, k_cache,
                                v_cache, num_tokens, heads, kv_heads, dim, vdim, rot_dims, eps, dt, opt,
                                reinterpret_cast<cudaStream_t>(stream));
}
void b200_window_attn_prep(const float* proj, int32_t ld, const float* bias, const float* q_norm_w,
                           const float* k_norm_w, const double* rot_freq, const int64_t* positions,
                           const int64_t* slot_mapping, float* q_out, void* k_cache, void* v_cache, int32_t num_tokens,
                           int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t rot_dims, float eps,
                           int32_t dt, int64_t stream) {
  b200_window_attn_prep_ex(proj, ld, bias, q_norm_w, k_norm_w, rot_freq, positions, slot_mapping, q_out, k_cache, v_cache,
                           num_tokens, heads, kv_heads, dim, vdim, rot_dims, eps, dt, nullptr, stream);
}
void b200_window_attn_ex(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                         const float* gate, int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                         const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens,
                         int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t window, int32_t keep_first,
                         float scale, float softcap, int32_t dt, void* workspace, const b200_attn_options* opt,
                         int64_t stream) {
  B200_CHECK_ARG(out && q && k_cache && v_cache && cu_seqlens_q && context_lens && block_tables && num_seqs > 0 &&
                     heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && (dt == 0 || dt == 1),
                 "window_attn: bad arguments");
  b200::launch_window_attn(out, q, k_cache, v_cache, sink, gate, ld_gate, cu_seqlens_q, context_lens, block_tables,
                           max_blocks_per_seq, num_seqs, num_tokens, heads, kv_heads, dim, vdim, window, keep_first,
                           scale, softcap, dt, workspace, opt, reinterpret_cast<cudaStream_t>(stream));
}
void b200_window_attn(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                      const float* gate, int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                      const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens,
                      int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t window, int32_t keep_first,
                      float scale, float softcap, int32_t dt, void* workspace, int64_t stream) {
  b200_window_attn_ex(out, q, k_cache, v_cache, sink, gate, ld_gate, cu_seqlens_q, context_lens, block_tables,
                      max_blocks_per_seq, num_seqs, num_tokens, heads, kv_heads, dim, vdim, window, keep_first, scale,
                      softcap, dt, workspace, nullptr, stream);
}
int64_t b200_window_attn_workspace_bytes(int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t vdim,
                                         int32_t window, int32_t keep_first) {
  return static_cast<int64_t>(b200::window_attn_workspace_bytes(num_tokens, heads, kv_heads, vdim, window, keep_first, 0));
}
int64_t b200_window_attn_workspace_bytes_ex(int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t v_heads,
                                            int32_t vdim, int32_t window, int32_t keep_first) {
  return static_cast<int64_t>(b200::window_attn_workspace_bytes(num_tokens, heads, kv_heads, vdim, window, keep_first,
                                                                v_heads));
}
}
