// Step runner of hybrid decoders with an fp32 residual stream: every launch of one ragged step (prompt portions and
// decoded tokens in one batch) on one GPU.  Sibling of model_runner.cpp (the fp16 LLaMA / Qwen2 plan); like it, the
// runner owns no device memory: weights, the paged latent cache, the state pools and one workspace come from the caller.
//
// Layer plan (parallel layer: mixer and feed-forward read one norm h of the stream x, both add into x):
//   h = norm(x)                                                    resid_rmsnorm        (fp32 in, operand dtype out)
//   latent attention:  [q | latent | k_rot] = h W_in^T             library GEMM (fp32 out)
//                      norm + rotary + cache write + query split   latent_prep
//                      q_abs[h] = q_plain[h] W_uk[h]               batched library GEMM into q_full
//                      latent_attn (window, sink)                  -> attention-weighted latents
//                      v[h] = lat[h] W_uv[h]^T ; x += v W_o^T      batched GEMM, cast, GEMM with beta = 1
//   delta rule:        [q | k | v | b | a | gate] = h W_in^T ; short_conv_silu on q | k | v ; delta_rule ;
//                      gated_group_norm (gate after the norm) ; x += . W_o^T
//   SSD:               [z | x | B | C | dt] = h W_in^T ; short_conv_silu on x | B | C ; ssd_scan ;
//                      gated_group_norm (gate before the norm) ; x += . W_o^T
//   window attention:  [q | k | v | gate] = h W_in^T ; window_attn_prep (biases, whole-projection q / k norms, rotary,
//                      K / V cache write) ; window_attn (window + kept first tokens, capped scores, sink, gate) ;
//                      dst (+)= scale . W_o^T (+ bias)
//   decay attention:   [q | k | v | gate | low] = h W_in^T ; lowrank_decay (per-channel decays) ; decay_attn ;
//                      gated_group_norm ; dst (+)= scale . W_o^T
//   experts:           router GEMM (fp32 out) -> moe_route -> sort -> grouped gate|up (SiLU * mul) -> grouped down ->
//                      combine into x ; shared expert: GEMM, silu_mul, GEMM with beta = 1 into x
// The residual add of every branch is the beta = 1 accumulation of its last matrix product (or the combine kernel).
// Sandwich layer (a norm before AND after each sublayer): the mixers of the layer (one, or two side by side with their
// scales) write their sum into y, then x += post_norm(y) (resid_add_rmsnorm); the dense gated feed-forward reads
// ff_norm(x), writes y, and x += ff_post_norm(y).
// Post-norm layer (results are normed on their way into the stream, inputs are not): the sublayers take x rounded to the
// operand dtype (cast_rows; fp32 runs read x in place): y = mixers(x), x += post_norm(y); y = ff(x), x += ff_post_norm(y), the
// feed-forward being the routed experts (plus their shared expert) or the dense gated one.
// Pre-norm layer (each sublayer behind its own norm, added times a factor): h = norm(x) -- RMS or dynamic tanh, with the
// token shift h[t] += (h[t-1] - h[t]) * shift where the layer has one (stream_norm) --, x += out_scale * mixer(h);
// h = ff_norm(x), x += ff_scale * ff(h).  With depth weights the layers' results X_0 (embedding) .. X_L are kept side by
// side, layer i works in place on slot i + 1 (which starts as its input), and depth_mix writes
// sum_j depth_w[j] X_j into slot i + 2 (the stream for the last layer), which is the next layer's input.
//   window attention with rotated values, a chunked mask or two score maps: the attention writes fp32, attn_finish
//                      combines the maps (a_0 - lambda a_1), turns rotated values back, norms per head, scales, gates
//   delta rule, channel form: [q | k | v | b | low_a | low_g] = h W_in^T ; short_conv_silu ; lowrank_decay (kind 1)
//                      -> decays per head and key channel ; delta_rule ; gate logits = low_g W_g2^T (fp32 product) ;
//                      gated_group_norm (sigmoid gate) ; x += . W_o^T
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <map>
#include <tuple>
#include <vector>

#include "../../../include/b200_vllm.h"
#include "../seqmix.cuh"

using namespace b200;
namespace b200 {
long long launch_count();
void launch_sample_topk_topp(uint32_t* out_ids, const float* logits, int B, int V, int k, float p, float t,
                             const uint64_t* seed_dev, cudaStream_t st);
}

namespace {
inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
}

struct b200_hybrid {
  b200_hybrid_config cfg;
  std::vector<b200_hybrid_layer> layers;
  std::vector<b200_hybrid_layer> sides;      // side mixer of layer i (sides[i].heads == 0: none)
  const void *embed = nullptr, *final_norm = nullptr, *lm_head = nullptr;
  const void* final_norm_b = nullptr;        // dynamic-tanh final norm: bias and the scalar inside the tanh
  float final_norm_alpha = 1.f;
  float* hist = nullptr;       // [num_layers + 1, T, width] results of the embedding and of every layer (depth weights)
  float* x0 = nullptr;         // the stream buffer of models without depth weights (x points here)
  uint8_t* ws = nullptr;
  float* trace = nullptr;
  // workspace carve-up
  float* x = nullptr;          // [T, width] residual stream
  float* y = nullptr;          // [T, width] output of a sublayer before the norm that follows it (sandwich layers)
  void* h = nullptr;           // [T, width] normed stream, operand dtype
  const void* hin = nullptr;   // what the sublayers of the current layer read: h, or x itself (fp32 post-norm layers)
  float* proj = nullptr;       // [T, max fused input projection]
  float* conv = nullptr;       // [T, max convolved channels]: output of the short convolution
  float* aux = nullptr;        // [T, max(heads (kv_rank + rot_dim), heads vdim)] fp32: q_full / scan output / expanded values
  void* opa = nullptr;         // [T, max(heads dim, heads vdim, 2 shared... )] operand dtype: q_plain, then the o-projection input
  void* lat = nullptr;         // [T, heads kv_rank] operand dtype: attention-weighted latents
  void* attn_ws = nullptr;     // parts of split attention rows (steps of few token rows)
  size_t attn_ws_rows = 0;     // token rows the parts are sized for
  float* rlog = nullptr;       // [T, experts]
  int32_t* top_idx = nullptr;
  float* top_w = nullptr;
  void* moe_ws = nullptr;
  float* sh = nullptr;         // [T, 2 shared_ff] fp32
  void* sha = nullptr;         // [T, shared_ff] operand dtype
  void* hr = nullptr;          // [R, width] final norm of the rows whose logits are wanted (read from x through out_rows)
  float* logits = nullptr;     // [R, vocab]
  // device staging of the host entry point
  uint32_t *s_ids = nullptr, *s_cu = nullptr, *s_ctx = nullptr, *s_bt = nullptr, *s_rows = nullptr, *s_out = nullptr;
  int64_t *s_pos = nullptr, *s_slot = nullptr;
  int32_t* s_state = nullptr;
  uint64_t* s_seed = nullptr;
  int samp_k = 0;
  bool samp_all = false;
  float samp_p = 1.f, samp_t = 1.f;
  int64_t launches = 0;
  // CUDA graphs of small steps (decoding, short portions), keyed by the host-side sizes that are kernel arguments:
  // (sequences, token rows, block-table width, output rows, ids wanted).  A shape is captured the second time it is
  // seen (the first run warms up lazily created library state); the step's inputs live in the static staging buffers.
  struct GraphEntry {
    int seen = 0;
    cudaGraphExec_t exec = nullptr;
  };
  std::map<std::tuple<int, int, int, int, int>, GraphEntry> graphs;
  void drop_graphs() {
    for (auto& g : graphs)
      if (g.second.exec) cudaGraphExecDestroy(g.second.exec);
    graphs.clear();
  }
};

constexpr int kGraphMaxRows = 256;
static bool graphs_enabled() {
  static int v = -1;
  if (v < 0) {
    const char* e = getenv("B200_HYBRID_GRAPHS");      // 0: every step is launched directly (A/B arm)
    v = (e && e[0] == '0') ? 0 : 1;
  }
  return v == 1;
}

static int in_rows(const b200_hybrid_layer& l) {
  switch (l.mixer) {
    case B200_MIXER_LATENT_ATTN:
      return l.heads * (l.dim + l.rot_dim) + (l.shared_cache ? 0 : l.kv_rank + l.rot_dim) + (l.gated ? l.heads : 0);
    case B200_MIXER_DELTA_RULE:
      if (l.chan_rank > 0) return 2 * l.kv_heads * l.dim + l.heads * l.vdim + l.heads + l.chan_rank + l.gate_rank;
      return 2 * l.kv_heads * l.dim + 2 * l.heads * l.vdim + 2 * l.heads;
    case B200_MIXER_WINDOW_ATTN: {
      const int maps = l.score_maps > 1 ? l.score_maps : 1;
      return maps * l.heads * l.dim +
             (l.shared_cache ? 0 : maps * l.kv_heads * l.dim + (l.v_from_k ? 0 : l.kv_heads * l.vdim)) +
             (l.gated == 2 ? l.heads * l.vdim : (l.gated ? l.heads : 0));
    }
    case B200_MIXER_DECAY_ATTN: return 2 * l.heads * l.dim + 2 * l.heads * l.vdim + l.decay_rank;
    default: return 2 * l.heads * l.vdim + 2 * l.kv_heads * l.state + l.heads;
  }
}

// window attention whose softmax-weighted sums pass attn_finish (fp32 sums, then maps / turn back / norm / gate)
static bool needs_finish(const b200_hybrid_layer& l) {
  return l.mixer == B200_MIXER_WINDOW_ATTN && (l.score_maps > 1 || l.v_rot_freq != nullptr || l.diff_norm != 0);
}

static int64_t carve(b200_hybrid* r, uint8_t* base) {
  const b200_hybrid_config& c = r->cfg;
  const size_t T = c.max_tokens, es = c.dt ? 4 : 2;
  size_t conv_n = 1, proj_n = 1, aux_n = 1, opa_n = 1, lat_n = 1, E = 1, top = 1, sh_n = 1, moe_bytes = 256, attn_bytes = 0;
  // rows up to which a step may split its attention rows: beyond two blocks per SM a split is never chosen
  r->attn_ws_rows = std::min<size_t>(T, 2 * static_cast<size_t>(sm_count()));
  std::vector<b200_hybrid_layer> all(r->layers);
  for (const b200_hybrid_layer& l : r->sides)
    if (l.heads > 0) all.push_back(l);
  for (const b200_hybrid_layer& l : all) {
    proj_n = std::max<size_t>(proj_n, in_rows(l));
    if (l.mixer == B200_MIXER_WINDOW_ATTN) {
      const int maps = l.score_maps > 1 ? l.score_maps : 1;
      aux_n = std::max<size_t>(aux_n, static_cast<size_t>(maps) * l.heads * l.dim);
      opa_n = std::max<size_t>(opa_n, static_cast<size_t>(l.heads) * l.vdim);
      if (needs_finish(l)) conv_n = std::max<size_t>(conv_n, static_cast<size_t>(maps) * l.heads * l.vdim);
      for (size_t rows = 1; rows <= r->attn_ws_rows; ++rows)
        attn_bytes = std::max(attn_bytes, window_attn_workspace_bytes(static_cast<int>(rows), maps * l.heads,
                                                                      maps * l.kv_heads, l.vdim, l.window, l.keep_first,
                                                                      l.kv_heads));
    } else if (l.mixer == B200_MIXER_DECAY_ATTN) {
      aux_n = std::max<size_t>(aux_n, static_cast<size_t>(l.heads) * l.vdim);
      opa_n = std::max<size_t>(opa_n, static_cast<size_t>(l.heads) * l.vdim);
      if (l.decay_rank > 0) conv_n = std::max<size_t>(conv_n, static_cast<size_t>(l.heads) * l.dim);
    } else if (l.mixer == B200_MIXER_LATENT_ATTN) {
      aux_n = std::max<size_t>(aux_n, static_cast<size_t>(l.heads) * std::max(l.kv_rank + l.rot_dim, l.vdim));
      opa_n = std::max<size_t>(opa_n, static_cast<size_t>(l.heads) * std::max(l.dim, l.vdim));
      lat_n = std::max<size_t>(lat_n, static_cast<size_t>(l.heads) * l.kv_rank);
      for (size_t rows = 1; rows <= r->attn_ws_rows; ++rows)
        attn_bytes = std::max(attn_bytes, latent_attn_workspace_bytes(static_cast<int>(rows), l.heads, l.kv_rank, l.window));
    } else {
      aux_n = std::max<size_t>(aux_n, static_cast<size_t>(l.heads) * l.vdim);
      opa_n = std::max<size_t>(opa_n, static_cast<size_t>(l.heads) * l.vdim);
      // (channel form of the delta rule: the decays and the gate logits follow the convolved rows)
      conv_n = std::max<size_t>(conv_n, l.mixer == B200_MIXER_DELTA_RULE
                                            ? 2 * static_cast<size_t>(l.kv_heads) * l.dim + static_cast<size_t>(l.heads) * l.vdim +
                                                  (l.chan_rank > 0 ? static_cast<size_t>(l.heads) * (l.dim + l.vdim) : 0)
                                            : static_cast<size_t>(l.heads) * l.vdim + 2 * static_cast<size_t>(l.kv_heads) * l.state);
    }
    if (l.experts > 0) {
      E = std::max<size_t>(E, l.experts + l.identity_experts);
      top = std::max<size_t>(top, l.top);
      moe_bytes = std::max<size_t>(moe_bytes, b200_moe_workspace_bytes(c.max_tokens, l.experts + l.identity_experts,
                                                                       l.top, c.width, l.expert_ff));
    }
    sh_n = std::max<size_t>(sh_n, l.shared_ff + (l.shared_gated ? 1 : 0));
  }
  size_t off = 0;
  auto take = [&](size_t bytes) {
    uint8_t* p = base ? base + off : nullptr;
    off = up256(off + bytes);
    return p;
  };
  bool depth = false;
  for (const b200_hybrid_layer& l : r->layers) depth = depth || l.depth_w != nullptr;
  r->x0 = r->x = (float*)take(T * c.width * 4);
  r->hist = depth ? (float*)take((static_cast<size_t>(c.num_layers) + 1) * T * c.width * 4) : nullptr;
  r->y = (float*)take(T * c.width * 4);
  r->h = take(T * c.width * es);
  r->proj = (float*)take(T * proj_n * 4);
  r->conv = (float*)take(T * conv_n * 4);
  r->aux = (float*)take(T * aux_n * 4);
  r->opa = take(T * opa_n * es);
  r->lat = take(T * lat_n * es);
  r->attn_ws = attn_bytes ? take(attn_bytes) : nullptr;
  r->rlog = (float*)take(T * E * 4);
  r->top_idx = (int32_t*)take(T * top * 4);
  r->top_w = (float*)take(T * top * 4);
  r->moe_ws = take(moe_bytes);
  r->sh = (float*)take(T * 2 * sh_n * 4);
  r->sha = take(T * sh_n * es);
  r->hr = take(T * c.width * es);
  r->logits = (float*)take(T * static_cast<size_t>(c.vocab) * 4);
  r->s_ids = (uint32_t*)take(T * 4);
  r->s_pos = (int64_t*)take(T * 8);
  r->s_slot = (int64_t*)take(T * 8);
  r->s_rows = (uint32_t*)take(T * 4);
  r->s_out = (uint32_t*)take(T * 4);
  r->s_cu = (uint32_t*)take((c.max_seqs + 1) * 4);
  r->s_ctx = (uint32_t*)take(c.max_seqs * 4);
  r->s_state = (int32_t*)take(c.max_seqs * 4);
  r->s_bt = (uint32_t*)take(static_cast<size_t>(c.max_seqs) * c.max_blocks_per_seq * 4);
  r->s_seed = (uint64_t*)take(8);
  return static_cast<int64_t>(off);
}

extern "C" {

b200_hybrid* b200_hybrid_new(const b200_hybrid_config* cfg) {
  if (!cfg || cfg->width <= 0 || cfg->vocab <= 0 || cfg->num_layers <= 0 || cfg->block_size != seqmix::kPage ||
      cfg->max_seqs <= 0 || cfg->max_tokens <= 0 || (cfg->dt != 0 && cfg->dt != 1)) {
    set_error(1, "hybrid_new: bad config");
    return nullptr;
  }
  auto* r = new b200_hybrid();
  r->cfg = *cfg;
  r->layers.resize(cfg->num_layers);
  r->sides.resize(cfg->num_layers);
  std::memset(r->layers.data(), 0, sizeof(b200_hybrid_layer) * cfg->num_layers);
  std::memset(r->sides.data(), 0, sizeof(b200_hybrid_layer) * cfg->num_layers);
  return r;
}

void b200_hybrid_free(b200_hybrid* r) {
  if (!r) return;
  r->drop_graphs();
  delete r;
}

// the mixer's own fields (shared by a layer's first mixer and its side mixer)
static bool mixer_ok(const b200_hybrid_layer* l) {
  bool ok = l->heads > 0 && l->vdim > 0 && l->w_in && l->w_o;
  if (l->mixer == B200_MIXER_WINDOW_ATTN)
    return ok && l->kv_heads > 0 && l->heads % l->kv_heads == 0 && l->dim > 0 && l->rot_dims % 2 == 0 &&
           l->rot_dims <= l->dim && (l->rot_dims == 0 || l->rot_freq) && l->kv_cache && l->v_cache &&
           (!l->v_from_k || l->vdim == l->dim) && l->gated >= 0 && l->gated <= 2 && l->score_maps >= 0 &&
           l->score_maps <= 2 && (l->score_maps < 2 || (!l->v_from_k && !l->sink)) && l->chunk >= 0 &&
           (!l->v_rot_freq || (l->vdim % 2 == 0 && !l->v_from_k));
  if (l->mixer == B200_MIXER_DECAY_ATTN)
    return ok && l->dim > 0 && l->dim <= 256 && l->rec_state && l->norm_groups > 0 &&
           (l->heads * l->vdim) % l->norm_groups == 0 && (l->out_norm_period == 0 || l->out_norm_w) &&
           (l->decay_rank > 0 ? (l->w_decay2 && l->decay_tau > 0.f) : l->head_decay != nullptr);
  return false;
}
void b200_hybrid_set_layer_side(b200_hybrid* r, int32_t layer, const b200_hybrid_layer* side) {
  if (layer < 0 || layer >= r->cfg.num_layers || !side) {
    set_error(1, "hybrid_set_layer_side: layer out of range");
    return;
  }
  if (!mixer_ok(side)) {
    set_error(1, "hybrid_set_layer_side: a side mixer is windowed attention or decayed linear attention, fully described");
    return;
  }
  r->sides[layer] = *side;
}

void b200_hybrid_set_layer(b200_hybrid* r, int32_t layer, const b200_hybrid_layer* l) {
  if (layer < 0 || layer >= r->cfg.num_layers || !l) {
    set_error(1, "hybrid_set_layer: layer out of range");
    return;
  }
  bool ok = l->heads > 0 && l->vdim > 0 && l->w_in && l->w_o;
  if (l->layout == B200_LAYOUT_SANDWICH)
    ok = ok && l->norm_w && l->post_norm_w && l->experts == 0 && (l->shared_ff == 0 || (l->ff_norm_w && l->ff_post_norm_w));
  else if (l->layout == B200_LAYOUT_POSTNORM)
    ok = ok && l->post_norm_w && ((l->shared_ff == 0 && l->experts == 0) || l->ff_post_norm_w);
  else
    ok = ok && l->norm_w && (l->layout == B200_LAYOUT_PARALLEL || l->layout == B200_LAYOUT_PRENORM);
  if (l->layout == B200_LAYOUT_PRENORM)
    ok = ok && ((l->shared_ff == 0 && l->experts == 0) || l->ff_norm_w) && (l->experts == 0 || l->ff_scale == 1.f);
  ok = ok && (l->norm_kind == B200_NORM_RMS || l->norm_kind == B200_NORM_DYNTANH) && (!l->shift_w || l->shift_state) &&
       ((!l->shift_w && !l->depth_w && !l->ff_up_bias && !l->ff_down_bias && l->norm_kind == B200_NORM_RMS) ||
        l->layout == B200_LAYOUT_PRENORM) &&
       ((!l->ff_up_bias && !l->ff_down_bias) || (l->shared_ff > 0 && l->shared_act == 1 && !l->shared_gated));
  if (l->mixer == B200_MIXER_WINDOW_ATTN || l->mixer == B200_MIXER_DECAY_ATTN)
    ok = ok && mixer_ok(l);
  else if (l->mixer == B200_MIXER_LATENT_ATTN)
    ok = ok && l->kv_rank > 0 && l->w_uk && l->w_uv && (l->shared_cache || l->latent_norm_w) && l->kv_cache &&
         l->rot_dims % 2 == 0 && l->rot_dims <= l->rot_dim && (l->rot_dims == 0 || l->rot_freq) &&
         (l->gated == 0 || l->gated == 1) && (!l->shared_cache || l->rot_dim == 0);
  else if (l->mixer == B200_MIXER_DELTA_RULE)
    ok = ok && l->kv_heads > 0 && l->heads % l->kv_heads == 0 && l->dim > 0 && l->conv_taps >= 1 && l->conv_w &&
         l->conv_state && l->rec_state && l->a_log && l->dt_bias && l->out_norm_w && l->chan_rank >= 0 &&
         l->gate_rank >= 0 && (l->chan_rank == 0 ? l->gate_rank == 0 : (l->w_decay2 && l->gate_rank > 0 && l->w_gate2));
  else if (l->mixer == B200_MIXER_SSD)
    ok = ok && l->kv_heads > 0 && l->heads % l->kv_heads == 0 && l->state > 0 && l->conv_taps >= 1 && l->conv_w &&
         l->conv_state && l->rec_state && l->a_log && l->dt_bias && l->out_norm_w && l->norm_groups > 0 &&
         (l->heads * l->vdim) % l->norm_groups == 0;
  else
    ok = false;
  if (l->experts > 0) {
    const int all = l->experts + l->identity_experts;
    ok = ok && l->identity_experts >= 0 && l->top > 0 && l->top <= all && l->expert_ff > 0 && l->w_router &&
         l->w_gate_up && l->w_down && (l->expert_act == 0 || l->expert_act == 1) && l->route_groups >= 0 &&
         (l->route_groups == 0 || (all % l->route_groups == 0 && l->route_keep >= 1 && l->route_keep <= l->route_groups &&
                                   l->top <= all / l->route_groups * l->route_keep));
  } else {
    ok = ok && l->identity_experts == 0;
  }
  if (l->shared_ff > 0)
    ok = ok && l->w_shared_gate_up && l->w_shared_down && (l->shared_act == 0 || l->shared_act == 1) &&
         (!l->shared_gated || l->shared_act == 1);
  if (!ok) {
    set_error(1, "hybrid_set_layer: inconsistent layer description");
    return;
  }
  r->layers[layer] = *l;
}

void b200_hybrid_set_globals(b200_hybrid* r, const void* embed, const void* final_norm, const void* lm_head) {
  r->embed = embed;
  r->final_norm = final_norm;
  r->lm_head = lm_head;
}

void b200_hybrid_set_final_norm(b200_hybrid* r, const void* bias, float alpha) {
  r->final_norm_b = bias;
  r->final_norm_alpha = alpha;
}

int64_t b200_hybrid_workspace_bytes(const b200_hybrid* r) {
  b200_hybrid tmp;
  tmp.cfg = r->cfg;
  tmp.layers = r->layers;
  tmp.sides = r->sides;
  return carve(&tmp, nullptr) + 256;
}

void b200_hybrid_set_workspace(b200_hybrid* r, void* workspace, int64_t bytes) {
  uint8_t* base = reinterpret_cast<uint8_t*>(up256(reinterpret_cast<size_t>(workspace)));
  const int64_t need = carve(r, base);
  if (r->hist)
    for (const b200_hybrid_layer& l : r->layers)
      if (l.layout != B200_LAYOUT_PRENORM) {
        set_error(1, "hybrid_set_workspace: depth weights need every layer in the pre-norm layout");
        return;
      }
  if (need + (base - reinterpret_cast<uint8_t*>(workspace)) > bytes) {
    set_error(1, "hybrid_set_workspace: workspace too small (set every layer before asking for its size)");
    return;
  }
  r->ws = base;
}

void b200_hybrid_set_layer_trace(b200_hybrid* r, float* buf) {
  r->trace = buf;
  r->drop_graphs();
}

int32_t b200_hybrid_set_sampling(b200_hybrid* r, int32_t strategy, int32_t k, float p, float t) {
  r->drop_graphs();              // k, p and t are kernel arguments of the captured sampler launch
  if (strategy == 0) {
    r->samp_all = false; r->samp_k = 0; r->samp_p = 1.f; r->samp_t = 1.f;
    return 0;
  }
  if (strategy < 0 || strategy > 4 || !(t > 0.f) || (strategy != 1 && (k < 1 || k > 256))) {
    set_error(1, "hybrid_set_sampling: unknown strategy or parameters out of range");
    return -1;
  }
  r->samp_all = strategy == 1; r->samp_k = strategy == 1 ? 0 : k; r->samp_p = p; r->samp_t = t;
  return 0;
}

void b200_hybrid_set_step_seed(b200_hybrid* r, uint64_t seed, int64_t stream) {
  if (!r->ws) {
    set_error(1, "hybrid_set_step_seed: workspace not set");
    return;
  }
  cudaMemcpyAsync(r->s_seed, &seed, 8, cudaMemcpyHostToDevice, reinterpret_cast<cudaStream_t>(stream));
}

int64_t b200_hybrid_launches_per_step(const b200_hybrid* r) { return r->launches; }

static void mixer_latent(b200_hybrid* r, const b200_hybrid_layer& l, const int64_t* positions, const int64_t* slots,
                         const uint32_t* cu, const uint32_t* ctx, const uint32_t* bt, int max_blocks, int B, int T,
                         float* dst, float alpha, float beta, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  const int H = l.heads, R = l.kv_rank + l.rot_dim, n_in = in_rows(l);
  gemm_f32out(r->hin, c.width, 0, l.w_in, c.width, 0, r->proj, n_in, 0, T, n_in, c.width, 1, 0.f, 0, c.dt, st);
  // a layer that shares another layer's cache brings queries only: nothing is normed or written
  launch_latent_prep(r->proj, n_in, r->opa, r->aux, l.shared_cache ? nullptr : l.kv_cache, (const float*)l.latent_norm_w,
                     l.rot_freq, l.rot_mag, positions, slots, T, H, l.dim, l.rot_dim, l.rot_dims, l.kv_rank, c.norm_eps,
                     c.dt, st);
  // q_abs[t, h, :] = q_plain[t, h, :] W_uk[h]  (W_uk[h] is [dim, kv_rank], i.e. stored [K, N])
  if (l.dim > 0)
    gemm_f32out(r->opa, H * l.dim, l.dim, l.w_uk, l.kv_rank, static_cast<long long>(l.dim) * l.kv_rank, r->aux, H * R, R,
                T, l.kv_rank, l.dim, H, 0.f, 1, c.dt, st);
  else
    cudaMemsetAsync(r->aux, 0, static_cast<size_t>(T) * H * R * 4, st);   // (rotated parts are rewritten by prep; dim == 0 is rejected upstream)
  const float* gate = l.gated ? r->proj + (n_in - H) : nullptr;          // the gate logits close the projection row
  launch_latent_attn(r->lat, r->aux, l.kv_cache, (const float*)l.sink, gate, n_in, cu, ctx, bt, max_blocks, B, T, H,
                     l.kv_rank, l.rot_dim, l.window, l.scale, c.dt,
                     static_cast<size_t>(T) <= r->attn_ws_rows ? r->attn_ws : nullptr, st);
  // v[t, h, :] = lat[t, h, :] W_uv[h]^T  (W_uv[h] is [vdim, kv_rank])
  gemm_f32out(r->lat, H * l.kv_rank, l.kv_rank, l.w_uv, l.kv_rank, static_cast<long long>(l.vdim) * l.kv_rank, r->aux,
              H * l.vdim, l.vdim, T, l.vdim, l.kv_rank, H, 0.f, 0, c.dt, st);
  const void* o_in = r->aux;
  if (!c.dt) {
    launch_cast_rows(r->opa, r->aux, H * l.vdim, T, H * l.vdim, 0, st);
    o_in = r->opa;
  }
  gemm_f32out_scaled(o_in, H * l.vdim, 0, l.w_o, H * l.vdim, 0, dst, c.width, 0, T, c.width, H * l.vdim, 1, alpha, beta, 0,
                     c.dt, st);
}

static void mixer_delta(b200_hybrid* r, const b200_hybrid_layer& l, const uint32_t* cu, const uint32_t* ctx,
                        const int32_t* state_slots, int B, int T, float* dst, float alpha, float beta, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  const int H = l.heads, Hk = l.kv_heads, n_in = in_rows(l);
  const int nq = Hk * l.dim, nv = H * l.vdim, nconv = 2 * nq + nv;
  gemm_f32out(r->hin, c.width, 0, l.w_in, c.width, 0, r->proj, n_in, 0, T, n_in, c.width, 1, 0.f, 0, c.dt, st);
  launch_short_conv_silu(r->conv, nconv, r->proj, n_in, (const float*)l.conv_w, (const float*)l.conv_b,
                         (float*)l.conv_state, state_slots, cu, ctx, B, T, nconv, l.conv_taps, st);
  const float* q = r->conv;
  const float* k = r->conv + nq;
  const float* v = r->conv + 2 * nq;
  const float* b_raw = r->proj + nconv;
  if (l.chan_rank > 0) {
    // decays per head and key channel, and the gate's logits, from the two low-rank halves that close the projection
    // row; the second factors are fp32 whatever the operand dtype (what enters the recurrence is not rounded)
    const int nd = H * l.dim;
    float* decay = r->conv + static_cast<size_t>(T) * nconv;
    float* gate2 = decay + static_cast<size_t>(T) * nd;
    const float* low_a = b_raw + H;
    const float* low_g = low_a + l.chan_rank;
    launch_lowrank_decay(decay, low_a, n_in, (const float*)l.w_decay2, (const float*)l.dt_bias, 1.f, (const float*)l.a_log,
                         l.dim, T, nd, l.chan_rank, st);
    launch_delta_rule(r->aux, q, k, v, nconv, b_raw, nullptr, n_in, nullptr, nullptr, decay, nd, (float*)l.rec_state,
                      state_slots, cu, ctx, B, H, Hk, l.dim, l.vdim, st);
    gemm_f32out(low_g, n_in, 0, l.w_gate2, l.gate_rank, 0, gate2, nv, 0, T, nv, l.gate_rank, 1, 0.f, 0, 1, st);
    launch_gated_group_norm(r->opa, r->aux, nv, gate2, nv, (const float*)l.out_norm_w, l.vdim, T, nv, l.vdim, c.norm_eps,
                            0, 1, c.dt, st);
    gemm_f32out_scaled(r->opa, nv, 0, l.w_o, nv, 0, dst, c.width, 0, T, c.width, nv, 1, alpha, beta, 0, c.dt, st);
    return;
  }
  const float* a_raw = b_raw + H;
  const float* gate = a_raw + H;
  launch_delta_rule(r->aux, q, k, v, nconv, b_raw, a_raw, n_in, (const float*)l.a_log, (const float*)l.dt_bias, nullptr,
                    0, (float*)l.rec_state, state_slots, cu, ctx, B, H, Hk, l.dim, l.vdim, st);
  launch_gated_group_norm(r->opa, r->aux, nv, gate, n_in, (const float*)l.out_norm_w, l.vdim, T, nv, l.vdim, c.norm_eps,
                          0, 0, c.dt, st);
  gemm_f32out_scaled(r->opa, nv, 0, l.w_o, nv, 0, dst, c.width, 0, T, c.width, nv, 1, alpha, beta, 0, c.dt, st);
}

static void mixer_ssd(b200_hybrid* r, const b200_hybrid_layer& l, const uint32_t* cu, const uint32_t* ctx,
                      const int32_t* state_slots, int B, int T, float* dst, float alpha, float beta, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  const int H = l.heads, G = l.kv_heads, N = l.state, inner = H * l.vdim, n_in = in_rows(l);
  const int nconv = inner + 2 * G * N;
  gemm_f32out(r->hin, c.width, 0, l.w_in, c.width, 0, r->proj, n_in, 0, T, n_in, c.width, 1, 0.f, 0, c.dt, st);
  const float* xbc = r->conv;
  launch_short_conv_silu(r->conv, nconv, r->proj + inner, n_in, (const float*)l.conv_w, (const float*)l.conv_b,
                         (float*)l.conv_state, state_slots, cu, ctx, B, T, nconv, l.conv_taps, st);
  launch_ssd_scan(r->aux, xbc, xbc + inner, xbc + inner + G * N, nconv, r->proj + inner + nconv, n_in, (const float*)l.a_log,
                  (const float*)l.dt_bias, (const float*)l.d_skip, (float*)l.rec_state, state_slots, cu, ctx, B, H, G, N,
                  l.vdim, st);
  launch_gated_group_norm(r->opa, r->aux, inner, r->proj, n_in, (const float*)l.out_norm_w, inner, T, inner,
                          inner / l.norm_groups, c.norm_eps, 1, 0, c.dt, st);
  gemm_f32out_scaled(r->opa, inner, 0, l.w_o, inner, 0, dst, c.width, 0, T, c.width, inner, 1, alpha, beta, 0, c.dt, st);
}

static void mixer_window(b200_hybrid* r, const b200_hybrid_layer& l, const int64_t* positions, const int64_t* slots,
                         const uint32_t* cu, const uint32_t* ctx, const uint32_t* bt, int max_blocks, int B, int T,
                         float* dst, float alpha, float beta, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  const int H = l.heads, G = l.kv_heads, n_in = in_rows(l), nv = H * l.vdim;
  const int maps = l.score_maps > 1 ? l.score_maps : 1;       // the maps' heads lie one map after the other
  const bool finish = needs_finish(l);
  gemm_f32out(r->hin, c.width, 0, l.w_in, c.width, 0, r->proj, n_in, 0, T, n_in, c.width, 1, 0.f, 0, c.dt, st);
  b200_attn_options opt;
  std::memset(&opt, 0, sizeof(opt));
  opt.head_norm = l.head_norm;
  opt.v_from_k = l.v_from_k;
  opt.q_temp_every = l.q_temp_every;
  opt.q_temp_coef = l.q_temp_coef;
  opt.gate_elems = l.gated == 2;
  opt.dist_slopes = (const float*)l.dist_slopes;
  opt.rot_half = l.rot_half;
  opt.rot_mag = l.rot_mag;
  opt.v_rot_freq = l.v_rot_freq;
  opt.v_heads = G;
  opt.chunk = l.chunk;
  opt.out_f32 = finish;
  opt.no_cache = l.shared_cache;
  launch_window_attn_prep(r->proj, n_in, (const float*)l.in_bias, (const float*)l.q_norm_w, (const float*)l.k_norm_w,
                          l.rot_freq, positions, slots, r->aux, l.kv_cache, l.v_cache, T, maps * H, maps * G, l.dim,
                          l.vdim, l.rot_dims, c.norm_eps, c.dt, &opt, st);
  const float* gate = l.gated ? r->proj + (n_in - (l.gated == 2 ? nv : H)) : nullptr;     // the gate logits close the row
  void* ws = static_cast<size_t>(T) <= r->attn_ws_rows ? r->attn_ws : nullptr;
  if (finish) {
    // fp32 sums of every map, then one kernel for all that follows them
    launch_window_attn(r->conv, r->aux, l.kv_cache, l.v_cache, (const float*)l.sink, nullptr, 0, cu, ctx, bt, max_blocks, B,
                       T, maps * H, maps * G, l.dim, l.vdim, l.window, l.keep_first, l.scale, l.softcap, c.dt, ws, &opt, st);
    launch_attn_finish(r->opa, r->conv, gate, n_in, l.gated == 2, positions, l.v_rot_freq, l.rot_half, maps, l.diff_lambda,
                       l.diff_norm, c.norm_eps, maps > 1 ? l.diff_out_scale : 1.f, T, H, l.vdim, c.dt, st);
  } else {
    launch_window_attn(r->opa, r->aux, l.kv_cache, l.v_cache, (const float*)l.sink, gate, n_in, cu, ctx, bt, max_blocks, B,
                       T, H, G, l.dim, l.vdim, l.window, l.keep_first, l.scale, l.softcap, c.dt, ws, &opt, st);
  }
  gemm_f32out_scaled(r->opa, nv, 0, l.w_o, nv, 0, dst, c.width, 0, T, c.width, nv, 1, alpha, beta, 0, c.dt, st);
  if (l.o_bias) launch_bias_rows(dst, (const float*)l.o_bias, alpha, T, c.width, st);
}

static void mixer_decay(b200_hybrid* r, const b200_hybrid_layer& l, const uint32_t* cu, const uint32_t* ctx,
                        const int32_t* state_slots, int B, int T, float* dst, float alpha, float beta, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  const int H = l.heads, nk = H * l.dim, nv = H * l.vdim, n_in = in_rows(l);
  gemm_f32out(r->hin, c.width, 0, l.w_in, c.width, 0, r->proj, n_in, 0, T, n_in, c.width, 1, 0.f, 0, c.dt, st);
  const float* q = r->proj;
  const float* k = q + nk;
  const float* v = k + nk;
  const float* gate = v + nv;
  const float* chan = nullptr;
  if (l.decay_rank > 0) {
    launch_lowrank_decay(r->conv, gate + nv, n_in, (const float*)l.w_decay2, (const float*)l.decay_bias, l.decay_tau,
                         nullptr, 1, T, nk, l.decay_rank, st);
    chan = r->conv;
  }
  launch_decay_attn(r->aux, q, k, v, n_in, chan ? nullptr : (const float*)l.head_decay, chan, nk, l.q_scale, l.k_scale,
                    l.qkv_act, (float*)l.rec_state, state_slots, cu, ctx, B, H, l.dim, l.vdim, st);
  launch_gated_group_norm(r->opa, r->aux, nv, gate, n_in, (const float*)(l.out_norm_period ? l.out_norm_w : nullptr),
                          l.out_norm_period ? l.out_norm_period : 1, T, nv, nv / l.norm_groups, c.norm_eps, 0, l.gate_act,
                          c.dt, st);
  gemm_f32out_scaled(r->opa, nv, 0, l.w_o, nv, 0, dst, c.width, 0, T, c.width, nv, 1, alpha, beta, 0, c.dt, st);
  if (l.o_bias) launch_bias_rows(dst, (const float*)l.o_bias, alpha, T, c.width, st);
}

// one mixer of a layer: dst = alpha * mixer(h) + beta * dst
static void run_mixer(b200_hybrid* r, const b200_hybrid_layer& l, const int64_t* positions, const int64_t* slot_mapping,
                      const uint32_t* cu, const uint32_t* ctx, const uint32_t* block_tables, const int32_t* state_slots,
                      int max_blocks, int B, int T, float* dst, float alpha, float beta, cudaStream_t st) {
  switch (l.mixer) {
    case B200_MIXER_LATENT_ATTN:
      mixer_latent(r, l, positions, slot_mapping, cu, ctx, block_tables, max_blocks, B, T, dst, alpha, beta, st);
      break;
    case B200_MIXER_DELTA_RULE: mixer_delta(r, l, cu, ctx, state_slots, B, T, dst, alpha, beta, st); break;
    case B200_MIXER_WINDOW_ATTN:
      mixer_window(r, l, positions, slot_mapping, cu, ctx, block_tables, max_blocks, B, T, dst, alpha, beta, st);
      break;
    case B200_MIXER_DECAY_ATTN: mixer_decay(r, l, cu, ctx, state_slots, B, T, dst, alpha, beta, st); break;
    default: mixer_ssd(r, l, cu, ctx, state_slots, B, T, dst, alpha, beta, st); break;
  }
}

// dense gated feed-forward of a sandwich layer: y = W_down (silu(W_gate h) * (W_up h))
static void dense_ffn(b200_hybrid* r, const b200_hybrid_layer& l, int T, cudaStream_t st) {
  const b200_hybrid_config& c = r->cfg;
  gemm_f32out(r->hin, c.width, 0, l.w_shared_gate_up, c.width, 0, r->sh, 2 * l.shared_ff, 0, T, 2 * l.shared_ff, c.width, 1,
              0.f, 0, c.dt, st);
  launch_silu_mul_f32(r->sha, r->sh, T, l.shared_ff, c.dt, st);
  gemm_f32out(r->sha, l.shared_ff, 0, l.w_shared_down, l.shared_ff, 0, r->y, c.width, 0, T, c.width, l.shared_ff, 1, 0.f,
              0, c.dt, st);
}

// routed experts and their shared expert: dst = (accumulate ? dst : 0) + experts(h) + shared(h).  `ident` / `ident_f32`:
// the rows that identity experts return (the sublayer's input before any rounding, where the layer has it in fp32).
// `scale` multiplies the shared / dense part (routed experts take none).
static void feed_forward(b200_hybrid* r, const b200_hybrid_layer& l, int T, float* dst, bool accumulate, const void* ident,
                         int ident_f32, cudaStream_t st, float scale = 1.f) {
  const b200_hybrid_config& c = r->cfg;
  if (l.experts > 0) {
    const int all = l.experts + l.identity_experts;
    gemm_f32out(r->hin, c.width, 0, l.w_router, c.width, 0, r->rlog, all, 0, T, all, c.width, 1, 0.f, 0, c.dt, st);
    launch_moe_route(r->rlog, (const float*)l.route_bias, T, all, l.top, l.route_groups, l.route_keep, l.route_scale,
                     r->top_idx, r->top_w, st);
    b200_moe_experts_ex(dst, r->hin, r->top_idx, r->top_w, l.w_gate_up, l.w_down, T, l.experts, l.identity_experts, l.top,
                        c.width, l.expert_ff, l.expert_act, accumulate ? 1 : 0, ident, ident_f32, c.dt, r->moe_ws,
                        reinterpret_cast<int64_t>(st));
    accumulate = true;
  }
  if (l.shared_ff > 0) {
    // SiLU-gated: [gate | up] rows; squared ReLU: up rows, closed by the one row of the token's gate where there is one
    const int rows = l.shared_act == 0 ? 2 * l.shared_ff : l.shared_ff + (l.shared_gated ? 1 : 0);
    gemm_f32out(r->hin, c.width, 0, l.w_shared_gate_up, c.width, 0, r->sh, rows, 0, T, rows, c.width, 1, 0.f, 0, c.dt, st);
    if (l.shared_act == 0)
      launch_silu_mul_f32(r->sha, r->sh, T, l.shared_ff, c.dt, st);
    else
      launch_relu2_f32(r->sha, r->sh, rows, T, l.shared_ff, l.shared_gated ? l.shared_ff : -1,
                       (const float*)l.ff_up_bias, c.dt, st);
    gemm_f32out_scaled(r->sha, l.shared_ff, 0, l.w_shared_down, l.shared_ff, 0, dst, c.width, 0, T, c.width, l.shared_ff,
                       1, scale, accumulate ? 1.f : 0.f, 0, c.dt, st);
    if (l.ff_down_bias) launch_bias_rows(dst, (const float*)l.ff_down_bias, scale, T, c.width, st);
  }
}

void b200_hybrid_step(b200_hybrid* r, const uint32_t* input_ids, const int64_t* positions, const int64_t* slot_mapping,
                      const uint32_t* cu, const uint32_t* ctx, const uint32_t* block_tables,
                      const int32_t* state_slots, const uint32_t* out_rows, int32_t B, int32_t T, int32_t max_blocks,
                      int32_t num_out, float* logits, uint32_t* out_ids, int64_t stream) {
  const b200_hybrid_config& c = r->cfg;
  if (!r->ws || !r->embed || !r->final_norm || !r->lm_head) {
    set_error(1, "hybrid_step: workspace or global weights not set");
    return;
  }
  if (B <= 0 || B > c.max_seqs || T <= 0 || T > c.max_tokens || num_out < 0 || num_out > T) {
    set_error(1, "hybrid_step: batch out of range");
    return;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const long long launches0 = launch_count();
  // the sublayers of post-norm layers take the un-normed stream: in bf16 runs the kernel that last wrote x also leaves its rounding in h
  const bool first_reads_stream = r->layers[0].layout == B200_LAYOUT_POSTNORM && !c.dt;
  // with depth weights the results of the embedding and of every layer lie side by side; layer i works in slot i + 1
  const size_t hstride = static_cast<size_t>(c.max_tokens) * c.width, xbytes = static_cast<size_t>(T) * c.width * 4;
  r->x = r->hist ? r->hist : r->x0;
  launch_embed_f32(r->x, r->embed, input_ids, positions, c.embed_pos_base, T, c.width, c.vocab, c.embed_scale, c.dt,
                   first_reads_stream ? r->h : nullptr, st);
  if (r->hist) {
    cudaMemcpyAsync(r->hist + hstride, r->hist, xbytes, cudaMemcpyDeviceToDevice, st);     // layer 0 starts from X_0
    r->x = r->hist + hstride;
  }
  bool h_is_x = first_reads_stream;          // h holds the bf16 rounding of the current x
  for (int i = 0; i < c.num_layers; ++i) {
    const b200_hybrid_layer& l = r->layers[i];
    const b200_hybrid_layer& side = r->sides[i];
    r->hin = r->h;
    if (l.layout == B200_LAYOUT_POSTNORM) {
      // sublayer input = x: rounded to bf16 for the products, in place for fp32 runs
      auto stream_in = [&]() {
        if (c.dt) r->hin = r->x;
        else if (!h_is_x) launch_cast_rows(r->h, r->x, c.width, T, c.width, 0, st);
      };
      void* cast = c.dt ? nullptr : r->h;
      stream_in();
      run_mixer(r, l, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->y, l.out_scale,
                0.f, st);
      if (side.heads > 0)
        run_mixer(r, side, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->y,
                  side.out_scale, 1.f, st);
      launch_resid_add_rmsnorm(r->x, r->y, (const float*)l.post_norm_w, T, c.width, c.norm_eps, c.norm_weight_offset,
                               cast, st);
      h_is_x = cast != nullptr;
      if (l.experts > 0 || l.shared_ff > 0) {
        stream_in();
        if (l.experts > 0) feed_forward(r, l, T, r->y, false, r->x, 1, st);
        else dense_ffn(r, l, T, st);
        launch_resid_add_rmsnorm(r->x, r->y, (const float*)l.ff_post_norm_w, T, c.width, c.norm_eps,
                                 c.norm_weight_offset, cast, st);
      }
      if (r->trace)
        cudaMemcpyAsync(r->trace + static_cast<size_t>(i) * c.max_tokens * c.width, r->x,
                        static_cast<size_t>(T) * c.width * 4, cudaMemcpyDeviceToDevice, st);
      continue;
    }
    h_is_x = false;
    if (l.layout == B200_LAYOUT_PRENORM) {
      launch_stream_norm(r->h, r->x, (const float*)l.norm_w, (const float*)l.norm_b, l.norm_alpha, l.norm_kind, c.norm_eps,
                         c.norm_weight_offset, nullptr, (const float*)l.shift_w, (float*)l.shift_state, state_slots, cu,
                         ctx, B, T, c.width, c.dt, st);
      run_mixer(r, l, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->x, l.out_scale,
                1.f, st);
      if (side.heads > 0)
        run_mixer(r, side, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->x,
                  side.out_scale, 1.f, st);
      if (l.experts > 0 || l.shared_ff > 0) {
        launch_stream_norm(r->h, r->x, (const float*)l.ff_norm_w, (const float*)l.ff_norm_b, l.ff_norm_alpha, l.norm_kind,
                           c.norm_eps, c.norm_weight_offset, nullptr, nullptr, nullptr, nullptr, nullptr, nullptr, 0, T,
                           c.width, c.dt, st);
        feed_forward(r, l, T, r->x, true, r->h, 0, st, l.ff_scale);
      }
      if (r->hist) {
        // what goes on: the weighted sum of the results so far, or (a layer without weights) this layer's result
        float* next = i + 1 < c.num_layers ? r->hist + static_cast<size_t>(i + 2) * hstride : r->x0;
        if (l.depth_w) launch_depth_mix(next, r->hist, hstride, (const float*)l.depth_w, i + 2, static_cast<size_t>(T) * c.width, st);
        else cudaMemcpyAsync(next, r->x, xbytes, cudaMemcpyDeviceToDevice, st);
        r->x = next;
      }
      if (r->trace)
        cudaMemcpyAsync(r->trace + static_cast<size_t>(i) * c.max_tokens * c.width, r->x, xbytes, cudaMemcpyDeviceToDevice,
                        st);
      continue;
    }
    launch_resid_rmsnorm(r->h, r->x, (const float*)l.norm_w, T, c.width, c.norm_eps, c.norm_weight_offset, nullptr,
                         c.dt, st);
    if (l.layout == B200_LAYOUT_SANDWICH) {
      run_mixer(r, l, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->y, l.out_scale,
                0.f, st);
      if (side.heads > 0)
        run_mixer(r, side, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->y,
                  side.out_scale, 1.f, st);
      launch_resid_add_rmsnorm(r->x, r->y, (const float*)l.post_norm_w, T, c.width, c.norm_eps, c.norm_weight_offset,
                               nullptr, st);
      if (l.shared_ff > 0) {
        launch_resid_rmsnorm(r->h, r->x, (const float*)l.ff_norm_w, T, c.width, c.norm_eps, c.norm_weight_offset, nullptr,
                             c.dt, st);
        dense_ffn(r, l, T, st);
        launch_resid_add_rmsnorm(r->x, r->y, (const float*)l.ff_post_norm_w, T, c.width, c.norm_eps,
                                 c.norm_weight_offset, nullptr, st);
      }
    } else {
      run_mixer(r, l, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->x, l.out_scale,
                1.f, st);
      if (side.heads > 0)
        run_mixer(r, side, positions, slot_mapping, cu, ctx, block_tables, state_slots, max_blocks, B, T, r->x,
                  side.out_scale, 1.f, st);
      feed_forward(r, l, T, r->x, true, r->h, 0, st);
    }
    if (r->trace)
      cudaMemcpyAsync(r->trace + static_cast<size_t>(i) * c.max_tokens * c.width, r->x,
                      static_cast<size_t>(T) * c.width * 4, cudaMemcpyDeviceToDevice, st);
  }
  if (num_out > 0) {
    if (c.final_norm_kind == B200_NORM_RMS)
      launch_resid_rmsnorm(r->hr, r->x, (const float*)r->final_norm, num_out, c.width, c.norm_eps, c.norm_weight_offset,
                           out_rows, c.dt, st);
    else
      launch_stream_norm(r->hr, r->x, (const float*)r->final_norm, (const float*)r->final_norm_b, r->final_norm_alpha,
                         c.final_norm_kind, c.norm_eps, c.norm_weight_offset, out_rows, nullptr, nullptr, nullptr, nullptr,
                         nullptr, 0, num_out, c.width, c.dt, st);
    float* lg = logits ? logits : r->logits;
    gemm_f32out(r->hr, c.width, 0, r->lm_head, c.width, 0, lg, c.vocab, 0, num_out, c.vocab, c.width, 1, 0.f, 0, c.dt,
                st);
    if (out_ids) {
      if (r->samp_k > 0 || r->samp_all)
        launch_sample_topk_topp(out_ids, lg, num_out, c.vocab, r->samp_all ? 0 : std::min(r->samp_k, c.vocab), r->samp_p,
                                r->samp_t, r->s_seed, st);
      else
        b200_argmax_f32(out_ids, lg, num_out, c.vocab, stream);
    }
  }
  r->launches = launch_count() - launches0;
}

int32_t b200_hybrid_step_host(b200_hybrid* r, const uint32_t* input_ids, const int64_t* positions,
                              const int64_t* slot_mapping, const uint32_t* cu, const uint32_t* ctx,
                              const uint32_t* block_tables, const int32_t* state_slots, const uint32_t* out_rows,
                              int32_t B, int32_t T, int32_t max_blocks, int32_t num_out, float* logits_host,
                              uint32_t* out_ids_host, int64_t stream) {
  const b200_hybrid_config& c = r->cfg;
  if (!r->ws || B <= 0 || B > c.max_seqs || T <= 0 || T > c.max_tokens || max_blocks > c.max_blocks_per_seq ||
      num_out < 0 || num_out > T) {
    set_error(1, "hybrid_step_host: bad arguments");
    return -1;
  }
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const auto H2D = cudaMemcpyHostToDevice;
  cudaMemcpyAsync(r->s_ids, input_ids, T * 4, H2D, st);
  cudaMemcpyAsync(r->s_pos, positions, T * 8, H2D, st);
  cudaMemcpyAsync(r->s_slot, slot_mapping, T * 8, H2D, st);
  cudaMemcpyAsync(r->s_cu, cu, (B + 1) * 4, H2D, st);
  cudaMemcpyAsync(r->s_ctx, ctx, B * 4, H2D, st);
  cudaMemcpyAsync(r->s_state, state_slots, B * 4, H2D, st);
  cudaMemcpyAsync(r->s_bt, block_tables, static_cast<size_t>(B) * max_blocks * 4, H2D, st);
  if (num_out > 0) cudaMemcpyAsync(r->s_rows, out_rows, num_out * 4, H2D, st);
  auto run = [&]() {
    b200_hybrid_step(r, r->s_ids, r->s_pos, r->s_slot, r->s_cu, r->s_ctx, r->s_bt, r->s_state, r->s_rows, B, T,
                     max_blocks, num_out, nullptr, out_ids_host ? r->s_out : nullptr, stream);
  };
  bool done = false;
  if (graphs_enabled() && !r->trace && T <= kGraphMaxRows && st != nullptr) {      // the legacy stream cannot capture
    if (r->graphs.size() > 512) r->drop_graphs();
    auto& g = r->graphs[std::make_tuple(B, T, max_blocks, num_out, out_ids_host ? 1 : 0)];
    if (!g.exec && g.seen++ >= 1 && !b200_last_error()) {
      cudaGraph_t graph = nullptr;
      if (cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed) == cudaSuccess) {
        const int64_t launches = r->launches;
        run();
        if (cudaStreamEndCapture(st, &graph) == cudaSuccess && graph && !b200_last_error())
          if (cudaGraphInstantiate(&g.exec, graph, 0) != cudaSuccess) g.exec = nullptr;
        if (graph) cudaGraphDestroy(graph);
        if (!g.exec) {
          cudaGetLastError();
          g.seen = -(1 << 30);          // this shape stays on direct launches
        }
        r->launches = launches;
      }
    }
    if (g.exec) {
      cudaGraphLaunch(g.exec, st);
      done = true;
    }
  }
  if (!done) run();
  if (num_out > 0 && logits_host)
    cudaMemcpyAsync(logits_host, r->logits, static_cast<size_t>(num_out) * c.vocab * 4, cudaMemcpyDeviceToHost, st);
  if (num_out > 0 && out_ids_host) cudaMemcpyAsync(out_ids_host, r->s_out, num_out * 4, cudaMemcpyDeviceToHost, st);
  const cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) {
    set_error(2, cudaGetErrorString(e));
    return -1;
  }
  return b200_last_error() ? -1 : 0;
}

}  // extern "C"
