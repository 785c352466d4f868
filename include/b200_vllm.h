/*
 * b200_vllm.h -- C ABI of the B200-native (sm_100a) forward hot path for vllm.rs.
 *
 * Drop-in boundary.  Every symbol below replaces one call the
 * reference crate makes into its un-vendored native dependency `attention-rs`
 * (or composes several of them into one fused launch).  Conventions are the
 * reference's own (src/utils/gptq.rs:100-200, 314-333):
 *   - raw device pointers, dims as int32, CUDA stream passed as int64 (CUstream cast);
 *   - the caller owns every buffer; outputs may be uninitialised on entry and are
 *     fully written; the callee never allocates, frees, synchronises or retains
 *     pointers (=> CUDA-graph capturable); scratch comes in through an explicit
 *     `workspace` pointer sized by the matching *_workspace_bytes() query;
 *   - `void` return like the reference FFI; failures are latched and can be read
 *     with b200_last_error()/b200_last_error_string() (0 = none).
 *   - index dtypes are the reference's: slot_mapping / positions int64,
 *     block_tables / context_lens / cu_seqlens uint32 (src/core/runner.rs:1243-1388).
 *
 * Native KV-cache layout (reference layout "L2", src/utils/kvcache_allocator.rs:150-173):
 *   K and V, per layer:  [num_blocks, block_size, num_kv_heads, head_dim]  fp16.
 *
 * Native quantised-weight layout ("B200 tile-major", produced by the prepack
 * entry points, same byte count as the checkpoint tensor so it can live in the
 * buffer the reference allocates for its Marlin repack, src/utils/gptq.rs:286-298):
 *   4-bit: u32 [N/128][K/64][2][128][4]  -- for out-channel tile nt, K chunk kc,
 *          half h, channel c, word w: the eight K values k = kc*64 + h*32 + w*8 + j,
 *          nibble p (p<4) holds j=2p, nibble p+4 holds j=2p+1.
 *   8-bit: u32 [N/128][K/64][4][128][4]  -- quarter q: k = kc*64 + q*16 + w*4 + j,
 *          byte j of the word holds K offset j (natural order).
 *   scales stay [K/G, N] fp16 and qzeros stay in checkpoint packing (AWQ or GPTQ).
 */
#ifndef B200_VLLM_H
#define B200_VLLM_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ errors */
int b200_last_error(void);                 /* 0 = ok, 1 = bad argument, 2 = CUDA error */
const char* b200_last_error_string(void);
void b200_clear_error(void);
int b200_abi_version(void);
/* kernels launched by this library since load (every launch site counts itself) */
int64_t b200_launch_count(void);

/* quantisation formats (checkpoint packing of qzeros / zero-point semantics) */
#define B200_QFMT_AWQ 0       /* zero = nibble (order 0,2,4,6,1,3,5,7), no +1           */
#define B200_QFMT_GPTQ 1      /* zero = field + 1 (sequential order); NULL qzeros => sym */

/* epilogue flags of b200_wna16_gemm_ex */
#define B200_EPI_NONE 0
#define B200_EPI_SILU_MUL 1   /* out[m, n] = silu(acc[m, n]) * acc[m, n + N/2], out is [M, N/2] */

/* ------------------------------------------------- quantised weight prepack
 * Replaces attention_rs::kernels::ffi::awq_repack (gptq.rs:316-324):
 *   in  : AWQ qweight  i32 [k, n_packed]   (n = n_packed * 32/bits)
 *   out : B200 tile-major layout, k*n_packed u32.                              */
void b200_awq_prepack(const void* in, void* out, int32_t k, int32_t n_packed, int32_t bits,
                      int64_t stream);
/* Replaces attention_rs::kernels::ffi::gptq_repack (gptq.rs:325-333):
 *   in  : GPTQ qweight i32 [k_packed, n]   (k = k_packed * 32/bits)            */
void b200_gptq_prepack(const void* in, void* out, int32_t k_packed, int32_t n, int32_t bits,
                       int64_t stream);

/* ------------------------------------------------- W4A16 / W8A16 GEMM
 * C[m, n] (fp16) = A[m, k] (fp16) x dequant(B)  with fp32 accumulation.
 * Replace marlin_awq_4bit_f16 / marlin_4bit_f16 (gptq.rs:118-146) and
 * gemm_half_q_half_alt (gptq.rs:183-195); same argument order as those.
 * `workspace`: b200_wna16_workspace_bytes() bytes, zero-initialised once by the
 * caller (the reference already allocates a zeroed workspace, wna16.rs:238-241);
 * the kernels leave it zeroed on exit.                                          */
void b200_marlin_awq_4bit_f16(const void* a, const int32_t* b, const void* scales,
                              const void* qzeros, const void* g_idx, void* c, int32_t m,
                              int32_t k, int32_t n, const void* workspace, int32_t group_size,
                              int64_t stream);
void b200_marlin_4bit_f16(const void* a, const int32_t* b, const void* scales,
                          const void* qzeros, const void* g_idx, void* c, int32_t m, int32_t k,
                          int32_t n, const void* workspace, int32_t group_size, int64_t stream);
/* bf16 flavour (replace marlin_awq_4bit_bf16 / marlin_4bit_bf16, gptq.rs:150-178; bf16 is the reference's
 * default dtype, utils/mod.rs:1919-1925): a, scales and c are bf16, same argument order and workspace.  Needs
 * k % 128 == 0 and group_size = 128 * 2^j (or <= 0 / >= k: one group per channel).  Decode-shaped calls
 * (m <= 32) are one launch of the stream-K tcgen05 kernel; larger m runs 32 rows per launch.            */
void b200_marlin_awq_4bit_bf16(const void* a, const int32_t* b, const void* scales,
                               const void* qzeros, const void* g_idx, void* c, int32_t m,
                               int32_t k, int32_t n, const void* workspace, int32_t group_size,
                               int64_t stream);
void b200_marlin_4bit_bf16(const void* a, const int32_t* b, const void* scales,
                           const void* qzeros, const void* g_idx, void* c, int32_t m, int32_t k,
                           int32_t n, const void* workspace, int32_t group_size, int64_t stream);
/* 8-bit GPTQ path (reference: gemm_half_q_half_alt, bits == 8).  Unlike the reference
 * symbol this takes the prepacked weight, an explicit group_size and a workspace.  */
void b200_gemm_half_q_half_8bit(const void* a, const uint32_t* qweight, const uint32_t* qzeros,
                                const void* scales, const int32_t* g_idx, void* c, int32_t m,
                                int32_t n, int32_t k, int32_t group_size, const void* workspace,
                                int64_t stream);
/* gemm_half_q_half_alt with the reference's EXACT signature (gptq.rs:183-195 call site, 316-324 declaration):
 * `qweight` is the checkpoint-format GPTQ tensor [k / (32/bits), n] as the loader leaves it on this path, no
 * group size, no workspace.  The group size is derived from g_idx (required; one cached 8-byte read), the
 * tile-major copy of the weight is made on first use and kept, the workspace is library-owned.  The first call
 * per tensor synchronises the stream; later calls do not.  b200_gemm_half_q_half_alt_release() frees all of it. */
void b200_gemm_half_q_half_alt(const void* a, const uint32_t* qweight, const uint32_t* qzeros,
                               const void* scales, const int32_t* g_idx, void* c, int32_t m, int32_t n,
                               int32_t k, int32_t bits, int64_t stream);
void b200_gemm_half_q_half_alt_release(void);
/* General entry: bits in {4,8}, qfmt AWQ/GPTQ, optional bias[n] (fp16, may be NULL),
 * epilogue flag.  variant: 0 = auto by m, 1 = flat GEMV (CUDA cores), 2 = tcgen05 (tile-split decode kernel for m <= 64),
 * 3 = tcgen05 with a single K split (direct store, workspace untouched; prefill),
 * 4 = the general tcgen05 kernel even for decode shapes (A/B testing),
 * 5 = the stream-K tcgen05 decode kernel (m <= 32, k % 128 == 0, group_size = 128 * 2^j). */
void b200_wna16_gemm_ex(const void* a, const void* b_packed, const void* scales,
                        const void* qzeros, const void* bias, void* c, int32_t m, int32_t k,
                        int32_t n, int32_t bits, int32_t group_size, int32_t qfmt,
                        int32_t epilogue, int32_t variant, void* workspace, int64_t stream);
int64_t b200_wna16_workspace_bytes(int32_t max_m, int32_t max_n);
/* Dequantise a prepacked weight to fp16 out[n, k] (row = output channel, K-major): the weight
 * operand of b200_dense_gemm_f16.  Large prefill steps dequantise a layer once and run the dense
 * tcgen05 GEMM instead of re-dequantising per token tile (no reference counterpart: Marlin
 * re-dequantises, gptq.rs:118-146).                                                      */
void b200_wna16_dequant_f16(const void* b_packed, const void* scales, const void* qzeros, void* out,
                            int32_t k, int32_t n, int32_t bits, int32_t group_size, int32_t qfmt,
                            int64_t stream);

/* ------------------------------------------------- dense fp16 GEMM (lm_head, fp16 linears)
 * C[m, n] = A[m, k] x W[n, k]^T ; out_f32 != 0 writes fp32 logits (llama.rs:311-320).
 * Replaces Linear::forward -> cuBLAS (linear.rs:75-123) with a tcgen05 kernel (TMA-fed SS-mode
 * MMA, CTA pairs for m > 128, weight-streaming swapped form for m <= 128).               */
void b200_dense_gemm_f16(const void* a, const void* w, void* c, int32_t m, int32_t n, int32_t k,
                         int32_t out_f32, int64_t stream);
/* Same with an optional fused bias[n] (fp16, may be NULL) and an explicit implementation:
 * mode -1 = default (env B200_DENSE), 0 = cuBLAS (the reference's own call, A/B baseline),
 * 1 = tcgen05 single-CTA tiles, 2 = tcgen05 CTA pairs.                                   */
void b200_dense_gemm_ex(const void* a, const void* w, const void* bias, void* c, int32_t m,
                        int32_t n, int32_t k, int32_t out_f32, int32_t mode, int64_t stream);

/* ------------------------------------------------- RoPE + KV-cache write
 * Replaces FusedRope::apply_inplace (rotary_emb.rs:88-104) followed by the cache
 * write inside PagedAttention::forward (attention.rs:808-820) in ONE launch.
 * q [T,H,D], k/v [T,Hkv,D] fp16, rotated in place (q,k); cos/sin [max_pos, rot_dim/2]
 * (fp16 or, when cos_sin_f32 != 0, fp32); positions int64 [T]; slot_mapping int64 [T]
 * (slot = block*block_size + offset; negative = skip the cache write).
 * k_cache/v_cache may be NULL (RoPE only).  interleaved = GPT-J style pairs.       */
void b200_rope_kv_write_f16(void* q, void* k, const void* v, const void* cos, const void* sin,
                            const int64_t* positions, const int64_t* slot_mapping,
                            void* k_cache, void* v_cache, int32_t num_tokens, int32_t num_heads,
                            int32_t num_kv_heads, int32_t head_dim, int32_t rot_dim,
                            int32_t block_size, int32_t interleaved, int32_t cos_sin_f32,
                            int64_t stream);
/* bf16 flavour (the reference's default dtype, utils/mod.rs:1919-1925): q / k / v, the caches and -- unless
 * cos_sin_f32 -- the cos / sin tables are bf16; same arithmetic (fp32 rotation, one rounding on store).            */
void b200_rope_kv_write_bf16(void* q, void* k, const void* v, const void* cos, const void* sin,
                             const int64_t* positions, const int64_t* slot_mapping,
                             void* k_cache, void* v_cache, int32_t num_tokens, int32_t num_heads,
                             int32_t num_kv_heads, int32_t head_dim, int32_t rot_dim,
                             int32_t block_size, int32_t interleaved, int32_t cos_sin_f32,
                             int64_t stream);
/* Same with an FP8 KV cache (`--fp8-kvcache`; kvcache_allocator.rs:188-193,776 allocates the caches as
 * U8 in the same [num_blocks, block_size, Hkv, D] shape): the rotated fp16 K row and the V row are
 * stored as e4m3 bytes (round to nearest even, saturating at +-448, scale 1 -- attention-rs's own
 * format is not source-visible, so this is the library's definition).  q / k are still rotated in
 * place as fp16.                                                                                   */
void b200_rope_kv_write_fp8kv_f16(void* q, void* k, const void* v, const void* cos, const void* sin,
                                  const int64_t* positions, const int64_t* slot_mapping,
                                  void* k_cache, void* v_cache, int32_t num_tokens, int32_t num_heads,
                                  int32_t num_kv_heads, int32_t head_dim, int32_t rot_dim,
                                  int32_t block_size, int32_t interleaved, int32_t cos_sin_f32,
                                  int64_t stream);
/* Cache write only (reshape_and_cache equivalent). */
void b200_kv_write_f16(const void* k, const void* v, void* k_cache, void* v_cache,
                       const int64_t* slot_mapping, int32_t num_tokens, int32_t num_kv_heads,
                       int32_t head_dim, int32_t block_size, int64_t stream);

/* attention_rs::cache::swap_blocks as called for CPU swap (runner.rs:1626-1645: once per layer for K and for
 * V, mapping = HashMap<src block, dst block>) and PD transfer (transfer/mod.rs:260-311): copies whole cache
 * blocks src[pairs[i][0]] -> dst[pairs[i][1]] in ONE launch.  block_bytes = bytes of one block of this cache
 * (block_size * Hkv * D * element size; multiple of 16).  pairs_dev: int64 [num_pairs][2] in DEVICE memory.
 * src / dst: device memory, pinned host memory (read / written by the kernel through UVA) or a peer GPU's
 * cache with peer access enabled.  Blocks must not overlap between src and dst ranges of one call.        */
void b200_swap_blocks(const void* src_cache, void* dst_cache, const int64_t* pairs_dev, int32_t num_pairs,
                      int64_t block_bytes, int64_t stream);

/* ------------------------------------------------- PD (prefill / decode) KV hand-off: wire frames + block movement
 * transfer/mod.rs:82-125 (KVTransferHandle / FinishedPrefillData / TransferMessage), comm.rs:384-410 (u32 LE length +
 * bincode 1.3.1 body) and the data legs of transfer/mod.rs:260-311,370-470.  A KV frame is built in place in a PINNED
 * host buffer: _frame_begin writes every field but the payloads and returns where layer l's K and V bytes go;
 * _export_blocks lets the copy kernel write them there from the paged caches (pairs = (server block, i));
 * _frame_parse gives the same offsets of a received frame and _import_blocks copies (i, local block) out of it.
 * _copy_blocks_peer is the LocalIpc leg: (server block, local block) between two GPUs' caches over NVLink.      */
typedef struct b200_pd_kv_header {
  uint64_t seq_id;
  uint32_t first_token;
  int32_t num_layers;
  uint64_t layer_bytes;        /* bytes of ONE layer's K (= V) payload: num_blocks * block bytes */
  uint64_t num_blocks;
  uint64_t sending_time;       /* ms since the epoch (mod.rs:383-386) */
  uint64_t num_cached_tokens;
} b200_pd_kv_header;
int64_t b200_pd_kv_frame_bytes(int32_t num_layers, int64_t layer_bytes);
int64_t b200_pd_kv_frame_begin(uint8_t* frame, int64_t cap, const b200_pd_kv_header* h, int64_t* k_off,
                               int64_t* v_off);
int32_t b200_pd_kv_frame_parse(const uint8_t* frame, int64_t len, b200_pd_kv_header* h, int64_t* k_off,
                               int64_t* v_off, int32_t max_layers);
/* The LocalIpc flavour of the same message (transfer/mod.rs:77,84-90): per layer a (K, V) pair of
 * CudaIpcMemHandle(64 handle bytes, tensor shape, SerializableDType: U8 0, U32 1, I64 2, BF16 3, F16 4, F32 5, F64 6)
 * and the server's block ids of the sequence (h->num_blocks of them; h->layer_bytes is unused).  k_handles / v_handles
 * are [num_layers][64] bytes as cudaIpcGetMemHandle returned them; every layer shares one shape and dtype.           */
int64_t b200_pd_ipc_frame(uint8_t* out, int64_t cap, const b200_pd_kv_header* h, const uint8_t* k_handles,
                          const uint8_t* v_handles, const uint64_t* shape, int32_t ndim, int32_t dtype,
                          const uint32_t* server_block_ids);
int32_t b200_pd_ipc_frame_parse(const uint8_t* frame, int64_t len, b200_pd_kv_header* h, uint8_t* k_handles,
                                uint8_t* v_handles, int32_t max_layers, uint64_t* shape, int32_t* ndim,
                                int32_t* dtype, uint32_t* server_block_ids, int32_t max_blocks);
/* kind 1 = AvailableTokenResponse(value), 3 = ReleaseKvCache(value); returns the frame length (16) */
int64_t b200_pd_frame_small(uint8_t* out, int64_t cap, int32_t kind, uint64_t value);
/* TransferMessage variant of a frame (0..3), -1 if malformed; *value for kinds 1 and 3 */
int32_t b200_pd_frame_kind(const uint8_t* frame, int64_t len, uint64_t* value);
void b200_pd_export_blocks(const void* const* k_caches, const void* const* v_caches, int32_t num_layers,
                           const int64_t* pairs_dev, int32_t n, int64_t block_bytes, uint8_t* frame,
                           const int64_t* k_off, const int64_t* v_off, int64_t stream);
void b200_pd_import_blocks(void* const* k_caches, void* const* v_caches, int32_t num_layers,
                           const int64_t* pairs_dev, int32_t n, int64_t block_bytes, const uint8_t* frame,
                           const int64_t* k_off, const int64_t* v_off, int64_t stream);
void b200_pd_copy_blocks_peer(const void* const* remote_k, const void* const* remote_v, void* const* local_k,
                              void* const* local_v, int32_t num_layers, const int64_t* pairs_dev, int32_t n,
                              int64_t block_bytes, int64_t stream);
int32_t b200_enable_peer_access(int32_t dev, int32_t peer);

/* ------------------------------------------------- engine <-> runner-process frames of the decode step
 * runner/mod.rs:168-295 (MessageType; u32 LE length + bincode 1.3.1; every frame is answered by ONE ack byte 0x01),
 * core/sequence.rs:52-83 (DecodeSequence), utils/config.rs:504-537 (SamplingParams).  A runner process built on this
 * library reads RunDecode, derives the step metadata (core/runner.rs:1243-1264), runs b200_runner_decode_host and
 * answers RunResponse; KVCacheSwap yields the (src, dst) pairs b200_swap_blocks takes.  MessageType variant indices:
 * RunDecode 4, RunResponse 5, FinishDecode 8, Heartbeat 14, KVCacheSwap 21, KVCacheSwapResponse 22, ClearBlocks 31,
 * ClearBlocksResponse 32, Shutdown 34.  Init / RunPrefill / RunEmbed carry whole Sequence / EngineConfig structs and
 * stay with the Rust host.                                                                                          */
typedef struct b200_wire_sampling {          /* the numeric fields of SamplingParams; has_* = Option is Some */
  int32_t has_temperature, has_max_tokens, ignore_eos, has_top_k, has_top_p, has_frequency_penalty,
      has_presence_penalty, reserved;
  float temperature, top_p, frequency_penalty, presence_penalty;
  int64_t max_tokens, top_k;
} b200_wire_sampling;
int32_t b200_wire_kind(const uint8_t* frame, int64_t len);
int32_t b200_wire_parse_run_decode(const uint8_t* frame, int64_t len, int32_t max_seqs, int32_t max_blocks,
                                   uint64_t* seq_ids, uint32_t* last_tokens, uint64_t* lens,
                                   uint64_t* last_block_tokens, uint32_t* block_table_last, uint32_t* block_tables,
                                   int32_t* num_blocks, b200_wire_sampling* sampling, int32_t* is_prefill);
int64_t b200_wire_frame_run_decode(uint8_t* out, int64_t cap, int32_t n, const uint64_t* seq_ids,
                                   const uint32_t* last_tokens, const uint64_t* lens,
                                   const uint64_t* last_block_tokens, const uint32_t* block_table_last,
                                   const uint32_t* block_tables, int32_t max_blocks, const int32_t* num_blocks,
                                   const b200_wire_sampling* sampling, int32_t is_prefill);
int64_t b200_wire_frame_run_response(uint8_t* out, int64_t cap, const uint32_t* ids, int32_t n);
int32_t b200_wire_parse_run_response(const uint8_t* frame, int64_t len, uint32_t* ids, int32_t cap);
int32_t b200_wire_parse_kv_swap(const uint8_t* frame, int64_t len, int64_t* pairs, int32_t cap, int32_t* swap_in);
int64_t b200_wire_frame_kv_swap(uint8_t* out, int64_t cap, const int64_t* pairs, int32_t n, int32_t swap_in);
int64_t b200_wire_frame_simple(uint8_t* out, int64_t cap, int32_t kind, int32_t payload_bytes, uint64_t value);
/* RunPrefill((Vec<Sequence>, bool)) (variant 3; Sequence as core/sequence.rs:32-50).  The engine side frames the
 * sequences `indices` of its scheduler; the runner side loads such a frame into a scheduler object used as a plain
 * sequence container (its running list is REPLACED; indices[0..n) = 0..n-1) and calls b200_prepare_prefill on it.
 * Fields the mirror does not keep travel as the reference's defaults (created_time 0, the Option fields None) and are
 * skipped on read; first_sampling (may be NULL) receives the SamplingParams of the first sequence, which pick the
 * step's strategy (core/runner.rs:1390-1570).  load returns n, or -1 malformed, -2 more than cap sequences, -3 a
 * sequence prepare_prefill cannot walk (other block size, short block table), -4 a sequence with images.           */
struct b200_scheduler;
int64_t b200_scheduler_frame_run_prefill(const struct b200_scheduler* s, const int32_t* indices, int32_t n,
                                         uint8_t* out, int64_t cap, int32_t is_prefill);
int32_t b200_scheduler_load_run_prefill(struct b200_scheduler* s, const uint8_t* frame, int64_t len,
                                        int32_t* indices, int32_t cap, int32_t* is_prefill,
                                        b200_wire_sampling* first_sampling);
/* Single-Sequence messages of the PD hand-off.  family 0 = runner IPC MessageType (runner/mod.rs:168-249): kind 15
 * TransferPrefill(Sequence), 18 ReceivePrefillResponse((bool, Option<Sequence>)), 23 KvCacheSend((Sequence, u32)),
 * 25 KvCacheReceive(Sequence); family 1 = client <-> PD server TransferMessage (transfer/mod.rs:113-122): kind 0
 * TransferPrefill(Sequence).  `extra` = the bool of kind 18 / the first token of kind 23; index < 0 with kind 18 frames
 * (extra, None).  load puts the sequence into the container as running[0]; returns 1, 0 (kind 18 with None), -1, -4.  */
int64_t b200_scheduler_frame_sequence(const struct b200_scheduler* s, int32_t index, int32_t family, int32_t kind,
                                      uint32_t extra, uint8_t* out, int64_t cap);
int32_t b200_scheduler_load_sequence(struct b200_scheduler* s, const uint8_t* frame, int64_t len, int32_t family,
                                     int32_t* kind, uint32_t* extra);
/* KvCacheReceiveResponse((bool, u32, usize, usize)) (variant 26): success, first token, the server's sending time
 * and the prefix-cache hit length recorded there (transfer/mod.rs:319).  parse returns 0, -1 malformed.            */
int64_t b200_wire_frame_kv_receive_response(uint8_t* out, int64_t cap, int32_t ok, uint32_t first_token, uint64_t sending_time,
                                            uint64_t num_cached_tokens);
int32_t b200_wire_parse_kv_receive_response(const uint8_t* frame, int64_t len, int32_t* ok, uint32_t* first_token,
                                            uint64_t* sending_time, uint64_t* num_cached_tokens);
void b200_wire_decode_metadata(int32_t n, const uint32_t* last_tokens, const uint64_t* lens,
                               const uint64_t* last_block_tokens, const uint32_t* block_table_last,
                               int32_t block_size, uint32_t* input_ids, int64_t* positions, int64_t* slot_mapping,
                               uint32_t* context_lens);

/* ------------------------------------------------- the reference's default-build cache layout ("L1")
 * kvcache_allocator.rs:150-173: without the flashattn / flashinfer features the caches are
 *   K [num_blocks, Hkv, D/x, block_size, x] (x = 16 / element size = 8),   V [num_blocks, Hkv, D, block_size].
 * These entry points read / write that layout directly (block_size 64, 16-bit elements; bf16 != 0 selects the bf16
 * arithmetic): a (block, head) tile is 64*D*2 contiguous bytes, K feeds the MMAs as it lies (8 x 16-byte core
 * matrices), V as a K-major operand.  Argument meaning as for the flash-layout functions of the same name.        */
void b200_kv_write_l1(const void* k, const void* v, void* k_cache, void* v_cache,
                      const int64_t* slot_mapping, int32_t num_tokens, int32_t num_kv_heads,
                      int32_t head_dim, int32_t block_size, int64_t stream);
void b200_rope_kv_write_l1(void* q, void* k, const void* v, const void* cos, const void* sin,
                           const int64_t* positions, const int64_t* slot_mapping,
                           void* k_cache, void* v_cache, int32_t num_tokens, int32_t num_heads,
                           int32_t num_kv_heads, int32_t head_dim, int32_t rot_dim,
                           int32_t block_size, int32_t interleaved, int32_t cos_sin_f32, int32_t bf16,
                           int64_t stream);
void b200_paged_attn_decode_l1(void* out, const void* q, const void* k_cache,
                               const void* v_cache, const uint32_t* block_tables,
                               const uint32_t* context_lens, int32_t batch, int32_t num_heads,
                               int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                               int32_t max_blocks_per_seq, int32_t num_blocks, float scale,
                               float softcap, int32_t window, void* workspace, int32_t bf16, int64_t stream);
void b200_attn_prefill_l1(void* out, const void* q, const void* k_cache, const void* v_cache,
                          const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                          const uint32_t* block_tables, int32_t batch, int32_t num_heads,
                          int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                          int32_t max_blocks_per_seq, int32_t num_blocks, int32_t max_seqlen_q,
                          int32_t num_tokens, int32_t mode, float scale, int32_t bf16, int64_t stream);

/* ------------------------------------------------- paged attention, decode
 * Replaces the decode branch of PagedAttention::forward (attention.rs:808-820).
 * out/q [B,H,D] fp16; block_tables u32 [B, max_blocks_per_seq] (zero padded);
 * context_lens u32 [B] (0 => row skipped, out row zeroed).  softcap <= 0 disables;
 * window <= 0 disables sliding window.  head_dim in {64,128}, block_size == 64,
 * H/Hkv <= 16.  Per-sequence lengths are read on the device (graph safe).  `workspace`:
 * b200_paged_attn_workspace_bytes() bytes, zeroed once by the caller (arrival counters;
 * the kernel leaves them zeroed).                                                    */
void b200_paged_attn_decode_f16(void* out, const void* q, const void* k_cache,
                                const void* v_cache, const uint32_t* block_tables,
                                const uint32_t* context_lens, int32_t batch, int32_t num_heads,
                                int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                                int32_t max_blocks_per_seq, int32_t num_blocks, float scale,
                                float softcap, int32_t window, void* workspace, int64_t stream);
/* bf16 flavour: q / out and both caches are bf16; S = Q K^T and P V run as bf16 x bf16 -> fp32 MMAs (P rounded
 * to bf16), softmax in fp32.  Same workspace.                                                                      */
void b200_paged_attn_decode_bf16(void* out, const void* q, const void* k_cache,
                                 const void* v_cache, const uint32_t* block_tables,
                                 const uint32_t* context_lens, int32_t batch, int32_t num_heads,
                                 int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                                 int32_t max_blocks_per_seq, int32_t num_blocks, float scale,
                                 float softcap, int32_t window, void* workspace, int64_t stream);
int64_t b200_paged_attn_workspace_bytes(int32_t batch, int32_t num_heads, int32_t head_dim,
                                        int32_t max_blocks_per_seq);
/* Decode attention over an FP8 (e4m3, scale 1) KV cache: same arguments, k_cache / v_cache are
 * u8 [num_blocks, 64, Hkv, 128]; half the HBM bytes per step.  head_dim must be 128.             */
void b200_paged_attn_decode_fp8kv_f16(void* out, const void* q, const void* k_cache,
                                      const void* v_cache, const uint32_t* block_tables,
                                      const uint32_t* context_lens, int32_t batch, int32_t num_heads,
                                      int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                                      int32_t max_blocks_per_seq, int32_t num_blocks, float scale,
                                      float softcap, int32_t window, void* workspace, int64_t stream);

/* ------------------------------------------------- paged attention, prefill (varlen causal)
 * Replaces the prefill branch of PagedAttention::forward (attention.rs:808-820) with the
 * metadata of prepare_prefill (runner.rs:978-1241).  q/out [T,H,D] fp16 (T = cu_seqlens_q[B]);
 * keys/values are read from the paged cache through block_tables for the whole context
 * [0, context_lens[b]) -- call b200_rope_kv_write_f16 for this step's tokens first.
 * context_lens may be NULL (no cached prefix: context = query length).  H/Hkv in {1,2,4,8}. */
void b200_attn_prefill_f16(void* out, const void* q, const void* k_cache, const void* v_cache,
                           const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                           const uint32_t* block_tables, int32_t batch, int32_t num_heads,
                           int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                           int32_t max_blocks_per_seq, int32_t num_blocks, int32_t max_seqlen_q,
                           float scale, int64_t stream);

/* Same, with the row count of q / out (num_tokens = cu_seqlens_q[batch], which the tcgen05 kernel's q
 * tensor map needs as a HOST value) and an explicit implementation: mode -1 = default (tcgen05 for
 * head_dim 128, env B200_PREFILL_ATTN), 0 = mma.sync kernel, 1 = tcgen05, 2 = tcgen05 bring-up switch. */
void b200_attn_prefill_ex_f16(void* out, const void* q, const void* k_cache, const void* v_cache,
                              const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                              const uint32_t* block_tables, int32_t batch, int32_t num_heads,
                              int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                              int32_t max_blocks_per_seq, int32_t num_blocks, int32_t max_seqlen_q,
                              int32_t num_tokens, int32_t mode, float scale, int64_t stream);
/* bf16 flavour (q / out / caches bf16; tcgen05 kind::f16 with bf16 operand formats, or the bf16 mma.sync kernel). */
void b200_attn_prefill_ex_bf16(void* out, const void* q, const void* k_cache, const void* v_cache,
                               const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                               const uint32_t* block_tables, int32_t batch, int32_t num_heads,
                               int32_t num_kv_heads, int32_t head_dim, int32_t block_size,
                               int32_t max_blocks_per_seq, int32_t num_blocks, int32_t max_seqlen_q,
                               int32_t num_tokens, int32_t mode, float scale, int64_t stream);

/* ------------------------------------------------- glue kernels (others.rs, mlp.rs, llama.rs) */
void b200_rmsnorm_f16(void* out, const void* x, const void* weight, int32_t num_tokens,
                      int32_t hidden, float eps, int64_t stream);
/* residual += x (fp16 rounding, as llama.rs:126-130); out = rmsnorm(residual) * weight */
void b200_add_rmsnorm_f16(void* out, void* residual, const void* x, const void* weight,
                          int32_t num_tokens, int32_t hidden, float eps, int64_t stream);
void b200_silu_mul_f16(void* out, const void* gate_up, int32_t num_tokens, int32_t inter,
                       int64_t stream);
/* bf16 flavours of the three (x / weight / residual / out bf16, fp32 math, the residual add rounds to bf16).
 * b200_embedding_f16, b200_gather_rows_f16, b200_kv_write_f16 and b200_swap_blocks move 16-bit elements without
 * arithmetic and serve bf16 tensors as they are.                                                                */
void b200_rmsnorm_bf16(void* out, const void* x, const void* weight, int32_t num_tokens,
                       int32_t hidden, float eps, int64_t stream);
void b200_add_rmsnorm_bf16(void* out, void* residual, const void* x, const void* weight,
                           int32_t num_tokens, int32_t hidden, float eps, int64_t stream);
void b200_silu_mul_bf16(void* out, const void* gate_up, int32_t num_tokens, int32_t inter,
                        int64_t stream);
void b200_embedding_f16(void* out, const void* table, const uint32_t* ids, int32_t num_tokens,
                        int32_t hidden, int32_t vocab, int64_t stream);
void b200_gather_rows_f16(void* out, const void* x, const uint32_t* rows, int32_t num_rows,
                          int32_t hidden, int64_t stream);
void b200_argmax_f32(uint32_t* out_ids, const float* logits, int32_t batch, int32_t vocab,
                     int64_t stream);
void b200_add_bias_f16(void* x, const void* bias, int32_t num_tokens, int32_t n, int64_t stream);

/* ------------------------------------------------- sampling (logits_processor.rs, runner.rs:1390-1570)
 * Device replacement of attention_rs::sampler::Sampler::sample_cuda (logits_processor.rs:226-229):
 * full-vocabulary softmax(logits / temperature) -> top_k (1..256) -> top-p cut on the
 * un-renormalised top-k probabilities -> multinomial (top_k = 0: Sampling::All, the whole vocabulary, no
 * cut); out_ids u32 [batch].  `seed_dev` points to
 * ONE u64 in device memory (the step seed, LogitsProcessor's rng.next_u64()), so a captured graph
 * changes it with a copy.  Row b draws u = f(seed, b) (this library's definition; the reference
 * kernel's is not source-visible).  Greedy (Sampling::ArgMax) is b200_argmax_f32.          */
void b200_sample_topk_topp_f32(uint32_t* out_ids, const float* logits, int32_t batch, int32_t vocab,
                               int32_t top_k, float top_p, float temperature,
                               const uint64_t* seed_dev, int64_t stream);
/* apply_batch_repeat_penalty (logits_processor.rs:308-343): context u32 [batch, context_cap] holds
 * each row's penalty window (the caller applies the "last 128 tokens once more than 128 exist"
 * rule of runner.rs:1522-1533), context_lens i32 [batch].  In place on fp32 logits.        */
void b200_apply_penalties_f32(float* logits, int32_t batch, int32_t vocab, const uint32_t* context,
                              const int32_t* context_lens, int32_t context_cap,
                              float frequency_penalty, float presence_penalty, int64_t stream);
/* LogitsProcessor::get_strategy + the (k, p, t) of sample_with_strategy (logits_processor.rs:48-70,
 * 208-216).  has_* = 0 is None.  Returns 0 ArgMax, 1 All, 2 TopK, 3 TopP, 4 TopKThenTopP.       */
int32_t b200_sampling_strategy(int32_t has_temperature, float temperature, int32_t has_top_k,
                               int64_t top_k, int32_t has_top_p, float top_p, int32_t* k, float* p,
                               float* t);
/* rand::rngs::StdRng::seed_from_u64 (logits_processor.rs:29-30): ChaCha12 keyed by the PCG32
 * expansion of the seed; next_u64 is the per-step kernel seed (logits_processor.rs:222-225).  */
typedef struct b200_rng b200_rng;
b200_rng* b200_rng_new(uint64_t seed);
void b200_rng_free(b200_rng*);
uint32_t b200_rng_next_u32(b200_rng*);
uint64_t b200_rng_next_u64(b200_rng*);

/* ------------------------------------------------- host side: block manager / scheduler
 * C++ mirror of src/core/{sequence,block_manager,scheduler}.rs and the input
 * preparation of src/core/runner.rs:952-1388.  Handles are opaque.               */
typedef struct b200_scheduler b200_scheduler;
b200_scheduler* b200_scheduler_new(int32_t num_blocks, int32_t block_size, int32_t max_num_seqs,
                                   int32_t max_num_batched_tokens, int32_t chunk_size,
                                   const uint32_t* eos_ids, int32_t num_eos);
void b200_scheduler_free(b200_scheduler*);
/* returns seq id (scheduler.rs:186-192) */
int64_t b200_scheduler_add(b200_scheduler*, const uint32_t* tokens, int32_t num_tokens,
                           int32_t max_tokens);
/* SamplingParams.stop_token_ids of a sequence that is still WAITING (id from add): num_stops token sequences
 * back to back in stop_tokens, lengths in stop_lens.  postprocess() then finishes the sequence when the sampled
 * token completes one of them (scheduler.rs:1309-1341: the head must equal the tail of the GENERATED tokens;
 * the stop token itself is not appended, like EOS).  Returns 0, -1 if the id is not waiting.             */
int32_t b200_scheduler_set_stop_sequences(b200_scheduler*, int64_t seq_id, const uint32_t* stop_tokens,
                                          const int32_t* stop_lens, int32_t num_stops);
/* schedule(): writes indices into `running` (<= cap); returns count, *is_prefill set.
 * Returns -1 on error (e.g. out of blocks).  (scheduler.rs:200-380)               */
int32_t b200_scheduler_schedule(b200_scheduler*, int32_t* indices, int32_t cap,
                                int32_t* is_prefill);
/* filter_prefill_finished (scheduler.rs:718-785): returns number finished; writes the
 * positions within `indices` (out_pos) and the new running indices (out_idx).      */
int32_t b200_scheduler_filter_prefill_finished(b200_scheduler*, const int32_t* indices,
                                               int32_t n, int32_t* out_pos, int32_t* out_idx);
void b200_scheduler_postprocess(b200_scheduler*, const int32_t* indices, int32_t n,
                                const uint32_t* tokens);
void b200_scheduler_clear_finished(b200_scheduler*);
int32_t b200_scheduler_num_running(const b200_scheduler*);
int32_t b200_scheduler_num_waiting(const b200_scheduler*);
int32_t b200_scheduler_num_free_blocks(const b200_scheduler*);
/* Prefix cache (src/core/prefix_cache.rs; block_manager.rs:179-221,275-299,346-442,552-604,
 * 657-672; scheduler.rs:60-104,288-337,617-620,1167-1175).  enable: max_tokens >= 0 is
 * `prefix_cache_max_tokens`, < 0 the default 65 % of the blocks; returns the capacity in blocks
 * (0 = disabled, as build_prefix_cache_config does).  Once enabled, allocate() shares the cached
 * full blocks of a matching prompt prefix (never the whole prompt), postprocess() inserts a
 * finished sequence's full blocks before dropping its references, and schedule() evicts 10 % of
 * the cache when a sequence cannot append or usage is over 95 %.  hash_block is the chain hash
 * (Rust DefaultHasher = SipHash-1-3, zero key, over parent u64 | len usize | tokens u32 LE).      */
int32_t b200_scheduler_enable_prefix_cache(b200_scheduler*, int64_t max_tokens);
int32_t b200_scheduler_prefix_cache_blocks(const b200_scheduler*);
int32_t b200_scheduler_evict_prefix_cache_blocks(b200_scheduler*, int32_t num_blocks);
int32_t b200_scheduler_block_ref_count(const b200_scheduler*, int32_t block_id);
/* free_block_ids in pop order; returns the count, copies up to cap */
int32_t b200_scheduler_free_block_ids(const b200_scheduler*, uint32_t* out, int32_t cap);
uint64_t b200_prefix_hash_block(uint64_t parent_hash, const uint32_t* tokens, int32_t n);
/* CPU swap of running sequences (block_manager.rs:69-78,255-272,878-1000; scheduler.rs:303-337,830-954), the
 * bookkeeping: enable with the number of CPU blocks (kvcache plan: num_cpu_blocks).  schedule() then swaps the
 * OLDEST sequence that cannot append out to CPU blocks when there is no prefix cache left to evict (and
 * another sequence keeps running), and brings ONE swapped sequence back per call once it has cooled down
 * 5 s, nothing is preempted and the cache has room.  The reference reads the wall clock; here the host sets it
 * (set_time_ms) before schedule().  The block copies themselves are NOT done here: after schedule() drain
 * pop_swap_op -- (src, dst) block pairs, GPU->CPU or CPU->GPU -- and run b200_swap_blocks per layer cache
 * before the step's forward.  Session ("Cached") sequences are out of scope.                              */
void b200_scheduler_enable_cpu_swap(b200_scheduler*, int32_t num_cpu_blocks);
void b200_scheduler_set_time_ms(b200_scheduler*, int64_t now_ms);
int32_t b200_scheduler_num_swapped(const b200_scheduler*);
int64_t b200_scheduler_swapped_seq_id(const b200_scheduler*, int32_t i);
int32_t b200_scheduler_free_cpu_block_ids(const b200_scheduler*, uint32_t* out, int32_t cap);
int32_t b200_scheduler_pop_swap_op(b200_scheduler*, int64_t* pairs, int32_t cap_pairs, int32_t* swap_in);
/* inspect a running sequence: returns token count; copies up to cap entries */
int32_t b200_scheduler_seq_info(const b200_scheduler*, int32_t running_idx, int64_t* seq_id,
                                int32_t* num_cached_tokens, int32_t* status,
                                int32_t* num_output_tokens);
int32_t b200_scheduler_seq_block_table(const b200_scheduler*, int32_t running_idx,
                                       uint32_t* out, int32_t cap);
int32_t b200_scheduler_seq_tokens(const b200_scheduler*, int32_t running_idx, uint32_t* out,
                                  int32_t cap);

/* prepare_decode (runner.rs:1243-1388) + prepare_block_tables (runner.rs:952-974).
 * Host output buffers sized [n] / [n * max_blocks_cap]; returns max_blocks (row
 * stride used) or -1 if max_blocks_cap is too small.  *max_context_len set.        */
int32_t b200_prepare_decode(const b200_scheduler*, const int32_t* indices, int32_t n,
                            uint32_t* input_ids, int64_t* positions, int64_t* slot_mapping,
                            uint32_t* context_lens, uint32_t* block_tables,
                            int32_t max_blocks_cap, int32_t* max_context_len);
/* prepare_prefill (runner.rs:978-1241).  Returns total tokens T (or -1 if cap too
 * small).  cu_seqlens_* are [n+1].  *has_context != 0 when block_tables /
 * context_lens were produced (some sequence has cached KV).                        */
int32_t b200_prepare_prefill(const b200_scheduler*, const int32_t* indices, int32_t n,
                             int32_t token_cap, uint32_t* input_ids, int64_t* positions,
                             int64_t* slot_mapping, uint32_t* cu_seqlens_q,
                             uint32_t* cu_seqlens_k, uint32_t* context_lens,
                             uint32_t* block_tables, int32_t max_blocks_cap,
                             int32_t* max_blocks, int32_t* max_seqlen_q, int32_t* max_seqlen_k,
                             int32_t* max_context_len, int32_t* has_context);

/* ------------------------------------------------- KV-cache planning (host, integer)
 * Mirror of KVCacheAllocator::{per_block_bytes, plan_allocation, auto_decide_params}
 * (src/utils/kvcache_allocator.rs:447-468, 553-612, 616-707) for dense (non-MLA, non-hybrid)
 * models.  `available_bytes` is what get_rank_available_memory returns: free * kv_fraction,
 * minimum over ranks.  user_max_num_seqs / user_max_model_len <= 0 mean "auto-decide".
 * Returns 0, or -1 for InvalidConfiguration, -2 for InsufficientGpuMemory.             */
typedef struct b200_kvcache_plan {
  int64_t per_block_bytes, num_gpu_blocks, num_cpu_blocks, max_num_seqs, max_model_len;
  int64_t kvcache_memory_bytes, max_num_batched_tokens;
} b200_kvcache_plan;
int32_t b200_kvcache_plan_allocation(int64_t available_bytes, int32_t num_layers,
                                     int32_t num_kv_heads, int32_t head_dim, int32_t num_shards,
                                     int32_t block_size, int32_t dtype_size,
                                     int64_t config_model_len, int64_t user_max_num_seqs,
                                     int64_t user_max_model_len, float cpu_mem_fold,
                                     b200_kvcache_plan* out);

/* ------------------------------------------------- model runner (decode step)
 * C++ mirror of ModelRunner::run for the decode branch (runner.rs:743-896) over
 * LLaMaForCausalLM::forward_inner (llama.rs:269-321): every launch of one decode
 * step, optionally captured into CUDA graphs per batch bucket (graph.rs:370-377).  */
typedef struct b200_model_config {
  int32_t hidden, num_layers, num_heads, num_kv_heads, head_dim, inter, vocab;
  int32_t bits, group_size, qfmt;      /* bits = 16 => dense fp16 weights              */
  int32_t block_size, num_blocks, max_blocks_per_seq, max_batch, max_pos;
  int32_t qkv_bias;                    /* Qwen2: q/k/v bias                            */
  int32_t cos_sin_f32;
  float rms_eps, attn_scale;
  int32_t tp_rank, tp_size;            /* shapes above are the LOCAL (per-rank) shard  */
  int32_t max_prefill_tokens;          /* 0 => decode only; else tokens per prefill step */
  int32_t kv_fp8;                      /* EngineConfig.fp8_kvcache: caches are e4m3 bytes (head_dim 128) */
} b200_model_config;

typedef struct b200_layer_weights {
  const void *input_norm, *post_norm;                 /* fp16 [hidden]                  */
  const void *qkv_w, *qkv_s, *qkv_z, *qkv_bias;       /* fused q|k|v along N            */
  const void *o_w, *o_s, *o_z;
  const void *gate_up_w, *gate_up_s, *gate_up_z;      /* fused gate|up along N          */
  const void *down_w, *down_s, *down_z;
  void *k_cache, *v_cache;
} b200_layer_weights;

typedef struct b200_runner b200_runner;
b200_runner* b200_runner_new(const b200_model_config* cfg);
void b200_runner_free(b200_runner*);
void b200_runner_set_layer(b200_runner*, int32_t layer, const b200_layer_weights* w);
void b200_runner_set_globals(b200_runner*, const void* embed, const void* final_norm,
                             const void* lm_head, const void* cos, const void* sin);
int64_t b200_runner_workspace_bytes(const b200_runner*);
void b200_runner_set_workspace(b200_runner*, void* workspace, int64_t bytes);
/* all-reduce hook for tensor parallelism: called on the stream after o_proj / down_proj
 * with (buf, count_halfs, user, stream); NULL => single GPU (distributed.rs:438-454).  */
typedef void (*b200_allreduce_fn)(void* buf, int64_t count, void* user, int64_t stream);
void b200_runner_set_allreduce(b200_runner*, b200_allreduce_fn fn, void* user);
/* One decode step from DEVICE inputs; logits (fp32 [B, vocab]) and/or greedy token
 * ids (u32 [B]) are written to device buffers (either may be NULL).                */
void b200_runner_decode_device(b200_runner*, const uint32_t* input_ids, const int64_t* positions,
                               const int64_t* slot_mapping, const uint32_t* block_tables,
                               const uint32_t* context_lens, int32_t batch, float* logits,
                               uint32_t* out_ids, int64_t stream);
/* ModelRunner::run equivalent for decode: HOST inputs (pinned), copies H2D, runs the
 * step (graph replay when captured for this bucket), copies token ids D2H and
 * synchronises the stream.  Returns 0 on success.                                   */
int32_t b200_runner_decode_host(b200_runner*, const uint32_t* input_ids,
                                const int64_t* positions, const int64_t* slot_mapping,
                                const uint32_t* block_tables, int32_t max_blocks,
                                const uint32_t* context_lens, int32_t batch,
                                uint32_t* out_ids_host, int64_t stream);
/* One prefill step (ModelRunner::run, prefill branch, runner.rs:743-896 with the metadata of
 * prepare_prefill): DEVICE inputs; T = num_tokens rows.  block_tables must cover every
 * sequence (keys are read from the paged cache after this step's KV write); context_lens may
 * be NULL when nothing is cached.  last_rows u32 [num_seqs] = cu_seqlens_q[1:] - 1
 * (llama.rs:306-310).  logits f32 [num_seqs, vocab] and/or greedy ids are written.        */
void b200_runner_prefill_device(b200_runner*, const uint32_t* input_ids, const int64_t* positions,
                                const int64_t* slot_mapping, const uint32_t* cu_seqlens_q,
                                const uint32_t* context_lens, const uint32_t* block_tables,
                                const uint32_t* last_rows, int32_t num_seqs, int32_t num_tokens,
                                int32_t max_seqlen_q, int32_t max_blocks, float* logits,
                                uint32_t* out_ids, int64_t stream);
/* Capture CUDA graphs for the given batch buckets (graph.rs:448-690). 0 on success. */
int32_t b200_runner_capture(b200_runner*, const int32_t* buckets, int32_t num_buckets,
                            int64_t stream);
int64_t b200_runner_launches_per_step(const b200_runner*);
/* Sampling of the decode / prefill steps: top_k == 0 => greedy argmax (default); otherwise the
 * device sampler above with these (k, p, t) (the strategy cached at prefill, runner.rs:1402-1510).
 * b200_runner_set_step_seed copies the step seed into the runner's device slot on `stream`
 * (call once per step before b200_runner_decode_host / _device; graph-replay safe).          */
void b200_runner_set_sampling(b200_runner*, int32_t top_k, float top_p, float temperature);
void b200_runner_set_step_seed(b200_runner*, uint64_t seed, int64_t stream);
/* The same from b200_sampling_strategy's result (0 ArgMax, 1 All, 2 TopK, 3 TopP, 4 TopKThenTopP) and its
 * (k, p, t): Sampling::All (temperature only, logits_processor.rs:199-207) draws from the whole vocabulary.
 * Any change of strategy or parameters drops the captured graphs (the values are kernel arguments).  0 / -1. */
int32_t b200_runner_set_sampling_strategy(b200_runner*, int32_t strategy, int32_t k, float p, float t);

/* ------------------------------------------------- engine step (engine.rs:1693-1757)
 * prepare_step -> run_forward -> finish_step of a DECODE batch in one native call: schedule(),
 * prepare_decode into pinned staging owned by the handle, b200_runner_decode_host, postprocess,
 * clear_finished.  b200_engine_step returns the number of sequences decoded (running indices at schedule
 * time, sequence ids and new tokens in the three output arrays, each sized >= max(max_batch, 5), any may be
 * NULL); 0 = nothing schedulable; -2 = the scheduler produced a PREFILL batch: *num_prefill indices are in
 * indices_out and the caller runs that step (b200_prepare_prefill / b200_runner_prefill_device /
 * filter_prefill_finished / postprocess); -1 = error.  The handle borrows the scheduler and the runner. */
typedef struct b200_engine b200_engine;
b200_engine* b200_engine_new(b200_scheduler* sched, b200_runner* runner, int32_t max_batch,
                             int32_t max_blocks_per_seq);
void b200_engine_free(b200_engine*);
/* CPU swap (scheduler.rs:303-337,830-954; runner.rs:1626-1645): per layer the GPU K / V caches and their
 * pinned-host mirrors.  b200_engine_step then runs every block copy schedule() queued BEFORE the step's
 * forward (a victim's GPU blocks may already belong to a sequence of the same batch); with swapping enabled
 * on the scheduler and no caches registered the step fails instead of decoding stale pages.  0 / -1.       */
int32_t b200_engine_set_swap_caches(b200_engine*, int32_t num_layers, void* const* gpu_k, void* const* gpu_v,
                                    void* const* cpu_k, void* const* cpu_v, int64_t block_bytes);
/* Seed of the sampling stream (StdRng::seed_from_u64, logits_processor.rs:29-30): once set, every decode step
 * pushes rng.next_u64() to the runner's device seed before the forward (logits_processor.rs:222-225).      */
void b200_engine_set_seed(b200_engine*, uint64_t seed);
int32_t b200_engine_step(b200_engine*, int32_t* indices_out, int64_t* seq_ids_out, uint32_t* tokens_out,
                         int32_t* num_prefill, int64_t stream);

/* ------------------------------------------------- tensor-parallel communicator
 * One process per GPU (runner/runner.rs:73-240).  NCCL communicator from a 128-byte unique id
 * (engine.rs:263, runner/mod.rs:33-58) + an optional one-shot NVLink all-reduce over
 * cudaIpc-mapped peer buffers for messages <= 1 MiB.  b200_allreduce_f16 is the in-place
 * equivalent of AllReduce::cuda_fwd (distributed.rs:335-395).                       */
typedef struct b200_comm b200_comm;
int32_t b200_nccl_unique_id(uint8_t* out128);
b200_comm* b200_comm_init_rank(const uint8_t* id128, int32_t rank, int32_t world);
int32_t b200_comm_enable_oneshot(b200_comm*, int64_t stream);
void b200_comm_set_force_nccl(b200_comm*, int32_t force);
void b200_comm_free(b200_comm*);
void b200_allreduce_f16(b200_comm*, void* buf, int64_t count, int64_t stream);
int32_t b200_comm_rank(const b200_comm*);
int32_t b200_comm_world(const b200_comm*);
/* the runner all-reduces o_proj / down_proj outputs through this communicator.  With the one-shot
 * path enabled, decode steps (batch <= 64) run the FUSED form: the row-parallel GEMM's tile
 * finalisers store their partial straight into every rank's receive buffer over NVLink and one
 * kernel waits for all ranks' tiles, sums them in rank order, adds the residual and applies the
 * next RMSNorm (3 launches and an NVLink round trip fewer per all-reduce; bit-identical to the
 * unfused GEMM -> all-reduce -> add+norm).  b200_runner_set_tp_fused: -1 env B200_TP_FUSED
 * (default on), 0 off, 1 on.                                                            */
void b200_runner_set_comm(b200_runner*, b200_comm*);
void b200_runner_set_tp_fused(b200_runner*, int32_t on);


/* ------------------------------------------------- hybrid decoders with an fp32 residual stream
 * Decoders whose layers pick one of several sequence mixers -- latent (compressed-KV) attention with an optional
 * sliding window and softmax sink, the gated delta rule, the SSD scan of Mamba-2 -- next to a routed mixture of
 * experts with a shared expert, both reading ONE norm of the stream (parallel layer).  Residual, norms, softmax,
 * router and recurrent state are fp32; `dt` picks the dtype of every matrix-product operand and of the latent cache
 * (0 = bf16, 1 = fp32, true fp32 products).  A step is a ragged batch: sequence b brings rows [cu[b], cu[b+1]) that
 * end at position context_lens[b] - 1, so prompt portions of any length and single decoded tokens mix freely.
 * Kernels: csrc/seq_norms.cu, latent_attn.cu, linear_recurrence.cu, moe.cu; launch plan: csrc/host/hybrid_runner.cpp. */
#define B200_MIXER_LATENT_ATTN 0
#define B200_MIXER_DELTA_RULE 1
#define B200_MIXER_SSD 2
#define B200_MIXER_WINDOW_ATTN 3            /* softmax attention, grouped K / V heads, paged K and V caches */
#define B200_MIXER_DECAY_ATTN 4             /* linear attention with a decayed state (fixed or per-channel decay) */
/* Layer layouts.  PARALLEL: mixer and feed-forward read ONE norm of the stream and add into it.  SANDWICH: every
 * sublayer has a norm before and after it: x += post_norm(mixer(norm(x))), then x += ff_post_norm(ff(ff_norm(x))).
 * In all layouts a layer may have a SIDE mixer (b200_hybrid_set_layer_side) that reads the same normed input; the mixers'
 * outputs are summed, each times its out_scale.                                                                   */
#define B200_LAYOUT_PARALLEL 0
#define B200_LAYOUT_SANDWICH 1
/* POSTNORM: every sublayer's result is normed before it joins the stream and nothing is normed on the way in:
 * x += post_norm(mixer(x)), then x += ff_post_norm(ff(x)), the inputs being x rounded to the operand dtype.  The feed-forward is the routed experts (with their
 * shared expert) when experts > 0, else the dense gated feed-forward (shared_ff), as in SANDWICH.                  */
#define B200_LAYOUT_POSTNORM 2
/* PRENORM: the sublayers follow one another, each behind its own norm of the stream and each added to it times a
 * factor: x += out_scale * mixer(norm(x)), then x += ff_scale * ff(ff_norm(x)).  The feed-forward is chosen as in
 * POSTNORM.  The mixer's input may pass a token shift first (shift_w), and the layer may close with an average over
 * the results of all layers so far (depth_w); both are described at b200_hybrid_layer.                              */
#define B200_LAYOUT_PRENORM 3
/* Norm kinds of the stream norms (norm_kind of a layer, final_norm_kind of the model).  RMS: x / sqrt(mean(x^2) + eps)
 * * (offset + w).  DYNTANH: tanh(alpha * x) * w + b, element by element, no mean or variance (eps is not used).   */
#define B200_NORM_RMS 0
#define B200_NORM_DYNTANH 1

void b200_resid_rmsnorm(void* out, const float* x, const float* w, int32_t num_tokens, int32_t width, float eps,
                        float w_offset, int32_t dt, int64_t stream);
/* gate_act: 0 SiLU, 1 sigmoid; w may be NULL (no weight) */
void b200_gated_group_norm(void* out, const float* y, int32_t ldy, const float* gate, int32_t ldg, const float* w,
                           int32_t w_period, int32_t num_tokens, int32_t channels, int32_t group, float eps,
                           int32_t gate_first, int32_t gate_act, int32_t dt, int64_t stream);
/* x fp32 [T, width] += y / sqrt(mean(y^2) + eps) * (w_offset + w): the norm after a sublayer and its residual sum */
void b200_resid_add_rmsnorm(float* x, const float* y, const float* w, int32_t num_tokens, int32_t width, float eps,
                            float w_offset, int64_t stream);
/* A norm of the stream with an optional token shift behind it.  n[t] = norm(x[t]) (kind B200_NORM_*; bias may be NULL);
 * with shift_w (fp32 [width]): out[t] = n[t] + (n[t-1] - n[t]) * shift_w, n[t-1] being the un-shifted norm of the
 * sequence's previous token: the row before in this step, or shift_state[slot] (fp32 [slots, width]) for the first row
 * of a portion, or zeros at position 0.  The un-shifted norm of a sequence's last row becomes its shift_state.  out has
 * dtype dt.  rows (u32, may be NULL; not with a shift): the stream rows to norm, out row r = norm(x[rows[r]]).       */
void b200_stream_norm(void* out, const float* x, const float* w, const float* bias, float alpha, int32_t kind,
                      float eps, float w_offset, const uint32_t* rows, const float* shift_w, float* shift_state,
                      const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                      int32_t num_seqs, int32_t num_tokens, int32_t width, int32_t dt, int64_t stream);
/* out fp32 [n] = sum over j < count of w[j] * hist[j * stride + i]: a weighted sum of `count` stored streams (w fp32
 * [count], on the device).  out may be one of the streams' successors but none of the `count` inputs.              */
void b200_depth_mix(float* out, const float* hist, int64_t stride, const float* w, int32_t count, int64_t n,
                    int64_t stream);
/* Windowed softmax attention with grouped K / V heads (csrc/window_attn.cu).  proj fp32 [T, ld] = [q: heads x dim |
 * k: kv_heads x dim | v: kv_heads x vdim | ...]; bias fp32 over q | k | v or NULL; q_norm_w / k_norm_w fp32 over the WHOLE
 * q / k projection or NULL (no norm); the first rot_dims entries of every q and k head are rotated as interleaved
 * pairs by position * rot_freq[i] (f64 [rot_dims / 2]).  Writes q_out fp32 [T, heads, dim] and the cache rows
 * k_cache [num_blocks, 64, kv_heads, dim], v_cache [num_blocks, 64, kv_heads, vdim] (dtype dt) at slot_mapping[t].  */
void b200_window_attn_prep(const float* proj, int32_t ld, const float* bias, const float* q_norm_w,
                           const float* k_norm_w, const double* rot_freq, const int64_t* positions,
                           const int64_t* slot_mapping, float* q_out, void* k_cache, void* v_cache, int32_t num_tokens,
                           int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t rot_dims, float eps,
                           int32_t dt, int64_t stream);
/* out [T, heads, vdim] (dtype dt).  Position i sees j <= i with i - j < window or j < keep_first (window <= 0: all);
 * score = cap * tanh(q.k * scale / cap) (softcap <= 0: no cap); sink fp32 [heads] joins the denominator (NULL: none);
 * gate fp32 [T, ld_gate]: head h's output is multiplied by sigmoid(gate[t, h]) (NULL: none).  workspace (may be NULL):
 * b200_window_attn_workspace_bytes() bytes; with it steps of few rows split a row's keys over several blocks.     */
void b200_window_attn(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                      const float* gate, int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                      const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens,
                      int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t window, int32_t keep_first,
                      float scale, float softcap, int32_t dt, void* workspace, int64_t stream);
int64_t b200_window_attn_workspace_bytes(int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t vdim,
                                         int32_t window, int32_t keep_first);
/* the same for a value cache of v_heads heads (b200_attn_options.v_heads) */
int64_t b200_window_attn_workspace_bytes_ex(int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t v_heads,
                                            int32_t vdim, int32_t window, int32_t keep_first);
/* Further options of the two calls above (a zeroed struct = the plain calls).
 *   head_norm   != 0: q_norm_w / k_norm_w are fp32 [dim], shared by all heads, and every head is RMS-normed on its own
 *   v_from_k    != 0: the projection row has no v block; the value row is a copy of the raw key row (bias added, before
 *                     the key norm and rotation), so vdim == dim
 *   q_temp_coef, q_temp_every: every > 0: the query at position p is multiplied by
 *                     1 + coef * ln(floor((p + 1) / every) + 1)                       (after norm and rotation)
 *   dist_slopes fp32 [heads] or NULL: the score of query position i against key position j is lowered by slope_h * (i - j)
 *                     (after scale and cap)
 *   gate_elems  != 0: the output gate has heads x vdim logits per token (one per output element) instead of heads   */
typedef struct b200_attn_options {
  int32_t head_norm, v_from_k, q_temp_every, gate_elems;
  float q_temp_coef;
  const float* dist_slopes;
  /* (fields below: zero = off)
   *   rot_half    != 0: rotary pairs are (i, i + rot_dims / 2) (the two halves of the rotated part) instead of (2i, 2i+1)
   *   rot_mag     != 0: cos and sin of the q / k rotation are multiplied by it (0 reads as 1)
   *   v_rot_freq  f64 [vdim / 2] or NULL: the value row of position j is rotated by j * v_rot_freq[m] over all of vdim
   *                     (same pair layout as rot_half says) before it is cached; b200_attn_finish turns a head's output
   *                     back by its own position
   *   v_heads     > 0: the value cache has v_heads heads and key head g reads value head g % v_heads (several score
   *                     maps over one set of values: the maps' key heads are laid out map after map); 0: kv_heads
   *   chunk       > 0: position i sees j <= i only if floor(i / chunk) == floor(j / chunk) (true positions, however a prompt is cut)
   *   out_f32     != 0: the attention writes fp32 whatever dt says (for b200_attn_finish)
   *   no_cache    != 0 (prep): the projection row holds queries only, nothing is written to a cache                  */
  int32_t rot_half;
  float rot_mag;
  const double* v_rot_freq;
  int32_t v_heads, chunk, out_f32, no_cache;
} b200_attn_options;
/* What follows the softmax-weighted sums where more than a gate does: out [T, heads, vdim] (dtype dt) from a fp32
 * [T, maps * heads, vdim] (map after map).  maps == 2: o = a[map 0] - lambda * a[map 1] (differential attention).
 * v_rot_freq (f64 [vdim / 2], or NULL): o is turned back by -position * v_rot_freq[m] (pairs as rot_half says).
 * head_norm != 0: o / sqrt(mean(o^2) + eps) over the head's vdim values, no weight.  Then o * out_scale, then the gate:
 * sigmoid(gate[t, h]) per head or, gate_elems != 0, sigmoid(gate[t, h * vdim + d]) per element (gate NULL: none).  */
void b200_attn_finish(void* out, const float* a, const float* gate, int32_t ld_gate, int32_t gate_elems,
                      const int64_t* positions, const double* v_rot_freq, int32_t rot_half, int32_t maps, float lambda,
                      int32_t head_norm, float eps, float out_scale, int32_t num_tokens, int32_t heads, int32_t vdim,
                      int32_t dt, int64_t stream);
void b200_window_attn_prep_ex(const float* proj, int32_t ld, const float* bias, const float* q_norm_w,
                              const float* k_norm_w, const double* rot_freq, const int64_t* positions,
                              const int64_t* slot_mapping, float* q_out, void* k_cache, void* v_cache,
                              int32_t num_tokens, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim,
                              int32_t rot_dims, float eps, int32_t dt, const b200_attn_options* opt, int64_t stream);
void b200_window_attn_ex(void* out, const float* q, const void* k_cache, const void* v_cache, const float* sink,
                         const float* gate, int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                         const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens,
                         int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int32_t window, int32_t keep_first,
                         float scale, float softcap, int32_t dt, void* workspace, const b200_attn_options* opt,
                         int64_t stream);
/* out fp32 [T, channels] = sigmoid(bias + low w2^T)^(1 / tau); low fp32 [T, rank] (row stride ld_low), w2 fp32
 * [channels, rank], bias fp32 [channels] or NULL.                                                                  */
void b200_lowrank_decay(float* out, const float* low, int32_t ld_low, const float* w2, const float* bias, float tau,
                        int32_t num_tokens, int32_t channels, int32_t rank, int64_t stream);
/* kind 0: as b200_lowrank_decay.  kind 1: out = exp(-exp(a_log[c / a_period]) * softplus(bias + low w2^T)), the decay
 * of a gated delta rule per key channel (a_log fp32 [channels / a_period]; tau is not used).                        */
void b200_lowrank_decay_ex(float* out, const float* low, int32_t ld_low, const float* w2, const float* bias, float tau,
                           int32_t kind, const float* a_log, int32_t a_period, int32_t num_tokens, int32_t channels,
                           int32_t rank, int64_t stream);
/* Linear attention with a decayed state: S <- diag(a_t) S + (k_scale k_t) v_t^T, o_t = S^T (q_scale q_t).  q, k fp32
 * [T, heads, dim], v [T, heads, vdim] (row stride ld); exactly one of head_decay fp32 [heads] (a constant per head)
 * and chan_decay fp32 [T, heads, dim] (row stride ld_decay); act != 0: SiLU on q, k and v first; out fp32
 * [T, heads, vdim]; state fp32 [slots, heads, dim, vdim].                                                          */
void b200_decay_attn(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* head_decay,
                     const float* chan_decay, int32_t ld_decay, float q_scale, float k_scale, int32_t act, float* state,
                     const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                     int32_t num_seqs, int32_t heads, int32_t dim, int32_t vdim, int64_t stream);
/* qc fp32 [T, ldq] = [q (heads x (dim + rot_dim)) | latent (kv_rank) | shared rotated key (rot_dim)] -> cache row at
 * slot_mapping[t] ([normed latent | rotated key], dtype dt), q_plain [T, heads, dim] (dtype dt) and the rotated query
 * parts in q_full [T, heads, kv_rank + rot_dim] fp32 (entries kv_rank.. of every head).  rot_freq f64 [rot_dims / 2]. */
void b200_latent_prep(const float* qc, int32_t ldq, void* q_plain, float* q_full, void* cache,
                      const float* latent_norm_w, const double* rot_freq, float rot_mag, const int64_t* positions,
                      const int64_t* slot_mapping, int32_t num_tokens, int32_t heads, int32_t dim, int32_t rot_dim,
                      int32_t rot_dims, int32_t kv_rank, float eps, int32_t dt, int64_t stream);
/* out [T, heads, kv_rank] (dtype dt) = softmax-weighted sum of cached latents; sink fp32 [heads] or NULL;
 * window <= 0: full causal context.  cache [num_blocks, 64, kv_rank + rot_dim].  workspace (may be NULL):
 * b200_latent_attn_workspace_bytes() bytes; with it, steps of few token rows split each row's keys over several
 * blocks and merge the parts (the result is the same softmax, summed in another order).                           */
void b200_latent_attn(void* out, const float* q_full, const void* cache, const float* sink,
                      const uint32_t* cu_seqlens_q, const uint32_t* context_lens, const uint32_t* block_tables,
                      int32_t max_blocks_per_seq, int32_t num_seqs, int32_t num_tokens, int32_t heads, int32_t kv_rank,
                      int32_t rot_dim, int32_t window, float scale, int32_t dt, void* workspace, int64_t stream);
int64_t b200_latent_attn_workspace_bytes(int32_t num_tokens, int32_t heads, int32_t kv_rank, int32_t window);
/* b200_latent_prep for a layer that shares another layer's latent cache: qc holds the queries only, nothing is
 * normed or written to a cache.                                                                                    */
void b200_latent_prep_queries(const float* qc, int32_t ldq, void* q_plain, float* q_full, const double* rot_freq,
                              float rot_mag, const int64_t* positions, int32_t num_tokens, int32_t heads, int32_t dim,
                              int32_t rot_dim, int32_t rot_dims, int32_t kv_rank, int32_t dt, int64_t stream);
/* b200_latent_attn with a per-head output gate: head h's output is multiplied by sigmoid(gate[t, h]), gate fp32
 * [T, ld_gate] (NULL: none).                                                                                        */
void b200_latent_attn_gated(void* out, const float* q_full, const void* cache, const float* sink, const float* gate,
                            int32_t ld_gate, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                            const uint32_t* block_tables, int32_t max_blocks_per_seq, int32_t num_seqs,
                            int32_t num_tokens, int32_t heads, int32_t kv_rank, int32_t rot_dim, int32_t window,
                            float scale, int32_t dt, void* workspace, int64_t stream);
/* Causal per-channel convolution + SiLU; state fp32 [slots, taps - 1, channels]; taps_w fp32 [channels, taps] (last
 * column = current token), bias fp32 [channels] or NULL.  out must not alias x (token chunks run in parallel).    */
void b200_short_conv_silu(float* out, int32_t ldo, const float* x, int32_t ldx, const float* taps_w, const float* bias,
                          float* state, const int32_t* state_slots, const uint32_t* cu_seqlens_q,
                          const uint32_t* context_lens, int32_t num_seqs, int32_t num_tokens, int32_t channels,
                          int32_t taps, int64_t stream);
/* q, k [T, kv_heads, dim], v [T, heads, vdim] (row stride ld), b_raw / a_raw [T, heads] (row stride ld_ba), all fp32;
 * out fp32 [T, heads, vdim]; state fp32 [slots, heads, dim, vdim].                                                 */
void b200_delta_rule(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* b_raw,
                     const float* a_raw, int32_t ld_ba, const float* a_log, const float* dt_bias, float* state,
                     const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                     int32_t num_seqs, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int64_t stream);
/* b200_delta_rule with one decay per head AND key channel: chan_decay fp32 [T, heads, dim] (row stride ld_decay) holds
 * the decays themselves (b200_lowrank_decay_ex kind 1), row i of S is multiplied by chan_decay[t, h, i].           */
void b200_delta_rule_chan(float* out, const float* q, const float* k, const float* v, int32_t ld, const float* b_raw,
                          int32_t ld_b, const float* chan_decay, int32_t ld_decay, float* state,
                          const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                          int32_t num_seqs, int32_t heads, int32_t kv_heads, int32_t dim, int32_t vdim, int64_t stream);
/* x [T, heads, vdim], Bm / Cm [T, groups, nstate] (row stride ld), dt_raw [T, heads] (row stride ld_dt), fp32;
 * out fp32 [T, heads, vdim]; state fp32 [slots, heads, nstate, vdim]; d_skip may be NULL.                          */
void b200_ssd_scan(float* out, const float* x, const float* Bm, const float* Cm, int32_t ld, const float* dt_raw,
                   int32_t ld_dt, const float* a_log, const float* dt_bias, const float* d_skip, float* state,
                   const int32_t* state_slots, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                   int32_t num_seqs, int32_t heads, int32_t groups, int32_t nstate, int32_t vdim, int64_t stream);
void b200_moe_route(const float* logits, int32_t num_tokens, int32_t experts, int32_t top, float scale,
                    int32_t* top_idx, float* top_w, int64_t stream);
int64_t b200_moe_workspace_bytes(int32_t num_tokens, int32_t experts, int32_t top, int32_t width, int32_t ff);
/* x fp32 [T, width] += sum over a token's choices of top_w * expert(h); w_gate_up [E, 2 ff, width] (gate rows first),
 * w_down [E, width, ff], h [T, width], all dtype dt.                                                               */
void b200_moe_experts(float* x, const void* h, const int32_t* top_idx, const float* top_w, const void* w_gate_up,
                      const void* w_down, int32_t num_tokens, int32_t experts, int32_t top, int32_t width, int32_t ff,
                      int32_t dt, void* workspace, int64_t stream);

/* Router with a selection bias and expert groups.  s = softmax(logits) over all `experts` outputs; the choice score of
 * expert e is s[e] + bias[e] (bias fp32 [experts] or NULL).  groups > 0: the outputs form `groups` equal runs of
 * neighbours, a run's score is its largest choice score, and only members of the `keep` best runs can be chosen.  The
 * `top` largest choice scores win (ties: lowest index); their weights are s (without the bias) times scale.       */
void b200_moe_route_ex(const float* logits, const float* bias, int32_t num_tokens, int32_t experts, int32_t top,
                       int32_t groups, int32_t keep, float scale, int32_t* top_idx, float* top_w, int64_t stream);
/* b200_moe_experts with an activation kind and identity experts; out = (accumulate ? out : 0) + sum over a token's
 * choices.  act 0: SiLU(gate) * up, w_up [E, 2 ff, width] (gate rows first); act 1: relu(up)^2, w_up [E, ff, width].
 * Indices >= experts (up to experts + identity - 1) are identity experts: their output is the token's own input row,
 * read from ident (fp32 when ident_f32 != 0, else dtype dt; [T, width]).  workspace: b200_moe_workspace_bytes with
 * experts + identity.                                                                                              */
void b200_moe_experts_ex(float* out, const void* h, const int32_t* top_idx, const float* top_w, const void* w_up,
                         const void* w_down, int32_t num_tokens, int32_t experts, int32_t identity, int32_t top,
                         int32_t width, int32_t ff, int32_t act, int32_t accumulate, const void* ident,
                         int32_t ident_f32, int32_t dt, void* workspace, int64_t stream);

typedef struct b200_hybrid_config {
  int32_t width, vocab, num_layers;
  int32_t dt;                               /* 0 = bf16 operands and cache, 1 = fp32 */
  int32_t block_size, num_blocks, max_blocks_per_seq;
  int32_t max_seqs, max_tokens;             /* per step */
  int32_t num_state_slots;
  float norm_eps, norm_weight_offset;       /* layer / final norms multiply by (offset + w) */
  float embed_scale;                        /* the embedding row is multiplied by it */
  float embed_pos_base;                     /* > 0: a sinusoidal position vector joins the embedding row: entry 2i is
                                               sin(p base^(-2i / width)), entry 2i + 1 the cosine of the same angle */
  int32_t final_norm_kind;                  /* B200_NORM_*; DYNTANH: see b200_hybrid_set_final_norm */
} b200_hybrid_config;

typedef struct b200_hybrid_layer {
  int32_t mixer;                            /* B200_MIXER_* */
  int32_t heads, kv_heads;                  /* kv_heads: q / k heads of the delta rule, B / C groups of the SSD scan */
  int32_t dim, rot_dim, rot_dims, vdim, kv_rank, window;
  int32_t state, conv_taps, norm_groups;
  float scale, rot_mag;
  int32_t experts, top, expert_ff, shared_ff;   /* experts == 0: no routed experts; shared_ff == 0: no shared expert */
  float route_scale;
  const void* norm_w;                       /* fp32 [width] */
  /* matrix-product weights, dtype dt, rows = outputs.  w_in fuses the mixer's input projections:
   *   latent attention: [q: heads x (dim + rot_dim) | latent: kv_rank | rotated key: rot_dim]
   *   delta rule:       [q: kv_heads x dim | k: kv_heads x dim | v: heads x vdim | b: heads | a: heads | gate: heads x vdim]
   *   SSD:              [z: heads x vdim | x: heads x vdim | B: groups x state | C: groups x state | dt: heads]      */
  const void *w_in, *w_uk, *w_uv, *w_o;
  /* small fp32 parameters */
  const void *latent_norm_w, *sink, *conv_w, *conv_b, *a_log, *dt_bias, *d_skip, *out_norm_w;
  const double* rot_freq;                   /* f64 [rot_dims / 2], device */
  const void *w_router, *w_gate_up, *w_down, *w_shared_gate_up, *w_shared_down;
  void *kv_cache, *conv_state, *rec_state;  /* caller-owned pools (see the kernels above for their shapes) */
  /* ---- layouts, side mixers, windowed attention and decayed linear attention */
  int32_t layout;                           /* B200_LAYOUT_*; SANDWICH: shared_ff is the dense gated feed-forward
                                               (w_shared_gate_up / w_shared_down), read through ff_norm_w */
  int32_t keep_first;                       /* window attention: the first keep_first positions stay visible */
  int32_t qkv_act;                          /* decay attention: != 0 SiLU on q, k and v */
  int32_t gate_act;                         /* decay attention output gate: 0 SiLU, 1 sigmoid */
  int32_t decay_rank;                       /* decay attention: > 0: per-channel decay from a low-rank projection */
  int32_t out_norm_period;                  /* decay attention: elements of out_norm_w (0: the norm has no weight);
                                               norm_groups = groups the heads x vdim outputs are normalised in */
  float softcap, q_scale, k_scale, decay_tau;
  float out_scale;                          /* the mixer's output is multiplied by it (every mixer; set it to 1) */
  /* w_in of the new mixers:
   *   window attention: [q: heads x dim | k: kv_heads x dim | v: kv_heads x vdim | gate: heads (if gated)]
   *   decay attention:  [q: heads x dim | k: heads x dim | v: heads x vdim | gate: heads x vdim | low: decay_rank] */
  const void *post_norm_w, *ff_norm_w, *ff_post_norm_w;     /* fp32 [width], SANDWICH layout */
  const void *in_bias, *o_bias;             /* fp32: over q | k | v of window attention; over the o-projection's outputs */
  const void *q_norm_w, *k_norm_w;          /* fp32, whole-projection norms of window attention (NULL: none) */
  const void *head_decay;                   /* fp32 [heads] (decay_rank == 0) */
  const void *w_decay2, *decay_bias;        /* fp32 [heads x dim, decay_rank], [heads x dim] */
  int32_t gated;                            /* window attention: != 0: per-head sigmoid output gate, logits last in w_in */
  void* v_cache;                            /* window attention: kv_cache holds K, v_cache V */
  /* ---- POSTNORM layers, attention with a distance bias, shared latent caches, routers with groups
   * gated (both attentions): 1 = one gate logit per head, 2 = one per output element (window attention only); the
   * logits are the last rows of w_in.  w_in of a latent attention with shared_cache: the queries (and gate) only. */
  int32_t head_norm, v_from_k;              /* window attention: see b200_attn_options */
  int32_t q_temp_every;
  float q_temp_coef;
  const void* dist_slopes;                  /* fp32 [heads] or NULL */
  int32_t shared_cache;                     /* latent attention: != 0: no latent projection of its own; kv_cache is
                                               another (earlier) layer's cache, which this layer only reads */
  int32_t expert_act, shared_act;           /* 0: SiLU(gate) * up ([gate | up] rows); 1: relu(up)^2 (up rows only) */
  int32_t identity_experts;                 /* router outputs experts .. experts + identity_experts - 1 return the input */
  int32_t route_groups, route_keep;         /* see b200_moe_route_ex (0: no groups) */
  int32_t shared_gated;                     /* != 0: one more row closes w_shared_gate_up; the shared expert's output is
                                               multiplied by the sigmoid of that row's product with the token */
  const void* route_bias;                   /* fp32 [experts + identity_experts] or NULL */
  /* ---- PRENORM layers, dynamic-tanh norms, token shift, depth average, rotated values, chunked and differential
   * attention, the delta rule with a decay per key channel, dense feed-forwards with biases */
  int32_t norm_kind;                        /* B200_NORM_* of norm_w (and ff_norm_w) */
  float norm_alpha, ff_norm_alpha;          /* DYNTANH: the scalar inside the tanh */
  const void *norm_b, *ff_norm_b;           /* DYNTANH: fp32 [width] bias (NULL: none) */
  const void* shift_w;                      /* fp32 [width] or NULL: token shift of the mixer's input (b200_stream_norm) */
  void* shift_state;                        /* fp32 [slots, width], caller-owned */
  const void* depth_w;                      /* fp32 [layer + 2] or NULL: the layer's result X_(layer+1) is kept, and what
                                               goes on is sum_j depth_w[j] X_j, X_0 being the embedding output */
  float ff_scale;                           /* PRENORM: the feed-forward's output is multiplied by it */
  const void *ff_up_bias, *ff_down_bias;    /* fp32 [shared_ff], [width] or NULL: biases of a squared-ReLU dense feed-forward */
  /* window attention (see b200_attn_options).  score_maps == 2: differential attention; w_in holds
   * [q: maps x heads x dim | k: maps x kv_heads x dim | v: kv_heads x vdim | gate], the maps one after the other, the
   * K cache has maps x kv_heads heads, the V cache kv_heads; out = (a_0 - diff_lambda a_1), RMS-normed per head without a
   * weight where diff_norm != 0, times diff_out_scale.  shared_cache != 0: w_in holds [q | gate] only and kv_cache /
   * v_cache are an earlier layer's, which this layer only reads.                                                      */
  int32_t rot_half, chunk, score_maps, diff_norm;
  float diff_lambda, diff_out_scale;
  const double* v_rot_freq;                 /* f64 [vdim / 2], device, or NULL */
  /* delta rule: chan_rank > 0: one decay per head and key channel from a low-rank projection, w_in =
   * [q | k | v | b: heads | low_a: chan_rank | low_g: gate_rank], decay = exp(-exp(a_log[h]) softplus(w_decay2 low_a +
   * dt_bias)) with w_decay2 fp32 [heads x dim, chan_rank], dt_bias fp32 [heads x dim]; gate_rank > 0: the output gate's
   * logits are w_gate2 low_g (w_gate2 fp32 [heads x vdim, gate_rank]) and the gate is a sigmoid (gate_act 1)          */
  int32_t chan_rank, gate_rank;
  const void* w_gate2;
} b200_hybrid_layer;

typedef struct b200_hybrid b200_hybrid;
b200_hybrid* b200_hybrid_new(const b200_hybrid_config* cfg);
void b200_hybrid_free(b200_hybrid*);
void b200_hybrid_set_layer(b200_hybrid*, int32_t layer, const b200_hybrid_layer* l);
/* A second mixer of the layer, beside the first: it reads the same normed input and its output (times out_scale) joins
 * the first one's.  Only the mixer's own fields of `side` are used (no norms, no feed-forward).  After set_layer.    */
void b200_hybrid_set_layer_side(b200_hybrid*, int32_t layer, const b200_hybrid_layer* side);
/* embed [vocab, width], lm_head [vocab, width] in dtype dt; final_norm fp32 [width] */
void b200_hybrid_set_globals(b200_hybrid*, const void* embed, const void* final_norm, const void* lm_head);
/* final norm of kind DYNTANH: bias fp32 [width] (may be NULL) and the scalar inside the tanh */
void b200_hybrid_set_final_norm(b200_hybrid*, const void* bias, float alpha);
int64_t b200_hybrid_workspace_bytes(const b200_hybrid*);
void b200_hybrid_set_workspace(b200_hybrid*, void* workspace, int64_t bytes);
/* fp32 [num_layers, max_tokens, width] device buffer that receives the residual stream after every layer (NULL: off) */
void b200_hybrid_set_layer_trace(b200_hybrid*, float* buf);
/* One step from DEVICE inputs.  out_rows u32 [num_out]: token rows whose logits are wanted (a sequence's last row
 * when generating); logits fp32 [num_out, vocab] and / or out_ids u32 [num_out] (either may be NULL) are written;
 * sampling as set by b200_hybrid_set_sampling (default greedy).                                                    */
void b200_hybrid_step(b200_hybrid*, const uint32_t* input_ids, const int64_t* positions, const int64_t* slot_mapping,
                      const uint32_t* cu_seqlens_q, const uint32_t* context_lens, const uint32_t* block_tables,
                      const int32_t* state_slots, const uint32_t* out_rows, int32_t num_seqs, int32_t num_tokens,
                      int32_t max_blocks, int32_t num_out, float* logits, uint32_t* out_ids, int64_t stream);
/* The same from HOST (pinned) inputs: H2D of the step's inputs, the step, D2H of ids and / or logits, stream sync. */
int32_t b200_hybrid_step_host(b200_hybrid*, const uint32_t* input_ids, const int64_t* positions,
                              const int64_t* slot_mapping, const uint32_t* cu_seqlens_q, const uint32_t* context_lens,
                              const uint32_t* block_tables, const int32_t* state_slots, const uint32_t* out_rows,
                              int32_t num_seqs, int32_t num_tokens, int32_t max_blocks, int32_t num_out,
                              float* logits_host, uint32_t* out_ids_host, int64_t stream);
int32_t b200_hybrid_set_sampling(b200_hybrid*, int32_t strategy, int32_t k, float p, float t);
void b200_hybrid_set_step_seed(b200_hybrid*, uint64_t seed, int64_t stream);
int64_t b200_hybrid_launches_per_step(const b200_hybrid*);

/* ------------------------------------------------- state slots and host-driven steps of the scheduler
 * Models with recurrent state give every running sequence one slot of `n` (enable_state_slots): schedule() admits a
 * waiting sequence only while a slot is free, finished / swapped-out sequences give theirs back.  A STREAMED sequence
 * is driven by the host instead of schedule(): open (takes a slot when slots are enabled), feed tokens (its block
 * table grows by whole blocks as needed), run them with b200_prepare_ragged, close (blocks and slot return).
 * b200_prepare_ragged builds the step metadata of ANY mix of running sequences.  mode 0 (a scheduled prefill chunk):
 * sequence i brings tokens [num_cached_tokens, + counts[i]) (counts NULL: min(chunk_size, the rest)); mode 1 (decode):
 * its last counts[i] tokens (NULL: 1); mode 2 (streamed): as mode 0 with counts NULL = everything fed since the last
 * step, and num_cached_tokens advances.  block_tables is [n, max_blocks_cap], zero padded.  Returns the number of
 * token rows, -1 when a capacity is too small, -2 for a bad index / count.                                           */
int32_t b200_scheduler_enable_state_slots(b200_scheduler*, int32_t n);
int32_t b200_scheduler_num_free_state_slots(const b200_scheduler*);
int32_t b200_scheduler_seq_state_slot(const b200_scheduler*, int32_t running_idx);
int64_t b200_scheduler_open(b200_scheduler*);
int32_t b200_scheduler_feed(b200_scheduler*, int64_t seq_id, const uint32_t* tokens, int32_t n);
int32_t b200_scheduler_close(b200_scheduler*, int64_t seq_id);
int32_t b200_scheduler_running_index(const b200_scheduler*, int64_t seq_id);
int32_t b200_prepare_ragged(b200_scheduler*, const int32_t* indices, const int32_t* counts, int32_t n, int32_t mode,
                            int32_t token_cap, int32_t max_blocks_cap, uint32_t* input_ids,
                            int64_t* positions, int64_t* slot_mapping, uint32_t* cu_seqlens_q, uint32_t* context_lens,
                            uint32_t* block_tables, int32_t* state_slots);

#ifdef __cplusplus
}
#endif
#endif /* B200_VLLM_H */
