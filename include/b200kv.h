/*
 * b200kv.h: C ABI of the B200 (sm_100a) decode-time KV-cache path.
 *
 * Three device operations and the host bookkeeping around them:
 *   append  : scatter each new token's MLA latent row (c_kv | k_rope, bf16) into the block-paged pool;
 *   gather  : copy a sequence's rows out of the pool through its block table;
 *   decode  : dense absorbed-MLA decode attention over the paged pool (split-KV on tcgen05 tensor
 *             cores) with a log-sum-exp merge of the split partials.
 *
 * Every entry point takes plain pointers, sizes and a CUDA stream handle passed as void*; nothing here
 * depends on a framework type. Device entry points enqueue work and return; an asynchronous fault
 * surfaces at the caller's next synchronisation, exactly as with the two-phase operator launches they
 * replace (reference: include/moe/core/op_table.hpp:1015). Return value: 0 on success, otherwise one
 * of the B200KV_ERR_* codes, whose values follow the reference's status convention
 * (include/moe/core/op_table.hpp:142-147). b200kv_last_error() gives the text for the calling thread.
 *
 * Pool layout (reference: src/memory/static_arena_manager.cpp:315-318, 571-580): a layer's cache is
 * two co-indexed row arrays, latent [rows][latent_dim] and rope [rows][rope_dim], rows = blocks x
 * block_size. Strides are in ELEMENTS (bf16). The fused 576-wide row of the benchmarks is the same
 * view with rope = latent + 512 and both row strides 576. The layer is chosen by the caller's base
 * pointers, as in src/pipeline/pipeline.cpp:391-395.
 */
#ifndef B200KV_H_
#define B200KV_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200KV_OK 0
#define B200KV_ERR_NULLPTR 161001 /* a required pointer was null            */
#define B200KV_ERR_INVALID 161002 /* a size, stride or alignment is refused */
#define B200KV_ERR_RUNTIME 361001 /* the CUDA runtime reported a failure    */

/* Codes a kernel records in the caller's status word (first error wins). */
#define B200KV_DEV_OK 0
#define B200KV_DEV_BAD_SLOT 1    /* append: slot >= pool_rows; detail = token index, slot           */
#define B200KV_DEV_BAD_BLOCK 2   /* gather/decode: block id out of range; detail = sequence, index  */
#define B200KV_DEV_TIMEOUT 3     /* a bounded wait inside a kernel ran out; detail = site, phase    */
#define B200KV_DEV_BAD_PLAN 4    /* decode: work partition inconsistent; detail = cta, value        */

/* MLA geometry of the reference model (include/moe/core/config.hpp:47,78-79,95). */
#define B200KV_LATENT_DIM 512
#define B200KV_ROPE_DIM 64
#define B200KV_HEADS 64

/* One layer's paged cache (device pointers, bf16). */
typedef struct b200kv_pool_view {
  void* latent;              /* [pool_rows][latent_row_stride] bf16, 16-byte aligned            */
  void* rope;                /* [pool_rows][rope_row_stride]  bf16, 16-byte aligned             */
  int64_t latent_row_stride; /* elements; multiple of 8                                          */
  int64_t rope_row_stride;   /* elements; multiple of 8                                          */
  int64_t pool_rows;         /* num_blocks * block_size                                          */
} b200kv_pool_view;

/* Device status word: int32[4] = {code, detail0, detail1, detail2}, zeroed by the caller. */
typedef int32_t b200kv_status_word;

const char* b200kv_last_error(void);
int32_t b200kv_abi_version(void);

/*
 * Host-side fault injection, for tests of failure handling. After b200kv_fault_inject(name, n) the next n calls
 * of the entry point `name` go through and the one after fails with B200KV_ERR_RUNTIME ("injected failure: name")
 * before anything reaches the device; then the hook disarms itself. The counterpart of the reference's
 * FailRuntimeCall(name, calls) (mock/runtime_faults.cpp:8-23, used by tests/mock_failure_teardown.cpp:153-184).
 * Names: the device entry points b200kv_append, b200kv_gather, b200kv_resolve_rows, b200kv_mla_decode,
 * b200kv_mla_decode_peer, b200kv_lse_merge, b200kv_peer_merge, b200kv_append_fused, b200kv_mx_quant_e4m3,
 * b200kv_indexer_topk, and b200kv_engine_step_upload (the per-step copy of b200kv_engine_begin_step).
 * No GPU fault is ever made. b200kv_fault_clear disarms and returns how many injected failures fired.
 */
int32_t b200kv_fault_inject(const char* entry_point, int32_t after_calls);
int64_t b200kv_fault_clear(void);

/*
 * Append. Replaces the launch of aclnnScatterPaKvCache planned at src/pipeline/pipeline.cpp:226-234
 * (prototype include/moe/core/op_table.hpp:365-372, cache mode "Norm"): for each token row t,
 *   pool.latent[slot[t]] = latent_src[t],  pool.rope[slot[t]] = rope_src[t].
 * slot is the flat row (block * block_size + offset); a negative slot marks padding and is skipped;
 * a slot >= pool_rows is recorded in `status` and skipped. Source strides in elements, multiple of 8.
 */
int32_t b200kv_append(const b200kv_pool_view* pool, const void* latent_src, int64_t src_latent_stride,
                      const void* rope_src, int64_t src_rope_stride, const int32_t* slot_mapping, int64_t n_tokens,
                      void* stream, b200kv_status_word* status);

/*
 * Gather. The standalone form of the block-table addressing that the reference hands to its fused
 * attention operator (block_table and block_size arguments, src/pipeline/pipeline.cpp:241,244):
 * logical token j of sequence b is pool row block_table[b*max_blocks + j/block_size]*block_size +
 * j%block_size; its latent and rope rows are copied to output row out_row_offsets[b] + j.
 * kv_len, block_table and out_row_offsets are device arrays (int32, int32, int64).
 */
int32_t b200kv_gather(const b200kv_pool_view* pool, const int32_t* block_table, int64_t max_blocks,
                      const int32_t* kv_len, int64_t batch, int64_t block_size, void* out_latent,
                      int64_t out_latent_stride, void* out_rope, int64_t out_rope_stride,
                      const int64_t* out_row_offsets, int64_t total_rows, void* stream,
                      b200kv_status_word* status);

/*
 * Decode attention. Replaces the launch of aclnnFusedInferAttentionScoreV5 planned at
 * src/pipeline/pipeline.cpp:235-249 (prototype include/moe/core/op_table.hpp:438-454; one query token
 * per sequence, layout TND, 64 query heads over one latent KV head): per sequence b and head h, over
 * logical tokens [kv_begin[b], kv_begin[b]+kv_len[b]) of the sequence's block table,
 *   s_j = scale*(q_lat[h].c_j + q_rope[h].r_j), p = softmax_j(s), out[h] = sum_j p_j c_j,
 *   lse[h] = max_j s_j + log sum_j exp(s_j - max).
 * q: bf16, element (b,h,k) at q[b*q_seq_stride + h*q_head_stride + k], k in [0,576).
 * out: bf16 [batch][heads][512]; lse: fp32 [batch][heads] or null.
 * partial_o/m/l: when non-null the call writes the UN-normalised shard result instead of out/lse
 *   (fp32 [batch][heads][512], [batch][heads], [batch][heads]) for a later b200kv_lse_merge across
 *   KV-range shards; kv_begin (device int32, multiple of block_size, or null for zero) selects the
 *   shard's first token.
 * workspace: device scratch of at least b200kv_mla_decode_workspace_bytes(); reused across calls on
 *   one stream. variant: B200KV_DECODE_AUTO, or force one implementation (tests, profiling).
 */
#define B200KV_DECODE_AUTO 0
#define B200KV_DECODE_SIMT 1   /* CUDA-core kernel: any geometry                            */
#define B200KV_DECODE_TCGEN05 2 /* tensor-core kernel: 64 heads, 512+64, block_size % 64 == 0 */

typedef struct b200kv_decode_args {
  const void* q;
  int64_t q_seq_stride;
  int64_t q_head_stride;
  b200kv_pool_view pool;
  const int32_t* block_table; /* device int32 [batch][max_blocks] */
  int64_t max_blocks;
  const int32_t* kv_len;   /* device int32 [batch]           */
  const int32_t* kv_begin; /* device int32 [batch] or null   */
  int32_t batch;
  int32_t heads;
  int32_t block_size;
  float scale;
  void* out;        /* bf16 [batch][heads][512] or null when partials are requested */
  float* lse;       /* fp32 [batch][heads] or null                                  */
  float* partial_o; /* fp32 [batch][heads][512] or null                             */
  float* partial_m; /* fp32 [batch][heads] or null                                  */
  float* partial_l; /* fp32 [batch][heads] or null                                  */
  void* workspace;
  size_t workspace_bytes;
  int32_t variant;
  int32_t max_ctas; /* 0 = one CTA per SM of the current device                     */
  /*
   * Append fused into the attention launch (tensor-core kernel, kv_begin null; both null = none): the new row
   * of sequence b, new_latent[b] (512 bf16) and new_rope[b] (64 bf16), row strides in elements (multiples of
   * 8), is written to the pool at the sequence's last position kv_len[b] - 1, through the block table, by the
   * CTA that attends over that position, before it reads the tile. The result equals b200kv_append with
   * slot_mapping[b] = block_table[b][(kv_len[b]-1) / block_size] * block_size + (kv_len[b]-1) % block_size
   * followed by the attention: the two stages the reference plans back to back
   * (src/pipeline/pipeline.cpp:226-249) as one launch. Sequences with kv_len 0 append nothing.
   */
  const void* new_latent;
  int64_t new_latent_stride;
  const void* new_rope;
  int64_t new_rope_stride;
  /*
   * B200KV_DECODE_STABLE_TABLES: block_table, kv_len and kv_begin were not written by the kernel that precedes
   * this call on the stream (the engine uploads them once per step, before the first layer:
   * src/pipeline/pipeline.cpp:515-519). The decode kernel is launched so that it may start while that kernel
   * drains; with this flag it finds its slice of the work and the rows of its first tiles before it waits for
   * that kernel, and only then reads Q, the new rows and the pool. Without it everything is read after the wait.
   */
  uint32_t flags;
  /*
   * Gathered rows (null = none): the call attends, for sequence b, over the pool rows row_index[b][0 .. kv_len[b])
   * (device int32, row stride row_index_stride elements; what b200kv_resolve_rows writes) instead of walking
   * block_table, which is then ignored together with block_size and max_blocks; kv_begin and the fused append
   * must be null. An entry that is not a row of the pool is recorded as B200KV_DEV_BAD_BLOCK. The tensor-core
   * kernel brings the rows in, 64 a tile, with 16-byte asynchronous copies that place them as a swizzled TMA
   * load would, so a top-k selection runs on the same tcgen05 pipeline as a dense history; the CUDA-core kernel
   * treats the list as a table of single-row blocks.
   */
  const int32_t* row_index;
  int64_t row_index_stride;
  /*
   * The output quantised as well (both null = no): out_fp8 [batch][heads][512] FP8 E4M3 and out_scale
   * [batch][heads][16] E8M0, block-32 MX along a head's row, bit for bit what b200kv_mx_quant_e4m3 gives on `out`
   * viewed as [batch][heads * 512]: the reference's stage after attention (attn_quant,
   * src/pipeline/pipeline.cpp:250-258) as the epilogue of the kernel that writes `out`, instead of a launch of its
   * own that reads `out` back. Needs `out` (not the partial_* form). The CUDA-core path runs the stand-alone
   * quantiser behind the attention.
   */
  void* out_fp8;
  void* out_scale;
} b200kv_decode_args;
#define B200KV_DECODE_STABLE_TABLES 1u

size_t b200kv_mla_decode_workspace_bytes(int32_t batch, int32_t heads, int32_t max_ctas);
int32_t b200kv_mla_decode(const b200kv_decode_args* args, void* stream, b200kv_status_word* status);

/*
 * Attention over a selected subset of a sequence's tokens (what a top-k indexer in front of attention hands
 * over; the reference vendors such an indexer but does not apply it, include/moe/pipeline/pipeline.hpp:57-66).
 * b200kv_resolve_rows turns the selection into pool rows: rows[b][j] = block_table[b][t / bs] * bs + t % bs for
 * t = token_index[b][j], j < n_selected[b] (the rest -1; a token outside the table or the pool is recorded
 * as B200KV_DEV_BAD_BLOCK). b200kv_mla_decode then attends over exactly those rows when it is given
 * row_index = rows, row_index_stride = max_selected and kv_len = n_selected (tensor-core kernel for 64 heads), or,
 * equivalently, block_table = rows, max_blocks = max_selected and block_size = 1 (a table of single-row blocks,
 * which runs on the CUDA-core kernel). All arrays device int32.
 */
int32_t b200kv_resolve_rows(const int32_t* block_table, int64_t max_blocks, int64_t block_size, const int32_t* token_index,
                            int64_t max_selected, const int32_t* n_selected, int64_t batch, int64_t pool_rows,
                            int32_t* rows, void* stream, b200kv_status_word* status);

/*
 * The selection itself: the sparse indexer the reference vendors in front of attention
 * (aclnnQuantLightningIndexer; contract mock/mock_ops.cpp:1118-1221, formula
 * third_party/ops_transformer/attention/quant_lightning_indexer/README.md). For sequence b and its one query
 * token of the step, every token t < kv_len[b] of the paged index-key cache scores
 *   score_t = sum_h w[b][h] * ReLU(q_scale[b][h] * k_scale[row_t] * (Q[b][h] . K[row_t])),
 * Q and K FP8 E4M3 vectors of 128, and index_out[b][0..k) receives the positions of the k best tokens, best
 * first (ties: lower position first; -1 beyond n_selected_out[b] = min(k, kv_len[b])). Two score kernels. The
 * exact one runs fixed fp32 fma chains on CUDA cores (csrc/kv_indexer.cu states them), so its selection is
 * reproducible bit for bit. The tensor-core one (csrc/kv_indexer_tc.cu: tcgen05 FP8 MMA, 128 tokens x 64 heads
 * a tile, keys through TMA) rounds the 128-term dot products differently: its scores agree to rounding error and
 * its selection can differ from the exact one between tokens whose scores are that close.
 * q fp8 [batch][heads][128] (heads <= 64); q_scale fp32 and weights bf16 [batch][heads]; key_pool fp8
 * [pool_rows][key_stride] (16-byte aligned, stride a multiple of 16) with k_scale fp32 [pool_rows], addressed
 * through block_table / block_size like the KV pool; k <= 2048; workspace of
 * b200kv_indexer_workspace_bytes(batch, max_kv_len) bytes holds the scores.
 */
typedef struct b200kv_indexer_args {
  const void* q;
  const float* q_scale;
  const void* weights;
  int32_t heads;
  const void* key_pool;
  int64_t key_stride;
  const float* k_scale;
  int64_t pool_rows;
  const int32_t* block_table;
  int64_t max_blocks;
  const int32_t* kv_len;
  int32_t batch;
  int32_t block_size;
  int64_t max_kv_len; /* the largest kv_len[b] (sizes the launch) */
  int32_t k;
  int32_t* index_out;      /* device int32 [batch][k] */
  int32_t* n_selected_out; /* device int32 [batch] */
  void* workspace;
  size_t workspace_bytes;
  int32_t variant; /* B200KV_INDEXER_AUTO, _EXACT or _TCGEN05 */
  /*
   * Optional: the selection as pool rows as well, device int32 [batch][k], rows_out[b][j] = block_table[b][t /
   * block_size] * block_size + t % block_size for t = index_out[b][j] (-1 beyond n_selected_out[b]): what
   * b200kv_resolve_rows makes of index_out with this block table, for a KV pool that shares the key cache's
   * paging, written by the select kernel itself. Feed it to b200kv_decode_args.row_index.
   */
  int32_t* rows_out;
} b200kv_indexer_args;
#define B200KV_INDEXER_AUTO 0    /* tensor cores where the geometry allows, else CUDA cores            */
#define B200KV_INDEXER_EXACT 1   /* CUDA cores: the fixed fp32 chains, reproducible bit for bit         */
#define B200KV_INDEXER_TCGEN05 2 /* tensor cores: heads <= 64, block_size % 64 == 0; refused otherwise */

size_t b200kv_indexer_workspace_bytes(int32_t batch, int64_t max_kv_len);
int32_t b200kv_indexer_topk(const b200kv_indexer_args* args, void* stream, b200kv_status_word* status);

/*
 * Decode attention without a caller workspace and without any device allocation. No counterpart in
 * the reference. Same arguments and results as b200kv_mla_decode (args->workspace, workspace_bytes and
 * variant are ignored; the tensor-core kernel runs, so the geometry it needs applies: 64 heads,
 * block_size % 64 == 0, 16-byte aligned q). The partial-result scratch is a fixed array inside the
 * library's device image, b200kv_mla_decode_static_scratch_bytes() bytes (8,421,376) on every GPU that
 * loads the library, held until the process exits. It covers grids of up to B200KV_STATIC_MAX_CTAS
 * CTAs: args->max_ctas = 0 means that many; a larger max_ctas is refused with B200KV_ERR_INVALID.
 * The first call on a device looks up the array's address (cudaGetSymbolAddress): make that first
 * call outside any stream capture. All calls share the one array, so two calls that overlap on the
 * GPU (different streams, no ordering between them) race; calls on one stream are safe.
 */
#define B200KV_STATIC_MAX_CTAS 32
size_t b200kv_mla_decode_static_scratch_bytes(void);
int32_t b200kv_mla_decode_static(const b200kv_decode_args* args, void* stream, b200kv_status_word* status);

/*
 * LSE merge of n_parts shard partials (the reduction that follows the KV-range split):
 *   M = max_r m_r, L = sum_r l_r e^{m_r-M}, out = sum_r O_r e^{m_r-M} / L, lse = M + log L.
 * partial_o: fp32 [n_parts][rows][512]; partial_m, partial_l: fp32 [n_parts][rows]; rows = batch*heads.
 * No counterpart in the reference (single device, include/moe/core/config.hpp:280).
 */
int32_t b200kv_lse_merge(const float* partial_o, const float* partial_m, const float* partial_l, int32_t n_parts,
                         int64_t rows, void* out_bf16, float* lse, void* stream);

/*
 * The same merge across GPUs, over peer memory instead of a collective library: every rank (one process per
 * GPU) pushes its shard's partials into every rank's exchange buffer with peer stores over NVLink, each value
 * as one 8-byte word that carries the call's epoch, and merges what arrives in its own buffer, in one kernel
 * and without fences or flags between the ranks: a reader that finds the epoch in a word has its value. The
 * wait for the peers' words is bounded (about a second: B200KV_DEV_TIMEOUT in the status word when a peer
 * does not arrive). No reference counterpart: the reference is a one-device engine; this is the exchange
 * step of the KV-range split.
 *   b200kv_peer_exchange_bytes   size of one rank's exchange buffer for `world` ranks (at most 16) and `rows`
 *                                rows (= batch * heads) per rank
 *   b200kv_peer_buffer_alloc     allocates and zero-fills it (cudaMalloc) and returns its 64-byte inter-process
 *                                handle, which the ranks exchange by any means (an all-gather of 64 bytes)
 *   b200kv_peer_buffer_open      maps a peer's buffer from its handle (peer access is enabled on first use)
 *   b200kv_peer_merge            peer_buffers[r] = rank r's buffer as seen from this process (own one at
 *                                [rank]); enqueues the kernel on `stream`. All ranks must call it
 *                                the same number of times; the call carries its own epoch on the device, so it
 *                                can be captured in a CUDA graph and replayed.
 */
size_t b200kv_peer_exchange_bytes(int32_t world, int64_t rows);
int32_t b200kv_peer_buffer_alloc(size_t bytes, void** ptr, unsigned char* handle64);
int32_t b200kv_peer_buffer_open(const unsigned char* handle64, void** ptr);
int32_t b200kv_peer_buffer_close(void* ptr);
int32_t b200kv_peer_buffer_free(void* ptr);
int32_t b200kv_peer_merge(void* const* peer_buffers, int32_t world, int32_t rank, int64_t rows, const float* partial_o,
                          const float* partial_m, const float* partial_l, void* out_bf16, float* lse, void* stream,
                          b200kv_status_word* status);
/*
 * Decode attention over this rank's KV-range shard and the merge across the ranks as one call of two kernels:
 * the decode kernel leaves its per-CTA partials in the workspace, and the kernel that merges them pushes the
 * shard's result straight into every rank's exchange buffer, waits (bounded) for the other ranks' and writes
 * the whole sequence's attention to args->out (bf16 [batch][64][512]; args->lse optional) on every rank. The
 * same as b200kv_mla_decode into partial_* followed by b200kv_peer_merge, without the kernel and the pass over
 * the partial in between. args->kv_begin / kv_len select the shard; partial_*, new_latent and new_rope must be
 * null; the exchange buffers are those of b200kv_peer_buffer_alloc for rows = batch * 64. Runs on the
 * tensor-core kernel for batches of fewer than 16 sequences (a long context is one sequence, or a few).
 */
int32_t b200kv_mla_decode_peer(const b200kv_decode_args* args, void* const* peer_buffers, int32_t world, int32_t rank,
                               void* stream, b200kv_status_word* status);

/*
 * The stages on either side of the path (the reference runs them as separate operators).
 *
 * Producer of the appended row, in one kernel instead of the reference's stages 6-8 (kv_a_norm, rope,
 * kv_cache_write: src/pipeline/pipeline.cpp:212-234): for token t, row kv_a[t] = [latent 512 | rope 64]
 * (the kv_a projection's output, src/memory/static_arena_manager.cpp:486-490) becomes
 *   latent' = RMSNorm(latent) * gamma   (epsilon eps; the reference passes 1e-6),
 *   rope'   = rotary embedding of rope, pairing element i with i + 32 (mode "half", pipeline.cpp:51),
 *             with the token's rows cos[t], sin[t] of 64 values (rope_cos / rope_sin [T, 64]),
 * and both are written to pool row slot_mapping[t] (negative: nothing is written; beyond the pool:
 * B200KV_DEV_BAD_SLOT in the status word). The same launch rotates q_rope [T][heads][64] in place when it
 * is given (the reference's rope stage rotates q and k together). latent_out, rope_out (may alias the rope
 * part of kv_a) and rstd_out, when non-null, also receive latent', rope' and the reciprocal RMS, as the
 * reference's activation buffers kv_latent_normed, k_rope and rstd do. All tensors bf16 except rstd (fp32);
 * strides in elements; every tensor 16-byte aligned with strides that are multiples of 8 (a cos / sin
 * stride of 0 shares one row among all tokens). The arithmetic is fixed to the operation (csrc/kv_stages.cu states it), so results do not
 * depend on the launch.
 */
typedef struct b200kv_producer_args {
  b200kv_pool_view pool;
  const void* kv_a;
  int64_t kv_a_stride;
  const void* gamma; /* bf16 [512] */
  float eps;
  const void* cos; /* bf16, row t at cos + t * cos_stride (a stride of 0 shares one row) */
  int64_t cos_stride;
  const void* sin;
  int64_t sin_stride;
  const int32_t* slot_mapping; /* device int32 [n_tokens] */
  int64_t n_tokens;
  void* q_rope; /* bf16 [n_tokens][heads][64] rotated in place, or null */
  int64_t q_token_stride;
  int64_t q_head_stride;
  int32_t heads;
  void* latent_out; /* bf16 [n_tokens][512] or null */
  int64_t latent_out_stride;
  void* rope_out; /* bf16 [n_tokens][64] or null */
  int64_t rope_out_stride;
  float* rstd_out; /* fp32 [n_tokens] or null */
} b200kv_producer_args;

int32_t b200kv_append_fused(const b200kv_producer_args* args, void* stream, b200kv_status_word* status);

/* The producer's two halves on their own, with the same arithmetic: y[r] = RMSNorm(x[r][0..511]) * gamma (the
 * reference's kv_a_norm stage) and the in-place rotation of x [tokens][vectors][64] by the token's cos/sin
 * row (its rope stage, for q_rope [T, 64, 64] and k_rope [T, 1, 64]). */
int32_t b200kv_rmsnorm512(const void* x, int64_t x_stride, const void* gamma, float eps, int64_t rows, void* y,
                          int64_t y_stride, float* rstd, void* stream);
int32_t b200kv_rope_half64(void* x, int64_t token_stride, int64_t vector_stride, const void* cos, int64_t cos_stride,
                           const void* sin, int64_t sin_stride, int64_t tokens, int32_t vectors, void* stream);

/*
 * Consumer of the attention output: block-32 MX quantisation along the last axis, the reference's stage 10
 * (attn_quant, src/pipeline/pipeline.cpp:250-258): x bf16 [rows][cols] -> q FP8 E4M3 [rows][cols] and one
 * E8M0 scale byte per 32 values, scales [rows][cols / 32]. Per block: e = floor(log2 max|x|) - 8 clamped to
 * [-127, 127] (an all-zero block: -127), scale byte = e + 127, q = e4m3(x * 2^-e) rounded to nearest even
 * and saturated at 448; a NaN anywhere in the block gives scale 0xFF and NaN values. cols a multiple of 32;
 * x and q 16-byte aligned, x_stride a multiple of 8, q_stride a multiple of 16 (elements).
 */
int32_t b200kv_mx_quant_e4m3(const void* x, int64_t x_stride, int64_t rows, int64_t cols, void* q, int64_t q_stride,
                             void* scales, int64_t scale_stride, void* stream);

/*
 * Seeded synthetic data on the device: dst[i] = bf16(scale * N(0,1)) for element counters
 * first_element + i of stream (seed, stream_id); splitmix64 counters, Box-Muller in double.
 * Bench and test utility; no counterpart in the reference.
 */
int32_t b200kv_fill_normal_bf16(void* dst, int64_t count, uint64_t seed, uint64_t stream_id,
                                uint64_t first_element, double scale, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Host bookkeeping: KV block pool (free list, per-sequence block tables, admission and release).
 * The reference reserves one block table and one slot per step and never fills the table
 * (src/memory/static_arena_manager.cpp:298-300, 581-582; slot = position,
 * src/pipeline/pipeline.cpp:515-519); batched decode needs the allocator below. It follows the
 * fixed-capacity, plan-then-commit, validate-with-arithmetic pattern of the reference's expert slot
 * pool (src/memory/exclusive_staging.cpp:313-399, 529-572): no allocation after create, a failed call
 * changes nothing.
 * ---------------------------------------------------------------------------------------------- */
typedef struct b200kv_block_pool b200kv_block_pool;

/* free_order: initial free-list order (num_blocks ids) or null for 0..num_blocks-1. */
b200kv_block_pool* b200kv_block_pool_create(int32_t num_blocks, int32_t block_size, int32_t max_seqs,
                                            int32_t max_blocks_per_seq, const int32_t* free_order);
void b200kv_block_pool_destroy(b200kv_block_pool* pool);
int32_t b200kv_block_pool_admit(b200kv_block_pool* pool, int32_t seq);
/* Extends `seq` by n_tokens; writes the new tokens' slots (flat pool rows) to slots_out[0..n). */
int32_t b200kv_block_pool_grow(b200kv_block_pool* pool, int32_t seq, int32_t n_tokens, int32_t* slots_out);
int32_t b200kv_block_pool_release(b200kv_block_pool* pool, int32_t seq);
/* Takes back the last n_tokens of `seq`; blocks that empties return to the FRONT of the free list, so that undoing
 * the most recent grows in reverse order restores tables, lengths and the free list exactly. */
int32_t b200kv_block_pool_ungrow(b200kv_block_pool* pool, int32_t seq, int32_t n_tokens);
int32_t b200kv_block_pool_free_count(const b200kv_block_pool* pool);
int32_t b200kv_block_pool_seq_len(const b200kv_block_pool* pool, int32_t seq);
/* Host views: table [max_seqs][max_blocks_per_seq] (unused entries 0), lens [max_seqs]. */
const int32_t* b200kv_block_pool_table(const b200kv_block_pool* pool);
const int32_t* b200kv_block_pool_lens(const b200kv_block_pool* pool);
/* Free list in queue order; returns the count written (<= capacity). */
int32_t b200kv_block_pool_export_free(const b200kv_block_pool* pool, int32_t* out, int32_t capacity);
/* O(blocks) invariant check; 0 when every block is owned exactly once, else B200KV_ERR_INVALID. */
int32_t b200kv_block_pool_validate(const b200kv_block_pool* pool);

/*
 * KV reservation geometry and paged-attention counters, as the reference computes them
 * (blocks per layer: src/memory/static_arena_manager.cpp:197; pool bytes: :315-318; reported block
 * count and utilisation: src/pipeline/pipeline.cpp:134-136, 532-534;
 * include/moe/diagnostics/inference_stats.hpp:21-28).
 */
typedef struct b200kv_reservation {
  int64_t blocks_per_layer;
  int64_t total_blocks;
  int64_t latent_bytes;
  int64_t rope_bytes;
  int64_t block_table_bytes;
  int64_t slot_mapping_bytes;
} b200kv_reservation;

int32_t b200kv_plan_reservation(int64_t max_context, int64_t block_size, int64_t layers, int64_t max_seqs,
                                int64_t tokens_per_step, b200kv_reservation* out);
double b200kv_utilisation(int64_t active_tokens, int64_t blocks_per_layer, int64_t block_size);
/* The "paged_attention" object of the reference's diagnostics JSON (include/moe/diagnostics/inference_stats.hpp:
 * 21-28, written by src/diagnostics/inference_stats.cpp:42-47), key for key and with its number formatting:
 * total_blocks_allocated = blocks_per_layer * layers, active_context_tokens, block_size, kv_cache_utilization.
 * Writes at most capacity - 1 characters and a terminator; returns the length of the whole text. */
int64_t b200kv_paged_attention_stats_json(int64_t blocks_per_layer, int64_t layers, int64_t active_tokens,
                                          int64_t block_size, char* buffer, int64_t capacity);

/* ------------------------------------------------------------------------------------------------
 * Static arena and the KV cache carved from it.
 * Replaces, for the KV spans, StaticMemoryArena::{Reserve, Commit, Address, NoteWorkspace,
 * CommitWorkspace, AssertWorkspaceFits, Seal, ValidateAlignment}
 * (src/memory/static_arena.cpp:88-124, 275-332) and the KV lines of StaticArenaManager
 * (src/memory/static_arena_manager.cpp:298-300, 315-318). Same three phases and the same refusals:
 * spans are 512-byte aligned by default, Commit performs ONE zero-filled device allocation, nothing
 * can be reserved after Commit, and after Seal nothing can allocate at all. A refusal returns
 * B200KV_ERR_INVALID (reserve: the negated code) with the reason in b200kv_last_error().
 * backend B200KV_ARENA_HOST_SIM serves page-aligned host memory, like the reference's simulated
 * device (src/core/device_ops.cpp:268-440), so that the latches can be tested without a GPU.
 * ---------------------------------------------------------------------------------------------- */
#define B200KV_ARENA_DEVICE 0
#define B200KV_ARENA_HOST_SIM 1
typedef struct b200kv_arena b200kv_arena;

b200kv_arena* b200kv_arena_create(int32_t backend);
void b200kv_arena_destroy(b200kv_arena* arena);
/* Returns a handle >= 0, or the negated error code. align 0 = 512. */
int64_t b200kv_arena_reserve(b200kv_arena* arena, const char* name, size_t bytes, size_t align);
int32_t b200kv_arena_commit(b200kv_arena* arena);
void* b200kv_arena_address(const b200kv_arena* arena, int64_t handle);
int64_t b200kv_arena_offset(const b200kv_arena* arena, int64_t handle);
size_t b200kv_arena_reserved_bytes(const b200kv_arena* arena);
size_t b200kv_arena_bytes(const b200kv_arena* arena);
int32_t b200kv_arena_allocations(const b200kv_arena* arena);
int32_t b200kv_arena_note_workspace(b200kv_arena* arena, uint64_t bytes);
int32_t b200kv_arena_commit_workspace(b200kv_arena* arena);
void* b200kv_arena_workspace(const b200kv_arena* arena);
uint64_t b200kv_arena_workspace_bytes(const b200kv_arena* arena);
int32_t b200kv_arena_workspace_fits(const b200kv_arena* arena, uint64_t bytes);
int32_t b200kv_arena_seal(b200kv_arena* arena);
int32_t b200kv_arena_sealed(const b200kv_arena* arena);
int32_t b200kv_arena_validate(const b200kv_arena* arena);

typedef struct b200kv_kv_cache {
  b200kv_reservation geometry;
  int64_t layers;
  int64_t block_size;
  int64_t max_seqs;
  int64_t block_table_handle; /* "kv.block_table": int32 [max_seqs][blocks_per_layer]     */
  int64_t slot_mapping_handle; /* "kv.slot_mapping": int32 [tokens_per_step]              */
  int64_t latent_handle;      /* "kv.latent_cache": bf16 [layers][blocks][block][512]      */
  int64_t rope_handle;        /* "kv.rope_cache":   bf16 [layers][blocks][block][64]       */
  int64_t max_blocks_per_seq; /* columns of the block table                                */
  int64_t seq_lens_handle;    /* "kv.seq_lens": int32 [max_seqs], or -1 (batched form only) */
} b200kv_kv_cache;

/* Reserves the four KV spans (RESERVE phase) with the reference's geometry: one sequence's blocks per layer,
 * blocks = ceil(max_context / block_size), a table of max_seqs rows of that many columns. */
int32_t b200kv_kv_cache_reserve(b200kv_arena* arena, int64_t max_context, int64_t block_size, int64_t layers,
                                int64_t max_seqs, int64_t tokens_per_step, b200kv_kv_cache* out);
/* The batched form of the same reservation (the reference keeps one token per step and one sequence,
 * src/memory/static_arena_manager.cpp:37-39, 298-300): a pool of num_blocks blocks per layer shared by max_seqs
 * sequences through b200kv_block_pool, a table [max_seqs][max_blocks_per_seq], slots for tokens_per_step
 * appended rows (a decode step appends one per sequence, a prefill chunk many) and the lengths [max_seqs],
 * all int32 and all carved from the same arena under the reference's span names. */
int32_t b200kv_kv_cache_reserve_batched(b200kv_arena* arena, int64_t num_blocks, int64_t block_size, int64_t layers,
                                        int64_t max_seqs, int64_t max_blocks_per_seq, int64_t tokens_per_step,
                                        b200kv_kv_cache* out);
/* One layer's pool view after Commit: base + layer * blocks * block_size * width * 2
 * (src/pipeline/pipeline.cpp:391-395). */
int32_t b200kv_kv_cache_layer_view(const b200kv_arena* arena, const b200kv_kv_cache* cache, int64_t layer,
                                   b200kv_pool_view* out);

/* ------------------------------------------------------------------------------------------------
 * The path as the engine drives it, batched. What Dsv4Pipeline::Build and ::DecodeStep do for the paged cache and
 * the attention stages (src/pipeline/pipeline.cpp:212-258, 496-537), for max_seqs sequences and for prefill chunks
 * of many tokens where the reference keeps one sequence and one token per step
 * (src/memory/static_arena_manager.cpp:37-39; src/pipeline/pipeline.cpp:40, 515-519; apps/moe_runner.cpp:434-439).
 *   create        Build: the KV spans reserved in a static arena, the attention workspace noted, one Commit, the
 *                 workspace, Seal; the block pool; one pinned block for the per-step upload. Nothing allocates
 *                 afterwards.
 *   admit/release a sequence enters with no tokens / leaves and its blocks return to the free list.
 *   begin_step    seqs[i] grows by new_tokens[i] tokens (null: one each, a decode step; more: a prefill chunk).
 *                 Plan, then commit: a step that does not fit (tokens per step, blocks per sequence, free blocks)
 *                 is refused and changes nothing. The step's table rows (row i = seqs[i]), lengths and slots go
 *                 to the device with ONE copy (the reference's slot mailbox, :515-519).
 *   layer_append  stages 6-8 of the reference's layer (kv_a_norm, rope, kv_cache_write) for the step's new tokens,
 *                 rows in step order (all tokens of seqs[0], then seqs[1], ...): b200kv_append_fused.
 *   layer_attend  stage 9 (decode attention of the step's sequences over their whole context) and, when out_fp8
 *                 is given, stage 10 (MX quantisation of the output): decode steps only.
 *   abort_step    a step one of whose launches failed is taken back as a whole.
 *   end_step      the step made no allocation (the reference asserts this per step, :502-503, 535-536) and the
 *                 block pool's invariants hold.
 * Tensors are device pointers, bf16, strides in elements; q is [n_seqs][64][576] with its rope part already
 * rotated or rotated in place by layer_append (q_rope). The status word lives in the arena.
 * ---------------------------------------------------------------------------------------------- */
typedef struct b200kv_engine b200kv_engine;
typedef struct b200kv_engine_config {
  int32_t layers;
  int32_t max_seqs;
  int32_t num_blocks;         /* per layer, shared by all sequences */
  int32_t block_size;         /* rows per block, a multiple of 64 */
  int32_t max_blocks_per_seq; /* columns of the block table */
  int32_t max_step_tokens;    /* new tokens per step: max_seqs for decode, a prefill chunk's total otherwise */
  float scale;                /* softmax scale */
  float eps;                  /* RMSNorm epsilon (the reference passes 1e-6) */
  int32_t backend;            /* B200KV_ARENA_DEVICE; B200KV_ARENA_HOST_SIM runs the bookkeeping without a GPU */
} b200kv_engine_config;

b200kv_engine* b200kv_engine_create(const b200kv_engine_config* config);
void b200kv_engine_destroy(b200kv_engine* engine);
const b200kv_arena* b200kv_engine_arena(const b200kv_engine* engine);
const b200kv_kv_cache* b200kv_engine_cache(const b200kv_engine* engine);
const b200kv_block_pool* b200kv_engine_block_pool(const b200kv_engine* engine);
b200kv_status_word* b200kv_engine_status(const b200kv_engine* engine);
int32_t b200kv_engine_admit(b200kv_engine* engine, int32_t seq);
int32_t b200kv_engine_release(b200kv_engine* engine, int32_t seq);
int32_t b200kv_engine_begin_step(b200kv_engine* engine, const int32_t* seqs, const int32_t* new_tokens, int32_t n_seqs,
                                 void* stream);
int32_t b200kv_engine_layer_append(b200kv_engine* engine, int32_t layer, const void* kv_a, int64_t kv_a_stride,
                                   const void* gamma, const void* cos, int64_t cos_stride, const void* sin,
                                   int64_t sin_stride, void* q_rope, int64_t q_token_stride, int64_t q_head_stride,
                                   void* stream);
int32_t b200kv_engine_layer_attend(b200kv_engine* engine, int32_t layer, const void* q, int64_t q_seq_stride,
                                   int64_t q_head_stride, void* out, void* out_fp8, void* out_scales, void* stream);
int32_t b200kv_engine_end_step(b200kv_engine* engine);
/* Abandons the step in flight (a launch of it failed): every sequence gives back what the step added, tables,
 * lengths and the free list are as before begin_step. */
int32_t b200kv_engine_abort_step(b200kv_engine* engine);
/* The "paged_attention" object of the reference's diagnostics for the engine's current state. */
int64_t b200kv_engine_stats_json(const b200kv_engine* engine, char* buffer, int64_t capacity);

/* ------------------------------------------------------------------------------------------------
 * Multi-GPU work partition (host). No counterpart in the reference, which runs on one device
 * (include/moe/core/config.hpp:280).
 * ---------------------------------------------------------------------------------------------- */
/* Batched decode: whole sequences to ranks by longest-processing-time greedy on context length.
 * rank_of_seq [n_seqs] receives each sequence's rank; tokens_per_rank [n_ranks] (or null) the loads. */
int32_t b200kv_partition_sequences(const int32_t* kv_len, int32_t n_seqs, int32_t n_ranks, int32_t* rank_of_seq,
                                   int64_t* tokens_per_rank);
/* One long sequence: shard `rank` is a contiguous block range; *begin is a multiple of block_size and
 * feeds b200kv_decode_args.kv_begin, *len feeds kv_len. The shard partials merge with b200kv_lse_merge. */
int32_t b200kv_split_kv_range(int32_t kv_len, int32_t block_size, int32_t n_ranks, int32_t rank, int32_t* begin,
                              int32_t* len);

#ifdef __cplusplus
}
#endif
#endif /* B200KV_H_ */
