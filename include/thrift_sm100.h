/*
 * libthrift_sm100 — C ABI of the sm_100a (B200) selective mixed-precision
 * attention library.
 *
 * This header replaces the compiled boundary of the reference project: the
 * plain-C++ kernel launchers that its csrc/bindings.cpp declares (lines 56-247)
 * and calls from the 27 pybind11 functions (lines 1454-1671).  Every entry point
 * takes raw device pointers, sizes and a CUDA stream (as void*), allocates
 * nothing and returns an int:
 *   0 = ok, < 0 = argument error (TA100_ERR_*), > 0 = a cudaError_t value.
 * State the library keeps per device: a status word that the decode kernels raise
 * when a bounded wait runs out (ta100_decode_status reads and clears it) and the
 * fixed scratch array of ta100_decode_attention_static; host side, a cache of that
 * array's device address behind a mutex.  Everything else is re-entrant.
 * Calls are asynchronous with respect to the host unless stated otherwise.
 *
 * Conventions
 *   - "16-bit" inputs are IEEE half (is_bf16 = 0) or bfloat16 (is_bf16 = 1).
 *   - NVFP4: e2m1 codes, one E4M3 scale per 16 values.  MXFP4: e2m1 codes, one
 *     E8M0 scale per 32 values (is_mxfp4 = 1).
 *   - Packed codes: byte i holds element 2i in bits 0..3 and 2i+1 in bits 4..7.
 *   - Row layouts: codes [heads, seq, D/2], scales [heads, seq, D/G].
 *   - Transposed layout (V): codes [heads, D, P/2], scales [heads, D, P/G] with
 *     P = ceil(seq/128)*128, groups running along the sequence.
 *   - Selection lists are int32, rank ordered, -1 padded.
 */
#ifndef THRIFT_SM100_H
#define THRIFT_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define TA100_OK 0
#define TA100_ERR_NULL (-1)
#define TA100_ERR_SHAPE (-2)
#define TA100_ERR_UNSUPPORTED (-3)
#define TA100_ERR_ALIGN (-4)
#define TA100_ERR_WORKSPACE (-5)
#define TA100_ERR_TENSOR_MAP (-6)
#define TA100_ERR_DEVICE_TIMEOUT (-7)
#define TA100_ERR_LIMIT (-8)
#define TA100_ERR_STATIC_SCRATCH (-9)
#define TA100_ERR_PAGE_TABLE (-10)

int ta100_version(void);
const char* ta100_status_string(int status);

/*
 * Diagnostics for the give-up path of the attention kernels (no counterpart in the reference, whose kernels
 * wait without bound).  Every device-side wait in this library is bounded by a cycle budget; when one runs
 * out the kernel raises a CTA-wide flag, every role drains, tensor memory is released and the launch's
 * status word reports TA100_ERR_DEVICE_TIMEOUT (ta100_prefill_status / ta100_decode_status).
 *   budget_cycles  cycle budget of later launches (<= 0 restores the default of 1e9 cycles)
 *   skip_loads     non-zero: the producer warps of later attention launches issue no copies at all, so the
 *                  consumers' waits run out while nothing asynchronous is in flight
 * Process-wide, not thread-safe: meant for tests only.
 */
int ta100_debug_set_wait(long long budget_cycles, int skip_loads);

/*
 * Quantise x [bs, seq, head_dim] (16-bit) to packed FP4 codes and block scales.
 * layout: 0 plain rows, 1 rows permuted inside every 32-row group (physical row p
 * holds logical row (p/8)*2 + ((p%8)/2)*8 + p%2), 2 transposed, 3 transposed +
 * permuted.  head_dim 64 or 128.
 * Replaces nvfp4_quantise / nvfp4_quantise_permute_seq / nvfp4_quantise_transpose /
 * nvfp4_quantise_transpose_permute_seq and the four mxfp4_* twins
 * (bindings.cpp:149-179; kernels csrc/cuda/sm120/nvfp4/quantization.cu:16,162,315,493
 * and csrc/cuda/sm120/mxfp4/quantization.cu:24,185,351,542).
 */
int ta100_quantize(const void* x, void* codes, void* scales, long long bs, int seq, int head_dim, int is_mxfp4,
                   int is_bf16, int layout, void* stream);

/*
 * Q, K and V of one attention call quantised by ONE launch (three parts of one grid):
 *   q [bs_q, seq_q, D]   -> q_codes [bs_q, seq_q, D/2],  q_scales [bs_q, seq_q, D/G]     (plain rows)
 *   k [bs_kv, seq_kv, D] -> k_codes [bs_kv, seq_kv, D/2], k_scales [bs_kv, seq_kv, D/G]  (rows; permuted as layout 1 of
 *                           ta100_quantize when k_permuted != 0: the prefill kernel's K layout)
 *   v [bs_kv, seq_kv, D] -> v_codes_t [bs_kv, D, P/2],    v_scales_t [bs_kv, D, P/G], P = seq_kv rounded up to 128
 * Outputs are bit-identical to three ta100_quantize calls with layouts 0, k_permuted and 2.
 * Replaces the three launches of QuantFormat.quantize_qkv / quantize_single_query_qkv
 * (src/thriftattention/quant/formats.py:55-79 of the reference).
 */
int ta100_quantize_qkv(const void* q, const void* k, const void* v, void* q_codes, void* q_scales, void* k_codes,
                       void* k_scales, void* v_codes_t, void* v_scales_t, long long bs_q, int seq_q, long long bs_kv,
                       int seq_kv, int head_dim, int is_mxfp4, int is_bf16, int k_permuted, void* stream);

/*
 * Per-block statistics of x [heads, seq, head_dim]: fp32 mean cast to the 16-bit
 * type, min and max, each [heads, seq/block, head_dim]; any output may be NULL.
 * Replaces the PyTorch pre-reductions of the reference (block_means,
 * src/thriftattention/selection/block_mean.py:44-54; block_minmax,
 * src/thriftattention/selection/quest.py:11-24).
 */
int ta100_block_stats(const void* x, void* mean, void* mn, void* mx, long long heads, int seq, int head_dim, int block,
                      int is_bf16, void* stream);

/*
 * Fused KV-cache append: one launch stores count new 16-bit K and V rows at token positions
 * [start, start + count) of a capacity-strided cache and brings every derived tensor up to date.
 *   k_new, v_new   [heads, k_count | v_count, D] 16-bit, contiguous; NULL = zero rows, or with
 *                  flags bit 0 (K) / bit 1 (V) = keep the cached rows and only re-quantise them
 *   k_hi, v_hi     [heads, capacity, D] 16-bit caches
 *   k_codes/k_scales   [heads, capacity, D/2] / [heads, capacity, D/G]   (plain row layout)
 *   v_codes_t/v_scales_t [heads, D, capacity/2] / [heads, D, capacity/G] (groups along tokens);
 *                  every G-token group touched by [start, start + v_count) is re-quantised, its
 *                  other tokens being read from v_hi
 *   k_mean, k_min, k_max [heads, capacity/stat_block, D] 16-bit, each may be NULL; refreshed for
 *                  the statistics blocks that [start, start + k_count) completes
 * capacity must be a multiple of 128; stat_block 64 or 128; G = 16 (NVFP4) or 32 (MXFP4).
 * Replaces ThriftAttentionCacheLayer.update and its helpers _quantize_k_range,
 * _quantize_v_range and _refresh_k_means
 * (src/thriftattention/integrations/transformers_cache.py:87-123, 308-351) and, with NULL
 * inputs, the re-quantisation of the zeroed tail in _zero_physical_tail (:237-253).
 */
int ta100_cache_append(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                       void* v_codes_t, void* v_scales_t, void* k_mean, void* k_min, void* k_max, long long heads,
                       int start, int k_count, int v_count, int capacity, int head_dim, int stat_block, int is_mxfp4,
                       int is_bf16, int flags, void* stream);

/*
 * The same append into a PAGED cache: the layout ta100_decode_attention reads through a page table.
 *   page_table     int32 [batch, max_pages]: physical page of logical 64-token page j of sequence b; entries that
 *                  the token range [start, start + count) (and, for V, its G-token groups) touches must be valid
 *                  pages in [0, pool_pages) - a row whose page is not is skipped
 *   k_hi, v_hi     [pool_pages, hkv, 64, D] 16-bit;  k_codes [pool_pages, hkv, 64, D/2], k_scales [.., 64, D/G]
 *   v_codes, v_scales  [pool_pages, hkv, D, 32], [pool_pages, hkv, D, 64/G]  (transposed inside a page)
 *   k_mean, k_min, k_max [batch*hkv, stat_blocks, D] by LOGICAL block, as for the contiguous cache
 *   k_new, v_new   [batch*hkv, count, D]
 * Growing a sequence is appending page ids to its row of the table; nothing is copied.  A page handed to a
 * sequence must hold zeros (the kernels read the rows behind the logical length as zero rows).  No counterpart
 * in the reference, whose cache grows by copying capacity-strided slabs (transformers_cache.py:255-306).
 */
int ta100_cache_append_paged(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                             void* v_codes, void* v_scales, void* k_mean, void* k_min, void* k_max, const void* page_table,
                             int max_pages, int pool_pages, int batch, int hkv, int stat_blocks, int start, int k_count,
                             int v_count, int head_dim, int stat_block, int is_mxfp4, int is_bf16, int flags, void* stream);

/*
 * Prefill block selection.  q_mean [heads, nq, D]; k_a / k_b [heads/group, nk, D].
 * quest = 0: score = q_mean . k_a (k_a = block means); quest = 1: Quest bound with
 * k_a = block minima, k_b = block maxima.  causal: blocks kb <= qb only.
 * out [heads, nq, sink + local + k]: the first `sink` and last `local` valid blocks
 * (forced, extension; pass 0 for the reference behaviour), then the k best of the
 * remaining blocks in rank order; -1 padded.  nk <= 2048.
 * Replaces block_mean_topk and quest_block_topk (bindings.cpp:181-203,
 * csrc/cuda/sm120/shared/block_selection.cu:24,231).
 */
int ta100_select_prefill(const void* q_mean, const void* k_a, const void* k_b, void* out, int heads, int group, int nq,
                         int nk, int head_dim, int k, int causal, int quest, int is_bf16, int sink, int local,
                         void* stream);

/*
 * Decode block selection.  q_grouped [flat_kv_heads, group, D]; k_a / k_b
 * [flat_kv_heads, cap_blocks, D]; score = max over the group; out
 * [flat_kv_heads, sink + local + k].  out_scores (NULL or fp32, same shape) receives the score
 * of every pick (+FLT_MAX for forced blocks, -FLT_MAX for padding): a shard of a longer sequence
 * sends them to its peers so that all derive the same global top-k.  out_stride (0 = sink + local + k) is the
 * distance between rows of out / out_scores in entries; entries past sink + local + k are padding.  Replaces
 * single_query_key_mean_topk, single_query_key_mean_topk_chunked and single_query_quest_topk
 * (bindings.cpp:205-247, block_selection.cu:127,339,450).
 */
int ta100_select_decode(const void* q_grouped, const void* k_a, const void* k_b, void* out, void* out_scores,
                        int flat_kv_heads, int group, int nk, int cap_blocks, int head_dim, int k, int quest, int is_bf16,
                        int sink, int local, int out_stride, void* stream);

/*
 * Decode selection with the KV sequence sharded over `world` GPUs (shard r owns pages
 * [r * total_pages / world, (r + 1) * total_pages / world)).  Every shard calls ta100_select_decode over its
 * own pages with out / out_scores laid out as one buffer [2, rows, width] (plane 0 ids, plane 1 scores) and
 * all-gathers it; `gathered` is the result [world, 2, rows, width].  The union of the shards' candidates is
 * ranked with the single-GPU key (score, then the reference's tie-break on the global page id) and the first
 * top_k are the global selection.  out [rows, sink + local + top_k] receives shard `rank`'s part as LOCAL page
 * ids: its forced pages first, picks at position sink + local + j when pick j lies in this shard, -1 elsewhere.
 * world * width <= 2048.  Exact ties in score are ranked by the global page id here and by the shard-local id
 * inside a shard's own pre-selection; the two orders agree when every shard begins at a multiple of 32 pages.
 * The reference has no multi-GPU path; the merge follows the same argument as its
 * chunked single-GPU top-k (block_selection.cu:443-447).
 */
int ta100_merge_page_candidates(const void* gathered, void* out, int rows, int world, int width, int rank,
                                int total_pages, int top_k, int sink, int local, void* stream);

/* Local windows: out [flat_heads, nq, k] (block_selection.cu:629) and
 * [flat_heads, k] (block_selection.cu:662); replace local_block_topk and
 * single_query_local_topk (bindings.cpp:213-224). */
int ta100_local_block_topk(void* out, long long flat_heads, int nq, int nk, int k, int causal, void* stream);
int ta100_single_query_local_topk(void* out, long long flat_heads, int nk, int k, void* stream);

/* sel [rows, k] -> mask [rows, words] of 64-bit words; replaces pack_topk_mask
 * (bindings.cpp:226-232, block_selection.cu:1260). */
int ta100_pack_topk_mask(const void* sel, void* mask, long long rows, int k, int nk, int words, void* stream);

/*
 * Fused prefill attention: the FP4 pass over non-selected KV blocks and the 16-bit
 * pass over the selected ones in ONE kernel (TMA -> shared memory -> tcgen05 MMA ->
 * tensor memory), online softmax in 64-column steps.
 *   q_hi [B*hq, sq, D], k_hi/v_hi [B*hkv, skv, D] with head stride kv_cap rows;  16-bit, needed when width > 0
 *   sel  [B*hq, sq/block, width] selected KV blocks of `block` (64 or 128) tokens;
 *        width = 0 -> pure FP4 attention
 *   q4/qs rows layout [B*hq, sq, ..]; k4/ks rows layout with head stride kv_cap rows
 *        (k_permuted = 1 when produced with layout 1); v4t/vst transposed layout with
 *        P = ceil(kv_cap/128)*128
 *   out  [B*hq, sq, D] 16-bit, or [B, sq, hq, D] with out_seq_major = 1 (the layout a Transformers
 *        attention function returns, integrations/transformers.py:168,184,200 of the reference, which
 *        transposes and copies instead)
 *   workspace: ta100_prefill_workspace_bytes(...) bytes, 256-byte aligned; holds
 *        re-tiled scale factors and a device status word
 *   round_partial = 1 rounds the running state to the 16-bit type between the two
 *        passes as the reference's two-kernel pipeline does
 *   max_ctas: 0 = one persistent CTA per SM
 * sq and skv multiples of 64, head_dim 64 or 128, skv <= 131072.  causal assumes query
 * row r sees keys <= r.
 * Replaces fp4_attention_{causal,noncausal}_{nvfp4,mxfp4} and
 * thrift_attention_{causal,noncausal}_{nvfp4,mxfp4} (bindings.cpp:56-147; kernels
 * csrc/cuda/sm120/nvfp4/fp4_attention.cu:18, thrift_attention.cu:22,454 and twins).
 */
size_t ta100_prefill_workspace_bytes(int batch, int hq, int hkv, int sq, int skv, int head_dim, int is_mxfp4);
int ta100_prefill_attention(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, int block,
                            const void* q4, const void* k4, const void* v4t, const void* qs, const void* ks,
                            const void* vst, void* out, void* workspace, size_t workspace_bytes, int batch, int hq,
                            int hkv, int sq, int skv, int kv_cap, int head_dim, int causal, int is_mxfp4, int is_bf16,
                            int k_permuted, int round_partial, int max_ctas, int out_seq_major, void* stream);
/* Synchronises `stream` and reports TA100_ERR_DEVICE_TIMEOUT if a bounded wait
 * inside the last prefill launch on this workspace gave up. */
int ta100_prefill_status(const void* workspace, int batch, int hq, int hkv, int sq, int skv, int head_dim, int is_mxfp4,
                         void* stream);

/*
 * Decode (single query token) attention over 64-token pages, split over the KV sequence.
 * Rows are the `group` (<= 16) query heads that share a KV head; head_dim 64 or 128:
 *   q_hi [B*hkv, group, D] 16-bit and its rows-layout quantisation q4 / qs
 *   K/V, contiguous cache (page_table = NULL): k4 / ks rows layout with head stride kv_cap rows
 *        (plain, not permuted), v4 / vs transposed layout with P = ceil(kv_cap/128)*128,
 *        k_hi / v_hi [B*hkv, kv_len, D] with head stride kv_cap rows
 *   K/V, paged pools (page_table int32 [B, max_pages] -> physical page in [0, pool_pages)):
 *        k4 [pool_pages, hkv, 64, D/2], ks [pool_pages, hkv, 64, D/G], v4 [pool_pages, hkv, D, 32],
 *        vs [pool_pages, hkv, D, 64/G], k_hi / v_hi [pool_pages, hkv, 64, D].  An entry outside the pool is
 *        never dereferenced: the kernel leaves that page out and ta100_decode_status reports
 *        TA100_ERR_PAGE_TABLE.  pool_pages is ignored for a contiguous cache.
 *   sel  [B*hkv, width] page ids kept in 16-bit (-1 entries ignored); width = 0 -> pure FP4
 * Chain s of `splits` walks pages [s*n/splits, (s+1)*n/splits): FP4 pages ascending, then the
 * selected pages ascending.  Partial results go to part_o [B*hkv, splits, group, D] (fp32,
 * un-normalised, in units of C = 2688 NVFP4 / 6 MXFP4) and part_ml [B*hkv, splits, group, 2]
 * (row max, row sum); with write_out = 1 they are merged into out [B*hkv, group, D] on the same
 * stream.  kv_len a multiple of 64, head_dim 64 or 128.
 * Replaces fp4_attention_single_query_{nvfp4,mxfp4} and thrift_attention_single_query_{nvfp4,mxfp4}
 * (bindings.cpp:79-92, 132-147; kernels csrc/cuda/sm120/nvfp4/single_query_attention.cu:795,1196,
 * single_query_fp4_attention.cu:718,1116 and twins).  The scratch the reference's binding allocates
 * per call (bindings.cpp:804-807) is the caller-provided part_o / part_ml.
 */
int ta100_decode_pick_splits(int flat_kv_heads, int npages);
size_t ta100_decode_workspace_bytes(int flat_kv_heads, int group, int head_dim, int splits);
int ta100_decode_attention(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width,
                           const void* q4, const void* k4, const void* v4, const void* qs, const void* ks, const void* vs,
                           const void* page_table, int max_pages, int pool_pages, void* out, void* part_o, void* part_ml, int batch,
                           int hkv, int group, int kv_len, int kv_cap, int head_dim, int is_mxfp4, int is_bf16, int splits,
                           int write_out, void* stream);

/*
 * Decode attention for callers that cannot allocate device memory (no counterpart in the
 * reference, whose binding allocates its split-KV workspace on every call).
 *
 * Meant for hosts that gave all free HBM to their own memory pool at start-up, so that a later
 * cudaMalloc would fail, and for latency-critical decode loops that must not take the device-wide
 * synchronisation cudaMalloc / cudaFree imply.  Inputs, `sel` and `out` are still the caller's;
 * only the split-KV partials (what ta100_decode_attention takes as part_o / part_ml) are kept in
 * a fixed 16 MiB device array inside the library, resident on every GPU that loads the library
 * until the process exits.  The call returns TA100_ERR_STATIC_SCRATCH when
 *   batch*hkv*splits*group*(head_dim + 2)*4 bytes (+ alignment)  >  ta100_decode_static_scratch_bytes(),
 * in which case lower `splits` or use ta100_decode_attention.  It never calls cudaMalloc, cudaFree
 * or any allocating routine.
 *
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress, with that
 * device current) and caches it; make that first call before starting any stream capture.  All
 * calls on a device share the array and it keeps the last call's contents: every call rewrites
 * each entry it reads, so no clearing is needed, but two calls that overlap on the GPU (for
 * example on different streams) race on it.  Results are identical to ta100_decode_attention with
 * write_out = 1 and the same `splits`.
 */
size_t ta100_decode_static_scratch_bytes(void);
int ta100_decode_attention_static(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width,
                                  const void* q4, const void* k4, const void* v4, const void* qs, const void* ks,
                                  const void* vs, const void* page_table, int max_pages, int pool_pages, void* out, int batch, int hkv,
                                  int group, int kv_len, int kv_cap, int head_dim, int is_mxfp4, int is_bf16, int splits,
                                  void* stream);

/*
 * Device status of the decode kernels on the current device.  Every wait inside the kernel is
 * bounded; when one runs out the kernel drains, releases its tensor memory and raises a flag.
 * This call synchronises with `stream`, returns TA100_ERR_DEVICE_TIMEOUT if the flag was raised
 * since the previous call (and clears it), TA100_ERR_PAGE_TABLE if a kernel skipped a page-table
 * entry that pointed outside the pool, else TA100_OK.  The reference kernels have no
 * counterpart: their launches are not checked at all
 * (csrc/cuda/sm120/nvfp4/single_query_attention.cu launch sites).
 */
int ta100_decode_status(void* stream);

/*
 * All-gather of a small per-rank buffer over NVLink peer memory in one kernel launch per rank - the exchange step of
 * the KV-sequence-sharded decode (page candidates; one (o, m, l) partial per head), where a library collective is
 * pure latency.  One process per GPU:
 *   ta100_peer_exchange_create   allocates this rank's region for `world` (<= 8) ranks x slot_bytes (a multiple of
 *                                16) and returns its 64-byte CUDA IPC handle; the ranks exchange the handles by any
 *                                means (e.g. an all-gather of bytes) and
 *   ta100_peer_exchange_open     map every peer's region (close / destroy undo the two).
 *   ta100_peer_all_gather        src [bytes] (<= slot_bytes, multiple of 16) of every rank -> out [world, bytes] on
 *                                every rank.  regions = host array of `world` device pointers, index = rank, own
 *                                region included.  The kernel stores src into slot `rank` of every region (plain
 *                                16-byte peer stores; no multicast, no loads from peer memory), publishes a flag on
 *                                every peer, waits with a cycle budget for the flags of all ranks in its own region
 *                                and copies the gathered rows to out.  The step counter lives in the region, so the
 *                                launch has the same arguments every step and replays from a CUDA graph.  Every rank
 *                                must call it the same number of times; the kernels of the ranks wait for each
 *                                other, so each rank needs a GPU of its own.
 *   ta100_peer_exchange_status   synchronises and returns TA100_ERR_DEVICE_TIMEOUT if a wait ran out (a peer never
 *                                arrived: out then holds zeros), clearing the mark.
 * No counterpart in the reference, which is single-GPU.
 */
int ta100_peer_exchange_create(int world, long long slot_bytes, void** region, unsigned char* handle64);
int ta100_peer_exchange_open(const unsigned char* handle64, void** region);
int ta100_peer_exchange_close(void* region);
int ta100_peer_exchange_destroy(void* region);
int ta100_peer_all_gather(const void* src, void* out, long long bytes, long long slot_bytes, int world, int rank,
                          void* const* regions, void* stream);
int ta100_peer_exchange_status(void* region, int world, long long slot_bytes, void* stream);

/*
 * Log-sum-exp merge of decode partials from `shards` producers (e.g. GPUs that each hold a slice
 * of the KV sequence): part_o [shards, flat_kv_heads, splits, group, D], part_ml [.., 2] ->
 * out [flat_kv_heads, group, D].  shard_stride_o / shard_stride_ml: floats between consecutive shards (0 = densely
 * packed), so that the two arrays may be the two parts of one all-gathered buffer per shard.  Same formula as
 * the reference's in-kernel merge (csrc/cuda/sm120/nvfp4/single_query_attention.cu:1562-1593).
 */
int ta100_merge_partials(const void* part_o, const void* part_ml, void* out, int shards, long long shard_stride_o,
                         long long shard_stride_ml, long long flat_kv_heads, int splits, int group, int head_dim,
                         int is_mxfp4, int is_bf16, void* stream);

/*
 * One decode step over a contiguous (capacity-strided) cache in a single call: quantise the grouped query
 * q [B*hkv, group, D] into the caller's q4 / qs, select top_k (+ sink + local) of the first n_select_blocks
 * 64-token blocks by block mean (stat_b = NULL, stat_a = means) or Quest (stat_a = minima, stat_b = maxima;
 * both [B*hkv, stat_cap_blocks, D]) into sel [B*hkv, top_k + sink + local], then split-KV attention and merge
 * into out [B*hkv, group, D].  The three launches are those of ta100_quantize, ta100_select_decode and
 * ta100_decode_attention with the same arguments; one call saves the host the per-call overhead, which at batch 1
 * exceeds the device time.  Replaces the body of cached_decode_attention
 * (integrations/transformers_cache.py:570-619 of the reference: quantize_single_query_qkv, select_key_blocks and
 * the single-query operator).
 */
int ta100_cached_decode_step(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                             const void* ks, const void* v4t, const void* vst, const void* stat_a, const void* stat_b,
                             void* sel, void* out, void* part_o, void* part_ml, int batch, int hkv, int group, int kv_len,
                             int kv_cap, int stat_cap_blocks, int n_select_blocks, int top_k, int sink, int local,
                             int head_dim, int is_mxfp4, int is_bf16, int splits, void* stream);

/*
 * The same step over a PAGED cache (pools and page table as for ta100_decode_attention; the block statistics are
 * indexed by logical block as above).  What a paged ThriftAttentionCache layer calls once per layer and token.
 */
int ta100_cached_decode_step_paged(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                                   const void* ks, const void* v4, const void* vs, const void* page_table, int max_pages,
                                   int pool_pages, const void* stat_a, const void* stat_b, void* sel, void* out,
                                   void* part_o, void* part_ml, int batch, int hkv, int group, int kv_len,
                                   int stat_cap_blocks, int n_select_blocks, int top_k, int sink, int local, int head_dim,
                                   int is_mxfp4, int is_bf16, int splits, void* stream);

/*
 * A generation step whose launches do not change from token to token.
 *
 * The three entries below read the number of cached tokens from device memory (len_dev: ONE int32 for the whole
 * batch with len_count = 1, or one per sequence with len_count = batch - a ragged batch) instead of
 * taking it as an argument, so that append + decode step of every layer, captured once in a CUDA graph, replay for
 * every later token: nothing on the host depends on the length any more (with a paged cache the page table is the
 * only other thing that changes, once per 64 tokens, in place).  A step is
 *     for every layer: ta100_cache_append_at(.., len_dev, n, 0, 1, 1, ..); ta100_cached_decode_step_at(.., len_dev, n, 1, ..)
 *     ta100_advance_length(len_dev, n, 1, capacity)
 * and computes bit for bit what ta100_cache_append[_paged] + ta100_cached_decode_step[_paged] compute when they are
 * given the same length, block counts and chain count as launch parameters.
 * No counterpart in the reference, whose cache keeps its length in Python (transformers_cache.py:64-84).
 *
 * ta100_cache_append_at: the append of ta100_cache_append (page_table NULL; capacity = tokens per head of the slabs)
 * or ta100_cache_append_paged (page_table given; capacity ignored) at position start_dev[sequence or 0] +
 * start_offset.  A range that would end beyond the capacity is not stored at all.
 */
int ta100_cache_append_at(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                          void* v_codes, void* v_scales, void* k_mean, void* k_min, void* k_max, const void* page_table,
                          int max_pages, int pool_pages, int batch, int hkv, int stat_blocks, int capacity,
                          const void* start_dev, int start_count, int start_offset, int k_count, int v_count, int head_dim,
                          int stat_block, int is_mxfp4, int is_bf16, int flags, void* stream);

/*
 * ta100_cached_decode_step_at: the step of ta100_cached_decode_step (page_table NULL) or _paged over
 * tokens = len_dev[sequence or 0] + len_offset cached tokens.  On the device: the kernel length is tokens rounded up to whole pages
 * (at least one), the blocks scored are the complete ones, n = tokens / 64; top_k >= 0 selects min(top_k, n) of
 * them, top_k < 0 selects max(1, round-half-even(fraction * n)) (0 when n == 0); the last `local` and then the first
 * `sink` blocks are forced as far as n minus the selected count leaves room (none when nothing is selected) - the
 * rule of cached_decode_attention (transformers_cache.py:570-619 with resolve_top_k, selection/counts.py).
 *   max_len      multiple of 64: the longest sequence the launch must cope with; fixes the grid (splits chains per
 *                KV head, ceil(max_len / 64 / splits) <= 1024 pages each) - chains beyond the pages of a shorter
 *                sequence write neutral partials
 *   sel, sel_stride   int32 [batch*hkv, sel_stride] selection rows, -1 padded; sel_stride >= the widest row, i.e.
 *                the counts above for max_len
 *   part_o, part_ml   as for ta100_decode_attention with `splits` chains
 * The 16-bit caches are always needed.  len_dev: int32, 4-byte aligned, on the device.
 */
int ta100_cached_decode_step_at(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                                const void* ks, const void* v4, const void* vs, const void* page_table, int max_pages,
                                int pool_pages, const void* stat_a, const void* stat_b, void* sel, int sel_stride, void* out,
                                void* part_o, void* part_ml, int batch, int hkv, int group, const void* len_dev,
                                int len_count, int len_offset, int max_len, int kv_cap, int stat_cap_blocks, int top_k,
                                double fraction, int sink, int local, int head_dim, int is_mxfp4, int is_bf16, int splits,
                                void* stream);

/*
 * The block counts ta100_cached_decode_step_at derives on the device for `tokens` cached tokens, computed on the host
 * (no GPU needed): counts4 = {complete blocks scored (at most 2048), blocks selected by score, forced sink blocks,
 * forced local blocks}.  Sizing helper (the widest selection row is counts4[1] + sink + local at the longest length)
 * and the statement of the rule that tests compare with resolve_top_k (src/thriftattention/selection/counts.py).
 */
int ta100_decode_step_counts(int tokens, int top_k, double fraction, int sink, int local, int* counts4);

/* len_dev[i] = min(len_dev[i] + count, limit) for i < len_count, in stream order: the end of a step. */
int ta100_advance_length(void* len_dev, int len_count, int count, int limit, void* stream);

/*
 * The merge of one producer's chains that stays a partial: part_o [flat_kv_heads, splits, group, D],
 * part_ml [.., 2] -> out_o [flat_kv_heads, 1, group, D] (fp32, units of C), out_ml [flat_kv_heads, 1, group, 2]
 * (row maximum, row sum), i.e. the same arrays with splits = 1.  A GPU that holds a slice of the KV sequence
 * reduces its own chains with this before the exchange, so that the bytes it sends do not grow with its chain
 * count; ta100_merge_partials(shards = N, splits = 1) finishes.  No counterpart in the reference (single GPU).
 */
int ta100_reduce_partials(const void* part_o, const void* part_ml, void* out_o, void* out_ml, long long flat_kv_heads,
                          int splits, int group, int head_dim, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* THRIFT_SM100_H */
