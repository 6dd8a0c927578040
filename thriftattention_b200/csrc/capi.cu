// C ABI of libthrift_sm100.so.  Declarations and contracts: include/thrift_sm100.h.
#include <cstddef>
#include <cstdint>

#include "common.cuh"

namespace ta100 {
int quantize_dispatch(const void*, void*, void*, long long, int, int, int, int, int, cudaStream_t);
int quantize_qkv_dispatch(const void*, const void*, const void*, void*, void*, void*, void*, void*, void*, long long, int,
                          long long, int, int, int, int, int, cudaStream_t);
int block_stats_dispatch(const void*, void*, void*, void*, long long, int, int, int, int, cudaStream_t);
int select_prefill_dispatch(const void*, const void*, const void*, void*, int, int, int, int, int, int, int, int, int, int,
                            int, cudaStream_t);
int select_decode_dispatch(const void*, const void*, const void*, void*, void*, int, int, int, int, int, int, int, int, int, int,
                           int, const DynLength*, cudaStream_t);
int merge_page_candidates_dispatch(const void*, void*, int, int, int, int, int, int, int, int, cudaStream_t);
int local_prefill_dispatch(void*, long long, int, int, int, int, cudaStream_t);
int local_decode_dispatch(void*, long long, int, int, cudaStream_t);
int pack_mask_dispatch(const void*, void*, long long, int, int, int, cudaStream_t);
size_t prefill_workspace_bytes(int, int, int, int, int, int, int);
int prefill_dispatch(const void*, const void*, const void*, const void*, int, int, const void*, const void*, const void*,
                     const void*, const void*, const void*, void*, void*, size_t, int, int, int, int, int, int, int, int,
                     int, int, int, int, int, int, cudaStream_t);
int prefill_status(const void*, int, int, int, int, int, int, int, cudaStream_t);
int decode_pick_splits(int, int);
size_t decode_workspace_bytes(int, int, int, int);
int decode_dispatch(const void*, const void*, const void*, const void*, int, const void*, const void*, const void*,
                    const void*, const void*, const void*, const void*, int, int, void*, void*, void*, int, int, int, int, int,
                    int, int, int, int, int, const void*, int, int, cudaStream_t);
int merge_dispatch(const void*, const void*, void*, int, long long, long long, long long, int, int, int, int, int,
                   cudaStream_t);
int reduce_partials_dispatch(const void*, const void*, void*, void*, long long, int, int, int, cudaStream_t);
int decode_status(cudaStream_t);
size_t decode_static_scratch_bytes();
int decode_static_dispatch(const void*, const void*, const void*, const void*, int, const void*, const void*, const void*,
                           const void*, const void*, const void*, const void*, int, int, void*, int, int, int, int, int, int, int,
                           int, int, cudaStream_t);
size_t peer_exchange_region_bytes(int, long long);
int peer_exchange_create(int, long long, void**, unsigned char*);
int peer_exchange_open(const unsigned char*, void**);
int peer_exchange_close(void*);
int peer_exchange_destroy(void*);
int peer_all_gather_dispatch(const void*, void*, long long, long long, int, int, void* const*, cudaStream_t);
int peer_exchange_status(void*, int, long long, cudaStream_t);
int cache_append_dispatch(const void*, const void*, void*, void*, void*, void*, void*, void*, void*, void*, void*, long long,
                          int, int, int, int, int, int, int, int, int, const void*, int, int, int, int, const void*, int,
                          cudaStream_t);
int advance_length_dispatch(void*, int, int, int, cudaStream_t);
}  // namespace ta100

namespace ta100 {
long long g_wait_budget_cycles = DEFAULT_WAIT_BUDGET;
int g_test_skip_loads = 0;
}  // namespace ta100

using namespace ta100;
static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int ta100_version(void) { return 100; }

int ta100_debug_set_wait(long long budget_cycles, int skip_loads) {
    g_wait_budget_cycles = budget_cycles > 0 ? budget_cycles : DEFAULT_WAIT_BUDGET;
    g_test_skip_loads = skip_loads ? 1 : 0;
    return TA100_OK;
}

const char* ta100_status_string(int status) {
    switch (status) {
        case TA100_OK: return "ok";
        case TA100_ERR_NULL: return "null pointer argument";
        case TA100_ERR_SHAPE: return "inconsistent or unsupported shape";
        case TA100_ERR_UNSUPPORTED: return "unsupported head_dim, block size or format";
        case TA100_ERR_ALIGN: return "pointer is not sufficiently aligned";
        case TA100_ERR_WORKSPACE: return "workspace too small";
        case TA100_ERR_TENSOR_MAP: return "tensor map creation failed";
        case TA100_ERR_DEVICE_TIMEOUT: return "a device-side wait timed out";
        case TA100_ERR_LIMIT: return "size beyond a compiled-in limit";
        case TA100_ERR_PAGE_TABLE:
            return "a page-table entry pointed outside the page pool; that page was left out of the attention";
        case TA100_ERR_STATIC_SCRATCH:
            return "problem needs more split-KV scratch than the library's fixed 16 MiB array; use ta100_decode_attention";
        default: return status > 0 ? cudaGetErrorString(static_cast<cudaError_t>(status)) : "unknown status";
    }
}

int ta100_quantize(const void* x, void* codes, void* scales, long long bs, int seq, int head_dim, int is_mxfp4,
                   int is_bf16, int layout, void* stream) {
    return quantize_dispatch(x, codes, scales, bs, seq, head_dim, is_mxfp4, is_bf16, layout, S(stream));
}

int ta100_quantize_qkv(const void* q, const void* k, const void* v, void* q_codes, void* q_scales, void* k_codes,
                       void* k_scales, void* v_codes_t, void* v_scales_t, long long bs_q, int seq_q, long long bs_kv,
                       int seq_kv, int head_dim, int is_mxfp4, int is_bf16, int k_permuted, void* stream) {
    return quantize_qkv_dispatch(q, k, v, q_codes, q_scales, k_codes, k_scales, v_codes_t, v_scales_t, bs_q, seq_q, bs_kv,
                                 seq_kv, head_dim, is_mxfp4, is_bf16, k_permuted, S(stream));
}

int ta100_block_stats(const void* x, void* mean, void* mn, void* mx, long long heads, int seq, int head_dim, int block,
                      int is_bf16, void* stream) {
    return block_stats_dispatch(x, mean, mn, mx, heads, seq, head_dim, block, is_bf16, S(stream));
}

int ta100_cache_append(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                       void* v_codes_t, void* v_scales_t, void* k_mean, void* k_min, void* k_max, long long heads,
                       int start, int k_count, int v_count, int capacity, int head_dim, int stat_block, int is_mxfp4,
                       int is_bf16, int flags, void* stream) {
    return cache_append_dispatch(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes_t, v_scales_t, k_mean, k_min, k_max,
                                 heads, start, k_count, v_count, capacity, head_dim, stat_block, is_mxfp4, is_bf16, flags,
                                 nullptr, 0, 0, 0, 0, nullptr, 0, S(stream));
}

int ta100_cache_append_paged(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                             void* v_codes, void* v_scales, void* k_mean, void* k_min, void* k_max, const void* page_table,
                             int max_pages, int pool_pages, int batch, int hkv, int stat_blocks, int start, int k_count,
                             int v_count, int head_dim, int stat_block, int is_mxfp4, int is_bf16, int flags, void* stream) {
    if (!page_table) return TA100_ERR_NULL;
    if (batch <= 0 || hkv <= 0) return TA100_ERR_SHAPE;
    return cache_append_dispatch(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes, v_scales, k_mean, k_min, k_max,
                                 static_cast<long long>(batch) * hkv, start, k_count, v_count, 0, head_dim, stat_block,
                                 is_mxfp4, is_bf16, flags, page_table, max_pages, pool_pages, hkv, stat_blocks, nullptr, 0,
                                 S(stream));
}

int ta100_cache_append_at(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                          void* v_codes, void* v_scales, void* k_mean, void* k_min, void* k_max, const void* page_table,
                          int max_pages, int pool_pages, int batch, int hkv, int stat_blocks, int capacity,
                          const void* start_dev, int start_count, int start_offset, int k_count, int v_count, int head_dim,
                          int stat_block, int is_mxfp4, int is_bf16, int flags, void* stream) {
    if (!start_dev) return TA100_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(start_dev) & 3) return TA100_ERR_ALIGN;
    if (start_count != 1 && start_count != batch) return TA100_ERR_SHAPE;
    return cache_append_dispatch(k_new, v_new, k_hi, v_hi, k_codes, k_scales, v_codes, v_scales, k_mean, k_min, k_max,
                                 static_cast<long long>(batch) * hkv, start_offset, k_count, v_count,
                                 page_table ? 0 : capacity, head_dim, stat_block, is_mxfp4, is_bf16, flags, page_table,
                                 max_pages, pool_pages, hkv, stat_blocks, start_dev, start_count > 1 ? 1 : 0, S(stream));
}

int ta100_decode_step_counts(int tokens, int top_k, double fraction, int sink, int local, int* counts4) {
    if (!counts4) return TA100_ERR_NULL;
    if (tokens < 0 || sink < 0 || local < 0) return TA100_ERR_SHAPE;
    DynLength d{};
    d.top_k = top_k;
    d.share = fraction;
    d.sink = sink;
    d.local = local;
    dyn_select_counts(d, tokens, 2048, counts4[0], counts4[1], counts4[2], counts4[3]);
    return TA100_OK;
}

int ta100_advance_length(void* len_dev, int len_count, int count, int limit, void* stream) {
    return advance_length_dispatch(len_dev, len_count, count, limit, S(stream));
}

int ta100_select_prefill(const void* q_mean, const void* k_a, const void* k_b, void* out, int heads, int group, int nq,
                         int nk, int head_dim, int k, int causal, int quest, int is_bf16, int sink, int local,
                         void* stream) {
    return select_prefill_dispatch(q_mean, k_a, k_b, out, heads, group, nq, nk, head_dim, k, causal, quest, is_bf16, sink,
                                   local, S(stream));
}

int ta100_select_decode(const void* q_grouped, const void* k_a, const void* k_b, void* out, void* out_scores,
                        int flat_kv_heads, int group, int nk, int cap_blocks, int head_dim, int k, int quest, int is_bf16,
                        int sink, int local, int out_stride, void* stream) {
    return select_decode_dispatch(q_grouped, k_a, k_b, out, out_scores, flat_kv_heads, group, nk, cap_blocks, head_dim, k,
                                  quest, is_bf16, sink, local, out_stride, nullptr, S(stream));
}

int ta100_merge_page_candidates(const void* gathered, void* out, int rows, int world, int width, int rank,
                                int total_pages, int top_k, int sink, int local, void* stream) {
    return merge_page_candidates_dispatch(gathered, out, rows, world, width, rank, total_pages, top_k, sink, local,
                                          S(stream));
}

int ta100_local_block_topk(void* out, long long flat_heads, int nq, int nk, int k, int causal, void* stream) {
    return local_prefill_dispatch(out, flat_heads, nq, nk, k, causal, S(stream));
}

int ta100_single_query_local_topk(void* out, long long flat_heads, int nk, int k, void* stream) {
    return local_decode_dispatch(out, flat_heads, nk, k, S(stream));
}

int ta100_pack_topk_mask(const void* sel, void* mask, long long rows, int k, int nk, int words, void* stream) {
    return pack_mask_dispatch(sel, mask, rows, k, nk, words, S(stream));
}

size_t ta100_prefill_workspace_bytes(int batch, int hq, int hkv, int sq, int skv, int head_dim, int is_mxfp4) {
    return prefill_workspace_bytes(batch, hq, hkv, sq, skv, head_dim, is_mxfp4);
}

int ta100_prefill_attention(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, int block,
                            const void* q4, const void* k4, const void* v4t, const void* qs, const void* ks,
                            const void* vst, void* out, void* workspace, size_t workspace_bytes, int batch, int hq,
                            int hkv, int sq, int skv, int kv_cap, int head_dim, int causal, int is_mxfp4, int is_bf16,
                            int k_permuted, int round_partial, int max_ctas, int out_seq_major, void* stream) {
    return prefill_dispatch(q_hi, k_hi, v_hi, sel, width, block, q4, k4, v4t, qs, ks, vst, out, workspace, workspace_bytes,
                            batch, hq, hkv, sq, skv, kv_cap, head_dim, causal, is_mxfp4, is_bf16, k_permuted,
                            round_partial, max_ctas, out_seq_major, S(stream));
}

int ta100_prefill_status(const void* workspace, int batch, int hq, int hkv, int sq, int skv, int head_dim, int is_mxfp4,
                         void* stream) {
    return prefill_status(workspace, batch, hq, hkv, sq, skv, head_dim, is_mxfp4, S(stream));
}

int ta100_decode_pick_splits(int flat_kv_heads, int npages) { return decode_pick_splits(flat_kv_heads, npages); }

size_t ta100_decode_workspace_bytes(int flat_kv_heads, int group, int head_dim, int splits) {
    return decode_workspace_bytes(flat_kv_heads, group, head_dim, splits);
}

int ta100_decode_attention(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width,
                           const void* q4, const void* k4, const void* v4, const void* qs, const void* ks, const void* vs,
                           const void* page_table, int max_pages, int pool_pages, void* out, void* part_o, void* part_ml, int batch,
                           int hkv, int group, int kv_len, int kv_cap, int head_dim, int is_mxfp4, int is_bf16, int splits,
                           int write_out, void* stream) {
    return decode_dispatch(q_hi, k_hi, v_hi, sel, width, q4, k4, v4, qs, ks, vs, page_table, max_pages, pool_pages, out, part_o,
                           part_ml, batch, hkv, group, kv_len, kv_cap, head_dim, is_mxfp4, is_bf16, splits, write_out,
                           nullptr, 0, 0, S(stream));
}

int ta100_cached_decode_step(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                             const void* ks, const void* v4t, const void* vst, const void* stat_a, const void* stat_b,
                             void* sel, void* out, void* part_o, void* part_ml, int batch, int hkv, int group, int kv_len,
                             int kv_cap, int stat_cap_blocks, int n_select_blocks, int top_k, int sink, int local,
                             int head_dim, int is_mxfp4, int is_bf16, int splits, void* stream) {
    const long long flat = static_cast<long long>(batch) * hkv;
    int rc = quantize_dispatch(q, q4, qs, flat, group, head_dim, is_mxfp4, is_bf16, 0, S(stream));
    if (rc != TA100_OK) return rc;
    const int width = top_k + sink + local;
    if (width > 0) {
        rc = select_decode_dispatch(q, stat_a, stat_b, sel, nullptr, static_cast<int>(flat), group, n_select_blocks,
                                    stat_cap_blocks, head_dim, top_k, stat_b != nullptr, is_bf16, sink, local, 0, nullptr,
                                    S(stream));
        if (rc != TA100_OK) return rc;
    }
    return decode_dispatch(q, k_hi, v_hi, width > 0 ? sel : nullptr, width, q4, k4, v4t, qs, ks, vst, nullptr, 0, 0, out, part_o,
                           part_ml, batch, hkv, group, kv_len, kv_cap, head_dim, is_mxfp4, is_bf16, splits, 1, nullptr, 0, 0,
                           S(stream));
}

int ta100_cached_decode_step_paged(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                                   const void* ks, const void* v4, const void* vs, const void* page_table, int max_pages,
                                   int pool_pages, const void* stat_a, const void* stat_b, void* sel, void* out,
                                   void* part_o, void* part_ml, int batch, int hkv, int group, int kv_len,
                                   int stat_cap_blocks, int n_select_blocks, int top_k, int sink, int local, int head_dim,
                                   int is_mxfp4, int is_bf16, int splits, void* stream) {
    if (!page_table) return TA100_ERR_NULL;
    const long long flat = static_cast<long long>(batch) * hkv;
    int rc = quantize_dispatch(q, q4, qs, flat, group, head_dim, is_mxfp4, is_bf16, 0, S(stream));
    if (rc != TA100_OK) return rc;
    const int width = top_k + sink + local;
    if (width > 0) {
        rc = select_decode_dispatch(q, stat_a, stat_b, sel, nullptr, static_cast<int>(flat), group, n_select_blocks,
                                    stat_cap_blocks, head_dim, top_k, stat_b != nullptr, is_bf16, sink, local, 0, nullptr,
                                    S(stream));
        if (rc != TA100_OK) return rc;
    }
    return decode_dispatch(q, k_hi, v_hi, width > 0 ? sel : nullptr, width, q4, k4, v4, qs, ks, vs, page_table, max_pages,
                           pool_pages, out, part_o, part_ml, batch, hkv, group, kv_len, kv_len, head_dim, is_mxfp4, is_bf16,
                           splits, 1, nullptr, 0, 0, S(stream));
}

int ta100_cached_decode_step_at(const void* q, void* q4, void* qs, const void* k_hi, const void* v_hi, const void* k4,
                                const void* ks, const void* v4, const void* vs, const void* page_table, int max_pages,
                                int pool_pages, const void* stat_a, const void* stat_b, void* sel, int sel_stride, void* out,
                                void* part_o, void* part_ml, int batch, int hkv, int group, const void* len_dev,
                                int len_count, int len_offset, int max_len, int kv_cap, int stat_cap_blocks, int top_k,
                                double fraction, int sink, int local, int head_dim, int is_mxfp4, int is_bf16, int splits,
                                void* stream) {
    if (!len_dev || !stat_a || !sel) return TA100_ERR_NULL;
    if (reinterpret_cast<uintptr_t>(len_dev) & 3) return TA100_ERR_ALIGN;
    if (max_len <= 0 || max_len % 64 != 0 || sel_stride <= 0) return TA100_ERR_SHAPE;
    if ((len_count != 1 && len_count != batch) || hkv <= 0) return TA100_ERR_SHAPE;
    const long long flat = static_cast<long long>(batch) * hkv;
    int rc = quantize_dispatch(q, q4, qs, flat, group, head_dim, is_mxfp4, is_bf16, 0, S(stream));
    if (rc != TA100_OK) return rc;
    DynLength dyn{};
    dyn.len = static_cast<const int32_t*>(len_dev);
    dyn.hkv_per_seq = len_count > 1 ? hkv : 0;
    dyn.offset = len_offset;
    dyn.top_k = top_k;
    dyn.share = fraction;
    dyn.sink = sink;
    dyn.local = local;
    rc = select_decode_dispatch(q, stat_a, stat_b, sel, nullptr, static_cast<int>(flat), group, max_len / 64,
                                stat_cap_blocks, head_dim, 0, stat_b != nullptr, is_bf16, 0, 0, sel_stride, &dyn, S(stream));
    if (rc != TA100_OK) return rc;
    return decode_dispatch(q, k_hi, v_hi, sel, sel_stride, q4, k4, v4, qs, ks, vs, page_table, max_pages, pool_pages, out,
                           part_o, part_ml, batch, hkv, group, max_len, page_table ? max_len : kv_cap, head_dim, is_mxfp4,
                           is_bf16, splits, 1, len_dev, len_count > 1 ? 1 : 0, len_offset, S(stream));
}

int ta100_decode_status(void* stream) { return decode_status(S(stream)); }

int ta100_peer_exchange_create(int world, long long slot_bytes, void** region, unsigned char* handle64) {
    return peer_exchange_create(world, slot_bytes, region, handle64);
}
int ta100_peer_exchange_open(const unsigned char* handle64, void** region) { return peer_exchange_open(handle64, region); }
int ta100_peer_exchange_close(void* region) { return peer_exchange_close(region); }
int ta100_peer_exchange_destroy(void* region) { return peer_exchange_destroy(region); }
int ta100_peer_all_gather(const void* src, void* out, long long bytes, long long slot_bytes, int world, int rank,
                          void* const* regions, void* stream) {
    return peer_all_gather_dispatch(src, out, bytes, slot_bytes, world, rank, regions, S(stream));
}
int ta100_peer_exchange_status(void* region, int world, long long slot_bytes, void* stream) {
    return peer_exchange_status(region, world, slot_bytes, S(stream));
}

int ta100_merge_partials(const void* part_o, const void* part_ml, void* out, int shards, long long shard_stride_o,
                         long long shard_stride_ml, long long flat_kv_heads, int splits, int group, int head_dim,
                         int is_mxfp4, int is_bf16, void* stream) {
    return merge_dispatch(part_o, part_ml, out, shards, shard_stride_o, shard_stride_ml, flat_kv_heads, splits, group,
                          head_dim, is_mxfp4, is_bf16, S(stream));
}

int ta100_reduce_partials(const void* part_o, const void* part_ml, void* out_o, void* out_ml, long long flat_kv_heads,
                          int splits, int group, int head_dim, void* stream) {
    return reduce_partials_dispatch(part_o, part_ml, out_o, out_ml, flat_kv_heads, splits, group, head_dim, S(stream));
}

size_t ta100_decode_static_scratch_bytes(void) { return decode_static_scratch_bytes(); }

int ta100_decode_attention_static(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width,
                                  const void* q4, const void* k4, const void* v4, const void* qs, const void* ks,
                                  const void* vs, const void* page_table, int max_pages, int pool_pages, void* out, int batch, int hkv,
                                  int group, int kv_len, int kv_cap, int head_dim, int is_mxfp4, int is_bf16, int splits,
                                  void* stream) {
    return decode_static_dispatch(q_hi, k_hi, v_hi, sel, width, q4, k4, v4, qs, ks, vs, page_table, max_pages, pool_pages, out, batch,
                                  hkv, group, kv_len, kv_cap, head_dim, is_mxfp4, is_bf16, splits, S(stream));
}

}  // extern "C"
