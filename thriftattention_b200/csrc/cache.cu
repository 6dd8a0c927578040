// Fused KV-cache append for generation.
//
// One launch per layer and step does what the reference cache does with several PyTorch slice
// copies and three extension calls (integrations/transformers_cache.py:87-123, 308-351):
//   * store the new 16-bit K and V rows at [start, start + count) of the capacity-strided cache,
//   * quantise the new K rows (plain row layout: codes [cap, D/2], scales [cap, D/G]),
//   * re-quantise every V group (G = 16 NVFP4 / 32 MXFP4 tokens, transposed layout
//     codes [D, cap/2], scales [D, cap/G]) that the new rows touch — tokens of such a group that
//     are not new are read back from the 16-bit cache,
//   * recompute mean / min / max of every statistics block that the new rows complete.
// The arithmetic of each piece is the one of the stand-alone quantise and block-statistics
// kernels, so a cache filled in any number of appends equals one filled in a single pass.
//
// Work is cut into independent CTA-sized items (K row bundles, 128-token V tiles, statistics
// blocks); an item reads new rows from the inputs and old rows from the cache, never a row that
// another item of the same launch writes, so no ordering between CTAs is needed.
//
// Two addressings of the cache tensors: capacity-strided slabs [heads, cap, ...], or pools of 64-token pages
// ([pool_pages, hkv, 64, ...]; V codes [pool_pages, hkv, D, 32]) behind a page table [batch, max_pages], the
// layout the decode kernel reads.  The statistics stay indexed by logical block in both.
#include "common.cuh"

namespace ta100 {

struct AppendParams {
    const uint16_t* k_new;
    const uint16_t* v_new;
    uint16_t* k_hi;
    uint16_t* v_hi;
    uint8_t* k_codes;
    uint8_t* k_scales;
    uint8_t* v_codes;
    uint8_t* v_scales;
    uint16_t* k_mean;
    uint16_t* k_min;
    uint16_t* k_max;
    int start, k_count, v_count, cap;
    const int32_t* start_dev;     // null, or the append position(s) in device memory: the kernel uses that + start
                                  // and the item counts below are upper bounds
    int start_per_seq;            // 0: start_dev[0] for every sequence; 1: start_dev[head / hkv]
    const int32_t* page_table;    // paged addressing: [batch, max_pages] -> physical page; nullptr = slabs
    int max_pages, pool_pages, hkv;
    int stat_blocks;              // statistics blocks per head in k_mean / k_min / k_max (their row stride)
    int k_keep, v_keep;           // with a null input: 1 = re-quantise the cached rows, 0 = store zero rows
    int n_k_items, n_v_items, n_s_items;
    int k_loop;                   // K row bundles per K item (more than one for bulk appends)
    int v_begin, v_end;           // group-aligned token range whose V groups are re-quantised
    int s_first, stat_block;
};

// Row of token `tok` of `head` in a [.., tokens, X]-shaped cache tensor (16-bit rows, K codes, K scales), in rows;
// -1 if the page table has no valid page there (the access is then skipped).
template <bool PAGED>
__device__ __forceinline__ long long cache_row(const AppendParams& p, long long head, int tok) {
    if constexpr (!PAGED) return head * p.cap + tok;
    const long long b = head / p.hkv, h = head - b * p.hkv;
    const int pg = tok >> 6;
    if (pg >= p.max_pages) return -1;
    const int page = p.page_table[b * p.max_pages + pg];
    if (page < 0 || page >= p.pool_pages) return -1;
    return (static_cast<long long>(page) * p.hkv + h) * 64 + (tok & 63);
}

// 16-byte chunk `cv` of token `tok`: from the new rows when the token is being appended, else from the cache.
template <int D, bool PAGED>
__device__ __forceinline__ uint4 row_chunk(const AppendParams& p, const uint16_t* __restrict__ fresh, const uint16_t* cache,
                                           int keep, int count, long long head, int tok, int cv, bool& is_new) {
    is_new = false;
    if (tok >= p.start && tok < p.start + count && !(fresh == nullptr && keep)) {
        is_new = true;
        if (fresh == nullptr) return make_uint4(0u, 0u, 0u, 0u);
        return __ldg(reinterpret_cast<const uint4*>(fresh + (head * count + (tok - p.start)) * D) + cv);
    }
    const long long row = cache_row<PAGED>(p, head, tok);
    if (row < 0) return make_uint4(0u, 0u, 0u, 0u);
    return *(reinterpret_cast<const uint4*>(cache + row * D) + cv);
}

template <int D, bool MX, bool BF16, bool PAGED>
__global__ void __launch_bounds__(128) cache_append_kernel(const AppendParams launch) {
    constexpr int G = MX ? 32 : 16;
    AppendParams p = launch;
    int n_v_real = p.n_v_items, n_s_real = p.n_s_items;
    if (launch.start_dev != nullptr) {
        // the position comes from device memory: the launch was cut for the worst case, the real ranges follow here
        const long long head0 = blockIdx.x / (launch.n_k_items + launch.n_v_items + launch.n_s_items);
        p.start = __ldg(launch.start_dev + (launch.start_per_seq ? head0 / launch.hkv : 0)) + launch.start;
        const int longest = p.k_count > p.v_count ? p.k_count : p.v_count;
        if (p.start < 0 || p.start > p.cap - longest) return;     // beyond the capacity: nothing is stored
        n_v_real = 0;
        n_s_real = 0;
        if (p.v_count > 0) {
            p.v_begin = p.start / G * G;
            p.v_end = cdiv(p.start + p.v_count, G) * G;
            n_v_real = cdiv(p.v_end, 128) - p.v_begin / 128;
        }
        if (p.k_count > 0 && (p.k_mean || p.k_min || p.k_max)) {
            p.s_first = p.start / p.stat_block;
            const int last = (p.start + p.k_count) / p.stat_block;
            n_s_real = last > p.s_first ? last - p.s_first : 0;
        }
    }
    constexpr int GPR = D / G;        // groups per row
    constexpr int ROWS = 128 / GPR;   // K rows per item
    constexpr int VEC = D / 8;        // 16-byte chunks per row
    constexpr int TILE_BYTES = 128 * (D + 8) * 2;
    __shared__ __align__(16) unsigned char smem[TILE_BYTES + D * 64 + D * 8];

    const int items = p.n_k_items + p.n_v_items + p.n_s_items;
    const long long head = blockIdx.x / items;
    int it = blockIdx.x % items;
    const int tid = threadIdx.x;

    if (it < p.n_k_items) {
        // ---------------------------------------------------------------- K rows: one thread per group
        const int c = tid % GPR;
        for (int b = 0; b < p.k_loop; ++b) {
            const int row = (it * p.k_loop + b) * ROWS + tid / GPR;
            if (row >= p.k_count) return;
            const int tok = p.start + row;
            uint32_t raw[G / 2];
            bool is_new = false;
            const long long krow = cache_row<PAGED>(p, head, tok);
            if (krow < 0) continue;
#pragma unroll
            for (int i = 0; i < G / 8; ++i) {
                const uint4 t = row_chunk<D, PAGED>(p, p.k_new, p.k_hi, p.k_keep, p.k_count, head, tok, c * (G / 8) + i, is_new);
                raw[4 * i + 0] = t.x; raw[4 * i + 1] = t.y; raw[4 * i + 2] = t.z; raw[4 * i + 3] = t.w;
                if (is_new) *(reinterpret_cast<uint4*>(p.k_hi + krow * D) + c * (G / 8) + i) = t;
            }
            uint32_t out[G / 8];
            uint8_t sb;
            quantise_group_regs<MX, BF16>(raw, out, sb);
            const long long gid = krow * GPR + c;
            if constexpr (MX) *reinterpret_cast<uint4*>(p.k_codes + gid * 16) = make_uint4(out[0], out[1], out[2], out[3]);
            else *reinterpret_cast<uint2*>(p.k_codes + gid * 8) = make_uint2(out[0], out[1]);
            p.k_scales[gid] = sb;
        }
        return;
    }
    it -= p.n_k_items;

    if (it < p.n_v_items) {
        if (it >= n_v_real) return;
        // ---------------------------------------------------------------- V: groups of one 128-token tile
        auto tile = reinterpret_cast<uint16_t(*)[D + 8]>(smem);
        auto out_codes = reinterpret_cast<uint8_t(*)[64]>(smem + TILE_BYTES);
        auto out_scales = reinterpret_cast<uint8_t(*)[8]>(smem + TILE_BYTES + D * 64);
        const int tok0 = (p.v_begin / 128 + it) * 128;
        const int lo = max(p.v_begin, tok0);
        const int hi = min(p.v_end, tok0 + 128);
        for (int i = tid; i < (hi - lo) * VEC; i += 128) {
            const int r = i / VEC, cv = i % VEC;
            const int tok = lo + r;
            bool is_new;
            const uint4 val = row_chunk<D, PAGED>(p, p.v_new, p.v_hi, p.v_keep, p.v_count, head, tok, cv, is_new);
            if (is_new) {
                const long long vrow = cache_row<PAGED>(p, head, tok);
                if (vrow >= 0) *(reinterpret_cast<uint4*>(p.v_hi + vrow * D) + cv) = val;
            }
            *reinterpret_cast<uint4*>(&tile[tok - tok0][cv * 8]) = val;
        }
        __syncthreads();
        const int g_first = (lo - tok0) / G;
        const int n_groups = (hi - lo) / G;
        for (int i = tid; i < D * n_groups; i += 128) {
            const int ch = i % D, grp = g_first + i / D;
            uint32_t raw[G / 2];
#pragma unroll
            for (int j = 0; j < G / 2; ++j) {
                const uint32_t a = tile[grp * G + 2 * j][ch];
                const uint32_t b = tile[grp * G + 2 * j + 1][ch];
                raw[j] = a | (b << 16);
            }
            uint32_t out[G / 8];
            uint8_t sb;
            quantise_group_regs<MX, BF16>(raw, out, sb);
#pragma unroll
            for (int w = 0; w < G / 8; ++w) *reinterpret_cast<uint32_t*>(&out_codes[ch][grp * (G / 2) + 4 * w]) = out[w];
            out_scales[ch][grp] = sb;
        }
        __syncthreads();
        // 8-byte pieces (16 tokens); consecutive threads write consecutive pieces of one channel row
        const int pc_first = (lo - tok0) / 16;
        const int n_pieces = (hi - lo) / 16;
        for (int i = tid; i < D * n_pieces; i += 128) {
            const int ch = i / n_pieces, pc = pc_first + i % n_pieces;
            long long dst;
            if constexpr (PAGED) {
                const long long row = cache_row<true>(p, head, tok0 + pc * 16);    // page row of the piece's first token
                if (row < 0) continue;
                dst = ((row >> 6) * D + ch) * 32 + (row & 63) / 2;                   // [page, h, D, 32]: (page * hkv + h) = row / 64
            } else {
                dst = (head * D + ch) * (p.cap / 2) + tok0 / 2 + pc * 8;
            }
            *reinterpret_cast<uint2*>(p.v_codes + dst) = *reinterpret_cast<const uint2*>(&out_codes[ch][pc * 8]);
        }
        for (int i = tid; i < D * n_groups; i += 128) {
            const int ch = i / n_groups, g = g_first + i % n_groups;
            long long dst;
            if constexpr (PAGED) {
                const long long row = cache_row<true>(p, head, tok0 + g * G);
                if (row < 0) continue;
                dst = ((row >> 6) * D + ch) * (64 / G) + (row & 63) / G;
            } else {
                dst = (head * D + ch) * (p.cap / G) + tok0 / G + g;
            }
            p.v_scales[dst] = out_scales[ch][g];
        }
        return;
    }
    it -= p.n_v_items;

    if (it < n_s_real) {
        // ---------------------------------------------------------------- statistics of one completed block
        // Same summation order as block_stats_kernel: eight row groups (row mod 8) accumulate in ascending
        // row order, the eight partial sums are added left to right, then divided by the block length.
        auto s_sum = reinterpret_cast<float(*)[D]>(smem);
        auto s_min = reinterpret_cast<float(*)[D]>(smem + 8 * D * 4);
        auto s_max = reinterpret_cast<float(*)[D]>(smem + 16 * D * 4);
        const int blk = p.s_first + it;
        if (tid < D) {
            const int cc = tid % VEC, rg = tid / VEC;
            float sum[8], lo[8], hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) { sum[i] = 0.0f; lo[i] = INFINITY; hi[i] = -INFINITY; }
            for (int r = rg; r < p.stat_block; r += 8) {
                bool is_new;
                const uint4 v = row_chunk<D, PAGED>(p, p.k_new, p.k_hi, p.k_keep, p.k_count, head, blk * p.stat_block + r, cc, is_new);
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const float a = In16<BF16>::to_f(static_cast<uint16_t>(w[i] & 0xFFFFu));
                    const float b = In16<BF16>::to_f(static_cast<uint16_t>(w[i] >> 16));
                    sum[2 * i] = __fadd_rn(sum[2 * i], a);
                    sum[2 * i + 1] = __fadd_rn(sum[2 * i + 1], b);
                    lo[2 * i] = fminf(lo[2 * i], a); lo[2 * i + 1] = fminf(lo[2 * i + 1], b);
                    hi[2 * i] = fmaxf(hi[2 * i], a); hi[2 * i + 1] = fmaxf(hi[2 * i + 1], b);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s_sum[rg][cc * 8 + i] = sum[i];
                s_min[rg][cc * 8 + i] = lo[i];
                s_max[rg][cc * 8 + i] = hi[i];
            }
        }
        __syncthreads();
        if (tid < D) {
            float total = s_sum[0][tid], l = s_min[0][tid], h = s_max[0][tid];
#pragma unroll
            for (int g = 1; g < 8; ++g) {
                total = __fadd_rn(total, s_sum[g][tid]);
                l = fminf(l, s_min[g][tid]);
                h = fmaxf(h, s_max[g][tid]);
            }
            const long long o = (head * p.stat_blocks + blk) * D + tid;
            if (p.k_mean) p.k_mean[o] = In16<BF16>::from_f(__fdiv_rn(total, static_cast<float>(p.stat_block)));
            if (p.k_min) p.k_min[o] = In16<BF16>::from_f(l);
            if (p.k_max) p.k_max[o] = In16<BF16>::from_f(h);
        }
    }
}

// Contiguous slabs: page_table = nullptr (max_pages, pool_pages, hkv, stat_blocks ignored; the statistics have
// capacity / stat_block blocks per head).  Paged pools: capacity = max_pages * 64 is the logical bound.
int cache_append_dispatch(const void* k_new, const void* v_new, void* k_hi, void* v_hi, void* k_codes, void* k_scales,
                          void* v_codes_t, void* v_scales_t, void* k_mean, void* k_min, void* k_max, long long heads,
                          int start, int k_count, int v_count, int capacity, int head_dim, int stat_block, int is_mx,
                          int is_bf16, int flags, const void* page_table, int max_pages, int pool_pages, int hkv,
                          int stat_blocks, const void* start_dev, int start_per_seq, cudaStream_t stream) {
    if (head_dim != 64 && head_dim != 128) return TA100_ERR_UNSUPPORTED;
    if (page_table) {
        if (max_pages <= 0 || pool_pages <= 0 || hkv <= 0 || heads % hkv != 0 || stat_blocks <= 0) return TA100_ERR_SHAPE;
        if (max_pages > 0x7FFFFFFF / 64) return TA100_ERR_LIMIT;
        capacity = max_pages * 64;
        if (capacity % 128 != 0) capacity += 64;     // only bounds the logical token range below
    }
    if (heads < 0 || start < 0 || k_count < 0 || v_count < 0 || capacity <= 0 || capacity % 128 != 0)
        return TA100_ERR_SHAPE;
    if (stat_block != 64 && stat_block != 128) return TA100_ERR_SHAPE;
    if (!start_dev && static_cast<long long>(start) + (k_count > v_count ? k_count : v_count) > capacity) return TA100_ERR_SHAPE;
    if (k_count > 0 && (!k_hi || !k_codes || !k_scales)) return TA100_ERR_NULL;
    if (v_count > 0 && (!v_hi || !v_codes_t || !v_scales_t)) return TA100_ERR_NULL;
    const uintptr_t all = reinterpret_cast<uintptr_t>(k_new) | reinterpret_cast<uintptr_t>(v_new) |
                          reinterpret_cast<uintptr_t>(k_hi) | reinterpret_cast<uintptr_t>(v_hi) |
                          reinterpret_cast<uintptr_t>(k_codes) | reinterpret_cast<uintptr_t>(v_codes_t);
    if (all & 15) return TA100_ERR_ALIGN;
    if (heads == 0 || (k_count == 0 && v_count == 0)) return TA100_OK;

    const int G = is_mx ? 32 : 16;
    AppendParams p{};
    p.k_new = static_cast<const uint16_t*>(k_new);
    p.v_new = static_cast<const uint16_t*>(v_new);
    p.k_hi = static_cast<uint16_t*>(k_hi);
    p.v_hi = static_cast<uint16_t*>(v_hi);
    p.k_codes = static_cast<uint8_t*>(k_codes);
    p.k_scales = static_cast<uint8_t*>(k_scales);
    p.v_codes = static_cast<uint8_t*>(v_codes_t);
    p.v_scales = static_cast<uint8_t*>(v_scales_t);
    p.k_mean = static_cast<uint16_t*>(k_mean);
    p.k_min = static_cast<uint16_t*>(k_min);
    p.k_max = static_cast<uint16_t*>(k_max);
    p.start = start; p.k_count = k_count; p.v_count = v_count; p.cap = capacity;
    p.start_dev = static_cast<const int32_t*>(start_dev);
    p.start_per_seq = (start_dev && start_per_seq) ? 1 : 0;
    if (p.start_per_seq && (hkv <= 0 || heads % hkv != 0)) return TA100_ERR_SHAPE;
    p.page_table = static_cast<const int32_t*>(page_table);
    p.max_pages = max_pages; p.pool_pages = pool_pages; p.hkv = hkv;
    p.stat_blocks = page_table ? stat_blocks : capacity / stat_block;
    p.k_keep = (flags & 1) ? 1 : 0;
    p.v_keep = (flags & 2) ? 1 : 0;
    p.stat_block = stat_block;
    const int rows_per_item = 128 / (head_dim / G);
    p.k_loop = k_count >= 2048 ? 8 : 1;
    p.n_k_items = cdiv(k_count, rows_per_item * p.k_loop);
    if (start_dev) {
        // wherever the range starts: its V groups reach at most G - 1 tokens beyond either end, and it completes at
        // most one statistics block more than it has whole blocks
        if (v_count > 0) p.n_v_items = (v_count + 2 * (G - 1) - 1) / 128 + 2;
        if (k_count > 0 && (k_mean || k_min || k_max)) p.n_s_items = k_count / stat_block + 1;
    } else {
        if (v_count > 0) {
            p.v_begin = start / G * G;
            p.v_end = cdiv(start + v_count, G) * G;
            p.n_v_items = cdiv(p.v_end, 128) - p.v_begin / 128;
        }
        if (k_count > 0 && (k_mean || k_min || k_max)) {
            p.s_first = start / stat_block;
            const int last = (start + k_count) / stat_block;
            p.n_s_items = last > p.s_first ? last - p.s_first : 0;
        }
    }
    const long long grid = heads * (p.n_k_items + p.n_v_items + p.n_s_items);
    if (grid > 0x7FFFFFFFLL) return TA100_ERR_LIMIT;
#define TA100_APPEND(DD, MXX, BFF)                                                                              \
    do {                                                                                                        \
        if (page_table) cache_append_kernel<DD, MXX, BFF, true><<<static_cast<unsigned>(grid), 128, 0, stream>>>(p);  \
        else cache_append_kernel<DD, MXX, BFF, false><<<static_cast<unsigned>(grid), 128, 0, stream>>>(p);       \
    } while (0)
    if (head_dim == 128) {
        if (is_mx) { if (is_bf16) TA100_APPEND(128, true, true); else TA100_APPEND(128, true, false); }
        else { if (is_bf16) TA100_APPEND(128, false, true); else TA100_APPEND(128, false, false); }
    } else {
        if (is_mx) { if (is_bf16) TA100_APPEND(64, true, true); else TA100_APPEND(64, true, false); }
        else { if (is_bf16) TA100_APPEND(64, false, true); else TA100_APPEND(64, false, false); }
    }
#undef TA100_APPEND
    return static_cast<int>(cudaGetLastError());
}

namespace {
__global__ void advance_length_kernel(int32_t* len, int n, int count, int limit) {
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        const long long v = static_cast<long long>(len[i]) + count;
        len[i] = static_cast<int32_t>(v > limit ? limit : (v < 0 ? 0 : v));
    }
}
}  // namespace

// len_dev[i] = min(len_dev[i] + count, limit) for the n lengths: the end of a generation step whose kernels read the
// length on the GPU.
int advance_length_dispatch(void* len_dev, int n, int count, int limit, cudaStream_t stream) {
    if (!len_dev) return TA100_ERR_NULL;
    if (limit < 0 || n < 1) return TA100_ERR_SHAPE;
    advance_length_kernel<<<1, 128, 0, stream>>>(static_cast<int32_t*>(len_dev), n, count, limit);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace ta100
