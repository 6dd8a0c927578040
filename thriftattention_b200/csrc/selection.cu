// Block selection: per-block statistics (mean / min / max), block-mean and
// Quest scoring with an exact warp top-k, decode variants with group-max
// scores, closed-form local windows and the index-list -> bitset packer.
//
// Score arithmetic is fixed so that results are reproducible bit for bit:
// lane l of a warp accumulates channels l, l+32, ... with fused multiply-adds,
// then the 32 partial sums are combined by an xor butterfly (deltas 16..1).
// Top-k is k rounds of arg-max with knock-out; ties go to the candidate whose
// index modulo 32 has the smallest 5-bit bit-reversal, then to the smaller index.
#include <cfloat>

#include "common.cuh"

namespace ta100 {

// ---------------------------------------------------------------------------
// Block statistics
// ---------------------------------------------------------------------------
// x [heads, seq, D] -> mean/min/max [heads, seq/block, D] (any may be null).
// Eight row groups accumulate rows r = g (mod 8) in ascending order in fp32; the
// eight partial sums are then added left to right and divided by `block`.
template <int D, bool BF16>
__global__ void __launch_bounds__(D) block_stats_kernel(const uint16_t* __restrict__ x, uint16_t* __restrict__ mean,
                                                        uint16_t* __restrict__ mn, uint16_t* __restrict__ mx,
                                                        long long n_blocks, int block) {
    constexpr int CHUNKS = D / 8;  // 16-byte chunks per row
    __shared__ float s_sum[8][D];
    __shared__ float s_min[8][D];
    __shared__ float s_max[8][D];
    const int cc = threadIdx.x % CHUNKS;
    const int rg = threadIdx.x / CHUNKS;  // 0..7
    for (long long blk = blockIdx.x; blk < n_blocks; blk += gridDim.x) {
        float sum[8], lo[8], hi[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) { sum[i] = 0.0f; lo[i] = INFINITY; hi[i] = -INFINITY; }
        const uint16_t* base = x + blk * block * D;
#pragma unroll 4
        for (int r = rg; r < block; r += 8) {
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(base + static_cast<long long>(r) * D) + cc);
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
        __syncthreads();
        {
            const int c = threadIdx.x;  // one channel per thread
            float total = s_sum[0][c], l = s_min[0][c], h = s_max[0][c];
#pragma unroll
            for (int g = 1; g < 8; ++g) {
                total = __fadd_rn(total, s_sum[g][c]);
                l = fminf(l, s_min[g][c]);
                h = fmaxf(h, s_max[g][c]);
            }
            const long long o = blk * D + c;
            if (mean) mean[o] = In16<BF16>::from_f(__fdiv_rn(total, static_cast<float>(block)));
            if (mn) mn[o] = In16<BF16>::from_f(l);
            if (mx) mx[o] = In16<BF16>::from_f(h);
        }
        __syncthreads();
    }
}

int block_stats_dispatch(const void* x, void* mean, void* mn, void* mx, long long heads, int seq, int d, int block,
                         int is_bf16, cudaStream_t stream) {
    if (!x) return TA100_ERR_NULL;
    if (d != 64 && d != 128) return TA100_ERR_UNSUPPORTED;
    if (block <= 0 || seq % block != 0) return TA100_ERR_SHAPE;
    const long long n_blocks = heads * (seq / block);
    if (n_blocks == 0) return TA100_OK;
    const int grid = static_cast<int>(n_blocks < NUM_SMS_HINT * 16LL ? n_blocks : NUM_SMS_HINT * 16LL);
    auto X = static_cast<const uint16_t*>(x);
    auto A = static_cast<uint16_t*>(mean);
    auto B = static_cast<uint16_t*>(mn);
    auto C = static_cast<uint16_t*>(mx);
    if (d == 128) {
        if (is_bf16) block_stats_kernel<128, true><<<grid, 128, 0, stream>>>(X, A, B, C, n_blocks, block);
        else block_stats_kernel<128, false><<<grid, 128, 0, stream>>>(X, A, B, C, n_blocks, block);
    } else {
        if (is_bf16) block_stats_kernel<64, true><<<grid, 64, 0, stream>>>(X, A, B, C, n_blocks, block);
        else block_stats_kernel<64, false><<<grid, 64, 0, stream>>>(X, A, B, C, n_blocks, block);
    }
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Scoring and top-k
// ---------------------------------------------------------------------------
template <int D, bool BF16, bool QUEST>
__device__ __forceinline__ float warp_score(const float (&q)[D / 32], const uint16_t* __restrict__ ka,
                                            const uint16_t* __restrict__ kb, int lane) {
    float dot = 0.0f;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
        const int e = lane + 32 * i;
        float k;
        if constexpr (QUEST) k = q[i] >= 0.0f ? In16<BF16>::to_f(kb[e]) : In16<BF16>::to_f(ka[e]);
        else k = In16<BF16>::to_f(ka[e]);
        dot = __fmaf_rn(q[i], k, dot);
    }
#pragma unroll
    for (int delta = 16; delta >= 1; delta >>= 1) dot = __fadd_rn(dot, __shfl_xor_sync(0xFFFFFFFFu, dot, delta));
    return dot;
}

// k rounds of arg-max over `scores[0..n)` (shared memory, one warp).
template <int ITEMS>
__device__ __forceinline__ void warp_topk_rounds(const float* scores, int n, int k, bool pad, int32_t* out, int lane) {
    float val[ITEMS];
#pragma unroll
    for (int i = 0; i < ITEMS; ++i) {
        const int idx = i * 32 + lane;
        val[i] = idx < n ? scores[idx] : -FLT_MAX;
    }
    for (int r = 0; r < k; ++r) {
        float best = val[0];
        int best_idx = lane;
#pragma unroll
        for (int i = 1; i < ITEMS; ++i)
            if (val[i] > best) { best = val[i]; best_idx = i * 32 + lane; }
#pragma unroll
        for (int delta = 16; delta >= 1; delta >>= 1) {
            const float ob = __shfl_xor_sync(0xFFFFFFFFu, best, delta);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, best_idx, delta);
            if (ob > best) { best = ob; best_idx = oi; }
        }
        best = __shfl_sync(0xFFFFFFFFu, best, 0);
        best_idx = __shfl_sync(0xFFFFFFFFu, best_idx, 0);
        const bool found = best > -FLT_MAX * 0.5f;
        if (lane == 0) out[r] = (found || !pad) ? best_idx : -1;
        if (found || !pad) {
#pragma unroll
            for (int i = 0; i < ITEMS; ++i)
                if (i * 32 + lane == best_idx) val[i] = -FLT_MAX;
        }
    }
}

// Sort key: high word orders scores descending (-0 counts as +0), low word is the tie-break rank.
__device__ __forceinline__ unsigned long long seld_key(float score, int page) {
    if (score == 0.0f) score = 0.0f;
    const uint32_t u = __float_as_uint(score);
    const uint32_t asc = (u >> 31) ? ~u : (u | 0x80000000u);
    const uint32_t tie = (__brev(static_cast<uint32_t>(page) & 31u) >> 27 << 16) | (static_cast<uint32_t>(page) >> 5);
    return (static_cast<unsigned long long>(~asc) << 32) | tie;
}
__device__ __forceinline__ float seld_key_score(unsigned long long key) {
    const uint32_t asc = ~static_cast<uint32_t>(key >> 32);
    return __uint_as_float((asc >> 31) ? (asc ^ 0x80000000u) : ~asc);
}
__device__ __forceinline__ int seld_key_page(unsigned long long key) {
    const uint32_t tie = static_cast<uint32_t>(key);
    return static_cast<int>((__brev(tie >> 16) >> 27) | ((tie & 0xFFFFu) << 5));
}

// The same k picks as warp_topk_rounds(pad = true) without k serial rounds (one warp, scores in shared memory):
// a four-digit radix selection finds the k-th largest score, the entries at or above it are gathered (at most
// SELP_CAND of them) and ranked by counting smaller 64-bit keys (descending score, then the arg-max rounds'
// tie-break: smallest 5-bit bit-reversal of idx mod 32, then smallest idx div 32).  Returns false without
// writing anything when more than SELP_CAND entries tie into the candidate set; the caller then runs the rounds.
// hist: 256 ints (reused for the candidate indices), keys: SELP_CAND 64-bit words, both private to the warp.
constexpr int SELP_CAND = 256;
__device__ __forceinline__ bool warp_topk_select(const float* scores, int n, int k, int32_t* out, int lane, int* hist,
                                                 unsigned long long* keys) {
    if (k <= 0) return true;
    auto image = [&](int i) -> uint32_t {       // ascending 32-bit image of the score
        float v = scores[i];
        if (v == 0.0f) v = 0.0f;
        const uint32_t u = __float_as_uint(v);
        return (u >> 31) ? ~u : (u | 0x80000000u);
    };
    uint32_t prefix = 0u;
    if (n > k) {
        int remaining = k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            for (int j = lane; j < 256; j += 32) hist[j] = 0;
            __syncwarp();
            for (int i = lane; i < n; i += 32) {
                const uint32_t key = image(i);
                if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1);
            }
            __syncwarp();
            int cnt[8], mine = 0;            // lane l owns digits 8l .. 8l+7; suffix sums over the lanes
#pragma unroll
            for (int j = 0; j < 8; ++j) { cnt[j] = hist[lane * 8 + j]; mine += cnt[j]; }
            int incl = mine;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                const int v = __shfl_down_sync(0xFFFFFFFFu, incl, d);
                if (lane + d < 32) incl += v;
            }
            const int excl = incl - mine;
            const bool owner = excl < remaining && remaining <= incl;
            int digit = 0, rest = 0;
            if (owner) {
                int seen = excl;
#pragma unroll
                for (int j = 7; j >= 0; --j) {
                    if (seen < remaining && remaining <= seen + cnt[j]) { digit = lane * 8 + j; rest = remaining - seen; break; }
                    seen += cnt[j];
                }
            }
            const int src = __ffs(__ballot_sync(0xFFFFFFFFu, owner)) - 1;
            digit = __shfl_sync(0xFFFFFFFFu, digit, src);
            remaining = __shfl_sync(0xFFFFFFFFu, rest, src);
            prefix |= static_cast<uint32_t>(digit) << shift;
            __syncwarp();
        }
    }
    // gather the entries at or above the threshold (all of them when n <= k)
    int* cand = hist;
    const uint32_t lt = (1u << lane) - 1u;
    int n_c = 0;
    for (int base = 0; base < n; base += 32) {
        const int i = base + lane;
        const bool take = i < n && image(i) >= prefix;
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, take);
        const int pos = n_c + __popc(m & lt);
        if (take && pos < SELP_CAND) cand[pos] = i;
        n_c += __popc(m);
    }
    if (n_c > SELP_CAND) return false;
    __syncwarp();
    for (int c = lane; c < n_c; c += 32) keys[c] = seld_key(scores[cand[c]], cand[c]);
    __syncwarp();
    for (int c = lane; c < n_c; c += 32) {
        const unsigned long long mine = keys[c];
        int rank = 0;
        for (int j = 0; j < n_c; ++j) rank += keys[j] < mine ? 1 : 0;
        if (rank < k) out[rank] = seld_key_score(mine) > -FLT_MAX * 0.5f ? seld_key_page(mine) : -1;
    }
    for (int r = n_c + lane; r < k; r += 32) out[r] = -1;
    return true;
}

__device__ __forceinline__ void topk_dispatch(const float* scores, int n, int k, bool pad, int32_t* out, int lane) {
    if (n <= 128) warp_topk_rounds<4>(scores, n, k, pad, out, lane);
    else if (n <= 512) warp_topk_rounds<16>(scores, n, k, pad, out, lane);
    else if (n <= 1024) warp_topk_rounds<32>(scores, n, k, pad, out, lane);
    else warp_topk_rounds<64>(scores, n, k, pad, out, lane);
}

// Prefill: one warp per (q head, q block); a CTA of 8 warps covers 8 consecutive
// q blocks of one head and shares the K statistics through shared memory.
// q_mean [heads, nq, D]; ka/kb [kv_heads, nk, D] (not expanded per q head).
// out [heads, nq, sink + local + k]: forced sink ids, forced local ids, then the
// top-k by rank, -1 padded.
constexpr int SEL_WARPS = 8;
constexpr int SEL_KTILE = 32;

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
                 "l"(src)
                 : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }


template <int D>
struct SelpSmem {
    static constexpr int ROW = D * 2 + 16;                    // padded statistics row: 16-byte reads by 32 lanes do not collide
    static constexpr int TILE = SEL_KTILE * ROW;
    static constexpr int QF = SEL_WARPS * D * 4;              // q rows as fp32
    static constexpr int QM = SEL_WARPS * (D / 2) * 4;        // Quest masks, one 16-bit mask per channel
    static constexpr int TOPK = SEL_WARPS * (256 * 4 + SELP_CAND * 8);   // per warp: histogram / candidates, keys
    static int total(int nk_pad) { return SEL_WARPS * nk_pad * 4 + 4 * TILE + QF + QM + TOPK; }   // two stages of [A | B]
};

// packed fp32x2 arithmetic (two partial sums per instruction) and 16-bit pair -> fp32 pair
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    unsigned long long ra, rb, rc, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rc) : "f"(c.x), "f"(c.y));
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(rd) : "l"(ra), "l"(rb), "l"(rc));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    unsigned long long ra, rb, rd;
    asm("mov.b64 %0, {%1, %2};" : "=l"(ra) : "f"(a.x), "f"(a.y));
    asm("mov.b64 %0, {%1, %2};" : "=l"(rb) : "f"(b.x), "f"(b.y));
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(rd) : "l"(ra), "l"(rb));
    float2 d;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(d.x), "=f"(d.y) : "l"(rd));
    return d;
}

template <bool BF16>
__device__ __forceinline__ float2 word_to_float2(uint32_t w) {
    if constexpr (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    else return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// Score of one (q row, key block) pair computed by ONE thread with the arithmetic of warp_score: 32 partial sums
// (channel c goes to partial c mod 32, fused multiply-adds in ascending channel order), then the xor-butterfly
// pairing 16, 8, 4, 2, 1 as plain additions — fp32 addition commutes, so the value is the warp's bit for bit.
template <int D, bool BF16, bool QUEST>
__device__ __forceinline__ float thread_score(const float4* __restrict__ qrow, const uint4* __restrict__ mrow,
                                              const uint4* __restrict__ ra, const uint4* __restrict__ rb) {
    float2 acc[16];
#pragma unroll
    for (int w = 0; w < 16; ++w) acc[w] = make_float2(0.0f, 0.0f);
#pragma unroll 1
    for (int i = 0; i < D / 32; ++i) {
#pragma unroll
        for (int v = 0; v < 4; ++v) {          // 8 channels per 16-byte chunk
            const uint4 a = ra[i * 4 + v];
            uint32_t kw[4] = {a.x, a.y, a.z, a.w};
            if constexpr (QUEST) {
                const uint4 b = rb[i * 4 + v];
                const uint4 m = mrow[i * 4 + v];
                kw[0] = (b.x & m.x) | (a.x & ~m.x);
                kw[1] = (b.y & m.y) | (a.y & ~m.y);
                kw[2] = (b.z & m.z) | (a.z & ~m.z);
                kw[3] = (b.w & m.w) | (a.w & ~m.w);
            }
            const float4 q0 = qrow[i * 8 + v * 2], q1 = qrow[i * 8 + v * 2 + 1];
            acc[v * 4 + 0] = fma2(make_float2(q0.x, q0.y), word_to_float2<BF16>(kw[0]), acc[v * 4 + 0]);
            acc[v * 4 + 1] = fma2(make_float2(q0.z, q0.w), word_to_float2<BF16>(kw[1]), acc[v * 4 + 1]);
            acc[v * 4 + 2] = fma2(make_float2(q1.x, q1.y), word_to_float2<BF16>(kw[2]), acc[v * 4 + 2]);
            acc[v * 4 + 3] = fma2(make_float2(q1.z, q1.w), word_to_float2<BF16>(kw[3]), acc[v * 4 + 3]);
        }
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) acc[w] = add2(acc[w], acc[w + 8]);
#pragma unroll
    for (int w = 0; w < 4; ++w) acc[w] = add2(acc[w], acc[w + 4]);
    acc[0] = add2(acc[0], acc[2]);
    acc[1] = add2(acc[1], acc[3]);
    acc[0] = add2(acc[0], acc[1]);
    return __fadd_rn(acc[0].x, acc[0].y);
}

template <int D, bool BF16, bool QUEST>
__global__ void __launch_bounds__(SEL_WARPS * 32) select_prefill_kernel(
    const uint16_t* __restrict__ q_mean, const uint16_t* __restrict__ ka, const uint16_t* __restrict__ kb,
    int32_t* __restrict__ out, int heads, int group, int nq, int nk, int k, int causal, int sink, int local) {
    using L = SelpSmem<D>;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    float* scores = reinterpret_cast<float*>(smem_raw);                              // [SEL_WARPS][nk_pad]
    const int nk_pad = (nk + 31) & ~31;
    uint8_t* s_tiles = smem_raw + SEL_WARPS * nk_pad * 4;                             // [2 stages][A | B][SEL_KTILE] padded rows
    float* qf = reinterpret_cast<float*>(s_tiles + 4 * L::TILE);                      // [SEL_WARPS][D]
    uint32_t* qm = reinterpret_cast<uint32_t*>(reinterpret_cast<uint8_t*>(qf) + L::QF);   // [SEL_WARPS][D/2]
    unsigned long long* tk_keys = reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(qm) + L::QM) +
                                  (threadIdx.x / 32) * SELP_CAND;
    int* tk_hist = reinterpret_cast<int*>(reinterpret_cast<uint8_t*>(qm) + L::QM + SEL_WARPS * SELP_CAND * 8) +
                   (threadIdx.x / 32) * 256;
    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    const int q_tiles = cdiv(nq, SEL_WARPS);
    const int width = sink + local + k;

    for (int work = blockIdx.x; work < heads * q_tiles; work += gridDim.x) {
        const int h = work / q_tiles;
        const int qb = (work - h * q_tiles) * SEL_WARPS + warp;
        const int kvh = h / group;
        const bool active = qb < nq;
        // this warp's q row as fp32, and for Quest an all-ones 16-bit mask per channel where q >= 0
        if (active) {
            for (int c = lane; c < D; c += 32)
                qf[warp * D + c] = In16<BF16>::to_f(q_mean[(static_cast<long long>(h) * nq + qb) * D + c]);
            __syncwarp();
            if constexpr (QUEST)
                for (int w = lane; w < D / 2; w += 32)
                    qm[warp * (D / 2) + w] = (qf[warp * D + 2 * w] >= 0.0f ? 0xFFFFu : 0u) |
                                             (qf[warp * D + 2 * w + 1] >= 0.0f ? 0xFFFF0000u : 0u);
            __syncwarp();
        }
        const int qb_hi = min((work - h * q_tiles) * SEL_WARPS + SEL_WARPS - 1, nq - 1);
        const int nk_need = causal ? min(nk, qb_hi + 1) : nk;
        const int nvalid = active ? (causal ? min(qb + 1, nk) : nk) : 0;
        const int n_sink = min(sink, nvalid);
        const int local_lo = max(nvalid - local, n_sink);
        float* my = scores + warp * nk_pad;
        const float4* qrow = reinterpret_cast<const float4*>(qf + warp * D);
        const uint4* mrow = reinterpret_cast<const uint4*>(qm + warp * (D / 2));
        // The statistics of 32 key blocks at a time stream through two shared-memory stages: tile t + 1 is on its way
        // (cp.async) while the warps score tile t.
        const int n_tiles = cdiv(nk_need, SEL_KTILE);
        auto issue = [&](int t) {
            const int b0 = t * SEL_KTILE;
            const int nb = min(SEL_KTILE, nk_need - b0);
            uint8_t* sa = s_tiles + (t & 1) * 2 * L::TILE;
            for (int i = threadIdx.x; i < nb * (D / 8); i += blockDim.x) {
                const int r = i / (D / 8), c = i - r * (D / 8);
                const long long g = (static_cast<long long>(kvh) * nk + b0 + r) * D + c * 8;
                cp_async16(sa + r * L::ROW + c * 16, ka + g);
                if constexpr (QUEST) cp_async16(sa + L::TILE + r * L::ROW + c * 16, kb + g);
            }
            cp_async_commit();
        };
        __syncthreads();                 // the previous item's readers are done with both stages
        if (n_tiles > 0) issue(0);
        for (int t = 0; t < n_tiles; ++t) {
            if (t + 1 < n_tiles) { issue(t + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncthreads();
            const int b0 = t * SEL_KTILE;
            const int nb = min(SEL_KTILE, nk_need - b0);
            const uint8_t* sa = s_tiles + (t & 1) * 2 * L::TILE;
            // one key block per lane
            const int b = b0 + lane;
            if (lane < nb && b < nvalid) {
                const float s = thread_score<D, BF16, QUEST>(qrow, mrow, reinterpret_cast<const uint4*>(sa + lane * L::ROW),
                                                             reinterpret_cast<const uint4*>(sa + L::TILE + lane * L::ROW));
                my[b] = (b < n_sink || b >= local_lo) ? -FLT_MAX : s;
            }
            __syncthreads();             // before this stage is refilled (tile t + 2)
        }
        __syncwarp();
        if (active) {
            int32_t* row = out + (static_cast<long long>(h) * nq + qb) * width;
            const int forced = n_sink + (nvalid - local_lo);
            for (int i = lane; i < forced; i += 32) row[i] = i < n_sink ? i : local_lo + (i - n_sink);
            if (!warp_topk_select(my, nvalid, k, row + forced, lane, tk_hist, tk_keys))
                topk_dispatch(my, nvalid, k, true, row + forced, lane);
            for (int i = forced + k + lane; i < width; i += 32) row[i] = -1;
        }
        __syncthreads();
    }
}

// Decode: one CTA (256 threads) per flat KV head.
//  1. scoring — 64-page tiles of the statistics stream through shared memory (cp.async, two stages);
//     four threads share a page and split the query group between them.  Each thread reproduces the
//     warp arithmetic above on its own: 32 partial sums (channel c goes to partial c mod 32, fused
//     multiply-adds in ascending channel order), then the xor-butterfly pairing 16, 8, 4, 2, 1 as plain
//     additions — fp32 addition commutes, so the value equals the warp's bit for bit.  Packed f32x2
//     instructions carry two partials each.
//  2. top-k — every page becomes a 64-bit key (descending score, then the tie-break rank of its index)
//     and the keys are sorted with a bitonic network in shared memory; the first k keys are the k
//     arg-max rounds' picks in the same order.
// q [flat, group, D]; ka/kb [flat, cap_blocks, D]; out [flat, sink + local + k].
constexpr int SELD_THREADS = 256;
constexpr int SELD_TILE = 64;       // pages per tile
constexpr int SELD_MAX_GROUP = 16;

constexpr int SELD_CAND_CAP = 512;   // exact re-scoring handles at most this many candidates

template <int D>
struct SeldSmem {
    static constexpr int ROW = D * 2 + 16;                       // padded statistics row (bytes)
    static constexpr int TILE_BYTES = SELD_TILE * ROW;
    static constexpr int QROW = D + 4;                            // floats per query row
    static constexpr int MROW = D / 2 + 4;                        // mask words per query row
    static constexpr int KEYS = 0;                                // 2048 x 8 B
    static constexpr int APPROX = KEYS + 2048 * 8;                // 2048 approximate scores
    static constexpr int CAND = APPROX + 2048 * 4;                // candidate page ids
    static constexpr int MISC = CAND + SELD_CAND_CAP * 4;         // counters
    static constexpr int QF = MISC + 64;
    static constexpr int QM = QF + SELD_MAX_GROUP * QROW * 4;
    static constexpr int TILES = QM + SELD_MAX_GROUP * MROW * 4;  // [2 stages][A | B]
    static constexpr int total(bool quest) { return TILES + 2 * (quest ? 2 : 1) * TILE_BYTES; }
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_row))));
}
template <bool BF16>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF16)
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    else
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Decode selection.  The exact score (see above) costs ~400 instructions per (page, head), far more than the
// 512 bytes of statistics it reads are worth, so the kernel ranks in two passes whenever it pays off:
//   pass 1  approximate scores of ALL pages with mma.sync (q split into its non-negative and negative parts,
//           so the Quest bound is a plain GEMM against [max | min]); every approximate score is within
//           delta = 2^-13 * max_g |q_g|_1 * max|statistics| of the exact one.  The products of two 16-bit
//           values are exact in fp32; what differs is the summation: the exact score rounds to nearest at
//           each of its <= 9 additions per value (<= 9 * 2^-24 relative to sum |q k|), the tensor core adds
//           up to 17 addends per MMA over 16 chained MMAs and its accumulation mode is not documented - a
//           truncating adder that aligns to the largest addend loses at most 2^-23 * sum |q k| per addend,
//           i.e. 16 * 17 * 2^-23 < 2^-14.9.  2^-13 covers both with a factor of three to spare;
//   pass 2  exact scores only for the pages that can still reach the top k: those whose approximate score
//           plus delta is at least the k-th largest (approximate score minus delta).
// Pages left out are provably below the exact k-th score, so the result is the one of scoring everything
// exactly.  With more than SELD_CAND_CAP candidates, few pages or a large query group, every page is scored
// exactly in one pass.
template <int D, bool BF16, bool QUEST>
__global__ void __launch_bounds__(SELD_THREADS, 2) select_decode_kernel(const uint16_t* __restrict__ q,
                                                                        const uint16_t* __restrict__ ka,
                                                                        const uint16_t* __restrict__ kb,
                                                                        int32_t* __restrict__ out,
                                                                        float* __restrict__ out_scores, int group,
                                                                        int nk_arg, int cap_blocks, int k_arg, int sink_arg,
                                                                        int local_arg, int out_stride, const DynLength dyn) {
    using L = SeldSmem<D>;
    // block counts: launch parameters, or derived from the sequence length in device memory
    int nk = nk_arg, k = k_arg, sink = sink_arg, local = local_arg;
    if (dyn.len != nullptr) {
        const int seq = dyn.hkv_per_seq > 0 ? static_cast<int>(blockIdx.x) / dyn.hkv_per_seq : 0;
        dyn_select_counts(dyn, max(0, __ldg(dyn.len + seq) + dyn.offset), min(cap_blocks, 2048), nk, k, sink, local);
        k = min(k, max(0, out_stride - sink - local));   // the host sizes the rows for the longest sequence
    }
    constexpr int VEC = D / 8;            // 16-byte chunks per statistics row
    constexpr int NARR = QUEST ? 2 : 1;
    extern __shared__ __align__(16) uint8_t smem_raw[];
    unsigned long long* keys = reinterpret_cast<unsigned long long*>(smem_raw + L::KEYS);
    float* approx = reinterpret_cast<float*>(smem_raw + L::APPROX);
    int* cand = reinterpret_cast<int*>(smem_raw + L::CAND);
    int* misc = reinterpret_cast<int*>(smem_raw + L::MISC);   // [0] candidates, [1] max |statistic| bits, [2] max |q|_1 bits
    float* qf = reinterpret_cast<float*>(smem_raw + L::QF);
    uint32_t* qm = reinterpret_cast<uint32_t*>(smem_raw + L::QM);
    uint8_t* tiles = smem_raw + L::TILES;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x;
    const int n_sink = min(sink, nk);
    const int local_lo = max(nk - local, n_sink);
    const int width = sink + local + k;
    const int forced = n_sink + (nk - local_lo);
    const bool two_pass = group <= 8 && nk >= 256 && k > 0 && k + forced < nk;

    // query group: fp32 values and, for Quest, one 16-bit mask per channel (all ones where q >= 0)
    for (int i = tid; i < group * D; i += SELD_THREADS) {
        const int g = i / D, c = i - g * D;
        qf[g * L::QROW + c] = In16<BF16>::to_f(q[(static_cast<long long>(h) * group + g) * D + c]);
    }
    if (tid < 4) misc[tid] = 0;
    __syncthreads();
    if constexpr (QUEST) {
        for (int i = tid; i < group * (D / 2); i += SELD_THREADS) {
            const int g = i / (D / 2), w = i - g * (D / 2);
            const uint32_t lo = qf[g * L::QROW + 2 * w] >= 0.0f ? 0xFFFFu : 0u;
            const uint32_t hi = qf[g * L::QROW + 2 * w + 1] >= 0.0f ? 0xFFFF0000u : 0u;
            qm[g * L::MROW + w] = lo | hi;
        }
    }
    if (two_pass && warp < group) {   // |q_g|_1, one warp per head
        float a1 = 0.0f;
        for (int c = lane; c < D; c += 32) a1 += fabsf(qf[warp * L::QROW + c]);
#pragma unroll
        for (int d = 16; d >= 1; d >>= 1) a1 += __shfl_xor_sync(0xFFFFFFFFu, a1, d);
        if (lane == 0) atomicMax(&misc[2], __float_as_int(a1));
    }

    // Statistics rows of list entries [t*64, t*64+64) -> shared-memory stage t & 1.  identity: entry i is page i.
    auto issue = [&](int t, int count, bool identity) {
        uint8_t* stage = tiles + (t & 1) * NARR * L::TILE_BYTES;
        const int p0 = t * SELD_TILE;
        const int rows = min(SELD_TILE, count - p0);
        for (int i = tid; i < rows * VEC; i += SELD_THREADS) {
            const int r = i / VEC, c = i - r * VEC;
            const int page = identity ? p0 + r : cand[p0 + r];
            const long long src = (static_cast<long long>(h) * cap_blocks + page) * D + c * 8;
            cp_async16(stage + r * L::ROW + c * 16, ka + src);
            if constexpr (QUEST) cp_async16(stage + L::TILE_BYTES + r * L::ROW + c * 16, kb + src);
        }
        cp_async_commit();
    };

    // Exact scores of `count` list entries into keys[entry] (the arithmetic of the reference's warp, one thread
    // per (page, head)).
    auto exact_pass = [&](int count, bool identity) {
        const int n_tiles = cdiv(count, SELD_TILE);
        const int pl = tid >> 2, sub = tid & 3;
        if (n_tiles > 0) issue(0, count, identity);
        for (int t = 0; t < n_tiles; ++t) {
            if (t + 1 < n_tiles) { issue(t + 1, count, identity); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
            __syncthreads();
            const uint8_t* stage = tiles + (t & 1) * NARR * L::TILE_BYTES;
            const int entry = t * SELD_TILE + pl;
            float best = -FLT_MAX;
            if (entry < count) {
                const uint4* ra = reinterpret_cast<const uint4*>(stage + pl * L::ROW);
                const uint4* rb = reinterpret_cast<const uint4*>(stage + L::TILE_BYTES + pl * L::ROW);
                for (int g = sub; g < group; g += 4) {
                    float2 acc[16];
#pragma unroll
                    for (int w = 0; w < 16; ++w) acc[w] = make_float2(0.0f, 0.0f);
                    const float4* qrow = reinterpret_cast<const float4*>(qf + g * L::QROW);
                    const uint4* mrow = reinterpret_cast<const uint4*>(qm + g * L::MROW);
#pragma unroll 1
                    for (int i = 0; i < D / 32; ++i) {
#pragma unroll
                        for (int v = 0; v < 4; ++v) {          // 8 channels per 16-byte chunk
                            const uint4 a = ra[i * 4 + v];
                            uint32_t kw[4] = {a.x, a.y, a.z, a.w};
                            if constexpr (QUEST) {
                                const uint4 b = rb[i * 4 + v];
                                const uint4 m = mrow[i * 4 + v];
                                kw[0] = (b.x & m.x) | (a.x & ~m.x);
                                kw[1] = (b.y & m.y) | (a.y & ~m.y);
                                kw[2] = (b.z & m.z) | (a.z & ~m.z);
                                kw[3] = (b.w & m.w) | (a.w & ~m.w);
                            }
                            const float4 q0 = qrow[i * 8 + v * 2], q1 = qrow[i * 8 + v * 2 + 1];
                            acc[v * 4 + 0] = fma2(make_float2(q0.x, q0.y), word_to_float2<BF16>(kw[0]), acc[v * 4 + 0]);
                            acc[v * 4 + 1] = fma2(make_float2(q0.z, q0.w), word_to_float2<BF16>(kw[1]), acc[v * 4 + 1]);
                            acc[v * 4 + 2] = fma2(make_float2(q1.x, q1.y), word_to_float2<BF16>(kw[2]), acc[v * 4 + 2]);
                            acc[v * 4 + 3] = fma2(make_float2(q1.z, q1.w), word_to_float2<BF16>(kw[3]), acc[v * 4 + 3]);
                        }
                    }
                    // butterfly pairing: partial j with j+16, then j+8, j+4, j+2, j+1
#pragma unroll
                    for (int w = 0; w < 8; ++w) acc[w] = add2(acc[w], acc[w + 8]);
#pragma unroll
                    for (int w = 0; w < 4; ++w) acc[w] = add2(acc[w], acc[w + 4]);
                    acc[0] = add2(acc[0], acc[2]);
                    acc[1] = add2(acc[1], acc[3]);
                    acc[0] = add2(acc[0], acc[1]);
                    const float s = __fadd_rn(acc[0].x, acc[0].y);
                    if (s > best) best = s;
                }
            }
            // the four threads of a page hold the maxima of their shares of the group
            {
                float o = __shfl_xor_sync(0xFFFFFFFFu, best, 1);
                if (o > best) best = o;
                o = __shfl_xor_sync(0xFFFFFFFFu, best, 2);
                if (o > best) best = o;
            }
            if (sub == 0 && entry < count) {
                const int page = identity ? entry : cand[entry];
                keys[entry] = seld_key((page < n_sink || page >= local_lo) ? -FLT_MAX : best, page);
            }
            __syncthreads();
        }
    };

    // ascending bitonic sort of keys[0, n)
    auto sort_keys = [&](int n) {
        for (int size = 2; size <= n; size <<= 1) {
            for (int stride = size >> 1; stride > 0; stride >>= 1) {
                __syncthreads();
                for (int t = tid; t < n / 2; t += SELD_THREADS) {
                    const int pos = 2 * t - (t & (stride - 1));
                    const unsigned long long a = keys[pos], b = keys[pos + stride];
                    const bool up = (pos & size) == 0;
                    if ((a > b) == up) { keys[pos] = b; keys[pos + stride] = a; }
                }
            }
        }
        __syncthreads();
    };
    auto pow2_at_least = [](int n) { int m = 2; while (m < n) m <<= 1; return m; };

    int n_sorted = 0;   // number of keys sorted at the end
    bool done = false;
    if (two_pass) {
        // ---------------- pass 1: approximate scores with tensor cores ----------------
        // Each warp takes 16 pages at a time straight from global memory: thread (r = lane/4, t = lane%4) reads
        // 16 contiguous bytes — channels 32 s + 8 t .. + 7 — of rows r and r + 8 for every 32-channel chunk s.
        // Those eight channels feed two m16n8k16 MMAs (slots k = 2t, 2t+1 and k = 2t+8, 2t+9 of each); the sum
        // over k does not care about the order as long as the q fragments below use the same assignment.
        constexpr int NSC = D / 32;
        uint32_t bp[NSC][2][2], bm[NSC][2][2];
        {
            const int gid = lane >> 2, t4 = lane & 3;
#pragma unroll
            for (int sc = 0; sc < NSC; ++sc)
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int hh = 0; hh < 2; ++hh) {
                        uint32_t w = 0u;
                        if (gid < group)
                            w = *reinterpret_cast<const uint32_t*>(q + (static_cast<long long>(h) * group + gid) * D +
                                                                   sc * 32 + 8 * t4 + 4 * j + 2 * hh);
                        const uint32_t neg = ((w & 0x8000u) ? 0xFFFFu : 0u) | ((w & 0x80000000u) ? 0xFFFF0000u : 0u);
                        bp[sc][j][hh] = w & ~neg;     // non-negative part of q
                        bm[sc][j][hh] = w & neg;      // negative part
                    }
        }
        uint32_t kabs2 = 0u;
        const int n_groups = cdiv(nk, 16);
        for (int grp = warp; grp < n_groups; grp += SELD_THREADS / 32) {
            const int pg0 = grp * 16 + (lane >> 2), pg1 = pg0 + 8;
            const int t4 = lane & 3;
            // rows past the end are read from the last page instead (in bounds) and ignored afterwards
            const long long r0 = (static_cast<long long>(h) * cap_blocks + min(pg0, nk - 1)) * D + 8 * t4;
            const long long r1 = (static_cast<long long>(h) * cap_blocks + min(pg1, nk - 1)) * D + 8 * t4;
            uint4 a0[NSC], a1[NSC], b0[QUEST ? NSC : 1], b1[QUEST ? NSC : 1];
#pragma unroll
            for (int sc = 0; sc < NSC; ++sc) {
                a0[sc] = __ldg(reinterpret_cast<const uint4*>(ka + r0 + sc * 32));
                a1[sc] = __ldg(reinterpret_cast<const uint4*>(ka + r1 + sc * 32));
                if constexpr (QUEST) {
                    b0[sc] = __ldg(reinterpret_cast<const uint4*>(kb + r0 + sc * 32));
                    b1[sc] = __ldg(reinterpret_cast<const uint4*>(kb + r1 + sc * 32));
                }
            }
            const uint32_t keep0 = pg0 < nk ? 0x7FFF7FFFu : 0u, keep1 = pg1 < nk ? 0x7FFF7FFFu : 0u;
            float c[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
            for (int sc = 0; sc < NSC; ++sc) {
                // MMA j uses words (2j, 2j+1) of the 16 bytes: fragment {row r: word 2j | row r+8: word 2j | row r: word 2j+1 | ...}
                const uint32_t fa[2][4] = {{a0[sc].x, a1[sc].x, a0[sc].y, a1[sc].y}, {a0[sc].z, a1[sc].z, a0[sc].w, a1[sc].w}};
                kabs2 = __vmaxu2(kabs2, __vmaxu2(__vmaxu2(a0[sc].x & keep0, a0[sc].y & keep0), __vmaxu2(a0[sc].z & keep0, a0[sc].w & keep0)));
                kabs2 = __vmaxu2(kabs2, __vmaxu2(__vmaxu2(a1[sc].x & keep1, a1[sc].y & keep1), __vmaxu2(a1[sc].z & keep1, a1[sc].w & keep1)));
                if constexpr (QUEST) {
                    const uint32_t fb[2][4] = {{b0[sc].x, b1[sc].x, b0[sc].y, b1[sc].y}, {b0[sc].z, b1[sc].z, b0[sc].w, b1[sc].w}};
                    kabs2 = __vmaxu2(kabs2, __vmaxu2(__vmaxu2(b0[sc].x & keep0, b0[sc].y & keep0), __vmaxu2(b0[sc].z & keep0, b0[sc].w & keep0)));
                    kabs2 = __vmaxu2(kabs2, __vmaxu2(__vmaxu2(b1[sc].x & keep1, b1[sc].y & keep1), __vmaxu2(b1[sc].z & keep1, b1[sc].w & keep1)));
#pragma unroll
                    for (int j = 0; j < 2; ++j) {
                        mma_16816<BF16>(c, fa[j], bm[sc][j][0], bm[sc][j][1]);   // minima meet the negative part of q
                        mma_16816<BF16>(c, fb[j], bp[sc][j][0], bp[sc][j][1]);   // maxima meet the non-negative part
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 2; ++j)
                        mma_16816<BF16>(c, fa[j], bp[sc][j][0] | bm[sc][j][0], bp[sc][j][1] | bm[sc][j][1]);
                }
            }
            // c0,c1: page lane/4, heads 2t,2t+1; c2,c3: page lane/4 + 8
            float lo = -FLT_MAX, hi = -FLT_MAX;
            if (2 * t4 < group) { lo = c[0]; hi = c[2]; }
            if (2 * t4 + 1 < group) { lo = fmaxf(lo, c[1]); hi = fmaxf(hi, c[3]); }
#pragma unroll
            for (int d = 1; d <= 2; d <<= 1) {
                lo = fmaxf(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, d));
                hi = fmaxf(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, d));
            }
            if (t4 == 0) {
                if (pg0 < nk) approx[pg0] = lo;
                if (pg1 < nk) approx[pg1] = hi;
            }
        }
        {   // largest |statistic| seen (16-bit patterns of non-negative values order like the values)
            uint32_t m16 = max(kabs2 & 0xFFFFu, kabs2 >> 16);
#pragma unroll
            for (int d = 16; d >= 1; d >>= 1) m16 = max(m16, __shfl_xor_sync(0xFFFFFFFFu, m16, d));
            if (lane == 0) atomicMax(&misc[1], static_cast<int>(m16));
        }
        __syncthreads();
        const float kabs = In16<BF16>::to_f(static_cast<uint16_t>(misc[1]));
        const float delta = __int_as_float(misc[2]) * kabs * (1.0f / 8192.0f);
        // ---------------- threshold: k-th largest lower bound, by radix selection ----------------
        // ascending 32-bit image of (approx - delta); forced pages rank lowest.  Four 8-bit digits, most
        // significant first: histogram of the keys that share the prefix found so far, then the digit whose
        // bucket holds the k-th largest.
        auto lower_key = [&](int i) -> uint32_t {
            if (i < n_sink || i >= local_lo) return 0u;
            float v = approx[i] - delta;
            if (v == 0.0f) v = 0.0f;
            const uint32_t u = __float_as_uint(v);
            return (u >> 31) ? ~u : (u | 0x80000000u);
        };
        int* hist = reinterpret_cast<int*>(keys);      // the key array is free until pass 2
        uint32_t prefix = 0u;
        int remaining = k;
        for (int shift = 24; shift >= 0; shift -= 8) {
            hist[tid] = 0;
            __syncthreads();
            for (int i = tid; i < nk; i += SELD_THREADS) {
                const uint32_t key = lower_key(i);
                if (shift == 24 || (key >> (shift + 8)) == (prefix >> (shift + 8))) atomicAdd(&hist[(key >> shift) & 255u], 1);
            }
            __syncthreads();
            if (warp == 0) {
                // lane l owns digits 8l .. 8l+7; walk from the largest digit down
                int cnt[8], mine = 0;
#pragma unroll
                for (int j = 0; j < 8; ++j) { cnt[j] = hist[lane * 8 + j]; mine += cnt[j]; }
                // inclusive suffix sums over the lanes
                int incl = mine;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int v = __shfl_down_sync(0xFFFFFFFFu, incl, d);
                    if (lane + d < 32) incl += v;
                }
                const int excl = incl - mine;                    // keys in digits above this lane's eight
                if (excl < remaining && remaining <= incl) {     // the k-th largest lies in this lane's digits
                    int seen = excl, digit = 0;
#pragma unroll
                    for (int j = 7; j >= 0; --j) {
                        if (seen < remaining && remaining <= seen + cnt[j]) { digit = lane * 8 + j; break; }
                        seen += cnt[j];
                    }
                    misc[3] = digit;
                    misc[0] = remaining - seen;                  // rank inside the chosen bucket
                }
            }
            __syncthreads();
            prefix |= static_cast<uint32_t>(misc[3]) << shift;
            remaining = misc[0];
            __syncthreads();
        }
        if (tid == 0) misc[0] = 0;
        float threshold;
        {
            // prefix 0 is the rank of a forced page: fewer than k free pages, so every one of them is a candidate
            const uint32_t u = (prefix >> 31) ? (prefix ^ 0x80000000u) : ~prefix;
            threshold = prefix == 0u ? -FLT_MAX : __uint_as_float(u);
        }
        __syncthreads();
        for (int i = tid; i < nk; i += SELD_THREADS) {
            if (i >= n_sink && i < local_lo && approx[i] + delta >= threshold) {
                const int slot = atomicAdd(&misc[0], 1);
                if (slot < SELD_CAND_CAP) cand[slot] = i;
            }
        }
        __syncthreads();
        const int n_cand = misc[0];
        if (n_cand <= SELD_CAND_CAP && isfinite(delta)) {
            // ---------------- pass 2: exact scores of the candidates ----------------
            n_sorted = pow2_at_least(n_cand);
            for (int i = tid; i < n_sorted; i += SELD_THREADS) keys[i] = ~0ull;
            __syncthreads();
            exact_pass(n_cand, false);
            // order the few candidates by counting: rank = number of smaller keys (keys are distinct)
            unsigned long long* sorted = keys + SELD_CAND_CAP;
            for (int i = tid; i < n_sorted; i += SELD_THREADS) sorted[i] = ~0ull;
            __syncthreads();
            for (int i = tid; i < n_cand; i += SELD_THREADS) {
                const unsigned long long mine = keys[i];
                int rank = 0;
                for (int j = 0; j < n_cand; ++j) rank += keys[j] < mine ? 1 : 0;
                sorted[rank] = mine;
            }
            __syncthreads();
            for (int i = tid; i < n_sorted; i += SELD_THREADS) keys[i] = sorted[i];
            __syncthreads();
            done = true;
        }
    }
    if (!done) {
        n_sorted = pow2_at_least(nk);
        __syncthreads();
        for (int i = tid; i < n_sorted; i += SELD_THREADS) keys[i] = ~0ull;
        __syncthreads();
        exact_pass(nk, true);
        sort_keys(n_sorted);
    }

    // rows are out_stride entries apart (>= width); the tail of a wider row is padding
    int32_t* row = out + static_cast<long long>(h) * out_stride;
    const bool pad = (sink + local) > 0;
    // optional scores of the picks (forced blocks +FLT_MAX, padding -FLT_MAX): what a shard of a longer
    // sequence sends to its peers so that all of them derive the same global top-k
    float* srow = out_scores ? out_scores + static_cast<long long>(h) * out_stride : nullptr;
    for (int i = tid; i < forced; i += SELD_THREADS) {
        row[i] = i < n_sink ? i : local_lo + (i - n_sink);
        if (srow) srow[i] = FLT_MAX;
    }
    for (int r = tid; r < k; r += SELD_THREADS) {
        int32_t id = -1;
        float sc = -FLT_MAX;
        if (r < n_sorted) {
            const unsigned long long key = keys[r];
            const bool real = key != ~0ull;
            const bool found = real && seld_key_score(key) > -FLT_MAX * 0.5f;
            if (found || (!pad && real)) { id = seld_key_page(key); sc = seld_key_score(key); }
        }
        row[forced + r] = id;
        if (srow) srow[forced + r] = sc;
    }
    for (int i = forced + k + tid; i < out_stride; i += SELD_THREADS) {
        row[i] = -1;
        if (srow) srow[i] = -FLT_MAX;
    }
}


int select_prefill_dispatch(const void* q_mean, const void* ka, const void* kb, void* out, int heads, int group, int nq,
                            int nk, int d, int k, int causal, int quest, int is_bf16, int sink, int local,
                            cudaStream_t stream) {
    if (!q_mean || !ka || !out || (quest && !kb)) return TA100_ERR_NULL;
    if (d != 64 && d != 128) return TA100_ERR_UNSUPPORTED;
    if (nk > 2048 || nk < 0 || k < 0 || group <= 0 || heads % group != 0) return TA100_ERR_SHAPE;
    if (sink + local + k == 0 || heads == 0 || nq == 0) return TA100_OK;
    const int nk_pad = (nk + 31) & ~31;
    const size_t smem = d == 128 ? SelpSmem<128>::total(nk_pad) : SelpSmem<64>::total(nk_pad);
    const long long work = static_cast<long long>(heads) * cdiv(nq, SEL_WARPS);
    const int grid = static_cast<int>(work < NUM_SMS_HINT * 8LL ? work : NUM_SMS_HINT * 8LL);
#define TA100_SEL(DD, BFF, QQ)                                                                                   \
    do {                                                                                                         \
        cudaFuncSetAttribute(select_prefill_kernel<DD, BFF, QQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,    \
                             static_cast<int>(smem));                                                            \
        select_prefill_kernel<DD, BFF, QQ><<<grid, SEL_WARPS * 32, smem, stream>>>(                              \
            static_cast<const uint16_t*>(q_mean), static_cast<const uint16_t*>(ka),                              \
            static_cast<const uint16_t*>(kb), static_cast<int32_t*>(out), heads, group, nq, nk, k, causal, sink, \
            local);                                                                                              \
    } while (0)
    if (d == 128) {
        if (is_bf16) { if (quest) TA100_SEL(128, true, true); else TA100_SEL(128, true, false); }
        else { if (quest) TA100_SEL(128, false, true); else TA100_SEL(128, false, false); }
    } else {
        if (is_bf16) { if (quest) TA100_SEL(64, true, true); else TA100_SEL(64, true, false); }
        else { if (quest) TA100_SEL(64, false, true); else TA100_SEL(64, false, false); }
    }
#undef TA100_SEL
    return static_cast<int>(cudaGetLastError());
}

// dyn (may be null): the block counts come from a sequence length in device memory; nk is then the largest block
// count the launch has to cope with, k / sink / local are ignored and out_stride (> 0) is the row width.
int select_decode_dispatch(const void* q, const void* ka, const void* kb, void* out, void* out_scores, int flat_heads, int group, int nk,
                           int cap_blocks, int d, int k, int quest, int is_bf16, int sink, int local, int out_stride,
                           const DynLength* dyn, cudaStream_t stream) {
    if (!q || !ka || !out || (quest && !kb)) return TA100_ERR_NULL;
    DynLength dl{};
    if (dyn && dyn->len) {
        dl = *dyn;
        if (out_stride <= 0 || dl.sink < 0 || dl.local < 0) return TA100_ERR_SHAPE;
        int n = 0, kk = 0, sk = 0, lc = 0;
        dyn_select_counts(dl, nk * 64, cap_blocks < 2048 ? cap_blocks : 2048, n, kk, sk, lc);
        if (out_stride < kk + dl.sink + dl.local) return TA100_ERR_SHAPE;   // counts only grow with the length
        k = kk; sink = 0; local = 0;
    }
    if (out_stride == 0) out_stride = sink + local + k;
    if (out_stride < sink + local + k) return TA100_ERR_SHAPE;
    if (d != 64 && d != 128) return TA100_ERR_UNSUPPORTED;
    if (nk > 2048 || nk < 0 || k < 0 || nk > cap_blocks || group <= 0) return TA100_ERR_SHAPE;
    if (!dl.len && (sink + local) == 0 && k > nk) return TA100_ERR_SHAPE;
    if (flat_heads == 0 || (!dl.len && sink + local + k == 0)) return TA100_OK;
    if (group > SELD_MAX_GROUP) return TA100_ERR_LIMIT;
#define TA100_SELD(DD, BFF, QQ)                                                                                \
    do {                                                                                                       \
        const int smem = SeldSmem<DD>::total(QQ);                                                              \
        cudaFuncSetAttribute(select_decode_kernel<DD, BFF, QQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        select_decode_kernel<DD, BFF, QQ><<<flat_heads, SELD_THREADS, smem, stream>>>(                         \
            static_cast<const uint16_t*>(q), static_cast<const uint16_t*>(ka), static_cast<const uint16_t*>(kb), \
            static_cast<int32_t*>(out), static_cast<float*>(out_scores), group, nk, cap_blocks, k, sink, local, \
            out_stride, dl);                                                                                   \
    } while (0)
    if (d == 128) {
        if (is_bf16) { if (quest) TA100_SELD(128, true, true); else TA100_SELD(128, true, false); }
        else { if (quest) TA100_SELD(128, false, true); else TA100_SELD(128, false, false); }
    } else {
        if (is_bf16) { if (quest) TA100_SELD(64, true, true); else TA100_SELD(64, true, false); }
        else { if (quest) TA100_SELD(64, false, true); else TA100_SELD(64, false, false); }
    }
#undef TA100_SELD
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// KV-sequence-sharded decode: global top-k from the shards' candidate lists
// ---------------------------------------------------------------------------
// Every shard runs select_decode_kernel over its own pages with out_scores and all-gathers its
// [2, rows, width] buffer (plane 0 page ids local to the shard, plane 1 fp32 scores; forced pages carry
// +FLT_MAX, padding -1 / -FLT_MAX).  Any page of the global top-k is in its shard's top-k, so sorting the
// union with the single-GPU key (score descending, then the tie-break rank of the GLOBAL page id) gives the
// single-GPU selection.  One CTA per row writes this shard's part of it as local page ids:
//   out[row] = [ this shard's forced pages | -1 ... up to sink+local | pick j if it lies in this shard else -1 ]
// Shard r owns pages [shard_page_begin(r), shard_page_begin(r + 1)): the even split r * total / world with every
// inner boundary moved to the nearest multiple of 32 pages.  The selection kernel cuts and orders exact ties by
// (bit-reversed page mod 32, page div 32) of its LOCAL page ids; with shard starts that are multiples of 32 this is
// the order of the global ids, so a tie at a shard's own cut is resolved as the single-GPU kernel resolves it.
// (A shard may come out empty when there are fewer than 32 pages per shard.)
__host__ __device__ inline int shard_page_begin(int r, int world, int total_pages) {
    if (r <= 0) return 0;
    if (r >= world) return total_pages;
    const long long even = static_cast<long long>(r) * total_pages / world;
    const long long aligned = (even + 16) / 32 * 32;
    return static_cast<int>(aligned < total_pages ? aligned : total_pages);
}
constexpr int MERGE_CAP = 2048;
__global__ void __launch_bounds__(256)
merge_page_candidates_kernel(const int32_t* __restrict__ gathered, int32_t* __restrict__ out, int rows, int world,
                             int width, int rank, int total_pages, int top_k, int sink, int local) {
    __shared__ unsigned long long keys[MERGE_CAP];
    const int row = blockIdx.x, tid = threadIdx.x;
    const int n = world * width;
    int n_sorted = 2;
    while (n_sorted < n) n_sorted <<= 1;
    const long long plane = static_cast<long long>(rows) * width;
    for (int i = tid; i < n_sorted; i += blockDim.x) {
        unsigned long long key = ~0ull;
        if (i < n) {
            const int r = i / width, j = i - r * width;
            const int32_t* base = gathered + static_cast<long long>(r) * 2 * plane + static_cast<long long>(row) * width + j;
            const int page = base[0];
            const float score = __int_as_float(base[plane]);
            if (page >= 0 && score < FLT_MAX && score > -FLT_MAX)
                key = seld_key(score, page + shard_page_begin(r, world, total_pages));
        }
        keys[i] = key;
    }
    for (int size = 2; size <= n_sorted; size <<= 1)
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int t = tid; t < n_sorted / 2; t += blockDim.x) {
                const int pos = 2 * t - (t & (stride - 1));
                const unsigned long long a = keys[pos], b = keys[pos + stride];
                const bool up = (pos & size) == 0;
                if ((a > b) == up) { keys[pos] = b; keys[pos + stride] = a; }
            }
        }
    __syncthreads();
    const int begin = shard_page_begin(rank, world, total_pages);
    const int end = shard_page_begin(rank + 1, world, total_pages);
    const int out_width = sink + local + top_k;
    int32_t* orow = out + static_cast<long long>(row) * out_width;
    const int32_t* mine = gathered + static_cast<long long>(rank) * 2 * plane + static_cast<long long>(row) * width;
    for (int i = tid; i < sink + local; i += blockDim.x) {
        // this shard's forced pages lead its own list
        const bool forced = i < width && mine[i] >= 0 && __int_as_float(mine[plane + i]) >= FLT_MAX;
        orow[i] = forced ? mine[i] : -1;
    }
    for (int j = tid; j < top_k; j += blockDim.x) {
        int32_t id = -1;
        if (j < n_sorted && keys[j] != ~0ull) {
            const int page = seld_key_page(keys[j]);
            if (page >= begin && page < end) id = page - begin;
        }
        orow[sink + local + j] = id;
    }
}

int merge_page_candidates_dispatch(const void* gathered, void* out, int rows, int world, int width, int rank,
                                   int total_pages, int top_k, int sink, int local, cudaStream_t stream) {
    if (!gathered || !out) return TA100_ERR_NULL;
    if (rows < 0 || world <= 0 || width < 0 || rank < 0 || rank >= world || total_pages < 0 || top_k < 0 || sink < 0 ||
        local < 0)
        return TA100_ERR_SHAPE;
    if (static_cast<long long>(world) * width > MERGE_CAP) return TA100_ERR_LIMIT;
    if (rows == 0 || sink + local + top_k == 0) return TA100_OK;
    merge_page_candidates_kernel<<<rows, 256, 0, stream>>>(static_cast<const int32_t*>(gathered),
                                                           static_cast<int32_t*>(out), rows, world, width, rank,
                                                           total_pages, top_k, sink, local);
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Local windows and bitset packing
// ---------------------------------------------------------------------------
__global__ void local_prefill_kernel(int32_t* __restrict__ out, long long rows, int nq, int nk, int k, int causal) {
    const long long total = rows * k;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const long long row = i / k;
        const int rank = static_cast<int>(i - row * k);
        const int qb = static_cast<int>(row % nq);
        int start, valid = k;
        if (causal) {
            const int end = min(qb, nk - 1);
            valid = min(end + 1, k);
            start = max(0, end - k + 1);
        } else {
            const int center = min(qb, nk - 1);
            const int max_start = max(nk - k, 0);
            start = min(max(center - k / 2, 0), max_start);
        }
        out[i] = rank < valid ? start + rank : -1;
    }
}

__global__ void local_decode_kernel(int32_t* __restrict__ out, long long rows, int nk, int k) {
    const long long total = rows * k;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = nk - k + static_cast<int>(i % k);
}

// sel [rows, k] -> mask [rows, words] (64-bit words, bit b of word w = block 64w + b).
__global__ void __launch_bounds__(128) pack_mask_kernel(const int32_t* __restrict__ sel,
                                                        unsigned long long* __restrict__ mask, long long rows, int k,
                                                        int nk, int words) {
    __shared__ unsigned long long s_words[32];
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        if (threadIdx.x < 32) s_words[threadIdx.x] = 0ull;
        __syncthreads();
        for (int i = threadIdx.x; i < k; i += blockDim.x) {
            const int b = sel[row * k + i];
            if (b >= 0 && b < nk && (b >> 6) < words && (b >> 6) < 32) atomicOr(&s_words[b >> 6], 1ull << (b & 63));
        }
        __syncthreads();
        if (threadIdx.x < words && threadIdx.x < 32) mask[row * words + threadIdx.x] = s_words[threadIdx.x];
        __syncthreads();
    }
}

int local_prefill_dispatch(void* out, long long rows_heads, int nq, int nk, int k, int causal, cudaStream_t stream) {
    if (k == 0 || rows_heads * nq == 0) return TA100_OK;
    if (!out) return TA100_ERR_NULL;
    const long long rows = rows_heads * nq;
    local_prefill_kernel<<<grid_for(rows * k, 256, 8), 256, 0, stream>>>(static_cast<int32_t*>(out), rows, nq, nk, k, causal);
    return static_cast<int>(cudaGetLastError());
}

int local_decode_dispatch(void* out, long long rows, int nk, int k, cudaStream_t stream) {
    if (k == 0 || rows == 0) return TA100_OK;
    if (!out) return TA100_ERR_NULL;
    if (k > nk) return TA100_ERR_SHAPE;
    local_decode_kernel<<<grid_for(rows * k, 256, 8), 256, 0, stream>>>(static_cast<int32_t*>(out), rows, nk, k);
    return static_cast<int>(cudaGetLastError());
}

int pack_mask_dispatch(const void* sel, void* mask, long long rows, int k, int nk, int words, cudaStream_t stream) {
    if (rows == 0 || words == 0) return TA100_OK;
    if (!sel || !mask) return TA100_ERR_NULL;
    if (words > 32) return TA100_ERR_LIMIT;
    const int grid = static_cast<int>(rows < NUM_SMS_HINT * 16LL ? rows : NUM_SMS_HINT * 16LL);
    pack_mask_kernel<<<grid, 128, 0, stream>>>(static_cast<const int32_t*>(sel), static_cast<unsigned long long*>(mask),
                                               rows, k, nk, words);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace ta100
