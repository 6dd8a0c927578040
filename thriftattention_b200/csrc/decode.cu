// Single-token (decode) selective mixed-precision attention, split over the KV
// sequence, plus the log-sum-exp merge of the partial results.
//
// One CTA per chain: chain s of a (sequence, KV head) pair walks pages
// [s*n/S, (s+1)*n/S) of 64 tokens — first the pages that are NOT selected (FP4 K/V),
// ascending, then the selected pages (16-bit K/V), ascending.  The kernel is
// HBM-bound, so the arithmetic is kept off the instruction pipes:
//   * pages arrive by TMA (tiled tensor maps over the contiguous cache or the page
//     pools) into a ring of shared-memory slots;
//   * S = Q K^T and O += P V are tcgen05 MMAs — block-scaled FP4 (the tensor core
//     applies the E4M3 / E8M0 scales) or f16/bf16 — with accumulators in tensor memory.
// The query group is tiny (G <= 16 heads), the MMA tile has 128 rows: every head is
// stored FOUR times, in rows 32*c + g (c = 0..3: one row per softmax warp), and the thread
// that owns row (g, c) handles token columns [16c, 16c+16) of each page - a warp's
// tensor-memory load takes one column address, so the quarter is the warp's.  Its P row is
// zero outside those columns, so the four O rows of a head are partial sums that are
// added once, at the end of the chain.  All four use the running row maximum of the
// whole 64-token page, as the reference does, because the quantisation of P
// (dynamic scale per 16 / 32 tokens, codes computed with the un-rounded scale) depends
// on it: the warps exchange their quarters' maxima through shared memory once per page.
//
// Warp roles (224 threads): warp 0 = page list + TMA producer (its 32 lanes also bring the K
// and V block scales of every page into the 512-byte atom order the tensor core reads),
// warp 1 = issuer of the S = Q K^T MMAs and tensor-memory owner, warp 2 = issuer of the
// O += P V MMAs (one thread needs some hundred cycles to issue the scale copies, MMAs and
// commits of a page, so the two streams are issued side by side), warps 3..6 = softmax.
// Two CTAs share an SM.
// The ring holds five FP4 pages in flight; when the chain turns to its 16-bit pages the same
// memory is re-cut into three 16 KB tiles.
// Every mbarrier wait is bounded; a timeout raises a CTA-wide abort flag, all roles
// drain, tensor memory is released and a status word is set.
#include <cfloat>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ta100 {

namespace {

constexpr int PAGE = 64;
constexpr int DEC_THREADS = 224;
constexpr int DEC_NS4 = 5;              // ring slots while the chain reads FP4 pages
constexpr int DEC_SLOT4_BYTES = 9728;   //   K4 4096 + V4 4096 + K scale atoms 1024 + V scale atom 512
constexpr int DEC_NS16 = 3;             // ring slots while it reads 16-bit pages (same memory, re-cut)
constexpr int DEC_SLOT16_BYTES = 16384; //   one K or V page
constexpr int DEC_RING_BYTES = 49152;
static_assert(DEC_NS4 * DEC_SLOT4_BYTES <= DEC_RING_BYTES && DEC_NS16 * DEC_SLOT16_BYTES <= DEC_RING_BYTES, "ring size");
static_assert(DEC_SLOT4_BYTES % 512 == 0, "FP4 slots keep the 64-byte-swizzle alignment");
constexpr int DEC_LIST_CAP = 1024;      // pages per chain
static_assert(2 * DEC_LIST_CAP * 4 <= DEC_RING_BYTES, "the idle page ring stages a chain's page-table entries and 16-bit keys");
constexpr int DEC_MAX_GROUP = 16;

// tensor-memory columns (256 allocated per CTA)
constexpr uint32_t DTM_O = 0;           // 128 columns
constexpr uint32_t DTM_S = 128;         // 64 columns
constexpr uint32_t DTM_SFA_Q = 192;     // up to 8 columns
constexpr uint32_t DTM_SFB_K = 200;     // up to 8 columns; second buffer at DTM_SFB_K2
constexpr uint32_t DTM_SFA_P = 208;     // two buffers of 4 columns
constexpr uint32_t DTM_SFB_V = 216;     // two buffers of 4 columns
constexpr uint32_t DTM_SFB_K2 = 224;    // up to 8 columns
constexpr uint32_t DTM_COLS = 256;

constexpr uint32_t L_FP16 = 0x80000000u;  // page-list flag: 16-bit page

__device__ int g_decode_status;           // wait site of a kernel whose bounded wait ran out, or STATUS_BAD_PAGE
constexpr int STATUS_BAD_PAGE = 1000;    // a page-table entry outside the pool was skipped


struct DecodeParams {
    const uint16_t* q_hi;   // [heads, G, D]
    const uint8_t* q4;      // [heads, G, D/2]
    const uint8_t* qs;      // [heads, G, D/g]
    const uint8_t* ks;      // K block scales: rows layout or page pool
    const uint8_t* vs;      // V block scales: transposed layout or page pool
    const int32_t* sel;     // [heads, width]
    const int32_t* page_table;  // [batch, max_pages] or null
    float* part_o;          // [heads, splits, G, D]
    float* part_ml;         // [heads, splits, G, 2]
    const int32_t* len_dev; // null, or the sequence length(s) in device memory: npages is then only the upper bound
    int len_per_seq;        // 0: len_dev[0] for every sequence; 1: len_dev[sequence]
    int len_offset;         // added to the length
    int heads, hkv, G, npages, cap_pages, max_pages, pool_pages, width, splits;
    int vs_row_stride;      // bytes between channel rows of vs (contiguous layout)
    float c2;               // (1/sqrt(d)) * log2(e)
    float sm_scale;         // 1/sqrt(d)
    long long budget;
    int skip_loads;         // diagnostics: the producer issues no copies
};

template <int D>
struct DecSmem {
    static constexpr int Q4 = 0;                          // 128 x D/2, 64-byte swizzle
    static constexpr int QSF = Q4 + 128 * D / 2;          // up to 2 atoms
    static constexpr int Q16 = QSF + 1024;                // 128 x D x 2, two 64-column halves, 128-byte swizzle
    static constexpr int P = Q16 + 128 * D * 2;           // 16 KB: two 4 KB FP4 buffers or one 16-bit tile
    static constexpr int SLOTS = P + 16384;
    static constexpr int PSF = SLOTS + DEC_RING_BYTES;    // two 512-byte atoms
    static constexpr int LIST = PSF + 1024;               // DEC_LIST_CAP x u32
    static constexpr int BITS = LIST + DEC_LIST_CAP * 4;  // 64 words: selected pages of the chain
    static constexpr int BARS = BITS + 256;
    static constexpr int TOTAL = BARS + 2048;
    // inside an FP4 slot
    static constexpr int K4 = 0, V4 = 4096, KSF = 8192, VSF = 9216;
    static_assert(Q16 % 1024 == 0 && P % 1024 == 0 && SLOTS % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static_assert(TOTAL <= 113 * 1024, "two CTAs must fit one SM");
};

struct DecBars {
    uint64_t q_ready, list_full;
    uint64_t f_full[DEC_NS4], f_empty[DEC_NS4];   // FP4 ring: page landed (TMA bytes + 32 scale-atom arrivals), released
    // 16-bit ring.  A slot alternates between K and V tiles and the two kinds are consumed by different warps; a
    // parity wait only works for a waiter that sees every phase of its barrier, so K and V arrivals are kept on
    // separate barriers (page j: K tile 2j and V tile 2j + 1, slot = tile mod 3, use index j / 3 on either kind).
    uint64_t hk_full[DEC_NS16], hv_full[DEC_NS16], h_empty[DEC_NS16];
    uint64_t s_full, s_free;
    uint64_t p_full[2], p_free[2];
    uint64_t epi_full;
    int n_total, n_fp4;
    uint32_t tmem_base;
    int abort_flag;
    int abort_code;     // which wait gave up first (development aid, reported through the status word)
    int bad_entry;      // a page-table entry pointed outside the pool
    float m_row[DEC_MAX_GROUP];
    float l_part[4][DEC_MAX_GROUP];
    uint64_t x_full;            // every softmax thread has published its quarter's maximum of the page
    float xch[2][4][32];        // [page parity][column quarter][head]: the quarters' maxima, exchanged between the warps
};
static_assert(sizeof(DecBars) <= 2048, "barrier block must fit its shared-memory slot");

__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// packed fp32x2 arithmetic (two values per instruction) and a three-input maximum
__device__ __forceinline__ uint64_t pack2f(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Page list of one chain (whole warp): FP4 pages ascending, then the selected pages ascending.
// An entry is the page's addressing key — the physical page times hkv plus the KV head for a page
// pool, the logical page for a contiguous cache — with L_FP16 set on 16-bit pages.
// A page-table entry outside [0, pool_pages) never becomes a key: the page is left out of the chain
// (nothing is read for it) and *bad_entry is raised so that the host learns of it.
// `stage` (shared memory, 2 x DEC_LIST_CAP words) first receives the chain's page-table entries in one sweep of
// independent loads (fetched inside the sweep below, every 32 pages would cost a round trip to global memory); its
// second half collects the keys of the selected pages while one sweep over the pages writes the FP4 keys straight
// into the list, and is appended to the list at the end.
__device__ void build_page_list(const DecodeParams& p, int h, int b, int kvh, int p_begin, int p_end, uint32_t* bits,
                                uint32_t* list, int32_t* stage, int& n_fp4, int& n_total, int lane, int* bad_entry) {
    for (int i = lane; i < 64; i += 32) bits[i] = 0u;
    if (p.page_table) {
        const int32_t* row = p.page_table + static_cast<long long>(b) * p.max_pages + p_begin;
#pragma unroll 4
        for (int i = lane; i < p_end - p_begin; i += 32) stage[i] = __ldg(row + i);
    }
    __syncwarp();
    for (int i = lane; i < p.width; i += 32) {
        const int id = p.sel[static_cast<long long>(h) * p.width + i];
        if (id >= p_begin && id < p_end) atomicOr(&bits[id >> 5], 1u << (id & 31));
    }
    __syncwarp();
    uint32_t* hi = reinterpret_cast<uint32_t*>(stage) + DEC_LIST_CAP;
    const uint32_t below = (1u << lane) - 1u;
    int n4 = 0, n16 = 0;
    for (int base = p_begin; base < p_end; base += 32) {
        const int pg = base + lane;
        bool take = pg < p_end;
        const bool is_sel = take && ((bits[pg >> 5] >> (pg & 31)) & 1u);
        uint32_t key = static_cast<uint32_t>(pg);
        if (take && p.page_table) {
            const int entry = stage[pg - p_begin];
            if (entry < 0 || entry >= p.pool_pages) {
                take = false;
                *bad_entry = 1;
            } else {
                key = static_cast<uint32_t>(entry) * static_cast<uint32_t>(p.hkv) + static_cast<uint32_t>(kvh);
            }
        }
        const uint32_t m4 = __ballot_sync(0xFFFFFFFFu, take && !is_sel);
        const uint32_t m16 = __ballot_sync(0xFFFFFFFFu, take && is_sel);
        if (take && !is_sel) list[n4 + __popc(m4 & below)] = key;
        if (take && is_sel) hi[n16 + __popc(m16 & below)] = key | L_FP16;
        n4 += __popc(m4);
        n16 += __popc(m16);
    }
    __syncwarp();
    for (int i = lane; i < n16; i += 32) list[n4 + i] = hi[i];
    n_fp4 = n4;
    n_total = n4 + n16;
}

template <int D, bool MX, bool BF16>
__global__ void __launch_bounds__(DEC_THREADS, 2)
decode_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap mapK4, const __grid_constant__ CUtensorMap mapV4,
              const __grid_constant__ CUtensorMap mapK16, const __grid_constant__ CUtensorMap mapV16) {
    using L = DecSmem<D>;
    constexpr uint32_t ROW4 = D / 2;                                   // bytes per FP4 row of Q / K
    constexpr uint32_t SWZ_QK = (ROW4 == 64) ? SWZ_64B : SWZ_32B;
    constexpr uint32_t SBO_QK = 8 * ROW4;
    constexpr int GRP = MX ? 32 : 16;
    constexpr int QK_ATOMS = MX ? 1 : D / 64;
    constexpr int KBLK = D / 64;
    constexpr float CSCALE = MX ? 6.0f : 2688.0f;
    constexpr float LOG2_C = MX ? 2.5849625007211562f : 11.392317422778761f;

    extern __shared__ __align__(1024) uint8_t smem[];
    DecBars& bars = *reinterpret_cast<DecBars*>(smem + L::BARS);
    uint32_t* list = reinterpret_cast<uint32_t*>(smem + L::LIST);
    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t sbase = smem_u32(smem);
    volatile int* abortp = &bars.abort_flag;
    const long long budget = p.budget;
    // bounded wait that remembers the first site that gave up
    auto waitc = [&](int code, uint64_t* bar, uint32_t parity) -> bool {
        if (mbar_wait(smem_u32(bar), parity, abortp, budget)) return true;
        atomicCAS(&bars.abort_code, 0, code);
        return false;
    };

    const int split = blockIdx.x, h = blockIdx.y;
    const int b = h / p.hkv, kvh = h - b * p.hkv;
    const int G = p.G;
    int npages = p.npages;
    if (p.len_dev != nullptr)
        npages = min(npages, max(1, cdiv(max(0, __ldg(p.len_dev + (p.len_per_seq ? b : 0)) + p.len_offset), PAGE)));
    const int p_begin = static_cast<int>(static_cast<long long>(split) * npages / p.splits);
    const int p_end = static_cast<int>(static_cast<long long>(split + 1) * npages / p.splits);
    const bool paged = p.page_table != nullptr;
    if (p_begin >= p_end) {
        // more chains than pages (only with a device-side length, whose launch is sized for the longest sequence):
        // a neutral partial, before anything is set up
        const long long pbase = (static_cast<long long>(h) * p.splits + split) * p.G;
        for (int i = tid; i < p.G * D; i += DEC_THREADS) p.part_o[pbase * D + i] = 0.0f;
        for (int i = tid; i < p.G; i += DEC_THREADS) { p.part_ml[(pbase + i) * 2] = -FLT_MAX; p.part_ml[(pbase + i) * 2 + 1] = 0.0f; }
        return;
    }

    if (tid == 0) {
        mbar_init(smem_u32(&bars.q_ready), 128);
        mbar_init(smem_u32(&bars.list_full), 1);
        mbar_init(smem_u32(&bars.s_full), 1);
        mbar_init(smem_u32(&bars.s_free), 128);
        mbar_init(smem_u32(&bars.epi_full), 128);
        mbar_init(smem_u32(&bars.x_full), 128);
        for (int i = 0; i < DEC_NS4; ++i) {
            mbar_init(smem_u32(&bars.f_full[i]), 33);   // lane 0's expect_tx arrival + one arrival per lane
            mbar_init(smem_u32(&bars.f_empty[i]), 1);
        }
        for (int i = 0; i < DEC_NS16; ++i) {
            mbar_init(smem_u32(&bars.hk_full[i]), 1);
            mbar_init(smem_u32(&bars.hv_full[i]), 1);
            mbar_init(smem_u32(&bars.h_empty[i]), 1);
        }
        for (int i = 0; i < 2; ++i) {
            mbar_init(smem_u32(&bars.p_full[i]), 128);
            mbar_init(smem_u32(&bars.p_free[i]), 1);
        }
        mbar_fence_init();
        bars.abort_flag = (sbase & 1023u) ? 1 : 0;
        bars.abort_code = 0;
        bars.bad_entry = 0;
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(&bars.tmem_base), DTM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = bars.tmem_base;

    if (warp == 0) {
        // =========================== page list + TMA producer ===========================
        if (lane == 0) {
            tma_prefetch_desc(&mapK4); tma_prefetch_desc(&mapV4);
            if (p.width > 0) { tma_prefetch_desc(&mapK16); tma_prefetch_desc(&mapV16); }
        }
        int n_fp4 = 0, n = 0;
        // the page ring is idle until the first copy below: its first 8 KB serve the list builder as scratch
        build_page_list(p, h, b, kvh, p_begin, p_end, reinterpret_cast<uint32_t*>(smem + L::BITS), list,
                        reinterpret_cast<int32_t*>(smem + L::SLOTS), n_fp4, n, lane, &bars.bad_entry);
        if (lane == 0) { bars.n_fp4 = n_fp4; bars.n_total = n; }
        __syncwarp();
        fence_proxy_async_smem();    // the staged entries were written and read through the generic proxy; copies follow
        __threadfence_block();
        if (lane == 0) mbar_arrive(smem_u32(&bars.list_full));
        // ---- FP4 pages: TMA for the codes; the lanes fetch the page's block scales two pages ahead and store
        //      them in atom order (word m0 * 4 + m1 holds the scales of row / channel 32 * m1 + m0) ----
        // K scales: D / GRP bytes per token row = KROW_WORDS 32-bit words (one 16-bit word for MXFP4 at D = 64);
        // V scales: PAGE / GRP bytes per channel row and page (4 NVFP4, 2 MXFP4)
        constexpr int KS_PAGE = PAGE * (D / GRP), VS_PAGE = D * (PAGE / GRP);
        constexpr int KROW_BYTES = D / GRP;
        constexpr int KROW_WORDS = KROW_BYTES >= 4 ? KROW_BYTES / 4 : 1;
        constexpr int KW = PAGE * KROW_WORDS / 32;   // K scale words per lane and page (4 or 2)
        constexpr int VW = D / 32;                   // V scale words per lane and page (4 or 2)
        auto load_sf = [&](int i, uint32_t (&kw)[4], uint32_t (&vw)[4]) {
            if (i >= n_fp4) return;
            const uint32_t key = list[i];
            const uint8_t* kp = paged ? p.ks + static_cast<long long>(key) * KS_PAGE
                                      : p.ks + (static_cast<long long>(h) * p.cap_pages + key) * KS_PAGE;
#pragma unroll
            for (int j = 0; j < KW; ++j) {
                if constexpr (KROW_BYTES >= 4) kw[j] = __ldg(reinterpret_cast<const uint32_t*>(kp) + lane + 32 * j);
                else kw[j] = __ldg(reinterpret_cast<const uint16_t*>(kp) + lane + 32 * j);
            }
#pragma unroll
            for (int j = 0; j < VW; ++j) {
                const int ch = lane + 32 * j;
                if constexpr (MX) {
                    const uint8_t* vp = paged ? p.vs + static_cast<long long>(key) * VS_PAGE + ch * 2
                                              : p.vs + (static_cast<long long>(h) * D + ch) * p.vs_row_stride + key * 2;
                    vw[j] = __ldg(reinterpret_cast<const uint16_t*>(vp));
                } else {
                    const uint8_t* vp = paged ? p.vs + static_cast<long long>(key) * VS_PAGE + ch * 4
                                              : p.vs + (static_cast<long long>(h) * D + ch) * p.vs_row_stride + key * 4;
                    vw[j] = __ldg(reinterpret_cast<const uint32_t*>(vp));
                }
            }
        };
        auto fp4_step = [&](int i, const uint32_t (&kw)[4], const uint32_t (&vw)[4]) -> bool {
            const uint32_t slot = i % DEC_NS4;
            if (!waitc(1, &bars.f_empty[slot], ((i / DEC_NS4) & 1) ^ 1)) return false;
            const uint32_t key = list[i];
            const int slab = paged ? static_cast<int>(key) : h;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&bars.f_full[slot]);
                const uint32_t sa = sbase + L::SLOTS + slot * DEC_SLOT4_BYTES;
                mbar_expect_tx(bar, PAGE * (D / 2) + D * (PAGE / 2));
                tma_load_3d(sa + L::K4, &mapK4, bar, 0, paged ? 0 : static_cast<int>(key) * PAGE, slab);
                tma_load_3d(sa + L::V4, &mapV4, bar, paged ? 0 : static_cast<int>(key) * (PAGE / 2), 0, slab);
            }
            uint8_t* sl = smem + L::SLOTS + slot * DEC_SLOT4_BYTES;
#pragma unroll
            for (int j = 0; j < KW; ++j) {
                const int w = lane + 32 * j;                     // word w: token w / KROW_WORDS, atom w % KROW_WORDS
                const int tok = w / KROW_WORDS, atom = w % KROW_WORDS;
                reinterpret_cast<uint32_t*>(sl + L::KSF + atom * 512)[(tok & 31) * 4 + (tok >> 5)] = kw[j];
            }
#pragma unroll
            for (int j = 0; j < VW; ++j) reinterpret_cast<uint32_t*>(sl + L::VSF)[lane * 4 + j] = vw[j];
            fence_proxy_async_smem();
            mbar_arrive(smem_u32(&bars.f_full[slot]));
            return true;
        };
        bool ok = !p.skip_loads;   // diagnostics: with skip_loads nothing is copied and the consumers' bounded waits run out
        if (ok) {
            // the scales of page i + 2 are requested when page i is handed over.  Measured: requests three or four
            // pages ahead make the step 3 - 11 % slower, and so does this loop written over an array of register sets
            // instead of the two named ones - keep it as it is.
            uint32_t kwa[4] = {0, 0, 0, 0}, vwa[4] = {0, 0, 0, 0}, kwb[4] = {0, 0, 0, 0}, vwb[4] = {0, 0, 0, 0};
            load_sf(0, kwa, vwa);
            load_sf(1, kwb, vwb);
            for (int i = 0; i < n_fp4 && ok; i += 2) {
                ok = fp4_step(i, kwa, vwa);
                if (!ok) break;
                load_sf(i + 2, kwa, vwa);
                if (i + 1 < n_fp4) {
                    ok = fp4_step(i + 1, kwb, vwb);
                    if (!ok) break;
                    load_sf(i + 3, kwb, vwb);
                }
            }
        }
        // ---- 16-bit pages: the ring is re-cut into 16 KB tiles once every FP4 slot has drained ----
        if (ok && n > n_fp4) {
            for (int sl = 0; sl < DEC_NS4 && ok; ++sl) {
                const int uses = (n_fp4 - sl + DEC_NS4 - 1) / DEC_NS4;   // FP4 pages that went through slot sl
                if (uses > 0) ok = waitc(1, &bars.f_empty[sl], (uses - 1) & 1);
            }
        }
        uint32_t t16 = 0;
        for (int i = n_fp4; i < n && ok; ++i) {
            const uint32_t key = list[i] & ~L_FP16;
            const int slab = paged ? static_cast<int>(key) : h;
            const int row0 = paged ? 0 : static_cast<int>(key) * PAGE;
            for (int which = 0; which < 2 && ok; ++which, ++t16) {   // K page, then V page
                const uint32_t slot = t16 % DEC_NS16;
                ok = waitc(2, &bars.h_empty[slot], ((t16 / DEC_NS16) & 1) ^ 1);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = smem_u32(which ? &bars.hv_full[slot] : &bars.hk_full[slot]);
                    const uint32_t sa = sbase + L::SLOTS + slot * DEC_SLOT16_BYTES;
                    mbar_expect_tx(bar, PAGE * D * 2);
                    for (int hf = 0; hf < D / 64; ++hf)
                        tma_load_3d(sa + hf * PAGE * 128, which ? &mapV16 : &mapK16, bar, hf * 64, row0, slab);
                }
            }
        }
    } else if (warp == 1) {
        // =========================== issuer of S = Q K^T ===========================
        // The whole warp runs this code with warp-uniform values; one elected lane issues each instruction.
        const uint32_t idesc_qk4 = make_idesc_fp4(128, PAGE, MX ? 1 : 0, 0, 0);
        const uint32_t idesc_qk16 = make_idesc_f16(128, PAGE, BF16 ? 1 : 0, 0, 0);
        bool ok = waitc(3, &bars.q_ready, 0) && waitc(4, &bars.list_full, 0);
        ok = __all_sync(0xFFFFFFFFu, ok);
        const int n = __shfl_sync(0xFFFFFFFFu, ok ? bars.n_total : 0, 0);
        const int n4 = __shfl_sync(0xFFFFFFFFu, ok ? bars.n_fp4 : 0, 0);
        const uint32_t tm = __shfl_sync(0xFFFFFFFFu, tmem, 0);
        tc_fence_after_sync();
        if (ok)
            for (int a = 0; a < QK_ATOMS; ++a)
                tmem_cp_sf_elect(tm + DTM_SFA_Q + a * 4, make_smem_desc(sbase + L::QSF + a * 512, 0, 128, SWZ_NONE));
        // ring position of step i: FP4 page -> slot i mod 5; 16-bit page -> tiles 2 (i - n4) (K) and + 1 (V)
        for (int i = 0; i < n && ok; ++i) {
            // operands of page i, and S of page i - 1 read by the softmax warps
            if (i < n4) {
                ok = waitc(5, &bars.f_full[i % DEC_NS4], (i / DEC_NS4) & 1);
            } else {
                const uint32_t j = i - n4, kt = 2u * j;
                ok = waitc(6, &bars.hk_full[kt % DEC_NS16], (j / DEC_NS16) & 1);
            }
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            // the K scale atoms go to tensor memory (two alternating buffers) before S of the previous page is free
            const uint32_t sfb = tm + ((i & 1) ? DTM_SFB_K2 : DTM_SFB_K);
            tc_fence_after_sync();
            if (i < n4) {
                const uint32_t sa = sbase + L::SLOTS + (i % DEC_NS4) * DEC_SLOT4_BYTES;
                for (int a = 0; a < QK_ATOMS; ++a)
                    tmem_cp_sf_elect(sfb + a * 4, make_smem_desc(sa + L::KSF + a * 512, 0, 128, SWZ_NONE));
            }
            if (i > 0) ok = waitc(7, &bars.s_free, (i - 1) & 1);
            ok = __all_sync(0xFFFFFFFFu, ok);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t d_t = tm + DTM_S;
            if (i < n4) {
                const uint32_t sa = sbase + L::SLOTS + (i % DEC_NS4) * DEC_SLOT4_BYTES;
                for (int kb = 0; kb < KBLK; ++kb) {
                    const uint64_t ad = make_smem_desc(sbase + L::Q4 + kb * 32, 16, SBO_QK, SWZ_QK);
                    const uint64_t bd = make_smem_desc(sa + L::K4 + kb * 32, 16, SBO_QK, SWZ_QK);
                    if constexpr (MX)
                        mma_mxfp4_elect(d_t, ad, bd, make_idesc_fp4(128, PAGE, 1, kb * 2, kb * 2), tm + DTM_SFA_Q, sfb, kb > 0);
                    else
                        mma_nvfp4_elect(d_t, ad, bd, idesc_qk4, tm + DTM_SFA_Q + kb * 4, sfb + kb * 4, kb > 0);
                }
            } else {
                const uint32_t kt = 2u * (i - n4);
                const uint32_t sa = sbase + L::SLOTS + (kt % DEC_NS16) * DEC_SLOT16_BYTES;
                for (int ks = 0; ks < D / 16; ++ks) {
                    const uint32_t hf = ks / 4, kk = ks % 4;
                    const uint64_t ad = make_smem_desc(sbase + L::Q16 + hf * 128 * 128 + kk * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = make_smem_desc(sa + hf * PAGE * 128 + kk * 32, 16, 1024, SWZ_128B);
                    mma_f16_elect(d_t, ad, bd, idesc_qk16, ks > 0);
                }
                tc_commit_elect(smem_u32(&bars.h_empty[kt % DEC_NS16]));   // the K page is free once S is computed
            }
            tc_commit_elect(smem_u32(&bars.s_full));
        }
    } else if (warp == 2) {
        // =========================== issuer of O += P V ===========================
        const uint32_t idesc_pv4 = make_idesc_fp4(128, D, MX ? 1 : 0, 0, 0);
        const uint32_t idesc_pv16 = make_idesc_f16(128, D, BF16 ? 1 : 0, 0, 1);
        bool ok = waitc(4, &bars.list_full, 0);
        const int n = ok ? bars.n_total : 0;
        const int n4 = ok ? bars.n_fp4 : 0;
        for (int i = 0; i < n && ok; ++i) {
            const bool fp16 = i >= n4;
            const uint32_t buf = i & 1;
            const uint32_t vt = 2u * (i - n4) + 1u;   // V tile of a 16-bit step
            ok = waitc(8, &bars.p_full[buf], (i >> 1) & 1);
            if (ok && fp16) ok = waitc(6, &bars.hv_full[vt % DEC_NS16], ((i - n4) / DEC_NS16) & 1);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint32_t d_t = tmem + DTM_O;
                const uint32_t acc = i > 0 ? 1u : 0u;
                if (!fp16) {
                    const uint32_t sa = sbase + L::SLOTS + (i % DEC_NS4) * DEC_SLOT4_BYTES;
                    const uint32_t sfa = tmem + DTM_SFA_P + buf * 4, sfb = tmem + DTM_SFB_V + buf * 4;
                    tmem_cp_sf(sfa, make_smem_desc(sbase + L::PSF + buf * 512, 0, 128, SWZ_NONE));
                    tmem_cp_sf(sfb, make_smem_desc(sa + L::VSF, 0, 128, SWZ_NONE));
                    const uint64_t ad = make_smem_desc(sbase + L::P + buf * 4096, 16, 256, SWZ_32B);
                    const uint64_t bd = make_smem_desc(sa + L::V4, 16, 256, SWZ_32B);
                    if constexpr (MX) mma_mxfp4(d_t, ad, bd, idesc_pv4, sfa, sfb, acc);
                    else mma_nvfp4(d_t, ad, bd, idesc_pv4, sfa, sfb, acc);
                    tc_commit(smem_u32(&bars.f_empty[i % DEC_NS4]));
                } else {
                    const uint32_t sa = sbase + L::SLOTS + (vt % DEC_NS16) * DEC_SLOT16_BYTES;
                    for (int ks = 0; ks < PAGE / 16; ++ks) {
                        const uint64_t ad = make_smem_desc(sbase + L::P + ks * 32, 16, 1024, SWZ_128B);
                        const uint64_t bd = make_smem_desc(sa + ks * 2048, PAGE * 128, 1024, SWZ_128B);
                        mma_f16(d_t, ad, bd, idesc_pv16, (acc == 0 && ks == 0) ? 0 : 1);
                    }
                    tc_commit(smem_u32(&bars.h_empty[vt % DEC_NS16]));
                }
                tc_commit(smem_u32(&bars.p_free[buf]));
            }
            __syncwarp();
        }
    } else {
        // =========================== softmax ===========================
        const int sub = warp & 3;                   // tensor-memory sub-partition of this warp
        const int row = sub * 32 + lane;            // tile row = tensor-memory lane = index among the 128 threads
        // Every query head occupies four rows of the tile, one per warp (rows g, 32 + g, 64 + g, 96 + g), and warp w
        // works on columns [16 w, 16 w + 16) of every head: the tensor-memory load of a warp takes one column address,
        // so a warp that needed all four quarters would load 64 columns per thread and keep 16.
        const int cq = sub;                         // column quarter handled by this warp
        const int g = lane;                         // query head of this row
        const bool active = g < G;
        const uint32_t lane_addr = static_cast<uint32_t>(sub * 32) << 16;
        const bool has_sel = p.width > 0;

        // ---- operand tiles written by hand: zero them, then place the query rows ----
        {
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
            for (int i = row; i < (L::Q16 - L::Q4) / 16; i += 128) reinterpret_cast<uint4*>(smem + L::Q4)[i] = z;
            if (has_sel)
                for (int i = row; i < 128 * D * 2 / 16; i += 128) reinterpret_cast<uint4*>(smem + L::Q16)[i] = z;
            for (int i = row; i < 16384 / 16; i += 128) reinterpret_cast<uint4*>(smem + L::P)[i] = z;
            for (int i = row; i < 1024 / 16; i += 128) reinterpret_cast<uint4*>(smem + L::PSF)[i] = z;
        }
        named_barrier_sync(1, 128);
        if (active) {
            const long long qrow = static_cast<long long>(h) * G + g;
            const uint4* q4row = reinterpret_cast<const uint4*>(p.q4 + qrow * (D / 2));
            if constexpr (D == 128) {
#pragma unroll
                for (int c = 0; c < 4; ++c)   // 64-byte row, 64-byte swizzle
                    *reinterpret_cast<uint4*>(smem + L::Q4 + row * 64 + ((c ^ ((row >> 1) & 3)) * 16)) = __ldg(q4row + c);
            } else {
#pragma unroll
                for (int c = 0; c < 2; ++c)   // 32-byte row, 32-byte swizzle
                    *reinterpret_cast<uint4*>(smem + L::Q4 + row * 32 + ((c ^ ((row >> 2) & 1)) * 16)) = __ldg(q4row + c);
            }
            const uint8_t* qsr = p.qs + qrow * (D / GRP);
#pragma unroll
            for (int a = 0; a < QK_ATOMS; ++a) {
                uint32_t word;
                if constexpr (D / GRP >= 4) word = __ldg(reinterpret_cast<const uint32_t*>(qsr) + a);
                else word = __ldg(reinterpret_cast<const uint16_t*>(qsr));
                reinterpret_cast<uint32_t*>(smem + L::QSF + a * 512)[lane * 4 + sub] = word;
            }
            if (has_sel) {
                const uint4* qh = reinterpret_cast<const uint4*>(p.q_hi + qrow * D);
#pragma unroll
                for (int hf = 0; hf < D / 64; ++hf)
#pragma unroll
                    for (int c = 0; c < 8; ++c)   // 128-byte row, 128-byte swizzle
                        *reinterpret_cast<uint4*>(smem + L::Q16 + hf * 128 * 128 + (row >> 3) * 1024 + (row & 7) * 128 +
                                                  ((c ^ (row & 7)) * 16)) = __ldg(qh + hf * 8 + c);
            }
        }
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&bars.q_ready));

        bool ok = waitc(21, &bars.list_full, 0);
        const int n = ok ? bars.n_total : 0;
        const int n4 = ok ? bars.n_fp4 : 0;

        float m_run = -FLT_MAX, l_run = 0.0f;
        bool prev_fp16 = false;
        for (int i = 0; i < n && ok; ++i) {
            const bool fp16 = i >= n4;
            ok = waitc(22, &bars.s_full, i & 1);
            if (!ok) break;
            tc_fence_after_sync();
            float s[16];
            {
                uint32_t r[16];
                tmem_ld16(tmem + lane_addr + DTM_S + 16 * cq, r);
                tmem_wait_ld();
#pragma unroll
                for (int j = 0; j < 16; ++j) s[j] = __uint_as_float(r[j]);
            }
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars.s_free));
            // running maximum of the whole page row: this quarter first
            // the P buffer of this step was last read by the PV of step i - 2: poll once now, look at the answer
            // only when the buffer is about to be written
            const uint32_t buf = i & 1;
            const uint32_t pf_parity = ((i >> 1) & 1) ^ 1;
            bool pf_ready = mbar_try_wait(smem_u32(&bars.p_free[buf]), pf_parity);
            float mx = fmaxf(max3(max3(s[0], s[1], s[2]), max3(s[3], s[4], s[5]), max3(s[6], s[7], s[8])),
                             max3(max3(s[9], s[10], s[11]), max3(s[12], s[13], s[14]), s[15]));
            // the other three quarters' maxima come from the other warps: published in shared memory, a barrier that
            // all 128 threads arrive at once per page (bounded wait, like every other), two buffers by page parity
            float mx_grp = mx;   // maximum of this thread's scale group: its 16 columns, 32 for MXFP4
            {
                float(*xq)[32] = bars.xch[i & 1];
                xq[cq][lane] = mx;
                mbar_arrive(smem_u32(&bars.x_full));
                ok = waitc(25, &bars.x_full, i & 1);
                if (!ok) break;
                if constexpr (MX) mx_grp = fmaxf(mx, xq[cq ^ 1][lane]);
                mx = fmaxf(max3(xq[0][lane], xq[1][lane], xq[2][lane]), xq[3][lane]);
            }
            const float m_new = fmaxf(m_run, mx);
            const bool changed = active && i > 0 && m_new > m_run;
            const float rescale = ex2((m_run - m_new) * p.c2);
            m_run = m_new;
            const bool need_rescale = __any_sync(0xFFFFFFFFu, changed);
            if ((need_rescale || fp16 || prev_fp16) && i > 0) {
                // O, or a P tile spanning both buffers, is about to be touched: both earlier PVs must be done
                if (!pf_ready) ok = waitc(23, &bars.p_free[buf], pf_parity);
                pf_ready = true;
                if (ok) ok = waitc(23, &bars.p_free[(i - 1) & 1], ((i - 1) >> 1) & 1);
                if (!ok) break;
                tc_fence_after_sync();
            }
            if (need_rescale) {
                const float f = changed ? rescale : 1.0f;
#pragma unroll 1
                for (int c = 0; c < D; c += 32) {
                    uint32_t r[32];
                    tmem_ld32(tmem + lane_addr + DTM_O + c, r);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * f);
                    tmem_st32(tmem + lane_addr + DTM_O + c, r);
                }
                tmem_wait_st();
            }
            if (!fp16) {
                // t = C p; group scale sf = amax(t) / 6 rounded to the scale format; codes = e2m1(t / sf), with
                // the un-rounded sf, as the reference computes them
                // amax(t) is t at the group's largest logit: the same operations on the same value
                const float amax = __fmul_rn(ex2(__fmul_rn(mx_grp - m_new, p.c2)), CSCALE);
                const float sfp = __fmul_rn(amax, 1.0f / 6.0f);
                const uint32_t sb = encode_scale<MX>(sfp);
                float inv = 0.0f;
                if (sfp > 1e-30f) asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(sfp));
                float t[16];
                {
                    const uint64_t mneg = pack2f(-m_new, -m_new), c2p = pack2f(p.c2, p.c2), cs = pack2f(CSCALE, CSCALE);
                    const uint64_t zero = pack2f(0.0f, 0.0f);
                    uint64_t acc0 = zero, acc1 = zero;
#pragma unroll
                    for (int j = 0; j < 16; j += 4) {
                        float a0, a1, b0, b1;
                        // (s - m) * c2 is exactly 0 at the row maximum, so p is exactly 1 there
                        unpack2f(mul2(add2(pack2f(s[j], s[j + 1]), mneg), c2p), a0, a1);
                        unpack2f(mul2(add2(pack2f(s[j + 2], s[j + 3]), mneg), c2p), b0, b1);
                        const uint64_t pa = pack2f(ex2(a0), ex2(a1)), pb = pack2f(ex2(b0), ex2(b1));
                        acc0 = add2(acc0, pa);
                        acc1 = add2(acc1, pb);
                        unpack2f(mul2(pa, cs), t[j], t[j + 1]);
                        unpack2f(mul2(pb, cs), t[j + 2], t[j + 3]);
                    }
                    float x, y;
                    unpack2f(add2(acc0, acc1), x, y);
                    l_run = fmaf(l_run, rescale, x + y);
                }
                uint32_t w0, w1;
                {
                    const uint64_t ip = pack2f(inv, inv);
                    float c[16];
#pragma unroll
                    for (int j = 0; j < 16; j += 2) unpack2f(mul2(pack2f(t[j], t[j + 1]), ip), c[j], c[j + 1]);
                    w0 = e2m1x8(c[0], c[1], c[2], c[3], c[4], c[5], c[6], c[7]);
                    w1 = e2m1x8(c[8], c[9], c[10], c[11], c[12], c[13], c[14], c[15]);
                }
                if (!pf_ready) {
                    ok = waitc(23, &bars.p_free[buf], pf_parity);
                    if (!ok) break;
                }
                if (active) {
                    // 128 rows x 32 bytes, 32-byte swizzle; this thread's 16 codes are bytes [8 cq, 8 cq + 8) of its row
                    uint8_t* dst = smem + L::P + buf * 4096 + (row >> 3) * 256 + (row & 7) * 32 +
                                   (((cq >> 1) ^ ((row >> 2) & 1)) * 16) + (cq & 1) * 8;
                    *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
                    const int sj = MX ? (cq >> 1) : cq;
                    reinterpret_cast<uint32_t*>(smem + L::PSF + buf * 512)[lane * 4 + sub] = sb << (8 * sj);
                }
            } else {
                float sum = 0.0f;
                uint32_t w[8];
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float a = ex2(fmaf(s[j] - m_new, p.c2, LOG2_C)), c = ex2(fmaf(s[j + 1] - m_new, p.c2, LOG2_C));
                    sum += a + c;
                    w[j >> 1] = In16<BF16>::pack2(a, c);
                }
                l_run = fmaf(l_run, rescale, sum * (1.0f / CSCALE));
                if (active) {
                    // 128 rows x 128 bytes, 128-byte swizzle; columns [16 cq, 16 cq + 16) are chunks 2 cq, 2 cq + 1
                    uint8_t* base = smem + L::P + (row >> 3) * 1024 + (row & 7) * 128;
                    if (!prev_fp16 && i > 0) {   // first 16-bit page: the row still holds FP4 codes
#pragma unroll
                        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(base + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                    *reinterpret_cast<uint4*>(base + (((2 * cq) ^ (row & 7)) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(base + (((2 * cq + 1) ^ (row & 7)) * 16)) = make_uint4(w[4], w[5], w[6], w[7]);
                }
            }
            fence_proxy_async_smem();
            tc_fence_before_sync();
            mbar_arrive(smem_u32(&bars.p_full[buf]));
            prev_fp16 = fp16;
        }

        // ---- end of chain: the four quarter rows of every head are added and written as one partial ----
        if (ok && n > 0) ok = waitc(23, &bars.p_free[(n - 1) & 1], ((n - 1) >> 1) & 1);
        if (ok) {
            tc_fence_after_sync();
            float* stage = reinterpret_cast<float*>(smem + L::SLOTS);   // [quarter][head][D]
#pragma unroll 1
            for (int c = 0; c < D; c += 32) {
                uint32_t r[32];
                tmem_ld32(tmem + lane_addr + DTM_O + c, r);
                tmem_wait_ld();
                if (active) {
                    uint4* dst = reinterpret_cast<uint4*>(stage + (cq * DEC_MAX_GROUP + g) * D + c);
#pragma unroll
                    for (int j = 0; j < 8; ++j) dst[j] = make_uint4(r[4 * j], r[4 * j + 1], r[4 * j + 2], r[4 * j + 3]);
                }
            }
            tc_fence_before_sync();
            if (active) {
                bars.l_part[cq][g] = l_run;
                if (cq == 0) bars.m_row[g] = m_run * p.sm_scale;
            }
            mbar_arrive(smem_u32(&bars.epi_full));
            ok = waitc(24, &bars.epi_full, 0);
        }
        if (ok) {
            const float* stage = reinterpret_cast<const float*>(smem + L::SLOTS);
            const long long pbase = (static_cast<long long>(h) * p.splits + split) * G;
            for (int gg = 0; gg < G && row < D; ++gg) {
                float o = stage[(0 * DEC_MAX_GROUP + gg) * D + row];
                o += stage[(1 * DEC_MAX_GROUP + gg) * D + row];
                o += stage[(2 * DEC_MAX_GROUP + gg) * D + row];
                o += stage[(3 * DEC_MAX_GROUP + gg) * D + row];
                p.part_o[(pbase + gg) * D + row] = o;
            }
            if (row < G) {
                p.part_ml[(pbase + row) * 2] = bars.m_row[row];
                p.part_ml[(pbase + row) * 2 + 1] = (bars.l_part[0][row] + bars.l_part[1][row]) + (bars.l_part[2][row] + bars.l_part[3][row]);
            }
        }
    }

    // ---- common exit ----
    if (bars.abort_flag != 0) {
        // copies and MMAs already issued must finish before shared and tensor memory are given back
        for (int i = 0; i < 25; ++i) __nanosleep(20000);
    }
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, DTM_COLS);
    if (bars.abort_flag != 0) {
        // a chain that gave up contributes nothing: neutral partials (row max -FLT_MAX, row sum 0) instead of
        // whatever the scratch memory held
        const long long pbase = (static_cast<long long>(h) * p.splits + split) * G;
        for (int i = tid; i < G * D; i += DEC_THREADS) p.part_o[pbase * D + i] = 0.0f;
        for (int i = tid; i < G; i += DEC_THREADS) { p.part_ml[(pbase + i) * 2] = -FLT_MAX; p.part_ml[(pbase + i) * 2 + 1] = 0.0f; }
    }
    if (tid == 0 && bars.abort_flag != 0) atomicCAS(&g_decode_status, 0, bars.abort_code != 0 ? bars.abort_code : 99);
    if (tid == 0 && bars.bad_entry != 0) atomicCAS(&g_decode_status, 0, STATUS_BAD_PAGE);
}

// out[row, :] = sum_s O_s e^{m_s - M} / (C sum_s l_s e^{m_s - M}); rows = heads * G
template <bool BF16>
__global__ void __launch_bounds__(128) merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                                    uint16_t* __restrict__ out, int shards, long long shard_stride_o,
                                                    long long shard_stride_ml, int splits, int G, int d, long long rows,
                                                    float c_scale) {
    // part_o is addressed as [shard][head][split][g][d]; one CTA per output row
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long head = row / G;
        const int g = static_cast<int>(row - head * G);
        float M = -FLT_MAX;
        for (int sh = 0; sh < shards; ++sh)
            for (int s = 0; s < splits; ++s)
                M = fmaxf(M, part_ml[sh * shard_stride_ml + ((head * splits + s) * G + g) * 2]);
        float den = 0.0f;
        float acc = 0.0f;
        for (int sh = 0; sh < shards; ++sh)
            for (int s = 0; s < splits; ++s) {
                const long long i = (head * splits + s) * G + g;
                const float w = __expf(part_ml[sh * shard_stride_ml + i * 2] - M);
                den = fmaf(part_ml[sh * shard_stride_ml + i * 2 + 1], w, den);
                if (threadIdx.x < d) acc = fmaf(part_o[sh * shard_stride_o + i * d + threadIdx.x], w, acc);
            }
        const float norm = den > 0.0f ? __fdiv_rn(1.0f, c_scale * den) : 0.0f;
        if (threadIdx.x < d) out[row * d + threadIdx.x] = In16<BF16>::from_f(acc * norm);
    }
}

// The same merge, but the result stays a partial: (sum_s O_s e^{m_s - M}, M, sum_s l_s e^{m_s - M}) as one split
// per head.  A rank of a KV-sequence-sharded step reduces its own chains with this before the exchange, so that
// what crosses NVLink does not grow with the number of chains.
__global__ void __launch_bounds__(128) reduce_partials_kernel(const float* __restrict__ part_o,
                                                              const float* __restrict__ part_ml,
                                                              float* __restrict__ out_o, float* __restrict__ out_ml,
                                                              int splits, int G, int d, long long rows) {
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const long long head = row / G;
        const int g = static_cast<int>(row - head * G);
        float M = -FLT_MAX;
        for (int s = 0; s < splits; ++s) M = fmaxf(M, part_ml[((head * splits + s) * G + g) * 2]);
        float den = 0.0f, acc = 0.0f;
        for (int s = 0; s < splits; ++s) {
            const long long i = (head * splits + s) * G + g;
            const float w = __expf(part_ml[i * 2] - M);
            den = fmaf(part_ml[i * 2 + 1], w, den);
            if (threadIdx.x < d) acc = fmaf(part_o[i * d + threadIdx.x], w, acc);
        }
        if (threadIdx.x < d) out_o[row * d + threadIdx.x] = acc;
        if (threadIdx.x == 0) { out_ml[row * 2] = M; out_ml[row * 2 + 1] = den; }
    }
}

}  // namespace

// Chains per (sequence, KV head).  A chain costs a fixed set-up (tensor-memory allocation, zeroed operand tiles,
// page list, filling and draining the page ring: measured as about the time of 15 pages) plus its pages, and the CTAs
// run in waves of two per SM; the count that minimises waves x (set-up + pages per chain) wins, the smaller count on
// a tie.  With many heads and short sequences that is ONE chain per head (256 heads x 256 pages: 209 us against 251
// with eight chains), with few heads it is as many chains as fill the GPU once.
int decode_pick_splits(int heads, int npages) {
    int sms = NUM_SMS_HINT;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (heads < 1) heads = 1;
    const long long resident = 2LL * sms;
    constexpr int SETUP_PAGES = 15;
    int lo = cdiv(npages, DEC_LIST_CAP);
    if (lo < 1) lo = 1;
    int hi = npages < 64 ? npages : 64;
    if (hi < lo) hi = lo;
    int best = lo;
    long long best_cost = -1;
    for (int s = lo; s <= hi; ++s) {
        const long long ctas = static_cast<long long>(heads) * s;
        const long long waves = (ctas + resident - 1) / resident;
        const long long cost = waves * (SETUP_PAGES + cdiv(npages, s));
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = s; }
        if (npages / s < 8) break;   // chains shorter than 8 pages are mostly set-up
    }
    return best;
}


size_t decode_workspace_bytes(int heads, int G, int d, int splits) {
    return static_cast<size_t>(heads) * splits * G * (d + 2) * sizeof(float);
}

// Reads and clears the device status word: TA100_ERR_DEVICE_TIMEOUT if a bounded wait inside a decode
// kernel of the current device ran out since the last call.  Synchronises with `stream`.
int decode_status(cudaStream_t stream) {
    cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    int flag = 0;
    e = cudaMemcpyFromSymbol(&flag, g_decode_status, sizeof(int));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (flag != 0) {
        const int zero = 0;
        cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
        if (flag == STATUS_BAD_PAGE) return TA100_ERR_PAGE_TABLE;
        fprintf(stderr, "libthrift_sm100: a decode kernel gave up waiting (wait site %d)\n", flag);
        return TA100_ERR_DEVICE_TIMEOUT;
    }
    return TA100_OK;
}

// See include/thrift_sm100.h (ta100_decode_attention).
int decode_dispatch(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, const void* q4,
                    const void* k4, const void* v4, const void* qs, const void* ks, const void* vs, const void* page_table,
                    int max_pages, int pool_pages, void* out, void* part_o, void* part_ml, int batch, int hkv, int G, int kv_len,
                    int kv_cap, int d, int is_mx, int is_bf16, int splits, int write_out, const void* len_dev, int len_per_seq,
                    int len_offset, cudaStream_t stream) {
    if (!q4 || !k4 || !v4 || !qs || !ks || !vs || !part_o || !part_ml) return TA100_ERR_NULL;
    if (write_out && !out) return TA100_ERR_NULL;
    if (width > 0 && (!q_hi || !k_hi || !v_hi || !sel)) return TA100_ERR_NULL;
    if (d != 128 && d != 64) return TA100_ERR_UNSUPPORTED;
    if (G < 1 || G > DEC_MAX_GROUP) return TA100_ERR_UNSUPPORTED;
    if (batch <= 0 || hkv <= 0 || kv_len <= 0 || kv_len % PAGE != 0 || kv_cap < kv_len) return TA100_ERR_SHAPE;
    if (!page_table && kv_cap % PAGE != 0) return TA100_ERR_SHAPE;
    const int heads = batch * hkv;
    const int npages = kv_len / PAGE;
    if (npages > 2048 || heads > 65535) return TA100_ERR_LIMIT;
    if (splits < 1 || splits > npages) return TA100_ERR_SHAPE;
    if (cdiv(npages, splits) > DEC_LIST_CAP) return TA100_ERR_LIMIT;
    const uintptr_t align = reinterpret_cast<uintptr_t>(k4) | reinterpret_cast<uintptr_t>(v4) |
                            reinterpret_cast<uintptr_t>(k_hi) | reinterpret_cast<uintptr_t>(v_hi) |
                            reinterpret_cast<uintptr_t>(q4) | reinterpret_cast<uintptr_t>(q_hi);
    if (align & 15) return TA100_ERR_ALIGN;
    if ((reinterpret_cast<uintptr_t>(ks) | reinterpret_cast<uintptr_t>(vs) | reinterpret_cast<uintptr_t>(qs)) & 3)
        return TA100_ERR_ALIGN;
    const int GRP = is_mx ? 32 : 16;
    const int P = cdiv(kv_cap, 128) * 128;
    const bool paged = page_table != nullptr;
    // a pool holds pool_pages x hkv slabs of one page each; the tensor maps end there and the kernel skips
    // page-table entries that point beyond it
    if (paged && (pool_pages <= 0 || max_pages < npages || static_cast<long long>(pool_pages) * hkv >= 0x7FFFFFFFll))
        return TA100_ERR_SHAPE;
    const uint64_t pool_slabs = paged ? static_cast<uint64_t>(pool_pages) * hkv : 1;

    CUtensorMap maps[4];
    memset(maps, 0, sizeof(maps));
    {
        int rc = 0;
        const uint64_t d2 = static_cast<uint64_t>(d / 2);
        {   // K codes: rows of d/2 bytes
            uint64_t dims[3] = {d2, paged ? uint64_t(PAGE) : uint64_t(kv_cap), paged ? pool_slabs : uint64_t(heads)};
            uint64_t str[2] = {d2, (paged ? uint64_t(PAGE) : uint64_t(kv_cap)) * d2};
            uint32_t box[3] = {static_cast<uint32_t>(d2), PAGE, 1};
            rc |= make_tensor_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, k4, dims, str, box,
                                  d == 128 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B);
        }
        {   // V codes, transposed: d rows of (tokens / 2) bytes
            const uint64_t rowb = paged ? uint64_t(PAGE / 2) : uint64_t(P / 2);
            uint64_t dims[3] = {rowb, uint64_t(d), paged ? pool_slabs : uint64_t(heads)};
            uint64_t str[2] = {rowb, rowb * d};
            uint32_t box[3] = {PAGE / 2, static_cast<uint32_t>(d), 1};
            rc |= make_tensor_map(&maps[1], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, v4, dims, str, box, CU_TENSOR_MAP_SWIZZLE_32B);
        }
        if (width > 0) {
            const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
            const uint64_t rows = paged ? uint64_t(PAGE) : uint64_t(kv_cap);
            uint64_t dims[3] = {uint64_t(d), rows, paged ? pool_slabs : uint64_t(heads)};
            uint64_t str[2] = {uint64_t(d) * 2, rows * d * 2};
            uint32_t box[3] = {64, PAGE, 1};
            rc |= make_tensor_map(&maps[2], dt, 3, k_hi, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
            rc |= make_tensor_map(&maps[3], dt, 3, v_hi, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
        } else {
            maps[2] = maps[0]; maps[3] = maps[0];
        }
        if (rc != 0) return TA100_ERR_TENSOR_MAP;
    }

    DecodeParams p;
    p.q_hi = static_cast<const uint16_t*>(q_hi); p.q4 = static_cast<const uint8_t*>(q4); p.qs = static_cast<const uint8_t*>(qs);
    p.ks = static_cast<const uint8_t*>(ks); p.vs = static_cast<const uint8_t*>(vs);
    p.sel = static_cast<const int32_t*>(sel); p.page_table = static_cast<const int32_t*>(page_table);
    p.part_o = static_cast<float*>(part_o); p.part_ml = static_cast<float*>(part_ml);
    p.len_dev = static_cast<const int32_t*>(len_dev); p.len_per_seq = len_per_seq ? 1 : 0; p.len_offset = len_offset;
    p.heads = heads; p.hkv = hkv; p.G = G; p.npages = npages; p.cap_pages = kv_cap / PAGE; p.max_pages = max_pages; p.pool_pages = pool_pages;
    p.width = width; p.splits = splits;
    p.vs_row_stride = P / GRP;
    p.sm_scale = static_cast<float>(1.0 / sqrt(static_cast<double>(d)));
    p.c2 = static_cast<float>((1.0 / sqrt(static_cast<double>(d))) * 1.4426950408889634);
    p.budget = g_wait_budget_cycles;
    p.skip_loads = g_test_skip_loads;
    const dim3 grid(splits, heads);
#define TA100_DEC(DD, MXX, BFF)                                                                               \
    do {                                                                                                      \
        const int smem = DecSmem<DD>::TOTAL;                                                                  \
        cudaFuncSetAttribute(decode_kernel<DD, MXX, BFF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        cudaFuncSetAttribute(decode_kernel<DD, MXX, BFF>, cudaFuncAttributePreferredSharedMemoryCarveout, 100); \
        decode_kernel<DD, MXX, BFF><<<grid, DEC_THREADS, smem, stream>>>(p, maps[0], maps[1], maps[2], maps[3]); \
    } while (0)
    if (d == 128) {
        if (is_mx) { if (is_bf16) TA100_DEC(128, true, true); else TA100_DEC(128, true, false); }
        else { if (is_bf16) TA100_DEC(128, false, true); else TA100_DEC(128, false, false); }
    } else {
        if (is_mx) { if (is_bf16) TA100_DEC(64, true, true); else TA100_DEC(64, true, false); }
        else { if (is_bf16) TA100_DEC(64, false, true); else TA100_DEC(64, false, false); }
    }
#undef TA100_DEC
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
    if (write_out) {
        const long long rows = static_cast<long long>(heads) * G;
        const int mgrid = static_cast<int>(rows < NUM_SMS_HINT * 8LL ? rows : NUM_SMS_HINT * 8LL);
        const float c = is_mx ? 6.0f : 2688.0f;
        if (is_bf16)
            merge_kernel<true><<<mgrid, 128, 0, stream>>>(p.part_o, p.part_ml, static_cast<uint16_t*>(out), 1, 0, 0, splits, G, d, rows, c);
        else
            merge_kernel<false><<<mgrid, 128, 0, stream>>>(p.part_o, p.part_ml, static_cast<uint16_t*>(out), 1, 0, 0, splits, G, d, rows, c);
        e = cudaGetLastError();
    }
    return static_cast<int>(e);
}

// Merge partials of `shards` ranks laid out as [shard][heads][splits][G][d] / [..][2].
// shard_stride_* = elements between consecutive shards (0: densely packed).
int merge_dispatch(const void* part_o, const void* part_ml, void* out, int shards, long long shard_stride_o,
                   long long shard_stride_ml, long long heads, int splits, int G, int d, int is_mx, int is_bf16,
                   cudaStream_t stream) {
    if (!part_o || !part_ml || !out) return TA100_ERR_NULL;
    if (d > 128 || shards < 1 || splits < 1) return TA100_ERR_SHAPE;
    const long long rows = heads * G;
    if (rows == 0) return TA100_OK;
    const long long dense_o = heads * splits * G * d, dense_ml = heads * splits * G * 2;
    if ((shard_stride_o != 0 && shard_stride_o < dense_o) || (shard_stride_ml != 0 && shard_stride_ml < dense_ml))
        return TA100_ERR_SHAPE;
    const long long so = shard_stride_o ? shard_stride_o : dense_o, sml = shard_stride_ml ? shard_stride_ml : dense_ml;
    const int mgrid = static_cast<int>(rows < NUM_SMS_HINT * 8LL ? rows : NUM_SMS_HINT * 8LL);
    const float c = is_mx ? 6.0f : 2688.0f;
    if (is_bf16)
        merge_kernel<true><<<mgrid, 128, 0, stream>>>(static_cast<const float*>(part_o), static_cast<const float*>(part_ml),
                                                      static_cast<uint16_t*>(out), shards, so, sml, splits, G, d, rows, c);
    else
        merge_kernel<false><<<mgrid, 128, 0, stream>>>(static_cast<const float*>(part_o), static_cast<const float*>(part_ml),
                                                       static_cast<uint16_t*>(out), shards, so, sml, splits, G, d, rows, c);
    return static_cast<int>(cudaGetLastError());
}

// Reduce the chains of every head to one partial per head: part_o [heads][splits][G][d] -> out_o [heads][1][G][d].
int reduce_partials_dispatch(const void* part_o, const void* part_ml, void* out_o, void* out_ml, long long heads,
                             int splits, int G, int d, cudaStream_t stream) {
    if (!part_o || !part_ml || !out_o || !out_ml) return TA100_ERR_NULL;
    if (d > 128 || d < 1 || splits < 1 || G < 1 || heads < 0) return TA100_ERR_SHAPE;
    const long long rows = heads * G;
    if (rows == 0) return TA100_OK;
    const int grid = static_cast<int>(rows < NUM_SMS_HINT * 8LL ? rows : NUM_SMS_HINT * 8LL);
    reduce_partials_kernel<<<grid, 128, 0, stream>>>(static_cast<const float*>(part_o), static_cast<const float*>(part_ml),
                                                     static_cast<float*>(out_o), static_cast<float*>(out_ml), splits, G, d,
                                                     rows);
    return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Allocation-free decode entry
// ---------------------------------------------------------------------------
// Some hosts cannot give this library device memory at call time: a serving
// process that has handed every free byte of HBM to its own pool at start-up
// (so a later cudaMalloc fails), or a latency-critical decode loop in which the
// implicit device-wide synchronisation of cudaMalloc / cudaFree is not
// acceptable.  For them the split-KV partials live in this fixed array, which
// every GPU that loads the library holds from load until process exit.
constexpr size_t STATIC_SCRATCH_BYTES = size_t(16) << 20;  // 16 MiB
static __device__ __align__(256) unsigned char g_decode_static_scratch[STATIC_SCRATCH_BYTES];

namespace {
constexpr int MAX_DEVICES = 64;
void* g_static_scratch_ptr[MAX_DEVICES] = {};
std::mutex g_static_scratch_mutex;

// The array's name is only a host-side handle: the device address has to be
// looked up, once per device, while that device is current.
int static_scratch_address(void** out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= MAX_DEVICES) return TA100_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_decode_static_scratch);
        if (e != cudaSuccess) return static_cast<int>(e);
        g_static_scratch_ptr[dev] = p;
    }
    *out = g_static_scratch_ptr[dev];
    return TA100_OK;
}
}  // namespace

size_t decode_static_scratch_bytes() { return STATIC_SCRATCH_BYTES; }

// Same computation as decode_dispatch with write_out = 1, but the partials go to
// the library's fixed scratch array instead of caller memory.  Nothing is
// allocated or freed here.  The scratch is shared by every call on the device
// and keeps the previous call's contents; each call overwrites every entry it
// later reads, so nothing needs clearing, but two calls that overlap on the GPU
// (different streams) would race on it.
int decode_static_dispatch(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, const void* q4,
                           const void* k4, const void* v4, const void* qs, const void* ks, const void* vs,
                           const void* page_table, int max_pages, int pool_pages, void* out, int batch, int hkv, int G,
                           int kv_len, int kv_cap, int d, int is_mx, int is_bf16, int splits, cudaStream_t stream) {
    if (batch <= 0 || hkv <= 0 || G <= 0 || splits <= 0 || d <= 0) return TA100_ERR_SHAPE;
    // bound every factor before multiplying them
    if (G > DEC_MAX_GROUP || d > 128 || splits > 4096 || static_cast<long long>(batch) * hkv > 65535) return TA100_ERR_STATIC_SCRATCH;
    const size_t n_o = static_cast<size_t>(batch) * hkv * splits * G * d * sizeof(float);
    const size_t n_ml = static_cast<size_t>(batch) * hkv * splits * G * 2 * sizeof(float);
    const size_t off_ml = (n_o + 255) & ~static_cast<size_t>(255);
    if (off_ml + n_ml > STATIC_SCRATCH_BYTES) return TA100_ERR_STATIC_SCRATCH;
    void* base = nullptr;
    const int rc = static_scratch_address(&base);
    if (rc != TA100_OK) return rc;
    unsigned char* b = static_cast<unsigned char*>(base);
    return decode_dispatch(q_hi, k_hi, v_hi, sel, width, q4, k4, v4, qs, ks, vs, page_table, max_pages, pool_pages, out, b, b + off_ml,
                           batch, hkv, G, kv_len, kv_cap, d, is_mx, is_bf16, splits, 1, nullptr, 0, 0, stream);
}

}  // namespace ta100
