// Fused selective mixed-precision prefill attention for sm_100a.
//
// One persistent CTA per SM walks (q head, 128-row q tile) work items, longest
// first.  Per item the KV sequence is consumed in 64-column sub-steps:
//   phase A  every sub-step whose KV block is NOT selected: block-scaled FP4
//            tcgen05 MMAs (S = Q4 K4^T, O += P4 V4) with P quantised to e2m1;
//   phase B  the selected blocks in list order: f16/bf16 tcgen05 MMAs.
// Both phases share one online softmax whose accumulator O lives in tensor memory
// for the whole item.
//
// What bounds this kernel is neither the tensor pipe (a sub-step's FP4 MMAs take ~130
// cycles) nor the special-function unit (one ex2 per score, 512 cycles per sub-step
// at 16 per cycle and SM; measured: removing every ex2 changes nothing) but the time
// one sub-step takes to pass through a softmax warp: that warp spends more time
// waiting - for S to land in tensor memory, for the previous P V to finish, for its
// own dependent instructions - than it spends computing.  So the sub-steps of an
// item are dealt round robin to FOUR sets of softmax warps: sub-step n of the CTA
// belongs to set n mod 4, has its own S buffer in tensor memory (4 x 64 columns)
// and its own P tile in shared memory, and each scheduler of the SM holds four
// softmax warps that are in four different sub-steps.  What ties consecutive
// sub-steps together is small and is handed from set to set through shared memory:
//   * the running row maximum (a chain of 32-arrival mbarriers per 32-row group);
//   * the rescale of O when a maximum moved: set n does it after P V of sub-step
//     n-1 completed and before it releases its own P tile, so the order in which
//     the reference updates its state is kept exactly;
//   * the row sum, which every set keeps for its own sub-steps (relative to the
//     maximum it saw last) and which is added up once per item.
//
// Warp roles (640 threads): warp 0 = producer (bulk copies of the packed K/V records, TMA for
// Q and the 16-bit tiles; it also builds the item's sub-step list in shared memory), warps 1
// and 2 = issuers of the S = Q K^T MMAs (even and odd sub-steps; warp 1 owns tensor memory),
// warp 3 = issuer of the O += P V MMAs, warps 4..19 = softmax (one thread per q row; warp w
// owns tensor-memory lanes 32*(w%4)..+31 and belongs to set (w-4)/4).
//
// Every mbarrier wait is bounded; a timeout raises a CTA-wide abort flag, all
// roles drain, tensor memory is released and a status word is set.  A parity
// wait is only sound for a waiter that sees every phase of its barrier, so every
// waiter here waits on each phase of the barriers it uses, also where the value
// behind the barrier is not needed - or, where noted, asks only about a phase that
// it knows to be the barrier's current or previous one.
#include <cfloat>
#include <climits>
#include <type_traits>

#include "common.cuh"
#include "sm100_ptx.cuh"

namespace ta100 {

namespace {


constexpr int QTILE = 128;
constexpr int STEP = 64;
constexpr int NSETS = 4;             // softmax warp sets = S buffers = P tiles
constexpr int NSLOTS = 6;            // K/V ring slots
constexpr int SLOT_BYTES = 16384;    // one FP4 sub-step (K4, V4, scale atoms) or one 16-bit K or V tile
constexpr int REC_BYTES = 9728;      // packed FP4 record of one (KV head, sub-step): K4 4096 | K scale atoms 1024 | V4 4096 | V scale atom 512
constexpr int PSET_BYTES = 16384;    // P tile of a set: 4 KB of e2m1 or 16 KB of 16-bit values
constexpr int NUM_THREADS = 32 * (4 + 4 * NSETS);   // 640 = 20 warps: 96 registers per thread
constexpr int SCHED_CAP = 2944;      // sub-step list entries per work item

// tensor-memory columns (all 512 of the SM)
constexpr uint32_t TM_O = 0;         // 128 columns
constexpr uint32_t TM_S = 128;       // NSETS buffers of 64 columns
constexpr uint32_t TM_SFA_Q = 384;   // up to 8 columns (issuer 0's copy; issuer 1's is TM_SFA_Q1)
constexpr uint32_t TM_SFA_Q1 = 448;
constexpr uint32_t TM_SFA_P = 392;   // 4 columns, constant
constexpr uint32_t TM_SFB_K = 400;   // NSETS buffers of 8 columns
constexpr uint32_t TM_SFB_V = 432;   // NSETS buffers of 4 columns
constexpr uint32_t TM_COLS = 512;

// sub-step list entry: bits 0..11 sub-step index, 12 = 16-bit, 13 / 14 = rows 0..63 / 64..127 take part
constexpr uint32_t E_FP16 = 1u << 12, E_P0 = 1u << 13, E_P1 = 1u << 14;

struct PrefillParams {
    int batch, hq_per_b, hkv_per_b, group;
    int sq, skv;
    int block;      // selection block size in tokens (64 or 128)
    int width;      // entries per selection row (0: pure FP4)
    int causal, round_partial;
    int out_seq_major;   // 0: out [B, Hq, Sq, D]; 1: out [B, Sq, Hq, D]
    int n_qtiles, n_items, nsteps_total, nkb;
    const int32_t* sel;
    const uint8_t* q_sf;
    const uint8_t* kv_rec;   // packed K/V records, one per (KV head, sub-step)
    uint16_t* out;
    int* status;
    float c2;  // (1/sqrt(d)) * log2(e)
    long long budget;
    int skip_loads;  // diagnostics: the producer issues no copies
};

// shared-memory carve-up (offsets from a 1024-byte aligned base)
template <int D>
struct Smem {
    static constexpr int Q4 = 0;                       // 128 x D/2
    static constexpr int QSF = Q4 + QTILE * D / 2;     // up to 2 atoms
    static constexpr int Q16 = QSF + 1024;             // 128 x D x 2
    static constexpr int P = Q16 + QTILE * D * 2;      // NSETS tiles
    static constexpr int SLOTS = P + NSETS * PSET_BYTES;
    static constexpr int CSF = SLOTS + NSLOTS * SLOT_BYTES;    // constant scale atom (512 B)
    static constexpr int BITS = CSF + 512;                     // 2 halves x 64 words
    static constexpr int BARS = BITS + 2 * 64 * 4;             // mbarriers and CTA-wide flags (1 KB)
    static constexpr int XCH = BARS + 1024;                    // row maxima and row sums handed between sets
    static constexpr int SCHED = XCH + sizeof(float) * 4 * NSETS * 32 * 5;   // SCHED_CAP x u16
    static constexpr int TOTAL = SCHED + SCHED_CAP * 2;
    // inside an FP4 slot
    static constexpr int K4 = 0, KSF = 4096, V4 = 5120, VSF = 9216;   // the record's layout: K4, K scale atoms, V4, V scale atom
    static_assert(Q16 % 1024 == 0 && P % 1024 == 0 && SLOTS % 1024 == 0, "swizzled tiles need 1024-byte alignment");
    static_assert(TOTAL <= 227 * 1024, "one CTA must fit the SM's shared memory");
};

struct Bars {
    uint64_t q_full, q_empty;
    uint64_t sched_full, sched_empty;
    uint64_t o_full;                                   // last P V of the item complete
    uint64_t k_full[NSLOTS], v_full[NSLOTS], slot_empty[NSLOTS];   // K part / V part of a slot landed; slot released
    uint64_t s_full[NSETS], s_free[NSETS];
    uint64_t p_full[NSETS][2], p_free[NSETS][2];       // P tile in buffer (use & 1) written; the P V that read it complete
    uint64_t mch[4][NSETS];                            // row maxima of (row group, set) published
    uint64_t trans[4];                                 // row sums of a row group published for the state rounding
    uint64_t lend[4];                                  // ... and for the end of the item
    int sched_n, sched_na;                             // entries; entries before the first 16-bit one
    uint32_t slot_last[NSLOTS];                        // producer's note of who used a slot last
    uint32_t tmem_base;
    int abort_flag;
};
static_assert(sizeof(Bars) <= 1024, "barrier block must fit its shared-memory slot");

// what the sets of one 32-row group hand to each other: [row group][set][lane]
struct Xch {
    float mrun[4][NSETS][32];       // running maximum after the set's latest sub-step
    float l_end[4][NSETS][32];      // row sum and its reference maximum at the end of the item
    float m_end[4][NSETS][32];
    float l_tr[4][NSETS][32];       // the same at the hand-over from the FP4 to the 16-bit phase
    float m_tr[4][NSETS][32];
};

struct ItemInfo {
    int h, t, kvh;
};

// Work items in launch order: all items of one KV head (its query heads x all q tiles, longest = latest tiles
// first) before the next KV head's.  The CTAs that run at the same time then read the K/V of one or two KV heads
// only, which stay in L2 while every q tile of those heads streams over them.
__device__ __forceinline__ ItemInfo decode_item(const PrefillParams& p, int item) {
    const int per_kv = p.n_qtiles * p.group;
    ItemInfo it;
    it.kvh = item / per_kv;                       // flat (batch, KV head)
    const int rem = item - it.kvh * per_kv;
    it.t = p.n_qtiles - 1 - rem / p.group;
    const int b = it.kvh / p.hkv_per_b;
    it.h = b * p.hq_per_b + (it.kvh - b * p.hkv_per_b) * p.group + rem % p.group;
    return it;
}

__device__ __forceinline__ bool bit_of(const uint32_t* b, int i) { return (b[i >> 5] >> (i & 31)) & 1u; }

// Builds the sub-step list of one work item (whole warp).  Order: every sub-step whose
// block is not selected, ascending; then the selected blocks of the first
// 64-row half in list order; then those of the second half that were not
// already visited.  Returns the number of entries, or -1 if the list overflows;
// n_fp4 receives the number of entries of the first kind.
__device__ __noinline__ int build_schedule(const PrefillParams& p, const ItemInfo& it, uint32_t* bits, uint16_t* sched, int lane,
                              int& n_fp4) {
    const int nqb = p.sq / p.block;
    const int row0 = it.t * QTILE;
    const int qb0 = row0 / p.block;
    const int qb1 = min((row0 + 64) / p.block, nqb - 1);
    const bool two = qb1 != qb0;
    const bool has_sel = p.width > 0;
    const int spb_shift = (p.block == 128) ? 1 : 0, spb = 1 << spb_shift;
    const int32_t* list0 = has_sel ? p.sel + (static_cast<long long>(it.h) * nqb + qb0) * p.width : nullptr;
    const int32_t* list1 = has_sel ? p.sel + (static_cast<long long>(it.h) * nqb + qb1) * p.width : nullptr;
    uint32_t* bits0 = bits;
    uint32_t* bits1 = two ? bits + 64 : bits;
    int last0, last1, nsteps;
    if (p.causal) {
        last0 = row0 + 63; last1 = row0 + 127;
        nsteps = min(p.nsteps_total, last1 / STEP + 1);
    } else {
        last0 = INT_MAX; last1 = INT_MAX;
        nsteps = p.nsteps_total;
    }
    // ---- bitsets of the selected blocks ----
    for (int i = lane; i < 128; i += 32) bits[i] = 0u;
    __syncwarp();
    if (has_sel) {
        for (int half = 0; half < (two ? 2 : 1); ++half) {
            const int32_t* list = half ? list1 : list0;
            for (int i = lane; i < p.width; i += 32) {
                const int id = list[i];
                if (id >= 0 && id < p.nkb) atomicOr(&bits[half * 64 + (id >> 5)], 1u << (id & 31));
            }
        }
    }
    __syncwarp();
    const uint32_t lt = (1u << lane) - 1u;
    int n = 0;
    // ---- phase A ----
    for (int base = 0; base < nsteps; base += 32) {
        const int st = base + lane;
        bool p0 = false, p1 = false;
        if (st < nsteps) {
            const int blk = st >> spb_shift;
            p0 = (st * STEP <= last0) && !(has_sel && bit_of(bits0, blk));
            p1 = (st * STEP <= last1) && !(has_sel && bit_of(bits1, blk));
        }
        const bool keep = p0 | p1;
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, keep);
        const int pos = n + __popc(m & lt);
        if (keep && pos < SCHED_CAP) sched[pos] = static_cast<uint16_t>(st | (p0 ? E_P0 : 0) | (p1 ? E_P1 : 0));
        n += __popc(m);
    }
    n_fp4 = n;
    // ---- phase B ----
    if (has_sel) {
        for (int pass = 0; pass < (two ? 2 : 1); ++pass) {
            const int32_t* list = pass ? list1 : list0;
            for (int base = 0; base < p.width; base += 32) {
                const int i = base + lane;
                const int id = i < p.width ? list[i] : -1;
                bool ok = id >= 0 && id < p.nkb;
                if (ok && pass == 1 && bit_of(bits0, id)) ok = false;  // already visited with the first half's list
                uint32_t e[2] = {0, 0};
                bool keep[2] = {false, false};
                if (ok) {
                    for (int sub = 0; sub < spb; ++sub) {
                        const int st = (id << spb_shift) + sub;
                        bool p0, p1;
                        if (pass == 0) {
                            p0 = st * STEP <= last0;
                            p1 = (st * STEP <= last1) && (!two || bit_of(bits1, id));
                        } else {
                            p0 = false;
                            p1 = st * STEP <= last1;
                        }
                        keep[sub] = (p0 | p1) && st < p.nsteps_total;
                        e[sub] = st | E_FP16 | (p0 ? E_P0 : 0) | (p1 ? E_P1 : 0);
                    }
                }
                const uint32_t m0 = __ballot_sync(0xFFFFFFFFu, keep[0]);
                const uint32_t m1 = __ballot_sync(0xFFFFFFFFu, keep[1]);
                int pos = n + __popc(m0 & lt) + __popc(m1 & lt);
                if (keep[0]) { if (pos < SCHED_CAP) sched[pos] = static_cast<uint16_t>(e[0]); ++pos; }
                if (keep[1] && pos < SCHED_CAP) sched[pos] = static_cast<uint16_t>(e[1]);
                n += __popc(m0) + __popc(m1);
            }
        }
    }
    __syncwarp();
    return n <= SCHED_CAP ? n : -1;
}

// Column maps inside a 64-column step.  With the "permuted" K layout physical
// row p of every 32-row group holds logical row perm32(p); logi[p] is the logical
// column of physical column p and phys[l] its inverse.
template <bool KPERM>
struct ColMap {
    int logi[STEP];
    int phys[STEP];
    constexpr ColMap() : logi(), phys() {
        for (int p = 0; p < STEP; ++p) {
            const int l = KPERM ? (p / 32) * 32 + perm32(p % 32) : p;
            logi[p] = l;
            phys[l] = p;
        }
    }
};

// packed fp32x2 arithmetic (two lanes per instruction)
__device__ __forceinline__ uint64_t pack2f(float a, float b) {
    uint64_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
    return r;
}
__device__ __forceinline__ void unpack2f(uint64_t v, float& a, float& b) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// p_j * scale for 64 logits: s[j] <- 2^(s[j] * c2 + bias); returns the sum of the results.
__device__ __forceinline__ float exp_scaled_64(float (&s)[STEP], float c2, float bias) {
    const uint64_t c2p = pack2f(c2, c2), bp = pack2f(bias, bias);
    uint64_t acc0 = pack2f(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
    for (int j = 0; j < STEP; j += 4) {
        float a, b, c, d;
        unpack2f(fma2(pack2f(s[j], s[j + 1]), c2p, bp), a, b);
        unpack2f(fma2(pack2f(s[j + 2], s[j + 3]), c2p, bp), c, d);
        s[j] = ex2(a); s[j + 1] = ex2(b); s[j + 2] = ex2(c); s[j + 3] = ex2(d);
        acc0 = add2(acc0, pack2f(s[j], s[j + 1]));
        acc1 = add2(acc1, pack2f(s[j + 2], s[j + 3]));
    }
    float x, y;
    unpack2f(add2(acc0, acc1), x, y);
    return x + y;
}

template <int D, bool MX, bool BF16, bool CAUSAL, bool KPERM>
__global__ void __launch_bounds__(NUM_THREADS, 1)
prefill_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap mapQ4, const __grid_constant__ CUtensorMap mapQ16,
               const __grid_constant__ CUtensorMap mapK16, const __grid_constant__ CUtensorMap mapV16) {
    using L = Smem<D>;
    constexpr int QK_ATOMS = MX ? 1 : D / 64;     // 512-byte scale atoms per tile for Q and K
    constexpr int KBLK = D / 64;                   // K=64 MMAs per QK^T (FP4)
    constexpr uint32_t ROW4 = D / 2;               // bytes per FP4 row of Q / K
    constexpr uint32_t SWZ_QK = (ROW4 == 64) ? SWZ_64B : SWZ_32B;
    constexpr uint32_t SBO_QK = 8 * ROW4;
    constexpr int HALVES = D / 64;                 // 64-column halves of a 16-bit row
    constexpr float CSCALE = MX ? 6.0f : 2688.0f;
    constexpr float CSCALE_INV = MX ? (1.0f / 6.0f) : (1.0f / 2688.0f);
    constexpr ColMap<KPERM> cmap{};

    // No static shared memory: the dynamic window then starts 1024-byte aligned, which the
    // 128-byte swizzled tiles need (checked below).
    extern __shared__ __align__(1024) uint8_t smem[];
    Bars& bars = *reinterpret_cast<Bars*>(smem + L::BARS);
    Xch& xch = *reinterpret_cast<Xch*>(smem + L::XCH);
    int& abort_flag = bars.abort_flag;
    uint32_t& tmem_base_s = bars.tmem_base;

    const int tid = threadIdx.x, warp = tid / 32, lane = tid % 32;
    const uint32_t sbase = smem_u32(smem);
    volatile int* abortp = &abort_flag;
    const long long budget = p.budget;
    uint16_t* sched = reinterpret_cast<uint16_t*>(smem + L::SCHED);

    if (tid == 0) {
        mbar_init(smem_u32(&bars.q_full), 1);
        mbar_init(smem_u32(&bars.q_empty), 2);
        mbar_init(smem_u32(&bars.sched_full), 1);
        mbar_init(smem_u32(&bars.sched_empty), 3 + 4 * NSETS);
        mbar_init(smem_u32(&bars.o_full), 1);
        for (int i = 0; i < NSLOTS; ++i) {
            bars.slot_last[i] = 0u;
            mbar_init(smem_u32(&bars.k_full[i]), 1);
            mbar_init(smem_u32(&bars.v_full[i]), 1);
            mbar_init(smem_u32(&bars.slot_empty[i]), 1);
        }
        for (int i = 0; i < NSETS; ++i) {
            mbar_init(smem_u32(&bars.s_full[i]), 1);
            mbar_init(smem_u32(&bars.s_free[i]), 128);
            mbar_init(smem_u32(&bars.p_full[i][0]), 128);
            mbar_init(smem_u32(&bars.p_full[i][1]), 128);
            mbar_init(smem_u32(&bars.p_free[i][0]), 1);
            mbar_init(smem_u32(&bars.p_free[i][1]), 1);
        }
        for (int g = 0; g < 4; ++g) {
            for (int i = 0; i < NSETS; ++i) mbar_init(smem_u32(&bars.mch[g][i]), 32);
            mbar_init(smem_u32(&bars.trans[g]), 32 * NSETS);
            mbar_init(smem_u32(&bars.lend[g]), 32 * NSETS);
        }
        mbar_fence_init();
        abort_flag = (sbase & 1023u) ? 1 : 0;
    }
    // constant scale atom for P: 448 (E4M3 0x7E) or 1.0 (E8M0 0x7F)
    for (int i = tid; i < 512 / 4; i += NUM_THREADS)
        reinterpret_cast<uint32_t*>(smem + L::CSF)[i] = MX ? 0x7F7F7F7Fu : 0x7E7E7E7Eu;
    fence_proxy_async_smem();
    if (warp == 1) {
        tmem_alloc(smem_u32(&tmem_base_s), TM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = tmem_base_s;

    if (warp == 0) {
        // =========================== producer ===========================
        if (lane == 0) {
            tma_prefetch_desc(&mapQ4);
            tma_prefetch_desc(&mapQ16); tma_prefetch_desc(&mapK16); tma_prefetch_desc(&mapV16);
        }
        uint32_t gslot = 0, gsub = 0;     // slots filled / sub-steps loaded so far by this CTA
        uint32_t epar = 0;                // bit s: parity of the next release of slot s through slot_empty
        int n_item = 0;
        bool ok = true;
        // A slot is free again when its last reader is done.  For an FP4 record that is the P V of its sub-step, whose
        // completion the issuer already signals on p_free (for the softmax warps); for a 16-bit tile the issuer that
        // read it commits slot_empty.  bars.slot_last[s] notes which: 0 = never used, bit 31 = slot_empty, else
        // 1 + the CTA-wide index of the sub-step.  When this warp asks about the sub-step's p_free phase, the next
        // phase of that barrier belongs to a sub-step 8 later, which is not even loaded yet: the barrier is in the
        // phase asked for or the one after it.
        auto wait_slot = [&](const uint32_t slot) -> bool {
            const uint32_t last = bars.slot_last[slot];
            if (last == 0u) return true;
            if (last & 0x80000000u) {
                const bool r = mbar_wait(smem_u32(&bars.slot_empty[slot]), (epar >> slot) & 1u, abortp, budget);
                epar ^= 1u << slot;
                return r;
            }
            const uint32_t u = last - 1u, set = u & (NSETS - 1), use = u / NSETS;
            return mbar_wait(smem_u32(&bars.p_free[set][use & 1]), (use >> 1) & 1, abortp, budget);
        };
        auto note_slot = [&](const uint32_t slot, const uint32_t v) {
            __syncwarp();
            if (lane == 0) bars.slot_last[slot] = v;
            __syncwarp();
        };
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n_item) {
            const ItemInfo it = decode_item(p, item);
            // ---- sub-step list (consumers must be done with the previous one) ----
            ok = mbar_wait(smem_u32(&bars.sched_empty), (n_item & 1) ^ 1, abortp, budget);
            if (!ok) break;
            int n_fp4 = 0;
            const int n = build_schedule(p, it, reinterpret_cast<uint32_t*>(smem + L::BITS), sched, lane, n_fp4);
            if (n < 0) { abort_flag = 1; ok = false; break; }
            if (lane == 0) { bars.sched_n = n; bars.sched_na = n_fp4; }
            __syncwarp();
            __threadfence_block();
            if (lane == 0) mbar_arrive(smem_u32(&bars.sched_full));
            if (p.skip_loads) break;   // diagnostics: nothing is copied, the consumers' bounded waits run out
            const bool has_sel = p.width > 0;
            // ---- Q tile ----
            ok = mbar_wait(smem_u32(&bars.q_empty), (n_item & 1) ^ 1, abortp, budget);
            if (!ok) break;
            if (lane == 0) {
                const uint32_t bar = smem_u32(&bars.q_full);
                mbar_expect_tx(bar, QTILE * ROW4 + QK_ATOMS * 512 + (has_sel ? QTILE * D * 2 : 0));
                tma_load_3d(sbase + L::Q4, &mapQ4, bar, 0, it.t * QTILE, it.h);
                bulk_load(sbase + L::QSF, p.q_sf + (static_cast<long long>(it.h) * p.n_qtiles + it.t) * QK_ATOMS * 512,
                          QK_ATOMS * 512, bar);
                if (has_sel)
                    for (int hf = 0; hf < HALVES; ++hf)
                        tma_load_3d(sbase + L::Q16 + hf * QTILE * 128, &mapQ16, bar, hf * 64, it.t * QTILE, it.h);
            }
            // ---- K/V sub-steps ----
            for (int i = 0; i < n && ok; ++i, ++gsub) {
                const uint32_t e = sched[i];
                const int st = e & 0xFFF;
                if (!(e & E_FP16)) {
                    const uint32_t slot = gslot % NSLOTS;
                    ok = wait_slot(slot);
                    if (!ok) break;
                    if (lane == 0) {
                        // one contiguous record: K4 and V4 tiles already in their swizzled shared-memory order + scale atoms
                        const uint32_t bar = smem_u32(&bars.k_full[slot]);
                        mbar_expect_tx(bar, REC_BYTES);
                        bulk_load(sbase + L::SLOTS + slot * SLOT_BYTES,
                                  p.kv_rec + (static_cast<long long>(it.kvh) * p.nsteps_total + st) * REC_BYTES, REC_BYTES, bar);
                    }
                    note_slot(slot, gsub + 1u);
                    gslot += 1;
                } else {
                    for (int which = 0; which < 2 && ok; ++which) {  // K tile, then V tile
                        const uint32_t slot = gslot % NSLOTS;
                        ok = wait_slot(slot);
                        if (!ok) break;
                        if (lane == 0) {
                            const uint32_t bar = smem_u32(which ? &bars.v_full[slot] : &bars.k_full[slot]);
                            const uint32_t sa = sbase + L::SLOTS + slot * SLOT_BYTES;
                            mbar_expect_tx(bar, STEP * D * 2);
                            for (int hf = 0; hf < HALVES; ++hf)
                                tma_load_3d(sa + hf * STEP * 128, which ? &mapV16 : &mapK16, bar, hf * 64, st * STEP, it.kvh);
                        }
                        note_slot(slot, 0x80000000u);
                        gslot += 1;
                    }
                }
            }
        }
    } else if (warp == 1 || warp == 2) {
        // =========================== S = Q K^T issuers ===========================
        // An issuer is a serial instruction stream that its sub-steps pass through one by one, and between the
        // softmax warps of its scheduler it gets an issue slot only every few cycles: a loop of some fifty
        // instructions bounds the whole CTA.  So there are two of these (S buffers are independent of each other):
        // issuer w takes the sub-steps whose CTA-wide index is w modulo 2 and walks past the others, keeping only the
        // ring position and the K-fill parities up to date.  Each has its own copy of Q's scale factors in tensor
        // memory, because tcgen05.cp and tcgen05.mma are ordered only within one thread.
        const uint32_t me = warp - 1;
        const uint32_t tm_sfa_q = tmem + (me ? TM_SFA_Q1 : TM_SFA_Q);
        uint32_t gsub = 0;                // sub-steps walked so far by this CTA
        uint32_t slot = 0, kpar = 0;      // ring position; bit s of kpar = parity of the next K-part fill of slot s
        int n_item = 0;
        bool ok = true;
        const uint32_t idesc_qk4 = make_idesc_fp4(128, STEP, MX ? 1 : 0, 0, 0);
        const uint32_t idesc_qk16 = make_idesc_f16(128, STEP, BF16 ? 1 : 0, 0, 0);
        const uint32_t bar_k_full = smem_u32(&bars.k_full[0]), bar_slot_empty = smem_u32(&bars.slot_empty[0]);
        const uint32_t bar_s_full = smem_u32(&bars.s_full[0]), bar_s_free = smem_u32(&bars.s_free[0]);
        const uint64_t qd0 = make_smem_desc(sbase + L::Q4, 16, SBO_QK, SWZ_QK);             // + 2 per 32-byte K block
        const uint64_t kd0 = make_smem_desc(sbase + L::SLOTS + L::K4, 16, SBO_QK, SWZ_QK);  // + slot * SLOT_BYTES / 16
        const uint64_t sfd0 = make_smem_desc(sbase + L::SLOTS + L::KSF, 0, 128, SWZ_NONE);
        auto next_slot = [&]() { if (++slot == NSLOTS) slot = 0; };
        // FP4 records and 16-bit K tiles land on k_full, 16-bit V tiles on v_full.  The parity of a slot's next K fill
        // is kept for every fill, also those of the other issuer's sub-steps; a slot is not filled again before the
        // sub-step that used it is through, so the barrier asked about is in the phase asked for or the one after it.
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n_item) {
            ok = mbar_wait(smem_u32(&bars.sched_full), n_item & 1, abortp, budget);
            if (!ok) break;
            const int n = bars.sched_n;
            ok = mbar_wait(smem_u32(&bars.q_full), n_item & 1, abortp, budget);
            if (!ok) break;
            tc_fence_after_sync();
            // index of this issuer's last sub-step of the item (Q is released behind it)
            int my_last = n - 1;
            if (((gsub + static_cast<uint32_t>(my_last)) & 1u) != me) my_last -= 1;
            if (my_last >= 0) {
                for (int a = 0; a < QK_ATOMS; ++a)
                    tmem_cp_sf_elect(tm_sfa_q + a * 4, make_smem_desc(sbase + L::QSF + a * 512, 0, 128, SWZ_NONE));
            } else if (lane == 0) {
                mbar_arrive(smem_u32(&bars.q_empty));
            }
            for (int i = 0; i < n && ok; ++i, ++gsub) {
                const uint32_t e = sched[i];
                const bool fp16 = e & E_FP16;
                const uint32_t kslot = slot, kp = (kpar >> slot) & 1u;
                kpar ^= 1u << slot;
                next_slot();
                if (fp16) next_slot();                              // the V tile's slot
                if ((gsub & 1u) != me) continue;
                const uint32_t set = gsub & (NSETS - 1), use = gsub / NSETS;
                const uint32_t d_t = tmem + TM_S + set * STEP;
                ok = mbar_wait(bar_k_full + kslot * 8, kp, abortp, budget) && mbar_wait(bar_s_free + set * 8, (use & 1) ^ 1, abortp, budget);
                if (!ok) break;
                tc_fence_after_sync();
                if (!fp16) {
                    const uint32_t soff = kslot * (SLOT_BYTES / 16);
                    const uint32_t sfb = tmem + TM_SFB_K + set * 8;
                    if (elect_one()) {
                        for (int a = 0; a < QK_ATOMS; ++a) tmem_cp_sf(sfb + a * 4, sfd0 + soff + a * 32);
                        for (int kb = 0; kb < KBLK; ++kb) {
                            if constexpr (MX)
                                mma_mxfp4(d_t, qd0 + kb * 2, kd0 + soff + kb * 2, make_idesc_fp4(128, STEP, 1, kb * 2, kb * 2),
                                          tm_sfa_q, sfb, kb > 0);
                            else
                                mma_nvfp4(d_t, qd0 + kb * 2, kd0 + soff + kb * 2, idesc_qk4, tm_sfa_q + kb * 4, sfb + kb * 4, kb > 0);
                        }
                        tc_commit(bar_s_full + set * 8);
                        if (i == my_last) tc_commit(smem_u32(&bars.q_empty));
                    }
                    __syncwarp();
                } else {
#pragma unroll 1
                    for (int ks = 0; ks < D / 16; ++ks) {
                        const uint32_t hf = ks / 4, kk = ks % 4;
                        const uint64_t ad = make_smem_desc(sbase + L::Q16 + hf * QTILE * 128 + kk * 32, 16, 1024, SWZ_128B);
                        const uint64_t bd = make_smem_desc(sbase + L::SLOTS + kslot * SLOT_BYTES + hf * STEP * 128 + kk * 32, 16, 1024,
                                                           SWZ_128B);
                        mma_f16_elect(d_t, ad, bd, idesc_qk16, ks > 0);
                    }
                    tc_commit_elect(bar_slot_empty + kslot * 8);    // the K tile is free once S is computed
                    tc_commit_elect(bar_s_full + set * 8);
                    if (i == my_last) tc_commit_elect(smem_u32(&bars.q_empty));
                }
            }
            if (lane == 0) mbar_arrive(smem_u32(&bars.sched_empty));
        }
    } else if (warp == 3) {
        // =========================== O += P V issuer ===========================
        // One thread issues every P V of the CTA, in list order (they add into the same accumulator), so this loop is
        // kept as short as it can be: an FP4 sub-step needs no wait for its V tile (it came with the K tile, which the
        // other issuer waited for before S, and P, existed) and no commit for its slot (the producer watches p_free).
        tmem_cp_sf_elect(tmem + TM_SFA_P, make_smem_desc(sbase + L::CSF, 0, 128, SWZ_NONE));
        uint32_t gsub = 0;
        uint32_t slot = 0, vpar = 0;      // ring position; bit s of vpar = parity of the next V-tile fill of slot s
        int n_item = 0;
        bool ok = true;
        const uint32_t idesc_pv4 = make_idesc_fp4(128, D, MX ? 1 : 0, 0, 0);
        const uint32_t idesc_pv16 = make_idesc_f16(128, D, BF16 ? 1 : 0, 0, 1);
        const uint32_t bar_v_full = smem_u32(&bars.v_full[0]), bar_slot_empty = smem_u32(&bars.slot_empty[0]);
        const uint32_t bar_p_full = smem_u32(&bars.p_full[0][0]), bar_p_free = smem_u32(&bars.p_free[0][0]);
        const uint32_t bar_o_full = smem_u32(&bars.o_full);
        const uint64_t pd0 = make_smem_desc(sbase + L::P, 16, 256, SWZ_32B);                 // + set * PSET_BYTES / 16 + buffer * 256
        const uint64_t vd0 = make_smem_desc(sbase + L::SLOTS + L::V4, 16, 256, SWZ_32B);     // + slot * SLOT_BYTES / 16
        const uint64_t sfd0 = make_smem_desc(sbase + L::SLOTS + L::VSF, 0, 128, SWZ_NONE);
        auto next_slot = [&]() { if (++slot == NSLOTS) slot = 0; };
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n_item) {
            ok = mbar_wait(smem_u32(&bars.sched_full), n_item & 1, abortp, budget);
            if (!ok) break;
            const int n = bars.sched_n, n_fp4 = bars.sched_na;
            int i = 0;
            // ---- FP4 sub-steps ----
            for (; i < n_fp4; ++i, ++gsub) {
                const uint32_t set = gsub & (NSETS - 1), use = gsub / NSETS, pb = set * 2 + (use & 1);
                ok = mbar_wait(bar_p_full + pb * 8, (use >> 1) & 1, abortp, budget);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t soff = slot * (SLOT_BYTES / 16);
                const uint32_t sfb = tmem + TM_SFB_V + set * 4;
                const uint64_t ad = pd0 + set * (PSET_BYTES / 16) + (use & 1) * 256;
                if (elect_one()) {
                    tmem_cp_sf(sfb, sfd0 + soff);
                    if constexpr (MX) mma_mxfp4(tmem + TM_O, ad, vd0 + soff, idesc_pv4, tmem + TM_SFA_P, sfb, i > 0);
                    else mma_nvfp4(tmem + TM_O, ad, vd0 + soff, idesc_pv4, tmem + TM_SFA_P, sfb, i > 0);
                    tc_commit(bar_p_free + pb * 8);
                    if (i + 1 == n) tc_commit(bar_o_full);
                }
                __syncwarp();
                next_slot();
            }
            // ---- 16-bit sub-steps ----
            for (; i < n && ok; ++i, ++gsub) {
                const uint32_t set = gsub & (NSETS - 1), use = gsub / NSETS, pb = set * 2 + (use & 1);
                next_slot();                                    // the K tile's slot
                const uint32_t vslot = slot;
                ok = mbar_wait(bar_v_full + vslot * 8, (vpar >> vslot) & 1u, abortp, budget) &&
                     mbar_wait(bar_p_full + pb * 8, (use >> 1) & 1, abortp, budget);
                vpar ^= 1u << vslot;
                if (!ok) break;
                next_slot();
                tc_fence_after_sync();
                const uint32_t pa = sbase + L::P + set * PSET_BYTES;
                const uint32_t va = sbase + L::SLOTS + vslot * SLOT_BYTES;
#pragma unroll 1
                for (int ks = 0; ks < STEP / 16; ++ks) {
                    const uint64_t ad = make_smem_desc(pa + ks * 32, 16, 1024, SWZ_128B);
                    const uint64_t bd = make_smem_desc(va + ks * 2048, STEP * 128, 1024, SWZ_128B);
                    mma_f16_elect(tmem + TM_O, ad, bd, idesc_pv16, (i == 0 && ks == 0) ? 0 : 1);
                }
                tc_commit_elect(bar_slot_empty + vslot * 8);
                tc_commit_elect(bar_p_free + pb * 8);
                if (i + 1 == n) tc_commit_elect(bar_o_full);
            }
            if (!ok) break;
            if (lane == 0) mbar_arrive(smem_u32(&bars.sched_empty));
        }
    } else {
        // =========================== softmax ===========================
        const int g = warp & 3;                   // 32-row group = tensor-memory sub-partition
        const uint32_t set = (warp - 4) >> 2;     // this warp runs the sub-steps with (CTA-wide index) mod 4 == set
        const uint32_t prev_set = (set + NSETS - 1) & (NSETS - 1);
        const int row = g * 32 + lane;            // row inside the q tile
        const int half = g >> 1;                  // 0: rows 0..63, 1: rows 64..127
        const uint32_t lane_addr = static_cast<uint32_t>(g * 32) << 16;
        const uint32_t tm_s = tmem + lane_addr + TM_S + set * STEP;
        uint8_t* const ptile = smem + L::P + set * PSET_BYTES;
        uint32_t gsub0 = 0;                       // CTA-wide index of the item's first sub-step
        int n_item = 0, n_nonempty = 0, n_trans = 0;
        bool ok = true, prev_wide = false;      // prev_wide: this set's previous sub-step wrote a 16-bit P tile
        for (int item = blockIdx.x; item < p.n_items && ok; item += gridDim.x, ++n_item) {
            const ItemInfo it = decode_item(p, item);
            ok = mbar_wait(smem_u32(&bars.sched_full), n_item & 1, abortp, budget);
            if (!ok) break;
            const int n = bars.sched_n, n_fp4 = bars.sched_na;
            const bool has_trans = p.round_partial && n_fp4 > 0 && n_fp4 < n;
            bool trans_sent = false;
            const int grow = it.t * QTILE + row;  // absolute query row
            float m_ref = -FLT_MAX, l_run = 0.0f; // this set's share of the row sum, relative to m_ref
            // one sub-step; the FP4 and the 16-bit kind are compiled separately (they are separate runs of the list)
            auto substep = [&](auto kind, const int i) -> bool {
                constexpr bool fp16 = decltype(kind)::value;
                const uint32_t gsub = gsub0 + i, use = gsub / NSETS;
                const uint32_t e = sched[i];
                const int col0 = (e & 0xFFF) * STEP;
                const bool part = e & (half ? E_P1 : E_P0);
                if (has_trans && !trans_sent && i >= n_fp4) {
                    xch.l_tr[g][set][lane] = l_run; xch.m_tr[g][set][lane] = m_ref;
                    mbar_arrive(smem_u32(&bars.trans[g]));
                    trans_sent = true;
                }
                ok = mbar_wait(smem_u32(&bars.s_full[set]), use & 1, abortp, budget);
                if (!ok) return false;
                tc_fence_after_sync();
                float s[STEP];
                {
                    uint32_t r0[32], r1[32];
                    tmem_ld32(tm_s, r0);
                    tmem_ld32(tm_s + 32, r1);
                    tmem_wait_ld();
#pragma unroll
                    for (int j = 0; j < 32; ++j) { s[j] = __uint_as_float(r0[j]); s[32 + j] = __uint_as_float(r1[j]); }
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&bars.s_free[set]));

                float m_loc = -FLT_MAX;
                if (part) {
                    if (CAUSAL && (col0 + STEP - 1 > grow)) {
#pragma unroll
                        for (int j = 0; j < STEP; ++j) {
                            const int lc = fp16 ? j : cmap.logi[j];
                            if (col0 + lc > grow) s[j] = -INFINITY;
                        }
                    }
                    float mx0 = -FLT_MAX, mx1 = -FLT_MAX, mx2 = -FLT_MAX, mx3 = -FLT_MAX;
#pragma unroll
                    for (int j = 0; j < STEP; j += 8) {
                        mx0 = max3(mx0, s[j], s[j + 1]);
                        mx1 = max3(mx1, s[j + 2], s[j + 3]);
                        mx2 = max3(mx2, s[j + 4], s[j + 5]);
                        mx3 = max3(mx3, s[j + 6], s[j + 7]);
                    }
                    m_loc = max3(fmaxf(mx0, mx1), mx2, mx3);
                }
                // running maximum: from the set that ran the previous sub-step, to the one that runs the next
                float m_prev = -FLT_MAX;
                if (gsub > 0) {
                    ok = mbar_wait(smem_u32(&bars.mch[g][prev_set]), ((gsub - 1) / NSETS) & 1, abortp, budget);
                    if (!ok) return false;
                    if (i > 0) m_prev = xch.mrun[g][prev_set][lane];
                }
                const float m_new = fmaxf(m_prev, m_loc);
                xch.mrun[g][set][lane] = m_new;
                mbar_arrive(smem_u32(&bars.mch[g][set]));
                const bool changed = m_new > m_prev;
                const float rescale_o = ex2((m_prev - m_new) * p.c2);
                const float rescale_l = ex2((m_ref - m_new) * p.c2);
                m_ref = m_new;
                const float mneg = -m_new * p.c2;
                l_run *= rescale_l;
                const bool transition = fp16 && has_trans && i == n_fp4;
                const bool need_rescale = __any_sync(0xFFFFFFFFu, changed && i > 0);

                // The set's P memory holds two FP4 tiles (buffer use & 1) or one 16-bit tile that spans both.  Buffer
                // b is free once the P V of the set's sub-step two uses ago completed; a 16-bit tile - this one or the
                // previous one - also involves the other buffer, whose latest reader is the previous use.
                const uint32_t pbuf = use & 1;
                ok = mbar_wait(smem_u32(&bars.p_free[set][pbuf]), ((use >> 1) & 1) ^ 1, abortp, budget);
                if (ok && (fp16 || prev_wide) && use > 0)
                    ok = mbar_wait(smem_u32(&bars.p_free[set][pbuf ^ 1]), ((use - 1) >> 1) & 1, abortp, budget);
                if (!ok) return false;
                prev_wide = fp16;
                if constexpr (!fp16) {
                    uint32_t w[STEP / 8];
                    if (part) {
                        // 6 p = 2^(s c2 - m c2 + log2 6): the e2m1 input directly
                        const float sum6 = exp_scaled_64(s, p.c2, mneg + 2.5849625007211562f);
                        l_run = fmaf(sum6, 1.0f / 6.0f, l_run);
#pragma unroll
                        for (int q8 = 0; q8 < STEP / 8; ++q8)
                            w[q8] = e2m1x8(s[cmap.phys[q8 * 8 + 0]], s[cmap.phys[q8 * 8 + 1]], s[cmap.phys[q8 * 8 + 2]],
                                           s[cmap.phys[q8 * 8 + 3]], s[cmap.phys[q8 * 8 + 4]], s[cmap.phys[q8 * 8 + 5]],
                                           s[cmap.phys[q8 * 8 + 6]], s[cmap.phys[q8 * 8 + 7]]);
                    } else {
#pragma unroll
                        for (int q8 = 0; q8 < STEP / 8; ++q8) w[q8] = 0u;
                    }
                    // 128 rows x 32 bytes, 32-byte swizzle
                    const uint32_t r8 = row & 7;
                    uint8_t* base = ptile + pbuf * 4096 + (row >> 3) * 256 + r8 * 32;
                    const uint32_t x = (r8 >> 2) & 1;
                    *reinterpret_cast<uint4*>(base + ((0 ^ x) * 16)) = make_uint4(w[0], w[1], w[2], w[3]);
                    *reinterpret_cast<uint4*>(base + ((1 ^ x) * 16)) = make_uint4(w[4], w[5], w[6], w[7]);
                } else {
                    // C p = 2^(s c2 - m c2 + log2 C): the 16-bit P operand directly.  128 rows x 128 bytes,
                    // 128-byte swizzle; eight values are exponentiated, packed and stored at a time.
                    constexpr float LOG2_C = MX ? 2.5849625007211562f : 11.392317422778761f;
                    const uint32_t r8 = row & 7;
                    uint8_t* base = ptile + (row >> 3) * 1024 + r8 * 128;
                    if (part) {
                        const uint64_t c2p = pack2f(p.c2, p.c2), bp = pack2f(mneg + LOG2_C, mneg + LOG2_C);
                        uint64_t acc0 = pack2f(0.0f, 0.0f), acc1 = acc0;
#pragma unroll
                        for (int c = 0; c < 8; ++c) {
                            float v[8];
#pragma unroll
                            for (int j = 0; j < 8; j += 2) {
                                float a0, a1;
                                unpack2f(fma2(pack2f(s[8 * c + j], s[8 * c + j + 1]), c2p, bp), a0, a1);
                                v[j] = ex2(a0); v[j + 1] = ex2(a1);
                            }
                            acc0 = add2(acc0, add2(pack2f(v[0], v[1]), pack2f(v[2], v[3])));
                            acc1 = add2(acc1, add2(pack2f(v[4], v[5]), pack2f(v[6], v[7])));
                            *reinterpret_cast<uint4*>(base + ((c ^ r8) * 16)) =
                                make_uint4(In16<BF16>::pack2(v[0], v[1]), In16<BF16>::pack2(v[2], v[3]),
                                           In16<BF16>::pack2(v[4], v[5]), In16<BF16>::pack2(v[6], v[7]));
                        }
                        float x, y;
                        unpack2f(add2(acc0, acc1), x, y);
                        l_run = fmaf(x + y, CSCALE_INV, l_run);
                    } else {
#pragma unroll
                        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(base + c * 16) = make_uint4(0u, 0u, 0u, 0u);
                    }
                }
                fence_proxy_async_smem();
                // O may be touched once the P V of the previous sub-step (another set's) has completed; the
                // issuer adds this sub-step's P V only after the arrival below.  Only a moved maximum (or the state
                // rounding) needs that wait: waiting every time would chain every sub-step behind the completion of
                // the one before it.  This warp does not see every phase of that barrier, but it has seen (above,
                // on its own buffer) the P V of sub-step gsub-8 complete, so the P V of gsub-9 - the previous reader
                // of the buffer asked about, committed earlier by the same thread - has completed as well and the
                // barrier is in the phase asked for or past it.
                if (gsub > 0 && (need_rescale || transition)) {
                    const uint32_t puse = (gsub - 1) / NSETS;
                    ok = mbar_wait(smem_u32(&bars.p_free[prev_set][puse & 1]), (puse >> 1) & 1, abortp, budget);
                    if (!ok) return false;
                }
                if (transition) {
                    // state rounding between the FP4 and the 16-bit phase (state before this sub-step's update):
                    // the row sum is the sum of the four sets' shares at their last FP4 sub-step
                    ok = mbar_wait(smem_u32(&bars.trans[g]), n_trans & 1, abortp, budget);
                    if (!ok) return false;
                    float l_prev = 0.0f;
#pragma unroll
                    for (int c = 0; c < NSETS; ++c)
                        l_prev = fmaf(xch.l_tr[g][c][lane], ex2((xch.m_tr[g][c][lane] - m_prev) * p.c2), l_prev);
                    tc_fence_after_sync();
                    const float norm = l_prev > 0.0f ? __fdiv_rn(CSCALE_INV, l_prev) : 0.0f;
                    const float back = l_prev * CSCALE * rescale_o;
#pragma unroll 1
                    for (int c = 0; c < D; c += 32) {
                        uint32_t r[32];
                        tmem_ld32(tmem + lane_addr + TM_O + c, r);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            const float v = __uint_as_float(r[j]) * norm;
                            r[j] = __float_as_uint(In16<BF16>::to_f(In16<BF16>::from_f(v)) * back);
                        }
                        tmem_st32(tmem + lane_addr + TM_O + c, r);
                    }
                    tmem_wait_st();
                } else if (need_rescale) {
                    // 64 columns per tensor-memory round trip (the scores' registers are free by now): this block sits
                    // on the chain that orders consecutive sub-steps, so its length counts
                    tc_fence_after_sync();
#pragma unroll 1
                    for (int c = 0; c < D; c += 64) {
                        uint32_t ra[32], rb[32];
                        tmem_ld32(tmem + lane_addr + TM_O + c, ra);
                        tmem_ld32(tmem + lane_addr + TM_O + c + 32, rb);
                        tmem_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            ra[j] = __float_as_uint(__uint_as_float(ra[j]) * rescale_o);
                            rb[j] = __float_as_uint(__uint_as_float(rb[j]) * rescale_o);
                        }
                        tmem_st32(tmem + lane_addr + TM_O + c, ra);
                        tmem_st32(tmem + lane_addr + TM_O + c + 32, rb);
                    }
                    tmem_wait_st();
                }
                tc_fence_before_sync();
                mbar_arrive(smem_u32(&bars.p_full[set][pbuf]));
                return true;
            };
            {
                int i = (set - gsub0) & (NSETS - 1);
                for (; i < n_fp4 && ok; i += NSETS) ok = substep(std::false_type{}, i);
                for (; i < n && ok; i += NSETS) ok = substep(std::true_type{}, i);
            }
            if (!ok) break;
            if (has_trans) {
                if (!trans_sent) {
                    xch.l_tr[g][set][lane] = l_run; xch.m_tr[g][set][lane] = m_ref;
                    mbar_arrive(smem_u32(&bars.trans[g]));
                }
                ++n_trans;
            }
            // ---- epilogue: the four sets of a row group add up their row sums and each normalises and
            //      stores a quarter of the output channels ----
            constexpr int DQ = D / NSETS;          // channels per set
            uint16_t* orow = p.out + (p.out_seq_major
                ? ((static_cast<long long>(it.h / p.hq_per_b) * p.sq + grow) * p.hq_per_b + it.h % p.hq_per_b) * D
                : (static_cast<long long>(it.h) * p.sq + grow) * D) + set * DQ;
            if (n > 0) {
                xch.l_end[g][set][lane] = l_run; xch.m_end[g][set][lane] = m_ref;
                mbar_arrive(smem_u32(&bars.lend[g]));
                ok = mbar_wait(smem_u32(&bars.lend[g]), n_nonempty & 1, abortp, budget);
                if (!ok) break;
                float m_fin = -FLT_MAX;
#pragma unroll
                for (int c = 0; c < NSETS; ++c) m_fin = fmaxf(m_fin, xch.m_end[g][c][lane]);
                float l_tot = 0.0f;
#pragma unroll
                for (int c = 0; c < NSETS; ++c)
                    l_tot = fmaf(xch.l_end[g][c][lane], ex2((xch.m_end[g][c][lane] - m_fin) * p.c2), l_tot);
                ok = mbar_wait(smem_u32(&bars.o_full), n_nonempty & 1, abortp, budget);
                if (!ok) break;
                ++n_nonempty;
                tc_fence_after_sync();
                const float norm = l_tot > 0.0f ? __fdiv_rn(CSCALE_INV, l_tot) : 0.0f;
                uint32_t r[DQ];
                if constexpr (DQ == 32) tmem_ld32(tmem + lane_addr + TM_O + set * DQ, r);
                else tmem_ld16(tmem + lane_addr + TM_O + set * DQ, r);
                tmem_wait_ld();
                if (grow < p.sq) {
#pragma unroll
                    for (int v4 = 0; v4 < DQ / 8; ++v4) {
                        uint32_t o[4];
#pragma unroll
                        for (int e2 = 0; e2 < 4; ++e2)
                            o[e2] = In16<BF16>::pack2(__uint_as_float(r[v4 * 8 + 2 * e2]) * norm,
                                                      __uint_as_float(r[v4 * 8 + 2 * e2 + 1]) * norm);
                        *reinterpret_cast<uint4*>(orow + v4 * 8) = make_uint4(o[0], o[1], o[2], o[3]);
                    }
                }
                tc_fence_before_sync();
            } else if (grow < p.sq) {
                for (int c = 0; c < DQ; c += 8) *reinterpret_cast<uint4*>(orow + c) = make_uint4(0, 0, 0, 0);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&bars.sched_empty));
            gsub0 += n;
        }
    }

    // ---- common exit ----
    if (abort_flag != 0) __nanosleep(20000);  // let copies already in flight land
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tmem, TM_COLS);
    if (tid == 0 && abort_flag != 0) atomicExch(p.status, 1);
}

// ---------------------------------------------------------------------------
// Scale-factor re-tiling: row-major scale bytes -> 512-byte tcgen05 atoms
//   atom[m0 * 16 + m1 * 4 + j] = scale(row = 32 * m1 + m0, j)
// ---------------------------------------------------------------------------
__global__ void retile_row_scales_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int heads,
                                         int rows_valid, long long head_stride_rows, int spr, int tile_rows,
                                         int ntiles, int natoms, int per_atom) {
    const long long total = static_cast<long long>(heads) * ntiles * natoms * 128;  // 4-byte words
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        const int wi = static_cast<int>(i & 127);
        const int m0 = wi >> 2, m1 = wi & 3;
        long long rest = i >> 7;
        const int atom = static_cast<int>(rest % natoms); rest /= natoms;
        const int tile = static_cast<int>(rest % ntiles);
        const int head = static_cast<int>(rest / ntiles);
        const int r_in_tile = 32 * m1 + m0;
        const long long row = static_cast<long long>(tile) * tile_rows + r_in_tile;
        uint32_t word = 0;
        if (r_in_tile < tile_rows && row < rows_valid) {
            const uint8_t* s = src + (head * head_stride_rows + row) * spr + atom * per_atom;
            for (int j = 0; j < per_atom; ++j) word |= static_cast<uint32_t>(s[j]) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(dst)[i] = word;
    }
}

// ---------------------------------------------------------------------------
// K/V packing for the attention kernel: one contiguous REC_BYTES record per (KV head, 64-token sub-step), laid out
// exactly as the kernel's ring slot: the K4 tile [64 keys x D/2 bytes] and the V4 tile [D channels x 32 bytes] in
// their swizzled shared-memory order (so that a plain bulk copy lands them ready for the tensor core: a tiled copy
// of 32- and 64-byte rows costs the copy engine a request per row, which is what held the whole kernel back), and
// the K and V block scales as 512-byte tcgen05 atoms  atom[m0 * 16 + m1 * 4 + j] = scale(row 32 * m1 + m0, j).
// One CTA of 256 threads per record.
// ---------------------------------------------------------------------------
template <int D>
__global__ void __launch_bounds__(256)
pack_kv_records_kernel(const uint8_t* __restrict__ k4, const uint8_t* __restrict__ ks, const uint8_t* __restrict__ v4t,
                       const uint8_t* __restrict__ vst, uint8_t* __restrict__ rec, int skv, long long kv_cap, int P, int nsteps,
                       int is_mx) {
    constexpr int ROW4 = D / 2, CPR = ROW4 / 16;            // bytes and 16-byte chunks per K4 row
    const int st = blockIdx.x, head = blockIdx.y, t = threadIdx.x;
    uint8_t* out = rec + (static_cast<long long>(head) * nsteps + st) * REC_BYTES;
    const int G = is_mx ? 32 : 16, spr = D / G, atoms = is_mx ? 1 : D / 64, per_atom = is_mx ? spr : 4;
    // K4: 64 rows; chunk c of row r goes to chunk c ^ f(r) (64-byte rows: f = (r >> 1) & 3; 32-byte rows: (r >> 2) & 1)
    for (int i = t; i < STEP * CPR; i += 256) {
        const int r = i / CPR, c = i % CPR;
        const long long row = static_cast<long long>(st) * STEP + r;
        uint4 val = make_uint4(0, 0, 0, 0);
        if (row < skv) val = *reinterpret_cast<const uint4*>(k4 + (head * kv_cap + row) * ROW4 + c * 16);
        const int cs = CPR == 4 ? (c ^ ((r >> 1) & 3)) : (c ^ ((r >> 2) & 1));
        *reinterpret_cast<uint4*>(out + r * ROW4 + cs * 16) = val;
    }
    // V4: D channel rows of 32 bytes (64 tokens), 32-byte swizzle
    for (int i = t; i < D * 2; i += 256) {
        const int r = i >> 1, c = i & 1;
        const uint4 val = *reinterpret_cast<const uint4*>(v4t + (static_cast<long long>(head) * D + r) * (P / 2) + st * 32 + c * 16);
        *reinterpret_cast<uint4*>(out + 5120 + r * 32 + ((c ^ ((r >> 2) & 1)) * 16)) = val;
    }
    // K scale atoms
    for (int i = t; i < atoms * 128; i += 256) {
        const int wi = i & 127, atom = i >> 7, m0 = wi >> 2, m1 = wi & 3;
        const int r_in = 32 * m1 + m0;
        const long long row = static_cast<long long>(st) * STEP + r_in;
        uint32_t word = 0;
        if (r_in < STEP && row < skv) {
            const uint8_t* src = ks + (head * kv_cap + row) * spr + atom * per_atom;
            for (int j = 0; j < per_atom; ++j) word |= static_cast<uint32_t>(src[j]) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(out + 4096)[i] = word;
    }
    // V scale atom: scale(channel 32 * m1 + m0, token group st * per + j)
    if (t < 128) {
        const int m0 = t >> 2, m1 = t & 3, ch = 32 * m1 + m0, per = STEP / G, pg = P / G;
        uint32_t word = 0;
        if (ch < D) {
            const uint8_t* src = vst + (static_cast<long long>(head) * D + ch) * pg + st * per;
            for (int j = 0; j < per; ++j) word |= static_cast<uint32_t>(src[j]) << (8 * j);
        }
        reinterpret_cast<uint32_t*>(out + 9216)[t] = word;
    }
}

struct WsLayout {
    size_t q_sf, kv_rec, status, total;
};

WsLayout ws_layout(int hq_flat, int hkv_flat, int sq, int skv, int d, int is_mx) {
    const int atoms = is_mx ? 1 : d / 64;
    const size_t n_qtiles = cdiv(sq, QTILE), nsteps = cdiv(skv, STEP);
    WsLayout w;
    w.q_sf = 0;
    w.kv_rec = w.q_sf + static_cast<size_t>(hq_flat) * n_qtiles * atoms * 512;
    w.status = w.kv_rec + static_cast<size_t>(hkv_flat) * nsteps * REC_BYTES;
    w.total = w.status + 256;
    return w;
}

template <int D, bool MX, bool BF16, bool CAUSAL, bool KPERM>
int launch_prefill_t(const PrefillParams& p, const CUtensorMap* maps, int grid, cudaStream_t stream) {
    auto kern = prefill_kernel<D, MX, BF16, CAUSAL, KPERM>;
    const int smem = Smem<D>::TOTAL;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
    if (e != cudaSuccess) return static_cast<int>(e);
    kern<<<grid, NUM_THREADS, smem, stream>>>(p, maps[0], maps[3], maps[4], maps[5]);
    return static_cast<int>(cudaGetLastError());
}

}  // namespace

size_t prefill_workspace_bytes(int batch, int hq, int hkv, int sq, int skv, int d, int is_mx) {
    return ws_layout(batch * hq, batch * hkv, sq, skv, d, is_mx).total;
}

// See include/thrift_sm100.h (ta100_prefill_attention) for the contract.
int prefill_dispatch(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, int block,
                     const void* q4, const void* k4, const void* v4t, const void* qs, const void* ks, const void* vst,
                     void* out, void* workspace, size_t workspace_bytes, int batch, int hq, int hkv, int sq, int skv,
                     int kv_cap, int d, int causal, int is_mx, int is_bf16, int k_permuted, int round_partial,
                     int max_ctas, int out_seq_major, cudaStream_t stream) {
    if (!q4 || !k4 || !v4t || !qs || !ks || !vst || !out || !workspace) return TA100_ERR_NULL;
    if (width > 0 && (!q_hi || !k_hi || !v_hi || !sel)) return TA100_ERR_NULL;
    if (d != 128 && d != 64) return TA100_ERR_UNSUPPORTED;
    if (block != 64 && block != 128) return TA100_ERR_UNSUPPORTED;
    if (batch <= 0 || hq <= 0 || hkv <= 0 || hq % hkv != 0 || sq <= 0 || skv <= 0) return TA100_ERR_SHAPE;
    if (sq % 64 != 0 || skv % 64 != 0 || kv_cap < skv) return TA100_ERR_SHAPE;
    if (width > 0 && (sq % block != 0 || skv % block != 0)) return TA100_ERR_SHAPE;
    if (skv / 64 > 2048 || width > 2048) return TA100_ERR_LIMIT;
    const int hq_flat = batch * hq, hkv_flat = batch * hkv;
    const WsLayout w = ws_layout(hq_flat, hkv_flat, sq, skv, d, is_mx);
    if (workspace_bytes < w.total) return TA100_ERR_WORKSPACE;
    if ((reinterpret_cast<uintptr_t>(workspace) & 255) != 0) return TA100_ERR_ALIGN;
    uint8_t* ws = static_cast<uint8_t*>(workspace);
    const int G = is_mx ? 32 : 16;
    const int spr = d / G;
    const int atoms = is_mx ? 1 : d / 64;
    const int per_atom = is_mx ? spr : 4;
    const int n_qtiles = cdiv(sq, QTILE), nsteps = cdiv(skv, STEP);
    const int P = cdiv(kv_cap, 128) * 128;

    cudaError_t e = cudaMemsetAsync(ws + w.status, 0, 4, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    {
        long long words = static_cast<long long>(hq_flat) * n_qtiles * atoms * 128;
        retile_row_scales_kernel<<<grid_for(words, 256, 8), 256, 0, stream>>>(
            static_cast<const uint8_t*>(qs), ws + w.q_sf, hq_flat, sq, sq, spr, QTILE, n_qtiles, atoms, per_atom);
        const dim3 pgrid(nsteps, hkv_flat);
        if (d == 128)
            pack_kv_records_kernel<128><<<pgrid, 256, 0, stream>>>(
                static_cast<const uint8_t*>(k4), static_cast<const uint8_t*>(ks), static_cast<const uint8_t*>(v4t),
                static_cast<const uint8_t*>(vst), ws + w.kv_rec, skv, kv_cap, P, nsteps, is_mx);
        else
            pack_kv_records_kernel<64><<<pgrid, 256, 0, stream>>>(
                static_cast<const uint8_t*>(k4), static_cast<const uint8_t*>(ks), static_cast<const uint8_t*>(v4t),
                static_cast<const uint8_t*>(vst), ws + w.kv_rec, skv, kv_cap, P, nsteps, is_mx);
        e = cudaGetLastError();
        if (e != cudaSuccess) return static_cast<int>(e);
    }

    CUtensorMap maps[6];
    memset(maps, 0, sizeof(maps));
    {
        const CUtensorMapSwizzle sw4 = (d / 2 == 64) ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B;
        int rc = 0;
        {
            uint64_t dims[3] = {static_cast<uint64_t>(d / 2), static_cast<uint64_t>(sq), static_cast<uint64_t>(hq_flat)};
            uint64_t str[2] = {static_cast<uint64_t>(d / 2), static_cast<uint64_t>(sq) * (d / 2)};
            uint32_t box[3] = {static_cast<uint32_t>(d / 2), QTILE, 1};
            rc |= make_tensor_map(&maps[0], CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, q4, dims, str, box, sw4);
        }
        if (width > 0) {
            const CUtensorMapDataType dt = is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
            {
                uint64_t dims[3] = {static_cast<uint64_t>(d), static_cast<uint64_t>(sq), static_cast<uint64_t>(hq_flat)};
                uint64_t str[2] = {static_cast<uint64_t>(d) * 2, static_cast<uint64_t>(sq) * d * 2};
                uint32_t box[3] = {64, QTILE, 1};
                rc |= make_tensor_map(&maps[3], dt, 3, q_hi, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
            }
            uint64_t dims[3] = {static_cast<uint64_t>(d), static_cast<uint64_t>(skv), static_cast<uint64_t>(hkv_flat)};
            // the 16-bit K/V share the capacity (row stride between heads) of the packed K
            uint64_t str[2] = {static_cast<uint64_t>(d) * 2, static_cast<uint64_t>(kv_cap) * d * 2};
            uint32_t box[3] = {64, STEP, 1};
            rc |= make_tensor_map(&maps[4], dt, 3, k_hi, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
            rc |= make_tensor_map(&maps[5], dt, 3, v_hi, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
        } else {
            maps[3] = maps[0]; maps[4] = maps[0]; maps[5] = maps[0];
        }
        if (rc != 0) return TA100_ERR_TENSOR_MAP;
    }

    PrefillParams p;
    p.batch = batch; p.hq_per_b = hq; p.hkv_per_b = hkv; p.group = hq / hkv;
    p.sq = sq; p.skv = skv; p.block = block; p.width = width;
    p.causal = causal; p.round_partial = round_partial; p.out_seq_major = out_seq_major ? 1 : 0;
    p.n_qtiles = n_qtiles; p.n_items = n_qtiles * hq_flat; p.nsteps_total = nsteps; p.nkb = skv / block;
    p.sel = static_cast<const int32_t*>(sel);
    p.q_sf = ws + w.q_sf; p.kv_rec = ws + w.kv_rec;
    p.out = static_cast<uint16_t*>(out);
    p.status = reinterpret_cast<int*>(ws + w.status);
    p.c2 = static_cast<float>((1.0 / sqrt(static_cast<double>(d))) * 1.4426950408889634);
    p.budget = g_wait_budget_cycles;
    p.skip_loads = g_test_skip_loads;

    int dev = 0, sms = NUM_SMS_HINT;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    int grid = p.n_items < sms ? p.n_items : sms;
    if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;

#define TA100_PF(DD, MXX, BFF, CC, KP) launch_prefill_t<DD, MXX, BFF, CC, KP>(p, maps, grid, stream)
#define TA100_PF2(DD, MXX, BFF)                                                                        \
    (causal ? (k_permuted ? TA100_PF(DD, MXX, BFF, true, true) : TA100_PF(DD, MXX, BFF, true, false))  \
            : (k_permuted ? TA100_PF(DD, MXX, BFF, false, true) : TA100_PF(DD, MXX, BFF, false, false)))
    int rc;
    if (d == 128) {
        if (is_mx) rc = is_bf16 ? TA100_PF2(128, true, true) : TA100_PF2(128, true, false);
        else rc = is_bf16 ? TA100_PF2(128, false, true) : TA100_PF2(128, false, false);
    } else {
        if (is_mx) rc = is_bf16 ? TA100_PF2(64, true, true) : TA100_PF2(64, true, false);
        else rc = is_bf16 ? TA100_PF2(64, false, true) : TA100_PF2(64, false, false);
    }
#undef TA100_PF2
#undef TA100_PF
    return rc;
}


// Reads back the device status word written by the last prefill launch that
// used `workspace` (synchronises the stream).
int prefill_status(const void* workspace, int batch, int hq, int hkv, int sq, int skv, int d, int is_mx,
                   cudaStream_t stream) {
    const WsLayout w = ws_layout(batch * hq, batch * hkv, sq, skv, d, is_mx);
    int st = 0;
    cudaError_t e = cudaMemcpyAsync(&st, static_cast<const uint8_t*>(workspace) + w.status, 4, cudaMemcpyDeviceToHost, stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess) return static_cast<int>(e);
    return st ? TA100_ERR_DEVICE_TIMEOUT : TA100_OK;
}

}  // namespace ta100
