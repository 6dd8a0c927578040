// Single-token (decode) selective mixed-precision attention, split over the KV
// sequence, plus the log-sum-exp merge of the partial results.
//
// Work decomposition: one warp (= one CTA) per chain; chain s of a (sequence,
// KV head) pair walks pages [s*n/S, (s+1)*n/S) of 64 tokens: first the pages that
// are NOT selected (FP4 K/V, P re-quantised to e2m1 with a per-group dynamic
// scale), ascending, then the selected pages (16-bit K/V), ascending.  Rows of
// the problem are the G <= 8 query heads that share the KV head.
//
// The kernel is HBM-bound; pages are streamed with cp.async into per-warp
// double buffers.  FP4 operands are dequantised exactly to f16 in registers
// (e2m1 x E4M3 products fit f16; for MXFP4 the E8M0 scales are applied in fp32
// per 32-wide group) and multiplied with mma.sync.m16n8k16, with the KV tokens
// (or head channels) on the M side and the query heads on the N side.
#include <cfloat>
#include <mutex>

#include "common.cuh"

namespace ta100 {

namespace {

constexpr int PAGE = 64;
constexpr int KROW = 80;    // padded shared-memory row of a 64-byte FP4 K row
constexpr int VROW = 48;    // padded row of a 32-byte FP4 V^T row
constexpr int HROW = 272;   // padded row of a 256-byte 16-bit row (D = 128)
constexpr int PROW = 72;    // f16 elements per row of the P staging tile (64 + 8)

struct DecodeParams {
    const uint16_t* q_hi;   // [heads, G, D]
    const uint8_t* q4;      // [heads, G, D/2]
    const uint8_t* qs;      // [heads, G, D/g]
    const uint8_t* k4;      // rows layout or page pool
    const uint8_t* ks;
    const uint8_t* v4;      // transposed layout or page pool
    const uint8_t* vs;
    const uint16_t* k_hi;   // [heads, kv_len, D] with head stride kv_cap rows, or page pool
    const uint16_t* v_hi;
    const int32_t* sel;     // [heads, width]
    const int32_t* page_table;  // [batch, max_pages] or null
    float* part_o;          // [heads, splits, G, D]
    float* part_ml;         // [heads, splits, G, 2]
    int heads, hkv, G, npages, cap_pages, max_pages, width, splits;
    long long v_head_stride;   // bytes between heads in v4 (contiguous layout)
    long long vs_head_stride;
    int v_row_stride, vs_row_stride;  // bytes between channel rows
    float sm_scale;
};

__device__ __forceinline__ void cp16(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
                 "l"(gsrc));
}
__device__ __forceinline__ void cp4(void* smem_dst, const void* gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst))),
                 "l"(gsrc));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// one byte of two e2m1 codes -> f16x2 (low nibble in the low half), exact
__device__ __forceinline__ uint32_t e2m1x2_to_h2(uint32_t byte) {
    uint32_t r;
    asm("{\n\t.reg .b8 b;\n\tcvt.u8.u32 b, %1;\n\tcvt.rn.f16x2.e2m1x2 %0, b;\n\t}\n" : "=r"(r) : "r"(byte));
    return r;
}
__device__ __forceinline__ uint32_t h2mul(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}
__device__ __forceinline__ uint32_t f2h2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void mma_f16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fragment for two consecutive k16 chunks from one 32-bit word of 8 e2m1 codes per row:
// codes 0,1 / 2,3 feed chunk 0 (k slots 2t,2t+1 / 2t+8,2t+9), codes 4,5 / 6,7 chunk 1.
__device__ __forceinline__ void word_to_frags(uint32_t w_lo_row, uint32_t w_hi_row, uint32_t scale_lo_h2,
                                              uint32_t scale_hi_h2, bool apply_scale, uint32_t (&a0)[4],
                                              uint32_t (&a1)[4]) {
    uint32_t l0 = e2m1x2_to_h2(w_lo_row & 0xFF), l1 = e2m1x2_to_h2((w_lo_row >> 8) & 0xFF);
    uint32_t l2 = e2m1x2_to_h2((w_lo_row >> 16) & 0xFF), l3 = e2m1x2_to_h2(w_lo_row >> 24);
    uint32_t h0 = e2m1x2_to_h2(w_hi_row & 0xFF), h1 = e2m1x2_to_h2((w_hi_row >> 8) & 0xFF);
    uint32_t h2 = e2m1x2_to_h2((w_hi_row >> 16) & 0xFF), h3 = e2m1x2_to_h2(w_hi_row >> 24);
    if (apply_scale) {
        l0 = h2mul(l0, scale_lo_h2); l1 = h2mul(l1, scale_lo_h2); l2 = h2mul(l2, scale_lo_h2); l3 = h2mul(l3, scale_lo_h2);
        h0 = h2mul(h0, scale_hi_h2); h1 = h2mul(h1, scale_hi_h2); h2 = h2mul(h2, scale_hi_h2); h3 = h2mul(h3, scale_hi_h2);
    }
    a0[0] = l0; a0[1] = h0; a0[2] = l1; a0[3] = h1;
    a1[0] = l2; a1[1] = h2; a1[2] = l3; a1[3] = h3;
}

template <bool MX>
__device__ __forceinline__ uint32_t scale_to_h2(uint8_t b) {
    const float f = decode_scale<MX>(b);
    return f2h2(f, f);
}

// shared-memory carve-up of one warp
struct WarpSmem {
    // FP4 phase: two page buffers
    static constexpr int K4 = 0;                         // [2][64][KROW]
    static constexpr int KS = K4 + 2 * PAGE * KROW;      // [2][64][8]
    static constexpr int V4 = KS + 2 * PAGE * 8;         // [2][128][VROW]
    static constexpr int VS = V4 + 2 * 128 * VROW;       // [2][128][4]
    static constexpr int FP4_END = VS + 2 * 128 * 4;
    // 16-bit phase: one page of K or V (aliases the FP4 buffers)
    static constexpr int H16 = 0;                        // [64][HROW]
    static constexpr int H16_END = PAGE * HROW;
    static constexpr int PT = (FP4_END > H16_END ? FP4_END : H16_END);  // P staging [8][PROW] f16
    static constexpr int FLAGS = PT + 8 * PROW * 2;      // selected-page flags, 1 byte per page (<= 2048)
    static constexpr int TOTAL = FLAGS + 2048;
};

template <bool MX, bool BF16>
__global__ void __launch_bounds__(32) decode_kernel(const DecodeParams p) {
    constexpr int D = 128;
    constexpr int GRP = MX ? 32 : 16;
    constexpr int SPR = D / GRP;           // K/Q scales per row
    constexpr float C = MX ? 6.0f : 2688.0f;
    extern __shared__ __align__(16) uint8_t sm[];
    const int lane = threadIdx.x, gl = lane >> 2, t = lane & 3;
    const int split = blockIdx.x, h = blockIdx.y;
    const int G = p.G;
    const int b = h / p.hkv, kvh = h - b * p.hkv;
    const int p_begin = static_cast<int>(static_cast<long long>(split) * p.npages / p.splits);
    const int p_end = static_cast<int>(static_cast<long long>(split + 1) * p.npages / p.splits);

    // ---- selected-page flags for this chain ----
    uint8_t* flags = sm + WarpSmem::FLAGS;
    for (int i = lane; i < p_end - p_begin; i += 32) flags[i] = 0;
    __syncwarp();
    for (int i = lane; i < p.width; i += 32) {
        const int id = p.sel[static_cast<long long>(h) * p.width + i];
        if (id >= p_begin && id < p_end) flags[id - p_begin] = 1;
    }
    __syncwarp();

    auto phys = [&](int page) -> long long {
        return p.page_table ? static_cast<long long>(p.page_table[static_cast<long long>(b) * p.max_pages + page]) * p.hkv + kvh
                            : static_cast<long long>(h) * p.cap_pages + page;
    };

    // ---- query fragments (B operands) ----
    // FP4: per span s (32 channels) and chunk c: b0b1 <- codes 8t+4c+{0,1}, b2b3 <- +{2,3} of head gl
    uint32_t qb4[4][2][2];
    float qscale[2][4];  // MX: scale of heads 2t, 2t+1 per span
    uint32_t qb16[8][2];
    {
        const bool live = gl < G;
        const uint8_t* qrow = p.q4 + (static_cast<long long>(h) * G + gl) * (D / 2);
        const uint8_t* qsr = p.qs + (static_cast<long long>(h) * G + gl) * SPR;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
            uint32_t w = live ? *reinterpret_cast<const uint32_t*>(qrow + s * 16 + 4 * t) : 0u;
            uint32_t a0[4], a1[4];
            uint32_t sc = 0;
            if (!MX && live) sc = scale_to_h2<false>(qsr[2 * s + (t >> 1)]);
            word_to_frags(w, 0u, sc, sc, !MX, a0, a1);
            qb4[s][0][0] = a0[0]; qb4[s][0][1] = a0[2];
            qb4[s][1][0] = a1[0]; qb4[s][1][1] = a1[2];
        }
        if (MX) {
#pragma unroll
            for (int e = 0; e < 2; ++e)
#pragma unroll
                for (int s = 0; s < 4; ++s) {
                    const int head = 2 * t + e;
                    qscale[e][s] = head < G ? decode_scale<true>(p.qs[(static_cast<long long>(h) * G + head) * SPR + s]) : 0.0f;
                }
        }
        const uint16_t* qh = p.q_hi ? p.q_hi + (static_cast<long long>(h) * G + gl) * D : nullptr;
#pragma unroll
        for (int kc = 0; kc < 8; ++kc) {
            qb16[kc][0] = (live && qh) ? *reinterpret_cast<const uint32_t*>(qh + kc * 16 + 2 * t) : 0u;
            qb16[kc][1] = (live && qh) ? *reinterpret_cast<const uint32_t*>(qh + kc * 16 + 8 + 2 * t) : 0u;
        }
    }

    // ---- running state for heads 2t and 2t+1 ----
    float m_run[2] = {-FLT_MAX, -FLT_MAX}, l_run[2] = {0.0f, 0.0f};
    float o[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) o[i][j] = 0.0f;

    __half* ptile = reinterpret_cast<__half*>(sm + WarpSmem::PT);

    // ================= FP4 pages =================
    auto issue_fp4 = [&](int page, int buf) {
        const long long pp = phys(page);
        const uint8_t* ksrc = p.k4 + pp * (PAGE * D / 2);
        uint8_t* kdst = sm + WarpSmem::K4 + buf * PAGE * KROW;
        for (int i = lane; i < PAGE * 4; i += 32) cp16(kdst + (i >> 2) * KROW + (i & 3) * 16, ksrc + i * 16);
        const uint8_t* kssrc = p.ks + pp * (PAGE * SPR);
        uint8_t* ksdst = sm + WarpSmem::KS + buf * PAGE * 8;
        for (int i = lane; i < PAGE * SPR / 16; i += 32) cp16(ksdst + i * 16, kssrc + i * 16);
        const uint8_t* vsrc;
        const uint8_t* vssrc;
        if (p.page_table) {
            vsrc = p.v4 + pp * (D * 32);
            vssrc = p.vs + pp * (D * (PAGE / GRP));
        } else {
            vsrc = p.v4 + static_cast<long long>(h) * p.v_head_stride + static_cast<long long>(page) * 32;
            vssrc = p.vs + static_cast<long long>(h) * p.vs_head_stride + static_cast<long long>(page) * (PAGE / GRP);
        }
        uint8_t* vdst = sm + WarpSmem::V4 + buf * 128 * VROW;
        for (int i = lane; i < D * 2; i += 32)
            cp16(vdst + (i >> 1) * VROW + (i & 1) * 16, vsrc + static_cast<long long>(i >> 1) * p.v_row_stride + (i & 1) * 16);
        uint8_t* vsdst = sm + WarpSmem::VS + buf * 128 * 4;
        if (p.page_table) {
            // pooled pages keep the scale bytes of a page contiguous
            for (int i = lane; i < D * (PAGE / GRP) / 16; i += 32) cp16(vsdst + i * 16, vssrc + i * 16);
        } else if (MX) {
            // two scale bytes per channel row: fetch the aligned 4-byte word that holds them
            for (int i = lane; i < D; i += 32) {
                const uint8_t* src = vssrc + static_cast<long long>(i) * p.vs_row_stride;
                cp4(vsdst + i * 4, reinterpret_cast<const uint8_t*>(reinterpret_cast<uintptr_t>(src) & ~static_cast<uintptr_t>(3)));
            }
        } else {
            for (int i = lane; i < D; i += 32) cp4(vsdst + i * 4, vssrc + static_cast<long long>(i) * p.vs_row_stride);
        }
        cp_commit();
    };

    // first non-selected page
    int cur = p_begin;
    while (cur < p_end && flags[cur - p_begin]) ++cur;
    int buf = 0;
    if (cur < p_end) issue_fp4(cur, 0);
    while (cur < p_end) {
        int nxt = cur + 1;
        while (nxt < p_end && flags[nxt - p_begin]) ++nxt;
        if (nxt < p_end) { issue_fp4(nxt, buf ^ 1); cp_wait<1>(); } else { cp_wait<0>(); }
        __syncwarp();
        const uint8_t* ksm = sm + WarpSmem::K4 + buf * PAGE * KROW;
        const uint8_t* kss = sm + WarpSmem::KS + buf * PAGE * 8;
        const uint8_t* vsm = sm + WarpSmem::V4 + buf * 128 * VROW;
        const uint8_t* vss = sm + WarpSmem::VS + buf * 128 * 4;
        // in the MX contiguous layout the two V scale bytes may sit in either half of the fetched word
        const int vs_off = (MX && !p.page_table) ? ((cur * (PAGE / GRP)) & 3) : 0;
        const int vs_srow = p.page_table ? (PAGE / GRP) : 4;  // bytes per channel row in the staged scales

        // ---- S^T = K Q^T : 4 tiles of 16 tokens ----
        float s_acc[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[mt][j] = 0.0f;
            const int r_lo = mt * 16 + gl, r_hi = r_lo + 8;
#pragma unroll
            for (int s = 0; s < 4; ++s) {
                const uint32_t w_lo = *reinterpret_cast<const uint32_t*>(ksm + r_lo * KROW + s * 16 + 4 * t);
                const uint32_t w_hi = *reinterpret_cast<const uint32_t*>(ksm + r_hi * KROW + s * 16 + 4 * t);
                uint32_t a0[4], a1[4];
                if (!MX) {
                    const uint32_t sc_lo = scale_to_h2<false>(kss[r_lo * 8 + 2 * s + (t >> 1)]);
                    const uint32_t sc_hi = scale_to_h2<false>(kss[r_hi * 8 + 2 * s + (t >> 1)]);
                    word_to_frags(w_lo, w_hi, sc_lo, sc_hi, true, a0, a1);
                    mma_f16_16816(s_acc[mt], a0, qb4[s][0][0], qb4[s][0][1]);
                    mma_f16_16816(s_acc[mt], a1, qb4[s][1][0], qb4[s][1][1]);
                } else {
                    word_to_frags(w_lo, w_hi, 0u, 0u, false, a0, a1);
                    float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_f16_16816(tmp, a0, qb4[s][0][0], qb4[s][0][1]);
                    mma_f16_16816(tmp, a1, qb4[s][1][0], qb4[s][1][1]);
                    const float k_lo = decode_scale<true>(kss[r_lo * 4 + s]), k_hi = decode_scale<true>(kss[r_hi * 4 + s]);
                    s_acc[mt][0] = fmaf(tmp[0], k_lo * qscale[0][s], s_acc[mt][0]);
                    s_acc[mt][1] = fmaf(tmp[1], k_lo * qscale[1][s], s_acc[mt][1]);
                    s_acc[mt][2] = fmaf(tmp[2], k_hi * qscale[0][s], s_acc[mt][2]);
                    s_acc[mt][3] = fmaf(tmp[3], k_hi * qscale[1][s], s_acc[mt][3]);
                }
            }
        }
        // ---- online softmax over the 64 tokens, per head (columns 2t, 2t+1) ----
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[mt][j] *= p.sm_scale;
            mx[0] = fmaxf(mx[0], fmaxf(s_acc[mt][0], s_acc[mt][2]));
            mx[1] = fmaxf(mx[1], fmaxf(s_acc[mt][1], s_acc[mt][3]));
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 4));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 8));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 16));
        }
        float resc[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float m_new = fmaxf(m_run[e], mx[e]);
            resc[e] = __expf(m_run[e] - m_new);
            m_run[e] = m_new;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { o[i][0] *= resc[0]; o[i][1] *= resc[1]; o[i][2] *= resc[0]; o[i][3] *= resc[1]; }
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            s_acc[mt][0] = __expf(s_acc[mt][0] - m_run[0]); s_acc[mt][2] = __expf(s_acc[mt][2] - m_run[0]);
            s_acc[mt][1] = __expf(s_acc[mt][1] - m_run[1]); s_acc[mt][3] = __expf(s_acc[mt][3] - m_run[1]);
            sum[0] += s_acc[mt][0] + s_acc[mt][2];
            sum[1] += s_acc[mt][1] + s_acc[mt][3];
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 4);
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 8);
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 16);
            l_run[e] = l_run[e] * resc[e] + sum[e];
        }
        // ---- P quantisation: dynamic scale per head and GRP tokens ----
        float p_scale_mx[2][2];  // MX: decoded scale per head and 32-token span
        constexpr int TILES_PER_GRP = GRP / 16;
#pragma unroll
        for (int g0 = 0; g0 < 4; g0 += TILES_PER_GRP) {
            float amax[2] = {0.0f, 0.0f};
#pragma unroll
            for (int mt = g0; mt < g0 + TILES_PER_GRP; ++mt) {
#pragma unroll
                for (int j = 0; j < 4; ++j) s_acc[mt][j] *= C;
                amax[0] = fmaxf(amax[0], fmaxf(s_acc[mt][0], s_acc[mt][2]));
                amax[1] = fmaxf(amax[1], fmaxf(s_acc[mt][1], s_acc[mt][3]));
            }
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                amax[e] = fmaxf(amax[e], __shfl_xor_sync(0xFFFFFFFFu, amax[e], 4));
                amax[e] = fmaxf(amax[e], __shfl_xor_sync(0xFFFFFFFFu, amax[e], 8));
                amax[e] = fmaxf(amax[e], __shfl_xor_sync(0xFFFFFFFFu, amax[e], 16));
            }
            float inv[2], deq[2];
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float sfp = __fdiv_rn(amax[e], 6.0f);
                inv[e] = __fdiv_rn(1.0f, sfp);
                deq[e] = decode_scale<MX>(encode_scale<MX>(sfp));
                if (MX) p_scale_mx[e][g0 / 2] = deq[e];
            }
#pragma unroll
            for (int mt = g0; mt < g0 + TILES_PER_GRP; ++mt) {
                // codes for (token gl / gl+8, heads 2t / 2t+1)
                const uint32_t c_lo = e2m1x2(s_acc[mt][0] * inv[0], s_acc[mt][1] * inv[1]);
                const uint32_t c_hi = e2m1x2(s_acc[mt][2] * inv[0], s_acc[mt][3] * inv[1]);
                const float v00 = e2m1_to_f(c_lo & 15u), v01 = e2m1_to_f(c_lo >> 4);
                const float v10 = e2m1_to_f(c_hi & 15u), v11 = e2m1_to_f(c_hi >> 4);
                const float d0 = MX ? 1.0f : deq[0], d1 = MX ? 1.0f : deq[1];
                const bool z0 = deq[0] == 0.0f, z1 = deq[1] == 0.0f;
                // staging tile: P[head][token]
                ptile[(2 * t) * PROW + mt * 16 + gl] = __float2half_rn(z0 ? 0.0f : v00 * d0);
                ptile[(2 * t + 1) * PROW + mt * 16 + gl] = __float2half_rn(z1 ? 0.0f : v01 * d1);
                ptile[(2 * t) * PROW + mt * 16 + gl + 8] = __float2half_rn(z0 ? 0.0f : v10 * d0);
                ptile[(2 * t + 1) * PROW + mt * 16 + gl + 8] = __float2half_rn(z1 ? 0.0f : v11 * d1);
            }
        }
        __syncwarp();
        // ---- O^T += V^T P^T : 8 tiles of 16 channels, 2 spans of 32 tokens ----
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            // B: P[head gl][tokens 32s + 8t + 4c + {0..3}]
            const uint2 pb0 = *reinterpret_cast<const uint2*>(ptile + gl * PROW + 32 * s + 8 * t);
            const uint2 pb1 = *reinterpret_cast<const uint2*>(ptile + gl * PROW + 32 * s + 8 * t + 4);
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                const int r_lo = dt * 16 + gl, r_hi = r_lo + 8;
                const uint32_t w_lo = *reinterpret_cast<const uint32_t*>(vsm + r_lo * VROW + s * 16 + 4 * t);
                const uint32_t w_hi = *reinterpret_cast<const uint32_t*>(vsm + r_hi * VROW + s * 16 + 4 * t);
                uint32_t a0[4], a1[4];
                if (!MX) {
                    const uint32_t sc_lo = scale_to_h2<false>(vss[r_lo * vs_srow + 2 * s + (t >> 1)]);
                    const uint32_t sc_hi = scale_to_h2<false>(vss[r_hi * vs_srow + 2 * s + (t >> 1)]);
                    word_to_frags(w_lo, w_hi, sc_lo, sc_hi, true, a0, a1);
                    mma_f16_16816(o[dt], a0, pb0.x, pb0.y);
                    mma_f16_16816(o[dt], a1, pb1.x, pb1.y);
                } else {
                    word_to_frags(w_lo, w_hi, 0u, 0u, false, a0, a1);
                    float tmp[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    mma_f16_16816(tmp, a0, pb0.x, pb0.y);
                    mma_f16_16816(tmp, a1, pb1.x, pb1.y);
                    const float v_lo = decode_scale<true>(vss[r_lo * vs_srow + vs_off + s]), v_hi = decode_scale<true>(vss[r_hi * vs_srow + vs_off + s]);
                    o[dt][0] = fmaf(tmp[0], v_lo * p_scale_mx[0][s], o[dt][0]);
                    o[dt][1] = fmaf(tmp[1], v_lo * p_scale_mx[1][s], o[dt][1]);
                    o[dt][2] = fmaf(tmp[2], v_hi * p_scale_mx[0][s], o[dt][2]);
                    o[dt][3] = fmaf(tmp[3], v_hi * p_scale_mx[1][s], o[dt][3]);
                }
            }
        }
        __syncwarp();
        cur = nxt;
        buf ^= 1;
    }

    // ================= selected pages (16-bit) =================
    uint8_t* hsm = sm + WarpSmem::H16;
    auto load16 = [&](const uint16_t* base, int page) {
        const uint16_t* src = base + phys(page) * (PAGE * D);  // same capacity stride as the packed K
        for (int i = lane; i < PAGE * 16; i += 32) cp16(hsm + (i >> 4) * HROW + (i & 15) * 16, reinterpret_cast<const uint8_t*>(src) + i * 16);
        cp_commit();
        cp_wait<0>();
        __syncwarp();
    };
    for (int page = p_begin; page < p_end; ++page) {
        if (!flags[page - p_begin]) continue;
        __syncwarp();
        load16(p.k_hi, page);
        float s_acc[4][4];
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[mt][j] = 0.0f;
#pragma unroll
            for (int kc = 0; kc < 8; ++kc) {
                uint32_t a[4];
                const uint8_t* r_lo = hsm + (mt * 16 + gl) * HROW + kc * 32 + 4 * t;
                const uint8_t* r_hi = r_lo + 8 * HROW;
                a[0] = *reinterpret_cast<const uint32_t*>(r_lo);
                a[1] = *reinterpret_cast<const uint32_t*>(r_hi);
                a[2] = *reinterpret_cast<const uint32_t*>(r_lo + 16);
                a[3] = *reinterpret_cast<const uint32_t*>(r_hi + 16);
                if (BF16) mma_bf16_16816(s_acc[mt], a, qb16[kc][0], qb16[kc][1]);
                else mma_f16_16816(s_acc[mt], a, qb16[kc][0], qb16[kc][1]);
            }
        }
        float mx[2] = {-FLT_MAX, -FLT_MAX};
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
#pragma unroll
            for (int j = 0; j < 4; ++j) s_acc[mt][j] *= p.sm_scale;
            mx[0] = fmaxf(mx[0], fmaxf(s_acc[mt][0], s_acc[mt][2]));
            mx[1] = fmaxf(mx[1], fmaxf(s_acc[mt][1], s_acc[mt][3]));
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 4));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 8));
            mx[e] = fmaxf(mx[e], __shfl_xor_sync(0xFFFFFFFFu, mx[e], 16));
        }
        float resc[2], sum[2] = {0.0f, 0.0f};
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const float m_new = fmaxf(m_run[e], mx[e]);
            resc[e] = __expf(m_run[e] - m_new);
            m_run[e] = m_new;
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) { o[i][0] *= resc[0]; o[i][1] *= resc[1]; o[i][2] *= resc[0]; o[i][3] *= resc[1]; }
        __syncwarp();
#pragma unroll
        for (int mt = 0; mt < 4; ++mt) {
            s_acc[mt][0] = __expf(s_acc[mt][0] - m_run[0]); s_acc[mt][2] = __expf(s_acc[mt][2] - m_run[0]);
            s_acc[mt][1] = __expf(s_acc[mt][1] - m_run[1]); s_acc[mt][3] = __expf(s_acc[mt][3] - m_run[1]);
            sum[0] += s_acc[mt][0] + s_acc[mt][2];
            sum[1] += s_acc[mt][1] + s_acc[mt][3];
            // P16 = 16-bit(C p), staged as [head][token]
            uint16_t* pt = reinterpret_cast<uint16_t*>(ptile);
            pt[(2 * t) * PROW + mt * 16 + gl] = In16<BF16>::from_f(s_acc[mt][0] * C);
            pt[(2 * t + 1) * PROW + mt * 16 + gl] = In16<BF16>::from_f(s_acc[mt][1] * C);
            pt[(2 * t) * PROW + mt * 16 + gl + 8] = In16<BF16>::from_f(s_acc[mt][2] * C);
            pt[(2 * t + 1) * PROW + mt * 16 + gl + 8] = In16<BF16>::from_f(s_acc[mt][3] * C);
        }
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 4);
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 8);
            sum[e] += __shfl_xor_sync(0xFFFFFFFFu, sum[e], 16);
            l_run[e] = l_run[e] * resc[e] + sum[e];
        }
        __syncwarp();
        load16(p.v_hi, page);
        // O^T += V^T P^T: A = V^T (channel rows, token k) read transposed from [token][channel]
#pragma unroll
        for (int kc = 0; kc < 4; ++kc) {
            const uint32_t b0 = *reinterpret_cast<const uint32_t*>(ptile + gl * PROW + kc * 16 + 2 * t);
            const uint32_t b1 = *reinterpret_cast<const uint32_t*>(ptile + gl * PROW + kc * 16 + 8 + 2 * t);
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                uint32_t a[4];
                // ldmatrix.trans: four 8x8 blocks of [token][channel] -> A fragment of V^T
                const int blk = lane >> 3, rr = lane & 7;
                const int tok = kc * 16 + (blk >> 1) * 8 + rr;
                const int ch = dt * 16 + (blk & 1) * 8;
                const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(hsm + tok * HROW + ch * 2));
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
                if (BF16) mma_bf16_16816(o[dt], a, b0, b1);
                else mma_f16_16816(o[dt], a, b0, b1);
            }
        }
    }

    // ---- partial results: O (units of C), m, l ----
    float* po = p.part_o + (static_cast<long long>(h) * p.splits + split) * G * D;
    float* pml = p.part_ml + (static_cast<long long>(h) * p.splits + split) * G * 2;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int head = 2 * t + e;
        if (head < G) {
#pragma unroll
            for (int dt = 0; dt < 8; ++dt) {
                po[head * D + dt * 16 + gl] = o[dt][e];
                po[head * D + dt * 16 + gl + 8] = o[dt][2 + e];
            }
            if (gl == 0) { pml[head * 2] = m_run[e]; pml[head * 2 + 1] = l_run[e]; }
        }
    }
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

}  // namespace

int decode_pick_splits(int heads, int npages) {
    // about two resident waves of single-warp chains (9 per SM) over the whole GPU
    int sms = NUM_SMS_HINT;
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    long long target = 2LL * 9 * sms;
    int splits = static_cast<int>((target + heads - 1) / (heads > 0 ? heads : 1));
    if (splits > npages) splits = npages;
    if (splits > 64) splits = 64;
    if (splits < 1) splits = 1;
    return splits;
}

size_t decode_workspace_bytes(int heads, int G, int d, int splits) {
    return static_cast<size_t>(heads) * splits * G * (d + 2) * sizeof(float);
}

// See include/thrift_sm100.h (ta100_decode_attention).
int decode_dispatch(const void* q_hi, const void* k_hi, const void* v_hi, const void* sel, int width, const void* q4,
                    const void* k4, const void* v4, const void* qs, const void* ks, const void* vs, const void* page_table,
                    int max_pages, void* out, void* part_o, void* part_ml, int batch, int hkv, int G, int kv_len, int kv_cap,
                    int d, int is_mx, int is_bf16, int splits, int write_out, cudaStream_t stream) {
    if (!q4 || !k4 || !v4 || !qs || !ks || !vs || !part_o || !part_ml) return TA100_ERR_NULL;
    if (write_out && !out) return TA100_ERR_NULL;
    if (width > 0 && (!q_hi || !k_hi || !v_hi || !sel)) return TA100_ERR_NULL;
    if (d != 128) return TA100_ERR_UNSUPPORTED;
    if (G < 1 || G > 8) return TA100_ERR_UNSUPPORTED;
    if (batch <= 0 || hkv <= 0 || kv_len <= 0 || kv_len % PAGE != 0 || kv_cap < kv_len) return TA100_ERR_SHAPE;
    if (!page_table && kv_cap % PAGE != 0) return TA100_ERR_SHAPE;
    const int heads = batch * hkv;
    const int npages = kv_len / PAGE;
    if (npages > 2048) return TA100_ERR_LIMIT;
    if (splits < 1 || splits > npages) return TA100_ERR_SHAPE;
    const int GRP = is_mx ? 32 : 16;
    const int P = cdiv(kv_cap, 128) * 128;
    DecodeParams p;
    p.q_hi = static_cast<const uint16_t*>(q_hi); p.q4 = static_cast<const uint8_t*>(q4); p.qs = static_cast<const uint8_t*>(qs);
    p.k4 = static_cast<const uint8_t*>(k4); p.ks = static_cast<const uint8_t*>(ks);
    p.v4 = static_cast<const uint8_t*>(v4); p.vs = static_cast<const uint8_t*>(vs);
    p.k_hi = static_cast<const uint16_t*>(k_hi); p.v_hi = static_cast<const uint16_t*>(v_hi);
    p.sel = static_cast<const int32_t*>(sel); p.page_table = static_cast<const int32_t*>(page_table);
    p.part_o = static_cast<float*>(part_o); p.part_ml = static_cast<float*>(part_ml);
    p.heads = heads; p.hkv = hkv; p.G = G; p.npages = npages; p.cap_pages = kv_cap / PAGE; p.max_pages = max_pages;
    p.width = width; p.splits = splits;
    if (page_table) {
        p.v_head_stride = 0; p.vs_head_stride = 0; p.v_row_stride = 32; p.vs_row_stride = PAGE / GRP;
    } else {
        p.v_head_stride = static_cast<long long>(d) * (P / 2); p.vs_head_stride = static_cast<long long>(d) * (P / GRP);
        p.v_row_stride = P / 2; p.vs_row_stride = P / GRP;
    }
    p.sm_scale = static_cast<float>(1.0 / sqrt(static_cast<double>(d)));
    const dim3 grid(splits, heads);
    const int smem = WarpSmem::TOTAL;
#define TA100_DEC(MXX, BFF)                                                                               \
    do {                                                                                                  \
        cudaFuncSetAttribute(decode_kernel<MXX, BFF>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem); \
        decode_kernel<MXX, BFF><<<grid, 32, smem, stream>>>(p);                                           \
    } while (0)
    if (is_mx) { if (is_bf16) TA100_DEC(true, true); else TA100_DEC(true, false); }
    else { if (is_bf16) TA100_DEC(false, true); else TA100_DEC(false, false); }
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
int merge_dispatch(const void* part_o, const void* part_ml, void* out, int shards, long long heads, int splits, int G, int d,
                   int is_mx, int is_bf16, cudaStream_t stream) {
    if (!part_o || !part_ml || !out) return TA100_ERR_NULL;
    if (d > 128 || shards < 1 || splits < 1) return TA100_ERR_SHAPE;
    const long long rows = heads * G;
    if (rows == 0) return TA100_OK;
    const long long so = heads * splits * G * d, sml = heads * splits * G * 2;
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
                           const void* page_table, int max_pages, void* out, int batch, int hkv, int G, int kv_len,
                           int kv_cap, int d, int is_mx, int is_bf16, int splits, cudaStream_t stream) {
    if (batch <= 0 || hkv <= 0 || G <= 0 || splits <= 0 || d <= 0) return TA100_ERR_SHAPE;
    const size_t n_o = static_cast<size_t>(batch) * hkv * splits * G * d * sizeof(float);
    const size_t n_ml = static_cast<size_t>(batch) * hkv * splits * G * 2 * sizeof(float);
    const size_t off_ml = (n_o + 255) & ~static_cast<size_t>(255);
    if (off_ml + n_ml > STATIC_SCRATCH_BYTES) return TA100_ERR_STATIC_SCRATCH;
    void* base = nullptr;
    const int rc = static_scratch_address(&base);
    if (rc != TA100_OK) return rc;
    unsigned char* b = static_cast<unsigned char*>(base);
    return decode_dispatch(q_hi, k_hi, v_hi, sel, width, q4, k4, v4, qs, ks, vs, page_table, max_pages, out, b, b + off_ml,
                           batch, hkv, G, kv_len, kv_cap, d, is_mx, is_bf16, splits, 1, stream);
}

}  // namespace ta100
