// NVFP4 / MXFP4 quantisers for Q, K (row layouts) and V (transposed layout).
//
// Arithmetic per group of G = 16 (NVFP4) or 32 (MXFP4) values, all IEEE fp32:
//   amax = max|x|; sf = amax / 6; byte = E4M3_rn_sat(sf) | E8M0_ceil_pow2(sf);
//   inv = decoded(byte) == 0 ? 0 : 1 / decoded(byte); code = e2m1_rn_sat(x * inv).
// Byte i of a group holds element 2i in the low nibble and 2i+1 in the high one.
// These kernels are bandwidth bound: 128-bit loads and stores, grids sized in
// multiples of the SM count with grid-stride loops.
#include "common.cuh"

namespace ta100 {

// Row layouts.  x [bs, seq, d] -> codes [bs, seq, d/2], scales [bs, seq, d/G].
// One thread per group; consecutive threads take consecutive groups so loads,
// code stores and scale stores are all contiguous across a warp.
// `cta` of `n_cta` CTAs work on the tensor (the whole grid, or the part of a fused launch that is given to it).
template <bool MX, bool BF16, bool PERMUTED>
__device__ __forceinline__ void quantize_rows_body(const uint16_t* __restrict__ x, uint8_t* __restrict__ codes,
                                                   uint8_t* __restrict__ scales, long long bs_seq, int seq, int d,
                                                   unsigned cta, unsigned n_cta) {
    constexpr int G = MX ? 32 : 16;
    const int groups_per_row = d / G;
    const long long total = bs_seq * groups_per_row;
    for (long long gid = cta * static_cast<long long>(blockDim.x) + threadIdx.x; gid < total;
         gid += static_cast<long long>(n_cta) * blockDim.x) {
        const long long row = gid / groups_per_row;
        const int c = static_cast<int>(gid - row * groups_per_row);
        long long src_row = row;
        bool valid = true;
        if constexpr (PERMUTED) {
            const long long b = row / seq;
            const int p = static_cast<int>(row - b * seq);
            const int logical = (p / 32) * 32 + perm32(p % 32);
            valid = logical < seq;
            src_row = b * seq + logical;
        }
        uint32_t raw[G / 2];
        if (valid) {
            const uint4* src = reinterpret_cast<const uint4*>(x + src_row * d + c * G);
#pragma unroll
            for (int i = 0; i < G / 8; ++i) {
                const uint4 t = __ldg(src + i);
                raw[4 * i + 0] = t.x; raw[4 * i + 1] = t.y; raw[4 * i + 2] = t.z; raw[4 * i + 3] = t.w;
            }
        } else {
#pragma unroll
            for (int i = 0; i < G / 2; ++i) raw[i] = 0;
        }
        uint32_t out[G / 8];
        uint8_t sb;
        quantise_group_regs<MX, BF16>(raw, out, sb);
        if constexpr (MX) {
            *reinterpret_cast<uint4*>(codes + gid * 16) = make_uint4(out[0], out[1], out[2], out[3]);
        } else {
            *reinterpret_cast<uint2*>(codes + gid * 8) = make_uint2(out[0], out[1]);
        }
        scales[gid] = sb;
    }
}

template <bool MX, bool BF16, bool PERMUTED>
__global__ void __launch_bounds__(256) quantize_rows_kernel(const uint16_t* __restrict__ x,
                                                            uint8_t* __restrict__ codes,
                                                            uint8_t* __restrict__ scales, long long bs_seq,
                                                            int seq, int d) {
    quantize_rows_body<MX, BF16, PERMUTED>(x, codes, scales, bs_seq, seq, d, blockIdx.x, gridDim.x);
}

// Transposed layout for V.  x [bs, seq, d] -> codes [bs, d, P/2], scales [bs, d, P/G],
// P = ceil(seq/128)*128; groups run along the sequence; rows >= seq are zero.
// One CTA stages a 128-token x d tile in shared memory, quantises down the
// columns and stages the packed result so that global stores are 16-byte wide
// and contiguous per channel row.
template <int D, bool MX, bool BF16, bool PERMUTED>
__device__ __forceinline__ void quantize_transposed_body(const uint16_t* __restrict__ x, uint8_t* __restrict__ codes,
                                                         uint8_t* __restrict__ scales, int bs, int seq, int padded,
                                                         unsigned cta, unsigned n_cta) {
    constexpr int G = MX ? 32 : 16;
    constexpr int TOK = 128;
    constexpr int GROUPS = TOK / G;  // per channel per tile
    // +2 element pad per row keeps the column reads conflict free
    __shared__ __align__(16) uint16_t tile[TOK][D + 8];
    __shared__ __align__(16) uint8_t out_codes[D][TOK / 2];
    __shared__ __align__(16) uint8_t out_scales[D][8];

    const int tiles_per_b = padded / TOK;
    for (int work = cta; work < bs * tiles_per_b; work += n_cta) {
        const int b = work / tiles_per_b;
        const int t = work - b * tiles_per_b;
        const int tok0 = t * TOK;
        // ---- load ----
        constexpr int VEC_PER_ROW = D / 8;
        for (int i = threadIdx.x; i < TOK * VEC_PER_ROW; i += blockDim.x) {
            const int r = i / VEC_PER_ROW, cv = i % VEC_PER_ROW;
            const int p = tok0 + r;
            int src = p;
            bool valid = p < seq;
            if constexpr (PERMUTED) {
                src = (p / 32) * 32 + perm32(p % 32);
                valid = valid && (src < seq);
            }
            uint4 val = make_uint4(0, 0, 0, 0);
            if (valid) val = __ldg(reinterpret_cast<const uint4*>(x + (static_cast<long long>(b) * seq + src) * D) + cv);
            *reinterpret_cast<uint4*>(&tile[r][cv * 8]) = val;
        }
        __syncthreads();
        // ---- quantise down the columns ----
        for (int i = threadIdx.x; i < D * GROUPS; i += blockDim.x) {
            const int ch = i % D, grp = i / D;
            uint32_t raw[G / 2];
#pragma unroll
            for (int j = 0; j < G / 2; ++j) {
                const uint32_t lo = tile[grp * G + 2 * j][ch];
                const uint32_t hi = tile[grp * G + 2 * j + 1][ch];
                raw[j] = lo | (hi << 16);
            }
            uint32_t out[G / 8];
            uint8_t sb;
            quantise_group_regs<MX, BF16>(raw, out, sb);
#pragma unroll
            for (int w = 0; w < G / 8; ++w) *reinterpret_cast<uint32_t*>(&out_codes[ch][grp * (G / 2) + 4 * w]) = out[w];
            out_scales[ch][grp] = sb;
        }
        __syncthreads();
        // ---- store ----
        for (int i = threadIdx.x; i < D * 4; i += blockDim.x) {
            const int ch = i / 4, part = i % 4;
            const uint4 val = *reinterpret_cast<const uint4*>(&out_codes[ch][part * 16]);
            *reinterpret_cast<uint4*>(codes + (static_cast<long long>(b) * D + ch) * (padded / 2) + tok0 / 2 + part * 16) = val;
        }
        for (int i = threadIdx.x; i < D; i += blockDim.x) {
            uint8_t* dst = scales + (static_cast<long long>(b) * D + i) * (padded / G) + tok0 / G;
            if constexpr (MX) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(&out_scales[i][0]);
            else *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(&out_scales[i][0]);
        }
        __syncthreads();
    }
}

template <int D, bool MX, bool BF16, bool PERMUTED>
__global__ void __launch_bounds__(256) quantize_transposed_kernel(const uint16_t* __restrict__ x,
                                                                  uint8_t* __restrict__ codes,
                                                                  uint8_t* __restrict__ scales, int bs, int seq,
                                                                  int padded) {
    quantize_transposed_body<D, MX, BF16, PERMUTED>(x, codes, scales, bs, seq, padded, blockIdx.x, gridDim.x);
}

// Q, K and V of one attention call in ONE launch: the grid is split into three parts, each running one of the
// bodies above on its tensor (Q rows, K rows - permuted for the prefill kernel, plain for decode - and V transposed).
struct QkvParams {
    const uint16_t *q, *k, *v;
    uint8_t *q_codes, *q_scales, *k_codes, *k_scales, *v_codes, *v_scales;
    long long q_rows, k_rows;   // bs * seq of Q and of K
    int seq_q, seq_kv, bs_kv, padded_kv, d;
    unsigned n_q, n_k, n_v;     // CTAs per part
};

template <int D, bool MX, bool BF16, bool KPERM>
__global__ void __launch_bounds__(256) quantize_qkv_kernel(const QkvParams p) {
    const unsigned b = blockIdx.x;
    if (b < p.n_q)
        quantize_rows_body<MX, BF16, false>(p.q, p.q_codes, p.q_scales, p.q_rows, p.seq_q, p.d, b, p.n_q);
    else if (b < p.n_q + p.n_k)
        quantize_rows_body<MX, BF16, KPERM>(p.k, p.k_codes, p.k_scales, p.k_rows, p.seq_kv, p.d, b - p.n_q, p.n_k);
    else
        quantize_transposed_body<D, MX, BF16, false>(p.v, p.v_codes, p.v_scales, p.bs_kv, p.seq_kv, p.padded_kv,
                                                     b - p.n_q - p.n_k, p.n_v);
}

template <bool MX, bool BF16>
static int launch_rows(const void* x, void* codes, void* scales, long long bs, int seq, int d, int permuted,
                       cudaStream_t stream) {
    const int G = MX ? 32 : 16;
    const long long total = bs * seq * (d / G);
    if (total == 0) return TA100_OK;
    const int grid = grid_for(total, 256, 16);
    if (permuted)
        quantize_rows_kernel<MX, BF16, true><<<grid, 256, 0, stream>>>(
            static_cast<const uint16_t*>(x), static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales), bs * seq, seq, d);
    else
        quantize_rows_kernel<MX, BF16, false><<<grid, 256, 0, stream>>>(
            static_cast<const uint16_t*>(x), static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales), bs * seq, seq, d);
    return static_cast<int>(cudaGetLastError());
}

template <int D, bool MX, bool BF16>
static int launch_transposed(const void* x, void* codes, void* scales, int bs, int seq, int permuted,
                             cudaStream_t stream) {
    const int padded = cdiv(seq, 128) * 128;
    const long long work = static_cast<long long>(bs) * (padded / 128);
    if (work == 0) return TA100_OK;
    int grid = static_cast<int>(work < NUM_SMS_HINT * 4LL ? work : NUM_SMS_HINT * 4LL);
    if (permuted)
        quantize_transposed_kernel<D, MX, BF16, true><<<grid, 256, 0, stream>>>(
            static_cast<const uint16_t*>(x), static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales), bs, seq, padded);
    else
        quantize_transposed_kernel<D, MX, BF16, false><<<grid, 256, 0, stream>>>(
            static_cast<const uint16_t*>(x), static_cast<uint8_t*>(codes), static_cast<uint8_t*>(scales), bs, seq, padded);
    return static_cast<int>(cudaGetLastError());
}

// layout: 0 plain, 1 permuted, 2 transposed, 3 transposed + permuted
int quantize_dispatch(const void* x, void* codes, void* scales, long long bs, int seq, int d, int is_mx,
                      int is_bf16, int layout, cudaStream_t stream) {
    if (!x || !codes || !scales) return bs * seq == 0 ? TA100_OK : TA100_ERR_NULL;
    if (d != 64 && d != 128) return TA100_ERR_UNSUPPORTED;
    if (layout < 0 || layout > 3 || bs < 0 || seq < 0) return TA100_ERR_SHAPE;
    if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(codes)) & 15) return TA100_ERR_ALIGN;
    const int perm = layout & 1;
    if (layout < 2) {
        if (is_mx) return is_bf16 ? launch_rows<true, true>(x, codes, scales, bs, seq, d, perm, stream)
                                  : launch_rows<true, false>(x, codes, scales, bs, seq, d, perm, stream);
        return is_bf16 ? launch_rows<false, true>(x, codes, scales, bs, seq, d, perm, stream)
                       : launch_rows<false, false>(x, codes, scales, bs, seq, d, perm, stream);
    }
    if (bs > 0x7FFFFFFF) return TA100_ERR_LIMIT;
    const int b = static_cast<int>(bs);
#define TA100_T(DD, MXX, BFF) launch_transposed<DD, MXX, BFF>(x, codes, scales, b, seq, perm, stream)
    if (d == 128) {
        if (is_mx) return is_bf16 ? TA100_T(128, true, true) : TA100_T(128, true, false);
        return is_bf16 ? TA100_T(128, false, true) : TA100_T(128, false, false);
    }
    if (is_mx) return is_bf16 ? TA100_T(64, true, true) : TA100_T(64, true, false);
    return is_bf16 ? TA100_T(64, false, true) : TA100_T(64, false, false);
#undef TA100_T
}

// See include/thrift_sm100.h (ta100_quantize_qkv) for the contract.
int quantize_qkv_dispatch(const void* q, const void* k, const void* v, void* q_codes, void* q_scales, void* k_codes,
                          void* k_scales, void* v_codes_t, void* v_scales_t, long long bs_q, int seq_q, long long bs_kv,
                          int seq_kv, int d, int is_mx, int is_bf16, int k_permuted, cudaStream_t stream) {
    if (!q || !k || !v || !q_codes || !q_scales || !k_codes || !k_scales || !v_codes_t || !v_scales_t) return TA100_ERR_NULL;
    if (d != 64 && d != 128) return TA100_ERR_UNSUPPORTED;
    if (bs_q <= 0 || bs_kv <= 0 || seq_q <= 0 || seq_kv <= 0) return TA100_ERR_SHAPE;
    if (bs_kv > 0x7FFFFFFF) return TA100_ERR_LIMIT;
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
         reinterpret_cast<uintptr_t>(q_codes) | reinterpret_cast<uintptr_t>(k_codes) | reinterpret_cast<uintptr_t>(v_codes_t)) & 15)
        return TA100_ERR_ALIGN;
    const int G = is_mx ? 32 : 16;
    QkvParams p;
    p.q = static_cast<const uint16_t*>(q); p.k = static_cast<const uint16_t*>(k); p.v = static_cast<const uint16_t*>(v);
    p.q_codes = static_cast<uint8_t*>(q_codes); p.q_scales = static_cast<uint8_t*>(q_scales);
    p.k_codes = static_cast<uint8_t*>(k_codes); p.k_scales = static_cast<uint8_t*>(k_scales);
    p.v_codes = static_cast<uint8_t*>(v_codes_t); p.v_scales = static_cast<uint8_t*>(v_scales_t);
    p.q_rows = bs_q * seq_q; p.k_rows = bs_kv * seq_kv;
    p.seq_q = seq_q; p.seq_kv = seq_kv; p.bs_kv = static_cast<int>(bs_kv); p.padded_kv = cdiv(seq_kv, 128) * 128; p.d = d;
    p.n_q = static_cast<unsigned>(grid_for(p.q_rows * (d / G), 256, 16));
    p.n_k = static_cast<unsigned>(grid_for(p.k_rows * (d / G), 256, 16));
    const long long v_work = bs_kv * (p.padded_kv / 128);
    p.n_v = static_cast<unsigned>(v_work < NUM_SMS_HINT * 4LL ? v_work : NUM_SMS_HINT * 4LL);
    const unsigned grid = p.n_q + p.n_k + p.n_v;
#define TA100_QKV(DD, MXX, BFF)                                                                    \
    do {                                                                                           \
        if (k_permuted) quantize_qkv_kernel<DD, MXX, BFF, true><<<grid, 256, 0, stream>>>(p);      \
        else quantize_qkv_kernel<DD, MXX, BFF, false><<<grid, 256, 0, stream>>>(p);                \
    } while (0)
    if (d == 128) {
        if (is_mx) { if (is_bf16) TA100_QKV(128, true, true); else TA100_QKV(128, true, false); }
        else { if (is_bf16) TA100_QKV(128, false, true); else TA100_QKV(128, false, false); }
    } else {
        if (is_mx) { if (is_bf16) TA100_QKV(64, true, true); else TA100_QKV(64, true, false); }
        else { if (is_bf16) TA100_QKV(64, false, true); else TA100_QKV(64, false, false); }
    }
#undef TA100_QKV
    return static_cast<int>(cudaGetLastError());
}

}  // namespace ta100
