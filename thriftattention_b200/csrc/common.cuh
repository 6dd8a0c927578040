// Shared device helpers: 16-bit input traits, exact FP4 / FP8 scale codecs and
// the status codes every C-ABI entry point returns.
#pragma once

#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

namespace ta100 {

// Return codes of the C ABI: 0 ok, negative = argument errors, positive = cudaError_t.
enum Status : int {
    TA100_OK = 0,
    TA100_ERR_NULL = -1,
    TA100_ERR_SHAPE = -2,
    TA100_ERR_UNSUPPORTED = -3,
    TA100_ERR_ALIGN = -4,
    TA100_ERR_WORKSPACE = -5,
    TA100_ERR_TENSOR_MAP = -6,
    TA100_ERR_DEVICE_TIMEOUT = -7,
    TA100_ERR_LIMIT = -8,
    TA100_ERR_STATIC_SCRATCH = -9,
    TA100_ERR_PAGE_TABLE = -10,
};

constexpr int NUM_SMS_HINT = 148;

// Diagnostics (see ta100_debug_set_wait): the cycle budget of every bounded device-side wait, and a switch that
// makes the producer warps of the attention kernels issue no copies at all, so that the consumers' waits run
// out with nothing asynchronous in flight - the only way to exercise the give-up path without a fault.
constexpr long long DEFAULT_WAIT_BUDGET = 1000000000LL;
extern long long g_wait_budget_cycles;
extern int g_test_skip_loads;

__host__ __device__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }

// Sequence length kept in DEVICE memory.  A generation loop whose launches must not change from token to token
// (one CUDA graph replayed for every token) stores the number of tokens in the cache in one int32 on the GPU;
// the append, selection and attention kernels read it when they start and derive from it what the host
// otherwise passes as launch parameters.  len == nullptr: the launch parameters hold.
struct DynLength {
    const int32_t* len;   // tokens in the cache when the step began (before its append): one int, or one per sequence
    int hkv_per_seq;      // 0: len[0] holds for every sequence; else KV heads per sequence - flat KV head h reads len[h / hkv_per_seq]
    int offset;           // added to the length: the tokens this step has appended before the reading kernel runs
    int top_k;            // >= 0: that many blocks (at most the complete ones); < 0: `share` of them
    double share;         // fraction of the complete 64-token blocks that are selected
    int sink, local;      // configured numbers of forced first / last blocks
};

__host__ __device__ inline long long round_half_even(double x) {
#ifdef __CUDA_ARCH__
    return __double2ll_rn(x);
#else
    const double f = static_cast<double>(static_cast<long long>(x));   // x >= 0 here
    const double r = x - f;
    long long v = static_cast<long long>(f);
    if (r > 0.5 || (r == 0.5 && (v & 1))) ++v;
    return v;
#endif
}

// Blocks scored (n), selected by score (k) and forced (sink, local) for `tokens` cached tokens: the rule of the
// cache's decode step - k = top_k or max(1, round-half-even(share * n)) capped by n; the last `local` and first
// `sink` blocks are forced as far as n - k leaves room, local first; nothing is forced when k == 0.
__host__ __device__ inline void dyn_select_counts(const DynLength& d, int tokens, int max_blocks, int& n, int& k, int& sink,
                                                  int& local) {
    n = tokens / 64;
    if (n > max_blocks) n = max_blocks;
    if (n < 0) n = 0;
    if (d.top_k >= 0) k = d.top_k < n ? d.top_k : n;
    else if (n <= 0 || !(d.share > 0.0)) k = 0;
    else if (d.share >= 1.0) k = n;
    else {
        long long r = round_half_even(d.share * static_cast<double>(n));
        if (r > n) r = n;
        if (r < 1) r = 1;
        k = static_cast<int>(r);
    }
    local = d.local < n - k ? d.local : n - k;
    if (local < 0) local = 0;
    sink = d.sink < n - k - local ? d.sink : n - k - local;
    if (sink < 0) sink = 0;
    if (k == 0) { sink = 0; local = 0; }
}

// Row permutation inside every group of 32 rows used by the "permuted" K layout.
__host__ __device__ constexpr int perm32(int x) { return (x / 8) * 2 + ((x % 8) / 2) * 8 + (x % 2); }

template <bool BF16>
struct In16;
template <>
struct In16<false> {
    using T = __half;
    using T2 = __half2;
    static __device__ __forceinline__ float to_f(uint16_t b) { return __half2float(__ushort_as_half(b)); }
    static __device__ __forceinline__ uint16_t from_f(float f) { return __half_as_ushort(__float2half_rn(f)); }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};
template <>
struct In16<true> {
    using T = __nv_bfloat16;
    using T2 = __nv_bfloat162;
    static __device__ __forceinline__ float to_f(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
    static __device__ __forceinline__ uint16_t from_f(float f) {
        return __bfloat16_as_ushort(__float2bfloat16_rn(f));
    }
    static __device__ __forceinline__ uint32_t pack2(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
};

// Two floats -> one byte of e2m1 codes: `lo` in bits 0..3, `hi` in bits 4..7.
// Round-to-nearest-even, saturating.
__device__ __forceinline__ uint32_t e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{\n\t"
        ".reg .b8 b;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b, %1, %2;\n\t"
        "cvt.u32.u8 %0, b;\n\t"
        "}\n"
        : "=r"(r)
        : "f"(hi), "f"(lo));
    return r;
}

// Eight floats (ascending element order) -> 32-bit word of packed e2m1.
__device__ __forceinline__ uint32_t e2m1x8(float v0, float v1, float v2, float v3, float v4, float v5, float v6,
                                           float v7) {
    uint32_t r;
    asm("{\n\t"
        ".reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3};\n\t"
        "}\n"
        : "=r"(r)
        : "f"(v0), "f"(v1), "f"(v2), "f"(v3), "f"(v4), "f"(v5), "f"(v6), "f"(v7));
    return r;
}

// Scale codecs.  E4M3: round-to-nearest-even, saturate to 448.  E8M0: smallest
// power of two >= x, saturating.
__device__ __forceinline__ uint8_t to_e4m3(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float from_e4m3(uint8_t b) {
    __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(b), __NV_E4M3);
    return __half2float(*reinterpret_cast<__half*>(&h));
}
__device__ __forceinline__ uint8_t to_e8m0(float x) {
    return static_cast<uint8_t>(__nv_cvt_float_to_e8m0(x, __NV_SATFINITE, cudaRoundPosInf));
}
__device__ __forceinline__ float from_e8m0(uint8_t b) {
    return b == 0 ? __uint_as_float(0x00400000u) : __uint_as_float(static_cast<uint32_t>(b) << 23);
}

template <bool MX>
__device__ __forceinline__ uint8_t encode_scale(float x) {
    if constexpr (MX) return to_e8m0(x);
    else return to_e4m3(x);
}
template <bool MX>
__device__ __forceinline__ float decode_scale(uint8_t b) {
    if constexpr (MX) return from_e8m0(b);
    else return from_e4m3(b);
}

// e2m1 code (4 bits) -> float.
__device__ __forceinline__ float e2m1_to_f(uint32_t c) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6
    const uint32_t mag = c & 7u;
    const float v = (mag == 0)   ? 0.0f
                    : (mag == 1) ? 0.5f
                                 : __uint_as_float(((126u + (mag >> 1)) << 23) | ((mag & 1u) << 22));
    return (c & 8u) ? -v : v;
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// One quantisation group (G = 16 NVFP4 / 32 MXFP4 values held as G/2 words of two 16-bit inputs):
// amax -> scale byte -> reciprocal of the DECODED scale -> e2m1 codes, all IEEE fp32.
template <bool MX, bool BF16>
__device__ __forceinline__ void quantise_group_regs(const uint32_t* raw /* G/2 words of 2x16-bit */,
                                                    uint32_t* codes /* G/8 words */, uint8_t& scale_byte) {
    constexpr int G = MX ? 32 : 16;
    float v[G];
    float amax = 0.0f;
#pragma unroll
    for (int i = 0; i < G / 2; ++i) {
        v[2 * i] = In16<BF16>::to_f(static_cast<uint16_t>(raw[i] & 0xFFFFu));
        v[2 * i + 1] = In16<BF16>::to_f(static_cast<uint16_t>(raw[i] >> 16));
        amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
    }
    const float sf = __fdiv_rn(amax, 6.0f);
    scale_byte = encode_scale<MX>(sf);
    const float sfq = decode_scale<MX>(scale_byte);
    const float inv = (sfq == 0.0f) ? 0.0f : __fdiv_rn(1.0f, sfq);
#pragma unroll
    for (int w = 0; w < G / 8; ++w) {
        codes[w] = e2m1x8(__fmul_rn(v[8 * w + 0], inv), __fmul_rn(v[8 * w + 1], inv), __fmul_rn(v[8 * w + 2], inv),
                          __fmul_rn(v[8 * w + 3], inv), __fmul_rn(v[8 * w + 4], inv), __fmul_rn(v[8 * w + 5], inv),
                          __fmul_rn(v[8 * w + 6], inv), __fmul_rn(v[8 * w + 7], inv));
    }
}

inline int grid_for(long long work_items, int threads, int per_sm) {
    long long blocks = (work_items + threads - 1) / threads;
    long long cap = static_cast<long long>(NUM_SMS_HINT) * per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return static_cast<int>(blocks);
}

}  // namespace ta100
