/*
 * CPU oracle for the selective mixed-precision attention path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file restates, in plain C, the arithmetic of
 * the reference's CUDA kernels so that the sm_100a kernels can be checked
 * against it.  Nothing in the product path may link or call it.
 *
 * Parity status: the reference's tests pin selection indices (small known
 * answers), resolve_top_k goldens and the local-window closed forms; those are
 * checked in tests/.  Quantised codes, scale bytes and attention values are
 * pinned by no reference test ("parity unpinned" for those): they follow this
 * file's reading of the reference sources cited on each function, with IEEE
 * fp32 division where the reference is compiled with fast-math.
 *
 * Citations are paths inside the reference project.
 */
#include <float.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ------------------------------------------------------------------------- */
/* Scalar formats                                                             */
/* ------------------------------------------------------------------------- */

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

float ora_half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000) << 16;
    int e = (h >> 10) & 31;
    uint32_t m = h & 0x3FF;
    if (e == 0) {
        if (m == 0) return u2f(sign);
        float v = ldexpf((float)m, -24);
        return sign ? -v : v;
    }
    if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
    return u2f(sign | ((uint32_t)(e + 112) << 23) | (m << 13));
}

/* round-to-nearest-even float -> IEEE half */
uint16_t ora_float_to_half(float f) {
    uint32_t x = f2u(f);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00 | ((ax > 0x7F800000u) ? 0x200 : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00); /* rounds to >= 65520 -> inf */
    if (ax < 0x33000001u) return sign;                        /* < 2^-25 (or == 2^-25 tie -> 0) */
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; }
    else { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7FFFFFu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1))) q++;
    return (uint16_t)(sign | (base + q));
}

float ora_bf16_to_float(uint16_t h) { return u2f((uint32_t)h << 16); }

uint16_t ora_float_to_bf16(float f) {
    uint32_t x = f2u(f);
    if ((x & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((x >> 16) | 0x40);
    uint32_t lsb = (x >> 16) & 1;
    x += 0x7FFFu + lsb;
    return (uint16_t)(x >> 16);
}

static inline float in_to_float(uint16_t bits, int is_bf16) {
    return is_bf16 ? ora_bf16_to_float(bits) : ora_half_to_float(bits);
}
static inline uint16_t float_to_out(float f, int is_bf16) {
    return is_bf16 ? ora_float_to_bf16(f) : ora_float_to_half(f);
}

/* e2m1, round-to-nearest-even, saturating; PTX cvt.rn.satfinite.e2m1x2.f32
 * (csrc/include/thriftattention/sm120/cuda_common.cuh:147-167). NaN -> +6. */
uint8_t ora_to_e2m1(float x) {
    if (x != x) return 0x7;
    uint8_t sign = (f2u(x) >> 31) ? 0x8 : 0x0;
    float a = fabsf(x);
    uint8_t c;
    if (a <= 0.25f) c = 0;
    else if (a < 0.75f) c = 1;
    else if (a <= 1.25f) c = 2;
    else if (a < 1.75f) c = 3;
    else if (a <= 2.5f) c = 4;
    else if (a < 3.5f) c = 5;
    else if (a <= 5.0f) c = 6;
    else c = 7;
    return (uint8_t)(sign | c);
}

static const float E2M1_VALUES[16] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f,
                                      -0.0f, -0.5f, -1.0f, -1.5f, -2.0f, -3.0f, -4.0f, -6.0f};
float ora_from_e2m1(uint8_t c) { return E2M1_VALUES[c & 15]; }

/* e4m3 (fn), round-to-nearest-even, saturate-to-finite (448); NaN -> 0x7F.
 * Matches __nv_fp8_e4m3(float) used at csrc/cuda/sm120/nvfp4/quantization.cu:63-65. */
uint8_t ora_to_e4m3(float x) {
    if (x != x) return 0x7F;
    uint8_t sign = (f2u(x) >> 31) ? 0x80 : 0x00;
    float a = fabsf(x);
    if (a >= 448.0f) return (uint8_t)(sign | 0x7E);
    if (a < ldexpf(1.0f, -10)) return sign; /* below half the smallest subnormal */
    int e;
    (void)frexpf(a, &e); /* a = f * 2^e, f in [0.5,1) */
    int exp = e - 1;     /* a in [2^exp, 2^(exp+1)) */
    if (exp < -6) exp = -6; /* subnormal range shares the 2^-6 scale */
    float scaled = ldexpf(a, 3 - exp); /* units of the mantissa lsb */
    float r = rintf(scaled);           /* RN-even under the default rounding mode */
    int q = (int)r;
    int biased;
    if (exp == -6 && q < 8) { biased = 0; }
    else {
        if (q >= 16) { q >>= 1; exp += 1; }
        biased = exp + 7; q -= 8;
    }
    if (biased > 15 || (biased == 15 && q > 6)) return (uint8_t)(sign | 0x7E);
    return (uint8_t)(sign | (biased << 3) | q);
}

float ora_from_e4m3(uint8_t b) {
    int e = (b >> 3) & 15, m = b & 7;
    float v;
    if (e == 15 && m == 7) return NAN;
    if (e == 0) v = ldexpf((float)m, -9);
    else v = ldexpf(1.0f + (float)m / 8.0f, e - 7);
    return (b & 0x80) ? -v : v;
}

/* e8m0: smallest power of two >= |x|, saturating; PTX cvt.rp.satfinite.ue8m0x2.f32
 * via __nv_cvt_float_to_e8m0(x, __NV_SATFINITE, cudaRoundPosInf)
 * (csrc/cuda/sm120/mxfp4/quantization.cu:14-16). */
uint8_t ora_to_e8m0(float x) {
    uint32_t u = f2u(x) & 0x7FFFFFFFu;
    if (u > 0x7F800000u) return 0xFF; /* NaN */
    uint32_t e = u >> 23, m = u & 0x7FFFFFu;
    if (e == 255) return 254;
    if (e == 0) return (m > 0x400000u) ? 1 : 0; /* (2^-127, 2^-126) rounds up to 2^-126; <= 2^-127 -> code 0 */
    if (m) e += 1;
    if (e > 254) e = 254;
    return (uint8_t)e;
}

float ora_from_e8m0(uint8_t b) {
    if (b == 0xFF) return NAN;
    return ldexpf(1.0f, (int)b - 127);
}

/* Row permutation inside every 32-row group (cuda_common.cuh:16-18). */
static inline int perm32(int x) { return (x / 8) * 2 + ((x % 8) / 2) * 8 + (x % 2); }
int ora_perm32(int x) { return perm32(x); }

/* ------------------------------------------------------------------------- */
/* Quantisers                                                                 */
/* ------------------------------------------------------------------------- */

/* One group of `g` values -> g/2 packed bytes and one scale byte.
 * nvfp4/quantization.cu:52-85, mxfp4/quantization.cu:67-107. */
static void quantise_group(const float* x, int g, int is_mx, uint8_t* codes, uint8_t* scale) {
    float amax = 0.0f;
    for (int i = 0; i < g; ++i) { float a = fabsf(x[i]); if (a > amax) amax = a; }
    float sf = amax / 6.0f;
    uint8_t sb = is_mx ? ora_to_e8m0(sf) : ora_to_e4m3(sf);
    float sfq = is_mx ? ora_from_e8m0(sb) : ora_from_e4m3(sb);
    float inv = (sfq == 0.0f) ? 0.0f : 1.0f / sfq;
    for (int i = 0; i < g; i += 2) {
        uint8_t lo = ora_to_e2m1(x[i] * inv);
        uint8_t hi = ora_to_e2m1(x[i + 1] * inv);
        codes[i / 2] = (uint8_t)(lo | (hi << 4));
    }
    *scale = sb;
}

/* x: [bs, seq, d] raw 16-bit; codes: [bs, seq, d/2]; scales: [bs, seq, d/g].
 * permuted != 0: physical row p of each 32-row group holds logical row perm32(p)
 * (nvfp4/quantization.cu:162-243). */
void ora_quantize_rows(const uint16_t* x, int bs, int seq, int d, int is_mx, int is_bf16, int permuted,
                       uint8_t* codes, uint8_t* scales) {
    const int g = is_mx ? 32 : 16;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < bs; ++b)
        for (int p = 0; p < seq; ++p) {
            int src = p;
            int valid = 1;
            if (permuted) {
                src = (p / 32) * 32 + perm32(p % 32);
                valid = src < seq;
            }
            float buf[32];
            for (int c = 0; c < d / g; ++c) {
                for (int i = 0; i < g; ++i)
                    buf[i] = valid ? in_to_float(x[((size_t)b * seq + src) * d + c * g + i], is_bf16) : 0.0f;
                quantise_group(buf, g, is_mx, codes + ((size_t)b * seq + p) * (d / 2) + c * (g / 2),
                               scales + ((size_t)b * seq + p) * (d / g) + c);
            }
        }
}

/* V layout: groups run along the sequence.  codes: [bs, d, P/2], scales: [bs, d, P/g],
 * P = ceil(seq/128)*128, rows >= seq read as zero (nvfp4/quantization.cu:315-428;
 * permuted variant :493-600 applies the row permutation before grouping). */
void ora_quantize_transposed(const uint16_t* x, int bs, int seq, int d, int is_mx, int is_bf16, int permuted,
                             uint8_t* codes, uint8_t* scales) {
    const int g = is_mx ? 32 : 16;
    const int P = ((seq + 127) / 128) * 128;
#pragma omp parallel for collapse(2) schedule(static)
    for (int b = 0; b < bs; ++b)
        for (int ch = 0; ch < d; ++ch) {
            float buf[32];
            for (int grp = 0; grp < P / g; ++grp) {
                for (int i = 0; i < g; ++i) {
                    int p = grp * g + i;
                    int src = p;
                    int valid = p < seq;
                    if (permuted) {
                        src = (p / 32) * 32 + perm32(p % 32);
                        valid = (src < seq) && (p < seq);
                    }
                    buf[i] = valid ? in_to_float(x[((size_t)b * seq + src) * d + ch], is_bf16) : 0.0f;
                }
                quantise_group(buf, g, is_mx, codes + ((size_t)b * d + ch) * (P / 2) + grp * (g / 2),
                               scales + ((size_t)b * d + ch) * (P / g) + grp);
            }
        }
}

/* Exact dequantisation helpers for the attention oracles. */
static void dequant_rows(const uint8_t* codes, const uint8_t* scales, size_t rows, int d, int is_mx, float* out) {
    const int g = is_mx ? 32 : 16;
#pragma omp parallel for schedule(static)
    for (long long r = 0; r < (long long)rows; ++r)
        for (int c = 0; c < d; ++c) {
            uint8_t byte = codes[(size_t)r * (d / 2) + c / 2];
            uint8_t code = (c & 1) ? (byte >> 4) : (byte & 15);
            uint8_t sb = scales[(size_t)r * (d / g) + c / g];
            float s = is_mx ? ora_from_e8m0(sb) : ora_from_e4m3(sb);
            out[(size_t)r * d + c] = E2M1_VALUES[code] * s;
        }
}

/* ------------------------------------------------------------------------- */
/* Block statistics (pre-reductions of the selection policies)                */
/* ------------------------------------------------------------------------- */

/* Per block of `block` rows and per channel: fp32 mean (cast to the 16-bit
 * type), min and max.  selection/block_mean.py:44-54, selection/quest.py:11-24.
 * Summation order: eight interleaved partial sums (rows r = j mod 8) added in
 * ascending row order, then the eight partials added left to right; this is the
 * order the CUDA kernel uses.  Any of mean/mn/mx may be NULL. */
void ora_block_stats(const uint16_t* x, int heads, int seq, int d, int block, int is_bf16, uint16_t* mean,
                     uint16_t* mn, uint16_t* mx) {
    const int nb = seq / block;
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < heads; ++h)
        for (int b = 0; b < nb; ++b)
            for (int c = 0; c < d; ++c) {
                float part[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                float lo = INFINITY, hi = -INFINITY;
                for (int r = 0; r < block; ++r) {
                    float v = in_to_float(x[((size_t)h * seq + (size_t)b * block + r) * d + c], is_bf16);
                    part[r & 7] += v;
                    if (v < lo) lo = v;
                    if (v > hi) hi = v;
                }
                float total = part[0];
                for (int j = 1; j < 8; ++j) total += part[j];
                size_t o = ((size_t)h * nb + b) * d + c;
                if (mean) mean[o] = float_to_out(total / (float)block, is_bf16);
                if (mn) mn[o] = float_to_out(lo, is_bf16);
                if (mx) mx[o] = float_to_out(hi, is_bf16);
            }
}

/* ------------------------------------------------------------------------- */
/* Selection                                                                  */
/* ------------------------------------------------------------------------- */

/* fp32 score with the reference kernel's summation tree: lane l accumulates
 * channels l, l+32, ... with fused multiply-adds, then an xor butterfly over
 * deltas 16..1 (csrc/cuda/sm120/shared/block_selection.cu:52-63, 264-278). */
static float warp_dot(const float* q, const float* kmin, const float* kmax, int d) {
    float lane[32];
    for (int l = 0; l < 32; ++l) {
        float acc = 0.0f;
        for (int c = l; c < d; c += 32) {
            float k = kmax ? (q[c] >= 0.0f ? kmax[c] : kmin[c]) : kmin[c];
            acc = fmaf(q[c], k, acc);
        }
        lane[l] = acc;
    }
    for (int delta = 16; delta >= 1; delta >>= 1) {
        float nxt[32];
        for (int l = 0; l < 32; ++l) nxt[l] = lane[l] + lane[l ^ delta];
        memcpy(lane, nxt, sizeof lane);
    }
    return lane[0];
}

/* k rounds of warp arg-max with knock-out (block_selection.cu:85-114): each
 * lane scans its strided candidates with strict '>', lanes are then combined by
 * an xor butterfly that keeps the own candidate on ties, lane 0 reports. */
static void warp_topk(float* scores, int n, int k, int pad_when_empty, int32_t* out) {
    for (int r = 0; r < k; ++r) {
        float best[32];
        int bidx[32];
        for (int l = 0; l < 32; ++l) {
            best[l] = -FLT_MAX;
            bidx[l] = l;
            if (l < n) best[l] = scores[l];
            for (int i = l + 32; i < n; i += 32)
                if (scores[i] > best[l]) { best[l] = scores[i]; bidx[l] = i; }
        }
        for (int delta = 16; delta >= 1; delta >>= 1) {
            float nb[32];
            int ni[32];
            for (int l = 0; l < 32; ++l) {
                nb[l] = best[l];
                ni[l] = bidx[l];
                if (best[l ^ delta] > best[l]) { nb[l] = best[l ^ delta]; ni[l] = bidx[l ^ delta]; }
            }
            memcpy(best, nb, sizeof best);
            memcpy(bidx, ni, sizeof bidx);
        }
        int found = best[0] > -FLT_MAX * 0.5f;
        if (pad_when_empty) out[r] = found ? bidx[0] : -1;
        else out[r] = bidx[0];
        if (found || !pad_when_empty) {
            if (bidx[0] < n) scores[bidx[0]] = -FLT_MAX;
        }
    }
}

/* Prefill selection.  q_mean: [heads, nq, d]; k_a/k_b: [kv_heads, nk, d] with
 * heads = kv_heads * group (the reference expands K statistics per Q head,
 * selection/quest.py:27-31).  quest != 0: k_a = k_min, k_b = k_max and the score
 * is the Quest bound (block_selection.cu:264-273); otherwise k_a = k_mean and the
 * score is the dot product (block_selection.cu:52-58).
 * Extension: `sink` leading and `local` trailing valid blocks are always kept and
 * excluded from the scored candidates; out row = [sink ids asc, local ids asc,
 * top-k by rank], -1 padded; width = sink + local + k. */
void ora_select_prefill(const uint16_t* q_mean, const uint16_t* k_a, const uint16_t* k_b, int heads, int group,
                        int nq, int nk, int d, int k, int causal, int quest, int is_bf16, int sink, int local,
                        int32_t* out) {
    const int width = sink + local + k;
#pragma omp parallel for collapse(2) schedule(dynamic, 8)
    for (int h = 0; h < heads; ++h)
        for (int qb = 0; qb < nq; ++qb) {
            const int kvh = h / group;
            float qf[256], ka[256], kb_[256];
            float* scores = (float*)malloc(sizeof(float) * (size_t)(nk > 0 ? nk : 1));
            for (int c = 0; c < d; ++c) qf[c] = in_to_float(q_mean[((size_t)h * nq + qb) * d + c], is_bf16);
            int nvalid = causal ? (qb + 1 < nk ? qb + 1 : nk) : nk;
            int n_sink = sink < nvalid ? sink : nvalid;
            int local_lo = nvalid - local;
            if (local_lo < n_sink) local_lo = n_sink;
            for (int b = 0; b < nk; ++b) {
                if (b >= nvalid || b < n_sink || b >= local_lo) { scores[b] = -FLT_MAX; continue; }
                for (int c = 0; c < d; ++c) {
                    ka[c] = in_to_float(k_a[((size_t)kvh * nk + b) * d + c], is_bf16);
                    if (quest) kb_[c] = in_to_float(k_b[((size_t)kvh * nk + b) * d + c], is_bf16);
                }
                scores[b] = warp_dot(qf, ka, quest ? kb_ : NULL, d);
            }
            int32_t* row = out + ((size_t)h * nq + qb) * width;
            int w = 0;
            for (int b = 0; b < n_sink; ++b) row[w++] = b;
            for (int b = local_lo; b < nvalid; ++b) row[w++] = b;
            warp_topk(scores, nk, k, 1, row + w);
            /* compact: move -1 padding of the forced part to the end */
            int filled = w;
            for (int i = 0; i < k; ++i) {
                int32_t v = row[w + i];
                if (v >= 0) row[filled++] = v;
            }
            for (int i = filled; i < width; ++i) row[i] = -1;
            free(scores);
        }
}

/* Decode selection: score = max over the `group` query heads of one KV head
 * (block_selection.cu:150-176, 365-391); no padding (rounds past the candidates
 * repeat the reference's behaviour only for k <= candidates, which callers ensure).
 * q: [flat_kv_heads, group, d]; k_a/k_b: [flat_kv_heads, cap_blocks, d].
 * Extension: sink/local forced blocks as in ora_select_prefill. */
void ora_select_decode(const uint16_t* q, const uint16_t* k_a, const uint16_t* k_b, int flat_kv_heads, int group,
                       int nk, int cap_blocks, int d, int k, int quest, int is_bf16, int sink, int local,
                       int32_t* out) {
    const int width = sink + local + k;
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < flat_kv_heads; ++h) {
        float* scores = (float*)malloc(sizeof(float) * (size_t)(nk > 0 ? nk : 1));
        float qf[256], ka[256], kb_[256];
        int n_sink = sink < nk ? sink : nk;
        int local_lo = nk - local;
        if (local_lo < n_sink) local_lo = n_sink;
        for (int b = 0; b < nk; ++b) {
            if (b < n_sink || b >= local_lo) { scores[b] = -FLT_MAX; continue; }
            for (int c = 0; c < d; ++c) {
                ka[c] = in_to_float(k_a[((size_t)h * cap_blocks + b) * d + c], is_bf16);
                if (quest) kb_[c] = in_to_float(k_b[((size_t)h * cap_blocks + b) * d + c], is_bf16);
            }
            float best = -FLT_MAX;
            for (int g = 0; g < group; ++g) {
                for (int c = 0; c < d; ++c) qf[c] = in_to_float(q[((size_t)h * group + g) * d + c], is_bf16);
                float s = warp_dot(qf, ka, quest ? kb_ : NULL, d);
                if (s > best) best = s;
            }
            scores[b] = best;
        }
        int32_t* row = out + (size_t)h * width;
        int w = 0;
        for (int b = 0; b < n_sink; ++b) row[w++] = b;
        for (int b = local_lo; b < nk; ++b) row[w++] = b;
        warp_topk(scores, nk, k, (sink + local) > 0, row + w);
        int filled = w;
        for (int i = 0; i < k; ++i) {
            int32_t v = row[w + i];
            if (v >= 0 || (sink + local) == 0) row[filled++] = v;
        }
        for (int i = filled; i < width; ++i) row[i] = -1;
        free(scores);
    }
}

/* Closed-form local windows (block_selection.cu:629-673). */
void ora_local_prefill(int rows_heads, int nq, int nk, int k, int causal, int32_t* out) {
    for (int h = 0; h < rows_heads; ++h)
        for (int qb = 0; qb < nq; ++qb) {
            int start = 0, valid = k;
            if (causal) {
                int end = qb < nk - 1 ? qb : nk - 1;
                valid = end + 1 < k ? end + 1 : k;
                start = end - k + 1 > 0 ? end - k + 1 : 0;
            } else {
                int center = qb < nk - 1 ? qb : nk - 1;
                int max_start = nk - k > 0 ? nk - k : 0;
                int s = center - k / 2 > 0 ? center - k / 2 : 0;
                start = s < max_start ? s : max_start;
            }
            for (int r = 0; r < k; ++r) out[((size_t)h * nq + qb) * k + r] = r < valid ? start + r : -1;
        }
}

void ora_local_decode(int flat_heads, int nk, int k, int32_t* out) {
    for (int h = 0; h < flat_heads; ++h)
        for (int r = 0; r < k; ++r) out[(size_t)h * k + r] = nk - k + r;
}

/* Index list -> 64-bit bitset words (block_selection.cu:1260-1285). */
void ora_pack_mask(const int32_t* sel, int rows, int k, int nk, int words, uint64_t* mask) {
    memset(mask, 0, sizeof(uint64_t) * (size_t)rows * words);
    for (int r = 0; r < rows; ++r)
        for (int i = 0; i < k; ++i) {
            int32_t b = sel[(size_t)r * k + i];
            if (b >= 0 && b < nk && (b >> 6) < words) mask[(size_t)r * words + (b >> 6)] |= 1ull << (b & 63);
        }
}

/* ------------------------------------------------------------------------- */
/* Prefill attention                                                          */
/* ------------------------------------------------------------------------- */

typedef struct {
    float m, l;
} row_state;

static inline float round_out(float v, int is_bf16) {
    uint16_t b = float_to_out(v, is_bf16);
    return in_to_float(b, is_bf16);
}

/*
 * Mixed FP4 / 16-bit prefill attention, all heads.
 *
 * Numerics follow csrc/cuda/sm120/nvfp4/thrift_attention.cu:188-447 (FP4 pass
 * over the non-selected blocks, ascending, in 64-column steps: block-scaled
 * dot, scale by 1/sqrt(d), causal mask, online softmax, P -> e2m1(6 p) with
 * scale 448 (NVFP4) or 1 (MXFP4), normalised partial rounded to the 16-bit
 * output type) and :509-737 (16-bit pass over the selected blocks in list
 * order, P -> 16-bit(C p)).  C = 2688 (NVFP4) or 6 (MXFP4).
 *
 * q_hi [hq, sq, d], k_hi/v_hi [hkv, skv, d] raw 16-bit; q4 [hq, sq, d/2] + qs;
 * k4 [hkv, kv_cap, d/2] + ks in *logical* row order (the reference's K row
 * permutation only relabels columns inside a block and is undone by its mask);
 * v4t [hkv, d, P/2] + vst with P = ceil(kv_cap/128)*128.
 * sel: [hq, nq_blocks, width] block ids (-1 padded) at granularity `block`, or
 * NULL / width 0 for pure FP4.  out [hq, sq, d] raw 16-bit.
 * round_partial != 0 reproduces the 16-bit rounding of the state between the two
 * passes (thrift_attention.cu:443-446, 524-529).
 * row_begin/row_end restrict the computed query rows (others are not written).
 */
void ora_prefill_attention(const uint16_t* q_hi, const uint16_t* k_hi, const uint16_t* v_hi, const uint8_t* q4,
                           const uint8_t* qs, const uint8_t* k4, const uint8_t* ks, const uint8_t* v4t,
                           const uint8_t* vst, const int32_t* sel, int width, int hq, int hkv, int sq, int skv,
                           int kv_cap, int d, int block, int causal, int is_mx, int is_bf16, int round_partial,
                           int row_begin, int row_end, uint16_t* out) {
    const int g = is_mx ? 32 : 16;
    const int group = hq / hkv;
    const int P = ((kv_cap + 127) / 128) * 128;
    const int STEP = 64;
    const float C = is_mx ? 6.0f : 448.0f * 6.0f;
    const float C_INV = is_mx ? 1.0f / 6.0f : 1.0f / (448.0f * 6.0f);
    const float p_scale = is_mx ? 1.0f : 448.0f;
    const float sm_scale = (float)(1.0 / sqrt((double)d));
    const int nkb = skv / block;
    const int nsteps_total = (skv + STEP - 1) / STEP;
    if (row_end > sq) row_end = sq;

    /* exact dequantised copies */
    float* qf = (float*)malloc(sizeof(float) * (size_t)hq * sq * d);
    float* kf = (float*)malloc(sizeof(float) * (size_t)hkv * skv * d);
    float* vf = (float*)malloc(sizeof(float) * (size_t)hkv * skv * d); /* [hkv, skv, d] */
    dequant_rows(q4, qs, (size_t)hq * sq, d, is_mx, qf);
    for (int h = 0; h < hkv; ++h)
        dequant_rows(k4 + (size_t)h * kv_cap * (d / 2), ks + (size_t)h * kv_cap * (d / g), (size_t)skv, d, is_mx,
                     kf + (size_t)h * skv * d);
#pragma omp parallel for collapse(2) schedule(static)
    for (int h = 0; h < hkv; ++h)
        for (int c = 0; c < d; ++c)
            for (int t = 0; t < skv; ++t) {
                uint8_t byte = v4t[((size_t)h * d + c) * (P / 2) + t / 2];
                uint8_t code = (t & 1) ? (byte >> 4) : (byte & 15);
                uint8_t sb = vst[((size_t)h * d + c) * (P / g) + t / g];
                float s = is_mx ? ora_from_e8m0(sb) : ora_from_e4m3(sb);
                vf[((size_t)h * skv + t) * d + c] = E2M1_VALUES[code] * s;
            }

#pragma omp parallel for collapse(2) schedule(dynamic, 4)
    for (int h = 0; h < hq; ++h)
        for (int r = row_begin; r < row_end; ++r) {
            const int kvh = h / group;
            const int qb = r / block;
            const int32_t* list = (sel && width > 0) ? sel + ((size_t)h * (sq / block) + qb) * width : NULL;
            /* bitset of selected blocks */
            uint8_t* is_sel = (uint8_t*)calloc((size_t)nkb + 1, 1);
            if (list)
                for (int i = 0; i < width; ++i)
                    if (list[i] >= 0 && list[i] < nkb) is_sel[list[i]] = 1;
            /* The reference bounds the kv loop by the 64-row tile's diagonal
             * (thrift_attention.cu:139-144); steps wholly above this row's own
             * diagonal are fully masked there and leave (m, l, O) unchanged, so
             * the per-row bound used here is equivalent. */
            const int tile_last = r;
            int nsteps = causal ? (r / STEP + 1 < nsteps_total ? r / STEP + 1 : nsteps_total) : nsteps_total;
            float m = -FLT_MAX, l = 0.0f;
            float O[256];
            float s[64], p[64];
            for (int c = 0; c < d; ++c) O[c] = 0.0f;
            const float* qrow = qf + ((size_t)h * sq + r) * d;

            for (int st = 0; st < nsteps; ++st) {
                const int col0 = st * STEP;
                if (list && is_sel[col0 / block]) continue;
                const int ncol = (skv - col0) < STEP ? (skv - col0) : STEP;
                float smax = -FLT_MAX;
                for (int j = 0; j < STEP; ++j) {
                    if (j >= ncol) { s[j] = -INFINITY; continue; }
                    const float* krow = kf + ((size_t)kvh * skv + col0 + j) * d;
                    float acc = 0.0f;
                    for (int c = 0; c < d; ++c) acc += qrow[c] * krow[c];
                    if (causal && (col0 + j) > r) acc = -INFINITY;
                    s[j] = acc * sm_scale;
                    if (s[j] > smax) smax = s[j];
                }
                float m_new = smax > m ? smax : m;
                float resc = expf(m - m_new);
                for (int c = 0; c < d; ++c) O[c] *= resc;
                m = m_new;
                float sum = 0.0f;
                for (int j = 0; j < STEP; ++j) { p[j] = expf(s[j] - m); sum += p[j]; }
                l = l * resc + sum;
                const int valid = m > -FLT_MAX * 0.5f;
                for (int j = 0; j < ncol; ++j) {
                    float pq = valid ? ora_from_e2m1(ora_to_e2m1(p[j] * 6.0f)) * p_scale : 0.0f;
                    if (pq == 0.0f) continue;
                    const float* vrow = vf + ((size_t)kvh * skv + col0 + j) * d;
                    for (int c = 0; c < d; ++c) O[c] += pq * vrow[c];
                }
            }

            if (list) {
                if (round_partial) {
                    float norm = l > 0.0f ? C_INV / l : 0.0f;
                    float back = l * C;
                    for (int c = 0; c < d; ++c) O[c] = round_out(O[c] * norm, is_bf16) * back;
                }
                const uint16_t* qh = q_hi + ((size_t)h * sq + r) * d;
                float q16[256];
                for (int c = 0; c < d; ++c) q16[c] = in_to_float(qh[c], is_bf16);
                for (int i = 0; i < width; ++i) {
                    int blk = list[i];
                    if (blk < 0 || blk >= nkb) continue;
                    if (causal && blk * block > tile_last) continue;
                    for (int sub = 0; sub < block / STEP; ++sub) {
                        const int col0 = blk * block + sub * STEP;
                        if (causal && col0 > tile_last) continue;
                        float smax = -FLT_MAX;
                        for (int j = 0; j < STEP; ++j) {
                            const uint16_t* kr = k_hi + ((size_t)kvh * skv + col0 + j) * d;
                            float acc = 0.0f;
                            for (int c = 0; c < d; ++c) acc += q16[c] * in_to_float(kr[c], is_bf16);
                            if (causal && (col0 + j) > r) acc = -INFINITY;
                            s[j] = acc * sm_scale;
                            if (s[j] > smax) smax = s[j];
                        }
                        float m_new = smax > m ? smax : m;
                        float resc = expf(m - m_new);
                        for (int c = 0; c < d; ++c) O[c] *= resc;
                        m = m_new;
                        float sum = 0.0f;
                        for (int j = 0; j < STEP; ++j) { p[j] = expf(s[j] - m); sum += p[j]; }
                        l = l * resc + sum;
                        for (int j = 0; j < STEP; ++j) {
                            float p16 = round_out(p[j] * C, is_bf16);
                            if (p16 == 0.0f) continue;
                            const uint16_t* vr = v_hi + ((size_t)kvh * skv + col0 + j) * d;
                            for (int c = 0; c < d; ++c) O[c] += p16 * in_to_float(vr[c], is_bf16);
                        }
                    }
                }
            }
            float norm = l > 0.0f ? C_INV / l : 0.0f;
            uint16_t* orow = out + ((size_t)h * sq + r) * d;
            for (int c = 0; c < d; ++c) orow[c] = float_to_out(O[c] * norm, is_bf16);
            free(is_sel);
        }
    free(qf);
    free(kf);
    free(vf);
}

/* ------------------------------------------------------------------------- */
/* Decode attention                                                           */
/* ------------------------------------------------------------------------- */

/*
 * Single-token mixed attention over a (logically contiguous) cache.
 * csrc/cuda/sm120/nvfp4/single_query_attention.cu:487-737 (FP4 pages, dynamic
 * per-16/32-column P scale), :277-461 (16-bit pages), split ranges :1246-1248,
 * merge :1551-1594.
 *
 * q_hi [heads, G, d] (heads = batch*kv_heads), q4/qs its quantisation;
 * k_hi/v_hi [heads, kv_len, d]; k4/ks [heads, kv_cap, d/2|d/g] plain order;
 * v4t/vst [heads, d, P/2|P/g]; sel [heads, width] page ids (64-token pages), may
 * contain -1.  `splits` sequential chains per head: chain s covers pages
 * [s*n/splits, (s+1)*n/splits); inside a chain FP4 pages ascending, then the
 * selected pages ascending.  out [heads, G, d].
 * If part_o != NULL the un-merged partials are also written:
 * part_o [heads, splits, G, d] (un-normalised, in units of C), part_ml [heads, splits, G, 2].
 */
void ora_decode_attention(const uint16_t* q_hi, const uint16_t* k_hi, const uint16_t* v_hi, const uint8_t* q4,
                          const uint8_t* qs, const uint8_t* k4, const uint8_t* ks, const uint8_t* v4t,
                          const uint8_t* vst, const int32_t* sel, int width, int heads, int G, int kv_len,
                          int kv_cap, int d, int is_mx, int is_bf16, int splits, uint16_t* out, float* part_o,
                          float* part_ml) {
    const int g = is_mx ? 32 : 16;
    const int P = ((kv_cap + 127) / 128) * 128;
    const int PAGE = 64;
    const int npages = (kv_len + PAGE - 1) / PAGE;
    const float C = is_mx ? 6.0f : 448.0f * 6.0f;
    const float sm_scale = (float)(1.0 / sqrt((double)d));
    if (splits < 1) splits = 1;
    if (splits > npages) splits = npages > 0 ? npages : 1;

#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < heads; ++h) {
        uint8_t* is_sel = (uint8_t*)calloc((size_t)npages + 1, 1);
        if (sel)
            for (int i = 0; i < width; ++i) {
                int32_t b = sel[(size_t)h * width + i];
                if (b >= 0 && b < npages) is_sel[b] = 1;
            }
        float* po = (float*)calloc((size_t)splits * G * d, sizeof(float));
        float* pm = (float*)malloc(sizeof(float) * (size_t)splits * G);
        float* pl = (float*)calloc((size_t)splits * G, sizeof(float));
        float* qd = (float*)malloc(sizeof(float) * (size_t)G * d);
        dequant_rows(q4 + (size_t)h * G * (d / 2), qs + (size_t)h * G * (d / g), (size_t)G, d, is_mx, qd);
        for (int s = 0; s < splits; ++s) {
            const int p_begin = (int)((long long)s * npages / splits);
            const int p_end = (int)((long long)(s + 1) * npages / splits);
            for (int gi = 0; gi < G; ++gi) {
                float m = -FLT_MAX, l = 0.0f;
                float* O = po + ((size_t)s * G + gi) * d;
                float sc[64], p[64];
                for (int pass = 0; pass < 2; ++pass)
                    for (int pg = p_begin; pg < p_end; ++pg) {
                        if ((int)is_sel[pg] != pass) continue;
                        const int col0 = pg * PAGE;
                        float smax = -FLT_MAX;
                        for (int j = 0; j < PAGE; ++j) {
                            const int t = col0 + j;
                            float acc = 0.0f;
                            if (pass == 0) {
                                /* rows past kv_len inside kv_cap are whatever the cache holds
                                 * (zero-filled by the cache); rows past kv_cap are zero. */
                                if (t < kv_cap) {
                                    const uint8_t* kc = k4 + ((size_t)h * kv_cap + t) * (d / 2);
                                    const uint8_t* kss = ks + ((size_t)h * kv_cap + t) * (d / g);
                                    for (int c = 0; c < d; ++c) {
                                        uint8_t byte = kc[c / 2];
                                        uint8_t code = (c & 1) ? (byte >> 4) : (byte & 15);
                                        float sv = is_mx ? ora_from_e8m0(kss[c / g]) : ora_from_e4m3(kss[c / g]);
                                        acc += qd[(size_t)gi * d + c] * (E2M1_VALUES[code] * sv);
                                    }
                                }
                            } else {
                                if (t < kv_len) {
                                    const uint16_t* kr = k_hi + ((size_t)h * kv_len + t) * d;
                                    const uint16_t* qr = q_hi + ((size_t)h * G + gi) * d;
                                    for (int c = 0; c < d; ++c)
                                        acc += in_to_float(qr[c], is_bf16) * in_to_float(kr[c], is_bf16);
                                }
                            }
                            sc[j] = acc * sm_scale;
                            if (sc[j] > smax) smax = sc[j];
                        }
                        float m_new = smax > m ? smax : m;
                        float resc = expf(m - m_new);
                        for (int c = 0; c < d; ++c) O[c] *= resc;
                        m = m_new;
                        float sum = 0.0f;
                        for (int j = 0; j < PAGE; ++j) { p[j] = expf(sc[j] - m); sum += p[j]; }
                        l = l * resc + sum;
                        if (pass == 0) {
                            for (int j0 = 0; j0 < PAGE; j0 += g) {
                                float amax = 0.0f;
                                for (int j = 0; j < g; ++j) { float t = p[j0 + j] * C; if (t > amax) amax = t; }
                                float sfp = amax / 6.0f;
                                float inv = 1.0f / sfp;
                                float sfq = is_mx ? ora_from_e8m0(ora_to_e8m0(sfp)) : ora_from_e4m3(ora_to_e4m3(sfp));
                                for (int j = 0; j < g; ++j) {
                                    const int t = col0 + j0 + j;
                                    float code_v = ora_from_e2m1(ora_to_e2m1(p[j0 + j] * C * inv));
                                    float pq = (sfq == 0.0f) ? 0.0f : code_v * sfq;
                                    if (pq == 0.0f || t >= P) continue;
                                    for (int c = 0; c < d; ++c) {
                                        uint8_t byte = v4t[((size_t)h * d + c) * (P / 2) + t / 2];
                                        uint8_t code = (t & 1) ? (byte >> 4) : (byte & 15);
                                        uint8_t sb = vst[((size_t)h * d + c) * (P / g) + t / g];
                                        float sv = is_mx ? ora_from_e8m0(sb) : ora_from_e4m3(sb);
                                        O[c] += pq * (E2M1_VALUES[code] * sv);
                                    }
                                }
                            }
                        } else {
                            for (int j = 0; j < PAGE; ++j) {
                                const int t = col0 + j;
                                if (t >= kv_len) continue;
                                float p16 = round_out(p[j] * C, is_bf16);
                                const uint16_t* vr = v_hi + ((size_t)h * kv_len + t) * d;
                                for (int c = 0; c < d; ++c) O[c] += p16 * in_to_float(vr[c], is_bf16);
                            }
                        }
                    }
                pm[(size_t)s * G + gi] = m;
                pl[(size_t)s * G + gi] = l;
            }
        }
        for (int gi = 0; gi < G; ++gi) {
            float M = -FLT_MAX;
            for (int s = 0; s < splits; ++s)
                if (pm[(size_t)s * G + gi] > M) M = pm[(size_t)s * G + gi];
            float den = 0.0f;
            float acc[256];
            for (int c = 0; c < d; ++c) acc[c] = 0.0f;
            for (int s = 0; s < splits; ++s) {
                float w = expf(pm[(size_t)s * G + gi] - M);
                den += pl[(size_t)s * G + gi] * w;
                for (int c = 0; c < d; ++c) acc[c] += po[((size_t)s * G + gi) * d + c] * w;
            }
            float norm = den > 0.0f ? 1.0f / (C * den) : 0.0f;
            for (int c = 0; c < d; ++c) out[((size_t)h * G + gi) * d + c] = float_to_out(acc[c] * norm, is_bf16);
        }
        if (part_o) {
            memcpy(part_o + (size_t)h * splits * G * d, po, sizeof(float) * (size_t)splits * G * d);
            for (int i = 0; i < splits * G; ++i) {
                part_ml[((size_t)h * splits * G + i) * 2 + 0] = pm[i];
                part_ml[((size_t)h * splits * G + i) * 2 + 1] = pl[i];
            }
        }
        free(is_sel); free(po); free(pm); free(pl); free(qd);
    }
}

/* Merge of per-shard decode partials (same formula as the in-kernel merge,
 * single_query_attention.cu:1562-1593): part_o [shards, rows, d] in units of C,
 * part_ml [shards, rows, 2]. */
void ora_merge_partials(const float* part_o, const float* part_ml, int shards, int rows, int d, float C,
                        int is_bf16, uint16_t* out) {
    for (int r = 0; r < rows; ++r) {
        float M = -FLT_MAX;
        for (int s = 0; s < shards; ++s) {
            float m = part_ml[((size_t)s * rows + r) * 2];
            if (m > M) M = m;
        }
        float den = 0.0f;
        float acc[256];
        for (int c = 0; c < d; ++c) acc[c] = 0.0f;
        for (int s = 0; s < shards; ++s) {
            float w = expf(part_ml[((size_t)s * rows + r) * 2] - M);
            den += part_ml[((size_t)s * rows + r) * 2 + 1] * w;
            for (int c = 0; c < d; ++c) acc[c] += part_o[((size_t)s * rows + r) * d + c] * w;
        }
        float norm = den > 0.0f ? 1.0f / (C * den) : 0.0f;
        for (int c = 0; c < d; ++c) out[(size_t)r * d + c] = float_to_out(acc[c] * norm, is_bf16);
    }
}
