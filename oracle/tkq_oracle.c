/*
 * tkq_oracle.c -- CPU restatement of the TileKernels quantization casts.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA kernels in
 * tilekernels_b200/csrc: the tests, the smoke check and the CPU-baseline leg of
 * the benchmark call it; the product never does.  It restates, in plain C, the
 * algorithms of the reference's PyTorch implementation (paths are relative to
 * the reference project root):
 *
 *   tile_kernels/torch/cast.py:62-221        cast()            -> tkqo_cast
 *   tile_kernels/torch/cast.py:224-252       convert_to_e2m1_bits -> f32_to_e2m1
 *   tile_kernels/torch/cast.py:40-59         cast_back()       -> tkqo_cast_back
 *   tile_kernels/torch/cast_e5m6.py:37-62    fp32 -> fp16 RTZ  -> f32_to_f16_rtz_bits
 *   tile_kernels/torch/cast_e5m6.py:65-100   12-bit rounding + 8-in-3-words packing
 *   tile_kernels/torch/cast_e5m6.py:135-218  cast_to_e5m6()    -> tkqo_cast_e5m6
 *   tile_kernels/torch/swiglu.py:47-88       swiglu_forward()  -> tkqo_swiglu_forward
 *   tile_kernels/torch/swiglu.py:98-226      swiglu_backward() -> tkqo_swiglu_backward
 *
 * The scale-factor *layouts* (column-major, packed ue8m0) are produced by the
 * numpy wrapper next to this file; this file always emits row-major fp32 scale
 * bits, exactly the `ds_int_rounded` of cast.py before step 6.
 *
 * Pinning: tests/test_oracle_golden.py compares every function here with
 * fixtures produced by the reference itself (tests/golden/make_golden.py).
 *
 * One deliberate difference, stated in the fixture test as well: exp() in
 * swiglu_forward.  torch's CPU exp is a vendor vector routine whose last bit
 * cannot be reproduced on a GPU, and CUDA's expf cannot be reproduced on a
 * CPU.  Both sides of this project therefore use the same FMA-only routine
 * (tkq_expf below, mirrored in csrc/tkq_common.cuh); it is within 1 ulp of
 * the true exponential on [-87, 88] and clamps its argument to that range.
 */
#include <math.h>
#include <stdint.h>
#include <string.h>

#define TKQO_DT_BF16 0
#define TKQO_DT_FP32 1

#define TKQO_FMT_E4M3 0
#define TKQO_FMT_E2M1 1

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

static inline float load_elem(const void* x, int dt, int64_t idx) {
    if (dt == TKQO_DT_BF16) return u2f((uint32_t)((const uint16_t*)x)[idx] << 16);
    return ((const float*)x)[idx];
}

/* ---- fp32 -> e4m3fn, round-to-nearest-even.  Callers clamp to +-448 first
 * (cast.py:186-187), so the overflow branch only maps what is left (NaN). ---- */
static inline uint8_t f32_to_e4m3fn(float f) {
    uint32_t u = f2u(f);
    uint8_t sign = (uint8_t)((u >> 24) & 0x80);
    u &= 0x7FFFFFFFu;
    if (u >= 0x43F00000u) return sign | 0x7F;          /* >= 480 or NaN: not reachable after the clamp */
    if (u < 0x3C800000u) {                              /* below 2^-6: subnormal target, step 2^-9 */
        float t = u2f(u) + 16384.0f;                    /* ulp(16384) = 2^-9: the add rounds RNE */
        return sign | (uint8_t)(f2u(t) - f2u(16384.0f));
    }
    uint32_t odd = (u >> 20) & 1u;
    u += 0x7FFFFu + odd;                                /* RNE on the 20 dropped bits */
    u -= (127u - 7u) << 23;                             /* re-bias 127 -> 7 */
    return sign | (uint8_t)(u >> 20);
}

/* ---- fp32 -> e2m1 (values 0, .5, 1, 1.5, 2, 3, 4, 6), RNE, saturating.
 * Same mapping as convert_to_e2m1_bits (cast.py:224-252): the code is the
 * number of midpoints below |v|, ties resolved to the even code. ---- */
static inline uint8_t f32_to_e2m1(float f) {
    uint32_t u = f2u(f);
    uint8_t sign = (uint8_t)((u >> 28) & 0x8);
    float a = u2f(u & 0x7FFFFFFFu);
    uint8_t c;
    if (!(a <= 5.0f)) c = 7;                            /* > 5, inf, NaN */
    else c = (uint8_t)((a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.0f));
    return sign | c;
}

static const float k_e2m1_values[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};

/* ---- fp32 -> fp16 bits, round toward zero (cast_e5m6.py:37-62). ---- */
static inline uint32_t f32_to_f16_rtz_bits(float f) {
    uint32_t x = f2u(f);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t exp = (x >> 23) & 0xFFu;
    uint32_t mant = x & 0x7FFFFFu;
    if (exp == 255) return sign | (mant ? 0x7FFFu : 0x7C00u);
    if (exp > 142) return sign | 0x7C00u;
    if (exp >= 113) return sign | ((exp - 112u) << 10) | (mant >> 13);
    if (exp >= 103) return sign | ((0x800000u | mant) >> (113u - exp + 13u));
    return sign;
}

/* ---- 12-bit e5m6 code: truncate the RTZ half to 12 bits, then round to
 * nearest even on the 17 low bits of the fp32 (cast_e5m6.py:76-80). ---- */
static inline uint32_t f32_to_e5m6(float f) {
    uint32_t c = f32_to_f16_rtz_bits(f) >> 4;
    uint32_t rem = f2u(f) & 0x1FFFFu;
    if ((c & 1u) + rem > 0x10000u) c += 1;
    return c & 0xFFFu;
}

/* ---- scale from a block maximum (cast.py:147-164).  Returns the dequant
 * scale bits (rounded up to a power of two when round_sf) and the multiplier
 * applied to the data. ---- */
static inline void scale_from_amax(float amax, float clamp_min, float max_q, int round_sf, uint32_t* sf_bits, float* q) {
    if (amax < clamp_min) amax = clamp_min;             /* torch.clamp(min=) */
    float ds = amax / max_q;
    uint32_t b = f2u(ds);
    if (round_sf) {
        b = (b + 0x007FFFFFu) & 0x7F800000u;
        *q = (b == 0 || u2f(b) == 0.0f) ? 0.0f : 1.0f / u2f(b);
    } else {
        *q = (b == 0) ? 0.0f : max_q / amax;
    }
    *sf_bits = b;
}

/*
 * tkqo_cast: blockwise cast of a 2-D tensor (cast.py:62-221 without the
 * QuantTensor-input branch).
 *   x            [T, H] elements of `in_dtype`, row stride `x_stride` elements
 *   fmt          e4m3 (1 byte/elem) or e2m1 (2 elems/byte, even index in the low nibble)
 *   (bm, bk)     scale block; edge blocks take the maximum over valid elements only
 *   clamp_min    < 0 selects the format default (1e-4 for e4m3, 6*2^-126 for e2m1)
 *   sf_pre       optional [ceil(T/bm), ceil(H/bk)] fp32 dequant scales ("cast only": data * (1/sf))
 *   out          [T, H] or [T, H/2] bytes
 *   sf_bits_out  [ceil(T/bm), ceil(H/bk)] uint32 scale bits, row-major (ignored with sf_pre; may be NULL)
 */
int tkqo_cast(const void* x, int in_dtype, int64_t T, int64_t H, int64_t x_stride, int fmt, int bm, int bk,
              int round_sf, float clamp_min, const float* sf_pre, uint8_t* out, uint32_t* sf_bits_out) {
    if (fmt != TKQO_FMT_E4M3 && fmt != TKQO_FMT_E2M1) return -1;
    if (fmt == TKQO_FMT_E2M1 && (H & 1)) return -1;
    const float max_q = fmt == TKQO_FMT_E4M3 ? 448.0f : 6.0f;
    if (clamp_min < 0.0f) clamp_min = fmt == TKQO_FMT_E4M3 ? 0.0001f : 6.0f * 0x1p-126f;
    const int64_t nbm = (T + bm - 1) / bm, nbk = (H + bk - 1) / bk;
    const int64_t out_stride = fmt == TKQO_FMT_E4M3 ? H : H / 2;

#pragma omp parallel for schedule(static) collapse(2)
    for (int64_t bi = 0; bi < nbm; ++bi) {
        for (int64_t bj = 0; bj < nbk; ++bj) {
            const int64_t r0 = bi * bm, r1 = r0 + bm < T ? r0 + bm : T;
            const int64_t c0 = bj * bk, c1 = c0 + bk < H ? c0 + bk : H;
            float q;
            if (sf_pre) {
                q = 1.0f / sf_pre[bi * nbk + bj];       /* sf.reciprocal(), cast.py:170 */
            } else {
                float amax = -1.0f;                      /* padding is excluded with -1, cast.py:142-144 */
                for (int64_t r = r0; r < r1; ++r)
                    for (int64_t c = c0; c < c1; ++c) {
                        float a = fabsf(load_elem(x, in_dtype, r * x_stride + c));
                        if (a > amax) amax = a;
                    }
                uint32_t b;
                scale_from_amax(amax, clamp_min, max_q, round_sf, &b, &q);
                if (sf_bits_out) sf_bits_out[bi * nbk + bj] = b;
            }
            for (int64_t r = r0; r < r1; ++r) {
                if (fmt == TKQO_FMT_E4M3) {
                    for (int64_t c = c0; c < c1; ++c) {
                        float v = load_elem(x, in_dtype, r * x_stride + c) * q;
                        if (v > max_q) v = max_q;        /* torch.clamp keeps NaN, as does this */
                        if (v < -max_q) v = -max_q;
                        out[r * out_stride + c] = f32_to_e4m3fn(v);
                    }
                } else {
                    for (int64_t c = c0; c < c1; c += 2) {  /* bk and H are even: pairs never straddle blocks */
                        uint8_t lo = f32_to_e2m1(load_elem(x, in_dtype, r * x_stride + c) * q);
                        uint8_t hi = f32_to_e2m1(load_elem(x, in_dtype, r * x_stride + c + 1) * q);
                        out[r * out_stride + c / 2] = (uint8_t)(lo | (hi << 4));
                    }
                }
            }
        }
    }
    return 0;
}

/*
 * tkqo_cast_back: dequantise (cast.py:40-59).  `sf` is row-major fp32
 * [ceil(T/bm), ceil(H/bk)]; out_fp32 is [T, H].
 */
int tkqo_cast_back(const uint8_t* q, int fmt, int64_t T, int64_t H, int bm, int bk, const float* sf, float* out_fp32) {
    const int64_t nbk = (H + bk - 1) / bk;
    static float e4m3_lut[256];
    static int lut_ready = 0;
    if (!lut_ready) {
        for (int i = 0; i < 256; ++i) {
            int e = (i >> 3) & 0xF, m = i & 7;
            float v = e == 0 ? ldexpf((float)m, -9) : ldexpf(1.0f + (float)m / 8.0f, e - 7);
            if ((i & 0x7F) == 0x7F) v = NAN;
            e4m3_lut[i] = (i & 0x80) ? -v : v;
        }
        lut_ready = 1;
    }
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < T; ++r)
        for (int64_t c = 0; c < H; ++c) {
            float v;
            if (fmt == TKQO_FMT_E4M3) v = e4m3_lut[q[r * H + c]];
            else {
                uint8_t byte = q[r * (H / 2) + c / 2];
                uint8_t code = (c & 1) ? (byte >> 4) : (byte & 0xF);
                v = k_e2m1_values[code & 7];
                if (code & 8) v = -v;
            }
            out_fp32[r * H + c] = v * sf[(r / bm) * nbk + c / bk];
        }
    return 0;
}

/*
 * tkqo_cast_e5m6 (cast_e5m6.py:135-218): per-row groups of `g` channels,
 * maximum 65024, clamp 1e-4.  Output: [T, H/8*3] little-endian uint32 words
 * (viewed as bytes by the caller) and row-major scale bits [T, H/g]; with
 * `ue8m0_bytes` the second output holds the exponent byte instead
 * (cast_e5m6.py:194-198: the rounded exponent, or the truncated one without round_sf).
 */
int tkqo_cast_e5m6(const void* x, int in_dtype, int64_t T, int64_t H, int64_t x_stride, int64_t g, int round_sf,
                   int ue8m0_bytes, uint32_t* out_words, uint32_t* sf_out) {
    if (H % 8 || g <= 0 || H % g || g % 8) return -1;     /* an octet of 8 codes never straddles two groups */
    const int64_t ng = H / g;
    const float max_v = 65024.0f, clamp_min = 1e-4f;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < T; ++r) {
        for (int64_t gi = 0; gi < ng; ++gi) {
            float amax = 0.0f;
            for (int64_t c = gi * g; c < (gi + 1) * g; ++c) {
                float a = fabsf(load_elem(x, in_dtype, r * x_stride + c));
                if (a > amax) amax = a;
            }
            if (amax < clamp_min) amax = clamp_min;
            float ds = amax / max_v;
            uint32_t b = f2u(ds);
            float q;
            uint32_t sf_word;
            if (round_sf) {
                int32_t e = (int32_t)((b - 1u) >> 23) + 1 - 127;
                int32_t ie = 127 - e;
                if (ie < 0) ie = 0;
                q = b == 0 ? 0.0f : u2f((uint32_t)ie << 23);
                sf_word = ue8m0_bytes ? (uint32_t)((e + 127) & 0xFF) : (uint32_t)(e + 127) << 23;
            } else {
                q = b == 0 ? 0.0f : max_v / amax;
                sf_word = ue8m0_bytes ? ((b >> 23) & 0xFFu) : b;
            }
            sf_out[r * ng + gi] = sf_word;
            for (int64_t c = gi * g; c < (gi + 1) * g; c += 8) {
                uint32_t h[8];
                for (int k = 0; k < 8; ++k) h[k] = f32_to_e5m6(load_elem(x, in_dtype, r * x_stride + c + k) * q);
                uint32_t* w = out_words + r * (H / 8 * 3) + (c / 8) * 3;
                w[0] = (h[0] << 20) | (h[1] << 8) | (h[2] >> 4);
                w[1] = (h[2] << 28) | (h[3] << 16) | (h[4] << 4) | (h[5] >> 8);
                w[2] = (h[5] << 24) | (h[6] << 12) | h[7];
            }
        }
    }
    return 0;
}

/*
 * tkqo_cast_back_e5m6 (cast_e5m6.py:103-132, 221-258): words -> 12-bit codes -> fp16 (code << 4) -> fp32,
 * times the row-major fp32 scale of the value's (bm x bk) block.
 */
static inline float f16_bits_to_f32(uint32_t h) {
    uint32_t sign = (h & 0x8000u) << 16, e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0) return u2f(sign) + (sign ? -1.0f : 1.0f) * ldexpf((float)m, -24) * (m != 0);
    if (e == 31) return u2f(sign | 0x7F800000u | (m << 13));
    return u2f(sign | ((e + 112u) << 23) | (m << 13));
}

int tkqo_cast_back_e5m6(const uint32_t* words, int64_t T, int64_t H, int bm, int bk, const float* sf, float* out_fp32) {
    if (H % 8) return -1;
    const int64_t nbk = (H + bk - 1) / bk;
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < T; ++r)
        for (int64_t o = 0; o < H / 8; ++o) {
            const uint32_t* w = words + r * (H / 8 * 3) + o * 3;
            uint32_t h[8] = {w[0] >> 16, w[0] >> 4, (w[0] << 8) | (w[1] >> 24), w[1] >> 12, w[1], (w[1] << 12) | (w[2] >> 20),
                             w[2] >> 8, w[2] << 4};
            for (int i = 0; i < 8; ++i) {
                int64_t c = o * 8 + i;
                out_fp32[r * H + c] = f16_bits_to_f32(h[i] & 0xFFF0u) * sf[(r / bm) * nbk + c / bk];
            }
        }
    return 0;
}

/* ---- exp(x), fp32, built from IEEE add/mul/fma and integer operations only, so that the CUDA copy
 * (csrc/tkq_common.cuh, tkq_expf) produces the same bits.  The argument is clamped to [-87, 88] (the
 * result stays a normal number; callers only use 1 + exp(x), for which the clamp changes nothing
 * below -87 and replaces +inf by 1.65e38 above 88).  x = j*ln2 + r with a two-constant ln2,
 * exp(r) = 1 + r + r^2 q(r) with a fitted degree-4 q, the last sum compensated, 2^j applied by adding
 * j to the exponent field (j sits in the low mantissa bits of t).
 * Measured: at most 0.77 ulp, 95% of results correctly rounded (tests/test_oracle_units.py). ---- */
float tkq_expf(float x) {
    x = fminf(fmaxf(x, -87.0f), 88.0f);
    const float shift = 12582912.0f;                        /* 1.5 * 2^23 */
    float t = fmaf(x, 1.4426950408889634f, shift);
    float jf = t - shift;
    float r = fmaf(jf, -0.693145751953125f, x);             /* ln2 high part, exact product */
    r = fmaf(jf, -1.428606765330187e-06f, r);               /* ln2 low part */
    float q = 0.001381455804221332f;
    q = fmaf(q, r, 0.008368736132979393f);
    q = fmaf(q, r, 0.04166838899254799f);
    q = fmaf(q, r, 0.1666652113199234f);
    q = fmaf(q, r, 0.4999999403953552f);
    float wl = (r * r) * q;                                 /* exp(r) = 1 + r + wl */
    float s = 1.0f + r;
    float e = (1.0f - s) + r;                               /* exact rounding error of s */
    float p = s + (e + wl);
    return u2f(f2u(p) + (f2u(t) << 23));
}

void tkqo_expf_array(const float* x, float* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = tkq_expf(x[i]);
}

/*
 * tkqo_swiglu_forward (swiglu.py:47-88): y[T, H] = silu(x[:, :H]) * x[:, H:]
 * in fp32, evaluated as (g / (1 + exp(-g))) * u, then times the row weight.
 *   clamp        < 0 disables; otherwise g = min(g, clamp), u = clamp(u, -clamp, clamp)
 *   counts       optional int64[3], incremented by the numbers of g > clamp, u > clamp, u < -clamp
 *   pos_to_token_topk / topk_weights: optional row weights; a negative position gives weight 0
 */
int tkqo_swiglu_forward(const void* x, int in_dtype, int64_t T, int64_t H, float clamp, int64_t* counts,
                        const int32_t* pos_to_token_topk, const float* topk_weights, float* y) {
    int64_t c0 = 0, c1 = 0, c2 = 0;
#pragma omp parallel for schedule(static) reduction(+ : c0, c1, c2)
    for (int64_t r = 0; r < T; ++r) {
        float w = 1.0f;
        if (pos_to_token_topk) w = pos_to_token_topk[r] >= 0 ? topk_weights[pos_to_token_topk[r]] : 0.0f;
        for (int64_t c = 0; c < H; ++c) {
            float g = load_elem(x, in_dtype, r * 2 * H + c);
            float u = load_elem(x, in_dtype, r * 2 * H + H + c);
            if (clamp >= 0.0f) {
                c0 += g > clamp;
                c1 += u > clamp;
                c2 += u < -clamp;
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            float v = g / (1.0f + tkq_expf(-g)) * u;
            if (pos_to_token_topk) v = v * w;
            y[r * H + c] = v;
        }
    }
    if (counts && clamp >= 0.0f) {
        counts[0] += c0;
        counts[1] += c1;
        counts[2] += c2;
    }
    return 0;
}

/*
 * tkqo_swiglu_backward (swiglu.py:152-226), on the already dequantised input x[T, 2H] (fp32) and the bf16
 * gradient d[T, H].  With g / u the two halves of a row, w the row's routing weight (0 for a negative
 * position), t = 1 + exp(-g), a = g / t * u, s = 1 / t, q = d * w * s:
 *   out[T, H]      = a * w
 *   x_grad[T, 2H]  = [q * u * fma(g, 1 - s, 1), q * g], 0 where the clamp was active (swiglu.py:200-211;
 *                    the fused multiply-add is the one elementwise_fma, swiglu.py:91-95, asks for)
 *   weight_grad[pos_to_token_topk[r]] = sum_c d * a   (summed in double; entries without a row keep the
 *                    caller's initial value, which the numpy wrapper sets to 0 as swiglu.py:217 does)
 *   clamp < 0 disables the clamp
 */
int tkqo_swiglu_backward(const float* x, const uint16_t* grad_out, int64_t T, int64_t H, float clamp,
                         const int32_t* pos_to_token_topk, const float* weight, float* out, float* x_grad,
                         float* weight_grad) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < T; ++r) {
        const int32_t index = pos_to_token_topk[r];
        const float w = index >= 0 ? weight[index] : 0.0f;
        double acc = 0.0;
        for (int64_t c = 0; c < H; ++c) {
            float g = x[r * 2 * H + c];
            float u = x[r * 2 * H + H + c];
            int clamped_g = 0, clamped_u = 0;
            if (clamp >= 0.0f) {
                clamped_g = g > clamp;
                clamped_u = u > clamp || u < -clamp;
                if (g > clamp) g = clamp;
                if (u > clamp) u = clamp;
                if (u < -clamp) u = -clamp;
            }
            const float d = u2f((uint32_t)grad_out[r * H + c] << 16);
            const float t = 1.0f + tkq_expf(-g);
            const float a = g / t * u;
            acc += (double)(d * a);
            const float s = 1.0f / t;
            const float q = d * w * s;
            out[r * H + c] = a * w;
            const float vg = q * u * fmaf(g, 1.0f - s, 1.0f);
            const float vu = q * g;
            x_grad[r * 2 * H + c] = clamped_g ? 0.0f : vg;
            x_grad[r * 2 * H + H + c] = clamped_u ? 0.0f : vu;
        }
        if (index >= 0) weight_grad[index] = (float)acc;
    }
    return 0;
}

/* element converters exported for the unit tests */
void tkqo_f32_to_e4m3_array(const float* x, uint8_t* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) {
        float v = x[i];
        if (v > 448.0f) v = 448.0f;
        if (v < -448.0f) v = -448.0f;
        y[i] = f32_to_e4m3fn(v);
    }
}
void tkqo_f32_to_e2m1_array(const float* x, uint8_t* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = f32_to_e2m1(x[i]);
}
void tkqo_f32_to_e5m6_array(const float* x, uint32_t* y, int64_t n) {
    for (int64_t i = 0; i < n; ++i) y[i] = f32_to_e5m6(x[i]);
}
