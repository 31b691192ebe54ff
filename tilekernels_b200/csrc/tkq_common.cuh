// Device-side building blocks shared by every cast kernel: wide global loads and
// stores, bf16 unpacking, the scale arithmetic, the saturating converters and the
// scale-factor addressing.  sm_100a only.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tkquant.h"

namespace tkq {

constexpr unsigned kFullMask = 0xffffffffu;

struct alignas(32) U32x8 {
    uint32_t v[8];
};
struct alignas(16) U32x4 {
    uint32_t v[4];
};

// ---------------------------------------------------------------------------
// Global memory access.  Inputs are read once and outputs written once, so
// loads bypass L1 (256-bit loads are also marked evict-first in L2, a hint PTX only
// accepts on that width); stores do not allocate in L1.
// sm_100 has 256-bit global loads: one instruction moves 16 bf16 per lane.
// ---------------------------------------------------------------------------
__device__ __forceinline__ U32x8 ldg256(const void* p) {
    U32x8 r;
    asm volatile("ld.global.nc.L1::no_allocate.L2::evict_first.v8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3]), "=r"(r.v[4]), "=r"(r.v[5]), "=r"(r.v[6]),
                   "=r"(r.v[7])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ U32x4 ldg128(const void* p) {
    U32x4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.v[0]), "=r"(r.v[1]), "=r"(r.v[2]), "=r"(r.v[3])
                 : "l"(p));
    return r;
}

__device__ __forceinline__ void stg128(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.global.L1::no_allocate.v4.b32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d)
                 : "memory");
}

// 256-bit store; p must be 32-byte aligned
__device__ __forceinline__ void stg256(void* p, const uint32_t* w) {
    asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}

__device__ __forceinline__ void stg64(void* p, uint32_t a, uint32_t b) {
    asm volatile("st.global.L1::no_allocate.v2.b32 [%0], {%1,%2};" ::"l"(p), "r"(a), "r"(b) : "memory");
}

__device__ __forceinline__ void stg32(void* p, uint32_t a) {
    asm volatile("st.global.L1::no_allocate.b32 [%0], %1;" ::"l"(p), "r"(a) : "memory");
}

// A 32-bit word holds two bf16: element 2i in the low half, 2i+1 in the high half.
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

// ---------------------------------------------------------------------------
// Scale arithmetic (reference: tile_kernels/quant/common.py:196-216 get_sf_and_inv;
// oracle form tile_kernels/torch/cast.py:147-164).
//   sf  = max(amax, clamp) / MAX                       IEEE division
//   inv = MAX / max(amax, clamp)                       second division, not 1/sf
// With rounding, sf becomes the next power of two >= sf and inv its exact
// reciprocal.  `e8` is the biased exponent byte stored in ue8m0 mode: the rounded
// exponent, or the truncated one when rounding is off (what the oracle stores).
// ---------------------------------------------------------------------------
struct Scale {
    float sf;
    float inv;
    uint32_t e8;
};

template <int FMT>
struct FmtTraits;
template <>
struct FmtTraits<TKQ_FMT_E4M3> {
    static constexpr float kMax = 448.0f;           // 1.75 * 2^8
    static constexpr uint32_t kMantCarry = 0x1FFFFFu;  // 0x800000 - mantissa(1.75) - 1
    static constexpr uint32_t kMaxExp = 8;
};
template <>
struct FmtTraits<TKQ_FMT_E2M1> {
    static constexpr float kMax = 6.0f;  // 1.5 * 2^2
    static constexpr uint32_t kMantCarry = 0x3FFFFFu;
    static constexpr uint32_t kMaxExp = 2;
};
template <>
struct FmtTraits<TKQ_FMT_E5M6> {
    static constexpr float kMax = 65024.0f;  // 1.984375 * 2^15
    static constexpr uint32_t kMantCarry = 0x01FFFFu;
    static constexpr uint32_t kMaxExp = 15;
};

// General form, any clamp and both rounding modes.
__device__ __forceinline__ Scale make_scale(float amax, float clamp_min, float max_q, bool round_sf) {
    Scale s;
    const float a = fmaxf(amax, clamp_min);
    const float sf = __fdiv_rn(a, max_q);
    const uint32_t bits = __float_as_uint(sf);
    if (!round_sf) {
        s.sf = sf;
        s.inv = bits == 0 ? 0.0f : __fdiv_rn(max_q, a);
        s.e8 = bits >> 23;
        return s;
    }
    // ceil(log2(sf)) as a biased exponent: 2^(e-127) >= sf > 2^(e-128)
    const uint32_t e = bits == 0 ? 0u : ((bits - 1u) >> 23) + 1u;
    s.sf = __uint_as_float(e << 23);
    s.inv = bits == 0 ? 0.0f : __uint_as_float((254u - e) << 23);
    s.e8 = e;
    return s;
}

// Power-of-two scales without the division.  With MAX = c * 2^p (1 <= c < 2) and a = m * 2^E:
// ceil(log2(RN(a / MAX))) = E - p + (m > c), so the biased exponent is ((bits(a) + kMantCarry) >> 23) - p.
// Equal to make_scale(..., round_sf = true) for every fp32 a with a / MAX normal (checked exhaustively on
// the CPU for the three formats); the caller guarantees that through clamp_min >= MAX * 2^-126.
template <int FMT>
__device__ __forceinline__ Scale make_scale_pow2(float amax, float clamp_min) {
    Scale s;
    const uint32_t bits = __float_as_uint(fmaxf(amax, clamp_min));
    const uint32_t e = ((bits + FmtTraits<FMT>::kMantCarry) >> 23) - FmtTraits<FMT>::kMaxExp;
    s.sf = __uint_as_float(e << 23);
    s.inv = __uint_as_float((254u - e) << 23);
    s.e8 = e;
    return s;
}

// kFast: the host established round_sf && clamp_min >= MAX * 2^-126.
template <int FMT>
__device__ __forceinline__ Scale make_scale_for(float amax, float clamp_min, bool round_sf, bool fast_pow2) {
    return fast_pow2 ? make_scale_pow2<FMT>(amax, clamp_min) : make_scale(amax, clamp_min, FmtTraits<FMT>::kMax, round_sf);
}

// max(|a|, |b|, |c|) in one instruction (three-input max of sm_100)
__device__ __forceinline__ float max3_abs(float a, float b, float c) {
    float d;
    asm("max.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// max of two pairs of unsigned 16-bit values; non-negative bf16 or f16 numbers order like their bit patterns
__device__ __forceinline__ uint32_t max_u16x2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("max.u16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

// Where a scale goes (reference: tile_kernels/quant/common.py:238-244 store_sf).
// m = token-block index, k = channel-block index.
__device__ __forceinline__ void store_sf_f32(void* sf, int64_t sf_stride, bool col_major, int64_t m, int64_t k,
                                             float v) {
    float* p = static_cast<float*>(sf);
    p[col_major ? k * sf_stride + m : m * sf_stride + k] = v;
}

__device__ __forceinline__ float load_sf_f32_row_major(const void* sf, int64_t sf_stride, int64_t m, int64_t k) {
    return static_cast<const float*>(sf)[m * sf_stride + k];
}

// Packed ue8m0: one 32-bit word holds the exponent bytes of channel blocks 4*kq .. 4*kq+3
// of token-block m; sf_stride counts bytes between consecutive kq.
__device__ __forceinline__ void store_sf_ue8m0_word(void* sf, int64_t sf_stride, int64_t m, int64_t kq, uint32_t word) {
    uint8_t* p = static_cast<uint8_t*>(sf) + kq * sf_stride + 4 * m;
    *reinterpret_cast<uint32_t*>(p) = word;
}

// One exponent byte of the packed layout.  When k is the last channel block the remaining bytes of its
// word are zeroed, so that the padding of the layout is deterministic.
__device__ __forceinline__ void store_sf_ue8m0_byte(void* sf, int64_t sf_stride, int64_t m, uint32_t k, uint32_t num_k,
                                                    uint32_t e8) {
    uint8_t* p = static_cast<uint8_t*>(sf) + static_cast<int64_t>(k >> 2) * sf_stride + 4 * m;
    p[k & 3] = static_cast<uint8_t>(e8);
    if (k == num_k - 1)
        for (uint32_t b = (k & 3) + 1; b < 4; ++b) p[b] = 0;
}

// ---------------------------------------------------------------------------
// Converters.  cvt.rn.satfinite rounds to nearest even and saturates to the
// largest finite value, which equals the reference's clamp-then-convert.
// The first source operand lands in the upper half of the result.
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t cvt_e4m3x2(float lo, float hi) {
    uint16_t r;
    asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
    return r;
}

// Four values -> four bytes (a in the lowest).  Both conversions and the merge of the two halves sit in one
// asm block so that the assembler can write each half of the result register directly.
__device__ __forceinline__ uint32_t cvt_e4m3x4(float a, float b, float c, float d) {
    uint32_t r;
    asm("{ .reg .b16 lo, hi;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 lo, %2, %1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f32 hi, %4, %3;\n\t"
        "mov.b32 %0, {lo, hi}; }"
        : "=r"(r)
        : "f"(a), "f"(b), "f"(c), "f"(d));
    return r;
}

// Two values -> one byte, `lo` in the low nibble.
__device__ __forceinline__ uint32_t cvt_e2m1x2(float lo, float hi) {
    uint32_t r;
    asm("{ .reg .b8 t; cvt.rn.satfinite.e2m1x2.f32 t, %1, %2; cvt.u32.u8 %0, t; }" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

__device__ __forceinline__ uint32_t cvt_e2m1x8(const float* v) {
    uint32_t r;
    asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n\t"
        "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n\t"
        "mov.b32 %0, {b0, b1, b2, b3}; }"
        : "=r"(r)
        : "f"(v[0]), "f"(v[1]), "f"(v[2]), "f"(v[3]), "f"(v[4]), "f"(v[5]), "f"(v[6]), "f"(v[7]));
    return r;
}

// fp32 -> 12-bit E5M6 code, the reference's definition: fp16 with round-toward-zero, cut to 12 bits, then
// round to nearest even on the 17 low bits of the fp32
// (reference: tile_kernels/quant/per_token_cast_to_e5m6_kernel.py:44-51).
__device__ __forceinline__ uint32_t cvt_e5m6(float v) {
    const uint32_t h = __half_as_ushort(__float2half_rz(v));
    uint32_t c = h >> 4;
    const uint32_t rem = __float_as_uint(v) & 0x1FFFFu;
    c += ((c & 1u) + rem > 0x10000u) ? 1u : 0u;
    return c & 0xFFFu;
}

// The same code for 2^-14 <= |v| < 65520 (the fp16-normal range), where the definition above is plain
// round-to-nearest-even of v to 1+6 significant bits followed by a re-bias of the exponent.  Everything that
// can run on the floating-point / multiply-add pipe does, because the integer pipe is what limits this cast:
//   * v is first scaled by 2^-112 (exact in this range), which re-biases the exponent for free;
//   * the rounding is a Veltkamp split, c = v * (2^17 + 1), hi = c - (c - v): v rounded to nearest even at
//     7 significant bits (checked against integer RNE for every mantissa of 44 binades on the CPU);
//   * hi >> 17 is then sign(1) | 000 | exponent(5) | mantissa(6); one multiply-add moves the sign from
//     bit 14 to bit 11.
__device__ __forceinline__ uint32_t mad_u32(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ uint32_t cvt_e5m6_normal(float v) {
    const float vs = __fmul_rn(v, 1.925929944387236e-34f);  // 2^-112
    const float c = __fmul_rn(vs, 131073.0f);
    const float hi = __fsub_rn(c, __fsub_rn(c, vs));
    const uint32_t bits = __float_as_uint(hi);
    const uint32_t t = bits >> 17;
    return mad_u32(bits >> 31, 0u - 0x3800u, t);  // t - sign * (2^14 - 2^11)
}

// min(|a|, |b|, |c|)
__device__ __forceinline__ float min3_abs(float a, float b, float c) {
    float d;
    asm("min.abs.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Eight codes -> three words (per_token_cast_to_e5m6_kernel.py:53-64).  The fields do not overlap, so every
// shift-and-or is written as a multiply-add.
__device__ __forceinline__ void pack_e5m6x8(const uint32_t* c, uint32_t* w) {
    w[0] = mad_u32(c[0], 1u << 20, mad_u32(c[1], 1u << 8, c[2] >> 4));
    w[1] = mad_u32(c[2], 1u << 28, mad_u32(c[3], 1u << 16, mad_u32(c[4], 1u << 4, c[5] >> 8)));
    w[2] = mad_u32(c[5], 1u << 24, mad_u32(c[6], 1u << 12, c[7]));
}

// ---------------------------------------------------------------------------
// exp(x) from IEEE add/mul/fma and integer operations only, so that the CPU checker
// (oracle/tkq_oracle.c, tkq_expf: same operations in the same order) reproduces it bit for bit;
// CUDA's own expf goes through the hardware ex2 approximation, which no CPU can reproduce.
// Argument clamped to [-87, 88]; within 1 ulp there; 18 instructions.
// ---------------------------------------------------------------------------
template <bool kClampArg>
__device__ __forceinline__ float tkq_expf_impl(float x) {
    if (kClampArg) x = fminf(fmaxf(x, -87.0f), 88.0f);
    const float shift = 12582912.0f;
    const float t = __fmaf_rn(x, 1.4426950408889634f, shift);
    const float jf = __fsub_rn(t, shift);
    float r = __fmaf_rn(jf, -0.693145751953125f, x);
    r = __fmaf_rn(jf, -1.428606765330187e-06f, r);
    float q = 0.001381455804221332f;
    q = __fmaf_rn(q, r, 0.008368736132979393f);
    q = __fmaf_rn(q, r, 0.04166838899254799f);
    q = __fmaf_rn(q, r, 0.1666652113199234f);
    q = __fmaf_rn(q, r, 0.4999999403953552f);
    const float wl = __fmul_rn(__fmul_rn(r, r), q);
    const float s = __fadd_rn(1.0f, r);
    const float e = __fadd_rn(__fsub_rn(1.0f, s), r);
    const float p = __fadd_rn(s, __fadd_rn(e, wl));
    return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}

__device__ __forceinline__ float tkq_expf(float x) { return tkq_expf_impl<true>(x); }

// silu(g) * u evaluated as (g / (1 + exp(-g))) * u with IEEE division
// (reference: tile_kernels/quant/swiglu_forward_and_per_token_cast_kernel.py:140-144).
__device__ __forceinline__ float swiglu(float g, float u) {
    const float d = __fadd_rn(1.0f, tkq_expf(-g));
    return __fmul_rn(__fdiv_rn(g, d), u);
}

// The same value for 2^-40 <= |g| <= 44 with g a bf16 number, in 12 fewer instructions:
//   * the argument of exp needs no clamp;
//   * g / d (d = 1 + exp(-g) in [1, 2^64)) is computed as reciprocal approximation, one Newton step, quotient,
//     exact residual, correction.  For bf16 numerators this sequence was compared with IEEE division on the
//     GPU for all 2^7 numerator mantissas x all 2^23 denominator mantissas over 41 exponent offsets and several
//     denominator binades: no difference (in this range no intermediate under- or overflows, so the result
//     depends on the two mantissas and the exponent difference only).
__device__ __forceinline__ float swiglu_bf16_in_range(float g, float u) {
    const float d = __fadd_rn(1.0f, tkq_expf_impl<false>(-g));
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(d));
    y = __fmaf_rn(y, __fmaf_rn(-d, y, 1.0f), y);
    const float q = __fmul_rn(g, y);
    return __fmul_rn(__fmaf_rn(__fmaf_rn(-d, q, g), y, q), u);
}

// ---------------------------------------------------------------------------
// Packed fp32 pairs.  sm_100 executes fma / add / mul on two IEEE binary32 values per issued instruction
// (fma.rn.f32x2 and friends); every element is rounded exactly as by the scalar instruction, so the pair forms
// below return the same bits as their scalar counterparts above at half the issue slots.  The kernels that are
// bound by instruction issue (fused SwiGLU casts) use them.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float2 splat2(float x) { return make_float2(x, x); }
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ float2 add2(float2 a, float2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ float2 mul2(float2 a, float2 b) { return __fmul2_rn(a, b); }

// tkq_expf_impl<false> on two arguments (no argument clamp: callers guarantee |x| <= 87)
__device__ __forceinline__ float2 tkq_expf2_noclamp(float2 x) {
    const float2 t = fma2(x, splat2(1.4426950408889634f), splat2(12582912.0f));
    const float2 jf = add2(t, splat2(-12582912.0f));
    float2 r = fma2(jf, splat2(-0.693145751953125f), x);
    r = fma2(jf, splat2(-1.428606765330187e-06f), r);
    float2 q = splat2(0.001381455804221332f);
    q = fma2(q, r, splat2(0.008368736132979393f));
    q = fma2(q, r, splat2(0.04166838899254799f));
    q = fma2(q, r, splat2(0.1666652113199234f));
    q = fma2(q, r, splat2(0.4999999403953552f));
    const float2 wl = mul2(mul2(r, r), q);
    const float2 s = add2(splat2(1.0f), r);
    const float2 e = add2(fma2(s, splat2(-1.0f), splat2(1.0f)), r);  // (1 - s) + r
    const float2 p = add2(s, add2(e, wl));
    return make_float2(__uint_as_float(mad_u32(__float_as_uint(t.x), 1u << 23, __float_as_uint(p.x))),
                       __uint_as_float(mad_u32(__float_as_uint(t.y), 1u << 23, __float_as_uint(p.y))));
}

// cvt_e5m6_normal for two values, with the scaling folded into the split: for v in the fp16-normal range
// c = v * (131073 * 2^-112) and d = fma(v, -2^-112, c) are exactly the c and c - vs of the scalar form (scaling
// by a power of two is exact there), so hi = c - d is the same number.
__device__ __forceinline__ void cvt_e5m6_normal2(float2 v, uint32_t& c0, uint32_t& c1) {
    const float2 c = mul2(v, splat2(131073.0f * 1.925929944387236e-34f));
    const float2 d = fma2(v, splat2(-1.925929944387236e-34f), c);
    const float2 hi = fma2(d, splat2(-1.0f), c);  // c - d
    const uint32_t b0 = __float_as_uint(hi.x), b1 = __float_as_uint(hi.y);
    c0 = mad_u32(b0 >> 31, 0u - 0x3800u, b0 >> 17);
    c1 = mad_u32(b1 >> 31, 0u - 0x3800u, b1 >> 17);
}

// 1 / d refined by one Newton step from the hardware approximation, for both elements
__device__ __forceinline__ float2 refined_rcp2(float2 d, float2 neg_d) {
    float2 y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y.x) : "f"(d.x));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y.y) : "f"(d.y));
    return fma2(y, fma2(neg_d, y, splat2(1.0f)), y);
}

// swiglu_bf16_in_range on two (gate, up) pairs
__device__ __forceinline__ float2 swiglu_bf16_in_range2(float2 g, float2 u) {
    const float2 d = add2(splat2(1.0f), tkq_expf2_noclamp(mul2(g, splat2(-1.0f))));
    const float2 neg_d = mul2(d, splat2(-1.0f));
    const float2 y = refined_rcp2(d, neg_d);
    const float2 q = mul2(g, y);
    return mul2(fma2(fma2(neg_d, q, g), y, q), u);
}

// ---------------------------------------------------------------------------
// Host-side helpers
// ---------------------------------------------------------------------------
int set_error(int code, const char* msg);          // records msg for tkq_last_error_string, returns code
int check_launch(const char* what);                 // cudaGetLastError -> return code
int device_sm_count();                              // cached per device

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace tkq
