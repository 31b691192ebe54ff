// "Sources": how a lane obtains the 16 consecutive fp32 values it owns.
//
// A source has a Raw type (the registers of the global loads, kept untouched so
// that several loads stay in flight), issue() that starts the loads, and
// unpack() that turns Raw into 16 floats.  Two families exist:
//   PlainSource<DT>   the input tensor itself (bf16 or fp32)
//   SwigluSource<DT>  silu(gate) * up (* row weight), gate at column c and up at
//                     column c + hidden of a [tokens, 2 * hidden] tensor
// 256-bit loads need 32-byte aligned addresses; `wide = false` falls back to pairs
// of 128-bit loads for tensors that are only 16-byte aligned.
#pragma once

#include "tkq_common.cuh"

namespace tkq {

template <int DT>
struct PlainSource;

template <>
struct PlainSource<TKQ_DT_BF16> {
    static constexpr int kElemBytes = 2;
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems * 2; }
    struct Raw {
        U32x8 a;
    };
    __device__ __forceinline__ static void zero(Raw& r) {
#pragma unroll
        for (int i = 0; i < 8; ++i) r.a.v[i] = 0;
    }
    // p points at the lane's first element; `wide` = p is 32-byte aligned
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool wide) {
        if (wide) {
            r.a = ldg256(p);
        } else {
            const U32x4 lo = ldg128(p), hi = ldg128(static_cast<const uint8_t*>(p) + 16);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                r.a.v[i] = lo.v[i];
                r.a.v[4 + i] = hi.v[i];
            }
        }
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = bf16_lo(r.a.v[i]);
            v[2 * i + 1] = bf16_hi(r.a.v[i]);
        }
    }
};

template <>
struct PlainSource<TKQ_DT_FP32> {
    static constexpr int kElemBytes = 4;
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems * 4; }
    struct Raw {
        U32x8 a, b;
    };
    __device__ __forceinline__ static void zero(Raw& r) {
#pragma unroll
        for (int i = 0; i < 8; ++i) r.a.v[i] = r.b.v[i] = 0;
    }
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool wide) {
        if (wide) {
            r.a = ldg256(p);
            r.b = ldg256(static_cast<const uint8_t*>(p) + 32);
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const U32x4 a = ldg128(static_cast<const uint8_t*>(p) + 16 * h);
                const U32x4 b = ldg128(static_cast<const uint8_t*>(p) + 32 + 16 * h);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    r.a.v[4 * h + i] = a.v[i];
                    r.b.v[4 * h + i] = b.v[i];
                }
            }
        }
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[i] = __uint_as_float(r.a.v[i]);
            v[8 + i] = __uint_as_float(r.b.v[i]);
        }
    }
};

// Clamp bookkeeping of the SwiGLU source: per-thread counters of clamped inputs.
struct ClampCounters {
    uint32_t gate_hi = 0, up_hi = 0, up_lo = 0;
};

template <int DT>
struct SwigluSource {
    using P = PlainSource<DT>;
    static constexpr int kElemBytes = P::kElemBytes;
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems * kElemBytes; }
    struct Raw {
        typename P::Raw g, u;
    };
    __device__ __forceinline__ static void zero(Raw& r) {
        P::zero(r.g);
        P::zero(r.u);
    }
    // p points at the lane's first gate element; the up half is `hidden` elements further
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool wide, int64_t hidden) {
        P::issue(r.g, p, wide);
        P::issue(r.u, static_cast<const uint8_t*>(p) + hidden * kElemBytes, wide);
    }
    // kClamp: apply the clamp; kCount: also count what was clamped; kWeight: multiply by w.
    // `bf16_gates`: every gate value that reaches the activation is a bf16 number (bf16 input and, if clamping,
    // a bf16-representable clamp value), which allows the cheaper in-range evaluation.
    template <bool kClamp, bool kCount, bool kWeight>
    __device__ __forceinline__ static void unpack(const Raw& r, float* v, float clamp, float w, ClampCounters& cnt,
                                                  bool bf16_gates) {
        float g[16], u[16];
        P::unpack(r.g, g);
        P::unpack(r.u, u);
        float lo = 1.0f, hi = 0.0f;  // smallest and largest gate magnitude of the chunk
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            lo = min3_abs(lo, g[i], g[i + 1]);
            hi = max3_abs(hi, g[i], g[i + 1]);
        }
        if (kClamp) {
            // the clamp (and its counters) only when something in the chunk can reach it: one maximum per two values
            // instead of three comparisons and three selects per value
            float u_hi = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i += 2) u_hi = max3_abs(u_hi, u[i], u[i + 1]);
            if (hi > clamp || u_hi > clamp) {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    if (kCount) {
                        cnt.gate_hi += g[i] > clamp;
                        cnt.up_hi += u[i] > clamp;
                        cnt.up_lo += u[i] < -clamp;
                    }
                    g[i] = g[i] > clamp ? clamp : g[i];
                    u[i] = u[i] > clamp ? clamp : u[i];
                    u[i] = u[i] < -clamp ? -clamp : u[i];
                }
                lo = 1.0f, hi = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    lo = min3_abs(lo, g[i], g[i + 1]);
                    hi = max3_abs(hi, g[i], g[i + 1]);
                }
            }
        }
        if (bf16_gates && lo >= 9.094947017729282e-13f && hi <= 44.0f) {  // 2^-40 <= |g| <= 44 for the whole chunk
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 y = swiglu_bf16_in_range2(make_float2(g[i], g[i + 1]), make_float2(u[i], u[i + 1]));
                v[i] = y.x;
                v[i + 1] = y.y;
            }
        } else if (hi <= 44.0f) {  // gates of any mantissa (fp32 input): exp without its clamp, IEEE division
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 g2 = make_float2(g[i], g[i + 1]);
                const float2 d = add2(splat2(1.0f), tkq_expf2_noclamp(mul2(g2, splat2(-1.0f))));
                const float2 y = mul2(make_float2(__fdiv_rn(g2.x, d.x), __fdiv_rn(g2.y, d.y)), make_float2(u[i], u[i + 1]));
                v[i] = y.x;
                v[i + 1] = y.y;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = swiglu(g[i], u[i]);
        }
        if (kWeight && w != 1.0f) {  // uniform over the row; multiplying by exactly 1 would change nothing
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __fmul_rn(v[i], w);
        }
    }
};

// Already quantized input (reference: the with_sf branch of tile_kernels/quant/per_token_cast_kernel.py:87-126
// and tile_kernels/torch/cast.py:86-97): FP8 e4m3 bytes or packed FP4 e2m1 nibbles plus one scale per input
// block.  A lane's 16 values lie in one input block (blocks are at least 32 wide), so unpack() takes the one
// scale and returns float(x) * scale, the fp32 product the reference forms before it takes the maximum.
template <int QFMT>
struct QuantSource;

template <>
struct QuantSource<TKQ_FMT_E4M3> {
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems; }
    struct Raw {
        U32x4 a;
    };
    __device__ __forceinline__ static void zero(Raw& r) { r.a.v[0] = r.a.v[1] = r.a.v[2] = r.a.v[3] = 0; }
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool) { r.a = ldg128(p); }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v, float scale) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const uint16_t pair = static_cast<uint16_t>(r.a.v[i] >> (16 * h));
                uint32_t f16x2;
                asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(f16x2) : "h"(pair));
                const __half2 hv = *reinterpret_cast<const __half2*>(&f16x2);
                const float2 t = mul2(__half22float2(hv), splat2(scale));
                v[4 * i + 2 * h] = t.x;
                v[4 * i + 2 * h + 1] = t.y;
            }
        }
    }
};

template <>
struct QuantSource<TKQ_FMT_E2M1> {
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems / 2; }
    struct Raw {
        uint32_t lo, hi;
    };
    __device__ __forceinline__ static void zero(Raw& r) { r.lo = r.hi = 0; }
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool) {
        asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(r.lo), "=r"(r.hi) : "l"(p));
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v, float scale) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t word = i < 4 ? r.lo : r.hi;
            const uint16_t byte = static_cast<uint16_t>((word >> (8 * (i & 3))) & 0xFFu);  // two codes, even index low
            uint32_t f16x2;
            asm("{ .reg .b8 t; cvt.u8.u16 t, %1; cvt.rn.f16x2.e2m1x2 %0, t; }" : "=r"(f16x2) : "h"(byte));
            const __half2 hv = *reinterpret_cast<const __half2*>(&f16x2);
            const float2 t = mul2(__half22float2(hv), splat2(scale));
            v[2 * i] = t.x;
            v[2 * i + 1] = t.y;
        }
    }
};

// ---------------------------------------------------------------------------
// The common tail of every cast: 16 scaled values of one lane -> packed codes.
// ---------------------------------------------------------------------------
__device__ __forceinline__ float absmax16(const float* v) {
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 16; i += 2) m = max3_abs(m, v[i], v[i + 1]);
    return m;
}

// e4m3: 16 bytes at out_row + col
__device__ __forceinline__ void quantize_store_e4m3x16(const float* v, float inv, uint8_t* dst) {
    float s[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {  // packed pairs: one issued instruction scales two values
        const float2 t = mul2(make_float2(v[i], v[i + 1]), splat2(inv));
        s[i] = t.x;
        s[i + 1] = t.y;
    }
    stg128(dst, cvt_e4m3x4(s[0], s[1], s[2], s[3]), cvt_e4m3x4(s[4], s[5], s[6], s[7]),
           cvt_e4m3x4(s[8], s[9], s[10], s[11]), cvt_e4m3x4(s[12], s[13], s[14], s[15]));
}

// e2m1: 8 bytes at out_row + col / 2
__device__ __forceinline__ void quantize_store_e2m1x16(const float* v, float inv, uint8_t* dst) {
    float s[16];
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        const float2 t = mul2(make_float2(v[i], v[i + 1]), splat2(inv));
        s[i] = t.x;
        s[i + 1] = t.y;
    }
    stg64(dst, cvt_e2m1x8(s), cvt_e2m1x8(s + 8));
}

}  // namespace tkq
