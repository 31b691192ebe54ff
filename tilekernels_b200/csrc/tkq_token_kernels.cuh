// Row-wise ("per-token") cast kernels.
//
// Work decomposition.  Every lane owns 16 consecutive values of one row, so a
// warp covers a 512-value span ("step") of a row per item:
//   * bf16 input: one 256-bit load per lane, 1 KB contiguous per warp
//   * e4m3 output: one 128-bit store per lane, 512 B contiguous per warp
//   * a 128-wide scale group is 8 adjacent lanes, reduced with 3 shuffles, and the
//     4 groups of a step are exactly one packed ue8m0 word
// group_cast_kernel handles scale groups of 16..128 values (LPG = lanes per group);
// row_cast_kernel handles one scale per row, reduced across the thread block.
#pragma once

#include <cstdlib>

#include "tkq_async.cuh"
#include "tkq_launch.cuh"
#include "tkq_sources.cuh"

namespace tkq {

struct TokenCastParams {
    const void* x;
    uint8_t* out;
    void* sf;
    int64_t x_stride;    // elements between rows of x
    int64_t sf_stride;   // see tkquant.h
    int64_t out_stride;  // bytes between rows of out
    int64_t num_tokens;
    int64_t hidden;          // values per row that are quantized (SwiGLU: half the input columns)
    uint32_t items_per_row;  // work items per row; an item is U consecutive 512-value steps
    uint32_t num_groups;     // scale groups per row
    uint32_t total_items;    // num_tokens * items_per_row
    uint32_t stride_rows;    // (warps in the grid) / items_per_row   -- the step of the grid-stride loop,
    uint32_t stride_items;   // (warps in the grid) % items_per_row      split so the loop needs no division
    uint32_t flags;
    float clamp_min;
    bool wide_loads;  // every row of x starts on a 32-byte boundary: 256-bit loads are legal
    bool fast_pow2;   // round_sf with a clamp that keeps the scale normal: division-free scale path
    // SwiGLU only
    const int32_t* pos_to_token_topk;
    const float* topk_weights;
    const int32_t* pos_to_expert;
    float swiglu_clamp;
    bool bf16_gates;  // SwiGLU: bf16 input and (no clamp or a bf16-representable clamp value)
    unsigned long long* clamped_count;
    // already quantized input only: its scales (layouts as for the output scales) and their block shape
    const void* in_sf;
    int64_t in_sf_stride;
    uint32_t in_sf_flags;  // TKQ_SF_COL_MAJOR, TKQ_SF_UE8M0
    uint32_t in_block_m, in_block_k;
    uint32_t in_shift_m1, in_shift_k1;  // 1 + log2 of the block sizes when they are powers of two, else 0 (divide)
};

// Fills in_shift_*1 from in_block_*.
inline void set_input_block_shifts(TokenCastParams& p) {
    auto shift1 = [](uint32_t v) -> uint32_t {
        if (v == 0 || (v & (v - 1)) != 0) return 0;
        uint32_t s = 0;
        while ((1u << s) < v) ++s;
        return s + 1;
    };
    p.in_shift_m1 = shift1(p.in_block_m);
    p.in_shift_k1 = shift1(p.in_block_k);
}

constexpr int kSourcePlain = 0, kSourceSwiglu = 1, kSourceQuant = 2;

// The input scale that applies to (row, col) of an already quantized input
// (reference: tile_kernels/quant/common.py:219-235 load_sf + transform_sf).
__device__ __forceinline__ float load_input_scale(const TokenCastParams& p, uint32_t row, uint32_t col) {
    const int64_t m = p.in_shift_m1 ? row >> (p.in_shift_m1 - 1) : row / p.in_block_m;
    const int64_t k = p.in_shift_k1 ? col >> (p.in_shift_k1 - 1) : col / p.in_block_k;
    if (p.in_sf_flags & TKQ_SF_UE8M0) {
        const uint8_t e = static_cast<const uint8_t*>(p.in_sf)[(k >> 2) * p.in_sf_stride + 4 * m + (k & 3)];
        return __uint_as_float(static_cast<uint32_t>(e) << 23);
    }
    const float* f = static_cast<const float*>(p.in_sf);
    return (p.in_sf_flags & TKQ_SF_COL_MAJOR) ? f[k * p.in_sf_stride + m] : f[m * p.in_sf_stride + k];
}

constexpr int kGroupThreads = 256;

__device__ __forceinline__ void flush_clamp_counters(const ClampCounters& cnt, unsigned long long* dst) {
    uint32_t a = cnt.gate_hi, b = cnt.up_hi, c = cnt.up_lo;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        a += __shfl_xor_sync(kFullMask, a, o);
        b += __shfl_xor_sync(kFullMask, b, o);
        c += __shfl_xor_sync(kFullMask, c, o);
    }
    if ((threadIdx.x & 31) == 0) {
        if (a) atomicAdd(dst + 0, static_cast<unsigned long long>(a));
        if (b) atomicAdd(dst + 1, static_cast<unsigned long long>(b));
        if (c) atomicAdd(dst + 2, static_cast<unsigned long long>(c));
    }
}

// kClampMode: 0 = no clamp, 1 = clamp, 2 = clamp and count (SwiGLU sources only)
// kLean: the flags are known at compile time to be the common production set -- power-of-two scales by the
//        division-free path, packed ue8m0 in the column-major layout, data and scales both written -- so that their
//        tests leave the loop.  Only the re-quantising cast is instantiated so (101 -> 93 us on [32768, 7168]); the
//        plain bf16 casts run slower in this form (cfg5 0.954 ms against 0.894 ms, FP4 97 us against 95 us)
template <class Src, int kKind, int FMT, int LPG, int U, int kClampMode, bool kLean = false>
__global__ void __launch_bounds__(kGroupThreads) group_cast_kernel(const TokenCastParams p) {
    constexpr bool kSwiglu = kKind == kSourceSwiglu;
    constexpr bool kQuant = kKind == kSourceQuant;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    const bool round_sf = kLean || (p.flags & TKQ_ROUND_SF);
    const bool col_major = kLean || (p.flags & TKQ_SF_COL_MAJOR);
    const bool ue8m0 = kLean || (p.flags & TKQ_SF_UE8M0);
    const bool sf_only = !kLean && (p.flags & TKQ_SF_ONLY);
    const bool cast_only = !kLean && (p.flags & TKQ_CAST_ONLY);
    const bool wide = p.wide_loads;
    const bool fast_pow2 = kLean || p.fast_pow2;
    const uint32_t hidden = static_cast<uint32_t>(p.hidden);
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    ClampCounters cnt;

    uint32_t row = warp / p.items_per_row;
    uint32_t sub = warp - row * p.items_per_row;
    for (uint32_t item = warp; item < p.total_items; item += nwarps) {
        const uint32_t col0 = sub * (512u * U) + lane * 16u;
        const uint32_t this_row = row;
        sub += p.stride_items;
        row += p.stride_rows;
        if (sub >= p.items_per_row) {
            sub -= p.items_per_row;
            ++row;
        }
        if (kSwiglu && p.pos_to_expert != nullptr && p.pos_to_expert[this_row] < 0) continue;  // warp-uniform

        typename Src::Raw raw[U];
        const uint8_t* src = xb + Src::bytes(static_cast<int64_t>(this_row) * p.x_stride + col0);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (col0 + u * 512u < hidden) {
                if constexpr (kSwiglu) Src::issue(raw[u], src + Src::bytes(u * 512), wide, p.hidden);
                else Src::issue(raw[u], src + Src::bytes(u * 512), wide);
            } else {
                Src::zero(raw[u]);
            }
        }
        float w = 1.0f;
        if constexpr (kSwiglu) {
            if (p.pos_to_token_topk != nullptr) {
                const int32_t pos = p.pos_to_token_topk[this_row];
                w = pos >= 0 ? p.topk_weights[pos] : 0.0f;
            }
        }
        uint8_t* out_row = p.out + static_cast<int64_t>(this_row) * p.out_stride;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const uint32_t col = col0 + u * 512u;
            if (U > 1 && col - lane * 16u >= hidden) break;  // warp-uniform: the whole step lies beyond the row
            float v[16];
            if constexpr (kSwiglu) Src::template unpack<(kClampMode > 0), (kClampMode > 1), true>(raw[u], v, p.swiglu_clamp, w, cnt, p.bf16_gates);
            else if constexpr (kQuant) Src::unpack(raw[u], v, col < hidden ? load_input_scale(p, this_row, col) : 0.0f);
            else Src::unpack(raw[u], v);
            const bool in_row = col < hidden;
            const uint32_t g = col / (16u * LPG);
            float inv;
            if (cast_only) {
                inv = in_row ? __fdiv_rn(1.0f, load_sf_f32_row_major(p.sf, p.sf_stride, this_row, g)) : 0.0f;
            } else {
                float amax = absmax16(v);
#pragma unroll
                for (int o = LPG / 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, o));
                const Scale s = make_scale_for<FMT>(amax, p.clamp_min, round_sf, fast_pow2);
                inv = s.inv;
                if (lane % LPG == 0 && in_row) {
                    if (ue8m0) store_sf_ue8m0_byte(p.sf, p.sf_stride, this_row, g, p.num_groups, s.e8);
                    else store_sf_f32(p.sf, p.sf_stride, col_major, this_row, g, s.sf);
                }
            }
            if (!sf_only && in_row) {
                if constexpr (FMT == TKQ_FMT_E4M3) quantize_store_e4m3x16(v, inv, out_row + col);
                else quantize_store_e2m1x16(v, inv, out_row + col / 2);
            }
        }
    }
    if constexpr (kSwiglu && kClampMode > 1) flush_clamp_counters(cnt, p.clamped_count);
}

// ---------------------------------------------------------------------------
// The re-quantising cast to e4m3 with one scale per 128 values, for rows of whole 1024-value steps on 32-byte
// boundaries and input blocks at least 32 wide.  A lane owns 32 consecutive values (one 256-bit load of FP8 or one
// 128-bit load of FP4, one 256-bit store: whole sectors), a group is four lanes.  The codes are widened to f16, which
// holds every e4m3 and e2m1 value; the group maximum is the largest f16 magnitude times the lane's input scale,
// rounded once (x -> fl(x * s) is monotone, so this is the maximum of the products the general kernel forms).
//   kPow2 (input scales ue8m0, output scales powers of two): an output value is the input value times
//     2^(e_in - e_out), exact in f16 (at most four significant bits, magnitude at most 448; what falls below f16's
//     2^-24 grid is far below half of e4m3's smallest step and rounds to zero either way), so the codes go
//     f16x2 -> one multiplication -> e4m3x2 and never become fp32.  2^(e_in - e_out) above f16's range (a group of
//     nothing but tiny codes) sends the lane's values through fp32.
//   otherwise: value * input scale * inverse output scale in fp32, rounded after each product as in the general kernel.
// Same bits as group_cast_kernel<QuantSource<QFMT>, ..., e4m3, 8, ...>.
// ---------------------------------------------------------------------------
template <int QFMT, bool kPow2>
__global__ void __launch_bounds__(kGroupThreads) requant32_kernel(const TokenCastParams p) {
    constexpr int kWords = QFMT == TKQ_FMT_E4M3 ? 8 : 4;  // 32 codes
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    uint32_t row = warp / p.items_per_row;
    uint32_t sub = warp - row * p.items_per_row;
    for (uint32_t item = warp; item < p.total_items; item += nwarps) {
        const uint32_t col = sub * 1024u + lane * 32u;
        const uint32_t this_row = row;
        sub += p.stride_items;
        row += p.stride_rows;
        if (sub >= p.items_per_row) {
            sub -= p.items_per_row;
            ++row;
        }
        const uint8_t* src = xb + (static_cast<int64_t>(this_row) * p.x_stride + col) * kWords / 8;
        uint32_t raw[kWords];
        if constexpr (QFMT == TKQ_FMT_E4M3) {
            const U32x8 r = ldg256(src);
#pragma unroll
            for (int i = 0; i < 8; ++i) raw[i] = r.v[i];
        } else {
            const U32x4 r = ldg128(src);
#pragma unroll
            for (int i = 0; i < 4; ++i) raw[i] = r.v[i];
        }
        const float s_in = load_input_scale(p, this_row, col);
        uint8_t* dst = p.out + static_cast<int64_t>(this_row) * p.out_stride + col;
        uint32_t h[16];  // the 32 values as f16 pairs
        if constexpr (QFMT == TKQ_FMT_E4M3) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                asm("{ .reg .b16 lo, hi;\n\t"
                    "mov.b32 {lo, hi}, %2;\n\t"
                    "cvt.rn.f16x2.e4m3x2 %0, lo;\n\t"
                    "cvt.rn.f16x2.e4m3x2 %1, hi; }"
                    : "=r"(h[2 * i]), "=r"(h[2 * i + 1])
                    : "r"(raw[i]));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                asm("{ .reg .b8 b0, b1, b2, b3;\n\t"
                    "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
                    "cvt.rn.f16x2.e2m1x2 %3, b3; }"
                    : "=r"(h[4 * i]), "=r"(h[4 * i + 1]), "=r"(h[4 * i + 2]), "=r"(h[4 * i + 3])
                    : "r"(raw[i]));
            }
        }
        // largest magnitude of the lane: non-negative f16 values order like their bit patterns
        uint32_t m2 = h[0] & 0x7FFF7FFFu;
#pragma unroll
        for (int i = 1; i < 16; ++i) m2 = max_u16x2(m2, h[i] & 0x7FFF7FFFu);
        const uint32_t m1 = max(m2 & 0xFFFFu, m2 >> 16);
        float amax = __fmul_rn(__half2float(__ushort_as_half(static_cast<unsigned short>(m1))), s_in);
        amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(kFullMask, amax, 2));
        const Scale s = kPow2 ? make_scale_pow2<TKQ_FMT_E4M3>(amax, p.clamp_min) : make_scale_for<TKQ_FMT_E4M3>(amax, p.clamp_min, round_sf, p.fast_pow2);
        if ((lane & 3u) == 0) {
            const uint32_t g = col >> 7;
            if (p.flags & TKQ_SF_UE8M0) store_sf_ue8m0_byte(p.sf, p.sf_stride, this_row, g, p.num_groups, s.e8);
            else store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, this_row, g, s.sf);
        }
        uint32_t w[8];
        bool through_f16 = kPow2;
        uint32_t rel = 0;
        if constexpr (kPow2) {
            const uint32_t e_in = __float_as_uint(s_in) >> 23;
            const int d = static_cast<int>(e_in) - static_cast<int>(s.e8);
            through_f16 = d <= 15 || m1 == 0u;
            // 2^d as f16 in both halves: normal from 2^-14, subnormal down to 2^-24, zero below (and for a zero input scale)
            rel = d >= -14 ? static_cast<uint32_t>(min(d, 15) + 15) << 10 : (d >= -24 ? 1u << (d + 24) : 0u);
            if (e_in == 0u) rel = 0u;
            rel |= rel << 16;
        }
        if (through_f16) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                asm("{ .reg .b16 c0, c1; .reg .b32 a, b;\n\t"
                    "mul.rn.f16x2 a, %1, %3;\n\t"
                    "mul.rn.f16x2 b, %2, %3;\n\t"
                    "cvt.rn.satfinite.e4m3x2.f16x2 c0, a;\n\t"
                    "cvt.rn.satfinite.e4m3x2.f16x2 c1, b;\n\t"
                    "mov.b32 %0, {c0, c1}; }"
                    : "=r"(w[i])
                    : "r"(h[2 * i]), "r"(h[2 * i + 1]), "r"(rel));
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float2 a = mul2(mul2(__half22float2(*reinterpret_cast<const __half2*>(&h[2 * i])), splat2(s_in)), splat2(s.inv));
                const float2 b = mul2(mul2(__half22float2(*reinterpret_cast<const __half2*>(&h[2 * i + 1])), splat2(s_in)), splat2(s.inv));
                w[i] = cvt_e4m3x4(a.x, a.y, b.x, b.y);
            }
        }
        stg256(dst, w);
    }
}

// ---------------------------------------------------------------------------
// One scale per row.  A thread block walks rows; each thread keeps K chunks of 16
// values in registers (chunk c = tid + k * blockDim.x), the block reduces the
// maximum through shared memory with a single barrier per row.
// ---------------------------------------------------------------------------
constexpr int kRowMaxThreads = 512;

// 16 values of a chunk held as raw 16-byte pieces (2 for bf16, 4 for fp32) -> floats.
template <int DT>
__device__ __forceinline__ void unpack_chunk(const uint4* raw, float* v) {
    if constexpr (DT == TKQ_DT_BF16) {
        const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = bf16_lo(w[i]);
            v[2 * i + 1] = bf16_hi(w[i]);
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            v[4 * q] = __uint_as_float(raw[q].x);
            v[4 * q + 1] = __uint_as_float(raw[q].y);
            v[4 * q + 2] = __uint_as_float(raw[q].z);
            v[4 * q + 3] = __uint_as_float(raw[q].w);
        }
    }
}


__device__ __forceinline__ float block_max(float m, float (*red)[32], int parity) {
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
    if (lane == 0) red[parity][warp] = m;
    __syncthreads();
    m = red[parity][lane < nw ? lane : 0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
    return m;
}

// Stores the single scale of a row in whichever layout was asked for.
__device__ __forceinline__ void store_row_scale(const TokenCastParams& p, int64_t row, const Scale& s) {
    if (p.flags & TKQ_SF_UE8M0) store_sf_ue8m0_word(p.sf, p.sf_stride, row, 0, s.e8);  // upper three bytes zero
    else store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, row, 0, s.sf);
}

template <class Src, bool kSwiglu, int FMT, int K, int kClampMode>
__global__ void __launch_bounds__(kRowMaxThreads) row_cast_kernel(const TokenCastParams p) {
    __shared__ float red[2][32];
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool wide = p.wide_loads;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    ClampCounters cnt;
    int parity = 0;
    for (int64_t row = blockIdx.x; row < p.num_tokens; row += gridDim.x) {
        if (kSwiglu && p.pos_to_expert != nullptr && p.pos_to_expert[row] < 0) continue;  // block-uniform
        typename Src::Raw raw[K];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int64_t col = (static_cast<int64_t>(threadIdx.x) + k * blockDim.x) * 16;
            if (col < p.hidden) {
                const uint8_t* src = xb + Src::bytes(row * p.x_stride + col);
                if constexpr (kSwiglu) Src::issue(raw[k], src, wide, p.hidden);
                else Src::issue(raw[k], src, wide);
            } else {
                Src::zero(raw[k]);
            }
        }
        float v[K][16];
        float amax = 0.0f;
        float w = 1.0f;
        if constexpr (kSwiglu) {
            if (p.pos_to_token_topk != nullptr) {
                const int32_t pos = p.pos_to_token_topk[row];
                w = pos >= 0 ? p.topk_weights[pos] : 0.0f;
            }
        }
#pragma unroll
        for (int k = 0; k < K; ++k) {
            if constexpr (kSwiglu)
                Src::template unpack<(kClampMode > 0), (kClampMode > 1), true>(raw[k], v[k], p.swiglu_clamp, w, cnt, p.bf16_gates);
            else
                Src::unpack(raw[k], v[k]);
            amax = fmaxf(amax, absmax16(v[k]));
        }
        amax = block_max(amax, red, parity);
        parity ^= 1;
        const Scale s = make_scale_for<FMT>(amax, p.clamp_min, round_sf, p.fast_pow2);
        if (threadIdx.x == 0) store_row_scale(p, row, s);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int64_t col = (static_cast<int64_t>(threadIdx.x) + k * blockDim.x) * 16;
            if (col < p.hidden) {
                if constexpr (FMT == TKQ_FMT_E4M3) quantize_store_e4m3x16(v[k], s.inv, p.out + row * p.out_stride + col);
                else quantize_store_e2m1x16(v[k], s.inv, p.out + row * p.out_stride + col / 2);
            }
        }
    }
    if constexpr (kSwiglu && kClampMode > 1) flush_clamp_counters(cnt, p.clamped_count);
}

// ---------------------------------------------------------------------------
// E5M6: one scale per row (maximum 65024), 12-bit codes, 8 codes in 3 words.
// A thread owns K chunks of 32 values = 4 octets = 12 output words = three 128-bit
// stores.  Rows whose length is not a multiple of 32 finish with per-octet stores.
// ---------------------------------------------------------------------------
template <int DT>
struct OctetLoader;
template <>
struct OctetLoader<TKQ_DT_BF16> {
    static constexpr int kElemBytes = 2;
    struct Raw {
        U32x4 a;
    };
    __device__ __forceinline__ static void zero(Raw& r) { r.a.v[0] = r.a.v[1] = r.a.v[2] = r.a.v[3] = 0; }
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool) { r.a = ldg128(p); }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = bf16_lo(r.a.v[i]);
            v[2 * i + 1] = bf16_hi(r.a.v[i]);
        }
    }
};
template <>
struct OctetLoader<TKQ_DT_FP32> {
    static constexpr int kElemBytes = 4;
    struct Raw {
        U32x8 a;
    };
    __device__ __forceinline__ static void zero(Raw& r) {
#pragma unroll
        for (int i = 0; i < 8; ++i) r.a.v[i] = 0;
    }
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
        for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r.a.v[i]);
    }
};

template <int DT, int K>
__global__ void __launch_bounds__(kRowMaxThreads) row_cast_e5m6_kernel(const TokenCastParams p) {
    using L = OctetLoader<DT>;
    __shared__ float red[2][32];
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    const bool wide = p.wide_loads;
    const bool wide_stores = (p.hidden % 32) == 0;  // then every chunk starts on a 16-byte boundary of the output row
    int parity = 0;
    for (int64_t row = blockIdx.x; row < p.num_tokens; row += gridDim.x) {
        typename L::Raw raw[K][4];
#pragma unroll
        for (int k = 0; k < K; ++k) {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                const int64_t col = (static_cast<int64_t>(threadIdx.x) + k * blockDim.x) * 32 + o * 8;
                if (col < p.hidden) L::issue(raw[k][o], xb + (row * p.x_stride + col) * L::kElemBytes, wide);
                else L::zero(raw[k][o]);
            }
        }
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                float v[8];
                L::unpack(raw[k][o], v);
#pragma unroll
                for (int i = 0; i < 8; i += 2) amax = max3_abs(amax, v[i], v[i + 1]);
            }
        }
        amax = block_max(amax, red, parity);
        parity ^= 1;
        const Scale s = make_scale_for<TKQ_FMT_E5M6>(amax, p.clamp_min, round_sf, p.fast_pow2);
        if (threadIdx.x == 0) store_row_scale(p, row, s);
        uint32_t* out_row = reinterpret_cast<uint32_t*>(p.out + row * p.out_stride);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const int64_t chunk = static_cast<int64_t>(threadIdx.x) + k * blockDim.x;
            uint32_t w[12];
#pragma unroll
            for (int o = 0; o < 4; ++o) {
                float v[8];
                uint32_t c[8];
                L::unpack(raw[k][o], v);
#pragma unroll
                for (int i = 0; i < 8; ++i) c[i] = cvt_e5m6(__fmul_rn(v[i], s.inv));
                pack_e5m6x8(c, w + 3 * o);
            }
            const int64_t col = chunk * 32;
            if (wide_stores) {
                if (col < p.hidden) {
                    uint32_t* dst = out_row + chunk * 12;
                    stg128(dst, w[0], w[1], w[2], w[3]);
                    stg128(dst + 4, w[4], w[5], w[6], w[7]);
                    stg128(dst + 8, w[8], w[9], w[10], w[11]);
                }
            } else {
#pragma unroll
                for (int o = 0; o < 4; ++o) {
                    if (col + o * 8 < p.hidden) {
                        uint32_t* dst = out_row + chunk * 12 + o * 3;
                        stg32(dst, w[3 * o]);
                        stg32(dst + 1, w[3 * o + 1]);
                        stg32(dst + 2, w[3 * o + 2]);
                    }
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------
// E5M6 with rows staged by the bulk-copy engine (used when hidden % 32 == 0 and a few rows fit in shared
// memory; row_cast_e5m6_kernel above is the fallback).
//
// A block walks rows b, b + grid, ...  Thread 0 keeps `stages - 1` rows ahead in flight: one
// cp.async.bulk per row into a ring of shared-memory stages, each completing on its own mbarrier.  The
// block reads a row from its stage, reduces the maximum (barrier 1, after which nobody reads the stage any
// more), converts, and writes the packed 12-bit codes back into the *same* stage (the output row is 3/4 of
// the input row).  After barrier 2 thread 0 sends the stage to global memory with one bulk store and
// refills the stage of the previous row, whose store has finished reading by then.  Loads and stores are
// asynchronous and fully coalesced, and the registers hold only the row being converted.
// ---------------------------------------------------------------------------
static __device__ unsigned int g_row_wait_failed = 0;

template <int DT, int K>
__global__ void __launch_bounds__(kRowMaxThreads) e5m6_row_pipeline_kernel(const TokenCastParams p, const uint32_t stages,
                                                                            const uint32_t stage_bytes) {
    constexpr int EB = DT == TKQ_DT_BF16 ? 2 : 4;
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full_bar[4];
    __shared__ float red[2][32];
    const uint32_t t = threadIdx.x;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const uint32_t in_bytes = static_cast<uint32_t>(p.hidden) * EB;
    const uint32_t out_bytes = static_cast<uint32_t>(p.out_stride);
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);

    if (t == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(full_bar + s, 1);
    }
    __syncthreads();
    const int64_t first = blockIdx.x, step = gridDim.x;
    const int64_t my_rows = first < p.num_tokens ? (p.num_tokens - first + step - 1) / step : 0;
    auto issue_row = [&](int64_t i) {  // thread 0 only
        const uint32_t s = static_cast<uint32_t>(i % stages);
        mbar_arrive_expect_tx(full_bar + s, in_bytes);
        bulk_load(ring + static_cast<size_t>(s) * stage_bytes, xb + (first + i * step) * p.x_stride * EB, in_bytes, full_bar + s);
    };
    if (t == 0) {
        for (int64_t i = 0; i + 1 < stages && i < my_rows; ++i) issue_row(i);
    }
    int parity_red = 0;
    for (int64_t i = 0; i < my_rows; ++i) {
        const uint32_t s = static_cast<uint32_t>(i % stages);
        const int64_t row = first + i * step;
        uint8_t* stage = ring + static_cast<size_t>(s) * stage_bytes;
        if (!mbar_wait(full_bar + s, static_cast<uint32_t>(i / stages) & 1u)) {
            atomicExch(&g_row_wait_failed, 1u);
            if (t == 0) {
                bulk_store_wait_all();  // rows already handed to the store engine still read this block's ring
                // rows requested ahead still target this block's ring: wait for them (bounded) before the block ends
                for (int64_t j = i + 1; j < my_rows && j < i + stages - 1; ++j)
                    mbar_wait(full_bar + static_cast<uint32_t>(j % stages), static_cast<uint32_t>(j / stages) & 1u);
            }
            return;
        }
        // the thread's K chunks of 16 values
        float v[K][16];
        float amax = 0.0f;
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const uint32_t chunk = t + k * blockDim.x;
            uint4 raw[EB];  // bf16: 2 x 16 bytes per chunk, fp32: 4 x 16 bytes
            if (chunk * 16 < p.hidden) {
                const uint4* src = reinterpret_cast<const uint4*>(stage + static_cast<size_t>(chunk) * 16 * EB);
#pragma unroll
                for (int q = 0; q < EB; ++q) raw[q] = src[q];
            } else {
#pragma unroll
                for (int q = 0; q < EB; ++q) raw[q] = make_uint4(0, 0, 0, 0);
            }
            unpack_chunk<DT>(raw, v[k]);
            amax = fmaxf(amax, absmax16(v[k]));
        }
        amax = block_max(amax, red, parity_red);  // barrier 1: every thread has its part of the row in registers
        parity_red ^= 1;
        const Scale sc = make_scale_for<TKQ_FMT_E5M6>(amax, p.clamp_min, round_sf, p.fast_pow2);
        if (t == 0) store_row_scale(p, row, sc);
#pragma unroll
        for (int k = 0; k < K; ++k) {
            const uint32_t chunk = t + k * blockDim.x;
            if (chunk * 16 >= p.hidden) continue;
            uint32_t c[16], w[6];
            float smallest = 1.0f;
#pragma unroll
            for (int j = 0; j < 16; j += 2) {  // packed pairs: one issued instruction scales two values
                const float2 scaled = mul2(make_float2(v[k][j], v[k][j + 1]), splat2(sc.inv));
                v[k][j] = scaled.x;
                v[k][j + 1] = scaled.y;
            }
#pragma unroll
            for (int j = 0; j < 16; j += 2) smallest = min3_abs(smallest, v[k][j], v[k][j + 1]);
            if (smallest >= 6.103515625e-05f) {  // every |v| >= 2^-14: the fp16-normal rules apply to the whole chunk
#pragma unroll
                for (int j = 0; j < 16; j += 2) cvt_e5m6_normal2(make_float2(v[k][j], v[k][j + 1]), c[j], c[j + 1]);
            } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) c[j] = cvt_e5m6(v[k][j]);
            }
            pack_e5m6x8(c, w);
            pack_e5m6x8(c + 8, w + 3);
            uint2* dst = reinterpret_cast<uint2*>(stage + static_cast<size_t>(chunk) * 24);
            dst[0] = make_uint2(w[0], w[1]);
            dst[1] = make_uint2(w[2], w[3]);
            dst[2] = make_uint2(w[4], w[5]);
        }
        fence_proxy_async_smem();  // the codes were written through the generic proxy, the store reads through the async proxy
        __syncthreads();           // barrier 2: the output row is complete in the stage
        if (t == 0) {
            bulk_store(p.out + row * p.out_stride, stage, out_bytes);
            const int64_t next = i + stages - 1;
            if (next < my_rows) {
                bulk_store_wait_read<1>();  // the store of the previous row (whose stage is refilled now) has read its data
                issue_row(next);
            }
        }
    }
    if (t == 0) bulk_store_wait_all();
}

// ---------------------------------------------------------------------------
// Host side: geometry of a group_cast_kernel launch.
// ---------------------------------------------------------------------------
// max_blocks_per_sm > 0 caps the resident blocks per SM below what the occupancy allows.
template <class Kernel>
int launch_group_kernel(Kernel kernel, TokenCastParams p, int unroll, int sm_limit, cudaStream_t stream, const char* what,
                        int max_blocks_per_sm = 0) {
    const int64_t steps = (p.hidden + 511) / 512;
    const int64_t items_per_row = (steps + unroll - 1) / unroll;
    const int64_t total = p.num_tokens * items_per_row;
    if (total >= (int64_t{1} << 31)) return set_error(TKQ_E_UNSUPPORTED, "more than 2^31 work items; split the token dimension");
    constexpr int kWarpsPerBlock = kGroupThreads / 32;
    int grid = grid_size(kernel, kGroupThreads, (total + kWarpsPerBlock - 1) / kWarpsPerBlock, 0, sm_limit);
    if (max_blocks_per_sm > 0) grid = static_cast<int>(std::min<int64_t>(grid, static_cast<int64_t>(device_sm_count()) * max_blocks_per_sm));
    const uint32_t nwarps = static_cast<uint32_t>(grid) * kWarpsPerBlock;
    p.items_per_row = static_cast<uint32_t>(items_per_row);
    p.total_items = static_cast<uint32_t>(total);
    p.stride_rows = nwarps / p.items_per_row;
    p.stride_items = nwarps % p.items_per_row;
    kernel<<<grid, kGroupThreads, 0, stream>>>(p);
    return check_launch(what);
}

// round_sf with a clamp that keeps clamp / MAX a normal number: the division-free scale path applies.
inline bool can_use_fast_pow2(unsigned flags, float clamp_min, float max_q) {
    return (flags & TKQ_ROUND_SF) && clamp_min >= max_q * 1.1754943508222875e-38f;
}

// The flag set the kLean instantiations of group_cast_kernel are compiled for.
inline bool lean_flags(const TokenCastParams& p) {
    return p.flags == (TKQ_ROUND_SF | TKQ_SF_COL_MAJOR | TKQ_SF_UE8M0) && p.fast_pow2;
}

}  // namespace tkq
