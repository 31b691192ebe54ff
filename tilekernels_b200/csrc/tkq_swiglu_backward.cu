// SwiGLU backward fused with the per-token e4m3 cast of the input gradient
// (reference: tile_kernels/quant/swiglu_backward_and_per_token_cast_kernel.py:16-155; oracle form
//  tile_kernels/torch/swiglu.py:98-226).
//
// Per expanded token (row) with gate part g = fp8(x[:, :H]) * sf and linear part u = fp8(x[:, H:]) * sf, incoming
// gradient d (bf16) and routing weight w (0 for an unused position):
//     t   = 1 + exp(-g)          a = g / t * u        s = 1 / t        q = d * w * s
//     out = a * w                                       (bf16)
//     dg  = q * u * fma(g, 1 - s, 1)    du = q * g      (0 where the forward clamp was active)
//     x_grad = [dg, du]                                 (bf16, and e4m3 with one scale per G = 32 / 128 values)
//     weight_grad[token, k] = sum over the row of d * a (0 where the (token, k) pair has no position)
//
// One warp owns a row: it walks the row in 512-column steps (a lane owns 16 consecutive columns of the gate
// half and the same 16 of the linear half), keeps the row's dot product in registers and writes it once.
// Every product is rounded separately (fp32, no contraction) except the one fused multiply-add the reference
// asks for; exp is the reproducible routine shared with the CPU oracle.
#include <cuda_bf16.h>

#include "tkq_launch.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

struct SwigluBackwardParams {
    const uint8_t* x;          // [rows, 2 * hidden] e4m3
    const float* x_sf;         // [rows, 2 * hidden / G]
    const uint8_t* grad_out;   // [rows, hidden] bf16
    const float* weight;       // [tokens * topk]
    const int32_t* pos_to_token_topk;  // [rows]
    const int32_t* token_topk_to_pos;  // [tokens * topk]
    uint8_t* out;              // [rows, hidden] bf16
    uint8_t* x_grad_fp8;       // [rows, 2 * hidden] e4m3
    float* x_grad_sf;          // [rows, 2 * hidden / G]
    uint8_t* x_grad;           // [rows, 2 * hidden] bf16
    float* weight_grad;        // [tokens * topk]
    uint32_t rows;
    uint32_t hidden;
    uint32_t steps;            // ceil(hidden / 512)
    uint32_t entries;          // tokens * topk
    float swiglu_clamp;
    float clamp_min;
    bool round_sf;
    bool fast_pow2;
    bool wide;                 // grad_out, out and x_grad are 32-byte aligned: 256-bit accesses
};

constexpr int kBackwardThreads = 128;
// Resident blocks per SM the register allocation aims at.  With the next step's loads in flight the kernel wants
// registers more than warps: measured best at 128 registers (4 blocks of 4 warps) without the clamp and at 168
// (3 blocks) with it; tighter limits spill and were 10-40 % slower.
template <bool kClamp>
constexpr int kBackwardBlocksPerSm = kClamp ? 3 : 4;

__device__ __forceinline__ void load_bf16x16(const uint8_t* p, bool wide, uint32_t* w) {
    if (wide) {
        const U32x8 a = ldg256(p);
#pragma unroll
        for (int i = 0; i < 8; ++i) w[i] = a.v[i];
    } else {
        const U32x4 a = ldg128(p), b = ldg128(p + 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            w[i] = a.v[i];
            w[4 + i] = b.v[i];
        }
    }
}

__device__ __forceinline__ void store_words8(uint8_t* p, bool wide, const uint32_t* w) {
    if (wide) {
        stg256(p, w);
    } else {
        stg128(p, w[0], w[1], w[2], w[3]);
        stg128(p + 16, w[4], w[5], w[6], w[7]);
    }
}

__device__ __forceinline__ void store_bf16x16(uint8_t* p, bool wide, const float* v) {
    uint32_t w[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        w[i] = *reinterpret_cast<const uint32_t*>(&b);
    }
    if (wide) {
        stg256(p, w);
    } else {
        stg128(p, w[0], w[1], w[2], w[3]);
        stg128(p + 16, w[4], w[5], w[6], w[7]);
    }
}

template <int LPG>
__device__ __forceinline__ float group_max(float m) {
#pragma unroll
    for (int o = 1; o < LPG; o *= 2) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    return m;
}

// The arithmetic of one lane's 16 columns, in one of three forms that give the same bits:
//   kPathBf16InRange  every gate is a bf16 number (an FP8 code times a power-of-two scale) of magnitude in
//                     [2^-40, 44] below the clamp: exp needs no argument clamp and both quotients come from ONE
//                     refined reciprocal (the sequence swiglu_bf16_in_range documents; for the numerator 1 and the
//                     3-bit FP8 mantissas it was compared with IEEE division for all 2^23 denominator mantissas of
//                     all 64 binades of [1, 2^64): no difference);
//   kPathInRange      gates of any mantissa with |g| <= 44 (FP8 codes times arbitrary fp32 scales): the same exp and
//                     the same reciprocal for s = 1 / t (its numerator is 1 whatever the gate is), IEEE division
//                     for g / t;
//   kPathGeneral      everything else: clamped exp argument, two IEEE divisions.
constexpr int kPathGeneral = 0, kPathBf16InRange = 1, kPathInRange = 2;

// Pairs of columns go through the packed fp32 instructions (two IEEE results per issued instruction).
template <bool kClamp, int kPath>
__device__ __forceinline__ float2 backward_chunk(const float* g, const float* u, const uint32_t* raw_d, float w, float clamp,
                                                 float2 acc, float* dg, float* du, uint32_t* o) {
    const float2 one = splat2(1.0f), minus_one = splat2(-1.0f), w2 = splat2(w);
#pragma unroll
    for (int i = 0; i < 16; i += 2) {
        float2 g2 = make_float2(g[i], g[i + 1]), u2 = make_float2(u[i], u[i + 1]);
        bool clamped_g0 = false, clamped_g1 = false, clamped_u0 = false, clamped_u1 = false;
        if constexpr (kClamp) {
            clamped_g0 = g2.x > clamp, clamped_g1 = g2.y > clamp;
            clamped_u0 = u2.x > clamp || u2.x < -clamp, clamped_u1 = u2.y > clamp || u2.y < -clamp;
            g2.x = clamped_g0 ? clamp : g2.x, g2.y = clamped_g1 ? clamp : g2.y;
            u2.x = u2.x > clamp ? clamp : u2.x, u2.y = u2.y > clamp ? clamp : u2.y;
            u2.x = u2.x < -clamp ? -clamp : u2.x, u2.y = u2.y < -clamp ? -clamp : u2.y;
        }
        const float2 d2 = make_float2(bf16_lo(raw_d[i >> 1]), bf16_hi(raw_d[i >> 1]));
        float2 ratio, s;  // g / t and 1 / t, both correctly rounded
        if constexpr (kPath == kPathBf16InRange) {
            const float2 t = add2(one, tkq_expf2_noclamp(mul2(g2, minus_one)));
            const float2 neg_t = mul2(t, minus_one);
            const float2 y = refined_rcp2(t, neg_t);
            s = fma2(fma2(neg_t, y, one), y, y);
            const float2 q0 = mul2(g2, y);
            ratio = fma2(fma2(neg_t, q0, g2), y, q0);
        } else if constexpr (kPath == kPathInRange) {
            const float2 t = add2(one, tkq_expf2_noclamp(mul2(g2, minus_one)));
            const float2 neg_t = mul2(t, minus_one);
            const float2 y = refined_rcp2(t, neg_t);
            s = fma2(fma2(neg_t, y, one), y, y);
            ratio = make_float2(__fdiv_rn(g2.x, t.x), __fdiv_rn(g2.y, t.y));
        } else {
            const float t0 = __fadd_rn(1.0f, tkq_expf(-g2.x)), t1 = __fadd_rn(1.0f, tkq_expf(-g2.y));
            ratio = make_float2(__fdiv_rn(g2.x, t0), __fdiv_rn(g2.y, t1));
            s = make_float2(__fdiv_rn(1.0f, t0), __fdiv_rn(1.0f, t1));
        }
        const float2 a = mul2(ratio, u2);
        acc = add2(acc, mul2(d2, a));
        const float2 q = mul2(mul2(d2, w2), s);
        const float2 out2 = mul2(a, w2);
        const __nv_bfloat162 b = __floats2bfloat162_rn(out2.x, out2.y);  // the weighted activation leaves as bf16 pairs
        o[i >> 1] = *reinterpret_cast<const uint32_t*>(&b);
        const float2 vg = mul2(mul2(q, u2), fma2(g2, fma2(s, minus_one, one), one));  // q * u * (1 + g * (1 - s))
        const float2 vu = mul2(q, g2);
        dg[i] = clamped_g0 ? 0.0f : vg.x;
        dg[i + 1] = clamped_g1 ? 0.0f : vg.y;
        du[i] = clamped_u0 ? 0.0f : vu.x;
        du[i + 1] = clamped_u1 ? 0.0f : vu.y;
    }
    return acc;
}

// G = 16 * LPG values per scale
template <int LPG, bool kClamp>
__global__ void __launch_bounds__(kBackwardThreads, kBackwardBlocksPerSm<kClamp>) swiglu_backward_kernel(const SwigluBackwardParams p) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t nthreads = gridDim.x * blockDim.x;
    const uint32_t hidden = p.hidden;
    const uint32_t groups_per_half = hidden / (16u * LPG);

    // (token, k) pairs that were routed nowhere get a zero gradient
    for (uint32_t e = tid; e < p.entries; e += nthreads)
        if (p.token_topk_to_pos[e] == -1) p.weight_grad[e] = 0.0f;

    // A warp walks its rows step by step; the loads of the NEXT step (or of the next row's first step) are issued
    // before the arithmetic of the current one, so their latency hides behind about 500 instructions.
    using Q8 = QuantSource<TKQ_FMT_E4M3>;
    struct StepInput {
        Q8::Raw g, u;
        uint32_t d[8];
        float sf_g, sf_u;
    };
    auto load_step = [&](StepInput& in, uint32_t row, uint32_t step) {
        const uint32_t col = step * 512u + lane * 16u;
        Q8::zero(in.g);
        Q8::zero(in.u);
#pragma unroll
        for (int i = 0; i < 8; ++i) in.d[i] = 0;
        in.sf_g = in.sf_u = 0.0f;
        if (row < p.rows && col < hidden) {  // whole scale groups are active or not: hidden is a multiple of G
            const uint8_t* x_row = p.x + static_cast<int64_t>(row) * 2 * hidden;
            const float* sf_row = p.x_sf + static_cast<int64_t>(row) * 2 * groups_per_half;
            const uint32_t group = col / (16u * LPG);
            Q8::issue(in.g, x_row + col, false);
            Q8::issue(in.u, x_row + hidden + col, false);
            load_bf16x16(p.grad_out + (static_cast<int64_t>(row) * hidden + col) * 2, p.wide, in.d);
            in.sf_g = __ldg(sf_row + group);
            in.sf_u = __ldg(sf_row + groups_per_half + group);
        }
    };
    auto load_index = [&](uint32_t row) { return row < p.rows ? p.pos_to_token_topk[row] : -1; };

    const uint32_t nwarps = nthreads >> 5;
    uint32_t row = tid >> 5, step = 0;
    StepInput cur, next;
    load_step(cur, row, 0);
    int32_t index = load_index(row), next_index = -1;
    float w = index >= 0 ? p.weight[index] : 0.0f;
    float2 acc2 = make_float2(0.0f, 0.0f);  // dot product of the lane's even and odd columns
    while (row < p.rows) {
        const bool last_step = step + 1 == p.steps;
        const uint32_t next_row = last_step ? row + nwarps : row, next_step = last_step ? 0 : step + 1;
        load_step(next, next_row, next_step);
        if (last_step) next_index = load_index(next_row);

        const uint32_t col = step * 512u + lane * 16u;
        const bool active = col < hidden;
        const uint32_t group = col / (16u * LPG);
        float g[16], u[16];
        Q8::unpack(cur.g, g, cur.sf_g);
        Q8::unpack(cur.u, u, cur.sf_u);
        float dg[16], du[16];
        uint32_t o[8];
        // pick the cheapest evaluation the chunk's gates allow (see backward_chunk)
        uint32_t low_bits = 0;
        float g_min = g[0], g_max = g[0];
#pragma unroll
        for (int i = 0; i < 16; i += 2) {
            low_bits |= __float_as_uint(g[i]) | __float_as_uint(g[i + 1]);
            g_min = min3_abs(g_min, g[i], g[i + 1]);
            g_max = max3_abs(g_max, g[i], g[i + 1]);
        }
        const bool in_range = g_max <= 44.0f;
        const bool bf16_in_range = in_range && (low_bits & 0xFFFFu) == 0 && g_min >= 0x1p-40f;
        bool reaches_clamp = false;  // chunks that cannot reach the clamp take the code without it
        if constexpr (kClamp) {
            float u_max = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i += 2) u_max = max3_abs(u_max, u[i], u[i + 1]);
            reaches_clamp = g_max > p.swiglu_clamp || u_max > p.swiglu_clamp;
        }
        if (reaches_clamp) {
            // clamped gates are at most the clamp value, which need not be a bf16 number: general mantissas
            if (in_range && p.swiglu_clamp <= 44.0f) acc2 = backward_chunk<true, kPathInRange>(g, u, cur.d, w, p.swiglu_clamp, acc2, dg, du, o);
            else acc2 = backward_chunk<true, kPathGeneral>(g, u, cur.d, w, p.swiglu_clamp, acc2, dg, du, o);
        } else if (bf16_in_range) {
            acc2 = backward_chunk<false, kPathBf16InRange>(g, u, cur.d, w, 0.0f, acc2, dg, du, o);
        } else if (in_range) {
            acc2 = backward_chunk<false, kPathInRange>(g, u, cur.d, w, 0.0f, acc2, dg, du, o);
        } else {
            acc2 = backward_chunk<false, kPathGeneral>(g, u, cur.d, w, 0.0f, acc2, dg, du, o);
        }
        const float amax_g = group_max<LPG>(absmax16(dg));  // the whole warp takes part in the shuffles
        const float amax_u = group_max<LPG>(absmax16(du));
        if (active) {
            const Scale scale_g = make_scale_for<TKQ_FMT_E4M3>(amax_g, p.clamp_min, p.round_sf, p.fast_pow2);
            const Scale scale_u = make_scale_for<TKQ_FMT_E4M3>(amax_u, p.clamp_min, p.round_sf, p.fast_pow2);
            if (lane % LPG == 0) {
                float* out_sf_row = p.x_grad_sf + static_cast<int64_t>(row) * 2 * groups_per_half;
                out_sf_row[group] = scale_g.sf;
                out_sf_row[groups_per_half + group] = scale_u.sf;
            }
            const int64_t half_off = static_cast<int64_t>(row) * hidden + col;      // in [rows, hidden]
            const int64_t full_off = static_cast<int64_t>(row) * 2 * hidden + col;  // in [rows, 2 * hidden]
            store_words8(p.out + half_off * 2, p.wide, o);
            store_bf16x16(p.x_grad + full_off * 2, p.wide, dg);
            store_bf16x16(p.x_grad + (full_off + hidden) * 2, p.wide, du);
            quantize_store_e4m3x16(dg, scale_g.inv, p.x_grad_fp8 + full_off);
            quantize_store_e4m3x16(du, scale_u.inv, p.x_grad_fp8 + full_off + hidden);
        }
        if (last_step) {
            float acc = __fadd_rn(acc2.x, acc2.y);
#pragma unroll
            for (int o2 = 16; o2 > 0; o2 >>= 1) acc = __fadd_rn(acc, __shfl_xor_sync(0xffffffffu, acc, o2));
            if (lane == 0 && index >= 0) p.weight_grad[index] = acc;
            acc2 = make_float2(0.0f, 0.0f);
            index = next_index;
            w = index >= 0 ? p.weight[index] : 0.0f;
        }
        cur = next;
        row = next_row;
        step = next_step;
    }
}

template <int LPG, bool kClamp>
static int launch_backward(const SwigluBackwardParams& p, cudaStream_t stream) {
    auto kernel = swiglu_backward_kernel<LPG, kClamp>;
    constexpr int kWarps = kBackwardThreads / 32;
    const int64_t blocks_of_work = std::max<int64_t>((static_cast<int64_t>(p.rows) + kWarps - 1) / kWarps,
                                                     (static_cast<int64_t>(p.entries) + kBackwardThreads - 1) / kBackwardThreads);
    const int grid = grid_size(kernel, kBackwardThreads, blocks_of_work, 0);
    kernel<<<grid, kBackwardThreads, 0, stream>>>(p);
    return check_launch("swiglu_backward_and_per_token_cast");
}

}  // namespace tkq

using namespace tkq;

extern "C" int tkq_swiglu_backward_and_per_token_cast(const void* x, const float* x_sf, const void* grad_out, const float* weight,
                                                      const int32_t* pos_to_token_topk, const int32_t* token_topk_to_pos,
                                                      int64_t num_expand_tokens, int64_t hidden, int64_t num_tokens,
                                                      int64_t num_topk, int64_t num_per_channels, float swiglu_clamp,
                                                      unsigned flags, void* out, void* x_grad_fp8, float* x_grad_sf,
                                                      void* x_grad, float* weight_grad, void* stream) {
    if (num_expand_tokens < 0 || hidden <= 0 || num_tokens < 0 || num_topk < 0)
        return set_error(TKQ_E_BAD_ARG, "swiglu_backward_and_per_token_cast: bad size");
    if (num_per_channels != 32 && num_per_channels != 128)
        return set_error(TKQ_E_UNSUPPORTED, "swiglu_backward_and_per_token_cast: num_per_channels must be 32 or 128");
    if (hidden % num_per_channels != 0)
        return set_error(TKQ_E_UNSUPPORTED, "swiglu_backward_and_per_token_cast: hidden must be a multiple of num_per_channels");
    if (flags & ~static_cast<unsigned>(TKQ_ROUND_SF))
        return set_error(TKQ_E_UNSUPPORTED, "swiglu_backward_and_per_token_cast: only TKQ_ROUND_SF applies (fp32 row-major scales)");
    if (num_expand_tokens == 0) return 0;  // the reference launches nothing either: weight_grad stays as it was
    if (!x || !x_sf || !grad_out || !weight || !pos_to_token_topk || !token_topk_to_pos || !out || !x_grad_fp8 || !x_grad_sf ||
        !x_grad || !weight_grad)
        return set_error(TKQ_E_BAD_ARG, "swiglu_backward_and_per_token_cast: null pointer");
    if (num_expand_tokens >= (int64_t{1} << 31) || num_tokens * num_topk >= (int64_t{1} << 31) || hidden >= (int64_t{1} << 30))
        return set_error(TKQ_E_UNSUPPORTED, "swiglu_backward_and_per_token_cast: more than 2^31 rows or routing entries");
    if (!aligned16(x) || !aligned16(grad_out) || !aligned16(out) || !aligned16(x_grad_fp8) || !aligned16(x_grad))
        return set_error(TKQ_E_ALIGNMENT, "swiglu_backward_and_per_token_cast: tensors must be 16-byte aligned");
    SwigluBackwardParams p{};
    p.x = static_cast<const uint8_t*>(x);
    p.x_sf = x_sf;
    p.grad_out = static_cast<const uint8_t*>(grad_out);
    p.weight = weight;
    p.pos_to_token_topk = pos_to_token_topk;
    p.token_topk_to_pos = token_topk_to_pos;
    p.out = static_cast<uint8_t*>(out);
    p.x_grad_fp8 = static_cast<uint8_t*>(x_grad_fp8);
    p.x_grad_sf = x_grad_sf;
    p.x_grad = static_cast<uint8_t*>(x_grad);
    p.weight_grad = weight_grad;
    p.rows = static_cast<uint32_t>(num_expand_tokens);
    p.hidden = static_cast<uint32_t>(hidden);
    p.steps = static_cast<uint32_t>((hidden + 511) / 512);
    p.entries = static_cast<uint32_t>(num_tokens * num_topk);
    p.swiglu_clamp = swiglu_clamp;
    p.clamp_min = 1e-4f;
    p.round_sf = (flags & TKQ_ROUND_SF) != 0;
    p.fast_pow2 = can_use_fast_pow2(flags, p.clamp_min, 448.0f);
    auto aligned32 = [](const void* q) { return reinterpret_cast<uintptr_t>(q) % 32 == 0; };
    p.wide = aligned32(grad_out) && aligned32(out) && aligned32(x_grad);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool clamp = swiglu_clamp >= 0.0f;
    if (num_per_channels == 128) return clamp ? launch_backward<8, true>(p, s) : launch_backward<8, false>(p, s);
    return clamp ? launch_backward<2, true>(p, s) : launch_backward<2, false>(p, s);
}
