// Fused SwiGLU + per-token e4m3 cast (scale groups of 128), bf16 input, rows staged by the bulk-copy engine.
//
// Work item: one row segment of up to 2048 activations; a block is 64 threads and every thread owns 32 activations
// of it, all in one scale group (4 lanes per group), so the per-item bookkeeping, the group reduction, the exact
// evaluation and the scale are paid once per 32 activations.  Thread 0 keeps `stages` items in flight, each as two cp.async.bulk copies (the gate columns and the up columns
// of the segment) into a ring of shared-memory stages that complete on one mbarrier per stage; all threads then
// compute from shared memory and write codes and scales straight to global memory.  Bytes in flight therefore do
// not depend on registers or on the number of resident warps.
//
// Arithmetic.  The reference evaluates y = g / (1 + exp(-g)) * u in fp32 and derives the scale of a group from
// max |y| (tile_kernels/quant/swiglu_forward_and_per_token_cast_kernel.py:140-160).  A reproducible exp and a
// correctly rounded division on every element cost about 25 instructions per activation, twice what a kernel
// that has to keep up with HBM can issue.  Here
//   * every activation is evaluated once with ex2.approx / rcp.approx (relative error below 2^-18 for gates
//     >= -80): these values become the FP8 codes, so a code can differ from the exactly evaluated one only when
//     the scaled activation lies within that error of a rounding boundary;
//   * the group maximum, which fixes the scale, is evaluated EXACTLY: every piece (8 values of one lane) whose
//     approximate values come within 2^-15 of the group's approximate maximum is "flagged" (normally one per
//     group: the one that holds the maximum); the 8 (gate, up) pairs of a flagged piece are evaluated again by the
//     4 lanes of the group, two pairs each as one packed evaluation, with the exact routine, and the group
//     maximum is taken over those exact values.  The margin is 8 times the error bound, so the exactly largest
//     element is always among the re-evaluated ones and the scale equals the scale of a fully exact evaluation
//     bit for bit;
//   * with power-of-two scales the exact evaluation is skipped whenever both ends of the interval that must hold
//     the exact maximum give the same exponent (almost always);
//   * a lane that holds a gate below -80 (where ex2 overflows and the error bound is lost) sends its warp's
//     whole step through the exact routine.
#pragma once

#include "tkq_async.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

constexpr int kSwThreads = 64;
constexpr int kSwSegment = kSwThreads * 32;              // activations per work item: 32 per thread
constexpr int kSwHalfBytes = kSwSegment * 2;             // bytes of the gate (or up) part of a stage
constexpr int kSwStageBytes = 2 * kSwHalfBytes;
constexpr int kSwMaxStages = 4;

static __device__ unsigned int g_swiglu_wait_failed = 0;

__device__ __forceinline__ float ex2_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float min3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// The exact value for two (gate, up) pairs: the packed in-range form where it applies, the general form otherwise.
__device__ __forceinline__ float2 swiglu_exact2(float2 g, float2 u, bool bf16_gates) {
    const float lo = fminf(fabsf(g.x), fabsf(g.y)), hi = fmaxf(fabsf(g.x), fabsf(g.y));
    if (bf16_gates && lo >= 9.094947017729282e-13f && hi <= 44.0f) return swiglu_bf16_in_range2(g, u);
    return make_float2(swiglu(g.x, u.x), swiglu(g.y, u.y));
}

// One element through the general exact routine, out of line: only the rare all-exact step calls it.
__device__ __noinline__ float swiglu_exact_element(float g, float u, float clamp, float w) {
    if (clamp >= 0.0f) {
        g = g > clamp ? clamp : g;
        u = u > clamp ? clamp : u;
        u = u < -clamp ? -clamp : u;
    }
    const float v = swiglu(g, u);
    return w != 1.0f ? __fmul_rn(v, w) : v;
}

// Maximum over the 4 lanes of a scale group.  (redux.sync with a sub-warp member mask was measured: it is emulated
// and costs far more than shuffle + max steps.)
__device__ __forceinline__ float group4_max(float m) {
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
    return fmaxf(m, __shfl_xor_sync(kFullMask, m, 2));
}

// fp32 scale and inverse of the e4m3 cast without the two IEEE divisions, same bits:
//   a / 448   = fma(fma(-448, q, a), c, q) with c = RN(1 / 448), q = a * c
//   448 / a   = reciprocal approximation, one Newton step, quotient, exact residual, correction
// Both were compared on the GPU with __fdiv_rn for all 2^23 mantissas of a over binades from 2^-100 to 2^110; the
// caller guarantees 1e-30 <= a <= 2^100 (nothing under- or overflows there), other values take make_scale.
__device__ __forceinline__ Scale make_scale_e4m3_nodiv(float amax, float clamp_min) {
    Scale s;
    const float a = fmaxf(amax, clamp_min);
    const float c = 1.0f / 448.0f;
    const float q = __fmul_rn(a, c);
    s.sf = __fmaf_rn(__fmaf_rn(-448.0f, q, a), c, q);
    float y = rcp_approx(a);
    y = __fmaf_rn(y, __fmaf_rn(-a, y, 1.0f), y);
    const float r = __fmul_rn(448.0f, y);
    s.inv = __fmaf_rn(__fmaf_rn(-a, r, 448.0f), y, r);
    s.e8 = __float_as_uint(s.sf) >> 23;
    return s;
}

// 8 activations (one 16-byte piece of the gate columns and of the up columns), approximately:
// y = g * (r * u) with r = rcp(1 + ex2(-g * log2 e)), times the row weight.  Returns the largest magnitude and
// lowers g_min to the smallest gate.
template <int kClampMode>
__device__ __forceinline__ float swiglu_approx_octet(const uint4 gw, const uint4 uw, float clamp, float w, ClampCounters& cnt,
                                                     float* y, float& g_min) {
    const uint32_t G[4] = {gw.x, gw.y, gw.z, gw.w}, U[4] = {uw.x, uw.y, uw.z, uw.w};
    float g[8], u[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        g[2 * i] = bf16_lo(G[i]);
        g[2 * i + 1] = bf16_hi(G[i]);
        u[2 * i] = bf16_lo(U[i]);
        u[2 * i + 1] = bf16_hi(U[i]);
    }
    if (kClampMode > 0) {
        float g_hi = 0.0f, u_hi = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            g_hi = max3(g_hi, g[i], g[i + 1]);
            u_hi = max3_abs(u_hi, u[i], u[i + 1]);
        }
        if (g_hi > clamp || u_hi > clamp) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (kClampMode > 1) {
                    cnt.gate_hi += g[i] > clamp;
                    cnt.up_hi += u[i] > clamp;
                    cnt.up_lo += u[i] < -clamp;
                }
                g[i] = g[i] > clamp ? clamp : g[i];
                u[i] = u[i] > clamp ? clamp : u[i];
                u[i] = u[i] < -clamp ? -clamp : u[i];
            }
        }
    }
#pragma unroll
    for (int i = 0; i < 8; i += 2) g_min = min3(g_min, g[i], g[i + 1]);
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float2 g2 = make_float2(g[i], g[i + 1]);
        const float2 e2 = mul2(g2, splat2(-1.4426950408889634f));
        const float2 d2 = add2(make_float2(ex2_approx(e2.x), ex2_approx(e2.y)), splat2(1.0f));
        const float2 r2 = make_float2(rcp_approx(d2.x), rcp_approx(d2.y));
        // g * (r * u): r * u can only lose bits to underflow where the product is far below any clamp
        const float2 v2 = mul2(g2, mul2(r2, make_float2(u[i], u[i + 1])));
        y[i] = v2.x;
        y[i + 1] = v2.y;
    }
    if (w != 1.0f) {  // uniform over the row
#pragma unroll
        for (int i = 0; i < 8; i += 2) {
            const float2 v2 = mul2(make_float2(y[i], y[i + 1]), splat2(w));
            y[i] = v2.x;
            y[i + 1] = v2.y;
        }
    }
    float m = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i += 2) m = max3_abs(m, y[i], y[i + 1]);
    return m;
}

// 8 values, scaled -> 8 e4m3 bytes in two words
__device__ __forceinline__ void quantize_e4m3x8(const float* v, float inv, uint32_t& w0, uint32_t& w1) {
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const float2 t = mul2(make_float2(v[i], v[i + 1]), splat2(inv));
        s[i] = t.x;
        s[i + 1] = t.y;
    }
    w0 = cvt_e4m3x4(s[0], s[1], s[2], s[3]);
    w1 = cvt_e4m3x4(s[4], s[5], s[6], s[7]);
}

// kClampMode: 0 = no clamp, 1 = clamp, 2 = clamp and count
//
// Thread mapping.  A warp covers 1024 consecutive activations of the item; the 4 lanes 4g .. 4g + 3 share scale
// group g of those (128 activations = 16 pieces of 8).  Lane i of a group owns the pieces 2i, 2i + 1 and 8 + 2i,
// 8 + 2i + 1: two runs of 16 consecutive activations, so that its codes leave as two 16-byte stores.  Its k-th load
// reads piece 8 (k / 2) + 2i + ((k % 2) xor (g % 2)): even and odd groups take the two pieces of a run in opposite
// order, and one load instruction of the warp touches every shared-memory bank exactly once.  32 activations per
// lane and item share ONE group reduction, ONE exact evaluation (the flagged piece: 8 pairs = 4 lanes x 2), one
// scale.
// kRouted: the call passes an expert mask and / or row weights (the plain form compiles without their checks)
// kFull:   hidden is a multiple of 2048, so every item is a full segment and every lane always has data
// kPairs:  the instruction schedule may interleave the lane's four pieces two at a time (about 95 registers, ten resident
//          blocks per SM) instead of one at a time (79 registers, twelve blocks).  Measured on [16384, 2 x 2048]: fp32
//          scales, whose exact pass needs the slack, 30.5 us in pairs with 10 blocks against 32.0 us singly with 12;
//          power-of-two scales 28.5 us singly with 8 blocks against 30.6 us in pairs with 10
template <int kClampMode, bool kRouted, bool kFull, bool kPairs>
__global__ void __launch_bounds__(kSwThreads, kPairs ? 10 : 12)
swiglu_group_pipeline_kernel(const TokenCastParams p, const uint32_t nseg, const uint32_t stages) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full_bar[kSwMaxStages];
    const uint32_t t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const uint32_t grp = lane >> 2, sub = lane & 3, parity = grp & 1;
    const uint32_t hidden = static_cast<uint32_t>(p.hidden);
    const uint32_t total = p.total_items;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool col_major = p.flags & TKQ_SF_COL_MAJOR;
    const bool ue8m0 = p.flags & TKQ_SF_UE8M0;
    const bool bf16_gates = p.bf16_gates;
    const bool fast_pow2 = p.fast_pow2;
    const float clamp = p.swiglu_clamp;
    const float clamp_min = p.clamp_min;
    // values below half the clamp of the maximum cannot decide a scale: no exact evaluation for them
    const float thr_floor = __fmul_rn(clamp_min, 0.5f);
    // first activation of the lane's group inside the item, and the byte offset of its first piece in a stage half
    const uint32_t group_col = warp * 1024 + grp * 128;
    const uint32_t piece0 = group_col * 2 + sub * 32;
    // byte offsets (inside a stage half) of the pieces the lane's four loads read
    const uint32_t off_a = piece0 + parity * 16, off_b = piece0 + (parity ^ 1u) * 16;
    ClampCounters cnt;

    if (t == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(full_bar + s, 1);
    }
    __syncthreads();

    // producer (thread 0): the next item to look at and the number of loads issued so far
    uint32_t p_item = blockIdx.x, p_loads = 0, p_stage = 0;
    const uint64_t policy = l2_evict_first_policy();  // the input is read once
    auto produce = [&](uint32_t limit) {
        while (p_loads < limit && p_item < total) {
            const uint32_t row = nseg == 1 ? p_item : p_item / nseg, seg = p_item - row * nseg;
            if (!kRouted || p.pos_to_expert == nullptr || p.pos_to_expert[row] >= 0) {
                const uint32_t col0 = seg * kSwSegment;
                const uint32_t bytes = min(static_cast<uint32_t>(kSwSegment), hidden - col0) * 2u;
                uint8_t* dst = ring + static_cast<size_t>(p_stage) * kSwStageBytes;
                const uint8_t* src = xb + (static_cast<int64_t>(row) * p.x_stride + col0) * 2;
                mbar_arrive_expect_tx(full_bar + p_stage, 2 * bytes);
                bulk_load_hint(dst, src, bytes, full_bar + p_stage, policy);
                bulk_load_hint(dst + kSwHalfBytes, src + static_cast<int64_t>(hidden) * 2, bytes, full_bar + p_stage, policy);
                ++p_loads;
                p_stage = p_stage + 1 == stages ? 0 : p_stage + 1;
            }
            p_item += gridDim.x;
        }
    };
    if (t == 0) produce(stages);

    uint32_t loads = 0, stage = 0, phase = 0;
    for (uint32_t item = blockIdx.x; item < total; item += gridDim.x) {
        const uint32_t row = nseg == 1 ? item : item / nseg, seg = item - row * nseg;
        if (kRouted && p.pos_to_expert != nullptr && p.pos_to_expert[row] < 0) continue;  // block-uniform
        // every thread is done with the stage of the previous load (its reads ordered before the refill)
        fence_proxy_async_smem();
        __syncthreads();
        if (t == 0) produce(loads + stages);
        const uint8_t* st = ring + static_cast<size_t>(stage) * kSwStageBytes;
        if (!mbar_wait(full_bar + stage, phase)) {
            atomicExch(&g_swiglu_wait_failed, 1u);
            if (t == 0) {  // the loads issued ahead still target this block's shared memory: wait for them (bounded) too
                uint32_t s2 = stage, ph2 = phase;
                for (uint32_t n = loads + 1; n < p_loads; ++n) {
                    s2 = s2 + 1 == stages ? 0 : s2 + 1;
                    ph2 ^= s2 == 0 ? 1u : 0u;
                    mbar_wait(full_bar + s2, ph2);
                }
            }
            return;
        }
        ++loads;
        stage = stage + 1 == stages ? 0 : stage + 1;
        phase ^= stage == 0 ? 1u : 0u;

        const uint32_t seg_col = seg * kSwSegment;
        const uint32_t width = kFull ? kSwSegment : min(static_cast<uint32_t>(kSwSegment), hidden - seg_col);  // a multiple of 128
        if (!kFull && warp * 1024 >= width) continue;     // warp-uniform: this warp's columns lie beyond the row
        const bool active = kFull || group_col < width;  // whole groups (4 lanes) are active or not
        float w = 1.0f;
        if (kRouted && p.pos_to_token_topk != nullptr) {
            const int32_t pos = p.pos_to_token_topk[row];
            w = pos >= 0 ? p.topk_weights[pos] : 0.0f;
        }

        // --- approximate evaluation of the lane's four pieces ---
        float y[4][8], piece_max[4];
        float g_min = 0.0f;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t off = ((k & 1) ? off_b : off_a) + (k >> 1) * 128;
            uint4 gw = make_uint4(0, 0, 0, 0), uw = make_uint4(0, 0, 0, 0);
            if (active) {
                gw = *reinterpret_cast<const uint4*>(st + off);
                uw = *reinterpret_cast<const uint4*>(st + kSwHalfBytes + off);
            }
            piece_max[k] = swiglu_approx_octet<kClampMode>(gw, uw, clamp, w, cnt, y[k], g_min);
            // keep the pieces apart in the instruction schedule (one by one, or two by two with kPairs): left alone, the
            // compiler interleaves all four, runs out of registers and spills (49 us instead of 32 us on
            // [16384, 2 x 2048]; with 96 registers for ten resident blocks it still spilled and took 34.6 us)
            if (kFull && (!kPairs || (k & 1))) asm volatile("" ::: "memory");
        }

        float amax;
        if (__any_sync(kFullMask, g_min < -80.0f)) {
            // rare: the whole step through the exact routine (the stage still holds the inputs)
            float m = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t off = ((k & 1) ? off_b : off_a) + (k >> 1) * 128;
                const uint16_t* gs = reinterpret_cast<const uint16_t*>(st + off);
                const uint16_t* us = reinterpret_cast<const uint16_t*>(st + kSwHalfBytes + off);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float gi = active ? __uint_as_float(static_cast<uint32_t>(gs[i]) << 16) : 0.0f;
                    const float ui = active ? __uint_as_float(static_cast<uint32_t>(us[i]) << 16) : 0.0f;
                    y[k][i] = swiglu_exact_element(gi, ui, kClampMode > 0 ? clamp : -1.0f, w);
                    m = fmaxf(m, fabsf(y[k][i]));
                }
            }
            amax = group4_max(m);
        } else {
            const float approx_max = group4_max(fmaxf(max3(piece_max[0], piece_max[1], piece_max[2]), piece_max[3]));
            bool undecided = true;
            if (fast_pow2) {
                // a power-of-two scale only depends on the binade of the maximum and on whether its mantissa exceeds
                // 1.75: when both ends of the interval that must contain the exact maximum give the same exponent,
                // the scale is decided without any exact evaluation
                const float lo_end = fmaxf(__fmaf_rn(approx_max, -3.0517578125e-05f, approx_max), clamp_min);
                const float hi_end = fmaxf(__fmaf_rn(approx_max, 3.0517578125e-05f, approx_max), clamp_min);
                constexpr uint32_t kCarry = FmtTraits<TKQ_FMT_E4M3>::kMantCarry;
                undecided = ((__float_as_uint(lo_end) + kCarry) >> 23) != ((__float_as_uint(hi_end) + kCarry) >> 23);
            }
            if (!__any_sync(kFullMask, undecided)) {
                amax = approx_max;
            } else {
                // --- which pieces can hold the exact maximum of their group: bit 4k + i = the k-th piece of lane i ---
                const float thr = fmaxf(__fmaf_rn(approx_max, -3.0517578125e-05f, approx_max), thr_floor);
                uint32_t todo = 0;
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    todo |= ((__ballot_sync(kFullMask, piece_max[k] >= thr) >> (lane & 28u)) & 0xFu) << (4 * k);
                // --- their 8 pairs again, exactly: two pairs per lane of the group ---
                float exact_max = 0.0f;
                while (true) {
                    if (todo != 0) {
                        const uint32_t h = __ffs(todo) - 1;
                        // bit h = 4k + i: the k-th piece of lane i of the group
                        const uint32_t off = group_col * 2 + (h >> 3) * 128 + (h & 3u) * 32 + ((((h >> 2) & 1u) ^ parity) << 4) + sub * 4;
                        const uint32_t gw = *reinterpret_cast<const uint32_t*>(st + off);
                        const uint32_t uw = *reinterpret_cast<const uint32_t*>(st + kSwHalfBytes + off);
                        float2 g2 = make_float2(bf16_lo(gw), bf16_hi(gw));
                        float2 u2 = make_float2(bf16_lo(uw), bf16_hi(uw));
                        if (kClampMode > 0) {
                            g2.x = g2.x > clamp ? clamp : g2.x;
                            g2.y = g2.y > clamp ? clamp : g2.y;
                            u2.x = fminf(fmaxf(u2.x, -clamp), clamp);
                            u2.y = fminf(fmaxf(u2.y, -clamp), clamp);
                        }
                        float2 f2 = swiglu_exact2(g2, u2, bf16_gates);
                        if (w != 1.0f) f2 = mul2(f2, splat2(w));
                        exact_max = max3_abs(exact_max, f2.x, f2.y);
                        todo &= todo - 1;
                    }
                    if (!__any_sync(kFullMask, todo != 0)) break;
                }
                amax = group4_max(exact_max);
            }
        }

        Scale sc;
        if (fast_pow2) sc = make_scale_pow2<TKQ_FMT_E4M3>(amax, clamp_min);
        else if (!round_sf && amax <= 1.2676506e30f) sc = make_scale_e4m3_nodiv(amax, clamp_min);
        else sc = make_scale(amax, clamp_min, 448.0f, round_sf);
        if (active) {
            if (sub == 0) {
                const uint32_t group_index = (seg_col + group_col) >> 7;
                if (ue8m0) store_sf_ue8m0_byte(p.sf, p.sf_stride, row, group_index, p.num_groups, sc.e8);
                else store_sf_f32(p.sf, p.sf_stride, col_major, row, group_index, sc.sf);
            }
            uint8_t* out_run0 = p.out + static_cast<int64_t>(row) * p.out_stride + seg_col + group_col + sub * 16;
#pragma unroll
            for (int run = 0; run < 2; ++run) {
                uint32_t a0, a1, b0, b1;
                quantize_e4m3x8(y[2 * run], sc.inv, a0, a1);
                quantize_e4m3x8(y[2 * run + 1], sc.inv, b0, b1);
                // odd groups hold the two pieces of a run in swapped order
                stg128(out_run0 + run * 64, parity ? b0 : a0, parity ? b1 : a1, parity ? a0 : b0, parity ? a1 : b1);
            }
        }
    }
    if constexpr (kClampMode > 1) flush_clamp_counters(cnt, p.clamped_count);
}

}  // namespace tkq
