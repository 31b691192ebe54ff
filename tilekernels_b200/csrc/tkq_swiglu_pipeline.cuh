// Fused SwiGLU + per-token e4m3 cast (scale groups of 128), bf16 input, rows staged by the bulk-copy engine.
//
// Work item: one row segment of up to 2048 activations (128 threads x 16).  Thread 0 keeps `stages` items in
// flight, each as two cp.async.bulk copies (the gate columns and the up columns of the segment) into a ring of
// shared-memory stages that complete on one mbarrier per stage; all threads then compute from shared memory and
// write codes and scales straight to global memory.  Bytes in flight therefore do not depend on registers or on
// the number of resident warps.
//
// Arithmetic.  The reference evaluates y = g / (1 + exp(-g)) * u in fp32 and derives the scale of a group from
// max |y| (tile_kernels/quant/swiglu_forward_and_per_token_cast_kernel.py:140-160).  A reproducible exp and a
// correctly rounded division on every element cost about 25 instructions per activation, twice what a kernel
// that has to keep up with HBM can issue.  Here
//   * every activation is evaluated once with ex2.approx / rcp.approx (relative error below 2^-18 for gates
//     >= -80): these values become the FP8 codes, so a code can differ from the exactly evaluated one only when
//     the scaled activation lies within that error of a rounding boundary;
//   * the group maximum, which fixes the scale, is evaluated EXACTLY: every lane whose approximate values come
//     within 2^-15 of the group's approximate maximum is "flagged" (normally one lane per group: the one that
//     holds the maximum), the 16 (gate, up) pairs of a flagged lane are evaluated again by the 8 lanes of the
//     group, two pairs each, with the exact routine, and the group maximum is taken over those exact values.
//     The margin is 8 times the error bound, so the exactly largest element is always among the re-evaluated
//     ones and the scale equals the scale of a fully exact evaluation bit for bit;
//   * a lane that holds a gate below -80 (where ex2 overflows and the error bound is lost) sends its warp's
//     whole step through the exact routine.
#pragma once

#include "tkq_async.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

constexpr int kSwThreads = 128;
constexpr int kSwSegment = kSwThreads * 16;        // activations per work item
constexpr int kSwHalfBytes = kSwSegment * 2;       // bytes of the gate (or up) part of a stage
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

__device__ __forceinline__ float group8_max(float m) {
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 1));
    m = fmaxf(m, __shfl_xor_sync(kFullMask, m, 2));
    return fmaxf(m, __shfl_xor_sync(kFullMask, m, 4));
}

// kClampMode: 0 = no clamp, 1 = clamp, 2 = clamp and count
template <int kClampMode>
__global__ void __launch_bounds__(kSwThreads, 8)
swiglu_group_pipeline_kernel(const TokenCastParams p, const uint32_t nseg, const uint32_t stages) {
    extern __shared__ __align__(128) uint8_t ring[];
    __shared__ uint64_t full_bar[kSwMaxStages];
    const uint32_t t = threadIdx.x, lane = t & 31;
    const uint32_t hidden = static_cast<uint32_t>(p.hidden);
    const uint32_t total = p.total_items;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool col_major = p.flags & TKQ_SF_COL_MAJOR;
    const bool ue8m0 = p.flags & TKQ_SF_UE8M0;
    const bool bf16_gates = p.bf16_gates;
    const float clamp = p.swiglu_clamp;
    // values below half the clamp of the maximum cannot decide a scale: no exact evaluation for them
    const float thr_floor = __fmul_rn(p.clamp_min, 0.5f);
    ClampCounters cnt;

    if (t == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(full_bar + s, 1);
    }
    __syncthreads();

    // producer (thread 0): the next item to look at and the number of loads issued so far
    uint32_t p_item = blockIdx.x, p_loads = 0, p_stage = 0;
    auto produce = [&](uint32_t limit) {
        while (p_loads < limit && p_item < total) {
            const uint32_t row = p_item / nseg, seg = p_item - row * nseg;
            if (p.pos_to_expert == nullptr || p.pos_to_expert[row] >= 0) {
                const uint32_t col0 = seg * kSwSegment;
                const uint32_t bytes = min(static_cast<uint32_t>(kSwSegment), hidden - col0) * 2u;
                uint8_t* dst = ring + static_cast<size_t>(p_stage) * kSwStageBytes;
                const uint8_t* src = xb + (static_cast<int64_t>(row) * p.x_stride + col0) * 2;
                mbar_arrive_expect_tx(full_bar + p_stage, 2 * bytes);
                bulk_load(dst, src, bytes, full_bar + p_stage);
                bulk_load(dst + kSwHalfBytes, src + static_cast<int64_t>(hidden) * 2, bytes, full_bar + p_stage);
                ++p_loads;
                p_stage = p_stage + 1 == stages ? 0 : p_stage + 1;
            }
            p_item += gridDim.x;
        }
    };
    if (t == 0) produce(stages);

    uint32_t loads = 0, stage = 0, phase = 0;
    for (uint32_t item = blockIdx.x; item < total; item += gridDim.x) {
        const uint32_t row = item / nseg, seg = item - row * nseg;
        if (p.pos_to_expert != nullptr && p.pos_to_expert[row] < 0) continue;  // block-uniform
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
        const uint32_t this_stage_next = stage + 1 == stages ? 0 : stage + 1;
        phase ^= this_stage_next == 0 ? 1u : 0u;
        stage = this_stage_next;

        const uint32_t col = seg * kSwSegment + t * 16;
        if (col - lane * 16 >= hidden) continue;  // warp-uniform: this warp's 512 columns lie beyond the row
        const bool active = col < hidden;          // whole groups of 8 lanes are active or not

        uint32_t G[8], U[8];
        if (active) {
            const uint4* gp = reinterpret_cast<const uint4*>(st + t * 32);
            const uint4* up = reinterpret_cast<const uint4*>(st + kSwHalfBytes + t * 32);
            const uint4 g0 = gp[0], g1 = gp[1], u0 = up[0], u1 = up[1];
            G[0] = g0.x, G[1] = g0.y, G[2] = g0.z, G[3] = g0.w, G[4] = g1.x, G[5] = g1.y, G[6] = g1.z, G[7] = g1.w;
            U[0] = u0.x, U[1] = u0.y, U[2] = u0.z, U[3] = u0.w, U[4] = u1.x, U[5] = u1.y, U[6] = u1.z, U[7] = u1.w;
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) G[i] = U[i] = 0;
        }
        float w = 1.0f;
        if (p.pos_to_token_topk != nullptr) {
            const int32_t pos = p.pos_to_token_topk[row];
            w = pos >= 0 ? p.topk_weights[pos] : 0.0f;
        }

        // --- approximate evaluation of the lane's 16 activations ---
        float y[16];
        float g_min = 0.0f;
        {
            float g[16], u[16];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                g[2 * i] = bf16_lo(G[i]);
                g[2 * i + 1] = bf16_hi(G[i]);
                u[2 * i] = bf16_lo(U[i]);
                u[2 * i + 1] = bf16_hi(U[i]);
            }
            if (kClampMode > 0) {
                float g_hi = 0.0f, u_hi = 0.0f;
#pragma unroll
                for (int i = 0; i < 16; i += 2) {
                    g_hi = max3(g_hi, g[i], g[i + 1]);
                    u_hi = max3_abs(u_hi, u[i], u[i + 1]);
                }
                if (g_hi > clamp || u_hi > clamp) {
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
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
            for (int i = 0; i < 16; i += 2) g_min = min3(g_min, g[i], g[i + 1]);
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 g2 = make_float2(g[i], g[i + 1]);
                const float2 e2 = mul2(g2, splat2(-1.4426950408889634f));
                const float2 d2 = add2(make_float2(ex2_approx(e2.x), ex2_approx(e2.y)), splat2(1.0f));
                const float2 r2 = make_float2(rcp_approx(d2.x), rcp_approx(d2.y));
                // g * (r * u): r * u can only lose bits to underflow where the product is far below any clamp
                const float2 v2 = mul2(g2, mul2(r2, make_float2(u[i], u[i + 1])));
                y[i] = v2.x;
                y[i + 1] = v2.y;
            }
        }
        if (w != 1.0f) {  // uniform over the row
#pragma unroll
            for (int i = 0; i < 16; i += 2) {
                const float2 v2 = mul2(make_float2(y[i], y[i + 1]), splat2(w));
                y[i] = v2.x;
                y[i + 1] = v2.y;
            }
        }

        float amax;
        if (__any_sync(kFullMask, g_min < -80.0f)) {
            // rare: the whole step through the exact routine (the stage still holds the inputs)
            const uint16_t* gs = reinterpret_cast<const uint16_t*>(st + t * 32);
            const uint16_t* us = reinterpret_cast<const uint16_t*>(st + kSwHalfBytes + t * 32);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
                const float gi = active ? __uint_as_float(static_cast<uint32_t>(gs[i]) << 16) : 0.0f;
                const float ui = active ? __uint_as_float(static_cast<uint32_t>(us[i]) << 16) : 0.0f;
                y[i] = swiglu_exact_element(gi, ui, kClampMode > 0 ? clamp : -1.0f, w);
            }
            amax = group8_max(absmax16(y));
        } else {
            // --- which lanes can hold the exact maximum of their group ---
            const float approx_max = group8_max(absmax16(y));
            const float thr = fmaxf(__fmaf_rn(approx_max, -3.0517578125e-05f, approx_max), thr_floor);
            bool near_max = false;
#pragma unroll
            for (int i = 0; i < 16; ++i) near_max = near_max || (fabsf(y[i]) >= thr);
            uint32_t todo = (__ballot_sync(kFullMask, near_max) >> (lane & 24u)) & 0xFFu;  // flagged lanes of my group
            // --- their 16 pairs again, exactly: two pairs per lane of the group ---
            float exact_max = 0.0f;
            while (true) {
                if (todo != 0) {
                    const uint32_t holder = (t & ~7u) + (__ffs(todo) - 1);
                    const uint32_t gw = *reinterpret_cast<const uint32_t*>(st + holder * 32 + (lane & 7u) * 4);
                    const uint32_t uw = *reinterpret_cast<const uint32_t*>(st + kSwHalfBytes + holder * 32 + (lane & 7u) * 4);
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
            amax = group8_max(exact_max);
        }

        const Scale sc = make_scale_for<TKQ_FMT_E4M3>(amax, p.clamp_min, round_sf, p.fast_pow2);
        if (active) {
            if ((lane & 7u) == 0) {
                const uint32_t grp = col >> 7;
                if (ue8m0) store_sf_ue8m0_byte(p.sf, p.sf_stride, row, grp, p.num_groups, sc.e8);
                else store_sf_f32(p.sf, p.sf_stride, col_major, row, grp, sc.sf);
            }
            quantize_store_e4m3x16(y, sc.inv, p.out + static_cast<int64_t>(row) * p.out_stride + col);
        }
    }
    if constexpr (kClampMode > 1) flush_clamp_counters(cnt, p.clamped_count);
}

}  // namespace tkq
