// C entry point of the fused SwiGLU + per-token e4m3 cast.
#include <algorithm>
#include <cstring>

#include "tkq_launch.cuh"
#include "tkq_swiglu_pipeline.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

// The staged kernel with approximate codes and exact scales (tkq_swiglu_pipeline.cuh): bf16 rows of at least 1024
// activations, scale groups of 128, a clamp of the maximum that keeps every decisive value a normal number.
static bool pipeline_applies(const TokenCastParams& p, int in_dtype, bool per_row_scale, unsigned flags) {
    return in_dtype == TKQ_DT_BF16 && !per_row_scale && p.hidden >= 1024 && p.clamp_min >= 1e-30f && !(flags & TKQ_EXACT_CODES);
}

template <int kClampMode, bool kRouted, bool kFull, bool kPairs>
static int launch_swiglu_pipeline(TokenCastParams p, int sm_limit, cudaStream_t stream) {
    auto kernel = swiglu_group_pipeline_kernel<kClampMode, kRouted, kFull, kPairs>;
    const int64_t nseg = (p.hidden + kSwSegment - 1) / kSwSegment;
    const int64_t total = p.num_tokens * nseg;
    if (total >= (int64_t{1} << 31)) return set_error(TKQ_E_UNSUPPORTED, "more than 2^31 work items; split the token dimension");
    // two stages of 8 KB: measured on B200, more stages cost resident blocks (shared memory) and were slower
    // (35.5 / 39.3 / 42.2 us with 2 / 3 / 4 stages on [16384, 2 x 2048])
    constexpr int kStages = 2;
    const int smem = kStages * kSwStageBytes;
    p.total_items = static_cast<uint32_t>(total);
    // Resident blocks per SM, measured on B200 (CUDA-graph replay, rows x [2 x 2048], us for 8 / 10 / 12 blocks of the
    // 79-register instantiation):
    //   power-of-two scales (exact pass almost never taken)   8192 rows 16.5 / 15.8 / 16.6;  16384 rows 28.5 / 29.9 / 32.6;
    //                                                          32768 rows 55.8 / 56.8 / 60.9   (odd counts are worse: 7: 32.4, 9: 31.2)
    //   fp32 scales (exact pass on every group wants warps)    8192 rows 18.7 / 17.8 / 17.5;  16384 rows 34.3 / 33.0 / 32.0;
    //                                                          32768 rows 64.2 / 61.9 / 60.1
    // and 30.5 us (16384 rows) for fp32 scales with 10 blocks of the instantiation that interleaves pieces in pairs.
    // So: fp32 scales take that instantiation with 10 blocks; power-of-two scales the other one with 8 blocks when every
    // block then still gets 10 or more items, else 10.
    const int occ = cached_occupancy(reinterpret_cast<const void*>(kernel), kSwThreads, smem);
    int sms = device_sm_count();
    if (sm_limit > 0) sms = std::min(sms, sm_limit);
    int best_k = 10;
    if (!kPairs) best_k = total >= int64_t{10} * 8 * sms ? 8 : 10;
    best_k = std::max(1, std::min(best_k, occ));
    const int grid = static_cast<int>(std::max<int64_t>(1, std::min<int64_t>(total, static_cast<int64_t>(sms) * best_k)));
    kernel<<<grid, kSwThreads, smem, stream>>>(p, static_cast<uint32_t>(nseg), kStages);
    return check_launch("swiglu_forward_and_per_token_cast (staged kernel)");
}

template <bool kRouted, bool kFull>
static int dispatch_swiglu_pipeline_clamp(const TokenCastParams& p, int sm_limit, cudaStream_t stream) {
    if (p.fast_pow2) {
        if (p.swiglu_clamp < 0.0f) return launch_swiglu_pipeline<0, kRouted, kFull, false>(p, sm_limit, stream);
        if (p.clamped_count == nullptr) return launch_swiglu_pipeline<1, kRouted, kFull, false>(p, sm_limit, stream);
        return launch_swiglu_pipeline<2, kRouted, kFull, false>(p, sm_limit, stream);
    }
    if (p.swiglu_clamp < 0.0f) return launch_swiglu_pipeline<0, kRouted, kFull, true>(p, sm_limit, stream);
    if (p.clamped_count == nullptr) return launch_swiglu_pipeline<1, kRouted, kFull, true>(p, sm_limit, stream);
    return launch_swiglu_pipeline<2, kRouted, kFull, true>(p, sm_limit, stream);
}

static int dispatch_swiglu_pipeline(const TokenCastParams& p, int sm_limit, cudaStream_t stream) {
    const bool routed = p.pos_to_expert != nullptr || p.pos_to_token_topk != nullptr;
    const bool full = p.hidden % kSwSegment == 0;
    if (routed) return full ? dispatch_swiglu_pipeline_clamp<true, true>(p, sm_limit, stream) : dispatch_swiglu_pipeline_clamp<true, false>(p, sm_limit, stream);
    return full ? dispatch_swiglu_pipeline_clamp<false, true>(p, sm_limit, stream) : dispatch_swiglu_pipeline_clamp<false, false>(p, sm_limit, stream);
}

int swiglu_wait_flag() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_swiglu_wait_failed, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_swiglu_wait_failed, &zero, sizeof(zero));
    return static_cast<int>(v);
}

template <int DT, int kClampMode>
static int launch_swiglu_group(const TokenCastParams& p, int sm_limit, cudaStream_t stream) {
    const char* what = "swiglu_forward_and_per_token_cast (group kernel)";
    // two input streams per step: 64 (bf16) or 128 (fp32) bytes per lane and step; one step per work item
    return launch_group_kernel(group_cast_kernel<SwigluSource<DT>, kSourceSwiglu, TKQ_FMT_E4M3, 8, 1, kClampMode>, p, 1, sm_limit, stream, what);
}

template <int DT, int kClampMode, int K>
static int launch_swiglu_row(const TokenCastParams& p, int threads, int sm_limit, cudaStream_t stream) {
    auto kernel = row_cast_kernel<SwigluSource<DT>, true, TKQ_FMT_E4M3, K, kClampMode>;
    const int grid = grid_size(kernel, threads, p.num_tokens, 0, sm_limit);
    kernel<<<grid, threads, 0, stream>>>(p);
    return check_launch("swiglu_forward_and_per_token_cast (row kernel)");
}

template <int DT, int kClampMode>
static int dispatch_swiglu(const TokenCastParams& p, bool per_row_scale, int sm_limit, cudaStream_t stream) {
    if (!per_row_scale) return launch_swiglu_group<DT, kClampMode>(p, sm_limit, stream);
    int k = 0, threads = 0;
    // K is capped at 2: the activations stay in registers as fp32 between the maximum and the conversion
    if (!row_shape(p.hidden / 16, kRowMaxThreads, &k, &threads) || k > 2)
        return set_error(TKQ_E_UNSUPPORTED, "swiglu cast: hidden too large for one scale per token (max 16384)");
    return k == 1 ? launch_swiglu_row<DT, kClampMode, 1>(p, threads, sm_limit, stream)
                  : launch_swiglu_row<DT, kClampMode, 2>(p, threads, sm_limit, stream);
}

template <int DT>
static int dispatch_clamp(const TokenCastParams& p, bool per_row_scale, int sm_limit, cudaStream_t stream) {
    if (p.swiglu_clamp < 0.0f) return dispatch_swiglu<DT, 0>(p, per_row_scale, sm_limit, stream);
    if (p.clamped_count == nullptr) return dispatch_swiglu<DT, 1>(p, per_row_scale, sm_limit, stream);
    return dispatch_swiglu<DT, 2>(p, per_row_scale, sm_limit, stream);
}

}  // namespace tkq

using namespace tkq;

extern "C" int tkq_swiglu_forward_and_per_token_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden,
                                                     int64_t num_per_channels, const int32_t* pos_to_token_topk,
                                                     const float* topk_weights, const int32_t* pos_to_expert,
                                                     float swiglu_clamp, long long* clamped_count, float sf_clamp_min,
                                                     int num_sms, unsigned flags, void* out, void* sf, int64_t sf_stride,
                                                     void* stream) {
    if (num_tokens < 0 || hidden <= 0 || (in_dtype != TKQ_DT_BF16 && in_dtype != TKQ_DT_FP32))
        return set_error(TKQ_E_BAD_ARG, "swiglu cast: bad size or dtype");
    if (num_tokens == 0) return 0;
    if (x == nullptr || out == nullptr || sf == nullptr) return set_error(TKQ_E_BAD_ARG, "swiglu cast: null pointer");
    if ((pos_to_token_topk == nullptr) != (topk_weights == nullptr))
        return set_error(TKQ_E_BAD_ARG, "swiglu cast: pos_to_token_topk and topk_weights go together");
    if (clamped_count != nullptr && swiglu_clamp < 0.0f)
        return set_error(TKQ_E_BAD_ARG, "swiglu cast: clamped_count needs a clamp value");
    if (flags & ~(TKQ_ROUND_SF | TKQ_SF_COL_MAJOR | TKQ_SF_UE8M0 | TKQ_SF_ONLY | TKQ_CAST_ONLY | TKQ_EXACT_CODES))
        return set_error(TKQ_E_BAD_ARG, "swiglu cast: unknown flag bit");
    if (flags & (TKQ_SF_ONLY | TKQ_CAST_ONLY)) return set_error(TKQ_E_UNSUPPORTED, "swiglu cast: sf-only / cast-only not defined");
    if ((flags & TKQ_SF_UE8M0) && !(flags & TKQ_SF_COL_MAJOR))
        return set_error(TKQ_E_UNSUPPORTED, "packed ue8m0 scales need the column-major layout");
    if (hidden % 128 != 0) return set_error(TKQ_E_UNSUPPORTED, "swiglu cast: hidden must be a multiple of 128");
    const bool per_row_scale = num_per_channels != 128;
    if (per_row_scale && num_per_channels != hidden)
        return set_error(TKQ_E_UNSUPPORTED, "swiglu cast: num_per_channels must be 128 or hidden");
    const int elem = in_dtype == TKQ_DT_BF16 ? 2 : 4;
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(sf) & 3u) || ((flags & TKQ_SF_UE8M0) && (sf_stride & 3)))
        return set_error(TKQ_E_ALIGNMENT, "swiglu cast: x and out must be 16-byte aligned, sf 4-byte aligned");

    TokenCastParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.x_stride = 2 * hidden;
    p.sf_stride = sf_stride;
    p.out_stride = hidden;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.flags = flags & ~TKQ_EXACT_CODES;
    p.clamp_min = sf_clamp_min < 0.0f ? 1e-4f : sf_clamp_min;
    p.wide_loads = (reinterpret_cast<uintptr_t>(x) % 32 == 0) && ((hidden * elem) % 32 == 0);
    p.pos_to_token_topk = pos_to_token_topk;
    p.topk_weights = topk_weights;
    p.pos_to_expert = pos_to_expert;
    p.swiglu_clamp = swiglu_clamp;
    {
        uint32_t clamp_bits;
        std::memcpy(&clamp_bits, &swiglu_clamp, 4);
        p.bf16_gates = in_dtype == TKQ_DT_BF16 && (swiglu_clamp < 0.0f || (clamp_bits & 0xFFFFu) == 0);
    }
    p.clamped_count = reinterpret_cast<unsigned long long*>(clamped_count);
    p.num_groups = per_row_scale ? 1u : static_cast<uint32_t>(hidden / 128);
    p.fast_pow2 = can_use_fast_pow2(flags, p.clamp_min, 448.0f);
    const int sm_limit = clamped_count != nullptr ? num_sms : 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (pipeline_applies(p, in_dtype, per_row_scale, flags)) return dispatch_swiglu_pipeline(p, sm_limit, s);
    return in_dtype == TKQ_DT_BF16 ? dispatch_clamp<TKQ_DT_BF16>(p, per_row_scale, sm_limit, s)
                                   : dispatch_clamp<TKQ_DT_FP32>(p, per_row_scale, sm_limit, s);
}
