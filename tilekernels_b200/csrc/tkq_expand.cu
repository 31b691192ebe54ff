// Row expansion into the fused expert layout, with the rows' scale factors
// (reference: tile_kernels/moe/expand_to_fused_kernel.py:15-94; oracle form tile_kernels/torch/expand_to_fused.py:6-91).
//
// The step after the cast in the MoE dispatch path: token t is copied to every expanded position
// token_topk_to_pos[t, k] >= 0, its scales go along (row-major, or into the column-major / packed-ue8m0 layout the
// grouped GEMM reads), and padding positions (pos_to_expert < 0) are zero-filled.  Pure data movement: a row is read
// once and written up to num_topk times.
//
// Phase 1 deals (token, 1024-byte step) items to warps grid-stride: a lane loads 32 bytes once (256-bit access; two
// 128-bit ones when only 16-byte alignment holds) and stores them to every routed position; the warp that owns
// step 0 of a row also moves its scales.  Phase 2 scans pos_to_expert, one position per lane, and clears the
// padded rows.
#include "tkq_launch.cuh"

namespace tkq {

struct ExpandParams {
    const uint8_t* x;
    const uint32_t* x_sf;   // [num_tokens, sf_words] or null
    const int32_t* token_topk_to_pos;
    const int32_t* pos_to_expert;
    uint8_t* out;
    uint32_t* out_sf;
    int64_t out_sf_stride;  // words between expanded rows (row-major) or between scale columns (column-major)
    uint32_t num_tokens;
    uint32_t num_expanded;
    uint32_t num_topk;
    uint32_t row_bytes;
    uint32_t steps;         // ceil(row_bytes / 1024)
    uint32_t sf_words;
    bool col_major;
    bool wide;
};

constexpr int kExpandThreads = 256;
constexpr int kSfWordsPerLane = 8;  // scale words of a row held in registers: 256 per warp

__device__ __forceinline__ void store32(uint8_t* p, bool wide, const uint32_t* w) {
    if (wide) {
        stg256(p, w);
    } else {
        stg128(p, w[0], w[1], w[2], w[3]);
        stg128(p + 16, w[4], w[5], w[6], w[7]);
    }
}

__device__ __forceinline__ uint32_t* sf_slot(const ExpandParams& p, uint32_t pos, uint32_t i) {
    return p.col_major ? p.out_sf + i * p.out_sf_stride + pos : p.out_sf + pos * p.out_sf_stride + i;
}

__global__ void __launch_bounds__(kExpandThreads) expand_to_fused_kernel(const ExpandParams p) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;

    // Phase 1: source rows.  Item = (token, 1024-byte step); a row is a multiple of 16 bytes, so the last lane of
    // a row may own a 16-byte half only.
    const uint32_t copy_items = p.num_tokens * p.steps;
    for (uint32_t item = warp; item < copy_items; item += nwarps) {
        const uint32_t row = item / p.steps;
        const uint32_t step = item - row * p.steps;
        const uint32_t off = step * 1024u + lane * 32u;
        const bool first_half = off < p.row_bytes, second_half = off + 16u < p.row_bytes;
        const int32_t my_pos = lane < p.num_topk ? p.token_topk_to_pos[static_cast<int64_t>(row) * p.num_topk + lane] : -1;
        // the row's scale words travel with step 0: up to 8 per lane are loaded once, ahead of the stores
        const bool with_sf = step == 0 && p.x_sf != nullptr;
        uint32_t sfw[kSfWordsPerLane];
#pragma unroll
        for (int j = 0; j < kSfWordsPerLane; ++j) {
            const uint32_t i = lane + 32u * j;
            sfw[j] = with_sf && i < p.sf_words ? __ldg(p.x_sf + static_cast<int64_t>(row) * p.sf_words + i) : 0u;
        }
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        const uint8_t* src = p.x + static_cast<int64_t>(row) * p.row_bytes + off;
        if (second_half && p.wide) {
            const U32x8 v = ldg256(src);
#pragma unroll
            for (int i = 0; i < 8; ++i) w[i] = v.v[i];
        } else {
            if (first_half) {
                const U32x4 v = ldg128(src);
                w[0] = v.v[0], w[1] = v.v[1], w[2] = v.v[2], w[3] = v.v[3];
            }
            if (second_half) {
                const U32x4 v = ldg128(src + 16);
                w[4] = v.v[0], w[5] = v.v[1], w[6] = v.v[2], w[7] = v.v[3];
            }
        }
        for (uint32_t k0 = 0; k0 < p.num_topk; k0 += 32) {
            const uint32_t count = min(32u, p.num_topk - k0);
            int32_t pos_k = my_pos;  // the first 32 slots were loaded with the row; further ones on demand
            if (k0 > 0) pos_k = lane < count ? p.token_topk_to_pos[static_cast<int64_t>(row) * p.num_topk + k0 + lane] : -1;
            uint32_t routed = __ballot_sync(0xffffffffu, pos_k >= 0);
            while (routed) {
                const int k = __ffs(routed) - 1;
                routed &= routed - 1;
                const uint32_t pos = static_cast<uint32_t>(__shfl_sync(0xffffffffu, pos_k, k));
                uint8_t* dst = p.out + static_cast<int64_t>(pos) * p.row_bytes + off;
                if (second_half) store32(dst, p.wide, w);
                else if (first_half) stg128(dst, w[0], w[1], w[2], w[3]);
                if (with_sf) {
#pragma unroll
                    for (int j = 0; j < kSfWordsPerLane; ++j) {
                        const uint32_t i = lane + 32u * j;
                        if (i < p.sf_words) *sf_slot(p, pos, i) = sfw[j];
                    }
                    for (uint32_t i = lane + 32u * kSfWordsPerLane; i < p.sf_words; i += 32)  // rows of more than 256 scale words
                        *sf_slot(p, pos, i) = __ldg(p.x_sf + static_cast<int64_t>(row) * p.sf_words + i);
                }
            }
        }
    }

    // Phase 2: padding rows.  Every lane looks at one expanded position; the warp then clears the padded ones.
    const uint32_t zero[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    for (uint32_t base = warp * 32u; base < p.num_expanded; base += nwarps * 32u) {
        const uint32_t mine = base + lane;
        uint32_t padded = __ballot_sync(0xffffffffu, mine < p.num_expanded && p.pos_to_expert[mine] < 0);
        while (padded) {
            const uint32_t pos = base + __ffs(padded) - 1;
            padded &= padded - 1;
            uint8_t* dst = p.out + static_cast<int64_t>(pos) * p.row_bytes;
            for (uint32_t off = lane * 32u; off < p.row_bytes; off += 1024u) {
                if (off + 16u < p.row_bytes) store32(dst + off, p.wide, zero);
                else stg128(dst + off, 0, 0, 0, 0);
            }
            if (p.x_sf != nullptr)
                for (uint32_t i = lane; i < p.sf_words; i += 32) *sf_slot(p, pos, i) = 0;
        }
    }
}

}  // namespace tkq

using namespace tkq;

extern "C" int tkq_expand_to_fused(const void* x, int64_t num_tokens, int64_t row_bytes, const void* x_sf, int64_t sf_words,
                                   const int32_t* token_topk_to_pos, int64_t num_topk, const int32_t* pos_to_expert,
                                   int64_t num_expanded_tokens, unsigned flags, void* out, void* out_sf, int64_t out_sf_stride,
                                   void* stream) {
    if (num_tokens < 0 || num_expanded_tokens < 0 || num_topk < 0 || row_bytes <= 0 || sf_words < 0)
        return set_error(TKQ_E_BAD_ARG, "expand_to_fused: bad size");
    if (flags & ~static_cast<unsigned>(TKQ_SF_COL_MAJOR))
        return set_error(TKQ_E_UNSUPPORTED, "expand_to_fused: only TKQ_SF_COL_MAJOR applies");
    if (num_tokens == 0) return 0;  // the reference launches nothing either, padding rows included
    if (x == nullptr || token_topk_to_pos == nullptr || pos_to_expert == nullptr || (out == nullptr && num_expanded_tokens > 0))
        return set_error(TKQ_E_BAD_ARG, "expand_to_fused: null pointer");
    if ((x_sf == nullptr) != (sf_words == 0) || (x_sf != nullptr && out_sf == nullptr && num_expanded_tokens > 0))
        return set_error(TKQ_E_BAD_ARG, "expand_to_fused: x_sf, sf_words and out_sf go together");
    if (row_bytes % 16 != 0) return set_error(TKQ_E_UNSUPPORTED, "expand_to_fused: a row must be a multiple of 16 bytes");
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(x_sf) & 3u) || (reinterpret_cast<uintptr_t>(out_sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "expand_to_fused: x and out must be 16-byte aligned, scales 4-byte aligned");
    if (num_expanded_tokens >= (int64_t{1} << 31) || row_bytes >= (int64_t{1} << 31) || sf_words >= (int64_t{1} << 31) ||
        num_tokens * ((row_bytes + 1023) / 1024) >= (int64_t{1} << 31))
        return set_error(TKQ_E_UNSUPPORTED, "expand_to_fused: more than 2^31 rows, work items or bytes per row");
    ExpandParams p{};
    p.x = static_cast<const uint8_t*>(x);
    p.x_sf = static_cast<const uint32_t*>(x_sf);
    p.token_topk_to_pos = token_topk_to_pos;
    p.pos_to_expert = pos_to_expert;
    p.out = static_cast<uint8_t*>(out);
    p.out_sf = static_cast<uint32_t*>(out_sf);
    p.out_sf_stride = out_sf_stride;
    p.num_tokens = static_cast<uint32_t>(num_tokens);
    p.num_expanded = static_cast<uint32_t>(num_expanded_tokens);
    p.num_topk = static_cast<uint32_t>(num_topk);
    p.row_bytes = static_cast<uint32_t>(row_bytes);
    p.steps = static_cast<uint32_t>((row_bytes + 1023) / 1024);
    p.sf_words = static_cast<uint32_t>(sf_words);
    p.col_major = (flags & TKQ_SF_COL_MAJOR) != 0;
    p.wide = row_bytes % 32 == 0 && reinterpret_cast<uintptr_t>(x) % 32 == 0 && reinterpret_cast<uintptr_t>(out) % 32 == 0;
    const int64_t items = std::max<int64_t>(num_tokens * p.steps, (num_expanded_tokens + 31) / 32);
    constexpr int kWarps = kExpandThreads / 32;
    const int grid = grid_size(expand_to_fused_kernel, kExpandThreads, (items + kWarps - 1) / kWarps, 0);
    expand_to_fused_kernel<<<grid, kExpandThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    return check_launch("expand_to_fused");
}
