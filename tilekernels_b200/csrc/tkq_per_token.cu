// C entry points of the per-token casts (FP8 e4m3, FP4 e2m1, E5M6).
#include <algorithm>
#include <cstdlib>

#include "tkq_launch.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

template <int DT, int FMT, int LPG>
static int launch_group(const TokenCastParams& p, cudaStream_t stream) {
    const char* what = "per_token_cast (group kernel)";
    // bytes per lane and step: 32 (bf16) or 64 (fp32)
    // measured on B200: many resident warps with one step each beat fewer warps with several steps in flight;
    // FP4 (half the output bytes per step) prefers two
    constexpr int kSteps = (DT == TKQ_DT_BF16 && FMT == TKQ_FMT_E2M1) ? 2 : 1;
    return launch_group_kernel(group_cast_kernel<PlainSource<DT>, kSourcePlain, FMT, LPG, kSteps, 0>, p, kSteps, 0, stream, what);
}

template <int DT, int FMT>
static int dispatch_group(const TokenCastParams& p, int64_t g, cudaStream_t stream) {
    switch (g) {
        case 16: return launch_group<DT, FMT, 1>(p, stream);
        case 32: return launch_group<DT, FMT, 2>(p, stream);
        case 64: return launch_group<DT, FMT, 4>(p, stream);
        case 128: return launch_group<DT, FMT, 8>(p, stream);
    }
    return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: num_per_channels must be 16, 32, 64, 128 or hidden");
}

template <int DT, int FMT, int K>
static int launch_row(const TokenCastParams& p, int threads, cudaStream_t stream) {
    auto kernel = row_cast_kernel<PlainSource<DT>, false, FMT, K, 0>;
    const int grid = grid_size(kernel, threads, p.num_tokens, 0);
    kernel<<<grid, threads, 0, stream>>>(p);
    return check_launch("per_token_cast (row kernel)");
}

template <int DT, int FMT>
static int dispatch_row(const TokenCastParams& p, cudaStream_t stream) {
    int k = 0, threads = 0;
    // blocks of up to 256 threads with more chunks per thread where the row allows it (cfg1's rows: 224 threads x 2
    // chunks, 16.5 us against 19.8 us with 448 x 1); the widest rows need 512 threads
    if (!row_shape(p.hidden / 16, 256, &k, &threads) && !row_shape(p.hidden / 16, kRowMaxThreads, &k, &threads))
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: hidden too large for one scale per token (max 32768)");
    switch (k) {
        case 1: return launch_row<DT, FMT, 1>(p, threads, stream);
        case 2: return launch_row<DT, FMT, 2>(p, threads, stream);
        default: return launch_row<DT, FMT, 4>(p, threads, stream);
    }
}

template <int DT, int K>
static int launch_e5m6(const TokenCastParams& p, int threads, cudaStream_t stream) {
    auto kernel = row_cast_e5m6_kernel<DT, K>;
    const int grid = grid_size(kernel, threads, p.num_tokens, 0);
    kernel<<<grid, threads, 0, stream>>>(p);
    return check_launch("per_token_cast_e5m6");
}

// The bulk-copy row pipeline: rows of hidden % 32 == 0 values that fit a shared-memory ring.
template <int DT, int K>
static int launch_e5m6_pipeline(const TokenCastParams& p, int threads, uint32_t stages, uint32_t stage_bytes, cudaStream_t stream) {
    auto kernel = e5m6_row_pipeline_kernel<DT, K>;
    const int smem = static_cast<int>(stages * stage_bytes);
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 200 * 1024)) return rc;
    const int grid = grid_size(kernel, threads, p.num_tokens, smem);
    kernel<<<grid, threads, smem, stream>>>(p, stages, stage_bytes);
    return check_launch("per_token_cast_e5m6 (row pipeline)");
}

template <int DT>
static int dispatch_e5m6(const TokenCastParams& p, cudaStream_t stream) {
    int k = 0, threads = 0;
    constexpr int EB = DT == TKQ_DT_BF16 ? 2 : 4;
    const uint32_t stage_bytes = static_cast<uint32_t>((p.hidden * EB + 127) / 128 * 128);
    if (p.hidden % 32 == 0 && stage_bytes <= 96 * 1024) {
        // small blocks (up to 128 threads, up to four chunks per thread) so that many blocks and their rings share an
        // SM: 134 us against 146 us with 256-thread blocks on [32768, 7168]
        if (row_shape(p.hidden / 16, 128, &k, &threads) || row_shape(p.hidden / 16, 256, &k, &threads) ||
            row_shape(p.hidden / 16, 512, &k, &threads)) {
            const uint32_t stages = stage_bytes <= 16 * 1024 ? 3u : 2u;
            switch (k) {
                case 1: return launch_e5m6_pipeline<DT, 1>(p, threads, stages, stage_bytes, stream);
                case 2: return launch_e5m6_pipeline<DT, 2>(p, threads, stages, stage_bytes, stream);
                default: return launch_e5m6_pipeline<DT, 4>(p, threads, stages, stage_bytes, stream);
            }
        }
    }
    if (!row_shape((p.hidden + 31) / 32, kRowMaxThreads, &k, &threads))
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast_e5m6: hidden too large (max 65536)");
    switch (k) {
        case 1: return launch_e5m6<DT, 1>(p, threads, stream);
        case 2: return launch_e5m6<DT, 2>(p, threads, stream);
        default: return launch_e5m6<DT, 4>(p, threads, stream);
    }
}

int row_wait_flag() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_row_wait_failed, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_row_wait_failed, &zero, sizeof(zero));
    return static_cast<int>(v);
}

template <int QFMT, int FMT>
static int dispatch_quant_group(const TokenCastParams& p, int64_t g, cudaStream_t stream) {
    const char* what = "per_token_cast (quantized input)";
    switch (g) {
        case 16: return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 1, 1, 0>, p, 1, 0, stream, what);
        case 32: return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 2, 1, 0>, p, 1, 0, stream, what);
        case 64: return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 4, 1, 0>, p, 1, 0, stream, what);
        case 128:
            // To e4m3, rows of whole 1024-value steps on 32-byte boundaries, input blocks at least 32 wide: the kernel with
            // 32 values per lane, in f16 arithmetic when both sides' scales are powers of two.  B200, FP8 [32768, 7168]
            // from 128x128 ue8m0 blocks: 101 us general kernel, 93 us with the flags fixed at compile time, 88 us with
            // two steps per warp, 79 us with this one.
            if constexpr (FMT == TKQ_FMT_E4M3) {
                const int64_t in_row_bytes = QFMT == TKQ_FMT_E4M3 ? p.x_stride : p.x_stride / 2;
                const bool rows32 = reinterpret_cast<uintptr_t>(p.x) % 32 == 0 && in_row_bytes % 32 == 0 && reinterpret_cast<uintptr_t>(p.out) % 32 == 0 &&
                                    p.out_stride % 32 == 0;
                if (!(p.flags & (TKQ_SF_ONLY | TKQ_CAST_ONLY)) && p.in_block_k % 32 == 0 && p.hidden % 1024 == 0 && rows32) {
                    // launch_group_kernel counts 512-value steps: two of them per step of this kernel
                    if ((p.in_sf_flags & TKQ_SF_UE8M0) && p.fast_pow2) return launch_group_kernel(requant32_kernel<QFMT, true>, p, 2, 0, stream, what);
                    return launch_group_kernel(requant32_kernel<QFMT, false>, p, 2, 0, stream, what);
                }
            }
            if (lean_flags(p)) {
                if (p.hidden >= 1024) return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 8, 2, 0, true>, p, 2, 0, stream, what);
                return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 8, 1, 0, true>, p, 1, 0, stream, what);
            }
            return launch_group_kernel(group_cast_kernel<QuantSource<QFMT>, kSourceQuant, FMT, 8, 1, 0>, p, 1, 0, stream, what);
    }
    return set_error(TKQ_E_UNSUPPORTED, "per_token_cast (quantized input): num_per_channels must be 16, 32, 64 or 128");
}

static int check_sf_flags(unsigned flags, const void* sf, int64_t sf_stride, const char** why) {
    if ((flags & TKQ_SF_UE8M0) && !(flags & TKQ_SF_COL_MAJOR)) {
        *why = "packed ue8m0 scales need the column-major layout";
        return TKQ_E_UNSUPPORTED;
    }
    if ((flags & TKQ_CAST_ONLY) && (flags & (TKQ_SF_UE8M0 | TKQ_SF_COL_MAJOR | TKQ_SF_ONLY))) {
        *why = "precomputed scales must be row-major fp32";
        return TKQ_E_UNSUPPORTED;
    }
    if ((reinterpret_cast<uintptr_t>(sf) & 3u) || ((flags & TKQ_SF_UE8M0) && (sf_stride & 3))) {
        *why = "scale storage must be 4-byte aligned";
        return TKQ_E_ALIGNMENT;
    }
    return 0;
}

}  // namespace tkq

using namespace tkq;

extern "C" int tkq_per_token_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, int64_t x_row_stride,
                                  int fmt, int64_t num_per_channels, unsigned flags, void* out, void* sf,
                                  int64_t sf_stride, void* stream) {
    if (fmt == TKQ_FMT_E5M6) {
        if (num_per_channels != hidden)
            return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: e5m6 needs num_per_channels == hidden");
        return tkq_per_token_cast_e5m6(x, in_dtype, num_tokens, hidden, x_row_stride, flags, out, sf, sf_stride, stream);
    }
    if (num_tokens < 0 || hidden <= 0 || x_row_stride < hidden || num_per_channels <= 0 ||
        (in_dtype != TKQ_DT_BF16 && in_dtype != TKQ_DT_FP32) || (fmt != TKQ_FMT_E4M3 && fmt != TKQ_FMT_E2M1))
        return set_error(TKQ_E_BAD_ARG, "per_token_cast: bad size, dtype or format");
    if (num_tokens == 0) return 0;
    const bool sf_only = flags & TKQ_SF_ONLY;
    if (x == nullptr || sf == nullptr || (!sf_only && out == nullptr))
        return set_error(TKQ_E_BAD_ARG, "per_token_cast: null pointer");
    const char* why = "";
    if (int rc = check_sf_flags(flags, sf, sf_stride, &why)) return set_error(rc, why);
    const int elem = in_dtype == TKQ_DT_BF16 ? 2 : 4;
    if (hidden % 16 != 0) return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: hidden must be a multiple of 16");
    if (!aligned16(x) || (x_row_stride * elem) % 16 != 0 || (!sf_only && !aligned16(out)))
        return set_error(TKQ_E_ALIGNMENT, "per_token_cast: x and out must be 16-byte aligned, rows too");

    TokenCastParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.x_stride = x_row_stride;
    p.sf_stride = sf_stride;
    p.out_stride = fmt == TKQ_FMT_E4M3 ? hidden : hidden / 2;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.flags = flags;
    p.clamp_min = fmt == TKQ_FMT_E4M3 ? 1e-4f : 6.0f * 1.1754943508222875e-38f;  // 6 * 2^-126
    p.wide_loads = (reinterpret_cast<uintptr_t>(x) % 32 == 0) && ((x_row_stride * elem) % 32 == 0);
    p.fast_pow2 = can_use_fast_pow2(flags, p.clamp_min, fmt == TKQ_FMT_E4M3 ? 448.0f : 6.0f);
    cudaStream_t s = static_cast<cudaStream_t>(stream);

    const bool group_kernel = num_per_channels == 16 || num_per_channels == 32 || num_per_channels == 64 ||
                              num_per_channels == 128;
    if (group_kernel) {
        p.num_groups = static_cast<uint32_t>((hidden + num_per_channels - 1) / num_per_channels);
        if (in_dtype == TKQ_DT_BF16)
            return fmt == TKQ_FMT_E4M3 ? dispatch_group<TKQ_DT_BF16, TKQ_FMT_E4M3>(p, num_per_channels, s)
                                       : dispatch_group<TKQ_DT_BF16, TKQ_FMT_E2M1>(p, num_per_channels, s);
        return fmt == TKQ_FMT_E4M3 ? dispatch_group<TKQ_DT_FP32, TKQ_FMT_E4M3>(p, num_per_channels, s)
                                   : dispatch_group<TKQ_DT_FP32, TKQ_FMT_E2M1>(p, num_per_channels, s);
    }
    if (num_per_channels != hidden)
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: num_per_channels must be 16, 32, 64, 128 or hidden");
    if (flags & (TKQ_SF_ONLY | TKQ_CAST_ONLY))
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast: sf-only / cast-only need num_per_channels < hidden");
    p.num_groups = 1;
    if (in_dtype == TKQ_DT_BF16)
        return fmt == TKQ_FMT_E4M3 ? dispatch_row<TKQ_DT_BF16, TKQ_FMT_E4M3>(p, s)
                                   : dispatch_row<TKQ_DT_BF16, TKQ_FMT_E2M1>(p, s);
    return fmt == TKQ_FMT_E4M3 ? dispatch_row<TKQ_DT_FP32, TKQ_FMT_E4M3>(p, s) : dispatch_row<TKQ_DT_FP32, TKQ_FMT_E2M1>(p, s);
}

extern "C" int tkq_per_token_cast_e5m6(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden,
                                       int64_t x_row_stride, unsigned flags, void* out, void* sf, int64_t sf_stride,
                                       void* stream) {
    if (num_tokens < 0 || hidden <= 0 || x_row_stride < hidden || (in_dtype != TKQ_DT_BF16 && in_dtype != TKQ_DT_FP32))
        return set_error(TKQ_E_BAD_ARG, "per_token_cast_e5m6: bad size or dtype");
    if (num_tokens == 0) return 0;
    if (x == nullptr || sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "per_token_cast_e5m6: null pointer");
    if (flags & (TKQ_SF_ONLY | TKQ_CAST_ONLY))
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast_e5m6: sf-only / cast-only are not defined for e5m6");
    const char* why = "";
    if (int rc = check_sf_flags(flags, sf, sf_stride, &why)) return set_error(rc, why);
    if (hidden % 8 != 0) return set_error(TKQ_E_UNSUPPORTED, "per_token_cast_e5m6: hidden must be a multiple of 8");
    const int elem = in_dtype == TKQ_DT_BF16 ? 2 : 4;
    if (!aligned16(x) || (x_row_stride * elem) % 16 != 0 || !aligned16(out))
        return set_error(TKQ_E_ALIGNMENT, "per_token_cast_e5m6: x and out must be 16-byte aligned, rows too");

    TokenCastParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.x_stride = x_row_stride;
    p.sf_stride = sf_stride;
    p.out_stride = hidden / 8 * 12;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.num_groups = 1;
    p.flags = flags;
    p.clamp_min = 1e-4f;
    p.wide_loads = (reinterpret_cast<uintptr_t>(x) % 32 == 0) && ((x_row_stride * elem) % 32 == 0);
    p.fast_pow2 = can_use_fast_pow2(flags, p.clamp_min, 65024.0f);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return in_dtype == TKQ_DT_BF16 ? dispatch_e5m6<TKQ_DT_BF16>(p, s) : dispatch_e5m6<TKQ_DT_FP32>(p, s);
}

extern "C" int tkq_per_token_cast_quantized(const void* x, int in_fmt, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride,
                                            int x_block_m, int x_block_k, int64_t num_tokens, int64_t hidden,
                                            int64_t x_row_stride, int fmt, int64_t num_per_channels, unsigned flags, void* out,
                                            void* sf, int64_t sf_stride, void* stream) {
    if (num_tokens < 0 || hidden <= 0 || x_row_stride < hidden || (in_fmt != TKQ_FMT_E4M3 && in_fmt != TKQ_FMT_E2M1) ||
        (fmt != TKQ_FMT_E4M3 && fmt != TKQ_FMT_E2M1) || x_block_m <= 0 || x_block_k <= 0)
        return set_error(TKQ_E_BAD_ARG, "per_token_cast (quantized input): bad size or format");
    if (num_tokens == 0) return 0;
    if (x == nullptr || x_sf == nullptr || sf == nullptr || out == nullptr)
        return set_error(TKQ_E_BAD_ARG, "per_token_cast (quantized input): null pointer");
    if (flags & (TKQ_SF_ONLY | TKQ_CAST_ONLY))
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast (quantized input): sf-only / cast-only are not defined");
    if ((x_sf_flags & TKQ_SF_UE8M0) && !(x_sf_flags & TKQ_SF_COL_MAJOR))
        return set_error(TKQ_E_UNSUPPORTED, "packed ue8m0 input scales need the column-major layout");
    const char* why = "";
    if (int rc = check_sf_flags(flags, sf, sf_stride, &why)) return set_error(rc, why);
    // a lane's 16 values must share one input scale and one 16-byte (FP8) or 8-byte (FP4) load
    if (hidden % 16 != 0 || x_block_k % 16 != 0)
        return set_error(TKQ_E_UNSUPPORTED, "per_token_cast (quantized input): hidden and the input block width must be multiples of 16");
    const int64_t row_bytes = in_fmt == TKQ_FMT_E4M3 ? x_row_stride : x_row_stride / 2;
    const int align = in_fmt == TKQ_FMT_E4M3 ? 16 : 8;
    if (reinterpret_cast<uintptr_t>(x) % align != 0 || row_bytes % align != 0 || !aligned16(out) ||
        (reinterpret_cast<uintptr_t>(x_sf) & 3u) != 0)
        return set_error(TKQ_E_ALIGNMENT, "per_token_cast (quantized input): x rows must be 16-byte (FP8) or 8-byte (FP4) aligned");

    TokenCastParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.x_stride = x_row_stride;
    p.sf_stride = sf_stride;
    p.out_stride = fmt == TKQ_FMT_E4M3 ? hidden : hidden / 2;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.flags = flags;
    p.clamp_min = fmt == TKQ_FMT_E4M3 ? 1e-4f : 6.0f * 1.1754943508222875e-38f;
    p.fast_pow2 = can_use_fast_pow2(flags, p.clamp_min, fmt == TKQ_FMT_E4M3 ? 448.0f : 6.0f);
    p.num_groups = static_cast<uint32_t>((hidden + num_per_channels - 1) / num_per_channels);
    p.in_sf = x_sf;
    p.in_sf_stride = x_sf_stride;
    p.in_sf_flags = x_sf_flags;
    p.in_block_m = static_cast<uint32_t>(x_block_m);
    p.in_block_k = static_cast<uint32_t>(x_block_k);
    set_input_block_shifts(p);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_fmt == TKQ_FMT_E4M3)
        return fmt == TKQ_FMT_E4M3 ? dispatch_quant_group<TKQ_FMT_E4M3, TKQ_FMT_E4M3>(p, num_per_channels, s)
                                   : dispatch_quant_group<TKQ_FMT_E4M3, TKQ_FMT_E2M1>(p, num_per_channels, s);
    return fmt == TKQ_FMT_E4M3 ? dispatch_quant_group<TKQ_FMT_E2M1, TKQ_FMT_E4M3>(p, num_per_channels, s)
                               : dispatch_quant_group<TKQ_FMT_E2M1, TKQ_FMT_E2M1>(p, num_per_channels, s);
}
