// Dequantisation: FP8 e4m3 / packed FP4 e2m1 / packed E5M6 data times its block scale -> bf16 or fp32.
// (reference: tile_kernels/quant/cast_back_kernel.py:19-143, tile_kernels/quant/cast_back_e5m6_kernel.py;
//  oracle form tile_kernels/torch/cast.py:40-59, tile_kernels/torch/cast_e5m6.py:103-132,221-258)
//
// Same decomposition as the casts: a lane owns 16 consecutive values of a row, a warp a 512-value step, work
// items (row, step) are dealt to warps grid-stride.  The product float(x) * scale is formed in fp32 and then
// rounded once to the output type, as the reference does.
#include <cuda_bf16.h>

#include "tkq_launch.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

// 16 E5M6 values = 2 octets = 6 little-endian words (tile_kernels/torch/cast_e5m6.py:103-132): a code is the
// top 12 bits of an fp16.
struct E5m6Source {
    struct Raw {
        uint32_t w[6];
    };
    __host__ __device__ static constexpr int64_t bytes(int64_t elems) { return elems / 2 * 3; }
    __device__ __forceinline__ static void zero(Raw& r) {
#pragma unroll
        for (int i = 0; i < 6; ++i) r.w[i] = 0;
    }
    __device__ __forceinline__ static void issue(Raw& r, const void* p, bool) {  // p is 8-byte aligned
        const uint8_t* b = static_cast<const uint8_t*>(p);
#pragma unroll
        for (int i = 0; i < 3; ++i)
            asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(r.w[2 * i]), "=r"(r.w[2 * i + 1]) : "l"(b + 8 * i));
    }
    __device__ __forceinline__ static float code_to_float(uint32_t f16_bits) {
        return __half2float(__ushort_as_half(static_cast<unsigned short>(f16_bits & 0xFFF0u)));
    }
    __device__ __forceinline__ static void unpack(const Raw& r, float* v, float scale) {
#pragma unroll
        for (int o = 0; o < 2; ++o) {
            const uint32_t w0 = r.w[3 * o], w1 = r.w[3 * o + 1], w2 = r.w[3 * o + 2];
            const uint32_t h[8] = {w0 >> 16, w0 >> 4, (w0 << 8) | (w1 >> 24), w1 >> 12, w1, (w1 << 12) | (w2 >> 20), w2 >> 8, w2 << 4};
#pragma unroll
            for (int i = 0; i < 8; ++i) v[8 * o + i] = __fmul_rn(code_to_float(h[i]), scale);
        }
    }
};

template <class Src, int OUT_DT>
__global__ void __launch_bounds__(kGroupThreads) cast_back_kernel(const TokenCastParams p) {
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t nwarps = (gridDim.x * blockDim.x) >> 5;
    const uint32_t hidden = static_cast<uint32_t>(p.hidden);
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    uint32_t row = warp / p.items_per_row;
    uint32_t sub = warp - row * p.items_per_row;
    for (uint32_t item = warp; item < p.total_items; item += nwarps) {
        const uint32_t col = sub * 512u + lane * 16u;
        const uint32_t this_row = row;
        sub += p.stride_items;
        row += p.stride_rows;
        if (sub >= p.items_per_row) {
            sub -= p.items_per_row;
            ++row;
        }
        if (col >= hidden) continue;
        typename Src::Raw raw;
        Src::issue(raw, xb + Src::bytes(static_cast<int64_t>(this_row) * p.x_stride + col), false);
        const float scale = load_input_scale(p, this_row, col);
        float v[16];
        Src::unpack(raw, v, scale);
        // a lane's output is 32 (bf16) or 64 (fp32) contiguous bytes at a 32-byte aligned address (out is 32-byte
        // aligned when wide_stores is set, hidden is a multiple of 16): one or two 256-bit stores
        if constexpr (OUT_DT == TKQ_DT_FP32) {
            float* dst = reinterpret_cast<float*>(p.out) + static_cast<int64_t>(this_row) * p.hidden + col;
            uint32_t w[16];
#pragma unroll
            for (int i = 0; i < 16; ++i) w[i] = __float_as_uint(v[i]);
            if (p.wide_loads) {
                stg256(dst, w);
                stg256(dst + 8, w + 8);
            } else {
#pragma unroll
                for (int q = 0; q < 4; ++q) stg128(dst + 4 * q, w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            }
        } else {
            uint32_t w[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                w[i] = *reinterpret_cast<const uint32_t*>(&b);
            }
            uint8_t* dst = p.out + (static_cast<int64_t>(this_row) * p.hidden + col) * 2;
            if (p.wide_loads) {
                stg256(dst, w);
            } else {
                stg128(dst, w[0], w[1], w[2], w[3]);
                stg128(dst + 16, w[4], w[5], w[6], w[7]);
            }
        }
    }
}

template <class Src>
static int launch_cast_back(const TokenCastParams& p, int out_dtype, cudaStream_t stream) {
    const char* what = "cast_back";
    // Resident blocks per SM (the occupancy allows 8), measured on B200 for e4m3 -> bf16, us with 4 / 5 / 6 / 8 blocks:
    // [32768, 7168] 124.5 / 115.3 / 116.3 / 123.6 (E5M6: 142.0 / 133.9 / 140.7 / 146.9); [8192, 7168] 34.2 / 31.6 / 30.8 /
    // 32.8; [4096, 7168] 18.2 / 17.1 / 16.4 / 16.4.  A write-heavy stream runs best with fewer warps in flight once
    // every warp has many items; fp32 output is flat (203-207 us).
    const int64_t items = p.num_tokens * ((p.hidden + 511) / 512);
    const int blocks_per_sm = items >= int64_t{48} * 5 * (kGroupThreads / 32) * device_sm_count() ? 5 : 6;
    if (out_dtype == TKQ_DT_BF16) return launch_group_kernel(cast_back_kernel<Src, TKQ_DT_BF16>, p, 1, 0, stream, what, blocks_per_sm);
    return launch_group_kernel(cast_back_kernel<Src, TKQ_DT_FP32>, p, 1, 0, stream, what, blocks_per_sm);
}

}  // namespace tkq

using namespace tkq;

extern "C" int tkq_cast_back(const void* x, int in_fmt, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride,
                             int x_block_m, int x_block_k, int64_t num_tokens, int64_t hidden, int out_dtype, void* out,
                             void* stream) {
    if (num_tokens < 0 || hidden <= 0 || x_block_m <= 0 || x_block_k <= 0 || (out_dtype != TKQ_DT_BF16 && out_dtype != TKQ_DT_FP32) ||
        (in_fmt != TKQ_FMT_E4M3 && in_fmt != TKQ_FMT_E2M1 && in_fmt != TKQ_FMT_E5M6))
        return set_error(TKQ_E_BAD_ARG, "cast_back: bad size, format or output type");
    if (num_tokens == 0) return 0;
    if (x == nullptr || x_sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "cast_back: null pointer");
    if ((x_sf_flags & TKQ_SF_UE8M0) && !(x_sf_flags & TKQ_SF_COL_MAJOR))
        return set_error(TKQ_E_UNSUPPORTED, "packed ue8m0 scales need the column-major layout");
    // a lane's 16 values share one scale and one aligned load: 16 bytes of FP8, 8 bytes of FP4, 24 bytes of E5M6
    if (hidden % 16 != 0 || x_block_k % 16 != 0)
        return set_error(TKQ_E_UNSUPPORTED, "cast_back: hidden and the scale block width must be multiples of 16");
    const uintptr_t xa = reinterpret_cast<uintptr_t>(x);
    const bool aligned = in_fmt == TKQ_FMT_E4M3 ? xa % 16 == 0 : xa % 8 == 0;
    if (!aligned || !aligned16(out) || (reinterpret_cast<uintptr_t>(x_sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "cast_back: x must be 16-byte (FP8) or 8-byte (FP4, E5M6) aligned, out 16-byte aligned");
    TokenCastParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.x_stride = hidden;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.in_sf = x_sf;
    p.in_sf_stride = x_sf_stride;
    p.in_sf_flags = x_sf_flags;
    p.in_block_m = static_cast<uint32_t>(x_block_m);
    p.in_block_k = static_cast<uint32_t>(x_block_k);
    set_input_block_shifts(p);
    p.wide_loads = reinterpret_cast<uintptr_t>(out) % 32 == 0;  // here: 256-bit *stores* are legal
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_fmt == TKQ_FMT_E4M3) return launch_cast_back<QuantSource<TKQ_FMT_E4M3>>(p, out_dtype, s);
    if (in_fmt == TKQ_FMT_E2M1) return launch_cast_back<QuantSource<TKQ_FMT_E2M1>>(p, out_dtype, s);
    return launch_cast_back<E5m6Source>(p, out_dtype, s);
}
