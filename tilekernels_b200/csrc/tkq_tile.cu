// Per-block and per-channel casts: 128 x 128 tiles staged in shared memory by the
// bulk-copy engine (TMA, untiled form: one cp.async.bulk per tile row, all
// completing on a single mbarrier; no tensor map and no multicast).
//
// Thread mapping inside a tile (256 threads): thread t owns the 16-column chunk
// c16 = t % 8 of rows t / 8 + 32 * i, i = 0..3.  A warp therefore covers 4 full
// rows per i, reads shared memory in whole rows and writes 4 x 128 B of e4m3 per
// store instruction.
#include "tkq_launch.cuh"
#include "tkq_sources.cuh"

namespace tkq {

constexpr int kTile = 128;
constexpr int kTileThreads = 256;

// Set when a kernel gave up waiting for its tile; read back by tkq_device_error().
__device__ unsigned int g_tile_wait_failed = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

// Bounded wait: returns false if the phase did not complete within the poll budget.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
    const uint32_t addr = smem_u32(bar);
    for (int i = 0; i < (1 << 22); ++i) {
        uint32_t done;
        asm volatile(
            "{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}

// global -> shared bulk copy; both addresses 16-byte aligned, bytes a multiple of 16
__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

struct TileParams {
    const void* x;
    uint8_t* out;
    void* sf;
    int64_t num_tokens;
    int64_t hidden;
    int64_t sf_stride;
    uint32_t tiles_k;  // tiles along the channel dimension
    uint32_t flags;
    float clamp_min;
};

template <int DT>
struct TileElem {
    static constexpr int kBytes = DT == TKQ_DT_BF16 ? 2 : 4;
};

// Reads the thread's 16 values of tile row `r` from shared memory.
template <int DT>
__device__ __forceinline__ void read_chunk(const uint8_t* tile, int r, int c16, float* v) {
    const uint8_t* p = tile + (static_cast<size_t>(r) * kTile + c16 * 16) * TileElem<DT>::kBytes;
    if constexpr (DT == TKQ_DT_BF16) {
        const uint4 a = *reinterpret_cast<const uint4*>(p), b = *reinterpret_cast<const uint4*>(p + 16);
        const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            v[2 * i] = bf16_lo(w[i]);
            v[2 * i + 1] = bf16_hi(w[i]);
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const float4 a = *reinterpret_cast<const float4*>(p + 16 * q);
            v[4 * q] = a.x;
            v[4 * q + 1] = a.y;
            v[4 * q + 2] = a.z;
            v[4 * q + 3] = a.w;
        }
    }
}

// Stages the tile (rows0.., cols0..) of x into shared memory and waits for it.
// Returns false (after raising the device error flag) if the wait ran out.
template <int DT>
__device__ __forceinline__ bool stage_tile(const TileParams& p, uint8_t* tile, uint64_t* bar, int64_t row0, int64_t col0,
                                           int valid_rows, int valid_cols) {
    constexpr int EB = TileElem<DT>::kBytes;
    const int t = threadIdx.x;
    if (t == 0) mbar_init(bar, 1);
    __syncthreads();
    const uint32_t row_bytes = static_cast<uint32_t>(valid_cols) * EB;
    if (t == 0) mbar_arrive_expect_tx(bar, row_bytes * static_cast<uint32_t>(valid_rows));
    if (t < valid_rows) {
        const uint8_t* src = static_cast<const uint8_t*>(p.x) + ((row0 + t) * p.hidden + col0) * EB;
        bulk_load(tile + static_cast<size_t>(t) * kTile * EB, src, row_bytes, bar);
    }
    if (!mbar_wait(bar, 0)) {
        atomicExch(&g_tile_wait_failed, 1u);
        return false;
    }
    return true;
}

// ---------------------------------------------------------------------------
// Per-block cast: one scale per (BM x BK) block, BM, BK in {32, 128}.
// ---------------------------------------------------------------------------
template <int DT, int FMT, int BM, int BK>
__global__ void __launch_bounds__(kTileThreads) per_block_cast_kernel(const TileParams p) {
    constexpr float kMaxQ = FMT == TKQ_FMT_E4M3 ? 448.0f : 6.0f;
    constexpr int NRB = kTile / BM, NCB = kTile / BK;  // scale blocks per tile
    constexpr int kLanesPerCb = BK / 16;                // lanes of a row that share a column block (2 or 8)
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* tile = smem;
    __shared__ uint64_t bar;
    __shared__ int amax_bits[NRB * NCB];

    const int t = threadIdx.x, lane = t & 31;
    const int c16 = t & 7, r_base = t >> 3;
    const int64_t tile_m = blockIdx.x / p.tiles_k, tile_k = blockIdx.x % p.tiles_k;
    const int64_t row0 = tile_m * kTile, col0 = tile_k * kTile;
    const int valid_rows = static_cast<int>(p.num_tokens - row0 < kTile ? p.num_tokens - row0 : kTile);
    const int valid_cols = static_cast<int>(p.hidden - col0 < kTile ? p.hidden - col0 : kTile);
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool cast_only = p.flags & TKQ_CAST_ONLY;
    const bool sf_only = p.flags & TKQ_SF_ONLY;

    if (t < NRB * NCB) amax_bits[t] = 0;
    if (!stage_tile<DT>(p, tile, &bar, row0, col0, valid_rows, valid_cols)) return;

    const bool col_ok = c16 * 16 < valid_cols;
    const int cb = c16 * 16 / BK;
    float v[4][16];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r_base + 32 * i;
        if (col_ok && r < valid_rows) {
            read_chunk<DT>(tile, r, c16, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[i][j] = 0.0f;
        }
    }

    const int64_t sf_m0 = row0 / BM, sf_k0 = col0 / BK;
    const int64_t num_kb = (p.hidden + BK - 1) / BK;
    float inv[4];
    if (cast_only) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rb = (r_base + 32 * i) / BM;
            const bool ok = col_ok && (r_base + 32 * i) < valid_rows;
            inv[i] = ok ? __fdiv_rn(1.0f, load_sf_f32_row_major(p.sf, p.sf_stride, sf_m0 + rb, sf_k0 + cb)) : 0.0f;
        }
    } else {
        // maxima per row block, combined over the lanes and warps that share the block
        float m[NRB];
#pragma unroll
        for (int rb = 0; rb < NRB; ++rb) m[rb] = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rb = NRB == 1 ? 0 : i;  // BM = 32: rows r_base + 32 i lie in row block i
            m[rb] = fmaxf(m[rb], absmax16(v[i]));
        }
#pragma unroll
        for (int rb = 0; rb < NRB; ++rb) {
#pragma unroll
            for (int o = kLanesPerCb / 2; o > 0; o >>= 1) m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], o));
            m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], 8));
            m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], 16));
            if (lane < 8 && (lane % kLanesPerCb) == 0) atomicMax(&amax_bits[rb * NCB + cb], __float_as_int(m[rb]));
        }
        __syncthreads();
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int rb = NRB == 1 ? 0 : i;
            const Scale s = make_scale(__int_as_float(amax_bits[rb * NCB + cb]), p.clamp_min, kMaxQ, round_sf);
            inv[i] = s.inv;
        }
        // one thread per scale block stores it
        if (t < NRB * NCB) {
            const int rb = t / NCB, kb = t % NCB;
            const int64_t m_idx = sf_m0 + rb, k_idx = sf_k0 + kb;
            if (rb * BM < valid_rows && kb * BK < valid_cols) {
                const Scale s = make_scale(__int_as_float(amax_bits[t]), p.clamp_min, kMaxQ, round_sf);
                if (p.flags & TKQ_SF_UE8M0) {
                    uint8_t* base = static_cast<uint8_t*>(p.sf) + (k_idx >> 2) * p.sf_stride + 4 * m_idx;
                    base[k_idx & 3] = static_cast<uint8_t>(s.e8);
                    if (k_idx == num_kb - 1)  // zero the unused bytes of the last word
                        for (int64_t b = (k_idx & 3) + 1; b < 4; ++b) base[b] = 0;
                } else {
                    store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, m_idx, k_idx, s.sf);
                }
            }
        }
    }
    if (sf_only) return;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r_base + 32 * i;
        if (col_ok && r < valid_rows) {
            const int64_t col = col0 + c16 * 16;
            if constexpr (FMT == TKQ_FMT_E4M3) quantize_store_e4m3x16(v[i], inv[i], p.out + (row0 + r) * p.hidden + col);
            else quantize_store_e2m1x16(v[i], inv[i], p.out + (row0 + r) * (p.hidden / 2) + col / 2);
        }
    }
}

// ---------------------------------------------------------------------------
// Per-channel cast: one scale per (128 tokens x 1 channel); e4m3 only.
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kTileThreads) per_channel_cast_kernel(const TileParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint8_t* tile = smem;
    __shared__ uint64_t bar;
    __shared__ int col_amax_bits[kTile];
    __shared__ float col_inv[kTile];

    const int t = threadIdx.x, lane = t & 31;
    const int c16 = t & 7, r_base = t >> 3;
    const int64_t tile_m = blockIdx.x / p.tiles_k, tile_k = blockIdx.x % p.tiles_k;
    const int64_t row0 = tile_m * kTile, col0 = tile_k * kTile;
    const int valid_rows = static_cast<int>(p.num_tokens - row0 < kTile ? p.num_tokens - row0 : kTile);
    const int valid_cols = static_cast<int>(p.hidden - col0 < kTile ? p.hidden - col0 : kTile);
    const bool round_sf = p.flags & TKQ_ROUND_SF;

    if (t < kTile) col_amax_bits[t] = 0;
    if (!stage_tile<DT>(p, tile, &bar, row0, col0, valid_rows, valid_cols)) return;

    const bool col_ok = c16 * 16 < valid_cols;
    float v[4][16];
    float cm[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) cm[j] = 0.0f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r_base + 32 * i;
        if (col_ok && r < valid_rows) {
            read_chunk<DT>(tile, r, c16, v[i]);
        } else {
#pragma unroll
            for (int j = 0; j < 16; ++j) v[i][j] = 0.0f;
        }
#pragma unroll
        for (int j = 0; j < 16; ++j) cm[j] = fmaxf(cm[j], fabsf(v[i][j]));
    }
    // combine the 4 rows a warp holds per chunk, then the 8 warps through shared-memory atomics
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 8));
        cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 16));
    }
    if (lane < 8) {
#pragma unroll
        for (int j = 0; j < 16; ++j) atomicMax(&col_amax_bits[c16 * 16 + j], __float_as_int(cm[j]));
    }
    __syncthreads();
    if (t < kTile) {
        const Scale s = make_scale(__int_as_float(col_amax_bits[t]), p.clamp_min, 448.0f, round_sf);
        col_inv[t] = s.inv;
        if (t < valid_cols) static_cast<float*>(p.sf)[tile_m * p.hidden + col0 + t] = s.sf;
    }
    __syncthreads();
    float inv[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) inv[j] = col_inv[c16 * 16 + j];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int r = r_base + 32 * i;
        if (col_ok && r < valid_rows) {
            float s[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) s[j] = __fmul_rn(v[i][j], inv[j]);
            stg128(p.out + (row0 + r) * p.hidden + col0 + c16 * 16, cvt_e4m3x4(s[0], s[1], s[2], s[3]),
                   cvt_e4m3x4(s[4], s[5], s[6], s[7]), cvt_e4m3x4(s[8], s[9], s[10], s[11]),
                   cvt_e4m3x4(s[12], s[13], s[14], s[15]));
        }
    }
}

template <class Kernel>
static int launch_tile(Kernel kernel, const TileParams& p, int elem_bytes, const char* what, cudaStream_t stream) {
    const int smem = kTile * kTile * elem_bytes;
    if (smem > 48 * 1024) {
        const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return set_error(static_cast<int>(e), "cudaFuncSetAttribute(max dynamic shared memory) failed");
    }
    const int64_t tiles = ((p.num_tokens + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31)) return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    kernel<<<static_cast<unsigned>(tiles), kTileThreads, smem, stream>>>(p);
    return check_launch(what);
}

template <int DT, int FMT>
static int dispatch_block(const TileParams& p, int bm, int bk, cudaStream_t s) {
    constexpr int EB = TileElem<DT>::kBytes;
    const char* what = "per_block_cast";
    if (bm == 128 && bk == 128) return launch_tile(per_block_cast_kernel<DT, FMT, 128, 128>, p, EB, what, s);
    if (bm == 32 && bk == 32) return launch_tile(per_block_cast_kernel<DT, FMT, 32, 32>, p, EB, what, s);
    if (bm == 128 && bk == 32) return launch_tile(per_block_cast_kernel<DT, FMT, 128, 32>, p, EB, what, s);
    if (bm == 32 && bk == 128) return launch_tile(per_block_cast_kernel<DT, FMT, 32, 128>, p, EB, what, s);
    return set_error(TKQ_E_UNSUPPORTED, "per_block_cast: block sizes must be 32 or 128");
}

}  // namespace tkq

using namespace tkq;

// Non-zero if any tile kernel of this process gave up waiting for its staged tile since the
// last call; reading clears the flag.  Synchronises the device.
extern "C" int tkq_device_error(void) {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tile_wait_failed, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tile_wait_failed, &zero, sizeof(zero));
    return static_cast<int>(v);
}

extern "C" int tkq_per_block_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, int fmt, int block_m,
                                  int block_k, unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream) {
    if (num_tokens < 0 || hidden <= 0 || (in_dtype != TKQ_DT_BF16 && in_dtype != TKQ_DT_FP32) ||
        (fmt != TKQ_FMT_E4M3 && fmt != TKQ_FMT_E2M1))
        return set_error(TKQ_E_BAD_ARG, "per_block_cast: bad size, dtype or format");
    if (num_tokens == 0) return 0;
    const bool sf_only = flags & TKQ_SF_ONLY;
    if (x == nullptr || sf == nullptr || (!sf_only && out == nullptr)) return set_error(TKQ_E_BAD_ARG, "per_block_cast: null pointer");
    if ((flags & TKQ_SF_UE8M0) && !(flags & TKQ_SF_COL_MAJOR))
        return set_error(TKQ_E_UNSUPPORTED, "packed ue8m0 scales need the column-major layout");
    if ((flags & TKQ_CAST_ONLY) && (flags & (TKQ_SF_UE8M0 | TKQ_SF_COL_MAJOR | TKQ_SF_ONLY)))
        return set_error(TKQ_E_UNSUPPORTED, "precomputed scales must be row-major fp32");
    if (hidden % 64 != 0) return set_error(TKQ_E_UNSUPPORTED, "per_block_cast: hidden must be a multiple of 64");
    if (!aligned16(x) || (!sf_only && !aligned16(out)) || (reinterpret_cast<uintptr_t>(sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "per_block_cast: x and out must be 16-byte aligned, sf 4-byte aligned");
    TileParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.sf_stride = sf_stride;
    p.tiles_k = static_cast<uint32_t>((hidden + kTile - 1) / kTile);
    p.flags = flags;
    p.clamp_min = fmt == TKQ_FMT_E4M3 ? 1e-4f : 6.0f * 1.1754943508222875e-38f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_dtype == TKQ_DT_BF16)
        return fmt == TKQ_FMT_E4M3 ? dispatch_block<TKQ_DT_BF16, TKQ_FMT_E4M3>(p, block_m, block_k, s)
                                   : dispatch_block<TKQ_DT_BF16, TKQ_FMT_E2M1>(p, block_m, block_k, s);
    return fmt == TKQ_FMT_E4M3 ? dispatch_block<TKQ_DT_FP32, TKQ_FMT_E4M3>(p, block_m, block_k, s)
                               : dispatch_block<TKQ_DT_FP32, TKQ_FMT_E2M1>(p, block_m, block_k, s);
}

extern "C" int tkq_per_channel_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, unsigned flags,
                                    void* out, void* sf, void* stream) {
    if (num_tokens < 0 || hidden <= 0 || (in_dtype != TKQ_DT_BF16 && in_dtype != TKQ_DT_FP32))
        return set_error(TKQ_E_BAD_ARG, "per_channel_cast: bad size or dtype");
    if (num_tokens == 0) return 0;
    if (x == nullptr || sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "per_channel_cast: null pointer");
    if (flags & ~TKQ_ROUND_SF) return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast: only TKQ_ROUND_SF is defined");
    if (num_tokens % 128 != 0 || hidden % 64 != 0)
        return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast: num_tokens % 128 == 0 and hidden % 64 == 0 required");
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "per_channel_cast: x and out must be 16-byte aligned, sf 4-byte aligned");
    TileParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = sf;
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.sf_stride = hidden;
    p.tiles_k = static_cast<uint32_t>((hidden + kTile - 1) / kTile);
    p.flags = flags;
    p.clamp_min = 1e-4f;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    return in_dtype == TKQ_DT_BF16
               ? launch_tile(per_channel_cast_kernel<TKQ_DT_BF16>, p, 2, "per_channel_cast", s)
               : launch_tile(per_channel_cast_kernel<TKQ_DT_FP32>, p, 4, "per_channel_cast", s);
}
