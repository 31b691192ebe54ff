// Per-block and per-channel casts over 128 x 128 tiles.  Two families:
//   * staged: tiles arrive in shared memory by TMA (cp.async.bulk.tensor.2d, one instruction per tile
//     completing on an mbarrier; no multicast), persistent blocks keep several tile loads in flight
//     (run_tile_pipeline) -- fp32 input, the 32-wide block shapes, the transposing casts, the
//     per-channel cast of the largest tensors;
//   * direct: bf16 tiles of the 128 x 128 per-block cast and of the per-channel cast are read with 256-bit
//     loads into registers and never staged, which measured faster at every size but the largest
//     (per_block_cast_direct_kernel, per_channel_cast_direct_kernel).
//
// Thread mapping inside a tile (256 threads): thread t owns the 16-column chunk
// c16 = t % 8 of rows t / 8 + 32 * i, i = 0..3.  A warp therefore covers 4 full
// rows per i, reads shared memory in whole rows and writes 4 x 128 B of e4m3 per
// store instruction.
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_bf16.h>

#include <cstring>
#include <type_traits>

#include "tkq_async.cuh"
#include "tkq_launch.cuh"
#include "tkq_token_kernels.cuh"

namespace tkq {

constexpr int kTile = 128;
constexpr int kTileThreads = 256;

// Set when a kernel gave up waiting for its tile; read back by tkq_device_error().
__device__ unsigned int g_tile_wait_failed = 0;
// Number of (row, 16-value chunk) pieces whose input scale the lossless re-blocking could not represent exactly.
__device__ unsigned int g_lossless_range_violations = 0;

struct TileParams {
    const void* x;
    uint8_t* out;
    void* sf;
    int64_t num_tokens;
    int64_t hidden;
    int64_t sf_stride;
    uint32_t tiles_k;    // tiles along the channel dimension
    uint32_t num_tiles;  // tiles_k * ceil(num_tokens / 128)
    uint32_t stages;     // shared-memory tile buffers per block
    uint32_t flags;
    float clamp_min;
    bool fast_pow2;
    const int32_t* pos_to_token;  // direct per-channel cast only: output row i reads x row pos_to_token[i] (negative: zeros)
};

template <int DT>
struct TileElem {
    static constexpr int kBytes = DT == TKQ_DT_BF16 ? 2 : 4;
    static constexpr int kTileBytes = kTile * kTile * kBytes;
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

// Where tile number `tile` sits in the tensor.
struct TileCoord {
    int64_t tile_m, tile_k, row0, col0;
    int valid_rows, valid_cols;
};

__device__ __forceinline__ TileCoord tile_coord(const TileParams& p, uint32_t tile) {
    TileCoord c;
    c.tile_m = tile / p.tiles_k;
    c.tile_k = tile - c.tile_m * p.tiles_k;
    c.row0 = c.tile_m * kTile;
    c.col0 = c.tile_k * kTile;
    c.valid_rows = static_cast<int>(p.num_tokens - c.row0 < kTile ? p.num_tokens - c.row0 : kTile);
    c.valid_cols = static_cast<int>(p.hidden - c.col0 < kTile ? p.hidden - c.col0 : kTile);
    return c;
}

// Called by one thread: arms the stage's barrier with the tile's byte count and issues the tile load.
template <int DT>
__device__ __forceinline__ void issue_tile(const TileParams& p, const CUtensorMap* tmap, uint32_t tile, uint8_t* stage,
                                           uint64_t* bar) {
    const TileCoord c = tile_coord(p, tile);
    mbar_arrive_expect_tx(bar, TileElem<DT>::kTileBytes);
    tma_load_tile(stage, tmap, static_cast<int32_t>(c.col0), static_cast<int32_t>(c.row0), bar);
}

// The tile pipeline shared by the tile kernels.  Blocks are persistent: block b handles tiles b, b + grid, ...;
// thread 0 keeps `stages` tile loads in flight.  Per tile every thread calls `read(tile, coord)`, which copies
// the thread's part of the tile from shared memory into registers; after the barrier that follows, the stage
// is refilled and `consume(i, coord)` does the arithmetic (it contains block-wide barriers, so every thread
// calls it).
template <int DT, class Read, class Consume>
__device__ __forceinline__ void run_tile_pipeline_rw(const TileParams& p, const CUtensorMap* tmap, uint8_t* smem, uint64_t* full_bar,
                                                     Read read, Consume consume) {
    const uint32_t t = threadIdx.x;
    const uint32_t stages = p.stages;
    if (t == 0) {
        for (uint32_t s = 0; s < stages; ++s) mbar_init(full_bar + s, 1);
    }
    __syncthreads();
    const uint32_t first = blockIdx.x, step = gridDim.x;
    const uint32_t my_tiles = first < p.num_tiles ? (p.num_tiles - first + step - 1) / step : 0;
    if (t == 0) {
        for (uint32_t i = 0; i < stages && i < my_tiles; ++i)
            issue_tile<DT>(p, tmap, first + i * step, smem + static_cast<size_t>(i) * TileElem<DT>::kTileBytes, full_bar + i);
    }
    for (uint32_t i = 0; i < my_tiles; ++i) {
        const uint32_t s = i % stages, parity = (i / stages) & 1;
        const TileCoord c = tile_coord(p, first + i * step);
        if (!mbar_wait(full_bar + s, parity)) {
            atomicExch(&g_tile_wait_failed, 1u);
            if (t == 0) {  // tiles requested ahead still target this block's shared memory: wait for them (bounded) too
                for (uint32_t j = i + 1; j < my_tiles && j < i + stages; ++j) mbar_wait(full_bar + j % stages, (j / stages) & 1);
            }
            return;
        }
        read(smem + static_cast<size_t>(s) * TileElem<DT>::kTileBytes, c);
        // the reads above went through the generic proxy, the refill below goes through the async proxy:
        // order them before the barrier that lets thread 0 overwrite the stage
        fence_proxy_async_smem();
        __syncthreads();  // the stage is free again
        if (t == 0 && i + stages < my_tiles)
            issue_tile<DT>(p, tmap, first + (i + stages) * step, smem + static_cast<size_t>(s) * TileElem<DT>::kTileBytes, full_bar + s);
        consume(i, c);
    }
}

// The row-major register mapping used by the per-block and per-channel casts: thread t holds the 16-column chunk
// t % 8 of rows t / 8 + 32 k, k = 0..3 (zeros outside the tensor); `consume(i, coord, v, col_ok)`.
template <int DT, class Consume>
__device__ __forceinline__ void run_tile_pipeline(const TileParams& p, const CUtensorMap* tmap, uint8_t* smem, uint64_t* full_bar,
                                                  Consume consume) {
    const int c16 = threadIdx.x & 7, r_base = threadIdx.x >> 3;
    float v[4][16];
    bool col_ok = false;
    run_tile_pipeline_rw<DT>(
        p, tmap, smem, full_bar,
        [&](const uint8_t* tile, const TileCoord& c) {
            col_ok = c16 * 16 < c.valid_cols;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r_base + 32 * k;
                if (col_ok && r < c.valid_rows) {
                    read_chunk<DT>(tile, r, c16, v[k]);
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[k][j] = 0.0f;
                }
            }
        },
        [&](uint32_t i, const TileCoord& c) { consume(i, c, v, col_ok); });
}

// ---------------------------------------------------------------------------
// Per-block cast: one scale per (BM x BK) block, BM, BK in {32, 128}.
// ---------------------------------------------------------------------------
template <int DT, int FMT, int BM, int BK>
__global__ void __launch_bounds__(kTileThreads) per_block_cast_kernel(const __grid_constant__ CUtensorMap tmap, const TileParams p) {
    constexpr int NRB = kTile / BM, NCB = kTile / BK;  // scale blocks per tile
    constexpr int kLanesPerCb = BK / 16;                // lanes of a row that share a column block (2 or 8)
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[8];
    __shared__ int amax_bits[2][NRB * NCB];  // double-buffered by tile parity

    const int t = threadIdx.x, lane = t & 31;
    const int c16 = t & 7, r_base = t >> 3;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool cast_only = p.flags & TKQ_CAST_ONLY;
    const bool sf_only = p.flags & TKQ_SF_ONLY;
    const int cb = c16 * 16 / BK;
    const int64_t num_kb = (p.hidden + BK - 1) / BK;
    if (t < 2 * NRB * NCB) (&amax_bits[0][0])[t] = 0;

    run_tile_pipeline<DT>(p, &tmap, smem, full_bar, [&](uint32_t i, const TileCoord& c, float (&v)[4][16], bool col_ok) {
        int* amax = amax_bits[i & 1];
        const int64_t sf_m0 = c.row0 / BM, sf_k0 = c.col0 / BK;
        float inv[4];
        if (cast_only) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int rb = (r_base + 32 * k) / BM;
                const bool ok = col_ok && (r_base + 32 * k) < c.valid_rows;
                inv[k] = ok ? __fdiv_rn(1.0f, load_sf_f32_row_major(p.sf, p.sf_stride, sf_m0 + rb, sf_k0 + cb)) : 0.0f;
            }
        } else {
            // maxima per row block, combined over the lanes and warps that share the block
            float m[NRB];
#pragma unroll
            for (int rb = 0; rb < NRB; ++rb) m[rb] = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int rb = NRB == 1 ? 0 : k;  // BM = 32: rows r_base + 32 k lie in row block k
                m[rb] = fmaxf(m[rb], absmax16(v[k]));
            }
#pragma unroll
            for (int rb = 0; rb < NRB; ++rb) {
#pragma unroll
                for (int o = kLanesPerCb / 2; o > 0; o >>= 1) m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], o));
                m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], 8));
                m[rb] = fmaxf(m[rb], __shfl_xor_sync(kFullMask, m[rb], 16));
                if (lane < 8 && (lane % kLanesPerCb) == 0) atomicMax(&amax[rb * NCB + cb], __float_as_int(m[rb]));
            }
            __syncthreads();
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int rb = NRB == 1 ? 0 : k;
                if (NRB == 1 && k > 0) {
                    inv[k] = inv[0];
                } else {
                    inv[k] = make_scale_for<FMT>(__int_as_float(amax[rb * NCB + cb]), p.clamp_min, round_sf, p.fast_pow2).inv;
                }
            }
            // one thread per scale block stores it
            if (t < NRB * NCB) {
                const int rb = t / NCB, kb = t % NCB;
                const int64_t m_idx = sf_m0 + rb, k_idx = sf_k0 + kb;
                if (rb * BM < c.valid_rows && kb * BK < c.valid_cols) {
                    const Scale s = make_scale_for<FMT>(__int_as_float(amax[t]), p.clamp_min, round_sf, p.fast_pow2);
                    if (p.flags & TKQ_SF_UE8M0) store_sf_ue8m0_byte(p.sf, p.sf_stride, m_idx, static_cast<uint32_t>(k_idx), static_cast<uint32_t>(num_kb), s.e8);
                    else store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, m_idx, k_idx, s.sf);
                }
            }
            // this tile's maxima were all read before the next tile's first barrier; clear the other buffer for it
            if (t < NRB * NCB) amax_bits[(i + 1) & 1][t] = 0;
        }
        if (sf_only) return;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = r_base + 32 * k;
            if (col_ok && r < c.valid_rows) {
                const int64_t col = c.col0 + c16 * 16;
                if constexpr (FMT == TKQ_FMT_E4M3) quantize_store_e4m3x16(v[k], inv[k], p.out + (c.row0 + r) * p.hidden + col);
                else quantize_store_e2m1x16(v[k], inv[k], p.out + (c.row0 + r) * (p.hidden / 2) + col / 2);
            }
        }
    });
}

// ---------------------------------------------------------------------------
// "Light" staging for the per-channel cast of the largest bf16 tensors: ONE tile buffer per block and nothing of the
// tile kept in registers (the tile is read from shared memory twice, for the maximum and for the conversion), so
// that about 40 registers suffice and six blocks share an SM.  The blocks of an SM are in different phases (waiting
// for their tile, reducing, converting, storing), which is what overlaps memory and arithmetic here.
// ---------------------------------------------------------------------------
template <int DT>
constexpr int kLightBlocksPerSm = DT == TKQ_DT_BF16 ? 6 : 3;

// ---------------------------------------------------------------------------
// The 128 x 128 per-block cast of bf16 input straight from global memory: a thread loads its four 32-byte pieces of
// the tile (rows t / 8 + 32 k, columns 16 (t % 8) ..) with 256-bit loads, keeps them packed in 32 registers for both
// passes (maximum, conversion), and the block combines the maxima through shared memory with ONE barrier per tile
// (the slot of the 8 warp maxima alternates between two rows).  No staging buffer, no asynchronous copy to wait
// for: with four to five blocks per SM the loads of one block overlap the arithmetic and stores of the others.
// ---------------------------------------------------------------------------
template <int FMT>
__global__ void __launch_bounds__(kTileThreads, 5) per_block_cast_direct_kernel(const TileParams p, const bool wide) {
    __shared__ float warp_max[2][kTileThreads / 32];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int c16 = t & 7, r_base = t >> 3;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const bool cast_only = p.flags & TKQ_CAST_ONLY;
    const bool sf_only = p.flags & TKQ_SF_ONLY;
    const int64_t num_kb = (p.hidden + kTile - 1) / kTile;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    uint32_t n = 0;
    for (uint32_t idx = blockIdx.x; idx < p.num_tiles; idx += gridDim.x, ++n) {
        const TileCoord c = tile_coord(p, idx);
        const bool col_ok = c16 * 16 < c.valid_cols;
        PlainSource<TKQ_DT_BF16>::Raw raw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = r_base + 32 * k;
            if (col_ok && r < c.valid_rows) PlainSource<TKQ_DT_BF16>::issue(raw[k], xb + ((c.row0 + r) * p.hidden + c.col0 + c16 * 16) * 2, wide);
            else PlainSource<TKQ_DT_BF16>::zero(raw[k]);
        }
        float inv;
        if (cast_only) {
            inv = __fdiv_rn(1.0f, load_sf_f32_row_major(p.sf, p.sf_stride, c.tile_m, c.tile_k));
        } else {
            float m = 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                float v[16];
                PlainSource<TKQ_DT_BF16>::unpack(raw[k], v);
                m = fmaxf(m, absmax16(v));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(kFullMask, m, o));
            if (lane == 0) warp_max[n & 1][warp] = m;
            __syncthreads();
            m = warp_max[n & 1][0];
#pragma unroll
            for (int w = 1; w < kTileThreads / 32; ++w) m = fmaxf(m, warp_max[n & 1][w]);
            const Scale s = make_scale_for<FMT>(m, p.clamp_min, round_sf, p.fast_pow2);
            inv = s.inv;
            if (t == 0) {
                if (p.flags & TKQ_SF_UE8M0) store_sf_ue8m0_byte(p.sf, p.sf_stride, c.tile_m, static_cast<uint32_t>(c.tile_k), static_cast<uint32_t>(num_kb), s.e8);
                else store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, c.tile_m, c.tile_k, s.sf);
            }
        }
        if (!sf_only && col_ok) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r_base + 32 * k;
                if (r >= c.valid_rows) continue;
                float v[16];
                PlainSource<TKQ_DT_BF16>::unpack(raw[k], v);
                const int64_t col = c.col0 + c16 * 16;
                if constexpr (FMT == TKQ_FMT_E4M3) quantize_store_e4m3x16(v, inv, p.out + (c.row0 + r) * p.hidden + col);
                else quantize_store_e2m1x16(v, inv, p.out + (c.row0 + r) * (p.hidden / 2) + col / 2);
            }
        }
    }
}

// ---------------------------------------------------------------------------
// The per-channel cast (128 tokens x 1 channel) of bf16 input straight from global memory, same thread mapping as the
// direct per-block cast.  Column maxima stay packed (two |bf16| per word, compared as unsigned 16-bit integers):
// over the thread's four rows, over the four lanes of a warp that hold the same columns (two shuffles), then over
// the eight warps through shared memory, where thread j < 128 finishes column j, computes its scale once and
// leaves the inverse for the conversion pass.  Two barriers per tile, nothing staged.
// ---------------------------------------------------------------------------
template <bool kGather>
__global__ void __launch_bounds__(kTileThreads, 4) per_channel_cast_direct_kernel(const TileParams p, const bool wide) {
    __shared__ __align__(16) uint32_t warp_colmax[kTileThreads / 32][kTile / 2];
    __shared__ __align__(16) float col_inv[kTile];
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int c16 = t & 7, r_base = t >> 3;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    const uint8_t* xb = static_cast<const uint8_t*>(p.x);
    for (uint32_t idx = blockIdx.x; idx < p.num_tiles; idx += gridDim.x) {
        const TileCoord c = tile_coord(p, idx);
        const bool col_ok = c16 * 16 < c.valid_cols;
        PlainSource<TKQ_DT_BF16>::Raw raw[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = r_base + 32 * k;
            int64_t src_row = c.row0 + r;
            bool ok = col_ok && r < c.valid_rows;
            if (kGather && ok) {
                src_row = p.pos_to_token[c.row0 + r];
                ok = src_row >= 0;
            }
            if (ok) PlainSource<TKQ_DT_BF16>::issue(raw[k], xb + (src_row * p.hidden + c.col0 + c16 * 16) * 2, wide);
            else PlainSource<TKQ_DT_BF16>::zero(raw[k]);
        }
        uint32_t cm[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t a = max_u16x2(raw[0].a.v[i] & 0x7FFF7FFFu, raw[1].a.v[i] & 0x7FFF7FFFu);
            const uint32_t b = max_u16x2(raw[2].a.v[i] & 0x7FFF7FFFu, raw[3].a.v[i] & 0x7FFF7FFFu);
            cm[i] = max_u16x2(a, b);
            cm[i] = max_u16x2(cm[i], __shfl_xor_sync(kFullMask, cm[i], 8));
            cm[i] = max_u16x2(cm[i], __shfl_xor_sync(kFullMask, cm[i], 16));
        }
        if (lane < 8) {
            uint4* dst = reinterpret_cast<uint4*>(&warp_colmax[warp][lane * 8]);
            dst[0] = make_uint4(cm[0], cm[1], cm[2], cm[3]);
            dst[1] = make_uint4(cm[4], cm[5], cm[6], cm[7]);
        }
        __syncthreads();
        if (t < kTile) {
            uint32_t m = warp_colmax[0][t >> 1];
#pragma unroll
            for (int w = 1; w < kTileThreads / 32; ++w) m = max_u16x2(m, warp_colmax[w][t >> 1]);
            const float amax = __uint_as_float((t & 1) ? (m & 0xFFFF0000u) : (m << 16));
            const Scale s = make_scale_for<TKQ_FMT_E4M3>(amax, p.clamp_min, round_sf, p.fast_pow2);
            col_inv[t] = s.inv;
            if (t < c.valid_cols) static_cast<float*>(p.sf)[c.tile_m * p.hidden + c.col0 + t] = s.sf;
        }
        __syncthreads();
        if (col_ok) {
            float inv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 a = reinterpret_cast<const float4*>(&col_inv[c16 * 16])[q];
                inv[4 * q] = a.x, inv[4 * q + 1] = a.y, inv[4 * q + 2] = a.z, inv[4 * q + 3] = a.w;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r_base + 32 * k;
                if (r >= c.valid_rows) continue;
                float v[16], q[16];
                PlainSource<TKQ_DT_BF16>::unpack(raw[k], v);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float2 y = mul2(make_float2(v[j], v[j + 1]), make_float2(inv[j], inv[j + 1]));
                    q[j] = y.x;
                    q[j + 1] = y.y;
                }
                stg128(p.out + (c.row0 + r) * p.hidden + c.col0 + c16 * 16, cvt_e4m3x4(q[0], q[1], q[2], q[3]),
                       cvt_e4m3x4(q[4], q[5], q[6], q[7]), cvt_e4m3x4(q[8], q[9], q[10], q[11]),
                       cvt_e4m3x4(q[12], q[13], q[14], q[15]));
            }
        }
    }
}

template <int DT>
__global__ void __launch_bounds__(kTileThreads, kLightBlocksPerSm<DT>) per_channel_cast_light_kernel(const __grid_constant__ CUtensorMap tmap,
                                                                                                     const TileParams p) {
    extern __shared__ __align__(128) uint8_t tile[];
    __shared__ uint64_t bar;
    __shared__ float half_max[2][kTile];
    __shared__ __align__(16) float col_inv[kTile];
    using Elem = typename std::conditional<DT == TKQ_DT_BF16, uint16_t, float>::type;
    const int t = threadIdx.x;
    const int ch = t & 127, half = t >> 7;
    const int c16 = t & 7, r_base = t >> 3;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    if (t == 0) mbar_init(&bar, 1);
    __syncthreads();
    uint32_t n = 0;
    for (uint32_t idx = blockIdx.x; idx < p.num_tiles; idx += gridDim.x, ++n) {
        const TileCoord c = tile_coord(p, idx);
        if (t == 0) issue_tile<DT>(p, &tmap, idx, tile, &bar);
        if (!mbar_wait(&bar, n & 1u)) {
            atomicExch(&g_tile_wait_failed, 1u);
            return;
        }
        // thread = (channel, 64 tokens): consecutive threads read consecutive channels, no bank conflicts
        const Elem* src = reinterpret_cast<const Elem*>(tile) + static_cast<size_t>(half) * 64 * kTile + ch;
        float m = 0.0f;
#pragma unroll 16
        for (int r = 0; r < 64; r += 2) {
            float a, b;
            if constexpr (DT == TKQ_DT_BF16) {
                a = __uint_as_float(static_cast<uint32_t>(src[r * kTile]) << 16);
                b = __uint_as_float(static_cast<uint32_t>(src[(r + 1) * kTile]) << 16);
            } else {
                a = src[r * kTile];
                b = src[(r + 1) * kTile];
            }
            m = max3_abs(m, a, b);
        }
        half_max[half][ch] = m;
        __syncthreads();
        if (t < kTile) {
            const Scale s = make_scale_for<TKQ_FMT_E4M3>(fmaxf(half_max[0][t], half_max[1][t]), p.clamp_min, round_sf, p.fast_pow2);
            col_inv[t] = s.inv;
            if (t < c.valid_cols) static_cast<float*>(p.sf)[c.tile_m * p.hidden + c.col0 + t] = s.sf;
        }
        __syncthreads();
        if (c16 * 16 < c.valid_cols) {
            float inv[16];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const float4 a = reinterpret_cast<const float4*>(&col_inv[c16 * 16])[q];
                inv[4 * q] = a.x, inv[4 * q + 1] = a.y, inv[4 * q + 2] = a.z, inv[4 * q + 3] = a.w;
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int r = r_base + 32 * k;
                if (r >= c.valid_rows) continue;
                float v[16], q[16];
                read_chunk<DT>(tile, r, c16, v);
#pragma unroll
                for (int j = 0; j < 16; j += 2) {
                    const float2 y = mul2(make_float2(v[j], v[j + 1]), make_float2(inv[j], inv[j + 1]));
                    q[j] = y.x;
                    q[j + 1] = y.y;
                }
                stg128(p.out + (c.row0 + r) * p.hidden + c.col0 + c16 * 16, cvt_e4m3x4(q[0], q[1], q[2], q[3]),
                       cvt_e4m3x4(q[4], q[5], q[6], q[7]), cvt_e4m3x4(q[8], q[9], q[10], q[11]),
                       cvt_e4m3x4(q[12], q[13], q[14], q[15]));
            }
        }
        fence_proxy_async_smem();
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------
// Per-channel cast: one scale per (128 tokens x 1 channel); e4m3 only.
// ---------------------------------------------------------------------------
template <int DT>
__global__ void __launch_bounds__(kTileThreads) per_channel_cast_kernel(const __grid_constant__ CUtensorMap tmap, const TileParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[8];
    __shared__ __align__(16) float warp_max[kTileThreads / 32][kTile];  // column maxima of each warp's 16 rows
    __shared__ float col_inv[kTile];

    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int c16 = t & 7, r_base = t >> 3;
    const bool round_sf = p.flags & TKQ_ROUND_SF;

    run_tile_pipeline<DT>(p, &tmap, smem, full_bar, [&](uint32_t, const TileCoord& c, float (&v)[4][16], bool col_ok) {
        float cm[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) cm[j] = max3_abs(fabsf(v[0][j]), v[1][j], max3_abs(0.0f, v[2][j], v[3][j]));
        // combine the 4 row groups a warp holds per chunk by shuffles, then the 8 warps through shared memory
        // (plain stores: every warp has its own row of warp_max)
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 8));
            cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 16));
        }
        if (lane < 8) {
            float4* dst = reinterpret_cast<float4*>(&warp_max[warp][c16 * 16]);
#pragma unroll
            for (int q = 0; q < 4; ++q) dst[q] = make_float4(cm[4 * q], cm[4 * q + 1], cm[4 * q + 2], cm[4 * q + 3]);
        }
        __syncthreads();
        if (t < kTile) {
            float m = warp_max[0][t];
#pragma unroll
            for (int w = 1; w < kTileThreads / 32; ++w) m = fmaxf(m, warp_max[w][t]);
            const Scale s = make_scale_for<TKQ_FMT_E4M3>(m, p.clamp_min, round_sf, p.fast_pow2);
            col_inv[t] = s.inv;
            if (t < c.valid_cols) static_cast<float*>(p.sf)[c.tile_m * p.hidden + c.col0 + t] = s.sf;
        }
        __syncthreads();
        float inv[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) inv[j] = col_inv[c16 * 16 + j];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = r_base + 32 * k;
            if (col_ok && r < c.valid_rows) {
                float q[16];
#pragma unroll
                for (int j = 0; j < 16; ++j) q[j] = __fmul_rn(v[k][j], inv[j]);
                stg128(p.out + (c.row0 + r) * p.hidden + c.col0 + c16 * 16, cvt_e4m3x4(q[0], q[1], q[2], q[3]),
                       cvt_e4m3x4(q[4], q[5], q[6], q[7]), cvt_e4m3x4(q[8], q[9], q[10], q[11]),
                       cvt_e4m3x4(q[12], q[13], q[14], q[15]));
            }
        }
    });
}

// ---------------------------------------------------------------------------
// Per-channel cast with transposed output: one scale per (NPT tokens x 1 channel), NPT = 32 or 128, data written
// as [hidden, num_tokens] (reference: tile_kernels/quant/per_channel_cast_and_transpose_kernel.py:85-123).
// The tile is read from shared memory in the transposed sense: thread t owns channel t % 128 and the 64 tokens
// (t / 128) * 64 ... of the tile, so a warp reads 64 contiguous bytes per token row (no bank conflicts), the
// column maximum is mostly thread-local, and 32 consecutive tokens of a channel leave as one 256-bit store.
// ---------------------------------------------------------------------------
template <int NPT>
__global__ void __launch_bounds__(kTileThreads) per_channel_cast_transpose_kernel(const __grid_constant__ CUtensorMap tmap,
                                                                                  const TileParams p) {
    constexpr int kBlocksPerThread = 64 / (NPT < 64 ? NPT : 64);  // scale blocks inside a thread's 64 tokens: 2 or 1
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[8];
    __shared__ float half_max[2][2][kTile];  // [tile parity][token half][channel], NPT = 128 only
    const int t = threadIdx.x;
    const int ch = t & 127, half = t >> 7;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    uint32_t packed[32];  // 64 bf16: tokens 2i (low half) and 2i + 1 (high half) of the thread's range

    run_tile_pipeline_rw<TKQ_DT_BF16>(
        p, &tmap, smem, full_bar,
        [&](const uint8_t* tile, const TileCoord&) {
            const uint16_t* src = reinterpret_cast<const uint16_t*>(tile) + static_cast<size_t>(half) * 64 * kTile + ch;
#pragma unroll
            for (int i = 0; i < 32; ++i)
                packed[i] = static_cast<uint32_t>(src[(2 * i) * kTile]) | (static_cast<uint32_t>(src[(2 * i + 1) * kTile]) << 16);
        },
        [&](uint32_t i, const TileCoord& c) {
            float m[kBlocksPerThread];
#pragma unroll
            for (int b = 0; b < kBlocksPerThread; ++b) {
                m[b] = 0.0f;
#pragma unroll
                for (int q = 0; q < 32 / kBlocksPerThread; ++q) {
                    const uint32_t w = packed[b * (32 / kBlocksPerThread) + q];
                    m[b] = max3_abs(m[b], bf16_lo(w), bf16_hi(w));
                }
            }
            if constexpr (NPT == 128) {
                half_max[i & 1][half][ch] = m[0];
                __syncthreads();
                m[0] = fmaxf(half_max[i & 1][0][ch], half_max[i & 1][1][ch]);
            }
            const bool ch_ok = ch < c.valid_cols;
            float inv[kBlocksPerThread];
#pragma unroll
            for (int b = 0; b < kBlocksPerThread; ++b) {
                const Scale s = make_scale_for<TKQ_FMT_E4M3>(m[b], p.clamp_min, round_sf, p.fast_pow2);
                inv[b] = s.inv;
                const int64_t sf_row = NPT == 128 ? c.tile_m : c.tile_m * (kTile / NPT) + half * kBlocksPerThread + b;
                const bool tokens_ok = NPT == 128 ? true : (half * 64 + b * NPT) < c.valid_rows;
                if (ch_ok && tokens_ok && (NPT != 128 || half == 0)) static_cast<float*>(p.sf)[sf_row * p.hidden + c.col0 + ch] = s.sf;
            }
            if (!ch_ok) return;
            uint8_t* dst = p.out + (c.col0 + ch) * p.num_tokens + c.row0 + half * 64;
            // 16 tokens = 8 packed words -> 16 bytes; two such groups leave as ONE 256-bit store, so that every lane
            // writes whole 32-byte sectors (lanes are num_tokens bytes apart: half-sector stores cost twice)
            const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
                if (half * 64 + g2 * 32 >= c.valid_rows) break;
                uint32_t o[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const float k = inv[kBlocksPerThread == 1 ? 0 : g2];
                    const uint32_t w0 = packed[g2 * 16 + 2 * q], w1 = packed[g2 * 16 + 2 * q + 1];
                    o[q] = cvt_e4m3x4(__fmul_rn(bf16_lo(w0), k), __fmul_rn(bf16_hi(w0), k), __fmul_rn(bf16_lo(w1), k),
                                      __fmul_rn(bf16_hi(w1), k));
                }
                if (wide && half * 64 + g2 * 32 + 16 < c.valid_rows) {
                    stg256(dst + g2 * 32, o);
                } else {
                    stg128(dst + g2 * 32, o[0], o[1], o[2], o[3]);
                    if (half * 64 + g2 * 32 + 16 < c.valid_rows) stg128(dst + g2 * 32 + 16, o[4], o[5], o[6], o[7]);
                }
            }
        });
}

// ---------------------------------------------------------------------------
// Fused SwiGLU + per-channel cast (+ transpose): the activation silu(gate) * up is formed in fp32, rounded to
// bf16, and that bf16 tile is cast with one scale per (NPT tokens x 1 channel), written either as
// [num_tokens, hidden] or transposed (reference:
// tile_kernels/quant/swiglu_forward_and_per_channel_cast_and_transpose_kernel.py:177-231; its test quantises
// the bf16-rounded activation, tests/quant/test_swiglu_forward_and_per_channel_cast_and_transpose.py:63-66).
// One block per 128 x 128 output tile: the activation tile is built in shared memory from plain vector loads
// of the two input halves, then read back in whichever register mapping suits the output layout.
// ---------------------------------------------------------------------------
struct SwigluChannelParams {
    const void* x;  // [num_tokens, 2 * hidden] bf16
    uint8_t* out;
    float* sf;
    int64_t num_tokens, hidden;
    uint32_t tiles_k;
    uint32_t flags;
    float clamp_min;
    float swiglu_clamp;  // < 0: none
    bool fast_pow2;
    bool bf16_gates;
    bool wide_loads;
};

template <int NPT, bool kTranspose>
__global__ void __launch_bounds__(kTileThreads) swiglu_per_channel_cast_kernel(const SwigluChannelParams p) {
    constexpr int NRB = kTile / NPT;  // scale blocks along the tokens of a tile: 1 or 4
    __shared__ __align__(16) uint16_t act[kTile][kTile];  // the bf16 activation tile
    __shared__ int col_amax_bits[NRB][kTile];
    __shared__ float col_inv[NRB][kTile];
    using Src = SwigluSource<TKQ_DT_BF16>;
    const int t = threadIdx.x, lane = t & 31;
    const int c16 = t & 7, r_base = t >> 3;
    const int64_t tile_m = blockIdx.x / p.tiles_k, tile_k = blockIdx.x % p.tiles_k;
    const int64_t row0 = tile_m * kTile, col0 = tile_k * kTile;
    const int valid_cols = static_cast<int>(p.hidden - col0 < kTile ? p.hidden - col0 : kTile);
    const bool col_ok = c16 * 16 < valid_cols;
    const bool round_sf = p.flags & TKQ_ROUND_SF;
    for (int i = t; i < NRB * kTile; i += kTileThreads) (&col_amax_bits[0][0])[i] = 0;

    // 1. activation tile -> shared memory (num_tokens is a multiple of 128: every tile row exists)
    ClampCounters unused;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = r_base + 32 * k;
        uint32_t w[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (col_ok) {
            typename Src::Raw raw;
            Src::issue(raw, static_cast<const uint8_t*>(p.x) + ((row0 + r) * 2 * p.hidden + col0 + c16 * 16) * 2, p.wide_loads, p.hidden);
            float y[16];
            if (p.swiglu_clamp >= 0.0f) Src::template unpack<true, false, false>(raw, y, p.swiglu_clamp, 1.0f, unused, p.bf16_gates);
            else Src::template unpack<false, false, false>(raw, y, 0.0f, 1.0f, unused, p.bf16_gates);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const __nv_bfloat162 b = __floats2bfloat162_rn(y[2 * j], y[2 * j + 1]);
                w[j] = *reinterpret_cast<const uint32_t*>(&b);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(&act[r][c16 * 16]);
        dst[0] = make_uint4(w[0], w[1], w[2], w[3]);
        dst[1] = make_uint4(w[4], w[5], w[6], w[7]);
    }
    __syncthreads();

    // 2. column maxima per scale block: thread t < 128 * NRB scans its channel over NPT tokens (conflict-free:
    //    consecutive threads read consecutive channels)
    for (int i = t; i < NRB * kTile; i += kTileThreads) {
        const int rb = i / kTile, ch = i % kTile;
        float m = 0.0f;
#pragma unroll 8
        for (int r = 0; r < NPT; r += 2)
            m = max3_abs(m, __uint_as_float(static_cast<uint32_t>(act[rb * NPT + r][ch]) << 16),
                         __uint_as_float(static_cast<uint32_t>(act[rb * NPT + r + 1][ch]) << 16));
        const Scale s = make_scale_for<TKQ_FMT_E4M3>(m, p.clamp_min, round_sf, p.fast_pow2);
        col_inv[rb][ch] = s.inv;
        if (ch < valid_cols) p.sf[(tile_m * NRB + rb) * p.hidden + col0 + ch] = s.sf;
    }
    __syncthreads();

    // 3. convert and store
    if constexpr (!kTranspose) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = r_base + 32 * k;
            if (!col_ok) continue;
            float v[16], q[16];
            read_chunk<TKQ_DT_BF16>(reinterpret_cast<const uint8_t*>(&act[0][0]), r, c16, v);
            const float* inv = col_inv[r / NPT] + c16 * 16;
#pragma unroll
            for (int j = 0; j < 16; ++j) q[j] = __fmul_rn(v[j], inv[j]);
            stg128(p.out + (row0 + r) * p.hidden + col0 + c16 * 16, cvt_e4m3x4(q[0], q[1], q[2], q[3]), cvt_e4m3x4(q[4], q[5], q[6], q[7]),
                   cvt_e4m3x4(q[8], q[9], q[10], q[11]), cvt_e4m3x4(q[12], q[13], q[14], q[15]));
        }
    } else {
        // thread = (channel, 64 tokens)
        const int ch = t & 127, half = t >> 7;
        if (ch < valid_cols) {
            uint8_t* dst = p.out + (col0 + ch) * p.num_tokens + row0 + half * 64;
            const bool wide = (reinterpret_cast<uintptr_t>(dst) & 31u) == 0;
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {  // 32 tokens of the channel: one 256-bit store (whole sectors per lane)
                const int r0 = half * 64 + g2 * 32;
                const float k = col_inv[r0 / NPT][ch];
                uint32_t o[8];
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    float f[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) f[e] = __fmul_rn(__uint_as_float(static_cast<uint32_t>(act[r0 + 4 * q + e][ch]) << 16), k);
                    o[q] = cvt_e4m3x4(f[0], f[1], f[2], f[3]);
                }
                if (wide) {
                    stg256(dst + g2 * 32, o);
                } else {
                    stg128(dst + g2 * 32, o[0], o[1], o[2], o[3]);
                    stg128(dst + g2 * 32 + 16, o[4], o[5], o[6], o[7]);
                }
            }
        }
    }
    (void)lane;
}

// ---------------------------------------------------------------------------
// Lossless FP4 -> FP8 re-blocking: the input is packed e2m1 with power-of-two scales per (in_bm x in_bk) block;
// the output is e4m3 with power-of-two scales per (out_bm x out_bk) block.  The output exponent of a block is the
// largest input exponent inside it minus 6 (not below 0); every value becomes fp4 * 2^(e_in - e_out), which e4m3
// represents exactly as long as e_in + 5 >= e_out (reference: tile_kernels/quant/per_block_cast_lossless_kernel.py:
// 96-131; where the reference asserts that condition on the device, this kernel rounds to nearest and counts).
// Tiles of 128 rows x 256 columns (a row of a tile is 128 bytes of input and 256 bytes of output); a thread owns four
// 32-value pieces (rows t / 8 + 32 k, columns 32 (t % 8) ..): 16 bytes in, one 32-byte sector out.
// ---------------------------------------------------------------------------
struct LosslessParams {
    TokenCastParams in;  // x, in_sf*, in_block_*, num_tokens, hidden
    void* sf;
    int64_t sf_stride;
    uint32_t tiles_k;    // ceil(hidden / 256)
    uint32_t flags;
    bool wide_stores;    // out is 32-byte aligned
};

// Resident blocks per SM and tiles copied ahead, measured on B200 for [32768, 7168] with 128 x 128 output blocks (352 MB
// moved; a device copy of as many bytes takes 54.9 us): 2 blocks / 1 tile ahead 61.6 us, 2 / 2 65.3, 2 / 3 64.8-67.4,
// 3 / 1 71.3, 3 / 2 71.6, 4 / 1 71.6, 1 / 2 72.3, 1 / 4 73.3, 1 / 8 91.0.  Two thirds of the traffic are writes: more
// blocks or deeper copies only add streams for the DRAM to interleave.
constexpr int kLosslessBlocksPerSm = 2;
constexpr int kLosslessDepth = 1;
constexpr int kLosslessCols = 256;

// A thread's part of one tile: the codes of its four pieces and, per piece, the input exponents of its two 16-value halves
// (equal unless the input blocks are 16 wide).
struct LosslessPieces {
    uint4 codes[4];
    uint32_t e_in[4][2];
};

// Tiles on their way to a block: every thread copies its own pieces (16 bytes of codes and the aligned words that hold
// the piece's input scales) to shared memory with asynchronous copies, kLosslessDepth tiles ahead, and reads back only
// what it copied itself, so that the copies need no barrier, only the thread's own wait_group.  Registers cannot
// hold that much: with the next tile in registers a thread had 32 bytes in flight and the kernel ran at 0.61 of the
// copy bandwidth.
struct LosslessStage {
    uint4 codes[4][kTileThreads];
    uint32_t scale_word[2][4][kTileThreads];
};

__device__ __forceinline__ void cp_async_16(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem_dst, const void* gmem_src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_u32(smem_dst)), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The aligned 32-bit word that holds the input scale of (row, col): the fp32 scale itself, or four packed ue8m0 bytes.
__device__ __forceinline__ const uint32_t* input_scale_word(const TokenCastParams& p, uint32_t row, uint32_t col) {
    const int64_t m = p.in_shift_m1 ? row >> (p.in_shift_m1 - 1) : row / p.in_block_m;
    const int64_t k = p.in_shift_k1 ? col >> (p.in_shift_k1 - 1) : col / p.in_block_k;
    if (p.in_sf_flags & TKQ_SF_UE8M0) return reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(p.in_sf) + (k >> 2) * p.in_sf_stride + 4 * m);
    const uint32_t* f = static_cast<const uint32_t*>(p.in_sf);
    return (p.in_sf_flags & TKQ_SF_COL_MAJOR) ? f + k * p.in_sf_stride + m : f + m * p.in_sf_stride + k;
}

// kFull: every row and column of the tile exists.  hidden is a multiple of 32, so a piece exists whole or not at all.
template <bool kFull>
__device__ __forceinline__ void lossless_issue(const LosslessParams& p, uint32_t tile_m, uint32_t tile_k, int t, int c32, int r_base, LosslessStage& st) {
    const uint32_t row0 = tile_m * kTile + r_base, col = tile_k * kLosslessCols + c32 * 32;
    const bool col_ok = kFull || col < static_cast<uint32_t>(p.in.hidden);
    const bool two_scales = p.in.in_block_k == 16;
    const uint8_t* src = static_cast<const uint8_t*>(p.in.x) + (static_cast<int64_t>(row0) * p.in.x_stride + col) / 2;
    const uint32_t pitch = static_cast<uint32_t>(p.in.x_stride) * 16u;  // bytes between a thread's pieces: 32 rows of packed FP4
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t r = row0 + 32 * k;
        if (kFull || (col_ok && r < static_cast<uint32_t>(p.in.num_tokens))) {
            cp_async_16(&st.codes[k][t], src + k * pitch);
            cp_async_4(&st.scale_word[0][k][t], input_scale_word(p.in, r, col));
            if (two_scales) cp_async_4(&st.scale_word[1][k][t], input_scale_word(p.in, r, col + 16));
        } else {
            st.codes[k][t] = make_uint4(0u, 0u, 0u, 0u);
            st.scale_word[0][k][t] = 0u;
            st.scale_word[1][k][t] = 0u;
        }
    }
}

// The thread's pieces of a tile whose copies have landed.
__device__ __forceinline__ void lossless_fetch(const LosslessParams& p, const LosslessStage& st, uint32_t tile_k, int t, int c32, LosslessPieces& q) {
    const uint32_t col = tile_k * kLosslessCols + c32 * 32;
    const bool ue8m0 = p.in.in_sf_flags & TKQ_SF_UE8M0;
    const bool two_scales = p.in.in_block_k == 16;
    const uint32_t k0 = p.in.in_shift_k1 ? col >> (p.in.in_shift_k1 - 1) : col / p.in.in_block_k;
    const uint32_t shift0 = ue8m0 ? 8u * (k0 & 3u) : 23u, shift1 = ue8m0 ? 8u * ((k0 + 1u) & 3u) : 23u;
    const uint32_t mask = ue8m0 ? 0xFFu : 0x1FFu;  // scales are positive: bit 8 of the shifted fp32 word is its sign, zero
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        q.codes[i] = st.codes[i][t];
        q.e_in[i][0] = (st.scale_word[0][i][t] >> shift0) & mask;
        q.e_in[i][1] = two_scales ? (st.scale_word[1][i][t] >> shift1) & mask : q.e_in[i][0];
    }
}

// 8 FP4 codes (one word, even index in the low nibble) times a power of two (the same f16 in both halves of
// `rel`) -> 8 e4m3 bytes.  The arithmetic stays in f16: a product is exact there (an FP4 value has one mantissa bit
// and rel >= 2^-14), so rounding it to e4m3 gives what the fp32 route of the other casts gives, in 3 instead of 5
// instructions per pair.
__device__ __forceinline__ void fp4x8_times_pow2_to_e4m3(uint32_t word, uint32_t rel, uint32_t& out0, uint32_t& out1) {
    asm("{ .reg .b8 b0, b1, b2, b3; .reg .b16 c0, c1, c2, c3; .reg .b32 h0, h1, h2, h3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %2;\n\t"
        "cvt.rn.f16x2.e2m1x2 h0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 h1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 h2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 h3, b3;\n\t"
        "mul.rn.f16x2 h0, h0, %3;\n\t"
        "mul.rn.f16x2 h1, h1, %3;\n\t"
        "mul.rn.f16x2 h2, h2, %3;\n\t"
        "mul.rn.f16x2 h3, h3, %3;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 c0, h0;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 c1, h1;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 c2, h2;\n\t"
        "cvt.rn.satfinite.e4m3x2.f16x2 c3, h3;\n\t"
        "mov.b32 %0, {c0, c1};\n\t"
        "mov.b32 %1, {c2, c3}; }"
        : "=r"(out0), "=r"(out1)
        : "r"(word), "r"(rel));
}

// 2^(e_in - e_out) as f16 in both halves of a word; counts the pieces the reference would assert on (e_in + 5 >= e_out,
// exact representability).  The difference is at most 6 (the block's maximum covers e_in); below 2^-14 every product is
// less than half of e4m3's smallest step and rounds to zero.
__device__ __forceinline__ uint32_t lossless_rel(uint32_t e_in, int e_out) {
    const int d = static_cast<int>(e_in) - e_out;
    if (d < -5) atomicAdd(&g_lossless_range_violations, 1u);
    const uint32_t h = d >= -14 ? static_cast<uint32_t>(d + 15) << 10 : 0u;
    return h | (h << 16);
}

// One tile: exponent maxima per output block (first over the lanes of the warp that hold pieces of the same block -- a
// warp is 4 rows x 8 pieces and its rows lie in one 32-row band -- then one shared-memory atomic per warp and block;
// one atomic per piece is a thousand atomics on a single word for 128 x 128 blocks), the block's barrier, scales, codes.
template <int OBM, int OBK, bool kFull>
__device__ __forceinline__ void lossless_tile(const LosslessParams& p, const LosslessPieces& cur, uint32_t tile_m, uint32_t tile_k, int* emax,
                                              int* emax_next, int t, int c32, int r_base) {
    constexpr int NRB = kTile / OBM, NCB = kLosslessCols / OBK;
    const uint32_t hidden = static_cast<uint32_t>(p.in.hidden);
    const uint32_t row0 = tile_m * kTile, col0 = tile_k * kLosslessCols;
    const int valid_rows = kFull ? kTile : static_cast<int>(min(static_cast<uint32_t>(p.in.num_tokens) - row0, static_cast<uint32_t>(kTile)));
    const int valid_cols = kFull ? kLosslessCols : static_cast<int>(min(hidden - col0, static_cast<uint32_t>(kLosslessCols)));
    const int cb = c32 * 32 / OBK;
    for (int i = t; i < NRB * NCB; i += kTileThreads) emax_next[i] = 0;

    int m[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) m[k] = static_cast<int>(max(cur.e_in[k][0], cur.e_in[k][1]));
    if constexpr (OBM == kTile) m[0] = max(max(m[0], m[1]), max(m[2], m[3]));
#pragma unroll
    for (int k = 0; k < (OBM == kTile ? 1 : 4); ++k) {
        if (OBK == 128) {
            m[k] = max(m[k], __shfl_xor_sync(kFullMask, m[k], 1));
            m[k] = max(m[k], __shfl_xor_sync(kFullMask, m[k], 2));
        }
        if (OBM >= 32) {
            m[k] = max(m[k], __shfl_xor_sync(kFullMask, m[k], 8));
            m[k] = max(m[k], __shfl_xor_sync(kFullMask, m[k], 16));
        }
    }
    if ((OBK == 32 || (c32 & 3) == 0) && (OBM < 32 || (t & 31) < 8)) {
        if constexpr (OBM == kTile) {
            atomicMax(&emax[cb], m[0]);
        } else {
#pragma unroll
            for (int k = 0; k < 4; ++k) atomicMax(&emax[((r_base + 32 * k) / OBM) * NCB + cb], m[k]);
        }
    }
    __syncthreads();
    for (int i = t; i < NRB * NCB; i += kTileThreads) {
        const int rb = i / NCB, kb = i % NCB;
        if (rb * OBM < valid_rows && kb * OBK < valid_cols) {
            const uint32_t e = emax[i] >= 6 ? emax[i] - 6 : 0;
            const int64_t m_idx = static_cast<int64_t>(tile_m) * NRB + rb;
            const uint32_t k_idx = tile_k * NCB + kb;
            if (p.flags & TKQ_SF_UE8M0) store_sf_ue8m0_byte(p.sf, p.sf_stride, m_idx, k_idx, (hidden + OBK - 1) / OBK, e);
            else store_sf_f32(p.sf, p.sf_stride, p.flags & TKQ_SF_COL_MAJOR, m_idx, k_idx, __uint_as_float(e << 23));
        }
    }
    if (!kFull && c32 * 32 >= valid_cols) return;  // after the tile's only barrier
    uint8_t* dst = p.in.out + (static_cast<int64_t>(row0 + r_base) * hidden + col0 + c32 * 32);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = r_base + 32 * k;
        if (kFull || r < valid_rows) {
            const int mx = emax[(r / OBM) * NCB + cb];
            const int e_out = mx >= 6 ? mx - 6 : 0;
            const uint32_t rel0 = lossless_rel(cur.e_in[k][0], e_out), rel1 = lossless_rel(cur.e_in[k][1], e_out);
            uint32_t w[8];
            fp4x8_times_pow2_to_e4m3(cur.codes[k].x, rel0, w[0], w[1]);
            fp4x8_times_pow2_to_e4m3(cur.codes[k].y, rel0, w[2], w[3]);
            fp4x8_times_pow2_to_e4m3(cur.codes[k].z, rel1, w[4], w[5]);
            fp4x8_times_pow2_to_e4m3(cur.codes[k].w, rel1, w[6], w[7]);
            uint8_t* d = dst + static_cast<uint32_t>(k) * 32u * hidden;
            if (p.wide_stores) {
                stg256(d, w);
            } else {
                stg128(d, w[0], w[1], w[2], w[3]);
                stg128(d + 16, w[4], w[5], w[6], w[7]);
            }
        }
    }
}

// Persistent blocks: block b takes tiles b, b + grid, ...; the copies of the tiles kLosslessDepth ahead are issued
// before the current one is reduced and stored.  The exponent maxima rotate over three buffers: the one for the next
// tile is cleared before this tile's barrier, when nobody reads it.  OBM x OBK is the output block (1 | 32 | 128) x (32 | 128).
template <int OBM, int OBK>
__global__ void __launch_bounds__(kTileThreads, kLosslessBlocksPerSm) per_block_cast_lossless_kernel(const LosslessParams p, const uint32_t num_tiles) {
    constexpr int NRB = kTile / OBM, NCB = kLosslessCols / OBK;
    constexpr int kStages = kLosslessDepth + 1;
    extern __shared__ __align__(16) uint8_t lossless_smem[];
    LosslessStage* const stages = reinterpret_cast<LosslessStage*>(lossless_smem);
    __shared__ int exp_max[3][NRB * NCB];
    const int t = threadIdx.x;
    const int c32 = t & 7, r_base = t >> 3;
    const uint32_t full_m = static_cast<uint32_t>(p.in.num_tokens) / kTile, full_k = static_cast<uint32_t>(p.in.hidden) / kLosslessCols;
    const uint32_t step_m = gridDim.x / p.tiles_k, step_k = gridDim.x - step_m * p.tiles_k;
    for (int i = t; i < NRB * NCB; i += kTileThreads) exp_max[0][i] = 0;
    __syncthreads();

    // (tile_m, tile_k) of the tile being processed and of the one being copied advance by the grid size without divisions
    auto advance = [&](uint32_t& m, uint32_t& k) {
        m += step_m;
        k += step_k;
        if (k >= p.tiles_k) {
            k -= p.tiles_k;
            ++m;
        }
    };
    auto issue = [&](uint32_t tile, uint32_t m, uint32_t k, uint32_t stage) {  // one group per tile slot, empty past the end
        if (tile < num_tiles) {
            if (m < full_m && k < full_k) lossless_issue<true>(p, m, k, t, c32, r_base, stages[stage]);
            else lossless_issue<false>(p, m, k, t, c32, r_base, stages[stage]);
        }
        cp_async_commit();
    };
    uint32_t tile = blockIdx.x;
    uint32_t cur_m = tile / p.tiles_k, cur_k = tile - cur_m * p.tiles_k;
    uint32_t nxt_tile = tile, nxt_m = cur_m, nxt_k = cur_k, nxt_stage = 0;
#pragma unroll
    for (int d = 0; d < kLosslessDepth; ++d) {
        issue(nxt_tile, nxt_m, nxt_k, nxt_stage);
        nxt_tile += gridDim.x;
        advance(nxt_m, nxt_k);
        ++nxt_stage;
    }
    uint32_t stage = 0, buf = 0;
    for (; tile < num_tiles; tile += gridDim.x) {
        issue(nxt_tile, nxt_m, nxt_k, nxt_stage);  // into the stage this thread emptied in the previous iteration
        nxt_tile += gridDim.x;
        advance(nxt_m, nxt_k);
        nxt_stage = nxt_stage == kStages - 1 ? 0 : nxt_stage + 1;
        cp_async_wait<kLosslessDepth>();
        LosslessPieces cur;
        lossless_fetch(p, stages[stage], cur_k, t, c32, cur);
        int* const a = exp_max[buf];
        buf = buf == 2 ? 0 : buf + 1;
        if (cur_m < full_m && cur_k < full_k) lossless_tile<OBM, OBK, true>(p, cur, cur_m, cur_k, a, exp_max[buf], t, c32, r_base);
        else lossless_tile<OBM, OBK, false>(p, cur, cur_m, cur_k, a, exp_max[buf], t, c32, r_base);
        advance(cur_m, cur_k);
        stage = stage == kStages - 1 ? 0 : stage + 1;
    }
    cp_async_wait<0>();
}

// cuTensorMapEncodeTiled through the runtime's driver entry-point lookup (no link against libcuda).
static PFN_cuTensorMapEncodeTiled_v12000 tensor_map_encoder() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
    }();
    return fn;
}

// Describes x as a [num_tokens, hidden] row-major tensor read in 128 x 128 boxes, out-of-range elements as zeros.
static int make_tensor_map(CUtensorMap* tmap, const void* x, int elem_bytes, int64_t num_tokens, int64_t hidden) {
    auto encode = tensor_map_encoder();
    if (encode == nullptr) return set_error(TKQ_E_UNSUPPORTED, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {static_cast<cuuint64_t>(hidden), static_cast<cuuint64_t>(num_tokens)};
    const cuuint64_t strides[1] = {static_cast<cuuint64_t>(hidden) * elem_bytes};
    const cuuint32_t box[2] = {kTile, kTile};
    const cuuint32_t elem_strides[2] = {1, 1};
    const CUresult r = encode(tmap, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2,
                              const_cast<void*>(x), dims, strides, box, elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return set_error(TKQ_E_UNSUPPORTED, "cuTensorMapEncodeTiled rejected the tensor (alignment or size)");
    return 0;
}

// Launch geometry: persistent blocks, two per SM, each with up to three tile buffers (about 100 KB).
template <class Kernel>
static int launch_tile(Kernel kernel, TileParams p, int elem_bytes, const char* what, cudaStream_t stream) {
    const int tile_bytes = kTile * kTile * elem_bytes;
    const int64_t tiles = ((p.num_tokens + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31) || p.num_tokens >= (int64_t{1} << 31))
        return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    alignas(64) CUtensorMap tmap;
    if (int rc = make_tensor_map(&tmap, p.x, elem_bytes, p.num_tokens, p.hidden)) return rc;
    const int sms = device_sm_count();
    const int blocks_per_sm = 2;  // three blocks with two stages each measured no faster
    const int grid = static_cast<int>(tiles < static_cast<int64_t>(sms) * blocks_per_sm ? tiles : static_cast<int64_t>(sms) * blocks_per_sm);
    const int max_stages = (100 * 1024) / tile_bytes;  // 3 bf16 tiles or 1 fp32 tile
    const int64_t tiles_per_block = (tiles + grid - 1) / grid;
    int stages = static_cast<int>(tiles_per_block < max_stages ? tiles_per_block : max_stages);
    if (stages < 1) stages = 1;
    p.num_tiles = static_cast<uint32_t>(tiles);
    p.stages = static_cast<uint32_t>(stages);
    const int smem = stages * tile_bytes;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), 100 * 1024)) return rc;
    kernel<<<grid, kTileThreads, smem, stream>>>(tmap, p);
    return check_launch(what);
}

// Launch of a light tile kernel: one tile buffer per block, as many resident blocks as the SM holds.
template <int DT, class Kernel>
static int launch_tile_light(Kernel kernel, TileParams p, const char* what, cudaStream_t stream) {
    constexpr int elem_bytes = TileElem<DT>::kBytes;
    const int64_t tiles = ((p.num_tokens + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31) || p.num_tokens >= (int64_t{1} << 31))
        return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    alignas(64) CUtensorMap tmap;
    if (int rc = make_tensor_map(&tmap, p.x, elem_bytes, p.num_tokens, p.hidden)) return rc;
    const int smem = TileElem<DT>::kTileBytes;
    if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), smem)) return rc;
    p.num_tiles = static_cast<uint32_t>(tiles);
    p.stages = 1;
    const int grid = grid_size(kernel, kTileThreads, tiles, smem);
    kernel<<<grid, kTileThreads, smem, stream>>>(tmap, p);
    return check_launch(what);
}

// Launch of a direct tile kernel (bf16 tiles held in registers).  Resident blocks per SM were measured on B200 for
// [7168, 2048] ... [32768, 7168]: up to 8 tiles per SM run fastest with every block resident (ramp and drain
// dominate), mid sizes with four blocks per SM, and the largest with three (more tiles in flight than that cost
// DRAM efficiency: 0.86 of the copy bandwidth with five blocks, 0.96 with three on [32768, 7168]).
template <class Kernel>
static int launch_tile_direct(Kernel kernel, TileParams p, int max_blocks_per_sm, const char* what, cudaStream_t stream) {
    const int64_t tiles = ((p.num_tokens + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31) || p.num_tokens >= (int64_t{1} << 31))
        return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    const int sms = device_sm_count();
    int per_sm = std::min(max_blocks_per_sm, cached_occupancy(reinterpret_cast<const void*>(kernel), kTileThreads, 0));
    if (tiles > int64_t{64} * sms) per_sm = std::min(per_sm, 3);
    else if (tiles > int64_t{8} * sms) per_sm = std::min(per_sm, 4);
    p.num_tiles = static_cast<uint32_t>(tiles);
    p.stages = 0;
    const int grid = static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(sms) * per_sm));
    kernel<<<grid, kTileThreads, 0, stream>>>(p, reinterpret_cast<uintptr_t>(p.x) % 32 == 0);
    return check_launch(what);
}

template <int DT, int FMT>
static int dispatch_block(const TileParams& p, int bm, int bk, cudaStream_t s) {
    constexpr int TB = TileElem<DT>::kBytes;
    const char* what = "per_block_cast";
    if (bm == 128 && bk == 128) {
        // bf16 tiles: the direct kernel (registers, no staging).  fp32 tiles (64 KB) go through the TMA ring kernel.
        if constexpr (DT == TKQ_DT_BF16) {
            return launch_tile_direct(per_block_cast_direct_kernel<FMT>, p, 5, what, s);
        } else return launch_tile(per_block_cast_kernel<DT, FMT, 128, 128>, p, TB, what, s);
    }
    if (bm == 32 && bk == 32) return launch_tile(per_block_cast_kernel<DT, FMT, 32, 32>, p, TB, what, s);
    if (bm == 128 && bk == 32) return launch_tile(per_block_cast_kernel<DT, FMT, 128, 32>, p, TB, what, s);
    if (bm == 32 && bk == 128) return launch_tile(per_block_cast_kernel<DT, FMT, 32, 128>, p, TB, what, s);
    return set_error(TKQ_E_UNSUPPORTED, "per_block_cast: block sizes must be 32 or 128");
}

// ---------------------------------------------------------------------------
// Fused per-channel cast: the per-channel cast of rows gathered through `pos_to_token` (a negative entry gives a
// row of zeros) and/or of FP8 input with one fp32 scale per (token, 128 channels), which is multiplied in before
// the maximum is taken (reference: tile_kernels/quant/per_channel_cast_fused_kernel.py:50-132,
// tile_kernels/torch/per_channel_cast_fused.py:9-44).  Gathered rows are not a rectangle, so this kernel reads
// its 128 x 128 tile with plain vector loads, one block per tile; the arithmetic is that of
// per_channel_cast_kernel.
// ---------------------------------------------------------------------------
constexpr int kInFp8 = 2;  // input kind next to TKQ_DT_BF16 / TKQ_DT_FP32

struct FusedChannelParams {
    const void* x;
    const float* x_sf;           // [num_tokens_in, hidden / 128], FP8 input only
    const int32_t* pos_to_token;  // [num_tokens_out] or null
    uint8_t* out;
    float* sf;
    int64_t num_tokens_in, num_tokens_out, hidden;
    uint32_t tiles_k;
    uint32_t flags;
    float clamp_min;
    bool fast_pow2;
    bool wide_loads;
};

template <int IN>
__global__ void __launch_bounds__(kTileThreads, 3) per_channel_cast_fused_kernel(const FusedChannelParams p) {
    __shared__ __align__(16) float warp_max[kTileThreads / 32][kTile];  // column maxima of each warp's 16 rows
    __shared__ __align__(16) float col_inv[kTile];
    using Src = typename std::conditional<IN == kInFp8, QuantSource<TKQ_FMT_E4M3>, PlainSource<IN == kInFp8 ? TKQ_DT_BF16 : IN>>::type;
    const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
    const int c16 = t & 7, r_base = t >> 3;
    const int64_t tile_m = blockIdx.x / p.tiles_k, tile_k = blockIdx.x % p.tiles_k;
    const int64_t row0 = tile_m * kTile, col0 = tile_k * kTile;
    const int valid_rows = static_cast<int>(p.num_tokens_out - row0 < kTile ? p.num_tokens_out - row0 : kTile);
    const int valid_cols = static_cast<int>(p.hidden - col0 < kTile ? p.hidden - col0 : kTile);
    const bool col_ok = c16 * 16 < valid_cols;
    const bool round_sf = p.flags & TKQ_ROUND_SF;

    // The four chunks stay in registers as loaded (8 words per chunk for bf16, 4 for FP8) and are unpacked twice,
    // for the maximum and for the conversion: fewer live registers, more resident blocks to hide the two
    // dependent loads (row index, then row).
    typename Src::Raw raw[4];
    float scale_in[4] = {1.0f, 1.0f, 1.0f, 1.0f};
    int64_t src_rows[4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = r_base + 32 * k;
        src_rows[k] = -1;
        if (col_ok && r < valid_rows) src_rows[k] = p.pos_to_token != nullptr ? p.pos_to_token[row0 + r] : row0 + r;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        Src::zero(raw[k]);
        if (src_rows[k] >= 0) {
            const int64_t elem = src_rows[k] * p.hidden + col0 + c16 * 16;
            Src::issue(raw[k], static_cast<const uint8_t*>(p.x) + Src::bytes(elem), p.wide_loads);
            if constexpr (IN == kInFp8) scale_in[k] = p.x_sf[src_rows[k] * (p.hidden / 128) + (col0 + c16 * 16) / 128];
        }
    }
    auto unpack = [&](int k, float* v) {
        if constexpr (IN == kInFp8) Src::unpack(raw[k], v, scale_in[k]);
        else Src::unpack(raw[k], v);
    };
    float cm[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) cm[j] = 0.0f;
#pragma unroll
    for (int k = 0; k < 4; k += 2) {
        float v0[16], v1[16];
        unpack(k, v0);
        unpack(k + 1, v1);
#pragma unroll
        for (int j = 0; j < 16; ++j) cm[j] = max3_abs(cm[j], v0[j], v1[j]);
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
        cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 8));
        cm[j] = fmaxf(cm[j], __shfl_xor_sync(kFullMask, cm[j], 16));
    }
    if (lane < 8) {
        float4* dst = reinterpret_cast<float4*>(&warp_max[warp][c16 * 16]);
#pragma unroll
        for (int q = 0; q < 4; ++q) dst[q] = make_float4(cm[4 * q], cm[4 * q + 1], cm[4 * q + 2], cm[4 * q + 3]);
    }
    __syncthreads();
    if (t < kTile) {
        float m = warp_max[0][t];
#pragma unroll
        for (int w = 1; w < kTileThreads / 32; ++w) m = fmaxf(m, warp_max[w][t]);
        const Scale s = make_scale_for<TKQ_FMT_E4M3>(m, p.clamp_min, round_sf, p.fast_pow2);
        col_inv[t] = s.inv;
        if (t < valid_cols) p.sf[tile_m * p.hidden + col0 + t] = s.sf;
    }
    __syncthreads();
    float inv[16];
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const float4 a = reinterpret_cast<const float4*>(&col_inv[c16 * 16])[q];
        inv[4 * q] = a.x, inv[4 * q + 1] = a.y, inv[4 * q + 2] = a.z, inv[4 * q + 3] = a.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int r = r_base + 32 * k;
        if (col_ok && r < valid_rows) {
            float v[16], q[16];
            unpack(k, v);
#pragma unroll
            for (int j = 0; j < 16; ++j) q[j] = __fmul_rn(v[j], inv[j]);
            stg128(p.out + (row0 + r) * p.hidden + col0 + c16 * 16, cvt_e4m3x4(q[0], q[1], q[2], q[3]),
                   cvt_e4m3x4(q[4], q[5], q[6], q[7]), cvt_e4m3x4(q[8], q[9], q[10], q[11]),
                   cvt_e4m3x4(q[12], q[13], q[14], q[15]));
        }
    }
}

}  // namespace tkq

using namespace tkq;

// Non-zero if any tile kernel of this process gave up waiting for its staged tile since the
// last call; reading clears the flag.  Synchronises the device.
int tkq::tile_wait_flag() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_tile_wait_failed, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_tile_wait_failed, &zero, sizeof(zero));
    return static_cast<int>(v);
}

static int lossless_violation_flag() {
    unsigned int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_lossless_range_violations, sizeof(v)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_lossless_range_violations, &zero, sizeof(zero));
    return v ? 1 : 0;
}

extern "C" int tkq_device_error(void) {
    const int a = tile_wait_flag(), b = row_wait_flag(), c = swiglu_wait_flag(), d = lossless_violation_flag();
    if (a < 0 || b < 0 || c < 0 || d < 0) return -1;
    return ((a | b | c) ? TKQ_DEVICE_WAIT_TIMEOUT : 0) | (d ? TKQ_DEVICE_LOSSLESS_RANGE : 0);
}

namespace tkq {
// Self-test of the bounded wait: one bulk copy of 16 bytes arrives on the first barrier (waited for with the
// default limit, so nothing is in flight afterwards); nothing ever arrives on the second one, and the wait on it
// gives up after `limit` polls, raises the flag and returns.
__global__ void bounded_wait_probe_kernel(const uint8_t* src, uint32_t limit, uint32_t* echo) {
    __shared__ __align__(16) uint8_t buf[16];
    __shared__ uint64_t bar[2];
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        mbar_init(bar + 1, 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(bar, 16);
        bulk_load(buf, src, 16, bar);
    }
    if (!mbar_wait(bar, 0)) {
        atomicExch(&g_tile_wait_failed, 1u);
        return;
    }
    if (threadIdx.x == 0 && echo != nullptr) *echo = *reinterpret_cast<const uint32_t*>(buf);
    if (!mbar_wait(bar + 1, 0, limit)) {
        atomicExch(&g_tile_wait_failed, 1u);
        return;
    }
}
}  // namespace tkq

extern "C" int tkq_selftest_bounded_wait(const void* src16, unsigned poll_limit, void* echo, void* stream) {
    if (src16 == nullptr || !aligned16(src16) || poll_limit == 0 || poll_limit > (1u << 16))
        return set_error(TKQ_E_BAD_ARG, "selftest_bounded_wait: 16-byte aligned source, poll limit in 1..65536");
    bounded_wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint8_t*>(src16), poll_limit,
                                                                               static_cast<uint32_t*>(echo));
    return check_launch("selftest_bounded_wait");
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
    p.fast_pow2 = (flags & TKQ_ROUND_SF) != 0;
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
    p.fast_pow2 = (flags & TKQ_ROUND_SF) != 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // bf16: the direct kernel, except for the largest shapes, where the staged light kernel (six blocks per SM)
    // measured a little faster (118 against 121 us on [32768, 7168]; 11.6 against 10.4 us on [7168, 2048])
    if (in_dtype == TKQ_DT_BF16 && (num_tokens / kTile) * p.tiles_k <= int64_t{64} * device_sm_count())
        return launch_tile_direct(per_channel_cast_direct_kernel<false>, p, 4, "per_channel_cast", s);
    return in_dtype == TKQ_DT_BF16
               ? launch_tile_light<TKQ_DT_BF16>(per_channel_cast_light_kernel<TKQ_DT_BF16>, p, "per_channel_cast", s)
               : launch_tile(per_channel_cast_kernel<TKQ_DT_FP32>, p, 4, "per_channel_cast", s);
}

extern "C" int tkq_per_channel_cast_fused(const void* x, int in_kind, const float* x_sf, const int32_t* pos_to_token,
                                          int64_t num_tokens_in, int64_t num_tokens_out, int64_t hidden, unsigned flags,
                                          void* out, void* sf, void* stream) {
    if (num_tokens_in < 0 || num_tokens_out < 0 || hidden <= 0 ||
        (in_kind != TKQ_DT_BF16 && in_kind != TKQ_DT_FP32 && in_kind != kInFp8))
        return set_error(TKQ_E_BAD_ARG, "per_channel_cast_fused: bad size or input kind");
    if (num_tokens_out == 0) return 0;
    if (x == nullptr || sf == nullptr || out == nullptr || (in_kind == kInFp8) != (x_sf != nullptr))
        return set_error(TKQ_E_BAD_ARG, "per_channel_cast_fused: null pointer (input scales go with FP8 input, and only with it)");
    if (flags & ~TKQ_ROUND_SF) return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast_fused: only TKQ_ROUND_SF is defined");
    if (hidden % 64 != 0 || (in_kind == kInFp8 && hidden % 128 != 0))
        return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast_fused: hidden % 64 == 0 (128 for FP8 input) required");
    if (num_tokens_out % (pos_to_token != nullptr ? 16 : 128) != 0)
        return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast_fused: output tokens must be a multiple of 128 (16 with pos_to_token)");
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "per_channel_cast_fused: x and out must be 16-byte aligned, sf 4-byte aligned");
    FusedChannelParams p{};
    p.x = x;
    p.x_sf = x_sf;
    p.pos_to_token = pos_to_token;
    p.out = static_cast<uint8_t*>(out);
    p.sf = static_cast<float*>(sf);
    p.num_tokens_in = num_tokens_in;
    p.num_tokens_out = num_tokens_out;
    p.hidden = hidden;
    p.tiles_k = static_cast<uint32_t>((hidden + kTile - 1) / kTile);
    p.flags = flags;
    p.clamp_min = 1e-4f;
    p.fast_pow2 = (flags & TKQ_ROUND_SF) != 0;
    const int elem = in_kind == TKQ_DT_BF16 ? 2 : 4;
    p.wide_loads = in_kind != kInFp8 && reinterpret_cast<uintptr_t>(x) % 32 == 0 && (hidden * elem) % 32 == 0;
    const int64_t tiles = ((num_tokens_out + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31)) return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (in_kind == TKQ_DT_BF16) {
        // bf16 rows, gathered or not: the direct per-channel kernel (packed column maxima), rows through pos_to_token
        TileParams q{};
        q.x = x;
        q.out = p.out;
        q.sf = sf;
        q.num_tokens = num_tokens_out;
        q.hidden = hidden;
        q.sf_stride = hidden;
        q.tiles_k = p.tiles_k;
        q.flags = flags;
        q.clamp_min = p.clamp_min;
        q.fast_pow2 = p.fast_pow2;
        q.pos_to_token = pos_to_token;
        return pos_to_token != nullptr ? launch_tile_direct(per_channel_cast_direct_kernel<true>, q, 4, "per_channel_cast_fused", s)
                                       : launch_tile_direct(per_channel_cast_direct_kernel<false>, q, 4, "per_channel_cast_fused", s);
    }
    const unsigned grid = static_cast<unsigned>(tiles);
    if (in_kind == TKQ_DT_FP32) per_channel_cast_fused_kernel<TKQ_DT_FP32><<<grid, kTileThreads, 0, s>>>(p);
    else per_channel_cast_fused_kernel<kInFp8><<<grid, kTileThreads, 0, s>>>(p);
    return check_launch("per_channel_cast_fused");
}

extern "C" int tkq_per_channel_cast_and_transpose(const void* x, int64_t num_tokens, int64_t hidden, int num_per_tokens,
                                                  unsigned flags, void* out, void* sf, void* stream) {
    if (num_tokens < 0 || hidden <= 0) return set_error(TKQ_E_BAD_ARG, "per_channel_cast_and_transpose: bad size");
    if (num_tokens == 0) return 0;
    if (x == nullptr || sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "per_channel_cast_and_transpose: null pointer");
    if (flags & ~TKQ_ROUND_SF) return set_error(TKQ_E_UNSUPPORTED, "per_channel_cast_and_transpose: only TKQ_ROUND_SF is defined");
    if (num_tokens % 128 != 0 || hidden % 64 != 0 || (num_per_tokens != 32 && num_per_tokens != 128))
        return set_error(TKQ_E_UNSUPPORTED,
                         "per_channel_cast_and_transpose: num_tokens % 128 == 0, hidden % 64 == 0, num_per_tokens 32 or 128 required");
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "per_channel_cast_and_transpose: x and out must be 16-byte aligned, sf 4-byte aligned");
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
    p.fast_pow2 = (flags & TKQ_ROUND_SF) != 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const char* what = "per_channel_cast_and_transpose";
    return num_per_tokens == 128 ? launch_tile(per_channel_cast_transpose_kernel<128>, p, 2, what, s)
                                 : launch_tile(per_channel_cast_transpose_kernel<32>, p, 2, what, s);
}

extern "C" int tkq_swiglu_forward_and_per_channel_cast(const void* x, int64_t num_tokens, int64_t hidden, int num_per_tokens,
                                                       int transpose, float swiglu_clamp, unsigned flags, void* out, void* sf,
                                                       void* stream) {
    if (num_tokens < 0 || hidden <= 0) return set_error(TKQ_E_BAD_ARG, "swiglu per-channel cast: bad size");
    if (num_tokens == 0) return 0;
    if (x == nullptr || sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "swiglu per-channel cast: null pointer");
    if (flags & ~TKQ_ROUND_SF) return set_error(TKQ_E_UNSUPPORTED, "swiglu per-channel cast: only TKQ_ROUND_SF is defined");
    if (num_tokens % 128 != 0 || hidden % 64 != 0 || (num_per_tokens != 32 && num_per_tokens != 128))
        return set_error(TKQ_E_UNSUPPORTED, "swiglu per-channel cast: num_tokens % 128 == 0, hidden % 64 == 0, num_per_tokens 32 or 128 required");
    if (!aligned16(x) || !aligned16(out) || (reinterpret_cast<uintptr_t>(sf) & 3u))
        return set_error(TKQ_E_ALIGNMENT, "swiglu per-channel cast: x and out must be 16-byte aligned, sf 4-byte aligned");
    SwigluChannelParams p{};
    p.x = x;
    p.out = static_cast<uint8_t*>(out);
    p.sf = static_cast<float*>(sf);
    p.num_tokens = num_tokens;
    p.hidden = hidden;
    p.tiles_k = static_cast<uint32_t>((hidden + kTile - 1) / kTile);
    p.flags = flags;
    p.clamp_min = 1e-4f;
    p.swiglu_clamp = swiglu_clamp;
    p.fast_pow2 = (flags & TKQ_ROUND_SF) != 0;
    uint32_t clamp_bits;
    std::memcpy(&clamp_bits, &swiglu_clamp, 4);
    p.bf16_gates = swiglu_clamp < 0.0f || (clamp_bits & 0xFFFFu) == 0;
    p.wide_loads = reinterpret_cast<uintptr_t>(x) % 32 == 0 && (hidden * 2) % 32 == 0;
    const int64_t tiles = (num_tokens / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31)) return set_error(TKQ_E_UNSUPPORTED, "too many tiles; split the token dimension");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const unsigned grid = static_cast<unsigned>(tiles);
    if (num_per_tokens == 128) {
        if (transpose) swiglu_per_channel_cast_kernel<128, true><<<grid, kTileThreads, 0, s>>>(p);
        else swiglu_per_channel_cast_kernel<128, false><<<grid, kTileThreads, 0, s>>>(p);
    } else {
        if (transpose) swiglu_per_channel_cast_kernel<32, true><<<grid, kTileThreads, 0, s>>>(p);
        else swiglu_per_channel_cast_kernel<32, false><<<grid, kTileThreads, 0, s>>>(p);
    }
    return check_launch("swiglu_forward_and_per_channel_cast_and_transpose");
}

extern "C" int tkq_per_block_cast_lossless(const void* x, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride, int x_block_m,
                                           int x_block_k, int64_t num_tokens, int64_t hidden, int64_t x_row_stride, int out_block_m,
                                           int out_block_k, unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream) {
    if (num_tokens < 0 || hidden <= 0 || x_row_stride < hidden || x_block_m <= 0 || x_block_k <= 0)
        return set_error(TKQ_E_BAD_ARG, "per_block_cast_lossless: bad size");
    if (num_tokens == 0) return 0;
    if (x == nullptr || x_sf == nullptr || sf == nullptr || out == nullptr) return set_error(TKQ_E_BAD_ARG, "per_block_cast_lossless: null pointer");
    if (((flags & TKQ_SF_UE8M0) && !(flags & TKQ_SF_COL_MAJOR)) || ((x_sf_flags & TKQ_SF_UE8M0) && !(x_sf_flags & TKQ_SF_COL_MAJOR)))
        return set_error(TKQ_E_UNSUPPORTED, "packed ue8m0 scales need the column-major layout");
    const bool bm_ok = out_block_m == 1 || out_block_m == 32 || out_block_m == 128;
    const bool bk_ok = out_block_k == 32 || out_block_k == 128;
    if (!bm_ok || !bk_ok || out_block_m % x_block_m != 0 || out_block_k % x_block_k != 0 || x_block_k % 16 != 0 || hidden % 32 != 0)
        return set_error(TKQ_E_UNSUPPORTED,
                         "per_block_cast_lossless: output blocks (1|32|128) x (32|128), multiples of the input block; hidden % 32 == 0");
    if (!aligned16(x) || (x_row_stride / 2) % 16 != 0 || !aligned16(out) ||
        (reinterpret_cast<uintptr_t>(sf) & 3u) || (reinterpret_cast<uintptr_t>(x_sf) & 3u) || ((flags & TKQ_SF_UE8M0) && (sf_stride & 3)) ||
        ((x_sf_flags & TKQ_SF_UE8M0) && (x_sf_stride & 3)))
        return set_error(TKQ_E_ALIGNMENT, "per_block_cast_lossless: x rows and out 16-byte aligned, scales 4-byte aligned");
    LosslessParams p{};
    p.in.x = x;
    p.in.out = static_cast<uint8_t*>(out);
    p.in.x_stride = x_row_stride;
    p.in.num_tokens = num_tokens;
    p.in.hidden = hidden;
    p.in.in_sf = x_sf;
    p.in.in_sf_stride = x_sf_stride;
    p.in.in_sf_flags = x_sf_flags;
    p.in.in_block_m = static_cast<uint32_t>(x_block_m);
    p.in.in_block_k = static_cast<uint32_t>(x_block_k);
    set_input_block_shifts(p.in);
    p.sf = sf;
    p.sf_stride = sf_stride;
    p.tiles_k = static_cast<uint32_t>((hidden + kLosslessCols - 1) / kLosslessCols);
    p.flags = flags;
    p.wide_stores = reinterpret_cast<uintptr_t>(out) % 32 == 0;
    const int64_t tiles = ((num_tokens + kTile - 1) / kTile) * p.tiles_k;
    if (tiles >= (int64_t{1} << 31) || num_tokens >= (int64_t{1} << 31) || x_row_stride >= (int64_t{1} << 24))
        return set_error(TKQ_E_UNSUPPORTED, "per_block_cast_lossless: more than 2^31 tokens or tiles, or rows of more than 2^24 values");
    const int sms = device_sm_count();
    const cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint32_t n = static_cast<uint32_t>(tiles);
    auto launch = [&](auto kernel) -> int {
        constexpr int kSmem = (kLosslessDepth + 1) * static_cast<int>(sizeof(LosslessStage));
        if (int rc = ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kSmem)) return rc;
        const int per_sm = std::min(kLosslessBlocksPerSm, cached_occupancy(reinterpret_cast<const void*>(kernel), kTileThreads, kSmem));
        const int grid = static_cast<int>(std::min<int64_t>(tiles, static_cast<int64_t>(sms) * std::max(per_sm, 1)));
        kernel<<<grid, kTileThreads, kSmem, st>>>(p, n);
        return 0;
    };
    int rc = 0;
    if (out_block_k == 128) {
        if (out_block_m == 128) rc = launch(per_block_cast_lossless_kernel<128, 128>);
        else if (out_block_m == 32) rc = launch(per_block_cast_lossless_kernel<32, 128>);
        else rc = launch(per_block_cast_lossless_kernel<1, 128>);
    } else {
        if (out_block_m == 128) rc = launch(per_block_cast_lossless_kernel<128, 32>);
        else if (out_block_m == 32) rc = launch(per_block_cast_lossless_kernel<32, 32>);
        else rc = launch(per_block_cast_lossless_kernel<1, 32>);
    }
    if (rc) return rc;
    return check_launch("per_block_cast_lossless");
}
