/*
 * tkquant.h -- C ABI of libtkquant.so: B200 (sm_100a) quantization casts.
 *
 * Every entry point takes plain device pointers and sizes, enqueues exactly one
 * kernel on `stream` (a cudaStream_t passed as void*; NULL = the legacy default
 * stream) and returns without synchronising.  Nothing here allocates, frees or
 * keeps a pointer after the launch.
 *
 * Return value: 0 on success; a positive cudaError_t if the launch failed; a
 * negative TKQ_E_* code when the arguments describe a case the library does not
 * implement (nothing was launched).  tkq_last_error_string() explains the last
 * non-zero return of the calling thread.
 *
 * Each function names the interface of the reference project (deepseek-ai
 * TileKernels; paths relative to that project) whose kernel launch it replaces.
 *
 * Scale-factor ("SF") storage, shared by all entry points
 * (reference: tile_kernels/quant/common.py:130-165 get_sf_shape/alloc_scaling_factors,
 *  :219-244 load_sf/store_sf):
 *   row-major fp32        sf[m * sf_stride + k]                      (float)
 *   TKQ_SF_COL_MAJOR      sf[k * sf_stride + m]                      (float)
 *   + TKQ_SF_UE8M0        sf[(k / 4) * sf_stride + 4 * m + k % 4]    (uint8 exponent bytes)
 * with m = token-block index, k = channel-block index and sf_stride in elements
 * of the stated type.  In packed mode the library also zeroes the bytes of a
 * 4-group word that lie beyond the last channel block.
 */
#ifndef TKQUANT_H_
#define TKQUANT_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types of `x` */
#define TKQ_DT_BF16 0
#define TKQ_DT_FP32 1

/* output formats */
#define TKQ_FMT_E4M3 0 /* 1 byte per element (float8_e4m3fn) */
#define TKQ_FMT_E2M1 1 /* 2 elements per byte, even index in the low nibble */
#define TKQ_FMT_E5M6 2 /* 8 elements in 3 little-endian uint32 words */

/* flag bits */
#define TKQ_ROUND_SF 1u     /* round the scale up to a power of two */
#define TKQ_SF_COL_MAJOR 2u /* column-major scale storage */
#define TKQ_SF_UE8M0 4u     /* exponent bytes, four per 32-bit word; needs TKQ_SF_COL_MAJOR */
#define TKQ_SF_ONLY 8u      /* compute and store scales only; `out` is not touched */
#define TKQ_CAST_ONLY 16u   /* read row-major fp32 scales from `sf`, store data only */
#define TKQ_EXACT_CODES 32u /* fused SwiGLU cast only: evaluate every activation with the exact routine (see there) */

/* negative return codes */
#define TKQ_E_BAD_ARG (-1)     /* null pointer, negative size, unknown enum */
#define TKQ_E_UNSUPPORTED (-2) /* shape/flag combination not implemented */
#define TKQ_E_ALIGNMENT (-3)   /* pointer or stride not aligned as documented */

/* Library version, major * 10000 + minor * 100 + patch. */
int tkq_version(void);

/* Text for the calling thread's last non-zero return value (never NULL). */
const char* tkq_last_error_string(void);

/*
 * Device-side conditions, reported without trapping.  This call synchronises the current device, returns the OR of
 * the bits below for what was raised on it since the last call (and clears them), 0 if nothing was, -1 if the
 * flags could not be read.  No counterpart in the reference.
 *
 *   TKQ_DEVICE_WAIT_TIMEOUT   a kernel that waits for asynchronous copies into shared memory (the per-block and
 *                             per-channel tile kernels, the E5M6 row pipeline, the staged SwiGLU cast) ran out of
 *                             polls (a limit that is seconds long), and returned early.  Outputs of that launch
 *                             are undefined: rows or tiles may be missing or partly written.
 *   TKQ_DEVICE_LOSSLESS_RANGE tkq_per_block_cast_lossless met an input scale more than 2^5 below its output
 *                             block's scale, where the reference's kernel asserts
 *                             (tile_kernels/quant/per_block_cast_lossless_kernel.py:128); those values were rounded
 *                             to nearest instead of being represented exactly.
 */
#define TKQ_DEVICE_WAIT_TIMEOUT 1
#define TKQ_DEVICE_LOSSLESS_RANGE 2
int tkq_device_error(void);

/*
 * Self-test of the bounded wait: launches one warp that receives 16 bytes from `src16` by bulk copy, writes the
 * first word to `echo` (optional), then waits `poll_limit` polls (1..65536) on a barrier nothing ever arrives on,
 * gives up, raises TKQ_DEVICE_WAIT_TIMEOUT and returns.  No copy is in flight when it returns and nothing faults
 * or hangs; tkq_device_error() afterwards reads 1, then 0.  No counterpart in the reference.
 */
int tkq_selftest_bounded_wait(const void* src16, unsigned poll_limit, void* echo, void* stream);

/*
 * Per-token cast to FP8 e4m3 or FP4 e2m1: one scale per (1 x num_per_channels) group.
 * Replaces the launch in tile_kernels/quant/per_token_cast_kernel.py:208-209
 * (kernel body :72-154; per_token_cast / _with_sf_only / _with_precomputed_sf, :223-302).
 *
 *   x             [num_tokens, hidden] bf16 or fp32, row stride x_row_stride elements, unit column stride
 *   num_per_channels  16, 32, 64, 128, or == hidden (one scale per token; hidden % 64 == 0)
 *   out           e4m3: [num_tokens, hidden] bytes; e2m1: [num_tokens, hidden / 2] bytes; contiguous
 *   sf            scale storage as described above (m = token, k = group); read with TKQ_CAST_ONLY
 * Alignment: x, out 16-byte aligned, hidden and x_row_stride multiples of 16 elements.
 */
int tkq_per_token_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, int64_t x_row_stride, int fmt,
                       int64_t num_per_channels, unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream);

/*
 * Per-token cast of an ALREADY QUANTIZED input: x holds FP8 e4m3 bytes or packed FP4 e2m1 nibbles with one
 * scale per (x_block_m x x_block_k) block; every value is float(x) * scale (an fp32 product), then cast as in
 * tkq_per_token_cast.  Replaces the same launch, tile_kernels/quant/per_token_cast_kernel.py:208-209, for the
 * `with_sf` input configuration (kernel body :87-126; input detection tile_kernels/quant/common.py:62-88).
 * The data are scaled as (x * scale_in) * inverse_out, the order of the reference's PyTorch implementation
 * (tile_kernels/torch/cast.py:93-97,174-176); the reference kernel folds the two factors first, which is the
 * same thing for power-of-two scales, the only case its tests use.
 *
 *   x             in_fmt e4m3: [num_tokens, hidden] bytes; e2m1: [num_tokens, hidden / 2] bytes;
 *                 x_row_stride in VALUES (twice the byte stride for e2m1)
 *   x_sf          input scales, m = token / x_block_m, k = channel / x_block_k, in the layout given by
 *                 x_sf_flags (0 = row-major fp32, TKQ_SF_COL_MAJOR, TKQ_SF_COL_MAJOR | TKQ_SF_UE8M0) with
 *                 x_sf_stride as sf_stride above
 *   num_per_channels  16, 32, 64 or 128; x_block_k a multiple of 16
 */
int tkq_per_token_cast_quantized(const void* x, int in_fmt, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride,
                                 int x_block_m, int x_block_k, int64_t num_tokens, int64_t hidden, int64_t x_row_stride,
                                 int fmt, int64_t num_per_channels, unsigned flags, void* out, void* sf, int64_t sf_stride,
                                 void* stream);

/*
 * Per-token cast to E5M6 (12-bit codes, one scale per token, maximum 65024, clamp 1e-4).
 * Replaces the launch in tile_kernels/quant/per_token_cast_to_e5m6_kernel.py:209-210
 * (kernel :108-154, float_to_e5m6 :33-64).
 *
 *   x      [num_tokens, hidden] bf16 or fp32, hidden % 8 == 0
 *   out    [num_tokens, hidden / 8 * 3] uint32 words, contiguous
 *   sf     one scale per token: k = 0 in the formulas above
 */
int tkq_per_token_cast_e5m6(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, int64_t x_row_stride,
                            unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream);

/*
 * Per-block cast: one scale per (block_m x block_k) tile, block sizes 32 or 128.
 * Replaces the launch in tile_kernels/quant/per_block_cast_kernel.py:191-192
 * (kernel :97-136; per_block_cast / _with_sf_only / _with_precomputed_sf, :205-276).
 *
 *   x      [num_tokens, hidden] bf16 or fp32, contiguous, hidden % 64 == 0
 *   out    e4m3 [num_tokens, hidden] or e2m1 [num_tokens, hidden / 2] bytes
 *   sf     m = token-block, k = channel-block
 */
int tkq_per_block_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, int fmt, int block_m,
                       int block_k, unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream);

/*
 * Per-channel cast to e4m3: one scale per (128 tokens x 1 channel).
 * Replaces the launch in tile_kernels/quant/per_channel_cast_fused_kernel.py:200-201
 * (kernel :50-132) for the plain-input case reached through
 * tile_kernels/quant/per_channel_cast_kernel.py:8-28.
 *
 *   x      [num_tokens, hidden] bf16 or fp32, contiguous, num_tokens % 128 == 0, hidden % 64 == 0
 *   out    [num_tokens, hidden] bytes
 *   sf     [num_tokens / 128, hidden] fp32 row-major, contiguous
 * flags: TKQ_ROUND_SF only.
 */
int tkq_per_channel_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden, unsigned flags, void* out,
                         void* sf, void* stream);

/*
 * Fused per-channel cast to e4m3: the per-channel cast (one scale per 128 output tokens x 1 channel) of
 *   - rows gathered through pos_to_token (out row i = x row pos_to_token[i]; a negative entry = a row of zeros), and/or
 *   - FP8 e4m3 input with one fp32 scale per (token, 128 channels): every value is float(x) * scale before the
 *     maximum is taken and the data are written as (x * scale) * inverse.
 * Replaces the launch in tile_kernels/quant/per_channel_cast_fused_kernel.py:200-201 (kernel :50-132) for the
 * cases tkq_per_channel_cast does not cover.
 *
 *   in_kind        TKQ_DT_BF16, TKQ_DT_FP32, or 2 = FP8 e4m3 bytes (then x_sf is required, hidden % 128 == 0)
 *   x              [num_tokens_in, hidden], contiguous
 *   x_sf           [num_tokens_in, hidden / 128] fp32, contiguous (FP8 input only, else NULL)
 *   pos_to_token   int32[num_tokens_out] or NULL (then num_tokens_out == num_tokens_in, a multiple of 128);
 *                  with it num_tokens_out must be a multiple of 16
 *   out            [num_tokens_out, hidden] bytes;  sf  [ceil(num_tokens_out / 128), hidden] fp32
 * flags: TKQ_ROUND_SF only.
 */
int tkq_per_channel_cast_fused(const void* x, int in_kind, const float* x_sf, const int32_t* pos_to_token,
                               int64_t num_tokens_in, int64_t num_tokens_out, int64_t hidden, unsigned flags, void* out,
                               void* sf, void* stream);

/*
 * Fused SwiGLU + per-channel e4m3 cast, optionally transposed: y = silu(x[:, :hidden]) * x[:, hidden:] in fp32
 * (optionally clamped as in tkq_swiglu_forward_and_per_token_cast), ROUNDED TO BF16, then one scale per
 * (num_per_tokens tokens x 1 channel), num_per_tokens = 32 or 128.
 * Replaces the launch in tile_kernels/quant/swiglu_forward_and_per_channel_cast_and_transpose_kernel.py:226-227.
 *
 *   x          [num_tokens, 2 * hidden] bf16, contiguous, num_tokens % 128 == 0, hidden % 64 == 0
 *   transpose  non-zero: out is [hidden, num_tokens]; zero: [num_tokens, hidden]
 *   sf         [num_tokens / num_per_tokens, hidden] fp32
 * flags: TKQ_ROUND_SF only.
 */
int tkq_swiglu_forward_and_per_channel_cast(const void* x, int64_t num_tokens, int64_t hidden, int num_per_tokens, int transpose,
                                            float swiglu_clamp, unsigned flags, void* out, void* sf, void* stream);

/*
 * Lossless FP4 -> FP8 re-blocking: packed e2m1 input with power-of-two scales per (x_block_m x x_block_k) block
 * becomes e4m3 with power-of-two scales per (out_block_m x out_block_k) block.  Output exponent of a block =
 * (largest input exponent inside it) - 6, not below 0; value = fp4 * 2^(e_in - e_out).
 * Replaces the launch in tile_kernels/quant/per_block_cast_lossless_kernel.py:201-202 (kernel :76-150).  The
 * reference asserts e_in + 5 >= e_out on the device (exact representability); this library rounds to nearest
 * where that does not hold and raises TKQ_DEVICE_LOSSLESS_RANGE (see tkq_device_error).
 *
 *   x          [num_tokens, hidden / 2] bytes, x_row_stride in VALUES; x_sf as in tkq_per_token_cast_quantized.
 *              x and every row of it 16-byte aligned (x_row_stride % 32 == 0); fewer than 2^24 values per row
 *   out blocks (1 | 32 | 128) x (32 | 128), multiples of the input block; hidden % 32 == 0
 *   flags      TKQ_SF_COL_MAJOR, TKQ_SF_UE8M0 for the output scales (always powers of two)
 */
int tkq_per_block_cast_lossless(const void* x, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride, int x_block_m,
                                int x_block_k, int64_t num_tokens, int64_t hidden, int64_t x_row_stride, int out_block_m,
                                int out_block_k, unsigned flags, void* out, void* sf, int64_t sf_stride, void* stream);

/*
 * Dequantise: out = float(x) * scale of the value's block, formed in fp32 and rounded once to bf16 or fp32.
 * Replaces the launches in tile_kernels/quant/cast_back_kernel.py:118-119 (cast_back, per_token_cast_back;
 * kernel :51-72) and tile_kernels/quant/cast_back_e5m6_kernel.py (cast_back_e5m6).
 *
 *   x          in_fmt e4m3: [num_tokens, hidden] bytes; e2m1: [num_tokens, hidden / 2] bytes;
 *              e5m6: [num_tokens, hidden / 8 * 3] uint32 words; contiguous
 *   x_sf       scales, m = token / x_block_m, k = channel / x_block_k, layout given by x_sf_flags
 *              (0 = row-major fp32, TKQ_SF_COL_MAJOR, TKQ_SF_COL_MAJOR | TKQ_SF_UE8M0), x_sf_stride as sf_stride above
 *   out_dtype  TKQ_DT_BF16 or TKQ_DT_FP32;  out  [num_tokens, hidden], contiguous
 * hidden and x_block_k must be multiples of 16.
 */
int tkq_cast_back(const void* x, int in_fmt, const void* x_sf, unsigned x_sf_flags, int64_t x_sf_stride, int x_block_m,
                  int x_block_k, int64_t num_tokens, int64_t hidden, int out_dtype, void* out, void* stream);

/*
 * Per-channel cast to e4m3 with transposed output: one scale per (num_per_tokens tokens x 1 channel),
 * num_per_tokens = 32 or 128; data written as [hidden, num_tokens].
 * Replaces the launch in tile_kernels/quant/per_channel_cast_and_transpose_kernel.py:120-121 (kernel :30-82).
 *
 *   x      [num_tokens, hidden] bf16, contiguous, num_tokens % 128 == 0, hidden % 64 == 0
 *   out    [hidden, num_tokens] bytes;  sf  [num_tokens / num_per_tokens, hidden] fp32
 * flags: TKQ_ROUND_SF only.
 */
int tkq_per_channel_cast_and_transpose(const void* x, int64_t num_tokens, int64_t hidden, int num_per_tokens, unsigned flags,
                                       void* out, void* sf, void* stream);

/*
 * Fused SwiGLU + per-token e4m3 cast: y = silu(x[:, :hidden]) * x[:, hidden:] in fp32
 * (times an optional per-row weight), then the per-token cast of y.
 * Replaces the launch in tile_kernels/quant/swiglu_forward_and_per_token_cast_kernel.py:255-256
 * (kernel :61-170).
 *
 *   x                  [num_tokens, 2 * hidden] bf16 or fp32, contiguous, hidden % 128 == 0
 *   num_per_channels   128 or hidden
 *   pos_to_token_topk  optional int32[num_tokens]; with topk_weights (fp32, flat) gives the row
 *                      weight topk_weights[pos]; a negative position leaves the weight undefined
 *                      in the reference -- here it is 0
 *   pos_to_expert      optional int32[num_tokens]; rows with a negative entry are skipped
 *                      (neither out nor sf is written for them)
 *   swiglu_clamp       < 0: no clamp; else gate = min(gate, c), up = clamp(up, -c, c)
 *   clamped_count      optional int64[3], atomically incremented by the numbers of
 *                      gate > c, up > c, up < -c (needs swiglu_clamp >= 0)
 *   sf_clamp_min       < 0: the format default 1e-4; else the lower clamp of the group maximum
 *   num_sms            > 0 limits the grid of the counting variant to the blocks that fit num_sms SMs
 *                      (tile_kernels/config.py:13-23); 0 = all SMs
 *   out                [num_tokens, hidden] bytes
 *
 * Arithmetic.  Scales (and clamp counters) are those of an evaluation of y with IEEE operations and a
 * reproducible exp (the routine the CPU checker shares), bit for bit, whatever kernel serves the call.  The FP8
 * codes: for bf16 input, groups of 128, hidden >= 1024 and sf_clamp_min >= 1e-30 the library uses a kernel that
 * evaluates y with the hardware's approximate exp2 and reciprocal (exact only around each group's maximum); a code
 * then differs from the exactly evaluated one only where the scaled activation lies within about 2^-18 of a rounding
 * boundary -- about one code in a million, by one step.  TKQ_EXACT_CODES in `flags` selects the exact evaluation of
 * every activation (at about two thirds of the speed); every other shape takes it anyway.
 */
int tkq_swiglu_forward_and_per_token_cast(const void* x, int in_dtype, int64_t num_tokens, int64_t hidden,
                                          int64_t num_per_channels, const int32_t* pos_to_token_topk,
                                          const float* topk_weights, const int32_t* pos_to_expert, float swiglu_clamp,
                                          long long* clamped_count, float sf_clamp_min, int num_sms, unsigned flags,
                                          void* out, void* sf, int64_t sf_stride, void* stream);

/*
 * SwiGLU backward fused with the per-token e4m3 cast of the input gradient.
 * Replaces the launch in tile_kernels/quant/swiglu_backward_and_per_token_cast_kernel.py:235-236
 * (kernel :34-152).  With g = x[:, :hidden] * x_sf, u = x[:, hidden:] * x_sf, d = grad_out, w = the row's
 * routing weight (0 for a negative position), t = 1 + exp(-g), a = g / t * u, s = 1 / t, q = d * w * s:
 *   out = a * w;   x_grad = [q * u * fma(g, 1 - s, 1),  q * g]  (0 where the forward clamp was active);
 *   weight_grad[pos_to_token_topk[row]] = sum(d * a);  weight_grad[e] = 0 where token_topk_to_pos[e] == -1.
 *
 *   x                  [num_expand_tokens, 2 * hidden] e4m3, contiguous, hidden % num_per_channels == 0
 *   x_sf               [num_expand_tokens, 2 * hidden / num_per_channels] fp32, contiguous
 *   grad_out           [num_expand_tokens, hidden] bf16, contiguous
 *   weight             [num_tokens, num_topk] fp32, contiguous
 *   pos_to_token_topk  int32[num_expand_tokens], flat (token * num_topk + k) index or negative
 *   token_topk_to_pos  int32[num_tokens, num_topk], row of x or -1
 *   num_per_channels   32 or 128
 *   swiglu_clamp       < 0: no clamp; else g = min(g, c), u = clamp(u, -c, c)
 *   flags              TKQ_ROUND_SF only
 *   out                [num_expand_tokens, hidden] bf16
 *   x_grad_fp8         [num_expand_tokens, 2 * hidden] e4m3;  x_grad_sf  fp32, the shape of x_sf
 *   x_grad             [num_expand_tokens, 2 * hidden] bf16
 *   weight_grad        [num_tokens, num_topk] fp32
 * num_expand_tokens == 0 launches nothing (weight_grad is left untouched, as in the reference).
 */
int tkq_swiglu_backward_and_per_token_cast(const void* x, const float* x_sf, const void* grad_out, const float* weight,
                                           const int32_t* pos_to_token_topk, const int32_t* token_topk_to_pos,
                                           int64_t num_expand_tokens, int64_t hidden, int64_t num_tokens, int64_t num_topk,
                                           int64_t num_per_channels, float swiglu_clamp, unsigned flags, void* out,
                                           void* x_grad_fp8, float* x_grad_sf, void* x_grad, float* weight_grad,
                                           void* stream);

/*
 * Expansion of token rows (and their scale factors) into the fused expert layout: out[pos] = x[t] for every
 * pos = token_topk_to_pos[t, k] >= 0; rows with pos_to_expert[pos] < 0 are zero-filled; other rows are left alone.
 * Replaces the launches in tile_kernels/moe/expand_to_fused_kernel.py:127-128 (expand_to_fused, x_sf = NULL) and
 * :196-197 (expand_to_fused_with_sf); kernel :44-92.
 *
 *   x                  [num_tokens, row_bytes] bytes, contiguous (any element type), row_bytes % 16 == 0
 *   x_sf, sf_words     optional [num_tokens, sf_words] 4-byte words (fp32 scales or packed ue8m0), contiguous;
 *                      NULL and 0 for a plain expansion
 *   token_topk_to_pos  int32[num_tokens, num_topk], expanded position or negative
 *   pos_to_expert      int32[num_expanded_tokens], negative = padding row
 *   flags              TKQ_SF_COL_MAJOR: out_sf is [sf_words, out_sf_stride] with one column per expanded row
 *                      (the TMA-aligned layout, out_sf_stride = align(num_expanded_tokens, 4));
 *                      else [num_expanded_tokens, out_sf_stride] row-major
 *   out                [num_expanded_tokens, row_bytes]
 * num_tokens == 0 launches nothing (padding rows are not cleared either, as in the reference).
 */
int tkq_expand_to_fused(const void* x, int64_t num_tokens, int64_t row_bytes, const void* x_sf, int64_t sf_words,
                        const int32_t* token_topk_to_pos, int64_t num_topk, const int32_t* pos_to_expert,
                        int64_t num_expanded_tokens, unsigned flags, void* out, void* out_sf, int64_t out_sf_stride,
                        void* stream);

#ifdef __cplusplus
}
#endif
#endif /* TKQUANT_H_ */
