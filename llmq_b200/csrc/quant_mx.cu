// Block-scaled (MX) quantisation of bf16 matrices for gemm_mx_tcgen05.cu: e4m3 values with one UE8M0 scale
// (a power of two, byte = exponent + 127) per 32 consecutive elements of the contraction axis.
//
// The scale of a block is the smallest power of two s with absmax / s <= 448, so nothing saturates and the block
// uses the top binade of e4m3.  Two forms per source matrix X[R, C] (row-major):
//   along rows    (transpose = 0): blocks run along C;  q[R, C],  operand rows = R, K = C
//   along columns (transpose = 1): blocks run along R;  q[C, R] (the transposed matrix), operand rows = C, K = R
// so both contraction axes of a linear layer (forward / input gradient vs weight gradient) get a K-major operand.
// Scales are written in the tiled layout the GEMM copies to tensor memory:
//   [K / 128][ceil(rows / tile_rows)][ceil(tile_rows / 128)][512],  byte (r % 32) * 16 + (r % 128 / 32) * 4 + block
// with tile_rows = 128 for the A operand and 224 for the B operand.  Padding bytes are zero (2^-127, never NaN).
#include "api.h"
#include "common.cuh"

namespace {

struct SfLayout {
    int tile_rows, chunks;
    long long n_tiles;
    __host__ __device__ long long offset(long long row, long long kblock) const {
        const long long tile = row / tile_rows;
        const int rt = static_cast<int>(row - tile * tile_rows);
        const int r = rt & 127;
        return (((kblock >> 2) * n_tiles + tile) * chunks + (rt >> 7)) * 512 + (r & 31) * 16 + (r >> 5) * 4 + (kblock & 3);
    }
    __host__ __device__ long long bytes(long long K) const { return (K / 128) * n_tiles * chunks * 512; }
};

SfLayout make_layout(long long rows, int tile_rows) {
    SfLayout l;
    l.tile_rows = tile_rows; l.chunks = (tile_rows + 127) / 128; l.n_tiles = (rows + tile_rows - 1) / tile_rows;
    return l;
}

// byte of the smallest power of two >= absmax / 448, and the reciprocal of that power as a float
__device__ __forceinline__ uint32_t mx_scale(float amax, float& inv) {
    uint32_t e = 0;
    if (amax > 0.f) {
        const uint32_t b = __float_as_uint(__fdiv_rn(amax, 448.f));      // exact at powers of two
        e = (b >> 23) + ((b & 0x7FFFFFu) ? 1u : 0u);
        e = e > 253u ? 253u : e;
    }
    inv = __uint_as_float((254u - e) << 23);
    return e;
}

__device__ __forceinline__ void quantise32(const float (&v)[32], float inv, uint4& lo, uint4& hi) {
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
        w[j] = pack_e4m3x2(v[4 * j] * inv, v[4 * j + 1] * inv) | (pack_e4m3x2(v[4 * j + 2] * inv, v[4 * j + 3] * inv) << 16);
    lo = make_uint4(w[0], w[1], w[2], w[3]);
    hi = make_uint4(w[4], w[5], w[6], w[7]);
}

// One thread per 32-element block; the four blocks of a K stage sit in neighbouring lanes and leave as one word.
__global__ void __launch_bounds__(256)
quantize_mx_rows_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const bf16* __restrict__ x, long long R, long long C, long long ld,
                        SfLayout lay) {
    const long long kblocks = C / 32;
    const long long total = R * kblocks;
    const long long idx = blockIdx.x * 256LL + threadIdx.x;
    const bool active = idx < total;
    const long long row = active ? idx / kblocks : 0, kb = active ? idx - row * kblocks : 0;
    float v[32];
    float amax = 0.f;
    if (active) {
        const uint4* src = reinterpret_cast<const uint4*>(x + row * ld + kb * 32);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 raw = __ldcs(src + g);
            const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(h[j]);
                v[g * 8 + 2 * j] = f.x; v[g * 8 + 2 * j + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
    }
    float inv;
    uint32_t e = mx_scale(amax, inv);
    if (active) {
        uint4 lo, hi;
        quantise32(v, inv, lo, hi);
        uint4* dst = reinterpret_cast<uint4*>(q + row * C + kb * 32);
        dst[0] = lo; dst[1] = hi;
    }
    // kblocks is a multiple of 4, so lanes 4i .. 4i+3 hold the four blocks of one (row, stage)
    const uint32_t lane = threadIdx.x & 31u;
    uint32_t word = e << (8 * (lane & 3u));
    word |= __shfl_xor_sync(0xffffffffu, word, 1);
    word |= __shfl_xor_sync(0xffffffffu, word, 2);
    if (active && (lane & 3u) == 0) *reinterpret_cast<uint32_t*>(sf + lay.offset(row, kb)) = word;
}

// Tile of 128 source rows (one K stage) x 128 source columns through shared memory; thread (column pair, block) quantises
// 32 values of two neighbouring source columns and writes 32 contiguous bytes of two rows of the transposed output.
constexpr int TC = 128, TR = 128, TPAD = 8;

// 32 source rows [kb * 32, kb * 32 + 32) of the column pair `cp` of the tile -> e4m3 blocks + scale bytes
__device__ __forceinline__ void quantise_column_pair(const bf16 (*tile)[TC + TPAD], int cp, int kb, uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                     long long c0, long long r0, long long R, const SfLayout& lay) {
    float v0[32], v1[32];
    float a0 = 0.f, a1 = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&tile[kb * 32 + i][2 * cp]));
        v0[i] = f.x; v1[i] = f.y;
        a0 = fmaxf(a0, fabsf(f.x)); a1 = fmaxf(a1, fabsf(f.y));
    }
    float inv;
    uint4 lo, hi;
    const long long col = c0 + 2 * cp;
    uint32_t e = mx_scale(a0, inv);
    quantise32(v0, inv, lo, hi);
    uint4* dst = reinterpret_cast<uint4*>(q + col * R + r0 + kb * 32);
    dst[0] = lo; dst[1] = hi;
    sf[lay.offset(col, r0 / 32 + kb)] = static_cast<uint8_t>(e);
    e = mx_scale(a1, inv);
    quantise32(v1, inv, lo, hi);
    dst = reinterpret_cast<uint4*>(q + (col + 1) * R + r0 + kb * 32);
    dst[0] = lo; dst[1] = hi;
    sf[lay.offset(col + 1, r0 / 32 + kb)] = static_cast<uint8_t>(e);
}

__global__ void __launch_bounds__(256)
quantize_mx_cols_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const bf16* __restrict__ x, long long R, long long C, long long ld,
                        SfLayout lay) {
    __shared__ __align__(16) bf16 tile[TR][TC + TPAD];
    const long long c0 = static_cast<long long>(blockIdx.x) * TC;
    const long long r0 = static_cast<long long>(blockIdx.y) * TR;
    for (int i = threadIdx.x; i < TR * TC / 8; i += 256) {
        const int r = i / (TC / 8), cg = i % (TC / 8);
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c0 + cg * 8 < C) raw = __ldcs(reinterpret_cast<const uint4*>(x + (r0 + r) * ld + c0 + cg * 8));
        *reinterpret_cast<uint4*>(&tile[r][cg * 8]) = raw;
    }
    __syncthreads();
    const int cp = threadIdx.x % (TC / 2), kb = threadIdx.x / (TC / 2);
    if (c0 + 2 * cp >= C) return;               // C is even: both columns of a pair exist or neither
    quantise_column_pair(tile, cp, kb, q, sf, c0, r0, R, lay);
}

// Both forms from one read of the source: the tile goes through shared memory once; every thread then quantises 32-row
// blocks of two source columns (-> transposed output) and two 32-column blocks of a source row.
__global__ void __launch_bounds__(256)
quantize_mx_both_kernel(uint8_t* __restrict__ q_rows, uint8_t* __restrict__ sf_rows, uint8_t* __restrict__ q_cols, uint8_t* __restrict__ sf_cols,
                        const bf16* __restrict__ x, long long R, long long C, long long ld, SfLayout lay_rows, SfLayout lay_cols) {
    __shared__ __align__(16) bf16 tile[TR][TC + TPAD];
    const long long c0 = static_cast<long long>(blockIdx.x) * TC;
    const long long r0 = static_cast<long long>(blockIdx.y) * TR;
    for (int i = threadIdx.x; i < TR * TC / 8; i += 256) {
        const int r = i / (TC / 8), cg = i % (TC / 8);
        *reinterpret_cast<uint4*>(&tile[r][cg * 8]) = __ldcs(reinterpret_cast<const uint4*>(x + (r0 + r) * ld + c0 + cg * 8));
    }
    __syncthreads();
    quantise_column_pair(tile, threadIdx.x % (TC / 2), threadIdx.x / (TC / 2), q_cols, sf_cols, c0, r0, R, lay_cols);
    // row blocks: 32 source columns of one source row; the tile holds 4 per row, two per thread
    const int row = threadIdx.x / 2;
    uint32_t e2 = 0;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int blk = (threadIdx.x % 2) * 2 + h;
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 raw = *reinterpret_cast<const uint4*>(&tile[row][blk * 32 + g * 8]);
            const __nv_bfloat162* hh = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __bfloat1622float2(hh[j]);
                v[g * 8 + 2 * j] = f.x; v[g * 8 + 2 * j + 1] = f.y;
                amax = fmaxf(amax, fmaxf(fabsf(f.x), fabsf(f.y)));
            }
        }
        float inv;
        uint4 lo, hi;
        e2 |= mx_scale(amax, inv) << (8 * h);
        quantise32(v, inv, lo, hi);
        uint4* dst = reinterpret_cast<uint4*>(q_rows + (r0 + row) * C + c0 + blk * 32);
        dst[0] = lo; dst[1] = hi;
    }
    // the tile spans one K stage of the row form (128 columns): blocks 2 * (t % 2) and + 1 are neighbouring bytes
    *reinterpret_cast<uint16_t*>(sf_rows + lay_rows.offset(r0 + row, c0 / 32 + (threadIdx.x % 2) * 2)) = static_cast<uint16_t>(e2);
}

}  // namespace

// Bytes of the scale-factor buffer of an operand with `rows` rows and contraction length K.
extern "C" long long llmq_mx_sf_bytes(long long rows, long long K, int tile_rows) { return make_layout(rows, tile_rows).bytes(K); }

// x: bf16 [R, C] with row pitch ld.  See the top of this file.  The contraction length (C, or R when transposing) must be a
// multiple of 128, C a multiple of 8, ld * 2 bytes and the base 16-byte aligned.
extern "C" int llmq_quantize_mx(void* q, void* sf, const void* x, long long R, long long C, long long ld, int transpose, int tile_rows,
                                cudaStream_t stream) {
    if (R <= 0 || C <= 0) return 0;
    const long long K = transpose ? R : C, rows = transpose ? C : R;
    if (K % 128 || C % 8 || ld % 8 || tile_rows < 32 || tile_rows > 256 || tile_rows % 32) return -5;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q) & 15u) || (reinterpret_cast<uintptr_t>(sf) & 3u)) return -3;
    const SfLayout lay = make_layout(rows, tile_rows);
    if (rows % tile_rows || tile_rows % 128) {
        cudaError_t e = cudaMemsetAsync(sf, 0, static_cast<size_t>(lay.bytes(K)), stream);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    if (!transpose) {
        const long long total = R * (C / 32);
        quantize_mx_rows_kernel<<<static_cast<unsigned int>((total + 255) / 256), 256, 0, stream>>>(
            static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), static_cast<const bf16*>(x), R, C, ld, lay);
    } else {
        dim3 grid(static_cast<unsigned int>((C + TC - 1) / TC), static_cast<unsigned int>(R / TR));
        quantize_mx_cols_kernel<<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(q), static_cast<uint8_t*>(sf), static_cast<const bf16*>(x), R, C,
                                                          ld, lay);
    }
    return LLMQ_LAUNCH_CHECK();
}

// Row form (q_rows [R, C], scales tiled by tile_rows_r) and column form (q_cols [C, R], tiled by tile_rows_c) of the same
// bf16 matrix from one pass over it.  R and C multiples of 128.
extern "C" int llmq_quantize_mx_both(void* q_rows, void* sf_rows, int tile_rows_r, void* q_cols, void* sf_cols, int tile_rows_c, const void* x,
                                     long long R, long long C, long long ld, cudaStream_t stream) {
    if (R <= 0 || C <= 0) return 0;
    if (R % 128 || C % 128 || ld % 8) return -5;
    if ((reinterpret_cast<uintptr_t>(x) & 15u) || (reinterpret_cast<uintptr_t>(q_rows) & 15u) || (reinterpret_cast<uintptr_t>(q_cols) & 15u)) return -3;
    for (int t : {tile_rows_r, tile_rows_c}) if (t < 32 || t > 256 || t % 32) return -5;
    const SfLayout lr = make_layout(R, tile_rows_r), lc = make_layout(C, tile_rows_c);
    if (R % tile_rows_r || tile_rows_r % 128) {
        cudaError_t e = cudaMemsetAsync(sf_rows, 0, static_cast<size_t>(lr.bytes(C)), stream);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    if (C % tile_rows_c || tile_rows_c % 128) {
        cudaError_t e = cudaMemsetAsync(sf_cols, 0, static_cast<size_t>(lc.bytes(R)), stream);
        if (e != cudaSuccess) return static_cast<int>(e);
    }
    dim3 grid(static_cast<unsigned int>(C / TC), static_cast<unsigned int>(R / TR));
    quantize_mx_both_kernel<<<grid, 256, 0, stream>>>(static_cast<uint8_t*>(q_rows), static_cast<uint8_t*>(sf_rows), static_cast<uint8_t*>(q_cols),
                                                      static_cast<uint8_t*>(sf_cols), static_cast<const bf16*>(x), R, C, ld, lr, lc);
    return LLMQ_LAUNCH_CHECK();
}
