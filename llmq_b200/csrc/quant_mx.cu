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

// Tile of 128 source rows (one K stage of the column form) x 64 source columns.  Input and outputs are staged in shared
// memory so that every global access is a run of full 32-byte sectors: the column form leaves as 64 rows x 128 bytes, the
// row form as 128 rows x 64 bytes.
constexpr int TC = 64, TR = 128, TPAD = 8;

struct MxTileSmem {
    bf16 in[TR][TC + TPAD];             // source tile
    uint8_t out_c[TC][TR + 16];         // transposed e4m3 tile (column form), 16 bytes of padding against bank conflicts
    uint8_t out_r[TR][TC + 16];         // e4m3 tile in source orientation (row form)
    uint32_t sf_c[TC];                  // the four block scales of every source column
};

__device__ __forceinline__ void load_tile(MxTileSmem& sm, const bf16* __restrict__ x, long long r0, long long c0, long long C, long long ld) {
    for (int i = threadIdx.x; i < TR * TC / 8; i += 256) {
        const int r = i / (TC / 8), cg = i % (TC / 8);
        uint4 raw = make_uint4(0, 0, 0, 0);
        if (c0 + cg * 8 < C) raw = __ldcs(reinterpret_cast<const uint4*>(x + (r0 + r) * ld + c0 + cg * 8));
        *reinterpret_cast<uint4*>(&sm.in[r][cg * 8]) = raw;
    }
}

// thread (column, block): 32 source rows of one source column -> shared memory; then the tile leaves in 128-byte rows
__device__ __forceinline__ void column_form(MxTileSmem& sm, uint8_t* __restrict__ q, uint8_t* __restrict__ sf, long long r0, long long c0,
                                            long long R, long long C, const SfLayout& lay) {
    const int col = threadIdx.x % TC, kb = threadIdx.x / TC;
    float v[32];
    float amax = 0.f;
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = __bfloat162float(sm.in[kb * 32 + i][col]);
        amax = fmaxf(amax, fabsf(v[i]));
    }
    float inv;
    uint4 lo, hi;
    const uint32_t e = mx_scale(amax, inv);
    quantise32(v, inv, lo, hi);
    *reinterpret_cast<uint4*>(&sm.out_c[col][kb * 32]) = lo;
    *reinterpret_cast<uint4*>(&sm.out_c[col][kb * 32 + 16]) = hi;
    reinterpret_cast<uint8_t*>(&sm.sf_c[col])[kb] = static_cast<uint8_t>(e);
    __syncthreads();
    for (int i = threadIdx.x; i < TC * TR / 16; i += 256) {
        const int row = i / (TR / 16), ch = i % (TR / 16);
        if (c0 + row < C) *reinterpret_cast<uint4*>(q + (c0 + row) * R + r0 + ch * 16) = *reinterpret_cast<const uint4*>(&sm.out_c[row][ch * 16]);
    }
    if (threadIdx.x < TC && c0 + threadIdx.x < C)
        *reinterpret_cast<uint32_t*>(sf + lay.offset(c0 + threadIdx.x, r0 / 32)) = sm.sf_c[threadIdx.x];
}

__global__ void __launch_bounds__(256)
quantize_mx_cols_kernel(uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const bf16* __restrict__ x, long long R, long long C, long long ld,
                        SfLayout lay) {
    __shared__ __align__(16) MxTileSmem sm;
    const long long c0 = static_cast<long long>(blockIdx.x) * TC;
    const long long r0 = static_cast<long long>(blockIdx.y) * TR;
    load_tile(sm, x, r0, c0, C, ld);
    __syncthreads();
    column_form(sm, q, sf, r0, c0, R, C, lay);
}

// Both forms from one read of the source.
__global__ void __launch_bounds__(256)
quantize_mx_both_kernel(uint8_t* __restrict__ q_rows, uint8_t* __restrict__ sf_rows, uint8_t* __restrict__ q_cols, uint8_t* __restrict__ sf_cols,
                        const bf16* __restrict__ x, long long R, long long C, long long ld, SfLayout lay_rows, SfLayout lay_cols) {
    __shared__ __align__(16) MxTileSmem sm;
    const long long c0 = static_cast<long long>(blockIdx.x) * TC;
    const long long r0 = static_cast<long long>(blockIdx.y) * TR;
    load_tile(sm, x, r0, c0, C, ld);
    __syncthreads();
    {   // row form: thread (row, half) quantises 32 source columns of one source row
        const int row = threadIdx.x / 2, blk = threadIdx.x % 2;
        float v[32];
        float amax = 0.f;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            const uint4 raw = *reinterpret_cast<const uint4*>(&sm.in[row][blk * 32 + g * 8]);
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
        const uint32_t e = mx_scale(amax, inv);
        quantise32(v, inv, lo, hi);
        *reinterpret_cast<uint4*>(&sm.out_r[row][blk * 32]) = lo;
        *reinterpret_cast<uint4*>(&sm.out_r[row][blk * 32 + 16]) = hi;
        // the two blocks of a row sit in neighbouring lanes and in neighbouring scale bytes (64 columns = half a K stage)
        const uint32_t pair = e | (__shfl_xor_sync(0xffffffffu, e, 1) << 8);
        if (blk == 0) *reinterpret_cast<uint16_t*>(sf_rows + lay_rows.offset(r0 + row, c0 / 32)) = static_cast<uint16_t>(pair);
    }
    column_form(sm, q_cols, sf_cols, r0, c0, R, C, lay_cols);       // contains the barrier that also covers out_r
    for (int i = threadIdx.x; i < TR * TC / 16; i += 256) {
        const int row = i / (TC / 16), ch = i % (TC / 16);
        *reinterpret_cast<uint4*>(q_rows + (r0 + row) * C + c0 + ch * 16) = *reinterpret_cast<const uint4*>(&sm.out_r[row][ch * 16]);
    }
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
