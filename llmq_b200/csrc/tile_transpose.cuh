// Shared-memory tile transpose of 1-byte elements, shared by the quantise + transpose kernels (quant.cu) and the SwiGLU
// recompute that only needs the transposed fp8 copy (act.cu).  A 128 x 128 byte tile sits in shared memory as 128 rows of 32
// words; word w of row r lives at w ^ (((r >> 4) & 7) << 2), which makes both the row-major stores (2, 4 or 16 bytes per
// thread) and the column reads (16 rows of one word column per thread) free of bank conflicts.
#pragma once
#include <cstdint>

// 4 x 4 byte transpose: words a..d hold bytes [x0 x1 x2 x3] of four consecutive rows; col[k] = [a_k b_k c_k d_k].
__device__ __forceinline__ void transpose_4x4_bytes(uint32_t a, uint32_t b, uint32_t c, uint32_t d, uint32_t (&col)[4]) {
    uint32_t t0 = __byte_perm(a, b, 0x5140), t1 = __byte_perm(c, d, 0x5140);
    uint32_t t2 = __byte_perm(a, b, 0x7362), t3 = __byte_perm(c, d, 0x7362);
    col[0] = __byte_perm(t0, t1, 0x5410);
    col[1] = __byte_perm(t0, t1, 0x7632);
    col[2] = __byte_perm(t2, t3, 0x5410);
    col[3] = __byte_perm(t2, t3, 0x7632);
}

// Index of word `w` (4 columns) of tile row `lr`.
__device__ __forceinline__ int tile_word_index(int lr, int w) { return lr * 32 + (w ^ (((lr >> 4) & 7) << 2)); }

// Writes the transposed tile: out_t[cols][rows], tile origin (r0, c0).  Thread = (16-row chunk rc, word column cw): eight
// lanes of equal cw write 128 contiguous bytes of one output row.  rows and cols are multiples of 16; 256 threads.
template <typename Q>
__device__ __forceinline__ void tile_store_transposed(const uint32_t* tile, Q* __restrict__ out_t, int r0, int c0, int rows, int cols) {
    static_assert(sizeof(Q) == 1, "1-byte outputs only");
    const int t = threadIdx.x;
    const int lane = t & 31, warp = t >> 5;
    const int rc = lane & 7, cw = warp * 4 + (lane >> 3);
    uint32_t w[16];
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j] = tile[(rc * 16 + j) * 32 + (cw ^ (rc << 2))];
    uint32_t o[4][4];            // o[g][k]: rows 4g..4g+3 of column k
#pragma unroll
    for (int g = 0; g < 4; ++g) transpose_4x4_bytes(w[4 * g], w[4 * g + 1], w[4 * g + 2], w[4 * g + 3], o[g]);
    const int r = r0 + rc * 16;
    if (r < rows) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            int c = c0 + cw * 4 + k;
            if (c < cols)
                *reinterpret_cast<uint4*>(out_t + static_cast<long long>(c) * rows + r) = make_uint4(o[0][k], o[1][k], o[2][k], o[3][k]);
        }
    }
}
