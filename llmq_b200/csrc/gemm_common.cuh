// Pieces shared by the one-CTA and the two-CTA tcgen05 GEMM kernels: launch parameters and the epilogue that
// moves one accumulator row block from tensor memory to global memory.
#pragma once
#include "ptx_sm100.cuh"
#include "common.cuh"

struct GemmParams {
    int M, N, K;
    int elem_bytes;        // 1 or 2
    int a_mn_major, b_mn_major;
    int a_fmt, b_fmt;      // instruction-descriptor format codes
    void* C;
    long long ldc;         // elements
    int c_dtype;           // 0 = bf16, 1 = fp32
    int accumulate;
    const void* bias;      // bf16 or fp32 (bias_dtype) or null, indexed by N
    int bias_dtype;
    const float* scale_a;  // optional dequant factors
    const float* scale_b;
    float alpha;
    float* absmax_out;     // optional
    unsigned int* status;  // error word
    // Optional: rows of B arrive from other GPUs (fused all-gather).  ready_flags[src] >= ready_gen means the rows
    // [src * ready_rows_per_src, (src+1) * ready_rows_per_src) of the stored B matrix are complete in local memory.
    const unsigned int* ready_flags;
    unsigned int ready_gen;
    int ready_rows_per_src;
    unsigned long long ready_limit_ns;
    // Optional: reduce-scatter fused into the kernel (CTA-pair kernel only).  Output row r belongs to rank
    // r / rs_shard_rows; the epilogue stores it into that rank's landing buffer, slot [this rank], over NVLink and
    // bumps the owner's arrival counter; after its last tile every CTA helps to sum this rank's `rs_world` slots
    // into the gradient shard.  rs_world == 0 switches all of this off.
    int rs_world, rs_rank, rs_shard_rows;
    void* rs_landing[8];            // landing buffer of every rank: [rs_world][rs_shard_rows][N] bf16
    unsigned int* rs_counter[8];    // arrival counter word of every rank
    unsigned int rs_target;         // local counter value once every source delivered all of its tiles
    void* rs_dst;                   // bf16 shard [rs_shard_rows][N]
    int rs_accumulate;              // dst += (stochastic rounding) instead of dst =
    float rs_scale;
    float* rs_norm_partials;        // optional, rs_num_partials floats: sum of squares of the new shard values
    int rs_num_partials;
    unsigned int rs_seed;
    unsigned long long rs_limit_ns;
    // Optional SwiGLU fused into the epilogue (CTA-pair kernel only, bf16 output).  ep_D = features D.
    //   ep_mode 1 (forward, N = 2D): the pair stages rows [f, f+128) (up) and [D+f, D+f+128) (gate) of B, so one
    //     accumulator tile holds up and gate of the same 128 features; C[M, 2D] gets both, ep_ptr[M, D] gets
    //     up * gate * sigmoid(gate), absmax_out tracks the latter.
    //   ep_mode 2 (backward, N = D): the accumulator is d(swiglu out); ep_ptr[M, 2D] holds [up | gate] on entry and
    //     [d_up | d_gate] on exit (in place), C is not written, absmax_out tracks the gradients.
    int ep_mode;
    void* ep_ptr;
    int ep_D;
    // Optional split-K (one-CTA kernel only): the K loop of every tile is cut into k_splits parts handled by different
    // CTAs; each writes its raw fp32 accumulator to partial[split][M][N] and a second kernel sums the parts and applies
    // the normal epilogue.  For outputs with fewer tiles than SMs and a long K (weight gradients of small models).
    int k_splits;
    float* partial;
    // CTA-pair kernel: 1 when the kernel's third tensor map describes C (bf16, plain store) and the epilogue may write
    // its staged 32 x 64 blocks with TMA stores instead of per-lane global stores
    int c_tma;
};

// Adds bias[col0 .. col0+31] to the 32 values of one accumulator chunk (every lane needs the same 32 bias values:
// vector loads that broadcast out of L1).
__device__ __forceinline__ void add_bias32(const GemmParams& p, int col0, float (&v)[32]) {
    if (p.bias_dtype == 0 && col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(static_cast<const __nv_bfloat16*>(p.bias) + col0) & 15u) == 0)) {
        const uint4* bp = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(p.bias) + col0);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
            uint4 bv = __ldg(bp + g);
            const __nv_bfloat162* bh = reinterpret_cast<const __nv_bfloat162*>(&bv);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __bfloat1622float2(bh[j]);
                v[g * 8 + 2 * j] += f.x; v[g * 8 + 2 * j + 1] += f.y;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < 32; ++j) {
            int cj = col0 + j;
            if (cj < p.N) {
                v[j] += p.bias_dtype == 0 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[cj])
                                          : static_cast<const float*>(p.bias)[cj];
            }
        }
    }
}

// Shared memory one epilogue warp needs for the coalescing store path of epilogue_rows (32 rows x 128 bytes).
constexpr int EPI_STAGE_BYTES_PER_WARP = 32 * 128;

// Each lane of the calling warp owns one accumulator row (TMEM lane); `t_row` addresses column 0 of that row
// block.  Applies alpha and bias, optionally adds the previous C, stores bf16 or fp32, tracks abs-max.
// The TMEM loads are warp-collective, so all lanes run the loop; only the stores are predicated on the row.
// `dst_row` (bf16, optional) redirects the stores of this lane's row to another buffer - possibly on a peer GPU -
// while an accumulating epilogue still reads the previous values from C.
//
// `stage` (optional, 128-byte aligned, EPI_STAGE_BYTES_PER_WARP bytes owned by this warp): plain bf16 outputs go
// through it 64 columns at a time.  Lane = row writes its 128 bytes as eight 16-byte chunks at chunk ^ (row & 7)
// (no bank conflicts), then eight lanes store the 128 contiguous bytes of one row, four rows per instruction.
// Straight from the accumulator layout every store instruction would touch 32 rows with 16 bytes each; with short K
// those scattered writes, not the tensor core, set the tile time (16384 x 37888 x 3584 e4m3: 1.62 ms against 1.46 ms
// with the stores removed).
__device__ __forceinline__ void epilogue_rows(const GemmParams& p, uint32_t t_row, int row, int col_base, int ncols,
                                              float alpha, float& tmax, __nv_bfloat16* dst_row = nullptr, uint8_t* stage = nullptr,
                                              const CUtensorMap* tmap_c = nullptr, int* stage_sel = nullptr) {
    using namespace sm100;
    const bool row_ok = row < p.M;
    // (`dst_row` redirection: the rows of one warp are consecutive rows of the same landing slot, N elements apart)
    const int lane_id = threadIdx.x & 31;
    __nv_bfloat16* const out_base = dst_row ? dst_row - static_cast<long long>(lane_id) * p.N
                                            : static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row - lane_id) * p.ldc;
    const long long out_ld = dst_row ? p.N : p.ldc;
    if (stage != nullptr && p.c_dtype == 0 && !p.accumulate && (p.N & 7) == 0 && (out_ld & 7) == 0 &&
        (reinterpret_cast<uintptr_t>(out_base) & 15u) == 0) {
        const int lane = lane_id;
        const int sub = lane >> 3, ch = lane & 7;
        const int row_base = row - lane;
        // With a tensor map for C the staged block leaves through one TMA store (box 64 columns x 32 rows, clipped at the
        // matrix edges) issued by lane 0; two staging buffers alternate, a buffer is rewritten once the store that read it
        // two blocks ago has finished reading (bulk-group accounting of lane 0).
        const bool use_tma = tmap_c != nullptr && p.c_tma != 0 && stage_sel != nullptr && dst_row == nullptr;
        uint32_t stage_addr = smem_u32(stage);
#pragma unroll 1
        for (int c = 0; c < ncols; c += 64) {
            const int col0 = col_base + c;
            if (col0 >= p.N) break;                    // uniform across the warp
            const bool second = col0 + 32 < p.N;       // uniform
            uint32_t r[2][32];
            tmem_ld_32x32b_x32(t_row + c, r[0]);
            if (second) tmem_ld_32x32b_x32(t_row + c + 32, r[1]);
            tmem_ld_wait();
            uint32_t packed[32];
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = (h == 0 || second) ? __uint_as_float(r[h][j]) * alpha : 0.f;
                if (p.bias && (h == 0 || second)) add_bias32(p, col0 + 32 * h, v);
                if (p.absmax_out && row_ok) {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + 32 * h + j < p.N) tmax = fmaxf(tmax, fabsf(v[j]));
                }
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                    packed[16 * h + j] = *reinterpret_cast<uint32_t*>(&b);
                }
            }
            if (use_tma) {
                stage_addr = smem_u32(stage) + static_cast<uint32_t>(*stage_sel) * EPI_STAGE_BYTES_PER_WARP;
                if (lane == 0) tma_store_wait_read<1>();
                __syncwarp();
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const uint32_t a = stage_addr + lane * 128 + ((i ^ (lane & 7)) << 4);
                asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(a), "r"(packed[4 * i]), "r"(packed[4 * i + 1]),
                             "r"(packed[4 * i + 2]), "r"(packed[4 * i + 3]) : "memory");
            }
            if (use_tma) {
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) { tma_store_2d(tmap_c, stage_addr, col0, row_base); tma_store_commit(); }
                *stage_sel ^= 1;
                continue;
            }
            __syncwarp();
            const int gcol = col0 + ch * 8;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int rr = 4 * j + sub;
                uint4 o;
                const uint32_t a = stage_addr + rr * 128 + ((ch ^ (rr & 7)) << 4);
                asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(o.x), "=r"(o.y), "=r"(o.z), "=r"(o.w) : "r"(a) : "memory");
                const int grow = row_base + rr;
                if (grow < p.M && gcol < p.N) *reinterpret_cast<uint4*>(out_base + rr * out_ld + gcol) = o;
            }
            __syncwarp();
        }
        return;
    }
#pragma unroll 1
    for (int c = 0; c < ncols; c += 32) {
        const int col0 = col_base + c;
        if (col0 >= p.N) break;                    // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) * alpha;
        if (p.bias) add_bias32(p, col0, v);
        if (row_ok) {
            const bool full = (col0 + 32 <= p.N);
            if (p.c_dtype == 0) {
                __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
                __nv_bfloat16* wp = dst_row ? dst_row + col0 : cp;
                if (full && (((reinterpret_cast<uintptr_t>(cp) | reinterpret_cast<uintptr_t>(wp)) & 15u) == 0)) {
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        uint4 o;
                        if (p.accumulate) {
                            uint4 old = *reinterpret_cast<const uint4*>(cp + g * 8);
                            const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&old);
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                float2 f = __bfloat1622float2(oh[j]);
                                v[g * 8 + 2 * j] += f.x; v[g * 8 + 2 * j + 1] += f.y;
                            }
                        }
                        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
                        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
                        *reinterpret_cast<uint4*>(wp + g * 8) = o;
                    }
                } else {
                    for (int j = 0; j < 32; ++j) {
                        if (col0 + j < p.N) {
                            if (p.accumulate) v[j] += __bfloat162float(cp[j]);
                            wp[j] = __float2bfloat16_rn(v[j]);
                        }
                    }
                }
            } else {
                float* cp = static_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col0;
                if (full && ((reinterpret_cast<uintptr_t>(cp) & 15u) == 0)) {
#pragma unroll
                    for (int g = 0; g < 8; ++g) {
                        float4 o = make_float4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
                        if (p.accumulate) {
                            float4 old = *reinterpret_cast<const float4*>(cp + g * 4);
                            o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                            v[g * 4] = o.x; v[g * 4 + 1] = o.y; v[g * 4 + 2] = o.z; v[g * 4 + 3] = o.w;
                        }
                        *reinterpret_cast<float4*>(cp + g * 4) = o;
                    }
                } else {
                    for (int j = 0; j < 32; ++j) {
                        if (col0 + j < p.N) {
                            if (p.accumulate) v[j] += cp[j];
                            cp[j] = v[j];
                        }
                    }
                }
            }
            if (p.absmax_out) {
#pragma unroll
                for (int j = 0; j < 32; ++j)
                    if (col0 + j < p.N) tmax = fmaxf(tmax, fabsf(v[j]));
            }
        }
    }
}

__device__ __forceinline__ float gemm_sigmoid(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }

__device__ __forceinline__ void load32_bf16(const __nv_bfloat16* p, float (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p + g * 8);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const float2 f = __bfloat1622float2(h[j]); v[g * 8 + 2 * j] = f.x; v[g * 8 + 2 * j + 1] = f.y; }
    }
}
__device__ __forceinline__ void store32_bf16(__nv_bfloat16* p, const float (&v)[32]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
        *reinterpret_cast<uint4*>(p + g * 8) = o;
    }
}

// SwiGLU forward epilogue: accumulator columns [0,128) = up, [128,256) = gate of features f0 .. f0+127 (all D and
// row pitches are multiples of 8 elements, so every 32-column chunk is 16-byte aligned).
__device__ __forceinline__ void epilogue_rows_swiglu_fwd(const GemmParams& p, uint32_t t_row, int row, int f0, float alpha, float& tmax) {
    using namespace sm100;
    const bool row_ok = row < p.M;
    __nv_bfloat16* crow = static_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
    __nv_bfloat16* srow = static_cast<__nv_bfloat16*>(p.ep_ptr) + static_cast<long long>(row) * p.ep_D;
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
        if (f0 + c >= p.ep_D) break;                 // uniform across the warp
        uint32_t ru[32], rg[32];
        tmem_ld_32x32b_x32(t_row + c, ru);
        tmem_ld_32x32b_x32(t_row + 128 + c, rg);
        tmem_ld_wait();
        if (row_ok) {
            float u[32], g[32], o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                // the saved projection is bf16: the activation is computed from the rounded values, like the separate kernel
                u[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(ru[j]) * alpha));
                g[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rg[j]) * alpha));
                o[j] = __bfloat162float(__float2bfloat16_rn(u[j] * g[j] * gemm_sigmoid(g[j])));
                tmax = fmaxf(tmax, fabsf(o[j]));
            }
            store32_bf16(crow + f0 + c, u);
            store32_bf16(crow + p.ep_D + f0 + c, g);
            store32_bf16(srow + f0 + c, o);
        }
    }
}

// SwiGLU backward epilogue over accumulator columns [0, ncols) = d(out) of features f0 ..
__device__ __forceinline__ void epilogue_rows_swiglu_bwd(const GemmParams& p, uint32_t t_row, int row, int f0, int ncols, float alpha, float& tmax) {
    using namespace sm100;
    const bool row_ok = row < p.M;
    __nv_bfloat16* urow = static_cast<__nv_bfloat16*>(p.ep_ptr) + static_cast<long long>(row) * 2 * p.ep_D;
#pragma unroll 1
    for (int c = 0; c < ncols; c += 32) {
        if (f0 + c >= p.ep_D) break;
        uint32_t rd[32];
        tmem_ld_32x32b_x32(t_row + c, rd);
        tmem_ld_wait();
        if (row_ok) {
            float u[32], g[32];
            load32_bf16(urow + f0 + c, u);
            load32_bf16(urow + p.ep_D + f0 + c, g);
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float d = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rd[j]) * alpha));   // d(out) as the bf16 the unfused path stores
                const float sg = gemm_sigmoid(g[j]);
                const float du = __bfloat162float(__float2bfloat16_rn(d * g[j] * sg));
                const float dg = __bfloat162float(__float2bfloat16_rn(d * u[j] * sg * (1.f + g[j] * (1.f - sg))));
                tmax = fmaxf(tmax, fmaxf(fabsf(du), fabsf(dg)));
                u[j] = du; g[j] = dg;
            }
            store32_bf16(urow + f0 + c, u);
            store32_bf16(urow + p.ep_D + f0 + c, g);
        }
    }
}

// Raw fp32 accumulator rows -> partial[split] (split-K); same lane / row convention as epilogue_rows.
__device__ __forceinline__ void epilogue_rows_partial(const GemmParams& p, uint32_t t_row, int row, int col_base, int ncols, int split) {
    using namespace sm100;
    const bool row_ok = row < p.M;
    float* prow = p.partial + (static_cast<long long>(split) * p.M + row) * p.N;
#pragma unroll 1
    for (int c = 0; c < ncols; c += 32) {
        const int col0 = col_base + c;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32b_x32(t_row + c, r);
        tmem_ld_wait();
        if (row_ok) {
            if (col0 + 32 <= p.N && ((reinterpret_cast<uintptr_t>(prow + col0) & 15u) == 0)) {
#pragma unroll
                for (int g = 0; g < 8; ++g)
                    *reinterpret_cast<float4*>(prow + col0 + g * 4) = make_float4(__uint_as_float(r[g * 4]), __uint_as_float(r[g * 4 + 1]),
                                                                                  __uint_as_float(r[g * 4 + 2]), __uint_as_float(r[g * 4 + 3]));
            } else {
                for (int j = 0; j < 32; ++j) if (col0 + j < p.N) prow[col0 + j] = __uint_as_float(r[j]);
            }
        }
    }
}
