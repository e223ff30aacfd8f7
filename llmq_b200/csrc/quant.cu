// abs-max reduction, per-tensor fp8 quantisation, transposes, dtype conversion, fill and normal init.
// Behavioural counterparts of src/kernels/{quant,transpose,convert,fill,random}.cu of the reference.
// Recipe: q = sat_fp8(x * QMAX / max(absmax, 1e-10)), dequant factor absmax / QMAX is written next to it.
// QMAX is 448 for e4m3 and 57344 for e5m2 (the reference uses 448 for both, which wastes the e5m2 range).
#include "api.h"
#include "common.cuh"
#include "tile_transpose.cuh"
#include <type_traits>

namespace {

int grid_for(long long work_items, int threads, int num_sms) {
    long long blocks = ceil_div_ll(work_items, threads);
    long long cap = static_cast<long long>(num_sms) * 8;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

template <typename T>
__global__ void __launch_bounds__(512) absmax_kernel(float* __restrict__ out, const T* __restrict__ x, long long n) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    float tmax = 0.f;
    const long long nvec = n / V::N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        V v = V::load(x + i * V::N);
#pragma unroll
        for (int k = 0; k < V::N; ++k) tmax = fmaxf(tmax, fabsf(to_float(v.v[k])));
    }
    if (blockIdx.x == 0) {
        for (long long i = nvec * V::N + threadIdx.x; i < n; i += blockDim.x) tmax = fmaxf(tmax, fabsf(to_float(x[i])));
    }
    block_absmax_commit(out, tmax, scratch);
}

template <typename Q> struct QMax;
template <> struct QMax<e4m3> { static constexpr float value = 448.f; };
template <> struct QMax<e5m2> { static constexpr float value = 57344.f; };
template <> struct QMax<bf16> { static constexpr float value = 1.f; };

template <typename T, typename Q>
__global__ void __launch_bounds__(512)
quantize_kernel(Q* __restrict__ out, float* __restrict__ scale_out, const T* __restrict__ x, const float* __restrict__ absmax, long long n) {
    using V = Vec16<T>;
    float mul = 1.f;
    if constexpr (sizeof(Q) == 1) {
        float am = fmaxf(*absmax, 1e-10f);
        mul = QMax<Q>::value / am;
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = am / QMax<Q>::value;
    } else {
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = 1.f;
    }
    const long long nvec = n / V::N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        V v = V::load_stream(x + i * V::N);
        alignas(16) Q q[V::N];
#pragma unroll
        for (int k = 0; k < V::N; ++k) q[k] = from_float<Q>(to_float(v.v[k]) * mul);
        constexpr int bytes = V::N * sizeof(Q);
        if constexpr (bytes == 16) *reinterpret_cast<uint4*>(out + i * V::N) = *reinterpret_cast<uint4*>(q);
        else if constexpr (bytes == 8) *reinterpret_cast<uint2*>(out + i * V::N) = *reinterpret_cast<uint2*>(q);
        else *reinterpret_cast<uint32_t*>(out + i * V::N) = *reinterpret_cast<uint32_t*>(q);
    }
    if (blockIdx.x == 0) {
        for (long long i = nvec * V::N + threadIdx.x; i < n; i += blockDim.x) out[i] = from_float<Q>(to_float(x[i]) * mul);
    }
}

// out[c][r] = f(in[r][c]) through a padded shared-memory tile; optionally quantises on the way.
template <typename T, typename Q, bool Quant>
__global__ void __launch_bounds__(256)
transpose_kernel(Q* __restrict__ out, float* __restrict__ scale_out, const T* __restrict__ in, const float* __restrict__ absmax,
                 int rows, int cols) {
    __shared__ float tile[32][33];
    float mul = 1.f;
    if constexpr (Quant) {
        float am = fmaxf(*absmax, 1e-10f);
        mul = QMax<Q>::value / am;
        if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0 && threadIdx.y == 0 && scale_out) *scale_out = am / QMax<Q>::value;
    }
    int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += 8) {
        int r = r0 + j, c = c0 + threadIdx.x;
        if (r < rows && c < cols) tile[j][threadIdx.x] = to_float(in[static_cast<long long>(r) * cols + c]);
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += 8) {
        int c = c0 + j, r = r0 + threadIdx.x;
        if (r < rows && c < cols) out[static_cast<long long>(c) * rows + r] = from_float<Q>(tile[threadIdx.x][j] * mul);
    }
}

// One 128 x 128 tile per CTA: reads in[rows][cols] (bf16/fp32: quantised with the given abs-max; 1-byte types: copied),
// optionally writes the row-major 1-byte copy, and writes the transposed 1-byte copy out_t[cols][rows] so that the
// weight-gradient GEMMs can read both operands K-major (the reference's quantize_and_transpose_with_abs_max,
// src/kernels/quant.cu:100-193, and its fp8 transpose_kernel).  The tile sits in shared memory as 128 rows of 32 words;
// word w of row r lives at w ^ (((r >> 4) & 7) << 2), which makes both the row-major stores and the column reads
// (16 rows of one word column per thread) free of bank conflicts.  Every global access is a 16-byte vector (8 bytes for
// the row-major copy of 2-byte inputs); rows and cols must be multiples of 16.
template <typename T, typename Q>
__global__ void __launch_bounds__(256)
tile_transpose_kernel(Q* __restrict__ out_rows, Q* __restrict__ out_t, float* __restrict__ scale_out, const T* __restrict__ in,
                      const float* __restrict__ absmax, int rows, int cols) {
    static_assert(sizeof(Q) == 1, "1-byte outputs only");
    __shared__ __align__(16) uint32_t tile[128 * 32];
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
    float mul = 1.f;
    if constexpr (sizeof(T) > 1) {
        float am = fmaxf(*absmax, 1e-10f);
        mul = QMax<Q>::value / am;
        if (blockIdx.x == 0 && blockIdx.y == 0 && t == 0 && scale_out) *scale_out = am / QMax<Q>::value;
    }
    if constexpr (sizeof(T) == 2) {
        // 16 threads per row (8 elements each), 16 rows per pass
        const int cc = t & 15, rr = t >> 4;
        uint4 v[8];
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            int r = r0 + p * 16 + rr, c = c0 + cc * 8;
            v[p] = (r < rows && c < cols) ? __ldcs(reinterpret_cast<const uint4*>(in + static_cast<long long>(r) * cols + c)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            int lr = p * 16 + rr, r = r0 + lr, c = c0 + cc * 8;
            const T* e = reinterpret_cast<const T*>(&v[p]);
            uint2 w;
            if constexpr (std::is_same<Q, e4m3>::value) {
                float f[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] = to_float(e[k]) * mul;
                w = pack_e4m3x8(f);
            } else {
                alignas(8) Q q[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) q[k] = from_float<Q>(to_float(e[k]) * mul);
                w = *reinterpret_cast<uint2*>(q);
            }
            if (out_rows && r < rows && c < cols) *reinterpret_cast<uint2*>(out_rows + static_cast<long long>(r) * cols + c) = w;
            *reinterpret_cast<uint2*>(&tile[lr * 32 + ((cc * 2) ^ (((lr >> 4) & 7) << 2))]) = w;
        }
    } else if constexpr (sizeof(T) == 4) {
        // 32 threads per row (4 elements each), 8 rows per pass
        const int cc = t & 31, rr = t >> 5;
#pragma unroll 4
        for (int p = 0; p < 16; ++p) {
            int lr = p * 8 + rr, r = r0 + lr, c = c0 + cc * 4;
            float4 f = (r < rows && c < cols) ? *reinterpret_cast<const float4*>(in + static_cast<long long>(r) * cols + c) : make_float4(0, 0, 0, 0);
            alignas(4) Q q[4] = {from_float<Q>(f.x * mul), from_float<Q>(f.y * mul), from_float<Q>(f.z * mul), from_float<Q>(f.w * mul)};
            uint32_t w = *reinterpret_cast<uint32_t*>(q);
            if (out_rows && r < rows && c < cols) *reinterpret_cast<uint32_t*>(out_rows + static_cast<long long>(r) * cols + c) = w;
            tile[lr * 32 + (cc ^ (((lr >> 4) & 7) << 2))] = w;
        }
    } else {
        // 1-byte input: 8 threads per row (16 bytes each), 32 rows per pass
        const int cc = t & 7, rr = t >> 3;
        uint4 v[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            int r = r0 + p * 32 + rr, c = c0 + cc * 16;
            v[p] = (r < rows && c < cols) ? __ldcs(reinterpret_cast<const uint4*>(in + static_cast<long long>(r) * cols + c)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            int lr = p * 32 + rr;
            *reinterpret_cast<uint4*>(&tile[lr * 32 + ((cc * 4) ^ (((lr >> 4) & 7) << 2))]) = v[p];
        }
    }
    __syncthreads();
    tile_store_transposed<Q>(tile, out_t, r0, c0, rows, cols);
}

// out[c][r] = in[r][c] for 2-byte elements, 64 x 64 tiles, 16-byte global accesses on both sides (rows and cols multiples
// of 8).  The row pitch of 66 halves (33 words) spreads a column walk over the banks.
__global__ void __launch_bounds__(256)
transpose16_kernel(uint16_t* __restrict__ out, const uint16_t* __restrict__ in, int rows, int cols) {
    __shared__ __align__(16) uint16_t tile[64 * 66];
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    const int sub = t >> 3, ch = t & 7;
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int lr = p * 32 + sub, r = r0 + lr, c = c0 + ch * 8;
        const uint4 v = (r < rows && c < cols) ? __ldcs(reinterpret_cast<const uint4*>(in + static_cast<long long>(r) * cols + c)) : make_uint4(0, 0, 0, 0);
        uint32_t* dst = reinterpret_cast<uint32_t*>(&tile[lr * 66 + ch * 8]);
        dst[0] = v.x; dst[1] = v.y; dst[2] = v.z; dst[3] = v.w;
    }
    __syncthreads();
#pragma unroll
    for (int p = 0; p < 2; ++p) {
        const int lc = p * 32 + sub;                            // column of the input tile = row of the output
        const int c = c0 + lc, r = r0 + ch * 8;
        uint16_t h[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) h[k] = tile[(ch * 8 + k) * 66 + lc];
        if (c < cols && r < rows) {
            uint4 o;
            o.x = h[0] | (static_cast<uint32_t>(h[1]) << 16); o.y = h[2] | (static_cast<uint32_t>(h[3]) << 16);
            o.z = h[4] | (static_cast<uint32_t>(h[5]) << 16); o.w = h[6] | (static_cast<uint32_t>(h[7]) << 16);
            *reinterpret_cast<uint4*>(out + static_cast<long long>(c) * rows + r) = o;
        }
    }
}

template <typename S, typename D>
__global__ void __launch_bounds__(512) convert_kernel(D* __restrict__ out, const S* __restrict__ in, long long n) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = from_float<D>(to_float(in[i]));
}

template <typename T>
__global__ void __launch_bounds__(512) fill_kernel(T* __restrict__ out, float value, long long n) {
    T v = from_float<T>(value);
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x)
        out[i] = v;
}

// N(mean, std) from a counter-based generator: element i of stream (seed, subsequence) gets the same value
// whatever the launch geometry or the sharding of the tensor (offset = index of out[0] in the full tensor).
template <typename T>
__global__ void __launch_bounds__(256)
normal_kernel(T* __restrict__ out, long long n, float mean, float std, unsigned long long seed, unsigned long long subsequence,
              long long offset) {
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < n;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        unsigned long long ctr = static_cast<unsigned long long>(i + offset);
        uint32_t s0 = static_cast<uint32_t>(seed) ^ hash_u32(static_cast<uint32_t>(subsequence) * 0x9e3779b9u + static_cast<uint32_t>(seed >> 32));
        uint32_t a = rng_u32(ctr * 2ull, s0), b = rng_u32(ctr * 2ull + 1ull, s0 ^ static_cast<uint32_t>(subsequence >> 32));
        float u1 = (a >> 8) * (1.0f / 16777216.0f) + (0.5f / 16777216.0f);
        float u2 = (b >> 8) * (1.0f / 16777216.0f);
        float z = sqrtf(-2.f * logf(u1)) * cospif(2.f * u2);
        out[i] = from_float<T>(mean + std * z);
    }
}

}  // namespace

extern "C" int llmq_abs_max(float* out, const void* x, long long n, int dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    if (dtype == 0) absmax_kernel<bf16><<<grid_for(n / 8 + 1, 512, num_sms), 512, 0, s>>>(out, static_cast<const bf16*>(x), n);
    else if (dtype == 3) absmax_kernel<float><<<grid_for(n / 4 + 1, 512, num_sms), 512, 0, s>>>(out, static_cast<const float*>(x), n);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_quantize(void* out, float* scale_out, const void* x, const float* absmax, long long n, int in_dtype,
                             int out_dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
#define Q_CASE(T, TC, Q, QC, VN)                                                                                   \
    if (in_dtype == TC && out_dtype == QC) {                                                                       \
        quantize_kernel<T, Q><<<grid_for(n / VN + 1, 512, num_sms), 512, 0, s>>>(static_cast<Q*>(out), scale_out,  \
                                                                                 static_cast<const T*>(x), absmax, n); \
        return LLMQ_LAUNCH_CHECK();                                                                                \
    }
    Q_CASE(bf16, 0, e4m3, 1, 8)
    Q_CASE(bf16, 0, e5m2, 2, 8)
    Q_CASE(bf16, 0, bf16, 0, 8)
    Q_CASE(float, 3, e4m3, 1, 4)
    Q_CASE(float, 3, e5m2, 2, 4)
    Q_CASE(float, 3, bf16, 0, 4)
#undef Q_CASE
    return -10;
}

extern "C" int llmq_transpose(void* out, float* scale_out, const void* in, const float* absmax, int rows, int cols,
                              int in_dtype, int out_dtype, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return 0;
    if (in_dtype == 0 && out_dtype == 0 && absmax == nullptr && rows % 8 == 0 && cols % 8 == 0 &&
        ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0) {
        transpose16_kernel<<<dim3(ceil_div_i(cols, 64), ceil_div_i(rows, 64)), 256, 0, s>>>(static_cast<uint16_t*>(out), static_cast<const uint16_t*>(in), rows, cols);
        return LLMQ_LAUNCH_CHECK();
    }
    dim3 grid(ceil_div_i(cols, 32), ceil_div_i(rows, 32)), block(32, 8);
#define T_CASE(T, TC, Q, QC, QUANT)                                                                                \
    if (in_dtype == TC && out_dtype == QC && (absmax != nullptr) == QUANT) {                                       \
        transpose_kernel<T, Q, QUANT><<<grid, block, 0, s>>>(static_cast<Q*>(out), scale_out, static_cast<const T*>(in), absmax, rows, cols); \
        return LLMQ_LAUNCH_CHECK();                                                                                \
    }
    T_CASE(bf16, 0, bf16, 0, false)
    T_CASE(float, 3, float, 3, false)
    T_CASE(e4m3, 1, e4m3, 1, false)
    T_CASE(e5m2, 2, e5m2, 2, false)
    T_CASE(bf16, 0, e4m3, 1, true)
    T_CASE(bf16, 0, e5m2, 2, true)
    T_CASE(float, 3, e4m3, 1, true)
#undef T_CASE
    return -10;
}

// out_rows (optional, [rows][cols]) and out_t ([cols][rows]) are 1-byte copies of in[rows][cols]; with a 2- or 4-byte
// input the values are quantised with *absmax first.  rows % 16 == 0 and cols % 16 == 0.
extern "C" int llmq_quantize_transpose(void* out_rows, void* out_t, float* scale_out, const void* in, const float* absmax, int rows,
                                       int cols, int in_dtype, int out_dtype, cudaStream_t s) {
    if (rows <= 0 || cols <= 0) return 0;
    if (rows % 16 != 0 || cols % 16 != 0 || out_t == nullptr) return -11;
    dim3 grid(ceil_div_i(cols, 128), ceil_div_i(rows, 128));
#define QT_CASE(T, TC, Q, QC)                                                                                         \
    if (in_dtype == TC && out_dtype == QC) {                                                                          \
        if (sizeof(T) > 1 && absmax == nullptr) return -12;                                                           \
        tile_transpose_kernel<T, Q><<<grid, 256, 0, s>>>(static_cast<Q*>(out_rows), static_cast<Q*>(out_t), scale_out, \
                                                         static_cast<const T*>(in), absmax, rows, cols);              \
        return LLMQ_LAUNCH_CHECK();                                                                                   \
    }
    QT_CASE(bf16, 0, e4m3, 1)
    QT_CASE(bf16, 0, e5m2, 2)
    QT_CASE(float, 3, e4m3, 1)
    QT_CASE(float, 3, e5m2, 2)
    QT_CASE(e4m3, 1, e4m3, 1)
    QT_CASE(e5m2, 2, e5m2, 2)
#undef QT_CASE
    return -10;
}

extern "C" int llmq_convert(void* out, const void* in, long long n, int in_dtype, int out_dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    int g = grid_for(n, 512, num_sms);
#define C_CASE(S, SC, D, DC)                                                                        \
    if (in_dtype == SC && out_dtype == DC) {                                                        \
        convert_kernel<S, D><<<g, 512, 0, s>>>(static_cast<D*>(out), static_cast<const S*>(in), n); \
        return LLMQ_LAUNCH_CHECK();                                                                 \
    }
    C_CASE(float, 3, bf16, 0)
    C_CASE(bf16, 0, float, 3)
    C_CASE(__half, 4, bf16, 0)
    C_CASE(__half, 4, float, 3)
    C_CASE(float, 3, __half, 4)
    C_CASE(bf16, 0, __half, 4)
    C_CASE(e4m3, 1, bf16, 0)
    C_CASE(e4m3, 1, float, 3)
    C_CASE(e5m2, 2, bf16, 0)
#undef C_CASE
    return -10;
}

extern "C" int llmq_fill(void* out, float value, long long n, int dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    int g = grid_for(n, 512, num_sms);
    if (dtype == 0) fill_kernel<bf16><<<g, 512, 0, s>>>(static_cast<bf16*>(out), value, n);
    else if (dtype == 3) fill_kernel<float><<<g, 512, 0, s>>>(static_cast<float*>(out), value, n);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_fill_normal(void* out, long long n, float mean, float std, unsigned long long seed,
                                unsigned long long subsequence, long long offset, int dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    int g = grid_for(n, 256, num_sms);
    if (dtype == 0) normal_kernel<bf16><<<g, 256, 0, s>>>(static_cast<bf16*>(out), n, mean, std, seed, subsequence, offset);
    else if (dtype == 3) normal_kernel<float><<<g, 256, 0, s>>>(static_cast<float*>(out), n, mean, std, seed, subsequence, offset);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}
