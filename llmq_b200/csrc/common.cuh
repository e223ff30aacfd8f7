// Device helpers shared by all kernels: 16-byte vector access, warp/block reductions, abs-max
// atomics, a counter-based hash RNG for stochastic rounding, and fp8 conversion.
#pragma once
#include <cstdint>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

typedef __nv_bfloat16 bf16;
typedef __nv_fp8_e4m3 e4m3;
typedef __nv_fp8_e5m2 e5m2;

#define LLMQ_LAUNCH_CHECK() static_cast<int>(cudaGetLastError())

__host__ __device__ constexpr long long ceil_div_ll(long long a, long long b) { return (a + b - 1) / b; }
__host__ __device__ constexpr int ceil_div_i(int a, int b) { return (a + b - 1) / b; }

// ------------------------------------------------------------------------------------------------
// Reductions
__device__ __forceinline__ float warp_reduce_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_reduce_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide reductions; `scratch` holds at least 32 floats of shared memory. All threads get the result.
__device__ __forceinline__ float block_reduce_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_reduce_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : 0.f;
    return warp_reduce_sum(r);
}
__device__ __forceinline__ float block_reduce_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_reduce_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? scratch[lane] : -INFINITY;
    return warp_reduce_max(r);
}

// abs-max values are non-negative floats, whose bit patterns order like unsigned integers
__device__ __forceinline__ void atomic_max_float(float* addr, float v) {
    atomicMax(reinterpret_cast<unsigned int*>(addr), __float_as_uint(v));
}
// Reduces a per-thread abs-max over the block and merges it into *dst (if dst != null).
__device__ __forceinline__ void block_absmax_commit(float* dst, float tmax, float* scratch) {
    if (!dst) return;
    tmax = block_reduce_max(tmax, scratch);
    if (threadIdx.x == 0 && tmax > 0.f) atomic_max_float(dst, tmax);
}

// ------------------------------------------------------------------------------------------------
// Element access for the supported storage types
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<bf16>(bf16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<e4m3>(e4m3 v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_float<e5m2>(e5m2 v) { return static_cast<float>(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_float<bf16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ e4m3 from_float<e4m3>(float v) { return e4m3(v); }   // saturating
template <> __device__ __forceinline__ e5m2 from_float<e5m2>(float v) { return e5m2(v); }

// Two floats -> two e4m3 bytes with one conversion instruction (saturating, round to nearest even).
__device__ __forceinline__ uint32_t pack_e4m3x2(float lo, float hi) {
    return static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(make_float2(lo, hi), __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ uint2 pack_e4m3x8(const float (&f)[8]) {
    uint2 r;
    r.x = pack_e4m3x2(f[0], f[1]) | (pack_e4m3x2(f[2], f[3]) << 16);
    r.y = pack_e4m3x2(f[4], f[5]) | (pack_e4m3x2(f[6], f[7]) << 16);
    return r;
}

// 16-byte vector of T
template <typename T>
struct alignas(16) Vec16 {
    static constexpr int N = 16 / sizeof(T);
    T v[N];
    __device__ __forceinline__ static Vec16 load(const T* p) {
        Vec16 r;
        *reinterpret_cast<uint4*>(r.v) = *reinterpret_cast<const uint4*>(p);
        return r;
    }
    __device__ __forceinline__ static Vec16 load_stream(const T* p) {   // read-once data
        Vec16 r;
        *reinterpret_cast<uint4*>(r.v) = __ldcs(reinterpret_cast<const uint4*>(p));
        return r;
    }
    __device__ __forceinline__ void store(T* p) const { *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(v); }
    __device__ __forceinline__ void store_stream(T* p) const { __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(v)); }
};

// ------------------------------------------------------------------------------------------------
// Division of a 31-bit index by a loop-invariant divisor with one multiply-high and a shift (the per-element
// index arithmetic of the streaming kernels would otherwise cost more instructions than their math).
struct FastDiv {
    uint32_t d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(uint32_t div) : d(div), mul(0), shr(0) {
        if (div > 1) {
            uint32_t lg = 0;
            while ((1ull << lg) < div) ++lg;
            const uint32_t p = 31 + lg;
            mul = static_cast<uint32_t>(((1ull << p) + div - 1) / div);
            shr = p - 32;
        }
    }
    // n < 2^31
    __device__ __forceinline__ uint32_t div(uint32_t n) const { return d == 1 ? n : (__umulhi(n, mul) >> shr); }
    __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const { q = div(n); r = n - q * d; }
};

// ------------------------------------------------------------------------------------------------
// Counter-based hash RNG.  The value depends only on (counter, seed), never on launch geometry, so
// that recomputation and different chunkings reproduce the same rounding decisions.
__device__ __forceinline__ uint32_t hash_u32(uint32_t x) {
    x ^= x >> 16; x *= 0x7feb352du;
    x ^= x >> 15; x *= 0x846ca68bu;
    x ^= x >> 16;
    return x;
}
__device__ __forceinline__ uint32_t rng_u32(uint64_t counter, uint32_t seed) {
    uint32_t lo = static_cast<uint32_t>(counter), hi = static_cast<uint32_t>(counter >> 32);
    return hash_u32(lo ^ hash_u32(hi + 0x9e3779b9u * (seed + 1u)) ^ (seed * 0x85ebca6bu));
}

// Stochastic rounding fp32 -> bf16: add 16 random bits below the bf16 mantissa and truncate.
__device__ __forceinline__ bf16 sr_bf16(float x, uint32_t rnd) {
    uint32_t bits = __float_as_uint(x);
    if ((bits & 0x7f800000u) == 0x7f800000u) return __float2bfloat16_rn(x);   // inf / nan
    bits += (rnd & 0xFFFFu);
    bits &= 0xFFFF0000u;
    return __float2bfloat16_rn(__uint_as_float(bits));    // exact
}
// Stochastic rounding to e4m3 of a value already scaled into the representable range.
__device__ __forceinline__ e4m3 sr_e4m3(float x, uint32_t rnd) {
    // e4m3 has 3 mantissa bits: make the rounding increment relative to the fp32 exponent
    float ax = fabsf(x);
    if (!(ax < 448.f)) return e4m3(x);
    if (ax < 0.015625f) {                 // subnormal range: fixed quantum 2^-9
        float q = 0.001953125f;
        float lo = floorf(x / q) * q;
        float frac = (x - lo) / q;
        float u = (rnd >> 8) * (1.0f / 16777216.0f);
        return e4m3(frac > u ? lo + q : lo);
    }
    uint32_t bits = __float_as_uint(x);
    bits += (rnd & 0xFFFFFu);             // 20 dropped mantissa bits
    bits &= 0xFFF00000u;
    return e4m3(__uint_as_float(bits));
}
template <typename T> __device__ __forceinline__ T sr_round(float x, uint32_t rnd);
template <> __device__ __forceinline__ float sr_round<float>(float x, uint32_t) { return x; }
template <> __device__ __forceinline__ bf16 sr_round<bf16>(float x, uint32_t rnd) { return sr_bf16(x, rnd); }

__device__ __forceinline__ float fast_sigmoid(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
