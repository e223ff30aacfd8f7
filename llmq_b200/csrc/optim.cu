// Optimiser-side kernels: AdamW with stochastic rounding (bf16 / fp32 / block-scaled e4m3 moments),
// global gradient norm with a deterministic reduction, and the stochastic-rounding vector add / reduce
// used for sharded gradient accumulation.
// Behavioural counterparts of src/kernels/{adamw,global_norm,vector_add}.cu of the reference.
#include <cstring>
#include "api.h"
#include "common.cuh"

namespace {

int grid_for(long long work_items, int threads, int num_sms) {
    long long blocks = ceil_div_ll(work_items, threads);
    long long cap = static_cast<long long>(num_sms) * 8;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

template <typename T> __device__ __forceinline__ void load8(float (&f)[8], const T* p);
template <> __device__ __forceinline__ void load8<bf16>(float (&f)[8], const bf16* p) {
    Vec16<bf16> v = Vec16<bf16>::load(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = __bfloat162float(v.v[i]);
}
template <> __device__ __forceinline__ void load8<float>(float (&f)[8], const float* p) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
template <> __device__ __forceinline__ void load8<e4m3>(float (&f)[8], const e4m3* p) {
    uint2 raw = *reinterpret_cast<const uint2*>(p);
    const e4m3* q = reinterpret_cast<const e4m3*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(q[i]);
}
template <typename T> __device__ __forceinline__ void store8_sr(T* p, const float (&f)[8], uint64_t ctr, uint32_t seed);
template <> __device__ __forceinline__ void store8_sr<bf16>(bf16* p, const float (&f)[8], uint64_t ctr, uint32_t seed) {
    Vec16<bf16> v;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        uint32_t r = rng_u32(ctr + i / 2, seed);         // 16 random bits per element
        v.v[i] = sr_bf16(f[i], r);
        v.v[i + 1] = sr_bf16(f[i + 1], r >> 16);
    }
    v.store(p);
}
template <> __device__ __forceinline__ void store8_sr<float>(float* p, const float (&f)[8], uint64_t, uint32_t) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// Random words for one thread-iteration (8 elements x {param, m, v}): one full hash of the element counter,
// then cheap multiply / xor-shift steps.  Depends only on (element index, seed), never on launch geometry.
struct SrWords {
    uint32_t h;
    __device__ __forceinline__ SrWords(uint64_t ctr, uint32_t seed) : h(rng_u32(ctr, seed)) {}
    __device__ __forceinline__ uint32_t get(uint32_t j) const {
        uint32_t x = (h + j * 0x9e3779b9u) * 0x85ebca6bu;
        x ^= x >> 15;
        x *= 0xc2b2ae35u;
        return x ^ (x >> 16);
    }
};
__device__ __forceinline__ float sqrt_approx(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
template <typename T> __device__ __forceinline__ void store8_srw(T* p, const float (&f)[8], const SrWords& w, uint32_t j0);
template <> __device__ __forceinline__ void store8_srw<bf16>(bf16* p, const float (&f)[8], const SrWords& w, uint32_t j0) {
    Vec16<bf16> v;
#pragma unroll
    for (int i = 0; i < 8; i += 2) {
        const uint32_t r = w.get(j0 + i / 2);
        v.v[i] = sr_bf16(f[i], r);
        v.v[i + 1] = sr_bf16(f[i + 1], r >> 16);
    }
    v.store(p);
}
template <> __device__ __forceinline__ void store8_srw<float>(float* p, const float (&f)[8], const SrWords&, uint32_t) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}

// One thread updates 8 consecutive parameters.  For e4m3 first moments 16 consecutive threads share one
// fp32 scale (128 elements); the scale is recomputed from the new values every step.
template <typename P, typename G, typename M, typename Vv>
__global__ void __launch_bounds__(256)
adamw_kernel(P* __restrict__ param, const G* __restrict__ grad, M* __restrict__ m_state, Vv* __restrict__ v_state,
             float* __restrict__ m_scales, long long n, float lr, float beta1, float beta2, float bc1, float bc2, float eps,
             float wd, const float* __restrict__ grad_scale, float* __restrict__ absmax_out, uint32_t seed, long long elem_offset,
             const float* __restrict__ hyper) {
    __shared__ float scratch[32];
    if (hyper) {
        // Step-dependent scalars from device memory: {lr, beta1, beta2, 1/(1-beta1^t), 1/(1-beta2^t), eps, weight decay,
        // seed bits}.  The launch itself is then the same every step and can be replayed from a CUDA graph; `wd` of the
        // launch selects (non-zero) or masks (zero) the weight decay, `seed` is added to the step's seed.
        lr = hyper[0]; beta1 = hyper[1]; beta2 = hyper[2]; bc1 = hyper[3]; bc2 = hyper[4]; eps = hyper[5];
        wd = wd != 0.f ? hyper[6] : 0.f;
        seed += __float_as_uint(hyper[7]);
    }
    const float gs = grad_scale ? *grad_scale : 1.f;
    float tmax = 0.f;
    const long long nvec = n / 8;
    const long long stride = static_cast<long long>(gridDim.x) * blockDim.x;
    // all threads of a 16-lane group must iterate together for the e4m3 path: round the loop bound up
    const long long nvec_pad = (nvec + 31) / 32 * 32;       // whole warps take part in the shuffles
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec_pad; i += stride) {
        const bool active = i < nvec;
        const long long e = i * 8;
        float p[8], g[8], m[8], v[8];
        if (active) {
            load8<P>(p, param + e);
            load8<G>(g, grad + e);
            load8<Vv>(v, v_state + e);
            load8<M>(m, m_state + e);
            if constexpr (sizeof(M) == 1) {
                float sc = m_scales[e / 128];
#pragma unroll
                for (int k = 0; k < 8; ++k) m[k] *= sc;
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) { p[k] = g[k] = m[k] = v[k] = 0.f; }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            float gk = g[k] * gs;
            m[k] = beta1 * m[k] + (1.f - beta1) * gk;
            v[k] = beta2 * v[k] + (1.f - beta2) * gk * gk;
            float mh = m[k] * bc1, vh = v[k] * bc2;
            p[k] -= lr * (__fdividef(mh, sqrt_approx(vh) + eps) + wd * p[k]);
        }
        const uint64_t ctr = static_cast<uint64_t>(e + elem_offset);
        const SrWords words(ctr, seed);
        if constexpr (sizeof(M) == 1) {
            float am = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) am = fmaxf(am, fabsf(m[k]));
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) am = fmaxf(am, __shfl_xor_sync(0xffffffffu, am, o));
            float sc = fmaxf(am, 1e-30f) / 448.f;
            if (active) {
                alignas(8) e4m3 q[8];
                float inv = 1.f / sc;
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    q[k] = sr_e4m3(m[k] * inv, words.get(4 + k));
                    q[k + 1] = sr_e4m3(m[k + 1] * inv, words.get(5 + k));
                }
                *reinterpret_cast<uint2*>(m_state + e) = *reinterpret_cast<uint2*>(q);
                if ((i & 15) == 0) m_scales[e / 128] = sc;
            }
        } else {
            if (active) store8_srw<M>(m_state + e, m, words, 4);
        }
        if (active) {
            store8_srw<Vv>(v_state + e, v, words, 12);
            if constexpr (sizeof(P) == 2) {
                Vec16<bf16> o;
#pragma unroll
                for (int k = 0; k < 8; k += 2) {
                    uint32_t r = words.get(k / 2);
                    o.v[k] = sr_bf16(p[k], r);
                    o.v[k + 1] = sr_bf16(p[k + 1], r >> 16);
                    tmax = fmaxf(tmax, fmaxf(fabsf(__bfloat162float(o.v[k])), fabsf(__bfloat162float(o.v[k + 1]))));
                }
                o.store(reinterpret_cast<bf16*>(param) + e);
            } else {
                store8_srw<float>(reinterpret_cast<float*>(param) + e, p, words, 0);
#pragma unroll
                for (int k = 0; k < 8; ++k) tmax = fmaxf(tmax, fabsf(p[k]));
            }
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// Sum of squares; block b adds its partial to out[b], so several tensors accumulate into the same
// partial vector in stream order and the result does not depend on atomics.
template <typename T>
__global__ void __launch_bounds__(512) norm_squared_kernel(float* __restrict__ out, const T* __restrict__ x, long long n) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    float s = 0.f;
    const long long nvec = n / V::N;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        V v = V::load(x + i * V::N);
#pragma unroll
        for (int k = 0; k < V::N; ++k) { float f = to_float(v.v[k]); s += f * f; }
    }
    if (blockIdx.x == 0)
        for (long long i = nvec * V::N + threadIdx.x; i < n; i += blockDim.x) { float f = to_float(x[i]); s += f * f; }
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) out[blockIdx.x] += s;
}

__global__ void __launch_bounds__(512) deterministic_sum_kernel(float* __restrict__ out, const float* __restrict__ in, int n) {
    __shared__ float scratch[32];
    float s = 0.f;
    for (int i = threadIdx.x; i < n; i += blockDim.x) s += in[i];
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) *out = s;
}

// io[0]: squared norm in -> norm out;  io[1]: multiplier that clips the gradient to `clip` (1 if no clipping)
__global__ void norm_finish_kernel(float* io, float clip, float* host_norm) {
    float nsq = io[0];
    float norm = sqrtf(nsq);
    float scale = 1.f;
    if (clip > 0.f && norm > clip) scale = clip / norm;
    if (!isfinite(norm)) scale = 0.f;          // a non-finite gradient must not reach the weights
    io[0] = norm;
    io[1] = scale;
    if (host_norm) *host_norm = norm;
}

// dst = SR(scale * (a + b))
template <typename T>
__global__ void __launch_bounds__(512)
vector_add_sr_kernel(T* dst, const T* a, const T* b, float scale, long long n, uint32_t seed) {
    const long long nvec = n / 8;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float fa[8], fb[8];
        load8<T>(fa, a + i * 8);
        load8<T>(fb, b + i * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) fa[k] = scale * (fa[k] + fb[k]);
        store8_sr<T>(dst + i * 8, fa, static_cast<uint64_t>(i * 8), seed);
    }
}

// dst = SR(scale * (sum_{k != skip} src[k * shard_stride + i] (+ dst[i] if accumulate)))
template <typename T>
__global__ void __launch_bounds__(512)
vector_reduce_sr_kernel(T* dst, const T* src, float scale, int n_shards, int skip, long long shard_stride, int accumulate,
                        long long n, uint32_t seed) {
    const long long nvec = n / 8;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        if (accumulate) load8<T>(acc, dst + i * 8);
        for (int sh = 0; sh < n_shards; ++sh) {
            if (sh == skip) continue;
            float f[8];
            load8<T>(f, src + sh * shard_stride + i * 8);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += f[k];
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] *= scale;
        store8_sr<T>(dst + i * 8, acc, static_cast<uint64_t>(i * 8), seed);
    }
}

}  // namespace

// dtype codes: param/grad: 0 bf16 | 3 fp32;  m: 0 | 3 | 1 (e4m3, needs m_scales and n % 128 == 0);  v: 0 | 3
extern "C" int llmq_adamw_hyper(void*, const void*, void*, void*, float*, long long, float, float, float, int, float, float, const float*, float*,
                                unsigned int, long long, int, int, int, int, int, const float*, cudaStream_t);

extern "C" int llmq_adamw(void* param, const void* grad, void* m, void* v, float* m_scales, long long n, float lr, float beta1,
                          float beta2, int step, float eps, float wd, const float* grad_scale, float* absmax_out,
                          unsigned int seed, long long elem_offset, int p_dtype, int g_dtype, int m_dtype, int v_dtype,
                          int num_sms, cudaStream_t s) {
    return llmq_adamw_hyper(param, grad, m, v, m_scales, n, lr, beta1, beta2, step, eps, wd, grad_scale, absmax_out, seed, elem_offset,
                            p_dtype, g_dtype, m_dtype, v_dtype, num_sms, nullptr, s);
}

// Fills the 8 host floats that `hyper` points the kernel at, with the same arithmetic as the by-value launch.
extern "C" void llmq_adamw_fill_hyper(float* out, float lr, float beta1, float beta2, int step, float eps, float wd, unsigned int seed) {
    out[0] = lr; out[1] = beta1; out[2] = beta2;
    out[3] = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
    out[4] = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
    out[5] = eps; out[6] = wd;
    memcpy(out + 7, &seed, sizeof(seed));
}

// Same, with the step-dependent scalars optionally read from 8 floats in device memory (see adamw_kernel).
extern "C" int llmq_adamw_hyper(void* param, const void* grad, void* m, void* v, float* m_scales, long long n, float lr, float beta1,
                                float beta2, int step, float eps, float wd, const float* grad_scale, float* absmax_out,
                                unsigned int seed, long long elem_offset, int p_dtype, int g_dtype, int m_dtype, int v_dtype,
                                int num_sms, const float* hyper, cudaStream_t s) {
    if (n <= 0) return 0;
    if (n % 8) return -1;
    if (m_dtype == 1 && (n % 128 || !m_scales)) return -2;
    const float bc1 = 1.f / (1.f - powf(beta1, static_cast<float>(step)));
    const float bc2 = 1.f / (1.f - powf(beta2, static_cast<float>(step)));
    int g = grid_for(n / 8, 256, num_sms);
#define A_CASE(P, PC, G, GC, M, MC, V, VC)                                                                          \
    if (p_dtype == PC && g_dtype == GC && m_dtype == MC && v_dtype == VC) {                                         \
        adamw_kernel<P, G, M, V><<<g, 256, 0, s>>>(static_cast<P*>(param), static_cast<const G*>(grad), static_cast<M*>(m), \
                                                   static_cast<V*>(v), m_scales, n, lr, beta1, beta2, bc1, bc2, eps, wd,   \
                                                   grad_scale, absmax_out, seed, elem_offset, hyper);               \
        return LLMQ_LAUNCH_CHECK();                                                                                 \
    }
    A_CASE(bf16, 0, bf16, 0, bf16, 0, bf16, 0)
    A_CASE(bf16, 0, bf16, 0, float, 3, float, 3)
    A_CASE(bf16, 0, bf16, 0, float, 3, bf16, 0)
    A_CASE(bf16, 0, bf16, 0, bf16, 0, float, 3)
    A_CASE(bf16, 0, bf16, 0, e4m3, 1, bf16, 0)
    A_CASE(bf16, 0, bf16, 0, e4m3, 1, float, 3)
    A_CASE(float, 3, float, 3, float, 3, float, 3)
    A_CASE(float, 3, float, 3, bf16, 0, bf16, 0)
    A_CASE(float, 3, bf16, 0, float, 3, float, 3)
    A_CASE(float, 3, bf16, 0, bf16, 0, bf16, 0)
#undef A_CASE
    return -10;
}

extern "C" int llmq_norm_squared(float* partials, const void* x, long long n, int dtype, int num_partials, cudaStream_t s) {
    if (n <= 0) return 0;
    if (dtype == 0) norm_squared_kernel<bf16><<<num_partials, 512, 0, s>>>(partials, static_cast<const bf16*>(x), n);
    else if (dtype == 3) norm_squared_kernel<float><<<num_partials, 512, 0, s>>>(partials, static_cast<const float*>(x), n);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_deterministic_sum(float* out, const float* in, int n, cudaStream_t s) {
    deterministic_sum_kernel<<<1, 512, 0, s>>>(out, in, n);
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_norm_finish(float* io, float clip, float* host_norm, cudaStream_t s) {
    norm_finish_kernel<<<1, 1, 0, s>>>(io, clip, host_norm);
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_vector_add_sr(void* dst, const void* a, const void* b, float scale, long long n, unsigned int seed, int dtype,
                                  int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    if (n % 8) return -1;
    int g = grid_for(n / 8, 512, num_sms);
    if (dtype == 0) vector_add_sr_kernel<bf16><<<g, 512, 0, s>>>(static_cast<bf16*>(dst), static_cast<const bf16*>(a), static_cast<const bf16*>(b), scale, n, seed);
    else if (dtype == 3) vector_add_sr_kernel<float><<<g, 512, 0, s>>>(static_cast<float*>(dst), static_cast<const float*>(a), static_cast<const float*>(b), scale, n, seed);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_vector_reduce_sr(void* dst, const void* src, float scale, int n_shards, int skip, long long shard_stride,
                                     int accumulate, long long n, unsigned int seed, int dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    if (n % 8) return -1;
    int g = grid_for(n / 8, 512, num_sms);
    if (dtype == 0) vector_reduce_sr_kernel<bf16><<<g, 512, 0, s>>>(static_cast<bf16*>(dst), static_cast<const bf16*>(src), scale, n_shards, skip, shard_stride, accumulate, n, seed);
    else if (dtype == 3) vector_reduce_sr_kernel<float><<<g, 512, 0, s>>>(static_cast<float*>(dst), static_cast<const float*>(src), scale, n_shards, skip, shard_stride, accumulate, n, seed);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}
