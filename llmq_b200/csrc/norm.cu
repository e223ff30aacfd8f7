// RMSNorm kernels: (fused residual +) RMSNorm forward with abs-max / direct fp8 emission, and the
// backward pass with a deterministic weight-gradient reduction.
// Behavioural counterpart of src/kernels/rmsnorm.cu:17-460 in the reference: y = T(x * rstd) * w with
// the intermediate rounded to the storage type (matches the HF modelling code), abs-max of y fused.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int NORM_THREADS = 256;

// One CTA per token row.  Pass 1 reads the row (adding the two residual inputs when fused, and writing
// the sum), pass 2 re-reads it from L1/L2 to normalise.  HBM traffic is one read + one write per tensor.
template <typename T>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_fwd_kernel(T* __restrict__ residual_out,      // may be null when not fused
                   T* __restrict__ y_out,             // may be null when only fp8 output is wanted
                   e4m3* __restrict__ q_out,          // optional direct fp8 output (needs known abs-max)
                   float* __restrict__ rstd_out,
                   const T* __restrict__ in_a, const T* __restrict__ in_b,   // in_b null -> plain norm of in_a
                   const T* __restrict__ weight, float eps, int C,
                   float* __restrict__ absmax_out, const float* __restrict__ known_absmax,
                   float* __restrict__ q_scale_out) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    const long long row = blockIdx.x;
    const T* a = in_a + row * C;
    const T* b = in_b ? in_b + row * C : nullptr;
    T* res = residual_out ? residual_out + row * C : nullptr;
    const T* x = res ? res : a;

    float ss = 0.f;
    for (int c = threadIdx.x * V::N; c < C; c += NORM_THREADS * V::N) {
        V va = V::load(a + c);
        if (b) {
            V vb = V::load_stream(b + c);
#pragma unroll
            for (int i = 0; i < V::N; ++i) va.v[i] = from_float<T>(to_float(va.v[i]) + to_float(vb.v[i]));
        }
        if (res) va.store(res + c);
#pragma unroll
        for (int i = 0; i < V::N; ++i) { float f = to_float(va.v[i]); ss += f * f; }
    }
    ss = block_reduce_sum(ss, scratch);     // contains __syncthreads: the residual writes are visible below
    const float rstd = rsqrtf(ss / C + eps);
    if (threadIdx.x == 0 && rstd_out) rstd_out[row] = rstd;

    float qmul = 0.f;
    if (q_out) {
        float am = fmaxf(*known_absmax, 1e-10f);
        qmul = 448.f / am;
        if (row == 0 && threadIdx.x == 0 && q_scale_out) *q_scale_out = am / 448.f;
    }
    float tmax = 0.f;
    for (int c = threadIdx.x * V::N; c < C; c += NORM_THREADS * V::N) {
        V vx = V::load(x + c);
        V vw = V::load(weight + c);
        V vy;
        alignas(8) e4m3 q[V::N];
#pragma unroll
        for (int i = 0; i < V::N; ++i) {
            T n = from_float<T>(to_float(vx.v[i]) * rstd);
            vy.v[i] = from_float<T>(to_float(n) * to_float(vw.v[i]));
            float f = to_float(vy.v[i]);
            tmax = fmaxf(tmax, fabsf(f));
            if (q_out) q[i] = e4m3(f * qmul);
        }
        if (y_out) vy.store(y_out + row * C + c);
        if (q_out) {
            if constexpr (V::N == 8) *reinterpret_cast<uint2*>(q_out + row * C + c) = *reinterpret_cast<uint2*>(q);
            else *reinterpret_cast<uint32_t*>(q_out + row * C + c) = *reinterpret_cast<uint32_t*>(q);
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// Backward.  Persistent CTAs walk over rows; each thread owns up to VPT 16-byte column vectors and keeps
// its share of the weight gradient in registers.  Partials go to scratch[gridDim.x][C] and a second
// kernel sums them in a fixed order (deterministic, no atomics).
template <typename T, int VPT>
__global__ void __launch_bounds__(NORM_THREADS)
rmsnorm_bwd_kernel(T* __restrict__ dinp,               // in: upstream residual gradient, out: += norm gradient
                   float* __restrict__ dw_partial,     // [gridDim.x, C]
                   const T* __restrict__ dout, const T* __restrict__ inp, const T* __restrict__ weight,
                   const float* __restrict__ rstd, int rows, int C, float* __restrict__ absmax_out) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    float dw[VPT][V::N];
#pragma unroll
    for (int k = 0; k < VPT; ++k)
#pragma unroll
        for (int i = 0; i < V::N; ++i) dw[k][i] = 0.f;
    float tmax = 0.f;

    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* dy = dout + row * C;
        const T* x = inp + row * C;
        T* dx = dinp + row * C;
        const float rs = rstd[row];
        // pass 1: dot = sum(w * dy * xhat)
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            int c = (k * NORM_THREADS + threadIdx.x) * V::N;
            if (c < C) {
                V vdy = V::load(dy + c), vx = V::load(x + c), vw = V::load(weight + c);
#pragma unroll
                for (int i = 0; i < V::N; ++i) {
                    float xh = to_float(vx.v[i]) * rs;
                    float g = to_float(vdy.v[i]);
                    dot += to_float(vw.v[i]) * g * xh;
                    dw[k][i] += g * xh;
                }
            }
        }
        dot = block_reduce_sum(dot, scratch) / C;
        // pass 2 (operands are L1/L2 resident)
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            int c = (k * NORM_THREADS + threadIdx.x) * V::N;
            if (c < C) {
                V vdy = V::load(dy + c), vx = V::load(x + c), vw = V::load(weight + c), vd = V::load(dx + c);
#pragma unroll
                for (int i = 0; i < V::N; ++i) {
                    float xh = to_float(vx.v[i]) * rs;
                    float g = (to_float(vw.v[i]) * to_float(vdy.v[i]) - xh * dot) * rs;
                    float r = to_float(vd.v[i]) + g;
                    vd.v[i] = from_float<T>(r);
                    tmax = fmaxf(tmax, fabsf(to_float(vd.v[i])));
                }
                vd.store(dx + c);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        int c = (k * NORM_THREADS + threadIdx.x) * V::N;
        if (c < C) {
#pragma unroll
            for (int i = 0; i < V::N; ++i) dw_partial[static_cast<long long>(blockIdx.x) * C + c + i] = dw[k][i];
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// Same contract, for rows of up to 4 column vectors per thread: the row's dout, inp and residual gradient are
// loaded once and stay in registers across the block-wide dot product (no second pass over L1 / L2), the norm
// weights are loaded once per CTA, and three CTAs share an SM so that their reductions overlap.
template <typename T, int VPT>
__global__ void __launch_bounds__(NORM_THREADS, VPT <= 2 ? 3 : 2)
rmsnorm_bwd_reg_kernel(T* __restrict__ dinp, float* __restrict__ dw_partial, const T* __restrict__ dout, const T* __restrict__ inp,
                       const T* __restrict__ weight, const float* __restrict__ rstd, int rows, int C, float* __restrict__ absmax_out) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    float dw[VPT][V::N];
    V vw[VPT];
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = (k * NORM_THREADS + threadIdx.x) * V::N;
        if (c < C) vw[k] = V::load(weight + c);
#pragma unroll
        for (int i = 0; i < V::N; ++i) dw[k][i] = 0.f;
    }
    float tmax = 0.f;
    const float inv_c = 1.f / C;
    for (long long row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* dy = dout + row * C;
        const T* x = inp + row * C;
        T* dx = dinp + row * C;
        V vdy[VPT], vx[VPT], vd[VPT];
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int c = (k * NORM_THREADS + threadIdx.x) * V::N;
            if (c < C) { vdy[k] = V::load_stream(dy + c); vx[k] = V::load_stream(x + c); vd[k] = V::load(dx + c); }
        }
        const float rs = rstd[row];
        float dot = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int c = (k * NORM_THREADS + threadIdx.x) * V::N;
            if (c < C) {
#pragma unroll
                for (int i = 0; i < V::N; ++i) {
                    const float xh = to_float(vx[k].v[i]) * rs;
                    const float g = to_float(vdy[k].v[i]);
                    dot += to_float(vw[k].v[i]) * g * xh;
                    dw[k][i] += g * xh;
                }
            }
        }
        dot = block_reduce_sum(dot, scratch) * inv_c;
#pragma unroll
        for (int k = 0; k < VPT; ++k) {
            const int c = (k * NORM_THREADS + threadIdx.x) * V::N;
            if (c < C) {
#pragma unroll
                for (int i = 0; i < V::N; ++i) {
                    const float xh = to_float(vx[k].v[i]) * rs;
                    const float g = (to_float(vw[k].v[i]) * to_float(vdy[k].v[i]) - xh * dot) * rs;
                    vd[k].v[i] = from_float<T>(to_float(vd[k].v[i]) + g);
                    tmax = fmaxf(tmax, fabsf(to_float(vd[k].v[i])));
                }
                vd[k].store(dx + c);
            }
        }
    }
#pragma unroll
    for (int k = 0; k < VPT; ++k) {
        const int c = (k * NORM_THREADS + threadIdx.x) * V::N;
        if (c < C) {
#pragma unroll
            for (int i = 0; i < V::N; ++i) dw_partial[static_cast<long long>(blockIdx.x) * C + c + i] = dw[k][i];
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// Column sums of the per-CTA partial rows.  A CTA owns 64 columns; its 16 thread rows walk the partial rows with a stride
// of 16 (28 loads per thread for 444 partial rows instead of 444 dependent loads in one thread) and are summed through
// shared memory in a fixed order, so the result does not depend on the schedule.
constexpr int RED_COLS = 64, RED_GROUPS = 16;
template <typename T>
__global__ void __launch_bounds__(RED_COLS * RED_GROUPS)
rmsnorm_bwd_reduce_kernel(T* __restrict__ dweight, const float* __restrict__ dw_partial, int nparts, int C, int accumulate) {
    __shared__ float part[RED_GROUPS][RED_COLS];
    const int x = threadIdx.x % RED_COLS, y = threadIdx.x / RED_COLS;
    const int c = blockIdx.x * RED_COLS + x;
    float s = 0.f;
    if (c < C) {
#pragma unroll 4
        for (int p = y; p < nparts; p += RED_GROUPS) s += dw_partial[static_cast<long long>(p) * C + c];
    }
    part[y][x] = s;
    __syncthreads();
    if (y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int g = 0; g < RED_GROUPS; ++g) t += part[g][x];
        if (accumulate) t += to_float(dweight[c]);
        dweight[c] = from_float<T>(t);
    }
}

template <typename T>
int launch_fwd(void* residual_out, void* y_out, void* q_out, float* rstd, const void* a, const void* b, const void* w,
               float eps, int rows, int C, float* absmax, const float* known_absmax, float* q_scale, cudaStream_t s) {
    if (C % Vec16<T>::N) return -1;
    rmsnorm_fwd_kernel<T><<<rows, NORM_THREADS, 0, s>>>(static_cast<T*>(residual_out), static_cast<T*>(y_out),
                                                        static_cast<e4m3*>(q_out), rstd, static_cast<const T*>(a),
                                                        static_cast<const T*>(b), static_cast<const T*>(w), eps, C, absmax,
                                                        known_absmax, q_scale);
    return LLMQ_LAUNCH_CHECK();
}

template <typename T>
int launch_bwd(void* dinp, void* dweight, float* scratch, const void* dout, const void* inp, const void* w,
               const float* rstd, int rows, int C, float* absmax, int accumulate_dw, int num_blocks, cudaStream_t s) {
    using V = Vec16<T>;
    if (C % V::N) return -1;
    int vecs = ceil_div_i(C / V::N, NORM_THREADS);
    if (num_blocks > rows) num_blocks = rows;
#define LAUNCH(VPT)                                                                                                   \
    rmsnorm_bwd_kernel<T, VPT><<<num_blocks, NORM_THREADS, 0, s>>>(static_cast<T*>(dinp), scratch,                    \
                                                                   static_cast<const T*>(dout), static_cast<const T*>(inp), \
                                                                   static_cast<const T*>(w), rstd, rows, C, absmax)
#define LAUNCH_REG(VPT)                                                                                               \
    rmsnorm_bwd_reg_kernel<T, VPT><<<num_blocks, NORM_THREADS, 0, s>>>(static_cast<T*>(dinp), scratch,                \
                                                                       static_cast<const T*>(dout), static_cast<const T*>(inp), \
                                                                       static_cast<const T*>(w), rstd, rows, C, absmax)
    if (vecs <= 1) LAUNCH_REG(1);
    else if (vecs <= 2) LAUNCH_REG(2);
    else if (vecs <= 4) LAUNCH_REG(4);
    else if (vecs <= 8) LAUNCH(8);
    else return -2;
#undef LAUNCH
#undef LAUNCH_REG
    int rc = LLMQ_LAUNCH_CHECK();
    if (rc) return rc;
    rmsnorm_bwd_reduce_kernel<T><<<ceil_div_i(C, RED_COLS), RED_COLS * RED_GROUPS, 0, s>>>(static_cast<T*>(dweight), scratch, num_blocks, C, accumulate_dw);
    return LLMQ_LAUNCH_CHECK();
}

}  // namespace

extern "C" int llmq_rmsnorm_forward(void* residual_out, void* y_out, void* q_out, float* rstd, const void* in_a,
                                    const void* in_b, const void* weight, float eps, int rows, int C, int dtype,
                                    float* absmax, const float* known_absmax, float* q_scale, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == 0) return launch_fwd<bf16>(residual_out, y_out, q_out, rstd, in_a, in_b, weight, eps, rows, C, absmax, known_absmax, q_scale, stream);
    if (dtype == 3) return launch_fwd<float>(residual_out, y_out, q_out, rstd, in_a, in_b, weight, eps, rows, C, absmax, known_absmax, q_scale, stream);
    return -10;
}

// scratch must hold num_blocks * C floats.
extern "C" int llmq_rmsnorm_backward(void* dinp, void* dweight, float* scratch, const void* dout, const void* inp,
                                     const void* weight, const float* rstd, int rows, int C, int dtype, float* absmax,
                                     int accumulate_dweight, int num_blocks, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (dtype == 0) return launch_bwd<bf16>(dinp, dweight, scratch, dout, inp, weight, rstd, rows, C, absmax, accumulate_dweight, num_blocks, stream);
    if (dtype == 3) return launch_bwd<float>(dinp, dweight, scratch, dout, inp, weight, rstd, rows, C, absmax, accumulate_dweight, num_blocks, stream);
    return -10;
}

// ------------------------------------------------------------------------------------------------
// RMSNorm backward for callers that must not allocate (see noalloc.h).
//
// The weight-gradient partials live in a file-scope device array instead of a caller-provided buffer.
// Every GPU that loads this library keeps the array resident until the process exits.
#include "noalloc.h"
#include <mutex>

static __device__ __align__(256) float g_noalloc_norm_scratch[LLMQ_NOALLOC_SCRATCH_FLOATS];

namespace {
std::mutex g_noalloc_mutex;
float* g_noalloc_scratch_ptr[64] = {};     // device address of the array, per device ordinal
}  // namespace

extern "C" int llmq_rmsnorm_backward_noalloc(void* dinp, void* dweight, const void* dout, const void* inp,
                                             const void* weight, const float* rstd, int rows, int C, int dtype,
                                             float* absmax, int accumulate_dweight, cudaStream_t stream) {
    if (rows <= 0) return 0;
    if (C <= 0 || C > LLMQ_NOALLOC_MAX_C) return LLMQ_NOALLOC_ERR_TOO_LARGE;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (dev < 0 || dev >= 64) return LLMQ_NOALLOC_ERR_DEVICE;
    float* scratch = nullptr;
    int sms = 0;
    {
        // One-time set-up per device, with that device current.  In host code the array's name is only a
        // handle for the runtime; the address a kernel can use comes from cudaGetSymbolAddress.
        std::lock_guard<std::mutex> lock(g_noalloc_mutex);
        if (!g_noalloc_scratch_ptr[dev]) {
            void* p = nullptr;
            e = cudaGetSymbolAddress(&p, g_noalloc_norm_scratch);
            if (e != cudaSuccess) return static_cast<int>(e);
            g_noalloc_scratch_ptr[dev] = static_cast<float*>(p);
        }
        scratch = g_noalloc_scratch_ptr[dev];
    }
    e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess) return static_cast<int>(e);
    // as many row-walking CTAs as the array can hold partial rows for, at most two per SM
    long long blocks = 2LL * sms;
    const long long fit = LLMQ_NOALLOC_SCRATCH_FLOATS / C;
    if (blocks > fit) blocks = fit;
    if (blocks < 1) return LLMQ_NOALLOC_ERR_TOO_LARGE;
    if (dtype == 0) return launch_bwd<bf16>(dinp, dweight, scratch, dout, inp, weight, rstd, rows, C, absmax, accumulate_dweight, static_cast<int>(blocks), stream);
    if (dtype == 3) return launch_bwd<float>(dinp, dweight, scratch, dout, inp, weight, rstd, rows, C, absmax, accumulate_dweight, static_cast<int>(blocks), stream);
    return -10;
}
