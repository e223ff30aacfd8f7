// Fused softmax cross-entropy over the vocabulary with in-place logit gradients, plus the small
// statistics kernels that go with it (per-position loss groups, log-sum-exp monitoring).
// Behavioural counterpart of src/kernels/fused_classifier.cu:20-342 and fused_classifier_tma.cu:40-273:
//   loss[row] += lse - logit[target];   dlogit = p * (dloss + z_reg * lse) - 1[target] * dloss;
//   rows whose target is -100 - or any other id outside [0, V), e.g. from a token file of a larger tokenizer - get
//   zero loss and zero gradient; the id never indexes memory.
// One CTA of 1024 threads owns a row.  Pass 1 streams the row once and keeps an online (max, sum);
// pass 2 re-reads the row (still L2 resident: a bf16 row of 152k logits is 300 KB) and overwrites it
// with the gradient using streaming stores, so HBM sees one read and one write per logit.
#include "api.h"
#include "common.cuh"

namespace {

constexpr int CE_THREADS = 1024;

template <typename T>
__global__ void __launch_bounds__(CE_THREADS, 1)
fused_ce_kernel(T* logits, float* __restrict__ losses, float* __restrict__ lse_out, const int* __restrict__ targets,
                float dloss, float z_reg, int rows, int V, long long ld, int write_dlogits) {
    __shared__ float s_max[32], s_sum[32];
    using Vt = Vec16<T>;
    const long long row = rows - 1 - static_cast<long long>(blockIdx.x);   // newest GEMM output first: L2 hits
    T* x = logits + row * ld;
    const int tgt = targets[row];
    const int nvec = V / Vt::N;
    if (tgt < 0 || tgt >= V) {                  // -100 = masked; other out-of-range ids are treated the same way
        if (write_dlogits) {
            Vt z;
#pragma unroll
            for (int k = 0; k < Vt::N; ++k) z.v[k] = from_float<T>(0.f);
            for (int i = threadIdx.x; i < nvec; i += CE_THREADS) z.store_stream(x + i * Vt::N);
            for (int i = nvec * Vt::N + threadIdx.x; i < V; i += CE_THREADS) x[i] = from_float<T>(0.f);
        }
        if (threadIdx.x == 0 && lse_out) lse_out[row] = 0.f;
        return;
    }
    constexpr float kLog2e = 1.4426950408889634f;
    // pass 1: online max / sum (base-2 domain)
    float m = -INFINITY, s = 0.f;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        Vt v = Vt::load(x + i * Vt::N);
        float lm = -INFINITY;
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) lm = fmaxf(lm, to_float(v.v[k]));
        if (lm > m) { s *= exp2f((m - lm) * kLog2e); m = lm; }
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) s += exp2f((to_float(v.v[k]) - m) * kLog2e);
    }
    for (int i = nvec * Vt::N + threadIdx.x; i < V; i += CE_THREADS) {
        float f = to_float(x[i]);
        if (f > m) { s *= exp2f((m - f) * kLog2e); m = f; }
        s += exp2f((f - m) * kLog2e);
    }
    // combine (max, sum) pairs across the block
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
        float nm = fmaxf(m, om);
        s = (m == -INFINITY ? 0.f : s * exp2f((m - nm) * kLog2e)) + (om == -INFINITY ? 0.f : os * exp2f((om - nm) * kLog2e));
        m = nm;
    }
    if (lane == 0) { s_max[warp] = m; s_sum[warp] = s; }
    __syncthreads();
    m = s_max[lane]; s = s_sum[lane];          // CE_THREADS / 32 == 32 warps
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float om = __shfl_xor_sync(0xffffffffu, m, o), os = __shfl_xor_sync(0xffffffffu, s, o);
        float nm = fmaxf(m, om);
        s = (m == -INFINITY ? 0.f : s * exp2f((m - nm) * kLog2e)) + (om == -INFINITY ? 0.f : os * exp2f((om - nm) * kLog2e));
        m = nm;
    }
    const float lse = logf(s) + m;
    const float tgt_logit = to_float(x[tgt]);
    __syncthreads();                            // everyone has read x[tgt] before it is overwritten
    if (threadIdx.x == 0) {
        losses[row] += lse - tgt_logit;
        if (lse_out) lse_out[row] = lse;
    }
    if (!write_dlogits) return;
    // pass 2: p * gscale = exp2(x*log2e + shift)
    const float gscale = dloss + z_reg * lse;
    const float shift = (gscale > 0.f ? log2f(gscale) : -INFINITY) - lse * kLog2e;
    for (int i = threadIdx.x; i < nvec; i += CE_THREADS) {
        Vt v = Vt::load(x + i * Vt::N);
        const int base = i * Vt::N;
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) {
            float g = exp2f(to_float(v.v[k]) * kLog2e + shift);
            if (base + k == tgt) g -= dloss;
            v.v[k] = from_float<T>(g);
        }
        v.store_stream(x + base);
    }
    for (int i = nvec * Vt::N + threadIdx.x; i < V; i += CE_THREADS) {
        float g = exp2f(to_float(x[i]) * kLog2e + shift);
        if (i == tgt) g -= dloss;
        x[i] = from_float<T>(g);
    }
}

// max and sum of the per-token LSE values (z-loss monitoring); out = {max, sum}
__global__ void __launch_bounds__(1024) lse_stats_kernel(float* __restrict__ out, const float* __restrict__ lse, long long n, int accumulate) {
    __shared__ float scratch[32];
    float m = -INFINITY, s = 0.f;
    for (long long i = threadIdx.x; i < n; i += blockDim.x) { float v = lse[i]; m = fmaxf(m, v); s += v; }
    m = block_reduce_max(m, scratch);
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) {
        if (accumulate) { out[0] = fmaxf(out[0], m); out[1] += s; }
        else { out[0] = m; out[1] = s; }
    }
}

// out[g] = sum over batch and over positions [g*group, (g+1)*group) of losses(B, T)
__global__ void __launch_bounds__(256) grouped_loss_kernel(float* __restrict__ out, const float* __restrict__ losses, int B, int T, int group) {
    __shared__ float scratch[32];
    const int g = blockIdx.x;
    const int t0 = g * group, t1 = min(T, t0 + group);
    float s = 0.f;
    for (int b = 0; b < B; ++b)
        for (int t = t0 + threadIdx.x; t < t1; t += blockDim.x) s += losses[static_cast<long long>(b) * T + t];
    s = block_reduce_sum(s, scratch);
    if (threadIdx.x == 0) out[g] = s;
}

}  // namespace

extern "C" int llmq_fused_classifier(void* logits, float* losses, float* lse_out, const int* targets, float dloss, float z_reg,
                                     int rows, int V, long long ld, int dtype, int write_dlogits, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (dtype == 0) {
        if (ld % 8) return -1;
        fused_ce_kernel<bf16><<<rows, CE_THREADS, 0, s>>>(static_cast<bf16*>(logits), losses, lse_out, targets, dloss, z_reg, rows, V, ld, write_dlogits);
    } else if (dtype == 3) {
        if (ld % 4) return -1;
        fused_ce_kernel<float><<<rows, CE_THREADS, 0, s>>>(static_cast<float*>(logits), losses, lse_out, targets, dloss, z_reg, rows, V, ld, write_dlogits);
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_lse_stats(float* out, const float* lse, long long n, int accumulate, cudaStream_t s) {
    lse_stats_kernel<<<1, 1024, 0, s>>>(out, lse, n, accumulate);
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_grouped_loss_sum(float* out, const float* losses, int B, int T, int group, cudaStream_t s) {
    int groups = ceil_div_i(T, group);
    if (groups <= 0) return 0;
    grouped_loss_kernel<<<groups, 256, 0, s>>>(out, losses, B, T, group);
    return LLMQ_LAUNCH_CHECK();
}
