// Per-head RMSNorm of the query and key heads of a packed (B, T, Hq + 2*Hkv, HS) tensor (Qwen3-style QK-norm).
// Part of the kernel API for parity with the reference (src/kernels/qk_norm.cu:60-446); like there it is not on
// the training path of the Llama / Qwen2 models.  One warp owns one (token, head) row.
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_fwd_kernel(T* out, float* __restrict__ rstd, const T* inp, const T* __restrict__ q_w, const T* __restrict__ k_w, float eps,
                   long long BT, int Hq, int Hkv, int HS) {
    const int H = Hq + 2 * Hkv, HN = Hq + Hkv;
    const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (w >= BT * HN) return;
    const long long bt = w / HN;
    const int h = static_cast<int>(w % HN);
    const T* x = inp + (bt * H + h) * HS;
    T* y = out + (bt * H + h) * HS;
    const T* wt = h < Hq ? q_w : k_w;
    float ss = 0.f;
    for (int c = lane; c < HS; c += 32) { float f = to_float(x[c]); ss += f * f; }
    ss = warp_reduce_sum(ss);
    const float rs = rsqrtf(ss / HS + eps);
    if (lane == 0) rstd[w] = rs;
    for (int c = lane; c < HS; c += 32) {
        T n = from_float<T>(to_float(x[c]) * rs);
        y[c] = from_float<T>(to_float(n) * to_float(wt[c]));
    }
}

// dinp = (w*dy - xhat * mean(w*dy*xhat)) * rstd ; dweight partials per block row-slice -> [slices][2][HS]
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_bwd_kernel(T* dinp, float* __restrict__ dw_partial, const T* dout, const T* inp, const T* __restrict__ q_w,
                   const T* __restrict__ k_w, const float* __restrict__ rstd, long long BT, int Hq, int Hkv, int HS) {
    extern __shared__ float sdw[];                       // [2][HS]
    const int H = Hq + 2 * Hkv, HN = Hq + Hkv;
    for (int i = threadIdx.x; i < 2 * HS; i += blockDim.x) sdw[i] = 0.f;
    __syncthreads();
    const int lane = threadIdx.x & 31, warps = blockDim.x >> 5;
    for (long long w = blockIdx.x * static_cast<long long>(warps) + (threadIdx.x >> 5); w < BT * HN;
         w += static_cast<long long>(gridDim.x) * warps) {
        const long long bt = w / HN;
        const int h = static_cast<int>(w % HN);
        const long long off = (bt * H + h) * HS;
        const T* wt = h < Hq ? q_w : k_w;
        const float rs = rstd[w];
        float dot = 0.f;
        for (int c = lane; c < HS; c += 32) dot += to_float(wt[c]) * to_float(dout[off + c]) * to_float(inp[off + c]) * rs;
        dot = warp_reduce_sum(dot) / HS;
        for (int c = lane; c < HS; c += 32) {
            const float xh = to_float(inp[off + c]) * rs, g = to_float(dout[off + c]);
            atomicAdd(&sdw[(h < Hq ? 0 : HS) + c], g * xh);
            dinp[off + c] = from_float<T>((to_float(wt[c]) * g - xh * dot) * rs);
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < 2 * HS; i += blockDim.x) dw_partial[static_cast<long long>(blockIdx.x) * 2 * HS + i] = sdw[i];
}

template <typename T>
__global__ void qk_norm_bwd_reduce_kernel(T* dq_w, T* dk_w, const float* __restrict__ partial, int slices, int HS, int accumulate) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 2 * HS) return;
    float s = 0.f;
    for (int k = 0; k < slices; ++k) s += partial[static_cast<long long>(k) * 2 * HS + i];
    T* dst = i < HS ? dq_w + i : dk_w + (i - HS);
    if (accumulate) s += to_float(*dst);
    *dst = from_float<T>(s);
}

}  // namespace

extern "C" int llmq_qk_norm_forward(void* out, float* rstd, const void* inp, const void* q_w, const void* k_w, float eps, long long BT,
                                    int Hq, int Hkv, int HS, int dtype, cudaStream_t s) {
    const long long rows = BT * (Hq + Hkv);
    if (rows <= 0) return 0;
    const unsigned int blocks = static_cast<unsigned int>(ceil_div_ll(rows * 32, 256));
    if (dtype == 0) qk_norm_fwd_kernel<bf16><<<blocks, 256, 0, s>>>(static_cast<bf16*>(out), rstd, static_cast<const bf16*>(inp), static_cast<const bf16*>(q_w), static_cast<const bf16*>(k_w), eps, BT, Hq, Hkv, HS);
    else if (dtype == 3) qk_norm_fwd_kernel<float><<<blocks, 256, 0, s>>>(static_cast<float*>(out), rstd, static_cast<const float*>(inp), static_cast<const float*>(q_w), static_cast<const float*>(k_w), eps, BT, Hq, Hkv, HS);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

// partial: slices * 2 * HS floats.  The value heads of dinp are left untouched.
extern "C" int llmq_qk_norm_backward(void* dinp, void* dq_w, void* dk_w, float* partial, const void* dout, const void* inp, const void* q_w,
                                     const void* k_w, const float* rstd, long long BT, int Hq, int Hkv, int HS, int slices, int accumulate,
                                     int dtype, cudaStream_t s) {
    if (BT <= 0) return 0;
    const int smem = 2 * HS * 4;
    if (dtype == 0) {
        qk_norm_bwd_kernel<bf16><<<slices, 256, smem, s>>>(static_cast<bf16*>(dinp), partial, static_cast<const bf16*>(dout), static_cast<const bf16*>(inp), static_cast<const bf16*>(q_w), static_cast<const bf16*>(k_w), rstd, BT, Hq, Hkv, HS);
        qk_norm_bwd_reduce_kernel<bf16><<<ceil_div_i(2 * HS, 128), 128, 0, s>>>(static_cast<bf16*>(dq_w), static_cast<bf16*>(dk_w), partial, slices, HS, accumulate);
    } else if (dtype == 3) {
        qk_norm_bwd_kernel<float><<<slices, 256, smem, s>>>(static_cast<float*>(dinp), partial, static_cast<const float*>(dout), static_cast<const float*>(inp), static_cast<const float*>(q_w), static_cast<const float*>(k_w), rstd, BT, Hq, Hkv, HS);
        qk_norm_bwd_reduce_kernel<float><<<ceil_div_i(2 * HS, 128), 128, 0, s>>>(static_cast<float*>(dq_w), static_cast<float*>(dk_w), partial, slices, HS, accumulate);
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}
