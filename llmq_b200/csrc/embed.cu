// Token embedding gather, its deterministic backward, and the bias gradient reduction.
// Behavioural counterparts of src/kernels/encoder.cu:23-249 and src/kernels/bias.cu:14-195 of the reference.
// The embedding backward works on token positions sorted by token id (sorted on the device by the
// caller): one CTA owns one distinct token, walks its positions in ascending order and adds the fp32
// sum to that embedding row, so the result is bitwise reproducible and needs no host-side bucketing.
#include "api.h"
#include "common.cuh"

namespace {

template <typename T>
__global__ void __launch_bounds__(256)
encoder_fwd_kernel(T* __restrict__ out, const int* __restrict__ tokens, const T* __restrict__ wte, long long BT, int C, int V) {
    using Vt = Vec16<T>;
    const int vec_per_row = C / Vt::N;
    const long long total = BT * vec_per_row;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long r = i / vec_per_row;
        int c = static_cast<int>(i - r * vec_per_row) * Vt::N;
        int tok = tokens[r];
        tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);           // out-of-range ids are clamped, never dereferenced
        Vt::load(wte + static_cast<long long>(tok) * C + c).store(out + r * C + c);
    }
}

// sorted_pos: positions (b*T + t) ordered by token id (stable);  seg_start[s] .. seg_start[s+1]: segment s;
// seg_token[s]: token id of the segment.
template <typename T>
__global__ void __launch_bounds__(256)
encoder_bwd_kernel(T* __restrict__ dwte, const T* __restrict__ dout, const int* __restrict__ sorted_pos,
                   const int* __restrict__ seg_start, const int* __restrict__ seg_token, int n_segments, int C) {
    using Vt = Vec16<T>;
    const int s = blockIdx.x;
    if (s >= n_segments) return;
    const int beg = seg_start[s], end = seg_start[s + 1];
    const long long tok = seg_token[s];
    for (int c = threadIdx.x * Vt::N; c < C; c += blockDim.x * Vt::N) {
        float acc[Vt::N];
        Vt cur = Vt::load(dwte + tok * C + c);
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) acc[k] = to_float(cur.v[k]);
        for (int j = beg; j < end; ++j) {
            Vt g = Vt::load_stream(dout + static_cast<long long>(sorted_pos[j]) * C + c);
#pragma unroll
            for (int k = 0; k < Vt::N; ++k) acc[k] += to_float(g.v[k]);
        }
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) cur.v[k] = from_float<T>(acc[k]);
        cur.store(dwte + tok * C + c);
    }
}

// dbias[c] (+)= scale * sum_rows dout[row, c].  Stage 1: grid (C/64 column groups, row slices) writes
// partial[slice][c]; stage 2 sums the slices in order.
template <typename T>
__global__ void __launch_bounds__(256)
bias_bwd_partial_kernel(float* __restrict__ partial, const T* __restrict__ dout, long long rows, int C) {
    __shared__ float tile[8][33];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;      // 32 columns x 8 row lanes
    const int c = blockIdx.x * 32 + cx;
    float s = 0.f;
    if (c < C) {
        for (long long r = blockIdx.y * 8 + ry; r < rows; r += static_cast<long long>(gridDim.y) * 8) s += to_float(dout[r * C + c]);
    }
    tile[ry][cx] = s;
    __syncthreads();
    if (ry == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += tile[k][cx];
        partial[static_cast<long long>(blockIdx.y) * C + c] = t;
    }
}

template <typename T>
__global__ void bias_bwd_final_kernel(T* __restrict__ dbias, const float* __restrict__ partial, int slices, int C,
                                      const float* __restrict__ scale_a, const float* __restrict__ scale_b, int accumulate) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float s = 0.f;
    for (int k = 0; k < slices; ++k) s += partial[static_cast<long long>(k) * C + c];
    if (scale_a) s *= *scale_a;
    if (scale_b) s *= *scale_b;
    if (accumulate) s += to_float(dbias[c]);
    dbias[c] = from_float<T>(s);
}

}  // namespace

extern "C" int llmq_encoder_forward(void* out, const int* tokens, const void* wte, long long BT, int C, int V, int dtype,
                                    int num_sms, cudaStream_t s) {
    if (BT <= 0) return 0;
    if (dtype == 0) {
        if (C % 8) return -1;
        long long blocks = ceil_div_ll(BT * (C / 8), 256);
        encoder_fwd_kernel<bf16><<<static_cast<int>(blocks < num_sms * 8LL ? blocks : num_sms * 8LL), 256, 0, s>>>(
            static_cast<bf16*>(out), tokens, static_cast<const bf16*>(wte), BT, C, V);
    } else if (dtype == 3) {
        if (C % 4) return -1;
        long long blocks = ceil_div_ll(BT * (C / 4), 256);
        encoder_fwd_kernel<float><<<static_cast<int>(blocks < num_sms * 8LL ? blocks : num_sms * 8LL), 256, 0, s>>>(
            static_cast<float*>(out), tokens, static_cast<const float*>(wte), BT, C, V);
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_encoder_backward(void* dwte, const void* dout, const int* sorted_pos, const int* seg_start,
                                     const int* seg_token, int n_segments, int C, int dtype, cudaStream_t s) {
    if (n_segments <= 0) return 0;
    if (dtype == 0) {
        if (C % 8) return -1;
        encoder_bwd_kernel<bf16><<<n_segments, 256, 0, s>>>(static_cast<bf16*>(dwte), static_cast<const bf16*>(dout), sorted_pos, seg_start, seg_token, n_segments, C);
    } else if (dtype == 3) {
        if (C % 4) return -1;
        encoder_bwd_kernel<float><<<n_segments, 256, 0, s>>>(static_cast<float*>(dwte), static_cast<const float*>(dout), sorted_pos, seg_start, seg_token, n_segments, C);
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

// partial must hold slices * C floats (slices <= 1024).  dout dtype: bf16 / fp32 / e4m3 / e5m2.
extern "C" int llmq_bias_backward(void* dbias, float* partial, const void* dout, long long rows, int C, int slices,
                                  const float* scale_a, const float* scale_b, int accumulate, int dout_dtype, int dbias_dtype,
                                  cudaStream_t s) {
    if (rows <= 0 || C <= 0) return 0;
    dim3 grid(ceil_div_i(C, 32), slices);
    if (dout_dtype == 0) bias_bwd_partial_kernel<bf16><<<grid, 256, 0, s>>>(partial, static_cast<const bf16*>(dout), rows, C);
    else if (dout_dtype == 3) bias_bwd_partial_kernel<float><<<grid, 256, 0, s>>>(partial, static_cast<const float*>(dout), rows, C);
    else if (dout_dtype == 1) bias_bwd_partial_kernel<e4m3><<<grid, 256, 0, s>>>(partial, static_cast<const e4m3*>(dout), rows, C);
    else if (dout_dtype == 2) bias_bwd_partial_kernel<e5m2><<<grid, 256, 0, s>>>(partial, static_cast<const e5m2*>(dout), rows, C);
    else return -10;
    int rc = LLMQ_LAUNCH_CHECK();
    if (rc) return rc;
    if (dbias_dtype == 0) bias_bwd_final_kernel<bf16><<<ceil_div_i(C, 256), 256, 0, s>>>(static_cast<bf16*>(dbias), partial, slices, C, scale_a, scale_b, accumulate);
    else if (dbias_dtype == 3) bias_bwd_final_kernel<float><<<ceil_div_i(C, 256), 256, 0, s>>>(static_cast<float*>(dbias), partial, slices, C, scale_a, scale_b, accumulate);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}
