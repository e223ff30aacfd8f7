// Token embedding gather, its deterministic backward, and the bias gradient reduction.
// Behavioural counterparts of src/kernels/encoder.cu:23-249 and src/kernels/bias.cu:14-195 of the reference.
// The embedding backward needs no sort and no host work (the reference bucket-sorts the tokens on the CPU,
// encoder.cu:187-221): a first kernel counts, for every position, how many earlier positions hold the same token
// (its rank) and how many positions hold it at all; in the second kernel the rank-0 position of every distinct
// token gathers the other positions of that token in ascending order and adds the fp32 sum to the embedding row.
// Launch sizes depend only on B*T, nothing is read back by the host, the result is bitwise reproducible.
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

// rank[p] = #{q < p : tok[q] == tok[p]},  count[p] = #{q : tok[q] == tok[p]}.  grid (ceil(BT/256), splits): every CTA
// compares its 256 positions with one slice of all positions (staged through shared memory, read as broadcasts) and
// adds its partial counts with integer atomics (exact, so the result does not depend on the order).  BT^2 compares:
// 2.7e8 for 16384 tokens, a few microseconds.
__global__ void __launch_bounds__(256)
token_rank_kernel(int* __restrict__ rank, int* __restrict__ count, const int* __restrict__ tokens, int BT) {
    __shared__ int chunk[2048];
    const int p = blockIdx.x * 256 + threadIdx.x;
    const int tok = p < BT ? tokens[p] : -1;
    const int per_split = (BT + gridDim.y - 1) / gridDim.y;
    const int q_begin = blockIdx.y * per_split, q_end = min(BT, q_begin + per_split);
    int r = 0, c = 0;
    for (int q0 = q_begin; q0 < q_end; q0 += 2048) {
        const int n = min(2048, q_end - q0);
        __syncthreads();
        for (int i = threadIdx.x; i < n; i += 256) chunk[i] = tokens[q0 + i];
        __syncthreads();
        const int before = min(n, max(0, p - q0));            // entries of this chunk with q < p
        int i = 0;
        for (; i < before; ++i) { const int m = chunk[i] == tok; r += m; c += m; }
        for (; i < n; ++i) c += chunk[i] == tok;
    }
    if (p < BT) {
        if (r) atomicAdd(rank + p, r);
        if (c) atomicAdd(count + p, c);
    }
}

// grid (BT, channel slices of 256 * vector width).  The CTA of position p works only if p is the first position of
// its token: it lists the later positions with the same token in ascending order (skipped when the token occurs once)
// and adds dout[p] + dout[those] to the token's embedding gradient row.
template <typename T>
__global__ void __launch_bounds__(256)
encoder_bwd_kernel(T* __restrict__ dwte, const T* __restrict__ dout, const int* __restrict__ tokens, const int* __restrict__ rank,
                   const int* __restrict__ count, int BT, int C, int V) {
    using Vt = Vec16<T>;
    constexpr int LIST = 1024;
    __shared__ int list[LIST];
    __shared__ int warp_cnt[8];
    const int p = blockIdx.x;
    if (rank[p] != 0) return;
    const long long tok = tokens[p];
    if (tok < 0 || tok >= V) return;                           // ids outside the vocabulary never index memory
    const int c = (blockIdx.y * 256 + threadIdx.x) * Vt::N;
    const bool active = c < C;
    float acc[Vt::N];
    Vt cur;
    if (active) {
        cur = Vt::load(dwte + tok * C + c);
        Vt g = Vt::load_stream(dout + static_cast<long long>(p) * C + c);
#pragma unroll
        for (int k = 0; k < Vt::N; ++k) acc[k] = to_float(cur.v[k]) + to_float(g.v[k]);
    }
    int remaining = count[p] - 1;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int q0 = p + 1;
    while (remaining > 0 && q0 < BT) {                          // uniform across the CTA
        // fill the list with up to LIST later positions of this token, in ascending order
        int filled = 0;
        while (filled + 256 <= LIST && q0 < BT && filled < remaining) {
            const int q = q0 + threadIdx.x;
            const bool m = q < BT && tokens[q] == static_cast<int>(tok);
            const unsigned ballot = __ballot_sync(0xffffffffu, m);
            if (lane == 0) warp_cnt[warp] = __popc(ballot);
            __syncthreads();
            int base = filled, total = 0;
#pragma unroll
            for (int w = 0; w < 8; ++w) { if (w < warp) base += warp_cnt[w]; total += warp_cnt[w]; }
            if (m) list[base + __popc(ballot & ((1u << lane) - 1u))] = q;
            filled += total;
            q0 += 256;
            __syncthreads();
        }
        if (active) {
            for (int j = 0; j < filled; ++j) {
                Vt g = Vt::load_stream(dout + static_cast<long long>(list[j]) * C + c);
#pragma unroll
                for (int k = 0; k < Vt::N; ++k) acc[k] += to_float(g.v[k]);
            }
        }
        remaining -= filled;
        __syncthreads();                                        // the list is rewritten in the next round
    }
    if (active) {
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

// Same sums for C % 4 == 0 with four columns per thread (one 4- / 8- / 16-byte load per row instead of four element loads;
// for 1-byte gradients a warp then reads 128 contiguous bytes of a row).  A CTA covers 128 columns; the row lanes are added
// in the same order as above, so both kernels give the same partials.
template <typename T>
__global__ void __launch_bounds__(256)
bias_bwd_partial_vec4_kernel(float* __restrict__ partial, const T* __restrict__ dout, long long rows, int C) {
    __shared__ float tile[8][32][5];
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int c = blockIdx.x * 128 + cx * 4;
    float s[4] = {0.f, 0.f, 0.f, 0.f};
    if (c < C) {
        struct alignas(sizeof(T) * 4) Quad { T v[4]; };
        for (long long r = blockIdx.y * 8 + ry; r < rows; r += static_cast<long long>(gridDim.y) * 8) {
            const Quad q = *reinterpret_cast<const Quad*>(dout + r * C + c);
#pragma unroll
            for (int k = 0; k < 4; ++k) s[k] += to_float(q.v[k]);
        }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) tile[ry][cx][k] = s[k];
    __syncthreads();
    if (ry == 0 && c < C) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float t = 0.f;
#pragma unroll
            for (int g = 0; g < 8; ++g) t += tile[g][cx][k];
            partial[static_cast<long long>(blockIdx.y) * C + c + k] = t;
        }
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

// dwte[tokens[p]] += dout[p] for all p, summed per token in ascending position order.  `scratch` holds 2 * BT ints
// (rank, count) and is cleared here.  Three launches on the stream, nothing comes back to the host.
extern "C" int llmq_encoder_backward(void* dwte, const void* dout, const int* tokens, int* scratch, int BT, int C, int V,
                                     int dtype, cudaStream_t s) {
    if (BT <= 0) return 0;
    if ((dtype == 0 && C % 8) || (dtype == 3 && C % 4)) return -1;
    if (dtype != 0 && dtype != 3) return -10;
    int* rank = scratch;
    int* count = scratch + BT;
    cudaError_t e = cudaMemsetAsync(scratch, 0, sizeof(int) * 2 * static_cast<size_t>(BT), s);
    if (e != cudaSuccess) return static_cast<int>(e);
    const int pblocks = ceil_div_i(BT, 256);
    int splits = 1;
    while (splits < 8 && pblocks * splits < 256 && BT / (splits * 2) >= 2048) splits *= 2;
    token_rank_kernel<<<dim3(pblocks, splits), 256, 0, s>>>(rank, count, tokens, BT);
    if (dtype == 0) {
        encoder_bwd_kernel<bf16><<<dim3(BT, ceil_div_i(C, 256 * 8)), 256, 0, s>>>(static_cast<bf16*>(dwte), static_cast<const bf16*>(dout), tokens, rank, count, BT, C, V);
    } else {
        encoder_bwd_kernel<float><<<dim3(BT, ceil_div_i(C, 256 * 4)), 256, 0, s>>>(static_cast<float*>(dwte), static_cast<const float*>(dout), tokens, rank, count, BT, C, V);
    }
    return LLMQ_LAUNCH_CHECK();
}

// partial must hold slices * C floats (slices <= 1024).  dout dtype: bf16 / fp32 / e4m3 / e5m2.
extern "C" int llmq_bias_backward(void* dbias, float* partial, const void* dout, long long rows, int C, int slices,
                                  const float* scale_a, const float* scale_b, int accumulate, int dout_dtype, int dbias_dtype,
                                  cudaStream_t s) {
    if (rows <= 0 || C <= 0) return 0;
    const bool vec4 = C % 4 == 0 && reinterpret_cast<uintptr_t>(dout) % 16 == 0;
    dim3 grid(ceil_div_i(C, vec4 ? 128 : 32), slices);
#define BIAS_PARTIAL(T)                                                                                             \
    do {                                                                                                            \
        if (vec4) bias_bwd_partial_vec4_kernel<T><<<grid, 256, 0, s>>>(partial, static_cast<const T*>(dout), rows, C); \
        else bias_bwd_partial_kernel<T><<<grid, 256, 0, s>>>(partial, static_cast<const T*>(dout), rows, C);       \
    } while (0)
    if (dout_dtype == 0) BIAS_PARTIAL(bf16);
    else if (dout_dtype == 3) BIAS_PARTIAL(float);
    else if (dout_dtype == 1) BIAS_PARTIAL(e4m3);
    else if (dout_dtype == 2) BIAS_PARTIAL(e5m2);
#undef BIAS_PARTIAL
    else return -10;
    int rc = LLMQ_LAUNCH_CHECK();
    if (rc) return rc;
    if (dbias_dtype == 0) bias_bwd_final_kernel<bf16><<<ceil_div_i(C, 256), 256, 0, s>>>(static_cast<bf16*>(dbias), partial, slices, C, scale_a, scale_b, accumulate);
    else if (dbias_dtype == 3) bias_bwd_final_kernel<float><<<ceil_div_i(C, 256), 256, 0, s>>>(static_cast<float*>(dbias), partial, slices, C, scale_a, scale_b, accumulate);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}
