// SwiGLU forward / backward and rotary position embedding kernels.
// Behavioural counterparts of src/kernels/swiglu.cu:21-405 and src/kernels/rope.cu:41-153 of the reference.
#include "api.h"
#include "common.cuh"
#include "tile_transpose.cuh"

namespace {

// i -> (i / per_row, i % per_row); multiply-high when the index space fits 31 bits, 64-bit division otherwise
__device__ __forceinline__ void split_index(long long i, long long total, int per_row, const FastDiv& fd, long long& r, int& c) {
    if (total < (1ll << 31)) {
        uint32_t q, m;
        fd.divmod(static_cast<uint32_t>(i), q, m);
        r = q; c = static_cast<int>(m);
    } else {
        r = i / per_row;
        c = static_cast<int>(i - r * per_row);
    }
}

// ------------------------------------------------------------------------------------------------
// SwiGLU.  Input rows are [up(D) | gate(D)];  out = up * gate * sigmoid(gate).
// With q_out the kernel emits e4m3 directly using an abs-max that is already known (recompute path).
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(T* __restrict__ out, e4m3* __restrict__ q_out, const T* __restrict__ inp, long long rows, int D,
                  float* __restrict__ absmax_out, const float* __restrict__ known_absmax, float* __restrict__ q_scale_out,
                  const FastDiv fd) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    const int vec_per_row = D / V::N;
    const long long total = rows * vec_per_row;
    float qmul = 0.f;
    if (q_out) {
        float am = fmaxf(*known_absmax, 1e-10f);
        qmul = 448.f / am;
        if (blockIdx.x == 0 && threadIdx.x == 0 && q_scale_out) *q_scale_out = am / 448.f;
    }
    float tmax = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long r; int c;
        split_index(i, total, vec_per_row, fd, r, c);
        c *= V::N;
        const T* up = inp + r * 2 * D + c;
        V vu = V::load_stream(up), vg = V::load_stream(up + D), vo;
        float f[V::N];
#pragma unroll
        for (int k = 0; k < V::N; ++k) {
            float u = to_float(vu.v[k]), g = to_float(vg.v[k]);
            vo.v[k] = from_float<T>(u * g * fast_sigmoid(g));
            f[k] = to_float(vo.v[k]);
            tmax = fmaxf(tmax, fabsf(f[k]));
        }
        if (out) vo.store(out + r * D + c);
        if (q_out) {
            if constexpr (V::N == 8) {
#pragma unroll
                for (int k = 0; k < 8; ++k) f[k] *= qmul;
                *reinterpret_cast<uint2*>(q_out + r * D + c) = pack_e4m3x8(f);
            } else {
                *reinterpret_cast<uint32_t*>(q_out + r * D + c) = pack_e4m3x2(f[0] * qmul, f[1] * qmul) | (pack_e4m3x2(f[2] * qmul, f[3] * qmul) << 16);
            }
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// SwiGLU recompute for the backward pass of an fp8 model: the only consumer of the recomputed activation is the
// weight-gradient GEMM of the down projection, which reads it transposed (K-major), so this kernel writes nothing but
// q_t[D][rows] = e4m3(swiglu(inp)[rows][D]) with the abs-max known from the forward pass.  One 128 x 128 tile per CTA; the
// values are rounded to T first, exactly like swiglu_fwd_kernel's q_out path, so the bytes are the same.
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_fwd_transposed_kernel(e4m3* __restrict__ q_t, const T* __restrict__ inp, int rows, int D, const float* __restrict__ known_absmax,
                             float* __restrict__ q_scale_out) {
    static_assert(sizeof(T) == 2, "16-bit activations");
    __shared__ __align__(16) uint32_t tile[128 * 32];
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
    const float am = fmaxf(*known_absmax, 1e-10f);
    const float qmul = 448.f / am;
    if (blockIdx.x == 0 && blockIdx.y == 0 && t == 0 && q_scale_out) *q_scale_out = am / 448.f;
    const int cc = t & 15, rr = t >> 4;                    // 16 threads per row (8 elements each), 16 rows per pass
    uint4 vu[8], vg[8];
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int r = r0 + p * 16 + rr, c = c0 + cc * 8;
        const bool ok = r < rows && c < D;
        const T* up = inp + static_cast<long long>(r) * 2 * D + c;
        vu[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up)) : make_uint4(0, 0, 0, 0);
        vg[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up + D)) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int p = 0; p < 8; ++p) {
        const int lr = p * 16 + rr;
        const T* u = reinterpret_cast<const T*>(&vu[p]);
        const T* g = reinterpret_cast<const T*>(&vg[p]);
        float f[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float uf = to_float(u[k]), gf = to_float(g[k]);
            f[k] = to_float(from_float<T>(uf * gf * fast_sigmoid(gf))) * qmul;
        }
        *reinterpret_cast<uint2*>(&tile[tile_word_index(lr, cc * 2)]) = pack_e4m3x8(f);
    }
    __syncthreads();
    tile_store_transposed<e4m3>(tile, q_t, r0, c0, rows, D);
}

// Backward: dinp = [d_up | d_gate]; dinp may alias inp (in-place over the saved up-projection).
template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(T* dinp, const T* __restrict__ dout, const T* inp, long long rows, int D, float* __restrict__ absmax_out,
                  const FastDiv fd) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    const int vec_per_row = D / V::N;
    const long long total = rows * vec_per_row;
    float tmax = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        long long r; int c;
        split_index(i, total, vec_per_row, fd, r, c);
        c *= V::N;
        const T* up = inp + r * 2 * D + c;
        V vu = V::load(up), vg = V::load(up + D), vd = V::load_stream(dout + r * D + c), du, dg;
#pragma unroll
        for (int k = 0; k < V::N; ++k) {
            float u = to_float(vu.v[k]), g = to_float(vg.v[k]), d = to_float(vd.v[k]);
            float s = fast_sigmoid(g);
            du.v[k] = from_float<T>(d * g * s);
            dg.v[k] = from_float<T>(d * u * s * (1.f + g * (1.f - s)));
            tmax = fmaxf(tmax, fmaxf(fabsf(to_float(du.v[k])), fabsf(to_float(dg.v[k]))));
        }
        du.store(dinp + r * 2 * D + c);
        dg.store(dinp + r * 2 * D + D + c);
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

// SwiGLU backward of an fp8 model whose GEMMs read K-major operands, in two passes that never write the 16-bit gradient:
// the only consumers of [d_up | d_gate] are the two GEMMs of the up projection, which read its e4m3 copy and the
// transpose of that copy.  The first pass finds the abs-max of the gradient (rounded to T, as swiglu_bwd_kernel would
// store it) and, while the up projection is in registers anyway, can emit the transposed e4m3 SwiGLU output that the
// weight-gradient GEMM of the down projection needs (the recompute of swiglu_fwd_transposed_kernel); the second pass
// recomputes the gradient and writes q_rows[rows][2D] and q_t[2D][rows].  Both passes work on 128 x 128 tiles of the D
// columns: one CTA reads the matching up, gate and dout tiles and owns both halves of the output.
template <typename T>
__device__ __forceinline__ void swiglu_bwd_values(const uint4& vu, const uint4& vg, const uint4& vd, float (&du)[8], float (&dg)[8]) {
    const T* u = reinterpret_cast<const T*>(&vu);
    const T* g = reinterpret_cast<const T*>(&vg);
    const T* d = reinterpret_cast<const T*>(&vd);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float uf = to_float(u[k]), gf = to_float(g[k]), df = to_float(d[k]);
        const float s = fast_sigmoid(gf);
        du[k] = to_float(from_float<T>(df * gf * s));
        dg[k] = to_float(from_float<T>(df * uf * s * (1.f + gf * (1.f - s))));
    }
}

template <typename T, bool WriteAct>
__global__ void __launch_bounds__(256)
swiglu_bwd_stats_kernel(float* __restrict__ absmax_out, e4m3* __restrict__ act_t, const T* __restrict__ dout, const T* __restrict__ inp,
                        int rows, int D, const float* __restrict__ act_absmax, float* __restrict__ act_scale_out) {
    static_assert(sizeof(T) == 2, "16-bit activations");
    __shared__ __align__(16) uint32_t tile[WriteAct ? 128 * 32 : 4];
    __shared__ float scratch[32];
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
    float qmul = 0.f;
    if constexpr (WriteAct) {
        const float am = fmaxf(*act_absmax, 1e-10f);
        qmul = 448.f / am;
        if (blockIdx.x == 0 && blockIdx.y == 0 && t == 0 && act_scale_out) *act_scale_out = am / 448.f;
    }
    const int cc = t & 15, rr = t >> 4;                    // 16 threads per row (8 elements each), 16 rows per pass
    float tmax = 0.f;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint4 vu[4], vg[4], vd[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int r = r0 + (h * 4 + p) * 16 + rr, c = c0 + cc * 8;
            const bool ok = r < rows && c < D;
            const T* up = inp + static_cast<long long>(r) * 2 * D + c;
            vu[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up)) : make_uint4(0, 0, 0, 0);
            vg[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up + D)) : make_uint4(0, 0, 0, 0);
            vd[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(dout + static_cast<long long>(r) * D + c)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            float du[8], dg[8];
            swiglu_bwd_values<T>(vu[p], vg[p], vd[p], du, dg);
#pragma unroll
            for (int k = 0; k < 8; ++k) tmax = fmaxf(tmax, fmaxf(fabsf(du[k]), fabsf(dg[k])));
            if constexpr (WriteAct) {
                const int lr = (h * 4 + p) * 16 + rr;
                const T* u = reinterpret_cast<const T*>(&vu[p]);
                const T* g = reinterpret_cast<const T*>(&vg[p]);
                float f[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const float uf = to_float(u[k]), gf = to_float(g[k]);
                    f[k] = to_float(from_float<T>(uf * gf * fast_sigmoid(gf))) * qmul;
                }
                *reinterpret_cast<uint2*>(&tile[tile_word_index(lr, cc * 2)]) = pack_e4m3x8(f);
            }
        }
    }
    if constexpr (WriteAct) {
        __syncthreads();
        tile_store_transposed<e4m3>(tile, act_t, r0, c0, rows, D);
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

template <typename T>
__global__ void __launch_bounds__(256)
swiglu_bwd_quant_kernel(e4m3* __restrict__ q_rows, e4m3* __restrict__ q_t, float* __restrict__ scale_out, const T* __restrict__ dout,
                        const T* __restrict__ inp, int rows, int D, const float* __restrict__ absmax) {
    static_assert(sizeof(T) == 2, "16-bit activations");
    __shared__ __align__(16) uint32_t tile_u[128 * 32];
    __shared__ __align__(16) uint32_t tile_g[128 * 32];
    const int t = threadIdx.x;
    const int c0 = blockIdx.x * 128, r0 = blockIdx.y * 128;
    const float am = fmaxf(*absmax, 1e-10f);
    const float mul = 448.f / am;
    if (blockIdx.x == 0 && blockIdx.y == 0 && t == 0 && scale_out) *scale_out = am / 448.f;
    const int cc = t & 15, rr = t >> 4;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        uint4 vu[4], vg[4], vd[4];
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int r = r0 + (h * 4 + p) * 16 + rr, c = c0 + cc * 8;
            const bool ok = r < rows && c < D;
            const T* up = inp + static_cast<long long>(r) * 2 * D + c;
            vu[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up)) : make_uint4(0, 0, 0, 0);
            vg[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(up + D)) : make_uint4(0, 0, 0, 0);
            vd[p] = ok ? __ldcs(reinterpret_cast<const uint4*>(dout + static_cast<long long>(r) * D + c)) : make_uint4(0, 0, 0, 0);
        }
#pragma unroll
        for (int p = 0; p < 4; ++p) {
            const int lr = (h * 4 + p) * 16 + rr, r = r0 + lr, c = c0 + cc * 8;
            float du[8], dg[8];
            swiglu_bwd_values<T>(vu[p], vg[p], vd[p], du, dg);
#pragma unroll
            for (int k = 0; k < 8; ++k) { du[k] *= mul; dg[k] *= mul; }
            const uint2 wu = pack_e4m3x8(du), wg = pack_e4m3x8(dg);
            if (r < rows && c < D) {
                e4m3* o = q_rows + static_cast<long long>(r) * 2 * D + c;
                *reinterpret_cast<uint2*>(o) = wu;
                *reinterpret_cast<uint2*>(o + D) = wg;
            }
            *reinterpret_cast<uint2*>(&tile_u[tile_word_index(lr, cc * 2)]) = wu;
            *reinterpret_cast<uint2*>(&tile_g[tile_word_index(lr, cc * 2)]) = wg;
        }
    }
    __syncthreads();
    // q_t is [2D][rows]: the d_up tile lands at rows c0.. of q_t, the d_gate tile at rows D + c0..; the column bound of each
    // call is the end of its half
    tile_store_transposed<e4m3>(tile_u, q_t, r0, c0, rows, D);
    tile_store_transposed<e4m3>(tile_g, q_t, r0, D + c0, rows, 2 * D);
}

// ------------------------------------------------------------------------------------------------
// RoPE on the packed (B, T, Hq + 2*Hkv, HS) tensor; query and key heads are rotated with the half-split
// pairing (d, d + HS/2), value heads are copied (or left alone when in place).  freqs is (T, HS/2, 2)
// fp32 {cos, sin}.  Backward is the conjugate rotation.
template <typename T, bool Backward>
__global__ void __launch_bounds__(256)
rope_kernel(T* out, const T* inp, const float* __restrict__ freqs, int B, int Tlen, int Hq, int Hkv, int HS,
            float* __restrict__ absmax_out, const FastDiv fd_vec, const FastDiv fd_h, const FastDiv fd_t) {
    __shared__ float scratch[32];
    using V = Vec16<T>;
    const int half = HS / 2;
    const int vec_per_half = half / V::N;
    const int H = Hq + 2 * Hkv;
    const long long total = static_cast<long long>(B) * Tlen * H * vec_per_half;
    float tmax = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        int v, h, t;
        long long bt;
        if (total < (1ll << 31)) {
            uint32_t rest, vv, hh, btt, bb, tt;
            fd_vec.divmod(static_cast<uint32_t>(i), rest, vv);
            fd_h.divmod(rest, btt, hh);
            fd_t.divmod(btt, bb, tt);
            v = static_cast<int>(vv); h = static_cast<int>(hh); t = static_cast<int>(tt); bt = btt;
        } else {
            v = static_cast<int>(i % vec_per_half);
            long long rest = i / vec_per_half;
            h = static_cast<int>(rest % H);
            bt = rest / H;
            t = static_cast<int>(bt % Tlen);
        }
        long long base = (bt * H + h) * HS + v * V::N;
        V x1 = V::load(inp + base), x2 = V::load(inp + base + half);
        if (h < Hq + Hkv) {
            const float* f = freqs + (static_cast<long long>(t) * half + v * V::N) * 2;
#pragma unroll
            for (int k = 0; k < V::N; ++k) {
                float c = f[2 * k], s = f[2 * k + 1];
                if (Backward) s = -s;
                float a = to_float(x1.v[k]), b = to_float(x2.v[k]);
                x1.v[k] = from_float<T>(a * c - b * s);
                x2.v[k] = from_float<T>(b * c + a * s);
            }
        } else if (out == inp && !absmax_out) {
            continue;
        }
        if (absmax_out) {
#pragma unroll
            for (int k = 0; k < V::N; ++k) tmax = fmaxf(tmax, fmaxf(fabsf(to_float(x1.v[k])), fabsf(to_float(x2.v[k]))));
        }
        if (!(out == inp && h >= Hq + Hkv)) {
            x1.store(out + base);
            x2.store(out + base + half);
        }
    }
    block_absmax_commit(absmax_out, tmax, scratch);
}

__global__ void rope_table_kernel(float* freqs, int Tlen, int half, float theta) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= Tlen * half) return;
    int t = i / half, d = i % half;
    // inverse frequency in double precision so long contexts keep their phase
    double inv = pow(static_cast<double>(theta), -static_cast<double>(2 * d) / (2.0 * half));
    double ang = t * inv;
    freqs[2 * i] = static_cast<float>(cos(ang));
    freqs[2 * i + 1] = static_cast<float>(sin(ang));
}

int grid_for(long long work_items, int threads, int num_sms) {
    long long blocks = ceil_div_ll(work_items, threads);
    long long cap = static_cast<long long>(num_sms) * 8;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

extern "C" int llmq_swiglu_forward(void* out, void* q_out, const void* inp, long long rows, int D, int dtype, float* absmax,
                                   const float* known_absmax, float* q_scale, int num_sms, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (dtype == 0) {
        if (D % 8) return -1;
        swiglu_fwd_kernel<bf16><<<grid_for(rows * (D / 8), 256, num_sms), 256, 0, s>>>(
            static_cast<bf16*>(out), static_cast<e4m3*>(q_out), static_cast<const bf16*>(inp), rows, D, absmax, known_absmax, q_scale, FastDiv(D / 8));
    } else if (dtype == 3) {
        if (D % 4) return -1;
        swiglu_fwd_kernel<float><<<grid_for(rows * (D / 4), 256, num_sms), 256, 0, s>>>(
            static_cast<float*>(out), static_cast<e4m3*>(q_out), static_cast<const float*>(inp), rows, D, absmax, known_absmax, q_scale, FastDiv(D / 4));
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_swiglu_backward(void* dinp, const void* dout, const void* inp, long long rows, int D, int dtype,
                                    float* absmax, int num_sms, cudaStream_t s) {
    if (rows <= 0) return 0;
    if (dtype == 0) {
        if (D % 8) return -1;
        swiglu_bwd_kernel<bf16><<<grid_for(rows * (D / 8), 256, num_sms), 256, 0, s>>>(
            static_cast<bf16*>(dinp), static_cast<const bf16*>(dout), static_cast<const bf16*>(inp), rows, D, absmax, FastDiv(D / 8));
    } else if (dtype == 3) {
        if (D % 4) return -1;
        swiglu_bwd_kernel<float><<<grid_for(rows * (D / 4), 256, num_sms), 256, 0, s>>>(
            static_cast<float*>(dinp), static_cast<const float*>(dout), static_cast<const float*>(inp), rows, D, absmax, FastDiv(D / 4));
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_rope(void* out, const void* inp, const float* freqs, int B, int T, int Hq, int Hkv, int HS, int dtype,
                         int backward, float* absmax, int num_sms, cudaStream_t s) {
    if (B <= 0 || T <= 0) return 0;
    const int H = Hq + 2 * Hkv;
    if (dtype == 0) {
        if ((HS / 2) % 8) return -1;
        constexpr int VN = 8;
        long long work = static_cast<long long>(B) * T * H * (HS / 2 / 8);
        int g = grid_for(work, 256, num_sms);
        if (backward) rope_kernel<bf16, true><<<g, 256, 0, s>>>(static_cast<bf16*>(out), static_cast<const bf16*>(inp), freqs, B, T, Hq, Hkv, HS, absmax, FastDiv(HS / 2 / VN), FastDiv(H), FastDiv(T));
        else rope_kernel<bf16, false><<<g, 256, 0, s>>>(static_cast<bf16*>(out), static_cast<const bf16*>(inp), freqs, B, T, Hq, Hkv, HS, absmax, FastDiv(HS / 2 / VN), FastDiv(H), FastDiv(T));
    } else if (dtype == 3) {
        if ((HS / 2) % 4) return -1;
        constexpr int VN = 4;
        long long work = static_cast<long long>(B) * T * H * (HS / 2 / 4);
        int g = grid_for(work, 256, num_sms);
        if (backward) rope_kernel<float, true><<<g, 256, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(inp), freqs, B, T, Hq, Hkv, HS, absmax, FastDiv(HS / 2 / VN), FastDiv(H), FastDiv(T));
        else rope_kernel<float, false><<<g, 256, 0, s>>>(static_cast<float*>(out), static_cast<const float*>(inp), freqs, B, T, Hq, Hkv, HS, absmax, FastDiv(HS / 2 / VN), FastDiv(H), FastDiv(T));
    } else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_rope_table(float* freqs, int T, int HS, float theta, cudaStream_t s) {
    int n = T * (HS / 2);
    if (n <= 0) return 0;
    rope_table_kernel<<<ceil_div_i(n, 256), 256, 0, s>>>(freqs, T, HS / 2, theta);
    return LLMQ_LAUNCH_CHECK();
}

// q_t[D][rows] (e4m3) = transpose of the quantised SwiGLU output; rows and D multiples of 16, bf16 input [rows][2D].
extern "C" int llmq_swiglu_forward_transposed(void* q_t, const void* inp, int rows, int D, const float* known_absmax, float* q_scale_out,
                                              int dtype, cudaStream_t s) {
    if (rows <= 0 || D <= 0) return 0;
    if (rows % 16 || D % 16 || !known_absmax) return -11;
    if (dtype != 0) return -10;
    dim3 grid(ceil_div_i(D, 128), ceil_div_i(rows, 128));
    swiglu_fwd_transposed_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<e4m3*>(q_t), static_cast<const bf16*>(inp), rows, D, known_absmax, q_scale_out);
    return LLMQ_LAUNCH_CHECK();
}

// Pass 1 of the fp8 SwiGLU backward: *absmax_out = max(*absmax_out, abs-max of [d_up | d_gate] rounded to the activation
// type); with act_t also act_t[D][rows] = transposed e4m3 SwiGLU output under the known abs-max *act_absmax.
// dout is [rows][D], inp [rows][2D] (bf16); rows and D multiples of 16.
extern "C" int llmq_swiglu_backward_stats(float* absmax_out, void* act_t, const void* dout, const void* inp, int rows, int D,
                                          const float* act_absmax, float* act_scale_out, int dtype, cudaStream_t s) {
    if (rows <= 0 || D <= 0) return 0;
    if (rows % 16 || D % 16 || !absmax_out || (act_t && !act_absmax)) return -11;
    if (dtype != 0) return -10;
    dim3 grid(ceil_div_i(D, 128), ceil_div_i(rows, 128));
    if (act_t)
        swiglu_bwd_stats_kernel<bf16, true><<<grid, 256, 0, s>>>(absmax_out, static_cast<e4m3*>(act_t), static_cast<const bf16*>(dout),
                                                                 static_cast<const bf16*>(inp), rows, D, act_absmax, act_scale_out);
    else
        swiglu_bwd_stats_kernel<bf16, false><<<grid, 256, 0, s>>>(absmax_out, nullptr, static_cast<const bf16*>(dout),
                                                                  static_cast<const bf16*>(inp), rows, D, nullptr, nullptr);
    return LLMQ_LAUNCH_CHECK();
}

// Pass 2: q_rows[rows][2D] and q_t[2D][rows] = e4m3([d_up | d_gate] * 448 / *absmax), *scale_out = *absmax / 448.
extern "C" int llmq_swiglu_backward_quant(void* q_rows, void* q_t, float* scale_out, const void* dout, const void* inp, int rows, int D,
                                          const float* absmax, int dtype, cudaStream_t s) {
    if (rows <= 0 || D <= 0) return 0;
    if (rows % 16 || D % 16 || !absmax || !q_rows || !q_t) return -11;
    if (dtype != 0) return -10;
    dim3 grid(ceil_div_i(D, 128), ceil_div_i(rows, 128));
    swiglu_bwd_quant_kernel<bf16><<<grid, 256, 0, s>>>(static_cast<e4m3*>(q_rows), static_cast<e4m3*>(q_t), scale_out,
                                                       static_cast<const bf16*>(dout), static_cast<const bf16*>(inp), rows, D, absmax);
    return LLMQ_LAUNCH_CHECK();
}
