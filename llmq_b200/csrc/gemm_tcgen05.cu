// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   C[M,N] (+)= alpha * A * B^T (+ bias[N]),   fp32 accumulation in tensor memory.
//
// Operands are bf16, 8-bit floats (e4m3 / e5m2) or - one-CTA kernel only - fp32 multiplied as tf32 (the GEMMs of an
// fp32 model: src/kernels/matmul.cpp:46-153 of the reference runs those through cuBLASLt).  Each operand may be stored K-major
// (row = M/N index, K contiguous) or MN-major (row = K index, M/N contiguous); the MN-major
// form is what lets the backward GEMMs (dX = dY * W, dW = dY^T * X) read the very same tensors
// as the forward pass without any transpose kernel.  alpha is the product of two optional
// per-tensor dequantisation factors read from device memory, so no host synchronisation is
// needed between the abs-max reduction and the GEMM.
//
// Replaces the cuBLASLt wrapper and the mma.sync kernel of the reference
// (src/kernels/matmul.cpp:46-153, src/kernels/gemm_mma.cu:21-291).
//
// Structure (192 threads per CTA, one CTA per SM):
//   warp 0     TMA producer: fills a 4-stage ring of 128x(128 B) A and 256x(128 B) B tiles
//   warp 1     MMA issuer (one elected lane): 4 tcgen05.mma per stage into one of two
//              128x256 fp32 accumulators in TMEM, tcgen05.commit to free the stage
//   warps 2-5  epilogue: tcgen05.ld the finished accumulator (while the other one is being
//              computed), scale, add bias, optionally add the previous C, track abs-max, store
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"
#include "gemm_common.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int ROW_BYTES = 128;            // one swizzle row
constexpr int STAGES = 4;
constexpr int A_STAGE_BYTES = BM * ROW_BYTES;   // 16 KiB
constexpr int B_STAGE_BYTES = BN * ROW_BYTES;   // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;            // two 256-column accumulators
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;


__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    // Grouped rasterisation: 16 row tiles share every column tile while it is hot in L2.
    constexpr int G = 16;
    int per_group = G * tiles_n;
    int group = t / per_group;
    int first_m = group * G;
    int gsz = min(tiles_m - first_m, G);
    int r = t - group * per_group;
    tm = first_m + (r % gsz);
    tn = r / gsz;
}

// Kind: MMA kind of ptx_sm100.cuh's mma_issue (0 bf16, 1 8-bit floats, 2 tf32 on fp32 operands).
template <int Kind>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 128B-swizzled tiles must start on a 1024-byte boundary
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    // bars[0..S) full, [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    const int bk = ROW_BYTES / p.elem_bytes;          // K elements per stage (K-major row)
    const int k_iters = (p.K + bk - 1) / bk;
    const int tiles_m = (p.M + BM - 1) / BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int splits = p.k_splits > 1 ? p.k_splits : 1;
    const int k_per_split = (k_iters + splits - 1) / splits;
    const int num_tiles = tiles_m * tiles_n * splits;           // work items: (tile, K split)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 128); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {
        tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            int stage = 0; uint32_t phase = 0;
            const int mn_chunk = ROW_BYTES / p.elem_bytes;     // M/N elements per 128-byte row (MN-major)
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn; tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
                const int k_begin = (t % splits) * k_per_split, k_end = min(k_iters, k_begin + k_per_split);
                for (int k = k_begin; k < k_end; ++k) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrEmptyWait); ok = false; break; }
                    uint32_t sa = smem_base + stage * STAGE_BYTES;
                    uint32_t sb = sa + A_STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), STAGE_BYTES);
                    if (!p.a_mn_major) {
                        tma_load_2d(sa, &tmap_a, full_bar(stage), k * bk, tm * BM);
                    } else {
                        // boxes of [bk K-rows][128 B of M]; BM*elem_bytes/128 boxes side by side
                        int nbox = BM * p.elem_bytes / ROW_BYTES;
                        for (int b = 0; b < nbox; ++b)
                            tma_load_2d(sa + b * (A_STAGE_BYTES / nbox), &tmap_a, full_bar(stage), tm * BM + b * mn_chunk, k * bk);
                    }
                    if (!p.b_mn_major) {
                        tma_load_2d(sb, &tmap_b, full_bar(stage), k * bk, tn * BN);
                    } else {
                        int nbox = BN * p.elem_bytes / ROW_BYTES;
                        for (int b = 0; b < nbox; ++b)
                            tma_load_2d(sb + b * (B_STAGE_BYTES / nbox), &tmap_b, full_bar(stage), tn * BN + b * mn_chunk, k * bk);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc = make_instr_desc(p.a_fmt, p.b_fmt, p.a_mn_major, p.b_mn_major, BM, BN);
            // K-major: 8-row groups are 1024 B apart, a K step of one MMA is 32 B inside the row.
            // MN-major: a K step of one MMA is (mma_k rows * 128 B); next 128 B chunk along M/N
            //           is one whole box (bk rows * 128 B) further on.
            const int mma_k = 32 / p.elem_bytes;
            const uint32_t box_bytes = static_cast<uint32_t>(bk) * ROW_BYTES;
            const uint32_t a_step = p.a_mn_major ? mma_k * ROW_BYTES : 32;
            const uint32_t b_step = p.b_mn_major ? mma_k * ROW_BYTES : 32;
            const uint32_t a_lbo = p.a_mn_major ? box_bytes : 16;
            const uint32_t b_lbo = p.b_mn_major ? box_bytes : 16;
            const uint32_t a_hi = desc_hi(1024), b_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_base, a_lbo), b_lo0 = desc_lo(smem_base + A_STAGE_BYTES, b_lbo);
            const uint32_t a_inc = a_step >> 4, b_inc = b_step >> 4;
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrTmemEmpty); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                const int k_begin = (t % splits) * k_per_split, k_end = min(k_iters, k_begin + k_per_split);
                for (int k = k_begin; k < k_end; ++k) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { atomicOr(p.status, kErrFullWait); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t alo = a_lo0 + stage * (STAGE_BYTES >> 4);
                    const uint32_t blo = b_lo0 + stage * (STAGE_BYTES >> 4);
                    mma_issue<Kind, false>(d_tmem, alo, a_hi, blo, b_hi, idesc, k > k_begin ? 1u : 0u);
                    mma_issue<Kind, false>(d_tmem, alo + a_inc, a_hi, blo + b_inc, b_hi, idesc, 1u);
                    mma_issue<Kind, false>(d_tmem, alo + 2 * a_inc, a_hi, blo + 2 * b_inc, b_hi, idesc, 1u);
                    mma_issue<Kind, false>(d_tmem, alo + 3 * a_inc, a_hi, blo + 3 * b_inc, b_hi, idesc, 1u);
                    mma_commit(empty_bar(stage));          // stage reusable once these MMAs have read it
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma_commit(tfull_bar(acc));                // accumulator complete
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps)
        const int q = warp & 3;                            // TMEM lane quarter this warp may access
        float alpha = p.alpha;
        if (p.scale_a) alpha *= *p.scale_a;
        if (p.scale_b) alpha *= *p.scale_b;
        float tmax = 0.f;
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int tm, tn; tile_coords(t / splits, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { if (lane == 0) atomicOr(p.status, kErrTmemFull); ok = false; break; }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
            if (splits > 1) epilogue_rows_partial(p, t_row, tm * BM + q * 32 + lane, tn * BN, BN, t % splits);
            else            epilogue_rows(p, t_row, tm * BM + q * 32 + lane, tn * BN, BN, alpha, tmax);
            tc_fence_before_sync();
            mbar_arrive(tempty_bar(acc));                  // 128 arrivals release the accumulator
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
        }
        if (p.absmax_out) {
            tmax = warp_reduce_max(tmax);
            if (lane == 0 && tmax > 0.f) atomic_max_float(p.absmax_out, tmax);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc(tmem_base, TMEM_COLS);
}

// Sum of the split-K parts + the normal epilogue (alpha, bias, accumulate, bf16 / fp32 store, abs-max).
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const GemmParams p, float alpha_host) {
    __shared__ float scratch[32];
    float alpha = alpha_host;
    if (p.scale_a) alpha *= *p.scale_a;
    if (p.scale_b) alpha *= *p.scale_b;
    const long long total = static_cast<long long>(p.M) * p.N;
    float tmax = 0.f;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < total; i += static_cast<long long>(gridDim.x) * 256) {
        const int col = static_cast<int>(i % p.N);
        const long long row = i / p.N;
        float v = 0.f;
        for (int s = 0; s < p.k_splits; ++s) v += p.partial[static_cast<long long>(s) * total + i];
        v *= alpha;
        if (p.bias) v += p.bias_dtype == 0 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p.bias)[col]) : static_cast<const float*>(p.bias)[col];
        if (p.c_dtype == 0) {
            __nv_bfloat16* c = static_cast<__nv_bfloat16*>(p.C) + row * p.ldc + col;
            if (p.accumulate) v += __bfloat162float(*c);
            *c = __float2bfloat16_rn(v);
        } else {
            float* c = static_cast<float*>(p.C) + row * p.ldc + col;
            if (p.accumulate) v += *c;
            *c = v;
        }
        tmax = fmaxf(tmax, fabsf(v));
    }
    if (p.absmax_out) block_absmax_commit(p.absmax_out, tmax, scratch);
}

// ------------------------------------------------------------------------------------------------
// Host side: tensor-map encoding through the driver entry point (no link-time libcuda dependency).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || !ptr)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

}  // namespace

// Encodes a 2-D tiled map over a row-major [rows, cols] matrix with leading dimension ld (elements).
// The box is [box_rows][128 bytes] with the 128-byte swizzle.  Returns 0 on success.
int llmq_encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, long long rows, long long cols,
                        long long ld, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) return -1;
    cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
    cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * elem_bytes};
    cuuint32_t box[2] = {static_cast<cuuint32_t>(128 / elem_bytes), static_cast<cuuint32_t>(box_rows)};
    cuuint32_t estr[2] = {1, 1};
    CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                             : (elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT8);
    CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int llmq_gemm_2cta_launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int num_sms, cudaStream_t stream);

// Tile-shape selection: 0 = automatic, 1 = force the one-CTA kernel, 2 = force the CTA-pair kernel.
static int g_gemm_mode = 0;
static int g_gemm_tma_store = 1;
extern "C" void llmq_gemm_set_tma_store(int on) { g_gemm_tma_store = on; }
extern "C" void llmq_gemm_set_mode(int mode) { g_gemm_mode = mode; }
// Split-K workspace of the calling thread's next GEMMs: `floats` fp32 elements at `ws` (0 switches split-K off).
// A GEMM uses it when its output has fewer than num_sms / 2 tiles of the one-CTA kernel and K is long enough.
static thread_local float* g_splitk_ws = nullptr;
static thread_local long long g_splitk_floats = 0;
extern "C" void llmq_gemm_set_splitk_workspace(float* ws, long long floats) { g_splitk_ws = ws; g_splitk_floats = floats; }

extern "C" int llmq_gemm_ready(const void*, const void*, void*, const void*, int, int, int, int, int, int, int, long long, long long, long long, int, int, int,
                               const float*, const float*, float, float*, unsigned int*, int, const unsigned int*, unsigned int, int, double, cudaStream_t);
static int gemm_impl(const void*, const void*, void*, const void*, int, int, int, int, int, int, int, long long, long long, long long, int, int, int,
                     const float*, const float*, float, float*, unsigned int*, int, const unsigned int*, unsigned int, int, double, const GemmParams*,
                     cudaStream_t);

extern "C" int llmq_gemm(const void* A, const void* B, void* C, const void* bias,
                         int M, int N, int K,
                         int ab_dtype,            // 0 bf16, 1 e4m3, 2 e5m2 (A), B shares the width
                         int b_dtype,
                         int a_mn_major, int b_mn_major,
                         long long lda, long long ldb, long long ldc,
                         int c_dtype, int bias_dtype, int accumulate,
                         const float* scale_a, const float* scale_b, float alpha,
                         float* absmax_out, unsigned int* status, int num_sms, cudaStream_t stream) {
    return llmq_gemm_ready(A, B, C, bias, M, N, K, ab_dtype, b_dtype, a_mn_major, b_mn_major, lda, ldb, ldc, c_dtype, bias_dtype, accumulate,
                           scale_a, scale_b, alpha, absmax_out, status, num_sms, nullptr, 0u, 0, 0.0, stream);
}

// Same, with the fused all-gather hook: rows of the stored B matrix are written by peer GPUs; ready_flags[src]
// reaching ready_gen marks source src's rows complete.  The producer warps poll the flags tile by tile.
extern "C" int llmq_gemm_ready(const void* A, const void* B, void* C, const void* bias,
                               int M, int N, int K, int ab_dtype, int b_dtype, int a_mn_major, int b_mn_major,
                               long long lda, long long ldb, long long ldc, int c_dtype, int bias_dtype, int accumulate,
                               const float* scale_a, const float* scale_b, float alpha, float* absmax_out, unsigned int* status,
                               int num_sms, const unsigned int* ready_flags, unsigned int ready_gen, int ready_rows_per_src,
                               double ready_limit_s, cudaStream_t stream) {
    return gemm_impl(A, B, C, bias, M, N, K, ab_dtype, b_dtype, a_mn_major, b_mn_major, lda, ldb, ldc, c_dtype, bias_dtype, accumulate, scale_a,
                     scale_b, alpha, absmax_out, status, num_sms, ready_flags, ready_gen, ready_rows_per_src, ready_limit_s, nullptr, stream);
}

// GEMM whose epilogue reduce-scatters the result over the data-parallel ranks (see gemm_tcgen05_2cta.cu).
// landing / counters: the landing buffer and the arrival counter of every rank (peer addresses); M must split
// into `world` row shards of a multiple of 32 rows, the output is bf16 with ldc == N.  `counter_target` is the
// value the local counter reaches after this call: every call adds world * (M / world / 32) * ceil(N / 256).
extern "C" int llmq_gemm_rs(const void* A, const void* B, void* C, int M, int N, int K, int ab_dtype, int b_dtype, int a_mn_major,
                            int b_mn_major, long long lda, long long ldb, int accumulate, const float* scale_a, const float* scale_b,
                            float alpha, unsigned int* status, int num_sms, void* const* landing, void* const* counters, int rank, int world,
                            unsigned int counter_target, void* shard_dst, int shard_accumulate, float shard_scale, float* norm_partials,
                            int num_partials, unsigned int seed, double limit_s, cudaStream_t stream) {
    if (world < 2 || world > 8 || M % world || (M / world) % 32 || M < 256 || N % 8) return -20;
    GemmParams rs{};
    rs.rs_world = world; rs.rs_rank = rank; rs.rs_shard_rows = M / world;
    for (int i = 0; i < world; ++i) { rs.rs_landing[i] = landing[i]; rs.rs_counter[i] = static_cast<unsigned int*>(counters[i]); }
    rs.rs_target = counter_target; rs.rs_dst = shard_dst; rs.rs_accumulate = shard_accumulate; rs.rs_scale = shard_scale;
    rs.rs_norm_partials = norm_partials; rs.rs_num_partials = num_partials > 0 ? num_partials : 1; rs.rs_seed = seed;
    rs.rs_limit_ns = static_cast<unsigned long long>(limit_s * 1e9);
    return gemm_impl(A, B, C, nullptr, M, N, K, ab_dtype, b_dtype, a_mn_major, b_mn_major, lda, ldb, N, 0, 0, accumulate, scale_a, scale_b, alpha,
                     nullptr, status, num_sms, nullptr, 0u, 0, 0.0, &rs, stream);
}

// GEMM with SwiGLU in the epilogue (see GemmParams::ep_mode).  mode 1: C[M, 2D] = A @ B^T with B = [up | gate] rows,
// aux[M, D] = swiglu(C).  mode 2: aux[M, 2D] ([up | gate] -> [d_up | d_gate], in place) from d(out) = A @ B^T, N = D.
// bf16 results; M >= 256, D a multiple of 128 (mode 1) / 8 (mode 2).  absmax_out follows the epilogue's output.
extern "C" int llmq_gemm_swiglu(const void* A, const void* B, void* C, void* aux, int mode, int M, int D, int K, int ab_dtype, int b_dtype,
                                int a_mn_major, int b_mn_major, long long lda, long long ldb, const float* scale_a, const float* scale_b,
                                float alpha, float* absmax_out, unsigned int* status, int num_sms, cudaStream_t stream) {
    if ((mode != 1 && mode != 2) || M < 256 || D % 8 || (mode == 1 && D % 128) || !aux || (mode == 1 && !C)) return -30;
    GemmParams ep{};
    ep.ep_mode = mode; ep.ep_ptr = aux; ep.ep_D = D;
    const int N = mode == 1 ? 2 * D : D;
    return gemm_impl(A, B, mode == 1 ? C : aux, nullptr, M, N, K, ab_dtype, b_dtype, a_mn_major, b_mn_major, lda, ldb, N, 0, 0, 0, scale_a, scale_b,
                     alpha, absmax_out, status, num_sms, nullptr, 0u, 0, 0.0, &ep, stream);
}

extern "C" unsigned int llmq_gemm_rs_arrivals(int M, int N, int world) {
    return static_cast<unsigned int>(world) * static_cast<unsigned int>(M / world / 32) * static_cast<unsigned int>((N + BN - 1) / BN);
}

static int gemm_impl(const void* A, const void* B, void* C, const void* bias,
                     int M, int N, int K, int ab_dtype, int b_dtype, int a_mn_major, int b_mn_major,
                     long long lda, long long ldb, long long ldc, int c_dtype, int bias_dtype, int accumulate,
                     const float* scale_a, const float* scale_b, float alpha, float* absmax_out, unsigned int* status,
                     int num_sms, const unsigned int* ready_flags, unsigned int ready_gen, int ready_rows_per_src,
                     double ready_limit_s, const GemmParams* rs, cudaStream_t stream) {
    auto width = [](int dt) { return dt == 0 ? 2 : (dt == 1 || dt == 2) ? 1 : (dt == 3 ? 4 : 0); };
    const int eb = width(ab_dtype);
    if (eb == 0 || width(b_dtype) != eb) return -2;
    if (eb == 4 && (rs != nullptr || ready_flags != nullptr)) return -2;      // fp32 operands: one-CTA kernel without fused collectives
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    // TMA needs 16-byte aligned bases and row pitches
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u)) return -3;
    if ((lda * eb) % 16 || (ldb * eb) % 16) return -4;

    CUtensorMap ta, tb;
    const int bk = 128 / eb;
    int rc;
    if (!a_mn_major) rc = llmq_encode_tmap_2d(&ta, A, eb, M, K, lda, BM);
    else             rc = llmq_encode_tmap_2d(&ta, A, eb, K, M, lda, bk);
    if (rc) return rc;
    // The CTA-pair kernel stages 128 rows of B per CTA; the one-CTA kernel stages all 256.
    const bool pair_kernel = eb != 4 && (rs != nullptr || ready_flags != nullptr || g_gemm_mode == 2 ||
                                         (g_gemm_mode == 0 && M >= 256 && static_cast<long long>(M) * N >= 256LL * 256 * 32));
    if (!b_mn_major) rc = llmq_encode_tmap_2d(&tb, B, eb, N, K, ldb, pair_kernel ? 128 : BN);
    else             rc = llmq_encode_tmap_2d(&tb, B, eb, K, N, ldb, bk);
    if (rc) return rc;

    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.elem_bytes = eb;
    p.a_mn_major = a_mn_major; p.b_mn_major = b_mn_major;
    p.a_fmt = ab_dtype == 3 ? 2 : (ab_dtype == 0 ? 1 : (ab_dtype == 1 ? 0 : 1));
    p.b_fmt = b_dtype == 3 ? 2 : (b_dtype == 0 ? 1 : (b_dtype == 1 ? 0 : 1));
    p.C = C; p.ldc = ldc; p.c_dtype = c_dtype; p.accumulate = accumulate;
    p.bias = bias; p.bias_dtype = bias_dtype;
    p.scale_a = scale_a; p.scale_b = scale_b; p.alpha = alpha;
    p.absmax_out = absmax_out; p.status = status;
    p.ready_flags = ready_flags; p.ready_gen = ready_gen; p.ready_rows_per_src = ready_rows_per_src > 0 ? ready_rows_per_src : 1;
    p.ready_limit_ns = static_cast<unsigned long long>(ready_limit_s * 1e9);
    if (rs) {
        p.ep_mode = rs->ep_mode; p.ep_ptr = rs->ep_ptr; p.ep_D = rs->ep_D;
        p.rs_world = rs->rs_world; p.rs_rank = rs->rs_rank; p.rs_shard_rows = rs->rs_shard_rows;
        for (int i = 0; i < 8; ++i) { p.rs_landing[i] = rs->rs_landing[i]; p.rs_counter[i] = rs->rs_counter[i]; }
        p.rs_target = rs->rs_target; p.rs_dst = rs->rs_dst; p.rs_accumulate = rs->rs_accumulate; p.rs_scale = rs->rs_scale;
        p.rs_norm_partials = rs->rs_norm_partials; p.rs_num_partials = rs->rs_num_partials; p.rs_seed = rs->rs_seed;
        p.rs_limit_ns = rs->rs_limit_ns;
    }

    if (pair_kernel) {
        // plain bf16 outputs leave the epilogue through TMA stores: a tensor map of C with 64-column x 32-row boxes
        CUtensorMap tc = ta;
        if (c_dtype == 0 && !accumulate && p.rs_world == 0 && p.ep_mode == 0 && (N % 8) == 0 && (ldc % 8) == 0 &&
            (reinterpret_cast<uintptr_t>(C) & 15u) == 0 && g_gemm_tma_store) {
            if (llmq_encode_tmap_2d(&tc, C, 2, M, N, ldc, 32) == 0) p.c_tma = 1;
        }
        return llmq_gemm_2cta_launch(ta, tb, tc, p, num_sms, stream);
    }

    static bool attr_set[64] = {};          // the attribute is per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set[dev & 63] = true;
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int k_iters = (K + bk - 1) / bk;
    int splits = 1;
    if (g_splitk_ws && tiles * 2 <= num_sms && k_iters >= 16) {
        splits = num_sms / tiles;
        if (splits > 8) splits = 8;
        if (splits > k_iters / 8) splits = k_iters / 8;
        while (splits > 1 && static_cast<long long>(splits) * M * N > g_splitk_floats) --splits;
        // every split must get at least one K step
        while (splits > 1 && (splits - 1) * ((k_iters + splits - 1) / splits) >= k_iters) --splits;
    }
    if (splits > 1) { p.k_splits = splits; p.partial = g_splitk_ws; }
    const int items = tiles * splits;
    int grid = items < num_sms ? items : num_sms;
    if (eb == 1)      gemm_tcgen05_kernel<1><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
    else if (eb == 2) gemm_tcgen05_kernel<0><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
    else              gemm_tcgen05_kernel<2><<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, p);
    if (splits > 1) {
        long long blocks = (static_cast<long long>(M) * N + 255) / 256;
        if (blocks > 4LL * num_sms) blocks = 4LL * num_sms;
        splitk_reduce_kernel<<<static_cast<unsigned int>(blocks), 256, 0, stream>>>(p, p.alpha);
    }
    return static_cast<int>(cudaGetLastError());
}
