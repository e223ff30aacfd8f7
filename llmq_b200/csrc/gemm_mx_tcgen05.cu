// Block-scaled (MX) e4m3 GEMM on tcgen05:  C[M,N] (+)= sum_k (A[m,k] * 2^(sa[m,k/32]-127)) * (B[n,k] * 2^(sb[n,k/32]-127)) (+ bias).
//
// Both operands are K-major e4m3 with one UE8M0 scale per 32 consecutive K elements
// (`tcgen05.mma.kind::mxf8f6f4.block_scale`): the tensor core applies the scales while it accumulates, so the
// dynamic range is set per 32-element block instead of per tensor, and no dequantisation factor is left for the
// epilogue.  The reference has no counterpart; its fp8 recipe is per-tensor (src/kernels/quant.cu:17-115).
//
// Structure: the persistent, warp-specialised layout of gemm_tcgen05.cu (TMA warp, MMA warp, 4 epilogue warps, two
// accumulators in tensor memory) with a 128 x 224 tile: two 224-column accumulators at columns 0 and 256 leave room
// for the scale factors, which the MMA reads from tensor memory (4 columns for A, 8 for B at columns 224..235).
//
// Scale-factor storage.  Per K stage (128 elements = 4 scale blocks) and per tile of rows the scales form chunks of
// 512 bytes = 128 rows x 4 blocks, byte offset (r % 32) * 16 + (r / 32) * 4 + block: exactly the image that
// `tcgen05.cp.32x128b.warpx4` copies to 4 tensor-memory columns (lane r % 32 of every lane quarter, column r / 32).
//   A: [K/128][ceil(M/128)][512]           B: [K/128][ceil(N/224)][2][512]   (rows 224..255 of a B tile are padding)
// quant_mx.cu writes this layout.  Scale bytes of padding rows must not be 0xFF (NaN); zero is used.
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"
#include "gemm_common.cuh"

using namespace sm100;

int llmq_encode_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, long long rows, long long cols, long long ld, int box_rows);

namespace {

constexpr int BM = 128;
constexpr int BN = 224;
constexpr int BK = 128;                          // e4m3 elements per stage = one 128-byte swizzle row
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * 128;                // 16 KiB
constexpr int B_BYTES = BN * 128;                // 28 KiB
constexpr int SFA_BYTES = 512, SFB_BYTES = 1024;
constexpr int SF_OFFSET = A_BYTES + B_BYTES;
constexpr int STAGE_BYTES = SF_OFFSET + 2048;    // keeps every stage on a 1024-byte boundary
constexpr int TX_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int ACC_STRIDE = 256;                  // accumulators at columns 0 and 256
constexpr int SFA_COL = 224, SFB_COL = 228;      // scale factors in the gap behind accumulator 0
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;

__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
// 32 rows x 16 bytes of shared memory (8-row groups 128 bytes apart, no swizzle) -> 4 tensor-memory columns, broadcast to
// the four lane quarters.
__device__ __forceinline__ void sf_copy(uint32_t tmem_col, uint32_t saddr) {
    const uint64_t desc = static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (static_cast<uint64_t>(128 >> 4) << 32) | (1ull << 46);
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col), "l"(desc) : "memory");
}
__device__ __forceinline__ void mma_mx(uint32_t tmem_d, uint32_t a_lo, uint32_t a_hi, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                       uint32_t sfa, uint32_t sfb, uint32_t accumulate) {
    asm volatile("{ .reg .pred p; .reg .b64 da, db; setp.ne.b32 p, %8, 0; mov.b64 da, {%1, %2}; mov.b64 db, {%3, %4};\n"
                 "  tcgen05.mma.cta_group::1.kind::mxf8f6f4.block_scale [%0], da, db, %5, [%6], [%7], p; }"
                 ::"r"(tmem_d), "r"(a_lo), "r"(a_hi), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(sfa), "r"(sfb), "r"(accumulate) : "memory");
}
// Instruction descriptor of the block-scaled kinds: e4m3 x e4m3, K-major, UE8M0 scales; byte `sf` of the scale words.
__host__ __device__ constexpr uint32_t mx_instr_desc(uint32_t m, uint32_t n, uint32_t sf) {
    return (sf << 4) | ((n >> 3) << 17) | (1u << 23) | ((m >> 4) << 24) | (sf << 29);
}

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
    constexpr int G = 16;
    const int per_group = G * tiles_n;
    const int group = t / per_group;
    const int first_m = group * G;
    const int gsz = min(tiles_m - first_m, G);
    const int r = t - group * per_group;
    tm = first_m + (r % gsz);
    tn = r / gsz;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const uint8_t* __restrict__ sfa, const uint8_t* __restrict__ sfb, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
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

    const int k_iters = p.K / BK;
    const int tiles_m = (p.M + BM - 1) / BM;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;

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
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
                for (int k = 0; k < k_iters; ++k) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrEmptyWait); ok = false; break; }
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    mbar_expect_tx(full_bar(stage), TX_BYTES);
                    tma_load_2d(sa, &tmap_a, full_bar(stage), k * BK, tm * BM);
                    tma_load_2d(sa + A_BYTES, &tmap_b, full_bar(stage), k * BK, tn * BN);
                    bulk_load(sa + SF_OFFSET, sfa + (static_cast<size_t>(k) * tiles_m + tm) * SFA_BYTES, SFA_BYTES, full_bar(stage));
                    bulk_load(sa + SF_OFFSET + SFA_BYTES, sfb + (static_cast<size_t>(k) * tiles_n + tn) * SFB_BYTES, SFB_BYTES, full_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t a_hi = desc_hi(1024), b_hi = desc_hi(1024);
            const uint32_t a_lo0 = desc_lo(smem_base, 16), b_lo0 = desc_lo(smem_base + A_BYTES, 16);
            const uint32_t t_sfa = tmem_base + SFA_COL, t_sfb = tmem_base + SFB_COL;
            int stage = 0; uint32_t phase = 0;
            int acc = 0; uint32_t acc_phase = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrTmemEmpty); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * ACC_STRIDE;
                for (int k = 0; k < k_iters; ++k) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { atomicOr(p.status, kErrFullWait); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t ssf = smem_base + stage * STAGE_BYTES + SF_OFFSET;
                    // copies and MMAs execute in issue order, so the scales of this stage replace the previous ones only
                    // after the MMAs that read those have run
                    sf_copy(t_sfa, ssf);
                    sf_copy(t_sfb, ssf + SFA_BYTES);
                    sf_copy(t_sfb + 4, ssf + SFA_BYTES + 512);
                    const uint32_t alo = a_lo0 + stage * (STAGE_BYTES >> 4);
                    const uint32_t blo = b_lo0 + stage * (STAGE_BYTES >> 4);
                    mma_mx(d_tmem, alo, a_hi, blo, b_hi, mx_instr_desc(BM, BN, 0), t_sfa, t_sfb, k > 0 ? 1u : 0u);
                    mma_mx(d_tmem, alo + 2, a_hi, blo + 2, b_hi, mx_instr_desc(BM, BN, 1), t_sfa, t_sfb, 1u);
                    mma_mx(d_tmem, alo + 4, a_hi, blo + 4, b_hi, mx_instr_desc(BM, BN, 2), t_sfa, t_sfb, 1u);
                    mma_mx(d_tmem, alo + 6, a_hi, blo + 6, b_hi, mx_instr_desc(BM, BN, 3), t_sfa, t_sfb, 1u);
                    mma_commit(empty_bar(stage));
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma_commit(tfull_bar(acc));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        const int q = warp & 3;
        float tmax = 0.f;
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
            int tm, tn; tile_coords(t, tiles_m, tiles_n, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { if (lane == 0) atomicOr(p.status, kErrTmemFull); ok = false; break; }
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_STRIDE;
            epilogue_rows(p, t_row, tm * BM + q * 32 + lane, tn * BN, BN, p.alpha, tmax);
            tc_fence_before_sync();
            mbar_arrive(tempty_bar(acc));
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

}  // namespace

// Rows per scale-factor tile of the B operand (the A operand uses 128).
extern "C" int llmq_gemm_mx_tile_n() { return BN; }

// A [M, K] and B [N, K] e4m3, K contiguous (lda / ldb in elements); sfa / sfb in the layout described at the top
// of this file; K a multiple of 128.  C bf16 (c_dtype 0) or fp32 (1), optional bias / accumulate / abs-max as llmq_gemm.
extern "C" int llmq_gemm_mx(const void* A, const void* B, const void* sfa, const void* sfb, void* C, const void* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int c_dtype, int bias_dtype, int accumulate, float alpha,
                            float* absmax_out, unsigned int* status, int num_sms, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % BK) return -5;
    if ((reinterpret_cast<uintptr_t>(A) & 15u) || (reinterpret_cast<uintptr_t>(B) & 15u) || (reinterpret_cast<uintptr_t>(sfa) & 15u) ||
        (reinterpret_cast<uintptr_t>(sfb) & 15u))
        return -3;
    if (lda % 16 || ldb % 16) return -4;
    CUtensorMap ta, tb;
    int rc = llmq_encode_tmap_2d(&ta, A, 1, M, K, lda, BM);
    if (rc) return rc;
    rc = llmq_encode_tmap_2d(&tb, B, 1, N, K, ldb, BN);
    if (rc) return rc;
    GemmParams p{};
    p.M = M; p.N = N; p.K = K; p.elem_bytes = 1;
    p.C = C; p.ldc = ldc; p.c_dtype = c_dtype; p.accumulate = accumulate;
    p.bias = bias; p.bias_dtype = bias_dtype; p.alpha = alpha;
    p.absmax_out = absmax_out; p.status = status;
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_mx_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set[dev & 63] = true;
    }
    const int tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = tiles < num_sms ? tiles : num_sms;
    gemm_mx_kernel<<<grid, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, static_cast<const uint8_t*>(sfa), static_cast<const uint8_t*>(sfb), p);
    return static_cast<int>(cudaGetLastError());
}
