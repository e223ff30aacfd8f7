// Causal grouped-query flash attention, forward and backward, on tcgen05 tensor cores (sm_100a).
//
// Operates directly on the packed post-RoPE tensor qkv (B, T, Hq + 2*Hkv, HS) through strided TMA maps,
// writes out (B, T, Hq, HS) and the per-row log-sum-exp (B, Hq, T); the backward pass produces the
// packed gradient dqkv with the same layout.  It takes the place of the cuDNN SDPA graphs and the
// scalar fallback kernel of the reference (src/kernels/cudnn_att.cpp:46-263, src/kernels/attention.cu).
//
// All three main kernels share one organisation.  A CTA owns a 128-row tile (queries for forward and dQ, keys for
// dK / dV) and has 19 warps: 16 compute warps (four warpgroups; thread (wg, r) owns row r = TMEM lane r and a quarter
// of the columns of every score tile), one warp whose lane 0 issues the score MMAs, one whose lane 0 issues the TMA
// loads and one whose lane 0 issues the accumulation MMAs.  MMA issue is synchronous with execution, so two issuing
// threads are needed to keep the tensor pipe busy while the other one waits for the compute warps.  Everything is
// handed over through mbarriers (one arrival per warp); score tiles are double buffered in tensor memory, the
// streamed operand (K / V, or Q / dO for dK / dV) sits in a ring of four shared-memory buffers.  Operands that are
// constant during a walk live in tensor memory as A operands where the 512 columns allow it (Q in forward, Q and dO
// in dQ; the bf16 probabilities of the forward pass too), so they are not re-read from shared memory by every MMA.
// The shared-memory tile of V / K / Q / dO doubles as an MN-major B operand, so no transposed copy is ever made.
//
// Backward is split into two deterministic kernels (no atomics):
//   * dK/dV: one CTA per (batch, kv head, 128 keys) walks over all query heads of the group and all
//     query blocks at or below the diagonal; dK and dV accumulate in TMEM across the whole walk.
//   * dQ   : one CTA per (batch, kv head, 128 queries) walks over the query heads of the group and their key
//     blocks; dQ accumulates in TMEM and is drained once per head.
// A small pre-pass computes delta = rowsum(dO * O).  Blocks with the longest walks are scheduled first.
#include <cstdlib>
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"

using namespace sm100;

namespace {

constexpr float kLog2e = 1.4426950408889634f;
// Backward kernels: four warpgroups share the 128 rows of a tile, each thread owns 16 score columns of its row, so
// every scheduler has four warps to hide the latency of the exp / TMEM / shared-memory chain.
constexpr int kBwdWarpgroups = 4;
constexpr int kBwdComputeThreads = 128 * kBwdWarpgroups;
constexpr int kBwdComputeWarps = kBwdComputeThreads / 32;
// + three single-lane helper warps: score-MMA issuer, TMA producer, accumulation-MMA issuer.  MMA issue is synchronous
// with execution (the queue is shallow), so two issuing threads keep the tensor pipe fed while the other one waits.
constexpr int kBwdThreads = kBwdComputeThreads + 96;
// barrier 1: the compute threads among themselves (barrier 0 is __syncthreads of the whole CTA)
// One arrival per warp (512 single arrivals on one shared-memory word would serialise): the lanes' earlier
// writes and fences are ordered before lane 0's releasing arrive by the warp barrier.
__device__ __forceinline__ void warp_arrive(uint32_t bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}
// barriers 2-5: the four warps (one per warpgroup) that share 32 rows of the tile
__device__ __forceinline__ void row_group_barrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(2 + group) : "memory"); }
__device__ __forceinline__ void compute_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kBwdComputeThreads) : "memory"); }

// 2^x with the hardware approximation (-inf -> 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

// low descriptor half of (base + byte offset); the base part is loop invariant, the offset a constant after unrolling
#define DLO(base, lbo, off) (desc_lo((base), (lbo)) + static_cast<uint32_t>((off) >> 4))
#define kDescHi desc_hi(1024)

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || !ptr) return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// bf16 tensor viewed as (B, T, W) with W contiguous; box = [box_rows along T][64 elements of W], 128B swizzle.
int encode_btw(CUtensorMap* out, const void* base, int B, int T, long long W, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return -1;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(W) * 2, static_cast<cuuint64_t>(W) * 2 * T};
    cuuint32_t box[3] = {64, static_cast<cuuint32_t>(box_rows), 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : 1000 + static_cast<int>(r);
}

struct AttnParams {
    int B, T, Hq, Hkv;
    float scale;                 // 1/sqrt(HS)
    bf16* out;                   // forward: (B,T,Hq,HS)
    float* lse;                  // (B,Hq,T), natural log
    const float* delta;          // (B,Hq,T)
    bf16* dqkv;                  // backward: packed gradient
    const bf16* qkv;             // backward: packed inputs and the output gradient as plain pointers
    const bf16* d_out;
    float* absmax;               // forward, optional: running abs-max of the output (for its fp8 quantisation)
    unsigned int* status;
};

// ------------------------------------------------------------------------------------------------
// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; HS / 8 lanes per row (one 16-byte load of each tensor per lane), so a
// warp covers 2 (HS = 128) or 4 (HS = 64) rows and every lane has work
template <int HS>
__global__ void __launch_bounds__(256)
attn_delta_kernel(float* __restrict__ delta, const bf16* __restrict__ o, const bf16* __restrict__ d_o, int B, int T, int Hq) {
    constexpr int LANES = HS / 8;                       // lanes per row
    static_assert(LANES == 8 || LANES == 16, "head sizes 64 and 128");
    const long long gid = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x;
    const long long w = gid / LANES;                    // row index over (b, t, h)
    const int sub = static_cast<int>(gid % LANES);
    const long long total = static_cast<long long>(B) * T * Hq;
    const bool active = w < total;
    float s = 0.f;
    if (active) {
        Vec16<bf16> a = Vec16<bf16>::load(o + w * HS + sub * 8), g = Vec16<bf16>::load(d_o + w * HS + sub * 8);
#pragma unroll
        for (int k = 0; k < 8; ++k) s += __bfloat162float(a.v[k]) * __bfloat162float(g.v[k]);
    }
#pragma unroll
    for (int off = LANES / 2; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (active && sub == 0) {
        const int h = static_cast<int>(w % Hq);
        const long long bt = w / Hq;
        const int t = static_cast<int>(bt % T);
        const long long b = bt / T;
        delta[(b * Hq + h) * T + t] = s;
    }
}

// ------------------------------------------------------------------------------------------------
// dK / dV.  Software pipeline over the (query head, query block) walk: while the threads turn S(it) / dP(it) into
// P^T and dS^T, the tensor core already computes S(it+1) / dP(it+1) (score tiles are double buffered in TMEM) and
// finishes dV / dK of tile it-1.  Q / dO tiles sit in a ring of four shared-memory buffers, loaded three tiles
// ahead; P^T / dS^T are kept in registers until the MMAs that read the previous pair have completed.
// 16 consecutive bf16 values (8 packed words): columns c0 .. c0+15 of row `row`
__device__ __forceinline__ void store_row_chunk16_swz_packed(uint8_t* tile, int row, int c0, const uint32_t (&v)[8]) {
    uint8_t* rowp = tile + row * 128;
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        const uint4 o = make_uint4(v[g * 4], v[g * 4 + 1], v[g * 4 + 2], v[g * 4 + 3]);
        const int u = (c0 >> 3) + g;
        *reinterpret_cast<uint4*>(rowp + ((u ^ (row & 7)) << 4)) = o;
    }
}
// 16 fp32 accumulator values of one row -> 16 bf16 in global memory (32 bytes)
__device__ __forceinline__ void store16_bf16(bf16* dst, const uint32_t (&r)[16]) {
#pragma unroll
    for (int g = 0; g < 2; ++g) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) ob[jj] = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * jj]), __uint_as_float(r[g * 8 + 2 * jj + 1]));
        *reinterpret_cast<uint4*>(dst + g * 8) = o;
    }
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

template <int HS>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_kv128,   // qkv, box 128 rows (K and V tiles)
                     const __grid_constant__ CUtensorMap tmap_q64,     // qkv, box 64 rows (Q tiles)
                     const __grid_constant__ CUtensorMap tmap_do64,    // dO, box 64 rows
                     const AttnParams p) {
    constexpr int BKV = 128, BQ = 64, NCH = HS / 64, NBUF = 4;
    constexpr int KV_BYTES = BKV * HS * 2, Q_BYTES = BQ * HS * 2, PT_BYTES = BKV * BQ * 2;
    constexpr uint32_t TMEM_COLS = 512;                       // S0 S1 | dP0 dP1 | dV | dK
    constexpr int CW = BQ / kBwdWarpgroups;                   // score columns per compute thread
    static_assert(CW == 16, "the column split below is written for 16 columns per thread");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = sK + KV_BYTES;
    uint8_t* sQ = sV + KV_BYTES;              // NBUF buffers
    uint8_t* sdO = sQ + NBUF * Q_BYTES;       // NBUF buffers
    uint8_t* sPT = sdO + NBUF * Q_BYTES;
    uint8_t* sdST = sPT + PT_BYTES;
    float* sLse = reinterpret_cast<float*>(sdST + PT_BYTES);      // [2][64] pre-multiplied by log2(e)
    float* sDelta = sLse + 2 * BQ;                                // [2][64]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + 2 * BQ);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    const bool issuer = warp == kBwdComputeWarps;             // MMA issuer (lane 0); its only other work is waiting
    const bool producer = warp == kBwdComputeWarps + 1;       // TMA producer (lane 0)
    const bool issuer2 = warp == kBwdComputeWarps + 2;        // issuer of the dV / dK MMAs (lane 0)
    const int wg = tid >> 7, r = tid & 127;                   // compute threads: column slice, row of the tile (TMEM lane)
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }
    // 1-D grid, key block slowest: the blocks with the longest walks (small kb) start first on every SM
    const int kb = blockIdx.x / (p.Hkv * p.B);
    const int kvh = (blockIdx.x % (p.Hkv * p.B)) % p.Hkv, b = (blockIdx.x % (p.Hkv * p.B)) / p.Hkv;
    const int G = p.Hq / p.Hkv;
    const int kv0 = kb * BKV;
    const int nqb = (p.T + BQ - 1) / BQ;
    const int qb_first = kv0 / BQ;
    const int per_head = nqb - qb_first;
    const int n_it = per_head * G;
    const int kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    // barriers: 0 kv | 1-4 q/dO ring | 5 sp (scores ready) | 6 acc (dV/dK MMAs of a tile done) | 7 p_ready (P^T/dS^T stored)
    //           8-9 s_free (score buffer read by all compute threads) | 10 second sp | 11-14 q/dO buffer free
    const uint32_t bar0 = smem_u32(bars);
    // Two score barriers, used alternately: the commit of tile it+2 needs every compute warp to have read tile it, so a
    // waiter can never miss a phase (with one barrier, tiles 0 and 1 can both complete before a slow warp looks).
    const uint32_t kv_bar = bar0, acc_bar = bar0 + 48, p_ready = bar0 + 56;
    auto sp_bar = [&](int it) { return (it & 1) ? bar0 + 80 : bar0 + 40; };
    auto qdo_bar = [&](int buf) { return bar0 + 8 + 8 * buf; };
    auto s_free = [&](int buf) { return bar0 + 64 + 8 * buf; };
    auto qdo_free = [&](int buf) { return bar0 + 88 + 8 * buf; };
    if (tid == 0) {
        for (int i = 0; i < 7; ++i) mbar_init(bar0 + 8 * i, 1);
        for (int i = 10; i < 15; ++i) mbar_init(bar0 + 8 * i, 1);
        mbar_init(p_ready, kBwdComputeWarps);
        mbar_init(s_free(0), kBwdComputeWarps);
        mbar_init(s_free(1), kBwdComputeWarps);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (issuer) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tdV = tmem + 4 * BQ, tdK = tmem + 4 * BQ + HS;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    auto tile_of = [&](int it, int& hq, int& qb) { hq = kvh * G + it / per_head; qb = qb_first + it % per_head; };
    bool ok = true;

    if (producer) {
        // ============================================================ TMA producer warp
        if ((tid & 31) == 0 && n_it > 0) {
            tma_prefetch_desc(&tmap_kv128); tma_prefetch_desc(&tmap_q64); tma_prefetch_desc(&tmap_do64);
            mbar_expect_tx(kv_bar, 2 * KV_BYTES);
            for (int c = 0; c < NCH; ++c) {
                tma_load_3d(smem_u32(sK) + c * (BKV * 128), &tmap_kv128, kv_bar, kcol + c * 64, kv0, b);
                tma_load_3d(smem_u32(sV) + c * (BKV * 128), &tmap_kv128, kv_bar, vcol + c * 64, kv0, b);
            }
            int hq = kvh * G, qb = qb_first;
            for (int it = 0; it < n_it; ++it) {
                const int buf = it % NBUF;
                // the buffer's previous tile, it - NBUF, has been consumed by its dV / dK MMAs
                if (it >= NBUF && !mbar_wait(qdo_free(buf), ((it / NBUF) - 1) & 1, abort_flag)) { atomicOr(p.status, kErrOther); break; }
                mbar_expect_tx(qdo_bar(buf), 2 * Q_BYTES);
                for (int c = 0; c < NCH; ++c) {
                    tma_load_3d(smem_u32(sQ) + buf * Q_BYTES + c * (BQ * 128), &tmap_q64, qdo_bar(buf), hq * HS + c * 64, qb * BQ, b);
                    tma_load_3d(smem_u32(sdO) + buf * Q_BYTES + c * (BQ * 128), &tmap_do64, qdo_bar(buf), hq * HS + c * 64, qb * BQ, b);
                }
                if (++qb == nqb) { qb = qb_first; ++hq; }
            }
        }
    } else if (issuer) {
        // ============================================================ MMA issuer warp
        if ((tid & 31) == 0 && n_it > 0) {
            const uint32_t idesc_st = make_instr_desc(1, 1, false, false, BKV, BQ);     // S^T = K Q^T, dP^T = V dO^T
            // scores of tile it: needs its Q / dO and, from tile 2 on, the score buffer read by every compute warp
            auto issue_sp = [&](int it) -> bool {
                const int buf = it % NBUF;
                if (!mbar_wait(qdo_bar(buf), (it / NBUF) & 1, abort_flag)) return false;
                if (it >= 2 && !mbar_wait(s_free(it & 1), ((it - 2) >> 1) & 1, abort_flag)) return false;
                tc_fence_after_sync();
                const uint32_t tS = tmem + (it & 1) * BQ, tdP = tmem + 2 * BQ + (it & 1) * BQ;
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tS, DLO(smem_u32(sK), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sQ) + buf * Q_BYTES, 16, (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi, idesc_st, k > 0);
                }
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tdP, DLO(smem_u32(sV), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sdO) + buf * Q_BYTES, 16, (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi, idesc_st, k > 0);
                }
                mma_commit(sp_bar(it));
                return true;
            };
            ok = mbar_wait(kv_bar, 0, abort_flag);
            for (int it = 0; it < n_it && ok; ++it) ok = issue_sp(it);
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else if (issuer2) {
        // ============================================================ dV / dK MMA issuer warp
        if ((tid & 31) == 0 && n_it > 0) {
            const uint32_t idesc_acc = make_instr_desc(1, 1, false, true, BKV, HS);      // dV += P^T dO, dK += dS^T Q
            for (int it = 0; it < n_it && ok; ++it) {
                if (!mbar_wait(p_ready, it & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const int buf = it % NBUF;
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k) {
                    mma_issue<false, false>(tdV, DLO(smem_u32(sPT), 16, k * 32), kDescHi,
                                            DLO(smem_u32(sdO) + buf * Q_BYTES, BQ * 128, k * (16 * 128)), kDescHi, idesc_acc, (it > 0 || k > 0));
                }
#pragma unroll
                for (int k = 0; k < BQ / 16; ++k) {
                    mma_issue<false, false>(tdK, DLO(smem_u32(sdST), 16, k * 32), kDescHi,
                                            DLO(smem_u32(sQ) + buf * Q_BYTES, BQ * 128, k * (16 * 128)), kDescHi, idesc_acc, (it > 0 || k > 0));
                }
                mma_commit(acc_bar);
                mma_commit(qdo_free(buf));
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else {
        // ============================================================ compute warps
        auto load_stats = [&](int it) {                         // lse (threads 0-63) and delta (64-127) of tile it
            if (tid >= 128) return;
            int hq, qb; tile_of(it, hq, qb);
            const int q = qb * BQ + (tid & 63);
            const long long si = (static_cast<long long>(b) * p.Hq + hq) * p.T + q;
            float* dst = (tid < 64 ? sLse : sDelta) + (it & 1) * BQ + (tid & 63);
            if (tid < 64) *dst = q < p.T ? p.lse[si] * kLog2e : INFINITY;
            else *dst = q < p.T ? p.delta[si] * p.scale : 0.f;       // delta pre-multiplied by the softmax scale
        };
        const float sl2 = p.scale * kLog2e;
        const int kv_row = kv0 + r;
        const int c0 = wg * CW;
        if (n_it > 0) load_stats(0);
        compute_barrier();
        // One tile; false when a wait ran out.  The caller still runs the barrier of every remaining tile, so that a
        // failure can never leave part of the CTA behind at a barrier.
        auto tile_body = [&](int it) -> bool {
            int hq, qb; tile_of(it, hq, qb);
            if (it + 1 < n_it) load_stats(it + 1);             // read after the barrier at the end of this tile
            if (!mbar_wait(sp_bar(it), (it >> 1) & 1, abort_flag)) return false;
            tc_fence_after_sync();
            const bool diag = qb * BQ < kv0 + BKV;              // some (kv, q) pairs have q < kv
            const float* lse_t = sLse + (it & 1) * BQ;
            const float* delta_t = sDelta + (it & 1) * BQ;
            const uint32_t tS = tmem + (it & 1) * BQ, tdP = tmem + 2 * BQ + (it & 1) * BQ;
            uint32_t ptp[CW / 2], dsp[CW / 2];
            {
                uint32_t rs[CW], rp[CW];
                tmem_ld_32x32b_x16(tS + lane_off + c0, rs);
                tmem_ld_32x32b_x16(tdP + lane_off + c0, rp);
                tmem_ld_wait();
                tc_fence_before_sync();
                warp_arrive(s_free(it & 1));                    // this score buffer may be overwritten
                float lse_c[CW], del_c[CW];
#pragma unroll
                for (int i = 0; i < CW; i += 4) {
                    *reinterpret_cast<float4*>(lse_c + i) = *reinterpret_cast<const float4*>(lse_t + c0 + i);
                    *reinterpret_cast<float4*>(del_c + i) = *reinterpret_cast<const float4*>(delta_t + c0 + i);
                }
                float pv[CW], ds[CW];
#pragma unroll
                for (int i = 0; i < CW; ++i) {
                    pv[i] = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -lse_c[i]));
                    ds[i] = fmaf(__uint_as_float(rp[i]), p.scale, -del_c[i]);
                }
                if (diag) {                                     // only tiles that touch the diagonal pay for the mask
                    const int lim = kv_row - qb * BQ - c0;      // columns below lim are above the diagonal (q < kv)
#pragma unroll
                    for (int i = 0; i < CW; ++i) if (i < lim) pv[i] = 0.f;
                }
#pragma unroll
                for (int i = 0; i < CW; i += 2) {
                    ptp[i / 2] = pack_bf16x2(pv[i], pv[i + 1]);
                    dsp[i / 2] = pack_bf16x2(pv[i] * ds[i], pv[i + 1] * ds[i + 1]);
                }
            }
            // P^T / dS^T of tile it-1 are read by its dV / dK MMAs until acc_bar completes
            if (it > 0 && !mbar_wait(acc_bar, (it - 1) & 1, abort_flag)) return false;
            store_row_chunk16_swz_packed(sPT, r, c0, ptp);
            store_row_chunk16_swz_packed(sdST, r, c0, dsp);
            fence_proxy_async_smem();
            warp_arrive(p_ready);
            return true;
        };
        for (int it = 0; it < n_it; ++it) {
            if (ok) ok = tile_body(it);
            compute_barrier();                                  // statistics of tile it+1 visible to all compute threads
        }
        if (ok && n_it > 0) ok = mbar_wait(acc_bar, (n_it - 1) & 1, abort_flag);
        tc_fence_after_sync();
        if (!ok && r == 0) atomicOr(p.status, kErrOther);
        if (ok && n_it > 0) {
            // The TMEM loads are warp-collective: every lane executes them, only the stores are predicated.
            const bool row_ok = kv_row < p.T;
            const int H = p.Hq + 2 * p.Hkv;
            const long long rbase = (static_cast<long long>(b) * p.T + (row_ok ? kv_row : 0)) * H;
            bf16* dk = p.dqkv + (rbase + p.Hq + kvh) * HS;
            bf16* dv = p.dqkv + (rbase + p.Hq + p.Hkv + kvh) * HS;
            __syncwarp();
            constexpr int ECW = HS / kBwdWarpgroups;           // output columns per thread
#pragma unroll
            for (int c = 0; c < ECW; c += 16) {
                const int col = wg * ECW + c;
                uint32_t rk[16], rv[16];
                tmem_ld_32x32b_x16(tdK + lane_off + col, rk);
                tmem_ld_32x32b_x16(tdV + lane_off + col, rv);
                tmem_ld_wait();
                if (row_ok) {
                    store16_bf16(dk + col, rk);
                    store16_bf16(dv + col, rv);
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (issuer) tmem_dealloc(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------
// dQ.  One CTA owns 128 query rows of one kv head and walks over the query heads of that group, and for every head
// over the key tiles up to the diagonal, so the start-up and drain costs of a CTA are paid once per group instead
// of once per head.  Q and dO of the current head live in tensor memory as the A operands of the score MMAs (they
// are constant during a key walk), K / V tiles stream through a ring of four shared-memory buffers three tiles
// ahead of the MMAs, S / dP are double buffered in TMEM, dQ accumulates in TMEM and is drained once per head.
template <int HS>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_kv64,    // qkv, box 64 rows
                   const AttnParams p) {
    constexpr int BQ = 128, BKV = 64, NCH = HS / 64, NBUF = 4;
    constexpr int KV_BYTES = BKV * HS * 2, DS_BYTES = BQ * BKV * 2;
    constexpr uint32_t TMEM_COLS = 512;                       // Q | dO (bf16 pairs, A operands) | S0 S1 | dP0 dP1 | dQ
    constexpr int CW = BKV / kBwdWarpgroups;
    static_assert(CW == 16, "the column split below is written for 16 columns per thread");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;                       // NBUF buffers
    uint8_t* sV = sK + NBUF * KV_BYTES;       // NBUF buffers
    uint8_t* sdS = sV + NBUF * KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + DS_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    const bool issuer = warp == kBwdComputeWarps, producer = warp == kBwdComputeWarps + 1, issuer2 = warp == kBwdComputeWarps + 2;
    const int wg = tid >> 7, r = tid & 127;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }
    const int nqb = (p.T + BQ - 1) / BQ;
    const int qb = nqb - 1 - blockIdx.x / (p.Hkv * p.B);        // 1-D grid, longest key walks first
    const int kvh = (blockIdx.x % (p.Hkv * p.B)) % p.Hkv, b = (blockIdx.x % (p.Hkv * p.B)) / p.Hkv;
    const int G = p.Hq / p.Hkv;
    const int q0 = qb * BQ;
    const int n_kv = min((p.T + BKV - 1) / BKV, (q0 + BQ) / BKV);
    const int total = n_kv * G;                                 // tiles of the whole walk, t = g * n_kv + j
    const int kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    // barriers: 0 head_ready | 1-4 k/v ring | 5, 10 sp (alternating) | 6 dq (dQ MMA of a tile done) | 7 p_ready | 8-9 s_free
    //           11-14 k/v buffer free
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t head_ready = bar0, dq_bar = bar0 + 48, p_ready = bar0 + 56;
    auto sp_bar = [&](int t) { return (t & 1) ? bar0 + 80 : bar0 + 40; };        // alternating, see the dK / dV kernel
    auto kv_bar = [&](int buf) { return bar0 + 8 + 8 * buf; };
    auto s_free = [&](int buf) { return bar0 + 64 + 8 * buf; };
    auto kv_free = [&](int buf) { return bar0 + 88 + 8 * buf; };
    if (tid == 0) {
        for (int i = 1; i < 7; ++i) mbar_init(bar0 + 8 * i, 1);
        for (int i = 10; i < 15; ++i) mbar_init(bar0 + 8 * i, 1);
        mbar_init(head_ready, kBwdComputeWarps);
        mbar_init(p_ready, kBwdComputeWarps);
        mbar_init(s_free(0), kBwdComputeWarps);
        mbar_init(s_free(1), kBwdComputeWarps);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (issuer) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tQ = tmem, tdO = tmem + HS / 2, tS0 = tmem + HS, tdP0 = tmem + HS + 2 * BKV, tdQ = tmem + HS + 4 * BKV;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;

    if (producer) {
        // ============================================================ TMA producer warp
        if ((tid & 31) == 0 && total > 0) {
            tma_prefetch_desc(&tmap_kv64);
            int j = 0;
            for (int t = 0; t < total; ++t) {
                const int buf = t % NBUF;
                // the buffer's previous tile, t - NBUF, has been consumed by its dQ MMA
                if (t >= NBUF && !mbar_wait(kv_free(buf), ((t / NBUF) - 1) & 1, abort_flag)) { atomicOr(p.status, kErrOther); break; }
                mbar_expect_tx(kv_bar(buf), 2 * KV_BYTES);
                for (int c = 0; c < NCH; ++c) {
                    tma_load_3d(smem_u32(sK) + buf * KV_BYTES + c * (BKV * 128), &tmap_kv64, kv_bar(buf), kcol + c * 64, j * BKV, b);
                    tma_load_3d(smem_u32(sV) + buf * KV_BYTES + c * (BKV * 128), &tmap_kv64, kv_bar(buf), vcol + c * 64, j * BKV, b);
                }
                if (++j == n_kv) j = 0;
            }
        }
    } else if (issuer) {
        // ============================================================ MMA issuer warp
        if ((tid & 31) == 0 && total > 0) {
            const uint32_t idesc_s = make_instr_desc(1, 1, false, false, BQ, BKV);
            // scores of tile t; needs its K / V tile and, from t = 2 on, the score buffer read by every compute warp
            auto issue_sp = [&](int t) -> bool {
                const int buf = t % NBUF;
                if (!mbar_wait(kv_bar(buf), (t / NBUF) & 1, abort_flag)) return false;
                if (t >= 2 && !mbar_wait(s_free(t & 1), ((t - 2) >> 1) & 1, abort_flag)) return false;
                tc_fence_after_sync();
                const uint32_t tS = tS0 + (t & 1) * BKV, tdP = tdP0 + (t & 1) * BKV;
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue_f16_tmem_a(tS, tQ + k * 8, DLO(smem_u32(sK) + buf * KV_BYTES, 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                         idesc_s, k > 0);
                }
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue_f16_tmem_a(tdP, tdO + k * 8, DLO(smem_u32(sV) + buf * KV_BYTES, 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                         idesc_s, k > 0);
                }
                mma_commit(sp_bar(t));
                return true;
            };
            int g = 0, j = 0;
            for (int t = 0; t < total && ok; ++t) {
                // the first tile of a head needs that head's Q / dO in tensor memory
                if (j == 0 && !mbar_wait(head_ready, g & 1, abort_flag)) { ok = false; break; }
                ok = issue_sp(t);
                if (++j == n_kv) { j = 0; ++g; }
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else if (issuer2) {
        // ============================================================ dQ MMA issuer warp
        if ((tid & 31) == 0 && total > 0) {
            const uint32_t idesc_dq = make_instr_desc(1, 1, false, true, BQ, HS);
            int j = 0;
            for (int t = 0; t < total && ok; ++t) {
                if (!mbar_wait(p_ready, t & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const int buf = t % NBUF;
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    mma_issue<false, false>(tdQ, DLO(smem_u32(sdS), 16, k * 32), kDescHi,
                                            DLO(smem_u32(sK) + buf * KV_BYTES, BKV * 128, k * (16 * 128)), kDescHi, idesc_dq, (j > 0 || k > 0));
                }
                mma_commit(dq_bar);
                mma_commit(kv_free(buf));
                if (++j == n_kv) j = 0;
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else {
        // ============================================================ compute warps
        const float sl2 = p.scale * kLog2e;
        const int row = q0 + r;
        const bool row_ok = row < p.T;
        const int c0 = wg * CW;
        const int H = p.Hq + 2 * p.Hkv;
        const bool stores_qdo = wg < HS / 32;                   // uniform per warp: the TMEM stores are warp-collective
        constexpr int ECW = HS / kBwdWarpgroups;                // dQ columns per thread
        // this thread's 32-element slices of the Q and dO rows of head hq (16 packed words each)
        auto load_qdo = [&](int hq, uint32_t (&wq)[16], uint32_t (&wo)[16]) {
            if (stores_qdo && row_ok) {
                const uint4* gq = reinterpret_cast<const uint4*>(p.qkv + ((static_cast<long long>(b) * p.T + row) * H + hq) * HS + wg * 32);
                const uint4* go = reinterpret_cast<const uint4*>(p.d_out + ((static_cast<long long>(b) * p.T + row) * p.Hq + hq) * HS + wg * 32);
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint4 x = __ldg(gq + q4), y = __ldg(go + q4);
                    wq[4 * q4] = x.x; wq[4 * q4 + 1] = x.y; wq[4 * q4 + 2] = x.z; wq[4 * q4 + 3] = x.w;
                    wo[4 * q4] = y.x; wo[4 * q4 + 1] = y.y; wo[4 * q4 + 2] = y.z; wo[4 * q4 + 3] = y.w;
                }
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 16; ++q4) { wq[q4] = 0u; wo[q4] = 0u; }
            }
        };
        auto store_qdo = [&](const uint32_t (&wq)[16], const uint32_t (&wo)[16]) {
            if (stores_qdo) {
                tmem_st_32x32b_x16(tQ + lane_off + wg * 16, wq);
                tmem_st_32x32b_x16(tdO + lane_off + wg * 16, wo);
                tmem_st_wait();
            }
            tc_fence_before_sync();
            warp_arrive(head_ready);
        };
        uint32_t wq[16], wo[16];
        load_qdo(kvh * G, wq, wo);
        store_qdo(wq, wo);
        for (int g = 0; g < G && ok; ++g) {
            const int h = kvh * G + g;
            if (g + 1 < G) load_qdo(h + 1, wq, wo);             // prefetch: consumed when this head's walk is over
            const long long si = (static_cast<long long>(b) * p.Hq + h) * p.T + row;
            const float lse2 = row_ok ? p.lse[si] * kLog2e : INFINITY;
            const float delta_s = row_ok ? p.delta[si] * p.scale : 0.f;
            for (int j = 0; j < n_kv && ok; ++j) {
                const int t = g * n_kv + j;
                if (!mbar_wait(sp_bar(t), (t >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const bool diag = (j + 1) * BKV > q0;
                const uint32_t tS = tS0 + (t & 1) * BKV, tdP = tdP0 + (t & 1) * BKV;
                uint32_t dsp[CW / 2];
                {
                    uint32_t rs[CW], rp[CW];
                    tmem_ld_32x32b_x16(tS + lane_off + c0, rs);
                    tmem_ld_32x32b_x16(tdP + lane_off + c0, rp);
                    tmem_ld_wait();
                    tc_fence_before_sync();
                    warp_arrive(s_free(t & 1));
                    float pv[CW];
#pragma unroll
                    for (int i = 0; i < CW; ++i) pv[i] = fast_exp2(fmaf(__uint_as_float(rs[i]), sl2, -lse2));
                    if (diag) {
                        const int lim = row - j * BKV - c0;     // columns above lim are beyond the diagonal (kv > q)
#pragma unroll
                        for (int i = 0; i < CW; ++i) if (i > lim) pv[i] = 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < CW; i += 2)
                        dsp[i / 2] = pack_bf16x2(pv[i] * fmaf(__uint_as_float(rp[i]), p.scale, -delta_s),
                                                 pv[i + 1] * fmaf(__uint_as_float(rp[i + 1]), p.scale, -delta_s));
                }
                // dS of tile t-1 is read by its dQ MMA until dq_bar completes
                if (t > 0 && !mbar_wait(dq_bar, (t - 1) & 1, abort_flag)) { ok = false; break; }
                store_row_chunk16_swz_packed(sdS, r, c0, dsp);
                fence_proxy_async_smem();
                warp_arrive(p_ready);
            }
            if (!ok) break;
            // ---- the head's walk is over: drain dQ, hand the next head's Q / dO to the tensor core, then store
            if (!mbar_wait(dq_bar, (g * n_kv + n_kv - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            uint32_t acc[ECW];
            __syncwarp();
#pragma unroll
            for (int c = 0; c < ECW; c += 16) tmem_ld_32x32b_x16(tdQ + lane_off + wg * ECW + c, *reinterpret_cast<uint32_t(*)[16]>(acc + c));
            tmem_ld_wait();
            if (g + 1 < G) store_qdo(wq, wo);
            if (row_ok) {
                bf16* dq = p.dqkv + ((static_cast<long long>(b) * p.T + row) * H + h) * HS + wg * ECW;
#pragma unroll
                for (int c = 0; c < ECW; c += 16) store16_bf16(dq + c, *reinterpret_cast<const uint32_t(*)[16]>(acc + c));
            }
        }
        if (!ok && r == 0) atomicOr(p.status, kErrOther);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (issuer) tmem_dealloc(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------
// Forward.  Same organisation as the dQ kernel: one CTA owns 128 query rows of one kv head and walks over the query
// heads of the group and, per head, over the 64-key tiles up to the diagonal.  Q lives in tensor memory as the A
// operand of S = Q K^T; the bf16 probabilities go back into tensor memory (two buffers) and are the A operand of
// O += P V, so neither Q nor P is ever re-read from shared memory; K / V stream through a ring of four buffers.
// Four threads share a row (16 score columns each): the row maximum is exchanged through shared memory once per
// tile, the row sum only at the end of a head.  O is rescaled only when a row maximum moved by more than 2^8 since
// the last rescale (the stale maximum keeps P <= 256, exact after the final normalisation).
template <int N> __device__ __forceinline__ void tmem_ld_cols(uint32_t addr, uint32_t (&r)[N]) {
    if constexpr (N == 32) tmem_ld_32x32b_x32(addr, r); else tmem_ld_32x32b_x16(addr, r);
}
template <int N> __device__ __forceinline__ void tmem_st_cols(uint32_t addr, const uint32_t (&r)[N]) {
    if constexpr (N == 32) tmem_st_32x32b_x32(addr, r); else tmem_st_32x32b_x16(addr, r);
}

template <int HS>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_kv64,    // qkv, box 64 rows
                const AttnParams p) {
    constexpr int BQ = 128, BKV = 64, NCH = HS / 64, NBUF = 4;
    constexpr int KV_BYTES = BKV * HS * 2;
    constexpr uint32_t TMEM_COLS = 512;                       // Q | S0 S1 | P0 P1 (bf16 pairs) | O
    constexpr int CW = BKV / kBwdWarpgroups;                  // score columns per thread
    constexpr int ECW = HS / kBwdWarpgroups;                  // output columns per thread
    constexpr float kRescaleThreshold = 8.f;                  // in log2 units
    static_assert(CW == 16, "the column split below is written for 16 columns per thread");
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;                       // NBUF buffers
    uint8_t* sV = sK + NBUF * KV_BYTES;       // NBUF buffers
    float* sMax = reinterpret_cast<float*>(sV + NBUF * KV_BYTES);     // [2][4][128] slice maxima of a tile
    float* sSum = sMax + 2 * kBwdWarpgroups * BQ;                      // [4][128] slice sums of a head
    uint64_t* bars = reinterpret_cast<uint64_t*>(sSum + kBwdWarpgroups * BQ);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 20);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    const bool issuer = warp == kBwdComputeWarps, producer = warp == kBwdComputeWarps + 1, issuer2 = warp == kBwdComputeWarps + 2;
    const int wg = tid >> 7, r = tid & 127;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }
    const int nqb = (p.T + BQ - 1) / BQ;
    const int qb = nqb - 1 - blockIdx.x / (p.Hkv * p.B);        // 1-D grid, longest key walks first
    const int kvh = (blockIdx.x % (p.Hkv * p.B)) % p.Hkv, b = (blockIdx.x % (p.Hkv * p.B)) / p.Hkv;
    const int G = p.Hq / p.Hkv;
    const int q0 = qb * BQ;
    const int n_kv = min((p.T + BKV - 1) / BKV, (q0 + BQ) / BKV);
    const int total = n_kv * G;                                 // tiles of the whole walk, t = g * n_kv + j
    const int kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    // barriers: 0 head_ready | 1-4 k/v ring | 5-6 s (scores ready) | 7-8 s_free | 9-10 p_ready | 11-12 p_free (PV of the
    //           tile done) | 13-16 k/v buffer free.  Two-entry sets alternate with the tile parity.
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t head_ready = bar0;
    auto kv_bar = [&](int buf) { return bar0 + 8 + 8 * buf; };
    auto s_bar = [&](int t) { return bar0 + 40 + 8 * (t & 1); };
    auto s_free = [&](int t) { return bar0 + 56 + 8 * (t & 1); };
    auto p_ready = [&](int t) { return bar0 + 72 + 8 * (t & 1); };
    auto p_free = [&](int t) { return bar0 + 88 + 8 * (t & 1); };
    auto kv_free = [&](int buf) { return bar0 + 104 + 8 * buf; };
    if (tid == 0) {
        mbar_init(head_ready, kBwdComputeWarps);
        for (int i = 0; i < 4; ++i) { mbar_init(kv_bar(i), 1); mbar_init(kv_free(i), 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(s_bar(i), 1); mbar_init(p_free(i), 1);
            mbar_init(s_free(i), kBwdComputeWarps); mbar_init(p_ready(i), kBwdComputeWarps);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (issuer) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tQ = tmem, tS0 = tmem + HS / 2, tP0 = tS0 + 2 * BKV, tO = tP0 + BKV;
    const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;

    if (producer) {
        // ============================================================ TMA producer warp
        if ((tid & 31) == 0 && total > 0) {
            tma_prefetch_desc(&tmap_kv64);
            int j = 0;
            for (int t = 0; t < total; ++t) {
                const int buf = t % NBUF;
                if (t >= NBUF && !mbar_wait(kv_free(buf), ((t / NBUF) - 1) & 1, abort_flag)) { atomicOr(p.status, kErrOther); break; }
                mbar_expect_tx(kv_bar(buf), 2 * KV_BYTES);
                for (int c = 0; c < NCH; ++c) {
                    tma_load_3d(smem_u32(sK) + buf * KV_BYTES + c * (BKV * 128), &tmap_kv64, kv_bar(buf), kcol + c * 64, j * BKV, b);
                    tma_load_3d(smem_u32(sV) + buf * KV_BYTES + c * (BKV * 128), &tmap_kv64, kv_bar(buf), vcol + c * 64, j * BKV, b);
                }
                if (++j == n_kv) j = 0;
            }
        }
    } else if (issuer) {
        // ============================================================ S = Q K^T issuer warp
        if ((tid & 31) == 0 && total > 0) {
            const uint32_t idesc_s = make_instr_desc(1, 1, false, false, BQ, BKV);
            int g = 0, j = 0;
            for (int t = 0; t < total && ok; ++t) {
                const int buf = t % NBUF;
                if (j == 0 && !mbar_wait(head_ready, g & 1, abort_flag)) { ok = false; break; }       // this head's Q is in tensor memory
                if (!mbar_wait(kv_bar(buf), (t / NBUF) & 1, abort_flag)) { ok = false; break; }
                if (t >= 2 && !mbar_wait(s_free(t), ((t - 2) >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue_f16_tmem_a(tS0 + (t & 1) * BKV, tQ + k * 8,
                                         DLO(smem_u32(sK) + buf * KV_BYTES, 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi, idesc_s, k > 0);
                }
                mma_commit(s_bar(t));
                if (++j == n_kv) { j = 0; ++g; }
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else if (issuer2) {
        // ============================================================ O += P V issuer warp
        if ((tid & 31) == 0 && total > 0) {
            const uint32_t idesc_o = make_instr_desc(1, 1, false, true, BQ, HS);
            int j = 0;
            for (int t = 0; t < total && ok; ++t) {
                if (!mbar_wait(p_ready(t), (t >> 1) & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const int buf = t % NBUF;
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    mma_issue_f16_tmem_a(tO, tP0 + (t & 1) * (BKV / 2) + k * 8,
                                         DLO(smem_u32(sV) + buf * KV_BYTES, BKV * 128, k * (16 * 128)), kDescHi, idesc_o, (j > 0 || k > 0));
                }
                mma_commit(p_free(t));
                mma_commit(kv_free(buf));
                if (++j == n_kv) j = 0;
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else {
        // ============================================================ compute warps
        const float sl2 = p.scale * kLog2e;
        const int row = q0 + r;
        const bool row_ok = row < p.T;
        const int c0 = wg * CW;
        const int H = p.Hq + 2 * p.Hkv;
        const bool stores_q = wg < HS / 32;                     // uniform per warp: the TMEM stores are warp-collective
        auto load_q = [&](int hq, uint32_t (&wq)[16]) {
            if (stores_q && row_ok) {
                const uint4* gq = reinterpret_cast<const uint4*>(p.qkv + ((static_cast<long long>(b) * p.T + row) * H + hq) * HS + wg * 32);
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) {
                    const uint4 x = __ldg(gq + q4);
                    wq[4 * q4] = x.x; wq[4 * q4 + 1] = x.y; wq[4 * q4 + 2] = x.z; wq[4 * q4 + 3] = x.w;
                }
            } else {
#pragma unroll
                for (int q4 = 0; q4 < 16; ++q4) wq[q4] = 0u;
            }
        };
        auto store_q = [&](const uint32_t (&wq)[16]) {
            if (stores_q) { tmem_st_32x32b_x16(tQ + lane_off + wg * 16, wq); tmem_st_wait(); }
            tc_fence_before_sync();
            warp_arrive(head_ready);
        };
        uint32_t wq[16];
        load_q(kvh * G, wq);
        store_q(wq);
        float m_ref = -INFINITY, l_part = 0.f, omax = 0.f;
        for (int g = 0; g < G; ++g) {
            const int h = kvh * G + g;
            if (g + 1 < G) load_q(h + 1, wq);                   // prefetch: consumed when this head's walk is over
            m_ref = -INFINITY; l_part = 0.f;
            for (int j = 0; j < n_kv; ++j) {
                const int t = g * n_kv + j;
                float sv[CW];
                // ---- scores of this thread's 16 columns, masked; slice maximum to shared memory
                if (ok) {
                    ok = mbar_wait(s_bar(t), (t >> 1) & 1, abort_flag);
                    if (ok) {
                        tc_fence_after_sync();
                        uint32_t rs[CW];
                        tmem_ld_32x32b_x16(tS0 + (t & 1) * BKV + lane_off + c0, rs);
                        tmem_ld_wait();
                        tc_fence_before_sync();
                        warp_arrive(s_free(t));
#pragma unroll
                        for (int i = 0; i < CW; ++i) sv[i] = __uint_as_float(rs[i]);
                        if ((j + 1) * BKV > q0) {               // tile touches the diagonal
                            const int lim = row - j * BKV - c0; // columns above lim are beyond the diagonal (kv > q)
#pragma unroll
                            for (int i = 0; i < CW; ++i) if (i > lim) sv[i] = -INFINITY;
                        }
                        float mx = sv[0];
#pragma unroll
                        for (int i = 1; i < CW; ++i) mx = fmaxf(mx, sv[i]);
                        sMax[((t & 1) * kBwdWarpgroups + wg) * BQ + r] = mx;
                    }
                }
                row_group_barrier(warp & 3);                              // every thread takes part, also after a failed wait
                if (!ok) continue;
                float m_tile = -INFINITY;
#pragma unroll
                for (int w4 = 0; w4 < kBwdWarpgroups; ++w4) m_tile = fmaxf(m_tile, sMax[((t & 1) * kBwdWarpgroups + w4) * BQ + r]);
                // ---- lazy rescale.  The TMEM loads / stores are warp-collective, so the decision is taken per warp; the
                // four warps that share rows see the same numbers and therefore decide alike.
                const bool need = j == 0 || (m_tile - m_ref) * sl2 > kRescaleThreshold;
                if (__any_sync(0xffffffffu, need)) {
                    const float m_new = fmaxf(m_ref, m_tile);
                    if (j > 0) {
                        const float alpha = fast_exp2((m_ref - m_new) * sl2);
                        l_part *= alpha;
                        // O is being accumulated by the PV MMAs of tile t-1: wait for them, then scale this thread's columns
                        if (!mbar_wait(p_free(t - 1), ((t - 1) >> 1) & 1, abort_flag)) { ok = false; continue; }
                        tc_fence_after_sync();
                        uint32_t ro[ECW];
                        tmem_ld_cols<ECW>(tO + lane_off + wg * ECW, ro);
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < ECW; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
                        tmem_st_cols<ECW>(tO + lane_off + wg * ECW, ro);
                        tmem_st_wait();
                    }
                    m_ref = m_new;
                }
                // ---- probabilities -> bf16 -> tensor memory (A operand of the PV MMA)
                const float moff = m_ref * sl2;
                uint32_t pw[CW / 2];
                float sum = 0.f;
#pragma unroll
                for (int i = 0; i < CW; i += 2) {
                    const float p0 = fast_exp2(fmaf(sv[i], sl2, -moff)), p1 = fast_exp2(fmaf(sv[i + 1], sl2, -moff));
                    sum += p0 + p1;
                    pw[i / 2] = pack_bf16x2(p0, p1);
                }
                l_part += sum;
                // this P buffer was read by the PV MMAs of tile t-2
                if (t >= 2 && !mbar_wait(p_free(t), ((t - 2) >> 1) & 1, abort_flag)) { ok = false; continue; }
                tc_fence_after_sync();
                __syncwarp();
                tmem_st_32x32b_x8(tP0 + (t & 1) * (BKV / 2) + lane_off + wg * (CW / 2), pw);
                tmem_st_wait();
                tc_fence_before_sync();
                warp_arrive(p_ready(t));
            }
            // ---- the head's walk is over: row sums, normalise, store; hand the next head's Q to the tensor core
            const int t_last = g * n_kv + n_kv - 1;
            if (ok) ok = mbar_wait(p_free(t_last), (t_last >> 1) & 1, abort_flag);
            tc_fence_after_sync();
            sSum[wg * BQ + r] = l_part;
            row_group_barrier(warp & 3);
            if (ok) {
                float l = 0.f;
#pragma unroll
                for (int w4 = 0; w4 < kBwdWarpgroups; ++w4) l += sSum[w4 * BQ + r];
                const float inv = 1.f / l;
                uint32_t ro[ECW];
                __syncwarp();
                tmem_ld_cols<ECW>(tO + lane_off + wg * ECW, ro);
                tmem_ld_wait();
                if (g + 1 < G) store_q(wq);
                if (row_ok) {
                    bf16* o = p.out + ((static_cast<long long>(b) * p.T + row) * p.Hq + h) * HS + wg * ECW;
#pragma unroll
                    for (int c = 0; c < ECW; c += 8) {
                        uint4 v;
                        __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                        for (int jj = 0; jj < 4; ++jj) {
                            vb[jj] = __floats2bfloat162_rn(__uint_as_float(ro[c + 2 * jj]) * inv, __uint_as_float(ro[c + 2 * jj + 1]) * inv);
                            const float2 f = __bfloat1622float2(vb[jj]);
                            omax = fmaxf(omax, fmaxf(fabsf(f.x), fabsf(f.y)));
                        }
                        *reinterpret_cast<uint4*>(o + c) = v;
                    }
                    if (wg == 0) p.lse[(static_cast<long long>(b) * p.Hq + h) * p.T + row] = m_ref * p.scale + logf(l);
                }
            }
            row_group_barrier(warp & 3);                                  // sSum is reused by the next head
        }
        if (!ok && r == 0) atomicOr(p.status, kErrOther);
        if (p.absmax) {
            omax = warp_reduce_max(omax);
            if ((tid & 31) == 0 && omax > 0.f) atomic_max_float(p.absmax, omax);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (issuer) tmem_dealloc(tmem, TMEM_COLS);
}

// Tag makes the static flag unique per kernel instantiation (several kernels share one signature).
template <int Tag, typename K>
int set_smem(K kernel, int bytes) {
    static bool done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return 2000 + static_cast<int>(e);
        done[dev & 63] = true;
    }
    return 0;
}

template <int HS>
int fwd_impl(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, float* absmax, unsigned int* status, cudaStream_t s) {
    const int H = Hq + 2 * Hkv;
    CUtensorMap tkv;
    int rc = encode_btw(&tkv, qkv, B, T, static_cast<long long>(H) * HS, 64);
    if (rc) return rc;
    constexpr int smem = 8 * 64 * HS * 2 + 3 * kBwdWarpgroups * 128 * 4 + 256;
    rc = set_smem<HS>(attn_fwd_kernel<HS>, smem);
    if (rc) return rc;
    AttnParams p{};
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.scale = 1.f / sqrtf(static_cast<float>(HS));
    p.out = static_cast<bf16*>(out); p.lse = lse; p.status = status; p.qkv = static_cast<const bf16*>(qkv); p.absmax = absmax;
    dim3 grid(((T + 127) / 128) * Hkv * B, 1, 1);
    attn_fwd_kernel<HS><<<grid, kBwdThreads, smem, s>>>(tkv, p);
    return LLMQ_LAUNCH_CHECK();
}

template <int HS>
int bwd_impl(void* dqkv, float* delta, const void* d_out, const void* out, const float* lse, const void* qkv, int B, int T,
             int Hq, int Hkv, unsigned int* status, cudaStream_t s) {
    const int H = Hq + 2 * Hkv;
    {
        long long rows = static_cast<long long>(B) * T * Hq;
        long long blocks = (rows * (HS / 8) + 255) / 256;
        attn_delta_kernel<HS><<<static_cast<unsigned int>(blocks), 256, 0, s>>>(delta, static_cast<const bf16*>(out), static_cast<const bf16*>(d_out), B, T, Hq);
        int rc = LLMQ_LAUNCH_CHECK();
        if (rc) return rc;
    }
    CUtensorMap t128, t64, tdo128, tdo64;
    int rc = encode_btw(&t128, qkv, B, T, static_cast<long long>(H) * HS, 128);
    if (!rc) rc = encode_btw(&t64, qkv, B, T, static_cast<long long>(H) * HS, 64);
    if (!rc) rc = encode_btw(&tdo128, d_out, B, T, static_cast<long long>(Hq) * HS, 128);
    if (!rc) rc = encode_btw(&tdo64, d_out, B, T, static_cast<long long>(Hq) * HS, 64);
    if (rc) return rc;
    AttnParams p{};
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.scale = 1.f / sqrtf(static_cast<float>(HS));
    p.lse = const_cast<float*>(lse); p.delta = delta; p.dqkv = static_cast<bf16*>(dqkv); p.status = status;
    p.qkv = static_cast<const bf16*>(qkv); p.d_out = static_cast<const bf16*>(d_out);
    {
        constexpr int smem = 2 * 128 * HS * 2 + 8 * 64 * HS * 2 + 2 * 128 * 64 * 2 + 4 * 64 * 4 + 256;
        rc = set_smem<1000 + HS>(attn_bwd_dkdv_kernel<HS>, smem);
        if (rc) return rc;
        dim3 grid(((T + 127) / 128) * Hkv * B, 1, 1);
        attn_bwd_dkdv_kernel<HS><<<grid, kBwdThreads, smem, s>>>(t128, t64, tdo64, p);
        rc = LLMQ_LAUNCH_CHECK();
        if (rc) return rc;
    }
    {
        constexpr int smem = 8 * 64 * HS * 2 + 128 * 64 * 2 + 256;
        rc = set_smem<2000 + HS>(attn_bwd_dq_kernel<HS>, smem);
        if (rc) return rc;
        dim3 grid(((T + 127) / 128) * Hkv * B, 1, 1);
        attn_bwd_dq_kernel<HS><<<grid, kBwdThreads, smem, s>>>(t64, p);
        rc = LLMQ_LAUNCH_CHECK();
    }
    return rc;
}

}  // namespace

int llmq_attention_forward_pingpong(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, float* absmax,
                                    unsigned int* status, cudaStream_t s);

// qkv (B,T,Hq+2Hkv,HS) bf16 -> out (B,T,Hq,HS) bf16, lse (B,Hq,T) fp32.  HS in {64, 128}.
// absmax (optional): atomic maximum of |out|, for the fp8 quantisation of the output.
extern "C" int llmq_attention_forward(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, int HS,
                                      float* absmax, unsigned int* status, cudaStream_t s) {
    if (B <= 0 || T <= 0) return 0;
    if (Hq % Hkv) return -1;
    if (HS == 64) return fwd_impl<64>(out, lse, qkv, B, T, Hq, Hkv, absmax, status, s);
    if (HS == 128) {
        // two query tiles per CTA, processed alternately (attention_fwd_pingpong.cu); LLMQ_ATTN_FWD_SINGLE=1 keeps the
        // one-tile kernel of this file for comparisons
        static const bool single = [] { const char* e = getenv("LLMQ_ATTN_FWD_SINGLE"); return e && e[0] == '1'; }();
        if (!single) return llmq_attention_forward_pingpong(out, lse, qkv, B, T, Hq, Hkv, absmax, status, s);
        return fwd_impl<128>(out, lse, qkv, B, T, Hq, Hkv, absmax, status, s);
    }
    return -2;
}

// dqkv (B,T,Hq+2Hkv,HS) is fully overwritten.  delta is scratch of B*Hq*T floats.
extern "C" int llmq_attention_backward(void* dqkv, float* delta, const void* d_out, const void* out, const float* lse,
                                       const void* qkv, int B, int T, int Hq, int Hkv, int HS, unsigned int* status,
                                       cudaStream_t s) {
    if (B <= 0 || T <= 0) return 0;
    if (Hq % Hkv) return -1;
    if (HS == 64) return bwd_impl<64>(dqkv, delta, d_out, out, lse, qkv, B, T, Hq, Hkv, status, s);
    if (HS == 128) return bwd_impl<128>(dqkv, delta, d_out, out, lse, qkv, B, T, Hq, Hkv, status, s);
    return -2;
}
