// Causal grouped-query flash attention, forward and backward, on tcgen05 tensor cores (sm_100a).
//
// Operates directly on the packed post-RoPE tensor qkv (B, T, Hq + 2*Hkv, HS) through strided TMA maps,
// writes out (B, T, Hq, HS) and the per-row log-sum-exp (B, Hq, T); the backward pass produces the
// packed gradient dqkv with the same layout.  It takes the place of the cuDNN SDPA graphs and the
// scalar fallback kernel of the reference (src/kernels/cudnn_att.cpp:46-263, src/kernels/attention.cu).
//
// Every CTA has 128 threads; thread i owns row i of the 128-row MMA tile (TMEM lane i), so softmax
// statistics never leave the thread.  Score tiles are produced in TMEM by tcgen05.mma, read back with
// tcgen05.ld, turned into bf16 probabilities in shared memory (128-byte swizzled, K-major) and fed to
// the second MMA.  The shared-memory tile of V (rows = key positions) doubles as an MN-major B operand,
// so no transposed copy of V, K, Q or dO is ever made.
//
// Backward is split into two deterministic kernels (no atomics):
//   * dK/dV: one CTA per (batch, kv head, 128 keys) walks over all query heads of the group and all
//     query blocks at or below the diagonal; dK and dV accumulate in TMEM across the whole walk.
//   * dQ   : one CTA per (batch, q head, 128 queries) walks over the key blocks; dQ accumulates in TMEM.
// A small pre-pass computes delta = rowsum(dO * O).
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"

using namespace sm100;

namespace {

constexpr float kLog2e = 1.4426950408889634f;

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

// Writes 32 consecutive bf16 values (columns c0 .. c0+31 of row `row`) into a [rows][64] K-major tile with
// the 128-byte swizzle: 16-byte unit u of a row lands at unit (u ^ (row & 7)).
__device__ __forceinline__ void store_row_chunk_swz(uint8_t* tile, int row, int c0, const float (&v)[32]) {
    uint8_t* rowp = tile + row * 128;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 o;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) ob[j] = __floats2bfloat162_rn(v[g * 8 + 2 * j], v[g * 8 + 2 * j + 1]);
        int u = (c0 >> 3) + g;
        *reinterpret_cast<uint4*>(rowp + ((u ^ (row & 7)) << 4)) = o;
    }
}

struct AttnParams {
    int B, T, Hq, Hkv;
    float scale;                 // 1/sqrt(HS)
    bf16* out;                   // forward: (B,T,Hq,HS)
    float* lse;                  // (B,Hq,T), natural log
    const float* delta;          // (B,Hq,T)
    bf16* dqkv;                  // backward: packed gradient
    unsigned int* status;
};

// ------------------------------------------------------------------------------------------------
// Forward.  O accumulates in TMEM across all key tiles (tcgen05.mma with accumulate); it is rescaled only when a
// row maximum moved by more than 2^8 since the last rescale (the stale maximum keeps P <= 256, exact in the
// final normalisation).  Score tiles are double buffered in TMEM and K / V in shared memory, so the tensor core
// computes S(j+1) while the threads run the softmax of tile j.
template <int HS>
__global__ void __launch_bounds__(128, 2)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv, const AttnParams p) {
    constexpr int BQ = 128, BKV = 64, NCH = HS / 64;
    constexpr int Q_BYTES = BQ * HS * 2, KV_BYTES = BKV * HS * 2, P_BYTES = BQ * BKV * 2;
    constexpr uint32_t TMEM_COLS = 256;                       // S0 | S1 | O
    constexpr float kRescaleThreshold = 8.f;                  // in log2 units
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sK = sQ + Q_BYTES;            // 2 buffers
    uint8_t* sV = sK + 2 * KV_BYTES;       // 2 buffers
    uint8_t* sP = sV + 2 * KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sP + P_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }   // swizzled tiles need 1 KiB alignment
    const int qb = gridDim.x - 1 - blockIdx.x;                // longest rows first
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.Hq / p.Hkv);
    const int q0 = qb * BQ;
    const int n_kv = min((p.T + BKV - 1) / BKV, (q0 + BQ) / BKV);
    const int qcol = h * HS, kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_bar = bar0, o_bar = bar0 + 8;
    auto k_bar = [&](int i) { return bar0 + 16 + 8 * i; };
    auto v_bar = [&](int i) { return bar0 + 32 + 8 * i; };
    auto s_bar = [&](int i) { return bar0 + 48 + 8 * i; };
    if (tid == 0) {
        for (int i = 0; i < 8; ++i) mbar_init(bar0 + 8 * i, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tO = tmem + 128;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

    auto load_k = [&](int j) {
        const int bi = j & 1;
        mbar_expect_tx(k_bar(bi), KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sK) + bi * KV_BYTES + c * (BKV * 128), &tmap_kv, k_bar(bi), kcol + c * 64, j * BKV, b);
    };
    auto load_v = [&](int j) {
        const int bi = j & 1;
        mbar_expect_tx(v_bar(bi), KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sV) + bi * KV_BYTES + c * (BKV * 128), &tmap_kv, v_bar(bi), vcol + c * 64, j * BKV, b);
    };
    const uint32_t idesc_s = make_instr_desc(1, 1, false, false, BQ, BKV);
    const uint32_t idesc_o = make_instr_desc(1, 1, false, true, BQ, HS);
    auto issue_s = [&](int j) {                               // S[j&1] = Q K(j)^T
        const int bi = j & 1;
#pragma unroll
        for (int k = 0; k < HS / 16; ++k) {
            mma_issue<false, false>(tmem + bi * 64, DLO(smem_u32(sQ), 16, (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi,
                                    DLO(smem_u32(sK), 16, bi * KV_BYTES + (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi, idesc_s, k > 0);
        }
        mma_commit(s_bar(bi));
    };

    bool ok = true;
    if (tid == 0) {
        tma_prefetch_desc(&tmap_q); tma_prefetch_desc(&tmap_kv);
        mbar_expect_tx(q_bar, Q_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sQ) + c * (BQ * 128), &tmap_q, q_bar, qcol + c * 64, q0, b);
        load_k(0); load_v(0);
        if (n_kv > 1) { load_k(1); load_v(1); }
        ok = mbar_wait(q_bar, 0, abort_flag) && mbar_wait(k_bar(0), 0, abort_flag);
        tc_fence_after_sync();
        if (ok) issue_s(0);
    }

    const float sl2 = p.scale * kLog2e;
    const int row = q0 + tid;
    float m_ref = -INFINITY, l = 0.f;

    for (int j = 0; j < n_kv && ok; ++j) {
        const int bi = j & 1;
        const uint32_t par = (j >> 1) & 1;
        if (!mbar_wait(s_bar(bi), par, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        if (tid == 0) {
            if (j + 1 < n_kv) {                               // next score tile runs on the tensor core during this softmax
                ok = mbar_wait(k_bar(bi ^ 1), ((j + 1) >> 1) & 1, abort_flag);
                tc_fence_after_sync();
                if (ok) issue_s(j + 1);
            }
            if (ok && j + 2 < n_kv) load_k(j + 2);            // K[bi] was released by S(j)
        }
        float s[64];
        __syncwarp();
        {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tmem + bi * 64 + lane_off, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) s[i] = __uint_as_float(r[i]);
            tmem_ld_32x32b_x32(tmem + bi * 64 + lane_off + 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) s[32 + i] = __uint_as_float(r[i]);
        }
        if ((j + 1) * BKV > q0) {                             // tile touches the diagonal
#pragma unroll
            for (int i = 0; i < 64; ++i) if (j * BKV + i > row) s[i] = -INFINITY;
        }
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 64; ++i) mx = fmaxf(mx, s[i]);
        // everything below needs PV(j-1) finished: it read P, and it wrote the O we may rescale
        if (j > 0) {
            if (!mbar_wait(o_bar, (j - 1) & 1, abort_flag)) { ok = false; break; }
            tc_fence_after_sync();
            if (tid == 0 && j + 1 < n_kv && j + 1 >= 2) load_v(j + 1);     // V[(j+1)&1] was released by PV(j-1)
        }
        const bool need = j == 0 ? true : (mx - m_ref) * sl2 > kRescaleThreshold;
        if (__any_sync(0xffffffffu, need)) {
            const float m_new = fmaxf(m_ref, mx);
            if (j > 0) {
                const float alpha = exp2f((m_ref - m_new) * sl2);
                l *= alpha;
#pragma unroll
                for (int c = 0; c < HS / 32; ++c) {
                    uint32_t r[32];
                    tmem_ld_32x32b_x32(tO + lane_off + c * 32, r);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
                    tmem_st_32x32b_x32(tO + lane_off + c * 32, r);
                }
                tmem_st_wait();
            }
            m_ref = m_new;
        }
        const float moff = m_ref * sl2;
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 64; ++i) { s[i] = exp2f(s[i] * sl2 - moff); sum += s[i]; }
        l += sum;
        {
            float t[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = s[i];
            store_row_chunk_swz(sP, tid, 0, t);
#pragma unroll
            for (int i = 0; i < 32; ++i) t[i] = s[32 + i];
            store_row_chunk_swz(sP, tid, 32, t);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            ok = mbar_wait(v_bar(bi), par, abort_flag);
            tc_fence_after_sync();
            if (ok) {
#pragma unroll
                for (int k = 0; k < BKV / 16; ++k) {
                    mma_issue<false, false>(tO, DLO(smem_u32(sP), 16, k * 32), kDescHi,
                                            DLO(smem_u32(sV), BKV * 128, bi * KV_BYTES + k * (16 * 128)), kDescHi, idesc_o, (j > 0 || k > 0));
                }
                mma_commit(o_bar);
            }
        }
    }
    if (ok && n_kv > 0) ok = mbar_wait(o_bar, (n_kv - 1) & 1, abort_flag);
    tc_fence_after_sync();
    if (!ok && tid == 0) atomicOr(p.status, kErrOther);

    if (ok) {
        const float inv = 1.f / l;
        bf16* o = p.out + ((static_cast<long long>(b) * p.T + (row < p.T ? row : 0)) * p.Hq + h) * HS;
        __syncwarp();
#pragma unroll
        for (int c = 0; c < HS / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tO + lane_off + c * 32, r);
            tmem_ld_wait();
            if (row < p.T) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 v;
                    __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        vb[jj] = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * jj]) * inv, __uint_as_float(r[g * 8 + 2 * jj + 1]) * inv);
                    *reinterpret_cast<uint4*>(o + c * 32 + g * 8) = v;
                }
            }
        }
        if (row < p.T) p.lse[(static_cast<long long>(b) * p.Hq + h) * p.T + row] = m_ref * p.scale + logf(l);
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------
// delta[b,h,t] = sum_d dO[b,t,h,d] * O[b,t,h,d]; one warp per row
template <int HS>
__global__ void __launch_bounds__(256)
attn_delta_kernel(float* __restrict__ delta, const bf16* __restrict__ o, const bf16* __restrict__ d_o, int B, int T, int Hq) {
    const long long w = (blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = static_cast<long long>(B) * T * Hq;
    if (w >= total) return;
    const int h = static_cast<int>(w % Hq);
    const long long bt = w / Hq;
    const int t = static_cast<int>(bt % T);
    const long long b = bt / T;
    float s = 0.f;
    for (int c = lane * 8; c < HS; c += 256) {
        Vec16<bf16> a = Vec16<bf16>::load(o + w * HS + c), g = Vec16<bf16>::load(d_o + w * HS + c);
#pragma unroll
        for (int k = 0; k < 8; ++k) s += __bfloat162float(a.v[k]) * __bfloat162float(g.v[k]);
    }
    s = warp_reduce_sum(s);
    if (lane == 0) delta[(b * Hq + h) * T + t] = s;
}

// ------------------------------------------------------------------------------------------------
// dK / dV
template <int HS>
__global__ void __launch_bounds__(128, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmap_kv128,   // qkv, box 128 rows (K and V tiles)
                     const __grid_constant__ CUtensorMap tmap_q64,     // qkv, box 64 rows (Q tiles)
                     const __grid_constant__ CUtensorMap tmap_do64,    // dO, box 64 rows
                     const AttnParams p) {
    constexpr int BKV = 128, BQ = 64, NCH = HS / 64;
    constexpr int KV_BYTES = BKV * HS * 2, Q_BYTES = BQ * HS * 2, PT_BYTES = BKV * BQ * 2;
    constexpr uint32_t TMEM_COLS = (2 * BQ + 2 * HS) <= 256 ? 256 : 512;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sK = smem;
    uint8_t* sV = sK + KV_BYTES;
    uint8_t* sQ = sV + KV_BYTES;            // 2 buffers
    uint8_t* sdO = sQ + 2 * Q_BYTES;        // 2 buffers
    uint8_t* sPT = sdO + 2 * Q_BYTES;
    uint8_t* sdST = sPT + PT_BYTES;
    float* sLse = reinterpret_cast<float*>(sdST + PT_BYTES);      // [64] pre-multiplied by log2(e)
    float* sDelta = sLse + BQ;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sDelta + BQ);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }
    const int kb = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int G = p.Hq / p.Hkv;
    const int kv0 = kb * BKV;
    const int nqb = (p.T + BQ - 1) / BQ;
    const int qb_first = kv0 / BQ;
    const int per_head = nqb - qb_first;
    const int n_it = per_head * G;
    const int kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t kv_bar = bar0, qdo_bar0 = bar0 + 8 /* +16 */, sp_bar = bar0 + 24, acc_bar = bar0 + 32;
    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(bar0 + 8 * i, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem, tdP = tmem + BQ, tdV = tmem + 2 * BQ, tdK = tmem + 2 * BQ + HS;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

    auto issue_qdo = [&](int it) {
        const int hq = kvh * G + it / per_head;
        const int qb = qb_first + it % per_head;
        const int buf = it & 1;
        const uint32_t bar = qdo_bar0 + 8 * buf;
        mbar_expect_tx(bar, 2 * Q_BYTES);
        for (int c = 0; c < NCH; ++c) {
            tma_load_3d(smem_u32(sQ) + buf * Q_BYTES + c * (BQ * 128), &tmap_q64, bar, hq * HS + c * 64, qb * BQ, b);
            tma_load_3d(smem_u32(sdO) + buf * Q_BYTES + c * (BQ * 128), &tmap_do64, bar, hq * HS + c * 64, qb * BQ, b);
        }
    };
    if (tid == 0 && n_it > 0) {
        tma_prefetch_desc(&tmap_kv128); tma_prefetch_desc(&tmap_q64); tma_prefetch_desc(&tmap_do64);
        mbar_expect_tx(kv_bar, 2 * KV_BYTES);
        for (int c = 0; c < NCH; ++c) {
            tma_load_3d(smem_u32(sK) + c * (BKV * 128), &tmap_kv128, kv_bar, kcol + c * 64, kv0, b);
            tma_load_3d(smem_u32(sV) + c * (BKV * 128), &tmap_kv128, kv_bar, vcol + c * 64, kv0, b);
        }
        issue_qdo(0);
    }

    const uint32_t idesc_st = make_instr_desc(1, 1, false, false, BKV, BQ);     // S^T = K Q^T, dP^T = V dO^T
    const uint32_t idesc_acc = make_instr_desc(1, 1, false, true, BKV, HS);      // dV += P^T dO, dK += dS^T Q
    const float sl2 = p.scale * kLog2e;
    const int kv_row = kv0 + tid;
    bool ok = true;

    for (int it = 0; it < n_it && ok; ++it) {
        const int hq = kvh * G + it / per_head;
        const int qb = qb_first + it % per_head;
        const int buf = it & 1;
        const uint32_t par = it & 1;
        if (tid == 0 && it + 1 < n_it) issue_qdo(it + 1);        // other buffer was released by acc_bar of it-1
        {
            const int q = qb * BQ + (tid & 63);
            const long long si = (static_cast<long long>(b) * p.Hq + hq) * p.T + q;
            if (tid < 64) sLse[tid] = q < p.T ? p.lse[si] * kLog2e : INFINITY;
            else sDelta[tid - 64] = q < p.T ? p.delta[si] : 0.f;
        }
        if (tid == 0) {
            if (it == 0) ok = mbar_wait(kv_bar, 0, abort_flag);
            ok = ok && mbar_wait(qdo_bar0 + 8 * buf, (it >> 1) & 1, abort_flag);
            tc_fence_after_sync();
            if (ok) {
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tS, DLO(smem_u32(sK), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sQ), 16, buf * Q_BYTES + (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi, idesc_st, k > 0);
                }
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tdP, DLO(smem_u32(sV), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sdO), 16, buf * Q_BYTES + (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi, idesc_st, k > 0);
                }
                mma_commit(sp_bar);
            }
        }
        __syncthreads();                                            // sLse / sDelta visible
        if (!mbar_wait(sp_bar, par, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        const bool diag = qb * BQ < kv0 + BKV;                      // some (kv, q) pairs have q < kv
        __syncwarp();
#pragma unroll
        for (int c = 0; c < BQ / 32; ++c) {
            uint32_t rs[32], rp[32];
            tmem_ld_32x32b_x32(tS + lane_off + c * 32, rs);
            tmem_ld_32x32b_x32(tdP + lane_off + c * 32, rp);
            tmem_ld_wait();
            float pt[32], ds[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                const int qi = c * 32 + i;
                float pv = exp2f(__uint_as_float(rs[i]) * sl2 - sLse[qi]);
                if (diag && (qb * BQ + qi < kv_row)) pv = 0.f;
                pt[i] = pv;
                ds[i] = pv * (__uint_as_float(rp[i]) - sDelta[qi]) * p.scale;
            }
            store_row_chunk_swz(sPT, tid, c * 32, pt);
            store_row_chunk_swz(sdST, tid, c * 32, ds);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int k = 0; k < BQ / 16; ++k) {
                mma_issue<false, false>(tdV, DLO(smem_u32(sPT), 16, k * 32), kDescHi,
                                        DLO(smem_u32(sdO), BQ * 128, buf * Q_BYTES + k * (16 * 128)), kDescHi, idesc_acc, (it > 0 || k > 0));
            }
#pragma unroll
            for (int k = 0; k < BQ / 16; ++k) {
                mma_issue<false, false>(tdK, DLO(smem_u32(sdST), 16, k * 32), kDescHi,
                                        DLO(smem_u32(sQ), BQ * 128, buf * Q_BYTES + k * (16 * 128)), kDescHi, idesc_acc, (it > 0 || k > 0));
            }
            mma_commit(acc_bar);
        }
        if (!mbar_wait(acc_bar, par, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
    }
    if (!ok && tid == 0) atomicOr(p.status, kErrOther);

    if (ok && n_it > 0) {
        // The TMEM loads are warp-collective: every lane executes them, only the stores are predicated.
        const bool row_ok = kv_row < p.T;
        const int H = p.Hq + 2 * p.Hkv;
        const long long rbase = (static_cast<long long>(b) * p.T + (row_ok ? kv_row : 0)) * H;
        bf16* dk = p.dqkv + (rbase + p.Hq + kvh) * HS;
        bf16* dv = p.dqkv + (rbase + p.Hq + p.Hkv + kvh) * HS;
        __syncwarp();
#pragma unroll
        for (int c = 0; c < HS / 32; ++c) {
            uint32_t rk[32], rv[32];
            tmem_ld_32x32b_x32(tdK + lane_off + c * 32, rk);
            tmem_ld_32x32b_x32(tdV + lane_off + c * 32, rv);
            tmem_ld_wait();
            if (row_ok) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 ok4, ov4;
                    __nv_bfloat162* kb2 = reinterpret_cast<__nv_bfloat162*>(&ok4);
                    __nv_bfloat162* vb2 = reinterpret_cast<__nv_bfloat162*>(&ov4);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) {
                        kb2[jj] = __floats2bfloat162_rn(__uint_as_float(rk[g * 8 + 2 * jj]), __uint_as_float(rk[g * 8 + 2 * jj + 1]));
                        vb2[jj] = __floats2bfloat162_rn(__uint_as_float(rv[g * 8 + 2 * jj]), __uint_as_float(rv[g * 8 + 2 * jj + 1]));
                    }
                    *reinterpret_cast<uint4*>(dk + c * 32 + g * 8) = ok4;
                    *reinterpret_cast<uint4*>(dv + c * 32 + g * 8) = ov4;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
}

// ------------------------------------------------------------------------------------------------
// dQ
template <int HS>
__global__ void __launch_bounds__(128, 2)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmap_q128,    // qkv, box 128 rows
                   const __grid_constant__ CUtensorMap tmap_kv64,    // qkv, box 64 rows
                   const __grid_constant__ CUtensorMap tmap_do128,   // dO, box 128 rows
                   const AttnParams p) {
    constexpr int BQ = 128, BKV = 64, NCH = HS / 64;
    constexpr int Q_BYTES = BQ * HS * 2, KV_BYTES = BKV * HS * 2, DS_BYTES = BQ * BKV * 2;
    constexpr uint32_t TMEM_COLS = (2 * BKV + HS) <= 256 ? 256 : 512;
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;
    uint8_t* sdO = sQ + Q_BYTES;
    uint8_t* sK = sdO + Q_BYTES;
    uint8_t* sV = sK + KV_BYTES;
    uint8_t* sdS = sV + KV_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(sdS + DS_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }
    const int qb = gridDim.x - 1 - blockIdx.x;
    const int h = blockIdx.y, b = blockIdx.z;
    const int kvh = h / (p.Hq / p.Hkv);
    const int q0 = qb * BQ;
    const int n_kv = min((p.T + BKV - 1) / BKV, (q0 + BQ) / BKV);
    const int kcol = (p.Hq + kvh) * HS, vcol = (p.Hq + p.Hkv + kvh) * HS;

    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_bar = bar0, k_bar = bar0 + 8, v_bar = bar0 + 16, sp_bar = bar0 + 24, dq_bar = bar0 + 32;
    if (tid == 0) {
        for (int i = 0; i < 5; ++i) mbar_init(bar0 + 8 * i, 1);
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 0) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;
    const uint32_t tS = tmem, tdP = tmem + BKV, tdQ = tmem + 2 * BKV;
    const uint32_t lane_off = static_cast<uint32_t>(warp * 32) << 16;

    if (tid == 0) {
        tma_prefetch_desc(&tmap_q128); tma_prefetch_desc(&tmap_kv64); tma_prefetch_desc(&tmap_do128);
        mbar_expect_tx(q_bar, 2 * Q_BYTES);
        for (int c = 0; c < NCH; ++c) {
            tma_load_3d(smem_u32(sQ) + c * (BQ * 128), &tmap_q128, q_bar, h * HS + c * 64, q0, b);
            tma_load_3d(smem_u32(sdO) + c * (BQ * 128), &tmap_do128, q_bar, h * HS + c * 64, q0, b);
        }
        mbar_expect_tx(k_bar, KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sK) + c * (BKV * 128), &tmap_kv64, k_bar, kcol + c * 64, 0, b);
        mbar_expect_tx(v_bar, KV_BYTES);
        for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sV) + c * (BKV * 128), &tmap_kv64, v_bar, vcol + c * 64, 0, b);
    }

    const uint32_t idesc_s = make_instr_desc(1, 1, false, false, BQ, BKV);
    const uint32_t idesc_dq = make_instr_desc(1, 1, false, true, BQ, HS);
    const float sl2 = p.scale * kLog2e;
    const int row = q0 + tid;
    const long long si = (static_cast<long long>(b) * p.Hq + h) * p.T + row;
    const float lse2 = row < p.T ? p.lse[si] * kLog2e : INFINITY;
    const float delta = row < p.T ? p.delta[si] : 0.f;
    bool ok = true;

    for (int j = 0; j < n_kv && ok; ++j) {
        const uint32_t par = j & 1;
        if (tid == 0) {
            if (j == 0) ok = mbar_wait(q_bar, 0, abort_flag);
            ok = ok && mbar_wait(k_bar, par, abort_flag) && mbar_wait(v_bar, par, abort_flag);
            tc_fence_after_sync();
            if (ok) {
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tS, DLO(smem_u32(sQ), 16, (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sK), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi, idesc_s, k > 0);
                }
#pragma unroll
                for (int k = 0; k < HS / 16; ++k) {
                    mma_issue<false, false>(tdP, DLO(smem_u32(sdO), 16, (k / 4) * (BQ * 128) + (k % 4) * 32), kDescHi,
                                            DLO(smem_u32(sV), 16, (k / 4) * (BKV * 128) + (k % 4) * 32), kDescHi, idesc_s, k > 0);
                }
                mma_commit(sp_bar);
            }
        }
        if (!mbar_wait(sp_bar, par, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        if (tid == 0 && j + 1 < n_kv) {                       // V tile is free again
            mbar_expect_tx(v_bar, KV_BYTES);
            for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sV) + c * (BKV * 128), &tmap_kv64, v_bar, vcol + c * 64, (j + 1) * BKV, b);
        }
        const bool diag = (j + 1) * BKV > q0;
        __syncwarp();
#pragma unroll
        for (int c = 0; c < BKV / 32; ++c) {
            uint32_t rs[32], rp[32];
            tmem_ld_32x32b_x32(tS + lane_off + c * 32, rs);
            tmem_ld_32x32b_x32(tdP + lane_off + c * 32, rp);
            tmem_ld_wait();
            float ds[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) {
                float pv = exp2f(__uint_as_float(rs[i]) * sl2 - lse2);
                if (diag && (j * BKV + c * 32 + i > row)) pv = 0.f;
                ds[i] = pv * (__uint_as_float(rp[i]) - delta) * p.scale;
            }
            store_row_chunk_swz(sdS, tid, c * 32, ds);
        }
        fence_proxy_async_smem();
        tc_fence_before_sync();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after_sync();
#pragma unroll
            for (int k = 0; k < BKV / 16; ++k) {
                mma_issue<false, false>(tdQ, DLO(smem_u32(sdS), 16, k * 32), kDescHi,
                                        DLO(smem_u32(sK), BKV * 128, k * (16 * 128)), kDescHi, idesc_dq, (j > 0 || k > 0));
            }
            mma_commit(dq_bar);
        }
        if (!mbar_wait(dq_bar, par, abort_flag)) { ok = false; break; }
        tc_fence_after_sync();
        if (tid == 0 && j + 1 < n_kv) {                       // K tile is free again
            mbar_expect_tx(k_bar, KV_BYTES);
            for (int c = 0; c < NCH; ++c) tma_load_3d(smem_u32(sK) + c * (BKV * 128), &tmap_kv64, k_bar, kcol + c * 64, (j + 1) * BKV, b);
        }
    }
    if (!ok && tid == 0) atomicOr(p.status, kErrOther);

    if (ok) {
        const int H = p.Hq + 2 * p.Hkv;
        bf16* dq = p.dqkv + ((static_cast<long long>(b) * p.T + row) * H + h) * HS;
        __syncwarp();
#pragma unroll
        for (int c = 0; c < HS / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32b_x32(tdQ + lane_off + c * 32, r);
            tmem_ld_wait();
            if (row < p.T) {
#pragma unroll
                for (int g = 0; g < 4; ++g) {
                    uint4 o4;
                    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj)
                        ob[jj] = __floats2bfloat162_rn(__uint_as_float(r[g * 8 + 2 * jj]), __uint_as_float(r[g * 8 + 2 * jj + 1]));
                    *reinterpret_cast<uint4*>(dq + c * 32 + g * 8) = o4;
                }
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 0) tmem_dealloc(tmem, TMEM_COLS);
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
int fwd_impl(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, unsigned int* status, cudaStream_t s) {
    const int H = Hq + 2 * Hkv;
    CUtensorMap tq, tkv;
    int rc = encode_btw(&tq, qkv, B, T, static_cast<long long>(H) * HS, 128);
    if (rc) return rc;
    rc = encode_btw(&tkv, qkv, B, T, static_cast<long long>(H) * HS, 64);
    if (rc) return rc;
    constexpr int smem = 128 * HS * 2 + 4 * 64 * HS * 2 + 128 * 64 * 2 + 128;
    rc = set_smem<HS>(attn_fwd_kernel<HS>, smem);
    if (rc) return rc;
    AttnParams p{};
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.scale = 1.f / sqrtf(static_cast<float>(HS));
    p.out = static_cast<bf16*>(out); p.lse = lse; p.status = status;
    dim3 grid((T + 127) / 128, Hq, B);
    attn_fwd_kernel<HS><<<grid, 128, smem, s>>>(tq, tkv, p);
    return LLMQ_LAUNCH_CHECK();
}

template <int HS>
int bwd_impl(void* dqkv, float* delta, const void* d_out, const void* out, const float* lse, const void* qkv, int B, int T,
             int Hq, int Hkv, unsigned int* status, cudaStream_t s) {
    const int H = Hq + 2 * Hkv;
    {
        long long rows = static_cast<long long>(B) * T * Hq;
        long long blocks = (rows * 32 + 255) / 256;
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
    {
        constexpr int smem = 2 * 128 * HS * 2 + 4 * 64 * HS * 2 + 2 * 128 * 64 * 2 + 2 * 64 * 4 + 128;
        rc = set_smem<1000 + HS>(attn_bwd_dkdv_kernel<HS>, smem);
        if (rc) return rc;
        dim3 grid((T + 127) / 128, Hkv, B);
        attn_bwd_dkdv_kernel<HS><<<grid, 128, smem, s>>>(t128, t64, tdo64, p);
        rc = LLMQ_LAUNCH_CHECK();
        if (rc) return rc;
    }
    {
        constexpr int smem = 2 * 128 * HS * 2 + 2 * 64 * HS * 2 + 128 * 64 * 2 + 128;
        rc = set_smem<2000 + HS>(attn_bwd_dq_kernel<HS>, smem);
        if (rc) return rc;
        dim3 grid((T + 127) / 128, Hq, B);
        attn_bwd_dq_kernel<HS><<<grid, 128, smem, s>>>(t128, t64, tdo128, p);
        rc = LLMQ_LAUNCH_CHECK();
    }
    return rc;
}

}  // namespace

// qkv (B,T,Hq+2Hkv,HS) bf16 -> out (B,T,Hq,HS) bf16, lse (B,Hq,T) fp32.  HS in {64, 128}.
extern "C" int llmq_attention_forward(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, int HS,
                                      unsigned int* status, cudaStream_t s) {
    if (B <= 0 || T <= 0) return 0;
    if (Hq % Hkv) return -1;
    if (HS == 64) return fwd_impl<64>(out, lse, qkv, B, T, Hq, Hkv, status, s);
    if (HS == 128) return fwd_impl<128>(out, lse, qkv, B, T, Hq, Hkv, status, s);
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
