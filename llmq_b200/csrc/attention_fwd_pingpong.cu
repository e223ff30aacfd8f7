// Causal grouped-query flash attention forward for head size 128: two query tiles per CTA, processed alternately.
//
// A CTA owns 256 consecutive queries of one (batch, query head) as two 128-row tiles A and B.  Each tile has its own
// softmax warpgroup (thread r owns row r = TMEM lane r and sees the whole 128-key score row, so the row maximum and the
// row sum need no exchange between threads), its own MMA-issuing thread and its own tensor-memory columns:
//
//     columns   0..127  S_A   (fp32 scores of the current key tile; the bf16 probabilities P_A overwrite columns 0..63)
//     columns 128..255  S_B
//     columns 256..383  O_A   (fp32 output accumulator)
//     columns 384..511  O_B
//
// Per 128-key tile j and query tile X the chain is  S_X = Q_X K_j^T  ->  softmax warpgroup X: max, exp2, bf16, P_X into
// tensor memory (handed over in two halves of 64 keys)  ->  O_X += P_X V_j (P is the A operand straight from tensor memory).  The two chains are independent,
// so while one tile's warpgroup computes exponentials the tensor core runs the other tile's MMAs; the single-tile
// kernel (attention_tcgen05.cu, still used for head size 64) left the tensor pipe idle during that time.
// K and V tiles stream through two shared-memory stages each (TMA, 128-byte swizzle); Q_A and Q_B stay in shared memory
// for the whole walk.  O is rescaled only when a row maximum moved by more than 2^8 since the last rescale (the stale
// maximum keeps P <= 256, which is exact after the final normalisation), and then by the row's own thread.
// Every wait is bounded: a wait that runs out sets the CTA's abort flag and the status word and all roles leave.
//
// Takes the place of the cuDNN SDPA forward graph of the reference (src/kernels/cudnn_att.cpp:46-160).
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"

using namespace sm100;

namespace {

constexpr int HS = 128;
constexpr int BQ = 128;                      // rows per query tile
constexpr int BKV = 128;                     // keys per tile
constexpr int TILE_BYTES = 128 * HS * 2;     // 32 KiB: Q, K and V tiles alike (two 64-column chunks of 128 rows x 128 bytes)
constexpr int CHUNK_BYTES = 128 * 128;
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 352;             // 4 + 4 softmax warps, TMA producer, MMA issuer A, MMA issuer B
constexpr uint32_t TMEM_COLS = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;     // in log2 units

struct FwdParams {
    int B, T, Hq, Hkv;
    float scale;
    int turns;                   // 1: the two softmax warpgroups take turns with their exponentials
    __nv_bfloat16* out;          // (B, T, Hq, HS)
    float* lse;                  // (B, Hq, T), natural log
    float* absmax;               // optional
    unsigned int* status;
};

__device__ __forceinline__ float ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void warp_arrive(uint32_t bar) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
}

#define DLO(base, lbo, off) (desc_lo((base), (lbo)) + static_cast<uint32_t>((off) >> 4))

// One work item = 256 consecutive queries of one (batch, query head).  Items are numbered with the longest key walks first
// (query block descending); a CTA walks the items  c, 2G-1-c, 2G+c, 4G-1-c, ...  (G = grid size): in every round of G items the
// order of the CTAs flips, which evens out the total walk length per CTA.
struct Item {
    int h, b, kvh, q0, nA, nB, n_max;
};
__device__ __forceinline__ int item_of(int it, int cta, int grid) { return it * grid + ((it & 1) ? grid - 1 - cta : cta); }
__device__ __forceinline__ Item decode_item(int item, const FwdParams& p, int nqb, int nt) {
    Item w;
    const int per_qb = p.Hq * p.B;
    const int qb = nqb - 1 - item / per_qb;
    const int rem = item % per_qb;
    w.h = rem % p.Hq;
    w.b = rem / p.Hq;
    w.kvh = w.h / (p.Hq / p.Hkv);
    w.q0 = qb * 2 * BQ;
    // key tiles each query tile walks over: everything up to and including its diagonal tile
    w.nA = min(2 * qb + 1, nt);
    w.nB = (w.q0 + BQ < p.T) ? min(2 * qb + 2, nt) : 0;
    w.n_max = max(w.nA, w.nB);
    return w;
}

// Persistent: one CTA per SM walks its items with every pipeline running across the item boundary.  The producer loads the
// next item's Q tiles as soon as the last score MMAs of the current item have read them and keeps the K / V stages rolling;
// an issuer starts the next item's first score tile while the softmax warpgroup still normalises and stores the current
// item's rows (it only has to wait for that before the first P V product overwrites O); tile A moves on to the next item
// while tile B walks its extra key tile.  All barrier phases are counted over the whole kernel.
__global__ void __launch_bounds__(NUM_THREADS, 1)
attn_fwd_pingpong_kernel(const __grid_constant__ CUtensorMap tmap_qkv,     // qkv as (B, T, W), box 128 rows x 64 columns
                         const FwdParams p) {
    extern __shared__ __align__(1024) uint8_t smem[];
    uint8_t* sQ = smem;                                   // [2 tiles][TILE_BYTES]
    uint8_t* sK = sQ + 2 * TILE_BYTES;                    // [KV_STAGES][TILE_BYTES]
    uint8_t* sV = sK + KV_STAGES * TILE_BYTES;            // [KV_STAGES][TILE_BYTES]
    uint64_t* bars = reinterpret_cast<uint64_t*>(sV + KV_STAGES * TILE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 24);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (smem_u32(smem) & 1023u) { if (tid == 0) atomicOr(p.status, kErrOther); return; }

    const int nqb = (p.T + 2 * BQ - 1) / (2 * BQ);
    const int nt = (p.T + BKV - 1) / BKV;                  // key tiles of the sequence
    const int total = nqb * p.Hq * p.B;
    const int cta = blockIdx.x, grid = gridDim.x;

    // barriers: 0 q_full | 1 q_empty | 2-3 k_full | 4-5 k_empty | 6-7 v_full | 8-9 v_empty | 10-11 s_full[X] | 12-13 p_ready[X]
    //           (first 64 keys) | 14-15 o_done[X] | 16-17 p_ready2[X] (second 64 keys) | 18-19 turn[X] (the exponentials of X
    //           may start) | 20-21 o_free[X] (the rows of X's previous item are stored, O may be overwritten).
    //           A waiter can be at most one completed phase behind on every barrier, so the parity test stays unambiguous.
    const uint32_t bar0 = smem_u32(bars);
    const uint32_t q_full = bar0, q_empty = bar0 + 8u;
    auto k_full = [&](int s) { return bar0 + 8u * (2 + s); };
    auto k_empty = [&](int s) { return bar0 + 8u * (4 + s); };
    auto v_full = [&](int s) { return bar0 + 8u * (6 + s); };
    auto v_empty = [&](int s) { return bar0 + 8u * (8 + s); };
    auto s_full = [&](int x) { return bar0 + 8u * (10 + x); };
    auto p_ready = [&](int x) { return bar0 + 8u * (12 + x); };
    auto o_done = [&](int x) { return bar0 + 8u * (14 + x); };
    auto p_ready2 = [&](int x) { return bar0 + 8u * (16 + x); };
    auto turn = [&](int x) { return bar0 + 8u * (18 + x); };
    auto o_free = [&](int x) { return bar0 + 8u * (20 + x); };
    if (tid == 0) {
        mbar_init(q_full, 1);
        mbar_init(q_empty, 2);                               // both issuers, every item
        for (int s = 0; s < KV_STAGES; ++s) {
            mbar_init(k_full(s), 1); mbar_init(v_full(s), 1);
            mbar_init(k_empty(s), 2); mbar_init(v_empty(s), 2);          // both issuers, every key tile (used or not)
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(s_full(x), 1); mbar_init(p_ready(x), 4); mbar_init(p_ready2(x), 4); mbar_init(o_done(x), 1);
            mbar_init(turn(x), 4); mbar_init(o_free(x), 4);
        }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 8) { tmem_alloc(smem_u32(tmem_slot), TMEM_COLS); tmem_relinquish(); }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *tmem_slot;

    if (warp == 8) {
        // ============================================================ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_qkv);
            uint32_t kv = 0;                                 // K / V stage fills so far
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int item = item_of(it, cta, grid);
                if (item >= total) break;
                const Item w = decode_item(item, p, nqb, nt);
                const int active = w.nB > 0 ? 2 : 1;
                const int qcol = w.h * HS, kcol = (p.Hq + w.kvh) * HS, vcol = (p.Hq + p.Hkv + w.kvh) * HS;
                if (it > 0 && !mbar_wait(q_empty, (it - 1) & 1, abort_flag)) { ok = false; break; }
                mbar_expect_tx(q_full, active * TILE_BYTES);
                for (int x = 0; x < active; ++x)
                    for (int c = 0; c < 2; ++c)
                        tma_load_3d(smem_u32(sQ) + x * TILE_BYTES + c * CHUNK_BYTES, &tmap_qkv, q_full, qcol + c * 64, w.q0 + x * BQ, w.b);
                for (int j = 0; j < w.n_max; ++j, ++kv) {
                    const int st = kv % KV_STAGES;
                    const uint32_t par = ((kv / KV_STAGES) - 1) & 1;
                    if (kv >= KV_STAGES && !mbar_wait(k_empty(st), par, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(k_full(st), TILE_BYTES);
                    for (int c = 0; c < 2; ++c)
                        tma_load_3d(smem_u32(sK) + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_qkv, k_full(st), kcol + c * 64, j * BKV, w.b);
                    if (kv >= KV_STAGES && !mbar_wait(v_empty(st), par, abort_flag)) { ok = false; break; }
                    mbar_expect_tx(v_full(st), TILE_BYTES);
                    for (int c = 0; c < 2; ++c)
                        tma_load_3d(smem_u32(sV) + st * TILE_BYTES + c * CHUNK_BYTES, &tmap_qkv, v_full(st), vcol + c * 64, j * BKV, w.b);
                }
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else if (warp >= 9) {
        // ============================================================ MMA issuer of query tile x
        const int x = warp - 9;
        if (lane == 0) {
            const uint32_t idesc_s = make_instr_desc(1, 1, false, false, BQ, BKV);       // S = Q K^T
            const uint32_t idesc_o = make_instr_desc(1, 1, false, true, BQ, HS);         // O += P V  (V read as MN-major B)
            const uint32_t hi = desc_hi(1024);
            const uint32_t tS = tmem + x * BKV, tO = tmem + 2 * BKV + x * HS;
            const uint32_t q_base = smem_u32(sQ) + x * TILE_BYTES;
            uint32_t kv = 0, tiles = 0, walks = 0;           // stage uses, key tiles of this query tile, items in which it had any
            bool ok = true;
            for (int it = 0; ok; ++it) {
                const int item = item_of(it, cta, grid);
                if (item >= total) break;
                const Item w = decode_item(item, p, nqb, nt);
                const int n = x == 0 ? w.nA : w.nB;
                if (!mbar_wait(q_full, it & 1, abort_flag)) { ok = false; break; }
                if (n == 0) mbar_arrive(q_empty);             // this tile does not exist in the item: its Q buffer was not loaded
                for (int j = 0; j < n && ok; ++j, ++kv, ++tiles) {
                    const int st = kv % KV_STAGES;
                    const uint32_t par = (kv / KV_STAGES) & 1;
                    if (!mbar_wait(k_full(st), par, abort_flag)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t k_base = smem_u32(sK) + st * TILE_BYTES;
#pragma unroll
                    for (int k = 0; k < HS / 16; ++k)
                        mma_issue<0, false>(tS, DLO(q_base, 16, (k / 4) * CHUNK_BYTES + (k % 4) * 32), hi,
                                            DLO(k_base, 16, (k / 4) * CHUNK_BYTES + (k % 4) * 32), hi, idesc_s, k > 0);
                    mma_commit(s_full(x));
                    mma_commit(k_empty(st));
                    if (j == n - 1) mma_commit(q_empty);      // the item's last read of this Q tile
                    if (!mbar_wait(v_full(st), par, abort_flag)) { ok = false; break; }
                    // the first product of an item overwrites O: the warpgroup must have stored the previous item's rows
                    if (j == 0 && walks > 0 && !mbar_wait(o_free(x), (walks - 1) & 1, abort_flag)) { ok = false; break; }
                    const uint32_t v_base = smem_u32(sV) + st * TILE_BYTES;
                    // P arrives in two halves of 64 keys (a barrier each): the first half's MMAs run while the warpgroup still
                    // exponentiates the second half
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        if (!mbar_wait(half == 0 ? p_ready(x) : p_ready2(x), tiles & 1, abort_flag)) { ok = false; break; }
                        tc_fence_after_sync();
#pragma unroll
                        for (int k = half * 4; k < half * 4 + 4; ++k)
                            mma_issue_f16_tmem_a(tO, tS + k * 8, DLO(v_base, CHUNK_BYTES, k * (16 * 128)), hi, idesc_o, (j > 0 || k > 0));
                    }
                    if (!ok) break;
                    mma_commit(o_done(x));
                    mma_commit(v_empty(st));
                }
                // the other tile may walk further: its stages still need this tile's arrival (wait for the stage's load first:
                // it is only issued once the stage's previous use was released by both tiles, so this arrival cannot be counted
                // towards that earlier phase)
                for (int j = n; j < w.n_max && ok; ++j, ++kv) {
                    const int st = kv % KV_STAGES;
                    const uint32_t par = (kv / KV_STAGES) & 1;
                    if (!mbar_wait(k_full(st), par, abort_flag)) { ok = false; break; }
                    mbar_arrive(k_empty(st));
                    if (!mbar_wait(v_full(st), par, abort_flag)) { ok = false; break; }
                    mbar_arrive(v_empty(st));
                }
                if (n > 0) ++walks;
            }
            if (!ok) { *abort_flag = 1u; atomicOr(p.status, kErrOther); }
        }
    } else {
        // ============================================================ softmax warpgroup of query tile x
        const int x = warp >> 2;
        const int r = tid & 127;
        const uint32_t lane_off = static_cast<uint32_t>((warp & 3) * 32) << 16;
        const uint32_t tS = tmem + x * BKV + lane_off, tO = tmem + 2 * BKV + x * HS + lane_off;
        const float sl2 = p.scale * kLog2e;
        float omax = 0.f;
        uint32_t tiles = 0, pairs = 0;                       // key tiles of this query tile so far; those walked together with the other tile
        bool ok = true;
        for (int it = 0; ok; ++it) {
            const int item = item_of(it, cta, grid);
            if (item >= total) break;
            const Item w = decode_item(item, p, nqb, nt);
            const int n = x == 0 ? w.nA : w.nB;
            const int q0 = w.q0, h = w.h, b = w.b;
            const int row = q0 + x * BQ + r;
            const bool row_ok = row < p.T;
            // The two warpgroups take turns with their exponentials for as long as both tiles have key tiles left: a warp alone on
            // its SM sub-partition keeps the MUFU unit busy (128 x 32 ex2 at 4 per clock), two at once only halve each other's
            // rate and then wait for the tensor pipe together.  A goes first; a warpgroup hands the turn over when its
            // exponentials are issued.  A's k-th wait (k >= 1) consumes B's arrival k-1, B's k-th wait A's arrival k.
            const int n_pair = (w.nB > 0 && p.turns) ? min(w.nA, w.nB) : 0;
            float m_ref = -INFINITY, l_sum = 0.f;
            for (int j = 0; j < n && ok; ++j, ++tiles) {
                if (!mbar_wait(s_full(x), tiles & 1, abort_flag)) { ok = false; break; }
                tc_fence_after_sync();
                const bool diag = (j + 1) * BKV > q0 + x * BQ;      // some keys of this tile lie beyond some rows of the tile
                const int lim = row - j * BKV;                      // columns above lim are masked (key > query)
                // ---- the whole score row at once: four loads in flight, one wait (the row stays in registers for both passes)
                uint32_t rs[128];
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) tmem_ld_32x32b_x32(tS + ch * 32, *reinterpret_cast<uint32_t(*)[32]>(rs + ch * 32));
                tmem_ld_wait();
                if (diag) {
#pragma unroll
                    for (int i = 0; i < 128; ++i) if (i > lim) rs[i] = __float_as_uint(-INFINITY);
                }
                float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
                for (int i = 0; i < 128; i += 4) {
                    mx0 = fmaxf(mx0, __uint_as_float(rs[i]));     mx1 = fmaxf(mx1, __uint_as_float(rs[i + 1]));
                    mx2 = fmaxf(mx2, __uint_as_float(rs[i + 2])); mx3 = fmaxf(mx3, __uint_as_float(rs[i + 3]));
                }
                const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
                // ---- lazy rescale of O (warp-collective tensor-memory accesses: the warp decides together)
                const bool need = j == 0 || (mx - m_ref) * sl2 > kRescaleThreshold;
                if (__any_sync(0xffffffffu, need)) {
                    const float m_new = need ? fmaxf(m_ref, mx) : m_ref;
                    if (j > 0) {
                        const float alpha = need ? ex2((m_ref - m_new) * sl2) : 1.f;
                        l_sum *= alpha;
                        if (!mbar_wait(o_done(x), (tiles - 1) & 1, abort_flag)) { ok = false; break; }      // PV of tile j-1 has landed
                        tc_fence_after_sync();
#pragma unroll 1
                        for (int ch = 0; ch < 4; ++ch) {
                            uint32_t ro[32];
                            tmem_ld_32x32b_x32(tO + ch * 32, ro);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) ro[i] = __float_as_uint(__uint_as_float(ro[i]) * alpha);
                            tmem_st_32x32b_x32(tO + ch * 32, ro);
                        }
                        tmem_st_wait();
                    }
                    m_ref = m_new;
                }
                // ---- this warpgroup's turn
                const bool paired = j < n_pair;
                if (paired && (x == 1 || pairs > 0)) {
                    if (!mbar_wait(turn(x), (x == 0 ? pairs - 1 : pairs) & 1, abort_flag)) { ok = false; break; }
                }
                // ---- probabilities -> bf16 -> tensor memory (over the first 64 score columns, which are in registers by now)
                const float moff = m_ref * sl2;
                float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t pw[16];
#pragma unroll
                    for (int i = 0; i < 32; i += 2) {
                        const float p0 = ex2(fmaf(__uint_as_float(rs[ch * 32 + i]), sl2, -moff));         // masked scores are -inf -> 0
                        const float p1 = ex2(fmaf(__uint_as_float(rs[ch * 32 + i + 1]), sl2, -moff));
                        sum0 += p0; sum1 += p1;
                        pw[i / 2] = pack2(p0, p1);
                    }
                    tmem_st_32x32b_x16(tS + ch * 16, pw);
                    if (ch == 1) {                                  // first 64 keys of P are complete: hand them over
                        tmem_st_wait();
                        tc_fence_before_sync();
                        warp_arrive(p_ready(x));
                    }
                }
                if (paired) { warp_arrive(turn(1 - x)); ++pairs; }      // every exponential of this tile is issued: the other tile's turn
                const float sum = sum0 + sum1;
                l_sum += sum;
                tmem_st_wait();
                tc_fence_before_sync();
                warp_arrive(p_ready2(x));
            }
            // ---- the walk is over: normalise and store this tile's rows, then release O to the next item
            if (ok && n > 0) ok = mbar_wait(o_done(x), (tiles - 1) & 1, abort_flag);
            tc_fence_after_sync();
            if (ok && n > 0) {
                const float inv = 1.f / l_sum;
                __nv_bfloat16* o = p.out + ((static_cast<long long>(b) * p.T + (row_ok ? row : 0)) * p.Hq + h) * HS;
#pragma unroll 1
                for (int ch = 0; ch < 4; ++ch) {
                    uint32_t ro[32];
                    tmem_ld_32x32b_x32(tO + ch * 32, ro);
                    tmem_ld_wait();
                    if (ch == 3) {                                  // the last of O is in registers
                        tc_fence_before_sync();
                        warp_arrive(o_free(x));
                    }
                    if (row_ok) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) {
                            uint4 v;
                            __nv_bfloat162* vb = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
                            for (int jj = 0; jj < 4; ++jj) {
                                vb[jj] = __floats2bfloat162_rn(__uint_as_float(ro[g * 8 + 2 * jj]) * inv, __uint_as_float(ro[g * 8 + 2 * jj + 1]) * inv);
                                const float2 f = __bfloat1622float2(vb[jj]);
                                omax = fmaxf(omax, fmaxf(fabsf(f.x), fabsf(f.y)));
                            }
                            *reinterpret_cast<uint4*>(o + ch * 32 + g * 8) = v;
                        }
                    }
                }
                if (row_ok) p.lse[(static_cast<long long>(b) * p.Hq + h) * p.T + row] = m_ref * p.scale + logf(l_sum);
            }
        }
        if (!ok) { *abort_flag = 1u; if (r == 0) atomicOr(p.status, kErrOther); }
        if (p.absmax) {
            omax = warp_reduce_max(omax);
            if (lane == 0 && omax > 0.f) atomic_max_float(p.absmax, omax);
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    if (warp == 8) tmem_dealloc(tmem, TMEM_COLS);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

}  // namespace

// Head size 128 only; same contract as llmq_attention_forward (which dispatches here).
int llmq_attention_forward_pingpong(void* out, float* lse, const void* qkv, int B, int T, int Hq, int Hkv, float* absmax,
                                    unsigned int* status, cudaStream_t s) {
    static EncodeTiledFn encode = nullptr;
    if (!encode) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess || !ptr) return -1;
        encode = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    const long long W = static_cast<long long>(Hq + 2 * Hkv) * HS;
    CUtensorMap tmap;
    cuuint64_t dims[3] = {static_cast<cuuint64_t>(W), static_cast<cuuint64_t>(T), static_cast<cuuint64_t>(B)};
    cuuint64_t strides[2] = {static_cast<cuuint64_t>(W) * 2, static_cast<cuuint64_t>(W) * 2 * T};
    cuuint32_t box[3] = {64, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = encode(&tmap, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(qkv), dims, strides, box, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return 1000 + static_cast<int>(r);
    constexpr int smem = (2 + 2 * KV_STAGES) * TILE_BYTES + 256;
    static bool attr_done[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_done[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(attn_fwd_pingpong_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e != cudaSuccess) return 2000 + static_cast<int>(e);
        attr_done[dev & 63] = true;
    }
    FwdParams p{};
    p.B = B; p.T = T; p.Hq = Hq; p.Hkv = Hkv; p.scale = 1.f / sqrtf(static_cast<float>(HS));
    p.out = static_cast<__nv_bfloat16*>(out); p.lse = lse; p.absmax = absmax; p.status = status;
    static const bool no_turns = [] { const char* e = getenv("LLMQ_ATTN_FWD_TURNS"); return e && e[0] == '0'; }();      // for A/B measurements
    p.turns = no_turns ? 0 : 1;
    const int nqb = (T + 2 * BQ - 1) / (2 * BQ);
    static int sms[64] = {};
    if (!sms[dev & 63]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return -2;
        sms[dev & 63] = n;
    }
    const long long total = static_cast<long long>(nqb) * Hq * B;
    const int grid = static_cast<int>(total < sms[dev & 63] ? total : sms[dev & 63]);       // one CTA per SM (shared memory, tensor memory)
    attn_fwd_pingpong_kernel<<<grid, NUM_THREADS, smem, s>>>(tmap, p);
    return LLMQ_LAUNCH_CHECK();
}
