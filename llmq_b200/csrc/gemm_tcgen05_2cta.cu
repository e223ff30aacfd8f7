// Two-CTA variant of the tcgen05 GEMM: a cluster of two CTAs on neighbouring SMs computes one 256x256 tile.
//
// Each CTA stages its own 128 rows of A and only half of the 256 rows of B per K step; tcgen05.mma with
// cta_group::2 reads both halves of B from the two shared memories, so per multiply-accumulate the pair moves
// a third less data out of L2 and shared memory than two independent 128x256 CTAs.  That is what lifts the
// kernel from the shared-memory / L2 limit of the one-CTA version towards the tensor-core limit.
//
// Roles per CTA (192 threads): warp 0 = TMA producer (both CTAs; completion bytes of both are credited to the
// leader's "full" barrier), warp 1 = MMA issuer (leader CTA only), warps 2-5 = epilogue of the CTA's own
// 128x256 accumulator.  Stage release and accumulator-ready signals go to both CTAs with two tcgen05.commit
// each; the peer's epilogue releases accumulators with a remote mbarrier arrive.  Every wait is bounded.
//
// Fused reduce-scatter (GemmParams::rs_*, used for the weight-gradient GEMMs of data-parallel ranks; takes the
// place of the reference's dW matmul followed by ncclReduceScatter and vector_add_sr, llama_gradients.cpp:50-77):
// the epilogue stores every output row straight into the landing buffer of the rank that owns the row, over
// NVLink, while the tensor core already works on the next tile; tiles are visited owner by owner starting with
// the right-hand neighbour, so a rank's own rows come last and the peers' contributions have landed by then.
// Each epilogue warp bumps the owner's arrival counter per tile (release, system scope).  After its last tile a
// CTA waits (bounded) for the local counter to show all sources, then the epilogue warps of all CTAs sum the
// `world` slots of this rank's rows, scale, add into the shard with stochastic rounding and collect the norm.
#include "ptx_sm100.cuh"
#include "api.h"
#include "common.cuh"
#include "gemm_common.cuh"
#include "peer_sync.cuh"

using namespace sm100;

namespace {

constexpr int BM = 128;              // rows per CTA (256 per pair)
constexpr int BN = 256;
constexpr int BN_HALF = 128;         // rows of B staged by each CTA
constexpr int ROW_BYTES = 128;
constexpr int STAGES = 6;
constexpr int A_STAGE_BYTES = BM * ROW_BYTES;        // 16 KiB
constexpr int B_STAGE_BYTES = BN_HALF * ROW_BYTES;   // 16 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 4;
// stages | 1 KiB for barriers and flags | two 1024-byte aligned staging buffers per epilogue warp | alignment slack
constexpr int EPI_STAGE_OFFSET = STAGES * STAGE_BYTES + 1024;
constexpr int SMEM_BYTES = EPI_STAGE_OFFSET + 2 * EPI_WARPS * EPI_STAGE_BYTES_PER_WARP + 1024;

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int rot, int& tm, int& tn) {
    constexpr int G = 8;             // 8 pair-rows (2048 rows of A) share each B tile while it is hot in L2
    int per_group = G * tiles_n;
    int group = t / per_group;
    int first_m = group * G;
    int gsz = min(tiles_m - first_m, G);
    int r = t - group * per_group;
    tm = first_m + (r % gsz) + rot;
    if (tm >= tiles_m) tm -= tiles_m;
    tn = r / gsz;
}

template <bool F8>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                         const __grid_constant__ CUtensorMap tmap_c, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
    // bars[0..S) full (used in the leader), [S..2S) empty, [2S..2S+2) tmem_full, [2S+2..2S+4) tmem_empty (leader)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4);
    volatile uint32_t* abort_flag = tmem_slot + 1;

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();           // 0 = leader
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * STAGES + 2 + a); };

    const int bk = ROW_BYTES / p.elem_bytes;
    const int k_iters = (p.K + bk - 1) / bk;
    const int tiles_m = (p.M + 2 * BM - 1) / (2 * BM);
    // SwiGLU forward mode: a column tile is 128 features, staged as 128 "up" rows + 128 "gate" rows of B
    const int tiles_n = p.ep_mode == 1 ? (p.ep_D + BN_HALF - 1) / BN_HALF : (p.N + BN - 1) / BN;
    const int num_tiles = tiles_m * tiles_n;
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    // fused reduce-scatter: start with the rows owned by the next rank, finish with our own
    const int rot = p.rs_world > 0 ? static_cast<int>((static_cast<long long>((p.rs_rank + 1) % p.rs_world) * p.rs_shard_rows) / (2 * BM)) : 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), 256); }
        *abort_flag = 0;
        mbar_init_fence();
    }
    if (warp == 1) {                                   // same warp index in both CTAs, as the pair allocation wants
        tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
        tmem_relinquish_pair();
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_arrive();                                  // barrier inits of both CTAs are visible cluster-wide
    cluster_wait();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer (both CTAs)
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            int stage = 0; uint32_t phase = 0;
            const int mn_chunk = ROW_BYTES / p.elem_bytes;
            bool ok = true;
            // Fused all-gather: B rows pushed by peer GPUs are consumed as soon as their source's flag shows the
            // current generation.  `seen` caches the sources already confirmed.
            uint32_t seen = 0;
            auto ensure_src = [&](int src) {
                if (!(seen >> src & 1u)) {
                    if (!peer::wait_flag(p.ready_flags + src, p.ready_gen, p.ready_limit_ns)) { atomicOr(p.status, kErrPeerFlag); *abort_flag = 1u; ok = false; }
                    peer::fence_before_tma_reads();
                    seen |= 1u << src;
                }
            };
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                int tm, tn; tile_coords(t, tiles_m, tiles_n, rot, tm, tn);
                const int row0 = (tm * 2 + static_cast<int>(rank)) * BM;               // this CTA's rows of A / C
                const int brow0 = p.ep_mode == 1 ? tn * BN_HALF + static_cast<int>(rank) * p.ep_D
                                                 : tn * BN + static_cast<int>(rank) * BN_HALF;   // this CTA's rows of B
                if (p.ready_flags && !p.b_mn_major && brow0 < p.N) {
                    const int last = min(brow0 + BN_HALF, p.N) - 1;
                    for (int src = brow0 / p.ready_rows_per_src; src <= last / p.ready_rows_per_src && ok; ++src) ensure_src(src);
                }
                for (int k = 0; k < k_iters && ok; ++k) {
                    if (p.ready_flags && p.b_mn_major) {
                        const int last = min(k * bk + bk, p.K) - 1;
                        for (int src = (k * bk) / p.ready_rows_per_src; src <= last / p.ready_rows_per_src && ok; ++src) ensure_src(src);
                        if (!ok) break;
                    }
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrEmptyWait); ok = false; break; }
                    const uint32_t sa = smem_base + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_STAGE_BYTES;
                    const uint32_t fb = map_to_cta(full_bar(stage), 0);                 // the leader's barrier
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * STAGE_BYTES);     // bytes of both CTAs
                    if (!p.a_mn_major) {
                        tma_load_2d_pair(sa, &tmap_a, fb, k * bk, row0);
                    } else {
                        int nbox = BM * p.elem_bytes / ROW_BYTES;
                        for (int b = 0; b < nbox; ++b)
                            tma_load_2d_pair(sa + b * (A_STAGE_BYTES / nbox), &tmap_a, fb, row0 + b * mn_chunk, k * bk);
                    }
                    if (!p.b_mn_major) {
                        tma_load_2d_pair(sb, &tmap_b, fb, k * bk, brow0);
                    } else {
                        int nbox = BN_HALF * p.elem_bytes / ROW_BYTES;
                        for (int b = 0; b < nbox; ++b)
                            tma_load_2d_pair(sb + b * (B_STAGE_BYTES / nbox), &tmap_b, fb, brow0 + b * mn_chunk, k * bk);
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = make_instr_desc(p.a_fmt, p.b_fmt, p.a_mn_major, p.b_mn_major, 2 * BM, BN);
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
            for (int t = pair; t < num_tiles && ok; t += num_pairs) {
                if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag)) { atomicOr(p.status, kErrTmemEmpty); ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int k = 0; k < k_iters; ++k) {
                    if (!mbar_wait(full_bar(stage), phase, abort_flag)) { atomicOr(p.status, kErrFullWait); ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t alo = a_lo0 + stage * (STAGE_BYTES >> 4);
                    const uint32_t blo = b_lo0 + stage * (STAGE_BYTES >> 4);
                    mma_issue<F8, true>(d_tmem, alo, a_hi, blo, b_hi, idesc, k > 0 ? 1u : 0u);
                    mma_issue<F8, true>(d_tmem, alo + a_inc, a_hi, blo + b_inc, b_hi, idesc, 1u);
                    mma_issue<F8, true>(d_tmem, alo + 2 * a_inc, a_hi, blo + 2 * b_inc, b_hi, idesc, 1u);
                    mma_issue<F8, true>(d_tmem, alo + 3 * a_inc, a_hi, blo + 3 * b_inc, b_hi, idesc, 1u);
                    mma_commit_pair(empty_bar(stage));                       // stage free in this CTA ...
                    mma_commit_pair(map_to_cta(empty_bar(stage), 1));        // ... and in the peer
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                mma_commit_pair(tfull_bar(acc));
                mma_commit_pair(map_to_cta(tfull_bar(acc), 1));
                if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (4 warps, both CTAs)
        const int q = warp & 3;
        uint8_t* stage = smem + EPI_STAGE_OFFSET + q * 2 * EPI_STAGE_BYTES_PER_WARP;            // coalescing buffers of this warp
        int stage_sel = 0;
        if (p.c_tma && lane == 0) tma_prefetch_desc(&tmap_c);
        float alpha = p.alpha;
        if (p.scale_a) alpha *= *p.scale_a;
        if (p.scale_b) alpha *= *p.scale_b;
        float tmax = 0.f;
        int acc = 0; uint32_t acc_phase = 0;
        bool ok = true;
        for (int t = pair; t < num_tiles && ok; t += num_pairs) {
            int tm, tn; tile_coords(t, tiles_m, tiles_n, rot, tm, tn);
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) { if (lane == 0) atomicOr(p.status, kErrTmemFull); ok = false; break; }
            tc_fence_after_sync();
            __syncwarp();
            const int row = (tm * 2 + static_cast<int>(rank)) * BM + q * 32 + lane;
            __nv_bfloat16* dst_row = nullptr;
            int owner = 0;
            if (p.rs_world > 0) {
                owner = min(((tm * 2 + static_cast<int>(rank)) * BM + q * 32) / p.rs_shard_rows, p.rs_world - 1);   // same for the whole warp
                const long long slot_row = static_cast<long long>(p.rs_rank) * p.rs_shard_rows + (row - owner * p.rs_shard_rows);
                dst_row = static_cast<__nv_bfloat16*>(p.rs_landing[owner]) + slot_row * p.N;
            }
            const uint32_t t_row = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * BN;
            if (p.ep_mode == 1)      epilogue_rows_swiglu_fwd(p, t_row, row, tn * BN_HALF, alpha, tmax);
            else if (p.ep_mode == 2) epilogue_rows_swiglu_bwd(p, t_row, row, tn * BN, BN, alpha, tmax);
            else                     epilogue_rows(p, t_row, row, tn * BN, BN, alpha, tmax, dst_row, stage, &tmap_c, &stage_sel);
            tc_fence_before_sync();
            mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));            // 2 x 128 arrivals at the leader
            if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
            if (p.rs_world > 0 && (tm * 2 + static_cast<int>(rank)) * BM + q * 32 < p.M) {
                __syncwarp();                                               // the rows of all lanes are stored
                if (lane == 0) {
                    __threadfence_system();
                    asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p.rs_counter[owner]), "r"(1u) : "memory");
                }
            }
        }
        if (p.rs_world > 0 && p.rs_dst != nullptr) {
            // ---- tail (only when the caller asked for it; otherwise a separate kernel on the collectives stream finishes):
            // sum the slots of this rank's rows once every source delivered
            volatile uint32_t* s_ok = abort_flag + 1;
            float* s_red = reinterpret_cast<float*>(const_cast<uint32_t*>(abort_flag + 2));
            if (warp == 2 && lane == 0) {
                bool got = ok && peer::wait_flag(p.rs_counter[p.rs_rank], p.rs_target, p.rs_limit_ns);
                if (!got) atomicOr(p.status, kErrPeerFlag);
                *s_ok = got ? 1u : 0u;
            }
            asm volatile("bar.sync 1, 128;" ::: "memory");
            if (*s_ok) {
                const int tid = threadIdx.x - 64;                           // 0..127
                const long long n_shard = static_cast<long long>(p.rs_shard_rows) * p.N;
                const long long nvec = n_shard / 8;
                const __nv_bfloat16* mine = static_cast<const __nv_bfloat16*>(p.rs_landing[p.rs_rank]);
                __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.rs_dst);
                float ss = 0.f;
                for (long long i = blockIdx.x * 128LL + tid; i < nvec; i += static_cast<long long>(gridDim.x) * 128) {
                    float a8[8];
#pragma unroll
                    for (int k = 0; k < 8; ++k) a8[k] = 0.f;
                    for (int s = 0; s < p.rs_world; ++s) {
                        const int src = (p.rs_rank + s) % p.rs_world;
                        Vec16<bf16> v = Vec16<bf16>::load_stream(mine + src * n_shard + i * 8);
#pragma unroll
                        for (int k = 0; k < 8; ++k) a8[k] += __bfloat162float(v.v[k]);
                    }
                    Vec16<bf16> o;
                    if (p.rs_accumulate) {
                        Vec16<bf16> old = Vec16<bf16>::load(dst + i * 8);
#pragma unroll
                        for (int k = 0; k < 8; k += 2) {
                            const uint32_t r = rng_u32(static_cast<uint64_t>(i) * 4 + k / 2, p.rs_seed);
                            o.v[k] = sr_bf16(a8[k] * p.rs_scale + __bfloat162float(old.v[k]), r);
                            o.v[k + 1] = sr_bf16(a8[k + 1] * p.rs_scale + __bfloat162float(old.v[k + 1]), r >> 16);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(a8[k] * p.rs_scale);
                    }
                    if (p.rs_norm_partials) {
#pragma unroll
                        for (int k = 0; k < 8; ++k) { float f = __bfloat162float(o.v[k]); ss += f * f; }
                    }
                    o.store(dst + i * 8);
                }
                if (p.rs_norm_partials) {
                    ss = warp_reduce_sum(ss);
                    if (lane == 0) s_red[q] = ss;
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (tid == 0) p.rs_norm_partials[blockIdx.x % p.rs_num_partials] += s_red[0] + s_red[1] + s_red[2] + s_red[3];
                }
            }
        }
        if (p.absmax_out) {
            tmax = warp_reduce_max(tmax);
            if (lane == 0 && tmax > 0.f) atomic_max_float(p.absmax_out, tmax);
        }
        if (p.c_tma && lane == 0) tma_store_wait<0>();          // the staged blocks have left shared memory and are written
    }

    // Neither CTA may leave while the other can still signal its barriers or read its shared memory.
    tc_fence_before_sync();
    __syncthreads();
    __syncwarp();
    cluster_arrive();
    cluster_wait();
    tc_fence_after_sync();
    if (warp == 1) tmem_dealloc_pair(tmem_base, TMEM_COLS);
}

}  // namespace

// Same contract as llmq_gemm (which dispatches here for problems with at least one full 256-row tile).
int llmq_gemm_2cta_launch(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const GemmParams& p, int num_sms, cudaStream_t stream) {
    static bool attr_set[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (!attr_set[dev & 63]) {
        cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tcgen05_2cta_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return static_cast<int>(e);
        attr_set[dev & 63] = true;
    }
    const int tiles = ((p.M + 2 * BM - 1) / (2 * BM)) * (p.ep_mode == 1 ? (p.ep_D + BN_HALF - 1) / BN_HALF : (p.N + BN - 1) / BN);
    int pairs = num_sms / 2;
    if (tiles < pairs) pairs = tiles;
    if (p.elem_bytes == 1) gemm_tcgen05_2cta_kernel<true><<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, p);
    else                   gemm_tcgen05_2cta_kernel<false><<<2 * pairs, NUM_THREADS, SMEM_BYTES, stream>>>(ta, tb, tc, p);
    return static_cast<int>(cudaGetLastError());
}
