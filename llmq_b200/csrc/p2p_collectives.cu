// Collectives issued from inside kernels over NVLink 5 / NVSwitch peer memory.
//
// Every rank owns a "symmetric heap": the same allocation on every GPU, mapped into every peer, so a tensor
// is named by (rank, byte offset).  Kernels get the table of the peers' base pointers and move the data
// themselves with ordinary loads / stores on peer addresses (or `multimem` loads that reduce inside the
// switch); there is no library collective on these paths.  These kernels take the place of the reference's
// NCCL calls on a side stream (src/utilities/comm.cpp:201-255) and of the separate passes around them:
//
//   quant_allgather : master shard -> (abs-max scaled e4m3 | plain copy) -> stored into the gather buffer of
//                     EVERY rank in one pass (convert_dtype_for_gather + ncclAllGather, llama_weights.cpp:472-504)
//   reduce_scatter  : this rank's rows of the gradient are read from every peer, summed in fp32, scaled, added
//                     into the persistent shard with stochastic rounding, and their squared norm is accumulated
//                     (ncclReduceScatter + vector_add_sr + global_norm_squared, llama_gradients.cpp:50-77)
//   signal / wait   : release-store of a generation number into every peer's flag word / bounded acquire-spin
//   allreduce_small : sum or max of a few floats (loss groups, norm^2, abs-max slots)
//
// Flags carry monotonically increasing generation numbers, never reset.  Waits give up after a time limit,
// set an error bit in the status word and let the kernel finish, so a lost peer cannot hang the GPU.
#include "api.h"
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "peer_sync.cuh"

namespace {

constexpr int MAX_PEERS = 8;
struct PeerTable { void* base[MAX_PEERS]; };

using peer::st_release_sys;
using peer::ld_acquire_sys;
using peer::wait_flag;

// ------------------------------------------------------------------------------------------------
// quantise (or copy) the local shard and store it into every rank's gather buffer
template <typename Q>
__global__ void __launch_bounds__(512)
quant_allgather_kernel(PeerTable peers, long long dst_offset_bytes, const bf16* __restrict__ src, long long n, int rank, int world,
                       const float* __restrict__ absmax, float* __restrict__ scale_out) {
    float mul = 1.f;
    if constexpr (sizeof(Q) == 1) {
        const float am = fmaxf(*absmax, 1e-10f);
        mul = 448.f / am;
        if (blockIdx.x == 0 && threadIdx.x == 0 && scale_out) *scale_out = am / 448.f;
    }
    const long long shard_bytes = n * static_cast<long long>(sizeof(Q));
    const long long nvec = n / 8;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        Vec16<bf16> v = Vec16<bf16>::load_stream(src + i * 8);
        if constexpr (sizeof(Q) == 1) {
            alignas(8) Q q[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) q[k] = Q(__bfloat162float(v.v[k]) * mul);
            const uint2 packed = *reinterpret_cast<uint2*>(q);
            for (int p = 0; p < world; ++p) {
                const int dst = (rank + p) % world;                 // start with the own copy, spread the rest
                char* base = static_cast<char*>(peers.base[dst]) + dst_offset_bytes + rank * shard_bytes;
                *reinterpret_cast<uint2*>(base + i * 8) = packed;
            }
        } else {
            const uint4 packed = *reinterpret_cast<uint4*>(v.v);
            for (int p = 0; p < world; ++p) {
                const int dst = (rank + p) % world;
                char* base = static_cast<char*>(peers.base[dst]) + dst_offset_bytes + rank * shard_bytes;
                *reinterpret_cast<uint4*>(base + i * 16) = packed;
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// flags[src_rank] of every peer <- gen   (one thread per peer; stores of earlier kernels are ordered before it)
__global__ void signal_kernel(PeerTable peers, long long flag_offset_bytes, int rank, int world, unsigned int gen) {
    __threadfence_system();
    if (threadIdx.x < world) {
        unsigned int* f = reinterpret_cast<unsigned int*>(static_cast<char*>(peers.base[threadIdx.x]) + flag_offset_bytes) + rank;
        st_release_sys(f, gen);
    }
}

__global__ void wait_kernel(const unsigned int* flags, int world, unsigned int gen, unsigned int* status, unsigned long long limit_ns) {
    if (threadIdx.x < world) {
        if (!wait_flag(flags + threadIdx.x, gen, limit_ns)) atomicOr(status, sm100::kErrPeerFlag);
    }
    __threadfence_system();
}

// ------------------------------------------------------------------------------------------------
// reduce-scatter of this rank's slice.  use_multimem: one load on the multicast address returns the sum over
// all ranks, reduced by the switch in fp32; otherwise `world` peer loads are summed here.
__device__ __forceinline__ void multimem_ld_reduce_bf16x8(const void* mc_addr, float (&f)[8]) {
    uint32_t r0, r1, r2, r3;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "l"(mc_addr) : "memory");
    const uint32_t r[4] = {r0, r1, r2, r3};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&r[k]));
        f[2 * k] = t.x; f[2 * k + 1] = t.y;
    }
}

__global__ void __launch_bounds__(512)
reduce_scatter_kernel(PeerTable peers, const void* mc_base, long long src_offset_bytes, long long n_shard, int rank, int world,
                      bf16* dst, int accumulate, float scale, float* __restrict__ norm_partials, unsigned int seed) {
    __shared__ float scratch[32];
    const long long nvec = n_shard / 8;
    const long long my_off = src_offset_bytes + rank * n_shard * 2;
    float ss = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc[8];
        if (mc_base) {
            multimem_ld_reduce_bf16x8(static_cast<const char*>(mc_base) + my_off + i * 16, acc);
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
            for (int p = 0; p < world; ++p) {
                const int srcr = (rank + p) % world;
                const bf16* s = reinterpret_cast<const bf16*>(static_cast<const char*>(peers.base[srcr]) + my_off) + i * 8;
                Vec16<bf16> v = Vec16<bf16>::load_stream(s);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(v.v[k]);
            }
        }
        Vec16<bf16> o;
        if (accumulate) {
            Vec16<bf16> old = Vec16<bf16>::load(dst + i * 8);
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                const uint32_t r = rng_u32(static_cast<uint64_t>(i) * 4 + k / 2, seed);
                o.v[k] = sr_bf16(acc[k] * scale + __bfloat162float(old.v[k]), r);
                o.v[k + 1] = sr_bf16(acc[k + 1] * scale + __bfloat162float(old.v[k + 1]), r >> 16);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(acc[k] * scale);
        }
        if (norm_partials) {
#pragma unroll
            for (int k = 0; k < 8; ++k) { float f = __bfloat162float(o.v[k]); ss += f * f; }
        }
        o.store(dst + i * 8);
    }
    if (norm_partials) {
        ss = block_reduce_sum(ss, scratch);
        if (threadIdx.x == 0) norm_partials[blockIdx.x] += ss;
    }
}

// ------------------------------------------------------------------------------------------------
// Owner side of the reduce-scatter that weight-gradient GEMMs start in their epilogue (gemm_tcgen05_2cta.cu pushes every
// output row into the owning rank's landing buffer and bumps its arrival counter per tile).  This kernel runs on the
// collectives stream: it waits (bounded) until the local counter shows all sources, then sums the `world` LOCAL slots,
// applies 1/world, adds into the gradient shard with stochastic rounding and collects the squared norm - the work of the
// reference's ncclReduceScatter + vector_add_sr + global-norm pass (llama_gradients.cpp:50-77) without holding the SMs of
// the GEMM while the peers are still sending.
__global__ void __launch_bounds__(512)
rs_finish_kernel(const bf16* __restrict__ landing, const unsigned int* counter, unsigned int target, long long n_shard, int rank, int world,
                 bf16* dst, int accumulate, float scale, float* __restrict__ norm_partials, unsigned int seed, unsigned int* status,
                 unsigned long long limit_ns) {
    __shared__ float scratch[32];
    __shared__ int arrived;
    if (threadIdx.x == 0) {
        const bool got = wait_flag(counter, target, limit_ns);
        if (!got) atomicOr(status, sm100::kErrPeerFlag);
        arrived = got ? 1 : 0;
        __threadfence_system();
    }
    __syncthreads();
    if (!arrived) return;
    const long long nvec = n_shard / 8;
    float ss = 0.f;
    for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < nvec;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
        float acc[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) acc[k] = 0.f;
        for (int s = 0; s < world; ++s) {
            const int src = (rank + s) % world;
            Vec16<bf16> v = Vec16<bf16>::load_stream(landing + src * n_shard + i * 8);
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] += __bfloat162float(v.v[k]);
        }
        Vec16<bf16> o;
        if (accumulate) {
            Vec16<bf16> old = Vec16<bf16>::load(dst + i * 8);
#pragma unroll
            for (int k = 0; k < 8; k += 2) {
                const uint32_t r = rng_u32(static_cast<uint64_t>(i) * 4 + k / 2, seed);
                o.v[k] = sr_bf16(acc[k] * scale + __bfloat162float(old.v[k]), r);
                o.v[k + 1] = sr_bf16(acc[k + 1] * scale + __bfloat162float(old.v[k + 1]), r >> 16);
            }
        } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) o.v[k] = __float2bfloat16_rn(acc[k] * scale);
        }
        if (norm_partials) {
#pragma unroll
            for (int k = 0; k < 8; ++k) { float f = __bfloat162float(o.v[k]); ss += f * f; }
        }
        o.store(dst + i * 8);
    }
    if (norm_partials) {
        ss = block_reduce_sum(ss, scratch);
        if (threadIdx.x == 0) norm_partials[blockIdx.x] += ss;
    }
}

// ------------------------------------------------------------------------------------------------
// small all-reduce: push my n floats into slot [rank] of every peer, flag, wait, reduce locally.  One CTA.
__global__ void __launch_bounds__(256)
allreduce_small_kernel(PeerTable peers, long long slots_offset_bytes, long long flag_offset_bytes, float* data, int n, int rank, int world,
                       int op /*0 sum, 1 max, 2 avg*/, unsigned int gen, unsigned int* status, unsigned long long limit_ns) {
    __shared__ int ok;
    // two slot sets, alternating by generation: a fast peer may already push generation g+1 while this rank still reads g
    slots_offset_bytes += static_cast<long long>(gen & 1u) * world * n * static_cast<long long>(sizeof(float));
    for (int p = 0; p < world; ++p) {
        float* slot = reinterpret_cast<float*>(static_cast<char*>(peers.base[p]) + slots_offset_bytes) + static_cast<long long>(rank) * n;
        for (int i = threadIdx.x; i < n; i += blockDim.x) slot[i] = data[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x < world) {
        unsigned int* f = reinterpret_cast<unsigned int*>(static_cast<char*>(peers.base[threadIdx.x]) + flag_offset_bytes) + rank;
        st_release_sys(f, gen);
    }
    if (threadIdx.x == 0) ok = 1;
    __syncthreads();
    if (threadIdx.x < world) {
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(static_cast<char*>(peers.base[rank]) + flag_offset_bytes) + threadIdx.x;
        if (!wait_flag(mine, gen, limit_ns)) { atomicOr(status, sm100::kErrPeerFlag); ok = 0; }
    }
    __threadfence_system();
    __syncthreads();
    if (!ok) return;
    const float* slots = reinterpret_cast<const float*>(static_cast<char*>(peers.base[rank]) + slots_offset_bytes);
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float r = op == 1 ? -INFINITY : 0.f;
        for (int p = 0; p < world; ++p) {
            float v = slots[static_cast<long long>(p) * n + i];
            r = op == 1 ? fmaxf(r, v) : r + v;
        }
        if (op == 2) r /= world;
        data[i] = r;
    }
}

PeerTable make_table(void* const* peer_bases, int world) {
    PeerTable t{};
    for (int i = 0; i < world && i < MAX_PEERS; ++i) t.base[i] = peer_bases[i];
    return t;
}
int grid_for(long long items, int threads, int num_sms, int per_sm) {
    long long blocks = ceil_div_ll(items, threads);
    long long cap = static_cast<long long>(num_sms) * per_sm;
    return static_cast<int>(blocks < cap ? (blocks > 0 ? blocks : 1) : cap);
}

}  // namespace

// out_dtype: 1 = e4m3 with per-tensor scale, 0 = bf16 copy.  n = elements of the local shard (multiple of 8).
extern "C" int llmq_p2p_quant_allgather(void* const* peer_bases, long long dst_offset_bytes, const void* src, long long n, int rank,
                                        int world, const float* absmax, float* scale_out, int out_dtype, int num_sms, cudaStream_t s) {
    if (n <= 0) return 0;
    if (n % 8 || world > MAX_PEERS) return -1;
    PeerTable t = make_table(peer_bases, world);
    int g = grid_for(n / 8, 512, num_sms, 2);
    if (out_dtype == 1) quant_allgather_kernel<e4m3><<<g, 512, 0, s>>>(t, dst_offset_bytes, static_cast<const bf16*>(src), n, rank, world, absmax, scale_out);
    else if (out_dtype == 0) quant_allgather_kernel<bf16><<<g, 512, 0, s>>>(t, dst_offset_bytes, static_cast<const bf16*>(src), n, rank, world, nullptr, nullptr);
    else return -10;
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_p2p_signal(void* const* peer_bases, long long flag_offset_bytes, int rank, int world, unsigned int gen, cudaStream_t s) {
    if (world > MAX_PEERS) return -1;
    signal_kernel<<<1, 32, 0, s>>>(make_table(peer_bases, world), flag_offset_bytes, rank, world, gen);
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_p2p_wait(const unsigned int* local_flags, int world, unsigned int gen, unsigned int* status, double limit_seconds,
                             cudaStream_t s) {
    wait_kernel<<<1, 32, 0, s>>>(local_flags, world, gen, status, static_cast<unsigned long long>(limit_seconds * 1e9));
    return LLMQ_LAUNCH_CHECK();
}

// n_shard = elements of this rank's slice (multiple of 8); the full tensor has world * n_shard bf16 elements at src_offset_bytes.
extern "C" int llmq_p2p_reduce_scatter(void* const* peer_bases, const void* multicast_base, long long src_offset_bytes, long long n_shard,
                                       int rank, int world, void* dst, int accumulate, float scale, float* norm_partials,
                                       int num_partials, unsigned int seed, int num_sms, cudaStream_t s) {
    if (n_shard <= 0) return 0;
    if (n_shard % 8 || world > MAX_PEERS) return -1;
    int g = norm_partials ? num_partials : grid_for(n_shard / 8, 512, num_sms, 2);
    reduce_scatter_kernel<<<g, 512, 0, s>>>(make_table(peer_bases, world), multicast_base, src_offset_bytes, n_shard, rank, world,
                                            static_cast<bf16*>(dst), accumulate, scale, norm_partials, seed);
    return LLMQ_LAUNCH_CHECK();
}

extern "C" int llmq_p2p_allreduce_small(void* const* peer_bases, long long slots_offset_bytes, long long flag_offset_bytes, float* data,
                                        int n, int rank, int world, int op, unsigned int gen, unsigned int* status, double limit_seconds,
                                        cudaStream_t s) {
    if (world > MAX_PEERS || n <= 0) return -1;
    allreduce_small_kernel<<<1, 256, 0, s>>>(make_table(peer_bases, world), slots_offset_bytes, flag_offset_bytes, data, n, rank, world, op,
                                             gen, status, static_cast<unsigned long long>(limit_seconds * 1e9));
    return LLMQ_LAUNCH_CHECK();
}

// landing: this rank's landing buffer [world][n_shard] bf16 (local memory); counter: its local arrival counter.
extern "C" int llmq_p2p_rs_finish(const void* landing, const unsigned int* counter, unsigned int target, long long n_shard, int rank,
                                  int world, void* dst, int accumulate, float scale, float* norm_partials, int num_partials,
                                  unsigned int seed, unsigned int* status, double limit_seconds, int num_sms, cudaStream_t s) {
    if (n_shard <= 0) return 0;
    if (n_shard % 8 || world > MAX_PEERS) return -1;
    int g = norm_partials ? num_partials : grid_for(n_shard / 8, 512, num_sms, 2);
    rs_finish_kernel<<<g, 512, 0, s>>>(static_cast<const bf16*>(landing), counter, target, n_shard, rank, world, static_cast<bf16*>(dst),
                                       accumulate, scale, norm_partials, seed, status, static_cast<unsigned long long>(limit_seconds * 1e9));
    return LLMQ_LAUNCH_CHECK();
}

// Copy-engine transfer between two device addresses of this process' address space; a peer GPU's mapped segment counts
// (--memcpy-all-gather / --memcpy-send-recv: the reference's cudaMemcpyAsync collectives, src/utilities/comm.cpp:570-618).
extern "C" int llmq_memcpy_d2d_async(void* dst, const void* src, long long bytes, cudaStream_t s) {
    if (bytes <= 0) return 0;
    return static_cast<int>(cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDeviceToDevice, s));
}
