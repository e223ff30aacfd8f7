// Benchmark driver for the UNMODIFIED reference (IST-DASLab/llmq), linked against its llmq-common library.
//
// It runs the reference's own training step through the reference's public C++ API and stock code path:
// TransformerConfig by model name, LLamaOptions as the `train` executable fills them, one rank thread per GPU
// (NCCLCommunicator::launch_threads_communicators, src/utilities/comm.cpp:472-498), LLamaModel::allocate_run_state /
// init_weights, then per optimizer step the loop of train.cpp:556-577: token batch into the model's pinned host
// buffers, forward, backward (grad-accum times), update, and the host read of loss and gradient norm.
// Nothing of this repository's own framework is linked or loaded.
//
// Output: one JSON line on stdout (rank 0) with the device-timed and the end-to-end duration of K steps.
// Device time: CUDA events on the model's main stream around the K steps, max over ranks.
// End to end: host clock around K steps that each include copying that step's tokens into the pinned input
// buffers (the H2D copy itself is issued by LLamaModel::forward) and reading loss and norm back on the host.

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <random>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "models/llama_model.h"
#include "models/llama_run_state.h"
#include "training/transformer_config.h"
#include "utilities/allocator.h"
#include "utilities/comm.h"
#include "utilities/dtype.h"
#include "utilities/tensor.h"

namespace {

struct Args {
    std::string Model = "Qwen2.5-7B";
    int GPUs = 1, Steps = 5, Warmup = 3, B = 8, T = 2048, GradAcc = 1, ZeroLevel = 0;
    std::string MatmulDType = "e4m3", ModelDType = "bf16", OptDType = "bf16";
    LLamaOptions Options;
};

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { \
    fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); std::exit(3); } } while (0)

bool flag(const char* a, const char* name) { return std::strcmp(a, name) == 0; }

Args parse(int argc, char** argv) {
    Args a;
    auto& o = a.Options;
    o.LMHeadChunks = 4;
    for (int i = 1; i < argc; ++i) {
        auto next = [&]() -> const char* { if (i + 1 >= argc) { fprintf(stderr, "missing value for %s\n", argv[i]); std::exit(2); } return argv[++i]; };
        const char* s = argv[i];
        if (flag(s, "--model")) a.Model = next();
        else if (flag(s, "--gpus")) a.GPUs = std::atoi(next());
        else if (flag(s, "--steps")) a.Steps = std::atoi(next());
        else if (flag(s, "--warmup")) a.Warmup = std::atoi(next());
        else if (flag(s, "--batch")) a.B = std::atoi(next());
        else if (flag(s, "--seq-len")) a.T = std::atoi(next());
        else if (flag(s, "--grad-accumulation")) a.GradAcc = std::atoi(next());
        else if (flag(s, "--zero-level")) a.ZeroLevel = std::atoi(next());
        else if (flag(s, "--matmul-dtype")) a.MatmulDType = next();
        else if (flag(s, "--model-dtype")) a.ModelDType = next();
        else if (flag(s, "--opt-dtype")) a.OptDType = next();
        else if (flag(s, "--lmhead-chunks")) o.LMHeadChunks = std::atoi(next());
        else if (flag(s, "--attn-bwd-chunks")) o.AttBwdChunks = std::atoi(next());
        else if (flag(s, "--recompute-swiglu")) o.RecomputeSwiGLu = true;
        else if (flag(s, "--recompute-norm")) o.RecomputeRMSNorm = true;
        else if (flag(s, "--recompute-ffn")) o.RecomputeFFN = true;
        else if (flag(s, "--recompute-qkv")) o.RecomputeQKV = true;
        else if (flag(s, "--recompute-att")) o.RecomputeAtt = true;
        else if (flag(s, "--recompute-block")) o.RecomputeBlock = true;
        else if (flag(s, "--offload-residual")) o.OffloadResidual = true;
        else if (flag(s, "--use-cuda-graphs")) o.UseCudaGraphs = true;
        else if (flag(s, "--offload-master")) o.OffloadMaster = true;
        else if (flag(s, "--offload-opt-m")) o.OffloadOptM = true;
        else if (flag(s, "--offload-opt-v")) o.OffloadOptV = true;
        else if (flag(s, "--persistent-quants")) o.PersistentQuants = true;
        else if (flag(s, "--custom-matmul")) o.UseCustomMatmul = true;
        else if (flag(s, "--debug-time-breakdown")) o.TriggerTimingEvents = true;
        else { fprintf(stderr, "unknown argument %s\n", s); std::exit(2); }
    }
    // the same implications as the reference's command line (train.cpp:229-254)
    if (a.ZeroLevel == 0) a.ZeroLevel = a.GPUs > 1 ? 3 : 1;
    if (a.ZeroLevel >= 3) o.ShardWeights = true;
    if (a.ZeroLevel >= 2) o.ShardGradients = true;
    if (o.RecomputeBlock) { o.RecomputeAtt = o.RecomputeFFN = o.RecomputeRMSNorm = true; }
    if (o.RecomputeAtt) o.RecomputeQKV = true;
    if (o.RecomputeFFN) o.RecomputeSwiGLu = true;
    o.MatmulType = dtype_from_str(a.MatmulDType);
    o.OptMomentumType = dtype_from_str(a.OptDType);
    o.OptVarianceType = dtype_from_str(a.OptDType);
    return a;
}

struct Result { float DeviceMs; float E2EMs; float Loss; float Norm; };

void run_rank(const Args& args, NCCLCommunicator& comm, Result* out) {
    const int B = args.B, T = args.T, GA = args.GradAcc;
    TransformerConfig config = create_config_from_name(args.Model, dtype_from_str(args.ModelDType));
    LLamaOptions options = args.Options;
    options.ModelType = config.DType;

    auto allocator = std::make_shared<TensorAllocator>();
    LLamaModel model{config, options, comm.rank(), comm.world_size(), allocator};
    model.allocate_run_state(options, comm, B, T);
    model.init_weights(comm);

    Tensor inputs = model.get_input_buffer();      // pinned host memory, (B, T) int32
    Tensor targets = model.get_target_buffer();

    // uniform-random token pool; every micro-step copies a fresh batch into the model's pinned buffers
    const int n_pool = std::min(256, GA * (args.Warmup + 2 * args.Steps));
    std::mt19937 gen(1234 + comm.rank());
    std::uniform_int_distribution<int> dist(0, config.VocabSize - 1);
    std::vector<std::vector<int>> pool(n_pool, std::vector<int>((size_t)B * (T + 1)));
    for (auto& p : pool) for (auto& v : p) v = dist(gen);

    auto load_batch = [&](int k) {
        const std::vector<int>& p = pool[k % n_pool];
        int* in = inputs.get<int>();
        int* tg = targets.get<int>();
        for (int b = 0; b < B; ++b) {
            std::memcpy(in + (size_t)b * T, p.data() + (size_t)b * (T + 1), sizeof(int) * T);
            std::memcpy(tg + (size_t)b * T, p.data() + (size_t)b * (T + 1) + 1, sizeof(int) * T);
        }
    };

    int step_no = 0, batch_no = 0;
    float loss = 0.f, norm = 0.f;
    auto one_step = [&](bool read_back) {
        for (int j = 0; j < GA; ++j) {
            load_batch(batch_no++);
            model.forward(inputs, comm, j);
            model.backward(inputs, targets, comm, 0.f, GA, j);
        }
        ++step_no;
        model.update(comm, 1e-5f, 0.9f, 0.95f, step_no, 1e-8f, 0.1f, 1.0f);
        CK(cudaDeviceSynchronize());                                   // as train.cpp:577 does after every update
        if (read_back) {
            loss = model.get_loss() / (float)((long)B * T * GA);      // waits for the backward-done event
            norm = model.get_norm();                                  // waits for the norm-done event
        }
    };

    for (int i = 0; i < args.Warmup; ++i) one_step(true);
    CK(cudaDeviceSynchronize());
    comm.barrier();

    cudaStream_t main_stream = model.run_state().MainStream;
    cudaEvent_t ev0, ev1;
    CK(cudaEventCreate(&ev0));
    CK(cudaEventCreate(&ev1));

    if (comm.rank() == 0) { printf("TIMED_BEGIN\n"); fflush(stdout); }
    // pass 1: device time of K steps
    CK(cudaEventRecord(ev0, main_stream));
    for (int i = 0; i < args.Steps; ++i) one_step(false);
    CK(cudaEventRecord(ev1, main_stream));
    CK(cudaDeviceSynchronize());
    float dev_ms = 0.f;
    CK(cudaEventElapsedTime(&dev_ms, ev0, ev1));
    comm.barrier();

    // pass 2: end to end, host clock, loss and norm read every step
    auto t0 = std::chrono::steady_clock::now();
    for (int i = 0; i < args.Steps; ++i) one_step(true);
    CK(cudaDeviceSynchronize());
    auto t1 = std::chrono::steady_clock::now();
    float e2e_ms = std::chrono::duration<float, std::milli>(t1 - t0).count();
    comm.barrier();
    if (comm.rank() == 0) { printf("TIMED_END\n"); fflush(stdout); }
    if (options.TriggerTimingEvents && comm.rank() == 0) {
        // phase times of the last step, read from the reference's own timing events (as logging.cpp:367-396 does)
        auto& rs = model.run_state();
        for (size_t i = 0; i < rs.TimingForwardStart.size() && i < (size_t)GA; ++i) {
            float fwd = 0.f, head = 0.f, bwd = 0.f;
            CK(cudaEventSynchronize(rs.TimingBackwardEnd.at(i)));
            CK(cudaEventElapsedTime(&fwd, rs.TimingForwardStart.at(i), rs.TimingForwardEnd.at(i)));
            CK(cudaEventElapsedTime(&head, rs.TimingHeadStart.at(i), rs.TimingHeadEnd.at(i)));
            CK(cudaEventElapsedTime(&bwd, rs.TimingBackwardStart.at(i), rs.TimingBackwardEnd.at(i)));
            fprintf(stderr, "breakdown micro-step %zu: fwd %.2f ms, head %.2f ms, bwd %.2f ms\n", i, fwd, head, bwd - head);
        }
        float opt = 0.f;
        CK(cudaEventSynchronize(rs.TimingOptimizerEnd));
        CK(cudaEventElapsedTime(&opt, rs.TimingOptimizerStart, rs.TimingOptimizerEnd));
        fprintf(stderr, "breakdown optimizer: %.2f ms\n", opt);
    }

    out[comm.rank()] = Result{dev_ms, e2e_ms, loss, norm};
}

}  // namespace

int main(int argc, char** argv) {
    Args args = parse(argc, argv);
    int available = 0;
    CK(cudaGetDeviceCount(&available));
    if (args.GPUs > available) {
        printf("{\"impl\": \"reference\", \"unavailable\": \"requested %d GPUs, %d visible\"}\n", args.GPUs, available);
        return 0;
    }
    std::vector<Result> results(args.GPUs);
    try {
        NCCLCommunicator::run_threads_communicators(args.GPUs, false, false,
            [&](NCCLCommunicator& comm) { run_rank(args, comm, results.data()); });
    } catch (const std::exception& e) {
        fprintf(stderr, "reference run failed: %s\n", e.what());
        return 1;
    }
    float dev_ms = 0.f, e2e_ms = 0.f;
    for (auto& r : results) { dev_ms = std::max(dev_ms, r.DeviceMs); e2e_ms = std::max(e2e_ms, r.E2EMs); }
    const double tokens = (double)args.B * args.T * args.GradAcc * args.GPUs * args.Steps;
    printf("{\"device_ms\": %.3f, \"e2e_ms\": %.3f, \"tokens\": %.0f, \"device_tok_s\": %.1f, \"e2e_tok_s\": %.1f, "
           "\"loss\": %.5f, \"norm\": %.5f, \"h2d_bytes_per_step\": %ld, \"d2h_bytes_per_step\": %ld}\n",
           dev_ms, e2e_ms, tokens, tokens / (dev_ms * 1e-3), tokens / (e2e_ms * 1e-3), results[0].Loss, results[0].Norm,
           (long)2 * args.B * args.T * 4 * args.GradAcc, (long)(3 + (args.T + 511) / 512) * 4);
    return 0;
}
