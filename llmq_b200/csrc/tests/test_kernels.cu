// Native unit tests of the kernel library: each case runs a kernel through its C entry point and compares it with a
// plain C++ reference on the host (role of the reference's Catch2 suite, src/testing/test-swiglu.cu, test-rope.cu,
// test-classifier.cu, test-gemm.cpp), plus the block-scaled e4m3 quantiser and GEMM.  Build: python -m llmq_b200.build --tests ; run: build/test_kernels
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

extern "C" {
int llmq_swiglu_forward(void*, void*, const void*, long long, int, int, float*, const float*, float*, int, cudaStream_t);
int llmq_swiglu_backward(void*, const void*, const void*, long long, int, int, float*, int, cudaStream_t);
int llmq_rope(void*, const void*, const float*, int, int, int, int, int, int, int, float*, int, cudaStream_t);
int llmq_rope_table(float*, int, int, float, cudaStream_t);
int llmq_fused_classifier(void*, float*, float*, const int*, float, float, int, int, long long, int, int, cudaStream_t);
int llmq_gemm(const void*, const void*, void*, const void*, int, int, int, int, int, int, int, long long, long long, long long, int, int, int,
              const float*, const float*, float, float*, unsigned int*, int, cudaStream_t);
int llmq_quantize_mx(void*, void*, const void*, long long, long long, long long, int, int, cudaStream_t);
long long llmq_mx_sf_bytes(long long, long long, int);
int llmq_gemm_mx_tile_n();
int llmq_gemm_mx(const void*, const void*, const void*, const void*, void*, const void*, int, int, int, long long, long long, long long, int, int, int,
                 float, float*, unsigned int*, int, cudaStream_t);
}

namespace {
int g_failed = 0, g_sms = 148;
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(2); } } while (0)

struct Rng { unsigned long long s; float next() { s = s * 6364136223846793005ull + 1442695040888963407ull; return ((s >> 40) & 0xFFFFFF) / 8388608.0f - 1.0f; } };
float bf(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
template <typename T> T* to_dev(const std::vector<T>& h) { T* d; CK(cudaMalloc(&d, h.size() * sizeof(T))); CK(cudaMemcpy(d, h.data(), h.size() * sizeof(T), cudaMemcpyHostToDevice)); return d; }
template <typename T> std::vector<T> to_host(const T* d, size_t n) { std::vector<T> h(n); CK(cudaMemcpy(h.data(), d, n * sizeof(T), cudaMemcpyDeviceToHost)); return h; }
std::vector<__nv_bfloat16> as_bf16(const std::vector<float>& v) { std::vector<__nv_bfloat16> o(v.size()); for (size_t i = 0; i < v.size(); ++i) o[i] = __float2bfloat16_rn(v[i]); return o; }

void report(const char* name, double max_err, double tol) {
    const bool ok = max_err <= tol && max_err == max_err;
    printf("%-28s max err %.4g (tol %.3g) %s\n", name, max_err, tol, ok ? "PASS" : "FAIL");
    if (!ok) ++g_failed;
}

void test_swiglu() {
    const int rows = 300, D = 512;
    Rng r{1};
    std::vector<float> x(static_cast<size_t>(rows) * 2 * D), dy(static_cast<size_t>(rows) * D);
    for (auto& v : x) v = bf(2.f * r.next());
    for (auto& v : dy) v = bf(r.next());
    auto dx = to_dev(as_bf16(x)); auto ddy = to_dev(as_bf16(dy));
    __nv_bfloat16* dout; CK(cudaMalloc(&dout, sizeof(__nv_bfloat16) * rows * D));
    float* dam; CK(cudaMalloc(&dam, 4)); CK(cudaMemset(dam, 0, 4));
    if (llmq_swiglu_forward(dout, nullptr, dx, rows, D, 0, dam, nullptr, nullptr, g_sms, 0)) { printf("swiglu_forward launch failed\n"); ++g_failed; return; }
    auto out = to_host(dout, static_cast<size_t>(rows) * D);
    double err = 0, am_ref = 0;
    for (int i = 0; i < rows; ++i) for (int c = 0; c < D; ++c) {
        const float u = x[static_cast<size_t>(i) * 2 * D + c], g = x[static_cast<size_t>(i) * 2 * D + D + c];
        const float ref = u * g / (1.f + std::exp(-g));
        err = std::fmax(err, std::fabs(__bfloat162float(out[static_cast<size_t>(i) * D + c]) - ref) / (1.0 + std::fabs(ref)));
        am_ref = std::fmax(am_ref, std::fabs(bf(ref)));
    }
    report("swiglu forward", err, 1e-2);
    report("swiglu forward abs-max", std::fabs(to_host(dam, 1)[0] - am_ref) / am_ref, 1e-2);
    // backward, in place over the input
    if (llmq_swiglu_backward(dx, ddy, dx, rows, D, 0, nullptr, g_sms, 0)) { printf("swiglu_backward launch failed\n"); ++g_failed; return; }
    auto g_out = to_host(dx, static_cast<size_t>(rows) * 2 * D);
    err = 0;
    for (int i = 0; i < rows; ++i) for (int c = 0; c < D; ++c) {
        const float u = x[static_cast<size_t>(i) * 2 * D + c], g = x[static_cast<size_t>(i) * 2 * D + D + c], d = dy[static_cast<size_t>(i) * D + c];
        const float s = 1.f / (1.f + std::exp(-g));
        const float du = d * g * s, dg = d * u * s * (1.f + g * (1.f - s));
        err = std::fmax(err, std::fabs(__bfloat162float(g_out[static_cast<size_t>(i) * 2 * D + c]) - du) / (1.0 + std::fabs(du)));
        err = std::fmax(err, std::fabs(__bfloat162float(g_out[static_cast<size_t>(i) * 2 * D + D + c]) - dg) / (1.0 + std::fabs(dg)));
    }
    report("swiglu backward", err, 1e-2);
    cudaFree(dx); cudaFree(ddy); cudaFree(dout); cudaFree(dam);
}

void test_rope() {
    const int B = 2, T = 96, Hq = 4, Hkv = 2, HS = 64, H = Hq + 2 * Hkv;
    const float theta = 10000.f;
    Rng r{2};
    std::vector<float> x(static_cast<size_t>(B) * T * H * HS);
    for (auto& v : x) v = bf(r.next());
    auto dx = to_dev(as_bf16(x));
    float* dfreq; CK(cudaMalloc(&dfreq, sizeof(float) * T * HS));
    __nv_bfloat16* dy; CK(cudaMalloc(&dy, sizeof(__nv_bfloat16) * x.size()));
    if (llmq_rope_table(dfreq, T, HS, theta, 0) || llmq_rope(dy, dx, dfreq, B, T, Hq, Hkv, HS, 0, 0, nullptr, g_sms, 0)) { printf("rope launch failed\n"); ++g_failed; return; }
    auto y = to_host(dy, x.size());
    double err = 0;
    for (int b = 0; b < B; ++b) for (int t = 0; t < T; ++t) for (int h = 0; h < H; ++h) for (int d = 0; d < HS / 2; ++d) {
        const size_t base = ((static_cast<size_t>(b) * T + t) * H + h) * HS;
        const double ang = t * std::pow(static_cast<double>(theta), -2.0 * d / HS);
        const float c = static_cast<float>(std::cos(ang)), s = static_cast<float>(std::sin(ang));
        const float a = x[base + d], bb = x[base + d + HS / 2];
        const float r1 = h < Hq + Hkv ? a * c - bb * s : a, r2 = h < Hq + Hkv ? bb * c + a * s : bb;
        err = std::fmax(err, std::fabs(__bfloat162float(y[base + d]) - r1));
        err = std::fmax(err, std::fabs(__bfloat162float(y[base + d + HS / 2]) - r2));
    }
    report("rope forward", err, 1.5e-2);
    // backward of forward is the identity on the rotated heads (orthogonal rotation)
    if (llmq_rope(dy, dy, dfreq, B, T, Hq, Hkv, HS, 0, 1, nullptr, g_sms, 0)) { printf("rope backward launch failed\n"); ++g_failed; return; }
    auto z = to_host(dy, x.size());
    err = 0;
    for (size_t i = 0; i < x.size(); ++i) err = std::fmax(err, std::fabs(__bfloat162float(z[i]) - x[i]));
    report("rope backward(forward(x))", err, 2.5e-2);
    cudaFree(dx); cudaFree(dy); cudaFree(dfreq);
}

void test_classifier() {
    const int rows = 70, V = 1000;
    const float dloss = 0.25f;
    Rng r{3};
    std::vector<float> lg(static_cast<size_t>(rows) * V);
    for (auto& v : lg) v = bf(4.f * r.next());
    std::vector<int> tg(rows);
    for (int i = 0; i < rows; ++i) tg[i] = (i % 7 == 3) ? -100 : (i * 37) % V;      // some rows are masked out
    auto dlg = to_dev(as_bf16(lg)); auto dtg = to_dev(tg);
    float *dloss_out, *dlse; CK(cudaMalloc(&dloss_out, 4 * rows)); CK(cudaMalloc(&dlse, 4 * rows));
    CK(cudaMemset(dloss_out, 0, 4 * rows));
    if (llmq_fused_classifier(dlg, dloss_out, dlse, dtg, dloss, 0.f, rows, V, V, 0, 1, 0)) { printf("classifier launch failed\n"); ++g_failed; return; }
    auto losses = to_host(dloss_out, rows); auto grads = to_host(dlg, lg.size());
    double el = 0, eg = 0;
    for (int i = 0; i < rows; ++i) {
        double mx = -1e30, sum = 0;
        for (int c = 0; c < V; ++c) mx = std::fmax(mx, lg[static_cast<size_t>(i) * V + c]);
        for (int c = 0; c < V; ++c) sum += std::exp(lg[static_cast<size_t>(i) * V + c] - mx);
        const double lse = mx + std::log(sum);
        const bool masked = tg[i] < 0;
        const double ref = masked ? 0.0 : lse - lg[static_cast<size_t>(i) * V + tg[i]];
        el = std::fmax(el, std::fabs(losses[i] - ref));
        for (int c = 0; c < V; ++c) {
            const double p = std::exp(lg[static_cast<size_t>(i) * V + c] - lse);
            const double g = masked ? 0.0 : (p - (c == tg[i] ? 1.0 : 0.0)) * dloss;
            eg = std::fmax(eg, std::fabs(__bfloat162float(grads[static_cast<size_t>(i) * V + c]) - g));
        }
    }
    report("classifier loss", el, 2e-3);
    report("classifier dlogits", eg, 2e-3);
    cudaFree(dlg); cudaFree(dtg); cudaFree(dloss_out); cudaFree(dlse);
}

void test_gemm(bool fp8) {
    const int M = 384, N = 320, K = 256;
    Rng r{fp8 ? 5ull : 4ull};
    std::vector<float> a(static_cast<size_t>(M) * K), b(static_cast<size_t>(N) * K), bias(N);
    for (auto& v : a) v = r.next();
    for (auto& v : b) v = r.next();
    for (auto& v : bias) v = bf(r.next());
    void *da, *db;
    if (fp8) {
        std::vector<__nv_fp8_e4m3> qa(a.size()), qb(b.size());
        for (size_t i = 0; i < a.size(); ++i) { qa[i] = __nv_fp8_e4m3(a[i]); a[i] = static_cast<float>(qa[i]); }
        for (size_t i = 0; i < b.size(); ++i) { qb[i] = __nv_fp8_e4m3(b[i]); b[i] = static_cast<float>(qb[i]); }
        da = to_dev(qa); db = to_dev(qb);
    } else {
        for (auto& v : a) v = bf(v);
        for (auto& v : b) v = bf(v);
        da = to_dev(as_bf16(a)); db = to_dev(as_bf16(b));
    }
    auto dbias = to_dev(as_bf16(bias));
    __nv_bfloat16* dc; CK(cudaMalloc(&dc, sizeof(__nv_bfloat16) * M * N));
    unsigned int* dstatus; CK(cudaMalloc(&dstatus, 4)); CK(cudaMemset(dstatus, 0, 4));
    const int dt = fp8 ? 1 : 0;
    if (llmq_gemm(da, db, dc, dbias, M, N, K, dt, dt, 0, 0, K, K, N, 0, 0, 0, nullptr, nullptr, 1.f, nullptr, dstatus, g_sms, 0)) { printf("gemm launch failed\n"); ++g_failed; return; }
    auto c = to_host(dc, static_cast<size_t>(M) * N);
    double err = 0;
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) {
        double acc = bias[j];
        for (int k = 0; k < K; ++k) acc += static_cast<double>(a[static_cast<size_t>(i) * K + k]) * b[static_cast<size_t>(j) * K + k];
        err = std::fmax(err, std::fabs(__bfloat162float(c[static_cast<size_t>(i) * N + j]) - acc) / (1.0 + std::fabs(acc)));
    }
    report(fp8 ? "gemm e4m3 + bias" : "gemm bf16 + bias", err, 1e-2);
    report("gemm status word", static_cast<double>(to_host(dstatus, 1)[0]), 0.0);
    cudaFree(da); cudaFree(db); cudaFree(dbias); cudaFree(dc); cudaFree(dstatus);
}
// Block-scaled e4m3: device quantiser -> host dequantisation through the tiled scale layout -> GEMM against a double sum.
std::vector<float> dequant_mx(const std::vector<__nv_fp8_e4m3>& q, const std::vector<unsigned char>& sf, int rows, int K, int tile_rows) {
    const int chunks = (tile_rows + 127) / 128, n_tiles = (rows + tile_rows - 1) / tile_rows;
    std::vector<float> out(q.size());
    for (int r = 0; r < rows; ++r) for (int k = 0; k < K; ++k) {
        const int kb = k / 32, tile = r / tile_rows, rt = r % tile_rows, rr = rt % 128;
        const size_t off = ((static_cast<size_t>(kb / 4) * n_tiles + tile) * chunks + rt / 128) * 512 + (rr % 32) * 16 + (rr / 32) * 4 + kb % 4;
        out[static_cast<size_t>(r) * K + k] = static_cast<float>(q[static_cast<size_t>(r) * K + k]) * std::ldexp(1.0f, static_cast<int>(sf[off]) - 127);
    }
    return out;
}

void test_gemm_mx() {
    const int M = 200, N = 300, K = 384, TN = llmq_gemm_mx_tile_n();
    Rng r{9ull};
    std::vector<float> a(static_cast<size_t>(M) * K), b(static_cast<size_t>(N) * K);
    // blocks of very different magnitude: a per-tensor scale would flush the small ones to zero
    for (size_t i = 0; i < a.size(); ++i) a[i] = bf(r.next() * std::ldexp(1.0f, static_cast<int>(i / 32 % 13) - 6));
    for (size_t i = 0; i < b.size(); ++i) b[i] = bf(r.next() * std::ldexp(1.0f, static_cast<int>(i / 32 % 11) - 5));
    auto da = to_dev(as_bf16(a)); auto db = to_dev(as_bf16(b));
    const size_t sfa_bytes = llmq_mx_sf_bytes(M, K, 128), sfb_bytes = llmq_mx_sf_bytes(N, K, TN);
    __nv_fp8_e4m3 *qa, *qb; unsigned char *sfa, *sfb; float* dc; unsigned int* dstatus;
    CK(cudaMalloc(&qa, a.size())); CK(cudaMalloc(&qb, b.size())); CK(cudaMalloc(&sfa, sfa_bytes)); CK(cudaMalloc(&sfb, sfb_bytes));
    CK(cudaMalloc(&dc, sizeof(float) * M * N)); CK(cudaMalloc(&dstatus, 4)); CK(cudaMemset(dstatus, 0, 4));
    int rc = llmq_quantize_mx(qa, sfa, da, M, K, K, 0, 128, 0);
    rc |= llmq_quantize_mx(qb, sfb, db, N, K, K, 0, TN, 0);
    rc |= llmq_gemm_mx(qa, qb, sfa, sfb, dc, nullptr, M, N, K, K, K, N, 1, 0, 0, 1.f, nullptr, dstatus, g_sms, 0);
    if (rc) { printf("block-scaled gemm launch failed (%d)\n", rc); ++g_failed; return; }
    auto c = to_host(dc, static_cast<size_t>(M) * N);
    auto fa = dequant_mx(to_host(qa, a.size()), to_host(sfa, sfa_bytes), M, K, 128);
    auto fb = dequant_mx(to_host(qb, b.size()), to_host(sfb, sfb_bytes), N, K, TN);
    double err = 0, qerr = 0;
    for (size_t i = 0; i < a.size(); i += 32) {          // every block reproduces its values to e4m3 precision of its own maximum
        double mx = 0, e = 0;
        for (int j = 0; j < 32; ++j) { mx = std::fmax(mx, std::fabs(a[i + j])); e = std::fmax(e, std::fabs(a[i + j] - fa[i + j])); }
        qerr = std::fmax(qerr, mx > 0 ? e / mx : 0.0);
    }
    for (int i = 0; i < M; ++i) for (int j = 0; j < N; ++j) {
        double acc = 0;
        for (int k = 0; k < K; ++k) acc += static_cast<double>(fa[static_cast<size_t>(i) * K + k]) * fb[static_cast<size_t>(j) * K + k];
        err = std::fmax(err, std::fabs(c[static_cast<size_t>(i) * N + j] - acc) / (1.0 + std::fabs(acc)));
    }
    report("quantize mx (per-block error)", qerr, 0.0626);
    report("gemm mx e4m3", err, 1e-3);      // fp32 accumulation over blocks whose magnitudes span 2^22
    report("gemm mx status word", static_cast<double>(to_host(dstatus, 1)[0]), 0.0);
    cudaFree(da); cudaFree(db); cudaFree(qa); cudaFree(qb); cudaFree(sfa); cudaFree(sfb); cudaFree(dc); cudaFree(dstatus);
}
}  // namespace

int main() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { printf("no CUDA device\n"); return 77; }
    cudaDeviceProp prop;
    CK(cudaGetDeviceProperties(&prop, dev));
    g_sms = prop.multiProcessorCount;
    test_swiglu();
    test_rope();
    test_classifier();
    test_gemm(false);
    test_gemm(true);
    test_gemm_mx();
    CK(cudaDeviceSynchronize());
    printf("%s\n", g_failed ? "SOME TESTS FAILED" : "ALL TESTS PASSED");
    return g_failed ? 1 : 0;
}
