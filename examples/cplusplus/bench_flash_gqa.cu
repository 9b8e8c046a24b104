// C++ bench harness for the GQA path.  It does what upstream's examples/cplusplus/test_decode_flash_gqa.cu does in
// one run -- random inputs, a CPU reference timed on the host cores (omp_get_wtime, thread count printed), the
// GPU launch timed with CUDA events, time / bandwidth / FLOP rate printed, relative error against the CPU reference
// printed -- with warm-up and repeated launches, decimal units, a pass/fail exit code, and a second case for the
// prefill forward (which upstream only has in Triton) through LaunchFlashGqaForwardBf16Kernel.
//
//   cmake -S . -B build -DCMAKE_CUDA_ARCHITECTURES=100a && cmake --build build -j       (see CMakeLists.txt), or
//   nvcc -std=c++17 -O3 -Xcompiler=-fopenmp -gencode arch=compute_100a,code=sm_100a -I include/cplusplus -I include \
//        examples/cplusplus/bench_flash_gqa.cu -L cuda_llm_ops_b200 -lcllo_flash_gqa \
//        -Xlinker -rpath=$PWD/cuda_llm_ops_b200 -o build/bench_flash_gqa
//   ./build/bench_flash_gqa [B S Hq Hkv iters]        decode shape (default: B=60 S=4096 Hq=128 Hkv=8, 50 launches)
//
// The CPU references below are plain two-pass softmax attention in fp32 with fp64 accumulation of the output; they
// are this harness's own checker, independent of the kernels' tiling.
#include "cuda_llm_ops.h"

#include <cuda_runtime.h>
#include <omp.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <random>
#include <vector>

#define CHECK(x)                                                                              \
    do {                                                                                      \
        cudaError_t e_ = (x);                                                                 \
        if (e_ != cudaSuccess) {                                                              \
            std::fprintf(stderr, "%s failed: %s\n", #x, cudaGetErrorString(e_));              \
            return 1;                                                                         \
        }                                                                                     \
    } while (0)

namespace {

constexpr int D = 128;

// N(0,1) rounded to bf16; every chunk of 2^20 elements has its own generator so that the fill runs on all cores
void fill_normal(std::vector<__nv_bfloat16>& dst, unsigned seed) {
    const long long n = static_cast<long long>(dst.size()), chunk = 1 << 20;
#pragma omp parallel for schedule(dynamic)
    for (long long c0 = 0; c0 < n; c0 += chunk) {
        std::mt19937 gen(seed * 7919u + static_cast<unsigned>(c0 / chunk));
        std::normal_distribution<float> dist(0.f, 1.f);
        const long long c1 = c0 + chunk < n ? c0 + chunk : n;
        for (long long i = c0; i < c1; ++i) dst[i] = __float2bfloat16(dist(gen));
    }
}

std::vector<float> to_float(const std::vector<__nv_bfloat16>& src) {
    std::vector<float> out(src.size());
#pragma omp parallel for
    for (long long i = 0; i < static_cast<long long>(src.size()); ++i) out[i] = __bfloat162float(src[i]);
    return out;
}

// softmax(scale * q . K^T) V for one query vector against keys [0, n) of one kv head; K/V rows are `stride` floats apart
void attend(const float* q, const float* k, const float* v, long long stride, int n, float scale, float* out,
            std::vector<float>& score) {
    float mx = -INFINITY;
    for (int s = 0; s < n; ++s) {
        const float* kr = k + s * stride;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) acc += q[d] * kr[d];
        score[s] = acc * scale;
        mx = std::fmax(mx, score[s]);
    }
    double o[D] = {0.0}, l = 0.0;
    for (int s = 0; s < n; ++s) {
        const float p = std::exp(score[s] - mx);
        const float* vr = v + s * stride;
        l += p;
        for (int d = 0; d < D; ++d) o[d] += static_cast<double>(p) * vr[d];
    }
    for (int d = 0; d < D; ++d) out[d] = static_cast<float>(o[d] / l);
}

double relative_error(const std::vector<float>& want, const std::vector<float>& got) {
    double num = 0.0, den = 0.0;
    for (size_t i = 0; i < want.size(); ++i) {
        num += (static_cast<double>(got[i]) - want[i]) * (static_cast<double>(got[i]) - want[i]);
        den += static_cast<double>(want[i]) * want[i];
    }
    return std::sqrt(num) / std::sqrt(den);
}

}  // namespace

// ---------------------------------------------------------------------------------------------------------------
// decode: Q [B,Hq,D], K/V [B,S,Hkv,D] (upstream's C++ layout), through upstream's launcher and through the C ABI
// ---------------------------------------------------------------------------------------------------------------
static int run_decode(int B, int S, int Hq, int Hkv, int iters) {
    const int G = Hq / Hkv;
    const size_t nq = static_cast<size_t>(B) * Hq * D, nkv = static_cast<size_t>(B) * S * Hkv * D;
    const float scale = 1.f / std::sqrt(static_cast<float>(D));
    std::vector<__nv_bfloat16> hq(nq), hk(nkv), hv(nkv), ho(nq);
    fill_normal(hq, 1u);
    fill_normal(hk, 2u);
    fill_normal(hv, 3u);

    // CPU reference, parallel over (batch, query head)
    const std::vector<float> fq = to_float(hq), fk = to_float(hk), fv = to_float(hv);
    std::vector<float> want(nq);
    const double c0 = omp_get_wtime();
#pragma omp parallel
    {
        std::vector<float> score(S);
#pragma omp for collapse(2) schedule(dynamic)
        for (int b = 0; b < B; ++b)
            for (int h = 0; h < Hq; ++h) {
                const size_t kv0 = (static_cast<size_t>(b) * S * Hkv + h / G) * D;
                attend(&fq[(static_cast<size_t>(b) * Hq + h) * D], &fk[kv0], &fv[kv0], static_cast<long long>(Hkv) * D, S,
                       scale, &want[(static_cast<size_t>(b) * Hq + h) * D], score);
            }
    }
    const double cpu_s = omp_get_wtime() - c0;
    const double bytes = 2.0 * nkv * 2 + 2.0 * nq * 2, flops = 4.0 * B * Hq * static_cast<double>(S) * D;
    std::printf("decode  B=%d S=%d Hq=%d Hkv=%d D=%d\n", B, S, Hq, Hkv, D);
    std::printf("  CPU reference             : %.3f s on %d threads, %.4f TB/s, %.4f TFLOP/s\n", cpu_s,
                omp_get_max_threads(), bytes / cpu_s / 1e12, flops / cpu_s / 1e12);

    __nv_bfloat16 *q, *k, *v, *o;
    float* inter;
    void* ws;
    CHECK(cudaMalloc(&q, nq * 2));
    CHECK(cudaMalloc(&k, nkv * 2));
    CHECK(cudaMalloc(&v, nkv * 2));
    CHECK(cudaMalloc(&o, nq * 2));
    CHECK(cudaMalloc(&inter, nq * 4));
    const size_t ws_bytes = cllo_gqa_decode_workspace_bytes(B, S, Hq, Hkv, D, 0);
    CHECK(cudaMalloc(&ws, ws_bytes));
    CHECK(cudaMemset(ws, 0, ws_bytes));
    CHECK(cudaMemcpy(q, hq.data(), nq * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(k, hk.data(), nkv * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(v, hv.data(), nkv * 2, cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CHECK(cudaStreamCreate(&stream));
    cudaEvent_t t0, t1;
    CHECK(cudaEventCreate(&t0));
    CHECK(cudaEventCreate(&t1));
    float ms = 0.f;
    int bad = 0;
    for (int variant = 0; variant < 2; ++variant) {
        CHECK(cudaMemset(o, 0, nq * 2));
        auto call = [&]() {
            if (variant == 0) {  // upstream's launcher signature: default stream, void
                LaunchFlashGqaBf16Kernel(q, k, v, scale, o, inter, B, S, Hq, Hkv, D);
                return CLLO_OK;
            }
            // the explicit C ABI: caller-owned (zeroed) workspace, caller's stream
            return cllo_gqa_decode_bf16(q, k, v, scale, o, ws, ws_bytes, B, S, Hq, Hkv, D,
                                        CLLO_KV_BSHD | CLLO_WS_COUNTERS_ZERO, 0, nullptr, stream);
        };
        cudaStream_t st = variant == 0 ? nullptr : stream;
        for (int i = 0; i < 5; ++i) {
            const int rc = call();
            if (rc != CLLO_OK) {
                std::fprintf(stderr, "decode call failed: %s\n", cllo_status_string(rc));
                return 1;
            }
        }
        CHECK(cudaStreamSynchronize(st));
        CHECK(cudaEventRecord(t0, st));
        for (int i = 0; i < iters; ++i) (void)call();
        CHECK(cudaEventRecord(t1, st));
        CHECK(cudaEventSynchronize(t1));
        CHECK(cudaEventElapsedTime(&ms, t0, t1));
        CHECK(cudaMemcpy(ho.data(), o, nq * 2, cudaMemcpyDeviceToHost));
        const double err = relative_error(want, to_float(ho)), us = ms / iters * 1e3;
        std::printf("  %-26s: %.1f us, %.3f TB/s, %.2f TFLOP/s, O error = %.3g\n",
                    variant == 0 ? "LaunchFlashGqaBf16Kernel" : "cllo_gqa_decode_bf16", us, bytes / us / 1e6,
                    flops / us / 1e6, err);
        if (!(err < 2e-2)) bad = 1;
    }
    cudaFree(q);
    cudaFree(k);
    cudaFree(v);
    cudaFree(o);
    cudaFree(inter);
    cudaFree(ws);
    cudaStreamDestroy(stream);
    return bad;
}

// ---------------------------------------------------------------------------------------------------------------
// prefill forward: Q/O [B,Hq,S,D], K/V [B,Hkv,S,D] (upstream's Triton layout), through LaunchFlashGqaForwardBf16Kernel.
// The CPU reference covers every `row_step`-th query row of every head (the whole problem is hundreds of GFLOP).
// ---------------------------------------------------------------------------------------------------------------
static int run_prefill(int B, int S, int Hq, int Hkv, bool causal, int iters, int row_step) {
    const int G = Hq / Hkv;
    const size_t nq = static_cast<size_t>(B) * Hq * S * D, nkv = static_cast<size_t>(B) * Hkv * S * D;
    const float scale = 1.f / std::sqrt(static_cast<float>(D));
    std::vector<__nv_bfloat16> hq(nq), hk(nkv), hv(nkv), ho(nq);
    fill_normal(hq, 11u);
    fill_normal(hk, 12u);
    fill_normal(hv, 13u);
    const std::vector<float> fq = to_float(hq), fk = to_float(hk), fv = to_float(hv);
    const int n_rows = (S + row_step - 1) / row_step;
    std::vector<float> want(static_cast<size_t>(B) * Hq * n_rows * D);
    double cpu_flops = 0.0;
    const double c0 = omp_get_wtime();
#pragma omp parallel reduction(+ : cpu_flops)
    {
        std::vector<float> score(S);
#pragma omp for collapse(2) schedule(dynamic)
        for (int bh = 0; bh < B * Hq; ++bh)
            for (int r = 0; r < n_rows; ++r) {
                const int b = bh / Hq, h = bh % Hq, row = r * row_step;
                const int n = causal ? row + 1 : S;
                const size_t kv0 = (static_cast<size_t>(b) * Hkv + h / G) * S * D;
                attend(&fq[(static_cast<size_t>(bh) * S + row) * D], &fk[kv0], &fv[kv0], D, n, scale,
                       &want[(static_cast<size_t>(bh) * n_rows + r) * D], score);
                cpu_flops += 4.0 * n * D;
            }
    }
    const double cpu_s = omp_get_wtime() - c0;
    const double flops = 4.0 * B * Hq * static_cast<double>(S) * S * D * (causal ? 0.5 : 1.0);
    std::printf("prefill %s  B=%d S=%d Hq=%d Hkv=%d D=%d\n", causal ? "causal" : "non-causal", B, S, Hq, Hkv, D);
    std::printf("  CPU reference             : %.3f s on %d threads for every %d-th query row, %.4f TFLOP/s\n", cpu_s,
                omp_get_max_threads(), row_step, cpu_flops / cpu_s / 1e12);

    __nv_bfloat16 *q, *k, *v, *o;
    float* lse;
    CHECK(cudaMalloc(&q, nq * 2));
    CHECK(cudaMalloc(&k, nkv * 2));
    CHECK(cudaMalloc(&v, nkv * 2));
    CHECK(cudaMalloc(&o, nq * 2));
    CHECK(cudaMalloc(&lse, static_cast<size_t>(B) * Hq * S * 4));
    CHECK(cudaMemcpy(q, hq.data(), nq * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(k, hk.data(), nkv * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemcpy(v, hv.data(), nkv * 2, cudaMemcpyHostToDevice));
    CHECK(cudaMemset(o, 0, nq * 2));
    cudaEvent_t t0, t1;
    CHECK(cudaEventCreate(&t0));
    CHECK(cudaEventCreate(&t1));
    for (int i = 0; i < 5; ++i) LaunchFlashGqaForwardBf16Kernel(q, k, v, scale, causal, o, lse, B, S, S, Hq, Hkv, D);
    CHECK(cudaDeviceSynchronize());
    CHECK(cudaEventRecord(t0));
    for (int i = 0; i < iters; ++i) LaunchFlashGqaForwardBf16Kernel(q, k, v, scale, causal, o, lse, B, S, S, Hq, Hkv, D);
    CHECK(cudaEventRecord(t1));
    CHECK(cudaEventSynchronize(t1));
    float ms = 0.f;
    CHECK(cudaEventElapsedTime(&ms, t0, t1));
    CHECK(cudaMemcpy(ho.data(), o, nq * 2, cudaMemcpyDeviceToHost));
    std::vector<float> got(want.size());
    for (int bh = 0; bh < B * Hq; ++bh)
        for (int r = 0; r < n_rows; ++r)
            for (int d = 0; d < D; ++d)
                got[(static_cast<size_t>(bh) * n_rows + r) * D + d] =
                    __bfloat162float(ho[(static_cast<size_t>(bh) * S + static_cast<size_t>(r) * row_step) * D + d]);
    const double err = relative_error(want, got), us = ms / iters * 1e3;
    std::printf("  %-26s: %.1f us, %.1f TFLOP/s, O error = %.3g (sampled rows)\n", "LaunchFlashGqaForwardBf16Kernel", us,
                flops / us / 1e6, err);
    cudaFree(q);
    cudaFree(k);
    cudaFree(v);
    cudaFree(o);
    cudaFree(lse);
    return err < 2e-2 ? 0 : 1;
}

int main(int argc, char** argv) {
    const int B = argc > 1 ? std::atoi(argv[1]) : 60, S = argc > 2 ? std::atoi(argv[2]) : 4096;
    const int Hq = argc > 3 ? std::atoi(argv[3]) : 128, Hkv = argc > 4 ? std::atoi(argv[4]) : 8;
    const int iters = argc > 5 ? std::atoi(argv[5]) : 50;
    if (B <= 0 || S <= 0 || Hq <= 0 || Hkv <= 0 || Hq % Hkv != 0 || iters <= 0) {
        std::fprintf(stderr, "usage: bench_flash_gqa [B S Hq Hkv iters]\n");
        return 1;
    }
    int bad = run_decode(B, S, Hq, Hkv, iters);
    // upstream's prefill benchmark shape (one sequence of 4096 tokens, 16 query heads on one kv head), both masks
    bad |= run_prefill(1, 4096, 16, 1, false, iters, 16);
    bad |= run_prefill(1, 4096, 16, 1, true, iters, 16);
    int detail[4];
    const int st = cllo_device_status(detail);
    std::printf("device status: %s; results %s\n", cllo_status_string(st), bad ? "OUT OF TOLERANCE" : "within tolerance");
    cllo_shutdown();
    return (st == CLLO_OK && !bad) ? 0 : 2;
}
