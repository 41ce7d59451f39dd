// Measurement aid for the bench report, not part of the step library: the FP32 fused-multiply-add rate this GPU
// sustains from registers, the denominator of the step kernel's FP32 roofline fraction.  Every thread runs
// independent FMA chains with no memory traffic; rate = 2 x FMAs / CUDA-event time.
#include <cuda_runtime.h>
#include <cstdint>

namespace {
constexpr int kChains = 8;

__global__ void __launch_bounds__(1024) fma_chains(float* sink, int iterations, float a, float b) {
    float x[kChains];
#pragma unroll
    for (int k = 0; k < kChains; ++k) x[k] = (float)(threadIdx.x + k) * 1.0e-3f;
    for (int it = 0; it < iterations; ++it) {
#pragma unroll
        for (int rep = 0; rep < 16; ++rep)
#pragma unroll
            for (int k = 0; k < kChains; ++k) x[k] = fmaf(x[k], a, b);
    }
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < kChains; ++k) total += x[k];
    if (total == 123.456f) sink[0] = total;          // keeps the chains alive without a store in the common case
}
}  // namespace

// Runs the FMA kernel `repeats` times on `device` and reports the best rate in TFLOP/s (one FMA = 2 FLOP) and the
// duration of that launch.  Returns a cudaError_t value, 0 on success.
extern "C" int nkb_probe_fp32_peak(int device, int repeats, float* out_tflops, float* out_ms) {
    cudaError_t err = cudaSetDevice(device);
    if (err != cudaSuccess) return (int)err;
    cudaDeviceProp prop{};
    if ((err = cudaGetDeviceProperties(&prop, device)) != cudaSuccess) return (int)err;
    float* sink = nullptr;
    if ((err = cudaMalloc(&sink, sizeof(float))) != cudaSuccess) return (int)err;
    const int blocks = prop.multiProcessorCount * 2, threads = 1024, iterations = 4096;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    float best = 0.f, best_ms = 0.f;
    for (int r = 0; r < repeats + 1; ++r) {          // the first launch warms up
        cudaEventRecord(e0, 0);
        fma_chains<<<blocks, threads>>>(sink, iterations, 0.999f, 1.0e-3f);
        cudaEventRecord(e1, 0);
        if ((err = cudaEventSynchronize(e1)) != cudaSuccess) break;
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        const double flop = 2.0 * kChains * 16.0 * iterations * (double)threads * blocks;
        const float tflops = (float)(flop / (ms * 1.0e-3) / 1.0e12);
        if (r > 0 && tflops > best) { best = tflops; best_ms = ms; }
    }
    cudaEventDestroy(e0); cudaEventDestroy(e1);
    cudaFree(sink);
    if (err != cudaSuccess) return (int)err;
    *out_tflops = best; *out_ms = best_ms;
    return 0;
}
