// Issue-rate probes: what the FP32 FMA pipe and the FP64 tensor-core (mma.sync m8n8k4) pipe of the
// current device deliver when nothing but independent FMAs / MMAs is issued from registers.
// The benchmark uses them as the live roofline denominators for SGEMM and DGEMM/DTRSM (the
// reference publishes its GEMM numbers against such a peak line too, doc/performance/
// clBLAS_2.6.0/S9150/peak_sp.csv and peak_dp.csv).
#include "common.h"

namespace cb200 {

namespace {

template <int ILP>
__global__ void __launch_bounds__(256) ffma_probe(float* out, int iters, float a, float b)
{
    float acc[ILP];
#pragma unroll
    for (int i = 0; i < ILP; i++) acc[i] = threadIdx.x * 0.001f + i;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < ILP; i++) acc[i] = fmaf(acc[i], a, b);
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < ILP; i++) s += acc[i];
    if (s == 12345.678f) out[0] = s;
}

template <int ILP>
__global__ void __launch_bounds__(256) dmma_probe(double* out, int iters, double a, double b)
{
    double c0[ILP], c1[ILP];
#pragma unroll
    for (int i = 0; i < ILP; i++) { c0[i] = threadIdx.x * 0.001 + i; c1[i] = i; }
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int i = 0; i < ILP; i++)
            asm volatile("mma.sync.aligned.m8n8k4.row.col.f64.f64.f64.f64 {%0,%1}, {%2}, {%3}, {%0,%1};"
                         : "+d"(c0[i]), "+d"(c1[i]) : "d"(a), "d"(b));
    }
    double s = 0.0;
#pragma unroll
    for (int i = 0; i < ILP; i++) s += c0[i] + c1[i];
    if (s == 12345.678) out[0] = s;
}

}  // namespace

}  // namespace cb200

using namespace cb200;

extern "C" double clblasB200ProbePeak(int kind, double seconds)
{
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -1.0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1.0;
    void* buf = nullptr;
    if (cudaMalloc(&buf, 256) != cudaSuccess) return -1.0;
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    const int blocks = sms * 4, threads = 256;
    const int iters = kind == 0 ? 40000 : 10000;
    // flops per launch
    const double fl = kind == 0 ? 2.0 * 16 * iters * (double)threads * blocks
                                : 2.0 * 8 * 8 * 4 * 8 * iters * (double)(threads / 32) * blocks;
    auto run = [&] {
        if (kind == 0) ffma_probe<16><<<blocks, threads>>>((float*)buf, iters, 1.0001f, 0.5f);
        else dmma_probe<8><<<blocks, threads>>>((double*)buf, iters, 1.0001, 0.5);
        count_launch();
    };
    run();
    cudaDeviceSynchronize();
    double best = 0.0, spent = 0.0;
    for (int rep = 0; rep < 1000 && spent < seconds * 1e3; rep++) {
        cudaEventRecord(e0);
        run();
        cudaEventRecord(e1);
        if (cudaEventSynchronize(e1) != cudaSuccess) { best = -1.0; break; }
        float ms = 0.f;
        cudaEventElapsedTime(&ms, e0, e1);
        spent += ms;
        const double tf = fl / (ms * 1e-3) * 1e-12;
        if (tf > best) best = tf;
    }
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(buf);
    if (cudaGetLastError() != cudaSuccess) return -1.0;
    return best;
}
