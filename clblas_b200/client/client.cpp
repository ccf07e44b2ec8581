// Native benchmark client for the B200 level-3 path, with the command line and the output lines
// of the reference's client (src/client/client.cpp:81-111 options, :574-592 timing loop and the
// two "BLAS kernel execution ..." lines; GFLOP/s formulas src/client/clfunc_xgemm.hpp:95-98 and
// src/client/clfunc_xtrsm.hpp:70-80; host data from srand(10), clfunc_xgemm.hpp:364-393; TRSM uses
// a diagonal A, clfunc_xtrsm.hpp:243-279).  Timing uses CUDA events around `apiCallCount`
// back-to-back enqueued calls, `profile` samples, samples further than 3 sigma from the mean
// pruned (src/client/statisticalTimer.cpp:267-289).  It also prints one CSV row in the schema of
// the reference's published sweeps (doc/performance/**.csv header).
//
//   clblas_b200_client -f gemm -r d -m 8192 -n 8192 -k 8192 --transposeA 1 -p 10 --apiCallCount 3
//
// --numQueues q   q command queues per call (src/client/client.cpp:108): streams on device 0, or spread over the
//                 devices of --devices d; GEMM cuts N into one stripe per queue.
// --roundtrip     the timed region includes writing the inputs from host memory and reading the result back
//                 (src/client/client.cpp:109, :522-556): the call goes through the host-matrix entry points.
// --validate      gemm, trsm, trmm: a sample of the result against a double-precision host evaluation (:111).
// --gpus g        one host thread per GPU, every thread calling the sharded entry point on its column block
//                 (GEMM column-major: columns of op(B) and C; TRSM Left: right-hand-side columns); the matrix that
//                 is shared is broadcast from GPU 0 inside every call.  Prints the whole-job GFLOP/s.
#include <cuda_runtime.h>

#include <algorithm>
#include <atomic>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <thread>
#include <vector>

#include "../../include/clblas_b200.h"

#define CUDA_OK(x)                                                                              \
    do {                                                                                        \
        cudaError_t e_ = (x);                                                                   \
        if (e_ != cudaSuccess) {                                                                \
            std::fprintf(stderr, "CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); \
            std::exit(2);                                                                       \
        }                                                                                       \
    } while (0)

struct Options {
    size_t M = 128, N = 128, K = 128, lda = 0, ldb = 0, ldc = 0, offA = 0, offB = 0, offC = 0;
    double alpha = 1.0, beta = 1.0;
    int order = 1, transA = 0, transB = 0, side = 0, uplo = 0, diag = 0, validate = 0, path = 0;
    int roundtrip = 0, gpus = 1, devices = 1;
    unsigned profile = 20, apiCallCount = 10, numQueues = 1;
    std::string function = "gemm", precision = "s";
};

static void usage()
{
    std::puts("clblas_b200_client options (same meaning as the clBLAS client):\n"
              "  -m/--sizem -n/--sizen -k/--sizek  --lda --ldb --ldc  --offA --offBX --offCY\n"
              "  --alpha --beta  -o/--order (0 row, 1 column)  --transposeA --transposeB (0/1/2)\n"
              "  -f/--function gemm|trsm|trmm|syrk|syr2k|symm  -r/--precision s|d|c|z  --side --uplo --diag\n"
              "  -p/--profile samples (20)  --apiCallCount calls per sample (10)  -v/--validate 0|1\n"
              "  --numQueues q [--devices d]  --roundtrip  --gpus g (sharded run, one thread per GPU)");
}

static bool parse(int argc, char** argv, Options& o)
{
    for (int i = 1; i < argc; i++) {
        std::string a = argv[i];
        auto val = [&]() -> const char* { return (i + 1 < argc) ? argv[++i] : "0"; };
        if (a == "-h" || a == "--help") return false;
        else if (a == "-m" || a == "--sizem") o.M = std::strtoull(val(), nullptr, 10);
        else if (a == "-n" || a == "--sizen") o.N = std::strtoull(val(), nullptr, 10);
        else if (a == "-k" || a == "--sizek") o.K = std::strtoull(val(), nullptr, 10);
        else if (a == "--lda") o.lda = std::strtoull(val(), nullptr, 10);
        else if (a == "--ldb") o.ldb = std::strtoull(val(), nullptr, 10);
        else if (a == "--ldc") o.ldc = std::strtoull(val(), nullptr, 10);
        else if (a == "--offA") o.offA = std::strtoull(val(), nullptr, 10);
        else if (a == "--offBX") o.offB = std::strtoull(val(), nullptr, 10);
        else if (a == "--offCY") o.offC = std::strtoull(val(), nullptr, 10);
        else if (a == "--alpha") o.alpha = std::atof(val());
        else if (a == "--beta") o.beta = std::atof(val());
        else if (a == "-o" || a == "--order") o.order = std::atoi(val());
        else if (a == "--transposeA") o.transA = std::atoi(val());
        else if (a == "--transposeB") o.transB = std::atoi(val());
        else if (a == "-f" || a == "--function") o.function = val();
        else if (a == "-r" || a == "--precision") o.precision = val();
        else if (a == "--side") o.side = std::atoi(val());
        else if (a == "--uplo") o.uplo = std::atoi(val());
        else if (a == "--diag") o.diag = std::atoi(val());
        else if (a == "-p" || a == "--profile") o.profile = (unsigned)std::atoi(val());
        else if (a == "--apiCallCount") o.apiCallCount = (unsigned)std::atoi(val());
        else if (a == "-v" || a == "--validate") o.validate = std::atoi(val());
        else if (a == "--path") o.path = std::atoi(val());      // clblasB200SetGemmPath (kernel family override)
        else if (a == "--numQueues") o.numQueues = (unsigned)std::max(1, std::atoi(val()));
        else if (a == "--devices") o.devices = std::max(1, std::atoi(val()));
        else if (a == "--roundtrip") o.roundtrip = 1;
        else if (a == "--gpus") o.gpus = std::max(1, std::atoi(val()));
        else { std::fprintf(stderr, "unknown option %s\n", a.c_str()); return false; }
    }
    return true;
}

// rows x cols of op(X) as stored: contiguous extent and number of strides
static void stored(int order, int trans, size_t rows, size_t cols, size_t& inner, size_t& outer)
{
    const bool tra = (order == 1 && trans == 0) || (order == 0 && trans != 0);
    inner = tra ? rows : cols;
    outer = tra ? cols : rows;
}

template <typename T>
static int run(const Options& o)
{
    const bool syr2k = o.function == "syr2k", symm = o.function == "symm";
    const bool gemm = o.function == "gemm" || syr2k || symm, syrk = o.function == "syrk";
    size_t ai, ao, bi, bo, ci = 0, co = 0;
    const size_t tri = o.side == 0 ? o.M : o.N;
    if (syr2k) {
        // A and B are N x K (K x N when transposed), C is N x N
        stored(o.order, o.transA, o.N, o.K, ai, ao);
        stored(o.order, o.transA, o.N, o.K, bi, bo);
        stored(o.order, 0, o.N, o.N, ci, co);
    } else if (symm) {
        ai = ao = tri;
        stored(o.order, 0, o.M, o.N, bi, bo);
        stored(o.order, 0, o.M, o.N, ci, co);
    } else if (gemm) {
        stored(o.order, o.transA, o.M, o.K, ai, ao);
        stored(o.order, o.transB, o.K, o.N, bi, bo);
        stored(o.order, 0, o.M, o.N, ci, co);
    } else if (syrk) {
        // A is N x K (K x N when transposed); the "B" buffer holds the N x N matrix C
        stored(o.order, o.transA, o.N, o.K, ai, ao);
        stored(o.order, 0, o.N, o.N, bi, bo);
    } else {
        ai = ao = tri;
        stored(o.order, 0, o.M, o.N, bi, bo);
    }
    const size_t lda = o.lda ? o.lda : ai, ldb = o.ldb ? o.ldb : bi, ldc = o.ldc ? o.ldc : ci;
    const size_t na = o.offA + (ao - 1) * lda + ai, nb = o.offB + (bo - 1) * ldb + bi;
    const size_t nc = gemm ? o.offC + (co - 1) * ldc + ci : 0;

    std::vector<T> hA(na), hB(nb), hC(nc ? nc : 1);
    std::srand(10);
    auto rnd = [] { return (T)((std::rand() % 20) - 10) / (T)10; };
    if (gemm || syrk) {
        for (auto& v : hA) v = rnd();
        for (auto& v : hB) v = rnd();
        for (auto& v : hC) v = rnd();
    } else {
        std::fill(hA.begin(), hA.end(), (T)0);
        for (size_t i = 0; i < tri; i++) hA[o.offA + i + i * lda] = (T)(1 + (std::rand() % 4));   // diagonal A, as the reference client
        for (auto& v : hB) v = rnd();
    }

    if (o.roundtrip) {
        // pinned host memory, as the copies of a roundtrip run want it
        CUDA_OK(cudaHostRegister(hA.data(), hA.size() * sizeof(T), cudaHostRegisterDefault));
        CUDA_OK(cudaHostRegister(hB.data(), hB.size() * sizeof(T), cudaHostRegisterDefault));
        CUDA_OK(cudaHostRegister(hC.data(), hC.size() * sizeof(T), cudaHostRegisterDefault));
    }
    T *dA, *dB, *dC = nullptr;
    CUDA_OK(cudaMalloc(&dA, na * sizeof(T)));
    CUDA_OK(cudaMalloc(&dB, nb * sizeof(T)));
    if (gemm) CUDA_OK(cudaMalloc(&dC, nc * sizeof(T)));
    CUDA_OK(cudaMemcpy(dA, hA.data(), na * sizeof(T), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dB, hB.data(), nb * sizeof(T), cudaMemcpyHostToDevice));
    if (gemm) CUDA_OK(cudaMemcpy(dC, hC.data(), nc * sizeof(T), cudaMemcpyHostToDevice));

    // queue 0 is the timing stream; further queues (--numQueues) live on device q % devices
    std::vector<cudaStream_t> streams(o.numQueues);
    std::vector<cudaEvent_t> done(o.numQueues);
    for (unsigned i = 0; i < o.numQueues; i++) {
        CUDA_OK(cudaSetDevice((int)(i % (unsigned)o.devices)));
        CUDA_OK(cudaStreamCreate(&streams[i]));
        CUDA_OK(cudaEventCreateWithFlags(&done[i], cudaEventDisableTiming));
    }
    CUDA_OK(cudaSetDevice(0));
    cudaStream_t stream = streams[0];
    clblasQueue* qs = reinterpret_cast<clblasQueue*>(streams.data());
    clblasEvent* evs = reinterpret_cast<clblasEvent*>(done.data());
    clblasQueue q = qs[0];
    const unsigned nq = o.numQueues;
    if (clblasSetup() != clblasSuccess) { std::fprintf(stderr, "clblasSetup failed\n"); return 2; }
    clblasB200SetGemmPath(o.path);
    const bool plain_gemm = o.function == "gemm";
    // after a call over several queues, queue 0 (the timing stream) waits for the others' events
    auto join = [&]() { for (unsigned i = 1; i < nq; i++) CUDA_OK(cudaStreamWaitEvent(stream, done[i], 0)); };

    auto call = [&]() -> clblasStatus {
        if (o.roundtrip && (plain_gemm || o.function == "trsm")) {
            // inputs from host memory, result back to host memory, inside the call
            if (plain_gemm) {
                if (sizeof(T) == 4)
                    return clblasB200SgemmHost((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                                               (float)o.alpha, hA.data(), o.offA, lda, hB.data(), o.offB, ldb, (float)o.beta, hC.data(), o.offC, ldc,
                                               1, &q, 0, nullptr, nullptr);
                return clblasB200DgemmHost((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                                           o.alpha, hA.data(), o.offA, lda, hB.data(), o.offB, ldb, o.beta, hC.data(), o.offC, ldc,
                                           1, &q, 0, nullptr, nullptr);
            }
            if (sizeof(T) == 4)
                return clblasB200StrsmHost((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                                           o.M, o.N, (float)o.alpha, hA.data(), o.offA, lda, hB.data(), o.offB, ldb, 1, &q, 0, nullptr, nullptr);
            return clblasB200DtrsmHost((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                                       o.M, o.N, o.alpha, hA.data(), o.offA, lda, hB.data(), o.offB, ldb, 1, &q, 0, nullptr, nullptr);
        }
        if (plain_gemm && nq > 1) {
            clblasStatus r;
            if (sizeof(T) == 4)
                r = clblasSgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                                (float)o.alpha, dA, o.offA, lda, dB, o.offB, ldb, (float)o.beta, dC, o.offC, ldc, nq, qs, 0, nullptr, evs);
            else
                r = clblasDgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                                o.alpha, dA, o.offA, lda, dB, o.offB, ldb, o.beta, dC, o.offC, ldc, nq, qs, 0, nullptr, evs);
            join();
            return r;
        }
        if (syr2k) {
            if (sizeof(T) == 4)
                return clblasSsyr2k((clblasOrder)o.order, (clblasUplo)o.uplo, (clblasTranspose)o.transA, o.N, o.K, (float)o.alpha,
                                    dA, o.offA, lda, dB, o.offB, ldb, (float)o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
            return clblasDsyr2k((clblasOrder)o.order, (clblasUplo)o.uplo, (clblasTranspose)o.transA, o.N, o.K, o.alpha,
                                dA, o.offA, lda, dB, o.offB, ldb, o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
        }
        if (symm) {
            if (sizeof(T) == 4)
                return clblasSsymm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, o.M, o.N, (float)o.alpha,
                                   dA, o.offA, lda, dB, o.offB, ldb, (float)o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
            return clblasDsymm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, o.M, o.N, o.alpha,
                               dA, o.offA, lda, dB, o.offB, ldb, o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
        }
        if (gemm) {
            if (sizeof(T) == 4)
                return clblasSgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                                   (float)o.alpha, dA, o.offA, lda, dB, o.offB, ldb, (float)o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
            return clblasDgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                               o.alpha, dA, o.offA, lda, dB, o.offB, ldb, o.beta, dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
        }
        if (syrk) {
            if (sizeof(T) == 4)
                return clblasSsyrk((clblasOrder)o.order, (clblasUplo)o.uplo, (clblasTranspose)o.transA, o.N, o.K, (float)o.alpha,
                                   dA, o.offA, lda, (float)o.beta, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
            return clblasDsyrk((clblasOrder)o.order, (clblasUplo)o.uplo, (clblasTranspose)o.transA, o.N, o.K, o.alpha,
                               dA, o.offA, lda, o.beta, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
        }
        if (o.function == "trmm") {
            if (sizeof(T) == 4)
                return clblasStrmm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                                   o.M, o.N, (float)o.alpha, dA, o.offA, lda, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
            return clblasDtrmm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                               o.M, o.N, o.alpha, dA, o.offA, lda, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
        }
        if (sizeof(T) == 4)
            return clblasStrsm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                               o.M, o.N, (float)o.alpha, dA, o.offA, lda, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
        return clblasDtrsm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag,
                           o.M, o.N, o.alpha, dA, o.offA, lda, dB, o.offB, ldb, 1, &q, 0, nullptr, nullptr);
    };

    clblasStatus st = call();          // untimed warm-up call (src/client/client.cpp:497)
    if (st != clblasSuccess) { std::fprintf(stderr, "call failed with status %d\n", (int)st); return 3; }
    CUDA_OK(cudaStreamSynchronize(stream));

    if (o.validate && gemm && !syr2k && !symm) {
        // spot check of 64 entries against a double-precision host evaluation of the same inputs
        std::vector<T> out(nc);
        CUDA_OK(cudaMemcpy(out.data(), dC, nc * sizeof(T), cudaMemcpyDeviceToHost));
        double worst = 0;
        for (int t = 0; t < 64; t++) {
            const size_t i = std::rand() % o.M, j = std::rand() % o.N;
            double acc = 0, mag = 0;
            for (size_t k = 0; k < o.K; k++) {
                const bool traA = (o.order == 1 && o.transA == 0) || (o.order == 0 && o.transA != 0);
                const bool traB = (o.order == 1 && o.transB == 0) || (o.order == 0 && o.transB != 0);
                const double a = hA[o.offA + (traA ? i + k * lda : i * lda + k)];
                const double b = hB[o.offB + (traB ? k + j * ldb : k * ldb + j)];
                acc += a * b;
                mag += std::fabs(a * b);
            }
            const size_t cidx = o.offC + (o.order == 1 ? i + j * ldc : i * ldc + j);
            const double want = o.alpha * acc + o.beta * hC[cidx];
            const double den = std::fabs(o.alpha) * mag + std::fabs(o.beta * hC[cidx]) + 1e-300;
            worst = std::max(worst, std::fabs((double)out[cidx] - want) / den);
        }
        const double u = sizeof(T) == 4 ? std::ldexp(1.0, -24) : std::ldexp(1.0, -53);
        std::printf("validation: max scaled error %.3e (bound 4*K*u = %.3e) %s\n", worst, 4.0 * o.K * u,
                    worst <= 4.0 * o.K * u ? "PASS" : "FAIL");
    }

    if (o.validate && !o.roundtrip && (o.function == "trsm" || o.function == "trmm")) {
        // eight columns (Left) or rows (Right) of the result against a double-precision host evaluation with the same
        // A: trsm by its residual alpha*B - op(A)*X, trmm by the product itself; both relative to |op(A)||.| + |.|
        std::vector<T> out(nb);
        CUDA_OK(cudaMemcpy(out.data(), dB, nb * sizeof(T), cudaMemcpyDeviceToHost));
        const bool left = o.side == 0, colmaj = o.order == 1, trsm = o.function == "trsm";
        auto a_at = [&](size_t i, size_t j) -> double {         // op(A)(i, j) of the triangular matrix, zero outside the triangle
            size_t r = o.transA ? j : i, c = o.transA ? i : j;
            const bool inside = o.uplo == 0 ? r <= c : r >= c;  // clblasUpper = 0
            if (!inside) return 0.0;
            if (r == c && o.diag == 0) return 1.0;              // clblasUnit = 0
            return (double)hA[o.offA + (colmaj ? r + c * lda : r * lda + c)];
        };
        auto b_idx = [&](size_t i, size_t j) { return o.offB + (colmaj ? i + j * ldb : i * ldb + j); };
        double worst = 0;
        const size_t other = left ? o.N : o.M;
        for (int t = 0; t < 8; t++) {
            const size_t sel = (size_t)std::rand() % other;
            for (size_t i = 0; i < tri; i++) {
                double acc = 0, mag = 0;
                for (size_t k = 0; k < tri; k++) {
                    const double a = left ? a_at(i, k) : a_at(k, i);
                    const double x = left ? (double)(trsm ? out : hB)[b_idx(k, sel)] : (double)(trsm ? out : hB)[b_idx(sel, k)];
                    acc += a * x;
                    mag += std::fabs(a * x);
                }
                const size_t bi_ = left ? b_idx(i, sel) : b_idx(sel, i);
                const double rhs = trsm ? o.alpha * (double)hB[bi_] : (double)out[bi_];
                const double lhs = trsm ? acc : o.alpha * acc;
                worst = std::max(worst, std::fabs(rhs - lhs) / (std::fabs(trsm ? 1.0 : o.alpha) * mag + std::fabs(rhs) + 1e-300));
            }
        }
        const double u = sizeof(T) == 4 ? std::ldexp(1.0, -24) : std::ldexp(1.0, -53);
        std::printf("validation: max scaled error %.3e (bound 4*n*u = %.3e) %s\n", worst, 4.0 * tri * u, worst <= 4.0 * tri * u ? "PASS" : "FAIL");
    }

    cudaEvent_t e0, e1;
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
    std::vector<double> ns;
    for (unsigned s = 0; s < o.profile; s++) {
        CUDA_OK(cudaEventRecord(e0, stream));
        for (unsigned c = 0; c < o.apiCallCount; c++) st = call();
        CUDA_OK(cudaEventRecord(e1, stream));
        CUDA_OK(cudaEventSynchronize(e1));
        float ms = 0;
        CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
        ns.push_back((double)ms * 1e6);
    }
    if (st != clblasSuccess) { std::fprintf(stderr, "call failed with status %d\n", (int)st); return 3; }

    auto mean_of = [](const std::vector<double>& v) { double s = 0; for (double x : v) s += x; return s / v.size(); };
    double mean = mean_of(ns), var = 0;
    for (double x : ns) var += (x - mean) * (x - mean);
    const double sd = std::sqrt(var / ns.size());
    std::vector<double> kept;
    for (double x : ns) if (std::fabs(x - mean) <= 3.0 * sd || sd == 0) kept.push_back(x);
    std::clog << "\tStatisticalTimer:: Pruning " << ns.size() - kept.size() << " samples from clfunc" << std::endl;
    mean = mean_of(kept.empty() ? ns : kept);
    const double per_call_ns = mean / o.apiCallCount;
    double flop;
    std::string formula;
    if (syr2k) { flop = 2.0 * o.N * (o.N + 1) * o.K; formula = "2*N*(N+1)*K/time"; }
    else if (symm) { flop = 2.0 * o.M * o.N * (o.side == 0 ? o.M : o.N); formula = o.side == 0 ? "2*M*M*N/time" : "2*M*N*N/time"; }
    else if (gemm) { flop = 2.0 * o.M * o.N * o.K; formula = "2.0*M*N*K/time"; }
    else if (syrk) { flop = (double)o.N * (o.N + 1) * o.K; formula = "N*(N+1)*K/time"; }
    else if (o.side == 0) { flop = (double)o.M * (o.M + 1) * o.N; formula = "M*(M+1)*N/time"; }
    else { flop = (double)o.M * (o.N + 1) * o.N; formula = "M*(N+1)*N/time"; }
    const double gflops = flop / per_call_ns;
    std::printf("BLAS kernel execution time < ns >: %.0f\n", per_call_ns);
    std::printf("BLAS kernel execution Gflops < %s >: %.2f\n", formula.c_str(), gflops);
    cudaDeviceProp prop;
    CUDA_OK(cudaGetDeviceProperties(&prop, 0));
    std::printf("m,n,k,lda,ldb,ldc,offa,offb,offc,alpha,beta,order,transa,transb,side,uplo,diag,function,device,library,label,GFLOPS\n");
    std::printf("%zu,%zu,%zu,%zu,%zu,%zu,%zu,%zu,%zu,%g,%g,%s,%s,%s,%s,%s,%s,%s%s,%s,clblas_b200,%s,%.2f\n", o.M, o.N, o.K, lda, ldb, ldc,
                o.offA, o.offB, o.offC, o.alpha, o.beta, o.order ? "column" : "row", o.transA ? "trans" : "none",
                o.transB ? "trans" : "none", o.side ? "right" : "left", o.uplo ? "lower" : "upper", o.diag ? "nonunit" : "unit",
                o.precision.c_str(), o.function.c_str(), prop.name, clblasB200LastGemmKernel(), gflops);

    cudaFree(dA); cudaFree(dB); if (dC) cudaFree(dC);
    for (auto s_ : streams) cudaStreamDestroy(s_);
    if (o.roundtrip) { cudaHostUnregister(hA.data()); cudaHostUnregister(hB.data()); cudaHostUnregister(hC.data()); }
    clblasTeardown();
    return 0;
}

// --gpus g: the sharded entry points, one host thread per GPU.  GEMM column-major (columns of op(B) and C split, A
// broadcast from GPU 0 inside every call) and TRSM column-major Left (right-hand-side columns split).  Time is taken on
// every GPU with CUDA events around the same calls, between two host-side barriers; the slowest GPU counts.
template <typename T>
static int run_sharded(const Options& o)
{
    const bool trsm = o.function == "trsm";
    if (o.order != 1 || (trsm && o.side != 0) || (!trsm && o.function != "gemm")) {
        std::fprintf(stderr, "--gpus: gemm (column-major) or trsm (column-major, Left)\n");
        return 1;
    }
    int ndev = 0;
    CUDA_OK(cudaGetDeviceCount(&ndev));
    const int G = o.gpus;
    if (G > ndev) { std::fprintf(stderr, "--gpus %d: only %d device(s)\n", G, ndev); return 1; }
    if (clblasSetup() != clblasSuccess) return 2;
    std::vector<clblasB200Comm> comms(G);
    if (clblasB200CommInitAll(comms.data(), G, nullptr) != clblasSuccess) { std::fprintf(stderr, "communicator set-up failed (NCCL available?)\n"); return 2; }
    std::vector<size_t> bounds(G + 1);
    clblasB200PlanShards(o.N, (unsigned)G, 128, bounds.data());
    std::vector<double> ms(G, 0.0);
    std::vector<int> status(G, 0);
    // a small sense-reversing barrier for the host threads
    struct Barrier { std::atomic<int> count{0}, phase{0}; int n; void wait() { const int p = phase.load(); if (count.fetch_add(1) + 1 == n) { count.store(0); phase.fetch_add(1); } else while (phase.load() == p) std::this_thread::yield(); } } bar;
    bar.n = G;
    auto worker = [&](int r) {
        CUDA_OK(cudaSetDevice(r));
        const size_t nl = bounds[r + 1] - bounds[r];
        const size_t am = trsm ? o.M : (o.transA ? o.K : o.M), an = trsm ? o.M : (o.transA ? o.M : o.K);      // A as stored
        const size_t lda = am, ldb = trsm ? o.M : (o.transB ? std::max<size_t>(nl, 1) : o.K), ldc = o.M;
        const size_t nbel = trsm ? o.M * std::max<size_t>(nl, 1) : (o.transB ? ldb * o.K : o.K * std::max<size_t>(nl, 1));
        // Only the root holds A on the host; a generator of its own per thread (std::rand serialises the threads on a lock,
        // which made the set-up of a 32768^2 problem take minutes).
        std::vector<T> hA(r == 0 ? am * an : 0), hB(nbel);
        unsigned long long lcg = 0x9E3779B97F4A7C15ull * (unsigned long long)(11 + r);
        auto next = [&lcg] { lcg = lcg * 6364136223846793005ull + 1442695040888963407ull; return (unsigned)(lcg >> 40); };
        auto rnd = [&next] { return (T)((int)(next() % 20) - 10) / (T)10; };
        if (r == 0) {
            if (trsm) { std::fill(hA.begin(), hA.end(), (T)0); for (size_t i = 0; i < o.M; i++) hA[i + i * lda] = (T)(1 + (next() % 4)); }
            else for (auto& v : hA) v = rnd();
        }
        for (auto& v : hB) v = rnd();
        T *dA, *dB, *dC = nullptr;
        CUDA_OK(cudaMalloc(&dA, am * an * sizeof(T)));
        CUDA_OK(cudaMalloc(&dB, hB.size() * sizeof(T)));
        if (r == 0) CUDA_OK(cudaMemcpy(dA, hA.data(), hA.size() * sizeof(T), cudaMemcpyHostToDevice));
        else CUDA_OK(cudaMemset(dA, 0xff, am * an * sizeof(T)));            // the broadcast has to fill it
        CUDA_OK(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(T), cudaMemcpyHostToDevice));
        if (!trsm) { CUDA_OK(cudaMalloc(&dC, o.M * std::max<size_t>(nl, 1) * sizeof(T))); CUDA_OK(cudaMemset(dC, 0, o.M * std::max<size_t>(nl, 1) * sizeof(T))); }
        cudaStream_t stream;
        CUDA_OK(cudaStreamCreate(&stream));
        clblasQueue q = reinterpret_cast<clblasQueue>(stream);
        auto call = [&]() -> clblasStatus {
            if (trsm) {
                if (sizeof(T) == 4)
                    return clblasB200StrsmSharded(clblasColumnMajor, clblasLeft, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag, o.M, nl,
                                                  (float)o.alpha, dA, 0, lda, dB, 0, ldb, comms[r], 0, 1, &q, 0, nullptr, nullptr);
                return clblasB200DtrsmSharded(clblasColumnMajor, clblasLeft, (clblasUplo)o.uplo, (clblasTranspose)o.transA, (clblasDiag)o.diag, o.M, nl,
                                              o.alpha, dA, 0, lda, dB, 0, ldb, comms[r], 0, 1, &q, 0, nullptr, nullptr);
            }
            if (sizeof(T) == 4)
                return clblasB200SgemmSharded(clblasColumnMajor, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, nl, o.K, (float)o.alpha,
                                              dA, 0, lda, dB, 0, ldb, (float)o.beta, dC, 0, ldc, comms[r], 0, 1, &q, 0, nullptr, nullptr);
            return clblasB200DgemmSharded(clblasColumnMajor, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, nl, o.K, o.alpha,
                                          dA, 0, lda, dB, 0, ldb, o.beta, dC, 0, ldc, comms[r], 0, 1, &q, 0, nullptr, nullptr);
        };
        clblasStatus st = call();
        CUDA_OK(cudaStreamSynchronize(stream));
        cudaEvent_t e0, e1;
        CUDA_OK(cudaEventCreate(&e0));
        CUDA_OK(cudaEventCreate(&e1));
        bar.wait();
        CUDA_OK(cudaEventRecord(e0, stream));
        for (unsigned sI = 0; sI < o.profile * o.apiCallCount && st == clblasSuccess; sI++) st = call();
        CUDA_OK(cudaEventRecord(e1, stream));
        CUDA_OK(cudaEventSynchronize(e1));
        bar.wait();
        float t = 0;
        CUDA_OK(cudaEventElapsedTime(&t, e0, e1));
        ms[r] = t;
        status[r] = (int)st;
        cudaFree(dA); cudaFree(dB); if (dC) cudaFree(dC);
        cudaStreamDestroy(stream);
    };
    std::vector<std::thread> th;
    for (int r = 0; r < G; r++) th.emplace_back(worker, r);
    for (auto& t : th) t.join();
    for (int r = 0; r < G; r++) if (status[r] != 0) { std::fprintf(stderr, "rank %d: status %d\n", r, status[r]); return 3; }
    const double worst_ms = *std::max_element(ms.begin(), ms.end());
    const double per_call_ns = worst_ms * 1e6 / ((double)o.profile * o.apiCallCount);
    const double flop = trsm ? (double)o.M * (o.M + 1) * o.N : 2.0 * o.M * o.N * o.K;
    std::printf("BLAS kernel execution time < ns >: %.0f\n", per_call_ns);
    std::printf("BLAS kernel execution Gflops < %s, %d GPUs >: %.2f\n", trsm ? "M*(M+1)*N/time" : "2.0*M*N*K/time", G, flop / per_call_ns);
    for (auto c : comms) clblasB200CommDestroy(c);
    clblasTeardown();
    return 0;
}

// Complex GEMM (-r c | z): interleaved (re, im) matrices, flops = 8*M*N*K as the reference client counts
// them (src/client/clfunc_xgemm.hpp:97 with the complex factor 4).
template <typename R>
static int run_complex(const Options& o)
{
    const bool trsm = o.function == "trsm";
    const size_t tri = o.side == 0 ? o.M : o.N;
    size_t ai, ao, bi, bo, ci, co;
    if (trsm) {
        ai = ao = tri;
        stored(o.order, 0, o.M, o.N, bi, bo);
    } else {
        stored(o.order, o.transA, o.M, o.K, ai, ao);
        stored(o.order, o.transB, o.K, o.N, bi, bo);
    }
    stored(o.order, 0, o.M, o.N, ci, co);
    const size_t lda = o.lda ? o.lda : ai, ldb = o.ldb ? o.ldb : bi, ldc = o.ldc ? o.ldc : ci;
    const size_t na = o.offA + (ao - 1) * lda + ai, nb = o.offB + (bo - 1) * ldb + bi, nc = o.offC + (co - 1) * ldc + ci;
    std::vector<R> hA(2 * na), hB(2 * nb), hC(2 * nc);
    std::srand(10);
    auto rnd = [] { return (R)((std::rand() % 20) - 10) / (R)10; };
    for (auto& v : hA) v = rnd();
    for (auto& v : hB) v = rnd();
    for (auto& v : hC) v = rnd();
    if (trsm) {     // diagonal A, as the reference client: repeated solves in place stay bounded
        std::fill(hA.begin(), hA.end(), (R)0);
        for (size_t i = 0; i < tri; i++) hA[2 * (o.offA + i + i * lda)] = (R)1;
    }
    R *dA, *dB, *dC;
    CUDA_OK(cudaMalloc(&dA, hA.size() * sizeof(R)));
    CUDA_OK(cudaMalloc(&dB, hB.size() * sizeof(R)));
    CUDA_OK(cudaMalloc(&dC, hC.size() * sizeof(R)));
    CUDA_OK(cudaMemcpy(dA, hA.data(), hA.size() * sizeof(R), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dB, hB.data(), hB.size() * sizeof(R), cudaMemcpyHostToDevice));
    CUDA_OK(cudaMemcpy(dC, hC.data(), hC.size() * sizeof(R), cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CUDA_OK(cudaStreamCreate(&stream));
    clblasQueue q = reinterpret_cast<clblasQueue>(stream);
    if (clblasSetup() != clblasSuccess) { std::fprintf(stderr, "clblasSetup failed\n"); return 2; }
    clblasB200SetGemmPath(o.path);
    auto call = [&]() -> clblasStatus {
        if (trsm) {
            if (sizeof(R) == 4)
                return clblasCtrsm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA,
                                   (clblasDiag)o.diag, o.M, o.N, floatComplex((float)o.alpha, 0.f), dA, o.offA, lda, dB, o.offB, ldb,
                                   1, &q, 0, nullptr, nullptr);
            return clblasZtrsm((clblasOrder)o.order, (clblasSide)o.side, (clblasUplo)o.uplo, (clblasTranspose)o.transA,
                               (clblasDiag)o.diag, o.M, o.N, doubleComplex(o.alpha, 0.0), dA, o.offA, lda, dB, o.offB, ldb,
                               1, &q, 0, nullptr, nullptr);
        }
        if (sizeof(R) == 4)
            return clblasCgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                               floatComplex((float)o.alpha, 0.f), dA, o.offA, lda, dB, o.offB, ldb, floatComplex((float)o.beta, 0.f),
                               dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
        return clblasZgemm((clblasOrder)o.order, (clblasTranspose)o.transA, (clblasTranspose)o.transB, o.M, o.N, o.K,
                           doubleComplex(o.alpha, 0.0), dA, o.offA, lda, dB, o.offB, ldb, doubleComplex(o.beta, 0.0),
                           dC, o.offC, ldc, 1, &q, 0, nullptr, nullptr);
    };
    clblasStatus st = call();
    if (st != clblasSuccess) { std::fprintf(stderr, "call failed with status %d\n", (int)st); return 3; }
    CUDA_OK(cudaStreamSynchronize(stream));
    cudaEvent_t e0, e1;
    CUDA_OK(cudaEventCreate(&e0));
    CUDA_OK(cudaEventCreate(&e1));
    double total_ms = 0;
    for (unsigned s = 0; s < o.profile; s++) {
        CUDA_OK(cudaEventRecord(e0, stream));
        for (unsigned c = 0; c < o.apiCallCount; c++) st = call();
        CUDA_OK(cudaEventRecord(e1, stream));
        CUDA_OK(cudaEventSynchronize(e1));
        float ms = 0;
        CUDA_OK(cudaEventElapsedTime(&ms, e0, e1));
        total_ms += ms;
    }
    if (st != clblasSuccess) { std::fprintf(stderr, "call failed with status %d\n", (int)st); return 3; }
    const double per_call_ns = total_ms * 1e6 / ((double)o.profile * o.apiCallCount);
    std::printf("BLAS kernel execution time < ns >: %.0f\n", per_call_ns);
    if (trsm)
        std::printf("BLAS kernel execution Gflops < 4*M*(M+1)*N/time >: %.2f\n",
                    4.0 * (o.side == 0 ? (double)o.M * (o.M + 1) * o.N : (double)o.M * (o.N + 1) * o.N) / per_call_ns);
    else
        std::printf("BLAS kernel execution Gflops < 8.0*M*N*K/time >: %.2f\n", 8.0 * o.M * o.N * o.K / per_call_ns);
    cudaFree(dA); cudaFree(dB); cudaFree(dC);
    cudaStreamDestroy(stream);
    clblasTeardown();
    return 0;
}

int main(int argc, char** argv)
{
    Options o;
    if (!parse(argc, argv, o)) { usage(); return 1; }
    if (o.function != "gemm" && o.function != "trsm" && o.function != "trmm" && o.function != "syrk" && o.function != "syr2k" && o.function != "symm") {
        std::fprintf(stderr, "function must be gemm, trsm, trmm, syrk, syr2k or symm\n");
        return 1;
    }
    if ((o.precision == "c" || o.precision == "z") && o.function != "gemm" && o.function != "trsm") {
        std::fprintf(stderr, "complex precisions are available for gemm and trsm\n");
        return 1;
    }
    if (o.gpus > 1) {
        if (o.precision == "s") return run_sharded<float>(o);
        if (o.precision == "d") return run_sharded<double>(o);
        std::fprintf(stderr, "--gpus: precision s or d\n");
        return 1;
    }
    if (o.precision == "c") return run_complex<float>(o);
    if (o.precision == "z") return run_complex<double>(o);
    if (o.precision == "s") return run<float>(o);
    if (o.precision == "d") return run<double>(o);
    std::fprintf(stderr, "precision must be s, d, c or z\n");
    return 1;
}
