// A C++ consumer of include/fnx_b200.h: compiled against the header and linked with libfnx_b200.so, it calls two
// operator entry points on the GPU the way a maintainer's scheduler would (device buffers, a stream, the err word).
// A drifted signature (an int for a size_t, a missing argument) fails here at compile or link time.
//   consumer <rows> <cols>   -> prints "ok <checksum>" ; exit code 0 on success
#include <cuda_runtime.h>

#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <vector>

#include "fnx_b200.h"

#define CK(x)                                                                      \
    do {                                                                           \
        if ((x) != 0) {                                                            \
            std::fprintf(stderr, "%s failed: %s\n", #x, fnx_last_error());         \
            return 2;                                                              \
        }                                                                          \
    } while (0)
#define CU(x)                                                                      \
    do {                                                                           \
        cudaError_t e_ = (x);                                                      \
        if (e_ != cudaSuccess) {                                                   \
            std::fprintf(stderr, "%s: %s\n", #x, cudaGetErrorString(e_));          \
            return 3;                                                              \
        }                                                                          \
    } while (0)

int main(int argc, char** argv) {
    const int rows = argc > 1 ? std::atoi(argv[1]) : 256, cols = argc > 2 ? std::atoi(argv[2]) : 1024, T = 3, E = 16, K = 4;
    cudaStream_t st;
    CU(cudaStreamCreate(&st));
    // a random IQ3_S matrix: fill, quantise, re-tile (all entry points of the header)
    const size_t n = (size_t) rows * cols, wb = fnx_iq3s_bytes(rows, cols);
    float *w, *x, *y, *wr, *logits, *topw;
    void *g, *tiles;
    unsigned* err;
    int *topi, *njobs;
    fnx_job* jobs;
    CU(cudaMalloc(&w, n * sizeof(float)));
    CU(cudaMalloc(&g, wb));
    CU(cudaMalloc(&tiles, wb));
    CU(cudaMalloc(&x, (size_t) T * cols * sizeof(float)));
    CU(cudaMalloc(&y, (size_t) T * rows * sizeof(float)));
    CU(cudaMalloc(&err, sizeof(unsigned)));
    CU(cudaMemset(err, 0, sizeof(unsigned)));
    CK(fnx_fill_normal(w, n, 0.02f, 7, 1, st));
    CK(fnx_iq3s_quantize(w, g, n, st));
    CK(fnx_iq3s_retile(g, tiles, (size_t) rows, (size_t) cols, st));
    CK(fnx_fill_normal(x, (size_t) T * cols, 1.0f, 7, 2, st));
    CK(fnx_dense(tiles, rows, cols, x, cols, T, nullptr, 1e-6f, y, rows, 0, err, st));
    // reference: the same product from the dequantised tiles
    CK(fnx_iq3s_dequant_tiles(tiles, w, (size_t) rows, (size_t) cols, st));
    std::vector<float> hw(n), hx((size_t) T * cols), hy((size_t) T * rows);
    CU(cudaStreamSynchronize(st));
    CU(cudaMemcpy(hw.data(), w, n * sizeof(float), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(hx.data(), x, hx.size() * sizeof(float), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(hy.data(), y, hy.size() * sizeof(float), cudaMemcpyDeviceToHost));
    double worst = 0, big = 0, sum = 0;
    for (int t = 0; t < T; ++t)
        for (int r = 0; r < rows; ++r) {
            double s = 0;
            for (int c = 0; c < cols; ++c) s += (double) hw[(size_t) r * cols + c] * hx[(size_t) t * cols + c];
            worst = std::fmax(worst, std::fabs(s - hy[(size_t) t * rows + r]));
            big = std::fmax(big, std::fabs(s));
            sum += hy[(size_t) t * rows + r];
        }
    if (worst > 2e-3 * big) {
        std::fprintf(stderr, "fnx_dense differs: %g of %g\n", worst, big);
        return 4;
    }
    // router: top-K of T rows over E experts
    CU(cudaMalloc(&wr, (size_t) (E + 1) * cols * sizeof(float)));
    CU(cudaMalloc(&logits, (size_t) T * (E + 1) * sizeof(float)));
    CU(cudaMalloc(&topw, (size_t) T * K * sizeof(float)));
    CU(cudaMalloc(&topi, (size_t) T * K * sizeof(int)));
    CU(cudaMalloc(&njobs, 2 * sizeof(int)));
    CU(cudaMemset(njobs, 0, 2 * sizeof(int)));
    CU(cudaMalloc(&jobs, (size_t) (T * K + 1) * sizeof(fnx_job)));
    CK(fnx_fill_normal(wr, (size_t) (E + 1) * cols, 0.02f, 7, 3, st));
    CK(fnx_router_route(wr, x, nullptr, 1e-6f, T, E, cols, K, 0, E, 1, logits, topi, topw, jobs, njobs, nullptr, err, st));
    CU(cudaStreamSynchronize(st));
    std::vector<int> hi((size_t) T * K), hn(2);
    std::vector<float> hl((size_t) T * (E + 1));
    unsigned herr = 0;
    CU(cudaMemcpy(hi.data(), topi, hi.size() * sizeof(int), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(hl.data(), logits, hl.size() * sizeof(float), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(hn.data(), njobs, 2 * sizeof(int), cudaMemcpyDeviceToHost));
    CU(cudaMemcpy(&herr, err, sizeof herr, cudaMemcpyDeviceToHost));
    for (int t = 0; t < T; ++t) {   // the first pick is the row's largest logit
        int best = 0;
        for (int e = 1; e < E; ++e)
            if (hl[(size_t) t * (E + 1) + e] > hl[(size_t) t * (E + 1) + best]) best = e;
        if (hi[(size_t) t * K] != best) {
            std::fprintf(stderr, "fnx_router_route: row %d picks %d first, the largest logit is %d\n", t, hi[(size_t) t * K], best);
            return 5;
        }
    }
    if (herr != 0 || hn[0] < 1 || hn[0] > T * K + 1) {
        std::fprintf(stderr, "err word %u, %d jobs\n", herr, hn[0]);
        return 6;
    }
    std::printf("ok %.6f %d\n", sum, hn[0]);
    return 0;
}
