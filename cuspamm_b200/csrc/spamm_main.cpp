// Command-line driver with the shape of the reference's `main` (cuSpAMM.cu:395-556): generate two matrices on the
// host, run SpAMM TESTTIME times on DEVICEDIM GPUs (C split by tile rows), print the parameter line and the mean
// time.  What para.h fixes at compile time is a command-line option here:
//
//   spamm_main [--n N | --m M --k K --nn N] [--devices D] [--tau T] [--iters I] [--warmup W]
//              [--matrix alg|exp|ones|sexp|ualg|uniform] [--tune RATE] [--float]
//
// --float is the counterpart of building the reference with USINGHALF 0 (para.h): float-level accuracy, here through
// the split-precision mode on the tensor cores.
//
// Defaults are the reference's: 2048^3, one device, tau = 1.548969, algebraic decay c=v=0.1, 10 iterations of which
// the first 5 are warm-up (para.h:1-14).  Differences: the mean is the true mean over the timed iterations (the
// reference divides 4 samples by 5, cuSpAMM.cu:545,549), every device is synchronised before the clock stops
// (cuSpAMM.cu:539 waits for one), inputs are float (the conversion to half happens on the GPU), and sizes that are
// not multiples of 32 are padded with zeros by the library (the reference extends its generated pattern into the
// padding or leaves it uninitialised, cuSpAMM.cu:410,425-430).
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <string>
#include <vector>

#include <cuda_runtime.h>

#include "../../include/spamm.h"

static int fail(const char *what, int st)
{
    fprintf(stderr, "%s: %s (%s)\n", what, spamm_status_string(st), spamm_last_cuda_error());
    return 1;
}

int main(int argc, char **argv)
{
    int M = 2048, K = 2048, N = 2048, devices = 1, iters = 10, warmup = 5;
    double tau = 1.548969, tune = -1.0;
    std::string matrix = "alg";
    bool split = false;
    for (int i = 1; i < argc; i++) {
        auto next = [&](const char *name) -> const char * {
            if (i + 1 >= argc) { fprintf(stderr, "%s needs a value\n", name); exit(2); }
            return argv[++i];
        };
        if (!strcmp(argv[i], "--n")) M = K = N = atoi(next("--n"));
        else if (!strcmp(argv[i], "--m")) M = atoi(next("--m"));
        else if (!strcmp(argv[i], "--k")) K = atoi(next("--k"));
        else if (!strcmp(argv[i], "--nn")) N = atoi(next("--nn"));
        else if (!strcmp(argv[i], "--devices")) devices = atoi(next("--devices"));
        else if (!strcmp(argv[i], "--tau")) tau = atof(next("--tau"));
        else if (!strcmp(argv[i], "--iters")) iters = atoi(next("--iters"));
        else if (!strcmp(argv[i], "--warmup")) warmup = atoi(next("--warmup"));
        else if (!strcmp(argv[i], "--matrix")) matrix = next("--matrix");
        else if (!strcmp(argv[i], "--tune")) tune = atof(next("--tune"));
        else if (!strcmp(argv[i], "--float")) split = true;
        else { fprintf(stderr, "unknown option %s\n", argv[i]); return 2; }
    }
    // the reference pads to multiples of 32 (main.h:54-56)
    const int Mp = (M + 31) / 32 * 32, Kp = (K + 31) / 32 * 32, Np = (N + 31) / 32 * 32;
    printf("input parameters: M=%d K=%d N=%d Norm=%f USINGHALF=%d devices=%d matrix=%s\n", Mp, Kp, Np, tau,
           split ? 0 : 1, devices, matrix.c_str());
    const int row_tiles = Mp / 32;
    if (devices <= 0 || iters <= warmup || row_tiles / devices <= 0) {
        printf("PART error! too many parts!\n");
        return 1;
    }
    float *h_A = nullptr, *h_B = nullptr, *h_C = nullptr;
    if (cudaMallocHost(&h_A, sizeof(float) * (size_t)M * K) != cudaSuccess ||
        cudaMallocHost(&h_B, sizeof(float) * (size_t)K * N) != cudaSuccess ||
        cudaMallocHost(&h_C, sizeof(float) * (size_t)M * N) != cudaSuccess) {
        fprintf(stderr, "host allocation failed\n");
        return 1;
    }
    int st = 0;
    if (matrix == "alg") { st |= spamm_gen_decay_alg(h_A, 0.1f, 0.1f, 0, M, K); st |= spamm_gen_decay_alg(h_B, 0.1f, 0.1f, 0, K, N); }
    else if (matrix == "ones") { st |= spamm_gen_ones(h_A, 0, M, K); st |= spamm_gen_ones(h_B, 0, K, N); }   // MATRIXNOR
    else if (matrix == "exp") { st |= spamm_gen_decay_exp(h_A, 1.0f, 0.1f, 0, M, K); st |= spamm_gen_decay_exp(h_B, 1.0f, 0.1f, 0, K, N); }
    else if (matrix == "sexp") { st |= spamm_gen_signed_exp(h_A, 0.1, 1, 0, M, K); st |= spamm_gen_signed_exp(h_B, 0.1, 2, 0, K, N); }
    else if (matrix == "ualg") { st |= spamm_gen_uniform_alg(h_A, 3, 0, M, K); st |= spamm_gen_uniform_alg(h_B, 4, 0, K, N); }
    else if (matrix == "uniform") { st |= spamm_gen_uniform(h_A, 5, 0, M, K); st |= spamm_gen_uniform(h_B, 6, 0, K, N); }
    else { fprintf(stderr, "unknown matrix kind %s\n", matrix.c_str()); return 2; }
    if (st) return fail("generator", st);

    std::vector<spamm_plan *> plan(devices, nullptr);
    std::vector<int> begin(devices), count(devices);
    for (int d = 0, b = 0; d < devices; d++) {          // device d owns tile rows [d*T/G, (d+1)*T/G), cuSpAMM.cu:503
        begin[d] = b;
        count[d] = (d == devices - 1) ? row_tiles - b : row_tiles / devices;
        b += count[d];
        if ((st = spamm_plan_create(&plan[d], M, K, N, begin[d], count[d], d))) return fail("spamm_plan_create", st);
        if (split && (st = spamm_plan_set_precision(plan[d], SPAMM_PRECISION_SPLIT)))
            return fail("spamm_plan_set_precision", st);
        if ((st = spamm_upload(plan[d], h_A + (size_t)begin[d] * 32 * K, h_B))) return fail("spamm_upload", st);
    }
    float norm = (float)tau;
    if (tune > 0) {                                     // TUNINGFLAG, main.h:35-38, cuSpAMM.cu:513-515
        double rate = 0;
        int it = 0;
        if ((st = spamm_norms(plan[0]))) return fail("spamm_norms", st);
        if ((st = spamm_tune_tau(plan[0], tune, 20, 0.01, &norm, &rate, &it))) return fail("spamm_tune_tau", st);
        printf("tuned Norm=%g valid ratio=%f after %d passes\n", norm, rate, it);
    }
    double sum = 0;
    for (int i = 0; i < iters; i++) {
        for (int d = 0; d < devices; d++) if ((st = spamm_sync(plan[d]))) return fail("spamm_sync", st);
        const auto t0 = std::chrono::steady_clock::now();
        for (int d = 0; d < devices; d++) if ((st = spamm_run(plan[d], norm))) return fail("spamm_run", st);
        for (int d = 0; d < devices; d++) if ((st = spamm_sync(plan[d]))) return fail("spamm_sync", st);
        const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (i >= warmup) sum += el;
    }
    int64_t survivors = 0;
    for (int d = 0; d < devices; d++) {
        int64_t s = 0;
        if ((st = spamm_get_counts(plan[d], nullptr, &s))) return fail("spamm_get_counts", st);
        survivors += s;
        if ((st = spamm_download_c(plan[d], h_C + (size_t)begin[d] * 32 * N))) return fail("spamm_download_c", st);
    }
    const double t = sum / (iters - warmup);
    const double total = (double)(Mp / 32) * (Kp / 32) * (Np / 32);
    printf("valid mul=%lld, simple mul=%.0f, rate=%f%%\n", (long long)survivors, total, 100.0 * survivors / total);
    printf("SpAMM time=%fs\n", t);
    printf("executed TFLOP/s=%f\n", 65536.0 * survivors / t / 1e12);
    for (int d = 0; d < devices; d++) spamm_plan_destroy(plan[d]);
    cudaFreeHost(h_A); cudaFreeHost(h_B); cudaFreeHost(h_C);
    return 0;
}
