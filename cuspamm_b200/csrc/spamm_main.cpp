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

    // all devices through one group: every device owns a block of C tile rows (cuSpAMM.cu:503), uploads its rows of A
    // and its share of B, and computes its share of B's norm map in every step
    spamm_group *group = nullptr;
    if ((st = spamm_group_create(&group, M, K, N, devices, nullptr))) return fail("spamm_group_create", st);
    if (split)
        for (int d = 0; d < devices; d++) {
            spamm_plan *pl = nullptr;
            if ((st = spamm_group_plan(group, d, &pl)) || (st = spamm_plan_set_precision(pl, SPAMM_PRECISION_SPLIT)))
                return fail("spamm_plan_set_precision", st);
        }
    if ((st = spamm_group_upload(group, h_A, h_B))) return fail("spamm_group_upload", st);
    float norm = (float)tau;
    if (tune > 0) {                                     // TUNINGFLAG, main.h:35-38, cuSpAMM.cu:513-515
        double rate = 0;
        int it = 0;
        spamm_plan *pl = nullptr;
        // as the reference: tuned on the first device's block of rows (every device would find its own value there)
        if ((st = spamm_group_run(group, norm)) || (st = spamm_group_sync(group))) return fail("spamm_group_run", st);
        if ((st = spamm_group_plan(group, 0, &pl))) return fail("spamm_group_plan", st);
        if ((st = spamm_tune_tau(pl, tune, 20, 0.01, &norm, &rate, &it))) return fail("spamm_tune_tau", st);
        printf("tuned Norm=%g valid ratio=%f after %d passes\n", norm, rate, it);
    }
    double sum = 0;
    for (int i = 0; i < iters; i++) {
        if ((st = spamm_group_sync(group))) return fail("spamm_group_sync", st);
        const auto t0 = std::chrono::steady_clock::now();
        if ((st = spamm_group_run(group, norm))) return fail("spamm_group_run", st);
        if ((st = spamm_group_sync(group))) return fail("spamm_group_sync", st);
        const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (i >= warmup) sum += el;
    }
    int64_t survivors = 0;
    if ((st = spamm_group_survivors(group, &survivors))) return fail("spamm_group_survivors", st);
    if ((st = spamm_group_download_c(group, h_C))) return fail("spamm_group_download_c", st);
    const double t = sum / (iters - warmup);
    const double total = (double)(Mp / 32) * (Kp / 32) * (Np / 32);
    printf("valid mul=%lld, simple mul=%.0f, rate=%f%%\n", (long long)survivors, total, 100.0 * survivors / total);
    printf("SpAMM time=%fs\n", t);
    printf("executed TFLOP/s=%f\n", 65536.0 * survivors / t / 1e12);
    spamm_group_destroy(group);
    cudaFreeHost(h_A); cudaFreeHost(h_B); cudaFreeHost(h_C);
    return 0;
}
