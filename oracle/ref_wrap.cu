// TEST INFRASTRUCTURE.  Thin extern "C" launchers around the reference's OWN kernels, so that the CPU checker
// and the CUDA path can be compared with what buaa-hipo/cuSpAMM itself computes on the same inputs.
//
// This file contains no reference code: build_ref.sh compiles it inside a scratch copy of the reference tree, where
// the #include below pulls in the reference's cuSpAMM.cu unmodified (its `main` renamed out of the way) with the
// matrix size of para.h set by the build script.  The reference's sizes are compile-time constants (para.h:6-8,
// main.h:54-56,73), hence one library per size.  Launch shapes are the reference's (cuSpAMM.cu:478,486,503,530).
#define main reference_main_not_used
#include "cuSpAMM.cu"
#undef main

extern "C" {

void ref_dims(int *m, int *k, int *n) { *m = M; *k = K; *n = N; }

// unroll_get_Fnorm_pri as launched at cuSpAMM.cu:478/495: one 128-thread block per tile
int ref_norm_fp32(const float *d_x, float *d_map, int rows, int cols)
{
    const int blocks = rows * cols / (LoNum * LoNum);
    unroll_get_Fnorm_pri<<<blocks, LoNum * LoNum / 8>>>(d_x, d_map, rows, cols, 0);
    return (int)cudaDeviceSynchronize();
}

// unroll_get_Fnorm_FP16 as launched at cuSpAMM.cu:486/503
int ref_norm_fp16(const half *d_x, float *d_map, int rows, int cols)
{
    const int blocks = rows * cols / (LoNum * LoNum);
    unroll_get_Fnorm_FP16<<<blocks, 32 * 4>>>(d_x, d_map, rows, cols, 0);
    return (int)cudaDeviceSynchronize();
}

// get_C_FP16_B32 as launched at cuSpAMM.cu:530 for `row_tiles` tile rows starting at tile row `row_offset`
int ref_get_c_fp16(const half *d_a, const float *d_norm_a, const half *d_b, const float *d_norm_b, float *d_c,
                   int row_offset, int row_tiles, float norm)
{
    const int blocks = row_tiles * (N / LoNum);
    get_C_FP16_B32<<<blocks, 32 * 4>>>(d_a, d_norm_a, d_b, d_norm_b, d_c, row_offset, norm);
    return (int)cudaDeviceSynchronize();
}

// One pass of the reference's timed region (cuSpAMM.cu:485-531, one device, PART 1) without a synchronisation: the
// norm map of B, the norm map of A, the gated multiply, on the default stream.  The caller brackets a number of
// calls with events on that stream to time the reference's kernels on this GPU.
int ref_timed_step_fp16(const half *d_a, float *d_norm_a, const half *d_b, float *d_norm_b, float *d_c, float norm)
{
    unroll_get_Fnorm_FP16<<<K * N / (LoNum * LoNum), 32 * 4>>>(d_b, d_norm_b, K, N, 0);
    unroll_get_Fnorm_FP16<<<M * K / (LoNum * LoNum), 32 * 4>>>(d_a, d_norm_a, M, K, 0);
    get_C_FP16_B32<<<(M / LoNum) * (N / LoNum), 32 * 4>>>(d_a, d_norm_a, d_b, d_norm_b, d_c, 0, norm);
    return (int)cudaGetLastError();
}

}  // extern "C"
