// Host-side input generators: the two deterministic decay generators of the reference (tool.cu:409-436) and the
// seeded families the benchmark configurations use.  Every element depends only on (seed, i, j), so a process can
// generate just the rows it owns.  Values are computed in double and rounded once to float.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdlib>
#include <thread>
#include <vector>

#include "../../include/spamm.h"

namespace {

inline uint64_t mix64(uint64_t z)
{
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}

// counter-based hash of (seed, i, j)
inline uint64_t hash3(uint64_t seed, uint64_t i, uint64_t j) { return mix64(mix64(mix64(seed) + i) + j); }

// uniform in [0, 1) with 53 bits
inline double u01(uint64_t h) { return (double)(h >> 11) * (1.0 / 9007199254740992.0); }

template <typename F>
void parallel_rows(int64_t rows, F &&fn)
{
    unsigned hw = std::thread::hardware_concurrency();
    int64_t nt = std::max<int64_t>(1, std::min<int64_t>(hw ? hw : 1, rows / 16));
    if (nt <= 1) {
        for (int64_t r = 0; r < rows; r++) fn(r);
        return;
    }
    std::vector<std::thread> th;
    th.reserve((size_t)nt);
    for (int64_t t = 0; t < nt; t++) {
        th.emplace_back([=, &fn] {
            const int64_t lo = rows * t / nt, hi = rows * (t + 1) / nt;
            for (int64_t r = lo; r < hi; r++) fn(r);
        });
    }
    for (auto &t : th) t.join();
}

bool bad(const float *out, int64_t row_begin, int64_t rows, int64_t cols)
{
    return !out || row_begin < 0 || rows < 0 || cols < 0;
}

}  // namespace

extern "C" {

int spamm_gen_decay_exp(float *out, float c, float v, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        for (int64_t j = 0; j < cols; j++)
            out[r * cols + j] = c * (float)std::pow((double)v, (double)std::llabs(i - j));
    });
    return SPAMM_OK;
}

int spamm_gen_decay_alg(float *out, float c, float v, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        for (int64_t j = 0; j < cols; j++)
            out[r * cols + j] = c / ((float)std::pow((double)std::llabs(i - j), (double)v) + 1.0f);
    });
    return SPAMM_OK;
}

int spamm_gen_ones(float *out, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        for (int64_t j = 0; j < cols; j++) out[r * cols + j] = 1.0f;
    });
    return SPAMM_OK;
}

int spamm_gen_signed_exp(float *out, double lambda, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    // exp(-lambda*d) once per distance
    const int64_t max_d = std::max<int64_t>(row_begin + rows, cols);
    std::vector<float> mag((size_t)max_d + 1);
    for (int64_t d = 0; d <= max_d; d++) mag[(size_t)d] = (float)std::exp(-lambda * (double)d);
    const float *m = mag.data();
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        for (int64_t j = 0; j < cols; j++) {
            const float v = m[std::llabs(i - j)];
            out[r * cols + j] = (hash3(seed, (uint64_t)i, (uint64_t)j) >> 63) ? -v : v;
        }
    });
    return SPAMM_OK;
}

int spamm_gen_uniform_alg(float *out, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        for (int64_t j = 0; j < cols; j++) {
            const double d = (double)std::llabs(i - j);
            const double u = 2.0 * u01(hash3(seed, (uint64_t)i, (uint64_t)j)) - 1.0;
            out[r * cols + j] = (float)(u / (d * d + 1.0));
        }
    });
    return SPAMM_OK;
}

int spamm_gen_uniform(float *out, uint64_t seed, int64_t row_begin, int64_t rows, int64_t cols)
{
    if (bad(out, row_begin, rows, cols)) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        for (int64_t j = 0; j < cols; j++)
            out[r * cols + j] = (float)(2.0 * u01(hash3(seed, (uint64_t)i, (uint64_t)j)) - 1.0);
    });
    return SPAMM_OK;
}

int spamm_gen_lattice(float *out, int L, uint64_t seed, int64_t row_begin, int64_t rows)
{
    if (!out || L <= 0 || row_begin < 0 || rows < 0) return SPAMM_ERR_INVALID;
    const int64_t n = (int64_t)L * L * L;
    if (row_begin + rows > n) return SPAMM_ERR_INVALID;
    parallel_rows(rows, [=](int64_t r) {
        const int64_t i = row_begin + r;
        const int64_t ix = i / ((int64_t)L * L), iy = (i / L) % L, iz = i % L;
        for (int64_t j = 0; j < n; j++) {
            const int64_t jx = j / ((int64_t)L * L), jy = (j / L) % L, jz = j % L;
            const double dx = (double)(ix - jx), dy = (double)(iy - jy), dz = (double)(iz - jz);
            const double dist = std::sqrt(dx * dx + dy * dy + dz * dz);
            const uint64_t h = hash3(seed, (uint64_t)std::min(i, j), (uint64_t)std::max(i, j));
            const double u = 0.5 + 0.5 * u01(h);
            const double v = u * std::exp(-dist);
            out[r * n + j] = (float)((h & 1ull) ? -v : v);
        }
    });
    return SPAMM_OK;
}

}  // extern "C"
