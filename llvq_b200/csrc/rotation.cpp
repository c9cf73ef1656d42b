#include "rotation.h"

#include <cmath>

namespace llvq {
namespace {

struct Rng {
    uint64_t state;
    uint64_t next() {
        state += 0x9E3779B97F4A7C15ull;
        uint64_t z = state;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        return z ^ (z >> 31);
    }
    double uniform() { return (double)(next() >> 11) * (1.0 / 9007199254740992.0); }
    double gaussian() {  // cosine branch of Box-Muller; u1 in (0, 1]
        const double u1 = ((double)(next() >> 11) + 1.0) * (1.0 / 9007199254740993.0);
        const double u2 = uniform();
        return std::sqrt(-2.0 * std::log(u1)) * std::cos(6.283185307179586476925286766559 * u2);
    }
};

}  // namespace

RotationTables build_rotation(int n, uint64_t seed) {
    RotationTables t;
    t.n = n;
    t.m = n & -n;
    t.k = n / t.m;
    Rng rng{seed};
    t.signbits.assign(((size_t)n + 31) / 32, 0u);
    for (int i = 0; i < n; ++i)
        if (rng.gaussian() < 0.0) t.signbits[i >> 5] |= 1u << (i & 31);
    // Gram-Schmidt on Gaussian rows, sums left to right (rotation.rs:215-235)
    const int k = t.k;
    std::vector<double> q((size_t)k * k, 0.0), row(k);
    for (int i = 0; i < k; ++i) {
        for (int c = 0; c < k; ++c) row[c] = rng.gaussian();
        for (int p = 0; p < i; ++p) {
            const double* prev = q.data() + (size_t)p * k;
            double d = 0.0;
            for (int c = 0; c < k; ++c) d += row[c] * prev[c];
            for (int c = 0; c < k; ++c) row[c] -= d * prev[c];
        }
        double nrm = 0.0;
        for (int c = 0; c < k; ++c) nrm += row[c] * row[c];
        nrm = std::sqrt(nrm);
        for (int c = 0; c < k; ++c) q[(size_t)i * k + c] = row[c] / nrm;
    }
    t.small.resize((size_t)k * k);
    for (size_t i = 0; i < t.small.size(); ++i) t.small[i] = (float)q[i];
    t.inv = (float)(1.0 / std::sqrt((double)t.m));
    return t;
}

}  // namespace llvq
