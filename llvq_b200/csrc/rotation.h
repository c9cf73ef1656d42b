// Host-side construction of the incoherence rotation Q = (Q_odd (x) H_m) D that a sealed matrix was
// quantised in (llvq-quant/src/rotation.rs:51-68): n = k * m with m the largest power of two dividing
// n, D a +-1 diagonal drawn from the matrix's rotation seed, H_m the orthogonal Walsh-Hadamard
// transform on each of the k groups of m coordinates, Q_odd a k x k orthogonal matrix from
// Gram-Schmidt on Gaussian rows. The tables are what the reference's host hands its kernel
// (RotationTables::build, llvq-llm/src/fused.rs:678-725): a sign bitmap (bit set = negative),
// Q_odd narrowed to f32, and 1/sqrt(m) computed in f64 and narrowed once.
#pragma once
#include <cstdint>
#include <vector>

namespace llvq {

constexpr int kRotMaxOdd = 32;  // largest odd factor served, as the reference's LLVQ_ROT_KMAX

struct RotationTables {
    int n = 0, m = 0, k = 0;
    std::vector<uint32_t> signbits;  // ceil(n / 32) words
    std::vector<float> small;        // k * k, row-major
    float inv = 0.0f;                // 1 / sqrt(m)
};

// Deterministic in (n, seed): SplitMix64 with Box-Muller normals (llvq-core/src/rng.rs:21-41).
RotationTables build_rotation(int n, uint64_t seed);

}  // namespace llvq
