// Small scalar helpers shared by the decoders (decode_tab.cuh): bit casts, the exact-division
// constants of a slot count, the quotient of a local rank by an arrangement count, byte permutes.
// Everything compiles as device code and as plain host C++ (the test-suite runs the host build
// against the CPU oracle).
#pragma once
#include <cstdint>
#include <cstring>

#include "codebook.h"
#include "portable.h"

namespace llvq {

struct Quad {
    unsigned int x, y, z, w;
};


template <typename T>
LLVQ_HD T ldg(const T* p) {
#if defined(__CUDA_ARCH__)
    return __ldg(p);
#else
    return *p;
#endif
}

LLVQ_HD float bits_to_float(unsigned int u) {
#if defined(__CUDA_ARCH__)
    return __uint_as_float(u);
#else
    float f;
    std::memcpy(&f, &u, 4);
    return f;
#endif
}

LLVQ_HD unsigned int float_to_bits(float f) {
#if defined(__CUDA_ARCH__)
    return __float_as_uint(f);
#else
    unsigned int u;
    std::memcpy(&u, &f, 4);
    return u;
#endif
}

// n = 2^a * o
LLVQ_CONSTEXPR int two_adic(int n) {
    int a = 0;
    while ((n & 1) == 0) {
        n >>= 1;
        ++a;
    }
    return a;
}
LLVQ_CONSTEXPR unsigned int odd_part(int n) {
    while ((n & 1) == 0) n >>= 1;
    return (unsigned int)n;
}
// inverse of an odd o modulo 2^32 (Newton iteration doubles the valid bits)
LLVQ_CONSTEXPR unsigned int inv_mod32(unsigned int o) {
    unsigned int x = o;  // correct to 3 bits
    for (int i = 0; i < 5; ++i) x *= 2u - o * x;
    return x;
}

// local = g * m + r with g < 4096, m < 2^31: quotient from a float estimate, fixed
// up exactly by the 64-bit remainder.
LLVQ_HD void divmod_odd(unsigned long long local, unsigned int m, float rcp, unsigned int* g, unsigned int* r) {
    const float lf = (float)(unsigned int)(local >> 32) * 4294967296.0f + (float)(unsigned int)local;
    unsigned int q = (unsigned int)(lf * rcp);
    long long rem = (long long)(local - (unsigned long long)q * m);
    if (rem < 0) {
        q -= 1;
        rem += m;
    } else if (rem >= (long long)m) {
        q += 1;
        rem -= m;
    }
    *g = q;
    *r = (unsigned int)rem;
}

// Byte permute of the 8 bytes {a, b} (CUDA __byte_perm semantics, selector nibbles 0-7).
LLVQ_HD unsigned int byte_perm32(unsigned int a, unsigned int b, unsigned int sel) {
#if defined(__CUDA_ARCH__)
    return __byte_perm(a, b, sel);
#else
    const unsigned long long v = (unsigned long long)b << 32 | a;
    unsigned int r = 0;
    for (int i = 0; i < 4; ++i) r |= (unsigned int)((v >> (8 * ((sel >> (4 * i)) & 7u))) & 0xffu) << (8 * i);
    return r;
#endif
}

}  // namespace llvq
