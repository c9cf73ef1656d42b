// Class-specialised scalar decoders of the cap-12 ball (47-bit index).
//
// A block is first classified (class search + local rank), then decoded by the
// routine of its class family, every lane of a warp running the same routine:
//
//   odd_fast<K>   odd coset, K thresholds per slot (K + 1 kinds). The 24-slot
//                 multiset unranking of llvq-search/src/fastdec.rs:173-194 with the
//                 candidate loop turned into K branch-free threshold compares per
//                 slot: T_j = M * C_j / n for the cumulative kind counts C_j, the slot
//                 holds kind #{j : rank >= T_j}. All arithmetic is 32-bit: arrangement
//                 counts of the cap-12 ball stay below 2^31, the division by the
//                 slot count n = 2^a * o is exact, so T_j = ((M * o^-1 mod 2^32) * C_j) >> a
//                 whenever T_j * 2^a < 2^32, which holds for every reachable state
//                 with n <= 23; the first slot (n = 24) takes a 64-bit product.
//   even_fast     even coset. The local rank is peeled into (r_sf, r_sw, r_off, r_on, g)
//                 exactly as llvq-search/src/index.rs:361-369 does, with the two
//                 divisions by a_off and a_on replaced by per-class magic multipliers;
//                 the on- and off-support arrangements come from tables indexed by
//                 (problem, rank) instead of being unranked slot by slot.
//
// Everything here compiles as device code and as plain host C++ (tests run the
// host build against the CPU oracle). Values are delivered in position order
// through emit(pos, value) with value already signed, as a float.
#pragma once
#include <cstdint>
#include <cstring>

#include "codebook.h"
#include "portable.h"

namespace llvq {

struct FastTables {
    const FastClass* cls;            // 301 records
    const unsigned long long* ends;  // offset + card per class
    const unsigned short* lut;       // class search accelerator
    const unsigned int* golay;       // 4096 codewords
    const unsigned int* lut_on;      // on-support arrangement table
    const unsigned int* lut_off;     // off-support arrangement table
    int lut_shift;
};

struct Quad {
    unsigned int x, y, z, w;
};

LLVQ_HD Quad load_quad(const FastClass* c, int q) {
#if defined(__CUDA_ARCH__)
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(c) + q);
    return Quad{v.x, v.y, v.z, v.w};
#else
    const unsigned int* p = reinterpret_cast<const unsigned int*>(c) + 4 * q;
    return Quad{p[0], p[1], p[2], p[3]};
#endif
}

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

// Result of the class search for one index of the cap-12 ball.
struct Classified {
    int ci;                    // class, or -1 for the origin, -2 for an index outside the ball
    unsigned int path;         // FastPath
    unsigned int arr;          // m_arr (odd) / a_off (even)
    unsigned long long local;  // rank inside the class
};

LLVQ_HD Classified classify12(const FastTables& T, unsigned long long idx) {
    Classified r;
    r.path = kPathSlow;
    r.arr = 0;
    r.local = 0;
    if (idx == 0 || idx > kN12) {
        r.ci = idx == 0 ? -1 : -2;
        return r;
    }
    const unsigned long long i = idx - 1;
    int ci = ldg(T.lut + (i >> T.lut_shift));
    while (i >= ldg(T.ends + ci)) ++ci;
    const Quad q0 = load_quad(T.cls + ci, 0);
    r.ci = ci;
    r.path = q0.w & 3u;
    r.arr = q0.z;
    r.local = i - ((unsigned long long)q0.y << 32 | q0.x);
    return r;
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

template <int K, class Emit>
LLVQ_HD void odd_fast(unsigned int rank, unsigned int m_arr, unsigned int cum, unsigned int sv, unsigned int cw,
                      Emit emit) {
    static_assert(K >= 1 && K <= 3, "one to three thresholds");
    unsigned int C[K];
    float f[K + 1];
#pragma unroll
    for (int j = 0; j < K; ++j) C[j] = (cum >> (8 * j)) & 0xffu;
#pragma unroll
    for (int j = 0; j <= K; ++j) f[j] = (float)(int)(signed char)((sv >> (8 * j)) & 0xffu);
    unsigned int R = rank, M = m_arr;
    const unsigned int ncw = ~cw;
#pragma unroll
    for (int pos = 0; pos < kDim; ++pos) {
        const int n = kDim - pos;
        unsigned int T[K];
        if (n == kDim) {
#pragma unroll
            for (int j = 0; j < K; ++j)
                T[j] = (unsigned int)(((unsigned long long)M * C[j]) >> 3) * 0xAAAAAAABu;  // / 8, then / 3
        } else {
            const int a = two_adic(n);
            const unsigned int o = odd_part(n);
            const unsigned int mo = o == 1 ? M : M * inv_mod32(o);
#pragma unroll
            for (int j = 0; j < K; ++j) T[j] = (mo * C[j]) >> a;
        }
        bool p[K];
#pragma unroll
        for (int j = 0; j < K; ++j) p[j] = R >= T[j];
        unsigned int lo = 0, hi = M;
#pragma unroll
        for (int j = 0; j < K; ++j) lo = p[j] ? T[j] : lo;
#pragma unroll
        for (int j = K - 1; j >= 0; --j) hi = p[j] ? hi : T[j];
        R -= lo;
        M = hi - lo;
        float fv = f[0];
#pragma unroll
        for (int j = 0; j < K; ++j) {
            C[j] -= p[j] ? 0u : 1u;
            fv = p[j] ? f[j + 1] : fv;
        }
        // a coordinate off the codeword support takes the negated value
        emit(pos, bits_to_float(float_to_bits(fv) ^ ((ncw << (31 - pos)) & 0x80000000u)));
    }
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

// 16 bits -> 32 bits, bit s moves to bit 2s
LLVQ_HD unsigned int spread16(unsigned int x) {
    x = (x | (x << 8)) & 0x00FF00FFu;
    x = (x | (x << 4)) & 0x0F0F0F0Fu;
    x = (x | (x << 2)) & 0x33333333u;
    x = (x | (x << 1)) & 0x55555555u;
    return x;
}

template <class Emit>
LLVQ_HD void even_fast(const FastTables& T, unsigned long long local, unsigned int a_off, const Quad& q1,
                       const Quad& q2, Emit emit) {
    const unsigned int a_on = q1.x & 0xffffu;
    const unsigned int w = (q1.x >> 16) & 0xffu;
    const unsigned int free_n = (q1.x >> 24) & 0x7fu;
    const unsigned int p_req = q1.x >> 31;
    const unsigned int wb = w - 1;
    const unsigned int r_sf = (unsigned int)local & ((1u << free_n) - 1u);
    const unsigned long long t = local >> free_n;
    const unsigned int r_sw = (unsigned int)t & ((1u << wb) - 1u);
    const unsigned int Q = (unsigned int)(t >> wb);  // < 2^28
    const unsigned int q = umulhi32(Q << 4, q1.y) >> (q1.w & 0xffu);
    const unsigned int r_off = Q - q * a_off;
    const unsigned int g = umulhi32(q << 4, q1.z) >> ((q1.w >> 8) & 0xffu);
    const unsigned int r_on = q - g * a_on;
    const unsigned int cw = ldg(T.golay + (q1.w >> 16) + g);
    // the last support sign is forced by the class parity (index.rs:386-388)
    const unsigned int sw = r_sw | ((((unsigned int)popc32(r_sw) & 1u) ^ p_req) << wb);
    unsigned int on = ldg(T.lut_on + q2.x + r_on) | (spread16(sw) << 1);  // (sign, kind) per support slot
    unsigned int off = ldg(T.lut_off + q2.y + r_off);                    // kind per off-support slot
    unsigned int sf = r_sf;
#pragma unroll
    for (int pos = 0; pos < kDim; ++pos) {
        const bool bit = (cw >> pos) & 1u;
        const unsigned int t = bit ? on : off;
        // |value| as a float without an integer->float conversion: the table byte is
        // dropped into the mantissa of 2^23 (0x4B000000) and 2^23 is subtracted.
        const unsigned int mag = byte_perm32(bit ? q2.z : q2.w, 0x4B000000u, (t & 3u) | 0x7440u);
        float val = bits_to_float(mag) - 8388608.0f;
        if (bit) on >>= 2; else off >>= 2;
        // support slot: the sign travels in bit 1 of its code; off-support slot: the next
        // free sign bit, consumed only by a non-zero value (the zero run is recognised by
        // its value, never by its kind index)
        const bool nz = !bit && mag != 0x4B000000u;
        const unsigned int sbit = bit ? (t << 30) : (sf << 31);
        val = bits_to_float(float_to_bits(val) ^ (sbit & 0x80000000u));
        if (nz) sf >>= 1;
        emit(pos, val);
    }
}

// Decode one cap-12 index with whichever routine its class calls for; returns the
// path taken (tests use this to make sure every family is exercised) or -1 for the
// origin / -2 for a refused index. `slow` is called as slow(idx) for the classes
// the fast families do not cover.
template <class Emit, class Slow>
LLVQ_HD int decode_fast_any(const FastTables& T, unsigned long long idx, Emit emit, Slow slow, float* scale) {
    const Classified c = classify12(T, idx);
    if (c.ci < 0) {
        for (int pos = 0; pos < kDim; ++pos) emit(pos, 0.0f);
        *scale = 0.0f;
        return c.ci;
    }
    const FastClass* rec = T.cls + c.ci;
    if (c.path == kPathSlow) {
        slow(idx);
        *scale = 0.0f;
        return (int)kPathSlow;
    }
    const Quad q1 = load_quad(rec, 1);
    if (c.path == kPathEven) {
        const Quad q2 = load_quad(rec, 2);
        const Quad q3 = load_quad(rec, 3);
        *scale = bits_to_float(q3.x);
        even_fast(T, c.local, c.arr, q1, q2, emit);
        return (int)kPathEven;
    }
    unsigned int g, r;
    divmod_odd(c.local, c.arr, bits_to_float(q1.w), &g, &r);
    const unsigned int cw = ldg(T.golay + g);
    *scale = bits_to_float(q1.z);
    if (c.path == kPathOdd2)
        odd_fast<2>(r, c.arr, q1.x, q1.y, cw, emit);
    else
        odd_fast<3>(r, c.arr, q1.x, q1.y, cw, emit);
    return (int)c.path;
}

}  // namespace llvq
