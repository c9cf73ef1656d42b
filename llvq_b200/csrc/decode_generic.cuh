// Generic device decoder of the v1 index map: any class of the cap-13 ball, all
// arithmetic in 64 bits. It is the reference semantics written for one thread
// (Indexer::decode, llvq-search/src/index.rs:334-435, with the exact recurrence
// M' = M * c / n of llvq-search/src/fastdec.rs:173-194) and serves the decode
// probes, the fingerprint check and the rare classes the fast paths hand over.
//
// The 24 coordinates come out in position order through a callback, so nothing
// is staged in local memory: an even class runs its on-support and off-support
// unranking problems interleaved, steered by the codeword bits.
#pragma once
#include <cstdint>

#include "codebook.h"
#include "portable.h"

namespace llvq {

struct DevTables {
    const DevClass* cls;
    const unsigned long long* ends;  // offset + card per class
    const unsigned short* lut;       // class search accelerator, key = (idx-1) >> lut_shift
    const unsigned int* golay;       // 4096 codewords, weight-major
    int lut_shift;
};

// x / n for n | x, x < 2^53: the IEEE quotient of two exactly representable
// numbers whose true quotient is representable is exact.
LLVQ_HD unsigned long long exact_div_small(unsigned long long x, int n) {
    return (unsigned long long)((double)x / (double)n);
}

// One slot of a multiset unranking: pick the first kind j whose interval holds
// `rank`, consume one item of it. cnt holds one count per byte.
template <typename CntT>
LLVQ_HD int unrank_step(unsigned long long& rank, unsigned long long& m, int& n,
                                           CntT& cnt, int k) {
    int chosen = k - 1;
    for (int j = 0; j < k; ++j) {
        const unsigned int c = (unsigned int)(cnt >> (8 * j)) & 0xffu;
        if (c == 0) continue;
        const unsigned long long mj = exact_div_small(m * c, n);
        if (rank < mj || j == k - 1) {
            m = mj;
            chosen = j;
            break;
        }
        rank -= mj;
    }
    cnt -= (CntT)1 << (8 * chosen);
    n -= 1;
    return chosen;
}

LLVQ_HD int find_class(const DevTables& T, unsigned long long i) {
    int ci = T.lut[i >> T.lut_shift];
    while (i >= T.ends[ci]) ++ci;
    return ci;
}

// Decode `idx` (0 = origin). `limit` is the ball size (N(12) or N(13)): indices
// above it are refused. Calls emit(pos, value) for pos = 0..23 in order and
// returns the shell m (0 for the origin, 255 for a refused index; a refused
// index emits zeros). *scale receives 1/sqrt(16 m) (0 for the origin).
template <class Emit>
LLVQ_HD int decode_generic(const DevTables& T, unsigned long long idx,
                                              unsigned long long limit, Emit emit, float* scale) {
    if (idx == 0 || idx > limit) {
#pragma unroll
        for (int pos = 0; pos < kDim; ++pos) emit(pos, 0);
        *scale = 0.0f;
        return idx == 0 ? 0 : 255;
    }
    const unsigned long long i = idx - 1;
    const int ci = find_class(T, i);
    const DevClass c = T.cls[ci];
    unsigned long long local = i - c.offset;
    *scale = c.inv_norm;

    unsigned long long rank_a, m_a = c.arr_a, rank_b = 0, m_b = c.arr_b;
    unsigned long long cnt_a = c.cnts_a;
    unsigned int cnt_b = c.cnts_b;
    int n_a, n_b = 0;
    unsigned int cw, sw = 0, sf = 0;
    if (c.odd) {
        rank_a = local % c.arr_a;
        cw = T.golay[local / c.arr_a];
        n_a = kDim;
    } else {
        sf = (unsigned int)local & ((1u << c.free_n) - 1u);
        local >>= c.free_n;
        const int wb = c.w ? c.w - 1 : 0;
        sw = (unsigned int)local & ((1u << wb) - 1u);
        local >>= wb;
        rank_b = local % c.arr_b;
        local /= c.arr_b;
        rank_a = local % c.arr_a;
        cw = T.golay[c.golay_base + (unsigned int)(local / c.arr_a)];
        // the last support sign is forced by the class parity (index.rs:386-388)
        if (c.w) sw |= (unsigned int)((popc32(sw) & 1) ^ c.p_req) << (c.w - 1);
        n_a = c.w;
        n_b = kDim - c.w;
    }
#pragma unroll 1
    for (int pos = 0; pos < kDim; ++pos) {
        const unsigned int bit = (cw >> pos) & 1u;
        int val;
        if (c.odd || bit) {
            const int j = unrank_step(rank_a, m_a, n_a, cnt_a, (int)c.n_a);
            const int v = (int)((c.vals_a >> (4 * j)) & 15u);
            if (c.odd) {
                // forced signs (index.rs:424-430): v = 3 (mod 4) is positive on the
                // codeword support and negative off it; v = 1 (mod 4) the opposite.
                const int a = (v & 3) == 3 ? v : -v;
                val = bit ? a : -a;
            } else {
                val = (sw & 1u) ? -v : v;
                sw >>= 1;
            }
        } else {
            const int j = unrank_step(rank_b, m_b, n_b, cnt_b, (int)c.n_b);
            const int v = (int)((c.vals_b >> (4 * j)) & 15u);
            val = v;
            if (v) {  // the zero run is recognised by its value, not by its kind index
                val = (sf & 1u) ? -v : v;
                sf >>= 1;
            }
        }
        emit(pos, val);
    }
    return c.shell;
}

// ---------------------------------------------------------------------------
// The same decoder restricted to the cap-12 ball, where every arrangement count
// is below 2^31: the unranking runs in 32-bit arithmetic and M * c / n is the exact
// division ((M * c) >> a) * o^-1 mod 2^32 for n = 2^a * o (the quotient is below
// 2^31, so its low 32 bits are the quotient). This is what the GEMV runs for the
// rare classes outside its table-driven families.
// ---------------------------------------------------------------------------

// o^-1 mod 2^32 | a << 32 for n = 2^a * o, n = 1..24 (index 0 unused)
#define LLVQ_EXACT_DIV_TABLE \
    { 0ull, \
      0x00000001ull | 0ull << 32, \
      0x00000001ull | 1ull << 32, \
      0xAAAAAAABull | 0ull << 32, \
      0x00000001ull | 2ull << 32, \
      0xCCCCCCCDull | 0ull << 32, \
      0xAAAAAAABull | 1ull << 32, \
      0xB6DB6DB7ull | 0ull << 32, \
      0x00000001ull | 3ull << 32, \
      0x38E38E39ull | 0ull << 32, \
      0xCCCCCCCDull | 1ull << 32, \
      0xBA2E8BA3ull | 0ull << 32, \
      0xAAAAAAABull | 2ull << 32, \
      0xC4EC4EC5ull | 0ull << 32, \
      0xB6DB6DB7ull | 1ull << 32, \
      0xEEEEEEEFull | 0ull << 32, \
      0x00000001ull | 4ull << 32, \
      0xF0F0F0F1ull | 0ull << 32, \
      0x38E38E39ull | 1ull << 32, \
      0x286BCA1Bull | 0ull << 32, \
      0xCCCCCCCDull | 2ull << 32, \
      0x3CF3CF3Dull | 0ull << 32, \
      0xBA2E8BA3ull | 1ull << 32, \
      0xE9BD37A7ull | 0ull << 32, \
      0xAAAAAAABull | 3ull << 32, }
static const unsigned long long kExactDivHost[25] = LLVQ_EXACT_DIV_TABLE;
#if defined(__CUDACC__)
static __device__ __constant__ unsigned long long kExactDivDev[25] = LLVQ_EXACT_DIV_TABLE;
#endif

LLVQ_HD unsigned long long exact_div_params(int n) {
#if defined(__CUDA_ARCH__)
    return kExactDivDev[n];
#else
    return kExactDivHost[n];
#endif
}

// One slot of a multiset unranking with all candidates evaluated at once. `cum` holds the running
// cumulative counts, one per byte (byte j = items left of kinds 0..j; bytes past the last kind equal n).
// The thresholds T_j = M * cum_j / n are exact integers (each M * c_i / n is), independent of one
// another, and the chosen kind is the number of thresholds at or below the rank: no loop-carried
// subtraction, so a single thread gets instruction-level parallelism out of it.
template <int KMAX, typename CumT>
LLVQ_HD int unrank_step32(unsigned int& rank, unsigned int& m, int& n, CumT& cum) {
    const unsigned long long prm = exact_div_params(n);
    const unsigned int inv = (unsigned int)prm, a = (unsigned int)(prm >> 32);
    // the thresholds ascend, so the last one at or below the rank is the lower bound of the chosen
    // kind and the first one above it (M if none) its upper bound
    unsigned int lo = 0, hi = m;
    int chosen = 0;
#pragma unroll
    for (int j = KMAX - 2; j >= 0; --j) {
        const unsigned int cj = (unsigned int)(cum >> (8 * j)) & 0xffu;
        const unsigned int t = (unsigned int)(((unsigned long long)m * cj) >> a) * inv;
        const bool below = rank >= t;  // t = M for the bytes past the last kind: never reached
        chosen += below ? 1 : 0;
        hi = below ? hi : t;
        lo = (below && t > lo) ? t : lo;
    }
    rank -= lo;
    m = hi - lo;
    CumT ones = 0;
#pragma unroll
    for (int j = 0; j < KMAX; ++j) ones |= (CumT)1 << (8 * j);
    cum -= ones << (8 * chosen);
    n -= 1;
    return chosen;
}

// The class-local half of decode_generic12: `local` is the rank of the point inside class `ci` of the
// cap-12 ball (what a caller that has already searched the class passes on, sparing a second search).
// Emits the 24 coordinates in position order, returns the shell.
template <class Emit>
LLVQ_HD int decode_class12(const DevTables& T, int ci, unsigned long long local, Emit emit, float* scale) {
    const DevClass c = T.cls[ci];
    *scale = c.inv_norm;
    unsigned int rank_a, m_a = (unsigned int)c.arr_a, rank_b = 0, m_b = (unsigned int)c.arr_b;
    // byte-wise prefix sums of the counts in one multiplication (no byte exceeds 24, so no carries)
    unsigned long long cum_a = c.cnts_a * 0x0101010101010101ull;
    unsigned int cum_b = c.cnts_b * 0x01010101u;
    int n_a, n_b = 0;
    unsigned int cw, sw = 0, sf = 0;
    if (c.odd) {
        // local = g * m_a + r with g < 4096: the quotient has 12 bits, so 32-bit pieces are enough
        unsigned int g = (unsigned int)(((float)(unsigned int)(local >> 32) * 4294967296.0f + (float)(unsigned int)local) /
                                        (float)m_a);
        long long rem = (long long)(local - (unsigned long long)g * m_a);  // float estimate, fixed up exactly
        while (rem < 0) {
            g -= 1;
            rem += m_a;
        }
        while (rem >= (long long)m_a) {
            g += 1;
            rem -= m_a;
        }
        rank_a = (unsigned int)rem;
        cw = T.golay[g];
        n_a = kDim;
    } else {
        sf = (unsigned int)local & ((1u << c.free_n) - 1u);
        local >>= c.free_n;
        const int wb = c.w ? c.w - 1 : 0;
        sw = (unsigned int)local & ((1u << wb) - 1u);
        local >>= wb;
        const unsigned int q = (unsigned int)local;  // gamma * a_on * a_off < 2^28
        rank_b = q % m_b;
        const unsigned int q2 = q / m_b;
        rank_a = q2 % m_a;
        cw = T.golay[c.golay_base + q2 / m_a];
        if (c.w) sw |= (unsigned int)((popc32(sw) & 1) ^ c.p_req) << (c.w - 1);
        n_a = c.w;
        n_b = kDim - c.w;
    }
#pragma unroll 1
    for (int pos = 0; pos < kDim; ++pos) {
        const unsigned int bit = (cw >> pos) & 1u;
        int val;
        if (c.odd || bit) {
            const int j = unrank_step32<8>(rank_a, m_a, n_a, cum_a);
            const int v = (int)((c.vals_a >> (4 * j)) & 15u);
            if (c.odd) {
                const int a = (v & 3) == 3 ? v : -v;
                val = bit ? a : -a;
            } else {
                val = (sw & 1u) ? -v : v;
                sw >>= 1;
            }
        } else {
            const int j = unrank_step32<4>(rank_b, m_b, n_b, cum_b);
            const int v = (int)((c.vals_b >> (4 * j)) & 15u);
            val = v;
            if (v) {
                val = (sf & 1u) ? -v : v;
                sf >>= 1;
            }
        }
        emit(pos, val);
    }
    return c.shell;
}

// Contract of decode_generic, for idx in the cap-12 ball (anything else is refused).
template <class Emit>
LLVQ_HD int decode_generic12(const DevTables& T, unsigned long long idx, Emit emit, float* scale) {
    if (idx == 0 || idx > kN12) {
#pragma unroll
        for (int pos = 0; pos < kDim; ++pos) emit(pos, 0);
        *scale = 0.0f;
        return idx == 0 ? 0 : 255;
    }
    const unsigned long long i = idx - 1;
    const int ci = find_class(T, i);
    return decode_class12(T, ci, i - T.cls[ci].offset, emit, scale);
}

// Big-endian 48-bit record of block b: idx = v >> 1, gain = v & 1
// (llvq-search/src/pack.rs:113-137, llvq-artifact/src/format.rs:362-368).
LLVQ_HD unsigned long long load_code48(const unsigned char* codes, size_t b) {
    const unsigned char* p = codes + 6 * b;
    unsigned long long v = 0;
#pragma unroll
    for (int t = 0; t < 6; ++t) v = (v << 8) | p[t];
    return v;
}

}  // namespace llvq
