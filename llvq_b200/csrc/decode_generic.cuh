// Generic device decoder of the v1 index map: any class of the cap-13 ball, all
// arithmetic in 64 bits. It is the reference semantics written for one thread
// (Indexer::decode, llvq-search/src/index.rs:334-435, with the exact recurrence
// M' = M * c / n of llvq-search/src/fastdec.rs:173-194) and serves the decode
// probes, the fingerprint check at start-up and the fallback GEMV kernel. The fused
// kernels decode with the table-driven routines of decode_tab.cuh instead.
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
