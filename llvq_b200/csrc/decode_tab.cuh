// State-table decoders of the cap-12 ball (47-bit index): one 24-weight block is
// turned into 24 signed bytes, position p in byte p % 4 of word p / 4, ready for
// four-way integer dot products.
//
// The bijection is the reference's (Indexer::decode, llvq-search/src/index.rs:334-435;
// FastDecoder::decode, llvq-search/src/fastdec.rs:321-399); only the way it is
// evaluated differs:
//
//   tab_decode_odd3   odd coset, up to three kinds. The multiset unranking of
//                     fastdec.rs:173-194 picks, at every slot, the first kind whose
//                     cumulative arrangement count exceeds the rank. Those counts
//                     depend only on the kinds still to place, so they are read from a
//                     table indexed by that state (one 8-byte load per slot) instead of
//                     being derived by M * c / n. The last six slots are one look-up in
//                     a table of all six-slot arrangements.
//   tab_decode_odd4   odd coset, four kinds: thresholds T_j = M * C_j / n in exact 32-bit
//                     arithmetic (n = 2^a * o: multiply by o^-1 mod 2^32, shift by a),
//                     same six-slot tail.
//   tab_decode_even   even coset: the local rank is peeled into (r_sf, r_sw, r_off, r_on, g)
//                     as index.rs:361-369 does, the two arrangements come from tables, and
//                     the support / off-support streams are merged into position order four
//                     coordinates at a time with byte permutes steered by the codeword.
//
// A decoder first builds, per coordinate, a 3-bit code into the class's table of
// (at most eight) signed values; one byte permute then turns four codes into four
// value bytes.
//
// All table reads go through TabView, which is shared memory on the device and a
// plain byte array on the host: the host build exists for the test-suite only.
#pragma once
#include <cstdint>
#include <cstring>

#include "decode_util.cuh"
#include "tab_tables.h"

namespace llvq {

constexpr int kClasses12 = 301;  // classes of the cap-12 ball

// Under nvcc the blob is addressed through the shared window (device code only: the host pass of
// nvcc never reads tables); a plain C++ compiler gets the byte array.
struct TabView {
#if defined(__CUDACC__)
    unsigned int base;  // shared-window address of the blob
#else
    const unsigned char* base;
#endif
    const OffEntry* lut_off;              // global memory
    const unsigned long long* lut_on3;    // global memory (rare classes only)
    TabLayout L;
};

LLVQ_HD unsigned int tab_ld16(const TabView& T, unsigned int off) {
#if defined(__CUDA_ARCH__)
    unsigned short v;
    asm("ld.shared.u16 %0, [%1];" : "=h"(v) : "r"(T.base + off));
    return v;
#elif !defined(__CUDACC__)
    unsigned short v;
    std::memcpy(&v, T.base + off, 2);
    return v;
#else
    return 0;
#endif
}
LLVQ_HD unsigned int tab_ld32(const TabView& T, unsigned int off) {
#if defined(__CUDA_ARCH__)
    unsigned int v;
    asm("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(T.base + off));
    return v;
#elif !defined(__CUDACC__)
    unsigned int v;
    std::memcpy(&v, T.base + off, 4);
    return v;
#else
    return 0;
#endif
}
struct Pair {
    unsigned int x, y;
};
LLVQ_HD Pair tab_ld64(const TabView& T, unsigned int off) {
    Pair p;
#if defined(__CUDA_ARCH__)
    asm("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(p.x), "=r"(p.y) : "r"(T.base + off));
#elif !defined(__CUDACC__)
    std::memcpy(&p, T.base + off, 8);
#else
    p.x = p.y = 0;
#endif
    return p;
}
LLVQ_HD Quad tab_ld128(const TabView& T, unsigned int off) {
    Quad q;
#if defined(__CUDA_ARCH__)
    asm("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "r"(T.base + off));
#elif !defined(__CUDACC__)
    std::memcpy(&q, T.base + off, 16);
#else
    q.x = q.y = q.z = q.w = 0;
#endif
    return q;
}
LLVQ_HD OffEntry tab_ld_off(const TabView& T, unsigned int i) {
#if defined(__CUDA_ARCH__)
    const uint4 v = __ldg(reinterpret_cast<const uint4*>(T.lut_off) + i);
    return OffEntry{v.x, v.y, v.z, v.w};
#else
    return T.lut_off[i];
#endif
}

// Result of the class search for one 48-bit record v = 2 idx + gain: family (TabFamily), or -1 for the
// origin and -2 for an index outside the ball; ci = class; local2 = 2 * (rank inside the class) + gain.
// The tables are read-only for the lifetime of a kernel, so their loads are plain (non-volatile) asm.
struct TabClassified {
    int fam = -1;
    int ci = 0;
    unsigned long long local2 = 0;
};

LLVQ_HD TabClassified tab_classify(const TabView& T, unsigned long long v) {
    TabClassified r;
    // bounds[c] = first record of class c (family in the top two bits). The accelerator names the class
    // of the first record of v's 2^36-wide bucket; nearly every record sits at most one class further
    // (one unconditional step), the few buckets that hold many small classes take the loop.
    const unsigned long long kMask = ~(3ull << 62);  // strips the family bits, keeps the 2^48 sentinel
    unsigned int ci = tab_ld16(T, T.L.lut + 2u * (unsigned int)(v >> 36));
    Pair e = tab_ld64(T, T.L.bounds + 8u * (ci + 1u));
    ci += v >= (((unsigned long long)e.y << 32 | e.x) & kMask) ? 1u : 0u;
    e = tab_ld64(T, T.L.bounds + 8u * (ci + 1u));
    while (v >= (((unsigned long long)e.y << 32 | e.x) & kMask)) {
        ++ci;
        e = tab_ld64(T, T.L.bounds + 8u * (ci + 1u));
    }
    const Pair o = tab_ld64(T, T.L.bounds + 8u * ci);
    r.ci = (int)ci;
    r.fam = v < 2 ? -1 : ci >= (unsigned int)kClasses12 ? -2 : (int)(o.y >> 30);
    r.local2 = v - (((unsigned long long)o.y << 32 | o.x) & kMask);
    return r;
}

// value bytes of the eight coordinates whose codes are the nibbles of `sel`
LLVQ_HD void tab_values8(unsigned int lo, unsigned int hi, unsigned int sel, unsigned int* v) {
    v[0] = byte_perm32(lo, hi, sel & 0xffffu);
    v[1] = byte_perm32(lo, hi, sel >> 16);
}

// Codeword bits as bit 2 of the eight nibbles of each selector word.
LLVQ_HD void tab_codeword_nibbles(const TabView& T, unsigned int cw, unsigned int* sel) {
    sel[0] = tab_ld32(T, T.L.spread + 4u * (cw & 0xffu)) << 2;
    sel[1] = tab_ld32(T, T.L.spread + 4u * ((cw >> 8) & 0xffu)) << 2;
    sel[2] = tab_ld32(T, T.L.spread + 4u * (cw >> 16)) << 2;
}

// The state-table walk: slots 0 .. 17 one threshold pair at a time, the last six from the tail table.
// Adds the kind of every slot (0, 1 or 2) to its nibble of sel[]. p = byte offset of the start state
// in the blob, R = rank of the arrangement.
LLVQ_HD void tab_walk3(const TabView& T, unsigned int p, unsigned int R, unsigned int* sel) {
#pragma unroll
    for (int slot = 0; slot < kDim - kTailSlots; ++slot) {
        const Pair t = tab_ld64(T, p);
        const bool p0 = R >= t.x, p1 = R >= t.y;
        R -= p1 ? t.y : (p0 ? t.x : 0u);
        p -= p1 ? kT3S2 : (p0 ? kT3S1 : kT3S0);
        const unsigned int one = 1u << (4 * (slot & 7));
        sel[slot >> 3] += (p0 ? one : 0u) + (p1 ? one : 0u);
    }
    const unsigned int tb = tab_ld32(T, p);
    sel[2] += tab_ld32(T, T.L.tail3 + 4u * (tb + R)) << (4 * ((kDim - kTailSlots) & 7));
}

// Odd coset, at most three kinds. V receives the 24 value bytes; returns 1/sqrt(16 m).
LLVQ_HD float tab_decode_odd3(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16);
    unsigned int g, R;
    divmod_odd(local, q0.z, bits_to_float(q1.x), &g, &R);
    const unsigned int cw = tab_ld32(T, T.L.golay + 4u * g);
    unsigned int sel[3];
    tab_codeword_nibbles(T, cw, sel);
    tab_walk3(T, T.L.t3 + q1.y, R, sel);
#pragma unroll
    for (int w = 0; w < 3; ++w) tab_values8(q1.z, q1.w, sel[w], V + 2 * w);
    return bits_to_float(q0.w);
}

// Even coset whose support is all 24 positions (rare): local = r_on << 23 | r_sw, one codeword, no
// off-support part. The 24-slot on-support arrangement is walked like an odd class's; the sign of a
// slot takes the place of the codeword bit. The last sign is forced by the class parity
// (index.rs:386-388).
LLVQ_HD float tab_decode_w24(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16);
    const unsigned int r_sw = (unsigned int)local & 0x7fffffu;
    const unsigned int sw = r_sw | ((((unsigned int)popc32(r_sw) & 1u) ^ q1.x) << 23);
    unsigned int sel[3];
    tab_codeword_nibbles(T, sw, sel);
    tab_walk3(T, T.L.t3 + q1.y, (unsigned int)(local >> 23), sel);
#pragma unroll
    for (int w = 0; w < 3; ++w) tab_values8(q1.z, q1.w, sel[w], V + 2 * w);
    return bits_to_float(q0.w);
}

// Even coset with an empty support (rare): local = r_off << free_n | r_sf. The 24-slot off-support
// arrangement is walked like an odd class's (the zero run is kind 2); every non-zero slot then takes
// the next sign bit, in position order.
LLVQ_HD float tab_decode_w0(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16);
    unsigned int sf = (unsigned int)local & ((1u << q1.x) - 1u);
    unsigned int sel[3] = {0u, 0u, 0u};
    tab_walk3(T, T.L.t3 + q1.y, (unsigned int)(local >> q1.x), sel);
#pragma unroll
    for (int w = 0; w < 3; ++w) {
#pragma unroll
        for (int s = 0; s < 8; ++s) {
            const bool nz = ((sel[w] >> (4 * s)) & 3u) != 2u;
            sel[w] |= nz ? (sf & 1u) << (4 * s + 2) : 0u;
            sf >>= nz ? 1 : 0;
        }
        tab_values8(q1.z, q1.w, sel[w], V + 2 * w);
    }
    return bits_to_float(q0.w);
}

// One slot of the unranking by thresholds T_j = M * C_j / n (C_j = cumulative kind counts), n = 2^a * o:
// multiply by o^-1 mod 2^32, shift by a. Exact while T_j * 2^a < 2^32, which holds for every state a
// cap-12 class with n <= 23 reaches; n = 24 takes a 64-bit product. Returns the kind (0 .. K).
template <int K>
LLVQ_HD unsigned int tab_threshold_slot(int n, unsigned int& R, unsigned int& M, unsigned int* C) {
    unsigned int Tj[K];
    if (n == kDim) {
#pragma unroll
        for (int j = 0; j < K; ++j) Tj[j] = (unsigned int)(((unsigned long long)M * C[j]) >> 3) * 0xAAAAAAABu;  // / 8, / 3
    } else {
        const int a = two_adic(n);
        const unsigned int o = odd_part(n);
        const unsigned int mo = o == 1 ? M : M * inv_mod32(o);
#pragma unroll
        for (int j = 0; j < K; ++j) Tj[j] = (mo * C[j]) >> a;
    }
    bool p[K];
#pragma unroll
    for (int j = 0; j < K; ++j) p[j] = R >= Tj[j];
    unsigned int lo = 0, hi = M, kind = 0;
#pragma unroll
    for (int j = 0; j < K; ++j) lo = p[j] ? Tj[j] : lo;
#pragma unroll
    for (int j = K - 1; j >= 0; --j) hi = p[j] ? hi : Tj[j];
    R -= lo;
    M = hi - lo;
#pragma unroll
    for (int j = 0; j < K; ++j) {
        C[j] -= p[j] ? 0u : 1u;
        kind += p[j] ? 1u : 0u;
    }
    return kind;
}

// Odd coset, four kinds.
LLVQ_HD float tab_decode_odd4(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16);
    unsigned int g, R;
    divmod_odd(local, q0.z, bits_to_float(q1.x), &g, &R);
    const unsigned int cw = tab_ld32(T, T.L.golay + 4u * g);
    unsigned int sel[3];
    tab_codeword_nibbles(T, cw, sel);
    unsigned int M = q0.z;
    unsigned int C[3] = {q1.y & 0xffu, (q1.y >> 8) & 0xffu, (q1.y >> 16) & 0xffu};
#pragma unroll
    for (int slot = 0; slot < kDim - kTailSlots; ++slot)
        sel[slot >> 3] += tab_threshold_slot<3>(kDim - slot, R, M, C) << (4 * (slot & 7));
    const unsigned int tb = tab_ld16(T, T.L.base4 + 2u * (C[0] + 7u * C[1] + 49u * C[2]));
    sel[2] += tab_ld32(T, T.L.tail4 + 4u * (tb + R)) << (4 * ((kDim - kTailSlots) & 7));
#pragma unroll
    for (int w = 0; w < 3; ++w) tab_values8(q1.z, q1.w, sel[w], V + 2 * w);
    return bits_to_float(q0.w);
}

// Odd coset, five kinds (one rare class): all 24 slots by thresholds; a slot's value is its kind's
// on-support value, negated off the codeword support.
LLVQ_HD float tab_decode_odd5(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16);
    unsigned int g, R;
    divmod_odd(local, q0.z, bits_to_float(q1.x), &g, &R);
    const unsigned int cw = tab_ld32(T, T.L.golay + 4u * g);
    unsigned int M = q0.z;
    unsigned int C[4] = {q1.y & 0xffu, (q1.y >> 8) & 0xffu, (q1.y >> 16) & 0xffu, q1.y >> 24};
#pragma unroll
    for (int k = 0; k < 6; ++k) V[k] = 0u;
#pragma unroll
    for (int slot = 0; slot < kDim; ++slot) {
        const unsigned int kind = tab_threshold_slot<4>(kDim - slot, R, M, C);
        const unsigned int on = byte_perm32(q1.z, q1.w, kind) & 0xffu;  // on-support value of the kind
        const unsigned int v = ((cw >> slot) & 1u) ? on : (0u - on) & 0xffu;
        V[slot >> 2] |= v << (8 * (slot & 3));
    }
    return bits_to_float(q0.w);
}

// (hi:lo) >> s, low half; s in [0, 64) (a shift of 64 or more never reaches a used nibble)
LLVQ_HD unsigned int tab_window(unsigned int lo, unsigned int hi, unsigned int s) {
#if defined(__CUDA_ARCH__)
    return s >= 32u ? hi >> (s & 31u) : __funnelshift_r(lo, hi, s);
#else
    const unsigned long long v = (unsigned long long)hi << 32 | lo;
    return s >= 64u ? 0u : (unsigned int)(v >> s);
#endif
}

// Even coset served from the arrangement tables. ON3 = the rare classes with three on-support kinds,
// whose on-support arrangements sit in a global table as kind nibbles.
template <bool ON3>
LLVQ_HD float tab_decode_even(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rec = T.L.cls + kClsStride * (unsigned int)ci;
    const Quad q0 = tab_ld128(T, rec), q1 = tab_ld128(T, rec + 16), q2 = tab_ld128(T, rec + 32);
    const Pair q3 = tab_ld64(T, rec + 48);  // vt_off_lo, vt_off_hi
    const unsigned int a_off = q0.z;
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
    const unsigned int cw = tab_ld32(T, T.L.golay + 4u * ((q1.w >> 16) + g));
    // the last support sign is forced by the class parity (index.rs:386-388)
    const unsigned int sw = r_sw | ((((unsigned int)popc32(r_sw) & 1u) ^ p_req) << wb);
    // support stream: nibble s = kind | sign << 2 of support slot s
    unsigned int on_lo = tab_ld32(T, T.L.spread + 4u * (sw & 0xffu)) << 2;
    unsigned int on_hi = tab_ld32(T, T.L.spread + 4u * ((sw >> 8) & 0xffu)) << 2;
    if (ON3) {
#if defined(__CUDA_ARCH__)
        const unsigned long long kn = __ldg(T.lut_on3 + q2.x + r_on);
#else
        const unsigned long long kn = T.lut_on3[q2.x + r_on];
#endif
        on_lo += (unsigned int)kn;
        on_hi += (unsigned int)(kn >> 32);
    } else {
        const unsigned int kon = tab_ld16(T, T.L.lut_on + 2u * (q2.x + r_on));
        on_lo += tab_ld32(T, T.L.spread + 4u * (kon & 0xffu));
        on_hi += tab_ld32(T, T.L.spread + 4u * (kon >> 8));
    }
    // off-support stream: nibble s = kind | sign << 2; a sign bit is consumed by every non-zero slot
    const OffEntry e = tab_ld_off(T, q2.y + r_off);
    const unsigned int nz = e.nz;
    const unsigned int s0 = tab_ld16(T, T.L.pd4 + 2u * ((nz & 15u) | (r_sf & 15u) << 4));
    const unsigned int s1 = tab_ld16(T, T.L.pd4 + 2u * (((nz >> 4) & 15u) | ((r_sf >> ((nz >> 16) & 15u)) & 15u) << 4));
    const unsigned int s2 = tab_ld16(T, T.L.pd4 + 2u * (((nz >> 8) & 15u) | ((r_sf >> ((nz >> 20) & 15u)) & 15u) << 4));
    const unsigned int s3 = tab_ld16(T, T.L.pd4 + 2u * (((nz >> 12) & 15u) | ((r_sf >> ((nz >> 24) & 15u)) & 15u) << 4));
    const unsigned int off_lo = e.klo | s0 | s1 << 16;
    const unsigned int off_hi = e.khi | s2 | s3 << 16;
    // merge: four positions at a time; the codeword nibble says which of them sit on the support
    unsigned int P = 0;  // support slots consumed, times 4
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        const unsigned int pe = tab_ld32(T, T.L.pat + 4u * ((cw >> (4 * k)) & 15u));
        const unsigned int onw = k == 0 ? on_lo : tab_window(on_lo, on_hi, P);
        const unsigned int offw = k == 0 ? off_lo : tab_window(off_lo, off_hi, 16u * k - P);
        const unsigned int A = byte_perm32(q2.z, q2.w, onw & 0xffffu);
        const unsigned int Bv = byte_perm32(q3.x, q3.y, offw & 0xffffu);
        V[k] = byte_perm32(A, Bv, pe & 0xffffu);
        P += (pe >> 16) << 2;
    }
    return bits_to_float(q0.w);
}

// The rare classes: word 15 of the record names the decoder. Returns 0 (and a zero block) for a class no
// decoder serves; the table builder leaves none.
LLVQ_HD float tab_decode_rare(const TabView& T, int ci, unsigned long long local, unsigned int* V) {
    const unsigned int rare = tab_ld32(T, T.L.cls + kClsStride * (unsigned int)ci + 60u);
    if (rare == kRareW24) return tab_decode_w24(T, ci, local, V);
    if (rare == kRareW0) return tab_decode_w0(T, ci, local, V);
    if (rare == kRareOn3) return tab_decode_even<true>(T, ci, local, V);
    if (rare == kRareOdd5) return tab_decode_odd5(T, ci, local, V);
    for (int k = 0; k < 6; ++k) V[k] = 0u;
    return 0.0f;
}

#if defined(__CUDACC__)
// The rare classes (0.07 % of the blocks) out of line, for the kernels: inlined, the four rare decoders add
// their registers and their code to the hot loop. Arguments and results travel by value (registers), not through a stack frame.
struct TabRareBlock {
    unsigned int v0, v1, v2, v3, v4, v5;
    float scale;
};
__device__ __noinline__ TabRareBlock tab_decode_rare_call(unsigned int tab_base, const OffEntry* lut_off,
                                                          const unsigned long long* lut_on3, TabLayout L, int ci,
                                                          unsigned long long local) {
    TabView T;
    T.base = tab_base;
    T.lut_off = lut_off;
    T.lut_on3 = lut_on3;
    T.L = L;
    unsigned int V[6];
    TabRareBlock r;
    r.scale = tab_decode_rare(T, ci, local, V);
    r.v0 = V[0]; r.v1 = V[1]; r.v2 = V[2]; r.v3 = V[3]; r.v4 = V[4]; r.v5 = V[5];
    return r;
}
#endif

// Decode one cap-12 index with whichever routine its class calls for. Returns the family
// (TabFamily; -1 origin, -2 refused index).
LLVQ_HD int tab_decode_any(const TabView& T, unsigned long long idx, unsigned int* V, float* scale) {
    TabClassified c;
    c.fam = -2;  // more than 47 bits: no record holds it
    if ((idx >> 47) == 0) c = tab_classify(T, idx << 1);
    const unsigned long long local = c.local2 >> 1;
    if (c.fam < 0) {
        for (int k = 0; k < 6; ++k) V[k] = 0;
        *scale = 0.0f;
        return c.fam;
    }
    switch ((unsigned int)c.fam) {
        case kFamOdd3: *scale = tab_decode_odd3(T, c.ci, local, V); break;
        case kFamOdd4: *scale = tab_decode_odd4(T, c.ci, local, V); break;
        case kFamEven: *scale = tab_decode_even<false>(T, c.ci, local, V); break;
        default: *scale = tab_decode_rare(T, c.ci, local, V); break;
    }
    return c.fam;
}

}  // namespace llvq
