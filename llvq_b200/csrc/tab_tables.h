// Tables of the state-table decoders (decode_tab.cuh) of the cap-12 ball.
//
// The decoders of decode_tab.cuh turn a 47-bit index into 24 signed bytes with
// as little arithmetic per coordinate as the bijection allows:
//
//   odd coset    the 24-slot multiset unranking (llvq-search/src/fastdec.rs:173-194)
//                walks a table of arrangement counts indexed by the remaining kind
//                counts: the thresholds of a slot are one load (no multiplication, no
//                division), the last six slots are one more load from a table of all
//                arrangements of six slots;
//   even coset   on- and off-support arrangements come from tables indexed by their
//                ranks (llvq-search/src/index.rs:361-401 peels the ranks), and are
//                merged into position order four coordinates at a time.
//
// Everything a CTA reads more than once per block lives in ONE contiguous blob
// that the kernels copy into shared memory; only the off-support arrangement
// table (6 MB) stays in global memory. TabLayout gives the byte offset of every
// section of the blob.
#pragma once
#include <cstdint>
#include <vector>

#include "codebook.h"

namespace llvq {

// Decode families of the cap-12 classes (two bits in the class record).
enum TabFamily : unsigned int {
    kFamRare = 0,  // the 30 rare classes (0.07 % of the ball): one of the TabRare decoders
    kFamOdd3 = 1,  // odd coset, at most three kinds: state table of thresholds
    kFamOdd4 = 2,  // odd coset, four kinds: thresholds by exact 32-bit division
    kFamEven = 3   // even coset: arrangement tables + position merge
};

// Decoder of a rare class (word 15 of its record).
enum TabRare : unsigned int {
    kRareNone = 0,
    kRareW24 = 1,   // even coset, support = all 24 positions: state-table walk of the on-support arrangement
    kRareW0 = 2,    // even coset, empty support: state-table walk of the off-support arrangement, signs deposited
    kRareOn3 = 3,   // even coset, three on-support kinds: the even decoder with a wider on-support table
    kRareOdd5 = 4   // odd coset, five kinds: thresholds by exact 32-bit division, no tail table
};

// Dimensions of the three-kind state table: counts (c0, c1, c2) of the kinds in class order
// (two-kind classes sit at c0 = 0). The strides are compile-time constants of the decoder.
constexpr int kT3D0 = 7, kT3D1 = 22, kT3D2 = 25;
constexpr unsigned int kT3S2 = 8;                      // bytes per state: (T0, T01)
constexpr unsigned int kT3S1 = kT3D2 * kT3S2;
constexpr unsigned int kT3S0 = kT3D1 * kT3S1;
constexpr int kTailSlots = 6;                          // slots served by the tail tables
constexpr unsigned int kOffLutCap = 131072;            // largest off-support arrangement count tabulated

struct TabLayout {
    // byte offsets of the sections inside the blob; every section starts 16-byte aligned
    // classification is keyed by the 48-bit record v = 2 idx + gain
    unsigned int lut;     // u16[4096]      by v >> 36: first class whose records reach past (v >> 36) << 36
    unsigned int bounds;  // u64[301 + 2]   bounds[c] = first record of class c | family << 62; bounds[301] = first
                          //                record outside the ball; bounds[302] = 2^48 (sentinel)
    unsigned int cls;     // 301 class records of kClsStride bytes
    unsigned int classify_bytes;  // [0, classify_bytes) is all that classification reads
    unsigned int golay;   // u32[4096]
    unsigned int spread;  // u32[256]   bit i of the byte -> bit 4 i
    unsigned int t3;      // uint2[kT3D0 * kT3D1 * kT3D2]   thresholds by state (tail base where c0+c1+c2 = 6)
    unsigned int tail3;   // u32[3^6]   kinds of the last six slots, one nibble each
    unsigned int tail4;   // u32[4^6]
    unsigned int base4;   // u16[343]   first tail4 entry of a state, by C0 + 7 C1 + 49 C2 (cumulative counts)
    unsigned int lut_on;  // u16[6512]  on-support arrangements: kind bit per support slot
    unsigned int pat;     // u32[16]    merge pattern of a codeword nibble: PRMT selector | popcount << 16
    unsigned int pd4;     // u16[256]   sign deposit of four off-support slots, by nz | signs << 4
    unsigned int total_bytes;
};

// 64-byte class record, read as 16-byte quads.
//   q0  w0, w1 unused; arr (odd: m_arr, even: a_off); scale = 1/sqrt(16 m) as float bits
//   odd   q1  rcp = 1/m_arr as float bits;
//             st0 = byte offset of the class's state inside the t3 section (three kinds), or the
//                   cumulative counts C0 | C1 << 8 | C2 << 16 (four kinds);
//             vt_lo, vt_hi = signed value of kind j off (byte j of vt_lo) and on (byte j of vt_hi)
//                   the codeword support
//   even  q1  geom = a_on | w << 16 | free_n << 24 | p_req << 31; m_off, m_on = magic multipliers;
//             sh = s_off | s_on << 8 | golay_base << 16
//         q2  on_base (entries of lut_on, or of lut_on3 for kRareOn3), off_base (entries of lut_off),
//             vt_on_lo = (+v0, +v1, +v2, 0), vt_on_hi = (-v0, -v1, -v2, 0)
//         q3  vt_off_lo = (f0, f1, f2, f3), vt_off_hi = (-f0, -f1, -f2, -f3)
//   rare  kRareW24: q1 = (p_req, st0, vt_lo = +v by kind, vt_hi = -v by kind)
//         kRareW0:  q1 = (free_n, st0, vt_lo = +f by kind, vt_hi = -f by kind); the zero run is kind 2
//         kRareOdd5: q1 = (rcp, C0 | C1 << 8 | C2 << 16 | C3 << 24, on-support values of kinds 0-3, of kind 4)
//   all   w[14] = shell m, w[15] = TabRare
struct alignas(16) TabClass {
    unsigned int w[16];
};
static_assert(sizeof(TabClass) == 64, "TabClass must stay 64 bytes");
// Records sit kClsStride bytes apart in the blob: an odd multiple of 16, so that the same quad of
// different classes falls into different bank groups of shared memory (a 64-byte stride would put
// every class on one of two).
constexpr unsigned int kClsStride = 80;

// Off-support arrangement of one rank: kinds as nibbles in slot order (x: slots 0-7, y: slots 8-15),
// z = non-zero slot mask | popcount of its low 4, 8, 12 bits << 16, 20, 24.
struct alignas(16) OffEntry {
    unsigned int klo, khi, nz, pad;
};

struct TabTablesHost {
    TabLayout layout;
    std::vector<unsigned char> blob;   // layout.total_bytes
    std::vector<OffEntry> lut_off;
    std::vector<unsigned long long> lut_on3;  // on-support arrangements of the three-kind classes: kind nibbles
    double slow_mass = 0.0;            // fraction of the ball no decoder of this file serves (must be 0)
    double family_mass[4] = {0, 0, 0, 0};
};

void build_tab_tables(const Codebook& cb, TabTablesHost& out);

}  // namespace llvq
